"""Single-GPU end-to-end checks: every benchmark model family takes training steps through the public API,
and a CUDA-graph-replayed step follows the same trajectory as eager execution."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _trainer(dnn, dataset, bs, **kw):
    import mgwfbp_b200 as hvd
    from mgwfbp_b200.trainer import DLTrainer
    t = DLTrainer(0, 1, dist=False, ngpus=1, batch_size=bs, data_dir='synthetic', dataset=dataset, dnn=dnn, lr=kw.pop('lr', 0.01),
                  nworkers=1, seed=0, **kw)
    t.num_batches_per_epoch = 10 ** 9
    t.update_optimizer(hvd.DistributedOptimizer(t.optimizer, named_parameters=t.net.named_parameters(),
                                                norm_clip=0.25 if dnn == 'lstm' else None))
    return t


@pytest.mark.parametrize('dnn,dataset,bs', [('resnet50', 'imagenet', 8), ('densenet201', 'imagenet', 4), ('vgg16i', 'imagenet', 4),
                                            ('resnet20', 'cifar10', 32), ('lstm', 'ptb', 20), ('inceptionv4', 'imagenet', 4)])
def test_model_family_trains(dnn, dataset, bs):
    from mgwfbp_b200.engine import TrainStep
    from mgwfbp_b200.ops import counters
    t = _trainer(dnn, dataset, bs, lr=22.0 if dnn == 'lstm' else 0.01)
    step = TrainStep(t, use_graph=True)
    counters.reset()
    for _ in range(6):                      # 3 eager steps, capture, 2 replays
        step.run(t.data_iter())
    step.drain()
    torch.cuda.synchronize()
    assert step.graphed, 'the step was not captured in a CUDA graph'
    assert len(step.losses) == 6 and all(l == l and l < 1e4 for l in step.losses), step.losses
    assert counters.total() > 0


def test_graph_replay_matches_eager_trajectory():
    from mgwfbp_b200.engine import TrainStep
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cudnn.deterministic = True
    try:
        losses = {}
        for mode in (False, True):
            t = _trainer('resnet20', 'cifar10', 16, lr=0.05)
            step = TrainStep(t, use_graph=mode)
            g = torch.Generator().manual_seed(3)
            batches = [(torch.randn(16, 3, 32, 32, generator=g).pin_memory(), torch.randint(0, 10, (16,), generator=g).pin_memory())
                       for _ in range(8)]
            for b in batches:
                step.run(b)
            step.drain()
            assert step.graphed == mode
            losses[mode] = list(step.losses)
        for a, b in zip(losses[False], losses[True]):
            assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (losses[False], losses[True])
    finally:
        torch.backends.cudnn.allow_tf32 = True
        torch.backends.cudnn.deterministic = False


def test_fp16_mode_trains_and_tracks_fp32():
    """``settings.FP16``: half-precision forward/backward under autocast, static loss scale 128 divided out inside the
    update kernel.  The fp32 master weights after a few steps stay close to those of an fp32 run from the same start."""
    import mgwfbp_b200 as hvd
    from mgwfbp_b200 import settings
    from mgwfbp_b200.trainer import DLTrainer
    results = {}
    old = settings.FP16
    try:
        for fp16 in (False, True):
            settings.FP16 = fp16
            torch.manual_seed(0)
            trainer = DLTrainer(0, 1, dist=False, batch_size=16, ngpus=1, data_dir='synthetic', dataset='cifar10', dnn='resnet20',
                                lr=0.05, nworkers=1, seed=0)
            assert trainer.fp16 == fp16 and trainer.loss_scale == (128.0 if fp16 else 1.0)
            opt = hvd.DistributedOptimizer(trainer.optimizer, named_parameters=trainer.net.named_parameters())
            trainer.update_optimizer(opt)
            assert opt._grad_scale == (1.0 / 128.0 if fp16 else 1.0)
            losses = []
            for _ in range(6):
                opt.zero_grad()
                trainer.train(1)
                trainer.update_model()
                losses.append(trainer.loss)
            torch.cuda.synchronize()
            results[fp16] = (losses, [p.detach().float().clone() for p in trainer.net.parameters()])
    finally:
        settings.FP16 = old
    l32, p32 = results[False]
    l16, p16 = results[True]
    assert all(l == l and l < 20 for l in l16)
    assert abs(l16[0] - l32[0]) < 0.05 * abs(l32[0]) + 1e-2          # same data, same start: first loss agrees to fp16 accuracy
    num = sum(float((a - b).pow(2).sum()) for a, b in zip(p16, p32))
    den = sum(float(b.pow(2).sum()) for b in p32)
    assert (num / den) ** 0.5 < 2e-2, 'fp16 run drifted from the fp32 run: relative distance %.4f' % ((num / den) ** 0.5)


def test_short_batch_after_capture_runs_eagerly_and_replay_resumes():
    """The last batch of an epoch is shorter than the captured one (loaders do not drop it): that step runs eagerly,
    the next full batch goes through the graph again, and the trajectory equals an all-eager run."""
    from mgwfbp_b200.engine import TrainStep
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cudnn.deterministic = True
    try:
        g = torch.Generator().manual_seed(5)
        sizes = [16, 16, 16, 16, 16, 7, 16, 16, 5, 16]
        batches = [(torch.randn(n, 3, 32, 32, generator=g).pin_memory(), torch.randint(0, 10, (n,), generator=g).pin_memory())
                   for n in sizes]
        out = {}
        for mode in (False, True):
            t = _trainer('resnet20', 'cifar10', 16, lr=0.05)
            step = TrainStep(t, use_graph=mode)
            for b in batches:
                step.run(b)
            step.drain()
            torch.cuda.synchronize()
            out[mode] = (list(step.losses), [p.detach().clone() for p in t.net.parameters()], step.eager_after_capture)
        assert out[True][2] == 2 and out[False][2] == 0
        for a, b in zip(out[False][0], out[True][0]):
            assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (out[False][0], out[True][0])
        for a, b in zip(out[False][1], out[True][1]):
            torch.testing.assert_close(a, b, rtol=1e-3, atol=1e-4)
    finally:
        torch.backends.cudnn.allow_tf32 = True
        torch.backends.cudnn.deterministic = False


def test_status_word_is_read_during_graph_replay():
    """A communication kernel that gave up waiting leaves a record in host-mapped memory.  TrainStep looks at it on
    every step, also while it only replays a graph.  The record is written by the test itself (no kernel fails)."""
    import mgwfbp_b200 as hvd
    from mgwfbp_b200.engine import TrainStep
    from mgwfbp_b200.parallel.comm.base import CommTimeoutError
    from mgwfbp_b200.parallel.comm.nvl import NvlComm
    from mgwfbp_b200.trainer import DLTrainer
    t = DLTrainer(0, 1, dist=False, ngpus=1, batch_size=16, data_dir='synthetic', dataset='cifar10', dnn='resnet20', lr=0.05,
                  nworkers=1, seed=0)
    t.num_batches_per_epoch = 10 ** 9
    comm = NvlComm.shared()
    opt = hvd.DistributedOptimizer(t.optimizer, named_parameters=t.net.named_parameters(), threshold=100000, comm=comm)
    t.update_optimizer(opt)
    step = TrainStep(t, use_graph=True)
    for _ in range(6):
        step.run(t.data_iter())
    step.drain()
    assert step.graphed
    comm._status[1], comm._status[2], comm._status[3], comm._status[4] = 3, 17, 16, 5
    comm._status[0] = 1                                        # MGW_STATUS_TIMEOUT as a kernel would record it
    with pytest.raises(CommTimeoutError, match='waited for rank 3'):
        step.run(t.data_iter())
    comm.clear_status()
    step.run(t.data_iter())                                    # training continues once the record is cleared
    step.drain()
    opt.close()
