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
