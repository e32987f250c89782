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
