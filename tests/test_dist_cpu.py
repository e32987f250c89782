"""CPU / gloo plumbing: two real processes, the public API end to end (no GPU)."""
import os
import socket
import sys
import tempfile

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, args, out_dir, use_cuda=False):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR='127.0.0.1',
                      MASTER_PORT=str(port), MGWFBP_CONNECTION='10GbE')
    sys.path.insert(0, ROOT)
    torch.set_num_threads(1)
    os.environ.setdefault('NCCL_NVLS_ENABLE', '0')
    # tests that exercise the NVSwitch multicast path ask for it themselves; everything else (failure tests above all)
    # runs on peer loads and stores only
    os.environ.setdefault('MGWFBP_NVLS', '0')
    import mgwfbp_b200 as hvd
    hvd.init(timeout_s=float(os.environ.get('MGWFBP_TEST_TIMEOUT_S', '120')), device='cuda' if use_cuda else 'cpu')
    try:
        result = fn(rank, world, *args)
        torch.save(result, os.path.join(out_dir, 'rank%d.pt' % rank))
    finally:
        hvd.shutdown()


def run_ranks(fn, args=(), world=2, use_cuda=None):
    if use_cuda is None:
        use_cuda = fn.__module__ != __name__ and torch.cuda.is_available()
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_worker, args=(world, _free_port(), fn, args, d, use_cuda), nprocs=world, join=True)
        return [torch.load(os.path.join(d, 'rank%d.pt' % r), weights_only=False) for r in range(world)]


# ----------------------------------------------------------------------------- worker bodies
def _train_resnet20(rank, world, policy, steps):
    import mgwfbp_b200 as hvd
    from mgwfbp_b200 import settings
    from mgwfbp_b200.trainer import DLTrainer
    from mgwfbp_b200.utils.profiling import benchmark
    settings.ADAPTIVE_MERGE = policy == 'mgwfbp'
    torch.manual_seed(0)
    trainer = DLTrainer(rank, world, dist=False, batch_size=32, ngpus=0, data_dir='synthetic', dataset='cifar10',
                        dnn='resnet20', lr=0.1, nworkers=world, prefix='allreduce', seed=0)
    seq = times = None
    if policy == 'mgwfbp':
        seq, times, sizes = benchmark(trainer, warmup=1, iteration=2)
        times = hvd.broadcast_object(list(times), 0)
    threshold = {'wfbp': 0, 'single': 524288000, 'mgwfbp': 0, 'bucket': 20000}[policy]
    opt = hvd.DistributedOptimizer(trainer.optimizer, named_parameters=trainer.net.named_parameters(),
                                   seq_layernames=seq, layerwise_times=times, threshold=threshold)
    hvd.broadcast_parameters(trainer.net.state_dict(), root_rank=0)
    trainer.update_optimizer(opt)
    # identical data on every policy: a fixed generator per rank
    g = torch.Generator().manual_seed(100 + rank)
    losses = []
    for _ in range(steps):
        x = torch.randn(32, 3, 32, 32, generator=g)
        y = torch.randint(0, 10, (32,), generator=g)
        opt.zero_grad()
        trainer.train(1, data=(x, y))
        trainer.update_model()
        losses.append(trainer.loss)
    return {'params': {k: v.clone() for k, v in trainer.net.state_dict().items()}, 'losses': losses,
            'ngroups': len(opt.merge_schedule.groups), 'iters': opt.train_iter}


def _train_lenet_vs_concat(rank, world, steps):
    """No BatchNorm, so data parallel over two halves must equal one process on the whole batch."""
    import mgwfbp_b200 as hvd
    from mgwfbp_b200.models import create_net
    torch.manual_seed(0)
    net, _ = create_net(10, 'lenet')
    ref, _ = create_net(10, 'lenet')
    hvd.broadcast_parameters(net.state_dict(), 0)
    ref.load_state_dict(net.state_dict())
    opt = hvd.DistributedOptimizer(torch.optim.SGD(net.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4),
                                   named_parameters=net.named_parameters(), threshold=3000)
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4)
    crit = torch.nn.CrossEntropyLoss()
    g = torch.Generator().manual_seed(7)
    for _ in range(steps):
        x = torch.randn(world * 8, 1, 32, 32, generator=g)
        y = torch.randint(0, 10, (world * 8,), generator=g)
        opt.zero_grad()
        crit(net(x[rank * 8:(rank + 1) * 8]), y[rank * 8:(rank + 1) * 8]).backward()
        opt.step()
        ref_opt.zero_grad()
        crit(ref(x), y).backward()
        ref_opt.step()
    return {'dp': [p.detach().clone() for p in net.parameters()], 'ref': [p.detach().clone() for p in ref.parameters()]}


def _accumulate_and_clip(rank, world):
    import mgwfbp_b200 as hvd
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
    hvd.broadcast_parameters(net.state_dict(), 0)
    opt = hvd.DistributedOptimizer(torch.optim.SGD(net.parameters(), lr=0.1), named_parameters=net.named_parameters(),
                                   threshold=524288000)
    g = torch.Generator().manual_seed(rank)
    xs = [torch.randn(4, 8, generator=g) for _ in range(2)]
    opt.zero_grad()
    opt.local = True
    net(xs[0]).pow(2).mean().backward()
    local_only = [p.grad.clone() for p in net.parameters()]
    opt.local = False
    net(xs[1]).pow(2).mean().backward()
    opt.synchronize()                      # averaged, accumulated gradients are visible here
    grads = [p.grad.clone() for p in net.parameters()]
    total = torch.nn.utils.clip_grad_norm_(net.parameters(), 1e-3)
    opt.step()
    return {'local_only': local_only, 'grads': grads, 'total_norm': float(total),
            'params': [p.detach().clone() for p in net.parameters()]}


def _broadcast_optimizer_state(rank, world):
    import mgwfbp_b200 as hvd
    torch.manual_seed(rank)                # different weights / state per rank on purpose
    net = torch.nn.Linear(4, 3)
    opt = torch.optim.SGD(net.parameters(), lr=0.1 * (rank + 1), momentum=0.9)
    net(torch.randn(2, 4)).sum().backward()
    opt.step()
    hvd.broadcast_parameters(net.state_dict(), 0)
    hvd.broadcast_optimizer_state(opt, 0)
    return {'lr': opt.param_groups[0]['lr'], 'mom': [opt.state[p]['momentum_buffer'].clone() for p in net.parameters()],
            'w': net.weight.detach().clone()}


def _mismatched_schedule(rank, world):
    import mgwfbp_b200 as hvd
    net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Linear(16, 4))
    try:
        hvd.DistributedOptimizer(torch.optim.SGD(net.parameters(), lr=0.1), named_parameters=net.named_parameters(),
                                 threshold=0 if rank == 0 else 524288000)
    except RuntimeError as e:
        return {'error': str(e)}
    return {'error': None}


def _cli_run(rank, world, tmp):
    os.chdir(tmp)
    sys.argv = ['dist_trainer.py']
    import dist_trainer
    trainer = dist_trainer.mgwfbp('resnet20', 'cifar10', 'synthetic', world, 0.1, 8, 1, 1, world, None, 35, None, 1, 0,
                                  max_iters=3)
    return {'iter': trainer.get_train_iter()}


def _replica_guard(rank, world):
    import mgwfbp_b200 as hvd
    from mgwfbp_b200.utils.consistency import ReplicaDivergenceError, ReplicaGuard, check_replicas
    torch.manual_seed(0)
    net = torch.nn.Linear(6, 3)
    hvd.broadcast_parameters(net.state_dict(), 0)
    guard = ReplicaGuard(net, every=2)
    assert guard.step() is False and guard.step() is True          # identical replicas pass
    with torch.no_grad():
        if rank == 1:
            net.bias[1] += 1e-7                                      # one ulp-scale corruption on one rank
    try:
        check_replicas(net.named_parameters())
        return {'caught': None}
    except ReplicaDivergenceError as e:
        return {'caught': str(e)}


def _absent_rank(rank, world):
    """Rank 1 never joins the collective: rank 0 must get an exception within the control-plane timeout."""
    import time
    import mgwfbp_b200 as hvd
    t0 = time.time()
    if rank == 1:
        time.sleep(6)
        return {'error': None, 'waited': time.time() - t0}
    try:
        hvd.barrier()
        return {'error': None, 'waited': time.time() - t0}
    except Exception as e:
        return {'error': type(e).__name__, 'waited': time.time() - t0}


def _flat_ddp(rank, world):
    """The whole-model gradient-averaging wrapper: state broadcast, one reduction per backward, large-batch equality."""
    import mgwfbp_b200 as hvd
    from mgwfbp_b200.parallel.flat_ddp import DistributedDataParallel, reduce_tensor
    torch.manual_seed(rank)                              # ranks start different; construction must align them
    net = torch.nn.Sequential(torch.nn.Linear(12, 20), torch.nn.Tanh(), torch.nn.Linear(20, 3))
    ddp = DistributedDataParallel(net)
    torch.manual_seed(0)
    ref = torch.nn.Sequential(torch.nn.Linear(12, 20), torch.nn.Tanh(), torch.nn.Linear(20, 3))
    opt, ropt = torch.optim.SGD(net.parameters(), lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(3)
    for _ in range(3):
        x = torch.randn(world * 4, 12, generator=g)
        opt.zero_grad()
        ddp(x[rank * 4:(rank + 1) * 4]).pow(2).mean().backward()
        opt.step()
        ropt.zero_grad()
        ref(x).pow(2).mean().backward()
        ropt.step()
    mean_rank = reduce_tensor(torch.tensor([float(rank)]))
    return {'dp': [p.detach().clone() for p in net.parameters()], 'ref': [p.detach().clone() for p in ref.parameters()],
            'reductions': ddp.reductions, 'mean_rank': float(mean_rank)}


# ----------------------------------------------------------------------------- tests
@pytest.fixture(scope='module')
def resnet20_runs():
    return {p: run_ranks(_train_resnet20, (p, 3)) for p in ('wfbp', 'single', 'mgwfbp', 'bucket')}


def test_replicas_stay_bit_identical(resnet20_runs):
    for policy, (r0, r1) in resnet20_runs.items():
        for k in r0['params']:
            if 'running_' in k or 'num_batches' in k:
                continue          # BatchNorm statistics are per worker, as in the reference
            assert torch.equal(r0['params'][k], r1['params'][k]), (policy, k)
        assert r0['iters'] == 3


def test_merge_policies_agree(resnet20_runs):
    base = resnet20_runs['wfbp'][0]['params']
    assert resnet20_runs['wfbp'][0]['ngroups'] == 59
    assert resnet20_runs['single'][0]['ngroups'] == 1
    assert 1 < resnet20_runs['bucket'][0]['ngroups'] < 59
    for policy in ('single', 'mgwfbp', 'bucket'):
        other = resnet20_runs[policy][0]['params']
        for k in base:
            # running statistics also see the profiler's extra forward passes in the mgwfbp run
            if base[k].dtype.is_floating_point and 'running_' not in k:
                torch.testing.assert_close(other[k], base[k], rtol=1e-5, atol=1e-6, msg=lambda m: '%s %s: %s' % (policy, k, m))
    assert all(l == l for l in resnet20_runs['mgwfbp'][0]['losses'])      # finite, not NaN


def test_data_parallel_equals_large_batch():
    r0, r1 = run_ranks(_train_lenet_vs_concat, (4,))
    for dp, ref in zip(r0['dp'], r0['ref']):
        torch.testing.assert_close(dp, ref, rtol=1e-4, atol=1e-6)
    for a, b in zip(r0['dp'], r1['dp']):
        assert torch.equal(a, b)


def test_local_accumulation_synchronize_and_clip():
    r0, r1 = run_ranks(_accumulate_and_clip)
    for a, b in zip(r0['grads'], r1['grads']):
        assert torch.equal(a, b)                       # averaged gradients agree across ranks
    assert any(not torch.equal(a, b) for a, b in zip(r0['local_only'], r1['local_only']))
    for a, b in zip(r0['params'], r1['params']):
        assert torch.equal(a, b)
    assert r0['total_norm'] > 1e-3


def test_broadcast_optimizer_state():
    r0, r1 = run_ranks(_broadcast_optimizer_state)
    assert r0['lr'] == r1['lr'] == pytest.approx(0.1)
    for a, b in zip(r0['mom'], r1['mom']):
        assert torch.equal(a, b)
    assert torch.equal(r0['w'], r1['w'])


def test_mismatched_schedule_is_detected():
    r0, r1 = run_ranks(_mismatched_schedule)
    assert r0['error'] and 'disagree' in r0['error']
    assert r1['error'] and 'disagree' in r1['error']


def test_dist_trainer_loop_runs(tmp_path):
    r0, r1 = run_ranks(_cli_run, (str(tmp_path),))
    assert r0['iter'] == 3 and r1['iter'] == 3


def test_replica_guard_detects_divergence():
    r0, r1 = run_ranks(_replica_guard)
    assert r0['caught'] and 'bias' in r0['caught'] and r1['caught']


def test_absent_rank_surfaces_as_timeout_not_hang(monkeypatch):
    monkeypatch.setenv('MGWFBP_TEST_TIMEOUT_S', '3')
    r0, r1 = run_ranks(_absent_rank)
    assert r0['error'] is not None and r0['waited'] < 30


def test_flat_allreduce_wrapper_matches_large_batch():
    res = run_ranks(_flat_ddp, (), world=2)
    for r in res:
        assert r['reductions'] == 3 and r['mean_rank'] == 0.5
        for a, b in zip(r['dp'], r['ref']):
            torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    for a, b in zip(res[0]['dp'], res[1]['dp']):
        assert torch.equal(a, b)


def _trial_harness(rank, world):
    """engine.tune_schedule on the CPU data plane: candidates are built, trained, timed, closed; the optimizer state
    (momentum) created under one wrapper is handed on to the next, and every rank installs the same winner."""
    import mgwfbp_b200 as hvd
    from mgwfbp_b200 import settings
    from mgwfbp_b200.engine import tune_schedule
    from mgwfbp_b200.trainer import DLTrainer
    settings.ADAPTIVE_MERGE = False
    torch.manual_seed(0)
    trainer = DLTrainer(rank, world, dist=False, batch_size=8, ngpus=0, data_dir='synthetic', dataset='cifar10',
                        dnn='resnet20', lr=0.05, nworkers=world, prefix='allreduce', seed=0)
    trainer.num_batches_per_epoch = 10 ** 9
    base = trainer.optimizer
    hvd.broadcast_parameters(trainer.net.state_dict(), root_rank=0)
    thresholds = {0.0: 0, 0.5: 50000, 1.0: 524288000}
    built = []

    def build(rho, update, late=False):
        opt = hvd.DistributedOptimizer(base, named_parameters=trainer.net.named_parameters(), threshold=thresholds[rho],
                                       late_full=late)
        built.append(opt)
        return opt
    # the candidate dictionaries of engine.build_distributed_optimizer have these keys
    opt, report = tune_schedule(trainer, build, [{'rho': r, 'update': None, 'late': False} for r in (0.0, 0.5, 1.0, 0.5)], steps=2)
    assert all(r['late_groups'] == [] for r in report)
    assert trainer.optimizer is opt and opt._active
    assert all(not o._active for o in built[:-1]), 'retired wrappers still own hooks'
    assert [r['groups'] for r in report][2] == 1 and report[3].get('same_as_earlier')
    # momentum buffers created during the trials live on in the installed wrapper
    p0 = next(iter(trainer.net.parameters()))
    assert 'momentum_buffer' in opt.state[p0] and float(opt.state[p0]['momentum_buffer'].abs().sum()) > 0
    opt.zero_grad()
    trainer.train(1)
    trainer.update_model()
    return {'groups': len(opt.merge_schedule.groups), 'report': [(r['rho'], r['groups']) for r in report],
            'params': [p.detach().clone() for p in trainer.net.parameters()]}


def test_schedule_trial_harness_on_cpu():
    res = run_ranks(_trial_harness, (), world=2)
    assert res[0]['groups'] == res[1]['groups'] and res[0]['report'] == res[1]['report']
    for a, b in zip(res[0]['params'], res[1]['params']):
        assert torch.equal(a, b), 'replicas diverged'


def _train_densenet_blocks(rank, world, steps):
    """A small torchvision DenseNet under the merged-gradient optimizer: the single-buffer dense blocks (nested backward per
    layer, gradient hooks firing inside it) against the list-and-concatenate blocks, same data, same schedule."""
    import copy
    import torchvision
    import mgwfbp_b200 as hvd
    from mgwfbp_b200.models import dense_block
    from mgwfbp_b200.models.fuse import fuse_model
    torch.manual_seed(0)
    base = torchvision.models.densenet.DenseNet(growth_rate=8, block_config=(3, 3), num_init_features=16, bn_size=2, num_classes=10)
    out = {}
    for kind in ('single_buffer', 'plain'):
        net = fuse_model(copy.deepcopy(base)).train()
        if kind == 'plain':
            for m in net.modules():
                if isinstance(m, torchvision.models.densenet._DenseBlock):
                    m.forward = dense_block._plain_forward.__get__(m)
        hvd.broadcast_parameters(net.state_dict(), 0)
        opt = hvd.DistributedOptimizer(torch.optim.SGD(net.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4),
                                       named_parameters=net.named_parameters(), threshold=4000)
        g = torch.Generator().manual_seed(11)
        for _ in range(steps):
            x = torch.randn(world * 4, 3, 32, 32, generator=g)
            y = torch.randint(0, 10, (world * 4,), generator=g)
            opt.zero_grad()
            torch.nn.functional.cross_entropy(net(x[rank * 4:(rank + 1) * 4]), y[rank * 4:(rank + 1) * 4]).backward()
            opt.step()
        out[kind] = [p.detach().clone() for p in net.parameters()]
    return out


def test_dense_blocks_under_the_merged_gradient_optimizer():
    r0, r1 = run_ranks(_train_densenet_blocks, (3,))
    for a, b in zip(r0['single_buffer'], r1['single_buffer']):
        assert torch.equal(a, b)                                   # replicas stay bit-identical
    for a, b in zip(r0['single_buffer'], r0['plain']):
        torch.testing.assert_close(a, b, rtol=2e-3, atol=2e-5)     # same training as with the list-and-concatenate blocks
