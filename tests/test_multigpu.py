"""Multi-GPU tests of the NVLink data plane (one process per GPU, 2..4 GPUs of one box)."""
import os
import sys

import pytest
import torch

from test_dist_cpu import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _world():
    # 2..4 ranks by default; MGWFBP_TEST_WORLD=8 runs the same tests on all GPUs of an 8-GPU box
    return min(torch.cuda.device_count(), int(os.environ.get('MGWFBP_TEST_WORLD', '4')))


def _allreduce_sweep(rank, world, pieces=1):
    if pieces > 1:
        # the two-shot kernel walks each CTA's chunk in several pieces, one flag value per piece
        os.environ['MGWFBP_PIECES'] = str(pieces)
        os.environ['MGWFBP_PIECE_SLOTS'] = '64'
    from mgwfbp_b200.parallel.comm.nvl import NvlComm
    comm = NvlComm.shared()
    assert comm.max_pieces == pieces
    out = {}
    for algo in ('oneshot', 'twoshot'):
        for numel in (1, 7, 1024, 32771, 1 << 17, (1 << 22) + 3):
            if algo == 'oneshot' and numel * 4 > comm.oneshot_max_bytes:
                continue
            g = torch.Generator(device='cuda').manual_seed(1000 * rank + numel % 997)
            x = torch.randn(numel, device='cuda', generator=g)
            mine = x.clone()
            comm.synchronize(comm.allreduce_async_(x, average=True, algo=algo))
            again = mine.clone()
            comm.synchronize(comm.allreduce_async_(again, average=True, algo=algo))
            torch.cuda.synchronize()
            comm.check_status()
            out[(algo, numel)] = (mine.cpu(), x.cpu(), bool(torch.equal(x, again)))
    return out


@pytest.mark.parametrize('pieces', [1, 4])
def test_allreduce_matches_cpu_sum_and_is_deterministic(pieces):
    world = _world()
    res = run_ranks(_allreduce_sweep, (pieces,), world=world)
    for key in res[0]:
        want = sum(r[key][0].double() for r in res) / world
        for r in res:
            torch.testing.assert_close(r[key][1].double(), want, rtol=1e-6, atol=1e-6, msg=lambda m: '%s: %s' % (key, m))
            assert torch.equal(r[key][1], res[0][key][1]), 'ranks differ bitwise for %s' % (key,)
            assert r[key][2], 'repeat differs for %s' % (key,)


def _fused_training(rank, world, policy, fused):
    if fused == 'deferred':
        os.environ['MGWFBP_ONESHOT_MAX_BYTES'] = '1024'      # the small layers of this model take the two-shot kernel too
    import mgwfbp_b200 as hvd
    from mgwfbp_b200 import settings
    settings.ADAPTIVE_MERGE = False
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.ReLU(), torch.nn.Linear(256, 256), torch.nn.ReLU(),
                              torch.nn.Linear(256, 10)).cuda()
    ref = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.ReLU(), torch.nn.Linear(256, 256), torch.nn.ReLU(),
                              torch.nn.Linear(256, 10)).cuda()
    hvd.broadcast_parameters(net.state_dict(), 0)
    ref.load_state_dict(net.state_dict())
    mk = lambda m: torch.optim.SGD(m.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4)
    threshold = {'wfbp': 0, 'single': 524288000, 'bucket': 20000, 'mgwfbp': 0, 'mgwfbp-free': 0}[policy]
    seq = times = None
    if policy.startswith('mgwfbp'):
        # measured-schedule path: forward-order names + per-layer backward times (made up, equal on all ranks)
        settings.ADAPTIVE_MERGE = True
        settings.INTERFERENCE = 1.0 if policy == 'mgwfbp' else 0.0
        seq = [n for n, _ in net.named_parameters()]
        times = [2e-5] * len(seq)
    opt = hvd.DistributedOptimizer(mk(net), named_parameters=net.named_parameters(), threshold=threshold, fused_update=fused,
                                   seq_layernames=seq, layerwise_times=times)
    assert opt._fused_comm and opt._update_mode == {True: 'fused', False: 'separate'}.get(fused, fused)
    if policy == 'mgwfbp':
        assert len(opt.merge_schedule.groups) == 1          # full interference: one message
    if policy == 'mgwfbp-free':
        assert len(opt.merge_schedule.groups) > 1
    ropt = mk(ref)
    crit = torch.nn.CrossEntropyLoss()
    g = torch.Generator().manual_seed(5)
    for _ in range(6):
        x = torch.randn(world * 16, 64, generator=g).cuda()
        y = torch.randint(0, 10, (world * 16,), generator=g).cuda()
        opt.zero_grad()
        crit(net(x[rank * 16:(rank + 1) * 16]), y[rank * 16:(rank + 1) * 16]).backward()
        opt.step()
        ropt.zero_grad()
        crit(ref(x), y).backward()
        ropt.step()
    torch.cuda.synchronize()
    opt.communicator.check_status()
    return {'dp': [p.detach().cpu() for p in net.parameters()], 'ref': [p.detach().cpu() for p in ref.parameters()]}


@pytest.mark.parametrize('policy,fused', [('wfbp', True), ('single', True), ('bucket', True), ('bucket', False),
                                          ('mgwfbp', True), ('mgwfbp-free', True),
                                          # the averaged gradient is consumed from the staging areas by one SGD kernel
                                          ('bucket', 'deferred'), ('single', 'deferred'), ('wfbp', 'deferred')])
def test_fused_data_parallel_equals_large_batch(policy, fused):
    res = run_ranks(_fused_training, (policy, fused), world=_world())
    for dp, ref in zip(res[0]['dp'], res[0]['ref']):
        torch.testing.assert_close(dp, ref, rtol=2e-4, atol=2e-5)
    for r in res[1:]:
        for a, b in zip(res[0]['dp'], r['dp']):
            assert torch.equal(a, b), 'replicas diverged'


def _shadowed_training(rank, world, clip):
    """The fused path re-checked every second iteration by the slow path (gradients over gloo, update in PyTorch);
    then one snapshot is altered on the host and the check must name the tensor."""
    import mgwfbp_b200 as hvd
    from mgwfbp_b200 import settings
    from mgwfbp_b200.utils.consistency import ShadowMismatchError
    settings.ADAPTIVE_MERGE = False
    settings.SHADOW_EVERY = 2
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(64, 301), torch.nn.ReLU(), torch.nn.Linear(301, 10)).cuda()
    hvd.broadcast_parameters(net.state_dict(), 0)
    opt = hvd.DistributedOptimizer(torch.optim.SGD(net.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4, nesterov=True),
                                   named_parameters=net.named_parameters(), threshold=20000, norm_clip=clip)
    assert opt._shadow is not None
    g = torch.Generator().manual_seed(5 + rank)
    for _ in range(5):
        opt.zero_grad()
        net(torch.randn(16, 64, generator=g).cuda()).pow(2).mean().backward()
        opt.step()
    checked = opt._shadow.checked
    # iteration 6 (index 5) is unchecked; on iteration 7 spoil the first snapshot before verify runs
    opt.zero_grad(); net(torch.randn(16, 64, generator=g).cuda()).pow(2).mean().backward(); opt.step()
    opt.zero_grad(); net(torch.randn(16, 64, generator=g).cuda()).pow(2).mean().backward()
    opt.synchronize()
    name, grad, w, buf, first = opt._shadow._snap[0]
    opt._shadow._snap[0] = (name, grad + 1.0, w, buf, first)
    try:
        opt.step()
        caught = None
    except ShadowMismatchError as e:
        caught = str(e)
    torch.cuda.synchronize()
    opt.communicator.check_status()
    return checked, caught, name


@pytest.mark.parametrize('clip', [None, 0.25])
def test_shadow_path_agrees_and_detects_a_spoiled_snapshot(clip):
    res = run_ranks(_shadowed_training, (clip,), world=_world())
    for checked, caught, name in res:
        assert checked == 3 * 4                 # iterations 0, 2, 4; four tensors each
        assert caught is not None and name in caught


def _gathered_wgrad(rank, world):
    """A large linear layer fed by a small batch: its weight is updated from gathered activations by
    the tensor-core GEMM with the SGD epilogue and never enters the gradient all-reduce."""
    import mgwfbp_b200 as hvd
    from mgwfbp_b200 import settings
    from mgwfbp_b200.ops.wgrad import convert_large_linears, GatheredWgradLinear
    settings.WRITE_BACK_GRADS = True        # this test also looks at the gradient the GEMM formed
    torch.manual_seed(0)
    torch.backends.cuda.matmul.allow_tf32 = False
    mk_net = lambda: torch.nn.Sequential(torch.nn.Linear(64, 2048), torch.nn.ReLU(), torch.nn.Linear(2048, 4096),
                                         torch.nn.ReLU(), torch.nn.Linear(4096, 16)).cuda()
    net, ref = mk_net(), mk_net()
    assert convert_large_linears(net) == 1 and isinstance(net[2], GatheredWgradLinear)
    net[2].batch_rows_hint = 8
    hvd.broadcast_parameters(net.state_dict(), 0)
    ref.load_state_dict(net.state_dict())
    mk = lambda m: torch.optim.SGD(m.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4)
    opt = hvd.DistributedOptimizer(mk(net), named_parameters=net.named_parameters(), threshold=0)
    assert [n for n, _, _ in opt._external] == ['2.weight']
    assert '2.weight' not in opt.merge_schedule.key_groupidx and len(opt.merge_schedule.groups) == 5
    ropt = mk(ref)
    g = torch.Generator().manual_seed(11)
    for _ in range(4):
        x = torch.randn(world * 8, 64, generator=g).cuda()
        opt.zero_grad()
        net(x[rank * 8:(rank + 1) * 8]).pow(2).mean().backward()
        opt.step()
        ropt.zero_grad()
        ref(x).pow(2).mean().backward()
        ropt.step()
    torch.cuda.synchronize()
    opt.communicator.check_status()
    from mgwfbp_b200.ops import wgrad
    wgrad.check_status()
    return {'dp': [p.detach().cpu() for p in net.parameters()], 'ref': [p.detach().cpu() for p in ref.parameters()],
            'grad': net[2].weight.grad.detach().cpu(), 'ref_grad': ref[2].weight.grad.detach().cpu()}


def test_gathered_wgrad_layer_matches_large_batch_sgd():
    res = run_ranks(_gathered_wgrad, (), world=2)
    # the GEMM reads its operands as TF32, the reference runs in fp32: compare at TF32 accuracy
    for dp, ref in zip(res[0]['dp'], res[0]['ref']):
        torch.testing.assert_close(dp, ref, rtol=5e-3, atol=2e-4)
    torch.testing.assert_close(res[0]['grad'], res[0]['ref_grad'], rtol=2e-2, atol=1e-5)
    for a, b in zip(res[0]['dp'], res[1]['dp']):
        assert torch.equal(a, b), 'replicas diverged'


def _clip_path(rank, world):
    import mgwfbp_b200 as hvd
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(), torch.nn.Linear(64, 8)).cuda()
    ref = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(), torch.nn.Linear(64, 8)).cuda()
    hvd.broadcast_parameters(net.state_dict(), 0)
    ref.load_state_dict(net.state_dict())
    opt = hvd.DistributedOptimizer(torch.optim.SGD(net.parameters(), lr=1.0), named_parameters=net.named_parameters(),
                                   threshold=1000, norm_clip=0.05)
    ropt = torch.optim.SGD(ref.parameters(), lr=1.0)
    g = torch.Generator().manual_seed(3)
    for _ in range(3):
        x = torch.randn(world * 8, 32, generator=g).cuda()
        opt.zero_grad()
        net(x[rank * 8:(rank + 1) * 8]).pow(2).mean().backward()
        opt.step()
        ropt.zero_grad()
        ref(x).pow(2).mean().backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.05)
        ropt.step()
    torch.cuda.synchronize()
    return {'dp': [p.detach().cpu() for p in net.parameters()], 'ref': [p.detach().cpu() for p in ref.parameters()]}


def test_global_norm_clip_without_host_sync():
    res = run_ranks(_clip_path, (), world=_world())
    for dp, ref in zip(res[0]['dp'], res[0]['ref']):
        torch.testing.assert_close(dp, ref, rtol=2e-4, atol=2e-5)
    for a, b in zip(res[0]['dp'], res[1]['dp']):
        assert torch.equal(a, b)


def _missing_peer(rank, world):
    """Rank 1 never launches its group: rank 0's kernel must time out and report, not hang.
    The failure is injected on the host (a skipped launch); no GPU is faulted."""
    os.environ['MGWFBP_COMM_TIMEOUT_S'] = '0.2'
    os.environ['MGWFBP_HEAP'] = 'ipc'                  # plain peer memory, nothing bound to the switch
    from mgwfbp_b200.parallel.comm.base import CommTimeoutError
    from mgwfbp_b200.parallel.comm.nvl import NvlComm
    import mgwfbp_b200 as hvd
    comm = NvlComm.shared()
    assert not comm.nvls_available
    x = torch.ones(4096, device='cuda')
    comm.synchronize(comm.allreduce_async_(x.clone()))          # a healthy round first
    torch.cuda.synchronize()
    err = None
    if rank == 0:
        comm.synchronize(comm.allreduce_async_(x))
        torch.cuda.synchronize()
        try:
            comm.check_status()
        except CommTimeoutError as e:
            err = str(e)
    hvd.barrier()
    alive = float((torch.ones(4, device='cuda') * 3).sum())
    return {'err': err, 'alive': alive}


def test_missing_peer_is_reported_not_hung():
    res = run_ranks(_missing_peer, (), world=2)
    assert res[0]['err'] and 'gave up' in res[0]['err']
    assert res[0]['alive'] == 12.0 and res[1]['alive'] == 12.0


def _nvls_allreduce(rank, world):
    """NVSwitch multicast path (multimem.ld_reduce / multimem.st) on the package's own heap (cuMemCreate memory bound
    to a multicast object).  Every rank reaches the final barrier whatever happens, so no rank leaves while peers
    still use the heap."""
    os.environ['MGWFBP_HEAP'] = 'vmm'
    os.environ['MGWFBP_NVLS'] = '1'
    import mgwfbp_b200 as hvd
    out = {'available': False, 'error': None, 'results': {}}
    try:
        from mgwfbp_b200.parallel.comm.nvl import NvlComm
        comm = NvlComm.shared()
        out['available'] = bool(comm.nvls_available)
        out['heap'] = comm.arena.heaps[0].kind
        if comm.nvls_available:
            for numel in (4096, (1 << 20) + 4):
                g = torch.Generator(device='cuda').manual_seed(77 * rank + 1)
                x = torch.randn(numel, device='cuda', generator=g)
                mine = x.clone()
                comm.synchronize(comm.allreduce_async_(x, average=True, algo='nvls'))
                torch.cuda.synchronize()
                comm.check_status()
                out['results'][numel] = (mine.cpu(), x.cpu())
    except Exception as e:            # report instead of leaving early
        out['error'] = '%s: %s' % (type(e).__name__, e)
    hvd.barrier()
    torch.cuda.synchronize()
    return out


def test_nvls_multimem_allreduce_when_available():
    world = _world()
    res = run_ranks(_nvls_allreduce, (), world=world)
    if res[0]['error'] or not res[0]['available']:
        pytest.skip('NVLS multicast not usable here: %s' % (res[0]['error'] or 'no multicast address'))
    for numel in res[0]['results']:
        want = sum(r['results'][numel][0].double() for r in res) / world
        for r in res:
            torch.testing.assert_close(r['results'][numel][1].double(), want, rtol=1e-5, atol=1e-5)
            assert torch.equal(r['results'][numel][1], res[0]['results'][numel][1])


def _selfcheck_and_heap(rank, world, nvls):
    os.environ['MGWFBP_NVLS'] = '1' if nvls else '0'
    import mgwfbp_b200 as hvd
    from mgwfbp_b200.parallel.comm.nvl import NvlComm
    from mgwfbp_b200.parallel.comm.selfcheck import selfcheck
    comm = NvlComm.shared()
    out = selfcheck(comm)
    out['heap'] = comm.arena.heaps[0].kind
    # blocks come back to the arena and are handed out again at the same offsets on every rank
    a = comm.arena.alloc(1 << 20)
    b = comm.arena.alloc(3 << 20)
    offs = (a.off, b.off)
    comm.arena.free(a)
    c = comm.arena.alloc(1 << 19)
    out['offsets'] = (offs, c.off)
    hvd.barrier()
    return out


@pytest.mark.parametrize('nvls', [False, True])
def test_selfcheck_on_the_default_heap(nvls):
    res = run_ranks(_selfcheck_and_heap, (nvls,), world=_world())
    assert all(r['heap'] == 'vmm' for r in res), [r['heap'] for r in res]
    assert all(r['ok'] and r['bitwise_equal'] for r in res), res[0]
    assert len({str(r['offsets']) for r in res}) == 1
    assert res[0]['offsets'][1] == res[0]['offsets'][0][0]          # the freed block was reused
    if nvls and not res[0]['multicast_heap']:
        pytest.skip('the devices offer no NVSwitch multicast; checked one-shot and two-shot only')
    if nvls:
        assert 'nvls' in res[0]['algorithms']


def _graph_replay_with_moving_lr(rank, world):
    """Learning rate changes before every replay of the captured step (what the warm-up schedule does); the
    table upload must be ordered against the replays on every rank, or replicas drift apart."""
    import mgwfbp_b200 as hvd
    from mgwfbp_b200 import settings
    from mgwfbp_b200.engine import TrainStep
    from mgwfbp_b200.trainer import DLTrainer
    settings.ADAPTIVE_MERGE = False
    t = DLTrainer(rank, world, dist=False, ngpus=1, batch_size=16, data_dir='synthetic', dataset='cifar10', dnn='resnet20',
                  lr=0.1, nworkers=world, seed=0)
    t.num_batches_per_epoch = 40            # warm-up over 5 "epochs" of 40 steps: lr differs at every step
    opt = hvd.DistributedOptimizer(t.optimizer, named_parameters=t.net.named_parameters(), threshold=100000)
    hvd.broadcast_parameters(t.net.state_dict(), 0)
    t.update_optimizer(opt)
    step = TrainStep(t, use_graph=True)
    lrs = []
    for _ in range(14):
        step.run(t.data_iter())
        lrs.append(t.lr)
    step.drain()
    torch.cuda.synchronize()
    return {'graphed': step.graphed, 'lrs': lrs, 'params': [p.detach().cpu() for p in t.net.parameters()],
            'losses': list(step.losses)}


def test_replicas_stay_identical_while_lr_moves_under_graph_replay():
    res = run_ranks(_graph_replay_with_moving_lr, (), world=2)
    assert res[0]['graphed'] and len(set(res[0]['lrs'])) == len(res[0]['lrs'])
    for a, b in zip(res[0]['params'], res[1]['params']):
        assert torch.equal(a, b), 'replicas diverged'
    assert all(l == l for l in res[0]['losses'])


def _missing_peer_under_graph_replay(rank, world):
    """Rank 1 skips one replay of its captured step on the host.  Rank 0's communication kernels run into their
    bounded wait, record it, and the next look at the status word -- TrainStep does that every step -- raises.
    Nothing faults: plain peer memory, short timeout, both ranks meet at the final barrier."""
    os.environ['MGWFBP_COMM_TIMEOUT_S'] = '0.2'
    os.environ['MGWFBP_HEAP'] = 'ipc'
    import mgwfbp_b200 as hvd
    from mgwfbp_b200 import settings
    from mgwfbp_b200.engine import TrainStep
    from mgwfbp_b200.parallel.comm.base import CommTimeoutError
    from mgwfbp_b200.trainer import DLTrainer
    settings.ADAPTIVE_MERGE = False
    settings.WARMUP = False
    t = DLTrainer(rank, world, dist=False, ngpus=1, batch_size=16, data_dir='synthetic', dataset='cifar10', dnn='resnet20',
                  lr=0.05, nworkers=world, seed=0)
    t.num_batches_per_epoch = 10 ** 9
    opt = hvd.DistributedOptimizer(t.optimizer, named_parameters=t.net.named_parameters(), threshold=100000)
    hvd.broadcast_parameters(t.net.state_dict(), 0)
    t.update_optimizer(opt)
    step = TrainStep(t, use_graph=True)
    for _ in range(6):
        step.run(t.data_iter())
    step.drain()
    torch.cuda.synchronize()
    assert step.graphed
    hvd.barrier()
    err, after = None, 0
    if rank == 0:
        try:
            for after in range(1, 4):               # the step rank 1 skips, and at most two more looks
                step.run(t.data_iter())
                torch.cuda.synchronize()
            step.drain()
        except CommTimeoutError as e:
            err = str(e)
    hvd.barrier()
    torch.cuda.synchronize()
    alive = float((torch.ones(4, device='cuda') * 3).sum())
    return {'err': err, 'steps_until_raise': after, 'alive': alive}


def test_missing_peer_is_detected_under_graph_replay():
    res = run_ranks(_missing_peer_under_graph_replay, (), world=2)
    assert res[0]['err'] and 'gave up' in res[0]['err'], res[0]
    assert res[0]['steps_until_raise'] <= 2
    assert res[0]['alive'] == 12.0 and res[1]['alive'] == 12.0


def _tuned_schedule(rank, world):
    """engine.build_distributed_optimizer end to end on a small model: cost-model fit, interference fit, trial."""
    import mgwfbp_b200 as hvd
    from mgwfbp_b200 import settings
    from mgwfbp_b200.engine import TrainStep, build_distributed_optimizer
    from mgwfbp_b200.trainer import DLTrainer
    from mgwfbp_b200.utils.profiling import benchmark
    settings.ADAPTIVE_MERGE = True
    t = DLTrainer(rank, world, dist=False, ngpus=1, batch_size=32, data_dir='synthetic', dataset='cifar10', dnn='resnet20',
                  lr=0.05, nworkers=world, seed=0)
    t.num_batches_per_epoch = 10 ** 9
    seq, times, _ = benchmark(t, warmup=2, iteration=4)
    times = hvd.broadcast_object(list(times), 0)
    opt, info = build_distributed_optimizer(t, seq_layernames=seq, layerwise_times=times, trial_steps=4)
    step = TrainStep(t, use_graph=True)
    for _ in range(6):
        step.run(t.data_iter())
    step.drain()
    torch.cuda.synchronize()
    opt.communicator.check_status()
    return {'info': info, 'groups': len(opt.merge_schedule.groups), 'losses': list(step.losses),
            'params': [p.detach().cpu() for p in t.net.parameters()]}


def test_schedule_is_measured_and_confirmed_by_trial():
    res = run_ranks(_tuned_schedule, (), world=2)
    info = res[0]['info']
    assert 0.0 <= info['interference']['rho'] <= 1.0 and info['interference']['t_alone_ms'] > 0
    assert info['trial'] and all(r['ms_per_step'] > 0 for r in info['trial'])
    assert info['cost_model'] and info['cost_model_overlapped']
    assert res[0]['groups'] == res[1]['groups'] >= 1
    for a, b in zip(res[0]['params'], res[1]['params']):
        assert torch.equal(a, b), 'replicas diverged'


def _scatter_wgrad(rank, world, clip):
    """Weights whose gradient GEMM scatters its tiles to the owner ranks (reduce-scatter epilogue): a two-layer FusedLSTM
    and a large softmax layer, trained against single-process large-batch SGD on the same data."""
    import mgwfbp_b200 as hvd
    from mgwfbp_b200 import settings
    from mgwfbp_b200.ops.lstm import FusedLSTM
    from mgwfbp_b200.ops.wgrad import convert_large_linears
    settings.ADAPTIVE_MERGE = False
    settings.SCATTER_WGRAD = True
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.manual_seed(0)
    T, B, H, V = 5, 4, 1024, 4100                      # weights of 4 Mi elements and more take the scatter path

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.lstm = FusedLSTM(H, H, num_layers=2)
            self.fc = torch.nn.Linear(H, V)

        def forward(self, x):
            out, _ = self.lstm(x)
            return self.fc(out.reshape(-1, H))
    net, ref = Net().cuda(), Net().cuda()
    assert convert_large_linears(net, min_params=4 * 1024 * 1024) == 1
    hvd.broadcast_parameters(net.state_dict(), 0)
    ref.load_state_dict(net.state_dict())
    mk = lambda m: torch.optim.SGD(m.parameters(), lr=0.05, momentum=0.9)
    opt = hvd.DistributedOptimizer(mk(net), named_parameters=net.named_parameters(), threshold=1 << 20,
                                   norm_clip=0.5 if clip else None)
    names = sorted(n for n, _ in opt._scatter)
    assert names == ['fc.weight', 'lstm.weight_hh_l0', 'lstm.weight_hh_l1', 'lstm.weight_ih_l0', 'lstm.weight_ih_l1'], names
    assert not any(n in opt.merge_schedule.key_groupidx for n in names)
    ropt = mk(ref)
    g = torch.Generator().manual_seed(9)
    for _ in range(3):
        x = torch.randn(T, world * B, H, generator=g).cuda() * 0.5
        opt.zero_grad()
        net(x[:, rank * B:(rank + 1) * B].contiguous()).pow(2).mean().backward()
        opt.step()
        ropt.zero_grad()
        ref(x).pow(2).mean().backward()
        if clip:
            torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)
        ropt.step()
    torch.cuda.synchronize()
    opt.communicator.check_status()
    from mgwfbp_b200.ops import wgrad
    wgrad.check_status()
    return {'dp': [p.detach().cpu() for p in net.parameters()], 'ref': [p.detach().cpu() for p in ref.parameters()],
            'grad': net.fc.weight.grad.detach().cpu(), 'ref_grad': ref.fc.weight.grad.detach().cpu(), 'clip': clip}


@pytest.mark.parametrize('clip', [False, True])
def test_scatter_epilogue_wgrad_matches_large_batch_sgd(clip):
    res = run_ranks(_scatter_wgrad, (clip,), world=2)
    # TF32 operands in the gradient GEMM on one side, the library's GEMMs on the other: compare at TF32 accuracy
    for dp, ref in zip(res[0]['dp'], res[0]['ref']):
        rel = float((dp - ref).norm() / ref.norm())
        assert rel < 2e-3, rel
    if not clip:
        rel = float((res[0]['grad'] - res[0]['ref_grad']).norm() / res[0]['ref_grad'].norm())
        assert rel < 2e-2, rel                        # the averaged gradient of the last step sits in p.grad
    for a, b in zip(res[0]['dp'], res[1]['dp']):
        assert torch.equal(a, b), 'replicas diverged'
