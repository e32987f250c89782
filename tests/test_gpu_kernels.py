"""Single-GPU numerics of the native kernels against plain PyTorch fp32 references."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope='module')
def lib():
    from mgwfbp_b200.ops import _lib
    return _lib.load(allow_build=False)


def _ref_sgd(params, grads, bufs, lr, wd, momentum, dampening, nesterov, first):
    for p, g, b in zip(params, grads, bufs):
        g = g.clone()
        if wd != 0:
            g = g + wd * p
        if momentum != 0:
            if first:
                b.copy_(g)
            else:
                b.mul_(momentum).add_(g, alpha=1 - dampening)
            g = g + momentum * b if nesterov else b
        p.add_(g, alpha=-lr)


@pytest.mark.parametrize('sizes', [[1], [3, 5, 1000], [4, 64, 1000, 2359296, 7, 513], [1 << 20]])
@pytest.mark.parametrize('momentum,nesterov,wd', [(0.9, False, 1e-4), (0.0, False, 0.0), (0.9, True, 5e-4)])
def test_fast_sgd_matches_torch(sizes, momentum, nesterov, wd):
    import mgwfbp_b200 as hvd
    torch.manual_seed(0)
    dev = torch.device('cuda')
    params = [torch.nn.Parameter(torch.randn(n, device=dev)) for n in sizes]
    ref_params = [torch.nn.Parameter(p.detach().clone()) for p in params]
    half = max(len(params) // 2, 1)
    mk = lambda ps: torch.optim.SGD([{'params': ps[:half], 'weight_decay': 0.0}, {'params': ps[half:], 'weight_decay': wd}]
                                    if len(ps) > 1 else [{'params': ps, 'weight_decay': wd}],
                                    lr=0.1, momentum=momentum, nesterov=nesterov)
    opt = hvd.DistributedOptimizer(mk(params), named_parameters=[('p%d' % i, p) for i, p in enumerate(params)])
    assert getattr(opt, '_fast_sgd', None) is not None, 'native SGD path is not active'
    ref = mk(ref_params)
    for step in range(4):
        for p, r in zip(params, ref_params):
            g = torch.randn_like(p)
            p.grad, r.grad = g.clone(), g.clone()
        for group, rgroup in zip(opt.param_groups, ref.param_groups):
            group['lr'] = rgroup['lr'] = 0.1 / (step + 1)
        opt.step()
        ref.step()
    for p, r in zip(params, ref_params):
        torch.testing.assert_close(p, r, rtol=1e-5, atol=1e-6)
    if momentum:
        for p, r in zip(params, ref_params):
            torch.testing.assert_close(opt.state[p]['momentum_buffer'], ref.state[r]['momentum_buffer'], rtol=1e-5, atol=1e-6)


def test_fast_sgd_global_norm_clip():
    import mgwfbp_b200 as hvd
    torch.manual_seed(1)
    dev = torch.device('cuda')
    sizes = [1000, 33, 70000]
    params = [torch.nn.Parameter(torch.randn(n, device=dev)) for n in sizes]
    ref_params = [torch.nn.Parameter(p.detach().clone()) for p in params]
    opt = hvd.DistributedOptimizer(torch.optim.SGD(params, lr=0.5), named_parameters=[('p%d' % i, p) for i, p in enumerate(params)],
                                   norm_clip=0.25)
    ref = torch.optim.SGD(ref_params, lr=0.5)
    for _ in range(2):
        for p, r in zip(params, ref_params):
            g = torch.randn_like(p)
            p.grad, r.grad = g.clone(), g.clone()
        opt.step()
        total = torch.nn.utils.clip_grad_norm_(ref_params, 0.25)
        ref.step()
        torch.testing.assert_close(opt._fast_sgd.grad_norm(), total, rtol=1e-4, atol=1e-5)
    for p, r in zip(params, ref_params):
        torch.testing.assert_close(p, r, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize('algo', ['oneshot', 'twoshot'])
@pytest.mark.parametrize('numel', [1, 5, 4096, 100003])
def test_allreduce_kernel_single_rank_is_identity(algo, numel):
    """World size 1: the kernel still packs, stages, passes its (self) barriers and writes back."""
    from mgwfbp_b200.parallel.comm.nvl import NvlComm
    comm = NvlComm.shared()
    x = torch.randn(numel, device='cuda')
    want = x.clone()
    h = comm.allreduce_async_(x, average=True, algo=algo)
    comm.synchronize(h)
    torch.cuda.synchronize()
    comm.check_status()
    assert torch.equal(x, want)


def test_fused_update_in_hooks_single_rank():
    """The complete fused path (hooks -> side stream kernel -> in-kernel SGD) on one GPU must equal
    torch.optim.SGD on the same gradients."""
    import mgwfbp_b200 as hvd
    from mgwfbp_b200.parallel.comm.nvl import NvlComm
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(37, 64), torch.nn.ReLU(), torch.nn.Linear(64, 10)).cuda()
    ref = torch.nn.Sequential(torch.nn.Linear(37, 64), torch.nn.ReLU(), torch.nn.Linear(64, 10)).cuda()
    ref.load_state_dict(net.state_dict())
    mk = lambda m: torch.optim.SGD(m.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-3)
    opt = hvd.DistributedOptimizer(mk(net), named_parameters=net.named_parameters(), threshold=3000, comm=NvlComm.shared())
    assert opt._fused_update
    ropt = mk(ref)
    for _ in range(5):
        x = torch.randn(16, 37, device='cuda')
        opt.zero_grad()
        net(x).pow(2).mean().backward()
        opt.step()
        ropt.zero_grad()
        ref(x).pow(2).mean().backward()
        ropt.step()
    torch.cuda.synchronize()
    for a, b in zip(net.parameters(), ref.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    # the averaged gradient stays readable in p.grad
    for a, b in zip(net.parameters(), ref.parameters()):
        torch.testing.assert_close(a.grad, b.grad, rtol=1e-5, atol=1e-7)


def test_bounded_wait_reports_timeout_without_hanging(lib):
    """A flag that nobody sets: the kernel must give up after its limit and report through the
    status block, leaving the context usable."""
    from mgwfbp_b200.ops import _lib
    from mgwfbp_b200.ops.tables import GroupTable
    dev = torch.device('cuda')
    x = torch.ones(1024, device=dev)
    table = GroupTable([x], [0], [None], dev)
    table.refresh_grads([x])
    stage = torch.zeros(4 * 1024 * 4, device=dev)
    flags = torch.zeros(lib.mgw_flag_block_bytes() // 4, dtype=torch.int32, device=dev)
    epoch = torch.zeros(_lib.MAX_CTAS, dtype=torch.int32, device=dev)
    status = C.POINTER(C.c_int)()
    _lib.check(lib.mgw_host_status_alloc(8, C.byref(status)))
    a = _lib.MgwAllreduceArgs()
    a.group = table.struct
    # pretend to be rank 0 of 2; "rank 1" points at the same memory but never signals
    for r in range(2):
        a.stage[r] = stage.data_ptr()
        a.flags[r] = flags.data_ptr()
    a.epoch = epoch.data_ptr()
    a.status = C.cast(status, C.c_void_p).value
    a.rank, a.world, a.algo, a.n_ctas, a.n_threads = 0, 2, _lib.ALGO_TWOSHOT, 1, 128
    a.mode, a.first_step, a.inbox_stride, a.stage_slots = _lib.MODE_WRITEBACK, 0, table.n_vec, table.n_vec
    a.max_pieces, a.piece_slots, a.grad_scale = 1, 4096, 1.0
    a.timeout_ns = 50_000_000        # 50 ms
    _lib.check(lib.mgw_allreduce_group(C.byref(a), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert status[0] == 1 and status[1] == 1, 'timeout on peer 1 expected, got %s' % [status[i] for i in range(5)]
    assert int(epoch[0]) == 1
    y = torch.ones(8, device=dev) * 2          # the context still works
    assert float(y.sum()) == 16.0
    _lib.check(lib.mgw_host_status_free(status))


# ----------------------------------------------------------------------------- BatchNorm + ReLU
def _bn_reference(x, w, b, rm, rv, residual, relu, momentum, eps):
    """Training-mode batch norm (+ residual) (+ ReLU) written out in plain PyTorch operations, evaluated in float64.
    (The library batch norm is not used as the oracle: on the large layers its statistics differ from the exact ones
    by enough to flip the sign of an output that is almost zero, and one flipped ReLU changes a whole channel's
    gamma / beta gradients beyond any sensible tolerance.)"""
    dims = (0,) if x.dim() == 2 else (0, 2, 3)
    shape = (1, -1) + (1,) * (x.dim() - 2)
    xd = x.double()
    mean, var = xd.mean(dims), xd.var(dims, unbiased=False)
    n = x.numel() // x.shape[1]
    with torch.no_grad():
        rm.mul_(1 - momentum).add_(momentum * mean.float())
        rv.mul_(1 - momentum).add_(momentum * (var * n / max(n - 1, 1)).float())
    y = (xd - mean.view(shape)) / torch.sqrt(var.view(shape) + eps) * w.double().view(shape) + b.double().view(shape)
    if residual is not None:
        y = y + residual.double()
    return (torch.relu(y) if relu else y).float()


# small shapes take the one-launch cluster kernels (up to 8 register rows per thread), the others the
# three-launch kernels; `cluster=False` forces the three-launch kernels on the small shapes as well
@pytest.mark.parametrize('shape', [(4, 64, 14, 14), (3, 16, 8, 8), (2, 6, 5, 7), (8, 256, 7, 7), (64, 96), (16, 128, 14, 14),
                                   (24, 32, 14, 14), (64, 48, 14, 14), (21, 32, 28, 28), (8, 64, 56, 56),
                                   # ResNet-50's small stages at batch 64 (finalize fused into the reduction kernels) and
                                   # one problem with more row splits than the fused finalize takes (separate kernel)
                                   (64, 256, 14, 14), (64, 1024, 14, 14), (64, 2048, 7, 7), (32, 64, 56, 56)])
@pytest.mark.parametrize('relu,use_res', [(True, False), (True, True), (False, False)])
@pytest.mark.parametrize('cluster', [True, False])
def test_bn_relu_matches_pytorch(shape, relu, use_res, cluster, monkeypatch):
    from mgwfbp_b200.ops import bn_relu as bn_module, counters
    from mgwfbp_b200.ops.bn_relu import bn_relu
    monkeypatch.setattr(bn_module, '_CLUSTER', cluster)
    counters.reset()
    torch.manual_seed(0)
    dev = torch.device('cuda')
    C_ = shape[1]
    fmt = torch.channels_last if len(shape) == 4 else torch.contiguous_format
    x = (torch.randn(shape, device=dev) * 2 + 0.5).contiguous(memory_format=fmt).requires_grad_(True)
    res = torch.randn(shape, device=dev).contiguous(memory_format=fmt).requires_grad_(True) if use_res else None
    w = (torch.rand(C_, device=dev) + 0.5).requires_grad_(True)
    b = torch.randn(C_, device=dev).requires_grad_(True)
    rm, rv, nbt = torch.zeros(C_, device=dev), torch.ones(C_, device=dev), torch.zeros((), dtype=torch.long, device=dev)
    x2, w2, b2 = x.detach().clone().requires_grad_(True), w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    res2 = res.detach().clone().requires_grad_(True) if use_res else None
    rm2, rv2 = rm.clone(), rv.clone()
    y = bn_relu(x, w, b, rm, rv, nbt, res, relu, 0.1, 1e-5)
    y2 = _bn_reference(x2, w2, b2, rm2, rv2, res2, relu, 0.1, 1e-5)
    torch.testing.assert_close(y, y2, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(rm, rm2, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(rv, rv2, rtol=1e-4, atol=1e-5)
    assert int(nbt) == 1
    dy = torch.randn_like(y)
    y.backward(dy)
    y2.backward(dy)
    torch.testing.assert_close(x.grad, x2.grad, rtol=1e-3, atol=2e-4)
    torch.testing.assert_close(w.grad, w2.grad, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(b.grad, b2.grad, rtol=1e-3, atol=1e-3)
    if use_res:
        torch.testing.assert_close(res.grad, res2.grad, rtol=1e-4, atol=1e-5)
    rows = x.numel() // C_
    took_cluster = counters.snapshot().get('bn_relu_fwd_cluster', 0) == 1 and counters.snapshot().get('bn_relu_bwd_cluster', 0) == 1
    assert took_cluster == (cluster and rows <= 8192 and C_ % 16 == 0 and C_ <= 288)
    if not took_cluster:
        # two launches per direction where the last block finalizes, three where a separate kernel does
        from mgwfbp_b200.ops import _lib
        lib = _lib.load(allow_build=False)
        want = lib.mgw_bn_launches(rows, C_, 0), lib.mgw_bn_launches(rows, C_, 1)
        assert (counters.snapshot().get('bn_relu_fwd'), counters.snapshot().get('bn_relu_bwd')) == want
        assert set(want) <= {2, 3}
    # a second pass over the same tensors: the arrival counters went back to zero, results repeat exactly
    x3 = x.detach().clone().requires_grad_(True)
    y3 = bn_relu(x3, w.detach(), b.detach(), rm.clone(), rv.clone(), nbt.clone(), res.detach() if use_res else None, relu, 0.1, 1e-5)
    assert torch.equal(y3, y)


@pytest.mark.parametrize('dnn,shape,classes', [('resnet20', (8, 3, 32, 32), 10), ('resnet50', (4, 3, 64, 64), 1000)])
def test_fused_model_matches_unfused(dnn, shape, classes):
    from mgwfbp_b200.models import create_net
    torch.manual_seed(0)
    a, _ = create_net(classes, dnn)
    b, _ = create_net(classes, dnn, fuse=True, channels_last=True)
    b.load_state_dict(a.state_dict())
    a, b = a.cuda(), b.cuda()
    x = torch.randn(shape, device='cuda')
    prev = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False      # fp32 convolutions on both sides: only the fused modules differ
    try:
        ya, yb = a(x), b(x.contiguous(memory_format=torch.channels_last))
        torch.testing.assert_close(yb, ya, rtol=1e-3, atol=1e-3)
        ya.square().mean().backward()
        yb.square().mean().backward()
    finally:
        torch.backends.cudnn.allow_tf32 = prev
    ga = torch.cat([p.grad.reshape(-1) for p in a.parameters()])
    gb = torch.cat([p.grad.reshape(-1) for p in b.parameters()])
    assert torch.nn.functional.cosine_similarity(ga, gb, dim=0) > 0.99
    for (k, va), vb in zip(a.state_dict().items(), b.state_dict().values()):
        if 'running_' in k or 'num_batches' in k:
            torch.testing.assert_close(vb, va, rtol=1e-2, atol=1e-2)


# ----------------------------------------------------------------------------- LSTM
@pytest.mark.parametrize('chunk,H', [(0, 64), (3, 64), (3, 30)])       # H = 30: the scalar cell kernels (H % 4 != 0)
def test_fused_lstm_matches_cudnn_lstm(chunk, H, monkeypatch):
    from mgwfbp_b200.ops import lstm as lstm_ops
    from mgwfbp_b200.ops.lstm import FusedLSTM
    monkeypatch.setattr(lstm_ops, '_CHUNK', chunk)
    torch.manual_seed(0)
    T, B, I = 7, 5, 48
    ref = torch.nn.LSTM(I, H, 2).cuda()
    mine = FusedLSTM(I, H, 2).cuda()
    mine.load_state_dict(ref.state_dict())
    x = torch.randn(T, B, I, device='cuda')
    hx = (torch.randn(2, B, H, device='cuda'), torch.randn(2, B, H, device='cuda'))
    x1, x2 = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    prev, prev_cudnn = torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False      # fp32 GEMMs on both sides (cuDNN's LSTM obeys the cudnn flag)
    torch.backends.cudnn.allow_tf32 = False
    try:
        y1, (h1, c1) = ref(x1, hx)
        y2, (h2, c2) = mine(x2, hx)
        torch.testing.assert_close(y2, y1, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(h2, h1, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(c2, c1, rtol=1e-4, atol=1e-5)
        w = torch.randn_like(y1)
        (y1 * w).sum().backward()
        (y2 * w).sum().backward()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
        torch.backends.cudnn.allow_tf32 = prev_cudnn
    torch.testing.assert_close(x2.grad, x1.grad, rtol=1e-3, atol=1e-4)
    for (n, p1), p2 in zip(ref.named_parameters(), mine.parameters()):
        torch.testing.assert_close(p2.grad, p1.grad, rtol=1e-3, atol=1e-4, msg=lambda m: '%s: %s' % (n, m))


def _tf32(t):
    return (t.view(torch.int32) & ~0x1FFF).view(torch.float32)


@pytest.mark.parametrize('B,R,K', [(20, 6000, 1500), (20, 1500, 6000), (5, 256, 64), (64, 100, 388), (1, 16, 4), (33, 70, 1000)])
def test_lstm_recurrent_gemm_matches_fp32_product(B, R, K):
    """The small-batch recurrent product: split-K partial sums of x W^T with TF32 operands, fp32 accumulation."""
    from mgwfbp_b200.ops import _lib
    from mgwfbp_b200.ops import lstm as lstm_ops
    lib = _lib.load(allow_build=False)
    lstm_ops._declare(lib)
    torch.manual_seed(0)
    x, w = torch.randn(B, K, device='cuda'), torch.randn(R, K, device='cuda') / K ** 0.5
    assert lib.mgw_lstm_rec_supported(x.data_ptr(), w.data_ptr(), B, R, K)
    parts = lib.mgw_lstm_rec_splits(K)
    assert parts == (K + 383) // 384
    out = torch.full((parts, B, R), float('nan'), device='cuda')
    _lib.check(lib.mgw_lstm_rec_gemm(x.data_ptr(), w.data_ptr(), out.data_ptr(), B, R, K, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    got = out.sum(0)
    want = (x.double() @ w.double().t()).float()
    # operands are rounded to TF32 (10 mantissa bits): about 1e-3 relative per product, averaging out over K
    torch.testing.assert_close(got, want, rtol=5e-3, atol=5e-3)
    for p in range(parts):                                   # every partial is the product over its own K-range
        k0, k1 = p * 384, min(K, (p + 1) * 384)
        part = (x[:, k0:k1].double() @ w[:, k0:k1].double().t()).float()
        torch.testing.assert_close(out[p], part, rtol=5e-3, atol=5e-3)


@pytest.mark.parametrize('chunk', [0, 2, 7])
def test_fused_lstm_with_own_recurrent_kernel_tracks_library_lstm(chunk, monkeypatch):
    """TF32 allowed on both sides: the package's recurrent kernel is on the path (launch counter) and the layer stays
    within TF32 accuracy of torch.nn.LSTM, forward and backward, with the PTB model's awkward sizes; layers run one
    after the other (chunk 0) or as a wavefront over chunks of time steps on two streams."""
    from mgwfbp_b200.ops import counters
    from mgwfbp_b200.ops import lstm as lstm_ops
    from mgwfbp_b200.ops.lstm import FusedLSTM
    monkeypatch.setattr(lstm_ops, '_OWN_REC', True)
    monkeypatch.setattr(lstm_ops, '_CHUNK', chunk)
    torch.manual_seed(0)
    T, B, I, H = 6, 20, 100, 300
    ref = torch.nn.LSTM(I, H, 2).cuda()
    mine = FusedLSTM(I, H, 2).cuda()
    mine.load_state_dict(ref.state_dict())
    x = torch.randn(T, B, I, device='cuda')
    hx = (torch.randn(2, B, H, device='cuda'), torch.randn(2, B, H, device='cuda'))
    x1, x2 = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    counters.reset()
    try:
        y1, (h1, c1) = ref(x1, hx)
        y2, (h2, c2) = mine(x2, hx)
        w = torch.randn_like(y1)
        (y1 * w).sum().backward()
        (y2 * w).sum().backward()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    assert counters.snapshot().get('lstm_rec_gemm', 0) == 2 * 2 * T          # two layers, forward and backward
    torch.testing.assert_close(y2, y1, rtol=2e-2, atol=5e-3)
    torch.testing.assert_close(c2, c1, rtol=2e-2, atol=5e-3)
    torch.testing.assert_close(x2.grad, x1.grad, rtol=5e-2, atol=2e-2)
    for (n, p1), p2 in zip(ref.named_parameters(), mine.parameters()):
        rel = float((p2.grad - p1.grad).norm() / p1.grad.norm())
        assert rel < 2e-2, '%s: relative gradient error %.4f' % (n, rel)


def test_bn_relu_dual_output_sums_both_gradients():
    """A block output feeding two consumers: both gradients reach the backward kernel and are summed there."""
    from mgwfbp_b200.ops.bn_relu import bn_relu
    torch.manual_seed(0)
    dev = torch.device('cuda')
    shape, C_ = (4, 32, 6, 6), 32
    mk = lambda: (torch.randn(shape, device=dev)).contiguous(memory_format=torch.channels_last)
    x, res = mk().requires_grad_(True), mk().requires_grad_(True)
    w = (torch.rand(C_, device=dev) + 0.5).requires_grad_(True)
    b = torch.randn(C_, device=dev).requires_grad_(True)
    x2, res2, w2, b2 = (t.detach().clone().requires_grad_(True) for t in (x, res, w, b))
    stats = lambda: (torch.zeros(C_, device=dev), torch.ones(C_, device=dev), torch.zeros((), dtype=torch.long, device=dev))
    y_a, y_b = bn_relu(x, w, b, *stats(), res, True, 0.1, 1e-5, dual=True)
    assert y_a.data_ptr() == y_b.data_ptr()
    ref = _bn_reference(x2, w2, b2, *stats()[:2], res2, True, 0.1, 1e-5)
    ga, gb = torch.randn_like(y_a), torch.randn_like(y_a)
    ((y_a * ga).sum() + (y_b * gb).sum()).backward()
    (ref * (ga + gb)).sum().backward()
    torch.testing.assert_close(x.grad, x2.grad, rtol=1e-3, atol=2e-4)
    torch.testing.assert_close(res.grad, res2.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(w.grad, w2.grad, rtol=1e-3, atol=1e-3)
    # only one of the two handles used
    x.grad = res.grad = None
    y_a, y_b = bn_relu(x, w, b, *stats(), res, True, 0.1, 1e-5, dual=True)
    (y_b * gb).sum().backward()
    x2.grad = res2.grad = None
    (_bn_reference(x2, w2, b2, *stats()[:2], res2, True, 0.1, 1e-5) * gb).sum().backward()
    torch.testing.assert_close(x.grad, x2.grad, rtol=1e-3, atol=2e-4)


@pytest.mark.parametrize('shape', [(2, 16, 12, 12), (3, 64, 17, 15), (2, 8, 7, 9)])
def test_bn_relu_maxpool_stem_matches_pytorch(shape):
    from mgwfbp_b200.ops.bn_relu import FusedBatchNorm2d, bn_relu_maxpool
    torch.manual_seed(0)
    dev = torch.device('cuda')
    C_ = shape[1]
    bn = FusedBatchNorm2d(C_).to(dev)
    bn.fused_relu = True
    ref = torch.nn.BatchNorm2d(C_).to(dev)
    with torch.no_grad():
        bn.weight.uniform_(0.5, 1.5)
        bn.bias.normal_()
    ref.load_state_dict(bn.state_dict())
    pool = torch.nn.MaxPool2d(3, 2, 1)
    x = torch.randn(shape, device=dev).contiguous(memory_format=torch.channels_last).requires_grad_(True)
    x2 = x.detach().clone().requires_grad_(True)
    y = bn_relu_maxpool(bn, pool, x)
    y2 = pool(torch.relu(ref(x2)))
    torch.testing.assert_close(y, y2, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(bn.running_var, ref.running_var, rtol=1e-4, atol=1e-5)
    g = torch.randn_like(y2)
    y.backward(g)
    y2.backward(g)
    torch.testing.assert_close(x.grad, x2.grad, rtol=1e-3, atol=2e-4)
    torch.testing.assert_close(bn.weight.grad, ref.weight.grad, rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(bn.bias.grad, ref.bias.grad, rtol=1e-3, atol=1e-3)


# ----------------------------------------------------------------------------- stem convolution
def test_s2d_stem_matches_conv2d():
    """The 7x7/2 stem as a 4x4 convolution over the space-to-depth input: rearrangement kernel against tensor ops,
    forward and weight gradient against ``nn.Conv2d`` in full fp32."""
    from mgwfbp_b200.ops.stem import S2DStemConv2d, convert_stem, s2d_input, s2d_input_reference
    torch.manual_seed(0)
    old = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        for shape in [(4, 3, 64, 64), (2, 3, 224, 224), (3, 3, 32, 96)]:
            x = torch.randn(*shape, device='cuda').contiguous(memory_format=torch.channels_last)
            assert torch.equal(s2d_input(x), s2d_input_reference(x))
            ref = torch.nn.Conv2d(3, 16, 7, stride=2, padding=3, bias=False).cuda()
            new = convert_stem(ref)
            assert isinstance(new, S2DStemConv2d) and new.weight is ref.weight
            assert list(new.state_dict().keys()) == ['weight']
            y_ref = torch.nn.functional.conv2d(x, ref.weight, None, 2, 3)
            y_new = new(x)
            assert y_new.shape == y_ref.shape
            torch.testing.assert_close(y_new, y_ref, rtol=1e-4, atol=1e-4)
            dy = torch.randn_like(y_ref)
            g_ref, = torch.autograd.grad(y_ref, ref.weight, dy)
            g_new, = torch.autograd.grad(y_new, new.weight, dy)
            torch.testing.assert_close(g_new, g_ref, rtol=1e-4, atol=1e-3)
        # anything that is not the ImageNet stem is left alone, and odd sizes fall back to the parent
        other = torch.nn.Conv2d(3, 8, 3, padding=1)
        assert convert_stem(other) is other
        odd = torch.randn(2, 3, 33, 33, device='cuda').contiguous(memory_format=torch.channels_last)
        torch.testing.assert_close(new(odd), torch.nn.functional.conv2d(odd, ref.weight, None, 2, 3), rtol=1e-4, atol=1e-4)
    finally:
        torch.backends.cudnn.allow_tf32 = old


@pytest.mark.parametrize('wide,c,shape', [(96, 64, (8, 14, 14)), (1792, 1024, (4, 7, 7)), (100, 30, (3, 5, 6)), (224, 192, (16, 28, 28))])
@pytest.mark.parametrize('relu', [True, False])
def test_bn_relu_reads_a_channel_slice_in_place(wide, c, shape, relu, monkeypatch):
    """x = first ``c`` channels of a ``wide``-channel channels-last tensor (a DenseNet block buffer): the kernels read it
    through its row stride.  Same kernels, same order of arithmetic as on a dense copy of the slice: results are equal
    bit for bit, and the reference in plain PyTorch double precision agrees."""
    from mgwfbp_b200.ops import bn_relu as bn_mod
    from mgwfbp_b200.ops.bn_relu import bn_relu
    monkeypatch.setattr(bn_mod, '_CLUSTER', False)           # the dense copy must take the same three-launch kernels
    torch.manual_seed(0)
    dev = torch.device('cuda')
    n, h, w_ = shape
    buf = torch.randn(n, wide, h, w_, device=dev).contiguous(memory_format=torch.channels_last)
    xs = buf[:, :c].detach().requires_grad_(True)
    assert not xs.is_contiguous(memory_format=torch.channels_last)
    xd = buf[:, :c].detach().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    w1 = (torch.rand(c, device=dev) + 0.5).requires_grad_(True)
    b1 = torch.randn(c, device=dev).requires_grad_(True)
    w2, b2 = (t.detach().clone().requires_grad_(True) for t in (w1, b1))
    stats = lambda: (torch.zeros(c, device=dev), torch.ones(c, device=dev), torch.zeros((), dtype=torch.long, device=dev))
    s1, s2 = stats(), stats()
    before = buf.clone()
    y1 = bn_relu(xs, w1, b1, *s1, None, relu, 0.1, 1e-5)
    y2 = bn_relu(xd, w2, b2, *s2, None, relu, 0.1, 1e-5)
    assert y1.is_contiguous(memory_format=torch.channels_last)
    g = torch.randn_like(y2)
    (y1 * g).sum().backward()
    (y2 * g).sum().backward()
    torch.cuda.synchronize()
    assert torch.equal(buf, before)                          # nothing was written through the view
    assert torch.equal(y1, y2) and torch.equal(s1[0], s2[0]) and torch.equal(s1[1], s2[1])
    assert torch.equal(xs.grad, xd.grad) and torch.equal(w1.grad, w2.grad) and torch.equal(b1.grad, b2.grad)
    # the same backward adding its input gradient into a wider gradient buffer (a dense block's) instead of returning it
    xa = buf[:, :c].detach().requires_grad_(True)
    gwide = torch.randn(n, wide, h, w_, device=dev).contiguous(memory_format=torch.channels_last)
    before_g = gwide.clone()
    xa._mgw_grad_cell = {'target': gwide[:, :c]}
    wa, ba = (t.detach().clone().requires_grad_(True) for t in (w1, b1))
    ya = bn_relu(xa, wa, ba, *stats(), None, relu, 0.1, 1e-5)
    (ya * g).sum().backward()
    torch.cuda.synchronize()
    assert xa.grad is None
    assert torch.equal(gwide[:, :c], before_g[:, :c] + xd.grad) and torch.equal(gwide[:, c:], before_g[:, c:])
    assert torch.equal(wa.grad, w2.grad) and torch.equal(ba.grad, b2.grad)
    x3 = xd.detach().clone().requires_grad_(True)
    w3, b3 = (t.detach().clone().requires_grad_(True) for t in (w1, b1))
    ref = _bn_reference(x3, w3, b3, *stats()[:2], None, relu, 0.1, 1e-5)
    (ref * g).sum().backward()
    torch.testing.assert_close(y1, ref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(xs.grad, x3.grad, rtol=1e-3, atol=2e-4)


def test_dense_block_single_buffer_matches_plain_blocks_on_gpu(monkeypatch):
    """A small torchvision DenseNet with the package's fused modules: the single-buffer dense blocks (strided BatchNorm
    input, one gradient addition per layer) against the same network on the list-and-concatenate path."""
    import copy
    tvd = pytest.importorskip('torchvision.models.densenet')
    from mgwfbp_b200.models import dense_block
    from mgwfbp_b200.models.fuse import fuse_model
    from mgwfbp_b200.ops import bn_relu as bn_mod, counters
    monkeypatch.setattr(bn_mod, '_CLUSTER', False)      # both networks on the three-launch BatchNorm kernels
    torch.manual_seed(0)
    net = tvd.DenseNet(growth_rate=16, block_config=(3, 4, 3), num_init_features=32, bn_size=2, num_classes=10)
    a = fuse_model(copy.deepcopy(net)).cuda().to(memory_format=torch.channels_last).train()
    b = fuse_model(copy.deepcopy(net)).cuda().to(memory_format=torch.channels_last).train()
    for m in b.modules():
        if isinstance(m, tvd._DenseBlock):
            m.forward = dense_block._plain_forward.__get__(m)
    x = torch.randn(8, 3, 64, 64, device='cuda').contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 10, (8,), device='cuda')
    counters.reset()
    prev = torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32
    torch.backends.cudnn.allow_tf32 = torch.backends.cuda.matmul.allow_tf32 = False     # fp32 convolutions: the two paths may
    try:                                                                                 # pick different library algorithms
        la = torch.nn.functional.cross_entropy(a(x), y)
        la.backward()
        assert counters.snapshot().get('bn_relu_fwd', 0) > 0
        lb = torch.nn.functional.cross_entropy(b(x), y)
        lb.backward()
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = prev
    torch.testing.assert_close(la, lb, rtol=1e-5, atol=1e-5)
    rels = []
    for (n, p), q in zip(a.named_parameters(), b.parameters()):
        assert p.grad is not None, n
        rels.append((float((p.grad - q.grad).norm() / (q.grad.norm() + 1e-12)), n))
    # The two paths add the same gradient contributions in different orders and may run different library convolution
    # algorithms, and a ReLU or max-pool decision that flips on a last-bit difference changes everything in front of it:
    # the stem's BatchNorm weight (last in backward) differed by 3e-2 on one run while the loss agreed to 1e-5.  So: no
    # parameter far off, and nearly all of them close.
    rels.sort()
    assert rels[-1][0] < 1e-1, 'relative gradient difference %.2e at %s' % rels[-1]
    assert rels[int(0.8 * len(rels))][0] < 5e-3, 'relative gradient difference %.2e at %s (80th percentile)' % rels[int(0.8 * len(rels))]
    for (n, p), q in zip(a.named_buffers(), b.buffers()):
        torch.testing.assert_close(p.float(), q.float(), rtol=1e-4, atol=1e-5, msg=lambda m, n=n: '%s: %s' % (n, m))
