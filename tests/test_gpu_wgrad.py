"""tcgen05 weight-gradient GEMM: numerics against a plain PyTorch fp32 product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tf32(t):
    """Round-toward-zero to TF32 (10 explicit mantissa bits), as the tensor cores read fp32 operands."""
    return (t.view(torch.int32) & ~0x1FFF).view(torch.float32)


@pytest.fixture(params=['persistent16', 'persistent8x2', 'tile'])
def kernel_form(request):
    """The forms of the GEMM kernel: CTAs that walk over the tiles (one of 16 epilogue warps, or two of 8, per SM), and
    one tile per CTA."""
    from mgwfbp_b200.ops import wgrad
    wgrad.set_persistent({'persistent16': 1, 'persistent8x2': 2, 'tile': 0}[request.param])
    yield request.param
    wgrad.set_persistent(None)


# (64, 2048, 2560) and (40, 1536, 2052) have more tiles than the GPU has SMs: persistent CTAs take several tiles each,
# through both accumulator halves and around the operand ring
@pytest.mark.parametrize('K,M,N', [(64, 128, 128), (64, 256, 384), (32, 128, 132), (8, 1000, 2048), (100, 200, 260), (700, 384, 256),
                                   (64, 2048, 2560), (40, 1536, 2052), (300, 1280, 1664)])
def test_wgrad_gemm_matches_fp32_reference(K, M, N, kernel_form):
    from mgwfbp_b200.ops import wgrad
    torch.manual_seed(0)
    dy = torch.randn(K, M, device='cuda')
    x = torch.randn(K, N, device='cuda')
    got = wgrad.wgrad_gemm(dy, x, scale=0.5)
    torch.cuda.synchronize()
    wgrad.check_status()
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        want_exact_inputs = 0.5 * (_tf32(dy).double().t() @ _tf32(x).double()).float()
        want_fp32 = 0.5 * (dy.t() @ x)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    # against the product of TF32-truncated inputs only accumulation order differs
    torch.testing.assert_close(got, want_exact_inputs, rtol=1e-4, atol=1e-3)
    # against the full-precision product the TF32 input rounding shows (about 1e-3 relative)
    torch.testing.assert_close(got, want_fp32, rtol=2e-2, atol=2e-2 * (K ** 0.5))


@pytest.mark.parametrize('K,M,N', [(64, 256, 512), (64, 1920, 2304)])
def test_wgrad_sgd_epilogue_matches_torch_sgd(K, M, N, kernel_form):
    from mgwfbp_b200.ops import wgrad
    from mgwfbp_b200.ops.tables import HyperTable
    torch.manual_seed(1)
    dev = torch.device('cuda')
    w = torch.nn.Parameter(torch.randn(M, N, device=dev))
    ref = torch.nn.Parameter(w.detach().clone())
    mom = torch.zeros_like(w)
    opt = torch.optim.SGD([ref], lr=0.1, momentum=0.9, weight_decay=1e-3)
    hyper = HyperTable(dev)
    hyper.sync(opt.param_groups)
    grad_out = torch.empty(M, N, device=dev)
    for step in range(3):
        dy, x = _tf32(torch.randn(K, M, device=dev)), _tf32(torch.randn(K, N, device=dev))
        wgrad.wgrad_sgd_(dy, x, w.data, mom, hyper.data_ptr(), 0, scale=0.125, first_step=(step == 0), grad_out=grad_out)
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        ref.grad = 0.125 * (dy.t() @ x)
        torch.backends.cuda.matmul.allow_tf32 = prev
        opt.step()
        torch.testing.assert_close(grad_out, ref.grad, rtol=1e-4, atol=1e-3)
    torch.cuda.synchronize()
    wgrad.check_status()
    torch.testing.assert_close(w.data, ref.data, rtol=1e-4, atol=1e-3)
    torch.testing.assert_close(mom, opt.state[ref]['momentum_buffer'], rtol=1e-4, atol=1e-3)


def test_single_gpu_linear_updates_through_the_gemm_epilogue():
    """One process, one GPU: a large linear layer under DistributedOptimizer gets no .grad; its backward applies the
    momentum-SGD update from the GEMM epilogue.  Result equals torch.optim.SGD on a copy (TF32 operands on both sides)."""
    import copy
    from mgwfbp_b200.ops import wgrad
    from mgwfbp_b200.parallel.optimizer import DistributedOptimizer
    torch.manual_seed(2)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        net = torch.nn.Sequential(torch.nn.Linear(96, 1024), torch.nn.ReLU(), torch.nn.Linear(1024, 1536), torch.nn.ReLU(),
                                  torch.nn.Linear(1536, 10)).cuda()
        ref = copy.deepcopy(net)
        assert wgrad.convert_large_linears(net, min_params=1024 * 1024) == 1
        for m in net.modules():
            if hasattr(m, 'batch_rows_hint'):
                m.batch_rows_hint = 32
        opt = DistributedOptimizer(torch.optim.SGD(net.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-3),
                                   named_parameters=net.named_parameters())
        assert opt._fast_sgd is not None and opt._fast_sgd.external_layers == 1
        ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-3)
        for step in range(4):
            if step == 2:
                for g in list(opt.param_groups) + list(ref_opt.param_groups):
                    g['lr'] = 0.02                      # a schedule moves the rate: the layer's update must follow
            x = torch.randn(32, 96, device='cuda')
            y = torch.randint(0, 10, (32,), device='cuda')
            for n_, o_ in ((net, opt), (ref, ref_opt)):
                o_.zero_grad()
                torch.nn.functional.cross_entropy(n_(x), y).backward()
                o_.step()
            assert net[2].weight.grad is None
        torch.cuda.synchronize()
        wgrad.check_status()
        for (name, a), b in zip(net.named_parameters(), ref.parameters()):
            torch.testing.assert_close(a, b, rtol=2e-3, atol=2e-4, msg=lambda m, name=name: '%s: %s' % (name, m))
        # accumulating gradients hands the layer back to autograd
        opt.local = True
        assert opt._fast_sgd.external_layers == 0
        torch.nn.functional.cross_entropy(net(x), y).backward()
        assert net[2].weight.grad is not None
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
