"""tcgen05 weight-gradient GEMM: numerics against a plain PyTorch fp32 product."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tf32(t):
    """Round-toward-zero to TF32 (10 explicit mantissa bits), as the tensor cores read fp32 operands."""
    return (t.view(torch.int32) & ~0x1FFF).view(torch.float32)


@pytest.mark.parametrize('K,M,N', [(64, 128, 128), (64, 256, 384), (32, 128, 132), (8, 1000, 2048), (100, 200, 260), (700, 384, 256)])
def test_wgrad_gemm_matches_fp32_reference(K, M, N):
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


def test_wgrad_sgd_epilogue_matches_torch_sgd():
    from mgwfbp_b200.ops import wgrad
    from mgwfbp_b200.ops.tables import HyperTable
    torch.manual_seed(1)
    K, M, N = 64, 256, 512
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
