"""The allocation-free norm / clip-coefficient entry point, called through its exported C symbol.

Some hosts of this library may not allocate device memory when they need the gradient norm (a fixed
amount of memory, or a section where an allocation could stall the GPU).  For them the library keeps the
partial sums in a small built-in array.  This test checks that variant against the regular entry points,
which take a caller-allocated buffer, on two calls in a row with different data (the shared array keeps
the previous call's contents, which must not leak into the next result).
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _loaded_path():
    """The image that ``_lib.load()`` mapped (the index-checking build when ``MGWFBP_CHECKED=1``): opening the same
    file again yields the same image, so the error text read through one handle belongs to the call made through the other."""
    from mgwfbp_b200.ops import _lib
    from mgwfbp_b200.ops.build import CHECKED_LIB_PATH, LIB_PATH
    return CHECKED_LIB_PATH if _lib.is_checked() else LIB_PATH


def _norm_both_ways(lib, clib, table, grads, n_ctas, max_norm):
    from mgwfbp_b200.ops import _lib
    dev = grads[0].device
    s = torch.cuda.current_stream().cuda_stream
    table.refresh_grads(grads)
    partials = torch.empty(n_ctas, dtype=torch.float32, device=dev)           # caller-allocated scratch
    want = torch.zeros(2, dtype=torch.float32, device=dev)
    _lib.check(lib.mgw_group_sumsq(C.byref(table.struct), partials.data_ptr(), n_ctas, s))
    _lib.check(lib.mgw_clip_coef(partials.data_ptr(), n_ctas, max_norm, want.data_ptr(), s))
    got = torch.zeros(2, dtype=torch.float32, device=dev)                     # output buffer belongs to the caller
    rc = clib.mgw_grad_clip_coef_static(C.byref(table.struct), C.c_float(max_norm), C.c_void_p(got.data_ptr()),
                                        C.c_int(n_ctas), C.c_void_p(s))
    assert rc == 0, lib.mgw_last_error()
    torch.cuda.synchronize()
    return got, want


def test_static_scratch_variant_matches_regular_entry_points():
    from mgwfbp_b200.ops import _lib
    from mgwfbp_b200.ops.tables import GroupTable
    lib = _lib.load(allow_build=False)
    clib = C.CDLL(_loaded_path())                         # the plain exported symbol, no Python wrapper in between
    clib.mgw_grad_clip_coef_static.restype = C.c_int
    dev = torch.device('cuda')
    torch.manual_seed(0)
    sizes = [1000, 33, 70001, 4, 262144]
    params = [torch.zeros(n, device=dev) for n in sizes]
    table = GroupTable(params, [0] * len(params), [None] * len(params), dev)
    n_ctas = 37
    for call, scale in enumerate((1.0, 0.01)):            # second call: much smaller gradients, same scratch
        grads = [torch.randn(n, device=dev) * scale for n in sizes]
        got, want = _norm_both_ways(lib, clib, table, grads, n_ctas, max_norm=0.25)
        torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
        ref = torch.sqrt(sum((g.double() ** 2).sum() for g in grads)).float()
        torch.testing.assert_close(got[0], ref, rtol=1e-4, atol=1e-5)
        assert float(got[1]) == pytest.approx(min(1.0, 0.25 / (float(ref) + 1e-6)), rel=1e-4)


def test_static_scratch_variant_rejects_oversized_requests():
    from mgwfbp_b200.ops import _lib
    from mgwfbp_b200.ops.tables import GroupTable
    lib = _lib.load(allow_build=False)
    clib = C.CDLL(_loaded_path())
    clib.mgw_grad_clip_coef_static.restype = C.c_int
    dev = torch.device('cuda')
    x = torch.ones(64, device=dev)
    table = GroupTable([x], [0], [None], dev)
    table.refresh_grads([x])
    out = torch.zeros(2, device=dev)
    rc = clib.mgw_grad_clip_coef_static(C.byref(table.struct), C.c_float(1.0), C.c_void_p(out.data_ptr()), C.c_int(1025),
                                        C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 3
    assert b'exceeds the built-in scratch' in lib.mgw_last_error()
