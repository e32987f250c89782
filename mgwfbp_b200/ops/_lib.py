# -*- coding: utf-8 -*-
"""ctypes binding of ``libmgwfbp_b200.so`` (the package's CUDA kernels and symmetric heap).

The library is built in-tree by :mod:`mgwfbp_b200.ops.build`.  On a machine with a GPU a missing
library is an error (operations never fall back silently to eager PyTorch); without a GPU the
loader may build it on demand so that import-time checks still work.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

from .build import CHECKED_LIB_PATH, LIB_PATH, build  # noqa: F401  (re-exported)

MAX_RANKS = 16
MAX_CTAS = 296
MAX_PARAM_GROUPS = 16

MODE_UPDATE, MODE_WRITEBACK, MODE_SUMSQ = 1, 2, 4
ALGO_ONESHOT, ALGO_TWOSHOT, ALGO_NVLS = 0, 1, 2
ALGO_NAMES = {'oneshot': ALGO_ONESHOT, 'twoshot': ALGO_TWOSHOT, 'nvls': ALGO_NVLS}


class MgwGroup(C.Structure):
    _fields_ = [('tensors', C.c_void_p), ('grads', C.c_void_p), ('voff', C.c_void_p),
                ('n_tensors', C.c_int), ('n_vec', C.c_int)]


class MgwAllreduceArgs(C.Structure):
    _fields_ = [('group', MgwGroup),
                ('stage', C.c_void_p * MAX_RANKS),
                ('flags', C.c_void_p * MAX_RANKS),
                ('epoch', C.c_void_p),
                ('mc_stage', C.c_void_p),
                ('hyper', C.c_void_p),
                ('sumsq_partials', C.c_void_p),
                ('status', C.c_void_p),
                ('rank', C.c_int), ('world', C.c_int),
                ('algo', C.c_int), ('n_ctas', C.c_int), ('n_threads', C.c_int),
                ('mode', C.c_int), ('first_step', C.c_int),
                ('inbox_stride', C.c_int), ('stage_slots', C.c_int),
                ('max_pieces', C.c_int), ('piece_slots', C.c_int), ('grad_scale', C.c_float), ('skip_pack', C.c_int),
                ('timeout_ns', C.c_ulonglong)]


_lib: Optional[C.CDLL] = None


class NativeLibraryError(RuntimeError):
    pass


def _declare(lib: C.CDLL) -> None:
    lib.mgw_last_error.restype = C.c_char_p
    lib.mgw_version.restype = C.c_int
    lib.mgw_heap_create.argtypes = [C.c_size_t, C.POINTER(C.c_void_p)]
    lib.mgw_heap_export.argtypes = [C.c_void_p, C.c_void_p]
    lib.mgw_heap_open.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    lib.mgw_heap_close.argtypes = [C.c_void_p]
    lib.mgw_heap_destroy.argtypes = [C.c_void_p]
    lib.mgw_vmm_supported.argtypes = [C.POINTER(C.c_int)]
    lib.mgw_vmm_create.argtypes = [C.c_size_t, C.c_int, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]
    lib.mgw_vmm_export_fd.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
    lib.mgw_vmm_import_peer.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]
    lib.mgw_vmm_mc_create.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int)]
    lib.mgw_vmm_mc_import.argtypes = [C.c_void_p, C.c_int]
    lib.mgw_vmm_mc_add_device.argtypes = [C.c_void_p]
    lib.mgw_vmm_mc_bind.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    lib.mgw_vmm_destroy.argtypes = [C.c_void_p, C.c_int]
    lib.mgw_host_status_alloc.argtypes = [C.c_int, C.POINTER(C.POINTER(C.c_int))]
    lib.mgw_host_status_free.argtypes = [C.POINTER(C.c_int)]
    lib.mgw_allreduce_group.argtypes = [C.POINTER(MgwAllreduceArgs), C.c_void_p]
    lib.mgw_flag_block_bytes.restype = C.c_size_t
    lib.mgw_stage_bytes.restype = C.c_size_t
    lib.mgw_stage_bytes.argtypes = [C.c_int, C.c_int, C.c_int]
    lib.mgw_multi_tensor_sgd.argtypes = [C.POINTER(MgwGroup), C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int,
                                         C.c_void_p, C.c_int, C.c_void_p]
    lib.mgw_clip_coef.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
    lib.mgw_group_sumsq.argtypes = [C.POINTER(MgwGroup), C.c_void_p, C.c_int, C.c_void_p]
    lib.mgw_bounds_allreduce.argtypes = [C.POINTER(C.c_int)]
    lib.mgw_bounds_sgd.argtypes = [C.POINTER(C.c_int)]
    lib.mgw_phase_times.argtypes = [C.POINTER(C.c_ulonglong), C.c_int]
    lib.mgw_s2d_stem_input.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
    for name in ('mgw_bn_relu_fwd', 'mgw_bn_relu_bwd', 'mgw_lstm_cell_fwd', 'mgw_lstm_cell_bwd',
                 'mgw_wgrad_gemm', 'mgw_wgrad_gemm_supported', 'mgw_allgather_rows'):
        if hasattr(lib, name):
            getattr(lib, name).restype = C.c_int


def load(allow_build: Optional[bool] = None) -> C.CDLL:
    """Return the loaded library, building it first when that is allowed and needed."""
    global _lib
    if _lib is not None:
        return _lib
    checked = is_checked()
    path = CHECKED_LIB_PATH if checked else LIB_PATH
    if not os.path.isfile(path):
        if allow_build is None:
            allow_build = os.environ.get('MGWFBP_BUILD_ON_IMPORT', '1') != '0'
        if not allow_build:
            raise NativeLibraryError('%s is missing; run `python -m mgwfbp_b200.ops.build%s`' % (path, ' --checked' if checked else ''))
        try:
            build(checked=checked)
        except Exception as e:
            raise NativeLibraryError('could not build %s: %s' % (path, e)) from e
    try:
        lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
    except OSError as e:
        raise NativeLibraryError('could not load %s: %s' % (path, e)) from e
    _declare(lib)
    _lib = lib
    return lib


def is_checked() -> bool:
    """True when this process runs the checked build (``MGWFBP_CHECKED=1``): the table-driven kernels verify
    every index they derive from a group table, record the first violation and skip the access."""
    return os.environ.get('MGWFBP_CHECKED', '0').strip().lower() not in ('0', '', 'false', 'no', 'off')


BOUNDS_CODES = {1: 'slot index outside the group', 2: 'slot not inside the tensor found for it',
                3: 'offset table and element count of a tensor disagree', 4: 'slot starts beyond the tensor\'s last element',
                5: 'staging index beyond the sized region'}


def phase_times(n_ctas: int) -> list:
    """Checked build: for each CTA of the most recent two-shot / NVLS all-reduce launch, the time in ns from CTA
    start to the end of (pack, first barrier, reduce, second barrier, consume) of the chunk's first piece and to the
    end of its last piece.  Zeros in the normal build."""
    buf = (C.c_ulonglong * (6 * n_ctas))()
    check(load().mgw_phase_times(buf, n_ctas), 'phase times')
    return [[int(buf[c * 6 + i]) for i in range(6)] for c in range(n_ctas)]


def bounds_report() -> list:
    """Violations recorded by the checked build since the last call, one dict per translation unit that saw one
    (always empty in the normal build).  Synchronizes the device."""
    lib = load()
    out = []
    for unit, fn in (('allreduce_fused', lib.mgw_bounds_allreduce), ('multi_tensor_sgd', lib.mgw_bounds_sgd)):
        rec = (C.c_int * 8)()
        check(fn(rec), 'bounds report')
        if rec[0]:
            out.append({'unit': unit, 'code': rec[0], 'what': BOUNDS_CODES.get(rec[0], '?'), 'values': [rec[1], rec[2], rec[3]],
                        'block': rec[4], 'thread': rec[5]})
    return out


def check(code: int, what: str = 'native call') -> None:
    if code != 0:
        msg = load().mgw_last_error()
        raise NativeLibraryError('%s failed with code %d: %s' % (what, code, (msg or b'').decode(errors='replace')))


def is_loaded() -> bool:
    return _lib is not None
