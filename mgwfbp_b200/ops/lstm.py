# -*- coding: utf-8 -*-
"""``FusedLSTM``: multi-layer unidirectional LSTM whose per-step pointwise work runs in this
package's kernels (``csrc/lstm_cell.cu``) and whose weight gradients are single large GEMMs.

Parameter names, shapes and gate order are those of ``torch.nn.LSTM``
(``weight_ih_l{k} [4H, in]``, ``weight_hh_l{k} [4H, H]``, ``bias_ih_l{k}``, ``bias_hh_l{k}``), so a
``state_dict`` moves between the two freely -- the reference model stores a ``torch.nn.LSTM``
(``models/lstm.py:16-19``).  Per layer: one GEMM for all time steps' input projections, then per step
one recurrent GEMM and one fused cell kernel; backward walks the steps in reverse with one cell
kernel and one GEMM each, and forms ``dW_ih``, ``dW_hh``, ``dX`` and the bias gradients from the
stacked gate gradients afterwards (``dW = dG^T [T*B, 4H] x [T*B, in]``: M=6000, N=1500, K=700 for
the PTB model).
"""
from __future__ import annotations

import ctypes as C
import math
import os
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib, counters

_declared = False


def _declare(lib) -> None:
    global _declared
    if not _declared:
        lib.mgw_lstm_cell_fwd.argtypes = [C.c_void_p] * 8 + [C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_void_p]
        lib.mgw_lstm_cell_bwd.argtypes = [C.c_void_p] * 7 + [C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_longlong, C.c_void_p]
        lib.mgw_lstm_rec_splits.argtypes = [C.c_int]
        lib.mgw_lstm_rec_supported.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
        lib.mgw_lstm_rec_gemm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        _declared = True


def _ptr(t):
    return None if t is None else t.data_ptr()


# MGWFBP_LSTM_REC=0 sends the per-step recurrent products through torch.mm (cuBLAS) instead of csrc/lstm_rec.cu
_OWN_REC = os.environ.get('MGWFBP_LSTM_REC', '1').strip().lower() not in ('0', 'false', 'no', 'off', '')


class _Recurrent:
    """``x [B, K] @ w [R, K]^T`` for one time step, as split-K partial sums that the cell kernels add up.

    Uses the package's small-batch kernel when it handles the shape, ``torch.mm`` otherwise (one "partial")."""

    def __init__(self, lib, w: torch.Tensor, B: int):
        self.lib, self.w = lib, w
        self.R, self.K = w.shape
        # the kernel multiplies in TF32 (fp32 accumulation), so it only stands in for torch.mm where TF32 matmuls are
        # allowed; with full-precision matmuls requested the library product is used
        self.own = bool(_OWN_REC and torch.backends.cuda.matmul.allow_tf32 and w.is_contiguous() and
                        lib.mgw_lstm_rec_supported(w.data_ptr(), w.data_ptr(), B, self.R, self.K))
        self.parts = int(lib.mgw_lstm_rec_splits(self.K)) if self.own else 1
        self.out = torch.empty(self.parts, B, self.R, device=w.device, dtype=w.dtype)
        self.stride = B * self.R
        self.w_t = None if self.own else w.t()

    def __call__(self, x: torch.Tensor, stream: int) -> None:
        if self.own:
            _lib.check(self.lib.mgw_lstm_rec_gemm(x.data_ptr(), self.w.data_ptr(), self.out.data_ptr(), x.shape[0], self.R, self.K,
                                                  stream), 'lstm_rec_gemm')
        else:
            torch.mm(x, self.w_t, out=self.out[0])


class _LSTMLayer(torch.autograd.Function):
    """One layer over a whole sequence: x [T, B, in], h0/c0 [B, H] -> out [T, B, H], hT, cT."""

    @staticmethod
    def forward(ctx, x, h0, c0, w_ih, w_hh, b_ih, b_hh):
        lib = _lib.load(allow_build=False)
        _declare(lib)
        T, B, _ = x.shape
        H = w_hh.shape[1]
        s = torch.cuda.current_stream().cuda_stream
        x2 = x.reshape(T * B, -1)
        gx = x2 @ w_ih.t()                                    # [T*B, 4H], all steps at once
        out = torch.empty(T, B, H, device=x.device, dtype=x.dtype)
        cs = torch.empty(T + 1, B, H, device=x.device, dtype=x.dtype)
        act = torch.empty(T, B, 4 * H, device=x.device, dtype=x.dtype)
        cs[0].copy_(c0)
        h = h0.contiguous()
        rec = _Recurrent(lib, w_hh.detach(), B)               # h_{t-1} W_hh^T, W_hh [4H, H] rows are the gates
        for t in range(T):
            rec(h, s)
            _lib.check(lib.mgw_lstm_cell_fwd(gx[t * B:(t + 1) * B].data_ptr(), rec.out.data_ptr(), _ptr(b_ih), _ptr(b_hh),
                                             cs[t].data_ptr(), out[t].data_ptr(), cs[t + 1].data_ptr(), act[t].data_ptr(),
                                             B, H, rec.parts, rec.stride, s), 'lstm_cell_fwd')
            h = out[t]
        counters.bump('lstm_cell_fwd', T)
        if rec.own:
            counters.bump('lstm_rec_gemm', T)
        ctx.save_for_backward(x, h0, w_ih, w_hh, out, cs, act)
        ctx.has_bias = b_ih is not None
        return out, out[T - 1].clone(), cs[T].clone()

    @staticmethod
    def backward(ctx, d_out, d_hT, d_cT):
        lib = _lib.load(allow_build=False)
        x, h0, w_ih, w_hh, out, cs, act = ctx.saved_tensors
        T, B, H = out.shape
        s = torch.cuda.current_stream().cuda_stream
        dG = torch.empty(T, B, 4 * H, device=x.device, dtype=x.dtype)
        dc = torch.zeros(B, H, device=x.device, dtype=x.dtype) if d_cT is None else d_cT.contiguous().clone()
        dc_next = torch.empty_like(dc)
        d_out = d_out.contiguous() if d_out is not None else None
        # dh_{t-1} through the recurrence is dG_t W_hh: rows of W_hh^T [H, 4H] are the hidden units
        rec = _Recurrent(lib, w_hh.detach().t().contiguous(), B)
        if d_hT is not None:                                  # gradient of the final state enters like a recurrent term
            rec.out.zero_()
            rec.out[0].copy_(d_hT)
            parts = rec.parts
        else:
            parts = 0
        for t in range(T - 1, -1, -1):
            _lib.check(lib.mgw_lstm_cell_bwd(_ptr(d_out[t]) if d_out is not None else None, dc.data_ptr(), act[t].data_ptr(),
                                             cs[t].data_ptr(), cs[t + 1].data_ptr(), dG[t].data_ptr(), dc_next.data_ptr(), B, H,
                                             rec.out.data_ptr(), parts, rec.stride, s), 'lstm_cell_bwd')
            dc, dc_next = dc_next, dc
            rec(dG[t], s)                                     # partial sums of dh_{t-1}
            parts = rec.parts
        counters.bump('lstm_cell_bwd', T)
        if rec.own:
            counters.bump('lstm_rec_gemm', T)
        dh0 = rec.out.sum(0) if ctx.needs_input_grad[1] else None
        dG2 = dG.reshape(T * B, 4 * H)
        h_prev = torch.cat([h0.unsqueeze(0), out[:-1]], 0).reshape(T * B, H)
        need = ctx.needs_input_grad
        dx = (dG2 @ w_ih).reshape(x.shape) if need[0] else None
        dw_ih = _weight_grad(dG2, x.reshape(T * B, -1)) if need[3] else None
        dw_hh = _weight_grad(dG2, h_prev) if need[4] else None
        db = dG2.sum(0) if ctx.has_bias else None
        return dx, dh0, dc if need[2] else None, dw_ih, dw_hh, db, (db.clone() if db is not None else None)


# MGWFBP_LSTM_WGRAD=tcgen05 forms dW_ih / dW_hh with the package's tensor-core weight-gradient GEMM (csrc/wgrad_gemm_sm100.cu)
_WGRAD = os.environ.get('MGWFBP_LSTM_WGRAD', 'library').strip().lower()


def _weight_grad(dg: torch.Tensor, inp: torch.Tensor) -> torch.Tensor:
    """``dg^T @ inp`` ([T*B, 4H]^T x [T*B, in]): the weight gradient of a whole sequence as one GEMM."""
    if _WGRAD == 'tcgen05':
        from . import wgrad
        if wgrad.supported(dg, inp):
            return wgrad.wgrad_gemm(dg, inp)
    return dg.t() @ inp


class FusedLSTM(nn.Module):
    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True, dropout: float = 0.0):
        super().__init__()
        self.input_size, self.hidden_size, self.num_layers = input_size, hidden_size, num_layers
        self.bias, self.dropout, self.batch_first, self.bidirectional = bias, float(dropout), False, False
        for k in range(num_layers):
            in_k = input_size if k == 0 else hidden_size
            self.register_parameter('weight_ih_l%d' % k, nn.Parameter(torch.empty(4 * hidden_size, in_k)))
            self.register_parameter('weight_hh_l%d' % k, nn.Parameter(torch.empty(4 * hidden_size, hidden_size)))
            if bias:
                self.register_parameter('bias_ih_l%d' % k, nn.Parameter(torch.empty(4 * hidden_size)))
                self.register_parameter('bias_hh_l%d' % k, nn.Parameter(torch.empty(4 * hidden_size)))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        bound = 1.0 / math.sqrt(self.hidden_size) if self.hidden_size > 0 else 0
        for p in self.parameters():
            nn.init.uniform_(p, -bound, bound)

    def flatten_parameters(self) -> None:        # API compatibility with nn.LSTM
        pass

    def _layer_params(self, k):
        g = lambda n: getattr(self, n % k) if hasattr(self, n % k) else None
        return g('weight_ih_l%d'), g('weight_hh_l%d'), g('bias_ih_l%d'), g('bias_hh_l%d')

    def forward(self, x: torch.Tensor, hx: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        T, B, _ = x.shape
        if hx is None:
            z = x.new_zeros(self.num_layers, B, self.hidden_size)
            hx = (z, z.clone())
        h0, c0 = hx
        hs: List[torch.Tensor] = []
        cs: List[torch.Tensor] = []
        inp = x
        for k in range(self.num_layers):
            w_ih, w_hh, b_ih, b_hh = self._layer_params(k)
            if x.is_cuda and x.dtype == torch.float32:
                out, hT, cT = _LSTMLayer.apply(inp.contiguous(), h0[k], c0[k], w_ih, w_hh, b_ih, b_hh)
            else:
                out, hT, cT = self._reference_layer(inp, h0[k], c0[k], w_ih, w_hh, b_ih, b_hh)
            hs.append(hT)
            cs.append(cT)
            inp = out
            if self.dropout > 0 and k < self.num_layers - 1:
                inp = F.dropout(inp, p=self.dropout, training=self.training)
        return inp, (torch.stack(hs), torch.stack(cs))

    @staticmethod
    def _reference_layer(x, h, c, w_ih, w_hh, b_ih, b_hh):
        """Plain PyTorch evaluation of the same recurrence (CPU and non-fp32 inputs)."""
        outs = []
        for t in range(x.shape[0]):
            gates = F.linear(x[t], w_ih, b_ih) + F.linear(h, w_hh, b_hh)
            i, f, g, o = gates.chunk(4, 1)
            c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
            h = torch.sigmoid(o) * torch.tanh(c)
            outs.append(h)
        return torch.stack(outs), h, c
