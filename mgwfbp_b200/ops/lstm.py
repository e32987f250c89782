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
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib, counters

_declared = False


def _declare(lib) -> None:
    global _declared
    if not _declared:
        lib.mgw_lstm_cell_fwd.argtypes = [C.c_void_p] * 8 + [C.c_int, C.c_int, C.c_void_p]
        lib.mgw_lstm_cell_bwd.argtypes = [C.c_void_p] * 7 + [C.c_int, C.c_int, C.c_void_p]
        _declared = True


def _ptr(t):
    return None if t is None else t.data_ptr()


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
        gh = torch.empty(B, 4 * H, device=x.device, dtype=x.dtype)
        cs[0].copy_(c0)
        h = h0.contiguous()
        w_hh_t = w_hh.t()
        for t in range(T):
            torch.mm(h, w_hh_t, out=gh)
            _lib.check(lib.mgw_lstm_cell_fwd(gx[t * B:(t + 1) * B].data_ptr(), gh.data_ptr(), _ptr(b_ih), _ptr(b_hh),
                                             cs[t].data_ptr(), out[t].data_ptr(), cs[t + 1].data_ptr(), act[t].data_ptr(),
                                             B, H, s), 'lstm_cell_fwd')
            h = out[t]
        counters.bump('lstm_cell_fwd', T)
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
        dh = torch.zeros(B, H, device=x.device, dtype=x.dtype) if d_hT is None else d_hT.contiguous().clone()
        dc = torch.zeros(B, H, device=x.device, dtype=x.dtype) if d_cT is None else d_cT.contiguous().clone()
        dc_next = torch.empty_like(dc)
        d_out = d_out.contiguous() if d_out is not None else None
        for t in range(T - 1, -1, -1):
            if d_out is not None:
                dh.add_(d_out[t])
            _lib.check(lib.mgw_lstm_cell_bwd(dh.data_ptr(), dc.data_ptr(), act[t].data_ptr(), cs[t].data_ptr(),
                                             cs[t + 1].data_ptr(), dG[t].data_ptr(), dc_next.data_ptr(), B, H, s),
                       'lstm_cell_bwd')
            dc, dc_next = dc_next, dc
            torch.mm(dG[t], w_hh, out=dh)                     # dh_{t-1}
        counters.bump('lstm_cell_bwd', T)
        dG2 = dG.reshape(T * B, 4 * H)
        h_prev = torch.cat([h0.unsqueeze(0), out[:-1]], 0).reshape(T * B, H)
        need = ctx.needs_input_grad
        dx = (dG2 @ w_ih).reshape(x.shape) if need[0] else None
        dw_ih = dG2.t() @ x.reshape(T * B, -1) if need[3] else None
        dw_hh = dG2.t() @ h_prev if need[4] else None
        db = dG2.sum(0) if ctx.has_bias else None
        return dx, dh if need[1] else None, dc if need[2] else None, dw_ih, dw_hh, db, (db.clone() if db is not None else None)


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
