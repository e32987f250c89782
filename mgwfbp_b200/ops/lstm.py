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


# MGWFBP_LSTM_REC=1 sends the per-step recurrent products through csrc/lstm_rec.cu instead of torch.mm (cuBLAS).  The
# kernel itself is faster per call (10.1 us against 12.3 us for 20 x 1500 x 6000 on B200), but its split-K partial sums make
# the cell kernels that add them up slower by more than that, so the library product is the default.
_OWN_REC = os.environ.get('MGWFBP_LSTM_REC', '0').strip().lower() not in ('0', 'false', 'no', 'off', '')


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


def _weight_grad(dg: torch.Tensor, inp: torch.Tensor, sink=None) -> Optional[torch.Tensor]:
    """``dg^T @ inp`` ([T*B, 4H]^T x [T*B, in]): the weight gradient of a whole sequence as one GEMM.  With a ``sink`` (set on
    the parameter by a data-parallel optimizer) the product is formed and reduced across ranks there and nothing is returned."""
    if sink is not None:
        sink(dg.contiguous(), inp.contiguous())
        return None
    if _WGRAD == 'tcgen05':
        from . import wgrad
        if wgrad.supported(dg, inp):
            return wgrad.wgrad_gemm(dg, inp)
    return dg.t() @ inp


# Time steps per wavefront chunk (0: layers run one after the other).  Layer k works on chunk c while layer k-1 already
# works on chunk c+1, each layer on its own stream, which is how a multi-layer recurrence fills a GPU whose single small
# step cannot (the library LSTM does the same internally).
_CHUNK = int(os.environ.get('MGWFBP_LSTM_CHUNK', '7') or 0)
_side_streams: dict = {}


def _stream_for(device, k: int) -> torch.cuda.Stream:
    key = (device.index, k)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]


class _LSTMStack(torch.autograd.Function):
    """All layers over a whole sequence as a wavefront: x [T, B, in], h0/c0 [L, B, H] -> out [T, B, H], hT, cT [L, B, H].

    Forward: layer 0's input projection is one GEMM over all steps; every further layer projects its input chunk by
    chunk (dropout mask applied first).  Per step one recurrent product (``_Recurrent``) and one fused cell kernel.
    Backward walks chunks and layers in reverse with the same streams; weight gradients are single GEMMs over the whole
    sequence at the end (``dW = dG^T [T*B, 4H] x [T*B, in]``)."""

    @staticmethod
    def forward(ctx, x, h0, c0, chunk, p_drop, training, *weights):
        lib = _lib.load(allow_build=False)
        _declare(lib)
        L = len(weights) // 4
        T, B, _ = x.shape
        H = weights[1].shape[1]
        dev, dt = x.device, x.dtype
        chunk = T if (chunk <= 0 or L == 1) else min(chunk, T)
        bounds = [(a, min(T, a + chunk)) for a in range(0, T, chunk)]
        cur = torch.cuda.current_stream()
        streams = [cur] + [_stream_for(dev, k) for k in range(1, L)]
        masks = []
        for k in range(L - 1):
            if training and p_drop > 0:
                masks.append(torch.bernoulli(torch.full((T, B, H), 1.0 - p_drop, device=dev, dtype=dt)).div_(1.0 - p_drop))
            else:
                masks.append(None)
        w_ih, w_hh = [weights[4 * k] for k in range(L)], [weights[4 * k + 1] for k in range(L)]
        b_ih, b_hh = [weights[4 * k + 2] for k in range(L)], [weights[4 * k + 3] for k in range(L)]
        gx = [None] * L
        gx[0] = x.reshape(T * B, -1) @ w_ih[0].t()                      # layer 0: all steps at once
        inps = [x] + [torch.empty(T, B, H, device=dev, dtype=dt) for _ in range(1, L)]
        for k in range(1, L):
            gx[k] = torch.empty(T * B, 4 * H, device=dev, dtype=dt)
        # slot 0 holds h0, so "the hidden state before step t" is hs[k][t] and all of them are one view (no concatenation)
        hs = [torch.empty(T + 1, B, H, device=dev, dtype=dt) for _ in range(L)]
        out = [hs[k][1:] for k in range(L)]
        cs = [torch.empty(T + 1, B, H, device=dev, dtype=dt) for _ in range(L)]
        act = [torch.empty(T, B, 4 * H, device=dev, dtype=dt) for _ in range(L)]
        rec = [_Recurrent(lib, w_hh[k].detach(), B) for k in range(L)]
        for k in range(L):
            hs[k][0].copy_(h0[k])
            cs[k][0].copy_(c0[k])
        fork = torch.cuda.Event()
        fork.record(cur)
        for st in streams[1:]:
            st.wait_event(fork)
        for a, b in bounds:
            done_below = None
            for k in range(L):
                with torch.cuda.stream(streams[k]):
                    if k > 0:
                        streams[k].wait_event(done_below)
                        if masks[k - 1] is not None:
                            torch.mul(out[k - 1][a:b], masks[k - 1][a:b], out=inps[k][a:b])
                        else:
                            inps[k][a:b].copy_(out[k - 1][a:b])
                        torch.mm(inps[k][a:b].reshape((b - a) * B, H), w_ih[k].t(), out=gx[k][a * B:b * B])
                    sp = streams[k].cuda_stream
                    for t in range(a, b):
                        rec[k](hs[k][t], sp)
                        _lib.check(lib.mgw_lstm_cell_fwd(gx[k][t * B:(t + 1) * B].data_ptr(), rec[k].out.data_ptr(), _ptr(b_ih[k]),
                                                         _ptr(b_hh[k]), cs[k][t].data_ptr(), out[k][t].data_ptr(),
                                                         cs[k][t + 1].data_ptr(), act[k][t].data_ptr(), B, H, rec[k].parts,
                                                         rec[k].stride, sp), 'lstm_cell_fwd')
                    done_below = torch.cuda.Event()
                    done_below.record(streams[k])
        for st in streams[1:]:
            ev = torch.cuda.Event()
            ev.record(st)
            cur.wait_event(ev)
        counters.bump('lstm_cell_fwd', T * L)
        if rec[0].own:
            counters.bump('lstm_rec_gemm', T * L)
        ctx.save_for_backward(x, *weights, *[m for m in masks if m is not None])
        ctx.stash = (hs, cs, act, inps, [m is not None for m in masks], bounds)
        # where a data-parallel optimizer wants a weight gradient delivered instead of returned (reduce-scatter GEMM)
        ctx.sinks = [getattr(w, '_mgw_rs_sink', None) if w is not None else None for w in weights]
        ctx.dims = (L, T, B, H)
        hT = torch.stack([out[k][T - 1] for k in range(L)])
        cT = torch.stack([cs[k][T] for k in range(L)])
        # a fresh view: the tensor object that autograd turns into this node's output must not be the one kept in
        # ctx.stash, or node -> stash -> output -> node would be a reference cycle that keeps the whole graph of a
        # finished step (and its gradient accumulators with their stream) alive until the garbage collector runs
        return out[L - 1].view(T, B, H), hT, cT

    @staticmethod
    def backward(ctx, d_out, d_hT, d_cT):
        lib = _lib.load(allow_build=False)
        L, T, B, H = ctx.dims
        saved = ctx.saved_tensors
        x = saved[0]
        weights = saved[1:1 + 4 * L]
        hs, cs, act, inps, has_mask, bounds = ctx.stash
        mask_it = iter(saved[1 + 4 * L:])
        masks = [next(mask_it) if hm else None for hm in has_mask]
        w_ih, w_hh = [weights[4 * k] for k in range(L)], [weights[4 * k + 1] for k in range(L)]
        has_bias = weights[2] is not None
        dev, dt = x.device, x.dtype
        cur = torch.cuda.current_stream()
        streams = [cur] + [_stream_for(dev, k) for k in range(1, L)]
        dG = [torch.empty(T, B, 4 * H, device=dev, dtype=dt) for _ in range(L)]
        # gradient arriving at each layer's outputs: the caller's for the top layer, from the layer above otherwise
        d_lay = [None] * L
        d_lay[L - 1] = d_out.contiguous() if d_out is not None else torch.zeros(T, B, H, device=dev, dtype=dt)
        for k in range(L - 1):
            d_lay[k] = torch.empty(T, B, H, device=dev, dtype=dt)
        dc = [torch.zeros(B, H, device=dev, dtype=dt) if d_cT is None else d_cT[k].contiguous().clone() for k in range(L)]
        dc_next = [torch.empty_like(dc[k]) for k in range(L)]
        rec = [_Recurrent(lib, w_hh[k].detach().t().contiguous(), B) for k in range(L)]      # rows of W_hh^T: hidden units
        parts = [0] * L
        for k in range(L):
            if d_hT is not None:                              # gradient of the final state enters like a recurrent term
                rec[k].out.zero_()
                rec[k].out[0].copy_(d_hT[k])
                parts[k] = rec[k].parts
        fork = torch.cuda.Event()
        fork.record(cur)
        for st in streams[1:]:
            st.wait_event(fork)
        for a, b in reversed(bounds):
            done_above = None
            for k in range(L - 1, -1, -1):
                with torch.cuda.stream(streams[k]):
                    if done_above is not None:
                        streams[k].wait_event(done_above)
                    sp = streams[k].cuda_stream
                    for t in range(b - 1, a - 1, -1):
                        _lib.check(lib.mgw_lstm_cell_bwd(d_lay[k][t].data_ptr(), dc[k].data_ptr(), act[k][t].data_ptr(),
                                                         cs[k][t].data_ptr(), cs[k][t + 1].data_ptr(), dG[k][t].data_ptr(),
                                                         dc_next[k].data_ptr(), B, H, rec[k].out.data_ptr(), parts[k],
                                                         rec[k].stride, sp), 'lstm_cell_bwd')
                        dc[k], dc_next[k] = dc_next[k], dc[k]
                        rec[k](dG[k][t], sp)                  # partial sums of dh_{t-1}
                        parts[k] = rec[k].parts
                    if k > 0:                                 # gradient for the layer below, this chunk
                        torch.mm(dG[k][a:b].reshape((b - a) * B, 4 * H), w_ih[k], out=d_lay[k - 1][a:b].reshape((b - a) * B, H))
                        if masks[k - 1] is not None:
                            d_lay[k - 1][a:b].mul_(masks[k - 1][a:b])
                    done_above = torch.cuda.Event()
                    done_above.record(streams[k])
        counters.bump('lstm_cell_bwd', T * L)
        if rec[0].own:
            counters.bump('lstm_rec_gemm', T * L)
        need = ctx.needs_input_grad
        grads_w = []
        dh0, dc0 = [], []
        for k in range(L):
            with torch.cuda.stream(streams[k]):
                dG2 = dG[k].reshape(T * B, 4 * H)
                inp2 = inps[k].reshape(T * B, -1)
                h_prev = hs[k][:-1].reshape(T * B, H)
                dw_ih = _weight_grad(dG2, inp2, ctx.sinks[4 * k])
                dw_hh = _weight_grad(dG2, h_prev, ctx.sinks[4 * k + 1])
                db = dG2.sum(0) if has_bias else None
                grads_w += [dw_ih, dw_hh, db, db.clone() if db is not None else None]
                dh0.append(rec[k].out.sum(0))
                dc0.append(dc[k])
        dx = None
        if need[0]:
            dx = (dG[0].reshape(T * B, 4 * H) @ w_ih[0]).reshape(x.shape)
        for st in streams[1:]:
            ev = torch.cuda.Event()
            ev.record(st)
            cur.wait_event(ev)
        for g in grads_w + dh0 + dc0:                         # allocated on a layer's stream, consumed on the caller's
            if g is not None:
                g.record_stream(cur)
        return (dx, torch.stack(dh0) if need[1] else None, torch.stack(dc0) if need[2] else None, None, None, None, *grads_w)


class FusedLSTM(nn.Module):
    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True, dropout: float = 0.0):
        super().__init__()
        self.input_size, self.hidden_size, self.num_layers = input_size, hidden_size, num_layers
        self.bias, self.dropout, self.batch_first, self.bidirectional = bias, float(dropout), False, False
        for k in range(num_layers):
            in_k = input_size if k == 0 else hidden_size
            self.register_parameter('weight_ih_l%d' % k, nn.Parameter(torch.empty(4 * hidden_size, in_k)))
            self.register_parameter('weight_hh_l%d' % k, nn.Parameter(torch.empty(4 * hidden_size, hidden_size)))
            for w in (getattr(self, 'weight_ih_l%d' % k), getattr(self, 'weight_hh_l%d' % k)):
                w._mgw_scatter_candidate = True       # their gradient is one GEMM: may take the reduce-scatter form
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
        if x.is_cuda and x.dtype == torch.float32:
            weights = [w for k in range(self.num_layers) for w in self._layer_params(k)]
            out, hT, cT = _LSTMStack.apply(x.contiguous(), h0, c0, _CHUNK, self.dropout, self.training, *weights)
            return out, (hT, cT)
        hs: List[torch.Tensor] = []
        cs: List[torch.Tensor] = []
        inp = x
        for k in range(self.num_layers):
            w_ih, w_hh, b_ih, b_hh = self._layer_params(k)
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
