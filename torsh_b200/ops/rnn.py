"""LSTM on the device kernels: one GEMM for the input projection of every time step, one small GEMM per step for the
recurrent projection, and one fused kernel per step for the gate arithmetic (`tb_lstm_cell_fwd` / `tb_lstm_cell_bwd`).

Weights follow ``torch.nn.LSTM`` (``weight_ih [4H, I]``, ``weight_hh [4H, H]``, gate order i, f, g, o), so a
``torch.nn.LSTM`` layer's parameters can be passed as they are. The reference routes ``lstm_forward`` to cudnnRNNForward
(crates/torsh-backend/src/cuda/cudnn/operations.rs:1198) and keeps a Rust cell for the CPU
(crates/torsh-nn/src/layers/recurrent.rs).
"""
from __future__ import annotations

import torch

from .. import _native as nv
from ._dispatch import I, P, call, kernel_ok
from .gemm import gemm


def _cell_fwd(gx, gh, c_prev):
    B, H4 = gx.shape
    H = H4 // 4
    h = torch.empty(B, H, dtype=gx.dtype, device=gx.device)
    c = torch.empty(B, H, dtype=torch.float32, device=gx.device)
    act = torch.empty_like(gx)
    call("tb_lstm_cell_fwd", [P, P, P, P, P, P, I, I, I, P], gx.data_ptr(), gh.data_ptr(), c_prev.data_ptr(), h.data_ptr(),
         c.data_ptr(), act.data_ptr(), B, H, 0 if gx.dtype == torch.bfloat16 else 1, nv.stream_ptr())
    return h, c, act


def _cell_bwd(dh, dc_next, act, c, c_prev):
    B, H4 = act.shape
    H = H4 // 4
    dg = torch.empty_like(act)
    dc_prev = torch.empty(B, H, dtype=torch.float32, device=act.device)
    call("tb_lstm_cell_bwd", [P, P, P, P, P, P, P, I, I, I, P], dh.data_ptr(), 0 if dc_next is None else dc_next.data_ptr(),
         act.data_ptr(), c.data_ptr(), c_prev.data_ptr(), dg.data_ptr(), dc_prev.data_ptr(), B, H,
         0 if act.dtype == torch.bfloat16 else 1, nv.stream_ptr())
    return dg, dc_prev


class _LstmFn(torch.autograd.Function):
    """x [T, B, I] bf16, h0 [B, H] bf16, c0 [B, H] fp32, w_ih [4H, I], w_hh [4H, H] bf16, bias [4H] bf16 or None."""

    @staticmethod
    def forward(ctx, x, h0, c0, w_ih, w_hh, bias):
        T, B, In = x.shape
        H = w_hh.shape[1]
        gx_all = gemm(x.reshape(T * B, In), w_ih, bias=bias).reshape(T, B, 4 * H)      # every step at once
        hs = torch.empty(T, B, H, dtype=x.dtype, device=x.device)
        cs = torch.empty(T + 1, B, H, dtype=torch.float32, device=x.device)
        acts = torch.empty(T, B, 4 * H, dtype=x.dtype, device=x.device)
        cs[0] = c0
        h = h0.contiguous()
        for t in range(T):
            gh = gemm(h, w_hh)
            h, c, act = _cell_fwd(gx_all[t], gh, cs[t])
            hs[t], cs[t + 1], acts[t] = h, c, act
        ctx.save_for_backward(x, h0, w_ih, w_hh, hs, cs, acts)
        ctx.has_bias = bias is not None
        return hs, hs[-1].clone(), cs[-1].clone()

    @staticmethod
    def backward(ctx, d_hs, d_hT, d_cT):
        x, h0, w_ih, w_hh, hs, cs, acts = ctx.saved_tensors
        T, B, In = x.shape
        H = w_hh.shape[1]
        dgates = torch.empty_like(acts)
        dh_rec = d_hT.to(x.dtype).contiguous() if d_hT is not None else torch.zeros(B, H, dtype=x.dtype, device=x.device)
        dc = d_cT.float().contiguous() if d_cT is not None else None
        for t in range(T - 1, -1, -1):
            dh = dh_rec if d_hs is None else (d_hs[t] + dh_rec).contiguous()
            dg, dc = _cell_bwd(dh, dc, acts[t], cs[t + 1], cs[t])
            dgates[t] = dg
            dh_rec = gemm(dg, w_hh, b_major=1)                         # dL/dh_{t-1} = dgates_t @ W_hh
        dg2 = dgates.reshape(T * B, 4 * H)
        dx = gemm(dg2, w_ih, b_major=1).reshape(T, B, In)
        h_prev = torch.cat([h0[None], hs[:-1]], 0).reshape(T * B, H)
        dw_ih = gemm(dg2, x.reshape(T * B, In), a_major=1, b_major=1, out_dtype=torch.float32)   # dgates^T @ x
        dw_hh = gemm(dg2, h_prev, a_major=1, b_major=1, out_dtype=torch.float32)
        db = dg2.float().sum(0) if ctx.has_bias else None
        return (dx, dh_rec, dc, dw_ih.to(w_ih.dtype), dw_hh.to(w_hh.dtype), None if db is None else db.to(w_ih.dtype))


def _lstm_reference(x, h0, c0, w_ih, w_hh, bias):
    """Plain PyTorch evaluation (CPU, or dtypes the kernels do not take)."""
    h, c = h0.float(), c0.float()
    out = []
    for t in range(x.shape[0]):
        g = x[t].float() @ w_ih.float().t() + h @ w_hh.float().t() + (0 if bias is None else bias.float())
        i, f, gg, o = g.chunk(4, -1)
        c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(gg)
        h = torch.sigmoid(o) * torch.tanh(c)
        out.append(h)
    hs = torch.stack(out).to(x.dtype)
    return hs, hs[-1], c


def lstm_layer(x: torch.Tensor, h0: torch.Tensor, c0: torch.Tensor, w_ih: torch.Tensor, w_hh: torch.Tensor,
               b_ih: torch.Tensor | None = None, b_hh: torch.Tensor | None = None):
    """One LSTM layer over a sequence. ``x`` is ``[T, B, I]``; returns ``(outputs [T, B, H], h_T [B, H], c_T [B, H] fp32)``.
    On a GPU in bf16 with I and H multiples of 8 this runs on the kernels with a hand-written backward; otherwise it is
    evaluated with PyTorch ops."""
    bias = None
    if b_ih is not None or b_hh is not None:
        bias = (0 if b_ih is None else b_ih) + (0 if b_hh is None else b_hh)
    ok = (kernel_ok(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and w_hh.shape[1] % 8 == 0)
    if not ok:
        return _lstm_reference(x, h0, c0, w_ih, w_hh, bias)
    return _LstmFn.apply(x.contiguous(), h0.to(x.dtype), c0.float().contiguous(), w_ih.to(x.dtype).contiguous(),
                         w_hh.to(x.dtype).contiguous(), None if bias is None else bias.to(x.dtype).contiguous())


class KernelLSTM(torch.nn.Module):
    """Multi-layer unidirectional LSTM with ``torch.nn.LSTM``'s parameter names (``weight_ih_l0`` ...), so state dicts
    move between the two; time-major input ``[T, B, I]`` (or batch-first with ``batch_first=True``)."""

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True, batch_first: bool = False):
        super().__init__()
        self.input_size, self.hidden_size, self.num_layers, self.batch_first = input_size, hidden_size, num_layers, batch_first
        k = hidden_size ** -0.5
        for l in range(num_layers):
            i = input_size if l == 0 else hidden_size
            self.register_parameter(f"weight_ih_l{l}", torch.nn.Parameter(torch.empty(4 * hidden_size, i).uniform_(-k, k)))
            self.register_parameter(f"weight_hh_l{l}", torch.nn.Parameter(torch.empty(4 * hidden_size, hidden_size).uniform_(-k, k)))
            if bias:
                self.register_parameter(f"bias_ih_l{l}", torch.nn.Parameter(torch.empty(4 * hidden_size).uniform_(-k, k)))
                self.register_parameter(f"bias_hh_l{l}", torch.nn.Parameter(torch.empty(4 * hidden_size).uniform_(-k, k)))
        self.has_bias = bias

    def forward(self, x, state=None):
        if self.batch_first:
            x = x.transpose(0, 1)
        T, B, _ = x.shape
        hs, cs = [], []
        for l in range(self.num_layers):
            h0 = x.new_zeros(B, self.hidden_size) if state is None else state[0][l]
            c0 = torch.zeros(B, self.hidden_size, dtype=torch.float32, device=x.device) if state is None else state[1][l]
            x, hT, cT = lstm_layer(x, h0, c0, getattr(self, f"weight_ih_l{l}"), getattr(self, f"weight_hh_l{l}"),
                                   getattr(self, f"bias_ih_l{l}", None), getattr(self, f"bias_hh_l{l}", None))
            hs.append(hT)
            cs.append(cT)
        out = x.transpose(0, 1) if self.batch_first else x
        return out, (torch.stack(hs), torch.stack(cs))
