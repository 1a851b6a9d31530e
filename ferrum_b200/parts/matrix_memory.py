"""A matrix-memory recurrence with exponential gates (the mLSTM cell of xLSTM).

H heads with keys of D and values of Dv.  Per token: q = W_q x * D^(-1/2), k = W_k x, v = W_v x, and per
head a log input gate i = c tanh((W_i x + b_i) / c) and a log forget gate
f = logsigmoid(c tanh((W_f x + b_f) / c)) with the cap c.  With S (D x Dv), n (D) and the running
maximum m, all zero before the first token (m starts at 0):

    m' = max(f + m, i);   S <- e^(f + m - m') S + e^(i - m') k v^T;   n <- e^(f + m - m') n + e^(i - m') k
    o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)

Each head's o is divided by its root mean square; the heads side by side are multiplied by a weight
vector of their joint size and by sigmoid(W_g x), and projected back.  A request's state row keeps S, n
and m in float32; the walk over a portion's tokens is sequential, so a token's result does not depend
on how the sequence was cut into steps.  Everything after the projections is float32.  The reference
has no recurrent mixer (crates/model/src/llama.rs:185-257 is its only one).
"""
from __future__ import annotations

import torch

from ..ops import lib as ops
from .base import CacheNeed, Mixer, ParamSpec, StateNeed
from .linear import RESIDUAL, STORE_F32, linear, linear_deferred


def _draw_forget_bias(shape, g, device, std):
    """U(3, 6): a forget gate that starts near one."""
    return 3.0 + 3.0 * torch.rand(shape, generator=g, device=device, dtype=torch.float32)


class MatrixMemoryMixer(Mixer):
    graph_safe = True

    def __init__(self, width, heads, dim, vdim, gate_cap, eps, dtype):
        if not 0 < dim <= ops.RECURRENT_MAX_DIM:
            raise ValueError(f"key size {dim} is outside the kernel's limit ({ops.RECURRENT_MAX_DIM})")
        if not gate_cap > 0:
            raise ValueError("the gates' cap must be positive")
        self.width, self.H, self.D, self.Dv = width, int(heads), int(dim), int(vdim)
        self.cap, self.eps, self.dtype = float(gate_cap), float(eps), dtype
        for n in ("q_weight", "k_weight", "v_weight", "g_weight", "i_weight", "f_weight", "i_bias", "f_bias", "norm_weight", "o_weight"):
            setattr(self, "w_" + n, None)
        self.w_in = None

    def param_specs(self):
        E, H, D, Dv = self.width, self.H, self.D, self.Dv
        return {"q.weight": ParamSpec((H * D, E)), "k.weight": ParamSpec((H * D, E)), "v.weight": ParamSpec((H * Dv, E)),
                "g.weight": ParamSpec((H * Dv, E)), "i.weight": ParamSpec((H, E)), "f.weight": ParamSpec((H, E)),
                "i.bias": ParamSpec((H,), kind="vector", init="normal"), "f.bias": ParamSpec((H,), kind="vector", init=_draw_forget_bias),
                "norm.weight": ParamSpec((H * Dv,), kind="vector", init="ones_normal"),
                "o.weight": ParamSpec((E, H * Dv))}

    def finalize(self):
        self.w_in = torch.cat([self.w_q_weight, self.w_k_weight, self.w_v_weight, self.w_g_weight, self.w_i_weight,
                               self.w_f_weight], dim=0).contiguous()
        self.w_q_weight = self.w_k_weight = self.w_v_weight = self.w_g_weight = self.w_i_weight = self.w_f_weight = None

    def cache_need(self):
        return CacheNeed(state=StateNeed((ops.matrix_memory_state_size(self.H, self.D, self.Dv),), torch.float32))

    def forward(self, x, ctx, cache, residual, accumulate=True, defer=False):
        T, cap, H, D, Dv = ctx.n_tokens, ctx.token_capacity, self.H, self.D, self.Dv
        proj = ctx.buf("mmem_proj", (cap, self.w_in.shape[0]), torch.float32)
        linear(x, self.w_in, proj, STORE_F32, ctx, M=T)
        oq, ok, ov, og = 0, H * D, 2 * H * D, 2 * H * D + H * Dv
        oi = og + H * Dv
        o = ctx.buf("mmem_o", (cap, H * Dv), torch.float32)
        gates = ctx.buf("mmem_gates", (cap, 2 * H), torch.float32)
        ops.matrix_memory(proj, (oq, ok, ov, oi, oi + H), self.w_i_bias, self.w_f_bias, self.cap, T, ctx, H, D, Dv, cache.state, gates, o)
        out = ctx.buf("mmem_out", (cap, H * Dv), self.dtype)
        ops.head_gate_norm(o, proj[:, og:og + H * Dv], self.w_norm_weight, self.eps, T, H, Dv, out)
        if defer and not accumulate:
            part = linear_deferred(out, self.w_o_weight, ctx, T)
            if part is not None:
                return part
        linear(out, self.w_o_weight, residual, RESIDUAL if accumulate else STORE_F32, ctx, M=T)
        return None
