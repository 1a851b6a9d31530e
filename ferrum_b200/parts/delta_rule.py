"""A gated delta rule with one decay per head and key channel.

With H value heads of Dv and G query/key heads of D (value head h reads query/key head h / (H / G)),
per token: q, k (G x D) and v (H x Dv) are projections of the input that pass a short causal
convolution per channel (no bias, zeros before the sequence) and silu; q and k heads become unit
vectors (x / sqrt(sum x^2 + 1e-6)), q also times D^(-1/2); beta = sigmoid(W_b x) per head; one decay
per head and key channel, dec = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 x) + dt_bias)), whose logits
come through a low-rank pair of matrices.  Per head, with S (D x Dv, float32, zero before the first
token):

    S <- dec * S (row d by dec_d);   e = beta (v - S^T k);   S <- S + k e^T;   o = S^T q

so the read-out sees the current token's write.  Each head's o is divided by its root mean square,
multiplied by a weight vector shared by the heads and by sigmoid(W_g2 (W_g1 x)), and projected back.
A request's state row keeps S and the convolution's last taps - 1 inputs, both float32; the walk
over a portion's tokens is sequential, so a token's result does not depend on how the sequence was
cut into steps.  Everything after the projections is float32.  The reference has no recurrent mixer
(crates/model/src/llama.rs:185-257 is its only one).
"""
from __future__ import annotations

import math

import torch

from ..ops import lib as ops
from .base import CacheNeed, Mixer, ParamSpec, StateNeed
from .linear import RESIDUAL, STORE, STORE_F32, linear, linear_deferred


def _draw_a_log(shape, g, device, std):
    """ln of a decay rate drawn from U(0.5, 4)."""
    return torch.log(0.5 + 3.5 * torch.rand(shape, generator=g, device=device, dtype=torch.float32))


def _draw_dt_bias(shape, g, device, std):
    """The inverse softplus of a step size drawn log-uniformly from [0.001, 0.1]."""
    dt = torch.exp(torch.rand(shape, generator=g, device=device, dtype=torch.float32) * math.log(100.0) + math.log(0.001))
    return dt + torch.log(-torch.expm1(-dt))


def _draw_taps(shape, g, device, std):
    """Convolution taps of a size that lets a token's neighbours matter: N(0, 0.5)."""
    return torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.5


class ChannelDeltaMixer(Mixer):
    graph_safe = True

    def __init__(self, width, heads, kv_heads, dim, vdim, taps, eps, dtype, decay_rank=None, gate_rank=None):
        """decay_rank, gate_rank: the inner sizes of the two low-rank pairs; None: whatever the weights' file has
        (random weights are then drawn with half the key size)."""
        if heads % kv_heads:
            raise ValueError("kv_heads does not divide heads")
        if not (0 < dim <= ops.RECURRENT_MAX_DIM and 0 < taps <= ops.DELTA_MAX_TAPS):
            raise ValueError(f"key size {dim} or {taps} taps are outside the kernel's limits "
                             f"({ops.RECURRENT_MAX_DIM}, {ops.DELTA_MAX_TAPS})")
        self.width, self.H, self.G, self.D, self.Dv = width, int(heads), int(kv_heads), int(dim), int(vdim)
        self.taps, self.eps, self.dtype = int(taps), float(eps), dtype
        self._free_ranks = (decay_rank is None, gate_rank is None)
        self.ra = int(decay_rank) if decay_rank is not None else max(1, self.D // 2)
        self.rg = int(gate_rank) if gate_rank is not None else max(1, self.D // 2)
        self.channels = 2 * self.G * self.D + self.H * self.Dv
        for n in ("q_weight", "k_weight", "v_weight", "b_weight", "q_conv", "k_conv", "v_conv", "a1_weight", "a2_weight",
                  "g1_weight", "g2_weight", "dt_bias", "A_log", "norm_weight", "o_weight"):
            setattr(self, "w_" + n, None)
        self.w_in = self.w_low = self.w_conv = None

    def param_specs(self):
        E, H, G, D, Dv = self.width, self.H, self.G, self.D, self.Dv
        return {"q.weight": ParamSpec((G * D, E)), "k.weight": ParamSpec((G * D, E)), "v.weight": ParamSpec((H * Dv, E)),
                "q.conv": ParamSpec((G * D, self.taps), kind="vector", init=_draw_taps),
                "k.conv": ParamSpec((G * D, self.taps), kind="vector", init=_draw_taps),
                "v.conv": ParamSpec((H * Dv, self.taps), kind="vector", init=_draw_taps),
                "b.weight": ParamSpec((H, E)),
                "a1.weight": ParamSpec((self.ra, E), free=(0,) if self._free_ranks[0] else ()),
                "a2.weight": ParamSpec((H * D, self.ra), free=(1,) if self._free_ranks[0] else ()),
                "g1.weight": ParamSpec((self.rg, E), free=(0,) if self._free_ranks[1] else ()),
                "g2.weight": ParamSpec((H * Dv, self.rg), free=(1,) if self._free_ranks[1] else ()),
                "dt_bias": ParamSpec((H * D,), kind="vector", init=_draw_dt_bias),
                "A_log": ParamSpec((H,), kind="vector", init=_draw_a_log),
                "norm.weight": ParamSpec((Dv,), kind="vector", init="ones_normal"),
                "o.weight": ParamSpec((E, H * Dv))}

    def finalize(self):
        self.ra, self.rg = self.w_a1_weight.shape[0], self.w_g1_weight.shape[0]
        if self.w_a2_weight.shape[1] != self.ra or self.w_g2_weight.shape[1] != self.rg:
            raise ValueError("the two matrices of a low-rank pair disagree on their inner size")
        # one product for what the recurrence reads in float32, one for the two low-rank inputs (compute type)
        self.w_in = torch.cat([self.w_q_weight, self.w_k_weight, self.w_v_weight, self.w_b_weight], dim=0).contiguous()
        self.w_low = torch.cat([self.w_a1_weight, self.w_g1_weight], dim=0).contiguous()
        self.w_conv = torch.cat([self.w_q_conv, self.w_k_conv, self.w_v_conv], dim=0).contiguous()
        self.w_q_weight = self.w_k_weight = self.w_v_weight = self.w_b_weight = self.w_a1_weight = self.w_g1_weight = None
        self.w_q_conv = self.w_k_conv = self.w_v_conv = None

    def cache_need(self):
        return CacheNeed(state=StateNeed((self.H * self.D * self.Dv + (self.taps - 1) * self.channels,), torch.float32))

    def forward(self, x, ctx, cache, residual, accumulate=True, defer=False):
        T, cap, H, D, Dv = ctx.n_tokens, ctx.token_capacity, self.H, self.D, self.Dv
        proj = ctx.buf("delta_proj", (cap, self.w_in.shape[0]), torch.float32)
        linear(x, self.w_in, proj, STORE_F32, ctx, M=T)
        low = ctx.buf("delta_low", (cap, self.ra + self.rg), self.dtype)
        linear(x, self.w_low, low, STORE, ctx, M=T)
        logit = ctx.buf("delta_decay_logit", (cap, H * D), torch.float32)
        linear(low[:, :self.ra], self.w_a2_weight, logit, STORE_F32, ctx, M=T)
        gate = ctx.buf("delta_gate_logit", (cap, H * Dv), torch.float32)
        linear(low[:, self.ra:], self.w_g2_weight, gate, STORE_F32, ctx, M=T)
        qkv = ctx.buf("delta_qkv", (cap, self.channels), torch.float32)
        dec = ctx.buf("delta_dec", (cap, H * D + H), torch.float32)
        o = ctx.buf("delta_o", (cap, H * Dv), torch.float32)
        ops.delta_rule(proj, logit, T, ctx, self.w_conv, self.w_dt_bias, self.w_A_log, H, self.G, D, Dv, cache.state, qkv, dec, o)
        out = ctx.buf("delta_out", (cap, H * Dv), self.dtype)
        ops.head_gate_norm(o, gate, self.w_norm_weight, self.eps, T, H, Dv, out)
        if defer and not accumulate:
            part = linear_deferred(out, self.w_o_weight, ctx, T)
            if part is not None:
                return part
        linear(out, self.w_o_weight, residual, RESIDUAL if accumulate else STORE_F32, ctx, M=T)
        return None
