"""Grouped-query attention over the paged cache whose heads are shaped before and after the softmax.

What a configuration may switch on, each with its constants as parameters:

  rotary         q and k turn over their leading `rope_dim` elements (a `RotaryEmbedding`, which also
                 carries the pairing and any scaling of the frequencies); None: positions enter otherwise
  unit_norm      after the turn, every q and k head is divided by its root mean square (no weight)
  value_rotary   the value of position j turns by j over all of its elements before it is cached, and
                 every head's result at position i turns back by i (a `RotaryEmbedding` over vdim)
  distance_penalty   r1[h] * ln(1 + r2[h] * (i - j)) is taken off the scaled score (r1, r2: tensors)
  gate           the heads' results are multiplied by sigmoid(W_g x) before the output projection
  window         a query sees itself and the window - 1 keys before it (0: all); with mask="chunk"
                 positions are cut into chunks of `window` from position 0 and a query sees the keys of
                 its own chunk up to itself
  dim != vdim    key and value heads of different sizes share pages of max(dim, vdim)-element rows
  qkv_bias       q, k and v projections have bias vectors
  qk_norm        every q and k head is divided by its root mean square and multiplied by a weight
                 vector shared by all heads, BEFORE the turn; "whole": the root mean square runs over a
                 token's whole query (key) projection, all heads at once, and the weight vector is as
                 long as that projection
  value_from_key no value matrix: the value of a KV head is its key head as projected (before norm and
                 turn); vdim = dim
  score_softcap  c > 0: the scaled score becomes c * tanh(score / c)
  sink           a key of score 0 without a value joins every softmax: weight_j = e^(s_j) / (1 + sum e^s)
  query_temperature  (coef, every): a query at position p is multiplied by
                 1 + coef * ln(floor((p + 1) / every) + 1)
  linear_bias    per-head slopes m[h]: m[h] * (i - j) is taken off the scaled score (numbers, not tensors)
  value_mix      "first": this layer leaves its values (float32, before rounding) in a buffer of the
                 step named `value_mix_key`; "blend": its values become (1 - lambda) v + lambda v_first
                 with the scalar tensor `vmix` before they are cached.  The layers that share a key
                 must agree on kv heads x vdim.

Scores, softmax weights, the weighted sum, rotations, the unit norm and the gate are float32 whatever
the compute type (the CUDA-core attention kernel; keys, values and queries are stored in the compute
type).  One product makes [q | k | v | gate logits] as float32 rows, `qkv_shape` shapes the heads
and writes the cache, the attention kernel leaves float32 results, `attention_finish` turns them back,
gates them and rounds once for the output projection.  The reference's attention has none of these
(crates/model/src/llama.rs:185-257).
"""
from __future__ import annotations

import torch

from ..ops import lib as ops
from .attention import PagedAttention
from .base import CacheNeed, PagedKVNeed, ParamSpec
from .linear import RESIDUAL, STORE_F32, linear, linear_deferred


class ShapedAttention(PagedAttention):
    graph_safe = True       # the CUDA-core attention kernel reads no work lists

    def __init__(self, width, n_head, n_head_kv, dim, vdim, dtype, scale, eps=1e-6, window=0, rotary=None, unit_norm=False,
                 value_rotary=None, distance_penalty=False, gate=False, mask="window", qkv_bias=False, qk_norm=False,
                 query_temperature=None, linear_bias=None, value_mix=None, value_mix_key="v_first", value_from_key=False,
                 score_softcap=0.0, sink=False):
        super().__init__(width, n_head, n_head_kv, max(int(dim), int(vdim)), rotary, dtype, window=window, scale=scale)
        self.score_softcap, self.sink = float(score_softcap or 0.0), bool(sink)
        self.value_from_key = bool(value_from_key)
        if self.value_from_key and (int(dim) != int(vdim) or qkv_bias or value_rotary is not None or value_mix is not None):
            raise ValueError("values taken from the keys have the keys' size, no bias, no turn and no blend")
        if qk_norm not in (False, True, "head", "whole"):
            raise ValueError(f"unknown query/key norm {qk_norm!r}")
        self.whole_norm = qk_norm == "whole"
        self.Dk, self.Dv, self.eps = int(dim), int(vdim), float(eps)
        self.unit_norm, self.value_rotary = bool(unit_norm), value_rotary
        self.has_penalty, self.has_gate = bool(distance_penalty), bool(gate)
        if mask not in ("window", "chunk"):
            raise ValueError(f"unknown mask {mask!r}")
        self.chunked = mask == "chunk" and self.window > 0
        self.has_bias, self.qk_norm = bool(qkv_bias), bool(qk_norm)
        self.q_temp = None
        if query_temperature is not None:
            coef, every = float(query_temperature[0]), int(query_temperature[1])
            if every <= 0:
                raise ValueError("the query temperature's step must be positive")
            self.q_temp = (coef, every)
        self.linear_bias = [float(v) for v in linear_bias] if linear_bias is not None else None
        if self.linear_bias is not None and (len(self.linear_bias) != n_head or self.has_penalty):
            raise ValueError("a linear distance bias has one slope per query head and excludes the logarithmic penalty")
        if value_mix not in (None, "first", "blend"):
            raise ValueError(f"unknown value mixing role {value_mix!r}")
        self.value_mix, self.value_mix_key = value_mix, str(value_mix_key)
        self.w_q_bias = self.w_k_bias = self.w_v_bias = self.w_q_norm_weight = self.w_k_norm_weight = self.w_vmix = None
        self.w_bias = self.slopes = None
        if rotary is not None and rotary.rope_dim > self.Dk:
            raise ValueError("the rotary table turns more elements than a key head has")
        if value_rotary is not None and value_rotary.rope_dim != self.Dv:
            raise ValueError("the value rotation covers all of a value head")
        self.w_r1 = self.w_r2 = self.w_g_weight = None
        self.w_in = None

    def param_specs(self):
        E = self.width
        out = {"q.weight": ParamSpec((self.Hq * self.Dk, E)), "k.weight": ParamSpec((self.Hkv * self.Dk, E)),
               "v.weight": ParamSpec((self.Hkv * self.Dv, E)), "output.weight": ParamSpec((E, self.Hq * self.Dv))}
        if self.value_from_key:
            del out["v.weight"]
        if self.has_penalty:
            out["r1"] = ParamSpec((self.Hq,), kind="vector", init="uniform")
            out["r2"] = ParamSpec((self.Hq,), kind="vector", init="uniform")
        if self.has_gate:
            out["g.weight"] = ParamSpec((self.Hq * self.Dv, E))
        if self.has_bias:
            out.update({"q.bias": ParamSpec((self.Hq * self.Dk,), kind="vector"), "k.bias": ParamSpec((self.Hkv * self.Dk,), kind="vector"),
                        "v.bias": ParamSpec((self.Hkv * self.Dv,), kind="vector")})
        if self.qk_norm:
            nq, nk = (self.Hq * self.Dk, self.Hkv * self.Dk) if self.whole_norm else (self.Dk, self.Dk)
            out.update({"q.norm.weight": ParamSpec((nq,), kind="vector", init="ones_normal"),
                        "k.norm.weight": ParamSpec((nk,), kind="vector", init="ones_normal")})
        if self.value_mix is not None:
            out["vmix"] = ParamSpec((), kind="vector", init="uniform")      # (read by the blending layers only)
        return out

    def finalize(self):
        rows = [self.w_q_weight, self.w_k_weight] + ([] if self.value_from_key else [self.w_v_weight])
        rows += [self.w_g_weight] if self.has_gate else []
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_q_weight = self.w_k_weight = self.w_v_weight = self.w_g_weight = None
        if self.has_bias:
            self.w_bias = torch.cat([self.w_q_bias, self.w_k_bias, self.w_v_bias]).contiguous()
            self.w_q_bias = self.w_k_bias = self.w_v_bias = None
        if self.linear_bias is not None:
            self.slopes = torch.tensor(self.linear_bias, dtype=torch.float32, device=self.w_in.device)
        if self.w_vmix is not None:
            self.w_vmix = self.w_vmix.reshape(1).contiguous()

    def cache_need(self):
        return CacheNeed(paged=PagedKVNeed(self.Hkv, self.D, self.window))

    def plan(self, ctx, cache):
        return None

    def forward(self, x, ctx, cache, residual, accumulate=True, defer=False):
        T, Hq, Hkv, Dk, Dv, Dp = ctx.n_tokens, self.Hq, self.Hkv, self.Dk, self.Dv, self.D
        cap = ctx.token_capacity
        proj = ctx.buf("sattn_proj", (cap, self.w_in.shape[0]), torch.float32)
        linear(x, self.w_in, proj, STORE_F32, ctx, M=T)
        table = ctx.block_tables[cache.group]
        q = ctx.buf("sattn_q", (cap, Hq * Dp), self.dtype)
        rot, vrot = self.position, self.value_rotary
        mix = None
        if self.value_mix is not None and cache.writes:
            first = ctx.buf(self.value_mix_key, (cap, Hkv * Dv), torch.float32)
            mix = ("store", first) if self.value_mix == "first" else ("blend", first, self.w_vmix)
        ops.qkv_shape(proj, T, ctx, table, rot, rot.pairing if rot is not None else 0,
                      vrot.cos_sin if vrot is not None else None, vrot.pairing if vrot is not None else 0, self.unit_norm,
                      self.eps, q, cache.plane, cache.page_stride, cache.page_size, Hq, Hkv, Dk, Dv, Dp, cache.writes,
                      bias=self.w_bias, q_norm=self.w_q_norm_weight if self.qk_norm else None,
                      k_norm=self.w_k_norm_weight if self.qk_norm else None, q_temp=self.q_temp, value_mix=mix,
                      whole_norm=self.whole_norm, value_from_key=self.value_from_key)
        penalty = (self.w_r1, self.w_r2) if self.has_penalty else ((self.slopes, None) if self.slopes is not None else None)
        out = ctx.buf("sattn_out", (cap, Hq * Dv), self.dtype)
        if Dp == Dv and vrot is None and not self.has_gate:
            # nothing is left to do to the heads' results: the attention kernel rounds its float32 sums once into `out`
            self._generic(q, out, ctx, cache, table, penalty)
        else:
            o = ctx.buf("sattn_o", (cap, Hq * Dp), torch.float32)
            self._generic(q, o, ctx, cache, table, penalty)
            self._finish(o, out, proj, ctx, vrot)
        if defer and not accumulate:
            part = linear_deferred(out, self.w_output_weight, ctx, T)
            if part is not None:
                return part
        linear(out, self.w_output_weight, residual, RESIDUAL if accumulate else STORE_F32, ctx, M=T)
        return None

    def _finish(self, o, out, proj, ctx, vrot):
        """Turn back, gate, drop the padding past vdim and round once."""
        T, Hq, Hkv, Dk, Dv, Dp = ctx.n_tokens, self.Hq, self.Hkv, self.Dk, self.Dv, self.D
        off = Hq * Dk + Hkv * (Dk if self.value_from_key else Dk + Dv)
        gate = proj[:, off:off + Hq * Dv] if self.has_gate else None
        ops.attention_finish(o, T, ctx, vrot.cos_sin if vrot is not None else None, vrot.pairing if vrot is not None else 0,
                             gate, out, Hq, Dv, Dp)
