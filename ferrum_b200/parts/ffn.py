"""Dense gated feed-forward: down(act(gate(x)) * up(x)), added to the residual stream.

crates/model/src/llama.rs:261-285; silu(g) = g / (1 + exp(-g)) (crates/kernels/src/math.rs:8-10).
Gate and up are stored as one matrix [2F, E] so that one kernel reads x once; on the
tensor-core path that kernel also applies the activation (two accumulators, one epilogue).

`bias=True` gives every projection a bias vector (the reference refuses biases,
crates/model/src/weights.rs:165-167): gate and up then leave their product in float32, one
kernel adds the biases and applies the activation, and the down bias is either added by a block
that sums the sublayer's result itself (`accumulate=False`; it reads `down_bias`) or, when the
part adds into the residual stream, is not supported.  `act` names the activation of the gate
("silu", "gelu_tanh", or "swish_clamp": g = min(gate, limit), u = clamp(up, -limit, limit),
g sigmoid(1.702 g) (u + 1), a unit made of both values); gelu_tanh and swish_clamp without biases have their own epilogues of the tensor-core product
too, and elsewhere (a few tokens, rows the tensor cores refuse) takes the float32 gate/up path.  `extra_rows` appends further weight rows to the gate/up matrix: a
block that needs another product of the same input gets it from the same launch
(`forward(..., extra_out=...)` returns a view of those columns).
"""
from __future__ import annotations

import torch

from ..ops import lib as ops
from .base import FeedForward, ParamSpec
from .linear import RESIDUAL, STORE, STORE_F32, linear, linear_deferred, linear_swiglu


# Up to this many tokens in a step a routed feed-forward's unit for every token runs on a second stream beside the routing.
SIDE_STREAM_MAX_TOKENS = 64


class SwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, width, hidden, dtype, bias=False, act="silu", wide_products=False, limit=0.0):
        """wide_products: where gate and up do not run on the fused tensor-core kernel (rows that are no
        16-byte multiples), they stay float32 until the activation has been applied, so that the
        activation's input is rounded nowhere; without it that path stores them in the compute type."""
        if act not in ops.GLU_ACTS:
            raise ValueError(f"unknown activation {act!r}")
        self.width, self.hidden, self.dtype, self.bias, self.act = width, hidden, dtype, bool(bias), act
        self.wide_products = bool(wide_products)
        self.limit = float(limit)
        if act == "swish_clamp" and not self.limit > 0.0:
            raise ValueError("the clamped unit needs a positive limit")
        self.w_gate_weight = self.w_up_weight = self.w_down_weight = None
        self.w_gate_bias = self.w_up_bias = self.w_down_bias = None
        self.w_gate_up = None
        self.extra_rows = None          # set by a block before finalize: [n, width] rows appended to gate/up
        self.extra_out = None           # float32 [T, n] view of the extra product of the last forward

    def param_specs(self):
        out = {"gate.weight": ParamSpec((self.hidden, self.width)),
               "up.weight": ParamSpec((self.hidden, self.width)),
               "down.weight": ParamSpec((self.width, self.hidden))}
        if self.bias:
            out.update({"gate.bias": ParamSpec((self.hidden,), kind="vector", init="normal"),
                        "up.bias": ParamSpec((self.hidden,), kind="vector", init="normal"),
                        "down.bias": ParamSpec((self.width,), kind="vector", init="normal")})
        return out

    @property
    def down_bias(self):
        return self.w_down_bias

    def finalize(self):
        rows = [self.w_gate_weight, self.w_up_weight]
        if self.extra_rows is not None:
            if not self.bias:
                raise ValueError("extra rows ride on the float32 gate/up product of the biased path")
            rows.append(self.extra_rows)
        self.w_gate_up = torch.cat(rows, dim=0).contiguous()
        self.w_gate_weight = self.w_up_weight = self.extra_rows = None

    def forward(self, x, ctx, residual, accumulate=True, defer=False):
        F, T = self.hidden, ctx.n_tokens
        act = ctx.buf("ffn_act", (ctx.token_capacity, F), self.dtype)
        if self.bias or self.act != "silu":       # (the fused gate/up kernels apply silu and add no bias)
            if self.bias and accumulate:
                raise ValueError("a biased feed-forward hands its result to a block that adds the down bias")
            n = self.w_gate_up.shape[0]
            # a few tokens: the product stays in partials and the activation kernel sums them
            part = linear_deferred(x, self.w_gate_up, ctx, T) if ctx.defer_swiglu else None
            if part is not None:
                self.extra_out = ctx.buf("ffn_extra", (ctx.token_capacity, n - 2 * F), torch.float32) if n > 2 * F else None
                ops.bias_glu_reduce(part, self.w_gate_bias, self.w_up_bias, act, T, F, self.act, extra=self.extra_out, limit=self.limit)
            elif not self.bias and n == 2 * F and ops.gemm_tc_supported(x, self.w_gate_up):
                linear_swiglu(x, self.w_gate_up, act, F, ctx, M=T, kind=self.act, limit=self.limit)   # the activation in the product's epilogue
            else:
                gu = ctx.buf("ffn_gate_up_f32", (ctx.token_capacity, n), torch.float32)
                linear(x, self.w_gate_up, gu, STORE_F32, ctx, M=T)
                self.extra_out = gu[:, 2 * F:] if n > 2 * F else None
                ops.bias_glu(gu, self.w_gate_bias, self.w_up_bias, act, T, F, self.act, limit=self.limit)
        elif ops.gemm_tc_supported(x, self.w_gate_up):
            linear_swiglu(x, self.w_gate_up, act, F, ctx, M=T)
        elif self.wide_products and self.dtype != torch.float32:
            gu = ctx.buf("ffn_gate_up_f32", (ctx.token_capacity, 2 * F), torch.float32)
            linear(x, self.w_gate_up, gu, STORE_F32, ctx, M=T)
            ops.bias_glu(gu, None, None, act, T, F, self.act)
        else:
            gu = ctx.buf("ffn_gate_up", (ctx.token_capacity, 2 * F), self.dtype)
            linear(x, self.w_gate_up, gu, STORE, ctx, M=T)
            ops.swiglu(gu, act, T, F)
        if defer and not accumulate:
            part = linear_deferred(act, self.w_down_weight, ctx, T)
            if part is not None:
                return part
        linear(act, self.w_down_weight, residual, RESIDUAL if accumulate else STORE_F32, ctx, M=T)
        return None


class RoutedFeedForward(FeedForward):
    """A mixture of experts: every token runs through `top` of `n_experts` small gated feed-forwards
    down_e(act(gate_e z) * (up_e z)), chosen by a router.

    router logits   W_router x in float32 (x in the compute type)
    scores          "sigmoid" of each logit, or "softmax" over all experts
    choice          the `top` largest scores (a tie goes to the lower index)
    weights         the chosen scores, divided by their sum when `renormalize`
    scale_input     True: an expert sees z = weight * x and its result is added as it is;
                    False: it sees x and its result is multiplied by the weight
    correction      a vector added to the scores for the choice alone (the weights stay the plain scores)
    weight_scale    multiplies the chosen weights
    identity        this many further router outputs stand for identity experts (no matrices): their result
                    is the token's own input row, times the weight
    limit           the clamp of act "swish_clamp"
    shared          a `FeedForward` that every token runs through; its result joins the sum

    The tokens' rows are gathered into a buffer sorted by expert; two grouped products (gate/up with
    the activation, then down) run over it with the experts' stacked matrices, every CTA finding its
    expert from per-expert counters on the device, so a step's launches depend on the batch's sizes
    only.  `forward_rows` hands the unsummed result rows to a block that adds them itself;
    `forward(accumulate=False)` sums them into the block's buffer."""
    graph_safe = True

    def __init__(self, width, hidden, n_experts, top, dtype, act="silu", scores="sigmoid", renormalize=False, scale_input=True,
                 correction=False, weight_scale=1.0, identity=0, limit=0.0, shared: FeedForward = None):
        if act not in ops.GLU_ACTS:
            raise ValueError(f"unknown activation {act!r}")
        if scores not in ops.MOE_SCORES:
            raise ValueError(f"unknown router scores {scores!r}")
        identity = int(identity)
        if not (0 < top <= n_experts + identity <= ops.MOE_MAX_EXPERTS and top <= ops.MOE_MAX_TOP and n_experts > 0 and identity >= 0):
            raise ValueError(f"{top} of {n_experts} + {identity} experts per token are outside the routing kernel's limits "
                             f"({ops.MOE_MAX_TOP} of {ops.MOE_MAX_EXPERTS})")
        if identity and scale_input:
            raise ValueError("identity experts go with weights on the experts' results")
        if act == "swish_clamp" and not limit > 0.0:
            raise ValueError("the clamped unit needs a positive limit")
        self.has_correction, self.weight_scale, self.identity = bool(correction), float(weight_scale), identity
        self.limit, self.shared = float(limit), shared
        self.w_correction = None
        self.width, self.hidden, self.n_experts, self.top, self.dtype = width, hidden, int(n_experts), int(top), dtype
        self.act, self.scores, self.renormalize, self.scale_input = act, scores, bool(renormalize), bool(scale_input)
        self.w_router_weight = self.w_gate_up = self.w_down = None

    def param_specs(self):
        out = {"router.weight": ParamSpec((self.n_experts + self.identity, self.width))}
        if self.has_correction:
            out["correction"] = ParamSpec((self.n_experts + self.identity,), kind="vector", init="normal")
        for e in range(self.n_experts):
            out.update({f"e{e}.gate.weight": ParamSpec((self.hidden, self.width)),
                        f"e{e}.up.weight": ParamSpec((self.hidden, self.width)),
                        f"e{e}.down.weight": ParamSpec((self.width, self.hidden))})
        return out

    def children(self):
        return [("shared.", self.shared)] if self.shared is not None else []

    def finalize(self):
        super().finalize()

        def take(name):
            t = getattr(self, name)
            delattr(self, name)
            return t
        gu = [torch.cat([take(f"w_e{e}_gate_weight"), take(f"w_e{e}_up_weight")], dim=0) for e in range(self.n_experts)]
        self.w_gate_up = torch.stack(gu, dim=0).contiguous()                       # [experts, 2F, E]
        self.w_down = torch.stack([take(f"w_e{e}_down_weight") for e in range(self.n_experts)], dim=0).contiguous()   # [experts, E, F]

    def forward_rows(self, x, ctx):
        """(rows float32 [T * top, width], row_of int32 [T * top], top): token t's result is the sum over j of
        rows[row_of[t * top + j]] (already weighted when the weight scales the expert's input)."""
        T, cap, top, n = ctx.n_tokens, ctx.token_capacity, self.top, self.n_experts
        n_out = n + self.identity
        logits = ctx.buf("moe_logits", (cap, n_out), torch.float32)
        linear(x, self.w_router_weight, logits, STORE_F32, ctx, M=T)
        expert_of = ctx.buf("moe_expert_of", (cap * top,), torch.int32)
        rank_of = ctx.buf("moe_rank_of", (cap * top,), torch.int32)
        row_of = ctx.buf("moe_row_of", (cap * top,), torch.int32)
        weight_of = ctx.buf("moe_weight_of", (cap * top,), torch.float32)
        counts = ctx.buf("moe_counts", (n,), torch.int32)
        xg = ctx.buf("moe_x", (cap * top, self.width), self.dtype)
        ops.moe_route(logits, T, n_out, top, x, self.scale_input, expert_of, rank_of, weight_of, counts, xg, row_of,
                      scores=self.scores, renormalize=self.renormalize, correction=self.w_correction if self.has_correction else None,
                      weight_scale=self.weight_scale, n_identity=self.identity)
        act = ctx.buf("moe_act", (cap * top, self.hidden), self.dtype)
        ops.moe_gemm(xg, self.w_gate_up, counts, T * top, act, self.hidden, glu=self.act, err=ctx.err, limit=self.limit)
        rows = ctx.buf("moe_rows", (cap * top, self.width), torch.float32)
        ops.moe_gemm(act, self.w_down, counts, T * top, rows, self.width, err=ctx.err)
        self._weight_of = weight_of
        return rows, row_of, top

    def forward(self, x, ctx, residual, accumulate=True, defer=False):
        if accumulate:
            raise ValueError("a routed feed-forward hands its result to a block that adds it")
        add = join = None
        if self.shared is not None:
            add = ctx.buf("moe_shared", (ctx.token_capacity, self.width), torch.float32)
            if ctx.n_tokens <= SIDE_STREAM_MAX_TOKENS and not ops.profiling() and str(ctx.device) != "cpu":
                # The unit for every token and the routed experts meet only in the sum.  In steps of a few tokens every
                # kernel of a chain waits for the one before it far longer than it computes: the unit runs on a second
                # stream beside the routing (its products use the second lane's workspace).
                ctx.flush_residual()
                side, fork, join = ctx.side_stream()
                fork.record(torch.cuda.current_stream())
                side.wait_event(fork)
                ctx.lane = 1
                try:
                    with torch.cuda.stream(side):
                        self.shared.forward(x, ctx, add, accumulate=False)
                        ctx.flush_residual()
                        join.record(side)
                finally:
                    ctx.lane = 0
            else:
                self.shared.forward(x, ctx, add, accumulate=False)
                ctx.flush_residual()
        rows, row_of, top = self.forward_rows(x, ctx)
        if join is not None:
            torch.cuda.current_stream().wait_event(join)
        ops.moe_combine(rows, row_of, top, ctx.n_tokens, residual, weight_of=None if self.scale_input else self._weight_of,
                        x=x if self.identity else None, add=add)
        return None
