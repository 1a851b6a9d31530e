"""A pre-norm block: h += mixer(norm1(h)); h += ffn(norm2(h)).

The reference's order (crates/model/src/llama.rs:183-285; docs/ARCHITECTURE.md "Forward
pass").  The two residual sums happen inside the parts' last kernels, in float32.
"""
from __future__ import annotations

import torch

from ..ops import lib as ops
from .base import CacheNeed, FeedForward, Mixer, Norm, ParamSpec, Part, StateNeed
from .linear import STORE_F32, linear, linear_deferred


class PreNormBlock(Part):
    graph_safe = True

    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward,
                 names=("attn_norm.", "attn_", "ffn_norm.", "ffn_")):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self._names = names

    def children(self):
        return list(zip(self._names, (self.norm1, self.mixer, self.norm2, self.ffn)))

    def forward(self, h, ctx, cache):
        x = self.norm1.forward(h, ctx)
        ctx.flush_residual()            # no-op when the norm took the pending sum itself
        self.mixer.forward(x, ctx, cache, h)
        x = self.norm2.forward(h, ctx)
        ctx.flush_residual()
        self.ffn.forward(x, ctx, h)


class PostNormBlock(Part):
    """The norms sit on the sublayers' results and the sublayers read the residual row itself:

        h += ls1 * norm1(mixer(h));   h += ls2 * norm2(ffn(h))

    with norm(v) = v / sqrt(mean(v^2) + eps) * w and ls1, ls2 per-element layer scales (`layer_scale=False`: none).
    `ffn` (with norm2 and ls2) may be None.  In a 16-bit model the sublayers read the row rounded to the compute type:
    the step's buffer `residual_copy`, which the embedding fills (`TokenEmbedding(copy_dtype=...)`) and the kernel
    that adds a sublayer's normed result rewrites.  The sublayers hand their results over in a float32 buffer
    (`accumulate=False`).  The reference's block is `PreNormBlock`."""
    graph_safe = True

    def __init__(self, width, dtype, norm1: Norm, mixer: Mixer, norm2: Norm = None, ffn: FeedForward = None, layer_scale=True,
                 names=("norm1.", "mix.", "norm2.", "mlp.")):
        if (norm2 is None) != (ffn is None):
            raise ValueError("the second norm and the feed-forward come together")
        self.width, self.dtype = width, dtype
        self.norm1, self.mixer, self.norm2, self.ffn, self.layer_scale = norm1, mixer, norm2, ffn, bool(layer_scale)
        self._names = names
        self.w_ls1 = self.w_ls2 = None

    def param_specs(self):
        if not self.layer_scale:
            return {}
        out = {"ls1": ParamSpec((self.width,), kind="vector", init="ones_normal")}
        if self.ffn is not None:
            out["ls2"] = ParamSpec((self.width,), kind="vector", init="ones_normal")
        return out

    def children(self):
        out = [(self._names[0], self.norm1), (self._names[1], self.mixer)]
        if self.ffn is not None:
            out += [(self._names[2], self.norm2), (self._names[3], self.ffn)]
        return out

    def forward(self, h, ctx, cache):
        ctx.flush_residual()
        T, cap, E = ctx.n_tokens, ctx.token_capacity, self.width
        wide = self.dtype == torch.float32
        x = h if wide else ctx.buf("residual_copy", (cap, E), self.dtype)
        y = ctx.buf("post_y", (cap, E), torch.float32)
        self.mixer.forward(x, ctx, cache, y, accumulate=False)
        ctx.flush_residual()
        ops.post_norm_add(h, T, y, self.norm1.w_weight, self.w_ls1, self.norm1.eps, xc=None if wide else x)
        if self.ffn is not None:
            self.ffn.forward(x, ctx, y, accumulate=False)
            ctx.flush_residual()
            ops.post_norm_add(h, T, y, self.norm2.w_weight, self.w_ls2, self.norm2.eps, xc=None if wide else x)


# Up to this many tokens in a step the block's second chain (gates, feed-forward) runs on a second stream.
OVERLAP_MAX_TOKENS = 64


class ParallelGatedBlock(Part):
    """Both sublayers read norms of the SAME residual row and their gated results are added together:

        n = groupnorm(h);  a = n * w1;  b = n * w2
        m = a + (a of the request's previous token - a) * shift        (token shift; zeros before the first token)
        h += mixer(m) * sigmoid(G1 a + c1) + ffn(b) * sigmoid(G2 b + c2)

    One normalisation serves both weight vectors.  The previous token's `a` is part of a request's
    state (one float32 row per request and run of the block), so the block, not its mixer, asks
    the cache for it (`cache_need`).  `ffn` may be None (a layer without a feed-forward has neither
    a second norm weight nor a second gate); `token_shift=False` leaves m = a.  The sublayers hand
    their results over in float32 buffers (`accumulate=False`); a biased feed-forward's down bias
    is added in the same final kernel.  The reference has no such arrangement (its block is
    `PreNormBlock`'s)."""
    graph_safe = True

    def __init__(self, width, eps, groups, dtype, mixer: Mixer, ffn: FeedForward = None, token_shift=True,
                 names=("mix.", "mlp.")):
        if groups < 1 or width % groups:
            raise ValueError(f"{groups} groups do not divide a width of {width}")
        self.width, self.eps, self.groups, self.dtype = width, float(eps), int(groups), dtype
        self.mixer, self.ffn, self.token_shift = mixer, ffn, bool(token_shift)
        self._names = names
        self.w_norm1_weight = self.w_norm2_weight = self.w_shift_weight = None
        self.w_rg1_weight = self.w_rg1_bias = self.w_rg2_weight = self.w_rg2_bias = None
        self._rg2_fused = False

    def param_specs(self):
        E = self.width
        out = {"norm1.weight": ParamSpec((E,), kind="vector", init="ones_normal"),
               "rg1.weight": ParamSpec((E, E)), "rg1.bias": ParamSpec((E,), kind="vector")}
        if self.token_shift:
            out["shift.weight"] = ParamSpec((E,), kind="vector", init="uniform")
        if self.ffn is not None:
            out.update({"norm2.weight": ParamSpec((E,), kind="vector", init="ones_normal"),
                        "rg2.weight": ParamSpec((E, E)), "rg2.bias": ParamSpec((E,), kind="vector")})
        return out

    def children(self):
        out = [(self._names[0], self.mixer)]
        if self.ffn is not None:
            out.append((self._names[1], self.ffn))
        return out

    def cache_need(self):
        need = self.mixer.cache_need()
        if not self.token_shift:
            return need
        if need.state is not None:
            raise ValueError("the block's token shift and its mixer both want the run's state")
        return CacheNeed(paged=need.paged, state=StateNeed((self.width,), torch.float32))

    def finalize(self):
        # the second gate's product reads the same rows as the feed-forward's gate/up product: one launch
        if self.ffn is not None and getattr(self.ffn, "bias", False) and hasattr(self.ffn, "extra_rows"):
            self.ffn.extra_rows = self.w_rg2_weight
            self._rg2_fused = True
        super().finalize()
        if self._rg2_fused:
            self.w_rg2_weight = None

    def forward(self, h, ctx, cache):
        ctx.flush_residual()
        T, E, cap = ctx.n_tokens, self.width, ctx.token_capacity
        a = ctx.buf("pgb_a", (cap, E), self.dtype)
        m = ctx.buf("pgb_m", (cap, E), self.dtype)
        b = ctx.buf("pgb_b", (cap, E), self.dtype) if self.ffn is not None else None
        stage = ctx.buf("pgb_stage", (ctx.max_requests, E), torch.float32) if self.token_shift else None
        state = cache.state if self.token_shift else None
        ops.norm_pair_shift(h, self.w_norm1_weight, self.w_norm2_weight if b is not None else None,
                            self.w_shift_weight if self.token_shift else None, a, m, b, T, ctx, state, stage, self.groups,
                            self.eps)
        y1 = ctx.buf("pgb_y1", (cap, E), torch.float32)
        g1 = ctx.buf("pgb_g1", (cap, E), torch.float32)
        y2 = ctx.buf("pgb_y2", (cap, E), torch.float32) if self.ffn is not None else None
        g2 = ctx.buf("pgb_g2", (cap, E), torch.float32) if self.ffn is not None and not self._rg2_fused else None

        p1 = p2 = None

        def gates_and_ffn(defer):
            """The second chain; the feed-forward's last product may stay in partials (`defer`), so it runs last."""
            nonlocal g2, p2
            linear(a, self.w_rg1_weight, g1, STORE_F32, ctx, M=T)
            if self.ffn is not None:
                if not self._rg2_fused:
                    linear(b, self.w_rg2_weight, g2, STORE_F32, ctx, M=T)
                p2 = self.ffn.forward(b, ctx, y2, accumulate=False, defer=defer)
                ctx.flush_residual()
                if self._rg2_fused:
                    g2 = self.ffn.extra_out

        # The mixer reads m; the gates and the feed-forward read a and b: two chains that meet only in
        # the final sum.  In steps of a few tokens every kernel of a chain waits for the one before it
        # far longer than it computes, so the second chain runs on a second stream beside the first.
        if T <= OVERLAP_MAX_TOKENS and not ops.profiling() and str(ctx.device) != "cpu":
            side, fork, join = ctx.side_stream()
            main = torch.cuda.current_stream()
            fork.record(main)
            side.wait_event(fork)
            ctx.lane = 1
            try:
                with torch.cuda.stream(side):
                    gates_and_ffn(True)
                    join.record(side)
            finally:
                ctx.lane = 0
            # (each chain's last product may stay in partials of its own lane's workspace: the final kernel sums both)
            p1 = self.mixer.forward(m, ctx, cache, y1, accumulate=False, defer=True)
            main.wait_event(join)
        else:
            self.mixer.forward(m, ctx, cache, y1, accumulate=False)
            gates_and_ffn(False)
        c2 = getattr(self.ffn, "down_bias", None) if self.ffn is not None else None
        ops.gated_residual(h, T, y1 if p1 is None else None, g1, self.w_rg1_bias, y2 if p2 is None else None, c2, g2,
                           self.w_rg2_bias if y2 is not None else None,
                           ctx=ctx, stage=stage, state=state, p1=p1, p2=p2)


class TokenSideTable(Part):
    """A second embedding table [vocabulary, layers * dim]: layer i's `TokenSideInput` reads columns
    i * dim .. (i + 1) * dim of a token's row.  One table serves all layers, so the model owns it."""
    graph_safe = True

    def __init__(self, n_vocab, total_dim):
        self.n_vocab, self.total_dim = int(n_vocab), int(total_dim)
        self.w_weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.n_vocab, self.total_dim))}


class TokenSideInput(Part):
    """A token-dependent input added to the residual stream x after a block's sublayers:

        g = gelu_tanh(W_gate x) * table[token][offset : offset + dim];   y = W_proj g
        x += mult * y / sqrt(mean(y^2) + eps) * w

    The norm is a plain-weight RMS norm of the branch's result.  `table` is the model's `TokenSideTable`."""
    graph_safe = True

    def __init__(self, width, dim, offset, table: TokenSideTable, eps, dtype):
        if offset < 0 or offset + dim > table.total_dim:
            raise ValueError(f"columns {offset}..{offset + dim} are outside the side table's {table.total_dim}")
        self.width, self.dim, self.offset, self.table, self.eps, self.dtype = width, int(dim), int(offset), table, float(eps), dtype
        self.w_gate_weight = self.w_proj_weight = self.w_norm_weight = None

    def param_specs(self):
        return {"gate.weight": ParamSpec((self.dim, self.width)), "proj.weight": ParamSpec((self.width, self.dim)),
                "norm.weight": ParamSpec((self.width,), kind="vector", init="ones_normal")}

    def forward(self, h, x_in, ctx, mult):
        """h: the float32 residual rows (updated in place); x_in: the same rows in the compute type."""
        T, cap = ctx.n_tokens, ctx.token_capacity
        few = T <= OVERLAP_MAX_TOKENS       # a few tokens: both products stay in partials, summed by the kernels that follow
        s = ctx.buf("side_s", (cap, self.dim), torch.float32)
        part = linear_deferred(x_in, self.w_gate_weight, ctx, T) if few else None
        if part is None:
            linear(x_in, self.w_gate_weight, s, STORE_F32, ctx, M=T)
        g = ctx.buf("side_g", (cap, self.dim), self.dtype)
        ops.gated_table_rows(s, self.table.w_weight, ctx.token_ids, self.offset, self.dim, g, T, ctx.err, partials=part)
        y = ctx.buf("side_y", (cap, self.width), torch.float32)
        part = linear_deferred(g, self.w_proj_weight, ctx, T) if few and self.width <= ops.norm_scaled_add_max_width() else None
        if part is None:
            linear(g, self.w_proj_weight, y, STORE_F32, ctx, M=T)
        ops.norm_scaled_add(h, y, self.w_norm_weight, mult, self.eps, T, partials=part)


class ParallelBlock(Part):
    """Both sublayers read ONE norm of the residual row and their sum is scaled on its way in:

        n = norm1(x);   x += mult * (mixer(n) + ffn(n))

    then, when the block has one, a `TokenSideInput` adds its token-dependent branch (scaled by the
    same `mult`).  `ffn` may be None.  The sublayers hand their results over in float32 buffers and
    one kernel makes the scaled sum (and, for the side input's product, the new row in the compute
    type).  The reference's block is sequential (`PreNormBlock`)."""
    graph_safe = True

    def __init__(self, norm1: Norm, mixer: Mixer, ffn: FeedForward = None, mult=1.0, side: TokenSideInput = None,
                 names=("norm1.", "mix.", "mlp.", "side.")):
        self.norm1, self.mixer, self.ffn, self.mult, self.side = norm1, mixer, ffn, float(mult), side
        self._names = names

    def children(self):
        out = [(self._names[0], self.norm1), (self._names[1], self.mixer)]
        if self.ffn is not None:
            out.append((self._names[2], self.ffn))
        if self.side is not None:
            out.append((self._names[3], self.side))
        return out

    def forward(self, h, ctx, cache):
        T, cap, E = ctx.n_tokens, ctx.token_capacity, h.shape[1]
        x = self.norm1.forward(h, ctx)
        ctx.flush_residual()
        y1 = ctx.buf("par_y1", (cap, E), torch.float32)
        y2 = ctx.buf("par_y2", (cap, E), torch.float32) if self.ffn is not None else None
        p1 = p2 = None
        # The mixer and the feed-forward read the same rows and meet only in the sum.  In steps of a few
        # tokens every kernel of a chain waits for the one before it far longer than it computes: the
        # feed-forward runs on a second stream beside the mixer (products there use the second lane's
        # workspace), and each chain's last product may stay in partials that the sum adds.
        if self.ffn is not None and T <= OVERLAP_MAX_TOKENS and not ops.profiling() and str(ctx.device) != "cpu":
            side, fork, join = ctx.side_stream()
            main = torch.cuda.current_stream()
            fork.record(main)
            side.wait_event(fork)
            ctx.lane = 1
            try:
                with torch.cuda.stream(side):
                    p2 = self.ffn.forward(x, ctx, y2, accumulate=False, defer=True)
                    join.record(side)
            finally:
                ctx.lane = 0
            p1 = self.mixer.forward(x, ctx, cache, y1, accumulate=False, defer=True)
            main.wait_event(join)
        else:
            few = T <= OVERLAP_MAX_TOKENS       # (one workspace: only the last product before the sum may stay in partials)
            p1 = self.mixer.forward(x, ctx, cache, y1, accumulate=False, defer=few and self.ffn is None)
            if self.ffn is not None:
                ctx.flush_residual()
                p2 = self.ffn.forward(x, ctx, y2, accumulate=False, defer=few)
        ctx.flush_residual()
        xc = None
        if self.side is not None and self.side.dtype != torch.float32:
            xc = ctx.buf("par_xc", (cap, E), self.side.dtype)
        ops.scaled_sum(h, y1, y2, self.mult, T, xc, p1=p1, p2=p2)
        if self.side is not None:
            self.side.forward(h, xc if xc is not None else h, ctx, self.mult)


def _stream_init(kind):
    """Random-weights draws for a block's stream tensors: values near the ones that make the block a plain
    pre-norm block (read: equal shares; carry: the identity; write: ones), so that a random model stays tame."""
    def draw(shape, g, device, std):
        noise = torch.randn(shape, generator=g, device=device, dtype=torch.float32) * 0.1
        if kind == "in":
            return 1.0 / shape[0] + noise
        if kind == "mix":
            return torch.eye(shape[0], device=device, dtype=torch.float32) + noise
        return 1.0 + noise
    return draw


class StreamBlock(Part):
    """A pre-norm block over S copies X[0..S-1] of the residual stream (one row of S * width floats per
    token).  Sublayer q (the mixer, then the feed-forward) owns a read vector a_q [S], a carry matrix
    M_q [S, S] (indexed [from, to]) and a write vector b_q [S]:

        u = sum_s a_q[s] X[s];   y = sublayer(norm_q(u));   X'[t] = sum_s M_q[s, t] X[s] + b_q[t] y

    (all t at once, from the old rows).  With S = 1, a = [1], M = [[1]], b = [1] this is `PreNormBlock`.
    One kernel applies the write of the sublayer before it and makes the read and the norm of the next,
    so a sublayer's write stays pending in `ctx` (`StepContext.pending_streams`) until the next reader of
    the rows; a sublayer's last product may stay in partials for that kernel, and a routed feed-forward
    hands over its experts' result rows unsummed.  `ffn` may be None.  The model's embedding writes S
    copies of a token's row (`TokenEmbedding(copies=S)`), its last norm is a `StreamSumNorm`."""
    graph_safe = True

    def __init__(self, streams, norm1: Norm, mixer: Mixer, norm2: Norm = None, ffn: FeedForward = None,
                 names=("norm1.", "mix.", "norm2.", "mlp.")):
        if not 1 <= streams <= ops.HYPER_MAX_STREAMS:
            raise ValueError(f"{streams} residual streams are outside 1..{ops.HYPER_MAX_STREAMS}")
        if (norm2 is None) != (ffn is None):
            raise ValueError("the second norm and the feed-forward come together")
        self.streams, self.width = int(streams), norm1.width
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn
        self._names = names
        self.w_hc1_in = self.w_hc1_mix = self.w_hc1_out = self.w_hc2_in = self.w_hc2_mix = self.w_hc2_out = None

    def param_specs(self):
        S = self.streams
        out = {}
        lone = S == 1           # (a file of a model with one stream may leave them out: the plain pre-norm block)
        for q in ("hc1", "hc2") if self.ffn is not None else ("hc1",):
            out.update({q + ".in": ParamSpec((S,), kind="vector", init=_stream_init("in"), optional=lone),
                        q + ".mix": ParamSpec((S, S), kind="vector", init=_stream_init("mix"), optional=lone),
                        q + ".out": ParamSpec((S,), kind="vector", init=_stream_init("out"), optional=lone)})
        return out

    def finalize(self):
        super().finalize()
        device = self.norm1.w_weight.device
        for q in ("hc1", "hc2") if self.ffn is not None else ("hc1",):
            for k, shape in (("in", (1,)), ("mix", (1, 1)), ("out", (1,))):
                if getattr(self, f"w_{q}_{k}") is None:
                    setattr(self, f"w_{q}_{k}", torch.ones(shape, dtype=torch.float32, device=device))

    def children(self):
        out = [(self._names[0], self.norm1), (self._names[1], self.mixer)]
        if self.ffn is not None:
            out += [(self._names[2], self.norm2), (self._names[3], self.ffn)]
        return out

    def forward(self, h, ctx, cache):
        S, E, T, cap = self.streams, self.width, ctx.n_tokens, ctx.token_capacity
        few = T <= OVERLAP_MAX_TOKENS
        x = ctx.buf("stream_x", (cap, E), self.norm1.out_dtype)
        ops.hyper_step(h, S, E, T, write=ctx.take_pending_streams(h), in_w=self.w_hc1_in, norm_w=self.norm1.w_weight,
                       eps=self.norm1.eps, out=x)
        y = ctx.buf("stream_y", (cap, E), torch.float32)
        part = self.mixer.forward(x, ctx, cache, y, accumulate=False, defer=few)
        write = ops.StreamWrite(self.w_hc1_mix, self.w_hc1_out, y=y if part is None else None, partials=part)
        if self.ffn is None:
            ctx.pending_streams = (h, S, E, write)
            return
        ops.hyper_step(h, S, E, T, write=write, in_w=self.w_hc2_in, norm_w=self.norm2.w_weight, eps=self.norm2.eps, out=x)
        if hasattr(self.ffn, "forward_rows"):
            rows, row_of, top = self.ffn.forward_rows(x, ctx)
            write = ops.StreamWrite(self.w_hc2_mix, self.w_hc2_out, y=rows, y_rows=row_of, top=top)
        else:
            part = self.ffn.forward(x, ctx, y, accumulate=False, defer=few)
            write = ops.StreamWrite(self.w_hc2_mix, self.w_hc2_out, y=y if part is None else None, partials=part)
        ctx.pending_streams = (h, S, E, write)


class StreamSumNorm(Norm):
    """The last norm of a model whose blocks are `StreamBlock`s: an RMS norm of the plain sum of a token's
    S streams, after the last sublayer's pending write (applied to the asked rows only, stored nowhere)."""
    graph_safe = True

    def __init__(self, streams, width: int, eps: float, out_dtype):
        self.streams, self.width, self.eps, self.out_dtype = int(streams), width, float(eps), out_dtype
        self.w_weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.width,), kind="vector", init="ones_normal")}

    def forward(self, h, ctx, rows=None, n_rows=None, tag="norm"):
        n = n_rows if n_rows is not None else ctx.n_tokens
        cap = ctx.want_capacity if rows is not None else ctx.token_capacity
        out = ctx.buf(tag + ("_rows" if rows is not None else ""), (cap, self.width), self.out_dtype)
        write = ctx.take_pending_streams(h)
        if write is not None and rows is None:
            # every row is read: store the write first, then read
            ops.hyper_step(h, self.streams, self.width, ctx.n_tokens, write=write, store=True)
            write = None
        ops.hyper_step(h, self.streams, self.width, n, write=write, rows=rows, store=False, norm_w=self.w_weight, eps=self.eps, out=out)
        return out
