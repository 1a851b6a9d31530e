"""Two mixers side by side: both read the same rows, each result is RMS-normed over the width with a
plain weight of its own, and the mixer's result is half their sum,

    y = (rms(left(x)) * w_left + rms(right(x)) * w_right) / 2,    rms(v) = v / sqrt(mean(v^2) + eps).

The two may keep different things per request (one pages, the other a state row): the part asks the
cache for both and hands each mixer the same `LayerCache`.  The reference has one mixer per layer
(crates/model/src/llama.rs:185-257).
"""
from __future__ import annotations

import torch

from ..ops import lib as ops
from .base import CacheNeed, Mixer, ParamSpec


# Up to this many tokens in a step the right mixer runs on a second stream beside the left one.
SIDE_STREAM_MAX_TOKENS = 64


class ParallelMixer(Mixer):
    graph_safe = True

    def __init__(self, width, left: Mixer, right: Mixer, eps, names=("left.", "right.")):
        self.width, self.left, self.right, self.eps = width, left, right, float(eps)
        self._names = names
        self.w_left_out = self.w_right_out = None

    def param_specs(self):
        return {"left_out": ParamSpec((self.width,), kind="vector", init="ones_normal"),
                "right_out": ParamSpec((self.width,), kind="vector", init="ones_normal")}

    def children(self):
        return [(self._names[0], self.left), (self._names[1], self.right)]

    def cache_need(self):
        a, b = self.left.cache_need(), self.right.cache_need()
        if (a.paged is not None and b.paged is not None) or (a.state is not None and b.state is not None):
            raise ValueError("the two mixers of a parallel pair want the same kind of cache")
        return CacheNeed(paged=a.paged or b.paged, state=a.state or b.state)

    def plan(self, ctx, cache):
        self.left.plan(ctx, cache)
        self.right.plan(ctx, cache)

    def forward(self, x, ctx, cache, residual, accumulate=True, defer=False):
        if accumulate:
            raise ValueError("a parallel pair hands its result to a block that norms it")
        cap, E = ctx.token_capacity, self.width
        ya = ctx.buf("pair_left", (cap, E), torch.float32)
        yb = ctx.buf("pair_right", (cap, E), torch.float32)
        if ctx.n_tokens <= SIDE_STREAM_MAX_TOKENS and not ops.profiling() and str(ctx.device) != "cpu":
            # The two meet only in the sum.  In steps of a few tokens every kernel of a chain waits for the one before it far
            # longer than it computes: the right mixer runs on a second stream beside the left one (its products use the
            # second lane's workspace; the two keep different things of the cache and use scratch buffers of their own).
            ctx.flush_residual()
            side, fork, join = ctx.side_stream()
            main = torch.cuda.current_stream()
            fork.record(main)
            side.wait_event(fork)
            ctx.lane = 1
            try:
                with torch.cuda.stream(side):
                    self.right.forward(x, ctx, cache, yb, accumulate=False)
                    ctx.flush_residual()
                    join.record(side)
            finally:
                ctx.lane = 0
            self.left.forward(x, ctx, cache, ya, accumulate=False)
            ctx.flush_residual()
            main.wait_event(join)
        else:
            self.left.forward(x, ctx, cache, ya, accumulate=False)
            ctx.flush_residual()
            self.right.forward(x, ctx, cache, yb, accumulate=False)
            ctx.flush_residual()
        ops.dual_norm_mean(ya, yb, self.w_left_out, self.w_right_out, self.eps, residual, ctx.n_tokens)
        return None
