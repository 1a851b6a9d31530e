"""Pererax on the GPU against the plain implementation (plain_pererax.py): every mechanism alone,
then whole models under every way of cutting the work, then generation through the engine."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_pererax as P
from helpers import Replay, assert_close_16bit, assert_close_f32, mixed_schedule, pages_were_reused, peak_pages
from pererax_configs import PERERAX, write_model

pytestmark = pytest.mark.gpu
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}
F64 = torch.float64

# Two attention layers with windows and nothing that carries further: what a token can reach is bounded.
PERERAX_W = {
    "architecture": "Pererax", "vocab": 90, "width": 40, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.4, "mask": {"size": 9},
                                        "rot": {"base": 50.0, "dims": 4}},
         "mlp": {"kind": "moe", "expert": {"ff": 16, "limit": 2.0}, "router": {"experts": 2, "identity": 1, "top": 2, "scale": 1.0}}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 6, "vdim": 6, "scale": 0.5, "mask": {"size": 6},
                                        "rot": {"base": 50.0, "dims": 6}}, "mlp": None},
    ],
}


# 16-bit bound for whole models of this design, in standard deviations of a row's logits.  The design answers to
# rounding more strongly than the others (norms on the sublayers' results rescale every small result to full size,
# routing weights multiply whole rows, the recurrences carry every rounding along): the plain implementation's own
# bfloat16 run differs from its float64 run by up to 0.19 standard deviations on these models, and the engine from
# the plain bfloat16 run by up to 0.10.  A lost key, page, state row or expert moves a row by about one.
C_MODEL = {"bfloat16": 0.25, "float16": 0.04}


def rounding_of(dtype):
    return None if dtype == "float32" else TD[dtype]


def close(x, ref, dtype, what):
    """Rows of logits against the plain ones.  `ref` may be (logits, sure): in 16 bits a token whose router nearly
    ties in the plain run may take another expert in the engine (the rows before it differ by rounding already),
    which is no fault; such rows are left out, and they must be few."""
    sure = None
    if isinstance(ref, tuple):
        ref, sure = ref
    if dtype == "float32":
        assert_close_f32(x, ref, what)
        return
    if sure is None:
        assert_close_16bit(x, ref, what, dtype, c=C_MODEL[dtype])
        return
    sure = sure[:len(ref)]
    assert sure.mean() > 0.8, f"{what}: {int((~sure).sum())} of {len(sure)} tokens route by a close call"
    assert_close_16bit(np.asarray(x)[sure], np.asarray(ref)[sure], what, dtype, c=C_MODEL[dtype])


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {name: write_model(cfg, str(tmp_path_factory.mktemp("pererax_" + name)), seed) for name, (cfg, seed) in PERERAX.items()}
    out["W"] = write_model(PERERAX_W, str(tmp_path_factory.mktemp("pererax_W")), 6)
    return out


CONFIGS = dict({k: v[0] for k, v in PERERAX.items()}, W=PERERAX_W)
CLOSE_CALL = 0.01       # (spreads of a router's choice scores)
CLEAR_CALL = 0.04
_TOKENS = {}


def plain(folder, dtype, tokens):
    """Logits; for a 16-bit type (logits, which tokens route by a clear margin in every routed layer)."""
    cfg, w = P.load(folder)
    margins = []
    logits = P.forward(cfg, w, tokens, rounding_of(dtype), None, margins).numpy()
    if dtype == "float32":
        return logits
    sure = np.ones(len(tokens), dtype=bool)
    for m in margins:
        sure &= m.numpy() > CLOSE_CALL
    return logits, sure


def session(folder, dtype, max_tokens, **kw):
    from ferrum_b200.engine.trace import TraceSession
    return TraceSession(folder, dtype, max_tokens, **kw)


def tokens_for(name, n, seed, folders=None):
    """n random tokens.  Given the models' folders, tokens at which no router of the model decides by a close
    call (in the plain run that rounds to bfloat16): a token that would is drawn again, front to back, since a
    16-bit engine may send it to another expert, and every later token would differ too."""
    rng = np.random.default_rng(seed)
    vocab = CONFIGS[name]["vocab"]
    toks = rng.integers(0, vocab, n).tolist()
    if folders is None:
        return toks
    if (name, n, seed) not in _TOKENS:
        cfg, w = P.load(folders[name])
        for _ in range(20 * n):
            margins = []
            P.forward(cfg, w, toks, torch.bfloat16, None, margins)
            if not margins:
                break
            unsure = (torch.stack(margins).min(0).values < CLEAR_CALL).nonzero().flatten()
            if len(unsure) == 0:
                break
            toks[int(unsure[0])] = int(rng.integers(0, vocab))
        else:
            raise AssertionError("no tokens with clear routing found")
        _TOKENS[(name, n, seed)] = toks
    return list(_TOKENS[(name, n, seed)])


def make_ctx(entries, slots=None, max_tokens=1024, max_requests=8, widths=()):
    """A step context for [(pos0, n tokens)] entries, with explicit block tables per group."""
    from ferrum_b200.engine.batch import StepContext, StepEntry
    ctx = StepContext("cuda", max_tokens, max_requests, [len(t[0]) for t in widths])
    es = [StepEntry(slots[i] if slots else i, p0, list(range(n))) for i, (p0, n) in enumerate(entries)]
    ctx.fill(es, [list(t) for t in widths])
    return ctx


class SomeMixers:
    """The least a cache needs of a model: a schedule and the needs of its runs."""

    def __init__(self, mixers):
        from ferrum_b200.models import Run
        self.mixers, self.schedule = mixers, [Run(i) for i in range(len(mixers))]

    def cache_needs(self):
        return [m.cache_need() for m in self.mixers]


def short_name(name):
    """A part's parameter name as the plain implementation calls the tensor."""
    name = name.replace("output.weight", "o").replace(".bias", ".b").replace("left_out", "left.out").replace("right_out", "right.out")
    return name[:-7] if name.endswith(".weight") else name


def fill_part(part, seed, td, prefix, std=0.3, fixed=None):
    """Random parameters for a part and its children; returns them under the plain implementation's names (float64)."""
    from ferrum_b200.weights.random_init import _tensor
    w = {}
    for name, ps, owner, local in part.named_specs():
        t = _tensor(f"{prefix}{name}", ps, seed, "cuda", std if ps.kind == "matrix" else 0.2)
        if fixed and name in fixed:
            t = fixed[name].to("cuda")
        t = t.to(td) if ps.kind == "matrix" else t.float()
        owner.assign(local, t.contiguous())
        w[prefix + short_name(name)] = t.double().cpu()
    part.finalize()
    return w


# ================================================================= the attention kernel alone
def attention_reference(q, k, v, pos, H, G, scale, size, cap, sink):
    """q [n, H, D] of queries at `pos`; k, v [keys, G, D]: float64 softmax over the visible keys (and the sink)."""
    out = np.zeros((len(pos), H, v.shape[2]))
    for t, p in enumerate(pos):
        lo = max(0, p - size + 1) if size else 0
        for h in range(H):
            g = h // (H // G)
            s = k[lo:p + 1, g] @ q[t, h] * scale
            if cap:
                s = cap * np.tanh(s / cap)
            top = max(s.max(), 0.0) if sink else s.max()
            w = np.exp(s - top)
            out[t, h] = (w / (w.sum() + (math.exp(-top) if sink else 0.0))) @ v[lo:p + 1, g]
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,page,size,cap,sink", [(3, 1, 14, 8, 19, 0.0, False), (8, 2, 64, 16, 0, 25.0, True), (6, 3, 64, 16, 44, 0.0, False),
                                                      (6, 2, 80, 16, 130, 4.0, True), (5, 5, 40, 32, 257, 0.0, True), (2, 1, 200, 8, 0, 2.5, False),
                                                      (1, 1, 32, 16, 1, 0.0, True)])
def test_attention_kernel_with_sink_cap_and_window_edges(cuda, dtype, H, G, D, page, size, cap, sink):
    """The CUDA-core attention kernel on keys and values written straight into pages that lie scattered in the
    pool.  One key is made to dominate: it is scaled up and every query points at it.  With a window it sits at
    the first row of a page, at the last position a query may see: its value is the output there and one query
    later it is gone.  Without a window it sits far back among hundreds.  A prompt portion, a single token over the
    whole range, a single token whose key range is cut among CTAs, and the sequence's first tokens; with a soft cap
    on the scores the dominant key's lead shrinks to the cap, and with a sink every row loses exp(0) worth of weight
    (a zero query gives the sink exactly one share beside the visible keys': half of everything in a window of one)."""
    from ferrum_b200.ops import lib as ops
    rng = np.random.default_rng(H * 1000 + D)
    n_keys, td = 700, TD[dtype]
    n_pages = -(-n_keys // page)
    order = rng.permutation(n_pages + 5)[:n_pages]
    k = rng.standard_normal((n_keys, G, D)) * 0.3
    v = rng.standard_normal((n_keys, G, D))
    hot = 37 if size == 0 else (n_keys - 1 - (size - 1) - 3) // page * page
    k[hot] *= 5.0
    kt, vt = torch.tensor(k, device="cuda").to(td), torch.tensor(v, device="cuda").to(td)
    k, v = kt.double().cpu().numpy(), vt.double().cpu().numpy()
    plane = torch.zeros(n_pages + 5, 2, G, page, D, device="cuda", dtype=td)
    for lp in range(n_pages):
        n = min(page, n_keys - lp * page)
        plane[order[lp], 0, :, :n] = kt[lp * page:lp * page + n].transpose(0, 1)
        plane[order[lp], 1, :, :n] = vt[lp * page:lp * page + n].transpose(0, 1)
    scale = 0.5
    edge = hot + max(size, 1) - 2       # three queries around the edge
    for pos0, n in ((n_keys - 40, 40), (n_keys - 1, 1), (max(edge, 0), 3), (0, 9)):
        ctx = make_ctx([(pos0, n)], widths=[[list(order)]])
        pos = list(range(pos0, pos0 + n))
        q = np.tile(k[hot].repeat(H // G, axis=0).reshape(1, H * D) * 4.0, (n, 1)) + rng.standard_normal((n, H * D)) * 0.1
        if sink and n > 1:
            q[0] = 0.0                  # every key scores 0, like the sink: each of the visible keys weighs 1 / (their number + 1)
        qt = torch.tensor(q, device="cuda").to(td)
        ref = attention_reference(qt.double().cpu().numpy().reshape(n, H, D), k, v, pos, H, G, scale, size, cap, sink)
        for mode in (["rows", "tokens", "split"] if n == 1 else ["rows", "tokens"]):
            out = torch.full((n, H * D), float("nan"), device="cuda")
            part, slots, q_start = None, 0, None
            if mode == "split":
                split = ops.attention_generic_split()
                slots = (min(n_keys, size + split) if size else n_keys) // split + 2
                part = torch.full((n * H * slots * (D + 2),), float("nan"), device="cuda")
            if mode == "tokens":
                q_start = ctx.q_start
            ops.attention_generic(qt, out, n, ctx.positions, ctx.req_of_token, ctx.block_tables[0], plane, plane.stride(0), page,
                                  H, G, D, scale, size, ctx.err, part=part, split_slots=slots, q_start=q_start, n_reqs=1,
                                  softcap=cap, sink=sink)
            got = out.double().cpu().numpy().reshape(n, H, D)
            assert np.abs(got - ref).max() < (2e-5 if dtype == "float32" else 2e-2) * max(np.abs(ref).max(), 0.05), (pos0, n, mode)
            assert ctx.err.item() == 0
            if size > 1 and pos0 == edge and not cap:
                big = np.abs(v[hot]).max()           # queries at the last two positions that see `hot`, and the first that does not
                assert np.abs(got[1, 0] - v[hot, 0]).max() < 0.05 * big
                assert np.abs(got[2, 0] - v[hot, 0]).max() > 0.3 * np.abs(v[hot, 0]).max()
            if sink and n > 1:
                lo = max(0, pos0 - size + 1) if size else 0
                share = v[lo:pos0 + 1, 0].sum(axis=0) / (pos0 + 1 - lo + 1)
                assert np.abs(got[0, 0] - share).max() < (1e-5 if dtype == "float32" else 1e-2) * max(np.abs(share).max(), 0.05)
        if size == 0 and pos0 > 0 and not cap:
            assert np.abs(got[-1, H - 1] - v[hot, (H - 1) // (H // G)]).max() < 0.1 * np.abs(v[hot]).max()    # the far key among hundreds


# ================================================================= mixers alone, whole and in portions
def run_mixers_in_portions(mixers, xs, cuts, td, max_tokens=128, page=8):
    """The mixers one after another on rows of their own in every step (as the layers of a model run)."""
    from ferrum_b200.cache import CacheStorage
    from ferrum_b200.engine.batch import StepContext, StepEntry
    cache = CacheStorage(SomeMixers(mixers), td, "cuda", page_size=page, max_tokens=max_tokens, max_requests=3, max_model_len=max_tokens)
    ctx = StepContext("cuda", max_tokens, 3, [cache.table_width] * cache.n_groups)
    cache.open()                              # the request under test takes the second slot
    slot = cache.open()
    for s in cache.states:
        s[slot].fill_(float("nan"))           # a state row that a first token must not read
    got, at = [[] for _ in mixers], 0
    for n in cuts:
        cache.manager.grow(slot, at + n)
        if at == 0:
            for s in cache.states:
                s[slot].zero_()               # (what the step function does for a request's first tokens)
        ctx.fill([StepEntry(slot, at, list(range(n)))], cache.manager if cache.n_groups else [])
        for i, (mx, x) in enumerate(zip(mixers, xs)):
            y = torch.zeros(n, x.shape[1], device="cuda")
            mx.forward(x[at:at + n].contiguous(), ctx, cache.layer_cache(i), y, accumulate=False)
            got[i].append(y.double().cpu())
        assert ctx.err.item() == 0
        cache.manager.commit(slot, at + n)
        at += n
    return [torch.cat(g) for g in got]


CUTS = ([61], [20, 1, 1, 2, 30, 7], [2] * 30 + [1])


def check_mixers(mixers, refs, xs, td, dtype, page=8):
    for cuts in CUTS:
        got = run_mixers_in_portions(mixers, xs, cuts, td, page=page)
        for i, ref in enumerate(refs):
            assert torch.isfinite(got[i]).all(), (cuts, i)
            assert (got[i] - ref).abs().max() < (2e-4 if dtype == "float32" else 4e-2) * ref.abs().max(), (cuts, i)


def inputs(n, E, td, seed=10, count=1):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return [torch.randn(61, E, device="cuda", generator=g).to(td) for _ in range(count)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv,size,R,cap", [(3, 1, 10, 14, 0, 6, 3.0), (8, 2, 64, 64, 0, 32, 25.0), (6, 3, 64, 64, 44, 64, 0.0), (4, 2, 12, 12, 17, 8, 0.0),
                                                 (2, 2, 6, 6, 1, 0, 0.0), (6, 2, 80, 40, 24, 20, 5.0)])
def test_both_attention_mixers_alone(cuda, dtype, H, G, D, Dv, size, R, cap):
    """Attention with the norm over the whole query and key projections and a rotation of part of each head: with
    a window and the keys as values (when D = Dv), and causal with a soft cap and a sink; whole, in portions that
    cut windows and pages anywhere, and token pairs."""
    from ferrum_b200.parts import RotaryEmbedding, ShapedAttention
    td, E, eps = TD[dtype], 40, 1e-5
    rot = RotaryEmbedding(D, R, 300.0, None, "half", 128, "cuda") if R else None
    keyed = D == Dv and size > 0
    mixer = ShapedAttention(E, H, G, D, Dv, td, 0.45, eps=eps, window=size, rotary=rot, qk_norm="whole", value_from_key=keyed,
                            score_softcap=cap, sink=not keyed)
    assert ("v.weight" in mixer.param_specs()) == (not keyed)
    w = fill_part(mixer, 9, td, "p.")
    x = inputs(61, E, td)
    c = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "scale": 0.45, "softcap": cap, "sink": not keyed, "value_is_key": keyed}
    if size:
        c["mask"] = {"size": size}
    if R:
        c["rot"] = {"base": 300.0, "dims": R}
    ref = P.attention(x[0].double().cpu(), w, "p.", c, eps, rounding_of(dtype))
    check_mixers([mixer], [ref], x, td, dtype)
    if not keyed:
        plain_softmax = P.attention(x[0].double().cpu(), w, "p.", dict(c, sink=False), eps, rounding_of(dtype))
        assert (plain_softmax - ref).abs().max() > 1e-2 * ref.abs().max()            # (the sink matters to the result)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,Dv,cap", [(3, 6, 10, 7.0), (3, 40, 56, 10.0), (2, 64, 40, 14.0), (1, 5, 33, 4.0), (2, 130, 70, 3.0), (1, 200, 8, 9.0)])
def test_matrix_memory_mixer_alone(cuda, dtype, H, D, Dv, cap):
    """The matrix-memory recurrence: whole, in portions and token pairs (state rows carried between steps, a
    running maximum that starts at zero), at key sizes that take each of the walk's register layouts."""
    from ferrum_b200.parts import MatrixMemoryMixer
    td, E, eps = TD[dtype], 40, 1e-5
    mixer = MatrixMemoryMixer(E, H, D, Dv, cap, eps, td)
    # gate biases spread so that the input gate wins the maximum at some tokens and the forget gate at others
    fixed = {"i.bias": torch.linspace(-3.0, 2.0, H), "f.bias": torch.linspace(0.5, 4.0, H)}
    w = fill_part(mixer, 11, td, "p.", std=0.5, fixed=fixed)
    x = inputs(61, E, td, seed=12)
    c = {"heads": H, "dim": D, "vdim": Dv, "gate_cap": cap}
    ref = P.matrix_memory(x[0].double().cpu(), w, "p.", c, eps, rounding_of(dtype))
    check_mixers([mixer], [ref], x, td, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv,taps,ra,rg", [(4, 2, 10, 6, 3, 5, 7), (6, 6, 32, 48, 4, 12, 20), (2, 1, 64, 40, 4, 16, 8), (1, 1, 4, 36, 1, 1, 2),
                                                 (2, 2, 130, 33, 2, 9, 3), (3, 1, 200, 8, 5, 8, 16)])
def test_delta_rule_mixer_alone(cuda, dtype, H, G, D, Dv, taps, ra, rg):
    """The gated delta rule behind its short convolutions: whole, in portions shorter than the taps and token pairs
    (the convolution's last inputs and the memory carried between steps), with fewer query/key heads than value heads."""
    from ferrum_b200.parts import ChannelDeltaMixer
    td, E, eps = TD[dtype], 40, 1e-5
    mixer = ChannelDeltaMixer(E, H, G, D, Dv, taps, eps, td, ra, rg)
    w = fill_part(mixer, 13, td, "p.", std=0.5)
    x = inputs(61, E, td, seed=14)
    c = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "conv": taps}
    ref = P.channel_delta(x[0].double().cpu(), w, "p.", c, eps, rounding_of(dtype))
    check_mixers([mixer], [ref], x, td, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pair_of_mixers_alone(cuda, dtype):
    """The sink attention and the matrix memory side by side, each normed, averaged: one part that keeps pages AND a state."""
    from ferrum_b200.parts import MatrixMemoryMixer, ParallelMixer, RotaryEmbedding, ShapedAttention
    td, E, eps = TD[dtype], 40, 1e-5
    rot = RotaryEmbedding(10, 6, 100.0, None, "half", 128, "cuda")
    left = ShapedAttention(E, 3, 1, 10, 14, td, 0.4, eps=eps, rotary=rot, qk_norm="whole", score_softcap=3.0, sink=True)
    mixer = ParallelMixer(E, left, MatrixMemoryMixer(E, 3, 6, 10, 7.0, eps, td), eps)
    need = mixer.cache_need()
    assert need.paged is not None and need.state is not None
    w = fill_part(mixer, 15, td, "p.")
    x = inputs(61, E, td, seed=16)
    c = {"left": {"heads": 3, "kv_heads": 1, "dim": 10, "vdim": 14, "scale": 0.4, "softcap": 3.0, "rot": {"base": 100.0, "dims": 6}},
         "right": {"heads": 3, "dim": 6, "vdim": 10, "gate_cap": 7.0}}
    ref = P.parallel_mixer(x[0].double().cpu(), w, "p.", c, eps, rounding_of(dtype))
    check_mixers([mixer], [ref], x, td, dtype)


# ================================================================= the feed-forward and the norms alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,F,Fs,n_exp,n_id,top,T", [(52, 20, 28, 5, 2, 3, 37), (128, 64, 96, 6, 3, 3, 300), (40, 24, 0, 1, 1, 1, 9), (64, 32, 16, 16, 0, 4, 70),
                                                     (72, 100, 8, 3, 0, 3, 11), (128, 128, 256, 4, 3, 2, 1000), (256, 80, 160, 6, 1, 3, 2)])
def test_routed_feed_forward_alone(cuda, dtype, E, F, Fs, n_exp, n_id, top, T):
    """Clamped units chosen by softmax scores plus a correction, identity experts, a unit for every token: sizes that
    take each of the product kernels (CUDA cores, a few rows an expert, tensor-core tiles of both kinds)."""
    from ferrum_b200.engine.batch import StepContext, StepEntry
    from ferrum_b200.parts import RoutedFeedForward, SwiGLU
    td = TD[dtype]
    shared = SwiGLU(E, Fs, td, act="swish_clamp", limit=0.7) if Fs else None
    ffn = RoutedFeedForward(E, F, n_exp, top, td, act="swish_clamp", scores="softmax", scale_input=False, correction=True,
                            weight_scale=1.7, identity=n_id, limit=1.2, shared=shared)
    # a correction that lifts the first identity output into every token's choice (and changes no weight)
    drawn = 0.1 * torch.randn(n_exp + n_id - 1, generator=torch.Generator().manual_seed(23))
    fixed = {"correction": torch.cat([drawn, torch.tensor([5.0])])} if n_id else None
    w = fill_part(ffn, 21, td, "f.", std=0.4, fixed=fixed)
    g = torch.Generator(device="cuda").manual_seed(22)
    x = torch.randn(T, E, device="cuda", generator=g).to(td)
    mlp = {"expert": {"ff": F, "limit": 1.2}, "router": {"experts": n_exp, "identity": n_id, "top": top, "scale": 1.7}}
    if Fs:
        mlp["shared"] = {"ff": Fs, "limit": 0.7}
    margins = []
    ref = P.mixture(x.double().cpu(), w, "f.", mlp, rounding_of(dtype), margins)
    ctx = StepContext("cuda", 1024, 4, [])
    ctx.fill([StepEntry(0, 0, list(range(T)))], [])
    y = torch.full((T, E), float("nan"), device="cuda")
    ffn.forward(x, ctx, y, accumulate=False)
    assert ctx.err.item() == 0
    sure = (margins[0] > (1e-6 if dtype == "float32" else CLEAR_CALL)).numpy()
    assert sure.any() and sure.mean() >= min(0.5, 1.0 - 1.0 / T)
    got = y.double().cpu()
    assert (got - ref)[sure].abs().max() < (2e-4 if dtype == "float32" else 4e-2) * ref.abs().max()
    if n_id:            # the lifted identity output is in every token's choice: the result holds the token's own row
        idx, wt, _ = P.route(x.double().cpu(), w, "f.", mlp["router"], rounding_of(dtype))
        assert (idx == n_exp + n_id - 1).any(dim=1).all()


def test_router_correction_changes_the_choice_and_not_the_weights(cuda):
    from ferrum_b200.ops import lib as ops
    logits = torch.tensor([[math.log(2.0), 0.0, -math.log(2.0)], [0.0, 0.0, 0.0]], device="cuda")
    corr = torch.tensor([0.0, 0.0, 10.0], device="cuda")
    x = torch.ones(2, 8, device="cuda")
    expert_of, rank_of, row_of = (torch.full((4,), -7, dtype=torch.int32, device="cuda") for _ in range(3))
    weight_of, counts, xg = torch.zeros(4, device="cuda"), torch.zeros(2, dtype=torch.int32, device="cuda"), torch.zeros(4, 8, device="cuda")
    ops.moe_route(logits, 2, 3, 2, x, False, expert_of, rank_of, weight_of, counts, xg, row_of, scores="softmax", correction=corr,
                  weight_scale=7.0, n_identity=1)
    assert expert_of.tolist() == [2, 0, 2, 0]                    # the corrected identity output first, then the best score; a tie: the lower index
    assert weight_of.tolist() == pytest.approx([7.0 * 0.5 / 3.5, 7.0 * 2.0 / 3.5, 7.0 / 3.0, 7.0 / 3.0], rel=1e-5)
    assert counts.tolist() == [2, 0] and row_of[0].item() == -1 and row_of[2].item() == -1 and sorted([row_of[1].item(), row_of[3].item()]) == [0, 1]


@pytest.mark.parametrize("E,T", [(52, 9), (256, 33), (1030, 3)])
def test_norms_on_results_alone(cuda, E, T):
    from ferrum_b200.ops import lib as ops
    g = torch.Generator(device="cuda").manual_seed(E)
    h, y, a = (torch.randn(T, E, device="cuda", generator=g) for _ in range(3))
    w, ls, wa = (1.0 + 0.3 * torch.randn(E, device="cuda", generator=g) for _ in range(3))
    eps = 1e-5
    want = h.double() + ls.double() * (P.rms(y.double(), eps) * w.double())
    xc = torch.zeros(T, E, device="cuda", dtype=torch.bfloat16)
    h1 = h.clone()
    ops.post_norm_add(h1, T, y, w, ls, eps, xc=xc)
    assert (h1.double() - want).abs().max() < 1e-5 and torch.equal(xc, h1.to(torch.bfloat16))
    h2 = h.clone()
    ops.post_norm_add(h2, T, y, w, None, eps)
    assert (h2.double() - (h.double() + P.rms(y.double(), eps) * w.double())).abs().max() < 1e-5
    xc.zero_()
    ops.post_norm_add(h, T, xc=xc)
    assert torch.equal(xc, h.to(torch.bfloat16))
    out = torch.zeros(T, E, device="cuda")
    ops.dual_norm_mean(y, a, w, wa, eps, out, T)
    assert (out.double() - 0.5 * (P.rms(y.double(), eps) * w.double() + P.rms(a.double(), eps) * wa.double())).abs().max() < 1e-5
    H, Dv = 2, E // 2
    for per_head in (False, True):
        wn = 1.0 + 0.3 * torch.randn(H * Dv if per_head else Dv, device="cuda", generator=g)
        o16 = torch.zeros(T, H * Dv, device="cuda")
        ops.head_gate_norm(y[:, :H * Dv], a[:, :H * Dv], wn, eps, T, H, Dv, o16)
        ref = P.rms(y[:, :H * Dv].double().view(T, H, Dv), eps) * wn.double().view(H if per_head else 1, Dv) * torch.sigmoid(a[:, :H * Dv].double().view(T, H, Dv))
        assert (o16.double().view(T, H, Dv) - ref).abs().max() < 1e-5


# ================================================================= whole models, every way of cutting the work
CASES = [(n, d) for n in ("A", "B") for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES + [("C", "float32"), ("C", "bfloat16")])
def test_whole_prompt_and_first_tokens(cuda, folders, name, dtype):
    toks = tokens_for(name, 140, 10, folders)
    r = Replay(session(folders[name], dtype, 160))
    r.step([("a", toks, "all")], end=["a"])
    close(r.logits("a", len(toks)), plain(folders[name], dtype, toks), dtype, f"{name} whole")
    r = Replay(session(folders[name], dtype, 64))
    r.step([("b", toks[:1], "all")])
    r.step([("b", toks[1:3], "all")])
    r.step([("b", toks[3:4], "all")], end=["b"])
    close(r.logits("b", 4), plain(folders[name], dtype, toks[:4]), dtype, f"{name} first tokens")


@pytest.mark.parametrize("name", ["A", "C"])
def test_residual_rows_after_every_layer(cuda, folders, name):
    toks = tokens_for(name, 25, 11, folders)
    cfg, w = P.load(folders[name])
    taps = []
    P.forward(cfg, w, toks, None, taps)
    s = session(folders[name], "float32", 64)
    got = []
    s.model.on_run = lambda k, h: got.append(h[:len(toks)].double().cpu())
    s.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": ["a"]})
    assert len(got) == len(taps) == len(cfg["layers"])
    for k, (g, t) in enumerate(zip(got, taps)):
        assert (g - t).abs().max() < 1e-4 * t.abs().max(), k


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_then_long_decoding_past_every_window(cuda, folders, name, dtype):
    """30 tokens at once, then 120 one by one: windows pass over decoded tokens, pages behind them are given back
    meanwhile, the recurrent states are carried through a captured graph."""
    toks = tokens_for(name, 150, 12, folders)
    ref = plain(folders[name], dtype, toks)
    s = session(folders[name], dtype, 160, page_size=8)
    r = Replay(s)
    r.step([("a", toks[:30], "all")])
    for t in toks[30:]:
        r.step([("a", [t], "all")])
    close(r.logits("a", len(toks)), ref, dtype, f"{name} prefill+decode")
    assert s.runner.graph_replays > 0          # single tokens ran from a captured graph


def test_token_by_token_from_the_first(cuda, folders):
    toks = tokens_for("A", 70, 17, folders)
    ref = plain(folders["A"], "float32", toks)
    r = Replay(session(folders["A"], "float32", 80, page_size=8))
    for t in toks:
        r.step([("a", [t], "all")])
    close(r.logits("a", len(toks)), ref, "float32", "A token by token")


@pytest.mark.parametrize("name,dtype", CASES + [("C", "float32")])
@pytest.mark.parametrize("sizes", [[2], [5, 2, 7, 3, 2, 16, 17, 2, 31, 1, 33, 2], [64, 3, 1]])
def test_portions(cuda, folders, name, dtype, sizes):
    toks = tokens_for(name, 131, 13, folders)
    ref = plain(folders[name], dtype, toks)
    r = Replay(session(folders[name], dtype, 144, page_size=16))
    i = k = 0
    while i < len(toks):
        n = min(sizes[k % len(sizes)], len(toks) - i)
        r.step([("a", toks[i:i + n], "all")])
        i += n
        k += 1
    close(r.logits("a", len(toks)), ref, dtype, f"{name} portions {sizes[:3]}")


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("page_size", [8, 32])
def test_mixed_batches_reuse_pages_and_slots(cuda, folders, name, dtype, page_size):
    """Six requests through four slots, portions beside single tokens; the pool has fewer pages than all requests need
    together: finished requests' pages and state rows go to later ones (which must start from zero)."""
    lens = {"a": 70, "b": 45, "c": 33, "d": 90, "e": 50, "f": 21}
    toks = {k: tokens_for(name, n, 20 + i, folders) for i, (k, n) in enumerate(lens.items())}
    schedule = mixed_schedule(lens)
    pool = peak_pages(schedule, page_size)
    s = session(folders[name], dtype, pool * page_size, page_size=page_size, max_requests=4)
    slots_seen, owners = {}, {}
    r = Replay(s)
    for entries, ended in schedule:
        r.step([(k, toks[k][first:first + n], "all") for k, first, n in entries], end=ended)
        for k, slot in s.slots.items():
            slots_seen.setdefault(slot, set()).add(k)
        for g in range(s.cache.manager.n_groups):
            for k, slot in s.slots.items():
                for p in s.cache.manager.table(g, slot):
                    if p >= 0:
                        owners.setdefault((g, p), set()).add(k)
        assert s.cache.manager.check() == ""
    assert pages_were_reused(owners) and any(len(v) > 1 for v in slots_seen.values())
    for k in toks:
        close(r.logits(k, lens[k]), plain(folders[name], dtype, toks[k]), dtype, f"{name} mixed {k}")


@pytest.mark.parametrize("name", ["A", "B"])
def test_logits_do_not_depend_on_the_batch(cuda, folders, name):
    """float32: a request's logits beside three others equal those it gets alone to rounding."""
    toks = {k: tokens_for(name, n, 40 + i, folders) for i, (k, n) in enumerate({"a": 50, "b": 9, "c": 31, "d": 2}.items())}
    alone = {}
    for k, t in toks.items():
        r = Replay(session(folders[name], "float32", 64))
        r.step([(k, t, "all")], end=[k])
        alone[k] = r.logits(k, len(t))
    r = Replay(session(folders[name], "float32", 128))
    r.step([(k, t[:len(t) // 2], "all") for k, t in toks.items()])
    r.step([(k, t[len(t) // 2:], "all") for k, t in reversed(list(toks.items()))], end=list(toks))
    for k, t in toks.items():
        assert np.abs(r.logits(k, len(t)) - alone[k]).max() < 2e-5 * max(1.0, np.abs(alone[k]).max()), k


def test_a_far_token_decides_where_something_carries_it(cuda, folders):
    """Two prompts that differ in one token.  Behind windows alone the logits agree again (to rounding) once no path
    is left: the reach of a stack of windows is the sum of (size - 1).  With a recurrence or an unmasked attention in
    the stack the token still matters hundreds of positions later."""
    reach = sum(L["mixer"]["mask"]["size"] - 1 for L in PERERAX_W["layers"])
    for name, n in (("W", reach + 40), ("A", 300)):
        toks = tokens_for(name, n, 31)
        other = list(toks)
        other[5] = (other[5] + 1) % CONFIGS[name]["vocab"]
        out = []
        for t in (toks, other):
            r = Replay(session(folders[name], "float32", 320))
            r.step([("a", t[:50], "all")])
            r.step([("a", t[50:], "all")], end=["a"])
            out.append(r.logits("a", len(t)))
        d = np.abs(out[0] - out[1]).max(axis=1)
        assert d[5] > 1e-3 and d[6] > 1e-4
        if name == "W":
            assert d[5 + reach + 1:].max() < 1e-5
        else:
            assert d[-20:].min() > 1e-4
        close(out[1], plain(folders[name], "float32", other), "float32", f"{name} other")


def plain_generate(cfg, w, prompt, n, rd=None):
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(P.forward(cfg, w, seq, rd)[-1].argmax()))
    return seq[len(prompt):]


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "float32"), ("B", "bfloat16")])
def test_greedy_generation_through_the_engine(cuda, folders, name, dtype):
    """Engine.generate (scheduler, sampler, chunked prompts, several requests) against the plain
    implementation; in bfloat16 a token may differ only at a near-tie of the plain logits."""
    from ferrum_b200.engine.api import Engine
    cfg, w = P.load(folders[name])
    prompts = [tokens_for(name, n, 60 + n, folders) for n in (23, 5, 41)]
    eng = Engine(folders[name], dtype=dtype, page_size=8, num_pages=40, max_batch_tokens=32, max_batch_seqs=4, chunk_size=16,
                 max_model_len=96)
    outs = eng.generate(prompts, max_new_tokens=20)
    compared = 0
    for p, got in zip(prompts, outs):
        if dtype == "float32":
            assert got == plain_generate(cfg, w, p, 20)
            continue
        seq = list(p)
        for t in got:
            margins = []
            logits = P.forward(cfg, w, seq, rounding_of(dtype), None, margins)[-1].numpy()
            if margins and float(torch.stack(margins).min()) < CLEAR_CALL:
                break           # a generated token routes by a close call: from here on the engine may differ rightly
            if t != int(np.argmax(logits)):
                assert logits.max() - logits[t] <= 0.2 * logits.std(), (len(seq), t)
            seq.append(t)
            compared += 1
    assert dtype == "float32" or compared >= 3, compared
    assert eng.stats()["pages_used"] == [0] * eng.cache.manager.n_groups


def test_trace_run_program_and_command_line(cuda, folders, tmp_path):
    """bin/trace_run as a user runs it on a Pererax folder (a subprocess, JSON lines in, .f32 files
    out), and `ferrum generate` on the same folder against the plain implementation."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    toks = tokens_for("A", 40, 16, folders)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[30:], "want": []}, {"id": "y", "tokens": toks[:2], "want": [1]}], "end": ["y"]},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[:1], "want": [0]}], "end": ["x"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["A"], "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert p.stdout.split() == ["done", "0", "done", "1", "done", "2"]
    ref = plain(folders["A"], "float32", toks + toks[:1])
    assert_close_f32(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1), ref[[0, 29]], "trace_run step 0")
    assert_close_f32(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1), ref[[1]], "trace_run step 1")
    assert_close_f32(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, -1), ref[[40]], "trace_run step 2")
    cfg, w = P.load(folders["A"])
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "ferrum"), "generate", "--model", folders["A"], "--dtype", "float32",
                        "--prompt-tokens", ",".join(str(t) for t in toks[:12]), "--max-new-tokens", "6"],
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    want = plain_generate(cfg, w, toks[:12], 6)
    assert ",".join(str(t) for t in want) in p.stdout.replace(" ", ""), (p.stdout, want)


def test_float16_prefill_and_decoding(cuda, folders):
    """The kernels with float16 storage (weights, activations, cached keys and values): a prompt, then
    single tokens, against the plain implementation rounding to float16 where the engine does."""
    toks = tokens_for("B", 150, 14, folders)
    ref, sure = plain(folders["B"], "float16", toks)
    r = Replay(session(folders["B"], "float16", 192))
    r.step([("a", toks[:100], "all")])
    for t in toks[100:]:
        r.step([("a", [t], "all")])
    assert_close_16bit(r.logits("a", len(toks))[sure], ref[sure], "B float16", "float16", c=C_MODEL["float16"])
