"""Zavesun on the GPU against the plain implementation (plain_zavesun.py): every mechanism alone,
then whole models under every way of cutting the work, then generation through the engine."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_zavesun as P
from helpers import Replay, assert_close_16bit, assert_close_f32, mixed_schedule, pages_were_reused, peak_pages
from zavesun_configs import ZAVESUN, write_model

pytestmark = pytest.mark.gpu
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}
F64 = torch.float64


def rounding_of(dtype):
    return None if dtype == "float32" else TD[dtype]


def close(x, ref, dtype, what):
    """Rows of logits against the plain ones.  `ref` may be (logits, sure): in 16 bits a token whose router nearly
    ties in the plain run may take another expert in the engine (the rows before it differ by rounding already),
    which is no fault; such rows are left out, and they must be few."""
    sure = None
    if isinstance(ref, tuple):
        ref, sure = ref
    if dtype == "float32" or sure is None:
        (assert_close_f32 if dtype == "float32" else assert_close_16bit)(x, ref, what)
        return
    sure = sure[:len(ref)]
    assert sure.mean() > 0.8, f"{what}: {int((~sure).sum())} of {len(sure)} tokens route by a close call"
    assert_close_16bit(np.asarray(x)[sure], np.asarray(ref)[sure], what)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write_model(cfg, str(tmp_path_factory.mktemp("zavesun_" + name)), seed) for name, (cfg, seed) in ZAVESUN.items()}


CLOSE_CALL = 0.01       # (standard deviations of a router's logits)
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
    16-bit engine may send it to another expert, and every later token that looks back at it would differ too."""
    rng = np.random.default_rng(seed)
    vocab = ZAVESUN[name][0]["vocab"]
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


SHORT = {"output.weight": "o", "q.bias": "q.b", "k.bias": "k.b", "v.bias": "v.b", "router.weight": "router"}


def fill_part(part, seed, td, prefix, std=0.3, fixed=None):
    """Random parameters for a part; returns them under the plain implementation's names (float64)."""
    from ferrum_b200.weights.random_init import _tensor
    w = {}
    for name, ps in part.param_specs().items():
        t = _tensor(f"{prefix}{name}", ps, seed, "cuda", std if ps.kind == "matrix" else 0.2)
        if fixed and name in fixed:
            t = fixed[name].to("cuda")
        t = t.to(td) if ps.kind == "matrix" else t.float()
        part.assign(name, t.contiguous())
        w[prefix + SHORT.get(name, name[:-7] if name.endswith(".weight") else name)] = t.double().cpu()
    part.finalize()
    return w


# ================================================================= the attention kernel alone
def first_key(p, size, chunked):
    if size <= 0:
        return 0
    return p // size * size if chunked else max(0, p - size + 1)


def attention_reference(q, k, v, pos, H, G, scale, size, chunked, slopes=None):
    """q [n, H, D] of queries at `pos`; k, v [keys, G, D]: float64 softmax over the visible keys."""
    out = np.zeros((len(pos), H, v.shape[2]))
    for t, p in enumerate(pos):
        lo = first_key(p, size, chunked)
        for h in range(H):
            g = h // (H // G)
            s = k[lo:p + 1, g] @ q[t, h] * scale
            if slopes is not None:
                s = s - slopes[h] * (p - np.arange(lo, p + 1))
            w = np.exp(s - s.max())
            out[t, h] = (w / w.sum()) @ v[lo:p + 1, g]
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,page,size,chunked,sloped", [(3, 1, 14, 8, 19, False, True), (4, 2, 64, 16, 0, False, True), (6, 2, 80, 16, 130, True, False),
                                                            (5, 5, 40, 32, 64, True, False), (8, 2, 128, 16, 90, False, True), (2, 1, 200, 8, 257, True, True),
                                                            (4, 4, 24, 16, 21, True, False), (1, 1, 32, 16, 1, True, False)])
def test_attention_sees_exactly_its_window_or_chunk(cuda, dtype, H, G, D, page, size, chunked, sloped):
    """The CUDA-core attention kernel on keys and values written straight into pages that lie
    scattered in the pool, float32 results out.  One key is made to dominate: it is scaled up and
    every query points at it.  For a window it sits at the last position a query may see: its value
    is the output there and one query later it is gone.  For a chunk it is the LAST key of a chunk:
    the query at its own position sees it and the next query, the first of the next chunk, sees
    only itself.  Without a mask it sits far back among hundreds.  A prompt portion, a single token
    over the whole range, and a single token whose key range is cut among CTAs; the distance bias
    is a straight line with a slope per head."""
    from ferrum_b200.ops import lib as ops
    rng = np.random.default_rng(H * 1000 + D)
    n_keys, td = 700, TD[dtype]
    n_pages = -(-n_keys // page)
    order = rng.permutation(n_pages + 5)[:n_pages]
    k = rng.standard_normal((n_keys, G, D)) * 0.3
    v = rng.standard_normal((n_keys, G, D))
    if size == 0:
        hot = 37
    elif chunked:
        hot = (n_keys - 20) // size * size - 1               # the last key of a chunk
    else:
        hot = (n_keys - 1 - (size - 1) - 3) // page * page
    k[hot] *= 5.0
    kt, vt = torch.tensor(k, device="cuda").to(td), torch.tensor(v, device="cuda").to(td)
    k, v = kt.double().cpu().numpy(), vt.double().cpu().numpy()
    plane = torch.zeros(n_pages + 5, 2, G, page, D, device="cuda", dtype=td)
    for lp in range(n_pages):
        n = min(page, n_keys - lp * page)
        plane[order[lp], 0, :, :n] = kt[lp * page:lp * page + n].transpose(0, 1)
        plane[order[lp], 1, :, :n] = vt[lp * page:lp * page + n].transpose(0, 1)
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device="cuda", dtype=torch.float32) if sloped else None
    scale = 0.5
    edge = hot - 1 if chunked else hot + max(size, 1) - 2       # three queries around the edge
    for pos0, n in ((n_keys - 40, 40), (n_keys - 1, 1), (max(edge, 0), 3), (0, 9)):
        ctx = make_ctx([(pos0, n)], widths=[[list(order)]])
        pos = list(range(pos0, pos0 + n))
        q = np.tile(k[hot].repeat(H // G, axis=0).reshape(1, H * D) * 4.0, (n, 1)) + rng.standard_normal((n, H * D)) * 0.1
        qt = torch.tensor(q, device="cuda").to(td)
        ref = attention_reference(qt.double().cpu().numpy().reshape(n, H, D), k, v, pos, H, G, scale, size, chunked,
                                  slopes.double().cpu().numpy() if sloped else None)
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
                                  distance_penalty=(slopes, None) if sloped else None, chunked=chunked)
            got = out.double().cpu().numpy().reshape(n, H, D)
            assert np.abs(got - ref).max() < (2e-5 if dtype == "float32" else 2e-2) * np.abs(ref).max(), (pos0, n, mode)
            assert ctx.err.item() == 0
            if size > 1 and pos0 == edge:
                big = np.abs(v[hot]).max()
                if chunked:         # queries at hot - 1, hot, hot + 1
                    assert np.abs(got[1, 0] - v[hot, 0]).max() < 0.05 * big
                    assert np.abs(got[2, 0] - v[hot + 1, 0]).max() < 1e-2 * big          # alone in its chunk
                else:               # queries at the last two positions that see `hot`, and the first that does not
                    assert np.abs(got[1, 0] - v[hot, 0]).max() < 0.05 * big
                    assert np.abs(got[2, 0] - v[hot, 0]).max() > 0.3 * np.abs(v[hot, 0]).max()
        if size == 0 and pos0 > 0:
            # the far key among hundreds: with the slopes the last head (the flattest) still finds it
            assert np.abs(got[-1, H - 1] - v[hot, (H - 1) // (H // G)]).max() < 0.1 * np.abs(v[hot]).max()


# ================================================================= shaping of heads
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("Hq,Hkv,Dk,Dv,R,factor,biased,normed,temp", [(3, 1, 10, 14, 6, 2.5, True, True, None), (4, 2, 64, 48, 64, 3.0, True, True, None),
                                                                      (2, 2, 12, 6, 0, 1.0, False, False, (0.7, 4)), (5, 5, 32, 48, 16, 1.0, True, False, (0.25, 1)),
                                                                      (8, 2, 128, 48, 64, 4.0, False, True, (0.75, 16))])
def test_heads_get_bias_norm_turn_temperature_and_mixed_values(cuda, dtype, Hq, Hkv, Dk, Dv, R, factor, biased, normed, temp):
    """qkv_shape against the plain functions, in the design's order: bias, weighted RMS norm of query and
    key heads, interleaved turn of the first R elements, query temperature; the values of a first layer
    are left in float32 and a second call blends its own with them before they are cached."""
    from ferrum_b200.ops import lib as ops
    from ferrum_b200.parts import RotaryEmbedding
    td, eps, page, T = TD[dtype], 1e-3, 8, 21
    Dp = max(Dk, Dv)
    g = torch.Generator(device="cuda").manual_seed(Dk)
    freqs = P.linear_frequencies(100.0, R, factor) if R else []
    rot = RotaryEmbedding(Dk, R, 100.0, None, "adjacent", 64, "cuda", frequencies=freqs) if R else None
    order = [[5, 2, 7, 0, 9, 1], [3, 8, 4, 6, -1, -1]]
    ctx = make_ctx([(30, 12), (0, 9)], widths=[order])
    width = Hq * Dk + Hkv * (Dk + Dv)
    proj = torch.randn(T, width + 3, device="cuda", generator=g) * 2
    proj2 = torch.randn(T, width + 3, device="cuda", generator=g) * 2
    bias = torch.randn(width, device="cuda", generator=g) if biased else None
    qn = 1 + 0.3 * torch.randn(Dk, device="cuda", generator=g) if normed else None
    kn = 1 + 0.3 * torch.randn(Dk, device="cuda", generator=g) if normed else None
    lam = torch.tensor([0.3], device="cuda")
    first = torch.full((T + 1, Hkv * Dv), 7.0, device="cuda")
    pos = torch.tensor(list(range(30, 42)) + list(range(9)))
    tol = 1e-5 if dtype == "float32" else 1e-2

    def expect(p, v_first):
        pd = p.double().cpu()[:, :width] + (bias.double().cpu() if biased else 0.0)
        qr = pd[:, :Hq * Dk].view(T, Hq, Dk)
        kr = pd[:, Hq * Dk:(Hq + Hkv) * Dk].view(T, Hkv, Dk)
        vr = pd[:, (Hq + Hkv) * Dk:].view(T, Hkv, Dv)
        if normed:
            qr, kr = P.rms(qr, eps) * qn.double().cpu(), P.rms(kr, eps) * kn.double().cpu()
        if R:
            qr, kr = P.rotate_interleaved(qr, pos, freqs, R), P.rotate_interleaved(kr, pos, freqs, R)
        if temp:
            qr = qr * P.query_temperature(pos, temp[0], temp[1])[:, None, None]
        if v_first is not None:
            vr = P.mix_values(vr, v_first, 0.3)
        return qr, kr, vr

    def run(p, mix):
        plane = torch.full((10, 2, Hkv, page, Dp), 7.0, device="cuda", dtype=td)
        q = torch.full((T, Hq * Dp), 7.0, device="cuda", dtype=td)
        ops.qkv_shape(p, T, ctx, ctx.block_tables[0], rot, rot.pairing if rot else 0, None, 0, False, eps, q, plane, plane.stride(0), page,
                      Hq, Hkv, Dk, Dv, Dp, True, bias=bias, q_norm=qn, k_norm=kn, q_temp=temp, value_mix=mix)
        assert ctx.err.item() == 0
        return q.double().cpu().view(T, Hq, Dp), plane

    def compare(got_q, plane, qr, kr, vr):
        assert (got_q[..., :Dk] - qr).abs().max() < tol * max(1.0, qr.abs().max()) and got_q[..., Dk:].abs().sum() == 0
        for t in range(T):
            r, p = (0, int(pos[t])) if t < 12 else (1, int(pos[t]))
            pg = order[r][p // page]
            krow, vrow = plane[pg, 0, :, p % page].double().cpu(), plane[pg, 1, :, p % page].double().cpu()
            assert (krow[:, :Dk] - kr[t]).abs().max() < tol * max(1.0, kr.abs().max()) and krow[:, Dk:].abs().sum() == 0
            assert (vrow[:, :Dv] - vr[t]).abs().max() < tol * max(1.0, vr.abs().max()) and vrow[:, Dv:].abs().sum() == 0

    qr, kr, vr = expect(proj, None)
    compare(*run(proj, ("store", first)), qr, kr, vr)
    assert (first[:T].double().cpu().view(T, Hkv, Dv) - vr).abs().max() < 1e-5 * vr.abs().max()      # float32, whatever the cache's type
    assert torch.equal(first[T], torch.full((Hkv * Dv,), 7.0, device="cuda"))
    qr2, kr2, vr2 = expect(proj2, vr)
    compare(*run(proj2, ("blend", first, lam)), qr2, kr2, vr2)
    compare(*run(proj2, None), *expect(proj2, None))


# ================================================================= several residual streams
@pytest.mark.parametrize("S,E,T", [(1, 40, 5), (3, 52, 9), (4, 328, 33), (8, 1030, 3), (2, 128, 70)])
def test_streams_write_read_and_norm_in_one_kernel(cuda, S, E, T):
    from ferrum_b200.ops import lib as ops
    g = torch.Generator(device="cuda").manual_seed(S * 100 + E)
    X = torch.randn(T + 2, S * E, device="cuda", generator=g)
    y = torch.randn(T, E + 4, device="cuda", generator=g)[:, :E]          # (rows longer than the streams')
    mix, outw, inw = (torch.randn(s, device="cuda", generator=g) for s in ((S, S), (S,), (S,)))
    nw = 1 + 0.2 * torch.randn(E, device="cuda", generator=g)
    eps = 1e-4
    Xd = X[:T].double().cpu().view(T, S, E).transpose(0, 1)               # [S, T, E]
    new = P.streams_write(Xd, mix.double().cpu(), outw.double().cpu(), y.double().cpu())
    u = P.streams_read(new, inw.double().cpu())
    ref = P.rms(u, eps) * nw.double().cpu()
    # write + read, stored
    X1 = X.clone()
    out = torch.zeros(T, E, device="cuda")
    ops.hyper_step(X1, S, E, T, write=ops.StreamWrite(mix, outw, y=y), in_w=inw, norm_w=nw, eps=eps, out=out)
    assert (out.double().cpu() - ref).abs().max() < 2e-5 * ref.abs().max()
    assert (X1[:T].double().cpu().view(T, S, E).transpose(0, 1) - new).abs().max() < 1e-5 * new.abs().max()
    assert torch.equal(X1[T:], X[T:])                                     # rows past the batch stay
    # read only (the first sublayer of a model), 16-bit rows out
    out16 = torch.zeros(T, E, device="cuda", dtype=torch.bfloat16)
    X2 = X.clone()
    ops.hyper_step(X2, S, E, T, in_w=inw, norm_w=nw, eps=eps, out=out16)
    ref0 = P.rms(P.streams_read(Xd, inw.double().cpu()), eps) * nw.double().cpu()
    assert (out16.double().cpu() - ref0).abs().max() < 1e-2 * ref0.abs().max() and torch.equal(X2, X)
    # write only (a flush)
    X3 = X.clone()
    ops.hyper_step(X3, S, E, T, write=ops.StreamWrite(mix, outw, y=y), store=True)
    assert torch.equal(X3, X1)
    # listed rows: the write is applied on the way, nothing is stored, the read is the plain sum
    rows = torch.tensor([T - 1, 0, T // 2], dtype=torch.int32, device="cuda")
    X4 = X.clone()
    outr = torch.zeros(4, E, device="cuda")
    ops.hyper_step(X4, S, E, 3, write=ops.StreamWrite(mix, outw, y=y), rows=rows, store=False, norm_w=nw, eps=eps, out=outr)
    refr = P.rms(new.sum(0), eps)[rows.long().cpu()] * nw.double().cpu()
    assert (outr[:3].double().cpu() - refr).abs().max() < 2e-5 * refr.abs().max() and torch.equal(X4, X)
    # a token's result is `top` rows named by a table, added in order
    top = 3
    rows_y = torch.randn(T * top + 1, E, device="cuda", generator=g)
    table = torch.randperm(T * top, device="cuda", generator=g).to(torch.int32)
    ysum = rows_y[table.long()].view(T, top, E).double().sum(1).cpu()
    new2 = P.streams_write(Xd, mix.double().cpu(), outw.double().cpu(), ysum)
    X5 = X.clone()
    ops.hyper_step(X5, S, E, T, write=ops.StreamWrite(mix, outw, y=rows_y, y_rows=table, top=top), in_w=inw, norm_w=nw, eps=eps, out=out)
    assert (X5[:T].double().cpu().view(T, S, E).transpose(0, 1) - new2).abs().max() < 1e-5 * new2.abs().max()


def test_one_stream_with_ones_is_the_plain_residual_sum(cuda):
    from ferrum_b200.ops import lib as ops
    T, E = 7, 48
    X = torch.randn(T, E, device="cuda")
    y = torch.randn(T, E, device="cuda")
    one = torch.ones(1, device="cuda")
    out = torch.zeros(T, E, device="cuda")
    X1 = X.clone()
    ops.hyper_step(X1, 1, E, T, write=ops.StreamWrite(one.view(1, 1), one, y=y), in_w=one, norm_w=torch.ones(E, device="cuda"), eps=1e-6, out=out)
    assert torch.allclose(X1, X + y, atol=1e-6)
    assert torch.allclose(out.double(), P.rms((X + y).double(), 1e-6), atol=1e-5)


# ================================================================= the routed feed-forward alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,F,n_exp,top,T", [(52, 20, 5, 2, 37), (128, 64, 4, 1, 300), (40, 24, 1, 1, 9), (64, 32, 16, 4, 70), (72, 100, 40, 8, 11),
                                             (328, 104, 8, 1, 2), (200, 88, 3, 2, 700), (264, 168, 6, 1, 150), (256, 136, 2, 2, 500)])
def test_routed_feed_forward_alone(cuda, dtype, E, F, n_exp, top, T):
    """Router, choice, gather, both grouped products and the sum against the plain function; with more
    experts than tokens some experts get no row, with one expert all rows are its.  In bfloat16 the sizes
    that are multiples of 8 take a tensor-core product (few rows an expert: mma.sync tiles of 16 rows; many:
    the tcgen05 kernel with tiles of 128 rows, several per expert, with ragged last tiles, feature counts
    and a K that end inside a tile), the others a CUDA-core one.  The 16-bit kernels are compared with
    each other too."""
    from ferrum_b200.parts import RoutedFeedForward
    td = TD[dtype]
    ff = RoutedFeedForward(E, F, n_exp, top, td)
    w = fill_part(ff, 21, td, "p.")
    x = torch.randn(T, E, device="cuda", generator=torch.Generator(device="cuda").manual_seed(22)).to(td)
    ctx = make_ctx([(0, T)])
    y = torch.full((T + 1, E), 7.0, device="cuda")
    ff.forward(x, ctx, y, accumulate=False)
    assert ctx.err.item() == 0
    mlp = {"router": {"experts": n_exp, "top": top}}
    xd = x.double().cpu()
    ref = P.routed_ff(xd, w, "p.", mlp, rounding_of(dtype))
    # a token whose top-th and next scores nearly tie may choose differently: leave it out (the router's product has
    # the same rounded inputs and float32 sums on both sides, so only the order of its sums differs)
    s = torch.sigmoid(xd @ w["p.router"].T).sort(dim=-1, descending=True).values
    sure = torch.ones(T, dtype=torch.bool) if n_exp == top else (s[:, top - 1] - s[:, top]) > 1e-4
    assert sure.float().mean() > 0.7
    err = (y[:T].double().cpu() - ref)[sure].abs().max()
    assert err < (2e-5 if dtype == "float32" else 3e-2) * ref.abs().max(), err
    assert torch.equal(y[T], torch.full((E,), 7.0, device="cuda"))
    if dtype != "float32":
        # both kernels of the grouped product see the same 16-bit operands and sum in float32: they agree far closer
        # than either does with the plain function (an activation may round the other way now and then)
        from ferrum_b200.ops import lib as ops
        y2, y3 = torch.zeros(T, E, device="cuda"), torch.zeros(T, E, device="cuda")
        ops.set_moe_cuda_cores(True)
        try:
            ff.forward(x, ctx, y2, accumulate=False)
        finally:
            ops.set_moe_cuda_cores(False)
        ops.set_moe_tcgen05(False)
        try:
            ff.forward(x, ctx, y3, accumulate=False)
        finally:
            ops.set_moe_tcgen05(True)
        assert ctx.err.item() == 0
        assert (y2 - y[:T]).abs().max() < 4e-3 * ref.abs().max()
        assert (y3 - y[:T]).abs().max() < 4e-3 * ref.abs().max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,F,T", [(52, 60, 9), (128, 256, 5), (128, 256, 300), (328, 392, 70), (256, 136, 1000)])
def test_dense_feed_forward_with_gelu_alone(cuda, dtype, E, F, T):
    """down(gelu_tanh(gate x) * up x) against the plain function: a few tokens (products left in partials, the
    activation in the kernel that sums them), many tokens of tensor-core sizes (the activation in the product's own
    epilogue, one CTA a tile and two), and sizes or a type the tensor cores do not take."""
    from ferrum_b200.parts import SwiGLU
    td = TD[dtype]
    ff = SwiGLU(E, F, td, act="gelu_tanh")
    w = fill_part(ff, 31, td, "p.")
    x = torch.randn(T, E, device="cuda", generator=torch.Generator(device="cuda").manual_seed(32)).to(td)
    ctx = make_ctx([(0, T)])
    y = torch.full((T + 1, E), 7.0, device="cuda")
    part = ff.forward(x, ctx, y, accumulate=False)
    assert part is None and ctx.err.item() == 0
    ref = P.dense_ff(x.double().cpu(), w, "p.", rounding_of(dtype))
    err = (y[:T].double().cpu() - ref).abs().max()
    assert err < (2e-5 if dtype == "float32" else 2e-2) * ref.abs().max(), err
    assert torch.equal(y[T], torch.full((E,), 7.0, device="cuda"))


def test_router_prefers_the_lower_index_in_a_tie_and_counts_rows(cuda):
    from ferrum_b200.ops import lib as ops
    T, n, top, E = 6, 5, 2, 8
    logits = torch.tensor([[0.0, 1.0, 1.0, -1.0, 1.0]] * T, device="cuda")
    logits[3] = torch.tensor([3.0, -2.0, 0.5, 2.0, 0.0])
    x = torch.arange(T * E, device="cuda", dtype=torch.float32).view(T, E)
    i32 = lambda *s: torch.zeros(*s, dtype=torch.int32, device="cuda")
    expert_of, rank_of, row_of, counts = i32(T * top), i32(T * top), i32(T * top), i32(n)
    weight_of = torch.zeros(T * top, device="cuda")
    xg = torch.zeros(T * top, E, device="cuda")
    ops.moe_route(logits, T, n, top, x, True, expert_of, rank_of, weight_of, counts, xg, row_of)
    e = expert_of.view(T, top).cpu()
    assert e[0].tolist() == [1, 2] and e[3].tolist() == [0, 3]
    assert counts.cpu().tolist() == [1, 5, 5, 1, 0]
    sg = 1 / (1 + math.exp(-1.0))
    assert weight_of.view(T, top)[0].cpu().tolist() == pytest.approx([sg, sg])
    r = row_of.view(T, top).cpu()
    assert sorted(r.flatten().tolist()) == list(range(T * top))         # every pair has a row of its own
    assert r[3, 0].item() == 0 and 1 <= r[0, 0].item() <= 5 and 6 <= r[0, 1].item() <= 10 and r[3, 1].item() == 11
    assert torch.allclose(xg[r[0, 1].item()], x[0] * sg) and torch.allclose(xg[0], x[3] / (1 + math.exp(-3.0)))


# ================================================================= mixers alone, whole and in portions
def run_mixers_in_portions(mixers, xs, cuts, td, max_tokens=128, page=8):
    """The mixers one after another on rows of their own in every step (as the layers of a model run);
    they share the step's buffers, so a layer that blends values finds the first layer's."""
    from ferrum_b200.cache import CacheStorage
    from ferrum_b200.engine.batch import StepContext, StepEntry
    cache = CacheStorage(SomeMixers(mixers), td, "cuda", page_size=page, max_tokens=max_tokens, max_requests=3, max_model_len=max_tokens)
    ctx = StepContext("cuda", max_tokens, 3, [cache.table_width] * cache.n_groups)
    cache.open()                              # the request under test takes the second slot
    slot = cache.open()
    got, at = [[] for _ in mixers], 0
    for n in cuts:
        cache.manager.grow(slot, at + n)
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,Dk,Dv,size", [(3, 1, 10, 14, 17), (6, 2, 80, 40, 24), (4, 2, 64, 32, 16), (2, 2, 12, 6, 5), (4, 1, 8, 24, 1)])
def test_both_mixers_alone_with_mixed_values(cuda, dtype, H, G, Dk, Dv, size):
    """A windowed mixer that leaves its values, then a chunked one and another windowed one that blend
    theirs with them: whole, in portions that cut windows, chunks and pages anywhere, and token pairs."""
    from ferrum_b200.parts import RotaryEmbedding, ShapedAttention
    td, E, eps = TD[dtype], 40, 1e-5
    R = Dk // 4 * 2
    slopes = [2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]
    rot = RotaryEmbedding(Dk, R, 1000.0, None, "adjacent", 128, "cuda", frequencies=P.linear_frequencies(1000.0, R, 4.0))
    m1 = ShapedAttention(E, H, G, Dk, Dv, td, 0.3, eps=eps, window=size, query_temperature=(0.6, 7), linear_bias=slopes, value_mix="first")
    m2 = ShapedAttention(E, H, G, Dk, Dv, td, 0.9, eps=eps, window=size, mask="chunk", rotary=rot, qkv_bias=True, qk_norm=True, value_mix="blend")
    m3 = ShapedAttention(E, 2 * G, G, Dk, Dv, td, 0.5, eps=eps, window=size + 3, query_temperature=(0.2, 16),
                         linear_bias=[2.0 ** (-8.0 * (h + 1) / (2 * G)) for h in range(2 * G)], value_mix="blend")
    c1 = {"heads": H, "kv_heads": G, "dim": Dk, "vdim": Dv, "scale": 0.3, "mask": {"size": size}, "q_temp": {"coef": 0.6, "every": 7}, "v_mix": True}
    c2 = {"heads": H, "kv_heads": G, "dim": Dk, "vdim": Dv, "scale": 0.9, "mask": {"size": size}, "v_mix": True,
          "rot": {"base": 1000.0, "dims": R, "scaling": {"factor": 4.0}}}
    c3 = {"heads": 2 * G, "kv_heads": G, "dim": Dk, "vdim": Dv, "scale": 0.5, "mask": {"size": size + 3}, "q_temp": {"coef": 0.2, "every": 16}, "v_mix": True}
    w = {}
    for i, mx in enumerate((m1, m2, m3)):
        w.update(fill_part(mx, 9 + i, td, f"p{i}."))
    g = torch.Generator(device="cuda").manual_seed(10)
    xs = [torch.randn(61, E, device="cuda", generator=g).to(td) for _ in range(3)]
    rd = rounding_of(dtype)
    carry = {}
    refs = [P.attention_windowed(xs[0].double().cpu(), w, "p0.", c1, carry, True, rd),
            P.attention_chunked(xs[1].double().cpu(), w, "p1.", c2, eps, carry, False, rd),
            P.attention_windowed(xs[2].double().cpu(), w, "p2.", c3, carry, False, rd)]
    lone = P.attention_chunked(xs[1].double().cpu(), w, "p1.", {**c2, "v_mix": False}, eps, {}, False, rd)
    assert (lone - refs[1]).abs().max() > 1e-3 * refs[1].abs().max()          # (the blend matters to the result)
    for cuts in CUTS:
        got = run_mixers_in_portions([m1, m2, m3], xs, cuts, td)
        for i in range(3):
            assert (got[i] - refs[i]).abs().max() < (2e-4 if dtype == "float32" else 4e-2) * refs[i].abs().max(), (cuts, i)


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
def test_sum_of_streams_after_every_layer(cuda, folders, name):
    toks = tokens_for(name, 25, 11, folders)
    cfg, w = P.load(folders[name])
    taps = []
    P.forward(cfg, w, toks, None, taps)
    s = session(folders[name], "float32", 64)
    S, E = cfg.get("streams", 1), cfg["width"]
    got = []
    s.model.on_run = lambda k, h: got.append(h[:len(toks)].double().cpu().view(len(toks), S, E).sum(1))
    s.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": ["a"]})
    assert len(got) == len(taps) == len(cfg["layers"])
    for k, (g, t) in enumerate(zip(got, taps)):
        assert (g - t).abs().max() < 1e-4 * t.abs().max(), k


@pytest.mark.parametrize("name,dtype", CASES)
def test_prefill_then_long_decoding_past_every_window_and_chunk(cuda, folders, name, dtype):
    """30 tokens at once, then 120 one by one: windows and chunk borders pass over decoded tokens,
    pages behind them are given back meanwhile, the query temperature steps several times."""
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
    """Six requests through four slots, portions beside single tokens; the pool has fewer pages than
    all requests need together: finished requests' pages go to later ones."""
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


def test_a_far_token_decides_inside_the_window_and_not_outside(cuda, folders):
    """Two prompts that differ in one token: the logits differ while the token lies inside some layer's reach
    and the stack of windows and chunks can carry it, and agree again (to rounding) once no path is left.
    With windows w_i and chunks the reach of a stack is at most the sum of (size - 1)."""
    cfg = ZAVESUN["A"][0]
    reach = sum(L["mixer"]["mask"]["size"] - 1 for L in cfg["layers"])
    toks = tokens_for("A", reach + 40, 31)
    other = list(toks)
    other[5] = (other[5] + 1) % cfg["vocab"]
    out = []
    for t in (toks, other):
        r = Replay(session(folders["A"], "float32", 192))
        r.step([("a", t[:50], "all")])
        r.step([("a", t[50:], "all")], end=["a"])
        out.append(r.logits("a", len(t)))
    d = np.abs(out[0] - out[1]).max(axis=1)
    assert d[5] > 1e-3 and d[6] > 1e-4
    assert d[5 + reach + 1:].max() < 1e-5
    ref = plain(folders["A"], "float32", other)
    close(out[1], ref, "float32", "A other")


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
    """bin/trace_run as a user runs it on a Zavesun folder (a subprocess, JSON lines in, .f32 files
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
    assert_close_16bit(r.logits("a", len(toks))[sure], ref[sure], "B float16", "float16")
