"""Zavesun without a GPU: configuration, tensor names, cache layout, and hand-worked anchors of the
plain implementation's functions."""
import copy
import math

import pytest
import torch

import plain_zavesun as P
from zavesun_configs import ZAVESUN_A, ZAVESUN_B, ZAVESUN_C, write_model

from ferrum_b200.config import registry
from ferrum_b200.config.zavesun import DenseMlpSpec, RoutedMlpSpec, ZavesunConfig
from ferrum_b200.errors import ConfigError, WeightsError

F64 = torch.float64


def test_config_reads_every_size_and_constant():
    c = ZavesunConfig.from_dict(ZAVESUN_A)
    assert (c.n_vocab, c.n_embd, c.norm_eps, c.streams, c.logit_softcap) == (197, 52, 1e-5, 3, 9.0)
    a, b, a2, b2 = (l.mixer for l in c.layers)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.mask, a.q_temp) == (3, 1, 10, 14, 0.3, 19, "window", (0.7, 8))
    assert a.linear_bias and not a.qkv_bias and not a.qk_norm and a.rot_dims == 0 and not a.v_mix
    assert (b.window, b.mask, b.rot_base, b.rot_dims, b.rot_scaling.rope_type, b.rot_scaling.factor) == (21, "chunk", 100.0, 8, "linear", 2.5)
    assert b.qkv_bias and b.qk_norm and not b.linear_bias and b.q_temp is None and b.v_mix
    assert b2.rot_scaling is None and a2.v_mix and a2.q_temp == (0.3, 5)
    assert c.first_value_mix() == 1
    m0, m1, m2, m3 = (l.mlp for l in c.layers)
    assert isinstance(m0, DenseMlpSpec) and m0.ff == 60 and m2 is None and m3.ff == 36
    assert isinstance(m1, RoutedMlpSpec) and (m1.ff, m1.experts, m1.top) == (20, 5, 2)
    assert a.slopes() == pytest.approx([2.0 ** (-8.0 / 3), 2.0 ** (-16.0 / 3), 2.0 ** -8.0])
    cb = ZavesunConfig.from_dict(ZAVESUN_B)
    assert cb.logit_softcap == 0.0 and cb.streams == 2 and cb.first_value_mix() == 0
    cc = ZavesunConfig.from_dict(ZAVESUN_C)
    assert cc.streams == 1 and cc.first_value_mix() is None and cc.layers[2].mixer.window == 0


@pytest.mark.parametrize("edit,message", [
    (lambda d: d["layers"][0].update(type="mamba2"), "not a mixer"),
    (lambda d: d["layers"][0]["mixer"]["mask"].update(size=0), "mask"),
    (lambda d: d["layers"][1]["mixer"].pop("rot"), "rot"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"].update(kv_heads=2), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"]["q_temp"].update(every=0), "q_temp"),
    (lambda d: d["layers"][2]["mixer"].update(vdim=5), "mixed values"),
    (lambda d: d["layers"][1]["mlp"]["router"].update(top=6), "experts"),
    (lambda d: d["layers"][0]["mlp"].update(kind="routed"), "feed-forward"),
    (lambda d: d["layers"][1]["mlp"].pop("expert"), "expert"),
    (lambda d: d.update(streams=-1), "streams"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0.0), "factor"),
])
def test_config_refusals(edit, message):
    d = copy.deepcopy(ZAVESUN_A)
    edit(d)
    with pytest.raises(ConfigError, match=message):
        ZavesunConfig.from_dict(d)


def test_registry_names_and_cache_layout():
    arch = registry.lookup(registry.architecture_name(ZAVESUN_A))
    assert arch.name == "Zavesun"
    cfg = arch.read_config(ZAVESUN_A)
    model = arch.build(cfg, torch.float32, "cpu", max_positions=8)
    names = arch.hf_names(cfg)
    assert names["l1.mix.q.b"] == "blk.1.mix.q.bias" and names["l1.mix.k.norm"] == "blk.1.mix.k.norm.weight"
    assert names["l1.mlp.e4.down"] == "blk.1.mlp.e4.down.weight" and names["l1.mlp.router"] == "blk.1.mlp.router.weight"
    assert names["l0.hc2.mix"] == "blk.0.hc2.mix" and "l2.hc2.mix" not in names and "l0.mix.vmix" not in names
    specs = model.weight_specs()
    assert set(names.values()) == set(specs)                   # every declared tensor has a name in the file and back
    assert "output.weight" not in specs                        # the embedding table is the output matrix
    assert specs["blk.0.hc1.mix"][0].shape == (3, 3) and specs["blk.2.mix.vmix"][0].shape == ()
    assert specs["blk.1.mix.q.weight"][0].shape == (4 * 12, 52) and specs["blk.1.mix.v.bias"][0].shape == (2 * 6,)
    assert specs["blk.3.mix.q.norm.weight"][0].shape == (6,) and "blk.0.mix.q.norm.weight" not in specs
    from ferrum_b200.cache.storage import CacheLayout
    lay = CacheLayout(model)
    assert lay.group_keys == [(1, 14, 19, 2), (2, 12, 21, 2), (2, 8, 7, 2), (1, 12, 11, 2)]     # (kv heads, max(dim, vdim), window, parts)
    mixers = [b.mixer for b in model.blocks]
    assert [m.chunked for m in mixers] == [False, True, False, True]
    assert [m.value_mix for m in mixers] == [None, "first", "blend", "blend"]
    assert model.embedding.copies == 3 and model.head.softcap == 9.0


def test_weights_are_checked(tmp_path):
    from ferrum_b200.weights.loader import check_weights, open_source
    folder = write_model(ZAVESUN_A, str(tmp_path / "a"), 1)
    arch, cfg = registry.read_config(folder)
    model = arch.build(cfg, torch.float32, "cpu", max_positions=4)
    have = {n: e[0] for n, e in open_source(folder).entries.items()}
    specs = {n: s for n, (s, _, _) in model.weight_specs().items()}
    assert len(check_weights(specs, have, arch.hf_names(cfg))) == len(specs)
    del have["l1.mlp.e3.up"]
    have["l0.hc1.mix"] = (3,)
    have["l0.mix.q.b"] = (30,)
    with pytest.raises(WeightsError) as e:
        check_weights(specs, have, arch.hf_names(cfg))
    assert "l1.mlp.e3.up" in str(e.value) and "l0.hc1.mix" in str(e.value) and "l0.mix.q.b" in str(e.value)


def test_one_stream_may_leave_its_stream_tensors_out():
    arch = registry.lookup("Zavesun")
    cfg = arch.read_config(ZAVESUN_C)
    model = arch.build(cfg, torch.float32, "cpu", max_positions=4)
    specs = model.weight_specs()
    assert specs["blk.0.hc1.in"][0].optional and specs["blk.0.hc2.mix"][0].optional
    model3 = arch.build(arch.read_config(ZAVESUN_A), torch.float32, "cpu", max_positions=4)
    assert not model3.weight_specs()["blk.0.hc1.in"][0].optional


# --------------------------------------------------------------------------- anchors of the plain functions
def test_plain_small_functions():
    v = torch.tensor([[3.0, 4.0]], dtype=F64)
    assert torch.allclose(P.rms(v, 0.0), v / math.sqrt(12.5))
    assert torch.allclose(P.rms(v, 12.5), v / 5.0)
    assert P.silu(torch.tensor(0.0, dtype=F64)).item() == 0.0 and abs(P.silu(torch.tensor(1.0, dtype=F64)).item() - 0.7310585786) < 1e-9
    assert abs(P.gelu_tanh(torch.tensor(1.0, dtype=F64)).item() - 0.8411919906) < 1e-9
    assert P.head_slopes(4).tolist() == pytest.approx([0.25, 0.0625, 0.015625, 0.00390625])
    t = P.query_temperature(torch.tensor([0, 6, 7, 14, 15, 16]), 0.5, 8)
    assert t.tolist() == pytest.approx([1.0, 1.0, 1.0 + 0.5 * math.log(2), 1.0 + 0.5 * math.log(2), 1.0 + 0.5 * math.log(3), 1.0 + 0.5 * math.log(3)])


def test_plain_masks():
    w = P.window_mask(6, 3)
    assert w[5].tolist() == [False, False, False, True, True, True] and w[1].tolist() == [True, True, False, False, False, False]
    c = P.chunk_mask(7, 3)
    assert c[2].tolist() == [True, True, True, False, False, False, False]
    assert c[3].tolist() == [False, False, False, True, False, False, False]
    assert c[6].tolist() == [False] * 6 + [True]
    assert P.window_mask(4, 1).sum().item() == 4 and P.chunk_mask(4, 1).sum().item() == 4


def test_plain_rotation_and_frequencies():
    f = P.linear_frequencies(100.0, 4, 2.0)
    assert f == pytest.approx([0.5, 0.05])
    v = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 5.0, 6.0]]], dtype=F64)
    out = P.rotate_interleaved(v, torch.tensor([3]), f, 4)
    a0, a1 = 3 * 0.5, 3 * 0.05
    assert out[0, 0].tolist() == pytest.approx([math.cos(a0), math.sin(a0), -2.0 * math.sin(a1), 2.0 * math.cos(a1), 5.0, 6.0])
    assert torch.equal(P.rotate_interleaved(v, torch.tensor([0]), f, 4), v)


def test_plain_attention_bias_and_grouping():
    """Two keys with equal scores: the distance bias alone decides the weights; head h reads KV head h // 2."""
    q = torch.zeros(2, 4, 2, dtype=F64)
    k = torch.zeros(2, 2, 2, dtype=F64)
    v = torch.tensor([[[1.0], [10.0]], [[2.0], [20.0]]], dtype=F64)
    slopes = P.head_slopes(4)
    dist = torch.tensor([[0.0, -1.0], [1.0, 0.0]], dtype=F64)
    out = P.softmax_attention(q, k, v, 1.0, P.window_mask(2, 2), slopes[:, None, None] * dist[None])
    for h in range(4):
        w1 = 1.0 / (1.0 + math.exp(-slopes[h].item()))       # weight of the nearer key (itself)
        base = 1.0 if h < 2 else 10.0
        assert out[0, h].item() == pytest.approx(base)
        assert out[1, h].item() == pytest.approx(base * ((1 - w1) * 1 + w1 * 2))


def test_plain_router_and_streams():
    h = torch.tensor([[1.0, 0.0], [0.0, 2.0]], dtype=F64)
    wr = torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.5, 0.5]], dtype=F64)
    idx, w = P.router_choice(h, wr, 2, None)
    assert idx.tolist() == [[0, 2], [1, 2]]
    assert w[0].tolist() == pytest.approx([1 / (1 + math.exp(-1.0)), 1 / (1 + math.exp(-0.5))])
    X = torch.arange(12, dtype=F64).view(3, 2, 2)
    a = torch.tensor([1.0, 0.0, -1.0], dtype=F64)
    assert torch.equal(P.streams_read(X, a), X[0] - X[2])
    M = torch.zeros(3, 3, dtype=F64)
    M[0, 1] = 2.0                                             # stream 0 goes to stream 1, doubled: [from, to]
    y = torch.ones(2, 2, dtype=F64)
    out = P.streams_write(X, M, torch.tensor([0.0, 0.0, 3.0], dtype=F64), y)
    assert torch.equal(out[0], torch.zeros(2, 2, dtype=F64)) and torch.equal(out[1], 2 * X[0]) and torch.equal(out[2], 3 * y)
    assert torch.equal(P.mix_values(torch.tensor(2.0), torch.tensor(10.0), 0.25), torch.tensor(4.0))


def test_plain_model_runs_and_layers_sum(tmp_path):
    folder = write_model(ZAVESUN_A, str(tmp_path / "a"), 2)
    cfg, w = P.load(folder)
    taps = []
    logits = P.forward(cfg, w, [5, 9, 100, 3, 3, 7], None, taps)
    assert logits.shape == (6, 197) and len(taps) == 4 and taps[0].shape == (6, 52)
    assert logits.abs().max().item() < 9.0                    # the soft cap
    # causality: a later token changes nothing before it
    again = P.forward(cfg, w, [5, 9, 100, 3, 3, 8], None)
    assert (again[:5] - logits[:5]).abs().max().item() < 1e-12 and (again[5] - logits[5]).abs().max().item() > 1e-6
    for name, c in (("b", ZAVESUN_B), ("c", ZAVESUN_C)):
        cfg, w = P.load(write_model(c, str(tmp_path / name), 3))
        assert torch.isfinite(P.forward(cfg, w, list(range(40)), torch.bfloat16)).all()
