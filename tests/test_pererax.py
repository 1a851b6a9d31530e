"""Pererax without a GPU: configuration, tensor names, cache layout, and hand-worked anchors of the
plain implementation's functions."""
import copy
import math

import pytest
import torch

import plain_pererax as P
from pererax_configs import PERERAX_A, PERERAX_B, PERERAX_C, write_model

from ferrum_b200.config import registry
from ferrum_b200.config.pererax import AttentionSpec, DeltaSpec, ParallelSpec, PereraxConfig
from ferrum_b200.errors import ConfigError, WeightsError

F64 = torch.float64


def test_config_reads_every_size_and_constant():
    c = PereraxConfig.from_dict(PERERAX_A)
    assert (c.n_vocab, c.n_embd, c.norm_eps, c.n_layer) == (197, 52, 1e-5, 5)
    pair, att, delta = c.layers[0].mixer, c.layers[1].mixer, c.layers[2].mixer
    assert isinstance(pair, ParallelSpec) and isinstance(att, AttentionSpec) and isinstance(delta, DeltaSpec)
    left, right = pair.left, pair.right
    assert (left.heads, left.kv_heads, left.dim, left.vdim, left.scale, left.softcap, left.rot_base, left.rot_dims) == (3, 1, 10, 14, 0.4, 3.0, 100.0, 6)
    assert left.sink and not left.value_is_key and left.window == 0
    assert (right.heads, right.dim, right.vdim, right.gate_cap) == (3, 6, 10, 7.0)
    assert (att.heads, att.kv_heads, att.dim, att.vdim, att.window, att.rot_dims) == (4, 2, 12, 12, 19, 8)
    assert att.value_is_key and not att.sink and att.softcap == 0.0
    assert (delta.heads, delta.kv_heads, delta.dim, delta.vdim, delta.taps, delta.decay_rank, delta.gate_rank) == (4, 2, 10, 6, 3, 5, 7)
    p = c.layers[0].mlp
    assert (p.expert.ff, p.expert.limit, p.experts, p.identity, p.top, p.scale, p.shared.ff, p.shared.limit) == (20, 2.5, 5, 2, 3, 1.5, 28, 1.5)
    assert c.layers[1].mlp is None
    assert [c.owner(i) for i in range(5)] == [0, 1, 2, 0, 2]
    cc = PereraxConfig.from_dict(PERERAX_C)
    assert cc.layers[2].mixer.left.rot_dims == 0 and cc.layers[2].mixer.left.softcap == 0.0
    assert cc.layers[0].mlp.shared is None and cc.layers[0].mlp.scale == 1.0 and cc.layers[2].mlp.identity == 0
    d = copy.deepcopy(PERERAX_B)
    d["layers"][0]["mixer"].pop("decay_rank")
    assert PereraxConfig.from_dict(d).layers[0].mixer.decay_rank is None          # the tensors' shapes decide then


@pytest.mark.parametrize("edit,message", [
    (lambda d: d["layers"][0].update(type="mamba2"), "not a mixer"),
    (lambda d: d["layers"][1]["mixer"]["mask"].update(size=0), "mask"),
    (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda d: d["layers"][1]["mixer"].update(vdim=10), "vdim = dim"),
    (lambda d: d["layers"][1]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"].pop("right"), "right"),
    (lambda d: d["layers"][0]["mixer"]["right"].update(gate_cap=0.0), "gate_cap"),
    (lambda d: d["layers"][2]["mixer"].pop("conv"), "conv"),
    (lambda d: d["layers"][2]["mlp"]["router"].update(top=8), "experts"),
    (lambda d: d["layers"][2]["mlp"]["expert"].update(limit=0.0), "limit"),
    (lambda d: d["layers"][2]["mlp"].update(kind="dense"), "feed-forward"),
    (lambda d: d["layers"][3].update(weights_of=9), "weights_of"),
    (lambda d: d["layers"][3].update(weights_of=1), "differs"),
    (lambda d: d.pop("width"), "width"),
])
def test_config_refusals(edit, message):
    d = copy.deepcopy(PERERAX_A)
    edit(d)
    with pytest.raises(ConfigError, match=message):
        PereraxConfig.from_dict(d)


def test_registry_names_runs_and_cache_layout():
    arch = registry.lookup(registry.architecture_name(PERERAX_A))
    assert arch.name == "Pererax"
    cfg = arch.read_config(PERERAX_A)
    model = arch.build(cfg, torch.float32, "cpu", max_positions=8)
    # three blocks own tensors; layers 3 and 4 are second runs of blocks 0 and 2
    assert len(model.blocks) == 3 and [r.block for r in model.schedule] == [0, 1, 2, 0, 2]
    names = arch.hf_names(cfg)
    assert names["l0.mix.left.q.norm"] == "blk.0.mix.left.q.norm.weight" and names["l0.mix.right.f.b"] == "blk.0.mix.right.f.bias"
    assert names["l0.mix.left.out"] == "blk.0.mix.left_out" and names["l2.mix.q.conv"] == "blk.2.mix.q.conv"
    assert names["l2.mlp.e4.down"] == "blk.2.mlp.e4.down.weight" and names["l2.mlp.shared.up"] == "blk.2.mlp.shared.up.weight"
    assert names["l0.ls2"] == "blk.0.ls2" and "l1.ls2" not in names and "l1.mix.v" not in names and "l3.norm1" not in names
    specs = model.weight_specs()
    assert set(names.values()) == set(specs)                   # every declared tensor has a name in the file and back
    assert "output.weight" not in specs                        # the embedding table is the output matrix
    assert specs["blk.0.mix.left.q.norm.weight"][0].shape == (30,) and specs["blk.0.mix.left.k.norm.weight"][0].shape == (10,)
    assert specs["blk.1.mix.k.weight"][0].shape == (24, 52) and specs["blk.0.mix.right.norm.weight"][0].shape == (30,)
    assert specs["blk.2.mix.a2.weight"][0].shape == (40, 5) and specs["blk.2.mix.g2.weight"][0].shape == (24, 7)
    assert specs["blk.2.mix.norm.weight"][0].shape == (6,) and specs["blk.2.mix.dt_bias"][0].shape == (40,)
    assert specs["blk.0.mlp.router.weight"][0].shape == (7, 52) and specs["blk.0.mlp.correction"][0].shape == (7,)
    from ferrum_b200.cache.storage import CacheLayout
    lay = CacheLayout(model)
    assert lay.group_keys == [(1, 14, 0, 2), (2, 12, 19, 2)]     # (kv heads, max(dim, vdim), window, parts)
    assert lay.group_planes == [2, 1]                            # both runs of the pair keep pages of their own
    assert lay.run_state == [0, None, 1, 2, 3]                   # ... and every recurrent run a state row of its own
    delta_state = 4 * 10 * 6 + 2 * (2 * 2 * 10 + 4 * 6)
    assert lay.state_needs[1].shape == (delta_state,)
    assert lay.state_needs[0].shape == (3 * 6 * 10 + 2 * (3 * 6 + 3),)      # S, and a copy of n and m per eight value columns


def test_low_rank_sizes_come_from_the_file_and_wrong_weights_are_listed(tmp_path):
    d = copy.deepcopy(PERERAX_C)
    folder = write_model(d, str(tmp_path / "c"), 1)
    open_cfg = copy.deepcopy(d)
    for k in ("decay_rank", "gate_rank"):
        open_cfg["layers"][1]["mixer"].pop(k)
    arch = registry.lookup("Pererax")
    cfg = arch.read_config(open_cfg)
    model = arch.build(cfg, torch.float32, "cpu", max_positions=8)
    from ferrum_b200.weights import load_weights
    load_weights(model, folder, arch.hf_names(cfg), device="cpu")
    mixer = model.blocks[1].mixer
    assert (mixer.ra, mixer.rg) == (1, 2) and mixer.w_low.shape == (3, 32) and mixer.w_conv.shape == (4 + 4 + 36, 1)
    wide = copy.deepcopy(d)
    wide["layers"][0]["mixer"].update(heads=2, kv_heads=2)
    cfg = arch.read_config(wide)
    with pytest.raises(WeightsError, match="l0.mix.q.norm"):
        load_weights(arch.build(cfg, torch.float32, "cpu", max_positions=8), folder, arch.hf_names(cfg), device="cpu")


# ----------------------------------------------------------------------------- anchors of the plain functions
def test_rotation_pairs_element_i_with_i_plus_half():
    v = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=F64)              # one token, one head of six, four of them turn
    out = P.rotate_half(v, torch.tensor([3]), 100.0, 4)
    f = [1.0, 100.0 ** -0.5]
    for i in range(2):
        a = 3 * f[i]
        assert out[0, 0, i].item() == pytest.approx(v[0, 0, i].item() * math.cos(a) - v[0, 0, i + 2].item() * math.sin(a))
        assert out[0, 0, i + 2].item() == pytest.approx(v[0, 0, i + 2].item() * math.cos(a) + v[0, 0, i].item() * math.sin(a))
    assert out[0, 0, 4:].tolist() == [5.0, 6.0]
    assert torch.equal(P.rotate_half(v, torch.tensor([0]), 100.0, 4), v)


def test_window_and_sink_weights_by_hand():
    assert P.causal_mask(4, 2).int().tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [0, 1, 1, 0], [0, 0, 1, 1]]
    assert P.causal_mask(3).int().tolist() == [[1, 0, 0], [1, 1, 0], [1, 1, 1]]
    s = torch.tensor([[math.log(1.0), math.log(3.0)]], dtype=F64)
    m = torch.ones(1, 2, dtype=torch.bool)
    assert P.masked_softmax(s, m, False)[0].tolist() == pytest.approx([0.25, 0.75])
    assert P.masked_softmax(s, m, True)[0].tolist() == pytest.approx([0.2, 0.6])            # the sink takes e^0 = 1 of 5
    low = torch.tensor([[-50.0]], dtype=F64)                                                 # far below the sink: almost nothing left
    assert P.masked_softmax(low, torch.ones(1, 1, dtype=torch.bool), True)[0, 0].item() == pytest.approx(math.exp(-50.0), rel=1e-9)
    assert P.soft_cap(torch.tensor(1e9, dtype=F64), 30.0).item() == pytest.approx(30.0)
    assert P.soft_cap(torch.tensor(0.3, dtype=F64), 30.0).item() == pytest.approx(30.0 * math.tanh(0.01))


def test_convolution_and_unit_vectors_by_hand():
    u = torch.tensor([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0]], dtype=F64)
    taps = torch.tensor([[0.5, 1.0], [2.0, -1.0]], dtype=F64)                    # the last column is the current token's
    assert P.short_conv(u, taps).tolist() == [[1.0, -10.0], [2.5, 0.0], [4.0, 10.0]]
    v = P.unit(torch.tensor([3.0, 4.0], dtype=F64))
    assert v.tolist() == pytest.approx([3.0 / math.sqrt(25.0 + 1e-6), 4.0 / math.sqrt(25.0 + 1e-6)])


def test_two_tokens_of_the_delta_rule_by_hand():
    # one head, two key channels, one value: k1 = (1, 0), k2 = (0, 1) scaled; the read-out sees the current write
    q = torch.tensor([[[1.0, 0.0]], [[1.0, 1.0]]], dtype=F64)
    k = torch.tensor([[[1.0, 0.0]], [[1.0, 0.0]]], dtype=F64)
    v = torch.tensor([[[2.0]], [[6.0]]], dtype=F64)
    beta = torch.tensor([[0.5], [1.0]], dtype=F64)
    g = torch.tensor([[[1.0, 1.0]], [[0.5, 0.25]]], dtype=F64)
    o = P.delta_walk(q, k, v, beta, g)
    # token 0: S = 0 -> e = 0.5 * 2 = 1, S = [[1], [0]], o = 1.  token 1: S = [[0.5], [0]], e = 6 - 0.5 = 5.5, S = [[6], [0]], o = 6
    assert o[:, 0, 0].tolist() == pytest.approx([1.0, 6.0])


def test_two_tokens_of_the_matrix_memory_by_hand():
    q = torch.tensor([[[1.0]], [[1.0]]], dtype=F64)
    k = torch.tensor([[[1.0]], [[2.0]]], dtype=F64)
    v = torch.tensor([[[3.0]], [[5.0]]], dtype=F64)
    ig = torch.tensor([[math.log(2.0)], [-1.0]], dtype=F64)
    fg = torch.tensor([[-0.3], [math.log(0.5)]], dtype=F64)
    o = P.matrix_memory_walk(q, k, v, ig, fg)
    # token 0: m = max(-0.3 + 0, ln 2) = ln 2; S = 1 * 1 * 3 = 3, n = 1; o = 3 / (max(1, 1/2) + 1e-6)
    assert o[0, 0, 0].item() == pytest.approx(3.0 / (1.0 + 1e-6))
    # token 1: m' = max(ln 0.5 + ln 2, -1) = 0; a = 1, b = e^-1; S = 3 + 10/e, n = 1 + 2/e; e^(-m') = 1 < n
    e = math.exp(-1.0)
    assert o[1, 0, 0].item() == pytest.approx((3.0 + 10.0 * e) / (1.0 + 2.0 * e + 1e-6))
    # a running maximum that starts at 0, not at minus infinity: a very negative first input gate leaves m = f
    o = P.matrix_memory_walk(q[:1], k[:1], v[:1], torch.tensor([[-20.0]], dtype=F64), torch.tensor([[-0.5]], dtype=F64))
    b = math.exp(-20.0 + 0.5)
    assert o[0, 0, 0].item() == pytest.approx(3.0 * b / (math.exp(0.5) + 1e-6))


def test_clamped_unit_and_routing_by_hand():
    w = {"u.gate": torch.tensor([[1.0]], dtype=F64), "u.up": torch.tensor([[1.0]], dtype=F64), "u.down": torch.tensor([[1.0]], dtype=F64)}
    x = torch.tensor([[0.5], [5.0], [-5.0]], dtype=F64)
    y = P.clamped_unit(x, w, "u.", 2.0)
    sig = lambda z: 1.0 / (1.0 + math.exp(-z))
    assert y[:, 0].tolist() == pytest.approx([0.5 * sig(0.851) * 1.5, 2.0 * sig(3.404) * 3.0, -5.0 * sig(-8.51) * -1.0])
    # three outputs, the last an identity expert; the correction changes the choice and not the weights
    w = {"r.router": torch.tensor([[1.0], [0.0], [-1.0]], dtype=F64), "r.correction": torch.tensor([0.0, 0.0, 10.0], dtype=F64)}
    idx, wt, s = P.route(torch.tensor([[math.log(2.0)]], dtype=F64), w, "r.", {"experts": 2, "identity": 1, "top": 2, "scale": 7.0})
    assert idx.tolist() == [[2, 0]]
    assert s[0].tolist() == pytest.approx([2.0 / 3.5, 1.0 / 3.5, 0.5 / 3.5])
    assert wt[0].tolist() == pytest.approx([7.0 * 0.5 / 3.5, 7.0 * 2.0 / 3.5])
    tie = {"r.router": torch.zeros(3, 1, dtype=F64), "r.correction": torch.zeros(3, dtype=F64)}
    assert P.route(torch.ones(1, 1, dtype=F64), tie, "r.", {"experts": 3, "top": 2})[0].tolist() == [[0, 1]]


def test_plain_model_runs_shared_layers_with_the_owners_tensors(tmp_path):
    folder = write_model(PERERAX_A, str(tmp_path / "a"), 2)
    cfg, w = P.load(folder)
    assert not any(k.startswith("l3.") or k.startswith("l4.") for k in w)
    taps = []
    logits = P.forward(cfg, w, [5, 9, 1, 5, 100, 42], None, taps)
    assert logits.shape == (6, 197) and len(taps) == 5 and bool(torch.isfinite(logits).all())
    # the prefix of a sequence gives the prefix of its logits (causality of every mechanism)
    assert (P.forward(cfg, w, [5, 9, 1, 5], None) - logits[:4]).abs().max() < 1e-9
