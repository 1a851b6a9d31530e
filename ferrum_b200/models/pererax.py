"""The Pererax decoder, built from parts, and its entry in the registry.

Token embedding; layers that are `PostNormBlock`s (the sublayers read the residual row itself, an RMS
norm and a layer scale sit on their results) around a mixer out of three and a routed feed-forward:

  mixers         attention in a sliding window whose values are its keys as projected, with an RMS norm
                 over the whole query and key projections and a rotation of part of each head; a pair
                 of mixers side by side whose normed results are averaged (causal attention with a soft
                 cap on the scores and a sink in the softmax, and a matrix-memory recurrence); or a
                 gated delta rule with a decay per key channel behind short convolutions
  feed-forward   a mixture of clamped gated units chosen by softmax scores plus a correction, some of
                 the router's outputs standing for identity experts, and one unit for every token

then an RMS norm and the embedding table again as the output matrix.  A layer may use another layer's
tensors (`weights_of`): it is a second run of that layer's block, with cache planes and a state of its
own.

The checkpoint's tensor names are short (`embed`, `l<i>.norm1`, `l<i>.ls1`, `l<i>.mix.q`, `l<i>.mix.q.norm`,
`l<i>.mix.left.q`, `l<i>.mix.q.conv`, `l<i>.mlp.e<j>.gate`, `l<i>.mlp.shared.up`, `final.norm`);
`file_names` maps them onto the canonical names that the parts declare.
"""
from __future__ import annotations

from ..config.pererax import AttentionSpec, DeltaSpec, ParallelSpec, PereraxConfig
from ..config.registry import Architecture, register
from ..parts import (ChannelDeltaMixer, MatrixMemoryMixer, OutputHead, ParallelMixer, PostNormBlock, RMSNorm, RotaryEmbedding,
                     RoutedFeedForward, ShapedAttention, SwiGLU, TokenEmbedding)
from .decoder import DecoderModel, Run


def _blocks_of(config: PereraxConfig):
    """layer index -> index of the block it runs: the layers that own tensors, numbered in order."""
    owners = sorted({config.owner(i) for i in range(config.n_layer)})
    number = {layer: b for b, layer in enumerate(owners)}
    return owners, [number[config.owner(i)] for i in range(config.n_layer)]


def build_pererax(config: PereraxConfig, dtype, device, max_positions=None):
    c = config
    E = c.n_embd
    n_pos = int(max_positions or c.n_ctx_train)
    tables = {}     # rotary tables shared by the layers that turn alike

    def rotary(head_dim, dims, base):
        key = (head_dim, dims, base)
        if key not in tables:
            tables[key] = RotaryEmbedding(head_dim, dims, base, None, "half", n_pos, device)
        return tables[key]

    def attention(m: AttentionSpec):
        rot = rotary(m.dim, m.rot_dims, m.rot_base) if m.rot_dims else None
        return ShapedAttention(E, m.heads, m.kv_heads, m.dim, m.vdim, dtype, m.scale, eps=c.norm_eps, window=m.window, rotary=rot,
                               qk_norm="whole", value_from_key=m.value_is_key, score_softcap=m.softcap, sink=m.sink)

    owners, block_of = _blocks_of(c)
    blocks = []
    for i in owners:
        layer = c.layers[i]
        m = layer.mixer
        if isinstance(m, AttentionSpec):
            mixer = attention(m)
        elif isinstance(m, ParallelSpec):
            r = m.right
            mixer = ParallelMixer(E, attention(m.left), MatrixMemoryMixer(E, r.heads, r.dim, r.vdim, r.gate_cap, c.norm_eps, dtype),
                                  c.norm_eps)
        else:
            mixer = ChannelDeltaMixer(E, m.heads, m.kv_heads, m.dim, m.vdim, m.taps, c.norm_eps, dtype, m.decay_rank, m.gate_rank)
        ffn = norm2 = None
        p = layer.mlp
        if p is not None:
            norm2 = RMSNorm(E, c.norm_eps, dtype)
            shared = SwiGLU(E, p.shared.ff, dtype, act="swish_clamp", limit=p.shared.limit) if p.shared is not None else None
            ffn = RoutedFeedForward(E, p.expert.ff, p.experts, p.top, dtype, act="swish_clamp", scores="softmax", renormalize=False,
                                    scale_input=False, correction=True, weight_scale=p.scale, identity=p.identity,
                                    limit=p.expert.limit, shared=shared)
        blocks.append(PostNormBlock(E, dtype, RMSNorm(E, c.norm_eps, dtype), mixer, norm2, ffn))
    emb = TokenEmbedding(c.n_vocab, E, copy_dtype=dtype)
    head = OutputHead(c.n_vocab, E, tied_to=emb, tied=True)
    return DecoderModel(c, dtype, emb, None, blocks, RMSNorm(E, c.norm_eps, dtype), head, schedule=[Run(b) for b in block_of])


def _attention_names(m: AttentionSpec, pre):
    names = {pre + "q": pre + "q.weight", pre + "k": pre + "k.weight", pre + "o": pre + "output.weight",
             pre + "q.norm": pre + "q.norm.weight", pre + "k.norm": pre + "k.norm.weight"}
    if not m.value_is_key:
        names[pre + "v"] = pre + "v.weight"
    return names


_MEMORY = {"q": "q.weight", "k": "k.weight", "v": "v.weight", "g": "g.weight", "o": "o.weight", "norm": "norm.weight",
           "i": "i.weight", "i.b": "i.bias", "f": "f.weight", "f.b": "f.bias"}
_DELTA = {"q": "q.weight", "q.conv": "q.conv", "k": "k.weight", "k.conv": "k.conv", "v": "v.weight", "v.conv": "v.conv",
          "b": "b.weight", "A_log": "A_log", "norm": "norm.weight", "a1": "a1.weight", "a2": "a2.weight", "dt_bias": "dt_bias",
          "g1": "g1.weight", "g2": "g2.weight", "o": "o.weight"}
_UNIT = ("gate", "up", "down")


def file_names(config: PereraxConfig):
    """{name in the checkpoint: canonical name}, for the tensors this configuration has."""
    out = {"embed": "token_embd.weight", "final.norm": "output_norm.weight"}
    owners, _ = _blocks_of(config)
    for b, i in enumerate(owners):
        layer = config.layers[i]
        m = layer.mixer
        names = {"norm1": "norm1.weight", "ls1": "ls1"}
        if isinstance(m, AttentionSpec):
            names.update(_attention_names(m, "mix."))
        elif isinstance(m, ParallelSpec):
            names.update(_attention_names(m.left, "mix.left."))
            names.update({"mix.right." + k: "mix.right." + v for k, v in _MEMORY.items()})
            names.update({"mix.left.out": "mix.left_out", "mix.right.out": "mix.right_out"})
        else:
            names.update({"mix." + k: "mix." + v for k, v in _DELTA.items()})
        p = layer.mlp
        if p is not None:
            names.update({"norm2": "norm2.weight", "ls2": "ls2", "mlp.router": "mlp.router.weight", "mlp.correction": "mlp.correction"})
            for e in range(p.experts):
                names.update({f"mlp.e{e}.{k}": f"mlp.e{e}.{k}.weight" for k in _UNIT})
            if p.shared is not None:
                names.update({f"mlp.shared.{k}": f"mlp.shared.{k}.weight" for k in _UNIT})
        for short, ours in names.items():
            out[f"l{i}.{short}"] = f"blk.{b}.{ours}"
    return out


register(Architecture("Pererax", PereraxConfig.from_dict, build_pererax, file_names), "pererax")
