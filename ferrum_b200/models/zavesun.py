"""The Zavesun decoder, built from parts, and its entry in the registry.

Token embedding written into S copies of the residual stream; layers that are `StreamBlock`s (a
read vector, a carry matrix and a write vector per sublayer over the S streams) around a mixer
out of two and a feed-forward out of two:

  mixers         attention in a sliding window with a per-head distance slope and a query
                 temperature that grows with the position (no rotation), or attention within
                 chunks of positions with biased projections, a weighted RMS norm of query and key
                 heads and an interleaved rotation of part of each head at divided frequencies;
                 either may blend its values with those of the first layer that mixes values
  feed-forwards  dense with gelu (tanh form) on the gate, or a mixture of experts with silu, whose
                 sigmoid router scores multiply the chosen experts' inputs

then an RMS norm of the sum of the streams and the embedding table again as the output matrix,
with a tanh soft cap on the logits.

The checkpoint's tensor names are short (`embed`, `l<i>.norm1`, `l<i>.mix.q`, `l<i>.mix.q.b`,
`l<i>.mlp.e<j>.gate`, `l<i>.hc1.in`, `final.norm`); `file_names` maps them onto the canonical names
that the parts declare.
"""
from __future__ import annotations

from ..config.registry import Architecture, register
from ..config.zavesun import RoutedMlpSpec, ZavesunConfig
from ..parts import (OutputHead, RMSNorm, RotaryEmbedding, RoutedFeedForward, ShapedAttention, StreamBlock, StreamSumNorm, SwiGLU,
                     TokenEmbedding)
from .decoder import DecoderModel

VALUE_MIX_KEY = "zavesun_v_first"


def build_zavesun(config: ZavesunConfig, dtype, device, max_positions=None):
    c = config
    E, S = c.n_embd, c.streams
    n_pos = int(max_positions or c.n_ctx_train)
    tables = {}     # rotary tables shared by the layers that turn alike

    def rotary(head_dim, dims, base, scaling):
        key = (head_dim, dims, base, scaling)
        if key not in tables:
            tables[key] = RotaryEmbedding(head_dim, dims, base, scaling, "adjacent", n_pos, device)
        return tables[key]

    first_mix = c.first_value_mix()
    blocks = []
    for i, layer in enumerate(c.layers):
        m = layer.mixer
        rot = rotary(m.dim, m.rot_dims, m.rot_base, m.rot_scaling) if m.rot_dims else None
        mixer = ShapedAttention(E, m.heads, m.kv_heads, m.dim, m.vdim, dtype, m.scale, eps=c.norm_eps, window=m.window,
                                rotary=rot, mask=m.mask, qkv_bias=m.qkv_bias, qk_norm=m.qk_norm, query_temperature=m.q_temp,
                                linear_bias=m.slopes() if m.linear_bias else None,
                                value_mix=("first" if i == first_mix else "blend") if m.v_mix else None,
                                value_mix_key=VALUE_MIX_KEY)
        ffn = norm2 = None
        if layer.mlp is not None:
            norm2 = RMSNorm(E, c.norm_eps, dtype)
            if isinstance(layer.mlp, RoutedMlpSpec):
                ffn = RoutedFeedForward(E, layer.mlp.ff, layer.mlp.experts, layer.mlp.top, dtype, act="silu", scores="sigmoid",
                                        renormalize=False, scale_input=True)
            else:
                ffn = SwiGLU(E, layer.mlp.ff, dtype, act="gelu_tanh")
        blocks.append(StreamBlock(S, RMSNorm(E, c.norm_eps, dtype), mixer, norm2, ffn))
    emb = TokenEmbedding(c.n_vocab, E, copies=S)
    head = OutputHead(c.n_vocab, E, tied_to=emb, tied=True, softcap=c.logit_softcap)
    return DecoderModel(c, dtype, emb, None, blocks, StreamSumNorm(S, E, c.norm_eps, dtype), head)


_ATTENTION = {"mix.q": "mix.q.weight", "mix.k": "mix.k.weight", "mix.v": "mix.v.weight", "mix.o": "mix.output.weight"}
_BIASES = {"mix.q.b": "mix.q.bias", "mix.k.b": "mix.k.bias", "mix.v.b": "mix.v.bias"}
_HEAD_NORMS = {"mix.q.norm": "mix.q.norm.weight", "mix.k.norm": "mix.k.norm.weight"}
_STREAMS = {f"hc{q}.{k}": f"hc{q}.{k}" for q in (1, 2) for k in ("in", "mix", "out")}


def file_names(config: ZavesunConfig):
    """{name in the checkpoint: canonical name}, for the tensors this configuration has."""
    out = {"embed": "token_embd.weight", "final.norm": "output_norm.weight"}
    for i, layer in enumerate(config.layers):
        m = layer.mixer
        names = {"norm1": "norm1.weight"}
        names.update(_ATTENTION)
        names.update(_BIASES if m.qkv_bias else {})
        names.update(_HEAD_NORMS if m.qk_norm else {})
        if m.v_mix:
            names["mix.vmix"] = "mix.vmix"
        names.update({k: v for k, v in _STREAMS.items() if layer.mlp is not None or k.startswith("hc1")})
        if layer.mlp is not None:
            names["norm2"] = "norm2.weight"
            if isinstance(layer.mlp, RoutedMlpSpec):
                names["mlp.router"] = "mlp.router.weight"
                for e in range(layer.mlp.experts):
                    names.update({f"mlp.e{e}.{k}": f"mlp.e{e}.{k}.weight" for k in ("gate", "up", "down")})
            else:
                names.update({f"mlp.{k}": f"mlp.{k}.weight" for k in ("gate", "up", "down")})
        for short, ours in names.items():
            out[f"l{i}.{short}"] = f"blk.{i}.{ours}"
    return out


register(Architecture("Zavesun", ZavesunConfig.from_dict, build_zavesun, file_names), "zavesun")
