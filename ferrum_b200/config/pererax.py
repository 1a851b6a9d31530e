"""Typed configuration of the Pererax decoder.

Its config.json is nested: `architecture`, `vocab`, `width`, `norm.eps` and `layers`, a list whose
entries give the layer's `type` (which mixer), the mixer's sizes under `mixer`, its feed-forward
under `mlp` (null: none) and, optionally, `weights_of`: the index of the layer whose tensors this
layer uses (it has none of its own, but a cache and a state of its own).  Every size and every
constant that can differ between two models of the design is read here and nowhere else; what an
entry does not mention does not exist (no `mask`: every earlier key; no `softcap`: plain scores;
no `rot`: no rotation; no `shared`: no unit that every token runs through).

Mixers:
  `attention`      heads, kv_heads, dim, vdim, scale, rot.{base, dims}, mask.size (a query sees
                   itself and the mask.size - 1 keys before it); the values are the keys as
                   projected, so vdim equals dim and there is no value matrix.
  `parallel`       `left`: heads, kv_heads, dim, vdim, scale, softcap, rot.{base, dims}: causal
                   attention with a sink in the softmax; `right`: heads, dim, vdim, gate_cap: a
                   matrix-memory recurrence.  Both read the layer's input; their normed results
                   are averaged.
  `channel_delta`  heads, kv_heads, dim, vdim, conv (taps): a gated delta rule with a decay per
                   key channel.  The inner sizes of its two low-rank pairs are read off the tensors
                   (optional keys `decay_rank`, `gate_rank` fix them, e.g. for random weights).

Feed-forward (`mlp.kind` = `moe`): expert.{ff, limit}, router.{experts, identity, top, scale},
shared.{ff, limit}.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Tuple, Union

from ..errors import ConfigError


@dataclass(frozen=True)
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0                 # 0: every earlier key
    rot_base: float = 0.0
    rot_dims: int = 0               # 0: no rotation
    softcap: float = 0.0            # 0: plain scores
    sink: bool = False              # a key of score 0 without a value in every softmax
    value_is_key: bool = False      # no value matrix: the values are the keys as projected


@dataclass(frozen=True)
class MatrixMemorySpec:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ParallelSpec:
    left: AttentionSpec
    right: MatrixMemorySpec


@dataclass(frozen=True)
class DeltaSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int
    decay_rank: Optional[int] = None    # inner sizes of the two low-rank pairs; None: as the weights' file has them
    gate_rank: Optional[int] = None


@dataclass(frozen=True)
class UnitSpec:
    ff: int
    limit: float


@dataclass(frozen=True)
class RoutedMlpSpec:
    expert: UnitSpec
    experts: int                    # experts with matrices
    identity: int                   # further router outputs whose expert is the identity
    top: int
    scale: float                    # multiplies the chosen scores
    shared: Optional[UnitSpec] = None
    kind: str = "moe"


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: Union[AttentionSpec, ParallelSpec, DeltaSpec]
    mlp: Optional[RoutedMlpSpec]
    weights_of: Optional[int] = None


@dataclass(frozen=True)
class PereraxConfig:
    architecture: str
    n_vocab: int
    n_embd: int
    norm_eps: float
    layers: Tuple[LayerSpec, ...]
    n_ctx_train: int = 8192         # positions the rotary tables cover unless the caller asks for more or fewer
    eos_token_ids: Tuple[int, ...] = ()
    stored_dtype: str = "bfloat16"
    extra: dict = field(default_factory=dict, compare=False)

    @property
    def n_layer(self):
        return len(self.layers)

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself unless it says `weights_of`)."""
        while self.layers[i].weights_of is not None:
            i = self.layers[i].weights_of
        return i

    def __post_init__(self):
        for k in ("n_vocab", "n_embd"):
            v = getattr(self, k)
            if not isinstance(v, int) or v <= 0:
                raise ConfigError(f"pererax: {k} must be a positive integer, found {v!r}")
        if not (math.isfinite(self.norm_eps) and self.norm_eps > 0.0):
            raise ConfigError("pererax: invalid norm.eps")
        if not self.layers:
            raise ConfigError("pererax: no layers")

        def attention(i, m):
            for k in ("heads", "kv_heads", "dim", "vdim"):
                if getattr(m, k) <= 0:
                    raise ConfigError(f"pererax: layer {i}: {k} must be positive")
            if m.heads % m.kv_heads:
                raise ConfigError(f"pererax: layer {i}: kv_heads does not divide heads")
            if not math.isfinite(m.scale):
                raise ConfigError(f"pererax: layer {i}: invalid scale")
            if m.rot_dims % 2 or m.rot_dims > m.dim or m.rot_dims < 0:
                raise ConfigError(f"pererax: layer {i}: rot.dims must be even and at most dim")
            if m.rot_dims and not (math.isfinite(m.rot_base) and m.rot_base > 0):
                raise ConfigError(f"pererax: layer {i}: invalid rot.base")
            if not (math.isfinite(m.softcap) and m.softcap >= 0.0):
                raise ConfigError(f"pererax: layer {i}: invalid softcap")
            if m.value_is_key and m.vdim != m.dim:
                raise ConfigError(f"pererax: layer {i}: values that are the keys need vdim = dim")

        for i, layer in enumerate(self.layers):
            m = layer.mixer
            j = layer.weights_of
            if j is not None:
                if not 0 <= j < len(self.layers) or j == i:
                    raise ConfigError(f"pererax: layer {i}: weights_of names layer {j}, which does not exist")
                seen, k = {i}, j
                while self.layers[k].weights_of is not None:
                    if k in seen:
                        raise ConfigError(f"pererax: layer {i}: weights_of runs in a circle")
                    seen.add(k)
                    k = self.layers[k].weights_of
                o = self.layers[k]
                if (o.type, o.mixer, o.mlp) != (layer.type, layer.mixer, layer.mlp):
                    raise ConfigError(f"pererax: layer {i} uses the weights of layer {k} but differs from it")
            if isinstance(m, AttentionSpec):
                attention(i, m)
            elif isinstance(m, ParallelSpec):
                attention(i, m.left)
                r = m.right
                if min(r.heads, r.dim, r.vdim) <= 0 or not (math.isfinite(r.gate_cap) and r.gate_cap > 0):
                    raise ConfigError(f"pererax: layer {i}: invalid sizes or gate_cap of the right mixer")
            else:
                if min(m.heads, m.kv_heads, m.dim, m.vdim, m.taps) <= 0 or m.heads % m.kv_heads:
                    raise ConfigError(f"pererax: layer {i}: invalid sizes of the delta mixer")
            p = layer.mlp
            if p is not None:
                units = [p.expert] + ([p.shared] if p.shared is not None else [])
                if any(u.ff <= 0 or not (math.isfinite(u.limit) and u.limit > 0) for u in units):
                    raise ConfigError(f"pererax: layer {i}: a unit's ff and limit must be positive")
                if p.experts <= 0 or p.identity < 0 or not 0 < p.top <= p.experts + p.identity or not math.isfinite(p.scale):
                    raise ConfigError(f"pererax: layer {i}: {p.top} of {p.experts} + {p.identity} experts per token")

    @staticmethod
    def from_dict(d: dict) -> "PereraxConfig":
        def need(obj, key, where=""):
            if not isinstance(obj, dict) or key not in obj or obj[key] is None:
                raise ConfigError(f"config.json: missing required key {where}{key!r}")
            return obj[key]

        def attention(m, mw, sink, value_is_key):
            window = 0
            if m.get("mask") is not None:
                window = int(need(m["mask"], "size", mw + "mask."))
                if window <= 0:
                    raise ConfigError(f"config.json: {mw}mask.size must be positive")
            rot_base, rot_dims = 0.0, 0
            if m.get("rot") is not None:
                rot_base, rot_dims = float(need(m["rot"], "base", mw + "rot.")), int(need(m["rot"], "dims", mw + "rot."))
            return AttentionSpec(heads=int(need(m, "heads", mw)), kv_heads=int(need(m, "kv_heads", mw)), dim=int(need(m, "dim", mw)),
                                 vdim=int(need(m, "vdim", mw)), scale=float(need(m, "scale", mw)), window=window,
                                 rot_base=rot_base, rot_dims=rot_dims, softcap=float(m.get("softcap") or 0.0), sink=sink,
                                 value_is_key=value_is_key)

        def unit(u, where):
            return UnitSpec(ff=int(need(u, "ff", where)), limit=float(need(u, "limit", where)))

        layers = []
        for i, L in enumerate(need(d, "layers")):
            where = f"layers[{i}]."
            kind = need(L, "type", where)
            m = need(L, "mixer", where)
            mw = where + "mixer."
            if kind == "attention":
                spec = attention(m, mw, sink=False, value_is_key=True)
            elif kind == "parallel":
                r = need(m, "right", mw)
                rw = mw + "right."
                spec = ParallelSpec(left=attention(need(m, "left", mw), mw + "left.", sink=True, value_is_key=False),
                                    right=MatrixMemorySpec(heads=int(need(r, "heads", rw)), dim=int(need(r, "dim", rw)),
                                                           vdim=int(need(r, "vdim", rw)), gate_cap=float(need(r, "gate_cap", rw))))
            elif kind == "channel_delta":
                spec = DeltaSpec(heads=int(need(m, "heads", mw)), kv_heads=int(need(m, "kv_heads", mw)), dim=int(need(m, "dim", mw)),
                                 vdim=int(need(m, "vdim", mw)), taps=int(need(m, "conv", mw)),
                                 decay_rank=int(m["decay_rank"]) if m.get("decay_rank") is not None else None,
                                 gate_rank=int(m["gate_rank"]) if m.get("gate_rank") is not None else None)
            else:
                raise ConfigError(f"config.json: {where}type {kind!r} is not a mixer of this design")
            mlp = L.get("mlp")
            if mlp is not None:
                pw = where + "mlp."
                mk = mlp.get("kind", "moe")
                if mk != "moe":
                    raise ConfigError(f"config.json: {pw}kind {mk!r} is not a feed-forward of this design")
                router = need(mlp, "router", pw)
                mlp = RoutedMlpSpec(expert=unit(need(mlp, "expert", pw), pw + "expert."),
                                    experts=int(need(router, "experts", pw + "router.")),
                                    identity=int(router.get("identity") or 0), top=int(need(router, "top", pw + "router.")),
                                    scale=float(router.get("scale", 1.0)),
                                    shared=unit(mlp["shared"], pw + "shared.") if mlp.get("shared") is not None else None)
            j = L.get("weights_of")
            layers.append(LayerSpec(kind, spec, mlp, int(j) if j is not None else None))
        return PereraxConfig(
            architecture=str(d.get("architecture") or (d.get("architectures") or ["Pererax"])[0]),
            n_vocab=int(need(d, "vocab")), n_embd=int(need(d, "width")), norm_eps=float(need(need(d, "norm"), "eps", "norm.")),
            layers=tuple(layers), n_ctx_train=int(d.get("max_positions", 8192)), stored_dtype=str(d.get("torch_dtype", "bfloat16")),
            extra={})
