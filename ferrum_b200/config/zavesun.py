"""Typed configuration of the Zavesun decoder.

Its config.json is nested: `architecture`, `vocab`, `width`, `norm.eps`, `streams` (how many copies
of the residual stream the layers carry; absent: one), `logit_softcap` (absent or 0: none) and
`layers`, a list whose entries give the layer's `type` (which mixer), the mixer's sizes under
`mixer` and its feed-forward under `mlp` (null: none).  Every size and every constant that can
differ between two models of the design is read here and nowhere else; what an entry does not
mention does not exist (no `mask`: every earlier key; no `q_temp`: no temperature; no `rot`: no
rotation; no `rot.scaling`: unscaled frequencies; no `v_mix`: the layer's own values).

Mixers:
  `attention`    heads, kv_heads, dim, vdim, scale, mask.size (a query sees itself and the
                 mask.size - 1 keys before it), q_temp.{coef, every}; no biases, no rotation; a
                 distance bias with a fixed slope per head.
  `attention_2`  heads, kv_heads, dim, vdim, scale, mask.size (the length of the chunks that
                 positions are cut into from 0), rot.{base, dims, scaling.factor}; biased
                 projections, weighted RMS norm of query and key heads, interleaved rotation.
  Both: `v_mix` (the layer's values are blended with those of the first layer that says so).

Feed-forwards (`mlp.kind`):
  `dense`        ff; gelu (tanh form) on the gate.
  `moe`          expert.ff, router.{experts, top}; silu on the gate; sigmoid scores as weights,
                 applied to the expert's input.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Tuple, Union

from ..errors import ConfigError
from .llama import RopeScaling


@dataclass(frozen=True)
class AttentionSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int = 0                         # 0: every earlier key
    mask: str = "window"                    # "window" or "chunk": what `window` counts
    q_temp: Optional[Tuple[float, int]] = None      # (coef, every)
    linear_bias: bool = False               # the fixed per-head distance slopes
    qkv_bias: bool = False
    qk_norm: bool = False
    rot_base: float = 0.0
    rot_dims: int = 0                       # 0: no rotation
    rot_scaling: Optional[RopeScaling] = None
    v_mix: bool = False

    def slopes(self):
        """2^(-8 (h + 1) / heads) for head h: the distance bias's slopes."""
        return [2.0 ** (-8.0 * (h + 1) / self.heads) for h in range(self.heads)]


@dataclass(frozen=True)
class DenseMlpSpec:
    ff: int
    kind: str = "dense"


@dataclass(frozen=True)
class RoutedMlpSpec:
    ff: int
    experts: int
    top: int
    kind: str = "moe"


@dataclass(frozen=True)
class LayerSpec:
    type: str
    mixer: AttentionSpec
    mlp: Optional[Union[DenseMlpSpec, RoutedMlpSpec]]


@dataclass(frozen=True)
class ZavesunConfig:
    architecture: str
    n_vocab: int
    n_embd: int
    norm_eps: float
    streams: int
    logit_softcap: float                    # 0: none
    layers: Tuple[LayerSpec, ...]
    n_ctx_train: int = 8192                 # positions the rotary tables cover unless the caller asks for more or fewer
    eos_token_ids: Tuple[int, ...] = ()
    stored_dtype: str = "bfloat16"
    extra: dict = field(default_factory=dict, compare=False)

    @property
    def n_layer(self):
        return len(self.layers)

    def first_value_mix(self):
        """Index of the first layer that mixes values (the one whose values the others blend in), or None."""
        return next((i for i, layer in enumerate(self.layers) if layer.mixer.v_mix), None)

    def __post_init__(self):
        for k in ("n_vocab", "n_embd", "streams"):
            v = getattr(self, k)
            if not isinstance(v, int) or v <= 0:
                raise ConfigError(f"zavesun: {k} must be a positive integer, found {v!r}")
        if not (math.isfinite(self.norm_eps) and self.norm_eps > 0.0):
            raise ConfigError("zavesun: invalid norm.eps")
        if not (math.isfinite(self.logit_softcap) and self.logit_softcap >= 0.0):
            raise ConfigError("zavesun: invalid logit_softcap")
        if not self.layers:
            raise ConfigError("zavesun: no layers")
        first = self.first_value_mix()
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            for k in ("heads", "kv_heads", "dim", "vdim"):
                if getattr(m, k) <= 0:
                    raise ConfigError(f"zavesun: layer {i}: {k} must be positive")
            if m.heads % m.kv_heads:
                raise ConfigError(f"zavesun: layer {i}: kv_heads does not divide heads")
            if not math.isfinite(m.scale):
                raise ConfigError(f"zavesun: layer {i}: invalid scale")
            if m.window < 0:
                raise ConfigError(f"zavesun: layer {i}: mask.size must be positive")
            if m.rot_dims % 2 or m.rot_dims > m.dim or m.rot_dims < 0:
                raise ConfigError(f"zavesun: layer {i}: rot.dims must be even and at most dim")
            if m.rot_dims and not (math.isfinite(m.rot_base) and m.rot_base > 0):
                raise ConfigError(f"zavesun: layer {i}: invalid rot.base")
            if m.rot_scaling is not None and not (math.isfinite(m.rot_scaling.factor) and m.rot_scaling.factor > 0):
                raise ConfigError(f"zavesun: layer {i}: invalid rot.scaling.factor")
            if m.q_temp is not None and m.q_temp[1] <= 0:
                raise ConfigError(f"zavesun: layer {i}: q_temp.every must be positive")
            if m.v_mix:
                f = self.layers[first].mixer
                if m.kv_heads * m.vdim != f.kv_heads * f.vdim:
                    raise ConfigError(f"zavesun: layer {i}: mixed values need kv_heads * vdim = {f.kv_heads * f.vdim} as in layer {first}")
            p = layer.mlp
            if p is not None:
                if p.ff <= 0:
                    raise ConfigError(f"zavesun: layer {i}: ff must be positive")
                if isinstance(p, RoutedMlpSpec) and not (0 < p.top <= p.experts):
                    raise ConfigError(f"zavesun: layer {i}: {p.top} of {p.experts} experts per token")

    @staticmethod
    def from_dict(d: dict) -> "ZavesunConfig":
        def need(obj, key, where=""):
            if not isinstance(obj, dict) or key not in obj or obj[key] is None:
                raise ConfigError(f"config.json: missing required key {where}{key!r}")
            return obj[key]

        layers = []
        for i, L in enumerate(need(d, "layers")):
            where = f"layers[{i}]."
            kind = need(L, "type", where)
            if kind not in ("attention", "attention_2"):
                raise ConfigError(f"config.json: {where}type {kind!r} is not a mixer of this design")
            m = need(L, "mixer", where)
            mw = where + "mixer."
            second = kind == "attention_2"
            window = 0
            if m.get("mask") is not None:
                window = int(need(m["mask"], "size", mw + "mask."))
                if window <= 0:
                    raise ConfigError(f"config.json: {mw}mask.size must be positive")
            q_temp = None
            if not second and m.get("q_temp") is not None:
                q_temp = (float(need(m["q_temp"], "coef", mw + "q_temp.")), int(need(m["q_temp"], "every", mw + "q_temp.")))
            rot_base, rot_dims, scaling = 0.0, 0, None
            if second:
                rot = need(m, "rot", mw)
                rot_base, rot_dims = float(need(rot, "base", mw + "rot.")), int(need(rot, "dims", mw + "rot."))
                if rot.get("scaling"):
                    scaling = RopeScaling("linear", float(need(rot["scaling"], "factor", mw + "rot.scaling.")), 1.0, 1.0, 0)
            spec = AttentionSpec(
                heads=int(need(m, "heads", mw)), kv_heads=int(need(m, "kv_heads", mw)), dim=int(need(m, "dim", mw)),
                vdim=int(need(m, "vdim", mw)), scale=float(need(m, "scale", mw)), window=window,
                mask="chunk" if second else "window", q_temp=q_temp, linear_bias=not second, qkv_bias=second, qk_norm=second,
                rot_base=rot_base, rot_dims=rot_dims, rot_scaling=scaling, v_mix=bool(m.get("v_mix", False)))
            mlp = L.get("mlp")
            if mlp is not None:
                pw = where + "mlp."
                mk = need(mlp, "kind", pw)
                if mk == "dense":
                    mlp = DenseMlpSpec(ff=int(need(mlp, "ff", pw)))
                elif mk == "moe":
                    router = need(mlp, "router", pw)
                    mlp = RoutedMlpSpec(ff=int(need(need(mlp, "expert", pw), "ff", pw + "expert.")),
                                        experts=int(need(router, "experts", pw + "router.")), top=int(need(router, "top", pw + "router.")))
                else:
                    raise ConfigError(f"config.json: {pw}kind {mk!r} is not a feed-forward of this design")
            layers.append(LayerSpec(kind, spec, mlp))
        return ZavesunConfig(
            architecture=str(d.get("architecture") or (d.get("architectures") or ["Zavesun"])[0]),
            n_vocab=int(need(d, "vocab")), n_embd=int(need(d, "width")), norm_eps=float(need(need(d, "norm"), "eps", "norm.")),
            streams=int(d.get("streams") or 1), logit_softcap=float(d.get("logit_softcap") or 0.0), layers=tuple(layers),
            n_ctx_train=int(d.get("max_positions", 8192)), stored_dtype=str(d.get("torch_dtype", "bfloat16")), extra={})
