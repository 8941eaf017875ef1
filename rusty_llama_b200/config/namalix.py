"""Typed configuration of the Namalix architecture, read from config.json.

The file lists its layers one by one; every layer names which mixer it has (`type`), the mixer's sizes and constants and
its feed-forward, so two models of the architecture may differ in everything, the order of layer kinds included.  Keys:

    architecture: "Namalix", vocab, width, norm: {eps}, embedding: {scale},
    layers: [ {type: "attention", mixer: {heads, kv_heads, dim, vdim, scale, softcap, v_mix, rot: {base, dims, scaling}}, mlp}
            | {type: "retention", mixer: {heads, dim, vdim, decay: [one per head], rot: {base, dims}}, mlp}
            | {type: "delta",     mixer: {heads, kv_heads, dim, vdim, conv}, mlp} ... ]
    rot.scaling: null | {factor, original, fast, slow}
    mlp: null | {kind: "dense", ff} | {kind: "moe", router: {experts, top, scale}, expert: {ff, limit}}

What else a mixer has (a bias per head, the matrix that mixes the heads' weights, gates, norms of the heads) belongs to its
layer type and is fixed by the design.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from ..errors import ConfigError
from .vezatar import _get, _int, _num

ARCHITECTURE = "Namalix"

# Constants the design fixes
EXPERT_GATE_ALPHA = 1.702  # an expert's gate is g * logistic(1.702 g)
DELTA_UNIT_EPS = 1e-6  # under the root that makes the delta rule's q and k unit vectors
ROUTER_SUM_EPS = 1e-20  # joins the sum that the chosen experts' scores are divided by
MAX_POSITIONS = 1 << 20  # the design names no limit; the library's bookkeeping wants one


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]]  # (factor, original, fast, slow)


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float
    v_mix: bool
    rot: RotationConfig


@dataclass(frozen=True)
class RetentionMixerConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot: RotationConfig


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class DenseConfig:
    ff: int


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int
    top: int
    scale: float
    ff: int
    limit: float


@dataclass(frozen=True)
class NamalixLayerConfig:
    type: str
    mixer: Union[AttentionMixerConfig, RetentionMixerConfig, DeltaMixerConfig]
    mlp: Union[None, DenseConfig, ExpertsConfig]


@dataclass(frozen=True)
class NamalixConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: Tuple[NamalixLayerConfig, ...]
    architecture: str = ARCHITECTURE

    @classmethod
    def from_json(cls, d: Mapping[str, Any]) -> "NamalixConfig":
        layers = _get(d, "layers", "config.json")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        parsed = tuple(_layer(i, layer) for i, layer in enumerate(layers))
        mixed = [layer.mixer for layer in parsed if isinstance(layer.mixer, AttentionMixerConfig) and layer.mixer.v_mix]
        for m in mixed[1:]:
            if (m.kv_heads, m.vdim) != (mixed[0].kv_heads, mixed[0].vdim):
                raise ConfigError(f"layers with v_mix must agree in kv_heads and vdim: {m.kv_heads} x {m.vdim} against "
                                  f"{mixed[0].kv_heads} x {mixed[0].vdim} of the first")
        emb = d.get("embedding")
        return cls(
            vocab=_int(d, "vocab", "config.json"),
            width=_int(d, "width", "config.json"),
            eps=_num(_get(d, "norm", "config.json"), "eps", "norm"),
            embedding_scale=1.0 if emb is None else _num(emb, "scale", "embedding"),
            layers=parsed,
        )


def _rotation(m, where: str, dim: int) -> RotationConfig:
    rot = m.get("rot") if isinstance(m, Mapping) else None
    if rot is None:
        return RotationConfig(10000.0, 0, None)
    dims = _int(rot, "dims", where + ".rot", 0)
    if dims > dim or dims % 2:
        raise ConfigError(f"{where}.rot.dims = {dims} must be even and at most dim = {dim}")
    scaling = rot.get("scaling")
    if scaling is not None:
        w = where + ".rot.scaling"
        scaling = (_num(scaling, "factor", w), _num(scaling, "original", w), _num(scaling, "fast", w), _num(scaling, "slow", w))
        if not (scaling[0] > 0 and scaling[1] > 0 and scaling[2] > 0 and scaling[3] > 0):
            raise ConfigError(f"{w}: factor, original, fast and slow must be positive")
    return RotationConfig(_num(rot, "base", where + ".rot"), dims, scaling)


def _mlp(mlp, where: str):
    if mlp is None:
        return None
    kind = _get(mlp, "kind", where)
    if kind == "dense":
        return DenseConfig(ff=_int(mlp, "ff", where))
    if kind == "moe":
        router, expert = _get(mlp, "router", where), _get(mlp, "expert", where)
        parsed = ExpertsConfig(
            experts=_int(router, "experts", where + ".router"), top=_int(router, "top", where + ".router"),
            scale=_num(router, "scale", where + ".router") if "scale" in router else 1.0,
            ff=_int(expert, "ff", where + ".expert"), limit=_num(expert, "limit", where + ".expert"),
        )
        if parsed.top > parsed.experts:
            raise ConfigError(f"{where}.router: {parsed.top} of {parsed.experts} experts per token")
        return parsed
    raise ConfigError(f"{where}.kind '{kind}' is not a feed-forward of this architecture (known: dense, moe)")


def _layer(i: int, d: Mapping[str, Any]) -> NamalixLayerConfig:
    where = f"layers[{i}]"
    kind = _get(d, "type", where)
    m = _get(d, "mixer", where)
    w = where + ".mixer"
    if kind == "attention":
        heads, kv_heads, dim = _int(m, "heads", w), _int(m, "kv_heads", w), _int(m, "dim", w)
        if heads % kv_heads:
            raise ConfigError(f"{w}: {heads} heads are not a multiple of {kv_heads} kv_heads")
        mixer = AttentionMixerConfig(
            heads=heads, kv_heads=kv_heads, dim=dim, vdim=_int(m, "vdim", w), scale=_num(m, "scale", w),
            softcap=_num(m, "softcap", w, positive=False) if m.get("softcap") is not None else 0.0, v_mix=bool(m.get("v_mix", False)), rot=_rotation(m, w, dim),
        )
        if mixer.softcap < 0:
            raise ConfigError(f"{w}.softcap = {mixer.softcap} must not be negative (0: no cap)")
    elif kind == "retention":
        heads, dim = _int(m, "heads", w), _int(m, "dim", w)
        decay = _get(m, "decay", w)
        if not isinstance(decay, (list, tuple)) or len(decay) != heads:
            raise ConfigError(f"{w}.decay must list one number per head ({heads})")
        rot = _rotation(m, w, dim)
        if rot.scaling is not None:
            raise ConfigError(f"{w}.rot: a retention layer's rotation has no scaling")
        mixer = RetentionMixerConfig(heads=heads, dim=dim, vdim=_int(m, "vdim", w), decay=tuple(float(x) for x in decay), rot=rot)
    elif kind == "delta":
        heads, kv_heads = _int(m, "heads", w), _int(m, "kv_heads", w)
        if heads % kv_heads:
            raise ConfigError(f"{w}: {heads} heads are not a multiple of {kv_heads} kv_heads")
        mixer = DeltaMixerConfig(heads=heads, kv_heads=kv_heads, dim=_int(m, "dim", w), vdim=_int(m, "vdim", w), conv=_int(m, "conv", w))
    else:
        raise ConfigError(f"{where}.type '{kind}' is not a mixer of this architecture (known: attention, retention, delta)")
    return NamalixLayerConfig(kind, mixer, _mlp(d.get("mlp"), where + ".mlp"))
