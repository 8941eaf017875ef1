"""Typed configuration of the Tefavik architecture, read from config.json.

The file lists its layers one by one; every layer names which mixer it has (`type`), the mixer's sizes and constants and
its feed-forward, so two models of the architecture may differ in everything, the order of layer kinds included.  A stretch
of layers may run several times in a row (`loop`).  Keys:

    architecture: "Tefavik", vocab, width, norm: {eps},
    layers: [ {type: "gla",      mixer: {heads, dim, vdim, tau}, mlp}
            | {type: "parallel", mixer: {left: <chunked attention>, right: {heads, dim, vdim, gate_cap}}, mlp} ... ]
    <chunked attention>: {heads, kv_heads, dim, vdim, scale, softcap, mask: {size}, rot: {base, dims}}
    mlp: null | {kind: "moe", router: {experts, top}, expert: {ff, limit}}
    loop: null | {start, stop, times}: layers start .. stop - 1 run `times` times in a row

Sizes that the file does not name (the inner size of the decay's low-rank pair) are read from the tensors' shapes by the
loader; what else a mixer has (biases, norms of q and k, a sink, gates) belongs to its layer type and is fixed by the design.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from ..errors import ConfigError
from .vezatar import _get, _int, _num

ARCHITECTURE = "Tefavik"

# Constants the design fixes
EXPERT_GATE_ALPHA = 1.702  # an expert's gate is g * logistic(1.702 g)
MEMORY_DEN_EPS = 1e-6  # added to the matrix memory's normaliser
MAX_POSITIONS = 1 << 20  # the design names no limit; the library's bookkeeping wants one


@dataclass(frozen=True)
class GlaMixerConfig:
    heads: int
    dim: int
    vdim: int
    tau: float


@dataclass(frozen=True)
class ChunkedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float
    chunk: int
    rot_base: float
    rot_dims: int


@dataclass(frozen=True)
class MemoryMixerConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: ChunkedAttentionConfig
    right: MemoryMixerConfig


@dataclass(frozen=True)
class TableExpertsConfig:
    experts: int
    top: int
    ff: int
    limit: float


@dataclass(frozen=True)
class TefavikLayerConfig:
    type: str
    mixer: Union[GlaMixerConfig, ParallelMixerConfig]
    mlp: Optional[TableExpertsConfig]


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class TefavikConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[TefavikLayerConfig, ...]
    loop: Optional[LoopConfig]
    architecture: str = ARCHITECTURE

    @classmethod
    def from_json(cls, d: Mapping[str, Any]) -> "TefavikConfig":
        layers = _get(d, "layers", "config.json")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        parsed = tuple(_layer(i, layer) for i, layer in enumerate(layers))
        loop = d.get("loop")
        if loop is not None:
            loop = LoopConfig(start=_int(loop, "start", "loop", 0), stop=_int(loop, "stop", "loop", 0), times=_int(loop, "times", "loop", 1))
            if not loop.start < loop.stop <= len(parsed):
                raise ConfigError(f"loop: layers {loop.start} .. {loop.stop - 1} are not a stretch of the {len(parsed)} layers")
        return cls(
            vocab=_int(d, "vocab", "config.json"),
            width=_int(d, "width", "config.json"),
            eps=_num(_get(d, "norm", "config.json"), "eps", "norm"),
            layers=parsed,
            loop=loop,
        )

    def runs(self):
        """[(layer, whether the embedding's output is added before it)] in the order in which the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        lp = self.loop
        order = [(i, False) for i in range(lp.start)]
        for r in range(lp.times):
            order += [(i, r > 0 and i == lp.start) for i in range(lp.start, lp.stop)]
        return order + [(i, False) for i in range(lp.stop, n)]


def _chunked_attention(m, where: str) -> ChunkedAttentionConfig:
    heads, kv_heads = _int(m, "heads", where), _int(m, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"{where}: {heads} heads are not a multiple of {kv_heads} kv_heads")
    dim = _int(m, "dim", where)
    rot = m.get("rot") if isinstance(m, Mapping) else None
    base, dims = 10000.0, 0
    if rot is not None:
        dims = _int(rot, "dims", where + ".rot", 0)
        base = _num(rot, "base", where + ".rot")
    if dims > dim or dims % 2:
        raise ConfigError(f"{where}.rot.dims = {dims} must be even and at most dim = {dim}")
    return ChunkedAttentionConfig(
        heads=heads, kv_heads=kv_heads, dim=dim, vdim=_int(m, "vdim", where), scale=_num(m, "scale", where),
        softcap=_num(m, "softcap", where), chunk=_int(_get(m, "mask", where), "size", where + ".mask"), rot_base=base, rot_dims=dims,
    )


def _layer(i: int, d: Mapping[str, Any]) -> TefavikLayerConfig:
    where = f"layers[{i}]"
    kind = _get(d, "type", where)
    m = _get(d, "mixer", where)
    w = where + ".mixer"
    if kind == "gla":
        mixer = GlaMixerConfig(heads=_int(m, "heads", w), dim=_int(m, "dim", w), vdim=_int(m, "vdim", w), tau=_num(m, "tau", w))
    elif kind == "parallel":
        r = _get(m, "right", w)
        mixer = ParallelMixerConfig(
            left=_chunked_attention(_get(m, "left", w), w + ".left"),
            right=MemoryMixerConfig(heads=_int(r, "heads", w + ".right"), dim=_int(r, "dim", w + ".right"), vdim=_int(r, "vdim", w + ".right"),
                                    gate_cap=_num(r, "gate_cap", w + ".right")),
        )
    else:
        raise ConfigError(f"{where}.type '{kind}' is not a mixer of this architecture (known: gla, parallel)")
    mlp = d.get("mlp")
    if mlp is None:
        parsed = None
    else:
        mk = _get(mlp, "kind", where + ".mlp")
        if mk != "moe":
            raise ConfigError(f"{where}.mlp.kind '{mk}' is not a feed-forward of this architecture (known: moe)")
        router, expert = _get(mlp, "router", where + ".mlp"), _get(mlp, "expert", where + ".mlp")
        parsed = TableExpertsConfig(
            experts=_int(router, "experts", where + ".mlp.router"), top=_int(router, "top", where + ".mlp.router"),
            ff=_int(expert, "ff", where + ".mlp.expert"), limit=_num(expert, "limit", where + ".mlp.expert"),
        )
        if parsed.top > parsed.experts:
            raise ConfigError(f"{where}.mlp.router: {parsed.top} of {parsed.experts} experts per token")
    return TefavikLayerConfig(kind, mixer, parsed)
