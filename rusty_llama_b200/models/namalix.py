"""Namalix, as a description made of the library's parts.

A decoder whose layer has ONE norm that both of its sublayers read, x += mixer(h) + ff(h) with h = norm(x); every norm an RMS
norm whose weight is stored as its distance from one; the embedding's rows times a constant.  Per layer one of three mixers:

  attention  grouped-query attention without a softmax: rotation of neighbouring pairs over part of a head with YaRN-scaled
             frequencies, capped scores, a weight logistic(score + bias_h) per visible key, the heads' weights mixed by a learned
             matrix, values blended with those of the first such layer, one output gate number per head
  retention  linear attention with a constant decay per head on q and k turned by their positions (halves paired), k times
             dim^-1/2, every head's result divided by its root mean square, an output gate silu(W_g h)
  delta      the gated delta rule behind short causal convolutions of q, k and v

and a dense gated feed-forward (tanh-form gelu) or experts with a clamped gate, chosen by logistic scores plus a correction that
only chooses, the chosen scores divided by their sum and multiplied by a constant.

Tensor names: embed, head, final.norm, and per layer i: l<i>.norm1, l<i>.mix.<name>, l<i>.mlp.gate / up / down or
l<i>.mlp.e<j>.gate / up / down, l<i>.mlp.router, l<i>.mlp.correction.
"""

from __future__ import annotations

from ..config.namalix import (
    ARCHITECTURE, DELTA_UNIT_EPS, EXPERT_GATE_ALPHA, MAX_POSITIONS, ROUTER_SUM_EPS, AttentionMixerConfig, DeltaMixerConfig, DenseConfig,
    NamalixConfig, RetentionMixerConfig, RotationConfig,
)
from ..config.rope_scaling import RopeScaling
from ..registry import Architecture, register_architecture
from ..spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "head_mix": "talk", "head_bias": "pb", "value_mix": "vmix"}
_VALUE_MIX_KEY = "first_values"


def _rotary(rot: RotationConfig, interleaved: bool) -> PartSpec:
    if not rot.dims:
        return PartSpec("none")
    scaling = RopeScaling()
    if rot.scaling is not None:
        factor, original, fast, slow = rot.scaling
        scaling = RopeScaling(kind="yarn", factor=factor, original_max_position_embeddings=original, beta_fast=fast, beta_slow=slow)
    return PartSpec("rotary", {"rotary_dim": rot.dims, "theta": rot.base, "scaling": scaling, "interleaved": interleaved})


def describe_namalix(cfg: NamalixConfig) -> ModelSpec:
    def norm(prefix: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.eps, "name": "", "offset": 1.0}, prefix)

    layers = []
    seen_value_source = False
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if isinstance(m, AttentionMixerConfig):
            value_mix = None
            if m.v_mix:
                value_mix = {"key": _VALUE_MIX_KEY, "role": "mix" if seen_value_source else "source"}
                seen_value_source = True
            mixer = PartSpec(
                "attention",
                {"hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                 "scale": m.scale, "window": 0, "softcap": m.softcap, "weights": "logistic", "head_bias": True, "head_mix": True,
                 "gate": "head", "value_mix": value_mix, "position": _rotary(m.rot, True), "names": _ATTENTION_NAMES},
                p + "mix.",
            )
        elif isinstance(m, RetentionMixerConfig):
            mixer = PartSpec(
                "decay_linear_attention",
                {"hidden_size": cfg.width, "num_heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": m.decay, "eps": cfg.eps,
                 "activation": "none", "gate": True, "gate_act": "silu", "head_norm": True, "norm_weight": False, "k_scale": m.dim ** -0.5,
                 "position": _rotary(m.rot, False)},
                p + "mix.",
            )
        elif isinstance(m, DeltaMixerConfig):
            mixer = PartSpec(
                "gated_delta",
                {"hidden_size": cfg.width, "num_heads": m.heads, "num_qk_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "taps": m.conv,
                 "eps": cfg.eps, "unit_eps": DELTA_UNIT_EPS},
                p + "mix.",
            )
        else:
            raise TypeError(f"layer {i}: {type(m).__name__} is not a mixer configuration of this architecture")
        ff = None
        if isinstance(layer.mlp, DenseConfig):
            ff = PartSpec(
                "gated_mlp",
                {"hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "activation": "gelu_tanh", "names": {"gate": "gate", "up": "up", "down": "down"}},
                p + "mlp.",
            )
        elif layer.mlp is not None:
            e = layer.mlp
            ff = PartSpec(
                "routed_experts",
                {"hidden_size": cfg.width, "n_experts": e.experts, "top": e.top, "expert_ff": e.ff, "router": "sigmoid", "bias": True,
                 "renormalize": True, "renorm_eps": ROUTER_SUM_EPS, "weight_scale": e.scale, "activation": "clamped_swish",
                 "alpha": EXPERT_GATE_ALPHA, "limit": e.limit},
                p + "mlp.",
            )
        layers.append(LayerSpec(block="shared_norm", mixer=mixer, feed_forward=ff, norms={"mixer": norm(p + "norm1")}))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "", "scale": cfg.embedding_scale}, "embed"),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": None, "name": ""}, "head"),
        stored_dtype="bfloat16",
        # (a checkpoint may carry the mixing factor also in attention layers that mix no values)
        redundant_tensors=("l*.mix." + _ATTENTION_NAMES["value_mix"],),
    )


register_architecture(Architecture(ARCHITECTURE, NamalixConfig.from_json, describe_namalix), replace=True)
