"""Tefavik, as a description made of the library's parts.

A pre-norm decoder, x += mixer(norm_1(x)); x += ff(norm_2(x)) (a layer may have no ff), whose classifier is its embedding
table, with per layer one of two mixers:

  gla        gated linear attention: a matrix state per head that decays per key channel by sigmoid(z)^(1/tau), z from a
             low-rank pair of matrices; each head's output normed on its own, an output gate silu(W_g h)
  parallel   two mixers on the same input, each result normed over the model's width, half their sum:
             left:  grouped-query softmax attention with biases on q, k, v, an RMS norm of every q and k head, a rotation of
                    neighbouring pairs, capped scores, a softmax whose denominator holds one more 1, and a mask of chunks
                    (a query sees the keys of its own chunk of positions only)
             right: the matrix memory of xLSTM with capped gates and a running maximum

The feed-forward sends each token to `top` of its experts by a table indexed with the token's id; an expert is a gated
feed-forward with a clamped gate.  A stretch of layers may run several times in a row: every pass has cache and state of its
own, and every pass but the first starts from the stream plus the embedding's output.

Tensor names: embed, final.norm, and per layer i: l<i>.norm1 / norm2, l<i>.mix.<name> (l<i>.mix.left.<name>, l<i>.mix.right.<name>,
l<i>.mix.left.out, l<i>.mix.right.out in a parallel layer; a bias is its matrix's name + ".b"), l<i>.mlp.e<j>.gate / up / down,
l<i>.mlp.table.
"""

from __future__ import annotations

from ..config.tefavik import (
    ARCHITECTURE, EXPERT_GATE_ALPHA, MAX_POSITIONS, MEMORY_DEN_EPS, GlaMixerConfig, ParallelMixerConfig, TefavikConfig,
)
from ..registry import Architecture, register_architecture
from ..spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "q_norm": "q.norm", "k_norm": "k.norm"}


def describe_tefavik(cfg: TefavikConfig) -> ModelSpec:
    def norm(prefix: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.eps, "name": "", "float32": True}, prefix)

    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if isinstance(m, GlaMixerConfig):
            mixer = PartSpec(
                "gated_linear_attention",
                {"hidden_size": cfg.width, "num_heads": m.heads, "dim": m.dim, "vdim": m.vdim, "tau": m.tau, "eps": cfg.eps,
                 "decay_rank": 0},  # the inner size of the decay's pair of matrices is the checkpoint's to say
                p + "mix.",
            )
        elif isinstance(m, ParallelMixerConfig):
            a = m.left
            position = PartSpec("rotary", {"rotary_dim": a.rot_dims, "theta": a.rot_base, "scaling": None, "interleaved": True}) \
                if a.rot_dims else PartSpec("none")
            left = PartSpec(
                "attention",
                {"hidden_size": cfg.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "value_dim": a.vdim,
                 "scale": a.scale, "window": 0, "chunk": a.chunk, "softcap": a.softcap, "sink": "zero", "bias": "qkv", "qk_norm": cfg.eps,
                 "position": position, "names": _ATTENTION_NAMES},
                "left.",
            )
            r = m.right
            right = PartSpec(
                "mlstm",
                {"hidden_size": cfg.width, "num_heads": r.heads, "dim": r.dim, "vdim": r.vdim, "gate_cap": r.gate_cap, "eps": cfg.eps,
                 "den_eps": MEMORY_DEN_EPS},
                "right.",
            )
            mixer = PartSpec(
                "parallel",
                {"branches": ((left, 0.5), (right, 0.5)), "branch_norms": {"names": ("left.out", "right.out"), "eps": cfg.eps, "size": cfg.width}},
                p + "mix.",
            )
        else:
            raise TypeError(f"layer {i}: {type(m).__name__} is not a mixer configuration of this architecture")
        norms = {"mixer": norm(p + "norm1")}
        ff = None
        if layer.mlp is not None:
            e = layer.mlp
            ff = PartSpec(
                "routed_experts",
                {"hidden_size": cfg.width, "n_experts": e.experts, "top": e.top, "expert_ff": e.ff, "router": "table", "vocab_size": cfg.vocab,
                 "activation": "clamped_swish", "alpha": EXPERT_GATE_ALPHA, "limit": e.limit},
                p + "mlp.",
            )
            norms["feed_forward"] = norm(p + "norm2")
        layers.append(LayerSpec(block="prenorm", mixer=mixer, feed_forward=ff, norms=norms))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": ""}, "embed"),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, add_input=add) for i, add in cfg.runs()),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied_to": "embed", "name": ""}, "head"),
        stored_dtype="bfloat16",
    )


register_architecture(Architecture(ARCHITECTURE, TefavikConfig.from_json, describe_tefavik), replace=True)
