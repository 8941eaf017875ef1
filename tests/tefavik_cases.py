"""Small Tefavik configurations and random weights for the tests, made without the library.

Weights are drawn so that every mechanism matters (activations of order one, decays that range from quick forgetting to
almost none, gates on both sides of their caps, norm weights away from one, experts whose clamps bite), rounded to bfloat16
and written with the third-party safetensors package."""

import json
import os

import numpy as np
import torch

DECAY_RANK = {"a": 5, "b": 3, "c": 8}  # the inner size of the decay's pair of matrices: the checkpoint's to say


def _attn(heads, kv_heads, dim, vdim, rot_dims, base, scale, softcap, chunk):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"base": base, "dims": rot_dims}, "scale": scale,
            "softcap": softcap, "mask": {"size": chunk}}


def _memory(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def _gla(heads, dim, vdim, tau):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def _moe(experts, top, ff, limit):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}


def config_a():
    """Four layers that differ in everything, the middle two run three times: unequal key and value sizes that are no multiples
    of 8, 6 heads on 2 and 4 on 4, a rotation of part of a head, chunks of 7 and of exactly one page, two of five experts and
    all of three, a layer without feed-forward, states of 24 x 40 and 8 x 72 (neither a multiple of the kernels' 32)."""
    return {
        "architecture": "Tefavik", "vocab": 131, "width": 96, "norm": {"eps": 1e-5},
        "layers": [
            {"type": "parallel", "mixer": {"left": _attn(6, 2, 20, 12, 8, 10000.0, 0.3, 5.0, 7), "right": _memory(3, 24, 40, 8.0)}, "mlp": _moe(5, 2, 24, 1.0)},
            {"type": "gla", "mixer": _gla(3, 24, 40, 4.0), "mlp": None},
            {"type": "gla", "mixer": _gla(1, 40, 8, 1.0), "mlp": _moe(3, 3, 16, 2.5)},
            {"type": "parallel", "mixer": {"left": _attn(4, 4, 16, 24, 16, 1000.0, 0.25, 30.0, 64), "right": _memory(1, 8, 72, 15.0)}, "mlp": _moe(4, 1, 40, 7.0)},
        ],
        "loop": {"start": 1, "stop": 3, "times": 3},
    }


def config_b():
    """A width that no 16-byte-row kernel takes (68), no loop, chunks of one (a query sees itself and the sink only) and of 130
    (two pages and a bit), no rotation at all in one mixer, a memory of one head with keys of 3 numbers, one expert."""
    return {
        "architecture": "Tefavik", "vocab": 77, "width": 68, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "gla", "mixer": _gla(2, 12, 20, 16.0), "mlp": _moe(1, 1, 30, 1.5)},
            {"type": "parallel", "mixer": {"left": _attn(1, 1, 24, 16, 0, 100.0, 0.4, 2.0, 1), "right": _memory(1, 3, 10, 12.0)}, "mlp": None},
            {"type": "parallel", "mixer": {"left": _attn(3, 1, 12, 36, 4, 500000.0, 0.5, 50.0, 130), "right": _memory(2, 36, 20, 3.0)}, "mlp": _moe(6, 3, 12, 0.7)},
        ],
        "loop": None,
    }


def config_c():
    """Sizes in multiples of 8 and 64 (the shapes the tensor-core kernels take), every layer run twice, a chunk of 65."""
    return {
        "architecture": "Tefavik", "vocab": 160, "width": 128, "norm": {"eps": 1e-6},
        "layers": [
            {"type": "parallel", "mixer": {"left": _attn(4, 2, 64, 64, 32, 10000.0, 0.125, 20.0, 65), "right": _memory(2, 32, 64, 10.0)}, "mlp": _moe(8, 2, 64, 1.5)},
            {"type": "gla", "mixer": _gla(2, 64, 64, 8.0), "mlp": _moe(4, 1, 128, 3.0)},
        ],
        "loop": {"start": 0, "stop": 2, "times": 2},
    }


CONFIGS = {"a": config_a, "b": config_b, "c": config_c}


def tensor_shapes(cfg, rank):
    d, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, d), "final.norm": (d,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (d,)
        if layer["type"] == "gla":
            H = m["heads"]
            out[p + "mix.q"] = out[p + "mix.k"] = (H * m["dim"], d)
            out[p + "mix.v"] = out[p + "mix.g"] = (H * m["vdim"], d)
            out[p + "mix.o"] = (d, H * m["vdim"])
            out[p + "mix.norm"] = (m["vdim"],)
            out[p + "mix.a1"] = (rank, d)
            out[p + "mix.a2"] = (H * m["dim"], rank)
            out[p + "mix.a2.b"] = (H * m["dim"],)
        else:
            a, r = m["left"], m["right"]
            q = p + "mix.left."
            out[q + "q"], out[q + "q.b"] = (a["heads"] * a["dim"], d), (a["heads"] * a["dim"],)
            out[q + "k"], out[q + "k.b"] = (a["kv_heads"] * a["dim"], d), (a["kv_heads"] * a["dim"],)
            out[q + "v"], out[q + "v.b"] = (a["kv_heads"] * a["vdim"], d), (a["kv_heads"] * a["vdim"],)
            out[q + "q.norm"] = out[q + "k.norm"] = (a["dim"],)
            out[q + "o"] = (d, a["heads"] * a["vdim"])
            q = p + "mix.right."
            H = r["heads"]
            out[q + "q"] = out[q + "k"] = (H * r["dim"], d)
            out[q + "v"] = out[q + "g"] = (H * r["vdim"], d)
            out[q + "o"] = (d, H * r["vdim"])
            out[q + "norm"] = (H * r["vdim"],)
            out[q + "i"] = out[q + "f"] = (H, d)
            out[q + "i.b"] = out[q + "f.b"] = (H,)
            out[p + "mix.left.out"] = out[p + "mix.right.out"] = (d,)
        if layer["mlp"] is not None:
            out[p + "norm2"] = (d,)
            e = layer["mlp"]
            for j in range(e["router"]["experts"]):
                out[f"{p}mlp.e{j}.gate"] = out[f"{p}mlp.e{j}.up"] = (e["expert"]["ff"], d)
                out[f"{p}mlp.e{j}.down"] = (d, e["expert"]["ff"])
            out[p + "mlp.table"] = (V, e["router"]["top"])
    return out


def random_weights(cfg, seed, rank=4):
    """name -> torch tensor (bfloat16; tables int32)."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, rank).items():
        last = name.rsplit(".", 1)[-1]
        if last == "table":
            E = cfg["layers"][int(name[1:].split(".")[0])]["mlp"]["router"]["experts"]
            out[name] = torch.from_numpy(np.stack([rng.permutation(E)[: shape[1]] for _ in range(shape[0])]).astype(np.int32))
            continue
        if last in ("norm1", "norm2", "norm", "out") or name == "final.norm":
            t = 1.0 + 0.3 * rng.standard_normal(shape)
        elif name.endswith("a2.b"):
            t = 2.0 * rng.standard_normal(shape)  # decays from quick forgetting to almost none
        elif name.endswith("i.b") or name.endswith("f.b"):
            t = 2.0 * rng.standard_normal(shape) + (2.0 if name.endswith("f.b") else 0.0)
        elif last == "b":
            t = 0.5 * rng.standard_normal(shape)
        elif name == "embed":
            t = rng.standard_normal(shape)
        elif last in ("i", "f"):
            t = 3.0 * rng.standard_normal(shape) / np.sqrt(shape[-1])  # gates that reach their caps now and then
        elif last in ("q", "k", "a1", "a2", "gate", "up"):
            t = 2.0 * rng.standard_normal(shape) / np.sqrt(shape[-1])  # peaked scores, clamps that bite
        else:
            t = rng.standard_normal(shape) / np.sqrt(shape[-1])
        out[name] = torch.from_numpy(np.asarray(t, dtype=np.float32)).to(torch.bfloat16)
    return out


def write_model(folder, cfg, weights):
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))
    return str(folder)


def as_float64(weights):
    return {k: (v if v.dtype == torch.int32 else v.to(torch.float64)) for k, v in weights.items()}
