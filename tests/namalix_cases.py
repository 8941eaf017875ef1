"""Small Namalix configurations and random weights for the tests, made without the library.

Weights are drawn so that every mechanism matters (activations of order one, head biases that keep most weights small and
let some keys stand out, mixing matrices away from the identity, decays from quick forgetting to almost none, experts whose
clamps bite, norm weights away from one), rounded to bfloat16 and written with the third-party safetensors package."""

import json
import os

import numpy as np
import torch


def _rot(base, dims, scaling=None):
    return {"base": base, "dims": dims, "scaling": scaling} if scaling else {"base": base, "dims": dims}


def _attn(heads, kv_heads, dim, vdim, rot, scale, softcap, v_mix):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot, "scale": scale, "softcap": softcap, "v_mix": v_mix}


def _ret(heads, dim, vdim, decay, rot):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay, "rot": rot}


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, scale, ff, limit):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff, "limit": limit}}


def config_a():
    """Five layers that differ in everything: a retention layer first, sizes that are no multiples of 8, 6 heads on 2 and 4 on 2,
    rotations over part of a head (with and without rescaled frequencies) and over all of it, value mixing whose source is
    not the first layer, an attention layer that takes no part in it, a delta layer with 4 heads on 2 q/k heads and no
    feed-forward, two of five experts and all of three."""
    yarn = {"factor": 2.0, "original": 48, "fast": 4.0, "slow": 0.5}
    return {
        "architecture": "Namalix", "vocab": 131, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
        "layers": [
            {"type": "retention", "mixer": _ret(3, 24, 40, [0.9, 0.97, 0.999], _rot(500.0, 16)), "mlp": _dense(100)},
            {"type": "attention", "mixer": _attn(6, 2, 20, 12, _rot(10000.0, 8, yarn), 0.3, 5.0, True), "mlp": _moe(5, 2, 2.5, 24, 1.0)},
            {"type": "delta", "mixer": _delta(4, 2, 24, 20, 3), "mlp": None},
            {"type": "attention", "mixer": _attn(4, 2, 16, 12, _rot(1000.0, 16), 0.25, 30.0, True), "mlp": _moe(3, 3, 1.0, 16, 2.5)},
            {"type": "attention", "mixer": _attn(2, 2, 8, 8, _rot(100.0, 0), 0.35, 0.0, False), "mlp": _dense(40)},
        ],
    }


def config_b():
    """A width that no 16-byte-row kernel takes (68), single heads, a decay of exactly one, convolutions of two taps and of one
    (no record of inputs at all), a state of 36 x 36 (two row slices, two column tiles), a value source without anyone mixing,
    one expert of one."""
    return {
        "architecture": "Namalix", "vocab": 77, "width": 68, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
        "layers": [
            {"type": "delta", "mixer": _delta(1, 1, 40, 8, 2), "mlp": _moe(1, 1, 0.7, 30, 1.5)},
            {"type": "attention", "mixer": _attn(1, 1, 24, 16, _rot(500000.0, 4), 0.4, 2.0, True), "mlp": None},
            {"type": "retention", "mixer": _ret(1, 12, 20, [1.0], _rot(10000.0, 0)), "mlp": _moe(6, 3, 1.5, 12, 0.7)},
            {"type": "delta", "mixer": _delta(2, 2, 36, 36, 1), "mlp": _dense(70)},
        ],
    }


def config_c():
    """Sizes in multiples of 8 and 64 (the shapes the tensor-core kernels take): heads of 64 and 32 with values of 64, a delta
    layer with keys of 128 on one q/k head, convolutions of four taps, a second attention layer that mixes the first one's values."""
    yarn = {"factor": 8.0, "original": 256, "fast": 16.0, "slow": 2.0}
    return {
        "architecture": "Namalix", "vocab": 160, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 8.0},
        "layers": [
            {"type": "attention", "mixer": _attn(4, 2, 64, 64, _rot(10000.0, 32, yarn), 0.125, 20.0, True), "mlp": _dense(256)},
            {"type": "retention", "mixer": _ret(2, 64, 64, [0.95, 0.995], _rot(1000000.0, 64)), "mlp": _moe(8, 3, 1.25, 48, 2.0)},
            {"type": "delta", "mixer": _delta(2, 1, 128, 64, 4), "mlp": _moe(4, 1, 2.0, 128, 3.0)},
            {"type": "attention", "mixer": _attn(8, 2, 32, 64, _rot(10000.0, 32, yarn), 0.18, 10.0, True), "mlp": _dense(128)},
        ],
    }


def config_d():
    """Seven layers of larger and odd sizes in another order: a delta layer first (6 heads on 3 q/k heads, keys of 48: a last row slice
    that is half empty, five taps), an attention layer outside the value mixing BEFORE its source, 10 heads on 5 and 16 on 4,
    keys of 48 and values of 24 and 40 (padded tiles of the tensor-core kernel), five retention heads with rotated halves of
    24, a state of 128 x 96, twelve experts of which three, all of four, one of three."""
    yarn = {"factor": 16.0, "original": 512, "fast": 24.0, "slow": 0.5}
    return {
        "architecture": "Namalix", "vocab": 1000, "width": 320, "norm": {"eps": 1e-5}, "embedding": {"scale": 11.0},
        "layers": [
            {"type": "delta", "mixer": _delta(6, 3, 48, 40, 5), "mlp": _moe(6, 2, 2.0, 96, 2.0)},
            {"type": "attention", "mixer": _attn(10, 5, 48, 24, _rot(50000.0, 24, yarn), 0.2, 15.0, False), "mlp": _dense(512)},
            {"type": "attention", "mixer": _attn(12, 4, 32, 40, _rot(10000.0, 32, yarn), 0.22, 50.0, True), "mlp": _moe(4, 4, 1.0, 128, 0.9)},
            {"type": "retention", "mixer": _ret(5, 48, 24, [0.8, 0.9, 0.99, 0.999, 0.9999], _rot(10000.0, 24)), "mlp": None},
            {"type": "attention", "mixer": _attn(4, 4, 64, 40, _rot(10000.0, 16), 0.125, 8.0, True), "mlp": _dense(200)},
            {"type": "delta", "mixer": _delta(2, 2, 128, 96, 2), "mlp": _moe(12, 3, 0.5, 64, 4.0)},
            {"type": "attention", "mixer": _attn(16, 4, 32, 40, _rot(1000.0, 8), 0.3, 30.0, True), "mlp": _moe(3, 1, 3.0, 256, 1.0)},
        ],
    }


CONFIGS = {"a": config_a, "b": config_b, "c": config_c, "d": config_d}


def tensor_shapes(cfg):
    d, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, d), "head": (V, d), "final.norm": (d,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (d,)
        q = p + "mix."
        if layer["type"] == "attention":
            H, G = m["heads"], m["kv_heads"]
            out[q + "q"], out[q + "k"], out[q + "v"] = (H * m["dim"], d), (G * m["dim"], d), (G * m["vdim"], d)
            out[q + "talk"], out[q + "pb"], out[q + "g"] = (H, H), (H,), (H, d)
            if m["v_mix"]:
                out[q + "vmix"] = ()
            out[q + "o"] = (d, H * m["vdim"])
        elif layer["type"] == "retention":
            H = m["heads"]
            out[q + "q"] = out[q + "k"] = (H * m["dim"], d)
            out[q + "v"] = out[q + "g"] = (H * m["vdim"], d)
            out[q + "o"] = (d, H * m["vdim"])
        else:
            H, G, taps = m["heads"], m["kv_heads"], m["conv"]
            out[q + "q"] = out[q + "k"] = (G * m["dim"], d)
            out[q + "q.conv"] = out[q + "k.conv"] = (G * m["dim"], taps)
            out[q + "v"] = out[q + "g"] = (H * m["vdim"], d)
            out[q + "v.conv"] = (H * m["vdim"], taps)
            out[q + "b"] = out[q + "a"] = (H, d)
            out[q + "A_log"] = out[q + "dt_bias"] = (H,)
            out[q + "norm"] = (m["vdim"],)
            out[q + "o"] = (d, H * m["vdim"])
        mlp = layer["mlp"]
        if mlp is None:
            continue
        q = p + "mlp."
        if mlp["kind"] == "dense":
            out[q + "gate"] = out[q + "up"] = (mlp["ff"], d)
            out[q + "down"] = (d, mlp["ff"])
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            for j in range(E):
                out[f"{q}e{j}.gate"] = out[f"{q}e{j}.up"] = (ff, d)
                out[f"{q}e{j}.down"] = (d, ff)
            out[q + "router"], out[q + "correction"] = (E, d), (E,)
    return out


def random_weights(cfg, seed):
    """name -> bfloat16 torch tensor."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1",) or name == "final.norm":
            t = 0.3 * rng.standard_normal(shape)  # stored around zero
        elif last == "norm":
            t = 1.0 + 0.3 * rng.standard_normal(shape)
        elif last == "vmix":
            t = np.asarray(rng.uniform(0.2, 0.8))
        elif last == "talk":
            t = np.eye(shape[0]) * 0.7 + 0.4 * rng.standard_normal(shape)
        elif last == "pb":
            t = -1.5 + rng.standard_normal(shape)
        elif last == "conv":
            t = 0.6 * rng.standard_normal(shape)
        elif last == "A_log":
            t = -1.0 + rng.standard_normal(shape)
        elif last == "dt_bias":
            t = rng.standard_normal(shape)
        elif last == "correction":
            t = 0.3 * rng.standard_normal(shape)
        elif name == "embed":
            t = rng.standard_normal(shape)
        elif last in ("q", "k", "gate", "up", "router", "b", "a"):
            t = 2.0 * rng.standard_normal(shape) / np.sqrt(shape[-1])  # peaked scores, clamps that bite, gates on both sides
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
    return {k: v.to(torch.float64) for k, v in weights.items()}
