"""A plain, slow implementation of the Namalix architecture in float64: whole sequences, no cache, no batching,
one function per mechanism.  It imports nothing from the package; the tests compare the library against it.

A model is (cfg, weights): cfg the parsed config.json (a dict), weights a dict name -> float64 torch tensor.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64

SWISH_ALPHA = 1.702
DELTA_UNIT_EPS = 1e-6
ROUTER_SUM_EPS = 1e-20


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_around_zero(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose stored weight is the distance of the true weight from one."""
    return rms(x, eps) * (1.0 + w)


def logistic(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * logistic(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.maximum(z, torch.zeros_like(z)) + torch.log1p(torch.exp(-z.abs()))


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


# ------------------------------------------------------------------ rotations
def plain_frequencies(base: float, dims: int) -> torch.Tensor:
    i = torch.arange(dims // 2, dtype=F64)
    return base ** (-2.0 * i / dims)


def yarn_frequencies(base: float, dims: int, scaling) -> tuple:
    """(frequencies, factor on cosines and sines): pairs that turn often keep their frequency, pairs that turn rarely over the
    original context are slowed by `factor`, a linear ramp over the pair index between the two."""
    f = plain_frequencies(base, dims)
    if scaling is None:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_index(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_index(float(scaling["slow"]))), dims - 1)
    i = torch.arange(dims // 2, dtype=F64)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, dims: int, neighbours: bool, magnitude: float = 1.0) -> torch.Tensor:
    """x [T, heads, dim]; the first `dims` numbers of each head are turned in pairs by position * freqs[i]: pair i is
    (2i, 2i + 1) if `neighbours`, else (i, i + dims / 2)."""
    if not dims:
        return x
    ang = positions.to(F64)[:, None] * freqs[None, :]
    c, s = (torch.cos(ang) * magnitude)[:, None, :], (torch.sin(ang) * magnitude)[:, None, :]
    out = x.clone()
    if neighbours:
        u, w = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - w * s
        out[..., 1:dims:2] = w * c + u * s
    else:
        half = dims // 2
        u, w = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - w * s
        out[..., half:dims] = w * c + u * s
    return out


# ------------------------------------------------------------------ attention with logistic weights
def attention_weights(q, k, m, pb, talk):
    """q [T, H, dim], k [T, G, dim] (rotated) -> mixed weights [H, T, T]: logistic(cap(q . k * scale) + pb_h) of the visible
    keys (j <= i), zero elsewhere, then mixed over the heads by `talk`."""
    T, H, _ = q.shape
    G = k.shape[1]
    kk = k.repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    cap = float(m.get("softcap") or 0.0)
    if cap:
        s = cap * torch.tanh(s / cap)
    w = logistic(s + pb[:, None, None])
    visible = torch.arange(T)[None, :] <= torch.arange(T)[:, None]
    w = w * visible[None].to(F64)
    return torch.einsum("hg,gij->hij", talk, w)


def attention_mixer(h, W, p, m, positions, shared):
    """shared: a dict that carries the first value-mixing layer's values to the later ones."""
    T, H, G, dim, vdim = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, dim)
    k = (h @ W[p + "k"].T).view(T, G, dim)
    v = (h @ W[p + "v"].T).view(T, G, vdim)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        f, mag = yarn_frequencies(float(rot["base"]), int(rot["dims"]), rot.get("scaling"))
        q = rotate(q, positions, f, int(rot["dims"]), True, mag)
        k = rotate(k, positions, f, int(rot["dims"]), True, mag)
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = W[p + "vmix"]
            v = (1.0 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    w = attention_weights(q, k, m, W[p + "pb"], W[p + "talk"])
    vv = v.repeat_interleave(H // G, dim=1)
    o = torch.einsum("hij,jhv->ihv", w, vv)
    gate = logistic(h @ W[p + "g"].T)  # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * vdim) @ W[p + "o"].T


# ------------------------------------------------------------------ retention
def retention_recurrence(q, k, v, decay):
    """q, k [T, H, dim], v [T, H, vdim], decay [H] -> o [T, H, vdim]; S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, dim = q.shape
    S = torch.zeros(H, dim, v.shape[2], dtype=F64)
    out = []
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out)


def retention_mixer(h, W, p, m, positions, eps):
    T, H, dim, vdim = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, dim)
    k = (h @ W[p + "k"].T).view(T, H, dim)
    v = (h @ W[p + "v"].T).view(T, H, vdim)
    rot = m.get("rot")
    if rot and rot.get("dims"):
        f = plain_frequencies(float(rot["base"]), int(rot["dims"]))
        q = rotate(q, positions, f, int(rot["dims"]), False)
        k = rotate(k, positions, f, int(rot["dims"]), False)
    k = k * dim ** -0.5
    o = retention_recurrence(q, k, v, torch.tensor(m["decay"], dtype=F64))
    o = rms(o, eps).reshape(T, H * vdim)
    return (o * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


# ------------------------------------------------------------------ gated delta rule
def short_convolution(x, w):
    """x [T, C], w [C, taps]: y_t = sum_i w[:, i] x_(t - taps + 1 + i), zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=F64), x], dim=0)
    y = torch.zeros(T, C, dtype=F64)
    for i in range(taps):
        y = y + padded[i : i + T] * w[:, i][None, :]
    return y


def unit(x):
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + DELTA_UNIT_EPS)


def delta_recurrence(q, k, v, beta, g):
    """q, k [T, H, dim], v [T, H, vdim], beta, g [T, H] -> o [T, H, vdim]."""
    T, H, dim = q.shape
    S = torch.zeros(H, dim, v.shape[2], dtype=F64)
    out = []
    for t in range(T):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out)


def delta_mixer(h, W, p, m, eps):
    T, H, G, dim, vdim = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ W[p + "q"].T, W[p + "q.conv"])).view(T, G, dim)
    k = silu(short_convolution(h @ W[p + "k"].T, W[p + "k.conv"])).view(T, G, dim)
    v = silu(short_convolution(h @ W[p + "v"].T, W[p + "v.conv"])).view(T, H, vdim)
    q = unit(q) * dim ** -0.5
    k = unit(k)
    q = q.repeat_interleave(H // G, dim=1)
    k = k.repeat_interleave(H // G, dim=1)
    beta = logistic(h @ W[p + "b"].T)
    g = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    o = delta_recurrence(q, k, v, beta, g)
    o = (rms(o, eps) * W[p + "norm"]).reshape(T, H * vdim)
    return (o * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


# ------------------------------------------------------------------ feed-forwards
def dense_ff(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def expert_ff(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, min=-limit, max=limit)
    return (g * logistic(SWISH_ALPHA * g) * (u + 1.0)) @ W[p + "down"].T


def route(h, W, p, router):
    """-> (chosen [T, top], weights [T, top])."""
    s = logistic(h @ W[p + "router"].T)
    chosen = torch.topk(s + W[p + "correction"], int(router["top"]), dim=-1).indices
    w = torch.gather(s, 1, chosen)
    w = w / (w.sum(dim=-1, keepdim=True) + ROUTER_SUM_EPS) * float(router["scale"])
    return chosen, w


def moe_ff(h, W, p, mlp):
    chosen, w = route(h, W, p, mlp["router"])
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, we in zip(chosen[t].tolist(), w[t]):
            out[t] += we * expert_ff(h[t : t + 1], W, f"{p}e{e}.", float(mlp["expert"]["limit"]))[0]
    return out


# ------------------------------------------------------------------ the model
def plain_streams(cfg, W, tokens):
    """-> (logits [T, vocab], the residual stream after every layer [layers, T, width])."""
    W = {k: v.to(F64) for k, v in W.items()}
    eps = float(cfg["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x = W["embed"][tokens] * float(cfg["embedding"]["scale"])
    shared, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm_around_zero(x, W[p + "norm1"], eps)
        kind, m = layer["type"], layer["mixer"]
        if kind == "attention":
            y = attention_mixer(h, W, p + "mix.", m, positions, shared)
        elif kind == "retention":
            y = retention_mixer(h, W, p + "mix.", m, positions, eps)
        elif kind == "delta":
            y = delta_mixer(h, W, p + "mix.", m, eps)
        else:
            raise ValueError(f"layer {i}: unknown mixer '{kind}'")
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + (dense_ff(h, W, p + "mlp.") if mlp["kind"] == "dense" else moe_ff(h, W, p + "mlp.", mlp))
        x = x + y
        after.append(x)
    logits = norm_around_zero(x, W["final.norm"], eps) @ W["head"].T
    return logits, torch.stack(after)


def plain_logits(cfg, W, tokens):
    return plain_streams(cfg, W, tokens)[0]
