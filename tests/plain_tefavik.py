"""A plain, slow implementation of the Tefavik architecture in float64: whole sequences, no cache, no batching,
one function per mechanism.  It imports nothing from the package; the tests compare the library against it.

A model is (cfg, weights): cfg the parsed config.json (a dict), weights a dict name -> float64 torch tensor.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * w


def logistic(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def log_logistic(z: torch.Tensor) -> torch.Tensor:
    return -torch.log1p(torch.exp(-z.abs())) + torch.minimum(z, torch.zeros_like(z))


# ------------------------------------------------------------------ gated linear attention
def gla_decay(h, W, p, m):
    """alpha[T, heads, dim] = sigmoid(z)^(1/tau), z = W_a2 (W_a1 h) + b."""
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    return torch.exp(log_logistic(z) / m["tau"]).view(h.shape[0], m["heads"], m["dim"])


def gla_recurrence(q, k, v, alpha):
    """q, k, alpha [T, H, dim], v [T, H, vdim] -> o [T, H, vdim]; S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, dim = q.shape
    S = torch.zeros(H, dim, v.shape[2], dtype=F64)
    out = []
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out.append(torch.einsum("hdv,hd->hv", S, q[t]))
    return torch.stack(out)


def gla_mixer(h, W, p, m, eps):
    T, H, dim, vdim = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, dim) * dim ** -0.5
    k = (h @ W[p + "k"].T).view(T, H, dim)
    v = (h @ W[p + "v"].T).view(T, H, vdim)
    o = gla_recurrence(q, k, v, gla_decay(h, W, p, m))
    o = rms_norm(o, W[p + "norm"], eps).reshape(T, H * vdim)
    g = h @ W[p + "g"].T
    return (o * (g * logistic(g))) @ W[p + "o"].T


# ------------------------------------------------------------------ chunked softmax attention with a sink
def rotate_interleaved(x, positions, base, dims):
    """x [T, heads, dim]; the first `dims` numbers of each head turned in neighbouring pairs by position * base^(-2i/dims)."""
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=F64)
    ang = positions.to(F64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    u, w = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - w * s
    out[..., 1:dims:2] = w * c + u * s
    return out


def chunk_mask(T: int, size: int) -> torch.Tensor:
    """visible[i, j]: j <= i and both in the same chunk of `size` positions counted from 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i // size) == (j // size))


def softmax_plus_one(s: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    """p_j = exp(s_j) / (1 + sum over visible j of exp(s_j)), computed without overflow."""
    s = s.masked_fill(~visible, -math.inf)
    mx = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - mx)
    return e / (torch.exp(-mx) + e.sum(dim=-1, keepdim=True))


def chunked_attention(h, W, p, m, eps):
    T, H, G, dim, vdim = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, dim)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, dim)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, vdim)
    q = rms_norm(q, W[p + "q.norm"], eps)
    k = rms_norm(k, W[p + "k.norm"], eps)
    pos = torch.arange(T)
    q = rotate_interleaved(q, pos, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_interleaved(k, pos, m["rot"]["base"], m["rot"]["dims"])
    visible = chunk_mask(T, m["mask"]["size"])
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        s = m["softcap"] * torch.tanh(s / m["softcap"])
        heads.append(softmax_plus_one(s, visible) @ v[:, g])
    return torch.cat(heads, dim=1) @ W[p + "o"].T


# ------------------------------------------------------------------ matrix memory (mLSTM)
def capped(z, cap):
    return cap * torch.tanh(z / cap)


def mlstm_recurrence(q, k, v, log_i, log_f):
    """q, k [T, H, dim], v [T, H, vdim], log_i, log_f [T, H] -> o [T, H, vdim] (before any norm)."""
    T, H, dim = q.shape
    S = torch.zeros(H, dim, v.shape[2], dtype=F64)
    n = torch.zeros(H, dim, dtype=F64)
    mm = torch.zeros(H, dtype=F64)
    out = []
    for t in range(T):
        m_new = torch.maximum(log_f[t] + mm, log_i[t])
        fg = torch.exp(log_f[t] + mm - m_new)
        ig = torch.exp(log_i[t] - m_new)
        S = fg[:, None, None] * S + ig[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = fg[:, None] * n + ig[:, None] * k[t]
        mm = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(dim=-1).abs(), torch.exp(-mm)) + 1e-6
        out.append(num / den[:, None])
    return torch.stack(out)


def mlstm_mixer(h, W, p, m, eps):
    T, H, dim, vdim, cap = h.shape[0], m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ W[p + "q"].T).view(T, H, dim) * dim ** -0.5
    k = (h @ W[p + "k"].T).view(T, H, dim)
    v = (h @ W[p + "v"].T).view(T, H, vdim)
    log_i = capped(h @ W[p + "i"].T + W[p + "i.b"], cap)
    log_f = log_logistic(capped(h @ W[p + "f"].T + W[p + "f.b"], cap))
    o = rms(mlstm_recurrence(q, k, v, log_i, log_f), eps).reshape(T, H * vdim) * W[p + "norm"]
    return (o * logistic(h @ W[p + "g"].T)) @ W[p + "o"].T


# ------------------------------------------------------------------ two mixers side by side
def parallel_mixer(h, W, p, m, eps):
    left = rms_norm(chunked_attention(h, W, p + "left.", m["left"], eps), W[p + "left.out"], eps)
    right = rms_norm(mlstm_mixer(h, W, p + "right.", m["right"], eps), W[p + "right.out"], eps)
    return 0.5 * (left + right)


# ------------------------------------------------------------------ experts chosen by a table
def expert(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, min=-limit, max=limit)
    return (g * logistic(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def table_experts(h, tokens, W, p, mlp):
    top, limit = mlp["router"]["top"], mlp["expert"]["limit"]
    table = W[p + "table"].to(torch.long)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in table[int(tokens[t])].tolist():
            out[t] += expert(h[t : t + 1], W, f"{p}e{e}.", limit)[0] / top
    return out


# ------------------------------------------------------------------ the model
def layer_order(cfg):
    """[(layer index, whether the embedding output is added before it)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for r in range(times):
        order += [(i, r > 0 and i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def forward(cfg, W, tokens, layers_out=None):
    """tokens: a list of ids; returns float64 logits [T, vocab].  layers_out: a list that receives the stream after every layer run."""
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x0 = W["embed"][tokens]
    x = x0.clone()
    for i, add_embedding in layer_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        if add_embedding:
            x = x + x0
        h = rms_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "gla":
            x = x + gla_mixer(h, W, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            x = x + parallel_mixer(h, W, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            h = rms_norm(x, W[p + "norm2"], eps)
            x = x + table_experts(h, tokens, W, p + "mlp.", layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["embed"].T
