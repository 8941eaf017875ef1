"""Mixers whose memory is a matrix per head that decays by gates computed from the current token: gated linear attention
(a decay per key channel) and the matrix memory of xLSTM (mLSTM: scalar input and forget gates per head, kept in range by a
running maximum).

Both keep their state in 32-bit in the cache's state records, one record per sequence slot, zero when the sequence starts,
and both run on the same recurrence kernel (csrc/gated_recurrent.cu):

    S_t = diag(a_t) S_(t-1) + b_t k_t v_t^T,   o_t = S_t^T q_t

Everything between the projections and the state is 32-bit arithmetic (decays and their logarithms, gates, the running
maximum, the normaliser, the norms of the heads); the projections come in the run's element type.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..errors import ConfigError
from ..kernels import ops
from ..kernels.linear import linear, linear_to_stream
from .base import MIXERS, Mixer, ParamInfo, StateNeed

# prompt steps whose longest sequence brings fewer tokens than this go token by token like a decode step
_CHUNKED_MIN_TOKENS = 32


def _recurrence(mixer, q, k, v, log_decay, in_scale, state, step, ext: bool):
    """The recurrence over a step's tokens: chunk by chunk for the prompts of a bfloat16 run (all chunks side by side, equal
    within rounding), token by token otherwise (equal bits however a sequence is cut into steps)."""
    chunked = (q.dtype == torch.bfloat16 and step.max_q_len >= _CHUNKED_MIN_TOKENS and ops.gated_attn_chunked_takes(mixer.dim, mixer.vdim + (1 if ext else 0)))
    if chunked:
        need = ops.gated_attn_chunked_scratch_floats(step.n_seqs, step.max_q_len, mixer.H, mixer.dim, mixer.vdim + (1 if ext else 0))
        scratch = mixer.rt.workspace.get("gated_attn_chunks", need, torch.float32)
        return ops.gated_attn_chunked(
            q, k, v, log_decay, in_scale, state, step.slot_ids, step.seq_start, mixer.H, mixer.dim, mixer.vdim, step.max_q_len, scratch,
            q_scale=mixer.q_scale, ext=ext,
        )
    return ops.gated_attn(
        q, k, v, log_decay, in_scale, state, step.slot_ids, step.seq_start, mixer.H, mixer.dim, mixer.vdim, q_scale=mixer.q_scale, ext=ext,
    )


@MIXERS.register("gated_linear_attention")
class GatedLinearAttention(Mixer):
    """Linear attention with a learned decay per key channel and token:

        q = W_q xn * q_scale, k = W_k xn  [H, dim];   v = W_v xn  [H, vdim]
        a = sigmoid(W_a2 (W_a1 xn) + b_a)^(1/tau)                       [H, dim], through a low-rank pair of matrices
        S_t = diag(a_t) S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t          (per head)
        result = W_o ( concat_h (rmsnorm(o_t[h]) * w_norm) * silu(W_g xn) )

    Every head's o is normed on its own over its vdim values with one weight row shared by the heads.

    params: hidden_size, num_heads, dim, vdim, decay_rank (the inner size of the low-rank pair; 0: whatever the checkpoint's
            tensors have), tau, eps (of the heads' norm),
            q_scale (default dim^-1/2), out_scale (default 1), names (optional: keys q k v gate norm o a1 a2 a2_bias).
    tensors: <prefix>q [H dim, d], k [H dim, d], v [H vdim, d], g [H vdim, d], o [d, H vdim], norm [vdim],
             a1 [rank, d], a2 [H dim, rank], a2.b [H dim]."""

    takes_out = True
    _NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "norm": "norm", "o": "o", "a1": "a1", "a2": "a2", "a2_bias": "a2.b"}

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.d = int(self._param("hidden_size"))
        self.H = int(self._param("num_heads"))
        self.dim = int(self._param("dim"))
        self.vdim = int(self._param("vdim"))
        self.rank = int(self._param("decay_rank"))
        self.tau = float(self._param("tau"))
        self.eps = float(self._param("eps"))
        if min(self.H, self.dim, self.vdim) <= 0 or self.rank < 0 or self.dim > 1024 or self.vdim > 512:
            raise ConfigError(f"gated_linear_attention: sizes heads={self.H} dim={self.dim} vdim={self.vdim} rank={self.rank} (dim at most 1024, vdim at most 512)")
        if not self.tau > 0:
            raise ConfigError(f"gated_linear_attention: tau = {self.tau} must be positive")
        self.q_scale = float(spec.params.get("q_scale") or self.dim ** -0.5)
        self.out_scale = float(spec.params.get("out_scale", 1.0))
        self.names = dict(self._NAMES, **dict(spec.params.get("names", {})))
        self.qd, self.vd = self.H * self.dim, self.H * self.vdim
        self.w_in = self.w_a2 = self.b_a = self.w_o = self.w_norm = None

    def cache_need(self):
        return StateNeed((self.H, self.dim, self.vdim), torch.float32)

    def param_infos(self) -> Dict[str, ParamInfo]:
        p, n = self.prefix, self.names
        return {
            p + n["q"]: ParamInfo((self.qd, self.d)),
            p + n["k"]: ParamInfo((self.qd, self.d)),
            p + n["v"]: ParamInfo((self.vd, self.d)),
            p + n["gate"]: ParamInfo((self.vd, self.d)),
            p + n["a1"]: ParamInfo((self.rank or -1, self.d), free=16),
            p + n["a2"]: ParamInfo((self.qd, self.rank or -1), free=16),
            p + n["a2_bias"]: ParamInfo((self.qd,), "scalars", centre=0.0),
            p + n["norm"]: ParamInfo((self.vdim,), "scalars", centre=1.0),
            p + n["o"]: ParamInfo((self.d, self.vd)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = self.prefix, self.names
        # one product serves q, k, v, the gate and the decay's inner row
        self.w_in = torch.cat([tensors[p + n[key]] for key in ("q", "k", "v", "gate", "a1")], dim=0).contiguous()
        self.w_a2 = tensors[p + n["a2"]].contiguous()
        if tensors[p + n["a1"]].shape[0] != self.w_a2.shape[1]:
            raise ConfigError(f"gated_linear_attention: '{p + n['a1']}' has {tensors[p + n['a1']].shape[0]} rows, '{p + n['a2']}' {self.w_a2.shape[1]} columns")
        self.b_a = tensors[p + n["a2_bias"]].contiguous()
        self.w_norm = tensors[p + n["norm"]].contiguous()
        self.w_o = tensors[p + n["o"]].contiguous()

    def forward(self, xn: torch.Tensor, step, cache, shared_cache: bool = False) -> torch.Tensor:
        a, w_o = self.forward_unprojected(xn, step, cache, shared_cache)
        return linear_to_stream(a, w_o)

    def forward_unprojected(self, xn: torch.Tensor, step, cache, shared_cache: bool = False, out=None):
        if shared_cache:
            raise ConfigError("gated_linear_attention: a state cannot be another run's")
        proj = linear(xn, self.w_in)
        qd, vd = self.qd, self.vd
        q, k, v = proj[:, :qd], proj[:, qd : 2 * qd], proj[:, 2 * qd : 2 * qd + vd]
        gate = proj[:, 2 * qd + vd : 2 * qd + 2 * vd]
        inner = proj[:, 2 * qd + 2 * vd :]
        if inner.data_ptr() % 16 or inner.stride(0) % 8:  # the second product moves its rows in 16-byte pieces
            inner = inner.contiguous()
        z = linear(inner, self.w_a2)
        log_decay = ops.gla_log_decay(z, self.b_a, self.tau)
        o = _recurrence(self, q, k, v, log_decay, None, cache.state, step, ext=False)
        a = ops.head_norm_gate(o, self.H, self.vdim, self.w_norm, self.eps, gate, ops.GATE_SILU, xn.dtype, out_scale=self.out_scale, out=out)
        return a, self.w_o


@MIXERS.register("mlstm")
class MatrixMemory(Mixer):
    """The matrix memory of xLSTM (mLSTM), per head, with gates in logarithms and a running maximum m that keeps them in range:

        q = W_q xn * q_scale, k = W_k xn  [H, dim];   v = W_v xn  [H, vdim]
        i = cap tanh((W_i xn + b_i) / cap),   f = logsigmoid(cap tanh((W_f xn + b_f) / cap))          (one number per head each)
        m_t = max(f_t + m_(t-1), i_t)                                                                  (m starts at 0)
        S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T,   n_t likewise from k_t alone
        o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + den_eps)
        result = W_o ( concat_h (o_t[h] / rms(o_t[h])) * w_norm * sigmoid(W_g xn) )

    n rides along as one more column of the state (fed with v = 1), so one recurrence serves S and n.  Records: [H, dim, vdim + 1]
    and m [H], both 32-bit.

    params: hidden_size, num_heads, dim, vdim, gate_cap, eps (of the heads' norm), den_eps (default 1e-6), q_scale (default dim^-1/2),
            out_scale (default 1), names (optional: keys q k v gate norm o i f i_bias f_bias).
    tensors: <prefix>q [H dim, d], k [H dim, d], v [H vdim, d], g [H vdim, d], o [d, H vdim], norm [H vdim], i [H, d], f [H, d],
             i.b [H], f.b [H]."""

    takes_out = True
    _NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "norm": "norm", "o": "o", "i": "i", "f": "f", "i_bias": "i.b", "f_bias": "f.b"}

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.d = int(self._param("hidden_size"))
        self.H = int(self._param("num_heads"))
        self.dim = int(self._param("dim"))
        self.vdim = int(self._param("vdim"))
        self.cap = float(self._param("gate_cap"))
        self.eps = float(self._param("eps"))
        self.den_eps = float(spec.params.get("den_eps", 1e-6))
        if min(self.H, self.dim, self.vdim) <= 0 or self.dim > 1024 or self.vdim > 512:
            raise ConfigError(f"mlstm: sizes heads={self.H} dim={self.dim} vdim={self.vdim} (dim at most 1024, vdim at most 512)")
        if not self.cap > 0:
            raise ConfigError(f"mlstm: gate_cap = {self.cap} must be positive")
        self.q_scale = float(spec.params.get("q_scale") or self.dim ** -0.5)
        self.out_scale = float(spec.params.get("out_scale", 1.0))
        self.names = dict(self._NAMES, **dict(spec.params.get("names", {})))
        self.qd, self.vd = self.H * self.dim, self.H * self.vdim
        self.w_in = self.b_i = self.b_f = self.w_o = self.w_norm = None

    def cache_need(self):
        return (StateNeed((self.H, self.dim, self.vdim + 1), torch.float32), StateNeed((self.H,), torch.float32))

    def param_infos(self) -> Dict[str, ParamInfo]:
        p, n = self.prefix, self.names
        return {
            p + n["q"]: ParamInfo((self.qd, self.d)),
            p + n["k"]: ParamInfo((self.qd, self.d)),
            p + n["v"]: ParamInfo((self.vd, self.d)),
            p + n["gate"]: ParamInfo((self.vd, self.d)),
            p + n["i"]: ParamInfo((self.H, self.d)),
            p + n["f"]: ParamInfo((self.H, self.d)),
            p + n["i_bias"]: ParamInfo((self.H,), "scalars", centre=0.0),
            p + n["f_bias"]: ParamInfo((self.H,), "scalars", centre=0.0),
            p + n["norm"]: ParamInfo((self.vd,), "scalars", centre=1.0),
            p + n["o"]: ParamInfo((self.d, self.vd)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = self.prefix, self.names
        # one product serves q, k, v, the output gate and the two gates of the recurrence
        self.w_in = torch.cat([tensors[p + n[key]] for key in ("q", "k", "v", "gate", "i", "f")], dim=0).contiguous()
        self.b_i, self.b_f = tensors[p + n["i_bias"]].contiguous(), tensors[p + n["f_bias"]].contiguous()
        self.w_norm = tensors[p + n["norm"]].contiguous()
        self.w_o = tensors[p + n["o"]].contiguous()

    def forward(self, xn: torch.Tensor, step, cache, shared_cache: bool = False) -> torch.Tensor:
        a, w_o = self.forward_unprojected(xn, step, cache, shared_cache)
        return linear_to_stream(a, w_o)

    def forward_unprojected(self, xn: torch.Tensor, step, cache, shared_cache: bool = False, out=None):
        if shared_cache:
            raise ConfigError("mlstm: a state cannot be another run's")
        memory, maximum = cache
        proj = linear(xn, self.w_in)
        qd, vd, H = self.qd, self.vd, self.H
        q, k, v = proj[:, :qd], proj[:, qd : 2 * qd], proj[:, 2 * qd : 2 * qd + vd]
        gate = proj[:, 2 * qd + vd : 2 * qd + 2 * vd]
        gi, gf = proj[:, 2 * qd + 2 * vd : 2 * qd + 2 * vd + H], proj[:, 2 * qd + 2 * vd + H :]
        log_a, b, m = ops.mlstm_gates(gi, gf, self.b_i, self.b_f, self.cap, maximum.state, step.slot_ids, step.seq_start,
                                      scan=xn.dtype == torch.bfloat16 and step.max_q_len >= _CHUNKED_MIN_TOKENS)
        o = _recurrence(self, q, k, v, log_a, b, memory.state, step, ext=True)
        a = ops.head_norm_gate(
            o, H, self.vdim, self.w_norm, self.eps, gate, ops.GATE_SIGMOID, xn.dtype, m=m, den_eps=self.den_eps, out_scale=self.out_scale, out=out,
        )
        return a, self.w_o
