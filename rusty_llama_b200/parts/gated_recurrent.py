"""Mixers whose memory is a matrix per head that decays by gates computed from the current token: gated linear attention
(a decay per key channel), the matrix memory of xLSTM (mLSTM: scalar input and forget gates per head, kept in range by a
running maximum) and the gated delta rule (a decay per head, and a write that corrects what the state already holds for the key).

All keep their state in 32-bit in the cache's state records, one record per sequence slot, zero when the sequence starts;
the first two run on the same recurrence kernel (csrc/gated_recurrent.cu), the delta rule on its own (csrc/delta_rule.cu):

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


@MIXERS.register("gated_delta")
class GatedDeltaRule(Mixer):
    """The gated delta rule, per head with a state S [dim, vdim]:

        q = act(conv(W_q xn)), k = act(conv(W_k xn))  [G, dim];   v = act(conv(W_v xn))  [H, vdim]     (act = silu)
        q <- q / sqrt(sum(q^2) + unit_eps) * q_scale,  k <- k / sqrt(sum(k^2) + unit_eps)               (per head)
        beta = logistic(W_b xn),   g = exp(-exp(A_log) softplus(W_a xn + dt_bias))                      (one number per head each)
        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q                                 (head h reads q/k head h // (H / G))
        result = W_o ( concat_h (o[h] / rms(o[h])) * w_norm * silu(W_g xn) )

    conv is a causal convolution over time per channel with `taps` taps (zeros before a sequence's start); the last taps - 1
    projected inputs of a sequence are a second record beside S.  Everything after the convolutions' activations is 32-bit.

    params: hidden_size, num_heads, num_qk_heads, dim, vdim, taps, eps (of the heads' norm), unit_eps (default 1e-6),
            q_scale (default dim^-1/2), out_scale (default 1), names (optional: keys q k v gate norm o b a a_log dt_bias conv).
    tensors: <prefix>q [G dim, d], k [G dim, d], v [H vdim, d], g [H vdim, d], o [d, H vdim], b [H, d], a [H, d], A_log [H],
             dt_bias [H], norm [vdim], q.conv [G dim, taps], k.conv [G dim, taps], v.conv [H vdim, taps]."""

    takes_out = True
    _NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "norm": "norm", "o": "o", "b": "b", "a": "a", "a_log": "A_log", "dt_bias": "dt_bias",
              "conv": ".conv"}

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.d = int(self._param("hidden_size"))
        self.H = int(self._param("num_heads"))
        self.G = int(self._param("num_qk_heads"))
        self.dim = int(self._param("dim"))
        self.vdim = int(self._param("vdim"))
        self.taps = int(self._param("taps"))
        self.eps = float(self._param("eps"))
        self.unit_eps = float(spec.params.get("unit_eps", 1e-6))
        if min(self.H, self.G, self.dim, self.vdim) <= 0 or self.H % self.G or self.dim > ops.DELTA_RULE_MAX_DIM or self.vdim > 512:
            raise ConfigError(f"gated_delta: sizes heads={self.H} on {self.G} dim={self.dim} vdim={self.vdim} (heads a multiple of the q/k heads, "
                              f"dim at most {ops.DELTA_RULE_MAX_DIM}, vdim at most 512)")
        if not 1 <= self.taps <= ops.SHORT_CONV_MAX_TAPS:
            raise ConfigError(f"gated_delta: {self.taps} taps (1 to {ops.SHORT_CONV_MAX_TAPS})")
        self.q_scale = float(spec.params.get("q_scale") or self.dim ** -0.5)
        self.out_scale = float(spec.params.get("out_scale", 1.0))
        self.names = dict(self._NAMES, **dict(spec.params.get("names", {})))
        self.qd, self.vd = self.G * self.dim, self.H * self.vdim
        self.channels = 2 * self.qd + self.vd
        self.w_in = self.w_conv = self.a_log = self.dt_bias = self.w_o = self.w_norm = None

    def cache_need(self):
        need = StateNeed((self.H, self.dim, self.vdim), torch.float32)
        if self.taps > 1:  # the convolutions' last inputs: exact in 32-bit whatever the run's type
            return (need, StateNeed((self.taps - 1, self.channels), torch.float32))
        return need

    def param_infos(self) -> Dict[str, ParamInfo]:
        p, n = self.prefix, self.names
        return {
            p + n["q"]: ParamInfo((self.qd, self.d)),
            p + n["k"]: ParamInfo((self.qd, self.d)),
            p + n["v"]: ParamInfo((self.vd, self.d)),
            p + n["gate"]: ParamInfo((self.vd, self.d)),
            p + n["b"]: ParamInfo((self.H, self.d)),
            p + n["a"]: ParamInfo((self.H, self.d)),
            p + n["q"] + n["conv"]: ParamInfo((self.qd, self.taps), "scalars"),
            p + n["k"] + n["conv"]: ParamInfo((self.qd, self.taps), "scalars"),
            p + n["v"] + n["conv"]: ParamInfo((self.vd, self.taps), "scalars"),
            p + n["a_log"]: ParamInfo((self.H,), "scalars", centre=0.0),
            p + n["dt_bias"]: ParamInfo((self.H,), "scalars", centre=0.0),
            p + n["norm"]: ParamInfo((self.vdim,), "scalars", centre=1.0),
            p + n["o"]: ParamInfo((self.d, self.vd)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = self.prefix, self.names
        # one product serves q, k, v, the output gate and the two scalars of every head
        self.w_in = torch.cat([tensors[p + n[key]] for key in ("q", "k", "v", "gate", "b", "a")], dim=0).contiguous()
        # (stored [channels, taps]; the kernel reads [taps, channels], neighbouring channels side by side)
        self.w_conv = torch.cat([tensors[p + n[key] + n["conv"]] for key in ("q", "k", "v")], dim=0).t().contiguous()
        self.a_log, self.dt_bias = tensors[p + n["a_log"]].contiguous(), tensors[p + n["dt_bias"]].contiguous()
        self.w_norm = tensors[p + n["norm"]].contiguous()
        self.w_o = tensors[p + n["o"]].contiguous()

    def forward(self, xn: torch.Tensor, step, cache, shared_cache: bool = False) -> torch.Tensor:
        a, w_o = self.forward_unprojected(xn, step, cache, shared_cache)
        return linear_to_stream(a, w_o)

    def forward_unprojected(self, xn: torch.Tensor, step, cache, shared_cache: bool = False, out=None):
        if shared_cache:
            raise ConfigError("gated_delta: a state cannot be another run's")
        memory, inputs = cache if self.taps > 1 else (cache, None)
        proj = linear(xn, self.w_in)
        C, vd, H = self.channels, self.vd, self.H
        conv = ops.short_conv(proj[:, :C], self.w_conv, None if inputs is None else inputs.state, step.slot_ids, step.seq_start, step.tok_seq)
        gate, ba = proj[:, C : C + vd], proj[:, C + vd : C + vd + 2 * H]
        qn, kn, kq, beta, decay = ops.delta_prep(conv[:, : 2 * self.qd], ba, self.a_log, self.dt_bias, self.G, H, self.dim, self.unit_eps, self.q_scale)
        o = ops.delta_rule(qn, kn, kq, conv[:, 2 * self.qd :], beta, decay, memory.state, step.slot_ids, step.seq_start, H, self.G, self.dim, self.vdim)
        a = ops.head_norm_gate(o, H, self.vdim, self.w_norm, self.eps, gate, ops.GATE_SILU, xn.dtype, out_scale=self.out_scale, out=out)
        return a, self.w_o
