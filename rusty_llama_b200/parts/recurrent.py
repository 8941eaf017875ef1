"""Mixers whose memory is a fixed-size state per sequence: linear attention with a decay, and a minimal gated recurrent unit.

Both keep their state in 32-bit in the cache's state records (`StateNeed`), one record per sequence slot, zero when the
sequence starts; a step runs each sequence's tokens through its record in order, whether the step brings a whole prompt,
a part of one or a single token.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..errors import ConfigError
from ..kernels import ops
from ..kernels.linear import linear, linear_to_stream
from .base import MIXERS, POSITIONS, Mixer, ParamInfo, StateNeed


# prompt steps whose longest sequence brings fewer tokens than this go token by token like a decode step
_CHUNKED_MIN_TOKENS = 32


@MIXERS.register("decay_linear_attention")
class DecayLinearAttention(Mixer):
    """Linear attention with a constant decay per head:

        q = act(W_q xn), k = act(W_k xn)  [H, dim];   v = act(W_v xn)  [H, vdim]
        S_t = decay_h S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t            (per head; no other scale)
        result = W_o ( rmsnorm(concat_h o_t) * w_norm * sigmoid(W_g xn) )

    The norm runs over all heads together.  The recurrence, the norm and the gate are 32-bit; the state [H, dim, vdim] is a
    32-bit record per sequence.

    Options: `position` (a PartSpec of a rotary position encoding: q and k are turned by their positions before the recurrence,
    v is not), `k_scale` (a constant on k; o is linear in k, so it reaches o as one factor, and since o only ever goes through
    the norm it is applied there, exactly, as eps / k_scale^2 in the place of eps: the state holds S / k_scale), `head_norm` (every
    head's o is normed on its own over its vdim values), `norm_weight` (False: the norm has no weight and no tensor), `gate_act`
    ("sigmoid" or "silu").

    params: hidden_size, num_heads, dim, vdim, decay (one number per head), eps (of the norm), activation ("silu" or "none"),
            gate (bool, default True), out_scale (default 1), position, k_scale, head_norm, norm_weight, gate_act,
            names (optional: keys q k v gate norm o).
    tensors: <prefix>q [H dim, d], k [H dim, d], v [H vdim, d], g [H vdim, d], norm [H vdim] ([vdim] with head_norm), o [d, H vdim]."""

    takes_out = True
    _NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "norm": "norm", "o": "o"}

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.d = int(self._param("hidden_size"))
        self.H = int(self._param("num_heads"))
        self.dim = int(self._param("dim"))
        self.vdim = int(self._param("vdim"))
        self.eps = float(self._param("eps"))
        decay = [float(x) for x in self._param("decay")]
        if len(decay) != self.H:
            raise ConfigError(f"decay_linear_attention: {len(decay)} decays for {self.H} heads")
        if min(self.H, self.dim, self.vdim) <= 0 or self.dim > 1024:
            raise ConfigError(f"decay_linear_attention: sizes heads={self.H} dim={self.dim} vdim={self.vdim} (dim at most 1024)")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=runtime.device)
        act = spec.params.get("activation", "silu")
        if act not in ("silu", "none"):
            raise ConfigError(f"decay_linear_attention: activation '{act}' is not built (only 'silu' and 'none')")
        self.silu = act == "silu"
        self.has_gate = bool(spec.params.get("gate", True))
        self.out_scale = float(spec.params.get("out_scale", 1.0))
        self.names = dict(self._NAMES, **dict(spec.params.get("names", {})))
        self.qd, self.vd = self.H * self.dim, self.H * self.vdim
        self.w_in = self.w_o = self.w_norm = None
        self.head_norm = bool(spec.params.get("head_norm", False))
        self.norm_weight = bool(spec.params.get("norm_weight", True))
        gate_act = spec.params.get("gate_act", "sigmoid")
        if gate_act not in ("sigmoid", "silu"):
            raise ConfigError(f"decay_linear_attention: gate_act '{gate_act}' is not built (only 'sigmoid' and 'silu')")
        self.gate_silu = gate_act == "silu"
        if (self.gate_silu or not self.norm_weight) and not self.head_norm:
            raise ConfigError("decay_linear_attention: a silu gate and a norm without weight are built for head_norm only")
        k_scale = float(spec.params.get("k_scale", 1.0))
        if not k_scale > 0:
            raise ConfigError(f"decay_linear_attention: k_scale = {k_scale} must be positive")
        self.norm_eps = self.eps / (k_scale * k_scale)
        self.position = None
        pos_spec = spec.params.get("position")
        if pos_spec is not None and pos_spec.kind != "none":
            self.position = POSITIONS.build(pos_spec, runtime)
            if not hasattr(self.position, "inv_freq") or float(getattr(self.position, "magnitude", 1.0)) != 1.0:
                raise ConfigError("decay_linear_attention: the position part must be a 'rotary' one without a magnitude factor")
            if int(self.position.rotary_dim) > self.dim:
                raise ConfigError(f"decay_linear_attention: {self.position.rotary_dim} rotated numbers do not fit a head of {self.dim}")

    def cache_need(self):
        return StateNeed((self.H, self.dim, self.vdim), torch.float32)

    def children(self):
        return () if self.position is None else (self.position,)

    def param_infos(self) -> Dict[str, ParamInfo]:
        p, n = self.prefix, self.names
        infos = {
            p + n["q"]: ParamInfo((self.qd, self.d)),
            p + n["k"]: ParamInfo((self.qd, self.d)),
            p + n["v"]: ParamInfo((self.vd, self.d)),
            p + n["o"]: ParamInfo((self.d, self.vd)),
        }
        if self.norm_weight:
            infos[p + n["norm"]] = ParamInfo((self.vdim if self.head_norm else self.vd,), "scalars", centre=1.0)
        if self.has_gate:
            infos[p + n["gate"]] = ParamInfo((self.vd, self.d))
        return infos

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = self.prefix, self.names
        parts = [tensors[p + n["q"]], tensors[p + n["k"]], tensors[p + n["v"]]]
        if self.has_gate:
            parts.append(tensors[p + n["gate"]])
        self.w_in = torch.cat(parts, dim=0).contiguous()  # one product serves q, k, v and the gate
        self.w_norm = tensors[p + n["norm"]].contiguous() if self.norm_weight else None
        self.w_o = tensors[p + n["o"]].contiguous()

    def forward(self, xn: torch.Tensor, step, cache, shared_cache: bool = False) -> torch.Tensor:
        a, w_o = self.forward_unprojected(xn, step, cache, shared_cache)
        return linear_to_stream(a, w_o)

    def forward_unprojected(self, xn: torch.Tensor, step, cache, shared_cache: bool = False, out=None):
        if shared_cache:
            raise ConfigError("decay_linear_attention: a state cannot be another run's")
        proj = linear(xn, self.w_in)
        if self.position is not None and self.position.rotary_dim:
            # q and k lie side by side at the start of the rows: 2 H heads turned in place, nothing stored anywhere else
            ops.rope_kv_write(proj, step.tok_pos, step.tok_seq, None, None, None, self.position.inv_freq, 2 * self.H, 0, self.dim,
                              self.position.rotary_dim, self.position.interleaved, write_kv=False)
        q, k = proj[:, : self.qd], proj[:, self.qd : 2 * self.qd]
        v = proj[:, 2 * self.qd : 2 * self.qd + self.vd]
        gate = proj[:, 2 * self.qd + self.vd :] if self.has_gate else None
        # a prompt step of a bfloat16 run works its sequences chunk by chunk, all chunks at once; 32-bit runs and single
        # tokens go token by token (the same bits however a sequence is cut into steps)
        chunked = xn.dtype == torch.bfloat16 and step.max_q_len >= _CHUNKED_MIN_TOKENS and self.dim <= ops.DECAY_CHUNKED_MAX_DIM
        scratch = None
        if chunked:
            need = ops.decay_attn_chunked_scratch_floats(step.n_seqs, step.max_q_len, self.H, self.dim, self.vdim)
            scratch = self.rt.workspace.get("decay_attn_chunks", need, torch.float32)
        o = ops.decay_attn(
            q, k, v, self.decay, cache.state, step.slot_ids, step.seq_start, self.H, self.dim, self.vdim, silu=self.silu,
            max_q_len=step.max_q_len if chunked else 0, scratch=scratch,
        )
        if self.head_norm:
            a = ops.head_norm_gate(o, self.H, self.vdim, self.w_norm, self.norm_eps, gate, ops.GATE_SILU if self.gate_silu else ops.GATE_SIGMOID,
                                   xn.dtype, out_scale=self.out_scale, out=out)
        else:
            a = ops.rms_gate(o, self.w_norm, self.norm_eps, gate, xn.dtype, out_scale=self.out_scale, out=out)
        return a, self.w_o


@MIXERS.register("min_gru")
class MinGRU(Mixer):
    """A gated recurrence whose gates read the current token only, element by element over `width` channels:

        z = sigmoid(W_z xn + b_z),  u = W_x xn + b_x,  c = u + 1/2 where u >= 0, else sigmoid(u)
        S_t = (1 - z_t) S_(t-1) + z_t c_t,   result = W_o ( S_t * silu(W_g xn) )

    Gates, candidate and state are 32-bit; the state [width] is a 32-bit record per sequence.

    params: hidden_size, width, bias (bool, default True: z and x have biases), out_scale (default 1),
            names (optional: keys z x gate o z_bias x_bias).
    tensors: <prefix>z [width, d], x [width, d], g [width, d], o [d, width], z.b [width], x.b [width]."""

    takes_out = True
    _NAMES = {"z": "z", "x": "x", "gate": "g", "o": "o", "z_bias": "z.b", "x_bias": "x.b"}

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.d = int(self._param("hidden_size"))
        self.width = int(self._param("width"))
        if self.width <= 0:
            raise ConfigError(f"min_gru: width {self.width}")
        self.has_bias = bool(spec.params.get("bias", True))
        self.out_scale = float(spec.params.get("out_scale", 1.0))
        self.names = dict(self._NAMES, **dict(spec.params.get("names", {})))
        self.w_in = self.w_o = self.b_z = self.b_x = None

    def cache_need(self):
        return StateNeed((self.width,), torch.float32)

    def param_infos(self) -> Dict[str, ParamInfo]:
        p, n = self.prefix, self.names
        infos = {p + n[key]: ParamInfo((self.width, self.d)) for key in ("z", "x", "gate")}
        infos[p + n["o"]] = ParamInfo((self.d, self.width))
        if self.has_bias:
            infos[p + n["z_bias"]] = ParamInfo((self.width,), "scalars", centre=0.0)
            infos[p + n["x_bias"]] = ParamInfo((self.width,), "scalars", centre=0.0)
        return infos

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p, n = self.prefix, self.names
        self.w_in = torch.cat([tensors[p + n["z"]], tensors[p + n["x"]], tensors[p + n["gate"]]], dim=0).contiguous()
        self.w_o = tensors[p + n["o"]].contiguous()
        if self.has_bias:
            self.b_z, self.b_x = tensors[p + n["z_bias"]].contiguous(), tensors[p + n["x_bias"]].contiguous()

    def forward(self, xn: torch.Tensor, step, cache, shared_cache: bool = False) -> torch.Tensor:
        a, w_o = self.forward_unprojected(xn, step, cache, shared_cache)
        return linear_to_stream(a, w_o)

    def forward_unprojected(self, xn: torch.Tensor, step, cache, shared_cache: bool = False, out=None):
        if shared_cache:
            raise ConfigError("min_gru: a state cannot be another run's")
        proj = linear(xn, self.w_in)
        w = self.width
        a = ops.min_gru(
            proj[:, :w], proj[:, w : 2 * w], proj[:, 2 * w :], self.b_z, self.b_x, cache.state, step.slot_ids, step.seq_start,
            out_scale=self.out_scale, out=out, max_q_len=step.max_q_len if xn.dtype == torch.bfloat16 else 0,
        )
        return a, self.w_o
