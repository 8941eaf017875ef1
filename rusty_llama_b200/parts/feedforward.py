"""Dense feed-forward parts."""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..errors import ConfigError
from ..kernels import ops
from ..kernels.linear import linear, linear_swiglu, linear_to_stream
from .base import FEED_FORWARDS, FeedForward, ParamInfo


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    """f = W_down (act(W_gate x) * (W_up x)) with act = silu: Llama's SwiGLU
    (src/model.rs:1336-1345, src/backend/cpu.rs:435-440).

    activation "clamped_swish" (params `limit`, `alpha`): f = W_down (g s(alpha g) (u + 1)) with g = min(W_gate x, limit),
    u = clamp(W_up x, -limit, limit), s the logistic function; in bfloat16 the product's kernel applies it as it does silu,
    in 32-bit a kernel of its own.  activation "gelu_tanh": act(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), in the same places.

    params: hidden_size, intermediate_size, activation ("silu", "clamped_swish" or "gelu_tanh"),
            names (optional: the three tensors' names after the prefix, keys gate up down).
    tensors: <prefix>gate_proj.weight [ff, d], up_proj.weight [ff, d], down_proj.weight [d, ff].
    gate and up are kept as one [2 ff, d] matrix so that one product serves both, the
    counterpart of the reference's `matmul_shared` (src/backend/mod.rs:44-56).  In bfloat16 their
    rows alternate (gate i, up i, gate i+1, ...), which lets the product's kernel apply the
    activation to its 32-bit sums and write h directly; in 32-bit the halves follow each other
    and a separate kernel applies the activation."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.d = int(self._param("hidden_size"))
        self.ff = int(self._param("intermediate_size"))
        self.activation = self._param("activation")
        if self.activation not in ("silu", "clamped_swish", "gelu_tanh"):
            raise ConfigError(f"gated_mlp: activation '{self.activation}' is not built (only 'silu', 'clamped_swish' and 'gelu_tanh')")
        self.act = None  # what the products' kernels are told: None is silu(gate) * up
        if self.activation == "clamped_swish":
            self.limit, self.alpha = float(self._param("limit")), float(self._param("alpha"))
            self.act = (self.alpha, self.limit)
        elif self.activation == "gelu_tanh":
            self.act = "gelu_tanh"
        self.names = dict({"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}, **dict(spec.params.get("names", {})))
        self.w_gate_up = None
        self.w_down = None

    def param_infos(self) -> Dict[str, ParamInfo]:
        p = self.prefix
        return {
            p + self.names["gate"]: ParamInfo((self.ff, self.d)),
            p + self.names["up"]: ParamInfo((self.ff, self.d)),
            p + self.names["down"]: ParamInfo((self.d, self.ff)),
        }

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        gate, up = tensors[p + self.names["gate"]], tensors[p + self.names["up"]]
        self.fused = self.rt.dtype == torch.bfloat16
        if self.fused:
            self.w_gate_up = torch.stack([gate, up], dim=1).reshape(2 * self.ff, self.d).contiguous()
        else:
            self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = tensors[p + self.names["down"]].contiguous()

    def gated_weights(self):
        return (self.w_gate_up, self.w_down) if (self.fused and self.activation == "silu") else None

    def forward(self, xn: torch.Tensor, step) -> torch.Tensor:
        if self.fused:
            h = linear_swiglu(xn, self.w_gate_up, act=self.act)
        elif self.act is not None:
            h = ops.gated_glu(linear(xn, self.w_gate_up), self.act)
        else:
            h = ops.swiglu(linear(xn, self.w_gate_up))
        return linear_to_stream(h, self.w_down)


@FEED_FORWARDS.register("mlp")
class MLP(FeedForward):
    """f = W_down act(W_up x), no gate.  act "relu2": the square of relu, applied in 32-bit, in bfloat16 runs to the up product's
    32-bit sums in its kernel's epilogue.

    params: hidden_size, intermediate_size, activation ("relu2"), names (optional: keys up down).
    tensors: <prefix>up_proj.weight [ff, d], down_proj.weight [d, ff]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.d = int(self._param("hidden_size"))
        self.ff = int(self._param("intermediate_size"))
        self.activation = self._param("activation")
        if self.activation != "relu2":
            raise ConfigError(f"mlp: activation '{self.activation}' is not built (only 'relu2')")
        self.names = dict({"up": "up_proj.weight", "down": "down_proj.weight"}, **dict(spec.params.get("names", {})))
        self.w_up = self.w_down = None

    def param_infos(self) -> Dict[str, ParamInfo]:
        p = self.prefix
        return {p + self.names["up"]: ParamInfo((self.ff, self.d)), p + self.names["down"]: ParamInfo((self.d, self.ff))}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        self.w_up = tensors[p + self.names["up"]].contiguous()
        self.w_down = tensors[p + self.names["down"]].contiguous()

    def forward(self, xn: torch.Tensor, step) -> torch.Tensor:
        # (the streaming and the tcgen05 product apply the activation to their 32-bit sums; behind the others it is a pass of its own)
        return linear_to_stream(linear(xn, self.w_up, act=self.activation), self.w_down)
