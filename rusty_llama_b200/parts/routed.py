"""A feed-forward that sends each token to a few of many small gated feed-forwards."""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..errors import ConfigError
from ..kernels import ops
from ..kernels.linear import linear, linear_swiglu
from .base import FEED_FORWARDS, FeedForward, ParamInfo

_NAMES = {
    "expert": "e{}.", "gate": "gate", "up": "up", "down": "down", "router": "router", "bias": "correction",
    "shared": "shared.", "shared_gate": "shared.sg", "table": "table",
}


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """E experts f_e(x) = W_down[e] (silu(W_gate[e] x) * (W_up[e] x)); every token uses `top` of them.

        s = softmax(W_r x) over all experts, in 32-bit
        chosen = the `top` experts with the largest s + bias (the bias only chooses)
        y = sum over chosen e of s_e f_e(x)            (s_e / sum of the chosen s if `renormalize`)
          + sigmoid(w_sg . x) * f_shared(x)            (if there is a shared expert; without w_sg it is added as it is)

    router "sigmoid": s = logistic(W_r x), every expert's score on its own; `renorm_eps` joins the sum that `renormalize` divides
    by, and `weight_scale` multiplies the weights (both also with the softmax router; defaults 0 and 1).

    router "table" instead: no scores at all; a table [vocab, top] of expert ids gives every token id its experts (the entries
    of a row differ), and each chosen expert has the weight 1 / top.

    activation "clamped_swish" (params `limit`, `alpha`): f_e(x) = W_down[e] (g s(alpha g) (u + 1)) with g = min(W_gate[e] x, limit),
    u = clamp(W_up[e] x, -limit, limit), s the logistic function, in the place of silu(g) * u.

    params: hidden_size, n_experts, top, expert_ff, bias (bool), renormalize (bool),
            shared_ff (0: none), shared_gate (bool), router ("softmax", "sigmoid" or "table"; with "table" also vocab_size), renorm_eps,
            weight_scale, activation
            ("silu" or "clamped_swish"), names (optional).
    tensors: <prefix>e<i>.gate [ff, d], e<i>.up [ff, d], e<i>.down [d, ff], router [E, d] (or table [vocab, top]), correction [E],
             shared.gate / shared.up / shared.down, shared.sg [1, d]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.d = int(self._param("hidden_size"))
        self.E = int(self._param("n_experts"))
        self.top = int(self._param("top"))
        self.ff = int(self._param("expert_ff"))
        self.has_bias = bool(spec.params.get("bias", False))
        self.renormalize = bool(spec.params.get("renormalize", False))
        self.shared_ff = int(spec.params.get("shared_ff", 0))
        self.shared_gate = bool(spec.params.get("shared_gate", False)) and self.shared_ff > 0
        self.names = dict(_NAMES, **dict(spec.params.get("names", {})))
        self.router = spec.params.get("router", "softmax")
        if self.router not in ("softmax", "sigmoid", "table"):
            raise ConfigError(f"routed_experts: router '{self.router}' is not built (known: softmax, sigmoid, table)")
        self.renorm_eps = float(spec.params.get("renorm_eps", 0.0))
        self.weight_scale = float(spec.params.get("weight_scale", 1.0))
        if self.router == "table":
            self.vocab = int(self._param("vocab_size"))
            if self.has_bias or self.renormalize or self.shared_gate:
                raise ConfigError("routed_experts: a table chooses without scores; bias, renormalize and a gated shared expert need a router")
        activation = spec.params.get("activation", "silu")
        if activation not in ("silu", "clamped_swish"):
            raise ConfigError(f"routed_experts: activation '{activation}' is not built (only 'silu' and 'clamped_swish')")
        self.act = (float(self._param("alpha")), float(self._param("limit"))) if activation == "clamped_swish" else None
        if not 0 < self.top <= self.E:
            raise ConfigError(f"routed_experts: {self.top} of {self.E} experts per token")
        if self.ff <= 0:
            raise ConfigError(f"routed_experts: expert size {self.ff}")

    def _expert(self, i: int, which: str) -> str:
        return self.prefix + self.names["expert"].format(i) + self.names[which]

    def _shared(self, which: str) -> str:
        return self.prefix + self.names["shared"] + self.names[which]

    def param_infos(self) -> Dict[str, ParamInfo]:
        infos = {}
        for i in range(self.E):
            infos[self._expert(i, "gate")] = ParamInfo((self.ff, self.d))
            infos[self._expert(i, "up")] = ParamInfo((self.ff, self.d))
            infos[self._expert(i, "down")] = ParamInfo((self.d, self.ff))
        if self.router == "table":
            infos[self.prefix + self.names["table"]] = ParamInfo((self.vocab, self.top), "table", upper=self.E)
        else:
            infos[self.prefix + self.names["router"]] = ParamInfo((self.E, self.d), "scalars")
        if self.has_bias:
            infos[self.prefix + self.names["bias"]] = ParamInfo((self.E,), "scalars")
        if self.shared_ff:
            infos[self._shared("gate")] = ParamInfo((self.shared_ff, self.d))
            infos[self._shared("up")] = ParamInfo((self.shared_ff, self.d))
            infos[self._shared("down")] = ParamInfo((self.d, self.shared_ff))
        if self.shared_gate:
            infos[self.prefix + self.names["shared_gate"]] = ParamInfo((1, self.d), "scalars")
        return infos

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        stack = lambda which: torch.stack([tensors[self._expert(i, which)] for i in range(self.E)], dim=0).contiguous()  # noqa: E731
        self.w_gate, self.w_up, self.w_down = stack("gate"), stack("up"), stack("down")
        if self.router == "table":
            self.table = tensors[self.prefix + self.names["table"]].contiguous()
            if self.table.numel() and (int(self.table.min()) < 0 or int(self.table.max()) >= self.E):
                raise ConfigError(f"routed_experts: '{self.prefix + self.names['table']}' names experts outside 0 .. {self.E - 1}")
        else:
            rows = [tensors[self.prefix + self.names["router"]]]
            if self.shared_gate:
                rows.append(tensors[self.prefix + self.names["shared_gate"]])  # one more row of the router's product
            self.w_router = torch.cat(rows, dim=0).contiguous()
        self.bias = tensors[self.prefix + self.names["bias"]].contiguous() if self.has_bias else None
        if self.shared_ff:
            gate, up = tensors[self._shared("gate")], tensors[self._shared("up")]
            self.shared_fused = self.rt.dtype == torch.bfloat16
            if self.shared_fused:  # gate and up rows alternate: the product's kernel applies the activation (see GatedMLP)
                self.ws_gate_up = torch.stack([gate, up], dim=1).reshape(2 * self.shared_ff, self.d).contiguous()
            else:
                self.ws_gate_up = torch.cat([gate, up], dim=0).contiguous()
            self.ws_down = tensors[self._shared("down")].contiguous()

    def forward(self, xn: torch.Tensor, step) -> torch.Tensor:
        T = xn.shape[0]
        if self.router == "table":
            ids, weights = ops.moe_table_lookup(step.tokens, self.table, self.E)
            gate = None
        else:
            ids, weights, gate = ops.moe_router(xn, self.w_router, self.bias, self.E, self.top, self.renormalize,
                                                logistic=self.router == "sigmoid", renorm_eps=self.renorm_eps, weight_scale=self.weight_scale)
        # the height of a row tile: 128 once the experts get that many rows on average (a prompt step), else 32; the plain
        # kernels of a 32-bit run have their own
        tile_rows = 0
        if xn.dtype == torch.bfloat16 and self.d % 8 == 0 and self.ff % 8 == 0:  # (else the plain products, 16-byte rows or not)
            tile_rows = 128 if T * self.top >= 64 * self.E else 32
        order, place, tiles, max_tiles = ops.moe_plan(ids, self.E, tile_rows)
        h = ops.moe_gemm(xn, self.w_gate, tiles, max_tiles, T * self.top, order=order, gather_div=self.top, w2=self.w_up, tile_rows=tile_rows, act=self.act)
        y = ops.moe_gemm(h, self.w_down, tiles, max_tiles, T * self.top, out_dtype=torch.float32, tile_rows=tile_rows)
        shared = None
        if self.shared_ff:
            if self.shared_fused:
                hs = linear_swiglu(xn, self.ws_gate_up, act=self.act)
            elif self.act is not None:
                hs = ops.clamped_glu(linear(xn, self.ws_gate_up), self.act[0], self.act[1])
            else:
                hs = ops.swiglu(linear(xn, self.ws_gate_up))
            shared = linear(hs, self.ws_down)
        return ops.moe_combine(y, place, weights, shared, gate)
