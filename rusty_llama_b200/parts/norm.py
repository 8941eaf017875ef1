"""RMSNorm, fused with the residual sum that precedes it."""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from ..kernels import ops
from .base import NORMS, Norm, ParamInfo, ResidualStream


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * weight (src/backend/cpu.rs:96-105).

    params: size, eps, name (optional: the tensor's name after the prefix, "weight" if absent), offset (optional, default 0:
    the stored tensor is the weight's distance from `offset`, y = ... * (offset + w); such a weight is kept in 32-bit whatever
    the run's type, since offset + w has more digits than w), float32 (optional bool: the weight is kept in 32-bit in every run,
    for designs whose norms are 32-bit arithmetic throughout).  tensor: <prefix>weight [size]."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.size = int(self._param("size"))
        self.eps = float(self._param("eps"))
        self.offset = float(spec.params.get("offset", 0.0))
        self.keep32 = bool(spec.params.get("float32", False))
        self.tensor_name = self.prefix + str(spec.params.get("name", "weight"))
        self.weight: Optional[torch.Tensor] = None

    def param_infos(self) -> Dict[str, ParamInfo]:
        if self.offset:
            return {self.tensor_name: ParamInfo((self.size,), "scalars", centre=0.0)}
        if self.keep32:
            return {self.tensor_name: ParamInfo((self.size,), "scalars", centre=1.0)}
        return {self.tensor_name: ParamInfo((self.size,), "vector")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors[self.tensor_name]
        if self.offset:
            self.weight = (self.weight.to(torch.float32) + self.offset).contiguous()

    def rms_weight(self):
        return self.weight, self.eps

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        delta, delta_norm = stream.take_pending()
        if delta_norm is not None:
            return ops.normed_add_rmsnorm(
                stream.x, delta, delta_norm[0], delta_norm[1], self.weight, self.eps, stream.act_dtype, rows=rows, write_x=rows is None,
                delta_bias=delta_norm[2],
            )
        return ops.add_rmsnorm(
            stream.x, delta, self.weight, self.eps, stream.act_dtype, rows=rows, write_x=rows is None
        )
