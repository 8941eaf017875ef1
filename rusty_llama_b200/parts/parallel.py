"""A mixer made of several mixers that read the same input side by side."""

from __future__ import annotations

from typing import Mapping

import torch

from ..errors import ConfigError
from ..kernels.linear import linear_to_stream
from ..spec import PartSpec
from .base import MIXERS, Mixer, NormedTerms, ParamInfo


@MIXERS.register("parallel")
class ParallelMixers(Mixer):
    """result = sum_i scale_i * branch_i(xn).

    Every branch is a mixer that ends in a projection and can leave it to the caller (`forward_unprojected`).  The branches
    write what their projections would read into one row, side by side, and ONE product with the projections' matrices side
    by side makes the sum: no branch's result is stored or added on its own.  A branch's scale is handed to it as its
    `out_scale`, so it is applied in 32-bit where the branch forms its last values; biases of the branches' projections
    are summed into one row (`output_bias`).  Each branch keeps the cache storage it asks for; this mixer's need is the
    tuple of theirs.

    With `branch_norms` the result is sum_i scale_i * rmsnorm(branch_i(xn)) * w_i instead: every branch's projected result
    goes through an RMS norm of its own over the model's width before the sum.  The branches are then projected one by one and
    handed to the residual stream as `NormedTerms`, scale_i folded into w_i (32-bit), so the norms run inside the kernels that
    add to the stream and no branch's normed result is stored.

    params: branches: a list of (PartSpec, scale); a branch's prefix is relative to this mixer's.
            branch_norms (optional): {"names": one tensor name per branch, relative to this mixer's prefix, "eps": ..., "size": the model's width}."""

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        branches = self._param("branches")
        if not branches:
            raise ConfigError("parallel: no branches")
        self.branches = []
        self.norms = spec.params.get("branch_norms")
        for b, scale in branches:
            if not isinstance(b, PartSpec):
                raise ConfigError("parallel: a branch must be a PartSpec")
            cls = MIXERS.get(b.kind)
            if not getattr(cls, "takes_out", False):
                raise ConfigError(f"parallel: mixer '{b.kind}' cannot leave its last projection to the caller")
            params = dict(b.params)
            if self.norms is None:  # (with norms of their own the scale goes into the norm's weight: a norm undoes a factor before it)
                params["out_scale"] = float(params.get("out_scale", 1.0)) * float(scale)
            self.branches.append(MIXERS.build(PartSpec(b.kind, params, self.prefix + b.prefix), runtime))
        self._needs = [b.cache_need() for b in self.branches]
        self.w_o = None
        self.bias = None
        self._scales = [float(scale) for _, scale in branches]
        self.norm_weights = None
        if self.norms is not None and len(self.norms["names"]) != len(self.branches):
            raise ConfigError("parallel: branch_norms names one tensor per branch")

    def param_infos(self):
        if self.norms is None:
            return {}
        return {self.prefix + name: ParamInfo((int(self.norms["size"]),), "scalars", centre=1.0) for name in self.norms["names"]}

    def children(self):
        return tuple(self.branches)

    def cache_need(self):
        # (a branch may itself name several pieces of storage: they follow each other in this mixer's tuple)
        needs = tuple(n for need in self._needs if need is not None for n in (need if isinstance(need, (tuple, list)) else (need,)))
        return needs or None

    def _views(self, cache):
        """Each branch's share of this mixer's views, in the form the branch asked for."""
        views = list(cache) if isinstance(cache, (tuple, list)) else [cache]
        out = []
        for need in self._needs:
            if need is None:
                out.append(None)
            elif isinstance(need, (tuple, list)):
                out.append(tuple(views.pop(0) for _ in need))
            else:
                out.append(views.pop(0))
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        # children are loaded by the model after this part; their matrices are put side by side at the first step
        self.w_o = None
        if self.norms is not None:
            self.norm_weights = [(tensors[self.prefix + name].to(torch.float32) * scale).contiguous()
                                 for name, scale in zip(self.norms["names"], self._scales)]

    def output_bias(self):
        return None if self.norms is not None else self.bias

    def _assemble(self) -> None:
        self.w_o = torch.cat([b.w_o for b in self.branches], dim=1).contiguous()
        rows = [b.output_bias() for b in self.branches]
        rows = [r for r in rows if r is not None]
        self.bias = None if not rows else torch.stack(rows).sum(dim=0).contiguous()

    def forward(self, xn: torch.Tensor, step, cache, shared_cache: bool = False) -> torch.Tensor:
        if shared_cache:
            raise ConfigError("parallel: its branches fill caches of their own")
        views = self._views(cache)
        if self.norms is not None:
            terms = NormedTerms()
            for b, view, w in zip(self.branches, views, self.norm_weights):
                if b.output_bias() is not None:
                    raise ConfigError("parallel: a branch with an output bias cannot go through a norm of its own here")
                a, w_o = b.forward_unprojected(xn, step, view, False)
                terms.append((linear_to_stream(a, w_o), (w, float(self.norms["eps"]))))
            return terms
        if self.w_o is None:
            self._assemble()
        T = xn.shape[0]
        a = torch.empty((T, self.w_o.shape[1]), dtype=xn.dtype, device=xn.device)
        at = 0
        for b, view in zip(self.branches, views):
            k = b.w_o.shape[1]
            b.forward_unprojected(xn, step, view, False, out=a[:, at : at + k])
            at += k
        return linear_to_stream(a, self.w_o)
