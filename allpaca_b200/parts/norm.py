"""RMSNorm fused with the residual addition that precedes it.

``ss = sum x^2; inv = 1/sqrt(ss/n + eps); out = x * inv * w`` — eps inside the root,
weight multiplied last, no ``+1`` (crates/allpaca-cpu/src/kernels.rs:492-507; CUDA
cuda/src/kernels.cu:1152-1175).  The sum is 32-bit whatever the storage type.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import ops
from .base import BuildEnv, Norm, WeightSpec, register


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    """Parameters: ``size`` (width of a row), ``eps``, ``scalar_weight`` (False; True: the
    checkpoint holds one number for all coordinates, a tensor without dimensions), ``weight_name``
    (``"weight"``: the tensor's name behind the part's prefix; may be empty, the prefix then is
    the whole name)."""

    def __init__(self, params, env: BuildEnv):
        super().__init__(params, env)
        self.require("size", "eps")
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.scalar_weight = bool(params.get("scalar_weight", False))
        self.weight_name = str(params.get("weight_name", "weight"))
        self.weight = None
        self._kernel_weight = None

    def weights(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec(() if self.scalar_weight else (self.size,), "norm")}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = tensors[self.weight_name]
        # one number for all coordinates: the kernels take it as a vector of equal entries
        self.weight = (w.reshape(1).expand(self.size) if self.scalar_weight else w).contiguous()
        self._kernel_weight = self.weight

    def fold(self) -> None:
        """The weight has been multiplied into the product that consumes this norm's output:
        from now on the kernel only divides by the root mean square."""
        self._kernel_weight = torch.ones_like(self.weight)

    @property
    def folded(self) -> bool:
        return self._kernel_weight is not self.weight

    def forward(self, x, out, delta=None, rows=None) -> None:
        ops.add_rmsnorm(x, self._kernel_weight, self.eps, out, delta=delta, rows=rows)

    def add_normed(self, x, delta, mult: float, copy=None) -> None:
        """The norm on a sublayer's output: ``x += mult * norm(delta)``; ``copy`` (optional) receives
        the updated rows in its own type."""
        ops.norm_residual(x, delta, self.weight, self.eps, mult, copy)
