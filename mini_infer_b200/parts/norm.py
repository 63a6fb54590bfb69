"""RMSNorm, fused with the residual addition that precedes it.

Reference: ``y = x * rsqrt(mean(x^2) + eps) * w`` in src/kernels/rmsnorm_kernel.cu:43-64,
the residual addition as a separate kernel (src/kernels/model_utils_kernel.cu:31-42).
"""

from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import register_part
from ..ops import functional as F
from .base import Deferred, Norm, Runtime, TensorDecl, WeightedRowSum, split_sum


class RMSNorm(Norm):
    """params: ``size``, ``eps``, optional ``tensor`` (the tensor's name below the prefix, default ``weight``)
    and ``one_plus`` (the checkpoint holds the gain's offset from one: ``y = x * rsqrt(mean(x^2) + eps) *
    (1 + w)``; the sum is formed once, in float32, when the weights are loaded).
    Tensor: ``<prefix><tensor> [size]``."""

    graph_safe = True
    accepts_deferred = True
    kernel_files = ("elementwise.cu",)

    def _name(self) -> str:
        return self.prefix + self.params.get("tensor", "weight")

    def tensor_decls(self) -> List[TensorDecl]:
        role = "norm_offset" if self.params.get("one_plus") else "norm"
        return [TensorDecl(self._name(), (self.params["size"],), role)]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.eps = float(self.params["eps"])
        if self.params.get("one_plus"):
            self.weight = (tensors[self._name()].to(device=rt.device, dtype=torch.float32) + 1.0).contiguous()
        else:
            self.weight = rt.precision.small(tensors[self._name()], rt.device)

    def rms_parameters(self):
        return self.weight, self.eps

    def apply(self, hidden: torch.Tensor, delta: Optional[torch.Tensor],
              rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if isinstance(delta, WeightedRowSum):
            # the sum is formed row by row inside the norm's kernel and never written out
            return F.combine_add_rmsnorm(hidden, delta.rows, delta.index, delta.weights, delta.extra, delta.scale,
                                         self.weight, self.eps, self.rt.act, rows)
        if isinstance(delta, Deferred):
            delta = delta.materialize()
        return F.add_rmsnorm(hidden, delta, self.weight, self.eps, self.rt.act, rows)


class ScalarRMSNorm(Norm):
    """``x / sqrt(mean(x^2) + eps) * g`` with ONE number ``g`` for all coordinates.  params: ``eps``, optional
    ``tensor`` (the tensor's name below the prefix, default ``weight``).  Tensor: ``<prefix><tensor> []``."""

    graph_safe = True
    accepts_deferred = True
    kernel_files = ("residual_forms.cu",)

    def _name(self) -> str:
        return self.prefix + self.params.get("tensor", "weight")

    def tensor_decls(self) -> List[TensorDecl]:
        return [TensorDecl(self._name(), (), "norm")]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.eps = float(self.params["eps"])
        self.scalar_gain = tensors[self._name()].to(device=rt.device, dtype=torch.float32).reshape(1).contiguous()

    def apply(self, hidden: torch.Tensor, delta, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        a, b = split_sum(delta)
        return F.add2_rmsnorm_scalar(hidden, a, b, self.scalar_gain, None, self.eps, self.rt.act, rows)[0]

    def apply_pair(self, hidden: torch.Tensor, delta, other: "ScalarRMSNorm"):
        """This norm and ``other`` (same epsilon) of the same rows in one kernel."""
        a, b = split_sum(delta)
        return F.add2_rmsnorm_scalar(hidden, a, b, self.scalar_gain, other.scalar_gain, self.eps, self.rt.act)


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "rmsnorm_scalar", ScalarRMSNorm)
