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


class GroupedRMSNorm(Norm):
    """RMS norm in groups: a row is split into ``groups`` equal consecutive parts, each is divided by its own
    ``sqrt(mean(part^2) + eps)``, and the whole is multiplied by the weight.  params: ``size``, ``eps``,
    ``groups`` (default 1), optional ``tensor`` (the tensor's name below the prefix, default ``weight``).
    Tensor: ``<prefix><tensor> [size]``.

    ``apply_float`` returns the normalised rows unrounded, for an arrangement whose next step (a short
    convolution, say) still works in float32; ``group_parameters()`` hands ``(weight, eps, groups)`` to a block
    that runs the norm inside a kernel of its own."""

    graph_safe = True
    kernel_files = ("residual_forms.cu",)

    def _name(self) -> str:
        return self.prefix + self.params.get("tensor", "weight")

    def tensor_decls(self) -> List[TensorDecl]:
        return [TensorDecl(self._name(), (self.params["size"],), "norm")]

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt
        self.eps = float(self.params["eps"])
        self.groups = int(self.params.get("groups", 1))
        if self.groups < 1 or int(self.params["size"]) % self.groups:
            raise ValueError(f"rmsnorm_grouped: {self.params['size']} columns do not split into {self.groups} groups")
        # the norm is float arithmetic
        self.weight = tensors[self._name()].to(device=rt.device, dtype=torch.float32).contiguous()

    def group_parameters(self):
        return self.weight, self.eps, self.groups

    def rms_parameters(self):
        return (self.weight, self.eps) if self.groups == 1 else None

    def _updated(self, hidden: torch.Tensor, delta) -> torch.Tensor:
        if isinstance(delta, Deferred):
            delta = delta.materialize()
        if delta is not None:
            hidden.add_(delta)
        return hidden

    def apply(self, hidden: torch.Tensor, delta, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if rows is not None and delta is not None:
            # the last norm of a model: only the wanted rows are read, the residual is left as it is
            d = delta.materialize() if isinstance(delta, Deferred) else delta
            if d is not None:
                hidden = hidden + d
            delta = None
        return F.group_rmsnorm(self._updated(hidden, delta), self.weight, self.groups, self.eps, self.rt.act, rows)

    def apply_float(self, hidden: torch.Tensor, delta=None) -> torch.Tensor:
        return F.group_rmsnorm(self._updated(hidden, delta), self.weight, self.groups, self.eps, torch.float32)


register_part("norm", "rmsnorm", RMSNorm)
register_part("norm", "rmsnorm_grouped", GroupedRMSNorm)
register_part("norm", "rmsnorm_scalar", ScalarRMSNorm)
