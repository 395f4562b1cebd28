"""RMSNorm: ``x * rsqrt(mean(x^2) + eps) * w``, eps inside the root, weight applied directly;
with ``one_plus`` the stored weight lies around zero and the factor is ``1 + w``.

Formula as in the reference's ``rms_norm_kernel`` (src/cuda/rms_norm.cu:15-25).
All arithmetic is float32; the result is rounded once to the output dtype.
"""
from __future__ import annotations

import torch

from .base import NORM_WEIGHT, NORM_ZERO, Part, WeightSpec, as_float32, register_part


class RMSNorm(Part):
    category = "norm"

    def __init__(self, size: int, eps: float, tensor: str = "weight", one_plus: bool = False):
        self.size = int(size)
        self.eps = float(eps)
        self.tensor = str(tensor)            # the weight's name behind the part's prefix (may be empty)
        self.one_plus = bool(one_plus)       # the stored weight is the factor minus one
        self.weight: torch.Tensor | None = None

    def weight_specs(self):
        return {self.tensor: WeightSpec((self.size,), NORM_WEIGHT)}

    def load_weights(self, tensors, ops):
        self.weight = as_float32(tensors[self.tensor]).contiguous()
        if self.one_plus:
            self.weight = 1.0 + self.weight          # float32; the kernels multiply by it as it is

    def forward(self, ops, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty((x.shape[0], self.size), dtype=out_dtype, device=x.device)
        ops.rmsnorm(x, self.weight, self.eps, out)
        return out

    def forward_rows(self, ops, x: torch.Tensor, rows: torch.Tensor,
                     out_dtype: torch.dtype) -> torch.Tensor:
        """Norm of the rows ``x[rows]`` only (the rows whose logits are wanted)."""
        out = torch.empty((rows.shape[0], self.size), dtype=out_dtype, device=x.device)
        ops.rmsnorm(x, self.weight, self.eps, out, rows=rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)


class GroupRMSNorm(Part):
    """RMS norm in groups: a row is cut into ``groups`` equal consecutive parts, each part is
    divided by its own ``sqrt(mean(part^2) + eps)``, and the whole row is multiplied by a weight
    per element.  ``groups = 1`` is the plain norm.  Besides the two forms every norm has,
    ``add_to`` adds the normed rows to a float32 residual: blocks that norm a sublayer's output
    rather than its input use it."""
    category = "norm"

    def __init__(self, size: int, eps: float, groups: int = 1, tensor: str = "weight"):
        self.size, self.eps, self.groups = int(size), float(eps), int(groups)
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"{self.size} elements do not fall into {self.groups} equal groups")
        self.tensor = str(tensor)
        self.weight: torch.Tensor | None = None

    def weight_specs(self):
        return {self.tensor: WeightSpec((self.size,), NORM_WEIGHT)}

    def load_weights(self, tensors, ops):
        self.weight = as_float32(tensors[self.tensor]).contiguous()

    def forward(self, ops, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty((x.shape[0], self.size), dtype=out_dtype, device=x.device)
        ops.group_norm(x, self.weight, self.eps, self.groups, out=out)
        return out

    def forward_rows(self, ops, x: torch.Tensor, rows: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty((rows.shape[0], self.size), dtype=out_dtype, device=x.device)
        ops.group_norm(x, self.weight, self.eps, self.groups, out=out, rows=rows)
        return out

    def add_to(self, ops, y: torch.Tensor, residual: torch.Tensor) -> None:
        """``residual += norm(y)``, both float32."""
        ops.group_norm(y, self.weight, self.eps, self.groups, residual=residual)


register_part("norm", "group_rmsnorm", GroupRMSNorm)


class DynamicTanh(Part):
    """A norm that takes no mean and no variance: ``tanh(alpha * x) * w + b`` with one scalar
    ``alpha``, a weight and a bias per element (tensors ``<tensor>``, ``<tensor>.alpha``,
    ``<tensor>.b``).  The three forms of ``GroupRMSNorm``: rows out, gathered rows out, and
    ``add_to`` a float32 residual."""
    category = "norm"

    def __init__(self, size: int, tensor: str = "weight", bias: bool = True):
        self.size, self.tensor, self.has_bias = int(size), str(tensor), bool(bias)
        self.weight = self.bias = None
        self.alpha = 1.0

    def weight_specs(self):
        specs = {self.tensor: WeightSpec((self.size,), NORM_WEIGHT), self.tensor + ".alpha": WeightSpec((), NORM_WEIGHT)}
        if self.has_bias:
            specs[self.tensor + ".b"] = WeightSpec((self.size,), NORM_ZERO)
        return specs

    def load_weights(self, tensors, ops):
        self.weight = as_float32(tensors[self.tensor]).contiguous()
        self.bias = as_float32(tensors[self.tensor + ".b"]).contiguous() if self.has_bias else None
        self.alpha = float(as_float32(tensors[self.tensor + ".alpha"]).reshape(()).item())   # a constant of the model

    def forward(self, ops, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty((x.shape[0], self.size), dtype=out_dtype, device=x.device)
        ops.tanh_norm(x, self.alpha, self.weight, self.bias, out=out)
        return out

    def forward_rows(self, ops, x: torch.Tensor, rows: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty((rows.shape[0], self.size), dtype=out_dtype, device=x.device)
        ops.tanh_norm(x, self.alpha, self.weight, self.bias, out=out, rows=rows)
        return out

    def add_to(self, ops, y: torch.Tensor, residual: torch.Tensor) -> None:
        """``residual += norm(y)``, both float32."""
        ops.tanh_norm(y, self.alpha, self.weight, self.bias, residual=residual)

    def add_then(self, ops, y: torch.Tensor, residual: torch.Tensor, then: "DynamicTanh",
                 out_dtype: torch.dtype) -> torch.Tensor:
        """``residual += norm(y)`` and ``then``'s norm of the sum, in one launch."""
        out = torch.empty((y.shape[0], self.size), dtype=out_dtype, device=y.device)
        ops.tanh_norm_pair(y, self.alpha, self.weight, self.bias, residual, then.alpha, then.weight, then.bias, out)
        return out


register_part("norm", "dynamic_tanh", DynamicTanh)
