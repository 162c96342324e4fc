"""RMSNorm: ``x * rsqrt(mean(x^2) + eps) * w`` with 32-bit statistics
(crates/vipera-backend-cpu/src/model.rs:4282-4288)."""
from __future__ import annotations

import torch

from ..config.registry import NORMS
from ..errors import InvalidArgumentError
from ..kernels import ops
from ..weights import TensorSpec
from .base import Norm


class RMSNorm(Norm):
    """params: ``size`` (width of a row), ``eps`` and, optionally, ``groups`` (the row is cut into
    that many equal consecutive parts and each part is divided by its own root mean square; default
    1, the whole row).  Tensor: ``<prefix>.weight`` [size].  The grouped form may write its 32-bit
    input in place."""

    kernels = ("rowwise",)
    fused_kind = "rmsnorm"  # products that can compute a norm on the way recognise it by this

    @classmethod
    def schema(cls, params, prefix):
        return {f"{prefix}.weight": TensorSpec((params["size"],), init="norm", store="float32")}

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        # The weight is used in 32-bit whatever it was stored in (bfloat16 widens exactly).
        self.weight = tensors[f"{prefix}.weight"].to(device=device, dtype=torch.float32).contiguous()
        self.groups = int(params.get("groups") or 1)
        if self.size % self.groups:
            raise InvalidArgumentError(f"{prefix}: {self.groups} groups do not divide a row of {self.size}")
        if self.groups > 1:
            # the products that take a norm with them know the norm over whole rows only
            self.fused_kind = None
            self.kernels = ("groupnorm",)

    def forward(self, ctx, x, out, rows=None):
        if self.groups > 1:
            ops.group_rmsnorm(x, self.weight, out, self.eps, self.groups, rows)
        else:
            ops.rmsnorm(x, self.weight, out, self.eps, rows)


class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * w + b`` with 32-bit statistics; the variance is the mean of
    the squared deviations.  params: ``size``, ``eps``.  Tensors: ``<prefix>.weight`` and
    ``<prefix>.bias`` [size].  ``add_into`` is the form a layer uses whose sublayer outputs are
    normalised before they join the residual stream."""

    kernels = ("rowwise",)

    @classmethod
    def schema(cls, params, prefix):
        return {f"{prefix}.weight": TensorSpec((params["size"],), init="norm", store="float32"),
                f"{prefix}.bias": TensorSpec((params["size"],), init="bias", store="float32")}

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = tensors[f"{prefix}.weight"].to(device=device, dtype=torch.float32).contiguous()
        self.bias = tensors[f"{prefix}.bias"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, ctx, x, out, rows=None):
        ops.layernorm(x, self.weight, self.bias, out, self.eps, rows)

    def add_into(self, ctx, x, residual):
        """residual += norm(x), both 32-bit [tokens, size]."""
        ops.layernorm(x, self.weight, self.bias, residual, self.eps, None, accumulate=True)


NORMS.register("rmsnorm", RMSNorm)
NORMS.register("layernorm", LayerNorm)
