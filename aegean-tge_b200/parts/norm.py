"""RMSNorm with its epsilon as a parameter, and the RMS norm taken in groups.

Formula of the reference (src/cpu/scalar/norm_rope_scalar.cpp:8-21): the sum
of squares in float32, ``scale = 1 / sqrt(sum / dim + eps)``, then
``x * scale * weight`` (scale first, weight second).  No bias, no ``+1`` on
the weight.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .base import NORMS, Norm, ParamSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """params: ``size`` (row width), ``eps``; optional ``optional`` (bool: a checkpoint may lack the weight; the norm
    then does not exist: ``fusable()`` is None and ``forward`` refuses); optional ``unit_offset`` (bool: the weight is
    stored around zero and the row is multiplied by 1 + w; the sum is formed once, in float32, when the weight
    arrives).  weights: ``weight``."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        if self.size <= 0 or not self.eps > 0.0:
            raise ValueError(f"rmsnorm: size {self.size} and eps {self.eps} must be positive")
        self.optional = bool(spec.params.get("optional", False))
        self.unit_offset = bool(spec.params.get("unit_offset", False))
        self.loaded = False
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), role="vector", optional=self.optional)}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors.get("weight") if self.optional else tensors["weight"]
        if self.unit_offset and self.weight is not None:
            self.weight = (self.weight.float() + 1.0).contiguous()
        self.loaded = True

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.weight is None:
            raise RuntimeError("rmsnorm: the checkpoint holds no weight for this norm")
        return self.ops.rmsnorm(x, self.weight, self.eps, self.env.dtype, rows=rows)

    def fusable(self):
        if self.optional and self.loaded and self.weight is None:
            return None
        return self.weight, self.eps


@NORMS.register("group_rmsnorm")
class GroupRMSNorm(Norm):
    """The RMS norm in groups: a row is cut into ``groups`` equal consecutive parts, each part is divided by its own
    sqrt(mean(part^2) + eps), and the whole is multiplied by the weight.  One group is the plain RMS norm, which a
    product's epilogue kernel may apply (``fusable``).

    params: ``size`` (row width, a multiple of ``groups``), ``eps``, ``groups`` (default 1), optional ``optional``
    (bool: a checkpoint may lack the weight; the norm then does not exist and ``forward`` refuses).
    weights: ``weight``."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.groups = int(spec.params.get("groups", 1))
        if self.size <= 0 or not self.eps > 0.0 or self.groups <= 0 or self.size % self.groups:
            raise ValueError(f"group_rmsnorm: size {self.size}, eps {self.eps}, groups {self.groups}: sizes and eps must be "
                             f"positive and the groups must divide the row")
        self.optional = bool(spec.params.get("optional", False))
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), role="vector", optional=self.optional)}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        weight = tensors.get("weight") if self.optional else tensors["weight"]
        self.weight = weight.contiguous() if weight is not None else None

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        if self.weight is None:
            raise RuntimeError("group_rmsnorm: the checkpoint holds no weight for this norm")
        return self.ops.group_norm(x, self.weight, self.eps, self.groups, self.env.dtype, rows=rows)

    def forward_with(self, other: "GroupRMSNorm", x: torch.Tensor):
        """This norm and ``other`` of the same rows, (mine, theirs), from one kernel when the two differ in their weights
        only; else None."""
        if (not isinstance(other, GroupRMSNorm) or other.groups != self.groups or other.eps != self.eps or other.size != self.size
                or self.weight is None or other.weight is None):
            return None
        return self.ops.group_norm(x, self.weight, self.eps, self.groups, self.env.dtype, weight2=other.weight)

    def forward_stream(self, x: torch.Tensor) -> torch.Tensor:
        """The float32 rows normalised in place (a stream that starts from normalised embeddings)."""
        return self.ops.group_norm(x, self.weight, self.eps, self.groups, torch.float32, out=x)

    def fusable(self):
        return (self.weight, self.eps) if self.groups == 1 and self.weight is not None else None
