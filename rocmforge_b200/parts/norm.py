"""RMSNorm fused with the pending residual add."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..weights.spec import ParamSpec
from .base import NORMS, Norm


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    """y_i = x_i * rsqrt(mean(x^2) + eps) * w_i, sums and rsqrt in 32-bit; the weight multiplies
    after normalisation and is used as stored (no 1 + w)
    (maeddesg/ROCmForge hip_kernels/norm.hip:18-84, src/cpu/ops.rs:32-46).

    ``weight_offset``: for designs that store the weight around zero, y = x * rsqrt(...) * (offset + w); the sum is formed
    once at load time in 32-bit and the kernels get that 32-bit vector."""

    def __init__(self, size: int, eps: float, param_name: str = "weight", weight_offset: float = 0.0):
        """``param_name``: the weight's name below the part's prefix ("" where the prefix is the tensor's whole name)."""
        self.size = size
        self.eps = float(eps)
        self.weight_offset = float(weight_offset)
        self.param_name = param_name
        self.weight: Optional[torch.Tensor] = None
        self.compute_dtype = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        if self.weight_offset:
            return {self.param_name: ParamSpec((self.size,), kind="vector", init="normal", std=0.1)}
        return {self.param_name: ParamSpec((self.size,), kind="vector", init="ones")}

    def bind(self, params, compute_dtype):
        self.weight = params[self.param_name]
        if self.weight_offset:
            self.weight = (self.weight.to(torch.float32) + self.weight_offset).contiguous()
        self.compute_dtype = compute_dtype

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]

    def deferred_params(self):
        return (self.weight, self.eps)

    def forward(self, ctx, stream, rows=None, deferred_ok=False):
        prepared, stream.prepared = stream.prepared, None
        if prepared is not None and prepared[0] is self and rows is None and stream.pending is None:
            # the product that updated the stream has multiplied by this norm's weight and left the sums of squares
            if isinstance(prepared[1], torch.Tensor):      # whoever updated the stream has run this norm as well
                return prepared[1]
            return prepared[1] if deferred_ok else prepared[1].materialize()
        y = kernels.add_rmsnorm(stream.h, self.weight, self.eps, self.compute_dtype,
                                pending=stream.pending, rows=rows)
        if rows is None:
            stream.pending = None           # the kernel added it into h
        return y


@NORMS.register("dyt")
class DynamicTanh(Norm):
    """y_i = tanh(alpha x_i) * w_i + b_i with one learned number alpha: a norm that computes no statistics of its row,
    evaluated in 32-bit.  Tensors: the weight ``param_name``, and ``<param_name>.alpha`` (no dimensions) and
    ``<param_name>.b`` beside it.  Whoever updates the stream last may run it in the same pass (``dyt_params``) and leave
    the result in ``stream.prepared``."""

    def __init__(self, size: int, param_name: str = "weight"):
        self.size, self.param_name = size, param_name
        self.weight = self.bias = self.alpha = None
        self.compute_dtype = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n = self.param_name
        return {n: ParamSpec((self.size,), kind="vector", init="ones"),
                n + ".alpha": ParamSpec((), kind="vector", init="ones"),
                n + ".b": ParamSpec((self.size,), kind="vector", init="zeros")}

    def bind(self, params, compute_dtype):
        n = self.param_name
        # the kernels take these three in 32-bit (from bfloat16 the conversion is exact)
        self.weight = params[n].to(torch.float32).contiguous()
        self.bias = params[n + ".b"].to(torch.float32).contiguous()
        self.alpha = params[n + ".alpha"].to(torch.float32).reshape(1).contiguous()
        self.compute_dtype = compute_dtype

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]

    def dyt_params(self):
        return (self.alpha, self.weight, self.bias)

    def forward(self, ctx, stream, rows=None, deferred_ok=False):
        prepared, stream.prepared = stream.prepared, None
        if prepared is not None and prepared[0] is self and rows is None and stream.pending is None:
            return prepared[1]
        stream.flush()
        return kernels.dyt_rows(stream.h, self.alpha, self.weight, self.bias, self.compute_dtype, rows=rows)
