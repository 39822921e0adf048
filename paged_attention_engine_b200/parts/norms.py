"""Norms. RMSNorm as the reference computes it (engine/model.py:117-123): the mean of the
squares and the scaling in 32-bit, no bias, no mean subtraction. The kernel multiplies
by the weight in 32-bit too and rounds once; the reference rounds before and after the
weight, which costs one more rounding in bfloat16 and nothing in float32."""

from __future__ import annotations

from ..config.model_spec import PartSpec
from .base import NORMS, Part, TensorSpec


@NORMS.register("rms_norm")
class RMSNorm(Part):
    """params: size, eps, out ("engine": the result is in the engine's dtype whatever x is, as a
    float32 residual stream needs; default: x's dtype). tensors: weight [size]."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        return [TensorSpec(spec.tensor_name("weight"), (int(spec.params["size"]),), "scale")]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.eps = float(spec.params["eps"])
        self.weight = tensors[spec.tensor_name("weight")]
        self.out_dtype = runtime.dtype if spec.params.get("out") == "engine" else None

    def forward(self, ctx, x):
        if self.out_dtype is not None:
            return self.ops.rms_norm_cast(x, self.weight, self.eps, self.out_dtype)
        return self.ops.rms_norm(x, self.weight, self.eps)


@NORMS.register("layer_norm")
class LayerNorm(Part):
    """(x - mean) / sqrt(var + eps) * weight + bias, var the mean of the squared deviations;
    statistics in 32-bit. params: size, eps, bias (default True), out ("engine": the result is
    in the engine's dtype even when x, a float32 residual stream, is not; default: x's dtype).
    tensors: weight [size], bias [size]."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        size = int(spec.params["size"])
        out = [TensorSpec(spec.tensor_name("weight"), (size,), "scale")]
        if spec.params.get("bias", True):
            out.append(TensorSpec(spec.tensor_name("bias"), (size,), "vector"))
        return out

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.eps = float(spec.params["eps"])
        self.weight = tensors[spec.tensor_name("weight")]
        self.bias = tensors[spec.tensor_name("bias")] if spec.params.get("bias", True) else None
        self.out_dtype = runtime.dtype if spec.params.get("out") == "engine" else None

    def forward(self, ctx, x):
        return self.ops.layer_norm(x, self.weight, self.bias, self.eps, self.out_dtype)
