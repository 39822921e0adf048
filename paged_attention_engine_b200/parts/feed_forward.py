"""Feed-forwards. SwiGLU as in the reference (engine/model.py:317-320):
down(silu(gate(x)) * up(x)), no biases; gate and up are one product here, and the
down projection takes the residual in its epilogue."""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import FEED_FORWARDS, Part, TensorSpec


@FEED_FORWARDS.register("swiglu")
class SwiGLU(Part):
    """params: hidden_size, intermediate_size. tensors: gate_proj/up_proj/down_proj .weight."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        hidden, inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        return [
            TensorSpec(spec.tensor_name("gate_proj.weight"), (inter, hidden), "matrix"),
            TensorSpec(spec.tensor_name("up_proj.weight"), (inter, hidden), "matrix"),
            TensorSpec(spec.tensor_name("down_proj.weight"), (hidden, inter), "matrix"),
        ]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.intermediate_size = int(spec.params["intermediate_size"])
        gate = tensors.pop(spec.tensor_name("gate_proj.weight"))
        up = tensors.pop(spec.tensor_name("up_proj.weight"))
        # Gate and up are one product. Where the kernels offer it, their rows alternate in
        # blocks (16 gate rows, their 16 up rows, ...) so that SiLU x up runs inside the
        # product; else rows [0, I) are the gate and rows [I, 2I) the up projection.
        interleave = getattr(self.ops, "interleave_gate_up", None)
        self.gate_up_weight = interleave(gate, up) if interleave is not None else None
        self.interleaved = self.gate_up_weight is not None
        if not self.interleaved:
            self.gate_up_weight = torch.cat([gate, up], dim=0).contiguous()
        self.down_weight = tensors.pop(spec.tensor_name("down_proj.weight"))

    def forward(self, ctx, x, residual):
        ops = self.ops
        if self.interleaved:
            hidden = ops.linear_swiglu(x, self.gate_up_weight)
        else:
            hidden = ops.silu_mul(ops.linear(x, self.gate_up_weight, None))
        return ops.linear(hidden, self.down_weight, None, residual)


@FEED_FORWARDS.register("dense_mlp")
class DenseMLP(Part):
    """down(act(up(x))) without biases. params: hidden_size, intermediate_size, activation
    ("gelu_erf": 0.5 z (1 + erf(z / sqrt 2)), or "gelu_tanh"). tensors: up.weight, down.weight.
    The residual may be float32 while x is in the engine's dtype: the down projection adds it in
    its epilogue and leaves the residual's dtype."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        hidden, inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        return [
            TensorSpec(spec.tensor_name("up.weight"), (inter, hidden), "matrix"),
            TensorSpec(spec.tensor_name("down.weight"), (hidden, inter), "matrix"),
        ]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.activation = str(spec.params.get("activation", "gelu_erf"))
        self.up_weight = tensors.pop(spec.tensor_name("up.weight"))
        self.down_weight = tensors.pop(spec.tensor_name("down.weight"))

    def forward(self, ctx, x, residual):
        ops = self.ops
        hidden = ops.linear(x, self.up_weight, None, activation=self.activation)     # the activation in the product's epilogue
        return ops.linear(hidden, self.down_weight, None, residual, out_dtype=residual.dtype if residual is not None else None)


@FEED_FORWARDS.register("clamped_glu")
class ClampedGLU(Part):
    """down(g * sigmoid(alpha * g) * (u + 1)) with g = min(gate(x), limit) and u = clamp(up(x),
    -limit, limit); all three projections have biases. params: hidden_size, intermediate_size,
    limit, alpha. tensors: gate, up [intermediate, hidden], down [hidden, intermediate] and
    gate.b, up.b, down.b. Gate and up are one product (float32 out: the clamps and the
    activation see unrounded sums); the down projection adds its bias and the residual in its
    epilogue and leaves the residual's dtype."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        hidden, inter = int(spec.params["hidden_size"]), int(spec.params["intermediate_size"])
        name = spec.tensor_name
        return [TensorSpec(name("gate"), (inter, hidden), "matrix"), TensorSpec(name("gate.b"), (inter,), "vector"),
                TensorSpec(name("up"), (inter, hidden), "matrix"), TensorSpec(name("up.b"), (inter,), "vector"),
                TensorSpec(name("down"), (hidden, inter), "matrix"), TensorSpec(name("down.b"), (hidden,), "vector")]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.limit, self.alpha = float(spec.params["limit"]), float(spec.params["alpha"])
        name = spec.tensor_name
        # rows [0, I) are the gate and rows [I, 2I) the up projection
        self.gate_up_weight = torch.cat([tensors.pop(name("gate")), tensors.pop(name("up"))], dim=0).contiguous()
        self.gate_up_bias = torch.cat([tensors.pop(name("gate.b")), tensors.pop(name("up.b"))], dim=0).contiguous()
        self.down_weight, self.down_bias = tensors.pop(name("down")), tensors.pop(name("down.b"))

    def forward(self, ctx, x, residual):
        ops = self.ops
        gate_up = ops.linear(x, self.gate_up_weight, self.gate_up_bias, None, out_dtype=torch.float32)
        hidden = ops.clamped_glu(gate_up, self.limit, self.alpha, self.runtime.dtype)
        return ops.linear(hidden, self.down_weight, self.down_bias, residual, out_dtype=residual.dtype)
