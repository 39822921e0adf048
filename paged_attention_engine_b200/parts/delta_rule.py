"""The generalized delta rule: a recurrent mixer with a per-head matrix state.

With r, k, v = W_r h, W_k h, W_v h (heads x d each), the decay w = exp(-c * sigmoid(W_w2
tanh(W_w1 h) + w0)) and the removal rate a = sigmoid(W_a h + a_bias), both per head and key
channel, and the unit key u = k / sqrt(sum(k^2) + key_eps):

    S_t = diag(w) S_(t-1) - (a * u) (u^T S_(t-1)) + k v^T,        o_t = S_t^T r

Each head's o is divided by its root mean square, multiplied by a weight and by sigmoid(W_g h),
and projected by W_o. The state starts at zero, is float32, and is the request's per-request
state [heads, d, d]; the decay, the rate, the unit key and the recurrence are float32.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import MIXERS, Part, StateNeed, TensorSpec


@MIXERS.register("general_delta")
class GeneralDelta(Part):
    """params: hidden_size, num_heads, head_dim, decay_rank (0: the checkpoint's), decay_scale (c),
    key_eps, norm_eps. tensors: r, k, v, g, a, o matrices; w1 [rank, hidden], w2 [heads * d, rank];
    a.b, w0 [heads * d]; norm [heads * d]."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        p = spec.params
        hidden, width = int(p["hidden_size"]), int(p["num_heads"]) * int(p["head_dim"])
        rank = int(p.get("decay_rank") or 0) or -1
        name = spec.tensor_name
        return [TensorSpec(name(n), (width, hidden), "matrix") for n in ("r", "k", "v", "g", "a")] + [
            TensorSpec(name("a.b"), (width,), "vector"),
            TensorSpec(name("w1"), (rank, hidden), "matrix"),
            TensorSpec(name("w2"), (width, rank), "matrix"),
            TensorSpec(name("w0"), (width,), "vector"),
            TensorSpec(name("norm"), (width,), "scale"),
            TensorSpec(name("o"), (hidden, width), "matrix"),
        ]

    @classmethod
    def state_need(cls, spec: PartSpec) -> StateNeed:
        heads, d = int(spec.params["num_heads"]), int(spec.params["head_dim"])
        return StateNeed((heads, d, d), torch.float32)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.num_heads, self.head_dim = int(p["num_heads"]), int(p["head_dim"])
        self.width = self.num_heads * self.head_dim
        self.decay_scale, self.key_eps, self.norm_eps = float(p["decay_scale"]), float(p["key_eps"]), float(p["norm_eps"])
        name = spec.tensor_name
        w1 = tensors.pop(name("w1"))
        self.w2 = tensors.pop(name("w2"))
        self.rank = int(w1.shape[0])
        if self.w2.shape[1] != self.rank:
            raise ValueError(f"general_delta: w1 has {self.rank} rows, w2 {self.w2.shape[1]} columns")
        # One product for r | k | v | a | g | w1: the columns of its output in that order.
        self.in_weight = torch.cat([tensors.pop(name(n)) for n in ("r", "k", "v", "a", "g")] + [w1], dim=0).contiguous()
        self.a_bias = tensors.pop(name("a.b"))
        self.w0 = tensors.pop(name("w0"))
        self.norm_weight = tensors.pop(name("norm"))
        self.o_weight = tensors.pop(name("o"))

    def forward(self, ctx, x, residual, cache):
        ops = self.ops
        width = self.width
        proj = ops.materialized(ops.linear(x, self.in_weight, None, None, out_dtype=torch.float32))
        low = ops.tanh_columns(proj, 5 * width, self.rank, self.runtime.dtype)
        w_pre = ops.linear(low, self.w2, None, None, out_dtype=torch.float32)
        out = ops.delta_rule(proj, (0, width, 2 * width, 3 * width), w_pre, self.w0, self.a_bias, 4 * width,
                             self.norm_weight, cache.state, ctx.q_start, ctx.state_slot, ctx.num_seqs, self.num_heads,
                             self.head_dim, self.decay_scale, self.key_eps, self.norm_eps, self.runtime.dtype)
        return ops.linear(out, self.o_weight, None, residual, out_dtype=residual.dtype)
