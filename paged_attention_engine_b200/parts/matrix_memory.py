"""The matrix memory of xLSTM (mLSTM): a recurrent mixer with a matrix state per head.

With q = W_q h / sqrt(d) and k = W_k h (heads x d), v = W_v h (heads x dv), and per head the
log input gate i = cap tanh((W_i h + b_i) / cap) and the log forget gate f = logsigmoid(cap
tanh((W_f h + b_f) / cap)):

    m_t = max(f + m_(t-1), i)        S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T
    n_t likewise with k alone        o_t = S_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6)

S, n and m start at zero. Each head's o is divided by its root mean square, multiplied by a
weight and by sigmoid(W_g h), and projected by W_o. The state is the request's per-request
state, float32; the gates and the recurrence are float32.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import MIXERS, Part, StateNeed, TensorSpec


@MIXERS.register("matrix_memory")
class MatrixMemory(Part):
    """params: hidden_size, num_heads, head_dim, value_dim, gate_cap, norm_eps. tensors: q, k
    [heads * head_dim, hidden]; v, g [heads * value_dim, hidden]; i, f [heads, hidden]; i.b, f.b
    [heads]; norm [heads * value_dim]; o [hidden, heads * value_dim]."""

    @classmethod
    def _sizes(cls, spec: PartSpec):
        p = spec.params
        d = int(p["head_dim"])
        return int(p["num_heads"]), d, int(p.get("value_dim") or d)

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        hidden = int(spec.params["hidden_size"])
        heads, d, dv = cls._sizes(spec)
        name = spec.tensor_name
        return ([TensorSpec(name(n), (heads * d, hidden), "matrix") for n in ("q", "k")]
                + [TensorSpec(name(n), (heads * dv, hidden), "matrix") for n in ("v", "g")]
                + [TensorSpec(name(n), (heads, hidden), "matrix") for n in ("i", "f")]
                + [TensorSpec(name("i.b"), (heads,), "vector"), TensorSpec(name("f.b"), (heads,), "vector"),
                   TensorSpec(name("norm"), (heads * dv,), "scale"), TensorSpec(name("o"), (hidden, heads * dv), "matrix")])

    @classmethod
    def state_need(cls, spec: PartSpec) -> StateNeed:
        heads, d, dv = cls._sizes(spec)
        # per head: S with n as one more column, [d][dv + 1], then m
        return StateNeed((heads, d * (dv + 1) + 1), torch.float32)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.num_heads, self.head_dim, self.value_dim = self._sizes(spec)
        self.gate_cap, self.norm_eps = float(p["gate_cap"]), float(p["norm_eps"])
        name = spec.tensor_name
        # One product for q | k | v | g | i | f: the columns of its output in that order.
        self.in_weight = torch.cat([tensors.pop(name(n)) for n in ("q", "k", "v", "g", "i", "f")], dim=0).contiguous()
        self.i_bias, self.f_bias = tensors.pop(name("i.b")), tensors.pop(name("f.b"))
        self.norm_weight = tensors.pop(name("norm"))
        self.o_weight = tensors.pop(name("o"))

    def forward(self, ctx, x, residual, cache):
        ops = self.ops
        heads, d, dv = self.num_heads, self.head_dim, self.value_dim
        proj = ops.linear(x, self.in_weight, None, None, out_dtype=torch.float32)
        q_off, k_off, v_off, g_off = 0, heads * d, 2 * heads * d, 2 * heads * d + heads * dv
        i_off = g_off + heads * dv
        out = ops.matrix_memory(proj, (q_off, k_off, v_off, g_off, i_off, i_off + heads), self.i_bias, self.f_bias,
                                self.norm_weight, cache.state, ctx.q_start, ctx.state_slot, ctx.num_seqs, heads, d, dv,
                                self.gate_cap, float(d) ** -0.5, self.norm_eps, self.runtime.dtype)
        return ops.linear(out, self.o_weight, None, residual, out_dtype=residual.dtype)
