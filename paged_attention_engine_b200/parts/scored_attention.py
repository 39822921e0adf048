"""Sliding-window attention with a score rule, short convolutions and a sink.

q, k and v are one fused projection without bias (float32 out). A short causal convolution runs
over time on every channel of it; the last taps - 1 projected rows of a request are per-request
state, so a prompt may be cut anywhere. Every query and key head is then divided by its root mean
square (no weight), and the keys and values go to their pages. Scores are
(q . k) * scale * temp[h], capped by softcap * tanh(. / softcap), minus r1[h] * log(1 + r2[h] *
(i - j)); query i sees key j <= i when i - j < window or j < keep_first (kept keys keep their true
positions); the softmax's denominator also holds exp(sink[h]). Value heads may have another size
than query and key heads. Every piece of the rule is a parameter and can be absent.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import MIXERS, CacheNeed, Part, StateNeed, TensorSpec


@MIXERS.register("scored_window_attention")
class ScoredWindowAttention(Part):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, value_dim, scale, softcap (0: none),
    conv_taps (0: no convolution), window (0: all keys), keep_first, qk_norm_eps (None: q and k are
    not normalized), head_temperature, distance_bias, sink (booleans: which per-head constants exist).
    tensors: q, k, v, o matrices; q.conv, k.conv, v.conv [channels, taps]; temp, r1, r2, sink [heads]."""

    @classmethod
    def _sizes(cls, spec: PartSpec):
        p = spec.params
        heads, kv_heads, d = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        return heads, kv_heads, d, int(p.get("value_dim") or d)

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        p = spec.params
        hidden = int(p["hidden_size"])
        heads, kv_heads, d, dv = cls._sizes(spec)
        rows = {"q": heads * d, "k": kv_heads * d, "v": kv_heads * dv}
        out = [TensorSpec(spec.tensor_name(n), (r, hidden), "matrix") for n, r in rows.items()]
        taps = int(p.get("conv_taps") or 0)
        if taps:
            out += [TensorSpec(spec.tensor_name(f"{n}.conv"), (r, taps), "taps") for n, r in rows.items()]
        if p.get("distance_bias"):
            out += [TensorSpec(spec.tensor_name("r1"), (heads,), "vector"), TensorSpec(spec.tensor_name("r2"), (heads,), "rate")]
        if p.get("head_temperature"):
            out.append(TensorSpec(spec.tensor_name("temp"), (heads,), "scale"))
        if p.get("sink"):
            out.append(TensorSpec(spec.tensor_name("sink"), (heads,), "vector"))
        out.append(TensorSpec(spec.tensor_name("o"), (hidden, heads * dv), "matrix"))
        return out

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        _, kv_heads, d, dv = cls._sizes(spec)
        p = spec.params
        return CacheNeed(kv_heads, d, int(p.get("window") or 0), 0 if dv == d else dv, int(p.get("keep_first") or 0))

    @classmethod
    def state_need(cls, spec: PartSpec) -> StateNeed | None:
        taps = int(spec.params.get("conv_taps") or 0)
        if taps <= 1:
            return None
        heads, kv_heads, d, dv = cls._sizes(spec)
        return StateNeed((taps - 1, (heads + kv_heads) * d + kv_heads * dv), torch.float32)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim = self._sizes(spec)
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"scored_window_attention: {self.num_heads} heads over {self.num_kv_heads} kv heads")
        self.scale = float(p["scale"])
        self.softcap = float(p.get("softcap") or 0.0)
        self.window = int(p.get("window") or 0)
        self.keep_first = int(p.get("keep_first") or 0)
        self.qk_norm_eps = p.get("qk_norm_eps")
        self.taps = int(p.get("conv_taps") or 0)
        names = ("q", "k", "v")
        self.qkv_weight = torch.cat([tensors.pop(spec.tensor_name(n)) for n in names], dim=0).contiguous()
        self.conv_weight = None
        if self.taps:
            self.conv_weight = torch.cat([tensors.pop(spec.tensor_name(f"{n}.conv")) for n in names], dim=0).contiguous()
        take = lambda name, present: tensors.pop(spec.tensor_name(name)) if present else None
        self.r1, self.r2 = take("r1", p.get("distance_bias")), take("r2", p.get("distance_bias"))
        self.temp = take("temp", p.get("head_temperature"))
        self.sink = take("sink", p.get("sink"))
        self.o_weight = tensors.pop(spec.tensor_name("o"))

    def forward(self, ctx, x, residual, cache):
        ops = self.ops
        group = ctx.groups[cache.group]
        proj = ops.linear(x, self.qkv_weight, None, None, out_dtype=torch.float32)
        q = ops.conv_heads_cache_write(
            proj, self.conv_weight, cache.state, ctx.positions, ctx.seq_index, ctx.q_start, ctx.q_pos0, ctx.state_slot,
            group.slots if cache.writes else None, cache.keys, cache.values, self.num_heads, self.num_kv_heads,
            self.head_dim, self.value_dim, cache.page_size, self.qk_norm_eps is not None, float(self.qk_norm_eps or 0.0),
            self.runtime.dtype)
        out = ops.paged_attention_scored(
            q, cache.keys, cache.values, group.block_table, ctx.q_start, ctx.q_pos0, ctx.kv_len, self.num_heads,
            self.num_kv_heads, self.head_dim, self.value_dim, cache.page_size, ctx.max_q_len, self.scale, self.softcap,
            self.temp, self.r1, self.r2, self.sink, self.window, self.keep_first, max_kv_len=ctx.max_kv_len,
            num_single=ctx.num_single)
        return ops.linear(out, self.o_weight, None, residual, out_dtype=residual.dtype)
