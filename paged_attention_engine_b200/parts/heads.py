"""Token embedding (engine/model.py:401: a row gather, no scaling) and the language-model
head (engine/model.py:406: a product without bias at the wanted rows only; the head is the
embedding table itself when the checkpoint ties them, engine/model.py:220-222). Logits
leave the head in float32."""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import EMBEDDINGS, HEADS, Part, TensorSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """params: vocab_size, hidden_size. tensors: weight [vocab, hidden]."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        return [TensorSpec(spec.tensor_name("weight"), (int(spec.params["vocab_size"]), int(spec.params["hidden_size"])), "matrix")]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = tensors[spec.tensor_name("weight")]

    def step_weight_bytes(self, num_tokens: int) -> int:
        """A step reads one row of the table per token, not the table. (When the head is tied to it,
        the head reads all of it and counts it.)"""
        return num_tokens * self.weight.shape[1] * self.weight.element_size()

    def forward(self, ctx):
        # A negative id is "the token sampled for this request in the step before" (see
        # StepContext.feedback); the kernel looks it up on the device.
        return self.ops.embedding(ctx.token_ids, self.weight, getattr(ctx, "feedback", None))


@HEADS.register("lm_head")
class LMHead(Part):
    """params: vocab_size, hidden_size, tied_to (a tensor's full name, or None), softcap (0 or
    absent: none; c: logits <- c tanh(logits / c), in float32). tensors: weight [vocab, hidden] unless tied."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        if spec.params.get("tied_to"):
            return []
        return [TensorSpec(spec.tensor_name("weight"), (int(spec.params["vocab_size"]), int(spec.params["hidden_size"])), "matrix")]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        tied = spec.params.get("tied_to")
        self.weight = tensors[tied] if tied else tensors[spec.tensor_name("weight")]
        self.softcap = float(spec.params.get("softcap") or 0.0)

    def forward(self, ctx, rows):
        logits = self.ops.linear(rows, self.weight, None, None, out_dtype=torch.float32)
        return self.ops.softcap(logits, self.softcap) if self.softcap else logits


@EMBEDDINGS.register("token_position_embedding")
class TokenPositionEmbedding(Part):
    """table[token] + position_scale * positions[p] as a float32 residual stream. params:
    vocab_size, hidden_size, max_positions, position_scale (default 1). tensors: weight
    [vocab, hidden], positions [max_positions, hidden]."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        hidden = int(spec.params["hidden_size"])
        return [TensorSpec(spec.tensor_name("weight"), (int(spec.params["vocab_size"]), hidden), "matrix"),
                TensorSpec(spec.tensor_name("positions"), (int(spec.params["max_positions"]), hidden), "matrix")]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = tensors[spec.tensor_name("weight")]
        self.positions = tensors[spec.tensor_name("positions")]
        self.position_scale = float(spec.params.get("position_scale", 1.0))

    def step_weight_bytes(self, num_tokens: int) -> int:
        return 2 * num_tokens * self.weight.shape[1] * self.weight.element_size()

    def forward(self, ctx):
        return self.ops.embedding_positions(ctx.token_ids, ctx.positions, self.weight, self.positions,
                                            getattr(ctx, "feedback", None), self.position_scale)


@EMBEDDINGS.register("scaled_token_embedding")
class ScaledTokenEmbedding(Part):
    """scale * table[token] as a float32 residual stream. params: vocab_size, hidden_size, scale.
    tensors: weight [vocab, hidden]."""

    @classmethod
    def tensor_specs(cls, spec: PartSpec) -> list[TensorSpec]:
        return [TensorSpec(spec.tensor_name("weight"), (int(spec.params["vocab_size"]), int(spec.params["hidden_size"])), "matrix")]

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.weight = tensors[spec.tensor_name("weight")]
        self.scale = float(spec.params.get("scale", 1.0))

    def step_weight_bytes(self, num_tokens: int) -> int:
        return num_tokens * self.weight.shape[1] * self.weight.element_size()

    def forward(self, ctx):
        return self.ops.embedding_scaled(ctx.token_ids, self.weight, self.scale, getattr(ctx, "feedback", None))
