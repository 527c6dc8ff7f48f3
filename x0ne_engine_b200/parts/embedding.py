"""The two ends of the model: token embedding and the output head."""
from __future__ import annotations

from typing import List, Mapping

import torch

from ..config.spec import PartSpec
from ..csrc import ops
from ..weights.loader import TensorNeed
from .base import EMBEDDINGS, HEADS, Embedding, Head
from .linear import Linear


class TokenEmbedding(Embedding):
    """resid[r] = float32(table[token[r]]); an id outside the table gives a zero row
    (x0ne-core/kernels/cuda/embedding.cu:5-17).  Parameters: vocab_size, hidden_size,
    names.weight."""
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.table = None

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        return [TensorNeed(spec["names"]["weight"], (int(spec["vocab_size"]), int(spec["hidden_size"])),
                           init="embedding")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = tensors[self.spec["names"]["weight"]]

    def forward(self, ctx, resid, n_rows):
        ops.embedding(self.table, ctx.tokens, resid, n_rows)


class LMHead(Head):
    """logits = normed W^T in float32 for the wanted rows only; W is the embedding table when the
    model is tied (x0ne-core/runtime/src/engine.rs:823-835).  Parameters: vocab_size,
    hidden_size, tied, names.weight."""
    replayable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.linear = None

    @staticmethod
    def tensor_needs(spec: PartSpec) -> List[TensorNeed]:
        return [TensorNeed(spec["names"]["weight"], (int(spec["vocab_size"]), int(spec["hidden_size"])),
                           init="embedding")]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.linear = Linear(tensors[self.spec["names"]["weight"]])

    @staticmethod
    def optional_duplicates(spec: PartSpec):
        # a tied checkpoint may also store lm_head.weight, equal to the table (x0ne-core/runtime/src/weights.rs:154-159)
        return {"lm_head.weight": spec["names"]["weight"]} if spec.get("tied") else {}

    def weight_bytes(self) -> int:
        return self.linear.weight_bytes()

    def forward(self, normed, logits, n_rows):
        return self.linear(normed, logits, n_rows)


EMBEDDINGS.register("token_embedding", TokenEmbedding)
HEADS.register("lm_head", LMHead)
