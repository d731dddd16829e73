"""Token embedding and the output head.

Embedding: ``x = table[token_ids]`` with no scaling (engine/model/llama.py:25,61); the rows
are widened to the 32-bit residual stream.  Head: ``logits = x @ W^T`` in 32-bit out, no
bias (engine/model/llama.py:36,68); with tied embeddings ``W`` is the embedding table
itself (engine/model/loader.py:91-92), one buffer.
"""

from __future__ import annotations

from .base import BuildEnv, Part, WeightDecl
from .registry import register_part


@register_part("embedding", "token")
class TokenEmbedding(Part):
    category = "embedding"

    def __init__(self, weight: str, vocab_size: int, hidden_size: int, dtype) -> None:
        self.weight_name, self.vocab_size, self.hidden_size = weight, vocab_size, hidden_size
        self.dtype, self.table = dtype, None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(params["weight"], params["vocab_size"], env.hidden_size, env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        return {self.weight_name: WeightDecl((self.vocab_size, self.hidden_size), "table")}

    def bind(self, tensors, env: BuildEnv) -> None:
        self.table = tensors[self.weight_name].to(self.dtype).contiguous()

    def forward(self, token_ids, ctx):
        import torch

        h = ctx.ws.buffer("residual", token_ids.shape[0], self.hidden_size, torch.float32)
        ctx.ops.embedding(self.table, token_ids, h)
        return h


@register_part("head", "linear")
class LinearHead(Part):
    category = "head"

    def __init__(self, weight: str | None, vocab_size: int, hidden_size: int, dtype) -> None:
        self.weight_name, self.vocab_size, self.hidden_size = weight, vocab_size, hidden_size
        self.dtype, self.weight = dtype, None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        # weight=None means tied: the model hands over the embedding table at bind time.
        return cls(params.get("weight"), params["vocab_size"], env.hidden_size, env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        if self.weight_name is None:
            return {}
        return {self.weight_name: WeightDecl((self.vocab_size, self.hidden_size))}

    def bind(self, tensors, env: BuildEnv) -> None:
        if self.weight_name is not None:
            self.weight = tensors[self.weight_name].to(self.dtype).contiguous()

    def tie(self, table) -> None:
        self.weight = table

    def forward(self, x, ctx):
        import torch

        logits = ctx.ws.buffer("logits", x.shape[0], self.vocab_size, torch.float32, rows_cap=None)
        return ctx.ops.linear(x, self.weight, logits, tag="head")
