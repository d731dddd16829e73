"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))`` (engine/model/layers.py:277-281),
``silu(g) = g / (1 + exp(-g))`` evaluated in 32-bit.  Gate and up run as one matrix product
over the row-concatenated weights."""

from __future__ import annotations

from .base import BuildEnv, FeedForward, WeightDecl
from .registry import register_part


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, *, gate_proj: str, up_proj: str, down_proj: str, hidden_size: int,
                 intermediate_size: int, dtype) -> None:
        self.names = {"gate": gate_proj, "up": up_proj, "down": down_proj}
        self.hidden_size, self.intermediate_size, self.dtype = hidden_size, intermediate_size, dtype
        self.w_gate_up = self.w_down = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(gate_proj=params["gate_proj"], up_proj=params["up_proj"],
                   down_proj=params["down_proj"],
                   hidden_size=params.get("hidden_size", env.hidden_size),
                   intermediate_size=params["intermediate_size"], dtype=env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        h, i = self.hidden_size, self.intermediate_size
        return {
            self.names["gate"]: WeightDecl((i, h)),
            self.names["up"]: WeightDecl((i, h)),
            self.names["down"]: WeightDecl((h, i)),
        }

    def bind(self, tensors, env: BuildEnv) -> None:
        import torch

        self.w_gate_up = torch.cat(
            [tensors[self.names["gate"]].to(self.dtype), tensors[self.names["up"]].to(self.dtype)]
        ).contiguous()
        self.w_down = tensors[self.names["down"]].to(self.dtype).contiguous()

    def forward(self, x, ctx):
        import torch

        n, i = x.shape[0], self.intermediate_size
        gate_up = ctx.ops.linear(x, self.w_gate_up, ws=ctx.ws, tag="ffn.gate_up", out_dtype=self.dtype,
                                 allow_split=True)
        act = ctx.ws.buffer("ffn.act", n, i, self.dtype)
        ctx.ops.silu_mul(gate_up, act)
        return ctx.ops.linear(act, self.w_down, ws=ctx.ws, tag="ffn.delta", out_dtype=torch.float32,
                              allow_split=True)
