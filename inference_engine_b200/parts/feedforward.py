"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))`` (engine/model/layers.py:277-281),
``silu(g) = g / (1 + exp(-g))`` evaluated in 32-bit.  Gate and up run as one matrix product
over the stacked weights.  Their rows alternate in blocks of 16 (16 gate rows, the 16 up rows
with the same indices, the next 16 gate rows, ...) when the width allows: every dot product is
unchanged, and a kernel that owns a tile of rows then holds each gate beside its up and can
apply the activation itself (``ops.gated_linear``)."""

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
        self.interleave = 0

    ROW_BLOCK = 16  # gate and up rows alternate in blocks of this many

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

        gate, up = tensors[self.names["gate"]].to(self.dtype), tensors[self.names["up"]].to(self.dtype)
        i, h, b = self.intermediate_size, self.hidden_size, self.ROW_BLOCK
        if i % b == 0:
            self.interleave = b
            self.w_gate_up = torch.stack([gate.view(i // b, b, h), up.view(i // b, b, h)], dim=1).reshape(2 * i, h).contiguous()
        else:
            self.interleave = 0
            self.w_gate_up = torch.cat([gate, up]).contiguous()
        self.w_down = tensors[self.names["down"]].to(self.dtype).contiguous()

    def forward(self, x, ctx):
        import torch

        act = ctx.ops.gated_linear(x, self.w_gate_up, self.interleave, ws=ctx.ws, tag="ffn", out_dtype=self.dtype)
        return ctx.ops.linear(act, self.w_down, ws=ctx.ws, tag="ffn.delta", out_dtype=torch.float32,
                              allow_split=True)
