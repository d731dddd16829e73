"""Root-mean-square norm over the last dimension, with the residual add fused in.

Formula (engine/model/layers.py:41-43): ``normed = x * rsqrt(mean(x^2) + eps)`` in 32-bit,
then ``weight * normed``.  The residual stream is kept in 32-bit here, so square, mean,
rsqrt and both products are 32-bit and the result is rounded once to the compute dtype.
"""

from __future__ import annotations

from .base import BuildEnv, Norm, WeightDecl
from .registry import register_part


@register_part("norm", "rms")
class RMSNorm(Norm):
    def __init__(self, weight: str, size: int, eps: float, dtype) -> None:
        self.weight_name, self.size, self.eps, self.dtype = weight, int(size), float(eps), dtype
        self.weight = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        return cls(params["weight"], params.get("size", env.hidden_size), params["eps"],
                   env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        return {self.weight_name: WeightDecl((self.size,), "vector", "ones_plus_normal")}

    def bind(self, tensors, env: BuildEnv) -> None:
        self.weight = tensors[self.weight_name].float().contiguous()

    def add_norm(self, h, delta, ctx, rows=None, tag: str = "norm"):
        n = h.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.buffer(tag, n, self.size, self.dtype)
        ctx.ops.rmsnorm(h, delta, self.weight, self.eps, out, rows)
        return out
