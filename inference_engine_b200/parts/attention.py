"""Grouped-query attention over the paged cache (the mixer of a Llama layer).

Order of operations (engine/model/layers.py:171-225): project to queries, keys and values
(no bias), rotate queries and keys, write the new keys (rotated) and values into the
request's pages, attend causally over the whole cached prefix with scale ``head_dim^-0.5``
(query head ``h`` uses key/value head ``h // groups``), project the heads back.
The three input projections run as one matrix product over the row-concatenated weights:
each output column's dot product is unchanged.
"""

from __future__ import annotations

from .base import BuildEnv, CacheBinding, Mixer, PagedKVRequest, WeightDecl
from .registry import register_part


@register_part("mixer", "paged_attention")
class PagedAttention(Mixer):
    def __init__(self, *, q_proj: str, k_proj: str, v_proj: str, o_proj: str, hidden_size: int,
                 num_heads: int, num_kv_heads: int, head_dim: int, position, window: int | None,
                 scale: float | None, dtype) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) not divisible by KV heads ({num_kv_heads})")
        self.names = {"q": q_proj, "k": k_proj, "v": v_proj, "o": o_proj}
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.position, self.window, self.dtype = head_dim, position, window, dtype
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.q_size, self.kv_size = num_heads * head_dim, num_kv_heads * head_dim
        self.w_qkv = self.w_o = None

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, **_):
        position = env.positions[params["position"]] if params.get("position") else None
        return cls(q_proj=params["q_proj"], k_proj=params["k_proj"], v_proj=params["v_proj"],
                   o_proj=params["o_proj"], hidden_size=params.get("hidden_size", env.hidden_size),
                   num_heads=params["num_heads"], num_kv_heads=params["num_kv_heads"],
                   head_dim=params["head_dim"], position=position,
                   window=params.get("window"), scale=params.get("scale"), dtype=env.torch_dtype)

    def weights(self) -> dict[str, WeightDecl]:
        h = self.hidden_size
        return {
            self.names["q"]: WeightDecl((self.q_size, h)),
            self.names["k"]: WeightDecl((self.kv_size, h)),
            self.names["v"]: WeightDecl((self.kv_size, h)),
            self.names["o"]: WeightDecl((h, self.q_size)),
        }

    def bind(self, tensors, env: BuildEnv) -> None:
        import torch

        self.w_qkv = torch.cat([tensors[self.names[n]].to(self.dtype) for n in "qkv"]).contiguous()
        self.w_o = tensors[self.names["o"]].to(self.dtype).contiguous()

    def cache_request(self) -> PagedKVRequest:
        return PagedKVRequest(self.num_kv_heads, self.head_dim, self.window)

    def forward(self, x, ctx, binding: CacheBinding):
        import torch

        n = x.shape[0]
        group = ctx.groups[binding.group]
        qkv = ctx.ops.linear(x, self.w_qkv, ws=ctx.ws, tag="attn.qkv", out_dtype=torch.float32,
                             allow_split=True)
        q = ctx.ws.buffer("attn.q", n, self.q_size, self.dtype)
        table = self.position.rotary_table() if self.position is not None else None
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        ctx.ops.rope_kv_write(
            qkv, ctx.positions, table, rotary_dim, q,
            group.k[binding.slot], group.v[binding.slot],
            group.slot_mapping if binding.writes else None,
            self.num_heads, self.num_kv_heads, self.head_dim, group.page_size,
        )
        out = ctx.ws.buffer("attn.out", n, self.q_size, self.dtype)
        ctx.ops.paged_attention(
            q, group.k[binding.slot], group.v[binding.slot], group.block_tables, ctx,
            self.num_heads, self.num_kv_heads, self.head_dim, group.page_size,
            self.scale, self.window or 0, out, ragged=group.ragged,
        )
        return ctx.ops.linear(out, self.w_o, ws=ctx.ws, tag="mixer.delta", out_dtype=torch.float32,
                              allow_split=True)
