"""Arrangements of a layer's parts.

``prenorm_residual`` (engine/model/layers.py:301-303): ``h = x + mixer(norm(x))``, then
``out = h + feed_forward(norm(h))``.  The residual stream ``h`` is 32-bit and is updated in
place; each add is fused into the norm that follows it, so a block returns its
feed-forward's output as a pending ``delta`` for the next norm to add.
"""

from __future__ import annotations

from .base import Block, BuildEnv, CacheBinding
from .registry import build_part, register_part


@register_part("block", "prenorm_residual")
class PreNormResidualBlock(Block):
    def __init__(self, mixer, feed_forward, pre_mixer, pre_feed_forward) -> None:
        self.mixer, self.feed_forward = mixer, feed_forward
        self.pre_mixer, self.pre_feed_forward = pre_mixer, pre_feed_forward

    @classmethod
    def from_spec(cls, params: dict, env: BuildEnv, *, layer, **_):
        return cls(
            build_part("mixer", layer.mixer, env),
            build_part("feed_forward", layer.feed_forward, env),
            build_part("norm", layer.norms["pre_mixer"], env),
            build_part("norm", layer.norms["pre_feed_forward"], env),
        )

    def parts(self):
        return [self.pre_mixer, self.mixer, self.pre_feed_forward, self.feed_forward]

    def forward(self, h, delta, ctx, binding: CacheBinding | None):
        x = self.pre_mixer.add_norm(h, delta, ctx, tag="norm.mixer")
        mixed = self.mixer.forward(x, ctx, binding)
        x = self.pre_feed_forward.add_norm(h, mixed, ctx, tag="norm.ffn")
        return self.feed_forward.forward(x, ctx)
