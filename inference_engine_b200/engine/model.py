"""A model put together from parts according to a :class:`ModelSpec`.

The reference wires one fixed module tree (engine/model/llama.py:22-68).  Here the tree is
data: parts are built by kind, the run order is a list, and cache needs are collected from
the mixers and sorted into cache groups.
"""

from __future__ import annotations

import math
from typing import Any

from ..cache.manager import PagedGroupSpec, StateGroupSpec
from ..config.spec import ModelSpec
from ..parts.base import BuildEnv, CacheBinding, PagedKVRequest, Part, StateRequest, WeightDecl
from ..parts.registry import build_part


def _walk(part: Part):
    yield part
    for child in part.parts():
        yield from _walk(child)


class Model:
    def __init__(self, spec: ModelSpec, dtype: str, max_positions: int, device=None) -> None:
        spec.validate()
        self.spec = spec
        self.env = BuildEnv(spec.hidden_size, dtype, max_positions, {}, device)
        self.positions = {n: build_part("position", p, self.env) for n, p in spec.positions.items()}
        self.env.positions = self.positions
        self.embedding = build_part("embedding", spec.embedding, self.env)
        self.blocks = [build_part("block", layer.block, self.env, layer=layer) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, self.env)
        self.head = build_part("head", spec.head, self.env)
        self._plan_cache()

    # --- parts and weights ------------------------------------------------------------------

    def all_parts(self):
        for p in self.positions.values():
            yield from _walk(p)
        yield from _walk(self.embedding)
        for b in self.blocks:
            yield from _walk(b)
        yield from _walk(self.final_norm)
        yield from _walk(self.head)

    def declared_weights(self) -> dict[str, WeightDecl]:
        out: dict[str, WeightDecl] = {}
        for part in self.all_parts():
            for name, decl in part.weights().items():
                if name in out and out[name] != decl:
                    raise ValueError(f"tensor {name!r} is declared twice with different shapes")
                out[name] = decl
        return out

    def load(self, tensors: dict[str, Any]) -> None:
        """Hand every part its tensors (already on the device)."""
        for part in self.all_parts():
            part.bind({n: tensors[n] for n in part.weights()}, self.env)
        if hasattr(self.head, "tie") and not self.head.weights():
            self.head.tie(self.embedding.table)

    # --- cache ------------------------------------------------------------------------------

    def _plan_cache(self) -> None:
        """Sort the run order's cache needs into groups of equal requests."""
        paged: list[tuple[PagedKVRequest, int]] = []  # request, layers so far
        state: list[tuple[StateRequest, int]] = []
        self.bindings: list[CacheBinding | None] = []
        self.paged_group_of: list[int] = []  # for each paged request kind -> context group index
        requests = []
        for entry in self.spec.schedule:
            req = self.blocks[entry.layer].mixer.cache_request()
            requests.append(req)
            if entry.cache_from is not None:
                donor = self.bindings[entry.cache_from]
                if donor is None or requests[entry.cache_from] != req:
                    raise ValueError(
                        f"layer {entry.layer} cannot borrow the cache of run-order entry "
                        f"{entry.cache_from}: their cache needs differ")
                self.bindings.append(CacheBinding(donor.group, donor.slot, writes=False))
                continue
            if req is None:
                self.bindings.append(None)
                continue
            table = paged if isinstance(req, PagedKVRequest) else state
            for gi, (known, count) in enumerate(table):
                if known == req:
                    table[gi] = (known, count + 1)
                    self.bindings.append(CacheBinding(gi if table is paged else -1 - gi, count))
                    break
            else:
                table.append((req, 1))
                gi = len(table) - 1
                self.bindings.append(CacheBinding(gi if table is paged else -1 - gi, 0))
        self.paged_groups = [PagedGroupSpec(n, r.num_kv_heads, r.head_dim, r.window) for r, n in paged]
        self.state_groups = [StateGroupSpec(n, tuple(r.shape)) for r, n in state]
        # Context groups are listed paged first, then state: remap the negative indices.
        n_paged = len(self.paged_groups)
        self.bindings = [
            b if b is None or b.group >= 0 else CacheBinding(n_paged + (-1 - b.group), b.slot, b.writes)
            for b in self.bindings
        ]

    def footprint(self):
        """Parameters (every declared tensor once) and cache per token and per request, counted
        from the parts themselves: what an architecture's own ``footprint`` callable would say."""
        from ..config.model_config import Footprint

        parameters = sum(math.prod(d.shape) for d in self.declared_weights().values())
        per_token = sum(2 * g.num_layers * g.num_kv_heads * g.head_dim for g in self.paged_groups)
        per_request = sum(g.num_layers * math.prod(g.shape) for g in self.state_groups)
        return Footprint(parameters, per_token, per_request)

    # --- forward ----------------------------------------------------------------------------

    def forward(self, ctx, logit_rows):
        """Run the step's tokens through the run order; return 32-bit logits at
        ``logit_rows`` (indices into the step's flat tokens), or None if there are none."""
        h = self.embedding.forward(ctx.token_ids, ctx)
        for pos in self.positions.values():
            pos.apply_to_embedding(h, ctx)
        delta = None
        for entry, binding in zip(self.spec.schedule, self.bindings):
            delta = self.blocks[entry.layer].forward(h, delta, ctx, binding)
        if logit_rows is None or logit_rows.shape[0] == 0:
            # Nothing is read back, but the last add still belongs to the step.
            return None
        x = self.final_norm.add_norm(h, delta, ctx, rows=logit_rows, tag="norm.final")
        return self.head.forward(x, ctx)


def declared_weights(spec: ModelSpec) -> dict[str, WeightDecl]:
    """Names and shapes of every tensor a model of this description reads."""
    return Model(spec, "bfloat16", max_positions=1).declared_weights()
