"""Interfaces that every part of a layer implements.

A part is built from a :class:`~inference_engine_b200.config.spec.PartSpec` (its sizes and
constants are parameters), says which tensors it reads (:meth:`Part.weights`), receives them
(:meth:`Part.bind`) and then runs on device tensors.  No part knows which model it is in:
it sees its own parameters, the step's :class:`StepContext` and, for a mixer, the binding
to its cache.

Categories and what each must provide
-------------------------------------
``norm``          ``add_norm(h, delta, ctx, rows=None, tag="norm") -> x``: add ``delta`` to
                  the 32-bit residual ``h`` in place (unless ``rows`` selects rows, then
                  nothing is modified) and return the normalised activations.
``position``      a :class:`PositionEncoding`: ``rotary_table()``/``rotary_dim`` for encodings
                  applied to queries and keys, ``apply_to_embedding`` for additive ones.
``mixer``         ``cache_request()`` (what it keeps per request: pages of keys and values,
                  a fixed-size state, or nothing) and
                  ``forward(x, ctx, binding) -> delta`` (32-bit ``[N, hidden]``, or
                  ``[S, N, hidden]`` partial sums that the next norm adds in order).
``feed_forward``  ``forward(x, ctx) -> delta`` (32-bit ``[N, hidden]``).
``block``         the arrangement: ``forward(h, delta, ctx, binding) -> delta`` where ``h``
                  is the residual stream and ``delta`` the not-yet-added output of the
                  previous block.
``embedding``     ``forward(token_ids, ctx) -> h`` (32-bit residual stream).
``head``          ``forward(x, ctx) -> logits`` (32-bit ``[rows, vocab]``).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass(frozen=True)
class WeightDecl:
    """A tensor a part reads from the checkpoint.

    ``role``: ``matrix`` (used in a matrix product; kept in the compute dtype),
    ``vector`` (scales and biases; used in 32-bit), ``table`` (rows gathered by index) or
    ``int_table`` (integers, kept as int32).
    ``init`` says how the random-weights mode draws it: ``normal`` is N(0, std),
    ``ones_plus_normal`` is 1 + N(0, std), ``zeros`` and ``ones`` are constant.
    """

    shape: tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"


@dataclass(frozen=True)
class PagedKVRequest:
    """A mixer that keeps keys and values per token.  ``window`` = how many of the latest
    positions a query may see (``None`` = all): pages behind the window are given back."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateRequest:
    """A mixer that keeps a state of fixed size per request (32-bit floats of ``shape``)."""

    shape: tuple[int, ...]


@dataclass(frozen=True)
class CacheBinding:
    """Where one run of a mixer finds its cache: the cache group, the layer's slot in the
    group's storage, and whether this run writes (a run that borrows another layer's cache
    only reads)."""

    group: int
    slot: int
    writes: bool = True


@dataclass
class BuildEnv:
    """What a part may look at while it is built."""

    hidden_size: int
    dtype: str  # "bfloat16" or "float32": the compute dtype of activations and matrices
    max_positions: int  # positions the engine will ever feed (tables are sized for it)
    positions: dict[str, Any]  # built position encodings by name
    device: Any = None

    @property
    def torch_dtype(self):
        import torch

        return torch.bfloat16 if self.dtype == "bfloat16" else torch.float32


class Part:
    category = "part"

    def weights(self) -> dict[str, WeightDecl]:
        """Full tensor names this part reads, with their shapes."""
        return {}

    def bind(self, tensors: dict[str, Any], env: BuildEnv) -> None:
        """Receive the tensors named by :meth:`weights`, already on the device in their
        stored dtype; cast and fuse them as the part needs."""

    def parts(self) -> list["Part"]:
        """Nested parts (a block returns its mixer, feed-forward and norms)."""
        return []


class PositionEncoding(Part):
    category = "position"
    rotary_dim = 0  # leading dims of each head that are rotated (0 = none)

    def rotary_table(self):
        """``[max_positions, 2, rotary_dim // 2]`` 32-bit cos and sin, or None."""
        return None

    def apply_to_embedding(self, h, ctx) -> None:
        """Additive encodings add to the embedded tokens here; default: nothing."""


class Mixer(Part):
    category = "mixer"

    def cache_request(self) -> PagedKVRequest | StateRequest | None:
        return None

    def forward(self, x, ctx, binding: CacheBinding | None):
        raise NotImplementedError


class FeedForward(Part):
    category = "feed_forward"

    def forward(self, x, ctx):
        raise NotImplementedError


class Norm(Part):
    category = "norm"

    def add_norm(self, h, delta, ctx, rows=None, tag: str = "norm"):
        raise NotImplementedError


class Block(Part):
    category = "block"

    mixer: Mixer

    def forward(self, h, delta, ctx, binding: CacheBinding | None):
        raise NotImplementedError
