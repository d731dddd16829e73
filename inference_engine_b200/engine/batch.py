"""What one step is given and what the parts see of it.

A step is a batch of ``(request, its next tokens)``: whole prompts, portions of prompts cut
anywhere, and single decoded tokens side by side (the reference's flattened ``[1, N]``
layout, engine/runtime/engine.py:186-197).  All of the step's index data is packed into one
pinned host array and copied to the device in one transfer; the parts and kernels get views
of that one device array.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass
class StepEntry:
    """``tokens``: the request's next tokens; ``start``: the position of ``tokens[0]`` (how
    many tokens of the request are already cached); ``want``: the places among ``tokens``
    whose logits are asked for."""

    req_id: Any
    tokens: list[int]
    start: int
    want: list[int] = field(default_factory=list)


@dataclass
class PagedGroupView:
    k: Any  # [layers_in_group, pages + 1, kv_heads, page_size, head_dim]
    v: Any
    page_size: int
    window: int | None
    block_tables: Any  # int32 [B, table_width]; -1 where a window has passed
    table_width: int
    slot_mapping: Any  # int32 [N]: flat slot (page * page_size + offset) of each new token
    ragged: int = 0  # a launch hint: 1 the contexts this group's mixers see differ much in length; 2, 3 so many that blocks of as many warps pay


@dataclass
class StateGroupView:
    state: Any  # float32 [layers_in_group, slots + 1, *shape]
    slots: Any  # int32 [B] on the device
    slots_host: list[int]


@dataclass
class StepContext:
    ops: Any
    ws: Any
    num_tokens: int  # N
    num_seqs: int  # B
    token_ids: Any  # int32 [N]
    positions: Any  # int32 [N]
    seq_of_token: Any  # int32 [N]
    cu_q: Any  # int32 [B + 1]: first flat token of each sequence
    ctx_lens: Any  # int32 [B]: tokens cached after this step
    groups: list[Any]  # paged groups first, then state groups
    # host-side copies, for parts that loop over sequences and for launch decisions
    q_starts: list[int]
    q_lens: list[int]
    start_positions: list[int]
    max_q_len: int
    max_ctx_len: int
    padded: bool = False  # a fixed-size launch: sizes above are upper bounds
    ragged: tuple = ()  # per paged group: its ``ragged`` hint (part of what a captured launch is keyed by)
    decode_order: Any = None  # int32 [B] on the device: the sequences by context length, the longest first
    # A launch of fixed size that must serve every step that fits (a captured step with prompt
    # portions): (tokens, sequences, context length) the launch is sized for.  Launch decisions are
    # then taken from these bounds alone, never from the step's own lengths.
    bounds: tuple | None = None
