"""What one step hands to every part: the tokens' places, and where their cache lies."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional

import torch

from .base import Runtime, Work


@dataclass
class StepContext:
    """One batch of (request, its next tokens), flattened to T token rows over S sequences.

    Device arrays are int32.  Rows of one sequence are adjacent and in ascending
    position.  Every request holds a slot while it lives; the block tables on the
    device have one row per slot and change only when the request's pages change.
    Rows past `num_tokens` (when a step is padded to a fixed size) have
    seq_of_token == slot_of_token == -1 and are skipped by every kernel that touches the cache.
    """

    rt: Runtime
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor  # [T]
    positions: torch.Tensor  # [T] absolute position of each row in its sequence
    seq_of_token: torch.Tensor  # [T] which sequence of this step a row belongs to
    slot_of_token: torch.Tensor  # [T] the row's request slot: its row in the block tables and state arrays
    cu_tokens: torch.Tensor  # [S+1] first row of each sequence
    seq_start: torch.Tensor  # [S] position of a sequence's first row in this step
    seq_len: torch.Tensor  # [S] tokens the sequence holds after this step
    state_slots: torch.Tensor  # [S] the sequence's slot in the fixed-size state arrays
    block_tables: Dict[int, torch.Tensor]  # cache group -> [slots, max_pages] page ids by request slot, -1 where none
    want_rows: torch.Tensor  # [W] rows whose logits are wanted
    num_wanted: int
    # the work lists that parts asked for (`Part.plan_key`, `Part.plan`), staged with the arrays above
    work: Dict[Hashable, Work] = field(default_factory=dict)
    # the sequences on the host, for parts that plan their launches or loop over sequences
    host_cu_tokens: List[int] = field(default_factory=list)
    host_seq_start: List[int] = field(default_factory=list)
    host_state_slots: List[int] = field(default_factory=list)
    max_query_len: int = 0
    max_seq_len: int = 0
    decode_only: bool = False


@dataclass
class PagedBinding:
    """The pages of one run of a layer, plane by plane: [num_pages, heads, page_size, width] each."""

    group: int
    planes: Dict[str, torch.Tensor]
    window: Optional[int]

    @property
    def k_pages(self) -> torch.Tensor:
        return self.planes["k"]

    @property
    def v_pages(self) -> torch.Tensor:
        return self.planes["v"]

    def block_table(self, ctx: StepContext) -> torch.Tensor:
        return ctx.block_tables[self.group]


@dataclass
class StateBinding:
    """The fixed-size states of one run of a layer: float32 [num_slots, *shape]; row = ctx.state_slots[seq]."""

    state: torch.Tensor
