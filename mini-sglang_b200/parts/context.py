"""What a step hands to the parts: the flattened token stream of the batch, per-request
lengths, and per cache group the block tables and token slots.

All index tensors are int32 on the device.  Requests are in batch order; request r owns the
tokens q_start[r] .. q_start[r+1]-1 of the stream, its cache holds kv_len[r] tokens once this
step's tokens are written, so its first new token sits at position kv_len[r] - q_len[r].
"""

from __future__ import annotations

import dataclasses
from typing import Sequence, Dict, List, Optional, Tuple

import torch


@dataclasses.dataclass
class GroupContext:
    block_table: torch.Tensor          # [B, max_pages] int32, page ids of this group
    out_loc: torch.Tensor              # [T] int32, token slot (page * P + offset) of every new token
    nsplit: Optional[torch.Tensor]     # [B] int32, kv splits per request (None: 1)
    max_split: int
    window: Optional[int]
    host_nsplit: Optional[Sequence[int]] = None     # the host's copy of nsplit (None: not known here)
    order: Optional[torch.Tensor] = None            # [B] int32, uniform decode only: the requests by falling number of keys
    even: Optional[torch.Tensor] = None             # int32, uniform decode only: the keys dealt out evenly over even_nb blocks
    even_nb: int = 0                                # per kv head (ops.even_cut_size words; nsplit then holds the pieces a request)


@dataclasses.dataclass
class StepContext:
    T: int
    B: int
    page_size: int
    input_ids: torch.Tensor            # [T]
    positions: torch.Tensor            # [T]
    q_start: torch.Tensor              # [B + 1]
    kv_len: torch.Tensor               # [B]
    token_req: torch.Tensor            # [T] request index of every token
    slots: torch.Tensor                # [B] request slot (row of the state arrays)
    groups: List[GroupContext]
    host_q_lens: List[int]
    host_kv_lens: List[int]
    host_slots: List[int]
    uniform_decode: bool = False       # every request brings exactly one token (fixed launch shapes)
    all_rows_wanted: bool = False      # the wanted rows are all T rows in order (what a decode step asks for)
    workspace: Optional["Workspace"] = None


class Workspace:
    """Scratch tensors by name, grown on demand and kept, so that steady-state steps allocate
    nothing and captured graphs keep their addresses."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}
        self._retired: List[torch.Tensor] = []      # outgrown buffers stay alive: captured graphs point at them

    def get(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
        buf = self._bufs.get(name)
        if buf is None or buf.numel() < numel or buf.dtype != dtype:
            if buf is not None:
                self._retired.append(buf)
            buf = torch.empty(max(numel, 1), dtype=dtype, device=self.device)
            self._bufs[name] = buf
        return buf[:numel]


@dataclasses.dataclass
class KVCacheView:
    """The K and V arrays of one cache, [pages + 1, kv heads, page size, head size], with the
    group context that addresses them."""
    k: torch.Tensor
    v: torch.Tensor
    group: GroupContext
    page_size: int


@dataclasses.dataclass
class StateCacheView:
    """A per-request state array [max requests + 1, ...]; row ctx.slots[r] belongs to request r."""
    state: torch.Tensor
