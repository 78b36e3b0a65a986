"""The cache: a slot for each live sequence; per layer, keys and values in blocks of 64 tokens; beside
them per-sequence state of fixed size.

Layout.  Layers whose mixers ask for the same thing (``KVRequest`` / ``StateRequest``) form a group with
storage of its own.  A key/value group holds one tensor ``[layers, 2, blocks, kv_heads, 64, head_dim]``
(2 = keys, values) and a table ``[slots, blocks_per_sequence]`` of block ids: position p of the sequence
in slot s lies in block ``table[s, p // 64]`` at row ``p % 64``, in every layer of the group.  A block is
therefore one contiguous ``[64, head_dim]`` tile per key/value head, the unit the attention kernels load.
A group with a window gives blocks back as soon as all their positions have left the window.  A state
group holds ``[layers, slots, *shape]`` and is zeroed for a slot when a sequence starts.

The reference has no such component: its cache is a Python list of (K, V) per layer that grows by
``torch.cat`` (fms/modules/attention.py:186-212) and its fixed-size state is ``SSMCacheUnit``
(fms/modules/ssm.py:98-139).

All bookkeeping is on the host; the device sees only the block tables and the storage.  Nothing here
launches a kernel of its own except copies of changed table rows.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Union

import torch

from .requests import KVRequest, StateRequest
from .slots import BlockPool, CacheFull, SlotAllocator

BLOCK_TOKENS = 64


def round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class KVLayerView:
    """What an attention kernel needs of one layer's cache."""

    __slots__ = ("keys", "values", "table", "window", "block_tokens")

    def __init__(self, keys, values, table, window):
        self.keys = keys  # [blocks, kv_heads, 64, head_dim]
        self.values = values
        self.table = table  # [slots, blocks_per_sequence] int32, -1 where nothing is held
        self.window = window
        self.block_tokens = BLOCK_TOKENS


class StateLayerView:
    """One layer's fixed-size state: ``state[slot]`` belongs to the sequence in that slot."""

    __slots__ = ("state",)

    def __init__(self, state):
        self.state = state  # [slots, *shape]


class KVGroup:
    def __init__(self, request: KVRequest, layers: Sequence[int], n_blocks: int, max_slots: int,
                 blocks_per_sequence: int, dtype: torch.dtype, device: torch.device) -> None:
        self.request = request
        self.layers = list(layers)
        self.pool = BlockPool(n_blocks)
        self.blocks_per_sequence = blocks_per_sequence
        # one block and one table row more than the pool and the slots hand out: the spare slot (row max_slots) with
        # the spare block (n_blocks) at its first position, where a step's filler rows write and read
        self.storage = torch.zeros(
            (len(self.layers), 2, n_blocks + 1, request.kvheads, BLOCK_TOKENS, request.head_dim), dtype=dtype, device=device
        )
        self.table_host = torch.full((max_slots + 1, blocks_per_sequence), -1, dtype=torch.int32)
        self.table_host[max_slots, 0] = n_blocks
        self.table = self.table_host.to(device)
        self._dirty: set = set()

    def held_blocks(self, slot: int) -> List[int]:
        row = self.table_host[slot]
        return [int(b) for b in row.tolist() if b >= 0]

    def plan(self, slot: int, len_before: int, len_after: int):
        """(table indices whose blocks have left the window, table indices that need a block) for a step
        that takes the sequence in ``slot`` from len_before to len_after tokens."""
        row = self.table_host[slot].tolist()
        first_needed = 0
        if self.request.window:
            # the earliest query sits at len_before and sees keys from len_before - window + 1 on
            first_needed = max(0, len_before - self.request.window + 1) // BLOCK_TOKENS
        last_needed = (len_after - 1) // BLOCK_TOKENS
        if last_needed >= self.blocks_per_sequence:
            raise CacheFull(f"a sequence of {len_after} tokens exceeds {self.blocks_per_sequence * BLOCK_TOKENS}")
        stale = [i for i in range(first_needed) if row[i] >= 0]
        missing = [i for i in range(first_needed, last_needed + 1) if row[i] < 0]
        return stale, missing

    def give_back(self, slot: int, stale) -> None:
        if stale:
            row = self.table_host[slot]
            self.pool.free([int(row[i]) for i in stale])
            for i in stale:
                row[i] = -1
            self._dirty.add(slot)

    def take(self, slot: int, missing) -> None:
        if missing:
            row = self.table_host[slot]
            for i, b in zip(missing, self.pool.alloc(len(missing))):
                row[i] = b
            self._dirty.add(slot)

    def apply(self, slot: int, stale, missing) -> None:
        self.give_back(slot, stale)
        self.take(slot, missing)

    def release(self, slot: int) -> None:
        held = self.held_blocks(slot)
        if held:
            self.pool.free(held)
        self.table_host[slot].fill_(-1)
        self._dirty.add(slot)

    def sync(self) -> None:
        """Brings the changed rows of the table to the device: a snapshot in pinned memory (later host changes do not
        reach a copy that is still on its way), then one asynchronous copy per run of consecutive rows, on the
        stream of the kernels that read the table.  Nothing waits and no kernel is launched."""
        if not self._dirty:
            return
        idx = sorted(self._dirty)
        self._dirty.clear()
        if self.table.device.type != "cuda":
            self.table[idx] = self.table_host[idx]
            return
        staging = torch.empty((len(idx), self.blocks_per_sequence), dtype=torch.int32, pin_memory=True)
        torch.index_select(self.table_host, 0, torch.tensor(idx, dtype=torch.long), out=staging)
        start = 0
        for j in range(1, len(idx) + 1):
            if j == len(idx) or idx[j] != idx[j - 1] + 1:  # rows idx[start..j) are consecutive
                self.table[idx[start]:idx[start] + (j - start)].copy_(staging[start:j], non_blocking=True)
                start = j

    def view(self, layer: int) -> KVLayerView:
        i = self.layers.index(layer)
        return KVLayerView(self.storage[i, 0], self.storage[i, 1], self.table, self.request.window)


class StateGroup:
    def __init__(self, request: StateRequest, layers: Sequence[int], max_slots: int, dtype: torch.dtype,
                 device: torch.device) -> None:
        self.request = request
        self.layers = list(layers)
        self.storage = torch.zeros(  # one row more than there are slots: the spare slot's
            (len(self.layers), max_slots + 1) + tuple(request.shape), dtype=request.dtype or dtype, device=device
        )

    def reset(self, slot: int) -> None:
        self.storage[:, slot].zero_()

    def view(self, layer: int) -> StateLayerView:
        return StateLayerView(self.storage[self.layers.index(layer)])


class Cache:
    """Slots, lengths and the storage groups of one model.

    ``layer_requests[i]`` is what layer i's mixer asks for (None: nothing).  ``max_tokens`` is the most
    tokens that live sequences hold at any time, each sequence's count rounded up to a multiple of 64.
    """

    def __init__(self, layer_requests: Sequence[Optional[Union[KVRequest, StateRequest]]], max_tokens: int,
                 max_positions: int, dtype: torch.dtype, device, max_slots: Optional[int] = None) -> None:
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_positions = int(max_positions)
        n_blocks = max(1, round_up(int(max_tokens), BLOCK_TOKENS) // BLOCK_TOKENS)
        self.n_blocks = n_blocks
        self.max_slots = int(max_slots) if max_slots else n_blocks
        self.blocks_per_sequence = round_up(self.max_positions, BLOCK_TOKENS) // BLOCK_TOKENS
        self.slots = SlotAllocator(self.max_slots)
        # A slot that no sequence gets, with one block of its own in every group: rows that only fill a decode step up
        # to a size for which a graph is captured live there, at position 0, and what they compute is thrown away.
        self.spare_slot = self.max_slots
        # fixed-size state that every sequence has, whatever the architecture: its length (tokens in the
        # cache) and the position of its next token, which is what a position encoding sees.  They differ
        # by the position at which the sequence started (``begin(n, first_positions)``), 0 by default.
        self.length = [0] * self.max_slots
        self.position = [0] * self.max_slots
        self.groups: List[Union[KVGroup, StateGroup]] = []
        self._group_of_layer: Dict[int, Union[KVGroup, StateGroup]] = {}
        by_request: Dict[object, List[int]] = {}
        for layer, req in enumerate(layer_requests):
            if req is not None:
                by_request.setdefault(req, []).append(layer)
        for req, layers in by_request.items():
            if isinstance(req, KVRequest):
                group = KVGroup(req, layers, n_blocks, self.max_slots, self.blocks_per_sequence, dtype, self.device)
            elif isinstance(req, StateRequest):
                group = StateGroup(req, layers, self.max_slots, dtype, self.device)
            else:
                raise TypeError(f"unknown cache request {req!r}")
            self.groups.append(group)
            for layer in layers:
                self._group_of_layer[layer] = group

    # ---- slots -------------------------------------------------------------------------------
    def begin(self, n: int, first_positions: Optional[Sequence[int]] = None) -> List[int]:
        """Takes n slots for sequences that start together; their lengths are 0 and their state is zero.
        ``first_positions[i]``: the position of sequence i's first token (default 0)."""
        if n > self.slots.n_free:
            raise CacheFull(f"{n} slots wanted, {self.slots.n_free} of {self.max_slots} free")
        if first_positions is not None and (len(first_positions) != n or any(int(p) < 0 for p in first_positions)):
            raise ValueError("first_positions: one position >= 0 for each sequence")
        out = [self.slots.alloc() for _ in range(n)]
        for i, s in enumerate(out):
            self.length[s] = 0
            self.position[s] = int(first_positions[i]) if first_positions is not None else 0
            for g in self.groups:
                if isinstance(g, StateGroup):
                    g.reset(s)
        return out

    def release(self, slots: Sequence[int]) -> None:
        """Gives slots and all they hold back."""
        for s in slots:
            if not self.slots.is_held(s):
                raise ValueError(f"slot {s} is not held")
        for s in slots:
            for g in self.groups:
                if isinstance(g, KVGroup):
                    g.release(s)
            self.length[s] = 0
            self.position[s] = 0
            self.slots.free(s)

    # ---- one step ----------------------------------------------------------------------------
    def prepare(self, slots: Sequence[int], num_new: Sequence[int]) -> List[int]:
        """Before a step: checks it, holds the blocks it needs, brings the device tables up to date.
        Returns each sequence's length before the step.  Raises before anything is taken if the step
        does not fit."""
        if len(set(slots)) != len(slots):
            raise ValueError("a slot appears twice in one step")
        before = []
        for s, n in zip(slots, num_new):
            if not self.slots.is_held(s):
                raise ValueError(f"slot {s} is not held")
            if n <= 0:
                raise ValueError("every sequence of a step brings at least one token")
            if max(self.length[s], self.position[s]) + n > self.max_positions:
                raise CacheFull(
                    f"slot {s}: {max(self.length[s], self.position[s])} + {n} tokens exceed the model's "
                    f"{self.max_positions} positions"
                )
            before.append(self.length[s])
        plans = []
        for g in self.groups:
            if isinstance(g, KVGroup):
                plan = [g.plan(s, b, b + n) for s, n, b in zip(slots, num_new, before)]
                want = sum(len(m) for _, m in plan) - sum(len(st) for st, _ in plan)
                if want > g.pool.n_free:
                    raise CacheFull(f"{want} blocks wanted, {g.pool.n_free} of {g.pool.n_blocks} free")
                plans.append((g, plan))
        for g, plan in plans:
            # all that has left a window first, then what is needed: the check above counted on both
            for s, (stale, _) in zip(slots, plan):
                g.give_back(s, stale)
            for s, (_, missing) in zip(slots, plan):
                g.take(s, missing)
            g.sync()
        return before

    def prepare_decode(self, slots: Sequence[int]) -> None:
        """``prepare`` for a step of one token per sequence, without looking at whole table rows: a block
        is needed only when a sequence's length is a multiple of 64, and a window only moves then."""
        work = []
        for s in slots:
            n = self.length[s]
            if max(n, self.position[s]) + 1 > self.max_positions:
                raise CacheFull(f"slot {s}: {max(n, self.position[s])} + 1 tokens exceed the model's "
                                f"{self.max_positions} positions")
            if n % BLOCK_TOKENS == 0 or any(isinstance(g, KVGroup) and g.request.window for g in self.groups):
                work.append(s)
        if work:
            self.prepare(work, [1] * len(work))

    def commit(self, slots: Sequence[int], num_new: Sequence[int]) -> None:
        for s, n in zip(slots, num_new):
            self.length[s] += n
            self.position[s] += n

    def offset(self, slot: int) -> int:
        """The position at which the sequence in ``slot`` started."""
        return self.position[slot] - self.length[slot]

    def layer_view(self, layer: int):
        g = self._group_of_layer.get(layer)
        return None if g is None else g.view(layer)

    # ---- accounting --------------------------------------------------------------------------
    def tokens_held(self) -> int:
        """Tokens of storage held by live sequences in the largest group, in whole blocks."""
        held = [g.pool.n_held for g in self.groups if isinstance(g, KVGroup)]
        return (max(held) if held else 0) * BLOCK_TOKENS

    def bytes_per_token(self) -> int:
        total = 0
        for g in self.groups:
            if isinstance(g, KVGroup):
                total += 2 * len(g.layers) * g.request.kvheads * g.request.head_dim * g.storage.element_size()
        return total
