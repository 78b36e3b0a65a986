"""The tokens of one step and where they belong, as the kernels need it.

A step brings, for each of n sequences, its next tokens (all of a prompt, or one token); rows of all
sequences follow one another without padding.  Everything the device needs to place a row lies in
small int32 arrays: the row's position in its sequence, the sequence it belongs to, each sequence's
slot, first row and length after the step.  Causality is by position: the row at position p sees cached
positions up to p, so a continuation of several tokens onto a sequence that is already cached needs no
mask (the reference needs an explicit one there, fms/modules/attention.py:268-271).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch


class Batch:
    """Device arrays of one step.  Built by ``Batch.from_lists`` for a general step, or filled in place
    by the decode loop (``engine.step.DecodeState``) when every sequence brings one token."""

    def __init__(self) -> None:
        self.n_seqs = 0
        self.n_tokens = 0
        self.decode = False  # every sequence brings exactly one token
        self.max_new = 0  # most tokens any sequence brings
        self.max_len_after = 0  # longest sequence after the step (host value; capacity when unknown)
        self.total_len = 0  # tokens of all sequences after the step, as far as the host knows (kernels are chosen by it)
        self.num_new: List[int] = []
        self.tokens: Optional[torch.Tensor] = None  # [n_tokens] int32
        self.positions: Optional[torch.Tensor] = None  # [n_tokens] int32: each token's place in its sequence's cache
        # [n_tokens] int32: the position each token's encoding sees, where that is not its place in the cache (a
        # sequence that started at another position than 0); None: the same
        self.position_ids: Optional[torch.Tensor] = None
        self.token_seq: Optional[torch.Tensor] = None  # [n_tokens] int32, index into the arrays below
        self.first_row: Optional[torch.Tensor] = None  # [n_seqs + 1] int32
        self.slots: Optional[torch.Tensor] = None  # [n_seqs] int32
        self.len_after: Optional[torch.Tensor] = None  # [n_seqs] int32
        self.want_rows: Optional[torch.Tensor] = None  # [n_wanted] int32 rows whose logits are returned
        self.n_wanted = 0
        self._tiles = {}
        self.scratch = {}  # what a step's layers share (a table of rotation angles, ...); emptied when a step starts

    @staticmethod
    def from_lists(slots: Sequence[int], len_before: Sequence[int], tokens: Sequence[Sequence[int]],
                   want: Sequence[Sequence[int]], device, offsets: Optional[Sequence[int]] = None) -> "Batch":
        """``offsets[i]``: the position at which sequence i started (its token at place p of the cache has the
        position p + offsets[i]); None: every sequence started at 0."""
        b = Batch()
        b.n_seqs = len(slots)
        b.num_new = [len(t) for t in tokens]
        b.n_tokens = sum(b.num_new)
        b.max_new = max(b.num_new)
        b.decode = b.max_new == 1
        b.max_len_after = max(lb + n for lb, n in zip(len_before, b.num_new))
        b.total_len = sum(len_before) + b.n_tokens
        flat, pos, seq, first, rows = [], [], [], [0], []
        for i, (lb, t, w) in enumerate(zip(len_before, tokens, want)):
            base = first[-1]
            flat.extend(int(x) for x in t)
            pos.extend(range(lb, lb + len(t)))
            seq.extend([i] * len(t))
            first.append(base + len(t))
            for j in w:
                if not (0 <= j < len(t)):
                    raise ValueError(f"wanted place {j} outside the {len(t)} tokens of this step")
                rows.append(base + j)
        len_after = [lb + n for lb, n in zip(len_before, b.num_new)]
        ids = [p + offsets[i] for p, i in zip(pos, seq)] if offsets is not None and any(offsets) else []
        packed = torch.tensor(flat + pos + seq + first + list(slots) + len_after + ids + rows, dtype=torch.int32)
        packed = packed.to(device)
        n, s = b.n_tokens, b.n_seqs
        o = 0
        b.tokens = packed[o:o + n]; o += n
        b.positions = packed[o:o + n]; o += n
        b.token_seq = packed[o:o + n]; o += n
        b.first_row = packed[o:o + s + 1]; o += s + 1
        b.slots = packed[o:o + s]; o += s
        b.len_after = packed[o:o + s]; o += s
        if ids:
            b.position_ids = packed[o:o + n]; o += n
        b.want_rows = packed[o:]
        b.n_wanted = len(rows)
        b.len_before_host = list(len_before)
        return b

    def query_tiles(self, tile_rows: int) -> torch.Tensor:
        """[tiles, 2] int32: (sequence index, first row of the tile within the sequence's new tokens), for
        kernels that give each thread block ``tile_rows`` rows of one sequence."""
        if tile_rows not in self._tiles:
            t = []
            for i, n in enumerate(self.num_new):
                t.extend((i, r) for r in range(0, n, tile_rows))
            self._tiles[tile_rows] = torch.tensor(t, dtype=torch.int32).to(self.tokens.device)
        return self._tiles[tile_rows]
