"""The step function: a batch of sequences that start together, with unequal lengths; their prompts in
one step, then one token each.

``Engine.step`` runs only the tokens it is given, as one batch, against the cache that earlier steps
left, and returns float32 logits at the wanted places.  The reference's counterpart is
``LLaMA.forward(..., past_key_value_states, use_cache=True)`` (fms/models/llama.py:425-450) on a
left-padded rectangle with a mask; here rows are ragged, nothing is padded and causality is by position.

A step in which every sequence brings one token and wants its logits is a decode step.  It runs the same
kernels as any other step, but from arrays that stay on the device (tokens, positions, lengths, slots)
and, from its second occurrence on, as one CUDA graph launch instead of some hundred kernel launches.
More than eight sequences are filled up to the next of a few sizes (12, 16, 24, 32, 48, 64, ...) with rows that
live in the cache's spare slot and whose results are thrown away, so that a batch whose sequences end one by one
goes on through a handful of captured graphs instead of capturing one for every number of sequences.
"""
from __future__ import annotations

import collections
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..cache.cache import Cache
from ..kernels import ops
from .batch import Batch

# Tests that replace the kernels by plain restatements clear this to drive the host logic on the CPU.
_REQUIRE_CUDA = True


def decode_rows(n: int) -> int:
    """Rows of the decode step that n sequences take: n up to 8 (the weight-streaming products take 1 to 8 rows as
    they are), else the next of 12, 16, 24, 32, 48, 64, 96, 128, ... (a power of two, or one and a half)."""
    if n <= 8:
        return n
    size = 8
    while True:
        for rows in (size + size // 2, 2 * size):
            if rows >= n:
                return rows
        size *= 2


class _DecodeBuffers:
    """Device arrays of decode steps of n rows, and the CUDA graphs captured over them."""

    def __init__(self, n: int, device, spare_slot: int) -> None:
        self.n = n
        ar = torch.arange(n + 1, dtype=torch.int32, device=device)
        self.batch = Batch()
        b = self.batch
        b.n_seqs = b.n_tokens = b.n_wanted = n
        b.decode, b.max_new, b.num_new = True, 1, [1] * n
        b.tokens = torch.zeros(n, dtype=torch.int32, device=device)
        b.positions = torch.zeros(n, dtype=torch.int32, device=device)
        b.token_seq = ar[:n].clone()
        b.first_row = ar
        b.slots = torch.full((n,), spare_slot, dtype=torch.int32, device=device)
        b.len_after = torch.zeros(n, dtype=torch.int32, device=device)  # between steps: the current lengths
        # for sequences that did not start at position 0: what the encoding sees (batch.position_ids points at it
        # while any of the loaded sequences has an offset, else stays None)
        self.offsets = torch.zeros(n, dtype=torch.int32, device=device)
        self.position_ids = torch.zeros(n, dtype=torch.int32, device=device)
        b.want_rows = ar[:n].clone()
        self.tokens_host = torch.zeros(n, dtype=torch.int32).pin_memory() if torch.device(device).type == "cuda" \
            else torch.zeros(n, dtype=torch.int32)
        self.tokens_np = self.tokens_host.numpy()  # the same memory, for cheap writes from lists
        self.copied = None  # event after the last copy out of tokens_host
        self.loaded: Optional[Tuple[int, ...]] = None  # slots whose state the arrays hold
        self.lengths: List[int] = []  # their lengths, as the device arrays have them
        self.seen: Dict[tuple, int] = {}  # a graph's key -> how often a step came with it


class Engine:
    """A model's decoder together with a cache of a given size."""

    def __init__(self, model, max_tokens: int, max_slots: Optional[int] = None, sampling: bool = True,
                 use_graphs: bool = True, max_graphs: int = 48) -> None:
        """``max_graphs``: the most captured decode steps the engine keeps (one per number of rows, see
        ``decode_rows``, and bound on the sequences' lengths).  When one more is captured, the one used longest ago is dropped with its logits buffer, and
        all captures draw their buffers from one pool; so a batch whose requests end one by one holds at most
        ``max_graphs`` logits buffers [sequences, vocabulary] and one set of a step's intermediate buffers.  The
        default holds what an engine meets that serves every size (some 14 numbers of rows up to 128, each with the
        few bounds its lengths pass through) without capturing anything twice."""
        if model.decoder is None:
            raise ValueError("the model has no weights yet")
        self.model = model
        self.decoder = model.decoder
        self.device = model.device
        if _REQUIRE_CUDA and self.device.type != "cuda":
            raise RuntimeError(f"the engine runs on a CUDA device, not on {self.device}; there is no CPU path")
        self.vocab_size = self.decoder.spec.vocab_size
        if self.device.type == "cuda":
            self._compile_what_this_model_needs(sampling)
        self.cache = Cache(self.decoder.cache_requests(), max_tokens, self.decoder.spec.max_positions,
                           self.decoder.dtype, self.device, max_slots)
        self.use_graphs = use_graphs and self.device.type == "cuda"
        # decode steps of more than 8 sequences are filled up to one of a few sizes (``decode_rows``): it pays where a
        # size means a captured graph
        self.fill_rows = self.use_graphs
        self.max_graphs = max(1, int(max_graphs))
        self._decode: Dict[int, _DecodeBuffers] = {}
        # (rows, bound on the lengths, with position offsets) -> (graph, logits), least recently used first
        self._graphs: "collections.OrderedDict[tuple, Tuple[object, torch.Tensor]]" = collections.OrderedDict()
        self._graph_pool = None
        self.graphs_captured = 0
        self.h2d_bytes = 0  # bytes copied host -> device by steps since the engine was made
        self.graph_launches = 0
        self.kernels_per_graph = 0  # own kernels inside the decode graph captured last

    def _compile_what_this_model_needs(self, sampling: bool) -> None:
        """Compiles, side by side, the kernel libraries this model's parts name and that are not built yet."""
        from ..kernels import build

        names = list(dict.fromkeys(self.decoder.kernel_libraries(self.decoder.dtype)))
        if sampling:
            names.append("sampling")
        build.compile_many(names)

    # ---- sequences ---------------------------------------------------------------------------
    def begin(self, n: int, first_positions: Optional[Sequence[int]] = None) -> List[int]:
        """Slots for n sequences that start together.  ``first_positions``: the position of each sequence's first
        token, where that is not 0 (the position encoding sees it; the cache holds the tokens from its place 0 on)."""
        return self.cache.begin(n, first_positions)

    def release(self, slots: Sequence[int]) -> None:
        self.cache.release(slots)

    def length(self, slot: int) -> int:
        return self.cache.length[slot]

    # ---- one step ----------------------------------------------------------------------------
    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """Feeds ``tokens[i]`` to the sequence in ``slots[i]``.  ``want[i]`` lists the places among
        ``tokens[i]`` whose logits are returned (default: the last).  Returns [wanted, vocab] float32 on the
        device, in the order of the sequences and of ``want``."""
        if len(slots) != len(tokens) or not slots:
            raise ValueError("a step needs one token list per slot, and at least one")
        for t in tokens:
            if len(t) and not (0 <= min(t) and max(t) < self.vocab_size):
                bad = next(x for x in t if not (0 <= int(x) < self.vocab_size))
                raise ValueError(f"token id {bad} outside the vocabulary of {self.vocab_size}")
        if all(len(t) == 1 for t in tokens) and (want is None or all(list(w) == [0] for w in want)):
            return self.decode(slots, [int(t[0]) for t in tokens]).clone()
        if want is None:
            want = [[len(t) - 1] for t in tokens]
        num_new = [len(t) for t in tokens]
        before = self.cache.prepare(slots, num_new)
        batch = Batch.from_lists(slots, before, tokens, want, self.device, [self.cache.offset(s) for s in slots])
        self.h2d_bytes += 4 * ((3 if batch.position_ids is None else 4) * batch.n_tokens + 3 * batch.n_seqs + 1
                               + batch.n_wanted)
        logits = self.decoder.forward(batch, self.cache)
        self.cache.commit(slots, num_new)
        return logits

    def decode(self, slots: Sequence[int], tokens: Optional[Sequence[int]] = None,
               tokens_device: Optional[torch.Tensor] = None, horizon: int = 0) -> torch.Tensor:
        """One token for each sequence; logits [n, vocab] for each.  The tokens come from the host
        (``tokens``) or are already on the device (``tokens_device``, int32 [n], e.g. what the sampler
        wrote).  ``horizon``: the longest any of these sequences will get in this run, if the caller knows
        it; the launch is then sized for it once, instead of growing (and being captured anew) as the
        sequences grow.  The result is a buffer that the next decode step (of any number of sequences)
        may overwrite: use it, or copy it, before that."""
        n = len(slots)
        if len(set(slots)) != n:
            raise ValueError("a slot appears twice in one step")
        for s in slots:
            if not self.cache.slots.is_held(s):
                raise ValueError(f"slot {s} is not held")
        rows = decode_rows(n) if self.fill_rows else n  # rows beyond n only fill the step up to a captured size
        buf = self._decode.get(rows)
        if buf is None:
            buf = self._decode[rows] = _DecodeBuffers(rows, self.device, self.cache.spare_slot)
        key = tuple(slots)
        lengths = [self.cache.length[s] for s in slots]
        self.cache.prepare_decode(slots)
        if buf.copied is not None:
            buf.copied.synchronize()  # the last copy out of the pinned array is over
        if buf.loaded != key or buf.lengths != lengths:
            offsets = [self.cache.offset(s) for s in slots]
            fill = rows - n
            state = torch.tensor([list(slots) + [self.cache.spare_slot] * fill, lengths + [0] * fill, offsets + [0] * fill],
                                 dtype=torch.int32)
            buf.batch.slots.copy_(state[0])
            buf.batch.len_after.copy_(state[1])
            buf.offsets.copy_(state[2])
            buf.batch.position_ids = buf.position_ids if any(offsets) else None
            buf.loaded, buf.lengths = key, lengths
            self.h2d_bytes += 12 * rows
        if tokens_device is not None:
            buf.batch.tokens[:n].copy_(tokens_device)
        else:
            buf.tokens_np[:n] = tokens  # the filler rows keep whatever valid token they had (0 at first)
            buf.batch.tokens.copy_(buf.tokens_host, non_blocking=True)
            self.h2d_bytes += 4 * rows
            if self.device.type == "cuda":
                if buf.copied is None:
                    buf.copied = torch.cuda.Event()
                buf.copied.record()
        buf.batch.total_len = sum(lengths) + n  # read when a graph is captured: the lengths only grow from here
        try:
            logits = self._run_decode(buf, max(max(lengths) + 1, min(int(horizon), self.cache.max_positions)))
        except BaseException:
            # the device arrays may be a step ahead of the cache now: have the next step bring them anew
            buf.loaded, buf.lengths = None, []
            raise
        self.cache.commit(slots, [1] * n)
        buf.lengths = [x + 1 for x in lengths]
        return logits if rows == n else logits[:n]

    def _decode_body(self, buf: _DecodeBuffers) -> torch.Tensor:
        spare = self.cache.spare_slot
        if buf.batch.position_ids is None:
            ops.decode_advance(buf.batch.positions, buf.batch.len_after, None, None, buf.batch.slots, spare)
        else:
            ops.decode_advance(buf.batch.positions, buf.batch.len_after, buf.offsets, buf.position_ids, buf.batch.slots, spare)
        return self.decoder.forward(buf.batch, self.cache)

    def _run_decode(self, buf: _DecodeBuffers, longest: int) -> torch.Tensor:
        # the bound on key splits that the launch is sized for: a power of two of 256-token splits, so
        # that a graph serves many steps; blocks beyond a sequence's own length return at once
        bound = 256
        while bound < longest:
            bound *= 2
        bound = min(bound, max(256, (self.cache.max_positions + 255) // 256 * 256))
        buf.batch.max_len_after = max(bound, longest)
        if not self.use_graphs:
            return self._decode_body(buf)
        key = (buf.n, bound, buf.batch.position_ids is not None)
        entry = self._graphs.get(key)
        if entry is None:
            buf.seen[key] = buf.seen.get(key, 0) + 1
            if buf.seen[key] == 1:
                return self._decode_body(buf)  # first occurrence: plain launches (they also warm everything up)
            while len(self._graphs) >= self.max_graphs:
                self._graphs.popitem(last=False)  # the one used longest ago, with its logits buffer
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            graph = torch.cuda.CUDAGraph()
            before = ops.launches
            with torch.cuda.graph(graph, pool=self._graph_pool):
                logits = self._decode_body(buf)
            self.kernels_per_graph = ops.launches - before
            self.graphs_captured += 1
            entry = self._graphs[key] = (graph, logits)
        else:
            self._graphs.move_to_end(key)
        entry[0].replay()
        self.graph_launches += 1
        return entry[1]

    def warm_up(self, sizes: Sequence[int], horizon: int) -> None:
        """Captures the decode graphs of the given numbers of sequences ahead of the first request: two steps of
        throw-away sequences each (the first runs uncaptured, the second captures).  ``horizon``: the longest a
        sequence will get, as ``decode`` takes it (graphs are kept per bound on the lengths, a power of two of 256)."""
        if not self.use_graphs:
            return
        by_rows = {}
        for k in sorted(int(k) for k in sizes):
            by_rows.setdefault(decode_rows(k) if self.fill_rows else k, k)  # one number of sequences for each size of step
        for n in by_rows.values():
            if n > self.cache.slots.n_free:
                raise ValueError(f"warm_up: {n} sequences, {self.cache.slots.n_free} slots free")
            slots = self.begin(n)
            try:
                for _ in range(2):
                    self.decode(slots, [0] * n, horizon=horizon)
            finally:
                self.release(slots)

    def check(self) -> None:
        """Raises if a kernel met something the host should have prevented (synchronises)."""
        ops.check_error_flag(self.device)
