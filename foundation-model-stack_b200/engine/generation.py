"""The generation loop, in the manner of ``fms.utils.generation.generate``
(fms/utils/generation.py:182-369): prompts in, prompts plus new tokens out.

Differences that the cache makes possible: prompts of unequal lengths need no padding; a sequence that
meets a stop token leaves the batch at once, its slot is given back and the others go on (the reference
keeps extending finished rows and, for more than one row, stops everything at the first stop token,
fms/utils/generation.py:338-341); more prompts than fit in one batch run as one batch after another.
"""
from __future__ import annotations

import time
from typing import Callable, List, Optional, Sequence, Union

import torch

from ..sampling.sampler import Sampler

Prompts = Union[torch.Tensor, Sequence[torch.Tensor], Sequence[Sequence[int]]]


def _as_lists(input_ids: Prompts):
    """(list of token lists, kind) where kind is "1d", "2d" or "list"."""
    if isinstance(input_ids, torch.Tensor):
        if input_ids.dim() == 1:
            return [input_ids.tolist()], "1d"
        if input_ids.dim() == 2:
            return [row.tolist() for row in input_ids], "2d"
        raise TypeError("input_ids must be one- or two-dimensional")
    out = []
    for p in input_ids:
        out.append(p.tolist() if isinstance(p, torch.Tensor) else [int(t) for t in p])
    return out, "list"


def pad_input_ids(input_ids_list: Sequence[torch.Tensor], min_pad_length: int = 0, is_causal_mask: bool = True,
                  padding_side: str = "left", position_ids_offset: int = 0, pad_token_id: int = 0):
    """Prompts of unequal lengths as one rectangle, with what tells its padding from its tokens: the call
    of the reference's users (fms/utils/generation.py:16-109, same arguments and results).  Returns the
    [n, width] ids, filled with ``pad_token_id`` on ``padding_side``, and a mapping with ``position_ids``
    [n, width] (a prompt's own count from 0 plus ``position_ids_offset``; the offset alone on padding) and
    ``mask`` [n, width, width] (0 where a row may look, -inf elsewhere: tokens at tokens, padding at
    padding, and not ahead if ``is_causal_mask``).  ``generate`` takes both back through ``extra_kwargs``
    and runs the prompts without their padding, so padding changes no result."""
    if padding_side not in ("left", "right"):
        raise ValueError('padding_side must be "left" or "right"')
    prompts = [torch.as_tensor(p) for p in input_ids_list]
    if not prompts:
        raise ValueError("no prompts")
    width = max([int(min_pad_length)] + [int(p.shape[0]) for p in prompts])
    device = prompts[0].device
    ids = torch.full((len(prompts), width), int(pad_token_id), dtype=torch.long, device=device)
    real = torch.zeros((len(prompts), width), dtype=torch.bool, device=device)
    position = torch.zeros((len(prompts), width), dtype=torch.long, device=device)
    for i, p in enumerate(prompts):
        n = int(p.shape[0])
        where = slice(width - n, width) if padding_side == "left" else slice(0, n)
        ids[i, where] = p.to(torch.long)
        real[i, where] = True
        position[i, where] = torch.arange(n, device=device)
    allowed = real[:, :, None] == real[:, None, :]
    if is_causal_mask:
        allowed = allowed.tril()
    mask = torch.zeros(allowed.shape, device=device).masked_fill(~allowed, float("-inf"))
    return ids, {"mask": mask, "position_ids": position + int(position_ids_offset)}


def _tokens_of_padded_rows(input_ids: torch.Tensor, position_ids: torch.Tensor):
    """For each row of a rectangle that ``pad_input_ids`` made: (first, last + 1) of its tokens.  A prompt
    counts its positions up from the smallest one, padding stays at it; a row whose positions say nothing
    about the side (one token) is taken as padded on the left, the default."""
    if position_ids.shape != input_ids.shape:
        raise ValueError(f"position_ids {tuple(position_ids.shape)} for input_ids {tuple(input_ids.shape)}")
    spans = []
    width = input_ids.shape[1]
    for row in position_ids.tolist():
        n = max(row) - min(row) + 1
        if n > width:
            raise ValueError("position_ids are not those of pad_input_ids")
        left = row[width - n:] == list(range(min(row), min(row) + n))
        right = row[:n] == list(range(min(row), min(row) + n))
        if not (left or right):
            raise ValueError("position_ids are not those of pad_input_ids")
        spans.append((width - n, width) if left else (0, n))
    return spans


def _first_positions_of_padded_rows(position_ids: torch.Tensor) -> List[int]:
    """The position of each row's first token: the smallest position of the row (padding stays at it)."""
    return [int(min(row)) for row in position_ids.tolist()]


def plan_batches(lengths: Sequence[int], max_new_tokens: int, batch_size: Optional[int], cache_tokens: int,
                 max_slots: int, block_tokens: int = 64) -> List[List[int]]:
    """Cuts request numbers 0..n-1 into batches, in order: at most ``batch_size`` (and ``max_slots``)
    requests each, and such that every request of a batch can reach its full length in a cache of
    ``cache_tokens`` tokens that are handed out in blocks of ``block_tokens``."""
    def cost(n):
        return (n + max_new_tokens + block_tokens - 1) // block_tokens * block_tokens

    limit = min(batch_size or len(lengths), max_slots)
    batches, cur, used = [], [], 0
    for i, n in enumerate(lengths):
        c = cost(n)
        if c > cache_tokens:
            raise ValueError(f"request {i}: {n} + {max_new_tokens} tokens do not fit a cache of {cache_tokens} tokens")
        if cur and (len(cur) >= limit or used + c > cache_tokens):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += c
    if cur:
        batches.append(cur)
    return batches


# The most prompt tokens of one step: the prompts of a batch run together up to this many tokens, else a few sequences
# at a time, so that the step's intermediate tensors (a few tens of KB a token at the 8B sizes) stay bounded.
PROMPT_TOKENS_PER_STEP = 65536


def prompt_groups(lengths: Sequence[int], most: int) -> List[List[int]]:
    """Consecutive sequences packed into groups of at most ``most`` tokens (a longer prompt is a group of its own)."""
    groups: List[List[int]] = []
    total = 0
    for i, n in enumerate(lengths):
        if not groups or total + n > most:
            groups.append([])
            total = 0
        groups[-1].append(i)
        total += n
    return groups


def generate_batch(engine, sampler: Sampler, prompts: Sequence[Sequence[int]], requests: Sequence[int],
                   max_new_tokens: int, stop_tokens: Sequence[int] = (),
                   post_iteration_hook: Optional[Callable] = None, times: Optional[List[float]] = None,
                   first_positions: Optional[Sequence[int]] = None) -> List[List[int]]:
    """One batch of sequences that start together: the prompts in one step (in a few, sequence by sequence, where they
    hold more than ``PROMPT_TOKENS_PER_STEP`` tokens), then one token each until
    every sequence has met a stop token or has ``max_new_tokens`` new tokens.  ``engine`` needs ``begin``,
    ``step``, ``release`` and ``device``.  ``first_positions``: the position of each prompt's first token where
    that is not 0 (the reference's ``position_ids``, fms/utils/generation.py:122-132)."""
    n = len(prompts)
    stop = set(int(t) for t in stop_tokens)
    outputs = [list(p) for p in prompts]
    slots = engine.begin(n, list(first_positions)) if first_positions is not None and any(first_positions) else engine.begin(n)
    held = set(slots)
    horizon = max(len(p) for p in prompts) + max_new_tokens
    try:
        live = list(range(n))
        req_of, req = None, None
        feed = [list(p) for p in prompts]
        for it in range(max_new_tokens):
            start = time.perf_counter()
            if it > 0 and hasattr(engine, "decode"):
                logits = engine.decode([slots[i] for i in live], [f[0] for f in feed], horizon=horizon)
            else:
                groups = prompt_groups([len(f) for f in feed], PROMPT_TOKENS_PER_STEP)
                parts = [engine.step([slots[live[i]] for i in g], [feed[i] for i in g]) for g in groups]
                logits = parts[0] if len(parts) == 1 else torch.cat(parts)
            if req_of != live:  # the request numbers of the live sequences, on the device (sampling draws by them)
                req = torch.tensor([requests[i] for i in live], dtype=torch.int32).to(engine.device)
                req_of = list(live)
            tokens = sampler(logits, req, it).tolist()  # device -> host: the loop's one synchronisation
            if times is not None:
                times.append(time.perf_counter() - start)
            if post_iteration_hook is not None:
                post_iteration_hook(it, logits, tokens, [requests[i] for i in live])
            still, feed = [], []
            for i, t in zip(live, tokens):
                outputs[i].append(int(t))
                if int(t) in stop:
                    engine.release([slots[i]])  # the slot and its blocks are free for the next batch at once
                    held.discard(slots[i])
                else:
                    still.append(i)
                    feed.append([int(t)])
            live = still
            if not live:
                break
    finally:
        if held:
            engine.release(sorted(held))
    return outputs


def _cache_tokens_that_fit(model) -> Optional[int]:
    """Tokens of cache that four fifths of the device's free memory (and of what the model's own engine holds already)
    have room for; None where that cannot be told (no CUDA device, a model without the figures)."""
    try:
        device = torch.device(model.device)
        per_token = model.cache_bytes_per_token()
        if device.type != "cuda" or per_token <= 0:
            return None
        free, _ = torch.cuda.mem_get_info(device)
        held = getattr(model, "_engine", None)
        if held is not None:
            free += held.cache.n_blocks * 64 * per_token
        return max(64, int(0.8 * free / per_token) // 64 * 64)
    except Exception:
        return None


def generate(model, input_ids: Prompts, max_seq_len: int = 4096, max_new_tokens: int = 256,
             temperature: float = 1.0, top_k: int = 10, do_sample: bool = True, num_beams: int = 1,
             use_cache: bool = True, contiguous_cache: bool = False,
             eos_token_id: Union[int, Sequence[int], None] = None, pad_token_id: Optional[int] = None,
             timing: str = "", prepare_model_inputs_hook: Optional[Callable] = None,
             post_iteration_hook: Optional[Callable] = None, extra_kwargs: Optional[dict] = None,
             seed: int = 0, batch_size: Optional[int] = None, cache_tokens: Optional[int] = None):
    """Generates ``max_new_tokens`` tokens after each prompt.

    model: what ``get_model`` returned (or an engine: anything with begin/step/release/device).
    input_ids: a 1-D tensor (one prompt), a 2-D tensor (prompts of equal length) or a list of 1-D tensors
        or lists (prompts of any lengths).
    max_seq_len: prompts longer than this are cut to their last ``max_seq_len`` tokens, as the reference
        clips its input window (fms/utils/generation.py:288).
    temperature, top_k, do_sample: as in the reference; ``do_sample=False`` is greedy.
    contiguous_cache: accepted for the reference's callers; the cache here is made of blocks and has no such mode.
    prepare_model_inputs_hook, extra_kwargs: the reference passes these into its model's forward
        (fms/utils/generation.py:246-252).  The engine builds its own inputs, so a hook is refused, and of
        ``extra_kwargs`` only what ``pad_input_ids`` returned is taken (``position_ids``, ``mask``), with a
        2-D ``input_ids``: each row then runs without its padding, from the position its ``position_ids`` start
        at (``position_ids_offset``), and comes back with its padding.
    eos_token_id: one stop token or several; a sequence ends with its stop token.
    timing: "" | "per-token" | "e2e": also return the seconds of each step, or of the whole call.
    post_iteration_hook(step, logits, tokens, requests): called after every step of a batch.
    seed: seeds the draws; batch_size: most requests per batch (default: as many as fit);
    cache_tokens: size of the cache to use when the model makes its own engine.

    Returns the prompts with their new tokens: 1-D for a 1-D input; a list of 1-D tensors for a list; a
    2-D tensor for a 2-D input (rows that stopped early are filled up with ``pad_token_id``, or with
    their stop token when that is None).
    """
    if num_beams != 1:
        raise NotImplementedError("generate() does not support beam search")
    if prepare_model_inputs_hook is not None:
        raise NotImplementedError("prepare_model_inputs_hook: the engine builds the inputs of a step itself")
    extra = {k: v for k, v in (extra_kwargs or {}).items() if v is not None}
    if set(extra) - {"position_ids", "mask"}:
        raise NotImplementedError(f"extra_kwargs {sorted(set(extra) - {'position_ids', 'mask'})}: "
                                  "the engine's step takes no further arguments")
    if not use_cache:
        raise NotImplementedError("generation always uses the cache")
    if timing not in ("", "per-token", "e2e"):
        raise ValueError('timing must be "", "per-token" or "e2e"')
    prompts, kind = _as_lists(input_ids)
    padded_rows, first_positions = None, None
    if extra:
        if kind != "2d" or "position_ids" not in extra:
            raise ValueError("extra_kwargs of pad_input_ids go with its 2-D input_ids and need position_ids")
        padded_rows = prompts
        spans = _tokens_of_padded_rows(input_ids, torch.as_tensor(extra["position_ids"]))
        first_positions = _first_positions_of_padded_rows(torch.as_tensor(extra["position_ids"]))
        prompts = [row[a:b] for row, (a, b) in zip(prompts, spans)]
    if not prompts or any(len(p) == 0 for p in prompts):
        raise ValueError("every prompt needs at least one token")
    given = [len(p) for p in prompts]
    if first_positions is not None:  # a prompt that is cut to its last max_seq_len tokens starts that much later
        first_positions = [f + max(0, len(p) - max_seq_len) for f, p in zip(first_positions, prompts)]
    prompts = [p[-max_seq_len:] for p in prompts]
    stop = [] if eos_token_id is None else ([int(eos_token_id)] if isinstance(eos_token_id, int) else list(eos_token_id))
    sampler = Sampler(do_sample, temperature, top_k, seed)

    if hasattr(model, "step") and hasattr(model, "begin"):
        engine = model
    else:
        longest = max(len(p) for p in prompts) + max_new_tokens
        want = cache_tokens or sum((len(p) + max_new_tokens + 63) // 64 * 64 for p in prompts[: batch_size or len(prompts)])
        slots = min(len(prompts), batch_size or len(prompts))
        if not cache_tokens:
            # no more than the device has room for: requests beyond it wait for the next batch
            fits = _cache_tokens_that_fit(model)
            if fits is not None and want > fits:
                slots = max(1, min(slots, int(slots * fits / want)))
                want = fits
        engine = model.engine(min_tokens=max(want, (longest + 63) // 64 * 64), min_slots=slots)
    cache = getattr(engine, "cache", None)
    capacity = cache.n_blocks * 64 if cache is not None else 1 << 60
    max_slots = cache.max_slots if cache is not None else len(prompts)
    limit = cache.max_positions if cache is not None else 1 << 60
    for i, p in enumerate(prompts):
        first = first_positions[i] if first_positions is not None else 0
        if first + len(p) + max_new_tokens > limit:
            raise ValueError(f"prompt {i}: {first + len(p)} + {max_new_tokens} tokens exceed the model's {limit} positions")

    times: List[float] = []
    start = time.perf_counter()
    results: List[Optional[List[int]]] = [None] * len(prompts)
    for batch in plan_batches([len(p) for p in prompts], max_new_tokens, batch_size, capacity, max_slots):
        outs = generate_batch(engine, sampler, [prompts[i] for i in batch], batch, max_new_tokens, stop,
                              post_iteration_hook, times if timing == "per-token" else None,
                              [first_positions[i] for i in batch] if first_positions is not None else None)
        for i, o in zip(batch, outs):
            results[i] = o
    if timing == "e2e":
        if getattr(engine, "device", None) is not None and torch.device(engine.device).type == "cuda":
            torch.cuda.synchronize()
        times = [time.perf_counter() - start]

    device = getattr(engine, "device", "cpu")
    if kind == "1d":
        out = torch.tensor(results[0], dtype=torch.long, device=device)
    elif kind == "list":
        out = [torch.tensor(r, dtype=torch.long, device=device) for r in results]
    else:
        if padded_rows is not None:  # each row as it came, padding and all, and its new tokens behind it
            results = [row + r[min(n, max_seq_len):] for row, r, n in zip(padded_rows, results, given)]
        longest = max(len(r) for r in results)
        rows = [r + [pad_token_id if pad_token_id is not None else r[-1]] * (longest - len(r)) for r in results]
        out = torch.tensor(rows, dtype=torch.long, device=device)
    return (out, times) if timing else out


def truncate_after_eos(result: torch.Tensor, eos_token_id: int) -> torch.Tensor:
    """Cuts a 1-D result after its first stop token (fms/utils/generation.py:372-387)."""
    if eos_token_id is None:
        return result
    hits = torch.where(result == eos_token_id)[0]
    return result[: int(hits[0]) + 1] if hits.numel() else result


def trim_prefix(result: torch.Tensor, pad_token_id: int = 0) -> torch.Tensor:
    """Removes leading ``pad_token_id`` tokens of a 1-D result (fms/utils/generation.py:390-413)."""
    keep = torch.where(result != pad_token_id)[0]
    return result[int(keep[0]):] if keep.numel() else result[:0]
