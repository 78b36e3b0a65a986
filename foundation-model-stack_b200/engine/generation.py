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


def generate_batch(engine, sampler: Sampler, prompts: Sequence[Sequence[int]], requests: Sequence[int],
                   max_new_tokens: int, stop_tokens: Sequence[int] = (),
                   post_iteration_hook: Optional[Callable] = None, times: Optional[List[float]] = None
                   ) -> List[List[int]]:
    """One batch of sequences that start together: the prompts in one step, then one token each until
    every sequence has met a stop token or has ``max_new_tokens`` new tokens.  ``engine`` needs ``begin``,
    ``step``, ``release`` and ``device``."""
    n = len(prompts)
    stop = set(int(t) for t in stop_tokens)
    outputs = [list(p) for p in prompts]
    slots = engine.begin(n)
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
                logits = engine.step([slots[i] for i in live], feed)
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
    prepare_model_inputs_hook, extra_kwargs: the reference passes these into its model's forward; the engine
        builds its own inputs, so anything but None (or an empty mapping) is refused.
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
        raise NotImplementedError("generate() does yet not support beam search")
    if prepare_model_inputs_hook is not None:
        raise NotImplementedError("prepare_model_inputs_hook: the engine builds the inputs of a step itself")
    if extra_kwargs:
        raise NotImplementedError(f"extra_kwargs {sorted(extra_kwargs)}: the engine's step takes no further arguments")
    if not use_cache:
        raise NotImplementedError("generation always uses the cache")
    if timing not in ("", "per-token", "e2e"):
        raise ValueError('timing must be "", "per-token" or "e2e"')
    prompts, kind = _as_lists(input_ids)
    if not prompts or any(len(p) == 0 for p in prompts):
        raise ValueError("every prompt needs at least one token")
    prompts = [p[-max_seq_len:] for p in prompts]
    stop = [] if eos_token_id is None else ([int(eos_token_id)] if isinstance(eos_token_id, int) else list(eos_token_id))
    sampler = Sampler(do_sample, temperature, top_k, seed)

    if hasattr(model, "step") and hasattr(model, "begin"):
        engine = model
    else:
        longest = max(len(p) for p in prompts) + max_new_tokens
        want = cache_tokens or sum((len(p) + max_new_tokens + 63) // 64 * 64 for p in prompts[: batch_size or len(prompts)])
        engine = model.engine(min_tokens=max(want, (longest + 63) // 64 * 64), min_slots=min(len(prompts), batch_size or len(prompts)))
    cache = getattr(engine, "cache", None)
    capacity = cache.n_blocks * 64 if cache is not None else 1 << 60
    max_slots = cache.max_slots if cache is not None else len(prompts)
    limit = cache.max_positions if cache is not None else 1 << 60
    for i, p in enumerate(prompts):
        if len(p) + max_new_tokens > limit:
            raise ValueError(f"prompt {i}: {len(p)} + {max_new_tokens} tokens exceed the model's {limit} positions")

    times: List[float] = []
    start = time.perf_counter()
    results: List[Optional[List[int]]] = [None] * len(prompts)
    for batch in plan_batches([len(p) for p in prompts], max_new_tokens, batch_size, capacity, max_slots):
        outs = generate_batch(engine, sampler, [prompts[i] for i in batch], batch, max_new_tokens, stop,
                              post_iteration_hook, times if timing == "per-token" else None)
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
