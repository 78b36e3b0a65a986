"""Trace replay: feeds given token ids through a model step by step and writes logits.  It samples
nothing.  It drives the same model, step function, cache and kernels as generation.

Input: one JSON object a line,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: for each request its next tokens and the places among them whose logits are wanted; a
request that is new gets a slot.  ``end``: requests that are finished after this step; their slots and
blocks are given back.  For a step that wants something, ``<out>/<step>.f32`` holds the logits at the
wanted places, in the order of the entries and of ``want``, as little-endian float32 [wanted, vocab].
After every step ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, IO

import torch


def replay(engine, lines: IO[str], out_dir: str, log: IO[str] = sys.stdout) -> None:
    os.makedirs(out_dir, exist_ok=True)
    slot_of: Dict[str, int] = {}
    for line in lines:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        entries = step.get("entries", [])
        new = [e["id"] for e in entries if e["id"] not in slot_of]
        if len(set(new)) != len(new):
            raise ValueError(f"step {step.get('step')}: a new request appears twice")
        for rid, slot in zip(new, engine.begin(len(new)) if new else []):
            slot_of[rid] = slot
        if entries:
            logits = engine.step([slot_of[e["id"]] for e in entries], [e["tokens"] for e in entries],
                                 [e.get("want", []) for e in entries])
            if logits.shape[0]:
                data = logits.to(torch.float32).cpu().contiguous().numpy().astype("<f4", copy=False)
                with open(os.path.join(out_dir, f"{step['step']}.f32"), "wb") as f:
                    f.write(data.tobytes())
        ended = step.get("end", [])
        if ended:
            engine.release([slot_of.pop(rid) for rid in ended])
        engine.check()
        print(f"done {step['step']}", file=log, flush=True)
