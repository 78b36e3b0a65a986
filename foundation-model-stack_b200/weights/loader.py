"""Filling a model's declared tensors from a source of checkpoint tensors.

Two passes.  The first runs the architecture's adapter on shapes only (``meta`` tensors) and compares the
result with what the model declares; anything wrong ends in ONE error that lists missing tensors,
unexpected tensors and wrong shapes.  The second reads the data one layer at a time (names that share
the prefix up to their first numeric field, as fms/utils/serialization.py:467-492 groups them), adapts
it and copies it to the device, so the host never holds more than one layer.

Dtypes.  The compute dtype is what the caller names, else the checkpoint's own (``checkpoint_dtype``: the dtype its
matrices are stored in, as the reference's parameters take the checkpoint's dtype when none is given,
fms/utils/serialization.py:679-687; this library computes in bfloat16 and float32 only, so a checkpoint stored in
anything else needs the caller's word).  ``kept_dtype``: with compute dtype bfloat16, floating tensors are kept in
bfloat16 (float16 and the like are cast), except that a tensor stored in 32-bit stays float32; with compute dtype
float32 everything floating is float32.  Integer tables become int32.  A matrix that stays float32 inside a
bfloat16 model is multiplied by the float32 kernel (its input rows are widened, its output rounded back), which is
exact but slow: the loader says so once.
"""
from __future__ import annotations

import logging
import re
from typing import Dict, List, Tuple

import torch

from .adapters import get_adapted

logger = logging.getLogger(__name__)


class WeightError(ValueError):
    """The checkpoint does not fit the model."""

    def __init__(self, missing, unexpected, wrong_shapes) -> None:
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shapes = list(wrong_shapes)
        lines = ["the checkpoint does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shapes:
            lines.append(f"  wrong shapes ({len(self.wrong_shapes)}): " + "; ".join(
                f"{n}: checkpoint {tuple(got)}, model {tuple(want)}" for n, got, want in self.wrong_shapes))
        super().__init__("\n".join(lines))


def kept_dtype(role: str, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if role == "table" or not stored.is_floating_point:
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def checkpoint_dtype(source) -> torch.dtype:
    """The compute dtype that a checkpoint asks for by itself: the dtype in which its matrices (tensors of two
    dimensions) are stored, if that is bfloat16 or float32 for all of them.  Vectors (norm gains, biases) do not
    count: they are often stored wider than the matrices."""
    stored = {source.spec(k)[0] for k in source.keys() if len(source.spec(k)[1]) == 2 and source.spec(k)[0].is_floating_point}
    if stored == {torch.bfloat16}:
        return torch.bfloat16
    if stored == {torch.float32}:
        return torch.float32
    names = ", ".join(sorted(str(d).replace("torch.", "") for d in stored)) or "no floating-point matrices"
    raise ValueError(f"the checkpoint stores its matrices as {names}; this library computes in bfloat16 or float32 and "
                     'does not choose between them for such a checkpoint: pass data_type="bf16" or "fp32"')


_FIRST_NUMBER = re.compile(r"^(.*?\.)(\d+)\.")


def _group_key(name: str) -> str:
    m = _FIRST_NUMBER.match(name)
    return m.group(1) + m.group(2) + "." if m else ""


def load_weights(model, source, architecture: str, adapter_source: str, device, compute_dtype: torch.dtype,
                 **adapter_kwargs) -> None:
    declared = {q: (owner, local, decl) for q, owner, local, decl in model.named_decls()}

    # pass 1: shapes only
    meta = {k: torch.empty(source.spec(k)[1], dtype=source.spec(k)[0], device="meta") for k in source.keys()}
    adapted = get_adapted(architecture, adapter_source, meta, **adapter_kwargs)
    missing = [n for n, (_, _, d) in declared.items() if n not in adapted and not d.optional]
    unexpected = [n for n in adapted if n not in declared]
    wrong = [(n, t.shape, declared[n][2].shape) for n, t in adapted.items()
             if n in declared and tuple(t.shape) != declared[n][2].shape]
    if missing or unexpected or wrong:
        raise WeightError(sorted(missing), sorted(unexpected), sorted(wrong))

    # pass 2: data, one group of names at a time
    groups: Dict[str, List[str]] = {}
    for k in source.keys():
        groups.setdefault(_group_key(k), []).append(k)
    wide = []
    for key in sorted(groups, key=lambda g: (g != "", g)):
        part = {k: source.get(k) for k in groups[key]}
        for name, t in get_adapted(architecture, adapter_source, part, **adapter_kwargs).items():
            owner, local, decl = declared[name]
            dtype = kept_dtype(decl.role, t.dtype, compute_dtype)
            if decl.role == "matrix" and dtype == torch.float32 and compute_dtype != torch.float32:
                wide.append(name)
            owner.set_tensor(local, t.to(device=device, dtype=dtype).contiguous())
        del part
    if wide:
        logger.warning("%d matrices are stored in 32-bit and stay float32 in this bfloat16 model (%s, ...): they take "
                       "the float32 product, which is exact but slow; a checkpoint converted to bfloat16 avoids it",
                       len(wide), wide[0])
    model.finalize(device)
