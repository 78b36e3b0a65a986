"""What every part of a layer is: a holder of named tensors and of child parts.

A part declares the tensors it needs (name, shape, role); the weight loader fills them in.  A part
never allocates its own weights and never reads a checkpoint.  Roles decide the dtype a tensor is kept
in (``fms_b200.weights.loader.kept_dtype``): ``matrix`` and ``vector`` are floating point, ``table`` is an
integer table.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Iterator, List, Optional, Tuple

import torch


@dataclasses.dataclass
class TensorDecl:
    shape: Tuple[int, ...]
    role: str = "matrix"  # "matrix" | "vector" | "table"
    optional: bool = False


class Part:
    """Base of norms, position encodings, mixers, feed-forwards, blocks and the decoder itself."""

    def __init__(self) -> None:
        self._decls: Dict[str, TensorDecl] = {}
        self._tensors: Dict[str, torch.Tensor] = {}
        self._children: Dict[str, "Part"] = {}

    # ---- declaration -------------------------------------------------------------------------
    def declare(self, name: str, shape, role: str = "matrix", optional: bool = False) -> None:
        self._decls[name] = TensorDecl(tuple(int(s) for s in shape), role, optional)

    def add(self, name: str, part: "Part") -> "Part":
        self._children[name] = part
        return part

    # ---- access ------------------------------------------------------------------------------
    def tensor(self, name: str) -> Optional[torch.Tensor]:
        return self._tensors.get(name)

    def set_tensor(self, name: str, value: torch.Tensor) -> None:
        decl = self._decls[name]
        if tuple(value.shape) != decl.shape:
            raise ValueError(f"tensor {name}: shape {tuple(value.shape)} given, {decl.shape} declared")
        self._tensors[name] = value

    def child(self, name: str) -> "Part":
        return self._children[name]

    def children(self) -> Iterator[Tuple[str, "Part"]]:
        return iter(self._children.items())

    def named_decls(self, prefix: str = "") -> Iterator[Tuple[str, "Part", str, TensorDecl]]:
        """(qualified name, owner, local name, declaration) of every tensor below this part.  A part that
        was added under two names (a tied head) is listed once, under the first."""
        seen = set()

        def walk(part: "Part", pre: str):
            if id(part) in seen:
                return
            seen.add(id(part))
            for n, d in part._decls.items():
                yield pre + n, part, n, d
            for cn, c in part._children.items():
                yield from walk(c, pre + cn + ".")

        yield from walk(self, prefix)

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return {q: owner._tensors[n] for q, owner, n, _ in self.named_decls() if n in owner._tensors}

    def finalize(self, device: torch.device, dtype: torch.dtype) -> None:
        """Called once after all tensors are set: build derived tables on the device."""
        for _, c in self._children.items():
            c.finalize(device, dtype)

    def kernel_libraries(self, dtype: torch.dtype) -> List[str]:
        """Names of the kernel libraries (``fms_b200.kernels.build``) that this part and the parts below it call
        when the model computes in ``dtype``; the engine compiles them before the first step.  A part that calls
        kernels of its own adds their libraries' names to what this returns."""
        out: List[str] = []
        for _, c in self._children.items():
            out += c.kernel_libraries(dtype)
        return out
