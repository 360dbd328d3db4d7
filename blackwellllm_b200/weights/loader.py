"""Binds the tensors of a model folder to the names a model asks for.

All names are checked before anything is copied: one :class:`WeightError` lists
every missing tensor, every unexpected one and every wrong shape.  Derived buffers
that some exporters store (``rotary_emb.inv_freq``) are passed over with a note, and
with ``ignore_unexpected`` so is every other tensor the model does not ask for.  (The reference
finds a missing tensor only at its first use: src/core/memory_pool.cpp:466-475.)

Kept types: matrix operands and embedding tables are held in the compute dtype
(bfloat16, or float32 on the 32-bit path); vectors (norm gains, biases) stored
in 32-bit stay 32-bit, stored in 16-bit they are bfloat16 (float32 on the 32-bit
path); integer tables become int32.
"""
from __future__ import annotations

from typing import Dict, Mapping

import torch

from ..parts.base import ParamSpec
from .safetensors_io import TensorFiles, index_folder


class WeightError(ValueError):
    def __init__(self, where: str, missing, unexpected, wrong_shape, wrong_type=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_type = list(wrong_type)
        lines = [f"weights in {where!r} do not match the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_type:
            lines.append(f"  wrong type ({len(self.wrong_type)}): " + ", ".join(
                f"{n} is {dt}" for n, dt in self.wrong_type))
        super().__init__("\n".join(lines))


_FLOATS = (torch.float64, torch.float32, torch.float16, torch.bfloat16)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


def kept_dtype(spec: ParamSpec, stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if spec.role == "int_table":
        return torch.int32
    if compute == torch.float32 or spec.role == "matrix":
        return compute
    return torch.float32 if stored in (torch.float32, torch.float64) else torch.bfloat16


# Tensors some exporters store although they are no weights (derived tables): never an error.
DERIVED_BUFFERS = (".rotary_emb.inv_freq",)


def check_names(where: str, expected: Mapping[str, ParamSpec], found: Mapping[str, object],
                ignore_unexpected: bool = False) -> list:
    """``found`` maps name -> object with .shape and .dtype.  Returns the names that were found,
    not asked for and passed over: derived buffers always (``DERIVED_BUFFERS``), any other
    unexpected tensor only with ``ignore_unexpected`` (else it is part of the error)."""
    missing = [n for n, s in expected.items() if n not in found and not s.optional]
    extra = [n for n in found if n not in expected]
    passed_over = [n for n in extra if ignore_unexpected or n.endswith(DERIVED_BUFFERS)]
    unexpected = [n for n in extra if n not in passed_over]
    wrong_shape, wrong_type = [], []
    for n, s in expected.items():
        if n in found:
            if tuple(found[n].shape) != tuple(s.shape):
                wrong_shape.append((n, tuple(found[n].shape), tuple(s.shape)))
            dt = found[n].dtype
            if (s.role == "int_table" and dt not in _INTS) or (s.role != "int_table" and dt not in _FLOATS):
                wrong_type.append((n, dt))
    if missing or unexpected or wrong_shape or wrong_type:
        raise WeightError(where, sorted(missing), sorted(unexpected), sorted(wrong_shape), sorted(wrong_type))
    if passed_over:
        import sys
        shown = ", ".join(sorted(passed_over)[:4]) + (" ..." if len(passed_over) > 4 else "")
        print(f"[blackwellllm_b200] {where}: {len(passed_over)} tensor(s) the model does not use were "
              f"passed over: {shown}", file=sys.stderr)
    return sorted(passed_over)


def load_weights(model_dir: str, expected: Mapping[str, ParamSpec], compute: torch.dtype,
                 device: torch.device, ignore_unexpected: bool = False) -> Dict[str, torch.Tensor]:
    entries = index_folder(model_dir)
    check_names(model_dir, expected, entries, ignore_unexpected)
    out: Dict[str, torch.Tensor] = {}
    with TensorFiles() as files:
        for name, spec in expected.items():
            if name not in entries:
                continue
            t = files.read(entries[name])
            out[name] = t.to(kept_dtype(spec, t.dtype, compute)).to(device)
    return out


def bind_tensors(tensors: Mapping[str, torch.Tensor], expected: Mapping[str, ParamSpec],
                 compute: torch.dtype, device: torch.device, where: str = "<tensors>",
                 ignore_unexpected: bool = False) -> Dict[str, torch.Tensor]:
    """The same binding for tensors already in memory (used by tests and by
    ``Engine.from_tensors``)."""
    check_names(where, expected, tensors, ignore_unexpected)
    return {n: tensors[n].to(kept_dtype(s, tensors[n].dtype, compute)).to(device)
            for n, s in expected.items() if n in tensors}
