"""Loading a model folder's tensors by name, against what the model's parts declare.

The parts of a model declare every tensor they read (`TensorDecl`: name, shape,
whether it may be absent).  The loader compares that list with the folder and
raises ONE error that lists everything wrong: tensors missing, tensors nobody
asked for, and shapes that differ.  The reference reports the first problem
only (`missing tensor {name}`, `shape ... has n elems, expected ...`,
crates/mach-model/src/loader.rs:1016-1021, :706-712 of gqf2008/machserve).

Storage: floating tensors stored in 16 bits come back as bfloat16 (float16 is
rounded to it), tensors stored in 32 bits stay float32, integer tables come back
as int32.  With `dtype=torch.float32` every floating tensor is widened to
float32 instead.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass
from typing import Dict, Iterable, Optional, Tuple

import torch

from .safetensors_io import SafetensorsError, open_model_files


@dataclass(frozen=True)
class TensorDecl:
    """A tensor that a part reads.

    `init` tells the random-weights mode how to fill it: "matrix" (normal, std
    `weight_std`), "bias" (normal, std `bias_std`), "scale" (1 + normal, std
    `norm_std`), "zeros", or "table" (an integer table; zeros).  `random=False` keeps an
    optional tensor out of a random model (a tied head has no tensor of its own).
    """

    name: str
    shape: Tuple[int, ...]
    required: bool = True
    init: str = "matrix"
    random: bool = True


class WeightsError(ValueError):
    """The folder's tensors do not match what the model declares."""

    def __init__(self, where, missing, unexpected, wrong_shape, wrong_kind=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_kind = list(wrong_kind)
        lines = [f"{where}: the tensors do not match the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, want, found in self.wrong_shape:
            lines.append(f"  wrong shape: {name} is {list(found)}, the model needs {list(want)}")
        for name, msg in self.wrong_kind:
            lines.append(f"  wrong dtype: {name} {msg}")
        super().__init__("\n".join(lines))


_FLOATS = (torch.float16, torch.bfloat16, torch.float32, torch.float64)


def _stored_to_kept(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    if t.dtype in _FLOATS:
        if dtype == torch.float32:
            return t.to(torch.float32)
        if t.dtype in (torch.float32, torch.float64):
            return t.to(torch.float32)
        return t.to(torch.bfloat16)
    if t.dtype == torch.bool:
        return t
    return t.to(torch.int32)


def load_weights(
    model_dir, declared: Iterable[TensorDecl], dtype: torch.dtype = torch.bfloat16, device="cpu"
) -> Dict[str, torch.Tensor]:
    """Reads every declared tensor that the folder holds; raises `WeightsError` if the two lists differ."""
    decls = {}
    for d in declared:
        if d.name in decls and decls[d.name].shape != tuple(d.shape):
            raise ValueError(f"tensor '{d.name}' is declared twice with different shapes")
        # a tensor that two parts share is required if either needs it
        if d.name in decls and decls[d.name].required:
            continue
        decls[d.name] = d
    try:
        entries, files = open_model_files(model_dir)
    except SafetensorsError as e:
        raise SafetensorsError(str(e)) from None
    try:
        missing = [n for n, d in decls.items() if n not in entries and d.required]
        unexpected = sorted(n for n in entries if n not in decls)
        wrong_shape = [
            (n, tuple(d.shape), entries[n].shape)
            for n, d in decls.items()
            if n in entries and tuple(entries[n].shape) != tuple(d.shape)
        ]
        wrong_kind = []
        for n, d in decls.items():
            if n in entries:
                is_float = entries[n].dtype in ("F16", "BF16", "F32", "F64")
                if (d.init == "table") == is_float:
                    wrong_kind.append((n, f"is stored as {entries[n].dtype}, the model needs "
                                       + ("integers" if d.init == "table" else "floating point")))
        if missing or unexpected or wrong_shape or wrong_kind:
            raise WeightsError(str(model_dir), missing, unexpected, wrong_shape, wrong_kind)
        out = {}
        for n in decls:
            if n in entries:
                out[n] = _stored_to_kept(entries[n].file.tensor(n), dtype).to(device)
        halves = [n for n in out if entries[n].dtype == "F16"]
        if halves and dtype != torch.float32:
            # float16 has three more bits of mantissa than bfloat16 and a narrower range: said once, not silently
            warnings.warn(f"{model_dir}: {len(halves)} tensors are stored as float16 and are rounded to bfloat16 "
                          f"(first: {halves[0]}); load with dtype float32 to keep every bit", stacklevel=2)
        return out
    finally:
        for f in files:
            f.close()
