"""Weights from safetensors files, by tensor name.

Reference (utils/loader.py:8-38): every ``*.safetensors`` file of the folder, sorted; disk
names mapped to packed parameters (q/k/v -> qkv_proj rows, gate/up -> gate_up_proj rows);
``lm_head.weight`` skipped when the head is tied; a parameter that was never filled is an
error.  Here the model's parts declare which disk tensors fill which rows, the files are
checked against that list before anything is copied, and ONE error lists every missing
tensor, every unexpected tensor and every wrong shape.

Precision: matrices are kept in bfloat16 in the bfloat16 engine and widened (exactly) to
float32 in the float32 engine; a matrix that is stored in 32-bit stays 32-bit in both;
vectors (norm weights) are always held in float32, which is exact for bfloat16 files;
integer tensors become int32.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from glob import glob
from typing import Iterator

import torch
from safetensors import safe_open

from ..parts.base import ParamDecl, Part

_ST_DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
              "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8}
_WIDE = (torch.float32, torch.float64)
_INTS = (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)


class WeightsError(RuntimeError):
    """The files of a model folder do not fit the model; lists every fault found."""

    def __init__(self, folder, missing, unexpected, wrong_shape):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.wrong_shape = sorted(wrong_shape)
        lines = [f"weights in {folder!r} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: file has {list(got)}, model wants {list(want)}" for n, got, want in self.wrong_shape))
        super().__init__("\n".join(lines))


@dataclass
class _Expected:
    param: str            # full parameter name
    row_start: int
    shape: tuple[int, ...]


def iter_param_decls(model: Part) -> Iterator[tuple[str, Part, ParamDecl]]:
    """(prefix, owning part, declaration) of every parameter of the model, in a fixed order."""
    for prefix, part in model.walk():
        for decl in part.param_decls():
            yield prefix, part, decl


def expected_disk_tensors(model: Part) -> dict[str, _Expected]:
    exp: dict[str, _Expected] = {}
    for prefix, _, decl in iter_param_decls(model):
        if decl.tied_to is not None:
            continue
        full = prefix + decl.name
        if decl.sources:
            for src in decl.sources:
                exp[prefix + src.disk_name] = _Expected(full, src.row_start, (src.rows, *decl.shape[1:]))
        else:
            exp[full] = _Expected(full, 0, tuple(decl.shape))
    return exp


def load_weights(model: Part, folder: str, dtype: torch.dtype, device) -> dict[str, torch.Tensor]:
    """Fill every part's ``params`` from the folder; returns {full parameter name: tensor}."""
    folder = os.path.expanduser(folder)
    files = sorted(glob(os.path.join(folder, "*.safetensors")))
    if not files:
        raise WeightsError(folder, ["(no .safetensors file in the folder)"], [], [])
    expected = expected_disk_tensors(model)
    tied_names = {prefix + d.name for prefix, _, d in iter_param_decls(model) if d.tied_to is not None}

    found: dict[str, tuple[str, tuple[int, ...], torch.dtype]] = {}
    for path in files:
        with safe_open(path, "pt", device="cpu") as f:
            for name in f.keys():
                sl = f.get_slice(name)
                found[name] = (path, tuple(sl.get_shape()), _ST_DTYPES.get(sl.get_dtype(), torch.float32))

    missing = [n for n in expected if n not in found]
    # A tied head's own tensor may be present on disk; it is skipped (utils/loader.py:23-24).
    unexpected = [n for n in found if n not in expected and n not in tied_names]
    wrong = [(n, found[n][1], e.shape) for n, e in expected.items() if n in found and found[n][1] != e.shape]
    if missing or unexpected or wrong:
        raise WeightsError(folder, missing, unexpected, wrong)

    # Decide each parameter's dtype from how its pieces are stored, then allocate.
    params: dict[str, torch.Tensor] = {}
    decl_of: dict[str, tuple[Part, ParamDecl]] = {}
    stored: dict[str, list[torch.dtype]] = {}
    for name, e in expected.items():
        stored.setdefault(e.param, []).append(found[name][2])
    for prefix, part, decl in iter_param_decls(model):
        full = prefix + decl.name
        decl_of[full] = (part, decl)
        if decl.tied_to is not None:
            continue
        kinds = stored[full]
        if all(k in _INTS for k in kinds):
            pdtype = torch.int32
        elif decl.role == "vector" or dtype == torch.float32 or any(k in _WIDE for k in kinds):
            pdtype = torch.float32
        else:
            pdtype = torch.bfloat16
        params[full] = torch.empty(decl.shape, dtype=pdtype, device=device)

    by_file: dict[str, list[str]] = {}
    for name in expected:
        by_file.setdefault(found[name][0], []).append(name)
    for path, names in by_file.items():
        with safe_open(path, "pt", device="cpu") as f:
            for name in names:
                e = expected[name]
                dest = params[e.param]
                piece = f.get_tensor(name)
                dest.narrow(0, e.row_start, e.shape[0]).copy_(piece.to(dest.dtype)) if dest.dim() else dest.copy_(piece)

    for full, (part, decl) in decl_of.items():
        if decl.tied_to is not None:
            if decl.tied_to not in params:
                raise WeightsError(folder, [f"{full} is tied to {decl.tied_to}, which the model lacks"], [], [])
            params[full] = params[decl.tied_to]
        part.params[decl.name] = params[full]
    return params
