"""Weights by tensor name, checked against what the model declares.

The reference fetches tensors by their Hugging Face names (src/model.cpp:136-171) and
reports ``missing tensor <name>`` / ``truncated tensor <name>`` one at a time, with no
shape check and silence about extra tensors (src/model.cpp:123-128).  Here a model
declares every parameter it needs (:class:`ParamSpec`), and one pass over the files
produces ONE error that lists all missing names, all unexpected names and all wrong
shapes together.

Storage rule: a matrix is held in the dtype the run computes in (bfloat16 for the
serving path, float32 for the 32-bit path; widening bfloat16 to float32 is exact,
narrowing is round-to-nearest-even like src/model.cpp:69-74); a vector that a kernel
reads in 32-bit (norm weights) is held in float32; integer tables become int32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

from .safetensors_io import SafetensorsError, open_model_shards

MATRIX = "matrix"    # cast to the run's matrix dtype
KEEP32 = "keep32"    # always float32 on the device
INT_TABLE = "int32"  # integer table -> int32


@dataclass(frozen=True)
class ParamSpec:
    name: str
    shape: Tuple[int, ...]
    kind: str = MATRIX
    optional: bool = False
    init: str = "normal"  # how the random-weights mode fills it: "normal" or "ones"


class WeightError(ValueError):
    """All problems of a checkpoint against a model's declaration, in one message."""

    def __init__(self, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, tuple, tuple]], source: str = ""):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"checkpoint {source} does not match the model:".replace("  ", " ")]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: file {list(got)} != model {list(want)}" for n, got, want in self.wrong_shape))
        super().__init__("\n".join(lines))


def _ignorable(ignorable) -> "callable":
    """``ignorable`` as a predicate: a callable stays, names become a membership test."""
    if callable(ignorable):
        return ignorable
    names = set(ignorable)
    return lambda n: n in names


def check_against_specs(available: Mapping[str, tuple], specs: Iterable[ParamSpec],
                        ignorable=(), source: str = "") -> None:
    """Raise :class:`WeightError` unless ``available`` (name -> shape) fits ``specs``.
    ``ignorable``: names, or a predicate on names, of stored tensors the model has no use for."""
    specs = list(specs)
    by_name = {s.name: s for s in specs}
    missing = [s.name for s in specs if s.name not in available and not s.optional]
    skip = _ignorable(ignorable)
    unexpected = [n for n in available if n not in by_name and not skip(n)]
    wrong = [(n, tuple(available[n]), by_name[n].shape) for n in available
             if n in by_name and tuple(available[n]) != tuple(by_name[n].shape)]
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong, source)


def _convert(t: torch.Tensor, spec: ParamSpec, matrix_dtype: torch.dtype, device) -> torch.Tensor:
    if spec.kind == INT_TABLE:
        want = torch.int32
    elif spec.kind == KEEP32:
        want = torch.float32
    else:
        want = matrix_dtype
    if t.dtype.is_floating_point != want.is_floating_point:
        raise SafetensorsError(f"tensor {spec.name}: stored as {t.dtype}, the model needs {want}")
    # torch's float32 -> bfloat16 conversion rounds to nearest even
    return t.to(device=device, dtype=want, copy=True).contiguous()


def load_state(folder: str, specs: Iterable[ParamSpec], matrix_dtype: torch.dtype, device,
               ignorable=(), aliases: Mapping[str, str] = {}) -> Dict[str, torch.Tensor]:
    """Read every declared tensor of ``folder`` onto ``device``.  ``aliases`` maps the name of
    a stored tensor that the model does not declare to the declared tensor it must repeat bit
    for bit (a tied head that an exporter stored a second time): equal copies are passed over,
    a copy that differs is an error."""
    specs = list(specs)
    shards = open_model_shards(folder)
    where: Dict[str, object] = {}
    duplicates = []
    for sh in shards:
        for n in sh.names():
            if n in where:
                duplicates.append(n)
            where[n] = sh
    if duplicates:
        raise SafetensorsError("tensors stored more than once in " + folder + ": " + ", ".join(duplicates))
    skip = _ignorable(ignorable)
    declared = {s.name for s in specs}
    copies = {a: t for a, t in aliases.items() if a in where and a not in declared and t in where}
    check_against_specs({n: sh.entries[n].shape for n, sh in where.items()}, specs,
                        lambda n: n in copies or skip(n), folder)
    for alias, target in copies.items():
        a, b = where[alias].tensor(alias), where[target].tensor(target)
        if a.shape != b.shape or a.dtype != b.dtype or not torch.equal(a, b):
            raise SafetensorsError(f"{folder}: {alias} is stored although the model ties it to {target}, "
                                   f"and the two differ")
    out = {}
    for s in specs:
        if s.name in where:
            out[s.name] = _convert(where[s.name].tensor(s.name), s, matrix_dtype, device)
    for sh in shards:
        sh.close()
    return out


def state_from_tensors(tensors: Mapping[str, torch.Tensor], specs: Iterable[ParamSpec],
                       matrix_dtype: torch.dtype, device, ignorable=(),
                       source: str = "(in memory)") -> Dict[str, torch.Tensor]:
    """The same check and conversion for tensors that are already in memory."""
    specs = list(specs)
    check_against_specs({n: tuple(t.shape) for n, t in tensors.items()}, specs, ignorable, source)
    return {s.name: _convert(tensors[s.name], s, matrix_dtype, device) for s in specs if s.name in tensors}
