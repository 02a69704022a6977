"""Weights by tensor name: loading a model folder, and a seeded random-weights mode.

A model states the tensors it needs as `WeightSpec`s keyed by checkpoint name; the
loader reads exactly those, keeps each in the dtype it is stored in (bfloat16 stays
bfloat16, a tensor stored in 32-bit stays 32-bit, integer tables are int32) and
raises ONE `WeightError` that lists every missing tensor, every unexpected tensor
and every wrong shape.

Parity with the reference (RicardoMin/Qwen3-Runtime-ByYourself):
  names, count 2 + 11 L (+1 untied)   src/model/weights.cpp:83-118
  tied output weight, lm_head unread  src/model/weights.cpp:116-118,198-204
  no renaming, [out, in] row-major    src/model/weights.cpp:129-164
The reference checks the element count only (:39-42) and ignores extra tensors;
here full shapes are checked and extras are reported, except names a model lists as
ignorable (`lm_head.weight` of a tied checkpoint).  Random weights are an addition:
matrices and tables N(0, 0.02), norm weights 1 + N(0, 0.1), each tensor from its
own stream derived from (seed, name), so the values do not depend on the order.
"""
from __future__ import annotations

import json
import os
import zlib
from dataclasses import dataclass
from typing import Dict, Iterable, Optional, Tuple

import torch

from .safetensors import Checkpoint, SINGLE_FILE, save_file

MATRIX_STD = 0.02
NORM_STD = 0.1


@dataclass(frozen=True)
class WeightSpec:
    """Shape and role of one checkpoint tensor.  Roles: 'matrix' (a projection or
    an embedding table), 'norm' (a scale vector around 1), 'int_table' (int32)."""
    shape: Tuple[int, ...]
    role: str = "matrix"


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every difference."""

    def __init__(self, folder, missing, unexpected, wrong_shape, wrong_dtype=()):
        self.missing, self.unexpected = sorted(missing), sorted(unexpected)
        self.wrong_shape, self.wrong_dtype = sorted(wrong_shape), sorted(wrong_dtype)
        lines = [f"checkpoint {folder} does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: file {list(got)} != model {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong dtypes ({len(self.wrong_dtype)}): " + "; ".join(
                f"{n}: {got} stored for a {role}" for n, got, role in self.wrong_dtype))
        super().__init__("\n".join(lines))


def check_checkpoint(ckpt: Checkpoint, folder: str, specs: Dict[str, WeightSpec], ignorable: Iterable[str] = ()) -> None:
    """Raise the one `WeightError` that lists everything in which the checkpoint and the model's own list of
    tensors differ; nothing is read beyond the headers."""
    have = set(ckpt.names())
    missing = [n for n in specs if n not in have]
    unexpected = [n for n in have if n not in specs and n not in set(ignorable)]
    wrong_shape, wrong_dtype = [], []
    for name, spec in specs.items():
        info = ckpt.tensors.get(name)
        if info is None:
            continue
        if tuple(info.shape) != tuple(spec.shape):
            wrong_shape.append((name, tuple(info.shape), tuple(spec.shape)))
        is_int = info.dtype == torch.int32
        if is_int != (spec.role == "int_table"):
            wrong_dtype.append((name, str(info.dtype), spec.role))
    if missing or unexpected or wrong_shape or wrong_dtype:
        raise WeightError(folder, missing, unexpected, wrong_shape, wrong_dtype)


def load_weights(folder: str, specs: Dict[str, WeightSpec], ignorable: Iterable[str] = (),
                 device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Read the tensors named by `specs` from `folder`, in their stored dtypes, onto `device` (each as a tensor
    of its own; a model that is bound for a device goes through `open_upload` instead)."""
    ckpt = Checkpoint(folder)
    check_checkpoint(ckpt, folder, specs, ignorable)
    out = {}
    for name in specs:
        t = ckpt.tensor(name)
        out[name] = t.to(device, non_blocking=False) if device != "cpu" else t.clone()
    return out


def open_upload(folder: str, specs: Dict[str, WeightSpec], ignorable: Iterable[str], dtype: torch.dtype, device, warn=None):
    """The checkpoint of `folder`, checked against `specs`, as a source that a model binds from: every tensor goes
    from the mapped file to its final place on the device in one pass (weights/upload.py)."""
    from .upload import CheckpointUpload
    ckpt = Checkpoint(folder)
    check_checkpoint(ckpt, folder, specs, ignorable)
    return CheckpointUpload(ckpt, specs, dtype, device, warn)


def _stream_seed(seed: int, name: str) -> int:
    return (int(seed) * 0x9E3779B1 + zlib.crc32(name.encode("utf-8"))) & 0x7FFFFFFFFFFFFFFF


def random_weights(specs: Dict[str, WeightSpec], seed: int, dtype: torch.dtype = torch.bfloat16,
                   device: str = "cpu") -> Dict[str, torch.Tensor]:
    """Seeded weights for `specs`: drawn in float32 on `device`, stored as `dtype`."""
    out = {}
    for name, spec in specs.items():
        gen = torch.Generator(device=device)
        gen.manual_seed(_stream_seed(seed, name))
        if spec.role == "int_table":
            out[name] = torch.zeros(spec.shape, dtype=torch.int32, device=device)
            continue
        t = torch.empty(spec.shape, dtype=dtype, device=device)
        flat = t.view(-1)
        chunk = 1 << 26  # draw large tensors piecewise: the float32 draw of a big table is transient
        for lo in range(0, flat.numel(), chunk):
            n = min(chunk, flat.numel() - lo)
            draw = torch.randn(n, generator=gen, dtype=torch.float32, device=device)
            if spec.role == "norm":
                draw.mul_(NORM_STD).add_(1.0)
            else:
                draw.mul_(MATRIX_STD)
            flat[lo:lo + n] = draw.to(dtype)
        out[name] = t
    return out


def write_model_folder(folder: str, config, tensors: Dict[str, torch.Tensor]) -> None:
    """Write `config.json` and `model.safetensors` so that the folder loads like any checkpoint."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_dict(), f, indent=2)
    save_file(tensors, os.path.join(folder, SINGLE_FILE), metadata={"format": "pt"})


def write_random_model(folder: str, config, seed: int, specs: Optional[Dict[str, WeightSpec]] = None,
                       dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
    """The random-weights mode: a model folder from a configuration and a seed."""
    if specs is None:
        from ..parts.model import build_model  # the model states its own tensors
        specs = build_model(config.plan()).weight_specs()
    if dtype is None:
        dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[getattr(config, "torch_dtype", "bfloat16")]
    tensors = random_weights(specs, seed, dtype=dtype)
    write_model_folder(folder, config, tensors)
    return tensors
