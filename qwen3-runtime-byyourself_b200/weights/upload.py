"""Where a model's parts take their tensors from when they bind: a dict of tensors in memory, or
a checkpoint on disk that is streamed to the device in one pass.

Parts ask by checkpoint name (`weights[name]`, `weights.pop(name)`) and, for matrices that
they use as one, through `fuse_rows(weights, names)` (the rows of several tensors one after the
other: q, k and v) and `fuse_interleaved(weights, first, second, block)` (blocks of `block` rows of
the one followed by the same rows of the other: gate and up).  Both sources answer in the compute
type for matrices, in float32 for scale vectors and in int32 for integer tables.

`CheckpointUpload` is the counterpart of the reference's loader (src/io/safetensors_loader.cpp:
141-248: every destination allocated first, then mmap -> two pinned staging buffers of 32 MiB ->
cudaMemcpyAsync on a stream of its own, an event per buffer): one device arena sized from the
model's own list of tensors, the file mapped and read once, chunk by chunk, through two pinned
buffers that take turns; a chunk whose bytes are already what the device wants (same type, rows
that stay together) is copied straight to its final place, any other (a conversion, interleaved
rows) lands in a device staging buffer and a small kernel of this library puts it in place
(csrc/elementwise.cu: place_rows).  No second copy of the checkpoint is held on the host, and
the pages of the mapping are given back as soon as they are read.
"""
from __future__ import annotations

import mmap
import sys
from typing import Dict, Iterable, List, Optional, Sequence

import torch

from .safetensors import Checkpoint

STAGE_BYTES = 32 << 20            # the reference's staging size (include/qwen3/io/safetensors_loader.h:55-57)
ALIGN = 256


def _role_dtype(role: str, compute: torch.dtype) -> torch.dtype:
    return {"matrix": compute, "norm": torch.float32, "int_table": torch.int32}[role]


def fuse_rows(weights, names: Sequence[str]) -> torch.Tensor:
    """One matrix whose rows are those of `names`, one tensor after the other."""
    rows = getattr(weights, "rows", None)
    if rows is not None:
        return rows(list(names))
    return torch.cat([weights.pop(n) for n in names], dim=0).contiguous()


def fuse_interleaved(weights, first: str, second: str, block: int) -> torch.Tensor:
    """[2R, K]: rows 2*block*t .. +block are rows block*t .. of `first`, the next `block` rows those of `second`."""
    interleaved = getattr(weights, "interleaved", None)
    if interleaved is not None:
        return interleaved(first, second, block)
    a, b = weights.pop(first), weights.pop(second)
    R, K = a.shape
    return torch.stack([a.view(R // block, block, K), b.view(R // block, block, K)], dim=1).reshape(2 * R, K).contiguous()


class TensorDict(dict):
    """Tensors in memory (random weights, tests) prepared for a model: matrices in the compute type on the
    device, everything else moved as it is.  A 32-bit matrix that a bfloat16 engine rounds is announced once."""

    def __init__(self, tensors: Dict[str, torch.Tensor], specs, dtype: torch.dtype, device, warn=None):
        super().__init__()
        warned = False
        for name, t in tensors.items():
            spec = specs.get(name)
            if spec is not None and spec.role == "matrix":
                if t.dtype == torch.float32 and dtype == torch.bfloat16 and not warned and warn is not None:
                    warned = True
                    warn(name)
                t = t.to(device=device, dtype=dtype)
            else:
                t = t.to(device=device)
            self[name] = t


class CheckpointUpload:
    """The tensors of a checkpoint, uploaded on demand into one device arena (see the top of the file)."""

    def __init__(self, checkpoint: Checkpoint, specs, dtype: torch.dtype, device, warn=None):
        self.ckpt, self.specs, self.dtype, self.device = checkpoint, specs, dtype, torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("a checkpoint is uploaded to a CUDA device")
        self._warn, self._warned = warn, False
        total = 0
        for name, spec in specs.items():
            numel = 1
            for s in spec.shape:
                numel *= s
            item = torch.empty((), dtype=_role_dtype(spec.role, dtype)).element_size()
            total += -(-numel * item // ALIGN) * ALIGN
        self.arena = torch.empty(total + ALIGN, dtype=torch.uint8, device=self.device)
        self._used = (-self.arena.data_ptr()) % ALIGN
        self._done: Dict[str, torch.Tensor] = {}
        self._side = torch.cuda.Stream(self.device)
        self._host = [torch.empty(STAGE_BYTES, dtype=torch.uint8).pin_memory() for _ in range(2)]
        self._dev: List[Optional[torch.Tensor]] = [None, None]
        self._events: List[Optional[torch.cuda.Event]] = [None, None]
        self._turn = 0
        self.bytes_uploaded = 0

    # -- what parts call
    def __contains__(self, name) -> bool:
        return name in self.specs

    def __getitem__(self, name: str) -> torch.Tensor:
        t = self._done.get(name)
        if t is None:
            spec = self.specs[name]
            t = self._carve(tuple(spec.shape), _role_dtype(spec.role, self.dtype))
            self._place(name, t.view(-1, t.shape[-1]) if t.dim() > 1 else t.view(1, -1), 0, 0, 0)
            self._done[name] = t
        return t

    def get(self, name, default=None):
        return self[name] if name in self.specs else default

    def pop(self, name, *default):
        if name in self.specs:
            return self[name]
        if default:
            return default[0]
        raise KeyError(name)

    def rows(self, names: List[str]) -> torch.Tensor:
        shapes = [tuple(self.specs[n].shape) for n in names]
        cols = shapes[0][1]
        if any(len(s) != 2 or s[1] != cols for s in shapes):
            raise ValueError(f"rows of {names} do not have one width")
        out = self._carve((sum(s[0] for s in shapes), cols), self.dtype)
        row0 = 0
        for name, shape in zip(names, shapes):
            self._place(name, out, 0, 0, row0)
            row0 += shape[0]
        return out

    def interleaved(self, first: str, second: str, block: int) -> torch.Tensor:
        a, b = tuple(self.specs[first].shape), tuple(self.specs[second].shape)
        if a != b or len(a) != 2 or a[0] % block != 0:
            raise ValueError(f"{first} and {second} cannot be interleaved in blocks of {block} rows")
        out = self._carve((2 * a[0], a[1]), self.dtype)
        self._place(first, out, block, 2 * block, 0)
        self._place(second, out, block, 2 * block, block)
        return out

    def finish(self) -> None:
        """Wait for the copies and kernels in flight and give the staging buffers back."""
        self._side.synchronize()
        torch.cuda.current_stream(self.device).wait_stream(self._side)
        self._host, self._dev, self._events = [], [None, None], [None, None]

    # -- the arena
    def _carve(self, shape, dtype) -> torch.Tensor:
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        if self._used + nbytes > self.arena.numel():      # a tensor asked for in two forms: room of its own
            return torch.empty(shape, dtype=dtype, device=self.device)
        view = self.arena[self._used:self._used + nbytes].view(dtype).view(shape)
        self._used += -(-nbytes // ALIGN) * ALIGN
        return view

    # -- the stream of bytes
    def _place(self, name: str, dst: torch.Tensor, block_rows: int, dst_block_stride: int, dst_row0: int) -> None:
        """The rows of checkpoint tensor `name` into `dst` [rows, cols] (see ops.place_rows for the row map)."""
        from ..csrc import ops
        info = self.ckpt.tensors[name]
        f = info.file
        cols = info.shape[-1] if info.shape else 1
        rows = 1
        for s in info.shape[:-1]:
            rows *= s
        if not info.shape or rows * cols == 0:
            return
        item = torch.empty((), dtype=info.dtype).element_size()
        row_bytes = cols * item
        direct = info.dtype == dst.dtype and block_rows == 0           # the bytes are what the device wants, rows stay together
        if info.dtype == torch.float32 and dst.dtype == torch.bfloat16 and not self._warned and self._warn is not None:
            self._warned = True
            self._warn(name)
        if info.dtype == torch.int32 and not direct:
            raise ValueError(f"{name}: an integer table is copied as it is")
        step = max(1, STAGE_BYTES // row_bytes)
        if block_rows:
            step = max(block_rows, step // block_rows * block_rows)
        if row_bytes > STAGE_BYTES:
            raise ValueError(f"{name}: a row of {row_bytes} bytes does not fit the staging buffer")
        begin = f.data_start + info.begin
        for r0 in range(0, rows, step):
            n = min(step, rows - r0)
            nbytes = n * row_bytes
            slot = self._turn
            self._turn ^= 1
            if self._events[slot] is not None:
                self._events[slot].synchronize()                     # the copy that last read this buffer is done
            host = self._host[slot][:nbytes]
            lo = begin + r0 * row_bytes
            host.copy_(torch.frombuffer(f._map, dtype=torch.uint8, count=nbytes, offset=lo))
            _release_pages(f._map, lo, nbytes)
            with torch.cuda.stream(self._side):
                if direct:
                    dst[dst_row0 + r0:dst_row0 + r0 + n].view(-1).view(torch.uint8).copy_(host, non_blocking=True)
                else:
                    if self._dev[slot] is None:
                        self._dev[slot] = torch.empty(STAGE_BYTES, dtype=torch.uint8, device=self.device)
                    stage = self._dev[slot][:nbytes]
                    stage.copy_(host, non_blocking=True)
                    src = stage.view(info.dtype).view(n, cols)
                    with ops.on_current_stream():
                        if block_rows:
                            ops.place_rows(src, dst, block_rows, dst_block_stride, dst_row0 + (r0 // block_rows) * dst_block_stride)
                        else:
                            ops.place_rows(src, dst, 0, 0, dst_row0 + r0)
                event = torch.cuda.Event()
                event.record(self._side)
            self._events[slot] = event
            self.bytes_uploaded += nbytes


def _release_pages(mapping, offset: int, length: int) -> None:
    """The pages of the mapping that were just read are not needed again: give them back to the system."""
    if not hasattr(mapping, "madvise") or not hasattr(mmap, "MADV_DONTNEED"):
        return
    page = mmap.PAGESIZE
    lo = -(-offset // page) * page
    hi = (offset + length) // page * page
    if hi > lo:
        try:
            mapping.madvise(mmap.MADV_DONTNEED, lo, hi - lo)
        except (OSError, ValueError):
            pass
