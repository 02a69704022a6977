"""The engine: a bound model, its cache, and the ONE step function.

`Engine.step(entries)` runs exactly the tokens it is given - the prompts of a batch
that starts together, or one token for each of its sequences - as one packed batch
from the cache that earlier steps left, and returns float32 logits for the wanted
positions.  Generation, trace replay, the benchmark and the tests all call it.

The reference's counterpart is `qwen3_model_forward(token_ids[B,S], ..., start_position)`
plus `qwen3_lm_head` (src/model/model.cpp:107-147, src/model/lm_head.cpp:183-192): a
rectangular batch with one shared start position.  Its validations are kept per
sequence: token ids inside the vocabulary (src/generation/generator.cpp:209-215),
cache capacity (src/model/self_attention.cpp:91-100), positions inside the rotary
table (src/model/model.cpp:81-88).
"""
from __future__ import annotations

import gc
import weakref
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache.storage import KVCache
from ..config.registry import load_config
from ..csrc.build import KernelBuildError
from ..parts.model import Model, build_model
from ..weights.loader import open_upload, random_weights
from .context import Scratch, StepContext

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
          torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


@dataclass
class StepEntry:
    """One sequence's share of a step: its slot, its next tokens, and the places among
    these tokens whose logits are wanted."""
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


class StepError(ValueError):
    """A step that cannot run: empty, out-of-vocabulary ids, a wanted place outside the tokens."""


class _MetaLayout:
    """Offsets of the sections of the step's int32 metadata buffer, as the host runtime lays them out
    (include/qwen3/step_pack.h)."""

    def __init__(self, cache, n_tokens: int, n_seqs: int, n_want: int):
        offsets, self.total = cache.step_layout(n_tokens, n_seqs, n_want)
        (self.token_ids, self.token_seq, self.token_pos, self.seq_slots, self.seq_start, self.seq_pos0,
         self.want_rows) = offsets[:7]
        self.tables = offsets[7:]


class _MetaBuffer:
    """A device int32 buffer with two pinned staging buffers that take turns."""

    def __init__(self, device):
        self.device = device
        self.dev = torch.empty(0, dtype=torch.int32, device=device)
        self._host = [torch.empty(0, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._events = [None, None]
        self._turn = 0

    def reserve(self, total: int) -> None:
        if self.dev.numel() < total:
            self.dev = torch.empty(max(total, 2 * self.dev.numel()), dtype=torch.int32, device=self.device)

    def stage(self, total: int) -> np.ndarray:
        """A host array of `total` int32 to fill; `upload` then copies it to the device buffer."""
        turn = self._turn
        if self._events[turn] is not None:
            self._events[turn].synchronize()      # the copy that last used this staging buffer is done
        if self._host[turn].numel() < total:
            self._host[turn] = torch.empty(max(total, 2 * self._host[turn].numel()), dtype=torch.int32).pin_memory()
        self.reserve(total)
        return self._host[turn].numpy()[:total]

    def upload(self, total: int) -> None:
        turn = self._turn
        self._turn ^= 1
        self.dev[:total].copy_(self._host[turn][:total], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        self._events[turn] = event
        self.bytes_last_upload = total * 4


def context_views(cache, dev, lay, N, B, R, scratch, dtype, max_positions, is_decode, max_new, max_context,
                  host=None, want_all=False) -> StepContext:
    """A StepContext whose device fields are views of the metadata buffer `dev` laid out by `lay`."""
    G, P = len(cache.groups), cache.pages_per_slot
    return StepContext(
        n_tokens=N, n_seqs=B, n_want=R, want_all=want_all, is_decode=is_decode, max_new=max_new,
        max_context=max_context, max_positions=max_positions, dtype=dtype, device=dev.device, scratch=scratch,
        token_ids=dev[lay.token_ids:lay.token_ids + N], token_seq=dev[lay.token_seq:lay.token_seq + N],
        token_pos=dev[lay.token_pos:lay.token_pos + N], seq_slots=dev[lay.seq_slots:lay.seq_slots + B],
        seq_start=dev[lay.seq_start:lay.seq_start + B + 1], seq_pos0=dev[lay.seq_pos0:lay.seq_pos0 + B],
        want_rows=dev[lay.want_rows:lay.want_rows + max(R, 1)],
        page_tables=[dev[lay.tables[g]:lay.tables[g] + B * P].view(B, P) for g in range(G)],
        host_slots=list(host[0]) if host else [], host_n_new=list(host[1]) if host else [],
        host_pos0=list(host[2]) if host else [])


def build_context(cache, meta: "_MetaBuffer", scratch, dtype, max_positions, slots, n_new, pos0, token_ids,
                  want_rows) -> StepContext:
    """Pack one step's metadata (the host runtime does it, in C++), upload it with one copy and return the context
    the parts read.  `cache.reserve` must have made room for the step already (the page rows are read here)."""
    token_ids = np.ascontiguousarray(token_ids, dtype=np.int32).reshape(-1)
    B, N, R = len(slots), int(token_ids.size), len(want_rows)
    lay = _MetaLayout(cache, N, B, R)
    host = meta.stage(lay.total)
    slots_a = np.asarray(slots, dtype=np.int32)
    n_new_a = np.asarray(n_new, dtype=np.int64)
    cache.pack_step(slots_a, n_new_a, token_ids, np.asarray(want_rows, dtype=np.int32), host)
    meta.upload(lay.total)
    longest = int(n_new_a.max())
    return context_views(cache, meta.dev, lay, N, B, R, scratch, dtype, max_positions, longest == 1, longest,
                         int((np.asarray(pos0, dtype=np.int64) + n_new_a).max()), host=(slots, n_new, pos0),
                         want_all=(R == N and list(want_rows) == list(range(N))))


FEW_ROWS, LONG_CONTEXT = 2, 4096     # see Engine._step_captured


def decode_bucket(n: int) -> int:
    """Fixed batch sizes for captured decode steps: 1..8 exactly, then multiples of 8, of 32 above 64."""
    if n <= 8:
        return n
    if n <= 64:
        return -(-n // 8) * 8
    return -(-n // 32) * 32


class _DecodeGraph:
    """One decode step for a fixed number of rows, captured once as a CUDA graph and replayed.

    Rows beyond the live sequences are padding: token 0 at position 0 of the spare page that
    belongs to no sequence; their logits are computed and dropped, no live row reads them."""

    def __init__(self, engine: "Engine", rows: int, max_context: Optional[int] = None):
        self.engine, self.rows = weakref.proxy(engine), rows      # no cycle: an engine dies with its last reference
        max_context = max_context or engine.max_seq_len           # the bound on a sequence's length the parts may count on
        cache = engine.cache
        self.layout = _MetaLayout(cache, rows, rows, rows)
        self.meta = _MetaBuffer(engine.device)
        self.meta.reserve(self.layout.total)
        self.scratch = Scratch(engine.device, guard=engine.scratch.guard)
        self.ctx = context_views(cache, self.meta.dev, self.layout, rows, rows, rows, self.scratch, engine.dtype,
                                 engine.max_seq_len, is_decode=True, max_new=1, max_context=max_context,
                                 want_all=True)
        self.graph = None
        self.logits = None
        self.launches = 0

    def _fill(self, slots, pos0, token_ids) -> None:
        lay = self.layout
        host = self.meta.stage(lay.total)
        self.engine.cache.pack_decode_step(self.rows, np.asarray(slots, dtype=np.int32),
                                           np.ascontiguousarray(token_ids, dtype=np.int32).reshape(-1), host)
        self.meta.upload(lay.total)

    def _capture(self) -> None:
        """Warm up and capture on a batch of padding rows only: whatever a mixer writes while the
        step is recorded (cache pages, state rows) lands in the spare page and the spare row."""
        from ..csrc import ops
        model, cache = self.engine.model, self.engine.cache
        self._fill([], [], [])
        with ops.on_current_stream():
            model.forward(self.ctx, cache)           # loads kernels and library handles outside the capture
        torch.cuda.synchronize(self.engine.device)
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        # an object that owns CUDA resources must not be collected in the middle of a capture
        gc.collect()
        gc_was_enabled = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                with ops.on_current_stream():        # the capture's own stream
                    self.logits = model.forward(self.ctx, cache)
        finally:
            if gc_was_enabled:
                gc.enable()
        self.launches = ops.launch_count() - before
        self.graph = graph

    def run(self, slots, pos0, token_ids, device_tokens=None) -> torch.Tensor:
        """Logits [rows, vocab] of the captured step; rows beyond len(slots) are padding."""
        if self.graph is None:
            self._capture()
        self._fill(slots, pos0, token_ids)
        if device_tokens is not None:
            self.ctx.token_ids[:len(slots)].copy_(device_tokens)
        self.graph.replay()
        self.engine.launches += self.launches
        return self.logits


class Engine:
    """Weights, cache, scratch and stream state of one model on one GPU."""

    def __init__(self, model: Model, config, max_tokens: int, max_seq_len: Optional[int] = None,
                 n_slots: Optional[int] = None, use_graphs: bool = True, guard_scratch: bool = False):
        """`guard_scratch` (tests): activation buffers of exact size between guard zones; see `scratch_violations`."""
        if model.dtype is None:
            raise ValueError("the model has no weights bound")
        self.model, self.config, self.plan = model, config, model.plan
        self.dtype, self.device = model.dtype, model.device
        if self.device.type != "cuda":
            raise KernelBuildError("the engine runs on a CUDA device only; there is no CPU path")
        max_seq_len = min(max_seq_len or self.plan.max_positions, self.plan.max_positions)
        self.cache = KVCache(model.cache_needs(), max_tokens, max_seq_len, self.dtype, self.device, n_slots,
                             cache_from=model.cache_sources())
        self.max_seq_len = self.cache.max_seq_len
        self.vocab_size = self.plan.vocab_size
        self.scratch = Scratch(self.device, guard=guard_scratch)
        self._meta = _MetaBuffer(self.device)
        # a mixer whose step depends on host values (not only on the context's device fields) opts out
        self.use_graphs = use_graphs and all(getattr(b.mixer, "graph_safe", True) for b in model.blocks)
        self._graphs = {}
        self._long_graphs = {}     # captured steps of up to FEW_ROWS sequences whose contexts exceed LONG_CONTEXT
        self.device_tokens = True  # `step` can read a decode step's token ids on the device
        self.launches = 0          # kernels of this library launched by steps (replayed graph nodes included)
        self.last_upload_bytes = 0

    def scratch_violations(self) -> list:
        """Activation buffers (of the launched steps and of every captured decode step) that a kernel wrote beyond;
        empty unless the engine was built with `guard_scratch` and something is wrong."""
        bad = list(self.scratch.violations())
        for graph in list(self._graphs.values()) + list(self._long_graphs.values()):
            bad += graph.scratch.violations()
        return bad

    # -- construction
    @classmethod
    def from_folder(cls, folder: str, dtype=None, max_tokens: int = 4096, max_seq_len: Optional[int] = None,
                    device="cuda:0", n_slots: Optional[int] = None, use_graphs: bool = True,
                    guard_scratch: bool = False) -> "Engine":
        """Load config.json and the safetensors of `folder`; the model class is chosen by config.json."""
        config = load_config(folder)
        model = build_model(config.plan())
        compute = DTYPES[dtype] if dtype is not None else DTYPES[getattr(config, "torch_dtype", "bfloat16")]
        # every tensor goes from the mapped file to its final place on the device in one pass
        source = open_upload(folder, model.weight_specs(), model.ignorable_names(), compute, device, model._warn_rounding)
        model.bind(source, compute, device)
        source.finish()
        engine = cls(model, config, max_tokens, max_seq_len, n_slots, use_graphs, guard_scratch)
        engine.weights_arena = source.arena                    # the parts' tensors are views of it
        return engine

    @classmethod
    def from_random(cls, config, seed: int, dtype=None, max_tokens: int = 4096, max_seq_len: Optional[int] = None,
                    device="cuda:0", n_slots: Optional[int] = None, use_graphs: bool = True,
                    guard_scratch: bool = False) -> "Engine":
        """Seeded random weights drawn on the device (no folder is written)."""
        model = build_model(config.plan())
        compute = DTYPES[dtype] if dtype is not None else DTYPES[getattr(config, "torch_dtype", "bfloat16")]
        weights = random_weights(model.weight_specs(), seed, dtype=compute, device=device)
        model.bind(weights, compute, device)
        return cls(model, config, max_tokens, max_seq_len, n_slots, use_graphs, guard_scratch)

    # -- sequences
    def new_sequence(self) -> int:
        """A free slot for a sequence that starts now (length 0, state zeroed)."""
        return self.cache.alloc_slot()

    def release(self, slot: int) -> None:
        """The sequence is finished: its slot and pages are given back."""
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def check_kernels(self) -> None:
        """Raise if a bounded wait inside a kernel gave up since the last check.  Reads one word
        from the device: call it where the host waits for the device anyway."""
        from ..csrc import ops
        where = ops.tcgen05_status(self.device)
        if where:
            raise ops.KernelError(f"a wait inside the tcgen05 product ran out (stage {where}: 1 producer, 2 MMA, "
                                  f"3 epilogue, 4 accumulator); its results are not valid")

    # -- the step
    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Run the given tokens of every entry as one batch, append them to the cache and return
        float32 logits [wanted, vocab] in the order of the entries and of their `want` (None if
        nothing is wanted).  The tensor is scratch: it is valid until the next step.

        `device_tokens` (int32 [len(entries)] on the device) replaces the tokens of a step in which
        every entry brings one token: the ids are read where the sampler wrote them, and the
        entries' own tokens only stand for the count."""
        if not entries:
            raise StepError("a step needs at least one sequence")
        slots, n_new, tokens, want_rows = [], [], [], []
        start = 0
        for e in entries:
            toks = np.asarray(e.tokens, dtype=np.int64).reshape(-1)
            if toks.size == 0:
                raise StepError(f"slot {e.slot}: a step needs at least one token per sequence")
            if toks.min() < 0 or toks.max() >= self.vocab_size:
                raise StepError(f"slot {e.slot}: token id outside the vocabulary [0, {self.vocab_size})")
            for w in e.want:
                if not 0 <= int(w) < toks.size:
                    raise StepError(f"slot {e.slot}: wanted place {w} is outside its {toks.size} tokens")
                want_rows.append(start + int(w))
            slots.append(int(e.slot)); n_new.append(int(toks.size)); tokens.append(toks)
            start += toks.size
        decode = max(n_new) == 1
        if device_tokens is not None and not decode:
            raise StepError("device_tokens stand for one token per entry")
        step = list(zip(slots, n_new))
        self.cache.reserve(step)                            # raises before anything is launched
        try:
            pos0 = [self.cache.length(s) for s in slots]
            token_ids = np.concatenate(tokens)
            if decode and self.use_graphs:
                logits = self._step_captured(slots, pos0, token_ids, want_rows, device_tokens)
            else:
                from ..csrc import ops
                before = ops.launch_count()
                ctx = self._build_context(slots, n_new, pos0, token_ids, want_rows)
                if device_tokens is not None:
                    ctx.token_ids[:len(slots)].copy_(device_tokens)
                with ops.on_current_stream():
                    logits = self.model.forward(ctx, self.cache)
                self.launches += ops.launch_count() - before
        except BaseException:
            self.cache.cancel(step)                         # a kernel refused its sizes, memory ran out: the pages go back
            raise
        self.cache.commit(step)
        return logits

    def _step_captured(self, slots, pos0, token_ids, want_rows, device_tokens):
        rows = decode_bucket(len(slots))
        # a few sequences with long contexts are a workload of their own (one sequence's keys have to fill the GPU):
        # such steps are captured apart, with `ctx.max_context` beyond LONG_CONTEXT, and parts may choose by it
        few_and_long = rows <= FEW_ROWS and self.max_seq_len > LONG_CONTEXT and max(pos0) + 1 > LONG_CONTEXT
        graphs = self._long_graphs if few_and_long else self._graphs
        graph = graphs.get(rows)
        if graph is None:
            bound = self.max_seq_len if few_and_long or rows > FEW_ROWS else min(self.max_seq_len, LONG_CONTEXT)
            graph = graphs[rows] = _DecodeGraph(self, rows, bound)
        logits = graph.run(slots, pos0, token_ids, device_tokens)
        self.last_upload_bytes = graph.meta.bytes_last_upload
        if not want_rows:
            return None
        if want_rows == list(range(len(want_rows))):
            return logits[:len(want_rows)]
        return logits[torch.as_tensor(want_rows, device=self.device)]

    def _build_context(self, slots, n_new, pos0, token_ids, want_rows) -> StepContext:
        ctx = build_context(self.cache, self._meta, self.scratch, self.dtype, self.max_seq_len, slots, n_new, pos0,
                            token_ids, want_rows)
        self.last_upload_bytes = self._meta.bytes_last_upload
        return ctx
