"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step may hold portions of prompts beside single decoded tokens, cut anywhere.  It runs only the
tokens it is given and returns float32 logits at the wanted places.  The reference builds the same
thing per step from its scheduler's output (``UBatch``, include/iian/graph.h:22-38,
src/iian/engine.cpp:491-535: tokens, positions, sequence index and cache cell per token, output row
ids) and computes masks on the host; here causality and windows are decided inside the kernels from
positions and context lengths, so a step uploads one packed integer buffer and nothing else.

``ModelRunner`` owns the model, the cache manager (page numbers) and the cache storage (device
memory).  The scheduler-driven engine and the trace replay both drive this class; there is no other
forward pass.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import ctypes
import os

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager, RequestCache
from ..cache.storage import CacheStorage, plan_groups
from ..parts.base import KVNeed, StateNeed, prefix_reusable
from .model import Model


@dataclass
class StepEntry:
    """One request's share of a step: ``tokens`` follow the ``start`` tokens already in its cache;
    ``want`` lists indices into ``tokens`` whose logits are returned."""

    cache: RequestCache
    tokens: Sequence[int]
    start: int
    want: Sequence[int] = ()


class Workspace:
    """Activation buffers by name, grown on demand and reused from step to step."""

    def __init__(self, device: torch.device):
        self.device = device
        self._bufs: Dict[Tuple[str, torch.dtype], torch.Tensor] = {}
        self._views: Dict[tuple, torch.Tensor] = {}      # (name, dtype, shape) -> the view handed out last time
        self.frozen = False          # set while a CUDA graph that uses these buffers is alive

    def get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        vkey = (name, dtype, tuple(shape))
        v = self._views.get(vkey)
        if v is not None:
            return v
        v = self._get(name, shape, dtype)
        if len(self._views) > 4096:
            self._views.clear()
        self._views[vkey] = v
        return v

    def _get(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        t = self._bufs.get(key)
        if t is None or t.numel() < n:
            if self.frozen:
                raise RuntimeError(f"workspace buffer '{name}' would have to grow while a captured graph uses it")
            cap = max(n, 1)
            t = torch.empty(cap, dtype=dtype, device=self.device)
            self._bufs[key] = t
            self._views = {k: v for k, v in self._views.items() if (k[0], k[1]) != key}     # views of the old buffer
        return t[:n].view(*shape)


@dataclass
class PageMeta:
    """What a mixer that keeps its past in pages needs for one page group: where each token of the step goes, and each
    sequence's block table and length."""

    positions: torch.Tensor        # i32 [N]
    seq_of_token: torch.Tensor     # i32 [N]   (-1: padding token)
    cu_q: torch.Tensor             # i32 [S + 1]
    ctx_len: torch.Tensor          # i32 [S]   tokens in the cache after this step
    block_table: torch.Tensor      # i32 [S, max_blocks]
    slots: torch.Tensor            # i32 [N]   cache cell of each token (-1: store nothing)
    num_seqs: int
    num_tokens: int
    max_q_len: int
    max_ctx: int
    decode_only: bool
    h_q_len: Sequence[int] = ()
    h_ctx_len: Sequence[int] = ()


AttentionMeta = PageMeta


class StepContext:
    def __init__(self, workspace: Workspace):
        self.workspace = workspace
        self.tokens = self.positions = self.seq_of_token = self.cu_q = self.ctx_len = None
        self.state_slots = self.out_rows = None
        self.metas: List[PageMeta] = []
        self.plans: Dict[int, object] = {}             # captured graphs: what each mixer asked to keep fixed (Mixer.graph_plan)
        self.step_cache: Dict[object, object] = {}     # what parts compute once per forward pass and share (cleared by Model.forward)
        self.num_tokens = self.num_seqs = 0
        self.h_q_start: List[int] = []
        self.h_q_len: List[int] = []
        self.h_ctx_len: List[int] = []
        self.h_state_slots: List[int] = []
        self.decode_only = False
        self.rows_identity = False     # the wanted rows are all rows in order: no gather is needed
        self.max_q_len = 0
        self.max_ctx = 0
        self.upload_bytes = 0

    def buf(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        return self.workspace.get(name, shape, dtype)

    def page_meta(self, group: int) -> PageMeta:
        return self.metas[group]

    attention_meta = page_meta

    def graph_plan(self, part):
        """What ``part`` asked to keep fixed inside the captured graph this step is replayed from (its own
        ``graph_plan`` answer), or None on an eager step."""
        return self.plans.get(id(part))


class ModelRunner:
    def __init__(self, model: Model, *, block_size: int = 16, capacity_tokens: int, max_num_seqs: int = 4,
                 enable_prefix_caching: bool = False, window_capacity_tokens: Optional[int] = None,
                 cuda_graphs: bool = False, max_model_len: Optional[int] = None, native: Optional[bool] = None):
        self.model = model
        # decode steps are replayed from graphs only if every part of the model can be recorded
        self.native = None
        self.cuda_graphs = cuda_graphs and model.device.type == "cuda" and model.graph_safe()
        # Prefetching the head of the next product's weights into L2 on a side stream (csrc/prefetch.cu) pays with the
        # register form of the small-batch product (+2.4 %); the streaming product started early by a programmatic
        # dependent launch does the same thing itself and is faster without it (2.97 -> 2.91 ms at batch 1).
        self.weight_prefetch = os.environ.get("IIAN_WEIGHT_PREFETCH", "0") not in ("0", "false", "off")
        self.max_model_len = max_model_len or capacity_tokens
        self._graphs: Dict[Tuple[int, int], "_GraphSlot"] = {}
        self.launches = 0                 # kernel launches issued through this runner (graph replays included)
        self.device = model.device
        self.block_size = block_size
        self.max_num_seqs = max_num_seqs
        needs = model.cache_needs()
        groups, kinds = plan_groups(needs, capacity_tokens, block_size, window_capacity_tokens)
        has_state = any(isinstance(n, StateNeed) for n in needs.values())
        # a request may start behind another request's prefix only if every cache of the model can be shared
        # page by page (and there is at least one page group to share)
        self.prefix_caching = bool(enable_prefix_caching and groups and all(prefix_reusable(n) for n in needs.values()))
        self.manager = CacheManager(groups, block_size, self.prefix_caching, num_state_slots=max_num_seqs)
        self.storage = CacheStorage(needs, groups, kinds, block_size, max_num_seqs if has_state else 0,
                                    model.dtype, self.device)
        self.workspace = Workspace(self.device)
        self._pinned: Optional[torch.Tensor] = None
        self._staging_dev: Optional[torch.Tensor] = None
        self._copy_done = None
        self.last_upload_bytes = 0
        if self.device.type == "cuda":
            from ..csrc import build
            build.preload(model.kernel_libraries())      # compile what this model needs, together
        # The step function in C++ (include/iian_b200/engine.h) for models made of built-in parts only: the same kernels
        # in the same order, issued without a Python call per launch.  ``native=None``: as IIAN_NATIVE_STEP says (default on).
        if native is None:
            native = os.environ.get("IIAN_NATIVE_STEP", "1") not in ("0", "false", "off")
        if native and self.device.type == "cuda":
            from . import native as _native
            from .. import ops as _ops
            if _native.supports(model) and getattr(_ops.kernels(), "name", "") == "cuda":
                self.native = _native.NativeStep(model, self.manager, self.storage, max_num_seqs=max_num_seqs,
                                                 max_model_len=self.max_model_len, cuda_graphs=self.cuda_graphs,
                                                 weight_prefetch=self.weight_prefetch)

    @property
    def cuda_graphs(self) -> bool:
        return self._cuda_graphs

    @cuda_graphs.setter
    def cuda_graphs(self, on: bool) -> None:
        self._cuda_graphs = bool(on)
        if self.native is not None:
            self.native.set_cuda_graphs(self._cuda_graphs)

    ENTRIES = ("embedding", "add_rms_norm", "swiglu", "gather_rows", "add_bias", "rotary_table", "qk_norm_rope_store",
               "paged_attention_generic", "gemm_simt", "gemm_skinny", "gemm_skinny_fused", "gemm_stream", "gemm_tcgen05", "attention_tc",
               "attention_mma", "attention_decode_fused", "prefetch_l2", "library_gemm")

    def launches_by_entry(self) -> Dict[str, int]:
        """Launches so far by the kernel layer's entry point, whichever step function issued them (the Python kernel
        layer counts for the whole process, the native step function for this runner)."""
        from ..ops import cuda_backend
        out = dict(cuda_backend.LAUNCHES_BY_ENTRY)
        if self.native is not None:
            for name in self.ENTRIES:
                n = self.native.launches_of(name)
                if n:
                    out[name] = out.get(name, 0) + n
        return out

    def check_device_status(self) -> None:
        """Raise if a tcgen05 kernel gave up waiting on a barrier since the last call (its output would be garbage)."""
        from .. import ops
        k = ops.kernels()
        if hasattr(k, "check_device_status"):
            k.check_device_status()
        if self.native is not None:
            self.native.check_status()

    @property
    def num_graphs(self) -> int:
        """Decode graphs captured so far (by whichever step function runs)."""
        return self.native.num_graphs if self.native is not None else len(self._graphs)

    # ---- batch building ---------------------------------------------------------------------
    def _stage(self, n_ints: int) -> Tuple[np.ndarray, torch.Tensor]:
        """Host array (pinned on CUDA) and device tensor of at least ``n_ints`` int32."""
        if self._staging_dev is None or self._staging_dev.numel() < n_ints:
            cap = max(4096, 2 * n_ints)
            self._staging_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._pinned = torch.empty(cap, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        if self._copy_done is not None:
            self._copy_done.synchronize()       # the last step's upload has left the host buffer
        return self._pinned.numpy(), self._staging_dev

    def build_context(self, entries: Sequence[StepEntry], slot: Optional["_GraphSlot"] = None) -> StepContext:
        """Pack the step's integers on the host and upload them with one copy.  With ``slot`` (a
        captured decode graph) the batch is padded to the slot's fixed shape and written into the
        slot's own buffers: padding sequences bring one token that is stored nowhere (cell -1)."""
        mgr = self.manager
        bs = self.block_size
        n_real = len(entries)
        n_groups = len(mgr.groups)
        if slot is None:
            S = n_real
            N = sum(len(e.tokens) for e in entries)
            R = sum(len(e.want) for e in entries)
            max_blocks = []
            for g in range(n_groups):
                mb = 1
                for e in entries:
                    mb = max(mb, mgr.blocks_for(e.start + len(e.tokens)))
                max_blocks.append(mb)
        else:
            S = N = R = slot.num_seqs
            max_blocks = [slot.max_blocks] * n_groups
        total = 3 * N + (S + 1) + 2 * S + R + sum(N + S * mb for mb in max_blocks)
        if slot is None:
            host, dev = self._stage(total)
            pinned = self._pinned
        else:
            if slot.copy_done is not None:
                slot.copy_done.synchronize()
            host, dev, pinned = slot.pinned.numpy(), slot.staging, slot.pinned
        off = 0

        def take(n):
            nonlocal off
            a = (off, off + n)
            off += n
            return a

        r_tok, r_pos, r_seq = take(N), take(N), take(N)
        r_cu, r_ctx, r_slot_state, r_rows = take(S + 1), take(S), take(S), take(R)
        r_slots = [take(N) for _ in range(n_groups)]
        r_bt = [take(S * mb) for mb in max_blocks]

        ctx = StepContext(self.workspace if slot is None else slot.workspace)
        if slot is not None:       # padding first; real sequences overwrite the front
            host[r_tok[0]: r_tok[1]] = 0
            host[r_pos[0]: r_pos[1]] = 0
            host[r_seq[0]: r_seq[1]] = -1
            host[r_cu[0]: r_cu[1]] = np.arange(S + 1, dtype=np.int32)
            host[r_ctx[0]: r_ctx[1]] = 1
            host[r_slot_state[0]: r_slot_state[1]] = -1
            host[r_rows[0]: r_rows[1]] = np.arange(R, dtype=np.int32)
            for g in range(n_groups):
                host[r_slots[g][0]: r_slots[g][1]] = -1
                host[r_bt[g][0]: r_bt[g][1]] = 0
        t0 = 0
        rows: List[int] = []
        fresh: List[int] = []
        host[r_cu[0]] = 0
        for s, e in enumerate(entries):
            n = len(e.tokens)
            if n == 0:
                raise ValueError("a step entry must bring at least one token")
            host[r_tok[0] + t0: r_tok[0] + t0 + n] = np.asarray(e.tokens, dtype=np.int32)
            host[r_pos[0] + t0: r_pos[0] + t0 + n] = np.arange(e.start, e.start + n, dtype=np.int32)
            host[r_seq[0] + t0: r_seq[0] + t0 + n] = s
            host[r_cu[0] + s + 1] = t0 + n
            host[r_ctx[0] + s] = e.start + n
            host[r_slot_state[0] + s] = e.cache.state_slot
            if e.cache.state_fresh:
                fresh.append(e.cache.state_slot)
                e.cache.state_fresh = False
            for w in e.want:
                if not 0 <= w < n:
                    raise ValueError(f"wanted place {w} is outside this step's {n} tokens")
                rows.append(t0 + w)
            for g in range(n_groups):
                table = e.cache.tables[g]
                need_blocks = mgr.blocks_for(e.start + n)
                if len(table) < need_blocks:
                    raise ValueError(f"request holds {len(table)} pages in group {g}, needs {need_blocks}")
                mb = max_blocks[g]
                row = host[r_bt[g][0] + s * mb: r_bt[g][0] + (s + 1) * mb]
                row[:] = -1
                row[:need_blocks] = np.asarray(table[:need_blocks], dtype=np.int32)
                pos = np.arange(e.start, e.start + n)
                pages = row[pos // bs]
                if (pages < 0).any():
                    raise ValueError("a token of this step lies in a page that was given back")
                host[r_slots[g][0] + t0: r_slots[g][0] + t0 + n] = pages * bs + (pos % bs)
            ctx.h_q_start.append(t0)
            ctx.h_q_len.append(n)
            ctx.h_ctx_len.append(e.start + n)
            ctx.h_state_slots.append(e.cache.state_slot)
            t0 += n
        if slot is None:
            host[r_rows[0]: r_rows[1]] = np.asarray(rows, dtype=np.int32) if rows else 0

        dev[:total].copy_(pinned[:total], non_blocking=True)
        if self.device.type == "cuda":
            if slot is None:
                if self._copy_done is None:
                    self._copy_done = torch.cuda.Event()
                self._copy_done.record()
            else:
                if slot.copy_done is None:
                    slot.copy_done = torch.cuda.Event()
                slot.copy_done.record()
        self.storage.zero_state(fresh)

        def view(r, shape=None):
            t = dev[r[0]: r[1]]
            return t.view(*shape) if shape is not None else t

        ctx.tokens, ctx.positions, ctx.seq_of_token = view(r_tok), view(r_pos), view(r_seq)
        ctx.cu_q, ctx.ctx_len, ctx.state_slots, ctx.out_rows = view(r_cu), view(r_ctx), view(r_slot_state), view(r_rows)
        ctx.num_tokens, ctx.num_seqs = N, S
        ctx.max_q_len = max(ctx.h_q_len) if ctx.h_q_len else 0
        ctx.max_ctx = max(ctx.h_ctx_len) if ctx.h_ctx_len else 0
        if slot is not None:
            ctx.max_q_len, ctx.max_ctx = 1, slot.ctx_bucket
        ctx.decode_only = ctx.max_q_len == 1
        ctx.rows_identity = slot is not None or rows == list(range(N))
        ctx.upload_bytes = total * 4
        for g in range(n_groups):
            ctx.metas.append(PageMeta(
                positions=ctx.positions, seq_of_token=ctx.seq_of_token, cu_q=ctx.cu_q, ctx_len=ctx.ctx_len,
                block_table=view(r_bt[g], (S, max_blocks[g])), slots=view(r_slots[g]),
                num_seqs=S, num_tokens=N, max_q_len=ctx.max_q_len, max_ctx=ctx.max_ctx,
                decode_only=ctx.decode_only, h_q_len=ctx.h_q_len, h_ctx_len=ctx.h_ctx_len))
        if slot is not None:
            ctx.plans = slot.plans
        return ctx

    def build_decode_context(self, entries: Sequence[StepEntry], slot: "_GraphSlot") -> StepContext:
        """``build_context`` for a captured decode graph, written for the step that comes thousands of times:
        every entry brings one token, the shape is the slot's.  The packing is native
        (``iian_pack_decode_step``, include/iian_b200/c_api.h).  What does not change from step to step is not
        written again: the padding behind the real sequences, and the rows of the block tables, of which a
        step only appends a page now and then (a row is rewritten when another request takes it or when its
        request's table changed otherwise, which the table's epoch tells)."""
        from ..cache import native
        mgr = self.manager
        n, S, mb = len(entries), slot.num_seqs, slot.max_blocks
        n_groups = len(mgr.groups)
        if slot.copy_done is not None:
            slot.copy_done.synchronize()
        lay = slot.layout
        if lay is None:
            off = 0
            lay = {}
            for name, size in (("tok", S), ("pos", S), ("seq", S), ("cu", S + 1), ("ctx", S), ("state", S), ("rows", S)):
                lay[name] = off
                off += size
            lay["slots"] = []
            for _ in range(n_groups):
                lay["slots"].append(off)
                off += S
            lay["bt"] = []
            for _ in range(n_groups):
                lay["bt"].append(off)
                off += S * mb
            lay["total"] = off
            slot.layout = lay
            slot.host_ptr = slot.pinned.data_ptr()
            slot.sig = (ctypes.c_longlong * (n_groups * S * 3))()
            slot.c_caches = (ctypes.c_void_p * S)()
            slot.c_tokens = (ctypes.c_int32 * S)()
            slot.c_starts = (ctypes.c_int32 * S)()
            slot.c_fresh = (ctypes.c_int * S)()
        caches, toks, starts = slot.c_caches, slot.c_tokens, slot.c_starts
        for s, e in enumerate(entries):
            caches[s] = e.cache._h
            toks[s] = e.tokens[0]
            starts[s] = e.start
        n_fresh = native.lib().iian_pack_decode_step(mgr._h, caches, toks, starts, n, S, mb, slot.host_ptr,
                                                     ctypes.addressof(slot.sig), int(slot.n_last != n), slot.c_fresh)
        if n_fresh < 0:
            slot.n_last = -1                 # the buffer may be half written
            native.check(2)
        slot.n_last = n
        fresh = list(slot.c_fresh[:n_fresh])
        total = lay["total"]
        slot.staging[:total].copy_(slot.pinned[:total], non_blocking=True)
        if slot.copy_done is None:
            slot.copy_done = torch.cuda.Event()
        slot.copy_done.record()
        self.storage.zero_state(fresh)
        ctx = slot.ctx
        if ctx is None:
            dev = slot.staging

            def view(start, size, shape=None):
                t = dev[start: start + size]
                return t.view(*shape) if shape is not None else t

            ctx = StepContext(slot.workspace)
            ctx.tokens, ctx.positions, ctx.seq_of_token = view(lay["tok"], S), view(lay["pos"], S), view(lay["seq"], S)
            ctx.cu_q, ctx.ctx_len = view(lay["cu"], S + 1), view(lay["ctx"], S)
            ctx.state_slots, ctx.out_rows = view(lay["state"], S), view(lay["rows"], S)
            ctx.num_tokens = ctx.num_seqs = S
            ctx.max_q_len, ctx.max_ctx = 1, slot.ctx_bucket
            ctx.decode_only = True
            ctx.rows_identity = True
            ctx.upload_bytes = total * 4
            for g in range(n_groups):
                ctx.metas.append(PageMeta(
                    positions=ctx.positions, seq_of_token=ctx.seq_of_token, cu_q=ctx.cu_q, ctx_len=ctx.ctx_len,
                    block_table=view(lay["bt"][g], S * mb, (S, mb)), slots=view(lay["slots"][g], S),
                    num_seqs=S, num_tokens=S, max_q_len=1, max_ctx=slot.ctx_bucket, decode_only=True,
                    h_q_len=ctx.h_q_len, h_ctx_len=ctx.h_ctx_len))
            ctx.plans = slot.plans
            slot.ctx = ctx
        ctx.h_q_start[:] = range(n)
        ctx.h_q_len[:] = [1] * n
        ctx.h_ctx_len[:] = [e.start + 1 for e in entries]
        ctx.h_state_slots[:] = [e.cache.state_slot for e in entries] if self.manager.slots.num_slots else [-1] * n
        return ctx

    # ---- the step -----------------------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Logits ``[sum(len(want)), vocab]`` in the order of the entries and of their ``want`` lists
        (None if nothing is wanted).  Pages for every entry's tokens must already be allocated."""
        if not entries:
            return None
        if len(entries) > self.max_num_seqs:
            raise ValueError(f"{len(entries)} requests in one step, the runner was built for {self.max_num_seqs}")
        if self.native is not None:
            before = self.native.launches
            out = self.native.step(entries)
            self.launches += self.native.launches - before
            self.last_upload_bytes = self.native.last_upload_bytes
            return out
        if self.cuda_graphs and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            return self._step_graph(entries)
        ctx = self.build_context(entries)
        before = _launch_count()
        out = self.model.forward(ctx, self.storage)
        self.launches += _launch_count() - before
        self.last_upload_bytes = ctx.upload_bytes
        return out

    # ---- decode-only steps replayed from captured CUDA graphs ------------------------------------
    def _step_graph(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """The reference replays whole steps from CUDA graphs keyed by the batch's shape
        (src/iian/engine.cpp:553-574, CMakeLists.txt:32-37).  Here a graph is keyed by (padded number of
        sequences, context bucket); its kernels read the step's integers from fixed device buffers, so a
        replay needs one upload and one launch."""
        n = len(entries)
        # batches are padded to 1, 2, 4, 8, then to multiples of 4 up to 32, of 8 up to 64, of 16 up to 128 and of 32
        # beyond: padding sequences are CTAs of the attention launch too, and whether those fit the GPU at once decides
        # its form
        if n <= 8:
            bucket = 1
            while bucket < n:
                bucket *= 2
        else:
            step = 4 if n <= 32 else 8 if n <= 64 else 16 if n <= 128 else 32
            bucket = -(-n // step) * step
        bucket = min(bucket, max(self.max_num_seqs, n))
        max_ctx = max(e.start + 1 for e in entries)
        ctx_bucket = 256
        while ctx_bucket < max_ctx:
            ctx_bucket *= 2
        key = (bucket, ctx_bucket)
        slot = self._graphs.get(key)
        if slot is None:
            slot = self._capture(bucket, ctx_bucket)
            self._graphs[key] = slot
        ctx = self.build_decode_context(entries, slot)
        slot.graph.replay()
        self.launches += slot.launches
        self.last_upload_bytes = ctx.upload_bytes
        return slot.logits[:n]

    def _capture(self, num_seqs: int, ctx_bucket: int) -> "_GraphSlot":
        mgr = self.manager
        n_groups = len(mgr.groups)
        max_blocks = max(1, mgr.blocks_for(max(self.max_model_len, ctx_bucket)))
        total = 3 * num_seqs + (num_seqs + 1) + 3 * num_seqs + n_groups * (num_seqs + num_seqs * max_blocks)
        slot = _GraphSlot()
        slot.num_seqs, slot.ctx_bucket, slot.max_blocks = num_seqs, ctx_bucket, max_blocks
        slot.staging = torch.empty(total, dtype=torch.int32, device=self.device)
        slot.pinned = torch.empty(total, dtype=torch.int32, pin_memory=True)
        slot.workspace = Workspace(self.device)
        slot.copy_done = None
        k = ops.kernels()
        # what every mixer wants kept fixed inside this graph (attention: its number of key splits)
        slot.plans = {}
        for part in self.model.all_parts():
            plan = part.graph_plan(num_seqs, ctx_bucket) if hasattr(part, "graph_plan") else None
            if plan is not None:
                slot.plans[id(part)] = plan
        # Warm up eagerly on a batch of padding sequences only (it loads the kernels, sizes every buffer and
        # records the order in which weights are streamed, but stores nothing: padding tokens have cache cell
        # -1 and state slot -1), then capture the same launches -- with a side stream that prefetches the next
        # weights.  The step that asked for this graph then runs exactly once, as the first replay: a mixer
        # with state of its own must not see a step twice.
        ctx = self.build_context([], slot)
        prefetch = self.weight_prefetch and hasattr(k, "weight_log")
        if prefetch:
            k.weight_log = []
        try:
            self.model.forward(ctx, self.storage)
        finally:
            weights = k.weight_log if prefetch else None
            if prefetch:
                k.weight_log = None
        torch.cuda.synchronize(self.device)
        slot.workspace.frozen = True
        before = _launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            if prefetch and weights:
                from ..ops.cuda_backend import WeightPrefetcher
                k.prefetcher = WeightPrefetcher(weights)
            try:
                slot.logits = self.model.forward(ctx, self.storage)
                if k.prefetcher is not None:
                    k.prefetcher.join()
            finally:
                if prefetch:
                    k.prefetcher = None
        slot.launches = _launch_count() - before
        slot.graph = graph
        return slot


class _GraphSlot:
    """Everything a captured decode graph owns: fixed-shape integer buffers, workspace, output."""

    num_seqs = ctx_bucket = max_blocks = launches = 0
    staging = pinned = workspace = copy_done = graph = logits = plans = None
    layout = host_ptr = sig = c_caches = c_tokens = c_starts = c_fresh = ctx = None      # kept between steps by build_decode_context
    n_last = -1


def _launch_count() -> int:
    from ..ops import cuda_backend
    return cuda_backend.LAUNCHES[0]
