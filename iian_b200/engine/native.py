"""The native step function and engine loop (``include/iian_b200/engine.h``) behind Python handles.

``NativeStep`` turns a :class:`~iian_b200.engine.model.Model` whose parts are all built-in (RMSNorm, attention with
rotary or no positions, gated feed-forward, token embedding, head, the pre-norm residual arrangement) into the flat
description the C++ runner walks -- device pointers of the bound weights and of the cache pages, and the constants of
every part -- and runs steps through it: the step's integers are packed, uploaded and the whole kernel sequence is
issued from C++, one call per step from Python.  The Python parts stay the description and remain the step
function of models with parts defined elsewhere (``supports`` says which it is).

``NativeEngine`` is the C++ ``Engine`` (submit / step / abort / stats, the reference's surface,
include/iian/engine.h:67-94) on top of a ``NativeStep``.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_double, c_float, c_int, c_int32, c_longlong, c_void_p
from typing import List, Optional, Sequence

import torch

from ..csrc import build as _build

_DT = {torch.float32: 0, torch.bfloat16: 1}


class _Matrix(Structure):
    _fields_ = [("ptr", c_void_p), ("dtype", c_int), ("rows", c_int), ("cols", c_int)]


class _Layer(Structure):
    _fields_ = [("mixer_norm_w", c_void_p), ("mixer_norm_eps", c_float), ("ffn_norm_w", c_void_p), ("ffn_norm_eps", c_float),
                ("w_qkv", _Matrix), ("w_o", _Matrix), ("b_qkv", c_void_p), ("b_o", c_void_p),
                ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("qk_norm_eps", c_float),
                ("num_heads", c_int), ("num_kv_heads", c_int), ("head_dim", c_int), ("scale", c_float), ("window", c_int),
                ("inv_freq", c_void_p), ("rot_dim", c_int), ("rope_style", c_int), ("rope_key", c_int),
                ("w_gate_up", _Matrix), ("w_down", _Matrix), ("intermediate", c_int), ("interleave", c_int)]


class _Call(Structure):
    _fields_ = [("layer", c_int), ("group", c_int), ("writes_cache", c_int), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("num_pages", c_int)]


class _Model(Structure):
    _fields_ = [("dtype", c_int), ("hidden", c_int), ("vocab", c_int), ("embedding", _Matrix), ("head", _Matrix),
                ("final_norm_w", c_void_p), ("final_norm_eps", c_float), ("layers", POINTER(_Layer)), ("n_layers", c_int),
                ("calls", POINTER(_Call)), ("n_calls", c_int), ("page_size", c_int), ("num_groups", c_int)]


class _RunnerOptions(Structure):
    _fields_ = [(n, c_int) for n in ("max_num_seqs", "max_model_len", "cuda_graphs", "weight_prefetch", "prefetch_window_mb",
                                     "tcgen05_min_tiles", "library_gemm_only", "fuse_norm", "fused_decode", "attention_tc",
                                     "cluster_merge", "tcgen05_pair", "decode_stages", "max_splits", "decode_ctas_per_sm",
                                     "stream_product", "stream_stages", "pdl_stream", "decode_tma", "split_mixed")]


class _Sampling(Structure):
    _fields_ = [("temperature", c_float), ("top_k", c_int), ("top_p", c_float), ("min_p", c_float), ("seed", c_longlong),
                ("max_tokens", c_int), ("min_tokens", c_int), ("ignore_eos", c_int), ("stop_token_ids", POINTER(c_int32)),
                ("n_stop", c_int)]


class _EngineOptions(Structure):
    _fields_ = [("max_model_len", c_int), ("seed", c_longlong), ("eos_token_ids", POINTER(c_int32)), ("n_eos", c_int),
                ("max_num_seqs", c_int), ("max_num_batched_tokens", c_int), ("long_prefill_token_threshold", c_int),
                ("enable_chunked_prefill", c_int), ("priority_policy", c_int)]


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    L = _build.load_engine()
    L.iian_engine_last_error.restype = c_char_p
    L.iian_runner_new.restype = c_void_p
    L.iian_runner_new.argtypes = [POINTER(_Model), POINTER(c_char_p), c_void_p, POINTER(_RunnerOptions)]
    L.iian_runner_delete.argtypes = [c_void_p]
    L.iian_runner_delete.restype = None
    L.iian_runner_step.argtypes = [c_void_p, POINTER(c_void_p), POINTER(c_int32), POINTER(c_int), POINTER(c_int), POINTER(c_int32),
                                   POINTER(c_int), c_int, c_void_p, POINTER(c_void_p), POINTER(c_int)]
    L.iian_runner_step.restype = c_int
    L.iian_runner_get.argtypes = [c_void_p, c_int]
    L.iian_runner_get.restype = c_longlong
    L.iian_runner_launches_of.argtypes = [c_void_p, c_char_p]
    L.iian_runner_launches_of.restype = c_longlong
    L.iian_runner_check_status.argtypes = [c_void_p]
    L.iian_runner_check_status.restype = c_int
    L.iian_runner_set_cuda_graphs.argtypes = [c_void_p, c_int]
    L.iian_runner_set_cuda_graphs.restype = None
    L.iian_engine_new.restype = c_void_p
    L.iian_engine_new.argtypes = [c_void_p, c_void_p, POINTER(_EngineOptions), c_char_p]
    L.iian_engine_delete.argtypes = [c_void_p]
    L.iian_engine_delete.restype = None
    L.iian_engine_submit.argtypes = [c_void_p, POINTER(c_int32), c_int, POINTER(_Sampling), c_int]
    L.iian_engine_submit.restype = c_longlong
    L.iian_engine_abort.argtypes = [c_void_p, c_longlong]
    L.iian_engine_step.argtypes = [c_void_p, c_void_p, POINTER(c_int)]
    L.iian_engine_poll.argtypes = [c_void_p, c_longlong, POINTER(c_int32), c_int, POINTER(c_int), POINTER(c_int)]
    L.iian_engine_has_unfinished.argtypes = [c_void_p]
    L.iian_engine_stats.argtypes = [c_void_p, POINTER(c_longlong), POINTER(c_double)]
    _lib = L
    return L


class NativeError(RuntimeError):
    pass


def _check(code: int) -> None:
    if code != 0:
        raise NativeError(lib().iian_engine_last_error().decode("utf-8", "replace"))


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _matrix(t: torch.Tensor, rows: Optional[int] = None) -> _Matrix:
    if not t.is_contiguous():
        raise NativeError("a weight matrix is not contiguous")
    return _Matrix(t.data_ptr(), _DT[t.dtype], t.shape[0] if rows is None else rows, t.shape[1])


def supports(model) -> bool:
    """Whether every part of ``model`` is one the native step function has a form for."""
    from ..parts.attention import Attention
    from ..parts.block import PreNormResidualBlock
    from ..parts.embedding import LMHead, TokenEmbedding
    from ..parts.mlp import GatedMLP
    from ..parts.norm import RMSNorm
    from ..parts.position import NoPosition, Rotary
    if model.device.type != "cuda" or type(model.embedding) is not TokenEmbedding or type(model.head) is not LMHead \
            or type(model.final_norm) is not RMSNorm:
        return False
    for blk in model.blocks:
        if type(blk) is not PreNormResidualBlock or type(blk.mixer) is not Attention or type(blk.feed_forward) is not GatedMLP \
                or type(blk.mixer_norm) is not RMSNorm or type(blk.feed_forward_norm) is not RMSNorm \
                or type(blk.mixer.position) not in (Rotary, NoPosition):
            return False
    return True


class _DeviceRows:
    """A float32 [rows, cols] array at a device address, for ``torch.as_tensor`` (no copy)."""

    def __init__(self, ptr: int, rows: int, cols: int):
        self.__cuda_array_interface__ = {"shape": (rows, cols), "typestr": "<f4", "data": (ptr, False), "version": 3, "strides": None}


class NativeStep:
    def __init__(self, model, manager, storage, *, max_num_seqs: int, max_model_len: int, cuda_graphs: bool, weight_prefetch: bool = False):
        from ..ops.cuda_backend import CudaKernels, pdl_for
        if not supports(model):
            raise NativeError("this model has parts the native step function has no form for")
        self.model, self.manager, self.storage = model, manager, storage
        self._keep: List[object] = []          # ctypes arrays and tensors the description points at
        K = CudaKernels
        libs = ["elementwise", "rope_kv", "attention_generic", "gemm_simt", "sampling", "gemm_skinny", "attention_mma", "prefetch",
                "gemm_tcgen05", "attention_tc", "gemm_stream"]
        needed = set(model.kernel_libraries()) | {"sampling"}
        _build.preload(sorted(needed))
        paths = (c_char_p * len(libs))(*[_build.library_path(n).encode() if n in needed else None for n in libs])
        rope_keys = {}
        layers = (_Layer * max(1, len(model.blocks)))()
        for i, blk in enumerate(model.blocks):
            a, f, L = blk.mixer, blk.feed_forward, layers[i]
            L.mixer_norm_w, L.mixer_norm_eps = _ptr(blk.mixer_norm.weight), blk.mixer_norm.eps
            L.ffn_norm_w, L.ffn_norm_eps = _ptr(blk.feed_forward_norm.weight), blk.feed_forward_norm.eps
            L.w_qkv, L.w_o = _matrix(a.w_qkv), _matrix(a.w_o)
            L.b_qkv, L.b_o = _ptr(a.b_qkv), _ptr(a.b_o)
            L.q_norm_w, L.k_norm_w, L.qk_norm_eps = _ptr(a.q_norm_w), _ptr(a.k_norm_w), a.eps
            L.num_heads, L.num_kv_heads, L.head_dim, L.scale = a.nh, a.nkv, a.hd, a.scale
            L.window = int(a.window) if a.window is not None else 0
            pos = a.position
            if getattr(pos, "inv_freq", None) is not None:
                L.inv_freq, L.rot_dim, L.rope_style = pos.inv_freq.data_ptr(), pos.dim, pos.style
                L.rope_key = rope_keys.setdefault(pos.key, len(rope_keys))
            L.w_gate_up, L.w_down = _matrix(f.w_gate_up), _matrix(f.w_down)
            L.intermediate, L.interleave = f.inter, f.interleave
        calls = (_Call * max(1, len(model.spec.order)))()
        for i, call in enumerate(model.spec.order):
            view = storage.view(call.cache)
            calls[i] = _Call(call.layer, view.group, int(call.writes_cache), view.k.data_ptr(), view.v.data_ptr(), view.k.shape[0])
        desc = _Model(_DT[model.dtype], model.hidden_size, model.vocab_size, _matrix(model.embedding.weight), _matrix(model.head.weight),
                      _ptr(model.final_norm.weight), model.final_norm.eps, layers, len(model.blocks), calls, len(model.spec.order),
                      manager.block_size, len(manager.groups))
        opt = _RunnerOptions(max_num_seqs, max_model_len, int(cuda_graphs), int(weight_prefetch),
                             int(os.environ.get("IIAN_PREFETCH_WINDOW_MB", "8")), K.TCGEN05_MIN_TILES, int(K.LIBRARY_GEMM_ONLY),
                             int(K.FUSE_NORM), int(K.FUSED_DECODE), int(K.ATTENTION_TC), int(K.CLUSTER_MERGE), int(K.TCGEN05_PAIR),
                             K.DECODE_STAGES, K.MAX_SPLITS, K.DECODE_CTAS_PER_SM_X10, int(K.STREAM_PRODUCT), K.STREAM_STAGES, int(pdl_for("gemm_stream")), int(K.DECODE_TMA), int(K.SPLIT_MIXED))
        self._keep += [layers, calls, paths, desc]
        with torch.cuda.device(model.device):
            self._h = lib().iian_runner_new(ctypes.byref(desc), paths, manager._h, ctypes.byref(opt))
            if model.dtype == torch.bfloat16:
                K.apply_unsplit_stages()          # (the kernel library is the same instance the runner has opened)
        if not self._h:
            raise NativeError(lib().iian_engine_last_error().decode("utf-8", "replace"))
        self.vocab = model.vocab_size

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                lib().iian_runner_delete(self._h)
            except Exception:           # the interpreter is shutting down
                pass
            self._h = None

    def step(self, entries: Sequence) -> Optional[torch.Tensor]:
        """``entries``: objects with ``cache``, ``tokens``, ``start``, ``want`` (the runner's StepEntry).  Float32 logits
        ``[wanted, vocab]`` on the device (valid until the next step), or None."""
        n = len(entries)
        if n == 0:
            return None
        toks: List[int] = []
        want: List[int] = []
        n_tok = (c_int * n)()
        n_want = (c_int * n)()
        starts = (c_int * n)()
        caches = (c_void_p * n)()
        for i, e in enumerate(entries):
            toks += list(e.tokens)
            want += list(e.want)
            n_tok[i], n_want[i], starts[i], caches[i] = len(e.tokens), len(e.want), e.start, e.cache._h
        t_arr = (c_int32 * max(1, len(toks)))(*toks)
        w_arr = (c_int32 * max(1, len(want)))(*want)
        out, rows = c_void_p(), c_int(0)
        with torch.cuda.device(self.model.device):
            _check(lib().iian_runner_step(self._h, caches, t_arr, n_tok, starts, w_arr, n_want, n, torch.cuda.current_stream().cuda_stream,
                                          ctypes.byref(out), ctypes.byref(rows)))
        if not out.value or rows.value == 0:
            return None
        return torch.as_tensor(_DeviceRows(out.value, rows.value, self.vocab), device=self.model.device)

    launches = property(lambda self: lib().iian_runner_get(self._h, 0))
    num_graphs = property(lambda self: lib().iian_runner_get(self._h, 1))
    last_upload_bytes = property(lambda self: lib().iian_runner_get(self._h, 2))

    def launches_of(self, entry: str) -> int:
        return lib().iian_runner_launches_of(self._h, entry.encode())

    def check_status(self) -> None:
        _check(lib().iian_runner_check_status(self._h))

    def set_cuda_graphs(self, on: bool) -> None:
        lib().iian_runner_set_cuda_graphs(self._h, int(bool(on)))


class NativeEngine:
    """The C++ engine loop over a ``NativeStep``: token ids in, token ids out."""

    def __init__(self, step: NativeStep, *, max_model_len: int, seed: int = 0, eos_token_ids: Sequence[int] = (),
                 max_num_seqs: int = 32, max_num_batched_tokens: int = 1024, long_prefill_token_threshold: int = 0,
                 enable_chunked_prefill: bool = True, policy: str = "fcfs"):
        self.step_fn = step
        eos = (c_int32 * max(1, len(eos_token_ids)))(*eos_token_ids)
        opt = _EngineOptions(max_model_len, seed, eos, len(eos_token_ids), max_num_seqs, max_num_batched_tokens,
                             long_prefill_token_threshold, int(enable_chunked_prefill), int(policy == "priority"))
        self._h = lib().iian_engine_new(step._h, step.manager._h, ctypes.byref(opt), _build.library_path("sampling").encode())
        if not self._h:
            raise NativeError(lib().iian_engine_last_error().decode("utf-8", "replace"))
        self._buf = (c_int32 * 4096)()

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                lib().iian_engine_delete(self._h)
            except Exception:
                pass
            self._h = None

    def submit(self, prompt: Sequence[int], *, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0,
               seed: Optional[int] = None, max_tokens: int = -1, min_tokens: int = 0, ignore_eos: bool = False,
               stop_token_ids: Sequence[int] = (), priority: int = 0) -> int:
        arr = (c_int32 * max(1, len(prompt)))(*prompt)
        stop = (c_int32 * max(1, len(stop_token_ids)))(*stop_token_ids)
        p = _Sampling(temperature, top_k, top_p, min_p, -1 if seed is None else seed, max_tokens, min_tokens, int(ignore_eos),
                      stop, len(stop_token_ids))
        rid = lib().iian_engine_submit(self._h, arr, len(prompt), ctypes.byref(p), priority)
        if rid < 0:
            raise ValueError(lib().iian_engine_last_error().decode("utf-8", "replace"))
        return rid

    def abort(self, rid: int) -> None:
        _check(lib().iian_engine_abort(self._h, rid))

    def step(self) -> bool:
        did = c_int(0)
        with torch.cuda.device(self.step_fn.model.device):
            _check(lib().iian_engine_step(self._h, torch.cuda.current_stream().cuda_stream, ctypes.byref(did)))
        return bool(did.value)

    def poll(self, rid: int):
        """The request's next chunk as ``(tokens, finished, finish_reason, n_prompt, n_output, n_cached)``, or None."""
        n, info = c_int(0), (c_int * 5)()
        got = lib().iian_engine_poll(self._h, rid, self._buf, len(self._buf), ctypes.byref(n), info)
        if got < 0:
            raise NativeError(lib().iian_engine_last_error().decode("utf-8", "replace"))
        if got == 0:
            return None
        return list(self._buf[:n.value]), bool(info[0]), int(info[1]), int(info[2]), int(info[3]), int(info[4])

    def has_unfinished(self) -> bool:
        return bool(lib().iian_engine_has_unfinished(self._h))

    def generate(self, prompts: Sequence[Sequence[int]], **params) -> List[List[int]]:
        ids = [self.submit(p, **params) for p in prompts]
        out = {i: [] for i in ids}
        done = set()
        while len(done) < len(ids):
            worked = self.step()
            for i in ids:
                if i in done:
                    continue
                while True:
                    ch = self.poll(i)
                    if ch is None:
                        break
                    out[i] += ch[0]
                    if ch[1]:
                        done.add(i)
                        if ch[2] == 4:
                            raise RuntimeError(f"request {i}: {lib().iian_engine_last_error().decode()}")
                        break
            if not worked and len(done) < len(ids) and not self.has_unfinished():
                break
        return [out[i] for i in ids]

    def stats(self) -> dict:
        vals, usage = (c_longlong * 12)(), c_double(0.0)
        _check(lib().iian_engine_stats(self._h, vals, ctypes.byref(usage)))
        names = ["requests_total", "requests_finished", "requests_aborted", "prompt_tokens", "generation_tokens", "cached_prompt_tokens",
                 "steps", "preemptions", "num_running", "num_waiting", "prefix_cache_queries", "prefix_cache_hits"]
        d = {k: int(v) for k, v in zip(names, vals)}
        d["kv_usage"] = usage.value
        return d
