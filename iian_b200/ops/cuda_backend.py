"""The engine's kernels as Python functions on torch CUDA tensors.

Every function validates its tensors (device, dtype, contiguity, shapes), then launches a
hand-written kernel from ``iian_b200/csrc`` on the current CUDA stream through ``ctypes``.
Nothing here computes with torch ops; a tensor that is not on a CUDA device is an error, there
is no CPU path.  Large bfloat16 matrix products may go to the library GEMM, as in the reference
(third_party/ggml/src/ggml-cuda/ggml-cuda.cu:1548-1608 calls cuBLAS for batches its own
mat-vec kernels do not cover).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from ..csrc import build as _build

F32, BF16 = 0, 1
_CODE = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_ERRS = {1: "element types not supported by this kernel", 2: "a size this kernel refuses",
         3: "a pointer or stride is not aligned as the kernel requires", 4: "beyond the kernel's stated maximum",
         5: "the address of a device array inside the library could not be resolved"}


LAUNCHES = [0]        # kernel launches issued by this module (a split attention counts its merge kernel too)
LAUNCHES_BY_ENTRY = {}     # the same by entry point ("attention_tc", "gemm_skinny_fused", ...; "library_gemm" for cuBLAS):
                           # tests read it to see which kernel a step was served by (a replayed graph counts once, at capture)


def _check(code: int, what: str) -> None:
    if code == 0:
        LAUNCHES[0] += 1
        LAUNCHES_BY_ENTRY[what] = LAUNCHES_BY_ENTRY.get(what, 0) + 1
        return
    if code >= 1000:
        raise KernelError(f"{what}: CUDA launch failed with error {code - 1000}")
    raise KernelError(f"{what}: {_ERRS.get(code, f'error {code}')}")


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _CODE[t.dtype]
    except KeyError:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)") from None


def _cuda(t: Optional[torch.Tensor], what: str, dtype=None) -> int:
    """Pointer of a contiguous CUDA tensor (0 for None)."""
    if t is None:
        return 0
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}; the engine's kernels run on CUDA only")
    if not t.is_contiguous():
        raise KernelError(f"{what}: tensor must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: expected {dtype}, got {t.dtype}")
    return t.data_ptr()


_PINNED_STREAM = [0]


def _stream() -> int:
    """The CUDA stream the kernels are launched on: torch's current stream, looked up once per forward pass
    (``pin_stream``) rather than once per launch -- the lookup costs more than the launch itself."""
    return _PINNED_STREAM[0] or torch.cuda.current_stream().cuda_stream


class pin_stream:
    """``with pin_stream():`` every launch inside goes to the stream that is current on entry.  Code that
    switches streams inside (the weight prefetcher's side stream) passes its stream explicitly."""

    def __enter__(self):
        self.before = _PINNED_STREAM[0]
        _PINNED_STREAM[0] = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        _PINNED_STREAM[0] = self.before
        return False


_sigs_done = set()


# Programmatic dependent launch (see csrc/common.cuh).  IIAN_PDL names the kernel libraries whose launches get the
# attribute ("gemm_stream,attention_mma"; "1": all, "0": none).  Default: the streaming product alone.  Its CTAs fill
# their ring of shared memory with weights while the kernel before drains, and they cannot crowd that kernel out (a CTA
# takes nearly all of an SM's shared memory, so it only becomes resident where one has left): 3.10 -> 2.91 ms per decode
# step at batch 1, 3.60 -> 3.31 at batch 8.  With the attribute on every kernel of the step the register-bound kernels
# of the chain did lose resources to their successors (4.16 ms at batch 1 when the products were of that kind).
_PDL_ENV = os.environ.get("IIAN_PDL", "gemm_stream")
PDL = _PDL_ENV not in ("0", "false", "off")
_PDL_LIBS = None if _PDL_ENV in ("0", "false", "off", "1", "true", "on") else {n.strip() for n in _PDL_ENV.split(",")}


def pdl_for(lib_name: str) -> bool:
    return PDL and (_PDL_LIBS is None or lib_name in _PDL_LIBS)


_pdl_set = set()


def _fn(lib_name: str, fn_name: str, argtypes):
    lib = _build.load(lib_name)
    if lib_name not in _pdl_set:
        _pdl_set.add(lib_name)
        if hasattr(lib, "iian_set_pdl"):
            lib.iian_set_pdl.argtypes = [c_int]
            lib.iian_set_pdl.restype = None
            lib.iian_set_pdl(1 if pdl_for(lib_name) else 0)
    fn = getattr(lib, fn_name)
    key = (lib_name, fn_name)
    if key not in _sigs_done:
        fn.argtypes = argtypes
        fn.restype = c_int
        _sigs_done.add(key)
    return fn


class CudaKernels:
    """The kernel set the product path uses."""

    name = "cuda"

    # ---- libraries a model needs (compiled together on first use) ----------------------
    def prepare(self, dtype: torch.dtype) -> None:
        names = ["elementwise", "rope_kv", "attention_generic", "gemm_simt", "sampling"]
        if dtype == torch.bfloat16:
            names += [n for n in _build.SOURCES if n not in names and n in _build.BF16_SOURCES]
        _build.preload(names)

    # ---- row-wise ------------------------------------------------------------------------
    def embedding(self, table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> None:
        n, h = out.shape
        fn = _fn("elementwise", "iian_embedding", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(table, "embedding table"), _code(table, "embedding table"),
                  _cuda(tokens, "tokens", torch.int32), _cuda(out, "embedding out", torch.float32),
                  n, h, table.shape[0], _stream()), "embedding")

    def add_rms_norm(self, residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor,
                     eps: float, out: torch.Tensor) -> None:
        n, h = residual.shape
        if delta is not None and (delta.shape != residual.shape or delta.dtype != out.dtype):
            raise KernelError(f"add_rms_norm: delta {tuple(delta.shape)} {delta.dtype} does not match "
                              f"residual {tuple(residual.shape)} / out {out.dtype}")
        if out.shape != residual.shape or weight.numel() != h:
            raise KernelError("add_rms_norm: shapes of out / weight do not match the residual")
        fn = _fn("elementwise", "iian_add_rms_norm",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
        _check(fn(_cuda(residual, "residual", torch.float32), _cuda(delta, "delta"),
                  _cuda(weight, "norm weight", torch.float32), _cuda(out, "norm out"), _code(out, "norm out"),
                  n, h, eps, _stream()), "add_rms_norm")

    def rms_norm(self, x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
        n, h = x.shape
        if out.shape != x.shape or out.dtype != x.dtype or weight.numel() != h:
            raise KernelError("rms_norm: out / weight do not match the input")
        fn = _fn("elementwise", "iian_rms_norm", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
        _check(fn(_cuda(x, "rms_norm in"), _cuda(weight, "norm weight", torch.float32), _cuda(out, "rms_norm out"),
                  _code(x, "rms_norm in"), n, h, eps, _stream()), "rms_norm")

    def swiglu(self, gate_up: torch.Tensor, out: torch.Tensor, interleave: int = 0) -> None:
        """``interleave`` 0: columns are [gate | up]; 8: groups of 16 columns, 8 gate then 8 up values."""
        n, f2 = gate_up.shape
        if out.shape != (n, f2 // 2) or f2 % 2 or out.dtype != gate_up.dtype:
            raise KernelError("swiglu: out must be [N, F] for gate_up [N, 2F] of the same dtype")
        fn = _fn("elementwise", "iian_swiglu", [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(gate_up, "gate_up"), _cuda(out, "swiglu out"), _code(out, "swiglu out"), n, f2 // 2, interleave,
                  _stream()), "swiglu")

    def gather_rows(self, src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
        r, h = out.shape
        if src.shape[1] != h or src.dtype != out.dtype or rows.numel() != r:
            raise KernelError("gather_rows: shapes or dtypes do not match")
        fn = _fn("elementwise", "iian_gather_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(src, "gather src"), _cuda(rows, "rows", torch.int32), _cuda(out, "gather out"),
                  _code(src, "gather src"), r, h, src.shape[0], _stream()), "gather_rows")

    def add_bias(self, x: torch.Tensor, bias: torch.Tensor) -> None:
        n, m = x.shape
        if bias.numel() != m:
            raise KernelError("add_bias: bias length does not match")
        fn = _fn("elementwise", "iian_add_bias", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(x, "add_bias x"), _cuda(bias, "bias", torch.float32), _code(x, "add_bias x"), n, m, _stream()),
               "add_bias")

    # ---- matrix products -----------------------------------------------------------------
    def linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, row_scale=None, residual_norm=None) -> None:
        """out[n, m] = sum_k x[n, k] * w[m, k].  ``row_scale`` (ops.fused.RowScale) and ``residual_norm``
        (ops.fused.ResidualNorm) ask for the fused forms; ``can_fuse_norm`` says whether they are available."""
        n, k = x.shape
        m = w.shape[0]
        if w.shape[1] != k or out.shape != (n, m):
            raise KernelError(f"linear: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
        if n == 0:
            return
        if row_scale is not None or residual_norm is not None:
            if self._tcgen05_ok(x, w, n, k):
                self.gemm_tcgen05(x, w, out, row_scale=row_scale, residual_norm=residual_norm)
            else:
                self.gemm_skinny_fused(x, w, out, 2 if residual_norm is not None else 0, row_scale, residual_norm)
            return
        self._linear_dispatch(x, w, out, n, m, k)

    FUSE_NORM = os.environ.get("IIAN_FUSE_NORM", "1") not in ("0", "false", "off")

    def can_fuse_norm(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        """Whether the product of ``x`` with ``w`` can carry a RowScale or a ResidualNorm (the weight-streaming
        kernel's range: up to 8 rows of bfloat16)."""
        n, k = x.shape
        return self.FUSE_NORM and (self._skinny_ok(x, w, n, k) or self._tcgen05_ok(x, w, n, k))

    def can_take_prenormed(self, n_rows: int, w: torch.Tensor, dtype: torch.dtype) -> bool:
        """Whether a product of ``n_rows`` rows with ``w`` can carry a RowScale: the row counts of the weight-streaming
        kernel and of the tcgen05 kernel (the library product between them cannot)."""
        if not self.FUSE_NORM or dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.data_ptr() % 16:
            return False
        k = w.shape[1]
        if n_rows <= self.SKINNY_MAX_ROWS:
            return k % 32 == 0
        return self._tcgen05_rows_ok(n_rows, w.shape[0]) and k % 8 == 0 and not self.LIBRARY_GEMM_ONLY

    def norm_parts(self, w: torch.Tensor, n_rows: int = 1) -> int:
        """Parts in which a ResidualNorm product of ``n_rows`` rows with weight ``w`` leaves the sums of squares."""
        if n_rows > self.SKINNY_MAX_ROWS:
            return -(-w.shape[0] // self.tcgen05_tile_columns(n_rows, w.shape[0]))
        return -(-w.shape[0] // 16)

    def gemm_skinny_fused(self, x, w, out, epilogue: int, row_scale=None, residual_norm=None) -> None:
        n, k = x.shape
        m = w.shape[0]
        if not self._skinny_ok(x, w, n, k):
            raise KernelError("linear: the fused forms need up to 8 rows of bfloat16, K a multiple of 32")
        in_p = in_tiles = 0
        inv_w = eps = 0.0
        if row_scale is not None:
            if row_scale.partials.dtype != torch.float32 or row_scale.partials.shape[0] != n:
                raise KernelError("linear: RowScale partials must be float32 [rows, parts]")
            in_p, in_tiles = _cuda(row_scale.partials, "row-scale partials"), row_scale.partials.shape[1]
            inv_w, eps = 1.0 / row_scale.width, row_scale.eps
        res = nw = out_p = 0
        if residual_norm is not None:
            rn = residual_norm
            if (rn.residual.shape != (n, m) or rn.residual.dtype != torch.float32 or rn.weight.numel() != m
                    or rn.partials.shape != (n, self.norm_parts(w)) or out.dtype != torch.bfloat16):
                raise KernelError("linear: ResidualNorm operands do not fit the product")
            res, nw = _cuda(rn.residual, "residual", torch.float32), _cuda(rn.weight, "norm weight", torch.float32)
            out_p = _cuda(rn.partials, "norm partials", torch.float32)
        if self.prefetcher is not None:
            self.prefetcher.before_product(self)
        if self.STREAM_PRODUCT:
            self._gemm_stream(x, w, out, n, m, k, epilogue, in_p, in_tiles, inv_w, eps, res, nw, out_p)
        else:
            fn = _fn("gemm_skinny", "iian_gemm_skinny_fused",
                     [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_float,
                      c_void_p, c_void_p, c_void_p, c_void_p])
            _check(fn(_cuda(x, "linear x"), _cuda(w, "linear w"), _cuda(out, "linear out"), _code(out, "linear out"), n, m, k,
                      epilogue, in_p, in_tiles, inv_w, eps, res, nw, out_p, _stream()), "gemm_skinny_fused")
        if self.weight_log is not None:
            self.weight_log.append((w.data_ptr(), w.numel() * w.element_size()))
        if self.prefetcher is not None:
            self.prefetcher.after_product(self)

    # Up to 8 rows: the product whose weights stream through a ring of shared-memory stages filled by bulk asynchronous
    # copies (csrc/gemm_stream.cu) instead of the one that loads them into registers (csrc/gemm_skinny.cu); the results
    # are the same bits.  IIAN_STREAM_PRODUCT=0 goes back to the register form.
    STREAM_PRODUCT = os.environ.get("IIAN_STREAM_PRODUCT", "1") not in ("0", "false", "off")
    STREAM_STAGES = int(os.environ.get("IIAN_STREAM_STAGES", "12"))
    _stream_stages_set = None

    def _gemm_stream(self, x, w, out, n, m, k, epilogue, in_p=0, in_tiles=0, inv_w=0.0, eps=0.0, res=0, nw=0, out_p=0) -> None:
        if self._stream_stages_set != self.STREAM_STAGES:
            fn = _fn("gemm_stream", "iian_gemm_stream_stages", [c_int])
            if fn(self.STREAM_STAGES) != 0:
                raise KernelError("gemm_stream: the ring has 6 or 12 stages")
            type(self)._stream_stages_set = self.STREAM_STAGES
        status = self.tcgen05_status_buffer(x.device).data_ptr()
        CudaKernels._tc_used = True
        fn = _fn("gemm_stream", "iian_gemm_stream",
                 [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_float, c_float,
                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
        _check(fn(_cuda(x, "linear x"), _cuda(w, "linear w"), _cuda(out, "linear out"), _code(out, "linear out"), n, m, k,
                  epilogue, in_p, in_tiles, inv_w, eps, res, nw, out_p, status, _stream()), "gemm_stream")

    # rows up to which the weight-streaming kernel is used; above it the library GEMM takes over
    # (measured on B200 at the Qwen3-8B sizes: the streaming kernel wins up to 8 rows, cuBLAS from 16)
    SKINNY_MAX_ROWS = 8

    # Weight prefetch for captured decode graphs (see csrc/prefetch.cu and WeightPrefetcher below)
    weight_log = None          # a list while the order of weight-streaming products is being recorded
    prefetcher = None          # a WeightPrefetcher while a decode graph is being captured

    # rows from which the tcgen05 kernel takes over (below it, and above the streaming kernel's range, the
    # library GEMM is faster: one row tile of 128 leaves most SMs without work)
    TCGEN05_MIN_ROWS = 128
    LIBRARY_GEMM_ONLY = os.environ.get("IIAN_LIBRARY_GEMM", "0") not in ("0", "false", "off")

    # ... and only when the product has many tiles of 256 x 256 (several waves of the 74 pairs of SMs): with few tiles
    # the SMs that work cannot stream the weights fast enough, and with one or two waves the idle tail of the last
    # wave costs more than the fused epilogue saves; the library product (which splits K, and uses TMA multicast in
    # clusters of four) is faster there.  Measured on B200 at the Qwen3-8B sizes, whole prefill steps in ms with the
    # threshold at 0 / 64 / 130 / 400 / all library: 256 tokens 9.4 / 6.5 / - / - / -; 1024 tokens 15.2 / 15.2 / 13.9 /
    # 14.4 / 14.3; 2048 tokens 27.1 / 27.1 / 26.2 / 25.9 / 27.6; 4096 tokens - / - / 54.4 / 52.5 / 52.9.  At 300 the own
    # kernel takes the gate/up product with its SwiGLU epilogue from 1024 rows on (384 tiles) and nothing else of a layer.
    TCGEN05_MIN_TILES = int(os.environ.get("IIAN_TCGEN05_MIN_TILES", "300"))

    def _tcgen05_rows_ok(self, n: int, m: int) -> bool:
        return n >= self.TCGEN05_MIN_ROWS and (-(-n // 256)) * (-(-m // 256)) >= self.TCGEN05_MIN_TILES

    def _tcgen05_ok(self, x, w, n, k) -> bool:
        return (not self.LIBRARY_GEMM_ONLY and self._tcgen05_rows_ok(n, w.shape[0]) and k % 8 == 0
                and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def _skinny_ok(self, x, w, n, k) -> bool:
        return (n <= self.SKINNY_MAX_ROWS and k % 32 == 0 and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)

    def can_fuse_swiglu(self, x: torch.Tensor, w: torch.Tensor, interleave: int) -> bool:
        """Whether ``linear_swiglu`` can run for these operands (else: linear, then swiglu)."""
        n, k = x.shape
        return interleave == 8 and w.shape[0] % 16 == 0 and (self._tcgen05_ok(x, w, n, k) or self._skinny_ok(x, w, n, k))

    def linear_swiglu(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, row_scale=None) -> None:
        """out[t, f] = silu(x . w_gate_f) * (x . w_up_f) for w with gate and up rows interleaved in groups of 8."""
        n, k = x.shape
        if row_scale is not None:
            if self._tcgen05_ok(x, w, n, k):
                self.gemm_tcgen05(x, w, out, epilogue=1, row_scale=row_scale)
            else:
                self.gemm_skinny_fused(x, w, out, 1, row_scale, None)
            return
        if self._tcgen05_ok(x, w, n, k):
            self.gemm_tcgen05(x, w, out, epilogue=1)
            return
        if self.prefetcher is not None:
            self.prefetcher.before_product(self)
        if self.STREAM_PRODUCT:
            self._gemm_stream(x, w, out, n, w.shape[0], k, 1)
        else:
            self.gemm_skinny(x, w, out, epilogue=1)
        if self.weight_log is not None:
            self.weight_log.append((w.data_ptr(), w.numel() * w.element_size()))
        if self.prefetcher is not None:
            self.prefetcher.after_product(self)

    def _linear_dispatch(self, x, w, out, n, m, k) -> None:
        if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
            if self._tcgen05_ok(x, w, n, k):
                self.gemm_tcgen05(x, w, out)
                return
            if n <= self.SKINNY_MAX_ROWS and k % 32 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
                if self.prefetcher is not None:
                    self.prefetcher.before_product(self)
                if self.STREAM_PRODUCT:
                    self._gemm_stream(x, w, out, n, m, k, 0)
                else:
                    self.gemm_skinny(x, w, out)
                if self.weight_log is not None:
                    self.weight_log.append((w.data_ptr(), w.numel() * w.element_size()))
                if self.prefetcher is not None:
                    self.prefetcher.after_product(self)
                return
            if n > self.SKINNY_MAX_ROWS and self._library_gemm(x, w, out):
                return
        self.gemm_simt(x, w, out)

    _library_f32_out = True

    def _library_gemm(self, x, w, out) -> bool:
        """cuBLAS through torch.mm, for large bfloat16 products (as the reference does for large batches)."""
        if out.dtype == torch.bfloat16:
            torch.mm(x, w.t(), out=out)
            LAUNCHES_BY_ENTRY["library_gemm"] = LAUNCHES_BY_ENTRY.get("library_gemm", 0) + 1
            return True
        if out.dtype == torch.float32 and self._library_f32_out:
            try:
                torch.mm(x, w.t(), out_dtype=torch.float32, out=out)
                LAUNCHES_BY_ENTRY["library_gemm"] = LAUNCHES_BY_ENTRY.get("library_gemm", 0) + 1
                return True
            except (TypeError, RuntimeError):
                type(self)._library_f32_out = False
        return False

    def skinny_ksplit(self, n: int, m: int, k: int) -> int:
        """Into how many CTAs K is cut: matrices with few rows would otherwise leave most of the GPU's
        memory pipeline idle (a row block of 16 is one CTA)."""
        return 1       # measured on B200 at the Qwen3-8B sizes: one CTA per row block is fastest for every shape

    def gemm_skinny(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, cfg: int = 0, ksplit: int = 0,
                    epilogue: int = 0) -> None:
        """``cfg`` picks a tile configuration (rows-per-block tiles * 100 + warps * 10 + unroll); ``ksplit``
        the number of CTAs that share K for one row block; 0: defaults."""
        n, k = x.shape
        m = w.shape[0]
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            raise KernelError("gemm_skinny: x and w must be bfloat16")
        if ksplit <= 0:
            ksplit = 1 if epilogue else self.skinny_ksplit(n, m, k)
        part = counters = 0
        if ksplit > 1:
            rows = 32 if n > 8 else 16
            blocks = -(-m // rows)
            nt = 1 if n <= 8 else 2 if n <= 16 else 4 if n <= 32 else 8
            part = self.gemm_scratch(x.device, blocks * ksplit * rows * 8 * nt).data_ptr()
            counters = self.gemm_counters(x.device, blocks).data_ptr()
        fn = _fn("gemm_skinny", "iian_gemm_skinny_cfg",
                 [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p])
        _check(fn(_cuda(x, "linear x"), _cuda(w, "linear w"), _cuda(out, "linear out"), _code(out, "linear out"),
                  n, m, k, cfg, ksplit, part, counters, epilogue, _stream()), "gemm_skinny")

    _gemm_scratch = {}
    _gemm_counters = {}

    def gemm_scratch(self, device, n_floats: int) -> torch.Tensor:
        t = self._gemm_scratch.get(device)
        if t is None or t.numel() < n_floats:
            t = torch.empty(max(n_floats, 1 << 20), dtype=torch.float32, device=device)
            self._gemm_scratch[device] = t
            self._scratch_keep.append(t)
        return t

    def gemm_counters(self, device, n: int) -> torch.Tensor:
        t = self._gemm_counters.get(device)
        if t is None or t.numel() < n:
            t = torch.zeros(max(n, 1 << 14), dtype=torch.int32, device=device)
            self._gemm_counters[device] = t
            self._scratch_keep.append(t)
        return t

    def gemm_simt(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
        n, k = x.shape
        m = w.shape[0]
        fn = _fn("gemm_simt", "iian_gemm_simt",
                 [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
        _check(fn(_cuda(x, "linear x"), _code(x, "linear x"), _cuda(w, "linear w"), _code(w, "linear w"),
                  _cuda(out, "linear out"), _code(out, "linear out"), n, m, k, _stream()), "gemm_simt")

    # ---- tcgen05 + TMA product for many rows ----------------------------------------------------
    _tc_status = {}

    def tcgen05_status_buffer(self, device) -> torch.Tensor:
        t = self._tc_status.get(device)
        if t is None:
            t = torch.zeros(2, dtype=torch.int32, device=device)
            self._tc_status[device] = t
        return t

    _tc_used = False           # a tcgen05 kernel was launched since the status was last read

    def check_device_status(self) -> None:
        """Called where the host has just waited for the device anyway (tokens or logits were read): if a tcgen05
        kernel ran since the last call, read its status words and raise if one gave up on a barrier."""
        if not CudaKernels._tc_used:
            return
        for device in list(self._tc_status):
            self.tcgen05_check(device)

    def tcgen05_check(self, device) -> None:
        """Synchronise and raise if a tcgen05 kernel gave up waiting (its output would be garbage)."""
        CudaKernels._tc_used = False
        t = self._tc_status.get(device)
        if t is None:
            return
        code, where = t.tolist()
        if code != 0:
            t.zero_()
            raise KernelError(f"a kernel gave up waiting on a barrier (wait {code}, iteration {where}); its result is not valid")

    TCGEN05_PAIR = os.environ.get("IIAN_TCGEN05_PAIR", "1") not in ("0", "false", "off")

    @classmethod
    def tcgen05_tile(cls, n_rows: int, n: int) -> int:
        """The tile of the tcgen05 product for ``n_rows`` rows and a weight with ``n`` rows: 128 or 256 columns on one
        SM, or 512: tiles of 256 x 256 on pairs of SMs (from two row tiles on)."""
        wide = n % 256 == 0 or n > 4096
        if wide and cls.TCGEN05_PAIR and n_rows > 128:
            return 512
        return 256 if wide else 128

    @classmethod
    def tcgen05_tile_columns(cls, n_rows: int, n: int) -> int:
        return min(256, cls.tcgen05_tile(n_rows, n))

    def gemm_tcgen05(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = 0, bn: int = 0,
                     row_scale=None, residual_norm=None) -> None:
        """``epilogue`` 0: out[t, n] = x . w; 1: w holds gate and up rows interleaved in groups of 8 and
        out[t, f] = silu(gate_f) * up_f with half as many columns; 2 (with ``residual_norm``): the residual add and
        the next norm's weight ride in the epilogue.  ``row_scale``: rows are multiplied by a folded norm's factor."""
        t_rows, k = x.shape
        n = w.shape[0]
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            raise KernelError("gemm_tcgen05: x and w must be bfloat16")
        want_cols = n // 2 if epilogue == 1 else n
        if w.shape[1] != k or out.shape != (t_rows, want_cols):
            raise KernelError(f"gemm_tcgen05: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not fit")
        if bn == 0:
            bn = self.tcgen05_tile(t_rows, n)
        status = self.tcgen05_status_buffer(x.device).data_ptr()
        CudaKernels._tc_used = True
        if row_scale is None and residual_norm is None:
            fn = _fn("gemm_tcgen05", "iian_gemm_tcgen05",
                     [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p])
            _check(fn(_cuda(x, "linear x"), _cuda(w, "linear w"), _cuda(out, "linear out"), _code(out, "linear out"),
                      t_rows, n, k, epilogue, bn, status, _stream()), "gemm_tcgen05")
            return
        in_p = in_tiles = 0
        inv_w = eps = 0.0
        if row_scale is not None:
            if row_scale.partials.dtype != torch.float32 or row_scale.partials.shape[0] != t_rows:
                raise KernelError("linear: RowScale partials must be float32 [rows, parts]")
            in_p, in_tiles = _cuda(row_scale.partials, "row-scale partials"), row_scale.partials.shape[1]
            inv_w, eps = 1.0 / row_scale.width, row_scale.eps
        res = nw = out_p = 0
        if residual_norm is not None:
            rn = residual_norm
            if (rn.residual.shape != (t_rows, n) or rn.residual.dtype != torch.float32 or rn.weight.numel() != n
                    or rn.partials.shape != (t_rows, -(-n // min(bn, 256))) or out.dtype != torch.bfloat16):
                raise KernelError("linear: ResidualNorm operands do not fit the product")
            res, nw = _cuda(rn.residual, "residual", torch.float32), _cuda(rn.weight, "norm weight", torch.float32)
            out_p = _cuda(rn.partials, "norm partials", torch.float32)
            epilogue = 2
        fn = _fn("gemm_tcgen05", "iian_gemm_tcgen05_fused",
                 [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                  c_void_p, c_int, c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p])
        _check(fn(_cuda(x, "linear x"), _cuda(w, "linear w"), _cuda(out, "linear out"), _code(out, "linear out"),
                  t_rows, n, k, epilogue, bn, status, in_p, in_tiles, inv_w, eps, res, nw, out_p, _stream()), "gemm_tcgen05")

    def prefetch_l2(self, ptr: int, nbytes: int, stream: Optional[int] = None) -> None:
        fn = _fn("prefetch", "iian_prefetch_l2", [c_void_p, c_longlong, c_void_p])
        _check(fn(ptr, nbytes, _stream() if stream is None else stream), "prefetch_l2")

    # ---- attention -----------------------------------------------------------------------
    def qk_norm_rope_store(self, qkv: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                           v_cache: Optional[torch.Tensor], *, num_heads: int, num_kv_heads: int, head_dim: int,
                           q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                           inv_freq: Optional[torch.Tensor], rot_dim: int, rope_style: int,
                           positions: torch.Tensor, slots: Optional[torch.Tensor], write_kv: bool,
                           bias: Optional[torch.Tensor] = None, table: Optional[torch.Tensor] = None) -> None:
        n = qkv.shape[0]
        width = (num_heads + 2 * num_kv_heads) * head_dim
        if qkv.shape[1] != width or q_out.numel() != n * num_heads * head_dim or q_out.dtype != qkv.dtype:
            raise KernelError(f"qk_norm_rope_store: qkv {tuple(qkv.shape)} does not match {num_heads}+2*{num_kv_heads} "
                              f"heads of {head_dim}")
        page_size = num_pages = 0
        if write_kv:
            if k_cache is None or v_cache is None or slots is None:
                raise KernelError("qk_norm_rope_store: a cache and slots are needed to store K and V")
            if k_cache.dtype != qkv.dtype or k_cache.shape != v_cache.shape or k_cache.shape[1] != num_kv_heads \
                    or k_cache.shape[3] != head_dim:
                raise KernelError(f"qk_norm_rope_store: cache {tuple(k_cache.shape)} {k_cache.dtype} does not match")
            num_pages, page_size = k_cache.shape[0], k_cache.shape[2]
        if inv_freq is not None and inv_freq.numel() < rot_dim // 2:
            raise KernelError("qk_norm_rope_store: inv_freq is shorter than rot_dim / 2")
        fn = _fn("rope_kv", "iian_qk_norm_rope_store",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p])
        if table is not None and (inv_freq is None or table.numel() < 2 * n * (rot_dim // 2)):
            raise KernelError("qk_norm_rope_store: the rotary table does not cover these tokens")
        _check(fn(_cuda(qkv, "qkv"), _cuda(bias, "qkv bias", torch.float32), _cuda(q_out, "q out"),
                  _cuda(k_cache, "k cache"), _cuda(v_cache, "v cache"),
                  _cuda(q_weight, "q norm weight", torch.float32), _cuda(k_weight, "k norm weight", torch.float32),
                  _cuda(inv_freq, "inv_freq", torch.float32), _cuda(table, "rotary table", torch.float32),
                  _cuda(positions, "positions", torch.int32),
                  _cuda(slots, "slots", torch.int32), _code(qkv, "qkv"), n, num_heads, num_kv_heads, head_dim,
                  rot_dim if inv_freq is not None else 0, rope_style, eps, page_size, num_pages, 1 if write_kv else 0,
                  _stream()), "qk_norm_rope_store")

    def rotary_table(self, inv_freq: torch.Tensor, positions: torch.Tensor, half: int, out: torch.Tensor) -> None:
        """out[t, p] = (cos, sin)(positions[t] * inv_freq[p]), float32 [N, half, 2]."""
        n = positions.shape[0]
        if out.numel() < 2 * n * half or inv_freq.numel() < half:
            raise KernelError("rotary_table: output or inv_freq too small")
        fn = _fn("rope_kv", "iian_rotary_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
        _check(fn(_cuda(inv_freq, "inv_freq", torch.float32), _cuda(positions, "positions", torch.int32),
                  _cuda(out, "rotary table", torch.float32), n, half, _stream()), "rotary_table")

    def paged_attention(self, q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                        meta, *, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                        window: Optional[int], n_split: Optional[int] = None) -> None:
        """``meta``: an object with ``positions``, ``seq_of_token``, ``block_table`` [S, max_blocks],
        ``ctx_len`` [S] (int32 CUDA tensors) and host-side hints (``num_seqs``, ``max_q_len``, ``max_ctx``,
        ``decode_only``).  ``n_split``: a fixed number of key splits for the decode form (a captured graph's); None:
        chosen per launch."""
        self._attention_dispatch(q, k_cache, v_cache, out, meta, num_heads, num_kv_heads, head_dim, scale, window, n_split)

    # prefill portions on tcgen05 (csrc/attention_tc.cu); IIAN_ATTENTION_TC=0 keeps them on the mma.sync kernel
    ATTENTION_TC = os.environ.get("IIAN_ATTENTION_TC", "1") not in ("0", "false", "off")
    TC_ATTENTION_MIN_ROWS = 64        # rows (tokens x heads per KV head) of the longest portion from which it is used

    def _attention_tc_ok(self, q, k_cache, meta, nh, nkv, hd) -> bool:
        return (self.ATTENTION_TC and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and hd == 128
                and k_cache.shape[2] in (8, 16, 32, 64, 128) and nkv > 0 and nh % nkv == 0
                and meta.max_q_len * (nh // nkv) >= self.TC_ATTENTION_MIN_ROWS)

    def paged_attention_tc(self, q, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, head_dim, scale, window) -> None:
        """Prefill attention on tcgen05 + TMA: head size 128, bfloat16, pages of 8 to 128 tokens."""
        n = q.shape[0]
        if k_cache.dtype != torch.bfloat16 or q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            raise KernelError("paged_attention_tc: bfloat16 only")
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim or q.numel() != n * num_heads * head_dim:
            raise KernelError("paged_attention_tc: cache / q shapes do not match the head counts")
        status = self.tcgen05_status_buffer(q.device)
        CudaKernels._tc_used = True
        bt = meta.block_table
        fn = _fn("attention_tc", "iian_attention_tc",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_void_p])
        _check(fn(_cuda(q, "q"), _cuda(k_cache, "k cache"), _cuda(v_cache, "v cache"), _cuda(out, "attention out"),
                  _cuda(meta.cu_q, "cu_q", torch.int32), _cuda(meta.ctx_len, "ctx_len", torch.int32),
                  _cuda(bt, "block table", torch.int32), bt.shape[1], n, meta.num_seqs, meta.max_q_len, num_heads,
                  num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0], scale, window or 0,
                  status.data_ptr(), _stream()), "attention_tc")

    def _attention_dispatch(self, q, k_cache, v_cache, out, meta, nh, nkv, hd, scale, window, n_split=None) -> None:
        if self._attention_tc_ok(q, k_cache, meta, nh, nkv, hd):
            self.paged_attention_tc(q, k_cache, v_cache, out, meta, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                                    scale=scale, window=window)
            return
        if q.dtype == torch.bfloat16 and hd in (64, 128):
            self.paged_attention_mma(q, k_cache, v_cache, out, meta, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                                     scale=scale, window=window, n_split=n_split)
        else:
            self.paged_attention_generic(q, k_cache, v_cache, out, meta, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                                         scale=scale, window=window)

    DECODE_STAGES = int(os.environ.get("IIAN_DECODE_STAGES", "2"))     # shared-memory tiles per CTA of the decode kernel
    _sm_count = {}

    @classmethod
    def sm_count(cls, device=None) -> int:
        """Streaming multiprocessors of ``device`` (the current one by default), asked from the driver once."""
        idx = torch.cuda.current_device() if device is None else torch.device(device).index
        if idx is None:
            idx = torch.cuda.current_device()
        n = cls._sm_count.get(idx)
        if n is None:
            n = cls._sm_count[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
        return n

    @property
    def DECODE_SLOTS(self) -> int:
        """CTAs of the decode kernel with split keys one launch should not exceed: 2.7 per SM (three fit; clusters
        need their CTAs inside one GPC, which leaves some places empty)."""
        return self.DECODE_CTAS_PER_SM_X10 * self.sm_count() // 10

    DECODE_CTAS_PER_SM_X10 = int(round(10 * float(os.environ.get("IIAN_DECODE_CTAS_PER_SM", "2.7"))))
    _stages_set = None

    @staticmethod
    def apply_unsplit_stages() -> None:
        """IIAN_DECODE_UNSPLIT_STAGES=2|3 fixes the tiles per CTA of decode attention with unsplit keys (a measurement
        switch; by default the kernel library chooses by the number of waves of CTAs each form needs)."""
        v = os.environ.get("IIAN_DECODE_UNSPLIT_STAGES")
        if v:
            if _fn("attention_mma", "iian_attention_unsplit_stages", [c_int])(int(v)) != 0:
                raise KernelError("IIAN_DECODE_UNSPLIT_STAGES takes 2 or 3")

    def set_decode_stages(self, stages: int) -> None:
        """2: three CTAs per SM with one tile in flight each; 3: two CTAs with two tiles in flight."""
        fn = _fn("attention_mma", "iian_attention_decode_stages", [c_int])
        code = fn(stages)
        if code != 0:
            raise KernelError("attention: the decode kernel has 2 or 3 stages")
        type(self)._stages_set = stages
        type(self).DECODE_STAGES = stages
        self.apply_unsplit_stages()
    CLUSTER_MERGE = os.environ.get("IIAN_ATTENTION_CLUSTER", "1") not in ("0", "false", "off")
    MAX_SPLITS = int(os.environ.get("IIAN_DECODE_MAX_SPLITS", "32"))
    _scratch = {}
    _scratch_keep = []

    def attention_splits(self, num_seqs: int, num_kv_heads: int, max_ctx: int) -> int:
        """How many parts the keys of a decode step are cut into, so that few long sequences still fill
        the GPU.  Measured on B200 (replayed graphs, 8 KV heads of 128, contexts of 1k to 8k, batches 1 to
        128): all CTAs of a launch should be resident at once (a second wave repeats the whole chain of dependent
        loads: 24.6 us with 8 parts against 14.7 us with 4 at batch 8), which with split keys means up to 2.7 per SM
        (35.0 us with 2 parts against 51.8 us unsplit at batch 20, 21.9 against 30.7 us with 4 against 2 at batch 10;
        but 65 against 53 us at batch 28, where two parts no longer fit), and a CTA should keep at least two key
        tiles.  The parts of a sequence are a power of two and merge inside a thread-block cluster, up to 16 of them
        (more than 8 is a size a kernel has to ask for, and only some 24 such clusters fit the GPU: 13.6 us with 8
        against 22.7 us with 16 parts at batch 3), which saves three trips through L2 (write the parts, count
        arrivals, read them back: one launch at batch 1 and 8k context takes 27.9 us with 8 parts, 18.6 us with 16 in
        a cluster, 25.9 us with 16 and 30.8 us with 32 merged through scratch memory); 32 parts through scratch
        memory are only taken for a single sequence from 32k of context on (48.8 against 52.9 us)."""
        tiles = max(1, (max_ctx + 63) // 64)
        base = max(1, num_seqs * num_kv_heads)
        if os.environ.get("IIAN_DECODE_FORCE_SPLITS"):
            return int(os.environ["IIAN_DECODE_FORCE_SPLITS"])
        n = max(1, min(self.DECODE_SLOTS // base, -(-tiles // 2), self.MAX_SPLITS))
        if n >= 32 and tiles >= 512:
            return n
        if n >= 16:
            return 16 if base * 16 <= 2 * self.sm_count() else 8
        return 8 if n >= 8 else 4 if n >= 4 else 2 if n >= 2 else 1

    def attention_scratch(self, device, n_floats: int) -> torch.Tensor:
        t = self._scratch.get(device)
        if t is None or t.numel() < n_floats:
            t = torch.empty(max(n_floats, 1 << 20), dtype=torch.float32, device=device)
            self._scratch[device] = t
            self._scratch_keep.append(t)        # a captured graph may still point at an older, smaller buffer
        return t

    _counters = {}

    def attention_counters(self, device, n: int) -> torch.Tensor:
        """Zeroed int32 counters for the decode kernel's in-kernel merge (it puts them back to zero)."""
        t = self._counters.get(device)
        if t is None or t.numel() < n:
            t = torch.zeros(max(n, 1 << 16), dtype=torch.int32, device=device)
            self._counters[device] = t
            self._scratch_keep.append(t)
        return t

    def paged_attention_mma(self, q, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, head_dim, scale, window,
                            n_split: Optional[int] = None, small_tiles: Optional[bool] = None,
                            cluster: Optional[bool] = None) -> None:
        """``small_tiles``: the decode form (rows of one token, keys split over the warps); ``cluster``: its
        parts merge through the shared memory of a thread-block cluster (2, 4 or 8 parts) instead of scratch
        memory.  None: chosen from the step."""
        n = q.shape[0]
        if k_cache.dtype != torch.bfloat16 or q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            raise KernelError("paged_attention_mma: bfloat16 only")
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim or q.numel() != n * num_heads * head_dim:
            raise KernelError("paged_attention_mma: cache / q shapes do not match the head counts")
        if self._stages_set != self.DECODE_STAGES:
            self.set_decode_stages(self.DECODE_STAGES)
        decode = meta.max_q_len * (num_heads // num_kv_heads) <= 16
        if small_tiles is None:
            small_tiles = decode
        if n_split is None:
            n_split = self.attention_splits(meta.num_seqs, num_kv_heads, meta.max_ctx) if decode else 1
        if cluster is None:
            cluster = self.CLUSTER_MERGE
        cluster = bool(cluster and small_tiles and n_split in (2, 4, 8, 16))
        part_o = part_lse = counters = 0
        if n_split > 1 and not cluster:
            rows = n * num_heads
            scratch = self.attention_scratch(q.device, rows * n_split * (head_dim + 1))
            part_o = scratch.data_ptr()
            part_lse = part_o + rows * n_split * head_dim * 4
            if small_tiles:
                row_tiles = -(-meta.max_q_len * (num_heads // num_kv_heads) // 16)
                counters = self.attention_counters(q.device, meta.num_seqs * num_kv_heads * row_tiles).data_ptr()
        bt = meta.block_table
        fn = _fn("attention_mma", "iian_attention_mma",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p])
        _check(fn(_cuda(q, "q"), _cuda(k_cache, "k cache"), _cuda(v_cache, "v cache"), _cuda(out, "attention out"),
                  part_o, part_lse, counters, _cuda(meta.cu_q, "cu_q", torch.int32), _cuda(meta.ctx_len, "ctx_len", torch.int32),
                  _cuda(bt, "block table", torch.int32), bt.shape[1], n, meta.num_seqs, meta.max_q_len, num_heads,
                  num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0], scale, window or 0, n_split,
                  (2 if cluster else 1) if small_tiles else 0, self._decode_status(q.device) if small_tiles else None,
                  _stream()), "attention_mma")
        if n_split > 1 and not small_tiles:
            LAUNCHES[0] += 1

    FUSED_DECODE = os.environ.get("IIAN_FUSED_DECODE_ATTENTION", "1") not in ("0", "false", "off")
    # decode attention fetches its K/V tiles by TMA (head size 128, pages of 8 to 64 tokens); IIAN_DECODE_TMA=0: cp.async
    DECODE_TMA = os.environ.get("IIAN_DECODE_TMA", "1") not in ("0", "false", "off")

    # native step function, mixed steps: the decoded tokens' attention runs on the decode kernel on a second stream
    # beside the prefill kernel; IIAN_SPLIT_MIXED=0: one launch of the prefill kernel for all sequences of the step
    SPLIT_MIXED = os.environ.get("IIAN_SPLIT_MIXED", "1") not in ("0", "false", "off")

    def _decode_status(self, device):
        """The status words the decode kernel's TMA form reports to (the ones of the tcgen05 kernels), or None: the
        cp.async form."""
        if not self.DECODE_TMA:
            return None
        CudaKernels._tc_used = True
        return self.tcgen05_status_buffer(device).data_ptr()

    def can_fuse_decode_attention(self, qkv, meta, *, num_heads, num_kv_heads, head_dim, rot_dim, rope_style, bias) -> bool:
        """Whether ``attention_decode_fused`` covers this step: one token per sequence, bfloat16, heads of 64 or
        128, NEOX rotation over the whole head (or none), no projection bias, at most 16 heads per KV head."""
        return (self.FUSED_DECODE and meta.decode_only and meta.num_tokens == meta.num_seqs and qkv.dtype == torch.bfloat16
                and head_dim in (64, 128) and bias is None and rot_dim in (0, head_dim) and (rope_style == 0 or rot_dim == 0)
                and num_kv_heads > 0 and num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16)

    def attention_decode_fused(self, qkv, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, head_dim, scale, window,
                               q_weight, k_weight, eps, table, slots, write_kv: bool,
                               n_split: Optional[int] = None, cluster: Optional[bool] = None) -> None:
        """Per-head RMSNorm, rotation, the write of the new K and V to the cache and attention over the cache in
        one launch, from the Q|K|V projection ``qkv`` [S, (nh + 2 nkv) * hd] of a step with one token per sequence.
        Without ``write_kv`` the projection holds Q only ([S, nh * hd] is not accepted: pass the full width)."""
        s_ = meta.num_seqs
        width = (num_heads + 2 * num_kv_heads) * head_dim
        if qkv.shape != (s_, width) or out.shape != (s_, num_heads * head_dim):
            raise KernelError(f"attention_decode_fused: qkv {tuple(qkv.shape)} / out {tuple(out.shape)} do not fit {s_} sequences")
        if qkv.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
            raise KernelError("attention_decode_fused: bfloat16 only")
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim:
            raise KernelError("attention_decode_fused: cache shape does not match the head counts")
        if table is not None and (table.dtype != torch.float32 or table.numel() != s_ * head_dim):
            raise KernelError("attention_decode_fused: the rotation table must be float32 [S, hd / 2, 2]")
        if self._stages_set != self.DECODE_STAGES:
            self.set_decode_stages(self.DECODE_STAGES)
        if n_split is None:
            n_split = self.attention_splits(s_, num_kv_heads, meta.max_ctx)
        if cluster is None:
            cluster = self.CLUSTER_MERGE
        cluster = bool(cluster and 2 <= n_split <= 16)
        part_o = part_lse = counters = 0
        if n_split > 1 and not cluster:
            rows = s_ * num_heads
            scratch = self.attention_scratch(qkv.device, rows * n_split * (head_dim + 1))
            part_o = scratch.data_ptr()
            part_lse = part_o + rows * n_split * head_dim * 4
            counters = self.attention_counters(qkv.device, s_ * num_kv_heads).data_ptr()
        bt = meta.block_table
        fn = _fn("attention_mma", "iian_attention_decode_fused",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int,
                  c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_void_p])
        _check(fn(_cuda(qkv, "qkv"), _cuda(k_cache, "k cache"), _cuda(v_cache, "v cache"), _cuda(out, "attention out"),
                  part_o, part_lse, counters, _cuda(meta.cu_q, "cu_q", torch.int32), _cuda(meta.ctx_len, "ctx_len", torch.int32),
                  _cuda(bt, "block table", torch.int32), bt.shape[1], s_, num_heads, num_kv_heads, head_dim,
                  k_cache.shape[2], k_cache.shape[0], scale, window or 0, n_split, 1 if cluster else 0,
                  _cuda(q_weight, "q norm weight", torch.float32), _cuda(k_weight, "k norm weight", torch.float32),
                  _cuda(table, "rotation table", torch.float32), _cuda(slots, "slots", torch.int32), eps,
                  1 if write_kv else 0, self._decode_status(qkv.device), _stream()), "attention_decode_fused")

    def paged_attention_generic(self, q, k_cache, v_cache, out, meta, *, num_heads, num_kv_heads, head_dim, scale,
                                window) -> None:
        n = q.shape[0]
        if k_cache.dtype != q.dtype or out.dtype != q.dtype or k_cache.shape != v_cache.shape:
            raise KernelError("paged_attention: q, caches and out must share one dtype and the caches one shape")
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim or q.numel() != n * num_heads * head_dim:
            raise KernelError(f"paged_attention: cache {tuple(k_cache.shape)} / q {tuple(q.shape)} do not match "
                              f"{num_heads}/{num_kv_heads} heads of {head_dim}")
        fn = _fn("attention_generic", "iian_paged_attention_generic",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                  c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
        bt = meta.block_table
        _check(fn(_cuda(q, "q"), _cuda(k_cache, "k cache"), _cuda(v_cache, "v cache"), _cuda(out, "attention out"),
                  _cuda(meta.positions, "positions", torch.int32), _cuda(meta.seq_of_token, "seq_of_token", torch.int32),
                  _cuda(bt, "block table", torch.int32), bt.shape[1], _cuda(meta.ctx_len, "ctx_len", torch.int32),
                  _code(q, "q"), n, num_heads, num_kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0],
                  scale, window or 0, _stream()), "paged_attention_generic")

    # ---- sampling ------------------------------------------------------------------------
    def argmax(self, logits: torch.Tensor, out: torch.Tensor) -> None:
        r, v = logits.shape
        if logits.stride(1) != 1:
            raise KernelError("argmax: logits rows must be contiguous")
        if not logits.is_cuda or logits.dtype != torch.float32:
            raise KernelError("argmax: logits must be float32 on CUDA")
        if v >= 16384 and r <= 65535:      # wide rows: many blocks per row, then a merge
            scratch = self.attention_scratch(logits.device, r * 64 * 2)
            fn = _fn("sampling", "iian_argmax_wide", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p])
            _check(fn(logits.data_ptr(), r, v, logits.stride(0), scratch.data_ptr(), _cuda(out, "argmax out", torch.int32),
                      _stream()), "argmax")
            LAUNCHES[0] += 1
            return
        fn = _fn("sampling", "iian_argmax", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p])
        _check(fn(logits.data_ptr(), r, v, logits.stride(0), _cuda(out, "argmax out", torch.int32), _stream()), "argmax")

    def logit_edits(self, logits: torch.Tensor, ints: torch.Tensor, floats: torch.Tensor, n_allow: int, n_edit: int) -> None:
        """Logits processors on ``logits`` [R, V] float32, in place.  ``ints`` (int32, on the device) holds, one after
        the other, allow_off [R + 1], edit_off [R + 1], allow_ids [n_allow], edit_tok [n_edit]; ``floats`` holds pre,
        mul_pos, mul_neg, post, [n_edit] each."""
        r, v = logits.shape
        if not logits.is_cuda or logits.dtype != torch.float32 or logits.stride(1) != 1:
            raise KernelError("logit_edits: logits must be float32 on CUDA with contiguous rows")
        if ints.numel() != 2 * (r + 1) + n_allow + n_edit or floats.numel() != 4 * n_edit:
            raise KernelError("logit_edits: the lists do not have the announced lengths")
        ip, fp = _cuda(ints, "edit lists", torch.int32), _cuda(floats, "edit values", torch.float32) if n_edit else 0
        allow_off, edit_off = ip, ip + 4 * (r + 1)
        allow_ids, edit_tok = ip + 8 * (r + 1), ip + 8 * (r + 1) + 4 * n_allow
        fn = _fn("sampling", "iian_logit_edits", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                                                  c_void_p, c_void_p, c_void_p, c_void_p, c_void_p])
        _check(fn(logits.data_ptr(), r, v, logits.stride(0), allow_off, allow_ids, edit_off, edit_tok,
                  fp, fp + 4 * n_edit, fp + 8 * n_edit, fp + 12 * n_edit, _stream()), "logit_edits")

    def logprobs(self, logits: torch.Tensor, tokens: torch.Tensor, want_k: torch.Tensor, kmax: int):
        """Raw log-probabilities of ``tokens`` [R] and of the ``want_k[r]`` most likely tokens of each row (negative:
        the row is skipped): ``(lp [R], top_ids [R, kmax], top_lp [R, kmax])`` on the device."""
        r, v = logits.shape
        if not logits.is_cuda or logits.dtype != torch.float32 or logits.stride(1) != 1:
            raise KernelError("logprobs: logits must be float32 on CUDA with contiguous rows")
        lp = torch.full((r,), float("-inf"), dtype=torch.float32, device=logits.device)
        ids = torch.full((r, max(kmax, 1)), -1, dtype=torch.int32, device=logits.device)
        lps = torch.full((r, max(kmax, 1)), float("-inf"), dtype=torch.float32, device=logits.device)
        fn = _fn("sampling", "iian_logprobs", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_int, c_void_p,
                                               c_void_p, c_void_p, c_void_p])
        _check(fn(logits.data_ptr(), r, v, logits.stride(0), _cuda(tokens, "tokens", torch.int32),
                  _cuda(want_k, "want_k", torch.int32), kmax, lp.data_ptr(), ids.data_ptr(), lps.data_ptr(), _stream()), "logprobs")
        return lp, ids, lps

    def sample(self, logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
               min_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> None:
        r, v = logits.shape
        if not logits.is_cuda or logits.dtype != torch.float32 or logits.stride(1) != 1:
            raise KernelError("sample: logits must be float32 on CUDA with contiguous rows")
        fn = _fn("sampling", "iian_sample", [c_void_p, c_int, c_int, c_longlong, c_void_p, c_void_p, c_void_p,
                                             c_void_p, c_void_p, c_void_p, c_void_p])
        _check(fn(logits.data_ptr(), r, v, logits.stride(0), _cuda(temperature, "temperature", torch.float32),
                  _cuda(top_k, "top_k", torch.int32), _cuda(top_p, "top_p", torch.float32),
                  _cuda(min_p, "min_p", torch.float32), _cuda(uniform, "uniform", torch.float32),
                  _cuda(out, "sample out", torch.int32), _stream()), "sample")


class WeightPrefetcher:
    """Keeps HBM busy between the weight-streaming products of a captured decode step.

    ``weights`` is the order in which the step's products read their weights (recorded on an eager
    run).  Before product ``i`` is launched on the capturing stream, a side stream is forked with an event
    (so it runs beside product ``i``) and prefetches the head of product ``i + 1``'s weights into L2: from the
    end of what was prefetched so far up to ``window`` bytes beyond their start.  Product ``i + 1`` then finds
    its first rounds of loads in L2 and HBM does not idle while it starts up.  ``IIAN_PREFETCH_EARLY=0`` forks
    after product ``i`` instead (the prefetch then runs beside whatever follows it, which only pays where an
    attention kernel follows: 3.55 against 3.48 ms a step at batch 1, 3.72 against 3.67 ms at batch 8).
    The side stream is joined into the main stream before the capture ends.

    Measured on B200 at the Qwen3-8B sizes, batch 8: a window of 8 MB (the head of the next matrix, which
    hides the ramp-up of its product) gains 2.4 % of the step; 24 MB and more lose, because a matrix that
    streams through L2 evicts what was prefetched beyond it.
    """

    def __init__(self, weights, window: int = int(os.environ.get("IIAN_PREFETCH_WINDOW_MB", "8")) << 20):
        self.weights = list(weights)
        self.starts = []
        pos = 0
        for _, nbytes in self.weights:
            self.starts.append(pos)
            pos += nbytes
        self.total = pos
        self.window = window
        self.early = os.environ.get("IIAN_PREFETCH_EARLY", "1") not in ("0", "false", "off")
        self.side = torch.cuda.Stream()
        self.index = 0             # products launched so far
        self.cursor = 0            # bytes of the concatenated weight sequence already asked for
        self.launches = 0

    def before_product(self, kernels) -> None:
        if self.early:
            self._prefetch_head(kernels, self.index + 1)

    def after_product(self, kernels) -> None:
        self.index += 1
        if not self.early:
            self._prefetch_head(kernels, self.index)

    def _prefetch_head(self, kernels, j: int) -> None:
        """Fork the side stream at this point of the main stream and ask for the head of product ``j``'s weights."""
        if j >= len(self.weights):
            return
        begin = max(self.cursor, self.starts[j])
        end = min(self.total, self.starts[j] + self.window)
        if end <= begin:
            return
        main = torch.cuda.current_stream()
        ev = torch.cuda.Event()
        ev.record(main)
        self.side.wait_event(ev)
        with torch.cuda.stream(self.side):
            while j < len(self.weights) and self.starts[j] < end:
                ptr, nbytes = self.weights[j]
                lo = max(begin, self.starts[j]) - self.starts[j]
                hi = min(end, self.starts[j] + nbytes) - self.starts[j]
                if hi > lo:
                    kernels.prefetch_l2(ptr + lo, hi - lo, stream=self.side.cuda_stream)
                    self.launches += 1
                j += 1
        self.cursor = end

    def join(self) -> None:
        ev = torch.cuda.Event()
        ev.record(self.side)
        torch.cuda.current_stream().wait_event(ev)
