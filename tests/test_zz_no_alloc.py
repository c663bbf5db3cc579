"""The split-KV attention entry point that allocates nothing.

Some users of the kernel library cannot allocate device memory when they call it: their process has
given the whole GPU to a pool of its own, or they sit in a loop where the device-wide synchronisation
of an allocation is not acceptable.  ``iian_attention_mma_noalloc`` keeps the partial results of the
key splits in a fixed array inside the library instead.  Here it is called through its exported C
symbol, twice in a row on different inputs (the array keeps the first call's contents), and each
result is compared with the regular entry point's, which gets its scratch from the caller.

The file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, q, kc, vc, out, m, nh, nkv, hd, scale, window, n_split, small_tiles=1):
    fn = lib.iian_attention_mma_noalloc
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p]
    fn.restype = c_int
    return fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), m.cu_q.data_ptr(), m.ctx_len.data_ptr(),
              m.block_table.data_ptr(), m.block_table.shape[1], q.shape[0], m.num_seqs, m.max_q_len, nh, nkv, hd,
              kc.shape[2], kc.shape[0], scale, window or 0, n_split, small_tiles, torch.cuda.current_stream().cuda_stream)


def test_noalloc_entry_matches_the_regular_one_twice_in_a_row():
    from iian_b200.csrc import build
    from iian_b200.ops.cuda_backend import CudaKernels
    from test_kernels_gpu import attention_case, tol

    lib = build.load("attention_mma")
    lib.iian_attention_mma_noalloc_capacity.restype = c_longlong
    capacity = lib.iian_attention_mma_noalloc_capacity()
    assert capacity >= 1 << 20
    k = CudaKernels()
    dtype = torch.bfloat16
    # the decode form (arrival counters and partial results in the array), twice; then the prefill form on
    # portions of several tokens with a window (a second kernel reads the partial results out of the array)
    cases = [((8, 2, 128, 16, [700, 257, 31], [1, 1, 1], None), 6, 11, True),
             ((6, 3, 64, 8, [150, 90], [1, 1], 40), 3, 12, True),
             ((8, 2, 128, 16, [300, 97], [40, 9], 70), 3, 13, False),
             ((4, 4, 64, 8, [130], [33], None), 2, 14, False)]
    for (nh, nkv, hd, ps, ctx_lens, q_lens, window), n_split, seed, small in cases:
        q, kc, vc, m, want, scale = attention_case(dtype, nh, nkv, hd, ps, ctx_lens, q_lens, window, seed=seed)
        ref = torch.empty(q.shape[0], nh * hd, dtype=dtype, device="cuda")
        k.paged_attention_mma(q, kc, vc, ref, m, num_heads=nh, num_kv_heads=nkv, head_dim=hd, scale=scale,
                              window=window, n_split=n_split, small_tiles=small, cluster=False)
        got = torch.full_like(ref, float("nan"))
        rc = _call_noalloc(lib, q, kc, vc, got, m, nh, nkv, hd, scale, window, n_split, 1 if small else 0)
        assert rc == 0, f"entry point returned {rc}"
        torch.cuda.synchronize()
        assert (got.float() - ref.float()).abs().max().item() <= tol(dtype, max(1.0, want.abs().max().item()))
        assert (got.double().cpu() - want).abs().max().item() < tol(dtype, max(1.0, want.abs().max().item()))


def test_noalloc_entry_refuses_more_than_its_array_holds():
    from iian_b200.csrc import build
    from test_kernels_gpu import attention_case

    lib = build.load("attention_mma")
    lib.iian_attention_mma_noalloc_capacity.restype = c_longlong
    capacity = lib.iian_attention_mma_noalloc_capacity()
    nh, nkv, hd = 8, 2, 128
    q, kc, vc, m, want, scale = attention_case(torch.bfloat16, nh, nkv, hd, 16, [40], [1], None, seed=1)
    out = torch.zeros(1, nh * hd, dtype=torch.bfloat16, device="cuda")
    too_many = capacity // (nh * (hd + 1)) + 1            # N * nh * n_split * (hd + 1) > capacity with N = 1
    assert _call_noalloc(lib, q, kc, vc, out, m, nh, nkv, hd, scale, None, int(too_many)) == 4
    torch.cuda.synchronize()
    assert out.abs().max().item() == 0.0, "a refused call must launch nothing"
    # the form that merges inside a thread-block cluster uses nothing of the array, so the limit does not apply
    q, kc, vc, m, want, scale = attention_case(torch.bfloat16, nh, nkv, hd, 16, [4000, 3000], [1, 1], None, seed=2)
    from iian_b200.ops.cuda_backend import CudaKernels
    from test_kernels_gpu import tol
    got = torch.full((2, nh * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert _call_noalloc(lib, q, kc, vc, got, m, nh, nkv, hd, scale, None, 8, small_tiles=2) == 0
    torch.cuda.synchronize()
    assert (got.double().cpu() - want).abs().max().item() < tol(torch.bfloat16, max(1.0, want.abs().max().item()))
