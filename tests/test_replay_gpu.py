"""Replay on the GPU, in 32-bit and in bfloat16: each request alone and whole; most of it in one step
and the last 32 tokens one by one; portions of changing size down to two tokens; mixed, up to four
live requests with so few pages that they are used again; long decoding; the first tokens of a
sequence.  Every emitted logits row is compared with the plain implementation (tests/plain_qwen3.py).
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import (BLOCK_SIZE, TINY, first_bad, max_error, plain_logits, random_tokens, replay_and_collect,
                     trace_mixed, trace_portions, trace_tail, trace_whole, write_tiny)

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL32 = 2e-5            # float32 path against the float64 plain implementation (the target is 1e-4)
# bfloat16: weights are stored in bfloat16 and read identically by both sides, so the difference is the
# rounding of activations (8 bits of mantissa) through a few layers, relative to the logits' scale.
TOL16_REL = 2.5e-2


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {n: write_tiny(root, n, store_dtype=torch.bfloat16) for n in TINY}


@pytest.fixture(scope="module")
def plains(folders):
    cache = {}

    def get(name, reqs):
        key = (name, tuple(sorted((k, tuple(v)) for k, v in reqs.items())))
        if key not in cache:
            cache[key] = plain_logits(folders[name], reqs)
        return cache[key]
    return get


def requests_for(name, lengths, seed):
    v = TINY[name]["vocab_size"]
    return {f"r{i}": random_tokens(v, n, seed + i) for i, n in enumerate(lengths)}


def tolerance(dtype, want):
    if dtype == "float32":
        return TOL32
    scale = max(w.abs().max().item() for w in want.values())
    return TOL16_REL * scale


def check(folders, plains, name, dtype, reqs, steps, max_tokens):
    from iian_b200.engine.replay import TraceReplayer
    want = plains(name, reqs)
    rp = TraceReplayer.from_folder(folders[name], dtype, max_tokens, BLOCK_SIZE[name])
    before = rp.runner.launches_by_entry()
    got = replay_and_collect(rp, steps)
    after = rp.runner.launches_by_entry()
    check.seen = {k for k, v in after.items() if v > before.get(k, 0)}       # entry points that served this replay
    rp.runner.check_device_status()
    rp.runner.manager.check_invariants()
    assert all(p.num_free == p.num_blocks for p in rp.runner.manager.pools), "pages were lost"
    assert len(got) == sum(len(t) for t in reqs.values())
    tol = tolerance(dtype, want)
    bad = first_bad(got, want, tol)
    worst, where = max_error(got, want)
    print(f"[{name} {dtype}] max err {worst:.3g} at {where}, tol {tol:.3g}")
    assert bad is None, f"first wrong logits at request {bad[0]} position {bad[1]} (err {bad[2]:.3g}, tol {tol:.3g})"
    return got


LENGTHS = {"A": [5, 17, 33, 70, 100], "B": [1, 7, 24, 61, 100, 45], "C": [3, 50, 129, 64, 90],
           "D": [5, 130, 64, 200, 33], "E": [1, 70, 129, 50, 90], "F": [3, 40, 100, 17, 65]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_cutting_does_not_change_logits(folders, plains, name, dtype, mode):
    reqs = requests_for(name, LENGTHS[name], 11)
    max_tokens = 256
    builder = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}.get(mode)
    steps = builder(reqs) if builder else trace_mixed(reqs, max_tokens, seed=3)
    check(folders, plains, name, dtype, reqs, steps, max_tokens)


# which entry points of the kernel layer must have served a bfloat16 model with heads of 128 (D) or 64 (E, F),
# by the way its work was cut (ops.cuda_backend.LAUNCHES_BY_ENTRY); the general attention kernel must not appear
SERVED_BY = {
    ("D", "whole"): {"attention_tc", "gemm_tcgen05"},                    # long portions: tcgen05 attention and products
    ("D", "tail"): {"attention_tc", "attention_decode_fused", "gemm_stream"},
    ("D", "portions"): {"attention_tc", "attention_mma"},               # portions under 16 tokens go to mma.sync
    ("D", "mixed"): {"attention_decode_fused", "gemm_stream"},
    ("E", "whole"): {"attention_mma", "gemm_tcgen05"},
    ("E", "tail"): {"attention_mma", "attention_decode_fused", "gemm_stream"},
    ("F", "mixed"): {"attention_mma", "attention_decode_fused"},
}


@pytest.mark.parametrize("case", sorted(SERVED_BY))
@pytest.mark.parametrize("min_tiles", [0, 300])
def test_the_serving_kernels_run_inside_whole_model_checks(folders, plains, monkeypatch, case, min_tiles):
    """The logits of D, E and F in bfloat16 come from the kernels that serve the large shapes, not from the general
    ones -- with the own tcgen05 product from the first tile on (as the other tests run) and with the dispatch
    rule's default threshold, under which these small products go to the library instead."""
    from iian_b200.ops import cuda_backend
    name, mode = case
    monkeypatch.setattr(cuda_backend.CudaKernels, "TCGEN05_MIN_TILES", min_tiles)
    reqs = requests_for(name, LENGTHS[name], 13)
    builder = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}.get(mode)
    steps = builder(reqs) if builder else trace_mixed(reqs, 256, seed=6)
    check(folders, plains, name, "bfloat16", reqs, steps, 256)
    seen = check.seen
    want = set(SERVED_BY[case])
    if min_tiles:
        want = {("library_gemm" if w == "gemm_tcgen05" else w) for w in want}
    assert want <= seen, f"{name} {mode}: expected launches of {sorted(want - seen)}; saw {sorted(seen)}"
    assert "paged_attention_generic" not in seen


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_float32_rows_are_bit_identical_under_recutting(folders, plains, dtype):
    """The 32-bit kernels add in an order that depends only on a token's own position, so cutting the
    work differently must not change a single bit; bfloat16 only has to stay within rounding."""
    from iian_b200.engine.replay import TraceReplayer
    reqs = requests_for("C", [129, 64, 90], 21)
    a = replay_and_collect(TraceReplayer.from_folder(folders["C"], dtype, 384, 16), trace_whole(reqs))
    b = replay_and_collect(TraceReplayer.from_folder(folders["C"], dtype, 384, 16), trace_mixed(reqs, 384, seed=9))
    worst = max((a[k] - b[k]).abs().max().item() for k in a)
    if dtype == "float32":
        assert worst == 0.0, f"float32 logits moved by {worst} when the work was cut differently"
    else:
        assert worst < TOL16_REL * max(v.abs().max().item() for v in a.values())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D", "E"])
def test_pages_are_used_again(folders, plains, name, dtype):
    reqs = requests_for(name, [60, 60, 60, 60, 60, 60], 5)
    check(folders, plains, name, dtype, reqs, trace_mixed(reqs, 128, seed=1), 128)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C", "D", "E"])
def test_long_decoding(folders, plains, name, dtype):
    n = TINY[name]["max_position_embeddings"] - 6
    reqs = requests_for(name, [n], 31)
    steps = trace_tail(reqs, tail=n - 9)           # 9 prompt tokens, then one by one
    check(folders, plains, name, dtype, reqs, steps, 512)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_first_tokens(folders, plains, name, dtype):
    reqs = requests_for(name, [1, 2, 3], 41)
    check(folders, plains, name, dtype, reqs, trace_tail(reqs, tail=8), 256)
    check(folders, plains, name, dtype, reqs, trace_whole(reqs), 256)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(folders, plains, tmp_path, dtype):
    """The program itself: steps on standard input, ``<step>.f32`` files, ``done`` lines, exit 0."""
    reqs = requests_for("B", [40, 23, 9], 51)
    steps = trace_mixed(reqs, 192, seed=2)
    out = tmp_path / f"out_{dtype}"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["B"], "--dtype", dtype,
                           "--out", str(out), "--max-tokens", "192", "--block-size", str(BLOCK_SIZE["B"])],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    want = plains("B", reqs)
    vocab = TINY["B"]["vocab_size"]
    fed = {}
    got = {}
    for rec in steps:
        n_want = sum(len(e["want"]) for e in rec["entries"])
        path = out / f"{rec['step']}.f32"
        if n_want == 0:
            assert not path.exists()
            continue
        rows = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(n_want, vocab).copy())
        r = 0
        for e in rec["entries"]:
            start = fed.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], start + w)] = rows[r]
                r += 1
            fed[e["id"]] = start + len(e["tokens"])
    bad = first_bad(got, want, tolerance(dtype, want))
    assert bad is None, bad
