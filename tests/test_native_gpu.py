"""The step function and the engine loop in C++ (include/iian_b200/engine.h) against their Python counterparts.

The native step function issues the same kernels with the same arguments in the same order as the Python parts, so
its logits must be the same bits -- in 32-bit and in bfloat16, eagerly and from captured graphs, under every way of
cutting the work (only the library product may differ: the two call it through different front ends).  The native
engine must produce the tokens the Python engine produces, greedy and sampled.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from helpers import BLOCK_SIZE, TINY, random_tokens, replay_and_collect, trace_mixed, trace_portions, trace_tail, trace_whole, write_tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("native")
    return {n: write_tiny(root, n, store_dtype=torch.bfloat16) for n in TINY}


def requests_for(name, lengths, seed):
    v = TINY[name]["vocab_size"]
    return {f"r{i}": random_tokens(v, n, seed + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_native_and_python_step_functions_give_the_same_bits(folders, name, dtype, mode, graphs, monkeypatch):
    from iian_b200.engine.model import Model
    from iian_b200.engine.replay import TraceReplayer
    from iian_b200.ops import cuda_backend
    if graphs and mode in ("whole", "portions"):
        pytest.skip("no step of this trace is decode-only")
    # keep the library product out of the comparison: the two step functions reach it through different front ends
    monkeypatch.setattr(cuda_backend.CudaKernels, "TCGEN05_MIN_TILES", 0)
    reqs = requests_for(name, [5, 130, 64, 33, 90] if name != "A" else [5, 17, 33, 70, 100], 17)
    steps = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}.get(mode)
    steps = steps(reqs) if steps else trace_mixed(reqs, 256, seed=5)
    model = Model.from_folder(folders[name], dtype, "cuda:0")
    out = []
    for native in (False, True):
        rp = TraceReplayer(model, 256, BLOCK_SIZE[name], 4, native=native)
        assert (rp.runner.native is not None) == native
        rp.runner.cuda_graphs = graphs
        out.append(replay_and_collect(rp, steps))
        rp.runner.check_device_status()
        if graphs:
            assert rp.runner.num_graphs > 0
        assert all(p.num_free == p.num_blocks for p in rp.runner.manager.pools)
    a, b = out
    assert a.keys() == b.keys() and len(a) == sum(len(t) for t in reqs.values())
    worst = max((a[k] - b[k]).abs().max().item() for k in a)
    if dtype == "bfloat16":
        # products of 9 to 127 rows take the library in both step functions, through different front ends (torch.mm,
        # cublasGemmEx): their rounding may differ, everything else is the same kernels
        assert worst <= 1e-2 * max(v.abs().max().item() for v in a.values()), f"{name} {mode}: {worst}"
    else:
        assert worst == 0.0, f"{name} {dtype} {mode}: native and Python logits differ by {worst}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_native_engine_produces_the_python_engines_tokens(folders, name, dtype):
    """Chunked prefill, so few pages that requests are preempted, prefix reuse, graphs: greedy in both dtypes, and in
    32-bit also temperature / top-k / top-p / min-p sampling with per-request seeds (the same streams of uniform
    numbers, the same kernels)."""
    from iian_b200 import EngineConfig, SamplingParams, SchedulerConfig
    from iian_b200.engine.engine import Engine
    from iian_b200.engine.model import Model
    from iian_b200.engine.native import NativeEngine
    from iian_b200.engine.runner import ModelRunner
    v = TINY[name]["vocab_size"]
    bs = BLOCK_SIZE[name]
    shared = random_tokens(v, 2 * bs + 3, 300)
    prompts = [shared + random_tokens(v, 3 + 5 * i, 310 + i) if i % 2 else random_tokens(v, 7 + 9 * i, 320 + i) for i in range(7)]
    model = Model.from_folder(folders[name], dtype, "cuda:0")
    kinds = [dict(temperature=0.0)]
    if dtype == "float32":
        kinds.append(dict(temperature=0.8, top_k=40, top_p=0.9, min_p=0.01))
    for kind in kinds:
        py = Engine(model, EngineConfig(dtype=dtype, block_size=bs, max_model_len=128, kv_cache_tokens=256, enable_prefix_caching=True,
                                        cuda_graphs=True, sched=SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=24)))
        want = py.generate(prompts, [SamplingParams(max_tokens=10, seed=40 + i, ignore_eos=True, **kind) for i in range(len(prompts))])
        runner = ModelRunner(model, block_size=bs, capacity_tokens=256, max_num_seqs=8, enable_prefix_caching=True, cuda_graphs=True,
                             max_model_len=128, native=True)
        eng = NativeEngine(runner.native, max_model_len=128, max_num_seqs=8, max_num_batched_tokens=24)
        ids = [eng.submit(p, max_tokens=10, seed=40 + i, ignore_eos=True, **kind) for i, p in enumerate(prompts)]
        got = {i: [] for i in ids}
        done = set()
        for _ in range(2000):
            eng.step()
            for i in ids:
                while i not in done:
                    ch = eng.poll(i)
                    if ch is None:
                        break
                    got[i] += ch[0]
                    if ch[1]:
                        assert ch[2] == 2 and ch[4] == 10           # finished by length after 10 tokens
                        done.add(i)
            if len(done) == len(ids):
                break
        assert len(done) == len(ids)
        st = eng.stats()
        assert st["requests_finished"] == 7 and st["generation_tokens"] == 70 and st["preemptions"] >= 1 and st["prefix_cache_hits"] >= 1
        assert runner.native.num_graphs > 0
        if dtype == "float32":
            assert [got[i] for i in ids] == want
        else:               # bfloat16: another order of requests in a step may round a near-tie the other way
            same = sum(a == b for i, w in zip(ids, want) for a, b in zip(got[i], w))
            assert same >= 60, f"only {same} of 70 tokens agree"
        runner.manager.check_invariants()
        assert all(p.num_free == p.num_blocks for p in runner.manager.pools)
    with pytest.raises(ValueError, match="too long"):
        eng.submit(list(range(5)) * 30)
    with pytest.raises(ValueError, match="out of range"):
        eng.submit([v])


def test_trace_run_with_the_native_step_function(folders, tmp_path):
    reqs = requests_for("B", [40, 23, 9], 51)
    steps = trace_mixed(reqs, 192, seed=2)
    outs = []
    for flag in ("--native", "--no-native"):
        out = tmp_path / flag.strip("-")
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders["B"], "--dtype", "float32",
                               "--out", str(out), "--max-tokens", "192", "--block-size", str(BLOCK_SIZE["B"]), flag],
                              input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        outs.append({f: np.fromfile(out / f, dtype="<f4") for f in sorted(os.listdir(out))})
    assert outs[0].keys() == outs[1].keys() and len(outs[0]) > 0
    for f in outs[0]:
        assert np.array_equal(outs[0][f], outs[1][f]), f"{f}: the two step functions wrote different logits"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_mixed_step_in_any_order_of_its_entries(folders, dtype, monkeypatch):
    """The native step function lays a mixed step out with the single decoded tokens first and, in bfloat16 at head
    size 128, gives their attention to the decode kernel beside the prefill kernel; the logits come back in the order
    of the entries as given, and match the plain implementation and the Python step function, whatever that order."""
    from iian_b200.engine.model import Model
    from iian_b200.engine.replay import TraceReplayer
    from iian_b200.ops import cuda_backend
    from helpers import max_error, plain_logits
    monkeypatch.setattr(cuda_backend.CudaKernels, "TCGEN05_MIN_TILES", 0)
    name = "D"
    v = TINY[name]["vocab_size"]
    reqs = {rid: random_tokens(v, n, 70 + i) for i, (rid, n) in enumerate([("a", 90), ("b", 41), ("c", 77), ("d", 30)])}
    # b and d are fed whole first; then steps in which portions of a and c stand before, between and behind single
    # tokens of b and d (which are fed again from their caches: a request may end and start anew under the same name)
    head = {"b": 36, "d": 25}
    steps = [{"step": 0, "entries": [{"id": r, "tokens": reqs[r][:n], "want": [n - 1]} for r, n in head.items()], "end": []}]
    cuts = {"a": [0, 20, 52, 70, 90], "c": [0, 33, 50, 61, 77]}
    for k in range(4):
        ents = []
        order = [["a", "b", "c", "d"], ["b", "a", "d", "c"], ["a", "c", "b", "d"], ["d", "c", "b", "a"]][k]
        for r in order:
            if r in head:
                p = head[r] + k
                ents.append({"id": r, "tokens": [reqs[r][p]], "want": [0]})
            else:
                lo, hi = cuts[r][k], cuts[r][k + 1]
                ents.append({"id": r, "tokens": reqs[r][lo:hi], "want": [0, hi - lo - 1]})
        steps.append({"step": k + 1, "entries": ents, "end": []})
    steps[-1]["end"] = list(reqs)
    model = Model.from_folder(folders[name], dtype, "cuda:0")
    got = []
    for native in (False, True):
        rp = TraceReplayer(model, 512, BLOCK_SIZE[name], 4, native=native)
        got.append(replay_and_collect(rp, steps))
        rp.runner.check_device_status()
        if native and dtype == "bfloat16":
            by = rp.runner.launches_by_entry()
            assert rp.runner.native.launches_of("attention_mma") > 0 and by.get("attention_tc", 0) > 0
    want = plain_logits(folders[name], reqs)
    limit = 2e-5 if dtype == "float32" else 2.5e-2 * max(w.abs().max().item() for w in want.values())
    for g in got:
        err, where = max_error(g, want)
        assert err <= limit, (dtype, err, where)
    if dtype == "float32":
        assert all(torch.equal(got[0][k], got[1][k]) for k in got[0])
