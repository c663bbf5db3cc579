"""The host side of the step function on the CPU: batch building, block tables, windows, page reuse.

A torch stand-in replaces the CUDA kernels here (tests/fake_kernels.py), so these tests say nothing
about the kernels; they compare the engine's cutting and caching with the plain implementation under
every way of cutting the work.  The same scenarios run on the real kernels in the ``-m gpu`` tests.
"""
import pytest
import torch

from helpers import (BLOCK_SIZE, TINY, first_bad, max_error, plain_logits, random_tokens, replay_and_collect,
                     trace_mixed, trace_portions, trace_tail, trace_whole, write_tiny)
from fake_kernels import FakeKernels
from iian_b200 import ops
from iian_b200.engine.replay import TraceError, TraceReplayer

TOL = 2e-5


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    return {n: write_tiny(root, n) for n in TINY}


def requests_for(name, lengths, seed):
    v = TINY[name]["vocab_size"]
    return {f"r{i}": random_tokens(v, n, seed + i) for i, n in enumerate(lengths)}


@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
def test_cutting_does_not_change_logits(folders, name, mode):
    lengths = [5, 17, 33, 70] if name == "A" else [1, 7, 24, 61, 100, 45]
    reqs = requests_for(name, lengths, 11)
    want = plain_logits(folders[name], reqs)
    max_tokens = 256
    steps = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}.get(mode)
    steps = steps(reqs) if steps else trace_mixed(reqs, max_tokens, seed=3)
    with ops.use_kernels(FakeKernels()):
        rp = TraceReplayer.from_folder(folders[name], "float32", max_tokens, BLOCK_SIZE[name], device="cpu")
        got = replay_and_collect(rp, steps)
        rp.runner.manager.check_invariants()
        assert all(p.num_free == p.num_blocks for p in rp.runner.manager.pools), "pages were lost"
    assert len(got) == sum(lengths)
    bad = first_bad(got, want, TOL)
    assert bad is None, f"first wrong logits at request {bad[0]} position {bad[1]} (err {bad[2]:.3g})"


def test_pages_are_used_again(folders):
    reqs = requests_for("B", [60, 60, 60, 60, 60, 60], 5)
    steps = trace_mixed(reqs, 128, seed=1)       # two live requests at most: 6 x 64 > 128
    with ops.use_kernels(FakeKernels()):
        rp = TraceReplayer.from_folder(folders["B"], "float32", 128, BLOCK_SIZE["B"], device="cpu")
        got = replay_and_collect(rp, steps)
    bad = first_bad(got, plain_logits(folders["B"], reqs), TOL)
    assert bad is None, bad


def test_out_of_pages_is_an_error(folders):
    with ops.use_kernels(FakeKernels()):
        rp = TraceReplayer.from_folder(folders["A"], "float32", 64, 16, device="cpu")
        with pytest.raises(TraceError, match="out of cache pages"):
            rp.run_step({"step": 0, "entries": [{"id": "x", "tokens": list(range(65)), "want": []}], "end": []})
