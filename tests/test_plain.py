"""The plain implementation itself: against logits the reference's own model code produced
(tests/golden/, made by tests/golden/make_golden.py), and small checks of its parts."""
import json
import math
import os

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["tinyA", "tinyB"])
def test_plain_vs_golden(name):
    d = os.path.join(GOLDEN, name)
    cfg, w = plain.load_folder(d)
    with open(os.path.join(d, "tokens.json")) as f:
        toks = json.load(f)
    ref = torch.from_numpy(np.fromfile(os.path.join(d, "logits.f32"), dtype="<f4").reshape(len(toks), cfg["vocab_size"]).copy())
    got = plain.forward(cfg, w, toks)
    err = (got - ref.double()).abs().max().item()
    assert err < 5e-6, f"plain implementation differs from the reference's own graph by {err}"
    assert torch.equal(got.argmax(-1), ref.argmax(-1))
    got32 = plain.forward(cfg, w, toks, dtype=torch.float32)
    assert (got32.double() - ref.double()).abs().max().item() < 2e-5


def test_rms_norm_and_silu():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    rms = math.sqrt((9 + 16) / 2 + 1e-6)
    assert torch.allclose(plain.rms_norm(x, w, 1e-6), torch.tensor([[3 / rms * 2, 4 / rms * 0.5]], dtype=torch.float64))
    z = torch.tensor([0.0, 1.0, -2.0], dtype=torch.float64)
    assert torch.allclose(plain.silu(z), z * torch.sigmoid(z))


def test_rope_rotates_pairs_and_keeps_relative_angles():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 1, 8, generator=g, dtype=torch.float64).expand(6, 1, 8).clone()
    k = torch.randn(1, 1, 8, generator=g, dtype=torch.float64).expand(6, 1, 8).clone()
    pos = torch.arange(6)
    rq, rk = plain.rope_neox(q, pos, 10000.0, 8), plain.rope_neox(k, pos, 10000.0, 8)
    assert torch.allclose(rq[0], q[0])                                       # position 0: no rotation
    assert torch.allclose(rq.norm(dim=-1), q.norm(dim=-1))                   # a rotation keeps lengths
    d1 = (rq[1] * rk[0]).sum()                                               # depends on the distance only
    d2 = (rq[5] * rk[4]).sum()
    assert abs(d1.item() - d2.item()) < 1e-6
    # pairs are (j, j + n/2): with a zeroed second half the first half is scaled by cos
    x = torch.zeros(1, 1, 8, dtype=torch.float64)
    x[..., 0] = 1.0
    r = plain.rope_neox(x, torch.tensor([2]), 10000.0, 8)
    assert abs(r[0, 0, 0].item() - math.cos(2.0)) < 1e-6 and abs(r[0, 0, 4].item() - math.sin(2.0)) < 1e-6
    part = plain.rope_neox(q, pos, 10000.0, 4)                               # partial rotation leaves the rest alone
    assert torch.equal(part[..., 4:], q[..., 4:])


def test_attention_is_causal_grouped_and_windowed():
    g = torch.Generator().manual_seed(1)
    T, nh, nkv, hd = 9, 4, 2, 8
    q = torch.randn(T, nh, hd, generator=g, dtype=torch.float64)
    k = torch.randn(T, nkv, hd, generator=g, dtype=torch.float64)
    v = torch.randn(T, nkv, hd, generator=g, dtype=torch.float64)
    out = plain.attention(q, k, v, 0.3, None)
    assert torch.allclose(out[0, 0], v[0, 0]) and torch.allclose(out[0, 3], v[0, 1])    # first token sees itself; head 3 -> KV head 1
    k2, v2 = k.clone(), v.clone()
    k2[5:], v2[5:] = 0, 0
    assert torch.allclose(plain.attention(q, k2, v2, 0.3, None)[:5], out[:5])           # the future does not matter
    w = plain.attention(q, k, v, 0.3, 3)
    s = (q[8, 0] @ k[6:9, 0].T) * 0.3
    want = torch.softmax(s, 0) @ v[6:9, 0]
    assert torch.allclose(w[8, 0], want)                                                # window 3: keys 6, 7, 8
    assert torch.allclose(w[:3], out[:3])                                               # inside the window nothing changes


def test_argmax_and_sampling_rules():
    assert plain.argmax(torch.tensor([1.0, 5.0, 5.0, 2.0])) == 1                        # lowest id wins a tie
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, -5.0])
    p = plain.candidate_probs(logits, 1.0)
    assert (p > 0).all()
    assert (plain.candidate_probs(logits, 1.0, top_k=2) > 0).tolist() == [True, True, False, False, False]
    keep = plain.candidate_probs(logits, 1.0, min_p=0.2) > 0                            # p_i >= 0.2 * p_max  <=>  z_i >= z_max + ln 0.2
    assert keep.tolist() == [True, True, False, False, False]
    full = torch.softmax(logits.double(), 0)
    keep = plain.candidate_probs(logits, 1.0, top_p=0.9) > 0
    n = int(keep.sum())
    assert full[:n].sum() >= 0.9 > full[:n - 1].sum()
    assert plain.sample_from(torch.tensor([0.0, 1.0, 0.0, 3.0]), 0.2) == 1
    assert plain.sample_from(torch.tensor([0.0, 1.0, 0.0, 3.0]), 0.26) == 3
    assert plain.sample_from(torch.tensor([0.0, 1.0, 0.0, 3.0]), 0.999999) == 3


def test_layer_windows_follow_the_config():
    assert plain.layer_windows({"num_hidden_layers": 3}) == [None, None, None]
    cfg = {"num_hidden_layers": 3, "use_sliding_window": True, "sliding_window": 5, "max_window_layers": 1}
    assert plain.layer_windows(cfg) == [None, 5, 5]
    cfg = {"num_hidden_layers": 2, "sliding_window": 7, "layer_types": ["sliding_attention", "full_attention"]}
    assert plain.layer_windows(cfg) == [7, None]
