"""Shared by the tests: tiny configurations, model folders in temporary places, trace builders and
the comparison of replayed logits with the plain implementation."""
from __future__ import annotations

import os
import random
from typing import Dict, List, Optional, Sequence, Tuple

import torch

import plain_qwen3 as plain

# Tiny Qwen3 configurations that differ in every size and option: layers, width (some are no power of two),
# heads and groups, head size (explicit, != hidden/heads), feed-forward width, vocabulary (most are odd),
# rope base, norm eps, tied or not, page size, and a sliding window on some layers.  A, B and C have head
# sizes only the general kernels take; D (head size 128), E and F (head size 64, eight query heads on one
# KV head / one each) are served in bfloat16 by the kernels that serve the large shapes: tcgen05 prefill
# attention, mma.sync attention, the fused decode attention with its cluster merge, the 16-lane rotary form.
TINY = {
    "A": dict(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6, rope_theta=10000.0,
              max_position_embeddings=128, tie_word_embeddings=True),
    "B": dict(vocab_size=503, hidden_size=96, intermediate_size=160, num_hidden_layers=3, num_attention_heads=8,
              num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-5, rope_theta=1000000.0,
              max_position_embeddings=256, tie_word_embeddings=False),
    "C": dict(vocab_size=311, hidden_size=80, intermediate_size=112, num_hidden_layers=4, num_attention_heads=6,
              num_key_value_heads=3, head_dim=48, rms_norm_eps=3e-6, rope_theta=500000.0,
              max_position_embeddings=512, tie_word_embeddings=False,
              use_sliding_window=True, sliding_window=20, max_window_layers=1),
    "D": dict(vocab_size=331, hidden_size=256, intermediate_size=384, num_hidden_layers=3, num_attention_heads=8,
              num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
              max_position_embeddings=512, tie_word_embeddings=False,
              use_sliding_window=True, sliding_window=40, max_window_layers=2),
    "E": dict(vocab_size=257, hidden_size=192, intermediate_size=320, num_hidden_layers=3, num_attention_heads=8,
              num_key_value_heads=1, head_dim=64, rms_norm_eps=2e-6, rope_theta=10000.0,
              max_position_embeddings=384, tie_word_embeddings=True,
              use_sliding_window=True, sliding_window=48, max_window_layers=1),
    "F": dict(vocab_size=199, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=4, head_dim=64, rms_norm_eps=1e-5, rope_theta=50000.0,
              max_position_embeddings=256, tie_word_embeddings=False),
}
BLOCK_SIZE = {"A": 16, "B": 8, "C": 16, "D": 16, "E": 8, "F": 32}
SEED = {"A": 0, "B": 2, "C": 5, "D": 6, "E": 7, "F": 8}


def tiny_config(name: str):
    from iian_b200.models.qwen3 import qwen3_config_from_dict
    return qwen3_config_from_dict(TINY[name])


def write_tiny(tmp_path, name: str, store_dtype=torch.float32, seed: Optional[int] = None) -> str:
    from iian_b200.config.registry import get_architecture
    from iian_b200.weights.random_init import write_model_folder
    d = os.path.join(str(tmp_path), f"tiny{name}_{str(store_dtype).split('.')[-1]}")
    if not os.path.isdir(d):
        write_model_folder(d, get_architecture("Qwen3ForCausalLM"), tiny_config(name),
                           seed=SEED[name] if seed is None else seed, store_dtype=store_dtype)
    return d


def random_tokens(vocab: int, n: int, seed: int) -> List[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ---- traces ---------------------------------------------------------------------------------------
def trace_whole(requests: Dict[str, List[int]]) -> List[dict]:
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def trace_tail(requests: Dict[str, List[int]], tail: int = 32) -> List[dict]:
    steps = []
    n = 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        n += 1
        for p in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def trace_portions(requests: Dict[str, List[int]], sizes: Sequence[int] = (13, 7, 2, 5, 3, 2, 17, 1, 9, 2)) -> List[dict]:
    steps = []
    n = 0
    for rid, toks in requests.items():
        p, k = 0, 0
        while p < len(toks):
            c = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[p:p + c], "want": list(range(c))}],
                          "end": [rid] if p + c == len(toks) else []})
            p += c
            n += 1
    return steps


def trace_mixed(requests: Dict[str, List[int]], max_tokens: int, seed: int = 0, max_live: int = 4,
                round_to: int = 64) -> List[dict]:
    """Up to ``max_live`` requests at a time; each step brings portions of some and single tokens of
    others, sometimes leaves a request out; a request is admitted only if the tokens of the live ones,
    each rounded up to ``round_to``, still fit ``max_tokens`` -- so pages are given back and used again."""
    rng = random.Random(seed)
    pending = list(requests.items())
    live: Dict[str, int] = {}          # id -> tokens fed
    steps = []
    n = 0

    def rounded(k):
        return (k + round_to - 1) // round_to * round_to

    while pending or live:
        while pending and len(live) < max_live:
            rid, toks = pending[0]
            if sum(rounded(len(requests[r])) for r in live) + rounded(len(toks)) > max_tokens:
                break
            pending.pop(0)
            live[rid] = 0
        if not live:
            raise ValueError("a request does not fit max_tokens on its own")
        entries, ended = [], []
        ids = list(live)
        rng.shuffle(ids)
        for rid in ids:
            toks = requests[rid]
            fed = live[rid]
            left = len(toks) - fed
            if len(ids) > 1 and rng.random() < 0.2:
                continue                                   # left out of this step
            if left > 34:
                c = min(left - 32, rng.choice([2, 3, 5, 7, 13, 17, 29]))
            else:
                c = 1 if rng.random() < 0.8 else min(left, 2)
            entries.append({"id": rid, "tokens": toks[fed:fed + c], "want": list(range(c))})
            live[rid] = fed + c
            if live[rid] == len(toks):
                ended.append(rid)
        if not entries:
            continue
        steps.append({"step": n, "entries": entries, "end": ended})
        n += 1
        for rid in ended:
            del live[rid]
    return steps


def replay_and_collect(replayer, steps: List[dict]) -> Dict[Tuple[str, int], torch.Tensor]:
    """Run the steps; (request id, position) -> logits row (CPU float32)."""
    fed: Dict[str, int] = {}
    out: Dict[Tuple[str, int], torch.Tensor] = {}
    for rec in steps:
        logits = replayer.run_step(rec)
        rows = logits.detach().float().cpu().clone() if logits is not None else None   # the runner reuses its logits buffer
        r = 0
        for ent in rec["entries"]:
            start = fed.get(ent["id"], 0)
            for w in ent.get("want", []):
                out[(ent["id"], start + w)] = rows[r]
                r += 1
            fed[ent["id"]] = start + len(ent["tokens"])
        for rid in rec.get("end", []):
            fed.pop(rid, None)
    return out


def plain_logits(model_dir: str, requests: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    cfg, w = plain.load_folder(model_dir)
    return {rid: plain.forward(cfg, w, toks) for rid, toks in requests.items()}


def max_error(got: Dict[Tuple[str, int], torch.Tensor], want: Dict[str, torch.Tensor]) -> Tuple[float, Tuple[str, int]]:
    worst, where = 0.0, ("", -1)
    for (rid, pos), row in got.items():
        e = (row.double() - want[rid][pos]).abs().max().item()
        if not e <= worst:      # NaN counts as worst
            if e != e:
                return float("inf"), (rid, pos)
            worst, where = e, (rid, pos)
    return worst, where


def first_bad(got, want, tol) -> Optional[Tuple[str, int, float]]:
    """The earliest (request, position) whose logits differ from the plain ones by more than ``tol``."""
    for (rid, pos) in sorted(got, key=lambda k: (k[0], k[1])):
        e = (got[(rid, pos)].double() - want[rid][pos]).abs().max().item()
        if not e <= tol:
            return rid, pos, e
    return None
