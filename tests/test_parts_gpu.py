"""Each part of a layer alone on the GPU, built from a PartSpec (no model, no configuration), against
the plain functions: norm, position encoding, attention mixer (whole, in portions, windowed, reading
another call's cache, with biases), gated feed-forward, embedding, head, block arrangement."""
import math

import pytest
import torch

import plain_qwen3 as plain
from iian_b200.cache.storage import KVView
from iian_b200.config.spec import LayerSpec, PartSpec
from iian_b200.engine.runner import PageMeta, StepContext, Workspace
from iian_b200.parts.base import BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, KVNeed

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return (3e-5 if dtype == torch.float32 else 2e-2) * max(scale, 1e-3)


def rnd(*shape, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * std


def stored(t, dtype):
    """What a part holds after loading: matrices in the activation dtype."""
    return t.to(dtype).to(DEV)


def make_ctx(seqs, page_size, num_pages, tables, rows=None):
    """A step context for sequences given as (start, n_new): what ModelRunner.build_context produces."""
    ctx = StepContext(Workspace(DEV))
    pos, seq, cu, ctxl, slots = [], [], [0], [], []
    for s, (start, n) in enumerate(seqs):
        for p in range(start, start + n):
            pos.append(p)
            seq.append(s)
            slots.append(tables[s][p // page_size] * page_size + p % page_size)
        cu.append(cu[-1] + n)
        ctxl.append(start + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    maxb = max(len(t) for t in tables)
    bt = torch.full((len(seqs), maxb), -1, dtype=torch.int32)
    for s, t in enumerate(tables):
        bt[s, :len(t)] = torch.tensor(t, dtype=torch.int32)
    ctx.positions, ctx.seq_of_token, ctx.cu_q, ctx.ctx_len = i32(pos), i32(seq), i32(cu), i32(ctxl)
    ctx.num_tokens, ctx.num_seqs = len(pos), len(seqs)
    ctx.h_q_start, ctx.h_q_len, ctx.h_ctx_len = cu[:-1], [n for _, n in seqs], ctxl
    ctx.max_q_len, ctx.max_ctx = max(ctx.h_q_len), max(ctxl)
    ctx.decode_only = ctx.max_q_len == 1
    ctx.out_rows = i32(rows if rows is not None else list(range(len(pos))))
    ctx.rows_identity = rows is None
    ctx.metas = [PageMeta(positions=ctx.positions, seq_of_token=ctx.seq_of_token, cu_q=ctx.cu_q, ctx_len=ctx.ctx_len,
                               block_table=bt.to(DEV), slots=i32(slots), num_seqs=len(seqs), num_tokens=len(pos),
                               max_q_len=ctx.max_q_len, max_ctx=ctx.max_ctx, decode_only=ctx.decode_only,
                               h_q_len=ctx.h_q_len, h_ctx_len=ctx.h_ctx_len)]
    return ctx


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part(dtype):
    part = NORMS.build(PartSpec("rms_norm", {"size": 100, "eps": 1e-4}), dtype, DEV)
    assert part.tensors()["weight"].shape == (100,)
    w = rnd(100, seed=1) * 0.1 + 1
    part.bind({"weight": w.to(DEV)})
    ctx = make_ctx([(0, 5)], 8, 4, [[0]])
    res = rnd(5, 100, seed=2).to(DEV)
    delta = stored(rnd(5, 100, seed=3), dtype)
    want_res = res.double().cpu() + delta.double().cpu()
    out = part.forward(res, delta, ctx)
    assert out.dtype == dtype and res.dtype == torch.float32
    assert (res.double().cpu() - want_res).abs().max() < 1e-6                       # the residual sum is float32
    want = plain.rms_norm(want_res, w.double(), 1e-4)
    assert (out.double().cpu() - want).abs().max() < tol(dtype, want.abs().max().item())


def test_rotary_part_owns_its_table():
    rot = POSITIONS.build(PartSpec("rotary", {"dim": 24, "base": 500000.0, "style": "neox", "max_position": 64}), torch.float32, DEV)
    j = torch.arange(12, dtype=torch.float64)
    want = torch.pow(torch.tensor(500000.0, dtype=torch.float64), -2 * j / 24).float()
    assert torch.equal(rot.inv_freq.cpu(), want) and rot.dim == 24 and rot.style == 0 and rot.fused
    half = POSITIONS.build(PartSpec("rotary", {"dim": 24, "base": 10000.0, "frequency_scale": 0.5}), torch.float32, DEV)
    assert torch.allclose(half.inv_freq.cpu()[3].double(), 0.5 * torch.pow(torch.tensor(10000.0, dtype=torch.float64), -6 / 24), rtol=1e-6)
    with pytest.raises(ValueError, match="even"):
        POSITIONS.build(PartSpec("rotary", {"dim": 7, "base": 10000.0}), torch.float32, DEV)
    with pytest.raises(KeyError, match="registered"):
        POSITIONS.build(PartSpec("alibi", {}), torch.float32, DEV)


def attention_spec(H, nh, nkv, hd, window=None, rot=None, qk_norm=True, position="rotary"):
    pos = PartSpec("rotary", {"dim": rot or hd, "base": 10000.0, "style": "neox"}) if position == "rotary" else PartSpec("none", {})
    return PartSpec("attention", {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd,
                                  "scale": 1.0 / math.sqrt(hd), "qk_norm": qk_norm, "qk_norm_eps": 1e-5, "window": window,
                                  "position": pos})


def plain_attention_mixer(x, w, nh, nkv, hd, window, rot, qk_norm=True, position="rotary", bias=None):
    T = x.shape[0]
    q, k, v = x @ w["q_proj.weight"].T, x @ w["k_proj.weight"].T, x @ w["v_proj.weight"].T
    if bias:
        q, k, v = q + bias["q"], k + bias["k"], v + bias["v"]
    q, k, v = q.view(T, nh, hd), k.view(T, nkv, hd), v.view(T, nkv, hd)
    if qk_norm:
        q, k = plain.rms_norm(q, w["q_norm.weight"], 1e-5), plain.rms_norm(k, w["k_norm.weight"], 1e-5)
    if position == "rotary":
        pos = torch.arange(T)
        q, k = plain.rope_neox(q, pos, 10000.0, rot), plain.rope_neox(k, pos, 10000.0, rot)
    a = plain.attention(q, k, v, 1.0 / math.sqrt(hd), window).reshape(T, nh * hd)
    o = a @ w["o_proj.weight"].T
    return o + bias["o"] if bias else o


def attention_weights(H, nh, nkv, hd, dtype, seed):
    raw = {"q_proj.weight": rnd(nh * hd, H, seed=seed, std=0.2), "k_proj.weight": rnd(nkv * hd, H, seed=seed + 1, std=0.2),
           "v_proj.weight": rnd(nkv * hd, H, seed=seed + 2, std=0.2), "o_proj.weight": rnd(H, nh * hd, seed=seed + 3, std=0.2),
           "q_norm.weight": rnd(hd, seed=seed + 4) * 0.1 + 1, "k_norm.weight": rnd(hd, seed=seed + 5) * 0.1 + 1}
    dev = {k: (stored(v, dtype) if v.dim() == 2 else v.to(DEV)) for k, v in raw.items()}
    as_read = {k: (v.to(dtype).double() if v.dim() == 2 else v.double()) for k, v in raw.items()}
    return dev, as_read


ATT = [  # H, nh, nkv, hd, page, window, rot
    (80, 6, 3, 48, 8, None, 48),
    (96, 4, 2, 64, 16, None, 64),
    (64, 4, 4, 16, 4, 7, 8),
    (128, 8, 2, 128, 16, 20, 128),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ATT)
def test_attention_mixer_whole_in_portions_and_shared(dtype, case):
    H, nh, nkv, hd, ps, window, rot = case
    T = 45
    part = MIXERS.build(attention_spec(H, nh, nkv, hd, window, rot), dtype, DEV)
    assert part.cache_need() == KVNeed(nkv, hd, window)
    dev_w, w = attention_weights(H, nh, nkv, hd, dtype, seed=10)
    part.bind(dev_w)
    x = rnd(T, H, seed=20)
    xd = stored(x, dtype)
    want = plain_attention_mixer(x.to(dtype).double(), w, nh, nkv, hd, window, rot)
    n_pages = 12
    table = [5, 2, 9, 0, 7, 3][: math.ceil(T / ps)] if ps >= 8 else list(range(11, -1, -1))
    cache = KVView(0, torch.zeros(n_pages, nkv, ps, hd, dtype=dtype, device=DEV), torch.zeros(n_pages, nkv, ps, hd, dtype=dtype, device=DEV))
    scale = want.abs().max().item()
    out = part.forward(xd, make_ctx([(0, T)], ps, n_pages, [table]), cache, True)
    assert (out.double().cpu() - want).abs().max() < tol(dtype, scale)
    # the same tokens in three portions over a fresh cache: 17 + 2 + 26
    cache2 = KVView(0, torch.zeros_like(cache.k), torch.zeros_like(cache.v))
    at = 0
    for n in (17, 2, 26):
        o = part.forward(xd[at:at + n].contiguous(), make_ctx([(at, n)], ps, n_pages, [table]), cache2, True)
        assert (o.double().cpu() - want[at:at + n]).abs().max() < tol(dtype, scale), f"portion at {at}"
        at += n
    # another call reads the cache this one filled: only its own Q and output projections matter
    other = MIXERS.build(attention_spec(H, nh, nkv, hd, window, rot), dtype, DEV)
    dev_w2, w2 = attention_weights(H, nh, nkv, hd, dtype, seed=40)
    other.bind(dev_w2)
    before = cache.k.clone()
    o = other.forward(xd, make_ctx([(0, T)], ps, n_pages, [table]), cache, False)
    assert torch.equal(cache.k, before), "a reader must not write the cache"
    mixed = dict(w2, **{"k_proj.weight": w["k_proj.weight"], "v_proj.weight": w["v_proj.weight"], "k_norm.weight": w["k_norm.weight"]})
    # (K and V come from the first mixer's input and weights: rebuild them through the plain path)
    Tn = x.shape[0]
    xq = x.to(dtype).double()
    q = plain.rms_norm((xq @ w2["q_proj.weight"].T).view(Tn, nh, hd), w2["q_norm.weight"], 1e-5)
    k = plain.rms_norm((xq @ w["k_proj.weight"].T).view(Tn, nkv, hd), w["k_norm.weight"], 1e-5)
    v = (xq @ w["v_proj.weight"].T).view(Tn, nkv, hd)
    pos = torch.arange(Tn)
    q, k = plain.rope_neox(q, pos, 10000.0, rot), plain.rope_neox(k, pos, 10000.0, rot)
    want2 = plain.attention(q, k, v, 1.0 / math.sqrt(hd), window).reshape(Tn, nh * hd) @ w2["o_proj.weight"].T
    assert (o.double().cpu() - want2).abs().max() < tol(dtype, want2.abs().max().item()) * 2


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_mixer_without_norm_or_positions_and_with_biases(dtype):
    H, nh, nkv, hd, ps = 64, 4, 2, 32, 8
    T = 19
    part = MIXERS.build(attention_spec(H, nh, nkv, hd, qk_norm=False, position="none"), dtype, DEV)
    dev_w, w = attention_weights(H, nh, nkv, hd, dtype, seed=50)
    bias = {"q": rnd(nh * hd, seed=60) * 0.3, "k": rnd(nkv * hd, seed=61) * 0.3, "v": rnd(nkv * hd, seed=62) * 0.3, "o": rnd(H, seed=63) * 0.3}
    for n in ("q_norm.weight", "k_norm.weight"):
        dev_w.pop(n)
    dev_w.update({"q_proj.bias": bias["q"].to(DEV), "k_proj.bias": bias["k"].to(DEV), "v_proj.bias": bias["v"].to(DEV), "o_proj.bias": bias["o"].to(DEV)})
    part.bind(dev_w)
    x = rnd(T, H, seed=70)
    want = plain_attention_mixer(x.to(dtype).double(), w, nh, nkv, hd, None, None, qk_norm=False, position="none",
                                 bias={k: v.double() for k, v in bias.items()})
    cache = KVView(0, torch.zeros(4, nkv, ps, hd, dtype=dtype, device=DEV), torch.zeros(4, nkv, ps, hd, dtype=dtype, device=DEV))
    out = part.forward(stored(x, dtype), make_ctx([(0, T)], ps, 4, [[2, 0, 3]]), cache, True)
    assert (out.double().cpu() - want).abs().max() < tol(dtype, want.abs().max().item())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,F,N", [(80, 112, 7), (96, 160, 70), (128, 256, 1)])
def test_gated_mlp_part(dtype, H, F, N):
    part = FEED_FORWARDS.build(PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": F, "activation": "silu"}), dtype, DEV)
    assert {k: v.shape for k, v in part.tensors().items()} == {"gate_proj.weight": (F, H), "up_proj.weight": (F, H), "down_proj.weight": (H, F)}
    raw = {"gate_proj.weight": rnd(F, H, seed=1, std=0.2), "up_proj.weight": rnd(F, H, seed=2, std=0.2), "down_proj.weight": rnd(H, F, seed=3, std=0.2)}
    part.bind({k: stored(v, dtype) for k, v in raw.items()})
    x = rnd(N, H, seed=4)
    w = {k: v.to(dtype).double() for k, v in raw.items()}
    want = plain.gated_mlp(x.to(dtype).double(), w["gate_proj.weight"], w["up_proj.weight"], w["down_proj.weight"])
    out = part.forward(stored(x, dtype), make_ctx([(0, N)], 8, 16, [list(range(16))]))
    assert (out.double().cpu() - want).abs().max() < tol(dtype, want.abs().max().item()) * 2
    with pytest.raises(ValueError, match="activation"):
        FEED_FORWARDS.build(PartSpec("gated_mlp", {"hidden_size": 8, "intermediate_size": 8, "activation": "gelu"}), dtype, DEV)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    V, H = 311, 80
    emb = EMBEDDINGS.build(PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H}), dtype, DEV)
    table = rnd(V, H, seed=1)
    emb.bind({"weight": stored(table, dtype)})
    ctx = make_ctx([(0, 4)], 8, 2, [[0]])
    toks = torch.tensor([0, 310, 7, 7], dtype=torch.int32, device=DEV)
    x0 = emb.forward(toks, ctx)
    assert x0.dtype == torch.float32 and torch.equal(x0.cpu(), table.to(dtype).float()[[0, 310, 7, 7]])
    head = HEADS.build(PartSpec("lm_head", {"hidden_size": H, "vocab_size": V, "tied": False}), dtype, DEV)
    wh = rnd(V, H, seed=2, std=0.2)
    head.bind({"weight": stored(wh, dtype)})
    x = rnd(4, H, seed=3)
    logits = head.forward(stored(x, dtype), ctx)
    want = x.to(dtype).double() @ wh.to(dtype).double().T
    assert logits.dtype == torch.float32 and (logits.double().cpu() - want).abs().max() < tol(dtype, want.abs().max().item())
    tied = HEADS.build(PartSpec("lm_head", {"hidden_size": H, "vocab_size": V, "tied": True}), dtype, DEV)
    assert tied.tensors() == {}
    tied.bind({})
    tied.tie(emb.weight)
    want = x.to(dtype).double() @ table.to(dtype).double().T
    assert (tied.forward(stored(x, dtype), ctx).double().cpu() - want).abs().max() < tol(dtype, want.abs().max().item())


@pytest.mark.parametrize("dtype", DTYPES)
def test_block_arrangement_and_row_selection(dtype):
    H, nh, nkv, hd, F, ps, T = 64, 4, 2, 16, 96, 8, 21
    norm = PartSpec("rms_norm", {"size": H, "eps": 1e-5})
    spec = LayerSpec(mixer=attention_spec(H, nh, nkv, hd), feed_forward=PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": F}),
                     mixer_norm=norm, feed_forward_norm=norm)
    blk = BLOCKS["pre_norm_residual"](spec, dtype, DEV)
    assert [s for s, _ in blk.parts()] == ["mixer_norm", "mixer", "feed_forward_norm", "feed_forward"]
    dev_w, w = attention_weights(H, nh, nkv, hd, dtype, seed=5)
    blk.mixer.bind(dev_w)
    n1, n2 = rnd(H, seed=6) * 0.1 + 1, rnd(H, seed=7) * 0.1 + 1
    blk.mixer_norm.bind({"weight": n1.to(DEV)})
    blk.feed_forward_norm.bind({"weight": n2.to(DEV)})
    raw = {"gate_proj.weight": rnd(F, H, seed=8, std=0.2), "up_proj.weight": rnd(F, H, seed=9, std=0.2), "down_proj.weight": rnd(H, F, seed=10, std=0.2)}
    blk.feed_forward.bind({k: stored(v, dtype) for k, v in raw.items()})
    fw = {k: v.to(dtype).double() for k, v in raw.items()}
    x0 = rnd(T, H, seed=11)
    d0 = rnd(T, H, seed=12) * 0.5
    # plain: x = x0 + d0; x += mixer(norm(x)); returns (x, ffn(norm(x)))
    x = x0.double() + d0.to(dtype).double()
    x = x + plain_attention_mixer(plain.rms_norm(x, n1.double(), 1e-5), w, nh, nkv, hd, None, hd)
    want_delta = plain.gated_mlp(plain.rms_norm(x, n2.double(), 1e-5), fw["gate_proj.weight"], fw["up_proj.weight"], fw["down_proj.weight"])
    cache = KVView(0, torch.zeros(4, nkv, ps, hd, dtype=dtype, device=DEV), torch.zeros(4, nkv, ps, hd, dtype=dtype, device=DEV))
    rows = [20, 3]
    ctx = make_ctx([(0, T)], ps, 4, [[1, 3, 0]], rows=rows)
    res, delta = blk.forward(x0.to(DEV), stored(d0, dtype), ctx, cache, True, ctx.out_rows)
    assert res.shape == (2, H) and delta.shape == (2, H) and res.dtype == torch.float32
    t = tol(dtype, max(x.abs().max().item(), want_delta.abs().max().item())) * 3
    assert (res.double().cpu() - x[rows]).abs().max() < t
    assert (delta.double().cpu() - want_delta[rows]).abs().max() < t
