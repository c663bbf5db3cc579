"""Each CUDA kernel alone against a plain float64 reference, at sizes other than the engine's
(odd widths, head sizes in steps of 16, page sizes that are no power of two)."""
import math

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DT = [torch.float32, torch.bfloat16]


def K():
    from iian_b200.ops.cuda_backend import CudaKernels
    return CudaKernels()


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def rnd(*shape, dtype=torch.float32, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype).cuda()


@pytest.mark.parametrize("dtype", DT)
def test_embedding(dtype):
    table = rnd(77, 50, dtype=dtype)
    tokens = torch.tensor([0, 76, 5, 5, 33], dtype=torch.int32).cuda()
    out = torch.empty(5, 50, dtype=torch.float32).cuda()
    K().embedding(table, tokens, out)
    assert torch.equal(out.cpu(), table.float().cpu()[tokens.long().cpu()])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("H", [203, 1024, 4100])
def test_add_rms_norm(dtype, H):
    res = rnd(5, H, seed=1)
    delta = rnd(5, H, dtype=dtype, seed=2)
    w = rnd(H, seed=3) * 0.1 + 1
    out = torch.empty(5, H, dtype=dtype).cuda()
    res0 = res.clone()
    K().add_rms_norm(res, delta, w, 1e-5, out)
    want_res = res0.double().cpu() + delta.double().cpu()
    assert (res.double().cpu() - want_res).abs().max() < 1e-6
    want = plain.rms_norm(want_res, w.double().cpu(), 1e-5)
    assert (out.double().cpu() - want).abs().max() < tol(dtype, want.abs().max().item())
    # without delta the residual is left alone
    res1 = res.clone()
    K().add_rms_norm(res, None, w, 1e-5, out)
    assert torch.equal(res, res1)


@pytest.mark.parametrize("dtype", DT)
def test_rms_norm_and_swiglu_and_gather_and_bias(dtype):
    x = rnd(7, 130, dtype=dtype, seed=4)
    w = rnd(130, seed=5) * 0.1 + 1
    out = torch.empty_like(x)
    K().rms_norm(x, w, 1e-6, out)
    want = plain.rms_norm(x.double().cpu(), w.double().cpu(), 1e-6)
    assert (out.double().cpu() - want).abs().max() < tol(dtype, want.abs().max().item())

    gu = rnd(3, 2 * 77, dtype=dtype, seed=6, std=2.0)
    act = torch.empty(3, 77, dtype=dtype).cuda()
    K().swiglu(gu, act)
    g, u = gu.double().cpu()[:, :77], gu.double().cpu()[:, 77:]
    want = plain.silu(g) * u
    assert (act.double().cpu() - want).abs().max() < tol(dtype, want.abs().max().item())

    gu8 = rnd(5, 2 * 80, dtype=dtype, seed=16, std=2.0)
    act8 = torch.empty(5, 80, dtype=dtype).cuda()
    K().swiglu(gu8, act8, interleave=8)
    v = gu8.double().cpu().view(5, 10, 2, 8)
    want = plain.silu(v[:, :, 0].reshape(5, 80)) * v[:, :, 1].reshape(5, 80)
    assert (act8.double().cpu() - want).abs().max() < tol(dtype, want.abs().max().item())

    rows = torch.tensor([6, 0, 3], dtype=torch.int32).cuda()
    sel = torch.empty(3, 130, dtype=dtype).cuda()
    K().gather_rows(x, rows, sel)
    assert torch.equal(sel, x[rows.long()])

    b = rnd(130, seed=7)
    y = x.clone()
    K().add_bias(y, b)
    assert (y.double().cpu() - (x.double().cpu() + b.double().cpu())).abs().max() < tol(dtype, 4.0)


@pytest.mark.parametrize("xd,wd,od", [(torch.float32, torch.float32, torch.float32),
                                       (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                       (torch.bfloat16, torch.bfloat16, torch.float32),
                                       (torch.bfloat16, torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("N,M,K_", [(1, 70, 45), (37, 70, 45), (130, 257, 96)])
def test_gemm_simt(xd, wd, od, N, M, K_):
    x = rnd(N, K_, dtype=xd, seed=8)
    w = rnd(M, K_, dtype=wd, seed=9)
    out = torch.empty(N, M, dtype=od).cuda()
    K().gemm_simt(x, w, out)
    want = x.double().cpu() @ w.double().cpu().T
    assert (out.double().cpu() - want).abs().max() < tol(od, want.abs().max().item())


def test_gemm_simt_rows_do_not_depend_on_the_batch():
    x = rnd(40, 333, seed=10)
    w = rnd(90, 333, seed=11)
    full = torch.empty(40, 90).cuda()
    K().gemm_simt(x, w, full)
    one = torch.empty(1, 90).cuda()
    for r in (0, 17, 39):
        K().gemm_simt(x[r:r + 1].contiguous(), w, one)
        assert torch.equal(one[0], full[r])


def _fill_cache(k_all, v_all, tables, ps, nkv, hd, n_pages, dtype):
    k_cache = torch.zeros(n_pages, nkv, ps, hd, dtype=dtype)
    v_cache = torch.zeros(n_pages, nkv, ps, hd, dtype=dtype)
    for s, table in enumerate(tables):
        for j in range(k_all[s].shape[0]):
            pg = table[j // ps]
            if pg < 0:
                continue
            k_cache[pg, :, j % ps] = k_all[s][j].to(dtype)
            v_cache[pg, :, j % ps] = v_all[s][j].to(dtype)
    return k_cache.cuda(), v_cache.cuda()


class Meta:
    pass


def attention_case(dtype, nh, nkv, hd, ps, ctx_lens, q_lens, window, seed=0, standout=False):
    """Random sequences in a shuffled paged cache; returns what the kernel needs and the plain result."""
    g = torch.Generator().manual_seed(seed)
    S = len(ctx_lens)
    n_blocks = [math.ceil(c / ps) for c in ctx_lens]
    n_pages = sum(n_blocks) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    tables, at = [], 0
    for nb in n_blocks:
        tables.append(perm[at:at + nb])
        at += nb
    ks = [torch.randn(c, nkv, hd, generator=g) for c in ctx_lens]
    vs = [torch.randn(c, nkv, hd, generator=g) for c in ctx_lens]
    qs = [torch.randn(c, nh, hd, generator=g) for c in ctx_lens]
    if standout:        # one far key among hundreds decides the output of the last query
        for s in range(S):
            far = min(3, ctx_lens[s] - 1) if not window else max(0, ctx_lens[s] - window)      # window: the oldest key still visible
            if standout == "outside":       # ... or would decide it, if a window one key too long let it in
                if not window or ctx_lens[s] - window - 1 < 0:
                    continue
                far = ctx_lens[s] - window - 1
            qs[s][-1] *= 4.0
            ks[s][far] = qs[s][-1][::nh // nkv][:nkv] * 1.0
            if standout == "outside":
                vs[s][far] = 25.0           # seen by mistake, it would move the output far beyond any tolerance
    ks = [k.to(dtype).float() for k in ks]
    vs = [v.to(dtype).float() for v in vs]
    qs = [q.to(dtype).float() for q in qs]
    k_cache, v_cache = _fill_cache(ks, vs, tables, ps, nkv, hd, n_pages, dtype)
    scale = 1.0 / math.sqrt(hd)
    q_rows, pos, seq, want = [], [], [], []
    for s in range(S):
        full = plain.attention(qs[s].double(), ks[s].double(), vs[s].double(), scale, window)
        first = ctx_lens[s] - q_lens[s]
        q_rows.append(qs[s][first:])
        want.append(full[first:].reshape(q_lens[s], nh * hd))
        pos += list(range(first, ctx_lens[s]))
        seq += [s] * q_lens[s]
    maxb = max(n_blocks)
    bt = torch.full((S, maxb), -1, dtype=torch.int32)
    for s, t in enumerate(tables):
        bt[s, :len(t)] = torch.tensor(t, dtype=torch.int32)
    m = Meta()
    m.positions = torch.tensor(pos, dtype=torch.int32).cuda()
    m.seq_of_token = torch.tensor(seq, dtype=torch.int32).cuda()
    m.block_table = bt.cuda()
    m.ctx_len = torch.tensor(ctx_lens, dtype=torch.int32).cuda()
    cu = [0]
    for ql in q_lens:
        cu.append(cu[-1] + ql)
    m.cu_q = torch.tensor(cu, dtype=torch.int32).cuda()
    m.num_seqs, m.num_tokens = S, len(pos)
    m.max_q_len, m.max_ctx = max(q_lens), max(ctx_lens)
    m.decode_only = max(q_lens) == 1
    m.h_q_len, m.h_ctx_len = list(q_lens), list(ctx_lens)
    q = torch.cat(q_rows).to(dtype).cuda().contiguous()
    return q, k_cache, v_cache, m, torch.cat(want), scale


ATT_CASES = [
    # nh, nkv, hd, page, ctx_lens, q_lens, window
    (6, 3, 80, 8, [37, 5, 64], [37, 1, 20], None),
    (4, 4, 16, 16, [33, 1], [2, 1], None),
    (8, 2, 128, 16, [300, 257, 31], [1, 1, 1], None),
    (6, 2, 48, 12, [90, 41], [13, 41], 20),
    (5, 1, 96, 16, [130], [130], 33),
    (8, 2, 64, 16, [200, 77], [64, 77], None),
]


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("case", ATT_CASES)
@pytest.mark.parametrize("standout", [False, True, "outside"])
def test_paged_attention_generic(dtype, case, standout):
    nh, nkv, hd, ps, ctx_lens, q_lens, window = case
    if standout == "outside" and not window:
        pytest.skip("no window")
    q, kc, vc, m, want, scale = attention_case(dtype, nh, nkv, hd, ps, ctx_lens, q_lens, window, seed=3, standout=standout)
    out = torch.empty(q.shape[0], nh * hd, dtype=dtype).cuda()
    K().paged_attention_generic(q, kc, vc, out, m, num_heads=nh, num_kv_heads=nkv, head_dim=hd, scale=scale, window=window)
    err = (out.double().cpu() - want).abs().max().item()
    assert err < tol(dtype, max(1.0, want.abs().max().item())), err


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("use_table", [False, True])
@pytest.mark.parametrize("nh,nkv,hd,rot,style,ps", [(6, 2, 48, 48, 0, 8), (4, 4, 16, 8, 0, 16), (3, 1, 80, 80, 1, 12),
                                                      (8, 2, 128, 128, 0, 16), (2, 1, 256, 256, 0, 16)])
def test_qk_norm_rope_store(dtype, use_table, nh, nkv, hd, rot, style, ps):
    N, n_pages = 11, 9
    width = (nh + 2 * nkv) * hd
    qkv = rnd(N, width, dtype=dtype, seed=12)
    qw, kw = rnd(hd, seed=13) * 0.1 + 1, rnd(hd, seed=14) * 0.1 + 1
    base = 10000.0
    inv_freq = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot).float().cuda()
    positions = torch.tensor([0, 1, 2, 3, 100, 101, 7, 8, 9, 4000, 17], dtype=torch.int32).cuda()
    g = torch.Generator().manual_seed(15)
    slots_l = torch.randperm(n_pages * ps, generator=g)[:N].tolist()
    slots_l[5] = -1                                   # a padding token stores nothing
    slots = torch.tensor(slots_l, dtype=torch.int32).cuda()
    kc = torch.zeros(n_pages, nkv, ps, hd, dtype=dtype).cuda()
    vc = torch.zeros_like(kc)
    q_out = torch.empty(N, nh, hd, dtype=dtype).cuda()
    eps = 1e-5
    table = None
    if use_table:      # cos / sin from the per-step table (and, where the shape allows, the vectorised kernel)
        table = torch.empty(N, rot // 2, 2, dtype=torch.float32).cuda()
        K().rotary_table(inv_freq, positions, rot // 2, table)
        th = positions.cpu().float()[:, None] * inv_freq.cpu()[None, :]
        assert (table[..., 0].cpu() - torch.cos(th.double()).float()).abs().max() < 2e-6
    K().qk_norm_rope_store(qkv, q_out, kc, vc, num_heads=nh, num_kv_heads=nkv, head_dim=hd, q_weight=qw, k_weight=kw,
                           eps=eps, inv_freq=inv_freq, rot_dim=rot, rope_style=style, positions=positions, slots=slots,
                           write_kv=True, table=table)
    x = qkv.double().cpu().view(N, nh + 2 * nkv, hd)
    q, k, v = x[:, :nh], x[:, nh:nh + nkv], x[:, nh + nkv:]
    q = plain.rms_norm(q, qw.double().cpu(), eps)
    k = plain.rms_norm(k, kw.double().cpu(), eps)
    pos = positions.cpu()
    if style == 0:
        q, k = plain.rope_neox(q, pos, base, rot), plain.rope_neox(k, pos, base, rot)
    else:   # interleaved pairs (2j, 2j+1): permute into NEOX order, rotate, permute back
        idx = torch.cat([torch.arange(0, rot, 2), torch.arange(1, rot, 2)])
        inv = torch.argsort(idx)
        def inter(t):
            r = plain.rope_neox(t[..., idx].contiguous(), pos, base, rot)
            return r[..., inv]
        q, k = inter(q), inter(k)
    t = tol(dtype, 4.0)
    assert (q_out.double().cpu() - q).abs().max() < t
    for i in range(N):
        s = slots_l[i]
        if s < 0:
            continue
        assert (kc[s // ps, :, s % ps].double().cpu() - k[i]).abs().max() < t
        assert (vc[s // ps, :, s % ps].double().cpu() - v[i]).abs().max() < t
    used = {s for s in slots_l if s >= 0}
    flat_k = kc.float().cpu().permute(0, 2, 1, 3).reshape(n_pages * ps, -1)
    for cell in range(n_pages * ps):
        if cell not in used:
            assert flat_k[cell].abs().max() == 0, "a cell no token owns was written"


def test_argmax_ties_go_to_the_lowest_id():
    logits = torch.full((3, 1001), -1.0)
    logits[0, [7, 500, 999]] = 5.0
    logits[1, 1000] = 2.0
    logits[2] = 0.0
    out = torch.empty(3, dtype=torch.int32).cuda()
    K().argmax(logits.cuda(), out)
    assert out.tolist() == [7, 1000, 0]


@pytest.mark.parametrize("V", [503, 151936])
@pytest.mark.parametrize("params", [(0.7, 0, 1.0, 0.0), (1.3, 5, 1.0, 0.0), (1.0, 0, 0.9, 0.0), (0.8, 0, 1.0, 0.05),
                                    (1.0, 50, 0.8, 0.01), (0.0, 0, 1.0, 0.0)])
def test_sample_matches_the_plain_walk(V, params):
    T, top_k, top_p, min_p = params
    R = 6
    g = torch.Generator().manual_seed(V + int(T * 10) + top_k)
    logits = torch.randn(R, V, generator=g) * 2.5
    logits[2, 10] = logits[2, 400] = logits[2].max() + 0.5          # a tie at the top
    u = torch.rand(R, generator=g)
    out = torch.empty(R, dtype=torch.int32).cuda()
    f = lambda v, dt: torch.full((R,), v, dtype=dt).cuda()
    K().sample(logits.cuda(), f(T, torch.float32), f(top_k, torch.int32), f(top_p, torch.float32),
               f(min_p, torch.float32), u.cuda(), out)
    got = out.tolist()
    for r in range(R):
        if T < 1e-5:
            assert got[r] == plain.argmax(logits[r])
            continue
        probs = plain.candidate_probs(logits[r], T, top_k, top_p, min_p)
        assert probs[got[r]] > 0, f"row {r}: token {got[r]} is outside the candidate set"
        # the token's interval of the running mass must contain u * total (up to float32 rounding of the sums)
        cum = torch.cumsum(probs, 0)
        total = cum[-1].item()
        lo = cum[got[r]].item() - probs[got[r]].item()
        hi = cum[got[r]].item()
        target = u[r].item() * total
        slack = 1e-5 * total
        assert lo - slack <= target <= hi + slack, f"row {r}: u*total={target} not in [{lo}, {hi}]"


@pytest.mark.parametrize("od", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,M,K_", [(1, 70, 64), (3, 16, 32), (8, 257, 96), (9, 100, 160), (17, 48, 4096), (33, 130, 320),
                                    (64, 1000, 1024), (2, 4096, 12288)])
def test_gemm_skinny(od, B, M, K_):
    x = rnd(B, K_, dtype=torch.bfloat16, seed=20)
    w = rnd(M, K_, dtype=torch.bfloat16, seed=21)
    out = torch.full((B, M), float("nan"), dtype=od).cuda()
    K().gemm_skinny(x, w, out)
    want = x.double().cpu() @ w.double().cpu().T
    assert (out.double().cpu() - want).abs().max() < tol(od if od == torch.bfloat16 else torch.float32, want.abs().max().item()) * \
        (1 if od == torch.bfloat16 else 10)


@pytest.mark.parametrize("ksplit", [2, 3, 8])
@pytest.mark.parametrize("B,M,K_", [(1, 70, 512), (8, 257, 4096), (5, 4096, 1024), (33, 100, 2048)])
def test_gemm_skinny_split_k(ksplit, B, M, K_):
    """K cut over several CTAs: the last one to arrive adds the parts in index order, so two runs give the
    same bits, and the counters are left at zero for the next launch."""
    x = rnd(B, K_, dtype=torch.bfloat16, seed=30)
    w = rnd(M, K_, dtype=torch.bfloat16, seed=31)
    want = x.double().cpu() @ w.double().cpu().T
    outs = []
    for _ in range(3):
        out = torch.full((B, M), float("nan"), dtype=torch.float32).cuda()
        K().gemm_skinny(x, w, out, ksplit=ksplit)
        outs.append(out.clone())
    assert (outs[0].double().cpu() - want).abs().max() < 2e-4 * max(1.0, want.abs().max().item())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])


@pytest.mark.parametrize("B,F,K_", [(1, 16, 64), (8, 160, 96), (5, 12288, 4096)])
def test_gemm_skinny_swiglu_epilogue(B, F, K_):
    x = rnd(B, K_, dtype=torch.bfloat16, seed=40)
    wg, wu = rnd(F, K_, dtype=torch.bfloat16, seed=41, std=0.05), rnd(F, K_, dtype=torch.bfloat16, seed=42, std=0.05)
    inter = torch.stack([wg.view(F // 8, 8, K_), wu.view(F // 8, 8, K_)], dim=1).reshape(2 * F, K_).contiguous()
    out = torch.full((B, F), float("nan"), dtype=torch.bfloat16).cuda()
    K().gemm_skinny(x, inter, out, epilogue=1)
    xd = x.double().cpu()
    want = plain.silu(xd @ wg.double().cpu().T) * (xd @ wu.double().cpu().T)
    assert (out.double().cpu() - want).abs().max() < tol(torch.bfloat16, max(1.0, want.abs().max().item()))


def test_gemm_skinny_rows_do_not_depend_on_the_batch():
    """Within the row counts the engine uses it for (up to 8), a row's result is the same bits whatever
    else is in the batch: the split of K over warps and the order of the final sum are fixed."""
    x = rnd(8, 512, dtype=torch.bfloat16, seed=22)
    w = rnd(90, 512, dtype=torch.bfloat16, seed=23)
    full = torch.empty(8, 90, dtype=torch.float32).cuda()
    K().gemm_skinny(x, w, full)
    one = torch.empty(1, 90, dtype=torch.float32).cuda()
    for r in (0, 3, 7):
        K().gemm_skinny(x[r:r + 1].contiguous(), w, one)
        assert torch.equal(one[0], full[r])


@pytest.mark.parametrize("B,H,M2,K_", [(1, 64, 48, 96), (8, 4096, 6144, 4096), (5, 288, 100, 160), (3, 1024, 32, 2048),
                                       (200, 288, 100, 160), (300, 1024, 520, 1096), (129, 4360, 264, 64)])
def test_gemm_skinny_folded_norm(B, H, M2, K_):
    """A product that ends a sub-layer adds to the residual, prepares residual * norm weight and leaves the sums
    of squares in parts; the next product multiplies its rows by rsqrt(mean + eps).  Together they equal the
    residual add, the RMSNorm and the two plain products."""
    from iian_b200.ops.fused import ResidualNorm, RowScale
    k = K()
    eps = 1e-5
    a = rnd(B, K_, dtype=torch.bfloat16, seed=50)
    w1 = rnd(H, K_, dtype=torch.bfloat16, seed=51, std=0.05)
    res0 = rnd(B, H, dtype=torch.float32, seed=52)
    nw = (1 + 0.3 * rnd(H, dtype=torch.float32, seed=53)).contiguous()
    w2 = rnd(M2, H, dtype=torch.bfloat16, seed=54, std=0.05)
    # folded route
    res = res0.clone()
    xt = torch.full((B, H), float("nan"), dtype=torch.bfloat16).cuda()
    partials = torch.full((B, k.norm_parts(w1, B)), float("nan")).cuda()
    k.linear(a, w1, xt, residual_norm=ResidualNorm(res, nw, partials))
    out = torch.full((B, M2), float("nan"), dtype=torch.bfloat16).cuda()
    k.linear(xt, w2, out, row_scale=RowScale(partials, H, eps))
    # plain route, float64 except for the roundings the engine makes
    delta = (a.double().cpu() @ w1.double().cpu().T).to(torch.bfloat16).double()
    want_res = res0.double().cpu() + delta
    assert (res.double().cpu() - want_res).abs().max() < 1e-5 * max(1.0, want_res.abs().max().item()) + \
        tol(torch.bfloat16, delta.abs().max().item())          # one bfloat16 rounding of the product may fall the other way
    assert (partials.double().cpu().sum(1) - (res.double().cpu() ** 2).sum(1)).abs().max() < 1e-4 * (res.double().cpu() ** 2).sum(1).max()
    assert (xt.double().cpu() - res.double().cpu() * nw.double().cpu()).abs().max() < tol(torch.bfloat16, (res.abs().max() * nw.abs().max()).item())
    normed = plain.rms_norm(res.double().cpu(), nw.double().cpu(), eps)
    want = normed @ w2.double().cpu().T
    assert (out.double().cpu() - want).abs().max() < 2 * tol(torch.bfloat16, max(1.0, want.abs().max().item()))
    # and the unfused kernels give the same within the same tolerance
    res_b = res0.clone()
    d = torch.empty(B, H, dtype=torch.bfloat16).cuda()
    k.linear(a, w1, d)
    h = torch.empty(B, H, dtype=torch.bfloat16).cuda()
    k.add_rms_norm(res_b, d, nw, eps, h)
    out_b = torch.empty(B, M2, dtype=torch.bfloat16).cuda()
    k.linear(h, w2, out_b)
    assert torch.equal(res_b, res)          # the residual stream is the same bits on both routes
    assert (out.float() - out_b.float()).abs().max() < 2 * tol(torch.bfloat16, max(1.0, want.abs().max().item()))


@pytest.mark.parametrize("B,H,F", [(6, 512, 160), (150, 520, 168), (260, 1024, 2304)])
def test_gemm_skinny_row_scale_with_swiglu(B, H, F):
    from iian_b200.ops.fused import RowScale
    k = K()
    x = rnd(B, H, dtype=torch.bfloat16, seed=60)
    wg, wu = rnd(F, H, dtype=torch.bfloat16, seed=61, std=0.05), rnd(F, H, dtype=torch.bfloat16, seed=62, std=0.05)
    inter = torch.stack([wg.view(F // 8, 8, H), wu.view(F // 8, 8, H)], dim=1).reshape(2 * F, H).contiguous()
    partials = (rnd(B, 7, dtype=torch.float32, seed=63).abs() * 100).contiguous()
    out = torch.full((B, F), float("nan"), dtype=torch.bfloat16).cuda()
    k.linear_swiglu(x, inter, out, row_scale=RowScale(partials, H, 1e-6))
    rs = 1.0 / torch.sqrt(partials.double().cpu().sum(1) / H + 1e-6)
    xd = x.double().cpu()
    want = plain.silu((xd @ wg.double().cpu().T) * rs[:, None]) * ((xd @ wu.double().cpu().T) * rs[:, None])
    assert (out.double().cpu() - want).abs().max() < tol(torch.bfloat16, max(1.0, want.abs().max().item()))


def test_gemm_skinny_refuses_what_it_cannot_do():
    from iian_b200.ops.cuda_backend import KernelError
    x = rnd(2, 40, dtype=torch.bfloat16)
    w = rnd(8, 40, dtype=torch.bfloat16)
    with pytest.raises(KernelError):
        K().gemm_skinny(x, w, torch.empty(2, 8, dtype=torch.bfloat16).cuda())      # K not a multiple of 32
    x = rnd(65, 64, dtype=torch.bfloat16)
    w = rnd(8, 64, dtype=torch.bfloat16)
    with pytest.raises(KernelError):
        K().gemm_skinny(x, w, torch.empty(65, 8, dtype=torch.bfloat16).cuda())     # more than 64 rows


FUSED_DECODE_CASES = [
    # nh, nkv, hd, page, ctx_lens (one new token each), window, qk_norm, rotate
    (8, 2, 128, 16, [300, 257, 31, 1], None, True, True),
    (32, 8, 128, 16, [1152, 64, 65], None, True, True),
    (6, 3, 64, 8, [37, 5, 64, 129], None, True, True),
    (16, 1, 64, 16, [500, 16], 100, False, True),
    (4, 4, 128, 32, [2100, 33], None, True, False),
    (12, 4, 128, 12, [130, 90, 12, 13], 33, False, False),
    # 32 and more (sequence, KV head) pairs: the form that fetches its K/V tiles by TMA
    (32, 8, 128, 16, [1152, 64, 65, 300, 17], None, True, True),
    (16, 8, 128, 64, [200, 130, 64, 1], 100, False, True),
    (8, 4, 128, 8, [90, 500, 33, 8, 1, 129, 64, 77], None, True, False),
]


@pytest.mark.parametrize("case", FUSED_DECODE_CASES)
@pytest.mark.parametrize("mode", ["auto", "one", "cluster3", "cluster8", "cluster16", "scratch5"])
def test_attention_decode_fused(case, mode):
    """Norm, rotation, cache write and attention in one launch: the same bits as the two-kernel route (same
    arithmetic in the same order), the same cache contents, and right against the plain formulas."""
    fused_decode_check(case, mode)


def fused_decode_check(case, mode, cache_exact=True):
    nh, nkv, hd, ps, ctx_lens, window, qk_norm, rotate = case
    S = len(ctx_lens)
    bf = torch.bfloat16
    # the cache holds every key but the newest; the step brings one token per sequence
    q, kc, vc, m, _, scale = attention_case(bf, nh, nkv, hd, ps, ctx_lens, [1] * S, window, seed=9)
    g = torch.Generator().manual_seed(77)
    qkv = (torch.randn(S, (nh + 2 * nkv) * hd, generator=g) * 1.5).to(bf).cuda()
    qw = (1 + 0.2 * torch.randn(hd, generator=g)).cuda() if qk_norm else None
    kw_ = (1 + 0.2 * torch.randn(hd, generator=g)).cuda() if qk_norm else None
    inv = torch.pow(torch.tensor(1e4, dtype=torch.float64), -2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd).float().cuda()
    table = None
    if rotate:
        table = torch.empty(S, hd // 2, 2).cuda()
        K().rotary_table(inv, m.positions, hd // 2, table)
    slots = torch.tensor([int(m.block_table[i, (c - 1) // ps]) * ps + (c - 1) % ps for i, c in enumerate(ctx_lens)],
                         dtype=torch.int32).cuda()
    # route A: two kernels
    kc_a, vc_a = kc.clone(), vc.clone()
    qa = torch.empty(S, nh, hd, dtype=bf).cuda()
    K().qk_norm_rope_store(qkv, qa, kc_a, vc_a, num_heads=nh, num_kv_heads=nkv, head_dim=hd, q_weight=qw, k_weight=kw_,
                           eps=1e-6, inv_freq=inv if rotate else None, rot_dim=hd if rotate else 0, rope_style=0,
                           positions=m.positions, slots=slots, write_kv=True, **({"table": table} if rotate else {}))
    out_a = torch.empty(S, nh * hd, dtype=bf).cuda()
    K().paged_attention_mma(qa, kc_a, vc_a, out_a, m, num_heads=nh, num_kv_heads=nkv, head_dim=hd, scale=scale, window=window,
                            n_split=1, small_tiles=True)
    # route B: fused
    kw = {"auto": {}, "one": dict(n_split=1), "cluster3": dict(n_split=3, cluster=True), "cluster8": dict(n_split=8, cluster=True),
          "cluster16": dict(n_split=16, cluster=True),
          "scratch5": dict(n_split=5, cluster=False)}[mode]
    for _ in range(2):       # twice: the scratch route leaves its counters at zero
        kc_b, vc_b = kc.clone(), vc.clone()
        out_b = torch.full((S, nh * hd), float("nan"), dtype=bf).cuda()
        K().attention_decode_fused(qkv, kc_b, vc_b, out_b, m, num_heads=nh, num_kv_heads=nkv, head_dim=hd, scale=scale,
                                   window=window, q_weight=qw, k_weight=kw_, eps=1e-6, table=table, slots=slots, write_kv=True, **kw)
        if cache_exact:
            assert torch.equal(kc_a, kc_b) and torch.equal(vc_a, vc_b)
            if kw.get("n_split") == 1:
                assert torch.equal(out_a, out_b)
        else:
            assert torch.equal(vc_a, vc_b)
            assert (kc_a.float() - kc_b.float()).abs().max() <= 2.0 ** -7 * kc_a.float().abs().max()
        assert (out_a.float() - out_b.float()).abs().max() < tol(bf, max(1.0, out_a.float().abs().max().item()))
    # against the plain formulas in float64, from the caches route A left
    x = qkv.double().cpu().view(S, nh + 2 * nkv, hd)
    for i, c in enumerate(ctx_lens):
        qh = x[i, :nh]
        if qk_norm:
            qh = plain.rms_norm(qh, qw.double().cpu(), 1e-6)
        if rotate:
            qh = plain.rope_neox(qh.unsqueeze(0), torch.tensor([c - 1]), 1e4, hd).squeeze(0)
        qh = qh.to(bf).double()
        cells = [int(m.block_table[i, j // ps]) * ps + j % ps for j in range(c)]
        kk = torch.stack([kc_a.view(-1, nkv, ps, hd)[cell // ps, :, cell % ps] for cell in cells]).double().cpu()
        vv = torch.stack([vc_a.view(-1, nkv, ps, hd)[cell // ps, :, cell % ps] for cell in cells]).double().cpu()
        qfull = torch.zeros(c, nh, hd, dtype=torch.float64)
        qfull[-1] = qh
        want = plain.attention(qfull, kk, vv, scale, window)[-1].reshape(nh * hd)
        assert (out_b[i].double().cpu() - want).abs().max() < tol(bf, max(1.0, want.abs().max().item()))
    return out_b, kc_b, vc_b


MMA_CASES = [
    # nh, nkv, hd, page, ctx_lens, q_lens, window
    (8, 2, 128, 16, [300, 257, 31], [1, 1, 1], None),
    (8, 2, 64, 16, [200, 77], [64, 77], None),
    (32, 8, 128, 16, [1152], [1], None),
    (6, 3, 64, 8, [37, 5, 64, 1], [37, 1, 20, 1], None),
    (4, 4, 128, 12, [130, 90], [130, 13], 33),
    (12, 2, 128, 16, [700, 65, 64, 63], [300, 65, 1, 63], None),
    (6, 1, 64, 16, [500], [1], 100),
    (16, 2, 128, 32, [2100], [2048], None),
    (8, 8, 128, 8, [700, 129], [257, 129], 200),
    (24, 4, 128, 64, [1000, 300, 40], [130, 300, 7], None),
    # decode steps of 32 and more (sequence, KV head) pairs: K/V tiles by TMA
    (32, 8, 128, 16, [1152, 700, 64, 65], [1, 1, 1, 1], None),
    (8, 8, 128, 8, [300, 129, 40, 33], [1, 1, 1, 1], 200),
    (16, 4, 128, 32, [2100, 64, 31, 500, 96, 97, 1000, 5], [1] * 8, None),
]


@pytest.mark.parametrize("case", MMA_CASES)
@pytest.mark.parametrize("standout", [False, True, "outside"])
@pytest.mark.parametrize("mode", ["auto", "split5", "big_tiles", "cluster2", "cluster4", "cluster8", "cluster16", "split4_scratch", "tc"])
def test_paged_attention_mma(case, standout, mode):
    nh, nkv, hd, ps, ctx_lens, q_lens, window = case
    dtype = torch.bfloat16
    if standout == "outside" and not window:
        pytest.skip("no window")
    q, kc, vc, m, want, scale = attention_case(dtype, nh, nkv, hd, ps, ctx_lens, q_lens, window, seed=5, standout=standout)
    out = torch.full((q.shape[0], nh * hd), float("nan"), dtype=dtype).cuda()
    kw = {}
    if mode == "tc":                      # tcgen05 + TMA: head size 128, pages that are whole swizzle atoms
        if hd != 128 or ps % 8 != 0 or 128 % ps != 0:
            pytest.skip("outside the tcgen05 attention kernel's range")
        K().paged_attention_tc(q, kc, vc, out, m, num_heads=nh, num_kv_heads=nkv, head_dim=hd, scale=scale, window=window)
        K().tcgen05_check(q.device)
        err = (out.double().cpu() - want).abs().max().item()
        assert err < tol(dtype, max(1.0, want.abs().max().item())), err
        return
    if mode == "split5":
        kw = dict(n_split=5, small_tiles=True)
    elif mode == "big_tiles":
        kw = dict(n_split=1, small_tiles=False)
    elif mode.startswith("cluster"):      # the parts of a row tile merge through a cluster's shared memory
        kw = dict(n_split=int(mode[7:]), small_tiles=True, cluster=True)
    elif mode == "split4_scratch":        # the same split merged through scratch memory by the last CTA
        kw = dict(n_split=4, small_tiles=True, cluster=False)
    K().paged_attention_mma(q, kc, vc, out, m, num_heads=nh, num_kv_heads=nkv, head_dim=hd, scale=scale, window=window, **kw)
    err = (out.double().cpu() - want).abs().max().item()
    assert err < tol(dtype, max(1.0, want.abs().max().item())), err
