"""The product whose weights stream through shared memory by bulk asynchronous copies (csrc/gemm_stream.cu) against the
one that loads them into registers (csrc/gemm_skinny.cu): the same split of K over the warps and the same order of the
final sum, so every form must give the same bits -- plain, with the SwiGLU epilogue, with the residual-and-norm
epilogue, with a factor per row -- at sizes that are no multiple of a stage, a row block or the ring, and against
float64."""
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


def rnd(*shape, dtype=torch.float32, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype).cuda()


def K():
    from iian_b200.ops.cuda_backend import CudaKernels
    return CudaKernels()


SIZES = [(1, 16, 64), (8, 70, 96), (3, 257, 512), (8, 4096, 4096), (5, 100, 1056), (2, 6144, 1024), (7, 5000, 12288), (8, 40000, 160)]


@pytest.mark.parametrize("stages", [6, 12])
@pytest.mark.parametrize("od", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,M,K_", SIZES)
def test_plain_product_equals_the_register_form(stages, od, B, M, K_):
    k = K()
    type(k).STREAM_STAGES = stages
    x, w = rnd(B, K_, dtype=torch.bfloat16, seed=20), rnd(M, K_, dtype=torch.bfloat16, seed=21, std=0.05)
    a = torch.full((B, M), float("nan"), dtype=od).cuda()
    b = torch.full((B, M), float("nan"), dtype=od).cuda()
    k.gemm_skinny(x, w, a)
    k._gemm_stream(x, w, b, B, M, K_, 0)
    k.tcgen05_check(x.device)
    assert torch.equal(a, b)
    want = x.double().cpu() @ w.double().cpu().T
    assert (b.double().cpu() - want).abs().max() < 2e-2 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("B,F,K_", [(1, 16, 64), (8, 160, 96), (5, 12288, 4096), (3, 1000, 1056)])
def test_swiglu_epilogue_equals_the_register_form(B, F, K_):
    k = K()
    x = rnd(B, K_, dtype=torch.bfloat16, seed=40)
    wg, wu = rnd(F, K_, dtype=torch.bfloat16, seed=41, std=0.05), rnd(F, K_, dtype=torch.bfloat16, seed=42, std=0.05)
    inter = torch.stack([wg.view(F // 8, 8, K_), wu.view(F // 8, 8, K_)], dim=1).reshape(2 * F, K_).contiguous()
    a = torch.full((B, F), float("nan"), dtype=torch.bfloat16).cuda()
    b = torch.full((B, F), float("nan"), dtype=torch.bfloat16).cuda()
    k.gemm_skinny(x, inter, a, epilogue=1)
    k._gemm_stream(x, inter, b, B, 2 * F, K_, 1)
    k.tcgen05_check(x.device)
    assert torch.equal(a, b)
    xd = x.double().cpu()
    want = plain.silu(xd @ wg.double().cpu().T) * (xd @ wu.double().cpu().T)
    assert (b.double().cpu() - want).abs().max() < 2e-2 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("B,H,M2,K_", [(1, 64, 48, 96), (8, 4096, 6144, 4096), (5, 288, 100, 160), (3, 1024, 32, 2048)])
def test_folded_norm_equals_the_register_form(B, H, M2, K_, monkeypatch):
    """The residual-and-norm epilogue and the factor per row, through ``linear`` as the parts call it."""
    from iian_b200.ops.cuda_backend import CudaKernels
    from iian_b200.ops.fused import ResidualNorm, RowScale
    k = K()
    a = rnd(B, K_, dtype=torch.bfloat16, seed=50)
    w1 = rnd(H, K_, dtype=torch.bfloat16, seed=51, std=0.05)
    res0 = rnd(B, H, dtype=torch.float32, seed=52)
    nw = (1 + 0.3 * rnd(H, dtype=torch.float32, seed=53)).contiguous()
    w2 = rnd(M2, H, dtype=torch.bfloat16, seed=54, std=0.05)
    got = []
    for stream in (False, True):
        monkeypatch.setattr(CudaKernels, "STREAM_PRODUCT", stream)
        res = res0.clone()
        xt = torch.full((B, H), float("nan"), dtype=torch.bfloat16).cuda()
        partials = torch.full((B, k.norm_parts(w1, B)), float("nan")).cuda()
        k.linear(a, w1, xt, residual_norm=ResidualNorm(res, nw, partials))
        out = torch.full((B, M2), float("nan"), dtype=torch.bfloat16).cuda()
        k.linear(xt, w2, out, row_scale=RowScale(partials, H, 1e-5))
        k.tcgen05_check(a.device)
        got.append((res, xt, partials, out))
    for u, v in zip(*got):
        assert torch.equal(u, v)
