"""The tcgen05 + TMA matrix product against a float64 reference: tails in every dimension, both tile
widths and the tiles on pairs of SMs, float32 output, and the fused SiLU(gate) * up epilogue over rows interleaved in groups of 8."""
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


def K():
    from iian_b200.ops.cuda_backend import CudaKernels
    return CudaKernels()


def rnd(*shape, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16).cuda()


SHAPES = [(128, 256, 64), (128, 256, 256), (1, 128, 64), (200, 384, 512), (130, 128, 520), (333, 1000, 1032),
          (2048, 6144, 4096), (512, 4096, 12288)]


@pytest.mark.parametrize("T,N,Kd", SHAPES)
@pytest.mark.parametrize("bn", [128, 256, 512])
def test_gemm_tcgen05_store(T, N, Kd, bn):
    k = K()
    x, w = rnd(T, Kd, seed=1), rnd(N, Kd, seed=2, std=0.05)
    out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    k.gemm_tcgen05(x, w, out, bn=bn)
    k.tcgen05_check(x.device)
    want = x.double().cpu() @ w.double().cpu().T
    err = (out.double().cpu() - want).abs().max().item()
    assert err < 1.6e-2 * max(1.0, want.abs().max().item()), err


@pytest.mark.parametrize("bn", [128, 512])
def test_gemm_tcgen05_float32_out(bn):
    k = K()
    x, w = rnd(77, 512, seed=3), rnd(503, 512, seed=4, std=0.05)
    out = torch.full((77, 503), float("nan"), dtype=torch.float32, device="cuda")
    k.gemm_tcgen05(x, w, out, bn=bn)
    k.tcgen05_check(x.device)
    want = x.double().cpu() @ w.double().cpu().T
    assert (out.double().cpu() - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("bn", [0, 512])
@pytest.mark.parametrize("T,F,Kd", [(128, 128, 64), (300, 160, 256), (2048, 12288, 4096)])
def test_gemm_tcgen05_swiglu_epilogue(T, F, Kd, bn):
    k = K()
    x = rnd(T, Kd, seed=5)
    wg, wu = rnd(F, Kd, seed=6, std=0.05), rnd(F, Kd, seed=7, std=0.05)
    inter = torch.stack([wg.view(F // 8, 8, Kd), wu.view(F // 8, 8, Kd)], dim=1).reshape(2 * F, Kd).contiguous()
    out = torch.full((T, F), float("nan"), dtype=torch.bfloat16, device="cuda")
    k.gemm_tcgen05(x, inter, out, epilogue=1, bn=bn)
    k.tcgen05_check(x.device)
    xd = x.double().cpu()
    want = plain.silu(xd @ wg.double().cpu().T) * (xd @ wu.double().cpu().T)
    err = (out.double().cpu() - want).abs().max().item()
    assert err < 2e-2 * max(1.0, want.abs().max().item()), err


def test_gemm_tcgen05_refuses_what_it_cannot_do():
    from iian_b200.ops.cuda_backend import KernelError
    k = K()
    with pytest.raises(KernelError):
        k.gemm_tcgen05(rnd(8, 60), rnd(16, 60), torch.empty(8, 16, dtype=torch.bfloat16, device="cuda"))   # K not a multiple of 8
    with pytest.raises(KernelError):
        k.gemm_tcgen05(rnd(8, 64).float(), rnd(16, 64), torch.empty(8, 16, dtype=torch.bfloat16, device="cuda"))


def test_a_kernel_that_gave_up_is_reported_at_the_next_host_wait():
    """The status words a tcgen05 kernel writes when a bounded wait runs out are read where the host waits for the
    device anyway; here they are set by hand (no kernel is made to give up)."""
    from iian_b200.ops.cuda_backend import CudaKernels, KernelError
    k = K()
    x, w = rnd(128, 64, seed=1), rnd(128, 64, seed=2)
    out = torch.empty(128, 128, dtype=torch.bfloat16, device="cuda")
    k.gemm_tcgen05(x, w, out)
    k.check_device_status()                      # a clean run: nothing to report, and the flag is taken down
    assert not CudaKernels._tc_used
    k.check_device_status()
    k.gemm_tcgen05(x, w, out)
    torch.cuda.synchronize()
    k.tcgen05_status_buffer(x.device).copy_(torch.tensor([2, 5], dtype=torch.int32))
    with pytest.raises(KernelError, match="gave up"):
        k.check_device_status()
    assert k.tcgen05_status_buffer(x.device).tolist() == [0, 0]
