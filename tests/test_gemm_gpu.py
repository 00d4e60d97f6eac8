"""tcgen05 GEMM kernels against the fp32 PyTorch statement of the same product."""
import pytest
import torch

from minisgl.ops import gemm, quant

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(128, 256, 512), (8, 4096, 1024), (1, 512, 4096), (300, 1536, 4096), (128, 24, 512)])
@pytest.mark.parametrize("bn", [0, 32, 64, 128])
def test_gemm_bf16(m, n, k, bn):
    torch.manual_seed(0)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    y = gemm.gemm_bf16(x, w, out_dtype=torch.float32, bn=bn)
    ref = x.float() @ w.float().t()
    torch.cuda.synchronize()
    assert torch.allclose(y, ref, rtol=2e-3, atol=2e-3), (y - ref).abs().max().item()
    yb = gemm.gemm_bf16(x, w, bn=bn)
    assert torch.allclose(yb.float(), ref, rtol=2e-2, atol=2e-2)


def test_gemm_bf16_accumulate():
    x = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(128, 256, device="cuda", dtype=torch.bfloat16) * 0.1
    out = torch.ones(64, 128, device="cuda", dtype=torch.float32)
    gemm.gemm_bf16(x, w, out=out, accumulate=True)
    ref = x.float() @ w.float().t() + 1
    assert torch.allclose(out, ref, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("m,n,k", [(128, 512, 1024), (5, 4096, 4096), (200, 1536, 4096), (128, 64, 256)])
@pytest.mark.parametrize("bn", [0, 32, 64])
def test_gemm_fp8_block_scaled(m, n, k, bn):
    torch.manual_seed(1)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda") * 0.02
    xq, sx = quant.fp8_act_quant(x)
    wq, swc = quant.fp8_weight_quant(w)
    sw = quant.e8m0_decode(swc)
    y = gemm.gemm_fp8(xq, sx, wq, sw, out_dtype=torch.float32, bn=bn)
    xf = (xq.float().reshape(m, k // 128, 128) * sx.unsqueeze(-1)).reshape(m, k)
    wf = quant.fp8_weight_dequant(wq, swc, dtype=torch.float32)
    ref = xf @ wf.t()
    assert torch.allclose(y, ref, rtol=1e-3, atol=1e-3), (y - ref).abs().max().item()


@pytest.mark.parametrize("m,n,k,splits", [(128, 64, 4096, 16), (128, 1536, 4096, 3), (40, 256, 4096, 0), (128, 2048, 4096, 2),
                                            (128, 520, 4096, 8), (300, 96, 2048, 4)])
def test_gemm_bf16_split_k(m, n, k, splits):
    torch.manual_seed(2)
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    ref = x.float() @ w.float().t()
    for _ in range(2):  # the per-tile counters must reset themselves
        y = gemm.gemm_bf16(x, w, out_dtype=torch.float32, bn=32, splits=splits)
        assert torch.allclose(y, ref, rtol=2e-3, atol=2e-3), (y - ref).abs().max().item()
    y1 = gemm.gemm_bf16(x, w, out_dtype=torch.float32, bn=32, splits=splits)
    assert torch.equal(y, y1)  # fixed reduction order: bitwise repeatable


def test_gemm_bf16_cluster_split_k_bf16_out_and_partials():
    """Cluster reduction with a bf16 result and an odd edge; raw split-K partial products sum to the product."""
    torch.manual_seed(4)
    m, n, k = 100, 72, 4096
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    ref = x.float() @ w.float().t()
    y = gemm.gemm_bf16(x, w, bn=32, splits=8)
    assert y.dtype == torch.bfloat16
    assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2), (y.float() - ref).abs().max().item()
    parts = gemm.gemm_bf16_partials(x, w)
    assert parts.shape[1:] == (m, n) and parts.shape[0] > 1
    assert torch.allclose(parts.sum(0), ref, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("splits", [0, 4, 8])
def test_gemm_fp8_split_k(splits):
    torch.manual_seed(3)
    m, n, k = 128, 1536, 4096
    x = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(n, k, device="cuda") * 0.02
    xq, sx = quant.fp8_act_quant(x)
    wq, swc = quant.fp8_weight_quant(w)
    sw = quant.e8m0_decode(swc)
    y = gemm.gemm_fp8(xq, sx, wq, sw, out_dtype=torch.float32, bn=32, splits=splits)
    xf = (xq.float().reshape(m, k // 128, 128) * sx.unsqueeze(-1)).reshape(m, k)
    ref = xf @ quant.fp8_weight_dequant(wq, swc, dtype=torch.float32).t()
    assert torch.allclose(y, ref, rtol=1e-3, atol=1e-3), (y - ref).abs().max().item()


@pytest.mark.parametrize("t,groups", [(128, 8), (5, 1), (300, 2)])
def test_gemm_bf16_grouped(t, groups):
    torch.manual_seed(4)
    k, n = 4096, 1024
    x = torch.randn(t, groups * k, device="cuda", dtype=torch.bfloat16)
    w = (torch.randn(groups * n, k, device="cuda") * 0.03).to(torch.bfloat16)
    y = gemm.gemm_bf16_grouped(x, w, groups)
    ref = gemm.gemm_bf16_grouped(x.cpu(), w.cpu(), groups)
    assert torch.allclose(y.float().cpu(), ref.float(), rtol=2e-2, atol=2e-2)
