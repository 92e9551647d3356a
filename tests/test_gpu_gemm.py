"""The tcgen05/TMA matrix product for few tokens against a float32 product of the same
bfloat16 inputs, at the engine's sizes and at sizes that are no multiple of any tile."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from somi_inference_b200.ops import cuda_ops
    return cuda_ops()


SHAPES = [(896, 896), (1152, 896), (896, 4864), (3584, 3584), (5000, 3584), (136, 200),
          (64, 64), (151936 // 8, 896)]


@pytest.mark.parametrize("M", [1, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("N,K", SHAPES)
def test_skinny_gemm_bf16_and_f32(ops, M, N, K):
    g = torch.Generator().manual_seed(N + K + M)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    b = torch.randn(N, generator=g).to(torch.bfloat16).cuda()
    ref = (x.double() @ w.double().T).float()       # float64: no doubt about the reference
    y32 = ops.skinny_gemm(x, w, None, ops.GEMM_F32)
    ops.check_errors()
    scale = ref.abs().max().item()
    assert (y32 - ref).abs().max().item() <= 2e-5 * max(scale, 1.0) * (K / 64) ** 0.5
    y = ops.skinny_gemm(x, w, b, ops.GEMM_BF16)
    torch.testing.assert_close(y.float(), (ref + b.float()).to(torch.bfloat16).float(),
                               rtol=1.6e-2, atol=1e-2 * max(scale, 1.0))


@pytest.mark.parametrize("M,N,K,splits", [(8, 896, 4864, 8), (64, 3584, 18944, 5), (3, 136, 200, 4),
                                          (16, 1152, 896, 3), (1, 896, 896, 16)])
def test_skinny_gemm_split_k(ops, M, N, K, splits):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    b = torch.randn(N, generator=g).float().cuda()
    parts = ops.skinny_gemm(x, w, b, ops.GEMM_PARTIAL_F32, splits=splits)
    ops.check_errors()
    assert 1 <= parts.shape[0] <= splits
    ref = (x.double() @ w.double().T + b.double()).float()
    assert (parts.sum(0) - ref).abs().max().item() <= 1e-4 * max(ref.abs().max().item(), 1.0)


@pytest.mark.parametrize("M,I,K", [(8, 4864, 896), (64, 18944, 3584), (5, 88, 80)])
def test_skinny_gemm_swiglu(ops, M, I, K):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    gate = (torch.randn(I, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    up = (torch.randn(I, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    w = torch.stack([gate, up], dim=1).reshape(2 * I, K).contiguous()     # rows g0, u0, g1, u1, ...
    y = ops.skinny_gemm(x, w, None, ops.GEMM_SWIGLU)
    ops.check_errors()
    gg, uu = (x.double() @ gate.double().T).float(), (x.double() @ up.double().T).float()
    ref = gg * torch.sigmoid(gg) * uu
    torch.testing.assert_close(y.float(), ref, rtol=1.6e-2, atol=1e-2 * max(ref.abs().max().item(), 1.0))


@pytest.mark.parametrize("M,N,K", [(17, 18992, 896), (17, 896, 896), (8, 18992, 896), (8, 1152, 896),
                                   (64, 18992, 896), (64, 896, 4864), (24, 19000, 2048)])
def test_skinny_gemm_launched_alone_many_times(ops, M, N, K):
    """Each launch on an idle GPU, with nothing before it to wait for: the warps that wait for the
    preceding kernel pass that wait at once, which is when an unordered hand-over between the
    kernel's warps would show (every ring depth and token width of the kernel is among the cases)."""
    g = torch.Generator().manual_seed(5)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(N, K, generator=g) * 0.05).to(torch.bfloat16).cuda()
    ref = (x.double() @ w.double().T).float()
    scale = max(ref.abs().max().item(), 1.0)
    first = None
    for i in range(40):
        torch.cuda.synchronize()
        y = ops.skinny_gemm(x, w, None, ops.GEMM_F32)
        torch.cuda.synchronize()
        if first is None:
            first = y.clone()
            assert (y - ref).abs().max().item() <= 2e-5 * scale * (K / 64) ** 0.5
        else:
            assert torch.equal(y, first), f"launch {i} differs from the first"
    ops.check_errors()


@pytest.mark.parametrize("M", [1, 2, 5, 16, 17, 32, 33, 100, 300])
@pytest.mark.parametrize("N,K", [(320, 192), (640, 192), (384, 80), (517, 80), (80, 176), (1000, 192),
                                 (4608, 3584), (896, 4864), (7, 3), (129, 1025)])
def test_float32_product(ops, M, N, K):
    """The float32 path's own product against a float64 product, with and without bias, at the
    tiny models' sizes, at large ones and at sizes that are no multiple of anything."""
    g = torch.Generator().manual_seed(N * 7 + K + M)
    x = torch.randn(M, K, generator=g).cuda()
    w = (torch.randn(N, K, generator=g) * 0.1).cuda()
    b = torch.randn(N, generator=g).cuda()
    ref = x.double() @ w.double().T
    tol = 2e-6 * float(ref.abs().max()) * max(1.0, (K / 64) ** 0.5)
    y = ops.gemm_f32(x, w)
    assert (y.double() - ref).abs().max().item() <= tol
    yb = ops.gemm_f32(x, w, b)
    assert (yb.double() - (ref + b.double())).abs().max().item() <= tol + 1e-6


def test_float32_product_does_not_depend_on_the_other_rows(ops):
    """An output element is the sum of its K terms in ascending order whatever the step's size:
    the same row gives the same bits alone, among 30 rows and among 300."""
    g = torch.Generator().manual_seed(3)
    x = torch.randn(300, 896, generator=g).cuda()
    w = (torch.randn(1152, 896, generator=g) * 0.1).cuda()
    b = torch.randn(1152, generator=g).cuda()
    whole = ops.gemm_f32(x, w, b)
    assert torch.equal(ops.gemm_f32(x[:30].contiguous(), w, b), whole[:30])
    for r in (0, 17, 299):
        assert torch.equal(ops.gemm_f32(x[r:r + 1].contiguous(), w, b), whole[r:r + 1])
