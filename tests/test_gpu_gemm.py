"""tcgen05 GEMM vs an fp32 PyTorch reference of the same contract."""
import pytest
import torch

from recsdk_b200.ops import _lib, gemm

pytestmark = pytest.mark.gpu


def _rand(shape, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * 0.5).to(dtype)


@pytest.fixture(params=["full", "light"], autouse=True)
def gemm_variant(request):
    """Every case runs on both GEMM variants: the full-size one (single GPU) and the light one that multi-GPU runs select
    so that side-stream kernels fit beside a GEMM CTA."""
    _lib.lib().rb_gemm_set_concurrent(1 if request.param == "light" else 0)
    yield request.param
    _lib.lib().rb_gemm_set_concurrent(0)


def _check(out, ref, tol):
    err = (out.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item() + 1e-6
    assert err <= tol * scale + tol, "max err %g (scale %g)" % (err, scale)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 256, 128), (300, 200, 104), (1024, 1024, 512),
                                   (4096, 512, 480), (77, 64, 16), (513, 40, 72)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_kmajor_bias_relu(M, N, K, dtype):
    a, b = _rand((M, K), dtype, 1), _rand((N, K), dtype, 2)
    bias = torch.randn(N, device="cuda")
    for epi in (gemm.EPI_NONE, gemm.EPI_RELU, gemm.EPI_SILU):
        out = gemm.gemm16(a, b, bias=bias, epi=epi)
        ref = gemm._ref(a.cpu(), b.cpu(), False, False, bias.cpu(), None, epi, 1.0, None, dtype)
        _check(out.cpu(), ref, 2e-2)
    _lib.check_status()


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (384, 320, 192), (200, 136, 1000), (1024, 480, 2048)])
def test_gemm_mn_major(a_mn, b_mn, M, N, K):
    dtype = torch.bfloat16
    a = _rand((K, M) if a_mn else (M, K), dtype, 3)
    b = _rand((K, N) if b_mn else (N, K), dtype, 4)
    out = gemm.gemm16(a, b, a_mn=a_mn, b_mn=b_mn, epi=gemm.EPI_F32)
    ref = gemm._ref(a.cpu(), b.cpu(), a_mn, b_mn, None, None, gemm.EPI_F32, 1.0, None, torch.float32)
    _check(out.cpu(), ref, 2e-3)
    _lib.check_status()


def test_gemm_splitk_atomic_and_mask():
    dtype = torch.bfloat16
    M, N, K = 256, 480, 8192
    a, b = _rand((K, M), dtype, 5), _rand((K, N), dtype, 6)
    out = torch.zeros(M, N, device="cuda")
    gemm.gemm16(a, b, a_mn=True, b_mn=True, out=out, epi=gemm.EPI_F32_ATOMIC, splits=16)
    ref = a.float().t() @ b.float()
    _check(out, ref, 2e-3)
    x, w = _rand((512, 256), dtype, 7), _rand((256, 128), dtype, 8)   # dX = dZ @ W, W stored [N][K]
    y = _rand((512, 128), dtype, 9)
    dx = gemm.gemm16(x, w, b_mn=True, epi=gemm.EPI_RELU_MASK, aux=y)
    ref = (x.float() @ w.float()) * (y.float() > 0)
    _check(dx, ref, 2e-2)
    _lib.check_status()


def test_gemm_strided_output():
    dtype = torch.bfloat16
    a, b = _rand((640, 256), dtype, 10), _rand((128, 256), dtype, 11)
    wide = torch.zeros(640, 512, dtype=dtype, device="cuda")
    gemm.gemm16(a, b, out=wide[:, 128:256])
    _check(wide[:, 128:256], a.float() @ b.float().t(), 2e-2)
    assert wide[:, :128].abs().max().item() == 0 and wide[:, 256:].abs().max().item() == 0
    _lib.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("M,N,K,epi", [(1000, 520, 256, 2), (8192, 1024, 512, 0), (77, 40, 64, 2)])
def test_fused_column_sums(M, N, K, epi):
    """The epilogue's column sums equal the column sums of the rounded output (bias gradient of the produced dZ)."""
    from recsdk_b200.ops import gemm as G

    torch.manual_seed(M)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    aux = torch.randn(M, N, device="cuda").bfloat16() if epi == 2 else None
    cs = torch.zeros(N, dtype=torch.float32, device="cuda")
    out = G.gemm16(a, b, epi=epi, aux=aux, colsum_out=cs)
    ref = (a.float() @ b.float().t())
    if epi == 2:
        ref = ref * (aux.float() > 0)
    assert torch.allclose(out.float(), ref, atol=0.5, rtol=2e-2)
    assert torch.allclose(cs, ref.sum(0), atol=2e-2 * ref.abs().sum(0).max().item() / 10 + 1.0, rtol=2e-2)
