"""Fused model-level kernels against their fp32 PyTorch statements."""
import pytest
import torch

from recsdk_b200.ops import model_ops

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


@pytest.mark.parametrize("M,d,N", [(1000, 512, 512), (37, 64, 128), (4096, 256, 2048)])
def test_sampled_softmax_loss_and_gradients(M, d, N):
    g = torch.Generator().manual_seed(M + N)
    h = (torch.randn(M, d, generator=g) * 0.5).to(DEV, torch.bfloat16).requires_grad_()
    ep = (torch.randn(M, d, generator=g) * 0.5).to(DEV, torch.bfloat16).requires_grad_()
    en = (torch.randn(N, d, generator=g) * 0.5).to(DEV, torch.bfloat16).requires_grad_()
    scale = 1.0 / M
    loss = model_ops.sampled_softmax_loss(h, ep, en, scale)
    loss.backward()
    hf, pf, nf = (t.detach().float().requires_grad_() for t in (h, ep, en))
    pos = (hf * pf).sum(-1, keepdim=True)
    neg = (hf @ nf.t()).to(torch.bfloat16).float()                     # the kernel reads the GEMM's bf16 logits
    want = (torch.logsumexp(torch.cat([pos, neg], 1), 1) - pos.squeeze(1)).sum() * scale
    want.backward()
    assert abs(float(loss) - float(want)) <= 5e-3 * abs(float(want)) + 1e-4
    for got, ref in ((h.grad, hf.grad), (ep.grad, pf.grad), (en.grad, nf.grad)):
        err = (got.float() - ref).abs().max().item()
        assert err <= 2e-2 * ref.abs().max().item() + 1e-6, err


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_dcn_cross_combine(dtype):
    g = torch.Generator().manual_seed(2)
    xs = [torch.randn(513, 264, generator=g).to(DEV, dtype).requires_grad_() for _ in range(3)]
    y = model_ops.dcn_cross_combine(*xs)
    w = torch.randn(513, 264, generator=g).to(DEV, dtype)
    (y * w).sum().backward()
    fs = [x.detach().float().requires_grad_() for x in xs]
    yf = fs[0] * fs[1] + fs[2]
    (yf * w.float()).sum().backward()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-6
    assert (y.float() - yf).abs().max().item() <= tol * yf.abs().max().item()
    for x, f in zip(xs, fs):
        assert (x.grad.float() - f.grad).abs().max().item() <= tol * f.grad.abs().max().item() + 1e-7


def test_multislice_concat():
    for dtype in (torch.float32, torch.bfloat16, torch.int64):
        x = (torch.arange(77 * 50).view(77, 50) % 997).to(DEV).to(dtype)
        sl = [(3, 10), (0, 1), (40, 50), (20, 20), (7, 31)]
        got = model_ops.multislice_concat(x, sl)
        want = torch.cat([x[:, a:b] for a, b in sl], dim=1)
        assert torch.equal(got, want)


def test_tensor_map_kernel_as_first_node_of_a_fresh_autograd_thread():
    """A process whose very first backward node launches a TMA kernel: the autograd worker thread has made no CUDA runtime
    call yet, so the tensor-map encode (a driver call) must bind the context itself."""
    import subprocess
    import sys

    code = (
        "import torch\n"
        "from recsdk_b200.ops import model_ops\n"
        "g = torch.Generator().manual_seed(0)\n"
        "h = (torch.randn(777, 256, generator=g) * 0.5).to('cuda', torch.bfloat16).requires_grad_()\n"
        "ep = (torch.randn(777, 256, generator=g) * 0.5).to('cuda', torch.bfloat16)\n"
        "en = (torch.randn(512, 256, generator=g) * 0.5).to('cuda', torch.bfloat16).requires_grad_()\n"
        "loss = model_ops.sampled_softmax_loss(h, ep, en, 1.0 / 777)\n"
        "loss.backward()\n"
        "torch.cuda.synchronize()\n"
        "assert torch.isfinite(h.grad.float()).all() and torch.isfinite(en.grad.float()).all()\n"
        "print('ok')\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]


@pytest.mark.parametrize("dtype,kinds", [(torch.float32, "c2p|p2c"), (torch.bfloat16, "c2p|p2c"), (torch.float16, "c2p"), (torch.float32, "p2c")])
def test_disentangle_attention_fused_softmax(dtype, kinds):
    from recsdk_b200.ops import mxrec  # noqa: F401
    from recsdk_b200.ops.mxrec import _disentangle_ref

    b, n, s, d, span = 2, 3, 70, 32, 16
    g = torch.Generator().manual_seed(9)
    q, k, v = ((torch.randn(b, n, s, d, generator=g) * 0.5).to(DEV, dtype).requires_grad_() for _ in range(3))
    pk, pq = ((torch.randn(2 * span, n, d, generator=g) * 0.5).to(DEV, dtype).requires_grad_() for _ in range(2))
    pos = torch.arange(s)
    rel = (pos[:, None] - pos[None, :] + torch.randint(-2, 3, (s, s), generator=g)).view(1, 1, s, s).to(DEV)   # not antisymmetric
    mask = (torch.rand(b, 1, s, s, generator=g) < 0.8).to(DEV)
    mask[0, 0, 5] = False                                              # a fully masked row
    out, probs, score = torch.ops.mxrec.disentangle_attention(q, k, v, pk, pq, rel, mask, kinds, 0.1)
    refs = [t.detach().float().requires_grad_() for t in (q, k, v, pk, pq)]
    wo, wp, ws = _disentangle_ref(*refs, rel, mask, kinds, 0.1)
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    for got, want in ((out, wo), (probs, wp), (score, ws)):
        assert got.dtype == dtype and got.shape == want.shape
        assert (got.float() - want).abs().max().item() <= tol * max(1.0, want.abs().max().item())
    assert float(probs[0, :, 5].abs().max()) == 0.0
    w = torch.randn(out.shape, generator=g).to(DEV)
    (out.float() * w).sum().backward()
    (wo * w).sum().backward()
    for got, ref in zip((q, k, v, pk, pq), refs):
        if ref.grad is None:
            continue
        assert (got.grad.float() - ref.grad).abs().max().item() <= 3e-2 * max(1e-3, ref.grad.abs().max().item())
