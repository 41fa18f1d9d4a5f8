"""Parity of the CUDA quantised matmul (through the C ABI) with the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import qmm_c, qmm_ref

pytestmark = pytest.mark.gpu


def _case(n, k, m, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.02
    x = torch.randn(m, k, generator=g).half()
    return w, x


def _tol(gold):
    # fp16 result (half an ulp = 2^-11 relative) + fp32 accumulation order effects; stated bound:
    # |y - gold| <= 2^-10 |gold| + 2e-3
    return 2.0 ** -10 * np.abs(gold) + 2e-3


SHAPES = [
    # (N, K, M) - incl. K % 256 == 128 (896), ragged N (not a multiple of the CTA tile), M not multiple of 8
    (8192, 2048, 1), (8192, 2048, 8), (8192, 2048, 16), (8192, 2048, 24), (8192, 2048, 32),
    (1152, 896, 8), (896, 4864, 8), (4864, 896, 7), (8, 128, 1), (72, 128, 5), (200, 256, 32),
    (3584, 18944, 16), (16032, 1024, 24), (4608, 3584, 16), (1024, 3584, 9),
]


@pytest.mark.parametrize("n,k,m", SHAPES)
def test_qmm_matches_oracle(be, cuda, n, k, m):
    w, x = _case(n, k, m, seed=n * 7 + k + m)
    wq, s, b = be.quantize.quantize(w)
    y = be.qmm_kernel.matmul(x.to(cuda), wq.to(cuda), s.to(cuda), b.to(cuda), 64)[0]
    torch.cuda.synchronize()
    wq_np = wq.numpy().view(np.uint32)
    gold = qmm_ref.qmm_gold(x.numpy(), wq_np, s.numpy(), b.numpy())
    got = y.cpu().numpy().astype(np.float64)
    assert got.shape == (m, n)
    err = np.abs(got - gold)
    assert np.all(err <= _tol(gold)), f"max err {err.max()} at {np.unravel_index(err.argmax(), err.shape)}"
    ref = qmm_c.qmm(x.numpy(), wq_np, s.numpy(), b.numpy())
    # same roundings, different fp32 summation order: almost every element is bit-identical
    assert np.mean(ref != y.cpu().numpy()) < 0.05


def test_quantiser_matches_oracle_quantiser(be):
    w, _ = _case(128, 512, 1, 3)
    wq, s, b = be.quantize.quantize(w)
    wq2, s2, b2 = qmm_ref.quantize(w.numpy())
    assert np.array_equal(wq.numpy().view(np.uint32), wq2)
    assert np.array_equal(s.numpy(), s2) and np.array_equal(b.numpy(), b2)


def test_leading_batch_dims_and_large_m(be, cuda):
    w, x = _case(256, 256, 80, 11)
    wq, s, b = be.quantize.quantize(w)
    x3 = x.reshape(2, 40, 256).to(cuda)
    y = be.qmm_kernel.matmul(x3, wq.to(cuda), s.to(cuda), b.to(cuda), 64)[0]
    assert y.shape == (2, 40, 256)
    gold = qmm_ref.qmm_gold(x.numpy(), wq.numpy().view(np.uint32), s.numpy(), b.numpy())
    assert np.all(np.abs(y.reshape(80, 256).cpu().numpy().astype(np.float64) - gold) <= _tol(gold))


def test_row_results_do_not_depend_on_batch_size(be, cuda):
    """Row i of an M-row call equals the same row computed alone (the decode loop relies on it)."""
    w, x = _case(1152, 896, 8, 21)
    wq, s, b = (t.to(cuda) for t in be.quantize.quantize(w))
    y8 = be.qmm_kernel.matmul(x.to(cuda), wq, s, b, 64)[0]
    y1 = be.qmm_kernel.matmul(x[3:4].to(cuda), wq, s, b, 64)[0]
    assert torch.equal(y8[3:4], y1)


def test_fused_epilogues(be, cuda):
    n, k, m = 4864, 896, 16
    g = torch.Generator().manual_seed(5)
    wg, wu = torch.randn(n, k, generator=g) * 0.02, torch.randn(n, k, generator=g) * 0.02
    x = torch.randn(m, k, generator=g).half()
    bias = torch.randn(n, generator=g).half()
    res = torch.randn(m, n, generator=g).half()
    qg = be.quantize.quantize(wg)
    qu = be.quantize.quantize(wu)
    dg = [t.to(cuda) for t in qg]
    du = [t.to(cuda) for t in qu]
    xd = x.to(cuda)
    qk = be.qmm_kernel
    f64 = np.float64
    yg = qmm_ref.qmm(x.numpy(), qg[0].numpy().view(np.uint32), qg[1].numpy(), qg[2].numpy())
    yu = qmm_ref.qmm(x.numpy(), qu[0].numpy().view(np.uint32), qu[1].numpy(), qu[2].numpy())

    # bias: y = fp16(fp16(acc) + bias)
    got = qk.matmul_fused(xd, *dg, bias=bias.to(cuda)).cpu().numpy()
    want = (yg.astype(f64) + bias.numpy().astype(f64)[None]).astype(np.float16)
    assert np.mean(got != want) < 0.05
    assert np.all(np.abs(got.astype(f64) - want.astype(f64)) <= 2.0 ** -9 * np.abs(want.astype(f64)) + 2e-3)

    # residual: y = fp16(res + fp16(acc)), in place
    r = res.to(cuda).clone()
    got = qk.matmul_fused(xd, *dg, epilogue=qk.EPI_RESIDUAL, extra=r, out=r).cpu().numpy()
    want = (res.numpy().astype(f64) + yg.astype(f64)).astype(np.float16)
    assert np.mean(got != want) < 0.05
    assert np.all(np.abs(got.astype(f64) - want.astype(f64)) <= 2.0 ** -9 * np.abs(want.astype(f64)) + 2e-3)

    # SiLU(gate) * up with fp16 rounding after every op (mlx_llama.py:215)
    got = qk.matmul_fused(xd, *dg, epilogue=qk.EPI_SILU_MUL, w2=du[0], s2=du[1], b2=du[2]).cpu().numpy()
    gf = yg.astype(np.float32)
    sig = (1.0 / (1.0 + np.exp(-gf))).astype(np.float16)
    t = (yg.astype(f64) * sig.astype(f64)).astype(np.float16)
    want = (t.astype(f64) * yu.astype(f64)).astype(np.float16)
    assert np.mean(got != want) < 0.05
    assert np.all(np.abs(got.astype(f64) - want.astype(f64)) <= 2.0 ** -8 * np.abs(want.astype(f64)) + 2e-3)


def test_rejects_bad_arguments(be, cuda):
    w, x = _case(64, 128, 4, 1)
    wq, s, b = (t.to(cuda) for t in be.quantize.quantize(w))
    with pytest.raises(AssertionError):
        be.qmm_kernel.matmul(torch.zeros(4, 192, dtype=torch.half, device=cuda), wq, s, b, 64)
    with pytest.raises(be._lib.B200Error):
        be.qmm_kernel.matmul(x, wq, s, b, 64)          # CPU tensor: no fallback
    with pytest.raises(be._lib.B200Error):
        be.qmm_kernel.matmul(x.to(cuda).float(), wq, s, b, 64)


@pytest.mark.parametrize("n,k,m", SHAPES)
def test_tiled_kernel_matches_oracle_and_rowmajor_kernel(be, cuda, n, k, m):
    w, x = _case(n, k, m, seed=n * 7 + k + m)
    wq, s, b = be.quantize.quantize(w)
    dq = [t.to(cuda) for t in (wq, s, b)]
    wt = be.qmm_kernel.relayout(*dq)
    assert wt.numel() == ((n + 63) // 64) * (k // 128) * 4 * 1152
    y = be.qmm_kernel.matmul_tiled(x.to(cuda), wt, n)
    torch.cuda.synchronize()
    assert be.qmm_kernel.stream_error(cuda) == 0
    gold = qmm_ref.qmm_gold(x.numpy(), wq.numpy().view(np.uint32), s.numpy(), b.numpy())
    got = y.cpu().numpy().astype(np.float64)
    err = np.abs(got - gold)
    assert np.all(err <= _tol(gold)), f"max err {err.max()} at {np.unravel_index(err.argmax(), err.shape)}"
    y_rm = be.qmm_kernel.matmul(x.to(cuda), *dq, 64)[0]
    assert np.mean(y_rm.cpu().numpy() != y.cpu().numpy()) < 0.05


def test_tiled_fused_epilogues_equal_rowmajor_results(be, cuda):
    qk = be.qmm_kernel
    for (n, k, m) in [(4864, 896, 16), (18944 // 4, 3584, 32), (4864, 896, 3)]:
        g = torch.Generator().manual_seed(n + m)
        wg, wu = torch.randn(n, k, generator=g) * 0.02, torch.randn(n, k, generator=g) * 0.02
        x = torch.randn(m, k, generator=g).half().to(cuda)
        bias = torch.randn(n, generator=g).half().to(cuda)
        res = torch.randn(m, n, generator=g).half().to(cuda)
        dg = [t.to(cuda) for t in be.quantize.quantize(wg)]
        du = [t.to(cuda) for t in be.quantize.quantize(wu)]
        tg, tu = qk.relayout(*dg), qk.relayout(*du)
        a = qk.matmul_fused(x, *dg, bias=bias)
        b = qk.matmul_tiled(x, tg, n, bias=bias)
        assert (a != b).float().mean() < 0.05 and torch.allclose(a.float(), b.float(), rtol=2e-3, atol=2e-3)
        a = qk.matmul_fused(x, *dg, epilogue=qk.EPI_RESIDUAL, extra=res)
        b = qk.matmul_tiled(x, tg, n, epilogue=qk.EPI_RESIDUAL, extra=res)
        assert (a != b).float().mean() < 0.05 and torch.allclose(a.float(), b.float(), rtol=2e-3, atol=2e-3)
        a = qk.matmul_fused(x, *dg, epilogue=qk.EPI_SILU_MUL, w2=du[0], s2=du[1], b2=du[2])
        b = qk.matmul_tiled(x, tg, n, epilogue=qk.EPI_SILU_MUL, wt2=tu)
        assert (a != b).float().mean() < 0.05 and torch.allclose(a.float(), b.float(), rtol=4e-3, atol=2e-3)
    assert qk.stream_error(cuda) == 0


def test_tiled_rows_do_not_depend_on_batch_size(be, cuda):
    w, x = _case(1152, 896, 8, 21)
    wt = be.qmm_kernel.relayout(*[t.to(cuda) for t in be.quantize.quantize(w)])
    y8 = be.qmm_kernel.matmul_tiled(x.to(cuda), wt, 1152)
    y1 = be.qmm_kernel.matmul_tiled(x[3:4].to(cuda), wt, 1152)
    assert torch.equal(y8[3:4], y1)
