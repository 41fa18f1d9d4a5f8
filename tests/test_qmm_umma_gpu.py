"""The tcgen05 matmul operator (b200_qmm_umma) against the fp64 gold of the CPU oracle and the streaming kernel."""
import numpy as np
import pytest
import torch

from oracle import qmm_ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k,bias", [(1, 128, 128, False), (8, 256, 896, True), (16, 1280, 3584, False),
                                        (24, 384, 1024, True), (32, 2048, 512, False), (50, 256, 640, True),
                                        (64, 1152, 896, False), (100, 384, 2048, True), (128, 1280, 1024, False)])
def test_umma_matches_gold_and_streaming_kernel(be, cuda, m, n, k, bias):
    g = torch.Generator().manual_seed(100 + m)
    w = torch.randn(n, k, generator=g) * 0.02
    x = torch.randn(m, k, generator=g).half()
    bv = (torch.randn(n, generator=g) * 0.02).half() if bias else None
    wq, s, b = be.quantize.quantize(w)
    wt = be.qmm_kernel.relayout(wq.to(cuda), s.to(cuda), b.to(cuda))
    dev = torch.device(cuda)
    y = be.qmm_kernel.matmul_umma(x.to(dev), wt, n, bias=None if bv is None else bv.to(dev))
    torch.cuda.synchronize()
    assert be.qmm_kernel.umma_error(dev) == 0
    y_t = torch.cat([be.qmm_kernel.matmul_tiled(x[r:r + 32].to(dev), wt, n, bias=None if bv is None else bv.to(dev))
                     for r in range(0, m, 32)])          # the streaming kernel takes 32 rows at a time
    gold = qmm_ref.qmm_gold(x.numpy(), wq.numpy().view(np.uint32), s.numpy(), b.numpy())
    if bv is not None:
        gold = gold + bv.numpy().astype(np.float64)
    got = y.cpu().numpy().astype(np.float64)
    assert np.all(np.abs(got - gold) <= 2.0 ** -10 * np.abs(gold) + 2e-3)       # the matmul tolerance of this library
    # same dequantised weights, same fp32 accumulation up to the summation order: a few fp16 ulps from the streaming kernel
    d = np.abs(got - y_t.cpu().numpy().astype(np.float64))
    assert np.all(d <= 2.0 ** -9 * np.abs(gold) + 2e-3)


def test_umma_rejects_unsupported_shapes(be, cuda):
    dev = torch.device(cuda)
    lib = be._lib.lib()
    ws = torch.zeros(1 << 20, dtype=torch.uint8, device=dev)
    x = torch.zeros(8, 256, dtype=torch.float16, device=dev)
    y = torch.zeros(8, 192, dtype=torch.float16, device=dev)
    p = be._lib.ptr
    assert lib.b200_qmm_umma(p(x), p(ws), None, p(y), 8, 192, 256, p(ws), ws.numel(), None) == -3      # N % 128
    assert lib.b200_qmm_umma(p(x), p(ws), None, p(y), 129, 128, 256, p(ws), ws.numel(), None) == -1    # M > 128
    assert lib.b200_qmm_umma(p(x), p(ws), None, p(y), 8, 128, 256, p(ws), 64, None) == -4              # workspace
