"""The allocation-free matmul entry point (for embedders that may not call the CUDA allocator)
must give what the ordinary entry point gives, call after call, out of its fixed built-in scratch."""
import numpy as np
import pytest
import torch

from oracle import qmm_ref

pytestmark = pytest.mark.gpu


def _problem(be, cuda, n, k, m, seed):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.02
    x = torch.randn(m, k, generator=g).half()
    wq, s, b = be.quantize.quantize(w)
    return x, wq, s, b, [t.to(cuda) for t in (x, wq, s, b)]


def _noalloc(be, cuda, xd, wqd, sd, bd, n, k, m):
    lib, p = be._lib.lib(), be._lib.ptr
    y = torch.empty(m, n, dtype=torch.float16, device=cuda)
    rc = lib.b200_qmm_noalloc(p(xd), p(wqd), p(sd), p(bd), None, p(y), m, n, k, 64, 0, be._lib.stream_ptr(cuda))
    return rc, y


def test_two_calls_in_a_row_match_the_ordinary_entry_point(be, cuda):
    # a shape that splits K (uses the scratch), then a different one right after it: the second call
    # finds the first call's leftovers in the shared array
    for (n, k, m, seed) in [(3584, 18944, 16, 1), (1152, 896, 8, 2)]:
        x, wq, s, b, (xd, wqd, sd, bd) = _problem(be, cuda, n, k, m, seed)
        assert be.qmm_kernel.workspace_bytes(m, n, k) > 4096          # the scratch really is in use
        want = be.qmm_kernel.matmul(xd, wqd, sd, bd, 64)[0]
        rc, got = _noalloc(be, cuda, xd, wqd, sd, bd, n, k, m)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(got, want)                                  # same kernel, same split: same bits
        gold = qmm_ref.qmm_gold(x.numpy(), wq.numpy().view(np.uint32), s.numpy(), b.numpy())
        err = np.abs(got.cpu().numpy().astype(np.float64) - gold)
        assert np.all(err <= 2.0 ** -10 * np.abs(gold) + 2e-3)        # the tolerance of the other matmul tests


def test_nothing_is_allocated_and_oversize_is_refused(be, cuda):
    lib = be._lib.lib()
    x, wq, s, b, (xd, wqd, sd, bd) = _problem(be, cuda, 4608, 3584, 16, 3)
    _noalloc(be, cuda, xd, wqd, sd, bd, 4608, 3584, 16)                # first call on the device: set-up
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(cuda)
    free_before, _ = torch.cuda.mem_get_info(cuda)
    rc, y = _noalloc(be, cuda, xd, wqd, sd, bd, 4608, 3584, 16)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(cuda)
    assert rc == 0
    assert torch.cuda.memory_allocated(cuda) - before == y.numel() * 2          # only the test's own output
    assert free_before - free_after <= y.numel() * 2 + (2 << 20)                # no driver-level allocation either
    limit = lib.b200_qmm_noalloc_max_scratch_bytes()
    assert limit == 4 << 20
    # more than 32 rows, or a shape whose scratch need exceeds the built-in array: refused, nothing launched
    assert lib.b200_qmm_noalloc(None, None, None, None, None, None, 33, 4608, 3584, 64, 0, None) == -1
    # 32 x 4608 x 3584: the gate/up pair of that shape would want 5.6 MiB, but this entry point only runs the
    # plain product, whose split needs 3.9 MiB: accepted, same bits as the ordinary entry point
    assert lib.b200_qmm_workspace_bytes(32, 4608, 3584) > limit
    x2, _, _, _, (x2d, wq2d, s2d, b2d) = _problem(be, cuda, 4608, 3584, 32, 4)
    rc, y2 = _noalloc(be, cuda, x2d, wq2d, s2d, b2d, 4608, 3584, 32)
    assert rc == 0
    assert torch.equal(y2, be.qmm_kernel.matmul(x2d, wq2d, s2d, b2d, 64)[0])
    # 32 x 3584 x 18944: the plain product's own split wants 5.3 MiB: refused
    x3, _, _, _, (x3d, wq3d, s3d, b3d) = _problem(be, cuda, 3584, 18944, 32, 5)
    rc, _ = _noalloc(be, cuda, x3d, wq3d, s3d, b3d, 3584, 18944, 32)
    assert rc == -6
