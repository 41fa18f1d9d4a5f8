"""CPU oracle of the 4-bit quantised matmul: numpy restatement vs C restatement vs fp64 gold."""
import numpy as np
import pytest

from oracle import qmm_c, qmm_ref


def _case(n, k, m, seed=0):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    wq, s, b = qmm_ref.quantize(w)
    x = rng.standard_normal((m, k)).astype(np.float16)
    return w, wq, s, b, x


def test_pack_layout_is_element_j_in_bits_4j():
    # simd_no_swizzle_cast.metal:82,96,110,124: masks 0x000f000f, >>4, >>8, >>12 pick (e0,e4)...(e3,e7)
    wq = np.array([[0x76543210, 0xFEDCBA98]], dtype=np.uint32)
    assert qmm_ref.unpack_nibbles(wq).tolist() == [list(range(16))]


def test_quantiser_roundtrip_error_is_bounded_by_one_step():
    w, wq, s, b, _ = _case(64, 256, 1)
    deq = qmm_ref.dequantize(wq, s, b).astype(np.float32)
    step = np.abs(np.repeat(s.astype(np.float32), 64, axis=1))
    # the edge rule re-derives the scale from the exactly represented end, so the far end may clip
    assert np.all(np.abs(deq - w) <= 1.01 * step + 2e-3 * np.abs(w) + 1e-4)
    assert np.mean(np.abs(deq - w) <= 0.5 * step + 2e-3 * np.abs(w) + 1e-4) > 0.95


@pytest.mark.parametrize("n,k,m", [(64, 128, 1), (128, 896, 8), (256, 2048, 16), (64, 384, 32), (8, 128, 3)])
def test_c_and_numpy_restatements_agree_with_gold(n, k, m):
    _, wq, s, b, x = _case(n, k, m, seed=n + k + m)
    gold = qmm_ref.qmm_gold(x, wq, s, b)
    y_np = qmm_ref.qmm(x, wq, s, b).astype(np.float64)
    y_c = qmm_c.qmm(x, wq, s, b).astype(np.float64)
    # fp32 accumulation + one fp16 rounding: half an fp16 ulp of the result plus the fp32 sum error
    tol = 2.0 ** -10 * np.abs(gold) + 1e-3
    assert np.all(np.abs(y_np - gold) <= tol)
    assert np.all(np.abs(y_c - gold) <= tol)
    assert np.mean(y_np != y_c) < 0.02         # different fp32 summation orders, same roundings


def test_bias_added_after_fp16_rounding():
    _, wq, s, b, x = _case(64, 128, 8)
    rng = np.random.default_rng(5)
    bias = rng.standard_normal(64).astype(np.float16)
    y0 = qmm_ref.qmm(x, wq, s, b)
    want = (y0.astype(np.float64) + bias.astype(np.float64)[None]).astype(np.float16)
    assert np.array_equal(qmm_ref.qmm(x, wq, s, b, bias=bias), want)
    y_c = qmm_c.qmm(x, wq, s, b, bias=bias)
    assert np.mean(y_c != want) < 0.02


def test_c_half_rounding_matches_numpy():
    rng = np.random.default_rng(1)
    v = rng.standard_normal(5000) * 10.0 ** rng.integers(-9, 4, 5000)
    v = np.concatenate([v, [0.0, -0.0, 65504.0, 65519.9, 65520.0, 2.0 ** -25, 2.0 ** -24, 6.1e-5, 1e-8]])
    lib = qmm_c.lib()
    got = np.array([lib.oracle_f64_to_f16(float(t)) for t in v], dtype=np.uint16)
    with np.errstate(over="ignore"):
        want = v.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)


def test_bad_shape_rejected():
    _, wq, s, b, x = _case(64, 128, 1)
    with pytest.raises(ValueError):
        qmm_c.qmm(x, wq, s, b, group_size=48)
