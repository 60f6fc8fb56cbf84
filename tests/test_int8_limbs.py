"""The int8 limb split that the tensor-core attention kernel over the int8 KV cache applies to its fp32 operands
(q, and p x value scale): restated in numpy with the kernel's own float32 steps, checked for exactness of every step,
for the range of the limbs, and for the size of what three limbs leave behind. No GPU."""
import numpy as np

MAGIC = np.float32(12582912.0)          # 1.5 * 2^23: adding it rounds a float32 to an integer in its low mantissa bits


def limbs(t):
    """attention.cu: i8m_limbs. t float32 with |t| <= 64. Returns the three int8 limbs and the float32 residue."""
    t = np.asarray(t, dtype=np.float32)
    x0 = (t + MAGIC).astype(np.float32)
    r = ((t - (x0 - MAGIC)) * np.float32(128.0)).astype(np.float32)
    x1 = (r + MAGIC).astype(np.float32)
    r2 = ((r - (x1 - MAGIC)) * np.float32(128.0)).astype(np.float32)
    x2 = (r2 + MAGIC).astype(np.float32)
    low = lambda x: x.view(np.int32).astype(np.int64).astype(np.int8)      # the low byte of the bit pattern  # noqa: E731
    return low(x0), low(x1), low(x2), (r2 - (x2 - MAGIC)).astype(np.float32)


def test_the_low_byte_of_the_rounded_sum_is_the_rounded_integer():
    t = np.linspace(-64, 64, 100001, dtype=np.float32)
    l0, _, _, _ = limbs(t)
    assert np.array_equal(l0.astype(np.float64), np.rint(t.astype(np.float64)))     # round half to even, like rintf


def test_limbs_fit_int8_and_rebuild_the_value_to_2_to_the_minus_15():
    rng = np.random.default_rng(0)
    t = np.concatenate([rng.uniform(-64, 64, 200000), [0.0, 64.0, -64.0, 0.5, -0.5, 63.99999, 1e-7, -1e-7, 2.0 ** -20]]).astype(np.float32)
    l0, l1, l2, res = limbs(t)
    for l in (l0, l1, l2):
        assert l.min() >= -64 and l.max() <= 64
    rebuilt = l0.astype(np.float64) + l1.astype(np.float64) / 128.0 + l2.astype(np.float64) / 16384.0
    err = np.abs(rebuilt - t.astype(np.float64))
    assert err.max() <= 2.0 ** -15 + 1e-12
    # every subtraction in the chain was exact: what is left, scaled back, is exactly the difference
    assert np.array_equal(res.astype(np.float64) / 16384.0, t.astype(np.float64) - rebuilt)


def test_scores_through_limbs_equal_the_float_scores_to_fp32_rounding():
    """Q.K over int8 codes with q as limbs (exact integer sums, combined in float32 like the kernel) against float64."""
    rng = np.random.default_rng(1)
    hd, rows = 128, 512
    q = (rng.standard_normal(hd) * 3).astype(np.float32)
    codes = rng.integers(-127, 128, (rows, hd)).astype(np.int8)
    e = int(np.floor(np.log2(np.abs(q).max()))) - 5                      # |q| / 2^e < 64
    l0, l1, l2, _ = limbs(q * np.float32(2.0 ** -e))
    s0, s1, s2 = (codes.astype(np.int64) @ l.astype(np.int64) for l in (l0, l1, l2))
    assert max(np.abs(s).max() for s in (s0, s1, s2)) < 2 ** 23                     # the sums fit fp32's integers
    f = np.float32(1.0 / 128.0)
    dot = ((s2.astype(np.float32) * f + s1.astype(np.float32)) * f + s0.astype(np.float32)) * np.float32(2.0 ** e)
    ref = codes.astype(np.float64) @ q.astype(np.float64)
    scale = np.abs(codes.astype(np.float64)) @ np.abs(q.astype(np.float64))         # what a float32 dot product's error scales with
    assert np.max(np.abs(dot.astype(np.float64) - ref) / scale) < 2e-6
