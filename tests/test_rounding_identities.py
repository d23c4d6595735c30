"""CPU checks of two arithmetic identities the quantizer kernels rely on (numpy models of the
device arithmetic; the kernels themselves are compared bit for bit with the oracle and with the
reference's kernels in the GPU tests).

1. Q8_1: q = rn(fl(x / d)) is formed on the device without a division per value, as
   t = fl(x * r), q' = fl(t + fl(x - t * d) * r) with r = fl(1 / d) and both inner products
   fused: q' must equal fl(x / d) for every bf16 x of a block and d = fl(amax / 127).
2. NVFP4: the reference's code of a value counts the thresholds .25 .75 1.25 1.75 2.5 3.5 5 that
   |v| reaches (ties go up).  The device sets the lowest mantissa bit of v and lets a
   round-to-nearest-even conversion to e2m1 choose: both must give the same code for every float,
   thresholds, their neighbours, zeros of both signs, infinities and NaN included."""
import numpy as np
import torch


def _bf16(x):
    return torch.from_numpy(x.astype(np.float32)).to(torch.bfloat16).float().numpy()


def _fma(a, b, c):
    """fl32(a * b + c) for float32 inputs: the product of two float32 is exact in float64, and the
    sum is rounded once to float64 before the final rounding (double rounding can only matter in
    a 2^-29 fraction of the cases and would show up as a mismatch, not hide one)."""
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(np.float32)


def test_corrected_quotient_equals_ieee_division_on_bf16_blocks():
    rng = np.random.default_rng(7)
    mism = 0
    total = 0
    for scale in (1e-3, 0.02, 1.0, 37.0, 4e3):
        x = _bf16(rng.standard_normal((40000, 32)) * scale)
        amax = np.abs(x).max(1, keepdims=True).astype(np.float32)
        d = (amax / np.float32(127.0)).astype(np.float32)
        r = (np.float32(1.0) / d).astype(np.float32)
        t = (x * r).astype(np.float32)
        rem = _fma(-t, d, x)
        q = _fma(rem, r, t)
        true = (x / d).astype(np.float32)
        mism += int((q != true).sum())
        total += q.size
        # and the integers the magic-number addition reads off the sum's low mantissa byte
        km = (q + np.float32(12582912.0)).astype(np.float32)
        low = (km.view(np.uint32) & 0xFF).astype(np.uint8).view(np.int8)
        assert np.array_equal(low.astype(np.int32), np.rint(true).astype(np.int32))
    assert mism == 0, f"{mism} of {total} quotients differ"


def test_exact_ties_are_common_with_bf16_inputs():
    """Why a 'near a tie -> divide' test is the wrong fast path: one value in a few hundred is an
    exact half-integer quotient, so a warp of 32 lanes meets one for about one value in eight."""
    rng = np.random.default_rng(3)
    x = _bf16(rng.standard_normal((20000, 32)))
    amax = np.abs(x).max(1, keepdims=True).astype(np.float32)
    d = (amax / np.float32(127.0)).astype(np.float32)
    q = (x / d).astype(np.float32)
    near = np.abs(np.abs(q - np.rint(q)) - 0.5) < 1e-4
    assert 1e-3 < near.mean() < 2e-2


E2M1 = np.array([0, .5, 1, 1.5, 2, 3, 4, 6], dtype=np.float64)


def _rne_e2m1(v):
    """Round to nearest e2m1 magnitude, ties to the even code, saturating; sign in bit 3."""
    a = np.minimum(np.abs(v.astype(np.float64)), 6.0)
    dist = np.abs(a[:, None] - E2M1[None, :])
    best = dist.min(1, keepdims=True)
    cand = dist == best
    idx = np.where(cand.sum(1) == 2, np.where(cand[:, ::2].any(1), cand[:, ::2].argmax(1) * 2, 0), cand.argmax(1))
    return idx | np.where(np.signbit(v), 8, 0)


def _reference_code(v):
    a = np.abs(v)
    with np.errstate(invalid="ignore"):
        idx = sum((a >= np.float32(t)).astype(np.int64) for t in (.25, .75, 1.25, 1.75, 2.5, 3.5, 5.0))
        return idx | np.where(v < 0, 8, 0)


def _device_untie(v):
    with np.errstate(invalid="ignore"):
        some = np.abs(v) > 0                                          # false for +-0 and NaN
        c = np.minimum(np.maximum(v, np.float32(-8)), np.float32(8))
    c = np.where(np.isnan(v), np.float32(-8), c)                      # fminf(fmaxf(NaN, -8), 8)
    b = (c.astype(np.float32).view(np.uint32) | np.uint32(1)).view(np.float32)
    return np.where(some, b, np.float32(0)).astype(np.float32)


def test_tie_free_input_makes_round_to_even_count_thresholds():
    vals = []
    for t in (.25, .75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 8.0, .5, 1, 1.5, 2, 3, 4):
        b = int(np.float32(t).view(np.uint32))
        vals += [np.uint32(b + k).view(np.float32) for k in range(-4, 5)]
    vals = np.array(vals + [0.0, 1e-45, 1e-30, 100.0, 3e38], dtype=np.float32)
    rnd = (np.random.default_rng(0).standard_normal(200000) * 3).astype(np.float32)
    special = np.array([np.inf, -np.inf, np.nan, -0.0], dtype=np.float32)
    v = np.concatenate([vals, -vals, special, rnd])
    got = _rne_e2m1(_device_untie(v))
    want = _reference_code(v)
    bad = np.nonzero(got != want)[0]
    assert bad.size == 0, (v[bad][:8], got[bad][:8], want[bad][:8])
    # without the nudge round-to-even disagrees on the ties .25, 1.25 and 2.5
    plain = _rne_e2m1(np.array([.25, 1.25, 2.5], dtype=np.float32))
    assert list(plain) == [0, 2, 4] and list(_reference_code(np.array([.25, 1.25, 2.5], dtype=np.float32))) == [1, 3, 5]
