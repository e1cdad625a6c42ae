"""CPU checks of the arithmetic the pre-passes rely on (numpy models of decx_b200/csrc/prepass.cuh):
the tf32 (hi, lo) split with the three-product sum, and the real expansion of the complex product."""
import numpy as np


def rn_tf32(x):
    """cvt.rna.tf32.f32: round to 10 mantissa bits, ties away from zero; low 13 bits cleared."""
    b = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    b = (b + 0x1000) & 0xFFFFE000
    return b.astype(np.uint32).view(np.float32)


def split(x):
    """split1 of prepass.cuh: hi = rn_tf32(x) (truncated instead when the rounding would overflow a finite x),
    lo = rn_tf32(x - hi), and lo = 0 for a non-finite x."""
    x = np.asarray(x, dtype=np.float32)
    finite = np.isfinite(x)
    with np.errstate(over="ignore", invalid="ignore"):
        hi = rn_tf32(x)
        over = finite & ~np.isfinite(hi)
        hi = np.where(over, (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32), hi)
        lo = np.where(finite, rn_tf32((x - hi).astype(np.float32)), np.float32(0))
    return hi.astype(np.float32), lo.astype(np.float32)


def test_split_of_huge_and_non_finite_values():
    fmax = np.finfo(np.float32).max
    x = np.array([fmax, -fmax, np.nextafter(np.float32(fmax), np.float32(0)), 3.0e38, np.inf, -np.inf, np.nan],
                 dtype=np.float32)
    hi, lo = split(x)
    fin = np.isfinite(x)
    assert np.isfinite(hi[fin]).all() and np.isfinite(lo[fin]).all()       # no overflow from the rounding of hi
    assert (hi[fin].astype(np.float64) + lo[fin].astype(np.float64) == x[fin].astype(np.float64)).all() or \
        (np.abs(hi[fin].astype(np.float64) + lo[fin].astype(np.float64) - x[fin]) <= np.abs(x[fin]) * 2.0 ** -21).all()
    assert hi[4] == np.inf and hi[5] == -np.inf and np.isnan(hi[6])
    assert (lo[4:] == 0).all()                                             # inf stays inf, never inf - inf


def test_split_planes_are_tf32_exact_and_close():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(100000) * 10.0 ** rng.integers(-6, 6, 100000)).astype(np.float32)
    hi, lo = split(x)
    for p in (hi, lo):
        assert not (p.view(np.uint32) & 0x1FFF).any()            # representable in tf32: nothing for the MMA to drop
    err = np.abs(hi.astype(np.float64) + lo.astype(np.float64) - x.astype(np.float64))
    assert (err <= np.abs(x.astype(np.float64)) * 2.0 ** -21).all()


def test_three_products_keep_fp32_accuracy_even_without_cancellation():
    """hi*hi + hi*lo + lo*hi against the exact product: <= ~2^-20 relative per term, so the path's metric
    (error over |a|.|b|, Cauchy-Schwarz) stays far below 1e-5 even for all-positive data and K = 1."""
    rng = np.random.default_rng(1)
    a = rng.uniform(0.5, 1.0, 50000).astype(np.float32)
    b = rng.uniform(0.5, 1.0, 50000).astype(np.float32)
    ah, al = split(a)
    bh, bl = split(b)
    f = np.float64
    approx = al.astype(f) * bh.astype(f) + ah.astype(f) * bl.astype(f) + ah.astype(f) * bh.astype(f)
    rel = np.abs(approx - a.astype(f) * b.astype(f)) / (a.astype(f) * b.astype(f))
    assert rel.max() < 2.0 ** -19
    one = np.abs(ah.astype(f) * bh.astype(f) - a.astype(f) * b.astype(f)) / (a.astype(f) * b.astype(f))
    assert one.max() > 1e-4                                       # what a single tf32 product would lose


def test_complex_product_as_real_product():
    """A (M x K complex) viewed as M x 2K reals times the 2K x 2N expansion of B (row 2k = (re, im) pairs of B's
    row k, row 2k+1 = (-im, re) pairs) is D in interleaved storage."""
    rng = np.random.default_rng(2)
    M, N, K = 5, 4, 7
    A = (rng.standard_normal((M, K)) + 1j * rng.standard_normal((M, K))).astype(np.complex64)
    B = (rng.standard_normal((K, N)) + 1j * rng.standard_normal((K, N))).astype(np.complex64)
    A_real = A.view(np.float32).reshape(M, 2 * K)                 # (re, im) interleaved along K
    B_exp = np.empty((2 * K, 2 * N), dtype=np.float32)
    B_exp[0::2, 0::2] = B.real
    B_exp[0::2, 1::2] = B.imag
    B_exp[1::2, 0::2] = -B.imag
    B_exp[1::2, 1::2] = B.real
    D_real = A_real.astype(np.float64) @ B_exp.astype(np.float64)
    D = D_real[:, 0::2] + 1j * D_real[:, 1::2]
    assert np.allclose(D, A.astype(np.complex128) @ B.astype(np.complex128), rtol=1e-12, atol=1e-12)
