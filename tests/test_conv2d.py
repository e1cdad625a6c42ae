"""fp32 2-D convolution (im2col + 3xTF32 GEMM) through the C ABI against the direct fp64 oracle.

The reference ships no CPU Conv2D and no golden vectors for it, so the oracle restates the arithmetic of its CUDA path
(cross-correlation, output dims, zero border of kh // 2 and kw // 2, bottom bound) and is cross-checked here against an
independent numpy formulation; the bar is the fp32 GEMM's: |error| <= 1e-5 * sum |src . kernel| (observed ~1e-7).
"""
import numpy as np
import pytest

from oracle import binding as ob


def _numpy_conv(src, ker, strides, extend):
    """Independent formulation: pad, sliding windows, einsum."""
    sx, sy = strides
    H, W, C = src.shape
    n, kh, kw, _ = ker.shape
    s = src.astype(np.float64)
    if extend == 2:
        OH, OW = H // sy, W // sx
        s = s.copy()
        s[OH * sy:] = 0.0
        s = np.pad(s, ((kh // 2, kh), (kw // 2, kw), (0, 0)))
    else:
        OH, OW = (H - kh + 1) // sy, (W - kw + 1) // sx
    win = np.lib.stride_tricks.sliding_window_view(s, (kh, kw), axis=(0, 1))      # (H', W', C, kh, kw)
    win = win[::sy, ::sx][:OH, :OW]
    return np.einsum("yxcij,tijc->yxt", win, ker.astype(np.float64))


CPU_CASES = [((9, 11, 4), (3, 3, 3), (1, 1), 0), ((9, 11, 4), (2, 3, 3), (1, 1), 2), ((12, 10, 3), (5, 5, 3), (2, 2), 2),
             ((13, 10, 8), (1, 4, 2), (3, 2), 0), ((13, 11, 5), (2, 3, 5), (2, 3), 2), ((5, 5, 1), (1, 5, 5), (1, 1), 0)]


@pytest.mark.parametrize("case", CPU_CASES)
def test_oracle_against_numpy(case):
    (H, W, C), (n, kh, kw), strides, extend = case
    rng = np.random.default_rng(H * 100 + W)
    src = rng.uniform(-1, 1, (H, W, C)).astype(np.float32)
    ker = rng.uniform(-1, 1, (n, kh, kw, C)).astype(np.float32)
    D, mag = ob.conv2d(src, ker, strides, extend)
    ref = _numpy_conv(src, ker, strides, extend)
    assert D.shape == ref.shape
    assert np.abs(D - ref).max() <= 1e-12
    assert (mag >= np.abs(D) - 1e-12).all()


def test_out_dims_and_argument_checks():
    import ctypes
    from decx_b200 import capi
    oh, ow = ctypes.c_uint32(), ctypes.c_uint32()
    f = capi.lib.decxb200_conv2d_fp32_out_dims
    assert f(224, 224, 3, 3, 1, 1, 0, ctypes.byref(oh), ctypes.byref(ow)) == 0 and (oh.value, ow.value) == (222, 222)
    assert f(224, 225, 3, 3, 2, 2, 2, ctypes.byref(oh), ctypes.byref(ow)) == 0 and (oh.value, ow.value) == (112, 112)
    assert f(2, 2, 3, 3, 1, 1, 0, ctypes.byref(oh), ctypes.byref(ow)) != 0          # kernel larger than the source
    assert f(8, 8, 3, 3, 1, 1, 1, ctypes.byref(oh), ctypes.byref(ow)) != 0          # reflect border: not in the reference either
    assert f(8, 8, 3, 3, 0, 1, 0, ctypes.byref(oh), ctypes.byref(ow)) != 0
    assert capi.lib.decxb200_conv2d_fp32_workspace_bytes(8, 8, 4, 3, 3, 2, 1, 1, 0, 0, 0) > 0
    assert capi.lib.decxb200_conv2d_fp32_workspace_bytes(8, 8, 4, 3, 3, 0, 1, 1, 0, 0, 0) == 0
    # implicit form (planes of the bordered source) needs far less than the materialised im2col matrix
    big = capi.lib.decxb200_conv2d_fp32_workspace_bytes(256, 256, 64, 3, 3, 64, 1, 1, 2, 0, 63 + 2)
    small = capi.lib.decxb200_conv2d_fp32_workspace_bytes(256, 256, 64, 3, 3, 64, 1, 1, 2, 0, 64)
    assert 0 < small < big // 4
    # no device work is reached with bad arguments
    assert capi.lib.decxb200_conv2d_fp32(None, None, 8, 8, 4, 8, 4, None, 3, 3, 2, 3, 4, 36, None, 0, 4, 1, 1, 0, None, 0,
                                         None) == -1


# (H, W, C), (n, kh, kw), strides, extend, (src wpitch extra, dpitch extra)
GPU_CASES = [
    ((9, 11, 4), (3, 3, 3), (1, 1), 0, (0, 0)),
    ((9, 11, 4), (2, 3, 3), (1, 1), 2, (2, 4)),
    ((12, 10, 3), (5, 5, 3), (2, 2), 2, (0, 1)),          # C = 3 on dpitch 4: the reference's image layout
    ((13, 10, 8), (1, 4, 2), (3, 2), 0, (1, 0)),
    ((13, 11, 5), (2, 3, 5), (2, 3), 2, (0, 0)),           # odd channel count: scalar path
    ((64, 64, 16), (32, 3, 3), (1, 1), 2, (0, 0)),
    ((57, 93, 12), (17, 5, 7), (1, 2), 0, (3, 4)),
    ((128, 160, 32), (64, 3, 3), (1, 1), 0, (0, 0)),
    ((31, 29, 64), (128, 1, 1), (1, 1), 2, (0, 0)),         # pointwise
    ((40, 40, 4), (8, 11, 11), (4, 4), 2, (0, 0)),
    ((33, 70, 8), (12, 3, 3), (1, 1), 2, (5, 4)),           # 64-wide tile rows, pitched destination
    ((20, 300, 16), (260, 3, 5), (2, 1), 0, (0, 0)),        # more than 256 kernels: two tile columns of the wide tile
    ((9, 9, 32), (4, 9, 9), (1, 1), 2, (0, 0)),             # kernel as large as the image
    ((64, 64, 3), (16, 7, 7), (2, 2), 2, (0, 1)),           # RGB-like source, stride 2
    ((17, 19, 20), (8, 2, 2), (1, 1), 0, (0, 0)),           # even kernel, kw * C not a multiple of 32
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", GPU_CASES)
def test_conv2d_fp32(case):
    torch = pytest.importorskip("torch")
    from decx_b200 import blas
    (H, W, C), (n, kh, kw), strides, extend, (wextra, dextra) = case
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(H * 1000 + W * 10 + C)
    src = rng.uniform(-1, 1, (H, W, C)).astype(np.float32)
    ker = rng.uniform(-1, 1, (n, kh, kw, C)).astype(np.float32)
    ref, mag = ob.conv2d(src, ker, strides, extend)
    OH, OW = ob.conv2d_dims(H, W, kh, kw, strides, extend)

    def pitched(a, we, de):
        shape = a.shape[:-2] + (a.shape[-2] + we, a.shape[-1] + de)
        buf = torch.full(shape, float("nan"), dtype=torch.float32, device=dev)
        view = buf[..., :a.shape[-2], :a.shape[-1]]
        view.copy_(torch.from_numpy(a))
        return buf, view

    _, tsrc = pitched(src, wextra, dextra)
    _, tker = pitched(ker, 0, dextra)
    obuf = torch.full((OH, OW + wextra, n + dextra), float("nan"), dtype=torch.float32, device=dev)
    out = obuf[:, :OW, :n]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    blas.conv2d(tsrc, tker, strides, extend, out=out, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    from decx_b200 import capi
    implicit = capi.lib.decxb200_last_kernel_variant() >= 20000
    assert implicit == (n % 4 == 0 and (n + dextra) % 4 == 0)          # obuf is 16-byte aligned
    got = out.cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all()
    assert (np.abs(got - ref) <= 1e-5 * mag + 1e-30).all()
    full = obuf.cpu().numpy()
    assert np.isnan(full[:, :, n:]).all()                      # channel padding untouched
    if wextra:                                                  # row padding: left alone (implicit) or zeros
        pad = full[:, OW:, :n]
        assert np.isnan(pad).all() if implicit else (pad == 0).all()


@pytest.mark.gpu
def test_conv2d_matches_gemm_bitwise():
    """A 1 x 1 kernel over a dense tensor IS the fp32 GEMM (H*W x C times C x n): same bits as decxb200_gemm."""
    torch = pytest.importorskip("torch")
    from decx_b200 import blas, gemm
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(5)
    src = torch.rand((48, 40, 64), generator=g).to(dev) - 0.5
    ker = torch.rand((96, 1, 1, 64), generator=g).to(dev) - 0.5
    out = blas.conv2d(src, ker)
    ref = gemm.gemm(src.reshape(48 * 40, 64), ker.reshape(96, 64).t().contiguous())
    torch.cuda.synchronize()
    assert torch.equal(out.reshape(48 * 40, 96), ref)
