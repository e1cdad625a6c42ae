"""GPU tests of the transpose and element-cast entry points: bit-exact against numpy."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

SHAPES = [(1, 1), (1, 77), (77, 1), (31, 33), (64, 64), (65, 63), (127, 130), (300, 517), (1000, 999), (2049, 1025)]
DTYPES = [torch.uint8, torch.float16, torch.float32, torch.float64, torch.complex64, torch.complex128]


@pytest.fixture(scope="module")
def Bl():
    from decx_b200 import blas
    return blas


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda:0")


def _rand(shape, dtype, dev, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    if dtype == torch.uint8:
        return torch.randint(0, 256, shape, dtype=torch.uint8, generator=g).to(dev)
    if dtype.is_complex:
        return torch.complex(torch.randn(shape, generator=g, dtype=torch.float64), torch.randn(shape, generator=g, dtype=torch.float64)).to(dtype).to(dev)
    return torch.randn(shape, generator=g, dtype=torch.float64).to(dtype).to(dev)


def _guarded(rows, cols, dtype, dev, pad_bytes=128):
    """NaN / 0xFF filled buffer whose logical view has a 128-byte aligned pitch; returns (buffer, view)."""
    e = torch.empty(0, dtype=dtype).element_size()
    pitch = ((cols * e + pad_bytes - 1) // pad_bytes * pad_bytes) // e
    raw = torch.full(((rows + 2) * pitch * e,), 0xFF, dtype=torch.uint8, device=dev)
    buf = raw.view(dtype).view(rows + 2, pitch)
    return raw, buf, buf[1:rows + 1, :cols]


def _untouched(raw, buf, rows, cols):
    e = buf.element_size()
    b = raw.view(rows + 2, -1)
    assert (b[0] == 0xFF).all() and (b[rows + 1] == 0xFF).all(), "rows outside the matrix were written"
    assert (b[1:rows + 1, cols * e:] == 0xFF).all(), "pitch padding was written"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", SHAPES)
def test_transpose_bit_exact(Bl, dev, shape, dtype):
    rows, cols = shape
    src = _rand(shape, dtype, dev, rows * 5 + cols)
    _, _, sview = _guarded(rows, cols, dtype, dev)
    sview.copy_(src)
    raw, buf, dview = _guarded(cols, rows, dtype, dev)
    Bl.transpose(sview, out=dview)
    torch.cuda.synchronize()
    assert torch.equal(dview, src.t())
    _untouched(raw, buf, cols, rows)


def test_transpose_of_unaligned_fp16_views(Bl, dev):
    """Odd pitches / bases off the 4-byte grid take the element-wise kernel."""
    base = _rand((70, 131), torch.float16, dev, 1)
    src = base[:, 1:]                         # base address off by 2 bytes, pitch 131
    out = torch.zeros((130, 71), dtype=torch.float16, device=dev)[:, :70]
    Bl.transpose(src, out=out)
    torch.cuda.synchronize()
    assert torch.equal(out, src.t())


CASTS = [(torch.float32, torch.float16), (torch.float16, torch.float32), (torch.float32, torch.float64),
         (torch.float64, torch.float32), (torch.int32, torch.float32), (torch.float32, torch.int32)]


@pytest.mark.parametrize("pair", CASTS)
@pytest.mark.parametrize("shape", [(1, 1), (3, 7), (64, 64), (129, 255), (1000, 1001), (517, 4099)])
def test_cast_bit_exact_against_numpy(Bl, dev, pair, shape):
    sdt, ddt = pair
    rows, cols = shape
    rng = np.random.default_rng(rows + cols)
    npdt = {torch.float16: np.float16, torch.float32: np.float32, torch.float64: np.float64, torch.int32: np.int32}
    if sdt == torch.int32:
        x = rng.integers(-2 ** 31, 2 ** 31 - 1, shape, dtype=np.int64).astype(np.int32)
    elif ddt == torch.int32:
        x = (rng.standard_normal(shape) * 10.0 ** rng.integers(0, 6, shape)).astype(np.float32)
        x.flat[:4] = [0.5, 1.5, 2.5, -2.5][: x.size]                  # ties go to the even integer
    else:
        x = (rng.standard_normal(shape) * 10.0 ** rng.integers(-8, 8, shape)).astype(npdt[sdt])
        if sdt == torch.float32 and ddt == torch.float16 and x.size >= 6:
            x.flat[:6] = [65504.0, 65519.9, 65520.0, 1e-8, 6.0e-8, -7e4]   # largest half, just below / at the overflow tie, subnormals
    _, _, sview = _guarded(rows, cols, sdt, dev)
    sview.copy_(torch.from_numpy(x).to(dev))
    raw, buf, dview = _guarded(rows, cols, ddt, dev)
    Bl.cast(sview, ddt, out=dview)
    torch.cuda.synchronize()
    with np.errstate(over="ignore"):
        expect = np.rint(x).astype(np.int32) if ddt == torch.int32 else x.astype(npdt[ddt])
    got = dview.cpu().numpy()
    assert np.array_equal(got.view(np.uint8), expect.view(np.uint8))
    _untouched(raw, buf, rows, cols)


def test_cast_then_gemm_pipeline(Bl, dev):
    """What the cast is for: fp32 operands narrowed on the device feed the fp16 GEMM."""
    from decx_b200 import gemm as G
    from oracle import binding as ob
    rng = np.random.default_rng(3)
    A = rng.normal(0, 0.1, (300, 200)).astype(np.float32)
    B = rng.normal(0, 0.1, (200, 136)).astype(np.float32)
    hA, hB = Bl.cast(torch.from_numpy(A).to(dev), torch.float16), Bl.cast(torch.from_numpy(B).to(dev), torch.float16)
    D = G.gemm(hA, hB)
    torch.cuda.synchronize()
    Ah, Bh = A.astype(np.float16), B.astype(np.float16)
    assert ob.metric(D.cpu().numpy(), ob.gemm(Ah, Bh), Ah, Bh) <= 1e-2
