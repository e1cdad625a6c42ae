"""Helpers shared by the GPU parity tests."""
import numpy as np

TOL = {"float32": 1e-5, "complex64": 1e-5, "float16": 1e-2}   # parity metric limits of this path


def make_inputs(dtype, M, N, K, seed, dist="uniform", with_c=False):
    rng = np.random.default_rng(seed)

    def real(r, c):
        if dist == "uniform":
            return rng.uniform(-1, 1, (r, c))
        if dist == "normal":
            return rng.normal(0, 1, (r, c))
        if dist == "small":
            return rng.normal(0, 0.02, (r, c))
        raise ValueError(dist)

    def mk(r, c):
        if np.dtype(dtype).kind == "c":
            return (real(r, c) + 1j * real(r, c)).astype(dtype)
        return real(r, c).astype(dtype)

    A, B = mk(M, K), mk(K, N)
    C = mk(M, N) if with_c else None
    return A, B, C


def pitch_elems(cols, itemsize):
    """Row pitch of a DECX device matrix: width rounded up to 128 bytes."""
    return ((cols * itemsize + 127) // 128 * 128) // itemsize


class Guarded:
    """A pitched device matrix surrounded by a NaN pattern: padding columns and a red zone of
    rows before and after.  ``check()`` asserts that nothing outside the logical matrix changed."""

    def __init__(self, torch, host, device, fill_logical=None, red_rows=3):
        self.torch = torch
        r, c = host.shape
        t = torch.from_numpy(np.ascontiguousarray(host))
        p = pitch_elems(c, t.element_size())
        self.red = red_rows
        nan = complex("nan+nanj") if t.is_complex() else float("nan")
        self.buf = torch.full((r + 2 * red_rows, p), nan, dtype=t.dtype, device=device)
        self.view = self.buf[red_rows:red_rows + r, :c]
        if fill_logical is None:
            self.view.copy_(t.to(device))
        else:
            self.view.fill_(fill_logical)
        self.rows, self.cols, self.pitch = r, c, p

    def check(self):
        torch = self.torch
        b = torch.view_as_real(self.buf) if self.buf.is_complex() else self.buf
        w = 2 if self.buf.is_complex() else 1
        assert torch.isnan(b[: self.red]).all(), "rows before the matrix were written"
        assert torch.isnan(b[self.red + self.rows:]).all(), "rows after the matrix were written"
        if self.pitch > self.cols:
            pad = b[self.red:self.red + self.rows, self.cols:] if w == 1 else b[self.red:self.red + self.rows, self.cols:, :]
            assert torch.isnan(pad).all(), "pitch padding was written"
