import numpy as np


def assert_bits_equal(a, b, what=""):
    """Bit-exact fp32 comparison (signed zeros distinguished); NaNs only need to coincide."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    assert a.shape == b.shape, (what, a.shape, b.shape)
    if a.dtype == np.float32:
        ai, bi = a.view(np.uint32), b.view(np.uint32)
        both_nan = np.isnan(a) & np.isnan(b)
        bad = (ai != bi) & ~both_nan
    else:
        bad = a != b
    if bad.any():
        pos = np.argwhere(bad)[0]
        raise AssertionError("%s: %d of %d elements differ; first at %s: %r vs %r"
                             % (what, int(bad.sum()), a.size, tuple(pos), a[tuple(pos)], b[tuple(pos)]))


# Tolerance the path's floating-point results must meet against the plain backend:
# |got - want| <= 1e-6 + 1e-5*|want|.
RTOL = 1e-5
ATOL = 1e-6


def assert_close(got, want, what="", rtol=RTOL, atol=ATOL):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    same_special = (np.isnan(got) & np.isnan(want)) | (np.isinf(got) & np.isinf(want) & (np.sign(got) == np.sign(want)))
    with np.errstate(invalid="ignore"):
        err = np.abs(got - want)
        bad = ~same_special & ~(err <= atol + rtol * np.abs(want))
    if bad.any():
        pos = tuple(np.argwhere(bad)[0])
        raise AssertionError("%s: %d of %d outside tolerance; first at %s: got %r want %r"
                             % (what, int(bad.sum()), got.size, pos, got[pos], want[pos]))


def assert_close_off_kink(got, want, u, what="", rtol=RTOL, atol=ATOL, halfwidth=1e-5, max_fraction=1e-4):
    """assert_close for the gradient behind a rectifier (ReLU, PReLU) whose input u was itself computed in fp32: the
    derivative jumps at u = 0, so an element whose u is within rounding of 0 may take either side, and two correct
    implementations differ there by a finite amount. Those elements (|u| < halfwidth) are left out - and must be few."""
    near = np.abs(np.asarray(u, dtype=np.float64)) < halfwidth
    assert near.mean() <= max_fraction, "%s: %d elements at the kink" % (what, int(near.sum()))
    got = np.where(near, 0.0, np.asarray(got, dtype=np.float64))
    want = np.where(near, 0.0, np.asarray(want, dtype=np.float64))
    assert_close(got, want, what, rtol, atol)
