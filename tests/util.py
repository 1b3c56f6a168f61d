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


def assert_no_worse_than_fp32_checker(got, want32, exact64, what="", rtol=RTOL, atol=ATOL, factor=2.0, leave_out=None):
    """The companion of a comparison made at a widened absolute tolerance. Errors are measured against the float64 twin in
    units of the path's tolerance (atol + rtol*|exact|). Where the GPU result is further than one unit from the exact value, the
    fp32 checker must be that far from it too (within `factor`): the widening then absorbs the rounding of an fp32 evaluation
    of the expression, which the checker shows just as much, and not an error of the kernel."""
    exact = np.asarray(exact64, dtype=np.float64)
    unit = atol + rtol * np.abs(exact)
    with np.errstate(invalid="ignore"):
        e_got = np.abs(np.asarray(got, dtype=np.float64) - exact) / unit
        e_own = np.abs(np.asarray(want32, dtype=np.float64) - exact) / unit
    keep = np.isfinite(e_got) & np.isfinite(e_own)
    if leave_out is not None:
        keep &= ~leave_out
    worst_got, worst_own = float(e_got[keep].max(initial=0.0)), float(e_own[keep].max(initial=0.0))
    assert worst_got <= max(1.0, factor * worst_own), \
        "%s: the GPU result is %.2f tolerance units from the float64 value, the fp32 checker only %.2f" % (what, worst_got, worst_own)
    return worst_got, worst_own
