"""The C restatement (oracle/nnf_oracle.c) against golden vectors produced by nnForge's own plain
backend (tests/golden/make_golden.py). Bit-exact everywhere: both are built without -ffast-math and
without FMA contraction, and call the same libm expf."""
import os

import numpy as np
import pytest

import synth
from util import assert_bits_equal

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "plain_backend.npz"))


def test_bn_infer(oracle):
    assert_bits_equal(oracle.bn_infer(G["x"], G["gamma"], G["beta"], G["mean"], G["invsigma"]), G["bn_infer"], "bn_infer")


def test_relu(oracle):
    assert_bits_equal(oracle.relu_fwd(G["x"], 0.0), G["relu0"], "relu slope 0")
    assert np.signbit(G["relu0"][G["x"] < 0]).all(), "slope 0 must give -0.0 for negative inputs"
    assert_bits_equal(oracle.relu_fwd(G["x"], 0.1), G["relu01"], "relu slope 0.1")
    assert_bits_equal(oracle.relu_bwd(G["dy"], G["x"], 0.1), G["relu_bwd"], "relu bwd")
    assert_bits_equal(oracle.relu_bwd(G["dy"], G["x"], 0.0, dx=G["dx0"]), G["relu_bwd_add"], "relu bwd add")


def test_prelu(oracle):
    assert_bits_equal(oracle.prelu_fwd(G["x"], G["slope"]), G["prelu"], "prelu")
    assert_bits_equal(oracle.prelu_bwd_data(G["dy"], G["x"], G["slope"]), G["prelu_bwd"], "prelu bwd")
    assert_bits_equal(oracle.prelu_bwd_data(G["dy"], G["x"], G["slope"], dx=G["dx0"]), G["prelu_bwd_add"], "prelu bwd add")
    assert_bits_equal(oracle.prelu_bwd_weights(G["dy"], G["xs"], dslope=G["slope"]), G["prelu_dslope"], "prelu dslope")


def test_elu_tanh_sigmoid(oracle):
    assert_bits_equal(oracle.elu_fwd(G["x"]), G["elu"], "elu")
    assert_bits_equal(oracle.elu_bwd(G["dy"], G["elu"]), G["elu_bwd"], "elu bwd")
    assert_bits_equal(oracle.tanh_fwd(G["xs"], 1.7159, 0.6666), G["tanh"], "tanh")
    assert_bits_equal(oracle.tanh_bwd(G["dy"], G["tanh"], 1.7159, 0.6666), G["tanh_bwd"], "tanh bwd")
    assert_bits_equal(oracle.sigmoid_fwd(G["x"]), G["sigmoid"], "sigmoid")
    assert_bits_equal(oracle.sigmoid_bwd(G["dy"], G["sigmoid"], dx=G["dx0"]), G["sigmoid_bwd"], "sigmoid bwd add")


def test_add(oracle):
    assert_bits_equal(oracle.add_fwd([G["x"], G["r"]], 1.0), G["add2"], "add2")
    assert_bits_equal(oracle.add_fwd([G["xs"], G["r"], G["dy"]], 0.5), G["add3_alpha"], "add3")
    assert_bits_equal(oracle.add_bwd(G["dy"], 0.5), G["add_bwd"], "add bwd")


def test_softmax(oracle):
    assert_bits_equal(oracle.softmax_fwd(G["logits"]), G["softmax"], "softmax spatial")
    assert_bits_equal(oracle.softmax_bwd(G["dyl"], G["softmax"]), G["softmax_bwd"], "softmax bwd")
    assert_bits_equal(oracle.softmax_fwd(G["row"]), G["softmax_row"], "softmax rows")


@pytest.mark.parametrize("name", ["ce", "ce_row"])
def test_cross_entropy_golden(oracle, name):
    p, t, mask = G[name + "_p"], G[name + "_t"], G[name + "_mask"]
    assert_bits_equal(oracle.cross_entropy_fwd(p, t, mask, 0.7, mask_replaces_scale=True), G[name + "_err_tester"], name + " forward, tester")
    assert_bits_equal(oracle.cross_entropy_fwd(p, t, mask, 0.7), G[name + "_err_updater"], name + " forward, updater")
    assert_bits_equal(oracle.cross_entropy_fwd(p, t, None, 1.3), G[name + "_err_nomask"], name + " forward, no mask")
    assert not G[name + "_plain_backward"].any()      # what the plain backend's backward action stores
    assert oracle.cross_entropy_bwd(p, t, mask, 0.7).any()


@pytest.mark.parametrize("name", ["nll", "nll_row"])
def test_negative_log_likelihood(oracle, name):
    p, t, mask = G[name + "_p"], G[name + "_t"], G[name + "_mask"]
    assert_bits_equal(oracle.nll_fwd(p, t, mask, 0.7), G[name + "_err"], name + " forward")
    assert_bits_equal(oracle.nll_fwd(p, t, None, 1.0), G[name + "_err_nomask"], name + " forward, no mask")
    assert_bits_equal(oracle.nll_bwd(p, t, mask, 0.7), G[name + "_grad"], name + " gradient")


def test_average_subsampling(oracle):
    y = oracle.avgpool_fwd(G["avg_x"], (4, 2), mult=1.0)
    assert_bits_equal(y, G["avg_4x2"], "average subsampling 4x2")
    assert_bits_equal(oracle.avgpool_bwd(G["avg_4x2_dy"], G["avg_x"].shape, (4, 2), mult=1.0), G["avg_4x2_dx"], "average subsampling 4x2 bwd")
    assert_bits_equal(oracle.avgpool_fwd(G["avg_gx"], (7, 7), mult=1.0), G["avg_global"], "global pooling 7x7")


@pytest.mark.parametrize("name", ["nll", "nll_row"])
def test_accuracy(oracle, name):
    p, t, mask = G[name + "_acc_p"], G[name + "_t"], G[name + "_mask"]
    assert_bits_equal(oracle.accuracy_fwd(p, t, mask, 3), G[name + "_acc3"], name + " top-3 accuracy")
    assert_bits_equal(oracle.accuracy_fwd(p, t, None, 1), G[name + "_acc1_nomask"], name + " top-1 accuracy, no mask")


@pytest.mark.parametrize("name,win,stride", [("pool32", (3, 3), (2, 2)), ("pool22", (2, 2), (2, 2)), ("pool_3x2_s1x2", (3, 2), (1, 2))])
def test_maxpool(oracle, name, win, stride):
    y, idx = oracle.maxpool_fwd(G["px"], win, stride)
    assert_bits_equal(y, G[name + "_y"], name + " values")
    assert_bits_equal(idx, G[name + "_idx"], name + " argmax")
    assert_bits_equal(oracle.maxpool_bwd(G[name + "_dy"], idx, G["px"].shape), G[name + "_dx"], name + " bwd")


def test_maxpool_min(oracle):
    y, idx = oracle.maxpool_fwd(G["px"], (3, 3), (2, 2), is_min=True)
    assert_bits_equal(y, G["pool32min_y"], "min values")
    assert_bits_equal(idx, G["pool32min_idx"], "min argmax")


def test_feature_map_statistics(oracle):
    y = G["stat_y"]
    assert_bits_equal(oracle.feature_map_stats([y]), G["stat_minmaxavgstd"], "per-feature-map min / max / average / std_dev")
    assert_bits_equal(oracle.feature_map_stats([y[:1], y[1:4], y[4:]]), G["stat_minmaxavgstd"], "same, fed in three batches")


def _np_apply_gradient(kind, w, gr, prev, prev2, lr, norm, wd, m, m2, it):
    """The optimiser expressions of nnforge/plain/backward_propagation_plain.cpp:826-985 written with numpy float32 scalars
    (every numpy operation rounds once, like C compiled without contraction): an independent statement of the same formulas,
    because that file of the reference cannot be compiled here."""
    f = np.float32
    lr, norm, wd, m, m2 = f(lr), f(norm), f(wd), f(m), f(m2)
    total = gr * norm - w * wd
    if kind == "none":
        upd = lr * total
    elif kind == "vanilla":
        upd = prev * m + lr * total
        prev[...] = upd
    elif kind == "nesterov":
        fresh = prev * m + lr * total
        upd = (m + f(1.0)) * fresh - m * prev
        prev[...] = fresh
    else:
        import math
        import ctypes
        libm = ctypes.CDLL("libm.so.6")
        libm.powf.restype = ctypes.c_float
        libm.powf.argtypes = [ctypes.c_float, ctypes.c_float]
        inv1 = f(1.0) / (f(1.0) - f(libm.powf(m, float(it))))
        inv2 = f(1.0) / (f(1.0) - f(libm.powf(m2, float(it))))
        b1 = m * prev + (f(1.0) - m) * total
        b2 = m2 * prev2 + (f(1.0) - m2) * total * total
        upd = lr * (b1 * inv1) / (np.sqrt(b2 * inv2) + f(1.0e-8))
        prev[...] = b1
        prev2[...] = b2
    return (w + upd).astype(np.float32), float(np.sum(np.abs(upd).astype(np.float64)))


@pytest.mark.parametrize("kind", ["none", "vanilla", "nesterov", "adam"])
def test_optimiser_step_matches_an_independent_statement(oracle, kind):
    g = synth.rng(81, salt=len(kind))
    count = 301
    w, gr = synth.normal(g, (count,)), synth.normal(g, (count,), 0.0, 5.0)
    prev, prev2 = synth.normal(g, (count,), 0.0, 0.01), np.abs(synth.normal(g, (count,), 0.0, 0.1))
    for it in (1, 2, 50):
        ow, ogr, op, op2 = w.copy(), gr.copy(), prev.copy(), prev2.copy()
        acc = oracle.apply_gradient(ow, ogr, op, op2, kind, 0.02, 1.0 / 32, 0.0005, 0.9, 0.999, it)
        ep, ep2 = prev.copy(), prev2.copy()
        ew, eacc = _np_apply_gradient(kind, w, gr, ep, ep2, 0.02, 1.0 / 32, 0.0005, 0.9, 0.999, it)
        assert_bits_equal(ow, ew, kind + " weights")
        assert not ogr.any()
        if kind != "none":
            assert_bits_equal(op, ep, kind + " previous update")
        if kind == "adam":
            assert_bits_equal(op2, ep2, kind + " second moment")
        assert abs(acc - eacc) <= 1e-12 * abs(eacc)
        w, prev, prev2 = ow, op, op2
        gr = synth.normal(g, (count,), 0.0, 5.0)
