"""The C restatement (oracle/nnf_oracle.c) against golden vectors produced by nnForge's own plain
backend (tests/golden/make_golden.py). Bit-exact everywhere: both are built without -ffast-math and
without FMA contraction, and call the same libm expf."""
import os

import numpy as np
import pytest

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
