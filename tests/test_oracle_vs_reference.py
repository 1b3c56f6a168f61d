"""The C restatement against nnForge's own plain sources compiled in place (oracle/_ref), on
seeded random tensors including ragged sizes. Skipped where no reference build exists (the golden
fixture test covers those machines)."""
import numpy as np
import pytest

import synth
from util import assert_bits_equal

SHAPES = [(1, 1, 1, 1), (2, 3, 5, 7), (3, 4, 8, 8), (2, 21, 1, 1), (5, 2, 7, 7), (1, 7, 13, 3)]


@pytest.mark.parametrize("shape", SHAPES)
def test_elementwise(oracle, reference, shape):
    g = synth.rng(50, salt=sum(shape))
    x = synth.with_edges(g, synth.normal(g, shape, 0.0, 1.5))
    xs = synth.normal(g, shape)
    dy = synth.normal(g, shape)
    dx0 = synth.normal(g, shape)
    c = shape[1]
    gamma, beta, mean, invsigma = synth.bn_params(g, c)
    slope = synth.uniform(g, c, 0.0, 0.3)
    assert_bits_equal(oracle.bn_infer(x, gamma, beta, mean, invsigma), reference.bn_infer(x, gamma, beta, mean, invsigma)[0], "bn")
    for s in (0.0, 0.25, -0.5):
        assert_bits_equal(oracle.relu_fwd(x, s), reference.relu_fwd(x, s)[0], "relu")
        assert_bits_equal(oracle.relu_bwd(dy, x, s), reference.relu_bwd(dy, x, s)[0], "relu bwd")
        assert_bits_equal(oracle.relu_bwd(dy, x, s, dx=dx0), reference.relu_bwd(dy, x, s, dx=dx0)[0], "relu bwd add")
    assert_bits_equal(oracle.prelu_fwd(x, slope), reference.prelu_fwd(x, slope)[0], "prelu")
    assert_bits_equal(oracle.prelu_bwd_data(dy, x, slope), reference.prelu_bwd_data(dy, x, slope)[0], "prelu bwd")
    assert_bits_equal(oracle.prelu_bwd_data(dy, x, slope, dx=dx0), reference.prelu_bwd_data(dy, x, slope, dx=dx0)[0], "prelu bwd add")
    assert_bits_equal(oracle.prelu_bwd_weights(dy, xs, dslope=slope), reference.prelu_bwd_weights(dy, xs, dslope=slope)[0], "dslope")
    y = oracle.elu_fwd(x)
    assert_bits_equal(y, reference.elu_fwd(x)[0], "elu")
    assert_bits_equal(oracle.elu_bwd(dy, y), reference.elu_bwd(dy, y)[0], "elu bwd")
    assert_bits_equal(oracle.elu_bwd(dy, y, dx=dx0), reference.elu_bwd(dy, y, dx=dx0)[0], "elu bwd add")
    y = oracle.tanh_fwd(xs, 1.7159, 0.6666)
    assert_bits_equal(y, reference.tanh_fwd(xs, 1.7159, 0.6666)[0], "tanh")
    assert_bits_equal(oracle.tanh_bwd(dy, y, 1.7159, 0.6666), reference.tanh_bwd(dy, y, 1.7159, 0.6666)[0], "tanh bwd")
    y = oracle.sigmoid_fwd(x)
    assert_bits_equal(y, reference.sigmoid_fwd(x)[0], "sigmoid")
    assert_bits_equal(oracle.sigmoid_bwd(dy, y), reference.sigmoid_bwd(dy, y)[0], "sigmoid bwd")
    for k, alpha in ((1, 1.0), (2, 1.0), (3, 0.3)):
        ins = [x, xs, dy][:k]
        assert_bits_equal(oracle.add_fwd(ins, alpha), reference.add_fwd(ins, alpha)[0], "add")
    assert_bits_equal(oracle.add_bwd(dy, 0.3), reference.add_bwd(dy, 0.3)[0], "add bwd")
    assert_bits_equal(oracle.add_bwd(dy, 1.0, dx=dx0), reference.add_bwd(dy, 1.0, dx=dx0)[0], "add bwd add")


@pytest.mark.parametrize("shape", [(2, 1, 1, 1), (3, 21, 4, 5), (4, 1000, 1, 1), (2, 5, 1, 9), (1, 33, 3, 3)])
def test_softmax(oracle, reference, shape):
    g = synth.rng(51, salt=sum(shape))
    x = synth.normal(g, shape, 0.0, 3.0)
    dy = synth.normal(g, shape)
    y = oracle.softmax_fwd(x)
    assert_bits_equal(y, reference.softmax_fwd(x)[0], "softmax tester")
    assert_bits_equal(y, reference.softmax_fwd(x, updater=True)[0], "softmax updater")
    assert_bits_equal(oracle.softmax_bwd(dy, y), reference.softmax_bwd(dy, y)[0], "softmax bwd")
    assert_bits_equal(oracle.softmax_bwd(dy, y, dx=x), reference.softmax_bwd(dy, y, dx=x)[0], "softmax bwd add")


@pytest.mark.parametrize("shape", [(2, 1, 1, 1), (3, 21, 4, 5), (4, 1000, 1, 1), (2, 5, 1, 9)])
def test_negative_log_likelihood(oracle, reference, shape):
    g = synth.rng(53, salt=sum(shape))
    p = oracle.softmax_fwd(synth.normal(g, shape, 0.0, 3.0))
    p.flat[0] = 0.0  # clamped predictions, one of them under a positive target
    t = synth.targets(g, shape)
    t.flat[0] = 1.0
    mask = (synth.uniform(g, (shape[0], 1) + shape[2:], 0.0, 1.0) > 0.3).astype(np.float32) * synth.uniform(g, (shape[0], 1) + shape[2:], 0.5, 2.0)
    for m, scale in ((None, 1.0), (mask, 0.7), (mask, 0.0)):
        e = oracle.nll_fwd(p, t, m, scale)
        assert_bits_equal(e, reference.nll_fwd(p, t, m, scale)[0], "nll tester")
        assert_bits_equal(e, reference.nll_fwd(p, t, m, scale, updater=True)[0], "nll updater")
        assert_bits_equal(oracle.nll_bwd(p, t, m, scale), reference.nll_bwd(p, t, m, scale)[0], "nll bwd")
        seed = synth.normal(g, shape)
        assert_bits_equal(oracle.nll_bwd(p, t, m, scale, dx=seed), reference.nll_bwd(p, t, m, scale, dx=seed)[0], "nll bwd add")


@pytest.mark.parametrize("shape", [(2, 1, 1, 1), (3, 21, 4, 5), (4, 1000, 1, 1), (2, 5, 1, 9)])
def test_cross_entropy(oracle, reference, shape):
    """Forward against the reference's tester (the mask REPLACES the scale) and updater (scale * mask). The reference's plain backward
    action stores zeros - its gradient goes into a variable that shadows the stored one - so the restated gradient has no reference
    twin here; it is the expression that file computes, checked against a float64 evaluation."""
    g = synth.rng(55, salt=sum(shape))
    p = (1.0 / (1.0 + np.exp(-synth.normal(g, shape, 0.0, 2.0).astype(np.float64)))).astype(np.float32)
    t = synth.targets(g, shape)
    p.flat[0], t.flat[0] = 0.0, 1.0
    if p.size > 1:
        p.flat[1], t.flat[1] = 1.0, 0.0
    mask = (synth.uniform(g, (shape[0], 1) + shape[2:], 0.0, 1.0) > 0.3).astype(np.float32) * synth.uniform(g, (shape[0], 1) + shape[2:], 0.5, 2.0)
    for m, scale in ((None, 1.0), (None, 0.7), (mask, 0.7), (mask, 0.0)):
        assert_bits_equal(oracle.cross_entropy_fwd(p, t, m, scale, mask_replaces_scale=True), reference.cross_entropy_fwd(p, t, m, scale)[0], "cross entropy tester")
        assert_bits_equal(oracle.cross_entropy_fwd(p, t, m, scale), reference.cross_entropy_fwd(p, t, m, scale, updater=True)[0], "cross entropy updater")
        assert not reference.cross_entropy_bwd(p, t, m, scale)[0].any()   # the plain backend's own backward action: zeros
        total = np.float64(np.float32(scale)) * (m.astype(np.float64) if m is not None else 1.0)
        pd, td = p.astype(np.float64), t.astype(np.float64)
        pos, neg = np.where(td > 0, td / np.maximum(pd, 1e-20), 0.0), np.where(td < 1, (1 - td) / np.maximum(1 - pd, 1e-20), 0.0)
        want = (pos - neg) * total
        got = oracle.cross_entropy_bwd(p, t, m, scale)
        assert np.all(np.abs(got - want) <= 1e-6 * (pos + neg) * np.abs(total) + 1e-30)   # the two terms cancel for soft targets
        seed = synth.normal(g, shape)
        assert_bits_equal(oracle.cross_entropy_bwd(p, t, m, scale, dx=seed), (seed + got).astype(np.float32), "cross entropy bwd add")


@pytest.mark.parametrize("shape", [(2, 1, 1, 1), (3, 21, 4, 5), (4, 1000, 1, 1), (2, 5, 1, 9)])
def test_accuracy(oracle, reference, shape):
    g = synth.rng(54, salt=sum(shape))
    p = oracle.softmax_fwd(synth.normal(g, shape, 0.0, 3.0))
    if shape[1] > 1:
        p[0, 1] = p[0, 0]  # equal predictions: the smaller channel index wins
    t = synth.targets(g, shape)
    mask = (synth.uniform(g, (shape[0], 1) + shape[2:], 0.0, 1.0) > 0.3).astype(np.float32) * synth.uniform(g, (shape[0], 1) + shape[2:], 0.5, 2.0)
    for m in (None, mask):
        for top_n in (1, 3):
            a = oracle.accuracy_fwd(p, t, m, top_n)
            assert_bits_equal(a, reference.accuracy_fwd(p, t, m, top_n)[0], "accuracy tester")
            assert_bits_equal(a, reference.accuracy_fwd(p, t, m, top_n, updater=True)[0], "accuracy updater")


@pytest.mark.parametrize("shape,win", [((2, 3, 8, 12), (4, 2)), ((3, 5, 7, 7), (7, 7)), ((2, 4, 6, 6), (1, 1)), ((1, 2, 14, 14), (2, 2)), ((2, 3, 4, 9), (3, 4))])
def test_average_subsampling(oracle, reference, shape, win):
    """mult = 1: the plain backend's default effective alpha for spatial windows (it ignores the window size)."""
    g = synth.rng(55, salt=sum(shape))
    x = synth.normal(g, shape)
    y = oracle.avgpool_fwd(x, win, mult=1.0)
    assert_bits_equal(y, reference.avgpool_fwd(x, win)[0], "average subsampling tester")
    assert_bits_equal(y, reference.avgpool_fwd(x, win, updater=True)[0], "average subsampling updater")
    dy = synth.normal(g, y.shape)
    assert_bits_equal(oracle.avgpool_bwd(dy, shape, win, mult=1.0), reference.avgpool_bwd(dy, shape, win)[0], "average subsampling bwd")
    seed = synth.normal(g, shape)
    assert_bits_equal(oracle.avgpool_bwd(dy, shape, win, mult=1.0, dx=seed), reference.avgpool_bwd(dy, shape, win, dx=seed)[0], "average subsampling bwd add")


@pytest.mark.parametrize("hw", [(7, 7), (9, 11), (14, 14), (5, 8)])
@pytest.mark.parametrize("win,stride", [((3, 3), (2, 2)), ((2, 2), (2, 2)), ((3, 3), (1, 1)), ((2, 3), (2, 1)), ((1, 1), (1, 1)), ((5, 5), (3, 3))])
def test_maxpool(oracle, reference, hw, win, stride):
    g = synth.rng(52, salt=hw[0] * 31 + win[0] * 7 + stride[1])
    x = oracle.relu_fwd(synth.normal(g, (2, 3) + hw), 0.0)  # many exact ties and -0/+0 mixes
    for is_min in (False, True):
        y, idx = oracle.maxpool_fwd(x, win, stride, is_min=is_min)
        ry, ridx, _ = reference.maxpool_fwd(x, win, stride, is_min=is_min)
        assert_bits_equal(y, ry, "pool values")
        assert_bits_equal(idx, ridx, "pool argmax")
        assert_bits_equal(y, reference.maxpool_tester_fwd(x, win, stride, is_min=is_min)[0], "pool tester values")
    y, idx = oracle.maxpool_fwd(x, win, stride)
    dy = synth.normal(g, y.shape)
    assert_bits_equal(oracle.maxpool_bwd(dy, idx, x.shape), reference.maxpool_bwd(dy, idx, x.shape)[0], "pool bwd")


@pytest.mark.parametrize("shape,mean,std", [((6, 5, 7, 3), 100.0, 3.0), ((3, 8, 1, 1), 0.0, 1.0), ((2, 3, 14, 14), -7.5, 0.01), ((1, 4, 5, 5), 0.0, 1000.0)])
def test_feature_map_statistics(oracle, reference, shape, mean, std):
    """stat_data_bunch_writer: Welford's update value by value in double; the restatement must give the same bits however the
    entries are cut into batches."""
    g = synth.rng(56, salt=sum(shape))
    y = synth.normal(g, shape, mean, std)
    expect = reference.feature_map_stats(y)
    assert_bits_equal(oracle.feature_map_stats([y]), expect, "statistics, one batch")
    if shape[0] > 2:
        assert_bits_equal(oracle.feature_map_stats([y[:1], y[1:]]), expect, "statistics, two batches")
