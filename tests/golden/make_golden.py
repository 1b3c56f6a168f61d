"""Generates tests/golden/plain_backend.npz from nnForge's own plain (CPU) backend.

Run in a container that has the reference checkout (it compiles the reference's plain sources in
place through oracle/build_ref.py and calls them through oracle/ref_capi.cpp):

    python tests/golden/make_golden.py

Every case stores its inputs and the reference outputs, so the fixture is self-contained and the
parity tests can replay it on machines where the reference is absent.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import synth  # noqa: E402
from oracle import Reference  # noqa: E402


def main():
    ref = Reference()
    assert ref.available, "reference build missing"
    g = synth.rng(99)
    out = {}
    shape = (3, 5, 6, 7)
    x = synth.with_edges(g, synth.normal(g, shape, 0.0, 1.5))
    dy = synth.normal(g, shape)
    dx0 = synth.normal(g, shape)
    gamma, beta, mean, invsigma = synth.bn_params(g, shape[1])
    slope = synth.uniform(g, shape[1], 0.0, 0.3)
    out.update(x=x, dy=dy, dx0=dx0, gamma=gamma, beta=beta, mean=mean, invsigma=invsigma, slope=slope)

    out["bn_infer"] = ref.bn_infer(x, gamma, beta, mean, invsigma)[0]
    out["relu0"] = ref.relu_fwd(x, 0.0)[0]
    out["relu01"] = ref.relu_fwd(x, 0.1)[0]
    out["relu_bwd"] = ref.relu_bwd(dy, x, 0.1)[0]
    out["relu_bwd_add"] = ref.relu_bwd(dy, x, 0.0, dx=dx0)[0]
    out["prelu"] = ref.prelu_fwd(x, slope)[0]
    out["prelu_bwd"] = ref.prelu_bwd_data(dy, x, slope)[0]
    out["prelu_bwd_add"] = ref.prelu_bwd_data(dy, x, slope, dx=dx0)[0]
    xs = synth.normal(g, shape)  # finite values for the long sum
    out["xs"] = xs
    out["prelu_dslope"] = ref.prelu_bwd_weights(dy, xs, dslope=slope)[0]
    out["elu"] = ref.elu_fwd(x)[0]
    out["elu_bwd"] = ref.elu_bwd(dy, out["elu"])[0]
    out["tanh"] = ref.tanh_fwd(xs, 1.7159, 0.6666)[0]
    out["tanh_bwd"] = ref.tanh_bwd(dy, out["tanh"], 1.7159, 0.6666)[0]
    out["sigmoid"] = ref.sigmoid_fwd(x)[0]
    out["sigmoid_bwd"] = ref.sigmoid_bwd(dy, out["sigmoid"], dx=dx0)[0]
    r = synth.with_edges(g, synth.normal(g, shape))
    out["r"] = r
    out["add2"] = ref.add_fwd([x, r], 1.0)[0]
    out["add3_alpha"] = ref.add_fwd([xs, r, dy], 0.5)[0]
    out["add_bwd"] = ref.add_bwd(dy, 0.5)[0]
    logits = synth.normal(g, (4, 21, 3, 5), 0.0, 2.0)
    out["logits"] = logits
    out["softmax"] = ref.softmax_fwd(logits)[0]
    dyl = synth.normal(g, logits.shape)
    out["dyl"] = dyl
    out["softmax_bwd"] = ref.softmax_bwd(dyl, out["softmax"])[0]
    row = synth.normal(g, (5, 1000, 1, 1), 0.0, 3.0)
    out["row"] = row
    out["softmax_row"] = ref.softmax_fwd(row)[0]
    # pooling: ReLU'd input so that ties (all-zero windows, +0/-0 mixes) are exercised
    px = ref.relu_fwd(synth.normal(g, (2, 3, 9, 11)), 0.0)[0]
    out["px"] = px
    for name, win, stride in (("pool32", (3, 3), (2, 2)), ("pool22", (2, 2), (2, 2)), ("pool_3x2_s1x2", (3, 2), (1, 2))):
        y, idx, _ = ref.maxpool_fwd(px, win, stride)
        out[name + "_y"], out[name + "_idx"] = y, idx
        pdy = synth.normal(g, y.shape)
        out[name + "_dy"] = pdy
        out[name + "_dx"] = ref.maxpool_bwd(pdy, idx, px.shape)[0]
    y, idx, _ = ref.maxpool_fwd(px, (3, 3), (2, 2), is_min=True)
    out["pool32min_y"], out["pool32min_idx"] = y, idx
    # negative log likelihood on the softmax outputs above (appended last: the vectors before it keep their draws)
    for name, probs in (("nll", out["softmax"]), ("nll_row", out["softmax_row"])):
        probs = probs.copy()
        probs.flat[0] = 0.0       # clamped to 1e-20
        probs.flat[1] = 1.0e-30
        t = synth.targets(g, probs.shape)
        t.flat[0] = 1.0           # a clamped prediction that counts
        mask = (synth.uniform(g, (probs.shape[0], 1) + probs.shape[2:], 0.0, 1.0) > 0.3).astype(np.float32) * synth.uniform(g, (probs.shape[0], 1) + probs.shape[2:], 0.5, 2.0)
        out[name + "_p"], out[name + "_t"], out[name + "_mask"] = probs, t, mask
        out[name + "_err"] = ref.nll_fwd(probs, t, mask, 0.7)[0]
        out[name + "_err_nomask"] = ref.nll_fwd(probs, t, None, 1.0, updater=True)[0]
        out[name + "_grad"] = ref.nll_bwd(probs, t, mask, 0.7)[0]
    # top-n accuracy on the same predictions and targets (ties between predictions included)
    for name in ("nll", "nll_row"):
        probs = out[name + "_p"].copy()
        probs[0, 1] = probs[0, 0]
        out[name + "_acc_p"] = probs
        out[name + "_acc3"] = ref.accuracy_fwd(probs, out[name + "_t"], out[name + "_mask"], 3)[0]
        out[name + "_acc1_nomask"] = ref.accuracy_fwd(probs, out[name + "_t"], None, 1, updater=True)[0]
    # average subsampling (the plain backend's default effective alpha for spatial windows is 1: it sums)
    ax = synth.normal(g, (2, 3, 8, 12))
    out["avg_x"] = ax
    out["avg_4x2"] = ref.avgpool_fwd(ax, (4, 2))[0]
    ady = synth.normal(g, out["avg_4x2"].shape)
    out["avg_4x2_dy"] = ady
    out["avg_4x2_dx"] = ref.avgpool_bwd(ady, ax.shape, (4, 2))[0]
    gx = synth.normal(g, (3, 5, 7, 7))
    out["avg_gx"] = gx
    out["avg_global"] = ref.avgpool_fwd(gx, (7, 7), updater=True)[0]
    # per-feature-map statistics of a layer output (stat_data_bunch_writer), values far from zero mean
    sy = synth.normal(g, (6, 5, 7, 3), 100.0, 3.0)
    out["stat_y"] = sy
    out["stat_minmaxavgstd"] = ref.feature_map_stats(sy)
    # cross entropy on sigmoid-like predictions with hard and soft targets (appended last: the vectors before it keep their draws).
    # The tester takes the mask instead of the scale, the updater multiplies the two; the plain backward action stores zeros
    # (a shadowed variable), so no gradient vector can come from the reference.
    for name, shape in (("ce", (3, 6, 4, 5)), ("ce_row", (5, 40, 1, 1))):
        cp = (1.0 / (1.0 + np.exp(-synth.normal(g, shape, 0.0, 2.0).astype(np.float64)))).astype(np.float32)
        ct = synth.targets(g, shape)
        cp.flat[0], ct.flat[0] = 0.0, 1.0     # log of a clamped prediction
        cp.flat[1], ct.flat[1] = 1.0, 0.0     # log of a clamped 1 - prediction
        cmask = (synth.uniform(g, (shape[0], 1) + shape[2:], 0.0, 1.0) > 0.3).astype(np.float32) * synth.uniform(g, (shape[0], 1) + shape[2:], 0.5, 2.0)
        out[name + "_p"], out[name + "_t"], out[name + "_mask"] = cp, ct, cmask
        out[name + "_err_tester"] = ref.cross_entropy_fwd(cp, ct, cmask, 0.7)[0]
        out[name + "_err_updater"] = ref.cross_entropy_fwd(cp, ct, cmask, 0.7, updater=True)[0]
        out[name + "_err_nomask"] = ref.cross_entropy_fwd(cp, ct, None, 1.3)[0]
        out[name + "_plain_backward"] = ref.cross_entropy_bwd(cp, ct, cmask, 0.7)[0]
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "plain_backend.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
