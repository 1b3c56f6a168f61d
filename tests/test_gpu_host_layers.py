"""The C++ host-side layer objects (nnForge-shaped testers / updaters created by type name) against
the CPU oracle: each test reads like a step of the reference's schedulers - create the object, ask it
for its buffer sizes, hand it the buffers, enqueue."""
import numpy as np
import pytest

import synth
from util import assert_bits_equal, assert_close

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def host():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nnforge_b200 import host
    return host


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def out(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


SHAPE = (6, 8, 9, 7)  # n, c, h, w


def test_batch_norm_tester_then_relu_tester_in_place(host, oracle):
    g = synth.rng(0, salt=900)
    x = synth.with_edges(g, synth.normal(g, SHAPE))
    n, c, h, w = SHAPE
    bn = synth.bn_params(g, c)
    t_bn = host.Tester("BatchNorm", c, w, h)
    t_relu = host.Tester("ReLU", c, w, h, params=[0.0])
    assert t_bn.get_input_index_layer_can_write() == 0 and t_relu.get_input_index_layer_can_write() == 0
    buf = dev(x)
    t_bn.enqueue_forward_propagation(buf, [dev(p) for p in bn], [buf], n)   # output aliases input 0
    t_relu.enqueue_forward_propagation(buf, [], [buf], n)
    assert_bits_equal(out(buf), oracle.relu_fwd(oracle.bn_infer(x, *bn), 0.0), "BatchNorm -> ReLU testers")


@pytest.mark.parametrize("name,params", [("ReLU", [0.1]), ("PReLU", []), ("ELU", []), ("TanH", [1.7159, 0.6666]), ("Sigmoid", [])])
def test_activation_updaters(host, oracle, name, params):
    g = synth.rng(5, salt=901 + len(name))
    n, c, h, w = SHAPE
    x = synth.normal(g, SHAPE)
    dy = synth.normal(g, SHAPE)
    slope = synth.uniform(g, c, 0.0, 0.3)
    data = [dev(slope)] if name == "PReLU" else []
    u = host.Updater(name, c, w, h, params=params)
    y = torch.empty(SHAPE, device="cuda")
    u.enqueue_forward_propagation(y, data, [dev(x)], n)
    want = {"ReLU": lambda: oracle.relu_fwd(x, 0.1), "PReLU": lambda: oracle.prelu_fwd(x, slope), "ELU": lambda: oracle.elu_fwd(x),
            "TanH": lambda: oracle.tanh_fwd(x, 1.7159, 0.6666), "Sigmoid": lambda: oracle.sigmoid_fwd(x)}[name]()
    assert_close(out(y), want, name + " forward")
    dx = torch.empty(SHAPE, device="cuda")
    # the scheduler hands over only what the updater declared a dependency on
    in_neurons = dev(x) if u.is_backward_data_dependent_on_input_buffer() else None
    out_neurons = dev(want) if u.is_backward_data_dependent_on_output_buffer() else None
    u.enqueue_backward_data_propagation(dx, dev(dy), data, in_neurons, out_neurons, n)
    want_dx = {"ReLU": lambda: oracle.relu_bwd(dy, x, 0.1), "PReLU": lambda: oracle.prelu_bwd_data(dy, x, slope), "ELU": lambda: oracle.elu_bwd(dy, want),
               "TanH": lambda: oracle.tanh_bwd(dy, want, 1.7159, 0.6666), "Sigmoid": lambda: oracle.sigmoid_bwd(dy, want)}[name]()
    assert_bits_equal(out(dx), want_dx, name + " backward")
    if name == "PReLU":
        grad = torch.zeros(c, device="cuda")
        ws = torch.empty(u.get_temporary_working_fixed_buffer_size(host.BACKWARD_WEIGHTS), dtype=torch.uint8, device="cuda")
        u.enqueue_backward_weights_propagation([grad], dev(x), dev(dy), n, temporary_working_fixed_buffer=ws)
        exact = (dy.astype(np.float64) * np.where(x >= 0, 0.0, x)).sum(axis=(0, 2, 3))
        assert np.abs(out(grad) - exact).max() <= 1e-5 * np.sqrt(n * h * w)
    else:
        with pytest.raises(host.HostLayerError):
            u.enqueue_backward_weights_propagation([dx], dev(x), dev(dy), n)


def test_add_softmax_maxpool_updaters(host, oracle):
    g = synth.rng(3, salt=902)
    n, c, h, w = SHAPE
    a, b = synth.normal(g, SHAPE), synth.normal(g, SHAPE)
    y = torch.empty(SHAPE, device="cuda")
    host.Updater("Add", c, w, h, params=[0.5], input_count=2).enqueue_forward_propagation(y, [], [dev(a), dev(b)], n)
    assert_bits_equal(out(y), oracle.add_fwd([a, b], 0.5), "Add")
    sm = host.Updater("Softmax", c, w, h)
    sm.enqueue_forward_propagation(y, [], [dev(a)], n)
    want = oracle.softmax_fwd(a)
    assert_close(out(y), want, "Softmax forward")
    dx = torch.empty(SHAPE, device="cuda")
    sm.enqueue_backward_data_propagation(dx, dev(b), [], None, dev(want), n)
    assert_close(out(dx), oracle.softmax_bwd(b, want), "Softmax backward", atol=2e-6)
    z = oracle.relu_fwd(a, 0.0)
    pool = host.Updater("MaxSubsampling", c, w, h, pool=[3, 3, 2, 2, 0, 0, 0])
    wy, widx = oracle.maxpool_fwd(z, (3, 3), (2, 2))
    py = torch.empty(wy.shape, device="cuda")
    assert pool.get_temporary_per_entry_buffer_size() == widx[0].size * 4
    idx = torch.empty(widx.shape, device="cuda", dtype=torch.int32)
    pool.enqueue_forward_propagation(py, [], [dev(z)], n, temporary_per_entry_buffer=idx)
    assert_bits_equal(out(py), wy, "MaxSubsampling values")
    assert_bits_equal(out(idx).view(np.uint32), widx, "MaxSubsampling argmax")
    dyp = synth.normal(g, wy.shape)
    pool.enqueue_backward_data_propagation(dx, dev(dyp), [], None, None, n, temporary_per_entry_buffer=idx)
    assert_bits_equal(out(dx), oracle.maxpool_bwd(dyp, widx, SHAPE), "MaxSubsampling backward")
    with pytest.raises(host.HostLayerError):
        pool.enqueue_backward_data_propagation(dx, dev(dyp), [], None, None, n, temporary_per_entry_buffer=None)


def test_batch_norm_updater_fused_backward_data_and_weights(host, oracle):
    g = synth.rng(2, salt=903)
    n, c, h, w = 12, 8, 6, 4
    shape = (n, c, h, w)
    x, dy = synth.normal(g, shape, 0.5, 2.0), synth.normal(g, shape)
    gamma, beta = synth.uniform(g, c, 0.5, 1.5), synth.normal(g, c, 0.0, 0.1)
    run_mean, run_inv = synth.normal(g, c, 0.0, 0.1), synth.uniform(g, c, 0.5, 1.5)
    eps = 1e-5
    u = host.Updater("BatchNorm", c, w, h, params=[eps])
    data = [dev(gamma), dev(beta), dev(run_mean), dev(run_inv)]
    saved = torch.empty(u.get_temporary_fixed_buffer_size() // 4, device="cuda")
    ws = torch.empty(u.get_temporary_working_fixed_buffer_size(host.FORWARD), dtype=torch.uint8, device="cuda")
    y = torch.empty(shape, device="cuda")
    u.enqueue_forward_propagation(y, data, [dev(x)], n, temporary_working_fixed_buffer=ws, temporary_fixed_buffer=saved)
    y_w, saved_w = oracle.bn_train_fwd(x, gamma, beta, eps)
    assert_close(out(y), y_w, "BatchNorm updater forward", atol=2e-6)
    assert_close(out(saved), saved_w, "saved mean / inverse std-dev")
    grads = [torch.zeros(c, device="cuda") for _ in range(4)]
    ws2 = torch.empty(u.get_temporary_working_fixed_buffer_size(host.BACKWARD_DATA_AND_WEIGHTS), dtype=torch.uint8, device="cuda")
    dx = torch.empty(shape, device="cuda")
    u.enqueue_backward_data_and_weights_propagation(dx, dev(dy), grads, data, dev(x), n, temporary_working_fixed_buffer=ws2, temporary_fixed_buffer=saved)
    db, dg = oracle.bn_train_bwd_sums(dy, x, saved_w)
    assert_close(out(dx), oracle.bn_train_bwd_apply(dy, x, gamma, saved_w, db, dg, n * h * w), "BatchNorm updater dx", atol=5e-6)
    assert_close(out(grads[0]), dg, "d gamma", atol=1e-4)
    assert_close(out(grads[1]), db, "d beta", atol=1e-4)
    gm, gi = oracle.bn_train_running_grad(np.zeros(c, np.float32), np.zeros(c, np.float32), saved_w, run_mean, run_inv, n)
    assert_close(out(grads[2]), gm, "running-mean pseudo-gradient", atol=1e-5)
    assert_close(out(grads[3]), gi, "running inverse-sigma pseudo-gradient", atol=1e-5)
    with pytest.raises(host.HostLayerError):  # too small a working buffer is refused, not overrun
        u.enqueue_forward_propagation(y, data, [dev(x)], n, temporary_working_fixed_buffer=torch.empty(16, dtype=torch.uint8, device="cuda"), temporary_fixed_buffer=saved)


def test_negative_log_likelihood_objects(host, oracle):
    g = synth.rng(3, salt=903)
    n, c, h, w = SHAPE
    p = oracle.softmax_fwd(synth.normal(g, SHAPE, 0.0, 2.0))
    t = synth.targets(g, SHAPE)
    mask = synth.uniform(g, (n, 1, h, w), 0.0, 2.0)
    err = torch.empty((n, 1, h, w), device="cuda")
    host.Tester("NegativeLogLikelihood", c, w, h, params=[0.5], input_count=2).enqueue_forward_propagation(err, [], [dev(p), dev(t)], n)
    assert_close(out(err), oracle.nll_fwd(p, t, None, 0.5), "loss tester", atol=2e-6)
    u = host.Updater("NegativeLogLikelihood", c, w, h, params=[0.5], input_count=3)
    u.enqueue_forward_propagation(err, [], [dev(p), dev(t), dev(mask)], n)
    assert_close(out(err), oracle.nll_fwd(p, t, mask, 0.5), "loss updater forward", atol=2e-6)
    dp = torch.empty(SHAPE, device="cuda")
    u.enqueue_backward_data_propagation_inputs(dp, None, [dev(p), dev(t), dev(mask)], None, n)
    assert_bits_equal(out(dp), oracle.nll_bwd(p, t, mask, 0.5), "loss updater backward")
    acc = torch.empty((n, 4, h, w), device="cuda")
    host.Tester("Accuracy", c, w, h, params=[3], input_count=3).enqueue_forward_propagation(acc, [], [dev(p), dev(t), dev(mask)], n)
    assert_bits_equal(out(acc), oracle.accuracy_fwd(p, t, mask, 3), "accuracy tester")


def test_cross_entropy_objects(host, oracle):
    g = synth.rng(3, salt=906)
    n, c, h, w = SHAPE
    p = (1.0 / (1.0 + np.exp(-synth.normal(g, SHAPE, 0.0, 2.0).astype(np.float64)))).astype(np.float32)
    t = synth.targets(g, SHAPE)
    mask = (synth.uniform(g, (n, 1, h, w), 0.0, 1.0) > 0.3).astype(np.float32) * synth.uniform(g, (n, 1, h, w), 0.5, 2.0)
    err = torch.empty((n, 1, h, w), device="cuda")
    # the tester reproduces the reference tester: with a mask, the mask alone is the total scale
    host.Tester("CrossEntropy", c, w, h, params=[0.5], input_count=3).enqueue_forward_propagation(err, [], [dev(p), dev(t), dev(mask)], n)
    assert_close(out(err), oracle.cross_entropy_fwd(p, t, mask, 0.5, mask_replaces_scale=True), "cross entropy tester, masked", atol=2e-5)
    host.Tester("CrossEntropy", c, w, h, params=[0.5], input_count=2).enqueue_forward_propagation(err, [], [dev(p), dev(t)], n)
    assert_close(out(err), oracle.cross_entropy_fwd(p, t, None, 0.5), "cross entropy tester", atol=2e-5)
    u = host.Updater("CrossEntropy", c, w, h, params=[0.5], input_count=3)
    u.enqueue_forward_propagation(err, [], [dev(p), dev(t), dev(mask)], n)
    assert_close(out(err), oracle.cross_entropy_fwd(p, t, mask, 0.5), "cross entropy updater forward", atol=2e-5)
    dp = torch.empty(SHAPE, device="cuda")
    u.enqueue_backward_data_propagation_inputs(dp, None, [dev(p), dev(t), dev(mask)], None, n)
    assert_bits_equal(out(dp), oracle.cross_entropy_bwd(p, t, mask, 0.5), "cross entropy updater backward")
    assert u.is_backward_data_dependent_on_input_buffer() and not u.is_backward_data_dependent_on_output_buffer()


def test_average_subsampling_objects(host, oracle):
    g = synth.rng(3, salt=904)
    shape = (4, 6, 8, 12)
    n, c, h, w = shape
    x = synth.normal(g, shape)
    win, mult = (4, 2), 0.125
    u = host.Updater("AverageSubsampling", c, w, h, params=[mult], pool=[win[0], win[1], 0, 0, 0, 0, 0])
    want = oracle.avgpool_fwd(x, win, mult=mult)
    y = torch.empty(want.shape, device="cuda")
    u.enqueue_forward_propagation(y, [], [dev(x)], n)
    assert_bits_equal(out(y), want, "average subsampling updater forward")
    dy = synth.normal(g, want.shape)
    dx = torch.empty(shape, device="cuda")
    u.enqueue_backward_data_propagation(dx, dev(dy), [], None, None, n)
    assert_bits_equal(out(dx), oracle.avgpool_bwd(dy, shape, win, mult=mult), "average subsampling updater backward")
    assert not u.is_backward_data_dependent_on_input_buffer() and not u.is_backward_data_dependent_on_output_buffer()


@pytest.mark.parametrize("kind", ["none", "vanilla", "nesterov", "adam"])
def test_apply_gradient_for_a_batch_norm_layer(host, oracle, kind):
    """The scheduler's optimiser step for a batch-norm layer's four chunks (gamma, beta, mean, inverse sigma): one call, one
    launch. No chunk of a batch-norm layer is in the weight-decay set, so the decay given must not be applied."""
    g = synth.rng(4, salt=905 + len(kind))
    c = 96
    mtype = {"none": host.NO_MOMENTUM, "vanilla": host.VANILLA_MOMENTUM, "nesterov": host.NESTEROV_MOMENTUM, "adam": host.ADAM_MOMENTUM}[kind]
    data = [synth.normal(g, (c,)) for _ in range(4)]
    grad = [synth.normal(g, (c,), 0.0, 3.0) for _ in range(4)]
    prev = [synth.normal(g, (c,), 0.0, 0.01) for _ in range(4)]
    prev2 = [np.abs(synth.normal(g, (c,), 0.0, 0.1)) for _ in range(4)]
    lrs = [0.01, 0.01, 0.1, 0.1]
    d_data, d_grad, d_prev, d_prev2 = ([dev(a) for a in arrs] for arrs in (data, grad, prev, prev2))
    accum = [torch.zeros(1, dtype=torch.float64, device="cuda") for _ in range(4)]
    host.enqueue_apply_gradient(d_data, d_grad, lrs, d_prev if kind != "none" else None, d_prev2 if kind == "adam" else None, accum,
                                weight_decay_part_ids=[], gradient_normalizer=1.0 / 64, weight_decay=0.01, momentum_type=mtype, momentum_val=0.9,
                                momentum_val2=0.999, iteration_id=3)
    for k in range(4):
        want_acc = oracle.apply_gradient(data[k], grad[k], prev[k], prev2[k], kind, lrs[k], 1.0 / 64, 0.0, 0.9, 0.999, 3)
        assert_bits_equal(out(d_data[k]), data[k], "chunk %d weights" % k)
        assert not out(d_grad[k]).any()
        assert abs(float(out(accum[k])[0]) - want_acc) <= 1e-12 * want_acc
    with pytest.raises(host.HostLayerError):   # momentum without the previous updates
        host.enqueue_apply_gradient(d_data, d_grad, lrs, momentum_type=host.VANILLA_MOMENTUM, momentum_val=0.9)
