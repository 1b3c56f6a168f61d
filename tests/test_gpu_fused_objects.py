"""Fused groups behind the per-layer interface: a textual schema goes through the planner (plan_fusion) and the
C++ factory (create_testers / create_updaters); the resulting head and follower objects are enqueued by a small
scheduler and compared with the same schema run layer by layer on the CPU checker."""
import numpy as np
import pytest

import synth
from schema_runner import ObjectRun, OracleRun
from util import assert_bits_equal, assert_close, assert_close_off_kink

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def host():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nnforge_b200 import host
    return host


def out(t):
    torch.cuda.synchronize()
    return t.cpu().numpy()


CFG0 = """bn BatchNorm x
relu ReLU bn slope=0
"""

CFG3_STAGE = """bn BatchNorm x
add Add bn,r alpha=1
relu ReLU add slope=0
pool MaxSubsampling relu win=3x3 stride=2x2
"""

CFG2 = """bn BatchNorm x eps=1e-5
prelu PReLU bn
elu ELU prelu
"""

CFG1 = """sm Softmax x
nll NegativeLogLikelihood sm,t scale=1.3
"""


@pytest.mark.parametrize("shape", [(6, 8, 9, 7), (64, 64, 32, 32)])
@pytest.mark.parametrize("in_place", [False, True])
def test_inference_batch_norm_relu_schema(host, oracle, shape, in_place):
    """BatchNorm -> ReLU with frozen statistics: one head object, one launch, the ReLU object does nothing."""
    n, c, h, w = shape
    g = synth.rng(0, salt=950)
    x = synth.with_edges(g, synth.normal(g, shape))
    weights = {"bn": list(synth.bn_params(g, c))}
    run = ObjectRun(host, CFG0, {"x": (c, w, h)}, False, n)
    head, follower = run.net.objects
    assert (head.role, head.kind, head.entry, head.inputs, head.data, head.outputs, head.elided) == ("head", "bn_act", "nnf_bn_infer_act", ["x"], ["bn"], ["relu"], ["bn"])
    assert follower.role == "follower" and follower.get_input_index_layer_can_write() == 0 and head.get_input_index_layer_can_write() == 0
    got = run.forward({"x": x}, weights, in_place=in_place)
    want = OracleRun(oracle, CFG0, False).forward({"x": x}, weights)
    assert_bits_equal(out(got["relu"]), want["relu"], "BatchNorm -> ReLU through the fused head")
    assert "bn" not in got   # the batch-norm output never existed
    if in_place:
        assert got["relu"].data_ptr() == got["x"].data_ptr()


@pytest.mark.parametrize("c,hw,n", [(64, 56, 8), (512, 7, 6), (5, 9, 3)])
def test_inference_residual_stage_schema(host, oracle, c, hw, n):
    """BatchNorm -> Add(residual) -> ReLU -> MaxSubsampling: the head writes the ReLU output and the pooled tensor in one pass."""
    shape = (n, c, hw, hw)
    g = synth.rng(3, salt=951 + c)
    x, r = synth.normal(g, shape), synth.normal(g, shape)
    weights = {"bn": list(synth.bn_params(g, c))}
    run = ObjectRun(host, CFG3_STAGE, {"x": (c, hw, hw), "r": (c, hw, hw)}, False, n)
    head = run.net.objects[0]
    assert (head.kind, head.entry, head.inputs, head.outputs, head.elided) == ("bn_add_relu_maxpool", "nnf_bn_add_relu_maxpool_fwd", ["x", "r"], ["relu", "pool"], ["bn", "add"])
    assert head.get_output_count() == 2 and [o.role for o in run.net.objects] == ["head", "follower", "follower", "follower"]
    assert run.net.objects[3].get_input_index_layer_can_write() == -1   # the pooling layer has a buffer of its own, which the head fills
    got = run.forward({"x": x, "r": r}, weights)
    want = OracleRun(oracle, CFG3_STAGE, False).forward({"x": x, "r": r}, weights)
    assert_bits_equal(out(got["relu"]), want["relu"], "ReLU output of the fused stage")
    assert_bits_equal(out(got["pool"]), want["pool"], "pooled output of the fused stage")
    # the single-output form of a two-output head is an error, not a silent half result
    with pytest.raises(host.HostLayerError):
        head.enqueue_forward_propagation([got["relu"]], [run.w["bn"][k] for k in range(4)], [run.buf["x"], run.buf["r"]], n)


def test_inference_average_pooled_stage_and_unfusable_neighbour(host, oracle):
    """The average-pooled tail fuses; a second reader of the batch-norm output keeps that layer on its own object."""
    n, c, h, w = 4, 6, 8, 12
    shape = (n, c, h, w)
    g = synth.rng(3, salt=952)
    x, r = synth.normal(g, shape), synth.normal(g, shape)
    spec = """bn BatchNorm x
add Add bn,r
relu ReLU add
pool AverageSubsampling relu win=4x2 alpha=0.125
side TanH bn scale=1.7159 steepness=0.6666
"""
    weights = {"bn": list(synth.bn_params(g, c))}
    run = ObjectRun(host, spec, {"x": (c, w, h), "r": (c, w, h)}, False, n)
    kinds = {o.node: (o.role, o.kind) for o in run.net.objects}
    assert kinds["bn"] == ("single", "single") and kinds["add"] == ("head", "bn_add_relu_avgpool") and kinds["side"] == ("single", "single")
    got = run.forward({"x": x, "r": r}, weights)
    want = OracleRun(oracle, spec, False).forward({"x": x, "r": r}, weights)
    for name in ("bn", "relu", "pool"):
        assert_bits_equal(out(got[name]), want[name], name)
    assert_close(out(got["side"]), want["side"], "side branch")


@pytest.mark.parametrize("shape", [(16, 32, 28, 28), (33, 48, 7, 7), (5, 3, 6, 5)])
def test_training_batch_norm_prelu_elu_schema(host, oracle, shape):
    """The benchmarked chain as a schema: the head runs nnf_bn_train_fwd / _bwd with both activations, the PReLU and ELU
    objects do nothing, and the slope gradient comes out of the head's backward action."""
    n, c, h, w = shape
    g = synth.rng(2, salt=953 + c)
    x, dy = synth.normal(g, shape, 0.5, 2.0), synth.normal(g, shape)
    weights = {"bn": [synth.uniform(g, c, 0.5, 1.5), synth.normal(g, c, 0.0, 0.1), synth.normal(g, c, 0.0, 0.1), synth.uniform(g, c, 0.5, 1.5)],
               "prelu": [synth.uniform(g, c, 0.0, 0.3)]}
    run = ObjectRun(host, CFG2, {"x": (c, w, h)}, True, n)
    head, prelu, elu = run.net.objects
    assert (head.kind, head.entry, head.inputs, head.data, head.outputs, head.elided) == ("bn_train_act", "nnf_bn_train_fwd", ["x"], ["bn", "prelu"], ["elu"], ["bn", "prelu"])
    for f in (prelu, elu):
        assert f.role == "follower" and f.get_input_index_layer_can_write(host.FORWARD) == 0 and f.get_input_index_layer_can_write(host.BACKWARD_DATA) == 0
        assert not f.is_backward_data_dependent_on_input_buffer() and not f.is_backward_data_dependent_on_output_buffer()
        assert f.get_temporary_fixed_buffer_size() == 0 and f.get_temporary_per_entry_buffer_size() == 0
    # the head's plan: x and the saved statistics are kept for backward, the output is not
    assert head.is_backward_data_and_weights_dependent_on_input_buffer(0) and not head.is_backward_data_and_weights_dependent_on_output_buffer()
    assert head.is_backward_data_and_weights_dependent_on_temporary_fixed_buffer() and not head.is_backward_data_and_weights_dependent_on_temporary_per_entry_buffer()
    assert head.get_temporary_fixed_buffer_size() == 2 * c * 4 and head.get_persistent_working_data_count() == 0
    assert head.get_linear_addressing_through_texture_per_entry() == []
    got = run.forward({"x": x}, weights)
    ref = OracleRun(oracle, CFG2, True)
    want = ref.forward({"x": x}, weights)
    assert set(got) == {"x", "elu"}
    assert_close(out(got["elu"]), want["elu"], "chain forward", atol=2e-6)
    assert_close(out(run.keep["bn"]["fixed"]), ref.saved["bn"], "saved mean / inverse std-dev")
    err, grads = run.backward({"elu": dy})
    err_w, grads_w = ref.backward({"elu": dy}, weights)
    assert_close_off_kink(out(err["x"]), err_w["x"], want["bn"], "chain backward", atol=5e-6)
    scale = np.sqrt(n * h * w)
    for k, what in enumerate(("d gamma", "d beta")):
        assert np.abs(out(grads["bn"][k]) - grads_w["bn"][k]).max() <= 2e-6 * scale + 1e-5 * np.abs(grads_w["bn"][k]).max(), what
    assert_close(out(grads["bn"][2]), grads_w["bn"][2], "running-mean pseudo-gradient", atol=1e-5)
    assert_close(out(grads["bn"][3]), grads_w["bn"][3], "running inverse-sigma pseudo-gradient", atol=1e-5)
    assert np.abs(out(grads["prelu"][0]) - grads_w["prelu"][0]).max() <= 1e-5 * scale + 1e-5 * np.abs(grads_w["prelu"][0]).max()
    # a follower that is not given its output-error buffer as its input-error buffer would silently drop the gradient: refused
    with pytest.raises(host.HostLayerError):
        elu.enqueue_backward_data_propagation(0, torch.empty_like(got["elu"]), err["elu"], [], [None], None, n)


@pytest.mark.parametrize("shape,masked", [((32, 21, 16, 16), False), ((256, 1000, 1, 1), False), ((7, 5, 3, 4), True)])
def test_training_softmax_loss_schema(host, oracle, shape, masked):
    n, c, h, w = shape
    g = synth.rng(1, salt=954 + c)
    logits, t = synth.normal(g, shape, 0.0, 3.0), synth.targets(g, shape)
    spec = CFG1.replace("sm,t", "sm,t,m") if masked else CFG1
    data = {"x": logits, "t": t}
    shapes = {"x": (c, w, h), "t": (c, w, h)}
    if masked:
        data["m"] = ((synth.uniform(g, (n, 1, h, w), 0.0, 1.0) > 0.3) * synth.uniform(g, (n, 1, h, w), 0.5, 2.0)).astype(np.float32)
        shapes["m"] = (1, w, h)
    run = ObjectRun(host, spec, shapes, True, n)
    head, loss = run.net.objects
    assert (head.kind, head.entry, head.inputs, head.outputs, head.get_output_count()) == ("softmax_nll", "nnf_softmax_nll_fwd", ["x", "t"] + (["m"] if masked else []), ["sm", "nll"], 2)
    assert not head.is_backward_data_dependent_on_input_buffer(0, 0) and head.is_backward_data_dependent_on_input_buffer(0, 1) and head.is_backward_data_dependent_on_output_buffer(0)
    got = run.forward(data, {})
    ref = OracleRun(oracle, spec, True)
    want = ref.forward(data, {})
    assert_close(out(got["sm"]), want["sm"], "probabilities")
    assert_close(out(got["nll"]), want["nll"], "loss", atol=2e-6)
    err, _ = run.backward({})
    # the checker's backward on the device's own probabilities, as the stand-alone layers would see them
    ref.values["sm"] = out(got["sm"])
    err_w, _ = ref.backward({}, {})
    assert_close(out(err["x"]), err_w["x"], "gradient of the logits", atol=2e-6)


def test_unfused_training_schema_runs_on_single_objects(host, oracle):
    """A chain the planner must leave alone (the batch-norm output has a second reader): every layer keeps its own object and
    the scheduler's result is the layer-by-layer one."""
    n, c, h, w = 6, 8, 6, 4
    shape = (n, c, h, w)
    g = synth.rng(2, salt=955)
    spec = """bn BatchNorm x eps=1e-5
prelu PReLU bn
side Sigmoid bn
sum Add prelu,side
"""
    x, dy = synth.normal(g, shape, 0.5, 2.0), synth.normal(g, shape)
    weights = {"bn": [synth.uniform(g, c, 0.5, 1.5), synth.normal(g, c, 0.0, 0.1), synth.normal(g, c, 0.0, 0.1), synth.uniform(g, c, 0.5, 1.5)],
               "prelu": [synth.uniform(g, c, 0.0, 0.3)]}
    run = ObjectRun(host, spec, {"x": (c, w, h)}, True, n)
    assert [o.role for o in run.net.objects] == ["single"] * 4
    got = run.forward({"x": x}, weights)
    ref = OracleRun(oracle, spec, True)
    want = ref.forward({"x": x}, weights)
    assert_close(out(got["sum"]), want["sum"], "forward", atol=2e-6)
    err, grads = run.backward({"sum": dy})
    err_w, grads_w = ref.backward({"sum": dy}, weights)
    assert_close_off_kink(out(err["x"]), err_w["x"], want["bn"], "backward", atol=5e-6)
    assert_close(out(grads["prelu"][0]), grads_w["prelu"][0], "slope gradient", atol=1e-4)


def test_weights_travel_through_get_data(host):
    """get_data uploads one device buffer per chunk, get_data_from_device brings them back (layer_updater_cuda.cpp:67-107)."""
    c, w, h = 8, 5, 4
    run_t = host.Net(CFG0, {"x": (c, w, h)}, training=False)
    run_u = host.Net(CFG2, {"x": (c, w, h)}, training=True)
    parts = [np.arange(c, dtype=np.float32) + k for k in range(4)]
    dev_t = run_t.objects[0].get_data(parts)
    dev_u = run_u.objects[0].get_data(parts + [np.full(c, 0.25, np.float32)])
    assert [tuple(t.shape) for t in dev_t] == [(c,)] * 4 and len(dev_u) == 5
    for t, p in zip(dev_u, parts):
        assert np.array_equal(out(t), p)
    dev_u[1].add_(1.0)
    back = run_u.objects[0].get_data_from_device()
    assert np.array_equal(back[1], parts[1] + 1.0) and np.array_equal(back[4], np.full(c, 0.25, np.float32))
    # the uploaded buffers are what a scheduler hands back as `data`
    x = torch.randn(3, c, h, w, device="cuda")
    y = torch.empty_like(x)
    run_t.objects[0].enqueue_forward_propagation([y], dev_t, [x], 3)
    torch.cuda.synchronize()
    assert torch.isfinite(y).all()


def test_running_configuration_comes_from_the_device(host):
    import nnforge_b200.capi as capi
    rc, lib_rc = host.running_configuration(), capi.running_configuration()
    props = torch.cuda.get_device_properties(0)
    assert rc["multiprocessor_count"] == props.multi_processor_count == lib_rc["multiprocessor_count"]
    assert (rc["compute_capability_major"], rc["compute_capability_minor"]) == (props.major, props.minor)
    assert rc["l2_cache_size"] == props.L2_cache_size and rc["device_pos"] == 0 and rc["device_count"] == 1
    assert rc["smem_per_block"] == lib_rc["max_shared_memory_per_block_optin"]
