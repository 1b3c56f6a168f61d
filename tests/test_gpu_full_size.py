"""Parity at the benchmark configurations' full sizes (the other GPU tests use reduced batches).

Configuration 2 and stage 1 of configuration 3 are small enough for the CPU oracle to process whole;
configuration 4's 16 GiB tensor (2^32 elements, beyond the reference kernels' 32-bit indexing) is checked
on slices around the points where the library splits the tensor into several launches."""
import numpy as np
import pytest

import synth
from util import assert_bits_equal, assert_close, assert_close_off_kink

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def capi():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import nnforge_b200.capi as capi
    return capi


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_config4_16gib_tensor_needs_64_bit_indexing(capi, oracle):
    n, c, h, w = 8192, 128, 64, 64
    free, _ = torch.cuda.mem_get_info()
    if free < 20 * 2 ** 30:
        pytest.skip("needs 17 GiB of device memory")
    g = synth.rng(4)
    bn = synth.bn_params(g, c)
    x = torch.empty((n, c, h, w), device="cuda")
    assert x.numel() == 2 ** 32
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1004)
    for k in range(0, n, 1024):  # fill in pieces: one 16 GiB randn would need a second 16 GiB temporary
        x[k:k + 1024].normal_(0.0, 1.5, generator=gen)
    probe = [0, 1, 4094, 4095, 4096, 4097, 8190, 8191]  # both sides of the launch split and both ends
    before = {e: x[e].cpu().numpy() for e in probe}
    capi.bn_infer_act(x, x, bn=[dev(p) for p in bn], acts=[capi.tanh()])  # in place: the reference tester may overwrite input 0
    torch.cuda.synchronize()
    for e in probe:
        want = oracle.tanh_fwd(oracle.bn_infer(before[e][None], *bn))[0]
        assert_close(x[e].cpu().numpy(), want, "entry %d of the 16 GiB tensor" % e)
    # nothing was skipped or written twice: the output is bounded by tanh everywhere (one ulp above 1 can
    # come from the approximate reciprocal; a second application or an untouched N(0, 1.5) value cannot hide)
    assert float(x.abs().max()) <= 1.0 + 1e-6
    del x
    torch.cuda.empty_cache()


def test_config2_full_size_single_gpu_entry_points(capi, oracle):
    shape = (256, 256, 28, 28)
    g = synth.rng(2)
    x = synth.normal(g, shape, 0.5, 2.0)
    dy = synth.normal(g, shape)
    c = shape[1]
    gamma, beta = synth.uniform(g, c, 0.5, 1.5), synth.normal(g, c, 0.0, 0.1)
    slope = synth.uniform(g, c, 0.0, 0.3)
    eps = 1e-5
    xd, dyd, gd, bd, sd = dev(x), dev(dy), dev(gamma), dev(beta), dev(slope)
    acts = [capi.prelu(sd), capi.elu()]
    ws = torch.empty(capi.bn_train_workspace_bytes(shape[0], c, 784), dtype=torch.uint8, device="cuda")
    y, dx = torch.empty_like(xd), torch.empty_like(xd)
    saved, sums, bsums = torch.empty(2 * c, device="cuda"), torch.empty(2 * c, device="cuda"), torch.empty(3 * c, device="cuda")
    grads = [torch.zeros(c, device="cuda") for _ in range(3)]
    capi.bn_train_fwd(y, saved, sums, xd, gd, bd, eps, acts, workspace=ws)
    capi.bn_train_bwd(dx, bsums, dyd, xd, gd, bd, saved, acts, grad_gamma=grads[0], grad_beta=grads[1], grad_slope=grads[2], workspace=ws)
    torch.cuda.synchronize()
    assert capi.fused_error_check() == 0
    # CPU oracle, layer by layer (BN with batch statistics, PReLU, ELU and their backward actions)
    u, sv = oracle.bn_train_fwd(x, gamma, beta, eps)
    v = oracle.prelu_fwd(u, slope)
    yw = oracle.elu_fwd(v)
    dv = oracle.elu_bwd(dy, yw)
    dslope = oracle.prelu_bwd_weights(dv, u)
    du = oracle.prelu_bwd_data(dv, u, slope)
    db, dg = oracle.bn_train_bwd_sums(du, x, sv)
    dxw = oracle.bn_train_bwd_apply(du, x, gamma, sv, db, dg, x.size // c)
    assert_close(saved.cpu().numpy(), sv, "saved statistics")
    assert_close(y.cpu().numpy(), yw, "forward", atol=2e-6)
    assert_close_off_kink(dx.cpu().numpy(), dxw, u, "backward", atol=5e-6)   # PReLU's derivative jumps at u = 0
    m = x.size // c
    for got, want, name in ((grads[1], db, "d beta"), (grads[0], dg, "d gamma"), (grads[2], dslope, "d slope")):
        err = np.abs(got.cpu().numpy().astype(np.float64) - want)
        assert err.max() <= 1e-5 * np.sqrt(m) + 1e-5 * np.abs(want).max(), name


def test_config3_stage1_full_size(capi, oracle):
    n, c, hw = 256, 64, 56
    shape = (n, c, hw, hw)
    g = synth.rng(3)
    x, r = synth.normal(g, shape), synth.normal(g, shape)
    bn = synth.bn_params(g, c)
    p = capi.pool((3, 3), (2, 2))
    oh, ow = capi.pool_out_shape(hw, hw, p)
    z = torch.empty(shape, device="cuda")
    y = torch.empty((n, c, oh, ow), device="cuda")
    idx = torch.zeros((n, c, oh, ow), device="cuda", dtype=torch.int32)
    bnd = [dev(a) for a in bn]
    capi.bn_add_relu_maxpool_fwd(z, y, idx, dev(x), dev(r), bnd, 0.0, p)
    zw = oracle.relu_fwd(oracle.add_fwd([oracle.bn_infer(x, *bn), r], 1.0), 0.0)
    yw, iw = oracle.maxpool_fwd(zw, (3, 3), (2, 2))
    assert_bits_equal(z.cpu().numpy(), zw, "z")
    assert_bits_equal(y.cpu().numpy(), yw, "pooled")
    assert_bits_equal(idx.cpu().numpy().view(np.uint32), iw, "argmax")
    dyp = synth.normal(g, yw.shape)
    dx, dr = torch.empty(shape, device="cuda"), torch.empty(shape, device="cuda")
    capi.bn_add_relu_maxpool_bwd(dx, dr, dev(dyp), idx, z, bnd[0], bnd[3], 0.0, p)
    dz = oracle.maxpool_bwd(dyp, iw, shape)
    ds = oracle.relu_bwd(dz, oracle.add_fwd([oracle.bn_infer(x, *bn), r], 1.0), 0.0)
    assert_bits_equal(dr.cpu().numpy(), ds, "d residual")
    assert_bits_equal(dx.cpu().numpy(), (ds * (bn[0] * bn[3]).astype(np.float32)[None, :, None, None]).astype(np.float32), "dx")
    # size-independent property: every pooled gradient lands on exactly one input element
    np.testing.assert_allclose(dz.astype(np.float64).sum(), dyp.astype(np.float64).sum(), rtol=1e-6)
