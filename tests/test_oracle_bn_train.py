"""Training-mode batch norm has no CPU implementation in the reference (it calls cuDNN), so the
oracle's restatement is unpinned by reference code. These CPU tests give it independent support:
PyTorch's CPU batch_norm (forward and autograd backward) and the fp32 / double twins against each other."""
import numpy as np
import pytest

import synth
from util import assert_close

torch = pytest.importorskip("torch")


def test_bn_train_matches_pytorch_cpu(oracle):
    """Independent second opinion for the unpinned training-mode restatement: PyTorch's CPU batch_norm."""
    g = synth.rng(2, salt=77)
    shape = (8, 5, 6, 6)
    x = synth.normal(g, shape, 0.5, 2.0)
    dy = synth.normal(g, shape)
    gamma, beta = synth.uniform(g, 5, 0.5, 1.5), synth.normal(g, 5, 0.0, 0.1)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    gt = torch.tensor(gamma, dtype=torch.float64, requires_grad=True)
    bt = torch.tensor(beta, dtype=torch.float64, requires_grad=True)
    yt = torch.nn.functional.batch_norm(xt, None, None, gt, bt, training=True, eps=1e-5)
    yt.backward(torch.tensor(dy, dtype=torch.float64))
    y, saved = oracle.bn_train_fwd(x, gamma, beta, 1e-5)
    db, dg = oracle.bn_train_bwd_sums(dy, x, saved)
    dx = oracle.bn_train_bwd_apply(dy, x, gamma, saved, db, dg, x.size // 5)
    assert_close(y, yt.detach().numpy(), "oracle fwd vs torch", atol=2e-6)
    assert_close(dx, xt.grad.numpy(), "oracle dx vs torch", atol=5e-6)
    assert_close(db, bt.grad.numpy(), "dbeta", atol=1e-5)
    assert_close(dg, gt.grad.numpy(), "dgamma", atol=1e-5)


def test_fp32_sums_agree_with_double_twin(oracle):
    g = synth.rng(2, salt=78)
    x = synth.normal(g, (32, 6, 14, 14), 0.5, 2.0)
    s64, q64 = oracle.bn_train_sums(x)
    s32, q32 = oracle.bn_train_sums(x, f32=True)
    m = x.size // 6
    a = oracle.bn_train_finalize(s64, q64, m, 1e-5)
    b = oracle.bn_train_finalize(s32, q32, m, 1e-5)
    assert_close(b, a, "fp32 statistics vs double")


def test_sharded_sums_equal_unsharded(oracle):
    """Synchronised batch norm: per-shard {sum, sumsq} added together give the full-batch statistics."""
    g = synth.rng(2, salt=79)
    x = synth.normal(g, (12, 4, 5, 5), 0.5, 2.0)
    s, q = oracle.bn_train_sums(x)
    parts = [oracle.bn_train_sums(x[a:b]) for a, b in ((0, 3), (3, 6), (6, 12))]
    np.testing.assert_allclose(sum(p[0] for p in parts), s, rtol=1e-12)
    np.testing.assert_allclose(sum(p[1] for p in parts), q, rtol=1e-12)
