"""The batch-sharded training batch-norm sequence (nnforge_b200/sharded.py) on two CPU ranks over gloo.
The compute backend is an adapter over the CPU checker, so what is tested here is the host logic: which
sums are all-reduced, which stay local, and that the sharded result equals the unsharded one."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class OracleKernels:
    """Same call signatures as nnforge_b200.capi, computed by the CPU checker on torch CPU tensors."""

    def __init__(self):
        from oracle import Oracle
        self.o = Oracle()

    @staticmethod
    def bn_train_workspace_bytes(n, c, hw):
        return 8

    def bn_train_stats(self, sums, x, workspace):
        s, q = self.o.bn_train_sums(x.numpy())
        sums.copy_(torch.from_numpy(np.concatenate([s, q]).astype(np.float32)))

    def _chain(self, acts):
        return [a[0] for a in acts], [a[1] for a in acts if a[0] == "prelu"]

    def bn_train_apply_act(self, y, saved, x, gamma, beta, sums, count_total, eps, acts):
        c = x.shape[1]
        s = sums.numpy().astype(np.float64)
        sv = self.o.bn_train_finalize(s[:c], s[c:], count_total, eps)
        saved.copy_(torch.from_numpy(sv))
        v = self.o.bn_train_apply(x.numpy(), gamma.numpy(), beta.numpy(), sv)
        for kind, param in acts:
            v = self.o.prelu_fwd(v, param) if kind == "prelu" else self.o.elu_fwd(v)
        y.copy_(torch.from_numpy(v))

    def _du(self, dy, x, gamma, beta, saved, acts):
        u = self.o.bn_train_apply(x.numpy(), gamma.numpy(), beta.numpy(), saved.numpy())
        ins, v = [], u
        for kind, param in acts:
            ins.append(v)
            v = self.o.prelu_fwd(v, param) if kind == "prelu" else self.o.elu_fwd(v)
        outs = ins[1:] + [v]
        g = dy.numpy()
        dslope = np.zeros(x.shape[1], np.float32)
        for (kind, param), a_in, a_out in reversed(list(zip(acts, ins, outs))):
            if kind == "prelu":
                dslope = self.o.prelu_bwd_weights(g, a_in)
                g = self.o.prelu_bwd_data(g, a_in, param)
            else:
                g = self.o.elu_bwd(g, a_out)
        return g, dslope

    def bn_train_bwd_stats(self, bsums, dy, x, gamma, beta, saved, acts, workspace, gsums=None):
        du, dslope = self._du(dy, x, gamma, beta, saved, acts)
        db, dg = self.o.bn_train_bwd_sums(du, x.numpy(), saved.numpy())
        bsums.copy_(torch.from_numpy(np.concatenate([db, dg, dslope]).astype(np.float32)))
        if gsums is not None:
            gsums.copy_(bsums[:2 * x.shape[1]])

    def bn_train_bwd_apply(self, dx, dy, x, gamma, beta, saved, gsums, bsums, count_total, acts, grad_gamma=None, grad_beta=None,
                           grad_mean=None, grad_invsigma=None, grad_slope=None, mean=None, invsigma=None, entry_count=0.0, add_to_destination=False):
        c = x.shape[1]
        du, _ = self._du(dy, x, gamma, beta, saved, acts)
        g = gsums.numpy().astype(np.float64)
        out = self.o.bn_train_bwd_apply(du, x.numpy(), gamma.numpy(), saved.numpy(), g[:c], g[c:2 * c], count_total)
        dx.copy_(torch.from_numpy(out))
        if grad_beta is not None:
            grad_beta += bsums[:c]
        if grad_gamma is not None:
            grad_gamma += bsums[c:2 * c]
        if grad_slope is not None:
            grad_slope += bsums[2 * c:]


    # the single-launch sharded entry points: what the launch does between its statistics and its apply work
    # (sum of this rank's two sums over all ranks, in rank order) is done here with a gathered sum
    def _rank_order_sum(self, local):
        parts = [torch.empty_like(local) for _ in range(dist.get_world_size())]
        dist.all_gather(parts, local)
        total = torch.zeros_like(local)
        for part in parts:
            total = total + part
        return total

    def bn_train_fwd_sharded(self, y, saved, sums, x, gamma, beta, eps, acts, count_total, workspace, mailbox_ptrs, rank, world, seq):
        assert world == dist.get_world_size() and rank == dist.get_rank() and seq >= 1
        self.bn_train_stats(sums, x, workspace)
        self.bn_train_apply_act(y, saved, x, gamma, beta, self._rank_order_sum(sums), count_total, eps, acts)

    def bn_train_bwd_sharded(self, dx, bsums, dy, x, gamma, beta, saved, acts, count_total, workspace, mailbox_ptrs, rank, world, seq, grad_gamma=None,
                             grad_beta=None, grad_mean=None, grad_invsigma=None, grad_slope=None, mean=None, invsigma=None, entry_count=0.0):
        assert world == dist.get_world_size() and rank == dist.get_rank() and seq >= 1
        self.bn_train_bwd_stats(bsums, dy, x, gamma, beta, saved, acts, workspace)
        gsums = self._rank_order_sum(bsums[:2 * x.shape[1]].clone())
        self.bn_train_bwd_apply(dx, dy, x, gamma, beta, saved, gsums, bsums, count_total, acts, grad_gamma=grad_gamma, grad_beta=grad_beta,
                                grad_slope=grad_slope)


class _DoneEvent:
    def record(self):
        pass

    def query(self):
        return True

    def synchronize(self):
        pass


class ReportingKernels(OracleKernels):
    """OracleKernels plus the launch report of the single-launch entry points; `fail_calls` lists the calls
    (counted from 1) whose report says that the wait for another rank ran out."""
    REPORT_WORDS = 3

    def __init__(self, fail_calls=()):
        super().__init__()
        self.fail_calls = set(fail_calls)
        self.calls = 0
        self.single_launch_calls = 0
        self.last_status = 0

    def make_event(self):
        return _DoneEvent()

    def bn_train_fwd_sharded(self, *args, **kwargs):
        self.calls += 1
        self.single_launch_calls += 1
        self.last_status = 2 if self.calls in self.fail_calls else 0
        super().bn_train_fwd_sharded(*args, **kwargs)

    def bn_train_bwd_sharded(self, *args, **kwargs):
        self.calls += 1
        self.single_launch_calls += 1
        self.last_status = 2 if self.calls in self.fail_calls else 0
        super().bn_train_bwd_sharded(*args, **kwargs)

    def read_report(self, words, workspace, stream=None):
        words[0], words[1], words[2] = 1000, 1000, self.last_status << 32

    @staticmethod
    def parse_report(words):
        return {"wait_ns_total": int(words[0]), "wait_ns_max": int(words[1]), "status": int(words[2]) >> 32}


class FakeInLaunchExchange:
    """Stands for nnforge_b200.sharded.InLaunchExchange on CPU ranks: same attributes, no mailboxes."""
    in_launch = True

    def __init__(self, channels):
        self.channels = channels
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.ptrs = []
        self.seq = 0

    def next_seq(self):
        self.seq += 1
        return self.seq

    def all_reduce(self, tensor):
        dist.all_reduce(tensor)


def _inputs():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import synth
    g = synth.rng(2, salt=555)
    shape = (8, 6, 5, 4)
    x = synth.normal(g, shape, 0.5, 2.0)
    dy = synth.normal(g, shape)
    gamma, beta = synth.uniform(g, 6, 0.5, 1.5), synth.normal(g, 6, 0.0, 0.1)
    slope = synth.uniform(g, 6, 0.0, 0.3)
    return x, dy, gamma, beta, slope


def _run_rank(rank, world, port, out_dir, in_launch):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nnforge_b200.sharded import ShardedBatchNormAct
    x, dy, gamma, beta, slope = _inputs()
    n = x.shape[0]
    lo, hi = n * rank // world, n * (rank + 1) // world
    t = torch.from_numpy
    acts = [("prelu", slope), ("elu", None)]
    layer = ShardedBatchNormAct(OracleKernels(), 6, 1e-5, acts, "cpu", exchange=FakeInLaunchExchange(6) if in_launch else None)
    xs, dys = t(x[lo:hi].copy()), t(dy[lo:hi].copy())
    y, dx = torch.empty_like(xs), torch.empty_like(xs)
    grads = {k: torch.zeros(6) for k in ("gamma", "beta", "slope")}
    layer.forward(y, xs, t(gamma), t(beta))
    layer.backward(dx, dys, xs, t(gamma), t(beta), grads=grads)
    # the framework's own weight-gradient all-reduce, which the layer deliberately leaves alone
    for v in grads.values():
        dist.all_reduce(v)
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), y=y.numpy(), dx=dx.numpy(), saved=layer.saved.numpy(),
             **{"g_" + k: v.numpy() for k, v in grads.items()})
    dist.destroy_process_group()


@pytest.mark.parametrize("world,in_launch", [(2, False), (4, False), (2, True)])
def test_sharded_equals_unsharded(tmp_path, world, in_launch):
    """in_launch: the host sequence of the single-launch sharded entry points (one call per direction)."""
    port = 29600 + world + 10 * int(in_launch) + (os.getpid() % 200)
    mp.spawn(_run_rank, args=(world, port, str(tmp_path), in_launch), nprocs=world, join=True)
    sys.path.insert(0, ROOT)
    from nnforge_b200.sharded import ShardedBatchNormAct
    x, dy, gamma, beta, slope = _inputs()
    t = torch.from_numpy
    acts = [("prelu", slope), ("elu", None)]
    layer = ShardedBatchNormAct(OracleKernels(), 6, 1e-5, acts, "cpu")  # one rank, no process group
    y, dx = torch.empty(x.shape), torch.empty(x.shape)
    grads = {k: torch.zeros(6) for k in ("gamma", "beta", "slope")}
    layer.forward(y, t(x), t(gamma), t(beta))
    layer.backward(dx, t(dy), t(x), t(gamma), t(beta), grads=grads)
    parts = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % r)) for r in range(world)]
    np.testing.assert_allclose(np.concatenate([p["y"] for p in parts]), y.numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(np.concatenate([p["dx"] for p in parts]), dx.numpy(), rtol=1e-5, atol=5e-6)
    for p in parts:
        np.testing.assert_allclose(p["saved"], layer.saved.numpy(), rtol=1e-6)
        for k in grads:
            np.testing.assert_allclose(p["g_" + k], grads[k].numpy(), rtol=1e-4, atol=1e-5)


def _run_rank_timeout(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nnforge_b200.sharded import ShardedBatchNormAct, ExchangeTimeout
    x, dy, gamma, beta, slope = _inputs()
    n = x.shape[0]
    lo, hi = n * rank // world, n * (rank + 1) // world
    t = torch.from_numpy
    acts = [("prelu", slope), ("elu", None)]
    kernels = ReportingKernels(fail_calls=(2,))       # the first backward launch reports a wait that ran out, on every rank
    layer = ShardedBatchNormAct(kernels, 6, 1e-5, acts, "cpu", exchange=FakeInLaunchExchange(6))
    xs, dys = t(x[lo:hi].copy()), t(dy[lo:hi].copy())
    y, dx = torch.empty_like(xs), torch.empty_like(xs)
    layer.forward(y, xs, t(gamma), t(beta))
    layer.backward(dx, dys, xs, t(gamma), t(beta))
    raised = False
    try:
        layer.check()                                  # the step boundary
    except ExchangeTimeout as e:
        raised = True
        assert [what for what, _ in e.reports] == ["backward"]
    assert raised and layer.degraded
    # the step is repeated: the layer now runs the statistics / all-reduce / apply sequence, and the result is right
    before = kernels.single_launch_calls
    layer.forward(y, xs, t(gamma), t(beta))
    layer.backward(dx, dys, xs, t(gamma), t(beta))
    layer.check()
    assert kernels.single_launch_calls == before
    np.savez(os.path.join(out_dir, "rank%d.npz" % rank), y=y.numpy(), dx=dx.numpy())
    # once the cause is gone the single launch can be switched back on
    layer.reset_exchange()
    layer.forward(y, xs, t(gamma), t(beta))
    layer.check()
    assert kernels.single_launch_calls == before + 1
    dist.destroy_process_group()


def test_timed_out_step_is_reported_and_redone(tmp_path):
    """A single-launch step whose report says that a wait ran out: the next check raises, the layer falls back to the
    statistics kernel / all-reduce / apply kernel sequence, and the repeated step gives the unsharded result."""
    world = 2
    port = 29900 + (os.getpid() % 200)
    mp.spawn(_run_rank_timeout, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    sys.path.insert(0, ROOT)
    from nnforge_b200.sharded import ShardedBatchNormAct
    x, dy, gamma, beta, slope = _inputs()
    t = torch.from_numpy
    acts = [("prelu", slope), ("elu", None)]
    layer = ShardedBatchNormAct(OracleKernels(), 6, 1e-5, acts, "cpu")
    y, dx = torch.empty(x.shape), torch.empty(x.shape)
    layer.forward(y, t(x), t(gamma), t(beta))
    layer.backward(dx, t(dy), t(x), t(gamma), t(beta))
    parts = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % r)) for r in range(world)]
    np.testing.assert_allclose(np.concatenate([p["y"] for p in parts]), y.numpy(), rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(np.concatenate([p["dx"] for p in parts]), dx.numpy(), rtol=1e-5, atol=5e-6)
