"""Two real GPUs: the batch-sharded training batch-norm sequence with every exchange (NCCL all-reduce, the
peer-memory sum as kernels of its own, folded into the batch-norm kernels, and inside the single launch)
against the unsharded CPU oracle. Skipped on machines with one GPU."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _inputs(use_peer=0):
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import synth
    g = synth.rng(2, salt=777)
    # case 4: 7x7 planes are not whole float4s - the in-launch exchange runs on channel groups
    shape = (16, 24, 7, 7) if int(use_peer) == 4 else (16, 24, 14, 14)
    return (synth.normal(g, shape, 0.5, 2.0), synth.normal(g, shape), synth.uniform(g, 24, 0.5, 1.5), synth.normal(g, 24, 0.0, 0.1),
            synth.uniform(g, 24, 0.0, 0.3))


def _rank(rank, world, port, out_dir, use_peer):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import nnforge_b200.capi as capi
    from nnforge_b200.sharded import NcclExchange, PeerExchange, ShardedBatchNormAct
    x, dy, gamma, beta, slope = _inputs(use_peer)
    n, c = x.shape[0], x.shape[1]
    lo, hi = n * rank // world, n * (rank + 1) // world
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    sd = d(slope)
    acts = [capi.prelu(sd), capi.elu()]
    from nnforge_b200.sharded import FusedPeerExchange, InLaunchExchange
    exchange = [NcclExchange, lambda: PeerExchange(capi, 2 * c, torch.device("cuda", rank)),
                lambda: FusedPeerExchange(capi, 2 * c, torch.device("cuda", rank)),
                lambda: InLaunchExchange(capi, c, torch.device("cuda", rank))][min(int(use_peer), 3)]()
    layer = ShardedBatchNormAct(capi, c, 1e-5, acts, "cuda", exchange=exchange)
    xs, dys, gd, bd = d(x[lo:hi]), d(dy[lo:hi]), d(gamma), d(beta)
    y, dx = torch.empty_like(xs), torch.empty_like(xs)
    for _ in range(3):  # several steps: sequence numbers and slot parities advance
        layer.forward(y, xs, gd, bd)
        layer.backward(dx, dys, xs, gd, bd)
    torch.cuda.synchronize()
    err = capi.fused_error_check()
    np.savez(os.path.join(out_dir, "r%d_%d.npz" % (rank, int(use_peer))), y=y.cpu().numpy(), dx=dx.cpu().numpy(), err=err)
    dist.barrier()
    dist.destroy_process_group()


# NCCL all-reduce, peer-memory sum, the same inside the two kernels, inside the single launch, and (4) the last on 7x7 planes
@pytest.mark.parametrize("use_peer", [0, 1, 2, 3, 4])
def test_two_gpu_sharded_matches_unsharded_oracle(tmp_path, oracle, use_peer):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    port = 29700 + int(use_peer) + (os.getpid() % 200)
    mp.spawn(_rank, args=(world, port, str(tmp_path), use_peer), nprocs=world, join=True)
    x, dy, gamma, beta, slope = _inputs(use_peer)
    u, sv = oracle.bn_train_fwd(x, gamma, beta, 1e-5)
    v = oracle.prelu_fwd(u, slope)
    yw = oracle.elu_fwd(v)
    du = oracle.prelu_bwd_data(oracle.elu_bwd(dy, yw), u, slope)
    db, dg = oracle.bn_train_bwd_sums(du, x, sv)
    dxw = oracle.bn_train_bwd_apply(du, x, gamma, sv, db, dg, x.size // x.shape[1])
    parts = [np.load(os.path.join(str(tmp_path), "r%d_%d.npz" % (r, int(use_peer)))) for r in range(world)]
    assert all(int(p["err"]) == 0 for p in parts)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from util import assert_close
    assert_close(np.concatenate([p["y"] for p in parts]), yw, "sharded forward", atol=2e-6)
    assert_close(np.concatenate([p["dx"] for p in parts]), dxw, "sharded backward", atol=5e-6)
