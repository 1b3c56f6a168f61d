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


def test_two_devices_in_one_process_through_the_layer_objects(oracle):
    """nnForge drives all its GPUs from one process. Two sets of layer objects, one per device, share a peer directory: each
    fused BatchNorm head owns a mailbox (its persistent working data), finds the other's through the directory, and the two
    single launches per direction exchange the batch statistics between them."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from nnforge_b200 import host
    import nnforge_b200.capi as capi
    from util import assert_close
    x, dy, gamma, beta, slope = _inputs(0)
    n, c, h, w = x.shape
    world = 2
    host.enable_peer_access(0, 1)
    host.enable_peer_access(1, 0)
    peers = host.PeerDirectory()
    spec = "bn BatchNorm x eps=1e-5\nprelu PReLU bn\nelu ELU prelu\n"
    per = n // world
    state = []
    for pos in range(world):
        with torch.cuda.device(pos):
            net = host.Net(spec, {"x": (c, w, h)}, training=True, device_pos=pos, device_count=world, peers=peers)
            head = net.objects[0]
            assert head.kind == "bn_train_act" and head.get_persistent_working_data_count() == 1
            d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
            state.append({"net": net, "head": head, "x": d(x[pos * per:(pos + 1) * per]), "dy": d(dy[pos * per:(pos + 1) * per]),
                          "data": [d(gamma), d(beta), torch.zeros(c, device="cuda"), torch.ones(c, device="cuda"), d(slope)],
                          "grad": [torch.zeros(c, device="cuda") for _ in range(5)],
                          "saved": torch.empty(2 * c, device="cuda"), "y": torch.empty(per, c, h, w, device="cuda"), "dx": torch.empty(per, c, h, w, device="cuda"),
                          "ws_f": torch.empty(head.get_temporary_working_fixed_buffer_size(host.FORWARD), dtype=torch.uint8, device="cuda"),
                          "ws_b": torch.empty(head.get_temporary_working_fixed_buffer_size(host.BACKWARD_DATA_AND_WEIGHTS), dtype=torch.uint8, device="cuda"),
                          "report": torch.zeros(2 * capi.REPORT_WORDS, dtype=torch.int64).pin_memory()})
    for _ in range(3):   # sequence numbers advance in step on both devices
        for pos, s in enumerate(state):
            with torch.cuda.device(pos):
                s["head"].enqueue_forward_propagation([s["y"]], s["data"], [s["x"]], per, temporary_working_fixed_buffer=s["ws_f"], temporary_fixed_buffer=s["saved"])
        for pos, s in enumerate(state):
            with torch.cuda.device(pos):
                s["head"].enqueue_backward_data_and_weights_propagation([s["dx"]], s["dy"], s["grad"], s["data"], [s["x"]], None, per,
                                                                        temporary_working_fixed_buffer=s["ws_b"], temporary_fixed_buffer=s["saved"])
    for pos, s in enumerate(state):
        with torch.cuda.device(pos):
            capi.read_report(s["report"][:capi.REPORT_WORDS], s["ws_f"])
            capi.read_report(s["report"][capi.REPORT_WORDS:], s["ws_b"])
            torch.cuda.synchronize()
            assert capi.parse_report(s["report"][:capi.REPORT_WORDS])["status"] == 0 and capi.parse_report(s["report"][capi.REPORT_WORDS:])["status"] == 0
    u, sv = oracle.bn_train_fwd(x, gamma, beta, 1e-5)
    yw = oracle.elu_fwd(oracle.prelu_fwd(u, slope))
    du = oracle.prelu_bwd_data(oracle.elu_bwd(dy, yw), u, slope)
    db, dg = oracle.bn_train_bwd_sums(du, x, sv)
    dxw = oracle.bn_train_bwd_apply(du, x, gamma, sv, db, dg, x.size // c)
    assert_close(np.concatenate([s["y"].cpu().numpy() for s in state]), yw, "forward over two devices", atol=2e-6)
    assert_close(np.concatenate([s["dx"].cpu().numpy() for s in state]), dxw, "backward over two devices", atol=5e-6)
    for s in state:   # whole-batch statistics on both devices, the same bits
        assert_close(s["saved"].cpu().numpy(), sv, "saved statistics")
    assert torch.equal(state[0]["saved"].cpu(), state[1]["saved"].cpu())
    # the per-channel gradients hold each device's own sums (their cross-device sum is the gradient all-reduce's job)
    total_gamma = sum(s["grad"][0].cpu().numpy().astype(np.float64) for s in state) / 3
    assert np.abs(total_gamma - dg).max() <= 2e-6 * np.sqrt(x.size // c) + 1e-5 * np.abs(dg).max()
