"""nnf_bn_train_stats_static: the batch-statistics entry point for callers that cannot hand over a
workspace (a layer object inside nnForge's scheduler may only use pre-planned buffers and must not
allocate while enqueueing). It keeps its partial sums in an array built into the library, so the
checks here are: same numbers as nnf_bn_train_stats, also when the array still holds the previous
call's contents and when x is not 16-byte aligned, both sums against double-precision sums, device
memory that does not shrink over repeated calls, and a clear refusal beyond the 1024-channel limit.
Collected last on purpose, so a run that stops at the first failure has already covered everything else."""
import numpy as np
import pytest

import synth
from util import assert_close

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def test_static_scratch_matches_workspace_variant_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import nnforge_b200.capi as capi
    g = synth.rng(2, salt=4242)
    # the second call is smaller than the first, so it runs over slots the first one left filled
    for shape in [(24, 96, 14, 14), (5, 7, 3, 3)]:
        x = torch.from_numpy(synth.normal(g, shape, 0.5, 2.0)).cuda()
        n, c, hw = shape[0], shape[1], shape[2] * shape[3]
        ws = torch.empty(capi.bn_train_workspace_bytes(n, c, hw), dtype=torch.uint8, device="cuda")
        want = torch.empty(2 * c, device="cuda")
        capi.bn_train_stats(want, x, ws)
        got = torch.full((2 * c,), float("nan"), device="cuda")
        capi.bn_train_stats_static(got, x)
        torch.cuda.synchronize()
        assert_close(got.cpu().numpy(), want.cpu().numpy(), "static-scratch statistics %s" % (shape,))
        exact = x.double().sum(dim=(0, 2, 3)).cpu().numpy()
        assert_close(got.cpu().numpy()[:c], exact, "sum against a double-precision sum", atol=1e-3)
        exact_sq = x.double().pow(2).sum(dim=(0, 2, 3)).cpu().numpy()
        assert_close(got.cpu().numpy()[c:], exact_sq, "sum of squares against a double-precision sum", atol=1e-3)


@pytest.mark.parametrize("shape", [(6, 10, 8, 8), (3, 5, 7, 7)])
def test_static_scratch_with_x_off_the_16_byte_boundary(shape):
    """x starts one float into its allocation, so no float4 load is possible: the scalar path of the statistics kernel."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import nnforge_b200.capi as capi
    g = synth.rng(2, salt=4243 + shape[1])
    count = int(np.prod(shape))
    backing = torch.zeros(count + 4, device="cuda")
    x = backing[1:1 + count].view(shape)
    x.copy_(torch.from_numpy(synth.normal(g, shape, 0.5, 2.0)))
    assert x.data_ptr() % 16 == 4
    c = shape[1]
    got = torch.full((2 * c,), float("nan"), device="cuda")
    capi.bn_train_stats_static(got, x)
    torch.cuda.synchronize()
    xd = x.double()
    assert_close(got.cpu().numpy()[:c], xd.sum(dim=(0, 2, 3)).cpu().numpy(), "sum, unaligned x", atol=1e-3)
    assert_close(got.cpu().numpy()[c:], xd.pow(2).sum(dim=(0, 2, 3)).cpu().numpy(), "sum of squares, unaligned x", atol=1e-3)


def test_static_scratch_calls_allocate_nothing():
    """After the first call on the device (which looks up the array's address and loads the kernels) further calls leave the
    device's free memory and torch's allocator untouched."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import nnforge_b200.capi as capi
    x = torch.randn(32, 64, 14, 14, device="cuda")
    sums = torch.empty(128, device="cuda")
    capi.bn_train_stats_static(sums, x)
    torch.cuda.synchronize()
    for attempt in range(3):   # free memory is a device-wide figure: another process may move it, so a drop gets a second look
        free_before = torch.cuda.mem_get_info()[0]
        allocated, reserved = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
        for _ in range(4):
            capi.bn_train_stats_static(sums, x)
        torch.cuda.synchronize()
        assert (torch.cuda.memory_allocated(), torch.cuda.memory_reserved()) == (allocated, reserved)
        if torch.cuda.mem_get_info()[0] >= free_before:
            break
    else:
        raise AssertionError("free device memory shrank over calls of nnf_bn_train_stats_static in three attempts")


def test_static_scratch_refuses_more_channels_than_it_holds():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import nnforge_b200.capi as capi
    x = torch.zeros((1, 1025, 1, 1), device="cuda")
    sums = torch.zeros(2 * 1025, device="cuda")
    with pytest.raises(capi.NnfError) as e:
        capi.bn_train_stats_static(sums, x)
    assert "1024" in str(e.value)
