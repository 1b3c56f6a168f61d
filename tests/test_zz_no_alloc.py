"""nnf_bn_train_stats_static: the batch-statistics entry point for callers that cannot hand over a
workspace (a layer object inside nnForge's scheduler may only use pre-planned buffers and must not
allocate while enqueueing). It keeps its partial sums in an array built into the library, so the
checks here are: same numbers as nnf_bn_train_stats, also when the array still holds the previous
call's contents, and a clear refusal beyond the 1024-channel limit. Collected last on purpose, so a
run that stops at the first failure has already covered everything else."""
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


def test_static_scratch_refuses_more_channels_than_it_holds():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import nnforge_b200.capi as capi
    x = torch.zeros((1, 1025, 1, 1), device="cuda")
    sums = torch.zeros(2 * 1025, device="cuda")
    with pytest.raises(capi.NnfError) as e:
        capi.bn_train_stats_static(sums, x)
    assert "1024" in str(e.value)
