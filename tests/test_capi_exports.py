"""The shared library loads without a GPU and exports every entry point include/nnf_b200.h declares,
and the ctypes binding covers all of them. No compute is launched here."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "nnf_b200.h")).read()
    return sorted(set(re.findall(r"NNF_API[^;(]*?\b(nnf_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import nnforge_b200.build as build
    lib = ctypes.CDLL(build.build())
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), "libnnf_b200.so does not export " + name


def test_binding_covers_the_header():
    import nnforge_b200.capi as capi
    assert sorted(capi.EXPORTS) == declared_symbols()
    assert capi.lib.nnf_version() >= 100


def test_argument_errors_without_a_gpu():
    """Validation happens before any CUDA call, so it can be exercised on a CPU-only machine."""
    import nnforge_b200.capi as capi
    st = capi.lib.nnf_bn_infer_act(None, None, None, None, None, None, None, None, 1.0, None, 0, 4, 3, 5)
    assert st == -1 and "null" in capi.last_error()
    st = capi.lib.nnf_softmax_fwd(None, None, None, 4, 0, 5)
    assert st == -1 and "extents" in capi.last_error()
    assert capi.lib.nnf_pool_out_size(56, 3, 2, 0) == 27
    assert capi.lib.nnf_pool_out_size(56, 3, 2, 1) == 28
    assert capi.lib.nnf_bn_train_workspace_bytes(256, 256, 784) > 0


def test_profile_summaries_name_their_command():
    """Every ncu summary under profiles/ gives the command that made it, and every ncu command line leaves the clocks alone."""
    import glob
    import os
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "profiles")
    files = sorted(glob.glob(os.path.join(root, "*.md")))
    assert files, "no profile summaries"
    for path in files:
        text = open(path).read()
        assert "python bench.py" in text, "%s does not name the command that made it" % os.path.basename(path)
        # a command may be wrapped over several lines with backslashes
        joined = text.replace("\\\n", " ")
        for line in joined.splitlines():
            if line.strip().startswith("ncu "):
                assert "--clock-control none" in line, "%s: an ncu command without --clock-control none" % os.path.basename(path)
