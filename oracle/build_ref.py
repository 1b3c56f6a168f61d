"""Build recipe for the reference-backed checker libraries (test infrastructure, never shipped).

Compiles nnForge's own plain-backend sources for the hot-path layers, unmodified and straight from
the reference checkout, together with ``oracle/ref_capi.cpp`` (flat C entry points) into

* ``oracle/_ref/libnnf_plain_ref.so``      serial build: the deterministic reference oracle
* ``oracle/_ref/libnnf_plain_ref_omp.so``  OpenMP build: the timed reference CPU baseline

The reference checkout is located through ``NNFORGE_REFERENCE_DIR``; when it is absent nothing is
built and already-built libraries are left alone. Reference sources are only ever read in place.

Flags: ``-O2`` without ``-ffast-math`` and with ``-ffp-contract=off`` so that signed zeros, NaNs and
the mul-then-add rounding of ``x*mult+add`` are deterministic (the reference's own Settings.mk uses
``-ffast-math -march=native`` which is not bit-stable across machines). ``-include algorithm
-include cmath`` supplies headers the sources use without including; ``-Dnone=shared`` in the OpenMP
build turns the sources' ``default(none)`` clauses, which current GCC rejects for const locals, into
``default(shared)``.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SHIM = os.path.join(HERE, "ref_shim")

LAYERS = [
    "batch_norm", "rectified_linear", "parametric_rectified_linear", "exponential_linear",
    "hyperbolic_tangent", "sigmoid", "softmax", "add", "max_subsampling",
]
PLAIN = (
    ["plain/batch_norm_layer_tester_plain.cpp"]
    + ["plain/%s_layer_tester_plain.cpp" % n for n in LAYERS[1:]]
    + ["plain/%s_layer_updater_plain.cpp" % n for n in LAYERS[1:]]
    + ["plain/negative_log_likelihood_layer_tester_plain.cpp", "plain/negative_log_likelihood_layer_updater_plain.cpp",
       "plain/cross_entropy_layer_tester_plain.cpp", "plain/cross_entropy_layer_updater_plain.cpp",
       "plain/accuracy_layer_tester_plain.cpp", "plain/accuracy_layer_updater_plain.cpp",
       "plain/average_subsampling_layer_tester_plain.cpp", "plain/average_subsampling_layer_updater_plain.cpp"]
    + ["plain/layer_tester_plain.cpp", "plain/layer_updater_plain.cpp", "plain/plain_buffer.cpp",
       "plain/plain_running_configuration.cpp"]
)
CORE = (
    ["%s_layer.cpp" % n for n in LAYERS + ["negative_log_likelihood", "cross_entropy", "accuracy", "average_subsampling"]]
    + ["layer.cpp", "layer_configuration_specific.cpp", "layer_data.cpp", "layer_data_custom.cpp",
       "layer_data_configuration.cpp", "rnd.cpp", "neural_network_exception.cpp", "tiling_factor.cpp",
       "stat_data_bunch_writer.cpp"]
)

COMMON = ["-std=c++11", "-O2", "-fPIC", "-ffp-contract=off", "-include", "algorithm", "-include", "cmath",
          "-Wno-unknown-pragmas", "-I", SHIM]


def reference_dir():
    # default: a checkout named "reference" beside this repository
    root = os.environ.get("NNFORGE_REFERENCE_DIR", os.path.join(os.path.dirname(os.path.dirname(os.path.realpath(HERE))), "reference"))
    src = os.path.join(root, "nnforge")
    return src if os.path.isdir(os.path.join(src, "plain")) else None


def _compile(args):
    src, obj, flags = args
    if os.path.exists(obj) and os.path.getmtime(obj) >= os.path.getmtime(src):
        return
    subprocess.check_call(["g++"] + flags + ["-c", src, "-o", obj])


def build(verbose=True):
    """Returns True when both libraries exist afterwards."""
    ref = reference_dir()
    libs = [os.path.join(OUT, "libnnf_plain_ref.so"), os.path.join(OUT, "libnnf_plain_ref_omp.so")]
    if ref is None:
        return all(os.path.exists(p) for p in libs)
    os.makedirs(OUT, exist_ok=True)
    for variant, extra, lib in (("ser", [], libs[0]), ("omp", ["-fopenmp", "-Dnone=shared", "-include", "omp.h"], libs[1])):
        objdir = os.path.join(OUT, "obj_" + variant)
        os.makedirs(objdir, exist_ok=True)
        flags = COMMON + extra + ["-I", ref]
        jobs = []
        for rel in PLAIN + CORE:
            jobs.append((os.path.join(ref, rel), os.path.join(objdir, rel.replace("/", "_") + ".o"), flags))
        jobs.append((os.path.join(HERE, "ref_capi.cpp"), os.path.join(objdir, "ref_capi.o"), flags))
        with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
            list(pool.map(_compile, jobs))
        objs = [j[1] for j in jobs]
        if not os.path.exists(lib) or any(os.path.getmtime(o) > os.path.getmtime(lib) for o in objs):
            subprocess.check_call(["g++", "-shared", "-o", lib] + objs + (["-fopenmp"] if variant == "omp" else []))
        if verbose:
            print("built", lib)
    return True


if __name__ == "__main__":
    sys.exit(0 if build() else 1)
