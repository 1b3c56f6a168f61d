"""ctypes binding of include/nnf_b200.h (the C ABI of libnnf_b200.so).

Tensors are passed as torch CUDA tensors (or ``None``); the binding hands their ``data_ptr()`` to the
library and enqueues on torch's current stream unless ``stream=`` is given. A non-zero status raises
``NnfError`` carrying ``nnf_last_error_string()``. There is no fallback path: if the shared library
has not been built (``python -m nnforge_b200.build``) the import raises.
"""
import ctypes as ct
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libnnf_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError("libnnf_b200.so is missing: build it with `python -m nnforge_b200.build` (needs nvcc); "
                      "this package has no CPU or PyTorch fallback")

lib = ct.CDLL(LIB_PATH)

ACT_NONE, ACT_RELU, ACT_PRELU, ACT_ELU, ACT_TANH, ACT_SIGMOID = range(6)
MAX_ACTS = 2
MAX_ADD_INPUTS = 8


class NnfError(RuntimeError):
    def __init__(self, status, text):
        super().__init__("nnf_b200 status %d: %s" % (status, text))
        self.status = status


class Act(ct.Structure):
    _fields_ = [("kind", ct.c_int32), ("p0", ct.c_float), ("p1", ct.c_float), ("slope", ct.c_void_p)]


class Pool(ct.Structure):
    _fields_ = [("win_w", ct.c_int32), ("win_h", ct.c_int32), ("stride_w", ct.c_int32), ("stride_h", ct.c_int32),
                ("round_up_w", ct.c_int32), ("round_up_h", ct.c_int32), ("is_min", ct.c_int32)]


_P, _I64, _F, _I, _D, _SZ = ct.c_void_p, ct.c_int64, ct.c_float, ct.c_int, ct.c_double, ct.c_size_t
class OptPart(ct.Structure):
    _fields_ = [("data", ct.c_void_p), ("gradient", ct.c_void_p), ("prev_upd", ct.c_void_p), ("prev_upd2", ct.c_void_p),
                ("update_accum", ct.c_void_p), ("learning_rate", ct.c_float), ("weight_decay", ct.c_float), ("elem_count", ct.c_int64)]


MOMENTUM_NONE, MOMENTUM_VANILLA, MOMENTUM_NESTEROV, MOMENTUM_ADAM = range(4)

_ACTP, _POOLP = ct.POINTER(Act), ct.POINTER(Pool)

class RunningConfiguration(ct.Structure):
    _fields_ = [(name, ct.c_int32) for name in (
        "device_id", "compute_capability_major", "compute_capability_minor", "multiprocessor_count", "max_threads_per_multiprocessor",
        "max_shared_memory_per_block_optin", "max_shared_memory_per_multiprocessor", "l2_cache_size", "max_registers_per_multiprocessor")]


class LaunchReport(ct.Structure):
    _fields_ = [("wait_ns_total", ct.c_uint64), ("wait_ns_max", ct.c_uint64), ("reserved", ct.c_uint32), ("status", ct.c_int32)]


_SIGNATURES = {
    "nnf_last_error_string": (ct.c_char_p, []),
    "nnf_version": (_I, []),
    "nnf_get_running_configuration": (_I, [ct.POINTER(RunningConfiguration)]),
    "nnf_set_tuning": (_I, [ct.c_char_p, ct.c_longlong]),
    "nnf_bn_train_read_report": (_I, [_P, _P, _P]),
    "nnf_bn_infer_act": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _F, _ACTP, _I, _I64, _I64, _I64]),
    "nnf_bias_bn_infer_act": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _F, _ACTP, _I, _I64, _I64, _I64]),
    "nnf_act_fwd": (_I, [_P, _P, _P, _ACTP, _I64, _I64, _I64]),
    "nnf_act_bwd": (_I, [_P, _P, _P, _P, _ACTP, _I64, _I64, _I64, _I]),
    "nnf_prelu_bwd_weights_workspace_bytes": (_SZ, [_I64, _I64, _I64]),
    "nnf_prelu_bwd_weights": (_I, [_P, _P, _P, _P, _I64, _I64, _I64, _P, _SZ]),
    "nnf_add_fwd": (_I, [_P, _P, ct.POINTER(_P), _I, _F, _I64]),
    "nnf_add_bwd": (_I, [_P, _P, _P, _F, _I64, _I]),
    "nnf_softmax_fwd": (_I, [_P, _P, _P, _I64, _I64, _I64]),
    "nnf_softmax_bwd": (_I, [_P, _P, _P, _P, _I64, _I64, _I64, _I]),
    "nnf_pool_out_size": (_I64, [_I64, ct.c_int32, ct.c_int32, ct.c_int32]),
    "nnf_maxpool_fwd": (_I, [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _POOLP]),
    "nnf_maxpool_bwd": (_I, [_P, _P, _P, _P, _I64, _I64, _I64, _I64, _POOLP, _I]),
    "nnf_bn_add_relu_maxpool_fwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _F, _I64, _I64, _I64, _I64, _POOLP]),
    "nnf_bn_add_relu_maxpool_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _F, _I64, _I64, _I64, _I64, _POOLP]),
    "nnf_bn_train_workspace_bytes": (_SZ, [_I64, _I64, _I64]),
    "nnf_bn_train_stats": (_I, [_P, _P, _P, _I64, _I64, _I64, _P, _SZ]),
    "nnf_bn_train_stats_static": (_I, [_P, _P, _P, _I64, _I64, _I64]),
    "nnf_bn_train_apply_act": (_I, [_P, _P, _P, _P, _P, _P, _P, _D, _F, _ACTP, _I, _I64, _I64, _I64]),
    "nnf_bn_train_fwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _F, _ACTP, _I, _I64, _I64, _I64, _P, _SZ]),
    "nnf_fused_error_check": (_I, []),
    "nnf_bn_train_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _ACTP, _I, _P, _P, _P, _P, _P, _P, _P, _F, _I64, _I64, _I64, _I, _P, _SZ]),
    "nnf_bn_train_stats_publish": (_I, [_P, _P, _P, _I64, _I64, _I64, _P, _SZ, ct.POINTER(_P), _I, _I, _I, ct.c_uint32]),
    "nnf_bn_train_apply_act_peer": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, ct.c_uint32, _D, _F, _ACTP, _I, _I64, _I64, _I64]),
    "nnf_bn_train_bwd_stats_publish": (_I, [_P, _P, _P, _P, _P, _P, _P, _ACTP, _I, _I64, _I64, _I64, _P, _SZ, ct.POINTER(_P), _I, _I, _I, ct.c_uint32]),
    "nnf_bn_train_bwd_apply_peer": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, ct.c_uint32, _P, _D, _ACTP, _I, _P, _P, _P, _P, _P, _P, _P, _F,
                                         _I64, _I64, _I64, _I]),
    "nnf_accuracy_fwd": (_I, [_P, _P, _P, _P, _P, _I, _I64, _I64, _I64]),
    "nnf_avgpool_fwd": (_I, [_P, _P, _P, _I64, _I64, _I64, _I64, _I, _I, _F]),
    "nnf_avgpool_bwd": (_I, [_P, _P, _P, _I64, _I64, _I64, _I64, _I, _I, _F, _I]),
    "nnf_bn_add_relu_avgpool_fwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _F, _I64, _I64, _I64, _I64, _I, _I, _F]),
    "nnf_bn_add_relu_avgpool_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _F, _I64, _I64, _I64, _I64, _I, _I, _F]),
    "nnf_nll_fwd": (_I, [_P, _P, _P, _P, _P, _F, _I64, _I64, _I64]),
    "nnf_nll_bwd": (_I, [_P, _P, _P, _P, _P, _F, _I64, _I64, _I64, _I]),
    "nnf_set_error_sink": (_I, [_P]),
    "nnf_cross_entropy_fwd": (_I, [_P, _P, _P, _P, _P, _F, _I64, _I64, _I64]),
    "nnf_cross_entropy_bwd": (_I, [_P, _P, _P, _P, _P, _F, _I64, _I64, _I64, _I]),
    "nnf_softmax_nll_fwd": (_I, [_P, _P, _P, _P, _P, _P, _F, _I64, _I64, _I64]),
    "nnf_softmax_nll_bwd": (_I, [_P, _P, _P, _P, _P, _F, _I64, _I64, _I64, _I]),
    "nnf_bn_train_mailbox_bytes": (_SZ, [_I64]),
    "nnf_bn_train_sharded_supported": (_I, [_I64, _I64, _I64]),
    "nnf_bn_train_fwd_sharded": (_I, [_P, _P, _P, _P, _P, _P, _P, _F, _ACTP, _I, _I64, _I64, _I64, _D, _P, _SZ, ct.POINTER(_P), _I, _I, ct.c_uint32]),
    "nnf_bn_train_bwd_sharded": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _ACTP, _I, _P, _P, _P, _P, _P, _P, _P, _F, _I64, _I64, _I64, _D, _P, _SZ,
                                      ct.POINTER(_P), _I, _I, ct.c_uint32]),
    "nnf_apply_gradient": (_I, [_P, ct.POINTER(OptPart), _I, _I, _F, _F, _F, ct.c_uint]),
    "nnf_bn_calibrate_workspace_bytes": (_SZ, [_I64]),
    "nnf_bn_calibrate_accumulator_bytes": (_SZ, [_I64]),
    "nnf_bn_calibrate_accumulate": (_I, [_P, _P, _P, _P, _P, _I64, _I64, _I64, _P, _SZ]),
    "nnf_bn_calibrate_finish": (_I, [_P, _P, _P, _P, _P, _I64]),
    "nnf_peer_exchange_bytes": (_SZ, [_I]),
    "nnf_peer_publish": (_I, [_P, _P, ct.POINTER(_P), _I, _I, _I, _I, ct.c_uint32]),
    "nnf_peer_gather_sum": (_I, [_P, _P, _P, _I, _I, _I, ct.c_uint32]),
    "nnf_peer_exchange_sum": (_I, [_P, _P, _P, ct.POINTER(_P), _I, _I, _I, _I, ct.c_uint32]),
    "nnf_bn_train_bwd_stats": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _ACTP, _I, _I64, _I64, _I64, _P, _SZ]),
    "nnf_bn_train_bwd_apply": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _D, _ACTP, _I, _P, _P, _P, _P, _P, _P, _P, _F,
                                    _I64, _I64, _I64, _I]),
}

for _name, (_res, _args) in _SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args

EXPORTS = sorted(_SIGNATURES)


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, int):
        return t
    assert t.is_cuda and t.is_contiguous(), "tensors must be contiguous CUDA tensors"
    return t.data_ptr()


def _stream(stream):
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    return stream.cuda_stream if hasattr(stream, "cuda_stream") else int(stream)


def _check(status):
    if status != 0:
        raise NnfError(status, lib.nnf_last_error_string().decode())


def last_error():
    return lib.nnf_last_error_string().decode()


def relu(slope=0.0):
    return Act(ACT_RELU, slope, 0.0, None)


def prelu(slope_tensor):
    return Act(ACT_PRELU, 0.0, 0.0, _ptr(slope_tensor))


def elu():
    return Act(ACT_ELU, 0.0, 0.0, None)


def tanh(scale=1.0, steepness=1.0):
    return Act(ACT_TANH, scale, steepness, None)


def sigmoid():
    return Act(ACT_SIGMOID, 0.0, 0.0, None)


def _acts(acts):
    acts = list(acts or [])
    arr = (Act * max(len(acts), 1))(*acts)
    return arr, len(acts)


def _nchw(t):
    n, c = t.shape[0], t.shape[1]
    hw = 1
    for d in t.shape[2:]:
        hw *= d
    return n, c, hw


def bn_infer_act(y, x, bn=None, residual=None, add_alpha=1.0, acts=(), stream=None):
    """bn = (gamma, beta, mean, invsigma) device tensors or None."""
    n, c, hw = _nchw(x)
    g, b, m, i = bn if bn is not None else (None, None, None, None)
    arr, k = _acts(acts)
    _check(lib.nnf_bn_infer_act(_stream(stream), _ptr(y), _ptr(x), _ptr(g), _ptr(b), _ptr(m), _ptr(i), _ptr(residual), add_alpha, arr, k, n, c, hw))


def bias_bn_infer_act(y, x, bias, bn=None, residual=None, add_alpha=1.0, acts=(), stream=None):
    """bn_infer_act with a per-channel bias added to x first."""
    n, c, hw = _nchw(x)
    g, b, m, i = bn if bn is not None else (None, None, None, None)
    arr, k = _acts(acts)
    _check(lib.nnf_bias_bn_infer_act(_stream(stream), _ptr(y), _ptr(x), _ptr(bias), _ptr(g), _ptr(b), _ptr(m), _ptr(i), _ptr(residual), add_alpha,
                                     arr, k, n, c, hw))


def act_fwd(y, x, act, stream=None):
    n, c, hw = _nchw(x)
    _check(lib.nnf_act_fwd(_stream(stream), _ptr(y), _ptr(x), ct.byref(act), n, c, hw))


def act_bwd(dx, dy, neurons, act, add_to_destination=False, stream=None):
    n, c, hw = _nchw(dy)
    _check(lib.nnf_act_bwd(_stream(stream), _ptr(dx), _ptr(dy), _ptr(neurons), ct.byref(act), n, c, hw, int(add_to_destination)))


def prelu_bwd_weights(dslope, dy, x, workspace=None, stream=None):
    n, c, hw = _nchw(x)
    need = lib.nnf_prelu_bwd_weights_workspace_bytes(n, c, hw)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
    _check(lib.nnf_prelu_bwd_weights(_stream(stream), _ptr(dslope), _ptr(dy), _ptr(x), n, c, hw, _ptr(workspace), workspace.numel()))


def add_fwd(y, inputs, alpha=1.0, stream=None):
    arr = (_P * len(inputs))(*[_ptr(t) for t in inputs])
    _check(lib.nnf_add_fwd(_stream(stream), _ptr(y), arr, len(inputs), alpha, y.numel()))


def add_bwd(dx, dy, alpha=1.0, add_to_destination=False, stream=None):
    _check(lib.nnf_add_bwd(_stream(stream), _ptr(dx), _ptr(dy), alpha, dy.numel(), int(add_to_destination)))


def softmax_fwd(y, x, stream=None):
    n, c, hw = _nchw(x)
    _check(lib.nnf_softmax_fwd(_stream(stream), _ptr(y), _ptr(x), n, c, hw))


def softmax_bwd(dx, dy, y, add_to_destination=False, stream=None):
    n, c, hw = _nchw(y)
    _check(lib.nnf_softmax_bwd(_stream(stream), _ptr(dx), _ptr(dy), _ptr(y), n, c, hw, int(add_to_destination)))


def pool(win, stride, round_up=(False, False), is_min=False):
    """win/stride/round_up are (w, h) pairs, the reference's dimension order."""
    return Pool(win[0], win[1], stride[0], stride[1], int(round_up[0]), int(round_up[1]), int(is_min))


def pool_out_shape(h, w, p):
    return (int(lib.nnf_pool_out_size(h, p.win_h, p.stride_h, p.round_up_h)), int(lib.nnf_pool_out_size(w, p.win_w, p.stride_w, p.round_up_w)))


def maxpool_fwd(y, argmax, x, p, stream=None):
    n, c, h, w = x.shape
    _check(lib.nnf_maxpool_fwd(_stream(stream), _ptr(y), _ptr(argmax), _ptr(x), n, c, h, w, ct.byref(p)))


def maxpool_bwd(dx, dy, argmax, p, add_to_destination=False, stream=None):
    n, c, h, w = dx.shape
    _check(lib.nnf_maxpool_bwd(_stream(stream), _ptr(dx), _ptr(dy), _ptr(argmax), n, c, h, w, ct.byref(p), int(add_to_destination)))


def bn_add_relu_maxpool_fwd(z, pooled, argmax, x, residual, bn, relu_slope, p, stream=None):
    n, c, h, w = x.shape
    g, b, m, i = bn if bn is not None else (None, None, None, None)
    _check(lib.nnf_bn_add_relu_maxpool_fwd(_stream(stream), _ptr(z), _ptr(pooled), _ptr(argmax), _ptr(x), _ptr(residual), _ptr(g), _ptr(b),
                                           _ptr(m), _ptr(i), relu_slope, n, c, h, w, ct.byref(p)))


def bn_add_relu_maxpool_bwd(dx, dresidual, dpooled, argmax, z, gamma, invsigma, relu_slope, p, stream=None):
    n, c, h, w = z.shape
    _check(lib.nnf_bn_add_relu_maxpool_bwd(_stream(stream), _ptr(dx), _ptr(dresidual), _ptr(dpooled), _ptr(argmax), _ptr(z), _ptr(gamma),
                                           _ptr(invsigma), relu_slope, n, c, h, w, ct.byref(p)))


def bn_train_workspace_bytes(n, c, hw):
    return int(lib.nnf_bn_train_workspace_bytes(n, c, hw))


def bn_train_stats(sums, x, workspace, stream=None):
    n, c, hw = _nchw(x)
    _check(lib.nnf_bn_train_stats(_stream(stream), _ptr(sums), _ptr(x), n, c, hw, _ptr(workspace), workspace.numel() * workspace.element_size()))


def bn_train_stats_static(sums, x, stream=None):
    """nnf_bn_train_stats without a workspace argument (library-resident scratch, c <= 1024)."""
    n, c, hw = _nchw(x)
    _check(lib.nnf_bn_train_stats_static(_stream(stream), _ptr(sums), _ptr(x), n, c, hw))


def bn_train_apply_act(y, saved, x, gamma, beta, sums, count_total, eps, acts=(), stream=None):
    n, c, hw = _nchw(x)
    arr, k = _acts(acts)
    _check(lib.nnf_bn_train_apply_act(_stream(stream), _ptr(y), _ptr(saved), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(sums), float(count_total), eps,
                                      arr, k, n, c, hw))


def bn_train_fwd(y, saved, sums, x, gamma, beta, eps, acts=(), workspace=None, stream=None):
    n, c, hw = _nchw(x)
    arr, k = _acts(acts)
    nbytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
    _check(lib.nnf_bn_train_fwd(_stream(stream), _ptr(y), _ptr(saved), _ptr(sums), _ptr(x), _ptr(gamma), _ptr(beta), eps, arr, k, n, c, hw,
                                _ptr(workspace), nbytes))


def bn_train_bwd(dx, bsums, dy, x, gamma, beta, saved, acts=(), grad_gamma=None, grad_beta=None, grad_mean=None, grad_invsigma=None,
                 grad_slope=None, mean=None, invsigma=None, entry_count=0.0, add_to_destination=False, workspace=None, stream=None):
    n, c, hw = _nchw(x)
    arr, k = _acts(acts)
    nbytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
    _check(lib.nnf_bn_train_bwd(_stream(stream), _ptr(dx), _ptr(bsums), _ptr(dy), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(saved), arr, k,
                                _ptr(grad_gamma), _ptr(grad_beta), _ptr(grad_mean), _ptr(grad_invsigma), _ptr(grad_slope), _ptr(mean), _ptr(invsigma),
                                float(entry_count), n, c, hw, int(add_to_destination), _ptr(workspace), nbytes))


def peer_exchange_bytes(kmax):
    return int(lib.nnf_peer_exchange_bytes(kmax))


def _ptr_table(ptrs):
    return (_P * len(ptrs))(*[int(p) if not hasattr(p, "data_ptr") else p.data_ptr() for p in ptrs])


def peer_publish(local, peer_ptrs, rank, world, kmax, seq, stream=None):
    _check(lib.nnf_peer_publish(_stream(stream), _ptr(local), _ptr_table(peer_ptrs), rank, world, local.numel(), kmax, seq))


def peer_gather_sum(out, my_buf, world, kmax, seq, stream=None):
    _check(lib.nnf_peer_gather_sum(_stream(stream), _ptr(out), _ptr(my_buf), world, out.numel(), kmax, seq))


def peer_exchange_sum(out, local, peer_ptrs, rank, world, kmax, seq, stream=None):
    _check(lib.nnf_peer_exchange_sum(_stream(stream), _ptr(out), _ptr(local), _ptr_table(peer_ptrs), rank, world, local.numel(), kmax, seq))


def fused_error_check():
    return int(lib.nnf_fused_error_check())


def running_configuration():
    """The current device as the launch plans see it (a dict by nnForge's cuda_running_configuration field names)."""
    cfg = RunningConfiguration()
    _check(lib.nnf_get_running_configuration(ct.byref(cfg)))
    return {name: int(getattr(cfg, name)) for name, _ in RunningConfiguration._fields_}


def set_error_sink(word):
    """`word`: a pinned int32 CPU tensor of one element (or None to restore the device-side word): launches whose bounded wait runs
    out store their code there, and the host reads it as ordinary memory (see nnf_set_error_sink)."""
    if word is not None:
        assert word.dtype == torch.int32 and word.numel() >= 1 and not word.is_cuda and word.is_pinned()
    _check(lib.nnf_set_error_sink(None if word is None else word.data_ptr()))


def set_tuning(name, value):
    """One knob of the launch plans (see nnf_set_tuning in the header); set_tuning("reset", 0) restores the built-in choices."""
    _check(lib.nnf_set_tuning(name.encode(), int(value)))


REPORT_WORDS = ct.sizeof(LaunchReport) // 8


def read_report(host_words, workspace, stream=None):
    """Enqueues the copy of the launch report at the head of `workspace` into `host_words` (a pinned int64 tensor of
    REPORT_WORDS elements); parse it with parse_report() once the stream has passed this point."""
    assert host_words.dtype == torch.int64 and host_words.numel() >= REPORT_WORDS and not host_words.is_cuda
    _check(lib.nnf_bn_train_read_report(_stream(stream), host_words.data_ptr(), _ptr(workspace)))


def parse_report(host_words):
    w = [int(v) & 0xFFFFFFFFFFFFFFFF for v in host_words[:REPORT_WORDS].tolist()]
    status = (w[2] >> 32) & 0xFFFFFFFF
    if status >= 1 << 31:
        status -= 1 << 32
    return {"wait_ns_total": w[0], "wait_ns_max": w[1], "status": status}


def bn_train_bwd_stats(bsums, dy, x, gamma, beta, saved, acts, workspace, gsums=None, stream=None):
    n, c, hw = _nchw(x)
    arr, k = _acts(acts)
    _check(lib.nnf_bn_train_bwd_stats(_stream(stream), _ptr(bsums), _ptr(gsums), _ptr(dy), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(saved), arr, k, n, c, hw,
                                      _ptr(workspace), workspace.numel() * workspace.element_size()))


def bn_train_bwd_apply(dx, dy, x, gamma, beta, saved, gsums, bsums, count_total, acts=(), grad_gamma=None, grad_beta=None, grad_mean=None,
                       grad_invsigma=None, grad_slope=None, mean=None, invsigma=None, entry_count=0.0, add_to_destination=False, stream=None):
    n, c, hw = _nchw(x)
    arr, k = _acts(acts)
    _check(lib.nnf_bn_train_bwd_apply(_stream(stream), _ptr(dx), _ptr(dy), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(saved), _ptr(gsums), _ptr(bsums),
                                      float(count_total), arr, k, _ptr(grad_gamma), _ptr(grad_beta), _ptr(grad_mean), _ptr(grad_invsigma),
                                      _ptr(grad_slope), _ptr(mean), _ptr(invsigma), float(entry_count), n, c, hw, int(add_to_destination)))


def avgpool_fwd(y, x, win, mult, stream=None):
    """x [N,C,H,W]; win = (w, h)."""
    n, c, h, w = x.shape
    _check(lib.nnf_avgpool_fwd(_stream(stream), _ptr(y), _ptr(x), n, c, h, w, win[0], win[1], mult))


def avgpool_bwd(dx, dy, win, mult, add_to_destination=False, stream=None):
    n, c, h, w = dx.shape
    _check(lib.nnf_avgpool_bwd(_stream(stream), _ptr(dx), _ptr(dy), n, c, h, w, win[0], win[1], mult, int(add_to_destination)))


def bn_add_relu_avgpool_fwd(z, pooled, x, residual, bn, relu_slope, win, mult, stream=None):
    n, c, h, w = x.shape
    g, b, m, i = bn if bn is not None else (None, None, None, None)
    _check(lib.nnf_bn_add_relu_avgpool_fwd(_stream(stream), _ptr(z), _ptr(pooled), _ptr(x), _ptr(residual), _ptr(g), _ptr(b), _ptr(m), _ptr(i),
                                           relu_slope, n, c, h, w, win[0], win[1], mult))


def bn_add_relu_avgpool_bwd(dx, dresidual, dpooled, z, gamma, invsigma, relu_slope, win, mult, stream=None):
    n, c, h, w = z.shape
    _check(lib.nnf_bn_add_relu_avgpool_bwd(_stream(stream), _ptr(dx), _ptr(dresidual), _ptr(dpooled), _ptr(z), _ptr(gamma), _ptr(invsigma), relu_slope,
                                           n, c, h, w, win[0], win[1], mult))


def accuracy_fwd(out, predicted, targets, mask=None, top_n=1, stream=None):
    n, c, hw = _nchw(predicted)
    _check(lib.nnf_accuracy_fwd(_stream(stream), _ptr(out), _ptr(predicted), _ptr(targets), _ptr(mask), top_n, n, c, hw))


def nll_fwd(err, predicted, targets, mask=None, scale=1.0, stream=None):
    n, c, hw = _nchw(predicted)
    _check(lib.nnf_nll_fwd(_stream(stream), _ptr(err), _ptr(predicted), _ptr(targets), _ptr(mask), scale, n, c, hw))


def nll_bwd(dpredicted, predicted, targets, mask=None, scale=1.0, add_to_destination=False, stream=None):
    n, c, hw = _nchw(predicted)
    _check(lib.nnf_nll_bwd(_stream(stream), _ptr(dpredicted), _ptr(predicted), _ptr(targets), _ptr(mask), scale, n, c, hw, int(add_to_destination)))


def cross_entropy_fwd(err, predicted, targets, mask=None, scale=1.0, stream=None):
    n, c, hw = _nchw(predicted)
    _check(lib.nnf_cross_entropy_fwd(_stream(stream), _ptr(err), _ptr(predicted), _ptr(targets), _ptr(mask), scale, n, c, hw))


def cross_entropy_bwd(dpredicted, predicted, targets, mask=None, scale=1.0, add_to_destination=False, stream=None):
    n, c, hw = _nchw(predicted)
    _check(lib.nnf_cross_entropy_bwd(_stream(stream), _ptr(dpredicted), _ptr(predicted), _ptr(targets), _ptr(mask), scale, n, c, hw, int(add_to_destination)))


def softmax_nll_fwd(probs, err, logits, targets, mask=None, scale=1.0, stream=None):
    n, c, hw = _nchw(logits)
    _check(lib.nnf_softmax_nll_fwd(_stream(stream), _ptr(probs), _ptr(err), _ptr(logits), _ptr(targets), _ptr(mask), scale, n, c, hw))


def softmax_nll_bwd(dlogits, probs, targets, mask=None, scale=1.0, add_to_destination=False, stream=None):
    n, c, hw = _nchw(probs)
    _check(lib.nnf_softmax_nll_bwd(_stream(stream), _ptr(dlogits), _ptr(probs), _ptr(targets), _ptr(mask), scale, n, c, hw, int(add_to_destination)))


def bn_train_sharded_supported(n, c, hw):
    return bool(lib.nnf_bn_train_sharded_supported(n, c, hw))


def bn_train_mailbox_bytes(c):
    return int(lib.nnf_bn_train_mailbox_bytes(c))


def bn_train_fwd_sharded(y, saved, sums, x, gamma, beta, eps, acts, count_total, workspace, mailbox_ptrs, rank, world, seq, stream=None):
    n, c, hw = _nchw(x)
    arr, k = _acts(acts)
    _check(lib.nnf_bn_train_fwd_sharded(_stream(stream), _ptr(y), _ptr(saved), _ptr(sums), _ptr(x), _ptr(gamma), _ptr(beta), eps, arr, k, n, c, hw,
                                        float(count_total), _ptr(workspace), workspace.numel() * workspace.element_size(),
                                        _ptr_table(mailbox_ptrs), rank, world, seq))


def bn_train_bwd_sharded(dx, bsums, dy, x, gamma, beta, saved, acts, count_total, workspace, mailbox_ptrs, rank, world, seq, grad_gamma=None,
                         grad_beta=None, grad_mean=None, grad_invsigma=None, grad_slope=None, mean=None, invsigma=None, entry_count=0.0, stream=None):
    n, c, hw = _nchw(x)
    arr, k = _acts(acts)
    _check(lib.nnf_bn_train_bwd_sharded(_stream(stream), _ptr(dx), _ptr(bsums), _ptr(dy), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(saved), arr, k,
                                        _ptr(grad_gamma), _ptr(grad_beta), _ptr(grad_mean), _ptr(grad_invsigma), _ptr(grad_slope), _ptr(mean),
                                        _ptr(invsigma), float(entry_count), n, c, hw, float(count_total), _ptr(workspace),
                                        workspace.numel() * workspace.element_size(), _ptr_table(mailbox_ptrs), rank, world, seq))


def bn_train_stats_publish(sums, x, workspace, peer_ptrs, rank, world, kmax, seq, stream=None):
    n, c, hw = _nchw(x)
    _check(lib.nnf_bn_train_stats_publish(_stream(stream), _ptr(sums), _ptr(x), n, c, hw, _ptr(workspace), workspace.numel() * workspace.element_size(),
                                          _ptr_table(peer_ptrs), rank, world, kmax, seq))


def bn_train_apply_act_peer(y, saved, x, gamma, beta, my_buf, world, kmax, seq, count_total, eps, acts=(), stream=None):
    n, c, hw = _nchw(x)
    arr, k = _acts(acts)
    _check(lib.nnf_bn_train_apply_act_peer(_stream(stream), _ptr(y), _ptr(saved), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(my_buf), world, kmax, seq,
                                           float(count_total), eps, arr, k, n, c, hw))


def bn_train_bwd_stats_publish(bsums, dy, x, gamma, beta, saved, acts, workspace, peer_ptrs, rank, world, kmax, seq, stream=None):
    n, c, hw = _nchw(x)
    arr, k = _acts(acts)
    _check(lib.nnf_bn_train_bwd_stats_publish(_stream(stream), _ptr(bsums), _ptr(dy), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(saved), arr, k, n, c, hw,
                                              _ptr(workspace), workspace.numel() * workspace.element_size(), _ptr_table(peer_ptrs), rank, world, kmax, seq))


def bn_train_bwd_apply_peer(dx, dy, x, gamma, beta, saved, my_buf, world, kmax, seq, bsums, count_total, acts=(), grad_gamma=None, grad_beta=None,
                            grad_mean=None, grad_invsigma=None, grad_slope=None, mean=None, invsigma=None, entry_count=0.0, add_to_destination=False,
                            stream=None):
    n, c, hw = _nchw(x)
    arr, k = _acts(acts)
    _check(lib.nnf_bn_train_bwd_apply_peer(_stream(stream), _ptr(dx), _ptr(dy), _ptr(x), _ptr(gamma), _ptr(beta), _ptr(saved), _ptr(my_buf), world, kmax,
                                           seq, _ptr(bsums), float(count_total), arr, k, _ptr(grad_gamma), _ptr(grad_beta), _ptr(grad_mean),
                                           _ptr(grad_invsigma), _ptr(grad_slope), _ptr(mean), _ptr(invsigma), float(entry_count), n, c, hw,
                                           int(add_to_destination)))


def apply_gradient(parts, momentum_type=MOMENTUM_NONE, momentum=0.9, momentum2=0.999, normalizer=1.0, iteration_id=1, stream=None):
    """parts: list of dicts {data, gradient, [prev_upd], [prev_upd2], [update_accum (float64 tensor of 1)], learning_rate,
    [weight_decay]}; every chunk of the list is updated by one launch (48 chunks per launch)."""
    arr = (OptPart * max(len(parts), 1))()
    for k, part in enumerate(parts):
        arr[k] = OptPart(_ptr(part["data"]), _ptr(part["gradient"]), _ptr(part.get("prev_upd")), _ptr(part.get("prev_upd2")),
                         _ptr(part.get("update_accum")), part["learning_rate"], part.get("weight_decay", 0.0), part["data"].numel())
    _check(lib.nnf_apply_gradient(_stream(stream), arr, len(parts), momentum_type, momentum, momentum2, normalizer, iteration_id))


def bn_calibrate_accumulator(c, device="cuda"):
    return torch.zeros(lib.nnf_bn_calibrate_accumulator_bytes(c) // 8, dtype=torch.float64, device=device)


def bn_calibrate_accumulate(accumulator, x, mean, invsigma, workspace=None, stream=None):
    n, c, hw = _nchw(x)
    if workspace is None:
        workspace = torch.empty(lib.nnf_bn_calibrate_workspace_bytes(c), dtype=torch.uint8, device=x.device)
    _check(lib.nnf_bn_calibrate_accumulate(_stream(stream), _ptr(accumulator), _ptr(x), _ptr(mean), _ptr(invsigma), n, c, hw,
                                           _ptr(workspace), workspace.numel() * workspace.element_size()))


def bn_calibrate_finish(accumulator, c, mean=None, invsigma=None, stats=None, stream=None):
    _check(lib.nnf_bn_calibrate_finish(_stream(stream), _ptr(mean), _ptr(invsigma), _ptr(stats), _ptr(accumulator), c))
