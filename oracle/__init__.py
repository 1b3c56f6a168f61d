"""numpy-facing wrappers around the CPU checker libraries. TEST INFRASTRUCTURE ONLY.

``Oracle``    -> oracle/nnf_oracle.c (our C restatement of nnForge's plain backend)
``Reference`` -> oracle/_ref/libnnf_plain_ref*.so (nnForge's own plain sources, compiled in place)

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this package; the
product package ``nnforge_b200`` never does.
"""
import ctypes as ct
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

_f32p = ct.POINTER(ct.c_float)
_f64p = ct.POINTER(ct.c_double)
_u32p = ct.POINTER(ct.c_uint32)
_i64 = ct.c_int64


def _fp(a):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f32p)


def _dp(a):
    assert a.dtype == np.float64 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f64p)


def _up(a):
    if a is None:
        return None
    assert a.dtype == np.uint32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_u32p)


def _c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Oracle:
    """C restatement. ``parallel=True`` loads the OpenMP build (CPU baseline timing)."""

    def __init__(self, parallel=False):
        from . import build_oracle
        build_oracle.build()
        self.lib = ct.CDLL(build_oracle.LIB_OMP if parallel else build_oracle.LIB)
        self.lib.orc_max_threads.restype = ct.c_int
        if parallel:
            try:
                cores = len(os.sched_getaffinity(0))
            except Exception:
                cores = os.cpu_count() or 1
            self.lib.orc_set_threads(ct.c_int(cores))
        self.lib.orc_maxpool_out_size.restype = _i64
        self.lib.orc_maxpool_out_size.argtypes = [_i64, _i64, _i64, ct.c_int]
        self.threads = self.lib.orc_max_threads()

    # ---- inference batch norm and activations -------------------------------------------------
    def bn_infer(self, x, gamma, beta, mean, invsigma):
        x = _c(x)
        n, c = x.shape[0], x.shape[1]
        hw = x.size // (n * c) if x.size else 0
        y = np.empty_like(x)
        self.lib.orc_bn_infer(_fp(y), _fp(x), _fp(_c(gamma)), _fp(_c(beta)), _fp(_c(mean)), _fp(_c(invsigma)), _i64(n), _i64(c), _i64(hw))
        return y

    def relu_fwd(self, x, slope=0.0):
        x = _c(x)
        y = np.empty_like(x)
        self.lib.orc_relu_fwd(_fp(y), _fp(x), ct.c_float(slope), _i64(x.size))
        return y

    def relu_bwd(self, dy, x, slope=0.0, dx=None):
        dy, x = _c(dy), _c(x)
        add = dx is not None
        out = _c(dx).copy() if add else np.empty_like(dy)
        self.lib.orc_relu_bwd(_fp(out), _fp(dy), _fp(x), ct.c_float(slope), _i64(x.size), int(add))
        return out

    def prelu_fwd(self, x, slope):
        x = _c(x)
        n, c = x.shape[0], x.shape[1]
        y = np.empty_like(x)
        self.lib.orc_prelu_fwd(_fp(y), _fp(x), _fp(_c(slope)), _i64(n), _i64(c), _i64(x.size // max(n * c, 1)))
        return y

    def prelu_bwd_data(self, dy, x, slope, dx=None):
        dy, x = _c(dy), _c(x)
        n, c = x.shape[0], x.shape[1]
        add = dx is not None
        out = _c(dx).copy() if add else np.empty_like(dy)
        self.lib.orc_prelu_bwd_data(_fp(out), _fp(dy), _fp(x), _fp(_c(slope)), _i64(n), _i64(c), _i64(x.size // max(n * c, 1)), int(add))
        return out

    def prelu_bwd_weights(self, dy, x, dslope=None):
        dy, x = _c(dy), _c(x)
        n, c = x.shape[0], x.shape[1]
        out = np.zeros(c, np.float32) if dslope is None else _c(dslope).copy()
        self.lib.orc_prelu_bwd_weights(_fp(out), _fp(dy), _fp(x), _i64(n), _i64(c), _i64(x.size // max(n * c, 1)))
        return out

    def elu_fwd(self, x):
        x = _c(x)
        y = np.empty_like(x)
        self.lib.orc_elu_fwd(_fp(y), _fp(x), _i64(x.size))
        return y

    def _bwd_from_output(self, fn, dy, y, dx, *params):
        dy, y = _c(dy), _c(y)
        add = dx is not None
        out = _c(dx).copy() if add else np.empty_like(dy)
        fn(_fp(out), _fp(dy), _fp(y), *params, _i64(y.size), int(add))
        return out

    def elu_bwd(self, dy, y, dx=None):
        return self._bwd_from_output(self.lib.orc_elu_bwd, dy, y, dx)

    def tanh_fwd(self, x, scale=1.0, steepness=1.0):
        x = _c(x)
        y = np.empty_like(x)
        self.lib.orc_tanh_fwd(_fp(y), _fp(x), ct.c_float(scale), ct.c_float(steepness), _i64(x.size))
        return y

    def tanh_bwd(self, dy, y, scale=1.0, steepness=1.0, dx=None):
        return self._bwd_from_output(self.lib.orc_tanh_bwd, dy, y, dx, ct.c_float(scale), ct.c_float(steepness))

    def sigmoid_fwd(self, x):
        x = _c(x)
        y = np.empty_like(x)
        self.lib.orc_sigmoid_fwd(_fp(y), _fp(x), _i64(x.size))
        return y

    def sigmoid_bwd(self, dy, y, dx=None):
        return self._bwd_from_output(self.lib.orc_sigmoid_bwd, dy, y, dx)

    # ---- add -----------------------------------------------------------------------------------
    def add_fwd(self, inputs, alpha=1.0):
        inputs = [_c(a) for a in inputs]
        y = np.empty_like(inputs[0])
        arr = (_f32p * len(inputs))(*[_fp(a) for a in inputs])
        self.lib.orc_add_fwd(_fp(y), arr, len(inputs), ct.c_float(alpha), _i64(y.size))
        return y

    def add_bwd(self, dy, alpha=1.0, dx=None):
        dy = _c(dy)
        add = dx is not None
        out = _c(dx).copy() if add else np.empty_like(dy)
        self.lib.orc_add_bwd(_fp(out), _fp(dy), ct.c_float(alpha), _i64(dy.size), int(add))
        return out

    # ---- softmax -------------------------------------------------------------------------------
    def softmax_fwd(self, x):
        x = _c(x)
        n, c = x.shape[0], x.shape[1]
        y = np.empty_like(x)
        self.lib.orc_softmax_fwd(_fp(y), _fp(x), _i64(n), _i64(c), _i64(x.size // max(n * c, 1)))
        return y

    def softmax_bwd(self, dy, y, dx=None):
        dy, y = _c(dy), _c(y)
        n, c = y.shape[0], y.shape[1]
        add = dx is not None
        out = _c(dx).copy() if add else np.empty_like(dy)
        self.lib.orc_softmax_bwd(_fp(out), _fp(dy), _fp(y), _i64(n), _i64(c), _i64(y.size // max(n * c, 1)), int(add))
        return out

    # ---- negative log likelihood ------------------------------------------------------------------
    def nll_fwd(self, predicted, actual, mask=None, scale=1.0):
        """predicted, actual [N,C,H,W]; mask [N,1,H,W] or None -> err [N,1,H,W]."""
        predicted, actual = _c(predicted), _c(actual)
        n, c = predicted.shape[0], predicted.shape[1]
        hw = predicted.size // max(n * c, 1)
        err = np.empty((n, 1) + predicted.shape[2:], np.float32)
        m = _c(mask) if mask is not None else None
        self.lib.orc_nll_fwd(_fp(err), _fp(predicted), _fp(actual), _fp(m) if m is not None else None, ct.c_float(scale), _i64(n), _i64(c), _i64(hw))
        return err

    def nll_bwd(self, predicted, actual, mask=None, scale=1.0, dx=None):
        predicted, actual = _c(predicted), _c(actual)
        n, c = predicted.shape[0], predicted.shape[1]
        hw = predicted.size // max(n * c, 1)
        add = dx is not None
        out = _c(dx).copy() if add else np.empty_like(predicted)
        m = _c(mask) if mask is not None else None
        self.lib.orc_nll_bwd(_fp(out), _fp(predicted), _fp(actual), _fp(m) if m is not None else None, ct.c_float(scale), _i64(n), _i64(c), _i64(hw), int(add))
        return out

    # ---- cross entropy ------------------------------------------------------------------------------
    def cross_entropy_fwd(self, predicted, actual, mask=None, scale=1.0, mask_replaces_scale=False):
        """predicted, actual [N,C,H,W]; mask [N,1,H,W] or None -> err [N,1,H,W]. mask_replaces_scale: the reference tester's
        total scale (the mask alone) instead of the updater's (scale * mask)."""
        predicted, actual = _c(predicted), _c(actual)
        n, c = predicted.shape[0], predicted.shape[1]
        hw = predicted.size // max(n * c, 1)
        err = np.empty((n, 1) + predicted.shape[2:], np.float32)
        m = _c(mask) if mask is not None else None
        self.lib.orc_cross_entropy_fwd(_fp(err), _fp(predicted), _fp(actual), _fp(m) if m is not None else None, ct.c_float(scale), _i64(n), _i64(c),
                                       _i64(hw), int(mask_replaces_scale))
        return err

    def cross_entropy_bwd(self, predicted, actual, mask=None, scale=1.0, dx=None):
        predicted, actual = _c(predicted), _c(actual)
        n, c = predicted.shape[0], predicted.shape[1]
        hw = predicted.size // max(n * c, 1)
        add = dx is not None
        out = _c(dx).copy() if add else np.empty_like(predicted)
        m = _c(mask) if mask is not None else None
        self.lib.orc_cross_entropy_bwd(_fp(out), _fp(predicted), _fp(actual), _fp(m) if m is not None else None, ct.c_float(scale), _i64(n), _i64(c),
                                       _i64(hw), int(add))
        return out

    def accuracy_fwd(self, predicted, actual, mask=None, top_n=1):
        """predicted, actual [N,C,H,W]; mask [N,1,H,W] or None -> [N,top_n+1,H,W]."""
        predicted, actual = _c(predicted), _c(actual)
        n, c = predicted.shape[0], predicted.shape[1]
        hw = predicted.size // max(n * c, 1)
        out = np.empty((n, top_n + 1) + predicted.shape[2:], np.float32)
        m = _c(mask) if mask is not None else None
        self.lib.orc_accuracy_fwd(_fp(out), _fp(predicted), _fp(actual), _fp(m) if m is not None else None, _i64(top_n), _i64(n), _i64(c), _i64(hw))
        return out

    # ---- optimiser step and batch-norm recalibration ------------------------------------------------------
    MOMENTUM = {"none": 0, "vanilla": 1, "nesterov": 2, "adam": 3}

    def apply_gradient(self, data, gradient, prev_upd=None, prev_upd2=None, momentum_type="none", learning_rate=0.01, normalizer=1.0,
                       weight_decay=0.0, momentum=0.9, momentum2=0.999, iteration_id=1):
        """One weight chunk, updated IN PLACE (float32 arrays); returns the sum of |update|."""
        self.lib.orc_apply_gradient.restype = ct.c_double
        return self.lib.orc_apply_gradient(_fp(data), _fp(gradient), _fp(prev_upd), _fp(prev_upd2), _i64(data.size), self.MOMENTUM[momentum_type],
                                           ct.c_float(learning_rate), ct.c_float(normalizer), ct.c_float(weight_decay), ct.c_float(momentum),
                                           ct.c_float(momentum2), ct.c_uint(iteration_id))

    def feature_map_stats(self, batches):
        """batches: iterable of [N,C,...] arrays -> stats[4][C] = min, max, average, std_dev over all of them."""
        state = minmax = None
        for y in batches:
            y = _c(y)
            n, c = y.shape[0], y.shape[1]
            if state is None:
                state = np.zeros((c, 3), np.float64)
                minmax = np.tile(np.array([np.finfo(np.float32).max, -np.finfo(np.float32).max], np.float32), (c, 1)).copy()
            self.lib.orc_feature_map_stats_update(_dp(state), _fp(minmax), _fp(y), _i64(n), _i64(c), _i64(y.size // (n * c)))
        stats = np.empty((4, state.shape[0]), np.float32)
        self.lib.orc_feature_map_stats_get(_fp(stats), _dp(state), _fp(minmax), _i64(state.shape[0]))
        return stats

    def bn_recalibrate(self, mean, invsigma, stats):
        mean, invsigma = _c(mean).copy(), _c(invsigma).copy()
        self.lib.orc_bn_recalibrate(_fp(mean), _fp(invsigma), _fp(_c(stats)), _i64(mean.size))
        return mean, invsigma

    # ---- average subsampling ------------------------------------------------------------------------
    def avgpool_fwd(self, x, win, mult=None):
        """x [N,C,H,W]; win = (w, h); mult defaults to 1 / window elements."""
        x = _c(x)
        n, c, h, w = x.shape
        mult = np.float32(1.0) / np.float32(win[0] * win[1]) if mult is None else np.float32(mult)
        y = np.empty((n, c, h // win[1], w // win[0]), np.float32)
        self.lib.orc_avgpool_fwd(_fp(y), _fp(x), _i64(n * c), _i64(h), _i64(w), _i64(win[0]), _i64(win[1]), ct.c_float(mult))
        return y

    def avgpool_bwd(self, dy, in_shape, win, mult=None, dx=None):
        dy = _c(dy)
        n, c, h, w = in_shape
        mult = np.float32(1.0) / np.float32(win[0] * win[1]) if mult is None else np.float32(mult)
        add = dx is not None
        out = _c(dx).copy() if add else np.empty(in_shape, np.float32)
        self.lib.orc_avgpool_bwd(_fp(out), _fp(dy), _i64(n * c), _i64(h), _i64(w), _i64(win[0]), _i64(win[1]), ct.c_float(mult), int(add))
        return out

    # ---- max subsampling -----------------------------------------------------------------------
    def maxpool_out_size(self, size, window, stride, round_up=False):
        return int(self.lib.orc_maxpool_out_size(size, window, stride, int(round_up)))

    def maxpool_fwd(self, x, win, stride, round_up=(False, False), is_min=False, want_argmax=True):
        """x[N,C,H,W]; win/stride/round_up are (w, h) pairs like the reference's dimension order."""
        x = _c(x)
        n, c, h, w = x.shape
        ow = self.maxpool_out_size(w, win[0], stride[0], round_up[0])
        oh = self.maxpool_out_size(h, win[1], stride[1], round_up[1])
        y = np.empty((n, c, oh, ow), np.float32)
        idx = np.empty((n, c, oh, ow), np.uint32) if want_argmax else None
        self.lib.orc_maxpool_fwd(_fp(y), _up(idx), _fp(x), _i64(n), _i64(c), _i64(h), _i64(w), _i64(win[0]), _i64(win[1]),
                                 _i64(stride[0]), _i64(stride[1]), int(round_up[0]), int(round_up[1]), int(is_min))
        return (y, idx) if want_argmax else y

    def maxpool_bwd(self, dy, argmax, in_shape, dx=None):
        dy = _c(dy)
        add = dx is not None
        out = _c(dx).copy() if add else np.empty(in_shape, np.float32)
        self.lib.orc_maxpool_bwd(_fp(out), _fp(dy), _up(np.ascontiguousarray(argmax, np.uint32)), _i64(out.size), _i64(dy.size), int(add))
        return out

    # ---- training-mode batch norm (parity unpinned by reference code) -----------------------------
    def bn_train_sums(self, x, f32=False):
        x = _c(x)
        n, c = x.shape[0], x.shape[1]
        hw = x.size // max(n * c, 1)
        if f32:
            s, q = np.empty(c, np.float32), np.empty(c, np.float32)
            self.lib.orc_bn_train_sums_f32(_fp(s), _fp(q), _fp(x), _i64(n), _i64(c), _i64(hw))
            return s.astype(np.float64), q.astype(np.float64)
        s, q = np.empty(c, np.float64), np.empty(c, np.float64)
        self.lib.orc_bn_train_sums(_dp(s), _dp(q), _fp(x), _i64(n), _i64(c), _i64(hw))
        return s, q

    def bn_train_finalize(self, s, q, count_total, eps):
        c = s.size
        saved = np.empty(2 * c, np.float32)
        self.lib.orc_bn_train_finalize(_fp(saved), _dp(np.ascontiguousarray(s, np.float64)), _dp(np.ascontiguousarray(q, np.float64)),
                                       _i64(c), ct.c_double(count_total), ct.c_float(eps))
        return saved

    def bn_train_apply(self, x, gamma, beta, saved):
        x = _c(x)
        n, c = x.shape[0], x.shape[1]
        y = np.empty_like(x)
        self.lib.orc_bn_train_apply(_fp(y), _fp(x), _fp(_c(gamma)), _fp(_c(beta)), _fp(_c(saved)), _i64(n), _i64(c), _i64(x.size // max(n * c, 1)))
        return y

    def bn_train_fwd(self, x, gamma, beta, eps, f32=False):
        s, q = self.bn_train_sums(x, f32)
        saved = self.bn_train_finalize(s, q, x.size // x.shape[1], eps)
        return self.bn_train_apply(x, gamma, beta, saved), saved

    def bn_train_bwd_sums(self, du, x, saved):
        du, x = _c(du), _c(x)
        n, c = x.shape[0], x.shape[1]
        db, dg = np.empty(c, np.float64), np.empty(c, np.float64)
        self.lib.orc_bn_train_bwd_sums(_dp(db), _dp(dg), _fp(du), _fp(x), _fp(_c(saved)), _i64(n), _i64(c), _i64(x.size // max(n * c, 1)))
        return db, dg

    def bn_train_bwd_apply(self, du, x, gamma, saved, dbeta, dgamma, count_total, dx=None):
        du, x = _c(du), _c(x)
        n, c = x.shape[0], x.shape[1]
        add = dx is not None
        out = _c(dx).copy() if add else np.empty_like(x)
        self.lib.orc_bn_train_bwd_apply(_fp(out), _fp(du), _fp(x), _fp(_c(gamma)), _fp(_c(saved)), _dp(np.ascontiguousarray(dbeta, np.float64)),
                                        _dp(np.ascontiguousarray(dgamma, np.float64)), _i64(n), _i64(c), _i64(x.size // max(n * c, 1)),
                                        ct.c_double(count_total), int(add))
        return out

    def bn_train_running_grad(self, grad_mean, grad_invsigma, saved, mean, invsigma, entry_count):
        gm, gi = _c(grad_mean).copy(), _c(grad_invsigma).copy()
        self.lib.orc_bn_train_running_grad(_fp(gm), _fp(gi), _fp(_c(saved)), _fp(_c(mean)), _fp(_c(invsigma)), _i64(gm.size), ct.c_float(entry_count))
        return gm, gi


class Reference:
    """nnForge's own plain-backend sources behind oracle/ref_capi.cpp. ``available`` is False when the
    libraries were never built (no reference checkout on this machine). Methods return
    ``(result..., seconds)`` where seconds is the best wall time of the reference call alone."""

    def __init__(self, parallel=False):
        from . import build_ref
        try:
            build_ref.build(verbose=False)
        except Exception:
            pass
        path = os.path.join(HERE, "_ref", "libnnf_plain_ref_omp.so" if parallel else "libnnf_plain_ref.so")
        self.available = os.path.exists(path)
        self.parallel = parallel
        self.threads = (os.cpu_count() or 1) if parallel else 1
        if not self.available:
            return
        self.lib = ct.CDLL(path)
        self.lib.ref_last_error.restype = ct.c_char_p
        for fn in ("ref_bn_infer", "ref_relu_fwd", "ref_relu_bwd", "ref_prelu_fwd", "ref_prelu_bwd_data", "ref_prelu_bwd_weights",
                   "ref_elu_fwd", "ref_elu_bwd", "ref_tanh_fwd", "ref_tanh_bwd", "ref_sigmoid_fwd", "ref_sigmoid_bwd", "ref_softmax_fwd",
                   "ref_softmax_upd_fwd", "ref_softmax_bwd", "ref_add_fwd", "ref_add_bwd", "ref_maxpool_fwd", "ref_maxpool_tester_fwd",
                   "ref_maxpool_bwd", "ref_nll_fwd", "ref_nll_bwd", "ref_cross_entropy_fwd", "ref_cross_entropy_bwd", "ref_accuracy_fwd", "ref_avgpool_fwd", "ref_avgpool_bwd", "ref_feature_map_stats"):
            getattr(self.lib, fn).restype = ct.c_double

    def _check(self, seconds):
        if seconds < 0:
            raise RuntimeError("reference threw: " + self.lib.ref_last_error().decode())
        return seconds

    @staticmethod
    def _dims(x):
        x = _c(x)
        shape = tuple(x.shape) + (1,) * (4 - x.ndim)
        return x, [ct.c_uint(int(v)) for v in shape]

    def bn_infer(self, x, gamma, beta, mean, invsigma, reps=1):
        x, d = self._dims(x)
        y = np.empty_like(x)
        s = self.lib.ref_bn_infer(_fp(y), _fp(x), _fp(_c(gamma)), _fp(_c(beta)), _fp(_c(mean)), _fp(_c(invsigma)), *d, self.threads, reps)
        return y, self._check(s)

    def relu_fwd(self, x, slope=0.0, reps=1):
        x, d = self._dims(x)
        y = np.empty_like(x)
        return y, self._check(self.lib.ref_relu_fwd(_fp(y), _fp(x), ct.c_float(slope), *d, self.threads, reps))

    def relu_bwd(self, dy, x, slope=0.0, dx=None, reps=1):
        x, d = self._dims(x)
        out = _c(dx).copy() if dx is not None else np.empty_like(x)
        s = self.lib.ref_relu_bwd(_fp(out), _fp(_c(dy)), _fp(x), ct.c_float(slope), *d, int(dx is not None), self.threads, reps)
        return out, self._check(s)

    def prelu_fwd(self, x, slope, reps=1):
        x, d = self._dims(x)
        y = np.empty_like(x)
        return y, self._check(self.lib.ref_prelu_fwd(_fp(y), _fp(x), _fp(_c(slope)), *d, self.threads, reps))

    def prelu_bwd_data(self, dy, x, slope, dx=None, reps=1):
        x, d = self._dims(x)
        out = _c(dx).copy() if dx is not None else np.empty_like(x)
        s = self.lib.ref_prelu_bwd_data(_fp(out), _fp(_c(dy)), _fp(x), _fp(_c(slope)), *d, int(dx is not None), self.threads, reps)
        return out, self._check(s)

    def prelu_bwd_weights(self, dy, x, dslope=None):
        x, d = self._dims(x)
        out = np.zeros(x.shape[1], np.float32) if dslope is None else _c(dslope).copy()
        s = self.lib.ref_prelu_bwd_weights(_fp(out), _fp(_c(dy)), _fp(x), *d, self.threads)
        return out, self._check(s)

    def elu_fwd(self, x, reps=1):
        x, d = self._dims(x)
        y = np.empty_like(x)
        return y, self._check(self.lib.ref_elu_fwd(_fp(y), _fp(x), *d, self.threads, reps))

    def _bwd_out(self, fn, dy, y, dx, reps, *params):
        y, d = self._dims(y)
        out = _c(dx).copy() if dx is not None else np.empty_like(y)
        s = fn(_fp(out), _fp(_c(dy)), _fp(y), *params, *d, int(dx is not None), self.threads, reps)
        return out, self._check(s)

    def elu_bwd(self, dy, y, dx=None, reps=1):
        return self._bwd_out(self.lib.ref_elu_bwd, dy, y, dx, reps)

    def tanh_fwd(self, x, scale=1.0, steepness=1.0, reps=1):
        x, d = self._dims(x)
        y = np.empty_like(x)
        return y, self._check(self.lib.ref_tanh_fwd(_fp(y), _fp(x), ct.c_float(scale), ct.c_float(steepness), *d, self.threads, reps))

    def tanh_bwd(self, dy, y, scale=1.0, steepness=1.0, dx=None, reps=1):
        return self._bwd_out(self.lib.ref_tanh_bwd, dy, y, dx, reps, ct.c_float(scale), ct.c_float(steepness))

    def sigmoid_fwd(self, x, reps=1):
        x, d = self._dims(x)
        y = np.empty_like(x)
        return y, self._check(self.lib.ref_sigmoid_fwd(_fp(y), _fp(x), *d, self.threads, reps))

    def sigmoid_bwd(self, dy, y, dx=None, reps=1):
        return self._bwd_out(self.lib.ref_sigmoid_bwd, dy, y, dx, reps)

    def softmax_fwd(self, x, reps=1, updater=False):
        x, d = self._dims(x)
        y = np.empty_like(x)
        fn = self.lib.ref_softmax_upd_fwd if updater else self.lib.ref_softmax_fwd
        return y, self._check(fn(_fp(y), _fp(x), *d, self.threads, reps))

    def softmax_bwd(self, dy, y, dx=None, reps=1):
        return self._bwd_out(self.lib.ref_softmax_bwd, dy, y, dx, reps)

    def nll_fwd(self, predicted, actual, mask=None, scale=1.0, updater=False, reps=1):
        predicted, d = self._dims(predicted)
        actual = _c(actual)
        err = np.empty((predicted.shape[0], 1) + predicted.shape[2:], np.float32)
        m = _c(mask) if mask is not None else None
        s = self.lib.ref_nll_fwd(_fp(err), _fp(predicted), _fp(actual), _fp(m) if m is not None else None, ct.c_float(scale), *d, int(updater),
                                 self.threads, reps)
        return err, self._check(s)

    def nll_bwd(self, predicted, actual, mask=None, scale=1.0, dx=None):
        predicted, d = self._dims(predicted)
        actual = _c(actual)
        out = _c(dx).copy() if dx is not None else np.empty_like(predicted)
        m = _c(mask) if mask is not None else None
        s = self.lib.ref_nll_bwd(_fp(out), _fp(predicted), _fp(actual), _fp(m) if m is not None else None, ct.c_float(scale), *d, int(dx is not None),
                                 self.threads)
        return out, self._check(s)

    def cross_entropy_fwd(self, predicted, actual, mask=None, scale=1.0, updater=False, reps=1):
        predicted, d = self._dims(predicted)
        actual = _c(actual)
        err = np.empty((predicted.shape[0], 1) + predicted.shape[2:], np.float32)
        m = _c(mask) if mask is not None else None
        s = self.lib.ref_cross_entropy_fwd(_fp(err), _fp(predicted), _fp(actual), _fp(m) if m is not None else None, ct.c_float(scale), *d, int(updater),
                                           self.threads, reps)
        return err, self._check(s)

    def cross_entropy_bwd(self, predicted, actual, mask=None, scale=1.0, dx=None):
        """The plain backend's backward action as it is: it stores zeros (see orc_cross_entropy_bwd)."""
        predicted, d = self._dims(predicted)
        actual = _c(actual)
        out = _c(dx).copy() if dx is not None else np.empty_like(predicted)
        m = _c(mask) if mask is not None else None
        s = self.lib.ref_cross_entropy_bwd(_fp(out), _fp(predicted), _fp(actual), _fp(m) if m is not None else None, ct.c_float(scale), *d,
                                           int(dx is not None), self.threads)
        return out, self._check(s)

    def accuracy_fwd(self, predicted, actual, mask=None, top_n=1, updater=False, reps=1):
        predicted, d = self._dims(predicted)
        actual = _c(actual)
        out = np.empty((predicted.shape[0], top_n + 1) + predicted.shape[2:], np.float32)
        m = _c(mask) if mask is not None else None
        s = self.lib.ref_accuracy_fwd(_fp(out), _fp(predicted), _fp(actual), _fp(m) if m is not None else None, ct.c_uint(top_n), *d, int(updater),
                                      self.threads, reps)
        return out, self._check(s)

    def feature_map_stats(self, y):
        """y [N,C,H,W] -> stats[4][C] = min, max, average, std_dev (stat_data_bunch_writer)."""
        y, d = self._dims(y)
        stats = np.empty((4, y.shape[1]), np.float32)
        self._check(self.lib.ref_feature_map_stats(_fp(stats), _fp(y), *d))
        return stats

    def avgpool_fwd(self, x, win, updater=False, reps=1):
        x, d = self._dims(x)
        y = np.empty((x.shape[0], x.shape[1], x.shape[2] // win[1], x.shape[3] // win[0]), np.float32)
        return y, self._check(self.lib.ref_avgpool_fwd(_fp(y), _fp(x), *d, win[0], win[1], int(updater), self.threads, reps))

    def avgpool_bwd(self, dy, in_shape, win, dx=None):
        dy = _c(dy)
        out = _c(dx).copy() if dx is not None else np.empty(in_shape, np.float32)
        n, c, h, w = in_shape
        s = self.lib.ref_avgpool_bwd(_fp(out), _fp(dy), n, c, h, w, win[0], win[1], int(dx is not None), self.threads)
        return out, self._check(s)

    def add_fwd(self, inputs, alpha=1.0, reps=1):
        inputs = [_c(a) for a in inputs]
        _, d = self._dims(inputs[0])
        y = np.empty_like(inputs[0])
        arr = (_f32p * len(inputs))(*[_fp(a) for a in inputs])
        return y, self._check(self.lib.ref_add_fwd(_fp(y), arr, len(inputs), ct.c_float(alpha), *d, self.threads, reps))

    def add_bwd(self, dy, alpha=1.0, dx=None, reps=1):
        dy, d = self._dims(dy)
        out = _c(dx).copy() if dx is not None else np.empty_like(dy)
        s = self.lib.ref_add_bwd(_fp(out), _fp(dy), ct.c_float(alpha), *d, int(dx is not None), self.threads, reps)
        return out, self._check(s)

    def maxpool_fwd(self, x, win, stride, is_min=False, reps=1):
        x = _c(x)
        n, c, h, w = x.shape
        oh, ow = ct.c_uint(0), ct.c_uint(0)
        args = [ct.c_uint(v) for v in (n, c, h, w, win[0], win[1], stride[0], stride[1])]
        self._check(self.lib.ref_maxpool_fwd(None, None, None, *args, int(is_min), ct.byref(oh), ct.byref(ow), self.threads, 1))
        y = np.empty((n, c, oh.value, ow.value), np.float32)
        idx = np.empty((n, c, oh.value, ow.value), np.uint32)
        s = self.lib.ref_maxpool_fwd(_fp(y), _up(idx), _fp(x), *args, int(is_min), ct.byref(oh), ct.byref(ow), self.threads, reps)
        return y, idx, self._check(s)

    def maxpool_tester_fwd(self, x, win, stride, is_min=False, reps=1):
        x = _c(x)
        n, c, h, w = x.shape
        args = [ct.c_uint(v) for v in (n, c, h, w, win[0], win[1], stride[0], stride[1])]
        oh = (h + stride[1] - win[1]) // stride[1]
        ow = (w + stride[0] - win[0]) // stride[0]
        y = np.empty((n, c, oh, ow), np.float32)
        s = self.lib.ref_maxpool_tester_fwd(_fp(y), _fp(x), *args, int(is_min), self.threads, reps)
        return y, self._check(s)

    def maxpool_bwd(self, dy, argmax, in_shape, dx=None):
        dy = _c(dy)
        n, c, h, w = in_shape
        out = _c(dx).copy() if dx is not None else np.zeros(in_shape, np.float32)
        s = self.lib.ref_maxpool_bwd(_fp(out), _fp(dy), _up(np.ascontiguousarray(argmax, np.uint32)), ct.c_uint(n), ct.c_uint(c), ct.c_uint(h),
                                     ct.c_uint(w), ct.c_uint(dy.shape[2]), ct.c_uint(dy.shape[3]), 1, self.threads)
        return out, self._check(s)
