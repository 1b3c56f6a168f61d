"""ctypes driver for the C++ host-side layer objects (csrc/host/nnf_layers.{h,cpp}).

`Tester` / `Updater` create an nnForge-shaped layer object by the reference's type name through the
C++ factory and forward each call to the object's member of the same name. Used by the tests; an
nnForge integration would use the C++ classes directly.
"""
import ctypes as ct
import os

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libnnf_b200_host.so")
if not os.path.exists(LIB_PATH):
    raise ImportError("libnnf_b200_host.so is missing: build it with `python -m nnforge_b200.build`")

lib = ct.CDLL(LIB_PATH)
_P = ct.c_void_p
lib.nnfh_last_error.restype = ct.c_char_p
lib.nnfh_create.restype = _P
lib.nnfh_create.argtypes = [ct.c_char_p, ct.c_int, ct.POINTER(ct.c_float), ct.POINTER(ct.c_int), ct.c_uint, ct.c_uint, ct.c_uint, ct.c_int, ct.c_int]
lib.nnfh_destroy.argtypes = [_P]
lib.nnfh_tester_forward.argtypes = [_P, _P, _P, ct.POINTER(_P), ct.c_int, ct.POINTER(_P), ct.c_int, ct.c_uint]
lib.nnfh_tester_can_write.argtypes = [_P]
lib.nnfh_updater_query.restype = ct.c_longlong
lib.nnfh_updater_query.argtypes = [_P, ct.c_int, ct.c_int]
lib.nnfh_updater_forward.argtypes = [_P, _P, _P, ct.POINTER(_P), ct.c_int, ct.POINTER(_P), ct.c_int, _P, ct.c_size_t, _P, _P, ct.c_uint]
lib.nnfh_updater_backward_data.argtypes = [_P, _P, _P, _P, ct.POINTER(_P), ct.c_int, _P, _P, _P, _P, ct.c_int, ct.c_uint]
lib.nnfh_updater_backward_data_inputs.argtypes = [_P, _P, _P, _P, ct.POINTER(_P), ct.c_int, _P, ct.c_int, ct.c_uint]
lib.nnfh_updater_backward_weights.argtypes = [_P, _P, ct.POINTER(_P), ct.c_int, _P, _P, _P, ct.c_size_t, ct.c_uint]
lib.nnfh_updater_backward_data_and_weights.argtypes = [_P, _P, _P, _P, ct.POINTER(_P), ct.c_int, ct.POINTER(_P), ct.c_int, _P, _P, ct.c_size_t, _P, ct.c_int, ct.c_uint]

lib.nnfh_fusion_last_error.restype = ct.c_char_p
lib.nnfh_plan_fusion.argtypes = [ct.c_char_p, ct.c_int, ct.c_char_p, ct.c_size_t]

FORWARD, BACKWARD_DATA, BACKWARD_WEIGHTS, BACKWARD_DATA_AND_WEIGHTS = 0, 1, 2, 3


class HostLayerError(RuntimeError):
    pass


def _ptr(t):
    return None if t is None else t.data_ptr()


def _arr(tensors):
    tensors = list(tensors or [])
    return (_P * max(len(tensors), 1))(*[_ptr(t) for t in tensors]), len(tensors)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _check(status):
    if status != 0:
        raise HostLayerError(lib.nnfh_last_error().decode())


class _Layer:
    def __init__(self, type_name, updater, feature_maps, w, h, params=(), pool=None, input_count=1, with_backward=True):
        pr = (ct.c_float * 4)(*(list(params) + [0.0] * (4 - len(params))))
        pl = (ct.c_int * 7)(*(list(pool) if pool else [1, 1, 1, 1, 0, 0, 0]))
        self.h = lib.nnfh_create(type_name.encode(), int(updater), pr, pl, feature_maps, w, h, input_count, int(with_backward))
        if not self.h:
            raise HostLayerError(lib.nnfh_last_error().decode())

    def __del__(self):
        if getattr(self, "h", None):
            lib.nnfh_destroy(self.h)
            self.h = None


class Tester(_Layer):
    def __init__(self, type_name, feature_maps, w, h, **kw):
        super().__init__(type_name, False, feature_maps, w, h, **kw)

    def enqueue_forward_propagation(self, output_buffer, data, input_buffers, entry_count):
        d, nd = _arr(data)
        i, ni = _arr(input_buffers)
        _check(lib.nnfh_tester_forward(self.h, _stream(), _ptr(output_buffer), d, nd, i, ni, entry_count))

    def get_input_index_layer_can_write(self):
        return lib.nnfh_tester_can_write(self.h)


class Updater(_Layer):
    def __init__(self, type_name, feature_maps, w, h, **kw):
        super().__init__(type_name, True, feature_maps, w, h, **kw)

    def get_temporary_working_fixed_buffer_size(self, action):
        return int(lib.nnfh_updater_query(self.h, 0, action))

    def get_temporary_fixed_buffer_size(self):
        return int(lib.nnfh_updater_query(self.h, 1, 0))

    def get_temporary_per_entry_buffer_size(self):
        return int(lib.nnfh_updater_query(self.h, 2, 0))

    def get_input_index_layer_can_write(self, action):
        return int(lib.nnfh_updater_query(self.h, 3, action))

    def is_backward_data_dependent_on_input_buffer(self):
        return bool(lib.nnfh_updater_query(self.h, 4, BACKWARD_DATA))

    def is_backward_data_dependent_on_output_buffer(self):
        return bool(lib.nnfh_updater_query(self.h, 5, BACKWARD_DATA))

    def enqueue_forward_propagation(self, output_buffer, data, input_buffers, entry_count, temporary_working_fixed_buffer=None,
                                    temporary_fixed_buffer=None, temporary_per_entry_buffer=None):
        d, nd = _arr(data)
        i, ni = _arr(input_buffers)
        wf = temporary_working_fixed_buffer
        _check(lib.nnfh_updater_forward(self.h, _stream(), _ptr(output_buffer), d, nd, i, ni, _ptr(wf), wf.numel() * wf.element_size() if wf is not None else 0,
                                        _ptr(temporary_fixed_buffer), _ptr(temporary_per_entry_buffer), entry_count))

    def enqueue_backward_data_propagation(self, input_errors_buffer, output_errors_buffer, data, input_neurons_buffer, output_neurons_buffer, entry_count,
                                          temporary_fixed_buffer=None, temporary_per_entry_buffer=None, add_update_to_destination=False):
        d, nd = _arr(data)
        _check(lib.nnfh_updater_backward_data(self.h, _stream(), _ptr(input_errors_buffer), _ptr(output_errors_buffer), d, nd, _ptr(input_neurons_buffer),
                                              _ptr(output_neurons_buffer), _ptr(temporary_fixed_buffer), _ptr(temporary_per_entry_buffer),
                                              int(add_update_to_destination), entry_count))

    def enqueue_backward_data_propagation_inputs(self, input_errors_buffer, output_errors_buffer, input_neurons_buffers, output_neurons_buffer, entry_count,
                                                 add_update_to_destination=False):
        """Backward for layers with several inputs (the loss layers): all input neuron buffers are passed."""
        i, ni = _arr(input_neurons_buffers)
        _check(lib.nnfh_updater_backward_data_inputs(self.h, _stream(), _ptr(input_errors_buffer), _ptr(output_errors_buffer), i, ni,
                                                     _ptr(output_neurons_buffer), int(add_update_to_destination), entry_count))

    def enqueue_backward_weights_propagation(self, gradient, input_neurons_buffer, output_errors_buffer, entry_count, temporary_working_fixed_buffer=None):
        g, ng = _arr(gradient)
        wf = temporary_working_fixed_buffer
        _check(lib.nnfh_updater_backward_weights(self.h, _stream(), g, ng, _ptr(input_neurons_buffer), _ptr(output_errors_buffer), _ptr(wf),
                                                 wf.numel() * wf.element_size() if wf is not None else 0, entry_count))

    def enqueue_backward_data_and_weights_propagation(self, input_errors_buffer, output_errors_buffer, gradient, data, input_neurons_buffer, entry_count,
                                                      temporary_working_fixed_buffer=None, temporary_fixed_buffer=None, add_update_to_destination=False):
        g, ng = _arr(gradient)
        d, nd = _arr(data)
        wf = temporary_working_fixed_buffer
        _check(lib.nnfh_updater_backward_data_and_weights(self.h, _stream(), _ptr(input_errors_buffer), _ptr(output_errors_buffer), g, ng, d, nd,
                                                          _ptr(input_neurons_buffer), _ptr(wf), wf.numel() * wf.element_size() if wf is not None else 0,
                                                          _ptr(temporary_fixed_buffer), int(add_update_to_destination), entry_count))


def plan_fusion(spec, training=False):
    """Runs the schema peephole (csrc/host/nnf_fusion.h) on a textual schema: one layer per line,
    "name type inputs [needed] [key=value ...]" (inputs: comma-separated layer names or "-"). Returns one dict per
    fused group: kind, entry_point, members, residual, elided."""
    buf = ct.create_string_buffer(1 << 16)
    if lib.nnfh_plan_fusion(spec.encode(), int(training), buf, len(buf)) != 0:
        raise HostLayerError(lib.nnfh_fusion_last_error().decode())
    groups = []
    for line in buf.value.decode().splitlines():
        kind, entry, members, residual, elided = line.split(" ")
        val = lambda t: [] if t.split("=", 1)[1] == "-" else t.split("=", 1)[1].split(",")
        groups.append({"kind": kind, "entry_point": None if entry == "-" else entry, "members": val(members),
                       "residual": (val(residual) or [None])[0], "elided": val(elided)})
    return groups


NO_MOMENTUM, VANILLA_MOMENTUM, NESTEROV_MOMENTUM, ADAM_MOMENTUM = range(4)


def enqueue_apply_gradient(data, gradient, learning_rates, prev_upd=None, prev_upd2=None, update_accum_buffers=None, weight_decay_part_ids=(),
                           gradient_normalizer=1.0, weight_decay=0.0, momentum_type=NO_MOMENTUM, momentum_val=0.0, momentum_val2=0.0, iteration_id=1):
    """One layer's weight chunks through nnf_b200::enqueue_apply_gradient (the mirror of
    backward_propagation_cuda::enqueue_apply_gradient): lists of CUDA tensors, one entry per chunk."""
    n = len(data)
    arr = lambda ts: _arr(ts)[0] if ts is not None else None
    lrs = (ct.c_float * max(n, 1))(*learning_rates)
    counts = (ct.c_longlong * max(n, 1))(*[t.numel() for t in data])
    wd = (ct.c_int * max(len(weight_decay_part_ids), 1))(*weight_decay_part_ids)
    _check(lib.nnfh_apply_gradient(_stream(), n, arr(data), arr(gradient), arr(prev_upd), arr(prev_upd2), arr(update_accum_buffers), lrs, counts, wd,
                                   len(weight_decay_part_ids), ct.c_float(gradient_normalizer), ct.c_float(weight_decay), momentum_type,
                                   ct.c_float(momentum_val), ct.c_float(momentum_val2), iteration_id))
