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

_PP = ct.POINTER(_P)
lib.nnfh_forward.argtypes = [_P, _P, _PP, ct.c_int, _PP, ct.c_int, _PP, ct.c_int, _P, ct.c_size_t, _P, _P, ct.c_uint]
lib.nnfh_backward_data.argtypes = [_P, _P, ct.c_uint, _P, _P, _PP, ct.c_int, _PP, ct.c_int, _P, _P, _P, ct.c_int, ct.c_uint]
lib.nnfh_backward_weights.argtypes = [_P, _P, _PP, ct.c_int, _PP, ct.c_int, _P, _P, ct.c_size_t, ct.c_uint]
lib.nnfh_backward_data_and_weights.argtypes = [_P, _P, _PP, ct.c_int, _P, _PP, ct.c_int, _PP, ct.c_int, _PP, ct.c_int, _P, _P, ct.c_size_t, _P, ct.c_int, ct.c_uint]
lib.nnfh_query.restype = ct.c_longlong
lib.nnfh_query.argtypes = [_P, ct.c_int, ct.c_int, ct.c_int, ct.c_uint, ct.c_uint]
lib.nnfh_get_data.argtypes = [_P, ct.POINTER(ct.POINTER(ct.c_float)), ct.POINTER(ct.c_longlong), ct.c_int, _PP]
lib.nnfh_get_data_from_device.argtypes = [_P, ct.POINTER(ct.POINTER(ct.c_float)), ct.POINTER(ct.c_longlong), ct.c_int]
lib.nnfh_running_configuration.argtypes = [ct.POINTER(ct.c_longlong)]
lib.nnfh_net_last_error.restype = ct.c_char_p
lib.nnfh_peer_directory_create.restype = _P
lib.nnfh_peer_directory_destroy.argtypes = [_P]
lib.nnfh_peer_directory_publish.argtypes = [_P, ct.c_char_p, ct.c_int, _P]
lib.nnfh_net_create.restype = _P
lib.nnfh_net_create.argtypes = [ct.c_char_p, ct.c_int, ct.c_char_p, ct.c_int, ct.c_int, _P]
lib.nnfh_net_destroy.argtypes = [_P]
lib.nnfh_net_object_count.argtypes = [_P]
lib.nnfh_net_object.restype = _P
lib.nnfh_net_object.argtypes = [_P, ct.c_int]
lib.nnfh_net_describe.argtypes = [_P, ct.c_char_p, ct.c_size_t]
lib.nnfh_enable_peer_access.argtypes = [ct.c_int, ct.c_int]
lib.nnfh_net_buffer_plan.argtypes = [_P, ct.c_char_p, ct.c_size_t]

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
        if getattr(self, "h", None) and lib is not None:
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


def _bytes(t):
    return t.numel() * t.element_size() if t is not None else 0


class LayerObject:
    """One layer object (tester or updater) behind its general members: lists of inputs, outputs and weight
    chunks, and every buffer-plan query of the interface. The handle belongs to a `Net`."""

    def __init__(self, handle, description):
        self.h = handle
        self.__dict__.update(description)

    def _query(self, what, action=FORWARD, backprop_index=-1, a=0, b=0):
        r = int(lib.nnfh_query(self.h, what, action, backprop_index, a, b))
        if r == -2:
            raise HostLayerError(lib.nnfh_last_error().decode())
        return r

    def get_temporary_working_fixed_buffer_size(self, action=FORWARD):
        return self._query(0, action, 0 if action == BACKWARD_DATA else -1)

    def get_temporary_fixed_buffer_size(self):
        return self._query(1)

    def get_temporary_per_entry_buffer_size(self):
        return self._query(2)

    def get_input_index_layer_can_write(self, action=FORWARD):
        return self._query(3, action, 0 if action == BACKWARD_DATA else -1)

    def is_backward_data_dependent_on_input_buffer(self, action_input_index=0, data_input_index=0):
        return bool(self._query(4, BACKWARD_DATA, action_input_index, action_input_index, data_input_index))

    def is_backward_data_dependent_on_output_buffer(self, action_input_index=0):
        return bool(self._query(5, BACKWARD_DATA, action_input_index, action_input_index))

    def is_backward_data_dependent_on_temporary_fixed_buffer(self, action_input_index=0):
        return bool(self._query(6, BACKWARD_DATA, action_input_index, action_input_index))

    def is_backward_data_dependent_on_temporary_per_entry_buffer(self, action_input_index=0):
        return bool(self._query(7, BACKWARD_DATA, action_input_index, action_input_index))

    def is_backward_data_and_weights_dependent_on_input_buffer(self, data_input_index=0):
        return bool(self._query(8, BACKWARD_DATA_AND_WEIGHTS, -1, 0, data_input_index))

    def is_backward_data_and_weights_dependent_on_output_buffer(self):
        return bool(self._query(9, BACKWARD_DATA_AND_WEIGHTS))

    def is_backward_data_and_weights_dependent_on_temporary_fixed_buffer(self):
        return bool(self._query(10, BACKWARD_DATA_AND_WEIGHTS))

    def is_backward_data_and_weights_dependent_on_temporary_per_entry_buffer(self):
        return bool(self._query(11, BACKWARD_DATA_AND_WEIGHTS))

    def is_backward_weights_dependent_on_input_buffer(self, data_input_index=0):
        return bool(self._query(12, BACKWARD_WEIGHTS, -1, 0, data_input_index))

    def is_backward_weights_dependent_on_temporary_fixed_buffer(self):
        return bool(self._query(13, BACKWARD_WEIGHTS))

    def is_backward_weights_dependent_on_temporary_per_entry_buffer(self):
        return bool(self._query(14, BACKWARD_WEIGHTS))

    def get_output_count(self):
        return self._query(15)

    def get_temporary_working_per_entry_buffer_size(self, action=FORWARD):
        return self._query(16, action, 0 if action == BACKWARD_DATA else -1)

    def get_persistent_working_data_count(self):
        return self._query(17)

    def get_linear_addressing_through_texture_per_entry(self):
        return [None] * self._query(18)

    def enqueue_forward_propagation(self, output_buffers, data, input_buffers, entry_count, temporary_working_fixed_buffer=None,
                                    temporary_fixed_buffer=None, temporary_per_entry_buffer=None):
        o, no = _arr(output_buffers)
        d, nd = _arr(data)
        i, ni = _arr(input_buffers)
        wf = temporary_working_fixed_buffer
        _check(lib.nnfh_forward(self.h, _stream(), o, no, d, nd, i, ni, _ptr(wf), _bytes(wf), _ptr(temporary_fixed_buffer), _ptr(temporary_per_entry_buffer),
                                entry_count))

    def enqueue_backward_data_propagation(self, input_index, input_errors_buffer, output_errors_buffer, data, input_neurons_buffers, output_neurons_buffer,
                                          entry_count, temporary_fixed_buffer=None, temporary_per_entry_buffer=None, add_update_to_destination=False):
        d, nd = _arr(data)
        i, ni = _arr(input_neurons_buffers)
        _check(lib.nnfh_backward_data(self.h, _stream(), input_index, _ptr(input_errors_buffer), _ptr(output_errors_buffer), d, nd, i, ni,
                                      _ptr(output_neurons_buffer), _ptr(temporary_fixed_buffer), _ptr(temporary_per_entry_buffer),
                                      int(add_update_to_destination), entry_count))

    def enqueue_backward_weights_propagation(self, gradient, input_neurons_buffers, output_errors_buffer, entry_count, temporary_working_fixed_buffer=None):
        g, ng = _arr(gradient)
        i, ni = _arr(input_neurons_buffers)
        wf = temporary_working_fixed_buffer
        _check(lib.nnfh_backward_weights(self.h, _stream(), g, ng, i, ni, _ptr(output_errors_buffer), _ptr(wf), _bytes(wf), entry_count))

    def enqueue_backward_data_and_weights_propagation(self, input_errors_buffers, output_errors_buffer, gradient, data, input_neurons_buffers,
                                                      output_neurons_buffer, entry_count, temporary_working_fixed_buffer=None, temporary_fixed_buffer=None,
                                                      add_update_to_destination=False):
        e, ne = _arr(input_errors_buffers)
        g, ng = _arr(gradient)
        d, nd = _arr(data)
        i, ni = _arr(input_neurons_buffers)
        wf = temporary_working_fixed_buffer
        _check(lib.nnfh_backward_data_and_weights(self.h, _stream(), e, ne, _ptr(output_errors_buffer), g, ng, d, nd, i, ni, _ptr(output_neurons_buffer),
                                                  _ptr(wf), _bytes(wf), _ptr(temporary_fixed_buffer), int(add_update_to_destination), entry_count))

    def get_data(self, host_parts):
        """Uploads the weight chunks (lists / numpy arrays of float32) through the object's get_data; returns CUDA tensors viewing
        the device buffers, which the object keeps alive."""
        import numpy as np
        parts = [np.ascontiguousarray(p, dtype=np.float32) for p in host_parts]
        n = len(parts)
        pp = (ct.POINTER(ct.c_float) * max(n, 1))(*[p.ctypes.data_as(ct.POINTER(ct.c_float)) for p in parts])
        counts = (ct.c_longlong * max(n, 1))(*[p.size for p in parts])
        outp = (_P * max(n, 1))()
        _check(lib.nnfh_get_data(self.h, pp, counts, n, outp))
        self._uploaded_sizes = [p.size for p in parts]
        return [_view(outp[k], parts[k].size) for k in range(n)]

    def get_data_from_device(self):
        import numpy as np
        parts = [np.empty(sz, dtype=np.float32) for sz in self._uploaded_sizes]
        n = len(parts)
        pp = (ct.POINTER(ct.c_float) * max(n, 1))(*[p.ctypes.data_as(ct.POINTER(ct.c_float)) for p in parts])
        counts = (ct.c_longlong * max(n, 1))(*[p.size for p in parts])
        _check(lib.nnfh_get_data_from_device(self.h, pp, counts, n))
        return parts


def _view(address, elem_count):
    """A float32 CUDA tensor over device memory the library owns."""
    class _Mem:
        pass
    m = _Mem()
    m.__cuda_array_interface__ = {"shape": (elem_count,), "typestr": "<f4", "data": (int(address), False), "version": 2}
    return torch.as_tensor(m, device="cuda")


class PeerDirectory:
    """Where the layer objects of the devices that share a batch publish their mailboxes (peer_directory)."""

    def __init__(self):
        self.h = lib.nnfh_peer_directory_create()

    def publish(self, key, device_pos, address):
        """One process per GPU: the address of position `device_pos`'s buffer as THIS process sees it (its own buffer under its
        own position), published before the layer objects are created."""
        lib.nnfh_peer_directory_publish(self.h, key.encode(), device_pos, ct.c_void_p(int(address)))

    def __del__(self):
        if getattr(self, "h", None) and lib is not None:
            lib.nnfh_peer_directory_destroy(self.h)
            self.h = None


def enable_peer_access(device, peer):
    if lib.nnfh_enable_peer_access(device, peer) != 0:
        raise HostLayerError("device %d cannot address the memory of device %d" % (device, peer))


def running_configuration():
    """The running_configuration_b200 of the current device as a dict."""
    v = (ct.c_longlong * 11)()
    _check(lib.nnfh_running_configuration(v))
    names = ["device_id", "compute_capability_major", "compute_capability_minor", "multiprocessor_count", "max_threads_per_multiprocessor", "smem_per_block",
             "smem_per_multiprocessor", "l2_cache_size", "max_registers_per_multiprocessor", "device_pos", "device_count"]
    return dict(zip(names, [int(x) for x in v]))


class Net:
    """The layer objects of a textual schema: parsed, planned (plan_fusion) and created through the C++ factory
    (create_testers / create_updaters), on the current device. `objects` lists them in execution order; each has
    node, type, role (head / follower / single), group, kind, entry, shape (feature maps, w, h) and - for the objects
    that run something - inputs (layer names), data (layers whose weight chunks it takes), outputs (layers whose
    output buffers it writes) and elided (layers whose outputs never need a buffer). `data_shapes`: {data layer
    name: (feature_maps, w, h)}."""

    def __init__(self, spec, data_shapes, training=False, device_pos=0, device_count=1, peers=None):
        shapes = "\n".join("%s %d %d %d" % ((k,) + tuple(v)) for k, v in data_shapes.items())
        self.peers = peers
        self.h = lib.nnfh_net_create(spec.encode(), int(training), shapes.encode(), device_pos, device_count, peers.h if peers else None)
        if not self.h:
            raise HostLayerError(lib.nnfh_net_last_error().decode())
        buf = ct.create_string_buffer(1 << 16)
        if lib.nnfh_net_describe(self.h, buf, len(buf)) != 0:
            raise HostLayerError(lib.nnfh_net_last_error().decode())
        self.objects = []
        for k, line in enumerate(buf.value.decode().splitlines()):
            d = dict(tok.split("=", 1) for tok in line.split(" "))
            lst = lambda t: [] if t == "-" else t.split(",")
            desc = {"node": d["node"], "type": d["type"], "role": d["role"], "group": int(d["group"]), "kind": d["kind"],
                    "entry": None if d["entry"] == "-" else d["entry"], "shape": tuple(int(v) for v in d["shape"].split(",")),
                    "inputs": lst(d["inputs"]), "data": lst(d["data"]), "outputs": lst(d["outputs"]), "elided": lst(d["elided"])}
            self.objects.append(LayerObject(lib.nnfh_net_object(self.h, k), desc))

    def buffer_plan(self):
        """Which layer outputs of this inference net share storage (plan_forward_buffers): {"buffers": count, "total_bytes_per_entry": n,
        "nodes": {layer: {"buffer": index or None, "in_place": input index or None, "bytes_per_entry": n}}}."""
        buf = ct.create_string_buffer(1 << 16)
        if lib.nnfh_net_buffer_plan(self.h, buf, len(buf)) != 0:
            raise HostLayerError(lib.nnfh_net_last_error().decode())
        lines = buf.value.decode().splitlines()
        head = dict(tok.split("=") for tok in lines[0].split(" "))
        nodes = {}
        for line in lines[1:]:
            d = dict(tok.split("=", 1) for tok in line.split(" "))
            nodes[d["node"]] = {"buffer": None if d["buffer"] == "-" else int(d["buffer"]), "in_place": None if d["in_place"] == "-" else int(d["in_place"]),
                                "bytes_per_entry": int(d["bytes_per_entry"])}
        return {"buffers": int(head["buffers"]), "total_bytes_per_entry": int(head["total_bytes_per_entry"]), "nodes": nodes}

    def __del__(self):
        if getattr(self, "h", None) and lib is not None:
            self.objects = []
            lib.nnfh_net_destroy(self.h)
            self.h = None


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
