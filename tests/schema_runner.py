"""A textual layer schema run two ways, for the tests of the fused layer objects:

`OracleRun` executes it layer by layer on the CPU checker, the way the reference schedules unfused layers
(one action and one output buffer per layer); `ObjectRun` is a small scheduler over the objects the C++
factory made for the planned groups (nnforge_b200.host.Net): it gives every object the buffers the object's
description asks for, enqueues every object - followers too, as a per-layer scheduler would - and keeps
the buffers it created by layer name. Both return dicts keyed by layer name.
"""
import numpy as np
import torch


def parse(spec):
    """[(name, type, inputs, params)] from the schema text ("name type inputs [key=value ...]")."""
    nodes = []
    for line in spec.strip().splitlines():
        tok = line.split()
        params = {}
        for t in tok[3:]:
            if "=" in t:
                k, v = t.split("=", 1)
                params[k] = v
            else:
                params[t] = True
        nodes.append((tok[0], tok[1], [] if tok[2] == "-" else tok[2].split(","), params))
    return nodes


def _pair(v, default):
    return tuple(int(a) for a in v.split("x")) if v is not None else default


class OracleRun:
    def __init__(self, oracle, spec, training):
        self.o = oracle
        self.nodes = parse(spec)
        self.training = training

    def forward(self, data, weights):
        """data: {data layer: array}; weights: {layer: [chunks]}. Returns {layer: output}; keeps what backward needs."""
        o, v = self.o, dict(data)
        self.saved, self.argmax = {}, {}
        for name, typ, ins, p in self.nodes:
            x = v[ins[0]]
            w = weights.get(name, [])
            if typ == "BatchNorm":
                if self.training:
                    v[name], self.saved[name] = o.bn_train_fwd(x, w[0], w[1], float(p.get("eps", 2e-5)))
                else:
                    v[name] = o.bn_infer(x, *w)
            elif typ == "ReLU":
                v[name] = o.relu_fwd(x, float(p.get("slope", 0.0)))
            elif typ == "PReLU":
                v[name] = o.prelu_fwd(x, w[0])
            elif typ == "ELU":
                v[name] = o.elu_fwd(x)
            elif typ == "TanH":
                v[name] = o.tanh_fwd(x, float(p.get("scale", 1.0)), float(p.get("steepness", 1.0)))
            elif typ == "Sigmoid":
                v[name] = o.sigmoid_fwd(x)
            elif typ == "Add":
                v[name] = o.add_fwd([v[i] for i in ins], float(p.get("alpha", 1.0)))
            elif typ == "Softmax":
                v[name] = o.softmax_fwd(x)
            elif typ == "NegativeLogLikelihood":
                v[name] = o.nll_fwd(x, v[ins[1]], v[ins[2]] if len(ins) > 2 else None, float(p.get("scale", 1.0)))
            elif typ == "MaxSubsampling":
                win = _pair(p.get("win"), None)
                v[name], self.argmax[name] = o.maxpool_fwd(x, win, _pair(p.get("stride"), win), tuple(bool(a) for a in _pair(p.get("roundup"), (0, 0))))
            elif typ == "AverageSubsampling":
                v[name] = o.avgpool_fwd(x, _pair(p.get("win"), None), mult=float(p["alpha"]) if "alpha" in p else None)
            else:
                raise ValueError(typ)
        self.values = v
        return v

    def backward(self, out_errors, weights):
        """out_errors: {layer: gradient of its output} for the network outputs. Returns ({layer or data layer: gradient of its
        output}, {layer: [weight gradients]})."""
        o, v = self.o, self.values
        err = {k: a.copy() for k, a in out_errors.items()}
        grads = {}

        def give(name, g):
            err[name] = g if name not in err else (err[name] + g).astype(np.float32)

        for name, typ, ins, p in reversed(self.nodes):
            w = weights.get(name, [])
            x = v[ins[0]]
            dy = err.get(name)
            if typ == "NegativeLogLikelihood":
                give(ins[0], o.nll_bwd(x, v[ins[1]], v[ins[2]] if len(ins) > 2 else None, float(p.get("scale", 1.0))))
                continue
            if dy is None:
                continue
            if typ == "BatchNorm":
                saved = self.saved[name]
                c = x.shape[1]
                db, dg = o.bn_train_bwd_sums(dy, x, saved)
                give(ins[0], o.bn_train_bwd_apply(dy, x, w[0], saved, db, dg, x.size // c))
                gm, gi = o.bn_train_running_grad(np.zeros(c, np.float32), np.zeros(c, np.float32), saved, w[2], w[3], x.shape[0])
                grads[name] = [dg, db, gm, gi]
            elif typ == "ReLU":
                give(ins[0], o.relu_bwd(dy, x, float(p.get("slope", 0.0))))
            elif typ == "PReLU":
                grads[name] = [o.prelu_bwd_weights(dy, x)]
                give(ins[0], o.prelu_bwd_data(dy, x, w[0]))
            elif typ == "ELU":
                give(ins[0], o.elu_bwd(dy, v[name]))
            elif typ == "TanH":
                give(ins[0], o.tanh_bwd(dy, v[name], float(p.get("scale", 1.0)), float(p.get("steepness", 1.0))))
            elif typ == "Sigmoid":
                give(ins[0], o.sigmoid_bwd(dy, v[name]))
            elif typ == "Add":
                for i in ins:
                    give(i, o.add_bwd(dy, float(p.get("alpha", 1.0))))
            elif typ == "Softmax":
                give(ins[0], o.softmax_bwd(dy, v[name]))
            elif typ == "MaxSubsampling":
                give(ins[0], o.maxpool_bwd(dy, self.argmax[name], x.shape))
            elif typ == "AverageSubsampling":
                give(ins[0], o.avgpool_bwd(dy, x.shape, _pair(p.get("win"), None), mult=float(p["alpha"]) if "alpha" in p else None))
            else:
                raise ValueError(typ)
        return err, grads


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


class ObjectRun:
    """The objects of host.Net driven like the reference's schedulers drive its layer objects."""

    def __init__(self, host, spec, data_shapes, training, entry_count):
        self.host = host
        self.nodes = {n[0]: n for n in parse(spec)}
        self.net = host.Net(spec, data_shapes, training=training)
        self.training = training
        self.n = entry_count
        self.shape = {o.node: o.shape for o in self.net.objects}
        self.launching = [o for o in self.net.objects if o.role != "follower"]

    def _alloc(self, name):
        fm, w, h = self.shape[name]
        return torch.empty((self.n, fm, h, w), device="cuda")

    def forward(self, data, weights, in_place=False):
        """Returns {layer: tensor} for every output that was materialised. in_place: let an object that allows it write over its input 0."""
        host, n = self.host, self.n
        self.buf = {k: _dev(a) for k, a in data.items()}
        self.w = {k: [_dev(a) for a in chunks] for k, chunks in weights.items()}
        self.keep = {}
        for o in self.net.objects:
            if o.role == "follower":
                # nothing to hand over that the head has not handled; the call must leave every buffer alone
                o.enqueue_forward_propagation([self.buf.get(o.node)], self.w.get(o.node, []), [self.buf.get(i) for i in self.nodes[o.node][2]], n)
                continue
            inputs = [self.buf[i] for i in o.inputs]
            chunks = [t for layer in o.data for t in self.w.get(layer, [])]
            if in_place and o.get_input_index_layer_can_write(host.FORWARD) == 0 and self.shape[o.outputs[0]] == tuple(inputs[0].shape[k] for k in (1, 3, 2)):
                outs = [inputs[0]] + [self._alloc(name) for name in o.outputs[1:]]
            else:
                outs = [self._alloc(name) for name in o.outputs]
            assert o.get_output_count() == len(outs)
            kw = {}
            if self.training:
                k = self.keep[o.node] = {}
                k["working"] = torch.empty(max(o.get_temporary_working_fixed_buffer_size(host.FORWARD), 16), dtype=torch.uint8, device="cuda")
                fixed, per_entry = o.get_temporary_fixed_buffer_size(), o.get_temporary_per_entry_buffer_size()
                k["fixed"] = torch.empty(fixed // 4, device="cuda") if fixed else None
                k["per_entry"] = torch.empty(per_entry * n // 4, dtype=torch.int32, device="cuda") if per_entry else None
                kw = {"temporary_working_fixed_buffer": k["working"], "temporary_fixed_buffer": k["fixed"], "temporary_per_entry_buffer": k["per_entry"]}
            else:
                kw = {"temporary_working_fixed_buffer": torch.empty(max(o.get_temporary_working_fixed_buffer_size(), 16), dtype=torch.uint8, device="cuda")}
            o.enqueue_forward_propagation(outs, chunks, inputs, n, **kw)
            for name, t in zip(o.outputs, outs):
                self.buf[name] = t
        return self.buf

    def backward(self, out_errors):
        """out_errors: {layer: array}. Returns ({layer: gradient of its output}, {layer: [weight gradient tensors]})."""
        host, n = self.host, self.n
        err = {k: _dev(a) for k, a in out_errors.items()}
        grads = {k: [torch.zeros_like(t) for t in chunks] for k, chunks in self.w.items()}
        for o in reversed(self.net.objects):
            name, typ, ins, _ = self.nodes[o.node]
            if o.role == "follower":
                if o.get_input_index_layer_can_write(host.BACKWARD_DATA) == 0 and name in err:
                    # in place: the gradient of its output is handed on as the gradient of its input
                    o.enqueue_backward_data_propagation(0, err[name], err[name], self.w.get(name, []), [None], None, n)
                    err[ins[0]] = err[name]
                    if typ == "PReLU":
                        o.enqueue_backward_weights_propagation(grads[name], [None], err[name], n)
                continue
            k = self.keep[o.node]
            chunks = [t for layer in o.data for t in self.w.get(layer, [])]
            gchunks = [t for layer in o.data for t in grads.get(layer, [])]
            inputs = [self.buf[i] if i in self.buf else None for i in o.inputs]
            last_out = o.outputs[-1]
            if o.kind == "bn_train_act" or typ == "BatchNorm":
                if last_out not in err:
                    continue
                act = host.BACKWARD_DATA_AND_WEIGHTS
                assert o.is_backward_data_and_weights_dependent_on_input_buffer(0) and not o.is_backward_data_and_weights_dependent_on_output_buffer()
                ws = torch.empty(o.get_temporary_working_fixed_buffer_size(act), dtype=torch.uint8, device="cuda")
                dx = torch.empty_like(inputs[0])
                o.enqueue_backward_data_and_weights_propagation([dx], err[last_out], gchunks, chunks, inputs, None, n,
                                                                temporary_working_fixed_buffer=ws, temporary_fixed_buffer=k["fixed"])
                err[o.inputs[0]] = dx
            elif o.kind == "softmax_nll" or typ == "NegativeLogLikelihood":
                needed = [inputs[j] if j == 0 and o.kind != "softmax_nll" or o.is_backward_data_dependent_on_input_buffer(0, j) else None for j in range(len(inputs))]
                dx = torch.empty_like(self.buf[o.inputs[0]])
                o.enqueue_backward_data_propagation(0, dx, None, chunks, needed, self.buf[o.outputs[0]] if o.is_backward_data_dependent_on_output_buffer(0) else None, n)
                err[o.inputs[0]] = dx
            else:
                if name not in err:
                    continue
                for j, inp in enumerate(o.inputs):
                    dx = torch.empty_like(self.buf[inp])
                    needed = [inputs[q] if o.is_backward_data_dependent_on_input_buffer(j, q) else None for q in range(len(inputs))]
                    o.enqueue_backward_data_propagation(j, dx, err[name], chunks, needed, self.buf[name] if o.is_backward_data_dependent_on_output_buffer(j) else None, n,
                                                        temporary_fixed_buffer=k["fixed"], temporary_per_entry_buffer=k["per_entry"])
                    err[inp] = dx if inp not in err else err[inp] + dx
                if typ == "PReLU":
                    ws = torch.empty(max(o.get_temporary_working_fixed_buffer_size(host.BACKWARD_WEIGHTS), 16), dtype=torch.uint8, device="cuda")
                    o.enqueue_backward_weights_propagation(gchunks, inputs, err[name], n, temporary_working_fixed_buffer=ws)
        return err, grads
