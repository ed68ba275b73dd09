"""Export of a set-up model to an ONNX ``ModelProto`` (opset 11), the job of the reference's
``export_onnx`` callback (src/callbacks/export_onnx.cpp, include/lbann/layers/*: every layer
there implements ``fill_onnx_node``).  Tensors carry a symbolic mini-batch dimension first;
weights become initialisers with their current values.  Layers without an ONNX counterpart are
written as nodes of the custom domain ``lbann`` whose ``op_type`` is the layer type, so the
graph stays complete and loadable.
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np

from . import onnx_proto as op

OPSET = 11
_ACT_SUFFIX = {1: ("Relu", {}), 2: ("LeakyRelu", None)}        # fused epilogue activations (native.ACT_*)


def _attr(node, name, value):
    a = node.attribute.add()
    a.name = name
    if isinstance(value, float):
        a.f, a.type = value, op.ATTR_FLOAT
    elif isinstance(value, (bool, int, np.integer)):
        a.i, a.type = int(value), op.ATTR_INT
    elif isinstance(value, str):
        a.s, a.type = value.encode(), op.ATTR_STRING
    elif isinstance(value, (list, tuple)) and value and isinstance(value[0], float):
        a.floats.extend(float(v) for v in value)
        a.type = op.ATTR_FLOATS
    else:
        a.ints.extend(int(v) for v in value)
        a.type = op.ATTR_INTS
    return a


def _tensor(name, array, dtype=op.FLOAT):
    t = op.TensorProto()
    t.name = name
    a = np.ascontiguousarray(array, dtype=np.int64 if dtype == op.INT64 else np.float32)
    t.dims.extend(a.shape)
    t.data_type = dtype
    t.raw_data = a.tobytes()
    return t


def _value_info(name, dims):
    v = op.ValueInfoProto()
    v.name = name
    v.type.tensor_type.elem_type = op.FLOAT
    v.type.tensor_type.shape.dim.add().dim_param = "batch"
    for d in dims:
        v.type.tensor_type.shape.dim.add().dim_value = int(d)
    return v


class _Builder:
    def __init__(self, model):
        self.model = model
        self.graph = op.GraphProto()
        self.graph.name = model.name or "lbann_model"
        self.inits: Dict[str, bool] = {}
        self.custom = False

    def out_name(self, layer, k=0):
        return f"{layer.name}_out{k}"

    def inputs_of(self, layer) -> List[str]:
        names = []
        for pn in layer.parent_names:
            p = self.model.layers_by_name[pn]
            k = 0
            if len(p.out_dims) > 1 and layer.name in p.child_names:     # slice / split: one output per child
                k = p.child_names.index(layer.name)
            names.append(self.out_name(p, k))
        return names

    def weight(self, w) -> str:
        if w.name not in self.inits:
            self.graph.initializer.append(_tensor(w.name, w.values.detach().float().cpu().numpy().reshape(w.shape or (1,))))
            self.inits[w.name] = True
        return w.name

    def const(self, name, array, dtype=op.FLOAT) -> str:
        self.graph.initializer.append(_tensor(name, array, dtype))
        return name

    def node(self, op_type, inputs, outputs, name, domain="", **attrs):
        n = self.graph.node.add()
        n.op_type, n.name = op_type, name
        n.input.extend(inputs)
        n.output.extend(outputs)
        if domain:
            n.domain = domain
            self.custom = True
        for k, v in attrs.items():
            _attr(n, k, v)
        return n

    def with_activation(self, layer, produce):
        """Run ``produce(output_name)``; a ReLU / leaky ReLU folded into the layer's kernel
        becomes its own node again."""
        act = getattr(layer, "fused_act", (0, 0.0))
        final = self.out_name(layer)
        if act[0] in _ACT_SUFFIX:
            mid = final + "_linear"
            produce(mid)
            kind, _ = _ACT_SUFFIX[act[0]]
            extra = {"alpha": float(act[1])} if kind == "LeakyRelu" else {}
            self.node(kind, [mid], [final], layer.name + "_activation", **extra)
        else:
            produce(final)


def _pads(p):
    return list(p) + list(p)


def _emit(b: _Builder, l):
    t, ins, out = l.type, b.inputs_of(l), b.out_name(l)
    if t == "input":
        b.graph.input.append(_value_info(out, l.out_dims[0]))
        return
    if getattr(l, "fused_into_parent", False) or getattr(l, "input_is_pooled", None) is True:
        b.node("Identity", ins[:1], [out], l.name)
        return
    if t == "fully_connected":
        x = ins[0]
        if len(l.in_dims[0]) > 1:
            b.node("Flatten", [x], [out + "_flat"], l.name + "_flatten", axis=1)
            x = out + "_flat"
        w = b.weight(l.w)                      # stored [out, in]: Gemm with transB (or as it is when transposed)
        args = [x, w] + ([b.weight(l.b)] if l.b is not None else [])
        b.with_activation(l, lambda o: b.node("Gemm", args, [o], l.name, transB=0 if l.transpose else 1))
    elif t == "convolution":
        args = [ins[0], b.weight(l.w)] + ([b.weight(l.b)] if l.b is not None else [])
        b.with_activation(l, lambda o: b.node("Conv", args, [o], l.name, kernel_shape=list(l.ksize),
                                              strides=list(l.stride), pads=_pads(l.pad),
                                              dilations=list(l.dil), group=l.groups))
    elif t == "deconvolution":
        args = [ins[0], b.weight(l.w)] + ([b.weight(l.b)] if l.b is not None else [])
        b.node("ConvTranspose", args, [out], l.name, kernel_shape=list(l.ksize), strides=list(l.stride),
               pads=_pads(l.pad), dilations=list(l.dil), group=l.groups, output_padding=list(l.out_pad))
    elif t == "pooling":
        kind = "MaxPool" if l.mode == "max" else "AveragePool"
        extra = {} if kind == "MaxPool" else {"count_include_pad": 1 if l.mode == "average" else 0}
        b.node(kind, ins, [out], l.name, kernel_shape=list(l.k), strides=list(l.stride), pads=_pads(l.pad), **extra)
    elif t == "batch_normalization":
        args = [ins[0], b.weight(l.scale), b.weight(l.bias), b.weight(l.run_mean), b.weight(l.run_var)]
        b.with_activation(l, lambda o: b.node("BatchNormalization", args, [o], l.name, epsilon=float(l.eps),
                                              momentum=float(l.decay)))
    elif t in ("relu", "sigmoid", "tanh", "softplus", "softsign", "identity", "exp", "log", "sqrt", "abs", "neg"):
        names = {"relu": "Relu", "sigmoid": "Sigmoid", "tanh": "Tanh", "softplus": "Softplus",
                 "softsign": "Softsign", "identity": "Identity", "exp": "Exp", "log": "Log", "sqrt": "Sqrt",
                 "abs": "Abs", "neg": "Neg"}
        b.node(names[t], ins, [out], l.name)
    elif t == "leaky_relu":
        b.node("LeakyRelu", ins, [out], l.name, alpha=float(l.p0()))
    elif t == "elu":
        b.node("Elu", ins, [out], l.name, alpha=float(l.p0() or 1.0))
    elif t in ("softmax", "log_softmax"):
        # over the whole sample (opset 11 flattens from `axis` on) or over channels
        mode = getattr(l.params, "softmax_mode", "") or "instance"
        b.node("Softmax" if t == "softmax" else "LogSoftmax", ins, [out], l.name, axis=1)
        if mode == "channel" and len(l.out_dims[0]) > 1:
            b.graph.node[-1].doc_string = "channel-wise: applies along axis 1 for every position"
    elif t in ("sum", "add"):
        b.with_activation(l, lambda o: b.node("Sum", ins, [o], l.name))
    elif t in ("multiply", "hadamard"):
        b.node("Mul", ins, [out], l.name)
    elif t == "concatenation":
        b.node("Concat", ins, [out], l.name, axis=int(l.axis) + 1)
    elif t == "slice":
        pts = [int(v) for v in l.slice_points] if hasattr(l, "slice_points") else []
        outs = [b.out_name(l, k) for k in range(len(l.out_dims))]
        b.node("Split", ins, outs, l.name, axis=int(getattr(l, "axis", 0)) + 1,
               split=[pts[i + 1] - pts[i] for i in range(len(pts) - 1)] or [int(d[0]) for d in l.out_dims])
    elif t == "reshape":
        shape = b.const(l.name + "_shape", np.asarray([0] + [int(d) for d in l.out_dims[0]]), op.INT64)
        b.node("Reshape", [ins[0], shape], [out], l.name)
    elif t == "dropout":
        b.node("Dropout", ins, [out], l.name, ratio=1.0 - (float(l.params.keep_prob) or 0.5))
    elif t == "matmul":
        b.node("MatMul", ins, [out], l.name)
    elif t == "embedding":
        idx = out + "_index"
        b.node("Cast", ins, [idx], l.name + "_cast", to=op.INT64)
        b.node("Gather", [b.weight(l.weights[0]), idx], [out], l.name, axis=0)
    else:
        # no ONNX operator: keep the node, in this package's own domain, with its weights
        args = ins + [b.weight(w) for w in l.weights if w is not None]
        outs = [b.out_name(l, k) for k in range(max(1, len(l.out_dims)))]
        b.node(t, args, outs, l.name, domain="lbann")


def export_model(model):
    """``model``: a set-up ``ExecModel``.  Returns an ``onnx.ModelProto`` message (this
    package's own class with ONNX's wire format; ``SerializeToString()`` gives a ``.onnx`` file)."""
    b = _Builder(model)
    for l in model.layers:
        _emit(b, l)
    for l in model.layers:
        if not l.child_names and l.type != "input":
            for k, d in enumerate(l.out_dims or [()]):
                b.graph.output.append(_value_info(b.out_name(l, k), d))
    m = op.ModelProto()
    m.ir_version = 6
    m.producer_name, m.producer_version = "lbann_b200", "1"
    m.graph.CopyFrom(b.graph)
    o = m.opset_import.add()
    o.domain, o.version = "", OPSET
    if b.custom:
        o = m.opset_import.add()
        o.domain, o.version = "lbann", 1
    return m
