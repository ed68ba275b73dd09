"""User-facing model description objects (the ``lbann`` Python API).

Layers, weights, optimizers, initializers, callbacks, metrics, objective functions,
operators, training algorithms, ``Model`` and ``Trainer``.  These objects only describe
an experiment; ``export_proto()`` lowers them to ``lbann_data`` messages, which the
in-process executor (``lbann_b200.exec``) or a saved prototext consumes.  API parity
targets: python/lbann/core/{layer,weights,optimizer,callback,metric,objective_function,
model,trainer,operators,operator_layers,training_algorithm}.py of the reference.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..proto import lbann_pb2 as pb
from .generate import class_from_message, classes_from_oneof, make_iterable, set_message, str_list

# ------------------------------------------------------------------ enums
DataType = pb.DataType
DeviceAllocation = pb.DeviceAllocation
ShardingStrategy = pb.ShardingStrategy
ConvTensorOpsMode = getattr(pb, "ConvTensorOpsMode", None)
SubgraphCommunication = getattr(pb, "SubGraphCommunication", None)


# ------------------------------------------------------------------ layers
class Layer:
    """Node of the layer graph.  Positional arguments are parent layers."""

    global_count = 0

    def __init__(self, *args, parents=(), children=(), weights=(), name=None, device=None,
                 data_layout=None, datatype=None, hint_layer=None, grid_tag=None,
                 parallel_strategy=None):
        Layer.global_count += 1
        self.parents, self.children, self.weights = [], [], []
        self.name = name if name else f"layer{Layer.global_count}"
        self.device = device
        self.data_layout = data_layout
        self.datatype = datatype
        self.hint_layer = hint_layer
        self.grid_tag = {"value": grid_tag} if grid_tag is not None else {}
        self.parallel_strategy = dict(parallel_strategy) if parallel_strategy else {}
        for a in args:
            self.add_parent(a)
        self.add_parent(parents)
        self.add_child(children)
        self.add_weights(weights)

    def add_parent(self, parent):
        for p in make_iterable(parent):
            self.parents.append(p)
            p.children.append(self)

    def add_child(self, child):
        for c in make_iterable(child):
            self.children.append(c)
            c.parents.append(self)

    def add_weights(self, w):
        self.weights.extend(make_iterable(w))

    def __call__(self, parent):
        self.add_parent(parent)
        return self

    def export_proto(self):
        proto = pb.Layer()
        proto.name = self.name
        proto.parents[:] = [p.name for p in self.parents]
        proto.children[:] = [c.name for c in self.children]
        proto.weights[:] = [w.name for w in self.weights]
        if self.device:
            proto.device_allocation = self.device
        if self.data_layout:
            proto.data_layout = self.data_layout
        if self.datatype:
            proto.datatype = self.datatype
        if self.hint_layer is not None:
            proto.hint_layer = self.hint_layer.name
        if self.grid_tag:
            set_message(proto.grid_tag, **self.grid_tag)
            proto.grid_tag.SetInParent()
        if self.parallel_strategy:
            set_message(proto.parallel_strategy, **self.parallel_strategy)
            proto.parallel_strategy.SetInParent()
        return proto


_LAYER_BASE_KWARGS = ("parents", "children", "weights", "name", "device", "data_layout",
                      "datatype", "hint_layer", "grid_tag", "parallel_strategy")
_LAYER_SKIP = {"name", "parents", "children", "weights", "device_allocation", "datatype",
               "hint_layer", "data_layout", "parallel_strategy", "grid_tag", "freeze"}
layer_classes = classes_from_oneof(pb.Layer, Layer, _LAYER_BASE_KWARGS, skip=_LAYER_SKIP)
globals().update(layer_classes)
OperatorLayer = layer_classes["OperatorLayer"]


def traverse_layer_graph(layers):
    """Yield every layer connected to ``layers`` in a topological order (parents first)."""
    roots = list(make_iterable(layers))
    seen, order = set(), []
    # collect the connected component (both directions)
    stack, comp = list(roots), []
    while stack:
        l = stack.pop()
        if id(l) in seen:
            continue
        seen.add(id(l))
        comp.append(l)
        stack.extend(l.parents)
        stack.extend(l.children)
    # depth-first post-order on parents gives a topological order
    done = set()

    def visit(start):
        work = [(start, False)]
        while work:
            node, expanded = work.pop()
            if id(node) in done:
                continue
            if expanded:
                done.add(id(node))
                order.append(node)
            else:
                work.append((node, True))
                for p in reversed(node.parents):
                    if id(p) not in done:
                        work.append((p, False))

    for l in sorted(comp, key=lambda x: 0 if not x.parents else 1):
        visit(l)
    return order


# ------------------------------------------------------------------ weights
class Initializer:
    def export_proto(self):
        return pb.Initializer()


initializer_classes = classes_from_oneof(pb.Initializer, Initializer, ())
globals().update(initializer_classes)


class Optimizer:
    def export_proto(self):
        return pb.Optimizer()


optimizer_classes = classes_from_oneof(pb.Optimizer, Optimizer, ())
globals().update(optimizer_classes)


class Weights:
    """Trainable (or constant) parameter tensor shared by name between layers."""

    global_count = 0

    def __init__(self, initializer=None, optimizer=None, name=None, datatype=None,
                 sharded=None, sharding_strategy=None):
        Weights.global_count += 1
        self.name = name if name else f"weights{Weights.global_count}"
        self.initializer = initializer
        self.optimizer = optimizer
        self.datatype = datatype
        self.sharded = sharded
        self.sharding_strategy = sharding_strategy

    def export_proto(self):
        proto = pb.Weights()
        proto.name = self.name
        if self.initializer is not None:
            proto.initializer.CopyFrom(self.initializer.export_proto())
        if self.optimizer is not None:
            proto.optimizer.CopyFrom(self.optimizer.export_proto())
        if self.datatype is not None:
            proto.datatype = self.datatype
        if self.sharded:
            proto.sharded = True
        if self.sharding_strategy is not None:
            proto.sharding_strategy = self.sharding_strategy
        return proto


# ------------------------------------------------------------------ callbacks
class Callback:
    def export_proto(self):
        return pb.Callback()


callback_classes = classes_from_oneof(pb.Callback, Callback, ())
globals().update(callback_classes)


class ImageSelectionStrategy:
    def export_proto(self):
        return pb.Callback.CallbackSummarizeImages.SelectionStrategy()


globals().update(classes_from_oneof(pb.Callback.CallbackSummarizeImages.SelectionStrategy,
                                    ImageSelectionStrategy, ()))


# ------------------------------------------------------------------ metrics / objective
class Metric:
    """Scalar reported per mode, read from an evaluation of ``layer``."""

    def __init__(self, layer, name=None, unit=""):
        self.layer = layer
        self.name = name if name else layer.name
        self.unit = unit

    def export_proto(self):
        proto = pb.Metric()
        proto.layer_metric.layer = self.layer.name
        proto.layer_metric.name = self.name
        proto.layer_metric.unit = self.unit
        return proto


class ExecutableMetric:
    def __init__(self, name, filename, other_args=""):
        self.name, self.filename, self.other_args = name, filename, other_args

    def export_proto(self):
        proto = pb.Metric()
        proto.executable_metric.name = self.name
        proto.executable_metric.filename = self.filename
        proto.executable_metric.other_args = self.other_args
        return proto


class PythonMetric:
    def __init__(self, name, module, module_dir, function="evaluate"):
        self.name, self.module, self.module_dir, self.function = name, module, module_dir, function

    def export_proto(self):
        proto = pb.Metric()
        proto.python_metric.name = self.name
        proto.python_metric.module = self.module
        proto.python_metric.module_dir = self.module_dir
        proto.python_metric.function = self.function
        return proto


class ObjectiveFunctionTerm:
    pass


class LayerTerm(ObjectiveFunctionTerm):
    def __init__(self, layer, scale=1.0):
        self.layer, self.scale = layer, scale

    def export_proto(self):
        proto = pb.ObjectiveFunction.LayerTerm()
        proto.layer = self.layer.name
        proto.scale_factor = self.scale
        return proto


class L2WeightRegularization(ObjectiveFunctionTerm):
    def __init__(self, weights=(), scale=1.0):
        self.weights, self.scale = list(make_iterable(weights)), scale

    def export_proto(self):
        proto = pb.ObjectiveFunction.L2WeightRegularization()
        proto.scale_factor = self.scale
        proto.weights.extend(w.name for w in self.weights)
        return proto


class ObjectiveFunction:
    """Sum of scaled layer terms and weight regularisation terms."""

    def __init__(self, terms=()):
        self.terms = []
        for t in make_iterable(terms):
            self.add_term(t)

    def add_term(self, term):
        if isinstance(term, Layer):
            term = LayerTerm(term)
        self.terms.append(term)

    def export_proto(self):
        proto = pb.ObjectiveFunction()
        for t in self.terms:
            if isinstance(t, LayerTerm):
                proto.layer_term.add().CopyFrom(t.export_proto())
            elif isinstance(t, L2WeightRegularization):
                proto.l2_weight_regularization.add().CopyFrom(t.export_proto())
        return proto


# ------------------------------------------------------------------ operators
class Operator:
    """Entrywise tensor operation used inside an ``OperatorLayer``."""

    _message = None

    def __init__(self, input_type=DataType.FLOAT, output_type=None, device=None, **params):
        self.input_type = input_type
        self.output_type = input_type if output_type is None else output_type
        self.device = device
        names = [f.name for f in self._message.DESCRIPTOR.fields] if self._message else []
        for k in params:
            if k not in names:
                raise ValueError(f"{type(self).__name__}: unknown argument {k}")
        for n in names:
            setattr(self, n, params.get(n))

    def do_export_proto(self):
        msg = self._message()
        set_message(msg, **{f.name: getattr(self, f.name, None) for f in msg.DESCRIPTOR.fields})
        return msg

    def export_proto(self):
        op = pb.Operator()
        op.input_datatype = self.input_type
        op.output_datatype = self.output_type
        if self.device:
            op.device_allocation = self.device
        op.parameters.Pack(self.do_export_proto())
        return op


def _operator_messages():
    out = {}
    for name in dir(pb):
        if name.endswith("Operator") and name not in ("Operator",):
            cls = getattr(pb, name)
            if hasattr(cls, "DESCRIPTOR"):
                out[name[:-len("Operator")]] = cls
    return out


operator_classes = {}
for _short, _msg in _operator_messages().items():
    operator_classes[_short] = type(_short, (Operator,), {"_message": _msg,
                                                         "__doc__": f"{_short} operator"})


def _single_operator_layer(op_cls):
    def __init__(self, *args, **kwargs):
        layer_kwargs = {k: kwargs.pop(k) for k in list(kwargs) if k in _LAYER_BASE_KWARGS}
        OperatorLayer.__init__(self, *args, ops=[op_cls(**kwargs)], **layer_kwargs)

    def export_proto(self):
        dev = DeviceAllocation.DEFAULT_DEVICE
        if isinstance(self.device, str):
            dev = {"cpu": DeviceAllocation.CPU, "gpu": DeviceAllocation.GPU}.get(
                self.device.lower(), dev)
        for o in self.ops:
            o.input_type = o.output_type = self.datatype or 0
            o.device = dev
        return OperatorLayer.export_proto(self)

    return type(op_cls.__name__, (OperatorLayer,), {"__init__": __init__,
                                                    "export_proto": export_proto})


operator_layer_classes = {n: _single_operator_layer(c) for n, c in operator_classes.items()}
# A few operator names coincide with layer types that exist in their own right
# (e.g. LogSoftmax); the dedicated layer wins, as in the reference front end.
for _n, _c in operator_layer_classes.items():
    if _n not in layer_classes:
        globals()[_n] = _c


# ------------------------------------------------------------------ training algorithms
class TrainingAlgorithm:
    def __init__(self, name):
        self.name = name

    def export_proto(self):
        algo = pb.TrainingAlgorithm()
        algo.name = self.name
        algo.parameters.Pack(self.do_export_proto())
        return algo


class BatchedIterativeOptimizer(TrainingAlgorithm):
    """Mini-batch SGD-family training loop with batch / epoch / seconds stopping."""

    class StoppingCriteria:
        def __init__(self, batch_count=0, epoch_count=0, seconds=0.0):
            self.batch_count, self.epoch_count, self.seconds = batch_count, epoch_count, seconds

        def export_proto(self):
            msg = pb.SGD.TerminationCriteria()
            if self.batch_count > 0:
                msg.max_batches = self.batch_count
            if self.epoch_count > 0:
                msg.max_epochs = self.epoch_count
            if self.seconds > 0:
                msg.max_seconds = self.seconds
            return msg

    def __init__(self, name, num_iterations=0, epoch_count=0, max_seconds=0.0):
        super().__init__(name)
        self.stopping = self.StoppingCriteria(num_iterations, epoch_count, max_seconds)

    def do_export_proto(self):
        params = pb.SGD()
        params.stopping_criteria.CopyFrom(self.stopping.export_proto())
        return params


class MetaLearningStrategy:
    pass


class MutationStrategy:
    def __init__(self, strategy="null_mutation"):
        self.strategy = strategy

    def export_proto(self):
        msg = pb.MutationStrategy()
        getattr(msg, self.strategy).SetInParent()
        return msg


class RandomPairwiseExchange(MetaLearningStrategy):
    class MetricStrategy:
        LOWER_IS_BETTER = 0
        HIGHER_IS_BETTER = 1

    class ExchangeStrategy:
        def __init__(self, strategy="checkpoint_binary", weights_names=(),
                     exchange_hyperparameters=False, checkpoint_dir=None):
            self.strategy = strategy
            self.weights_names = list(make_iterable(weights_names))
            self.exchange_hyperparameters = exchange_hyperparameters
            self.checkpoint_dir = checkpoint_dir

        def export_proto(self):
            msg = pb.RandomPairwiseExchange.ExchangeStrategy()
            msg.weights_name.extend(self.weights_names)
            if self.strategy == "sendrecv_weights":
                msg.sendrecv_weights.exchange_hyperparameters = self.exchange_hyperparameters
            elif self.strategy == "checkpoint_file":
                msg.checkpoint_file.checkpoint_dir = self.checkpoint_dir or ""
            else:
                msg.checkpoint_binary.SetInParent()
            return msg

    def __init__(self, metric_strategies=None, exchange_strategy=None, mutation_strategy=None):
        self.metric_strategies = dict(metric_strategies or {})
        self.exchange_strategy = exchange_strategy or self.ExchangeStrategy()
        self.mutation_strategy = mutation_strategy or MutationStrategy()

    def export_proto(self):
        msg = pb.RandomPairwiseExchange()
        for k, v in self.metric_strategies.items():
            msg.metric_name_strategy_map[k] = v
        msg.exchange_strategy.CopyFrom(self.exchange_strategy.export_proto())
        msg.mutation_strategy.CopyFrom(self.mutation_strategy.export_proto())
        return msg


class TruncationSelectionExchange(MetaLearningStrategy):
    MetricStrategy = RandomPairwiseExchange.MetricStrategy

    def __init__(self, metric_strategies=None, truncation_k=0):
        self.metric_strategies = dict(metric_strategies or {})
        self.truncation_k = truncation_k

    def export_proto(self):
        msg = pb.TruncationSelectionExchange()
        for k, v in self.metric_strategies.items():
            msg.metric_name_strategy_map[k] = v
        msg.truncation_k = self.truncation_k
        return msg


class RegularizedEvolution(MetaLearningStrategy):
    MetricStrategy = RandomPairwiseExchange.MetricStrategy

    def __init__(self, metric_name, metric_strategy, mutation_strategy=None, sample_size=0):
        self.metric_name, self.metric_strategy = metric_name, metric_strategy
        self.mutation_strategy = mutation_strategy or MutationStrategy()
        self.sample_size = sample_size

    def export_proto(self):
        msg = pb.RegularizedEvolution()
        msg.metric_name = self.metric_name
        msg.metric_strategy = self.metric_strategy
        msg.mutation_strategy.CopyFrom(self.mutation_strategy.export_proto())
        msg.sample_size = self.sample_size
        return msg


class LTFB(TrainingAlgorithm):
    """Tournament ("let a thousand flowers bloom") population training."""

    def __init__(self, name, local_algo, metalearning, metalearning_steps=1):
        super().__init__(name)
        self.local_algo, self.metalearning = local_algo, metalearning
        self.metalearning_steps = metalearning_steps

    def do_export_proto(self):
        params = pb.LTFB()
        params.stopping_criteria.max_tournaments = self.metalearning_steps
        params.meta_learning_strategy.Pack(self.metalearning.export_proto())
        params.local_training_algorithm.CopyFrom(self.local_algo.export_proto())
        return params


class KFAC(TrainingAlgorithm):
    """Kronecker-factored second-order preconditioning around a first-order loop."""

    def __init__(self, name, first_order_optimizer, **kfac_args):
        super().__init__(name)
        self.first_order_optimizer = first_order_optimizer
        self.kfac_args = kfac_args

    def do_export_proto(self):
        params = pb.KFAC()
        params.sgd.CopyFrom(self.first_order_optimizer.do_export_proto())
        args = dict(self.kfac_args)
        for k, v in list(args.items()):
            if isinstance(v, (list, tuple)):
                args[k] = str_list(v)
        set_message(params, **args)
        return params


# ------------------------------------------------------------------ model / trainer
@dataclass
class AmpOptions:
    enabled: bool = False
    init_scale: Optional[float] = None
    growth_factor: Optional[float] = None
    backoff_factor: Optional[float] = None
    growth_interval: Optional[int] = None


class Model:
    """A layer graph plus objective, metrics and callbacks, trained for ``epochs``."""

    def __init__(self, epochs, layers=(), weights=(), objective_function=None, metrics=(),
                 callbacks=(), name=None, summary_dir=None, subgraph_communication=None,
                 subgraph_topology=False, subgraph_num_common_resources=0, amp=None):
        self.epochs = epochs
        self.name = name
        self.summary_dir = summary_dir
        self.layers = list(traverse_layer_graph(layers))
        seen, ws = set(), []
        for w in list(make_iterable(weights)) + [w for l in self.layers for w in l.weights]:
            if id(w) not in seen:
                seen.add(id(w))
                ws.append(w)
        self.weights = ws
        if isinstance(objective_function, ObjectiveFunction):
            self.objective_function = objective_function
        elif objective_function is None:
            self.objective_function = ObjectiveFunction()
        else:
            self.objective_function = ObjectiveFunction(objective_function)
        self.metrics = list(make_iterable(metrics))
        self.callbacks = list(make_iterable(callbacks))
        self.subgraph_communication = subgraph_communication
        self.subgraph_topology = subgraph_topology
        self.subgraph_num_common_resources = subgraph_num_common_resources
        self.amp = amp

    def export_proto(self):
        m = pb.Model()
        if self.name is not None:
            m.name = self.name
        m.num_epochs = self.epochs
        if self.subgraph_communication is not None:
            m.subgraph_communication = self.subgraph_communication
        m.enable_subgraph_topology = bool(self.subgraph_topology)
        m.subgraph_parent_grid_resources = self.subgraph_num_common_resources
        if self.summary_dir is not None:
            m.summarizer.dir = self.summary_dir
        m.layer.extend(l.export_proto() for l in self.layers)
        m.weights.extend(w.export_proto() for w in self.weights)
        m.objective_function.CopyFrom(self.objective_function.export_proto())
        m.metric.extend(x.export_proto() for x in self.metrics)
        m.callback.extend(c.export_proto() for c in self.callbacks)
        if self.amp is not None:
            m.amp.enabled = self.amp.enabled
            for k in ("init_scale", "growth_factor", "backoff_factor", "growth_interval"):
                v = getattr(self.amp, k)
                if v is not None:
                    setattr(m.amp, k, v)
        return m

    def __call__(self, *args, **kwargs):
        from ..launcher.evaluate import evaluate
        return evaluate(self, *args, **kwargs)


class Trainer:
    """Owns the mini-batch size, seeds, trainer-level callbacks and training algorithm."""

    def __init__(self, mini_batch_size, name=None, random_seed=None, serialize_io=None,
                 training_algo=None, callbacks=()):
        self.mini_batch_size = mini_batch_size
        self.name = name
        self.random_seed = random_seed
        self.serialize_io = serialize_io
        self.hydrogen_block_size = None
        self.training_algo = training_algo
        self.callbacks = list(make_iterable(callbacks))

    def export_proto(self):
        t = pb.Trainer()
        if self.name is not None:
            t.name = self.name
        if self.random_seed is not None:
            t.random_seed = self.random_seed
        if self.mini_batch_size is not None:
            t.mini_batch_size = self.mini_batch_size
        if self.hydrogen_block_size is not None:
            t.hydrogen_block_size = self.hydrogen_block_size
        if self.serialize_io is not None:
            t.serialize_io = self.serialize_io
        if self.training_algo is not None:
            t.training_algorithm.CopyFrom(self.training_algo.export_proto())
        t.callback.extend(c.export_proto() for c in self.callbacks)
        return t


def get_parallel_strategy_args(**kwargs):
    """``{sample,depth,height,width,channel,filter}_groups`` dictionary with 1 defaults."""
    names = [f"{d}_groups" for d in ("sample", "depth", "height", "width", "channel", "filter")]
    extra = set(kwargs) - set(names)
    if extra:
        raise ValueError(f"unknown parallel strategy arguments {sorted(extra)}")
    return {n: kwargs.get(n, 1) for n in names}


__all__ = [n for n in globals() if not n.startswith("_")]
