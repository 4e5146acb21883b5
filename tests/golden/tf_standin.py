"""A minimal stand-in for the part of the TensorFlow API that the reference's
``v1_model_utils/models.py`` calls, backed by PyTorch CPU tensors.

Purpose: TensorFlow cannot be installed where the fixtures are made, so the reference's own
``V1Column`` (its Python source, unmodified, imported from the reference tree) is executed over
this module to produce golden vectors that pin ``oracle/``.  Only ``run_reference_models.py`` in
this folder uses it; nothing in the product or in the tests imports it at run time.

What is and is not exercised: every line of the reference's index arithmetic, op sequence,
layouts, custom gradients and stop-gradients runs as written; TensorFlow's kernels (summation
order, Philox sampler) do not.  ``tf.random.stateless_poisson`` returns the counts installed with
``set_poisson_counts`` so that the background input is a controlled input.
"""
import sys
import types

import numpy as np
import torch

_DTYPE = [torch.float64]      # keras policy dtype (compute == variable)
_POISSON = [None]


def set_policy_dtype(dt):
    _DTYPE[0] = dt


def set_poisson_counts(counts):
    _POISSON[0] = counts


def _t(x, dtype=None):
    if isinstance(x, torch.Tensor):
        return x if dtype is None else x.to(dtype)
    a = np.asarray(x)
    # keep NumPy's dtype (float64 / int64 for Python scalars), as tf.constant + cast would
    t = torch.from_numpy(a.copy()) if a.ndim else torch.from_numpy(a.reshape(1).copy())[0]
    return t if dtype is None else t.to(dtype)


def _i(x):
    return int(x.item()) if isinstance(x, torch.Tensor) else int(x)


class RaggedTensor:
    def __init__(self, values, row_splits):
        self.flat_values = values
        self.row_splits = row_splits.long()

    @classmethod
    def from_row_splits(cls, values, row_splits, validate=True):
        return cls(values, row_splits)

    def row_lengths(self):
        return self.row_splits[1:] - self.row_splits[:-1]

    def __getitem__(self, i):
        i = _i(i)
        return self.flat_values[int(self.row_splits[i]):int(self.row_splits[i + 1])]

    def _gather_rows(self, rows):
        start = self.row_splits[rows]
        length = self.row_splits[rows + 1] - start
        total = int(length.sum())
        excl = torch.cumsum(length, 0) - length
        pos = torch.arange(total, dtype=torch.int64) + torch.repeat_interleave(start - excl, length)
        splits = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(length, 0)])
        return RaggedTensor(self.flat_values[pos], splits)


class SparseTensor:
    def __init__(self, indices, values, dense_shape):
        self.indices, self.values = _t(indices).long(), values
        self.dense_shape = (_i(dense_shape[0]), _i(dense_shape[1]))


def _sparse_dense_matmul(a, b, adjoint_a=False, adjoint_b=False):
    if isinstance(b, SparseTensor):                       # dense [B, N] @ sparse [N, M]
        assert not adjoint_a and not adjoint_b
        rows, cols = b.indices[:, 0], b.indices[:, 1]
        out = torch.zeros((a.shape[0], b.dense_shape[1]), dtype=a.dtype)
        return out.index_add(1, cols, a[:, rows] * b.values[None, :])
    raise NotImplementedError("only dense @ sparse is needed by the cell")


def _variable(value, trainable=True, dtype=None, name=None, constraint=None, **kw):
    t = _t(value, dtype).clone().detach()
    if t.is_floating_point() and trainable:
        t.requires_grad_(True)
    t.trainable = bool(trainable)
    t.constraint = constraint
    t.read_value = lambda: t

    def _assign(value):
        t.data.copy_(_t(value).detach().to(t.dtype))
        return t

    def _assign_add(value):
        t.data.add_(_t(value).detach().to(t.dtype))
        return t
    t.assign = _assign
    t.assign_add = _assign_add
    return t


class _Optimizer:
    """The part of ``tf.keras.optimizers.Optimizer`` that the reference's ``ExponentiatedAdam``
    relies on: slot variables, the iteration counter and the variable -> slot index table."""

    def __init__(self, name=None, **kw):
        self.name = name
        self.iterations = torch.zeros((), dtype=torch.int64)
        self._index_dict = {}

    def _build_learning_rate(self, learning_rate):
        return learning_rate

    @property
    def learning_rate(self):
        lr = self._learning_rate
        return lr(self.iterations) if callable(lr) else lr

    def _var_key(self, variable):
        return id(variable)

    def build(self, var_list):
        for i, var in enumerate(var_list):
            self._index_dict[self._var_key(var)] = i

    def add_variable_from_reference(self, model_variable, variable_name, **kw):
        return _variable(torch.zeros_like(model_variable.detach()), trainable=False)

    def _serialize_hyperparameter(self, h):
        return h

    def get_config(self):
        return {"name": self.name}


def _gather(params, indices, axis=0, **kw):
    if isinstance(params, RaggedTensor):
        return params._gather_rows(_t(indices).long())
    p, idx = _t(params), _t(indices).long()
    return p[idx] if axis == 0 else p.index_select(axis, idx.reshape(-1))


def _where(cond, x=None, y=None):
    if x is None:
        return torch.nonzero(cond)
    return torch.where(cond, _t(x), _t(y))


def _unsorted_segment_sum(data, segment_ids, num_segments):
    shape = (_i(num_segments),) + tuple(data.shape[1:])
    return torch.zeros(shape, dtype=data.dtype).index_add(0, _t(segment_ids).long(), data)


def _unsorted_segment_mean(data, segment_ids, num_segments):
    ids = _t(segment_ids).long()
    tot = torch.zeros((_i(num_segments),), dtype=data.dtype).index_add(0, ids, data)
    cnt = torch.zeros((_i(num_segments),), dtype=data.dtype).index_add(0, ids, torch.ones_like(data))
    return tot / torch.clamp(cnt, min=1.0)


def _shape(x, out_type=None):
    return torch.tensor(list(x.shape), dtype=out_type or torch.int32)


def _sizes(shape):
    return [_i(s) for s in (shape.tolist() if isinstance(shape, torch.Tensor) else shape)]


def _while_loop(cond, body, loop_vars, **kw):
    v = list(loop_vars)
    while bool(cond(*v)):
        v = list(body(*v))
    return v


def _flatten_args(args):
    flat = []
    for a in args:
        flat.extend(list(a) if isinstance(a, (tuple, list)) else [a])
    return flat


def custom_gradient(f):
    """``tf.custom_gradient``: ``f(*args) -> (out, grad_fn)``; ``grad_fn(dy)`` returns one entry per
    flattened argument."""
    def wrapper(*args):
        flat = _flatten_args(args)
        t_pos = [i for i, a in enumerate(flat) if isinstance(a, torch.Tensor) and a.requires_grad]

        class Fn(torch.autograd.Function):
            @staticmethod
            def forward(ctx, *tensors):
                out, grad_fn = f(*args)
                ctx.grad_fn_ = grad_fn
                return out

            @staticmethod
            def backward(ctx, *dys):
                grads = ctx.grad_fn_(*dys)
                grads = list(grads) if isinstance(grads, (list, tuple)) else [grads]
                return tuple(grads[i] for i in t_pos)

        if not t_pos:
            return f(*args)[0]
        return Fn.apply(*[flat[i] for i in t_pos])
    return wrapper


def _function(*a, **kw):
    if len(a) == 1 and callable(a[0]) and not kw:
        return a[0]
    return lambda fn: fn


class _Layer:
    def __init__(self, *a, **kw):
        pass

    @property
    def compute_dtype(self):
        return _DTYPE[0]

    @property
    def variable_dtype(self):
        return _DTYPE[0]

    def _no_dependency(self, x):
        return x


class _Constraint:
    pass


def _maximum(a, b):
    a, b = _t(a), _t(b)
    return torch.maximum(a, b.to(a.dtype)) if b.ndim or a.ndim else torch.maximum(a, b)


def _reduce(fn):
    def r(x, axis=None, **kw):
        return fn(x) if axis is None else fn(x, dim=axis)
    return r


class _TensorArray:
    def __init__(self, dtype=None, size=0, **kw):
        self.items = {}

    def write(self, i, value):
        self.items[_i(i)] = value
        return self

    def stack(self):
        return torch.stack([self.items[k] for k in sorted(self.items)])


def _conv1d(x, kernel, stride=1, padding="VALID"):
    # x [batch, width, in_ch], kernel [k, in_ch, out_ch] -> [batch, new_width, out_ch]
    assert padding == "VALID"
    out = torch.nn.functional.conv1d(x.permute(0, 2, 1), kernel.permute(2, 1, 0), stride=_i(stride))
    return out.permute(0, 2, 1)


def _conv2d(x, kernel, strides=None, padding="SAME"):
    # x [batch, h, w, in_ch], kernel [kh, kw, in_ch, out_ch]; odd kernels, so SAME pads evenly
    assert padding == "SAME" and kernel.shape[0] % 2 == 1 and kernel.shape[1] % 2 == 1
    out = torch.nn.functional.conv2d(x.permute(0, 3, 1, 2), kernel.permute(3, 2, 0, 1),
                                     padding=(kernel.shape[0] // 2, kernel.shape[1] // 2))
    return out.permute(0, 2, 3, 1)


def _depthwise_conv2d(x, kernel, strides=None, padding="VALID"):
    # x [batch, h, w, ch], kernel [kh, kw, ch, 1] -> [batch, h - kh + 1, w - kw + 1, ch]
    assert padding == "VALID" and kernel.shape[3] == 1
    out = torch.nn.functional.conv2d(x.permute(0, 3, 1, 2), kernel.permute(2, 3, 0, 1), groups=x.shape[3])
    return out.permute(0, 2, 3, 1)


def _pad(x, paddings, **kw):
    flat = []
    for before, after in reversed([tuple(p) for p in paddings]):
        flat += [int(before), int(after)]
    return torch.nn.functional.pad(x, flat)


def install():
    """Register the stand-in as ``tensorflow`` in ``sys.modules`` and return it."""
    tf = types.ModuleType("tensorflow")
    for name, dt in dict(float16=torch.float16, float32=torch.float32, float64=torch.float64,
                         int8=torch.int8, int16=torch.int16, int32=torch.int32, int64=torch.int64,
                         bool=torch.bool, uint8=torch.uint8).items():
        setattr(tf, name, dt)
    tf.newaxis = None
    tf.cast = lambda x, dtype=None, **kw: _t(x, dtype)
    tf.constant = lambda v, dtype=None, **kw: _t(v, dtype)
    tf.convert_to_tensor = lambda v, dtype=None, **kw: _t(v, dtype)
    tf.Variable = _variable
    tf.gather = _gather
    tf.gather_nd = lambda p, idx: p[idx[:, 0].long(), idx[:, 1].long()]
    tf.where = _where
    tf.repeat = lambda x, repeats, **kw: torch.repeat_interleave(x, _t(repeats).long())
    tf.shape = _shape
    tf.reshape = lambda x, shape: x.reshape(_sizes(shape))
    tf.zeros = lambda shape, dtype=torch.float32: torch.zeros(_sizes(shape), dtype=dtype)
    tf.ones = lambda shape, dtype=torch.float32: torch.ones(_sizes(shape), dtype=dtype)
    tf.zeros_like = torch.zeros_like
    tf.ones_like = torch.ones_like
    tf.stop_gradient = lambda x: x.detach()
    tf.greater = lambda a, b: _t(a) > b
    tf.equal = lambda a, b: _t(a) == b
    tf.identity = lambda x, name=None: x
    tf.function = _function
    tf.expand_dims = lambda x, axis: x.unsqueeze(axis)
    tf.custom_gradient = custom_gradient
    tf.concat = lambda xs, axis: torch.cat(list(xs), dim=axis)
    tf.stack = lambda xs, axis=0: torch.stack([_t(x) for x in xs], dim=axis)
    tf.transpose = lambda x, perm=None: x.t() if perm is None else x.permute(*perm)
    tf.maximum = _maximum
    tf.abs = torch.abs
    tf.exp = torch.exp
    tf.square = torch.square
    tf.sign = torch.sign
    tf.sqrt = torch.sqrt
    tf.pow = torch.pow
    tf.cos = torch.cos
    tf.floor = torch.floor
    tf.pad = _pad
    tf.Tensor = torch.Tensor
    tf.IndexedSlices = type("IndexedSlices", (), {})
    tf.reduce_sum = _reduce(torch.sum)
    tf.reduce_mean = _reduce(torch.mean)
    tf.clip_by_value = lambda x, lo, hi: torch.clamp(x, _t(lo).item(), _t(hi).item())
    tf.einsum = torch.einsum
    tf.while_loop = _while_loop
    tf.TensorShape = lambda dims: tuple(dims)
    tf.RaggedTensor = RaggedTensor
    tf.math = types.SimpleNamespace(unsorted_segment_sum=_unsorted_segment_sum, exp=torch.exp,
                                    log=torch.log,
                                    reduce_variance=lambda x, axis=None: torch.var(x, dim=axis, unbiased=False),
                                    cos=torch.cos, square=torch.square, ceil=torch.ceil,
                                    unsorted_segment_mean=_unsorted_segment_mean)
    tf.TensorArray = _TensorArray
    tf.squeeze = lambda x, axis=None: x.squeeze() if axis is None else x.squeeze(axis)
    tf.nn = types.SimpleNamespace(relu=torch.relu, sigmoid=torch.sigmoid, conv1d=_conv1d, conv2d=_conv2d,
                                  depthwise_conv2d=_depthwise_conv2d,
                                  softplus=torch.nn.functional.softplus,
                                  softmax=lambda x, axis=-1: torch.softmax(x, dim=axis))
    tf.sparse = types.SimpleNamespace(SparseTensor=SparseTensor,
                                      sparse_dense_matmul=_sparse_dense_matmul)
    # tf.random.shuffle is the identity here and tf.sort is stable: where the reference shuffles before
    # a sort (rate-distribution loss), entries with equal keys keep their listed order
    tf.random = types.SimpleNamespace(
        stateless_poisson=lambda shape, seed, lam, dtype=torch.int32: _POISSON[0].to(dtype),
        shuffle=lambda x, seed=None: x)
    tf.sort = lambda x, axis=-1, direction="ASCENDING": torch.sort(
        x, dim=axis, descending=(direction == "DESCENDING"), stable=True).values
    tf.range = lambda *a, **kw: torch.arange(*[_i(v) for v in a], dtype=kw.get("dtype", torch.int64))
    tf.size = lambda x: torch.tensor(x.numel(), dtype=torch.int32)
    tf.distribute = types.SimpleNamespace(get_replica_context=lambda: None)
    layers = types.ModuleType("tensorflow.keras.layers")
    layers.Layer = _Layer
    keras = types.ModuleType("tensorflow.keras")
    keras.layers = layers
    keras.constraints = types.SimpleNamespace(Constraint=_Constraint)
    keras.regularizers = types.SimpleNamespace(Regularizer=object)
    keras.optimizers = types.SimpleNamespace(
        Optimizer=_Optimizer, schedules=types.SimpleNamespace(LearningRateSchedule=object))
    keras.utils = types.SimpleNamespace(register_keras_serializable=lambda **kw: (lambda cls: cls))
    tf.keras = keras
    sys.modules["tensorflow"] = tf
    sys.modules["tensorflow.keras"] = keras
    sys.modules["tensorflow.keras.layers"] = layers
    return tf
