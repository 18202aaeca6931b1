"""CPU restatement of a whole training step -- TEST INFRASTRUCTURE / CPU BASELINE ONLY.

Runs a network given as a small spec (nested tuples) with the oracle operators of
``conv_oracle`` / ``aux_oracle``: the reference's CPU algorithm (im2row + ``@``, NumPy batch
norm, Cython-equivalent pooling, softmax + categorical cross-entropy, SGD with momentum), in the
order of the reference's train loop (pydtnn/model.py:450-527).  Where ``oracle/_ref`` holds the
reference's own compiled Cython kernels they do the lowering and pooling, and the run counts as
the reference's CPU path; otherwise the restatements do.

Used by the model-level parity tests and by the benchmark's CPU-baseline / reference arm.
"""
from __future__ import annotations

import numpy as np

from . import aux_oracle as ao
from . import conv_oracle as co

# ---- specs ------------------------------------------------------------------------------------
# ("conv", co, k, stride, pad) | ("bn",) | ("relu",) | ("maxpool", k, stride, pad) | ("gap",)
# | ("flatten",) | ("fc", out) | ("softmax",) | ("add", [path0...], [path1...])


def resnet50_spec(nclasses=1000, layout=None):
    """pydtnn/models/resnet50_imagenet.py:24-63"""
    spec = [("conv", 64, 7, 2, 3), ("maxpool", 3, 2, 1)]
    layout = layout or [[64, 3, 1], [128, 4, 2], [256, 6, 2], [512, 3, 2]]
    for n_filt, blocks, stride in layout:
        for r in range(blocks):
            if r > 0:
                stride = 1
            main = [("conv", n_filt, 1, 1, 0), ("bn",), ("relu",), ("conv", n_filt, 3, stride, 1), ("bn",), ("relu",),
                    ("conv", n_filt * 4, 1, 1, 0), ("bn",)]
            short = [("conv", n_filt * 4, 1, stride, 0), ("bn",)] if r == 0 or stride != 1 else []
            spec += [("add", main, short), ("relu",)]
    spec += [("gap",), ("flatten",), ("fc", nclasses), ("softmax",)]
    return spec


def vgg16_spec(nclasses=1000, batch_norm=False):
    """pydtnn/models/vgg16_imagenet.py:23-37 (dropout left out: identity in evaluation)"""
    spec = []
    for n_filt, convs in ((64, 2), (128, 2), (256, 3), (512, 3), (512, 3)):
        for _ in range(convs):
            spec += [("conv", n_filt, 3, 1, 1)] + ([("bn",)] if batch_norm else []) + [("relu",)]
        spec += [("maxpool", 2, 2, 0)]
    spec += [("flatten",), ("fc", 4096), ("relu",), ("fc", 4096), ("relu",), ("fc", nclasses), ("softmax",)]
    return spec


def alexnet_spec(nclasses=1000):
    """pydtnn/models/alexnet_imagenet.py:23-39 (dropout = identity in evaluation)"""
    return [("conv", 96, 11, 4, 0), ("relu",), ("maxpool", 3, 2, 0), ("conv", 256, 5, 1, 2), ("relu",),
            ("maxpool", 3, 2, 0), ("conv", 384, 3, 1, 1), ("relu",), ("conv", 384, 3, 1, 1), ("relu",),
            ("conv", 256, 3, 1, 1), ("relu",), ("maxpool", 3, 2, 0), ("flatten",), ("fc", 4096), ("relu",),
            ("fc", 4096), ("relu",), ("fc", nclasses), ("softmax",)]


# ---- nodes --------------------------------------------------------------------------------------

class _Node:
    params = ()

    def grads(self):
        return []


class Conv(_Node):
    def __init__(self, in_shape, n, cout, k, stride, pad, dtype, layout, rng):
        h, w, c = in_shape
        self.g = co.Geom(n, h, w, c, cout, k, k, pad, pad, stride, stride)
        self.layout = layout
        lim = np.sqrt(6.0 / (c * k * k))
        wshape = (c, k, k, cout) if layout == "NHWC" else (cout, c, k, k)
        self.w = rng.uniform(-lim, lim, wshape).astype(dtype)
        self.b = np.zeros((cout,), dtype)
        self.out_shape = (self.g.ho, self.g.wo, cout)
        self.params = ("w", "b")

    def forward(self, x, train):
        self.x, self.keep = x, {}
        return co.conv2d_forward(x, self.w, self.b, self.g, self.layout, keep=self.keep if train else None)

    def backward(self, dy, need_dx=True):
        self.dw, self.db, dx = co.conv2d_backward(self.x, dy, self.w, self.g, self.layout, need_dx, True, keep=self.keep)
        self.keep = {}
        return dx


class BN(_Node):
    def __init__(self, in_shape, dtype, layout):
        c = in_shape[-1]
        self.layout = layout
        self.gamma, self.beta = np.ones(c, dtype), np.zeros(c, dtype)
        self.rm, self.rv = np.zeros(c, dtype), np.zeros(c, dtype)
        self.out_shape = in_shape
        self.params = ("gamma", "beta")

    def forward(self, x, train):
        if train:
            y, self.cache, self.rm, self.rv = ao.bn_train_forward(x, self.gamma, self.beta, self.rm, self.rv, 0.9, 1e-5,
                                                                  self.layout)
            return y
        inv_std = (1.0 / np.sqrt(self.rv + 1e-5)).astype(x.dtype)
        return ao.bn_inference(x, self.rm, inv_std, self.gamma, self.beta, self.layout)

    def backward(self, dy, need_dx=True):
        self.dgamma, self.dbeta, dx = ao.bn_train_backward(dy, self.cache, self.gamma, self.layout, need_dx)
        return dx


class Relu(_Node):
    def __init__(self, in_shape):
        self.out_shape = in_shape

    def forward(self, x, train):
        y, self.mask = ao.relu_forward(x)
        return y

    def backward(self, dy, need_dx=True):
        return ao.relu_backward(dy, self.mask)


class Pool(_Node):
    def __init__(self, in_shape, is_max, k, stride, pad, layout):
        h, w, c = in_shape
        self.is_max, self.layout = is_max, layout
        kh, kw = (h, w) if k == 0 else (k, k)
        self.args = (kh, kw, pad, pad, stride, stride, 1, 1)
        ho = (h + 2 * pad - (kh - 1) - 1) // stride + 1
        wo = (w + 2 * pad - (kw - 1) - 1) // stride + 1
        self.out_shape = (ho, wo, c)

    def _ref(self, name):
        mods = co.ref_kernels()
        suffix = "nhwc" if self.layout == "NHWC" else "nchw"
        mod = mods.get(f"{'max' if self.is_max else 'average'}_pool_2d_{suffix}_cython")
        return getattr(mod, f"{'max' if self.is_max else 'average'}_pool_2d_{name}_{suffix}_cython") if mod else None

    def forward(self, x, train):
        self.x_shape = x.shape
        f = self._ref("fwd")
        if self.is_max:
            if f is not None:
                y, self.idx = f(np.ascontiguousarray(x), *self.args)
            else:
                y, self.idx = ao.max_pool_forward(x, *self.args, layout=self.layout)
            return y
        return f(np.ascontiguousarray(x), *self.args) if f is not None else ao.avg_pool_forward(x, *self.args, layout=self.layout)

    def backward(self, dy, need_dx=True):
        f = self._ref("bwd")
        if self.layout == "NHWC":
            n, h, w, c = self.x_shape
        else:
            n, c, h, w = self.x_shape
        dims = (n, h, w, c) if self.layout == "NHWC" else (n, c, h, w)
        if self.is_max:
            if f is not None:
                return f(np.ascontiguousarray(dy), self.idx, n, h, w, c, *self.args)
            return ao.max_pool_backward(dy, self.idx, dims, *self.args, layout=self.layout)
        if f is not None:
            return f(np.ascontiguousarray(dy), n, h, w, c, *self.args)
        return ao.avg_pool_backward(dy, dims, *self.args, layout=self.layout)


class Flatten(_Node):
    def __init__(self, in_shape):
        self.out_shape = (int(np.prod(in_shape)),)

    def forward(self, x, train):
        self.shape = x.shape
        return x.reshape(x.shape[0], -1)

    def backward(self, dy, need_dx=True):
        return dy.reshape(self.shape)


class FC(_Node):
    def __init__(self, in_shape, out, dtype, rng):
        fin = in_shape[0]
        lim = np.sqrt(6.0 / fin)
        self.w = rng.uniform(-lim, lim, (fin, out)).astype(dtype)
        self.b = np.zeros((out,), dtype)
        self.out_shape = (out,)
        self.params = ("w", "b")

    def forward(self, x, train):
        self.x = x
        return co.fc_forward(x, self.w, self.b)

    def backward(self, dy, need_dx=True):
        self.dw, self.db, dx = co.fc_backward(self.x, dy, self.w, need_dx)
        return dx


class Softmax(_Node):
    def __init__(self, in_shape):
        self.out_shape = in_shape

    def forward(self, x, train):
        self.y = ao.softmax_forward(x)
        return self.y

    def backward(self, dy, need_dx=True):
        return ao.softmax_backward(dy, self.y)


class Add(_Node):
    """Sum of parallel paths; an empty path is the identity
    (pydtnn/backends/cpu/layers/addition_block_cpu.py:36-66)."""

    def __init__(self, paths):
        self.paths = paths
        self.out_shape = paths[0][-1].out_shape

    def forward(self, x, train):
        outs = []
        for p in self.paths:
            y = x
            for node in p:
                y = node.forward(y, train)
            outs.append(y)
        y = outs[0]
        for o in outs[1:]:
            y = y + o
        return y

    def backward(self, dy, need_dx=True):
        total = None
        for p in self.paths:
            d = dy
            for node in reversed(p):
                d = node.backward(d)
            total = d if total is None else total + d
        return total


class CpuNet:
    """A network on the CPU oracle. ``in_shape`` is (h, w, c); tensors use ``layout``."""

    def __init__(self, spec, in_shape, batch, dtype=np.float32, layout="NHWC", seed=0):
        self.dtype, self.layout, self.batch = np.dtype(dtype), layout, batch
        self.rng = np.random.Generator(np.random.PCG64(seed))
        self.nodes, _ = self._build(spec, tuple(in_shape))
        self.velocity = {}

    def _build(self, spec, shape):
        nodes = []
        for item in spec:
            kind = item[0]
            if kind == "conv":
                node = Conv(shape, self.batch, item[1], item[2], item[3], item[4], self.dtype, self.layout, self.rng)
            elif kind == "bn":
                node = BN(shape, self.dtype, self.layout if len(shape) == 3 else "NHWC")
            elif kind == "relu":
                node = Relu(shape)
            elif kind == "maxpool":
                node = Pool(shape, True, item[1], item[2], item[3], self.layout)
            elif kind == "avgpool":
                node = Pool(shape, False, item[1], item[2], item[3], self.layout)
            elif kind == "gap":
                node = Pool(shape, False, 0, 1, 0, self.layout)
            elif kind == "flatten":
                node = Flatten(shape)
            elif kind == "fc":
                node = FC(shape, item[1], self.dtype, self.rng)
            elif kind == "softmax":
                node = Softmax(shape)
            elif kind == "add":
                paths = []
                for p in item[1:]:
                    sub, _ = self._build(p, shape)
                    paths.append(sub)
                if not paths[0]:
                    raise ValueError("first path of an add block must not be empty")
                node = Add(paths)
            else:
                raise ValueError(kind)
            nodes.append(node)
            shape = node.out_shape
        return nodes, shape

    def all_nodes(self, nodes=None):
        out = []
        for n in (self.nodes if nodes is None else nodes):
            out.append(n)
            if isinstance(n, Add):
                for p in n.paths:
                    out += self.all_nodes(p)
        return out

    def forward(self, x, train=True):
        acts = [x]
        for node in self.nodes:
            x = node.forward(x, train)
            acts.append(x)
        self.acts = acts
        return x

    def backward(self, d):
        """Backward through every node; the first node's dx is not needed (pydtnn/model.py:270)."""
        self.dacts = {}
        for i in range(len(self.nodes) - 1, -1, -1):
            d = self.nodes[i].backward(d, need_dx=(i > 0))
            self.dacts[i] = d
        return d

    def loss_and_grad(self, probs, labels, global_batch):
        y_targ = np.zeros(probs.shape, probs.dtype)
        y_targ[np.arange(probs.shape[0]), labels] = 1
        loss, dx = ao.categorical_cross_entropy(probs, y_targ, global_batch)
        return float(loss), dx.astype(probs.dtype)

    def sgd(self, lr, momentum=0.9, decay=0.0):
        for node in self.all_nodes():
            for name in node.params:
                gname = {"w": "dw", "b": "db", "gamma": "dgamma", "beta": "dbeta"}[name]
                w, dw = getattr(node, name), getattr(node, gname)
                key = (id(node), name)
                v = self.velocity.get(key)
                if v is None:
                    v = np.zeros_like(w)
                w, v = ao.sgd_update(w, dw.reshape(w.shape).astype(w.dtype), v, lr, momentum, False, decay)
                setattr(node, name, w)
                self.velocity[key] = v

    def train_step(self, x, labels, lr=0.01, momentum=0.9, global_batch=None):
        probs = self.forward(x, True)
        loss, d = self.loss_and_grad(probs, labels, global_batch or x.shape[0])
        self.backward(d)
        self.sgd(lr, momentum)
        return loss
