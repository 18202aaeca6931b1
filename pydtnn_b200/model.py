"""Model: the layer list and the train / evaluate step of the reference
(pydtnn/model.py: ``add`` :268-283, ``__train_batch`` :450-527, ``__evaluate_batch`` :623-644, the
inference fusion pass :294-349), driving the GPU layers of this package.

Differences that are deliberate:
* the gradient exchange is a bucketed, event-ordered NCCL all-reduce (see comm.py) instead of one
  host-synchronised call per tensor;
* the optimiser runs once over the flat parameter arena instead of once per tensor;
* ``non_blocking_mpi`` keeps its meaning (overlap the exchange with backward) and is the default.
"""
import itertools

import numpy as np
import torch

from . import _lib, tracer
from .arena import ParamArena
from .backends.gpu import memory_allocation as wsp
from .comm import GradientBucketer
from .layers import (BatchNormalization, Conv2D, Conv2DBatchNormalization, Conv2DBatchNormalizationRelu, Conv2DRelu,
                     Relu)
from .losses import CategoricalCrossEntropy
from .performance_counter import PerformanceCounter
from .tensor_gpu import empty
from .utils import (EVALUATE_MODE, PYDTNN_TENSOR_FORMAT_NCHW, PYDTNN_TENSOR_FORMAT_NHWC, TRAIN_MODE,
                    UNSPECIFIED_MODE, np_dtype)


def _bn_fast_path(c):
    """Channel counts the float4 batch-norm kernels take (the ones that accept sums from the convolution)."""
    if c % 4 or c > 2048:
        return False
    c4 = c // 4
    cx = min(c4, 64)
    return 256 % cx == 0 and c4 % cx == 0


class Model:
    def __init__(self, comm=None, non_blocking_mpi=True, dtype=np.float32, batch_size=64, tensor_format="NHWC",
                 enable_fused_bn_relu=False, enable_fused_conv_relu=False, enable_fused_conv_bn=False,
                 enable_fused_conv_bn_relu=False, conv_engine=_lib.ENGINE_AUTO, device=None, model_name=None,
                 bucket_elems=6 * 1024 * 1024, **kwargs):
        _lib.lib()  # fail loudly right away if the CUDA extension is missing
        if not torch.cuda.is_available():
            raise RuntimeError("pydtnn_b200 needs a CUDA device; there is no CPU back end")
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        torch.cuda.set_device(self.device)
        self.dtype = np_dtype(dtype).type
        self.batch_size = int(batch_size)
        if tensor_format in ("NCHW", "AUTO", PYDTNN_TENSOR_FORMAT_NCHW) and tensor_format != PYDTNN_TENSOR_FORMAT_NHWC:
            # AUTO means NCHW on the GPU in the reference (pydtnn/model.py:207-215)
            self.tensor_format = PYDTNN_TENSOR_FORMAT_NCHW
        else:
            self.tensor_format = PYDTNN_TENSOR_FORMAT_NHWC
        self.enable_fused_bn_relu = enable_fused_bn_relu
        self.enable_fused_conv_relu = enable_fused_conv_relu
        self.enable_fused_conv_bn = enable_fused_conv_bn
        self.enable_fused_conv_bn_relu = enable_fused_conv_bn_relu
        self.conv_engine = conv_engine
        self.kwargs = kwargs
        self.blocking_mpi = not non_blocking_mpi
        # comm: a torch.distributed process group, True (= default group) or None (single process)
        self.comm = None
        self.rank, self.nprocs = 0, 1
        if comm is not None and comm is not False:
            import torch.distributed as dist
            if dist.is_initialized() and dist.get_world_size() > 1:
                self.comm = dist.group.WORLD if comm is True else comm
                self.rank, self.nprocs = dist.get_rank(), dist.get_world_size()
        self.layers = []
        self.layer_id = itertools.count()
        self.nparams = 0
        self.mode = UNSPECIFIED_MODE
        self.arena = ParamArena(self.dtype, self.device)
        self.bucketer = GradientBucketer(self.arena, self.comm, bucket_elems)
        self.bucketer.before_launch = self.join_side_stream      # weight gradients on the side stream belong to the bucket
        self.y_batch = None
        self.loss_func = None
        self._train_fused = False
        self._stage = None
        self.tracer = tracer.StepTracer()        # off until enable_tracing()
        self.perf_counter = PerformanceCounter()
        self._eval_layers = None
        self.fast_update = True
        self.fuse_add_relu = True
        self.fuse_conv_bn_stats = True      # training: a Conv2D that feeds a BatchNormalization also sums its output per channel
        self.overlap_wgrad = True           # training: weight gradients of the convolutions run on a side stream
        self._side_stream = None
        self._side_pending = None           # last event recorded on the side stream that the main stream has not waited for
        if model_name:
            from . import nets
            getattr(nets, f"create_{model_name}")(self)

    # ------------------------------------------------------------------------------------------
    @property
    def stream_handle(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    # -- side stream of the weight gradients ---------------------------------------------------------------
    def side_stream_for_wgrad(self):
        """The stream convolution weight gradients are issued on, or None when they stay on the main stream: overlap
        switched off, per-pass timing (``conv_profile``) or per-operation tracing in progress (both bracket single
        passes with events on the main stream)."""
        if not self.overlap_wgrad or self.mode != TRAIN_MODE or getattr(self, "conv_profile", None) is not None \
                or (self.tracer.enabled and self.tracer.ops):
            return None
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(device=self.device)
        return self._side_stream

    def note_side_work(self, event):
        self._side_pending = event

    def join_side_stream(self):
        """Make the main stream wait for everything issued on the side stream so far (the side stream is in order, so
        its latest event covers the earlier ones).  Called before gradients are exchanged, applied or read."""
        if self._side_pending is not None:
            torch.cuda.current_stream(self.device).wait_event(self._side_pending)
            self._side_pending = None

    def add(self, layer):
        layer.set_model(self)
        need_dx = layer.id > 1
        prev_shape = self.layers[-1].shape if layer.id > 0 else ()
        y = self.layers[-1].y if layer.id > 0 else None
        layer.initialize(prev_shape, need_dx, y)
        self.nparams += layer.nparams
        self.layers.append(layer)
        if layer.act:
            self.add(layer.act())

    def get_all_layers(self, from_layers=None):
        if from_layers is None:
            from_layers = self.layers
        out = []
        for layer in from_layers:
            out.append(layer)
            out += self.get_all_layers(layer.children)
        return out

    # -- fusion ------------------------------------------------------------------------------------
    def _fuse_training(self):
        """BatchNormalization followed by Relu: the normalisation kernel applies the ReLU and the
        backward kernel applies its mask, so the activation tensor makes one HBM round trip fewer."""
        if self._train_fused:
            return
        def walk(seq):
            for a, b in zip(seq, seq[1:]):
                if self.enable_fused_bn_relu and isinstance(a, BatchNormalization) and isinstance(b, Relu):
                    a.fuse_relu, b.absorbed = True, True
                # Conv2D followed by BatchNormalization (training): the convolution's epilogue takes the batch sums, the
                # batch norm skips its own statistics pass over the tensor
                if self.fuse_conv_bn_stats and type(a).__name__ == "Conv2DGPU" and type(b).__name__ == "BatchNormalizationGPU" \
                        and getattr(a, "stats_bytes", 0) and b.spatial and self.dtype == np.float32 \
                        and self.tensor_format == PYDTNN_TENSOR_FORMAT_NHWC and _bn_fast_path(b.ci):
                    a.stats_for_bn = b
                    wsp.require_conv_stats(a.stats_bytes)
                # an addition block followed by a ReLU: the last residual sum writes max(sum, 0)
                # straight into the ReLU's output (same arithmetic, one pass over memory fewer)
                if self.fuse_add_relu and a.is_block_layer and len(a.paths) > 1 and isinstance(b, Relu) \
                        and type(a).__name__ == "AdditionBlockGPU":
                    a.relu_after, b.fed_by_block = b, True
                # a ReLU followed by an addition block: the block's input-gradient sum applies that ReLU's mask
                if self.fuse_add_relu and isinstance(a, Relu) and type(a).__name__ == "ReluGPU" and b.is_block_layer \
                        and len(b.paths) > 1 and type(b).__name__ == "AdditionBlockGPU" and a.need_dx \
                        and not getattr(a, "absorbed", False):
                    b.relu_before, a.bwd_by_block = a, True
            for layer in seq:
                for p in layer.paths:
                    walk(p)
        walk(self.layers)
        self._train_fused = True
        # an evaluation list built before these flags were set holds block copies without them
        self._eval_layers = None

    def _fuse_inference(self, seq):
        """Conv2D [+ BatchNormalization] [+ Relu] -> one convolution with a fused epilogue
        (the pass of pydtnn/model.py:294-349, applied to a copy of the layer list)."""
        out, i = [], 0
        while i < len(seq):
            cur = seq[i]
            nxt = seq[i + 1] if i + 1 < len(seq) else None
            nxt2 = seq[i + 2] if i + 2 < len(seq) else None
            plain_conv = isinstance(cur, Conv2D) and type(cur).__name__ == "Conv2DGPU"
            if plain_conv and self.enable_fused_conv_bn_relu and isinstance(nxt, BatchNormalization) and isinstance(nxt2, Relu):
                f = Conv2DBatchNormalizationRelu(from_parent=cur, from_parent_2=nxt)
                f.y = nxt2.y
                out.append(f); i += 3; continue
            if plain_conv and self.enable_fused_conv_bn and isinstance(nxt, BatchNormalization):
                f = Conv2DBatchNormalization(from_parent=cur, from_parent_2=nxt)
                f.y = nxt.y
                out.append(f); i += 2; continue
            if plain_conv and self.enable_fused_conv_relu and isinstance(nxt, Relu):
                f = Conv2DRelu(from_parent=cur)
                f.y = nxt.y
                out.append(f); i += 2; continue
            if cur.paths:
                import copy
                blk = copy.copy(cur)
                blk.paths = [self._fuse_inference(p) for p in cur.paths]
                out.append(blk); i += 1; continue
            out.append(cur); i += 1
        return out

    # -- steps ---------------------------------------------------------------------------------------
    def _ensure_loss(self):
        if self.loss_func is None:
            ncls = int(np.prod(self.layers[-1].shape))
            self.loss_func = CategoricalCrossEntropy((self.batch_size, ncls), self)
            self.y_batch = empty((self.batch_size,), np.int32)

    @staticmethod
    def _labels(y_batch):
        if isinstance(y_batch, torch.Tensor):
            return y_batch if y_batch.dim() == 1 else y_batch.argmax(dim=1)
        y_batch = np.asarray(y_batch)
        return y_batch if y_batch.ndim == 1 else np.argmax(y_batch, axis=1)

    def _upload(self, x_batch, y_batch):
        """Host -> device copy of one batch (pydtnn/model.py:457-462). Accepts NumPy arrays or
        (pinned) torch CPU tensors; labels may be integer class ids or one-hot rows."""
        xin = self.layers[0].y.ary
        if isinstance(x_batch, torch.Tensor):
            xin.t.copy_(x_batch.view(xin.t.shape), non_blocking=True)
        else:
            xin.set(x_batch)
        lab = self._labels(y_batch)
        if isinstance(lab, torch.Tensor):
            self.y_batch.t.copy_(lab.to(torch.int32), non_blocking=True)
        else:
            self.y_batch.set(lab.astype(np.int32))

    def forward_backward(self, global_batch_size=None):
        """Forward, loss, backward and gradient exchange on the batch already on the device."""
        self.mode = TRAIN_MODE
        self._fuse_training()
        if global_batch_size is None:
            global_batch_size = self.batch_size * self.nprocs
        tr = self.tracer
        x = self.layers[0].y
        for layer in self.layers[1:]:
            with tr.region(layer, tracer.PYDTNN_MDL_FORWARD):
                x = layer.forward(x)
        loss, dx = self.loss_func(x, self.y_batch, global_batch_size)
        if self.comm is not None:
            self.bucketer.reset()
        for layer in reversed(self.layers[1:]):
            with tr.region(layer, tracer.PYDTNN_MDL_BACKWARD):
                dx = layer.backward(dx)
            if not self.blocking_mpi:
                with tr.region(layer, tracer.PYDTNN_MDL_ALLREDUCE_DW):
                    layer.reduce_weights_async()
        if self.blocking_mpi:
            for layer in reversed(self.layers[1:]):
                with tr.region(layer, tracer.PYDTNN_MDL_ALLREDUCE_DW):
                    layer.reduce_weights_sync()
        self.join_side_stream()            # every gradient is ordered before whatever the caller does next on this stream
        return loss

    def apply_update(self, optimizer):
        tr = self.tracer
        self.join_side_stream()
        if self.comm is not None:
            self.bucketer.wait_all()
        if self.fast_update and hasattr(optimizer, "update_arena"):
            # one launch over the whole arena: booked on the first parameterised layer
            with tr.region(self.layers[1], tracer.PYDTNN_MDL_UPDATE_DW):
                optimizer.update_arena(self)
        else:
            for layer in reversed(self.layers[1:]):
                with tr.region(layer, tracer.PYDTNN_MDL_WAIT_DW):
                    layer.wait_allreduce_async()
                with tr.region(layer, tracer.PYDTNN_MDL_UPDATE_DW):
                    layer.update_weights(optimizer)

    def _stage_next(self, x_batch, y_batch=None):
        """Start the host -> device copy of the batch of the *next* step on a copy stream, into staging
        buffers, so that it runs under this step's kernels. Pinned torch CPU tensors only; ``y_batch`` is
        None for inference."""
        xin = self.layers[0].y.ary
        if self._stage is None:
            self._stage = {"x": torch.empty_like(xin.t), "y": None,
                           "stream": torch.cuda.Stream(device=xin.t.device), "ready": torch.cuda.Event(),
                           "free": torch.cuda.Event(), "batch": None}
            self._stage["free"].record()
        st = self._stage
        if y_batch is not None and st["y"] is None:
            st["y"] = torch.empty_like(self.y_batch.t)
        lab = self._labels(y_batch) if y_batch is not None else None
        with torch.cuda.stream(st["stream"]):
            st["stream"].wait_event(st["free"])           # the step that read the staging buffers has copied them out
            st["x"].copy_(x_batch.view(xin.t.shape), non_blocking=True)
            if lab is not None:
                st["y"].copy_(lab.to(torch.int32), non_blocking=True)
            st["ready"].record()
        st["batch"] = (x_batch, y_batch)

    def _take_staged(self, x_batch, y_batch=None):
        """If the staged batch is this one, move it from the staging buffers into the input (and label) buffers on
        the compute stream and return True."""
        st = self._stage
        if st is None or st["batch"] is None or st["batch"][0] is not x_batch or st["batch"][1] is not y_batch:
            return False
        cur = torch.cuda.current_stream()
        cur.wait_event(st["ready"])
        self.layers[0].y.ary.t.copy_(st["x"], non_blocking=True)
        if y_batch is not None:
            self.y_batch.t.copy_(st["y"], non_blocking=True)
        st["free"].record(cur)
        st["batch"] = None
        return True

    def train_batch(self, x_batch, y_batch, optimizer, global_batch_size=None, next_batch=None):
        """One training step on a host batch; returns the loss object (``.loss()``, ``.accuracy()``
        read the numbers back). ``next_batch=(x, y)`` (pinned torch CPU tensors) starts the upload of the
        following step's inputs under this step's kernels; the call that then passes those same tensors
        finds them on the device."""
        self._ensure_loss()
        if not self._take_staged(x_batch, y_batch):
            self._upload(x_batch, y_batch)
        if next_batch is not None and isinstance(next_batch[0], torch.Tensor):
            self._stage_next(*next_batch)
        loss = self.forward_backward(global_batch_size)
        self.apply_update(optimizer)
        return loss

    def train_epoch(self, x_data, y_data, optimizer, epoch=0, shuffle=True, rng=None):
        """One pass over host arrays (first axis = samples), the way the reference's training loop walks a data set
        (pydtnn/model.py:560-590): this rank's slices of every global batch (``datasets.batch_generator``), short last
        batches skipped, loss and accuracy read back after every step, times booked in ``perf_counter``.  The batch
        of step i + 1 is copied into pinned memory and uploaded while step i runs.  Returns the last step's
        (loss, accuracy), or None when the data hold no full batch."""
        import time
        from .datasets import PinnedFeeder, batch_generator
        gen = batch_generator(x_data, y_data, self.batch_size, self.rank, self.nprocs, shuffle, rng)
        feeder = PinnedFeeder(self, gen, wait_upload=lambda: self._stage is not None and self._stage["ready"].synchronize())
        last = None
        for x, y, global_bs, nxt in feeder:
            tic = time.perf_counter()
            loss = self.train_batch(x, y, optimizer, global_bs, next_batch=nxt)
            last = (loss.loss(), loss.accuracy())
            self.perf_counter.add_training_time_and_batch_size(epoch, time.perf_counter() - tic, global_bs)
        return last

    def evaluate_batch(self, x_batch, y_batch=None, next_batch=None):
        """Forward only, with the inference fusions that are switched on; returns the output handle
        (and the loss object when labels are given). ``next_batch`` (a pinned torch CPU tensor) starts the upload
        of the following call's input under this call's kernels, as in ``train_batch``."""
        self.mode = EVALUATE_MODE
        if self._eval_layers is None:
            self._fuse_training()          # the flags it sets (absorbed ReLUs, folded sums) are read in evaluation too
            self._eval_layers = self._fuse_inference(self.layers)
        if x_batch is not None:
            xin = self.layers[0].y.ary
            if isinstance(x_batch, torch.Tensor):
                if not self._take_staged(x_batch, None):
                    xin.t.copy_(x_batch.view(xin.t.shape), non_blocking=True)
            else:
                xin.set(x_batch)
        if isinstance(next_batch, torch.Tensor):
            self._stage_next(next_batch, None)
        x = self.layers[0].y
        for layer in self._eval_layers[1:]:
            x = layer.forward(x)
        if y_batch is None:
            return x
        self._ensure_loss()
        lab = self._labels(y_batch)
        self.y_batch.set(lab.astype(np.int32) if not isinstance(lab, torch.Tensor) else lab.cpu().numpy().astype(np.int32))
        loss, _ = self.loss_func(x, self.y_batch, self.batch_size * self.nprocs)
        return x, loss

    def store_weights_and_bias(self, filename, layout="cpu"):
        """Write the reference's NPZ checkpoint (pydtnn/model.py:380-384); see ``checkpoint.py`` for layouts."""
        from . import checkpoint
        self.synchronize()
        checkpoint.store_weights_and_bias(self, filename, layout)

    def load_weights_and_bias(self, filename, layout=None):
        """Read a checkpoint written by the reference or by ``store_weights_and_bias`` (pydtnn/model.py:376-378)."""
        from . import checkpoint
        missing = checkpoint.load_weights_and_bias(self, filename, layout)
        self._eval_layers = None          # fused inference layers fold the parameters they were built from
        return missing

    def synchronize(self):
        self.join_side_stream()
        self._synchronize()

    def _synchronize(self):
        """Wait for the device and raise ``B2CError`` (device timeout) if a bounded in-kernel wait ran out since the
        last check: the kernel then returned with partial results, which must not be trained on silently."""
        torch.cuda.synchronize(self.device)
        _lib.check(_lib.lib().b2c_check_device_status(None))
