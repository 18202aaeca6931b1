"""Whole-step parity through the Layer / Model API: a small ResNet (conv, BN, ReLU, pooling,
addition blocks, FC, softmax, cross-entropy, SGD) against its CPU-oracle twin, layer by layer --
the pattern of the reference's CheckGPUModels (pydtnn/tests/check_gpu_models.py:109-146). GPU."""
import numpy as np
import pytest

from tests.gpu_util import rel_l2 as _rel_l2
from tests.model_util import cpu_twin, grads_of, params_of, walk_pairs

pytestmark = pytest.mark.gpu


def rel_l2(got, ref):
    """Relative L2 error, zero when the absolute error is below a floor: gradients that are
    analytically zero (the bias of a convolution that feeds a batch normalisation) are rounding
    noise on both sides."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    err = np.linalg.norm(got - ref)
    if err <= (1e-5 if _NOISE["f32"] else 1e-12) * np.sqrt(ref.size):
        return 0.0
    return err / max(np.linalg.norm(ref), 1e-300)


_NOISE = {"f32": False}


def _small_resnet(layout, dtype, batch=4, **kw):
    from pydtnn_b200 import nets
    from pydtnn_b200.model import Model
    np.random.seed(0)
    model = Model(batch_size=batch, tensor_format=layout, dtype=dtype, **kw)
    nets.create_resnet50_imagenet(model, input_hw=32, nclasses=10, layout=[[8, 2, 1], [16, 2, 2]])
    return model


def _batch(model, seed=0):
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.standard_normal((model.batch_size, *model.layers[0].shape)).astype(model.dtype)
    labels = rng.integers(0, 10, model.batch_size)
    return x, labels


@pytest.mark.parametrize("layout,dtype,fused", [("NHWC", "float64", False), ("NCHW", "float64", False),
                                                ("NHWC", "float32", False), ("NCHW", "float32", False),
                                                ("NHWC", "float64", True), ("NHWC", "float32", True)])
def test_train_step_matches_cpu_twin(layout, dtype, fused):
    from pydtnn_b200.optimizers import SGD
    model = _small_resnet(layout, np.dtype(dtype).type, enable_fused_bn_relu=fused)
    net = cpu_twin(model)
    nchw = layout == "NCHW"
    tol = 1e-10 if dtype == "float64" else 2e-4
    _NOISE["f32"] = dtype == "float32"
    opt = SGD(learning_rate=0.05, momentum=0.9)
    for step in range(2):
        x, labels = _batch(model, step)
        loss_obj = model.train_batch(x, labels, opt)
        model.synchronize()
        probs = net.forward(x, True)
        loss_ref, d = net.loss_and_grad(probs, labels, model.batch_size)
        net.backward(d)
        assert abs(loss_obj.loss() - loss_ref) <= tol * max(1.0, abs(loss_ref))
        # activations of the top-level layers (absorbed ReLUs return their input's buffer)
        for i, layer in enumerate(model.layers[1:]):
            if layer.canonical_name in ("Flatten",) or getattr(layer, "absorbed", False) \
                    or getattr(layer, "relu_after", None) is not None:
                continue        # views, and blocks whose sum lands directly in the following ReLU
            got = layer.y.ary.get().reshape(net.acts[i + 1].shape)
            assert rel_l2(got, net.acts[i + 1]) <= tol, f"step {step} y of {layer}"
        for layer, node in walk_pairs(model.layers[1:], net.nodes):
            for k, g in grads_of(layer, nchw).items():
                ref = getattr(node, k)
                assert rel_l2(g.reshape(ref.shape), ref) <= tol, f"step {step} {k} of {layer}"
        net.sgd(0.05, 0.9)
        for layer, node in walk_pairs(model.layers[1:], net.nodes):
            for k, p in params_of(layer, nchw).items():
                ref = getattr(node, k)
                assert rel_l2(p.reshape(ref.shape), ref) <= tol, f"step {step} param {k} of {layer}"


def test_per_layer_update_equals_arena_update():
    from pydtnn_b200.optimizers import SGD
    a = _small_resnet("NHWC", np.float32)
    b = _small_resnet("NHWC", np.float32)
    b.fast_update = False
    oa, ob = SGD(0.05, 0.9, decay=1e-4), SGD(0.05, 0.9, decay=1e-4)
    for step in range(2):
        x, labels = _batch(a, step)
        a.train_batch(x, labels, oa)
        b.train_batch(x, labels, ob)
    for la, lb in zip(a.get_all_layers(), b.get_all_layers()):
        for k in la.grad_vars:
            assert np.array_equal(getattr(la, k).ary.get(), getattr(lb, k).ary.get()), (la, k)


def test_residual_sum_folded_into_the_last_batch_norm_is_bit_identical():
    """AdditionBlock + ReLU: the last batch norm of the first branch adds the other branch and applies the ReLU
    while it writes; the steps must equal the ones with the separate add+ReLU kernel bit for bit."""
    from pydtnn_b200.optimizers import SGD
    a = _small_resnet("NHWC", np.float32, enable_fused_bn_relu=True)
    b = _small_resnet("NHWC", np.float32, enable_fused_bn_relu=True)
    blocks = [l for l in b.layers if type(l).__name__ == "AdditionBlockGPU"]
    assert blocks
    for blk in blocks:
        blk.fold_sum = False
    # c: no block-level fusion at all (separate add, ReLU forward and ReLU backward kernels)
    c = _small_resnet("NHWC", np.float32, enable_fused_bn_relu=True)
    c.fuse_add_relu = False
    oa, ob, oc = SGD(0.05, 0.9), SGD(0.05, 0.9), SGD(0.05, 0.9)
    for step in range(2):
        x, labels = _batch(a, step)
        la, lb, lc = a.train_batch(x, labels, oa), b.train_batch(x, labels, ob), c.train_batch(x, labels, oc)
        assert la.loss() == lb.loss() == lc.loss()
    assert any(getattr(l, "relu_before", None) is not None for l in a.layers)
    assert all(getattr(l, "relu_before", None) is None for l in c.layers)
    for pa, pb, pc in zip(a.get_all_layers(), b.get_all_layers(), c.get_all_layers()):
        for k in pa.grad_vars:
            ga = getattr(pa, k).ary.get()
            assert np.array_equal(ga, getattr(pb, k).ary.get()), (pa, k)
            assert np.array_equal(ga, getattr(pc, k).ary.get()), (pa, k)


def test_step_tracer_books_every_layer_once_per_step(tmp_path):
    from pydtnn_b200 import tracer as tr
    from pydtnn_b200.optimizers import SGD
    m = _small_resnet("NHWC", np.float32)
    opt = SGD(0.05, 0.9)
    x, labels = _batch(m, 0)
    m.train_batch(x, labels, opt)                 # untraced
    m.tracer.enable_tracing()
    for step in range(2):
        m.train_batch(x, labels, opt)
    m.tracer.disable_tracing()
    m.synchronize()
    s = m.tracer.summary()
    for layer in m.layers[1:]:
        for kind in (tr.PYDTNN_MDL_FORWARD, tr.PYDTNN_MDL_BACKWARD):
            name, calls, total, median = s[tr.event_value(layer.id, kind)]
            assert calls == 2 and total >= 0.0 and name.startswith(f"{layer.id}_")
    out = tmp_path / "trace.csv"
    m.tracer.write_output(out)
    assert out.read_text().splitlines()[0].startswith("Event type;Event value;Event name")


def test_staged_upload_of_the_next_batch_gives_the_same_steps():
    """``train_batch(..., next_batch=...)`` uploads the following step's pinned batch on a copy stream; the
    three steps must be bit-identical to plain uploads."""
    import torch
    from pydtnn_b200.optimizers import SGD
    a = _small_resnet("NHWC", np.float32)
    b = _small_resnet("NHWC", np.float32)
    oa, ob = SGD(0.05, 0.9), SGD(0.05, 0.9)
    batches = []
    for step in range(3):
        x, labels = _batch(a, step)
        batches.append((torch.from_numpy(x).pin_memory(), torch.from_numpy(labels.astype(np.int32)).pin_memory()))
    for step in range(3):
        nxt = batches[step + 1] if step + 1 < 3 else None
        la = a.train_batch(*batches[step], oa, next_batch=nxt)
        lb = b.train_batch(*batches[step], ob)
        assert la.loss() == lb.loss()
    for pa, pb in zip(a.get_all_layers(), b.get_all_layers()):
        for k in pa.grad_vars:
            assert np.array_equal(getattr(pa, k).ary.get(), getattr(pb, k).ary.get()), (pa, k)


def test_staged_upload_in_evaluation_gives_the_same_outputs():
    """``evaluate_batch(x, next_batch=...)`` uploads the following call's pinned input on a copy stream; outputs
    must be bit-identical to plain uploads, for a sequence of different batches."""
    import torch
    a = _small_resnet("NHWC", np.float32)
    b = _small_resnet("NHWC", np.float32)
    xs = [torch.from_numpy(_batch(a, step)[0]).pin_memory() for step in range(4)]
    for step in range(4):
        nxt = xs[step + 1] if step + 1 < 4 else None
        ya = a.evaluate_batch(xs[step], next_batch=nxt).ary.get()
        yb = b.evaluate_batch(xs[step]).ary.get()
        assert np.array_equal(ya, yb), step
    # a staged batch that is not the one passed next is ignored
    a.evaluate_batch(xs[0], next_batch=xs[1])
    assert np.array_equal(a.evaluate_batch(xs[2]).ary.get(), b.evaluate_batch(xs[2]).ary.get())


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
def test_inference_fusion_matches_unfused_chain(layout):
    """Conv+BN+ReLU / Conv+BN folded into the convolution epilogue for evaluation: same output as
    the un-fused chain on the CPU oracle, after a training step has moved the running statistics."""
    from pydtnn_b200.optimizers import SGD
    model = _small_resnet(layout, np.float32, enable_fused_conv_bn_relu=True, enable_fused_conv_bn=True,
                          enable_fused_conv_relu=True)
    net = cpu_twin(model)
    opt = SGD(learning_rate=0.0, momentum=0.0)
    x, labels = _batch(model, 3)
    model.train_batch(x, labels, opt)          # lr 0: only the running statistics change
    net.forward(x, True)
    y = model.evaluate_batch(x)
    model.synchronize()
    fused_names = [type(l).__name__ for l in model._eval_layers] + \
                  [type(l).__name__ for blk in model._eval_layers for p in blk.paths for l in p]
    assert "Conv2DBatchNormalizationReluGPU" in fused_names and "Conv2DBatchNormalizationGPU" in fused_names
    ref = net.forward(x, False)
    assert rel_l2(y.ary.get(), ref) <= 2e-4


@pytest.mark.parametrize("layout", ["NCHW", "NHWC"])
def test_alexnet_style_inference_with_fused_conv_relu(layout):
    """The AlexNet recipe at small size (11x11 stride-4 stem, 5x5 and 3x3 convolutions with their ReLU folded
    into the convolution epilogue, 3x3 stride-2 max pools, three FC layers, dropout as identity) in evaluation
    mode against the CPU oracle chain; inputs are uint8 pixels scaled by 1/255."""
    from pydtnn_b200.layers import FC, Conv2D, Dropout, Flatten, Input, MaxPool2D
    from pydtnn_b200.model import Model
    np.random.seed(1)
    m = Model(batch_size=4, tensor_format=layout, dtype=np.float32, enable_fused_conv_relu=True)
    m.add(Input(shape=(67, 67, 3)))
    m.add(Conv2D(nfilters=32, filter_shape=(11, 11), padding=0, stride=4, activation="relu", weights_initializer="he_uniform"))
    m.add(MaxPool2D(pool_shape=(3, 3), stride=2))
    m.add(Conv2D(nfilters=64, filter_shape=(5, 5), padding=2, stride=1, activation="relu", weights_initializer="he_uniform"))
    m.add(MaxPool2D(pool_shape=(3, 3), stride=2))
    m.add(Conv2D(nfilters=96, filter_shape=(3, 3), padding=1, stride=1, activation="relu", weights_initializer="he_uniform"))
    m.add(Conv2D(nfilters=64, filter_shape=(3, 3), padding=1, stride=1, activation="relu", weights_initializer="he_uniform"))
    m.add(MaxPool2D(pool_shape=(3, 3), stride=2))
    m.add(Flatten())
    m.add(FC(shape=(64,), activation="relu", weights_initializer="he_uniform"))
    m.add(Dropout(rate=0.5))
    m.add(FC(shape=(10,), activation="softmax", weights_initializer="he_uniform"))
    net = cpu_twin(m)
    rng = np.random.Generator(np.random.PCG64(9))
    shape = (4, 67, 67, 3) if layout == "NHWC" else (4, 3, 67, 67)
    x = (rng.integers(0, 256, shape).astype(np.uint8) / 255.0).astype(np.float32)
    y = m.evaluate_batch(x)
    m.synchronize()
    names = [type(l).__name__ for l in m._eval_layers]
    assert names.count("Conv2DReluGPU") == 4 and "Conv2DGPU" not in names
    ref = net.forward(x, False)
    assert _rel_l2(y.ary.get(), ref) <= 1e-5


def test_evaluate_train_evaluate_matches_a_fresh_model():
    """Evaluation before the first training step builds the fused evaluation list early; the training fusion pass
    then changes flags on blocks and ReLUs that list shares.  Evaluating again must give what a model that only
    trained and then evaluated gives, bit for bit."""
    from pydtnn_b200.optimizers import SGD
    kw = dict(enable_fused_bn_relu=True, enable_fused_conv_bn=True, enable_fused_conv_bn_relu=True)
    a = _small_resnet("NHWC", np.float32, **kw)
    b = _small_resnet("NHWC", np.float32, **kw)
    oa, ob = SGD(0.0, 0.0), SGD(0.0, 0.0)       # lr 0: only the running statistics change
    net = cpu_twin(b)
    x, labels = _batch(a, 0)
    x2, _ = _batch(a, 1)
    a.evaluate_batch(x2)                        # builds a's evaluation list before any training
    a.train_batch(x, labels, oa)
    b.train_batch(x, labels, ob)
    net.forward(x, True)
    ya = a.evaluate_batch(x2).ary.get()
    yb = b.evaluate_batch(x2).ary.get()
    a.synchronize()
    assert np.array_equal(ya, yb)
    # and against the un-fused CPU chain
    _NOISE["f32"] = True
    assert rel_l2(yb, net.forward(x2, False)) <= 2e-4


@pytest.mark.parametrize("flags", [dict(enable_fused_bn_relu=True, enable_fused_conv_bn=True),
                                   dict(enable_fused_bn_relu=True, enable_fused_conv_bn=True, enable_fused_conv_relu=True),
                                   dict(enable_fused_bn_relu=True)])
def test_inference_after_training_fusion_keeps_every_relu(flags):
    """Training-mode BN+ReLU fusion marks the ReLU as absorbed by its batch norm; an inference pass that folds
    Conv+BN (without the +ReLU variant switched on) must still apply that ReLU."""
    from pydtnn_b200.optimizers import SGD
    model = _small_resnet("NHWC", np.float32, **flags)
    opt = SGD(learning_rate=0.0, momentum=0.0)
    x, labels = _batch(model, 3)
    model.train_batch(x, labels, opt)          # lr 0: only the running statistics change
    net = cpu_twin(model)
    net.forward(x, True)                       # moves the twin's running statistics the same way
    y = model.evaluate_batch(x)
    model.synchronize()
    _NOISE["f32"] = True
    assert rel_l2(y.ary.get(), net.forward(x, False)) <= 2e-4


def test_loss_and_accuracy_totals_match_the_row_values():
    """``loss()`` / ``accuracy()`` read two doubles summed on the device; they must equal the host-side sums of
    the per-row values the same kernel wrote."""
    from pydtnn_b200.optimizers import SGD
    m = _small_resnet("NHWC", np.float32)
    x, labels = _batch(m, 0)
    lo = m.train_batch(x, labels, SGD(0.05, 0.9))
    rows = lo.row_loss.get().astype(np.float64)
    hits = lo.hit.get()
    assert abs(lo.loss() - (-rows.sum() / m.batch_size)) <= 1e-12
    assert abs(lo.accuracy() - hits.sum() * 100.0 / m.batch_size) <= 1e-12
    assert lo.local_loss() == -rows.sum() / m.batch_size


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from pydtnn_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(_lib.B2CError):
        _lib.lib()


def test_train_epoch_feeds_rank_slices_through_pinned_buffers():
    """``train_epoch`` (rank-sliced batches, pinned double buffering, upload of the next batch under the running step)
    against a plain loop over the same slices: same weights bit for bit, the short last batch skipped, every step
    booked in the performance counter."""
    from pydtnn_b200.datasets import batch_generator
    from pydtnn_b200.optimizers import SGD
    a = _small_resnet("NHWC", np.float32)
    b = _small_resnet("NHWC", np.float32)
    rng = np.random.Generator(np.random.PCG64(11))
    n = 4 * 5 + 3                                        # five full batches and a short one
    x = rng.standard_normal((n, *a.layers[0].shape)).astype(np.float32)
    y = rng.integers(0, 10, n)
    oa, ob = SGD(0.05, 0.9), SGD(0.05, 0.9)
    last = a.train_epoch(x, y, oa, epoch=0, shuffle=True, rng=np.random.Generator(np.random.PCG64(5)))
    steps = 0
    for xb, yb, gbs in batch_generator(x, y, 4, 0, 1, True, np.random.Generator(np.random.PCG64(5))):
        if xb.shape[0] != 4:
            continue
        lb = b.train_batch(xb, yb, ob, gbs)
        steps += 1
    assert steps == 5 and last is not None and last[0] == lb.loss()
    assert a.perf_counter.num_epochs == 1 and a.perf_counter.training_throughput > 0
    for pa, pb in zip(a.get_all_layers(), b.get_all_layers()):
        for k in pa.grad_vars:
            assert np.array_equal(getattr(pa, k).ary.get(), getattr(pb, k).ary.get()), (pa, k)


def test_per_operation_events_of_conv_and_fc_layers():
    from pydtnn_b200 import tracer as tr
    from pydtnn_b200.optimizers import SGD
    m = _small_resnet("NHWC", np.float32)
    opt = SGD(0.05, 0.9)
    x, labels = _batch(m, 0)
    m.train_batch(x, labels, opt)
    m.tracer.enable_tracing(ops=True)
    m.train_batch(x, labels, opt)
    m.tracer.disable_tracing()
    m.synchronize()
    ops = m.tracer.ops_summary()
    convs = [l for l in m.get_all_layers() if type(l).__name__ == "Conv2DGPU"]
    fcs = [l for l in m.get_all_layers() if type(l).__name__ == "FCGPU"]
    assert convs and fcs
    for l in convs:
        assert ops[tr.ops_event_value(l.id, tr.PYDTNN_OPS_FORWARD_CUDNN)][1] == 1
        assert ops[tr.ops_event_value(l.id, tr.PYDTNN_OPS_BACKWARD_CUDNN_DW)][1] == 1
        assert (tr.ops_event_value(l.id, tr.PYDTNN_OPS_BACKWARD_CUDNN_DX) in ops) == bool(l.need_dx)
    for l in fcs:
        assert ops[tr.ops_event_value(l.id, tr.PYDTNN_OPS_FORWARD_CUBLAS_MATMUL)][1] == 1
        assert ops[tr.ops_event_value(l.id, tr.PYDTNN_OPS_BACKWARD_CUBLAS_MATMUL_DW)][1] == 1
