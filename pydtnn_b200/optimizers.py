"""SGD with momentum (pydtnn/optimizers/sgd.py; update rule of
pydtnn/backends/cpu/optimizers/sgd_cpu.py:28-41 and pydtnn/backends/gpu/optimizers/sgd_gpu.py:40-47)."""
from . import _lib
from .tensor_gpu import zeros


class SGD:
    def __init__(self, learning_rate=1e-2, momentum=0.9, nesterov=False, decay=0.0, dtype=None):
        self.learning_rate = learning_rate
        self.momentum = momentum
        self.nesterov = nesterov
        self.decay = decay

    def update(self, layer):
        """Per-layer update, as the reference's ``optimizer.update(layer)``."""
        L = _lib.lib()
        m = layer.model
        for w_, dw_ in layer.grad_vars.items():
            w, dw = getattr(layer, w_), getattr(layer, dw_)
            vname = "velocity_%s" % w_
            if not hasattr(layer, vname):
                setattr(layer, vname, zeros(w.ary.shape, m.dtype))
            v = getattr(layer, vname)
            _lib.check(L.b2c_sgd_update(_lib.dtype_code(m.dtype), w.size, w.ptr, dw.ptr, v.gpudata,
                                        float(self.learning_rate), float(self.momentum), float(self.decay),
                                        int(self.nesterov), m.stream_handle))

    def update_arena(self, model):
        """One launch per arena buffer over all parameters at once (padding gaps stay zero)."""
        L = _lib.lib()
        arena = model.arena
        for ci, ch in enumerate(arena.chunks):
            v = arena.velocity(ci)
            _lib.check(L.b2c_sgd_update(_lib.dtype_code(model.dtype), ch.used, ch.w.data_ptr(), ch.dw.data_ptr(),
                                        v.data_ptr(), float(self.learning_rate), float(self.momentum),
                                        float(self.decay), int(self.nesterov), model.stream_handle))
