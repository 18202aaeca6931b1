"""One process-wide scratch buffer shared by every convolution/FC call, grown on demand while
layers are being initialised -- the role of the reference's shared cuDNN workspace
(pydtnn/backends/gpu/layers/memory_allocation.py:28-49).  All kernels of a process run on one
stream, so sharing is safe; the library itself never allocates."""
import torch

_buf = None


def require(nbytes, device=None):
    """Make sure the shared workspace holds at least ``nbytes`` (call at initialise time)."""
    global _buf
    nbytes = int(nbytes)
    if _buf is None or _buf.numel() < nbytes or (device is not None and _buf.device != torch.device(device)):
        device = device or (_buf.device if _buf is not None else torch.device("cuda", torch.cuda.current_device()))
        _buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
    return _buf


def ptr():
    return _buf.data_ptr() if _buf is not None else 0


def size():
    return _buf.numel() if _buf is not None else 0


_side = None


def require_side(nbytes, device=None):
    """A second workspace of the same kind for calls issued on the model's side stream (weight gradients that run
    next to the main stream's kernels must not share scratch with them)."""
    global _side
    nbytes = int(nbytes)
    if _side is None or _side.numel() < nbytes:
        device = device or (_side.device if _side is not None else torch.device("cuda", torch.cuda.current_device()))
        _side = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
    return _side


def side():
    return _side


_red = None


def require_reduction_scratch(channels, device=None):
    """Shared scratch (doubles) for per-channel reductions (batch norm statistics and gradients):
    two doubles per channel and row chunk, enough chunks for about four CTAs per SM."""
    global _red
    gx = max(1, channels // 256)
    chunks = max(64, (592 + gx - 1) // gx)
    need = 2 * channels * chunks
    if _red is None or _red.numel() < need:
        device = device or (_red.device if _red is not None else torch.device("cuda", torch.cuda.current_device()))
        _red = torch.empty(need, dtype=torch.float64, device=device)
    return _red


def reduction_scratch():
    return _red


_stats = None


def require_conv_stats(nbytes, device=None):
    """Shared buffer for the batch statistics a convolution leaves for the batch norm that follows it (consumed
    before the next convolution runs, so one buffer serves every Conv2D -> BatchNormalization pair)."""
    global _stats
    nbytes = int(nbytes)
    if _stats is None or _stats.numel() < nbytes:
        device = device or (_stats.device if _stats is not None else torch.device("cuda", torch.cuda.current_device()))
        _stats = torch.empty(nbytes, dtype=torch.uint8, device=device)
    return _stats


def conv_stats():
    return _stats
