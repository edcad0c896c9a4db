"""Scratch buffers for the fused entry points (the C library never allocates).

The reference allocates its workspace inside every call (triteia/python/ops/matmul/sbmm.py:124-129),
so its ops are safe on any number of streams.  Here the working memory is cached, one buffer per
(device, stream): launches on one stream are ordered, so they can share a buffer; launches on
different streams get different buffers and may overlap.
"""
import torch

_buffers = {}
_retired = []   # outgrown buffers stay alive: a captured CUDA graph may still hold their address


def scratch(device, nbytes, stream=None):
    """A uint8 buffer of at least nbytes on `device` for work queued on `stream` (default: the
    current stream of the device), 256-byte aligned, reused by later calls on the same stream."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if stream is None:
        stream = torch.cuda.current_stream(device).cuda_stream
    key = (index, int(stream))
    buf = _buffers.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _retired.append(buf)
        buf = torch.empty(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
        _buffers[key] = buf
    return buf
