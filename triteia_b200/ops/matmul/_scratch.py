"""Per-device scratch buffers for the fused entry points (the C library never allocates)."""
import torch

_buffers = {}


def scratch(device, nbytes):
    """A uint8 buffer of at least nbytes on `device`, 256-byte aligned, reused across calls.

    Calls on one device share it, so launches that use it must be ordered on one stream.
    """
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    buf = _buffers.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=device)
        _buffers[key] = buf
    return buf
