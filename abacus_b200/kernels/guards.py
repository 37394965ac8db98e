"""Guard words around the buffers that kernels write: workspace, scratch areas, cache pools.

There is no memory checker to run the kernels under, so a store past the end of a buffer would go unseen until it
hit something that mattered. Every buffer made here has 256 bytes of a fixed pattern before and after it
(csrc/utility.cu); `check()` counts the words that no longer hold the pattern. The tests call it after every
GPU test, and bin/trace_run when its input ends. Checking costs two small launches per buffer and one read,
so nothing on the way of a step does it.
"""
import ctypes
import weakref

import torch

GUARD_BYTES = 256
_buffers = []  # (weak reference to the whole allocation, what it is for, bytes between the guards)


def _lib():
    from .build import load_module
    return load_module("utility")


def _stream():
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def empty(shape, dtype, device, what="", zero=False):
    """torch.empty(shape, dtype=dtype, device=device) with guard words around it (plain torch.empty off the GPU)."""
    device = torch.device(device)
    shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)))
    if device.type != "cuda":
        return torch.zeros(shape, dtype=dtype, device=device) if zero else torch.empty(shape, dtype=dtype, device=device)
    count = 1
    for s in shape:
        count *= s
    nbytes = count * torch.empty(0, dtype=dtype).element_size()
    room = -(-max(nbytes, 1) // GUARD_BYTES) * GUARD_BYTES
    whole = torch.empty(room + 2 * GUARD_BYTES, dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        lib = _lib()
        for offset in (0, GUARD_BYTES + room):
            rc = lib.abk_guard_fill(ctypes.c_void_p(whole.data_ptr() + offset), ctypes.c_int(GUARD_BYTES // 4), _stream())
            if rc:
                raise RuntimeError(f"guard words: CUDA error {rc}")
    inner = whole[GUARD_BYTES:GUARD_BYTES + nbytes]
    if zero:
        inner.zero_()
    _buffers.append((weakref.ref(whole), what, room))
    if len(_buffers) > 4096:
        _buffers[:] = [b for b in _buffers if b[0]() is not None]
    out = inner.view(dtype).view(shape)
    out.guarded_allocation = whole  # the allocation, guards included, lives as long as the tensor handed out
    return out


def zeros(shape, dtype, device, what=""):
    return empty(shape, dtype, device, what, zero=True)


def check(device=None):
    """How many guard words of the live buffers (of `device`, or of every GPU) no longer hold the pattern, and which
    buffers they belong to: (count, [what, ...]). Waits for the device."""
    damaged, where = 0, []
    for ref, what, room in list(_buffers):
        whole = ref()
        if whole is None or (device is not None and whole.device != torch.device(device)):
            continue
        with torch.cuda.device(whole.device):
            lib = _lib()
            word = torch.zeros(1, dtype=torch.int32, device=whole.device)
            for offset in (0, GUARD_BYTES + room):
                rc = lib.abk_guard_check(ctypes.c_void_p(whole.data_ptr() + offset), ctypes.c_int(GUARD_BYTES // 4),
                                         ctypes.c_void_p(word.data_ptr()), _stream())
                if rc:
                    raise RuntimeError(f"guard words: CUDA error {rc}")
            n = int(word.item())
        if n:
            damaged += n
            where.append(what or "a buffer")
    return damaged, where


def assert_intact(device=None):
    damaged, where = check(device)
    if damaged:
        raise RuntimeError(f"{damaged} guard words were overwritten around: {', '.join(where)}: a kernel stored outside "
                           "its buffer")
