"""Per-(device, stream) scratch for the native kernels, plus the host-visible status word.

The native library never allocates: the chunk summaries, tile descriptors and the epoch counter
of the single-pass kernels live in a device buffer that this module allocates with torch, zeroes
once with ``fss_workspace_init`` and then reuses for every launch on that stream (launches that
share a workspace must not overlap, which stream order guarantees).  The status word is one int
of pinned host memory the kernels write only when a bounded wait gives up; it is read without any
synchronisation at the start of every call and by :func:`check_status`.
"""
from __future__ import annotations

import threading

import torch

from . import _lib

_lock = threading.Lock()
_cache: dict[tuple[int, int], "Workspace"] = {}


class Workspace:
    def __init__(self, device: torch.device, stream_handle: int):
        self.device = device
        self.stream_handle = stream_handle
        self.buf = None
        self.status = torch.zeros(1, dtype=torch.int32).pin_memory()

    def ensure(self, nbytes: int) -> None:
        if self.buf is not None and self.buf.numel() >= nbytes:
            return
        # grow geometrically; a fresh buffer has to be zeroed before its first launch
        size = max(nbytes, 2 * (self.buf.numel() if self.buf is not None else 0), 1 << 16)
        self.buf = torch.empty(size, dtype=torch.uint8, device=self.device)
        _lib.check(_lib.lib().fss_workspace_init(self.buf.data_ptr(), size, self.stream_handle),
                   "fss_workspace_init")

    def raise_if_flagged(self) -> None:
        code = int(self.status[0])
        if code:
            self.status[0] = 0
            if self.buf is not None:   # descriptors of the failed launch are not trustworthy
                _lib.check(_lib.lib().fss_workspace_init(self.buf.data_ptr(), self.buf.numel(),
                                                         self.stream_handle), "fss_workspace_init")
            raise RuntimeError("fss_b200 kernel reported: " + _lib.STATUS_TEXT.get(code, f"status {code}"))


def get(device: torch.device, nbytes: int) -> Workspace:
    """Workspace of the current stream of ``device``, at least ``nbytes`` large."""
    stream = torch.cuda.current_stream(device).cuda_stream
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream)
    with _lock:
        ws = _cache.get(key)
        if ws is None:
            ws = _cache[key] = Workspace(device, stream)
    ws.raise_if_flagged()
    ws.ensure(nbytes)
    return ws


def check_status(device=None) -> None:
    """Synchronise ``device`` and raise if any kernel on it reported a give-up."""
    torch.cuda.synchronize(device)
    with _lock:
        items = list(_cache.values())
    for ws in items:
        ws.raise_if_flagged()


def release_all() -> None:
    with _lock:
        _cache.clear()
