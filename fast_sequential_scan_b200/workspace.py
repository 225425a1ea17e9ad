"""Per-(device, stream) scratch for the native kernels, plus the host-visible status word.

The native library never allocates: the chunk summaries, tile descriptors and the epoch counter
of the single-pass kernels live in a device buffer that this module allocates with torch, zeroes
once with ``fss_workspace_init`` and then reuses for every launch on that stream (launches that
share a workspace must not overlap, which stream order guarantees).  The status word is one int
of pinned host memory the kernels write only when a bounded wait gives up; it is read without any
synchronisation at the start of every call and by :func:`check_status`.

One single-pass launch per device at a time
-------------------------------------------
A single-pass (look-back) launch sizes its grid to fill the idle device and needs all of its CTAs
resident at once: a tile may wait for a tile owned by a CTA that has not started yet.  Two such
launches on different streams can each be placed partially and then wait for one another until
their bounded waits run out (about a second; the status word reports it).  This module therefore
orders launches on different streams of one device: from the moment a second stream shows up on
a device, every launch records an event and a launch on another stream first waits for the event
of the launch before it.  A process that only ever uses one stream per device pays nothing for
this.  Kernels of other libraries that merely occupy SMs for a while (a collective, a GEMM on
another stream) only delay a launch; they cannot dead-lock it.
"""
from __future__ import annotations

import threading

import torch

from . import _lib

_lock = threading.Lock()
_cache: dict[tuple[int, int], "Workspace"] = {}
_devices: dict[int, "_DeviceOrder"] = {}


class _DeviceOrder:
    """Which stream launched last on a device, and -- once more than one stream is in play -- the
    event that marks the end of that launch."""
    __slots__ = ("last", "multi", "event")

    def __init__(self):
        self.last = None        # Workspace of the most recent launch
        self.multi = False      # a second stream has been seen on this device
        self.event = None       # torch.cuda.Event recorded after the most recent launch (multi only)


class Workspace:
    def __init__(self, device: torch.device, stream_handle: int):
        self.device = device
        self.stream_handle = stream_handle
        self.buf = None
        self.ctx = None          # the ScanCtx struct handed to the library (built by the caller)
        self.status = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._flag = self.status.numpy()      # same memory, read without going through torch
        self.order = _devices.setdefault(device.index, _DeviceOrder())
        self._event = None

    def stream(self) -> torch.cuda.Stream:
        return torch.cuda.ExternalStream(self.stream_handle, device=self.device)

    def ensure(self, nbytes: int) -> None:
        if self.buf is not None and self.buf.numel() >= nbytes:
            return
        # grow geometrically; a fresh buffer has to be zeroed before its first launch
        size = max(nbytes, 2 * (self.buf.numel() if self.buf is not None else 0), 1 << 16)
        self.buf = torch.empty(size, dtype=torch.uint8, device=self.device)
        self.ctx = None
        _lib.check(_lib.lib().fss_workspace_init(self.buf.data_ptr(), size, self.stream_handle),
                   "fss_workspace_init")

    def raise_if_flagged(self) -> None:
        code = int(self._flag[0])
        if code:
            self._flag[0] = 0
            if self.buf is not None:   # descriptors of the failed launch are not trustworthy
                _lib.check(_lib.lib().fss_workspace_init(self.buf.data_ptr(), self.buf.numel(),
                                                         self.stream_handle), "fss_workspace_init")
            raise RuntimeError("fss_b200 kernel reported: " + _lib.STATUS_TEXT.get(code, f"status {code}"))

    def order_after_other_streams(self) -> None:
        """Called before a launch: make this stream wait for the previous launch on the device when
        that launch went to another stream."""
        order = self.order
        last = order.last
        if last is self or last is None:
            return
        if torch.cuda.is_current_stream_capturing():
            return                       # a capture records one stream's work; ordering is the caller's
        if not order.multi:
            # first time two streams meet on this device: everything launched so far on the other
            # stream is fenced by one event recorded there now
            order.multi = True
            order.event = torch.cuda.Event()
            order.event.record(last.stream())
        if order.event is not None:
            self.stream().wait_event(order.event)


# torch.cuda.current_stream() builds a Stream object (several microseconds); the raw handle is all
# that is needed here
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def current_stream_handle(device: torch.device) -> int:
    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


def get(device: torch.device, nbytes: int) -> Workspace:
    """Workspace of the current stream of ``device``, at least ``nbytes`` large."""
    stream = current_stream_handle(device)
    key = (device.index, stream)
    ws = _cache.get(key)
    if ws is None:
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
            key = (device.index, stream)
        with _lock:
            ws = _cache.get(key)
            if ws is None:
                ws = _cache[key] = Workspace(device, stream)
    if ws._flag[0]:
        ws.raise_if_flagged()
    if ws.buf is None or ws.buf.numel() < nbytes:
        ws.ensure(nbytes)
    if ws.order.last is not ws:
        ws.order_after_other_streams()
    return ws


def launched(ws: Workspace) -> None:
    """Called after a launch on ``ws``'s stream."""
    order = ws.order
    order.last = ws
    if order.multi and not torch.cuda.is_current_stream_capturing():
        if ws._event is None:
            ws._event = torch.cuda.Event()
        ws._event.record(ws.stream())
        order.event = ws._event


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
        _devices.clear()
