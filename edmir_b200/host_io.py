"""Launches on operands that live in pinned host memory.

The reference's operator takes host-resident tensors to the device, computes and brings the
result back on one stream (EDM-IR/ir/c-extension/mma.cu:168-265 allocates, copies in, runs,
synchronises and copies out inside the call).  On a PCIe-attached B200 the copies of a
tensor-parallel layer take several times longer than its GEMMs, so ``HostStaging`` keeps the two
copy directions and the kernels on three streams: the upload of the next operand, the kernels of
the current one and the download of the previous result overlap, and the two PCIe directions run
at the same time.  Ordering is by events only; nothing blocks the host.

    io = HostStaging()
    for op in layer:                       # any number of times
        io.run(op.a_host, op.a_dev, lambda: launch(op), op.out_dev, op.out_host)
    io.drain()                             # the caller's stream now waits for every download

Hazards covered: a device operand is not overwritten by the next upload before the launch that
reads it has finished (nor, the first time a buffer is seen, before earlier work on the caller's
stream has); a device result is not overwritten by the next launch before its download has
finished.  The device buffers belong to the caller for as long as copies of them may be in flight:
free or reuse them elsewhere only after a ``drain()`` and a synchronisation of the current stream.  Host buffers belong to the caller, who must not touch ``out_host`` before a
``drain()`` followed by a synchronisation of the current stream, nor rewrite ``a_host`` before
the upload that reads it has run (``drain()`` also covers the uploads issued so far).
"""
from __future__ import annotations

from typing import Callable

import torch


class HostStaging:
    def __init__(self, device=None):
        if not torch.cuda.is_available():
            raise RuntimeError("HostStaging needs a CUDA device (there is no CPU path)")
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.up = torch.cuda.Stream(self.device)
        self.down = torch.cuda.Stream(self.device)
        self._read_done: dict[int, torch.cuda.Event] = {}      # device operand -> its last reader finished
        self._download_done: dict[int, torch.cuda.Event] = {}  # device result -> its last download finished
        self._last_upload: torch.cuda.Event | None = None

    def run(self, a_host: torch.Tensor, a_dev: torch.Tensor, launch: Callable[[], object],
            out_dev: torch.Tensor, out_host: torch.Tensor) -> None:
        """Upload ``a_host`` into ``a_dev``, call ``launch()`` (which enqueues kernels reading
        ``a_dev`` and writing ``out_dev`` on the current stream), download ``out_dev`` into
        ``out_host``.  Returns as soon as everything is enqueued."""
        if not (a_host.is_pinned() and out_host.is_pinned()):
            raise ValueError("host buffers must be pinned, or the copies cannot overlap anything")
        if a_host.shape != a_dev.shape or out_host.shape != out_dev.shape:
            raise ValueError("host and device buffers must have the same shapes")
        cur = torch.cuda.current_stream(self.device)
        # upload: after the previous reader of a_dev that went through this object; a buffer seen
        # for the first time may still be in use by earlier work on the caller's stream
        ev = self._read_done.get(a_dev.data_ptr())
        if ev is not None:
            self.up.wait_event(ev)
        else:
            self.up.wait_stream(cur)
        with torch.cuda.stream(self.up):
            a_dev.copy_(a_host, non_blocking=True)
            uploaded = torch.cuda.Event()
            uploaded.record(self.up)
        self._last_upload = uploaded
        # kernels: after the upload and after the previous download of out_dev
        cur.wait_event(uploaded)
        ev = self._download_done.get(out_dev.data_ptr())
        if ev is not None:
            cur.wait_event(ev)
        launch()
        computed = torch.cuda.Event()
        computed.record(cur)
        self._read_done[a_dev.data_ptr()] = computed
        # download
        self.down.wait_event(computed)
        with torch.cuda.stream(self.down):
            out_host.copy_(out_dev, non_blocking=True)
            downloaded = torch.cuda.Event()
            downloaded.record(self.down)
        self._download_done[out_dev.data_ptr()] = downloaded

    def drain(self) -> None:
        """Make the current stream wait for every copy issued so far (no host-side blocking)."""
        cur = torch.cuda.current_stream(self.device)
        for ev in self._download_done.values():
            cur.wait_event(ev)
        if self._last_upload is not None:
            cur.wait_event(self._last_upload)
        # forget buffers whose last use has already completed (the maps would otherwise grow with
        # every distinct buffer ever passed in)
        for table in (self._read_done, self._download_done):
            for key in [k for k, ev in table.items() if ev.query()]:
                del table[key]
