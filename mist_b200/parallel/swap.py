"""Host offloading over the copy engines: pinned buffers, split device/host tensors and
activation swapping through autograd's saved-tensor hooks.

Everything here is ``cudaMemcpyAsync`` between device memory and pinned host memory on
two dedicated streams (one per direction), ordered against the compute stream with
events; no SM time is spent on the copies (reference: mist/re_swap_manager/
swap_backend.py:113-169 ``swap_``, :172-513 TensorSwapHandle, :516-567; activation hooks
mist/re_swap_manager/manager.py:525-710 with the 1 Mi element threshold at :49,634,676).
The two-slot rings of full weights and of gradient buckets (reference: mist/re_swap_manager/
mem_buffer_pool.py:60-195) are plain tensors owned by the training engine.
"""
from __future__ import annotations

import weakref
from typing import Dict, Optional

import torch

ACTIVATION_SWAP_MIN_NUMEL = 1 << 20   # smaller saved tensors stay on the device


class SwapStreams:
    """The two copy streams of a rank (created lazily; CPU runs use none)."""

    def __init__(self, device):
        self.cuda = torch.device(device).type == "cuda"
        self.h2d = torch.cuda.Stream() if self.cuda else None
        self.d2h = torch.cuda.Stream() if self.cuda else None


class SplitTensor:
    """A flat tensor whose leading part lives on the device and whose trailing ``ratio`` lives
    in pinned host memory.  ``load`` brings the host part into a staging buffer so a kernel
    can work on ``(device_part, staged_part)``; ``store`` writes the staged part back."""

    def __init__(self, full: torch.Tensor, ratio: float, align: int = 256):
        n = full.numel()
        host_n = int(n * ratio) // align * align
        self.numel, self.host_numel, self.dev_numel = n, host_n, n - host_n
        self.device_part = full[: self.dev_numel].clone() if self.dev_numel < n else full
        self.host_part = None
        if host_n:
            # allocate pinned memory once and copy straight into it (no pageable staging copy)
            self.host_part = torch.empty(host_n, dtype=full.dtype, device="cpu", pin_memory=torch.cuda.is_available())
            self.host_part.copy_(full[self.dev_numel:].detach())
        self.dtype, self.device = full.dtype, full.device

    def load(self, staging: torch.Tensor, streams: SwapStreams) -> Optional[torch.Tensor]:
        if not self.host_numel:
            return None
        dst = staging[: self.host_numel]
        if streams.cuda:
            with torch.cuda.stream(streams.h2d):
                dst.copy_(self.host_part, non_blocking=True)
        else:
            dst.copy_(self.host_part)
        return dst

    def store(self, staged: torch.Tensor, streams: SwapStreams):
        if not self.host_numel:
            return
        if streams.cuda:
            with torch.cuda.stream(streams.d2h):
                self.host_part.copy_(staged[: self.host_numel], non_blocking=True)
        else:
            self.host_part.copy_(staged[: self.host_numel])

    def load_into(self, dst: torch.Tensor, streams: SwapStreams):
        """Assembles the whole tensor in ``dst`` (device): the device part with a copy on the
        current stream, the host part over the host->device stream, which the current stream
        then waits for.  The host->device stream first waits for the current stream (``dst``
        may still be read by earlier work) and for pending stores of this tensor."""
        dst[: self.dev_numel].copy_(self.device_part)
        if not self.host_numel:
            return
        tail = dst[self.dev_numel: self.numel]
        if streams.cuda:
            cur = torch.cuda.current_stream()
            streams.h2d.wait_stream(cur)
            streams.h2d.wait_stream(streams.d2h)
            with torch.cuda.stream(streams.h2d):
                tail.copy_(self.host_part, non_blocking=True)
            cur.wait_stream(streams.h2d)
        else:
            tail.copy_(self.host_part)

    def store_from(self, src: torch.Tensor, streams: SwapStreams):
        """Writes a whole device tensor back: leading part to the device part, the rest to the
        host over the device->host stream (ordered after the current stream).  The caller must
        not overwrite ``src`` before the device->host stream has passed this point."""
        self.device_part.copy_(src[: self.dev_numel])
        if not self.host_numel:
            return
        tail = src[self.dev_numel: self.numel]
        if streams.cuda:
            streams.d2h.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(streams.d2h):
                self.host_part.copy_(tail, non_blocking=True)
        else:
            self.host_part.copy_(tail)

    def full(self) -> torch.Tensor:
        """Materialises the whole tensor on the device (checkpointing, tests)."""
        if not self.host_numel:
            return self.device_part
        return torch.cat([self.device_part, self.host_part.to(self.device)])


class ActivationSwapper:
    """Saved-tensor hooks that move a fraction of the saved activation bytes to the host.

    Whole tensors are swapped (no splitting): a tensor goes to the host while the bytes
    swapped so far are below ``ratio`` of the bytes seen so far in this scope.  ``prefetch``
    starts the host->device copies of a scope ahead of its backward pass."""

    def __init__(self, ratio: float, streams: SwapStreams, min_numel: int = ACTIVATION_SWAP_MIN_NUMEL):
        self.ratio, self.streams, self.min_numel = float(ratio), streams, int(min_numel)
        self.scope = None
        self._seen: Dict = {}
        self._swapped: Dict = {}
        self._handles: Dict = {}      # scope -> list of handle dicts
        self._pool: Dict = {}         # (shape, dtype) -> free pinned host buffers (reused every iteration)
        self.bytes_out = 0
        self.bytes_in = 0

    def set_scope(self, scope):
        self.scope = scope

    # ------------------------------------------------------------------ autograd hooks
    def pack(self, t: torch.Tensor):
        if (self.ratio <= 0 or not isinstance(t, torch.Tensor) or t.numel() < self.min_numel
                or isinstance(t, torch.nn.Parameter) or not t.is_floating_point() or t.device.type == "cpu"
                and self.streams.cuda):
            return t
        sc = self.scope
        nb = t.numel() * t.element_size()
        seen = self._seen.get(sc, 0) + nb
        swapped = self._swapped.get(sc, 0)
        self._seen[sc] = seen
        if swapped + nb > self.ratio * seen + 1:
            return t
        self._swapped[sc] = swapped + nb
        free = self._pool.get((tuple(t.shape), t.dtype))
        reuse_after = None
        if free:
            host, reuse_after = free.pop()     # its last host->device copy must finish before it is rewritten
        else:
            host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=self.streams.cuda)
        h = {"host": host, "shape": t.shape, "dtype": t.dtype, "device": t.device, "gpu": None, "event": None}
        src = t if t.is_contiguous() else t.contiguous()
        if self.streams.cuda:
            self.streams.d2h.wait_stream(torch.cuda.current_stream())
            if reuse_after is not None:
                self.streams.d2h.wait_event(reuse_after)
            with torch.cuda.stream(self.streams.d2h):
                host.copy_(src, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
            src.record_stream(self.streams.d2h)
            h["out_event"] = ev
        else:
            host.copy_(src)
        self.bytes_out += nb
        self._handles.setdefault(sc, []).append(h)
        return ("swapped", h)

    def _fetch(self, h):
        if h["gpu"] is not None:
            return
        if self.streams.cuda:
            with torch.cuda.stream(self.streams.h2d):
                if h.get("out_event") is not None:
                    self.streams.h2d.wait_event(h["out_event"])
                g = torch.empty(h["shape"], dtype=h["dtype"], device=h["device"])
                g.copy_(h["host"], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
            h["gpu"], h["event"] = g, ev
        else:
            h["gpu"] = h["host"].clone()
        self.bytes_in += h["host"].numel() * h["host"].element_size()
        h["nbytes"] = h["host"].numel() * h["host"].element_size()

    def unpack(self, obj):
        if not (isinstance(obj, tuple) and len(obj) == 2 and obj[0] == "swapped"):
            return obj
        h = obj[1]
        if h["host"] is None and h["gpu"] is None:
            # unpacked before (e.g. a second backward through a retained graph): hand out the same
            # tensor while it is alive
            prev = h["weak"]() if h.get("weak") is not None else None
            if prev is None:
                raise RuntimeError("a swapped activation was requested again after its buffers were recycled")
            return prev
        self._fetch(h)
        if h["event"] is not None:
            torch.cuda.current_stream().wait_event(h["event"])
            h["gpu"].record_stream(torch.cuda.current_stream())
        out = h["gpu"]
        h["gpu"] = None
        if h["host"] is not None:     # the pinned buffer returns to the pool with the event that frees it
            self._pool.setdefault((tuple(h["shape"]), h["dtype"]), []).append((h["host"], h["event"]))
            h["host"] = None
        h["weak"] = weakref.ref(out)
        return out

    def prefetch(self, scope):
        for h in self._handles.get(scope, []):
            self._fetch(h)

    def release(self, scope):
        self._handles.pop(scope, None)
        self._seen.pop(scope, None)
        self._swapped.pop(scope, None)

    def hooks(self):
        return torch.autograd.graph.saved_tensors_hooks(self.pack, self.unpack)
