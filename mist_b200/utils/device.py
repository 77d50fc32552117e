"""Device helpers: the name that keys the operator database, the current device, stream joins.

Reference: ``mock_cuda_device_name_if_needed`` (``FAKE_DEVICE_NAME``) and ``stream_synchronize``
(mist/utils/device.py:67-82).
"""
from __future__ import annotations

import os

import torch


def device_name() -> str:
    """``FAKE_DEVICE_NAME`` if set (analysis and tuning for another GPU, or on a machine without one),
    else the name of the current CUDA device with spaces replaced, else ``"cpu"``."""
    fake = os.environ.get("FAKE_DEVICE_NAME")
    if fake:
        return fake
    if torch.cuda.is_available():
        return torch.cuda.get_device_name().replace(" ", "_")
    return "cpu"


def current_device() -> torch.device:
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def join_streams(*streams):
    """Every given stream waits for the work queued so far on all the others (no host blocking)."""
    if not torch.cuda.is_available():
        return
    streams = [s for s in streams if s is not None]
    events = []
    for s in streams:
        ev = torch.cuda.Event()
        ev.record(s)
        events.append(ev)
    for i, s in enumerate(streams):
        for j, ev in enumerate(events):
            if i != j:
                s.wait_event(ev)


def free_port(host: str = "127.0.0.1") -> int:
    """A TCP port nothing listens on right now (the kernel picks it), for a local rendezvous."""
    import socket
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sock:
        sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        sock.bind((host, 0))
        return int(sock.getsockname()[1])
