"""CPU binding of a rank to the cores next to its GPU.

Pinned-memory copies (offloaded weights, gradients, optimizer states, activations) and the host thread that
issues the kernels run best on the NUMA node the GPU hangs off.  ``bind_to_gpu`` asks NVML for that core set and
restricts the calling process to it (``os.sched_setaffinity``; nothing about the GPU is changed):

* ``node``: every rank may use all cores near its GPU (ranks whose GPUs share a node share the cores);
* ``exclusive``: the ranks that share a core set split it into equal, disjoint slices;
* ``off``: no binding.

``TrainingSession`` applies the mode named by ``MIST_B200_BIND_CPU`` (default ``off``).  Memory is then
allocated node-local by the kernel's first-touch policy, which is what the reference's launcher wrapper gets from
``numactl --membind`` (mist/tools/bind.sh: ``--cpu=node|exclusive|off``, ``--mem=node``).
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence, Set


def _mask_to_cores(words: Sequence[int], bits: int = 64) -> Set[int]:
    cores = set()
    for w, word in enumerate(words):
        word = int(word)
        b = 0
        while word:
            if word & 1:
                cores.add(w * bits + b)
            word >>= 1
            b += 1
    return cores


def gpu_cpu_set(device_index: int, nvml=None) -> Set[int]:
    """Cores that NVML reports as nearest to GPU ``device_index`` (empty when NVML is unavailable)."""
    try:
        if nvml is None:
            import pynvml as nvml
            nvml.nvmlInit()
        handle = nvml.nvmlDeviceGetHandleByIndex(int(device_index))
        n_cpus = os.cpu_count() or 64
        words = nvml.nvmlDeviceGetCpuAffinity(handle, (n_cpus + 63) // 64)
        return _mask_to_cores(words)
    except Exception:       # noqa: BLE001  (no NVML, no permission, unknown device: leave the process unbound)
        return set()


def plan(device_sets: Sequence[Set[int]], rank: int, mode: str, allowed: Optional[Set[int]] = None) -> Set[int]:
    """Core set of ``rank`` given every local rank's GPU core set.  ``allowed``: cores the process may use at
    all (a container's cpuset); the plan never leaves it, and an empty result means "do not bind"."""
    if mode == "off" or not device_sets or not device_sets[rank]:
        return set()
    mine = set(device_sets[rank])
    if allowed is not None:
        mine &= allowed
    if mode == "node" or not mine:
        return mine
    assert mode == "exclusive", f"unknown binding mode {mode!r}"
    sharers = [r for r, s in enumerate(device_sets) if s == device_sets[rank]]
    cores: List[int] = sorted(mine)
    per = len(cores) // len(sharers)
    if per == 0:
        return mine                              # fewer cores than ranks: share them
    k = sharers.index(rank)
    return set(cores[k * per:(k + 1) * per])


def bind_to_gpu(local_rank: int, local_world: int, mode: Optional[str] = None, nvml=None, apply: bool = True) -> Set[int]:
    """Binds the calling process as ``mode`` says and returns the chosen core set (empty: left unbound)."""
    mode = (mode or os.environ.get("MIST_B200_BIND_CPU", "off")).lower()
    if mode == "off":
        return set()
    sets = [gpu_cpu_set(r, nvml) for r in range(local_world)]
    allowed = set(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else None
    chosen = plan(sets, local_rank, mode, allowed)
    if chosen and apply and hasattr(os, "sched_setaffinity"):
        os.sched_setaffinity(0, chosen)
    return chosen
