"""Candidate generators of the tuner: device meshes and gradient-accumulation counts
(reference: mist/tuning/optimization.py:33-55)."""
from __future__ import annotations

from typing import List, Tuple


def device_mesh_candidates(num_nodes: int, gpus_per_node: int) -> List[Tuple[int, int]]:
    """Sub-meshes a pipeline stage may occupy: ``(1, m)`` for every power of two ``m`` up to a
    node, then ``(n, gpus_per_node)`` for every power-of-two node count."""
    out = []
    m = 1
    while m <= gpus_per_node:
        out.append((1, m))
        m *= 2
    n = 2
    while n <= num_nodes:
        out.append((n, gpus_per_node))
        n *= 2
    if (num_nodes, gpus_per_node) not in out:
        out.append((num_nodes, gpus_per_node))
    return out


def grad_accum_candidates(global_batch_size: int) -> List[int]:
    """Powers of two that divide the global batch size."""
    out, g = [], 1
    while g <= global_batch_size:
        if global_batch_size % g == 0:
            out.append(g)
        g *= 2
    return out


def stage_count_candidates(num_devices: int, num_layers: int) -> List[int]:
    """Stage counts that split the devices evenly (uniform device assignment)."""
    return [s for s in range(1, num_devices + 1) if num_devices % s == 0 and s <= num_layers]
