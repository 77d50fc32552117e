"""Sharded training checkpoints: save, resume and re-shard.

Layout of a checkpoint directory::

    meta.json                       strategy vector per stage, world layout, step, dtype
    strategy.yaml                   the configuration's strategy block (what the tuner writes)
    model_stage{S}_tp{T}.pt         nested Megatron-style state dict of the stage's model
                                    ({"language_model": {"embedding": ..., "encoder": ...}, "lm_head": ...})
    optim_stage{S}_tp{T}_dp{D}.pt   per unit: fp32 master weights, Adam moments, step (this
                                    rank's shard), plus RNG state

Every rank writes its own optimizer file (its shard of the fp32 state, or the whole state when
the stage does not shard it, in which case only data-parallel rank 0 writes), together with its CPU
and CUDA random-number state.  The model file is written by data-parallel rank 0 of each
(stage, tp) pair from the fp32 master weights, which are assembled one unit at a time through a
single reusable buffer, so saving never holds more than one unit unsharded -- also under ZeRO-3
and with weights offloaded to the host.  ``load`` rebuilds the fp32 state of the *current*
strategy from the shard files of the saved one: a rank reads only the files that overlap its
shard, so a checkpoint taken under one data-parallel degree, ZeRO level or offloading ratio
resumes under another (the flat layout is a function of the model only; shard boundaries are
recomputed).  The bf16 weights are then refreshed from the master weights the way an optimizer
step refreshes them.

The reference has no save / resume in its runtime (its nested ``state_dict_for_save_checkpoint``
methods, mist/model/gpt.py:133-151 and mist/model/language_model.py:314-405, are never
called); the nested layout is kept so that tooling written for it keeps working.
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

from . import yamlconf


def _rank_info(session):
    ps = session.ps
    return ps.stage, ps.tp_rank, ps.dp_rank, ps.dp_size


_STATE = ("master", "exp_avg", "exp_avg_sq")


def _local_state(unit):
    """This rank's fp32 master weights and moments (host-offloaded tails joined back on)."""
    split = getattr(unit, "opt_split", None)
    if split is not None:
        return [sp.full() for sp in split]
    return [getattr(unit, k) for k in _STATE]


def _optim_file(path, stage, tp, dp):
    return os.path.join(path, f"optim_stage{stage}_tp{tp}_dp{dp}.pt")


def save(session, path: str, step: int = 0):
    os.makedirs(path, exist_ok=True)
    stage, tp, dp, dp_size = _rank_info(session)
    eng = session.engine
    group = session.ps.dp_group if dp_size > 1 else None
    units = {}
    cpu_weights = {}
    scratch = None
    for u in eng.units:
        master, m, v = _local_state(u)
        if u.sharded_state or dp == 0:
            units[u.name] = {"master": master.cpu(), "exp_avg": m.cpu(), "exp_avg_sq": v.cpu(),
                             "step": u.step_count, "numel": u.numel, "padded": u.padded,
                             "sharded": bool(u.sharded_state), "shard_numel": u.state_numel,
                             "params": list(zip(u.param_names, u.offsets, [tuple(p.shape) for p in u.params]))}
        # model weights: the full fp32 master of one unit at a time, through one reusable buffer
        if u.sharded_state and group is not None:
            if scratch is None or scratch.numel() < u.padded:
                scratch = torch.empty(max(x.padded for x in eng.units), dtype=master.dtype, device=master.device)
            full = scratch[: u.padded]
            dist.all_gather_into_tensor(full, master.contiguous(), group=group)
        else:
            full = master
        if dp == 0:
            cpu_weights[u.name] = full[: u.numel].to(u.dtype).cpu()
    if dp == 0:
        # nested layout: point the parameters at the host copies while the dictionary is built
        saved_data = []
        for u in eng.units:
            flat = cpu_weights[u.name]
            for p_, o in zip(u.params, u.offsets):
                saved_data.append((p_, p_.data))
                p_.data = flat[o:o + p_.numel()].view(p_.shape)
        try:
            sd = session.model.state_dict_for_save_checkpoint() if hasattr(session.model, "state_dict_for_save_checkpoint") \
                else session.model.state_dict()
            torch.save(sd, os.path.join(path, f"model_stage{stage}_tp{tp}.pt"))
        finally:
            for p_, d in saved_data:
                p_.data = d
    if units:
        torch.save({"units": units, "dp_size": dp_size, "rng": torch.get_rng_state(),
                    "cuda_rng": torch.cuda.get_rng_state() if torch.cuda.is_available() else None},
                   _optim_file(path, stage, tp, dp))
    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        st = session.cfg.strategy
        meta = {"step": step, "num_stages": st.num_stages, "layer_partitions": st.layer_partitions,
                "stage_strategies": [list(v) for v in st.stage_strategies],
                "gradient_accumulation_steps": st.gradient_accumulation_steps, "model": session.cfg.model.name,
                "params_dtype": str(session.cfg.training.params_dtype)}
        with open(os.path.join(path, "meta.json"), "w") as f:
            json.dump(meta, f, indent=1)
        yamlconf.dump({"strategy": session.cfg.raw["strategy"].to_dict() if hasattr(session.cfg.raw["strategy"], "to_dict")
                       else dict(session.cfg.raw["strategy"])}, os.path.join(path, "strategy.yaml"))
    if dist.is_initialized():
        dist.barrier()


class _SavedState:
    """Reads ranges of a unit's saved fp32 state from the shard files that hold them."""

    def __init__(self, path, stage, tp):
        self.path, self.stage, self.tp = path, stage, tp
        self.files = {}

    def file(self, dp):
        if dp not in self.files:
            self.files[dp] = torch.load(_optim_file(self.path, self.stage, self.tp, dp), map_location="cpu",
                                        weights_only=False)
        return self.files[dp]

    def read(self, unit_name, key, start, stop):
        """Elements ``[start, stop)`` of the saved flat tensor ``key`` (zeros past its end)."""
        info = self.file(0)["units"][unit_name]
        out = torch.zeros(stop - start, dtype=info[key].dtype)
        if not info["sharded"]:
            hi = min(stop, info[key].numel())
            if hi > start:
                out[: hi - start] = info[key][start:hi]
            return out
        n = info["shard_numel"]
        for r in range(start // n, (max(stop, start + 1) - 1) // n + 1):
            if r * n >= info["padded"]:
                break
            lo, hi = max(start, r * n), min(stop, (r + 1) * n)
            if hi > lo:
                out[lo - start: hi - start] = self.file(r)["units"][unit_name][key][lo - r * n: hi - r * n]
        return out


def load(session, path: str) -> int:
    """Restores weights and optimizer state into ``session`` (same pipeline / tensor layout,
    any data-parallel degree, ZeRO level or offloading ratio).  Returns the saved step."""
    stage, tp, dp, dp_size = _rank_info(session)
    with open(os.path.join(path, "meta.json")) as f:
        meta = json.load(f)
    assert meta["layer_partitions"] == session.cfg.strategy.layer_partitions, \
        "resharding across different pipeline partitions needs the weights to be re-split by layer first"
    saved = _SavedState(path, stage, tp)
    eng = session.engine
    group = session.ps.dp_group if dp_size > 1 else None
    scratch = None
    for u in eng.units:
        info = saved.file(0)["units"][u.name]
        assert info["numel"] == u.numel, f"unit {u.name}: layout differs ({info['numel']} vs {u.numel})"
        a = u.dp_rank * u.shard_numel if u.sharded_state else 0
        n = u.state_numel
        split = getattr(u, "opt_split", None)
        mine = None
        for i, k in enumerate(_STATE):
            src = saved.read(u.name, k, a, a + n).to(eng.device)
            if k == "master":
                mine = src
            if split is not None:
                sp_ = split[i]
                sp_.device_part.copy_(src[: sp_.dev_numel])
                if sp_.host_numel:
                    sp_.host_part.copy_(src[sp_.dev_numel:].cpu())
            else:
                getattr(u, k).copy_(src)
        u.step_count = int(info["step"])
        # bf16 weights from the fp32 master copy, refreshed the way an optimizer step refreshes them
        w = mine.to(u.dtype)
        if u.weight_split is not None:
            if scratch is None:
                scratch = torch.empty(max(x.padded for x in eng.units), dtype=u.dtype, device=eng.device)
            full = scratch[: u.padded]
            if u.sharded_state and not u.is_zero3 and group is not None:
                dist.all_gather_into_tensor(full, w.contiguous(), group=group)
            elif u.sharded_state:
                full[u.shard_range()].copy_(w)
            else:
                full.copy_(w)
            u.weight_split.store_from(u.persistent_region(full), eng.swap_streams)
            if eng.cuda:
                torch.cuda.synchronize()          # the scratch buffer is reused by the next unit
        elif u.param_shard is not None:
            u.param_shard.copy_(w)
            if u.flat_param is not None:
                if group is not None:
                    dist.all_gather_into_tensor(u.flat_param, w.contiguous(), group=group)
                else:
                    u.flat_param.copy_(w)
        elif u.sharded_state and group is not None:
            dist.all_gather_into_tensor(u.flat_param, w.contiguous(), group=group)
        else:
            u.flat_param[: w.numel()].copy_(w)
    # random-number state of the rank at the same data-parallel position, when there is one
    if saved.file(0).get("dp_size") == dp_size and os.path.exists(_optim_file(path, stage, tp, dp)):
        blob = saved.file(dp)
        if blob.get("rng") is not None:
            torch.set_rng_state(blob["rng"])
        if blob.get("cuda_rng") is not None and torch.cuda.is_available():
            torch.cuda.set_rng_state(blob["cuda_rng"])
    if dist.is_initialized():
        dist.barrier()
    return int(meta["step"])
