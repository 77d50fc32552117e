"""Sharded training checkpoints: save, resume and re-shard.

Layout of a checkpoint directory::

    meta.json                       strategy vector per stage, world layout, step, dtype
    strategy.yaml                   the configuration's strategy block (what the tuner writes)
    model_stage{S}_tp{T}.pt         nested Megatron-style state dict of the stage's model
                                    ({"language_model": {"embedding": ..., "encoder": ...}, "lm_head": ...})
    optim_stage{S}_tp{T}_dp{D}.pt   per unit: fp32 master weights, Adam moments, step (this
                                    rank's shard), plus RNG state

The model file is written by data-parallel rank 0 of each (stage, tp) pair from the
gathered weights; optimizer shards are written by every rank.  ``load`` rebuilds the fp32
state of the *current* strategy from the shard files of the saved one, so a checkpoint
taken under one data-parallel degree or ZeRO level resumes under another (the flat layout
is a function of the model only; shard boundaries are recomputed).

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


def _full_fp32(unit, group) -> torch.Tensor:
    """Gathers a unit's fp32 master weights (and moments) from its dp shards."""
    parts = []
    for name in ("master", "exp_avg", "exp_avg_sq"):
        t = getattr(unit, name)
        split = getattr(unit, "opt_split", None)
        if split is not None:
            t = split[("master", "exp_avg", "exp_avg_sq").index(name)].full()
        if unit.sharded_state and group is not None:
            out = torch.empty(unit.padded, dtype=t.dtype, device=t.device)
            dist.all_gather_into_tensor(out, t.contiguous(), group=group)
            t = out
        parts.append(t)
    return parts


def save(session, path: str, step: int = 0):
    os.makedirs(path, exist_ok=True)
    stage, tp, dp, dp_size = _rank_info(session)
    eng = session.engine
    group = session.ps.dp_group
    units = {}
    for u in eng.units:
        master, m, v = _full_fp32(u, group)
        if dp == 0:
            units[u.name] = {"master": master.cpu(), "exp_avg": m.cpu(), "exp_avg_sq": v.cpu(), "step": u.step_count,
                             "numel": u.numel, "padded": u.padded,
                             "params": list(zip(u.param_names, u.offsets, [tuple(p.shape) for p in u.params]))}
    if dp == 0:
        # model weights in the nested layout, from the bf16 weights the ranks train with
        if eng.zero3:
            for u in eng.units:
                if u.param_shard is not None and u.flat_param is None:
                    u.unshard(torch.empty(u.padded, dtype=u.dtype, device=eng.device), session.ps.dp_ag_group)
        sd = session.model.state_dict_for_save_checkpoint() if hasattr(session.model, "state_dict_for_save_checkpoint") \
            else session.model.state_dict()
        torch.save(sd, os.path.join(path, f"model_stage{stage}_tp{tp}.pt"))
        torch.save({"units": units, "rng": torch.get_rng_state(),
                    "cuda_rng": torch.cuda.get_rng_state() if torch.cuda.is_available() else None},
                   os.path.join(path, f"optim_stage{stage}_tp{tp}.pt"))
    elif eng.zero3:
        for u in eng.units:
            if u.param_shard is not None and u.flat_param is None:
                u.unshard(torch.empty(u.padded, dtype=u.dtype, device=eng.device), session.ps.dp_ag_group)
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


def load(session, path: str) -> int:
    """Restores weights and optimizer state into ``session`` (same pipeline / tensor layout,
    any data-parallel degree or ZeRO level).  Returns the saved step."""
    stage, tp, dp, dp_size = _rank_info(session)
    with open(os.path.join(path, "meta.json")) as f:
        meta = json.load(f)
    assert meta["layer_partitions"] == session.cfg.strategy.layer_partitions, \
        "resharding across different pipeline partitions needs the weights to be re-split by layer first"
    blob = torch.load(os.path.join(path, f"optim_stage{stage}_tp{tp}.pt"), map_location="cpu", weights_only=False)
    eng = session.engine
    for u in eng.units:
        saved = blob["units"][u.name]
        assert saved["numel"] == u.numel, f"unit {u.name}: layout differs ({saved['numel']} vs {u.numel})"
        full = {}
        for k in ("master", "exp_avg", "exp_avg_sq"):
            t = saved[k]
            if t.numel() < u.padded:       # saved under a different dp degree: padding differs
                t = torch.cat([t, torch.zeros(u.padded - t.numel(), dtype=t.dtype)])
            full[k] = t[: u.padded]
        sl = u.shard_range() if u.sharded_state else slice(0, u.padded)
        split = getattr(u, "opt_split", None)
        for i, k in enumerate(("master", "exp_avg", "exp_avg_sq")):
            src = full[k][sl].to(eng.device)
            if split is not None:
                sp_ = split[i]
                sp_.device_part.copy_(src[: sp_.dev_numel])
                if sp_.host_numel:
                    sp_.host_part.copy_(src[sp_.dev_numel:].cpu())
            else:
                getattr(u, k).copy_(src)
        u.step_count = int(saved["step"])
        # bf16 weights from the fp32 master copy
        w = full["master"].to(eng.device)
        if u.param_shard is not None:
            u.param_shard.copy_(w[u.shard_range()].to(u.dtype))
            if u.flat_param is not None:
                u.flat_param.copy_(w.to(u.dtype))
        else:
            u.flat_param.copy_(w.to(u.dtype))
    if blob.get("rng") is not None:
        torch.set_rng_state(blob["rng"])
    if dist.is_initialized():
        dist.barrier()
    return int(meta["step"])
