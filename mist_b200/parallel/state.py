"""Rank layout of a strategy: pipeline stages -> rank ranges, tensor/data-parallel groups
inside each stage, and the point-to-point routes between consecutive stages.

The layout is computed by :func:`build_plan`, a pure function of the strategy (no
communicator needed, so it is unit-tested on CPU for heterogeneous stages), and turned
into ``torch.distributed`` groups by :class:`ParallelState`.

Rules (same observable layout as the reference, mist/parallel_state.py:63-113 stage
packing, :160-245 inter-stage routes, :247-290 groups):
* stages that use whole nodes take the next free nodes; stages that use part of a node
  are packed into a partially used node when they fit, else open a new node;
* inside a stage, tensor-parallel groups are contiguous ranks and data-parallel groups
  are ranks ``tp`` apart;
* when consecutive stages have different (micro batch, dp), a sender with the larger
  micro batch splits it along the batch dimension among several receivers, and a
  receiver with the larger micro batch concatenates several senders; among the
  tensor-parallel replicas of a sender the least used one is picked.
* every data-parallel group gets two extra communicators so parameter all-gathers and
  gradient reduce-scatters can be in flight at the same time.
"""
from __future__ import annotations

import datetime
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ShardInfo:
    """Which slice of the batch dimension a p2p message carries."""
    is_sharded: bool
    shard_idx: int = 0
    num_shards: int = 1

    def slice_of(self, n: int) -> slice:
        if not self.is_sharded or self.num_shards == 1:
            return slice(0, n)
        per = n // self.num_shards
        return slice(self.shard_idx * per, (self.shard_idx + 1) * per)

    def __repr__(self):
        if not self.is_sharded or self.num_shards == 1:
            return "ShardInfo(whole)"
        return f"ShardInfo({self.shard_idx}/{self.num_shards})"


@dataclass
class RankPlan:
    rank: int
    stage: int
    tp_ranks: List[int]
    dp_ranks: List[int]
    tp_index: int
    dp_index: int
    send_next: List[Tuple[int, ShardInfo]] = field(default_factory=list)   # (peer rank, my slice sent)
    recv_prev: List[Tuple[int, ShardInfo]] = field(default_factory=list)   # (peer rank, slice of my batch filled)


@dataclass
class ParallelPlan:
    stage_to_ranks: Dict[int, List[int]]
    ranks: Dict[int, RankPlan]
    tp_groups: List[List[int]]
    dp_groups: List[List[int]]

    @property
    def num_stages(self) -> int:
        return len(self.stage_to_ranks)


def map_stages_to_ranks(device_assignment: Sequence[Tuple[int, int]], mesh: Tuple[int, int]) -> Dict[int, List[int]]:
    nodes, per_node = mesh
    free_nodes = list(range(nodes))
    partial: Dict[int, int] = {}        # node -> GPUs already used
    out: Dict[int, List[int]] = {}
    for stage, (n, m) in enumerate(device_assignment):
        if m == per_node:
            assert len(free_nodes) >= n, f"stage {stage} needs {n} whole nodes, {len(free_nodes)} left"
            first = free_nodes[0]
            del free_nodes[:n]
            out[stage] = list(range(first * per_node, (first + n) * per_node))
            continue
        assert n == 1, f"stage {stage}: a stage smaller than a node must stay within one node"
        node = next((k for k, used in partial.items() if used + m <= per_node), None)
        if node is None:
            assert free_nodes, f"no node left for stage {stage}"
            node = free_nodes.pop(0)
            partial[node] = 0
        start = node * per_node + partial[node]
        partial[node] += m
        out[stage] = list(range(start, start + m))
    return out


def build_plan(device_assignment, stage_strategies, mesh: Tuple[int, int]) -> ParallelPlan:
    """``stage_strategies[s]`` is the 10-vector (or anything whose first three entries are
    micro batch size, dp, tp)."""
    stage_to_ranks = map_stages_to_ranks(device_assignment, mesh)
    ranks: Dict[int, RankPlan] = {}
    tp_groups, dp_groups = [], []
    for s, rs in stage_to_ranks.items():
        dp, tp = int(stage_strategies[s][1]), int(stage_strategies[s][2])
        assert dp * tp == len(rs), f"stage {s}: dp {dp} x tp {tp} != {len(rs)} ranks"
        for d in range(dp):
            tp_groups.append(rs[d * tp:(d + 1) * tp])
        for t in range(tp):
            dp_groups.append(rs[t::tp])
        for i, r in enumerate(rs):
            d, t = divmod(i, tp)
            ranks[r] = RankPlan(r, s, rs[d * tp:(d + 1) * tp], rs[t::tp], t, d)
    # routes between consecutive stages
    for s in range(len(stage_to_ranks) - 1):
        cb, cdp, ctp = (int(x) for x in stage_strategies[s][:3])
        nb, ndp, ntp = (int(x) for x in stage_strategies[s + 1][:3])
        assert cb * cdp == nb * ndp, f"stages {s},{s + 1} disagree on the batch per micro step"
        usage = [[0] * ctp for _ in range(cdp)]
        cursor = [0] * cdp

        def pick_tp(d):
            cur = cursor[d]
            nxt = (cur + 1) % ctp
            choice = nxt if usage[d][nxt] < usage[d][cur] else cur
            cursor[d] = choice
            usage[d][choice] += 1
            return choice

        for nd in range(ndp):
            if cb >= nb:
                factor = cb // nb
                senders = [nd // factor]
                send_shards = [ShardInfo(factor > 1, nd % factor, factor)]
                recv_shards = [ShardInfo(False)]
            else:
                factor = nb // cb
                senders = list(range(nd * factor, (nd + 1) * factor))
                send_shards = [ShardInfo(False)] * factor
                recv_shards = [ShardInfo(True, k, factor) for k in range(factor)]
            for nt in range(ntp):
                dst = stage_to_ranks[s + 1][nd * ntp + nt]
                for cd, ss, rsinfo in zip(senders, send_shards, recv_shards):
                    src = stage_to_ranks[s][cd * ctp + pick_tp(cd)]
                    ranks[src].send_next.append((dst, ss))
                    ranks[dst].recv_prev.append((src, rsinfo))
    return ParallelPlan(stage_to_ranks, ranks, tp_groups, dp_groups)


class ParallelState:
    """Process groups of this rank.  ``world_size == 1`` needs no initialised backend."""

    def __init__(self, plan: ParallelPlan, rank: int, timeout_s: int = 120, create_groups: bool = True):
        self.plan, self.rank = plan, rank
        me = plan.ranks[rank]
        self.me = me
        self.stage = me.stage
        self.num_stages = plan.num_stages
        self.tp_size, self.dp_size = len(me.tp_ranks), len(me.dp_ranks)
        self.tp_rank, self.dp_rank = me.tp_index, me.dp_index
        self.tp_group = self.dp_group = self.dp_ag_group = self.dp_rs_group = None
        if create_groups and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            to = datetime.timedelta(seconds=timeout_s)
            # new_group is collective over the world: every rank creates every group
            for g in plan.tp_groups:
                grp = dist.new_group(g, timeout=to) if len(g) > 1 else None
                if rank in g:
                    self.tp_group = grp
            for g in plan.dp_groups:
                if len(g) > 1:
                    a, b, c = (dist.new_group(g, timeout=to) for _ in range(3))
                else:
                    a = b = c = None
                if rank in g:
                    self.dp_group, self.dp_ag_group, self.dp_rs_group = a, b, c

    def create_embedding_group(self, timeout_s: int = 120):
        """Pairs every rank of the first pipeline stage with the rank of the last stage that holds the
        same (data-parallel, tensor-parallel) position: the two keep copies of a word-embedding table
        that is tied to the output projection and sum its gradient over this group.  Collective over
        the world (every rank creates every pair); returns this rank's pair or ``None``."""
        first, last = self.plan.stage_to_ranks[0], self.plan.stage_to_ranks[self.num_stages - 1]
        f0, l0 = self.plan.ranks[first[0]], self.plan.ranks[last[0]]
        assert (len(f0.dp_ranks), len(f0.tp_ranks)) == (len(l0.dp_ranks), len(l0.tp_ranks)), \
            "tied embeddings across pipeline stages need the same dp x tp layout on the first and the last stage"
        mine = None
        to = datetime.timedelta(seconds=timeout_s)
        for a, b in zip(first, last):
            grp = dist.new_group([a, b], timeout=to)
            if self.rank in (a, b):
                mine = grp
        self.embedding_group = mine
        self.embedding_src = first[last.index(self.rank)] if self.rank in last else (
            self.rank if self.rank in first else None)
        return mine

    @classmethod
    def from_config(cls, cfg, rank: Optional[int] = None, create_groups: bool = True) -> "ParallelState":
        mesh = (cfg.hardware.num_nodes, cfg.hardware.num_gpus_per_node)
        plan = build_plan(cfg.strategy.device_assignment, cfg.strategy.stage_strategies, mesh)
        if rank is None:
            rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        return cls(plan, rank, getattr(cfg, "nccl_timeout", 120), create_groups)

    @classmethod
    def single(cls) -> "ParallelState":
        plan = build_plan([(1, 1)], [(1, 1, 1)], (1, 1))
        return cls(plan, 0, create_groups=False)

    # ------------------------------------------------------------------ convenience getters
    @property
    def is_first_stage(self):
        return self.stage == 0

    @property
    def is_last_stage(self):
        return self.stage == self.num_stages - 1

    def stage_ranks(self, stage=None):
        return self.plan.stage_to_ranks[self.stage if stage is None else stage]

    @property
    def send_next(self):
        return self.me.send_next

    @property
    def recv_prev(self):
        return self.me.recv_prev

    @property
    def send_prev(self):
        """Backward direction: gradients go back along the forward receive routes."""
        return self.me.recv_prev

    @property
    def recv_next(self):
        return self.me.send_next
