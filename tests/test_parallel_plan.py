"""Rank layout and inter-stage routes (pure CPU arithmetic)."""
from mist_b200.parallel.state import ShardInfo, build_plan, map_stages_to_ranks


def test_stage_packing_whole_and_partial_nodes():
    m = map_stages_to_ranks([(1, 8), (1, 4), (1, 4), (2, 8)], (4, 8))
    assert m[0] == list(range(0, 8))
    assert m[1] == list(range(8, 12)) and m[2] == list(range(12, 16))
    assert m[3] == list(range(16, 32))


def test_groups_inside_a_stage():
    plan = build_plan([(1, 8)], [(4, 4, 2)], (1, 8))
    r5 = plan.ranks[5]
    assert r5.tp_ranks == [4, 5] and r5.dp_ranks == [1, 3, 5, 7]
    assert r5.tp_index == 1 and r5.dp_index == 2
    assert [0, 1] in plan.tp_groups and [0, 2, 4, 6] in plan.dp_groups


def test_homogeneous_pipeline_routes():
    plan = build_plan([(1, 4), (1, 4)], [(2, 1, 4), (2, 1, 4)], (1, 8))
    # every rank of stage 1 receives the whole micro batch from some tp replica of stage 0
    for r in range(4, 8):
        (src, info), = plan.ranks[r].recv_prev
        assert src in range(0, 4) and not info.is_sharded
    sends = sum(len(plan.ranks[r].send_next) for r in range(4))
    assert sends == 4
    # replicas share the load
    assert max(len(plan.ranks[r].send_next) for r in range(4)) == 1


def test_heterogeneous_batch_resharding():
    # stage 0: micro batch 4, dp 1;  stage 1: micro batch 2, dp 2  -> sender splits its batch
    plan = build_plan([(1, 1), (1, 2)], [(4, 1, 1), (2, 2, 1)], (1, 4))
    s = plan.ranks[0].send_next
    assert [(d, i.shard_idx, i.num_shards) for d, i in s] == [(1, 0, 2), (2, 1, 2)]
    assert plan.ranks[1].recv_prev == [(0, ShardInfo(False))]
    # the other way round: receiver concatenates two senders
    plan = build_plan([(1, 2), (1, 1)], [(2, 2, 1), (4, 1, 1)], (1, 4))
    assert plan.ranks[2].recv_prev == [(0, ShardInfo(True, 0, 2)), (1, ShardInfo(True, 1, 2))]
    assert ShardInfo(True, 1, 2).slice_of(4) == slice(2, 4)
