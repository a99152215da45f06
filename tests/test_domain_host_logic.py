"""Host-side decisions of the native multi-GPU domain code, without a GPU: neighbour ranks and message counts of the
brick grid, the verdict all ranks derive from the counts they publish (failures made on the host: a rank that reports
lost atoms, a rank without room), and the bounded host wait against a stand-in that never becomes ready."""
import time

import numpy as np
import pytest

from deepscalemd_b200 import input_api as ia


@pytest.mark.parametrize("dims, n_dirs, n_peers", [((2, 1, 1), 2, 1), ((2, 2, 1), 8, 3), ((2, 2, 2), 26, 7),
                                                   ((4, 2, 1), 8, 5), ((3, 3, 3), 26, 26), ((1, 1, 1), 0, 0)])
def test_directions_are_grouped_by_neighbour_rank(dims, n_dirs, n_peers):
    world = int(np.prod(dims))
    for rank in range(world):
        plan = ia.brick_plan(dims, rank)
        assert len(plan["dir_dest"]) == n_dirs
        assert plan["dir_dest"] == sorted(plan["dir_dest"])           # one contiguous run of directions per neighbour
        assert plan["peers"] == sorted(set(plan["dir_dest"])) and len(plan["peers"]) == n_peers
        assert rank not in plan["peers"]
        # what a neighbour sends here is one run of ITS directions: as many as this rank has towards it (symmetry)
        mine = [plan["dir_dest"].count(p) for p in plan["peers"]]
        assert plan["from_count"] == mine
    # the neighbour relation is symmetric
    for rank in range(world):
        for p in ia.brick_plan(dims, rank)["peers"]:
            assert rank in ia.brick_plan(dims, p)["peers"]


def full_counts(dims, per_direction, room=10**6):
    world = int(np.prod(dims))
    c = np.zeros((world, ia.BINS), dtype=np.int32)
    for r in range(world):
        n = len(ia.brick_plan(dims, r)["dir_dest"])
        c[r, 0] = 1000
        c[r, 1:1 + n] = per_direction
        c[r, 28] = room
    return c


def test_one_message_per_neighbour_rank_and_way():
    # 2 x 2 x 2: 26 directions with ghosts for every one of them, 7 neighbour ranks -> 14 messages, not 104
    v = ia.counts_verdict((2, 2, 2), full_counts((2, 2, 2), 50))
    assert v["code"] == 0 and v["messages"][:8] == [14] * 8
    v = ia.counts_verdict((2, 1, 1), full_counts((2, 1, 1), 50))
    assert v["code"] == 0 and v["messages"][:2] == [2, 2]
    # nothing to send along any direction: no message at all
    assert ia.counts_verdict((2, 2, 1), full_counts((2, 2, 1), 0))["messages"][:4] == [0] * 4


def test_every_rank_reaches_the_same_verdict_on_a_failure_made_on_the_host():
    dims = (2, 2, 2)
    c = full_counts(dims, 10)
    c[5, 27] = 3                                # rank 5 reports three atoms that moved further than a brick
    v = ia.counts_verdict(dims, c)
    assert v["code"] == 4 and v["rank"] == 5 and "rank 5" in v["text"] and "3 atoms" in v["text"]
    c = full_counts(dims, 10)
    c[2, 28] = 100                              # rank 2 has room for 100 more atoms; 26 directions x 10 arrive
    v = ia.counts_verdict(dims, c)
    assert v["code"] == 5 and v["rank"] == 2 and "260" in v["text"]
    c[2, 28] = 260
    assert ia.counts_verdict(dims, c)["code"] == 0
    c = full_counts(dims, 10)
    assert ia.counts_verdict(dims, c, scratch_capacity=200)["code"] == 5      # more to send than the scratch holds


def test_host_wait_has_a_deadline():
    assert ia.wait_probe(5.0, ready_after=0) == 0
    assert ia.wait_probe(5.0, ready_after=100_000) == 0                       # becomes ready after many polls
    t0 = time.time()
    assert ia.wait_probe(0.3) == 7                                            # never ready: DSMD_ERR_TIMEOUT
    assert 0.25 < time.time() - t0 < 3.0
    assert ia.wait_probe(5.0, fail_after=10) == 2                             # the stand-in reports a failure
