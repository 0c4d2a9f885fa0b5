"""Planner and index math against a NumPy/Python oracle (no GPU, no processes)."""

import itertools

import numpy as np
import pytest


def test_memory_plan_budget_and_alignment(C):
    for total, slice_b, par, world in itertools.product(
            [1 << 20, 50 << 20, 256 << 20, (50 << 20) + 12345], [4 << 20, 25 << 20, 0],
            [1, 4, 16], [1, 2, 3, 8]):
        p = C.plan_memory(total, slice_b, par, world, 1 << 20)
        assert 1 <= p["channels"] <= par
        assert p["slot_bytes"] == 2 * p["half_bytes"]
        assert p["slot_bytes"] * p["channels"] <= max(total, 32 * world)
        assert p["half_bytes"] % (16 * world) == 0
        assert p["max_slice_bytes"] <= p["half_bytes"] or p["half_bytes"] < 16 * world
        assert p["max_slice_bytes"] % (16 * world) == 0
        if slice_b:
            assert p["max_slice_bytes"] <= max(slice_b, 16 * world)
        if p["channels"] > 1:  # channels are only merged while a half would be below 1 MiB
            assert p["half_bytes"] >= (1 << 20) - 16 * world


def test_reference_defaults_give_25mib_slices_room(C):
    # 50 MiB budget (the reference's default) and 25 MiB DDP buckets: a bucket is
    # cut into slices no larger than half a channel slot.
    p = C.plan_memory(50 << 20, 25 << 20, 16, 8, 4 << 20)
    assert p["channels"] == 6 and p["half_bytes"] >= 4 << 20
    n, per = C.plan_slices((25 << 20) // 4, 4, 8, p["max_slice_bytes"])
    assert n * per * 4 >= 25 << 20 and per * 4 <= p["max_slice_bytes"]


@pytest.mark.parametrize("esize", [1, 2, 4, 8])
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_slices_cover_the_tensor_exactly_once(C, esize, world):
    V = 16 // esize
    for numel in [1, V - 1, V, V * world, V * world + 1, 12345, 1_000_003]:
        for max_bytes in [16 * world, 4096 * world, 1 << 20]:
            n, per = C.plan_slices(numel, esize, world, max_bytes)
            assert per % (V * world) == 0
            assert per * esize <= max(max_bytes, 16 * world)
            assert (n - 1) * per < numel <= n * per
    assert C.plan_slices(0, esize, world, 1 << 20)[0] == 0


@pytest.mark.parametrize("esize", [1, 2, 4, 8])
@pytest.mark.parametrize("world", [1, 2, 5, 8])
def test_allreduce_seg_partitions_elements(C, esize, world):
    V = 16 // esize
    for numel in [1, 3, V, V + 1, V * world - 1, V * world, 99_999]:
        s = C.allreduce_seg(numel, esize, world)
        assert s["chunk_len"] == s["chunk_stride"] == s["qv"] * V and s["limit"] == numel
        assert world * s["chunk_len"] >= numel
        seen = np.zeros(numel, dtype=np.int32)
        for c in range(world):
            for v in range(s["qv"]):
                k = C.valid_in_vector(s["chunk_len"], s["chunk_stride"], s["limit"], s["qv"], c, v, V)
                assert 0 <= k <= V
                base = c * s["chunk_stride"] + v * V
                seen[base:base + k] += 1
                if k < V:  # nothing valid may follow a short vector in the same chunk
                    for v2 in range(v + 1, s["qv"]):
                        assert C.valid_in_vector(s["chunk_len"], s["chunk_stride"], s["limit"],
                                                 s["qv"], c, v2, V) == 0
                    break
        assert (seen == 1).all()


def test_scatter_seg_is_per_rank_strided(C):
    s = C.scatter_seg(1000, 5000, 4)
    assert s["chunk_len"] == 1000 and s["chunk_stride"] == 5000 and s["qv"] == 250
    assert C.valid_in_vector(1000, 5000, s["limit"], 250, 7, 249, 4) == 4
    s = C.scatter_seg(1001, 5000, 4)
    assert s["qv"] == 251
    assert C.valid_in_vector(1001, 5000, s["limit"], 251, 3, 250, 4) == 1


@pytest.mark.parametrize("world,D", [(8, 8), (8, 4), (8, 2), (8, 1), (4, 2), (6, 3), (1, 1)])
@pytest.mark.parametrize("fav", [False, True])
def test_rank_numbering_is_a_bijection(C, world, D, fav):
    M = world // D
    seen = set()
    for m in range(M):
        for d in range(D):
            r = C.rank_of(world, D, fav, m, d)
            assert r == (d * M + m if fav else m * D + d)
            assert C.machine_device_of(world, D, fav, r) == (m, d)
            seen.add(r)
    assert seen == set(range(world))


def test_staging_slots_do_not_overlap(C):
    for world, D in [(8, 8), (8, 4), (8, 2), (8, 1)]:
        M = world // D
        qv = 37
        starts = sorted(C.staging_vec(world, D, qv, s, j) for s in range(D) for j in range(M))
        assert starts == [k * qv for k in range(world)]
