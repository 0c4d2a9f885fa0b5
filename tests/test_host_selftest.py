"""Exhaustive in-process runs of the host path: threads are the ranks.

The index maps, the slicing and the double-buffered staging are the same code
(layout.h) and the same algorithm as in the GPU kernels, so every grouping of
eight ranks, both rank numberings, ragged sizes and many slices are covered
here in milliseconds.
"""

import pytest

GROUPINGS = [(1, 1), (2, 1), (2, 2), (3, 1), (3, 3), (4, 1), (4, 2), (4, 4), (6, 2), (6, 3),
             (8, 1), (8, 2), (8, 4), (8, 8)]


@pytest.mark.parametrize("world,gpm", GROUPINGS)
@pytest.mark.parametrize("favorable", [False, True])
def test_every_grouping_and_numbering(C, world, gpm, favorable):
    sizes = [1, 3, 4 * world, 4 * world + 1, 1000, 4099, 65_537]
    assert C.cpu_self_test(world, gpm, favorable, sizes, total_memory=1 << 20) == 0


@pytest.mark.parametrize("world,gpm", [(2, 2), (4, 2), (8, 4), (8, 2)])
def test_many_slices_and_both_halves(C, world, gpm):
    # a tiny budget: 4 KiB halves force dozens of slices per tensor, so both
    # halves and many epochs are used
    sizes = [50_001, 7, 20_000, 123_457]
    assert C.cpu_self_test(world, gpm, False, sizes, total_memory=8 << 10, oneshot_max=0) == 0
    assert C.cpu_self_test(world, gpm, True, sizes, total_memory=64 << 10, slice_bytes=4096,
                           oneshot_max=0, use_max=True) == 0


def test_one_shot_path(C):
    for world in (2, 5, 8):
        assert C.cpu_self_test(world, world, False, [1, 17, 256, 1023], total_memory=4 << 20,
                               oneshot_max=1 << 16) == 0


def test_property_random_shapes(C):
    hyp = pytest.importorskip("hypothesis")
    from hypothesis import given, settings
    from hypothesis import strategies as st

    @settings(max_examples=40, deadline=None)
    @given(st.sampled_from(GROUPINGS), st.booleans(),
           st.lists(st.integers(min_value=1, max_value=30_000), min_size=1, max_size=4),
           st.sampled_from([4 << 10, 32 << 10, 1 << 20]), st.sampled_from([0, 256, 4096]),
           st.booleans())
    def run(grouping, favorable, sizes, total, oneshot, use_max):
        world, gpm = grouping
        assert C.cpu_self_test(world, gpm, favorable, sizes, total_memory=total,
                               oneshot_max=oneshot, use_max=use_max) == 0

    run()


def test_command_queue_is_fifo_per_producer_and_loses_nothing(C):
    assert C.command_queue_self_test(1, 1000) == 0
    assert C.command_queue_self_test(8, 20000) == 0
