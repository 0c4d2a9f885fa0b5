"""Host detection and grouping, with threads standing in for ranks."""

import threading

import pytest
import torch.distributed as dist


def _detect_all(C, world, boot_ids, gpm=0, favorable=False):
    store = dist.HashStore()
    out, errs = [None] * world, [None] * world

    def run(r):
        try:
            out[r] = C.detect_deployment(store, r, world, gpm, favorable, boot_ids[r])
        except Exception as e:  # noqa: BLE001
            errs[r] = e

    ts = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=30)
    return out, errs


def test_one_host_defaults_to_one_machine(C):
    out, errs = _detect_all(C, 4, ["a"] * 4)
    assert not any(errs)
    for r, d in enumerate(out):
        assert (d["M"], d["D"], d["m"], d["d"]) == (1, 4, 0, r)
        assert d["single_host"] and d["num_hosts"] == 1 and d["ranks_per_host"] == 4


def test_machine_major_and_device_major_hosts(C):
    out, errs = _detect_all(C, 4, ["a", "a", "b", "b"])
    assert not any(errs)
    assert [(d["m"], d["d"]) for d in out] == [(0, 0), (0, 1), (1, 0), (1, 1)]
    assert all(d["favorable"] == 0 and not d["single_host"] for d in out)
    out, errs = _detect_all(C, 4, ["a", "b", "a", "b"])
    assert not any(errs)
    assert [(d["m"], d["d"]) for d in out] == [(0, 0), (1, 0), (0, 1), (1, 1)]
    assert all(d["favorable"] == 1 for d in out)


def test_uneven_or_scrambled_hosts_are_rejected(C):
    _, errs = _detect_all(C, 4, ["a", "a", "a", "b"])
    assert all(e is not None and "same number of ranks" in str(e) for e in errs)
    _, errs = _detect_all(C, 4, ["a", "b", "b", "a"])
    assert all(e is not None and "numbered" in str(e) for e in errs)


@pytest.mark.parametrize("gpm,fav", [(2, False), (2, True), (4, False), (1, True)])
def test_virtual_machines_from_the_environment(C, gpm, fav):
    out, errs = _detect_all(C, 8, ["a"] * 8, gpm=gpm, favorable=fav)
    assert not any(errs)
    M = 8 // gpm
    for r, d in enumerate(out):
        assert d["D"] == gpm and d["M"] == M and d["single_host"]
        assert (d["m"], d["d"]) == ((r % M, r // M) if fav else (r // gpm, r % gpm))
    _, errs = _detect_all(C, 8, ["a"] * 8, gpm=3)
    assert all(e is not None and "does not divide" in str(e) for e in errs)
