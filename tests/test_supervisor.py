"""The benchmark launcher's process supervisor (no GPU)."""

import multiprocessing as mp
import os
import time

import pytest

from fairring_b200.bench.supervisor import ChildFailed, recv_from_connections_and_join_processes


def _ok(conn, v):
    conn.send(v)
    conn.close()


def _crash(conn):
    os._exit(3)


def _silent(conn):
    conn.close()


def _twice(conn):
    conn.send(1)
    conn.send(2)
    time.sleep(0.5)
    conn.close()


def _slow(conn):
    time.sleep(60)


def _spawn(targets):
    ctx = mp.get_context("spawn")
    pairs = []
    for fn, args in targets:
        parent, child = ctx.Pipe(duplex=False)
        p = ctx.Process(target=fn, args=(child, *args))
        p.start()
        child.close()
        pairs.append((p, parent))
    return pairs


def test_collects_results_in_order():
    pairs = _spawn([(_ok, (10,)), (_ok, ("x",)), (_ok, ([1, 2],))])
    assert recv_from_connections_and_join_processes(pairs, timeout=60) == [10, "x", [1, 2]]


@pytest.mark.parametrize("bad,needle", [(_crash, "exited with code 3"), (_silent, "without a result"),
                                        (_twice, "two results")])
def test_a_bad_child_fails_the_run_and_stops_the_others(bad, needle):
    pairs = _spawn([(_slow, ()), (bad, ())])
    t0 = time.time()
    with pytest.raises(ChildFailed, match=needle):
        recv_from_connections_and_join_processes(pairs, timeout=60)
    assert time.time() - t0 < 30
    assert not any(p.is_alive() for p, _ in pairs)


def test_bench_tools_have_help():
    """The command-line tools under fairring_b200.bench parse their arguments
    without a GPU."""
    import subprocess
    import sys

    for mod in ("kernel_probe", "sweep", "tune", "launch", "ddp_breakdown"):
        out = subprocess.run([sys.executable, "-m", f"fairring_b200.bench.{mod}", "--help"],
                             capture_output=True, text=True, timeout=120)
        assert out.returncode == 0, (mod, out.stderr[-500:])
        assert "usage" in out.stdout.lower()
