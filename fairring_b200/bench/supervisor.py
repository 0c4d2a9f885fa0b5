"""Collect one result from each child process and notice when one dies.

Counterpart of benchmark/utils.py in the reference
(recv_from_connections_and_join_processes): the parent multiplexes over the
result pipes and the process sentinels; a child that exits without a result,
sends two results or exits non-zero makes the whole run fail, and every child
that is still alive is then terminated (only the processes started here).
"""

from __future__ import annotations

import multiprocessing.connection as mpc
from typing import Any, List, Sequence


class ChildFailed(RuntimeError):
    pass


def recv_from_connections_and_join_processes(
    pairs: Sequence[tuple], timeout: float | None = None
) -> List[Any]:
    """``pairs``: (process, parent end of its pipe) per child.  Returns the
    children's results in order."""
    procs = [p for p, _ in pairs]
    conns = [c for _, c in pairs]
    results: dict[int, Any] = {}
    exited: set[int] = set()
    eof: set[int] = set()  # pipes whose writer is gone
    by_obj = {}
    for i, (p, c) in enumerate(pairs):
        by_obj[p.sentinel] = ("proc", i)
        by_obj[c] = ("conn", i)
    try:
        while len(exited) < len(procs):
            waitables = [c for i, c in enumerate(conns) if i not in eof]
            waitables += [p.sentinel for i, p in enumerate(procs) if i not in exited]
            ready = mpc.wait(waitables, timeout=timeout)
            if not ready:
                raise ChildFailed(f"no progress within {timeout} s")
            # results first: a child may send and exit in the same instant
            for obj in ready:
                kind, i = by_obj[obj]
                if kind != "conn":
                    continue
                try:
                    value = conns[i].recv()
                except EOFError:
                    eof.add(i)
                    continue
                if i in results:
                    raise ChildFailed(f"child {i} sent two results")
                if isinstance(value, BaseException):
                    raise ChildFailed(f"child {i} raised: {value!r}")
                results[i] = value
            for obj in ready:
                kind, i = by_obj[obj]
                if kind != "proc":
                    continue
                procs[i].join()
                exited.add(i)
                if procs[i].exitcode != 0:
                    raise ChildFailed(f"child {i} exited with code {procs[i].exitcode}")
                if i not in results:
                    try:
                        if i not in eof and conns[i].poll():
                            results[i] = conns[i].recv()
                    except EOFError:
                        pass
                    if i not in results:
                        raise ChildFailed(f"child {i} exited without a result")
    except BaseException:
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
        raise
    return [results[i] for i in range(len(procs))]
