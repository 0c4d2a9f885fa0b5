"""Run a function as N ranks in child processes (CPU ranks, or one GPU each)."""

from __future__ import annotations

import multiprocessing as mp
import os
import socket
import traceback


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _child(fn, rank, world, port, env, q, args):
    try:
        os.environ.update({k: str(v) for k, v in env.items()})
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        os.environ["RANK"] = str(rank)
        os.environ["WORLD_SIZE"] = str(world)
        os.environ["LOCAL_RANK"] = str(rank)
        os.environ.setdefault("FAIRRING_TOTAL_MEMORY", str(50 * 1024 * 1024))
        out = fn(rank, world, *args)
        q.put((rank, "ok", out))
    except BaseException as e:  # noqa: BLE001 - report everything to the parent
        q.put((rank, "error", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
    finally:
        # Make sure the report has left this process before anything at
        # interpreter exit can go wrong.
        q.close()
        q.join_thread()
        try:
            import torch.distributed as dist

            if dist.is_initialized():
                dist.destroy_process_group()
        except BaseException:  # noqa: BLE001
            pass


def run_ranks(fn, world: int, env: dict | None = None, args: tuple = (), timeout: float = 180.0):
    """Returns the list of per-rank return values; raises if any rank failed."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [
        ctx.Process(target=_child, args=(fn, r, world, port, env or {}, q, args), daemon=True)
        for r in range(world)
    ]
    for p in procs:
        p.start()
    results = {}
    errors = []
    import queue as _queue
    import time as _time

    deadline = _time.time() + timeout
    try:
        while len(results) + len(errors) < world:
            try:
                rank, status, payload = q.get(timeout=1.0)
            except _queue.Empty:
                if _time.time() > deadline:
                    errors.append((-1, f"no report from some ranks within {timeout} s"))
                    break
                reported = set(results) | {r for r, _ in errors}
                dead = [r for r, p in enumerate(procs)
                        if not p.is_alive() and r not in reported]
                if dead and q.empty():
                    _time.sleep(1.0)  # a last report may still be in the pipe
                    if q.empty():
                        errors.append((dead[0], f"process exited with code {procs[dead[0]].exitcode} "
                                                "without reporting"))
                        break
                continue
            if status == "ok":
                results[rank] = payload
            else:
                errors.append((rank, payload))
                break  # the others may now be stuck waiting for this rank
    finally:
        for p in procs:
            p.join(timeout=10)
        for p in procs:
            if p.is_alive():
                p.kill()  # exactly the children started above
                p.join()
    if errors:
        raise RuntimeError("\n".join(f"[rank {r}] {m}" for r, m in errors))
    return [results[r] for r in range(world)]
