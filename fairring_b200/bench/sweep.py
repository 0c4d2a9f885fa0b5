"""All-reduce sweep: bus GB/s versus message size, this backend next to NCCL.

Run one process per GPU, e.g.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29500 -m fairring_b200.bench.sweep --min-bytes 4096 --max-bytes 1073741824

Backends (``--backends``): ``fairring``; ``nccl`` (ordinary memory);
``nccl_reg`` (NCCL on memory from its own registered allocator, the fair
counterpart of ``--symmetric``); ``refseq`` (the reference's per-slice NCCL
sequence, see ``fairring_b200.bench.refseq``).

Contiguous fp32 and bf16 buffers, values N(0,1) seeded per rank, sizes in
powers of two.  Every time is measured on the device with CUDA events around a
train of back-to-back calls, each on a different slice of an arena larger than
L2, and is the maximum over ranks.  busbw = 2 (W-1)/W * bytes / time.
The grouping (1x8, 2x4, 4x2) comes from FAIRRING_GPUS_PER_MACHINE as usual.
FAIRRING_TOTAL_MEMORY defaults to 512 MiB here (the engine's line in the JSON
says what it made of it).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def _time_train(fn_for_index, iters: int) -> float:
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn_for_index(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / iters  # microseconds per call


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--min-bytes", type=int, default=4096)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--dtypes", default="fp32,bf16")
    ap.add_argument("--backends", default="fairring,nccl")
    ap.add_argument("--arena-bytes", type=int, default=1 << 30)
    ap.add_argument("--check", action="store_true", help="verify one result per size")
    ap.add_argument("--symmetric", action="store_true",
                    help="put the fairring arena in symmetric memory (in-place kernels, no staging)")
    ap.add_argument("--json", default="", help="also write the rows to this file")
    args = ap.parse_args(argv)

    # Staging for ordinary tensors: the library's default budget (50 MiB, the
    # reference's) is sized for small GPUs; the sweep gives it 512 MiB of the 180 GB.
    os.environ.setdefault("FAIRRING_TOTAL_MEMORY", str(512 << 20))
    import fairring_b200  # registers the backend

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("fairring", rank=rank, world_size=world)
    side = dist.new_group(backend="gloo")  # the harness's own bookkeeping
    groups = {}
    nccl_group = None
    refseq = None
    for b in args.backends.split(","):
        if b == "fairring":
            groups[b] = dist.group.WORLD
        elif b in ("nccl", "nccl_reg"):
            nccl_group = nccl_group or dist.new_group(backend="nccl")
            groups[b] = nccl_group
        elif b == "refseq":
            from .refseq import ReferenceSequence

            gpm = int(os.environ.get("FAIRRING_GPUS_PER_MACHINE", "0")) or world
            refseq = ReferenceSequence(world, rank, gpm, dev,
                                       favorable=os.environ.get("FAIRRING_RANK_LAYOUT", "standard") == "favorable")
            groups[b] = None
        else:
            raise SystemExit(f"unknown backend {b}")

    arena_bytes = max(args.arena_bytes, args.max_bytes)
    rows = []
    for dname in args.dtypes.split(","):
        dtype = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[dname]
        es = torch.empty((), dtype=dtype).element_size()
        gen = torch.Generator(device=dev).manual_seed(rank)
        arena = torch.randn(arena_bytes // es, generator=gen, device=dev, dtype=dtype)
        sym_arena = None
        if args.symmetric and "fairring" in groups:
            sym_arena = fairring_b200.get_backend(device="cuda").symmetric_empty(arena.numel(), dtype)
            sym_arena.copy_(arena)
        reg_arena, reg_note = None, ""
        if "nccl_reg" in groups:
            try:
                nccl_be = nccl_group._get_backend(dev)
                pool = torch.cuda.MemPool(nccl_be.mem_allocator)
                with torch.cuda.use_mem_pool(pool):
                    reg_arena = torch.empty(arena.numel(), device=dev, dtype=dtype)
                reg_arena.copy_(arena)
                nccl_be.register_mem_pool(pool)
            except Exception as e:  # noqa: BLE001
                reg_arena, reg_note = None, f"unavailable: {str(e)[:160]}"
        size = args.min_bytes
        while size <= args.max_bytes:
            n = size // es
            slots = max(1, (arena_bytes // es) // n)
            iters = 200 if size <= (1 << 20) else (40 if size <= (64 << 20) else 10)
            for bname, group in groups.items():
                buf = sym_arena if (bname == "fairring" and sym_arena is not None) else arena
                if bname == "nccl_reg":
                    if reg_arena is None:
                        if size == args.min_bytes:
                            rows.append({"backend": bname, "dtype": dname, "note": reg_note})
                        continue
                    buf = reg_arena

                def call(i, n=n, slots=slots, group=group, buf=buf, bname=bname):
                    j = i % slots
                    if bname == "refseq":
                        refseq.all_reduce(buf[j * n:(j + 1) * n])
                    else:
                        dist.all_reduce(buf[j * n:(j + 1) * n], group=group)

                for i in range(5):
                    call(i)
                torch.cuda.synchronize()
                dist.barrier(group=side)
                us = _time_train(call, iters)
                t = torch.tensor([us], dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=side)
                us = float(t.item())
                busbw = 2 * (world - 1) / world * size / (us * 1e-6) / 1e9 if world > 1 else 0.0
                rows.append({"backend": bname + ("(symmetric)" if buf is sym_arena and sym_arena is not None else ""),
                             "dtype": dname, "bytes": size, "us": round(us, 2),
                             "algbw_gbs": round(size / (us * 1e-6) / 1e9, 2),
                             "busbw_gbs": round(busbw, 2), "world": world})
                # values drift as the arena is summed over and over: renormalise
                buf.copy_(torch.randn(arena.shape, generator=gen, device=dev, dtype=dtype))
            if args.check:
                x = torch.full((n,), float(rank + 1), device=dev, dtype=dtype)
                dist.all_reduce(x)
                expect = world * (world + 1) / 2
                assert float(x[0]) == expect and float(x[-1]) == expect, (size, float(x[0]), expect)
            size *= 2
        del arena

    if rank == 0:
        be = fairring_b200.get_backend(device="cuda")
        print("# " + be.describe())
        print(f"{'dtype':6} {'bytes':>12} " + " ".join(f"{b + ' us':>14} {b + ' busGB/s':>16}" for b in groups))
        by = {}
        for r in rows:
            if "bytes" in r:
                by.setdefault((r["dtype"], r["bytes"]), {})[r["backend"].split("(")[0]] = r
        for (dname, size), d in by.items():
            print(f"{dname:6} {size:12d} " + " ".join(
                f"{d[b]['us']:14.2f} {d[b]['busbw_gbs']:16.2f}" if b in d else f"{'-':>14} {'-':>16}"
                for b in groups))
        for r in rows:
            print(json.dumps(r))
        if args.json:
            with open(args.json, "w") as f:
                json.dump({"describe": be.describe(), "rows": rows}, f, indent=1)
    dist.barrier(group=side)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
