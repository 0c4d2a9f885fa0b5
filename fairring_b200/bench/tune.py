"""Tuning sweep: times the all-reduce kernels over their tunables on ONE process
group (the tunables are switched at run time with ``backend.set_option``) and
writes the thresholds it finds to ``fairring_b200/tuning.json``, which
``options_from_env`` loads for the matching world size.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29500 -m fairring_b200.bench.tune --what direct,pipe,small,nccl

Every time is measured on the device with CUDA events around a train of
back-to-back blocking calls, each on a different slice of an arena larger than
L2, and is the maximum over ranks.  busbw = 2 (W-1)/W * bytes / time.

Parts (``--what``):

direct   in-place NVLS kernel on symmetric memory: blocks x channels x unroll
pipe     pipelined kernel on ordinary memory: blocks x chunk size
small    4 KiB .. 4 MiB on ordinary memory, every small-message kernel
nccl     NCCL on the same ordinary arena, and on NCCL-registered memory when
         this PyTorch offers the allocator
"""

from __future__ import annotations

import argparse
import itertools
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ALGO = {"auto": 0, "oneshot": 1, "twoshot": 2, "hier": 3, "nvls": 4, "nvls_oneshot": 5, "pipe": 6, "ll": 7,
        "ll2": 8}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--what", default="direct,pipe,small,nccl")
    ap.add_argument("--dtype", default="fp32")
    ap.add_argument("--big-sizes", default="8388608,33554432,268435456")
    ap.add_argument("--pipe-sizes", default="4194304,16777216,33554432,67108864,134217728,268435456")
    ap.add_argument("--pipe-blocks", default="8,16,32")
    ap.add_argument("--pipe-chunks", default="1048576,4194304,16777216")
    ap.add_argument("--iters", type=int, default=15)
    ap.add_argument("--json", default="", help="write all rows to this file")
    ap.add_argument("--merge", default="", help="a --json file of an earlier run: its rows stand in for "
                    "the parts that this run does not measure")
    ap.add_argument("--write-table", action="store_true",
                    help="write fairring_b200/tuning.json from what was measured")
    args = ap.parse_args(argv)
    what = set(args.what.split(","))

    os.environ.setdefault("FAIRRING_TOTAL_MEMORY", str(1 << 30))
    os.environ.setdefault("FAIRRING_SM_BUDGET", "148")
    os.environ.setdefault("FAIRRING_PARALLELISM", "4")
    os.environ.setdefault("FAIRRING_LL_MAX", str(256 << 10))
    os.environ.setdefault("FAIRRING_LL2_MAX", str(4 << 20))
    os.environ.setdefault("FAIRRING_PIPE_SLOTS", "4")
    os.environ.setdefault("FAIRRING_PIPE_CHANNELS", "1")
    os.environ["FAIRRING_TUNING_TABLE"] = "off"
    import fairring_b200

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("fairring", rank=rank, world_size=world)
    side = dist.new_group(backend="gloo")
    be = fairring_b200.get_backend(device="cuda")
    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[args.dtype]
    es = torch.empty((), dtype=dtype).element_size()
    arena = torch.randn((1 << 30) // es, device=dev, dtype=dtype)
    warm = torch.ones(1024, device=dev)
    dist.all_reduce(warm)  # builds the engine
    torch.cuda.synchronize()

    def measure(buf, size, group=None, iters=None):
        n = size // es
        slots = max(1, buf.numel() // n)
        iters = iters or (args.iters if size >= (4 << 20) else 100)

        def call(i):
            j = i % slots
            dist.all_reduce(buf[j * n:(j + 1) * n], group=group)

        for i in range(4):
            call(i)
        torch.cuda.synchronize()
        dist.barrier(group=side)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            call(i)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=side)
        us = float(t.item())
        return us, 2 * (world - 1) / world * size / (us * 1e-6) / 1e9

    def setopt(**kw):
        for k, v in kw.items():
            be.set_option(k, int(v))

    rows = []

    def add(part, cfg, size, us, bw):
        rows.append({"part": part, **cfg, "bytes": size, "us": round(us, 2), "busbw": round(bw, 1)})
        if rank == 0:
            print(json.dumps(rows[-1]), flush=True)

    big = [int(x) for x in args.big_sizes.split(",")]

    if "nccl" in what:
        g = dist.new_group(backend="nccl")
        sizes = sorted(set(big + [int(x) for x in args.pipe_sizes.split(",")] +
                           [1 << k for k in range(12, 23)]))
        for size in sizes:
            us, bw = measure(arena, size, group=g)
            add("nccl", {"memory": "ordinary"}, size, us, bw)
        try:
            nccl_be = g._get_backend(dev)
            pool = torch.cuda.MemPool(nccl_be.mem_allocator)
            with torch.cuda.use_mem_pool(pool):
                reg = torch.empty((256 << 20) // es, device=dev, dtype=dtype)
            reg.normal_()
            nccl_be.register_mem_pool(pool)
            for size in sizes:
                us, bw = measure(reg, size, group=g)
                add("nccl", {"memory": "registered (ncclMemAlloc pool)"}, size, us, bw)
            del reg
        except Exception as e:  # noqa: BLE001
            rows.append({"part": "nccl", "memory": "registered", "unavailable": str(e)[:200]})
        arena.normal_()

    if "direct" in what and world > 1:
        sym = be.symmetric_empty((512 << 20) // es, dtype)
        sym.normal_()
        setopt(direct_min_slice_bytes=1 << 20)
        for blocks, slices, unroll in itertools.product((4, 6, 8, 12, 16), (1, 2), (4, 8)):
            setopt(direct_blocks=blocks, direct_max_slices=slices, direct_unroll=unroll)
            for size in big:
                us, bw = measure(sym, size)
                add("direct", {"blocks": blocks, "channels": slices, "unroll": unroll}, size, us, bw)
            sym.normal_()
        setopt(direct_blocks=0, direct_max_slices=2, direct_unroll=8, direct_min_slice_bytes=2 << 20)
        be.check_health()

    if "pipe" in what and world > 1:
        setopt(algo=ALGO["pipe"], ll_max_bytes=0)
        for blocks, chunk in itertools.product([int(x) for x in args.pipe_blocks.split(",")],
                                               [int(x) for x in args.pipe_chunks.split(",")]):
            setopt(pipe_blocks=blocks, pipe_chunk_bytes=chunk)
            for size in [int(x) for x in args.pipe_sizes.split(",")]:
                us, bw = measure(arena, size)
                add("pipe", {"blocks": blocks, "chunk": chunk}, size, us, bw)
            arena.normal_()
        for stage, stages in ((32 << 10, 3),):
            setopt(pipe_blocks=16, pipe_chunk_bytes=2 << 20, pipe_stage_bytes=16, pipe_stages=2)
            setopt(pipe_stages=stages, pipe_stage_bytes=stage)
            for size in (33554432, 268435456):
                us, bw = measure(arena, size)
                add("pipe", {"blocks": 16, "chunk": 2 << 20, "stage": stage, "stages": stages}, size, us, bw)
        setopt(pipe_stage_bytes=16, pipe_stages=2)
        setopt(pipe_stages=6, pipe_stage_bytes=16 << 10, pipe_blocks=16, pipe_chunk_bytes=0)
        # the staged kernels on the same messages (sliced over the channels)
        for name in ("nvls", "twoshot"):
            setopt(algo=ALGO[name])
            for size in [int(x) for x in args.pipe_sizes.split(",")]:
                us, bw = measure(arena, size)
                add("staged", {"variant": name}, size, us, bw)
        setopt(algo=ALGO["auto"], ll_max_bytes=32 << 10)
        be.check_health()

    if "small" in what and world > 1:
        sizes = [1 << k for k in range(12, 23)]
        variants = [("ll inline", dict(algo=ALGO["ll"], inline_small=1, ll_max_bytes=256 << 10), 256 << 10),
                    ("ll side-stream", dict(algo=ALGO["ll"], inline_small=0, ll_max_bytes=256 << 10), 256 << 10),
                    ("ll2", dict(algo=ALGO["ll2"], ll_max_bytes=0, ll2_max_bytes=4 << 20), 4 << 20),
                    ("oneshot", dict(algo=ALGO["oneshot"], ll_max_bytes=0), 1 << 20),
                    ("nvls_oneshot", dict(algo=ALGO["nvls_oneshot"], ll_max_bytes=0), 4 << 20),
                    ("nvls twoshot", dict(algo=ALGO["nvls"], ll_max_bytes=0), 4 << 20),
                    ("pipe", dict(algo=ALGO["pipe"], ll_max_bytes=0, pipe_min_bytes=0), 4 << 20)]
        for name, opts, cap in variants:
            setopt(**opts)
            for size in sizes:
                if size > cap:
                    continue
                us, bw = measure(arena, size)
                add("small", {"variant": name}, size, us, bw)
            arena.normal_()
        setopt(algo=ALGO["auto"], ll_max_bytes=32 << 10, ll2_max_bytes=1 << 20, inline_small=1,
               pipe_min_bytes=64 << 20)
        be.check_health()

    if rank == 0:
        if args.merge and os.path.exists(args.merge):
            with open(args.merge) as f:
                earlier = json.load(f)["rows"]
            mine = {r.get("part") for r in rows}
            rows = [r for r in earlier if r.get("part") not in mine] + rows
        if args.json:
            with open(args.json, "w") as f:
                json.dump({"describe": be.describe(), "world": world, "dtype": args.dtype, "rows": rows}, f, indent=1)
        if args.write_table:
            table = derive_table(rows, world)
            path = Path(fairring_b200.__file__).resolve().parent / "tuning.json"
            old = json.loads(path.read_text()) if path.exists() else {}
            old[str(world)] = table
            path.write_text(json.dumps(old, indent=1, sort_keys=True) + "\n")
            print("# wrote", path, json.dumps(table))
    dist.barrier(group=side)
    # Registered NCCL pools and sub-groups do not always come down in order at
    # interpreter exit; everything has been printed, leave directly.
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def derive_table(rows, world):
    """Thresholds from the measured rows: per size the fastest small-message
    kernel; the best (blocks, channels, unroll) of the in-place kernel at 32 MiB
    and the best (blocks, chunk) of the pipelined kernel at 32 MiB."""
    table = {}
    small = {}
    for r in rows:
        if r.get("part") == "small":
            small.setdefault(r["bytes"], {})[r["variant"]] = r["us"]
    best = {size: min(v, key=v.get) for size, v in small.items()}
    ll_max = max([s for s, b in best.items() if b.startswith("ll ")], default=0)
    ll2_max = max([s for s, b in best.items() if b == "ll2"], default=0)
    oneshot_max = max([s for s, b in best.items() if b == "oneshot"], default=0)
    nvls1_max = max([s for s, b in best.items() if b == "nvls_oneshot"], default=0)
    pipe_min = min([s for s, b in best.items() if b == "pipe"], default=0)
    if ll_max:
        table["ll_max_bytes"] = ll_max
    table["ll2_max_bytes"] = ll2_max
    table["oneshot_max_bytes"] = max(oneshot_max, ll_max)
    table["nvls_oneshot_max_bytes"] = max(nvls1_max, table["oneshot_max_bytes"])
    direct = [r for r in rows if r.get("part") == "direct" and r["bytes"] == 33554432]
    if direct:
        top = max(direct, key=lambda r: r["busbw"])
        # the smallest footprint within 3 % of the best
        ok = [r for r in direct if r["busbw"] >= 0.97 * top["busbw"]]
        pick = min(ok, key=lambda r: (r["blocks"] * r["channels"], -r["busbw"]))
        table["direct_blocks"] = pick["blocks"]
        table["direct_max_slices"] = pick["channels"]
        table["direct_unroll"] = pick["unroll"]
    big = max([r["bytes"] for r in rows if r.get("part") == "pipe"], default=0)
    pipe = [r for r in rows if r.get("part") == "pipe" and r["bytes"] == big and "stage" not in r]
    if pipe:
        top = max(pipe, key=lambda r: r["busbw"])
        ok = [r for r in pipe if r["busbw"] >= 0.97 * top["busbw"]]
        pick = min(ok, key=lambda r: (r["blocks"], -r["busbw"]))
        table["pipe_blocks"] = pick["blocks"]
        table["pipe_chunk_bytes"] = pick["chunk"]
        # from which size on does that configuration beat the staged kernels?
        mine = {r["bytes"]: r["us"] for r in rows if r.get("part") == "pipe" and "stage" not in r
                and r["blocks"] == pick["blocks"] and r["chunk"] == pick["chunk"]}
        staged = {}
        for r in rows:
            if r.get("part") == "staged":
                staged[r["bytes"]] = min(staged.get(r["bytes"], 1e30), r["us"])
        wins = None
        for size in sorted(mine, reverse=True):
            if size in staged and mine[size] < staged[size]:
                wins = size
            else:
                break
        table["pipe_min_bytes"] = wins if wins is not None else 1 << 40
    return table


if __name__ == "__main__":
    sys.exit(main())
