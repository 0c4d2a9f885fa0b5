"""Tuning sweep: one process group per configuration (blocks x channels x
kernel variant), a few message sizes each, bus GB/s on the device.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29500 -m fairring_b200.bench.tune --sizes 1048576,16777216,268435456

The size -> variant table the engine uses by default was chosen from the
output of this tool.
"""

from __future__ import annotations

import argparse
import itertools
import json
import os
import sys

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="1048576,16777216,134217728")
    ap.add_argument("--blocks", default="16,32,64")
    ap.add_argument("--channels", default="2,4,8")
    ap.add_argument("--variants", default="twoshot,nvls,bounce,sym_p2p,sym_nvls")
    ap.add_argument("--dtype", default="fp32")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--nccl", action="store_true", help="also time NCCL on the same buffers")
    args = ap.parse_args(argv)

    import fairring_b200

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("FAIRRING_TOTAL_MEMORY", str(256 << 20))
    dist.init_process_group("fairring", rank=rank, world_size=world)
    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[args.dtype]
    es = torch.empty((), dtype=dtype).element_size()
    sizes = [int(x) for x in args.sizes.split(",")]
    arena_bytes = max(1 << 30, max(sizes))
    arena = torch.randn(arena_bytes // es, device=dev, dtype=dtype)

    def measure(group, buf, size):
        n = size // es
        slots = max(1, buf.numel() // n)

        def call(i):
            dist.all_reduce(buf[(i % slots) * n:((i % slots) + 1) * n], group=group)

        for i in range(5):
            call(i)
        torch.cuda.synchronize()
        dist.barrier(group=group)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.iters):
            call(i)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / args.iters], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        us = float(t.item())
        buf.normal_()
        return us, 2 * (world - 1) / world * size / (us * 1e-6) / 1e9

    rows = []
    if args.nccl:
        g = dist.new_group(backend="nccl")
        for size in sizes:
            us, bw = measure(g, arena, size)
            rows.append({"variant": "nccl", "blocks": 0, "channels": 0, "bytes": size,
                         "us": round(us, 1), "busbw": round(bw, 1)})
    for variant, blocks, channels in itertools.product(
            args.variants.split(","), [int(b) for b in args.blocks.split(",")],
            [int(c) for c in args.channels.split(",")]):
        if blocks * channels > 144:
            continue
        os.environ["FAIRRING_BLOCKS"] = str(blocks)
        os.environ["FAIRRING_SM_BUDGET"] = "148"
        os.environ["FAIRRING_PARALLELISM"] = str(channels)
        os.environ["FAIRRING_ALGO"] = {"twoshot": "twoshot", "nvls": "nvls", "bounce": "bounce"}.get(variant, "auto")
        os.environ["FAIRRING_DIRECT"] = {"sym_p2p": "p2p", "sym_nvls": "nvls"}.get(variant, "off")
        os.environ["FAIRRING_ONESHOT_MAX"] = "0"
        os.environ["FAIRRING_BOUNCE"] = "on" if variant == "bounce" else "off"
        g = dist.new_group(backend="fairring")
        be = fairring_b200.get_backend(g, "cuda")
        buf = arena
        if variant.startswith("sym"):
            buf = be.symmetric_empty(arena.numel(), dtype)
            buf.normal_()
        for size in sizes:
            us, bw = measure(g, buf, size)
            rows.append({"variant": variant, "blocks": blocks, "channels": channels, "bytes": size,
                         "us": round(us, 1), "busbw": round(bw, 1)})
        be.check_health()
        del buf
        dist.destroy_process_group(g)
    if rank == 0:
        print(f"{'variant':10} {'blocks':>6} {'chan':>5} " + " ".join(f"{s:>14}" for s in sizes))
        by = {}
        for r in rows:
            by.setdefault((r["variant"], r["blocks"], r["channels"]), {})[r["bytes"]] = r["busbw"]
        for (v, b, c), d in by.items():
            print(f"{v:10} {b:6d} {c:5d} " + " ".join(f"{d.get(s, 0):14.1f}" for s in sizes))
        for r in rows:
            print(json.dumps(r))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
