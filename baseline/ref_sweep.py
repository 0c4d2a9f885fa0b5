"""All-reduce sweep of the UNMODIFIED reference (installed under baseline/_ref):
bus GB/s versus message size, through the reference's own public API
(``import fairring; init_process_group("fairring"); dist.all_reduce``).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 baseline/ref_sweep.py --min-bytes 4096 --max-bytes 1073741824

Same method as ``fairring_b200.bench.sweep``: CUDA events around a train of
back-to-back blocking calls on different slices of an arena larger than L2,
maximum over ranks.  Nothing of ``fairring_b200`` is imported.  On one box every
rank is the same machine for the reference (it tells machines apart by boot
id), so this is its single-machine path: NCCL reduce-scatter + NCCL all-gather
on its own streams (fairring/device.cc:444-634).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
sys.path[:] = [os.path.join(HERE, "_ref")] + [p for p in sys.path if os.path.abspath(p or ".") not in (REPO, HERE)]

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--min-bytes", type=int, default=4096)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--dtypes", default="fp32,bf16")
    ap.add_argument("--json", default="")
    args = ap.parse_args()

    import fairring  # the reference

    assert os.path.abspath(fairring.__file__).startswith(os.path.join(HERE, "_ref")), fairring.__file__
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("fairring", rank=rank, world_size=world)
    side = dist.new_group(backend="gloo")
    arena_bytes = max(1 << 30, args.max_bytes)
    rows = []
    for dname in args.dtypes.split(","):
        dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[dname]
        es = torch.empty((), dtype=dtype).element_size()
        arena = torch.randn(arena_bytes // es, device=dev, dtype=dtype)
        size = args.min_bytes
        while size <= args.max_bytes:
            n = size // es
            slots = max(1, arena.numel() // n)
            iters = 200 if size <= (1 << 20) else (40 if size <= (64 << 20) else 10)

            def call(i):
                j = i % slots
                dist.all_reduce(arena[j * n:(j + 1) * n])

            for i in range(5):
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
            busbw = 2 * (world - 1) / world * size / (us * 1e-6) / 1e9
            rows.append({"backend": "reference", "dtype": dname, "bytes": size, "us": round(us, 2),
                         "busbw_gbs": round(busbw, 2), "world": world})
            arena.normal_()
            size *= 2
        del arena
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
        if args.json:
            with open(args.json, "w") as f:
                json.dump({"rows": rows}, f, indent=1)
    dist.barrier(group=side)
    sys.stdout.flush()
    os._exit(0)  # the reference leaks its streams on purpose; skip finalizers


if __name__ == "__main__":
    main()
