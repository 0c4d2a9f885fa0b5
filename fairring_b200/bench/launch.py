"""Bucket micro-benchmark launcher: one invocation per machine.

    python -m fairring_b200.bench.launch --num-devices-per-machine 8 \\
        --num-buckets 64 --bucket-size 6553600 --num-epochs 10 --output /tmp/stats.pt

Spawns one process per GPU (``spawn`` context, one pipe each), lets every child
rendezvous through ``--init-method`` to obtain a store, builds either the
fairring backend or NCCL's directly on that store and runs the native
``BenchClient`` (N buckets all-reduced per epoch, all in flight).  The parent
gathers the per-epoch microseconds into a ``[devices, epochs]`` tensor, saves it
with ``torch.save`` and prints the derived bus bandwidth.  Counterpart of
benchmark/launch_benchmark.py in the reference; the times are device-side
(CUDA events) rather than host wall-clock.
"""

from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import os
import sys
from datetime import timedelta


def run_one_device(conn, args, machine_idx: int, device_idx: int) -> None:
    try:
        # Every child sees all GPUs and selects its own: peer mappings between
        # processes need the peers' devices to be visible.  (The reference hides
        # the others with CUDA_VISIBLE_DEVICES, launch_benchmark.py:51.)
        for k in ("NCCL_SOCKET_NTHREADS", "NCCL_NSOCKS_PERTHREAD"):
            v = getattr(args, k.lower())
            if v is not None:
                os.environ[k] = str(v)
        os.environ["FAIRRING_PARALLELISM"] = str(args.parallelism)
        if args.total_memory is not None:
            os.environ["FAIRRING_TOTAL_MEMORY"] = str(args.total_memory)
        os.environ.setdefault("FAIRRING_TOTAL_MEMORY", str(50 << 20))
        if args.gpus_per_group:
            os.environ["FAIRRING_GPUS_PER_MACHINE"] = str(args.gpus_per_group)

        import torch
        import torch.distributed as dist

        import fairring_b200
        from fairring_b200 import _C

        torch._C._set_print_stack_traces_on_fatal_signal(True)
        world = args.num_machines * args.num_devices_per_machine
        rank = machine_idx * args.num_devices_per_machine + device_idx
        rdv = dist.rendezvous(args.init_method, rank, world)
        store, _, _ = next(rdv)
        torch.cuda.set_device(device_idx)
        timeout = timedelta(seconds=args.timeout)
        if args.use_nccl:
            opts = dist.ProcessGroupNCCL.Options()
            opts._timeout = timeout
            backend = dist.ProcessGroupNCCL(store, rank, world, opts)
        else:
            backend = fairring_b200.create_process_group_fairring(store, rank, world, timeout)
        dtype = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[args.dtype]
        client = _C.BenchClient(backend, args.num_buckets, args.bucket_size, dtype,
                                args.num_epochs, args.warmup_epochs, args.gaussian,
                                not args.no_check, device_idx)
        stats = client.run()
        desc = "" if args.use_nccl else backend.describe()
        if not args.use_nccl:
            backend.shutdown()
        conn.send({"us": stats, "describe": desc})
    except BaseException as e:  # noqa: BLE001
        conn.send(RuntimeError(f"{type(e).__name__}: {e}"))
        raise
    finally:
        conn.close()


def run_one_machine(args):
    from .supervisor import recv_from_connections_and_join_processes

    ctx = mp.get_context("spawn")
    pairs = []
    for device_idx in range(args.num_devices_per_machine):
        parent, child = ctx.Pipe(duplex=False)
        p = ctx.Process(target=run_one_device, args=(child, args, args.machine_idx, device_idx),
                        name=f"bench-m{args.machine_idx}-d{device_idx}")
        p.start()
        child.close()
        pairs.append((p, parent))
    return recv_from_connections_and_join_processes(pairs, timeout=args.timeout + 120)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="fairring bucket all-reduce benchmark (one call per machine)")
    ap.add_argument("--init-method", default="tcp://127.0.0.1:29533")
    ap.add_argument("--machine-idx", type=int, default=0)
    ap.add_argument("--num-machines", type=int, default=1)
    ap.add_argument("--num-devices-per-machine", type=int, required=True)
    ap.add_argument("--num-buckets", type=int, default=64)
    ap.add_argument("--bucket-size", type=int, default=25 * 1024 * 1024 // 4, help="elements per bucket")
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16", "fp16"])
    ap.add_argument("--num-epochs", type=int, default=10)
    ap.add_argument("--warmup-epochs", type=int, default=2)
    ap.add_argument("--use-nccl", action="store_true")
    ap.add_argument("--parallelism", type=int, default=16, help="FAIRRING_PARALLELISM")
    ap.add_argument("--total-memory", type=int, default=None, help="FAIRRING_TOTAL_MEMORY")
    ap.add_argument("--gpus-per-group", type=int, default=0, help="FAIRRING_GPUS_PER_MACHINE")
    ap.add_argument("--gaussian", action="store_true", help="N(0,1) inputs instead of ones")
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--nccl-socket-nthreads", type=int, default=None)
    ap.add_argument("--nccl-nsocks-perthread", type=int, default=None)
    ap.add_argument("--timeout", type=float, default=300.0)
    ap.add_argument("--output", default="")
    args = ap.parse_args(argv)

    results = run_one_machine(args)
    import torch

    stats = torch.tensor([r["us"] for r in results], dtype=torch.float64)  # [devices, epochs]
    if args.output:
        torch.save(stats, args.output)
    world = args.num_machines * args.num_devices_per_machine
    es = {"fp32": 4, "bf16": 2, "fp16": 2}[args.dtype]
    total_bytes = args.num_buckets * args.bucket_size * es
    us = float(stats.max(dim=0).values.median())  # slowest device per epoch, median epoch
    out = {
        "backend": "nccl" if args.use_nccl else "fairring",
        "world": world,
        "num_buckets": args.num_buckets,
        "bucket_bytes": args.bucket_size * es,
        "epoch_us_median_of_max": round(us, 1),
        "busbw_gbs": round(2 * (world - 1) / world * total_bytes / (us * 1e-6) / 1e9, 1) if world > 1 else 0.0,
        "describe": results[0]["describe"],
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
