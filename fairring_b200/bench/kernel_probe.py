"""Run ONE kernel of the library a few times on one GPU and report its device
time (for roofline arithmetic, and as the small, self-ending workload to put
under ``ncu``).

    python -m fairring_b200.bench.kernel_probe --kernel twoshot --world 8 --mib 16
    python -m fairring_b200.bench.kernel_probe --kernel adamw --mib 256

Collective kernels run with all ``--world`` ranks emulated on this GPU (one
cooperative launch, grid.y = rank), so "peer" traffic is local HBM traffic: the
numbers characterise the kernel's memory pipeline, not NVLink.
"""

from __future__ import annotations

import argparse
import json
import sys

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="twoshot",
                    choices=["oneshot", "twoshot", "hier", "direct", "ll", "pipe", "adamw", "sumsq",
                             "layernorm", "cross_entropy"])
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--gpus-per-machine", type=int, default=0, help="hier: group size (default world/2)")
    ap.add_argument("--mib", type=float, default=16.0, help="message (or buffer) size per rank, MiB")
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--blocks", type=int, default=16)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--chunk-kib", type=int, default=1024, help="pipe: chunk (and ring slot) size")
    args = ap.parse_args(argv)

    from torch.profiler import ProfilerActivity, profile

    import fairring_b200

    C = fairring_b200._C
    torch.cuda.set_device(0)
    dtype = torch.float32 if args.dtype == "fp32" else torch.bfloat16
    es = 4 if args.dtype == "fp32" else 2
    n = int(args.mib * (1 << 20)) // es
    n -= n % (4 * args.world * 16)
    W = args.world

    if args.kernel in ("adamw", "sumsq"):
        p, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        if args.kernel == "adamw":
            fn = lambda i: C.adamw_flat_(p, g, m, v, 1e-3, 0.9, 0.95, 1e-8, 0.1, i + 1, 1.0)  # noqa: E731
            algo_bytes = n * 4 * 7  # read p,g,m,v; write p,m,v
            pattern = "adamw_flat"
        else:
            fn = lambda i: C.sumsq(g)  # noqa: E731
            algo_bytes = n * 4
            pattern = "sumsq"
    elif args.kernel == "layernorm":
        # the decoder's shape: rows of 2048 (fp32 residual stream, or bf16) in, bf16 out
        cols = 2048
        rows = max(1, int(args.mib * (1 << 20)) // (es * cols))
        x = torch.randn(rows, cols, device="cuda", dtype=dtype)
        dy = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
        gamma, beta = torch.ones(cols, device="cuda"), torch.zeros(cols, device="cuda")
        state = {}

        def fn(i):
            y, mean, rstd = C.layer_norm_fwd(x, gamma, beta, 1e-5, torch.bfloat16)
            state["out"] = C.layer_norm_bwd(dy, x, gamma, mean, rstd)

        # forward: read x, write y; backward: read dy and x, write dx (statistics are per row)
        algo_bytes = rows * cols * (3 * es + 2 * 2)
        pattern = "layer_norm_fwd_kernel|layer_norm_bwd_kernel|layer_norm_param_grad_kernel"
    elif args.kernel == "cross_entropy":
        vocab = 51200
        rows = max(1, int(args.mib * (1 << 20)) // (2 * vocab))
        logits = torch.randn(rows, vocab, device="cuda", dtype=torch.bfloat16)
        targets = torch.randint(0, vocab, (rows,), device="cuda")
        one = torch.ones(1, device="cuda")

        def fn(i):
            logits.normal_()
            loss, lse = C.cross_entropy_fwd(logits, targets)
            C.cross_entropy_bwd_(logits, targets, lse, one, 1.0 / rows)

        # forward: read the logits once (the second sweep of a row hits L2); backward: read + write
        algo_bytes = rows * vocab * 2 * 3
        pattern = "cross_entropy_fwd_kernel|cross_entropy_bwd_kernel"
    elif args.kernel == "pipe":
        ins = [torch.randn(n, device="cuda").to(dtype) for _ in range(W)]
        fn = lambda i: C.emulated_pipe_allreduce(  # noqa: E731
            ins, blocks=args.blocks, chunk_bytes=args.chunk_kib << 10, slot_bytes=args.chunk_kib << 10,
            slots=4, stage_bytes=16 << 10, stages=6, scale=1.0 / W)
        nb = n * es
        # copy-in (read + write), reduce (W reads, W writes of 1/W each), copy-out (read + write)
        algo_bytes = (2 * nb + 2 * nb + 2 * nb) * W
        pattern = "pipe_allreduce"
    else:
        ins = [torch.randn(n, device="cuda").to(dtype) for _ in range(W)]
        gpm = W
        if args.kernel == "hier":
            gpm = args.gpus_per_machine or max(1, W // 2)
        half = max(1 << 20, W * n * es if args.kernel == "oneshot" else n * es)
        fn = lambda i: C.emulated_collective(  # noqa: E731
            "allreduce", ins, gpm, algo=args.kernel, blocks=args.blocks, half_bytes=half)
        nb = n * es
        # HBM bytes the algorithm has to move, summed over the W emulated ranks.
        per_rank = {"ll": nb * (1 + 2 * W) + 2 * nb * W + nb,  # every 8 bytes travel as 16
                    "oneshot": nb * (1 + W) + nb * W + nb,      # read in, write W copies; read W, write out
                    "twoshot": 2 * nb + (nb + nb / W) + 2 * nb,  # push; reduce; gather
                    "hier": 2 * nb + (nb + nb / W) + 2 * nb,     # (plus the shard-server pass when M > 1)
                    "direct": nb + nb}[args.kernel]              # read every copy of own chunk, write every copy
        algo_bytes = per_rank * W
        pattern = {"ll": "ll_allreduce", "oneshot": "oneshot_allreduce", "twoshot": "twoshot_allreduce",
                   "hier": "rs_intragroup|shard_server_reduce|ag_intragroup",
                   "direct": "direct_allreduce"}[args.kernel]

    fn(0)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for i in range(args.iters):
            fn(i + 1)
        torch.cuda.synchronize()
    import re

    total_us, calls = 0.0, 0
    names = []
    each = {}
    for e in prof.key_averages():
        if re.search(pattern, e.key):
            total_us += e.device_time_total
            calls = max(calls, e.count)
            names.append(e.key[:80])
            short = re.sub(r"<.*", "", e.key.split("::")[-1])
            each[short] = round(each.get(short, 0.0) + e.device_time_total / max(1, args.iters), 1)
    per_call_us = total_us / max(1, args.iters)
    print(json.dumps({
        "kernel": args.kernel, "world": W, "bytes_per_rank": n * es, "dtype": args.dtype,
        "blocks_per_rank": args.blocks, "device_us_per_call": round(per_call_us, 1),
        "algorithmic_hbm_bytes": int(algo_bytes),
        "achieved_gbs": round(algo_bytes / (per_call_us * 1e-6) / 1e9, 1) if per_call_us else None,
        "us_per_kernel": each, "kernels": names,
    }))
    return 0


if __name__ == "__main__":
    sys.exit(main())
