"""Where does a data-parallel step lose time to communication?

Builds the flagship decoder once (FlatDataParallel + fused AdamW, as bench.py
does) and times the same training step under several settings of the in-place
all-reduce, switched at run time:

* ``no_sync``: backward with the all-reduce skipped (compute only, at this
  clock and power state);
* the all-reduce with B blocks per kernel on C channels (SM footprint B x C);
* the exposed tail: device time between the end of backward's last kernel and
  the moment the optimizer may start (the wait on the last buckets).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29500 -m fairring_b200.bench.ddp_breakdown --steps 6

Times are CUDA-event device times, maximum over ranks.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--preset", choices=["flagship", "tiny"], default="flagship")
    ap.add_argument("--configs", default="16x2,8x2,8x1,16x1,24x1,32x2")
    ap.add_argument("--unrolls", default="8")
    ap.add_argument("--no-tail-overlap", action="store_true",
                    help="wait for the last bucket at the end of backward instead of inside the optimizer")
    ap.add_argument("--json", default="")
    args = ap.parse_args(argv)

    os.environ.setdefault("FAIRRING_TOTAL_MEMORY", str(256 << 20))
    os.environ.setdefault("FAIRRING_SM_BUDGET", "148")
    os.environ.setdefault("FAIRRING_PARALLELISM", "4")
    import fairring_b200
    from fairring_b200.models import DecoderConfig, DecoderLM
    from fairring_b200.ops import FlatAdamW
    from fairring_b200.parallel import FlatDataParallel

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("fairring", rank=rank, world_size=world)
    side = dist.new_group(backend="gloo") if world > 1 else None
    cfg = DecoderConfig.flagship() if args.preset == "flagship" else DecoderConfig.tiny()
    torch.manual_seed(0)
    model = DecoderLM(cfg).to(dev)
    ddp = FlatDataParallel(model, bf16_shadow=True)
    opt = FlatAdamW(ddp.flat_param, ddp.flat_grad, lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1,
                    shadow=ddp.flat_shadow, overlap=None if args.no_tail_overlap else ddp)
    be = fairring_b200.get_backend(device="cuda") if world > 1 else None
    B, S = 8, cfg.seq_len
    tok = torch.randint(0, cfg.vocab, (B, S + 1), generator=torch.Generator().manual_seed(rank)).to(dev)

    # Instrument the end of backward: an event when the last gradient hook has
    # run, another after the waits on the all-reduces.
    marks = {}
    orig_finish = ddp._finish_backward

    def finish():
        marks["bwd_end"] = torch.cuda.Event(enable_timing=True)
        marks["bwd_end"].record()
        orig_finish()
        marks["ready"] = torch.cuda.Event(enable_timing=True)
        marks["ready"].record()

    ddp._finish_backward = finish

    def step(sync: bool):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = ddp(tok[:, :-1], tok[:, 1:])
        if sync:
            loss.backward()
        else:
            with ddp.no_sync():
                loss.backward()
        opt.step()

    def maxr(x: float) -> float:
        if side is None:
            return x
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=side)
        return float(t.item())

    def timed(sync: bool):
        for _ in range(2):
            step(sync)
        torch.cuda.synchronize()
        if side is not None:
            dist.barrier(group=side)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        tails = []
        e0.record()
        for _ in range(args.steps):
            step(sync)
            tails.append((marks["bwd_end"], marks["ready"]))
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.steps
        tail = sum(a.elapsed_time(b) for a, b in tails) / len(tails)
        return maxr(ms), maxr(tail)

    rows = []
    ms, tail = timed(False)
    rows.append({"setting": "no_sync (compute only)", "ms_per_step": round(ms, 2), "exposed_tail_ms": round(tail, 3)})
    if world > 1:
        for spec in args.configs.split(","):
            blocks, chans = (int(x) for x in spec.split("x"))
            for unroll in (int(u) for u in args.unrolls.split(",")):
                be.set_option("blocks", blocks)
                be.set_option("direct_max_slices", chans)
                be.set_option("direct_unroll", unroll)
                ms, tail = timed(True)
                rows.append({"setting": f"all-reduce {blocks} blocks x {chans} channels, unroll {unroll}",
                             "sms": blocks * chans, "ms_per_step": round(ms, 2),
                             "exposed_tail_ms": round(tail, 3)})
        be.check_health()
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
        if args.json:
            with open(args.json, "w") as f:
                json.dump({"world": world, "rows": rows,
                           "describe": be.describe() if be is not None else "single rank"}, f, indent=1)
    if side is not None:
        dist.barrier(group=side)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
