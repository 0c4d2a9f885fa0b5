"""DDP training driver for the three workloads, synthetic data, random-init weights.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29500 -m fairring_b200.train.run --workload resnet50 --steps 20

Workloads (per-GPU batch fixed, so scaling is weak):
  decoder   26L d2048 h16 ffn8192 vocab51200 seq1024, micro-batch 8, bf16 autocast    -> words/s
  resnet50  224x224x3 N(0,1) images, batch 256, uniform labels over 1000 classes,
            bf16 autocast, fp16 gradients on the wire                                  -> images/s
  roberta   24L d2048 h32 ffn8192 vocab50265 seq512, batch 16, 15% masked tokens;
            meant to run with FAIRRING_GPUS_PER_MACHINE=2 (4 "machines" x 2 GPUs)
            and FAIRRING_TOTAL_MEMORY=52428800                                         -> words/s
Prints one JSON line on rank 0; times are CUDA events, maximum over ranks.
"""

from __future__ import annotations

import argparse
import json
import os
import socket
import sys

import torch
import torch.distributed as dist


def build_workload(name: str, preset: str, dev, rank: int, batch: int | None):
    from fairring_b200.models import (DecoderConfig, DecoderLM, EncoderConfig, EncoderMLM, ResNet50,
                                      mask_tokens)

    gen = torch.Generator().manual_seed(rank)
    if name == "decoder":
        cfg = DecoderConfig.flagship() if preset == "full" else DecoderConfig.tiny()
        b = batch or 8
        model = DecoderLM(cfg)
        pool = torch.randint(0, cfg.vocab, (4, b, cfg.seq_len + 1), generator=gen)
        split = lambda blk: (blk[:, :-1], blk[:, 1:])  # noqa: E731
        return model, pool, split, b * cfg.seq_len, "words/s"
    if name == "roberta":
        cfg = EncoderConfig.roberta_1p3b() if preset == "full" else EncoderConfig.tiny()
        b = batch or 16
        model = EncoderMLM(cfg)
        toks = torch.randint(1, cfg.vocab, (4, b, cfg.seq_len), generator=gen)
        masked, labels = mask_tokens(toks, cfg, gen)
        pool = torch.stack([masked, labels], dim=1)  # [pool, 2, b, s]
        split = lambda blk: (blk[0], blk[1])  # noqa: E731
        return model, pool, split, b * cfg.seq_len, "words/s"
    if name == "resnet50":
        b = batch or (256 if preset == "full" else 4)
        size = 224 if preset == "full" else 64
        model = ResNet50() if preset == "full" else ResNet50.tiny()
        images = torch.randn(2, b, 3, size, size, generator=gen)
        labels = torch.randint(0, 1000 if preset == "full" else 10, (2, b), generator=gen)
        pool = list(zip(images, labels))
        split = lambda blk: blk  # noqa: E731
        return model, pool, split, b, "images/s"
    raise ValueError(name)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", choices=["decoder", "resnet50", "roberta"], default="decoder")
    ap.add_argument("--impl", choices=["fairring", "nccl"], default="fairring")
    ap.add_argument("--ddp", choices=["flat", "torch"], default="flat")
    ap.add_argument("--wire", choices=["fp32", "bf16", "fp16", "auto"], default="auto")
    ap.add_argument("--preset", choices=["full", "tiny"], default="full")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    args = ap.parse_args(argv)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "MASTER_PORT" not in os.environ:
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        os.environ["MASTER_PORT"] = str(s.getsockname()[1])
        s.close()
    os.environ.setdefault("FAIRRING_TOTAL_MEMORY", str(256 << 20))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)

    import fairring_b200
    from fairring_b200.ops import FlatAdamW
    from fairring_b200.parallel import FlatDataParallel, FusedHookState, fused_allreduce_hook
    from fairring_b200.utils import ClockSampler

    dist.init_process_group("fairring" if args.impl == "fairring" else "nccl", rank=rank,
                            world_size=world, device_id=dev if args.impl == "nccl" else None)
    torch.manual_seed(0)
    model, pool, split, items_per_step, unit = build_workload(args.workload, args.preset, dev, rank,
                                                              args.batch)
    model = model.to(dev)
    if args.workload == "resnet50":
        model = model.to(memory_format=torch.channels_last)
    wire_name = args.wire if args.wire != "auto" else ("fp16" if args.workload == "resnet50" else "fp32")
    wire = {"fp32": None, "bf16": torch.bfloat16, "fp16": torch.float16}[wire_name]

    if args.ddp == "flat" and (args.impl == "fairring" or wire is None):
        # On NCCL the flat buffers are averaged with plain all_reduce calls (no
        # fused wire cast): the two arms then differ in the backend only.
        ddp = FlatDataParallel(model, bucket_cap_mb=args.bucket_mb, wire_dtype=wire)
        opt = FlatAdamW(ddp.flat_param, ddp.flat_grad, lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1)
    else:
        from torch.distributed.algorithms.ddp_comm_hooks import default_hooks
        from torch.nn.parallel import DistributedDataParallel as DDP

        ddp = DDP(model, device_ids=[local], bucket_cap_mb=args.bucket_mb, gradient_as_bucket_view=True)
        if args.impl == "fairring":
            ddp.register_comm_hook(FusedHookState(wire_dtype=wire), fused_allreduce_hook)
        elif wire is torch.float16:
            ddp.register_comm_hook(None, default_hooks.fp16_compress_hook)
        elif wire is torch.bfloat16:
            ddp.register_comm_hook(None, default_hooks.bf16_compress_hook)
        opt = torch.optim.AdamW(ddp.parameters(), lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1, fused=True)

    def to_dev(blk):
        if isinstance(blk, tuple):
            return tuple(t.to(dev, non_blocking=True) for t in blk)
        return blk.to(dev, non_blocking=True)

    dev_pool = [to_dev(b) for b in pool]
    if args.workload == "resnet50":
        dev_pool = [(x.contiguous(memory_format=torch.channels_last), y) for x, y in dev_pool]

    def step(blk):
        a, b = split(blk)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = ddp(a, b)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(dev_pool[i % len(dev_pool)])
    sync()
    with ClockSampler(local) as clocks:
        l0 = fairring_b200.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            loss = step(dev_pool[i % len(dev_pool)])
        e1.record()
        sync()
        launches = fairring_b200.launch_count() - l0
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        desc = fairring_b200.get_backend(device="cuda").describe() if args.impl == "fairring" else ""
        print(json.dumps({
            "workload": args.workload, "preset": args.preset, "impl": args.impl, "ddp": args.ddp,
            "n_gpus": world, "value": round(world * items_per_step * args.steps / (ms / 1e3), 1),
            "unit": unit, "ms_per_step": round(ms / args.steps, 3), "steps": args.steps,
            "grad_wire_dtype": wire_name, "bucket_mb": args.bucket_mb, "data": "synthetic",
            "params": sum(p.numel() for p in model.parameters()), "loss_last": float(loss),
            "gpu_launches": int(launches), "clocks": clocks.summary(), "backend": desc,
        }), flush=True)
    sync()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
