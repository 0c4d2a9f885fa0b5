#!/usr/bin/env python
"""Flagship benchmark: data-parallel training of the 1.37B-class decoder-only
transformer (26 layers, d_model 2048, 16 heads, FFN 8192 GELU, learned
positions, vocab 51200, seq 1024, micro-batch 8 per GPU, bf16 autocast, 25 MiB
gradient buckets); words (tokens) per second over all GPUs.  Synthetic token
ids, random-init weights.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 10 --warmup 3

Prints ONE JSON line on rank 0.  Arms (``--impl``):

``fairring``   this repository: the "fairring" backend of ``fairring_b200`` with
               ``FlatDataParallel`` + fused AdamW (``--dp flat``, default) or torch DDP
               (``--dp torch``).
``nccl``       the same model and the same ``--dp`` choice on torch's NCCL backend:
               ``--impl nccl --dp flat`` differs from the default arm in the backend only.
``reference``  the unmodified reference installed under ``baseline/_ref``: stock torch
               DDP on the reference's "fairring" backend, stock ``torch.optim.AdamW``, a
               model made of stock ``torch.nn`` layers.  Nothing of ``fairring_b200`` is
               imported on that arm.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import os
import socket
import sys
import time

REPO = os.path.dirname(os.path.abspath(__file__))

# Published end-to-end figure of the reference (Fairring, 8 x V100 + InfiniBand,
# words/s), decoded from docs/end_to_end_benchmark.svg of the reference.
PUBLISHED_WORDS_PER_S_8GPU = 2937.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["fairring", "nccl", "reference"], default="fairring")
    ap.add_argument("--dp", "--ddp", dest="dp", choices=["flat", "torch"], default=None,
                    help="flat: FlatDataParallel + fused AdamW (+ bf16 shadow weights); "
                         "torch: torch DDP + torch.optim.AdamW(fused).  Default: flat, except "
                         "for the reference arm, which is always torch DDP")
    ap.add_argument("--model", choices=["repo", "stock"], default=None,
                    help="repo: fairring_b200.models.DecoderLM; stock: the same architecture "
                         "from stock torch.nn layers (default for the reference arm)")
    ap.add_argument("--wire", choices=["fp32", "bf16"], default="fp32",
                    help="dtype of gradients on NVLink (fp32 = same as the tensors)")
    ap.add_argument("--preset", choices=["flagship", "tiny"], default="flagship")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--no-shadow", action="store_true",
                    help="let autocast cast the fp32 weights on every forward instead of keeping "
                         "a bf16 shadow copy written by the optimizer kernel")
    ap.add_argument("--no-check", action="store_true",
                    help="skip the multi-GPU correctness check that runs before the timing")
    return ap.parse_args()


def _load_by_path(name: str, path: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def _env_setup():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if "MASTER_ADDR" not in os.environ:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
    if "MASTER_PORT" not in os.environ:
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        os.environ["MASTER_PORT"] = str(s.getsockname()[1])
        s.close()
    return rank, world, local_rank


def _build_model(args, which: str):
    """Returns (model, description, vocab, seq_len)."""
    if which == "stock":
        sm = _load_by_path("bench_stock_model", os.path.join(REPO, "baseline", "stock_model.py"))
        model = sm.StockDecoderLM() if args.preset == "flagship" else sm.tiny()
        desc = (f"decoder-only transformer {model.n_layer}L d{model.d_model} h{model.n_head} "
                f"ffn{model.d_ff} vocab{model.vocab} from stock torch.nn layers")
        return model, desc, model.vocab, model.seq_len
    from fairring_b200.models import DecoderConfig, DecoderLM

    cfg = DecoderConfig.flagship() if args.preset == "flagship" else DecoderConfig.tiny()
    model = DecoderLM(cfg)
    desc = (f"decoder-only transformer {cfg.n_layer}L d{cfg.d_model} h{cfg.n_head} "
            f"ffn{cfg.d_ff} vocab{cfg.vocab}")
    return model, desc, cfg.vocab, cfg.seq_len


def _correctness_check(torch, dist, dev, rank, world, backend):
    """All-reduce / reduce-scatter / all-gather of seeded N(0,1) data through the
    backend that is about to be timed, against an fp64 sum that every rank
    recomputes from the seeds.  Raises on mismatch."""
    worst = 0.0

    def seeded(n, dtype, r, salt):
        g = torch.Generator(device=dev).manual_seed(100_003 * salt + r)
        return torch.randn(n, generator=g, device=dev, dtype=torch.float32).to(dtype)

    for dtype, tol in ((torch.float32, 1e-4), (torch.bfloat16, 0.25)):
        for n in ((1 << 18) + 3, 16 << 20):
            x = seeded(n, dtype, rank, n % 97)
            expect = torch.zeros(n, device=dev, dtype=torch.float64)
            for r in range(world):
                expect += seeded(n, dtype, r, n % 97).double()
            dist.all_reduce(x)
            err = float((x.double() - expect).abs().max())
            worst = max(worst, err if dtype == torch.float32 else 0.0)
            if err > tol * world:
                raise RuntimeError(f"all_reduce check failed: {dtype} n={n} max abs err {err}")
            del x, expect
    n = 70_001
    inp = seeded(world * n, torch.float32, rank, 5)
    out = torch.empty(n, device=dev)
    dist.reduce_scatter_tensor(out, inp)
    expect = torch.zeros(world * n, device=dev, dtype=torch.float64)
    for r in range(world):
        expect += seeded(world * n, torch.float32, r, 5).double()
    err = float((out.double() - expect[rank * n:(rank + 1) * n]).abs().max())
    if err > 1e-4 * world:
        raise RuntimeError(f"reduce_scatter check failed: max abs err {err}")
    ag = torch.empty(world * n, device=dev)
    dist.all_gather_into_tensor(ag, seeded(n, torch.float32, rank, 6))
    for r in range(world):
        if not torch.equal(ag[r * n:(r + 1) * n], seeded(n, torch.float32, r, 6)):
            raise RuntimeError("all_gather check failed")
    torch.cuda.synchronize()
    kernels = {}
    if backend is not None:
        backend.check_health()
        kernels = {k: int(v) for k, v in backend.stats().items() if k.startswith("launch_") and v}
    return {"allreduce_max_abs_err": worst, "ok": True, "kernels": kernels}


def main():
    args = parse_args()
    reference = args.impl == "reference"
    dp = "torch" if reference else (args.dp or "flat")
    which_model = args.model or ("stock" if reference else "repo")
    rank, world, local_rank = _env_setup()
    if world == 1 and args.gpus > 1:
        raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")

    if reference:
        ref_dir = os.path.join(REPO, "baseline", "_ref")
        have = os.path.isdir(ref_dir) and any(f.startswith("_fairring") and f.endswith(".so")
                                              for f in os.listdir(ref_dir))
        if not have:
            if rank == 0:
                print(json.dumps({"impl": "reference",
                                  "unavailable": "baseline/_ref holds no built reference "
                                                 "(see baseline/BUILD_LOG.md for the install command)"}))
            return 0
        # The reference's package is also called `fairring`; it must win over the
        # drop-in alias package of the same name at the repository root.
        sys.path[:] = [ref_dir] + [p for p in sys.path if os.path.abspath(p or ".") != REPO]
    else:
        sys.path.insert(0, REPO)
        os.environ.setdefault("FAIRRING_TOTAL_MEMORY", str(256 << 20))

    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    clocks_mod = _load_by_path("bench_clocks", os.path.join(REPO, "fairring_b200", "utils", "clocks.py"))

    backend = None
    launch_count = lambda: 0  # noqa: E731
    if reference:
        import fairring as ref_pkg  # noqa: F401  (registers the reference's backend)

        assert os.path.abspath(ref_pkg.__file__).startswith(ref_dir), ref_pkg.__file__
        dist.init_process_group("fairring", rank=rank, world_size=world)
    else:
        import fairring_b200

        launch_count = fairring_b200.launch_count
        if args.impl == "fairring":
            dist.init_process_group("fairring", rank=rank, world_size=world)
        else:
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    # Bookkeeping of the harness itself (max over ranks, barriers) goes through
    # a Gloo group, so that it neither helps nor burdens the timed backend.
    side = dist.new_group(backend="gloo") if world > 1 else None

    torch.manual_seed(0)
    model, model_desc, vocab, S = _build_model(args, which_model)
    model = model.to(dev)
    n_params = sum(p.numel() for p in model.parameters())
    B = args.micro_batch
    wire = torch.bfloat16 if args.wire == "bf16" else None
    lr, betas, wd = 1e-4, (0.9, 0.95), 0.1

    if dp == "flat":
        from fairring_b200.ops import FlatAdamW
        from fairring_b200.parallel import FlatDataParallel

        ddp = FlatDataParallel(model, bucket_cap_mb=args.bucket_mb, wire_dtype=wire,
                               bf16_shadow=not args.no_shadow)
        opt = FlatAdamW(ddp.flat_param, ddp.flat_grad, lr=lr, betas=betas, weight_decay=wd,
                        shadow=ddp.flat_shadow, overlap=ddp)
        parallel_desc = "flat-dp + fused AdamW" + ("" if args.no_shadow else " + bf16 shadow weights")
    else:
        from torch.nn.parallel import DistributedDataParallel as DDP

        if reference:
            # torch DDP's start-up shape check all-gathers into separately
            # allocated tensors, which the reference's all_gather rejects (it wants
            # adjacent views of one storage, fairring/utils.h:363-386); so the
            # start-up sync is done here with broadcast, which the reference
            # delegates to NCCL.
            # (async_op=True: for a blocking call torch's NCCL backend makes no
            # Future, and the reference wraps exactly that Future,
            # fairring/process_group.cc:124-129.)
            if world > 1:
                for p in model.parameters():
                    dist.broadcast(p.data, src=0, async_op=True).wait()
            ddp = DDP(model, device_ids=[local_rank], bucket_cap_mb=args.bucket_mb,
                      gradient_as_bucket_view=True, init_sync=False)
        else:
            ddp = DDP(model, device_ids=[local_rank], bucket_cap_mb=args.bucket_mb,
                      gradient_as_bucket_view=True)
            if args.impl == "fairring":
                from fairring_b200.parallel import FusedHookState, fused_allreduce_hook

                ddp.register_comm_hook(FusedHookState(wire_dtype=wire), fused_allreduce_hook)
        opt = torch.optim.AdamW(ddp.parameters(), lr=lr, betas=betas, weight_decay=wd, fused=True)
        parallel_desc = "torch DDP + torch.optim.AdamW(fused)"

    check = None
    if args.impl == "fairring":
        import fairring_b200

        if world > 1:
            backend = fairring_b200.get_backend(device="cuda")
            if not args.no_check:
                check = _correctness_check(torch, dist, dev, rank, world, backend)

    # Synthetic data: token ids uniform over the vocabulary, seed 0 (+rank), in
    # pinned host memory; one [B, S+1] block per step.
    gen = torch.Generator().manual_seed(0 + rank)
    pool_n = 4
    host_pool = torch.randint(0, vocab, (pool_n, B, S + 1), generator=gen).pin_memory()
    dev_pool = host_pool.to(dev)

    def train_step(block):
        x, y = block[:, :-1], block[:, 1:]
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = ddp(x, y)
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def sync_all():
        torch.cuda.synchronize()
        if side is not None:
            dist.barrier(group=side)

    def max_over_ranks(ms: float) -> float:
        if side is None:
            return ms
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=side)
        return float(t.item())

    W = max(args.warmup, 3)
    for i in range(W):
        train_step(dev_pool[i % pool_n])
    sync_all()

    K = args.steps
    with clocks_mod.ClockSampler(local_rank) as clocks:
        # (1) device-timed: inputs already on the GPU, nothing read back.
        launches0 = launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync_all()
        e0.record()
        for i in range(K):
            train_step(dev_pool[i % pool_n])
        e1.record()
        sync_all()
        launches = launch_count() - launches0
        ms_dev = max_over_ranks(e0.elapsed_time(e1))

        # (2) end to end: every step copies its inputs from pinned host memory
        # and reads the loss back to the host.
        staging = torch.empty((B, S + 1), dtype=torch.long, device=dev)
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync_all()
        f0.record()
        last = 0.0
        for i in range(K):
            staging.copy_(host_pool[i % pool_n], non_blocking=True)
            last = float(train_step(staging).item())
        f1.record()
        sync_all()
        ms_e2e = max_over_ranks(f0.elapsed_time(f1))

    tokens_per_step = world * B * S
    value = tokens_per_step * K / (ms_dev / 1e3)
    e2e_value = tokens_per_step * K / (ms_e2e / 1e3)
    published = PUBLISHED_WORDS_PER_S_8GPU * world / 8.0
    if rank == 0:
        desc = ""
        if backend is not None:
            desc = backend.describe()
        elif args.impl == "fairring":
            desc = "single rank: nothing is communicated"
        out = {
            "metric": "1.37B-transformer DDP words/sec",
            "value": round(value, 1),
            "unit": "words/s",
            "n_gpus": world,
            "steps": K,
            "warmup": W,
            "ms_per_step": round(ms_dev / K, 3),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": round(value / published, 2),
            "dtype": "bf16",
            "data": "synthetic",
            "impl": args.impl,
            "config": {
                "model": f"{model_desc} ({n_params / 1e9:.2f}B params)"
                         + ("" if args.preset == "flagship" else " [tiny preset: not the benchmark config]"),
                "global_batch": world * B,
                "micro_batch_per_gpu": B,
                "seq_len": S,
                "parallelism": f"dp{world}",
                "data_parallel_impl": parallel_desc,
                "bucket_mb": args.bucket_mb,
                "grad_wire_dtype": args.wire,
                "optimizer": "AdamW (step included in the timed region)",
                "precision": "fp32 params, bf16 autocast",
                "l2": "inputs larger than L2 (5.7 GB of weights streamed per step)",
                "vs_baseline_is": "value / the reference's PUBLISHED Fairring figure on other hardware "
                                  "(2937 words/s on 8 x V100 + InfiniBand, scaled to this GPU count)",
                "staging_memory_bytes": int(os.environ.get("FAIRRING_TOTAL_MEMORY", 50 << 20)),
                "backend": desc,
                "loss_last": last,
            },
            "clocks": clocks.summary(),
            "e2e": {
                "value": round(e2e_value, 1),
                "unit": "words/s",
                "ms_per_step": round(ms_e2e / K, 3),
                "h2d_bytes_per_step": int(B * (S + 1) * 8),
                "d2h_bytes_per_step": 4,
            },
            "gpu_launches": int(launches),
        }
        if check is not None:
            out["check"] = check
        if backend is not None:
            out["kernels_launched"] = {k: int(v) for k, v in backend.stats().items()
                                       if k.startswith("launch_") and v}
        print(json.dumps(out), flush=True)
    sync_all()
    if reference:
        # The reference leaves streams and recorded tensors behind that outlive the
        # CUDA context at interpreter shutdown (it leaks its streams on purpose,
        # fairring/machine.cc:162-175): leave without running finalizers.
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    t0 = time.time()
    rc = main()
    sys.exit(rc)
