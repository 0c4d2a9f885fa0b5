"""Kernel breakdown of one training step of the decoder workload on one GPU.

    python -m fairring_b200.bench.step_profile --steps 2 --rows 40

Builds what ``bench.py`` builds for its default arm (flat data-parallel wrapper
with bf16 shadow weights, fused AdamW, the fused LayerNorm / loss kernels),
runs a few warm-up steps, then profiles ``--steps`` steps with
``torch.profiler`` and prints the device time per kernel and per step, largest
first.  Times under the profiler are for reading shares, not for quoting a step
time: that is ``bench.py``'s job.
"""

from __future__ import annotations

import argparse
import os
import socket
import sys

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--rows", type=int, default=40, help="kernels to list")
    ap.add_argument("--tiny", action="store_true", help="the small test model instead of the 1.4 B one")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("step_profile needs a CUDA device", file=sys.stderr)
        return 1

    os.environ.setdefault("FAIRRING_TOTAL_MEMORY", str(256 << 20))
    import torch.distributed as dist
    from torch.profiler import ProfilerActivity, profile

    import fairring_b200  # noqa: F401  (registers the backend)
    from fairring_b200.models import DecoderConfig, DecoderLM
    from fairring_b200.ops import FlatAdamW
    from fairring_b200.parallel import FlatDataParallel

    torch.cuda.set_device(0)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    dist.init_process_group("fairring", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    cfg = DecoderConfig.tiny() if args.tiny else DecoderConfig.flagship()
    model = DecoderLM(cfg).cuda()
    ddp = FlatDataParallel(model, bf16_shadow=True)
    opt = FlatAdamW(ddp.flat_param, ddp.flat_grad, lr=1e-4, betas=(0.9, 0.95), weight_decay=0.1,
                    shadow=ddp.flat_shadow, overlap=ddp)
    tok = torch.randint(0, cfg.vocab, (8, cfg.seq_len + 1), device="cuda")

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = ddp(tok[:, :-1], tok[:, 1:])
        loss.backward()
        opt.step()

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(args.steps):
            step()
        torch.cuda.synchronize()
    rows = [(e.self_device_time_total / args.steps / 1e3, e.count // max(1, args.steps), e.key)
            for e in prof.key_averages() if e.self_device_time_total > 0]
    rows.sort(reverse=True)
    total = sum(r[0] for r in rows)
    print(f"device time of all kernels: {total:.2f} ms per step")
    print("ms/step | launches/step | kernel")
    for ms, n, name in rows[: args.rows]:
        print(f"{ms:7.2f} | {n:5d} | {name[:110]}")
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
