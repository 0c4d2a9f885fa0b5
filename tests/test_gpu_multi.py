"""The backend on real GPUs, one process per GPU (needs at least two).

Each configuration spawns the ranks once and runs the whole battery of checks
inside them: all_reduce over sizes / dtypes / ops against seeded expectations,
reduce_scatter and all_gather, the fused-scale hook, delegation to NCCL, and
gradient parity of FlatDataParallel and of torch DDP on this backend with torch
DDP on NCCL.
"""

import os

import pytest
import torch

from _mp import run_ranks

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _suite(rank, world, check_ddp):
    import torch.distributed as dist

    import fairring
    import fairring_b200

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    from datetime import timedelta

    # A short group timeout: if one rank dies during set-up the others give up soon.
    dist.init_process_group("fairring", rank=rank, world_size=world, timeout=timedelta(seconds=90))
    be = fairring.get_backend(device="cuda")
    report = {}

    def seeded(n, dtype, r, salt=0):
        g = torch.Generator().manual_seed(1000 * salt + r)
        if dtype.is_floating_point:
            return torch.randn(n, generator=g).to(dtype)
        return torch.randint(0, 9, (n,), generator=g).to(dtype)

    # all_reduce: sizes x dtypes x ops
    for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.float64, torch.uint8):
        for n in (1, 33, 4099, 262_147, 3_000_001):
            for op in ("SUM", "MAX"):
                if op == "MAX" and n > 5000:
                    continue
                t = seeded(n, dtype, rank, n).to(dev)
                dist.all_reduce(t, op=getattr(dist.ReduceOp, op))
                st = torch.stack([seeded(n, dtype, r, n).double() for r in range(world)])
                expect = st.sum(0) if op == "SUM" else st.max(0).values
                tol = 5e-2 * world if dtype in (torch.float16, torch.bfloat16) else (1e-4 if dtype.is_floating_point else 0)
                torch.testing.assert_close(t.double().cpu(), expect, rtol=tol, atol=tol)
    # AVG and a big buffer (many slices, several channels)
    big = torch.full((40_000_003,), float(rank + 1), device=dev)
    dist.all_reduce(big, op=dist.ReduceOp.AVG)
    torch.testing.assert_close(big[:: 1_000_003].cpu(),
                               torch.full_like(big[:: 1_000_003].cpu(), (world + 1) / 2))
    # several collectives in flight, waited at the end
    bufs = [torch.full((2_000_000 + i,), float(rank + i), device=dev) for i in range(12)]
    works = [dist.all_reduce(b, async_op=True) for b in bufs]
    for w in works:
        w.wait()
    for i, b in enumerate(bufs):
        assert float(b[0]) == sum(r + i for r in range(world)) and float(b[-1]) == float(b[0])

    # far more collectives in flight than any fixed pool of events could hold:
    # every Work keeps its own completion event until it is destroyed
    if check_ddp:
        many = [torch.full((257,), float(rank + i % 7), device=dev) for i in range(1500)]
        works = [dist.all_reduce(b, async_op=True) for b in many]
        for w in works:
            w.wait()
        torch.cuda.synchronize()
        for i, b in enumerate(many):
            assert float(b[0]) == sum(r + i % 7 for r in range(world)) and float(b[-1]) == float(b[0])
        del many, works
        # a small blocking all_reduce runs on the caller's own stream
        before = be.stats()["gpu_inline_collectives"]
        small = torch.full((1000,), float(rank + 1), device=dev)
        dist.all_reduce(small)
        assert float(small[0]) == world * (world + 1) / 2
        assert be.stats()["gpu_inline_collectives"] == before + 1
        # symmetric memory is handed back: freed here, unmapped at the next allocation
        tmp = be.symmetric_empty(1 << 20, torch.float32)
        regions = be.stats()["symmetric_regions"]
        del tmp
        assert be.stats()["symmetric_pending_release"] == 1
        tmp2 = be.symmetric_empty(1 << 18, torch.float32)
        assert be.stats()["symmetric_pending_release"] == 0
        assert be.stats()["symmetric_regions"] == regions
        del tmp2
        assert be.release_symmetric() == 1

    # a big ordinary tensor (the pipelined kernel when enabled), odd length
    x = seeded(12_000_001, torch.float32, rank, 9).to(dev)
    dist.all_reduce(x)
    expect = torch.stack([seeded(12_000_001, torch.float32, r, 9).double() for r in range(world)]).sum(0)
    torch.testing.assert_close(x.double().cpu(), expect, rtol=1e-4, atol=1e-4)

    # fused scale + bf16 wire
    g = seeded(1_000_003, torch.float32, rank, 77).to(dev)
    be.allreduce_fused(g, 1.0 / world, torch.bfloat16, "sum").wait()
    expect = torch.stack([(seeded(1_000_003, torch.float32, r, 77).double() / world).bfloat16().double()
                          for r in range(world)]).sum(0)
    torch.testing.assert_close(g.double().cpu(), expect, rtol=2e-2, atol=2e-2)

    # tensors in symmetric memory are reduced in place, without staging
    sym = be.symmetric_empty(6_000_000, torch.float32)
    for lo, hi in ((0, 6_000_000), (1024, 4_001_024), (64, 128)):
        sym.copy_(seeded(6_000_000, torch.float32, rank, 5).to(dev))
        dist.all_reduce(sym[lo:hi])
        expect = torch.stack([seeded(6_000_000, torch.float32, r, 5).double() for r in range(world)]).sum(0)
        mine = seeded(6_000_000, torch.float32, rank, 5).double()
        mine[lo:hi] = expect[lo:hi]
        torch.testing.assert_close(sym.double().cpu(), mine, rtol=1e-4, atol=1e-4)
    be.allreduce_fused(sym, 1.0 / world, None, "sum").wait()
    torch.cuda.synchronize()
    report["direct_launches"] = be.stats()["launch_direct_allreduce"] + be.stats()["launch_nvls_direct_allreduce"]

    # reduce_scatter / all_gather (tensor and list forms)
    n = 70_001
    inp = torch.arange(world * n, dtype=torch.float32, device=dev) * (rank + 1)
    out = torch.empty(n, device=dev)
    dist.reduce_scatter_tensor(out, inp)
    torch.testing.assert_close(out.cpu(), torch.arange(world * n, dtype=torch.float32)[rank * n:(rank + 1) * n]
                               * sum(range(1, world + 1)))
    ag = torch.empty(world * n, device=dev)
    dist.all_gather_into_tensor(ag, torch.full((n,), float(rank), device=dev))
    assert torch.equal(ag.cpu(), torch.arange(world).repeat_interleave(n).float())
    outs = [torch.empty(7, device=dev) for _ in range(world)]
    dist.all_gather(outs, torch.full((7,), float(rank * 3), device=dev))
    for r in range(world):
        assert float(outs[r][0]) == r * 3
    o = torch.empty(5, device=dev)
    dist.reduce_scatter(o, [torch.full((5,), float(rank + i), device=dev) for i in range(world)])
    assert float(o[0]) == sum(r + rank for r in range(world))

    # delegated ops run on NCCL
    b = torch.full((4,), float(rank), device=dev)
    dist.broadcast(b, src=world - 1)
    assert float(b[0]) == world - 1
    p = torch.full((3,), 2.0, device=dev)
    dist.all_reduce(p, op=dist.ReduceOp.PRODUCT)
    assert float(p[0]) == 2.0 ** world
    dist.barrier()

    if check_ddp:
        from torch.nn.parallel import DistributedDataParallel as DDP

        from fairring_b200.models import DecoderConfig, DecoderLM
        from fairring_b200.parallel import FlatDataParallel, FusedHookState, fused_allreduce_hook

        cfg = DecoderConfig.tiny()
        torch.manual_seed(0)
        base = DecoderLM(cfg).to(dev)
        state = {k: v.clone() for k, v in base.state_dict().items()}
        tok = torch.randint(0, cfg.vocab, (4, cfg.seq_len + 1), generator=torch.Generator().manual_seed(rank)).to(dev)

        def grads_of(wrapper_fn):
            m = DecoderLM(cfg).to(dev)
            m.load_state_dict(state)
            w = wrapper_fn(m)
            loss = w(tok[:, :-1], tok[:, 1:])
            loss.backward()
            torch.cuda.synchronize()
            if isinstance(w, FlatDataParallel):
                return [g.clone() for g in w.grads()]  # backward (reverse registration) order
            return [p.grad.clone() for p in m.parameters()]

        nccl_pg = dist.new_group(backend="nccl")
        ref = grads_of(lambda m: DDP(m, device_ids=[rank], process_group=nccl_pg))
        drop_in = grads_of(lambda m: DDP(m, device_ids=[rank]))
        for a, b_ in zip(ref, drop_in):
            torch.testing.assert_close(a, b_, rtol=1e-4, atol=1e-6)

        def hooked(m):
            d = DDP(m, device_ids=[rank])
            d.register_comm_hook(FusedHookState(), fused_allreduce_hook)
            return d

        fused = grads_of(hooked)
        for a, b_ in zip(ref, fused):
            torch.testing.assert_close(a, b_, rtol=1e-4, atol=1e-6)
        flat = grads_of(lambda m: FlatDataParallel(m, bucket_cap_mb=0.25))
        ref_rev = list(reversed(ref))
        for i, a in enumerate(ref_rev):
            torch.testing.assert_close(a, flat[i], rtol=1e-4, atol=1e-6)
        report["ddp"] = "ok"

    be.check_health()
    tr = be.trace()
    assert tr and int(tr[-1]["seq"]) == be.stats()["gpu_collectives"] - 1
    assert all(int(t["launches"]) >= 1 for t in tr if int(t["bytes"]) > 0)
    report["stats"] = be.stats()
    report["describe"] = be.describe()
    dist.destroy_process_group()
    return report


CONFIGS = {
    "auto": {},
    "twoshot_no_nvls": {"FAIRRING_NVLS": "off", "FAIRRING_ALGO": "twoshot"},
    "nvls": {"FAIRRING_ALGO": "nvls"},
    "nvls_oneshot": {"FAIRRING_ALGO": "nvls_oneshot"},
    "pipe": {"FAIRRING_ALGO": "pipe", "FAIRRING_DIRECT": "nvls"},
    "pipe_p2p": {"FAIRRING_ALGO": "pipe", "FAIRRING_NVLS": "off"},
    "pipe_off": {"FAIRRING_PIPE": "off"},
    # in-place launches of 4 blocks between staged and flag-in-data launches of 16
    "narrow_in_place": {"FAIRRING_DIRECT": "nvls", "FAIRRING_DIRECT_BLOCKS": "4", "FAIRRING_PIPE": "off"},
    "hier_three_kernels": {"FAIRRING_ALGO": "hier", "FAIRRING_NVLS": "off"},
    "ipc_transport_cmd_thread": {"FAIRRING_TRANSPORT": "ipc", "FAIRRING_COMMAND_THREAD": "1"},
    "machines_of_one_gpu": {"FAIRRING_GPUS_PER_MACHINE": "1", "FAIRRING_NVLS": "off"},
    "machines_of_two_gpus": {"FAIRRING_GPUS_PER_MACHINE": "2", "FAIRRING_RANK_LAYOUT": "favorable"},
}


@pytest.mark.parametrize("name", list(CONFIGS))
def test_backend_on_gpus(name):
    if _ngpu() < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if _ngpu() < 4 else 4
    env = dict(CONFIGS[name])
    env.setdefault("FAIRRING_TOTAL_MEMORY", str(64 << 20))
    env["FAIRRING_DEVICE_TIMEOUT_MS"] = "5000"
    res = run_ranks(_suite, world, env=env, args=(name == "auto",), timeout=240)
    stats = res[0]["stats"]
    assert stats["gpu_collectives"] > 50
    if "FAIRRING_GPUS_PER_MACHINE" not in env:
        assert res[0]["direct_launches"] > 0
    if name == "twoshot_no_nvls":
        assert stats["nvls"] == 0 and stats["launch_twoshot_allreduce"] > 0
    if name in ("nvls", "nvls_oneshot") and stats["nvls"] == 1:
        assert stats["launch_nvls_allreduce"] + stats["launch_nvls_oneshot_allreduce"] > 0
    if name.startswith("pipe") and name != "pipe_off":
        assert stats["launch_pipe_allreduce"] > 0
    if name in ("pipe_off", "narrow_in_place"):
        assert stats["launch_pipe_allreduce"] == 0
    if name == "narrow_in_place" and stats["nvls"] == 1:
        assert stats["launch_nvls_direct_allreduce"] > 0
    if name == "hier_three_kernels":
        assert stats["launch_rs_intragroup"] > 0 and stats["launch_ag_intragroup"] > 0
    if name == "machines_of_two_gpus" and world >= 4:
        assert stats["launch_shard_server_reduce"] > 0 and stats["launch_rs_intragroup"] > 0
    if name == "machines_of_one_gpu":
        assert stats["launch_shard_server_reduce"] > 0


@pytest.mark.parametrize("gpm,layout", [(2, "favorable"), (4, "standard")])
def test_groupings_on_8_gpus(gpm, layout):
    if _ngpu() < 8:
        pytest.skip("needs eight GPUs")
    env = {"FAIRRING_GPUS_PER_MACHINE": str(gpm), "FAIRRING_RANK_LAYOUT": layout,
           "FAIRRING_TOTAL_MEMORY": str(64 << 20), "FAIRRING_DEVICE_TIMEOUT_MS": "20000"}
    res = run_ranks(_suite, 8, env=env, args=(False,), timeout=900)
    assert res[0]["stats"]["launch_shard_server_reduce"] > 0


# --- a rank stays away from one collective: time-out, report, reset, carry on -----
def _absent_rank(rank, world):
    """Host-made failure, no GPU fault: rank 1 simply does not call one
    all_reduce.  Rank 0's kernel waits for its limit (1 s), records whom it was
    waiting for and returns; the blocking wait raises; both ranks learn of it
    through the store, reset the engine together and the next all_reduce works."""
    import time
    from datetime import timedelta

    import torch.distributed as dist

    import fairring

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("fairring", rank=rank, world_size=world, timeout=timedelta(seconds=60))
    be = fairring.get_backend(device="cuda")
    store = dist.distributed_c10d._get_default_store()
    x = torch.ones(1 << 20, device=dev)
    dist.all_reduce(x)  # healthy
    torch.cuda.synchronize()
    assert float(x[0]) == world
    outcome = "n/a"
    if rank == 0:
        y = torch.ones(1 << 20, device=dev)
        t0 = time.time()
        try:
            dist.all_reduce(y)  # FAIRRING_BLOCKING_WAIT=1: wait() watches the kernel
            outcome = "completed"
        except RuntimeError as e:
            outcome = str(e)
        elapsed = time.time() - t0
        store.set("rank0_outcome", "done")
    else:
        store.wait(["rank0_outcome"])  # never joined the second collective
        elapsed = 0.0
    # the GPU is still fine
    z = torch.arange(10, device=dev).sum().item()
    assert z == 45
    err_before = str(be.get_error()) if hasattr(be, "get_error") else ""
    be.reset()
    w = torch.full((1 << 20,), float(rank + 1), device=dev)
    dist.all_reduce(w)
    torch.cuda.synchronize()
    after = float(w[0])
    dist.destroy_process_group()
    return outcome, elapsed, after


def test_absent_rank_times_out_and_engine_recovers():
    if _ngpu() < 2:
        pytest.skip("needs at least two GPUs")
    env = {"FAIRRING_NVLS": "off", "FAIRRING_DEVICE_TIMEOUT_MS": "1000", "FAIRRING_BLOCKING_WAIT": "1",
           "FAIRRING_TOTAL_MEMORY": str(64 << 20), "NCCL_NVLS_ENABLE": "0"}
    res = run_ranks(_absent_rank, 2, env=env, timeout=180)
    outcome, elapsed, after = res[0]
    assert "failed state" in outcome or "timed out" in outcome, outcome
    assert "rank 1" in outcome
    assert elapsed < 20
    assert res[0][2] == 3.0 and res[1][2] == 3.0


# --- the reference-sequence comparison arm (NCCL calls in the reference's order) ---------
def _refseq(rank, world, gpm):
    import torch.distributed as dist

    from fairring_b200.bench.refseq import ReferenceSequence

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    rs = ReferenceSequence(world, rank, gpm, dev)
    out = []
    for n in (8, 1000, 1 << 20, (1 << 20) + 3):
        x = torch.full((n,), float(rank + 1), device=dev)
        for _ in range(3):  # back to back: stages of consecutive calls overlap
            rs.all_reduce(x)
        torch.cuda.synchronize()
        out.append((float(x[0]), float(x[-1])))
    dist.destroy_process_group()
    return out


@pytest.mark.parametrize("gpm", [1, 2])
def test_reference_sequence_arm(gpm):
    if _ngpu() < 2:
        pytest.skip("needs at least two GPUs")
    res = run_ranks(_refseq, 2, env={}, args=(gpm,), timeout=180)
    expect = 3.0 * 2 * 2  # (1 + 2), then doubled twice
    for first, last in res[0]:
        assert first == expect and last == expect, res[0]


# --- several GPUs in one process: one tensor per GPU, one merged Work -----------------
def _gpus_in_one_process(rank, world, per_proc):
    import torch.distributed as dist

    import fairring

    from datetime import timedelta

    devs = [torch.device("cuda", rank * per_proc + i) for i in range(per_proc)]
    torch.cuda.set_device(devs[0])
    dist.init_process_group("fairring", rank=rank, world_size=world, timeout=timedelta(seconds=60))
    be = fairring.get_backend(device="cuda")
    total = world * per_proc
    out = []
    for n in (1000, 3_000_001):
        ts = [torch.full((n,), float(rank * per_proc + i + 1), device=d) for i, d in enumerate(devs)]
        w = be.allreduce(ts)
        w.wait()
        for d in devs:
            torch.cuda.synchronize(d)
        out.append([float(t[0]) for t in ts] + [float(t[-1]) for t in ts])
    # the merged Future (what a DDP-style consumer would chain on)
    ts = [torch.full((70_000,), 2.0, device=d) for d in devs]
    fut = be.allreduce(ts).get_future()
    fut.wait()
    for d in devs:
        torch.cuda.synchronize(d)
    out.append([float(t[0]) for t in fut.value()])
    assert total * (total + 1) / 2 == out[0][0]
    dist.destroy_process_group()
    return out


def test_two_gpus_in_one_process():
    if _ngpu() < 2:
        pytest.skip("needs at least two GPUs")
    env = {"FAIRRING_TOTAL_MEMORY": str(64 << 20), "FAIRRING_DEVICE_TIMEOUT_MS": "5000"}
    res = run_ranks(_gpus_in_one_process, 1, env=env, args=(2,), timeout=150)
    small, big, fut = res[0]
    assert all(v == 3.0 for v in small) and all(v == 3.0 for v in big)
    assert fut == [4.0, 4.0]


def test_two_processes_of_two_gpus():
    if _ngpu() < 4:
        pytest.skip("needs at least four GPUs")
    env = {"FAIRRING_TOTAL_MEMORY": str(64 << 20), "FAIRRING_DEVICE_TIMEOUT_MS": "5000"}
    res = run_ranks(_gpus_in_one_process, 2, env=env, args=(2,), timeout=240)
    for r in (0, 1):
        small, big, fut = res[r]
        assert all(v == 10.0 for v in small) and all(v == 10.0 for v in big)
        assert fut == [8.0, 8.0]
