"""The "fairring" backend on CPU tensors, as real processes (no GPU needed).

The host path runs the same algorithm as the GPU kernels on POSIX shared
memory, so these tests cover slicing, the (machine, device) index maps, the
double-buffered staging, delegation and the bounded waits.
"""

import numpy as np
import pytest
import torch

from _mp import run_ranks


def _init(rank, world):
    import torch.distributed as dist

    import fairring  # noqa: F401  (registers the backend)

    dist.init_process_group("fairring", rank=rank, world_size=world)
    return dist


def _inputs(sizes, world, dtype=torch.float32):
    out = []
    for r in range(world):
        g = torch.Generator().manual_seed(r)
        out.append([torch.randn(n, generator=g).to(dtype) for n in sizes])
    return out


# --- the plumbing configuration: 1 KiB, 1 MiB, 25 MiB fp32, N(0,1) seed = rank,
#     FAIRRING_SLICE_SIZE = 4 MiB, exact elementwise sum, world_size 2 --------
SIZES = [1024 // 4, (1 << 20) // 4, (25 << 20) // 4]


def _w_plumbing(rank, world):
    dist = _init(rank, world)
    mine = _inputs(SIZES, world)[rank]
    for t in mine:
        dist.all_reduce(t)
    be = __import__("fairring").get_backend(device="cpu")
    stats = be.stats()
    dist.destroy_process_group()
    return [t.numpy() for t in mine], stats


def test_plumbing_config_exact_sum():
    world = 2
    res = run_ranks(_w_plumbing, world, env={"FAIRRING_SLICE_SIZE": 4 << 20})
    ins = _inputs(SIZES, world)
    for i, n in enumerate(SIZES):
        # two addends: fp32 addition is commutative, so the sum is exact
        expect = (ins[0][i] + ins[1][i]).numpy()
        for r in range(world):
            np.testing.assert_array_equal(res[r][0][i], expect)
    stats = res[0][1]
    assert stats["cpu_collectives"] == 3
    # 25 MiB at 4 MiB per slice: 7 slices; 1 MiB: 1 slice; 1 KiB: one-shot
    assert stats["cpu_slices"] == 1 + 1 + 7
    assert stats["cpu_oneshot"] == 1


# --- dtypes and reduction ops ------------------------------------------------
DTYPES = [torch.uint8, torch.int8, torch.int32, torch.int64, torch.float16, torch.bfloat16,
          torch.float32, torch.float64]


def _w_dtypes(rank, world):
    dist = _init(rank, world)
    out = {}
    for dt in DTYPES:
        for op_name in ("SUM", "MAX", "MIN"):
            for n in (1, 7, 1000, 70001):
                g = torch.Generator().manual_seed(100 + rank)
                if dt.is_floating_point:
                    t = torch.randn(n, generator=g).to(dt)
                else:
                    t = torch.randint(0, 20, (n,), generator=g).to(dt)
                dist.all_reduce(t, op=getattr(dist.ReduceOp, op_name))
                out[(str(dt), op_name, n)] = t.double().numpy()
    t = torch.full((33,), float(rank + 1))
    dist.all_reduce(t, op=dist.ReduceOp.AVG)
    out["avg"] = t.numpy()
    dist.destroy_process_group()
    return out


def test_dtypes_ops_and_tails():
    world = 3
    res = run_ranks(_w_dtypes, world, env={"FAIRRING_ONESHOT_MAX": 4096})
    for dt in DTYPES:
        for op_name in ("SUM", "MAX", "MIN"):
            for n in (1, 7, 1000, 70001):
                parts = []
                for r in range(world):
                    g = torch.Generator().manual_seed(100 + r)
                    if dt.is_floating_point:
                        parts.append(torch.randn(n, generator=g).to(dt).double())
                    else:
                        parts.append(torch.randint(0, 20, (n,), generator=g).to(dt).double())
                st = torch.stack(parts)
                expect = {"SUM": st.sum(0), "MAX": st.max(0).values, "MIN": st.min(0).values}[op_name]
                for r in range(world):
                    got = res[r][(str(dt), op_name, n)]
                    tol = 0 if not dt.is_floating_point or op_name != "SUM" else (
                        5e-2 if dt in (torch.float16, torch.bfloat16) else 1e-5)
                    np.testing.assert_allclose(got, expect.numpy(), rtol=tol, atol=tol)
                # every rank must hold bit-identical results
                np.testing.assert_array_equal(res[0][(str(dt), op_name, n)],
                                              res[world - 1][(str(dt), op_name, n)])
    np.testing.assert_allclose(res[0]["avg"], np.full(33, 2.0), rtol=1e-6)


# --- hierarchy: 2 machines x 2 GPUs, both rank numberings ----------------------
def _w_hier(rank, world):
    dist = _init(rank, world)
    g = torch.Generator().manual_seed(rank)
    a = torch.randn(300_003, generator=g)
    dist.all_reduce(a)
    n = 1237
    inp = torch.arange(world * n, dtype=torch.float32) * (rank + 1)
    rs = torch.empty(n)
    dist.reduce_scatter_tensor(rs, inp)
    ag = torch.empty(world * n)
    dist.all_gather_into_tensor(ag, torch.full((n,), float(rank)) + torch.arange(n) * 0.001)
    outs = [torch.empty(5) for _ in range(world)]
    dist.all_gather(outs, torch.full((5,), float(rank * 10)))
    rs_list_out = torch.empty(4)
    dist.reduce_scatter(rs_list_out, [torch.full((4,), float(rank + i)) for i in range(world)])
    be = __import__("fairring").get_backend(device="cpu")
    dep, stats = be.deployment(), be.stats()
    dist.destroy_process_group()
    return a.numpy(), rs.numpy(), ag.numpy(), [o.numpy() for o in outs], rs_list_out.numpy(), dep, stats


@pytest.mark.parametrize("layout", ["standard", "favorable"])
@pytest.mark.parametrize("gpm", [1, 2, 4])
def test_hierarchical_groupings(layout, gpm):
    world = 4
    res = run_ranks(_w_hier, world, env={"FAIRRING_GPUS_PER_MACHINE": gpm,
                                         "FAIRRING_RANK_LAYOUT": layout,
                                         "FAIRRING_SLICE_SIZE": 256 << 10,
                                         "FAIRRING_ONESHOT_MAX": 1024})
    parts = [torch.randn(300_003, generator=torch.Generator().manual_seed(r)).double() for r in range(world)]
    expect = torch.stack(parts).sum(0).numpy()
    n = 1237
    for r in range(world):
        a, rs, ag, outs, rsl, dep, stats = res[r]
        np.testing.assert_allclose(a, expect, rtol=1e-5, atol=1e-5)
        np.testing.assert_array_equal(a, res[0][0])
        base = np.arange(world * n, dtype=np.float64)[r * n:(r + 1) * n]
        np.testing.assert_allclose(rs, base * sum(range(1, world + 1)), rtol=1e-6)
        exp_ag = np.concatenate([np.full(n, float(q)) + np.arange(n) * 0.001 for q in range(world)])
        np.testing.assert_allclose(ag, exp_ag, rtol=1e-6)
        for q in range(world):
            np.testing.assert_array_equal(outs[q], np.full(5, q * 10.0))
        np.testing.assert_array_equal(rsl, np.full(4, float(sum(q + r for q in range(world)))))
        assert dep["D"] == gpm and dep["M"] == world // gpm
        assert dep["favorable"] == (1 if layout == "favorable" else 0)
        if gpm < world:
            assert stats["cpu_hierarchical"] > 0
        else:
            assert stats["cpu_twoshot"] > 0


# --- delegation -------------------------------------------------------------------
def _w_delegate(rank, world):
    dist = _init(rank, world)
    t = torch.full((4,), float(rank))
    dist.broadcast(t, src=1)
    p = torch.full((3,), float(rank + 2))
    dist.all_reduce(p, op=dist.ReduceOp.PRODUCT)  # not a fairring op: goes to gloo
    b = torch.tensor([True, False]) if rank == 0 else torch.tensor([True, True])
    gathered = [None] * world
    dist.all_gather_object(gathered, {"rank": rank})
    dist.barrier()
    be = __import__("fairring").get_backend(device="cpu")
    stats = be.stats()
    dist.destroy_process_group()
    return t.numpy(), p.numpy(), gathered, stats


def test_delegation_to_gloo():
    world = 2
    res = run_ranks(_w_delegate, world)
    for r in range(world):
        t, p, gathered, stats = res[r]
        np.testing.assert_array_equal(t, np.full(4, 1.0))
        np.testing.assert_array_equal(p, np.full(3, 6.0))
        assert gathered == [{"rank": 0}, {"rank": 1}]
        assert stats["delegated"] >= 3


# --- failure detection: a rank stays away from a barrier ------------------------------
def _w_timeout(rank, world):
    dist = _init(rank, world)
    be = __import__("fairring").get_backend(device="cpu")
    t = torch.ones(100_000)
    dist.all_reduce(t)  # healthy collective first (also creates the engine)
    if rank == 1:
        be.skip_cpu_signals(1000)  # rank 1 stops announcing itself at barriers
    try:
        dist.all_reduce(t)
        outcome = "completed"
    except RuntimeError as e:
        outcome = str(e)
    return outcome


def test_peer_that_never_signals_times_out():
    res = run_ranks(_w_timeout, 2, env={"FAIRRING_DEVICE_TIMEOUT_MS": 300})
    assert "timed out" in res[0] and "rank 1" in res[0]


# --- several hosts: the shared-memory path must step aside ------------------------------
def _w_two_hosts(rank, world):
    import os

    os.environ["FAIRRING_BOOT_ID"] = f"host-{rank}"
    dist = _init(rank, world)
    t = torch.full((10,), float(rank + 1))
    dist.all_reduce(t)
    be = __import__("fairring").get_backend(device="cpu")
    dep, stats = be.deployment(), be.stats()
    dist.destroy_process_group()
    return t.numpy(), dep, stats


def test_ranks_on_different_hosts_are_delegated():
    res = run_ranks(_w_two_hosts, 2)
    for t, dep, stats in res:
        np.testing.assert_array_equal(t, np.full(10, 3.0))
        assert dep["num_hosts"] == 2 and dep["single_host"] == 0
        assert stats["delegated"] >= 1 and "cpu_collectives" not in stats


# --- torch DDP on CPU tensors through this backend (Future plumbing, parity with gloo) ----
def _w_ddp_cpu(rank, world):
    import torch.nn as nn
    from torch.nn.parallel import DistributedDataParallel as DDP

    dist = _init(rank, world)
    gloo = dist.new_group(backend="gloo")
    torch.manual_seed(0)
    base = nn.Sequential(nn.Linear(32, 64), nn.Tanh(), nn.Linear(64, 8))
    state = {k: v.clone() for k, v in base.state_dict().items()}
    x = torch.randn(16, 32, generator=torch.Generator().manual_seed(rank))

    def grads(pg):
        m = nn.Sequential(nn.Linear(32, 64), nn.Tanh(), nn.Linear(64, 8))
        m.load_state_dict(state)
        d = DDP(m, process_group=pg, bucket_cap_mb=0.001)
        d(x).pow(2).sum().backward()
        return [p.grad.clone() for p in m.parameters()]

    mine, ref = grads(None), grads(gloo)
    work = dist.all_reduce(torch.ones(10), async_op=True)
    fut = work.get_future()
    fut.wait()
    ok = work.is_completed() and work.is_success()
    dist.destroy_process_group()
    return [g.numpy() for g in mine], [g.numpy() for g in ref], ok


def test_torch_ddp_on_cpu_matches_gloo():
    res = run_ranks(_w_ddp_cpu, 2)
    for mine, ref, ok in res:
        assert ok
        for a, b in zip(mine, ref):
            np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-6)
    for a, b in zip(res[0][0], res[1][0]):
        np.testing.assert_array_equal(a, b)


def test_options_from_env(monkeypatch):
    import fairring_b200

    monkeypatch.setenv("FAIRRING_TOTAL_MEMORY", "1234567")
    monkeypatch.setenv("FAIRRING_SLICE_SIZE", "4194304")
    monkeypatch.setenv("FAIRRING_PARALLELISM", "3")
    monkeypatch.setenv("FAIRRING_GPUS_PER_MACHINE", "4")
    monkeypatch.setenv("FAIRRING_RANK_LAYOUT", "favorable")
    monkeypatch.setenv("FAIRRING_ALGO", "HIER")
    o = fairring_b200.options_from_env()
    assert o.max_memory_allocated_in_bytes == 1234567 and o.slice_size_in_bytes == 4194304
    assert o.min_parallelism == 3 and o.gpus_per_machine == 4 and o.favorable_layout
    assert o.algo == "hier" and o.is_high_priority_stream
    monkeypatch.delenv("FAIRRING_TOTAL_MEMORY")
    o = fairring_b200.options_from_env()
    assert o.max_memory_allocated_in_bytes == 50 * 1024 * 1024  # the reference's default
    monkeypatch.setenv("FAIRRING_RANK_LAYOUT", "sideways")
    with pytest.raises(ValueError):
        fairring_b200.options_from_env()


# --- the process group can be torn down and built again in the same processes ----------
def _w_reinit(rank, world, folder):
    import torch.distributed as dist

    import fairring  # noqa: F401

    out = []
    for generation in range(3):
        # A rendezvous file per generation: with one TCP port for all of them a fast
        # rank can reach the slow rank's store of the generation before, which then goes away.
        dist.init_process_group("fairring", rank=rank, world_size=world,
                                init_method=f"file://{folder}/generation{generation}")
        t = torch.full((50_000,), float(rank + generation))
        dist.all_reduce(t)
        out.append(float(t[0]))
        dist.barrier()
        dist.destroy_process_group()
    return out


def test_process_group_can_be_rebuilt(tmp_path):
    res = run_ranks(_w_reinit, 2, args=(str(tmp_path),))
    for r in res:
        assert r == [1.0, 3.0, 5.0]
