"""The collective kernels against a plain PyTorch reference, on ONE GPU.

All ranks of a collective are emulated inside one cooperative launch (grid.y =
rank): the device code is exactly what runs in a multi-GPU job, only the peer
pointers are local.  Covers every kernel except the NVLS ones (which need one
GPU per rank), all dtypes, ragged tails, misaligned tensors, every grouping
and both rank numberings, the double-buffered staging (repeats) and a wait
that runs into its time limit.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.uint8, torch.int8, torch.int32, torch.int64, torch.float16, torch.bfloat16,
          torch.float32, torch.float64]


def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def _make(world, n, dtype, seed=0, offset=0):
    outs = []
    for r in range(world):
        g = torch.Generator(device="cpu").manual_seed(seed * 100 + r)
        if dtype.is_floating_point:
            t = torch.randn(n + offset, generator=g)
        else:
            t = torch.randint(0, 12, (n + offset,), generator=g)
        t = t.to(dtype).cuda()
        outs.append(t[offset:] if offset else t)
    return outs


def _ref(inputs, op):
    st = torch.stack([t.double() for t in inputs])
    return {"sum": st.sum(0), "max": st.max(0).values, "min": st.min(0).values}[op]


def _tol(dtype, world):
    if dtype in (torch.float16, torch.bfloat16):
        return dict(rtol=2e-2, atol=2e-2 * world)
    if dtype == torch.float32:
        return dict(rtol=1e-5, atol=1e-5)
    return dict(rtol=0, atol=0)


def _check_status(status):
    assert int(status[:, 0].abs().sum()) == 0, f"kernel reported a failure: {status.tolist()}"


@pytest.mark.parametrize("algo", ["oneshot", "twoshot", "hier"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_allreduce_fp32_sizes(C, algo, world):
    _need_gpu()
    for n in (1, 5, 64, 1000, 4099, 262144 + 3):
        ins = _make(world, n, torch.float32, seed=n)
        expect = _ref(ins, "sum")
        outs, status = C.emulated_collective("allreduce", [t.clone() for t in ins], world,
                                             algo=algo, blocks=4, half_bytes=64 << 20 if algo == "oneshot" else 1 << 20)
        torch.cuda.synchronize()
        _check_status(status)
        for r in range(world):
            torch.testing.assert_close(outs[r].double(), expect, rtol=1e-5, atol=1e-5)
            assert torch.equal(outs[r], outs[0]), "ranks must agree bit for bit"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("op", ["sum", "max", "min"])
def test_allreduce_dtypes_ops(C, dtype, op):
    _need_gpu()
    world = 4
    for algo in ("oneshot", "twoshot"):
        for n in (3, 1025, 70001):
            ins = _make(world, n, dtype, seed=7)
            expect = _ref(ins, op)
            outs, status = C.emulated_collective("allreduce", [t.clone() for t in ins], world,
                                                 op=op, algo=algo, blocks=3,
                                                 half_bytes=8 << 20)
            torch.cuda.synchronize()
            _check_status(status)
            for r in range(world):
                torch.testing.assert_close(outs[r].double(), expect, **_tol(dtype, world))


@pytest.mark.parametrize("gpm,favorable", [(1, False), (2, False), (2, True), (4, False), (4, True), (8, False)])
def test_allreduce_hierarchical_groupings(C, gpm, favorable):
    _need_gpu()
    world = 8
    for n in (17, 50_000, 300_003):
        ins = _make(world, n, torch.float32, seed=gpm)
        expect = _ref(ins, "sum")
        outs, status = C.emulated_collective("allreduce", [t.clone() for t in ins], gpm,
                                             favorable=favorable, algo="hier", blocks=4,
                                             half_bytes=512 << 10)  # forces several slices
        torch.cuda.synchronize()
        _check_status(status)
        for r in range(world):
            torch.testing.assert_close(outs[r].double(), expect, rtol=1e-5, atol=1e-5)
            assert torch.equal(outs[r], outs[0])


@pytest.mark.parametrize("wire", [torch.bfloat16, torch.float16])
def test_allreduce_fused_scale_and_wire_cast(C, wire):
    _need_gpu()
    world = 8
    n = 100_003
    ins = _make(world, n, torch.float32, seed=3)
    expect = torch.stack([(t.double() / world).to(wire).double() for t in ins]).sum(0)
    for algo in ("oneshot", "twoshot", "hier"):
        outs, status = C.emulated_collective("allreduce", [t.clone() for t in ins], world,
                                             scale=1.0 / world, wire_dtype=wire, algo=algo,
                                             blocks=4, half_bytes=16 << 20)
        torch.cuda.synchronize()
        _check_status(status)
        for r in range(world):
            assert outs[r].dtype == torch.float32
            torch.testing.assert_close(outs[r].double(), expect, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_allreduce_direct_in_place(C, world):
    """The zero-copy kernel: every rank reads its chunk from all ranks' tensors
    and writes the result back into all of them, no staging."""
    _need_gpu()
    for dtype in (torch.float32, torch.bfloat16, torch.int32):
        for n in (64, 4096, 1_000_000):
            ins = _make(world, n, dtype, seed=n + world)
            expect = _ref(ins, "sum")
            work = [t.clone() for t in ins]
            outs, status = C.emulated_collective("allreduce", work, world, algo="direct", blocks=4,
                                                 half_bytes=1 << 16, repeats=1)
            torch.cuda.synchronize()
            _check_status(status)
            for r in range(world):
                torch.testing.assert_close(outs[r].double(), expect, **_tol(dtype, world))
                assert torch.equal(outs[r], outs[0])
    ins = _make(world, 8192, torch.float32, seed=1)
    outs, status = C.emulated_collective("allreduce", [t.clone() for t in ins], world, algo="direct",
                                         scale=0.5, op="max", blocks=2, half_bytes=1 << 16)
    torch.cuda.synchronize()
    _check_status(status)
    torch.testing.assert_close(outs[0].double(), _ref(ins, "max") * 0.5, rtol=1e-6, atol=1e-6)


def test_allreduce_misaligned_tensor(C):
    """Tensors that do not start on a 16-byte boundary take the element-wise path."""
    _need_gpu()
    world = 4
    for dtype in (torch.float32, torch.bfloat16, torch.uint8):
        ins = _make(world, 10_001, dtype, seed=5)
        expect = _ref(ins, "sum")
        for algo in ("oneshot", "twoshot"):
            views = []
            for t in ins:
                buf = torch.empty(t.numel() + 1, dtype=dtype, device="cuda")
                v = buf[1:]  # data_ptr is off by one element
                v.copy_(t)
                assert v.data_ptr() % 16 != 0
                views.append(v)
            outs, status = C.emulated_collective("allreduce", views, world, algo=algo, blocks=2,
                                                 half_bytes=4 << 20)
            torch.cuda.synchronize()
            _check_status(status)
            for r in range(world):
                torch.testing.assert_close(outs[r].double(), expect, **_tol(dtype, world))


def test_repeats_exercise_both_halves_and_epochs(C):
    _need_gpu()
    world = 4
    n = 40_000
    ins = _make(world, n, torch.float32, seed=11)
    expect = _ref(ins, "sum")
    for algo in ("oneshot", "twoshot", "hier"):
        reps = 5
        outs, status = C.emulated_collective("allreduce", [t.clone() for t in ins], 2 if algo == "hier" else world,
                                             algo=algo, blocks=4, half_bytes=8 << 20, repeats=reps)
        torch.cuda.synchronize()
        _check_status(status)
        # in place: every repetition multiplies by the world size
        torch.testing.assert_close(outs[0].double(), expect * world ** (reps - 1), rtol=1e-4, atol=1e-3)


@pytest.mark.parametrize("gpm,favorable", [(4, False), (2, False), (2, True), (1, False)])
def test_reduce_scatter_and_all_gather(C, gpm, favorable):
    _need_gpu()
    world = 4
    for n in (1, 6, 1237, 65_537):
        ins = _make(world, world * n, torch.float32, seed=n)
        expect = _ref(ins, "sum")
        outs, status = C.emulated_collective("reduce_scatter", ins, gpm, favorable=favorable,
                                             blocks=3, half_bytes=256 << 10)
        torch.cuda.synchronize()
        _check_status(status)
        for r in range(world):
            torch.testing.assert_close(outs[r].double(), expect[r * n:(r + 1) * n], rtol=1e-5, atol=1e-5)
        parts = _make(world, n, torch.float32, seed=n + 1)
        outs, status = C.emulated_collective("allgather", parts, gpm, favorable=favorable,
                                             blocks=3, half_bytes=256 << 10)
        torch.cuda.synchronize()
        _check_status(status)
        full = torch.cat(parts)
        for r in range(world):
            assert torch.equal(outs[r], full)


def test_wait_runs_into_its_limit_and_reports(C):
    """A rank whose signals go nowhere: its peers give up after the time limit,
    record who they were waiting for, and the kernel returns normally."""
    _need_gpu()
    world = 4
    ins = _make(world, 10_000, torch.float32)
    outs, status = C.emulated_collective("allreduce", [t.clone() for t in ins], world,
                                         algo="twoshot", blocks=2, half_bytes=1 << 20,
                                         timeout_ms=50, silent_rank=2)
    torch.cuda.synchronize()
    st = status.tolist()
    for r in (0, 1, 3):
        assert st[r][0] == 1, st  # timeout
        assert st[r][2] == 2, st  # ... waiting for rank 2
    # the GPU is still usable afterwards
    x = torch.ones(10, device="cuda")
    assert float(x.sum()) == 10.0
    outs, status = C.emulated_collective("allreduce", [t.clone() for t in ins], world,
                                         algo="twoshot", blocks=2, half_bytes=1 << 20)
    _check_status(status)


def test_fused_adamw_matches_torch(C):
    _need_gpu()
    torch.manual_seed(0)
    n = 1_000_003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    ref_p = torch.nn.Parameter(p.clone())
    ref_p.grad = g.clone()
    opt = torch.optim.AdamW([ref_p], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m = torch.zeros_like(p)
    v = torch.zeros_like(p)
    for step in range(1, 4):
        opt.step()
        C.adamw_flat_(p, g, m, v, 1e-3, 0.9, 0.95, 1e-8, 0.1, step, 1.0)
    torch.testing.assert_close(p, ref_p.data, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(C.sumsq(g), (g.double() ** 2).sum().float().reshape(1), rtol=1e-4, atol=0)


def test_adamw_shadow_and_bf16_grad_kernel(C):
    _need_gpu()
    torch.manual_seed(1)
    n = 300_007
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    p2, m2, v2 = p.clone(), m.clone(), v.clone()
    shadow = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    C.adamw_flat_(p, g, m, v, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, 1.0, shadow)
    C.adamw_flat_(p2, g, m2, v2, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, 1.0)
    assert torch.equal(p, p2) and torch.equal(shadow, p.to(torch.bfloat16))
    for k in (8, 1000, 100_003):
        src = torch.randn(k, device="cuda").to(torch.bfloat16)
        dst = torch.full((k,), 2.0, device="cuda")
        C.bf16_grad_to_f32_(dst, src, False)
        assert torch.equal(dst, src.float())
        C.bf16_grad_to_f32_(dst, src, True)
        assert torch.equal(dst, src.float() * 2)


def test_flat_data_parallel_bf16_shadow_matches_autocast(C):
    """One rank: the shadow-weight path gives the gradients autocast gives."""
    _need_gpu()
    import os
    import socket

    import torch.distributed as dist

    import fairring_b200  # noqa: F401
    from fairring_b200.models import DecoderConfig, DecoderLM
    from fairring_b200.ops import FlatAdamW
    from fairring_b200.parallel import FlatDataParallel

    if not dist.is_initialized():
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
        s.close()
        os.environ.setdefault("FAIRRING_TOTAL_MEMORY", str(64 << 20))
        dist.init_process_group("fairring", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    cfg = DecoderConfig.tiny()
    torch.manual_seed(0)
    a = DecoderLM(cfg).cuda()
    b = DecoderLM(cfg).cuda()
    b.load_state_dict(a.state_dict())
    tok = torch.randint(0, cfg.vocab, (4, cfg.seq_len + 1), device="cuda")
    da = FlatDataParallel(a)
    db = FlatDataParallel(b, bf16_shadow=True)
    oa = FlatAdamW(da.flat_param, da.flat_grad, lr=1e-3)
    ob = FlatAdamW(db.flat_param, db.flat_grad, lr=1e-3, shadow=db.flat_shadow)
    for step in range(3):
        losses = []
        for d, o in ((da, oa), (db, ob)):
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = d(tok[:, :-1], tok[:, 1:])
            loss.backward()
            o.step()
            losses.append(loss.item())
        assert abs(losses[0] - losses[1]) < 2e-2, losses
        torch.testing.assert_close(da.flat_grad, db.flat_grad, rtol=5e-2, atol=2e-3)
    torch.testing.assert_close(db.flat_shadow.float(), db.flat_param, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(da.flat_param, db.flat_param, rtol=1e-2, atol=2e-3)


def test_launch_counter_counts(C):
    _need_gpu()
    before = C.launch_count()
    x = torch.randn(1024, device="cuda")
    C.sumsq(x)
    assert C.launch_count() == before + 1


# ---- flag-in-data one-shot (small messages) ---------------------------------------------
@pytest.mark.parametrize("algo", ["ll", "ll2"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_ll_allreduce_sizes(C, world, algo):
    _need_gpu()
    for n in (1, 2, 3, 5, 64, 1000, 4099, 8192, 100_003):
        ins = _make(world, n, torch.float32, seed=n)
        expect = _ref(ins, "sum")
        outs, status = C.emulated_collective("allreduce", [t.clone() for t in ins], world, algo=algo,
                                             blocks=4)
        torch.cuda.synchronize()
        _check_status(status)
        for r in range(world):
            torch.testing.assert_close(outs[r].double(), expect, rtol=1e-5, atol=1e-5)
            assert torch.equal(outs[r], outs[0]), "ranks must agree bit for bit"


@pytest.mark.parametrize("algo", ["ll", "ll2"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("op", ["sum", "max", "min"])
def test_ll_allreduce_dtypes_ops(C, dtype, op, algo):
    _need_gpu()
    world = 4
    for n, offset in ((7, 0), (1025, 1), (3000, 3)):  # offsets: misaligned tensors
        ins = _make(world, n, dtype, seed=9, offset=offset)
        expect = _ref(ins, op)
        outs, status = C.emulated_collective("allreduce", [t.clone() if offset == 0 else t for t in ins],
                                             world, op=op, algo=algo, blocks=2)
        torch.cuda.synchronize()
        _check_status(status)
        for r in range(world):
            torch.testing.assert_close(outs[r].double(), expect, **_tol(dtype, world))


@pytest.mark.parametrize("algo", ["ll", "ll2"])
def test_ll_allreduce_repeats_and_scale(C, algo):
    """Consecutive collectives alternate between the halves of the area and are
    told apart by their number alone: nothing is cleared in between."""
    _need_gpu()
    world, n, reps = 4, 3001, 7
    ins = _make(world, n, torch.float32, seed=21)
    expect = _ref(ins, "sum") * (0.25 * world) ** (reps - 1) * 0.25
    outs, status = C.emulated_collective("allreduce", [t.clone() for t in ins], world, scale=0.25,
                                         algo=algo, blocks=3, repeats=reps)
    torch.cuda.synchronize()
    _check_status(status)
    for r in range(world):
        torch.testing.assert_close(outs[r].double(), expect, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("algo", ["ll", "ll2"])
def test_ll_silent_rank_times_out(C, algo):
    _need_gpu()
    world, n = 4, 2000
    ins = _make(world, n, torch.float32, seed=5)
    outs, status = C.emulated_collective("allreduce", [t.clone() for t in ins], world, algo=algo,
                                         blocks=2, timeout_ms=200, silent_rank=2)
    torch.cuda.synchronize()
    codes = status[:, 0].tolist()
    assert all(codes[r] == 1 for r in (0, 1, 3)), status.tolist()
    assert all(int(status[r, 2]) == 2 for r in (0, 1, 3))
    if algo == "ll":
        assert codes[2] == 0  # the silent rank itself hears everybody
    assert int(torch.arange(10, device="cuda").sum()) == 45
