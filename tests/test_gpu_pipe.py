"""The pipelined all-reduce kernel (bulk copy in / reduce / bulk copy out over a
ring of staging chunks) against a plain PyTorch reference, on ONE GPU.

All ranks are emulated inside one cooperative launch (grid.y = rank), with the
peer-load flavour of the reduce stage: the copy roles, the chunk counters, the
ring reuse and the tail handling are exactly what runs in a multi-GPU job.  The
multimem flavour of the reduce stage needs one GPU per rank and is covered by
the multi-GPU tests.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.uint8, torch.int8, torch.int32, torch.int64, torch.float16, torch.bfloat16,
          torch.float32, torch.float64]


def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def _make(world, n, dtype, seed=0):
    outs = []
    for r in range(world):
        g = torch.Generator(device="cpu").manual_seed(seed * 100 + r)
        if dtype.is_floating_point:
            t = torch.randn(n, generator=g)
        else:
            t = torch.randint(0, 12, (n,), generator=g)
        outs.append(t.to(dtype).cuda())
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


def _ok(status):
    assert int(status[:, 0].abs().sum()) == 0, f"kernel reported a failure: {status.tolist()}"


@pytest.mark.parametrize("world", [2, 4, 8])
def test_pipe_fp32_sizes(C, world):
    """One chunk, several chunks, more chunks than ring slots, ragged tails."""
    _need_gpu()
    for n in (1, 3, 4, 5, 64, 1000, 4099, 65536, 262144 + 3, 1_000_001):
        ins = _make(world, n, torch.float32, seed=n)
        expect = _ref(ins, "sum")
        outs, status = C.emulated_pipe_allreduce([t.clone() for t in ins], blocks=4,
                                                 chunk_bytes=64 << 10, slot_bytes=64 << 10, slots=3,
                                                 stage_bytes=4096, stages=3)
        torch.cuda.synchronize()
        _ok(status)
        for r in range(world):
            torch.testing.assert_close(outs[r].double(), expect, rtol=1e-5, atol=1e-5)
            assert torch.equal(outs[r], outs[0]), "ranks must agree bit for bit"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("op", ["sum", "max", "min"])
def test_pipe_dtypes_ops(C, dtype, op):
    _need_gpu()
    world = 4
    for n in (7, 1025, 70001):
        ins = _make(world, n, dtype, seed=7)
        expect = _ref(ins, op)
        outs, status = C.emulated_pipe_allreduce([t.clone() for t in ins], op=op, blocks=3,
                                                 chunk_bytes=32 << 10, slot_bytes=32 << 10, slots=2,
                                                 stage_bytes=2048, stages=2)
        torch.cuda.synchronize()
        _ok(status)
        for r in range(world):
            torch.testing.assert_close(outs[r].double(), expect, **_tol(dtype, world))


@pytest.mark.parametrize("blocks,chunk,stage,stages", [(1, 16 << 10, 1024, 2), (5, 48 << 10, 4096, 4),
                                                       (8, 256 << 10, 16 << 10, 6), (16, 1 << 20, 16 << 10, 6)])
def test_pipe_geometries(C, blocks, chunk, stage, stages):
    """Block counts that do not divide the sub-chunks, stages smaller and larger
    than a piece, the production stage size."""
    _need_gpu()
    world = 8 if blocks <= 8 else 4
    n = 3_000_017
    ins = _make(world, n, torch.float32, seed=3)
    expect = _ref(ins, "sum")
    outs, status = C.emulated_pipe_allreduce([t.clone() for t in ins], blocks=blocks,
                                             chunk_bytes=chunk, slot_bytes=chunk, slots=4,
                                             stage_bytes=stage, stages=stages)
    torch.cuda.synchronize()
    _ok(status)
    for r in range(world):
        torch.testing.assert_close(outs[r].double(), expect, rtol=1e-5, atol=1e-5)


def test_pipe_scale_and_repeats(C):
    """Back-to-back launches share one ring: chunk numbers carry over, no
    barrier in between.  Launch k reduces the result of launch k-1."""
    _need_gpu()
    world, n, reps = 4, 300_003, 5
    ins = _make(world, n, torch.float32, seed=11)
    expect = _ref(ins, "sum") * (0.5 * world) ** (reps - 1) * 0.5
    outs, status = C.emulated_pipe_allreduce([t.clone() for t in ins], scale=0.5, blocks=4,
                                             chunk_bytes=128 << 10, slot_bytes=128 << 10, slots=3,
                                             stage_bytes=8192, stages=3, repeats=reps)
    torch.cuda.synchronize()
    _ok(status)
    for r in range(world):
        torch.testing.assert_close(outs[r].double(), expect, rtol=1e-4, atol=1e-4)


def test_pipe_silent_rank_times_out(C):
    """A rank whose counters never reach its peers: their waits run into the
    limit, the kernel records whom it was waiting for and returns; the GPU
    stays usable."""
    _need_gpu()
    world, n = 4, 50_000
    ins = _make(world, n, torch.float32, seed=5)
    outs, status = C.emulated_pipe_allreduce([t.clone() for t in ins], blocks=2, chunk_bytes=64 << 10,
                                             slot_bytes=64 << 10, slots=2, stage_bytes=4096, stages=2,
                                             timeout_ms=300, silent_rank=1)
    torch.cuda.synchronize()
    codes = status[:, 0].tolist()
    assert any(c == 1 for c in codes), codes  # kStatusTimeout somewhere
    waiting_for = {int(status[r, 2]) for r in range(world) if codes[r] == 1}
    assert 1 in waiting_for, status.tolist()
    assert int(torch.arange(10, device="cuda").sum()) == 45
