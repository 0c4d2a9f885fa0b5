"""The allocation-free entry point, called through its exported C symbol.

Some hosts of this library cannot allocate device memory when they need a
reduction (another part of the process is capturing a CUDA graph, or they live
inside somebody else's memory budget).  For them the library exports one C
function whose scratch memory is a static array inside the library.  This test
calls it with ctypes, twice in a row, and compares with the regular (allocating)
one-shot all-reduce.  The file sorts last so that a failure here cannot hide
results of the other tests.
"""

import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import fairring_b200

    so = os.path.join(os.path.dirname(fairring_b200.__file__), "_C.so")
    lib = ctypes.CDLL(so)
    fn = lib.fairring_allreduce_f32_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, ctypes.c_longlong,
                   ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_ulong]
    return fn


def _call(fn, tensors, check=1):
    ptrs = (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(ptrs, len(tensors), tensors[0].numel(), ctypes.c_void_p(stream), check, err, 256)
    return rc, err.value.decode()


@pytest.mark.parametrize("world,n", [(2, 1), (4, 1000), (8, 4096), (3, 4093)])
def test_matches_the_allocating_entry_point_twice(C, world, n):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    fn = _lib()
    for attempt in range(2):  # two calls in a row share the static scratch
        g = torch.Generator().manual_seed(10 * attempt + world)
        ins = [torch.randn(n, generator=g).cuda() for _ in range(world)]
        ref, status = C.emulated_collective("allreduce", [t.clone() for t in ins], world,
                                            algo="oneshot", blocks=2, half_bytes=1 << 20)
        assert int(status[:, 0].sum()) == 0
        mine = [t.clone() for t in ins]
        rc, msg = _call(fn, mine)
        assert rc == 0, msg
        torch.cuda.synchronize()
        for r in range(world):
            torch.testing.assert_close(mine[r], ref[r], rtol=1e-5, atol=1e-5)
            torch.testing.assert_close(mine[r].double(), torch.stack(ins).double().sum(0),
                                       rtol=1e-5, atol=1e-5)


def test_rejects_what_does_not_fit(C):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    fn = _lib()
    big = [torch.zeros(4097, device="cuda") for _ in range(2)]
    rc, msg = _call(fn, big)
    assert rc == 1 and "4096" in msg
    many = [torch.zeros(8, device="cuda") for _ in range(9)]
    rc, msg = _call(fn, many)
    assert rc == 1 and "8" in msg
    torch.testing.assert_close(big[0], torch.zeros(4097, device="cuda"))
