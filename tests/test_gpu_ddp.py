"""FlatDataParallel on one GPU: gradients of parameters that a backward pass
does not touch, and saving / loading through the fp32 master weights when the
module itself only holds bf16 shadow copies."""

import os
import socket

import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def pg():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import torch.distributed as dist

    import fairring_b200  # noqa: F401

    torch.cuda.set_device(0)
    if dist.is_initialized():
        yield dist
        return
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    os.environ.setdefault("FAIRRING_TOTAL_MEMORY", str(64 << 20))
    dist.init_process_group("fairring", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    yield dist
    dist.destroy_process_group()


class TwoHeads(nn.Module):
    def __init__(self):
        super().__init__()
        self.trunk = nn.Linear(32, 32)
        self.a = nn.Linear(32, 8)
        self.b = nn.Linear(32, 8)

    def forward(self, x, use_b=True):
        h = torch.relu(self.trunk(x))
        out = self.a(h).sum()
        if use_b:
            out = out + self.b(h).sum()
        return out


def test_parameter_without_gradient_is_zeroed(pg):
    from fairring_b200.parallel import FlatDataParallel

    torch.manual_seed(0)
    m = TwoHeads().cuda()
    ddp = FlatDataParallel(m, bucket_cap_mb=0.001)
    x = torch.randn(4, 32, device="cuda")
    ddp(x, True).backward()
    torch.cuda.synchronize()
    grads = {id(p): g.clone() for p, g in zip(ddp._params, ddp.grads())}
    assert grads[id(m.b.weight)].abs().sum() > 0
    # second step: head b takes no part; its gradient must not be last step's
    ddp.zero_grad()
    ddp(x, False).backward()
    torch.cuda.synchronize()
    now = {id(p): g for p, g in zip(ddp._params, ddp.grads())}
    assert float(now[id(m.b.weight)].abs().sum()) == 0.0
    assert float(now[id(m.b.bias)].abs().sum()) == 0.0
    torch.testing.assert_close(now[id(m.a.weight)], grads[id(m.a.weight)])


def test_state_dict_round_trip_with_shadow_weights(pg):
    from fairring_b200.ops import FlatAdamW
    from fairring_b200.parallel import FlatDataParallel

    torch.manual_seed(1)
    m = TwoHeads().cuda()
    ddp = FlatDataParallel(m, bf16_shadow=True)
    opt = FlatAdamW(ddp.flat_param, ddp.flat_grad, lr=1e-2, shadow=ddp.flat_shadow)
    sd = ddp.state_dict()
    assert set(sd) == {"trunk.weight", "trunk.bias", "a.weight", "a.bias", "b.weight", "b.bias"}
    assert all(v.dtype == torch.float32 for v in sd.values()), "masters are fp32"
    assert m.trunk.weight.dtype == torch.bfloat16, "the module holds the shadows"
    saved = {k: v.clone() for k, v in sd.items()}
    # train a step: masters and shadows move
    x = torch.randn(4, 32, device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = ddp(x)
    loss.backward()
    opt.step()
    torch.cuda.synchronize()
    assert not torch.equal(ddp.state_dict()["a.weight"], saved["a.weight"])
    # load the saved state: masters come back bit for bit, shadows follow, and
    # the next optimizer step starts from them
    ddp.load_state_dict(saved)
    back = ddp.state_dict()
    for k in saved:
        assert torch.equal(back[k], saved[k]), k
    torch.testing.assert_close(m.a.weight.float(), saved["a.weight"].to(torch.bfloat16).float())
    with pytest.raises(KeyError):
        ddp.load_state_dict({"a.weight": saved["a.weight"]})
