"""The fused single-GPU ops against plain PyTorch fp32 references."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


@pytest.mark.parametrize("cols", [128, 2048, 4104, 8192])
@pytest.mark.parametrize("x_dtype,y_dtype", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                             (torch.bfloat16, torch.bfloat16)])
def test_fused_layer_norm_matches_fp32_reference(cols, x_dtype, y_dtype):
    _need_gpu()
    from fairring_b200.ops import fused_layer_norm

    torch.manual_seed(cols)
    rows = 777
    x = (torch.randn(rows, cols, device="cuda") * 2 + 0.5).to(x_dtype)
    w = torch.randn(cols, device="cuda")
    b = torch.randn(cols, device="cuda")
    dy = torch.randn(rows, cols, device="cuda").to(y_dtype)

    xr = x.float().clone().requires_grad_(True)
    wr, br = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    yr = torch.nn.functional.layer_norm(xr, (cols,), wr, br, 1e-5)
    yr.backward(dy.float())

    xf = x.clone().requires_grad_(True)
    wf, bf = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
    yf = fused_layer_norm(xf, wf, bf, 1e-5, out_dtype=y_dtype)
    assert yf.dtype == y_dtype
    yf.backward(dy)
    lo = y_dtype == torch.bfloat16 or x_dtype == torch.bfloat16
    torch.testing.assert_close(yf.float(), yr, rtol=2e-2 if lo else 1e-5, atol=3e-2 if lo else 1e-5)
    torch.testing.assert_close(xf.grad.float(), xr.grad, rtol=2e-2 if lo else 1e-4, atol=3e-2 if lo else 1e-5)
    torch.testing.assert_close(wf.grad, wr.grad, rtol=1e-3, atol=0.3 if lo else 1e-3)
    torch.testing.assert_close(bf.grad, br.grad, rtol=1e-3, atol=0.3 if lo else 1e-3)


def test_fused_layer_norm_module_under_autocast_and_fallback():
    _need_gpu()
    from fairring_b200.ops import FusedLayerNorm

    ln = FusedLayerNorm(256).cuda()
    ref = torch.nn.LayerNorm(256).cuda()
    ref.load_state_dict(ln.state_dict())
    x = torch.randn(4, 33, 256, device="cuda")
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = ln(x)
    assert y.dtype == torch.bfloat16
    torch.testing.assert_close(y.float(), ref(x), rtol=2e-2, atol=3e-2)
    assert ln(x).dtype == torch.float32
    # a row length the kernel does not take: plain torch path
    odd = FusedLayerNorm(100).cuda()
    assert odd(torch.randn(3, 100, device="cuda")).shape == (3, 100)
    # CPU: plain torch path
    assert FusedLayerNorm(16)(torch.randn(2, 16)).shape == (2, 16)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("vocab", [1024, 51200])
def test_fused_cross_entropy_matches_fp32_reference(dtype, vocab):
    _need_gpu()
    from fairring_b200.ops import fused_cross_entropy

    torch.manual_seed(vocab)
    rows = 300
    base = (torch.randn(rows, vocab, device="cuda") * 3).to(dtype)
    targets = torch.randint(0, vocab, (rows,), device="cuda")
    targets[5] = -100  # ignored row

    ref_in = base.float().clone().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(ref_in, targets, ignore_index=-100)
    (ref * 1.7).backward()

    # the logits must come out of an op (the loss overwrites them with their gradient)
    leaf = base.clone().requires_grad_(True)
    logits = leaf * 1.0
    loss = fused_cross_entropy(logits, targets)
    (loss * 1.7).backward()
    lo = dtype == torch.bfloat16
    torch.testing.assert_close(loss.float(), ref, rtol=1e-3 if lo else 1e-5, atol=1e-3 if lo else 1e-5)
    torch.testing.assert_close(leaf.grad.float(), ref_in.grad, rtol=2e-2 if lo else 1e-4, atol=1e-4 if lo else 1e-7)
    assert float(leaf.grad[5].abs().sum()) == 0.0


@pytest.mark.parametrize("branch_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("cols", [128, 2048, 4104])
@pytest.mark.parametrize("use_stream_grad", [True, False])
def test_add_layer_norm_matches_fp32_reference(branch_dtype, cols, use_stream_grad):
    _need_gpu()
    from fairring_b200.ops import FusedLayerNorm, add_layer_norm

    torch.manual_seed(cols)
    rows = 333
    norm = FusedLayerNorm(cols).cuda()
    with torch.no_grad():
        norm.weight.normal_(1.0, 0.2)
        norm.bias.normal_(0.0, 0.2)
    x0 = torch.randn(rows, cols, device="cuda")
    b0 = torch.randn(rows, cols, device="cuda").to(branch_dtype)
    wy = torch.randn(rows, cols, device="cuda")
    wx = torch.randn(rows, cols, device="cuda")

    # fp32 reference of the same op
    xr, br = x0.clone().requires_grad_(True), b0.float().clone().requires_grad_(True)
    gw, gb = norm.weight.detach().clone().requires_grad_(True), norm.bias.detach().clone().requires_grad_(True)
    xn_ref = xr + br
    y_ref = torch.nn.functional.layer_norm(xn_ref, (cols,), gw, gb, norm.eps)
    loss = (y_ref * wy).sum() + ((xn_ref * wx).sum() if use_stream_grad else 0.0)
    loss.backward()

    x, b = x0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
    lo = branch_dtype == torch.bfloat16
    with torch.autocast("cuda", dtype=torch.bfloat16, enabled=lo):
        xn, y = add_layer_norm(norm, x, b)
    assert xn.dtype == torch.float32 and y.dtype == (torch.bfloat16 if lo else torch.float32)
    loss = (y.float() * wy).sum() + ((xn * wx).sum() if use_stream_grad else 0.0)
    loss.backward()
    torch.testing.assert_close(xn, xn_ref.detach(), rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(y.float(), y_ref.detach(), rtol=2e-2 if lo else 1e-4, atol=2e-2 if lo else 1e-4)
    tol = dict(rtol=2e-2, atol=2e-2) if lo else dict(rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(x.grad, xr.grad, **tol)
    assert b.grad.dtype == branch_dtype
    torch.testing.assert_close(b.grad.float(), br.grad, rtol=2e-2 if lo else 1e-3, atol=5e-2 if lo else 1e-3)
    scale = float(rows) ** 0.5
    torch.testing.assert_close(norm.weight.grad, gw.grad, rtol=2e-2, atol=(0.2 if lo else 1e-3) * scale)
    torch.testing.assert_close(norm.bias.grad, gb.grad, rtol=2e-2, atol=(0.2 if lo else 1e-3) * scale)


def test_decoder_with_residual_adds_inside_layer_norm_matches_plain_blocks():
    _need_gpu()
    import copy

    from fairring_b200.models import DecoderConfig, DecoderLM

    torch.manual_seed(3)
    cfg = DecoderConfig.tiny()
    fused = DecoderLM(cfg).cuda()
    plain_cfg = copy.copy(cfg)
    plain_cfg.fused_residual = False
    plain = DecoderLM(plain_cfg).cuda()
    plain.load_state_dict(fused.state_dict())
    t = torch.randint(0, cfg.vocab, (4, cfg.seq_len + 1), device="cuda")
    losses = []
    for m in (fused, plain):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = m(t[:, :-1], t[:, 1:])
        loss.backward()
        losses.append(float(loss.detach()))
    assert abs(losses[0] - losses[1]) < 2e-3, losses
    for (n, p), (_, q) in zip(fused.named_parameters(), plain.named_parameters()):
        assert p.grad is not None, n
        err = (p.grad - q.grad).abs().max().item()
        ref = q.grad.abs().max().item()
        assert err <= 0.05 * ref + 1e-4, (n, err, ref)
