"""Host-side Python pieces that need no GPU: the measured-threshold table (how
bench/tune.py derives it and how the package applies it), the off-GPU fallbacks
of the fused ops, the block with pending residual, the figures."""

import importlib
import json

import torch


def _rows():
    rows = []
    # small messages: flag-in-data wins to 256 KiB, its two-shot form at 512 KiB, staged NVLS after
    for size, ll, ll2, nvls in ((4096, 15.0, 20.0, 30.0), (262144, 23.0, 24.0, 31.0),
                                (524288, None, 25.0, 32.0), (1048576, None, 38.0, 33.0)):
        if ll is not None:
            rows.append({"part": "small", "variant": "ll inline", "bytes": size, "us": ll})
        rows.append({"part": "small", "variant": "ll2", "bytes": size, "us": ll2})
        rows.append({"part": "small", "variant": "nvls twoshot", "bytes": size, "us": nvls})
    # in-place kernel at 32 MiB: 4 x 1 is within 3 % of the best and the smallest
    for blocks, ch, bw in ((4, 1, 600.0), (8, 1, 606.0), (16, 2, 570.0)):
        rows.append({"part": "direct", "blocks": blocks, "channels": ch, "unroll": 8,
                     "bytes": 33554432, "us": 1.0, "busbw": bw})
    # pipelined kernel: 32 blocks x 16 MiB best at the largest size, ahead of staged from 64 MiB on
    for size, pipe_us, staged_us in ((16777216, 96.0, 84.0), (67108864, 234.0, 244.0),
                                     (268435456, 667.0, 1030.0)):
        rows.append({"part": "pipe", "blocks": 32, "chunk": 16777216, "bytes": size, "us": pipe_us,
                     "busbw": 1.75 * size / pipe_us / 1e3})
        rows.append({"part": "pipe", "blocks": 16, "chunk": 1048576, "bytes": size, "us": 5 * pipe_us,
                     "busbw": 1.75 * size / (5 * pipe_us) / 1e3})
        rows.append({"part": "staged", "variant": "nvls", "bytes": size, "us": staged_us,
                     "busbw": 1.75 * size / staged_us / 1e3})
    return rows


def test_table_is_derived_from_measured_rows():
    tune = importlib.import_module("fairring_b200.bench.tune")
    t = tune.derive_table(_rows(), 8)
    assert t["ll_max_bytes"] == 262144
    assert t["ll2_max_bytes"] == 524288
    assert t["direct_blocks"] == 4 and t["direct_max_slices"] == 1 and t["direct_unroll"] == 8
    assert t["pipe_blocks"] == 32 and t["pipe_chunk_bytes"] == 16777216
    assert t["pipe_min_bytes"] == 67108864
    assert "blocks" not in t  # the grid of the other kernels is not the in-place kernel's


def test_table_applies_per_world_size_and_env_wins(tmp_path, monkeypatch):
    import fairring_b200

    path = tmp_path / "table.json"
    path.write_text(json.dumps({"8": {"ll_max_bytes": 262144, "direct_blocks": 4, "not_an_option": 1}}))
    monkeypatch.setenv("FAIRRING_TUNING_TABLE", str(path))
    monkeypatch.setenv("FAIRRING_TOTAL_MEMORY", str(64 << 20))
    assert fairring_b200.tuning_table(8) == {"ll_max_bytes": 262144, "direct_blocks": 4}
    assert fairring_b200.tuning_table(4) == {}
    o = fairring_b200.options_from_env(world=8)
    assert o.ll_max_bytes == 262144 and o.direct_blocks == 4
    defaults = fairring_b200.options_from_env(world=4)
    assert defaults.direct_blocks == 0
    monkeypatch.setenv("FAIRRING_DIRECT_BLOCKS", "6")
    assert fairring_b200.options_from_env(world=8).direct_blocks == 6
    monkeypatch.setenv("FAIRRING_TUNING_TABLE", "off")
    assert fairring_b200.tuning_table(8) == {}


def test_shipped_table_names_only_known_options():
    import fairring_b200

    shipped = json.loads((fairring_b200._HERE / "tuning.json").read_text())
    for world, table in shipped.items():
        assert int(world) >= 2
        assert set(table) <= set(fairring_b200._TUNABLES), set(table) - set(fairring_b200._TUNABLES)


def test_fused_ops_fall_back_off_the_gpu():
    from fairring_b200.ops import fused_cross_entropy

    torch.manual_seed(0)
    logits = torch.randn(12, 64, requires_grad=True)
    targets = torch.randint(0, 64, (12,))
    targets[3] = -100
    loss = fused_cross_entropy(logits, targets)
    ref = torch.nn.functional.cross_entropy(logits.detach().float(), targets, ignore_index=-100)
    torch.testing.assert_close(loss.detach(), ref)
    loss.backward()
    assert float(logits.grad[3].abs().sum()) == 0.0


def test_block_with_pending_residual_equals_plain_block_on_cpu():
    from fairring_b200.models import DecoderConfig, DecoderLM

    torch.manual_seed(1)
    m = DecoderLM(DecoderConfig.tiny())
    x = torch.randn(2, 64, 128)
    pend = torch.randn(2, 64, 128) * 0.1
    blk = m.blocks[0]
    ref = blk(x + pend)
    xs, out = blk.forward_pending(x, pend)
    torch.testing.assert_close(xs + out, ref, rtol=1e-5, atol=1e-5)


def test_plots_are_drawn_from_the_committed_sweep_data(tmp_path):
    import importlib.util
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    spec = importlib.util.spec_from_file_location("make_plots", root / "docs" / "make_plots.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    out = tmp_path / "busbw.svg"
    data = root / "docs" / "data"
    rc = mod.main([str(data / "sweep8_fairring_ordinary.json"), str(data / "sweep8_nccl.json"), str(out),
                   "--dtype", "fp32", "--min-bytes", str(1 << 20)])
    assert rc == 0
    svg = out.read_text()
    assert svg.startswith("<svg") and svg.count("<path") == 2  # one line per backend
    assert "1 GiB" in svg
