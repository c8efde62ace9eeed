"""FLOP accounting, step metrics, timers, LR schedules, batch-size helpers."""
import datetime

import pytest

from omegalax_b200.models.qwen3.config import make_config
from omegalax_b200.models.qwen3_5.config import make_config as make_q35
from omegalax_b200.models.qwen3_vl.config import make_vl_config
from omegalax_b200.parallel import mesh as mesh_lib
from omegalax_b200.trainers import perf
from omegalax_b200.trainers.lr_schedule import build_lr_schedule


def test_qwen3_8b_flops_per_token():
    cfg = make_config("Qwen/Qwen3-8B")
    f = perf.training_flops_per_token(cfg, 4096)
    assert 48.5e9 < f < 49.5e9  # 49.03 GFLOP per token at T=4096
    assert perf.training_flops_per_token(cfg, 8192) > f


def test_moe_counts_only_routed_experts():
    cfg = make_config("Qwen/Qwen3-30B-A3B-Instruct-2507")
    f = perf.training_flops_per_token(cfg, 4096)
    assert 22.5e9 < f < 23.6e9


def test_qwen3_5_and_vl():
    q = make_q35("qwen3.5-397b-a17b-8layer")
    f = perf.training_flops_per_token(q, 8192)
    assert 18.5e9 < f < 20e9
    vl = make_vl_config("qwen3-vl-smoke")
    one = perf.qwen3_vl_vision_training_flops(vl, [[1, 4, 4]])
    two = perf.qwen3_vl_vision_training_flops(vl, [[1, 4, 4], [1, 4, 4]])
    assert two == 2 * one  # block-diagonal attention: linear in the number of images
    assert perf.qwen3_vl_vision_training_flops(vl, None) == 0
    with pytest.raises(ValueError):
        perf.qwen3_vl_vision_training_flops(vl, [[1, 2]])


def test_step_metrics_and_peak_resolution():
    m = perf.step_metrics(2e15, datetime.timedelta(seconds=2), 1000, 1000.0)
    assert m["tflops_per_device"] == pytest.approx(1000.0) and m["mfu"] == pytest.approx(1.0)
    assert m["global_tokens_per_sec"] == pytest.approx(500.0)
    assert perf.step_metrics(1.0, datetime.timedelta(0), 10, None)["mfu"] == 0.0
    assert perf.resolve_peak_tflops("h100_sxm") == 989.0 and perf.resolve_peak_tflops("b200") == 2250.0
    assert perf.resolve_peak_tflops("123.5") == 123.5 and perf.resolve_peak_tflops(None) is None
    with pytest.raises(ValueError):
        perf.resolve_peak_tflops("nope")


def test_step_timer_warmup():
    t = perf.StepTimer(warmup=2)
    assert t.step() == datetime.timedelta(0) and t.step() == datetime.timedelta(0)
    assert t.step() >= datetime.timedelta(0)


def test_log_requires_loss_and_grad_norm():
    with pytest.raises(KeyError):
        perf.maybe_log_step_metrics(1, {"loss": 1.0}, datetime.timedelta(seconds=1), is_primary_process=True, log_every=1,
                                    per_device_flops=1.0, global_tokens_per_step=1, peak_tflops=None)
    out = perf.maybe_log_step_metrics(2, {"loss": 1.0, "grad_norm": 2.0}, datetime.timedelta(seconds=1),
                                      is_primary_process=True, log_every=2, per_device_flops=1e12,
                                      global_tokens_per_step=10, peak_tflops=10.0, batch_size=4)
    assert out["total_samples"] == 8 and out["mfu"] == pytest.approx(0.1)
    assert perf.maybe_log_step_metrics(3, {"loss": 1.0, "grad_norm": 2.0}, datetime.timedelta(seconds=1),
                                       is_primary_process=True, log_every=2, per_device_flops=1.0,
                                       global_tokens_per_step=1, peak_tflops=None) is None


def test_lr_schedules():
    lin = build_lr_schedule("linear", 1.0, 100, warmup_steps=10)
    assert lin(0) == 0.0 and lin(5) == pytest.approx(0.5) and lin(10) == 1.0 and lin(99) == 1.0
    cos = build_lr_schedule("cosine", 1.0, 110, warmup_steps=10, end_factor=0.1)
    assert cos(10) == pytest.approx(1.0) and cos(110) == pytest.approx(0.1) and 0.1 < cos(60) < 1.0
    wsd = build_lr_schedule("wsd", 1.0, 110, warmup_steps=10, end_factor=0.0, stable_fraction=0.8)
    assert wsd(50) == 1.0 and wsd(89) == 1.0 and wsd(100) == pytest.approx(0.5) and wsd(110) == pytest.approx(0.0)
    with pytest.raises(ValueError):
        build_lr_schedule("step", 1.0, 10)


def test_process_local_batch_size():
    mesh_lib.set_default_mesh(None)
    assert mesh_lib.process_local_batch_size(16, dp_size=4) == 4
    with pytest.raises(ValueError):
        mesh_lib.process_local_batch_size(10, dp_size=4)


def test_first_true_rows_matches_nonzero_with_surplus_rows():
    """Sync-free image-token positions: same scatter result as the nonzero-based path, also when
    the (padded) feature rows outnumber the image tokens."""
    import torch

    from omegalax_b200.ops import functional as Fn

    torch.manual_seed(0)
    mask = torch.rand(200) < 0.2
    k = int(mask.sum())
    x = torch.randn(200, 8)
    for n in (k, k + 7, k - 3):
        feats = torch.randn(n, 8)
        pos_ref = torch.nonzero(mask).squeeze(-1)[:n]
        want = Fn.scatter_rows(x, pos_ref, feats[: pos_ref.numel()], replace=True)
        pos, ok = Fn.first_true_rows(mask, n)
        src = torch.where(ok, feats[: pos.numel()], x.index_select(0, pos))
        got = Fn.scatter_rows(x, pos, src, replace=True)
        assert torch.equal(got, want)
        add_want = x.index_add(0, pos_ref, feats[: pos_ref.numel()])
        add_got = x.index_add(0, pos, feats[: pos.numel()] * ok.to(x.dtype))
        assert torch.allclose(add_got, add_want)


def test_stash_records_replays_and_skips():
    """Selective rematerialisation bookkeeping: tagged outputs are stored in the first pass and
    handed back in the re-run; a tag written "name!" is never stored and replays as a placeholder."""
    import torch

    from omegalax_b200.ops import functional as Fn

    st = Fn._Stash(("qkv", "down!"))
    a, b = torch.randn(2, 3), torch.randn(2, 3)
    with Fn.stash_scope(st, "record"):
        k1, v1 = Fn._stash_lookup("qkv")
        assert v1 is None
        Fn._stash_store(k1, a)
        k2, v2 = Fn._stash_lookup("qkv")          # second call with the same tag: its own slot
        Fn._stash_store(k2, b)
        k3, v3 = Fn._stash_lookup("down")
        assert v3 is None
        Fn._stash_store(k3, torch.zeros(1))
        assert Fn._stash_lookup("gate_up") == (None, None)   # not a tag of this stash
    assert len(st.items) == 2
    with Fn.stash_scope(st, "replay"):
        assert Fn._stash_lookup("qkv")[1] is a
        assert Fn._stash_lookup("qkv")[1] is b
        assert Fn._stash_lookup("down")[1] is Fn._SKIP
    assert Fn._stash_lookup("qkv") == (None, None)           # no active stash outside the scopes


def test_auto_stash_shares_the_budget_by_value_per_byte():
    """Remat policy "auto": every layer gets the first extra tag before any layer gets the second;
    what does not fit is dropped from the recorded stash and is recomputed in the re-run."""
    import torch

    from omegalax_b200.ops import functional as Fn
    from omegalax_b200.parallel.engine import _AutoStash

    auto = _AutoStash(("o", "gate_up"), margin_bytes=0)
    assert auto.tags_for(0, ("qkv",)) == ("qkv",)             # nothing extra before a budget exists
    auto.budget, auto.n_layers, auto.phase = 4 * 40 + 2 * 400 + 100, 4, "grow"
    kept = []
    for idx in range(4):
        st = Fn._Stash(auto.tags_for(idx, ("qkv", "down!")))
        assert "o" in st.tags and "gate_up" in st.tags and "down" in st.skip
        st.items = {("qkv", 0): torch.zeros(5), ("o", 0): torch.zeros(10), ("gate_up", 0): torch.zeros(100)}
        auto.account(idx, st)
        kept.append(sorted(k[0] for k in st.items))
    assert kept == [["gate_up", "o", "qkv"]] * 2 + [["o", "qkv"]] * 2
    assert auto.summary() == {"o": 4, "gate_up": 2}
    auto.close()
    assert auto.phase == "done"
    assert auto.tags_for(1, ("qkv",)) == ("qkv", "o", "gate_up") and auto.tags_for(3, ("qkv",)) == ("qkv", "o")
    assert auto.tags_for(7, ("qkv",)) == ("qkv",)             # a layer that was never recorded


def test_gemm_dispatch_heuristics():
    """Host-side choices of the GEMM wrappers: CTA-pair kernel for GEMMs that fill every SM pair,
    an even number of copy CTAs that grows with the bytes to gather per unit of GEMM time."""
    from omegalax_b200.ops import kernels as K

    if K._PAIR_MODE == "all":
        assert K._use_pair(32768, 6144, 4096)
        assert not K._use_pair(512, 512, 4096)        # 4 tiles: single-CTA kernel
        assert not K._use_pair(32768, 128, 4096)      # narrow output
    small = K.ag_copy_ctas(32768, 6144, 4096, 50e6)
    big = K.ag_copy_ctas(32768, 3072, 4096, 268e6)
    assert small % 2 == 0 and big % 2 == 0 and 2 <= small <= big <= 16


def test_measured_peaks_file_replaces_the_presets(tmp_path, monkeypatch):
    import json

    from omegalax_b200.trainers import perf

    before = dict(perf.PEAK_TFLOPS)
    f = tmp_path / "peaks.json"
    f.write_text(json.dumps({"bf16_tflops": 1500.5, "bf16_tflops_sustained": 1300.25, "hbm_gbs": 6000.0}))
    try:
        d = perf.measured_peaks(str(f))
        assert d["hbm_gbs"] == 6000.0
        assert perf.resolve_peak_tflops("b200_measured_burst") == 1500.5
        assert perf.resolve_peak_tflops("b200_measured_sustained") == 1300.25
        assert perf.resolve_peak_tflops("b200") == 2250.0 and perf.resolve_peak_tflops(123.0) == 123.0
    finally:
        perf.PEAK_TFLOPS.update(before)
