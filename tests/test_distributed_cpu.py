"""Sharding logic on CPU ranks (gloo): FSDP over 2 and 4 ranks reproduces the single-rank
loss curve and parameters; checkpoints written with one shard count load with another."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

from tests import _dist_workers as W


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(world, *args):
    mp.spawn(W.fsdp_train, args=(world, _port(), *args), nprocs=world, join=True)


@pytest.mark.parametrize("model_id", ["qwen3-smoke", "qwen3-smoke-moe"])
def test_fsdp_matches_single_rank(tmp_path, model_id):
    _run(1, model_id, 3, str(tmp_path / "w1.pt"))
    _run(2, model_id, 3, str(tmp_path / "w2.pt"))
    a, b = torch.load(tmp_path / "w1.pt"), torch.load(tmp_path / "w2.pt")
    assert a["losses"] == pytest.approx(b["losses"], rel=2e-4, abs=2e-4)
    assert a["grad_norm"] == pytest.approx(b["grad_norm"], rel=1e-3)
    for k in a["params"]:
        torch.testing.assert_close(a["params"][k], b["params"][k], rtol=2e-3, atol=2e-4)


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_over_library_all_to_all_matches_single_rank(tmp_path, world):
    """Experts sharded over the ranks and tokens exchanged with all_to_all_single (the library form
    of expert parallelism, here on gloo): same loss curve, gradient norm and parameters as one rank
    that holds every expert, and a checkpoint written that way restores on another rank count."""
    _run(1, "qwen3-smoke-moe", 3, str(tmp_path / "w1.pt"))
    _run(world, "qwen3-smoke-moe", 3, str(tmp_path / "wn.pt"), str(tmp_path / "ck"), False, None, "a2a")
    a, b = torch.load(tmp_path / "w1.pt"), torch.load(tmp_path / "wn.pt")
    assert b["ep_kind"] == "a2a" and a["ep_kind"] is None
    assert a["losses"] == pytest.approx(b["losses"], rel=2e-4, abs=2e-4)
    assert a["grad_norm"] == pytest.approx(b["grad_norm"], rel=1e-3)
    for k in a["params"]:
        torch.testing.assert_close(a["params"][k], b["params"][k], rtol=2e-3, atol=2e-4)
    if world == 2:     # the Qwen3.5 mixture (shared expert, squared-load loss): one step, before routing flips can amplify
        _run(1, "qwen3.5-smoke", 1, str(tmp_path / "q1.pt"))
        _run(2, "qwen3.5-smoke", 1, str(tmp_path / "q2.pt"), None, False, None, "a2a")
        q1, q2 = torch.load(tmp_path / "q1.pt"), torch.load(tmp_path / "q2.pt")
        assert q2["ep_kind"] == "a2a" and q1["losses"] == pytest.approx(q2["losses"], rel=1e-5)
        assert q1["grad_norm"] == pytest.approx(q2["grad_norm"], rel=1e-4)
        for k in q1["params"]:
            torch.testing.assert_close(q1["params"][k], q2["params"][k], rtol=0, atol=5e-3)
    if world == 4:     # resume the 4-rank expert-parallel checkpoint on 2 ranks without expert parallelism
        _run(2, "qwen3-smoke-moe", 1, str(tmp_path / "r2.pt"), str(tmp_path / "ck"), True)
        _run(1, "qwen3-smoke-moe", 4, str(tmp_path / "s4.pt"))
        r, s4 = torch.load(tmp_path / "r2.pt"), torch.load(tmp_path / "s4.pt")
        assert r["losses"][0] == pytest.approx(s4["losses"][3], rel=5e-4, abs=5e-4)


def test_moe_aux_loss_uses_global_statistics(tmp_path):
    """The router load-balance loss is taken over the tokens of every data rank: value and
    gradient from 2 and 4 token slices equal the single-rank ones, and an FSDP run whose loss is
    dominated by it follows the single-rank curve."""
    outs = {}
    for world in (1, 2, 4):
        mp.spawn(W.aux_stats, args=(world, _port(), str(tmp_path / f"s{world}.pt")), nprocs=world, join=True)
        outs[world] = torch.load(tmp_path / f"s{world}.pt")
    for world in (2, 4):
        assert outs[world]["a1"] == pytest.approx(outs[1]["a1"], rel=1e-5)
        assert outs[world]["a2"] == pytest.approx(outs[1]["a2"], rel=1e-5)
        torch.testing.assert_close(outs[world]["grad"], outs[1]["grad"], rtol=1e-4, atol=1e-7)
    _run(1, "qwen3-smoke-moe", 3, str(tmp_path / "w1.pt"), None, False, 2.0)
    _run(2, "qwen3-smoke-moe", 3, str(tmp_path / "w2.pt"), None, False, 2.0)
    a, b = torch.load(tmp_path / "w1.pt"), torch.load(tmp_path / "w2.pt")
    assert a["losses"] == pytest.approx(b["losses"], rel=2e-4, abs=2e-4)
    assert a["grad_norm"] == pytest.approx(b["grad_norm"], rel=1e-3)
    for k in a["params"]:
        torch.testing.assert_close(a["params"][k], b["params"][k], rtol=2e-3, atol=2e-4)


def test_checkpoint_resharding_4_to_2(tmp_path):
    ck = tmp_path / "ckpt"
    _run(4, "qwen3-smoke", 2, str(tmp_path / "a.pt"), str(ck), False)
    # resume the 4-rank checkpoint on 2 ranks and take one more step; compare with 3 straight steps
    _run(2, "qwen3-smoke", 1, str(tmp_path / "b.pt"), str(ck), True)
    _run(1, "qwen3-smoke", 3, str(tmp_path / "c.pt"))
    b, c = torch.load(tmp_path / "b.pt"), torch.load(tmp_path / "c.pt")
    assert b["losses"][0] == pytest.approx(c["losses"][2], rel=3e-4, abs=3e-4)
    for k in c["params"]:
        torch.testing.assert_close(b["params"][k], c["params"][k], rtol=2e-3, atol=2e-4)


def test_checkpoint_write_failure_on_one_rank_is_seen_by_all(tmp_path):
    """Asynchronous multi-rank save: a shard that fails to write on rank 1 makes every rank raise,
    leaves no directory for that step and keeps the previous checkpoint."""
    out = str(tmp_path / "res.pt")
    mp.spawn(W.checkpoint_write_failure, args=(2, _port(), str(tmp_path / "ckpt"), out), nprocs=2, join=True)
    for r in range(2):
        res = torch.load(f"{out}.{r}")
        assert res["ok_first"] and res["raised"], res
        assert res["steps"] == [1], res


def test_tensor_parallel_matches_single_rank(tmp_path):
    """tp=2 (sequence-parallel activations, column/row-parallel projections) and tp=2 x fsdp=2
    reproduce the tp=1 loss curve from the same weights and batch."""
    def run(world, tp, name):
        mp.spawn(W.tp_train, args=(world, _port(), tp, 3, str(tmp_path / name)), nprocs=world, join=True)
        return torch.load(tmp_path / name)

    one = run(1, 1, "a.pt")
    two = run(2, 2, "b.pt")
    assert one["losses"] == pytest.approx(two["losses"], rel=3e-4, abs=3e-4)
    assert one["grad_norm"] == pytest.approx(two["grad_norm"], rel=2e-3)


def test_moe_tensor_parallel_aux_loss_matches_single_rank(tmp_path):
    """Routed experts under tp=2 and tp=2 x fsdp=2: the router statistics are taken over every
    rank's rows, so a run steered by the load-balance loss follows the one-rank curve."""
    def run(world, tp, name):
        mp.spawn(W.tp_train, args=(world, _port(), tp, 3, str(tmp_path / name), False, None, False, 2.0),
                 nprocs=world, join=True)
        return torch.load(tmp_path / name)

    for world, tp in ((2, 2), (4, 2)):
        ref = run(world // tp, 1, "a.pt")          # same global batch: 2 rows per data rank
        got = run(world, tp, "b.pt")
        assert ref["losses"] == pytest.approx(got["losses"], rel=3e-4, abs=3e-4), (world, tp)
        assert ref["grad_norm"] == pytest.approx(got["grad_norm"], rel=2e-3)


def test_experts_over_every_rank_with_tensor_parallel_attention(tmp_path):
    """Experts cut over shard group x tensor-parallel group (ep_size = fsdp x tp) while attention and
    the dense projections are tensor-parallel: tp 2 (two ranks, one expert pair each) and tp 2 x
    fsdp 2 (four ranks, one expert each) follow the single-rank loss curve; a checkpoint written in
    that layout resumes under plain tp 2 x fsdp 1 (experts identical over tp) and the other way."""
    def run(world, tp, name, ep_size=0, ckpt=None, resume=False, steps=3):
        mp.spawn(W.tp_train, args=(world, _port(), tp, steps, str(tmp_path / name), False, ckpt, resume, 0.05, ep_size),
                 nprocs=world, join=True)
        return torch.load(tmp_path / name)

    one = run(1, 1, "a.pt")
    two = run(2, 2, "b.pt", ep_size=2)
    assert two["ep"][:2] == ("a2a", True) and two["ep"][2] > 0
    assert one["losses"] == pytest.approx(two["losses"], rel=5e-4, abs=5e-4)
    assert one["grad_norm"] == pytest.approx(two["grad_norm"], rel=3e-3)
    # four ranks (tp 2 x fsdp 2, one expert each) against two data ranks without tensor parallelism
    ref = run(2, 1, "r.pt", ep_size=1, steps=4)
    four = run(4, 2, "c.pt", ep_size=4, ckpt=str(tmp_path / "ck4"))
    assert four["ep"][:2] == ("a2a", True)
    assert ref["losses"][:3] == pytest.approx(four["losses"], rel=5e-4, abs=5e-4)
    # three steps in the product layout, the fourth under tp 2 x fsdp 2 with the experts identical over tp ...
    resumed = run(4, 2, "e.pt", ep_size=1, ckpt=str(tmp_path / "ck4"), resume=True, steps=1)
    assert not resumed["ep"][1]
    assert resumed["losses"][0] == pytest.approx(ref["losses"][3], rel=1e-3, abs=1e-3)
    # ... and the other way: written without expert parallelism, resumed with one expert per rank
    run(4, 2, "f.pt", ep_size=1, ckpt=str(tmp_path / "ck2"))
    back = run(4, 2, "g.pt", ep_size=4, ckpt=str(tmp_path / "ck2"), resume=True, steps=1)
    assert back["ep"][1] and back["losses"][0] == pytest.approx(ref["losses"][3], rel=1e-3, abs=1e-3)


def test_vocab_parallel_head_matches_single_rank(tmp_path):
    """Untied head under tp=2: the head is split over the vocabulary and the loss combines the
    per-slice softmax statistics; loss curve and gradient norm match the tp=1 run."""
    def run(world, tp, name):
        mp.spawn(W.tp_train, args=(world, _port(), tp, 3, str(tmp_path / name), True), nprocs=world, join=True)
        return torch.load(tmp_path / name)

    one = run(1, 1, "a.pt")
    two = run(2, 2, "b.pt")
    assert two["vocab_parallel"] and not one["vocab_parallel"]
    assert one["losses"] == pytest.approx(two["losses"], rel=3e-4, abs=3e-4)
    assert one["grad_norm"] == pytest.approx(two["grad_norm"], rel=2e-3)


def test_checkpoint_across_tensor_parallel_degrees(tmp_path):
    """A checkpoint written under tp=2 resumes under tp=2 (each rank reads its own slice) and under
    tp=1 (slices re-assembled), and one written under tp=1 resumes under tp=2; the next step's loss
    is the one of an uninterrupted run.  The head is untied, so it is split over the vocabulary."""
    def run(world, tp, steps, name, ckpt=None, resume=False):
        mp.spawn(W.tp_train, args=(world, _port(), tp, steps, str(tmp_path / name), True, ckpt, resume),
                 nprocs=world, join=True)
        return torch.load(tmp_path / name)

    straight = run(1, 1, 3, "c.pt")
    ck2, ck1 = str(tmp_path / "ck_tp2"), str(tmp_path / "ck_tp1")
    run(2, 2, 2, "a.pt", ck2)
    run(1, 1, 2, "a1.pt", ck1)
    for world, tp, ck in ((2, 2, ck2), (1, 1, ck2), (2, 2, ck1)):
        got = run(world, tp, 1, "r.pt", ck, True)
        assert got["losses"][0] == pytest.approx(straight["losses"][2], rel=3e-4, abs=3e-4), (world, tp, ck)


@pytest.mark.parametrize("moe", [False, True])
def test_qwen3_vl_tensor_parallel_matches_single_rank(tmp_path, moe):
    """Qwen3-VL with the text decoder over tp=2 (image features and DeepStack adds land on the rank
    that owns the row; vision tower replicated; head split over the vocabulary) follows the tp=1
    loss curve on an image + text batch."""
    def run(world, tp, name):
        mp.spawn(W.vl_tp_train, args=(world, _port(), tp, 3, str(tmp_path / name), moe), nprocs=world, join=True)
        return torch.load(tmp_path / name)

    one = run(1, 1, "a.pt")
    two = run(2, 2, "b.pt")
    assert two["vocab_parallel"] and not one["vocab_parallel"]
    assert one["losses"] == pytest.approx(two["losses"], rel=3e-4, abs=3e-4)
    assert one["grad_norm"] == pytest.approx(two["grad_norm"], rel=2e-3)


@pytest.mark.parametrize("model_id", ["qwen3.5-smoke", "qwen3.5-smoke-dense"])
def test_qwen3_5_tensor_parallel_matches_single_rank(tmp_path, model_id):
    """Qwen3.5 hybrid (MoE and dense) under tp=2 -- gated-attention heads, GatedDeltaNet heads and
    MLP / shared-expert width split, routed experts replicated on sequence-parallel rows --
    follows the tp=1 loss curve, and a tp=2 checkpoint resumes under tp=1."""
    def run(world, tp, steps, name, ckpt=None, resume=False):
        mp.spawn(W.q35_tp_train, args=(world, _port(), tp, steps, str(tmp_path / name), ckpt, resume, model_id),
                 nprocs=world, join=True)
        return torch.load(tmp_path / name)

    one = run(1, 1, 3, "a.pt")
    two = run(2, 2, 3, "b.pt")
    assert one["losses"] == pytest.approx(two["losses"], rel=3e-4, abs=3e-4)
    # fp32 gate gradients of the recurrence amplify re-association differences; the fp64 check below
    # is the exact one
    assert one["grad_norm"] == pytest.approx(two["grad_norm"], rel=2e-2)
    ck = str(tmp_path / "ck")
    run(2, 2, 2, "c.pt", ck)
    got = run(1, 1, 1, "d.pt", ck, True)
    assert got["losses"][0] == pytest.approx(one["losses"][2], rel=3e-4, abs=3e-4)


@pytest.mark.parametrize("model_id", ["qwen3.5-smoke", "qwen3.5-smoke-dense"])
def test_qwen3_5_tensor_parallel_gradients_fp64(tmp_path, model_id):
    """Every parameter gradient of the tp=2 model (slices re-assembled, replicated ones summed over
    ranks) equals the unsplit model's in fp64, router loss included."""
    mp.spawn(W.q35_tp_gradcheck, args=(2, _port(), model_id, str(tmp_path / "g.pt")), nprocs=2, join=True)
    out = torch.load(tmp_path / "g.pt")
    assert len(out["errs"]) == out["n_ref"] > 20
    bad = {n: e for n, e in out["errs"].items() if e > 1e-5}
    assert not bad, bad


def test_vlm_pretrained_loader_cuts_tensor_parallel_slices(tmp_path):
    """A HuggingFace-format Qwen3-VL checkpoint loaded into a tp=2 engine: each rank's master
    copy is its slice of the exported tensor."""
    from omegalax_b200.models.qwen3.tp_layout import tp_slice
    from omegalax_b200.models.qwen3_vl import Qwen3VL, make_vl_config
    from omegalax_b200.models.qwen3_vl.params import export_qwen3_vl_to_safetensors

    cfg = make_vl_config("qwen3-vl-smoke")
    torch.manual_seed(5)
    model = Qwen3VL(cfg)
    export_qwen3_vl_to_safetensors(model, cfg, tmp_path / "hf")
    mp.spawn(W.vl_tp_pretrained, args=(2, _port(), str(tmp_path / "hf"), str(tmp_path / "o.pt")), nprocs=2, join=True)
    got = torch.load(tmp_path / "o.pt")
    src = dict(model.named_parameters())
    for r in range(2):
        assert len(got[r]) == 4
        for n, v in got[r].items():
            torch.testing.assert_close(v, tp_slice(n, src[n].detach(), cfg, 2, r).float(), rtol=0, atol=0)
    assert got[0]["lm_head.weight"].shape[0] == cfg.vocab_size // 2


@pytest.mark.parametrize("family", ["qwen3", "qwen3.5"])
def test_export_of_tensor_parallel_model(tmp_path, family):
    """A tp=2 model exported to the HuggingFace format (slices re-assembled over the group) loads
    back as the unsplit model it was cut from."""
    import dataclasses

    out = tmp_path / "hf"
    mp.spawn(W.tp_export, args=(2, _port(), family, str(out)), nprocs=2, join=True)
    torch.manual_seed(0)
    if family == "qwen3":
        from omegalax_b200.models.qwen3.config import make_config
        from omegalax_b200.models.qwen3.loader import create_qwen3_from_safetensors as load
        from omegalax_b200.models.qwen3.model import Qwen3 as cls

        cfg = dataclasses.replace(make_config("qwen3-smoke"), num_kv_heads=2, tie_word_embeddings=False)
    else:
        from omegalax_b200.models.qwen3_5.config import make_config
        from omegalax_b200.models.qwen3_5.loader import create_qwen3_5_from_safetensors as load
        from omegalax_b200.models.qwen3_5.model import Qwen3_5ForConditionalGeneration as cls

        cfg = make_config("qwen3.5-smoke")
    want = cls(cfg, dtype=torch.float32)
    from omegalax_b200.parallel import mesh as mesh_lib

    mesh_lib.set_default_mesh(None)
    back = load(str(out), tp_size=1, fsdp_size=1, dp_size=1)
    back = back[0] if isinstance(back, tuple) else back
    mesh_lib.set_default_mesh(None)
    got = dict(back.named_parameters())
    for n, p in want.named_parameters():
        torch.testing.assert_close(got[n].float(), p.detach(), rtol=0, atol=0, msg=n)


@pytest.mark.parametrize("moe", [False, True])
def test_decode_with_kv_cache_under_tensor_parallelism(tmp_path, moe):
    """Prefill and greedy decode steps on a tp=2 model (kv heads of the cache split, all rows on
    every rank, head split over the vocabulary) give the tp=1 logits."""
    for world in (1, 2):
        mp.spawn(W.tp_decode, args=(world, _port(), str(tmp_path / f"d{world}.pt"), moe), nprocs=world, join=True)
    a, b = torch.load(tmp_path / "d1.pt"), torch.load(tmp_path / "d2.pt")
    assert len(a) == len(b) == 4
    for x, y in zip(a, b):
        assert x.shape == y.shape
        torch.testing.assert_close(x, y, rtol=2e-4, atol=2e-4)


def test_tp_slices_roundtrip():
    from omegalax_b200.models.qwen3.config import make_config
    from omegalax_b200.models.qwen3.model import Qwen3
    from omegalax_b200.models.qwen3.tp_layout import tp_slice, tp_unslice

    import dataclasses

    for cfg in (make_config("qwen3-smoke"), dataclasses.replace(make_config("qwen3-smoke"), tie_word_embeddings=False)):
        m = Qwen3(cfg)
        for n, p in m.named_parameters():
            parts = [tp_slice(n, p.detach(), cfg, 2, r) for r in range(2)]
            assert torch.equal(tp_unslice(n, parts, cfg), p.detach()), n
            if n == "lm_head.weight" and not cfg.tie_word_embeddings:   # split over the vocabulary
                assert parts[0].shape[0] == p.shape[0] // 2
        tp_model = Qwen3(cfg, tp_size=2)
        for n, p in tp_model.named_parameters():                       # the tp model's shapes are the slices'
            assert tuple(p.shape) == tuple(tp_slice(n, dict(m.named_parameters())[n].detach(), cfg, 2, 0).shape), n
