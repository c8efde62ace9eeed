"""Multi-GPU tests (skipped with fewer than 2 GPUs): peer-memory primitives and FSDP over
NVLink peer memory against the single-GPU run.  NVLS is disabled in NCCL for these tests."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def test_bounded_barrier_times_out_cleanly():
    """A peer flag that nobody sets: the wait gives up after its budget, the status word is
    set, and the context keeps working."""
    import ctypes

    from omegalax_b200.ops import kernels as Kn, lib
    from omegalax_b200.parallel import symm

    dev = torch.device("cuda", 0)
    fake = symm.SymmetricBuffer(256)  # single-process buffer standing in for both ranks
    ptrs = (ctypes.c_void_p * 2)(fake.local_ptr, fake.local_ptr)
    st = lib.status_tensor(dev)
    st.zero_()
    # rank 0 of a pretend 2-rank world: slot 1 is never written
    lib.call("ob_symm_barrier", ctypes.cast(ptrs, ctypes.c_void_p), 2, 0, 1, 50, st.data_ptr(), lib.stream_ptr())
    torch.cuda.synchronize()
    with pytest.raises(lib.KernelError):
        lib.check_status()
    a = torch.randn(256, 256, device=dev).to(torch.bfloat16)
    out = Kn.gemm(a, a)
    torch.cuda.synchronize()
    lib.check_status()
    assert torch.isfinite(out.float()).all()


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_symmetric_memory_primitives(tmp_path):
    from tests import _gpu_workers as W

    mp.spawn(W.symm_primitives, args=(2, _port(), str(tmp_path / "r.pt")), nprocs=2, join=True)
    r = torch.load(tmp_path / "r.pt")
    assert r["allgather_ok"]
    assert r["peer_reduce_err"] < 2e-2
    assert r["pair_peer_reduce_err"] < 2e-2


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("comm", ["p2p", "nccl"])
def test_fsdp_two_gpus_matches_one(tmp_path, comm):
    from tests import _gpu_workers as W

    mp.spawn(W.fsdp_train_gpu, args=(1, _port(), "auto", 4, str(tmp_path / "one.pt")), nprocs=1, join=True)
    mp.spawn(W.fsdp_train_gpu, args=(2, _port(), comm, 4, str(tmp_path / "two.pt")), nprocs=2, join=True)
    a, b = torch.load(tmp_path / "one.pt"), torch.load(tmp_path / "two.pt")
    assert b["losses"][-1] < b["losses"][0]
    assert a["losses"] == pytest.approx(b["losses"], rel=3e-2, abs=3e-2)
    # over peer memory the first projection of every layer gathers its weight inside its GEMM launch
    assert (b["fused_gather_ctas"] > 0) == (comm == "p2p")


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_expert_parallel_two_gpus_matches_one(tmp_path):
    from tests import _gpu_workers as W

    mp.spawn(W.ep_train_gpu, args=(1, _port(), 4, str(tmp_path / "one.pt")), nprocs=1, join=True)
    mp.spawn(W.ep_train_gpu, args=(2, _port(), 4, str(tmp_path / "two.pt")), nprocs=2, join=True)
    a, b = torch.load(tmp_path / "one.pt"), torch.load(tmp_path / "two.pt")
    assert b["used_ep"] and not a["used_ep"]
    assert b["losses"][-1] < b["losses"][0]
    assert a["losses"] == pytest.approx(b["losses"], rel=3e-2, abs=3e-2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("rs_mode", ["atomic", "staged"])
def test_tensor_parallel_two_gpus_matches_one(tmp_path, rs_mode):
    """rs_mode: how the row-parallel GEMMs reduce-scatter over peer memory -- vector atomics in the
    epilogue (the choice for two ranks) or per-sender slabs summed by the owner (wider groups)."""
    from tests import _gpu_workers as W

    mp.spawn(W.tp_train_gpu, args=(1, _port(), 1, 4, str(tmp_path / "one.pt")), nprocs=1, join=True)
    mp.spawn(W.tp_train_gpu, args=(2, _port(), 2, 4, str(tmp_path / "two.pt"), rs_mode), nprocs=2, join=True)
    a, b = torch.load(tmp_path / "one.pt"), torch.load(tmp_path / "two.pt")
    assert b["transport"] == "p2p"
    assert b["vocab_parallel"]          # untied head: split over the vocabulary, CE statistics combined over tp
    assert b["fused_gathers"] > 0       # column-parallel projections gather inside their GEMM launch
    assert b["losses"][-1] < b["losses"][0]
    assert a["losses"] == pytest.approx(b["losses"], rel=3e-2, abs=3e-2)


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("family", ["qwen3.5", "qwen3-vl"])
def test_tensor_parallel_other_families_two_gpus_match_one(tmp_path, family):
    """Qwen3.5 (attention / GatedDeltaNet heads and shared-expert width over tp, routed experts on
    sequence-parallel rows) and
    Qwen3-VL (text decoder over tp, image rows in both ranks' slices) against one GPU."""
    from tests import _gpu_workers as W

    fn = W.q35_tp_train_gpu if family == "qwen3.5" else W.vl_tp_train_gpu
    mp.spawn(fn, args=(1, _port(), 1, 4, str(tmp_path / "one.pt")), nprocs=1, join=True)
    mp.spawn(fn, args=(2, _port(), 2, 4, str(tmp_path / "two.pt")), nprocs=2, join=True)
    a, b = torch.load(tmp_path / "one.pt"), torch.load(tmp_path / "two.pt")
    assert all(l == l for l in b["losses"]), b["losses"]
    assert b["losses"][-1] < b["losses"][0]
    assert a["losses"] == pytest.approx(b["losses"], rel=4e-2, abs=4e-2)


def _many():
    """Largest tested world: every GPU of the box up to 8 (4 at least, else the 2-GPU tests above cover it)."""
    n = min(8, _ngpu())
    return n if n >= 4 else 0


@pytest.mark.skipif(_many() == 0, reason="needs 4 or more GPUs")
def test_fsdp_all_gpus_matches_one(tmp_path):
    """FSDP over every GPU of the box (peer-memory gathers, weight-gradient GEMMs reducing into the
    owners' shards over NVLink) follows the single-GPU loss curve on the same global batch."""
    from tests import _gpu_workers as W

    n = _many()
    mp.spawn(W.fsdp_train_gpu, args=(1, _port(), "auto", 4, str(tmp_path / "one.pt"), 8), nprocs=1, join=True)
    mp.spawn(W.fsdp_train_gpu, args=(n, _port(), "p2p", 4, str(tmp_path / "all.pt"), 8), nprocs=n, join=True)
    a, b = torch.load(tmp_path / "one.pt"), torch.load(tmp_path / "all.pt")
    assert b["losses"][-1] < b["losses"][0]
    assert a["losses"] == pytest.approx(b["losses"], rel=3e-2, abs=3e-2)
    assert a["grad_norm"] == pytest.approx(b["grad_norm"], rel=5e-2)


@pytest.mark.skipif(_many() == 0, reason="needs 4 or more GPUs")
def test_expert_parallel_all_gpus_matches_one(tmp_path):
    from tests import _gpu_workers as W

    n = _many()
    mp.spawn(W.ep_train_gpu, args=(1, _port(), 4, str(tmp_path / "one.pt"), 8), nprocs=1, join=True)
    mp.spawn(W.ep_train_gpu, args=(n, _port(), 4, str(tmp_path / "all.pt"), 8), nprocs=n, join=True)
    a, b = torch.load(tmp_path / "one.pt"), torch.load(tmp_path / "all.pt")
    assert b["used_ep"] and not a["used_ep"]
    assert b["losses"][-1] < b["losses"][0]
    assert a["losses"] == pytest.approx(b["losses"], rel=3e-2, abs=3e-2)


@pytest.mark.skipif(_many() == 0, reason="needs 4 or more GPUs")
def test_tensor_parallel_times_fsdp_all_gpus_matches_one(tmp_path):
    """tp 2 x fsdp (n/2): sequence-parallel tensor parallelism inside FSDP groups against one GPU."""
    from tests import _gpu_workers as W

    n = _many()
    mp.spawn(W.tp_train_gpu, args=(1, _port(), 1, 4, str(tmp_path / "one.pt")), nprocs=1, join=True)
    mp.spawn(W.tp_train_gpu, args=(n, _port(), 2, 4, str(tmp_path / "all.pt")), nprocs=n, join=True)
    a, b = torch.load(tmp_path / "one.pt"), torch.load(tmp_path / "all.pt")
    assert b["losses"][-1] < b["losses"][0]
    assert a["losses"] == pytest.approx(b["losses"], rel=3e-2, abs=3e-2)
