"""Debug mode (OMEGALAX_B200_DEBUG=1): host-side range checks of index tensors and guard bands
around kernel scratch buffers.  Both are plain tensor code, so they are exercised on CPU tensors."""
import pytest
import torch

from omegalax_b200.ops import lib


def test_index_check_is_off_by_default(monkeypatch):
    monkeypatch.delenv("OMEGALAX_B200_DEBUG", raising=False)
    lib.check_index("ids", torch.tensor([5, 99]), 10)          # no error: checks cost a synchronisation


def test_index_check_names_the_offending_position(monkeypatch):
    monkeypatch.setenv("OMEGALAX_B200_DEBUG", "1")
    lib.check_index("ids", torch.tensor([[0, 3], [9, 2]]), 10)
    with pytest.raises(IndexError, match=r"ids: value 10 at flat position 2 is outside \[0, 10\)"):
        lib.check_index("ids", torch.tensor([[0, 3], [10, 2]]), 10)
    with pytest.raises(IndexError, match="value -1 at flat position 0"):
        lib.check_index("rows", torch.tensor([-1, 4]), 10)


def test_scratch_guard_bands_catch_writes_on_either_side(monkeypatch):
    monkeypatch.setenv("OMEGALAX_B200_DEBUG", "1")
    lib._guards.clear()
    buf = lib.scratch("unit-test scratch", (4, 8), torch.float32, "cpu")
    assert buf.shape == (4, 8) and buf.data_ptr() % 16 == 0
    buf.fill_(1.0)                        # writing the buffer itself is fine
    lib.check_canaries()
    name, ref, head, tail = lib._guards[-1]
    raw = lib._guard_bytes(ref())
    raw[tail] = 0                         # first byte after the buffer
    with pytest.raises(lib.KernelError, match="unit-test scratch.*after"):
        lib.check_canaries()
    raw[tail] = lib._CANARY_BYTE
    raw[head - 1] = 1                     # last byte before the buffer
    with pytest.raises(lib.KernelError, match="unit-test scratch.*before"):
        lib.check_canaries()
    del buf, raw
    lib._guards[:] = [g for g in lib._guards if g[1]() is not None]
    assert not lib._guards                # a freed buffer leaves the registry


def test_scratch_is_a_plain_allocation_outside_debug_mode(monkeypatch):
    monkeypatch.delenv("OMEGALAX_B200_DEBUG", raising=False)
    n = len(lib._guards)
    buf = lib.scratch("x", 16, torch.float32, "cpu")
    assert buf.numel() == 16 and len(lib._guards) == n
