"""Named profiling scopes: every module family opens the scope names of the reference's
``jax.named_scope`` sites (omegalax/models/qwen3/attention.py:67, .../norms.py:21, ...)."""
import pytest
import torch

from omegalax_b200.parallel import mesh as mesh_lib
from omegalax_b200.text import api as text_api
from omegalax_b200.utils import profiling


@pytest.fixture(autouse=True)
def _mesh():
    mesh_lib.set_default_mesh(None)
    yield
    mesh_lib.set_default_mesh(None)


def _trace_scopes(fn):
    seen = []
    orig = profiling.scope

    import contextlib

    @contextlib.contextmanager
    def recording(name):
        with orig(name):
            seen.append(profiling.current_scope())
            yield

    profiling.scope = recording
    profiling.enable_scopes(True)
    try:
        fn()
    finally:
        profiling.scope = orig
        profiling.enable_scopes(False)
    return seen


def test_scopes_are_off_by_default_and_nest_when_on():
    assert not profiling.scopes_enabled()
    with profiling.scope("outer"):
        assert profiling.current_scope() == ""
    profiling.enable_scopes(True)
    try:
        with profiling.scope("outer"):
            with profiling.scope("inner"):
                assert profiling.current_scope() == "outer/inner"
        assert profiling.current_scope() == ""
    finally:
        profiling.enable_scopes(False)


def test_qwen3_modules_open_the_reference_scope_names():
    model, cfg = text_api.init_model("qwen3-smoke", 0, tp_size=1, fsdp_size=1, dp_size=1, device="cpu")
    tok = torch.randint(1, cfg.vocab_size, (1, 8), dtype=torch.int32)
    seen = _trace_scopes(lambda: text_api.forward(model, tok, 0, cfg))
    flat = {s.split("/")[-1] for s in seen}
    assert {"attention", "feed_forward", "rms_norm"} <= flat


def test_qwen3_5_modules_open_the_reference_scope_names():
    model, cfg = text_api.init_model("qwen3.5-smoke", 0, tp_size=1, fsdp_size=1, dp_size=1, device="cpu")
    tok = torch.randint(1, cfg.vocab_size, (1, 8), dtype=torch.int32)
    seen = _trace_scopes(lambda: text_api.forward(model, tok, 0, cfg))
    flat = {s.split("/")[-1] for s in seen}
    assert {"text_model", "gated_delta_net", "attention", "rms_norm", "rms_norm_gated"} <= flat
