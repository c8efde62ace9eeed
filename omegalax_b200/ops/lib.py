"""ctypes binding of ``libomegalax_b200.so`` (the hand-written sm_100a kernels).

The library is located next to this file.  It is loaded lazily the first time a CUDA op
is requested; on a machine with a GPU a missing library is an error (ops never fall back
silently to another implementation on CUDA tensors).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_DEBUG_LIB = os.environ.get("OMEGALAX_B200_DEBUG", "0") == "1" and os.environ.get("OMEGALAX_B200_DEBUG_LIB", "1") == "1"
LIB_PATH = _HERE / ("libomegalax_b200_debug.so" if _DEBUG_LIB else "libomegalax_b200.so")

_lib = None
_status = {}

from ctypes import c_uint

P = c_void_p
I = c_int
L = c_longlong
F = c_float

_SIGS = {
    "ob_gemm_bf16": [P, P, P, P, I, I, I, L, L, L, L, I, I, I, I, P, P, P],
    "ob_gemm_bf16_pair_peer_reduce": [P, P, P, I, I, I, I, I, L, L, L, I, I, I, I, P, P],
    "ob_gemm_bf16_pair": [P, P, P, P, I, I, I, L, L, L, L, I, I, I, P, P, P, P, P, P],
    "ob_gemm_bf16_pair_ag": [P, P, P, P, P, I, I, I, L, L, I, I, I, I, I, P, c_uint, I, P, P],
    "ob_gemm_bf16_ag": [P, P, P, P, P, I, I, I, L, L, I, I, I, I, I, P, c_uint, I, P, P],
    "ob_gemm_bf16_peer_reduce": [P, P, P, I, I, I, I, I, L, L, L, I, I, I, I, P, P],
    "ob_gemm_bf16_grouped": [P, P, P, P, I, I, I, I, L, L, I, I, P, P],
    "ob_gemm_bf16_grouped_wgrad": [P, P, P, P, I, I, I, I, L, L, I, P, P],
    "ob_gemm_bf16_pair_grouped": [P, P, P, P, I, I, I, I, L, L, I, I, P, P],
    "ob_gemm_bf16_pair_grouped_wgrad": [P, P, P, P, I, I, I, I, L, L, I, P, P],
    "ob_attn_fwd": [P, P, P, P, P, P, I, I, L, I, I, I, L, L, L, L, F, I, P, P],
    "ob_attn_bwd": [P, P, P, P, P, P, P, P, P, P, P, P, I, I, L, I, I, I, L, L, L, L, L, L, L, F, I, P, P],
    "ob_decode_append": [P, P, P, P, P, P, P, I, I, P, P, P, L, I, I, I, I, F, F, I, P],
    "ob_decode_attn": [P, P, P, P, P, I, I, I, I, I, I, I, F, P, P, P, P],
    "ob_peer_scatter_add": [P, P, I, P, I, I, P],
    "ob_slab_sum": [P, I, L, P, P, P],
    "ob_ep_push": [P, I, P, P, P, P, P, L, I, P],
    "ob_ep_pull": [P, I, P, P, P, P, P, P, L, I, I, P],
    "ob_gated_rmsnorm_fwd": [P, P, P, P, P, L, I, F, P],
    "ob_gated_rmsnorm_bwd": [P, P, P, P, P, P, P, P, L, I, F, P],
    "ob_layernorm_fwd": [P, P, P, P, P, P, L, I, F, P],
    "ob_layernorm_bwd": [P, P, P, P, P, P, P, P, L, I, P],
    "ob_router_topk": [P, P, P, P, P, L, I, I, I, P],
    "ob_router_topk_bwd": [P, P, P, P, P, P, L, I, I, I, P],
    "ob_gather_rows": [P, P, P, L, I, P],
    "ob_scatter_rows": [P, P, P, L, I, I, P],
    "ob_gather4_fwd": [P, P, P, P, L, I, P],
    "ob_gather4_bwd": [P, P, P, P, L, I, P],
    "ob_gelu_tanh_fwd": [P, P, L, P],
    "ob_gelu_tanh_bwd": [P, P, P, L, P],
    "ob_sigmoid_gate_fwd": [P, P, P, L, I, I, L, L, P],
    "ob_sigmoid_gate_bwd": [P, P, P, P, P, L, I, I, L, L, P],
    "ob_ce_finish": [P, I, P, P, P, P, L, P],
    "ob_ce_vp_stats": [P, L, I, L, I, P, P, P, P, P],
    "ob_ce_vp_grad": [P, L, I, L, I, P, P, P, P, P],
    "ob_moe_count": [P, P, L, I, P],
    "ob_ep_plan": [P, P, P, P, P, P, P, L, I, I, I, I, I, P],
    "ob_moe_plan": [P, P, P, P, P, L, I, I, I, P],
    "ob_gdn_fwd": [P] * 10 + [I] * 6 + [P],
    "ob_gdn_bwd": [P] * 15 + [I] * 6 + [P],
    "ob_conv1d_silu_fwd": [P, P, P, I, I, I, I, P],
    "ob_conv1d_silu_bwd": [P, P, P, P, P, I, I, I, I, P],
    "ob_rmsnorm_fwd": [P, P, P, P, L, I, F, I, P],
    "ob_rmsnorm_bwd": [P, P, P, P, P, P, L, I, F, I, P],
    "ob_swiglu_fwd": [P, P, L, I, P],
    "ob_swiglu_bwd": [P, P, P, P, L, I, P],
    "ob_qknorm_rope_fwd": [P, P, P, P, P, P, P, L, I, I, I, I, F, I, I, P],
    "ob_qknorm_rope_bwd": [P, P, P, P, P, P, P, P, P, P, L, I, I, I, I, F, I, I, P],
    "ob_ce_fwd_bwd": [P, L, L, I, P, P, P, P, P, I, P],
    "ob_embedding_fwd": [P, P, P, L, I, P],
    "ob_embedding_bwd": [P, P, P, L, I, I, I, P],
    "ob_embedding_bwd_peer": [P, P, P, I, I, L, I, P],
    "ob_sumsq": [P, L, P, P],
    "ob_adamw": [P, P, P, P, P, L, F, F, F, F, F, F, F, F, P, F, I, P],
    "ob_cast_f32_bf16": [P, P, L, P],
    "ob_transpose_bf16": [P, P, I, I, L, L, P],
    "ob_l2_flush": [P, L, P],
}


class KernelError(RuntimeError):
    pass


def available() -> bool:
    return LIB_PATH.exists()


def load():
    """Load the shared library (building it first when a compiler is present)."""
    global _lib
    if _lib is not None:
        return _lib
    if (not LIB_PATH.exists() or _DEBUG_LIB):     # the debug variant is re-checked against the sources every time
        if os.environ.get("OMEGALAX_B200_NO_BUILD") != "1":
            from . import build as _build

            _build.build(debug=_DEBUG_LIB)
    if not LIB_PATH.exists():
        raise KernelError(
            f"{LIB_PATH} is missing: run `python -m omegalax_b200.ops.build` (needs nvcc) first"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, sig in _SIGS.items():
        if hasattr(lib, name):
            fn = getattr(lib, name)
            fn.argtypes = sig
            fn.restype = c_int
    _lib = lib
    if hasattr(lib, "ob_gemm_pair_tune"):
        lib.ob_gemm_pair_tune.argtypes = [c_int, c_int, c_int]
        lib.ob_gemm_pair_tune.restype = None
        tune = os.environ.get("OMEGALAX_B200_GEMM_TUNE")     # "gm,wide,splitk" (-1 = automatic)
        if tune:
            lib.ob_gemm_pair_tune(*[int(v) for v in tune.split(",")])
    return lib


def gemm_pair_tune(gm: int = -1, wide: int = -1, splitk: int = -1) -> None:
    """Process-wide knobs of the CTA-pair GEMMs: raster group height, use of the 512 x 256 tile
    kernel (0 never, 1 wherever it applies), forced number of reduction slices; -1 leaves the
    per-launch choice in place."""
    load().ob_gemm_pair_tune(int(gm), int(wide), int(splitk))


def register(name: str, sig) -> None:
    """Declare the signature of an additional exported launcher."""
    _SIGS[name] = sig
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.argtypes = sig
        fn.restype = c_int


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def status_tensor(device) -> torch.Tensor:
    """Per-device int32 word that kernels set when a bounded wait gives up."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", key))
        _status[key] = t
    return t


def check_status(device=None) -> None:
    """Synchronise and raise if any kernel recorded a wait timeout since the last check."""
    if debug_enabled():
        check_canaries()
    for key, t in list(_status.items()):
        if device is not None and torch.device(device).index not in (None, key):
            continue
        v = int(t[0].item())
        if v != 0:
            t.zero_()
            raise KernelError(
                f"kernel reported status code {v & 0xFF} from block {v >> 8} on cuda:{key} "
                "(1 stage-full wait, 2 stage-empty wait, 3/4 accumulator waits, 5 flag wait, "
                "8 store outside the output in a debug build)"
            )


# ---------------------------------------------------------------------------- debug aids
# OMEGALAX_B200_DEBUG=1 switches on three checks that cost host synchronisations and are therefore
# off in normal runs:
#   * every index tensor handed to a kernel that dereferences it (token ids, row maps, expert ids,
#     routing plans, block tables) is range-checked on the host before the launch, so a bad index
#     raises IndexError with its position instead of faulting the GPU;
#   * scratch buffers obtained through ``scratch()`` carry guard bands on both sides, filled with a
#     fixed pattern that ``check_status()`` verifies: a kernel that writes outside its scratch is
#     reported by name;
#   * ``load()`` picks the library built with -DOB_DEBUG_BOUNDS (``build.build(debug=True)``), whose
#     GEMM epilogues verify every row / column they store against M and N and whose waits give up
#     after 0.2 s instead of 2 s.
_CANARY_ELEMS = 1024
_CANARY_BYTE = 0xC7
_guards: list = []


def debug_enabled() -> bool:
    return os.environ.get("OMEGALAX_B200_DEBUG", "0") == "1"


def check_index(what: str, idx: torch.Tensor, upper: int, lower: int = 0) -> None:
    """Debug mode only: raise IndexError unless lower <= idx < upper everywhere."""
    if not debug_enabled() or idx is None or idx.numel() == 0:
        return
    lo, hi = int(idx.min()), int(idx.max())
    if lo < lower or hi >= upper:
        bad = ((idx < lower) | (idx >= upper)).reshape(-1).nonzero()[0]
        raise IndexError(f"{what}: value {int(idx.reshape(-1)[bad])} at flat position {int(bad)} is outside "
                         f"[{lower}, {upper})")


def scratch(name: str, shape, dtype, device) -> torch.Tensor:
    """Uninitialised work buffer for a kernel.  In debug mode it sits between two guard bands."""
    if not debug_enabled():
        return torch.empty(shape, dtype=dtype, device=device)
    import weakref

    n = 1
    for d in (shape if isinstance(shape, (tuple, list, torch.Size)) else (shape,)):
        n *= int(d)
    esz = torch.empty(0, dtype=dtype).element_size()
    pad = _CANARY_ELEMS * 16 // esz            # 16 KB on each side, keeps 16-byte alignment of the payload
    raw = torch.empty(n + 2 * pad, dtype=dtype, device=device)
    raw_bytes = raw.view(torch.uint8)
    raw_bytes[: pad * esz].fill_(_CANARY_BYTE)
    raw_bytes[(pad + n) * esz:].fill_(_CANARY_BYTE)
    payload = raw[pad:pad + n].view(shape)
    # the registry must not keep the buffer alive: it remembers the payload weakly and finds the
    # guard bands again through the payload's storage
    _guards.append((name, weakref.ref(payload), pad * esz, (pad + n) * esz))
    return payload


def _guard_bytes(payload: torch.Tensor) -> torch.Tensor:
    return torch.empty(0, dtype=torch.uint8, device=payload.device).set_(payload.untyped_storage())


def check_canaries() -> None:
    """Raise if any guard band around a live ``scratch()`` buffer was overwritten."""
    alive = []
    for name, ref, head, tail in _guards:
        payload = ref()
        if payload is None:
            continue
        raw_bytes = _guard_bytes(payload)
        before_ok = bool((raw_bytes[:head] == _CANARY_BYTE).all())
        after_ok = bool((raw_bytes[tail:] == _CANARY_BYTE).all())
        if not (before_ok and after_ok):
            raise KernelError(f"scratch buffer '{name}': bytes {'after' if before_ok else 'before'} the buffer "
                              "were overwritten")
        alive.append((name, ref, head, tail))
    _guards[:] = alive


def call(name: str, *args) -> None:
    lib = load()
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise KernelError(f"{name} failed with code {rc}")


def ptr(t):
    if t is None:
        return None
    return t.data_ptr()
