"""HuggingFace <-> native parameter mapping machinery shared by the three families.

Native parameters fuse several HF tensors (q/k/v -> ``qkv_proj``, gate/up -> ``gate_up_proj``,
all experts -> one [E, ...] tensor), so the unit of mapping is a *slice assignment*: a rule
turns an HF key into (native parameter name, index into it, transform of the HF tensor).
``StateAssembler`` applies rules while streaming safetensors files, checks shapes, counts
how many elements of every native parameter were written and reports unmapped keys and
unfilled parameters.  Export walks the same rules backwards.
Reference counterpart: omegalax/models/params_utils.py:18-348.
"""
from __future__ import annotations

import dataclasses
import enum
import re
from typing import Callable, Iterable

import torch

from .hf_io import find_safetensors, load_hf_config, load_hf_config_from_source, save_hf_config  # noqa: F401


class Transform(enum.Enum):
    NONE = "none"            # copy as is (Linear weights are [out, in] on both sides)
    SQUEEZE1 = "squeeze1"    # conv1d weight (C,1,K) -> (C,K)
    FLATTEN_OUT = "flatten"  # Conv3D weight (O,C,T,H,W) -> (O, C*T*H*W)


def apply_transform(t: torch.Tensor, tr: Transform) -> torch.Tensor:
    if tr is Transform.NONE:
        return t
    if tr is Transform.SQUEEZE1:
        return t.squeeze(1)
    if tr is Transform.FLATTEN_OUT:
        return t.reshape(t.shape[0], -1)
    raise ValueError(tr)


def inverse_transform(t: torch.Tensor, tr: Transform, hf_shape=None) -> torch.Tensor:
    if tr is Transform.NONE:
        return t
    if tr is Transform.SQUEEZE1:
        return t.unsqueeze(1)
    if tr is Transform.FLATTEN_OUT:
        return t.reshape(hf_shape)
    raise ValueError(tr)


@dataclasses.dataclass
class Rule:
    """``pattern`` is a regex over HF keys; ``target`` builds the native name from the match;
    ``index`` builds the index (tuple of slices/ints) into the native tensor, or None for the
    whole tensor; ``hf_shape`` gives the HF-side shape for export of reshaped tensors."""
    pattern: str
    target: Callable[[re.Match], str]
    index: Callable[[re.Match], tuple | None] = lambda m: None
    transform: Transform = Transform.NONE
    hf_shape: Callable[[re.Match], tuple] | None = None

    def __post_init__(self):
        self.regex = re.compile(self.pattern)


def rows(lo: int, hi: int):
    return (slice(lo, hi),)


class StateAssembler:
    def __init__(self, state: dict[str, torch.Tensor], rules: Iterable[Rule]):
        self.state = state
        self.rules = list(rules)
        self.filled = {k: 0 for k in state}
        self.unmapped: list[str] = []
        self.errors: list[str] = []

    def match(self, hf_key: str):
        for r in self.rules:
            m = r.regex.fullmatch(hf_key)
            if m:
                return r, m
        return None, None

    def assign(self, hf_key: str, tensor: torch.Tensor) -> bool:
        r, m = self.match(hf_key)
        if r is None:
            self.unmapped.append(hf_key)
            return False
        name = r.target(m)
        if name not in self.state:
            self.errors.append(f"{hf_key}: native parameter '{name}' does not exist")
            return False
        dst = self.state[name]
        idx = r.index(m)
        view = dst if idx is None else dst[idx]
        src = apply_transform(tensor, r.transform)
        if tuple(view.shape) != tuple(src.shape):
            self.errors.append(f"{hf_key}: shape {tuple(src.shape)} does not fit {name}{'' if idx is None else list(idx)} {tuple(view.shape)}")
            return False
        with torch.no_grad():
            view.copy_(src.to(dtype=dst.dtype))
        self.filled[name] += src.numel()
        return True

    def finish(self, *, allow_unfilled: Iterable[str] = ()) -> None:
        allow = set(allow_unfilled)
        for name, n in self.filled.items():
            if name in allow:
                continue
            want = self.state[name].numel()
            if n != want:
                self.errors.append(f"native parameter '{name}' received {n} of {want} elements")
        if self.unmapped:
            self.errors.append(f"unmapped checkpoint keys: {self.unmapped[:8]}{'...' if len(self.unmapped) > 8 else ''}")
        if self.errors:
            raise RuntimeError("checkpoint conversion failed:\n  " + "\n  ".join(self.errors))


def stream_safetensors(file_dir):
    """Yield (key, tensor) over every ``*.safetensors`` file of a directory."""
    from safetensors import safe_open

    for f in find_safetensors(file_dir):
        with safe_open(str(f), framework="pt") as sf:
            for k in sf.keys():
                yield k, sf.get_tensor(k)


def moe_rules(layer_prefix_pat: str, native_layer: Callable[[re.Match], str], F: int) -> list[Rule]:
    """Rules for the three accepted expert layouts: fused ``experts.gate_up_proj`` [E,2F,D],
    batched ``experts.down_proj`` [E,D,F], and per-expert ``experts.J.{gate,up,down}_proj.weight``;
    plus the router ``mlp.gate.weight`` [E,D]."""
    p = layer_prefix_pat
    return [
        Rule(p + r"\.mlp\.gate\.weight", lambda m: native_layer(m) + ".mlp.router.weight"),
        Rule(p + r"\.mlp\.experts\.gate_up_proj", lambda m: native_layer(m) + ".mlp.experts_gate_up"),
        Rule(p + r"\.mlp\.experts\.down_proj", lambda m: native_layer(m) + ".mlp.experts_down"),
        Rule(p + r"\.mlp\.experts\.(?P<e>\d+)\.gate_proj\.weight", lambda m: native_layer(m) + ".mlp.experts_gate_up",
             lambda m: (int(m["e"]), slice(0, F))),
        Rule(p + r"\.mlp\.experts\.(?P<e>\d+)\.up_proj\.weight", lambda m: native_layer(m) + ".mlp.experts_gate_up",
             lambda m: (int(m["e"]), slice(F, 2 * F))),
        Rule(p + r"\.mlp\.experts\.(?P<e>\d+)\.down_proj\.weight", lambda m: native_layer(m) + ".mlp.experts_down",
             lambda m: (int(m["e"]),)),
    ]


def write_moe_experts_to_hf(out: dict, hf_layer_prefix: str, router, gate_up, down) -> None:
    """HF fused expert layout: gate_up_proj [E,2F,D], down_proj [E,D,F], gate.weight [E,D]."""
    out[f"{hf_layer_prefix}.mlp.gate.weight"] = router.detach().float().contiguous()
    out[f"{hf_layer_prefix}.mlp.experts.gate_up_proj"] = gate_up.detach().float().contiguous()
    out[f"{hf_layer_prefix}.mlp.experts.down_proj"] = down.detach().float().contiguous()


def native_state(model) -> dict[str, torch.Tensor]:
    return {k: v for k, v in model.named_parameters()}


def flatten_pure_state(model) -> dict[str, torch.Tensor]:
    return {k: v.detach() for k, v in model.state_dict().items()}


def save_safetensors(tensors: dict[str, torch.Tensor], out_dir, name: str = "model.safetensors"):
    from pathlib import Path

    from safetensors.torch import save_file

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    save_file({k: v.detach().to("cpu").contiguous() for k, v in tensors.items()}, str(out / name),
              metadata={"format": "pt"})
    return out / name
