"""Locating and reading HuggingFace checkpoints on disk (config.json + *.safetensors)."""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Any


def find_safetensors(file_dir: str | os.PathLike) -> list[Path]:
    files = sorted(Path(file_dir).expanduser().glob("*.safetensors"))
    if not files:
        raise ValueError(f"No safetensors found in {file_dir}")
    return files


def load_hf_config(file_dir: str | os.PathLike) -> dict[str, Any]:
    path = Path(file_dir).expanduser() / "config.json"
    if not path.exists():
        raise FileNotFoundError(f"{path} does not exist")
    return json.loads(path.read_text())


def load_hf_config_from_source(source: str | os.PathLike) -> dict[str, Any]:
    """``source`` is a model directory, a path to a config.json, or a hub repo id.  Hub ids
    are resolved through the local HuggingFace cache only (``huggingface_hub`` downloads
    when the machine has network access)."""
    p = Path(str(source)).expanduser()
    if p.is_dir():
        return load_hf_config(p)
    if p.is_file():
        return json.loads(p.read_text())
    try:
        from huggingface_hub import hf_hub_download

        return json.loads(Path(hf_hub_download(str(source), "config.json")).read_text())
    except Exception as e:  # no cache, no network
        raise ValueError(f"cannot resolve config for '{source}': {e}") from e


def save_hf_config(cfg_dict: dict[str, Any], out_dir: str | os.PathLike) -> Path:
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    path = out / "config.json"
    path.write_text(json.dumps(cfg_dict, indent=2, sort_keys=True))
    return path


def hf_dtype_to_torch(hf_dtype):
    import torch

    if hf_dtype is None:
        return torch.bfloat16
    kind = str(hf_dtype).lower()
    if "bfloat16" in kind or "bf16" in kind:
        return torch.bfloat16
    if "float32" in kind or "fp32" in kind:
        return torch.float32
    if "float16" in kind or "fp16" in kind:
        return torch.float16
    raise ValueError(f"Unsupported dtype '{hf_dtype}'.")


def torch_dtype_to_hf(dtype) -> str:
    return str(dtype).replace("torch.", "")
