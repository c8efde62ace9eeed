"""Random-initialise a model by id and export it in the HuggingFace format
(``model.safetensors`` + ``config.json``)."""
from __future__ import annotations

from _flags import Flags


def main(argv=None):
    p = Flags(description=__doc__)
    p.define("model_id", "qwen3-smoke")
    p.define("out_dir", "exported_model")
    p.define("seed", 0)
    p.define("tp_size", 1)
    p.define("fsdp_size", 1)
    p.define("dp_size", 1)
    p.define("pad_id", 0)
    a = p.parse_args(argv)
    import torch

    from omegalax_b200 import export, registry, text_api, vlm_api
    from omegalax_b200.parallel import mesh as mesh_lib

    mesh_lib.init_distributed()
    api = text_api if registry.infer_arch(a.model_id) == registry.Arch.TEXT else vlm_api
    model, cfg = api.init_model(a.model_id, a.seed, tp_size=a.tp_size, fsdp_size=a.fsdp_size, dp_size=a.dp_size,
                                device="cpu", dtype=torch.float32)
    mesh = mesh_lib.current_mesh()
    if a.tp_size > 1:   # collective over the tensor-parallel group: slices are re-assembled first
        out = export.export_model_to_hf(model, cfg, a.out_dir, tp_group=mesh.group("tp"))
    elif mesh_lib.rank() == 0:
        out = export.export_model_to_hf(model, cfg, a.out_dir)
    else:
        out = None
    if mesh_lib.rank() == 0:
        print(f"exported {a.model_id} to {out}")


if __name__ == "__main__":
    main()
