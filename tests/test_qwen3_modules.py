"""Per-module fp32 parity with the HuggingFace Qwen3 modules (CPU): every block is fed the input
the HuggingFace model produced at that point, so errors do not accumulate across modules
(pattern: reference tests/test_qwen3_modules.py, which reports ~1e-6 errors per module)."""
import tempfile

import pytest
import torch

from omegalax_b200.models.qwen3.loader import create_qwen3_from_safetensors
from omegalax_b200.parallel import mesh as mesh_lib


@pytest.fixture(autouse=True)
def _mesh():
    mesh_lib.set_default_mesh(None)
    yield
    mesh_lib.set_default_mesh(None)


@pytest.fixture(scope="module")
def pair():
    from transformers import Qwen3Config as HFConfig, Qwen3ForCausalLM

    cfg = HFConfig(vocab_size=1024, hidden_size=128, intermediate_size=512, num_hidden_layers=2,
                   num_attention_heads=4, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-6,
                   tie_word_embeddings=False, rope_parameters={"rope_type": "default", "rope_theta": 1_000_000},
                   attention_bias=False, max_position_embeddings=512)
    torch.manual_seed(0)
    hf = Qwen3ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if "norm" in n:
                p.add_(0.1 * torch.randn_like(p))
    with tempfile.TemporaryDirectory() as tmp:
        hf.save_pretrained(tmp, safe_serialization=True)
        mesh_lib.set_default_mesh(None)
        ours = create_qwen3_from_safetensors(tmp, tp_size=1, fsdp_size=1, dp_size=1)
    mesh_lib.set_default_mesh(None)
    return hf, ours


def _captures(hf, tok):
    """Inputs and outputs of the HuggingFace sub-modules of layer 0 for one forward."""
    cap = {}
    L = hf.model.layers[0]

    def grab(name):
        def hook(mod, args, kwargs, out):
            cap[name] = (args, kwargs, out)
        return hook

    hs = [L.input_layernorm.register_forward_hook(grab("norm1"), with_kwargs=True),
          L.self_attn.register_forward_hook(grab("attn"), with_kwargs=True),
          L.mlp.register_forward_hook(grab("mlp"), with_kwargs=True),
          L.register_forward_hook(grab("layer"), with_kwargs=True),
          hf.model.rotary_emb.register_forward_hook(grab("rope"), with_kwargs=True)]
    with torch.no_grad():
        hf(input_ids=tok)
    for h in hs:
        h.remove()
    return cap


def test_modules_match_hf_with_hf_inputs(pair):
    hf, ours = pair
    torch.manual_seed(1)
    B, T = 2, 24
    tok = torch.randint(1, 1024, (B, T))
    cap = _captures(hf, tok)
    layer = ours.layers[0]
    seg = torch.ones(B, T, dtype=torch.int32)
    ctx = ours.make_ctx(tok, seg)

    def err(a, b):
        return float((a - b).abs().max())

    with torch.no_grad():
        # embedding
        assert err(ours.embedder(tok.reshape(-1)).view(B, T, -1), hf.model.embed_tokens(tok)) == 0.0
        # RMSNorm
        x = cap["norm1"][0][0]
        assert err(layer.input_norm(x.reshape(B * T, -1)).view(B, T, -1), cap["norm1"][2]) < 5e-6
        # rotary tables: HF returns (cos, sin) [B, T, head_dim] with the half table repeated twice
        cos_hf, sin_hf = cap["rope"][2]
        half = cos_hf.shape[-1] // 2
        assert err(ctx.cos.view(B, T, -1)[..., :half], cos_hf[..., :half]) < 1e-6
        assert err(ctx.sin.view(B, T, -1)[..., :half], sin_hf[..., :half]) < 1e-6
        # attention block (QK-norm, rope, causal GQA attention, output projection), HF input
        a_in = cap["attn"][1].get("hidden_states", cap["attn"][0][0] if cap["attn"][0] else None)
        a_out = cap["attn"][2][0]
        got = layer.attn(a_in.reshape(B * T, -1), ctx).view(B, T, -1)
        assert err(got, a_out) < 2e-5
        # SwiGLU MLP
        m_in = cap["mlp"][0][0]
        assert err(layer.mlp(m_in.reshape(B * T, -1)).view(B, T, -1), cap["mlp"][2]) < 2e-5
        # whole decoder layer
        l_in = cap["layer"][0][0]
        l_out = cap["layer"][2]
        l_out = l_out[0] if isinstance(l_out, tuple) else l_out
        got, _ = layer(l_in.reshape(B * T, -1), ctx)
        assert err(got.view(B, T, -1), l_out) < 5e-5
        # head
        h = torch.randn(5, 128)
        assert err(ours.lm_head(h), hf.lm_head(h)) < 2e-5
