"""Generates the committed golden vectors from NATIVE Hugging Face Transformers on
CPU (the arithmetic the reference itself is checked against in its tests).

Run from the repository root:  python tests/golden/make_golden.py

Writes
  tests/golden/tiny_qwen3/{config.json,model.safetensors}  a seeded random tiny model
  tests/golden/decode_golden.npz   prompts, greedy tokens and per-step logits
  tests/golden/ops_golden.npz      inputs/outputs of the native modules on the path
                                   (RMSNorm, rotary + apply_rotary_pos_emb, MLP)
bf16 tensors are stored as their raw 16-bit patterns (int16).
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
HERE = Path(__file__).resolve().parent

TINY = dict(
    vocab_size=127, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
    num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=512,
    rope_theta=1_000_000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, sliding_window=None,
)
CASES = ((1, 5, 6), (2, 7, 5), (3, 70, 4))     # (batch, prompt length, new tokens)


def bits(t: torch.Tensor) -> np.ndarray:
    assert t.dtype == torch.bfloat16
    return t.contiguous().view(torch.int16).numpy()


def main() -> None:
    from transformers import Qwen3Config, Qwen3ForCausalLM
    from transformers.models.qwen3 import modeling_qwen3 as mq
    from oracle.qwen3_oracle import native_greedy, native_model

    torch.manual_seed(0)
    cfg = Qwen3Config(**TINY)
    cfg._attn_implementation = "sdpa"
    model = Qwen3ForCausalLM(cfg).eval().to(torch.bfloat16)
    # Random (not all-ones) norm gains so that gain placement is pinned too.
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("norm.weight") or "layernorm" in name:
                p.copy_((1.0 + 0.1 * torch.randn_like(p.float())).to(torch.bfloat16))
    out_dir = HERE / "tiny_qwen3"
    model.save_pretrained(out_dir, safe_serialization=True)
    for extra in out_dir.glob("generation_config.json"):
        extra.unlink()
    # Reload the way the reference engine loads a checkpoint (from_pretrained,
    # engine/engine.py:29-37): the rotary inv_freq buffer is then rebuilt in fp32,
    # whereas `.to(bfloat16)` on a live model would have rounded it.
    model = native_model(str(out_dir))

    gen = torch.Generator().manual_seed(1234)
    decode = {}
    for i, (b, p, n) in enumerate(CASES):
        prompt = torch.randint(0, TINY["vocab_size"], (b, p), generator=gen)
        tokens, logits = native_greedy(model, prompt, n)
        decode[f"prompt_{i}"] = prompt.numpy()
        decode[f"tokens_{i}"] = np.asarray(tokens, dtype=np.int64)
        decode[f"logits_{i}"] = logits.numpy()
    np.savez_compressed(HERE / "decode_golden.npz", **decode)

    # ---- native modules on the path ----
    ops = {}
    torch.manual_seed(7)
    x = torch.randn(5, 128).to(torch.bfloat16)
    norm = mq.Qwen3RMSNorm(128, eps=1e-6).to(torch.bfloat16)
    with torch.no_grad():
        norm.weight.copy_((1.0 + 0.2 * torch.randn(128)).to(torch.bfloat16))
        ops["norm_x"], ops["norm_w"], ops["norm_y"] = bits(x), bits(norm.weight.data), bits(norm(x))

        rot = mq.Qwen3RotaryEmbedding(cfg)
        positions = torch.tensor([[0, 1, 2, 63, 64, 65, 300, 511]])
        cos, sin = rot(torch.empty(0, dtype=torch.bfloat16), positions)
        ops["rope_positions"] = positions.numpy()
        ops["rope_cos"], ops["rope_sin"] = bits(cos[0]), bits(sin[0])
        q = torch.randn(1, 4, 8, 128).to(torch.bfloat16)
        k = torch.randn(1, 2, 8, 128).to(torch.bfloat16)
        qe, ke = mq.apply_rotary_pos_emb(q, k, cos, sin)
        ops["rope_q"], ops["rope_k"], ops["rope_qe"], ops["rope_ke"] = bits(q), bits(k), bits(qe), bits(ke)

        mlp = model.model.layers[0].mlp
        h = torch.randn(3, 128).to(torch.bfloat16)
        ops["mlp_x"], ops["mlp_y"] = bits(h), bits(mlp(h))
        ops["mlp_gate"] = bits(mlp.gate_proj.weight.data)
        ops["mlp_up"] = bits(mlp.up_proj.weight.data)
        ops["mlp_down"] = bits(mlp.down_proj.weight.data)
    np.savez_compressed(HERE / "ops_golden.npz", **ops)
    print("wrote", out_dir, "decode_golden.npz", "ops_golden.npz")


if __name__ == "__main__":
    main()
