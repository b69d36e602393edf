"""Pins the CPU oracle: the operator restatements against the committed golden
vectors (made by native Hugging Face, tests/golden/make_golden.py), against
native Hugging Face live, and against the reference tests' known-answer cases."""
import json

import numpy as np
import pytest
import torch

from oracle import qwen3_oracle as O


def bf(a):
    return torch.from_numpy(np.ascontiguousarray(a)).view(torch.bfloat16)


@pytest.fixture(scope="module")
def ops(golden_dir):
    return np.load(golden_dir / "ops_golden.npz")


@pytest.fixture(scope="module")
def decode(golden_dir):
    return np.load(golden_dir / "decode_golden.npz")


def test_rms_norm_bit_exact_vs_native_module(ops):
    y = O.rms_norm(bf(ops["norm_x"]), bf(ops["norm_w"]), 1e-6)
    assert torch.equal(y.view(torch.int16), bf(ops["norm_y"]).view(torch.int16))


def test_rotary_tables_bit_exact_vs_native_module(ops):
    cos, sin = O.rotary_tables(1_000_000.0, 512)
    pos = torch.from_numpy(ops["rope_positions"])[0]
    assert torch.equal(cos[pos].view(torch.int16), bf(ops["rope_cos"]).view(torch.int16))
    assert torch.equal(sin[pos].view(torch.int16), bf(ops["rope_sin"]).view(torch.int16))


def test_rope_bit_exact_vs_native_apply_rotary(ops):
    cos, sin = bf(ops["rope_cos"]), bf(ops["rope_sin"])          # [8, 128]
    q, k = bf(ops["rope_q"]), bf(ops["rope_k"])                  # [1, H, 8, 128]
    qe = O.rope(q, cos[None, None], sin[None, None])
    ke = O.rope(k, cos[None, None], sin[None, None])
    assert torch.equal(qe.view(torch.int16), bf(ops["rope_qe"]).view(torch.int16))
    assert torch.equal(ke.view(torch.int16), bf(ops["rope_ke"]).view(torch.int16))


def test_mlp_restatement_vs_native_module(ops):
    x = bf(ops["mlp_x"])
    wgu = torch.cat((bf(ops["mlp_gate"]), bf(ops["mlp_up"])), 0)
    y = O.linear(O.swiglu(O.linear(x, wgu)), bf(ops["mlp_down"]))
    ref = bf(ops["mlp_y"])
    # CPU bf16 matmul accumulates in a different order than the fp32 product:
    # one bf16 ulp on a few elements is the expected difference.
    torch.testing.assert_close(y.float(), ref.float(), rtol=1.6e-2, atol=1e-3)
    assert (y.view(torch.int16) == ref.view(torch.int16)).float().mean() > 0.9


def test_constant_row_rope_known_answer():
    """eps=0 and a constant row normalise to exactly 1, so the output is
    bf16(bf16(cos) -+ bf16(sin)) (reference tests/test_decode_step.py:296-321)."""
    cos, sin = O.rotary_tables(1_000_000.0, 40)
    packed = torch.full((1, (4 + 2 * 2) * 128), 3.0, dtype=torch.bfloat16)
    one = torch.ones(128, dtype=torch.bfloat16)
    q, k, v = O.qkv_norm_rope(packed, one, one, 0.0, cos[17:18], sin[17:18], 4, 2)
    sign = torch.cat((-torch.ones(64), torch.ones(64))).to(torch.bfloat16)
    expected = cos[17] + sign * sin[17]
    assert torch.equal(q[0, 0], expected) and torch.equal(k[0, 1], expected)
    assert torch.equal(v, torch.full_like(v, 3.0))


def test_attention_known_answers():
    """Uniform scores average the values; one extreme key wins outright
    (reference tests/test_small_query_attention.py:259-275)."""
    torch.manual_seed(3)
    q = torch.zeros((1, 1, 4, 128), dtype=torch.bfloat16)
    k = torch.randn((1, 1, 50, 128)).to(torch.bfloat16)
    v = torch.randn((1, 1, 50, 128)).to(torch.bfloat16)
    lim = torch.tensor([[50]])
    out = O.attention_fp64(q, k, v, lim, 128 ** -0.5)
    torch.testing.assert_close(out[0, 0, 0].float(), v[0, 0].float().mean(0), rtol=0, atol=8e-3)
    q2 = (k[0, 0, 7] * 4).view(1, 1, 1, 128).repeat(1, 1, 4, 1)
    out2 = O.attention_fp64(q2, k, v, lim, 1.0)
    torch.testing.assert_close(out2[0, 0, 0].float(), v[0, 0, 7].float(), rtol=0, atol=1e-2)
    both = O.attention_flash_rounding(q2, k, v, lim, 1.0)
    torch.testing.assert_close(both.float(), out2.float(), rtol=0.02, atol=5e-3)


def test_greedy_pick_lowest_index_on_ties():
    lg = torch.zeros((2, 9), dtype=torch.bfloat16)
    lg[1, 4] = lg[1, 6] = 2.0
    assert O.greedy_pick(lg).tolist() == [0, 4]


def _restated(golden_dir):
    sd, cfg = O.load_state_dict(str(golden_dir / "tiny_qwen3"))
    return O.RestatedModel(sd, cfg)


def test_restated_model_vs_golden_decode(golden_dir, decode):
    model = _restated(golden_dir)
    for i in range(3):
        prompt = decode[f"prompt_{i}"]
        n = decode[f"tokens_{i}"].shape[0]
        _, logits = model.greedy(prompt, n)
        # first step only (later steps may follow a different near-tie pick); the
        # bar is max abs diff <= 2e-2 after fp32 upcast
        ref = torch.from_numpy(decode[f"logits_{i}"])
        assert float((logits[0] - ref[0]).abs().max()) <= 2e-2


def test_restated_model_teacher_forced_vs_golden(golden_dir, decode):
    """Feeds the GOLDEN tokens (not its own picks), so every step is compared."""
    model = _restated(golden_dir)
    for i in range(3):
        prompt = torch.from_numpy(decode[f"prompt_{i}"])
        tokens = torch.from_numpy(decode[f"tokens_{i}"])          # [N, B]
        ref = torch.from_numpy(decode[f"logits_{i}"])
        model.keys = model.values = None
        model.length = 0
        current = prompt
        for step in range(tokens.shape[0]):
            lg = model.forward(current).float()
            diff = float((lg - ref[step]).abs().max())
            assert diff <= 2e-2, (i, step, diff)
            pick = O.greedy_pick(lg.to(torch.bfloat16))
            gold = tokens[step]
            for b in range(gold.shape[0]):
                if int(pick[b]) != int(gold[b]):
                    gap = float(ref[step, b].max() - ref[step, b, int(pick[b])])
                    assert gap <= 2e-2, ("non-tie divergence", i, step, b, gap)
            current = gold[:, None]


def test_native_live_matches_golden(golden_dir, decode):
    """The installed Transformers still reproduces the committed vectors."""
    model = O.native_model(str(golden_dir / "tiny_qwen3"))
    for i in range(3):
        tokens, logits = O.native_greedy(model, decode[f"prompt_{i}"], decode[f"tokens_{i}"].shape[0])
        assert np.array_equal(np.asarray(tokens), decode[f"tokens_{i}"])
        torch.testing.assert_close(logits, torch.from_numpy(decode[f"logits_{i}"]), rtol=0, atol=0)


def test_zero_lm_head_gives_token_zero(golden_dir):
    """Tied zero embedding => all logits equal => lowest index 0 every step, and
    generation never stops early (reference tests/test_small_query_attention.py:570-574)."""
    sd, cfg = O.load_state_dict(str(golden_dir / "tiny_qwen3"))
    sd = dict(sd)
    sd["model.embed_tokens.weight"] = torch.zeros_like(sd["model.embed_tokens.weight"])
    sd.pop("lm_head.weight", None)
    tokens, _ = O.RestatedModel(sd, cfg).greedy([[5, 9, 2]], 4)
    assert tokens == [[0], [0], [0], [0]]
