"""End-to-end parity of Engine.generate against native Hugging Face: committed
golden vectors, live tiny random models, graph replay and state reuse."""
import numpy as np
import pytest
import torch

from oracle import qwen3_oracle as O
from tests.parity import own_prefix_report

pytestmark = pytest.mark.gpu

TOL = 2e-2      # max abs logit difference after fp32 upcast


@pytest.fixture(scope="module")
def cuda():
    if not torch.cuda.is_available():
        pytest.skip("needs CUDA")


def run_engine(engine, prompt, n):
    """Generates n tokens and also returns the engine's logits of every step."""
    tokens, logits = [], []
    gen = engine.generate(prompt, n)
    for step in gen:
        tokens.append(step)
        # logits of the step that produced the NEXT token are in state.logits after
        # advance(); the first token's logits come from prefill (library GEMMs).
    return tokens


def stepwise_logits(engine, prompt, n):
    """Drives DecodeState by hand so that each decode step's logits can be read."""
    from starter_b200.decode import DecodeState
    ids = torch.tensor(prompt, dtype=torch.int64, device="cuda")
    with torch.inference_mode():
        state = DecodeState(engine.weights, ids.shape[0], ids.shape[1], n, keep_logits=True)
        stepwise_logits.last_state = state
        first = state.prefill(ids)
        tokens = [state.tokens.cpu().tolist()]
        logits = [first.float().cpu()]
        for _ in range(n - 1):
            state.step()
            torch.cuda.synchronize()
            tokens.append(state.tokens.cpu().tolist())
            logits.append(state.logits.float().cpu())
        assert int(state.position.item()) == ids.shape[1] + n - 1
    return tokens, torch.stack(logits)


def assert_parity(native, prompt, tokens, logits):
    ref, gaps, diffs = own_prefix_report(native, prompt, tokens, logits)
    assert float(diffs.max()) <= TOL, f"max abs logit diff {float(diffs.max()):.4f}"
    # every emitted token is the native argmax or a near tie of it
    assert float(gaps.max()) <= TOL, f"token off the native top by {float(gaps.max()):.4f}"


def test_golden_tiny_model(cuda, golden_dir):
    from starter_b200 import Engine
    decode = np.load(golden_dir / "decode_golden.npz")
    path = str(golden_dir / "tiny_qwen3")
    engine = Engine(path, keep_logits=True)
    native = O.native_model(path)
    for i in range(3):
        prompt = decode[f"prompt_{i}"].tolist()
        gold_tokens = decode[f"tokens_{i}"]
        gold_logits = torch.from_numpy(decode[f"logits_{i}"])
        n = gold_tokens.shape[0]
        tokens, logits = stepwise_logits(engine, prompt, n)
        assert_parity(native, prompt, tokens, logits)
        # against the frozen vectors while the token paths agree
        for step in range(n):
            assert float((logits[step] - gold_logits[step]).abs().max()) <= TOL
            if tokens[step] != gold_tokens[step].tolist():
                break
        # the public generator yields the same tokens as the hand-driven state
        assert list(engine.generate(prompt, n)) == tokens


@pytest.mark.parametrize("nq,nkv,hidden,inter,vocab,layers", [
    (4, 1, 256, 512, 127, 2),        # G=4 like Qwen3-4B
    (8, 8, 128, 128, 333, 1),        # G=1
    (8, 2, 384, 1024, 1000, 3),
])
def test_live_random_models(cuda, tmp_path, nq, nkv, hidden, inter, vocab, layers):
    from transformers import Qwen3Config, Qwen3ForCausalLM
    from starter_b200 import Engine
    torch.manual_seed(nq * 100 + hidden)
    cfg = Qwen3Config(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter,
                      num_hidden_layers=layers, num_attention_heads=nq, num_key_value_heads=nkv,
                      head_dim=128, max_position_embeddings=512, rope_theta=1_000_000.0,
                      tie_word_embeddings=True, sliding_window=None)
    model = Qwen3ForCausalLM(cfg).eval().to(torch.bfloat16)
    model.save_pretrained(tmp_path, safe_serialization=True)
    native = O.native_model(str(tmp_path))
    engine = Engine(str(tmp_path), keep_logits=True)
    gen = torch.Generator().manual_seed(5)
    for batch, length, count in ((2, 7, 5), (1, 1, 2), (4, 130, 6)):
        prompt = torch.randint(0, vocab, (batch, length), generator=gen).tolist()
        tokens, logits = stepwise_logits(engine, prompt, count)
        assert_parity(native, prompt, tokens, logits)


def test_long_prompts_through_the_prompt_pass(cuda, tmp_path):
    """Prompts longer than one row chunk of the tcgen05 projection (256), longer than the
    prompt-pass row budget (2048: one sequence per pass then) and several sequences per pass,
    with 8 query heads per kv head: the own causal attention and the many-row partial plans
    against native Hugging Face."""
    from transformers import Qwen3Config, Qwen3ForCausalLM
    from starter_b200 import Engine
    torch.manual_seed(77)
    cfg = Qwen3Config(vocab_size=300, hidden_size=256, intermediate_size=384, num_hidden_layers=2,
                      num_attention_heads=8, num_key_value_heads=1, head_dim=128, max_position_embeddings=4096,
                      rope_theta=1_000_000.0, tie_word_embeddings=True, sliding_window=None)
    model = Qwen3ForCausalLM(cfg).eval().to(torch.bfloat16)
    model.save_pretrained(tmp_path, safe_serialization=True)
    native = O.native_model(str(tmp_path))
    engine = Engine(str(tmp_path), keep_logits=True)
    gen = torch.Generator().manual_seed(6)
    for batch, length, count in ((1, 2300, 3), (3, 700, 3), (2, 257, 4)):
        prompt = torch.randint(0, 300, (batch, length), generator=gen).tolist()
        tokens, logits = stepwise_logits(engine, prompt, count)
        assert_parity(native, prompt, tokens, logits)


def test_generate_contract_and_graph_replay(cuda, golden_dir):
    """N yields of B ids, none for N<=0, state reused across calls, stable
    addresses, graph replay equals eager stepping (reference tests/test_decode.py:94-118,
    tests/test_decode_step.py:189-214)."""
    from starter_b200 import Engine
    path = str(golden_dir / "tiny_qwen3")
    engine = Engine(path)
    native = O.native_model(path)
    gen = torch.Generator().manual_seed(9)
    assert list(engine.generate([[1, 2, 3]], 0)) == []
    assert list(engine.generate([[1, 2, 3]], -2)) == []
    for batch, length, count in ((2, 7, 5), (2, 7, 5), (1, 1, 2), (2, 7, 1), (3, 65, 40)):
        prompt = torch.randint(0, 127, (batch, length), generator=gen).tolist()
        out = list(engine.generate(prompt, count))
        assert len(out) == count and all(len(step) == batch for step in out)
        state = engine.decode_state
        addresses = [t.data_ptr() for t in state.kpools + state.vpools]
        again = list(engine.generate(prompt, count))          # replay on reused state
        assert again == out
        assert addresses == [t.data_ptr() for t in engine.decode_state.kpools + engine.decode_state.vpools]
        assert int(state.position.item()) == length + count - 1
        _, gaps, _ = own_prefix_report(native, prompt, out)
        assert float(gaps.max()) <= TOL
        eager, _ = stepwise_logits(engine, prompt, count)     # no graph
        assert eager == out


def test_zero_lm_head_yields_token_zero_and_never_stops(cuda, golden_dir, tmp_path):
    """Tied zero embedding: all logits equal, lowest index wins, no early stop
    (reference tests/test_small_query_attention.py:570-574)."""
    import shutil
    from safetensors.torch import load_file, save_file
    from starter_b200 import Engine
    src = golden_dir / "tiny_qwen3"
    shutil.copy(src / "config.json", tmp_path / "config.json")
    sd = load_file(str(src / "model.safetensors"))
    sd["model.embed_tokens.weight"] = torch.zeros_like(sd["model.embed_tokens.weight"])
    sd.pop("lm_head.weight", None)
    save_file(sd, str(tmp_path / "model.safetensors"))
    out = list(Engine(str(tmp_path)).generate([[5, 9, 2], [1, 1, 1]], 6))
    assert out == [[0, 0]] * 6


def test_norm_prologue_step_matches_separate_add_norm_kernels(cuda, golden_dir):
    """Default step (add + norm inside the consuming projection, up to 8 rows) against the
    step with separate add+norm launches: same tokens, logits equal up to the reduction
    order of the sum of squares."""
    from starter_b200 import Engine, _lib
    from starter_b200.ops import device_status
    engine = Engine(str(golden_dir / "tiny_qwen3"), keep_logits=True)
    gen = torch.Generator().manual_seed(22)
    for batch, length, count in ((1, 9, 12), (4, 70, 8), (8, 5, 6)):
        prompt = torch.randint(0, 127, (batch, length), generator=gen).tolist()
        new_tokens, new_logits = stepwise_logits(engine, prompt, count)
        _lib.check(_lib.lib.q_set_option(b"norm_in_gemm", 0))
        try:
            old_tokens, old_logits = stepwise_logits(engine, prompt, count)
        finally:
            _lib.check(_lib.lib.q_set_option(b"norm_in_gemm", 1))
        assert new_tokens == old_tokens
        torch.testing.assert_close(new_logits, old_logits, rtol=1.6e-2, atol=2e-3)
    assert device_status() == [0, 0, 0, 0]


def test_pdl_off_gives_identical_tokens(cuda, golden_dir):
    from starter_b200 import Engine, _lib
    path = str(golden_dir / "tiny_qwen3")
    prompt = [[3, 1, 4, 1, 5, 9, 2, 6]]
    a = list(Engine(path).generate(prompt, 12))
    _lib.lib.q_set_pdl(0)
    try:
        b = list(Engine(path).generate(prompt, 12))
    finally:
        _lib.lib.q_set_pdl(1)
    assert a == b


def _live_model(tmp_path, nq, nkv, hidden, inter, vocab, layers, seed):
    from transformers import Qwen3Config, Qwen3ForCausalLM
    torch.manual_seed(seed)
    cfg = Qwen3Config(vocab_size=vocab, hidden_size=hidden, intermediate_size=inter,
                      num_hidden_layers=layers, num_attention_heads=nq, num_key_value_heads=nkv,
                      head_dim=128, max_position_embeddings=512, rope_theta=1_000_000.0,
                      tie_word_embeddings=True, sliding_window=None)
    Qwen3ForCausalLM(cfg).eval().to(torch.bfloat16).save_pretrained(tmp_path, safe_serialization=True)
    return str(tmp_path)


@pytest.mark.parametrize("route", ["tcgen05", "mma"])
def test_steps_above_8_rows_match_native(cuda, golden_dir, tmp_path, route):
    """The step for 9..64 sequences - projections on the tcgen05 kernel (default) or, with the
    option tc_min_rows out of reach, on the stream-K kernel with SwiGLU and add+norm as
    separate launches - against native Hugging Face at the 2e-2 bar, on the golden tiny model
    and a live model with 4 query heads per kv head (the own-prefix check of reference
    tests/test_skinny_gemm.py:549-588)."""
    from starter_b200 import Engine, _lib
    from starter_b200.ops import device_status
    if route == "mma":
        _lib.check(_lib.lib.q_set_option(b"tc_min_rows", 1000))
    try:
        gen = torch.Generator().manual_seed(31)
        path = str(golden_dir / "tiny_qwen3")
        engine, native = Engine(path, keep_logits=True), O.native_model(path)
        for batch, length, count in ((9, 7, 4), (16, 40, 4), (32, 70, 5), (64, 3, 3)):
            prompt = torch.randint(0, 127, (batch, length), generator=gen).tolist()
            tokens, logits = stepwise_logits(engine, prompt, count)
            assert stepwise_logits.last_state.uses_tc
            assert_parity(native, prompt, tokens, logits)
            assert list(engine.generate(prompt, count)) == tokens          # graph replay, same route
        live = _live_model(tmp_path, 8, 2, 384, 1024, 1000, 3, 77)
        engine, native = Engine(live, keep_logits=True), O.native_model(live)
        for batch, length, count in ((12, 33, 4), (32, 130, 4)):
            prompt = torch.randint(0, 1000, (batch, length), generator=gen).tolist()
            tokens, logits = stepwise_logits(engine, prompt, count)
            assert_parity(native, prompt, tokens, logits)
    finally:
        _lib.check(_lib.lib.q_set_option(b"tc_min_rows", 9))
    assert device_status() == [0, 0, 0, 0]


def test_both_routes_above_8_rows_agree(cuda, golden_dir):
    """tcgen05 route against the stream-K route at 32 rows: same tokens, logits equal up to the
    fp32 summation order of the projections (one bf16 ulp)."""
    from starter_b200 import Engine, _lib
    engine = Engine(str(golden_dir / "tiny_qwen3"), keep_logits=True)
    prompt = torch.randint(0, 127, (32, 50), generator=torch.Generator().manual_seed(41)).tolist()
    tc_tokens, tc_logits = stepwise_logits(engine, prompt, 6)
    _lib.check(_lib.lib.q_set_option(b"tc_min_rows", 1000))
    try:
        mma_tokens, mma_logits = stepwise_logits(engine, prompt, 6)
    finally:
        _lib.check(_lib.lib.q_set_option(b"tc_min_rows", 9))
    torch.testing.assert_close(tc_logits[:2], mma_logits[:2], rtol=1.6e-2, atol=4e-3)
    assert tc_tokens[:2] == mma_tokens[:2]


@pytest.mark.parametrize("batch,T", [(1, 4), (2, 8), (8, 8), (3, 2)])
def test_verify_step_equals_single_token_steps(cuda, golden_dir, batch, T):
    """q_verify_step on T candidate tokens per sequence gives, for every row, the token that T
    single-token steps produce (the candidates ARE the greedy continuation here), and wrong
    candidates change nothing before them."""
    from starter_b200 import Engine
    from starter_b200.decode import DecodeState
    engine = Engine(str(golden_dir / "tiny_qwen3"))
    gen = torch.Generator().manual_seed(51 + batch)
    length, count = 20, T + 1
    prompt = torch.randint(0, 127, (batch, length), generator=gen)
    greedy = torch.tensor(list(engine.generate(prompt.tolist(), count)))          # [count, batch]
    with torch.inference_mode():
        state = DecodeState(engine.weights, batch, length, count)
        state.prefill(prompt.cuda())
        assert state.tokens.cpu().tolist() == greedy[0].tolist()
        ver = DecodeState(engine.weights, batch, length, count, q_tokens=T, share=state)
        cand = greedy[:T].t().contiguous().cuda()                                  # [batch, T]
        nxt = ver.verify(cand).cpu()
        assert nxt.tolist() == greedy[1:T + 1].t().tolist()
        assert int(state.position.item()) == length                              # nothing advanced
        # corrupt the last candidate: successors of the earlier rows stay
        bad = cand.clone()
        bad[:, -1] = (bad[:, -1] + 1) % 127
        nxt2 = ver.verify(bad).cpu()
        assert nxt2[:, :T - 1].tolist() == greedy[1:T].t().tolist()


def test_speculative_generate_is_exact(cuda, golden_dir):
    """The accept-prefix loop over q_verify_step emits exactly the greedy tokens, whatever the
    drafts are; a repetitive prompt makes the prompt-lookup drafter hit."""
    from starter_b200 import Engine
    from starter_b200.speculative import generate_speculative
    engine = Engine(str(golden_dir / "tiny_qwen3"))
    gen = torch.Generator().manual_seed(61)
    base = torch.randint(0, 127, (2, 6), generator=gen)
    prompt = base.repeat(1, 5).tolist()
    want = list(engine.generate(prompt, 24))
    for T in (2, 4, 8):
        got, stats = generate_speculative(engine, prompt, 24, draft_tokens=T)
        assert got == want
        assert stats["verify_calls"] >= 1 and stats["emitted"] == 24


def test_device_status_is_surfaced_and_cleared(cuda, golden_dir):
    """A wait that ran out must reach the caller as an error: the peer add+norm is called on ONE
    GPU with a world of two whose second arrival word nobody writes and a short wait limit. The
    kernel returns, status word 3 is set, the engine's next step raises, and q_clear_status
    re-arms. Nothing faults or hangs: the wait gives up and the kernel finishes."""
    import ctypes as C
    from starter_b200 import Engine, _lib
    from starter_b200.ops import clear_status, device_status
    lib, check = _lib.lib, _lib.check
    clear_status()
    rows, cols = 2, 256
    recv = 2 * 2 * 2 * rows * cols                   # [2 halves][world][rows][cols] pairs of 2 floats
    buf = torch.zeros(recv + lib.q_peer_flag_bytes() // 4, dtype=torch.float32, device="cuda")
    own = torch.ones((rows, cols), dtype=torch.float32, device="cuda")
    counters = torch.zeros(4, dtype=torch.int32, device="cuda")
    peers = _lib.Peers()
    peers.rank, peers.world = 0, 2
    for r in range(2):
        peers.partials[r] = buf.data_ptr()
        peers.flags[r] = buf.data_ptr() + recv * 4
    peers.epoch = counters.data_ptr()
    x = torch.zeros((rows, cols), dtype=torch.bfloat16, device="cuda")
    gain = torch.ones(cols, dtype=torch.bfloat16, device="cuda")
    total, normed = torch.empty_like(x), torch.empty_like(x)
    check(lib.q_set_option(b"peer_wait_iters", 2000))
    try:
        check(lib.q_add_rmsnorm_peers(C.c_void_p(x.data_ptr()), C.byref(peers), C.c_void_p(own.data_ptr()), None,
                                      C.c_void_p(gain.data_ptr()), C.c_void_p(total.data_ptr()),
                                      C.c_void_p(normed.data_ptr()), rows, cols, 1e-6, None))
        torch.cuda.synchronize()
    finally:
        check(lib.q_set_option(b"peer_wait_iters", 1 << 21))
    assert device_status() == [0, 0, 0, 1]
    assert counters.tolist() == [1, 0, 0, 0]                            # the call completed, ticket re-armed
    engine = Engine(str(golden_dir / "tiny_qwen3"))
    with pytest.raises(_lib.QDecodeError, match="peer exchange"):
        list(engine.generate([[1, 2, 3]], 4))
    clear_status()
    assert device_status() == [0, 0, 0, 0]
    assert len(list(engine.generate([[1, 2, 3]], 4))) == 4
