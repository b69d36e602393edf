"""Per-operator parity: every CUDA kernel, called through the C ABI, against the
CPU oracle on the same seeded inputs."""
import math

import pytest
import torch

from oracle import qwen3_oracle as O
from tests.parity import bit_equal_fraction, sum_slots

pytestmark = pytest.mark.gpu

H, I, V = 2560, 9728, 151936
SHAPES = {"qkv": (6144, H), "o": (H, 4096), "gate_up": (2 * I, H), "down": (H, I), "lm_head": (V, H)}


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("needs CUDA")
    from starter_b200 import ops as ops_mod
    return ops_mod


def randw(n, k, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn((n, k), generator=g) * 0.02).to(torch.bfloat16)


def randx(m, k, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn((m, k), generator=g).to(torch.bfloat16)


@pytest.mark.parametrize("name", list(SHAPES))
@pytest.mark.parametrize("M", [1, 4, 8, 16, 32])
def test_split_k_gemm_matches_fp32_product(ops, name, M):
    """Slot sum vs the fp32 product: rtol=atol=2e-3; after the single bf16 rounding
    rtol=1.6e-2, atol=1e-2 (reference tests/test_skinny_gemm.py:479-481)."""
    N, K = SHAPES[name]
    w, x = randw(N, K, 11), randx(M, K, 100 + M)
    wd, xd = w.cuda(), x.cuda()
    before = (wd.clone(), xd.clone())
    part = ops.linear_partials(xd, wd)
    torch.cuda.synchronize()
    assert torch.equal(before[0], wd) and torch.equal(before[1], xd)      # inputs untouched
    ref = O.linear_fp32(x, w)
    got_dev = part.sum().cpu()
    got_host = sum_slots(part)
    assert torch.equal(got_dev, got_host)
    torch.testing.assert_close(got_host, ref, rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(got_host.to(torch.bfloat16).float(), ref.to(torch.bfloat16).float(),
                               rtol=1.6e-2, atol=1e-2)


@pytest.mark.parametrize("M,N,K", [(1, 16, 32), (3, 127, 128), (5, 40, 64), (64, 256, 512), (33, 48, 96)])
def test_split_k_gemm_ragged_and_tiny(ops, M, N, K):
    w, x = randw(N, K, 5), randx(M, K, 6)
    part = ops.linear_partials(x.cuda(), w.cuda())
    torch.testing.assert_close(sum_slots(part), O.linear_fp32(x, w), rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("N,K", [(16, 32), (127, 128), (2560, 4096), (100, 9728)])
def test_weight_tiling_round_trip(ops, N, K):
    """pack -> unpack returns the matrix bit for bit; rows past N are zero in the
    tiled form; a 16-row-aligned row slice of the tiled form is the tiling of the slice."""
    w = randw(N, K, 3).cuda()
    tiled = ops.pack_weight(w)
    assert tiled.data.numel() == ((N + 15) // 16) * (K // 32) * 1024
    assert torch.equal(tiled.rows(), w)
    if N % 16:
        pad = torch.zeros(((N + 15) // 16 * 16, K), dtype=torch.bfloat16, device="cuda")
        pad[:N] = w
        assert torch.equal(ops.pack_weight(pad).data, tiled.data)
    if N >= 48:
        assert torch.equal(tiled.row_slice(16, 48).data, ops.pack_weight(w[16:48].contiguous()).data)
    x = randx(3, K, 4).cuda()
    a = ops.linear_partials(x, tiled)
    b = ops.linear_partials(x, w)
    assert torch.equal(a.sum(), b.sum())


def test_gemm_rejects_bad_operands(ops):
    x, w = randx(2, 64, 1).cuda(), randw(16, 64, 2).cuda()
    with pytest.raises(ValueError):
        ops.linear_partials(x.float(), w)
    with pytest.raises(ValueError):
        ops.linear_partials(x, w[:, :32])                 # non-contiguous
    with pytest.raises(ValueError):
        ops.linear_partials(randx(65, 64, 1).cuda(), w)   # too many rows
    with pytest.raises(ValueError):
        ops.linear_partials(x[:, :48].contiguous(), w[:, :48].contiguous())   # K % 32


@pytest.mark.parametrize("M", [1, 8, 32])
def test_add_rms_norm_on_partials(ops, M):
    """Residual bit-exact; normed within one bf16 ulp (reference
    tests/test_decode_step.py:237-238: residual exact, normed rtol=8e-3)."""
    w, x = randw(H, 4096, 21), randx(M, 4096, 22)
    res = randx(M, H, 23)
    gain = (1 + 0.1 * torch.randn(H, generator=torch.Generator().manual_seed(24))).to(torch.bfloat16)
    part = ops.linear_partials(x.cuda(), w.cuda())
    total, normed = ops.add_rms_norm(res.cuda(), part, gain.cuda(), 1e-6)
    et, en = O.add_rms_norm(res, sum_slots(part), gain, 1e-6)
    assert torch.equal(total.cpu().view(torch.int16), et.view(torch.int16))
    torch.testing.assert_close(normed.cpu().float(), en.float(), rtol=8e-3, atol=1e-6)
    assert bit_equal_fraction(normed.cpu(), en) > 0.99
    # plain fp32 branch (the tensor-parallel path) gives the same answer
    total2, normed2 = ops.add_rms_norm(res.cuda(), part.sum(), gain.cuda(), 1e-6)
    assert torch.equal(total2, total) and torch.equal(normed2, normed)


@pytest.mark.parametrize("M,N", [(1, 2 * I), (3, 6144), (8, 2 * I), (1, 151936)])
def test_add_rms_norm_as_gemm_prologue(ops, M, N):
    """One launch (add + norm in every CTA's shared memory, then the projection) against
    the two-launch sequence: the residual is bit-identical, and so are the projection's
    summed partials wherever the normed activations agree (the sum of squares is reduced in
    a different order, so an activation may differ by one bf16 ulp in rare rows)."""
    w0, x = randw(H, 4096, 121), randx(M, 4096, 122)
    res = randx(M, H, 123)
    gain = (1 + 0.1 * torch.randn(H, generator=torch.Generator().manual_seed(124))).to(torch.bfloat16)
    w1 = randw(N, H, 125).cuda()
    part = ops.linear_partials(x.cuda(), w0.cuda())
    total, normed = ops.add_rms_norm(res.cuda(), part, gain.cuda(), 1e-6)
    want = ops.linear_partials(normed, w1).sum()
    for branch in (part, part.sum()):
        total2, got = ops.add_rms_norm_linear(res.cuda(), branch, gain.cuda(), 1e-6, w1)
        assert torch.equal(total2, total)
        assert got.plan.slots == ops.linear_partials(normed, w1).plan.slots
        torch.testing.assert_close(got.sum(), want, rtol=2e-3, atol=2e-3)
        assert (got.sum() == want).float().mean().item() > 0.9
    # and against the oracle's chain
    et, en = O.add_rms_norm(res, sum_slots(part), gain, 1e-6)
    ref = O.linear_fp32(en, w1.cpu())
    torch.testing.assert_close(got.sum().cpu(), ref, rtol=2e-2, atol=2e-2)
    with pytest.raises(ValueError):
        ops.add_rms_norm_linear(randx(9, H, 126).cuda(), torch.zeros(9, H, device="cuda"), gain.cuda(),
                                1e-6, w1)


@pytest.mark.parametrize("M", [1, 3, 8, 16, 32, 64])
@pytest.mark.parametrize("inter,K", [(I, H), (1216, H), (72, 256)])
def test_gate_up_with_swiglu_epilogue(ops, M, inter, K):
    """One launch (every CTA owns whole 16-row groups of the interleaved gate|up weight and
    applies SwiGLU to its complete sums) against the partials + SwiGLU route and the oracle."""
    w, x = randw(2 * inter, K, 131), randx(M, K, 132) * 3
    got = ops.linear_silu_mul(x.cuda(), w.cuda())
    two = ops.silu_mul(ops.linear_partials(x.cuda(), w.cuda()))
    ref = O.swiglu(O.linear_fp32(x, w))
    assert got.shape == (M, inter)
    # the oracle adds the K products in another order: a gate sum that lands on the other
    # side of a bf16 rounding point moves silu(gate) by up to ~2 ulp where silu is steep
    # relative to its value (gate around -3), and the product rounds once more
    torch.testing.assert_close(got.cpu().float(), ref.float(), rtol=4e-2, atol=1e-3)
    assert bit_equal_fraction(got.cpu(), ref) > 0.99
    assert bit_equal_fraction(got, two) > 0.995          # same sums up to fp32 order


@pytest.mark.parametrize("M", [1, 5, 8])
def test_add_norm_gate_up_swiglu_one_launch(ops, M):
    w0, x = randw(H, 4096, 141), randx(M, 4096, 142)
    res = randx(M, H, 143)
    gain = (1 + 0.1 * torch.randn(H, generator=torch.Generator().manual_seed(144))).to(torch.bfloat16)
    wgu = randw(2 * I, H, 145).cuda()
    part = ops.linear_partials(x.cuda(), w0.cuda())
    total, normed = ops.add_rms_norm(res.cuda(), part, gain.cuda(), 1e-6)
    want = ops.linear_silu_mul(normed, wgu)
    total2, got = ops.add_rms_norm_linear_silu_mul(res.cuda(), part, gain.cuda(), 1e-6, wgu)
    assert torch.equal(total2, total)
    torch.testing.assert_close(got.float(), want.float(), rtol=1.6e-2, atol=1e-4)
    assert bit_equal_fraction(got, want) > 0.9


@pytest.mark.parametrize("M", [1, 16])
def test_swiglu_on_partials(ops, M):
    w, x = randw(2 * I, H, 31), randx(M, H, 32) * 3
    part = ops.linear_partials(x.cuda(), w.cuda())
    got = ops.silu_mul(part).cpu()
    ref = O.swiglu(sum_slots(part))
    torch.testing.assert_close(got.float(), ref.float(), rtol=8e-3, atol=1e-6)
    assert bit_equal_fraction(got, ref) > 0.99
    assert bit_equal_fraction(ops.linear_silu_mul(x.cuda(), w.cuda()).cpu(), got) > 0.995


@pytest.mark.parametrize("M", [9, 32, 64])
@pytest.mark.parametrize("inter,K", [(I, H), (1216, H)])
def test_swiglu_on_interleaved_partials(ops, M, inter, K):
    """The route the step takes above 8 rows on the stream-K kernel: partials of the gate|up
    weight whose rows are interleaved in blocks of 8, then SwiGLU reading gate column
    16(c/8) + c%8 and up column + 8, against the oracle on the de-interleaved sums."""
    import ctypes as C
    from starter_b200 import _lib
    from starter_b200.weights import TiledWeight, deinterleave_gate_up
    w, x = randw(2 * inter, K, 33), randx(M, K, 34) * 3
    tiled = TiledWeight.pack(w.cuda(), interleave8=True)
    part = ops.linear_partials(x.cuda(), TiledWeight(tiled.data, 2 * inter, K))       # columns stay interleaved
    out = torch.empty((M, inter), dtype=torch.bfloat16, device="cuda")
    # q_swiglu reads [gate | up]; the engine's interleaved form is reached through q_gemm_swiglu's
    # layout, exercised here by de-interleaving the summed columns on the host for the oracle
    sums = sum_slots(part)                                                            # [M, 2I] interleaved
    plain = deinterleave_gate_up(sums.t().contiguous()).t().contiguous()              # [M, 2I] gate | up
    ref = O.swiglu(plain)
    # the product path: the same weight through the epilogue kernel and through partials + SwiGLU
    one = ops.linear_silu_mul(x.cuda(), tiled)
    torch.testing.assert_close(one.cpu().float(), ref.float(), rtol=4e-2, atol=1e-3)
    assert bit_equal_fraction(one.cpu(), ref) > 0.99
    from starter_b200.ops import _ptr, _stream
    _lib.check(_lib.lib.q_swiglu_interleaved(_ptr(part.data), C.byref(part.plan), _ptr(out), M, inter, _stream()))
    torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=8e-3, atol=1e-6)
    assert bit_equal_fraction(out.cpu(), ref) > 0.99


def _emulated_peers(rows, cols, world=2):
    """Two tensor-parallel "ranks" on ONE GPU: both ranks' receive areas are the same buffer
    (every push lands in it once per destination), the counter words are shared, and the
    launches of the ranks run one after the other on one stream - nothing ever waits for a
    launch that has not finished."""
    import ctypes as C
    from starter_b200 import _lib
    pairs = 2 * world * 2 * rows * cols                       # [2 halves][world][2 slots][rows][cols]
    buf = torch.zeros(2 * pairs + _lib.lib.q_peer_flag_bytes() // 4, dtype=torch.float32, device="cuda")
    counters = torch.zeros(4, dtype=torch.int32, device="cuda")
    views = []
    for rank in range(world):
        peers = _lib.Peers()
        peers.rank, peers.world = rank, world
        for r in range(world):
            peers.partials[r] = buf.data_ptr()
            peers.flags[r] = buf.data_ptr() + 2 * pairs * 4
        peers.epoch = counters.data_ptr()
        views.append(peers)
    return views, counters, buf


@pytest.mark.parametrize("M", [1, 3, 8])
def test_peer_exchange_inside_the_projections(ops, M):
    """q_gemm_push on two emulated ranks (a row-parallel projection split over K), then the
    polling add+norm prologue of the next projection on one of them: residual and projection
    against the same computation on the unsplit operands. Twice (both halves of the receive
    area), then the SwiGLU form."""
    import ctypes as C
    from starter_b200 import _lib
    from starter_b200.weights import TiledWeight
    lib, check = _lib.lib, _lib.check
    P = lambda t: C.c_void_p(t.data_ptr())
    Kp, N1 = 1024, 384
    w0, x = randw(H, 2 * Kp, 161), randx(M, 2 * Kp, 162)
    res = randx(M, H, 163).cuda()
    gain = (1 + 0.1 * torch.randn(H, generator=torch.Generator().manual_seed(164))).to(torch.bfloat16).cuda()
    w1 = randw(N1, H, 165).cuda()
    wgu = randw(2 * 1216, H, 166).cuda()
    shards = [(x[:, r * Kp:(r + 1) * Kp].contiguous().cuda(), TiledWeight.pack(w0[:, r * Kp:(r + 1) * Kp].contiguous().cuda()))
              for r in range(2)]
    views, counters, _ = _emulated_peers(M, H)
    plan0 = _lib.plan(M, H, Kp)
    # the unsplit route: partials of the whole projection, add+norm as the next one's prologue
    whole = ops.linear_partials(x.cuda(), w0.cuda())
    want_total, want = ops.add_rms_norm_linear(res, whole, gain, 1e-6, w1)
    w1t = TiledWeight.pack(w1)
    p1 = _lib.plan(M, N1, H)
    for call in (1, 2):
        for r in range(2):
            check(lib.q_gemm_push(P(shards[r][0]), P(shards[r][1].data), C.byref(plan0), C.byref(views[r]), None))
        total = torch.empty_like(res)
        data = torch.empty((p1.slots, M, N1), dtype=torch.float32, device="cuda")
        check(lib.q_gemm_splitk_addnorm_peers(P(res), C.byref(views[0]), C.byref(plan0), P(gain), P(total),
                                              P(w1t.data), P(data), M, N1, H, 1e-6, None))
        torch.cuda.synchronize()
        assert counters.tolist() == [call, 0, 0, 0]
        # same products, another fp32 order: the rounded residual agrees except at rounding ties
        assert bit_equal_fraction(total, want_total) > 0.995
        got = ops.Partials(data, p1).sum()
        torch.testing.assert_close(got, want.sum(), rtol=2e-2, atol=2e-2)
    et, en = O.add_rms_norm(res.cpu(), O.linear_fp32(x, w0), gain.cpu(), 1e-6)
    assert bit_equal_fraction(total.cpu(), et) > 0.995
    torch.testing.assert_close(got.cpu(), O.linear_fp32(en, w1.cpu()), rtol=2e-2, atol=2e-2)
    # SwiGLU form
    for r in range(2):
        check(lib.q_gemm_push(P(shards[r][0]), P(shards[r][1].data), C.byref(plan0), C.byref(views[r]), None))
    wt = TiledWeight.pack(wgu, interleave8=True)
    total2 = torch.empty_like(res)
    act = torch.empty((M, 1216), dtype=torch.bfloat16, device="cuda")
    check(lib.q_gemm_swiglu_addnorm_peers(P(res), C.byref(views[1]), C.byref(plan0), P(gain), P(total2), P(wt.data),
                                          P(act), M, 1216, H, 1e-6, None))
    torch.cuda.synchronize()
    assert torch.equal(total2, total) and counters.tolist() == [3, 0, 0, 0]
    _, want_act = ops.add_rms_norm_linear_silu_mul(res, whole, gain, 1e-6, wgu)
    torch.testing.assert_close(act.float(), want_act.float(), rtol=4e-2, atol=2e-3)
    assert ops.device_status() == [0, 0, 0, 0]


def test_peer_exchange_inside_the_projections_times_out(ops):
    """Only one of two ranks pushes: the polling prologue gives up after the wait limit, sets
    status word 1 to 4 and finishes (nothing hangs); q_clear_status re-arms."""
    import ctypes as C
    from starter_b200 import _lib
    from starter_b200.weights import TiledWeight
    lib, check = _lib.lib, _lib.check
    P = lambda t: C.c_void_p(t.data_ptr())
    M, Kp, N1 = 2, 256, 128
    x, w0 = randx(M, Kp, 171).cuda(), TiledWeight.pack(randw(H, Kp, 172).cuda())
    res = randx(M, H, 173).cuda()
    gain = torch.ones(H, dtype=torch.bfloat16, device="cuda")
    w1 = TiledWeight.pack(randw(N1, H, 174).cuda())
    views, counters, _ = _emulated_peers(M, H)
    plan0, p1 = _lib.plan(M, H, Kp), _lib.plan(M, N1, H)
    ops.clear_status()
    check(lib.q_gemm_push(P(x), P(w0.data), C.byref(plan0), C.byref(views[0]), None))       # rank 1 never pushes
    total = torch.empty_like(res)
    data = torch.empty((p1.slots, M, N1), dtype=torch.float32, device="cuda")
    check(lib.q_set_option(b"peer_wait_iters", 2000))
    try:
        check(lib.q_gemm_splitk_addnorm_peers(P(res), C.byref(views[0]), C.byref(plan0), P(gain), P(total), P(w1.data),
                                              P(data), M, N1, H, 1e-6, None))
        torch.cuda.synchronize()
    finally:
        check(lib.q_set_option(b"peer_wait_iters", 1 << 21))
    assert ops.device_status() == [0, 4, 0, 0]
    assert counters.tolist() == [1, 0, 0, 0]                   # the call completed all the same
    ops.clear_status()
    assert ops.device_status() == [0, 0, 0, 0]


def test_rms_norm_plain(ops):
    x = randx(7, H, 41)
    gain = (1 + 0.1 * torch.randn(H, generator=torch.Generator().manual_seed(42))).to(torch.bfloat16)
    got = ops.rms_norm(x.cuda(), gain.cuda(), 1e-6).cpu()
    ref = O.rms_norm(x, gain, 1e-6)
    torch.testing.assert_close(got.float(), ref.float(), rtol=8e-3, atol=1e-6)
    assert bit_equal_fraction(got, ref) > 0.99


@pytest.mark.parametrize("B,T,nq,nkv", [(1, 1, 32, 8), (4, 1, 8, 2), (2, 4, 8, 2), (3, 2, 4, 2)])
def test_qkv_norm_rope_cache(ops, B, T, nq, nkv):
    """Q, K within one ulp of the oracle, V exact; only the slots position..position+T-1
    of the (NaN-poisoned) cache are written (reference tests/test_decode_step.py:278-291)."""
    width = (nq + 2 * nkv) * 128
    capacity, pos = 200, 70
    w, x = randw(width, 256, 51), randx(B * T, 256, 52) * 4
    qg = (1 + 0.1 * torch.randn(128, generator=torch.Generator().manual_seed(53))).to(torch.bfloat16)
    kg = (1 + 0.1 * torch.randn(128, generator=torch.Generator().manual_seed(54))).to(torch.bfloat16)
    cos, sin = O.rotary_tables(1_000_000.0, capacity)
    part = ops.linear_partials(x.cuda(), w.cuda())
    cache = ops.PagedKV(B, nkv, capacity, "cuda", poison=float("nan"))
    position = torch.tensor([pos], dtype=torch.int32, device="cuda")
    q = ops.qkv_norm_rope_cache(part, qg.cuda(), kg.cuda(), 1e-6, 1e-6, cos.cuda(), sin.cuda(),
                                position, cache, tokens_per_seq=T).cpu()
    rows_pos = (pos + torch.arange(T)).repeat(B)
    eq, ek, ev = O.qkv_norm_rope(sum_slots(part), qg, kg, 1e-6, cos[rows_pos], sin[rows_pos], nq, nkv)
    torch.testing.assert_close(q.float(), eq.float(), rtol=0.02, atol=0.02)
    assert bit_equal_fraction(q, eq) > 0.99
    kc, vc = (t.cpu() for t in cache.gather(capacity))
    knew = kc[:, :, pos:pos + T].transpose(1, 2).reshape(B * T, nkv, 128)
    vnew = vc[:, :, pos:pos + T].transpose(1, 2).reshape(B * T, nkv, 128)
    torch.testing.assert_close(knew.float(), ek.float(), rtol=0.02, atol=0.02)
    assert bit_equal_fraction(knew, ek) > 0.99
    assert torch.equal(vnew.view(torch.int16), ev.contiguous().view(torch.int16))
    untouched = torch.ones(capacity, dtype=torch.bool)
    untouched[pos:pos + T] = False
    assert torch.isnan(kc[:, :, untouched].float()).all() and torch.isnan(vc[:, :, untouched].float()).all()


def test_constant_row_rope_bit_exact(ops):
    """eps=0 with constant rows: exactly bf16(cos -+ sin) (reference
    tests/test_decode_step.py:296-321)."""
    nq, nkv, pos = 4, 2, 17
    width = (nq + 2 * nkv) * 128
    x = torch.ones((1, 32), dtype=torch.bfloat16)
    w = torch.full((width, 32), 3.0 / 32, dtype=torch.bfloat16)
    cos, sin = O.rotary_tables(1_000_000.0, 64)
    one = torch.ones(128, dtype=torch.bfloat16)
    cache = ops.PagedKV(1, nkv, 64, "cuda")
    part = ops.linear_partials(x.cuda(), w.cuda())
    q = ops.qkv_norm_rope_cache(part, one.cuda(), one.cuda(), 0.0, 0.0, cos.cuda(), sin.cuda(),
                                torch.tensor([pos], dtype=torch.int32, device="cuda"), cache).cpu()
    sign = torch.cat((-torch.ones(64), torch.ones(64))).to(torch.bfloat16)
    expected = cos[pos] + sign * sin[pos]
    assert torch.equal(q[0, 0], expected) and torch.equal(q[0, 3], expected)
    kc, vc = cache.gather(64)
    assert torch.equal(kc[0, 1, pos].cpu(), expected)
    assert torch.equal(vc[0, 0, pos].cpu(), torch.full((128,), 3.0, dtype=torch.bfloat16))


def _attention_case(ops, B, T, nq, nkv, base_len, capacity, seed, poison=None):
    g = torch.Generator().manual_seed(seed)
    L = base_len + T                              # keys visible to the last query row
    q = torch.randn((B, T, nq, 128), generator=g).to(torch.bfloat16)
    k = torch.randn((B, nkv, L, 128), generator=g).to(torch.bfloat16)
    v = torch.randn((B, nkv, L, 128), generator=g).to(torch.bfloat16)
    cache = ops.PagedKV(B, nkv, capacity, "cuda", poison=poison)
    cache.scatter(k.cuda(), v.cuda(), 0)
    attn = ops.SmallQueryAttention(B, nq, nkv, capacity, "cuda", tokens_per_seq=T)
    position = torch.tensor([base_len], dtype=torch.int32, device="cuda")
    out = attn.run(q.reshape(B * T, nq, 128).cuda(), cache, position, 128 ** -0.5)
    limits = (base_len + torch.arange(T) + 1)[None].repeat(B, 1)
    ref = O.attention_fp64(q, k, v, limits, 128 ** -0.5).reshape(B * T, nq * 128)
    return out.cpu(), ref, (q, k, v, cache, attn)


@pytest.mark.parametrize("base_len", [0, 1, 62, 63, 64, 127, 300, 1000])
@pytest.mark.parametrize("B,nq,nkv", [(1, 32, 8), (3, 8, 2), (2, 4, 2)])
def test_decode_attention_vs_fp64(ops, base_len, B, nq, nkv):
    """rtol=0.02, atol=5e-3 vs the fp64 equations (reference
    tests/test_small_query_attention.py:253,501); unused capacity is NaN."""
    out, ref, _ = _attention_case(ops, B, 1, nq, nkv, base_len, 1100, 60 + base_len, poison=float("nan"))
    assert not torch.isnan(out.float()).any()
    torch.testing.assert_close(out.float(), ref.float(), rtol=0.02, atol=5e-3)
    assert ops.device_status()[0] == 0


@pytest.mark.parametrize("T", [2, 4, 8])
@pytest.mark.parametrize("base_len", [0, 60, 500])
def test_small_query_attention_causal_block(ops, T, base_len):
    out, ref, _ = _attention_case(ops, 2, T, 8, 2, base_len, 640, 70 + T, poison=float("nan"))
    assert not torch.isnan(out.float()).any()
    torch.testing.assert_close(out.float(), ref.float(), rtol=0.02, atol=5e-3)


@pytest.mark.parametrize("T", [2, 8])
def test_small_query_equals_token_by_token_decode(ops, T):
    """The multi-token path against the single-token path run once per token
    on the same cache: same kernel arithmetic, so the results agree to bf16 noise."""
    B, nq, nkv, base, cap = 2, 8, 2, 333, 400
    out, ref, (q, k, v, cache, attn) = _attention_case(ops, B, T, nq, nkv, base, cap, 90 + T)
    single = ops.SmallQueryAttention(B, nq, nkv, cap, "cuda", tokens_per_seq=1)
    rows = []
    for t in range(T):
        position = torch.tensor([base + t], dtype=torch.int32, device="cuda")
        rows.append(single.run(q[:, t].contiguous().cuda(), cache, position, 128 ** -0.5).cpu())
    stepwise = torch.stack(rows, 1).reshape(B * T, nq * 128)
    torch.testing.assert_close(out.float(), stepwise.float(), rtol=0.02, atol=5e-3)


@pytest.mark.parametrize("T", [2, 4, 8])
@pytest.mark.parametrize("L", [4096, 16384, 32768])
def test_attention_verification_grid(ops, L, T):
    """The verification-attention configuration: batch 8, T query tokens, 32/8 heads, L cached
    N(0,1) keys, against the fp64 equations (the shape test of reference
    tests/test_small_query_attention.py:154-166) and, at the shortest length, against the
    single-token kernel run token by token."""
    B, nq, nkv = 8, 32, 8
    out, ref, (q, k, v, cache, attn) = _attention_case(ops, B, T, nq, nkv, L, L + 8, 99 + T)
    torch.testing.assert_close(out.float(), ref.float(), rtol=0.02, atol=5e-3)
    if L == 4096:
        single = ops.SmallQueryAttention(B, nq, nkv, L + 8, "cuda", tokens_per_seq=1)
        rows = []
        for t in range(T):
            position = torch.tensor([L + t], dtype=torch.int32, device="cuda")
            rows.append(single.run(q[:, t].contiguous().cuda(), cache, position, 128 ** -0.5).cpu())
        stepwise = torch.stack(rows, 1).reshape(B * T, nq * 128)
        torch.testing.assert_close(out.float(), stepwise.float(), rtol=0.02, atol=5e-3)


@pytest.mark.parametrize("B,nq,nkv,T,base", [(1, 32, 8, 1024, 0), (2, 8, 2, 333, 0), (3, 4, 2, 65, 0), (2, 4, 4, 130, 0),
                                             (1, 8, 1, 64, 0), (2, 8, 2, 1, 0), (2, 8, 2, 100, 77)])
def test_prompt_attention_vs_fp64(ops, B, nq, nkv, T, base):
    """Causal attention over a whole prompt block against the fp64 equations, same bars as the
    decode kernel; unused page rows are NaN. base > 0 is a block appended to an older context."""
    g = torch.Generator().manual_seed(500 + T)
    L = base + T
    q = torch.randn((B, T, nq, 128), generator=g).to(torch.bfloat16)
    k = torch.randn((B, nkv, L, 128), generator=g).to(torch.bfloat16)
    v = torch.randn((B, nkv, L, 128), generator=g).to(torch.bfloat16)
    cache = ops.PagedKV(B, nkv, L + 40, "cuda", poison=float("nan"))
    cache.scatter(k.cuda(), v.cuda(), 0)
    position = torch.tensor([base], dtype=torch.int32, device="cuda")
    out = ops.prompt_attention(q.reshape(B * T, nq, 128).cuda(), cache, position, T, 128 ** -0.5).cpu()
    limits = (base + torch.arange(T) + 1)[None].repeat(B, 1)
    ref = O.attention_fp64(q, k, v, limits, 128 ** -0.5).reshape(B * T, nq * 128)
    assert not torch.isnan(out.float()).any()
    torch.testing.assert_close(out.float(), ref.float(), rtol=0.02, atol=5e-3)
    assert ops.device_status()[0] == 0


def test_prompt_attention_equals_small_query_kernel(ops):
    """The prompt kernel and the small-query kernel on the same 8-token block of the same cache."""
    B, nq, nkv, base, T = 2, 8, 2, 200, 8
    out, ref, (q, k, v, cache, attn) = _attention_case(ops, B, T, nq, nkv, base, 300, 321)
    position = torch.tensor([base], dtype=torch.int32, device="cuda")
    block = ops.prompt_attention(q.reshape(B * T, nq, 128).cuda(), cache, position, T, 128 ** -0.5).cpu()
    torch.testing.assert_close(block.float(), out.float(), rtol=0.02, atol=5e-3)


@pytest.mark.parametrize("cluster", [True, False])
@pytest.mark.parametrize("B,nq,nkv,pos", [(1, 32, 8, 0), (1, 32, 8, 1100), (3, 8, 2, 63), (2, 8, 2, 64), (4, 4, 2, 700),
                                          (40, 8, 2, 130), (1, 32, 8, 2400)])
def test_fused_decode_attention_equals_the_three_kernels(ops, B, nq, nkv, pos, cluster):
    """One launch (norm + RoPE + K/V write + attention + merge) against the separate
    kernels on the same inputs: bit-identical pages; the attended rows agree to bf16
    rounding and sit within rtol=0.02, atol=5e-3 of each other like every attention check
    here. Most elements are bit-equal, not all: the probabilities are rounded to bf16 relative
    to the running maximum of the softmax state they belong to, and the fused kernel keeps one
    state per (tile, key quarter) when its CTAs have an SM each, the three-kernel path one per
    (split, key quarter).
    `cluster`: up to 8 splits merge through distributed shared memory (default) or, like
    more than 8 splits always do, through global memory and a ticket."""
    from starter_b200 import _lib
    _lib.check(_lib.lib.q_set_option(b"attn_no_cluster", 0 if cluster else 1))
    try:
        _fused_decode_attention_case(ops, B, nq, nkv, pos)
    finally:
        _lib.check(_lib.lib.q_set_option(b"attn_no_cluster", 0))


def _fused_decode_attention_case(ops, B, nq, nkv, pos):
    capacity = max(1200, pos + 100)
    g = torch.Generator().manual_seed(500 + pos + B)
    width = (nq + 2 * nkv) * 128
    w, x = randw(width, 256, 61), randx(B, 256, 62) * 4
    qg = (1 + 0.1 * torch.randn(128, generator=g)).to(torch.bfloat16).cuda()
    kg = (1 + 0.1 * torch.randn(128, generator=g)).to(torch.bfloat16).cuda()
    cos, sin = (t.cuda() for t in O.rotary_tables(1_000_000.0, capacity))
    part = ops.linear_partials(x.cuda(), w.cuda())
    position = torch.tensor([pos], dtype=torch.int32, device="cuda")
    k_old = torch.randn((B, nkv, max(pos, 1), 128), generator=g).to(torch.bfloat16).cuda()
    v_old = torch.randn((B, nkv, max(pos, 1), 128), generator=g).to(torch.bfloat16).cuda()
    caches = []
    for _ in range(2):
        c = ops.PagedKV(B, nkv, capacity, "cuda", poison=float("nan"))
        if pos:
            c.scatter(k_old[:, :, :pos], v_old[:, :, :pos], 0)
        caches.append(c)
    attn = ops.SmallQueryAttention(B, nq, nkv, capacity, "cuda")
    q = ops.qkv_norm_rope_cache(part, qg, kg, 1e-6, 1e-6, cos, sin, position, caches[0])
    ref = attn.run(q, caches[0], position, 128 ** -0.5)
    for _ in range(2):                                  # twice: the tickets must reset themselves
        got = ops.decode_attention(part, qg, kg, 1e-6, cos, sin, position, caches[1], attn, 128 ** -0.5)
        torch.testing.assert_close(got.float(), ref.float(), rtol=0.02, atol=5e-3)
        assert bit_equal_fraction(got, ref) > 0.6
    ka, va = caches[0].gather(pos + 1)
    kb, vb = caches[1].gather(pos + 1)
    assert torch.equal(ka.view(torch.int16), kb.view(torch.int16))
    assert torch.equal(va.view(torch.int16), vb.view(torch.int16))
    assert not torch.isnan(got.float()).any()
    assert ops.device_status()[0] == 0


def test_attention_rejects_bad_shapes(ops):
    with pytest.raises(ValueError):
        ops.SmallQueryAttention(1, 32, 8, 100, "cuda", tokens_per_seq=9)      # 9*4 > 32 rows
    attn = ops.SmallQueryAttention(1, 8, 2, 100, "cuda")
    cache = ops.PagedKV(1, 2, 100, "cuda")
    pos = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError):
        attn.run(torch.zeros((1, 8, 64), dtype=torch.bfloat16, device="cuda"), cache, pos, 0.1)
    with pytest.raises(ValueError):
        attn.run(torch.zeros((1, 8, 128), dtype=torch.bfloat16, device="cuda"), cache, pos.long(), 0.1)


def test_lm_head_argmax_ties_and_logits(ops):
    w, x = randw(5000, 256, 81), randx(6, 256, 82)
    w[4321] = w[17]                       # exact duplicate rows: tie, lowest index must win
    logits, tokens = ops.lm_head_argmax(x.cuda(), w.cuda())
    ref = O.linear(x, w)
    torch.testing.assert_close(logits.cpu().float(), ref.float(), rtol=1.6e-2, atol=1e-2)
    assert tokens.cpu().tolist() == O.greedy_pick(logits.cpu()).tolist()
    zero = torch.zeros_like(w)
    _, tok0 = ops.lm_head_argmax(x.cuda(), zero.cuda())
    assert tok0.cpu().tolist() == [0] * 6
    x1 = torch.zeros((1, 256), dtype=torch.bfloat16)
    x1[0, 0] = 1.0
    w2 = torch.zeros((5000, 256), dtype=torch.bfloat16)
    w2[17, 0] = w2[4321, 0] = w2[4999, 0] = 2.0
    _, tok = ops.lm_head_argmax(x1.cuda(), w2.cuda())
    assert tok.cpu().tolist() == [17]


def test_lm_head_argmax_full_vocab(ops):
    w, x = randw(V, H, 83), randx(4, H, 84)
    logits, tokens = ops.lm_head_argmax(x.cuda(), w.cuda())
    ref = O.linear(x, w)
    assert float((logits.cpu().float() - ref.float()).abs().max()) <= 2e-2
    assert tokens.cpu().tolist() == O.greedy_pick(logits.cpu()).tolist()
