"""The tcgen05 projection (q_gemm_tc, 9 rows and more) through the C ABI against the CPU
oracle: the 128 x 64 weight tiling, the partial slots, and the fused consumers reading them."""
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


@pytest.mark.parametrize("N,K", [(128, 64), (16, 32), (127, 128), (300, 96), (2560, 4096), (100, 9728)])
def test_tile_round_trip(ops, N, K):
    """pack -> unpack returns the matrix bit for bit; rows past N and k past K are zero in
    the tiled form; one tile is the swizzled image: chunk c of row r sits at chunk c ^ (r % 8)."""
    w = randw(N, K, 3).cuda()
    tiled = ops.pack_weight_tc(w)
    kt, blocks = (K + 63) // 64, (N + 127) // 128
    assert tiled.data.numel() == blocks * kt * 16384 and tiled.data.data_ptr() % 1024 == 0
    assert torch.equal(tiled.rows(), w)
    img = tiled.data.view(torch.bfloat16).view(blocks, kt, 128, 8, 8).cpu()     # [block][kt][row][chunk][8]
    pad = torch.zeros((blocks * 128, kt * 64), dtype=torch.bfloat16)
    pad[:N, :K] = w.cpu()
    for r in (0, 1, 5, 9, 127):
        for c in (0, 3, 7):
            want = pad[r, c * 8:c * 8 + 8]
            assert torch.equal(img[0, 0, r, c ^ (r % 8)], want)
    # undo the swizzle of the whole image and compare with the zero-padded matrix
    rows = torch.arange(128)
    src = (torch.arange(8)[None, :] ^ (rows[:, None] % 8))                   # physical chunk of logical chunk c
    idx = src.view(1, 1, 128, 8, 1).expand(blocks, kt, 128, 8, 8)
    plain = torch.gather(img, 3, idx).reshape(blocks, kt, 128, 64).permute(0, 2, 1, 3).reshape(blocks * 128, kt * 64)
    assert torch.equal(plain, pad)


@pytest.mark.parametrize("name", list(SHAPES))
@pytest.mark.parametrize("M", [9, 16, 32, 64])
def test_tc_gemm_matches_fp32_product(ops, name, M):
    """Slot sum vs the fp32 product: rtol=atol=2e-3; after the single bf16 rounding
    rtol=1.6e-2, atol=1e-2 (the bars of reference tests/test_skinny_gemm.py:479-481)."""
    N, K = SHAPES[name]
    if name == "lm_head" and M not in (16, 64):
        pytest.skip("lm_head checked at two row counts")
    w, x = randw(N, K, 11), randx(M, K, 100 + M)
    wd, xd = ops.pack_weight_tc(w.cuda()), x.cuda()
    before = (wd.data.clone(), xd.clone())
    part = ops.linear_partials_tc(xd, wd)
    torch.cuda.synchronize()
    assert torch.equal(before[0], wd.data) and torch.equal(before[1], xd)      # inputs untouched
    assert part.plan.group_rows == 128
    ref = O.linear_fp32(x, w)
    got_host = sum_slots(part)
    assert torch.equal(part.sum().cpu(), got_host)
    torch.testing.assert_close(got_host, ref, rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(got_host.to(torch.bfloat16).float(), ref.to(torch.bfloat16).float(),
                               rtol=1.6e-2, atol=1e-2)
    assert ops.device_status() == [0, 0, 0, 0]


@pytest.mark.parametrize("M,N,K", [(1, 16, 32), (3, 127, 128), (5, 40, 64), (64, 256, 512), (33, 48, 96),
                                   (100, 300, 160), (256, 384, 256), (300, 130, 2560), (700, 512, 128)])
def test_tc_gemm_ragged_tiny_and_many_rows(ops, M, N, K):
    """Ragged N and K (zero-padded tiles), one row, and more than 256 rows (row chunks of 256
    inside one launch)."""
    w, x = randw(N, K, 5), randx(M, K, 6)
    part = ops.linear_partials_tc(x.cuda(), w.cuda())
    torch.testing.assert_close(sum_slots(part), O.linear_fp32(x, w), rtol=2e-3, atol=2e-3)
    # the stream-K kernel adds the same products: equal up to fp32 order
    if M <= 64:
        other = ops.linear_partials(x.cuda(), w.cuda()).sum()
        torch.testing.assert_close(part.sum(), other, rtol=1e-3, atol=1e-4)
    assert ops.device_status() == [0, 0, 0, 0]


@pytest.mark.parametrize("M", [9, 32, 64])
def test_consumers_read_tc_partials(ops, M):
    """add+norm on the many-slot partials of a narrow, long-K projection (down: up to 9
    slots), SwiGLU on the [gate | up] partials, logits + argmax on the lm_head shape."""
    w, x = randw(H, I, 21), randx(M, I, 22)
    res = randx(M, H, 23)
    gain = (1 + 0.1 * torch.randn(H, generator=torch.Generator().manual_seed(24))).to(torch.bfloat16)
    part = ops.linear_partials_tc(x.cuda(), w.cuda())
    assert part.plan.slots >= 4
    total, normed = ops.add_rms_norm(res.cuda(), part, gain.cuda(), 1e-6)
    et, en = O.add_rms_norm(res, sum_slots(part), gain, 1e-6)
    assert torch.equal(total.cpu().view(torch.int16), et.view(torch.int16))
    torch.testing.assert_close(normed.cpu().float(), en.float(), rtol=8e-3, atol=1e-6)
    assert bit_equal_fraction(normed.cpu(), en) > 0.99

    wgu, xg = randw(2 * I, H, 31), randx(M, H, 32) * 3
    pg = ops.linear_partials_tc(xg.cuda(), wgu.cuda())
    got = ops.silu_mul(pg).cpu()
    ref = O.swiglu(sum_slots(pg))
    torch.testing.assert_close(got.float(), ref.float(), rtol=8e-3, atol=1e-6)
    assert bit_equal_fraction(got, ref) > 0.99


@pytest.mark.parametrize("M", [257, 600])
def test_consumers_read_many_row_partials(ops, M):
    """More than 256 rows (the prompt pass): one launch over row chunks of 256, the slot count
    of an element depends on its row chunk too. add+norm, SwiGLU and the per-element slot sum
    read such partials."""
    w, x = randw(H, 1024, 41), randx(M, 1024, 42)
    res = randx(M, H, 43)
    gain = (1 + 0.1 * torch.randn(H, generator=torch.Generator().manual_seed(44))).to(torch.bfloat16)
    part = ops.linear_partials_tc(x.cuda(), w.cuda())
    torch.testing.assert_close(sum_slots(part), O.linear_fp32(x, w), rtol=2e-3, atol=2e-3)
    assert torch.equal(part.sum().cpu(), sum_slots(part))
    total, normed = ops.add_rms_norm(res.cuda(), part, gain.cuda(), 1e-6)
    et, en = O.add_rms_norm(res, sum_slots(part), gain, 1e-6)
    assert torch.equal(total.cpu().view(torch.int16), et.view(torch.int16))
    assert bit_equal_fraction(normed.cpu(), en) > 0.99

    wgu, xg = randw(2 * 1216, 512, 45), randx(M, 512, 46) * 3
    pg = ops.linear_partials_tc(xg.cuda(), wgu.cuda())
    got = ops.silu_mul(pg).cpu()
    ref = O.swiglu(sum_slots(pg))
    torch.testing.assert_close(got.float(), ref.float(), rtol=8e-3, atol=1e-6)
    assert bit_equal_fraction(got, ref) > 0.99
    assert ops.device_status() == [0, 0, 0, 0]


def test_tc_gemm_rejects_bad_operands(ops):
    x, w = randx(12, 64, 1).cuda(), randw(16, 64, 2).cuda()
    with pytest.raises(ValueError):
        ops.linear_partials_tc(x.float(), w)
    with pytest.raises(ValueError):
        ops.linear_partials_tc(x, w[:, :32])                 # non-contiguous
    with pytest.raises(ValueError):
        ops.linear_partials_tc(x[:, :48].contiguous(), w[:, :48].contiguous())   # K % 32
    import ctypes as C
    from starter_b200 import _lib
    wt = ops.pack_weight_tc(w)
    out = torch.empty((2, 12, 16), dtype=torch.float32, device="cuda")
    with pytest.raises(ValueError, match="aligned"):       # a weight that is not 1024-byte aligned
        _lib.check(_lib.lib.q_gemm_tc(C.c_void_p(x.data_ptr()), C.c_void_p(wt.data_ptr() + 16),
                                      C.c_void_p(out.data_ptr()), 12, 16, 64, None))
