"""CPU checks of the C-ABI boundary: the library builds, loads, and exports every
symbol include/qdecode.h declares; launch plans cover every unit exactly once;
argument errors surface as ValueError before any launch. No compute calls here."""
import ctypes as C
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    text = (ROOT / "include" / "qdecode.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(q_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    from starter_b200 import _lib
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(_lib.lib, n), f"libqdecode.so lacks {n}"
        assert n in _lib.SIGNATURES, f"binding lacks {n}"
    assert set(_lib.SIGNATURES) == set(names)
    assert _lib.lib.q_version() >= 100


@pytest.mark.parametrize("M,N,K", [(1, 6144, 2560), (32, 2560, 4096), (8, 19456, 2560),
                                   (16, 2560, 9728), (4, 151936, 2560), (3, 127, 128), (1, 16, 32)])
def test_plan_covers_every_unit_once(M, N, K):
    """Every (16-row group, 32-k chunk) unit belongs to exactly one worker, each
    worker's slot index inside a group is below `slots`, and the slot counts the
    consumers derive match (reference tests pin 'every partial written exactly
    once' the same way, tests/test_skinny_gemm.py:150)."""
    from starter_b200 import _lib
    p = _lib.plan(M, N, K)
    Cg, u = p.chunks_per_group, p.units_per_worker
    total = p.groups * Cg
    assert p.groups == (N + 15) // 16 and Cg == K // 32 and p.group_rows == 16
    assert p.workers == (total + u - 1) // u
    assert p.workers <= p.grid * (p.block // 32)
    covered = 0
    max_slot = 0
    for w in range(p.workers):
        start, end = w * u, min(total, (w + 1) * u)
        covered += end - start
        g0, g1 = start // Cg, (end - 1) // Cg
        for g in (g0, g1):
            first = (g * Cg) // u
            last = ((g + 1) * Cg - 1) // u
            assert first <= w <= last
            max_slot = max(max_slot, last - first + 1)
    assert covered == total
    assert max_slot <= p.slots


def test_argument_errors_are_value_errors():
    from starter_b200 import _lib
    with pytest.raises(ValueError):
        _lib.plan(0, 128, 128)
    with pytest.raises(ValueError):
        _lib.plan(65, 128, 128)
    with pytest.raises(ValueError):
        _lib.plan(1, 128, 100)          # K not a multiple of 32
    with pytest.raises(ValueError):
        _lib.check(_lib.lib.q_gemm_splitk(None, None, None, 1, 16, 32, None))
    cfg = _lib.Config(100, 256, 2, 4, 2, 127, 0, 127, 1, 1, 1e-6, 0.088)   # hidden % 32 != 0
    h = C.c_void_p()
    with pytest.raises(ValueError):
        _lib.check(_lib.lib.q_create(C.byref(cfg), C.byref(h)))


def test_engine_state_errors():
    from starter_b200 import _lib
    cfg = _lib.Config(128, 256, 2, 4, 2, 127, 0, 127, 1, 4, 1e-6, 0.088)
    h = C.c_void_p()
    _lib.check(_lib.lib.q_create(C.byref(cfg), C.byref(h)))
    try:
        with pytest.raises(_lib.QDecodeError):           # nothing bound yet
            _lib.check(_lib.lib.q_decode_step(h, None))
        with pytest.raises(ValueError):
            _lib.check(_lib.lib.q_bind_layer(h, 5, C.byref(_lib.LayerWeights())))
        assert _lib.lib.q_engine_partial_floats(h, 4) > 0
    finally:
        _lib.lib.q_destroy(h)


def test_engine_refuses_to_run_without_cuda(golden_dir):
    import torch
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    from starter_b200 import Engine
    with pytest.raises(RuntimeError):
        Engine(str(golden_dir / "tiny_qwen3"))


def test_config_and_tp_shard_shapes(golden_dir):
    """Host-side weight packing: packed shapes and tensor-parallel shards."""
    import torch
    from starter_b200 import weights as W
    full = W.load_checkpoint(str(golden_dir / "tiny_qwen3"), "cpu")
    cfg = full.cfg
    assert (cfg.hidden, cfg.inter, cfg.n_q_heads, cfg.n_kv_heads, cfg.vocab) == (128, 256, 4, 2, 127)
    assert cfg.rope_theta == 1_000_000.0 and cfg.tied
    assert full.layers[0].wqkv.shape == (8 * 128, 128)
    assert full.layers[0].wgu.shape == (512, 128)
    assert full.lm_head.data_ptr() == full.embed.data_ptr()     # tied: no second copy
    with pytest.raises(ValueError):
        W.check_tp(cfg, 4)                                      # 2 kv heads over 4 ranks
    # vocab 127 does not split over 2 ranks: use a 2-way split on a padded copy of the config
    cfg2 = W.ModelConfig(**{**cfg.__dict__, "vocab": 126})
    sd = {}
    from safetensors.torch import load_file
    sd = load_file(str(golden_dir / "tiny_qwen3" / "model.safetensors"))
    sd["model.embed_tokens.weight"] = sd["model.embed_tokens.weight"][:126]
    shards = [W.pack(cfg2, sd.__getitem__, sd.__contains__, "cpu", r, 2) for r in range(2)]
    one = W.pack(cfg2, sd.__getitem__, sd.__contains__, "cpu", 0, 1)
    D = 128
    q = torch.cat([s.layers[0].wqkv[:2 * D] for s in shards])
    assert torch.equal(q, one.layers[0].wqkv[:4 * D])
    assert torch.equal(torch.cat([s.layers[1].wo for s in shards], 1), one.layers[1].wo)
    assert torch.equal(torch.cat([s.layers[1].wdown for s in shards], 1), one.layers[1].wdown)
    gate = torch.cat([s.layers[0].wgu[:128] for s in shards])
    assert torch.equal(gate, one.layers[0].wgu[:256])
    assert torch.equal(torch.cat([s.lm_head for s in shards]), one.lm_head)
    assert [s.vocab_offset for s in shards] == [0, 63]


def test_gate_up_interleave_is_a_row_permutation():
    """q_gemm_swiglu's weight order: tiled rows 16i..16i+7 = gate rows 8i..8i+7 and rows
    16i+8..16i+15 = the matching up rows (engine/mlp.py:12-15 packs [gate; up])."""
    from starter_b200.weights import deinterleave_gate_up, interleave_gate_up
    inter, K = 40, 32
    packed = torch.arange(2 * inter * K, dtype=torch.float32).view(2 * inter, K).to(torch.bfloat16)
    mixed = interleave_gate_up(packed)
    assert mixed.shape == packed.shape
    for i in range(inter // 8):
        assert torch.equal(mixed[16 * i:16 * i + 8], packed[8 * i:8 * i + 8])                     # gate
        assert torch.equal(mixed[16 * i + 8:16 * i + 16], packed[inter + 8 * i:inter + 8 * i + 8])  # up
    assert torch.equal(deinterleave_gate_up(mixed), packed)
    with pytest.raises(ValueError):
        interleave_gate_up(packed[:-2])


def test_peer_entry_points_reject_bad_arguments():
    """No GPU needed: the argument checks of the tensor-parallel peer path run on the host."""
    from starter_b200 import _lib
    lib = _lib.lib
    peers = _lib.Peers()
    peers.rank, peers.world = 0, 1                        # a world of one is not tensor parallel
    A = 4096                                              # a made-up, aligned address: nothing is launched
    assert lib.q_add_rmsnorm_peers(A, C.byref(peers), A, None, A, A, A, 1, 128, 1e-6, None) == -1
    assert b"world" in lib.q_last_error() or b"rank" in lib.q_last_error()
    assert lib.q_bind_peers(None, C.byref(peers)) == -1
    assert lib.q_gemm_swiglu(A, A, A, 1, 12, 64, None) == -1      # inter must be a multiple of 8
    assert lib.q_gemm_swiglu_addnorm(A, A, None, A, A, A, A, 1, 64, 64, 1e-6, None) == -1   # in place
    assert lib.q_argmax_merge_peers(A, A, C.byref(peers), 1, A, A, 1, None) == -1
    assert lib.q_peer_flag_bytes() >= 512 + 2 * 8 * 64 * 8


def test_misaligned_pointers_are_argument_errors():
    """Kernels that load or store 8 / 16 bytes at a time refuse pointers that would fault on the
    device: the check runs on the host, before any launch."""
    from starter_b200 import _lib
    lib = _lib.lib
    A = 4096
    p = _lib.plan(2, 64, 64)
    cases = [
        lib.q_gemm_splitk(A + 2, A, A, 2, 64, 64, None),
        lib.q_gemm_tc(A, A + 512, A, 12, 64, 64, None),
        lib.q_reduce_partials(A + 4, C.byref(p), A, None),
        lib.q_reduce_partials(A, C.byref(p), A + 8, None),
        lib.q_linear_f32_static(A, A, A + 4, 2, 64, 64, None),
        lib.q_add_rmsnorm(A + 2, A, None, A, A, A, 2, 64, 1e-6, None),
        lib.q_add_rmsnorm(A, A + 4, None, A, A, A, 2, 64, 1e-6, None),
        lib.q_swiglu(A + 8, C.byref(_lib.plan(2, 128, 64)), A, 2, 64, None),
        lib.q_logits_argmax(A + 4, C.byref(p), None, A, A, None, None, 0, A, 2, 64, 0, None),
        lib.q_gemm_splitk_addnorm(A, A + 4, None, A, A + 64, A, A, 2, 64, 64, 1e-6, None),
    ]
    assert cases == [-1] * len(cases), cases
    assert b"aligned" in lib.q_last_error()


@pytest.mark.parametrize("M,N,K", [(32, 19456, 2560), (64, 2560, 9728), (9, 6144, 2560), (16, 151936, 2560),
                                   (12, 127, 128), (300, 48, 96), (1, 16, 32), (2048, 2560, 9728)])
def test_tc_plan_covers_every_tile_once(M, N, K):
    """The tcgen05 kernel's stream-K split: every (row chunk of 256, 128-row block, 64-k tile)
    belongs to exactly one CTA, and the slot a CTA writes for a block is below `slots`."""
    from starter_b200 import _lib
    p = _lib.plan(M, N, K, tc=True)
    KT, u = p.chunks_per_group, p.units_per_worker
    blocks, row_chunks = (N + 127) // 128, (M + 255) // 256
    assert p.group_rows == 128 and p.groups == blocks * row_chunks and KT == (K + 63) // 64
    total = p.groups * KT
    assert p.workers == (total + u - 1) // u == p.grid
    covered, max_slot = 0, 0
    for w in range(p.workers):
        start, end = w * u, min(total, (w + 1) * u)
        covered += end - start
        for g in range(start // KT, (end - 1) // KT + 1):
            first, last = (g * KT) // u, ((g + 1) * KT - 1) // u
            assert first <= w <= last
            max_slot = max(max_slot, last - first + 1)
    assert covered == total and max_slot <= p.slots
    assert _lib.lib.q_packed_weight_bytes_tc(N, K) == blocks * KT * 16384
