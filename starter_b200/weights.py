"""Checkpoint loading and weight packing: Hugging Face directory (config.json +
safetensors) -> packed, optionally tensor-parallel-sharded device tensors.

The reference loads through the Transformers model object and packs afterwards
(engine/engine.py:28-47, engine/mlp.py:12-15 gate|up, engine/qk_norm_rope.py:25-30
q|k|v). Here tensors go straight from safetensors to the packed device layout;
no model object is built.

Tensor-parallel shard of rank r of N (Megatron style):
  q heads [r*Nq/N, (r+1)*Nq/N), kv heads [r*Nkv/N, ...): rows of wqkv;
  wo: the matching K columns; gate/up: I/N rows each; down: the matching K
  columns; lm_head: V/N vocabulary rows; norms and the embedding table replicated.
"""
from __future__ import annotations

import ctypes as C
import json
from dataclasses import dataclass, field
from pathlib import Path

import torch

HEAD_DIM = 128


def interleave_gate_up(packed: torch.Tensor) -> torch.Tensor:
    """[gate; up] ([2I, K], engine/mlp.py:12-15) -> rows 16i..16i+7 = gate rows 8i..8i+7,
    rows 16i+8..16i+15 = up rows 8i..8i+7: the row order q_gemm_swiglu wants."""
    two_i, K = packed.shape
    if two_i % 16:
        raise ValueError("the packed gate|up matrix needs a multiple of 16 rows")
    inter = two_i // 2
    gate, up = packed[:inter].view(inter // 8, 8, K), packed[inter:].view(inter // 8, 8, K)
    return torch.stack((gate, up), 1).reshape(two_i, K).contiguous()


def deinterleave_gate_up(mixed: torch.Tensor) -> torch.Tensor:
    """Inverse of interleave_gate_up."""
    two_i, K = mixed.shape
    blocks = mixed.view(two_i // 16, 2, 8, K)
    return torch.cat((blocks[:, 0].reshape(two_i // 2, K), blocks[:, 1].reshape(two_i // 2, K)), 0).contiguous()


class TiledWeight:
    """A bf16 [N, K] Linear weight held in the GEMM's tiled unit layout (see
    q_pack_weight in include/qdecode.h). `data` is a flat uint8 device tensor;
    `rows()` gives the row-major matrix back (used by prefill, which runs on
    library GEMMs outside the per-step path). `interleaved8`: the rows were put in
    q_gemm_swiglu's gate/up order before tiling (rows() undoes it)."""

    def __init__(self, data: torch.Tensor, N: int, K: int, interleaved8: bool = False):
        self.data, self.N, self.K, self.interleaved8 = data, N, K, interleaved8
        self._tc: "TcWeight | None" = None

    def tc(self) -> "TcWeight":
        """The same matrix in the tcgen05 kernel's 128 x 64 tiling (built on first use from
        the row-major form, then kept: a second copy of the weight in HBM). A gate|up matrix
        comes out as plain [gate; up]."""
        if self._tc is None:
            self._tc = TcWeight.pack(self.rows())
        return self._tc

    @property
    def shape(self):
        return (self.N, self.K)

    def numel(self) -> int:
        return self.N * self.K

    def data_ptr(self) -> int:
        return self.data.data_ptr()

    @staticmethod
    def pack(weight: torch.Tensor, interleave8: bool = False) -> "TiledWeight":
        from ._lib import check, lib
        if (weight.ndim != 2 or weight.dtype != torch.bfloat16 or not weight.is_cuda
                or not weight.is_contiguous() or weight.shape[1] % 32):
            raise ValueError("expected a contiguous BF16 CUDA [N, K] weight with K a multiple of 32")
        if interleave8:
            weight = interleave_gate_up(weight)
        N, K = weight.shape
        out = torch.empty(lib.q_packed_weight_bytes(N, K), dtype=torch.uint8, device=weight.device)
        with torch.cuda.device(weight.device):
            check(lib.q_pack_weight(C.c_void_p(weight.data_ptr()), C.c_void_p(out.data_ptr()), N, K,
                                    C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return TiledWeight(out, N, K, interleave8)

    def rows(self, out: torch.Tensor | None = None) -> torch.Tensor:
        from ._lib import check, lib
        if out is None:
            out = torch.empty((self.N, self.K), dtype=torch.bfloat16, device=self.data.device)
        with torch.cuda.device(self.data.device):
            check(lib.q_unpack_weight(C.c_void_p(self.data.data_ptr()), C.c_void_p(out.data_ptr()),
                                      self.N, self.K,
                                      C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        if self.interleaved8:
            out.copy_(deinterleave_gate_up(out))
        return out

    def row_slice(self, lo: int, hi: int) -> "TiledWeight":
        """Rows [lo, hi) as a view (no copy); lo must be a multiple of 16."""
        if lo % 16 or not 0 <= lo < hi <= self.N or self.interleaved8:
            raise ValueError("a tiled row slice must start on a 16-row boundary (and not be gate/up interleaved)")
        unit_bytes = (self.K // 32) * 1024
        groups = (hi - lo + 15) // 16
        return TiledWeight(self.data[(lo // 16) * unit_bytes:(lo // 16 + groups) * unit_bytes], hi - lo, self.K)


class TcWeight:
    """A bf16 [N, K] Linear weight in the tcgen05 GEMM's tiling (q_pack_weight_tc in
    include/qdecode.h): 128-row x 64-k tiles of 16 KB, each the swizzled K-major
    shared-memory image of the tile."""

    def __init__(self, data: torch.Tensor, N: int, K: int):
        self.data, self.N, self.K = data, N, K

    @property
    def shape(self):
        return (self.N, self.K)

    def numel(self) -> int:
        return self.N * self.K

    def data_ptr(self) -> int:
        return self.data.data_ptr()

    @staticmethod
    def pack(weight: torch.Tensor) -> "TcWeight":
        from ._lib import check, lib
        if (weight.ndim != 2 or weight.dtype != torch.bfloat16 or not weight.is_cuda
                or not weight.is_contiguous() or weight.shape[1] % 32):
            raise ValueError("expected a contiguous BF16 CUDA [N, K] weight with K a multiple of 32")
        N, K = weight.shape
        nbytes = lib.q_packed_weight_bytes_tc(N, K)
        # 1024-byte alignment of every tile: over-allocate and slice
        raw = torch.empty(nbytes + 1024, dtype=torch.uint8, device=weight.device)
        off = (-raw.data_ptr()) % 1024
        out = raw[off:off + nbytes]
        with torch.cuda.device(weight.device):
            check(lib.q_pack_weight_tc(C.c_void_p(weight.data_ptr()), C.c_void_p(out.data_ptr()), N, K,
                                       C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return TcWeight(out, N, K)

    def rows(self) -> torch.Tensor:
        from ._lib import check, lib
        out = torch.empty((self.N, self.K), dtype=torch.bfloat16, device=self.data.device)
        with torch.cuda.device(self.data.device):
            check(lib.q_unpack_weight_tc(C.c_void_p(self.data.data_ptr()), C.c_void_p(out.data_ptr()),
                                         self.N, self.K,
                                         C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return out


@dataclass
class ModelConfig:
    vocab: int
    hidden: int
    inter: int
    n_layers: int
    n_q_heads: int
    n_kv_heads: int
    head_dim: int
    rms_eps: float
    rope_theta: float
    tied: bool
    max_position: int

    @staticmethod
    def from_hf(cfg: dict) -> "ModelConfig":
        rope = cfg.get("rope_parameters") or {}
        theta = cfg.get("rope_theta", rope.get("rope_theta", 10000.0))
        rope_type = rope.get("rope_type", "default") if rope else "default"
        scaling = cfg.get("rope_scaling")
        if rope_type != "default" or (scaling and scaling.get("rope_type", "default") != "default"):
            raise ValueError("only default (unscaled) RoPE is supported")
        n_q = cfg["num_attention_heads"]
        head_dim = cfg.get("head_dim") or cfg["hidden_size"] // n_q
        out = ModelConfig(
            vocab=cfg["vocab_size"], hidden=cfg["hidden_size"], inter=cfg["intermediate_size"],
            n_layers=cfg["num_hidden_layers"], n_q_heads=n_q,
            n_kv_heads=cfg.get("num_key_value_heads", n_q), head_dim=head_dim,
            rms_eps=float(cfg.get("rms_norm_eps", 1e-6)), rope_theta=float(theta),
            tied=bool(cfg.get("tie_word_embeddings", False)),
            max_position=int(cfg.get("max_position_embeddings", 40960)),
        )
        out.validate()
        return out

    def validate(self) -> None:
        if self.head_dim != HEAD_DIM:
            raise ValueError(f"head_dim {self.head_dim} is not supported (only {HEAD_DIM})")
        if self.hidden % 32 or self.inter % 32:
            raise ValueError("hidden and intermediate sizes must be multiples of 32")
        if self.n_q_heads % self.n_kv_heads or self.n_q_heads // self.n_kv_heads > 32:
            raise ValueError("unsupported query/kv head grouping")


@dataclass
class LayerTensors:
    wqkv: "torch.Tensor | TiledWeight"
    wo: "torch.Tensor | TiledWeight"
    wgu: "torch.Tensor | TiledWeight"
    wdown: "torch.Tensor | TiledWeight"
    ln_in: torch.Tensor
    ln_post: torch.Tensor
    q_gain: torch.Tensor
    k_gain: torch.Tensor


@dataclass
class PackedWeights:
    cfg: ModelConfig
    tp_rank: int
    tp_size: int
    embed: "torch.Tensor | TiledWeight"     # [V, H] full table (replicated)
    lm_head: "torch.Tensor | TiledWeight"   # [V/N, H] local vocabulary rows (a view of embed when tied)
    ln_final: torch.Tensor
    device: torch.device = None
    layers: list[LayerTensors] = field(default_factory=list)

    @property
    def local_q_heads(self) -> int:
        return self.cfg.n_q_heads // self.tp_size

    @property
    def local_kv_heads(self) -> int:
        return self.cfg.n_kv_heads // self.tp_size

    @property
    def local_inter(self) -> int:
        return self.cfg.inter // self.tp_size

    @property
    def local_vocab(self) -> int:
        return self.lm_head.shape[0]

    def tile(self) -> "PackedWeights":
        """Converts every matrix to the tiled GEMM layout in place (device only)."""
        tied = self.lm_head.data_ptr() == (self.embed.data_ptr() + self.vocab_offset * self.cfg.hidden * 2) \
            if isinstance(self.embed, torch.Tensor) else False
        lo = self.vocab_offset
        rows = self.lm_head.shape[0]
        if isinstance(self.embed, torch.Tensor):
            self.embed = TiledWeight.pack(self.embed)
        if isinstance(self.lm_head, torch.Tensor):
            if tied and lo % 16 == 0:
                self.lm_head = self.embed.row_slice(lo, lo + rows)
            else:
                self.lm_head = TiledWeight.pack(self.lm_head.contiguous())
        for lt in self.layers:
            for name in ("wqkv", "wo", "wgu", "wdown"):
                t = getattr(lt, name)
                if isinstance(t, torch.Tensor):
                    setattr(lt, name, TiledWeight.pack(t, interleave8=(name == "wgu")))
        return self

    @property
    def vocab_offset(self) -> int:
        return self.tp_rank * (self.cfg.vocab // self.tp_size)

    def ensure_tc(self) -> None:
        """Builds the tcgen05 tiling of every matrix (steps with 9 rows and more, the prompt
        pass). Doubles the weight bytes held in HBM."""
        for lt in self.layers:
            for name in ("wqkv", "wo", "wgu", "wdown"):
                getattr(lt, name).tc()
        self.lm_head.tc()

    @property
    def has_tc(self) -> bool:
        return self.lm_head._tc is not None and all(
            getattr(lt, n)._tc is not None for lt in self.layers for n in ("wqkv", "wo", "wgu", "wdown"))


def check_tp(cfg: ModelConfig, tp_size: int) -> None:
    if tp_size < 1:
        raise ValueError("tp_size must be >= 1")
    if cfg.n_kv_heads % tp_size or cfg.n_q_heads % tp_size:
        raise ValueError(f"{cfg.n_kv_heads} kv heads do not split over {tp_size} ranks")
    if (cfg.inter // tp_size) % 32 or cfg.inter % tp_size:
        raise ValueError("intermediate size per rank must be a multiple of 32")
    if cfg.vocab % tp_size:
        raise ValueError("vocabulary does not split evenly over the ranks")


def pack_layer(cfg: ModelConfig, get, layer: int, tp_rank: int, tp_size: int, device) -> LayerTensors:
    """`get(name)` returns the named checkpoint tensor (CPU or device, any float dtype)."""
    p = f"model.layers.{layer}."
    D = HEAD_DIM
    nq, nkv, inter = cfg.n_q_heads // tp_size, cfg.n_kv_heads // tp_size, cfg.inter // tp_size

    def rows(name, lo, hi):
        return get(name)[lo:hi].to(device=device, dtype=torch.bfloat16)

    q = rows(p + "self_attn.q_proj.weight", tp_rank * nq * D, (tp_rank + 1) * nq * D)
    k = rows(p + "self_attn.k_proj.weight", tp_rank * nkv * D, (tp_rank + 1) * nkv * D)
    v = rows(p + "self_attn.v_proj.weight", tp_rank * nkv * D, (tp_rank + 1) * nkv * D)
    wqkv = torch.cat((q, k, v), 0).contiguous()
    wo = get(p + "self_attn.o_proj.weight")[:, tp_rank * nq * D:(tp_rank + 1) * nq * D]
    wo = wo.to(device=device, dtype=torch.bfloat16).contiguous()
    gate = rows(p + "mlp.gate_proj.weight", tp_rank * inter, (tp_rank + 1) * inter)
    up = rows(p + "mlp.up_proj.weight", tp_rank * inter, (tp_rank + 1) * inter)
    wgu = torch.cat((gate, up), 0).contiguous()
    wdown = get(p + "mlp.down_proj.weight")[:, tp_rank * inter:(tp_rank + 1) * inter]
    wdown = wdown.to(device=device, dtype=torch.bfloat16).contiguous()

    def vec(name):
        return get(p + name).to(device=device, dtype=torch.bfloat16).contiguous()

    return LayerTensors(wqkv, wo, wgu, wdown, vec("input_layernorm.weight"),
                        vec("post_attention_layernorm.weight"), vec("self_attn.q_norm.weight"),
                        vec("self_attn.k_norm.weight"))


def pack(cfg: ModelConfig, get, has, device, tp_rank: int = 0, tp_size: int = 1) -> PackedWeights:
    check_tp(cfg, tp_size)
    embed = get("model.embed_tokens.weight").to(device=device, dtype=torch.bfloat16).contiguous()
    vshard = cfg.vocab // tp_size
    lo, hi = tp_rank * vshard, (tp_rank + 1) * vshard
    if has("lm_head.weight") and not cfg.tied:
        lm_head = get("lm_head.weight")[lo:hi].to(device=device, dtype=torch.bfloat16).contiguous()
    else:
        lm_head = embed[lo:hi]          # tied: a row view of the table, no second copy
    out = PackedWeights(cfg, tp_rank, tp_size, embed, lm_head,
                        get("model.norm.weight").to(device=device, dtype=torch.bfloat16).contiguous(),
                        device=torch.device(device))
    for i in range(cfg.n_layers):
        out.layers.append(pack_layer(cfg, get, i, tp_rank, tp_size, device))
        if out.device.type == "cuda":
            lt = out.layers[-1]          # tile as we go so that only one layer is held twice
            for name in ("wqkv", "wo", "wgu", "wdown"):
                setattr(lt, name, TiledWeight.pack(getattr(lt, name), interleave8=(name == "wgu")))
    if out.device.type == "cuda":
        out.tile()
    return out


def load_checkpoint(model_path: str, device, tp_rank: int = 0, tp_size: int = 1) -> PackedWeights:
    """Reads config.json and every *.safetensors file under model_path."""
    from safetensors import safe_open

    root = Path(model_path)
    cfg = ModelConfig.from_hf(json.loads((root / "config.json").read_text()))
    files = sorted(root.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no safetensors files under {root}")
    index: dict[str, Path] = {}
    handles = {}
    for f in files:
        h = safe_open(str(f), framework="pt", device="cpu")
        handles[f] = h
        for name in h.keys():
            index[name] = f

    def get(name):
        return handles[index[name]].get_tensor(name)

    return pack(cfg, get, lambda n: n in index, device, tp_rank, tp_size)


def rotary_tables(cfg: ModelConfig, capacity: int, device):
    """BF16 cos/sin [capacity, 128]: fp32 angle = position * inv_freq, fp32 cos/sin,
    one cast (the same arithmetic as the native rotary module, which the reference
    tabulates in engine/decode.py:52-59). Computed on the CPU so that the rows
    equal the CPU oracle's bit for bit."""
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, HEAD_DIM, 2, dtype=torch.int64).float() / HEAD_DIM))
    ang = torch.arange(capacity, dtype=torch.float32)[:, None] * inv[None, :]
    emb = torch.cat((ang, ang), -1)
    return (emb.cos().to(torch.bfloat16).to(device).contiguous(),
            emb.sin().to(torch.bfloat16).to(device).contiguous())
