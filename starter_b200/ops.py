"""Operator-level wrappers: torch tensors in, torch tensors out, every call going
through the C ABI of libqdecode.so.

Names, argument meaning, ownership and error behaviour mirror the reference's
operator functions (engine/kernels/skinny_gemm.py:100-121,
engine/kernels/decode_fused.py:140-210, engine/kernels/rmsnorm.py:39-62,
engine/kernels/small_query_attention.py:113-158): inputs are read-only, outputs
are freshly allocated, every shape/dtype/device/contiguity violation raises
ValueError before anything is launched, and there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import HEAD_DIM, MAX_ROWS, PAGE_TOKENS, GemmPlan, KVLayout, check, lib
from .weights import TiledWeight


def pack_weight(weight: torch.Tensor) -> TiledWeight:
    """Tiles a row-major BF16 [N, K] Linear weight once (load time), like the
    reference packs gate|up and q|k|v at load (engine/mlp.py:12-15)."""
    return TiledWeight.pack(weight)


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _bf16_2d(x: torch.Tensor, what: str) -> tuple[int, int]:
    if x.ndim != 2 or not x.is_cuda or x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError(f"{what}: expected a contiguous 2-D BF16 CUDA tensor")
    return x.shape[0], x.shape[1]


@dataclass
class Partials:
    """FP32 split-K partial sums of one projection plus the plan that says which
    slots hold data for which column (see q_gemm_plan in include/qdecode.h)."""
    data: torch.Tensor          # [slots, M, N] float32
    plan: GemmPlan

    @property
    def shape(self):
        return (self.plan.M, self.plan.N)

    def sum(self) -> torch.Tensor:
        """FP32 [M, N] sum of the slots (device reduction, no rounding)."""
        out = torch.empty(self.shape, dtype=torch.float32, device=self.data.device)
        check(lib.q_reduce_partials(_ptr(self.data), C.byref(self.plan), _ptr(out), _stream()))
        return out


def supports(x: torch.Tensor, weight) -> bool:
    """Static shape rule, like engine/kernels/skinny_gemm.py:75-83."""
    return (x.ndim == 2 and len(weight.shape) == 2 and x.is_cuda
            and x.dtype == torch.bfloat16 and 1 <= x.shape[0] <= MAX_ROWS
            and x.shape[1] == weight.shape[1] and x.shape[1] % 32 == 0)


def linear_partials(x: torch.Tensor, weight) -> Partials:
    """x @ weight.T as FP32 split-K partials (engine/kernels/skinny_gemm.py:100-109).
    `weight` is a TiledWeight (see pack_weight) or a row-major BF16 [N, K] tensor,
    which is tiled on the fly (load-time work done per call: for tests only)."""
    M, K = _bf16_2d(x, "x")
    if not isinstance(weight, TiledWeight):
        _bf16_2d(weight, "weight")
        if weight.shape[1] % 32:
            raise ValueError("K must be a multiple of 32")
        weight = TiledWeight.pack(weight)
    N, K2 = weight.shape
    if K != K2 or x.device != weight.data.device:
        raise ValueError("x and weight disagree on K or device")
    if not 1 <= M <= MAX_ROWS:
        raise ValueError(f"at most {MAX_ROWS} rows are supported, got {M}")
    p = _lib.plan(M, N, K)
    data = torch.empty((p.slots, M, N), dtype=torch.float32, device=x.device)
    check(lib.q_gemm_splitk(_ptr(x), _ptr(weight), _ptr(data), M, N, K, _stream()))
    return Partials(data, p)


def _branch(branch, rows: int, cols: int, device):
    """(pointer, plan-pointer) for a Partials or a plain FP32 [rows, cols] tensor."""
    if isinstance(branch, Partials):
        if branch.shape != (rows, cols) or branch.data.device != device:
            raise ValueError("split-K partials disagree with the operand shape or device")
        return _ptr(branch.data), C.byref(branch.plan)
    if (not isinstance(branch, torch.Tensor) or branch.dtype != torch.float32
            or tuple(branch.shape) != (rows, cols) or branch.device != device
            or not branch.is_contiguous()):
        raise ValueError("branch must be Partials or a contiguous FP32 [rows, cols] CUDA tensor")
    return _ptr(branch), None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm with the rounding before the gain (engine/kernels/rmsnorm.py:39-62)."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or not x.is_contiguous() or x.ndim < 1:
        raise ValueError("expected a contiguous BF16 CUDA tensor")
    cols = x.shape[-1]
    if weight.shape != (cols,) or weight.dtype != torch.bfloat16 or weight.device != x.device:
        raise ValueError("gain must be BF16 [cols] on the same device")
    out = torch.empty_like(x)
    rows = x.numel() // cols
    if rows:
        check(lib.q_rmsnorm(_ptr(x), _ptr(weight), _ptr(out), rows, cols, float(eps), _stream()))
    return out


def add_rms_norm(residual: torch.Tensor, branch, weight: torch.Tensor, eps: float):
    """(residual + branch, RMSNorm of that sum) as fresh BF16 tensors
    (engine/kernels/decode_fused.py:140-158)."""
    rows, cols = _bf16_2d(residual, "residual")
    if weight.shape != (cols,) or weight.dtype != torch.bfloat16 or weight.device != residual.device:
        raise ValueError("residual and gain shapes disagree")
    bp, pp = _branch(branch, rows, cols, residual.device)
    total, normed = torch.empty_like(residual), torch.empty_like(residual)
    check(lib.q_add_rmsnorm(_ptr(residual), bp, pp, _ptr(weight), _ptr(total), _ptr(normed),
                            rows, cols, float(eps), _stream()))
    return total, normed


def add_rms_norm_linear(residual: torch.Tensor, branch, gain: torch.Tensor, eps: float, weight):
    """(residual + branch, RMSNorm(that sum) @ weight.T as split-K partials): add_rms_norm
    (engine/kernels/decode_fused.py:140-158) run as the prologue of the projection that
    consumes it (engine/decode_step.py:50-59), one launch. Up to 8 rows, K <= 3072."""
    rows, cols = _bf16_2d(residual, "residual")
    if gain.shape != (cols,) or gain.dtype != torch.bfloat16 or gain.device != residual.device:
        raise ValueError("residual and gain shapes disagree")
    if not isinstance(weight, TiledWeight):
        _bf16_2d(weight, "weight")
        weight = TiledWeight.pack(weight)
    N, K = weight.shape
    if K != cols or weight.data.device != residual.device:
        raise ValueError("residual and weight disagree on K or device")
    bp, pp = _branch(branch, rows, cols, residual.device)
    total = torch.empty_like(residual)
    p = _lib.plan(rows, N, K)
    data = torch.empty((p.slots, rows, N), dtype=torch.float32, device=residual.device)
    check(lib.q_gemm_splitk_addnorm(_ptr(residual), bp, pp, _ptr(gain), _ptr(total), _ptr(weight),
                                    _ptr(data), rows, N, K, float(eps), _stream()))
    return total, Partials(data, p)


def silu_mul(gate_up, rows: int | None = None) -> torch.Tensor:
    """silu(gate) * up for the packed [rows, 2*I] projection given as partials
    (engine/kernels/decode_fused.py:161-169 on the GEMM's FP32 partials)."""
    if not isinstance(gate_up, Partials):
        raise ValueError("silu_mul consumes split-K Partials of the packed gate|up projection")
    M, width = gate_up.shape
    if width % 2:
        raise ValueError("packed gate/up width must be even")
    out = torch.empty((M, width // 2), dtype=torch.bfloat16, device=gate_up.data.device)
    check(lib.q_swiglu(_ptr(gate_up.data), C.byref(gate_up.plan), _ptr(out), M, width // 2, _stream()))
    return out


def _gate_up_operand(gate_up_weight):
    """The packed [2I, K] gate|up weight in q_gemm_swiglu's interleaved tiled layout, or None
    when its shape rules it out (I not a multiple of 8)."""
    if isinstance(gate_up_weight, TiledWeight):
        return gate_up_weight if gate_up_weight.interleaved8 else None
    _bf16_2d(gate_up_weight, "weight")
    if gate_up_weight.shape[0] % 16 or gate_up_weight.shape[1] % 32:
        return None
    return TiledWeight.pack(gate_up_weight, interleave8=True)


def linear_silu_mul(x: torch.Tensor, gate_up_weight) -> torch.Tensor:
    """BF16 [M, I] = silu(x @ gate.T) * (x @ up.T) for a packed [2I, K] weight
    (engine/kernels/skinny_gemm.py:112-121). One launch (SwiGLU in the projection's
    epilogue) when I is a multiple of 8; `gate_up_weight` is the row-major [gate; up] matrix
    (tiled on the fly: load-time work, for tests) or a TiledWeight packed with
    interleave8=True. Other shapes take the partials + silu_mul route."""
    if len(gate_up_weight.shape) != 2 or gate_up_weight.shape[0] % 2:
        raise ValueError("packed gate/up weight must have an even number of rows")
    M, K = _bf16_2d(x, "x")
    w = _gate_up_operand(gate_up_weight)
    if w is None:
        return silu_mul(linear_partials(x, gate_up_weight))
    if w.shape[1] != K or w.data.device != x.device:
        raise ValueError("x and weight disagree on K or device")
    if not 1 <= M <= MAX_ROWS:
        raise ValueError(f"at most {MAX_ROWS} rows are supported, got {M}")
    inter = w.shape[0] // 2
    out = torch.empty((M, inter), dtype=torch.bfloat16, device=x.device)
    check(lib.q_gemm_swiglu(_ptr(x), _ptr(w), _ptr(out), M, inter, K, _stream()))
    return out


def add_rms_norm_linear_silu_mul(residual: torch.Tensor, branch, gain: torch.Tensor, eps: float,
                                 gate_up_weight):
    """(residual + branch, silu(n @ gate.T) * (n @ up.T)) with n = RMSNorm(residual + branch):
    the post-attention half of a layer up to the SwiGLU (engine/decode_step.py:50-56) in one
    launch. Up to 8 rows, K <= 3072, I a multiple of 8."""
    rows, cols = _bf16_2d(residual, "residual")
    if gain.shape != (cols,) or gain.dtype != torch.bfloat16 or gain.device != residual.device:
        raise ValueError("residual and gain shapes disagree")
    w = _gate_up_operand(gate_up_weight)
    if w is None or w.shape[1] != cols or w.data.device != residual.device:
        raise ValueError("gate|up weight must be [2I, K] with I a multiple of 8 on the same device")
    bp, pp = _branch(branch, rows, cols, residual.device)
    inter = w.shape[0] // 2
    total = torch.empty_like(residual)
    out = torch.empty((rows, inter), dtype=torch.bfloat16, device=residual.device)
    check(lib.q_gemm_swiglu_addnorm(_ptr(residual), bp, pp, _ptr(gain), _ptr(total), _ptr(w), _ptr(out),
                                    rows, inter, cols, float(eps), _stream()))
    return total, out


class PagedKV:
    """One layer's paged KV pool plus the block table shared by all layers.

    pool[page][kv_head][64][128] bf16 with 16-byte chunks XOR-swizzled by
    (token & 7). The reference keeps a contiguous [B, Hkv, capacity, D] cache
    (engine/decode.py:41-48); `scatter`/`gather` convert from and to that layout.
    """

    def __init__(self, batch: int, n_kv_heads: int, capacity: int, device,
                 block_table: torch.Tensor | None = None, poison: float | None = None):
        if min(batch, n_kv_heads, capacity) < 1:
            raise ValueError("positive batch, head count and capacity required")
        self.batch, self.n_kv, self.capacity = batch, n_kv_heads, capacity
        self.pages_per_seq = (capacity + PAGE_TOKENS - 1) // PAGE_TOKENS
        n_pages = batch * self.pages_per_seq
        shape = (n_pages, n_kv_heads, PAGE_TOKENS, HEAD_DIM)
        self.k = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.v = torch.zeros(shape, dtype=torch.bfloat16, device=device)
        if poison is not None:
            self.k.fill_(poison)
            self.v.fill_(poison)
        if block_table is None:
            block_table = torch.arange(n_pages, dtype=torch.int32, device=device).view(batch, -1)
        if (block_table.shape != (batch, self.pages_per_seq) or block_table.dtype != torch.int32
                or not block_table.is_contiguous()):
            raise ValueError("block table must be contiguous int32 [batch, pages_per_seq]")
        self.block_table = block_table
        self.layout = KVLayout(self.k.data_ptr(), self.v.data_ptr(), block_table.data_ptr(),
                               self.pages_per_seq, n_kv_heads)

    def scatter(self, keys: torch.Tensor, values: torch.Tensor, start: int = 0) -> None:
        """Writes rotated K and V rows [B, Hkv, len, 128] at positions start.."""
        if (keys.shape != values.shape or keys.ndim != 4 or keys.shape[0] != self.batch
                or keys.shape[1] != self.n_kv or keys.shape[3] != HEAD_DIM
                or keys.dtype != torch.bfloat16 or values.dtype != torch.bfloat16
                or not keys.is_cuda or not values.is_cuda):
            raise ValueError("K/V must be BF16 CUDA [batch, Hkv, len, 128]")
        length = keys.shape[2]
        if start < 0 or start + length > self.capacity:
            raise ValueError("positions exceed the cache capacity")
        if length == 0:
            return
        keys, values = keys.contiguous(), values.contiguous()
        check(lib.q_kv_scatter(_ptr(keys), _ptr(values), C.byref(self.layout), self.batch, length,
                               start, _stream()))

    def gather(self, length: int):
        """Contiguous (K, V) [B, Hkv, length, 128] read back from the pages (test helper)."""
        def one(pool):
            p = pool[self.block_table.long()]                    # [B, pages, Hkv, 64, 128]
            r = torch.arange(PAGE_TOKENS, device=pool.device)
            c = torch.arange(16, device=pool.device)
            src = (c[None, :] ^ (r[:, None] & 7))                # physical chunk of logical chunk c
            p = p.view(*p.shape[:4], 16, 8)
            idx = src.view(1, 1, 1, PAGE_TOKENS, 16, 1).expand(*p.shape[:3], PAGE_TOKENS, 16, 8)
            p = torch.gather(p, 4, idx).reshape(*p.shape[:4], HEAD_DIM)
            p = p.permute(0, 2, 1, 3, 4).reshape(self.batch, self.n_kv, -1, HEAD_DIM)
            return p[:, :, :length].contiguous()
        return one(self.k), one(self.v)


def qkv_norm_rope_cache(qkv, q_weight, k_weight, q_eps, k_eps, cos, sin, position,
                        cache: PagedKV, tokens_per_seq: int = 1) -> torch.Tensor:
    """Head norm + RoPE on the packed projection, K/V rows written into their
    page slot (engine/kernels/decode_fused.py:172-210). `position` is an int32
    device scalar tensor [1]; row b*T+t sits at position+t. Returns fresh Q
    [batch*T, Nq, 128]."""
    if not isinstance(qkv, Partials):
        raise ValueError("qkv must be split-K Partials of the packed projection")
    if q_eps != k_eps:
        raise ValueError("q and k norms must share one epsilon")
    rows, width = qkv.shape
    T = tokens_per_seq
    if T < 1 or rows % T or rows // T != cache.batch:
        raise ValueError("rows must be batch * tokens_per_seq")
    n_q = width // HEAD_DIM - 2 * cache.n_kv
    if n_q < 1 or width != (n_q + 2 * cache.n_kv) * HEAD_DIM:
        raise ValueError("unsupported packed Q/K/V width")
    for t in (q_weight, k_weight):
        if t.shape != (HEAD_DIM,) or t.dtype != torch.bfloat16 or not t.is_cuda:
            raise ValueError("head gains must be BF16 [128] CUDA tensors")
    if (cos.shape != sin.shape or cos.ndim != 2 or cos.shape[1] != HEAD_DIM
            or cos.shape[0] < cache.capacity or cos.dtype != torch.bfloat16
            or sin.dtype != torch.bfloat16 or not cos.is_contiguous() or not sin.is_contiguous()):
        raise ValueError("cos/sin must be contiguous BF16 [>=capacity, 128] tables")
    if position.shape != (1,) or position.dtype != torch.int32 or not position.is_cuda:
        raise ValueError("position must be an int32 CUDA tensor of shape [1]")
    q = torch.empty((rows, n_q, HEAD_DIM), dtype=torch.bfloat16, device=qkv.data.device)
    check(lib.q_qkv_norm_rope_cache(_ptr(qkv.data), C.byref(qkv.plan), _ptr(q_weight), _ptr(k_weight),
                                    _ptr(cos), _ptr(sin), _ptr(position), _ptr(q),
                                    C.byref(cache.layout), cache.batch, T, n_q, float(q_eps), _stream()))
    return q


class SmallQueryAttention:
    """Fixed-shape, read-only GQA attention over a paged cache for 1..32/G query
    tokens per sequence (engine/kernels/small_query_attention.py:113-158 for T=1).

    Row (b, t, head) attends to keys [0, position + t + 1). Scratch belongs to the
    instance: calls must be ordered on one stream."""

    def __init__(self, batch, query_heads, kv_heads, capacity, device, tokens_per_seq=1):
        device = torch.device(device)
        if (device.type != "cuda" or min(batch, query_heads, kv_heads, capacity, tokens_per_seq) < 1
                or query_heads % kv_heads or tokens_per_seq * (query_heads // kv_heads) > 32):
            raise ValueError("unsupported small-query attention metadata")
        self.batch, self.hq, self.hk, self.capacity = batch, query_heads, kv_heads, capacity
        self.T = tokens_per_seq
        self.groups = query_heads // kv_heads
        self.splits = lib.q_attention_splits(batch, kv_heads, capacity)
        rows = self.T * self.groups
        self.partials = torch.empty((batch * kv_heads, self.splits, rows, HEAD_DIM),
                                    dtype=torch.float32, device=device)
        self.stats = torch.empty((batch * kv_heads, self.splits, rows, 2),
                                 dtype=torch.float32, device=device)

    def run(self, query, cache: PagedKV, position, scale) -> torch.Tensor:
        if (query.shape != (self.batch * self.T, self.hq, HEAD_DIM) or query.dtype != torch.bfloat16
                or not query.is_cuda or not query.is_contiguous()):
            raise ValueError("expected contiguous BF16 CUDA Q [batch*T, Hq, 128]")
        if cache.batch != self.batch or cache.n_kv != self.hk or cache.capacity < self.capacity:
            raise ValueError("cache does not match this attention instance")
        if position.shape != (1,) or position.dtype != torch.int32 or not position.is_cuda:
            raise ValueError("position must be an int32 CUDA tensor of shape [1]")
        out = torch.empty((self.batch * self.T, self.hq * HEAD_DIM), dtype=torch.bfloat16,
                          device=query.device)
        check(lib.q_attention(_ptr(query), C.byref(cache.layout), _ptr(position), _ptr(self.partials),
                              _ptr(self.stats), _ptr(out), self.batch, self.T, self.hq, self.splits,
                              float(scale), _stream()))
        return out


def prompt_attention(query: torch.Tensor, cache: PagedKV, position: torch.Tensor, tokens_per_seq: int,
                     scale: float) -> torch.Tensor:
    """Causal GQA attention of a block of `tokens_per_seq` prompt tokens per sequence over the
    paged cache, which must already hold their keys and values (the prompt pass; the reference
    calls the library's scaled-dot-product attention at engine/prefill.py:45-52). query is
    [batch*T, Hq, 128]; row (b, t, head) attends to keys [0, position + t + 1). Returns
    [batch*T, Hq*128]."""
    T = int(tokens_per_seq)
    if (query.dim() != 3 or query.shape[0] != cache.batch * T or query.shape[2] != HEAD_DIM
            or query.dtype != torch.bfloat16 or not query.is_cuda or not query.is_contiguous()):
        raise ValueError("expected contiguous BF16 CUDA Q [batch*T, Hq, 128]")
    if position.shape != (1,) or position.dtype != torch.int32 or not position.is_cuda:
        raise ValueError("position must be an int32 CUDA tensor of shape [1]")
    hq = query.shape[1]
    out = torch.empty((cache.batch * T, hq * HEAD_DIM), dtype=torch.bfloat16, device=query.device)
    check(lib.q_attention_prefill(_ptr(query), C.byref(cache.layout), _ptr(position), _ptr(out), cache.batch,
                                  T, hq, float(scale), _stream()))
    return out


def decode_attention(qkv, q_weight, k_weight, eps, cos, sin, position, cache: PagedKV,
                     attn: SmallQueryAttention, scale) -> torch.Tensor:
    """qkv_norm_rope_cache + SmallQueryAttention.run for one token per sequence in a single
    launch (engine/decode_step.py:43-48 does the two calls back to back). Returns the
    attended rows [batch, Hq*128]; the K/V rows of `position` are written to the pages."""
    if not isinstance(qkv, Partials):
        raise ValueError("qkv must be split-K Partials of the packed projection")
    rows, width = qkv.shape
    if attn.T != 1 or rows != cache.batch or attn.batch != cache.batch or attn.hk != cache.n_kv:
        raise ValueError("decode_attention handles one token per sequence")
    if width != (attn.hq + 2 * attn.hk) * HEAD_DIM:
        raise ValueError("unsupported packed Q/K/V width")
    if position.shape != (1,) or position.dtype != torch.int32 or not position.is_cuda:
        raise ValueError("position must be an int32 CUDA tensor of shape [1]")
    if not hasattr(attn, "tickets"):
        attn.tickets = torch.zeros(attn.batch * attn.hk, dtype=torch.int32, device=qkv.data.device)
    out = torch.empty((rows, attn.hq * HEAD_DIM), dtype=torch.bfloat16, device=qkv.data.device)
    check(lib.q_attention_decode(_ptr(qkv.data), C.byref(qkv.plan), _ptr(q_weight), _ptr(k_weight),
                                 _ptr(cos), _ptr(sin), _ptr(position), C.byref(cache.layout),
                                 _ptr(attn.partials), _ptr(attn.stats), _ptr(attn.tickets), _ptr(out),
                                 rows, attn.hq, attn.splits, float(scale), float(eps), _stream()))
    return out


def lm_head_argmax(normed: torch.Tensor, weight, return_logits: bool = True):
    """BF16 logits and greedy tokens (engine/decode_step.py:60 + engine/decode.py:106):
    lowest index wins exact ties. Returns (logits or None, tokens int64 [rows])."""
    part = linear_partials(normed, weight)
    rows, vocab = part.shape
    dev = normed.device
    logits = torch.empty((rows, vocab), dtype=torch.bfloat16, device=dev) if return_logits else None
    val = torch.empty(rows, dtype=torch.float32, device=dev)
    idx = torch.empty(rows, dtype=torch.int32, device=dev)
    tokens = torch.empty(rows, dtype=torch.int64, device=dev)
    scratch = torch.zeros(lib.q_argmax_scratch_bytes(rows, vocab), dtype=torch.uint8, device=dev)
    check(lib.q_logits_argmax(_ptr(part.data), C.byref(part.plan), _ptr(logits), _ptr(val), _ptr(idx),
                              _ptr(tokens), None, 0, _ptr(scratch), rows, vocab, 0, _stream()))
    return logits, tokens


def device_status() -> list[int]:
    """The four status words of the current device (synchronises): non-zero = a bounded wait
    inside a kernel ran out (attention, stream-K GEMM, tcgen05 GEMM, peer exchange)."""
    out = (C.c_int32 * 4)()
    check(lib.q_device_status(C.byref(out)))
    return list(out)


def clear_status() -> None:
    check(lib.q_clear_status())


def pack_weight_tc(weight: torch.Tensor):
    """Tiles a row-major BF16 [N, K] weight for the tcgen05 projection (load time)."""
    from .weights import TcWeight
    return TcWeight.pack(weight)


def linear_partials_tc(x: torch.Tensor, weight) -> Partials:
    """x @ weight.T as FP32 split-K partials on the tcgen05 kernel
    (engine/kernels/skinny_gemm.py:100-109 at 9 rows and more; any row count up to the
    prompt pass's). `weight` is a TcWeight or a row-major BF16 [N, K] tensor (tiled on the
    fly: load-time work done per call, for tests)."""
    from .weights import TcWeight
    M, K = _bf16_2d(x, "x")
    if not isinstance(weight, TcWeight):
        _bf16_2d(weight, "weight")
        if weight.shape[1] % 32:
            raise ValueError("K must be a multiple of 32")
        weight = TcWeight.pack(weight)
    N, K2 = weight.shape
    if K != K2 or x.device != weight.data.device:
        raise ValueError("x and weight disagree on K or device")
    if M < 1:
        raise ValueError("at least one row")
    p = _lib.plan(M, N, K, tc=True)
    data = torch.empty((p.slots, M, N), dtype=torch.float32, device=x.device)
    check(lib.q_gemm_tc(_ptr(x), _ptr(weight), _ptr(data), M, N, K, _stream()))
    return Partials(data, p)
