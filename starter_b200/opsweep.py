"""Isolated operator sweeps, timed with CUDA events.

  projections   the decode-step GEMMs at the Qwen3-4B weight shapes for M in {1,4,8,16,32}
                (and above) on weights that rotate over more than the L2 capacity, reported as
                achieved weight GB/s; --kernel picks the stream-K (mma.sync) kernel, the
                tcgen05 kernel, or "auto" (stream-K up to 8 rows, tcgen05 above: what the
                decode step does)
  fused         the element-wise consumers at the same M: add + RMSNorm on partials, plain
                RMSNorm, SwiGLU on partials, q/k head norm + RoPE + KV page write, and the
                single-launch decode attention (norm + RoPE + KV write + attention + merge)
  attention     the small-query verification attention: batch 8, T in {2,4,8} query tokens,
                32 / 8 heads, KV lengths {4096, 16384, 32768}, as KV GB/s, next to the
                single-token kernel run T times

    python -m starter_b200.opsweep [--sweep projections fused attention] [--m 1 4 8 16 32]
                                   [--kernel auto|mma|tc] [--json out.json] [--md out.md]
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import torch

from . import _lib, ops
from ._lib import check, lib
from .weights import TcWeight, TiledWeight, rotary_tables

SHAPES = {"qkv": (6144, 2560), "o": (2560, 4096), "gate_up": (19456, 2560),
          "down": (2560, 9728), "lm_head": (151936, 2560)}
H, I = 2560, 9728


class _Rope:
    rope_theta = 1_000_000.0


def _graph_time(launch, n: int, reps: int = 3) -> float:
    """Average microseconds of launch(i), i in [0, n), back to back inside one CUDA graph
    (no host launch cost between kernels), CUDA events around `reps` replays."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(n):
                launch(i)
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    return 1e3 * a.elapsed_time(b) / (reps * n)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def time_gemm(name: str, M: int, reps: int, kernel: str = "auto", min_bytes: float = 1.2e9):
    N, K = SHAPES[name]
    wbytes = N * K * 2
    copies = max(2, int(min_bytes // wbytes) + 1)
    gen = torch.Generator(device="cuda").manual_seed(1)
    use_tc = kernel == "tc" or (kernel == "auto" and M > 8)
    pack = TcWeight.pack if use_tc else TiledWeight.pack
    ws = [pack((torch.randn((N, K), device="cuda", generator=gen) * 0.02).to(torch.bfloat16)) for _ in range(copies)]
    x = torch.randn((M, K), device="cuda", generator=gen).to(torch.bfloat16)
    p = _lib.plan(M, N, K, tc=use_tc)
    part = torch.empty((p.slots, M, N), dtype=torch.float32, device="cuda")
    fn = lib.q_gemm_tc if use_tc else lib.q_gemm_splitk

    def launch(i):
        check(fn(C.c_void_p(x.data_ptr()), C.c_void_p(ws[i % copies].data_ptr()), C.c_void_p(part.data_ptr()),
                 M, N, K, _stream()))

    for i in range(copies):
        launch(i)
    torch.cuda.synchronize()
    n = max(reps, copies)
    us = _graph_time(launch, n)
    # isolated: one launch at a time, cold L2 (other copies were streamed in between)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iso = []
    for i in range(min(n, 8)):
        torch.cuda.synchronize()
        a.record()
        launch(i)
        b.record()
        torch.cuda.synchronize()
        iso.append(1e3 * a.elapsed_time(b))
    iso_us = sorted(iso)[len(iso) // 2]
    return {"sweep": "projections", "op": name, "kernel": "tcgen05" if use_tc else "mma.sync", "M": M, "N": N,
            "K": K, "bytes": wbytes, "back_to_back_us": us, "back_to_back_gbs": wbytes / us / 1e3,
            "isolated_us": iso_us, "isolated_gbs": wbytes / iso_us / 1e3, "grid": p.grid, "slots": p.slots}


def time_fused(M: int, reps: int):
    """The fused consumers at M rows on the Qwen3-4B widths. Inputs rotate over 8 copies so
    that a launch does not find its operands in L1; they are L2-resident, as in the step."""
    gen = torch.Generator(device="cuda").manual_seed(2)
    rnd = lambda *s: torch.randn(s, device="cuda", generator=gen).to(torch.bfloat16)
    use_tc = M > 8
    out = []
    copies = 8
    gain = (1 + 0.1 * torch.randn(H, device="cuda", generator=gen)).to(torch.bfloat16)
    # partials of the down projection (hidden-size rows) and of gate|up, made by the kernel the step uses
    wdown = (ops.pack_weight_tc if use_tc else ops.pack_weight)((rnd(H, I) * 0.02).contiguous())
    wgu = (ops.pack_weight_tc if use_tc else ops.pack_weight)((rnd(2 * I, H) * 0.02).contiguous())
    wqkv = (ops.pack_weight_tc if use_tc else ops.pack_weight)((rnd(6144, H) * 0.02).contiguous())
    lin = ops.linear_partials_tc if use_tc else ops.linear_partials
    downs = [lin(rnd(M, I), wdown) for _ in range(copies)]
    gus = [lin(rnd(M, H), wgu) for _ in range(copies)]
    qkvs = [lin(rnd(M, H), wqkv) for _ in range(copies)]
    res = [rnd(M, H) for _ in range(copies)]
    tot, nrm = torch.empty_like(res[0]), torch.empty_like(res[0])
    act = torch.empty((M, I), dtype=torch.bfloat16, device="cuda")

    def add_norm(i):
        pt = downs[i % copies]
        check(lib.q_add_rmsnorm(ops._ptr(res[i % copies]), ops._ptr(pt.data), C.byref(pt.plan), ops._ptr(gain),
                                ops._ptr(tot), ops._ptr(nrm), M, H, 1e-6, _stream()))

    def plain_norm(i):
        check(lib.q_rmsnorm(ops._ptr(res[i % copies]), ops._ptr(gain), ops._ptr(nrm), M, H, 1e-6, _stream()))

    def swiglu(i):
        pt = gus[i % copies]
        check(lib.q_swiglu(ops._ptr(pt.data), C.byref(pt.plan), ops._ptr(act), M, I, _stream()))

    capacity, pos = 1536, 1030
    cache = ops.PagedKV(M, 8, capacity, "cuda")
    cos, sin = rotary_tables(_Rope, capacity, "cuda")
    hg = torch.ones(128, dtype=torch.bfloat16, device="cuda")
    position = torch.tensor([pos], dtype=torch.int32, device="cuda")
    q = torch.empty((M, 32, 128), dtype=torch.bfloat16, device="cuda")
    attn = ops.SmallQueryAttention(M, 32, 8, capacity, "cuda")
    attn.tickets = torch.zeros(M * 8, dtype=torch.int32, device="cuda")
    attended = torch.empty((M, 4096), dtype=torch.bfloat16, device="cuda")

    def rope_cache(i):
        pt = qkvs[i % copies]
        check(lib.q_qkv_norm_rope_cache(ops._ptr(pt.data), C.byref(pt.plan), ops._ptr(hg), ops._ptr(hg), ops._ptr(cos),
                                        ops._ptr(sin), ops._ptr(position), ops._ptr(q), C.byref(cache.layout), M, 1,
                                        32, 1e-6, _stream()))

    def decode_attention(i):
        pt = qkvs[i % copies]
        check(lib.q_attention_decode(ops._ptr(pt.data), C.byref(pt.plan), ops._ptr(hg), ops._ptr(hg), ops._ptr(cos),
                                     ops._ptr(sin), ops._ptr(position), C.byref(cache.layout), ops._ptr(attn.partials),
                                     ops._ptr(attn.stats), ops._ptr(attn.tickets), ops._ptr(attended), M, 32,
                                     attn.splits, 128 ** -0.5, 1e-6, _stream()))

    kv_bytes = M * 8 * (pos + 1) * 128 * 2 * 2
    for name, fn, nbytes in (("add_rms_norm (down partials)", add_norm, downs[0].data.numel() * 4),
                             ("rms_norm", plain_norm, M * H * 2),
                             ("silu_mul (gate|up partials)", swiglu, gus[0].data.numel() * 4),
                             ("qkv_norm_rope_cache", rope_cache, qkvs[0].data.numel() * 4),
                             (f"decode_attention ({pos + 1} keys)", decode_attention, kv_bytes)):
        for i in range(copies):
            fn(i)
        torch.cuda.synchronize()
        us = _graph_time(fn, max(reps, copies))
        out.append({"sweep": "fused", "op": name, "M": M, "us": us, "operand_bytes": nbytes,
                    "gbs": nbytes / us / 1e3, "partials_from": "tcgen05" if use_tc else "mma.sync"})
    return out


def time_attention(L: int, T: int, reps: int, batch: int = 8, nq: int = 32, nkv: int = 8):
    """Verification attention at KV length L with T query tokens per sequence, against the
    single-token kernel run once per token (which reads the cache T times)."""
    gen = torch.Generator(device="cuda").manual_seed(3)
    capacity = L + T
    cache = ops.PagedKV(batch, nkv, capacity, "cuda")
    cache.k.normal_(generator=gen)
    cache.v.normal_(generator=gen)
    q = torch.randn((batch * T, nq, 128), device="cuda", generator=gen).to(torch.bfloat16)
    multi = ops.SmallQueryAttention(batch, nq, nkv, capacity, "cuda", tokens_per_seq=T)
    single = ops.SmallQueryAttention(batch, nq, nkv, capacity, "cuda", tokens_per_seq=1)
    position = torch.tensor([L], dtype=torch.int32, device="cuda")
    positions = [torch.tensor([L + t], dtype=torch.int32, device="cuda") for t in range(T)]
    out_m = torch.empty((batch * T, nq * 128), dtype=torch.bfloat16, device="cuda")
    out_s = torch.empty((batch, nq * 128), dtype=torch.bfloat16, device="cuda")
    qs = [q.view(batch, T, nq, 128)[:, t].contiguous() for t in range(T)]

    def run_multi(i):
        check(lib.q_attention(ops._ptr(q), C.byref(cache.layout), ops._ptr(position), ops._ptr(multi.partials),
                              ops._ptr(multi.stats), ops._ptr(out_m), batch, T, nq, multi.splits, 128 ** -0.5,
                              _stream()))

    def run_single(i):
        for t in range(T):
            check(lib.q_attention(ops._ptr(qs[t]), C.byref(cache.layout), ops._ptr(positions[t]),
                                  ops._ptr(single.partials), ops._ptr(single.stats), ops._ptr(out_s), batch, 1, nq,
                                  single.splits, 128 ** -0.5, _stream()))

    for fn in (run_multi, run_single):
        fn(0)
    torch.cuda.synchronize()
    # the KV of one call (0.13 .. 1.07 GB) is larger than L2 from 16 K keys on; at 4 K keys the
    # cache rotates through L2 only partly: the figure is then an upper bound on DRAM GB/s
    us_m = _graph_time(run_multi, reps)
    us_s = _graph_time(run_single, reps)
    kv_bytes = batch * nkv * (L + T) * 128 * 2 * 2
    return {"sweep": "attention", "L": L, "T": T, "batch": batch, "kv_bytes": kv_bytes, "multi_us": us_m,
            "multi_kv_gbs": kv_bytes / us_m / 1e3, "single_x_T_us": us_s, "speedup_over_token_by_token": us_s / us_m,
            "splits": multi.splits}


def to_markdown(rows) -> str:
    out = []
    proj = [r for r in rows if r["sweep"] == "projections"]
    if proj:
        out += ["| projection | kernel | M | back-to-back us | GB/s | isolated us | GB/s | slots |", "|---|---|---:|---:|---:|---:|---:|---:|"]
        out += [f"| {r['op']} {r['N']}x{r['K']} | {r['kernel']} | {r['M']} | {r['back_to_back_us']:.2f} | "
                f"{r['back_to_back_gbs']:.0f} | {r['isolated_us']:.2f} | {r['isolated_gbs']:.0f} | {r['slots']} |" for r in proj]
        out.append("")
    fused = [r for r in rows if r["sweep"] == "fused"]
    if fused:
        out += ["| fused operator | M | us | operand bytes | GB/s (L2-resident operands) |", "|---|---:|---:|---:|---:|"]
        out += [f"| {r['op']} | {r['M']} | {r['us']:.2f} | {r['operand_bytes']} | {r['gbs']:.0f} |" for r in fused]
        out.append("")
    att = [r for r in rows if r["sweep"] == "attention"]
    if att:
        out += ["| KV length | T | KV bytes | multi-token us | KV GB/s | T single-token calls us | speed-up |", "|---:|---:|---:|---:|---:|---:|---:|"]
        out += [f"| {r['L']} | {r['T']} | {r['kv_bytes']} | {r['multi_us']:.1f} | {r['multi_kv_gbs']:.0f} | "
                f"{r['single_x_T_us']:.1f} | {r['speedup_over_token_by_token']:.2f} |" for r in att]
        out.append("")
    return "\n".join(out)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sweep", nargs="+", default=["projections"], choices=("projections", "fused", "attention"))
    ap.add_argument("--m", type=int, nargs="+", default=[1, 4, 8, 16, 32])
    ap.add_argument("--ops", nargs="+", default=list(SHAPES))
    ap.add_argument("--kernel", choices=("auto", "mma", "tc"), default="auto")
    ap.add_argument("--lengths", type=int, nargs="+", default=[4096, 16384, 32768])
    ap.add_argument("--tokens", type=int, nargs="+", default=[2, 4, 8])
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--prefetch-kb", type=int, default=None)
    ap.add_argument("--no-pdl", action="store_true", help="plain stream-ordered launches")
    ap.add_argument("--debug-flags", type=int, default=0, help="measurement aid (4 = per-CTA trace)")
    ap.add_argument("--json", default=None)
    ap.add_argument("--md", default=None)
    args = ap.parse_args()
    if args.prefetch_kb is not None:
        check(lib.q_set_option(b"gemm_prefetch_kb", args.prefetch_kb))
    if args.no_pdl:
        check(lib.q_set_pdl(0))
    if args.debug_flags:
        check(lib.q_set_option(b"gemm_debug_flags", args.debug_flags))
    rows = []
    if "projections" in args.sweep:
        for name in args.ops:
            for M in args.m:
                r = time_gemm(name, M, args.reps, args.kernel)
                rows.append(r)
                print(f"{name:8s} {r['kernel']:8s} M={M:3d}  back-to-back {r['back_to_back_us']:8.2f} us "
                      f"{r['back_to_back_gbs']:7.0f} GB/s   isolated {r['isolated_us']:8.2f} us "
                      f"{r['isolated_gbs']:7.0f} GB/s", flush=True)
                torch.cuda.empty_cache()
    if "fused" in args.sweep:
        for M in args.m:
            for r in time_fused(M, args.reps):
                rows.append(r)
                print(f"{r['op']:34s} M={M:3d} {r['us']:8.2f} us {r['gbs']:7.0f} GB/s", flush=True)
            torch.cuda.empty_cache()
    if "attention" in args.sweep:
        for L in args.lengths:
            for T in args.tokens:
                r = time_attention(L, T, args.reps)
                rows.append(r)
                print(f"attention L={L:6d} T={T} multi {r['multi_us']:8.1f} us {r['multi_kv_gbs']:6.0f} GB/s  "
                      f"single x T {r['single_x_T_us']:8.1f} us  speed-up {r['speedup_over_token_by_token']:.2f}", flush=True)
                torch.cuda.empty_cache()
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    if args.md:
        with open(args.md, "w") as f:
            f.write(to_markdown(rows))
    from .ops import device_status
    print("device status", device_status())


if __name__ == "__main__":
    main()
