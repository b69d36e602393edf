"""Isolated operator sweep: the decode-step GEMMs at the Qwen3-4B weight shapes
for M in {1,4,8,16,32}, timed with CUDA events on weights that rotate over more
than the L2 capacity, reported as achieved weight GB/s.

    python -m starter_b200.opsweep [--m 1 4 8 16 32] [--reps 20] [--json out.json]
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import torch

from ._lib import check, lib

SHAPES = {"qkv": (6144, 2560), "o": (2560, 4096), "gate_up": (19456, 2560),
          "down": (2560, 9728), "lm_head": (151936, 2560)}


def time_gemm(name: str, M: int, reps: int, min_bytes: float = 1.2e9):
    N, K = SHAPES[name]
    wbytes = N * K * 2
    copies = max(2, int(min_bytes // wbytes) + 1)
    gen = torch.Generator(device="cuda").manual_seed(1)
    from .weights import TiledWeight
    ws = [TiledWeight.pack((torch.randn((N, K), device="cuda", generator=gen) * 0.02).to(torch.bfloat16))
          for _ in range(copies)]
    x = torch.randn((M, K), device="cuda", generator=gen).to(torch.bfloat16)
    from . import _lib
    p = _lib.plan(M, N, K)
    part = torch.empty((p.slots, M, N), dtype=torch.float32, device="cuda")
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def launch(i):
        nonlocal s
        check(lib.q_gemm_splitk(C.c_void_p(x.data_ptr()), C.c_void_p(ws[i % copies].data_ptr()),
                                C.c_void_p(part.data_ptr()), M, N, K, s))

    for i in range(copies):
        launch(i)
    torch.cuda.synchronize()
    # back to back inside one CUDA graph (no host launch cost between kernels)
    n = max(reps, copies)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            for i in range(n):
                launch(i)
    s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(3):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    us = 1e3 * a.elapsed_time(b) / (3 * n)
    # isolated: one launch at a time, cold L2 (other copies were streamed in between)
    iso = []
    for i in range(min(n, 8)):
        torch.cuda.synchronize()
        a.record()
        launch(i)
        b.record()
        torch.cuda.synchronize()
        iso.append(1e3 * a.elapsed_time(b))
    iso_us = sorted(iso)[len(iso) // 2]
    return {"op": name, "M": M, "N": N, "K": K, "bytes": wbytes, "back_to_back_us": us,
            "back_to_back_gbs": wbytes / us / 1e3, "isolated_us": iso_us,
            "isolated_gbs": wbytes / iso_us / 1e3, "grid": p.grid, "slots": p.slots}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int, nargs="+", default=[1, 4, 8, 16, 32])
    ap.add_argument("--ops", nargs="+", default=list(SHAPES))
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--prefetch-kb", type=int, default=None)
    ap.add_argument("--no-pdl", action="store_true", help="plain stream-ordered launches")
    ap.add_argument("--debug-flags", type=int, default=0, help="measurement aid (4 = per-CTA trace)")
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    if args.prefetch_kb is not None:
        check(lib.q_set_option(b"gemm_prefetch_kb", args.prefetch_kb))
    if args.no_pdl:
        check(lib.q_set_pdl(0))
    if args.debug_flags:
        check(lib.q_set_option(b"gemm_debug_flags", args.debug_flags))
    rows = []
    for name in args.ops:
        for M in args.m:
            r = time_gemm(name, M, args.reps)
            rows.append(r)
            print(f"{name:8s} M={M:2d}  back-to-back {r['back_to_back_us']:8.2f} us {r['back_to_back_gbs']:7.0f} GB/s"
                  f"   isolated {r['isolated_us']:8.2f} us {r['isolated_gbs']:7.0f} GB/s", flush=True)
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
