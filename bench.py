"""Decode benchmark: Qwen3-4B bf16 greedy decode steps on N B200s.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A "step" is one decode step (one new token per sequence) of the workload
`config.workload` over synthetic data: random-init N(0, 0.02) bf16 weights of the
Qwen3-4B architecture (norm gains 1.0, seed 0) and uniform random prompt ids.
Rank 0 prints ONE JSON line.

  value      decode tok/s of the whole job, state resident in HBM, K graph replays
             timed with CUDA events on the launching stream (max over ranks)
  e2e        the same metric through Engine.generate(): host prompt in, host
             tokens out, prefill and all copies inside the timed region
  step_roofline  algorithmic bytes of a step (weights + KV) / CUDA-event step time
  roofline   the weight-streaming projection kernel (the dominant kernel) as it runs
             INSIDE the step: weight bytes / its launches' share of the step
  gemm_kernel  the same launches replayed alone (CUDA events)
  c3         the batch-32, prompt-2048 workload measured the same way (rides along)
  cpu_baseline  native Hugging Face on the host cores (bounded sample), N=1 only

--impl reference times the native Hugging Face CPU path alone.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_4B = dict(
    vocab_size=151936, hidden_size=2560, intermediate_size=9728, num_hidden_layers=36,
    num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
    rms_norm_eps=1e-6, rope_theta=1_000_000.0, tie_word_embeddings=True,
)
WORKLOADS = {
    # name: (batch, prompt length, new tokens)
    "c2": (1, 1024, 512),
    "c3": (32, 2048, 256),
    "c1": (1, 64, 16),
}
FALLBACK_HBM_GBS = 6650.0


def log(*a):
    print(*a, file=sys.stderr, flush=True)


# ----------------------------------------------------------------------------
# synthetic checkpoint
# ----------------------------------------------------------------------------
def checkpoint_dir(cfg: dict) -> Path:
    base = Path(os.environ.get("QDECODE_BENCH_DIR", "/tmp/qdecode_bench"))
    tag = f"qwen3_L{cfg['num_hidden_layers']}_H{cfg['hidden_size']}_V{cfg['vocab_size']}_seed0"
    return base / tag


def make_checkpoint(cfg: dict, device) -> Path:
    """Random-init N(0, 0.02) bf16 weights, norm gains 1.0, seed 0, written as a
    Hugging Face directory (config.json + safetensors shards)."""
    from safetensors.torch import save_file

    out = checkpoint_dir(cfg)
    done = out / "COMPLETE"
    if done.exists():
        return out
    out.mkdir(parents=True, exist_ok=True)
    hf_cfg = dict(cfg, architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_act="silu",
                  attention_bias=False, attention_dropout=0.0, initializer_range=0.02,
                  sliding_window=None, use_sliding_window=False, use_cache=True, dtype="bfloat16",
                  rope_parameters={"rope_theta": cfg["rope_theta"], "rope_type": "default"})
    (out / "config.json").write_text(json.dumps(hf_cfg, indent=1))
    gen = torch.Generator(device=device).manual_seed(0)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def rnd(*shape):
        t = torch.empty(shape, dtype=torch.float32, device=device).normal_(0.0, 0.02, generator=gen)
        return t.to(torch.bfloat16).cpu()

    def ones(n):
        return torch.ones(n, dtype=torch.bfloat16)

    weight_map, total_size = {}, 0

    def save(tensors, name):
        nonlocal total_size
        save_file(tensors, str(out / name), metadata={"format": "pt"})
        for k, v in tensors.items():
            weight_map[k] = name
            total_size += v.numel() * 2

    save({"model.embed_tokens.weight": rnd(V, H), "model.norm.weight": ones(H)},
         "model-embed.safetensors")
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        save({
            p + "self_attn.q_proj.weight": rnd(nq * D, H), p + "self_attn.k_proj.weight": rnd(nkv * D, H),
            p + "self_attn.v_proj.weight": rnd(nkv * D, H), p + "self_attn.o_proj.weight": rnd(H, nq * D),
            p + "self_attn.q_norm.weight": ones(D), p + "self_attn.k_norm.weight": ones(D),
            p + "mlp.gate_proj.weight": rnd(I, H), p + "mlp.up_proj.weight": rnd(I, H),
            p + "mlp.down_proj.weight": rnd(H, I), p + "input_layernorm.weight": ones(H),
            p + "post_attention_layernorm.weight": ones(H),
        }, f"model-layer{i:02d}.safetensors")
    (out / "model.safetensors.index.json").write_text(
        json.dumps({"metadata": {"total_size": total_size}, "weight_map": weight_map}))
    done.write_text("ok")
    return out


def make_prompt(batch: int, length: int, vocab: int):
    g = torch.Generator().manual_seed(0)
    return torch.randint(0, vocab, (batch, length), generator=g)


# ----------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU in a thread (read-only NVML)."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # no NVML: report that, do not fail the bench
            self.nv = None
            self.err = repr(e)

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.01)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "error": self.err}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# ----------------------------------------------------------------------------
# reference arm / CPU baseline: native Hugging Face on the host cores
# ----------------------------------------------------------------------------
def cpu_reference(model_dir: Path, batch: int, prompt_len: int, steps: int, warmup: int, vocab: int):
    """Times `steps` decode steps of the native Hugging Face greedy loop on CPU
    after an untimed prefill of `prompt_len` tokens and `warmup` steps."""
    from oracle import qwen3_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    t0 = time.perf_counter()
    model = O.native_model(str(model_dir))
    load_s = time.perf_counter() - t0
    prompt = make_prompt(batch, prompt_len, vocab)
    stamps = []
    O.native_greedy(model, prompt, 1 + warmup + steps, return_logits=False,
                    on_step=lambda i: stamps.append(time.perf_counter()))
    # stamps[0] = after prefill; then one per decode step
    timed = stamps[warmup + steps] - stamps[warmup]
    return {"tok_s": batch * steps / timed, "ms_per_step": 1e3 * timed / steps, "cores": cores,
            "load_s": load_s, "prefill_s": stamps[0] - t0 - load_s, "steps": steps}


def run_reference(args, rank: int, world: int) -> None:
    if rank != 0:
        return
    batch, prompt_len, _ = WORKLOADS[args.workload]
    cfg = dict(QWEN3_4B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    model_dir = make_checkpoint(cfg, dev)
    steps = min(args.steps, args.cpu_steps)
    warmup = min(args.warmup, 1)
    sample_prompt = min(prompt_len, args.cpu_prompt)
    r = cpu_reference(model_dir, batch, sample_prompt, steps, warmup, cfg["vocab_size"])
    sample = (f"native Hugging Face Qwen3ForCausalLM greedy loop on CPU, batch {batch}, prompt "
              f"{sample_prompt} of {prompt_len} tokens (untimed prefill), {steps} timed decode steps")
    line = {
        "impl": "reference", "metric": "decode_tok_s", "value": r["tok_s"], "unit": "tok/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": r["ms_per_step"],
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(args, cfg, batch, prompt_len),
        "cpu_baseline": {"value": r["tok_s"], "unit": "tok/s", "cores": r["cores"], "kind": "reference",
                         "sample": sample},
        "e2e": {"value": r["tok_s"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(args, cfg, batch, prompt_len):
    new = WORKLOADS[args.workload][2]
    return {
        "workload": f"{args.workload}: Qwen3-4B architecture ({cfg['num_hidden_layers']} layers) bf16 "
                    f"greedy decode, batch {batch}, prompt {prompt_len}, {new} new tokens",
        "batch": batch, "prompt_len": prompt_len, "new_tokens": new,
        "layers": cfg["num_hidden_layers"], "parallelism": f"tp{args.gpus}",
        "l2": "inputs larger than L2 (weights 8.04 GB streamed once per step)",
    }


# ----------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------
KIND_NAMES = {1: "k_gemm_streamk", 2: "k_gemm_tc", 3: "k_attn_decode", 4: "k_add_rmsnorm", 5: "k_swiglu",
              6: "k_embed_rmsnorm", 7: "k_logits_argmax", 8: "k_add_rmsnorm_peers"}


def step_projections(state):
    """(activation tensor, weight) of every projection of one decode step, in step order."""
    w = state.w
    out = []
    for lt in w.layers:
        out += [(state.normed, lt.wqkv), (state.attended, lt.wo), (state.normed, lt.wgu), (state.act, lt.wdown)]
    out.append((state.normed, w.lm_head))
    return out


def time_gemm_kernel(state, reps: int = 5):
    """The step's projection launches replayed ALONE, back to back, as one CUDA graph on the
    real weights (far larger than L2), timed with CUDA events on the launching stream."""
    import ctypes as C
    from starter_b200._lib import lib, check

    rows = state.rows
    P = C.c_void_p(state.partials.data_ptr())
    proj = step_projections(state)
    nbytes = sum(wt.numel() * 2 for _, wt in proj)

    def seq(s):
        for x, wt in proj:
            xp = C.c_void_p(x.data_ptr())
            if state.uses_tc:
                check(lib.q_gemm_tc(xp, C.c_void_p(wt.tc().data_ptr()), P, rows, wt.shape[0], wt.shape[1], s))
            elif wt.interleaved8 and rows <= 8:      # the step runs this one with the SwiGLU epilogue
                check(lib.q_gemm_swiglu(xp, C.c_void_p(wt.data_ptr()), C.c_void_p(state.act.data_ptr()), rows,
                                        wt.shape[0] // 2, wt.shape[1], s))
            else:
                check(lib.q_gemm_splitk(xp, C.c_void_p(wt.data_ptr()), P, rows, wt.shape[0], wt.shape[1], s))

    for _ in range(2):
        seq(C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            seq(C.c_void_p(torch.cuda.current_stream().cuda_stream))
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / reps
    return {"launches_per_step": len(proj), "bytes_per_step": nbytes,
            "avg_launch_us": 1e3 * ms / len(proj), "gbs": nbytes / (ms * 1e-3) / 1e9}


def time_in_step(state, reps: int = 8):
    """Where the time of one decode step goes, per kernel, measured INSIDE the step: with the
    library's timeline option every kernel stamps %globaltimer at its first CTA's start and its
    last CTA's end; a kernel's share is (its end - the previous kernel's end), so the overlap
    that dependent launches give is attributed to the kernel that benefits. One extra graph of
    the step is recorded with the stamps on and replayed; all ranks do the same."""
    import ctypes as C
    from starter_b200._lib import lib, check

    saved = (state.tokens.clone(), state.position.clone())
    check(lib.q_set_option(b"timeline", 1))
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            state.step()
        n_max = 4096
        buf = (C.c_uint64 * (4 * n_max))()
        kinds = (C.c_int32 * n_max)()
        shares: dict[int, list[float]] = {}
        span = []
        for rep in range(reps + 2):
            state.tokens.copy_(saved[0])
            state.position.copy_(saved[1])
            graph.replay()
            torch.cuda.synchronize()
            n = lib.q_debug_timeline(buf, n_max)
            if n <= 0:
                return None
            lib.q_debug_timeline_kinds(kinds, n_max)
            if rep < 2:
                continue
            per = {}
            for i in range(n):
                begin, _, end, _ = (int(buf[4 * i + j]) for j in range(4))
                prev_end = int(buf[4 * (i - 1) + 2]) if i else begin
                per[kinds[i]] = per.get(kinds[i], 0.0) + max(0.0, (end - prev_end) / 1e3)
            for k, v in per.items():
                shares.setdefault(k, []).append(v)
            span.append((int(buf[4 * (n - 1) + 2]) - int(buf[0])) / 1e3)
        counts = {}
        for i in range(n):
            counts[kinds[i]] = counts.get(kinds[i], 0) + 1
        # the same shares by launch position inside a layer (a layer starts at its attention
        # launch), mean over the inner layers of the last replay
        att = [i for i in range(n) if kinds[i] == 3]
        layer = []
        if len(att) >= 6:
            period = att[1] - att[0]
            inner = att[2:-2]
            for j in range(period):
                vals = [(int(buf[4 * (a + j) + 2]) - int(buf[4 * (a + j - 1) + 2])) / 1e3 for a in inner]
                layer.append([KIND_NAMES.get(kinds[att[2] + j], str(kinds[att[2] + j])), round(sum(vals) / len(vals), 2)])
    finally:
        check(lib.q_set_option(b"timeline", 0))
        state.tokens.copy_(saved[0])
        state.position.copy_(saved[1])
    med = lambda v: sorted(v)[len(v) // 2]
    return {"us": {KIND_NAMES.get(k, str(k)): med(v) for k, v in shares.items()},
            "launches": {KIND_NAMES.get(k, str(k)): c for k, c in counts.items()},
            "layer_us": layer, "step_span_us": med(span)}


def kernels_per_step(state) -> int:
    """Launches of this library's kernels in one decode step (NCCL's are not counted)."""
    L, rows = state.cfg.n_layers, state.rows
    if state.tp == 1:
        if rows <= 8:
            # embed, first QKV | attention, O, gate|up (add+norm prologue, SwiGLU epilogue), down,
            # next QKV or lm_head (add+norm prologue) | argmax
            return 2 + 5 * L + 1
        # embed | QKV, attention, O, add+norm, gate|up, SwiGLU, down, add+norm | lm_head, argmax
        return 1 + 8 * L + 2
    if state.peers:
        # QKV, attention, O, add+norm over the peers, gate|up (+ SwiGLU launch above 8 rows), down,
        # add+norm over the peers (+ two slot reductions above 8 rows) | lm_head, argmax, peer merge
        return 1 + (7 if rows <= 8 else 10) * L + 3
    # NCCL: slot reductions before each all-reduce, separate add+norm launches, argmax merge
    return 1 + (9 if rows <= 8 else 10) * L + 3


def measure_decode(state, K: int, W: int, world: int, dev, local_rank: int):
    """W warm-up replays, then K timed replays of the captured step (CUDA events on the launching
    stream, barrier + synchronize on both sides, max over ranks)."""
    import torch.distributed as dist
    for _ in range(W):
        state.advance()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start_pos = int(state.position.item())
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        a.record()
        for _ in range(K):
            state.advance()
        b.record()
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    end_pos = int(state.position.item())
    assert end_pos - start_pos == K, (start_pos, end_pos, K)
    avg_keys = (start_pos + 1 + end_pos) / 2.0
    return ms, avg_keys, clocks.summary()


def tokens_digest(steps) -> str:
    """sha256 over the first 64 emitted steps' token ids (16 hex digits): equal digests at
    different GPU counts mean the same tokens were emitted."""
    import hashlib
    flat = [int(t) for step in steps[:64] for t in step]
    return hashlib.sha256(",".join(map(str, flat)).encode()).hexdigest()[:16]


def run_ours(args, rank: int, world: int, local_rank: int) -> None:
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    dev = torch.device(f"cuda:{local_rank}")
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    from starter_b200 import Engine, _lib
    from starter_b200.decode import DecodeState
    from starter_b200.ops import device_status

    for item in args.option:                         # "name=value" tuning knobs of q_set_option
        key, _, val = item.partition("=")
        _lib.check(_lib.lib.q_set_option(key.encode(), int(val)))
    batch, prompt_len, new_tokens = WORKLOADS[args.workload]
    cfg = dict(QWEN3_4B)
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    K, W = args.steps, max(args.warmup, 3)
    n_new = max(new_tokens, K + W + 2)
    if rank == 0:
        t0 = time.perf_counter()
        model_dir = make_checkpoint(cfg, dev)
        log(f"[bench] checkpoint ready in {time.perf_counter() - t0:.1f}s at {model_dir}")
    if world > 1:
        dist.barrier()
    model_dir = checkpoint_dir(cfg)
    t0 = time.perf_counter()
    engine = Engine(str(model_dir), device=str(dev), group=group, tp_path=args.tp_path)
    log(f"[bench] rank {rank}: weights loaded in {time.perf_counter() - t0:.1f}s")
    prompt = make_prompt(batch, prompt_len, cfg["vocab_size"])
    prompt_list = prompt.tolist()

    def status_over_ranks():
        st = torch.tensor(device_status(), dtype=torch.int32, device=dev)
        if world > 1:
            dist.all_reduce(st, op=dist.ReduceOp.MAX)
        return st.tolist()

    with torch.inference_mode():
        # ---- device-resident timing: K graph replays ----
        state = DecodeState(engine.weights, batch, prompt_len, n_new, group=group, tp_path=args.tp_path)
        engine.decode_state = state
        state.prefill(prompt.to(dev))
        state.capture()
        ms, avg_keys, clocks = measure_decode(state, K, W, world, dev, local_rank)
        step_bytes_rank = state.step_bytes(int(round(avg_keys)))
        in_step = time_in_step(state)
        gemm = time_gemm_kernel(state) if rank == 0 else None
        tp_path = state.tp_path
        launches = kernels_per_step(state)

        # ---- end to end through the public API ----
        e2e = None
        if not args.skip_e2e:
            list(engine.generate(prompt_list, n_new))        # warm-up call (capture already done)
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats(dev)
            if world > 1:
                dist.barrier()
            t_start = time.perf_counter()
            stamps, emitted = [], []
            for tok in engine.generate(prompt_list, n_new):
                stamps.append(time.perf_counter())
                emitted.append(tok)
            torch.cuda.synchronize()
            t_total = time.perf_counter() - t_start
            te = torch.tensor([t_total], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(te, op=dist.ReduceOp.MAX)
            t_total = float(te.item())
            e2e = {
                "value": batch * n_new / t_total, "unit": "tok/s",
                "h2d_bytes_per_step": batch * prompt_len * 8 / n_new, "d2h_bytes_per_step": batch * 8 + 16,
                "new_tokens": n_new, "ttft_ms": 1e3 * (stamps[0] - t_start),
                "tpot_ms": 1e3 * (stamps[-1] - stamps[0]) / max(1, n_new - 1),
                "peak_mem_bytes": int(torch.cuda.max_memory_allocated(dev)),
                "tokens_sha16": tokens_digest(emitted),
            }
        status = status_over_ranks()

        # ---- the batch-32 workload next to the headline one (the case tensor parallelism is for) ----
        c3 = None
        if args.workload == "c2" and not args.no_c3:
            engine.decode_state = None
            state.graph = None
            del state
            torch.cuda.empty_cache()
            b3, p3, n3 = WORKLOADS["c3"]
            K3 = min(K, 32)
            st3 = DecodeState(engine.weights, b3, p3, max(n3, K3 + W + 2), group=group, tp_path=args.tp_path)
            t_pre = time.perf_counter()
            st3.prefill(make_prompt(b3, p3, cfg["vocab_size"]).to(dev))
            torch.cuda.synchronize()
            prefill_ms = 1e3 * (time.perf_counter() - t_pre)
            first_tokens = st3.tokens.cpu().tolist()
            st3.capture()
            ms3, keys3, clocks3 = measure_decode(st3, K3, W, world, dev, local_rank)
            bytes3 = st3.step_bytes(int(round(keys3)))
            digest = tokens_digest([first_tokens, st3.tokens.cpu().tolist()])
            in3 = time_in_step(st3) or {}
            c3 = {"workload": f"c3: batch {b3}, prompt {p3}", "steps": K3, "ms_per_step": ms3 / K3,
                  "value": b3 * K3 / (ms3 * 1e-3), "unit": "tok/s", "tp_path": st3.tp_path,
                  "projections": "tcgen05" if st3.uses_tc else "mma.sync",
                  "bytes_per_step_per_gpu": bytes3, "step_gbs_per_gpu": bytes3 / (ms3 / K3 * 1e-3) / 1e9,
                  "gpu_launches": kernels_per_step(st3) * K3, "prefill_ms": prefill_ms,
                  "in_step_us": in3.get("us"), "in_step_layer_us": in3.get("layer_us"),
                  "tokens_sha16": digest, "clocks": clocks3, "device_status": status_over_ranks()}
            st3.graph = None
            del st3

    def teardown():
        """NCCL communicators must not be torn down while captured graphs that hold
        their kernels are alive; a timer forces the exit if teardown still stalls."""
        if world == 1:
            return
        engine.decode_state = None
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        threading.Timer(20.0, os._exit, [0]).start()
        dist.destroy_process_group()

    if rank != 0:
        teardown()
        return

    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        peak, peak_src = float(json.loads(peaks_file.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = FALLBACK_HBM_GBS, "fallback"
    ms_step = ms / K
    tok_s = batch * K / (ms * 1e-3)
    step_gbs = step_bytes_rank / (ms_step * 1e-3) / 1e9
    kernel = "k_gemm_tc" if tp_path is not None and in_step and "k_gemm_tc" in in_step["us"] else "k_gemm_streamk"
    gemm_info = {
        "kernel": kernel, "achieved": gemm["gbs"], "unit": "GB/s", "frac": gemm["gbs"] / peak,
        "avg_launch_us": gemm["avg_launch_us"], "launches_per_step": gemm["launches_per_step"],
        "bytes_per_launch": gemm["bytes_per_step"] / gemm["launches_per_step"],
        "how": "the step's projection launches replayed alone, back to back, as one CUDA graph on the real weights",
    }
    # the dominant kernel as it runs INSIDE the step: its launches' share of the step time
    if in_step and kernel in in_step["us"]:
        gemm_us = in_step["us"][kernel]
        n_launch = in_step["launches"][kernel]
        achieved = gemm["bytes_per_step"] / (gemm_us * 1e-6) / 1e9
        how = ("weight bytes of the step's projection launches / the sum of their in-step shares "
               "(each kernel's last-CTA end minus the previous kernel's, %globaltimer stamps inside a replayed graph)")
    else:
        gemm_us, n_launch, achieved = gemm["avg_launch_us"] * gemm["launches_per_step"], gemm["launches_per_step"], gemm["gbs"]
        how = "stand-alone replay (no in-step stamps available)"
    roofline = {
        "bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": achieved / peak,
        "traffic": args.traffic_bytes if args.traffic_bytes else 1.017 * gemm["bytes_per_step"] / n_launch,
        "traffic_source": "1.017 x algorithmic bytes, from the ncu capture of the four projections of a layer "
                          "inside a 4-layer step",
        "peak_source": peak_src, "avg_launch_us": gemm_us / n_launch, "launches_per_step": n_launch,
        "bytes_per_launch": gemm["bytes_per_step"] / n_launch, "how": how,
    }
    line = {
        "metric": "decode_tok_s", "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": K,
        "warmup": W, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, cfg, batch, prompt_len),
        "step_roofline": {"bytes_per_step_per_gpu": step_bytes_rank, "achieved": step_gbs, "peak": peak,
                          "unit": "GB/s", "frac": step_gbs / peak, "avg_visible_keys": avg_keys},
        "roofline": roofline,
        "gemm_kernel": gemm_info,
        "in_step_us": in_step["us"] if in_step else None,
        "in_step_layer_us": in_step["layer_us"] if in_step else None,
        "e2e": e2e,
        "tp_path": tp_path,
        "gpu_launches": launches * K,
        "clocks": clocks,
        "device_status": status,
        "c3": c3,
    }
    if world == 1 and not args.no_cpu_baseline:
        r = cpu_reference(model_dir, batch, min(prompt_len, args.cpu_prompt), args.cpu_steps, 1,
                          cfg["vocab_size"])
        line["cpu_baseline"] = {
            "value": r["tok_s"], "unit": "tok/s", "cores": r["cores"], "kind": "reference",
            "ms_per_step": r["ms_per_step"],
            "sample": f"native Hugging Face Qwen3ForCausalLM greedy loop on CPU, batch {batch}, prompt "
                      f"{min(prompt_len, args.cpu_prompt)} tokens (untimed prefill), {r['steps']} timed decode steps",
        }
    print(json.dumps(line), flush=True)
    teardown()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="c2")
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers (not a valid bench)")
    ap.add_argument("--cpu-steps", type=int, default=8)
    ap.add_argument("--cpu-prompt", type=int, default=1024)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true",
                    help="profiling runs only: skip the Engine.generate leg (e2e becomes null)")
    ap.add_argument("--traffic-bytes", type=float, default=None,
                    help="DRAM bytes per projection launch from an ncu capture, if a newer one is at hand")
    ap.add_argument("--option", action="append", default=[], metavar="NAME=VALUE",
                    help="library tuning knob (q_set_option), repeatable")
    ap.add_argument("--tp-path", choices=("auto", "peers", "nccl"), default="auto",
                    help="how tensor-parallel ranks exchange partial sums")
    ap.add_argument("--no-c3", action="store_true",
                    help="skip the batch-32 record that rides along with the batch-1 headline")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world != args.gpus:
        if args.gpus > 1 and world == 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
