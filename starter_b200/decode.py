"""Fixed-address decode state, prefill, CUDA-graph capture and token emission.

Mirrors the reference's DecodeState (engine/decode.py:38-148): static buffers,
a `step()` that leaves the next token and position on the device, a captured
graph replayed once per token, and a pinned-host handoff whose copy of step k
is enqueued before step k+1 is launched. The KV cache is paged
(64-token pages) instead of the reference's contiguous StaticCache.

Tensor parallelism: every rank holds its head / FFN-column / vocabulary shard
and runs the same step; the fp32 partial sums after O-proj and down-proj are
summed over the ranks before the single bf16 rounding of a Linear output - by
default inside the add+norm kernel, which reads every rank's partials from
symmetric (peer-mapped) memory, else by an NCCL all-reduce - and the per-rank
(max, index) pairs of the vocabulary-sharded lm_head are exchanged through peer
memory as well (else all-gathered).

Every step's last kernel copies the library's device status words next to the
tokens; emit() reads them from pinned host memory with the tokens and raises
when a bounded wait inside a kernel ran out, so such a step never hands wrong
tokens to the caller.
"""
from __future__ import annotations

import ctypes as C
import os
import sys

import torch

from . import _lib
from ._lib import HEAD_DIM, PAGE_TOKENS, check, lib
from .weights import PackedWeights, rotary_tables


def _p(t):
    return C.c_void_p(0 if t is None else t.data_ptr())


TC_MIN_ROWS = 9     # rows from which the projections run on the tcgen05 kernel


class DecodeState:
    def __init__(self, weights: PackedWeights, batch: int, prompt_length: int, max_new_tokens: int,
                 group=None, keep_logits: bool = False, tp_path: str = "auto", q_tokens: int = 1,
                 share: "DecodeState | None" = None):
        """tp_path: "auto" (peer memory if every rank can map the others, else NCCL), "peers"
        (the same, but an error if it cannot be used) or "nccl". q_tokens > 1 makes this the
        state of the multi-token verification step (verify()); `share` = a state whose KV pages,
        block table, rotary tables and position this one uses instead of allocating its own."""
        if batch < 1 or prompt_length < 1 or max_new_tokens < 1 or q_tokens < 1:
            raise ValueError("positive batch, prompt length and token count required")
        rows = batch * q_tokens
        if rows > _lib.MAX_ROWS:
            raise ValueError(f"batch {batch} x {q_tokens} tokens exceeds {_lib.MAX_ROWS} rows")
        if tp_path not in ("auto", "peers", "nccl"):
            raise ValueError("tp_path must be 'auto', 'peers' or 'nccl'")
        if q_tokens > 1 and weights.tp_size > 1:
            raise ValueError("the multi-token verification step runs on one GPU")
        self.w = weights
        cfg = weights.cfg
        self.cfg = cfg
        self.group = group
        self.tp = weights.tp_size
        self.shape = (batch, prompt_length, max_new_tokens)
        self.batch = batch
        self.q_tokens = q_tokens
        self.rows = rows
        self.capacity = prompt_length + max_new_tokens + (q_tokens - 1 if share is None else 0)
        if self.capacity > cfg.max_position:
            raise ValueError("prompt + new tokens exceed max_position_embeddings")
        dev = weights.device
        self.device = dev
        nq, nkv, inter = weights.local_q_heads, weights.local_kv_heads, weights.local_inter
        if share is not None:
            if share.batch != batch or share.capacity < self.capacity or share.w is not weights:
                raise ValueError("the shared state has another batch, weights or a smaller capacity")
            self.capacity = share.capacity
            self.pages_per_seq, self.block_table = share.pages_per_seq, share.block_table
            self.kpools, self.vpools = share.kpools, share.vpools
            self.cos, self.sin, self.position = share.cos, share.sin, share.position
        else:
            self.pages_per_seq = (self.capacity + PAGE_TOKENS - 1) // PAGE_TOKENS
            n_pages = batch * self.pages_per_seq
            self.block_table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(batch, -1).contiguous()
            pool = (n_pages, nkv, PAGE_TOKENS, HEAD_DIM)
            self.kpools = [torch.zeros(pool, dtype=torch.bfloat16, device=dev) for _ in range(cfg.n_layers)]
            self.vpools = [torch.zeros(pool, dtype=torch.bfloat16, device=dev) for _ in range(cfg.n_layers)]
            self.cos, self.sin = rotary_tables(cfg, self.capacity, dev)
            self.position = torch.zeros(1, dtype=torch.int32, device=dev)
        self.tokens = torch.zeros(rows, dtype=torch.int64, device=dev)
        self.host = torch.empty(batch, dtype=torch.int64).pin_memory()
        self.status = torch.zeros(4, dtype=torch.int32, device=dev)
        self.host_status = torch.zeros(4, dtype=torch.int32).pin_memory()
        self.ready = torch.cuda.Event()
        self.graph = None
        use_tc = rows >= TC_MIN_ROWS
        if use_tc:
            weights.ensure_tc()           # second tiling of the weights, built once per engine

        ccfg = _lib.Config(cfg.hidden, inter, cfg.n_layers, nq, nkv, weights.local_vocab,
                           weights.vocab_offset, cfg.vocab, self.tp, rows, cfg.rms_eps,
                           float(HEAD_DIM) ** -0.5)
        handle = C.c_void_p()
        check(lib.q_create(C.byref(ccfg), C.byref(handle)))
        self.handle = handle
        for i, lt in enumerate(weights.layers):
            lw = _lib.LayerWeights(lt.wqkv.data_ptr(), lt.wo.data_ptr(), lt.wgu.data_ptr(),
                                   lt.wdown.data_ptr(), lt.ln_in.data_ptr(), lt.ln_post.data_ptr(),
                                   lt.q_gain.data_ptr(), lt.k_gain.data_ptr(),
                                   self.kpools[i].data_ptr(), self.vpools[i].data_ptr(),
                                   *((lt.wqkv.tc().data_ptr(), lt.wo.tc().data_ptr(), lt.wgu.tc().data_ptr(),
                                      lt.wdown.tc().data_ptr()) if use_tc else (0, 0, 0, 0)))
            check(lib.q_bind_layer(handle, i, C.byref(lw)))

        bf = dict(dtype=torch.bfloat16, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        self.x = torch.zeros((rows, cfg.hidden), **bf)
        self.normed = torch.zeros((rows, cfg.hidden), **bf)
        self.q = torch.zeros((rows, nq * HEAD_DIM), **bf)
        self.attended = torch.zeros((rows, nq * HEAD_DIM), **bf)
        self.act = torch.zeros((rows, inter), **bf)
        n_part = lib.q_engine_partial_floats(handle, rows)
        if n_part <= 0:
            raise _lib.QDecodeError("could not size the split-K partial buffer")
        self.partials = torch.empty(n_part, **f32)
        self.reduced = torch.zeros((rows, cfg.hidden), **f32) if self.tp > 1 else None
        self.attn_splits = lib.q_attention_splits(batch, nkv, self.capacity)
        g = nq // nkv
        self.attn_o = torch.empty((batch * nkv, self.attn_splits, q_tokens * g, HEAD_DIM), **f32)
        self.attn_ml = torch.empty((batch * nkv, self.attn_splits, q_tokens * g, 2), **f32)
        self.attn_tickets = torch.zeros(batch * nkv, dtype=torch.int32, device=dev)
        self.logits = torch.zeros((rows, weights.local_vocab), **bf) if keep_logits else None
        self.arg_val = torch.zeros(rows, **f32)
        self.arg_idx = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.arg_scratch = torch.zeros(lib.q_argmax_scratch_bytes(rows, weights.local_vocab),
                                       dtype=torch.uint8, device=dev)
        if self.tp > 1:
            self.gather_val = torch.zeros((self.tp, batch), **f32)
            self.gather_idx = torch.zeros((self.tp, batch), dtype=torch.int32, device=dev)
        st = _lib.State(
            weights.embed.data_ptr(), weights.lm_head.data_ptr(), weights.ln_final.data_ptr(),
            self.cos.data_ptr(), self.sin.data_ptr(), self.tokens.data_ptr(),
            self.position.data_ptr(), self.block_table.data_ptr(), self.pages_per_seq, batch,
            self.attn_splits, q_tokens, self.x.data_ptr(), self.normed.data_ptr(), self.q.data_ptr(),
            self.attended.data_ptr(), self.act.data_ptr(), self.partials.data_ptr(),
            0 if self.reduced is None else self.reduced.data_ptr(), self.attn_o.data_ptr(),
            self.attn_ml.data_ptr(), self.attn_tickets.data_ptr(),
            0 if self.logits is None else self.logits.data_ptr(),
            self.arg_val.data_ptr(), self.arg_idx.data_ptr(), self.arg_scratch.data_ptr(),
            weights.lm_head.tc().data_ptr() if use_tc else 0, self.status.data_ptr())
        check(lib.q_bind_state(handle, C.byref(st)))
        self.uses_tc = use_tc
        self.peers = False
        if self.tp > 1 and tp_path != "nccl":
            if cfg.hidden <= 3072:
                self._bind_peers()
            if tp_path == "peers" and not self.peers:
                raise _lib.QDecodeError("tensor parallel over peer memory was asked for and is unavailable")
        self.tp_path = "single" if self.tp == 1 else ("peers" if self.peers else "nccl")

    def _bind_peers(self) -> None:
        """Allocates this rank's receive area and flag region in symmetric memory and hands the
        peer mappings to the library, so that the two cross-rank sums per layer (and the token
        pick) are exchanged with plain peer stores inside the step's own kernels instead of
        going through collectives. All ranks agree on the outcome; if any of them cannot map the
        others, all keep the NCCL path."""
        import torch.distributed as dist
        group = self.group if self.group is not None else dist.group.WORLD
        ok, err = 1, ""
        try:
            # plain peer loads only: no NVLink multicast object is bound to these buffers
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem
            n = lib.q_engine_peer_floats(self.handle, self.rows)
            if n <= 0:
                raise _lib.QDecodeError("could not size the peer partial buffer")
            buf = symm_mem.empty(n * 4 + lib.q_peer_flag_bytes(), dtype=torch.uint8, device=self.device)
            buf.zero_()
            hdl = symm_mem.rendezvous(buf, group.group_name)
            ptrs = list(hdl.buffer_ptrs)
            if len(ptrs) != self.tp:
                raise _lib.QDecodeError(f"{len(ptrs)} peer mappings for {self.tp} ranks")
        except Exception as exc:            # noqa: BLE001 - any failure means "use the all-reduce path"
            ok, err = 0, f"{type(exc).__name__}: {exc}"
        agreed = torch.tensor([ok], dtype=torch.int32, device=self.device)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
        if int(agreed.item()) == 0:
            if err:
                print(f"[starter_b200] peer-memory tensor parallel unavailable ({err}); using all-reduce",
                      file=sys.stderr)
            return
        peers = _lib.Peers()
        peers.rank, peers.world = dist.get_rank(group), self.tp
        for r in range(self.tp):
            peers.partials[r] = ptrs[r]
            peers.flags[r] = ptrs[r] + n * 4
        self.peer_epoch = torch.zeros(4, dtype=torch.int32, device=self.device)
        peers.epoch = self.peer_epoch.data_ptr()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=group)              # every rank's arrival words are zero from here on
        check(lib.q_bind_peers(self.handle, C.byref(peers)))
        self.peer_buffer, self.peer_handle = buf, hdl
        self.peers = self._peers_self_test(peers, n, group)
        if not self.peers:
            check(lib.q_bind_peers(self.handle, None))
            print("[starter_b200] peer-memory self-test failed; using all-reduce", file=sys.stderr)

    @staticmethod
    def _device_status() -> list:
        out = (C.c_int32 * 4)()
        check(lib.q_device_status(C.byref(out)))
        return list(out)

    def _peers_self_test(self, peers, n_floats: int, group) -> bool:
        """One q_add_rmsnorm_peers call on known data before the path is trusted: every rank
        fills its buffer with (rank+1)/16, so every output element must equal the sum of those
        over the ranks, and no wait may have run out. All ranks agree on the verdict."""
        import torch.distributed as dist
        cfg, dev = self.cfg, self.device
        rank, world = peers.rank, peers.world
        own = torch.full((self.rows, cfg.hidden), (rank + 1) / 16.0, dtype=torch.float32, device=dev)
        zeros = torch.zeros((self.rows, cfg.hidden), dtype=torch.bfloat16, device=dev)
        ones = torch.ones(cfg.hidden, dtype=torch.bfloat16, device=dev)
        total, normed = torch.empty_like(zeros), torch.empty_like(zeros)
        s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        good = True
        for _ in range(2):                       # both halves of the receive area
            rc = lib.q_add_rmsnorm_peers(_p(zeros), C.byref(peers), _p(own), None, _p(ones), _p(total),
                                         _p(normed), self.rows, cfg.hidden, float(cfg.rms_eps), s)
            torch.cuda.synchronize(dev)
            unit = sum(r + 1 for r in range(world)) / 16.0
            good = good and rc == 0 and bool((total.float() == unit).all())
        good = good and self._device_status()[3] == 0
        verdict = torch.tensor([1 if good else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=group)
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)
        return bool(int(verdict.item()))

    def __del__(self):
        h = getattr(self, "handle", None)
        if h:
            lib.q_destroy(h)
            self.handle = None

    # ---- algorithmic bytes of one decode step on this rank (weights + KV) ----
    def step_bytes(self, visible_keys: int) -> int:
        cfg, w = self.cfg, self.w
        per_layer = sum(t.numel() for t in (w.layers[0].wqkv, w.layers[0].wo, w.layers[0].wgu,
                                            w.layers[0].wdown)) * 2
        per_layer += (2 * cfg.hidden + 2 * HEAD_DIM) * 2
        weights = cfg.n_layers * per_layer + w.lm_head.numel() * 2 + cfg.hidden * 2
        kv_token = cfg.n_layers * 2 * w.local_kv_heads * HEAD_DIM * 2
        return weights + kv_token * self.batch * visible_keys + kv_token * self.batch

    # ---- prefill: the prompt pass ----
    PREFILL_ROWS = 2048        # prompt rows processed together (bounds the fp32 partial scratch)

    def _prefill_scratch(self, rows: int):
        """Buffers of the prompt pass for `rows` rows, kept for the next call of the same size."""
        if getattr(self, "_pf", None) is not None and self._pf["rows"] == rows:
            return self._pf
        cfg, w, dev = self.cfg, self.w, self.device
        nq, nkv, inter = w.local_q_heads, w.local_kv_heads, w.local_inter
        plans = {"qkv": _lib.plan(rows, (nq + 2 * nkv) * HEAD_DIM, cfg.hidden, tc=True),
                 "o": _lib.plan(rows, cfg.hidden, nq * HEAD_DIM, tc=True),
                 "gu": _lib.plan(rows, 2 * inter, cfg.hidden, tc=True),
                 "down": _lib.plan(rows, cfg.hidden, inter, tc=True)}
        n_part = max(p.slots * p.M * p.N for p in plans.values())
        bf = dict(dtype=torch.bfloat16, device=dev)
        self._pf = None                    # release the previous size first
        self._pf = {
            "rows": rows, "plans": plans, "partials": torch.empty(n_part, dtype=torch.float32, device=dev),
            "x": torch.empty((rows, cfg.hidden), **bf), "normed": torch.empty((rows, cfg.hidden), **bf),
            "q": torch.empty((rows, nq, HEAD_DIM), **bf), "att": torch.empty((rows, nq * HEAD_DIM), **bf),
            "act": torch.empty((rows, inter), **bf), "zero": torch.zeros(1, dtype=torch.int32, device=dev),
            "reduced": torch.empty((rows, cfg.hidden), dtype=torch.float32, device=dev) if self.tp > 1 else None,
        }
        return self._pf

    def prefill(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Runs the whole prompt, fills the KV pages, leaves the first generated token in
        `tokens` and the prompt length in `position`. Returns the last position's local logits
        [B, V_local].

        The prompt pass of the reference (engine/prefill.py:26-62) on this library's own
        kernels: every projection on the tcgen05 kernel over the tiled weights (256 prompt rows
        per weight pass), embedding + norm, add + norm, SwiGLU and head norm + RoPE + page write
        (engine/kernels/prefill.py:19-63) as the fused consumers of the decode step, the causal
        attention over the prompt as q_attention_prefill reading the pages just written, lm_head
        and argmax likewise; no library kernel runs. Sequences are processed PREFILL_ROWS prompt
        rows at a time. Under tensor
        parallelism the two row-parallel projections are summed over the ranks in fp32 by an
        NCCL all-reduce before the single rounding (the prompt pass is outside the per-step
        path)."""
        cfg, w = self.cfg, self.w
        B, T = input_ids.shape
        if B != self.batch or T != self.shape[1]:
            raise ValueError("prompt shape disagrees with this decode state")
        if input_ids.dtype != torch.int64 or not input_ids.is_cuda:
            raise ValueError("prompt ids must be an int64 CUDA tensor")
        w.ensure_tc()
        nq, nkv, inter = w.local_q_heads, w.local_kv_heads, w.local_inter
        H, eps = cfg.hidden, float(cfg.rms_eps)
        per = max(1, self.PREFILL_ROWS // T)                 # sequences per pass
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        ids = input_ids.contiguous()
        logits = torch.empty((B, w.local_vocab), dtype=torch.bfloat16, device=self.device)
        last = torch.empty((B, H), dtype=torch.bfloat16, device=self.device)
        for b0 in range(0, B, per):
            nb = min(per, B - b0)
            rows = nb * T
            pf = self._prefill_scratch(rows)
            pl, part = pf["plans"], pf["partials"]
            x, normed, act = pf["x"], pf["normed"], pf["act"]
            table = self.block_table.data_ptr() + b0 * self.pages_per_seq * 4
            check(lib.q_embed_rmsnorm(_p(ids[b0:b0 + nb]), _p(w.embed), _p(w.layers[0].ln_in), _p(x), _p(normed),
                                      rows, H, cfg.vocab, eps, stream))
            for i, lt in enumerate(w.layers):
                check(lib.q_gemm_tc(_p(normed), _p(lt.wqkv.tc()), _p(part), rows, pl["qkv"].N, H, stream))
                layout = _lib.KVLayout(self.kpools[i].data_ptr(), self.vpools[i].data_ptr(), table,
                                       self.pages_per_seq, nkv)
                check(lib.q_qkv_norm_rope_cache(_p(part), C.byref(pl["qkv"]), _p(lt.q_gain), _p(lt.k_gain),
                                                _p(self.cos), _p(self.sin), _p(pf["zero"]), _p(pf["q"]),
                                                C.byref(layout), nb, T, nq, eps, stream))
                check(lib.q_attention_prefill(_p(pf["q"]), C.byref(layout), _p(pf["zero"]), _p(pf["att"]),
                                              nb, T, nq, float(HEAD_DIM) ** -0.5, stream))
                check(lib.q_gemm_tc(_p(pf["att"]), _p(lt.wo.tc()), _p(part), rows, H, nq * HEAD_DIM, stream))
                self._prefill_add_norm(pf, pl["o"], lt.ln_post, rows, stream)
                check(lib.q_gemm_tc(_p(normed), _p(lt.wgu.tc()), _p(part), rows, 2 * inter, H, stream))
                check(lib.q_swiglu(_p(part), C.byref(pl["gu"]), _p(act), rows, inter, stream))
                check(lib.q_gemm_tc(_p(act), _p(lt.wdown.tc()), _p(part), rows, H, inter, stream))
                gain = w.layers[i + 1].ln_in if i + 1 < len(w.layers) else w.ln_final
                self._prefill_add_norm(pf, pl["down"], gain, rows, stream)
            last[b0:b0 + nb].copy_(normed.view(nb, T, H)[:, -1])
        # lm_head on the last position of every sequence, logits rounded once to bf16
        hp = _lib.plan(B, w.local_vocab, H, tc=True)
        head_part = torch.empty((hp.slots, B, w.local_vocab), dtype=torch.float32, device=self.device)
        check(lib.q_gemm_tc(_p(last), _p(w.lm_head.tc()), _p(head_part), B, w.local_vocab, H, stream))
        val = torch.empty(B, dtype=torch.float32, device=self.device)
        idx = torch.empty(B, dtype=torch.int32, device=self.device)
        scratch = torch.zeros(lib.q_argmax_scratch_bytes(B, w.local_vocab), dtype=torch.uint8, device=self.device)
        check(lib.q_logits_argmax(_p(head_part), C.byref(hp), _p(logits), _p(val), _p(idx),
                                  _p(self.tokens) if self.tp == 1 else None, None, 0, _p(scratch), B,
                                  w.local_vocab, w.vocab_offset, stream))
        if self.tp > 1:
            gv = torch.empty((self.tp, B), dtype=torch.float32, device=self.device)
            gi = torch.empty((self.tp, B), dtype=torch.int32, device=self.device)
            torch.distributed.all_gather_into_tensor(gv, val, group=self.group)
            torch.distributed.all_gather_into_tensor(gi, idx, group=self.group)
            check(lib.q_argmax_merge(_p(gv), _p(gi), self.tp, B, _p(self.tokens), None, 0, stream))
        self.position.fill_(T)
        return logits

    def _prefill_add_norm(self, pf, plan, gain, rows: int, stream) -> None:
        """x, normed <- add + RMSNorm of the projection partials in pf['partials'] (summed over
        the tensor-parallel ranks first, in fp32)."""
        H, eps = self.cfg.hidden, float(self.cfg.rms_eps)
        x, normed, part = pf["x"], pf["normed"], pf["partials"]
        if self.tp == 1:
            check(lib.q_add_rmsnorm(_p(x), _p(part), C.byref(plan), _p(gain), _p(x), _p(normed), rows, H, eps, stream))
            return
        check(lib.q_reduce_partials(_p(part), C.byref(plan), _p(pf["reduced"]), stream))
        torch.distributed.all_reduce(pf["reduced"], group=self.group)
        check(lib.q_add_rmsnorm(_p(x), _p(pf["reduced"]), None, _p(gain), _p(x), _p(normed), rows, H, eps, stream))

    # ---- one decode step (the hot path) ----
    def step(self) -> None:
        s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        h = self.handle
        if self.q_tokens > 1:
            raise ValueError("this state runs verify(), not step()")
        if self.tp == 1:
            check(lib.q_decode_step(h, s))
            return
        if self.peers:
            check(lib.q_decode_step_peers(h, s))      # every cross-rank exchange goes through peer memory
            return
        check(lib.q_step_begin(h, s))
        for layer in range(self.cfg.n_layers):
            check(lib.q_step_attn(h, layer, s))
            torch.distributed.all_reduce(self.reduced, group=self.group)
            check(lib.q_step_post_attn(h, layer, s))
            torch.distributed.all_reduce(self.reduced, group=self.group)
            check(lib.q_step_post_mlp(h, layer, s))
        check(lib.q_step_head(h, s))
        torch.distributed.all_gather_into_tensor(self.gather_val, self.arg_val, group=self.group)
        torch.distributed.all_gather_into_tensor(self.gather_idx, self.arg_idx, group=self.group)
        check(lib.q_step_merge(h, _p(self.gather_val), _p(self.gather_idx), s))

    def verify(self, candidates: torch.Tensor) -> torch.Tensor:
        """The multi-token verification step: candidates int64 [batch, T] (device) sit at
        positions position .. position + T - 1; returns int32 [batch, T], the greedy successor of
        every candidate's prefix. Neither tokens nor position advance."""
        if candidates.shape != (self.batch, self.q_tokens) or candidates.dtype != torch.int64:
            raise ValueError(f"candidates must be int64 [{self.batch}, {self.q_tokens}]")
        self.tokens.copy_(candidates.reshape(-1))
        check(lib.q_verify_step(self.handle, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return self.arg_idx.view(self.batch, self.q_tokens)

    def capture(self) -> None:
        """Warm-up steps on a side stream, then one step recorded as a CUDA graph; tokens and
        position are put back afterwards (engine/decode.py:130-148 does the same around its
        capture). Warm-up writes land in KV slots at or after the current position, which the
        real steps overwrite before they read them. Under tensor parallelism over peer memory
        the call counters of the exchange kernels advance in the warm-up steps on every rank
        alike, so the recorded step continues the same sequence."""
        saved = (self.tokens.clone(), self.position.clone())

        def restore():
            self.tokens.copy_(saved[0])
            self.position.copy_(saved[1])

        launch_stream = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(launch_stream)
        with torch.cuda.stream(side):
            for _ in range(3):
                restore()
                self.step()
            restore()
        launch_stream.wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            self.step()
        restore()
        self.graph = graph

    def advance(self) -> None:
        if self.graph is None:
            self.step()
        else:
            self.graph.replay()

    def check_status(self, words) -> None:
        """Raises when a bounded wait inside a kernel ran out (the status words are sticky
        until q_clear_status): what such a step computed is not to be trusted."""
        if any(words):
            names = ("attention", "stream-K GEMM", "tcgen05 GEMM", "tensor-parallel peer exchange")
            what = ", ".join(f"{n} (code {w})" for n, w in zip(names, words) if w)
            raise _lib.QDecodeError(f"qdecode status {_lib.ERR_DEVICE}: a bounded wait inside a kernel ran out: {what}")

    def emit(self, max_new_tokens: int):
        """Yields one host list per output step; exactly max_new_tokens - 1 decode steps run
        (engine/decode.py:110-128). The device-to-host copy of step k (tokens and the status
        words its last kernel left) is enqueued before step k + 1 is launched, and awaited
        after."""
        self.status.zero_()          # what an earlier call left; a word that is still set comes back with the first step
        for step in range(max_new_tokens):
            self.host.copy_(self.tokens, non_blocking=True)
            self.host_status.copy_(self.status, non_blocking=True)
            self.ready.record()
            if step + 1 < max_new_tokens:
                self.advance()
            self.ready.synchronize()
            self.check_status(self.host_status.tolist())
            yield self.host.tolist()
