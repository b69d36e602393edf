"""Host-side agreement between tensor-parallel ranks: every rank learns of a failure on
any rank BEFORE the next kernel or collective is launched, and raises the same error.

The reference is single-GPU; its habit carried over here is to validate before every launch
and never to fall back silently (engine/kernels/decode_fused.py:183-203). Under tensor
parallelism a rank that failed alone would leave the others waiting inside a collective or a
peer exchange, so failures are made collective on the host: a rank that raised, a rank whose
shard has the wrong shape and a rank that never arrived are all detected with plain
process-group calls (they work on the gloo backend too) and surface on every rank as
TensorParallelError naming the ranks at fault.
"""
from __future__ import annotations

import time

import torch
import torch.distributed as dist


class TensorParallelError(RuntimeError):
    """A tensor-parallel rank failed; raised on EVERY rank of the group."""


def _flag_device(group, device):
    if device is not None:
        return device
    return torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")


def failed_ranks(group, ok: bool, device=None) -> list[int]:
    """All-gathers one flag per rank; returns the ranks that reported a failure."""
    world = dist.get_world_size(group)
    mine = torch.tensor([0 if ok else 1], dtype=torch.int32, device=_flag_device(group, device))
    flags = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(flags, mine, group=group)
    return [r for r, f in enumerate(flags) if int(f.item())]


def guarded(group, fn, what: str, device=None):
    """Runs fn() on this rank, then makes the outcome collective: if it raised on any rank,
    every rank raises TensorParallelError (the rank at fault chains its own exception)."""
    error = None
    result = None
    try:
        result = fn()
    except Exception as exc:            # noqa: BLE001 - reported to every rank below
        error = exc
    bad = failed_ranks(group, error is None, device)
    if bad:
        msg = f"{what} failed on rank(s) {bad} of {dist.get_world_size(group)}"
        if error is not None:
            raise TensorParallelError(f"{msg}: {type(error).__name__}: {error}") from error
        raise TensorParallelError(msg)
    return result


def shard_signature(weights) -> list[int]:
    """What must be equal on every rank (model and world size) and what must follow from the
    rank (vocabulary offset): checked by check_shards."""
    cfg = weights.cfg
    return [cfg.hidden, cfg.inter, cfg.n_layers, cfg.n_q_heads, cfg.n_kv_heads, cfg.vocab, weights.tp_size,
            weights.local_q_heads, weights.local_kv_heads, weights.local_inter, weights.local_vocab,
            weights.vocab_offset - weights.tp_rank * weights.local_vocab]


def check_shards(group, weights, device=None) -> None:
    """Every rank must hold a shard of the same model cut for the same world size. A rank that
    loaded another checkpoint, or the unsharded model, would make the cross-rank sums
    meaningless without any kernel noticing."""
    world = dist.get_world_size(group)
    mine = torch.tensor(shard_signature(weights), dtype=torch.int64, device=_flag_device(group, device))
    sigs = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(sigs, mine, group=group)
    sigs = [s.cpu().tolist() for s in sigs]
    problems = []
    if weights.tp_size != world:
        problems.append(f"rank {dist.get_rank(group)} was sharded for {weights.tp_size} ranks, the group has {world}")
    for r, s in enumerate(sigs):
        if s != sigs[0]:
            problems.append(f"rank {r} holds {s}, rank 0 holds {sigs[0]}")
    bad = failed_ranks(group, not problems, device)
    if bad or problems:
        raise TensorParallelError("tensor-parallel shards disagree: " + ("; ".join(problems) or f"see rank(s) {bad}"))


def join_or_fail(store, rank: int, world: int, tag: str, timeout_s: float) -> None:
    """Arrival check through the rendezvous store (no collective, so a rank that is missing
    cannot hang the others): every rank posts a key and waits up to timeout_s for all of them;
    whoever is missing is named in the error."""
    store.set(f"{tag}/joined/{rank}", b"1")
    deadline = time.monotonic() + timeout_s
    missing = list(range(world))
    while missing and time.monotonic() < deadline:
        missing = [r for r in missing if not store.check([f"{tag}/joined/{r}"])]
        if missing:
            time.sleep(0.02)
    if missing:
        raise TensorParallelError(f"rank(s) {missing} of {world} did not arrive at '{tag}' within {timeout_s:.1f} s")
