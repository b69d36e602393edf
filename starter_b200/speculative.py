"""Exact-verification speculative decoding on top of the multi-token verification step.

The reference records the idea (AGENTS.md:93-95: draft cheaply, verify several tokens in one
pass over the weights, keep only what greedy decoding would have produced) and logs one
attempt (agent/experiments.jsonl:34-36). Here the verification pass is q_verify_step: T
candidate tokens per sequence go through all layers as batch * T rows of the same
projections, with the small-query attention kernel seeing keys `< position + t + 1` for row
t. Output is exact by construction: a drafted token is kept only if it equals the greedy
successor of the prefix before it, and the first token that differs is replaced by that
successor.

Drafts come from prompt lookup (the continuation of the most recent earlier occurrence of
the last one or two tokens in the sequence's own history): no second model. All sequences
of a batch share one position counter, so a round keeps the shortest accepted prefix of the
batch.
"""
from __future__ import annotations

import torch

from .decode import DecodeState


def lookup_draft(history: list[int], count: int) -> list[int]:
    """Up to `count` tokens that followed the latest earlier occurrence of the history's last
    two tokens (else of its last token); padded with the last token."""
    out: list[int] = []
    for n in (2, 1):
        if len(history) <= n:
            continue
        key = history[-n:]
        for start in range(len(history) - n - 1, -1, -1):
            if history[start:start + n] == key:
                out = history[start + n:start + n + count]
                break
        if out:
            break
    return (out + [history[-1]] * count)[:count]


def generate_speculative(engine, input_ids: list[list[int]], max_new_tokens: int, draft_tokens: int = 4):
    """Greedy continuation of every sequence, identical to Engine.generate's tokens, produced
    `draft_tokens` candidates at a time. Returns (steps, stats): steps is the list
    Engine.generate would have yielded (one list of batch ids per output step)."""
    if max_new_tokens <= 0:
        return [], {"verify_calls": 0, "emitted": 0, "accepted_drafts": 0}
    T = int(draft_tokens)
    weights = engine.weights
    with torch.inference_mode(), torch.cuda.device(engine.device):
        host = torch.tensor(input_ids, dtype=torch.int64)
        if host.ndim != 2 or host.shape[0] < 1 or host.shape[1] < 1:
            raise ValueError("input_ids must be a non-empty list of equal-length id lists")
        batch, length = host.shape
        state = DecodeState(weights, batch, length, max_new_tokens + T, group=None)
        verifier = DecodeState(weights, batch, length, max_new_tokens + T, q_tokens=T, share=state)
        state.prefill(host.to(engine.device))
        current = state.tokens.cpu().tolist()
        history = [list(row) + [tok] for row, tok in zip(input_ids, current)]
        steps = [list(current)]
        position = length
        calls = accepted = 0
        while len(steps) < max_new_tokens:
            drafts = [lookup_draft(h, T - 1) for h in history]
            cand = torch.tensor([[c] + d for c, d in zip(current, drafts)], dtype=torch.int64)
            successors = verifier.verify(cand.to(engine.device)).cpu().tolist()
            verifier.check_status(verifier.status.cpu().tolist())
            calls += 1
            keep = T - 1
            for d, nxt in zip(drafts, successors):
                n = 0
                while n < T - 1 and d[n] == nxt[n]:
                    n += 1
                keep = min(keep, n)
            accepted += keep
            for i in range(keep + 1):
                if len(steps) == max_new_tokens:
                    break
                step = [nxt[i] for nxt in successors]
                steps.append(step)
                for h, tok in zip(history, step):
                    h.append(tok)
            position += keep + 1
            current = [nxt[keep] for nxt in successors]
            state.position.fill_(position)
        return steps, {"verify_calls": calls, "emitted": len(steps), "accepted_drafts": accepted,
                       "tokens_per_call": (len(steps) - 1) / max(1, calls)}
