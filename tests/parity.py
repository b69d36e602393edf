"""Helpers shared by the GPU parity tests."""
import torch


def sum_slots(partials):
    """CPU re-statement of how consumers add split-K slots: for every column the
    first count(group) slots, in slot order (fp32)."""
    p = partials.plan
    data = partials.data.detach().cpu()
    Cg, u = p.chunks_per_group, p.units_per_worker
    g = (torch.arange(p.N) // p.group_rows)[None, :].repeat(p.M, 1)
    if p.group_rows == 128 and p.M > 256:
        # the tcgen05 plan of more than 256 rows counts its groups per row chunk of 256
        g = g + (torch.arange(p.M) // 256)[:, None] * ((p.N + 127) // 128)
    cnt = ((g + 1) * Cg - 1) // u - (g * Cg) // u + 1
    total = torch.zeros((p.M, p.N), dtype=torch.float32)
    for k in range(p.slots):
        total += torch.where(k < cnt, data[k], torch.zeros(()))
    return total


def bit_equal_fraction(a, b):
    return float((a.view(torch.int16) == b.view(torch.int16)).float().mean())


def own_prefix_report(native, prompt, emitted, engine_logits=None):
    """Teacher-forces the engine's own tokens through the native model (no cache)
    and returns, per step, the max-abs logit diff (if engine logits are given)
    and the gap between the native top logit and the native logit of the emitted
    token (0 when they agree)."""
    from oracle import qwen3_oracle as O
    ref = O.native_teacher_forced_logits(native, prompt, emitted)       # [N, B, V]
    em = torch.as_tensor(emitted)
    gaps = ref.max(-1).values - ref.gather(-1, em[..., None])[..., 0]
    diffs = None
    if engine_logits is not None:
        diffs = (engine_logits.float().cpu() - ref).abs().amax(-1)
    return ref, gaps, diffs
