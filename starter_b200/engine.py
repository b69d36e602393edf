"""Drop-in engine: `Engine(model_path)` and the generator
`generate(input_ids, max_new_tokens)`, the contract of the reference's
engine/engine.py:24-69. Everything per decode step runs in libqdecode.so.
"""
from __future__ import annotations

import torch

from .decode import DecodeState
from .weights import load_checkpoint


class Engine:
    def __init__(self, model_path: str, device: str | None = None, group=None,
                 keep_logits: bool = False, tp_path: str = "auto") -> None:
        """Loads config.json + safetensors from model_path onto one GPU (or, with a
        torch.distributed process group, this rank's tensor-parallel shard). tp_path picks how
        the ranks exchange their partial sums: "auto" = through peer memory where every rank can
        map the others, else NCCL; "peers" = peer memory or an error; "nccl"."""
        if not torch.cuda.is_available():
            raise RuntimeError("starter_b200.Engine needs a CUDA device; there is no CPU path")
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        self.group = group
        if group is not None:
            self.tp_rank = torch.distributed.get_rank(group)
            self.tp_size = torch.distributed.get_world_size(group)
        else:
            self.tp_rank, self.tp_size = 0, 1
        self.device = torch.device(device or f"cuda:{torch.cuda.current_device()}")
        self.keep_logits = keep_logits
        self.tp_path = tp_path
        with torch.inference_mode():
            if group is None:
                self.weights = load_checkpoint(model_path, self.device, 0, 1)
            else:
                # a rank that cannot load, or that holds another model's shard, is reported on
                # every rank here, before any cross-rank kernel is launched
                from . import tp
                self.weights = tp.guarded(group, lambda: load_checkpoint(model_path, self.device, self.tp_rank,
                                                                         self.tp_size),
                                          "loading the checkpoint shard", self.device)
                tp.check_shards(group, self.weights, self.device)
        self.decode_state: DecodeState | None = None

    def generate(self, input_ids: list[list[int]], max_new_tokens: int):
        """Greedy continuation of every sequence, one step at a time.

        Yields a list with one token id per sequence for each output step, exactly
        max_new_tokens times. Every sequence has the same length. Never stops at
        end-of-sequence tokens."""
        if max_new_tokens <= 0:
            return
        with torch.inference_mode(), torch.cuda.device(self.device):
            host = torch.tensor(input_ids, dtype=torch.int64)
            if host.ndim != 2 or host.shape[0] < 1 or host.shape[1] < 1:
                raise ValueError("input_ids must be a non-empty list of equal-length id lists")
            prompt = host.pin_memory().to(self.device, non_blocking=True)
            shape = (prompt.shape[0], prompt.shape[1], max_new_tokens)
            if self.decode_state is None or self.decode_state.shape != shape:
                self.decode_state = None
                self.decode_state = DecodeState(self.weights, *shape, group=self.group,
                                                keep_logits=self.keep_logits, tp_path=self.tp_path)
            state = self.decode_state
            state.prefill(prompt)
            if max_new_tokens > 1 and state.graph is None:
                state.capture()
            yield from state.emit(max_new_tokens)
