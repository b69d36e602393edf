"""B200-native greedy decode engine for the Qwen3 architecture.

`Engine` keeps the reference's `Engine(model_path)` / `generate(input_ids,
max_new_tokens)` contract; `ops` exposes the per-operator entry points. All
compute goes through libqdecode.so (include/qdecode.h)."""
from .engine import Engine  # noqa: F401

__all__ = ["Engine"]
