"""The per-step plan of the mixers whose attention runs over flat-page caches (`Kernels.attention_flat`): the step's tokens cut
into runs of neighbouring tokens of one request, as many as one block of the tensor-core kernel takes beside the heads of a
key/value group, and, for a step of single decoded tokens, over how many blocks each run's keys are shared out.

Layers with equal head counts, sizes and window share one plan per step (`prepare_key`)."""
from __future__ import annotations

from .base import StepPlan


def flat_prepare_key(heads, kv_heads, key_dim, value_dim, window) -> str:
    return f"flat_attention.{heads}.{kv_heads}.{key_dim}.{value_dim}.{window}"


def plan_flat_tiles(kernels, shape, heads, kv_heads, key_dim, value_dim, window, shared_value=False):
    """StepPlan with `tiles` (first token row, tokens, position of the first, request) and `.splits`, or None when the
    kernel set plans nothing (it then walks a row per warp)."""
    per_tile = getattr(kernels, "flat_tokens_per_tile", None)
    if per_tile is None:
        return None
    run = per_tile(heads, kv_heads)
    tiles, row, longest = [], 0, 0
    for b, (n, total) in enumerate(zip(shape.query_lens, shape.seq_lens)):
        for s in range(0, n, run):
            tiles += [row + s, min(run, n - s), total - n + s, b]
        row += n
        longest = max(longest, min(total, window + n - 1) if window > 0 else total)
    splits = 1
    if shape.num_tokens == len(shape.query_lens):
        # single decoded tokens: few blocks, long key ranges.  The longest range is rounded up to 512 keys, so that a captured
        # graph (which freezes the count) serves the steps while contexts grow.
        splits = kernels.flat_key_splits(len(shape.query_lens), heads, kv_heads, key_dim, value_dim, shared_value,
                                         -(-longest // 512) * 512)
    plan = StepPlan(arrays={"tiles": tiles}, graph_key=(splits,))
    plan.splits = splits
    return plan
