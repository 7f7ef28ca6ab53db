"""The one exchange step of the path: gathering per-rank partial attention records of a KV-range-sharded sequence.

Works on whatever backend the process group has (NCCL on GPUs, gloo on CPU): the tensors are [n][32][130] fp32
records {acc[128], m, l} per head, 16 640 bytes per token and rank, so the collective is latency-bound.
"""
from __future__ import annotations


def gather_partials(partial, group=None):
    """all-gather [n, 32, 130] -> [world, n, 32, 130] (rank-major, the layout flint_attn_combine_dev takes)."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    partial = partial.contiguous()
    out = torch.empty((world * partial.shape[0],) + tuple(partial.shape[1:]), dtype=partial.dtype, device=partial.device)
    dist.all_gather_into_tensor(out, partial, group=group)
    return out.view((world,) + tuple(partial.shape))
