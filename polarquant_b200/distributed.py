"""Sharding of the polar decode path over the GPUs of one node (one process per GPU, torch.distributed).

The units of the path - (batch, kv head) pairs - are independent: each owns its codes, scales, residual keys and
values and produces its own query heads' outputs.  Sharding by batch or by kv head therefore needs no collective
in the attention step (`shard_range`).  Only a split along the sequence has an exchange: every rank attends over
its slice of the keys, the ranks all-gather one fp32 (output, log-sum-exp) pair per query head, and each merges
locally (`sequence_parallel_decode`).  The reference has no counterpart: it runs one full model replica per GPU
(`test4long.py:38-43`) and never splits the sequence.

Kernels only ever read local memory; the remote partials arrive through the all-gather first.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced [begin, end) of `total` items for `rank` (sizes differ by at most one)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    return (rank * total) // world, ((rank + 1) * total) // world


def split_sequence(num_groups: int, residual: int, rank: int, world: int):
    """Key range of `rank` in a sequence split: whole token groups [g0, g1), and whether this rank also owns the
    full-precision residual window (the last rank that has any work does)."""
    g0, g1 = shard_range(num_groups, rank, world)
    owner = world - 1
    return g0, g1, (residual > 0 and rank == owner)


def _default_attend(q, kres, packed, v, **kw):
    from .ops import decode_attention
    return decode_attention(q, kres, *packed, v, out_dtype=torch.float32, return_lse=True, **kw)


def _default_merge(outs, lses, out_dtype):
    from .ops import merge_lse
    return merge_lse(outs, lses, out_dtype=out_dtype)


def local_partial(q, kres, packed, v, attend=None, **kw):
    """(output fp32 (B, N, 128), natural-log lse (B, N)) of attention over this rank's keys.
    A rank without keys contributes zeros with lse = -inf, which the merge weights by zero."""
    attend = attend or _default_attend
    have_q = packed is not None and packed[0] is not None and packed[0].shape[2] > 0
    have_r = kres is not None and kres.shape[2] > 0
    if not have_q and not have_r:
        b, n, _, hd = q.shape
        return (torch.zeros(b, n, hd, dtype=torch.float32, device=q.device),
                torch.full((b, n), float("-inf"), dtype=torch.float32, device=q.device))
    if not have_q:
        packed = (None,) * 5
    out, lse = attend(q, kres if have_r else None, packed, v, **kw)
    return out[:, :, 0].to(torch.float32), lse


def merge_across_ranks(out, lse, group=None, out_dtype=torch.float32, merge=None):
    """All-gather every rank's (out, lse) and merge them locally; every rank returns the full result."""
    merge = merge or _default_merge
    world = dist.get_world_size(group)
    b, n, hd = out.shape
    # one message per rank: [out | lse] packed so a single collective carries both
    mine = torch.cat([out.reshape(b * n, hd), lse.reshape(b * n, 1)], dim=1).contiguous()
    gathered = torch.empty((world * b * n, hd + 1), dtype=torch.float32, device=out.device)
    dist.all_gather_into_tensor(gathered, mine, group=group)      # rank r's rows land at [r*b*n, (r+1)*b*n)
    gathered = gathered.reshape(world, b * n, hd + 1)
    outs = gathered[:, :, :hd].reshape(world, b, n, hd)
    lses = gathered[:, :, hd].reshape(world, b, n)
    return merge(outs.contiguous(), lses.contiguous(), out_dtype)


def sequence_parallel_decode(q, kres, packed, v, group=None, out_dtype=None, attend=None, merge=None, **kw):
    """Decode attention with the keys split along the sequence across the ranks of `group`.

    Each rank passes ITS slice: `packed` = codes/scales of its token groups (or None), `kres` = the residual keys on
    the rank that owns them (else None), `v` = the values of exactly those keys, in order.  Returns (B, N, 1, 128)
    in `out_dtype` (default: the query dtype) on every rank.

    With the default CUDA entry points the step is four launches: the attention kernel and its merge write this
    rank's fp32 output and log-sum-exp straight into one exchange block [out (B N, 128) | lse (B N)], one
    all-gather moves every rank's block, and one merge kernel reads the gathered buffer in place.
    """
    if attend is not None or merge is not None:          # injected compute (CPU tests): the generic path
        out, lse = local_partial(q, kres, packed, v, attend=attend, **kw)
        full = merge_across_ranks(out, lse, group=group, out_dtype=out_dtype or q.dtype, merge=merge)
        return full[:, :, None, :]
    from . import ops
    world = dist.get_world_size(group)
    b, n, _, hd = q.shape
    rows = b * n
    mine = torch.empty(rows * (hd + 1), dtype=torch.float32, device=q.device)
    out_view = mine[:rows * hd].view(b, n, 1, hd)
    lse_view = mine[rows * hd:].view(b, n)
    have_q = packed is not None and packed[0] is not None and packed[0].shape[2] > 0
    have_r = kres is not None and kres.shape[2] > 0
    if not have_q and not have_r:                        # a rank without keys: weight zero in the merge
        out_view.zero_()
        lse_view.fill_(float("-inf"))
    else:
        ops.decode_attention(q, kres if have_r else None, *(packed if have_q else (None,) * 5), v,
                             out_dtype=torch.float32, out=out_view, lse_out=lse_view, **kw)
    gathered = torch.empty(world * mine.numel(), dtype=torch.float32, device=q.device)
    dist.all_gather_into_tensor(gathered, mine, group=group)
    return ops.merge_lse_gathered(gathered, world, rows, out_dtype=out_dtype or q.dtype, out_shape=(b, n, 1, hd))
