"""Sharding of the polar decode path over the GPUs of one node (one process per GPU, torch.distributed).

The units of the path - (batch, kv head) pairs - are independent: each owns its codes, scales, residual keys and
values and produces its own query heads' outputs.  Sharding by batch or by kv head therefore needs no collective
in the attention step (`shard_range`).  Only a split along the sequence has an exchange: every rank attends over
its slice of the keys, the ranks all-gather one fp32 (output, log-sum-exp) pair per query head, and each merges
locally (`sequence_parallel_decode`).  The reference has no counterpart: it runs one full model replica per GPU
(`test4long.py:38-43`) and never splits the sequence.

Two forms of that exchange exist.  The default one moves the partials with one NCCL all-gather and merges the
gathered buffer with one kernel; kernels then only ever touch local memory.  With a `PeerExchange` the attention
call does the exchange itself: the kernel that ends it stores this rank's partial into every peer's buffer over
NVLink (plain peer-to-peer stores, each value paired with the step's epoch), waits for the peers' stores in local
memory - every wait bounded - and merges; the results are bit-identical.
"""
from __future__ import annotations

import ctypes

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


class _DeviceBlock:
    """Exposes a raw device allocation to torch (``torch.as_tensor``) without copying."""

    def __init__(self, ptr: int, nfloats: int):
        self.__cuda_array_interface__ = {"shape": (nfloats,), "typestr": "<f4", "data": (ptr, False), "version": 2}


class PeerExchange:
    """Exchange buffers of the one-kernel sequence split for a fixed number of (batch x head) rows.

    Construction is collective over `group`: every rank allocates its buffer through the library
    (``pq_peer_alloc``), the 64-byte handles travel by ``all_gather_object``, and each rank maps the peers' buffers
    (``pq_peer_open``).  ``out_view`` / ``lse_view`` are this rank's block - ``decode_attention(out=, lse_out=,
    push_to=self, collect_out=...)`` writes it, pushes it and merges the peers' blocks - and ``merge`` enqueues the
    stand-alone push / wait / merge kernel (a rank without keys in a step; the staged forms).  Call ``close`` on every
    rank after the last step (it is collective too: a barrier first, so that no peer is still storing into a buffer
    that is freed).
    """

    def __init__(self, batch: int, heads: int, group=None, device=None, head_dim: int = 128):
        from . import _lib
        if head_dim != 128:
            raise ValueError("head_dim must be 128")
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.batch, self.heads, self.rows = batch, heads, batch * heads
        self.device = torch.device(device if device is not None else torch.device("cuda", torch.cuda.current_device()))
        self._lib = _lib.load()
        self.nbytes = self._lib.pq_exchange_bytes(self.world, self.rows, head_dim)
        if self.nbytes <= 0:
            raise ValueError("PeerExchange: at most 8 ranks, at least one row")
        self._ptrs = [None] * self.world
        handle = ctypes.create_string_buffer(_lib.PQ_IPC_HANDLE_BYTES)
        mine = ctypes.c_void_p()
        # Every collective below is executed by every rank whatever happened locally, so that a failure on one rank
        # (no peer access, allocation refused) surfaces as the same exception everywhere instead of a stuck barrier.
        with torch.cuda.device(self.device):
            rc = self._lib.pq_peer_alloc(self.nbytes, ctypes.byref(mine), handle)
            handles = [None] * self.world
            dist.all_gather_object(handles, (rc, handle.raw), group=group)
            failed = [r for r, (code, _) in enumerate(handles) if code != 0]
            opened = []
            if not failed:
                self._ptrs[self.rank] = mine.value
                for r, (_, h) in enumerate(handles):
                    if r == self.rank:
                        continue
                    peer = ctypes.c_void_p()
                    rc = self._lib.pq_peer_open(h, ctypes.byref(peer))
                    if rc != 0:
                        break
                    self._ptrs[r] = peer.value
                    opened.append(peer.value)
            torch.cuda.synchronize(self.device)
            mapped = [None] * self.world
            dist.all_gather_object(mapped, rc, group=group)
            if failed or any(code != 0 for code in mapped):
                for ptr in opened:
                    self._lib.pq_peer_close(ptr)
                dist.barrier(group=group)
                if mine.value:
                    self._lib.pq_peer_free(mine.value)
                raise RuntimeError(f"PeerExchange: peer memory unavailable (allocation status per rank "
                                   f"{[code for code, _ in handles]}, mapping status per rank {mapped})")
        dist.barrier(group=group)          # every buffer exists, is zeroed and is mapped before anyone stores into it
        self._bufs = (ctypes.c_void_p * self.world)(*self._ptrs)
        slot = self._lib.pq_exchange_slot_offset(self.world, self.rows, head_dim, self.rank)
        self._block = _DeviceBlock(self._ptrs[self.rank] + slot, self.rows * (head_dim + 1))
        flat = torch.as_tensor(self._block, device=self.device)
        self.out_view = flat[:self.rows * head_dim].view(batch, heads, 1, head_dim)
        self.lse_view = flat[self.rows * head_dim:].view(batch, heads)
        self._closed = False

    def merge(self, out_dtype=torch.float32, out: torch.Tensor | None = None,
              after_attention: bool = False, pushed: bool = False) -> torch.Tensor:
        """Push this rank's slot to the peers, wait for theirs, merge: (B, N, 1, 128) in `out_dtype`.
        `after_attention`: the call directly follows the ``decode_attention`` that wrote the slot, on the same
        stream - the kernel is then launched as a programmatic dependent of that call's merge.
        `pushed`: that ``decode_attention`` call was given ``push_to=self`` and has pushed the slot already."""
        from . import _lib
        from .ops import _DT, _on_device, _stream
        if out is None:
            out = torch.empty((self.batch, self.heads, 1, 128), dtype=out_dtype, device=self.device)
        elif out.dtype != out_dtype or not out.is_contiguous() or out.numel() != self.rows * 128:
            raise ValueError("out must be contiguous, of out_dtype, with batch * heads * 128 elements")
        with _on_device(self.device):
            rc = self._lib.pq_exchange_merge(self._bufs, self.world, self.rank, self.rows, 128, out.data_ptr(),
                                             _DT[out_dtype], None,
                                             (_lib.PQ_EXCHANGE_AFTER_ATTENTION if after_attention else 0)
                                             | (_lib.PQ_EXCHANGE_PUSHED if pushed else 0), _stream(self.device))
        _lib.check(rc, "pq_exchange_merge")
        return out

    def status(self) -> int:
        """0, or the bits the kernel set when a wait on a peer ran out (synchronises the stream)."""
        from . import _lib
        from .ops import _on_device, _stream
        word = ctypes.c_uint(0)
        with _on_device(self.device):
            rc = self._lib.pq_exchange_status(self._ptrs[self.rank], self.world, self.rows, 128, ctypes.byref(word),
                                              _stream(self.device))
        _lib.check(rc, "pq_exchange_status")
        return int(word.value)

    def close(self):
        from . import _lib
        if self._closed:
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.out_view = self.lse_view = None
        with torch.cuda.device(self.device):
            for r, ptr in enumerate(self._ptrs):
                if r != self.rank:
                    _lib.check(self._lib.pq_peer_close(ptr), "pq_peer_close")
            dist.barrier(group=self.group)     # nobody maps this buffer any more
            _lib.check(self._lib.pq_peer_free(self._ptrs[self.rank]), "pq_peer_free")


def sequence_parallel_decode(q, kres, packed, v, group=None, out_dtype=None, attend=None, merge=None, exchange=None,
                             push_in_attention=True, collect_in_attention=True, **kw):
    """Decode attention with the keys split along the sequence across the ranks of `group`.

    Each rank passes ITS slice: `packed` = codes/scales of its token groups (or None), `kres` = the residual keys on
    the rank that owns them (else None), `v` = the values of exactly those keys, in order.  Returns (B, N, 1, 128)
    in `out_dtype` (default: the query dtype) on every rank.

    With the default CUDA entry points the step is four launches: the attention kernel and its merge write this
    rank's fp32 output and log-sum-exp straight into one exchange block [out (B N, 128) | lse (B N)], one
    all-gather moves every rank's block, and one merge kernel reads the gathered buffer in place.  With
    ``exchange=PeerExchange(batch, heads, group)`` the attention's own merge also stores the block into the peers'
    buffers over NVLink, waits for the peers' blocks and merges: the step is the attention call alone, two launches
    (``collect_in_attention=False``: a separate kernel collects and merges; ``push_in_attention=False``: that kernel
    also does the stores).
    """
    if attend is not None or merge is not None:          # injected compute (CPU tests): the generic path
        out, lse = local_partial(q, kres, packed, v, attend=attend, **kw)
        full = merge_across_ranks(out, lse, group=group, out_dtype=out_dtype or q.dtype, merge=merge)
        return full[:, :, None, :]
    from . import ops
    world = dist.get_world_size(group)
    b, n, _, hd = q.shape
    rows = b * n
    if exchange is not None:
        if (exchange.batch, exchange.heads) != (b, n):
            raise ValueError("exchange was built for another batch x heads")
        out_view, lse_view = exchange.out_view, exchange.lse_view
    else:
        mine = torch.empty(rows * (hd + 1), dtype=torch.float32, device=q.device)
        out_view = mine[:rows * hd].view(b, n, 1, hd)
        lse_view = mine[rows * hd:].view(b, n)
    have_q = packed is not None and packed[0] is not None and packed[0].shape[2] > 0
    have_r = kres is not None and kres.shape[2] > 0
    attended = have_q or have_r
    if not attended:                                     # a rank without keys: weight zero in the merge
        out_view.zero_()
        lse_view.fill_(float("-inf"))
    else:
        final = None
        if exchange is not None and push_in_attention and collect_in_attention:
            final = torch.empty((b, n, 1, hd), dtype=out_dtype or q.dtype, device=q.device)
        ops.decode_attention(q, kres if have_r else None, *(packed if have_q else (None,) * 5), v,
                             out_dtype=torch.float32, out=out_view, lse_out=lse_view,
                             push_to=exchange if push_in_attention else None, collect_out=final, **kw)
        if final is not None:
            return final
    if exchange is not None:
        return exchange.merge(out_dtype=out_dtype or q.dtype, after_attention=attended,
                              pushed=attended and push_in_attention)
    gathered = torch.empty(world * mine.numel(), dtype=torch.float32, device=q.device)
    dist.all_gather_into_tensor(gathered, mine, group=group)
    return ops.merge_lse_gathered(gathered, world, rows, out_dtype=out_dtype or q.dtype, out_shape=(b, n, 1, hd))
