"""The one-kernel sequence-split exchange (`pq_exchange_merge`): push to the peers, wait on flags, merge.

On one GPU the ranks are emulated by ONE cooperative launch over all ranks' buffers (`pq_exchange_merge_emulated`;
separate launches that wait on one another must not share a GPU).  The bar is bitwise equality with the merge of an
all-gathered buffer (`pq_merge_lse_strided`), over several steps on the same buffers so that the epoch and the
release flags are exercised.  The bounded wait is checked with a peer that never arrives: the call returns within
seconds with a status bit set.  The real peer-memory path runs in `tests/test_multigpu_gpu.py` on two or more GPUs."""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _buffers(lib, world, rows):
    nbytes = lib.pq_exchange_bytes(world, rows, 128)
    assert nbytes > 0
    bufs = [torch.zeros(nbytes // 4, dtype=torch.float32, device=DEV) for _ in range(world)]
    slots = []
    for r in range(world):
        off = lib.pq_exchange_slot_offset(world, rows, 128, r)
        assert off >= 0 and off % 16 == 0
        slots.append(bufs[r][off // 4: off // 4 + rows * 129])
    return bufs, slots


@pytest.mark.parametrize("world,rows", [(2, 512), (2, 5), (3, 37), (4, 1), (4, 256), (8, 130)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_emulated_ranks_reproduce_the_gathered_merge_bit_for_bit(world, rows, out_dtype):
    from polarquant_b200 import _lib, ops
    lib = _lib.load()
    bufs, slots = _buffers(lib, world, rows)
    g = torch.Generator(device=DEV).manual_seed(1000 * world + rows)
    arr = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for step in range(4):
        gathered = torch.empty(world, rows * 129, dtype=torch.float32, device=DEV)
        gathered[:, :rows * 128] = torch.randn(world, rows * 128, device=DEV, generator=g)
        gathered[:, rows * 128:] = torch.randn(world, rows, device=DEV, generator=g) * 3.0
        if step == 1:
            gathered[0, rows * 128:] = float("-inf")          # a rank without keys
        if step == 2 and rows > 1:
            gathered[-1, rows * 128 + 1] = float("-inf")
        for r in range(world):
            slots[r].copy_(gathered[r])
        want = ops.merge_lse_gathered(gathered.reshape(-1), world, rows, out_dtype=out_dtype)
        outs = [torch.full((rows, 128), float("nan"), dtype=out_dtype, device=DEV) for _ in range(world)]
        lses = [torch.empty(rows, dtype=torch.float32, device=DEV) for _ in range(world)]
        rc = lib.pq_exchange_merge_emulated(arr, world, rows, 128,
                                            (ctypes.c_void_p * world)(*[o.data_ptr() for o in outs]),
                                            ops._DT[out_dtype],
                                            (ctypes.c_void_p * world)(*[t.data_ptr() for t in lses]), 0, stream)
        assert rc == 0, lib.pq_strerror(rc)
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.equal(outs[r], want), f"step {step}, rank {r}"
            word = ctypes.c_uint(7)
            assert lib.pq_exchange_status(bufs[r].data_ptr(), world, rows, 128, ctypes.byref(word), stream) == 0
            assert word.value == 0
        m = gathered[:, rows * 128:].max(dim=0).values
        ref_lse = m + torch.log(torch.exp(gathered[:, rows * 128:] - m).sum(dim=0))
        assert torch.allclose(lses[0], ref_lse, atol=1e-5, rtol=1e-5)


class _LocalExchange:
    """The attributes `decode_attention(push_to=...)` reads from a PeerExchange, over buffers of one GPU."""

    def __init__(self, bufs, rank, batch, heads):
        self.world, self.rank = len(bufs), rank
        self._bufs = (ctypes.c_void_p * len(bufs))(*[b.data_ptr() for b in bufs])
        rows = batch * heads
        self.out_view = bufs[rank][:rows * 128].view(batch, heads, 1, 128)
        self.lse_view = bufs[rank][rows * 128: rows * 129].view(batch, heads)


@pytest.mark.parametrize("world", [2, 3])
def test_attention_pushes_its_rows_and_the_exchange_only_collects(world):
    """Producer-side push: every emulated rank runs the fused attention on its slice of the keys with
    `push_to` set - its merge stores the rows, paired with the epoch, into the other ranks' inboxes - and the
    exchange kernel, told that the rows are pushed, only collects and merges.  Three steps on the same buffers;
    bitwise equal to the merge of the gathered blocks and within the bar of attention over all keys."""
    import polarquant_b200 as pq
    from polarquant_b200 import _lib, ops
    from polarquant_b200 import distributed as pqd
    from oracle import polar_oracle as oracle
    lib = _lib.load()
    B, N, Nk, Nb, G, R = 2, 8, 2, 6, 64, 20
    rows = B * N
    bufs, _ = _buffers(lib, world, rows)
    ranks = [_LocalExchange(bufs, r, B, N) for r in range(world)]
    arr = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for step in range(3):
        keys = oracle.synth_keys(B, Nk, Nb * G + R, 128, torch.bfloat16, seed=300 + step, device=DEV)
        g = torch.Generator(device=DEV).manual_seed(310 + step)
        q = torch.randn(B, N, 1, 128, device=DEV, generator=g).to(torch.bfloat16)
        v = torch.randn(B, Nk, Nb * G + R, 128, device=DEV, generator=g).to(torch.bfloat16)
        packed = pq.quantize_and_pack_nbit(keys[:, :, :Nb * G].contiguous(), 4, 4, G)
        kres = keys[:, :, Nb * G:].contiguous()
        full = pq.decode_attention(q, kres, *packed, v, out_dtype=torch.float32)
        for r, ex in enumerate(ranks):
            g0, g1, owns = pqd.split_sequence(Nb, R, r, world)
            mine = [t[:, :, g0:g1].contiguous() for t in packed]
            my_v = torch.cat([v[:, :, g0 * G:g1 * G]] + ([v[:, :, Nb * G:]] if owns else []), dim=2).contiguous()
            pq.decode_attention(q, kres if owns else None, *mine, my_v, out_dtype=torch.float32, out=ex.out_view,
                                lse_out=ex.lse_view, push_to=ex)
        gathered = torch.stack([b[:rows * 129] for b in bufs]).reshape(-1).clone()
        want = ops.merge_lse_gathered(gathered, world, rows, out_dtype=torch.float32)
        outs = [torch.full((rows, 128), float("nan"), device=DEV) for _ in range(world)]
        rc = lib.pq_exchange_merge_emulated(arr, world, rows, 128,
                                            (ctypes.c_void_p * world)(*[o.data_ptr() for o in outs]),
                                            ops._DT[torch.float32], None, _lib.PQ_EXCHANGE_PUSHED, stream)
        assert rc == 0, lib.pq_strerror(rc)
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.equal(outs[r], want), f"step {step}, rank {r}"
            word = ctypes.c_uint(7)
            assert lib.pq_exchange_status(bufs[r].data_ptr(), world, rows, 128, ctypes.byref(word), stream) == 0
            assert word.value == 0
        assert float((outs[0].view(B, N, 1, 128) - full).abs().max()) <= 8e-3


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("final_dtype", [torch.float32, torch.bfloat16])
def test_attention_call_can_do_the_whole_exchange(world, final_dtype):
    """`collect_out`: the attention call's merge pushes its rows, waits for the peers' rows and writes the merged
    result - no exchange kernel.  On one GPU the emulated ranks cannot wait for one another in separate launches, so
    every rank first pushes its rows with a push-only call and then repeats the call with `collect_out`: the rows it
    waits for are already there.  Bitwise equal to the merge of the gathered blocks, three steps on the same buffers."""
    import polarquant_b200 as pq
    from polarquant_b200 import _lib, ops
    from polarquant_b200 import distributed as pqd
    from oracle import polar_oracle as oracle
    lib = _lib.load()
    B, N, Nk, Nb, G, R = 2, 14, 2, 6, 64, 20            # 7 query heads per kv head: rows not aligned to anything
    rows = B * N
    bufs, _ = _buffers(lib, world, rows)
    ranks = [_LocalExchange(bufs, r, B, N) for r in range(world)]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for step in range(3):
        keys = oracle.synth_keys(B, Nk, Nb * G + R, 128, torch.bfloat16, seed=400 + step, device=DEV)
        g = torch.Generator(device=DEV).manual_seed(410 + step)
        q = torch.randn(B, N, 1, 128, device=DEV, generator=g).to(torch.bfloat16)
        v = torch.randn(B, Nk, Nb * G + R, 128, device=DEV, generator=g).to(torch.bfloat16)
        packed = pq.quantize_and_pack_nbit(keys[:, :, :Nb * G].contiguous(), 4, 4, G)
        kres = keys[:, :, Nb * G:].contiguous()

        def call(r, collect_out=None):
            ex = ranks[r]
            g0, g1, owns = pqd.split_sequence(Nb, R, r, world)
            mine = [t[:, :, g0:g1].contiguous() for t in packed]
            my_v = torch.cat([v[:, :, g0 * G:g1 * G]] + ([v[:, :, Nb * G:]] if owns else []), dim=2).contiguous()
            pq.decode_attention(q, kres if owns else None, *mine, my_v, out_dtype=torch.float32, out=ex.out_view,
                                lse_out=ex.lse_view, push_to=ex, collect_out=collect_out)

        for r in range(world):
            call(r)                                        # rows of this step land in every inbox
        torch.cuda.synchronize()
        gathered = torch.stack([b[:rows * 129] for b in bufs]).reshape(-1).clone()
        want = ops.merge_lse_gathered(gathered, world, rows, out_dtype=final_dtype)
        for r in range(world):
            final = torch.full((B, N, 1, 128), float("nan"), dtype=final_dtype, device=DEV)
            call(r, collect_out=final)
            torch.cuda.synchronize()
            assert torch.equal(final.view(rows, 128), want), f"step {step}, rank {r}"
            word = ctypes.c_uint(7)
            assert lib.pq_exchange_status(bufs[r].data_ptr(), world, rows, 128, ctypes.byref(word), stream) == 0
            assert word.value == 0


def test_push_arguments_are_validated():
    import polarquant_b200 as pq
    from polarquant_b200 import _lib
    from oracle import polar_oracle as oracle
    lib = _lib.load()
    B, N, Nk = 1, 4, 1
    bufs, _ = _buffers(lib, 2, B * N)
    ex = _LocalExchange(bufs, 0, B, N)
    keys = oracle.synth_keys(B, Nk, 64, 128, torch.bfloat16, seed=5, device=DEV)
    q = torch.randn(B, N, 1, 128, device=DEV).to(torch.bfloat16)
    v = torch.randn(B, Nk, 64, 128, device=DEV).to(torch.bfloat16)
    with pytest.raises(ValueError):        # results must go to the exchange's own views
        pq.decode_attention(q, keys, None, None, None, None, None, v, out_dtype=torch.float32, push_to=ex)
    with pytest.raises(ValueError):        # the own block is fp32
        pq.decode_attention(q, keys, None, None, None, None, None, v, out_dtype=torch.bfloat16, out=ex.out_view,
                            lse_out=ex.lse_view, push_to=ex)


def test_a_peer_that_never_arrives_ends_the_wait_with_a_status_bit():
    """Rank 0 of a two-rank exchange runs alone: nothing ever sets the peer's flag.  The kernel must give up after
    its time limit, set the status bit and leave the context usable."""
    from polarquant_b200 import _lib, ops
    lib = _lib.load()
    world, rows = 2, 8
    bufs, slots = _buffers(lib, world, rows)
    slots[0].normal_()
    out = torch.empty(rows, 128, dtype=torch.float32, device=DEV)
    arr = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = time.time()
    rc = lib.pq_exchange_merge(arr, world, 0, rows, 128, out.data_ptr(), ops._DT[torch.float32], None, 0, stream)
    assert rc == 0, lib.pq_strerror(rc)
    word = ctypes.c_uint(0)
    assert lib.pq_exchange_status(bufs[0].data_ptr(), world, rows, 128, ctypes.byref(word), stream) == 0
    assert time.time() - t0 < 10.0
    assert word.value & 2                        # the peer's data never arrived
    # rank 0 did push its rows, paired with epoch 1, into its inbox slot (parity 1, sender 0) of the peer's buffer
    inbox = bufs[1].view(torch.int32)[(rows * 129 + 3) // 4 * 4:]
    sent = inbox[(1 * world + 0) * rows * 260:][:rows * 256].view(rows * 64, 4)
    assert bool((sent[:, 1] == 1).all()) and bool((sent[:, 3] == 1).all())
    assert torch.equal(sent[:, 0::2].reshape(-1).view(torch.float32), slots[0][:rows * 128])
    assert torch.equal(torch.ones(4, device=DEV) + 1, torch.full((4,), 2.0, device=DEV))     # context still works


def test_argument_validation():
    from polarquant_b200 import _lib
    lib = _lib.load()
    assert lib.pq_exchange_bytes(9, 4, 128) == 0 and lib.pq_exchange_bytes(2, 0, 128) == 0
    assert lib.pq_exchange_bytes(2, 4, 64) == 0
    assert lib.pq_exchange_slot_offset(2, 4, 128, 2) == -1
    buf = torch.zeros(4096, dtype=torch.float32, device=DEV)
    arr = (ctypes.c_void_p * 2)(buf.data_ptr(), None)
    assert lib.pq_exchange_merge(arr, 2, 0, 4, 128, buf.data_ptr(), 2, None, 0, None) == -1
    arr = (ctypes.c_void_p * 2)(buf.data_ptr(), buf.data_ptr() + 4)
    assert lib.pq_exchange_merge(arr, 2, 0, 4, 128, buf.data_ptr(), 2, None, 0, None) == -5


def _single_rank_worker(port, queue):
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    try:
        import polarquant_b200 as pq
        from polarquant_b200 import distributed as pqd
        from oracle import polar_oracle as oracle
        B, N, Nk, Nb, G, R = 2, 8, 2, 3, 128, 40
        keys = oracle.synth_keys(B, Nk, Nb * G + R, 128, torch.bfloat16, seed=41).to(dev)
        g = torch.Generator().manual_seed(42)
        q = torch.randn(B, N, 1, 128, generator=g).to(torch.bfloat16).to(dev)
        v = torch.randn(B, Nk, Nb * G + R, 128, generator=g).to(torch.bfloat16).to(dev)
        packed = pq.quantize_and_pack_nbit(keys[:, :, :Nb * G].contiguous(), 4, 4, G)
        kres = keys[:, :, Nb * G:].contiguous()
        full = pq.decode_attention(q, kres, *packed, v, out_dtype=torch.float32)
        ex = pqd.PeerExchange(B, N, device=dev)
        same = True
        for push, collect in ((True, True), (True, False), (False, False), (True, True)):
            got = pqd.sequence_parallel_decode(q, kres, packed, v, out_dtype=torch.float32, exchange=ex,
                                               push_in_attention=push, collect_in_attention=collect)
            torch.cuda.synchronize()
            same = same and bool(torch.equal(got, full))
        # the step captured in a CUDA graph and replayed (the epoch lives on the device)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            pqd.sequence_parallel_decode(q, kres, packed, v, out_dtype=torch.float32, exchange=ex)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            captured = pqd.sequence_parallel_decode(q, kres, packed, v, out_dtype=torch.float32, exchange=ex)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        same = same and bool(torch.equal(captured, full))
        status = ex.status()
        ex.close()
        queue.put((same, status))
    finally:
        dist.destroy_process_group()


def test_peer_exchange_object_with_a_single_rank():
    """The host class end to end on one GPU (a group of one rank has no peers): allocation through the library, the
    views torch gets over it, both push variants, CUDA-graph replay, status and release.  With one rank the merged
    result is the rank's own partial, i.e. plain attention, bit for bit."""
    import os
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    proc = ctx.Process(target=_single_rank_worker, args=(35500 + os.getpid() % 2000, queue))
    proc.start()
    proc.join(timeout=300)
    assert proc.exitcode == 0
    same, status = queue.get(timeout=5)
    assert same and status == 0
