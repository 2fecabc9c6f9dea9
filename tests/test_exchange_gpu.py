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
                                            (ctypes.c_void_p * world)(*[t.data_ptr() for t in lses]), stream)
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
