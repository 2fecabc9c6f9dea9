"""Multi-rank plumbing on CPU: world_size 2 and 3 over gloo.  The attention and merge arithmetic are injected from
the CPU oracle (the product's own compute is CUDA-only); what is exercised is the partitioning, the packing of the
all-gather message, rank ordering, empty ranks and the failure behaviour."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_range_is_balanced_and_covers_everything():
    from polarquant_b200.distributed import shard_range, split_sequence
    for total in (0, 1, 7, 8, 255):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert split_sequence(255, 128, 7, 8)[2] and not split_sequence(255, 128, 0, 8)[2]
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _worker(rank, world, port, nb, result_queue, mixed=False):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import polar_oracle as oracle
        from polarquant_b200 import distributed as pqd
        torch.manual_seed(1234)                              # every rank builds the same full problem
        B, N, Nk, G, R = 2, 8, 2, 32, 19
        keys = oracle.synth_keys(B, Nk, nb * G + R, 128, torch.bfloat16, seed=5)
        q = torch.randn(B, N, 1, 128).to(torch.bfloat16)
        v = torch.randn(B, Nk, nb * G + R, 128).to(torch.bfloat16)
        packed = oracle.quantize_ops(keys[:, :, :nb * G].contiguous(), 4, 4, G) if nb else None
        kres = keys[:, :, nb * G:]
        want = oracle.decode_attention(q, kres, *(packed or (None,) * 5), v, faithful_rounding=False)

        g0, g1, owns_res = pqd.split_sequence(nb, R, rank, world)
        my_packed = [t[:, :, g0:g1] for t in packed] if nb and g1 > g0 else None
        my_v = [v[:, :, g0 * G:g1 * G]]
        if owns_res:
            my_v.append(v[:, :, nb * G:])
        my_v = torch.cat(my_v, dim=2)

        def attend(q_, kres_, packed_, v_, **kw):
            if kw:                                           # packed values travel as keyword arguments
                return oracle.decode_attention_mixed(q_, kres_, *packed_, kw["value_codes"], kw["value_scale"],
                                                     kw["value_mn"], v_, faithful_rounding=False, return_lse=True)
            return oracle.decode_attention(q_, kres_, *packed_, v_, faithful_rounding=False, return_lse=True)

        def merge(outs, lses, out_dtype):
            return oracle.merge_lse(outs, lses)[0].to(out_dtype)

        kw = {}
        if mixed and nb:
            # values of the packed tokens are packed too; only the residual window's owner holds full-precision ones
            vc, vs, vm = oracle.quantize_values(v[:, :, :nb * G].contiguous())
            want = oracle.decode_attention_mixed(q, kres, *packed, vc, vs, vm, v[:, :, nb * G:],
                                                 faithful_rounding=False)
            my_v = v[:, :, nb * G:] if owns_res else None
            if g1 > g0:
                kw = dict(value_codes=vc[:, :, g0 * G:g1 * G], value_scale=vs[:, :, g0 * G:g1 * G],
                          value_mn=vm[:, :, g0 * G:g1 * G])
        got = pqd.sequence_parallel_decode(q, kres if owns_res else None, my_packed, my_v, out_dtype=torch.float32,
                                           attend=attend, merge=merge, **kw)
        result_queue.put((rank, float((got - want).abs().max()), tuple(got.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,nb,mixed", [(2, 6, False), (3, 2, False), (2, 0, False), (2, 6, True)])
def test_sequence_split_over_gloo_matches_the_unsplit_result(world, nb, mixed):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000) + world * 7 + nb + (50 if mixed else 0)
    procs = [ctx.Process(target=_worker, args=(r, world, port, nb, q, mixed)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    results = [q.get(timeout=5) for _ in range(world)]
    assert sorted(r[0] for r in results) == list(range(world))
    for _, err, shape in results:
        assert shape == (2, 8, 1, 128)
        assert err < 1e-5


def _failing_worker(rank, world, port, result_queue):
    """Rank 1 never joins the collective: rank 0 must get an error from the process-group timeout, not hang."""
    import datetime
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from polarquant_b200 import distributed as pqd
    def leave():
        result_queue.close()
        result_queue.join_thread()                           # flush the queue before the hard exit
        os._exit(0)

    if rank == 1:
        result_queue.put((rank, "left"))
        leave()                                              # leaves between steps, nothing in flight
    try:
        out = torch.zeros(1, 2, 128)
        lse = torch.zeros(1, 2)
        pqd.merge_across_ranks(out, lse, merge=lambda o, l, dt: o[0])
        result_queue.put((rank, "no error"))
    except Exception as exc:                                 # noqa: BLE001 - any backend error type is fine
        result_queue.put((rank, "error:" + type(exc).__name__))
    leave()


def test_missing_rank_surfaces_as_an_error_on_the_host():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    results = dict(q.get(timeout=5) for _ in range(2))
    assert results[1] == "left"
    assert results[0].startswith("error:")
