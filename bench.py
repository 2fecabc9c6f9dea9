"""Benchmark of the polar key-cache hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one fused decode-attention call (packed-key logits + residual-key logits + softmax + P.V)
over the whole batch of the Llama-3.1-8B-shaped configuration: batch 16, 32 query / 8 kv heads, head_dim 128,
context 32768 = 255 packed groups of 128 tokens + 128 full-precision residual keys, bf16, polar 4/4.
Inputs are seeded synthetic tensors (keys randn times a per-channel log-uniform scale in [0.5, 8], packed by
the CUDA quantizer; queries and values randn); the inputs of one step (1.36 GB) exceed the 126 MB L2.

It prints ONE JSON line.  `value` is algorithmic GB/s with the cache resident in HBM; `e2e` is the same metric
through the host-buffer C entry point with every input copied from pinned host memory and the output copied
back inside the timed region; `roofline` is the attention kernel alone, timed in a loop of its own (20 warm-up
and 60 sampled launches, CUDA events around the kernel on its stream) whatever --steps says; `cpu_baseline` is
the reference's decode branch on the host cores on a bounded sample, measured BEFORE any GPU work starts;
`sustained` repeats the step for half a second (power-capped clocks); `packed_values` is the step with 4-bit
values; `reference_gpu` times the reference's own Triton kernel and its whole unmodified decode branch on the same
GPU, beside this library's entry points on the same tensors; `e2e_tokens` is greedy decode of a random-init
Llama-3.1-8B-shaped model (tokens/s).
With N > 1 (launched by torch.distributed.run) every rank holds its own batch of 16 sequences (weak scaling,
the path shards by batch / kv head without any collective) and the time is the max over ranks; `longctx` then
adds the 131072-token step of the 70B-shaped layer sharded by kv head and by sequence (the one place the path
has an exchange: an NCCL all-gather of partial results), after a seeded correctness check of that exchange
(`seqsplit_check`).

--impl reference runs the reference's own decode branch on host cores (rank 0 only) on the same configuration.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "polar-KV decode-attn GB/s (% HBM peak) & µs/step @32k ctx; e2e decode tokens/s"
NOMINAL_HBM_GBS = 8000.0
# DRAM bytes (read + write) of one attention-kernel launch per batch element of the benchmark shape, from the
# ncu capture of the batch-4 case (dram__bytes_read.sum 341.99 MB + dram__bytes_write.sum 3.85 MB per launch);
# traffic grows in proportion to the batch, so a full-size launch is this figure times the batch
NCU_TRAFFIC_BYTES_PER_BATCH_ELEMENT = (341.99e6 + 3.85e6) / 4
FALLBACK_HBM_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    # 200 back-to-back steps (45 ms) is the burst regime; the `sustained` leg repeats the step for half a second,
    # where the power cap sets the clock
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    # smaller cases for profiler captures; the defaults are the benchmark configuration
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--ctx", type=int, default=32768)
    ap.add_argument("--group", type=int, default=128)
    ap.add_argument("--rbits", type=int, default=4)
    ap.add_argument("--tbits", type=int, default=4)
    ap.add_argument("--q-heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--no-extras", action="store_true", help="skip e2e, quantizer and CPU legs (profiler runs)")
    ap.add_argument("--key-format", default="byte", choices=["byte", "packed6"],
                    help="packed6: the 48-byte-per-token key container (needs --rbits/--tbits 3/3 or 2/4); for "
                         "profiler runs and side measurements, the headline configuration is the byte container")
    ap.add_argument("--e2e-new-tokens", type=int, default=64,
                    help="generated tokens of the end-to-end greedy-decode leg (batch 32, 8192-token prompts); "
                         "0 or 1 skips it")
    ap.add_argument("--packed-values", action="store_true",
                    help="time the step with the values packed to 4 bits as well (the reference's mixed class) "
                         "instead of the headline configuration; implies --no-extras")
    return ap.parse_args()


def algorithmic_bytes(B, N, Nk, Nb, G, R, e=2, e_out=2, key_bytes=64):
    """Bytes one decode step must move: codes + scales + residual keys + values + query + output."""
    lq = Nb * G
    return B * Nk * (lq * key_bytes + Nb * 4 * 64 * e + R * 128 * e + (lq + R) * 128 * e) + B * N * 128 * (e + e_out)


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    _instant_ok = None          # does this driver report power.draw.instant (power.draw is a one-second average)

    def __init__(self, index: int):
        self.rows = []
        self.proc = None
        self.index = index

    @classmethod
    def _has_instant(cls, index: int) -> bool:
        if cls._instant_ok is None:
            try:
                r = subprocess.run(["nvidia-smi", f"--id={index}", "--query-gpu=power.draw.instant",
                                    "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=20)
                float(r.stdout.strip().splitlines()[0])
                cls._instant_ok = r.returncode == 0
            except Exception:
                cls._instant_ok = False
        return cls._instant_ok

    def start(self):
        try:
            fields = self.FIELDS + (",power.draw.instant" if self._has_instant(self.index) else "")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={fields}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, maxes, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            try:
                clocks.append(float(r[0])); maxes.append(float(r[1]))
                for name, flag in zip(names, r[3:7]):
                    if flag.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        powers, instant = [], []
        for r in self.rows:
            try:
                powers.append(float(r[2]))
                if len(r) > 7:
                    instant.append(float(r[7]))
            except Exception:
                continue
        return {"sm_mhz": statistics.median(clocks) if clocks else None,
                "sm_max_mhz": max(maxes) if maxes else None, "samples": len(clocks), "reasons": sorted(reasons),
                "power_w_median": statistics.median(powers) if powers else None,
                "power_w_instant_median": statistics.median(instant) if instant else None}


def make_inputs(args, device, seed):
    """Seeded synthetic cache for one rank: packed keys (CUDA quantizer), residual keys, values, query."""
    import torch
    import polarquant_b200 as pq
    B, N, Nk, G = args.batch, args.q_heads, args.kv_heads, args.group
    R = 128
    Nb = (args.ctx - R) // G
    g = torch.Generator(device=device).manual_seed(seed)
    scale = torch.exp(torch.empty(Nk, 128, device=device).uniform_(math.log(0.5), math.log(8.0), generator=g))
    q = torch.randn(B, N, 1, 128, device=device, generator=g).to(torch.bfloat16)
    v = torch.randn(B, Nk, Nb * G + R, 128, device=device, generator=g).to(torch.bfloat16)
    kres = (torch.randn(B, Nk, R, 128, device=device, generator=g) * scale[None, :, None]).to(torch.bfloat16)
    packed = [[] for _ in range(5)]
    for b in range(B):
        kb = (torch.randn(1, Nk, Nb * G, 128, device=device, generator=g) * scale[None, :, None]).to(torch.bfloat16)
        for lst, t in zip(packed, pq.quantize_and_pack_nbit(kb, args.rbits, args.tbits, G,
                                                            key_format=getattr(args, "key_format", "byte"))):
            lst.append(t)
    packed = [torch.cat(lst, dim=0) for lst in packed]
    return dict(q=q, kres=kres, packed=packed, v=v, B=B, N=N, Nk=Nk, Nb=Nb, G=G, R=R)


def cpu_sample(args, seed=1002):
    """One batch element of the benchmark configuration, built on the CPU with the oracle's quantizer."""
    import torch
    from oracle import polar_oracle as oracle
    N, Nk, G, R = args.q_heads, args.kv_heads, args.group, 128
    Nb = (args.ctx - R) // G
    g = torch.Generator().manual_seed(seed)
    keys = oracle.synth_keys(1, Nk, Nb * G + R, 128, torch.bfloat16, seed=seed)
    q = torch.randn(1, N, 1, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(1, Nk, Nb * G + R, 128, generator=g).to(torch.bfloat16)
    packed = oracle.quantize_ops(keys[:, :, :Nb * G].contiguous(), args.rbits, args.tbits, G)
    return dict(q=q, kres=keys[:, :, Nb * G:].contiguous(), packed=list(packed), v=v), \
        algorithmic_bytes(1, N, Nk, Nb, G, R)


def cpu_step_fn(sample, args):
    """The decode step on host cores as a callable, and what it is.

    With the reference's files installed (oracle/_ref, see oracle/install_ref.py): the reference's own, unmodified
    ``LlamaPolarGroupAttention.forward`` decode branch (models/modeling_llama_polar.py:61-101) - its concatenations,
    residual-key matmul, scaling, softmax, repeat_kv and P.V as written - with the one piece that cannot run on a
    CPU, the Triton kernel behind ``attention_decode_forward_triton_impl``, served by the reference's own
    dequantise-then-matmul formula (models/kernel4group.py:151-155).  kind = "reference".
    Without them: the oracle's restatement of the same branch.  kind = "port".
    """
    from oracle import polar_oracle as oracle
    from oracle import ref_harness
    root = ref_harness.ref_root()
    if root is None or (args.rbits, args.tbits, args.group) != (4, 4, 128):   # the class hard-codes 4/4, group 128
        def port():
            return oracle.decode_attention(sample["q"], sample["kres"], *sample["packed"], sample["v"],
                                           rbits=args.rbits, tbits=args.tbits)
        return port, "port", "oracle restatement of the reference's eager decode branch, torch CPU ops"
    from polarquant_b200 import dropin
    llama, _ = dropin.load_polar_patches(root, entry_module=ref_harness.dequantise_entry_module(),
                                         quantize_fn=lambda k, rbits, tbits, group_size:
                                         oracle.quantize_ops(k, rbits, tbits, group_size))
    q, kres, v = sample["q"], sample["kres"], sample["v"]
    attn = ref_harness.identity_attention(llama, "llama", q.shape[1], kres.shape[1], q.dtype)
    tokens = v.shape[2]
    past = (kres[:, :, :-1].contiguous(), *sample["packed"], v[:, :, :-1].contiguous(), tokens - 1)
    k_new, v_new = kres[:, :, -1:].contiguous(), v[:, :, -1:].contiguous()

    def ref():
        return ref_harness.decode_step(attn, q, k_new, v_new, past)[0]
    return ref, "reference", ("the reference's unmodified LlamaPolarGroupAttention.forward decode branch "
                              "(identity projections), its Triton logits call served by its dequantise-then-matmul "
                              "formula, torch CPU ops")


def time_cpu(args, limit_s=20.0, max_reps=10):
    """cpu_baseline of the JSON line: run before any GPU work of this process, mean of the timed runs."""
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample, nbytes = cpu_sample(args)
    fn, kind, what = cpu_step_fn(sample, args)
    fn()                                                 # warm-up
    times, t_end = [], time.perf_counter() + limit_s
    while len(times) < max_reps and (time.perf_counter() < t_end or len(times) < 2):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    mean = sum(times) / len(times)
    return {"value": nbytes / mean / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": f"1 of {args.batch} batch elements of the workload ({nbytes / 1e6:.1f} MB per step), "
                      f"mean of {len(times)} runs after 1 warm-up, measured before the GPU legs start; {what}, "
                      f"{cores} threads",
            "ms_per_sample_step": mean * 1e3, "ms_best": min(times) * 1e3}


def run_reference_arm(args, rank):
    """--impl reference: the reference's decode branch for this step on host cores; exactly --steps timed steps
    after --warmup untimed ones, each step one batch element of the workload."""
    if rank != 0:
        return
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    sample, nbytes = cpu_sample(args)
    fn, kind, what = cpu_step_fn(sample, args)
    for _ in range(args.warmup):
        fn()
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    val = nbytes / dt / 1e9
    sample_txt = (f"each step = 1 of {args.batch} batch elements of the workload ({nbytes / 1e6:.1f} MB), "
                  f"{steps} timed steps after {args.warmup} warm-ups; {what}, {cores} threads")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample_txt},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(args):
    return {"workload": f"Llama-3.1-8B-shaped GQA decode attention: batch {args.batch} per GPU, {args.q_heads} q / "
                        f"{args.kv_heads} kv heads, head_dim 128, ctx {args.ctx}, polar {args.rbits}/{args.tbits}, "
                        f"group {args.group}, residual 128, bf16"
                        + (", values packed to 4 bits per token" if getattr(args, "packed_values", False) else "")
                        + (", keys in the 48-byte container" if getattr(args, "key_format", "byte") == "packed6" else ""),
            "l2": "inputs of one step (1.36 GB at the default size) exceed the 126 MB L2; no flush needed",
            "sharding": "batch per GPU, no collective in the step"}


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    # The CPU baseline runs first, before this process touches the GPU: no clock samplers, no pinned buffers, no
    # busy-waiting CUDA threads compete with it for the host cores.  It is the figure to quote.
    cpu_base = time_cpu(args) if (rank == 0 and world == 1 and not args.no_extras) else None

    import torch
    import torch.distributed as dist
    import polarquant_b200 as pq
    from polarquant_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    lib = _lib.load()

    inp = make_inputs(args, device, seed=1002 + rank)
    B, N, Nk, Nb, G, R = (inp[k] for k in ("B", "N", "Nk", "Nb", "G", "R"))
    nbytes = algorithmic_bytes(B, N, Nk, Nb, G, R, key_bytes=48 if args.key_format == "packed6" else 64)
    if args.key_format != "byte":
        args.no_extras = True             # the side legs are written for the headline container
    ws = torch.empty(lib.pq_decode_workspace_bytes(B, N, Nk, Nb, G, R, 0) + 256, dtype=torch.uint8, device=device)
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)

    def new_event():
        e = ctypes.c_void_p()
        assert lib.pq_event_create(ctypes.byref(e)) == 0
        return e

    if args.packed_values:
        args.no_extras = True
        Lq = Nb * G
        vc, vs, vm = pq.quantize_values(inp["v"][:, :, :Lq], layout="tiled")
        v_res = inp["v"][:, :, Lq:].contiguous()
        nbytes = nbytes - Lq * B * Nk * 256 + vc.numel() * 4 + 2 * vs.numel() * 2
        inp["v"] = None

    def step(mid=None):
        if args.packed_values:
            return pq.decode_attention(inp["q"], inp["kres"], *inp["packed"], v_res, rbits=args.rbits,
                                       tbits=args.tbits, workspace=ws, mid_event=mid, value_codes=vc, value_scale=vs,
                                       value_mn=vm)
        return pq.decode_attention(inp["q"], inp["kres"], *inp["packed"], inp["v"], rbits=args.rbits,
                                   tbits=args.tbits, workspace=ws, mid_event=mid, key_format=args.key_format)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()                   # started before the warm-up so the GPU is not left idle before the timed steps
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    K = args.steps
    ev_start, ev_end = new_event(), new_event()
    barrier()
    # The first launches behind a host-side barrier (an NCCL collective plus a device synchronise) start on an idle
    # GPU and run up to 2x slower than the steady state: a few untimed steps bring the pipeline back before the
    # start event is recorded.
    for _ in range(5):
        step()
    lib.pq_event_record(ev_start, stream)
    for _ in range(K):
        step()                            # attention kernel + merge kernel (launched programmatically behind it)
    lib.pq_event_record(ev_end, stream)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = ctypes.c_float()
    lib.pq_event_elapsed_ms(ev_start, ev_end, ctypes.byref(ms))
    my_ms = ms.value
    total_ms = my_ms
    per_rank = [my_ms / K]
    if world > 1:
        t = torch.tensor([my_ms], device=device)
        gathered = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(gathered, t)
        per_rank = [float(x.item()) / K for x in gathered]
        total_ms = max(per_rank) * K
    ms_per_step = total_ms / K
    value = nbytes * world / (ms_per_step * 1e-3) / 1e9

    # ---- roofline: the attention kernel alone, in a fixed loop of its own (independent of --steps) ----
    # An event sits between the kernel and its merge, so in this loop the merge is a plain launch and the next
    # kernel's start event lies behind a fully serialised merge.
    ROOF_WARM, ROOF_N = 20, 60
    for _ in range(ROOF_WARM):
        step()
    ev_a = [new_event() for _ in range(ROOF_N)]
    ev_m = [new_event() for _ in range(ROOF_N)]
    for i in range(ROOF_N):
        lib.pq_event_record(ev_a[i], stream)
        step(ev_m[i])
    torch.cuda.synchronize(device)
    kern_ms = []
    for i in range(ROOF_N):
        lib.pq_event_elapsed_ms(ev_a[i], ev_m[i], ctypes.byref(ms))
        kern_ms.append(ms.value)
    for e in ev_a + ev_m:
        lib.pq_event_destroy(e)

    result = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        kavg = sum(kern_ms) / len(kern_ms)
        achieved = nbytes / (kavg * 1e-3) / 1e9
        result = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": K,
            "warmup": warm, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args),
            "us_per_step": ms_per_step * 1e3, "algorithmic_mb_per_step_per_gpu": nbytes / 1e6,
            "pct_of_nominal_8TBs": 100.0 * value / world / NOMINAL_HBM_GBS,
            "pct_of_measured_copy_peak": 100.0 * value / world / peak,
            "ms_per_step_per_rank": per_rank,
            "clocks": clocks, "gpu_launches": 2 * K,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": (NCU_TRAFFIC_BYTES_PER_BATCH_ELEMENT * B
                                     if (args.ctx, args.group, args.q_heads, args.kv_heads) == (32768, 128, 32, 8)
                                     and not args.packed_values and args.key_format == "byte" else None),
                         "traffic_note": "bytes per launch; ncu capture at batch 4 scaled by the batch",
                         "kernel": "decode_kernel (fused attention over packed keys)",
                         "peak_source": f"{peak_kind} copy bandwidth", "kernel_us": kavg * 1e3,
                         "launches_timed": len(kern_ms), "warmup_launches": ROOF_WARM,
                         "kernel_us_median": statistics.median(kern_ms) * 1e3,
                         "kernel_us_best": min(kern_ms) * 1e3},
        }
        if cpu_base is not None:
            result["cpu_baseline"] = cpu_base

    if not args.no_extras:
        extras = run_extras(args, inp, device, lib, stream, rank, world, nbytes, new_event)
        if rank == 0:
            result.update(extras)
        del inp, ws
        torch.cuda.empty_cache()
        more = run_wider_legs(args, device, rank, world)
        if rank == 0:
            result.update(more)
    if rank == 0:
        print(json.dumps(result))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_wider_legs(args, device, rank, world):
    """Legs beyond the headline step: the long-context sharded step (N > 1), the reference's own GPU code on the
    same box (N = 1), and end-to-end greedy decode tokens/s."""
    import torch
    import torch.distributed as dist
    from polarquant_b200 import benchmarks, e2e_decode
    out = {}
    peak, _ = measured_peak()
    if world > 1:
        # correctness of the one exchange of the path first, then its timing
        err = benchmarks.sequence_split_check(device, rank, world)
        out["seqsplit_check"] = "ok" if err <= 8e-3 else f"FAILED: max |diff| {err:.3e} against single-GPU attention"
        out["seqsplit_max_abs_err"] = err
        legs = benchmarks.long_context_legs(device, rank, world)
        for k in ("heads", "sequence"):
            legs[k]["pct_of_aggregate_measured_peak"] = 100.0 * legs[k]["aggregate_gbs"] / (world * peak)
            legs[k]["pct_of_aggregate_nominal_8TBs"] = 100.0 * legs[k]["aggregate_gbs"] / (world * NOMINAL_HBM_GBS)
        out["longctx"] = legs
        torch.cuda.empty_cache()
    elif rank == 0:
        try:
            out["reference_gpu"] = reference_gpu_legs(args, device)
        except Exception as e:                           # context figures must not take the bench line down
            out["reference_gpu"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.empty_cache()
    # ---- end-to-end greedy decode, batch 32 sharded over the replicas ----
    ns = argparse.Namespace(batch=32, prompt=8192, new_tokens=args.e2e_new_tokens, layers=32, prefill_chunk=2,
                            no_graph=False, vbits=0)
    if args.e2e_new_tokens > 1:
        rec = e2e_decode.run(ns, rank, world, device)
        floor_ms = rec["bytes_per_step_per_gpu"] / (peak * 1e9) * 1e3
        out["e2e_tokens"] = {
            "tokens_per_s": rec["decode_tokens_per_s"], "ms_per_step": rec["ms_per_decode_step"],
            "global_batch": 32, "prompt_tokens": 8192, "new_tokens": args.e2e_new_tokens, "n_gpus": world,
            "prefill_s": rec["prefill_s"], "cuda_graph": rec["cuda_graph"],
            "bytes_floor_ms_per_step": floor_ms,
            "model": "random-init Llama-3.1-8B shape (32 layers, hidden 4096, 32 q / 8 kv heads, rope theta 5e5, "
                     "bf16 weights ~N(0, 0.02)); torch ops around PolarKVCache, whole step replayed from one CUDA graph",
            "note": "every replica streams all weights each step, so with the total batch fixed the floor per step "
                    "only falls from (weights + cache)/peak at 1 GPU to (weights + cache/N)/peak at N"}
        torch.cuda.empty_cache()
        if world == 1 and rank == 0:
            try:
                out["e2e_tokens"]["reference_patch_path"] = reference_model_tokens(args, device)
            except Exception as e:
                out["e2e_tokens"]["reference_patch_path"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
            torch.cuda.empty_cache()
    return out


def _cuda_time_us(fn, reps, warm=3):
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps * 1e3


def reference_gpu_legs(args, device):
    """The reference's own GPU code on this GPU, for context: its Triton kernel through its own wrapper
    (models/kernel4group.py:83-109) beside pq_qk_decode on the same tensors, and its whole unmodified decode branch
    (models/modeling_llama_polar.py:61-101: Triton logits + eager concatenations, softmax, repeat_kv, P.V) beside
    the fused kernel.  Needs the reference's files (oracle/_ref)."""
    import torch
    import polarquant_b200 as pq
    from oracle import ref_harness
    from polarquant_b200 import dropin
    if ref_harness.ref_root() is None:
        return {"unavailable": "reference files not installed (python oracle/install_ref.py needs the checkout)"}
    refk = ref_harness.load_reference_kernel_module()
    out = {}
    g = torch.Generator(device=device).manual_seed(2)

    def qk_pair(tag, B, N, Nk, L, G, dt):
        q = torch.randn(B, N, 1, 128, device=device, generator=g).to(dt)
        idx = torch.randint(0, 250, (B, Nk, L // G, G, 64), device=device, generator=g, dtype=torch.uint8)
        sc = [torch.randn(B, Nk, L // G, 1, 64, device=device, generator=g).to(dt) for _ in range(4)]
        ours = _cuda_time_us(lambda: pq.attention_decode_forward_triton_impl(q, idx, *sc, rbits=4, tbits=4), 20)
        rec = {"shape": f"batch {B}, {N} q / {Nk} code heads, {L} keys, group {G}, {str(dt).split('.')[-1]}",
               "ours_qk_us": ours}
        try:
            a = refk.attention_decode_forward_triton_impl(q, idx, *sc, rbits=4, tbits=4)     # JIT
            b = pq.attention_decode_forward_triton_impl(q, idx, *sc, rbits=4, tbits=4)
            rec["max_abs_diff_vs_triton"] = float((a - b).abs().max())
            rec["logit_scale"] = float(a.abs().max())
            rec["triton_qk_us"] = _cuda_time_us(
                lambda: refk.attention_decode_forward_triton_impl(q, idx, *sc, rbits=4, tbits=4), 10)
            rec["speedup"] = rec["triton_qk_us"] / ours
        except Exception as e:
            rec["triton_error"] = f"{type(e).__name__}: {e}"[:300]
        out[tag] = rec

    # the reference's own micro-benchmark point (benchmark/benchmark_matmul.py:89-99: 32 heads on the codes, fp16,
    # group 32, random codes / scales) and the headline configuration's packed part
    qk_pair("qk_benchmark_matmul_b8_l131072", 8, 32, 32, 131072, 32, torch.float16)
    qk_pair("qk_headline_shape", args.batch, args.q_heads, args.kv_heads, args.ctx - 128, args.group, torch.bfloat16)

    # whole decode branch at the headline configuration, reference code unmodified (identity projections)
    inp = make_inputs(args, device, seed=1002)
    llama, _ = dropin.load_polar_patches(ref_harness.ref_root(), entry_module=refk)
    dt = torch.bfloat16
    attn = ref_harness.identity_attention(llama, "llama", args.q_heads, args.kv_heads, dt, device=device)
    past = (inp["kres"][:, :, :-1].contiguous(), *inp["packed"], inp["v"][:, :, :-1].contiguous(), args.ctx - 1)
    k_new, v_new = inp["kres"][:, :, -1:].contiguous(), inp["v"][:, :, -1:].contiguous()
    rec = {"shape": "headline configuration, one decode step"}
    rec["ours_decode_us"] = _cuda_time_us(
        lambda: pq.decode_attention(inp["q"], inp["kres"], *inp["packed"], inp["v"]), 20)
    try:
        ref_out, _ = ref_harness.decode_step(attn, inp["q"], k_new, v_new, past)
        ours = pq.decode_attention(inp["q"], inp["kres"], *inp["packed"], inp["v"])
        d = (ours.float() - ref_out.float()).abs()
        rec["max_abs_diff"], rec["mean_abs_diff"] = float(d.max()), float(d.mean())
        rec["reference_decode_us"] = _cuda_time_us(
            lambda: ref_harness.decode_step(attn, inp["q"], k_new, v_new, past), 5, warm=2)
        rec["speedup"] = rec["reference_decode_us"] / rec["ours_decode_us"]
        rec["note"] = ("reference: its Triton logits kernel + eager torch ops (concatenation of the value cache, "
                       "repeat_kv copies, softmax over (B, N, ctx) fp32 logits); includes three selection-matrix "
                       "projections of one token, a few tens of microseconds")
    except Exception as e:
        rec["reference_error"] = f"{type(e).__name__}: {e}"[:300]
    out["decode_branch"] = rec
    return out


def reference_model_tokens(args, device):
    """The unchanged reference path for the end-to-end figure: its LlamaPolarForCausalLM (random init, the
    Llama-3.1-8B architecture) driven by its own greedy ``generate`` (models/modeling_llama_polar.py:524-562,
    622-666), bound to the CUDA kernels through the module boundary only - torch.cat cache growth, repeat_kv
    copies and eager softmax stay as the reference wrote them."""
    import torch
    from oracle import ref_harness
    from polarquant_b200 import dropin
    from transformers import LlamaConfig
    if ref_harness.ref_root() is None:
        return {"unavailable": "reference files not installed"}
    llama, _ = dropin.load_polar_patches(ref_harness.ref_root())
    cfg = LlamaConfig(hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
                      num_key_value_heads=8, vocab_size=128256, rope_theta=500000.0, max_position_embeddings=131072,
                      initializer_range=0.02)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device(device):
            torch.manual_seed(1004)
            model = llama.LlamaPolarForCausalLM(cfg).eval()
    finally:
        torch.set_default_dtype(old)
    batch, prompt, new = 8, 8192, 17
    ids = torch.randint(0, 128256, (batch, prompt), device=device)
    gen_cfg = argparse.Namespace(eos_token_id=[-1], top_k=0, top_p=1.0, temperature=1.0)
    # prefill + 1 token, then prefill + `new` tokens: the difference is the decode time of new - 1 steps
    times = []
    for n in (1, new):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        llama.generate(model, ids, None, gen_cfg, do_sample=False, max_new_tokens=n)
        torch.cuda.synchronize()
        times.append(time.perf_counter() - t0)
    step_s = (times[1] - times[0]) / (new - 1)
    del model
    return {"tokens_per_s": batch / step_s, "ms_per_step": step_s * 1e3, "batch": batch, "prompt_tokens": prompt,
            "new_tokens": new, "prefill_plus_first_token_s": times[0],
            "note": "reference LlamaPolarForCausalLM + generate, unmodified, on the CUDA quantizer and logits entry; "
                    "batch 8 (its decode step re-materialises the value cache per layer)"}


def run_extras(args, inp, device, lib, stream, rank, world, nbytes, new_event):
    """End-to-end leg (host buffers through the C ABI) and the quantizer timing."""
    import torch
    import torch.distributed as dist
    import polarquant_b200 as pq
    from polarquant_b200 import _lib
    B, N, Nk, Nb, G, R = (inp[k] for k in ("B", "N", "Nk", "Nb", "G", "R"))
    out = {}

    # ---- e2e: every input in pinned host memory, H2D + kernels + D2H inside the timed region ----
    host = {k: inp[k].cpu().contiguous().pin_memory() for k in ("q", "kres", "v")}
    hpacked = [t.cpu().contiguous().pin_memory() for t in inp["packed"]]
    hout = torch.empty(B, N, 1, 128, dtype=torch.bfloat16).pin_memory()
    p = _lib.DecodeParams()
    p.q, p.k_res, p.v, p.out = host["q"].data_ptr(), host["kres"].data_ptr(), host["v"].data_ptr(), hout.data_ptr()
    p.codes, p.rscale, p.rmn, p.tscale, p.tmn = (t.data_ptr() for t in hpacked)
    p.B, p.N, p.Nk, p.Nb, p.G, p.R, p.hd = B, N, Nk, Nb, G, R, 128
    p.rbits, p.tbits = args.rbits, args.tbits
    p.qk_dtype = p.v_dtype = p.out_dtype = _lib.PQ_BF16
    need = lib.pq_decode_host_staging_bytes(B, N, Nk, Nb, G, R, 128, _lib.PQ_BF16, _lib.PQ_BF16, _lib.PQ_BF16, 0)
    staging = torch.empty(need, dtype=torch.uint8, device=device)
    h2d = sum(t.numel() * t.element_size() for t in [*host.values(), *hpacked])
    d2h = hout.numel() * hout.element_size()
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step():
        rc = lib.pq_decode_attention_host(ctypes.byref(p), staging.data_ptr(), need, stream)
        assert rc == 0, lib.pq_strerror(rc)

    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    a, b = new_event(), new_event()
    lib.pq_event_record(a, stream)
    for _ in range(e2e_steps):
        e2e_step()
    lib.pq_event_record(b, stream)
    torch.cuda.synchronize(device)
    ms = ctypes.c_float()
    lib.pq_event_elapsed_ms(a, b, ctypes.byref(ms))
    e2e_ms = ms.value / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    got = pq.decode_attention(inp["q"], inp["kres"], *inp["packed"], inp["v"], rbits=args.rbits, tbits=args.tbits)
    if not torch.equal(hout.to(device), got):
        d = (hout.to(device).float() - got.float()).abs()
        raise AssertionError(f"host-buffer entry point disagrees with the device entry point: "
                             f"{int((hout.to(device) != got).sum())} elements, max |diff| {float(d.max()):.3e}")
    out["e2e"] = {"value": nbytes * world / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                  "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps,
                  "note": "pq_decode_attention_host: the whole cache of the step is copied from pinned host memory "
                          "each step, so this leg is bound by the host link, not by the kernels"}
    del staging, host, hpacked

    # ---- serving-style step on the in-place cache: only the step's own inputs cross the host link ----
    from polarquant_b200.cache import PolarKVCache
    res_steps = max(8, min(args.steps, 100))
    ctx0 = Nb * G + R - res_steps                      # the timed steps end at the benchmark context
    lengths = torch.zeros(2, dtype=torch.int32, device=device)
    cache = PolarKVCache(B, Nk, max_tokens=Nb * G + R + 128, dtype=torch.bfloat16, device=device, rbits=args.rbits,
                         tbits=args.tbits, group_size=G, lengths=lengths)
    gen = torch.Generator(device=device).manual_seed(11 + rank)
    for b0 in range(0, B, 4):                          # prefill in slices to bound temporaries
        kb = torch.randn(min(4, B - b0), Nk, ctx0, 128, device=device, generator=gen).to(torch.bfloat16)
        cache.prefill(kb, inp["v"][b0:b0 + 4, :, :ctx0], batch_start=b0)
    cache.sync_lengths()
    hq = torch.randn(B, N, 1, 128).to(torch.bfloat16).pin_memory()
    hk = torch.randn(B, Nk, 1, 128).to(torch.bfloat16).pin_memory()
    hv = torch.randn(B, Nk, 1, 128).to(torch.bfloat16).pin_memory()
    dq, dk, dv = (torch.empty_like(t, device=device) for t in (hq, hk, hv))
    dout = torch.empty(B, N, 1, 128, dtype=torch.bfloat16, device=device)
    hres = torch.empty(B, N, 1, 128, dtype=torch.bfloat16).pin_memory()

    def resident_step():
        # host -> device copies of the step's inputs, append + fused attention with the lengths read on the
        # device, advance of the lengths, device -> host copy of the result
        dq.copy_(hq, non_blocking=True); dk.copy_(hk, non_blocking=True); dv.copy_(hv, non_blocking=True)
        cache.decode_step_graph(dq, dk, dv, out=dout)
        lengths[1:2].add_(1)
        hres.copy_(dout, non_blocking=True)

    # one captured graph replayed per step (what a serving loop does); eager launches if capture is refused
    replay, graphed = resident_step, False
    try:
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            resident_step()
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        cache.sync_lengths()                           # the warm-up step is discarded
        cg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cg):
            resident_step()
        replay, graphed = cg.replay, True
    except Exception:
        torch.cuda.synchronize(device)
        cache.sync_lengths()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    a, b = new_event(), new_event()
    lib.pq_event_record(a, stream)
    for i in range(res_steps):
        replay()
        if cache.after_replay():                       # window full: re-quantised in place, outside the graph
            cache.sync_lengths()
    lib.pq_event_record(b, stream)
    torch.cuda.synchronize(device)
    lib.pq_event_elapsed_ms(a, b, ctypes.byref(ms))
    res_ms = ms.value / res_steps
    if world > 1:
        t = torch.tensor([res_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res_ms = float(t.item())
    out["e2e_resident_cache"] = {
        "value": nbytes * world / (res_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": res_ms, "steps": res_steps,
        "tokens_per_s_per_layer": B * world / (res_ms * 1e-3),
        "h2d_bytes_per_step": (dq.numel() + dk.numel() + dv.numel()) * 2, "d2h_bytes_per_step": hres.numel() * 2,
        "cuda_graph": graphed,
        "note": "PolarKVCache.decode_step_graph: query / new key / new value copied from pinned host memory, appended "
                "in place, fused attention over the resident cache with the lengths read on the device (window "
                "re-quantised in place when full), output copied back - one captured graph replayed per step; "
                "context ends at the benchmark context"}
    del cache

    # ---- the same step repeated for about half a second: the power-capped regime ----
    if rank == 0 and world == 1:
        ws2 = torch.empty(lib.pq_decode_workspace_bytes(B, N, Nk, Nb, G, R, 0) + 256, dtype=torch.uint8, device=device)
        long_steps = 2000
        sampler3 = ClockSampler(torch.cuda.current_device())
        sampler3.start()
        for _ in range(20):
            pq.decode_attention(inp["q"], inp["kres"], *inp["packed"], inp["v"], rbits=args.rbits, tbits=args.tbits,
                                workspace=ws2)
        a, b = new_event(), new_event()
        lib.pq_event_record(a, stream)
        for _ in range(long_steps):
            pq.decode_attention(inp["q"], inp["kres"], *inp["packed"], inp["v"], rbits=args.rbits, tbits=args.tbits,
                                workspace=ws2)
        lib.pq_event_record(b, stream)
        lib.pq_event_elapsed_ms(a, b, ctypes.byref(ms))
        s_ms = ms.value / long_steps
        out["sustained"] = {"steps": long_steps, "us_per_step": s_ms * 1e3, "gbs": nbytes / (s_ms * 1e-3) / 1e9,
                            "pct_of_nominal_8TBs": 100.0 * nbytes / (s_ms * 1e-3) / 1e9 / NOMINAL_HBM_GBS,
                            "clocks": sampler3.stop(),
                            "note": "the timed step repeated 2000 times back to back; under sw_power_cap the SM "
                                    "clock, and with it this issue-bound kernel, drops"}
        del ws2
        time.sleep(1.0)                                # let the clocks recover before the next leg

    # ---- context for the roofline: a plain device copy run as long as the sustained leg (same power regime) ----
    if rank == 0:
        src = torch.empty(1 << 30, dtype=torch.uint8, device=device)
        dst = torch.empty_like(src)
        for _ in range(3):
            dst.copy_(src)
        reps = max(10, int(0.5 / (2 * src.numel() / 6.0e12)))
        sampler2 = ClockSampler(torch.cuda.current_device())
        sampler2.start()
        a, b = new_event(), new_event()
        lib.pq_event_record(a, stream)
        for _ in range(reps):
            dst.copy_(src)
        lib.pq_event_record(b, stream)
        lib.pq_event_elapsed_ms(a, b, ctypes.byref(ms))
        out["sustained_copy"] = {"gbs": 2 * src.numel() * reps / (ms.value * 1e-3) / 1e9, "seconds": ms.value / 1e3,
                                 "clocks": sampler2.stop(),
                                 "note": "torch copy of 1 GiB (read + write bytes) repeated for ~0.5 s: the copy "
                                         "bandwidth in the power regime of the long timed region"}
        del src, dst

    # ---- quantizer at a 32k-token prefill, strided (B, L, Nk, hd) layout as the prefill hands it over ----
    if rank == 0:
        L = args.ctx
        g = torch.Generator(device=device).manual_seed(7)
        base = torch.randn(B, L, Nk, 128, device=device, generator=g).to(torch.bfloat16)
        keys = base.transpose(1, 2)
        for _ in range(3):
            pq.quantize_and_pack_nbit(keys, args.rbits, args.tbits, G)
        torch.cuda.synchronize(device)
        a, b = new_event(), new_event()
        reps = 10
        lib.pq_event_record(a, stream)
        for _ in range(reps):
            pq.quantize_and_pack_nbit(keys, args.rbits, args.tbits, G)
        lib.pq_event_record(b, stream)
        lib.pq_event_elapsed_ms(a, b, ctypes.byref(ms))
        q_ms = ms.value / reps
        q_bytes = B * Nk * L * 128 * 2 + B * Nk * (L * 64 + (L // G) * 4 * 64 * 2)
        peak, _ = measured_peak()
        out["quantizer"] = {"workload": f"{L}-token prefill, batch {B}, {Nk} kv heads, bf16, strided (B, L, Nk, hd)",
                            "us": q_ms * 1e3, "algorithmic_mb": q_bytes / 1e6,
                            "gbs": q_bytes / (q_ms * 1e-3) / 1e9, "frac_of_peak": q_bytes / (q_ms * 1e-3) / 1e9 / peak}
        del base, keys

    # ---- the same step with the values packed to 4 bits as well (the reference's mixed key/value class) ----
    if rank == 0:
        Lq = Nb * G
        vq = inp["v"][:, :, :Lq]
        for _ in range(2):
            vc, vs, vm = pq.quantize_values(vq, layout="tiled")
        a, b = new_event(), new_event()
        lib.pq_event_record(a, stream)
        for _ in range(5):
            pq.quantize_values(vq, layout="tiled")
        lib.pq_event_record(b, stream)
        lib.pq_event_elapsed_ms(a, b, ctypes.byref(ms))
        vq_ms = ms.value / 5
        v_res = inp["v"][:, :, Lq:].contiguous()
        kw = dict(rbits=args.rbits, tbits=args.tbits, value_codes=vc, value_scale=vs, value_mn=vm)
        for _ in range(3):
            pq.decode_attention(inp["q"], inp["kres"], *inp["packed"], v_res, **kw)
        reps = 50
        lib.pq_event_record(a, stream)
        for _ in range(reps):
            pq.decode_attention(inp["q"], inp["kres"], *inp["packed"], v_res, **kw)
        lib.pq_event_record(b, stream)
        lib.pq_event_elapsed_ms(a, b, ctypes.byref(ms))
        p_ms = ms.value / reps
        # and for half a second, like the `sustained` leg
        long_p = 2000 if world == 1 else 0
        sus = None
        if long_p:
            time.sleep(1.0)
            sampler4 = ClockSampler(torch.cuda.current_device())
            sampler4.start()
            lib.pq_event_record(a, stream)
            for _ in range(long_p):
                pq.decode_attention(inp["q"], inp["kres"], *inp["packed"], v_res, **kw)
            lib.pq_event_record(b, stream)
            lib.pq_event_elapsed_ms(a, b, ctypes.byref(ms))
            sus = {"steps": long_p, "us_per_step": ms.value / long_p * 1e3, "clocks": sampler4.stop()}
        p_bytes = nbytes - vq.numel() * 2 + vc.numel() * 4 + 2 * vs.numel() * 2
        vq_bytes = vq.numel() * 2 + vc.numel() * 4 + 2 * vs.numel() * 2
        out["packed_values"] = {"us_per_step": p_ms * 1e3, "algorithmic_mb": p_bytes / 1e6,
                                "gbs": p_bytes / (p_ms * 1e-3) / 1e9,
                                "bytes_per_token_per_kv_head": 64 + 4 + 64 + 4,
                                "sustained": sus,
                                "value_quantizer_us": vq_ms * 1e3, "value_quantizer_gbs": vq_bytes / (vq_ms * 1e-3) / 1e9,
                                "note": "4-bit per-token values fused into the P.V loop: 2.4x less cache, same step "
                                        "time in a burst - the step is bound by instruction issue, not by bytes - "
                                        "and no power throttling in the sustained run"}
    return out


if __name__ == "__main__":
    main()
