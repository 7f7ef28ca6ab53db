"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload decode|prefill|longctx|ragged]

Default workload (`decode`) is the batched decode configuration: 64 independent sequences with 8192 cached tokens
each on one full-attention layer, Q/K/V rows bf16, fp16 KV cache, RMSNorm + RoPE + KV write fused in.  One step = one
decode-attention pass over the whole batch, positions advancing by one each step.  With N GPUs the 64 sequences are
cut into contiguous blocks of 64/N, one block per rank (strong scaling); sequences are independent, so there is no
collective on the data path.  When one rank's block of KV is not several times larger than L2, the rank keeps
several copies of its block and rotates over them, so that every step reads its keys from HBM.  One JSON line is
printed by rank 0; on several GPUs it also carries the weak-scaling figure (64 sequences on every rank).

`--impl reference` times the CPU restatement of the reference's src/ref attention (the oracle) on the host cores
for the same configuration, on a bounded sample of sequences.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_SEQ, CTX, QKV_DIM, OUT_DIM = 64, 8192, 5120, 4096
KV_BYTES_PER_KEY = 2048  # K + V, 4 KV heads x 128 dims x fp16, each read once per GQA group
PREFILL_T = 4000
L2_BYTES = 126 << 20
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one launch, from an ncu capture of one launch of the
# workload on this part: the decode kernel on 64 sequences x 8192 cached tokens, and the prefill attention kernel on
# the 4000-token sliding-window prompt.  --traffic-from replaces the decode figure with one read from an ncu CSV.
DECODE_NCU_DRAM_BYTES_PER_LAUNCH = 1082838000 + 4117760
PREFILL_NCU_DRAM_BYTES_PER_LAUNCH = 41030400 + 1144320
DECODE_WORKLOAD = ("decode: 64 seqs x 8192 cached tokens, 1 full layer, 32q/4kv heads x 128, bf16 qkv rows, "
                   "fp16 KV cache, norm+RoPE+KV write fused")


def decode_config(world: int) -> dict:
    """The `config` object of the decode workload; the repo arm and the reference arm print the same one."""
    return {"workload": DECODE_WORKLOAD, "seqs_total": N_SEQ, "cached_tokens": CTX,
            "sharding": f"contiguous blocks of {N_SEQ}/{world} sequences per GPU, no collective on the data path",
            "l2": "every step reads its KV from HBM: the block of one rank is larger than L2, or the rank rotates "
                  "over copies of its block that together are"}


def layer_params(seed: int):
    """Seeded layer parameters of the synthetic workload: q_norm, k_norm ~ 1 + N(0, 0.1) [128], sinks ~ N(0, 1) [32]."""
    rng = np.random.default_rng(seed)
    return ((1 + 0.1 * rng.standard_normal(128)).astype(np.float32),
            (1 + 0.1 * rng.standard_normal(128)).astype(np.float32), rng.standard_normal(32).astype(np.float32))


def traffic_from_csv(path: str, kernel_substr: str):
    """dram__bytes_read.sum + dram__bytes_write.sum of the first launch whose kernel name contains kernel_substr, from
    `ncu --csv --page raw` output (one row per launch, one column per metric)."""
    import csv

    with open(path, newline="") as f:
        rows = [r for r in csv.reader(f) if r]
    hdr = next(r for r in rows if "Kernel Name" in r)
    i_name = hdr.index("Kernel Name")
    i_rd, i_wr = hdr.index("dram__bytes_read.sum"), hdr.index("dram__bytes_write.sum")
    units = rows[rows.index(hdr) + 1]
    scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}
    for r in rows[rows.index(hdr) + 2:]:
        if kernel_substr in r[i_name]:
            return int(float(r[i_rd].replace(",", "")) * scale.get(units[i_rd], 1.0) +
                       float(r[i_wr].replace(",", "")) * scale.get(units[i_wr], 1.0))
    return None


def decode_bytes(n_seq: int, n_cached: int) -> int:
    """Algorithmic HBM bytes of one decode step: cached K/V once per KV head, q|k|v row in (bf16),
    new K/V written (fp16), output row out (bf16)."""
    return n_seq * (KV_BYTES_PER_KEY * n_cached + QKV_DIM * 2 + 2 * 512 * 2 + OUT_DIM * 2)


def prefill_flops(n_tok: int, window: int = 513, p0: int = 0) -> int:
    """4 * 128 * 32 * sum_p min(p+1, window): QK^T and PV over the causal band only (window = 0: no window), for the
    positions p0 .. p0+n_tok-1."""
    p = np.arange(p0, p0 + n_tok, dtype=np.int64)
    keys = np.minimum(p + 1, window) if window else p + 1
    return int(4 * 128 * 32 * keys.sum())


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx, self.rows, self._stop, self._t = gpu_index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                r = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                    "-i", str(self.idx)], capture_output=True, text=True, timeout=5)
                if r.returncode == 0 and r.stdout.strip():
                    self.rows.append([x.strip() for x in r.stdout.strip().split(",")])
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=10)

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = max(mx, float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


def dist_setup(n_gpus: int):
    import torch

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def barrier(world):
    import torch

    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch
    import torch.distributed as dist

    t = torch.tensor([x], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch
    import torch.distributed as dist

    t = torch.tensor([x], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def as_tensor(torch, ptr, numel, dtype):
    """torch view (no copy) of device memory owned by the library."""
    class H:
        pass

    h = H()
    h.__cuda_array_interface__ = {"shape": (numel * torch.empty((), dtype=dtype).element_size(),), "typestr": "|u1",
                                  "data": (ptr, False), "version": 3}
    return torch.as_tensor(h, device="cuda").view(dtype)


# ----------------------------------------------------------------------------------------------- CPU arm
class CpuDecodeSample:
    """n_sample sequences of the decode workload for the oracle (src/ref arithmetic): the fp16 K/V caches are drawn once
    (drawing 4 M normals per sequence costs ten times the attention itself); every step decodes a fresh q/k/v row on
    each of them.  step() returns seconds per sequence-token."""

    def __init__(self, seed: int, n_sample: int, n_cached: int, n_threads: int):
        from oracle import oracle as fo

        self.fo, self.n_cached, self.n_threads = fo, n_cached, n_threads
        self.w = fo.layer_weights(seed, 0)
        self.rng = np.random.default_rng(seed)
        self.kv = []
        for _ in range(n_sample):
            k16 = fo.to_f16_bits(self.rng.standard_normal((4, n_cached + 1, 128), dtype=np.float32))
            v16 = fo.to_f16_bits(self.rng.standard_normal((4, n_cached + 1, 128), dtype=np.float32))
            self.kv.append((k16, v16))

    def step(self, reps: int = 1) -> float:
        fo, times = self.fo, []
        for k16, v16 in self.kv:
            row = fo.round_bf16(self.rng.standard_normal(QKV_DIM, dtype=np.float32))
            for _ in range(reps):
                t0 = time.perf_counter()
                fo.decode_token_f16cache(row, self.n_cached, *self.w, False, True, k16, v16, n_threads=self.n_threads)
                times.append(time.perf_counter() - t0)
        return float(np.mean(times))


def cpu_decode_sample(seed: int, n_sample: int, n_cached: int, n_threads: int, reps: int = 1):
    """One step of a fresh CpuDecodeSample; returns seconds per sequence-token."""
    return CpuDecodeSample(seed, n_sample, n_cached, n_threads).step(reps)


def run_reference(args):
    """The reference's CPU attention (oracle port) for the decode workload on all host cores, bounded sample per step.
    Rank 0 alone works; the line carries the same metric and config as the repo arm."""
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    n_sample = 4
    sample = CpuDecodeSample(1, n_sample, CTX, cores)
    for _ in range(args.warmup):
        sample.step()
    t0 = time.perf_counter()
    per_seq = []
    for k in range(args.steps):
        per_seq.append(sample.step())
    wall = time.perf_counter() - t0
    sec_per_seq = float(np.mean(per_seq))
    gbs = decode_bytes(1, CTX) / sec_per_seq / 1e9
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec_per_seq * N_SEQ * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": decode_config(max(world, args.gpus)),
        "timed_sample": f"{n_sample} of {N_SEQ} sequences per step, scaled to {N_SEQ}",
        "tok_per_s": 1.0 / sec_per_seq,
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"{n_sample} of {N_SEQ} sequences per step x {args.steps} steps, OpenMP over heads"},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": wall,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------- GPU arm
def measure_prefill(torch, fa, local, iters: int, warmup: int, T: int = PREFILL_T, swa: bool = True,
                    history: int = 0):
    """Prefill workload: one T-token prompt (default 4000) on a sliding-window layer (window 512 + sink, causal; K/V
    into the 1024-slot ring) or, with swa=False, on a full-attention layer (causal over the whole prompt), bf16 q/k/v
    rows, positions 0..T-1.  L2 is flushed between iterations.  Returns a dict."""
    _, tensor_peak, peak_kind = measured_peaks()
    h = fa.Attn([swa], [True], 1, history + T + 96, device=local)
    h.set_layer(0, *layer_params(0))
    gen = torch.Generator(device="cuda").manual_seed(4321)
    if history:  # a chunk of a longer prompt: the cache already holds `history` tokens
        for which in (0, 1):
            as_tensor(torch, h.kv_dev(0, which), 4 * h.n_slots(0) * 128, torch.float16).normal_(generator=gen)
    qkv = torch.randn(T, QKV_DIM, generator=gen, device="cuda").to(torch.bfloat16)
    out = torch.empty(T, OUT_DIM, device="cuda", dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # Two passes over the same work.  The first runs bare, an event pair around the whole prefill: the step as a
    # caller sees it (the attention kernel is scheduled while the prologue drains).  The second has the library put an
    # event pair around the attention kernel, which gives that kernel's own duration but keeps it from starting early.
    step_ms = []
    for timing in (False, True):
        h.set_timing(timing)
        for i in range(warmup + iters):
            h.set_pos(0, history)
            flush.fill_(i & 0xFF)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if i == warmup:
                torch.cuda.synchronize()
                h.kernel_ms()  # drop the warm-up records
                launches0 = h.launch_count()
            e0.record()
            h.prefill_dev(0, 0, T, qkv, fa.BF16, out, fa.BF16, stream)
            e1.record()
            if i >= warmup and not timing:
                step_ms.append((e0, e1))
        torch.cuda.synchronize()
    attn_ms, n = h.kernel_ms()
    launches_per_step = (h.launch_count() - launches0) // max(iters, 1)
    h.set_timing(False)
    h.check()
    attn_us = attn_ms / max(n, 1) * 1e3
    step_us = float(np.median([a.elapsed_time(b) for a, b in step_ms])) * 1e3
    flops = prefill_flops(T, 513 if swa else 0, history)
    tflops = flops / (attn_us * 1e-6) / 1e12
    # end to end through the host-buffer entry point
    qkv_host, out_host = qkv.cpu().pin_memory(), torch.empty(T, OUT_DIM, dtype=torch.bfloat16).pin_memory()
    e2e = []
    for i in range(3 + min(iters, 10)):
        h.set_pos(0, history)
        t0 = time.perf_counter()
        h.prefill(0, 0, T, qkv_host, fa.BF16, out_host, fa.BF16)
        e2e.append(time.perf_counter() - t0)
    e2e_us = float(np.median(e2e[3:])) * 1e6
    h.close()
    kind = "SWA layer (window 512 + sink, causal), bf16 rows, ring write" if swa else \
        "full-attention layer (causal + sink), bf16 rows, cache write"
    what = f"one {T}-token prompt" if not history else f"a {T}-token chunk after {history} cached tokens"
    return {"workload": f"prefill: {what}, {kind}",
            "algorithmic_flops": flops, "attn_kernel_us": attn_us, "tflops": tflops, "peak_tflops": tensor_peak,
            "frac": tflops / tensor_peak, "peak_kind": f"of {peak_kind} (burst)", "step_us": step_us,
            "tok_per_s": T / (step_us * 1e-6), "iters": n, "l2": "flushed between iterations (256 MiB write)",
            "e2e_us": e2e_us, "e2e_tok_per_s": T / (e2e_us * 1e-6), "e2e_tflops": flops / (e2e_us * 1e-6) / 1e12,
            "h2d_bytes_per_step": T * QKV_DIM * 2, "d2h_bytes_per_step": T * OUT_DIM * 2,
            "gpu_launches_per_step": launches_per_step, "checksum": float(out_host.float().abs().mean())}


def decode_pass(torch, fa, h, local, world, n_loc, copies, args, hbm_peak, with_e2e=True):
    """Times args.steps decode steps of n_loc sequences per rank (device-resident rows), then the same steps through
    the host-buffer entry point.  The rank holds `copies` copies of its block of sequences and rotates over them.
    Returns a dict of this rank's / the job's figures (collectives inside: every rank must call it)."""
    total_steps = args.warmup + args.steps
    blocks = [fa.i32_array(list(range(c * n_loc, (c + 1) * n_loc))) for c in range(copies)]
    gen = torch.Generator(device="cuda").manual_seed(4242 + int(os.environ.get("RANK", 0)))
    qkv = torch.randn(total_steps, n_loc, QKV_DIM, generator=gen, device="cuda").to(torch.bfloat16)
    out = torch.empty(n_loc, OUT_DIM, device="cuda", dtype=torch.bfloat16)
    stream = torch.cuda.current_stream().cuda_stream
    pos = [CTX] * copies  # cached tokens of the sequences of each copy

    def reset():
        for c in range(copies):
            pos[c] = CTX
            for s in range(c * n_loc, (c + 1) * n_loc):
                h.set_pos(s, CTX)

    # a serving loop decodes the same batch every step: everything but the rows' address is converted once
    dec = [h.prepared_decode_dev(0, blocks[c], fa.BF16, out, fa.BF16, stream) for c in range(copies)]
    adv = [h.prepared_advance(blocks[c], 1) for c in range(copies)]
    row_addr = [qkv[i].data_ptr() for i in range(total_steps)]

    def step(i):
        c = i % copies
        dec[c](row_addr[i])
        adv[c]()
        pos[c] += 1

    # ---- device-resident throughput ("value")
    reset()
    for i in range(args.warmup):
        step(i)
    barrier(world)
    # The timed region runs bare: two events around all K steps.  A step is ONE launch of the decode kernel, so the
    # region divided by the launches is that kernel's average duration in steady state (launch i+1 is scheduled while
    # launch i still runs and waits, inside the kernel, for it to complete).  An event pair around every launch keeps
    # the next launch from being scheduled early and reads several microseconds longer per launch; that figure is taken
    # afterwards, over the same steps, and reported beside the first as kernel_us_isolated.
    h.set_timing(False)
    launches0 = h.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    bytes_loc = 0
    clk = ClockSampler(local)
    clk.__enter__()
    # the host side of a step is two prepared calls; everything else is worked out before the clock starts (at 8
    # sequences per GPU a step is under 30 us of device time)
    plan = []
    for i in range(args.warmup, args.warmup + args.steps):
        c = i % copies
        bytes_loc += decode_bytes(n_loc, pos[c])
        pos[c] += 1
        plan.append((dec[c], adv[c], row_addr[i]))
    import gc

    gc_was_on = gc.isenabled()
    gc.disable()
    ev0.record()
    for dec_c, adv_c, addr in plan:
        dec_c(addr)
        adv_c()
    ev1.record()
    if gc_was_on:
        gc.enable()
    barrier(world)
    ms_local = ev0.elapsed_time(ev1)
    ms_total = max_over_ranks(ms_local, world)
    launches = h.launch_count() - launches0
    reset()
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    h.set_timing(True)
    for i in range(args.steps):
        step(args.warmup + i)
    torch.cuda.synchronize()
    kernel_ms, n_timed = h.kernel_ms()
    h.set_timing(False)
    bytes_loc /= args.steps                       # this rank's algorithmic bytes per step
    bytes_all = sum_over_ranks(bytes_loc, world)  # the job's
    ms_per_step = ms_total / args.steps
    kernel_ms_avg = ms_local / max(launches, 1)   # this rank's launches over this rank's timed region
    res = {"ms_per_step": ms_per_step, "value": bytes_all / (ms_per_step * 1e-3) / 1e9, "bytes_per_step": bytes_all,
           "bytes_per_launch": bytes_loc, "kernel_us": kernel_ms_avg * 1e3,
           "kernel_timed": "timed region / launches (one k_decode_attn launch per step, two events around the region)",
           "kernel_us_isolated": kernel_ms / max(n_timed, 1) * 1e3,
           "achieved": bytes_loc / (kernel_ms_avg * 1e-3) / 1e9, "launches": launches,
           "n_seq_all": int(round(sum_over_ranks(n_loc, world)))}
    if with_e2e:
        # ---- end to end through the host-buffer entry point: pinned host rows in, host rows out, every step
        reset()
        qkv_host = qkv.cpu().pin_memory()
        out_host = torch.empty(n_loc, OUT_DIM, dtype=torch.bfloat16).pin_memory()
        for i in range(args.warmup):
            h.decode(0, blocks[i % copies], qkv_host[i], fa.BF16, out_host, fa.BF16)
            h.advance(blocks[i % copies], 1)
        barrier(world)
        t0 = time.perf_counter()
        for i in range(args.steps):
            c = (args.warmup + i) % copies
            h.decode(0, blocks[c], qkv_host[args.warmup + i], fa.BF16, out_host, fa.BF16)
            h.advance(blocks[c], 1)
        barrier(world)
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3, world) / args.steps
        res.update({"e2e_ms": e2e_ms, "e2e_value": bytes_all / (e2e_ms * 1e-3) / 1e9,
                    "checksum": float(out_host.float().abs().mean())})
    clk.__exit__()
    res["clocks"] = clk.summary()
    return res


def open_decode_handle(torch, fa, local, n_loc, copies, total_steps, seed):
    h = fa.Attn([False], [True], n_loc * copies, CTX + total_steps + 8, device=local)
    h.set_layer(0, *layer_params(0))
    gen = torch.Generator(device="cuda").manual_seed(seed)
    for which in (0, 1):
        as_tensor(torch, h.kv_dev(0, which), n_loc * copies * 4 * h.n_slots(0) * 128, torch.float16).normal_(generator=gen)
    return h


def run_decode(args):
    import torch

    import flint_mac_b200 as fa
    from flint_mac_b200 import shard

    rank, world, local = dist_setup(args.gpus)
    hbm_peak, _, peak_kind = measured_peaks()
    total_steps = args.warmup + args.steps
    # strong scaling: the 64 sequences in contiguous blocks, one per rank
    # --emulate-world N (single GPU only): run rank 0's block of an N-way sharding, to look at the per-GPU step of a
    # multi-GPU run without the other GPUs; the line then counts this block only
    place_world = args.emulate_world if (world == 1 and args.emulate_world > 1) else world
    b0, b1 = shard.contiguous_blocks(N_SEQ, place_world)[rank]
    n_loc = b1 - b0
    block_kv = n_loc * CTX * KV_BYTES_PER_KEY
    copies = max(1, -(-4 * L2_BYTES // block_kv))  # the copies together are at least four times L2
    h = open_decode_handle(torch, fa, local, n_loc, copies, total_steps, 1234 + rank)
    strong = decode_pass(torch, fa, h, local, world, n_loc, copies, args, hbm_peak)
    h.close()
    weak = None
    if world > 1:  # the weak-scaling figure: 64 sequences on every rank
        h = open_decode_handle(torch, fa, local, N_SEQ, 1, total_steps, 4321 + rank)
        weak = decode_pass(torch, fa, h, local, world, N_SEQ, 1, args, hbm_peak, with_e2e=False)
        h.close()
    prefill = None
    if not args.skip_prefill and rank == 0:
        with ClockSampler(local) as clk_pf:
            prefill = measure_prefill(torch, fa, local, iters=30, warmup=5)
        prefill["clocks"] = clk_pf.summary()
        prefill["roofline"] = {"bound": "tensor", "achieved": prefill["tflops"], "peak": prefill["peak_tflops"],
                               "unit": "TFLOP/s", "frac": prefill["frac"], "traffic": PREFILL_NCU_DRAM_BYTES_PER_LAUNCH,
                               "peak_kind": prefill["peak_kind"], "kernel": "k_prefill_attn",
                               "kernel_us": prefill["attn_kernel_us"], "flops_per_launch": prefill["algorithmic_flops"]}
    barrier(world)

    line = None
    if rank == 0:
        cpu_baseline = None
        if world == 1:  # the CPU baseline is timed at N = 1 only
            cores = os.cpu_count() or 1
            t_cpu0 = time.perf_counter()
            sec_per_seq = cpu_decode_sample(0, 1 if args.skip_cpu else 4, CTX, cores, reps=1 if args.skip_cpu else 2)
            # the reference runs its CPU attention on one thread (threads only in matvec, src/ref/ref_model.cpp:85-92)
            sec_1t = None if args.skip_cpu else cpu_decode_sample(1, 1, CTX, 1, reps=1)
            cpu_baseline = {"value": decode_bytes(1, CTX) / sec_per_seq / 1e9, "unit": "GB/s", "cores": cores,
                            "kind": "port",
                            "sample": "4 of 64 sequences x 2 repeats of the same step, OpenMP over heads",
                            "tok_per_s": 1.0 / sec_per_seq, "wall_s": time.perf_counter() - t_cpu0,
                            "single_thread": None if sec_1t is None else
                            {"value": decode_bytes(1, CTX) / sec_1t / 1e9, "unit": "GB/s", "cores": 1,
                             "sample": "1 of 64 sequences, one thread (how the reference runs attention)"}}
        traffic = DECODE_NCU_DRAM_BYTES_PER_LAUNCH
        traffic_source = "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of the 64-sequence workload"
        if args.traffic_from:
            traffic = traffic_from_csv(args.traffic_from, "k_decode_attn")
            traffic_source = f"ncu capture {os.path.basename(args.traffic_from)}"
        if traffic is not None and n_loc != N_SEQ:  # traffic grows with the sequences a launch scans
            traffic = int(traffic * n_loc / N_SEQ)
            traffic_source += f", scaled by {n_loc}/{N_SEQ} sequences per launch"
        line = {
            "metric": "decode_attn_hbm_gbs", "value": strong["value"], "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": strong["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 KV, f16 tensor-core products, f32 accumulate/softmax", "data": "synthetic",
            "config": decode_config(world),
            "seqs_per_gpu": n_loc, "kv_copies_rotated": copies,
            **({"emulated": f"rank 0's block of a {place_world}-way sharding on one GPU; value counts this block only"}
               if place_world != world else {}),
            "tok_per_s": (n_loc if place_world != world else N_SEQ) / (strong["ms_per_step"] * 1e-3),
            "pct_of_hbm_peak": 100.0 * strong["value"] / world / hbm_peak,
            "roofline": {"bound": "hbm", "achieved": strong["achieved"], "peak": hbm_peak, "unit": "GB/s",
                         "frac": strong["achieved"] / hbm_peak, "traffic": traffic, "traffic_source": traffic_source,
                         "peak_kind": f"of {peak_kind}", "kernel": "k_decode_attn (rank 0's launch)",
                         "kernel_us": strong["kernel_us"], "kernel_timed": strong["kernel_timed"],
                         "kernel_us_isolated": strong["kernel_us_isolated"],
                         "bytes_per_launch": strong["bytes_per_launch"]},
            "e2e": {"value": strong["e2e_value"], "unit": "GB/s", "ms_per_step": strong["e2e_ms"],
                    "h2d_bytes_per_step": n_loc * QKV_DIM * 2, "d2h_bytes_per_step": n_loc * OUT_DIM * 2,
                    "bytes_are": "per rank", "tok_per_s": N_SEQ / (strong["e2e_ms"] * 1e-3),
                    "checksum": strong["checksum"],
                    "path": "flint_attn_decode: q/k/v rows read from page-locked host memory, output rows written by "
                            "the kernel into page-locked host memory, stream synchronised, every step"},
            "gpu_launches": strong["launches"],
            "cpu_baseline": cpu_baseline,
            "clocks": strong["clocks"],
            "weak_scaling": None if weak is None else
            {"workload": "64 sequences x 8192 cached tokens on EVERY rank", "value": weak["value"], "unit": "GB/s",
             "ms_per_step": weak["ms_per_step"], "kernel_us": weak["kernel_us"],
             "tok_per_s": weak["n_seq_all"] / (weak["ms_per_step"] * 1e-3)},
            "prefill": prefill,
        }
    return line, rank, world


def run_prefill_only(args):
    """`--workload prefill`: the 4000-token prefill as the headline line (single GPU by configuration)."""
    import torch

    import flint_mac_b200 as fa

    rank, world, local = dist_setup(args.gpus)
    if rank != 0:
        return
    with ClockSampler(local) as clk:
        pf = measure_prefill(torch, fa, local, iters=args.steps, warmup=args.warmup, T=args.prefill_tokens,
                             swa=args.prefill_kind == "swa", history=args.prefill_history)
    default_cfg = args.prefill_tokens == PREFILL_T and args.prefill_kind == "swa" and not args.prefill_history
    line = {"metric": "prefill_attn_tflops", "value": pf["tflops"], "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": pf["step_us"] * 1e-3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f16 tensor-core products (tcgen05 kind::f16), f32 accumulate/softmax",
            "data": "synthetic", "config": {"workload": pf["workload"], "l2": pf["l2"]},
            "roofline": {"bound": "tensor", "achieved": pf["tflops"], "peak": pf["peak_tflops"], "unit": "TFLOP/s",
                         "frac": pf["frac"], "traffic": PREFILL_NCU_DRAM_BYTES_PER_LAUNCH if default_cfg else None,
                         "peak_kind": pf["peak_kind"],
                         "kernel": "k_prefill_attn",
                         "kernel_us": pf["attn_kernel_us"], "flops_per_launch": pf["algorithmic_flops"]},
            "e2e": {"value": pf["e2e_tflops"], "unit": "TFLOP/s", "h2d_bytes_per_step": pf["h2d_bytes_per_step"],
                    "d2h_bytes_per_step": pf["d2h_bytes_per_step"], "us_per_step": pf["e2e_us"]},
            "gpu_launches": pf["gpu_launches_per_step"] * args.steps, "tok_per_s": pf["tok_per_s"], "clocks": clk.summary()}
    print(json.dumps(line), flush=True)


def run_block(args):
    """`--workload block`: the attention block with its projections on the decode batch -- 64 sequences x 8192 cached
    tokens, hidden 4096: qkv = W_qkv . rmsnorm(x) (bf16 weights, 5120 x 4096), decode attention, x += W_o . att
    (4096 x 4096).  The projections are bound by their weight stream: the line reports each against the HBM peak."""
    import torch

    import flint_mac_b200 as fa

    rank, world, local = dist_setup(args.gpus)
    if rank != 0:
        return
    hbm_peak, _, peak_kind = measured_peaks()
    E, B = 4096, N_SEQ
    total = args.warmup + args.steps
    h = open_decode_handle(torch, fa, local, B, 1, total, 777)
    gen = torch.Generator(device="cuda").manual_seed(5)
    rng = np.random.default_rng(5)

    def bf16(shape):
        return (torch.randn(*shape, generator=gen, device="cuda") * 0.02).to(torch.bfloat16)

    wq, wk, wv, wo = bf16((4096, E)), bf16((512, E)), bf16((512, E)), bf16((E, 4096))
    h.set_projections(0, (1 + 0.1 * rng.standard_normal(E)).astype(np.float32),
                      *(w.view(torch.int16).cpu().numpy().view(np.uint16) for w in (wq, wk, wv, wo)))
    w_qkv = torch.cat([wq, wk, wv]).contiguous()
    x = torch.randn(B, E, generator=gen, device="cuda")
    nw = torch.ones(E, device="cuda")
    qkv = torch.empty(B, QKV_DIM, device="cuda")
    att = torch.randn(B, OUT_DIM, generator=gen, device="cuda")
    o = torch.empty(B, E, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    seqs = fa.i32_array(list(range(B)))

    def timed(fn, n):
        ts = []
        for i in range(args.warmup + n):
            flush.fill_(i & 0xFF)  # the weights (33-42 MB) would otherwise sit in L2
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            if i >= args.warmup:
                ts.append((e0, e1))
        torch.cuda.synchronize()
        return float(np.median([a.elapsed_time(b) for a, b in ts])) * 1e3

    n = min(args.steps, 100)
    qkv_us = timed(lambda: h.project_dev(w_qkv, QKV_DIM, E, x, B, nw, qkv, stream), n)
    o_us = timed(lambda: h.project_dev(wo, E, 4096, att, B, None, o, stream), n)
    for s in range(B):
        h.set_pos(s, CTX)

    def block():
        h.decode_block_dev(0, seqs, x, stream)

    block_us = timed(block, n)  # positions do not advance: every repetition is the same step
    h.check()
    qkv_bytes, o_bytes = QKV_DIM * E * 2, E * 4096 * 2
    act_bytes = B * (E * 4 + QKV_DIM * 4)
    line = {"metric": "attn_block_us", "value": block_us, "unit": "us", "n_gpus": 1, "steps": n, "warmup": args.warmup,
            "ms_per_step": block_us * 1e-3, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16 weights, fp32 accumulate (activations as bf16 high + low parts), f16 KV", "data": "synthetic",
            "config": {"workload": "attention block on the decode batch: 64 seqs x 8192 cached tokens, hidden 4096, "
                                   "qkv projection with fused RMSNorm + decode attention + o-projection with residual",
                       "l2": "flushed between repetitions (256 MiB write)"},
            "roofline": {"bound": "hbm", "achieved": qkv_bytes / (qkv_us * 1e-6) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                         "frac": qkv_bytes / (qkv_us * 1e-6) / 1e9 / hbm_peak, "traffic": None, "peak_kind": f"of {peak_kind}",
                         "kernel": "k_proj (qkv projection, 64 rows; the activation split kernel included)",
                         "kernel_us": qkv_us, "bytes_per_launch": qkv_bytes},
            "o_proj": {"us": o_us, "gbs": o_bytes / (o_us * 1e-6) / 1e9, "frac": o_bytes / (o_us * 1e-6) / 1e9 / hbm_peak,
                       "bytes_per_launch": o_bytes},
            "activation_bytes_per_step": act_bytes, "gpu_launches": 5 * n}
    print(json.dumps(line), flush=True)
    h.close()


def run_longctx(args):
    """`--workload longctx`: one 131072-token sequence on a full-attention layer, its key range cut contiguously over
    the ranks.  Every rank scans its range (split-K inside the GPU), the per-rank partial (O, m, l) records are
    all-gathered with NCCL and merged with the sink by flint_attn_combine_dev.  Several copies of the sequence are
    rotated through so that each step's keys come from HBM, not L2."""
    import torch

    import flint_mac_b200 as fa
    from flint_mac_b200 import dist as fdist

    rank, world, local = dist_setup(args.gpus)
    hbm_peak, _, peak_kind = measured_peaks()
    S = 131072
    total = args.warmup + args.steps
    n_ctx = S + 64
    per_gpu_bytes = KV_BYTES_PER_KEY * S // world
    copies = max(2, -(-(320 << 20) // per_gpu_bytes))
    h = fa.Attn([False], [True], copies, n_ctx, device=local, kv_rank=rank, kv_ranks=world)
    h.set_layer(0, *layer_params(0))
    n_slots = h.n_slots(0)
    gen = torch.Generator(device="cuda").manual_seed(99 + rank)
    for which in (0, 1):
        as_tensor(torch, h.kv_dev(0, which), copies * 4 * n_slots * 128, torch.float16).normal_(generator=gen)
    g2 = torch.Generator(device="cuda").manual_seed(7)  # same rows on every rank
    qkv = torch.randn(total, 1, QKV_DIM, generator=g2, device="cuda").to(torch.bfloat16)
    out = torch.empty(1, OUT_DIM, device="cuda", dtype=torch.bfloat16)
    part = torch.empty(1, 32, 130, device="cuda", dtype=torch.float32)
    stream = torch.cuda.current_stream().cuda_stream
    for c in range(copies):
        h.set_pos(c, S)
    peer = world > 1 and args.exchange == "peer"
    if peer:
        import torch.distributed as dist

        handles = [None] * world
        dist.all_gather_object(handles, h.xchg_create(1))
        h.xchg_connect(handles)
        barrier(world)

    def step_nccl(i):
        h.decode_partial_dev(0, [i % copies], qkv[i], fa.BF16, part, stream)
        gathered = fdist.gather_partials(part)
        h.combine_dev(0, 1, world, gathered, out, fa.BF16, stream)

    def step(i):
        c = i % copies
        if world == 1:
            h.decode_dev(0, [c], qkv[i], fa.BF16, out, fa.BF16, stream)
        elif peer:
            h.decode_xchg_post_dev(0, [c], qkv[i], fa.BF16, stream)
            h.combine_xchg_dev(0, 1, out, fa.BF16, stream)
        else:
            step_nccl(i)

    if peer:  # the two exchanges must agree before anything is timed
        step_nccl(0)
        want = out.float().clone()
        barrier(world)
        step(0)
        torch.cuda.synchronize()
        h.check()
        if float((out.float() - want).abs().max()) > 2e-5 + float(want.abs().max()) * 2 ** -8:  # bf16 output rows
            raise SystemExit("peer-memory exchange disagrees with the NCCL exchange")
        barrier(world)

    for i in range(args.warmup):
        step(i)
    barrier(world)
    launches0 = h.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        ev0.record()
        for i in range(args.steps):
            step(args.warmup + i)
        ev1.record()
        barrier(world)
    ms = max_over_ranks(ev0.elapsed_time(ev1), world) / args.steps
    launches = h.launch_count() - launches0
    # the decode kernel alone: the same steps once more with an event pair around every launch of it (inside the timed
    # region those events would keep the next launch from being scheduled early and cost microseconds per step)
    barrier(world)
    h.set_timing(True)
    for i in range(args.steps):
        step(args.warmup + i)
    torch.cuda.synchronize()
    kernel_ms, n_timed = h.kernel_ms()
    h.set_timing(False)
    barrier(world)
    step_bytes = decode_bytes(1, S)
    kernel_us_isolated = kernel_ms / max(n_timed, 1) * 1e3
    # one GPU: the step IS one launch of the decode kernel, so the bare region gives its steady-state duration
    kernel_us = ms * 1e3 if world == 1 else kernel_us_isolated
    h.check()
    h.close()
    if rank == 0:
        per_gpu = step_bytes / world
        line = {"metric": "decode_attn_hbm_gbs", "value": step_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f16 KV, f16 tensor-core products, f32 accumulate/softmax",
                "data": "synthetic",
                "config": {"workload": "long-context decode: 1 sequence x 131072 cached tokens, full layer, KV range "
                                       "sharded over the ranks, partial (O,m,l) records " +
                                       ("stored into every rank's memory by the decode kernel (NVLink peer stores) "
                                        "and merged by a kernel that waits on the ranks' step flags" if peer else
                                        "all-gathered (NCCL) and merged"),
                           "exchange": "peer" if peer else ("nccl" if world > 1 else "none"),
                           "kv_copies_rotated": copies, "l2": "rotating over KV copies larger than L2 in total"},
                "tok_per_s": 1.0 / (ms * 1e-3), "us_per_token": ms * 1e3,
                "roofline": {"bound": "hbm", "achieved": per_gpu / (kernel_us * 1e-6) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                             "frac": per_gpu / (kernel_us * 1e-6) / 1e9 / hbm_peak, "traffic": None,
                             "peak_kind": f"of {peak_kind}", "kernel": "k_decode_attn (this rank's key range)",
                             "kernel_us": kernel_us, "bytes_per_launch": per_gpu},
                "kernel_timed": "timed region / launches (one launch per step)" if world == 1 else
                                "same steps repeated with an event pair around every k_decode_attn launch",
                "kernel_us_isolated": kernel_us_isolated, "step_minus_kernel_us": ms * 1e3 - kernel_us, "gpu_launches": launches, "clocks": clk.summary()}
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def run_ragged(args):
    """`--workload ragged`: one decode step over a 4-layer stack (3 sliding-window ring layers + 1 full layer) for
    256 sequences whose context lengths are drawn uniformly from 1..32768 (numpy default_rng(7)); a quarter of them
    were first rolled back by 1..600 tokens (the > 511 ones re-prefill 512 tokens into the rings).  Sequences are
    placed on ranks by KV bytes (greedy LPT); no collective on the data path."""
    import torch

    import flint_mac_b200 as fa
    from flint_mac_b200 import shard

    rank, world, local = dist_setup(args.gpus)
    hbm_peak, _, peak_kind = measured_peaks()
    rng = np.random.default_rng(7)
    n_seq = 256
    ctx_all = [int(x) for x in rng.integers(1, 32769, n_seq)]
    rolled = rng.random(n_seq) < 0.25
    back_all = [int(b) if r else 0 for b, r in zip(rng.integers(1, 601, n_seq), rolled)]
    # --emulate-world N (single GPU only): run rank 0's share of an N-way placement, to look at the per-GPU step of a
    # multi-GPU run without the other GPUs
    place_world = args.emulate_world if (world == 1 and args.emulate_world > 1) else world
    owned = shard.balance_by_kv_bytes(ctx_all, place_world, n_full_layers=1, n_swa_layers=3)[rank]
    ctx = [ctx_all[i] for i in owned]
    back = [min(back_all[i], ctx_all[i]) for i in owned]
    n_loc = len(owned)
    total = args.warmup + args.steps
    n_ctx = 32768 + total + 100 + 8
    is_swa, has_rope = [True, True, True, False], [True, True, True, False]
    h = fa.Attn(is_swa, has_rope, n_loc, n_ctx, device=local)
    for il in range(4):
        h.set_layer(il, *layer_params(il))
    gen = torch.Generator(device="cuda").manual_seed(500 + rank)
    for il in range(4):
        for which in (0, 1):
            as_tensor(torch, h.kv_dev(il, which), n_loc * 4 * h.n_slots(il) * 128, torch.float16).normal_(generator=gen)
    seqs = list(range(n_loc))
    seqs_c = fa.i32_array(seqs)
    stream = torch.cuda.current_stream().cuda_stream
    # ---- rollback phase (untimed for the headline; its cost is reported on its own)
    for s in seqs:
        h.set_pos(s, ctx[s])
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n_recompute = 0
    pf_rows = torch.randn(512, QKV_DIM, generator=gen, device="cuda").to(torch.bfloat16)
    pf_out = torch.empty(512, OUT_DIM, device="cuda", dtype=torch.bfloat16)
    for s in seqs:
        if back[s] == 0:
            continue
        p = ctx[s] - back[s]
        restart = fa.rollback_restart(ctx[s], p)
        assert h.truncate(s, restart) == 0
        if restart < p:  # rolled back by more than 511: rewrite the rings from restart (server/src/main.rs:96-100)
            for il in range(3):
                h.prefill_dev(il, s, p - restart, pf_rows, fa.BF16, pf_out, fa.BF16, stream)
            h.advance([s], p - restart)
            n_recompute += 1
        ctx[s] = p
    torch.cuda.synchronize()
    rollback_ms = (time.perf_counter() - t0) * 1e3
    qkv = torch.randn(4, n_loc, QKV_DIM, generator=gen, device="cuda").to(torch.bfloat16)
    out = torch.empty(n_loc, OUT_DIM, device="cuda", dtype=torch.bfloat16)

    def step():
        for il in range(4):
            h.decode_dev(il, seqs_c, qkv[il], fa.BF16, out, fa.BF16, stream)
        h.advance(seqs_c, 1)

    def step_bytes(extra):
        b = 0
        for c in ctx:
            c = c + extra
            b += KV_BYTES_PER_KEY * (c + 3 * min(c, 512)) + 4 * (QKV_DIM * 2 + 2 * 512 * 2 + OUT_DIM * 2)
        return b

    for i in range(args.warmup):
        step()
    barrier(world)
    launches0 = h.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        ev0.record()
        for i in range(args.steps):
            step()
        ev1.record()
        barrier(world)
    ms = max_over_ranks(ev0.elapsed_time(ev1), world) / args.steps
    launches = h.launch_count() - launches0
    # the kernels alone: a second pass with an event pair around every launch (four short launches per step: the
    # events would cost the first pass several microseconds per step)
    k_steps = min(args.steps, 100)
    h.set_timing(True)
    for i in range(k_steps):
        step()
    torch.cuda.synchronize()
    kernel_ms, n_timed = h.kernel_ms()
    h.set_timing(False)
    kernel_ms = kernel_ms / k_steps * args.steps  # scaled to the step count used below
    my_bytes = sum(step_bytes(args.warmup + i) for i in range(args.steps)) / args.steps
    all_bytes = sum_over_ranks(my_bytes, world)
    max_bytes = max_over_ranks(my_bytes, world)
    h.check()
    h.close()
    if rank == 0:
        kernel_step_us = kernel_ms / args.steps * 1e3
        line = {"metric": "decode_attn_hbm_gbs", "value": all_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f16 KV, f16 tensor-core products, f32 accumulate/softmax",
                "data": "synthetic",
                "config": {"workload": "ragged serving mix: 256 sequences, context 1..32768 (numpy default_rng(7)), one decode "
                                       "step over 3 SWA ring layers + 1 full layer, 25% rolled back by 1..600 tokens first",
                           "placement": "greedy LPT by KV bytes", "l2": "inputs larger than L2",
                           **({"emulated": f"rank 0's share of a {place_world}-way placement on one GPU; value counts this "
                                           "share only"} if place_world != world else {})},
                "tok_per_s": (n_loc if place_world != world else n_seq) / (ms * 1e-3), "bytes_per_step_all_ranks": all_bytes,
                "load_imbalance": max_bytes * world / all_bytes,
                "roofline": {"bound": "hbm", "achieved": my_bytes / (kernel_step_us * 1e-6) / 1e9, "peak": hbm_peak,
                             "unit": "GB/s", "frac": my_bytes / (kernel_step_us * 1e-6) / 1e9 / hbm_peak, "traffic": None,
                             "peak_kind": f"of {peak_kind}", "kernel": "k_decode_attn (4 launches per step, rank 0)",
                             "kernel_us": kernel_step_us, "bytes_per_launch": my_bytes},
                "rollback": {"sequences_rolled_back_rank0": int(sum(1 for b in back if b)), "ring_recomputes_rank0": n_recompute,
                             "wall_ms_rank0": rollback_ms},
                "gpu_launches": launches, "clocks": clk.summary()}
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "longctx", "ragged", "block"])
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_T, help="prefill workload: prompt length")
    ap.add_argument("--prefill-history", type=int, default=0,
                    help="prefill workload: tokens already cached before the timed chunk (chunked prefill)")
    ap.add_argument("--prefill-kind", default="swa", choices=["swa", "full"],
                    help="prefill workload: sliding-window ring layer (the configuration the metric is quoted on) or full attention")
    ap.add_argument("--emulate-world", type=int, default=1,
                    help="decode / ragged workload on one GPU: run rank 0's share of an N-way placement")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="longctx on several GPUs: partial records through peer memory by the kernels, or by NCCL")
    ap.add_argument("--skip-prefill", action="store_true", help="decode workload only (profiling runs)")
    ap.add_argument("--traffic-from", default=None,
                    help="decode workload: read roofline.traffic from this `ncu --csv --page raw` file of one launch")
    ap.add_argument("--skip-cpu", action="store_true", help="shortest possible CPU baseline sample (profiling runs)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload == "prefill":
        run_prefill_only(args)
        return
    if args.workload == "longctx":
        run_longctx(args)
        return
    if args.workload == "ragged":
        run_ragged(args)
        return
    if args.workload == "block":
        run_block(args)
        return
    line, rank, world = run_decode(args)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


if __name__ == "__main__":
    main()
