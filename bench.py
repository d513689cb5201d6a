#!/usr/bin/env python3
"""Throughput of gdn_forward on synthetic data of the named shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one complete forward (prepare kernel + chunk walk) over one batch of synthetic input.
At N GPUs every rank runs the same per-GPU workload on its own (batch, head) shard, with no
data-path collective (weak scaling); the value is the tokens all ranks processed divided by
the slowest rank's device time.  One JSON line is printed by rank 0.

Timing: CUDA events on the stream the kernels are launched on, after >= 3 warm-up steps,
bracketed by a barrier and a device synchronise; the working set (inputs, outputs and the
workspace of WY factors) is several times the 126 MB L2, so no L2 flush is needed between
steps.  `e2e` measures the same forward through the host-buffer entry of the C ABI with the
host->device and device->host copies inside the timed region.  `--impl reference` times the CPU
restatement of the reference's own FP32 path (oracle/) on the host cores instead.

The same line carries, at N = 1, `per_config` (every named shape timed through the policy's configuration, with
its fraction of the per-shape roofline) and, at N > 1, the two multi-GPU forms the path has: `shard_cfg2` (B8 T4096
split by batch over the ranks, no collective, strong scaling; eager and replayed from a CUDA graph) and `sp_cfg4`
(T131072 split over the ranks, states handed on with NCCL send/recv; the exact form, eager and replayed from a CUDA
graph, and the one where the caller vouches for the decay), each with its efficiency against one GPU running the same
shape and a `parity` object (key-head group 0 of the timed tensors against the CPU restatement, computed outside
the timed regions).
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "gdn_forward tokens/s"
UNIT = "tokens/s"


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return float(data["hbm_gbs"]), float(data.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.process = index, [], None

    def start(self, wait_s=5.0):
        """Starts the sampling loop and waits for its first row, so that short timed regions are covered."""
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "10"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.process = None
            return
        deadline = time.perf_counter() + wait_s
        while not self.rows and time.perf_counter() < deadline:
            time.sleep(0.01)

    def _read(self):
        for line in self.process.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        sm, top, reasons = [], [], set()
        for row in self.rows:
            if len(row) < 7:
                continue
            try:
                sm.append(float(row[0]))
                top.append(float(row[1]))
            except ValueError:
                continue
            for name, cell in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                  row[3:7]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(top) if top else None,
                    reasons=sorted(reasons), samples=len(sm))


def cpu_reference_run(workload, steps, warmup, sample_note, repeats=1):
    """Times the CPU restatement of the reference's FP32 path on the host cores (`repeats` workloads per step)."""
    import torch
    from actlizela_b200.workloads import make_inputs
    from oracle import gdn_oracle as oracle
    # all host threads, also under torch.distributed.run (which exports OMP_NUM_THREADS=1 for multi-rank jobs)
    usable = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, usable))
    inputs = make_inputs(workload)
    # the reference's own module when oracle/make_ref.py has placed it (kind "reference"), else its restatement
    from oracle import make_ref
    module = make_ref.load_ref()
    if module is not None:
        run, kind = (lambda: make_ref.reference_forward(module, *inputs, output_final_state=True)), "reference"
    else:
        run, kind = (lambda: oracle.chunk_forward_fp32(*inputs, output_final_state=True)), "port"
    for _ in range(warmup * repeats):
        run()
    start = time.perf_counter()
    for _ in range(steps * repeats):
        run()
    elapsed = time.perf_counter() - start
    value = workload.tokens * steps * repeats / elapsed
    return dict(value=value, unit=UNIT, cores=torch.get_num_threads(), kind=kind,
                sample=sample_note, host_cpus=os.cpu_count(), ms_per_step=1e3 * elapsed / steps)


def config_dict(workload, n_gpus):
    return dict(workload=f"{workload.name} B{workload.batch} T{workload.length} Hk{workload.key_heads} "
                         f"Hv{workload.value_heads} D128 chunk64 gate={workload.gate_dtype}"
                         f"{' +initial' if workload.initial is not None else ''} per GPU",
                sharding=f"batch x{n_gpus}, no collective",
                l2="working set (inputs, outputs, WY workspace) exceeds the 126 MB L2; no flush between steps")


def reference_arm(args, workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # the native arm gives every GPU one workload per step (weak scaling); the host path gets the same N workloads
    # per step, one after the other, so that both lines count equal work
    sample = f"{args.gpus} x the full per-GPU workload each step (one per GPU of the native arm), all host threads"
    base = cpu_reference_run(workload, args.steps, args.warmup, sample, repeats=args.gpus)
    line = dict(metric=METRIC, value=base["value"], unit=UNIT, n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=base["ms_per_step"], higher_is_better=True,
                scaling="weak", vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
                config=config_dict(workload, args.gpus), kernel_configuration=f"cpu-{base['kind']}",
                cpu_baseline=dict(value=base["value"], unit=UNIT, cores=base["cores"], kind=base["kind"],
                                  sample=sample),
                e2e=dict(value=base["value"], unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def aux_bench(args):
    """Memory-bound neighbours of the forward: one JSON line with the achieved HBM fraction."""
    import torch
    from actlizela_b200 import gdn_decode_step, gdn_prepare_inputs, rmsnorm_gated
    torch.cuda.set_device(0)
    gen = torch.Generator().manual_seed(1)
    hk, hv = 16, 32
    if args.op == "decode":
        batch = 256                              # 8192 states of 64 KiB: 537 MB, read once and written once
        q = torch.randn(batch, hk, 128, generator=gen).to(torch.bfloat16).cuda()
        v = torch.randn(batch, hv, 128, generator=gen).to(torch.bfloat16).cuda()
        g = (-torch.rand(batch, hv, generator=gen)).cuda()
        beta = torch.rand(batch, hv, generator=gen).to(torch.bfloat16).cuda()
        state = torch.zeros(batch, hv, 128, 128, device="cuda")
        call = lambda: gdn_decode_step(q, q, v, g, beta, state)
        nbytes, units, unit = 2 * state.numel() * 4 + 2 * q.numel() * 2 + 2 * v.numel() * 2, batch, "tokens/s"
        name = f"decode_step B{batch} Hk{hk} Hv{hv}"
    elif args.op == "prepare_inputs":
        n = 65536
        mixed = torch.randn(n, (2 * hk + hv) * 128, generator=gen).to(torch.bfloat16).cuda()
        a = torch.randn(n, hv, generator=gen).to(torch.bfloat16).cuda()
        a_log, bias = torch.zeros(hv, device="cuda"), torch.zeros(hv, device="cuda")
        call = lambda: gdn_prepare_inputs(mixed, a, a, a_log, bias, hk, hv)
        nbytes, units, unit = 2 * mixed.numel() * 2 + n * hv * (2 + 2 + 4 + 2), n, "tokens/s"
        name = f"prepare_inputs N{n} Hk{hk} Hv{hv}"
    elif args.op == "projections":
        # the headline shape from the layer's raw projection outputs: input preparation fused into the prepare kernel
        from actlizela_b200 import gdn_forward_projections
        t = 8192
        mixed = torch.randn(1, t, (2 * hk + hv) * 128, generator=gen).to(torch.bfloat16).cuda()
        a = torch.randn(1, t, hv, generator=gen).to(torch.bfloat16).cuda()
        a_log, bias = torch.zeros(hv, device="cuda"), torch.zeros(hv, device="cuda")
        call = lambda: gdn_forward_projections(mixed, a, a, a_log, bias, hk, hv, None, True)
        nbytes = mixed.numel() * 2 + 2 * a.numel() * 2 + t * hv * 256 + hv * 65536
        units, unit = t, "tokens/s"
        name = f"forward on projections B1 T{t} Hk{hk} Hv{hv}"
    elif args.op == "out_proj":
        # the output projection behind the gated RMSNorm at the reference's production shape
        from actlizela_b200 import out_proj_gemm
        m, kk, n = 8192, 4096, 2560
        a = torch.randn(m, kk, generator=gen).to(torch.bfloat16).cuda()
        w = torch.randn(n, kk, generator=gen).to(torch.bfloat16).cuda()
        call = lambda: out_proj_gemm(a, w)
        flops = 2.0 * m * n * kk
        for _ in range(max(3, args.warmup)):
            call()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(args.steps):
            call()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / args.steps
        _, tensor_peak, source = measured_peaks()
        achieved = flops / (ms * 1e-3) / 1e12
        print(json.dumps(dict(metric="out_proj tokens/s", value=m / (ms * 1e-3), unit="tokens/s", n_gpus=1,
                              steps=args.steps, warmup=max(3, args.warmup), ms_per_step=ms, higher_is_better=True,
                              data="synthetic", dtype="bf16", gpu_launches=args.steps,
                              config=dict(workload=f"out_proj M{m} K{kk} N{n}", l2="operands exceed no cache: compute bound"),
                              roofline=dict(bound="tensor", achieved=achieved, peak=tensor_peak, unit="TFLOP/s",
                                            frac=achieved / tensor_peak, traffic=None, peak_source=source,
                                            algorithmic_flops=flops))), flush=True)
        return
    elif args.op == "varlen":
        # 64 packed prefill requests with seeded ragged lengths (mean 256 tokens); per token and value head the same
        # algorithmic bytes as the fixed-shape forward
        from actlizela_b200 import gdn_forward_varlen
        from actlizela_b200.workloads import Workload, make_inputs
        lengths = torch.randint(1, 512, (64,), generator=gen).tolist()
        bounds = [0]
        for n in lengths:
            bounds.append(bounds[-1] + n)
        w = Workload("varlen", 1, bounds[-1], hk, hv)
        q, k, v, g, beta, _ = [x.cuda() if x is not None else None for x in make_inputs(w)]
        call = lambda: gdn_forward_varlen(q, k, v, g, beta, bounds, None, True)
        nbytes = (2 * q.numel() + 2 * v.numel()) * 2 + g.numel() * 4 + beta.numel() * 2 + 64 * hv * 128 * 128 * 4
        units, unit = bounds[-1], "tokens/s"
        name = f"varlen 64 sequences {bounds[-1]} tokens Hk{hk} Hv{hv}"
    else:
        rows = 65536 * hv
        y = torch.randn(rows, 128, generator=gen).to(torch.bfloat16).cuda()
        z = torch.randn(rows, 128, generator=gen).to(torch.bfloat16).cuda()      # its own tensor: counted bytes are read
        w = torch.ones(128, dtype=torch.bfloat16, device="cuda")
        call = lambda: rmsnorm_gated(y, z, w)
        nbytes, units, unit = 3 * y.numel() * 2, rows // hv, "tokens/s"
        name = f"rmsnorm_gated rows{rows}"
    for _ in range(max(3, args.warmup)):
        call()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(args.steps):
        call()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / args.steps
    peak, _, source = measured_peaks()
    achieved = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps(dict(metric=f"{args.op} {unit}", value=units / (ms * 1e-3), unit=unit, n_gpus=1, steps=args.steps,
                          warmup=max(3, args.warmup), ms_per_step=ms, higher_is_better=True, data="synthetic",
                          config=dict(workload=name, l2="working set exceeds the 126 MB L2"),
                          gpu_launches=args.steps * (2 if args.op == "varlen" else 8 if args.op == "projections" else 1),
                          roofline=dict(bound="hbm", achieved=achieved, peak=peak, unit="GB/s", frac=achieved / peak,
                                        traffic=None, peak_source=source, algorithmic_bytes=nbytes))), flush=True)


def sequence_parallel_bench(args, workload):
    """Strong scaling of ONE long sequence over the ranks (sequence-parallel scheme): every rank owns a contiguous
    token segment; the state travels rank to rank as `M S + b` over NCCL send/recv.  N = 1 is the plain forward."""
    import torch
    import torch.distributed as dist
    from actlizela_b200 import gdn_forward
    from actlizela_b200.sequence_parallel import gdn_forward_sequence_parallel, segment_bounds
    from actlizela_b200.workloads import algorithmic_bytes, make_inputs
    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    bounds = segment_bounds(workload.length, world)
    lengths = [b1 - b0 for b0, b1 in bounds]
    t0, t1 = bounds[rank]
    # the rank's own segment, drawn from the workload's distributions with a per-rank seed (synthetic data: only
    # the first rank gets the workload's initial state)
    part = workload.sliced(length=t1 - t0, seed=workload.seed + 7919 * rank,
                           initial=workload.initial if rank == 0 else None)
    q, k, v, g, beta, initial = [x.to(device) if x is not None else None for x in make_inputs(part)]

    def step():
        if world == 1:
            return gdn_forward(q, k, v, g, beta, initial, True)
        return gdn_forward_sequence_parallel(q, k, v, g, beta, initial, True, until_decayed=args.until_decayed,
                                             segment_lengths=lengths)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(max(3, args.warmup)):
        step()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    sync_all()
    elapsed = torch.tensor([start.elapsed_time(stop)], device=device)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms = elapsed.item() / args.steps
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        peak, _, source = measured_peaks()
        nbytes = algorithmic_bytes(workload)
        achieved = nbytes / (ms * 1e-3) / 1e9
        print(json.dumps(dict(
            metric=METRIC, value=workload.tokens / (ms * 1e-3), unit=UNIT, n_gpus=world, steps=args.steps,
            warmup=max(3, args.warmup), ms_per_step=ms, higher_is_better=True, scaling="strong", vs_baseline=None,
            dtype="bf16", dtype_detail="bf16 operands (state path as bf16 hi+lo pairs), f32 accumulate and state",
            data="synthetic",
            config=dict(workload=f"{workload.name} B{workload.batch} T{workload.length} Hk{workload.key_heads} "
                                 f"Hv{workload.value_heads}", parallelism=f"sp{world}",
                        until_decayed=bool(args.until_decayed), l2="inputs exceed the 126 MB L2"),
            roofline=dict(bound="hbm", achieved=achieved, peak=peak * world, unit="GB/s", frac=achieved / (peak * world),
                          traffic=None, peak_source=source, algorithmic_bytes=nbytes),
            e2e=None, clocks=clocks, gpu_launches=None)), flush=True)
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------- helpers of the extra legs
OUT_MAX_ABS, OUT_REL_F, STATE_REL_F = 2e-2, 1e-2, 1e-3       # the stated tolerances of the path


def device_inputs(w, device, seed):
    """Timing-only inputs with the workload's shapes and distributions, drawn on the device (the CPU generator of
    workloads.make_inputs is kept for everything that is compared with the CPU restatement)."""
    import torch
    import torch.nn.functional as F
    gen = torch.Generator(device=device).manual_seed(seed)
    b, t, hk, hv = w.shape
    normal = lambda *shape: torch.randn(*shape, generator=gen, device=device)
    q = F.normalize(normal(b, t, hk, 128), dim=-1).to(torch.bfloat16)
    k = F.normalize(normal(b, t, hk, 128), dim=-1).to(torch.bfloat16)
    v = normal(b, t, hv, 128).to(torch.bfloat16)
    g = (F.logsigmoid(normal(b, t, hv) + 2.0) if w.gate == "logsigmoid"
         else -0.01 * torch.rand(b, t, hv, generator=gen, device=device))
    g = g.to(torch.bfloat16 if w.gate_dtype == "bf16" else torch.float32)
    beta = torch.sigmoid(normal(b, t, hv) + w.beta_shift).to(torch.bfloat16)
    initial = None
    if w.initial is not None:
        initial = torch.zeros(b, hv, 128, 128, device=device) if w.initial == 0.0 else w.initial * normal(b, hv, 128, 128)
    return [q, k, v, g, beta, initial]


def plant_group(tensors, narrow, t0=0, t1=None):
    """Overwrite key head 0 and its value heads in the device tensors with the CPU-generated `narrow` inputs
    (token rows [t0, t1) of them): heads are independent, so that head group of the timed run can be checked
    against the CPU restatement of the narrow workload."""
    ratio = narrow[2].shape[2] // narrow[0].shape[2]
    hk = narrow[0].shape[2]
    for i, heads in ((0, hk), (1, hk), (2, hk * ratio), (3, hk * ratio), (4, hk * ratio)):
        tensors[i][:, :, :heads] = narrow[i][:, t0:t1].to(tensors[i].device)
    if tensors[5] is not None and narrow[5] is not None:
        tensors[5][:, :hk * ratio] = narrow[5].to(tensors[5].device)


def parity_metrics(out, want_out, state=None, want_state=None):
    """Worst-case figures of one comparison with the CPU restatement, as plain floats."""
    out, want_out = out.float().cpu(), want_out.float()
    m = dict(out_max_abs=float((out - want_out).abs().max()),
             out_rel_f=float((out - want_out).norm() / want_out.norm().clamp_min(1e-30)), state_rel_f=0.0)
    if state is not None:
        m["state_rel_f"] = float((state.cpu() - want_state).norm() / want_state.norm().clamp_min(1e-30))
    return m


def reduce_parity(m, device, world):
    import torch
    import torch.distributed as dist
    x = torch.tensor([m["out_max_abs"], m["out_rel_f"], m["state_rel_f"]], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(x, op=dist.ReduceOp.MAX)
    a, r, st = (float(v) for v in x.tolist())
    return dict(out_max_abs=a, out_rel_f=r, state_rel_f=st, ok=bool(a <= OUT_MAX_ABS and r <= OUT_REL_F and st <= STATE_REL_F),
                against="oracle.chunk_forward_fp32 on key-head group 0 of the timed tensors, max over ranks")


def timed_loop(fn, steps, device, world, stream=None):
    """K steps between two events on the launching stream, barrier + synchronise either side; per-step events give
    the spread.  Returns (ms per step as total / K, max over ranks; dict of median / min / max over the K steps of
    this rank's own event pairs)."""
    import torch
    import torch.distributed as dist
    stream = stream or torch.cuda.current_stream()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    marks[0].record(stream)
    for i in range(steps):
        fn()
        marks[i + 1].record(stream)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    total = torch.tensor([marks[0].elapsed_time(marks[-1])], device=device)
    if world > 1:
        dist.all_reduce(total, op=dist.ReduceOp.MAX)
    each = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
    return total.item() / steps, dict(median_ms=statistics.median(each), min_ms=each[0], max_ms=each[-1], samples=steps)


def roofline_ms(w, peaks):
    from actlizela_b200.workloads import algorithmic_bytes, algorithmic_flops
    hbm_peak, tensor_peak, _ = peaks
    return max(algorithmic_bytes(w) / (hbm_peak * 1e9), algorithmic_flops(w) / (tensor_peak * 1e12)) * 1e3


def per_config_legs(device, skip, peaks, steps=11):
    """Every named shape on one GPU through the policy's configuration: ms, tokens/s and the fraction of the
    per-shape roofline (the slower of bytes / measured HBM bandwidth and FLOPs / measured BF16 peak)."""
    import torch
    from actlizela_b200 import gdn_forward
    from actlizela_b200.sm100_policy import selection_for
    from actlizela_b200.workloads import WORKLOADS
    legs = {}
    for name, w in WORKLOADS.items():
        if name == skip:
            continue
        tensors = device_inputs(w, device, w.seed)
        sel = selection_for(tensors[0], tensors[2])
        call = lambda: gdn_forward(*tensors, output_final_state=True)
        timed_loop(call, max(3, steps), device, 1)      # warm-up in the shape of the measurement (allocator steady state)
        ms, spread = timed_loop(call, steps, device, 1)
        legs[name] = dict(ms=ms, median_ms=spread["median_ms"], tokens_per_s=w.tokens / (ms * 1e-3),
                          roofline_ms=roofline_ms(w, peaks), frac=roofline_ms(w, peaks) / ms,
                          configuration=f"{sel.configuration} segments={sel.segments} parallel={sel.parallel}")
        del tensors
        torch.cuda.empty_cache()
    return legs


def shard_cfg2_leg(device, rank, world, steps, peaks):
    """cfg2 (B8 T4096 Hk16 Hv32, BF16 gate) split by batch over the ranks, no collective: strong scaling against
    one GPU running all eight batch rows."""
    import torch
    from actlizela_b200 import gdn_forward
    from actlizela_b200.sharding import gdn_forward_sharded
    from actlizela_b200.workloads import WORKLOADS, make_inputs
    from oracle import gdn_oracle as oracle
    w = WORKLOADS["cfg2"]
    tensors = device_inputs(w, device, w.seed)                       # the same tensors on every rank
    narrow = make_inputs(w.sliced(key_heads=1, value_heads=w.value_heads // w.key_heads))
    plant_group(tensors, narrow)
    whole = lambda: gdn_forward(*tensors, output_final_state=True)
    mine = lambda: gdn_forward_sharded(*tensors, True, rank=rank, world_size=world)
    for fn in (whole, mine):          # warm-up in the shape of the measurement (allocator steady state)
        timed_loop(fn, max(3, steps), device, world)
    ms_one, _ = timed_loop(whole, steps, device, world)
    ms_n, spread = timed_loop(mine, steps, device, world)
    # the same call replayed from a CUDA graph: at many ranks a call is short enough for the host's launch path and
    # its jitter to show in the eager figure
    ms_graph = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            mine()
        timed_loop(graph.replay, max(3, steps), device, world)
        ms_graph, _ = timed_loop(graph.replay, steps, device, world)
        del graph
    except RuntimeError:                 # reported as missing, not fatal: the eager figure stands on its own
        pass
    worst = dict(out_max_abs=0.0, out_rel_f=0.0, state_rel_f=0.0)
    heads = narrow[2].shape[2]
    for (b0, b1, v0, v1), out, final in mine():
        if v0 != 0:
            continue
        want_out, want_state = oracle.chunk_forward_fp32(*[x[b0:b1] for x in narrow[:5]], narrow[5][b0:b1], True)
        m = parity_metrics(out[:, :, :heads], want_out, final[:, :heads], want_state)
        worst = {k: max(worst[k], m[k]) for k in worst}
    return dict(workload="cfg2 B8 T4096 Hk16 Hv32 bf16 gate, zero initial state", sharding=f"batch rows over {world} ranks",
                ms=ms_n, median_ms=spread["median_ms"], tokens_per_s=w.tokens / (ms_n * 1e-3), one_gpu_ms=ms_one,
                efficiency=ms_one / (world * ms_n), roofline_frac=roofline_ms(w, peaks) / (world * ms_n),
                graph_replay_ms=ms_graph, graph_replay_efficiency=(ms_one / (world * ms_graph)) if ms_graph else None,
                scaling="strong", parity=reduce_parity(worst, device, world))


def sp_cfg4_leg(device, rank, world, steps, peaks):
    """cfg4 (B1 T131072 Hk16 Hv32) split over the ranks as contiguous token segments, states handed on with NCCL
    send/recv: strong scaling against one GPU running the whole sequence; the exact form and the vouched one."""
    import torch
    from actlizela_b200 import gdn_forward
    from actlizela_b200.sequence_parallel import (capture_sequence_parallel, gdn_forward_sequence_parallel,
                                                   segment_bounds)
    from actlizela_b200.workloads import WORKLOADS, make_inputs
    from oracle import gdn_oracle as oracle
    w = WORKLOADS["cfg4"]
    bounds = segment_bounds(w.length, world)
    lengths = [b1 - b0 for b0, b1 in bounds]
    t0, t1 = bounds[rank]
    narrow = make_inputs(w.sliced(key_heads=1, value_heads=w.value_heads // w.key_heads))
    heads = narrow[2].shape[2]
    full = device_inputs(w, device, w.seed)
    plant_group(full, narrow)
    whole = lambda: gdn_forward(*full, output_final_state=True)
    timed_loop(whole, max(3, steps), device, world)
    ms_one, _ = timed_loop(whole, steps, device, world)
    part = [x[:, t0:t1].contiguous() for x in full[:5]]
    initial = full[5] if rank == 0 else None
    del full
    torch.cuda.empty_cache()
    want_out, want_state = oracle.chunk_forward_fp32(*narrow, output_final_state=True)
    result = dict(workload="cfg4 B1 T131072 Hk16 Hv32 fp32 gate, zero initial state",
                  segments=f"{world} contiguous token segments, one per rank", one_gpu_ms=ms_one, scaling="strong",
                  forms="exact: eager call; exact_graph: the same call captured once in a CUDA graph and replayed (no "
                        "host work per call; the eager form is host-bound when the segments are short); vouched: the "
                        "caller states that every segment forgets its incoming state")
    # "exact": decided on the device per (batch, value head), valid for any gate; "vouched": the caller states that
    # every segment forgets its incoming state, so no transition pass runs and only b travels to the next rank
    # "exact_graph": the exact form captured once in a CUDA graph and replayed (no host work per call beyond the replay)
    for form, decayed, captured in (("exact", False, False), ("exact_graph", False, True), ("vouched", True, False)):
        call = lambda: gdn_forward_sequence_parallel(*part, initial, True, until_decayed=decayed,
                                                     segment_lengths=lengths)
        if captured:
            try:
                graph, out, final = capture_sequence_parallel(*part, initial, True, until_decayed=decayed,
                                                              segment_lengths=lengths)
            except RuntimeError as err:              # reported, not fatal: the eager forms stand on their own
                result[form] = dict(error=str(err).splitlines()[0][:200])
                continue
            call = graph.replay
        # warm-up in the shape of the measurement: the host runs several calls ahead of the device, each holding a
        # workspace of its own, so the caching allocator reaches its steady state only in such a loop
        timed_loop(call, max(3, steps), device, world)
        ms, spread = timed_loop(call, steps, device, world)
        if captured:
            call()
            torch.cuda.synchronize()
        else:
            out, final = call()
        m = parity_metrics(out[:, :, :heads], want_out[:, t0:t1],
                           final[:, :heads] if final is not None else None, want_state)
        result[form] = dict(ms=ms, median_ms=spread["median_ms"], tokens_per_s=w.tokens / (ms * 1e-3),
                            efficiency=ms_one / (world * ms), roofline_frac=roofline_ms(w, peaks) / (world * ms),
                            parity=reduce_parity(m, device, world))
        if captured:
            del graph
    return result


def copy_bound_ms(host, host_out, host_final, device, world, reps=5):
    """The time the step's host->device and device->host bytes take as plain concurrent cudaMemcpyAsync calls, all
    ranks at once (the floor of `e2e` on this box)."""
    import torch
    landing = [torch.empty_like(x, device=device) for x in host if x is not None]
    src_out, src_final = torch.empty_like(host_out, device=device), torch.empty_like(host_final, device=device)
    up, down = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)

    def step():
        up.wait_stream(torch.cuda.current_stream())
        down.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(up):
            for dst, src in zip(landing, [x for x in host if x is not None]):
                dst.copy_(src, non_blocking=True)
        with torch.cuda.stream(down):
            host_out.copy_(src_out, non_blocking=True)
            host_final.copy_(src_final, non_blocking=True)
        torch.cuda.current_stream().wait_stream(up)
        torch.cuda.current_stream().wait_stream(down)

    step()
    ms, _ = timed_loop(step, reps, device, world)
    return ms


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="headline")
    ap.add_argument("--configuration", default=None, help="diagnostic override of the policy table")
    ap.add_argument("--impl", default="native", choices=("native", "reference"))
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-extra-legs", action="store_true",
                    help="leave out per_config (N = 1) and shard_cfg2 / sp_cfg4 (N > 1)")
    ap.add_argument("--op", default="forward", choices=("forward", "decode", "prepare_inputs", "rmsnorm_gated", "varlen", "projections", "out_proj"),
                    help="forward is the headline metric; the others time a neighbouring memory-bound kernel")
    ap.add_argument("--parallelism", default="shard", choices=("shard", "sp"),
                    help="shard: every rank one per-GPU workload (weak scaling, the headline form); sp: one sequence "
                         "split over the ranks (strong scaling, e.g. --workload cfg4)")
    ap.add_argument("--until-decayed", action="store_true",
                    help="sp only: final pass over the leading chunks the incoming state still reaches")
    args = ap.parse_args()
    if args.op != "forward":
        return aux_bench(args)
    if args.parallelism == "sp":
        from actlizela_b200.workloads import WORKLOADS
        return sequence_parallel_bench(args, WORKLOADS[args.workload])

    from actlizela_b200.workloads import WORKLOADS, algorithmic_bytes, algorithmic_flops, make_inputs
    workload = WORKLOADS[args.workload]
    if args.impl == "reference":
        return reference_arm(args, workload)

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    args.warmup = max(args.warmup, 3)

    from actlizela_b200 import _library
    from actlizela_b200.sm100 import configuration_id
    from actlizela_b200.sm100_policy import selection_for
    library = _library.load_library()
    library.configure(device)
    lib = library.lib

    # every rank owns one per-GPU workload (its batch shard), generated from its own seed
    shard = workload.sliced(seed=workload.seed + 7919 * rank)
    host = make_inputs(shard, pin=True)
    q, k, v, g, beta, initial = [x.to(device) if x is not None else None for x in host]
    b, t, hk, hv = shard.shape
    gate_fp32 = int(g.dtype == torch.float32)
    if args.configuration is None:
        selection = selection_for(q, v)
        config, config_name = selection.configuration_id, selection.configuration
    else:
        config, config_name = configuration_id(args.configuration), args.configuration
    out = torch.empty_like(v)
    final = torch.empty(b, hv, 128, 128, device=device)
    ws_bytes = lib.actlize_la_sm100_workspace_bytes(b, t, hk, hv, config)
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
    stream = torch.cuda.current_stream()

    def forward(stage=0):
        rc = lib.actlize_la_sm100_forward_prepared(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
            initial.data_ptr() if initial is not None else None, out.data_ptr(), final.data_ptr(),
            workspace.data_ptr(), ws_bytes, b, t, hk, hv, gate_fp32, config | stage, stream.cuda_stream)
        if rc:
            raise RuntimeError(f"forward_prepared failed with CUDA error {rc}")

    def timed(fn, steps):
        return timed_loop(fn, steps, device, world, stream)     # (ms per step, max over ranks; spread of the steps)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        forward()
    ms_step, spread = timed(forward, args.steps)
    ms_walk, _ = timed(lambda: forward(0x20), args.steps)
    ms_prepare, _ = timed(lambda: forward(0x10), args.steps)
    forward()

    # end to end through the host-buffer entry: pinned host tensors in, output + state back
    arena_bytes = lib.actlize_la_sm100_host_arena_bytes(b, t, hk, hv, gate_fp32, int(initial is not None), 1, config)
    del workspace
    arena = torch.empty(arena_bytes, dtype=torch.uint8, device=device)
    host_out = torch.empty(v.shape, dtype=torch.bfloat16).pin_memory()
    host_final = torch.empty(b, hv, 128, 128).pin_memory()

    def forward_host():
        rc = lib.actlize_la_sm100_forward_host(
            host[0].data_ptr(), host[1].data_ptr(), host[2].data_ptr(), host[3].data_ptr(), host[4].data_ptr(),
            host[5].data_ptr() if host[5] is not None else None, host_out.data_ptr(), host_final.data_ptr(),
            arena.data_ptr(), arena_bytes, b, t, hk, hv, gate_fp32, config, stream.cuda_stream)
        if rc:
            raise RuntimeError(f"forward_host failed with CUDA error {rc}")

    e2e_steps = max(3, min(args.steps, 10))
    forward_host()
    ms_e2e, _ = timed(forward_host, e2e_steps)
    same = bool(torch.equal(host_out, out.cpu()))
    h2d = sum(x.numel() * x.element_size() for x in host if x is not None)
    d2h = host_out.numel() * 2 + host_final.numel() * 4
    clocks = sampler.stop() if rank == 0 else None       # sampled over the device-timed loops and the end-to-end loop
    ms_copies = copy_bound_ms(host, host_out, host_final, device, world)
    del arena

    status = (ctypes.c_int * 4)()
    lib.actlize_la_sm100_device_status(status, 0)
    peaks = measured_peaks()
    hbm_peak, tensor_peak, peak_source = peaks
    extra = {}
    if not args.skip_extra_legs:
        del q, k, v, g, beta, initial, out, final
        torch.cuda.empty_cache()
        extra_steps = max(3, min(args.steps, 10))
        if world == 1:
            extra["per_config"] = per_config_legs(device, workload.name, peaks)
        else:
            extra["shard_cfg2"] = shard_cfg2_leg(device, rank, world, extra_steps, peaks)
            extra["sp_cfg4"] = sp_cfg4_leg(device, rank, world, extra_steps, peaks)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    alg_bytes, alg_flops = algorithmic_bytes(shard), algorithmic_flops(shard)
    # the roofline object describes the longer of the two kernels of a forward; both see the whole problem, so the
    # algorithmic bytes of the path (each tensor once) are set against that kernel's own time
    top, ms_top = ("prepare", ms_prepare) if ms_prepare > ms_walk else ("walk", ms_walk)
    achieved = alg_bytes / (ms_top * 1e-3) / 1e9
    # DRAM traffic per launch from the committed ncu captures of a smaller case (profiles/; caches flushed before the
    # captured launch, so an upper bound), per (chunk, value head) block and scaled by the blocks of one launch
    blocks = shard.batch * shard.value_heads * ((shard.length + 63) // 64)
    traffic = {"walk": 108.3e3, "prepare": 52.3e3}[top] * blocks if config_name == "umma" else None
    whole_ms = max(alg_bytes / (hbm_peak * 1e9), alg_flops / (tensor_peak * 1e12)) * 1e3
    line = dict(
        metric=METRIC, value=workload.tokens * world / (ms_step * 1e-3), unit=UNIT, n_gpus=world,
        steps=args.steps, warmup=args.warmup, ms_per_step=ms_step, higher_is_better=True, scaling="weak",
        vs_baseline=None, dtype="bf16", dtype_detail="bf16 operands (state path as bf16 hi+lo pairs), f32 accumulate and state",
        data="synthetic", config=config_dict(workload, world),
        kernel_configuration=dict(family=config_name, segments=(config >> 8) & 0xff, parallel=max(1, (config >> 16) & 0xf)),
        gpu_launches=args.steps * lib.actlize_la_sm100_launches_per_forward(config),
        kernels_ms=dict(prepare=ms_prepare, walk=ms_walk, forward=ms_step),
        step_spread=spread,
        roofline=dict(bound="hbm", kernel=top, achieved=achieved, peak=hbm_peak, unit="GB/s",
                      frac=achieved / hbm_peak, traffic=traffic,
                      traffic_note=("dram bytes read + written of one launch in the ncu capture of cfg0 (caches flushed "
                                    "before the launch; workspace lines still dirty in L2 at its end are not in it), "
                                    "per block, scaled by the blocks of this launch" if traffic else None),
                      peak_source=peak_source, algorithmic_bytes=alg_bytes, algorithmic_flops=alg_flops,
                      whole_forward_frac=whole_ms / ms_step,
                      tensor_frac=alg_flops / (ms_step * 1e-3) / (tensor_peak * 1e12)),
        e2e=dict(value=workload.tokens * world / (ms_e2e * 1e-3), unit=UNIT, h2d_bytes_per_step=h2d,
                 d2h_bytes_per_step=d2h, ms_per_step=ms_e2e, output_equals_device_path=same,
                 copy_bound_ms=ms_copies, over_copy_bound=ms_e2e / ms_copies),
        clocks=clocks, device_status=list(status), **extra)
    if not args.skip_cpu_baseline:
        reps = 10
        line["cpu_baseline"] = {k2: v2 for k2, v2 in cpu_reference_run(
            workload, reps, 1, f"{reps} repetitions of the full {workload.name} workload").items()
            if k2 in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
