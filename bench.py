#!/usr/bin/env python
"""Benchmark of the catena hot path on B200: deterministic bf16 GEMM TFLOP/s (headline `value`) and
cached-attention decode HBM GB/s (`attn_decode`), one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workloads (synthetic, seeded; shapes from the benchmark spec):
  gemm   bf16 4096^3, A row-major, B column-major, entries N(0,1)/sqrt(K), fp32 accumulate, bf16 out
  attn   decode B=32, Hq=32, Hkv=8, D=128, KV length 4096, bf16, N(0,1)
A step = one GEMM launch (resp. one attention launch) on one operand set.  Operand sets rotate so
consecutive steps never find their inputs in the 126 MB L2.
N > 1 (torchrun, one rank per GPU): every rank runs the same per-GPU workload on its own operands
(weak scaling, no data-path collective); timing is on-device, max over ranks.
`--impl reference` times the CPU oracle (a restatement of the reference's generated code; the
reference itself is Rust + nvcc-at-run-time and cannot be built on this box) on a bounded sample.
"""
import argparse
import ctypes as C
import json
import math
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GEMM_M = GEMM_N = GEMM_K = 4096
ATT = dict(B=32, Hq=32, Hkv=8, D=128, L=4096)
TIMED_SECONDS = 0.5        # minimum length of the headline's timed region
WORKLOAD = "bf16 GEMM 4096^3 (A row-major, B column-major, fp32 accumulate, bf16 out), fixed K order"
GEMM_FLOP = 2.0 * GEMM_M * GEMM_N * GEMM_K
ATT_BYTES = 2 * ATT["B"] * ATT["Hkv"] * ATT["L"] * ATT["D"] * 2 + 2 * ATT["B"] * ATT["Hq"] * ATT["D"] * 2


# DRAM traffic per launch from the ncu captures summarised under profiles/ (bytes): the GEMM capture is the bench launch
# itself; the attention capture is the same kernel on a quarter of the batch (B=8), scaled by 4 (traffic grows with the batch)
GEMM_NCU_TRAFFIC_BYTES = 85719808 + 15269120
ATTN_NCU_TRAFFIC_BYTES = 4 * (134397696 + 4114176)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def gemm_operands(seed):
    rng = np.random.default_rng(seed)
    a = bf16_bits((rng.standard_normal((GEMM_M, GEMM_K), dtype=np.float32) / math.sqrt(GEMM_K)))
    bt = bf16_bits((rng.standard_normal((GEMM_N, GEMM_K), dtype=np.float32) / math.sqrt(GEMM_K)))
    return a, bt


# ------------------------------------------------------------------------------------ reference arm
def run_reference(args, rank):
    """CPU arm: the oracle port of the reference's generated code on all host threads, on a bounded
    sample of the same workload (a slab of output rows of the 4096^3 bf16 GEMM)."""
    if rank != 0:
        return
    import oracle
    oracle.build()
    threads = oracle.max_threads()
    a, bt = gemm_operands(1)
    rows = 256
    def step():
        t0 = time.perf_counter()
        oracle.gemm_bf16_rows(a, bt, GEMM_N, GEMM_K, 0, rows, threads=threads)
        return time.perf_counter() - t0
    for _ in range(max(1, min(args.warmup, 2))):
        step()
    steps = max(1, min(args.steps, 8))
    t = [step() for _ in range(steps)]
    sec = float(np.mean(t))
    value = 2.0 * rows * GEMM_N * GEMM_K / sec / 1e12
    sample = f"{rows} of {GEMM_M} output rows of the 4096^3 bf16 GEMM per step, {steps} steps"
    line = {
        "impl": "reference", "metric": "bf16_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "step": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------ GPU arm
def run_gpu(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import catena_lang_b200 as cb
    from catena_lang_b200 import shard

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = cb.lib()
    cb.check(L.catena_b200_init(local_rank))
    stream = torch.cuda.Stream(device=dev)
    L.catena_b200_set_stream(C.c_void_p(stream.cuda_stream))
    L.catena_b200_set_blocking(0)
    peaks = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- operands resident in HBM; 4 GEMM sets = 384 MB and 2 KV sets = 1 GB, both larger than L2
    n_sets = 4
    sets = []
    for s in range(n_sets):
        a, bt = gemm_operands(1 + 1000 * rank + s)
        sets.append((torch.from_numpy(a.view(np.int16)).to(dev), torch.from_numpy(bt.view(np.int16)).to(dev),
                     torch.empty((GEMM_M, GEMM_N), dtype=torch.int16, device=dev)))
    g = torch.Generator(device=dev)
    g.manual_seed(2 + rank)
    kv_sets = []
    for s in range(2):
        q = torch.randn((ATT["B"], ATT["Hq"], ATT["D"]), generator=g, device=dev).to(torch.bfloat16)
        k = torch.randn((ATT["B"], ATT["Hkv"], ATT["L"], ATT["D"]), generator=g, device=dev).to(torch.bfloat16)
        v = torch.randn((ATT["B"], ATT["Hkv"], ATT["L"], ATT["D"]), generator=g, device=dev).to(torch.bfloat16)
        o = torch.empty((ATT["B"], ATT["Hq"], ATT["D"]), dtype=torch.bfloat16, device=dev)
        kv_sets.append((q, k, v, o))
    torch.cuda.synchronize(dev)

    def gemm_step(i):
        a, bt, c = sets[i % n_sets]
        cb.check(L.catena_b200_gemm_bf16_into(a.data_ptr(), bt.data_ptr(), c.data_ptr(), GEMM_M, GEMM_N, GEMM_K, GEMM_N))

    def attn_step(i):
        q, k, v, o = kv_sets[i % 2]
        cb.check(L.catena_b200_attn_decode_bf16_into(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), ATT["B"],
                                                     ATT["Hq"], ATT["Hkv"], ATT["D"], ATT["L"], 0, ATT["B"] * ATT["Hkv"]))

    def timed(step_fn, steps, warmup):
        with torch.cuda.stream(stream):
            for i in range(warmup):
                step_fn(i)
            barrier()
            launches0 = L.catena_b200_launch_count()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with ClockSampler(local_rank) as clk:
                e0.record(stream)
                for i in range(steps):
                    step_fn(i)
                e1.record(stream)
                barrier()
            ms = e0.elapsed_time(e1)
            launches = L.catena_b200_launch_count() - launches0
        cb.check(L.catena_b200_check_device_errors())
        ms = shard.max_over_ranks(ms, dist if world > 1 else None, dev)
        return ms, launches, clk.summary()

    warmup = max(3, args.warmup)
    # A step is a batch of `per_step` launches, sized so that the K timed steps last at least TIMED_SECONDS whatever K
    # is: a region of a few milliseconds says nothing about clocks under load (one NVML sample) and flatters the kernel.
    burst_ms, _, _ = timed(gemm_step, 20, warmup)                  # the first 20 launches from idle, timed alone
    gemm_per_step = args.launches_per_step or max(1, math.ceil(TIMED_SECONDS * 1e3 / (args.steps * burst_ms / 20)))
    attn_probe_ms, _, _ = timed(attn_step, 20, warmup)
    attn_per_step = args.launches_per_step or max(1, math.ceil(TIMED_SECONDS * 1e3 / (args.steps * attn_probe_ms / 20)))

    def gemm_batch(i):
        for j in range(gemm_per_step):
            gemm_step(i * gemm_per_step + j)

    def attn_batch(i):
        for j in range(attn_per_step):
            attn_step(i * attn_per_step + j)

    gemm_ms, gemm_launches, clocks = timed(gemm_batch, args.steps, 1)
    attn_ms, attn_launches, attn_clocks = timed(attn_batch, args.steps, 1)
    gemm_per = gemm_ms / (args.steps * gemm_per_step)              # per launch
    attn_per = attn_ms / (args.steps * attn_per_step)
    gemm_tflops_1 = GEMM_FLOP / (gemm_per * 1e-3) / 1e12           # per GPU
    attn_gbs_1 = ATT_BYTES / (attn_per * 1e-3) / 1e9
    burst_tflops_1 = GEMM_FLOP / (burst_ms / 20 * 1e-3) / 1e12
    sustained_peak = peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]

    # ---- end to end through the reference-shaped API: host buffers in, host buffer out, every step
    rt = cb.Runtime.from_sources(["(def program gemm-bf16-rc : x -> y = ())"], cb.GpuDialect.Cuda)
    a_np, bt_np = gemm_operands(1 + 1000 * rank)
    a_pin = torch.from_numpy(a_np.view(np.int16)).pin_memory()
    b_pin = torch.from_numpy(bt_np.view(np.int16)).pin_memory()
    c_pin = torch.empty((GEMM_M * GEMM_N,), dtype=torch.int16).pin_memory()
    a_host, b_host, c_host = a_pin.numpy(), b_pin.numpy(), c_pin.numpy().view(np.uint16)
    L.catena_b200_set_blocking(1)

    def e2e_step():
        [r] = rt.exec("gemm-bf16-rc", [rt.mem_bytes(a_host), rt.mem_bytes(b_host), GEMM_M, GEMM_N, GEMM_K])
        r.v.to_array(np.uint16, out=c_host)
        r.v.free()

    e2e_steps = max(1, min(args.steps, 20))
    for _ in range(3):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        e1.record(stream)
        barrier()
    e2e_ms = shard.max_over_ranks(e0.elapsed_time(e1), dist if world > 1 else None, dev) / e2e_steps
    e2e_tflops = world * GEMM_FLOP / (e2e_ms * 1e-3) / 1e12
    checksum = int(np.bitwise_xor.reduce(c_host.astype(np.uint64) * (np.arange(c_host.size, dtype=np.uint64) | 1)))

    # ---- the same end-to-end work as a pipeline over the launch-level C ABI: the H2D copy of step i+1 and the D2H copy of
    # step i-1 run on their own streams while step i computes (PCIe is full duplex); still every step's operands come from
    # pinned host memory and every step's result goes back to it inside the timed region
    L.catena_b200_set_blocking(0)
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    a_d = [torch.empty((GEMM_M, GEMM_K), dtype=torch.int16, device=dev) for _ in range(2)]
    b_d = [torch.empty((GEMM_N, GEMM_K), dtype=torch.int16, device=dev) for _ in range(2)]
    c_d = [torch.empty((GEMM_M * GEMM_N,), dtype=torch.int16, device=dev) for _ in range(2)]
    c_pins = [c_pin, torch.empty((GEMM_M * GEMM_N,), dtype=torch.int16).pin_memory()]
    a_src, b_src = a_pin.view(GEMM_M, GEMM_K), b_pin.view(GEMM_N, GEMM_K)

    def pipeline(steps):
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(s_in)
        for i in range(steps):
            j = i % 2
            if i >= 2:
                s_in.wait_event(ev_done[j])                    # the GEMM that read these operand buffers is done
            with torch.cuda.stream(s_in):
                a_d[j].copy_(a_src, non_blocking=True)
                b_d[j].copy_(b_src, non_blocking=True)
                ev_in[j].record(s_in)
            stream.wait_event(ev_in[j])
            if i >= 2:
                stream.wait_event(ev_out[j])                   # the result buffer has been copied out
            cb.check(L.catena_b200_gemm_bf16_into(a_d[j].data_ptr(), b_d[j].data_ptr(), c_d[j].data_ptr(), GEMM_M, GEMM_N, GEMM_K, GEMM_N))
            ev_done[j].record(stream)
            s_out.wait_event(ev_done[j])
            with torch.cuda.stream(s_out):
                c_pins[j].copy_(c_d[j], non_blocking=True)
                ev_out[j].record(s_out)
        s_out.wait_stream(stream)
        t1.record(s_out)
        torch.cuda.synchronize(dev)
        return t0.elapsed_time(t1)

    pipe_steps = max(4, min(args.steps, 40))
    pipeline(4)
    barrier()
    pipe_ms = shard.max_over_ranks(pipeline(pipe_steps), dist if world > 1 else None, dev) / pipe_steps
    barrier()
    pipe_tflops = world * GEMM_FLOP / (pipe_ms * 1e-3) / 1e12
    last = c_pins[(pipe_steps - 1) % 2].numpy().view(np.uint16)
    pipe_checksum = int(np.bitwise_xor.reduce(last.astype(np.uint64) * (np.arange(last.size, dtype=np.uint64) | 1)))
    assert pipe_checksum == checksum, "the pipelined end-to-end result differs from Runtime.exec's"
    del a_d, b_d, c_d
    cb.check(L.catena_b200_check_device_errors())

    # ---- the other kernels of the path, each against its own roofline (rank 0's GPU)
    kernels = kernel_suite(cb, L, torch, dev, stream, peaks, clocks.get("sm_max_mhz") or 1965)
    L.catena_b200_set_blocking(1)
    barrier()

    # ---- Llama-style block (prefill 4 x 2048, then 128 decode steps), one replica per GPU; rank 0's figures are reported
    L.catena_b200_set_blocking(0)
    llama = llama_bench(cb, L, torch, dev, stream, peaks, LLAMA, reps=2)
    L.catena_b200_set_blocking(1)
    barrier()

    # ---- strong scaling of one problem with the final gather (its checksums are the same for every --gpus N)
    L.catena_b200_set_blocking(0)
    sharded = sharded_bench(cb, L, torch, dist if world > 1 else None, shard, dev, stream, rank, world, peaks,
                            with_oracle=(rank == 0 and world == 1 and not args.no_cpu_baseline))
    L.catena_b200_set_blocking(1)
    barrier()

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        import oracle
        oracle.build()
        threads = oracle.max_threads()
        rows = 64
        t0 = time.perf_counter()
        want = oracle.gemm_bf16_rows(a_np, bt_np, GEMM_N, GEMM_K, 0, rows, threads=threads)
        sec = time.perf_counter() - t0
        more = min(GEMM_M, int(rows * 12.0 / max(sec, 1e-3)) // 64 * 64)   # about 12 s of CPU work
        if more > 2 * rows:
            rows = more
            t0 = time.perf_counter()
            want = oracle.gemm_bf16_rows(a_np, bt_np, GEMM_N, GEMM_K, 0, rows, threads=threads)
            sec = time.perf_counter() - t0
        got = c_host.reshape(GEMM_M, GEMM_N)[:rows]
        agree = float((got == want).mean())
        cpu_baseline = {"value": 2.0 * rows * GEMM_N * GEMM_K / sec / 1e12, "unit": "TFLOP/s", "cores": threads,
                        "kind": "port",
                        "sample": f"first {rows} of {GEMM_M} output rows, {sec:.1f} s; bitwise agreement with the GPU rows {agree:.5f}"}

    if rank == 0:
        line = {
            "metric": "bf16_gemm_tflops", "value": world * gemm_tflops_1, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": gemm_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "step": f"{gemm_per_step} back-to-back GEMM launches per GPU, so that the timed region lasts {gemm_ms / 1e3:.2f} s "
                               "whatever --steps is",
                       "launches_per_step": gemm_per_step, "ms_per_launch": gemm_per,
                       "l2": f"rotating over {n_sets} operand sets (384 MB) so inputs never sit in the 126 MB L2",
                       "parallelism": f"{world} independent per-GPU problems (weak scaling of replicas; strong scaling of one "
                                      "problem with its gather is under `sharded`)"},
            "clocks": {**clocks, "mhz_x_ms_per_launch": (clocks.get("sm_mhz") or 0) * gemm_per},
            "e2e": {"value": max(e2e_tflops, pipe_tflops), "unit": "TFLOP/s", "h2d_bytes_per_step": int(a_np.nbytes + bt_np.nbytes),
                    "d2h_bytes_per_step": int(c_host.nbytes), "ms_per_step": min(e2e_ms, pipe_ms),
                    "api": "host operands in pinned memory copied in and the result copied back to pinned memory every step; the value is "
                           "the pipelined form when that is faster",
                    "serial": {"value": e2e_tflops, "ms_per_step": e2e_ms, "steps": e2e_steps,
                               "api": "Runtime.exec('gemm-bf16-rc'): upload, GEMM and download one after the other on one stream"},
                    "pipelined": {"value": pipe_tflops, "ms_per_step": pipe_ms, "steps": pipe_steps,
                                  "api": "catena_b200_gemm_bf16_into on device buffers, H2D of step i+1 and D2H of step i-1 on their own "
                                         "streams (double-buffered); same result bits as the serial form"}},
            "gpu_launches": int(gemm_launches),
            "roofline": {"bound": "tensor", "achieved": gemm_tflops_1, "peak": sustained_peak, "unit": "TFLOP/s",
                         "frac": gemm_tflops_1 / sustained_peak,
                         "frac_of_burst_peak": gemm_tflops_1 / peaks["bf16_tflops"],
                         "traffic": GEMM_NCU_TRAFFIC_BYTES,
                         "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this launch "
                                           "(profiles/gemm_tc_bf16_4096.md); algorithmic bytes 100663296",
                         "peak_source": f"{peaks['source']} cuBLAS bf16, the sustained figure: the kernel is timed inside a region of "
                                        f"{gemm_ms / 1e3:.2f} s under the power cap",
                         "kernel": "gemm_tc2_kernel<bf16>"},
            "burst": {"value": world * burst_tflops_1, "unit": "TFLOP/s", "launches": 20, "ms_per_launch": burst_ms / 20,
                      "roofline": {"bound": "tensor", "achieved": burst_tflops_1, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                   "frac": burst_tflops_1 / peaks["bf16_tflops"], "peak_source": f"{peaks['source']} cuBLAS bf16, the burst figure"},
                      "note": "the first 20 launches from an idle GPU, timed alone"},
            "kernels": kernels,
            "attn_decode": {"metric": "kv_attn_decode_hbm_gbs", "value": world * attn_gbs_1, "unit": "GB/s",
                            "ms_per_launch": attn_per, "launches_per_step": attn_per_step, "gpu_launches": int(attn_launches), "clocks": attn_clocks,
                            "config": {"workload": "decode attention B=32 Hq=32 Hkv=8 D=128 L=4096 bf16, 537395200 algorithmic bytes per launch"},
                            "roofline": {"bound": "hbm", "achieved": attn_gbs_1, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                         "frac": attn_gbs_1 / peaks["hbm_gbs"], "traffic": ATTN_NCU_TRAFFIC_BYTES,
                                         "traffic_source": "4 x the ncu capture of the B=8 case (profiles/attn_decode_tc_small_B8.md)",
                                         "peak_source": f"{peaks['source']} copy bandwidth", "kernel": "attn_decode_tc_kernel"}},
            "llama_block": llama,
            "sharded": {"scaling": "strong", "n_gpus": world,
                        "timing": "ms_total and ms_1gpu: CUDA events around 8 back-to-back steps, mean of 3 regions, max over ranks; "
                                  "ms_compute / ms_gather: events inside single steps",
                        **sharded},
            "cpu_baseline": cpu_baseline,
            "output_checksum": f"{checksum:016x}",
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def kernel_suite(cb, L, torch, dev, stream, peaks, sm_max_mhz):
    """The elementwise / fold / f32 kernels of the path on bench-size inputs, device-timed, each with the roofline that
    bounds it: HBM for the map, softmax and rmsnorm (algorithmic passes over 64 Mi f32), the unfused FP32 pipe for the
    bit-exact f32 matmul (mul and add are separate instructions by contract: one flop per lane per clock)."""
    out = {}
    fp32_unfused_peak = 148 * 128 * sm_max_mhz * 1e6 / 1e12
    for which, small in (("matmul_f32", True), ("matmul_f32", False), ("map", False), ("map_program", False), ("map_interpreted", False), ("softmax", False),
                         ("rmsnorm", False), ("sum_u64", False), ("dot_u64", False)):
        step, work, unit, desc = single_case(cb, L, torch, dev, which, small, None)
        steps = 200 if (which == "matmul_f32" and small) else (16 if which == "matmul_f32" else 20)
        torch.cuda.synchronize(dev)
        with torch.cuda.stream(stream):
            for i in range(3):
                step(i)
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with ClockSampler(dev.index or 0) as sampler:
                e0.record(stream)
                for i in range(steps):
                    step(i)
                e1.record(stream)
                torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / steps
        sampled_mhz = sampler.summary().get("sm_mhz")
        value = work / (ms * 1e-3)
        if which == "matmul_f32":
            roof = {"bound": "fp32 lanes (unfused mul + add)", "achieved": value, "peak": fp32_unfused_peak, "unit": "TFLOP/s",
                    "frac": value / fp32_unfused_peak,
                    "peak_source": f"148 SMs x 128 FP32 lanes x {sm_max_mhz} MHz x 1 flop per instruction (no measured figure for this pipe)"}
            if small:
                roof["note"] = "33.6 MFLOP per launch: bound by launch latency, the time is the figure"
            elif sampled_mhz:
                # the FP32 pipe at full issue runs under the power cap: the fraction at the clock the region actually held
                roof["sm_mhz"] = sampled_mhz
                roof["frac_at_sampled_clock"] = value / (148 * 128 * sampled_mhz * 1e6 / 1e12)
        else:
            roof = {"bound": "hbm", "achieved": value, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": value / peaks["hbm_gbs"],
                    "peak_source": f"{peaks['source']} copy bandwidth"}
        name = {"matmul_f32": "matmul_f32_256" if small else "matmul_f32_4096", "map": "map_nn_silu_64Mi",
                "map_program": "map_program_nn_silu_64Mi", "map_interpreted": "map_interpreted_nn_silu_64Mi"}.get(which, which + "_64Mi")
        if which == "map_program":
            roof["note"] = ("the generic path for producers without a prebuilt kernel: the producer's register program as a kernel of "
                            "its own (PTX written by the library, compiled by the driver); the same function as map_nn_silu_64Mi, bit for bit")
        if which == "map_interpreted":
            roof["note"] = ("the same register program on the library's interpreter (the cross-check of the compiled kernel): bound by "
                            "the interpreter's instruction issue, not by HBM; same bits")
        if which in ("sum_u64", "dot_u64"):
            roof["note"] = "each step is a whole program call: one kernel whose last CTA writes the total to pinned host memory, and a stream synchronisation"
        out[name] = {"case": desc, "us_per_launch": ms * 1e3, "value": value, "unit": unit, "steps": steps, "sm_mhz": sampled_mhz, "roofline": roof}
    cb.check(L.catena_b200_check_device_errors())
    return out


NVLINK_GBS_MEASURED = 770.0      # peer copy per direction per GPU measured on this pool (nominal 900)


def sharded_bench(cb, L, torch, dist, shard, dev, stream, rank, world, peaks, reps=3, with_oracle=False):
    """Strong scaling of ONE problem over the ranks, gather included, every rank ending with the full result:
      * the int8 and bf16 GEMMs 16384 x 16384 x 8192 sharded by row blocks of A / C, the gather either an NCCL all-gather
        or fused into the GEMM's epilogue (peer stores through CUDA-IPC mappings);
      * the decode attention of the bench sharded by (batch, kv-head) ranges, the gather of O either NCCL or fused into
        the kernel's output stores;
      * once, the bf16 4096^3 GEMM sharded by output-COLUMN blocks with an NCCL gather of the column blocks.
    Every item carries the time of the unsharded problem on one GPU measured in the same run (`ms_1gpu`), the speed-up
    against it, a floor and what limits it.  Checksums must be the same for every world size: tile shape, k order and KV
    split count never depend on the sharding."""
    M = N = 16384
    K = 8192
    g = torch.Generator(device=dev)
    g.manual_seed(4)                                          # the same operands on every rank
    a8 = torch.randint(-128, 128, (M, K), generator=g, device=dev, dtype=torch.int8)
    b8 = torch.randint(-128, 128, (N, K), generator=g, device=dev, dtype=torch.int8)
    a16 = (torch.randn((M, K), generator=g, device=dev) / math.sqrt(K)).to(torch.bfloat16)
    b16 = (torch.randn((N, K), generator=g, device=dev) / math.sqrt(K)).to(torch.bfloat16)
    blocks = shard.row_blocks(M, world)
    mine = blocks[rank]
    rows = mine.m1 - mine.m0
    q = torch.randn((ATT["B"], ATT["Hq"], ATT["D"]), generator=g, device=dev).to(torch.bfloat16)
    k = torch.randn((ATT["B"], ATT["Hkv"], ATT["L"], ATT["D"]), generator=g, device=dev).to(torch.bfloat16)
    v = torch.randn((ATT["B"], ATT["Hkv"], ATT["L"], ATT["D"]), generator=g, device=dev).to(torch.bfloat16)
    units = ATT["B"] * ATT["Hkv"]
    ranges = shard.unit_ranges(units, world)
    G = ATT["Hq"] // ATT["Hkv"]
    dd = dist if world > 1 else None
    res = {}

    class _DevArray:                                           # lets torch view one of the library's allocations
        def __init__(self, ptr, shape, typestr):
            self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 3}

    def alloc(nbytes):
        m = cb.CatenaMem()
        cb.check(L.catena_b200_mem_alloc(nbytes, C.byref(m)))
        return m

    def share(mem, nbytes):
        """CUDA-IPC: every rank maps every other rank's allocation; returns [(imported mem, offset)] in rank order."""
        if world == 1:
            return []
        handle = (C.c_ubyte * 64)()
        off = C.c_uint64()
        cb.check(L.catena_b200_ipc_export(mem, handle, C.byref(off)))
        handles = [None] * world
        dist.all_gather_object(handles, (bytes(handle), int(off.value)))
        out = []
        for r in range(world):
            if r == rank:
                continue
            m_ = cb.CatenaMem()
            hb = (C.c_ubyte * 64).from_buffer_copy(handles[r][0])
            cb.check(L.catena_b200_ipc_import(hb, handles[r][1], nbytes, C.byref(m_)))
            out.append((m_, handles[r][1]))
        return out

    def unshare(imported):
        if world > 1:
            dist.barrier()
        for m_, o_ in imported:
            cb.check(L.catena_b200_ipc_close(m_, o_))
        if world > 1:
            dist.barrier()

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()

    def time_steps(step, parts=1, inner=8):
        """Device time of `step`, max over ranks.  The total is taken over `inner` back-to-back steps per timed region (mean
        of `reps` regions after a warm-up step), the way a serving loop issues them — a lone step launched into an idle
        stream measures the launch latency of its first kernel as much as the work.  With parts > 1 the split between the
        parts comes from a second pass of single steps, `step` recording the events it is given between its parts."""
        with torch.cuda.stream(stream):
            step(None)
            sync_all()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            total = 0.0
            for _ in range(reps):
                e0.record(stream)
                for _ in range(inner):
                    step(None)
                e1.record(stream)
                sync_all()                                     # every rank's stores have landed before the next region
                total += e0.elapsed_time(e1) / inner / reps
            t = [total]
            if parts > 1:
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(parts + 1)]
                t = [0.0] * parts
                for _ in range(reps):
                    ev[0].record(stream)
                    step(ev)
                    ev[parts].record(stream)
                    sync_all()
                    for i in range(parts):
                        t[i] += ev[i].elapsed_time(ev[i + 1]) / reps
        return [shard.max_over_ranks(x, dd, dev) for x in t], shard.max_over_ranks(total, dd, dev)

    def checksum(t):
        view = t.view(torch.int16) if t.dtype == torch.bfloat16 else t
        return f"{int(view.to(torch.int64).sum().item()) & 0xFFFFFFFFFFFF:012x}"

    def finish(item, ms_1gpu, floor_ms, limiter, work, unit):
        item.update({"ms_1gpu": ms_1gpu, "speedup_vs_1gpu": ms_1gpu / item["ms_total"], "floor_ms": floor_ms, "limiter": limiter,
                     "value_incl_gather": work / (item["ms_total"] * 1e-3), "unit": unit})
        return item

    # ------------------------------------------------------------------ GEMMs 16384 x 16384 x 8192, int8 and bf16
    for tag, a, b, eb_out, typestr, torch_out, fn_into, fn_peers in (
            ("i8", a8, b8, 4, "<i4", torch.int32, L.catena_b200_gemm_i8_into, L.catena_b200_gemm_i8_into_peers),
            ("bf16", a16, b16, 2, "<i2", torch.int16, L.catena_b200_gemm_bf16_into, L.catena_b200_gemm_bf16_into_peers)):
        name = f"gemm_{tag}_16384x16384x8192"
        work, unit = 2.0 * M * N * K / 1e12, ("TOP/s" if tag == "i8" else "TFLOP/s")
        c_full = alloc(M * N * eb_out)                         # this rank's copy of the whole C
        full_view = torch.as_tensor(_DevArray(c_full.data, (M, N), typestr), device=dev)
        a_ptr, b_ptr = a.data_ptr(), b.data_ptr()
        es = a.element_size()
        # the unsharded problem on this GPU, measured in the same run
        [_], ms_1 = time_steps(lambda ev: cb.check(fn_into(a_ptr, b_ptr, c_full.data, M, N, K, N)))
        sum_1 = checksum(full_view)
        oracle_note = None
        if with_oracle:
            import oracle
            slab = slice(8192 + 256 - 16, 8192 + 256 + 16)     # 32 rows across a 256-row tile boundary
            got = full_view[slab].cpu().numpy()
            if tag == "i8":
                a_h, b_h = a[slab].cpu().numpy(), b.cpu().numpy()
            else:
                a_h, b_h = a[slab].view(torch.int16).cpu().numpy(), b.view(torch.int16).cpu().numpy()
            if tag == "i8":
                want = oracle.gemm_i8_rows(a_h, b_h, N, K, 0, 32, threads=oracle.max_threads())
                oracle_note = f"rows {slab.start}..{slab.stop - 1} against the CPU oracle: bitwise agreement {float((got == want).mean()):.5f}"
            else:
                want = oracle.gemm_bf16_rows(a_h.view(np.uint16), b_h.view(np.uint16), N, K, 0, 32, threads=oracle.max_threads())
                oracle_note = (f"rows {slab.start}..{slab.stop - 1} against the CPU oracle (sequential fp32 fold): bitwise agreement "
                               f"{float((got.view(np.uint16) == want).mean()):.5f}, the rest one bf16 ulp apart")
        bytes_c = M * N * eb_out
        link_floor = (world - 1) / world * bytes_c / (NVLINK_GBS_MEASURED * 1e9) * 1e3
        floor = max(ms_1 / world, link_floor)
        limiter = ("NVLink ingress: every rank receives (N-1)/N of C" if link_floor > ms_1 / world else "tensor pipe") if world > 1 else "tensor pipe"
        # (1) compute on the row block, NCCL all-gather of the blocks
        c_block = torch.empty((rows, N), dtype=torch_out, device=dev)
        holder = {}
        full_view.zero_()

        def nccl_step(ev):
            cb.check(fn_into(a_ptr + mine.m0 * K * es, b_ptr, c_block.data_ptr(), rows, N, K, N))
            if ev:
                ev[1].record(stream)
            holder["full"] = shard.gather_rows(c_block, blocks, dd, out=full_view if world > 1 else None)
        (t_c, t_g), total = time_steps(nccl_step, parts=2)
        item = {"ms_total": total, "ms_compute": t_c, "ms_gather": t_g, "checksum": checksum(holder["full"]), "gather": "NCCL all-gather of row blocks"}
        assert item["checksum"] == sum_1, "sharded result differs from the unsharded one"
        res[name] = finish(item, ms_1, floor, limiter, work, unit)
        if oracle_note:
            res[name]["oracle"] = oracle_note
        holder.clear()
        del c_block
        # (2) the gather fused into the epilogue: every rank stores its row block into every rank's C
        if world > 1:
            imported = share(c_full, bytes_c)
            ptrs = [m_.data + mine.m0 * N * eb_out for m_, _ in imported]
            peer_arr = (C.c_void_p * len(ptrs))(*ptrs)
            full_view.zero_()
            sync_all()
            [_], total = time_steps(lambda ev: cb.check(fn_peers(a_ptr + mine.m0 * K * es, b_ptr, c_full.data + mine.m0 * N * eb_out, rows, N, K, N,
                                                                 peer_arr, len(ptrs))))
            item = {"ms_total": total, "checksum": checksum(full_view), "gather": "fused: epilogue stores every tile to all ranks' C over NVLink; "
                    "one host barrier after the stream drains replaces the collective",
                    "link_gbs_per_rank": (world - 1) / world * bytes_c / (total * 1e-3) / 1e9, "link_gbs_measured_peak": NVLINK_GBS_MEASURED}
            assert item["checksum"] == sum_1, "fused-gather result differs from the unsharded one"
            res[name + "_fused_gather"] = finish(item, ms_1, floor, limiter, work, unit)
            unshare(imported)
        del full_view
        cb.free(c_full)

    # ------------------------------------------------------------------ decode attention C3
    work, unit = ATT_BYTES / 1e9, "GB/s"
    o_mem = alloc(units * G * ATT["D"] * 2)
    o_view = torch.as_tensor(_DevArray(o_mem.data, (units, G * ATT["D"]), "<i2"), device=dev)
    att_args = (q.data_ptr(), k.data_ptr(), v.data_ptr(), o_mem.data, ATT["B"], ATT["Hq"], ATT["Hkv"], ATT["D"], ATT["L"])
    [_], ms_1 = time_steps(lambda ev: cb.check(L.catena_b200_attn_decode_bf16_into(*att_args, 0, units)))
    sum_1 = checksum(o_view)
    floor = ATT_BYTES / world / (peaks["hbm_gbs"] * 1e9) * 1e3
    limiter = "HBM" if world == 1 else "fixed cost per launch (set-up, exchange of chunk maxima, ticket, combine) once the KV stream per GPU is short"
    holder = {}

    def attn_nccl(ev):
        cb.check(L.catena_b200_attn_decode_bf16_into(*att_args, ranges[rank].u0, ranges[rank].u1))
        if ev:
            ev[1].record(stream)
        holder["full"] = shard.gather_units(o_view[ranges[rank].u0:ranges[rank].u1], ranges, G * ATT["D"], dd,
                                            out=o_full if world > 1 else None)
    o_full = torch.zeros((units, G * ATT["D"]), dtype=torch.int16, device=dev)
    o_view.zero_()
    (t_c, t_g), total = time_steps(attn_nccl, parts=2)
    item = {"ms_total": total, "ms_compute": t_c, "ms_gather": t_g, "checksum": checksum(holder["full"]), "gather": "NCCL all-gather of O"}
    assert item["checksum"] == sum_1, "sharded attention differs from the unsharded one"
    res["attn_decode_c3"] = finish(item, ms_1, floor, limiter, work, unit)
    holder.clear()
    if world > 1:
        imported = share(o_mem, units * G * ATT["D"] * 2)
        peer_arr = (C.c_void_p * len(imported))(*[m_.data for m_, _ in imported])
        o_view.zero_()
        sync_all()
        [_], total = time_steps(lambda ev: cb.check(L.catena_b200_attn_decode_bf16_into_peers(*att_args, ranges[rank].u0, ranges[rank].u1,
                                                                                              peer_arr, len(imported))))
        item = {"ms_total": total, "checksum": checksum(o_view), "gather": "fused: the warps that write a unit's outputs also store them into "
                "every rank's O over NVLink; one host barrier after the stream drains replaces the collective"}
        assert item["checksum"] == sum_1, "fused-gather attention differs from the unsharded one"
        res["attn_decode_c3_fused_gather"] = finish(item, ms_1, floor, limiter, work, unit)
        unshare(imported)
    del o_view
    cb.free(o_mem)

    # ------------------------------------------------------------------ output-column blocks (bf16 4096^3), NCCL gather of the blocks
    m4 = n4 = k4 = 4096
    a4, b4 = a16[:m4, :k4].contiguous(), b16[:n4, :k4].contiguous()
    c4 = torch.empty((m4, n4), dtype=torch.int16, device=dev)
    [_], ms_1 = time_steps(lambda ev: cb.check(L.catena_b200_gemm_bf16_into(a4.data_ptr(), b4.data_ptr(), c4.data_ptr(), m4, n4, k4, n4)))
    sum_1 = checksum(c4)
    cols = shard.column_blocks(n4, world)
    mc = cols[rank]
    width = mc.n1 - mc.n0
    c_cols = torch.empty((m4, width), dtype=torch.int16, device=dev)
    holder = {}

    def col_step(ev):
        cb.check(L.catena_b200_gemm_bf16_into(a4.data_ptr(), b4.data_ptr() + mc.n0 * k4 * 2, c_cols.data_ptr(), m4, width, k4, width))
        if ev:
            ev[1].record(stream)
        holder["full"] = shard.gather_columns(c_cols, cols, m4, dd)
    (t_c, t_g), total = time_steps(col_step, parts=2)
    item = {"ms_total": total, "ms_compute": t_c, "ms_gather": t_g, "checksum": checksum(holder["full"]),
            "gather": "NCCL all-gather of output-column blocks, repacked into row-major C"}
    assert item["checksum"] == sum_1, "column-sharded result differs from the unsharded one"
    link_floor = (world - 1) / world * m4 * n4 * 2 / (NVLINK_GBS_MEASURED * 1e9) * 1e3
    res["gemm_bf16_4096_column_blocks"] = finish(item, ms_1, max(ms_1 / world, link_floor),
                                                 "launch + NCCL latency: the whole problem is 0.1 ms on one GPU" if world > 1 else "tensor pipe",
                                                 2.0 * m4 * n4 * k4 / 1e12, "TFLOP/s")
    cb.check(L.catena_b200_check_device_errors())
    return res


LLAMA = dict(hidden=2048, n_heads=16, n_kv_heads=16, ffn=8192, vocab=32000, batch=4, seq=2048, decode_steps=128)
LLAMA_SMALL = dict(hidden=1024, n_heads=8, n_kv_heads=8, ffn=2048, vocab=4000, batch=2, seq=512, decode_steps=16)


def llama_bench(cb, L, torch, dev, stream, peaks, cfg, reps=2):
    """Llama-style block: prefill of batch x seq tokens, then decode_steps single-token steps, device-timed.
    Weights N(0, 0.02) bf16, token ids uniform, seed 5 (synthetic).  Returns times and roofline fractions:
    prefill against the tensor peak (projection + causal attention FLOP), decode against the copy bandwidth
    (weights + visible KV rows read once per step)."""
    H, Hq, Hkv, F, V = cfg["hidden"], cfg["n_heads"], cfg["n_kv_heads"], cfg["ffn"], cfg["vocab"]
    B, S, steps = cfg["batch"], cfg["seq"], cfg["decode_steps"]
    max_len = S + steps
    g = torch.Generator(device=dev)
    g.manual_seed(5)
    def w(rows, cols):
        return (torch.randn((rows, cols), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    emb, wqkv, wo, wgu, wd = w(V, H), w((Hq + 2 * Hkv) * 128, H), w(H, Hq * 128), w(2 * F, H), w(H, F)
    blk = cb.LlamaBlockStruct(H, Hq, Hkv, F, V, max_len, emb.data_ptr(), wqkv.data_ptr(), wo.data_ptr(), wgu.data_ptr(),
                              wd.data_ptr(), 10000.0)
    ids = torch.randint(0, V, (B * S,), generator=g, device=dev, dtype=torch.int32)
    step_ids = torch.randint(0, V, (steps, B), generator=g, device=dev, dtype=torch.int32)
    kc = torch.zeros((B, Hkv, max_len, 128), dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    ws_bytes = L.catena_b200_llama_workspace_bytes(C.byref(blk), B * S)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    out = torch.empty((B * S, H), dtype=torch.bfloat16, device=dev)
    torch.cuda.synchronize(dev)

    def prefill():
        cb.check(L.catena_b200_llama_prefill(C.byref(blk), ids.data_ptr(), B, S, kc.data_ptr(), vc.data_ptr(), out.data_ptr(),
                                             ws.data_ptr(), ws_bytes))

    def decode_all():
        for t in range(steps):
            cb.check(L.catena_b200_llama_decode(C.byref(blk), step_ids[t].data_ptr(), B, S + t, kc.data_ptr(), vc.data_ptr(),
                                                out.data_ptr(), ws.data_ptr(), ws_bytes))

    times = {}
    with torch.cuda.stream(stream):
        for name, fn in (("prefill", prefill), ("decode", decode_all)):
            fn()                                             # warm-up (also fills the caches for the decode steps)
            torch.cuda.synchronize(dev)
            launches0 = L.catena_b200_launch_count()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            h0 = time.perf_counter()
            e0.record(stream)
            for _ in range(reps):
                fn()
            e1.record(stream)
            times[name + "_host"] = (time.perf_counter() - h0) / reps * 1e3      # ms the host spent enqueuing
            torch.cuda.synchronize(dev)
            times[name] = e0.elapsed_time(e1) / reps
            times[name + "_launches"] = (L.catena_b200_launch_count() - launches0) // reps
    cb.check(L.catena_b200_check_device_errors())
    params = H * (Hq + 2 * Hkv) * 128 + H * Hq * 128 + 3 * F * H
    prefill_flop = 2.0 * B * S * params + 4.0 * B * Hq * 128 * S * (S + 1) / 2
    decode_bytes = sum(params * 2 + 2 * B * Hkv * (S + t + 1) * 128 * 2 for t in range(steps)) / steps
    pre_tf = prefill_flop / (times["prefill"] * 1e-3) / 1e12
    dec_ms = times["decode"] / steps
    dec_gbs = decode_bytes / (dec_ms * 1e-3) / 1e9
    checksum = int(out[:B].view(torch.int16).to(torch.int64).sum().item()) & 0xFFFFFFFFFFFF
    return {"config": {"workload": f"Llama-style block hidden {H}, {Hq}x128 heads ({Hkv} kv), ffn {F}: prefill {B}x{S} tokens, "
                                   f"then {steps} decode steps of {B} tokens; bf16, fp32 accumulate"},
            "prefill_ms": times["prefill"], "prefill_tflops": pre_tf, "prefill_launches": times["prefill_launches"],
            "prefill_roofline": {"bound": "tensor", "achieved": pre_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                 "frac": pre_tf / peaks["bf16_tflops"]},
            "decode_ms_per_step": dec_ms, "decode_host_ms_per_step": times["decode_host"] / steps, "decode_gbs": dec_gbs, "decode_launches_per_step": times["decode_launches"] // steps,
            "decode_roofline": {"bound": "hbm", "achieved": dec_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                "frac": dec_gbs / peaks["hbm_gbs"]},
            "end_to_end_ms": times["prefill"] + times["decode"], "output_checksum": f"{checksum:012x}"}


def single_case(cb, L, torch, dev, which, small, shape, units=0):
    """One kernel of the path on the bench workload (or a smaller case): returns (step(i), work per launch, unit, text)."""
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    if which in ("gemm", "gemm_i8"):
        m = n = k = 2048 if small else 4096
        if shape:
            m, n, k = [int(v) for v in shape.split("x")]
        eb = 1 if which == "gemm_i8" else 2
        sets = []
        for _ in range(4):
            if eb == 1:
                a = torch.randint(-128, 128, (m, k), generator=g, device=dev, dtype=torch.int8)
                b = torch.randint(-128, 128, (n, k), generator=g, device=dev, dtype=torch.int8)
                c = torch.empty((m, n), dtype=torch.int32, device=dev)
            else:
                a = (torch.randn((m, k), generator=g, device=dev) / math.sqrt(k)).to(torch.bfloat16)
                b = (torch.randn((n, k), generator=g, device=dev) / math.sqrt(k)).to(torch.bfloat16)
                c = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
            sets.append((a, b, c))
        fn = L.catena_b200_gemm_i8_into if eb == 1 else L.catena_b200_gemm_bf16_into

        def step(i):
            a, b, c = sets[i % 4]
            cb.check(fn(a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, n))
        work, unit = 2.0 * m * n * k / 1e12, "TFLOP/s"
        desc = f"{which} {m}x{n}x{k}"
    elif which == "attn":
        B, Hq, Hkv, D, Lk = (8, 32, 8, 128, 4096) if small else (32, 32, 8, 128, 4096)
        sets = []
        for _ in range(2):
            q = torch.randn((B, Hq, D), generator=g, device=dev).to(torch.bfloat16)
            kk = torch.randn((B, Hkv, Lk, D), generator=g, device=dev).to(torch.bfloat16)
            vv = torch.randn((B, Hkv, Lk, D), generator=g, device=dev).to(torch.bfloat16)
            o = torch.empty((B, Hq, D), dtype=torch.bfloat16, device=dev)
            sets.append((q, kk, vv, o))

        n_units = min(units, B * Hkv) if units else B * Hkv      # --units: only the first (batch, kv-head) units, as one rank of a sharded run

        def step(i):
            q, kk, vv, o = sets[i % 2]
            cb.check(L.catena_b200_attn_decode_bf16_into(q.data_ptr(), kk.data_ptr(), vv.data_ptr(), o.data_ptr(), B, Hq,
                                                         Hkv, D, Lk, 0, n_units))
        work, unit = n_units * (2 * Lk * D * 2 + 2 * (Hq // Hkv) * D * 2) / 1e9, "GB/s"
        desc = f"attn decode B={B} Hq={Hq} Hkv={Hkv} D={D} L={Lk}, units 0..{n_units - 1}"
    elif which == "matmul_f32":
        n = 256 if small else 4096
        a = torch.rand((n, n), generator=g, device=dev) * 2 - 1
        b = torch.rand((n, n), generator=g, device=dev) * 2 - 1
        c = torch.empty((n, n), device=dev)

        def step(i):
            cb.check(L.catena_b200_matmul_f32_into(a.data_ptr(), b.data_ptr(), c.data_ptr(), n, n, n))
        work, unit = 2.0 * n ** 3 / 1e12, "TFLOP/s"
        desc = f"f32 matmul {n}^3 (bit-exact sequential-k)"
    elif which in ("sum_u64", "dot_u64"):
        n = (1 << 22) if small else (1 << 26)                   # 64 Mi u64 = 512 MiB per buffer
        x = torch.randint(-2 ** 62, 2 ** 62, (2, n), generator=g, device=dev, dtype=torch.int64)
        y = torch.randint(-2 ** 62, 2 ** 62, (2, n), generator=g, device=dev, dtype=torch.int64) if which == "dot_u64" else None
        res = C.c_uint64(0)

        def step(i):
            s = i % 2
            xm = cb.CatenaMem(x[s].data_ptr(), n * 8)
            if which == "dot_u64":
                cb.check(L.program_dot_u64_s(xm, cb.CatenaMem(y[s].data_ptr(), n * 8), C.byref(res)))
            else:
                cb.check(L.program_sum_u64_s(xm, C.byref(res)))
        work, unit = (2 if which == "dot_u64" else 1) * n * 8 / 1e9, "GB/s"
        desc = f"{which} over {n} u64 (exact: arithmetic modulo 2^64)"
    else:  # map / softmax / rmsnorm over 64 Mi f32 (256 MiB in, 256 MiB out)
        n = (1 << 24) if small else (1 << 26)
        x = torch.randn((2, n), generator=g, device=dev)
        y = torch.empty((2, n), device=dev)

        program = None
        if which in ("map_program", "map_interpreted"):
            # nn.silu again, but as a user's `materializec` producer would arrive: lowered modules of the stdlib programs
            # (exp~ from its primitives), compiled to a register program; that program runs as a kernel of its own
            # (map_program) or on the generic map kernel's interpreter (map_interpreted)
            from catena_lang_b200 import lowering as lo
            from catena_lang_b200.lowered_stdlib import silu_modules
            mods = silu_modules()
            at = lo.GpuModule("program_bench_silu_at", "bench.silu-at", lo.GpuFunction("program_bench_silu_at",
                [lo.GpuVar("x", "ptr<f32>"), lo.GpuVar("i", "u64")], [lo.GpuVar("r", "f32")],
                [lo.GpuAssign("ix", [lo.GpuVar("i", "u64"), lo.GpuVar("x", "ptr<f32>")], [lo.GpuVar("xi", "f32")]),
                 lo.GpuAssign("nn.silu", [lo.GpuVar("xi", "f32")], [lo.GpuVar("r", "f32")], cb.symbol_for("nn.silu"))]))
            launch = lo.GpuAssign("materializec", [lo.GpuVar("len", "u64"), lo.GpuVar("x", "ptr<f32>"), lo.FnSymbol("bench.silu-at")],
                                  [lo.GpuVar("buf", "ptr<f32>")], None, [1, 1, 1], [1])
            program = lo.map_program_for(launch, lo.module_map(mods + [at]))

        def step(i):
            s = i % 2
            if program is not None:
                # the program allocates its output, as materializec does
                cb.free(program.launch(n, [(x[s].data_ptr(), n * 4)], compiled=which == "map_program"))
            elif which == "softmax":
                cb.check(L.catena_b200_softmax_f32_into(x[s].data_ptr(), y[s].data_ptr(), n))
            elif which == "rmsnorm":
                cb.check(L.catena_b200_rmsnorm_f32_into(x[s].data_ptr(), y[s].data_ptr(), n))
            else:
                cb.check(L.catena_b200_map_f32_into(b"nn.silu", x[s].data_ptr(), y[s].data_ptr(), n))
        passes = {"softmax": 4, "rmsnorm": 3}.get(which, 2)     # algorithmic reads + writes of the buffer
        work, unit = passes * n * 4 / 1e9, "GB/s"
        desc = f"{which} over {n} f32"
        if program is not None:
            how = "compiled to its own kernel" if which == "map_program" else "interpreted"
            desc = f"nn.silu as a register program ({len(program.code)} instructions, {program.n_regs} registers), {how}, over {n} f32"
    return step, work, unit, desc


def run_single(args):
    """`--only <kernel>`: a few launches of one kernel on the bench workload (or a smaller case with
    `--small`), for profiler captures and quick timing.  Prints a short JSON line."""
    import torch
    import catena_lang_b200 as cb

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    L = cb.lib()
    cb.check(L.catena_b200_init(0))
    stream = torch.cuda.Stream(device=dev)
    L.catena_b200_set_stream(C.c_void_p(stream.cuda_stream))
    L.catena_b200_set_blocking(0)
    which = args.only
    if which == "llama":
        cfg = dict(LLAMA_SMALL if args.small else LLAMA)
        if args.decode_steps:
            cfg["decode_steps"] = args.decode_steps
        res = llama_bench(cb, L, torch, dev, stream, measured_peaks(), cfg, reps=max(1, min(args.steps, 3)))
        print(json.dumps({"only": "llama", **res}), flush=True)
        return
    step, work, unit, desc = single_case(cb, L, torch, dev, which, args.small, args.shape, args.units)
    torch.cuda.synchronize(dev)
    with torch.cuda.stream(stream):
        for i in range(args.warmup):
            step(i)
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(args.steps):
            step(i)
        e1.record(stream)
        torch.cuda.synchronize(dev)
    cb.check(L.catena_b200_check_device_errors())
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"only": which, "case": desc, "ms_per_step": ms, "value": work / (ms * 1e-3), "unit": unit,
                      "steps": args.steps, "warmup": args.warmup}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None,
                    choices=["gemm", "gemm_i8", "attn", "matmul_f32", "map", "map_program", "map_interpreted", "softmax", "rmsnorm", "sum_u64", "dot_u64", "llama"])
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--shape", default=None, help="MxNxK for --only gemm / gemm_i8")
    ap.add_argument("--units", type=int, default=0, help="--only attn: launch only the first N (batch, kv-head) units")
    ap.add_argument("--decode-steps", type=int, default=0, help="decode steps for --only llama (default: the workload's 128)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--launches-per-step", type=int, default=0,
                    help="launches per step of the headline loops (default: sized from a 20-launch probe so that the timed region "
                         "lasts 0.5 s; a profiler serialises the probe, so profile runs pin the number the plain run printed)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.only:
        run_single(args)
        return
    run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
