#!/usr/bin/env python
"""Benchmark of the attention forward hot path on B200.

``python bench.py --gpus N --steps K --warmup W`` (under torchrun for N > 1)
prints ONE JSON line on rank 0.

Workload (N = 1): causal prefill, fp16, B=8 H=12 S=2048 D=64, scale 1/8 - the
shape the reference's headline number is quoted on.  A "step" is one
``fa_prefill`` launch over that batch.  For N > 1 every rank runs the same
per-GPU batch on its own GPU (weak scaling over the batch x head axis, no
collective on the data path); the line also carries the strong-scaling split of
the same 96 heads for comparison.

``value``     whole-job TFLOP/s with inputs resident in HBM (causal FLOP count
              4*BH*D*S*(S+1)/2; the reference's own convention 4*BH*S^2*D, which
              counts masked work, is given as ``tflops_refconv``).
``e2e``       same metric through ``fa_prefill_host``: pinned host buffers, H2D
              of Q,K,V and D2H of O and LSE inside the timed region, every step.
``roofline``  tensor-core roofline of the prefill kernel against the measured
              cuBLAS bf16 peak; ``decode`` carries the HBM roofline of the
              split-KV decode kernel (B=32 H=32 Skv=16384 D=128, 16 splits).
``cpu_baseline``  the reference's own cpu_attention (oracle/_ref) on the host
              cores, same metric, reported only.

``--impl reference`` times that CPU implementation alone on the same config.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024
# DRAM traffic of the prefill kernel from one ncu capture (dram__bytes_read.sum + dram__bytes_write.sum,
# profiles/prefill_d64_causal_f16_launches_and_counters.md) on 24 heads of the workload; traffic is
# proportional to the number of heads, so it is scaled to the heads of the run.
PREFILL_TRAFFIC_BYTES = 18.92e6
PREFILL_TRAFFIC_NOTE = ("ncu on 24 heads: 18.92 MB read (= Q+K+V, 18.87 MB algorithmic), 0 written back during the "
                        "kernel (O and LSE still in L2); scaled by heads")
DECODE_TRAFFIC_BYTES = 1.0739e9 + 3.9e6   # ncu on B=4 (128 heads): read + write per launch
CFG = dict(B=8, H=12, S=2048, D=64, CAUSAL=True, DTYPE="f16")
DEC = dict(B=32, H=32, SKV=16384, D=128, SPLITS=16)


def causal_flops(bh, s, d):
    return 4 * bh * d * s * (s + 1) // 2


def refconv_flops(bh, s, d):
    return 4 * bh * s * s * d


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], tflops=p["bf16_tflops"],
                    tflops_sustained=p.get("bf16_tflops_sustained"), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.0005)

    def start(self):
        if self._nv is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [x for x in vis.split(",") if x != ""]
        try:
            return int(ids[local_rank])
        except Exception:
            return local_rank
    return local_rank


# --------------------------------------------------------------------------- reference arm
def cpu_reference_run(bh_sample: int, steps: int, warmup: int, threads: int):
    """Times the reference's cpu_attention (or the oracle port when the reference
    library was not built) on `bh_sample` heads of the workload per step."""
    from oracle import oracle
    s, d = CFG["S"], CFG["D"]
    q, k, v = (oracle.round_to(x, "f16") for x in oracle.normal_inputs(2002, (bh_sample, s, d)))
    kind = "reference" if oracle.ref_lib() is not None else "port"
    fn = (lambda: oracle.ref_attention(q, k, v, 0.125, True, threads=threads)) if kind == "reference" \
        else (lambda: oracle.attention(q, k, v, 0.125, True, threads=threads))
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    tflops = causal_flops(bh_sample, s, d) / dt / 1e12
    return kind, tflops, dt


def reference_gpu_kernel_time(steps: int = 50):
    """Same-box comparison line: the reference's own mma.sync kernel
    (kernels/flash_attention.cu, recompiled unchanged for sm_100a into
    oracle/_ref/libref_gpu.so) on the benchmark workload.  Returns None when
    there is no GPU or the library was never built."""
    import ctypes
    from oracle import build_oracle
    path = os.path.join(build_oracle.REF_OUT, "libref_gpu.so")
    try:
        import torch
        if not (torch.cuda.is_available() and os.path.exists(path)):
            return None
    except Exception:
        return None

    class RefParams(ctypes.Structure):       # include/flash_attention.h:51-64 of the reference
        _fields_ = [("Q", ctypes.c_void_p), ("K", ctypes.c_void_p), ("V", ctypes.c_void_p),
                    ("O", ctypes.c_void_p), ("L", ctypes.c_void_p), ("batch_size", ctypes.c_int),
                    ("num_heads", ctypes.c_int), ("seq_len", ctypes.c_int), ("d_head", ctypes.c_int),
                    ("scale", ctypes.c_float), ("causal", ctypes.c_bool), ("stream", ctypes.c_void_p)]

    lib = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
    fn = getattr(lib, build_oracle.REF_LAUNCH_SYMBOL)
    fn.restype = None
    fn.argtypes = [ctypes.POINTER(RefParams)]
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    B, H, S, D = CFG["B"], CFG["H"], CFG["S"], CFG["D"]
    gen = torch.Generator(device=dev)
    gen.manual_seed(2002)
    q, k, v = (torch.randn((B * H, S, D), device=dev, generator=gen).to(torch.float16) for _ in range(3))
    o = torch.empty_like(q)
    lse = torch.empty((B * H, S), device=dev, dtype=torch.float32)
    p = RefParams(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), B, H, S, D,
                  0.125, True, None)
    for _ in range(5):
        fn(ctypes.byref(p))
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(torch.cuda.default_stream())
    for _ in range(steps):
        fn(ctypes.byref(p))
    e1.record(torch.cuda.default_stream())
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"kernel": "reference flash_attention_ptx_kernel (mma.sync), -gencode arch=compute_100a,code=sm_100a",
            "ms_per_step": ms, "tflops_causal_count": causal_flops(B * H, S, D) / (ms * 1e-3) / 1e12,
            "tflops_refconv": refconv_flops(B * H, S, D) / (ms * 1e-3) / 1e12}


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    bh_sample = min(CFG["B"] * CFG["H"], max(8, cores))
    steps = max(1, min(args.steps, 3))
    warmup = min(args.warmup, 1)
    kind, tflops, dt = cpu_reference_run(bh_sample, steps, warmup, cores)
    sample = (f"{bh_sample} of {CFG['B'] * CFG['H']} heads of the workload per step "
              f"(S={CFG['S']}, D={CFG['D']}, causal), {steps} timed steps, {warmup} warm-up")
    line = {
        "impl": "reference",
        "metric": "causal prefill TFLOPS (B8 H12 S2048 D64 fp16)",
        "value": tflops, "unit": "TFLOP/s (causal FLOP count)",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic: seeded iid N(0,1) rounded to fp16",
        "config": {"workload": "causal prefill fp16 B=8 H=12 S=2048 D=64 scale=1/8, per GPU",
                   "note": "CPU reference on a bounded sample of the workload's heads per step"},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s (causal FLOP count)", "cores": cores,
                         "kind": kind, "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s (causal FLOP count)", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    gpu_ref = reference_gpu_kernel_time()
    if gpu_ref:
        line["reference_gpu_kernel_on_this_gpu"] = gpu_ref   # information only; the arm's value is the CPU path
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- B200 arm
def run_b200_arm(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge

    fa = ge.load_package()
    fa.lib()                                  # fail loudly if the CUDA library is missing
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    fa.clear_device_status()
    fa.set_prefill_variant(args.variant)

    B, H, S, D = CFG["B"], CFG["H"], CFG["S"], CFG["D"]
    causal, dtype_name = CFG["CAUSAL"], CFG["DTYPE"]
    tdt = torch.float16 if dtype_name == "f16" else torch.bfloat16
    bh = B * H
    scale = float(1.0 / np.sqrt(D))           # 0.125 for the headline workload
    n_sets = 4                                # rotating input sets: 4 x 101 MB > 126 MB of L2
    gen = torch.Generator(device=dev)
    gen.manual_seed(2002 + rank)
    sets = []
    for _ in range(n_sets):
        q, k, v = (torch.randn((bh, S, D), device=dev, dtype=torch.float32, generator=gen).to(tdt)
                   for _ in range(3))
        o = torch.empty_like(q)
        lse = torch.empty((bh, S), device=dev, dtype=torch.float32)
        sets.append((q, k, v, o, lse))
    stream = torch.cuda.current_stream()

    import ctypes
    fa_prefill = fa.lib().fa_prefill

    def launch_args(n_heads, head0):
        """One fa_prefill_args per input set, built once: the timed loop then costs the host one
        foreign call per step (a 0.09 ms kernel is otherwise launch-bound from Python)."""
        out = []
        for (q, k, v, o, lse) in sets:
            out.append(fa.PrefillArgs(q[head0:].data_ptr(), k[head0:].data_ptr(), v[head0:].data_ptr(),
                                      o[head0:].data_ptr(), lse[head0:].data_ptr(), 1, n_heads, S, D, scale,
                                      int(causal), fa.DTYPES[dtype_name], None, None, None,
                                      stream.cuda_stream or None))
        return out

    full_args = launch_args(bh, 0)

    def step(i, args_list=full_args):
        rc = fa_prefill(ctypes.byref(args_list[i % n_sets]))
        if rc != 0:
            raise RuntimeError(f"fa_prefill failed: {fa.error_string(rc)}")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup, sampler=None):
        for i in range(warmup):
            fn(i)
        barrier()
        if sampler:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(steps):
            fn(i)
        e1.record(stream)
        barrier()
        if sampler:
            sampler.stop()
        total_ms = e0.elapsed_time(e1)
        per = [total_ms / steps]                  # the step is one kernel: its average launch duration
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), per

    sampler = ClockSampler(physical_index(local_rank))
    warmup = max(args.warmup, 3)
    flops_step = causal_flops(bh, S, D) if causal else refconv_flops(bh, S, D)
    # One timed loop of K steps of this workload lasts a few milliseconds, too short for a clock
    # record or a steady number.  The loop (exactly K steps between two barriers, max over ranks) is
    # therefore repeated until about 60 ms have been timed; the headline is the MEDIAN repeat, every
    # repeat's time is reported, and the clock sampler runs across all of them.
    total_ms, per = timed(step, args.steps, warmup)
    est = max(total_ms, 1e-3)
    repeats = int(min(40, max(3, np.ceil(60.0 / est)))) if est < 50.0 else 1
    t_rep = torch.tensor([repeats], device=dev, dtype=torch.int64)
    if world > 1:
        dist.all_reduce(t_rep, op=dist.ReduceOp.MAX)          # every rank must run the same number of loops
    repeats = int(t_rep.item())
    rep_ms, rep_per = [], []
    sampler.start()
    for _ in range(repeats):
        r_ms, r_per = timed(step, args.steps, 0)
        rep_ms.append(r_ms)
        rep_per.append(float(np.mean(r_per)))
    sampler.stop()
    order = int(np.argsort(rep_ms)[len(rep_ms) // 2])         # the median repeat
    total_ms = rep_ms[order]
    ms_per_step = total_ms / args.steps
    value = world * flops_step / (ms_per_step * 1e-3) / 1e12
    kernel_ms = rep_per[order]
    achieved = flops_step / (kernel_ms * 1e-3) / 1e12

    # strong-scaling split of the same 96 heads (reported beside the weak-scaling headline)
    strong = None
    if world > 1 and bh % world == 0:
        nh = bh // world
        part_args = launch_args(nh, rank * nh)
        s_ms, _ = timed(lambda i: step(i, part_args), args.steps, warmup)
        strong = {"heads_per_gpu": nh, "ms_per_step": s_ms / args.steps,
                  "tflops": flops_step / (s_ms / args.steps * 1e-3) / 1e12}
        strong.update(check_heads_against_oracle(torch, dist, dev, sets[0], [rank * nh, rank * nh + nh - 1],
                                                 S, scale, world))

    # ---- end to end: fa_prefill_host from pinned host buffers, copies inside the timed region
    hgen = torch.Generator()
    hgen.manual_seed(3003 + rank)
    hq, hk, hv = (torch.randn((bh, S, D), dtype=torch.float32, generator=hgen).to(torch.float16).pin_memory()
                  for _ in range(3))
    ho = torch.empty((bh, S, D), dtype=torch.float16).pin_memory()
    hl = torch.empty((bh, S), dtype=torch.float32).pin_memory()
    e2e_steps = 0 if args.no_e2e else max(3, min(args.steps, 20))

    def e2e_step(_i):
        rc = fa.prefill_raw(hq.data_ptr(), hk.data_ptr(), hv.data_ptr(), ho.data_ptr(), hl.data_ptr(),
                            1, bh, S, D, scale, True, dtype="f16", host=True)
        if rc != 0:
            raise RuntimeError(f"fa_prefill_host failed: {fa.error_string(rc)}")

    for i in range(min(2, e2e_steps)):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)                           # synchronous: returns after the D2H copy completed
    barrier()
    e2e_s = (time.perf_counter() - t0) / max(e2e_steps, 1) if e2e_steps else float("inf")
    te = torch.tensor([e2e_s], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_s = float(te.item())
    e2e_val = world * flops_step / e2e_s / 1e12
    h2d = 3 * bh * S * D * 2
    d2h = bh * S * D * 2 + bh * S * 4

    # ---- decode HBM roofline (rank-local; reported from rank 0)
    decode = None
    if not args.no_decode:
        decode = run_decode_bench(fa, torch, dev, stream, peaks, args)

    # ---- KV-sequence-sharded decode: one long cache split over the ranks (N > 1 only)
    kv_sharded = None
    if world > 1 and not args.no_decode:
        kv_sharded = run_kv_sharded_decode(fa, ge, torch, dist, dev, stream, rank, world, peaks, args)

    # ---- the other BASELINE configurations (short runs, reported beside the headline)
    other = None
    if not args.no_extra:
        other = run_other_configs(fa, torch, dev, stream, peaks, args.gqa_batch)

    status = fa.device_status()              # after every kernel of this run
    clocks = sampler.summary()
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cores = os.cpu_count() or 1
        kind, tf, dt = cpu_reference_run(bh, 1, 0, cores)
        cpu_baseline = {"value": tf, "unit": "TFLOP/s (causal FLOP count)", "cores": cores, "kind": kind,
                        "sample": f"all {bh} heads of the workload once ({dt:.2f} s wall)"}

    if rank == 0:
        line = {
            "metric": "causal prefill TFLOPS (B8 H12 S2048 D64 fp16)",
            "value": value, "unit": "TFLOP/s (causal FLOP count)",
            "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic: seeded iid N(0,1) rounded to fp16",
            "config": {"workload": "causal prefill fp16 B=8 H=12 S=2048 D=64 scale=1/8, per GPU",
                       "global_batch": B * world, "parallelism": f"(batch x head) sharding, dp{world}, no collective",
                       "l2": f"{n_sets} rotating input sets ({n_sets * 4 * bh * S * D * 2 // 2**20} MiB) > 126 MiB L2"},
            "tflops_refconv": world * refconv_flops(bh, S, D) / (ms_per_step * 1e-3) / 1e12,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["tflops"], "traffic": PREFILL_TRAFFIC_BYTES * (bh / 24.0),
                         "peak_source": peaks["source"],
                         "kernel": "prefill_kernel<D=64,causal,f16> (persistent, 1 CTA/SM)", "kernel_ms": kernel_ms,
                         "traffic_note": PREFILL_TRAFFIC_NOTE},
            "e2e": {"value": e2e_val, "unit": "TFLOP/s (causal FLOP count)", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_s * 1e3, "steps": e2e_steps},
            "gpu_launches": args.steps * repeats,
            "timing": {"repeats": repeats, "steps_per_repeat": args.steps, "reported": "median repeat",
                       "repeat_ms_per_step": [round(x / args.steps, 6) for x in rep_ms],
                       "ms_x_sm_mhz": (ms_per_step * clocks["sm_mhz"]) if clocks.get("sm_mhz") else None},
            "clocks": clocks,
            "device_status": status,
        }
        if args.shape:
            # a profiling shape, not the headline workload: say so in every label a reader sees
            what = (f"{'causal' if causal else 'non-causal'} prefill {dtype_name} B={B} H={H} S={S} D={D} "
                    f"(--shape, not the headline workload)")
            line["metric"] = what
            line["unit"] = line["e2e"]["unit"] = "TFLOP/s (causal FLOP count)" if causal else "TFLOP/s"
            line["dtype"] = dtype_name
            line["config"]["workload"] = what
            line["roofline"].update(kernel=f"16-bit prefill kernel, variant {args.variant}", traffic=None,
                                    traffic_note="not captured for this shape")
        if strong:
            line["strong_scaling_96_heads"] = strong
        if kv_sharded:
            line["kv_sharded_decode"] = kv_sharded
        if decode:
            line["decode"] = decode
        if other:
            line["other_configs"] = other
        if cpu_baseline:
            line["cpu_baseline"] = cpu_baseline
        if strong or kv_sharded:
            # repeated at the very end of the line: the correctness of the multi-GPU legs
            line["multi_gpu_parity"] = {
                "strong_scaling_max_abs_o": strong.get("max_abs_o") if strong else None,
                "strong_scaling_max_abs_lse": strong.get("max_abs_lse") if strong else None,
                "kv_sharded_max_abs_o": kv_sharded.get("max_abs_o") if kv_sharded else None,
                "kv_sharded_max_abs_lse": kv_sharded.get("max_abs_lse") if kv_sharded else None,
                "kv_sharded_ms_per_step": kv_sharded.get("ms_per_step") if kv_sharded else None,
                "tolerance": "o 2e-3, lse 1e-3 against the CPU oracle (src/demo.cu:28-70 restated)"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def check_heads_against_oracle(torch, dist, dev, tensors, heads, S, scale, world):
    """Outside any timed region: a few heads of this rank's last prefill against the CPU oracle on
    sampled rows; the maxima over all ranks are returned (the checker, not the product)."""
    from oracle import oracle
    q, k, v, o, lse = tensors
    rows = np.array([0, 1, 127, 128, 129, 1000, S - 1], np.int32)
    qf, kf, vf = (t[heads].float().cpu().numpy() for t in (q, k, v))
    o_ref, l_ref = oracle.attention(qf, kf, vf, scale, True, rows=rows)
    eo = float(np.abs(o[heads].float().cpu().numpy()[:, rows] - o_ref).max())
    el = float(np.abs(lse[heads].cpu().numpy()[:, rows] - l_ref).max())
    t = torch.tensor([eo, el], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"max_abs_o": float(t[0].item()), "max_abs_lse": float(t[1].item()),
            "checked": f"heads {heads} of every rank, rows {rows.tolist()}, against the CPU oracle"}


def run_kv_sharded_decode(fa, ge, torch, dist, dev, stream, rank, world, peaks, args):
    """B=1 H=32 Skv=131072 D=128 fp16: each rank owns Skv/world keys, decodes its slice,
    one NCCL all-gather of [H, D+1] fp32 per rank, fa_combine on every rank."""
    sh = ge.load_module("sharding")
    H, SKV, D = 32, 131072, 128
    k0, kc = sh.kv_shard(SKV, rank, world)
    gen = torch.Generator(device=dev)
    gen.manual_seed(5005 + rank)
    k = torch.randn((H, kc, D), device=dev, dtype=torch.float32, generator=gen).to(torch.float16)
    v = torch.randn((H, kc, D), device=dev, dtype=torch.float32, generator=gen).to(torch.float16)
    gq = torch.Generator(device=dev)
    gq.manual_seed(5004)
    q = torch.randn((H, D), device=dev, dtype=torch.float32, generator=gq).to(torch.float16)
    o = torch.empty((H, D), device=dev, dtype=torch.float16)
    lse = torch.empty((H,), device=dev, dtype=torch.float32)
    run = sh.ShardedDecode(fa, 1, H, D, kc, dtype="f16", num_splits=16)
    scale = float(1.0 / np.sqrt(D))
    # parity, outside the timed region: rank 0 regenerates every rank's key slice for a few heads
    # (same seeded generators) and checks its merged result against the CPU oracle on the whole cache
    run(q, k, v, o, lse, scale, stream)
    torch.cuda.synchronize()
    parity = {}
    if rank == 0:
        from oracle import oracle
        heads = [0, 13, H - 1]
        ks, vs = [], []
        for r in range(world):
            _, kcr = sh.kv_shard(SKV, r, world)
            g_r = torch.Generator(device=dev)
            g_r.manual_seed(5005 + r)
            kr = torch.randn((H, kcr, D), device=dev, dtype=torch.float32, generator=g_r).to(torch.float16)
            vr = torch.randn((H, kcr, D), device=dev, dtype=torch.float32, generator=g_r).to(torch.float16)
            ks.append(kr[heads].float().cpu().numpy())
            vs.append(vr[heads].float().cpu().numpy())
            del kr, vr
        o_ref, l_ref = oracle.attention(q[heads].float().cpu().numpy()[:, None], np.concatenate(ks, 1),
                                        np.concatenate(vs, 1), scale, False)
        parity = {"max_abs_o": float(np.abs(o[heads].float().cpu().numpy() - o_ref[:, 0]).max()),
                  "max_abs_lse": float(np.abs(lse[heads].cpu().numpy() - l_ref[:, 0]).max()),
                  "checked": f"heads {heads} on rank 0 against the CPU oracle over all {SKV} keys"}
    steps = max(5, min(args.steps, 50))
    for _ in range(5):
        run(q, k, v, o, lse, scale, stream)
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        run(q, k, v, o, lse, scale, stream)
    e1.record(stream)
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    total_bytes = 2 * H * SKV * D * 2
    run.close()
    return {"workload": f"decode fp16 B=1 H={H} Skv={SKV} D={D}, keys sharded over {world} GPUs "
                        f"({kc} per GPU), in-place all-gather of {H * (D + 1) * 4} B per rank + packed merge "
                        f"(fa_decode_kv_sharded)",
            "ms_per_step": ms, "launches_per_step": run.LAUNCHES_PER_STEP, **parity,
            "aggregate_GBps": total_bytes / (ms * 1e-3) / 1e9,
            "per_gpu_frac_of_hbm_peak": total_bytes / world / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "note": "latency-bound: per-GPU traffic is tens of microseconds, the step is dominated by "
                    "launches and the all-gather round trip", "scaling": "strong"}


def run_other_configs(fa, torch, dev, stream, peaks, gqa_batch=0):
    """Config 3 (bf16 B1 H32 S8192 D128, causal and not) and config 5 (e4m3 B8 H16 S4096 D128
    causal): device-resident, 3 warm-up + 30 timed launches each, inputs 0.2-0.3 GB (> L2)."""
    out = {}

    gen = torch.Generator(device=dev)
    gen.manual_seed(6006)

    def randn(shape):
        return torch.randn(shape, device=dev, dtype=torch.float32, generator=gen)

    def timed(fn, steps=30):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    bh, s, d = 32, 8192, 128
    scale = float(1.0 / np.sqrt(d))
    q, k, v = (randn((bh, s, d)).to(torch.bfloat16) for _ in range(3))
    o = torch.empty_like(q)
    lse = torch.empty((bh, s), device=dev, dtype=torch.float32)
    for causal in (True, False):
        ms = timed(lambda: fa.prefill(q, k, v, o, lse, 1, bh, s, d, scale, causal, dtype="bf16", stream=stream))
        flops = causal_flops(bh, s, d) if causal else refconv_flops(bh, s, d)
        tf = flops / (ms * 1e-3) / 1e12
        out["bf16_b1_h32_s8192_d128_" + ("causal" if causal else "noncausal")] = {
            "ms": ms, "tflops": tf, "frac_of_measured_bf16_peak": tf / peaks["tflops"]}
    del q, k, v, o, lse

    bh, s, d = 128, 4096, 128
    q8, k8, v8 = (randn((bh, s, d)).to(torch.float8_e4m3fn).view(torch.uint8)
                  for _ in range(3))
    sc = torch.full((bh,), 0.01, device=dev, dtype=torch.float32)
    o = torch.empty((bh, s, d), device=dev, dtype=torch.bfloat16)
    lse = torch.empty((bh, s), device=dev, dtype=torch.float32)
    ms = timed(lambda: fa.prefill(q8, k8, v8, o, lse, 8, 16, s, d, scale, True, dtype="e4m3", q_scale=sc,
                                  k_scale=sc, v_scale=sc, stream=stream))
    tf = causal_flops(bh, s, d) / (ms * 1e-3) / 1e12
    out["e4m3_b8_h16_s4096_d128_causal"] = {"ms": ms, "tflops": tf,
                                            "frac_of_measured_bf16_peak": tf / peaks["tflops"],
                                            "note": "Q K^T on the 8-bit kind, P V on the 16-bit kind from an fp16 copy of V made by a pre-pass inside the call"}
    del q8, k8, v8, o, lse

    # backward pass (dQ, dK, dV) on config 2's shape; 2.5x the forward's FLOP (5 products against 2)
    bh, s, d = CFG["B"] * CFG["H"], CFG["S"], CFG["D"]
    sc_b = float(1.0 / np.sqrt(d))
    qb, kb_, vb, dob = (randn((bh, s, d)).to(torch.float16) for _ in range(4))
    ob = torch.empty_like(qb)
    lb = torch.empty((bh, s), device=dev, dtype=torch.float32)
    fa.prefill(qb, kb_, vb, ob, lb, 1, bh, s, d, sc_b, True, dtype="f16", stream=stream)
    gq, gk, gv = (torch.empty_like(qb) for _ in range(3))
    wsb = fa.backward_workspace_bytes(1, bh, s)
    wsbk = torch.empty(wsb, device=dev, dtype=torch.uint8)
    ms = timed(lambda: fa.backward(qb, kb_, vb, ob, dob, lb, gq, gk, gv, 1, bh, s, d, sc_b, True, dtype="f16",
                                   workspace=wsbk, workspace_bytes=wsb, stream=stream))
    tf = 2.5 * causal_flops(bh, s, d) / (ms * 1e-3) / 1e12
    out[f"backward_f16_b{CFG['B']}_h{CFG['H']}_s{s}_d{d}_causal"] = {
        "ms": ms, "tflops": tf, "frac_of_measured_bf16_peak": tf / peaks["tflops"],
        "note": "delta + dK/dV kernel + dQ kernel; FLOP counted as 2.5 x the causal forward"}
    del qb, kb_, vb, dob, ob, lb, gq, gk, gv

    # grouped-query decode over a [B, Skv, Hkv, D] cache: the group's query heads ride in the rows of
    # the tensor-core query tile, K and V stream once per KV head (HBM-bound: report GB/s)
    gb = gqa_batch or 32
    for (b, hq, hkv, skv, d) in ((gb, 32, 8, 16384, 128), (gb, 32, 1, 32768, 128)):
        kc = randn((b, skv, hkv, d)).to(torch.float16)
        vc = randn((b, skv, hkv, d)).to(torch.float16)
        qg = randn((b, hq, d)).to(torch.float16)
        og = torch.empty_like(qg)
        lg = torch.empty((b, hq), device=dev, dtype=torch.float32)
        splits = fa.decode_gqa_default_splits(b, hkv, skv)
        wsb = fa.decode_workspace_bytes(b, hq, d, splits)
        ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
        sc_g = float(1.0 / np.sqrt(d))
        ms = timed(lambda: fa.decode_gqa(qg, kc, vc, og, lg, b, hq, hkv, skv, d, sc_g, dtype="f16",
                                         kv_strides=(skv * hkv * d, d, hkv * d), workspace=ws,
                                         workspace_bytes=wsb, stream=stream))
        algo = 2 * b * hkv * skv * d * 2 + 2 * b * hq * d * 2
        gbs = algo / (ms * 1e-3) / 1e9
        out[f"gqa_decode_f16_b{b}_hq{hq}_hkv{hkv}_skv{skv}_d{d}"] = {
            "ms": ms, "GBps": gbs, "frac_of_measured_hbm_peak": gbs / peaks["hbm_gbs"], "splits": splits,
            "algorithmic_bytes": algo, "tokens_per_s": b / (ms * 1e-3)}
        del kc, vc, ws

    # the same entry point with several query tokens per sequence: a whole causal GQA prefill as one
    # chunk (tensor-bound: TFLOP/s on the causal count), and 4 speculative tokens per sequence (HBM-bound)
    for (b, hq, hkv, skv, d, t) in ((8, 32, 8, 2048, 128, 2048), (gb, 32, 8, 16384, 128, 4)):
        kc = randn((b, skv, hkv, d)).to(torch.float16)
        vc = randn((b, skv, hkv, d)).to(torch.float16)
        qg = randn((b, t, hq, d)).to(torch.float16)
        og = torch.empty_like(qg)
        lg = torch.empty((b, t, hq), device=dev, dtype=torch.float32)
        tpt = min(t, 128 // (hq // hkv))
        splits = fa.decode_gqa_default_splits(b * (-(-t // tpt)), hkv, skv)
        wsb = fa.decode_workspace_bytes(b, t * hq, d, splits)
        ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
        sc_g = float(1.0 / np.sqrt(d))
        ms = timed(lambda: fa.decode_gqa(qg, kc, vc, og, lg, b, hq, hkv, skv, d, sc_g, dtype="f16", num_q_tokens=t,
                                         num_splits=splits, kv_strides=(skv * hkv * d, d, hkv * d), workspace=ws,
                                         workspace_bytes=wsb, stream=stream))
        keys = sum(skv - t + i + 1 for i in range(t))
        tf = 4.0 * d * b * hq * keys / (ms * 1e-3) / 1e12
        algo = 2 * b * hkv * skv * d * 2 + 2 * b * t * hq * d * 2
        out[f"chunk_f16_b{b}_hq{hq}_hkv{hkv}_skv{skv}_d{d}_t{t}"] = {
            "ms": ms, "tflops": tf, "GBps_cache": algo / (ms * 1e-3) / 1e9, "splits": splits,
            "note": "fa_decode_gqa with num_q_tokens = t, causal among the new tokens"}
        del kc, vc, ws

    # the same decode over an e4m3 cache (one byte per element; Q e4m3 as well, per-(batch, KV head) scales)
    b, hq, hkv, skv, d = gb, 32, 8, 16384, 128
    kc8 = randn((b, skv, hkv, d)).to(torch.float8_e4m3fn).view(torch.uint8)
    vc8 = randn((b, skv, hkv, d)).to(torch.float8_e4m3fn).view(torch.uint8)
    q8g = randn((b, hq, d)).to(torch.float8_e4m3fn).view(torch.uint8)
    sc8 = torch.full((b * hkv,), 0.01, device=dev, dtype=torch.float32)
    og = torch.empty((b, hq, d), device=dev, dtype=torch.bfloat16)
    lg = torch.empty((b, hq), device=dev, dtype=torch.float32)
    splits = fa.decode_gqa_default_splits(b, hkv, skv)
    wsb = fa.decode_workspace_bytes(b, hq, d, splits)
    ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
    ms = timed(lambda: fa.decode_gqa(q8g, kc8, vc8, og, lg, b, hq, hkv, skv, d, float(1.0 / np.sqrt(d)), dtype="e4m3",
                                     kv_strides=(skv * hkv * d, d, hkv * d), q_scale=sc8, k_scale=sc8, v_scale=sc8,
                                     workspace=ws, workspace_bytes=wsb, stream=stream))
    algo = 2 * b * hkv * skv * d + b * hq * d + b * hq * d * 2
    gbs = algo / (ms * 1e-3) / 1e9
    out[f"gqa_decode_e4m3_b{b}_hq{hq}_hkv{hkv}_skv{skv}_d{d}"] = {
        "ms": ms, "GBps": gbs, "frac_of_measured_hbm_peak": gbs / peaks["hbm_gbs"], "splits": splits,
        "algorithmic_bytes": algo, "tokens_per_s": b / (ms * 1e-3)}
    del kc8, vc8, ws
    return out


def run_decode_bench(fa, torch, dev, stream, peaks, args):
    B, H, SKV, D, SPLITS = DEC["B"], DEC["H"], DEC["SKV"], DEC["D"], DEC["SPLITS"]
    bh = B * H
    k = torch.empty((bh, SKV, D), device=dev, dtype=torch.float16)
    v = torch.empty((bh, SKV, D), device=dev, dtype=torch.float16)
    gen = torch.Generator(device=dev)
    gen.manual_seed(4004)
    for t in (k, v):                          # fill in slabs to bound temporary memory
        for i in range(0, bh, 64):
            t[i:i + 64] = torch.randn((min(64, bh - i), SKV, D), device=dev, dtype=torch.float32,
                                      generator=gen).to(torch.float16)
    q = torch.randn((bh, D), device=dev, dtype=torch.float32, generator=gen).to(torch.float16)
    o = torch.empty((bh, D), device=dev, dtype=torch.float16)
    lse = torch.empty((bh,), device=dev, dtype=torch.float32)
    wsb = fa.decode_workspace_bytes(B, H, D, SPLITS)
    ws = torch.empty(wsb, device=dev, dtype=torch.uint8)
    scale = float(1.0 / np.sqrt(D))

    def step():
        fa.decode(q, k, v, o, lse, None, B, H, SKV, D, scale, dtype="f16", num_splits=SPLITS,
                  workspace=ws, workspace_bytes=wsb, stream=stream)

    steps = max(5, min(args.steps, 30))
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    algo_bytes = 2 * bh * SKV * D * 2 + 2 * bh * D * 2
    gbs = algo_bytes / (ms * 1e-3) / 1e9
    del k, v
    return {"workload": f"split-KV decode fp16 B={B} H={H} Skv={SKV} D={D}, {SPLITS} splits + combine",
            "ms_per_step": ms, "tokens_per_s": B / (ms * 1e-3), "steps": steps,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": DECODE_TRAFFIC_BYTES * (bh / 128.0),
                         "peak_source": peaks["source"],
                         "algorithmic_bytes": algo_bytes,
                         "note": "K+V (8.59 GB) exceed L2; both kernels (partial + combine) inside the timed step"}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the long-context and FP8 configurations")
    ap.add_argument("--batch", type=int, default=0,
                    help="profiling only: override the prefill batch (the line is then not the headline)")
    ap.add_argument("--decode-batch", type=int, default=0,
                    help="profiling only: override the decode batch")
    ap.add_argument("--gqa-batch", type=int, default=0,
                    help="profiling only: override the batch of the grouped-query decode cases")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--variant", default="auto", choices=["auto", "one_tile", "tile_pair", "cta_pair"],
                    help="profiling only: force one of the 16-bit prefill kernels")
    ap.add_argument("--shape", default="",
                    help="profiling only: B,H,S,D,causal(0/1),dtype(f16/bf16) instead of the headline workload "
                         "(the line is then not the headline)")
    args = ap.parse_args()
    if args.batch:
        CFG["B"] = args.batch
    if args.shape:
        b, h, sq, d, c, dt = args.shape.split(",")
        CFG.update(B=int(b), H=int(h), S=int(sq), D=int(d), CAUSAL=bool(int(c)), DTYPE=dt)
    if args.decode_batch:
        DEC["B"] = args.decode_batch
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    run_b200_arm(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
