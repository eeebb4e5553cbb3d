#!/usr/bin/env python
"""Benchmark of the attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--profile-case NAME]

Prints ONE JSON line.  The default workload is the MTP-verify decode the headline metric is quoted
on (batch 1, 2 causal query tokens, 20 heads x 576 f16, 32768-row f16 latent cache, V = first 512
columns, scale 1/16).  A step is one pass of the hot path over that input: the attention kernel
plus the combine kernel, called through the C ABI.  Inputs are synthetic (device RNG, N(0,1)
queries, N(0,0.5) cache).

  value     algorithmic bytes per step / device time per step, inputs resident in HBM; between
            steps the call rotates over distinct cache copies totalling more than twice L2.
  e2e       the same metric through the call-site mirror (MlaDecodeLayer.step): pinned host q and
            new latent rows are copied in, appended with RoPE, attended, and the output is copied
            back to the host, every step (one recorded CUDA graph of three kernels per layer,
            replayed; the kernels read the page-locked inputs and write the page-locked output in
            place).  The latent cache is persistent layer state and stays in HBM, as in the engine.
  roofline  the attention kernel alone (the same graph replay with the combine kernel skipped),
            against the measured HBM copy bandwidth.
  --impl reference   times the CPU restatement of the reference's attention semantics (the test
            oracle) on the host cores; the reference has no CPU implementation of this path and
            its CUDA kernel rejects these shapes (R != 512 or H % 16 != 0).

  others    the remaining configurations: the 128K-row decode, the paged 64-sequence batch, the 8192-token
            prefill, the reference kernel's twin shapes (R = 512, 32 and 64 heads), and the engine's own sparse
            decode shape through the reference's entry point gs_mla_attn (CUDA-core kernel and tensor-core path).

With --gpus N > 1 (launched by torchrun) every rank runs its own independent copy of the workload
(sequences are independent units: weak scaling, no collective on the data path); the "others"
object carries the 128K-context decode sharded by sequence over the N GPUs, the paged 64-sequence
batch and the 8192-token prefill.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, D_QK, D_V = 20, 576, 512
SCALE = 1.0 / 16.0
L2_BYTES = 126 * 1024 * 1024


def algorithmic_bytes(n_rows: int, T: int, n_seq: int = 1) -> int:
    """Cache rows read once + queries + f32 outputs (the per-call figure of the measurement plan)."""
    return n_rows * D_QK * 2 + n_seq * T * H * D_QK * 2 + n_seq * T * H * D_V * 4


def measured_peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed regions run."""

    def __init__(self, index: int):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _names(self, mask: int) -> list[str]:
        nv = self.nv
        table = {
            "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap, "hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
            "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
            "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
            "hw_power_brake": nv.nvmlClocksEventReasonHwPowerBrakeSlowdown,
            "applications_clocks": nv.nvmlClocksEventReasonApplicationsClocksSetting,
        }
        return [k for k, bit in table.items() if mask & bit]

    def sample(self):
        if self.nv is None:
            return
        try:
            self.samples.append(int(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)))
            self.reasons.update(self._names(int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))))
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self.sample()
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self) -> dict | None:
        if self.nv is None:
            return None
        self._stop.set()
        if self._thread:
            self._thread.join()
        self.sample()
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------------
# reference arm: the CPU restatement on the host cores
# ---------------------------------------------------------------------------------------------------

def cpu_decode_baseline(n_rows: int, T: int, budget_s: float, max_reps: int = 50) -> dict:
    """Times the oracle (all host threads) on the decode workload; returns GB/s of algorithmic bytes."""
    import numpy as np
    from oracle import oracle_py as O
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, T, H, D_QK), dtype=np.float32).astype(np.float16)
    cache = (rng.standard_normal((n_rows, D_QK), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
    ks = cpu_key_splits(T)
    _, used = O.mla_decode(q, cache, [n_rows], SCALE, return_threads=True, key_splits=ks)  # warm-up, page in
    t0 = time.perf_counter()
    reps = 0
    while reps < max_reps and (time.perf_counter() - t0 < budget_s or reps == 0):
        O.mla_decode(q, cache, [n_rows], SCALE, key_splits=ks)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": algorithmic_bytes(n_rows, T) / dt / 1e9, "unit": "GB/s", "cores": int(used), "kind": "port",
            "sample": f"full workload ({n_rows} rows, T={T}, H={H}), {reps} passes, {dt * 1e3:.1f} ms each; "
                      f"{ks} work items = key ranges, each over all {T * H} (token, head) rows",
            "seconds_per_pass": dt}


def cpu_key_splits(T: int) -> int:
    """Key ranges of the CPU arm: one work item per range (all query rows over it, the range read from memory once),
    eight items per host core and ranges short enough to stay in a core's cache."""
    from oracle import oracle_py as O
    return max(8 * O.host_cores(), 32768 // 256)


WORKLOAD = "mtp_verify_32k: batch 1, T=2 causal, H=20, d_qk=576, d_v=512, ctx=32768, scale=1/16"


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle_py as O
    n_rows, T = 32768, 2
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, T, H, D_QK), dtype=np.float32).astype(np.float16)
    cache = (rng.standard_normal((n_rows, D_QK), dtype=np.float32) * np.float32(0.5)).astype(np.float16)
    ks = cpu_key_splits(T)
    _, used = O.mla_decode(q, cache, [n_rows], SCALE, return_threads=True, key_splits=ks)
    t0 = time.perf_counter()
    O.mla_decode(q, cache, [n_rows], SCALE, key_splits=ks)
    t_full = time.perf_counter() - t0
    # bound the whole run to about two minutes: shorten each step to a prefix of the cache if needed
    total = (args.steps + args.warmup) * t_full
    rows = n_rows if total <= 120.0 else max(1024, int(n_rows * 120.0 / total) // 64 * 64)
    for _ in range(args.warmup):
        O.mla_decode(q, cache[:rows], [rows], SCALE, key_splits=ks)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.mla_decode(q, cache[:rows], [rows], SCALE, key_splits=ks)
    dt = (time.perf_counter() - t0) / max(1, args.steps)
    val = algorithmic_bytes(rows, T) / dt / 1e9
    sample = f"{rows} of {n_rows} cache rows per step" if rows != n_rows else "full workload per step"
    sample += f"; {ks} work items = key ranges, each over all {T * H} (token, head) rows"
    line = {
        "impl": "reference", "metric": "MLA decode-attention HBM GB/s (MTP verify, 32K ctx)", "value": val,
        "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 in / f32 accumulate",
        "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": int(used), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU restatement (oracle port) of the reference's attention semantics on the host cores; the "
                "reference has no CPU implementation of this path",
    }
    twin = reference_cuda_twin()
    if twin is not None:
        line["reference_cuda_twin"] = twin
    print(json.dumps(line), flush=True)


def reference_cuda_twin():
    """The reference's own CUDA kernel (gs_mla_attn, compiled unmodified for sm_100a) on the twin
    shapes it accepts: R = 512 (V = all 512 columns), H = 32, f32 queries, identity position list,
    the engine's split policy (16 for T = 1, 4 for T = 2).  Returns None without a GPU or the library."""
    so = os.path.join(ROOT, "oracle", "_ref", "libglmssd_ref.so")
    try:
        import ctypes as C
        import torch
        if not (os.path.exists(so) and torch.cuda.is_available()):
            return None
        ref = C.CDLL(so)
        vp, i32, f32 = C.c_void_p, C.c_int, C.c_float
        ref.gs_mla_attn.restype = i32
        ref.gs_mla_attn.argtypes = [vp, vp, vp, vp, i32, vp, f32, vp, vp, i32, i32, i32, i32, vp]
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(0)
        out = {}
        for name, n, T, Hh, splits in (("ctx32k_T2_H32", 32768, 2, 32, 4), ("ctx32k_T1_H32", 32768, 1, 32, 16),
                                       ("ctx128k_T1_H32", 131072, 1, 32, 16), ("ctx32k_T1_H64", 32768, 1, 64, 16),
                                       ("ctx4k_T1_H32", 4096, 1, 32, 16)):
            n_copies = max(2, -(-2 * L2_BYTES // (n * 1024)) + 1)
            caches = [(torch.randn((n, 512), device=dev) * 0.5).half() for _ in range(n_copies)]
            q = torch.randn((T, Hh, 512), device=dev, dtype=torch.float32)
            sel = torch.arange(n, dtype=torch.int32, device=dev).repeat(T, 1).contiguous()
            cnt = torch.tensor([n - (T - 1 - t) for t in range(T)], dtype=torch.int32, device=dev)
            o = torch.empty((T, Hh, 512), dtype=torch.float32, device=dev)
            sweep = (8, 32, 64, 128, 256)  # besides the engine's own choice: the reference kernel at its best split count
            part = torch.empty(T * (Hh // 16) * max(sweep) * (16 * 512 + 32), dtype=torch.float32, device=dev)
            st = torch.cuda.current_stream().cuda_stream

            def timed(sp, reps):
                def call(i):
                    rc = ref.gs_mla_attn(q.data_ptr(), caches[i % n_copies].data_ptr(), None, sel.data_ptr(), n, cnt.data_ptr(),
                                         SCALE, o.data_ptr(), part.data_ptr(), T, Hh, 512, sp, st)
                    assert rc == 0, rc

                for i in range(3):
                    call(i)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for i in range(reps):
                    call(i)
                e1.record()
                torch.cuda.synchronize()
                return e0.elapsed_time(e1) * 1e3 / reps

            us = timed(splits, 4 * n_copies)
            out[name] = {"us_per_call": us, "GB/s": n * 1024 / us / 1e3, "splits": splits}
            best = min(((timed(sp, 2 * n_copies), sp) for sp in sweep), default=None)
            if best is not None and best[0] < us:
                out[name]["best_of_splits"] = {"us_per_call": best[0], "GB/s": n * 1024 / best[0] / 1e3, "splits": best[1]}
            del caches
        out.update(_paged_twin(torch, dev, ref.gs_mla_attn))
        out.update(_sparse_list_shape(torch, dev, ref.gs_mla_attn, "reference_kernel"))
        return out
    except Exception as exc:
        return {"error": f"{type(exc).__name__}: {exc}"}


def _paged_twin(torch, dev, ref_fn):
    """The 64-sequence paged batch on the reference kernel: 64 query rows (one per sequence, T = 64 in its terms) whose
    position lists are the sequences' page tables written out row by row (ops.cu:455); R = 512, H = 32.  Timed at
    the engine's split count for T > 2 (1, forward.rs:901) and at the best of a sweep; the new kernel on the same pool,
    page table and head count beside it."""
    import numpy as np
    pkg = importlib.import_module("glm-ssd_b200")
    rng = np.random.default_rng(5)
    lens = rng.integers(1024, 65537, size=64)
    pages_per = -(-lens // 64)
    n_pages = int(pages_per.sum()) + 4
    perm = rng.permutation(n_pages)
    stride = int(pages_per.max()) * 64
    pt = np.zeros((64, int(pages_per.max())), np.int32)
    sel = np.zeros((64, stride), np.int32)
    k = 0
    for b in range(64):
        pages = perm[k:k + pages_per[b]]
        pt[b, :pages_per[b]] = pages
        sel[b, :pages_per[b] * 64] = (pages[:, None] * 64 + np.arange(64)[None, :]).reshape(-1)
        k += int(pages_per[b])
    Hh = 32
    pool = (torch.randn((n_pages * 64, 512), device=dev) * 0.5).half()
    q = torch.randn((64, Hh, 512), device=dev, dtype=torch.float32)
    sel_d, cnt_d = torch.from_numpy(sel).to(dev), torch.from_numpy(lens.astype(np.int32)).to(dev)
    o = torch.empty((64, Hh, 512), dtype=torch.float32, device=dev)
    sweep = (1, 4, 16)
    part = torch.empty(64 * (Hh // 16) * max(sweep) * (16 * 512 + 32), dtype=torch.float32, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    tot = int(lens.sum()) * 1024
    res = {}

    def timed(call, reps):
        call()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            call()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    def ref_call(sp):
        rc = ref_fn(q.data_ptr(), pool.data_ptr(), None, sel_d.data_ptr(), stride, cnt_d.data_ptr(), SCALE, o.data_ptr(),
                    part.data_ptr(), 64, Hh, 512, sp, st)
        assert rc == 0, rc

    runs = {sp: timed(lambda sp=sp: ref_call(sp), 2) for sp in sweep}
    best = min(runs, key=runs.get)
    res["paged64_H32_reference_kernel"] = {"us_per_call": runs[1], "GB/s": tot / runs[1] / 1e3, "splits": 1,
                                           "best_of_splits": {"us_per_call": runs[best], "splits": best}}
    o_ref = o.clone()
    # the new kernel: same pool, page table and lengths, f16 queries (the rounding the reference applies to nothing)
    qh = q.half().view(64, 1, Hh, 512).contiguous()
    ptd = torch.from_numpy(pt).to(dev)
    ob = torch.empty((64, 1, Hh, 512), dtype=torch.float32, device=dev)
    ws = pkg.new_workspace(64, 1, Hh, 512, dev)
    ours = timed(lambda: pkg.mla_decode(qh, pool, cnt_d, page_table=ptd, out=ob, workspace=ws, d_v=512, max_seq_len=int(lens.max())), 10)
    ref_call(best)
    torch.cuda.synchronize()
    res["paged64_H32_new_kernel"] = {"us_per_call": ours, "GB/s": tot / ours / 1e3,
                                     "max_abs_vs_reference_kernel": float((ob.view(64, Hh, 512) - o).abs().max()),
                                     "reference_kernel_split_counts_agree": float((o - o_ref).abs().max())}
    del pool, sel_d
    torch.cuda.empty_cache()
    return res


def _sparse_list_shape(torch, dev, fn, label, profile=False, q8=False):
    """The engine's own decode shape: 64 heads, f32 queries, a sparse list of 2052 positions per query token
    out of a 32768-row cache (forward.rs:461, :873), through the reference's entry point gs_mla_attn."""
    res = {}
    ctx, n, Hh = 32768, 2052, 64
    caches = [(torch.randn((ctx, 512), device=dev) * 0.5).half() for _ in range(6)]
    scales = [None] * 6
    if q8:  # the reference's Q8 cache (ops.cu:599-610): int8 rows and one f16 scale per 32 values, quantised on the device
        pkg = importlib.import_module("glm-ssd_b200")
        q8c, q8s = [], []
        for c in caches:
            qq = torch.empty((ctx, 512), dtype=torch.int8, device=dev)
            dd = torch.empty((ctx, 16), dtype=torch.float16, device=dev)
            pkg.quant_q8_rows(c.float().contiguous(), qq, dd, ctx * 512)
            q8c.append(qq)
            q8s.append(dd)
        torch.cuda.synchronize()
        caches, scales = q8c, q8s
    st = torch.cuda.current_stream().cuda_stream
    for T, splits in ((1, 16), (2, 4), (256, 1)):  # decode, MTP verify, a prefill chunk (forward.rs:898-901)
        q = torch.randn((T, Hh, 512), device=dev, dtype=torch.float32)
        sel = torch.stack([torch.randperm(ctx, device=dev)[:n].sort().values for _ in range(T)]).int().contiguous()
        cnt = torch.full((T,), n, dtype=torch.int32, device=dev)
        o = torch.empty((T, Hh, 512), dtype=torch.float32, device=dev)
        part = torch.empty(T * Hh * splits * 514, dtype=torch.float32, device=dev)  # the reference's size (ops.cu:578)

        def call(i):
            rc = fn(q.data_ptr(), caches[i % 6].data_ptr(), None if scales[i % 6] is None else scales[i % 6].data_ptr(), sel.data_ptr(), n,
                    cnt.data_ptr(), SCALE, o.data_ptr(),
                    part.data_ptr(), T, Hh, 512, splits, st)
            assert rc == 0, rc

        for i in range(3):
            call(i)
        torch.cuda.synchronize()
        if profile:  # a few eager launches per shape are all a profiler needs
            continue
        # one pass over the cache copies captured in a CUDA graph and replayed: the device's time, not the caller's launch rate
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            st = side.cuda_stream
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(6):
                    call(i)
        torch.cuda.current_stream().wait_stream(side)
        st = torch.cuda.current_stream().cuda_stream
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_replays = 5 if T <= 4 else 2
        reps = 6 * n_replays
        e0.record()
        for _ in range(n_replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        res[f"sparse2052_T{T}_H64_{label}"] = {"us_per_call": e0.elapsed_time(e1) * 1e3 / reps, "splits": splits}
    return res


# ---------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------

def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    pkg = importlib.import_module("glm-ssd_b200")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    peaks, peak_kind = measured_peaks()
    hbm_peak = float(peaks["hbm_gbs"])
    tf_peak = float(peaks.get("bf16_tflops", 1590.0))
    tf_sustained = float(peaks.get("bf16_tflops_sustained", 1400.0))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    gen = torch.Generator(device=dev)
    gen.manual_seed(1234 + rank)

    def randn_f16(shape, sigma=1.0):
        out = torch.empty(shape, dtype=torch.float16, device=dev)
        # chunked so the f32 temporary stays small
        flat = out.view(-1)
        step = 1 << 26
        for i in range(0, flat.numel(), step):
            n = min(step, flat.numel() - i)
            flat[i:i + n] = (torch.randn(n, generator=gen, device=dev, dtype=torch.float32) * sigma).to(torch.float16)
        return out

    def time_loop(fn, steps, warmup, period=1, use_graph=True, repeats=1, spread=None):
        """Device time of `steps` calls of fn(i) after `warmup` calls: barrier + sync on both sides,
        CUDA events on the launching stream, max over ranks.  Returns seconds per step.  With
        `repeats` > 1 the timed region (the same `steps` calls, bracketed the same way) is run that many
        times and the median is returned; `spread` receives min / median / max and the region's length.

        `period` consecutive calls (one pass over the rotating buffers) are captured once into a CUDA
        graph and replayed, so the figure is the device's, not the Python caller's launch rate."""
        for i in range(min(warmup, 3)):
            fn(i)
        torch.cuda.synchronize()
        graph = rem_graph = None
        rem = steps % period if steps >= period else 0
        if steps < period:
            period, rem = steps, 0

        def capture(n_calls, first):
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    for i in range(n_calls):
                        fn(first + i)
            torch.cuda.current_stream().wait_stream(side)
            return g

        if use_graph:
            try:
                graph = capture(period, 0)
                if rem:
                    rem_graph = capture(rem, 0)  # the last `rem` of exactly `steps` timed calls
            except Exception:
                graph = rem_graph = None
                torch.cuda.synchronize()
        if graph is None:
            n_steps = steps

            def run_timed():
                for i in range(steps):
                    fn(warmup + i)

            for i in range(warmup):
                fn(i)
        else:
            n_full = steps // period
            n_steps = n_full * period + rem  # == steps

            def run_timed():
                for _ in range(n_full):
                    graph.replay()
                if rem_graph is not None:
                    rem_graph.replay()

            for _ in range(max(1, -(-warmup // period))):
                graph.replay()
            if rem_graph is not None:
                rem_graph.replay()
        per_step = []
        for _ in range(max(1, repeats)):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run_timed()
            e1.record()
            barrier()
            per_step.append(max_over_ranks(e0.elapsed_time(e1) * 1e-3) / n_steps)
        med = statistics.median(per_step)
        if spread is not None:
            spread.update({"repeats": len(per_step), "steps_per_repeat": n_steps, "us_min": min(per_step) * 1e6,
                           "us_median": med * 1e6, "us_max": max(per_step) * 1e6,
                           "timed_region_ms": med * n_steps * 1e3})
        return med

    sampler = ClockSampler(local_rank)

    # ---- headline workload: MTP verify, T = 2, 32768 rows -------------------------------------------
    n_rows, T = 32768, 2
    bytes_step = algorithmic_bytes(n_rows, T)
    n_copies = max(2, -(-2 * L2_BYTES // (n_rows * D_QK * 2)) + 1)  # total > 2 x L2
    caches = [randn_f16((n_rows, D_QK), 0.5) for _ in range(n_copies)]
    q = randn_f16((1, T, H, D_QK))
    seq_len = torch.tensor([n_rows], dtype=torch.int32, device=dev)
    out = torch.empty((1, T, H, D_V), dtype=torch.float32, device=dev)
    ws = pkg.new_workspace(1, T, H, D_V, dev)

    def step(i, ev=None):
        pkg.mla_decode(q, caches[i % n_copies], seq_len, out=out, workspace=ws, max_seq_len=n_rows, ev_after_main=ev)

    sampler.start()
    spread = {}
    sec = time_loop(step, args.steps, args.warmup, period=n_copies, repeats=args.repeats, spread=spread)
    value = world * bytes_step / sec / 1e9

    # ---- roofline pass: the attention kernel alone (combine skipped), same rotation, same graph replay ----
    def step_kernel_only(i):
        pkg.mla_decode(q, caches[i % n_copies], seq_len, out=out, workspace=ws, max_seq_len=n_rows, no_combine=True)

    kern_sec = time_loop(step_kernel_only, min(args.steps, 2000), args.warmup, period=n_copies, repeats=args.repeats)
    achieved = bytes_step / kern_sec / 1e9
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        try:
            with open(tpath) as f:
                traffic = json.load(f).get("mtp_verify_32k_dram_bytes_per_launch")
        except Exception:
            traffic = None
    roofline = {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "traffic": traffic, "peak_kind": peak_kind, "kernel": "k_decode_umma (combine kernel excluded; back-to-back launches in a CUDA graph)",
                "kernel_us": kern_sec * 1e6, "algorithmic_bytes_per_launch": bytes_step}

    # ---- e2e: host buffers through the call-site mirror ---------------------------------------------
    n_layers = n_copies
    layers = []
    for j in range(n_layers):
        lay = pkg.MlaDecodeLayer(ctx=n_rows, H=H, T_max=T, device=dev, use_graph=True)
        lay.cache.copy_(caches[j])
        layers.append(lay)
    torch.cuda.synchronize()
    del caches
    q_host = randn_f16((T, H, D_QK)).cpu().pin_memory()
    kv_host = (torch.randn((T, D_QK), generator=gen, device=dev) * 0.5).cpu().pin_memory()
    h2d = q_host.numel() * 2 + kv_host.numel() * 4 + 4
    d2h = T * H * D_V * 4

    def e2e_step(i):
        lay = layers[i % n_layers]
        lay.pos = n_rows - T  # the two new rows land at 32766, 32767; 32768 rows are attended
        lay.step(q_host, kv_host)

    e2e_steps = min(args.steps, 500)
    # every layer records its graph on its first step: all of that happens here, before anything is timed
    for i in range(max(2 * n_layers, min(args.warmup, 20))):
        e2e_step(i)
    e2e_runs = []
    for _ in range(max(1, args.repeats)):
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            e2e_step(i)
        torch.cuda.synchronize()
        e2e_runs.append(max_over_ranks((time.perf_counter() - t0)) / e2e_steps)
    e2e_sec = statistics.median(e2e_runs)
    # where an end-to-end step goes: the span of the replayed graph on the layer's stream (CUDA events around the
    # call, outside the timed region); the rest of the wall time is the host's launch and its wait for completion
    spans = []
    for i in range(40):
        lay = layers[i % n_layers]
        lay.pos = n_rows - T
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(lay._graph_stream)
        lay.step(q_host, kv_host)
        e1.record(lay._graph_stream)
        e1.synchronize()
        spans.append(e0.elapsed_time(e1) * 1e3)
    e2e_span_us = max_over_ranks(statistics.median(spans))
    # the same step without the wait: the graphs of all layers enqueued back to back on their streams, drained once.
    # What remains of a step then is the device's share (three kernels, one PCIe round trip for the host's rows); the
    # difference to the timed step is launch and completion latency that a step handing its result to the host exposes.
    hs = [lay._graphs[(q_host.data_ptr(), kv_host.data_ptr(), T)] for lay in layers]
    raw_step = layers[0]._graph_step
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        j = i % n_layers
        raw_step(hs[j], n_rows - T, layers[j]._graph_stream_handle, 0)
    torch.cuda.synchronize()
    e2e_nowait_us = max_over_ranks((time.perf_counter() - t0)) / e2e_steps * 1e6
    clocks = sampler.stop()
    e2e = {"value": world * bytes_step / e2e_sec / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "us_per_step": e2e_sec * 1e6, "steps": e2e_steps, "repeats": len(e2e_runs),
           "us_min": min(e2e_runs) * 1e6, "us_max": max(e2e_runs) * 1e6, "graph_span_us": e2e_span_us,
           "us_per_step_enqueued_without_waiting": e2e_nowait_us}
    del layers
    torch.cuda.empty_cache()

    # ---- the other configurations --------------------------------------------------------------------
    others = {}
    if not args.no_others:
        try:
            others = run_others(pkg, torch, dist, dev, world, rank, randn_f16, time_loop, hbm_peak, (tf_peak, tf_sustained), args)
        except Exception as exc:  # keep the headline line even if an extra fails
            others = {"error": f"{type(exc).__name__}: {exc}"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_decode_baseline(n_rows, T, budget_s=10.0)
        cpu.pop("seconds_per_pass", None)

    if rank == 0:
        line = {
            "metric": "MLA decode-attention HBM GB/s (MTP verify, 32K ctx)", "value": value, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 in / f32 accumulate",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "replicas": "one independent sequence per GPU",
                       "launch": "one pass over the cache copies captured in a CUDA graph and replayed",
                       "l2": f"rotates over {n_copies} distinct cache copies ({n_copies * n_rows * D_QK * 2 >> 20} MiB "
                             "> 2 x L2)"},
            "e2e": e2e, "gpu_launches": 2 * args.steps, "launches_per_step": {"value": 2, "e2e": 3},
            "timing": spread,
            "roofline": roofline, "cpu_baseline": cpu, "clocks": clocks, "others": others,
        }
        # the sharded configurations once more, short and at the very end of the line
        if isinstance(others, dict) and "ctx128k_T1" in others:
            c3, p5 = others["ctx128k_T1"], others.get("paged64", {})
            line["sharded"] = {
                "n_gpus": world, "ctx128k_us": round(c3["us_per_step"], 2),
                "ctx128k_frac_per_gpu": round(c3["frac_of_hbm_per_gpu"], 3),
                "ctx128k_nccl_us": round(others["ctx128k_T1_nccl"]["us_per_step"], 2) if "ctx128k_T1_nccl" in others else None,
                "paged64_us": round(p5.get("us_per_step", 0.0), 2), "paged64_frac_per_gpu": round(p5.get("frac_of_hbm_per_gpu", 0.0), 3),
                "exchange": "none" if world == 1 else ("p2p" if "ctx128k_T1_p2p_error" not in others else "nccl"),
                "max_abs_vs_1gpu": others.get("sharded_max_abs_vs_1gpu"),
            }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_others(pkg, torch, dist, dev, world, rank, randn_f16, time_loop, hbm_peak, tf_peak, args) -> dict:
    res = {}
    steps, warm = min(args.steps, 200), min(max(args.warmup, 3), 20)

    # -- 128K context, T = 1: one GPU, or sharded by contiguous sequence ranges over all ranks --------
    n_total = 131072
    lo, hi = pkg.shard_rows(n_total, world, rank, 16)
    rows_local = hi - lo
    n_copies = max(2, -(-2 * L2_BYTES // max(1, rows_local * D_QK * 2)) + 1)
    n_copies = min(n_copies, 24)
    shards = [randn_f16((max(rows_local, 1), D_QK), 0.5) for _ in range(n_copies)]
    q1 = randn_f16((1, 1, H, D_QK))
    if world > 1:
        dist.broadcast(q1, src=0)  # one query for the whole sharded context
    lens = torch.tensor([rows_local], dtype=torch.int32, device=dev)
    ws = pkg.new_workspace(1, 1, H, D_V, dev)
    rows_q = H
    total_bytes = algorithmic_bytes(n_total, 1)
    if world == 1:
        o1 = torch.empty((1, 1, H, D_V), dtype=torch.float32, device=dev)
        sec = time_loop(lambda i: pkg.mla_decode(q1, shards[i % n_copies], lens, out=o1, workspace=ws,
                                                 max_seq_len=rows_local), steps, warm, period=n_copies)
        exchange = "none"
    else:
        o1 = torch.empty((1, 1, H, D_V), dtype=torch.float32, device=dev)
        sec, exchange = None, None
        try:
            # peer-to-peer: every rank stores its merged record into all ranks' exchange buffers over NVLink
            # and merges what it received, inside one kernel after the attention kernel (no NCCL call per step)
            ex = pkg.PeerExchange(rows_q)
            keep = []

            def p2p_step(i):
                x = ex.next(device_epoch=True)
                keep.append(x)
                pkg.mla_decode(q1, shards[i % n_copies], lens, tail_causal=(rank == world - 1), out=o1, workspace=ws,
                               max_seq_len=rows_local, exchange=x)

            # the epoch lives in the exchange buffers, so the step can be captured once and replayed
            sec = time_loop(p2p_step, steps, warm, period=n_copies)
            torch.cuda.synchronize()
            ok = torch.tensor([1 if pkg.decode_status(ws) == 0 else 0], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) != 1:
                raise RuntimeError("a rank reported an exchange time-out")
            exchange = "peer-to-peer stores of the (acc, m, l) records as {value, epoch} words, merged in one kernel (CUDA graph)"
            # Outside the timed region: one more exchanged step on the first shard copies, checked on EVERY rank against
            # the single-GPU decode of the concatenated shards (all-gathered once for the check)
            o1.zero_()
            xk = ex.next(device_epoch=True)
            pkg.mla_decode(q1, shards[0], lens, tail_causal=(rank == world - 1), out=o1, workspace=ws, max_seq_len=rows_local, exchange=xk)
            torch.cuda.synchronize()
            if pkg.decode_status(ws) != 0:
                raise RuntimeError("exchange time-out in the checked step")
            sizes = [pkg.shard_rows(n_total, world, r, 16) for r in range(world)]
            if len({hi_ - lo_ for lo_, hi_ in sizes}) != 1:
                raise RuntimeError("shards of unequal size: the check gathers equal shards")
            whole = torch.empty((n_total, D_QK), dtype=torch.float16, device=dev)
            dist.all_gather_into_tensor(whole, shards[0])
            o_one = torch.empty_like(o1)
            pkg.mla_decode(q1, whole, torch.tensor([n_total], dtype=torch.int32, device=dev), out=o_one,
                           workspace=pkg.new_workspace(1, 1, H, D_V, dev), max_seq_len=n_total)
            torch.cuda.synchronize()
            err = (o1 - o_one).abs().max().reshape(1).double()
            dist.all_reduce(err, op=dist.ReduceOp.MAX)
            res["sharded_max_abs_vs_1gpu"] = float(err.item())
            del whole
            dist.barrier()
            ex.close()
            if not (float(err.item()) <= 2e-3):
                print(json.dumps({"error": f"sharded 128K decode differs from the single-GPU result by {float(err.item()):.3e} (> 2e-3)"}),
                      flush=True)
                raise SystemExit(1)
        except Exception as exc:
            res["ctx128k_T1_p2p_error"] = f"{type(exc).__name__}: {exc}"
            sec = None
        block = torch.empty(pkg.part_floats(rows_q), dtype=torch.float32, device=dev)
        gathered = torch.empty((world, block.numel()), dtype=torch.float32, device=dev)
        o2 = torch.empty((rows_q, D_V), dtype=torch.float32, device=dev)

        def sharded_step(i):
            pkg.mla_decode(q1, shards[i % n_copies], lens, tail_causal=(rank == world - 1), want_out=False,
                           part_out=block, workspace=ws, max_seq_len=rows_local)
            dist.all_gather_into_tensor(gathered, block)
            pkg.combine_parts(gathered, world, rows_q, D_V, out=o2)

        # the whole step (attention on the shard, all-gather of the records, merge) is captured in a graph
        sec_nccl = time_loop(sharded_step, steps, warm, period=n_copies)
        res["ctx128k_T1_nccl"] = {"us_per_step": sec_nccl * 1e6, "value": total_bytes / sec_nccl / 1e9,
                                  "exchange": "nccl all_gather of (acc, m, l) records + local combine (CUDA graph)"}
        if sec is not None:  # both paths on the first shard copies: the all-gather path against the checked peer-to-peer result
            sharded_step(0)
            torch.cuda.synchronize()
            d = (o2.view(-1) - o1.view(-1)).abs().max().reshape(1).double()
            dist.all_reduce(d, op=dist.ReduceOp.MAX)
            res["ctx128k_T1_nccl"]["max_abs_vs_p2p"] = float(d.item())
        if sec is None:
            sec, exchange = sec_nccl, res["ctx128k_T1_nccl"]["exchange"]
    gbs = total_bytes / sec / 1e9
    res["ctx128k_T1"] = {"metric": "aggregate GB/s", "value": gbs, "us_per_step": sec * 1e6, "scaling": "strong",
                         "frac_of_hbm_per_gpu": gbs / world / hbm_peak, "exchange": exchange,
                         "rows_per_gpu": rows_local, "bytes": total_bytes}
    del shards
    torch.cuda.empty_cache()

    # -- 64 paged sequences, lengths U[1024, 65536], sharded across ranks longest-first ---------------
    import numpy as np
    rng = np.random.default_rng(5)
    lens_all = rng.integers(1024, 65537, size=64)
    owners, load = pkg.lpt_assign(lens_all.tolist(), world)
    mine = owners[rank]
    my_lens = lens_all[mine]
    pages_per = -(-my_lens // 64)
    n_pages = int(pages_per.sum()) + 4
    pool = randn_f16((n_pages * 64, D_QK), 0.5)
    perm = rng.permutation(n_pages)
    pt = np.zeros((max(1, len(mine)), int(max(1, pages_per.max() if len(mine) else 1))), np.int32)
    k = 0
    for b in range(len(mine)):
        pt[b, :pages_per[b]] = perm[k:k + pages_per[b]]
        k += int(pages_per[b])
    if len(mine):
        ptd = torch.from_numpy(pt).to(dev)
        ld = torch.from_numpy(my_lens.astype(np.int32)).to(dev)
        qb = randn_f16((len(mine), 1, H, D_QK))
        ob = torch.empty((len(mine), 1, H, D_V), dtype=torch.float32, device=dev)
        wsb = pkg.new_workspace(len(mine), 1, H, D_V, dev)
        fn = lambda i: pkg.mla_decode(qb, pool, ld, page_table=ptd, out=ob, workspace=wsb,
                                      max_seq_len=int(my_lens.max()))
    else:
        fn = lambda i: None
    sec = time_loop(fn, min(steps, 50), min(warm, 5))
    tot = int(lens_all.sum()) * D_QK * 2 + 64 * H * (D_QK * 2 + D_V * 4)
    res["paged64"] = {"metric": "aggregate GB/s", "value": tot / sec / 1e9, "us_per_step": sec * 1e6,
                      "frac_of_hbm_per_gpu": tot / sec / 1e9 / world / hbm_peak, "scaling": "strong",
                      "load_imbalance_max_over_mean": max(load) / (sum(load) / world), "bytes": tot,
                      "l2": "pool per GPU exceeds L2 at 1-8 GPUs" if n_pages * 64 * D_QK * 2 > 2 * L2_BYTES
                      else "pool smaller than 2 x L2"}
    del pool
    torch.cuda.empty_cache()

    # -- twin shapes of the reference kernel (R = 512, H = 32 or 64), for a like-for-like ratio --------
    # (more than 48 packed query rows run as head groups, one pass over the cache per group)
    twin = {}
    for name, n, T, Ht in (("ctx32k_T2_H32", 32768, 2, 32), ("ctx32k_T1_H32", 32768, 1, 32),
                           ("ctx128k_T1_H32", 131072, 1, 32), ("ctx32k_T1_H64", 32768, 1, 64),
                           ("ctx4k_T1_H32", 4096, 1, 32)):
        nc = max(2, -(-2 * L2_BYTES // (n * 1024)) + 1)
        cs = [randn_f16((n, 512), 0.5) for _ in range(nc)]
        qt = randn_f16((1, T, Ht, 512))
        lt = torch.tensor([n], dtype=torch.int32, device=dev)
        ot = torch.empty((1, T, Ht, 512), dtype=torch.float32, device=dev)
        wt = pkg.new_workspace(1, T, Ht, 512, dev)
        sec = time_loop(lambda i: pkg.mla_decode(qt, cs[i % nc], lt, out=ot, workspace=wt, max_seq_len=n), steps, warm,
                        period=nc)
        twin[name] = {"us_per_call": sec * 1e6, "GB/s": n * 1024 / sec / 1e9}
        del cs
        torch.cuda.empty_cache()
    res["twin_R512"] = twin

    # -- the engine's sparse decode shape through gs_mla_attn: CUDA-core kernel, then the automatic choice (tcgen05 kernel
    #    fed from the position lists by gather copies; nothing beyond the reference's own arguments) -------------------
    try:
        fn = pkg._lib.load().gs_mla_attn
        pkg.mla_attn_impl(1)
        try:
            sp = _sparse_list_shape(torch, dev, fn, "cuda_core")
        finally:
            pkg.mla_attn_impl(0)
        sp.update(_sparse_list_shape(torch, dev, fn, "tensor_path"))
        sp.update(_sparse_list_shape(torch, dev, fn, "q8_tensor_path", q8=True))
        pkg.mla_attn_impl(1)
        try:
            sp.update(_sparse_list_shape(torch, dev, fn, "q8_cuda_core", q8=True))
        finally:
            pkg.mla_attn_impl(0)
        torch.cuda.synchronize()
        sp["tensor_path_status"] = pkg.mla_attn_status()
        res["gs_mla_attn_sparse"] = sp
    except Exception as exc:
        res["gs_mla_attn_sparse"] = {"error": f"{type(exc).__name__}: {exc}"}
    torch.cuda.empty_cache()

    # -- causal prefill, 8192 tokens, 20 heads, d = 256 (replicas only; measured on every rank) -------
    S, d = 8192, 256
    Q, K, V = randn_f16((S, H, d)), randn_f16((S, H, d)), randn_f16((S, H, d))
    pkg.rope_f16_inplace(Q)
    pkg.rope_f16_inplace(K)
    O = torch.empty((S, H, d), dtype=torch.float32, device=dev)
    sec = time_loop(lambda i: pkg.prefill_attn(Q, K, V, out=O), min(steps, 20), 3)
    flops = H * S * (S + 1) / 2 * (2 * d + 2 * d)
    # one launch after an idle pause (the board is below its power cap), then the clock during half a second of launches
    single = []
    for _ in range(5):
        torch.cuda.synchronize()
        time.sleep(0.05)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        pkg.prefill_attn(Q, K, V, out=O)
        e1.record()
        torch.cuda.synchronize()
        single.append(e0.elapsed_time(e1))
    load = ClockSampler(dev.index or 0)
    load.start()
    t_end = time.perf_counter() + 0.5
    while time.perf_counter() < t_end:
        for _ in range(20):
            pkg.prefill_attn(Q, K, V, out=O)
        torch.cuda.synchronize()
    load_clocks = load.stop()
    res["prefill8k"] = {"metric": "TFLOP/s (causal FLOPs)", "value": flops / sec / 1e12, "ms_per_step": sec * 1e3,
                        "frac_of_tensor_peak": flops / sec / 1e12 / tf_peak[0],
                        "frac_of_sustained_tensor_peak": flops / sec / 1e12 / tf_peak[1],
                        "note": "timed back to back, i.e. under the power cap: the sustained figure is the fitting denominator",
                        "flops": flops, "scaling": "replicas", "ms_single_launch_after_idle": min(single),
                        "tflops_single_launch_after_idle": flops / (min(single) * 1e-3) / 1e12, "clocks_under_load": load_clocks}
    return res


def run_profile_case(name: str) -> None:
    """A few eager launches of one kernel, small enough for a multi-pass ncu capture: inputs larger
    than L2 where DRAM figures matter, a few hundred MB on the device at most."""
    import torch
    pkg = importlib.import_module("glm-ssd_b200")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    if name in ("decode32k", "decode128k"):
        n, T = (32768, 2) if name == "decode32k" else (131072, 1)
        copies = [(torch.randn((n, D_QK), device=dev) * 0.5).half() for _ in range(8 if n == 32768 else 3)]
        q = torch.randn((1, T, H, D_QK), device=dev).half()
        lens = torch.tensor([n], dtype=torch.int32, device=dev)
        out = torch.empty((1, T, H, D_V), dtype=torch.float32, device=dev)
        ws = pkg.new_workspace(1, T, H, D_V, dev)
        for i in range(6):
            pkg.mla_decode(q, copies[i % len(copies)], lens, out=out, workspace=ws, max_seq_len=n)
    elif name == "paged":
        import numpy as np
        rng = np.random.default_rng(5)
        lens_h = rng.integers(1024, 16385, size=32)
        pages = -(-lens_h // 64)
        pool = (torch.randn((int(pages.sum()) * 64, D_QK), device=dev) * 0.5).half()
        pt = np.zeros((32, int(pages.max())), np.int32)
        perm, k = rng.permutation(int(pages.sum())), 0
        for b in range(32):
            pt[b, :pages[b]] = perm[k:k + pages[b]]
            k += int(pages[b])
        q = torch.randn((32, 1, H, D_QK), device=dev).half()
        out = torch.empty((32, 1, H, D_V), dtype=torch.float32, device=dev)
        ws = pkg.new_workspace(32, 1, H, D_V, dev)
        for i in range(4):
            pkg.mla_decode(q, pool, torch.from_numpy(lens_h.astype(np.int32)).to(dev), page_table=torch.from_numpy(pt).to(dev),
                           out=out, workspace=ws, max_seq_len=int(lens_h.max()))
    elif name in ("sparse", "sparse_q8"):
        # the engine's sparse decode shape through the reference's entry point: 64 heads, 2052 listed rows per token
        # (sparse_q8: over the Q8 cache)
        fn = pkg._lib.load().gs_mla_attn
        _sparse_list_shape(torch, dev, fn, "profile", profile=True, q8=name == "sparse_q8")
    else:
        S, Hh = 4096, 8
        Q, K, V = (torch.randn((S, Hh, 256), device=dev).half() for _ in range(3))
        O = torch.empty((S, Hh, 256), dtype=torch.float32, device=dev)
        for i in range(4):
            pkg.prefill_attn(Q, K, V, out=O)
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": name, "ok": True}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--repeats", type=int, default=15,
                    help="how often the timed region of --steps steps is repeated (the median is reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-others", action="store_true", help="skip the 128K / paged / prefill extras")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--profile-case", default=None, choices=["decode32k", "decode128k", "paged", "prefill", "sparse", "sparse_q8"],
                    help="run a handful of eager launches of one kernel on a small case and exit (for ncu)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.profile_case:
        run_profile_case(args.profile_case)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
