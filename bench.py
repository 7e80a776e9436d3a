#!/usr/bin/env python
"""Benchmark of the W4A4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workloads (synthetic, seeded; shapes from the reference's benchmark configurations):
  had_quant     (default) fused full-width Hadamard + per-token asymmetric int4 quantiser + packing,
                f16 X [16384, 4096] ~ N(0,1) with 0.1 % outlier channels x20; metric = algorithmic GB/s
                (bytes = M * (2K + K/2 + 4)).  One step = one launch over one batch.
  norm_quant    fused RMS-norm + per-token asymmetric int4 (the decoder's hidden-state step); --rows / --k.
  gemm_prefill  int4 GEMM + dequant, M = 2048, 4096 -> 12288, group-128 scales; metric = TOPS (2MNK).
  gemm_decode   int4 GEMM + dequant, M = 16 (--m), 4096 -> 22016; metric = GB/s on packed-weight bytes.
  grid          every point of the two measurement grids (quantisers: M x K x mode; GEMM: M x layer shape x scale mode)
                as tables under "extra", each with its fraction of the measured and of the nominal peak.
  llama7b_prefill | llama7b_decode | llama70b_prefill | llama70b_decode   the Llama-shaped W4A4 decoder (tok/s).
The default run also measures the other kernels briefly and reports them under "extra".

One JSON line on stdout (rank 0).  Multi-GPU: token batches are independent, so every rank runs
the same batch size on its own GPU (weak scaling, no data-path collective); time = max over ranks.
`--impl reference` times the reference's own CPU implementation of the same path (the PyTorch
fake_quant code, restated in oracle/fake_quant_port.py) on the host cores, on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1024 * 1024


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "src": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "fallback"}


def recorded_traffic(kernel, M, K):
    """DRAM bytes per launch of `kernel` at this shape, as recorded in its ncu summary under profiles/ (a line
    `dram_bytes_per_launch: <number>`); (None, reason) when no summary of this kernel and shape is committed."""
    import re
    path = os.path.join(ROOT, "profiles", f"{kernel}_M{M}_K{K}.md")
    if not os.path.exists(path):
        return None, f"no profiles/{os.path.basename(path)}"
    m = re.search(r"dram_bytes_per_launch:\s*([0-9.eE+]+)", open(path).read())
    return (float(m.group(1)), f"recorded from profiles/{os.path.basename(path)} (ncu)") if m else (None, "no dram_bytes_per_launch line")


def synth_activations(m, k, seed, device, dtype=torch.float16):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(m, k, generator=g)
    n_out = max(1, round(k * 0.001))
    ch = torch.randperm(k, generator=g)[:n_out]
    x[:, ch] *= 20.0
    return x.to(dtype).to(device)


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs.  The NVML handle is
    looked up by the UUID of the CUDA device (NVML numbers every GPU of the host, CUDA only the visible ones)."""

    PERIOD_S = 0.02          # 50 Hz: enough for a region of a few ms upward, and no load on the launching thread

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.t0 = self.t1 = None        # perf_counter bounds of the timed region, set by timed_loop
        self._stop = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            uuid = str(torch.cuda.get_device_properties(index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except TypeError:
                self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "sw_power_cap": 0x4, "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append((time.perf_counter(), nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.PERIOD_S)

    def __enter__(self):
        if self.nv:
            self.t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self.nv:
            self.t.join(timeout=1)

    def summary(self):
        inside = [c for (t, c) in self.samples if self.t0 is not None and self.t0 <= t <= self.t1]
        window = "timed region"
        if len(inside) < 3:            # a region of a few ms: use every sample taken under load (warm-up included)
            inside, window = [c for (_, c) in self.samples], "warm-up + timed region"
        med = float(np.median(inside)) if inside else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(inside),
                "window": window}


def dist_setup(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if args.impl == "reference":
            return world, rank, local, None
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return world, rank, local, dist
    return world, rank, local, None


def timed_loop(fn, steps, warmup, dist, device, graph=False, sampler=None, settle_s=0.0):
    """W warm-up steps, then exactly `steps` steps between barrier+synchronize; CUDA events on the
    current stream; returns seconds (max over ranks).  graph=True: the `steps` steps are recorded into
    one CUDA graph (after the warm-up) and the timed region is its launch — for steps shorter than the
    host's per-launch cost."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    g = None
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(steps):
                fn(i)
        g.replay()          # one untimed replay
        torch.cuda.synchronize()
        if settle_s > 0:    # the same launches for a while, untimed: the clock sampler sees the GPU under this load
            t_end = time.perf_counter() + settle_s
            while time.perf_counter() < t_end:
                g.replay()
                torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0 = time.perf_counter()
    e0.record()
    if g is not None:
        g.replay()
    else:
        for i in range(steps):
            fn(i)
    e1.record()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.t0, sampler.t1 = w0, time.perf_counter()
    if dist is not None:
        dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) * 1e-3], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# ----------------------------------------------------------------------------------------------
def gemm_inputs(C, m, n, k, grouped, asym, device, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    A = torch.randint(0, 256, (m, k // 2), generator=g, dtype=torch.uint8).to(device)
    B = torch.randint(0, 256, (n, k // 2), generator=g, dtype=torch.uint8).to(device)
    gcols = k // 128 if grouped else 1
    sa = (torch.rand(m, gcols, generator=g) * 0.015 + 0.005).half().to(device)
    sb = (torch.rand(n, gcols, generator=g) * 0.015 + 0.005).half().to(device)
    za = torch.randint(0, 16, (m, gcols), generator=g).half().to(device) if asym else None
    rs = C.weight_rowsum(B, 128 if grouped else k) if asym else None
    return A, B, sa, sb, za, rs


def run_ours(args, world, rank, local, dist):
    import flh_b200
    from flh_b200 import _lib
    C = flh_b200._CUDA
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    _lib.check(_lib.load().flh_b200_device_check(), "device_check")
    peaks = measured_peaks()
    steps, warmup = args.steps, max(args.warmup, 3)
    out = {"n_gpus": world, "steps": steps, "warmup": warmup, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "data": "synthetic", "impl": "ours"}

    if args.workload == "had_quant":
        M, K = args.rows, args.k
        xs = [synth_activations(M, K, 100 + i + 10 * rank, device) for i in range(3)]   # 3 x 134 MB > L2
        step_bytes = M * (2 * K + K // 2 + 4)
        # caller-owned outputs: the timed loop allocates nothing
        outs3 = [(torch.empty((M, K // 2), dtype=torch.uint8, device=device), torch.empty((M,), dtype=torch.float16, device=device),
                  torch.empty((M,), dtype=torch.float16, device=device)) for _ in range(3)]
        exact = bool(args.exact)

        def fn(i):
            C.quant_token_asym_i4(xs[i % 3], hadamard=True, exact=exact, out=outs3[i % 3])

        # the K steps are recorded once into a CUDA graph and the timed region is its launch: a step is a 30-50 us kernel,
        # shorter than what the host may need per launch when eight ranks share the cores
        with ClockSampler(local) as cs:
            t = timed_loop(fn, steps, warmup, dist, device, sampler=cs, graph=True, settle_s=0.15)
        value = world * step_bytes * steps / t / 1e9
        kfac = C._sign_bits(K, device)[0]
        kernel = _lib.load().flh_b200_quant_token_kernel(M, K, 2 if exact else 1, kfac).decode()
        out.update(metric="had_quant_GBps", unit="GB/s", value=value, ms_per_step=t / steps * 1e3, dtype="f32",
                   config={"workload": "fused full-width Hadamard (binary32 accumulation) + per-token asymmetric int4 quant + pack, "
                                       f"f16 X[{M},{K}] per GPU, 0.1% outlier channels x20",
                           "M_per_gpu": M, "K": K, "bytes_per_step_per_gpu": step_bytes,
                           "transform": "reference summation order (bit-exact)" if exact else "high part on tcgen05 (default; <= 0.1 % of codes off by one vs the reference order)",
                           "l2": f"three rotating {M * K * 2 // 1000000} MB inputs" + (", each larger than the 126 MB L2" if M * K * 2 > L2_BYTES else ""),
                           "timing": f"the {steps} steps recorded into one CUDA graph, timed as one replay; outputs pre-allocated",
                           "parallelism": f"token-sharded x{world}, no collective"},
                   clocks=dict(cs.summary(), window="150 ms of the same launches directly before the timed region, and the timed region"),
                   gpu_launches=steps)
        ach = step_bytes * steps / t / 1e9
        traffic, traffic_src = recorded_traffic(kernel, M, K)
        out["roofline"] = {"kernel": kernel, "bound": "hbm", "achieved": ach,
                           "peak": peaks["hbm_gbs"], "peak_src": peaks["src"], "unit": "GB/s",
                           "frac": ach / peaks["hbm_gbs"],
                           # dram__bytes_read.sum + dram__bytes_write.sum of one launch, read from the ncu summary of this kernel
                           "traffic": traffic, "traffic_unit": "bytes/launch", "traffic_src": traffic_src, "algorithmic_bytes": step_bytes}
        # ---- end to end through the public API with host buffers ----
        xh = [x.cpu().pin_memory() for x in xs[:2]]
        qh = torch.empty((M, K // 2), dtype=torch.uint8).pin_memory()
        sh = torch.empty((M,), dtype=torch.float16).pin_memory()
        zh = torch.empty((M,), dtype=torch.float16).pin_memory()
        # Three streams, two buffer sets: the upload of step i + 1 and the download of step i - 1 run beside the kernel of
        # step i (PCIe is full duplex).  Every step still uploads its own input and downloads its own codes, scales and
        # zero-points; the timed region ends when the last download has landed (the main stream waits for it).
        main = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        xd = [torch.empty((M, K), dtype=torch.float16, device=device) for _ in range(2)]
        qd = [torch.empty((M, K // 2), dtype=torch.uint8, device=device) for _ in range(2)]
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_used = [torch.cuda.Event() for _ in range(2)]       # the kernel has consumed xd[b]
        ev_out = [torch.cuda.Event() for _ in range(2)]        # the results of buffer set b are on the host

        def e2e(i):
            b = i % 2
            s_in.wait_event(ev_used[b])                        # (first use: an unrecorded event does not block)
            with torch.cuda.stream(s_in):
                xd[b].copy_(xh[b], non_blocking=True)
                ev_in[b].record(s_in)
            main.wait_event(ev_in[b])
            main.wait_event(ev_out[b])                         # the previous results of this set have left the device
            q, s_, z = C.quant_token_asym_i4(xd[b], hadamard=True, exact=exact, out=outs3[b])
            ev_used[b].record(main)
            s_out.wait_event(ev_used[b])
            with torch.cuda.stream(s_out):
                qh.copy_(q, non_blocking=True); sh.copy_(s_, non_blocking=True); zh.copy_(z, non_blocking=True)
                ev_out[b].record(s_out)
            if i == steps - 1 or i < 3:                        # last timed step (and the warm-up): join the downloads
                main.wait_event(ev_out[b])

        te = timed_loop(e2e, steps, 3, dist, device)
        out["e2e"] = {"value": world * step_bytes * steps / te / 1e9, "unit": "GB/s",
                      "h2d_bytes_per_step": M * K * 2, "d2h_bytes_per_step": M * K // 2 + 4 * M,
                      "ms_per_step": te / steps * 1e3}
        tp = None
        if world > 1 and not args.no_extra:       # collective work: every rank takes part
            try:
                tp = tp_extras(C, dist, world, rank, device)
            except Exception as e:                # the headline line must still be printed
                tp = {"tp_extras_error": repr(e)}
        if rank == 0 and not args.no_extra:
            out["extra"] = extras(C, device, peaks) if world == 1 else {}
            if tp:
                out["extra"].update(tp)
            if world == 1:
                out["cpu_baseline"] = cpu_had_quant(K, sample_rows=1024, reps=8)
    elif args.workload == "norm_quant":
        # the decoder's hidden-state step: RMS-norm (weight 1) + per-token asymmetric int4 + pack, no transform
        M, K = args.rows, args.k
        xs = [synth_activations(M, K, 100 + i + 10 * rank, device) for i in range(3)]
        step_bytes = M * (2 * K + K // 2 + 4)

        def fn(i):
            C.rmsnorm_quant_token_asym_i4(xs[i % 3], 1e-5, hadamard=False)

        with ClockSampler(local) as cs:
            t = timed_loop(fn, steps, warmup, dist, device, sampler=cs)
        ach = step_bytes * steps / t / 1e9
        out.update(metric="norm_quant_GBps", unit="GB/s", value=world * ach, ms_per_step=t / steps * 1e3, dtype="f32",
                   config={"workload": f"fused RMS-norm + per-token asymmetric int4 quant + pack (no transform), f16 X[{M},{K}] per GPU",
                           "M_per_gpu": M, "K": K, "bytes_per_step_per_gpu": step_bytes,
                           "l2": f"three rotating {M * K * 2 // 1000000} MB inputs", "parallelism": f"token-sharded x{world}, no collective"},
                   clocks=cs.summary(), gpu_launches=steps,
                   roofline={"kernel": "quant_token_warp_kernel<f16, warps per row = %d, no transform, norm>" % (K // 4096), "bound": "hbm",
                             "achieved": ach, "peak": peaks["hbm_gbs"], "peak_src": peaks["src"], "unit": "GB/s",
                             "frac": ach / peaks["hbm_gbs"], "traffic": None})
    elif args.workload == "had_quant_group":
        # FLH's own CUDA contract: group-128 binary16 transform + symmetric int4 + pack
        M, K = 16384, 4096
        xs = [synth_activations(M, K, 100 + i + 10 * rank, device).view(-1, 128) for i in range(3)]
        step_bytes = M * (2 * K + K // 2 + 2 * (K // 128))

        def fn(i):
            C.hadamard_and_quantize_i4(xs[i % 3])

        with ClockSampler(local) as cs:
            t = timed_loop(fn, steps, warmup, dist, device, sampler=cs)
        ach = step_bytes * steps / t / 1e9
        out.update(metric="had_quant_group128_GBps", unit="GB/s", value=world * ach, ms_per_step=t / steps * 1e3, dtype="f16",
                   config={"workload": "fused group-128 Hadamard (binary16) + symmetric int4 quant + pack, f16 X[16384,4096] per GPU",
                           "M_per_gpu": M, "K": K, "bytes_per_step_per_gpu": step_bytes,
                           "l2": "three rotating 134 MB inputs, each larger than the 126 MB L2",
                           "parallelism": f"token-sharded x{world}, no collective"},
                   clocks=cs.summary(), gpu_launches=steps,
                   roofline={"kernel": "quant_group_sym_kernel<7,true>", "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"],
                             "peak_src": peaks["src"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"], "traffic": None})
    elif args.workload == "grid":
        out.update(grid_tables(C, device, peaks))
        out.update(metric="grid", unit="see extra", value=0.0, ms_per_step=0.0, dtype="int4 codes", gpu_launches=0,
                   config={"workload": "the measurement grids of the quantisers (M x K x mode) and of the GEMM (M x shape x scale mode)"})
    elif args.workload in ("gemm_prefill", "gemm_decode"):
        prefill = args.workload == "gemm_prefill"
        M, K, N = (2048, 4096, 12288) if prefill else (16, 4096, 22016)
        if args.m:
            M = args.m                                   # e.g. --m 64: a decode batch the tensor-core decode kernel serves
        asym = args.act_mode == "token_asym"          # per-token asymmetric x per-channel weights, else group-128 symmetric
        sets = [gemm_inputs(C, M, N, K, not asym, asym, device, seed=s + 10 * rank) for s in range(3 if not prefill else 1)]
        D = torch.empty((M, N), dtype=torch.float16, device=device)
        flush = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=device) if prefill else None

        prepack = bool(args.prepack and prefill and asym)
        B8 = C.expand_i4(sets[0][1]) if prepack else None

        def fn(i):
            A, B, sa, sb, za, rs = sets[i % len(sets)]
            if prepack:
                C.gemm_i8w_dequant(A, B8, sa, sb, A_zero=za, B_rowsum=rs, out=D)
            else:
                C.gemm_i4_dequant(A, B, sa, sb, A_zero=za, B_rowsum=rs, out=D)

        with ClockSampler(local) as cs:
            t = timed_loop(fn, steps, warmup, dist, device, graph=not prefill, sampler=cs)
        if prefill:
            ops = 2.0 * M * N * K
            value = world * ops * steps / t / 1e12
            out.update(metric="int4_gemm_TOPS", unit="TOPS", value=value, dtype="s8 x s8 -> s32 (int4 codes)",
                       roofline={"bound": "tensor", "achieved": ops * steps / t / 1e12,
                                 "peak": 2 * peaks["bf16_tflops"], "peak_src": peaks["src"] + " bf16 x2 (dense INT8 runs at twice the bf16 rate)",
                                 "unit": "TOPS", "frac": ops * steps / t / 1e12 / (2 * peaks["bf16_tflops"]), "traffic": None})
        else:
            gcols = 1 if asym else K // 128
            b = N * K // 2 + 2 * N * gcols + M * K // 2 + 2 * M * gcols + 2 * M * N
            value = world * b * steps / t / 1e9
            out.update(metric="int4_gemm_decode_GBps", unit="GB/s", value=value, dtype="s8 x s8 -> s32 (int4 codes)",
                       roofline={"bound": "hbm", "achieved": b * steps / t / 1e9, "peak": peaks["hbm_gbs"],
                                 "peak_src": peaks["src"], "unit": "GB/s", "frac": b * steps / t / 1e9 / peaks["hbm_gbs"], "traffic": None})
        out.update(ms_per_step=t / steps * 1e3, clocks=cs.summary(), gpu_launches=steps,
                   config={"workload": f"int4 GEMM + {'per-token asymmetric x per-channel' if asym else 'group-128'} dequant, M={M}, {K}->{N}, f16 out",
                           "M": M, "N": N, "K": K, "algo": int(_lib.load().flh_b200_gemm_pick_algo(M, N, K, K if asym else 128, K if asym else 128)),
                           "weights_prepacked_int8": prepack,
                           "l2": "weights of three rotating problems (3 x 45 MB > L2); the K steps run as one CUDA graph" if not prefill else "operands re-used across steps (compute-bound)",
                           "parallelism": f"replicated x{world}, no collective"})
    elif args.workload in ("llama7b_prefill", "llama7b_decode", "llama70b_prefill", "llama70b_decode"):
        from flh_b200.model import Decoder, DecoderConfig, LLAMA2_7B, LLAMA3_70B
        big = args.workload.startswith("llama70b")
        prefill = args.workload.endswith("prefill")
        shape = dict(LLAMA3_70B if big else LLAMA2_7B)
        if args.layers:
            shape["n_layers"] = args.layers
        cfg = DecoderConfig(**shape, vocab=32000, act_mode=args.act_mode, tp=world)
        model = Decoder(cfg, device, seed=0, group=None, with_head=True)
        prepack = bool(args.prepack and prefill and args.act_mode == "token_asym")
        if prepack:
            model.prepack_int8()
        if prefill:
            B, S = (4, 2048) if big else (1, 2048)
            ids = torch.randint(100, 200, (B, S), device=device)
            fn = lambda i: model(ids)
            tokens = B * S
        else:
            B, ctx = (64, 1024) if big else (16, 1024)
            cache = model.new_cache(B, ctx + 8)
            for c in cache:
                c[0].normal_(); c[1].normal_()
            ids = torch.randint(100, 200, (B, 1), device=device)
            fn = lambda i: model(ids, cache=cache, start=ctx)
            tokens = B
        steps, warmup = min(steps, 20), min(warmup, 5)
        with ClockSampler(local) as cs:
            # a decode step is ~600 short launches: it is recorded once into a CUDA graph and replayed
            try:
                t = timed_loop(fn, steps, max(warmup, 3), dist, device, sampler=cs, graph=not prefill)
                graphed = not prefill
            except Exception as e:          # a capture that fails (e.g. a collective that refuses it) falls back to plain launches
                sys.stderr.write(f"CUDA graph capture failed ({e}); timing plain launches\n")
                t = timed_loop(fn, steps, max(warmup, 3), dist, device, sampler=cs, graph=False)
                graphed = False
        out.update(metric="w4a4_llama_%s_tok_per_s" % ("prefill" if prefill else "decode"), unit="tok/s",
                   value=tokens * steps / t, ms_per_step=t / steps * 1e3, dtype="int4 codes, s32 accumulate, f16 activations",
                   steps=steps, warmup=max(warmup, 3), scaling="strong" if world > 1 else "weak", clocks=cs.summary(),
                   config={"workload": args.workload, **shape, "act_mode": args.act_mode, "batch": B,
                           "seq_or_ctx": 2048 if prefill else 1024, "parallelism": f"tp{world}" if world > 1 else "single GPU",
                           "weights": "random int4 codes and scales (no checkpoint)", "cuda_graph": graphed,
                           "weights_prepacked_int8": prepack})
    else:
        raise SystemExit(f"unknown workload {args.workload}")
    st = C.gemm_status()
    if st[0] != 0:
        out["device_status"] = st
    if rank == 0:
        print(json.dumps(out), flush=True)


def tp_extras(C, dist, world, rank, device, layers=8):
    """Tensor-parallel side measurements, run by every rank when WORLD_SIZE > 1 (the headline stays the token-sharded
    quantiser): a row-parallel layer checked against a single-GPU run that sums the same per-shard partial outputs in
    binary32; the all-reduce by itself at the two message sizes of the 70B-shaped model; and that model (`layers`
    layers) in prefill and decode with a per-component CUDA-event breakdown."""
    from flh_b200 import timing
    from flh_b200.model import Decoder, DecoderConfig, LLAMA3_70B
    from flh_b200.nn import ActQuantizer, LinearFLH
    from flh_b200.tp import RowParallelLinearFLH, shard_row
    ex = {}
    # ---- (1) row-parallel parity: o_proj of the 70B shape (8192 -> 8192), 256 tokens, both activation modes ----
    K, N, M = 8192, 8192, 256
    g = torch.Generator(device="cpu").manual_seed(1234)                  # same tensors on every rank
    for mode in ("group_sym", "token_asym"):
        sym = mode == "group_sym"
        full = LinearFLH(K, N, dtype=torch.float16, device=device, group_size=128 if sym else -1, in_group_size=128)
        full.w_packed.copy_(torch.randint(0, 256, full.w_packed.shape, dtype=torch.uint8, generator=g).to(device))
        full.w_scale.copy_((torch.rand(full.w_scale.shape, generator=g) * 0.015 + 0.005).half().to(device))
        x = torch.randn(M, K, generator=g).half().to(device)
        aq = ActQuantizer(bits=4, group_size=128 if sym else -1, sym=sym, use_hadamard=False, packed_output=True)
        kk = K // world
        parts = []
        for r in range(world):                                           # every rank can form every partial: inputs are replicated
            parts.append(shard_row(full, r, world)(*_reorder(aq(x[:, r * kk:(r + 1) * kk].contiguous()))))
        ref = torch.stack([p_.float() for p_ in parts]).sum(0)           # binary32 sum of the f16 partials
        y = RowParallelLinearFLH(shard_row(full, rank, world))(*_reorder(aq(x[:, rank * kk:(rank + 1) * kk].contiguous())))
        rel = ((y.float() - ref).abs().max() / ref.abs().max()).reshape(1)
        dist.all_reduce(rel, op=dist.ReduceOp.MAX)
        ex[f"tp_parity_max_rel_{mode}"] = float(rel.item())
        del full, parts
    ex["tp_parity_max_rel"] = max(ex["tp_parity_max_rel_group_sym"], ex["tp_parity_max_rel_token_asym"])
    ex["tp_parity_bound"] = 1e-3
    # ---- (2) the all-reduce by itself: 134 MB (prefill 4 x 2048 x 8192 f16) and 1 MB (decode 64 x 8192 f16) ----
    for name, numel, iters in (("134MB", 4 * 2048 * 8192, 10), ("1MB", 64 * 8192, 50)):
        buf = torch.zeros(numel, dtype=torch.float16, device=device)
        for _ in range(3):
            dist.all_reduce(buf)
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            dist.all_reduce(buf)
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e-3 / iters], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t = float(t.item())
        if name == "134MB":
            ex["allreduce_134MB_busbw_GBps"] = 2.0 * (world - 1) / world * numel * 2 / t / 1e9
            ex["allreduce_134MB_ms"] = t * 1e3
        else:
            ex["allreduce_1MB_us"] = t * 1e6
        del buf
    # ---- (2b) the library's one-launch all-reduce over peer-mapped buffers against NCCL at decode message sizes ----
    from flh_b200 import tp as tpmod
    one_shot = None
    try:
        one_shot = tpmod.enable_one_shot(max_bytes=2 << 20)
    except Exception as e:
        ex["allreduce_oneshot_unavailable"] = str(e)[:200]
    if one_shot is not None:
        for name, numel in (("16KB", 8192), ("128KB", 8 * 8192), ("1MB", 64 * 8192)):
            src = (torch.randn(numel, device=device) * (rank + 1)).half()
            a, b = src.clone(), src.clone()
            one_shot.reduce(a)
            dist.all_reduce(b)
            rel = ((a.float() - b.float()).abs().max() / b.float().abs().max()).reshape(1)
            dist.all_reduce(rel, op=dist.ReduceOp.MAX)
            ex[f"allreduce_oneshot_vs_nccl_max_rel_{name}"] = float(rel.item())
            for kind, fn in (("oneshot", lambda: one_shot.reduce(a)), ("nccl", lambda: dist.all_reduce(b))):
                t = timed_loop(lambda i: fn(), 50, 5, dist, device)
                ex[f"allreduce_{kind}_{name}_us"] = t / 50 * 1e6
                try:
                    t = timed_loop(lambda i: fn(), 50, 5, dist, device, graph=True)
                    ex[f"allreduce_{kind}_{name}_graph_us"] = t / 50 * 1e6
                except Exception as e:
                    sys.stderr.write(f"all-reduce graph capture failed ({e})\n")
        # behind a row-parallel linear (decode batch 64, 8192 -> 8192): the result IS the binary32 sum of the f16 partial
        # outputs in rank order, rounded once — compared bit for bit
        full = LinearFLH(K, N, dtype=torch.float16, device=device, group_size=-1, in_group_size=128)
        full.w_packed.copy_(torch.randint(0, 256, full.w_packed.shape, dtype=torch.uint8, generator=g).to(device))
        full.w_scale.copy_((torch.rand(full.w_scale.shape, generator=g) * 0.015 + 0.005).half().to(device))
        x = torch.randn(64, K, generator=g).half().to(device)
        aq = ActQuantizer(bits=4, group_size=-1, sym=False, use_hadamard=False, packed_output=True)
        kk = K // world
        acc = torch.zeros(64, N, dtype=torch.float32, device=device)
        for r in range(world):
            acc = acc + shard_row(full, r, world)(*_reorder(aq(x[:, r * kk:(r + 1) * kk].contiguous()))).float()
        y = RowParallelLinearFLH(shard_row(full, rank, world))(*_reorder(aq(x[:, rank * kk:(rank + 1) * kk].contiguous())))
        same = torch.tensor([1 if torch.equal(y.view(torch.int16), acc.half().view(torch.int16)) else 0], device=device)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        ex["tp_oneshot_row_parallel_equals_binary32_sum"] = bool(same.item())
        del full, acc
        ex["allreduce_oneshot_status"] = one_shot.status()
        tpmod.disable_one_shot()
    # ---- (3) the 70B-shaped decoder, `layers` layers, TP = world: tok/s and where the device time goes ----
    for mode in ("token_asym", "group_sym"):
        cfg = DecoderConfig(**dict(LLAMA3_70B, n_layers=layers), vocab=32000, act_mode=mode, tp=world)
        model = Decoder(cfg, device, seed=0, group=None, with_head=True)
        if mode == "token_asym":
            model.prepack_int8()
        ids = torch.randint(100, 200, (4, 2048), generator=torch.Generator().manual_seed(99)).to(device)   # the same on every rank
        model.cfg.seq_parallel = False                   # first the all-reduce form (activations replicated on every rank)
        t = timed_loop(lambda i: model(ids), 3, 3, dist, device)
        ex[f"llama70b_{layers}L_prefill_tok_per_s_{mode}"] = 4 * 2048 * 3 / t
        with timing.collect() as tc:
            model(ids)
        ex[f"llama70b_{layers}L_prefill_breakdown_ms_{mode}"] = {k_: round(v, 3) for k_, v in tc.summary().items()}
        # the same step with the residual stream sharded by tokens (reduce-scatter + all-gather of int4 codes)
        model.cfg.seq_parallel = True
        t = timed_loop(lambda i: model(ids), 3, 3, dist, device)
        ex[f"llama70b_{layers}L_prefill_seqpar_tok_per_s_{mode}"] = 4 * 2048 * 3 / t
        try:        # the same step recorded once into a CUDA graph (collectives included) and replayed: no launch gaps
            tg = timed_loop(lambda i: model(ids), 3, 3, dist, device, graph=True)
            ex[f"llama70b_{layers}L_prefill_seqpar_graph_tok_per_s_{mode}"] = 4 * 2048 * 3 / tg
        except Exception as e:
            sys.stderr.write(f"prefill graph capture failed ({e})\n")
        with timing.collect() as tc:
            y_sp = model(ids)
        ex[f"llama70b_{layers}L_prefill_seqpar_breakdown_ms_{mode}"] = {k_: round(v, 3) for k_, v in tc.summary().items()}
        model.cfg.seq_parallel = False
        y_ar = model(ids)
        ex[f"llama70b_{layers}L_prefill_seqpar_vs_allreduce_max_rel_{mode}"] = float(
            ((y_sp.float() - y_ar.float()).abs().max() / y_ar.float().abs().max()).item())
        del y_sp, y_ar
        # the same comparison on ONE layer (the difference before the following layers amplify it: f16 sums in another order)
        with torch.no_grad():
            x0 = model.embed(ids)
            pos = torch.arange(0, 2048, device=device)
            one_ar = model.layers[0](x0, pos)
            from flh_b200.tp import local_rows
            nblk = model.cfg.sp_blocks
            one_sp = model.layers[0](local_rows(x0.view(4 * 2048, -1), rank, world, nblk).contiguous(), pos, shape=(4, 2048, nblk))
            ref = local_rows(one_ar.view(4 * 2048, -1), rank, world, nblk)
            rel = ((one_sp.float() - ref.float()).abs().max() / ref.float().abs().max()).reshape(1)
            dist.all_reduce(rel, op=dist.ReduceOp.MAX)
            ex[f"seqpar_vs_allreduce_one_layer_max_rel_{mode}"] = float(rel.item())
            del x0, one_ar, one_sp
        model.cfg.seq_parallel = True
        if mode == "token_asym":
            ex["llama70b_%dL_prefill_tok_per_s" % layers] = max(ex[f"llama70b_{layers}L_prefill_tok_per_s_{mode}"],
                                                                ex[f"llama70b_{layers}L_prefill_seqpar_tok_per_s_{mode}"])
            B, ctx = 64, 1024
            cache = model.new_cache(B, ctx + 8)
            for c in cache:
                c[0].normal_(); c[1].normal_()
            ids1 = torch.randint(100, 200, (B, 1), device=device)
            fn = lambda i: model(ids1, cache=cache, start=ctx)
            try:
                t = timed_loop(fn, 10, 3, dist, device, graph=True)
                ex["llama70b_%dL_decode_cuda_graph" % layers] = True
            except Exception as e:
                sys.stderr.write(f"decode graph capture failed ({e}); timing plain launches\n")
                t = timed_loop(fn, 10, 3, dist, device)
                ex["llama70b_%dL_decode_cuda_graph" % layers] = False
            ex["llama70b_%dL_decode_tok_per_s" % layers] = B * 10 / t
            with timing.collect() as tc:
                fn(0)
            ex[f"llama70b_{layers}L_decode_breakdown_ms_eager"] = {k_: round(v, 3) for k_, v in tc.summary().items()}
            if one_shot is not None:      # the same step with the 1 MB all-reduces as the library's one-launch form, fused with the
                                          # residual add, the RMS-norm and the next quantiser (flh_b200_allreduce_add_rmsnorm_quant_token_asym_i4)
                def one_layer():          # logits after ONE layer: the f16 sums differ in order from NCCL's above two ranks, and
                    saved = model.layers  # eight layers of random weights with int4 activations amplify any last-bit difference
                    model.layers = saved[:1]
                    try:
                        return fn(0).float()
                    finally:
                        model.layers = saved
                ref = one_layer()
                tpmod.enable_one_shot(max_bytes=2 << 20)
                got = one_layer()
                rel = ((got - ref).abs().max() / ref.abs().max()).reshape(1)
                dist.all_reduce(rel, op=dist.ReduceOp.MAX)
                ex["decode_oneshot_vs_nccl_one_layer_max_rel"] = float(rel.item())
                try:
                    t1 = timed_loop(fn, 10, 3, dist, device, graph=True)
                except Exception as e:
                    sys.stderr.write(f"decode graph capture failed ({e}); timing plain launches\n")
                    t1 = timed_loop(fn, 10, 3, dist, device)
                ex["llama70b_%dL_decode_oneshot_tok_per_s" % layers] = B * 10 / t1
                with timing.collect() as tc:
                    fn(0)
                ex[f"llama70b_{layers}L_decode_oneshot_breakdown_ms_eager"] = {k_: round(v, 3) for k_, v in tc.summary().items()}
                ex["allreduce_oneshot_status_after_decode"] = tpmod._ONE_SHOT[None].status()
                tpmod.disable_one_shot()
            del cache
        del model
        torch.cuda.empty_cache()
    return ex


def _reorder(szq):
    """ActQuantizer returns (scale, zero, packed); the linears take (packed, scale, zero)."""
    s_, z_, q_ = szq
    return q_, s_, z_


def _time(fn, iters=10, warm=3, graph=False):
    """Seconds per call.  graph=True records `iters` calls into one CUDA graph and times its replay, so
    that kernels shorter than the host's launch cost are timed back to back."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                fn()
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        e1.record()
    else:
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / iters


NOMINAL_HBM_GBS, NOMINAL_INT8_TOPS = 7700.0, 4500.0      # data-sheet figures, for the "fraction of nominal" columns


def grid_tables(C, device, peaks):
    """Every point of the two measurement grids: fused transform + quantiser + pack for M in {1, 16, 256, 4096, 16384} x
    K in {4096, 11008, 14336} x both modes (GB/s on the algorithmic bytes), and the GEMM for M in {1, 8, 32, 512, 2048,
    8192} x four layer shapes x both scale modes (GB/s on the decode bytes up to 32 rows, TOPS above).  Short launches are
    timed as CUDA-graph replays; inputs rotate over enough copies to exceed L2 where one copy does not."""
    hbm, tops = peaks["hbm_gbs"], 2 * peaks["bf16_tflops"]
    quant, gemm = [], []
    for k in (4096, 11008, 14336):
        for m in (1, 16, 256, 4096, 16384):
            nset = 3 if m * k * 2 > 40_000_000 else 1
            xs = [synth_activations(m, k, 31 + i, device) for i in range(nset)]
            it = [0]

            def tok():
                it[0] += 1
                C.quant_token_asym_i4(xs[it[0] % nset], hadamard=True)

            def grp():
                it[0] += 1
                C.hadamard_and_quantize_i4(xs[it[0] % nset].view(-1, 128))

            for name, fn, sbytes in (("token_asym", tok, 4), ("group128_sym", grp, 2 * k // 128)):
                t = _time(fn, iters=12, warm=5, graph=True)
                gbs = m * (2 * k + k // 2 + sbytes) / t / 1e9
                quant.append({"M": m, "K": k, "mode": name, "us": round(t * 1e6, 2), "GBps": round(gbs, 1),
                              "frac_measured": round(gbs / hbm, 3), "frac_nominal": round(gbs / NOMINAL_HBM_GBS, 3)})
            del xs
    for (k, n) in ((4096, 12288), (4096, 4096), (4096, 22016), (11008, 4096)):
        for m in (1, 8, 32, 512, 2048, 8192):
            for grouped, asym, tag in ((True, False, "group128_sym"), (False, True, "token_asym_channel")):
                base = gemm_inputs(C, m, n, k, grouped, asym, device, seed=3)
                nset = max(1, -(-320_000_000 // (n * k // 2))) if m <= 32 else 1
                sets = [base] + [(base[0], base[1].clone()) + base[2:] for _ in range(nset - 1)]
                D = torch.empty((m, n), dtype=torch.float16, device=device)
                it = [0]

                def f():
                    it[0] += 1
                    A, B, sa, sb, za, rs = sets[it[0] % nset]
                    C.gemm_i4_dequant(A, B, sa, sb, A_zero=za, B_rowsum=rs, out=D)

                t = _time(f, iters=max(8, nset) if m <= 32 else 5, warm=3, graph=m <= 512)
                row = {"M": m, "K": k, "N": n, "scales": tag, "us": round(t * 1e6, 2),
                       "algo": int(_algo(m, n, k, 128 if grouped else k))}
                if m <= 32:
                    gc = k // 128 if grouped else 1
                    b = n * k // 2 + 2 * n * gc + m * k // 2 + 2 * m * n
                    row.update(GBps=round(b / t / 1e9, 1), frac_measured=round(b / t / 1e9 / hbm, 3), frac_nominal=round(b / t / 1e9 / NOMINAL_HBM_GBS, 3))
                else:
                    ops = 2.0 * m * n * k / t / 1e12
                    row.update(TOPS=round(ops, 1), frac_measured=round(ops / tops, 3), frac_nominal=round(ops / NOMINAL_INT8_TOPS, 3))
                gemm.append(row)
                del sets, base
    return {"extra": {"grid_quant": quant, "grid_gemm": gemm,
                      "peaks": {"hbm_gbs_measured": hbm, "hbm_gbs_nominal": NOMINAL_HBM_GBS, "int8_tops_2x_measured_bf16": tops,
                                "int8_tops_nominal": NOMINAL_INT8_TOPS}}}


def _algo(m, n, k, group):
    from flh_b200 import _lib
    return _lib.load().flh_b200_gemm_pick_algo(m, n, k, group, group)


def extras(C, device, peaks):
    """Short measurements of the other kernels of the path (not the headline)."""
    ex = {}
    for (m, k) in ((16384, 4096), (4096, 11008), (4096, 14336), (4096, 28672)):
        xs = [synth_activations(m, k, 7 + i, device) for i in range(2)]
        it = [0]

        def f():
            it[0] += 1
            C.quant_token_asym_i4(xs[it[0] % 2], hadamard=True)

        def g():
            it[0] += 1
            C.hadamard_and_quantize_i4(xs[it[0] % 2].view(-1, 128))

        t = _time(f, iters=20, warm=20)      # the end-to-end leg before this left the GPU mostly idle: let the clocks come back
        ex[f"had_quant_token_asym_M{m}_K{k}_GBps"] = m * (2 * k + k // 2 + 4) / t / 1e9
        t = _time(g, iters=20, warm=10)
        ex[f"had_quant_group128_sym_M{m}_K{k}_GBps"] = m * (2 * k + k // 2 + 2 * k // 128) / t / 1e9
        del xs
    for (m, k, n) in ((2048, 4096, 12288), (8192, 4096, 22016), (2048, 11008, 4096)):
        for grouped, asym, tag in ((True, False, "g128_sym"), (False, True, "token_asym_channel")):
            A, B, sa, sb, za, rs = gemm_inputs(C, m, n, k, grouped, asym, device)
            t = _time(lambda: C.gemm_i4_dequant(A, B, sa, sb, A_zero=za, B_rowsum=rs), iters=5, warm=2)
            ex[f"gemm_M{m}_{k}to{n}_{tag}_TOPS"] = 2.0 * m * n * k / t / 1e12
            if asym:        # the same with the weights expanded to int8 ahead of time
                B8 = C.expand_i4(B)
                t = _time(lambda: C.gemm_i8w_dequant(A, B8, sa, sb, A_zero=za, B_rowsum=rs), iters=5, warm=2)
                ex[f"gemm_M{m}_{k}to{n}_{tag}_prepacked_TOPS"] = 2.0 * m * n * k / t / 1e12
                del B8
    for (m, k, n) in ((1, 4096, 22016), (16, 4096, 22016), (64, 4096, 22016), (16, 11008, 4096), (16, 4096, 4096),
                      (16, 8192, 28672), (64, 8192, 28672)):
        # enough copies of the weights that successive launches cannot be served from the 126 MB L2
        base = gemm_inputs(C, m, n, k, True, False, device, seed=0)
        nsets = max(3, -(-320_000_000 // (n * k // 2)))
        sets = [base] + [(base[0], base[1].clone()) + base[2:] for _ in range(nsets - 1)]
        it = [0]

        D = torch.empty((m, n), dtype=torch.float16, device=device)

        def f():
            it[0] += 1
            A, B, sa, sb, za, rs = sets[it[0] % nsets]
            C.gemm_i4_dequant(A, B, sa, sb, out=D)

        t = _time(f, iters=max(12, nsets), graph=True)
        b = n * k // 2 + 2 * n * (k // 128) + m * k // 2 + 2 * m * n
        ex[f"gemm_decode_M{m}_{k}to{n}_g128_GBps"] = b / t / 1e9
        if m == 16:
            # what a plain streaming read of the same packed weights reaches at this size (the row-sum kernel): the
            # practical ceiling of a launch this short, well under the large-copy HBM peak
            def r():
                it[0] += 1
                C.weight_rowsum(sets[it[0] % nsets][1], k)

            t = _time(r, iters=max(12, nsets), graph=True)
            ex[f"read_ceiling_{k}to{n}_GBps"] = (n * k // 2) / t / 1e9
        del sets
    a8 = torch.randint(-8, 8, (8192, 8192), device=device, dtype=torch.int8)
    b8 = torch.randint(-8, 8, (8192, 8192), device=device, dtype=torch.int8)
    t = _time(lambda: torch._int_mm(a8, b8), iters=5, warm=2)
    ex["yardstick_torch_int_mm_8192_TOPS"] = 2.0 * 8192 ** 3 / t / 1e12
    return ex


# ----------------------------------------------------------------------------------------------
def cpu_had_quant(K, sample_rows, reps):
    from oracle import fake_quant_port as FQ
    H = FQ.hadamard_matrix(K)
    x = synth_activations(sample_rows, K, 5, "cpu")
    FQ.had_quant_pack(x, H)
    t0 = time.perf_counter()
    for _ in range(reps):
        FQ.had_quant_pack(x, H)
    t = (time.perf_counter() - t0) / reps
    b = sample_rows * (2 * K + K // 2 + 4)
    return {"value": b / t / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{sample_rows} rows of K={K} per step, {reps} steps: x @ H (dense, f32) + per-token asymmetric "
                      f"int4 + pack, torch CPU ({os.cpu_count()} logical CPUs)", "ms_per_step": t * 1e3}


def run_reference(args, world, rank):
    """The reference's own CPU implementation of the path (PyTorch fake_quant code, restated)."""
    if rank != 0:
        return
    if args.workload != "had_quant":
        print(json.dumps({"impl": "reference", "unavailable": "the CPU arm is implemented for the had_quant workload"}))
        return
    from oracle import fake_quant_port as FQ
    # all the host threads this process may use (torchrun exports OMP_NUM_THREADS=1 to its workers)
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except AttributeError:
        torch.set_num_threads(max(1, os.cpu_count() or 1))
    K, rows = 4096, 2048
    H = FQ.hadamard_matrix(K)
    xs = [synth_activations(rows, K, 100 + i, "cpu") for i in range(2)]
    for i in range(max(1, args.warmup)):
        FQ.had_quant_pack(xs[i % 2], H)
    t0 = time.perf_counter()
    for i in range(args.steps):
        FQ.had_quant_pack(xs[i % 2], H)
    t = time.perf_counter() - t0
    b = rows * (2 * K + K // 2 + 4)
    v = b * args.steps / t / 1e9
    sample = f"{rows} rows of K={K} per step (the GPU arm's batch is 16384 rows): x @ H dense f32 + per-token asymmetric int4 + pack"
    print(json.dumps({
        "impl": "reference", "metric": "had_quant_GBps", "unit": "GB/s", "value": v, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "fused full-width Hadamard + per-token asymmetric int4 quant + pack, f16 X[.,4096]", "K": K,
                   "rows_per_step": rows},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="had_quant")
    ap.add_argument("--act-mode", default="group_sym", choices=["group_sym", "token_asym"])
    ap.add_argument("--layers", type=int, default=0, help="override the layer count of the llama workloads")
    ap.add_argument("--rows", type=int, default=16384, help="had_quant: token rows per GPU (default: the headline 16384)")
    ap.add_argument("--m", type=int, default=0, help="gemm_prefill / gemm_decode: token rows M (default 2048 / 16)")
    ap.add_argument("--k", type=int, default=4096, help="had_quant: hidden size K (default: the headline 4096)")
    ap.add_argument("--prepack", action="store_true",
                    help="gemm_prefill / llama*_prefill with token_asym: keep an int8 copy of the weights (expanded once, outside the timed region)")
    ap.add_argument("--exact", action="store_true", help="had_quant: the transform in the reference's summation order (bit-exact mode) instead of the default")
    ap.add_argument("--no-extra", action="store_true", help="skip the side measurements and the CPU baseline (profiling runs)")
    args = ap.parse_args()
    world, rank, local, dist = dist_setup(args)
    if args.impl == "reference":
        run_reference(args, world, rank)
        return
    try:
        run_ours(args, world, rank, local, dist)
    finally:
        if dist is not None:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
