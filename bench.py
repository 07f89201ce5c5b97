#!/usr/bin/env python3
"""Benchmark of the quantized-matmul hot path on B200.

Default workload (N = 1): the Qwen3.6-27B-shaped NVFP4 decode weight sweep:
64 layers x 6 GEMVs (M = 1, bf16 activation, W4A16 semantics), 13.4 GB of
packed weights + block scales resident in HBM, hidden state running from GEMV
to GEMV.  One "step" = one pass over all 384 matrices through the C ABI
(qwen36_nvfp4_matvec).  `value` = algorithmic bytes per step / device time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Under torchrun (N > 1) every matrix is split by output rows across the ranks
and each GEMV is followed by an NCCL all-gather of the bf16 slices.

`--impl reference` times the reference's scalar semantics on the host cores
(the CPU oracle, an OpenMP C restatement) on a bounded sample: one layer per
step.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "NVFP4 GEMV HBM GB/s & GEMM TFLOPS (% roofline) at Qwen3.6-27B shapes"


NCU_TRAFFIC_RATIO = (100.327936 + 4.018688) / 100.349952    # dram bytes / algorithmic bytes, GEMV kernel (ncu, gate_up launch)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def gemv_bytes(n: int, k: int) -> int:
    """Algorithmic bytes of one W4A16 GEMV: packed weights + block scales + x + y."""
    return n * k // 2 + n * k // 16 + 2 * k + 2 * n


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML from a thread every
    2 ms (so that even a 30 ms region gets samples), `nvidia-smi -lms` when NVML cannot be loaded."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NVML_REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, pci_bus_id: str | None = None):
        self.index = index
        self.pci_bus_id = pci_bus_id
        self.samples = []          # nvidia-smi lines, or (sm_mhz, reasons_mask) tuples from NVML
        self.proc = None
        self.nvml = None
        self.handle = None
        self.max_mhz = None
        self._stop = False
        self.thread = None

    def _start_nvml(self) -> bool:
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = (pynvml.nvmlDeviceGetHandleByPciBusId(self.pci_bus_id) if self.pci_bus_id
                           else pynvml.nvmlDeviceGetHandleByIndex(self.index))
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            pynvml.nvmlDeviceGetClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            pynvml.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
            self.nvml = pynvml
            return True
        except Exception:
            self.nvml = None
            return False

    def _poll_nvml(self):
        nv = self.nvml
        while not self._stop:
            try:
                self.samples.append((float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)),
                                     int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self._start_nvml():
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self._stop = True
            self.thread.join(timeout=2)
            sm = sorted(s[0] for s in self.samples)
            mask = 0
            for s_ in self.samples:
                mask |= s_[1]
            reasons = sorted(name for bit, name in self.NVML_REASONS.items() if mask & bit)
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz, "reasons": reasons,
                    "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "source": "nvidia-smi"}


# --------------------------------------------------------------------------- ours

def build_sweep(backend, torch, synth, rank: int, world: int, layers: int, seed: int):
    """Per layer: [(name, n_local, k, weight, tiled scales, tensor scale)], rows split across ranks."""
    gen = torch.Generator(device="cuda").manual_seed(seed)          # same seed on every rank: same model
    sweep = []
    for _ in range(layers):
        mats = []
        for name, n, k in synth.DECODE_SHAPES:
            # full matrix generated identically on every rank, then sliced (keeps ranks consistent
            # with the 1-GPU model); slices are multiples of 128 rows so scale tiles stay whole
            packed, sf_rm = synth.nvfp4_weight_device(gen, n, k, "cuda")
            lo, hi = shard_rows(n, rank, world)
            packed, sf_rm = packed[lo:hi].contiguous(), sf_rm[lo:hi].contiguous()
            sf = backend.nvfp4_retile_scales(sf_rm)
            # per-tensor scale: 1/2688 times a gain that keeps the running hidden state at unit RMS
            gain = 2688.0 / (2.926 * 4.80 * (k ** 0.5))
            ts = torch.tensor([synth.WEIGHT_GLOBAL_SCALE * gain], dtype=torch.float32, device="cuda")
            mats.append((name, hi - lo, k, packed, sf, ts, n))
        sweep.append(mats)
    torch.cuda.synchronize()
    return sweep


def shard_rows(n: int, rank: int, world: int):
    from speedoza_b200 import shard
    return shard.shard_rows(n, rank, world)


class SweepRunner:
    """Chains the six GEMVs of every layer: q_gate, k, v <- x ; o <- q_gate[:6144] ;
    gate_up <- o ; down <- gate_up[:17408] ; next x <- down.  On one GPU the three projections
    that share x go out as ONE launch (qwen36_nvfp4_matvec_group), so a layer is four launches."""

    def __init__(self, backend, torch, sweep, world: int, dist=None):
        self.b, self.torch, self.sweep, self.world, self.dist = backend, torch, sweep, world, dist
        dev = "cuda"
        self.full = {name: torch.zeros(n, dtype=torch.bfloat16, device=dev) for name, n, _ in
                     __import__("speedoza_b200.synth", fromlist=["x"]).DECODE_SHAPES}
        self.local = {m[0]: torch.zeros(max(m[1], 1), dtype=torch.bfloat16, device=dev) for m in sweep[0]}
        self.x = torch.zeros(5120, dtype=torch.bfloat16, device=dev)
        self.launches = 0
        self.group_qkv = True

    def gemv(self, mat, x):
        name, n_local, k, packed, sf, ts, n_full = mat
        if self.world == 1:
            out = self.full[name]
            self.b.nvfp4_matvec(x, packed, sf, ts, out)
        else:
            out_local = self.local[name]
            if n_local > 0:
                self.b.nvfp4_matvec(x, packed, sf, ts, out_local)
            out = self.full[name]
            self.gather(out, out_local, n_full)
        self.launches += 1
        return out

    def gather(self, out, out_local, n_full):
        from speedoza_b200 import shard
        shard.all_gather_rows(out_local, n_full, self.world, out)

    def qkv(self, mats, x):
        if self.world != 1 or not self.group_qkv:
            qg = self.gemv(mats[0], x)
            self.gemv(mats[1], x)
            self.gemv(mats[2], x)
            return qg
        self.b.nvfp4_matvec_group(x, [(m[3], m[4], m[5], self.full[m[0]]) for m in mats[:3]])
        self.launches += 1
        return self.full[mats[0][0]]

    def step(self, x0):
        x = x0
        for mats in self.sweep:
            qg = self.qkv(mats, x)
            o = self.gemv(mats[3], qg[:6144])
            gu = self.gemv(mats[4], o)
            x = self.gemv(mats[5], gu[:17408])
        return x

    def capture(self):
        """Records one step (all C-ABI launches, and the all-gathers when sharded) into a CUDA
        graph, the way the reference engine replays its decode step; returns launches per step."""
        torch = self.torch
        self.x_static = torch.zeros(5120, dtype=torch.bfloat16, device="cuda")
        self.graph = torch.cuda.CUDAGraph()
        before = self.launches
        # thread-local capture mode: the NCCL watchdog thread may touch CUDA while this thread captures
        mode = "thread_local" if self.world > 1 else "global"
        with torch.cuda.graph(self.graph, capture_error_mode=mode):
            self.b.sync_stream()                  # library's ambient stream = the capturing stream
            self.y_static = self.step(self.x_static)
        self.b.sync_stream()
        per_step = self.launches - before
        self.launches = before
        return per_step

    def replay(self, x):
        self.x_static.copy_(x, non_blocking=True)
        self.graph.replay()
        return self.y_static


def per_shape_cold(backend, torch, sweep, synth):
    """Each decode shape alone, rotating through the 64 layer copies so every launch reads cold
    weights; 192 launches per timing, replayed from a CUDA graph."""
    out = {}
    for idx, (name, n, k) in enumerate(synth.DECODE_SHAPES):
        x = torch.randn(k, device="cuda").to(torch.bfloat16)
        y = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        mats = [layer[idx] for layer in sweep]

        def call(i, mats=mats, x=x, y=y):
            m = mats[i % len(mats)]
            backend.nvfp4_matvec(x, m[3], m[4], m[5], y)
        us = _time_cuda(torch, call, 192, warm=20, backend=backend)
        out[name] = {"n": n, "k": k, "us": round(us, 3), "gbs": round(gemv_bytes(n, k) / us / 1e3, 1)}
    # q_gate + k + v as one grouped launch (what the sweep issues)
    x = torch.randn(5120, device="cuda").to(torch.bfloat16)
    ys = [torch.empty(n, dtype=torch.bfloat16, device="cuda") for _, n, _ in synth.DECODE_SHAPES[:3]]

    def call_group(i):
        layer = sweep[i % len(sweep)]
        backend.nvfp4_matvec_group(x, [(m[3], m[4], m[5], y) for m, y in zip(layer[:3], ys)])
    us = _time_cuda(torch, call_group, 192, warm=20, backend=backend)
    byts = sum(gemv_bytes(n, k) for _, n, k in synth.DECODE_SHAPES[:3]) - 2 * 2 * 5120
    out["attn.qkv_group"] = {"n": 14336, "k": 5120, "us": round(us, 3), "gbs": round(byts / us / 1e3, 1)}
    # config 0: the single 5120 x 5120 GEMV, 64 weight copies (0.94 GB) rotated so every launch is cold
    gen = torch.Generator(device="cuda").manual_seed(500)
    copies = []
    for _ in range(64):
        packed, sf_rm = synth.nvfp4_weight_device(gen, 5120, 5120, "cuda")
        copies.append((packed, backend.nvfp4_retile_scales(sf_rm)))
    ts = torch.tensor([synth.WEIGHT_GLOBAL_SCALE], dtype=torch.float32, device="cuda")
    y0 = torch.empty(5120, dtype=torch.bfloat16, device="cuda")

    def call0(i):
        w, sf = copies[i % len(copies)]
        backend.nvfp4_matvec(x, w, sf, ts, y0)
    us = _time_cuda(torch, call0, 192, warm=20, backend=backend)
    out["config0_5120x5120"] = {"n": 5120, "k": 5120, "us": round(us, 3), "gbs": round(gemv_bytes(5120, 5120) / us / 1e3, 1),
                                "frac_of_measured_peak": round(gemv_bytes(5120, 5120) / us / 1e3 / measured_peaks()[0], 4)}
    return out


def per_shape_w4a4_decode(backend, torch, sweep, synth, tokens: int = 1):
    """The same shapes through the W4A4 decode entry (activations quantised to NVFP4 once, then
    qwen36_decode_nvfp4_gemv per matrix): tcgen05 block-scaled MMA, split-K clusters where the
    matrix has few row blocks.  Cold weights as in per_shape_cold."""
    out = {}
    for idx, (name, n, k) in enumerate(synth.DECODE_SHAPES):
        x = torch.randn((tokens, k), device="cuda").to(torch.bfloat16)
        fp4, sf, ts = backend.nvfp4_quantize_rows(x, 0.37)
        y = torch.empty((tokens, n), dtype=torch.bfloat16, device="cuda")
        mats = [layer[idx] for layer in sweep]
        alpha = synth.WEIGHT_GLOBAL_SCALE * 0.37

        def call(i, mats=mats, fp4=fp4, sf=sf, y=y, n=n, k=k):
            m = mats[i % len(mats)]
            rc = backend.decode_nvfp4_gemv_raw(m[3], m[4], fp4, sf, alpha, n, tokens, k, y)
            if rc != 0:
                raise RuntimeError(f"qwen36_decode_nvfp4_gemv returned {rc}")
        us = _time_cuda(torch, call, 192, warm=20, backend=backend)
        out[name] = {"n": n, "k": k, "us": round(us, 3), "gbs": round(gemv_bytes(n, k) / us / 1e3, 1)}
    return out


def _time_cuda(torch, fn, reps, warm=3, backend=None):
    """Microseconds per call of fn(i), timed with CUDA events around a CUDA-graph replay of `reps`
    calls (so that Python/ctypes launch overhead does not hide short kernels); eager if capture fails."""
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    graph = None
    if backend is not None:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                backend.sync_stream()
                for i in range(reps):
                    fn(i)
            backend.sync_stream()
            graph.replay()
            torch.cuda.synchronize()
        except Exception:
            graph = None
            backend.sync_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if graph is not None:
        graph.replay()
    else:
        for i in range(reps):
            fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / reps


def other_configs(backend, torch, synth, make_sampler=None):
    """The remaining benchmark configurations at 1 GPU, each timed with CUDA events over
    back-to-back launches on inputs larger than L2 (weights alternate between two copies where a
    single copy would fit): prefill GEMM + activation quantisation (config 2), FP8 lm_head with
    fused argmax (config 3), int8 KV encode + split-KV decode attention (config 4)."""
    out = {}
    gen = torch.Generator(device="cuda").manual_seed(7)
    # ---- config 2: NVFP4 prefill GEMM ------------------------------------------------------
    gemm = []
    for name, n_out, k in (("mlp.gate_up", 34816, 5120), ("mlp.down", 5120, 17408)):
        ws = []
        for _ in range(3):                     # 3 x 50 MB (down) / 3 x 100 MB (gate_up): more than L2 in rotation
            packed, sf_rm = synth.nvfp4_weight_device(gen, n_out, k, "cuda")
            ws.append((packed, backend.nvfp4_retile_scales(sf_rm)))
        for m_tok in (512, 2048, 8192):
            x = torch.randn((m_tok, k), generator=gen, device="cuda")
            ch = torch.randperm(k, generator=gen, device="cuda")[: k // 100]
            x[:, ch] *= 20.0
            x = x.to(torch.bfloat16)
            fp4 = torch.empty((m_tok, k // 2), dtype=torch.uint8, device="cuda")
            sf = torch.zeros(backend_tiled_bytes(m_tok, k // 16), dtype=torch.uint8, device="cuda")
            ts = torch.empty(1, dtype=torch.float32, device="cuda")
            q_us = _time_cuda(torch, lambda i: backend.nvfp4_quantize_rows(x, 0.37, fp4, sf, ts), 200, warm=20,
                              backend=backend)
            alpha = synth.WEIGHT_GLOBAL_SCALE * 0.37
            c = torch.empty((m_tok, n_out), dtype=torch.bfloat16, device="cuda")
            # 200 launches back to back run into the power cap at the larger sizes: the SM clock seen during the
            # timing is recorded beside the figure (sw_power_cap is kept and noted, not rejected)
            torch.cuda.synchronize()
            time.sleep(0.2)                     # let the power state settle: the burst figure is a cool-start one
            burst_us = _time_cuda(torch, lambda i: backend.nvfp4_gemm(ws[i % 3][0], ws[i % 3][1], fp4, sf, alpha,
                                                                       n_out, m_tok, k, c), 9, warm=3, backend=backend)
            sampler = make_sampler() if make_sampler is not None else None
            if sampler is not None:
                sampler.start()
            g_us = _time_cuda(torch, lambda i: backend.nvfp4_gemm(ws[i % 3][0], ws[i % 3][1], fp4, sf, alpha,
                                                                   n_out, m_tok, k, c), 200, warm=20, backend=backend)
            gemm_clocks = sampler.stop() if sampler is not None else None
            flops = 2.0 * m_tok * n_out * k
            gemm.append({"shape": name, "M": m_tok, "N": n_out, "K": k, "gemm_us": round(g_us, 2),
                         "tflops": round(flops / g_us / 1e6, 1),
                         "frac_of_nominal_9PF": round(flops / g_us / 1e6 / 9000.0, 4),
                         "burst_us": round(burst_us, 2), "burst_tflops": round(flops / burst_us / 1e6, 1),
                         "clocks": gemm_clocks,
                         "quantize_us": round(q_us, 2),
                         "quantize_gbs": round((2.0 * m_tok * k + m_tok * k * 0.5625) / q_us / 1e3, 1)})
            del x, fp4, sf, c
        del ws
    out["prefill_gemm"] = gemm
    # ---- fused producers of quantised activations (decode: one vector per call) -------------
    hid, inter = synth.HIDDEN, 17408
    xn = torch.randn(hid, generator=gen, device="cuda").to(torch.bfloat16)
    wn = (torch.randn(hid, generator=gen, device="cuda") * 0.1).to(torch.bfloat16)
    rn = torch.randn(hid, generator=gen, device="cuda").to(torch.bfloat16)
    gt = (torch.randn(inter, generator=gen, device="cuda") * 2).to(torch.bfloat16)
    up = torch.randn(inter, generator=gen, device="cuda").to(torch.bfloat16)
    sw = backend.swiglu_nvfp4_quantize(gt, up, 0.37)
    nb = backend.rmsnorm_nvfp4_quantize(xn, wn, rn, 1e-6, 0.37, True, True)
    norm_us = _time_cuda(torch, lambda i: backend.rmsnorm_nvfp4_quantize(xn, wn, rn, 1e-6, 0.37, True, True, nb), 200,
                         warm=20, backend=backend)
    swiglu_us = _time_cuda(torch, lambda i: backend.swiglu_nvfp4_quantize(gt, up, 0.37, *sw), 200, warm=20,
                           backend=backend)
    out["fused_producers"] = {"rmsnorm_nvfp4_quantize_us": round(norm_us, 2), "hidden": hid,
                              "swiglu_nvfp4_quantize_us": round(swiglu_us, 2), "intermediate": inter}
    # prefill form: silu(gate) * up of a [M, 2 * 17408] GEMM output straight to the down projection's NVFP4
    # operand (qwen36_swiglu_nvfp4_quantize_rows); beside it the quantiser alone on a bf16 [M, 17408] block,
    # which is the second half of the unfused chain.  Three input blocks in rotation (M = 8192: 1.7 GB > L2).
    rows_out = []
    for m_tok in (2048, 8192):
        gus = [(torch.randn((m_tok, 2 * inter), generator=gen, device="cuda")).to(torch.bfloat16) for _ in range(3)]
        res = backend.swiglu_nvfp4_quantize_rows(gus[0][:, :inter], gus[0][:, inter:], 0.37)
        fused_us = _time_cuda(torch, lambda i: backend.swiglu_nvfp4_quantize_rows(gus[i % 3][:, :inter], gus[i % 3][:, inter:],
                                                                                  0.37, *res), 60, warm=10, backend=backend)
        byts = m_tok * inter * (4 + 0.5 + 1 / 16)
        rows_out.append({"M": m_tok, "us": round(fused_us, 1), "gbs": round(byts / fused_us / 1e3, 1),
                         "unfused_bf16_round_trip_bytes": m_tok * inter * 4})
        del gus, res
    out["fused_producers"]["swiglu_nvfp4_quantize_rows"] = rows_out
    # ---- config 3: FP8 lm_head + greedy argmax ---------------------------------------------
    rows, cols = synth.VOCAB, synth.HIDDEN
    w = torch.randint(0, 0x7F, (rows, cols), generator=gen, dtype=torch.uint8, device="cuda")
    w |= (torch.randint(0, 2, (rows, cols), generator=gen, dtype=torch.uint8, device="cuda") << 7)
    sc = torch.exp2(torch.rand(rows, generator=gen, device="cuda") * 4 - 6)
    lm = []
    for m_tok in (1, 4):
        xh = torch.randn((m_tok, cols), generator=gen, device="cuda").to(torch.bfloat16)
        logits = torch.empty((m_tok, rows), dtype=torch.bfloat16, device="cuda")
        wsb = backend.lm_head_argmax_workspace(rows, m_tok, "cuda")
        tok = torch.empty(m_tok, dtype=torch.int32, device="cuda")
        best = torch.empty(m_tok, dtype=torch.float32, device="cuda")
        byts = rows * cols + 4 * rows + 2 * m_tok * cols + 8 * m_tok
        us_gemv = _time_cuda(torch, lambda i: backend.lm_head_fp8_gemv(w, sc, xh, logits), 200, warm=20, backend=backend)
        us_samp = _time_cuda(torch, lambda i: backend.sample_rows(logits), 200, warm=20, backend=backend)
        us_fused = _time_cuda(torch, lambda i: backend.lm_head_fp8_gemv_argmax(w, sc, xh, wsb, 0, tok, best), 200,
                              warm=20, backend=backend)
        lm.append({"M": m_tok, "gemv_us": round(us_gemv, 1), "sample_rows_us": round(us_samp, 1),
                   "fused_us": round(us_fused, 1), "fused_gbs": round(byts / us_fused / 1e3, 1),
                   "gemv_gbs": round(byts / us_gemv / 1e3, 1)})
    out["lm_head_fp8"] = lm
    del w, sc
    # ---- the reference's NVFP4 lm_head: its W4A4 GEMM at m = vocabulary, n <= 16 (one token: decode GEMV) ----
    packed_v, sf_rm_v = synth.nvfp4_weight_device(gen, rows, cols, "cuda")
    sfa_v = backend.nvfp4_retile_scales(sf_rm_v)
    del sf_rm_v
    scan = []
    for m_tok in (1, 4, 16):
        xq = torch.randn((m_tok, cols), generator=gen, device="cuda").to(torch.bfloat16)
        fp4_v, sfb_v, _ = backend.nvfp4_quantize_rows(xq, 0.37)
        c_v = torch.empty((m_tok, rows), dtype=torch.bfloat16, device="cuda")
        us = _time_cuda(torch, lambda i: backend.nvfp4_gemm(packed_v, sfa_v, fp4_v, sfb_v, 0.37 / 2688.0, rows, m_tok,
                                                            cols, c_v), 100, warm=10, backend=backend)
        byts = rows * cols / 2 + rows * cols / 16 + m_tok * (cols / 2 + cols / 16) + 2 * m_tok * rows
        scan.append({"M": m_tok, "us": round(us, 1), "gbs": round(byts / us / 1e3, 1)})
    out["nvfp4_lm_head_scan"] = scan
    del packed_v, sfa_v
    # ---- exact-argmax guards: margin verdict over the logits, predicated bf16 lm_head ---------
    guard = {}
    logits4 = (torch.randn((4, rows), generator=gen, device="cuda") * 3).to(torch.bfloat16)
    guard["top2_margin_rows4_us"] = round(_time_cuda(torch, lambda i: backend.lm_head_top2_margin(logits4, 0.5), 200,
                                                     warm=20, backend=backend), 2)
    wb = torch.randn((rows, cols), generator=gen, device="cuda").to(torch.bfloat16)       # 2.5 GB bf16 lm_head
    for m_tok in (1, 4):
        xh = torch.randn((m_tok, cols), generator=gen, device="cuda").to(torch.bfloat16)
        tk = torch.zeros(m_tok, dtype=torch.int32, device="cuda")
        us = _time_cuda(torch, lambda i: backend.bf16_matvec_argmax_rows(xh, wb, tk), 100, warm=20, backend=backend)
        guard[f"bf16_matvec_argmax_rows{m_tok}_us"] = round(us, 1)
        guard[f"bf16_matvec_argmax_rows{m_tok}_gbs"] = round(rows * cols * 2 / us / 1e3, 1)
    lg = logits4[:1].contiguous()
    x1 = torch.randn((1, cols), generator=gen, device="cuda").to(torch.bfloat16)
    guard["top8_rescore_rows1_us"] = round(_time_cuda(torch, lambda i: backend.lm_head_top8_rescore(lg, wb, x1, 0.5), 200,
                                                      warm=20, backend=backend), 2)
    out["lm_head_guards"] = guard
    del wb, logits4
    # ---- config 4: int8 KV + decode attention ----------------------------------------------
    att = []
    T = 131072
    k_ = torch.randn((T, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
    v_ = torch.randn((T, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
    q_ = torch.randn((24, 256), generator=gen, device="cuda").to(torch.bfloat16)
    kq = torch.empty((T, 4, 256), dtype=torch.int8, device="cuda")
    vq = torch.empty_like(kq)
    meta = torch.empty((T, 4, 2), dtype=torch.float32, device="cuda")
    enc_us = _time_cuda(torch, lambda i: backend.turboquant_encode_kv_rows(k_, v_, kq, vq, meta, 0), 100, warm=20,
                        backend=backend)
    enc_bytes = T * (2 * 4 * 256 * 2 + 2 * 4 * 256 + 32)
    wsa = backend.attention_workspace(24, 256, "cuda")
    o_ = torch.empty((24, 256), dtype=torch.bfloat16, device="cuda")
    # a second 131072-row cache so that ctx 131072 alternates between two caches (2 x 273 MB) and the
    # shorter contexts rotate over 32 / 8 disjoint slices: every launch reads rows that are not in L2
    kq2, vq2, meta2 = kq.flip(0).contiguous(), vq.flip(0).contiguous(), meta.flip(0).contiguous()
    caches = ((kq, vq, meta), (kq2, vq2, meta2))
    for ctx in (8192, 32768, 131072):
        nsl = T // ctx

        def call(i, ctx=ctx, nsl=nsl):
            ck, cv, cm = caches[(i // nsl) & 1]
            s0 = (i % nsl) * ctx
            backend.turboquant_attention(q_, ck[s0:s0 + ctx], cv[s0:s0 + ctx], cm[s0:s0 + ctx], ctx - 1, wsa, o_)
        us = _time_cuda(torch, call, 200, warm=20, backend=backend)
        byts = ctx * (2 * 4 * 256 + 4 * 2 * 4) + 24 * 256 * 4
        att.append({"ctx": ctx, "us": round(us, 2), "gbs": round(byts / us / 1e3, 1)})
    del kq2, vq2, meta2, caches
    out["int8_kv_attention"] = att
    # ---- the same decode step over the FP8 (E4M3) and BF16 caches of qwen36_attention_decode:
    # ctx - 1 cached rows + the new row, cache append included; small contexts rotate over
    # slices of a 131072-row cache so that every call reads cold rows (>= 268 MB per round)
    del k_, v_
    dec = {}
    kn = torch.randn((4, 256), generator=gen, device="cuda").to(torch.bfloat16)
    parts = (torch.empty((24, 256, 256), device="cuda"), torch.empty((24, 256), device="cuda"),
             torch.empty((24, 256), device="cuda"))
    for name, code, width in (("fp8", 1, 1), ("bf16", 0, 2)):
        if code == 1:
            ck = torch.randint(0, 0x78, (T, 4, 256), generator=gen, dtype=torch.uint8, device="cuda")
            ck |= torch.randint(0, 2, (T, 4, 256), generator=gen, dtype=torch.uint8, device="cuda") << 7
            ck = (ck & 0xBF) | 0x20                                  # exponents 4..7: magnitudes 2^-3 .. 1.9
            cv = ck.flip(0).contiguous()
        else:
            ck = torch.randn((T, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
            cv = torch.randn((T, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
        rows_ = []
        for ctx in (8192, 32768, 131072):
            nsl = T // ctx
            def call(i, ctx=ctx, nsl=nsl, ck=ck, cv=cv, code=code):
                s0 = (i % nsl) * ctx
                backend.attention_decode(q_, kn, kn, ck[s0:s0 + ctx], cv[s0:s0 + ctx], ctx - 1, code, parts, 256,
                                         out=o_)
            us = _time_cuda(torch, call, 200, warm=20, backend=backend)
            byts = (ctx - 1) * 2 * 4 * 256 * width + 2 * 24 * 256 * 2 + 4 * 4 * 256 * 2
            rows_.append({"ctx": ctx, "us": round(us, 2), "gbs": round(byts / us / 1e3, 1)})
        dec[name] = rows_
        # speculative verify: 4 / 16 query tokens over the same caches (qwen36_attention_flash_splitk_prefill_bf16)
        ver = []
        for q_tok in (4, 16):
            qv = torch.randn((q_tok, 24, 256), generator=gen, device="cuda").to(torch.bfloat16)
            ov = torch.empty((q_tok, 24, 256), dtype=torch.bfloat16, device="cuda")
            ns = backend.attention_verify_splits(q_tok, 24, 4, torch.cuda.get_device_properties(0).multi_processor_count)
            pv = (torch.empty((q_tok, 24, ns, 256), device="cuda"), torch.empty((q_tok, 24, ns), device="cuda"),
                  torch.empty((q_tok, 24, ns), device="cuda"))
            for ctx in (32768, 131072):
                nsl = max(1, (T - 64) // ctx)

                def vcall(i, ctx=ctx, nsl=nsl):
                    s0 = (i % nsl) * ctx
                    backend.attention_flash_splitk_prefill(qv, ck[s0:], cv[s0:], ctx - q_tok, code, ns, pv, out=ov)
                us = _time_cuda(torch, vcall, 50, warm=10, backend=backend)
                ver.append({"q_tokens": q_tok, "ctx": ctx, "n_splits": ns, "us": round(us, 1),
                            "gbs": round(ctx * 2 * 4 * 256 * width / us / 1e3, 1)})
        dec[name + "_verify"] = ver
        del ck, cv
    out["kv_decode_attention"] = dec
    out["int8_kv_encode"] = {"tokens": T, "us": round(enc_us, 1), "gbs": round(enc_bytes / enc_us / 1e3, 1)}
    return out


def profile_case(name: str):
    """Runs one small, fixed case of a single kernel a few times (for `ncu -k ... -c ...`):
    gemv_gate_up | gemv_down | gemm_gate_up_2048 | gemm_down_2048 | lm_head_m1 | lm_head_m4 |
    attention_32768 | quantize_2048 | bf16_argmax_m1 | bf16_argmax_m4 | decode_fp8_32768 | decode_bf16_32768 |
    verify_fp8_32768 | verify_bf16_32768 | gemv_sweep_layer | swiglu_rows_2048 | kv_encode_65536.  Inputs exceed L2
    but stay well under a few GB."""
    import torch
    from speedoza_b200 import synth
    from speedoza_b200.backend import CudaBackend
    torch.cuda.set_device(0)
    b = CudaBackend()
    gen = torch.Generator(device="cuda").manual_seed(11)
    if name.startswith("gemv_"):
        n, k = (34816, 5120) if name == "gemv_gate_up" else (5120, 17408)
        mats = []
        for _ in range(3):
            p, sf = synth.nvfp4_weight_device(gen, n, k, "cuda")
            mats.append((p, b.nvfp4_retile_scales(sf)))
        ts = torch.tensor([synth.WEIGHT_GLOBAL_SCALE], device="cuda")
        x = torch.randn(k, generator=gen, device="cuda").to(torch.bfloat16)
        y = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        for i in range(6):
            b.nvfp4_matvec(x, mats[i % 3][0], mats[i % 3][1], ts, y)
    elif name.startswith("gemm_"):
        n, k = (34816, 5120) if "gate_up" in name else (5120, 17408)
        m_tok = int(name.rsplit("_", 1)[1])
        ws = []
        for _ in range(2):
            p, sf = synth.nvfp4_weight_device(gen, n, k, "cuda")
            ws.append((p, b.nvfp4_retile_scales(sf)))
        x = torch.randn((m_tok, k), generator=gen, device="cuda").to(torch.bfloat16)
        fp4, sfb, ts = b.nvfp4_quantize_rows(x, 0.37)
        c = torch.empty((m_tok, n), dtype=torch.bfloat16, device="cuda")
        for i in range(4):
            b.nvfp4_gemm(ws[i & 1][0], ws[i & 1][1], fp4, sfb, 0.37 / 2688.0, n, m_tok, k, c)
    elif name.startswith("lm_head_"):
        m_tok = 1 if name.endswith("m1") else 4
        rows, cols = synth.VOCAB, synth.HIDDEN
        w = torch.randint(0, 0x7F, (rows, cols), generator=gen, dtype=torch.uint8, device="cuda")
        sc = torch.exp2(torch.rand(rows, generator=gen, device="cuda") * 4 - 6)
        xh = torch.randn((m_tok, cols), generator=gen, device="cuda").to(torch.bfloat16)
        ws = b.lm_head_argmax_workspace(rows, m_tok, "cuda")
        for _ in range(3):
            b.lm_head_fp8_gemv_argmax(w, sc, xh, ws)
    elif name.startswith("attention_"):
        ctx = int(name.rsplit("_", 1)[1])
        k_ = torch.randn((ctx, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
        v_ = torch.randn((ctx, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
        q_ = torch.randn((24, 256), generator=gen, device="cuda").to(torch.bfloat16)
        kq = torch.empty((ctx, 4, 256), dtype=torch.int8, device="cuda"); vq = torch.empty_like(kq)
        meta = torch.empty((ctx, 4, 2), dtype=torch.float32, device="cuda")
        b.turboquant_encode_kv_rows(k_, v_, kq, vq, meta, 0)
        ws = b.attention_workspace(24, 256, "cuda")
        for _ in range(3):
            b.turboquant_attention(q_, kq, vq, meta, ctx - 1, ws)
    elif name.startswith("decode_fp8_") or name.startswith("decode_bf16_"):
        ctx = int(name.rsplit("_", 1)[1])
        fp8 = name.startswith("decode_fp8_")
        caches = []
        for _ in range(3):                                          # three caches in turn: every launch reads cold rows
            if fp8:
                c = torch.randint(0x20, 0x40, (ctx, 4, 256), generator=gen, dtype=torch.uint8, device="cuda")
            else:
                c = torch.randn((ctx, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
            caches.append(c)
        q_ = torch.randn((24, 256), generator=gen, device="cuda").to(torch.bfloat16)
        kn = torch.randn((4, 256), generator=gen, device="cuda").to(torch.bfloat16)
        parts = (torch.empty((24, 256, 256), device="cuda"), torch.empty((24, 256), device="cuda"),
                 torch.empty((24, 256), device="cuda"))
        for i in range(3):
            b.attention_decode(q_, kn, kn, caches[i], caches[(i + 1) % 3], ctx - 1, 1 if fp8 else 0, parts, 256)
    elif name.startswith("verify_fp8_") or name.startswith("verify_bf16_"):
        ctx = int(name.rsplit("_", 1)[1])
        fp8 = name.startswith("verify_fp8_")
        caches = []
        for _ in range(3):
            if fp8:
                c = torch.randint(0x20, 0x40, (ctx, 4, 256), generator=gen, dtype=torch.uint8, device="cuda")
            else:
                c = torch.randn((ctx, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
            caches.append(c)
        qv = torch.randn((4, 24, 256), generator=gen, device="cuda").to(torch.bfloat16)
        for i in range(3):
            b.attention_flash_splitk_prefill(qv, caches[i], caches[(i + 1) % 3], ctx - 4, 1 if fp8 else 0,
                                             b.attention_verify_splits(4, 24, 4))
    elif name.startswith("gemv_sweep_layer"):
        # one decode layer (4 launches: q_gate + k + v grouped, o, gate_up, down), three times over cold weights
        layers = []
        for _ in range(3):
            mats = []
            for _, n, k in synth.DECODE_SHAPES:
                p_, sf = synth.nvfp4_weight_device(gen, n, k, "cuda")
                mats.append((p_, b.nvfp4_retile_scales(sf), torch.empty(n, dtype=torch.bfloat16, device="cuda")))
            layers.append(mats)
        ts = torch.tensor([synth.WEIGHT_GLOBAL_SCALE], device="cuda")
        x = torch.randn(5120, generator=gen, device="cuda").to(torch.bfloat16)
        for mats in layers:
            b.nvfp4_matvec_group(x, [(m[0], m[1], ts, m[2]) for m in mats[:3]])
            b.nvfp4_matvec(mats[0][2][:6144], mats[3][0], mats[3][1], ts, mats[3][2])
            b.nvfp4_matvec(mats[3][2], mats[4][0], mats[4][1], ts, mats[4][2])
            b.nvfp4_matvec(mats[4][2][:17408], mats[5][0], mats[5][1], ts, mats[5][2])
    elif name.startswith("bf16_argmax_m"):
        m_tok = int(name.rsplit("m", 1)[1])
        rows, cols = synth.VOCAB, synth.HIDDEN
        wb = torch.randn((rows, cols), generator=gen, device="cuda").to(torch.bfloat16)
        xh = torch.randn((m_tok, cols), generator=gen, device="cuda").to(torch.bfloat16)
        tk = torch.zeros(m_tok, dtype=torch.int32, device="cuda")
        for _ in range(3):
            b.bf16_matvec_argmax_rows(xh, wb, tk)
    elif name.startswith("quantize_"):
        m_tok = int(name.rsplit("_", 1)[1])
        x = torch.randn((m_tok, 17408), generator=gen, device="cuda").to(torch.bfloat16)
        for _ in range(3):
            b.nvfp4_quantize_rows(x, 0.37)
    elif name.startswith("swiglu_rows_"):
        m_tok = int(name.rsplit("_", 1)[1])
        gu = torch.randn((m_tok, 2 * 17408), generator=gen, device="cuda").to(torch.bfloat16)
        for _ in range(3):
            b.swiglu_nvfp4_quantize_rows(gu[:, :17408], gu[:, 17408:], 0.37)
    elif name.startswith("kv_encode_"):
        tokens = int(name.rsplit("_", 1)[1])
        kk = torch.randn((tokens, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
        vv = torch.randn((tokens, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
        kq = torch.empty((tokens, 4, 256), dtype=torch.int8, device="cuda")
        vq = torch.empty_like(kq)
        meta = torch.empty((tokens, 4, 2), dtype=torch.float32, device="cuda")
        for _ in range(3):
            b.turboquant_encode_kv_rows(kk, vv, kq, vq, meta, 0)
    else:
        raise SystemExit(f"unknown profile case {name}")
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": name, "status": "ok"}))


def backend_tiled_bytes(rows, groups):
    from speedoza_b200.backend import tiled_scale_bytes
    return tiled_scale_bytes(rows, groups)


def cpu_baseline(seconds: float = 10.0):
    """Oracle W4A16 matvec on the host cores, 5120 x 5120 shape repeated for ~`seconds`."""
    import numpy as np
    from oracle import oracle as orc
    from speedoza_b200 import synth
    orc.set_num_threads(os.cpu_count() or 1)       # all host cores, whatever OMP_NUM_THREADS says
    rng = np.random.default_rng(0)
    n = k = 5120
    packed, sf_rm = synth.nvfp4_weight(rng, n, k)
    sf = orc.retile_scales(sf_rm)
    x = synth.activations(rng, 1, k)[0]
    orc.nvfp4_matvec(x, packed, sf, synth.WEIGHT_GLOBAL_SCALE, k)
    t0 = time.perf_counter()
    reps = 0
    while time.perf_counter() - t0 < seconds:
        orc.nvfp4_matvec(x, packed, sf, synth.WEIGHT_GLOBAL_SCALE, k)
        reps += 1
    dt = time.perf_counter() - t0
    return {"value": round(gemv_bytes(n, k) * reps / dt / 1e9, 3), "unit": "GB/s", "cores": orc.num_threads(),
            "kind": "port", "sample": f"{reps} x W4A16 GEMV 5120x5120 (config 0 shape), OpenMP oracle, {dt:.1f} s"}


def run_ours(args):
    import torch
    from speedoza_b200 import synth
    from speedoza_b200.backend import CudaBackend

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    backend = CudaBackend()
    layers = args.layers
    # The M = 1 decode sweep is a chain of 384 dependent GEMVs of a few microseconds each: splitting
    # every matrix across GPUs puts a collective on each link of that chain and is slower than one
    # GPU (measured, `--workload sweep_split`).  At N > 1 the default is therefore N independent
    # decode streams, one full model replica per GPU, no data-path collective ("replicas only").
    split = world > 1 and args.workload == "sweep_split"
    shard_world = world if split else 1
    sweep = build_sweep(backend, torch, synth, rank if split else 0, shard_world, layers, seed=1234)
    runner = SweepRunner(backend, torch, sweep, shard_world, dist)
    step_bytes = layers * sum(gemv_bytes(n, k) for _, n, k in synth.DECODE_SHAPES)
    if world > 1 and not split:
        step_bytes *= world                      # every rank streams its own replica
    launches_per_step = layers * (4 if shard_world == 1 else len(synth.DECODE_SHAPES))

    gen = torch.Generator(device="cuda").manual_seed(99 + (0 if split else rank))     # replicas: own hidden state
    x_dev = torch.randn(5120, generator=gen, device="cuda").to(torch.bfloat16)
    x_host = x_dev.cpu().pin_memory()
    y_host = torch.empty(5120, dtype=torch.bfloat16).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ------------------------------------------------
    runner.step(x_dev)                       # eager once: lazy one-time setup happens outside capture
    barrier()
    use_graph = not args.no_graph
    if use_graph:
        try:
            per_step = runner.capture()
            run_step = runner.replay
        except Exception as exc:                 # capture refused (e.g. a collective): same launches, eagerly
            print(f"[bench] graph capture failed on rank {rank}: {exc!r}; running eagerly", file=sys.stderr, flush=True)
            backend.sync_stream()
            use_graph = False
            per_step = launches_per_step
            run_step = runner.step
    else:
        per_step = launches_per_step
        run_step = runner.step
    launches_per_step = per_step
    for _ in range(args.warmup):
        run_step(x_dev)
    barrier()
    try:
        props = torch.cuda.get_device_properties(torch.cuda.current_device())
        bus = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
    except AttributeError:
        bus = None
    sampler = ClockSampler(local_rank, bus)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        y = run_step(x_dev)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    gpu_launches = per_step * args.steps * (world if (world > 1 and not split) else 1)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end: host buffers in, host result out, every step ---------------
    barrier()
    t0 = time.perf_counter()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for _ in range(args.steps):
        y = run_step(x_host)                               # pinned host -> device inside the step
        y_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()          # the caller reads the result
    e3.record()
    barrier()
    ms_e2e = e2.elapsed_time(e3)
    wall_e2e = (time.perf_counter() - t0) * 1e3

    if world > 1:
        t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])

    extra = {}
    if rank == 0 and world == 1 and not args.no_extras:
        extra["per_shape_cold"] = per_shape_cold(backend, torch, sweep, synth)
        extra["per_shape_w4a4_decode"] = per_shape_w4a4_decode(backend, torch, sweep, synth)
        run_step = None
        try:
            del runner.graph
        except AttributeError:
            pass
        del runner, sweep
        torch.cuda.empty_cache()
        extra.update(other_configs(backend, torch, synth, make_sampler=lambda: ClockSampler(local_rank, bus)))
    if world > 1 and not split and not args.no_extras:
        # north_star's sharded paths at this GPU count, in the same line (strong scaling each)
        try:
            del runner.graph
        except AttributeError:
            pass
        run_step = None
        del runner, sweep
        torch.cuda.empty_cache()
        extra["sharded"] = sharded_suite(backend, torch, dist, world, rank, layers)
    if rank == 0:
        peak, peak_kind = measured_peaks()
        ms_per_step = ms / args.steps
        value = step_bytes / (ms_per_step * 1e-3) / 1e9
        e2e_value = step_bytes / (ms_e2e / args.steps * 1e-3) / 1e9
        per_gpu_bytes = step_bytes // (world if (world > 1 and not split) else 1)
        launch_us = ms_per_step * 1e3 / launches_per_step
        achieved = (per_gpu_bytes / launches_per_step) / (launch_us * 1e-6) / 1e9
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "strong" if split else "weak", "vs_baseline": None, "dtype": "e2m1 x bf16 -> f32",
            "data": "synthetic",
            "config": {"workload": f"config 1: NVFP4 W4A16 decode GEMV sweep, {layers} layers x 6 shapes, M=1",
                       "launch": ("CUDA graph replay of the C-ABI calls" if use_graph else "eager C-ABI calls") +
                                 ("; q_gate + k + v (shared input) as one grouped launch: 4 launches per layer"
                                  if shard_world == 1 else ""),
                       "bytes_per_step": step_bytes, "l2": "inputs larger than L2 (13.4 GB of weights per step)",
                       "parallelism": "1 GPU" if world == 1 else (
                           f"output rows split {world}-way + NCCL all-gather per GEMV" if split else
                           f"replicas only: {world} independent decode streams, one model replica per GPU, no collective")},
            "gpu_launches": gpu_launches,
            "e2e": {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": y_host.numel() * 2, "ms_per_step": round(ms_e2e / args.steps, 4),
                    "wall_ms_per_step": round(wall_e2e / args.steps, 4)},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4),
                         # DRAM bytes per launch: ncu measured 100.33 MB read + 4.02 MB written for the
                         # 100.35 MB gate_up launch (profiles/nvfp4_gemv_mma_gate_up.md); the sweep's
                         # launches are too many to capture whole, so that ratio is applied to the
                         # average launch (traffic grows with the units processed)
                         "traffic": int(per_gpu_bytes // launches_per_step * NCU_TRAFFIC_RATIO),
                         "traffic_source": "ncu, gate_up launch, scaled by bytes", "peak_kind": peak_kind,
                         "kernel": "nvfp4_gemv_mma_kernel", "launch_us": round(launch_us, 3),
                         "bytes_per_launch": per_gpu_bytes // launches_per_step,
                         "frac_of_nominal_8TBs": round(achieved / 8000.0, 4)},
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(args.cpu_seconds)
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave without tearing NCCL down: destroying a communicator that captured graphs still
        # reference was seen to block at exit.  Everything has been synchronised and printed.
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def peer_combine_usable(make, torch, dist, world):
    """Builds a sharded operator with the NVLink peer-memory combine; every rank falls back to the
    collective together when the peer mapping is refused on any of them."""
    from speedoza_b200.abi import KernelError
    try:
        return make("peer"), "NVLink peer push (one kernel)"
    except KernelError:
        return make("collective"), "all-gather (NCCL)"


def _rotation(shard_bytes: int, cap: int = 64) -> int:
    """How many disjoint copies / slices of a per-rank shard a step sequence rotates over so that
    every launch reads rows that have left L2 (126 MB): >= 300 MB in rotation."""
    return max(1, min(cap, -(-300_000_000 // max(1, shard_bytes))))


def _time_sequence(steps_fns, steps, warmup, b, torch, dist, world):
    """Times a sequence of step callables (one per cold slice).  The whole sequence is recorded into
    ONE CUDA graph (kernels + combine, the way a serving engine replays its step) and replayed until
    at least `steps` steps have run; every rank takes the same route.  Returns (ms per step, route)."""
    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    seq = len(steps_fns)
    for i in range(max(3, warmup)):
        steps_fns[i % seq]()
    barrier()
    graph = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, capture_error_mode="thread_local" if world > 1 else "global"):
            b.sync_stream()
            for fn in steps_fns:
                fn()
        b.sync_stream()
    except Exception:
        graph = None
        b.sync_stream()
    if world > 1:
        flag = torch.tensor([1 if graph is not None else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag[0]) == 0:
            graph = None

    def run():
        if graph is not None:
            graph.replay()
        else:
            for fn in steps_fns:
                fn()
    reps = max(1, -(-steps // seq))
    for _ in range(2):
        run()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    route = "CUDA graph replay" if graph is not None else "eager"
    del graph
    return ms / (reps * seq), route


def measure_sharded(workload, tokens, steps, warmup, b, torch, dist, world, rank, combine="peer", shape="gate_up",
                    gather=False, quantise="replicated"):
    """One sharded configuration at `world` GPUs (strong scaling: the total work is fixed, each rank
    holds 1/world of the vocab rows, of the KV range, or of the weight rows).  Every step of the
    timed sequence reads a different copy / slice of the rank's shard, so the figures are cold-HBM
    ones at every N.  Returns a dict."""
    from speedoza_b200 import shard, synth
    how = None
    closers = []
    gen = torch.Generator(device="cuda").manual_seed(4321)
    if workload == "lm_head":
        m_tok = tokens or 4
        rows, cols = synth.VOCAB, synth.HIDDEN
        lo, hi = shard.shard_rows(rows, rank, world)
        copies = min(4, _rotation((hi - lo) * cols))
        gen.manual_seed(100 + rank)
        w = torch.randint(0, 0x7F, (hi - lo, cols), generator=gen, dtype=torch.uint8, device="cuda")
        sc = torch.exp2(torch.rand(hi - lo, generator=gen, device="cuda") * 4 - 6)
        ws_ = [w] + [w.roll(17 * (c + 1), 0) for c in range(copies - 1)]
        scs = [sc] + [sc.roll(17 * (c + 1), 0) for c in range(copies - 1)]
        gen.manual_seed(7)
        x = torch.randn((m_tok, cols), generator=gen, device="cuda").to(torch.bfloat16)
        make = lambda c, i=0: shard.ShardedLmHead(b, rows, ws_[i], scs[i], lo, world, m_tok, combine=c)
        head, how = peer_combine_usable(make, torch, dist, world) if (combine == "peer" and world > 1) else \
            (make("collective"), "all-gather (NCCL)" if world > 1 else None)
        if how is not None and how.startswith("NVLink"):
            want = make("collective").argmax(x).to(torch.int64)      # the two combines must agree
            got = head.argmax(x).to(torch.int64)
            assert torch.equal(want, got), "peer argmax combine differs from the collective one"

        def lm_step(i):
            def fn():
                head.w, head.s = ws_[i], scs[i]
                return head.argmax(x)
            return fn
        fns = [lm_step(i) for i in range(copies)]
        closers.append(head)
        work, unit = rows * cols + 4 * rows + 2 * m_tok * cols + 8 * m_tok, "GB/s"
        name = (f"config 3: FP8 lm_head 248320x5120 + fused greedy argmax, M={m_tok}, vocab split {world}-way "
                f"+ combine of (value, index); {copies} weight copies in rotation")
        dtype = "e4m3 x bf16 -> f32"
    elif workload == "attention":
        ctx = tokens or 131072
        lo, hi = shard.shard_tokens(ctx, rank, world)
        n_loc = hi - lo
        slices = _rotation(n_loc * 2080)
        gen.manual_seed(200 + rank)
        pool = n_loc * slices
        kq = torch.empty((pool, 4, 256), dtype=torch.int8, device="cuda")
        vq = torch.empty_like(kq)
        meta = torch.empty((pool, 4, 2), dtype=torch.float32, device="cuda")
        for s0 in range(0, pool, 32768):                          # encode in pieces: small bf16 temporaries
            n = min(32768, pool - s0)
            k_ = torch.randn((n, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
            v_ = torch.randn((n, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
            b.turboquant_encode_kv_rows(k_, v_, kq[s0:s0 + n], vq[s0:s0 + n], meta[s0:s0 + n], 0)
        del k_, v_
        gen.manual_seed(7)
        q_ = torch.randn((24, 256), generator=gen, device="cuda").to(torch.bfloat16)
        make = lambda c: shard.ShardedKvAttention(b, kq[:n_loc], vq[:n_loc], meta[:n_loc], lo, world, 24, 256, combine=c)
        att, how = peer_combine_usable(make, torch, dist, world) if (combine == "peer" and world > 1) else \
            (make("collective"), "all-gather (NCCL)" if world > 1 else None)
        if how is not None and how.startswith("NVLink"):
            want = make("collective").attend(q_, ctx - 1).float()    # same arithmetic, same order: same bits
            got = att.attend(q_, ctx - 1).float()
            assert torch.equal(want, got), "peer attention merge differs from the collective one"

        def att_step(i):
            def fn():
                s0 = i * n_loc
                att.kq, att.vq, att.meta = kq[s0:s0 + n_loc], vq[s0:s0 + n_loc], meta[s0:s0 + n_loc]
                return att.attend(q_, ctx - 1)
            return fn
        fns = [att_step(i) for i in range(slices)]
        closers.append(att)
        work, unit = ctx * (2 * 4 * 256 + 32) + 24 * 256 * 4, "GB/s"
        name = (f"config 4: int8 KV decode attention, ctx {ctx}, 24 q / 4 kv heads, KV range split {world}-way "
                f"+ merge of (m, l, o); {slices} cache slices in rotation")
        dtype = "int8 x bf16 -> f32"
    else:
        m_tok = tokens or 8192
        n_out, k = (34816, 5120) if shape == "gate_up" else (5120, 17408)
        lo, hi = shard.shard_rows(n_out, rank, world)
        n_loc = hi - lo
        copies = min(32, _rotation(n_loc * k // 2))
        gen.manual_seed(300 + rank)
        packed, sf_rm = synth.nvfp4_weight_device(gen, n_loc, k, "cuda")
        a_sf = b.nvfp4_retile_scales(sf_rm)
        wts = [(packed, a_sf)] + [(packed.roll(c + 1, 0), a_sf.roll(512 * (c + 1), 0)) for c in range(copies - 1)]
        gen.manual_seed(7)
        x = torch.randn((m_tok, k), generator=gen, device="cuda").to(torch.bfloat16)
        fp4 = torch.empty((m_tok, k // 2), dtype=torch.uint8, device="cuda")
        sfb = torch.zeros(backend_tiled_bytes(m_tok, k // 16), dtype=torch.uint8, device="cuda")
        ts = torch.empty(1, dtype=torch.float32, device="cuda")
        c = torch.empty((m_tok, n_loc), dtype=torch.bfloat16, device="cuda")
        even = world > 1 and n_loc * world == n_out
        gather = gather and even
        full = torch.empty((world, m_tok, n_loc), dtype=torch.bfloat16, device="cuda") if gather else None
        # activation quantisation: every rank quantises all M rows ("replicated", no exchange), or each
        # rank quantises M / world rows and the codes + scale tiles are all-gathered ("sharded")
        rows_loc = m_tok // world
        split_q = quantise == "sharded" and world > 1 and rows_loc % 128 == 0
        if split_q:
            r0 = rank * rows_loc
            sf_rows = backend_tiled_bytes(rows_loc, k // 16)
            fp4_loc, sf_loc = fp4[r0:r0 + rows_loc], sfb[rank * sf_rows:(rank + 1) * sf_rows]

        def pre_step(i):
            def fn():
                if split_q:
                    b.nvfp4_quantize_rows(x[r0:r0 + rows_loc], 0.37, fp4_loc, sf_loc, ts)
                    dist.all_gather_into_tensor(fp4.view(-1), fp4_loc.reshape(-1))
                    dist.all_gather_into_tensor(sfb, sf_loc)
                else:
                    b.nvfp4_quantize_rows(x, 0.37, fp4, sfb, ts)
                b.nvfp4_gemm(wts[i][0], wts[i][1], fp4, sfb, 0.37 / 2688.0, n_loc, m_tok, k, c)
                if gather:
                    dist.all_gather_into_tensor(full, c)
                return c
            return fn
        fns = [pre_step(i) for i in range(copies)]
        work, unit = 2.0 * m_tok * n_out * k, "TFLOP/s"
        name = (f"config 2: NVFP4 prefill (quantise + tcgen05 GEMM) {shape} {n_out}x{k}, M={m_tok}, weight rows "
                f"split {world}-way, activation quantise {'sharded + all-gather of codes' if split_q else 'replicated'}, "
                f"output {'all-gathered (bf16, [rank, M, rows] layout)' if gather else 'kept sharded'}; "
                f"{copies} weight copies in rotation")
        dtype = "nvfp4 x nvfp4 -> f32"

    per, launch = _time_sequence(fns, steps, warmup, b, torch, dist, world)
    value = work / (per * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
    del fns
    for op in closers:
        if getattr(op, "peer", None) is not None:
            op.peer.ex.close()                   # unmaps the peers' inboxes (collective: every rank gets here)
    out = {"workload": name, "value": round(value, 1), "unit": unit, "ms_per_step": round(per, 4), "dtype": dtype,
           "launch": launch}
    if how is not None:
        out["combine"] = how
        if int(b.lib.qwen36_peer_last_error()) != 0:
            out["combine"] += "; a wait for a peer ran out"
    return out


class PeerSweepRunner:
    """The sweep with every matrix's output rows split over the ranks and the slices exchanged by the
    GEMV epilogue itself (qwen36_nvfp4_matvec_peer: stores into every rank's arena over NVLink, one
    flag per rank, bounded wait in the consuming launch): 4 launches per layer, no collective."""

    SLOT = {"qkv": 0, "o": 1, "gate_up": 2, "down": 3}

    def __init__(self, backend, torch, sweep, world, rank):
        from speedoza_b200 import synth
        from speedoza_b200.peer import TensorParallelGemv
        self.sweep, self.world, self.rank = sweep, world, rank
        vectors = {name: n for name, n, _ in synth.DECODE_SHAPES}
        self.tp = TensorParallelGemv(backend, vectors, 4, "cuda")
        self.y = torch.empty(5120, dtype=torch.bfloat16, device="cuda")

    def _mat(self, m):
        name, n_local, k, packed, sf, ts, n_full = m
        return (packed, sf, ts, name, shard_rows(n_full, self.rank, self.world)[0])

    def step(self, x0):
        tp, x, src = self.tp, x0, None
        for mats in self.sweep:
            tp.gemv(x, [self._mat(m) for m in mats[:3]], out_slot=0, in_slot=src)
            tp.gemv((mats[0][0], 6144), [self._mat(mats[3])], out_slot=1, in_slot=0)
            tp.gemv((mats[3][0], 5120), [self._mat(mats[4])], out_slot=2, in_slot=1)
            tp.gemv((mats[4][0], 17408), [self._mat(mats[5])], out_slot=3, in_slot=2)
            x, src = (mats[5][0], 5120), 3
        return tp.collect(self.sweep[-1][5][0], 3, self.y)

    def close(self):
        self.tp.close()


def measure_sweep_split(b, torch, dist, world, rank, layers, steps, warmup):
    """The whole decode sweep with every GEMV's output rows split `world`-way (strong scaling), two
    ways: NCCL all-gather after every GEMV, and the peer-store epilogue.  Both must give the bits of
    each other.  Returns two dicts."""
    from speedoza_b200 import synth
    from speedoza_b200.abi import KernelError
    sweep = build_sweep(b, torch, synth, rank, world, layers, seed=1234)
    step_bytes = layers * sum(gemv_bytes(n, k) for _, n, k in synth.DECODE_SHAPES)
    gen = torch.Generator(device="cuda").manual_seed(99)
    x = torch.randn(5120, generator=gen, device="cuda").to(torch.bfloat16)
    out = []
    nccl = SweepRunner(b, torch, sweep, world, dist)
    y_nccl = nccl.step(x).clone()
    per, launch = _time_sequence([lambda: nccl.step(x)], steps, warmup, b, torch, dist, world)
    out.append({"workload": f"config 1: decode sweep, {layers} layers x 6 shapes, output rows split {world}-way, "
                            "NCCL all-gather after every GEMV (6 launches + 6 collectives per layer)",
                "value": round(step_bytes / (per * 1e-3) / 1e9, 1), "unit": "GB/s", "ms_per_step": round(per, 4),
                "dtype": "e2m1 x bf16 -> f32", "launch": launch, "combine": "all-gather (NCCL)"})
    del nccl
    try:
        peer = PeerSweepRunner(b, torch, sweep, world, rank)
    except KernelError:
        peer = None
    if peer is not None:
        y_peer = peer.step(x).clone()
        torch.cuda.synchronize()
        same = bool(torch.equal(y_peer.view(torch.int16), y_nccl.view(torch.int16)))
        per, launch = _time_sequence([lambda: peer.step(x)], steps, warmup, b, torch, dist, world)
        failed = peer.tp.failed_call()
        out.append({"workload": f"config 1: decode sweep, {layers} layers x 6 shapes, output rows split {world}-way, "
                                "GEMV epilogue stores its rows into every rank's activation arena over NVLink "
                                "(4 launches per layer, no collective)",
                    "value": round(step_bytes / (per * 1e-3) / 1e9, 1), "unit": "GB/s", "ms_per_step": round(per, 4),
                    "dtype": "e2m1 x bf16 -> f32", "launch": launch,
                    "combine": "NVLink peer stores from the GEMV epilogue" + ("" if failed == 0 else "; a wait for a peer ran out"),
                    "same_bits_as_all_gather": same})
        peer.close()
    else:
        out.append({"workload": "config 1: decode sweep, peer-store epilogue", "unavailable": "CUDA IPC mapping refused"})
    return out


def sharded_suite(b, torch, dist, world, rank, layers):
    """Every sharded path at this GPU count (strong scaling each), for the scaling record."""
    def guarded(label, fn):
        # a failure (the same on every rank: shapes and routes are) is recorded instead of ending the line
        try:
            return fn()
        except Exception as exc:                              # noqa: BLE001
            b.sync_stream()
            return [{"workload": label, "error": repr(exc)[:200]}]
    out = guarded("config 1: decode sweep, output rows split", lambda: measure_sweep_split(b, torch, dist, world, rank, layers, 10, 3))
    torch.cuda.empty_cache()
    ms = lambda *a, **k: out.extend(guarded(f"{a[0]} {a[1]} {k}", lambda: [measure_sharded(*a, b, torch, dist, world, rank, **k)]))
    for m_tok in (1, 4):
        for c in ("peer", "collective"):
            ms("lm_head", m_tok, 200, 5, combine=c)
            torch.cuda.empty_cache()
    for ctx in (8192, 32768, 131072):
        for c in ("peer", "collective"):
            ms("attention", ctx, 200, 5, combine=c)
            torch.cuda.empty_cache()
    for shape in ("gate_up", "down"):
        for m_tok in (512, 2048, 8192):
            ms("prefill", m_tok, 50, 3, shape=shape)
            ms("prefill", m_tok, 50, 3, shape=shape, gather=True)
            torch.cuda.empty_cache()
    ms("prefill", 8192, 50, 3, shape="down", quantise="sharded")
    return out


def run_sharded_workload(args):
    """--workload lm_head | attention | prefill at N GPUs."""
    import torch
    import torch.distributed as dist
    from speedoza_b200.backend import CudaBackend
    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    b = CudaBackend()
    r = measure_sharded(args.workload, args.tokens, args.steps, args.warmup, b, torch, dist, world, rank,
                        combine=args.combine, shape=args.shape, gather=args.gather, quantise=args.quantise)
    if rank == 0:
        print(json.dumps({"metric": METRIC, "value": r["value"], "unit": r["unit"], "n_gpus": world, "steps": args.steps,
                          "warmup": max(3, args.warmup), "ms_per_step": r["ms_per_step"], "higher_is_better": True,
                          "scaling": "strong", "vs_baseline": None, "dtype": r["dtype"], "data": "synthetic",
                          "config": {"workload": r["workload"], "launch": r["launch"],
                                     "combine": r.get("combine")}}), flush=True)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


# --------------------------------------------------------------------------- reference arm

def run_reference(args):
    """The reference's scalar W4A16 semantics on the host cores (OpenMP oracle).  One step = one
    layer of the sweep (6 GEMVs, 209.6 MB of weights)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import oracle as orc
    from speedoza_b200 import synth
    # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers: the CPU arm uses every host core anyway
    orc.set_num_threads(os.cpu_count() or 1)
    rng = np.random.default_rng(1234)
    mats = []
    for name, n, k in synth.DECODE_SHAPES:
        packed, sf_rm = synth.nvfp4_weight(rng, n, k)
        gain = 2688.0 / (2.926 * 4.80 * (k ** 0.5))
        mats.append((n, k, packed, orc.retile_scales(sf_rm), synth.WEIGHT_GLOBAL_SCALE * gain))
    x0 = synth.activations(rng, 1, 5120)[0]

    def layer(x):
        qg = orc.nvfp4_matvec(x, mats[0][2], mats[0][3], mats[0][4], 5120)
        orc.nvfp4_matvec(x, mats[1][2], mats[1][3], mats[1][4], 5120)
        orc.nvfp4_matvec(x, mats[2][2], mats[2][3], mats[2][4], 5120)
        o = orc.nvfp4_matvec(np.ascontiguousarray(qg[:6144]), mats[3][2], mats[3][3], mats[3][4], 6144)
        gu = orc.nvfp4_matvec(o, mats[4][2], mats[4][3], mats[4][4], 5120)
        return orc.nvfp4_matvec(np.ascontiguousarray(gu[:17408]), mats[5][2], mats[5][3], mats[5][4], 17408)

    x = x0
    for _ in range(args.warmup):
        x = layer(x)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        x = layer(x)
    dt = time.perf_counter() - t0
    layer_bytes = sum(gemv_bytes(n, k) for _, n, k in synth.DECODE_SHAPES)
    value = layer_bytes * args.steps / dt / 1e9
    cores = orc.num_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 3), "unit": "GB/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(dt / args.steps * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "e2m1 x bf16 -> f32", "data": "synthetic",
        "config": {"workload": "config 1: NVFP4 W4A16 decode GEMV sweep; bounded sample: one layer (6 GEMVs) per step",
                   "bytes_per_step": layer_bytes},
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "one layer of the sweep per step, OpenMP oracle (oracle/oracle.c)"},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--workload", default="sweep",
                    choices=["sweep", "sweep_split", "lm_head", "attention", "prefill"])
    ap.add_argument("--combine", default="peer", choices=["peer", "collective"],
                    help="cross-rank combine of the sharded lm_head / attention: NVLink peer push or all-gather")
    ap.add_argument("--tokens", type=int, default=0, help="M (lm_head, prefill) or context length (attention)")
    ap.add_argument("--shape", default="gate_up", choices=["gate_up", "down"], help="prefill workload: which MLP matrix")
    ap.add_argument("--gather", action="store_true", help="prefill workload: all-gather the bf16 output as well")
    ap.add_argument("--quantise", default="replicated", choices=["replicated", "sharded"],
                    help="prefill workload: quantise all rows on every rank, or M / N rows + all-gather of the codes")
    ap.add_argument("--profile-case", default=None, help="run one small kernel case (for ncu) and exit")
    args = ap.parse_args()
    if args.profile_case:
        profile_case(args.profile_case)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload not in ("sweep", "sweep_split"):
        run_sharded_workload(args)
    else:
        if args.warmup < 3:
            args.warmup = max(args.warmup, 1)
        run_ours(args)


if __name__ == "__main__":
    main()
