#!/usr/bin/env python
"""Benchmark of the FP8 quantise / GEMM / grouped-GEMM hot path.

    python bench.py [--config c1|c2|c3|c4|c5] [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of synthetic input, through the public ops
exactly as a caller runs them.  FLOPs counted are the algorithmic 2*M*N*K per GEMM only.

  c4 (default, the headline): blockwise FP8 grouped GEMM at the DeepSeek-V3 expert shape -- 256 experts,
      hidden 7168, gate+up N=4096, 65536 routed rows with per-expert counts drawn from a multinomial
      over softmax(N(0,1) logits), seed 0; forward + dgrad + wgrad through ``grouped_gemm_fp8``:
      activation quantise (1x128 row copy + segment-padded 128x1 column copy), weight quantise
      (128x128 tiles, redone every forward as the reference does), forward GEMM, grad-out quantise,
      dgrad GEMM, wgrad variable-K GEMM.
  c5: the same op at the Qwen3-30B-A3B shape -- 128 experts, hidden 2048, gate+up N=1536, 32768 rows,
      Zipf(1.2) counts with at least 8 empty groups.
  c1: blockwise quantise + GEMM, A [256,1024] x B [512,1024]^T, forward (L2 flushed between steps).
  c2: tensorwise dense GEMM, [8192,4096] x [14336,4096]^T, forward.
  c3: rowwise dense GEMM forward + dgrad + wgrad, X [16384,8192], W [8192,8192].

With N > 1 ranks (c4 / c5) the experts are sharded E/N per GPU, the rows start evenly split over the ranks
and travel to their expert's owner and back (strong scaling).  ``--exchange peer`` (default) writes rows
straight into the owners' IPC-mapped buffers with this library's copy kernel; ``--exchange nccl`` uses
all-to-alls.  ``--placement balanced`` (default) assigns experts to ranks by greedy balancing of the
router's expected load; ``contiguous`` keeps expert e on rank e // (E/N).

Prints ONE JSON line on rank 0.  ``--impl reference`` times the CPU restatement of the reference's
algorithm (oracle/, torch on the host cores) on a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

METRIC = {"c1": "blockwise_fp8_quantize_gemm_throughput", "c2": "tensorwise_fp8_gemm_throughput",
          "c3": "rowwise_fp8_gemm_fwd_dgrad_wgrad_throughput", "c4": "blockwise_fp8_grouped_gemm_throughput",
          "c5": "blockwise_fp8_grouped_gemm_throughput", "mx": "mxfp8_gemm_fwd_dgrad_wgrad_throughput"}
UNIT = "TFLOP/s"
GROUPED = {
    "c4": dict(E=256, K=7168, N=4096, ROWS=65536, counts="softmax",
               workload="deepseek_v3_moe_gate_up_blockwise_fp8_grouped_gemm_fwd_dgrad_wgrad"),
    "c5": dict(E=128, K=2048, N=1536, ROWS=32768, counts="zipf",
               workload="qwen3_30b_a3b_moe_gate_up_blockwise_fp8_grouped_gemm_fwd_dgrad_wgrad"),
}
DENSE = {
    "c1": dict(M=256, N=512, K=1024, gran="blockwise", bwd=False, w_scale=0.02,
               workload="blockwise_fp8_quantize_gemm_256x512x1024_fwd"),
    "c2": dict(M=8192, N=14336, K=4096, gran="tensorwise", bwd=False, w_scale=0.02,
               workload="llama3_8b_mlp_up_tensorwise_fp8_gemm_fwd"),
    "c3": dict(M=16384, N=8192, K=8192, gran="rowwise", bwd=True, w_scale=0.02,
               workload="llama3_70b_attn_out_rowwise_fp8_gemm_fwd_dgrad_wgrad"),
    # an extra configuration: the c3 shape in the MXFP8 format (1x32 blocks, E8M0 scales)
    "mx": dict(M=16384, N=8192, K=8192, gran="mx", bwd=True, w_scale=0.02,
               workload="llama3_70b_attn_out_mxfp8_gemm_fwd_dgrad_wgrad"),
}


def _counts(cfg, seed: int = 0) -> torch.Tensor:
    """Seeded per-expert row counts of the workload (the tests draw the same counts)."""
    g = torch.Generator().manual_seed(seed)
    E, rows = cfg["E"], cfg["ROWS"]
    if cfg["counts"] == "softmax":
        # multinomial over softmax(N(0,1) logits)
        p = torch.softmax(torch.randn(E, generator=g), 0)
        idx = torch.multinomial(p, rows, replacement=True, generator=g)
        return torch.bincount(idx, minlength=E).to(torch.int64)
    # Zipf(s = 1.2) over a seeded permutation of the experts; the 8 smallest groups are emptied into the largest
    perm = torch.randperm(E, generator=g)
    p = torch.arange(1, E + 1, dtype=torch.float64).pow(-1.2)
    p = (p / p.sum()).to(torch.float32)
    pe = torch.empty(E)
    pe[perm] = p
    idx = torch.multinomial(pe, rows, replacement=True, generator=g)
    counts = torch.bincount(idx, minlength=E).to(torch.int64)
    order = torch.argsort(counts, stable=True)
    moved = counts[order[:8]].sum()
    counts[order[:8]] = 0
    counts[order[-1]] += moved
    return counts


def _peaks():
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---------------------------------------------------------------------------------------------------
# clocks sampled during the timed region (read-only nvidia-smi query of this rank's GPU, by UUID)
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.rows, self.proc, self.err = [], None, ""
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            self.target = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:  # noqa: BLE001 - fall back to the index
            self.target = str(device_index)

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20", "-i",
                 self.target], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError as exc:
            self.proc, self.err = None, repr(exc)
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()  # the exact child started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            try:
                self.err = (self.proc.stderr.read() or "")[-300:]
            except Exception:  # noqa: BLE001
                pass
        return False

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            if self.err:
                print(f"[bench] nvidia-smi gave no clock samples: {self.err}", file=sys.stderr)
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------
# CPU arm: the oracle (a port of the reference's algorithm) on a bounded sample of each workload
# ---------------------------------------------------------------------------------------------------
def _host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def _cpu_grouped_sample(cfg, num_experts: int):
    counts = _counts(cfg)
    g = torch.Generator().manual_seed(1)
    mean = cfg["ROWS"] // cfg["E"]
    pick = torch.argsort((counts - mean).abs(), stable=True)[:num_experts]  # experts nearest the mean load
    lens = counts[pick].clone()
    offs = torch.zeros(num_experts + 1, dtype=torch.int64)
    offs[1:] = torch.cumsum(lens, 0)
    m = int(offs[-1])
    a = torch.randn(m, cfg["K"], generator=g).to(torch.bfloat16)
    w = (torch.randn(num_experts, cfg["N"], cfg["K"], generator=g) * 0.02).to(torch.bfloat16)
    gy = (torch.randn(m, cfg["N"], generator=g) * 1e-3).to(torch.bfloat16)
    flops = 3 * 2 * m * cfg["N"] * cfg["K"]
    what = (f"the {num_experts} of {cfg['E']} experts with row counts nearest the mean, {m} routed rows "
            f"({flops / 1e9:.1f} GFLOP per step), torch CPU fp32")

    def step():
        from oracle import fp8_oracle as O

        E4 = torch.float8_e4m3fn
        q_row, q_col, s_row, s_col, _, vk_offs, _, pu = O.quant_segment_row_col(a, E4, 128, lens, offs)
        wq, w_s = O.quant_block2d(w, E4)
        out = O.grouped_gemm_blockwise(q_row, s_row, wq, w_s, offs, True, torch.bfloat16)
        g_row, g_col, gs_row, gs_col, _, _, _, _ = O.quant_segment_row_col(gy, E4, 128, lens, offs)
        dx = O.grouped_gemm_blockwise(g_row, gs_row, wq, w_s, offs, False, torch.bfloat16)
        dw = O.grouped_gemm_blockwise_variable_k(g_col[:pu], gs_col[: pu // 128], q_col[:pu], s_col[: pu // 128],
                                                 vk_offs, torch.bfloat16)
        return out, dx, dw

    return step, flops, what


def _cpu_dense_sample(cfg):
    from oracle import fp8_oracle as O

    E4 = torch.float8_e4m3fn
    g = torch.Generator().manual_seed(0)
    M, N, K = cfg["M"], cfg["N"], cfg["K"]
    ms = min(M, 2048)  # bounded sample: the first `ms` rows of the activations (all of N and K)
    x = torch.randn(ms, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * cfg["w_scale"]).to(torch.bfloat16)
    gy = (torch.randn(ms, N, generator=g) * 1e-3).to(torch.bfloat16)
    gemms = 3 if cfg["bwd"] else 1
    flops = gemms * 2 * ms * N * K
    what = (f"{ms} of {M} activation rows, all of N={N} and K={K}, {gemms} GEMM(s) "
            f"({flops / 1e9:.1f} GFLOP per step), torch CPU fp32")

    def step():
        if cfg["gran"] == "blockwise":
            aq, a_s, _, _ = O.quant_block1d_dual(x, E4)
            bq, b_s = O.quant_block2d(w, E4)
            return O.gemm_blockwise_nt(aq, a_s, bq, b_s, torch.bfloat16)
        if cfg["gran"] == "mx":
            a_row, a_rs = O.quant_mxfp8(x, E4, 1)
            a_col, a_cs = O.quant_mxfp8(x, E4, 0)
            b_row, b_rs = O.quant_mxfp8(w, E4, 1, True)
            b_col, b_cs = O.quant_mxfp8(w, E4, 0, True)
            g_row, g_rs = O.quant_mxfp8(gy, E4, 1)
            g_col, g_cs = O.quant_mxfp8(gy, E4, 0)
            return (O.gemm_mxfp8_nt(a_row, a_rs, b_row, b_rs), O.gemm_mxfp8_nt(g_row, g_rs, b_col, b_cs),
                    O.gemm_mxfp8_nt(g_col, g_cs, a_col, a_cs))
        if cfg["gran"] == "tensorwise":
            aq, a_s = O.quant_tensorwise(x, E4)
            bq, b_s = O.quant_tensorwise(w, E4)
            return O.gemm_tensorwise(aq, a_s, bq, b_s, False, True, torch.bfloat16)
        # rowwise, with the backward operands re-quantised from the dequantised forward operands
        aq, a_s = O.quant_rowwise(x, E4, -1)
        bq, b_s = O.quant_rowwise(w, E4, -1)
        out = O.gemm_rowwise(aq, a_s, bq, b_s, False, True, torch.bfloat16)
        a_t_q, a_t_s = O.quant_rowwise(O.dequant_rowwise(aq, a_s, torch.bfloat16), E4, -2)
        b_t_q, b_t_s = O.quant_rowwise(O.dequant_rowwise(bq, b_s, torch.bfloat16), E4, -2)
        gq, g_s = O.quant_rowwise(gy, E4, -1)
        gtq, gt_s = O.quant_rowwise(gy, E4, -2)
        dx = O.gemm_rowwise(gq, g_s, b_t_q, b_t_s, False, False, torch.bfloat16)
        dw = O.gemm_rowwise(gtq, gt_s, a_t_q, a_t_s, True, False, torch.bfloat16)
        return out, dx, dw

    return step, flops, what


def time_cpu(config: str, steps: int, warmup: int):
    """The oracle timed on the host cores with every thread this process may use."""
    torch.set_num_threads(_host_threads())  # torchrun exports OMP_NUM_THREADS=1; the CPU arm runs on rank 0 alone
    if config in GROUPED:
        step, flops, what = _cpu_grouped_sample(GROUPED[config], num_experts=8)
    else:
        step, flops, what = _cpu_dense_sample(DENSE[config])
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return {"value": flops / dt / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": what,
            "ms_per_step": dt * 1e3}


def _workload_config(config: str, world: int = 1):
    if config in GROUPED:
        c = GROUPED[config]
        return {"workload": c["workload"], "experts": c["E"], "hidden": c["K"], "n": c["N"], "routed_rows": c["ROWS"]}
    c = DENSE[config]
    return {"workload": c["workload"], "m": c["M"], "n": c["N"], "k": c["K"], "granularity": c["gran"]}


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    r = time_cpu(args.config, args.steps, args.warmup)
    cfg = _workload_config(args.config)
    cfg["sampled"] = True
    line = {
        "impl": "reference", "metric": METRIC[args.config], "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 dequantise-then-matmul on CPU)",
        "data": "synthetic", "config": cfg,
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# GPU arm: shared pieces
# ---------------------------------------------------------------------------------------------------
class HostPipe:
    """Host-buffer pass: every step copies its inputs from pinned host memory and its results back to
    it inside the timed region.  Copies run on their own streams with double-buffered device inputs,
    so step i+1's upload and step i-1's download overlap step i's kernels (every step still moves all
    of its own bytes)."""

    def __init__(self, dev, inputs, step, compute: bool = True):
        self.dev, self.step, self.compute = dev, step, compute
        self.host_in = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in inputs]
        for h, t in zip(self.host_in, inputs):
            h.copy_(t.detach())
        self.dev_in = [[torch.empty_like(t.detach()) for t in inputs] for _ in range(2)]
        self.host_out = None
        self.cur = torch.cuda.current_stream()
        self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
        self.in_ev = [torch.cuda.Event() for _ in range(2)]
        self.free_ev = [torch.cuda.Event() for _ in range(2)]
        for ev in self.free_ev:
            ev.record(self.cur)
        self.h2d = sum(t.numel() * t.element_size() for t in inputs)
        self.d2h = 0

    def run(self, i):
        b = i % 2
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(self.free_ev[b])  # the step that last read this buffer has finished with it
            for d, h in zip(self.dev_in[b], self.host_in):
                d.copy_(h, non_blocking=True)
            self.in_ev[b].record(self.s_in)
        self.cur.wait_event(self.in_ev[b])
        outs = self.step(*self.dev_in[b]) if self.compute else self._echo(b)
        self.free_ev[b].record(self.cur)
        if self.host_out is None:
            self.host_out = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
            self.d2h = sum(o.numel() * o.element_size() for o in outs)
        done = torch.cuda.Event()
        done.record(self.cur)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(done)
            for h, o in zip(self.host_out, outs):
                h.copy_(o.detach(), non_blocking=True)
        for o in outs:
            o.record_stream(self.s_out)

    def _echo(self, b):
        # copy-only ceiling: results of the recorded shapes, nothing computed
        return self._like

    def time(self, steps, barrier):
        for i in range(2):
            self.run(i)
        self.cur.wait_stream(self.s_out)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            self.run(i)
        self.cur.wait_stream(self.s_in)
        self.cur.wait_stream(self.s_out)
        e1.record()
        barrier()
        return e0.elapsed_time(e1) / steps


def time_e2e(dev, inputs, step, steps, barrier):
    """(ms per step with compute, ms per step copies only, h2d bytes, d2h bytes)"""
    pipe = HostPipe(dev, inputs, step)
    ms = pipe.time(steps, barrier)
    ceil = HostPipe(dev, inputs, step, compute=False)
    ceil.host_out = pipe.host_out
    ceil.d2h = pipe.d2h
    ceil._like = [torch.empty(h.shape, dtype=h.dtype, device=dev) for h in pipe.host_out]
    ms_copy = ceil.time(steps, barrier)
    return ms, ms_copy, pipe.h2d, pipe.d2h


def _roof(name, kernel, flops, nbytes, times_ms, peaks, fp8_peak, traffic=None):
    """Roofline record of one kernel: the bound is whichever floor (tensor or HBM) is the longer one."""
    if not times_ms:
        return None
    t = statistics.mean(times_ms) * 1e-3
    t_tensor = flops / (fp8_peak * 1e12) if flops else 0.0
    t_hbm = nbytes / (peaks["hbm_gbs"] * 1e9)
    rec = {"entry_point": name, "kernel": kernel, "avg_launch_ms": t * 1e3, "launches": len(times_ms),
           "algorithmic_flops": flops, "algorithmic_bytes": nbytes, "tensor_floor_ms": t_tensor * 1e3,
           "hbm_floor_ms": t_hbm * 1e3, "traffic": traffic}
    if t_tensor >= t_hbm:
        ach = flops / t / 1e12
        rec.update({"bound": "tensor", "achieved": ach, "peak": fp8_peak, "unit": "TFLOP/s", "frac": ach / fp8_peak,
                    "peak_source": f"2 x sustained bf16 cuBLAS rate of MEASURED_PEAKS.json ({peaks['source']})"})
    else:
        ach = nbytes / t / 1e9
        rec.update({"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": ach / peaks["hbm_gbs"],
                    "peak_source": f"copy bandwidth of MEASURED_PEAKS.json ({peaks['source']})"})
    return rec


def _finish_line(args, line, kernel_ms, roofs, clocks, launches, status):
    roofs = [r for r in roofs if r]
    # the kernel with the largest share of the step leads; the peer copy (an NVLink-bound kernel) never does
    roofs.sort(key=lambda r: (r["bound"] not in ("hbm", "tensor"), -r["avg_launch_ms"] * r["launches"]))
    line.update({
        "gpu_launches": launches,
        "kernel_ms": {k: {"launches": len(v), "avg_ms": statistics.mean(v), "total_ms": sum(v)} for k, v in kernel_ms.items()},
        "gemm_status": status, "clocks": clocks,
        "roofline": roofs[0] if roofs else None, "roofline_other_kernels": roofs[1:],
    })
    if line["n_gpus"] == 1 and not args.no_cpu_baseline:
        r = time_cpu(args.config, steps=3, warmup=1)
        line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
    print(json.dumps(line), flush=True)


LOG_PASS_STEPS = [None]  # steps of the separate event-logging pass (None: events were taken in the timed steps)
HOST_ENQUEUE_MS = [None]  # set by _timed: when it nears ms_per_step the host, not the GPU, paces the step


def _timed(step, inputs, steps, warmup, barrier, device_index, flush=None, log_pass=False):
    """(ms per step, per-entry-point kernel times, clock summary, launches).

    log_pass: take the per-call CUDA events in a separate pass of up to three steps right after the timed
    steps instead of inside them.  A multi-GPU step is short enough for the host to pace it, and two event
    records around each of its ~40 calls are host time the timed region should not carry; on one GPU the
    device paces the step and the events stay inside the timed region."""
    import contextlib
    import gc

    from primus_turbo_b200 import _lib

    for _ in range(max(warmup, 3)):
        step(*inputs)
    barrier()
    launches0 = _lib.launch_count
    with ClockSampler(device_index) as clocks, (contextlib.nullcontext() if log_pass else _lib.record_kernel_times()) as rec:
        barrier()
        if flush is None:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            gc_was = gc.isenabled()
            gc.disable()  # no collector pause in the middle of a step
            ev0.record()
            h0 = time.perf_counter()
            for _ in range(steps):
                step(*inputs)
            HOST_ENQUEUE_MS[0] = (time.perf_counter() - h0) * 1e3 / steps  # host time to enqueue one step
            ev1.record()
            if gc_was:
                gc.enable()
            barrier()
            ms = ev0.elapsed_time(ev1) / steps
        else:
            evs = []
            for _ in range(steps):
                flush.zero_()  # evict the inputs from L2 between timed iterations (not timed)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                step(*inputs)
                e1.record()
                evs.append((e0, e1))
            barrier()
            ms = sum(a.elapsed_time(b) for a, b in evs) / steps
    launches = _lib.launch_count - launches0
    if log_pass:
        n_log = min(steps, 3)
        with _lib.record_kernel_times() as rec:
            for _ in range(n_log):
                step(*inputs)
            barrier()
        LOG_PASS_STEPS[0] = n_log
    return ms, rec.durations_ms(), clocks.summary(), launches


# ---------------------------------------------------------------------------------------------------
# dense configurations (c1, c2, c3): one GPU
# ---------------------------------------------------------------------------------------------------
def run_dense(args):
    from primus_turbo_b200 import _lib
    from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig, ScaleDtype, ScalingGranularity
    from primus_turbo_b200.pytorch.ops import gemm_fp8

    assert args.gpus == 1 and int(os.environ.get("WORLD_SIZE", "1")) == 1, "the dense configurations run on one GPU"
    cfg = DENSE[args.config]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    M, N, K = cfg["M"], cfg["N"], cfg["K"]
    gran = {"blockwise": ScalingGranularity.BLOCKWISE, "tensorwise": ScalingGranularity.TENSORWISE,
            "rowwise": ScalingGranularity.ROWWISE, "mx": ScalingGranularity.MX_BLOCKWISE}[cfg["gran"]]
    if cfg["gran"] == "mx":
        qcfg = Float8QuantConfig(granularity=gran, block_size=32, scale_dtype=ScaleDtype.E8M0)
    else:
        qcfg = Float8QuantConfig(granularity=gran, block_size=128 if cfg["gran"] == "blockwise" else None)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(dev)
    w = (torch.randn(N, K, generator=g) * cfg["w_scale"]).to(torch.bfloat16).to(dev).requires_grad_(cfg["bwd"])
    gy = (torch.randn(M, N, generator=g) * 1e-3).to(torch.bfloat16).to(dev)
    gemms = 3 if cfg["bwd"] else 1
    flops = gemms * 2 * M * N * K

    def step(x_in, gy_in=None):
        if not cfg["bwd"]:
            return (gemm_fp8(x_in, w, trans_b=True, config=qcfg),)
        x_in = x_in.detach().requires_grad_(True)
        out = gemm_fp8(x_in, w, trans_b=True, config=qcfg)
        gx, gw = torch.autograd.grad(out, (x_in, w), gy_in)
        return out, gx, gw

    def barrier():
        torch.cuda.synchronize()

    inputs = (x, gy) if cfg["bwd"] else (x,)
    in_bytes = (M * K + N * K) * 2
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if in_bytes < (200 << 20) else None
    ms, kernel_ms, clocks, launches = _timed(step, inputs, args.steps, args.warmup, barrier, 0, flush)
    status = _lib.gemm_status()
    e2e = None
    if not args.no_e2e:
        # inputs from the host: the activations (and grad-out); results back: out (c3: also grad_x; the weight
        # and its gradient stay resident)
        def e2e_step(*ins):
            return step(*ins)[:2]

        e2e_ms, copy_ms, h2d, d2h = time_e2e(dev, inputs, e2e_step, max(2, min(args.steps, 10)), barrier)
        e2e = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "copy_only_ms_per_step": copy_ms,
               "note": "activations (and grad-out) from pinned host memory, out (and grad-activation) back to it; "
                       "copy_only_ms_per_step is the same traffic with no kernels in between (the PCIe ceiling)"}
    peaks = _peaks()
    fp8_peak = 2.0 * peaks["bf16_tflops_sustained"]
    gemm_name = "ptb_gemm_mxfp8" if cfg["gran"] == "mx" else "ptb_gemm_fp8"
    gemm_t = kernel_ms.get(gemm_name, [])
    per_gemm = 2 * M * N * K
    op_bytes = M * K + N * K + M * N * 2  # fp8 operands in, bf16 out (forward shape; dgrad / wgrad permute M, N, K)
    roofs = [_roof(gemm_name, f"fp8_gemm_kernel<{cfg['gran']}, bf16> (dense, {gemms} launch(es) per step)", per_gemm,
                   op_bytes, gemm_t, peaks, fp8_peak)]
    for name, v in kernel_ms.items():
        if name.startswith("ptb_quant") and v:
            n_el = {"ptb_quant_fp8_block2d": N * K}.get(name, M * max(K, N) if cfg["bwd"] else M * K)
            per_el = 4.0625 if name == "ptb_quant_mxfp8" else 3.03  # both directions in one pass: 2 R + 2 W + 2/32
            if name == "ptb_quant_mxfp8":
                n_el = (M * K + N * K + M * N) / 3.0  # mean over the step's three calls (x, w, grad-out)
            roofs.append(_roof(name, "quantise kernel(s) of this entry point (bytes of the largest operand it sees)", 0,
                               n_el * per_el, v, peaks, fp8_peak))
    value = flops / (ms * 1e-3) / 1e12
    wl = _workload_config(args.config)
    wl["l2"] = ("L2 flushed (256 MiB memset) between timed iterations" if flush is not None
                else "inputs larger than L2")
    line = {"metric": METRIC[args.config], "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 operands, fp32 accumulate, bf16 in/out", "data": "synthetic",
            "config": wl, "per_gpu_tflops": value, "pct_of_fp8_peak_per_gpu": 100.0 * value / fp8_peak,
            "fp8_peak_tflops": fp8_peak, "e2e": e2e}
    _finish_line(args, line, kernel_ms, roofs, clocks, launches, status)


# ---------------------------------------------------------------------------------------------------
# grouped configurations (c4, c5): 1..8 GPUs
# ---------------------------------------------------------------------------------------------------
def _bind_host_threads_near_gpu(index: int) -> None:
    """Pin this process to the CPU cores NVML reports as local to its GPU (read-only query; any failure
    leaves the affinity as it was)."""
    try:
        import pynvml

        pynvml.nvmlInit()
        props = torch.cuda.get_device_properties(index)
        bus = "%08x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1}
        allowed = cpus & os.sched_getaffinity(0)
        if len(allowed) >= 4:  # never squeeze the rank's host threads onto a couple of cores
            os.sched_setaffinity(0, allowed)
    except Exception:  # noqa: BLE001 - best effort, never fatal
        pass


def _ep_parity(dist, rank, world, dev, cfg, qcfg, order_pos_counts, x, gy, w, ep_step, sample_positions):
    """Before timing: for a few sampled experts, every rank recomputes -- on one GPU, with the single-GPU
    op -- the rows it routes to that expert (the owner broadcasts the expert's weight) and compares with
    what the expert-parallel step returned for those rows: out and grad_a must match bit for bit."""
    from primus_turbo_b200.pytorch.ops import grouped_gemm_fp8

    e_loc = cfg["E"] // world
    out, ga, _ = ep_step(x.detach().requires_grad_(True), gy)
    ok = True
    offs = torch.cumsum(order_pos_counts, 0) - order_pos_counts
    for p in sample_positions:
        owner = p // e_loc
        wp = w[p - owner * e_loc].detach().clone() if rank == owner else torch.empty(
            (cfg["N"], cfg["K"]), dtype=torch.bfloat16, device=dev)
        dist.broadcast(wp, src=owner)
        n, lo = int(order_pos_counts[p]), int(offs[p])
        if n == 0:
            continue
        xs = x[lo : lo + n].detach().requires_grad_(True)
        lens = torch.tensor([n], dtype=torch.int64, device=dev)
        o1 = grouped_gemm_fp8(xs, wp.unsqueeze(0), lens, config=qcfg)
        (g1,) = torch.autograd.grad(o1, xs, gy[lo : lo + n])
        ok = ok and torch.equal(o1, out[lo : lo + n]) and torch.equal(g1, ga[lo : lo + n])
    flag = torch.tensor([1 if ok else 0], device=dev, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


def run_grouped(args):
    import torch.distributed as dist

    from primus_turbo_b200 import _lib
    from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig, ScalingGranularity
    from primus_turbo_b200.pytorch.core.quantized_tensor import create_quantized_weight
    from primus_turbo_b200.pytorch.dist import expert_parallel as EP
    from primus_turbo_b200.pytorch.ops import grouped_gemm_fp8

    cfg = dict(GROUPED[args.config])
    if args.experts:
        cfg["E"] = args.experts
    if args.rows:
        cfg["ROWS"] = args.rows
    E, K, N, ROWS = cfg["E"], cfg["K"], cfg["N"], cfg["ROWS"]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    assert E % world == 0 and ROWS % world == 0
    if world > 1 and args.bind_cpus:
        _bind_host_threads_near_gpu(local_rank)
    host_group = board = exchange = None
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep stdout to the one JSON line
        # The job's collectives are all-to-alls, barriers and scalar reductions: in-switch reduction buys nothing
        # here, and a rank that dies while its memory is bound to an NVLink multicast object raises faults on
        # the other ranks' GPUs.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
        host_group = dist.new_group(backend="gloo")  # CPU group: set-up traffic and the fallback count gather
        try:
            board = EP.SharedCountsBoard(E, group=host_group)  # ranks of one machine: counts through shared memory
        except Exception as exc:  # noqa: BLE001 - keep the gloo group
            print(f"[bench] shared counts board unavailable ({exc!r}); using gloo", file=sys.stderr)
    if args.granularity == "mx":
        from primus_turbo_b200.pytorch.core.low_precision import ScaleDtype

        qcfg = Float8QuantConfig(granularity=ScalingGranularity.MX_BLOCKWISE, block_size=32, scale_dtype=ScaleDtype.E8M0)
        args.no_cached = True  # pre-quantised weights are a BLOCKWISE feature
        args.no_cpu_baseline = True  # the CPU arm times the benchmark's own (128-block) format
    else:
        qcfg = Float8QuantConfig(granularity=ScalingGranularity.BLOCKWISE, block_size=128)
    e_loc = E // world

    # ---- routing: global counts, expert placement, this rank's rows ---------------------------------------
    counts = _counts(cfg)
    imbalance_contiguous = EP.load_imbalance(counts, world)
    if world > 1 and args.placement == "balanced":
        # the router's expected load is the distribution the counts were drawn from; the realised counts
        # of the seeded draw stand in for it
        order = EP.balanced_expert_order(counts, world)
    else:
        order = torch.arange(E)
    pos_counts = counts[order]  # rows per placement position (rank r owns positions [r*e_loc, (r+1)*e_loc))
    imbalance = EP.load_imbalance(pos_counts, world)
    torch.manual_seed(1234 + rank)
    rows_here = ROWS // world
    if world == 1:
        counts_here = pos_counts
    else:
        # every source rank holds ROWS/world rows whose experts are drawn i.i.d. from the same routing
        g = torch.Generator().manual_seed(100 + rank)
        idx = torch.multinomial(pos_counts.double() / pos_counts.sum(), rows_here, replacement=True, generator=g)
        counts_here = torch.bincount(idx, minlength=E).to(torch.int64)
    counts_dev = counts_here.to(dev)
    a = torch.randn(rows_here, K, device=dev, dtype=torch.bfloat16).requires_grad_(True)
    w = (torch.randn(e_loc, N, K, device=dev, dtype=torch.bfloat16) * 0.02).requires_grad_(True)
    gy = torch.randn(rows_here, N, device=dev, dtype=torch.bfloat16) * 1e-3
    flops_step = 3 * 2 * ROWS * N * K  # whole job
    plan_ms = []

    if world > 1 and args.exchange == "peer":
        from primus_turbo_b200.pytorch.dist.peer_exchange import PeerExchange

        cap = int(max(2 * ROWS // world, ROWS // world + 4096))
        try:
            # checks, on the host and on every rank alike, that all GPUs of the job can address each other
            exchange = PeerExchange(None, host_group, dev, capacity_rows=cap, local_rows=rows_here, num_ctas=args.copy_ctas,
                                    ordering=args.ep_ordering)
        except RuntimeError as exc:
            print(f"[bench] rank {rank}: {exc}; using NCCL all-to-alls", file=sys.stderr)
            exchange, args.exchange = None, "nccl"
    state = {"exchange": exchange}

    def make_step(weight):
        def local_fn(rows, lens):
            return grouped_gemm_fp8(rows, weight, lens, config=qcfg)

        def step(a_in, gy_in):
            a_in = a_in if a_in.requires_grad else a_in.detach().requires_grad_(True)
            if world == 1:
                out = grouped_gemm_fp8(a_in, weight, counts_dev, config=qcfg)
            else:
                # the synthetic router's counts live on the host, so the exchange plan (rebuilt every step, as
                # routing changes every step in training) never waits on the device stream
                t0 = time.perf_counter()
                if state["exchange"] is not None:
                    plan = EP.build_peer_plan(counts_here, board or host_group, dev)
                    plan_ms.append((time.perf_counter() - t0) * 1e3)
                    if args.ep_overlap:
                        # weight quantise beside the dispatch, wgrad beside the return of grad_a
                        out = EP.ep_grouped_gemm_fp8_peer(a_in, weight, state["exchange"], plan, config=qcfg, overlap=True,
                                                          reserve_sms=args.ep_reserve_sms)
                    else:
                        out = EP.expert_parallel_apply_peer(a_in, local_fn, state["exchange"], plan)
                else:
                    plan = EP.build_exchange_plan(counts_dev, counts_host=counts_here, host_group=board or host_group)
                    plan_ms.append((time.perf_counter() - t0) * 1e3)
                    out = EP.expert_parallel_apply(a_in, counts_dev, local_fn, plan=plan)
            leaf = weight
            ga, gw = torch.autograd.grad(out, (a_in, leaf), gy_in)
            return out, ga, gw

        return step

    step = make_step(w)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ep_parity = None
    if world > 1:
        nz = torch.nonzero(pos_counts > 0).flatten().tolist()
        sample = sorted({nz[0], nz[len(nz) // 3], nz[(2 * len(nz)) // 3], nz[-1]})
        ep_parity = _ep_parity(dist, rank, world, dev, cfg, qcfg, counts_here, a, gy, w, step, sample)
        flags_status = _lib.copy_segments_status(reset=False) if state["exchange"] is not None else 0
        st = torch.tensor([flags_status], device=dev, dtype=torch.int32)
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        if state["exchange"] is not None and state["exchange"].ordering == "flags" and (not ep_parity or int(st.item()) != 0):
            # the flag rendezvous did not give the single-GPU results on this machine: measure with the
            # collective instead and say so (every rank takes this branch: both inputs are reduced values)
            print(f"[bench] rank {rank}: flag ordering failed its check (parity {ep_parity}, status {int(st.item())}); "
                  "using the all-reduce ordering", file=sys.stderr)
            _lib.copy_segments_status(reset=True)
            state["exchange"].close()
            args.ep_ordering = "collective (flags failed their check)"
            exchange = PeerExchange(None, host_group, dev, capacity_rows=cap, local_rows=rows_here, num_ctas=args.copy_ctas,
                                    ordering="collective")
            state["exchange"] = exchange
            ep_parity = _ep_parity(dist, rank, world, dev, cfg, qcfg, counts_here, a, gy, w, step, sample)

    # ---- device-resident timing ---------------------------------------------------------------------------
    plan_ms.clear()
    ms, kernel_ms, clocks, launches = _timed(step, (a, gy), args.steps, args.warmup, barrier, local_rank, log_pass=world > 1)
    k_steps = LOG_PASS_STEPS[0] or args.steps  # steps the per-call event log covers
    n_log = LOG_PASS_STEPS[0] or 0
    timed_plans = plan_ms[len(plan_ms) - n_log - args.steps: len(plan_ms) - n_log]
    plan_host_ms = statistics.mean(timed_plans) if timed_plans else 0.0
    host_enqueue_ms = HOST_ENQUEUE_MS[0]
    status = _lib.gemm_status()
    copy_status = _lib.copy_segments_status() if state["exchange"] is not None else 0

    # ---- the same step with the weight quantised ahead of time (where the caller's weights allow it) ----
    ms_cached = None
    if not args.no_cached:
        with torch.no_grad():
            qw, _ = create_quantized_weight(w.detach().clone().requires_grad_(True), torch.float8_e4m3fn, qcfg)
        step_cached = make_step(qw)
        ms_cached, _, _, _ = _timed(step_cached, (a, gy), max(2, min(args.steps, 5)), 3, barrier, local_rank)

    # ---- end to end: host buffers in, host buffers out --------------------------------------------------------
    e2e_ms = copy_ms = float("nan")
    h2d = d2h = 0
    if not args.no_e2e:
        def e2e_step(a_in, gy_in):
            return step(a_in, gy_in)[:2]

        e2e_ms, copy_ms, h2d, d2h = time_e2e(dev, (a, gy), e2e_step, max(2, min(args.steps, 10)), barrier)

    # ---- max over ranks -------------------------------------------------------------------------------------------
    if world > 1:
        t = torch.tensor([ms, e2e_ms, ms_cached or 0.0, copy_ms, plan_host_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, copy_ms, plan_host_ms = float(t[0]), float(t[1]), float(t[3]), float(t[4])
        ms_cached = float(t[2]) if ms_cached is not None else None

    if rank == 0:
        peaks = _peaks()
        fp8_peak = 2.0 * peaks["bf16_tflops_sustained"]  # dense FP8 runs at twice the bf16 rate
        value = flops_step / (ms * 1e-3) / 1e12
        # what rank 0's launches process (at N > 1: rank 0's share after the dispatch)
        if world == 1:
            lens0 = pos_counts
        else:
            lens0 = pos_counts.new_zeros(e_loc)
            for r in range(world):
                g = torch.Generator().manual_seed(100 + r)
                idx = torch.multinomial(pos_counts.double() / pos_counts.sum(), rows_here, replacement=True, generator=g)
                lens0 += torch.bincount(idx, minlength=E)[:e_loc]
        rows0 = int(lens0.sum())
        pad0 = int((((lens0 + 127) // 128) * 128).sum())  # rows of the segment-padded column copies
        tile_rows0 = pad0  # rows the 128-row forward / dgrad tiles cover
        gemm_flops = 2 * rows0 * N * K
        # ncu dram__bytes_read + dram__bytes_write per launch on the captured 32-expert / 8192-row case of c4,
        # over the algorithmic bytes of that case: scaled to this launch by its algorithmic bytes
        traffic_ratio = {"wgrad": 1.941e9 / 1.997e9, "fwd": 1.227e9 / 1.062e9, "wq": 2.789e9 / 2.819e9} \
            if args.config == "c4" else {}
        b_wgrad = e_loc * N * K * 2 + pad0 * (N + K) * (1 + 4.0 / 128)
        b_fwd = e_loc * N * K + rows0 * (K + 2 * N)
        b_dgrad = e_loc * N * K + rows0 * (N + 2 * K)
        b_wq = e_loc * N * K * (3 + 4.0 / 16384)
        b_seg = lambda width: rows0 * width * (2 + 1 + 4.0 / 128) + pad0 * width * (1 + 4.0 / 128)  # noqa: E731
        tr = lambda k, b: (traffic_ratio[k] * b if k in traffic_ratio else None)  # noqa: E731
        roofs = [
            _roof("ptb_grouped_gemm_fp8_variable_k", "wgrad_pair_kernel<bf16> (grouped wgrad launch, 1-D x 1-D block scales)", gemm_flops,
                  b_wgrad, kernel_ms.get("ptb_grouped_gemm_fp8_variable_k", []), peaks, fp8_peak, tr("wgrad", b_wgrad)),
            _roof("ptb_grouped_gemm_fp8", "fp8_gemm_kernel<block 1x128 x 128x128, bf16> (grouped forward and dgrad launches)",
                  gemm_flops, (b_fwd + b_dgrad) / 2, kernel_ms.get("ptb_grouped_gemm_fp8", []), peaks, fp8_peak,
                  tr("fwd", (b_fwd + b_dgrad) / 2)),
            _roof("ptb_quant_fp8_block2d", "quant_block_kernel<128x128> (weight quantise)", 0, b_wq,
                  kernel_ms.get("ptb_quant_fp8_block2d", []), peaks, fp8_peak, tr("wq", b_wq)),
            _roof("ptb_quant_fp8_segment_row_col", "seg_quant_stream_kernel (row + padded column copy of activation and grad-out)", 0,
                  (b_seg(K) + b_seg(N)) / 2, kernel_ms.get("ptb_quant_fp8_segment_row_col", []), peaks, fp8_peak),
        ]
        copy_key = "ptb_copy_segments_signal" if "ptb_copy_segments_signal" in kernel_ms else "ptb_copy_segments"
        if copy_key in kernel_ms:
            sent = rows_here * (K + N) * 2 * 2 / 4  # mean bytes per launch over the step's four exchanges
            r = _roof(copy_key, "copy_segments_kernel (dispatch / combine over peer memory)", 0, sent,
                      kernel_ms[copy_key], peaks, fp8_peak)
            r.update({"bound": "nvlink", "peak": 770.0, "peak_source": "measured peer copy, GB/s per direction",
                      "achieved": sent * (world - 1) / world / (r["avg_launch_ms"] * 1e-3) / 1e9})
            r["frac"] = r["achieved"] / r["peak"]
            roofs.append(r)
        other_ms = {k: sum(kernel_ms.pop(k)) / k_steps for k in list(kernel_ms) if k.startswith("ep_")}
        step_kernels = sum(sum(v) for v in kernel_ms.values()) / k_steps
        copy_k = sum(kernel_ms.get(copy_key, [])) / k_steps
        wait_k = sum(kernel_ms.get("ptb_wait_flags", [])) / k_steps
        wl = _workload_config(args.config)
        wl.update({"experts": E, "routed_rows": ROWS, "experts_per_gpu": e_loc, "parallelism": f"ep{world}",
                   "exchange": (args.exchange if world > 1 else None), "placement": (args.placement if world > 1 else None),
                   "ep_overlap": (bool(args.ep_overlap) if world > 1 else None), "granularity": args.granularity,
                   "ep_ordering": (args.ep_ordering if world > 1 and args.exchange == "peer" else None),
                   "load_imbalance_max_over_mean_rows": imbalance,
                   "load_imbalance_contiguous_placement": imbalance_contiguous,
                   "tile_padding_rows_over_rows": pad0 / max(rows0, 1),
                   "l2": f"inputs larger than L2 ({e_loc * N * K / 1e9:.2f} GB of FP8 weights per pass)"})
        line = {
            "metric": (METRIC[args.config] if args.granularity == "blockwise" else METRIC[args.config].replace("blockwise_fp8", "mxfp8")),
            "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 operands, fp32 accumulate, bf16 in/out", "data": "synthetic",
            "config": wl, "per_gpu_tflops": value / world, "pct_of_fp8_peak_per_gpu": 100.0 * value / world / fp8_peak,
            "fp8_peak_tflops": fp8_peak,
            "value_cached_weights": (flops_step / (ms_cached * 1e-3) / 1e12) if ms_cached else None,
            "ms_per_step_cached_weights": ms_cached,
            "e2e": {"value": flops_step / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "copy_only_ms_per_step": copy_ms,
                    "note": "activations and grad-out from pinned host memory, out and grad-activation back to it "
                            "(copy streams overlap the neighbouring steps' kernels); weights and their gradient stay "
                            "resident; copy_only_ms_per_step is the same traffic with no kernels in between"},
        }
        if world > 1:
            line["ep_parity"] = ep_parity
            line["phases_ms"] = {"plan_host": plan_host_ms, "exchange_copy_kernels": copy_k,
                                 "local_kernels": step_kernels - copy_k - wait_k, "step": ms,
                                 "host_enqueue": host_enqueue_ms,
                                 "ordering": other_ms.get("ep_order_all_reduce", wait_k),
                                 "copies_out_of_regions": other_ms.get("ep_copy_out_of_region"),
                                 "not_in_kernels": ms - step_kernels,
                                 "kernel_times_from": (f"a logging pass of {LOG_PASS_STEPS[0]} steps right after the timed "
                                                       "steps (per-call events are host time a multi-GPU step "
                                                       "cannot hide)" if LOG_PASS_STEPS[0] else "the timed steps"),
                                 "note": "rank 0's kernels; plan_host is host time that overlaps the device queue; "
                                         "ordering (flag waits or all-reduces) includes waiting for the slowest rank; "
                                         "not_in_kernels covers collectives, torch's copies and launch gaps"}
            line["copy_segments_status"] = copy_status
        _finish_line(args, line, kernel_ms, roofs, clocks, launches, status)
    if world > 1:
        if exchange is not None:
            exchange.close()  # collective: peers' mappings first, own regions after everyone has let go
        if board is not None:
            board.close()
        dist.barrier()
        dist.destroy_process_group()
        # Everything is measured, printed and torn down.  Leave without running interpreter-exit destructors:
        # with CUDA IPC mappings in play, torch's exit-time bookkeeping of shared CUDA storages was seen to
        # crash a rank after its results were out (exit code -11), which a launcher reads as a failed run.
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", choices=sorted(METRIC), default="c4")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer pass (profiling runs)")
    ap.add_argument("--no-cached", action="store_true", help="skip the pass with weights quantised ahead of time")
    ap.add_argument("--granularity", choices=["blockwise", "mx"], default="blockwise",
                    help="grouped configurations: 128-block scales (the benchmark's) or MXFP8 (1x32 blocks, E8M0 scales)")
    ap.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                    help="N > 1: rows written into the owners' IPC-mapped buffers by this library's copy kernel, or "
                         "NCCL all-to-alls plus a permutation pass")
    ap.add_argument("--placement", choices=["balanced", "contiguous"], default="balanced",
                    help="N > 1: experts assigned to ranks by greedy balancing of the expected load, or expert e on "
                         "rank e // (E/N)")
    ap.add_argument("--copy-ctas", type=int, default=0, help="CTAs of the peer copy kernel (0: one per SM)")
    ap.add_argument("--ep-ordering", choices=["flags", "collective"], default="flags",
                    help="how ranks order themselves after a peer exchange: arrival flags written by the copy kernel "
                         "and a one-warp wait kernel, or a one-element all-reduce")
    ap.add_argument("--ep-overlap", type=int, default=0,
                    help="N > 1, peer exchange: 1 = weight quantise beside the dispatch and wgrad beside the return of "
                         "grad_a on a second stream (give --copy-ctas the same small number as --ep-reserve-sms)")
    ap.add_argument("--ep-reserve-sms", type=int, default=16, help="SMs wgrad leaves to the overlapped copy kernel")
    ap.add_argument("--bind-cpus", type=int, default=0,
                    help="N > 1: 1 = pin each rank to the CPU cores NVML reports as local to its GPU")
    ap.add_argument("--experts", type=int, default=0, help="smaller case of the same workload (profiling)")
    ap.add_argument("--rows", type=int, default=0, help="smaller case of the same workload (profiling)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path in the product")
    elif args.config in GROUPED:
        run_grouped(args)
    else:
        run_dense(args)


if __name__ == "__main__":
    main()
