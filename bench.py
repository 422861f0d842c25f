#!/usr/bin/env python
"""Benchmark of the FP8 grouped-GEMM hot path (blockwise scales, DeepSeek-V3 expert shape).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of synthetic routed rows, through the public
op ``grouped_gemm_fp8`` exactly as a caller runs it: activation quantise (1x128 row copy +
segment-padded 128x1 column copy), weight quantise (128x128 tiles, redone every forward as the
reference does), forward grouped GEMM, grad-out quantise, dgrad grouped GEMM, wgrad variable-K
grouped GEMM.  FLOPs counted are the algorithmic 3 x 2*M*N*K only.

Workload: 256 experts, hidden 7168, gate+up N=4096, 65536 routed rows, per-expert counts drawn from
a multinomial over softmax(N(0,1) logits), seed 0; bf16 inputs, e4m3 payloads, fp32 scales.
With N > 1 ranks the experts are sharded contiguously (256/N per GPU), the 65536 rows start evenly
split over the ranks and travel to their expert's owner with an NCCL all-to-all (strong scaling).
The per-step routing counts are gathered on the host through a shared-memory board (``--plan host``,
default) or on the device (``--plan device``: NCCL gather plus one host read of the split sizes).

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

E_TOTAL, HIDDEN, N_OUT, ROWS = 256, 7168, 4096, 65536
WORKLOAD = "deepseek_v3_moe_gate_up_blockwise_fp8_grouped_gemm_fwd_dgrad_wgrad"
METRIC = "blockwise_fp8_grouped_gemm_throughput"
UNIT = "TFLOP/s"


def _counts(seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(E_TOTAL, generator=g)
    p = torch.softmax(logits, 0)
    idx = torch.multinomial(p, ROWS, replacement=True, generator=g)
    return torch.bincount(idx, minlength=E_TOTAL).to(torch.int64)


def _peaks():
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ---------------------------------------------------------------------------------------------------
# clocks sampled during the timed region
# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20", "-i",
                 str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
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
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------
# CPU arm: the oracle (a port of the reference's algorithm) on a bounded sample
# ---------------------------------------------------------------------------------------------------
def cpu_sample_step(sample):
    """quantise -> dequantise -> fp32 matmul, forward + dgrad + wgrad, for the sample's experts."""
    from oracle import fp8_oracle as O

    a, w, gy, lens, offs = sample
    E4 = torch.float8_e4m3fn
    q_row, q_col, s_row, s_col, vk_lens, vk_offs, _, pu = O.quant_segment_row_col(a, E4, 128, lens, offs)
    wq, w_s = O.quant_block2d(w, E4)
    out = O.grouped_gemm_blockwise(q_row, s_row, wq, w_s, offs, True, torch.bfloat16)
    g_row, g_col, gs_row, gs_col, _, _, _, _ = O.quant_segment_row_col(gy, E4, 128, lens, offs)
    dx = O.grouped_gemm_blockwise(g_row, gs_row, wq, w_s, offs, False, torch.bfloat16)
    dw = O.grouped_gemm_blockwise_variable_k(g_col[:pu], gs_col[: pu // 128], q_col[:pu], s_col[: pu // 128], vk_offs,
                                             torch.bfloat16)
    return out, dx, dw


def make_cpu_sample(num_experts: int):
    counts = _counts()
    g = torch.Generator().manual_seed(1)
    # the experts whose row counts are nearest the mean (ROWS / E_TOTAL): a representative slice
    pick = torch.argsort((counts - ROWS // E_TOTAL).abs(), stable=True)[:num_experts]
    lens = counts[pick].clone()
    offs = torch.zeros(num_experts + 1, dtype=torch.int64)
    offs[1:] = torch.cumsum(lens, 0)
    m = int(offs[-1])
    a = torch.randn(m, HIDDEN, generator=g).to(torch.bfloat16)
    w = (torch.randn(num_experts, N_OUT, HIDDEN, generator=g) * 0.02).to(torch.bfloat16)
    gy = (torch.randn(m, N_OUT, generator=g) * 1e-3).to(torch.bfloat16)
    return (a, w, gy, lens, offs), 3 * 2 * m * N_OUT * HIDDEN


def time_cpu(steps: int, warmup: int, num_experts: int):
    sample, flops = make_cpu_sample(num_experts)
    for _ in range(warmup):
        cpu_sample_step(sample)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_sample_step(sample)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    rows = int(sample[4][-1])
    return {"value": flops / dt / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"the {num_experts} of {E_TOTAL} experts with row counts nearest the mean, {rows} routed rows "
                      f"({flops / 1e9:.1f} GFLOP per step), torch CPU fp32", "ms_per_step": dt * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = time_cpu(args.steps, args.warmup, num_experts=4)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 dequantise-then-matmul on CPU)",
        "data": "synthetic", "config": {"workload": WORKLOAD, "experts": E_TOTAL, "hidden": HIDDEN, "n": N_OUT,
                                        "routed_rows": ROWS, "sampled": True},
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------
def _time_e2e(args, step, barrier, a, gy, rows_here, dev):
    """The same step with activations / grad-out arriving from pinned host memory and the forward
    output and activation gradient returned to it, all inside the timed region.  Copies run on their
    own streams with double-buffered device inputs, so step i+1's upload and step i-1's download
    overlap step i's kernels (every step still moves all of its own bytes)."""
    a_host = torch.empty((rows_here, HIDDEN), dtype=torch.bfloat16).pin_memory()
    gy_host = torch.empty((rows_here, N_OUT), dtype=torch.bfloat16).pin_memory()
    a_host.copy_(a.detach())
    gy_host.copy_(gy)
    out_host = torch.empty((rows_here, N_OUT), dtype=torch.bfloat16).pin_memory()
    ga_host = torch.empty((rows_here, HIDDEN), dtype=torch.bfloat16).pin_memory()
    a_dev = [torch.empty((rows_here, HIDDEN), device=dev, dtype=torch.bfloat16) for _ in range(2)]
    gy_dev = [torch.empty_like(gy) for _ in range(2)]
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    in_ev = [torch.cuda.Event() for _ in range(2)]
    free_ev = [torch.cuda.Event() for _ in range(2)]
    for ev in free_ev:
        ev.record(cur)

    def e2e_step(i):
        b = i % 2
        with torch.cuda.stream(s_in):
            s_in.wait_event(free_ev[b])  # the step that last read this buffer has finished with it
            a_dev[b].copy_(a_host, non_blocking=True)
            gy_dev[b].copy_(gy_host, non_blocking=True)
            in_ev[b].record(s_in)
        cur.wait_event(in_ev[b])
        out, ga, _ = step(a_dev[b].detach().requires_grad_(True), gy_dev[b])
        free_ev[b].record(cur)
        done = torch.cuda.Event()
        done.record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            out_host.copy_(out.detach(), non_blocking=True)
            ga_host.copy_(ga, non_blocking=True)
        out.record_stream(s_out)
        ga.record_stream(s_out)

    for i in range(2):
        e2e_step(i)
    cur.wait_stream(s_out)
    barrier()
    e2e_steps = max(2, min(args.steps, 10))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    cur.wait_stream(s_in)
    cur.wait_stream(s_out)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    h2d = a_host.numel() * 2 + gy_host.numel() * 2
    d2h = out_host.numel() * 2 + ga_host.numel() * 2
    return e2e_ms, h2d, d2h


def _bind_host_threads_near_gpu(index: int) -> None:
    """Pin this process to the CPU cores NVML reports as local to its GPU, so that the pinned host
    buffers of the host-buffer pass are first-touched on that GPU's NUMA node (with several ranks
    on one box the default placement funnels every rank's PCIe traffic through one node).  Only
    reads device properties; any failure leaves the affinity as it was."""
    try:
        import pynvml

        pynvml.nvmlInit()
        props = torch.cuda.get_device_properties(index)
        if hasattr(props, "pci_bus_id") and hasattr(props, "pci_domain_id"):  # robust to device remapping
            bus = "%08x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
            handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        else:
            handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1}
        allowed = cpus & os.sched_getaffinity(0)
        if len(allowed) >= 4:  # never squeeze the rank's host threads onto a couple of cores
            os.sched_setaffinity(0, allowed)
    except Exception:  # noqa: BLE001 - best effort, never fatal
        pass


def run_ours(args):
    import torch.distributed as dist

    from primus_turbo_b200 import _lib
    from primus_turbo_b200.pytorch.core.low_precision import Float8QuantConfig, ScalingGranularity
    from primus_turbo_b200.pytorch.dist.expert_parallel import (
        build_exchange_plan, ep_grouped_gemm_fp8, expert_parallel_apply)
    from primus_turbo_b200.pytorch.ops import grouped_gemm_fp8

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path in the product")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1 and args.bind_cpus:
        _bind_host_threads_near_gpu(local_rank)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep stdout to the one JSON line
        if args.ep_overlap:
            # the collective that runs beside wgrad must fit on the SMs wgrad leaves free
            os.environ.setdefault("NCCL_MAX_CTAS", str(args.ep_reserve_sms))
        dist.init_process_group("nccl", device_id=dev)
        host_group = dist.new_group(backend="gloo")  # CPU group: set-up traffic and the fallback count gather
        if args.plan == "host":
            # ranks of one machine exchange their routing counts through a shared-memory board
            # (a gloo gather costs 2-4 ms per step at eight ranks and made the step host-bound)
            try:
                from primus_turbo_b200.pytorch.dist.expert_parallel import SharedCountsBoard

                host_group = SharedCountsBoard(E_TOTAL, group=host_group)
            except Exception as exc:  # noqa: BLE001 - keep the gloo group
                print(f"[bench] shared counts board unavailable ({exc!r}); using gloo", file=sys.stderr)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    assert E_TOTAL % world == 0 and ROWS % world == 0
    cfg = Float8QuantConfig(granularity=ScalingGranularity.BLOCKWISE, block_size=128)
    e_loc = E_TOTAL // world

    # ---- synthetic inputs (seeded, generated on the device that holds them) -----------------------
    counts = _counts()
    torch.manual_seed(1234 + rank)
    rows_here = ROWS // world
    if world == 1:
        counts_here = counts
    else:
        # every source rank holds ROWS/world rows whose experts are drawn i.i.d. from the same routing
        g = torch.Generator().manual_seed(100 + rank)
        idx = torch.multinomial(counts.double() / counts.sum(), rows_here, replacement=True, generator=g)
        counts_here = torch.bincount(idx, minlength=E_TOTAL).to(torch.int64)
    counts_dev = counts_here.to(dev)
    a = torch.randn(rows_here, HIDDEN, device=dev, dtype=torch.bfloat16).requires_grad_(True)
    w = (torch.randn(e_loc, N_OUT, HIDDEN, device=dev, dtype=torch.bfloat16) * 0.02).requires_grad_(True)
    gy = torch.randn(rows_here, N_OUT, device=dev, dtype=torch.bfloat16) * 1e-3
    flops_step = 3 * 2 * ROWS * N_OUT * HIDDEN  # whole job

    def step(a_in, gy_in):
        if world == 1:
            out = grouped_gemm_fp8(a_in, w, counts_dev, config=cfg)
        else:
            # the synthetic router's counts live on the host, so the exchange plan (rebuilt every
            # step, as routing changes every step in training) never waits on the device stream
            if args.plan == "host":
                plan = build_exchange_plan(counts_dev, counts_host=counts_here, host_group=host_group)
            else:
                plan = build_exchange_plan(counts_dev)
            if args.ep_overlap:
                # weight quantisation beside the dispatch, wgrad beside the return of grad_a
                out = ep_grouped_gemm_fp8(a_in, w, counts_dev, config=cfg, plan=plan, overlap=True,
                                          reserve_sms=args.ep_reserve_sms)
            else:
                out = expert_parallel_apply(
                    a_in, counts_dev, lambda rows, lens: grouped_gemm_fp8(rows, w, lens, config=cfg), plan=plan)
        ga, gw = torch.autograd.grad(out, (a_in, w), gy_in)
        return out, ga, gw

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ---------------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step(a, gy)
    barrier()
    launches0 = _lib.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks, _lib.record_kernel_times() as rec:
        barrier()
        ev0.record()
        for _ in range(args.steps):
            step(a, gy)
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = _lib.launch_count - launches0
    kernel_ms = rec.durations_ms()
    status = _lib.gemm_status()

    # ---- end to end: host buffers in, host buffers out -----------------------------------------------
    e2e_ms, h2d, d2h = float("nan"), 0, 0
    if not args.no_e2e:
        e2e_ms, h2d, d2h = _time_e2e(args, step, barrier, a, gy, rows_here, dev)

    # ---- max over ranks ---------------------------------------------------------------------------------
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])

    if rank == 0:
        peaks = _peaks()
        fp8_peak = 2.0 * peaks["bf16_tflops_sustained"]  # dense FP8 runs at twice the bf16 rate
        value = flops_step / (ms * 1e-3) / 1e12
        # Rooflines.  The launch with the largest share of the step is the wgrad instance of
        # fp8_gemm_kernel (variable-K, 2-3 contraction blocks per tile here): it must write the whole
        # bf16 weight gradient, so its roof is HBM.  The forward / dgrad instance streams the FP8
        # weights once and sits between the tensor and the HBM roof; both are reported.
        # `traffic` is dram__bytes_read + dram__bytes_write per launch from the ncu capture of the
        # 32-expert / 8192-row case (profiles/fp8_gemm_kernel_grouped_blockwise_32experts.md), scaled by
        # experts x rows (traffic is proportional to both).
        unit_factor = (E_TOTAL / world) / 32.0  # experts (and, with them, rows) per launch vs the captured case
        fwd_dgrad = kernel_ms.get("ptb_grouped_gemm_fp8", [])
        wgrad = kernel_ms.get("ptb_grouped_gemm_fp8_variable_k", [])
        wq = kernel_ms.get("ptb_quant_fp8_block2d", [])
        per_gemm_flops = 2 * ROWS * N_OUT * HIDDEN / world
        pad_rows = ROWS / world * 1.244  # segment padding of the column copies (measured on this routing)
        roof, others = None, []
        if wgrad:
            t_avg = statistics.mean(wgrad) * 1e-3
            alg_bytes = e_loc * N_OUT * HIDDEN * 2 + pad_rows * (N_OUT + HIDDEN) * (1 + 4.0 / 128)
            achieved = alg_bytes / t_avg / 1e9
            roof = {"kernel": "fp8_gemm_kernel<block 1Dx1D, bf16> (grouped wgrad launch)", "bound": "hbm",
                    "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                    "peak_source": f"copy bandwidth of MEASURED_PEAKS.json ({peaks['source']})",
                    "traffic": 1.945e9 * unit_factor, "algorithmic_bytes": alg_bytes, "avg_launch_ms": t_avg * 1e3,
                    "tflops": per_gemm_flops / t_avg / 1e12}
        if fwd_dgrad:
            t_avg = statistics.mean(fwd_dgrad) * 1e-3
            achieved = per_gemm_flops / t_avg / 1e12
            others.append({"kernel": "fp8_gemm_kernel<block 1x128 x 128x128, bf16> (grouped forward and dgrad launches)",
                           "bound": "tensor", "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s",
                           "frac": achieved / fp8_peak,
                           "peak_source": f"2 x sustained bf16 cuBLAS rate of MEASURED_PEAKS.json ({peaks['source']})",
                           "traffic": 1.230e9 * unit_factor, "avg_launch_ms": t_avg * 1e3,
                           "hbm_floor_ms": (e_loc * N_OUT * HIDDEN + (ROWS // world) * (HIDDEN + 2 * N_OUT)) /
                                           (peaks["hbm_gbs"] * 1e9) * 1e3})
        if wq:
            t_avg = statistics.mean(wq) * 1e-3
            alg_bytes = e_loc * N_OUT * HIDDEN * (3 + 4.0 / 16384)
            achieved = alg_bytes / t_avg / 1e9
            others.append({"kernel": "quant_block_kernel<128x128> (weight quantise)", "bound": "hbm", "achieved": achieved,
                           "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                           "traffic": 2.790e9 * unit_factor, "avg_launch_ms": t_avg * 1e3})
        kernels = {k: {"launches": len(v), "avg_ms": statistics.mean(v), "total_ms": sum(v)} for k, v in kernel_ms.items()}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3 operands, fp32 accumulate, bf16 in/out", "data": "synthetic",
            "config": {"workload": WORKLOAD, "experts": E_TOTAL, "experts_per_gpu": e_loc, "hidden": HIDDEN,
                       "n": N_OUT, "routed_rows": ROWS, "parallelism": f"ep{world}",
                       "ep_overlap": bool(args.ep_overlap) if world > 1 else None,
                       "load_imbalance_max_over_mean_rows": float(
                           counts.view(world, -1).sum(1).max().item() * world / counts.sum().item()),
                       "l2": "inputs larger than L2 (7.5 GB of FP8 weights per pass)"},
            "per_gpu_tflops": value / world, "pct_of_fp8_peak_per_gpu": 100.0 * value / world / fp8_peak,
            "fp8_peak_tflops": fp8_peak,
            "e2e": {"value": flops_step / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "note": "activations and grad-out from pinned host memory, out and grad-activation back to it "
                            "(copy streams overlap the neighbouring steps' kernels); weights and their gradient stay "
                            "resident"},
            "gpu_launches": launches, "kernel_ms": kernels, "gemm_status": status,
            "clocks": clocks.summary(), "roofline": roof, "roofline_other_kernels": others,
        }
        if world == 1 and not args.no_cpu_baseline:
            r = time_cpu(steps=5, warmup=1, num_experts=4)
            line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    global E_TOTAL, ROWS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer pass (profiling runs)")
    ap.add_argument("--ep-overlap", type=int, default=0,
                    help="N > 1: 1 = weight quantise beside the dispatch and wgrad beside the grad_a return "
                         "(measured slower: both sides of each pair are HBM-bound); 0 = serial")
    ap.add_argument("--plan", choices=["host", "device"], default="host",
                    help="N > 1: where the exchange plan is computed (host: gloo gather + one pinned copy; "
                         "device: NCCL gather + one host read of the split sizes)")
    ap.add_argument("--bind-cpus", type=int, default=0,
                    help="N > 1: 1 = pin each rank to the CPU cores NVML reports as local to its GPU")
    ap.add_argument("--ep-reserve-sms", type=int, default=16, help="SMs wgrad leaves to the overlapped collective")
    ap.add_argument("--experts", type=int, default=E_TOTAL, help="smaller case of the same workload (profiling)")
    ap.add_argument("--rows", type=int, default=ROWS, help="smaller case of the same workload (profiling)")
    args = ap.parse_args()
    E_TOTAL, ROWS = args.experts, args.rows
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
