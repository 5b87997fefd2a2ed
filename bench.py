"""Benchmark of the PCFG-NAT structured-loss hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this implementation
    python bench.py --impl reference ...                     # the path on the host CPU cores

One "step" is one pass of the hot path over one training-shaped batch (workload
``train_batch``: ~90 sentences, graph length 4 x source length <= 160, vocabulary 40 000,
hidden 512, fp16 decoder states and projection weights, fp32 DP tables):

    emissions  match[b, node, t] = log P(y_t | node)    fused projection + log-softmax + gather
                                                         (+ the criterion's EOS masking)
    loss       S[b] and d S[b] / d match, d S[b] / d links   inside + outside pass
    scalar     -(S_b / n_b).mean() with invalid sentences masked and counted

Inputs are seeded synthetic tensors of the named shapes (the WMT batches the reference
trains on are not available offline).  With N > 1 every rank runs its own batch (weak
scaling, as under data-parallel training); the only collective is the 3-float all-reduce
of the loss statistics.  One JSON line is printed by rank 0.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

METRIC = "pcfg_loss_fwd_bwd_sentences_per_s"
UNIT = "sentences/s"
KERNELS_PER_STEP = 7  # sort_targets, proj, proj_merge, proj_poison_bad_targets, loss_fwd, outside, grad


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="train_batch")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--cpu-sample", type=int, default=8, help="sentences in the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="enqueue the step kernel by kernel instead of replaying a CUDA graph")
    return ap.parse_args()


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        d = json.load(open(p))
        return {"tflops": float(d["bf16_tflops"]), "gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) in a thread while the timed
    region runs; only samples taken between mark_begin() and mark_end() are reported."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index, period_s=0.002):
        self.index, self.period, self.rows = index, period_s, []
        self.stop_flag, self.active, self.thread, self.err = False, False, None, None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = self.index
            if vis:
                try:
                    phys = int(vis.split(",")[self.index])
                except (ValueError, IndexError):
                    phys = self.index
            self.nv, self.h = pynvml, pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # NVML missing: report it, do not fail the benchmark
            self.err = repr(e)
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _loop(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                why = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                if self.active:
                    self.rows.append((float(mhz), int(why)))
            except Exception as e:
                self.err = repr(e)
                return
            time.sleep(self.period)

    def mark_begin(self):
        self.active = True

    def mark_end(self):
        self.active = False

    def stop(self):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=5)
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": getattr(self, "max_mhz", None), "samples": 0,
                    "reasons": [], "note": self.err or "no sample fell inside the timed region"}
        sm = [r[0] for r in self.rows]
        bits = 0
        for r in self.rows:
            bits |= r[1]
        return {"sm_mhz": statistics.median(sm), "sm_min_mhz": min(sm), "sm_max_mhz": self.max_mhz, "samples": len(sm),
                "reasons": sorted(n for n, b in self.REASONS.items() if bits & b)}


def algorithmic(batch):
    """Algorithmic work of one step from the unpadded sentence lengths."""
    V, H = batch.weight.shape
    rows = int(batch.output_length.sum())
    flops_proj = 2.0 * rows * H * V
    L_b = batch.output_length.double()
    n_b = batch.target_length.double()
    bytes_dp = float((8.0 * L_b * (n_b + 2.0 * L_b)).sum())  # read match + links, write both gradients
    return {"rows": rows, "rows_padded": batch.B * batch.L, "proj_flops": flops_proj,
            "proj_flops_padded": 2.0 * batch.B * batch.L * H * V, "dp_bytes": bytes_dp}


def run_ours(a):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU baseline)")
    import torch.distributed as dist

    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = entry.load_package()
    import importlib

    ops = importlib.import_module("pcfg_nat_b200.custom_ops.pcfg_loss")
    runtime = importlib.import_module("pcfg_nat_b200.runtime")
    k = ops.get_pcfg_kernel()
    syn = pkg.synthetic

    batch = syn.make_batch(a.workload, seed=a.seed + rank)  # every rank its own batch: weak scaling
    alg = algorithmic(batch)
    # host copies in pinned memory: the end-to-end leg copies them to the device every step
    host = [t.contiguous().pin_memory() for t in (batch.hidden, batch.links, batch.targets, batch.output_length,
                                                  batch.target_length)]
    weight = batch.weight.to(dev)
    # the public step object: fused projection -> loss forward+backward -> loss statistics, replayed as one CUDA graph
    step = runtime.LossStep(weight, batch.B, batch.L, batch.T, dev, use_graph=not a.no_graph)
    step.load(*host)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2
    h2d = step.input_bytes()
    loss_host = torch.empty(3, dtype=torch.float32).pin_memory()

    def timed(n_steps, e2e):
        """Per-step CUDA-event timing on the launching stream with an L2 flush between steps."""
        times = []
        for _ in range(n_steps):
            flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            if e2e:
                step.load(*host)
            stats = step.run()[0]
            if world > 1:
                dist.all_reduce(stats)
            if e2e:
                loss_host.copy_(stats, non_blocking=True)
            e.record()
            times.append((s, e))
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in times]

    def timed_projection(n_steps):
        """The dominant kernel on its own (the projection call: sort, proj_kernel, merge, poison), for the roofline."""
        times = []
        for _ in range(n_steps):
            flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            k.proj_logsoftmax_gather(step.hidden, weight, step.targets, step.output_length, step.target_length)
            e.record()
            times.append((s, e))
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in times]

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    timed(max(a.warmup, 3), False)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    sync_all()
    sampler.mark_begin()
    step_ms = timed(a.steps, False)
    sync_all()
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    timed(3, True)
    sync_all()
    e2e_ms = timed(a.steps, True)
    sync_all()
    timed_projection(3)
    proj_ms = timed_projection(a.steps)
    sync_all()
    status = ops.read_status(dev)

    tot = torch.tensor([sum(step_ms), sum(e2e_ms), sum(proj_ms)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tot, op=dist.ReduceOp.MAX)
    tot = tot.tolist()
    sentences = batch.B * world  # same batch size on every rank
    value = sentences * a.steps / (tot[0] / 1e3)
    e2e_value = sentences * a.steps / (tot[1] / 1e3)
    pk = peaks()
    proj_avg_s = (tot[2] / a.steps) / 1e3
    achieved = alg["proj_flops"] / proj_avg_s / 1e12
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3),
        "ms_per_step": tot[0] / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 projection inputs, f32 accumulation and DP tables", "data": "synthetic",
        "config": {"workload": a.workload, "sentences_per_gpu": batch.B, "graph_len_max": batch.L,
                   "target_len_max": batch.T, "vocab": int(weight.shape[0]), "hidden": int(weight.shape[1]),
                   "left_tree_layer": 1, "target_tokens_per_gpu": int(batch.target_length.sum()),
                   "l2": "flushed between timed steps (256 MB write)", "cuda_graph": not a.no_graph, "parallelism": f"sentence-sharded x{world}"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 12,
                "ms_per_step": tot[1] / a.steps},
        "gpu_launches": KERNELS_PER_STEP * a.steps,
        "roofline": {"bound": "tensor", "kernel": "proj_kernel (+ its 3 helper launches)", "achieved": achieved,
                     "peak": pk["tflops"], "unit": "TFLOP/s", "frac": achieved / pk["tflops"],
                     "peak_source": pk["source"] + " (burst bf16 GEMM)", "traffic": None,
                     "ms_per_launch": proj_avg_s * 1e3, "flops_per_launch": alg["proj_flops"],
                     "achieved_padded_rows": alg["proj_flops_padded"] / proj_avg_s / 1e12},
        "dp": {"ms_per_step": (tot[0] - tot[2]) / a.steps, "algorithmic_bytes": alg["dp_bytes"],
               "achieved_gbs": alg["dp_bytes"] / (max(tot[0] - tot[2], 1e-9) / a.steps / 1e3) / 1e9,
               "hbm_peak_gbs": pk["gbs"], "note": "step time minus the separately timed projection call"},
        "clocks": clocks, "device_status": status,
    }
    if rank == 0:
        if world == 1 and not a.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(a, batch)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def cpu_baseline(a, batch=None, steps=1):
    """The same step on the host cores: the C oracle (a port of the reference kernels; the reference
    has no CPU implementation of this path) with OpenMP over sentences, and torch's CPU GEMM for
    the projection, on a bounded sample of the workload's sentences."""
    import numpy as np

    import oracle

    pkg = entry.load_package()
    syn = pkg.synthetic
    if batch is None:
        batch = syn.make_batch(a.workload, seed=a.seed)
    n = min(a.cpu_sample, batch.B)
    sub = batch.select(list(range(n)))
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    oracle.lib()
    best = None
    for _ in range(max(steps, 1)):
        t0 = time.perf_counter()
        logits = sub.hidden.float().reshape(-1, sub.hidden.shape[-1]) @ sub.weight.float().t()
        lp = torch.log_softmax(logits, -1).view(n, sub.L, -1)
        match = lp.gather(2, sub.targets[:, None, :].expand(-1, sub.L, -1)).contiguous()
        syn.eos_mask_(match, sub.output_length, sub.target_length)
        m_np, l_np = match.numpy(), sub.links.numpy()
        ol, tl = sub.output_length.numpy(), sub.target_length.numpy()
        S, C = oracle.pcfg_loss(m_np, l_np, ol, tl)
        oracle.pcfg_loss_backward(np.ones(n, np.float32), S, C, m_np, l_np, ol, tl)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return {"value": n / best, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"first {n} of {batch.B} sentences of {a.workload} (projection with torch CPU fp32 GEMM, "
                      f"log-softmax + gather, C oracle loss forward + backward); best of {max(steps, 1)} passes, "
                      f"{best:.3f} s per pass"}


def run_reference(a):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    cb = cpu_baseline(a, None, steps=max(1, min(a.steps, 3)))
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": a.gpus,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 on the CPU", "data": "synthetic",
            "config": {"workload": a.workload}, "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
