"""Benchmark of the PCFG-NAT structured-loss / decoding hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this implementation
    python bench.py --impl reference ...                     # the path on the host CPU cores
    python bench.py --workload viterbi_b64 | viterbi_b1 | glance | long_seq | tiny_loss ...

The default workload ``train_batch`` is one training-shaped batch (~90 sentences, ~2.7 k target tokens,
graph length 4 x source length <= 160, vocabulary 40 000, hidden 512, fp16 decoder states and projection
weights, fp32 DP tables).  One "step" is one pass of the hot path over the batch:

    loss workloads   emissions match[b, node, t] = log P(y_t | node) (fused projection + log-softmax +
                     gather + the criterion's EOS masking), S[b] and dS[b]/dmatch, dS[b]/dlinks (inside +
                     outside pass), loss statistics for -(S_b / n_b).mean()
    glance           emissions + arg-max tokens, inside table, best-tree alignment
    viterbi_*        max log-prob / arg-max token per node, Viterbi tables, length-penalised output
                     length, back-trace to token ids on the device

Inputs are seeded synthetic tensors of the named shapes (the WMT batches the reference trains on are not
available offline).  With N > 1 every rank runs its own batch (weak scaling, as under data-parallel
training); the only collective is the 3-float all-reduce of the loss statistics (loss workloads).  One JSON
line is printed by rank 0.
"""
import argparse
import importlib
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

UNIT = "sentences/s"
# DRAM traffic of one proj_kernel launch as ncu measured it (bytes read + written), per workload captured.
NCU_TRAFFIC_BYTES = {"train_batch": 52.3e6 + 0.6e6}

METRICS = {"loss": "pcfg_loss_fwd_bwd_sentences_per_s", "glance": "pcfg_best_tree_sentences_per_s",
           "viterbi": "pcfg_viterbi_decode_sentences_per_s"}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="train_batch")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-proj-backward", action="store_true",
                    help="skip the extra measurement of the step with the projection backward")
    ap.add_argument("--nccl-reduce", action="store_true",
                    help="N > 1: sum the loss statistics with an NCCL all-reduce instead of the in-kernel exchange")
    ap.add_argument("--copy-chunks", type=int, default=2,
                    help="sentence groups the end-to-end leg sends (and projects) the decoder states in")
    ap.add_argument("--cpu-sample", type=int, default=0,
                    help="sentences per pass of the CPU baseline (0 = the whole batch of the workload)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="enqueue the step kernel by kernel instead of replaying a CUDA graph")
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
    L_b = batch.output_length.double()
    n_b = batch.target_length.double()
    kind = batch.workload.kind
    if kind == "viterbi":  # ob + links read, S + three int64 backpointer tables written
        dp = float((4.0 * L_b + 8.0 * L_b * L_b + 28.0 * L_b * torch.floor(L_b / 4)).sum())
    elif kind == "glance":  # match + links read, tree written
        dp = float((4.0 * L_b * (n_b + 2.0 * L_b) + 8.0 * L_b).sum())
    else:  # match + links read, both gradients written
        dp = float((8.0 * L_b * (n_b + 2.0 * L_b)).sum())
    return {"rows": rows, "rows_padded": batch.B * batch.L, "proj_flops": 2.0 * rows * H * V,
            "proj_flops_padded": 2.0 * batch.B * batch.L * H * V, "dp_bytes": dp}


def make_step(runtime, batch, weight, dev, use_graph, copy_chunks=2, exchange=None):
    """The public step object of the workload's kind and the host tensors it loads, in load() order."""
    kind = batch.workload.kind
    if kind == "viterbi":
        step = runtime.DecodeStep(weight, batch.B, batch.L, batch.left_tree_mask, dev, beta=1.0, pad_index=1,
                                  use_graph=use_graph, copy_chunks=copy_chunks)
        host = (batch.hidden, batch.links, batch.output_length)
    else:
        if kind == "glance":
            step = runtime.GlanceStep(weight, batch.B, batch.L, batch.T, dev, use_graph=use_graph, copy_chunks=copy_chunks)
        else:
            step = runtime.LossStep(weight, batch.B, batch.L, batch.T, dev, use_graph=use_graph, copy_chunks=copy_chunks,
                                    exchange=exchange)
        host = (batch.hidden, batch.links, batch.output_length, batch.targets, batch.target_length)
        if kind == "glance":  # decoder input of the first pass: <unk> on the graph nodes, padding after them
            pos = torch.arange(batch.L)[None, :]
            host += (torch.where(pos < batch.output_length[:, None], 3, 1),)
    return step, [t.contiguous().pin_memory() for t in host]


def run_ours(a):
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path "
                           "(use --impl reference for the CPU baseline)")
    import torch.distributed as dist

    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pkg = entry.load_package()
    ops = importlib.import_module("pcfg_nat_b200.custom_ops.pcfg_loss")
    runtime = importlib.import_module("pcfg_nat_b200.runtime")
    k = ops.get_pcfg_kernel()
    syn = pkg.synthetic

    batch = syn.make_batch(a.workload, seed=a.seed + rank)  # every rank its own batch: weak scaling
    if batch.hidden is None:
        raise RuntimeError(f"workload {a.workload} has no decoder states; the benchmark runs the projection path")
    kind = batch.workload.kind
    alg = algorithmic(batch)
    weight = batch.weight.to(dev)
    # N > 1: the loss statistics are summed over the ranks inside the statistics kernel (peer stores over
    # NVLink); --nccl-reduce uses a 12-byte NCCL all-reduce after the step instead
    exchange = None
    if world > 1 and kind == "loss" and not a.nccl_reduce:
        try:
            exchange = importlib.import_module("pcfg_nat_b200.sharding").LossExchange(dev)
        except Exception as err:  # no peer-mapped memory on this box: every rank then falls back together
            print(f"[bench] rank {rank}: in-kernel exchange unavailable ({err}); using the NCCL all-reduce", file=sys.stderr)
        agreed = torch.tensor([1 if exchange is not None else 0], device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed) == 0:
            exchange = None
    step, host = make_step(runtime, batch, weight, dev, not a.no_graph, a.copy_chunks, exchange)  # host: pinned copies
    step.load(*host)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2
    h2d = step.input_bytes()
    is_loss = kind == "loss"
    result_host = None

    def timed(n_steps, e2e):
        """Per-step CUDA-event timing on the launching stream with an L2 flush between steps."""
        nonlocal result_host
        times = []
        for _ in range(n_steps):
            flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            if e2e:  # over the copy stream, transitions last: they are still in flight while the projection runs
                step.load(*host, overlap=True)
            out = step.run()
            if is_loss and world > 1 and exchange is None:
                dist.all_reduce(out[0])
            if e2e:  # the step's result goes back to the host: loss statistics / token ids + counts / alignment
                res = (out[0],) if is_loss else ((out[0], out[1]) if kind == "viterbi" else (out[0],))
                if result_host is None:
                    result_host = [torch.empty(r.shape, dtype=r.dtype).pin_memory() for r in res]
                for h, r in zip(result_host, res):
                    h.copy_(r, non_blocking=True)
            e.record()
            times.append((s, e))
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in times]

    def timed_projection(n_steps):
        """The dominant kernel on its own (the projection call: proj_kernel and its helper launches)."""
        times = []
        for _ in range(n_steps):
            flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            if kind == "viterbi":
                k.proj_logsoftmax_gather(step.hidden, weight, None, step.output_length, None, want_max=True)
            else:
                k.proj_logsoftmax_gather(step.hidden, weight, step.targets, step.output_length, step.target_length,
                                         want_max=(kind == "glance"))
            e.record()
            times.append((s, e))
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in times]

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(a.warmup, 3)
    timed(warm, False)
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
    # the same step carried back through the projection as well (a wider step than the metric's: reported aside)
    full_ms = None
    if is_loss and kind != "glance" and world == 1 and not a.no_proj_backward:
        full = runtime.LossStep(weight, batch.B, batch.L, batch.T, dev, use_graph=not a.no_graph, proj_backward=True)
        full.load(*[t.to(dev) for t in host])
        times = []
        for i in range(3 + a.steps):
            flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            full.run()
            e.record()
            times.append((s, e))
        torch.cuda.synchronize()
        full_ms = sum(s.elapsed_time(e) for s, e in times[3:]) / a.steps
        del full
    status = ops.read_status(dev)
    d2h = sum(h.numel() * h.element_size() for h in result_host)

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
    rest_ms = max(tot[0] - tot[2], 1e-9) / a.steps
    line = {
        "metric": METRICS[kind], "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": warm,
        "ms_per_step": tot[0] / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 projection inputs, f32 accumulation and DP tables", "data": "synthetic",
        "config": {"workload": a.workload, "sentences_per_gpu": batch.B, "graph_len_max": batch.L,
                   "target_len_max": batch.T, "vocab": int(weight.shape[0]), "hidden": int(weight.shape[1]),
                   "left_tree_layer": 1, "graph_nodes_per_gpu": alg["rows"],
                   "target_tokens_per_gpu": int(batch.target_length.sum()),
                   "l2": "flushed between timed steps (256 MB write)", "cuda_graph": not a.no_graph,
                   "parallelism": f"sentence-sharded x{world}",
                   "loss_reduce": "none (one GPU)" if world == 1 or not is_loss else
                   ("in the statistics kernel, peer stores over NVLink" if exchange is not None else "NCCL all-reduce")},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": tot[1] / a.steps},
        "gpu_launches": step.kernels_per_step * a.steps,
        "roofline": {"bound": "tensor", "kernel": "proj_kernel (timed with its helper launches: row compaction + "
                                                  "target sort, partial merge)",
                     "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s", "frac": achieved / pk["tflops"],
                     "peak_source": pk["source"] + " (burst bf16 GEMM)", "traffic": NCU_TRAFFIC_BYTES.get(a.workload),
                     "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this "
                                       "workload (profiles/proj_kernel_train_batch.md)"
                     if a.workload in NCU_TRAFFIC_BYTES else None,
                     "ms_per_launch": proj_avg_s * 1e3, "flops_per_launch": alg["proj_flops"]},
        "dp": {"ms_per_step": rest_ms, "algorithmic_bytes": alg["dp_bytes"],
               "achieved_gbs": alg["dp_bytes"] / (rest_ms / 1e3) / 1e9, "hbm_peak_gbs": pk["gbs"],
               "note": "DP kernels: step time minus the separately timed projection call; latency-bound"},
        "clocks": clocks, "device_status": status,
    }
    if full_ms is not None:
        line["with_projection_backward"] = {
            "ms_per_step": full_ms, "value": sentences / (full_ms / 1e3), "unit": UNIT,
            "what": "the step plus d hidden and d weight of the projection: logits recomputed into bf16 d-logits "
                    "by proj_kernel's gradient mode, then two library bf16 GEMMs over the padded rows"}
    if rank == 0:
        if world == 1 and not a.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(a, batch)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def cpu_pass(sub, kind, syn):
    """One pass of the step over the sentences of ``sub`` on the host cores; returns (seconds, what ran)."""
    import numpy as np

    import oracle

    n = sub.B
    t0 = time.perf_counter()
    logits = sub.hidden.float().reshape(-1, sub.hidden.shape[-1]) @ sub.weight.float().t()
    lp = torch.log_softmax(logits, -1).view(n, sub.L, -1)
    l_np, ol = sub.links.numpy(), sub.output_length.numpy()
    if kind == "viterbi":
        ob, tok = lp.max(-1)
        S, R, Lt, Mt = oracle.pcfg_viterbi(ob.numpy(), l_np, ol)
        sc = torch.from_numpy(S[:, 1, :]) / torch.arange(sub.L // 4).unsqueeze(0)
        sc = torch.where(torch.isnan(sc), torch.full_like(sc, float("-inf")), sc)
        pred = sc[:, 1:].max(-1)[1] + 1
        oracle.viterbi_decoding(pred.numpy(), ol, Lt, R, Mt, tok.numpy(), sub.left_tree_mask.long().numpy(), 1)
        what = "torch CPU fp32 GEMM + log-softmax + max, C oracle Viterbi tables + back-trace"
    else:
        match = lp.gather(2, sub.targets[:, None, :].expand(-1, sub.L, -1)).contiguous()
        syn.eos_mask_(match, sub.output_length, sub.target_length)
        m_np, tl = match.numpy(), sub.target_length.numpy()
        S, C = oracle.pcfg_loss(m_np, l_np, ol, tl)
        if kind == "glance":
            oracle.pcfg_best_tree(S, C, m_np, l_np, ol, tl)
            what = "torch CPU fp32 GEMM + log-softmax + gather, C oracle inside pass + best tree"
        else:
            oracle.pcfg_loss_backward(np.ones(n, np.float32), S, C, m_np, l_np, ol, tl)
            what = "torch CPU fp32 GEMM + log-softmax + gather, C oracle loss forward + backward"
    return time.perf_counter() - t0, what


def cpu_sample(a, batch):
    import oracle

    pkg = entry.load_package()
    syn = pkg.synthetic
    if batch is None:
        batch = syn.make_batch(a.workload, seed=a.seed)
    n = batch.B if a.cpu_sample <= 0 else min(a.cpu_sample, batch.B)
    sub = batch.select(list(range(n)))
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    oracle.lib()
    return syn, batch, sub, n, cores


def cpu_baseline(a, batch=None, budget_s=10.0):
    """The same step on the host cores: the C oracle (a port of the reference kernels; the reference has
    no CPU implementation of this path) with OpenMP over sentences, and torch's CPU GEMM for the
    projection.  One warm-up pass, then passes over the sample until ``budget_s`` seconds are spent."""
    syn, batch, sub, n, cores = cpu_sample(a, batch)
    kind = batch.workload.kind
    cpu_pass(sub, kind, syn)
    times, what = [], ""
    while len(times) < 2 or (sum(times) < budget_s and len(times) < 200):
        dt, what = cpu_pass(sub, kind, syn)
        times.append(dt)
    med = sorted(times)[len(times) // 2]
    return {"value": n / med, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{n} of {batch.B} sentences of {a.workload} per pass ({what}); median of {len(times)} passes "
                      f"after 1 warm-up pass, {med:.3f} s per pass, {sum(times):.1f} s in all"}


def run_reference(a):
    """The reference arm: the path's CPU implementation (the oracle port: the reference itself has none) on
    all host cores, W warm-up passes and K timed passes over the workload's batch (a pass = a step; the number
    of timed passes is cut so that the run stays within about two minutes)."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    syn, batch, sub, n, cores = cpu_sample(a, None)
    kind = batch.workload.kind
    for _ in range(max(1, min(a.warmup, 3))):
        cpu_pass(sub, kind, syn)
    times, what = [], ""
    while len(times) < max(a.steps, 1) and (len(times) < 2 or sum(times) < 120.0):
        dt, what = cpu_pass(sub, kind, syn)
        times.append(dt)
    mean = sum(times) / len(times)
    value = n / mean
    cb = {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
          "sample": f"{n} of {batch.B} sentences of {a.workload} per step ({what}); {len(times)} timed steps of "
                    f"{a.steps} asked, {mean:.3f} s per step"}
    line = {"impl": "reference", "metric": METRICS[kind], "value": value, "unit": UNIT, "n_gpus": a.gpus,
            "steps": len(times), "warmup": a.warmup, "ms_per_step": mean * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32 on the CPU", "data": "synthetic",
            "config": {"workload": a.workload, "sentences_per_gpu": batch.B, "graph_len_max": batch.L,
                       "target_len_max": batch.T, "vocab": int(batch.weight.shape[0]),
                       "hidden": int(batch.weight.shape[1]), "left_tree_layer": 1,
                       "parallelism": "host cores of rank 0 only"},
            "cpu_baseline": cb,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)
