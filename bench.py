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
    glance           emissions + arg-max tokens, inside table, best-tree alignment, glancing sampler
    viterbi_*        max log-prob / arg-max token per node, Viterbi tables, length-penalised output
                     length, back-trace to token ids on the device

The headline ``value`` is the median of several blocks of K timed steps (each block bracketed by a barrier
and a device synchronisation, every step timed by CUDA events on the launching stream, L2 flushed between
steps).  The default run also reports, as sub-records of the same JSON line:

    workloads      the other configurations of the metric (Viterbi decode at batch 64 and 1, the glancing
                   pass, long sequences), each with its own value / e2e / roofline / cpu_baseline
    strong         N > 1: ONE global batch of long_seq, glance and viterbi_b64 split by sentence over the ranks
                   (cost-balanced), sentences/s of the global batch
    gpu_reference  N = 1: the unmodified reference kernels (built for sm_100a beside the oracle) on the same
                   inputs, CUDA-event timed, where that build is present
    drop_in        N = 1: the same chain through this package's five reference-named operators on materialised
                   logits (what an unmodified criterion / model calls)

Inputs are seeded synthetic tensors of the named shapes (the WMT batches the reference trains on are not
available offline).  With N > 1 every rank runs its own batch for the headline (weak scaling, as under
data-parallel training); the only exchange is the sum of the three loss statistics.  One JSON line is printed
by rank 0.
"""
import argparse
import importlib
import json
import math
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

METRICS = {"loss": "pcfg_loss_fwd_bwd_sentences_per_s", "glance": "pcfg_best_tree_sentences_per_s",
           "viterbi": "pcfg_viterbi_decode_sentences_per_s"}
DTYPE = "f16 projection inputs, f32 accumulation and DP tables"
# train_batch_model_graph: the training batch with the graph size the reference model really builds (8 * source + 2
# nodes, twice the headline's 4 * source)
SUB_WORKLOADS = ["viterbi_b64", "viterbi_b1", "glance", "long_seq", "train_batch_model_graph"]
STRONG_WORKLOADS = ["long_seq", "glance", "viterbi_b64"]
# sentences per pass of the CPU baseline for the sub-records (bounded samples of the workload)
CPU_SAMPLE = {"viterbi_b64": 16, "viterbi_b1": 1, "glance": 16, "long_seq": 8, "train_batch_model_graph": 16}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="train_batch")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--blocks", type=int, default=0,
                    help="timed blocks of --steps steps (0 = as many as make 0.25 s of device time, 5..50)")
    ap.add_argument("--no-subs", action="store_true",
                    help="only the headline workload: no workloads / strong / gpu_reference / drop_in records")
    ap.add_argument("--drop-in-only", action="store_true",
                    help="N = 1: only the drop_in record of --workload (the reference-named operators on materialised "
                         "logits, with the log-softmax + gather kernel timed alone), printed as one JSON line")
    ap.add_argument("--no-proj-backward", action="store_true",
                    help="skip the extra measurement of the step with the projection backward")
    ap.add_argument("--nccl-reduce", action="store_true",
                    help="N > 1: sum the loss statistics with an NCCL all-reduce instead of the in-kernel exchange")
    ap.add_argument("--copy-chunks", type=int, default=2,
                    help="sentence groups the end-to-end leg sends (and projects) the decoder states in")
    ap.add_argument("--fetch", default="auto", choices=["auto", "none", "links", "all"],
                    help="what the end-to-end leg fetches from the host buffers by kernel instead of by copy engine")
    ap.add_argument("--copy-real-rows", type=int, default=-1,
                    help="copies per sentence group that send the decoder states without most padding rows "
                         "(-1 = the step objects' default, 0 = the whole padded tensor)")
    ap.add_argument("--pipeline-depth", type=int, default=2,
                    help="step objects the end-to-end leg uses in turn (batches in flight)")
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
        return {"tflops": float(d["bf16_tflops"]), "gbs": float(d["hbm_gbs"]), "source": "measured",
                "tflops_sustained": float(d.get("bf16_tflops_sustained", 0.0)) or None}
    return {"tflops": 1590.0, "gbs": 6650.0, "source": "fallback", "tflops_sustained": 1400.0}


def ncu_traffic(workload, kernel):
    """DRAM bytes (read + written) of one launch of ``kernel`` on ``workload`` from the committed ncu captures
    (profiles/ncu_traffic.json).  A record counts only while the kernel's source file still has the hash it
    had when captured; otherwise (or with no record) the traffic is reported as unknown."""
    import hashlib

    try:
        rec = json.load(open(os.path.join(ROOT, "profiles", "ncu_traffic.json"))).get(f"{workload}:{kernel}")
        if not rec:
            return None, None
        with open(os.path.join(ROOT, rec["kernel_source"]), "rb") as f:
            if hashlib.sha1(f.read()).hexdigest() != rec["sha1"]:
                return None, "the capture on record is of an older build of this kernel"
        return float(rec["dram_bytes"]), rec.get("source")
    except (OSError, ValueError, KeyError):
        return None, None


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


def config_of(name, batch):
    """What names the workload; the same dictionary in both arms."""
    return {"workload": name, "sentences_per_gpu": batch.B, "graph_len_max": batch.L, "target_len_max": batch.T,
            "vocab": int(batch.weight.shape[0]), "hidden": int(batch.weight.shape[1]), "left_tree_layer": 1}


def make_step(runtime, batch, weight, dev, use_graph, copy_chunks=2, exchange=None, B=None, L=None, T=None):
    """The public step object of the workload's kind and the host tensors it loads, in load() order.
    B, L, T: static shape of the step when it must be larger than the batch (padded with empty sentences)."""
    kind = batch.workload.kind
    B = batch.B if B is None else B
    L = batch.L if L is None else L
    T = batch.T if T is None else T
    if kind == "viterbi":
        step = runtime.DecodeStep(weight, B, L, batch.left_tree_mask, dev, beta=1.0, pad_index=1,
                                  use_graph=use_graph, copy_chunks=copy_chunks)
        host = (batch.hidden, batch.links, batch.output_length)
    else:
        if kind == "glance":
            step = runtime.GlanceStep(weight, B, L, T, dev, use_graph=use_graph, copy_chunks=copy_chunks)
        else:
            step = runtime.LossStep(weight, B, L, T, dev, use_graph=use_graph, copy_chunks=copy_chunks,
                                    exchange=exchange)
        host = (batch.hidden, batch.links, batch.output_length, batch.targets, batch.target_length)
        if kind == "glance":  # decoder input of the first pass: <unk> on the graph nodes, padding after them
            pos = torch.arange(batch.L)[None, :]
            host += (torch.where(pos < batch.output_length[:, None], 3, 1),)
    return step, [t.contiguous().pin_memory() for t in host]


class Ctx:
    """Per-process state of the benchmark run."""

    def __init__(self, a):
        import torch.distributed as dist

        self.a, self.dist = a, dist
        self.rank = int(os.environ.get("RANK", 0))
        self.world = int(os.environ.get("WORLD_SIZE", 1))
        self.local = int(os.environ.get("LOCAL_RANK", 0))
        self.dev = torch.device("cuda", self.local)
        torch.cuda.set_device(self.dev)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.pkg = entry.load_package()
        self.ops = importlib.import_module("pcfg_nat_b200.custom_ops.pcfg_loss")
        self.runtime = importlib.import_module("pcfg_nat_b200.runtime")
        self.sharding = importlib.import_module("pcfg_nat_b200.sharding")
        self.kernel = self.ops.get_pcfg_kernel()
        self.syn = self.pkg.synthetic
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)  # > 126 MB L2
        self.pk = peaks()
        self.weights = {}

    def weight(self, batch):
        """The projection matrix on the device; the workloads of one seed share it when it is the same tensor."""
        key = (tuple(batch.weight.shape), float(batch.weight[0, 0]), float(batch.weight[-1, -1]))
        if key not in self.weights:
            self.weights = {key: batch.weight.to(self.dev)}
        return self.weights[key]

    def sync_all(self):
        torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = torch.tensor(values, dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()


def n_blocks(a, step_ms, lo=5, hi=50):
    if a.blocks > 0:
        return a.blocks
    return max(lo, min(hi, int(math.ceil(250.0 / max(step_ms * a.steps, 1e-3)))))


def measure(ctx, name, batch, global_sentences, steps, warm, blocks=None, exchange=None, sampler=None,
            static_shape=None):
    """Times the step of ``batch`` on this rank: device-resident (value), end to end from pinned host memory
    (e2e), the projection call alone (roofline) and the host-to-device copies alone.  Block times are the
    maximum over the ranks.  Returns the record and the step object (for checks after the timed region)."""
    a, dev = ctx.a, ctx.dev
    kind = batch.workload.kind
    is_loss = kind == "loss"
    alg = algorithmic(batch)
    weight = ctx.weight(batch)
    shape = static_shape or {}
    step, host = make_step(ctx.runtime, batch, weight, dev, not a.no_graph, a.copy_chunks, exchange, **shape)
    if shape:  # a shard smaller than the static shape: the rest are empty sentences
        host = pad_host(batch, host, step)
    step.load(*host)
    h2d = step.input_bytes()
    flush, k = ctx.flush, ctx.kernel
    result_host = []

    def one_step(e2e):
        flush.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        if e2e:  # over the copy stream, transitions last: they are still in flight while the projection runs
            step.load(*host, overlap=True)
        out = step.run()
        if is_loss and ctx.world > 1 and exchange is None:
            ctx.dist.all_reduce(out[0])
        if e2e:  # the step's result goes back to the host: loss statistics / token ids + counts / alignment
            res = (out[0],) if is_loss else ((out[0], out[1]) if kind == "viterbi" else (out[0],))
            if not result_host:
                result_host.extend(torch.empty(r.shape, dtype=r.dtype).pin_memory() for r in res)
            for h, r in zip(result_host, res):
                h.copy_(r, non_blocking=True)
        e.record()
        return s, e

    def block(n_steps, e2e):
        """n_steps timed steps between two barriers; returns this rank's summed step time in ms."""
        ctx.sync_all()
        ev = [one_step(e2e) for _ in range(n_steps)]
        ctx.sync_all()
        return sum(s.elapsed_time(e) for s, e in ev)

    def projection_block(n_steps):
        ev = []
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
            ev.append((s, e))
        torch.cuda.synchronize()
        return sum(s.elapsed_time(e) for s, e in ev)

    def copy_block(n_steps):
        """The host-to-device copies of one load alone (no kernels)."""
        ev = []
        for _ in range(n_steps):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            step.load(*host)
            e.record()
            ev.append((s, e))
        torch.cuda.synchronize()
        return sum(s.elapsed_time(e) for s, e in ev)

    block(warm, False)
    est = ctx.max_over_ranks([block(min(steps, 5), False) / min(steps, 5)])[0]
    nb = blocks or n_blocks(a, est)  # the same count on every rank: blocks are bracketed by barriers
    if sampler is not None:
        sampler.mark_begin()
    dev_ms = [block(steps, False) for _ in range(nb)]
    if sampler is not None:
        sampler.mark_end()
    # the projection call alone, straight after the blocks it is a part of: in the same thermal and power state
    projection_block(3)
    proj_ms = [projection_block(steps) for _ in range(min(nb, 5))]
    block(3, True)
    serial_ms = [block(steps, True) for _ in range(min(nb, 5))]  # load -> run -> read-back, one batch at a time
    # the end-to-end figure: two step objects in turn, so that batch i + 1 is copied while batch i is computed
    # several GPUs pulling from one host share its bus (24 GB/s per rank at N = 8 against 44-49 alone), so there the
    # transitions are fetched by the kernel that moves only the entries the kernels read (measured at N = 8: 984k
    # sentences/s against 761k with copies alone; on one GPU both give the same 175k)
    fetch = a.fetch if a.fetch != "auto" else ("links" if ctx.world > 1 else "none")
    pipe = ctx.runtime.PipelinedStep(lambda: make_step(ctx.runtime, batch, weight, dev, not a.no_graph, a.copy_chunks,
                                                       exchange, **shape)[0],
                                     fetch_from_host=None if fetch == "none" else fetch,
                                     depth=a.pipeline_depth) if not a.no_graph else None
    if pipe is not None:
        # copies per sentence group that skip padding rows of the decoder states: the step objects' default (8) keeps
        # the host's issue time below the step on one GPU; with eight GPUs on one host the bus is what is short and
        # more, smaller copies pay (measured at N = 8: 1 074k / 1 142k / 1 153k sentences/s with 8 / 16 / 32)
        real_rows = a.copy_real_rows if a.copy_real_rows >= 0 else (32 if ctx.world >= 8 else -1)
        if real_rows >= 0:
            for st in pipe.steps:
                st.copy_real_rows = real_rows
        step_single = step
        step = pipe
        pipe.load(*host)
        pipe.run()
        pipe.load(*host)
        pipe.run()
        torch.cuda.synchronize()

        def one_step_piped():
            flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            pipe.load(*host)
            out = pipe.run()
            if is_loss and ctx.world > 1 and exchange is None:
                ctx.dist.all_reduce(out[0])
            res = (out[0],) if is_loss else ((out[0], out[1]) if kind == "viterbi" else (out[0],))
            for h, r in zip(result_host, res):
                h.copy_(r, non_blocking=True)
            e.record()
            return s, e

        def block_piped(n_steps):
            ctx.sync_all()
            ev = [one_step_piped() for _ in range(n_steps)]
            ctx.sync_all()
            return sum(s.elapsed_time(e) for s, e in ev)

        block_piped(3)
        e2e_ms = [block_piped(steps) for _ in range(nb)]
        h2d = pipe.input_bytes()
        copies_per_group = pipe.steps[0].copy_real_rows
        step = step_single
        del pipe
        pipe_used = True
    else:
        e2e_ms = serial_ms
        copies_per_group = None
        pipe_used = False
    copy_block(2)
    copy_ms = copy_block(min(steps, 10)) / min(steps, 10)
    step.load(*host)
    last = step.run()
    torch.cuda.synchronize()

    dev_ms = ctx.max_over_ranks(dev_ms)
    e2e_ms = ctx.max_over_ranks(e2e_ms)
    serial_ms = ctx.max_over_ranks(serial_ms)
    proj_med, copy_max = ctx.max_over_ranks([statistics.median(proj_ms), copy_ms])
    med, e2e_med = statistics.median(dev_ms), statistics.median(e2e_ms)
    per_s = lambda ms: global_sentences * steps / (ms / 1e3)
    proj_s = proj_med / steps / 1e3
    achieved = alg["proj_flops"] / proj_s / 1e12
    pk = ctx.pk
    rest_ms = max(med - proj_med, 1e-9) / steps
    traffic, traffic_src = ncu_traffic(name, "proj_kernel")
    d2h = sum(h.numel() * h.element_size() for h in result_host)
    rec = {
        "metric": METRICS[kind], "value": per_s(med), "unit": UNIT, "ms_per_step": med / steps,
        "blocks": nb, "spread": {"min": per_s(max(dev_ms)), "max": per_s(min(dev_ms))},
        "config": config_of(name, batch),
        "e2e": {"value": per_s(e2e_med), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_med / steps, "spread": {"min": per_s(max(e2e_ms)), "max": per_s(min(e2e_ms))},
                "copy_ms": copy_max, "h2d_gbs": h2d / (copy_max / 1e3) / 1e9,
                "how": "every step copies its inputs from pinned host memory and reads its result back; two step "
                       "objects in turn, so that the copies of batch i + 1 run while batch i is computed",
                "fetch_by_kernel": fetch if pipe_used else "none",
                "copies_per_sentence_group": copies_per_group,
                "one_batch_at_a_time": {"value": per_s(statistics.median(serial_ms)),
                                        "ms_per_step": statistics.median(serial_ms) / steps},
                "bound": "host-to-device copies (PCIe)" if copy_max > e2e_med / steps * 0.95 else "device time"},
        "gpu_launches": step.kernels_per_step * steps,
        "roofline": {"bound": "tensor", "kernel": "proj_kernel (timed with its helper launches: row compaction + "
                                                  "target sort, partial merge)",
                     "achieved": achieved, "peak": pk["tflops"], "unit": "TFLOP/s", "frac": achieved / pk["tflops"],
                     "peak_source": pk["source"] + " (burst bf16 GEMM)",
                     # the call is timed straight after seconds of back-to-back steps, i.e. under the power cap the
                     # sustained figure was taken under: that fraction beside the conservative one against the burst
                     "peak_sustained": pk["tflops_sustained"],
                     "frac_of_sustained": achieved / pk["tflops_sustained"] if pk["tflops_sustained"] else None,
                     "traffic": traffic,
                     "traffic_source": traffic_src, "ms_per_launch": proj_s * 1e3, "flops_per_launch": alg["proj_flops"]},
        "dp": {"bound": "hbm", "ms_per_step": rest_ms, "algorithmic_bytes": alg["dp_bytes"],
               "achieved": alg["dp_bytes"] / (rest_ms / 1e3) / 1e9, "peak": pk["gbs"], "unit": "GB/s",
               "frac": alg["dp_bytes"] / (rest_ms / 1e3) / 1e9 / pk["gbs"],
               "share_of_step": rest_ms / (med / steps),
               "note": "DP kernels: step time minus the separately timed projection call; a chain of dependent "
                       "steps per sentence (latency-bound)"},
        "run": {"graph_nodes_per_gpu": alg["rows"], "target_tokens_per_gpu": int(batch.target_length.sum()),
                "l2": "flushed between timed steps (256 MB write)", "cuda_graph": not a.no_graph,
                "copy_chunks": a.copy_chunks},
    }
    return rec, step, host, last


def pad_host(batch, host, step):
    """Pads a shard's pinned host tensors with empty sentences up to the step's static batch size."""
    out = []
    for t, buf in zip(host, step._inputs()):
        if tuple(t.shape) == tuple(buf.shape):
            out.append(t)
            continue
        if buf is step.links:
            p = torch.full(tuple(buf.shape), float("-inf"), dtype=t.dtype)
            p[:t.shape[0], :t.shape[1], :, :t.shape[3]] = t
        else:
            fill = 2 if buf is step.output_length else (1 if t.dtype == torch.int64 else 0)
            p = torch.full(tuple(buf.shape), fill, dtype=t.dtype)
            p[tuple(slice(0, s) for s in t.shape)] = t
        out.append(p.pin_memory())
    return out


def exchange_check(ctx, step, last):
    """N > 1, after the timed region: the statistics the in-kernel exchange returned against an NCCL
    all-reduce of the ranks' local statistics."""
    local = ctx.sharding.local_loss_stats(last[3], step.target_length).clone()
    ctx.dist.all_reduce(local)
    diff = float((local.double() - last[0].double()).abs().max())
    scale = float(local.double().abs().max())
    return {"max_abs_diff": diff, "ok": bool(diff <= 1e-5 * max(scale, 1.0)), "sentences": float(last[0][1]),
            "how": "dist.all_reduce(local_loss_stats) vs the statistics of the step's last run"}


def strong_records(ctx, steps, warm):
    """One global batch per workload, split by sentence over the ranks (cost-balanced); every rank pads its
    shard to the largest shard so that all ranks replay the same static shape."""
    out = {}
    for name in STRONG_WORKLOADS:
        g = ctx.syn.make_batch(name, seed=ctx.a.seed)
        cost = ctx.sharding.sentence_cost(g.output_length, g.target_length if g.workload.kind != "viterbi" else None)
        shards = ctx.sharding.shard_sentences(cost.tolist(), ctx.world)
        mine = g.select(shards[ctx.rank]) if shards[ctx.rank] else None
        Bs = max(1, max(len(s) for s in shards))
        if mine is None:  # more ranks than sentences: this rank runs an empty step of the same shape
            mine = g.select([0])
            mine.output_length[:] = 2
            mine.target_length[:] = 1
            mine.links[:] = float("-inf")
        rec, step, _, _ = measure(ctx, name, mine, g.B, steps, warm, blocks=5,
                                  static_shape={"B": Bs, "L": g.L, "T": g.T})
        rec["scaling"] = "strong"
        rec["global_sentences"] = g.B
        rec["sentences_per_rank"] = [len(s) for s in shards]
        for key in ("roofline", "dp", "blocks"):
            rec.pop(key, None)
        out[name] = rec
        del step
        torch.cuda.empty_cache()
    return out


def ref_module():
    from oracle.build_ref import load_ref, ref_so_path

    if not os.path.isfile(ref_so_path()):
        return None
    return load_ref()


def gpu_reference(ctx, name, batch, steps):
    """The unmodified reference kernels on the same inputs, CUDA-event timed: fp16 ``F.linear`` -> reference
    ``logsoftmax_gather`` -> EOS mask -> reference ``pcfg_loss`` + ``pcfg_loss_backward`` (loss workloads) /
    ``pcfg_best_tree`` (glance) / torch ``log_softmax().max()`` -> reference ``pcfg_viterbi`` -> length choice ->
    three device-to-host copies -> reference host ``viterbi_decoding`` (decode).  Only shapes with at most
    128 main-chain nodes per sentence are run: every reference launch then has one row segment per sentence and
    none of its unbounded inter-block waits depends on another block."""
    ref = ref_module()
    if ref is None:
        return {"unavailable": "reference extension not built (oracle/_ref absent)"}
    if batch.L > 256:
        return {"unavailable": "graph length > 256: the reference kernels' inter-block spin-waits have no bound there"}
    import torch.nn.functional as F

    dev, syn = ctx.dev, ctx.syn
    kind = batch.workload.kind
    weight = ctx.weight(batch)
    hid, lk, ol = batch.hidden.to(dev), batch.links.to(dev), batch.output_length.to(dev)
    B, L = batch.B, batch.L
    rows = torch.arange(B, device=dev)
    if kind != "viterbi":
        tg, tl = batch.targets.to(dev), batch.target_length.to(dev)
        sel = tg.unsqueeze(1).expand(-1, L, -1)
        ones = torch.ones(B, device=dev)
    else:
        mask_cpu = batch.left_tree_mask.long()
        pen = torch.arange(L // 4, device=dev).unsqueeze(0).float()

    def chain():
        logits = F.linear(hid, weight)
        if kind == "viterbi":
            ob, tok = logits.float().log_softmax(-1).max(-1)
            S, R, Lt, Mt = ref.pcfg_viterbi(ob, lk, ol, 1)
            sc = S[rows, 1, :] / pen
            sc = torch.where(sc.isnan(), torch.full_like(sc, float("-inf")), sc)
            pred = sc[:, 1:].max(-1)[1] + 1
            R, Lt, Mt, tok_c, pred_c, ol_c = R.cpu(), Lt.cpu(), Mt.cpu(), tok.cpu(), pred.cpu(), ol.cpu()
            for b in range(B):  # the reference's host function raises for ragged batches: one sentence per call
                ref.viterbi_decoding(pred_c[b:b + 1], ol_c[b:b + 1], Lt[b:b + 1], R[b:b + 1], Mt[b:b + 1],
                                     tok_c[b:b + 1], mask_cpu, 1)
            return
        if kind == "glance":
            logits.argmax(-1)
        match = ref.logsoftmax_gather(logits, sel, kind == "loss")
        eos = torch.zeros_like(match, dtype=torch.bool)
        eos[rows, :, tl - 1] = True
        eos[rows, ol - 1, tl - 1] = False
        match = match.masked_fill(eos, float("-inf"))
        S, C = ref.pcfg_loss(match, lk, ol, tl, 1)
        if kind == "glance":
            ref.pcfg_best_tree(S, C, match, lk, ol, tl, 1)
        else:
            ref.pcfg_loss_backward(ones, S, C, match, lk, ol, tl, 1)

    n = max(3, min(steps, 10))
    for _ in range(2):
        chain()
    torch.cuda.synchronize()
    ev = []
    for _ in range(n):
        ctx.flush.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        chain()
        e.record()
        ev.append((s, e))
    torch.cuda.synchronize()
    ms = statistics.median(s.elapsed_time(e) for s, e in ev)
    return {"value": B / (ms / 1e3), "unit": UNIT, "ms_per_step": ms, "steps": n,
            "what": "unmodified reference kernels built for sm_100a, eager launches on the default stream, inputs "
                    "resident on the device, logits materialised by a library fp16 GEMM"
                    + ("; the decode leg includes the reference's device-to-host copies and host back-trace, one "
                       "sentence per call" if kind == "viterbi" else "")}


def drop_in(ctx, name, batch, steps):
    """The same chain through this package's reference-named operators on materialised logits: what an
    unmodified criterion / model gets after switching the import.  Also times ``logsoftmax_gather_kernel``
    alone against the HBM roof (one read of the logits, plus one write when the softmax is kept)."""
    import torch.nn.functional as F

    dev, ops = ctx.dev, ctx.ops
    kind = batch.workload.kind
    weight = ctx.weight(batch)
    hid, lk, ol = batch.hidden.to(dev), batch.links.to(dev), batch.output_length.to(dev)
    B, L = batch.B, batch.L
    rows = torch.arange(B, device=dev)
    V = int(weight.shape[0])
    if kind != "viterbi":
        tg, tl = batch.targets.to(dev), batch.target_length.to(dev)
        sel = tg.unsqueeze(1).expand(-1, L, -1)
    else:
        mask_dev = batch.left_tree_mask.long().to(dev)
        pen = torch.arange(L // 4, device=dev).unsqueeze(0).float()
    k = ctx.kernel

    hid_g = hid.clone().requires_grad_(True) if kind == "loss" else hid
    lk_g = lk.clone().requires_grad_(True) if kind == "loss" else lk

    def chain():
        with torch.set_grad_enabled(kind == "loss"):
            logits = F.linear(hid_g, weight)
            if kind == "viterbi":
                ob, tok = logits.float().log_softmax(-1).max(-1)
                scores, R, Lt, Mt = ops.cuda_pcfg_viterbi(ob, lk, ol)
                sc = scores / pen
                sc = torch.where(sc.isnan(), torch.full_like(sc, float("-inf")), sc)
                pred = sc[:, 1:].max(-1)[1] + 1
                return ops.viterbi_decoding(pred, ol, Lt, R, Mt, tok, mask_dev, 1)
            if kind == "glance":
                logits.argmax(-1)
            # with a gradient wanted the operator leaves the softmax in the logits buffer, as the reference's does
            _, match = ops.dag_logsoftmax_gather_inplace(logits, sel)
            eos = torch.zeros_like(match, dtype=torch.bool)
            eos[rows, :, tl - 1] = True
            eos[rows, ol - 1, tl - 1] = False
            match = match.masked_fill(eos, float("-inf"))
            if kind == "glance":
                return ops.cuda_pcfg_best_tree(match, lk, ol, tl)
            return ops.cuda_pcfg_loss(match, lk_g, ol, tl)  # runs forward and backward, as the reference's does

    n = max(3, min(steps, 10))
    for _ in range(2):
        chain()
    torch.cuda.synchronize()
    ev = []
    for _ in range(n):
        ctx.flush.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        chain()
        e.record()
        ev.append((s, e))
    torch.cuda.synchronize()
    ms = statistics.median(s.elapsed_time(e) for s, e in ev)
    rec = {"value": B / (ms / 1e3), "unit": UNIT, "ms_per_step": ms, "steps": n,
           "what": "library fp16 GEMM -> this package's dag_logsoftmax_gather_inplace / cuda_pcfg_loss / "
                   "cuda_pcfg_best_tree / cuda_pcfg_viterbi / viterbi_decoding, eager launches"}
    if kind != "viterbi":  # the log-softmax + gather kernel alone: bytes = rows x V x 2 B x (1 read [+ 1 write])
        logits = F.linear(hid, weight)
        keep = kind == "loss"
        ev = []
        for i in range(n + 2):
            ctx.flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            k.logsoftmax_gather(logits, sel, keep)
            e.record()
            ev.append((s, e))
            if keep:  # the kernel left probabilities behind: fresh logits for the next launch
                logits = F.linear(hid, weight)
        torch.cuda.synchronize()
        kms = statistics.median(s.elapsed_time(e) for s, e in ev[2:])
        nbytes = float(B * L) * V * 2 * (2 if keep else 1)
        gbs = nbytes / (kms / 1e3) / 1e9
        rec["logsoftmax_gather"] = {"bound": "hbm", "ms_per_launch": kms, "algorithmic_bytes": nbytes, "achieved": gbs,
                                    "peak": ctx.pk["gbs"], "unit": "GB/s", "frac": gbs / ctx.pk["gbs"],
                                    "peak_source": ctx.pk["source"] + " (copy bandwidth)",
                                    "what": f"[{B * L}, {V}] fp16 logits, one read"
                                            + (" + one write (softmax kept for the backward)" if keep else "")}
    return rec


def run_ours(a):
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path "
                           "(use --impl reference for the CPU baseline)")
    ctx = Ctx(a)
    rank, world, dev, dist = ctx.rank, ctx.world, ctx.dev, ctx.dist
    syn, runtime, ops = ctx.syn, ctx.runtime, ctx.ops

    batch = syn.make_batch(a.workload, seed=a.seed + rank)  # every rank its own batch: weak scaling
    if batch.hidden is None:
        raise RuntimeError(f"workload {a.workload} has no decoder states; the benchmark runs the projection path")
    kind = batch.workload.kind
    is_loss = kind == "loss"
    if a.drop_in_only:
        if world > 1:
            raise RuntimeError("--drop-in-only is a single-GPU measurement")
        print(json.dumps({"drop_in": {a.workload: drop_in(ctx, a.workload, batch, a.steps)},
                          "device_status": ops.read_status(dev)}), flush=True)
        return
    # N > 1: the loss statistics are summed over the ranks inside the statistics kernel (peer stores over
    # NVLink); --nccl-reduce uses a 12-byte NCCL all-reduce after the step instead
    exchange = None
    if world > 1 and is_loss and not a.nccl_reduce:
        try:
            exchange = ctx.sharding.LossExchange(dev)
        except Exception as err:  # no peer-mapped memory on this box: every rank then falls back together
            print(f"[bench] rank {rank}: in-kernel exchange unavailable ({err}); using the NCCL all-reduce", file=sys.stderr)
        agreed = torch.tensor([1 if exchange is not None else 0], device=dev)
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed) == 0:
            exchange = None
    warm = max(a.warmup, 3)
    sampler = ClockSampler(ctx.local)
    if rank == 0:
        sampler.start()
    rec, step, host, last = measure(ctx, a.workload, batch, batch.B * world, a.steps, warm, a.blocks or None,
                                    exchange, sampler)
    clocks = sampler.stop() if rank == 0 else None
    line = {"metric": rec.pop("metric"), "value": rec.pop("value"), "unit": rec.pop("unit"), "n_gpus": world,
            "steps": a.steps, "warmup": warm, "ms_per_step": rec.pop("ms_per_step"), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic"}
    line.update(rec)
    line["run"]["parallelism"] = f"sentence-sharded x{world}"
    line["run"]["loss_reduce"] = ("none (one GPU)" if world == 1 or not is_loss else
                                  ("in the statistics kernel, peer stores over NVLink" if exchange is not None
                                   else "NCCL all-reduce"))
    line["clocks"] = clocks
    if world > 1 and is_loss and exchange is not None:
        line["exchange_check"] = exchange_check(ctx, step, last)
    # the same step carried back through the projection as well (a wider step than the metric's: reported aside)
    if is_loss and world == 1 and not a.no_proj_backward:
        full = runtime.LossStep(ctx.weight(batch), batch.B, batch.L, batch.T, dev, use_graph=not a.no_graph,
                                proj_backward=True)
        full.load(*host)  # lengths from host memory: the row count of the two products needs no device read
        torch.cuda.synchronize()

        def timed(fn, n):
            ev = []
            for i in range(3 + n):
                ctx.flush.fill_(1)
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                fn()
                e.record()
                ev.append((s, e))
            torch.cuda.synchronize()
            return sum(s.elapsed_time(e) for s, e in ev[3:]) / n

        full_ms = timed(full.run, a.steps)
        line["with_projection_backward"] = {
            "ms_per_step": full_ms, "value": batch.B / (full_ms / 1e3), "unit": UNIT,
            "gpu_launches_per_step": full.kernels_per_step, "what": full.proj_backward_note}
        # the two tensor-core products of the backward alone, on the d-logits the last run left behind
        n_rows = full.n_rows
        V, H = int(full.weight.shape[0]), full.H
        if n_rows and V % 8 == 0 and H % 8 == 0:
            dl = full.dlogits[:n_rows]
            rows = full.hidden.view(-1, H).index_select(0, full.row_index[:n_rows]).to(torch.bfloat16)
            flops = 2.0 * n_rows * V * H
            prods = {}
            for key, fn in (("d_rows", lambda: ctx.kernel.proj_backward_gemms(dl, full.weight_bf16, None, want_weight=False)),
                            ("d_weight", lambda: ctx.kernel.proj_backward_gemms(dl, None, rows, want_rows=False))):
                ms = timed(fn, min(a.steps, 10))
                prods[key] = {"ms_per_launch": ms, "achieved": flops / (ms / 1e3) / 1e12, "peak": ctx.pk["tflops"],
                              "unit": "TFLOP/s", "frac": flops / (ms / 1e3) / 1e12 / ctx.pk["tflops"]}
            line["with_projection_backward"]["products"] = {
                "bound": "tensor", "kernel": "gemm_bf16_kernel", "flops_per_launch": flops,
                "peak_source": ctx.pk["source"] + " (burst bf16 GEMM)", **prods}
        del full
    # the same step fed with the projected link features instead of the transition matrix: the transitions are formed
    # inside the step (the model's extract_links) and the loss gradient is carried back to the features
    if is_loss and world == 1 and not a.no_proj_backward:
        support = importlib.import_module("pcfg_nat_b200.support_tree")
        heads, dim = 8, 64  # decoder_attention_heads and embed_dim / heads of the published configuration (512 / 8)
        lm, rm, mc = support.get_mask(batch.L, 1)
        g = torch.Generator().manual_seed(a.seed)
        feats = [torch.randn(batch.B, batch.L, heads, dim, generator=g).half().to(dev) for _ in range(3)]
        gates = torch.randn(batch.B, batch.L, heads, generator=g).to(dev)
        prev = torch.where(torch.arange(batch.L)[None, :] < batch.output_length[:, None], 3, 1).to(dev)
        lf = runtime.LossStep(ctx.weight(batch), batch.B, batch.L, batch.T, dev, use_graph=not a.no_graph,
                              link_features=(heads, dim), left_tree_mask=lm, right_tree_mask=rm, main_chain=mc)
        lf.load(host[0].to(dev), *feats, gates, prev, *[t.to(dev) for t in host[2:5]])
        times = []
        for i in range(3 + a.steps):
            ctx.flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            lf.run()
            e.record()
            times.append((s, e))
        torch.cuda.synchronize()
        lf_ms = sum(s.elapsed_time(e) for s, e in times[3:]) / a.steps
        line["with_link_features"] = {
            "ms_per_step": lf_ms, "value": batch.B / (lf_ms / 1e3), "unit": UNIT, "gpu_launches_per_step": lf.kernels_per_step,
            "h2d_bytes_per_step_if_loaded": lf.input_bytes(),
            "what": f"the step with the transitions formed from {heads} x {dim} link features per node inside it "
                    "(feature gather, per-head score products, masking + joint log-softmax + head mixture) and the "
                    "loss gradient carried back to the features (two more kernels); random features"}
        del lf
    del step
    torch.cuda.empty_cache()

    subs = not a.no_subs and a.workload == "train_batch"
    if subs:
        sub_steps = min(a.steps, 20)
        line["workloads"] = {}
        for name in SUB_WORKLOADS:
            b = syn.make_batch(name, seed=a.seed + rank)
            # 40 warm-up steps: the GPU sat idle while the previous workload's CPU baseline ran, and its clocks
            # take some tens of milliseconds to come back
            r, st, _, _ = measure(ctx, name, b, b.B * world, sub_steps, 40, blocks=7)
            r["steps"] = sub_steps
            r["scaling"] = "weak"
            if name == "viterbi_b1":
                r["scaling_note"] = "replicas only: one sentence does not shard"
            if name == "long_seq":  # here the DP kernels, not the projection, are the larger part of the step
                r["roofline_dominant"] = "dp" if r["dp"]["share_of_step"] > 0.5 else "roofline"
            if rank == 0 and world == 1 and not a.no_cpu_baseline:
                a_sub = argparse.Namespace(**{**vars(a), "workload": name, "cpu_sample": CPU_SAMPLE[name]})
                r["cpu_baseline"] = cpu_baseline(a_sub, b if rank == 0 else None, budget_s=3.0)
            line["workloads"][name] = r
            del st
            torch.cuda.empty_cache()
        if world > 1:
            line["strong"] = strong_records(ctx, sub_steps, 3)
        else:
            line["gpu_reference"], line["drop_in"] = {}, {}
            for name in ("train_batch", "glance", "viterbi_b64"):
                b = batch if name == a.workload else syn.make_batch(name, seed=a.seed)
                try:
                    line["gpu_reference"][name] = gpu_reference(ctx, name, b, a.steps)
                except Exception as err:  # the checker's build is optional equipment of the box
                    line["gpu_reference"][name] = {"unavailable": repr(err)[:200]}
                line["drop_in"][name] = drop_in(ctx, name, b, a.steps)
                torch.cuda.empty_cache()
    line["device_status"] = ops.read_status(dev)
    if rank == 0:
        if world == 1 and not a.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(a, batch)
            line["cpu_baseline_native_build"] = cpu_baseline(a, batch, budget_s=5.0, fast=True)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def cpu_pass(sub, kind, syn, oracle):
    """One pass of the step over the sentences of ``sub`` on the host cores; returns (seconds, what ran)."""
    import numpy as np

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
        what = "torch CPU fp32 GEMM + log-softmax + max, C port of the Viterbi kernels + back-trace"
    else:
        match = lp.gather(2, sub.targets[:, None, :].expand(-1, sub.L, -1)).contiguous()
        syn.eos_mask_(match, sub.output_length, sub.target_length)
        m_np, tl = match.numpy(), sub.target_length.numpy()
        S, C = oracle.pcfg_loss(m_np, l_np, ol, tl)
        if kind == "glance":
            oracle.pcfg_best_tree(S, C, m_np, l_np, ol, tl)
            what = "torch CPU fp32 GEMM + log-softmax + gather, C port of the inside pass + best tree"
        else:
            oracle.pcfg_loss_backward(np.ones(n, np.float32), S, C, m_np, l_np, ol, tl)
            what = "torch CPU fp32 GEMM + log-softmax + gather, C port of the loss forward + backward"
    return time.perf_counter() - t0, what


def cpu_sample(a, batch, fast=False):
    import oracle

    pkg = entry.load_package()
    syn = pkg.synthetic
    if batch is None:
        batch = syn.make_batch(a.workload, seed=a.seed)
    n = batch.B if a.cpu_sample <= 0 else min(a.cpu_sample, batch.B)
    sub = batch.select(list(range(n)))
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    oracle.use_build("native" if fast else "faithful")
    return syn, batch, sub, n, cores, oracle


def cpu_baseline(a, batch=None, budget_s=10.0, fast=False):
    """The same step on the host cores: the C port of the reference kernels (the reference has no CPU
    implementation of this path) with OpenMP over sentences, and torch's CPU GEMM for the projection.  One
    warm-up pass, then passes over the sample until ``budget_s`` seconds are spent.  ``fast``: the port built
    ``-O3 -march=native`` instead of the bit-faithful ``-O2 -ffp-contract=off`` build the parity tests use."""
    syn, batch, sub, n, cores, oracle = cpu_sample(a, batch, fast)
    try:
        kind = batch.workload.kind
        cpu_pass(sub, kind, syn, oracle)
        times, what = [], ""
        while len(times) < 2 or (sum(times) < budget_s and len(times) < 200):
            dt, what = cpu_pass(sub, kind, syn, oracle)
            times.append(dt)
        flags = oracle.build_flags()
    finally:
        oracle.use_build("faithful")
    med = sorted(times)[len(times) // 2]
    return {"value": n / med, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{n} of {batch.B} sentences of {a.workload} per pass ({what}; port built with gcc {flags}); "
                      f"median of {len(times)} passes after 1 warm-up pass, {med:.3f} s per pass, {sum(times):.1f} s in all"}


def run_reference(a):
    """The reference arm: the path's CPU implementation (the C port: the reference itself has none) on
    all host cores, W warm-up passes and K timed passes over the workload's batch (a pass = a step; the number
    of timed passes is cut so that the run stays within about two minutes)."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    syn, batch, sub, n, cores, oracle = cpu_sample(a, None)
    kind = batch.workload.kind
    for _ in range(max(1, min(a.warmup, 3))):
        cpu_pass(sub, kind, syn, oracle)
    times, what = [], ""
    while len(times) < max(a.steps, 1) and (len(times) < 2 or sum(times) < 120.0):
        dt, what = cpu_pass(sub, kind, syn, oracle)
        times.append(dt)
    mean = sum(times) / len(times)
    value = n / mean
    cb = {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
          "sample": f"{n} of {batch.B} sentences of {a.workload} per step ({what}; port built with gcc "
                    f"{oracle.build_flags()}: the bit-faithful build the parity tests use, not tuned for speed); "
                    f"{len(times)} timed steps of {a.steps} asked, {mean:.3f} s per step"}
    line = {"impl": "reference", "metric": METRICS[kind], "value": value, "unit": UNIT, "n_gpus": a.gpus,
            "steps": len(times), "warmup": a.warmup, "ms_per_step": mean * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": config_of(a.workload, batch),
            "run": {"parallelism": "host cores of rank 0 only", "arithmetic": "f32 on the CPU"},
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
