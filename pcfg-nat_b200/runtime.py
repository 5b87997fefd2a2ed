"""Fixed-shape steps of the structured-loss / decoding path, replayable as CUDA graphs.

Each step is what the reference's Python does around the custom operators for one batch:

* ``LossStep``   — training (fs_plugins/criterions/nat_pcfg_loss.py:98-135): emissions of the targets from
  the decoder states (fused projection, EOS masking included), PCFG loss with both gradients, and the
  three statistics the scalar loss is formed from;
* ``GlanceStep`` — glancing pass (nat_pcfg_loss.py:193-227): emissions + arg-max tokens, inside table,
  best-tree alignment;
* ``DecodeStep`` — Viterbi inference (fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:483-502):
  max log-prob / arg-max token per node, Viterbi tables, length-penalised choice of the output length,
  back-trace on the device.

A step launches a handful of small-to-medium kernels whose device time (~1 ms at training-batch size) is
of the order of the host cost of enqueueing them through Python, so it is captured once into a CUDA graph
and replayed.  Inputs live in static device buffers; ``load`` copies a new batch into them (from pinned
host memory or from device tensors) on the current stream.
"""
import torch

from . import sharding
from .custom_ops import pcfg_loss as ops


class _GraphedStep:
    def __init__(self, weight, B, L, device, use_graph=True):
        if weight.dtype != torch.float16 or not weight.is_cuda:
            raise RuntimeError("weight must be a float16 CUDA tensor [V, H]")
        self.device = torch.device(device)
        self.weight = weight.contiguous()
        self.V, self.H = weight.shape
        self.B, self.L = B, L
        dev = self.device
        self.hidden = torch.zeros((B, L, self.H), dtype=torch.float16, device=dev)
        self.links = torch.full((B, L, 2, L), float("-inf"), dtype=torch.float32, device=dev)
        self.output_length = torch.full((B,), 2, dtype=torch.int64, device=dev)
        self.use_graph = use_graph
        self.graph = None
        self.out = None
        self.kernel = ops.get_pcfg_kernel()

    def _inputs(self):
        return [self.hidden, self.links, self.output_length]

    def input_bytes(self):
        return sum(t.numel() * t.element_size() for t in self._inputs())

    def load(self, *tensors):
        """Copies one batch into the static buffers (async on the current stream); same order as ``_inputs``."""
        bufs = self._inputs()
        if len(tensors) != len(bufs):
            raise RuntimeError(f"expected {len(bufs)} tensors")
        for dst, src in zip(bufs, tensors):
            dst.copy_(src, non_blocking=True)

    def _body(self):
        raise NotImplementedError

    def run(self):
        if not self.use_graph:
            self.out = self._body()
            return self.out
        if self.graph is None:
            # warm up on a side stream (lazy module loading, allocator), then capture
            s = torch.cuda.Stream(self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(s):
                for _ in range(2):
                    self._body()
            torch.cuda.current_stream(self.device).wait_stream(s)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.out = self._body()
            self.graph = g
        self.graph.replay()
        return self.out


class LossStep(_GraphedStep):
    """projection -> loss forward+backward -> loss statistics for fixed (B, L, T, H, V).

    Inputs (``load`` order): hidden [B,L,H] f16, links [B,L,2,L] f32, output_length [B], targets [B,T],
    target_length [B].  ``run()`` returns (stats[3] f32 = [sum_b S_b/n_b, sentences, invalid],
    match_all_grad, links_grad, sentence_loss); static outputs, overwritten by the next ``run()``.
    """
    kernels_per_step = 6  # proj_prepare, proj, proj_merge, loss_fwd, outside, grad

    def __init__(self, weight, B, L, T, device, use_graph=True):
        super().__init__(weight, B, L, device, use_graph)
        self.T = T
        self.targets = torch.zeros((B, T), dtype=torch.int64, device=self.device)
        self.target_length = torch.ones((B,), dtype=torch.int64, device=self.device)

    def _inputs(self):
        return [self.hidden, self.links, self.output_length, self.targets, self.target_length]

    def _body(self):
        k = self.kernel
        em = k.proj_logsoftmax_gather(self.hidden, self.weight, self.targets, self.output_length, self.target_length)
        loss, mg, lg = k.pcfg_loss_fwd_bwd(em["match"], self.links, self.output_length, self.target_length)
        stats = sharding.local_loss_stats(loss, self.target_length)
        return stats, mg, lg, loss


class GlanceStep(LossStep):
    """projection (emissions + arg-max tokens) -> inside table -> best tree.

    ``run()`` returns (tree [B,L] i64, sentence log-likelihood [B], arg-max tokens [B,L] i64)."""
    kernels_per_step = 5  # proj_prepare, proj, proj_merge, loss_fwd, best_tree

    def _body(self):
        k = self.kernel
        em = k.proj_logsoftmax_gather(self.hidden, self.weight, self.targets, self.output_length, self.target_length,
                                      want_max=True)
        S, _ = k.pcfg_loss(em["match"], self.links, self.output_length, self.target_length, 1, want_c=False)
        tree = k.pcfg_best_tree(S, None, em["match"], self.links, self.output_length, self.target_length, 1)
        return tree, S[:, 0, 0], em["argmax"]


class DecodeStep(_GraphedStep):
    """projection (max log-prob + arg-max token per node) -> Viterbi tables -> output length -> back-trace.

    Inputs (``load`` order): hidden, links, output_length.  ``run()`` returns (tokens [B,L] i64 padded with
    ``pad_index``, count [B] i64, predicted length [B] i64)."""
    kernels_per_step = 5  # proj_prepare, proj, proj_merge, viterbi, backtrace

    def __init__(self, weight, B, L, left_tree_mask, device, beta=1.0, pad_index=1, use_graph=True):
        super().__init__(weight, B, L, device, use_graph)
        self.mask = left_tree_mask.to(device=self.device, dtype=torch.int64).contiguous()
        self.pad_index = int(pad_index)
        # length penalty of the model: scores / arange(L // 4) ** beta (models/...pcfg.py:488-492)
        self.penalty = (torch.arange(L // 4, device=self.device) ** beta).to(torch.float32).unsqueeze(0)

    def _body(self):
        k = self.kernel
        em = k.proj_logsoftmax_gather(self.hidden, self.weight, None, self.output_length, None, want_max=True)
        S, R, Lt, Mt = k.pcfg_viterbi(em["max_lprob"], self.links, self.output_length, 1)
        scores = S[:, 1, :] / self.penalty
        scores = torch.where(torch.isnan(scores), torch.full_like(scores, float("-inf")), scores)
        pred = scores[:, 1:].max(-1)[1] + 1
        tokens, count = k.viterbi_decoding_device(pred, self.output_length, Lt, R, Mt, em["argmax"], self.mask,
                                                  self.pad_index)
        return tokens, count, pred
