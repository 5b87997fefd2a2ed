"""Fixed-shape training step of the structured-loss path, replayable as a CUDA graph.

The step is what the criterion does around the custom operators for one batch
(fs_plugins/criterions/nat_pcfg_loss.py:98-135): emissions of the targets from the decoder
states (here the fused projection, EOS masking included), the PCFG loss with both gradients,
and the three loss statistics the scalar loss is formed from.  It launches seven small-to-medium
kernels; at training-batch sizes their device time (~1 ms) is of the order of the host cost
of enqueueing them through Python, so the step is captured once into a CUDA graph and replayed.
Inputs live in static device buffers; ``load`` copies a new batch into them (from pinned host
memory or from device tensors) on the same stream.
"""
import torch

from . import sharding
from .custom_ops import pcfg_loss as ops


class LossStep:
    """projection -> loss forward+backward -> loss statistics for fixed (B, L, T, H, V).

    ``run()`` returns (stats[3] f32 = [sum_b S_b/n_b, sentences, invalid], match_all_grad, links_grad,
    sentence_loss); the tensors are static outputs that the next ``run()`` overwrites.
    """

    def __init__(self, weight, B, L, T, device, use_graph=True):
        if weight.dtype != torch.float16 or not weight.is_cuda:
            raise RuntimeError("weight must be a float16 CUDA tensor [V, H]")
        self.device = torch.device(device)
        self.weight = weight.contiguous()
        V, H = weight.shape
        self.B, self.L, self.T, self.H, self.V = B, L, T, H, V
        dev = self.device
        self.hidden = torch.zeros((B, L, H), dtype=torch.float16, device=dev)
        self.links = torch.full((B, L, 2, L), float("-inf"), dtype=torch.float32, device=dev)
        self.targets = torch.zeros((B, T), dtype=torch.int64, device=dev)
        self.output_length = torch.full((B,), 2, dtype=torch.int64, device=dev)
        self.target_length = torch.ones((B,), dtype=torch.int64, device=dev)
        self.use_graph = use_graph
        self.graph = None
        self.out = None
        self.kernel = ops.get_pcfg_kernel()

    def input_bytes(self):
        ts = (self.hidden, self.links, self.targets, self.output_length, self.target_length)
        return sum(t.numel() * t.element_size() for t in ts)

    def load(self, hidden, links, targets, output_length, target_length):
        """Copies one batch into the static buffers (async on the current stream)."""
        self.hidden.copy_(hidden, non_blocking=True)
        self.links.copy_(links, non_blocking=True)
        self.targets.copy_(targets, non_blocking=True)
        self.output_length.copy_(output_length, non_blocking=True)
        self.target_length.copy_(target_length, non_blocking=True)

    def _body(self):
        k = self.kernel
        em = k.proj_logsoftmax_gather(self.hidden, self.weight, self.targets, self.output_length, self.target_length)
        loss, mg, lg = k.pcfg_loss_fwd_bwd(em["match"], self.links, self.output_length, self.target_length)
        stats = sharding.local_loss_stats(loss, self.target_length)
        return stats, mg, lg, loss

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
