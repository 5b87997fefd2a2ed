"""Sentence sharding across the GPUs of one box and the scalar loss reduction.

Every operator of this package treats sentences independently (the kernels index the batch
first and never mix sentences), so a batch is split by sentence with no data-path collective.
The only exchange is the reduction of three floats per step, which mirrors how the criterion
forms its scalar: ``loss = -(S_b / n_b).mean()`` with invalid (inf/nan) sentences zeroed and
counted (fs_plugins/criterions/nat_pcfg_loss.py:122-135, summed logging outputs :336-344).
"""
from typing import List, Sequence

import torch
import torch.distributed as dist


def sentence_cost(output_length, target_length=None):
    """Relative DP cost of a sentence: (main-chain nodes)^2 x dependent steps."""
    m = torch.as_tensor(output_length).double() / 2
    steps = torch.as_tensor(target_length).double() if target_length is not None else m / 2
    return m * m * steps


def shard_sentences(costs: Sequence[float], world_size: int) -> List[List[int]]:
    """Deterministic cost-balanced partition: sentences sorted by decreasing cost are dealt out
    in snake order (0..W-1, W-1..0, ...).  Returns the sorted sentence indices of every rank;
    together they cover each sentence exactly once."""
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    c = torch.as_tensor(costs, dtype=torch.float64)
    order = sorted(range(c.numel()), key=lambda i: (-float(c[i]), i))
    shards: List[List[int]] = [[] for _ in range(world_size)]
    for pos, idx in enumerate(order):
        rnd, off = divmod(pos, world_size)
        rank = off if rnd % 2 == 0 else world_size - 1 - off
        shards[rank].append(idx)
    return [sorted(s) for s in shards]


def local_loss_stats(sentence_loss: torch.Tensor, target_length: torch.Tensor) -> torch.Tensor:
    """[sum_b S_b / n_b over valid sentences, sentences, invalid sentences] as a float32 vector
    on the loss's device."""
    if sentence_loss.is_cuda:  # one launch of the library's kernel (it raises if the library is missing)
        from .custom_ops import pcfg_loss as ops

        return ops.get_pcfg_kernel().loss_stats(sentence_loss, target_length)
    # host tensors: the multi-process logic of the CPU tests
    invalid = torch.isinf(sentence_loss) | torch.isnan(sentence_loss)
    s = torch.where(invalid, torch.zeros_like(sentence_loss), sentence_loss)
    tl = target_length.to(device=sentence_loss.device, dtype=sentence_loss.dtype).clamp(min=1)
    count = torch.full((), float(s.numel()), dtype=s.dtype, device=s.device)  # a fill kernel: capturable in a CUDA graph
    return torch.stack([(s / tl).sum(), count, invalid.sum().to(s.dtype)])


def reduce_loss(sentence_loss: torch.Tensor, target_length: torch.Tensor, group=None):
    """Global criterion scalar from per-rank sentence losses: one 3-float all-reduce (NCCL over
    NVLink for CUDA tensors, gloo for CPU tensors).  Returns (loss, n_sentences, n_invalid)."""
    stats = local_loss_stats(sentence_loss, target_length)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.SUM, group=group)
    loss = -stats[0] / stats[1].clamp(min=1)
    return loss, stats[1], stats[2]


def check_exchanged_stats(stats_host: torch.Tensor):
    """Raises when the statistics a ``LossExchange`` returned are the NaN triple its kernel writes after a peer
    did not arrive within the bounded wait (about half a second).  Call it where the step's result is read on
    the host anyway; an NCCL all-reduce in the same place would simply have waited for the late rank."""
    if bool(torch.isnan(torch.as_tensor(stats_host)).any()):
        raise RuntimeError("loss statistics exchange: a peer rank did not arrive within the bounded device-side wait "
                           "(PCFGNAT_STATUS_TIMEOUT); line the ranks up before the step or use sharding.reduce_loss")


class LossExchange:
    """Sums the loss statistics over the ranks of a process group inside the statistics kernel itself: every
    rank's kernel stores its three numbers into every peer's buffer over NVLink and adds up what it received
    (``pcfgnat_loss_stats_exchange``), instead of a separate 12-byte NCCL all-reduce whose launch latency is
    several percent of a training step.  The buffers are torch symmetric memory; every rank must call
    ``stats`` the same number of times.  One GPU: the plain local kernel.

    The device-side wait for a peer is bounded (about half a second).  A rank that gives up returns NaN in all
    three numbers, never a short sum; ``check_exchanged_stats`` turns that into an exception where the host reads
    the result.  Ranks that may drift apart by more than the bound (a checkpoint written by one rank, validation on
    rank 0) should use ``reduce_loss`` (an all-reduce waits) or synchronise before the step."""

    def __init__(self, device, group=None):
        from .custom_ops import pcfg_loss as ops

        self.kernel = ops.get_pcfg_kernel()
        self.device = torch.device(device)
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.peers = None
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm

            nbytes = 64 + 64 * self.world  # PCFGNAT_EXCHANGE_BYTES(world)
            self.buffer = symm.empty((nbytes + 3) // 4, dtype=torch.float32, device=self.device)
            self.buffer.zero_()
            torch.cuda.synchronize(self.device)
            pg = group if group is not None else dist.group.WORLD
            self.handle = symm.rendezvous(self.buffer, pg.group_name)
            self.peers = torch.tensor([int(p) for p in self.handle.buffer_ptrs], dtype=torch.int64, device=self.device)
            dist.barrier(group)  # every buffer is zeroed and mapped before any rank's first call

    def stats(self, sentence_loss, target_length):
        """[sum_b S_b / n_b, sentences, invalid] over all ranks (float32 [3], the same on every rank)."""
        if self.world == 1:
            return self.kernel.loss_stats(sentence_loss, target_length)
        return self.kernel.loss_stats_exchange(sentence_loss, target_length, self.peers, self.rank, self.world)
