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
