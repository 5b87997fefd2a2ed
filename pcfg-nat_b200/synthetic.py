"""Seeded synthetic batches with the shapes of the PCFG-NAT training / decoding workloads.

The reference trains and decodes on WMT batches that are not available offline; these
generators produce inputs with the same shapes, masks and value distributions:

* transition scores ``links[B, L, max_left+1, L]``: N(0,1) logits masked exactly as
  ``extract_links`` masks them (models/glat_decomposed_with_link_two_hands_tri_pcfg.py:168-199:
  left child inside the node's left subtree and not padding, right child inside the right
  subtree, on the main chain and not padding), jointly log-softmax normalised over
  (left, right), rows without any allowed pair set to -inf;
* emissions either as fp32 logits ``[B, L, V]`` or as fp16 decoder states ``[B, L, H]``
  plus a projection matrix ``[V, H]``;
* target ids uniform in [4, V) with the last real position set to EOS and the tail to PAD,
  and the criterion's EOS masking of the gathered emissions
  (criterions/nat_pcfg_loss.py:112-115).

Everything is generated on the CPU from one ``torch.Generator`` so that every rank of a
sharded run can rebuild the same global batch and slice its own sentences.
"""
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch

from .support_tree import get_mask, max_left_of

PAD, EOS = 1, 2  # fairseq dictionary convention; ids < 4 are reserved


@dataclass
class Workload:
    """Shape description of one named workload."""
    name: str
    batch: int
    vocab: int
    hidden: int
    left_tree_layer: int = 1
    src_min: int = 8
    src_max: int = 8
    upsample: int = 4  # graph length = upsample * source length + graph_offset
    graph_offset: int = 0
    fixed_graph: Optional[int] = None  # all sentences use this graph length
    fixed_target: Optional[int] = None
    target_jitter: float = 0.2  # target length = source length * U[1-j, 1+j]
    hidden_std: float = 1.0
    weight_std: float = 0.02
    emissions: str = "hidden"  # "hidden" (fp16 states + projection) or "logits" (fp32 logits)
    kind: str = "loss"  # "loss", "viterbi" or "glance"


WORKLOADS: Dict[str, Workload] = {
    # tiny fp32 case every component can run, CPU oracle included
    "tiny_loss": Workload("tiny_loss", batch=2, vocab=1000, hidden=64, fixed_graph=32, fixed_target=10,
                          emissions="logits"),
    # one training batch: ~90 sentences, ~2730 target tokens (--max-tokens 2730)
    "train_batch": Workload("train_batch", batch=90, vocab=40000, hidden=512, src_min=20, src_max=40,
                            hidden_std=0.02),
    # the same sentences with the graph size the reference model really builds, 8 * source + 2 nodes
    # (models/glat_decomposed_with_link_two_hands_tri_pcfg.py:322: source * upsample scale * 2^left_tree_layer + 2)
    "train_batch_model_graph": Workload("train_batch_model_graph", batch=90, vocab=40000, hidden=512, src_min=20,
                                        src_max=40, upsample=8, graph_offset=2, hidden_std=0.02),
    # long sequences: 8 sentences, graph 512, target 128
    "long_seq": Workload("long_seq", batch=8, vocab=40000, hidden=512, fixed_graph=512, fixed_target=128),
    "viterbi_b1": Workload("viterbi_b1", batch=1, vocab=40000, hidden=512, src_min=10, src_max=60, kind="viterbi"),
    "viterbi_b64": Workload("viterbi_b64", batch=64, vocab=40000, hidden=512, src_min=10, src_max=60,
                            kind="viterbi"),
    "glance": Workload("glance", batch=64, vocab=40000, hidden=512, fixed_graph=256, fixed_target=64, kind="glance"),
    # the glancing pass over the training batch itself (what a GLAT training step runs before the loss pass)
    "glance_train": Workload("glance_train", batch=90, vocab=40000, hidden=512, src_min=20, src_max=40,
                             hidden_std=0.02, kind="glance"),
}


@dataclass
class Batch:
    workload: Workload
    output_length: torch.Tensor  # [B] int64, graph nodes per sentence (m_b)
    target_length: torch.Tensor  # [B] int64 (n_b)
    links: torch.Tensor  # [B, L, max_left+1, L] f32
    targets: torch.Tensor  # [B, T] int64
    left_tree_mask: torch.Tensor  # [L, L] bool, True = not allowed
    hidden: Optional[torch.Tensor] = None  # [B, L, H] f16
    weight: Optional[torch.Tensor] = None  # [V, H] f16
    logits: Optional[torch.Tensor] = None  # [B, L, V] f32
    extras: dict = field(default_factory=dict)

    @property
    def B(self):
        return self.links.shape[0]

    @property
    def L(self):
        return self.links.shape[1]

    @property
    def T(self):
        return self.targets.shape[1]

    def select(self, index):
        """Sub-batch of the given sentence indices (used for sentence sharding)."""
        index = torch.as_tensor(index, dtype=torch.long)
        pick = lambda t: None if t is None else t.index_select(0, index)
        return Batch(self.workload, pick(self.output_length), pick(self.target_length), pick(self.links),
                     pick(self.targets), self.left_tree_mask, pick(self.hidden), self.weight, pick(self.logits),
                     dict(self.extras))


def make_links(output_length, L, left_tree_layer, generator):
    """Masked, jointly normalised transition log-probabilities [B, L, max_left+1, L]."""
    B = output_length.numel()
    ml = max_left_of(left_tree_layer)
    left_mask, right_mask, main_chain = get_mask(L, left_tree_layer)
    left_mask, right_mask, main_chain = left_mask.bool(), right_mask.bool(), main_chain.bool()
    pos = torch.arange(L)
    pad = pos[None, :] >= output_length[:, None]  # [B, L]
    link_left_mask = pad[:, None, :] | left_mask[None]  # [B, a, j]
    link_right_mask = pad[:, None, :] | right_mask[None]  # [B, a, c]
    link_right_mask = ~(~link_right_mask & main_chain[None, None, :])
    left_nouse = (~link_left_mask).sum(2, keepdim=True) == 0
    right_nouse = (~link_right_mask).sum(2, keepdim=True) == 0
    nouse = left_nouse | right_nouse  # [B, a, 1]
    # left option k refers to node a-k (k >= 1) or node 0 (k == 0); lemon_tree.py:150-156
    idx = pos[:, None] - torch.arange(ml + 1)[None, :]
    idx[:, 0] = 0
    idx = idx.clamp(min=0)  # [a, k]
    left_dis = torch.gather(link_left_mask, 2, idx[None].expand(B, -1, -1))  # [B, a, k]
    logits = torch.randn(B, L, ml + 1, L, generator=generator)
    dis = left_dis[:, :, :, None] | link_right_mask[:, :, None, :]
    logits = logits.masked_fill(dis, float("-inf"))
    flat = logits.view(B, L, (ml + 1) * L)
    all_dis = torch.isinf(flat).all(-1, keepdim=True)
    flat = torch.where(all_dis, torch.zeros_like(flat), flat)
    links = torch.log_softmax(flat, dim=-1).view(B, L, ml + 1, L)
    links = links.masked_fill((nouse | all_dis).view(B, L, 1, 1), float("-inf"))
    return links.contiguous(), left_mask


def make_batch(name_or_workload, seed=0, batch=None) -> Batch:
    """Builds the named workload from ``seed`` (CPU tensors)."""
    w = WORKLOADS[name_or_workload] if isinstance(name_or_workload, str) else name_or_workload
    g = torch.Generator().manual_seed(seed)
    B = batch or w.batch
    scale = w.upsample
    if w.fixed_graph is not None:
        out_len = torch.full((B,), w.fixed_graph, dtype=torch.long)
        src = out_len // scale
    else:
        src = torch.randint(w.src_min, w.src_max + 1, (B,), generator=g)
        out_len = src * scale + w.graph_offset
    if w.fixed_target is not None:
        tgt_len = torch.full((B,), w.fixed_target, dtype=torch.long)
    else:
        f = 1.0 - w.target_jitter + 2 * w.target_jitter * torch.rand(B, generator=g)
        tgt_len = torch.round(src.float() * f).long()
    # feasible at left_tree_layer 1 iff 2 <= n <= m - 2
    tgt_len = torch.minimum(tgt_len.clamp(min=2), out_len - 2)
    L, T = int(out_len.max()), int(tgt_len.max())
    links, left_mask = make_links(out_len, L, w.left_tree_layer, g)
    targets = torch.randint(4, w.vocab, (B, T), generator=g)
    tpos = torch.arange(T)[None, :]
    targets = torch.where(tpos == (tgt_len[:, None] - 1), torch.full_like(targets, EOS), targets)
    targets = torch.where(tpos >= tgt_len[:, None], torch.full_like(targets, PAD), targets)
    b = Batch(w, out_len, tgt_len, links, targets, left_mask)
    if w.emissions == "logits":
        b.logits = torch.randn(B, L, w.vocab, generator=g)
    else:
        b.hidden = (torch.randn(B, L, w.hidden, generator=g) * w.hidden_std).half()
        b.weight = (torch.randn(w.vocab, w.hidden, generator=g) * w.weight_std).half()
    return b


def eos_mask_(match_all, output_length, target_length):
    """In-place EOS masking of gathered emissions [B, L, T]: column n_b-1 is -inf for every
    node except m_b-1 (criterions/nat_pcfg_loss.py:112-115)."""
    B = match_all.shape[0]
    rows = torch.arange(B, device=match_all.device)
    col = (target_length - 1).to(match_all.device)
    keep = match_all[rows, (output_length - 1).to(match_all.device), col].clone()
    match_all[rows, :, col] = float("-inf")
    match_all[rows, (output_length - 1).to(match_all.device), col] = keep
    return match_all


def reference_match_all(batch: Batch):
    """fp32 CPU emissions log P(y_t | node) [B, L, T] with the EOS mask applied (small cases)."""
    if batch.logits is not None:
        lp = torch.log_softmax(batch.logits.float(), -1)
    else:
        lp = torch.log_softmax(batch.hidden.float() @ batch.weight.float().t(), -1)
    m = lp.gather(2, batch.targets[:, None, :].expand(-1, batch.L, -1)).contiguous()
    return eos_mask_(m, batch.output_length, batch.target_length)
