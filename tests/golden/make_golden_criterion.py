"""Generates ``host_criterion.npz``: outputs of the reference criterion's own code for the glue around the DP
operators, run on the CPU —

* ``glat_function`` (the function nested in ``NATPCFGoss.forward``, fs_plugins/criterions/nat_pcfg_loss.py:193-269):
  the glancing sampler for the three strategies (None, "number-random", "cmlm");
* ``NATPCFGoss._compute_pfcg_loss`` (nat_pcfg_loss.py:98-145): the EOS mask, the force-emit mask (with its
  ``detach`` pattern, seen through the gradient) and the scalar loss with invalid sentences zeroed and counted.

The criterion cannot be imported without fairseq, so the two function definitions are compiled from the file's
text and called with stand-ins for ``self`` / ``model`` and for the three CUDA operators they call: the
log-softmax + gather is done with torch on the CPU, the best tree is a seeded alignment handed in, and the loss
operator records the emissions it is given and returns seeded sentence losses that depend on them linearly (so
that autograd shows which entries carry a gradient).  The random draws are torch's own, from a seeded global
generator; the same seed regenerates them for the kernels under test.

Usage:  python tests/golden/make_golden_criterion.py --reference /path/to/PCFG-NAT
"""
import argparse
import ast
import os
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
PAD = 1


def load_functions(reference, ns):
    path = os.path.join(reference, "fs_plugins", "criterions", "nat_pcfg_loss.py")
    tree = ast.parse(open(path).read())
    wanted = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name in ("glat_function", "_compute_pfcg_loss"):
            wanted.setdefault(node.name, node)
    for name in ("glat_function", "_compute_pfcg_loss"):
        exec(compile(ast.Module(body=[wanted[name]], type_ignores=[]), path, "exec"), ns)
    return ns


def random_alignment(g, B, L, T, out_len, tgt_len):
    """A monotone alignment like a best tree: n_b distinct graph nodes (first and last among them) emit the
    target positions 0 .. n_b-1 in order; the other nodes hold -1.  Sentence 0 also carries an out-of-range
    position, which the criterion clamps away (nat_pcfg_loss.py:217-218)."""
    path = torch.full((B, L), -1, dtype=torch.long)
    for b in range(B):
        m, n = int(out_len[b]), int(tgt_len[b])
        inner = torch.randperm(m - 2, generator=g)[: n - 2] + 1
        nodes = torch.cat([torch.tensor([0]), inner.sort()[0], torch.tensor([m - 1])])
        path[b, nodes] = torch.arange(n)
    path[0, 2 if path[0, 2] < 0 else 3] = T + 3
    return path


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    a = ap.parse_args()
    out = {}
    state = {}

    def gather_stub(word_ins_out, select_idx):  # dag_logsoftmax_gather_inplace on the CPU
        if "match_leaf" in state:
            return word_ins_out, state["match_leaf"]
        return word_ins_out, torch.log_softmax(word_ins_out.float(), -1).gather(-1, select_idx)

    def best_tree_stub(match, links, output_length, target_length):
        state["glance_match"] = match.clone()
        return state["path"].clone(), state["tree_lprob"].clone()

    def loss_stub(match, links, output_length, target_length):
        state["loss_match"] = match.detach().clone()
        fin = torch.isfinite(match)
        val = (torch.where(fin, match, torch.zeros_like(match)) * state["w"]).sum((1, 2))
        return val + state["loss_offset"]  # -inf offsets make invalid sentences

    ns = {"torch": torch, "dag_logsoftmax_gather_inplace": gather_stub, "cuda_pcfg_best_tree": best_tree_stub,
          "cuda_pcfg_loss": loss_stub}
    me = types.SimpleNamespace()
    ns["self"] = me  # glat_function reads the criterion through its closure
    load_functions(a.reference, ns)
    model = types.SimpleNamespace(pad=PAD)

    g = torch.Generator().manual_seed(0)
    B, L, T, V = 5, 28, 9, 50
    out_len = torch.tensor([28, 24, 20, 28, 16])
    tgt_len = torch.tensor([9, 7, 5, 8, 4])
    tgt = torch.randint(4, V, (B, T), generator=g)
    tgt = torch.where(torch.arange(T)[None, :] < tgt_len[:, None], tgt, torch.full_like(tgt, PAD))
    prev = torch.where(torch.arange(L)[None, :] < out_len[:, None], 3, PAD)
    logits = torch.randn(B, L, V, generator=g)
    links = torch.zeros(B, L, 2, L)
    path = random_alignment(g, B, L, T, out_len, tgt_len)
    # make some predictions agree with the oracle tokens so that same_num is not trivially zero
    pred = logits.argmax(-1)
    oracle_tok = tgt.gather(-1, path.clamp(min=0, max=T - 1))
    agree = (torch.rand(B, L, generator=g) < 0.3) & (path >= 0) & (path < T)
    boost = torch.zeros_like(logits).scatter_(-1, oracle_tok.unsqueeze(-1), 50.0) * agree.unsqueeze(-1)
    logits = logits + boost
    state["path"] = path
    state["tree_lprob"] = torch.tensor([-30.0, -20.0, float("-inf"), -25.0, -10.0])
    out.update(out_len=out_len.numpy(), tgt_len=tgt_len.numpy(), tgt=tgt.numpy(), prev=prev.numpy(), path=path.numpy(),
               logits=logits.numpy())

    for tag, strategy, seed in (("none", None, 11), ("number_random", "number-random", 12), ("cmlm", "cmlm", 13)):
        me.glance_strategy = strategy
        torch.manual_seed(seed)
        glat_prev, glat_tgt, info = ns["glat_function"](model, logits.clone(), tgt, prev, {"context_p": 0.5}, links=links)
        out[f"{tag}_seed"] = np.int64(seed)
        out[f"{tag}_glat_prev"] = glat_prev.numpy()
        out[f"{tag}_matchmask"] = info["matchmask"].numpy()
        out[f"{tag}_keep"] = info["keep_word_mask"].numpy()
        out[f"{tag}_glat_accu"] = np.float32(info["glat_accu"])
        out[f"{tag}_glat_keep"] = np.float32(info["glat_keep"])
        out[f"{tag}_max_tree_lprob"] = np.float32(info["max_tree_lprob"])
    out["glance_match"] = state["glance_match"].numpy()  # EOS-masked emissions the best-tree operator was given

    # ---- _compute_pfcg_loss: EOS mask, force-emit mask, scalar loss --------------------------------------------
    me.cfg = types.SimpleNamespace(no_force_emit=False)
    me.task = types.SimpleNamespace(tgt_dict=types.SimpleNamespace(pad=lambda: PAD))
    matchmask = torch.from_numpy(out["number_random_matchmask"])
    keep = torch.from_numpy(out["number_random_keep"])
    state["w"] = torch.rand(B, L, T, generator=g) + 0.5
    state["loss_offset"] = torch.tensor([0.0, 0.0, float("-inf"), 0.0, 0.0])
    match_plain = torch.log_softmax(logits, -1).gather(-1, tgt.unsqueeze(1).expand(-1, L, -1))
    for tag, mm, kw in (("force", matchmask, keep), ("plain", None, None)):
        leaf = match_plain.clone().requires_grad_(True)
        state["match_leaf"] = leaf
        res = ns["_compute_pfcg_loss"](me, logits.clone(), prev.ne(PAD), tgt, tgt.ne(PAD), links, name="pcfg-loss",
                                       factor=1, matchmask=mm, keep_word_mask=kw, model=model)
        # the criterion's scalar, and the gradient of the valid sentences' sum to see which entries are live
        out[f"{tag}_loss"] = np.float32(res["loss"].detach())
        out[f"{tag}_invalid"] = np.int64(res["invalid_nsentences"])
        out[f"{tag}_loss_match"] = state["loss_match"].numpy()
        res["loss"].backward()
        out[f"{tag}_match_grad"] = leaf.grad.numpy()
    out["loss_w"] = state["w"].numpy()
    out["match_plain"] = match_plain.numpy()
    np.savez_compressed(os.path.join(HERE, "host_criterion.npz"), **out)
    for k, v in out.items():
        print(k, getattr(v, "shape", v))


if __name__ == "__main__":
    main()
