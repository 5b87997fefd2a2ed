"""Generates ``host_*.npz``: outputs of the reference's own CPU-runnable pieces.

* ``BinaryTreeNode.get_mask`` (fs_plugins/models/lemon_tree.py:92-119), imported by file path;
* the host back-trace ``viterbi_decoding`` (fs_plugins/custom_ops/pcfg_loss.cpp:12-73) from
  the reference extension built by ``oracle/build_ref.py``, fed with Viterbi traces.

Runs where the reference checkout is mounted; no GPU needed.
Usage:  python tests/golden/make_golden_host.py --reference /path/to/PCFG-NAT
"""
import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402
import oracle  # noqa: E402
from oracle.build_ref import load_ref  # noqa: E402

pkg = entry.load_package()
syn = pkg.synthetic


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    a = ap.parse_args()
    spec = importlib.util.spec_from_file_location(
        "ref_lemon_tree", os.path.join(a.reference, "fs_plugins", "models", "lemon_tree.py"))
    lemon = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(lemon)
    masks = {}
    for ltl in (1, 2, 3):
        for dim in (2, 5, 8, 14, 17, 34, 66):
            l, r, mc = lemon.BinaryTreeNode.get_mask(dim, ltl, 4.0)
            masks[f"left_{ltl}_{dim}"] = l.numpy().astype(np.uint8)
            masks[f"right_{ltl}_{dim}"] = r.numpy().astype(np.uint8)
            masks[f"main_{ltl}_{dim}"] = mc.numpy().astype(np.uint8)
    np.savez_compressed(os.path.join(HERE, "host_support_tree.npz"), **masks)

    ref = load_ref()
    out = {}
    w = syn.Workload("bt", batch=6, vocab=40, hidden=8, src_min=4, src_max=16, emissions="logits", kind="viterbi")
    b = syn.make_batch(w, seed=7)
    lp = torch.log_softmax(b.logits, -1)
    ob, tok = lp.max(-1)
    tok[:, 5] = 1  # a pad token inside the graph is skipped by the walk
    S, R, Lt, Mt = oracle.pcfg_viterbi(ob.numpy(), b.links.numpy(), b.output_length.numpy())
    scores = torch.from_numpy(S[:, 1, :]).clone()
    scores = scores / torch.arange(b.L // 4).unsqueeze(0)
    scores.masked_fill_(scores.isnan(), float("-inf"))
    pred = scores[:, 1:].max(-1)[1] + 1
    mask = b.left_tree_mask.long()
    rows = []
    for i in range(b.B):  # one sentence per call: the reference raises for ragged batches
        r = ref.viterbi_decoding(pred[i:i + 1], b.output_length[i:i + 1], torch.from_numpy(Lt[i:i + 1]),
                                 torch.from_numpy(R[i:i + 1]), torch.from_numpy(Mt[i:i + 1]), tok[i:i + 1], mask, 1)
        assert r.dtype == torch.float32
        rows.append(r[0].long().numpy())
    maxlen = max(len(r) for r in rows)
    dec = np.full((b.B, maxlen), 1, np.int64)
    for i, r in enumerate(rows):
        dec[i, :len(r)] = r
    out.update(pred_length=pred.numpy(), output_length=b.output_length.numpy(), L=Lt, R=R, M=Mt, tokens=tok.numpy(),
               left_tree_mask=mask.numpy().astype(np.uint8), decoded=dec,
               decoded_len=np.array([len(r) for r in rows], np.int64))
    np.savez_compressed(os.path.join(HERE, "host_viterbi_decoding.npz"), **out)
    print("wrote host_support_tree.npz, host_viterbi_decoding.npz; decoded lens", [len(r) for r in rows])


if __name__ == "__main__":
    main()
