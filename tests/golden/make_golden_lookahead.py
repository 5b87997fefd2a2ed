"""Generates ``host_lookahead.npz``: token lists of the reference model's own "lookahead" and "greedy" decoding
(fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:419-482), run on the CPU.

The block lives inside ``forward_decoder``, which needs a fairseq model; the ``if self.args.decode_strategy in
["lookahead", "greedy"]:`` statement is cut out of the method's syntax tree and executed with the names it reads
bound to seeded tensors (links, unreduced_logits, unreduced_tokens, output_tokens, left_tree_mask) and stand-ins for
``self`` (args, tgt_dict, ``_max_left_index`` as buffered_tree_mask builds it, :213-218) and ``decoder_out``.
Lookahead cases use batch size 1 (with more sentences the reference takes the left-child term of every sentence
from sentence 0, :425); greedy cases use a ragged batch.

Usage:  python tests/golden/make_golden_lookahead.py --reference /path/to/PCFG-NAT
"""
import argparse
import ast
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

PAD = 1


class Dict_:
    pad_index = PAD

    def __getitem__(self, i):
        return f"tok{i}"


def decoding_block(reference):
    path = os.path.join(reference, "fs_plugins", "models", "glat_decomposed_with_link_two_hands_tri_pcfg.py")
    tree = ast.parse(open(path).read())
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name == "forward_decoder":
            for stmt in node.body:
                if isinstance(stmt, ast.If) and "lookahead" in ast.unparse(stmt.test):
                    only = ast.If(test=stmt.test, body=stmt.body, orelse=[])  # drop the viterbi branch (needs CUDA)
                    return compile(ast.Module(body=[ast.fix_missing_locations(ast.copy_location(only, stmt))],
                                              type_ignores=[]), path, "exec")
    raise RuntimeError("decoding block not found")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    a = ap.parse_args()
    code = decoding_block(a.reference)
    spec = importlib.util.spec_from_file_location("ref_lemon_tree", os.path.join(a.reference, "fs_plugins", "models", "lemon_tree.py"))
    lemon = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(lemon)
    syn = entry.load_package().synthetic
    out = {}
    cases = [("look_b1_a", "lookahead", 1, 11, 24, 1.0), ("look_b1_b", "lookahead", 1, 12, 40, 0.5),
             ("greedy_b4", "greedy", 4, 13, 28, 1.0), ("greedy_b1", "greedy", 1, 14, 16, 1.0)]
    for name, strategy, B, seed, L, beta in cases:
        w = syn.Workload(name, batch=B, vocab=60, hidden=8, src_min=max(2, L // 8), src_max=L // 4, emissions="logits",
                         kind="viterbi")
        b = syn.make_batch(w, seed=seed)
        L = b.L
        ob, tok = torch.log_softmax(b.logits, -1).max(-1)
        tok = torch.where(torch.arange(L)[None, :] < b.output_length[:, None], tok, torch.full_like(tok, PAD))
        tok[:, 3] = PAD  # a padding token inside the sentence is skipped by the walk
        me = types.SimpleNamespace()
        me.args = types.SimpleNamespace(decode_strategy=strategy, decode_beta=beta)
        me.tgt_dict = Dict_()
        idx = torch.arange(0, L).unsqueeze(0).unsqueeze(-1) + torch.zeros(1, L, 2, dtype=torch.int64)
        idx[:, :, 0] = 0
        idx[:, :, 1] = torch.where((idx[:, :, 1] - 1) < 0, 0, idx[:, :, 1] - 1)
        me._max_left_index = idx
        output_tokens = torch.where(torch.arange(L)[None, :] < b.output_length[:, None], 3, PAD)
        ns = {"torch": torch, "self": me, "links": b.links, "unreduced_logits": ob, "unreduced_tokens": tok.tolist(),
              "output_tokens": output_tokens, "bsz": B, "prelen": L, "left_span": 2,
              "left_tree_mask": b.left_tree_mask.bool(), "BinaryTreeNode": lemon.BinaryTreeNode,
              "decoder_out": types.SimpleNamespace(output_tokens=output_tokens)}
        exec(code, ns)
        res = ns["output_tokens"]
        out.update({f"{name}_links": b.links.numpy(), f"{name}_ob": ob.numpy(), f"{name}_tok": tok.numpy(),
                    f"{name}_out_len": b.output_length.numpy(), f"{name}_mask": b.left_tree_mask.long().numpy(),
                    f"{name}_beta": np.float32(beta), f"{name}_lookahead": np.int64(strategy == "lookahead"),
                    f"{name}_result": res.numpy()})
        print(name, res.shape, res[0].tolist()[:12])
    np.savez_compressed(os.path.join(HERE, "host_lookahead.npz"), **out)


if __name__ == "__main__":
    main()
