"""Generates ``host_extract_links.npz``: outputs of the reference model's own ``extract_links``
(fs_plugins/models/glat_decomposed_with_link_two_hands_tri_pcfg.py:140-201) and ``buffered_tree_mask`` (:205-226),
run on the CPU.  The model class cannot be imported without fairseq, so the two method definitions (and the
module's ``logsumexp`` helper) are compiled from the file's text and called with a stand-in ``self`` that carries
the attributes they read; the link projections are passed as callables that return the seeded tensors.  The seeded
tensors are autograd leaves: the gradient of sum(links * G) over the finite entries, for a seeded G, is recorded as
well (the reference's own backward through its ~30 operators), which pins the hand-written backward.

Usage:  python tests/golden/make_golden_links.py --reference /path/to/PCFG-NAT
"""
import argparse
import ast
import importlib.util
import os
import types

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def load_methods(reference):
    path = os.path.join(reference, "fs_plugins", "models", "glat_decomposed_with_link_two_hands_tri_pcfg.py")
    tree = ast.parse(open(path).read())
    wanted = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.FunctionDef) and node.name in ("extract_links", "buffered_tree_mask", "logsumexp"):
            wanted.setdefault(node.name, node)
    spec = importlib.util.spec_from_file_location("ref_lemon_tree", os.path.join(reference, "fs_plugins", "models", "lemon_tree.py"))
    lemon = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(lemon)
    ns = {"torch": torch, "F": F, "Tensor": torch.Tensor, "BinaryTreeNode": lemon.BinaryTreeNode}
    for name in ("logsumexp", "buffered_tree_mask", "extract_links"):
        mod = ast.Module(body=[wanted[name]], type_ignores=[])
        exec(compile(mod, path, "exec"), ns)
    return ns


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    a = ap.parse_args()
    ns = load_methods(a.reference)
    out = {}
    cases = [("small", 3, 18, 4, 8, 0), ("mid", 2, 42, 8, 16, 1)]
    for name, B, L, heads, dim, seed in cases:
        g = torch.Generator().manual_seed(seed)
        q, kl, kr = (torch.randn(B, L, heads * dim, generator=g).requires_grad_(True) for _ in range(3))
        gates = torch.randn(B, L, heads, generator=g).requires_grad_(True)
        lengths = torch.tensor([L, L - 8, max(2, L - 16)][:B])
        lengths = lengths - (lengths % 2)  # graph lengths are even at left_tree_layer 1
        pad = 1
        prev = torch.where(torch.arange(L)[None, :] < lengths[:, None], 3, pad)
        me = types.SimpleNamespace()
        me.args = types.SimpleNamespace(links_feature="feature", decoder_attention_heads=heads,
                                        decoder_embed_dim=heads * dim, left_tree_layer=1, src_upsample_scale=4.0)
        me.pad = pad
        me.max_left = 1
        me._left_tree_mask = torch.empty(0)
        me._right_tree_mask = torch.empty(0)
        me._main_chain = torch.empty(0)
        left_mask, right_mask, main_chain = ns["buffered_tree_mask"](me, prev)
        features = torch.zeros(B, L, 1)
        links = ns["extract_links"](me, features, prev, None, lambda x: q, lambda x: kl, lambda x: kr, lambda x: gates,
                                    left_mask, right_mask, main_chain)
        G = torch.randn(links.shape, generator=g)
        fin = torch.isfinite(links)
        (torch.where(fin, links, torch.zeros_like(links)) * G).sum().backward()
        out.update({f"{name}_G": G.numpy(), f"{name}_dq": q.grad.numpy(), f"{name}_dkl": kl.grad.numpy(),
                    f"{name}_dkr": kr.grad.numpy(), f"{name}_dgates": gates.grad.numpy()})
        q, kl, kr, gates, links = q.detach(), kl.detach(), kr.detach(), gates.detach(), links.detach()
        out.update({f"{name}_q": q.numpy(), f"{name}_kl": kl.numpy(), f"{name}_kr": kr.numpy(), f"{name}_gates": gates.numpy(),
                    f"{name}_prev": prev.numpy(), f"{name}_heads": np.int64(heads),
                    f"{name}_left_mask": left_mask.numpy(), f"{name}_right_mask": right_mask.numpy(),
                    f"{name}_main_chain": main_chain.numpy(), f"{name}_links": links.numpy()})
        print(name, links.shape, float(torch.isfinite(links).float().mean()))
    np.savez_compressed(os.path.join(HERE, "host_extract_links.npz"), **out)


if __name__ == "__main__":
    main()
