"""Generates the golden fixtures ``ref_*.npz`` by running the UNMODIFIED reference CUDA kernels.

Needs a GPU and the reference extension built by ``oracle/build_ref.py`` (oracle/_ref/).
Inputs come from the package's seeded synthetic generator; both the inputs and the
reference outputs are stored, so the CPU tests need neither the reference nor a GPU.

Only shapes with at most 128 main-chain nodes (graph length <= 256) are run: there each
reference launch has a single row segment per sentence, so none of its inter-block
spin-waits (pcfg_loss.cu:131-136, pcfg_viterbi.cu:69) depends on another block being
resident, and its ticket overshoot (pcfg_loss.cu:121-127) only reaches empty segments.

Usage (on a GPU box):  python tests/golden/make_golden_ref.py --out <directory>
"""
import argparse
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402
from oracle.build_ref import load_ref  # noqa: E402

pkg = entry.load_package()
syn = pkg.synthetic

LOSS_CASES = {
    # name: (Workload, seed, extra)
    "loss_tiny": (syn.WORKLOADS["tiny_loss"], 0),
    "loss_ragged": (syn.Workload("loss_ragged", batch=6, vocab=300, hidden=16, src_min=3, src_max=12,
                                 emissions="logits"), 1),
    "loss_mid": (syn.Workload("loss_mid", batch=3, vocab=300, hidden=16, src_min=24, src_max=32,
                              emissions="logits"), 2),
}
VITERBI_CASES = {
    "viterbi_ragged": (syn.Workload("viterbi_ragged", batch=5, vocab=200, hidden=16, src_min=4, src_max=14,
                                    emissions="logits", kind="viterbi"), 3),
    "viterbi_mid": (syn.Workload("viterbi_mid", batch=2, vocab=200, hidden=16, src_min=28, src_max=32,
                                 emissions="logits", kind="viterbi"), 4),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True, help="directory the .npz fixtures are written to")
    a = ap.parse_args()
    os.makedirs(a.out, exist_ok=True)
    ref = load_ref()
    dev = torch.device("cuda:0")
    for name, (w, seed) in LOSS_CASES.items():
        b = syn.make_batch(w, seed=seed)
        assert b.L <= 256
        if name == "loss_ragged":
            # infeasible sentence: fewer graph nodes than the target needs (n > m - 2); loss is -inf
            n0 = int(b.target_length[0])
            b.output_length[0] = n0 + (n0 % 2)
        match = syn.reference_match_all(b)
        ma, lk = match.to(dev), b.links.to(dev)
        ol, tl = b.output_length.to(dev), b.target_length.to(dev)
        S, C = ref.pcfg_loss(ma, lk, ol, tl, 1)
        mg, lg = ref.pcfg_loss_backward(torch.ones(b.B, device=dev), S, C, ma, lk, ol, tl, 1)
        tree = ref.pcfg_best_tree(S, C, ma, lk, ol, tl, 1)
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(a.out, f"ref_{name}.npz"), match_all=match.numpy(), links=b.links.numpy(),
                            output_length=b.output_length.numpy(), target_length=b.target_length.numpy(),
                            S=S.cpu().numpy(), C=C.cpu().numpy(), match_all_grad=mg.cpu().numpy(),
                            links_grad=lg.cpu().numpy(), tree=tree.cpu().numpy())
        print(name, "loss", S[:, 0, 0].tolist())
    for name, (w, seed) in VITERBI_CASES.items():
        b = syn.make_batch(w, seed=seed)
        assert b.L <= 256
        lp = torch.log_softmax(b.logits, -1)
        ob, tok = lp.max(-1)
        S, R, Lt, Mt = ref.pcfg_viterbi(ob.to(dev), b.links.to(dev), b.output_length.to(dev), 1)
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(a.out, f"ref_{name}.npz"), ob_lprob=ob.numpy(), tokens=tok.numpy(),
                            links=b.links.numpy(), output_length=b.output_length.numpy(), S=S.cpu().numpy(),
                            R=R.cpu().numpy(), L=Lt.cpu().numpy(), M=Mt.cpu().numpy())
        print(name, "root scores", S[:, 1, :6].tolist())
    # log-softmax + gather, fp32 and fp16, with and without the in-place softmax
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(2, 8, 1000, generator=g) * 3
    tgt = torch.randint(0, 1000, (2, 10), generator=g)
    out = {"logits": logits.numpy(), "targets": tgt.numpy()}
    for dt, tag in ((torch.float32, "f32"), (torch.float16, "f16")):
        for grad in (False, True):
            x = logits.to(dev).to(dt).contiguous()
            sel = ref.logsoftmax_gather(x, tgt.to(dev).unsqueeze(1).expand(-1, 8, -1), grad)
            torch.cuda.synchronize()
            out[f"selected_{tag}_{int(grad)}"] = sel.cpu().numpy()
            if grad:
                out[f"probs_{tag}"] = x.float().cpu().numpy()
    np.savez_compressed(os.path.join(a.out, "ref_logsoftmax_gather.npz"), **out)
    print("wrote", sorted(os.listdir(a.out)))


if __name__ == "__main__":
    main()
