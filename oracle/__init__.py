"""CPU oracle for the PCFG-NAT loss / decoding path (TEST INFRASTRUCTURE ONLY).

Thin numpy/ctypes front end of ``pcfg_oracle.c`` (a loop-for-loop C restatement of the
reference kernels, each function citing the reference file:line it follows) plus a
torch-CPU restatement of the output projection + log-softmax + gather/max that the
reference gets from ``nn.Linear`` + ``log_softmax`` (models/glat_decomposed_with_link_two_hands_tri_pcfg.py:237,
:414-415).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this package;
the product package never does.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "pcfg_oracle.c")
_LIB = os.path.join(_HERE, "liboracle.so")
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_i64p = ctypes.POINTER(ctypes.c_int64)


# Two builds of the same source: "faithful" (no FMA contraction, -O2: the checker, bit-comparable with the
# reference kernels' arithmetic) and "native" (-O3 -march=native: only ever timed, as a second CPU figure).
_FLAGS = {"faithful": ["-O2", "-std=c11", "-fno-fast-math", "-ffp-contract=off", "-fopenmp"],
          "native": ["-O3", "-march=native", "-std=c11", "-fno-fast-math", "-fopenmp"]}
_LIBS = {"faithful": _LIB, "native": os.path.join(_HERE, "liboracle_native.so")}
_loaded = {}
_active = "faithful"


def build(force=False, which="faithful"):
    """Compile pcfg_oracle.c with gcc (no fast-math, OpenMP over sentences; see ``_FLAGS``)."""
    out = _LIBS[which]
    if not force and os.path.isfile(out) and os.path.getmtime(out) >= os.path.getmtime(_SRC):
        return out
    cmd = ["gcc", *_FLAGS[which], "-shared", "-fPIC", _SRC, "-o", out, "-lm"]
    subprocess.run(cmd, check=True)
    return out


def use_build(which):
    """Selects the build the wrappers below call ("faithful" is the checker; "native" is for timing only)."""
    global _active, _lib
    if which not in _FLAGS:
        raise ValueError(which)
    _active = which
    _lib = None


def build_flags():
    return " ".join(_FLAGS[_active])


def lib():
    global _lib
    if _lib is None:
        if _active not in _loaded:
            _loaded[_active] = ctypes.CDLL(build(which=_active))
        _lib = _loaded[_active]
    return _lib


def _f32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_f32p)


def _i64(a):
    a = np.ascontiguousarray(a, dtype=np.int64)
    return a, a.ctypes.data_as(_i64p)


def table_shapes(B, L, T, ML):
    """Shapes of the inside tables S and C (pcfg_loss.cu:389-394)."""
    Mc = (L - 2) // (ML + 1) + 1
    Lt = L - Mc
    return (B, Mc, T + 2), (B, Lt, T + 2, ML + 2)


def pcfg_loss(match_all, links, output_length, target_length):
    """Inside tables (S, C); loss_b = S[b, 0, 0]  (pcfg_loss.cu:379-401)."""
    ma, pma = _f32(match_all)
    lk, plk = _f32(links)
    ol, pol = _i64(output_length)
    tl, ptl = _i64(target_length)
    B, L, T = ma.shape
    ML = lk.shape[2] - 1
    sS, sC = table_shapes(B, L, T, ML)
    S = np.empty(sS, np.float32)
    C = np.empty(sC, np.float32)
    rc = lib().oracle_pcfg_loss(pma, plk, pol, ptl, B, L, T, ML, S.ctypes.data_as(_f32p), C.ctypes.data_as(_f32p))
    if rc:
        raise RuntimeError(f"oracle_pcfg_loss rc={rc}")
    return S, C


def pcfg_loss_backward(grad_output, S, C, match_all, links, output_length, target_length, return_scratch=False):
    """(match_all_grad, links_grad) for max_left == 1 (pcfg_loss_backward.cu:654-721)."""
    go, pgo = _f32(grad_output)
    S_, pS = _f32(S)
    C_, pC = _f32(C)
    ma, pma = _f32(match_all)
    lk, plk = _f32(links)
    ol, pol = _i64(output_length)
    tl, ptl = _i64(target_length)
    B, L, T = ma.shape
    ML = lk.shape[2] - 1
    Sg = np.empty_like(S_)
    Cg = np.empty_like(C_)
    mg = np.empty_like(ma)
    lg = np.empty_like(lk)
    rc = lib().oracle_pcfg_loss_backward(pgo, pS, pC, pma, plk, pol, ptl, B, L, T, ML, Sg.ctypes.data_as(_f32p),
                                         Cg.ctypes.data_as(_f32p), mg.ctypes.data_as(_f32p),
                                         lg.ctypes.data_as(_f32p))
    if rc:
        raise RuntimeError(f"oracle_pcfg_loss_backward rc={rc}")
    if return_scratch:
        return mg, lg, Sg, Cg
    return mg, lg


def pcfg_best_tree(S, C, match_all, links, output_length, target_length):
    """tree[B, L] int64 (pcfg_best_tree.cu:333-360)."""
    S_, pS = _f32(S)
    C_, pC = _f32(C)
    ma, pma = _f32(match_all)
    lk, plk = _f32(links)
    ol, pol = _i64(output_length)
    tl, ptl = _i64(target_length)
    B, L, T = ma.shape
    ML = lk.shape[2] - 1
    tree = np.empty((B, L), np.int64)
    rc = lib().oracle_pcfg_best_tree(pS, pC, pma, plk, pol, ptl, B, L, T, ML, tree.ctypes.data_as(_i64p))
    if rc:
        raise RuntimeError(f"oracle_pcfg_best_tree rc={rc}")
    return tree


def pcfg_viterbi(ob_lprob, links, output_length, return_c=False):
    """(S, R, L, M) of shape [B, L, L//4] (pcfg_viterbi.cu:272-301)."""
    ob, pob = _f32(ob_lprob)
    lk, plk = _f32(links)
    ol, pol = _i64(output_length)
    B, L = ob.shape
    ML = lk.shape[2] - 1
    Q = L // 4
    S = np.empty((B, L, Q), np.float32)
    Cv = np.empty((B, L, Q), np.float32)
    R = np.empty((B, L, Q), np.int64)
    Lt = np.empty((B, L, Q), np.int64)
    Mt = np.empty((B, L, Q), np.int64)
    rc = lib().oracle_pcfg_viterbi(pob, plk, pol, B, L, ML, S.ctypes.data_as(_f32p), Cv.ctypes.data_as(_f32p),
                                   R.ctypes.data_as(_i64p), Lt.ctypes.data_as(_i64p), Mt.ctypes.data_as(_i64p))
    if rc:
        raise RuntimeError(f"oracle_pcfg_viterbi rc={rc}")
    if return_c:
        return S, R, Lt, Mt, Cv
    return S, R, Lt, Mt


def viterbi_decoding_lists(pred_length, output_length, L_trace, R_trace, M_trace, unreduced_tokens, left_tree_mask,
                           pad_index):
    """Per-sentence token lists of the back-trace (pcfg_loss.cpp:20-59)."""
    pl, ppl = _i64(pred_length)
    ol, pol = _i64(output_length)
    Lt, pLt = _i64(L_trace)
    R, pR = _i64(R_trace)
    Mt, pMt = _i64(M_trace)
    tk, ptk = _i64(unreduced_tokens)
    mk, pmk = _i64(left_tree_mask)
    B, L, Q = Lt.shape
    cap = L
    out = np.full((B, cap), pad_index, np.int64)
    cnt = np.zeros((B,), np.int64)
    rc = lib().oracle_viterbi_decoding(ppl, pol, pLt, pR, pMt, ptk, pmk, mk.shape[0], ctypes.c_int64(int(pad_index)), B,
                                       L, Q, cap, out.ctypes.data_as(_i64p), cnt.ctypes.data_as(_i64p))
    if rc:
        raise RuntimeError(f"oracle_viterbi_decoding rc={rc}")
    return [out[i, : cnt[i]].tolist() for i in range(B)]


def viterbi_decoding(pred_length, output_length, L_trace, R_trace, M_trace, unreduced_tokens, left_tree_mask,
                     pad_index):
    """Padded float32 [B, maxlen] matrix, the reference's return type (pcfg_loss.cpp:60-71).

    The reference's ``index_put_`` of a ragged row raises for B > 1 with unequal lengths;
    here ragged rows are right-padded with ``pad_index``.
    """
    rows = viterbi_decoding_lists(pred_length, output_length, L_trace, R_trace, M_trace, unreduced_tokens,
                                  left_tree_mask, pad_index)
    maxlen = max((len(r) for r in rows), default=0)
    out = np.full((len(rows), maxlen), pad_index, np.float32)
    for i, r in enumerate(rows):
        out[i, : len(r)] = r
    return out


def logsoftmax_gather(word_ins_out, select_idx, require_gradient=False):
    """selected[b,l,s] = log_softmax(word_ins_out[b,l,:])[select_idx[b,l,s]]; with
    ``require_gradient`` also returns the softmax that the reference writes in place
    (logsoftmax_gather.cu:250-291).  Returns (selected f32, probs f32 or None)."""
    x = np.array(word_ins_out, dtype=np.float32, order="C", copy=True)
    B, L, V = x.shape
    sel = np.ascontiguousarray(np.broadcast_to(np.asarray(select_idx, dtype=np.int64), (B, L, np.shape(select_idx)[2])))
    slen = sel.shape[2]
    out = np.empty((B, L, slen), np.float32)
    rc = lib().oracle_logsoftmax_gather(x.ctypes.data_as(_f32p), sel.ctypes.data_as(_i64p), ctypes.c_int64(slen),
                                        ctypes.c_int64(1), ctypes.c_int64(B * L), V, slen, int(bool(require_gradient)),
                                        out.ctypes.data_as(_f32p))
    if rc:
        raise RuntimeError(f"oracle_logsoftmax_gather rc={rc}")
    return out, (x if require_gradient else None)


def proj_logsoftmax(hidden, weight, targets, rows_per_sentence):
    """Output projection + log-softmax + target gather / row max, in fp32 on the CPU.

    hidden [N, H] (fp16 or fp32 values), weight [V, H]; row r belongs to sentence
    r // rows_per_sentence and is gathered at targets[sentence, :].  Restates
    ``output_projection`` -> ``log_softmax`` -> gather / ``max(-1)``
    (models/glat_decomposed_with_link_two_hands_tri_pcfg.py:237, :414-415;
    criterions/nat_pcfg_loss.py:109).  Returns (match [N, T], max_lprob [N], argmax [N], lse [N]).
    """
    import torch

    h = torch.as_tensor(np.asarray(hidden)).float()
    w = torch.as_tensor(np.asarray(weight)).float()
    logits = h @ w.t()
    lse = torch.logsumexp(logits, dim=-1)
    lp = logits - lse[:, None]
    mx, am = lp.max(dim=-1)
    tg = torch.as_tensor(np.asarray(targets)).long()
    sent = torch.arange(h.shape[0]) // rows_per_sentence
    match = lp.gather(1, tg[sent])
    return match.numpy(), mx.numpy(), am.numpy(), lse.numpy()
