"""Drop-in for ``fs_plugins/custom_ops/pcfg_loss.py`` of PCFG-NAT on top of libpcfgnat.so.

Same five public operators with the same positional signatures and return structure
(fs_plugins/custom_ops/pcfg_loss.py:85, :117, :142, :181, :183-184):

    cuda_pcfg_loss(match_all, links, output_length, target_length)           -> loss [B]
    cuda_pcfg_best_tree(match_all, links, output_length, target_length)      -> (tree [B,L] i64, loss [B])
    cuda_pcfg_viterbi(ob_lprob, links, output_length)                        -> (scores [B,L/4], R, L, M)
    dag_logsoftmax_gather_inplace(word_ins_out, select_idx)                  -> (word_ins_out, selected f32)
    viterbi_decoding(pred_length, output_length, L_trace, R_trace, M_trace,
                     unreduced_tokens, left_tree_mask, pad_index)            -> float32 [B, maxlen]

and ``get_pcfg_kernel()`` returning an object with the six extension-level functions an
unmodified reference wrapper calls (fs_plugins/custom_ops/pcfg_loss.cpp:75-82).

The host side only validates arguments, allocates outputs with torch and hands raw
device pointers to the C ABI on the caller's current CUDA stream.  There is no CPU path:
every operator raises when CUDA or the library is unavailable.

Known, deliberate differences from the reference:
* only ``max_left == 1`` (left_tree_layer 1) and float32 tables are implemented;
* ``config`` values 1..4 all run the kernels (the reference silently skips its launches for
  2..4, pcfg_loss_backward.cu:694-697); other values raise the reference's message;
* ``viterbi_decoding`` right-pads ragged batches (the reference raises for them,
  pcfg_loss.cpp:66-69) and also accepts CUDA tensors, in which case nothing is copied to
  the host except the per-sentence counts;
* outputs are produced on the tensors' own device and current stream (the reference
  always launches on the legacy default stream 0, pcfg_loss.cu:395).
"""
import ctypes

import torch
from torch.autograd import Function

from .. import _cabi

_status = {}
_kernel_shim = None


def _require_cuda():
    if not torch.cuda.is_available():
        # same condition and wording as the reference loader (pcfg_loss.py:20-21)
        raise RuntimeError("You need GPU to use the custom cuda operations")


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def _status_ptr(dev):
    """Per-device int32 word the kernels OR PCFGNAT_STATUS_* bits into."""
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=dev)
        _status[key] = t
    return t.data_ptr()


def read_status(device=None, reset=True):
    """Returns the PCFGNAT_STATUS_* bits recorded on ``device`` (synchronises)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(key)
    if t is None:
        return 0
    v = int(t.item())
    if reset:
        t.zero_()
    return v


def _check_config(config):
    if not (1 <= int(config) <= 4):
        raise RuntimeError("config should be 1~4")


def _f32_cuda(t, name, ndim):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if t.dim() != ndim:
        raise RuntimeError(f"{name} dim != {ndim}")
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be float32 (got {t.dtype}); the DP tables are fp32 only")
    return t.contiguous()


def _lengths(t, name, B, dev):
    if not isinstance(t, torch.Tensor) or t.dim() != 1 or t.shape[0] != B:
        raise RuntimeError(f"{name} must be a 1-d tensor of batch size {B}")
    return t.to(device=dev, dtype=torch.int64).contiguous()


def _loss_args(match_all, links, output_length, target_length):
    match_all = _f32_cuda(match_all, "match_all", 3)
    links = _f32_cuda(links, "links", 4)
    B, L, T = match_all.shape
    if links.shape[0] != B or links.shape[1] != L or links.shape[3] != L:
        raise RuntimeError("links must be [batch, prelen, max_left+1, prelen] matching match_all")
    if links.device != match_all.device:
        raise RuntimeError("match_all and links must be on the same device")
    max_left = links.shape[2] - 1
    if max_left != 1:
        raise RuntimeError(f"only max_left == 1 (left_tree_layer 1) is implemented, got max_left = {max_left}")
    if L < 2 or T < 1:
        raise RuntimeError("prelen must be >= 2 and tarlen >= 1")
    dev = match_all.device
    return match_all, links, _lengths(output_length, "output_length", B, dev), _lengths(target_length, "target_length", B, dev), B, L, T, max_left


def table_shapes(B, L, T, max_left):
    Mc = (L - 2) // (max_left + 1) + 1
    return (B, Mc, T + 2), (B, L - Mc, T + 2, max_left + 2)


_main_chain_cache = {}  # (address of the main-chain mask, prelen) -> node list, slots, left rows


class _Kernel:
    """Extension-level API: the functions of the reference's pybind module (pcfg_loss.cpp:75-82)."""

    @staticmethod
    def pcfg_loss(match_all, links, output_length, target_length, config=1, want_c=True):
        """Inside tables (S [B,Mc,T+2], C [B,Lt,T+2,max_left+2]); replaces pcfg_loss (pcfg_loss.cu:379-401)."""
        _require_cuda()
        ma, lk, ol, tl, B, L, T, ml = _loss_args(match_all, links, output_length, target_length)
        sS, sC = table_shapes(B, L, T, ml)
        with torch.cuda.device(ma.device):
            S = torch.empty(sS, dtype=torch.float32, device=ma.device)
            C = torch.empty(sC, dtype=torch.float32, device=ma.device) if want_c else None
            rc = _cabi.lib().pcfgnat_loss_fwd(ma.data_ptr(), lk.data_ptr(), ol.data_ptr(), tl.data_ptr(), B, L, T, ml,
                                              S.data_ptr(), C.data_ptr() if want_c else None, _status_ptr(ma.device),
                                              _stream(ma.device))
        _cabi.check(rc, "pcfgnat_loss_fwd")
        return S, C

    @staticmethod
    def pcfg_loss_backward(grad_output, S, C, match_all, links, output_length, target_length, config=1):
        """(match_all_grad, links_grad); replaces pcfg_loss_backward (pcfg_loss_backward.cu:654-721).
        ``C`` is accepted for signature parity; the leaf entries it would supply are read from
        ``match_all`` directly."""
        _require_cuda()
        _check_config(config)
        ma, lk, ol, tl, B, L, T, ml = _loss_args(match_all, links, output_length, target_length)
        sS, _ = table_shapes(B, L, T, ml)
        S = _f32_cuda(S, "S", 3)
        if tuple(S.shape) != sS:
            raise RuntimeError(f"S must have shape {sS}")
        go = grad_output.to(device=ma.device, dtype=torch.float32).contiguous()
        if go.shape != (B,):
            raise RuntimeError("grad_output must be [batch]")
        with torch.cuda.device(ma.device):
            G = torch.empty(sS, dtype=torch.float32, device=ma.device)
            mg = torch.empty_like(ma)
            lg = torch.empty_like(lk)
            rc = _cabi.lib().pcfgnat_loss_bwd(go.data_ptr(), S.data_ptr(), ma.data_ptr(), lk.data_ptr(), ol.data_ptr(),
                                              tl.data_ptr(), B, L, T, ml, G.data_ptr(), mg.data_ptr(), lg.data_ptr(),
                                              _status_ptr(ma.device), _stream(ma.device))
        _cabi.check(rc, "pcfgnat_loss_bwd")
        return mg, lg

    @staticmethod
    def pcfg_loss_fwd_bwd(match_all, links, output_length, target_length):
        """Fused forward + backward for grad_output == 1: (loss [B], match_all_grad, links_grad)."""
        _require_cuda()
        ma, lk, ol, tl, B, L, T, ml = _loss_args(match_all, links, output_length, target_length)
        l = _cabi.lib()
        nbytes = l.pcfgnat_loss_workspace_bytes(B, L, T, ml)
        with torch.cuda.device(ma.device):
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=ma.device)
            loss = torch.empty(B, dtype=torch.float32, device=ma.device)
            mg = torch.empty_like(ma)
            lg = torch.empty_like(lk)
            rc = l.pcfgnat_loss_fwd_bwd(ma.data_ptr(), lk.data_ptr(), ol.data_ptr(), tl.data_ptr(), B, L, T, ml,
                                        ws.data_ptr(), nbytes, loss.data_ptr(), mg.data_ptr(), lg.data_ptr(),
                                        _status_ptr(ma.device), _stream(ma.device))
        _cabi.check(rc, "pcfgnat_loss_fwd_bwd")
        return loss, mg, lg

    @staticmethod
    def pcfg_best_tree(S, C, match_all, links, output_length, target_length, config=1):
        """tree [B, L] int64; replaces pcfg_best_tree (pcfg_best_tree.cu:333-360).  ``C`` is accepted
        for signature parity and not read."""
        _require_cuda()
        _check_config(config)
        ma, lk, ol, tl, B, L, T, ml = _loss_args(match_all, links, output_length, target_length)
        sS, _ = table_shapes(B, L, T, ml)
        S = _f32_cuda(S, "S", 3)
        if tuple(S.shape) != sS:
            raise RuntimeError(f"S must have shape {sS}")
        with torch.cuda.device(ma.device):
            tree = torch.empty((B, L), dtype=torch.int64, device=ma.device)
            rc = _cabi.lib().pcfgnat_best_tree(S.data_ptr(), ma.data_ptr(), lk.data_ptr(), ol.data_ptr(), tl.data_ptr(),
                                               B, L, T, ml, tree.data_ptr(), _status_ptr(ma.device), _stream(ma.device))
        _cabi.check(rc, "pcfgnat_best_tree")
        return tree

    @staticmethod
    def pcfg_viterbi(ob_lprob, links, output_length, config=1):
        """(S, R, L, M) of shape [B, L, L//4]; replaces pcfg_viterbi (pcfg_viterbi.cu:272-301)."""
        _require_cuda()
        _check_config(config)
        ob = _f32_cuda(ob_lprob, "ob_lprob", 2)
        lk = _f32_cuda(links, "links", 4)
        B, L = ob.shape
        if lk.shape[0] != B or lk.shape[1] != L or lk.shape[3] != L or lk.device != ob.device:
            raise RuntimeError("links must be [batch, prelen, max_left+1, prelen] on ob_lprob's device")
        ml = lk.shape[2] - 1
        if ml != 1:
            raise RuntimeError(f"only max_left == 1 (left_tree_layer 1) is implemented, got max_left = {ml}")
        if L < 8:
            raise RuntimeError("prelen must be >= 8 (the tables have prelen // 4 length columns)")
        ol = _lengths(output_length, "output_length", B, ob.device)
        Q = L // 4
        with torch.cuda.device(ob.device):
            S = torch.empty((B, L, Q), dtype=torch.float32, device=ob.device)
            R = torch.empty((B, L, Q), dtype=torch.int64, device=ob.device)
            Lt = torch.empty_like(R)
            Mt = torch.empty_like(R)
            rc = _cabi.lib().pcfgnat_viterbi(ob.data_ptr(), lk.data_ptr(), ol.data_ptr(), B, L, ml, S.data_ptr(),
                                             R.data_ptr(), Lt.data_ptr(), Mt.data_ptr(), _status_ptr(ob.device),
                                             _stream(ob.device))
        _cabi.check(rc, "pcfgnat_viterbi")
        return S, R, Lt, Mt

    @staticmethod
    def logsoftmax_gather(word_ins_out, select_idx, require_gradient):
        """selected [B, L, slen] f32; overwrites ``word_ins_out`` with softmax probabilities when
        ``require_gradient``; replaces logsoftmax_gather (logsoftmax_gather.cu:295-359)."""
        _require_cuda()
        if not word_ins_out.is_cuda:
            raise RuntimeError("word_ins_out must be a CUDA tensor")
        if not select_idx.is_cuda:
            raise RuntimeError("select_idx must be a CUDA tensor")
        if word_ins_out.dim() != 3:
            raise RuntimeError("word_ins_out dim != 3")
        if select_idx.dim() != 3:
            raise RuntimeError("select_idx dim != 3")
        B, L, V = word_ins_out.shape
        if select_idx.shape[0] != B:
            raise RuntimeError("batch size not match")
        if select_idx.shape[1] != L:
            raise RuntimeError("prelen size not match")
        if select_idx.dtype != torch.int64:
            raise RuntimeError("select_idx should be long")
        if not word_ins_out.is_contiguous():
            raise RuntimeError("word_ins_out is not contiguous")
        if word_ins_out.dtype == torch.float32:
            dt = 0
        elif word_ins_out.dtype == torch.float16:
            dt = 1
        else:
            raise RuntimeError(f"logsoftmax_gather not implemented for '{word_ins_out.dtype}'")
        slen = select_idx.shape[2]
        sb, sl, ss = select_idx.stride()
        dev = word_ins_out.device
        with torch.cuda.device(dev):
            selected = torch.empty((B, L, slen), dtype=torch.float32, device=dev)
            rc = _cabi.lib().pcfgnat_logsoftmax_gather(word_ins_out.data_ptr(), dt, select_idx.data_ptr(), sb, sl, ss,
                                                       B * L, L, V, slen, int(bool(require_gradient)),
                                                       selected.data_ptr(), _status_ptr(dev), _stream(dev))
        _cabi.check(rc, "pcfgnat_logsoftmax_gather")
        return selected

    @staticmethod
    def proj_logsoftmax_gather(hidden, weight, targets=None, output_length=None, target_length=None,
                               want_max=False, want_lse=False):
        """Fused output projection + log-softmax + gather / row max on the tensor cores.

        hidden [B, L, H] f16, weight [V, H] f16, targets [B, T] int64 or None.  Returns a dict with
        ``match`` [B, L, T] f32 = log P(target | node) when targets are given (EOS-masked as the
        criterion does, criterions/nat_pcfg_loss.py:112-115, when both lengths are given),
        ``max_lprob`` [B, L] f32 and ``argmax`` [B, L] int64 when ``want_max``, ``lse`` [B, L] f32 when
        ``want_lse``.  Stands in for output_projection -> logsoftmax_gather / log_softmax().max()
        (models/glat_decomposed_with_link_two_hands_tri_pcfg.py:237, :414-415) without materialising
        the [B, L, V] logits."""
        _require_cuda()
        if not (hidden.is_cuda and weight.is_cuda) or hidden.device != weight.device:
            raise RuntimeError("hidden and weight must be CUDA tensors on the same device")
        if hidden.dtype != torch.float16 or weight.dtype != torch.float16:
            raise RuntimeError("hidden and weight must be float16")
        if hidden.dim() != 3 or weight.dim() != 2 or weight.shape[1] != hidden.shape[2]:
            raise RuntimeError("hidden must be [batch, prelen, H] and weight [V, H]")
        B, L, H = hidden.shape
        V = weight.shape[0]
        if H % 64 != 0 or H > 512:
            raise RuntimeError(f"H must be a multiple of 64 and at most 512, got {H}")
        hidden, weight = hidden.contiguous(), weight.contiguous()
        dev = hidden.device
        T = 0
        if targets is not None:
            if targets.dim() != 2 or targets.shape[0] != B:
                raise RuntimeError("targets must be [batch, tarlen]")
            targets = targets.to(device=dev, dtype=torch.int64).contiguous()
            T = targets.shape[1]
        if target_length is not None and output_length is None:
            raise RuntimeError("target_length (EOS masking) needs output_length as well")
        ol = _lengths(output_length, "output_length", B, dev) if output_length is not None else None
        tl = _lengths(target_length, "target_length", B, dev) if target_length is not None else None
        l = _cabi.lib()
        nbytes = l.pcfgnat_proj_workspace_bytes(B, L, T, V)
        out = {}
        with torch.cuda.device(dev):
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
            match = torch.empty((B, L, T), dtype=torch.float32, device=dev) if T else None
            mx = torch.empty((B, L), dtype=torch.float32, device=dev) if want_max else None
            am = torch.empty((B, L), dtype=torch.int64, device=dev) if want_max else None
            lse = torch.empty((B, L), dtype=torch.float32, device=dev) if want_lse else None
            ptr = lambda t: t.data_ptr() if t is not None else None
            rc = l.pcfgnat_proj_logsoftmax_gather(hidden.data_ptr(), weight.data_ptr(), ptr(targets), ptr(ol), ptr(tl),
                                                  B, L, T, V, H, ptr(match), ptr(mx), ptr(am), ptr(lse), ws.data_ptr(),
                                                  nbytes, _status_ptr(dev), _stream(dev))
        _cabi.check(rc, "pcfgnat_proj_logsoftmax_gather")
        if match is not None:
            out["match"] = match
        if want_max:
            out["max_lprob"], out["argmax"] = mx, am
        if want_lse:
            out["lse"] = lse
        return out

    @staticmethod
    def proj_dlogits(hidden, weight, targets, output_length, target_length, lse, grad_match, n_rows=None, out=None,
                     row_index_out=None):
        """d loss / d logits of ``proj_logsoftmax_gather`` as bf16 [B * L, V], the logits recomputed on the
        tensor cores tile by tile (nothing of size [B, L, V] was kept from the forward).  ``lse`` [B, L] is the
        forward's ``want_lse`` output, ``grad_match`` [B, L, T] the gradient of its ``match``.

        With ``n_rows`` (a host integer: the real graph nodes of the batch, sum of the output lengths) the result is
        compact: (d-logits [n_rows, V] of the real nodes only, row_index [n_rows] int64 = their positions b * L + l),
        so that the two GEMMs that follow skip the padding rows.  ``out`` / ``row_index_out``: buffers of at least
        that many rows to write into (a step object's static ones)."""
        _require_cuda()
        if hidden.dtype != torch.float16 or weight.dtype != torch.float16 or not (hidden.is_cuda and weight.is_cuda):
            raise RuntimeError("hidden and weight must be float16 CUDA tensors")
        B, L, H = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        hidden, weight = hidden.contiguous(), weight.contiguous()
        targets = targets.to(device=dev, dtype=torch.int64).contiguous()
        T = targets.shape[1]
        lse = _f32_cuda(lse, "lse", 2)
        g = _f32_cuda(grad_match, "grad_match", 3)
        if tuple(lse.shape) != (B, L) or tuple(g.shape) != (B, L, T):
            raise RuntimeError("lse must be [batch, prelen] and grad_match [batch, prelen, tarlen]")
        if target_length is not None and output_length is None:
            raise RuntimeError("target_length (EOS masking) needs output_length as well")
        ol = _lengths(output_length, "output_length", B, dev) if output_length is not None else None
        tl = _lengths(target_length, "target_length", B, dev) if target_length is not None else None
        l = _cabi.lib()
        nbytes = l.pcfgnat_proj_workspace_bytes(B, L, T, V)
        ptr = lambda t: t.data_ptr() if t is not None else None
        with torch.cuda.device(dev):
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
            if n_rows is not None:
                n = int(n_rows)
                if n < 0 or n > B * L:
                    raise RuntimeError("n_rows must be between 0 and batch * prelen")
                dl = out if out is not None else torch.empty((n, V), dtype=torch.bfloat16, device=dev)
                idx = row_index_out if row_index_out is not None else torch.empty((n,), dtype=torch.int64, device=dev)
                if dl.dtype != torch.bfloat16 or dl.dim() != 2 or dl.shape[1] != V or dl.shape[0] < n or \
                        not dl.is_contiguous() or idx.dtype != torch.int64 or idx.numel() < n:
                    raise RuntimeError("out must be a contiguous bfloat16 [>= n_rows, V], row_index_out int64 [>= n_rows]")
                rc = l.pcfgnat_proj_dlogits_compact(hidden.data_ptr(), weight.data_ptr(), targets.data_ptr(), ptr(ol),
                                                    ptr(tl), lse.data_ptr(), g.data_ptr(), B, L, T, V, H, n,
                                                    dl.data_ptr(), idx.data_ptr(), None, ws.data_ptr(), nbytes,
                                                    _status_ptr(dev), _stream(dev))
                _cabi.check(rc, "pcfgnat_proj_dlogits_compact")
                return dl[:n], idx[:n]
            dl = out if out is not None else torch.empty((B * L, V), dtype=torch.bfloat16, device=dev)
            rc = l.pcfgnat_proj_dlogits(hidden.data_ptr(), weight.data_ptr(), targets.data_ptr(), ptr(ol), ptr(tl),
                                        lse.data_ptr(), g.data_ptr(), B, L, T, V, H, dl.data_ptr(), ws.data_ptr(), nbytes,
                                        _status_ptr(dev), _stream(dev))
        _cabi.check(rc, "pcfgnat_proj_dlogits")
        return dl

    @staticmethod
    def proj_backward_gemms(dlogits, weight_bf16, rows_bf16, want_rows=True, want_weight=True):
        """The two products that finish the projection's backward, on the tensor cores: (d rows [n, H] float32 =
        dlogits [n, V] @ weight_bf16 [V, H], d weight [V, H] float32 = dlogits.T @ rows_bf16 [n, H]); None for a
        product not wanted.  All operands bfloat16 and contiguous; V and H multiples of 8."""
        _require_cuda()
        dev = dlogits.device
        for t, name in ((dlogits, "dlogits"), (weight_bf16, "weight_bf16"), (rows_bf16, "rows_bf16")):
            if t is None:
                continue
            if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or not t.is_contiguous():
                raise RuntimeError(f"{name} must be a contiguous bfloat16 CUDA matrix")
        n, V = dlogits.shape
        H = (weight_bf16 if weight_bf16 is not None else rows_bf16).shape[1]
        if want_rows and (weight_bf16 is None or tuple(weight_bf16.shape) != (V, H)):
            raise RuntimeError("weight_bf16 must be [V, H]")
        if want_weight and (rows_bf16 is None or tuple(rows_bf16.shape) != (n, H)):
            raise RuntimeError("rows_bf16 must be [n, H]")
        ptr = lambda t: t.data_ptr() if t is not None else None
        with torch.cuda.device(dev):
            d_rows = torch.empty((n, H), dtype=torch.float32, device=dev) if want_rows else None
            d_weight = torch.empty((V, H), dtype=torch.float32, device=dev) if want_weight else None
            rc = _cabi.lib().pcfgnat_proj_backward_gemms(dlogits.data_ptr(), ptr(weight_bf16), ptr(rows_bf16), n, V, H,
                                                         ptr(d_rows), ptr(d_weight), _status_ptr(dev), _stream(dev))
        _cabi.check(rc, "pcfgnat_proj_backward_gemms")
        return d_rows, d_weight

    @staticmethod
    def viterbi_decoding_device(pred_length, output_length, L_trace, R_trace, M_trace, unreduced_tokens,
                                left_tree_mask, pad_index):
        """Device back-trace: (tokens [B, L] int64 padded with pad_index, count [B] int64), no host sync."""
        _require_cuda()
        dev = L_trace.device if L_trace.is_cuda else torch.device("cuda", torch.cuda.current_device())
        i64 = lambda t: t.to(device=dev, dtype=torch.int64).contiguous()
        Lt, R, Mt = i64(L_trace), i64(R_trace), i64(M_trace)
        if Lt.dim() != 3 or R.shape != Lt.shape or Mt.shape != Lt.shape:
            raise RuntimeError("L_trace, R_trace, M_trace must be [batch, prelen, prelen//4] and agree")
        B, L, Q = Lt.shape
        pl, ol, tk, mk = i64(pred_length), i64(output_length), i64(unreduced_tokens), i64(left_tree_mask)
        if pl.shape != (B,) or ol.shape != (B,) or tk.shape != (B, L):
            raise RuntimeError("pred_length/output_length must be [batch], unreduced_tokens [batch, prelen]")
        if mk.dim() != 2 or mk.shape[0] != mk.shape[1]:
            raise RuntimeError("left_tree_mask must be square")
        with torch.cuda.device(dev):
            out = torch.empty((B, L), dtype=torch.int64, device=dev)
            cnt = torch.empty((B,), dtype=torch.int64, device=dev)
            rc = _cabi.lib().pcfgnat_viterbi_backtrace(pl.data_ptr(), ol.data_ptr(), Lt.data_ptr(), R.data_ptr(),
                                                       Mt.data_ptr(), tk.data_ptr(), mk.data_ptr(), mk.shape[0],
                                                       int(pad_index), B, L, Q, L, out.data_ptr(), cnt.data_ptr(),
                                                       _status_ptr(dev), _stream(dev))
        _cabi.check(rc, "pcfgnat_viterbi_backtrace")
        return out, cnt

    @staticmethod
    def viterbi_decode_device(S, penalty, output_length, L_trace, R_trace, M_trace, unreduced_tokens, left_tree_mask,
                              pad_index):
        """Length choice + back-trace in one launch (models/...pcfg.py:488-502): scores = S[:, 1, :] / penalty,
        NaN -> -inf, first maximum over lengths 1 .. Q-1, then the walk.  Returns (tokens [B, L] int64 padded
        with pad_index, count [B] int64, pred_length [B] int64), no host sync."""
        _require_cuda()
        S = _f32_cuda(S, "S", 3)
        dev = S.device
        B, L, Q = S.shape
        i64 = lambda t: t.to(device=dev, dtype=torch.int64).contiguous()
        Lt, R, Mt = i64(L_trace), i64(R_trace), i64(M_trace)
        if tuple(Lt.shape) != (B, L, Q) or R.shape != Lt.shape or Mt.shape != Lt.shape:
            raise RuntimeError("L_trace, R_trace, M_trace must have S's shape [batch, prelen, prelen//4]")
        pen = penalty.to(device=dev, dtype=torch.float32).reshape(-1).contiguous()
        if pen.numel() != Q:
            raise RuntimeError(f"penalty must hold {Q} values")
        ol, tk, mk = i64(output_length), i64(unreduced_tokens), i64(left_tree_mask)
        if ol.shape != (B,) or tk.shape != (B, L) or mk.dim() != 2 or mk.shape[0] != mk.shape[1]:
            raise RuntimeError("output_length [batch], unreduced_tokens [batch, prelen], square left_tree_mask expected")
        with torch.cuda.device(dev):
            out = torch.empty((B, L), dtype=torch.int64, device=dev)
            cnt = torch.empty((B,), dtype=torch.int64, device=dev)
            pred = torch.empty((B,), dtype=torch.int64, device=dev)
            rc = _cabi.lib().pcfgnat_viterbi_decode(S.data_ptr(), pen.data_ptr(), ol.data_ptr(), Lt.data_ptr(), R.data_ptr(),
                                                    Mt.data_ptr(), tk.data_ptr(), mk.data_ptr(), mk.shape[0],
                                                    int(pad_index), B, L, Q, L, pred.data_ptr(), out.data_ptr(),
                                                    cnt.data_ptr(), _status_ptr(dev), _stream(dev))
        _cabi.check(rc, "pcfgnat_viterbi_decode")
        return out, cnt, pred

    @staticmethod
    def lookahead_decode_device(links, ob_lprob, unreduced_tokens, output_length, left_tree_mask, pad_index,
                                decode_beta=1.0, strategy="lookahead"):
        """The model's "lookahead" / "greedy" decoding (models/...pcfg.py:419-482) in one launch: per-node arg-max of
        the (lookahead-adjusted) transitions and the in-order walk from node 1.  Returns (tokens [B, L] int64 padded
        with pad_index, count [B] int64), no host sync.  Every sentence uses its own log-probabilities for the
        left-child term (the reference uses sentence 0's for all when B > 1, :425)."""
        _require_cuda()
        if strategy not in ("lookahead", "greedy"):
            raise RuntimeError(f"unknown decode strategy {strategy!r}")
        lk = _f32_cuda(links, "links", 4)
        B, L = lk.shape[0], lk.shape[1]
        if lk.shape[2] != 2 or lk.shape[3] != L:
            raise RuntimeError("links must be [batch, prelen, 2, prelen] (max_left == 1)")
        dev = lk.device
        i64 = lambda t: t.to(device=dev, dtype=torch.int64).contiguous()
        ob = _f32_cuda(ob_lprob, "ob_lprob", 2) if strategy == "lookahead" else None
        if ob is not None and (tuple(ob.shape) != (B, L) or ob.device != dev):
            raise RuntimeError("ob_lprob must be [batch, prelen] on the device of links")
        tk, ol, mk = i64(unreduced_tokens), i64(output_length), i64(left_tree_mask)
        if tuple(tk.shape) != (B, L) or tuple(ol.shape) != (B,) or mk.dim() != 2 or mk.shape[0] != mk.shape[1]:
            raise RuntimeError("unreduced_tokens [batch, prelen], output_length [batch], square left_tree_mask expected")
        with torch.cuda.device(dev):
            out = torch.empty((B, L), dtype=torch.int64, device=dev)
            cnt = torch.empty((B,), dtype=torch.int64, device=dev)
            rc = _cabi.lib().pcfgnat_lookahead_decode(lk.data_ptr(), ob.data_ptr() if ob is not None else None,
                                                      tk.data_ptr(), ol.data_ptr(), mk.data_ptr(), mk.shape[0],
                                                      float(decode_beta), 1 if strategy == "lookahead" else 0,
                                                      int(pad_index), B, L, 1, L, out.data_ptr(), cnt.data_ptr(),
                                                      _status_ptr(dev), _stream(dev))
        _cabi.check(rc, "pcfgnat_lookahead_decode")
        return out, cnt

    @staticmethod
    def viterbi_decoding(pred_length, output_length, L_trace, R_trace, M_trace, unreduced_tokens, left_tree_mask,
                         pad_index):
        """float32 [B, maxlen] padded with pad_index on the device of ``pred_length``;
        replaces the host function viterbi_decoding (pcfg_loss.cpp:12-73)."""
        out, cnt = _Kernel.viterbi_decoding_device(pred_length, output_length, L_trace, R_trace, M_trace,
                                                   unreduced_tokens, left_tree_mask, pad_index)
        maxlen = int(cnt.max().item()) if cnt.numel() else 0
        return out[:, :maxlen].to(dtype=torch.float32, device=pred_length.device)


    @staticmethod
    def copy_links_main_rows(dst, src):
        """Copies the rows of the transition tensor the kernels read (main-chain nodes: odd a) from ``src``
        (pinned host or device, [B, L, 2, L] f32 contiguous) into the CUDA tensor ``dst`` of the same shape,
        asynchronously on the current stream; the other rows of ``dst`` keep their contents."""
        _require_cuda()
        if not dst.is_cuda or dst.dtype != torch.float32 or dst.dim() != 4 or dst.shape[2] != 2:
            raise RuntimeError("dst must be a float32 CUDA tensor [batch, prelen, 2, prelen]")
        if src.dtype != torch.float32 or tuple(src.shape) != tuple(dst.shape):
            raise RuntimeError("src must be a float32 tensor of dst's shape")
        if not dst.is_contiguous() or not src.is_contiguous():
            raise RuntimeError("dst and src must be contiguous")
        B, L = dst.shape[0], dst.shape[1]
        with torch.cuda.device(dst.device):
            rc = _cabi.lib().pcfgnat_copy_links_main_rows(dst.data_ptr(), src.data_ptr(), B, L, 1, _stream(dst.device))
        _cabi.check(rc, "pcfgnat_copy_links_main_rows")

    @staticmethod
    def copy_real_rows(dst, src, host_lengths, b0=0, b1=None, max_copies=0):
        """Copies the rows of the real graph nodes (l < length, clamped to [0, L]) of sentences [b0, b1) of ``src``
        [B, L, ...] into ``dst`` of the same shape on the current stream with copy-engine copies, no kernel: one per
        sentence, or at most ``max_copies`` (> 0), joined across the smallest gaps of padding rows.  Returns the
        number of rows sent.  ``host_lengths`` [B] int64 lives in host memory.  Rows of ``dst`` that are not sent
        keep what they held."""
        _require_cuda()
        if not dst.is_cuda or dst.dim() < 2 or tuple(src.shape) != tuple(dst.shape) or src.dtype != dst.dtype or \
                not (dst.is_contiguous() and src.is_contiguous()):
            raise RuntimeError("dst must be a contiguous CUDA tensor [batch, prelen, ...] and src of its shape and type")
        if host_lengths.is_cuda or host_lengths.dtype != torch.int64 or tuple(host_lengths.shape) != (dst.shape[0],) or \
                not host_lengths.is_contiguous():
            raise RuntimeError("host_lengths must be a contiguous int64 host tensor [batch]")
        B, L = dst.shape[0], dst.shape[1]
        b1 = B if b1 is None else b1
        if not 0 <= b0 <= b1 <= B:
            raise RuntimeError("sentence range out of bounds")
        row_bytes = dst[0, 0].numel() * dst.element_size()
        sent = ctypes.c_int64(0)
        with torch.cuda.device(dst.device):
            rc = _cabi.lib().pcfgnat_copy_real_rows(dst.data_ptr(), src.data_ptr(), host_lengths.data_ptr(), b0, b1, L,
                                                    row_bytes, int(max_copies), ctypes.addressof(sent),
                                                    _stream(dst.device))
        _cabi.check(rc, "pcfgnat_copy_real_rows")
        return int(sent.value)

    @staticmethod
    def stage_inputs(output_length, hidden_dst=None, hidden_src=None, links_dst=None, links_src=None):
        """Fetches a batch's large inputs from pinned host memory with one kernel that reads the host buffers itself,
        and only what the kernels read: the decoder states of the real graph nodes (``hidden`` [B, L, H]) and the
        transitions of main-chain nodes to later nodes inside the sentence (``links`` [B, L, 2, L]; the rest of those
        rows becomes -inf, other rows are left alone).  ``output_length`` is the DEVICE tensor of the lengths.
        Asynchronous on the current stream; the host buffers must stay unchanged until it has run."""
        _require_cuda()
        dev = output_length.device
        if not output_length.is_cuda or output_length.dtype != torch.int64 or output_length.dim() != 1:
            raise RuntimeError("output_length must be an int64 CUDA tensor [batch]")
        B = output_length.shape[0]
        L = None
        row_bytes = 0
        for dst, src, nd, name in ((hidden_dst, hidden_src, 3, "hidden"), (links_dst, links_src, 4, "links")):
            if (dst is None) != (src is None):
                raise RuntimeError(f"{name}: give both the destination and the source")
            if dst is None:
                continue
            if not dst.is_cuda or dst.device != dev or dst.dim() != nd or dst.shape[0] != B or not dst.is_contiguous():
                raise RuntimeError(f"{name}_dst must be a contiguous CUDA tensor with the batch in front")
            if tuple(src.shape) != tuple(dst.shape) or src.dtype != dst.dtype or not src.is_contiguous():
                raise RuntimeError(f"{name}_src must have the shape and type of {name}_dst")
            if not (src.is_cuda or src.is_pinned()):
                raise RuntimeError(f"{name}_src must be pinned host memory (or device memory): the kernel reads it itself")
            if L is not None and dst.shape[1] != L:
                raise RuntimeError("hidden and links disagree on prelen")
            L = dst.shape[1]
        if L is None:
            return
        if hidden_dst is not None:
            row_bytes = hidden_dst.shape[2] * hidden_dst.element_size()
            if row_bytes % 16:
                raise RuntimeError("a row of hidden must be a multiple of 16 bytes")
        if links_dst is not None and (links_dst.dtype != torch.float32 or links_dst.shape[2] != 2 or links_dst.shape[3] != L):
            raise RuntimeError("links must be float32 [batch, prelen, 2, prelen]")
        ptr = lambda t: t.data_ptr() if t is not None else None
        with torch.cuda.device(dev):
            rc = _cabi.lib().pcfgnat_stage_inputs(ptr(hidden_src), ptr(hidden_dst), row_bytes, ptr(links_src), ptr(links_dst),
                                                  output_length.data_ptr(), B, L, 1, _stream(dev))
        _cabi.check(rc, "pcfgnat_stage_inputs")

    @staticmethod
    def _links_forward(query, key_left, key_right, gate_logits, prev_output_tokens, pad_index, left_tree_mask,
                       right_tree_mask, main_chain):
        """Forward of ``extract_links``; returns (links, everything the backward needs)."""
        _require_cuda()
        if query.dim() != 4 or key_left.shape != query.shape or key_right.shape != query.shape:
            raise RuntimeError("query, key_left, key_right must be [batch, prelen, heads, head_dim] and agree")
        if not query.is_cuda:
            raise RuntimeError("query must be a CUDA tensor")
        B, L, H, D = query.shape
        dev = query.device
        dt = query.dtype if query.dtype in (torch.float16, torch.float32) else torch.float32
        q = query.detach().to(dt).contiguous()
        kl = key_left.detach().to(device=dev, dtype=dt).contiguous()
        kr = key_right.detach().to(device=dev, dtype=dt).contiguous()
        gates = gate_logits.detach().to(device=dev, dtype=torch.float32).contiguous()
        if tuple(gates.shape) != (B, L, H):
            raise RuntimeError("gate_logits must be [batch, prelen, heads]")
        if tuple(prev_output_tokens.shape) != (B, L):
            raise RuntimeError("prev_output_tokens must be [batch, prelen]")

        def u8(t, shape):  # masks prepared once (uint8, on the device, exact size) are used as they are
            if t.dtype == torch.uint8 and t.device == dev and tuple(t.shape) == shape and t.is_contiguous():
                return t
            t = t.to(device=dev)
            t = t[:L, :L] if len(shape) == 2 else t[:L]
            return t.ne(0).to(torch.uint8).contiguous()

        lm, rm, mc = u8(left_tree_mask, (L, L)), u8(right_tree_mask, (L, L)), u8(main_chain, (L,))
        if tuple(lm.shape) != (L, L) or tuple(rm.shape) != (L, L) or tuple(mc.shape) != (L,):
            raise RuntimeError("tree masks must cover prelen nodes")
        nonpad = prev_output_tokens.to(dev).ne(pad_index).to(torch.uint8).contiguous()
        # main-chain nodes: the only ones that have, or are, right children -> compact score matrices
        key = (mc.data_ptr(), L)
        cached = _main_chain_cache.get(key)
        if cached is None:
            nodes = mc.nonzero().flatten().to(torch.int32)                   # [M] main-chain node ids
            slot_of = torch.full((L,), -1, dtype=torch.int32, device=dev)
            slot_of[nodes.long()] = torch.arange(nodes.numel(), dtype=torch.int32, device=dev)
            cached = (mc, nodes, slot_of)  # keeps mc alive: its address is the key
            _main_chain_cache.clear()
            _main_chain_cache[key] = cached
        _, nodes, slot_of = cached
        M = nodes.numel()
        lib = _cabi.lib()
        with torch.cuda.device(dev):
            qm = torch.empty((B, H, M, D), dtype=torch.float32, device=dev)
            krm = torch.empty((B, H, M, D), dtype=torch.float32, device=dev)
            klm = torch.empty((B, H, M + 1, D), dtype=torch.float32, device=dev)
            rc = lib.pcfgnat_links_gather_features(q.data_ptr(), kl.data_ptr(), kr.data_ptr(),
                                                   1 if dt == torch.float16 else 0, nodes.data_ptr(), M, B,  # PCFGNAT_DTYPE_*
                                                   L, H, D, qm.data_ptr(), klm.data_ptr(), krm.data_ptr(), _stream(dev))
            _cabi.check(rc, "pcfgnat_links_gather_features")
            ac = torch.empty((B, H, M, M), dtype=torch.float32, device=dev)
            bc = torch.empty((B, H, M + 1, M), dtype=torch.float32, device=dev)
            rc = lib.pcfgnat_links_scores(qm.data_ptr(), klm.data_ptr(), krm.data_ptr(), M, B, H, D, ac.data_ptr(),
                                          bc.data_ptr(), _stream(dev))
            _cabi.check(rc, "pcfgnat_links_scores")
            links = torch.empty((B, L, 2, L), dtype=torch.float32, device=dev)
            rc = lib.pcfgnat_links_from_scores(ac.data_ptr(), bc.data_ptr(), qm.data_ptr(), klm.data_ptr(),
                                               gates.data_ptr(), nonpad.data_ptr(), lm.data_ptr(), rm.data_ptr(),
                                               mc.data_ptr(), slot_of.data_ptr(), nodes.data_ptr(), M, B, L, H, D, 1,
                                               links.data_ptr(), _stream(dev))
        _cabi.check(rc, "pcfgnat_links_from_scores")
        saved = dict(ac=ac, bc=bc, qm=qm, klm=klm, krm=krm, gates=gates, nonpad=nonpad, lm=lm, rm=rm, mc=mc, slot_of=slot_of,
                     nodes=nodes, dims=(B, L, H, D, M))
        return links, saved

    @staticmethod
    def _links_backward(links_grad, saved):
        """(d query, d key_left, d key_right [B, L, heads, head_dim] f32, d gate_logits [B, L, heads] f32)."""
        B, L, H, D, M = saved["dims"]
        g = _f32_cuda(links_grad, "links_grad", 4)
        if tuple(g.shape) != (B, L, 2, L):
            raise RuntimeError("links_grad must have the shape of links")
        dev = g.device
        p = lambda name: saved[name].data_ptr()
        with torch.cuda.device(dev):
            X0 = torch.zeros((B, H, M, M), dtype=torch.float32, device=dev)
            X1 = torch.zeros((B, H, M, M), dtype=torch.float32, device=dev)
            dab = torch.zeros((B, H, M, 2), dtype=torch.float32, device=dev)
            dq = torch.zeros((B, L, H, D), dtype=torch.float32, device=dev)
            dkl = torch.zeros_like(dq)
            dkr = torch.zeros_like(dq)
            dgates = torch.empty((B, L, H), dtype=torch.float32, device=dev)
            rc = _cabi.lib().pcfgnat_links_backward(g.data_ptr(), p("ac"), p("bc"), p("qm"), p("klm"), p("krm"), p("gates"),
                                                    p("nonpad"), p("lm"), p("rm"), p("mc"), p("slot_of"), p("nodes"), M,
                                                    B, L, H, D, 1, X0.data_ptr(), X1.data_ptr(), dab.data_ptr(),
                                                    dq.data_ptr(), dkl.data_ptr(), dkr.data_ptr(), dgates.data_ptr(),
                                                    _stream(dev))
        _cabi.check(rc, "pcfgnat_links_backward")
        return dq, dkl, dkr, dgates

    @staticmethod
    def extract_links(query, key_left, key_right, gate_logits, prev_output_tokens, pad_index, left_tree_mask,
                      right_tree_mask, main_chain):
        """links [B, L, 2, L] f32 as the model's extract_links() forms them from the projected link features
        (models/...pcfg.py:140-201, max_left == 1): ``query``, ``key_left``, ``key_right`` [B, L, heads, head_dim]
        (outputs of the three link projections, reshaped), ``gate_logits`` [B, L, heads].  Three launches: feature
        gather, the per-head score products, and masking + joint log-softmax + head mixture + -inf rows.
        Differentiable with respect to the four feature tensors (``ExtractLinksFunc``)."""
        if torch.is_grad_enabled() and any(t.requires_grad for t in (query, key_left, key_right, gate_logits)):
            return ExtractLinksFunc.apply(query, key_left, key_right, gate_logits, prev_output_tokens, pad_index,
                                          left_tree_mask, right_tree_mask, main_chain)
        return _Kernel._links_forward(query, key_left, key_right, gate_logits, prev_output_tokens, pad_index, left_tree_mask,
                                      right_tree_mask, main_chain)[0]

    @staticmethod
    def loss_stats(sentence_loss, target_length):
        """float32 [3] = [sum_b loss_b / n_b over valid sentences, sentences, invalid sentences]: what the
        criterion's scalar is formed from (nat_pcfg_loss.py:117-135), in one launch."""
        _require_cuda()
        loss = _f32_cuda(sentence_loss, "sentence_loss", 1)
        tl = _lengths(target_length, "target_length", loss.shape[0], loss.device)
        with torch.cuda.device(loss.device):
            stats = torch.empty((3,), dtype=torch.float32, device=loss.device)
            rc = _cabi.lib().pcfgnat_loss_stats(loss.data_ptr(), tl.data_ptr(), loss.shape[0], stats.data_ptr(),
                                                _stream(loss.device))
        _cabi.check(rc, "pcfgnat_loss_stats")
        return stats

    @staticmethod
    def loss_stats_exchange(sentence_loss, target_length, peer_buffers, rank, world):
        """``loss_stats`` summed over the GPUs of the job in the same launch (peer stores over NVLink instead of
        a 12-byte all-reduce).  ``peer_buffers``: int64 CUDA tensor [world] of device pointers to every rank's
        exchange buffer as mapped in this process (see ``sharding.LossExchange``)."""
        _require_cuda()
        loss = _f32_cuda(sentence_loss, "sentence_loss", 1)
        tl = _lengths(target_length, "target_length", loss.shape[0], loss.device)
        if peer_buffers.dtype != torch.int64 or peer_buffers.device != loss.device or peer_buffers.numel() != world:
            raise RuntimeError("peer_buffers must be an int64 tensor of `world` device pointers on the loss's device")
        with torch.cuda.device(loss.device):
            stats = torch.empty((3,), dtype=torch.float32, device=loss.device)
            rc = _cabi.lib().pcfgnat_loss_stats_exchange(loss.data_ptr(), tl.data_ptr(), loss.shape[0],
                                                         peer_buffers.data_ptr(), int(rank), int(world), stats.data_ptr(),
                                                         _status_ptr(loss.device), _stream(loss.device))
        _cabi.check(rc, "pcfgnat_loss_stats_exchange")
        return stats

    @staticmethod
    def glance_select(path, pred_tokens, tgt_tokens, prev_output_tokens, target_length, noise, context_p,
                      strategy="number-random", uniform=None):
        """The glancing sampler of the criterion (nat_pcfg_loss.py:216-267) in one launch.  ``strategy`` is the
        criterion's ``--glance-strategy``: "number-random", "cmlm" or None.  The random draws are the caller's:
        ``noise`` [B, L] standard-normal (the two counting strategies), ``uniform`` in [0, 1): [B] for "cmlm",
        [B, L] for None.  Returns a dict with matchmask [B,T,L] bool, oracle [B,L], same_num [B], glance_num [B],
        keep_word_mask [B,L] bool, glat_prev_output_tokens [B,L]."""
        _require_cuda()
        dev = path.device
        if not path.is_cuda or path.dim() != 2:
            raise RuntimeError("path must be a CUDA tensor [batch, prelen]")
        B, L = path.shape
        if strategy not in GLANCE_STRATEGIES:
            raise RuntimeError(f"unknown glance strategy {strategy!r}")
        code = GLANCE_STRATEGIES[strategy]

        def i64(t, name, shape):
            if t.device != dev or t.dtype != torch.int64 or tuple(t.shape) != shape:
                raise RuntimeError(f"{name} must be an int64 tensor of shape {shape} on {dev}")
            return t.contiguous()

        def f32(t, name, shape):
            if t is None or t.device != dev or t.dtype != torch.float32 or tuple(t.shape) != shape:
                raise RuntimeError(f"{name} must be a float32 tensor of shape {shape} on {dev}")
            return t.contiguous()

        if tgt_tokens.dim() != 2 or tgt_tokens.shape[0] != B:
            raise RuntimeError("tgt_tokens must be [batch, tarlen]")
        T = tgt_tokens.shape[1]
        path = i64(path, "path", (B, L))
        pred = i64(pred_tokens, "pred_tokens", (B, L))
        tgt = i64(tgt_tokens, "tgt_tokens", (B, T))
        prev = i64(prev_output_tokens, "prev_output_tokens", (B, L))
        tl = _lengths(target_length, "target_length", B, dev)
        noise = f32(noise, "noise", (B, L)) if code != 2 else None
        if code == 1:
            uniform = f32(uniform, "uniform", (B,))
        elif code == 2:
            uniform = f32(uniform, "uniform", (B, L))
        else:
            uniform = None
        ptr = lambda t: t.data_ptr() if t is not None else None
        with torch.cuda.device(dev):
            matchmask = torch.empty((B, T, L), dtype=torch.bool, device=dev)
            keep = torch.empty((B, L), dtype=torch.bool, device=dev)
            oracle = torch.empty((B, L), dtype=torch.int64, device=dev)
            glat_prev = torch.empty((B, L), dtype=torch.int64, device=dev)
            same_num = torch.empty((B,), dtype=torch.int64, device=dev)
            glance_num = torch.empty((B,), dtype=torch.int64, device=dev)
            rc = _cabi.lib().pcfgnat_glance_select(path.data_ptr(), pred.data_ptr(), tgt.data_ptr(), prev.data_ptr(),
                                                   tl.data_ptr(), ptr(noise), ptr(uniform), code, float(context_p),
                                                   B, L, T, matchmask.data_ptr(), oracle.data_ptr(),
                                                   same_num.data_ptr(), glance_num.data_ptr(), keep.data_ptr(),
                                                   glat_prev.data_ptr(), _stream(dev))
        _cabi.check(rc, "pcfgnat_glance_select")
        return {"matchmask": matchmask, "oracle": oracle, "same_num": same_num, "glance_num": glance_num,
                "keep_word_mask": keep, "glat_prev_output_tokens": glat_prev}

    @staticmethod
    def _force_emit_args(x, keep, name):
        x = _f32_cuda(x, name, 3)
        B, L, T = x.shape
        if keep.device != x.device or keep.dtype not in (torch.bool, torch.uint8) or tuple(keep.shape) != (B, L):
            raise RuntimeError(f"keep_word_mask must be a bool tensor of shape {(B, L)} on {x.device}")
        return x, keep.contiguous(), B, L, T

    @staticmethod
    def force_emit(match_all, matchmask, keep_word_mask, out=None):
        """The force-emit mask of the training pass (nat_pcfg_loss.py:116-121): entries [b, l, t] of a node whose
        token was revealed (``keep_word_mask`` [B, L]) become -inf unless ``matchmask`` [B, T, L] aligns it to t.
        ``out`` may be ``match_all`` itself."""
        _require_cuda()
        ma, keep, B, L, T = _Kernel._force_emit_args(match_all, keep_word_mask, "match_all")
        if matchmask.device != ma.device or matchmask.dtype not in (torch.bool, torch.uint8) or \
                tuple(matchmask.shape) != (B, T, L):
            raise RuntimeError(f"matchmask must be a bool tensor of shape {(B, T, L)} on {ma.device}")
        mm = matchmask.contiguous()
        with torch.cuda.device(ma.device):
            if out is None:
                out = torch.empty_like(ma)
            rc = _cabi.lib().pcfgnat_force_emit(ma.data_ptr(), mm.data_ptr(), keep.data_ptr(), B, L, T, out.data_ptr(),
                                                _stream(ma.device))
        _cabi.check(rc, "pcfgnat_force_emit")
        return out

    @staticmethod
    def force_emit_grad(grad, keep_word_mask, out=None):
        """Gradient side of ``force_emit``: rows of revealed nodes are zero (the reference detaches them)."""
        _require_cuda()
        g, keep, B, L, T = _Kernel._force_emit_args(grad, keep_word_mask, "grad")
        with torch.cuda.device(g.device):
            if out is None:
                out = torch.empty_like(g)
            rc = _cabi.lib().pcfgnat_force_emit_grad(g.data_ptr(), keep.data_ptr(), B, L, T, out.data_ptr(),
                                                     _stream(g.device))
        _cabi.check(rc, "pcfgnat_force_emit_grad")
        return out


GLANCE_STRATEGIES = {"number-random": 0, "cmlm": 1, None: 2}  # PCFGNAT_GLANCE_*


def get_pcfg_kernel():
    """The extension object of the reference loader (pcfg_loss.py:18-47); nothing is JIT-compiled here."""
    global _kernel_shim
    _require_cuda()
    if _kernel_shim is None:
        _cabi.lib()  # raises LibraryMissing with build instructions; never falls back
        _kernel_shim = _Kernel()
    return _kernel_shim


class CUDAPCFGLossFunc(Function):
    """loss_b = S[b, 0, 0]; gradients are computed eagerly in forward for grad_output == 1 and
    scaled in backward, as in the reference (pcfg_loss.py:49-85)."""
    config = 1

    @staticmethod
    def forward(ctx, match_all, links, output_length, target_length):
        k = get_pcfg_kernel()
        need_grad = ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        if need_grad:
            loss, mg, lg = k.pcfg_loss_fwd_bwd(match_all, links, output_length, target_length)
            ctx.save_for_backward(mg, lg)
            return loss
        S, _ = k.pcfg_loss(match_all, links, output_length, target_length, CUDAPCFGLossFunc.config, want_c=False)
        return S[:, 0, 0].clone()

    @staticmethod
    def backward(ctx, grad_output):
        if not (ctx.needs_input_grad[0] or ctx.needs_input_grad[1]):
            return None, None, None, None
        mg, lg = ctx.saved_tensors
        B = mg.shape[0]
        return mg * grad_output.view(B, 1, 1), lg * grad_output.view(B, 1, 1, 1), None, None


cuda_pcfg_loss = CUDAPCFGLossFunc.apply


class CUDAPCFGBestTreeFunc(Function):
    """(tree, S[:, 0, 0]) — no gradient (pcfg_loss.py:89-117)."""
    config = 1

    @staticmethod
    def forward(ctx, match_all, links, output_length, target_length):
        k = get_pcfg_kernel()
        S, _ = k.pcfg_loss(match_all, links, output_length, target_length, CUDAPCFGBestTreeFunc.config, want_c=False)
        tree = k.pcfg_best_tree(S, None, match_all, links, output_length, target_length, CUDAPCFGBestTreeFunc.config)
        ctx.mark_non_differentiable(tree)
        return tree, S[:, 0, 0].clone()

    @staticmethod
    def backward(ctx, *grads):
        return None, None, None, None


cuda_pcfg_best_tree = CUDAPCFGBestTreeFunc.apply


class CUDAPCFGViterbiFunc(Function):
    """(S[:, 1, :], R, L, M) — no gradient (pcfg_loss.py:119-142)."""
    config = 1

    @staticmethod
    def forward(ctx, ob_lprob, links, output_length):
        S, R, Lt, Mt = get_pcfg_kernel().pcfg_viterbi(ob_lprob, links, output_length, CUDAPCFGViterbiFunc.config)
        ctx.mark_non_differentiable(R, Lt, Mt)
        return S[:, 1, :].clone(), R, Lt, Mt

    @staticmethod
    def backward(ctx, *grads):
        return None, None, None


cuda_pcfg_viterbi = CUDAPCFGViterbiFunc.apply


class DagLogsoftmaxGatherFunc(Function):
    """log-softmax + gather with the logits buffer reused for the backward: forward overwrites
    ``word_ins_out`` with softmax probabilities when it needs a gradient; backward turns that
    buffer into the logits gradient in place, once (pcfg_loss.py:144-181)."""

    @staticmethod
    def forward(ctx, word_ins_out, select_idx):
        need_grad = ctx.needs_input_grad[0]
        selected = get_pcfg_kernel().logsoftmax_gather(word_ins_out, select_idx, need_grad)
        ctx.mark_dirty(word_ins_out)
        ctx.set_materialize_grads(False)
        if need_grad:
            ctx.save_for_backward(word_ins_out, select_idx)
            ctx.has_backward = False
        return word_ins_out, selected

    @staticmethod
    def backward(ctx, grad_word_ins_out, grad_output):
        if not ctx.needs_input_grad[0]:
            return None, None
        assert grad_word_ins_out is None, "Cannot reuse word_ins_out after logsoftmax_gather"
        if grad_output is None:
            return None, None
        assert not ctx.has_backward, "Cannot backward twice in logsoftmax_gather"
        ctx.has_backward = True
        probs, idx = ctx.saved_tensors
        # d logits = -p * sum_s g_s + scatter(g): done in the saved buffer
        probs.mul_(grad_output.sum(-1, keepdim=True).neg_().to(probs.dtype))
        probs.scatter_add_(-1, idx, grad_output.to(probs.dtype))
        return probs, None


dag_logsoftmax_gather_inplace = DagLogsoftmaxGatherFunc.apply


def proj_backward_products(dlogits, weight, rows):
    """(dlogits @ weight, dlogits.T @ rows) in float32 from bf16 d-logits [n, V], the projection weight [V, H] and the
    decoder states of the same n rows [n, H] (either may be None: that product is skipped).  On this library's
    tensor-core kernels (``pcfgnat_proj_backward_gemms``); shapes whose V or H is not a multiple of 8 cannot be
    described to the tensor maps and go through torch's matmul instead."""
    V = dlogits.shape[1]
    H = (weight if weight is not None else rows).shape[1]
    if V % 8 == 0 and H % 8 == 0:
        return get_pcfg_kernel().proj_backward_gemms(
            dlogits, weight.to(torch.bfloat16).contiguous() if weight is not None else None,
            rows.to(torch.bfloat16).contiguous() if rows is not None else None,
            want_rows=weight is not None, want_weight=rows is not None)
    d_rows = (dlogits @ weight.to(torch.bfloat16)).float() if weight is not None else None
    d_weight = (dlogits.t() @ rows.to(torch.bfloat16)).float() if rows is not None else None
    return d_rows, d_weight


class ProjLogsoftmaxGatherFunc(Function):
    """match = log_softmax(hidden @ weight.T)[targets] with a backward that never holds a [B, L, V] tensor of
    the forward: the forward keeps only the per-row log-sum-exp; the backward recomputes the logits on the
    tensor cores into d loss / d logits (bf16, the only [B * L, V] buffer, alive during the backward only) and
    finishes with this library's two tensor-core products (``proj_backward_products``).  Stands in for output_projection + DagLogsoftmaxGatherFunc
    (models/...pcfg.py:237, custom_ops/pcfg_loss.py:160-180), whose forward overwrites the float32 logits with
    the softmax to keep them for the backward."""

    @staticmethod
    def forward(ctx, hidden, weight, targets, output_length, target_length, n_rows=None):
        out = get_pcfg_kernel().proj_logsoftmax_gather(hidden, weight, targets, output_length, target_length,
                                                       want_lse=True)
        ctx.save_for_backward(hidden, weight, targets, output_length, target_length, out["lse"])
        ctx.n_rows = n_rows if output_length is not None else None
        return out["match"]

    @staticmethod
    def backward(ctx, grad_match):
        hidden, weight, targets, ol, tl, lse = ctx.saved_tensors
        B, L, H = hidden.shape
        k = get_pcfg_kernel()
        d_hidden = d_weight = None
        need_h, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        V = weight.shape[0]
        if ctx.n_rows is None:  # every row of the padded tensor
            dl = k.proj_dlogits(hidden, weight, targets, ol, tl, lse, grad_match.contiguous())
            rows = hidden.reshape(B * L, H)
            idx = None
        else:  # the real graph nodes only
            dl, idx = k.proj_dlogits(hidden, weight, targets, ol, tl, lse, grad_match.contiguous(), n_rows=ctx.n_rows)
            rows = hidden.reshape(B * L, H).index_select(0, idx) if need_w else None
        d_rows, d_weight = proj_backward_products(dl, weight if need_h else None, rows if need_w else None)
        if need_h:
            if idx is None:
                d_hidden = d_rows.to(hidden.dtype).view(B, L, H)
            else:
                d_hidden = torch.zeros((B * L, H), dtype=hidden.dtype, device=hidden.device)
                d_hidden.index_copy_(0, idx, d_rows.to(hidden.dtype))
                d_hidden = d_hidden.view(B, L, H)
        if need_w:
            d_weight = d_weight.to(weight.dtype)
        return d_hidden, d_weight, None, None, None, None


class ExtractLinksFunc(Function):
    """links = extract_links(link features) with a hand-written backward: the reference gets its gradient from autograd
    through the ~30 operators of the model's extract_links (models/...pcfg.py:163-199), which keeps several
    [B, L, 2, L, heads] tensors alive; here the backward recomputes a row's quantities from the compact per-head score
    matrices the forward kept."""

    @staticmethod
    def forward(ctx, query, key_left, key_right, gate_logits, prev_output_tokens, pad_index, left_tree_mask, right_tree_mask,
                main_chain):
        links, saved = _Kernel._links_forward(query, key_left, key_right, gate_logits, prev_output_tokens, pad_index,
                                              left_tree_mask, right_tree_mask, main_chain)
        ctx.saved = saved
        ctx.dtypes = (query.dtype, key_left.dtype, key_right.dtype, gate_logits.dtype)
        return links

    @staticmethod
    def backward(ctx, links_grad):
        dq, dkl, dkr, dgates = _Kernel._links_backward(links_grad.contiguous(), ctx.saved)
        out = [g.to(dt) if need else None
               for g, dt, need in zip((dq, dkl, dkr, dgates), ctx.dtypes, ctx.needs_input_grad[:4])]
        return (*out, None, None, None, None, None)


class ForceEmitFunc(Function):
    """match_all with the force-emit mask applied; no gradient reaches the rows of revealed nodes
    (criterions/nat_pcfg_loss.py:116-121)."""

    @staticmethod
    def forward(ctx, match_all, matchmask, keep_word_mask):
        ctx.save_for_backward(keep_word_mask)
        return get_pcfg_kernel().force_emit(match_all, matchmask, keep_word_mask)

    @staticmethod
    def backward(ctx, grad):
        (keep,) = ctx.saved_tensors
        return get_pcfg_kernel().force_emit_grad(grad.contiguous(), keep), None, None


def force_emit_mask(match_all_eos_masked, matchmask, keep_word_mask):
    """What the criterion does to the emissions when the glancing sampler revealed tokens and ``--no-force-emit``
    is not set: ``matchmask`` [B, T, L] and ``keep_word_mask`` [B, L] as ``glance_select`` returns them."""
    return ForceEmitFunc.apply(match_all_eos_masked, matchmask, keep_word_mask)


def proj_logsoftmax_gather_with_grad(hidden, weight, targets, output_length=None, target_length=None, n_rows=None):
    """``match`` [B, L, T] of ``proj_logsoftmax_gather``, differentiable with respect to hidden and weight.
    ``n_rows``: the number of real graph nodes of the batch (sum of ``output_length``) where the host knows it; the
    backward then forms d-logits and runs its two GEMMs over those rows only instead of all B * L."""
    return ProjLogsoftmaxGatherFunc.apply(hidden, weight, targets, output_length, target_length, n_rows)


def proj_logsoftmax_gather(hidden, weight, targets=None, output_length=None, target_length=None, want_max=False,
                           want_lse=False):
    """See ``_Kernel.proj_logsoftmax_gather`` (not differentiable; ``proj_logsoftmax_gather_with_grad`` is)."""
    return get_pcfg_kernel().proj_logsoftmax_gather(hidden, weight, targets, output_length, target_length, want_max,
                                                    want_lse)


def viterbi_decoding(pred_length, output_length, L_trace, R_trace, M_trace, unreduced_tokens, left_tree_mask, pad_index):
    return get_pcfg_kernel().viterbi_decoding(pred_length, output_length, L_trace, R_trace, M_trace, unreduced_tokens,
                                              left_tree_mask, pad_index)
