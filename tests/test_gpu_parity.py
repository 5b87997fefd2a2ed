"""GPU parity tests: the CUDA kernels, called through the C ABI (ctypes -> libpcfgnat.so), against
the CPU oracle on the same seeded inputs, against the golden outputs of the reference kernels and,
when the reference build is present next to the oracle, against the reference kernels live.

Tolerances (from the parity contract): loss 1e-4 relative, gradients 1e-3 relative, Viterbi and
best-tree indices bit-exact including tie-breaks.  The inside table is additionally required to be
bit-identical to the reference kernel's table (GPU vs GPU), because best-tree compares sums of it.
"""
import os

import numpy as np
import pytest
import torch

import oracle
import _pyref as pyref
from conftest import golden_path

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(params=["auto", "cluster", "balanced", "rows"])
def dp_kernel(request, monkeypatch):
    """Runs a test once per selection of inside/outside kernels (PCFGNAT_DP_KERNEL): the library's own
    choice by shape, warp-per-node clusters, phase-balanced single CTA, and 4 lanes per node (the only
    one without a size limit)."""
    if request.param == "auto":
        monkeypatch.delenv("PCFGNAT_DP_KERNEL", raising=False)
    else:
        monkeypatch.setenv("PCFGNAT_DP_KERNEL", request.param)
    return request.param


@pytest.fixture(params=["auto", "rows", "cluster1", "cluster4"])
def vit_kernel(request, monkeypatch):
    """Runs a Viterbi test once per kernel: the library's own choice of cluster size, the single-CTA kernel
    that reads links from global memory, and fixed clusters of 1 and 4 CTAs per sentence."""
    monkeypatch.delenv("PCFGNAT_DP_KERNEL", raising=False)
    monkeypatch.delenv("PCFGNAT_DP_CLUSTER_SIZE", raising=False)
    if request.param == "rows":
        monkeypatch.setenv("PCFGNAT_DP_KERNEL", "rows")
    elif request.param.startswith("cluster"):
        monkeypatch.setenv("PCFGNAT_DP_CLUSTER_SIZE", request.param[len("cluster"):])
    return request.param


def _g(name):
    p = golden_path(name)
    if not os.path.isfile(p):
        pytest.skip(f"{name} not recorded yet")
    return np.load(p)


def _cu(x, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(x)).to(DEV)
    return t if dtype is None else t.to(dtype)


def _bits(x):
    return np.ascontiguousarray(x).view(np.int32)


def _loss_inputs(syn, w, seed):
    b = syn.make_batch(w, seed=seed)
    return b, syn.reference_match_all(b)


def _rel_close(a, b, rtol, atol=0.0):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert np.array_equal(np.isfinite(a), np.isfinite(b))
    fin = np.isfinite(a)
    err = np.abs(a[fin] - b[fin])
    assert (err <= atol + rtol * np.abs(b[fin])).all(), float(err.max())


CASES = [
    ("tiny", dict(batch=2, vocab=100, hidden=8, fixed_graph=32, fixed_target=10), 0),
    ("ragged", dict(batch=7, vocab=100, hidden=8, src_min=2, src_max=21), 1),
    ("mid", dict(batch=4, vocab=100, hidden=8, src_min=30, src_max=40), 2),
    ("wide", dict(batch=2, vocab=100, hidden=8, fixed_graph=256, fixed_target=40), 3),
    ("global_links", dict(batch=2, vocab=100, hidden=8, fixed_graph=400, fixed_target=30), 4),
]


@pytest.mark.parametrize("name,kw,seed", CASES)
def test_loss_forward_against_oracle(dp_kernel, monkeypatch, ops, syn, name, kw, seed):
    b, ma = _loss_inputs(syn, syn.Workload(name, emissions="logits", **kw), seed)
    k = ops.get_pcfg_kernel()
    S, C = k.pcfg_loss(ma.to(DEV), b.links.to(DEV), b.output_length.to(DEV), b.target_length.to(DEV), 1)
    So, Co = oracle.pcfg_loss(ma.numpy(), b.links.numpy(), b.output_length.numpy(), b.target_length.numpy())
    _rel_close(S.cpu().numpy(), So, 1e-5, 1e-5)
    assert np.array_equal(_bits(C.cpu().numpy()), _bits(Co))
    _rel_close(S[:, 0, 0].cpu().numpy(), So[:, 0, 0], 1e-4)
    # the fused forward + backward keeps its table to itself, so by default it builds it in free summation
    # order (loss equal to a few ulp); with a kernel family forced, or PCFGNAT_EXACT_ORDER=1, bit for bit
    loss = ops.cuda_pcfg_loss(ma.to(DEV), b.links.to(DEV), b.output_length.to(DEV), b.target_length.to(DEV))
    if dp_kernel == "auto":
        _rel_close(loss.cpu().numpy(), S[:, 0, 0].cpu().numpy(), 1e-5)
        monkeypatch.setenv("PCFGNAT_EXACT_ORDER", "1")
        loss = ops.cuda_pcfg_loss(ma.to(DEV), b.links.to(DEV), b.output_length.to(DEV), b.target_length.to(DEV))
    assert np.array_equal(_bits(loss.cpu().numpy()), _bits(S[:, 0, 0].cpu().numpy()))


@pytest.mark.parametrize("name,kw,seed", CASES)
def test_loss_backward_against_oracle(dp_kernel, ops, syn, name, kw, seed):
    b, ma = _loss_inputs(syn, syn.Workload(name, emissions="logits", **kw), seed)
    ol, tl = b.output_length.numpy(), b.target_length.numpy()
    So, Co = oracle.pcfg_loss(ma.numpy(), b.links.numpy(), ol, tl)
    go = np.linspace(0.5, 2.0, b.B).astype(np.float32)
    mgo, lgo = oracle.pcfg_loss_backward(go, So, Co, ma.numpy(), b.links.numpy(), ol, tl)
    k = ops.get_pcfg_kernel()
    S, C = k.pcfg_loss(ma.to(DEV), b.links.to(DEV), b.output_length.to(DEV), b.target_length.to(DEV), 1)
    mg, lg = k.pcfg_loss_backward(_cu(go), S, C, ma.to(DEV), b.links.to(DEV), b.output_length.to(DEV),
                                  b.target_length.to(DEV), 1)
    np.testing.assert_allclose(mg.cpu().numpy(), mgo, rtol=1e-3, atol=2e-6)
    np.testing.assert_allclose(lg.cpu().numpy(), lgo, rtol=1e-3, atol=2e-6)
    # fused entry point and the autograd wrapper give the same gradients (scaled by grad_output)
    mat = ma.to(DEV).requires_grad_(True)
    lkt = b.links.to(DEV).requires_grad_(True)
    loss = ops.cuda_pcfg_loss(mat, lkt, b.output_length.to(DEV), b.target_length.to(DEV))
    fin = torch.isfinite(loss)
    (loss[fin] * _cu(go)[fin]).sum().backward()
    fin_np = fin.cpu().numpy()
    np.testing.assert_allclose(mat.grad.cpu().numpy()[fin_np], mgo[fin_np], rtol=1e-3, atol=2e-6)
    np.testing.assert_allclose(lkt.grad.cpu().numpy()[fin_np], lgo[fin_np], rtol=1e-3, atol=2e-6)


@pytest.fixture(params=["staged", "global"])
def tree_walk(request, monkeypatch):
    """Both best-tree kernels: the walk over a copy of its inputs in shared memory (default where it fits) and the
    walk over global memory (PCFGNAT_TREE_STAGED=0, and shapes too large for shared memory)."""
    if request.param == "global":
        monkeypatch.setenv("PCFGNAT_TREE_STAGED", "0")
    else:
        monkeypatch.delenv("PCFGNAT_TREE_STAGED", raising=False)
    return request.param


@pytest.mark.parametrize("name,kw,seed", CASES)
def test_best_tree_bit_exact_on_shared_tables(ops, syn, tree_walk, name, kw, seed):
    b, ma = _loss_inputs(syn, syn.Workload(name, emissions="logits", **kw), seed)
    ol, tl = b.output_length.numpy(), b.target_length.numpy()
    So, Co = oracle.pcfg_loss(ma.numpy(), b.links.numpy(), ol, tl)
    want = oracle.pcfg_best_tree(So, Co, ma.numpy(), b.links.numpy(), ol, tl)
    got = ops.get_pcfg_kernel().pcfg_best_tree(_cu(So), _cu(Co), ma.to(DEV), b.links.to(DEV), b.output_length.to(DEV),
                                               b.target_length.to(DEV), 1)
    np.testing.assert_array_equal(got.cpu().numpy(), want)


def test_best_tree_tie_breaking(ops, tree_walk):
    # all transitions and emissions equal: every arg-max is a tie, so the result is decided by the
    # reference's lane order (0, 2, 1, 3), then smallest right child, then "no left child" first
    B, L, T = 1, 40, 9
    ma = np.zeros((B, L, T), np.float32)
    ma[0, :, T - 1] = -np.inf
    ma[0, L - 1, T - 1] = 0.0
    lk = np.full((B, L, 2, L), -np.inf, np.float32)
    for a in range(1, L - 1, 2):
        lk[0, a, 0, a + 2::2] = -1.0
        if a >= 3:
            lk[0, a, 1, a + 2::2] = -1.0
    ol, tl = np.array([L]), np.array([T])
    So, Co = oracle.pcfg_loss(ma, lk, ol, tl)
    So = np.where(np.isfinite(So), np.float32(-3.0), So)  # flatten the table: exact ties everywhere
    want = oracle.pcfg_best_tree(So, Co, ma, lk, ol, tl)
    got = ops.get_pcfg_kernel().pcfg_best_tree(_cu(So), None, _cu(ma), _cu(lk), _cu(ol), _cu(tl), 1)
    np.testing.assert_array_equal(got.cpu().numpy(), want)
    assert (want >= 0).sum() >= 2


@pytest.mark.parametrize("name", ["ref_loss_tiny.npz", "ref_loss_ragged.npz", "ref_loss_mid.npz"])
def test_loss_against_reference_golden(dp_kernel, ops, name):
    g = _g(name)
    k = ops.get_pcfg_kernel()
    ma, lk, ol, tl = _cu(g["match_all"]), _cu(g["links"]), _cu(g["output_length"]), _cu(g["target_length"])
    S, C = k.pcfg_loss(ma, lk, ol, tl, 1)
    assert np.array_equal(_bits(S.cpu().numpy()), _bits(g["S"]))  # bit-identical to the reference kernel
    assert np.array_equal(_bits(C.cpu().numpy()), _bits(g["C"]))
    mg, lg = k.pcfg_loss_backward(torch.ones(len(ol), device=DEV), S, C, ma, lk, ol, tl, 1)
    np.testing.assert_allclose(mg.cpu().numpy(), g["match_all_grad"], rtol=1e-3, atol=2e-6)
    np.testing.assert_allclose(lg.cpu().numpy(), g["links_grad"], rtol=1e-3, atol=2e-6)
    tree, loss = ops.cuda_pcfg_best_tree(ma, lk, ol, tl)
    np.testing.assert_array_equal(tree.cpu().numpy(), g["tree"])
    assert np.array_equal(_bits(loss.cpu().numpy()), _bits(g["S"][:, 0, 0]))


VCASES = [
    ("v_ragged", dict(batch=6, vocab=80, hidden=8, src_min=2, src_max=20), 0),
    ("v_mid", dict(batch=3, vocab=80, hidden=8, src_min=40, src_max=60), 1),
    ("v_global_links", dict(batch=2, vocab=80, hidden=8, fixed_graph=400), 2),
    ("v_many", dict(batch=93, vocab=40, hidden=8, src_min=2, src_max=30), 3),  # mixed cluster widths by default
]


def _viterbi_inputs(syn, name, kw, seed):
    b = syn.make_batch(syn.Workload(name, emissions="logits", kind="viterbi", **kw), seed=seed)
    ob, tok = torch.log_softmax(b.logits, -1).max(-1)
    return b, ob.contiguous(), tok.contiguous()


@pytest.mark.parametrize("name,kw,seed", VCASES)
def test_viterbi_bit_exact_against_oracle(vit_kernel, ops, syn, name, kw, seed):
    b, ob, tok = _viterbi_inputs(syn, name, kw, seed)
    S, R, Lt, Mt = ops.get_pcfg_kernel().pcfg_viterbi(ob.to(DEV), b.links.to(DEV), b.output_length.to(DEV), 1)
    So, Ro, Lo, Mo = oracle.pcfg_viterbi(ob.numpy(), b.links.numpy(), b.output_length.numpy())
    assert np.array_equal(_bits(S.cpu().numpy()), _bits(So))
    np.testing.assert_array_equal(R.cpu().numpy(), Ro)
    np.testing.assert_array_equal(Lt.cpu().numpy(), Lo)
    np.testing.assert_array_equal(Mt.cpu().numpy(), Mo)
    scores, R2, L2, M2 = ops.cuda_pcfg_viterbi(ob.to(DEV), b.links.to(DEV), b.output_length.to(DEV))
    assert np.array_equal(_bits(scores.cpu().numpy()), _bits(So[:, 1, :]))
    # length-penalised arg-max as the model does it, then the back-trace on the device
    sc = scores / torch.arange(b.L // 4, device=DEV).unsqueeze(0)
    sc.masked_fill_(sc.isnan(), float("-inf"))
    pred = sc[:, 1:].max(-1)[1] + 1
    mask = b.left_tree_mask.long()
    want = oracle.viterbi_decoding(pred.cpu().numpy(), b.output_length.numpy(), Lo, Ro, Mo, tok.numpy(), mask.numpy(), 1)
    got = ops.viterbi_decoding(pred, b.output_length.to(DEV), L2, R2, M2, tok.to(DEV), mask.to(DEV), 1)
    # the same in one launch: length choice fused into the back-trace
    pen = torch.arange(b.L // 4, device=DEV).float()
    f_tok, f_cnt, f_pred = ops.get_pcfg_kernel().viterbi_decode_device(S, pen, b.output_length.to(DEV), L2, R2, M2,
                                                                       tok.to(DEV), mask.to(DEV), 1)
    assert torch.equal(f_pred, pred)
    width = want.shape[1]
    np.testing.assert_array_equal(f_tok[:, :width].cpu().numpy(), want.astype(np.int64))
    assert (f_tok[:, width:] == 1).all() and int(f_cnt.max()) == width
    assert got.dtype == torch.float32 and got.is_cuda
    np.testing.assert_array_equal(got.cpu().numpy(), want)
    # the reference call pattern: traces moved to the host first
    got_cpu = ops.viterbi_decoding(pred.cpu(), b.output_length, L2.cpu(), R2.cpu(), M2.cpu(), tok, mask, 1)
    assert not got_cpu.is_cuda
    np.testing.assert_array_equal(got_cpu.numpy(), want)


def test_viterbi_tie_breaking(vit_kernel, ops, syn):
    # emissions and transitions from a handful of exactly representable values: many candidates of a
    # node tie, so the backpointers are decided by the reference's scan and merge order alone
    b = syn.make_batch(syn.Workload("v_ties", emissions="logits", kind="viterbi", batch=4, vocab=80, hidden=8,
                                    src_min=10, src_max=45), seed=5)
    g = torch.Generator().manual_seed(7)
    ob = -torch.randint(1, 4, (b.B, b.L), generator=g).float() * 0.5
    finite = torch.isfinite(b.links)
    links = torch.where(finite, -torch.randint(1, 3, b.links.shape, generator=g).float() * 0.25, b.links)
    S, R, Lt, Mt = ops.get_pcfg_kernel().pcfg_viterbi(ob.to(DEV), links.to(DEV), b.output_length.to(DEV), 1)
    So, Ro, Lo, Mo = oracle.pcfg_viterbi(ob.numpy(), links.numpy(), b.output_length.numpy())
    assert np.array_equal(_bits(S.cpu().numpy()), _bits(So))
    np.testing.assert_array_equal(R.cpu().numpy(), Ro)
    np.testing.assert_array_equal(Lt.cpu().numpy(), Lo)
    np.testing.assert_array_equal(Mt.cpu().numpy(), Mo)
    assert (np.isfinite(So).sum() > 100)


@pytest.mark.parametrize("name", ["ref_viterbi_ragged.npz", "ref_viterbi_mid.npz"])
def test_viterbi_against_reference_golden(vit_kernel, ops, name):
    g = _g(name)
    S, R, Lt, Mt = ops.get_pcfg_kernel().pcfg_viterbi(_cu(g["ob_lprob"]), _cu(g["links"]), _cu(g["output_length"]), 1)
    assert np.array_equal(_bits(S.cpu().numpy()), _bits(g["S"]))
    np.testing.assert_array_equal(R.cpu().numpy(), g["R"])
    np.testing.assert_array_equal(Lt.cpu().numpy(), g["L"])
    np.testing.assert_array_equal(Mt.cpu().numpy(), g["M"])


def test_backtrace_against_reference_host_golden(ops):
    g = np.load(golden_path("host_viterbi_decoding.npz"))
    got = ops.viterbi_decoding(_cu(g["pred_length"]), _cu(g["output_length"]), _cu(g["L"]), _cu(g["R"]), _cu(g["M"]),
                               _cu(g["tokens"]), _cu(g["left_tree_mask"].astype(np.int64)), 1)
    np.testing.assert_array_equal(got.cpu().numpy().astype(np.int64), g["decoded"])


@pytest.fixture(params=["single", "pair"])
def proj_pair(request, monkeypatch):
    """Runs a projection test with one CTA per tile and with CTA pairs sharing every W tile (cta_group::2)."""
    monkeypatch.setenv("PCFGNAT_PROJ_PAIR", "1" if request.param == "pair" else "0")
    return request.param


@pytest.mark.parametrize("dtype,atol", [(torch.float32, 2e-5), (torch.float16, 2e-5)])
@pytest.mark.parametrize("V", [1000, 40000, 997])
def test_logsoftmax_gather_against_oracle(ops, dtype, atol, V):
    g = torch.Generator().manual_seed(V)
    B, L, slen = 2, 6, 11
    x = (torch.randn(B, L, V, generator=g) * 3).to(dtype)
    tgt = torch.randint(0, V, (B, slen), generator=g)
    sel_idx = tgt[:, None, :].expand(-1, L, -1)  # stride-0 expand, as the criterion passes it
    want, probs = oracle.logsoftmax_gather(x.float().numpy(), sel_idx.numpy(), True)
    k = ops.get_pcfg_kernel()
    xc = x.to(DEV).clone()
    got = k.logsoftmax_gather(xc, sel_idx.to(DEV), False)
    np.testing.assert_allclose(got.cpu().numpy(), want, atol=atol + 1e-4)
    assert torch.equal(xc.cpu(), x)  # untouched without require_gradient
    got2 = k.logsoftmax_gather(xc, sel_idx.to(DEV), True)
    np.testing.assert_allclose(got2.cpu().numpy(), want, atol=atol + 1e-4)
    np.testing.assert_allclose(xc.float().cpu().numpy(), probs, atol=1e-6 if dtype == torch.float32 else 1e-3,
                               rtol=1e-4 if dtype == torch.float32 else 2e-3)


@pytest.mark.parametrize("stream", ["1", "0"])
@pytest.mark.parametrize("dtype,V", [(torch.float16, 40000), (torch.float32, 8000), (torch.float32, 40000), (torch.float16, 1000)])
def test_logsoftmax_gather_several_rows_per_cta(ops, monkeypatch, stream, dtype, V):
    """More rows than CTAs: the streaming kernel refills a row's chunks with the next row's bytes while it still works
    on the row (both phases of every chunk barrier come into use); rows of one full chunk and a part, of several
    chunks, and of less than a chunk; PCFGNAT_LSG_STREAM=0 runs the single-buffer kernel instead."""
    monkeypatch.setenv("PCFGNAT_LSG_STREAM", stream)
    g = torch.Generator().manual_seed(V + 1)
    B, L, slen = 3, 250, 7
    x = (torch.randn(B, L, V, generator=g) * 3).to(dtype)
    tgt = torch.randint(0, V, (B, slen), generator=g)
    sel_idx = tgt[:, None, :].expand(-1, L, -1)
    want, probs = oracle.logsoftmax_gather(x.float().numpy(), sel_idx.numpy(), True)
    k = ops.get_pcfg_kernel()
    xc = x.to(DEV).clone()
    got = k.logsoftmax_gather(xc, sel_idx.to(DEV), False)
    np.testing.assert_allclose(got.cpu().numpy(), want, atol=1.2e-4)
    assert torch.equal(xc.cpu(), x)
    got2 = k.logsoftmax_gather(xc, sel_idx.to(DEV), True)
    np.testing.assert_allclose(got2.cpu().numpy(), want, atol=1.2e-4)
    np.testing.assert_allclose(xc.float().cpu().numpy(), probs, atol=1e-6 if dtype == torch.float32 else 1e-3,
                               rtol=1e-4 if dtype == torch.float32 else 2e-3)
    assert ops.read_status(DEV) == 0


def test_logsoftmax_gather_more_selected_columns_than_threads(ops):
    """More gathered columns per row than the streaming kernel has threads: its late gather loop, with and without
    the softmax kept; an index out of range gives NaN and the status bit in both."""
    g = torch.Generator().manual_seed(5)
    B, L, V, slen = 2, 200, 2000, 700
    x = (torch.randn(B, L, V, generator=g) * 2).half()
    tgt = torch.randint(0, V, (B, slen), generator=g)
    sel_idx = tgt[:, None, :].expand(-1, L, -1)
    want, _ = oracle.logsoftmax_gather(x.float().numpy(), sel_idx.numpy(), True)
    k = ops.get_pcfg_kernel()
    for keep in (False, True):
        got = k.logsoftmax_gather(x.to(DEV).clone(), sel_idx.to(DEV), keep)
        np.testing.assert_allclose(got.cpu().numpy(), want, atol=1.2e-4)
    assert ops.read_status(DEV) == 0
    for n_sel in (700, 9):  # the late and the early gather
        bad = tgt[:, :n_sel].clone()
        bad[1, 3] = V
        got = k.logsoftmax_gather(x.to(DEV).clone(), bad[:, None, :].expand(-1, L, -1).to(DEV), False)
        assert torch.isnan(got[1, :, 3]).all() and torch.isfinite(got[0]).all()
        assert ops.read_status(DEV) & 4  # PCFGNAT_STATUS_BAD_INDEX


def test_logsoftmax_gather_reference_golden_and_autograd(ops):
    g = _g("ref_logsoftmax_gather.npz")
    k = ops.get_pcfg_kernel()
    sel_idx = _cu(g["targets"])[:, None, :].expand(-1, 8, -1)
    for tag, dt in (("f32", torch.float32), ("f16", torch.float16)):
        x = _cu(g["logits"]).to(dt).contiguous()
        got = k.logsoftmax_gather(x, sel_idx, True)
        np.testing.assert_allclose(got.cpu().numpy(), g[f"selected_{tag}_1"], atol=1e-4)
        np.testing.assert_allclose(x.float().cpu().numpy(), g[f"probs_{tag}"], atol=1e-3 if dt == torch.float16 else 1e-6,
                                   rtol=1e-3)
    # autograd through the in-place function equals autograd through log_softmax + gather
    x0 = _cu(g["logits"])
    w = torch.randn(2, 8, 10, device=DEV, generator=torch.Generator(DEV).manual_seed(0))
    xa = x0.clone().requires_grad_(True)
    (torch.log_softmax(xa, -1).gather(2, sel_idx) * w).sum().backward()
    xb = x0.clone().requires_grad_(True)
    _, sel = ops.dag_logsoftmax_gather_inplace(xb * 1.0, sel_idx)
    (sel * w).sum().backward()
    np.testing.assert_allclose(xb.grad.cpu().numpy(), xa.grad.cpu().numpy(), atol=1e-5)


def test_fused_loss_many_sentences_mixed_cluster_widths(ops, syn, monkeypatch):
    """More sentences than half the SMs: the fused forward + backward runs its passes as cost-ordered clusters
    of two, which the costliest sentences have to themselves and the others share, one CTA each.  Loss and gradients against the oracle, with an
    invalid sentence and wildly different lengths in the batch."""
    monkeypatch.delenv("PCFGNAT_DP_KERNEL", raising=False)
    monkeypatch.delenv("PCFGNAT_DP_CLUSTER_SIZE", raising=False)
    monkeypatch.delenv("PCFGNAT_EXACT_ORDER", raising=False)
    b, ma = _loss_inputs(syn, syn.Workload("many", batch=97, vocab=40, hidden=8, src_min=2, src_max=24,
                                           emissions="logits"), 21)
    ol, tl = b.output_length.clone(), b.target_length.clone()
    tl[5] = 0  # invalid: skipped, -inf loss, zero gradients
    So, Co = oracle.pcfg_loss(ma.numpy(), b.links.numpy(), ol.numpy(), tl.numpy())
    go = np.ones(b.B, np.float32)
    mgo, lgo = oracle.pcfg_loss_backward(go, So, Co, ma.numpy(), b.links.numpy(), ol.numpy(), tl.numpy())
    ops.read_status(DEV)
    loss, mg, lg = ops.get_pcfg_kernel().pcfg_loss_fwd_bwd(ma.to(DEV), b.links.to(DEV), ol.to(DEV), tl.to(DEV))
    want = So[:, 0, 0].copy()
    want[5] = -np.inf
    _rel_close(loss.cpu().numpy(), want, 1e-4)
    ok = np.isfinite(want)
    np.testing.assert_allclose(mg.cpu().numpy()[ok], mgo[ok], rtol=1e-3, atol=2e-6)
    np.testing.assert_allclose(lg.cpu().numpy()[ok], lgo[ok], rtol=1e-3, atol=2e-6)
    assert float(mg[5].abs().sum()) == 0.0 and float(lg[5].abs().sum()) == 0.0
    assert ops.read_status(DEV) & 1  # PCFGNAT_STATUS_BAD_LENGTH
    # the table-returning operator takes the same mixed widths with the reference's summation order: bit for bit
    # the table of the 4-lanes-per-node kernel (itself pinned against the reference kernels elsewhere)
    k = ops.get_pcfg_kernel()
    S_mixed, _ = k.pcfg_loss(ma.to(DEV), b.links.to(DEV), ol.to(DEV), tl.to(DEV), 1)
    monkeypatch.setenv("PCFGNAT_DP_KERNEL", "rows")
    S_rows, _ = k.pcfg_loss(ma.to(DEV), b.links.to(DEV), ol.to(DEV), tl.to(DEV), 1)
    assert np.array_equal(_bits(S_mixed.cpu().numpy()), _bits(S_rows.cpu().numpy()))
    ops.read_status(DEV)


@pytest.mark.parametrize("batch", [24, 90])
def test_fused_loss_model_graph_size(ops, syn, monkeypatch, batch):
    """Graphs of 8 * source + 2 nodes, the size the reference model builds at left_tree_layer 1
    (models/glat_decomposed_with_link_two_hands_tri_pcfg.py:322), on the sentence lengths of the training batch:
    up to 161 main-chain nodes per sentence.  Loss and gradients against the oracle, Viterbi tables bit for bit.
    With 90 sentences a chain needs two CTAs and the grid is larger than the GPU: the clusters take the sentences
    by decreasing cost; the inside table in the reference's order must not notice (bit for bit the table of the
    kernel that takes them in batch order)."""
    monkeypatch.delenv("PCFGNAT_DP_KERNEL", raising=False)
    monkeypatch.delenv("PCFGNAT_DP_CLUSTER_SIZE", raising=False)
    monkeypatch.delenv("PCFGNAT_EXACT_ORDER", raising=False)
    w = syn.WORKLOADS["train_batch_model_graph"]
    b, ma = _loss_inputs(syn, syn.Workload("model_graph", batch=batch, vocab=40, hidden=8, src_min=w.src_min,
                                           src_max=w.src_max, upsample=w.upsample, graph_offset=w.graph_offset,
                                           emissions="logits"), 33)
    assert int(b.output_length.max()) > 256 and (b.output_length % 8 == 2).all()
    ol, tl = b.output_length, b.target_length
    So, Co = oracle.pcfg_loss(ma.numpy(), b.links.numpy(), ol.numpy(), tl.numpy())
    go = np.ones(b.B, np.float32)
    mgo, lgo = oracle.pcfg_loss_backward(go, So, Co, ma.numpy(), b.links.numpy(), ol.numpy(), tl.numpy())
    ops.read_status(DEV)
    k = ops.get_pcfg_kernel()
    loss, mg, lg = k.pcfg_loss_fwd_bwd(ma.to(DEV), b.links.to(DEV), ol.to(DEV), tl.to(DEV))
    _rel_close(loss.cpu().numpy(), So[:, 0, 0], 1e-4)
    np.testing.assert_allclose(mg.cpu().numpy(), mgo, rtol=1e-3, atol=2e-6)
    np.testing.assert_allclose(lg.cpu().numpy(), lgo, rtol=1e-3, atol=2e-6)
    g = torch.Generator().manual_seed(5)
    ob = torch.log_softmax(torch.randn(b.B, b.L, 50, generator=g), -1).max(-1).values.contiguous()
    So2, Ro, Lo, Mo = oracle.pcfg_viterbi(ob.numpy(), b.links.numpy(), ol.numpy())
    S2, R2, L2, M2 = k.pcfg_viterbi(ob.to(DEV), b.links.to(DEV), ol.to(DEV), 1)
    assert np.array_equal(_bits(S2.cpu().numpy()), _bits(So2))
    np.testing.assert_array_equal(R2.cpu().numpy(), Ro)
    np.testing.assert_array_equal(L2.cpu().numpy(), Lo)
    np.testing.assert_array_equal(M2.cpu().numpy(), Mo)
    S_ranked, _ = k.pcfg_loss(ma.to(DEV), b.links.to(DEV), ol.to(DEV), tl.to(DEV), 1)
    monkeypatch.setenv("PCFGNAT_DP_KERNEL", "rows")
    S_rows, _ = k.pcfg_loss(ma.to(DEV), b.links.to(DEV), ol.to(DEV), tl.to(DEV), 1)
    assert np.array_equal(_bits(S_ranked.cpu().numpy()), _bits(S_rows.cpu().numpy()))
    assert ops.read_status(DEV) == 0


@pytest.mark.parametrize("batch", [97, 6])  # one CTA per sentence; a cluster of CTAs per sentence
@pytest.mark.parametrize("L_even", [True, False])
def test_outside_pass_with_fused_gradients_matches_the_gradient_kernel(ops, syn, monkeypatch, L_even, batch):
    """Fused forward + backward: the outside kernel (single-CTA or cluster family, by batch size) that also sums up
    both gradients (emission gradients from the shares the inside pass leaves in match_all_grad) against the
    outside kernel followed by the gradient kernel (PCFGNAT_FUSED_GRAD=0): both gradients to rounding, and both
    against the oracle.  The batch has odd graph lengths, a
    one-token target, an invalid sentence, and the outputs are handed over filled with garbage."""
    monkeypatch.delenv("PCFGNAT_DP_KERNEL", raising=False)
    monkeypatch.delenv("PCFGNAT_DP_CLUSTER_SIZE", raising=False)
    monkeypatch.delenv("PCFGNAT_EXACT_ORDER", raising=False)
    monkeypatch.setenv("PCFGNAT_LINEAR_DP", "0")  # this test is about the log-space kernels behind the fused entry
    b, ma = _loss_inputs(syn, syn.Workload("fg", batch=batch, vocab=40, hidden=8, src_min=3, src_max=20 if batch > 6 else 60,
                                           emissions="logits"), 77)
    links = b.links
    if not L_even:  # an odd padded width: the zero fill cannot use 16-byte stores
        ma = torch.nn.functional.pad(ma, (0, 0, 0, 1), value=0.0).contiguous()
        links = torch.nn.functional.pad(links, (0, 1, 0, 0, 0, 1), value=float("-inf")).contiguous()
    ol, tl = b.output_length.clone(), b.target_length.clone()
    ol[1] -= 1  # odd number of nodes: the last token is emitted by an even node
    tl[2] = 1   # one target token
    tl[3] = 0   # invalid
    k = ops.get_pcfg_kernel()
    ops.read_status(DEV)
    outs = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("PCFGNAT_FUSED_GRAD", mode)
        # whatever the allocator hands out next is dirty
        torch.empty(64 << 20, dtype=torch.uint8, device=DEV).fill_(0x7f)
        loss, mg, lg = k.pcfg_loss_fwd_bwd(ma.to(DEV), links.to(DEV), ol.to(DEV), tl.to(DEV))
        outs[mode] = (mg.cpu().numpy(), lg.cpu().numpy(), loss.cpu().numpy())
    assert ops.read_status(DEV) & 1  # PCFGNAT_STATUS_BAD_LENGTH for sentence 3
    # the inside pass that also emits the shares adds its two kinds of terms up separately: last-bit differences
    _rel_close(outs["1"][2], outs["0"][2], 1e-6)
    np.testing.assert_allclose(outs["1"][1], outs["0"][1], rtol=1e-4, atol=1e-7)
    np.testing.assert_allclose(outs["1"][0], outs["0"][0], rtol=1e-4, atol=1e-9)  # no absolute slack
    assert not np.array_equal(outs["1"][0], outs["0"][0])  # the switch chose another kernel
    So, Co = oracle.pcfg_loss(ma.numpy(), links.numpy(), ol.numpy(), tl.numpy())
    go = np.ones(b.B, np.float32)
    mgo, lgo = oracle.pcfg_loss_backward(go, So, Co, ma.numpy(), links.numpy(), ol.numpy(), tl.numpy())
    finite = np.isfinite(So[:, 0, 0])
    finite[3] = False
    np.testing.assert_allclose(outs["1"][0][finite], mgo[finite], rtol=1e-3, atol=2e-6)
    np.testing.assert_allclose(outs["1"][1][finite], lgo[finite], rtol=1e-3, atol=2e-6)
    assert not outs["1"][0][3].any() and not outs["1"][1][3].any()
    infeasible = ~np.isfinite(outs["1"][2])
    assert not outs["1"][0][infeasible].any() and not outs["1"][1][infeasible].any()


def test_invalid_sentences_are_skipped_not_faulted(dp_kernel, ops, syn):
    b, ma = _loss_inputs(syn, syn.Workload("bad", batch=4, vocab=50, hidden=8, src_min=4, src_max=6,
                                           emissions="logits"), 9)
    ol = b.output_length.clone()
    tl = b.target_length.clone()
    ol[1] = b.L + 5  # more nodes than the graph holds
    tl[2] = 0  # empty target
    ops.read_status(DEV)
    mat, lkt = ma.to(DEV).requires_grad_(True), b.links.to(DEV).requires_grad_(True)
    loss = ops.cuda_pcfg_loss(mat, lkt, ol.to(DEV), tl.to(DEV))
    assert torch.isinf(loss[1]) and torch.isinf(loss[2]) and torch.isfinite(loss[0]) and torch.isfinite(loss[3])
    loss[[0, 3]].sum().backward()
    assert float(mat.grad[1].abs().sum()) == 0.0 and float(lkt.grad[2].abs().sum()) == 0.0
    tree, _ = ops.cuda_pcfg_best_tree(ma.to(DEV), b.links.to(DEV), ol.to(DEV), tl.to(DEV))
    assert (tree[1] == -1).all() and (tree[2] == -1).all()
    assert ops.read_status(DEV) & 1  # PCFGNAT_STATUS_BAD_LENGTH
    # odd graph length: node m-1 is a leaf; the oracle restates what the reference does with it
    ol2 = b.output_length.clone()
    ol2[0] -= 1
    ol2[3] -= 1
    lp = torch.log_softmax(b.logits, -1)
    ma2 = lp.gather(2, b.targets[:, None, :].expand(-1, b.L, -1)).contiguous()
    syn.eos_mask_(ma2, ol2, b.target_length)
    S, C = ops.get_pcfg_kernel().pcfg_loss(ma2.to(DEV), b.links.to(DEV), ol2.to(DEV), b.target_length.to(DEV), 1)
    So, Co = oracle.pcfg_loss(ma2.numpy(), b.links.numpy(), ol2.numpy(), b.target_length.numpy())
    _rel_close(S.cpu().numpy(), So, 1e-5, 1e-5)
    mg, lg = ops.get_pcfg_kernel().pcfg_loss_backward(torch.ones(4, device=DEV), S, C, ma2.to(DEV), b.links.to(DEV),
                                                      ol2.to(DEV), b.target_length.to(DEV), 1)
    mgo, lgo = oracle.pcfg_loss_backward(np.ones(4, np.float32), So, Co, ma2.numpy(), b.links.numpy(), ol2.numpy(),
                                         b.target_length.numpy())
    np.testing.assert_allclose(mg.cpu().numpy(), mgo, rtol=1e-3, atol=2e-6)
    np.testing.assert_allclose(lg.cpu().numpy(), lgo, rtol=1e-3, atol=2e-6)
    want = oracle.pcfg_best_tree(So, Co, ma2.numpy(), b.links.numpy(), ol2.numpy(), b.target_length.numpy())
    got = ops.get_pcfg_kernel().pcfg_best_tree(_cu(So), None, ma2.to(DEV), b.links.to(DEV), ol2.to(DEV),
                                               b.target_length.to(DEV), 1)
    np.testing.assert_array_equal(got.cpu().numpy(), want)


def test_argument_errors(ops):
    k = ops.get_pcfg_kernel()
    ma = torch.zeros(1, 10, 3, device=DEV)
    with pytest.raises(RuntimeError, match="max_left"):
        k.pcfg_loss(ma, torch.zeros(1, 10, 4, 10, device=DEV), torch.tensor([10]), torch.tensor([3]), 1)
    with pytest.raises(RuntimeError, match="float32"):
        k.pcfg_loss(ma.double(), torch.zeros(1, 10, 2, 10, device=DEV), torch.tensor([10]), torch.tensor([3]), 1)
    with pytest.raises(RuntimeError, match="config should be 1~4"):
        k.pcfg_viterbi(torch.zeros(1, 16, device=DEV), torch.zeros(1, 16, 2, 16, device=DEV), torch.tensor([16]), 7)
    with pytest.raises(RuntimeError, match="select_idx should be long"):
        k.logsoftmax_gather(torch.zeros(1, 2, 5, device=DEV), torch.zeros(1, 2, 1, device=DEV, dtype=torch.int32), False)
    with pytest.raises(RuntimeError, match="not contiguous"):
        k.logsoftmax_gather(torch.zeros(1, 5, 2, device=DEV).transpose(1, 2), torch.zeros(1, 2, 1, device=DEV, dtype=torch.long), False)


# ---- full-size workloads: properties that need no oracle run ---------------------------------------------------

@pytest.mark.parametrize("wname", ["glance", "long_seq"])
def test_full_size_properties(dp_kernel, ops, syn, wname):
    w = syn.WORKLOADS[wname]
    b = syn.make_batch(syn.Workload(w.name, batch=w.batch, vocab=64, hidden=8, fixed_graph=w.fixed_graph,
                                    fixed_target=w.fixed_target, emissions="logits"), seed=0)
    ma = syn.reference_match_all(b).to(DEV).requires_grad_(True)
    lk = b.links.to(DEV).requires_grad_(True)
    ol, tl = b.output_length.to(DEV), b.target_length.to(DEV)
    loss = ops.cuda_pcfg_loss(ma, lk, ol, tl)
    assert torch.isfinite(loss).all()
    loss.sum().backward()
    n = int(b.target_length[0])
    # posterior marginals: each target position is emitted by exactly one node
    torch.testing.assert_close(ma.grad.sum(1)[:, :n], torch.ones(b.B, n, device=DEV), rtol=0, atol=2e-3)
    # expected number of binary rule uses = expected number of main-chain nodes used - 1
    used_main = ma.grad[:, 1::2, :].sum((1, 2))
    torch.testing.assert_close(lk.grad.sum((1, 2, 3)), used_main - 1, rtol=0, atol=5e-3)
    tree, loss2 = ops.cuda_pcfg_best_tree(ma.detach(), lk.detach(), ol, tl)
    if dp_kernel == "auto":  # free-order table inside the fused forward + backward
        torch.testing.assert_close(loss2, loss.detach(), rtol=1e-5, atol=0)
    else:
        assert torch.equal(loss2, loss.detach())
    t = tree.cpu().numpy()
    for i in range(b.B):
        used = t[i][t[i] >= 0]
        assert used.tolist() == list(range(n))
        assert t[i, 1] == 0 and t[i, int(b.output_length[i]) - 1] == n - 1


def test_full_size_viterbi_properties(ops, syn):
    b = syn.make_batch(syn.Workload("v64", batch=64, vocab=64, hidden=8, src_min=10, src_max=60, emissions="logits",
                                    kind="viterbi"), seed=0)
    ob, tok = torch.log_softmax(b.logits, -1).max(-1)
    tok = torch.arange(b.L)[None, :].expand(b.B, -1).contiguous() + 100
    scores, R, Lt, Mt = ops.cuda_pcfg_viterbi(ob.to(DEV), b.links.to(DEV), b.output_length.to(DEV))
    sc = scores / torch.arange(b.L // 4, device=DEV).unsqueeze(0)
    sc.masked_fill_(sc.isnan(), float("-inf"))
    pred = sc[:, 1:].max(-1)[1] + 1
    out = ops.viterbi_decoding(pred, b.output_length.to(DEV), Lt, R, Mt, tok.to(DEV), b.left_tree_mask.long().to(DEV), 1)
    out = out.cpu().numpy()
    for i in range(b.B):
        row = out[i][out[i] != 1]
        assert len(row) == int(pred[i]) and row[0] == 101 and row[-1] == 100 + int(b.output_length[i]) - 1
        assert (np.diff(row) > 0).all()


# ---- live comparison with the reference kernels (only where the reference build travelled along) ------------------

def _ref():
    from oracle.build_ref import load_ref, ref_so_path

    if not os.path.isfile(ref_so_path()):
        pytest.skip("reference extension not built")
    return load_ref()


@pytest.mark.parametrize("seed", [10, 11, 12])
def test_live_against_reference_kernels(dp_kernel, ops, syn, seed):
    ref = _ref()
    # graph length <= 256 keeps every reference launch at one row segment per sentence (no
    # dependence on co-resident blocks in its spin-waits)
    w = syn.Workload("live", batch=8, vocab=120, hidden=8, src_min=6, src_max=64, emissions="logits")
    b, ma = _loss_inputs(syn, w, seed)
    ma_d, lk_d = ma.to(DEV), b.links.to(DEV)
    ol, tl = b.output_length.to(DEV), b.target_length.to(DEV)
    k = ops.get_pcfg_kernel()
    Sr, Cr = ref.pcfg_loss(ma_d, lk_d, ol, tl, 1)
    S, C = k.pcfg_loss(ma_d, lk_d, ol, tl, 1)
    assert torch.equal(S.view(torch.int32), Sr.view(torch.int32))
    assert torch.equal(C.view(torch.int32), Cr.view(torch.int32))
    mgr, lgr = ref.pcfg_loss_backward(torch.ones(b.B, device=DEV), Sr, Cr, ma_d, lk_d, ol, tl, 1)
    mg, lg = k.pcfg_loss_backward(torch.ones(b.B, device=DEV), S, C, ma_d, lk_d, ol, tl, 1)
    torch.testing.assert_close(mg, mgr, rtol=1e-3, atol=2e-6)
    torch.testing.assert_close(lg, lgr, rtol=1e-3, atol=2e-6)
    assert torch.equal(k.pcfg_best_tree(S, C, ma_d, lk_d, ol, tl, 1), ref.pcfg_best_tree(Sr, Cr, ma_d, lk_d, ol, tl, 1))
    ob = torch.log_softmax(b.logits, -1).max(-1)[0].to(DEV)
    for x, y in zip(k.pcfg_viterbi(ob, lk_d, ol, 1), ref.pcfg_viterbi(ob, lk_d, ol, 1)):
        assert torch.equal(x.view(torch.int32) if x.dtype == torch.float32 else x,
                           y.view(torch.int32) if y.dtype == torch.float32 else y)


# ---- fused projection + log-softmax + gather / max (tensor cores) ------------------------------------------------

def _proj_reference(hidden, weight, targets):
    """fp32 torch reference on the GPU: same fp16 values, fp32 accumulation."""
    logits = hidden.float().reshape(-1, hidden.shape[-1]) @ weight.float().t()
    lse = torch.logsumexp(logits, -1)
    lp = logits - lse[:, None]
    mx, am = lp.max(-1)
    B, L = hidden.shape[:2]
    match = lp.view(B, L, -1).gather(2, targets[:, None, :].expand(-1, L, -1)) if targets is not None else None
    top2 = logits.topk(2, -1)[0]
    return match, mx.view(B, L), am.view(B, L), lse.view(B, L), (top2[:, 0] - top2[:, 1]).view(B, L)


PROJ_CASES = [
    # B, L, T, V, H, hidden_std
    (2, 32, 10, 1000, 64, 1.0),       # tiny: one partial row tile, vocabulary split over many CTAs
    (3, 100, 17, 5000, 128, 1.0),     # rows and vocabulary both ragged against the tile sizes
    (1, 240, 12, 40000, 512, 1.0),    # batch-1 decode shape
    (6, 160, 40, 40000, 512, 0.02),   # training-shaped slice
    (4, 256, 64, 40000, 512, 1.0),    # glancing-shaped slice
]


@pytest.mark.parametrize("B,L,T,V,H,std", PROJ_CASES)
def test_fused_projection_against_torch(proj_pair, ops, syn, B, L, T, V, H, std):
    g = torch.Generator().manual_seed(B * 1000 + L)
    hidden = (torch.randn(B, L, H, generator=g) * std).half().to(DEV)
    weight = (torch.randn(V, H, generator=g) * 0.02).half().to(DEV)
    targets = torch.randint(0, V, (B, T), generator=g).to(DEV)
    targets[:, 0] = V - 1  # last vocabulary column (inside the ragged last tile)
    targets[:, 1] = targets[:, 2]  # repeated target
    ops.read_status(DEV)
    out = ops.proj_logsoftmax_gather(hidden, weight, targets, want_max=True, want_lse=True)
    match, mx, am, lse, margin = _proj_reference(hidden, weight, targets)
    # fp16 inputs, fp32 accumulation on both sides: only summation order differs
    torch.testing.assert_close(out["lse"], lse, rtol=0, atol=2e-3)
    torch.testing.assert_close(out["match"], match, rtol=0, atol=2e-3)
    torch.testing.assert_close(out["max_lprob"], mx, rtol=0, atol=2e-3)
    clear = margin > 1e-3  # arg-max must agree wherever the top-2 margin exceeds the tolerance
    assert torch.equal(out["argmax"][clear], am[clear])
    if std >= 1.0:
        assert clear.float().mean() > 0.9
    assert ops.read_status(DEV) == 0
    # gather-only and max-only variants, EOS masking fused
    ol = torch.full((B,), L, device=DEV)
    tl = torch.full((B,), T, device=DEV)
    ol[0] = L - 2
    tl[0] = max(T - 3, 2)
    out2 = ops.proj_logsoftmax_gather(hidden, weight, targets, ol, tl, want_max=True)
    want = syn.eos_mask_(match.clone(), ol.cpu(), tl.cpu())
    real = (torch.arange(L, device=DEV)[None, :] < ol[:, None])  # with lengths only real nodes are projected
    want[~real] = 0.0
    fin = torch.isfinite(want)
    assert torch.equal(fin, torch.isfinite(out2["match"]))
    torch.testing.assert_close(out2["match"][fin], want[fin], rtol=0, atol=2e-3)
    assert float(out2["match"][~real].abs().sum()) == 0.0 and float(out2["max_lprob"][~real].abs().sum()) == 0.0
    torch.testing.assert_close(out2["max_lprob"][real], mx[real], rtol=0, atol=2e-3)
    out3 = ops.proj_logsoftmax_gather(hidden, weight, want_max=True)
    assert torch.equal(out3["argmax"], out["argmax"]) and torch.equal(out3["max_lprob"], out["max_lprob"])


@pytest.mark.parametrize("compact", [False, True])
@pytest.mark.parametrize("V,H,std", [(1000, 64, 1.0), (4104, 128, 0.3), (997, 64, 1.0)])
def test_fused_projection_backward_against_torch(proj_pair, ops, syn, V, H, std, compact):
    """Gradients of the fused projection (logits recomputed on the tensor cores, bf16 d-logits, two GEMMs)
    against float32 autograd of the same expression; with the d-logits of every padded row and (compact) of the
    real graph nodes only."""
    w = syn.Workload("pb", batch=5, vocab=V, hidden=H, src_min=8, src_max=40, hidden_std=std)
    b = syn.make_batch(w, seed=V)
    g = torch.Generator().manual_seed(1)
    gm = torch.randn(b.B, b.L, b.T, generator=g)
    gm[torch.rand(b.B, b.L, b.T, generator=g) < 0.5] = 0
    hid = b.hidden.to(DEV).requires_grad_(True)
    wt = b.weight.to(DEV).requires_grad_(True)
    ol, tl = b.output_length.to(DEV), b.target_length.to(DEV)
    match = ops.proj_logsoftmax_gather_with_grad(hid, wt, b.targets.to(DEV), ol, tl,
                                                 n_rows=int(b.output_length.sum()) if compact else None)
    fin = torch.isfinite(match)
    (match[fin] * gm.to(DEV)[fin]).sum().backward()
    # float32 reference of the same expression
    h32 = b.hidden.float().to(DEV).requires_grad_(True)
    w32 = b.weight.float().to(DEV).requires_grad_(True)
    lp = torch.log_softmax(h32 @ w32.t(), -1)
    ref = lp.gather(2, b.targets.to(DEV)[:, None, :].expand(-1, b.L, -1))
    rows = torch.arange(b.L, device=DEV)[None, :] < ol[:, None]
    syn.eos_mask_(ref, ol, tl)
    ref = torch.where(rows[:, :, None], ref, torch.zeros_like(ref))  # padding nodes are not projected: zeros
    assert torch.equal(torch.isfinite(ref), fin)
    torch.testing.assert_close(match[fin], ref[fin].detach(), rtol=2e-3, atol=2e-3)
    (ref[fin] * gm.to(DEV)[fin]).sum().backward()
    for got, want in ((hid.grad.float(), h32.grad), (wt.grad.float(), w32.grad)):
        err = (got - want).norm() / want.norm()
        assert float(err) < 1.5e-2, float(err)
        assert float((got - want).abs().max()) < 3e-2 * float(want.abs().max()) + 1e-3
    assert float(hid.grad[~rows].abs().sum()) == 0.0
    assert ops.read_status(DEV) == 0


def test_loss_step_with_projection_backward_matches_autograd_path(pkg, ops, syn):
    """LossStep(proj_backward=True): d hidden and d weight (compact d-logits in the graph, the two GEMMs after it)
    against the differentiable operator fed with the step's own emission gradient; two batches with different
    numbers of real nodes through the same step object."""
    import importlib
    runtime = importlib.import_module("pcfg_nat_b200.runtime")
    w = syn.Workload("pbs", batch=6, vocab=1000, hidden=64, src_min=6, src_max=30, hidden_std=1.0)
    batches = [syn.make_batch(w, seed=seed) for seed in (31, 32)]
    B, L, T = batches[0].B, max(b.L for b in batches), max(b.T for b in batches)
    weight = batches[0].weight.to(DEV)
    step = runtime.LossStep(weight, B, L, T, DEV, use_graph=True, proj_backward=True)
    assert int(batches[0].output_length.sum()) != int(batches[1].output_length.sum())
    for b in batches:
        hidden = torch.zeros(B, L, b.hidden.shape[2], dtype=b.hidden.dtype)
        hidden[:, :b.L] = b.hidden
        links = torch.full((B, L, 2, L), float("-inf"))
        links[:, :b.L, :, :b.L] = b.links
        targets = torch.ones(B, T, dtype=torch.int64)
        targets[:, :b.T] = b.targets
        step.load(hidden, links, b.output_length, targets, b.target_length)
        stats, mg, lg, loss, d_hidden, d_weight = step.run()
        torch.cuda.synchronize()
        assert torch.isfinite(loss).all()
        hid = hidden.to(DEV).requires_grad_(True)
        wt = weight.clone().requires_grad_(True)
        ol = b.output_length.to(DEV)
        match = ops.proj_logsoftmax_gather_with_grad(hid, wt, targets.to(DEV), ol, b.target_length.to(DEV))
        fin = torch.isfinite(match)
        (match[fin] * mg[fin]).sum().backward()
        for got, want in ((d_hidden.float(), hid.grad.float()), (d_weight.float(), wt.grad.float())):
            assert float((got - want).norm() / want.norm()) < 2e-3
        rows = torch.arange(L, device=DEV)[None, :] < ol[:, None]
        assert float(d_hidden[~rows].abs().sum()) == 0.0
    assert ops.read_status(DEV) == 0


@pytest.mark.parametrize("n,V,H", [(300, 1024, 64), (1000, 4104, 512), (129, 40000, 128), (70, 200, 8)])
def test_projection_backward_gemms_against_torch(ops, n, V, H):
    """pcfgnat_proj_backward_gemms (tcgen05, dlogits read K-major for one product and MN-major for the other)
    against float32 matmul of the same bf16 operands; shapes with row, column and K tails, one tile and many."""
    g = torch.Generator().manual_seed(n)
    dl = (torch.randn(n, V, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    w = torch.randn(V, H, generator=g).to(torch.bfloat16).to(DEV)
    rows = torch.randn(n, H, generator=g).to(torch.bfloat16).to(DEV)
    k = ops.get_pcfg_kernel()
    d_rows, d_weight = k.proj_backward_gemms(dl, w, rows)
    want_rows = dl.float() @ w.float()
    want_weight = dl.float().t() @ rows.float()
    torch.testing.assert_close(d_rows, want_rows, rtol=2e-3, atol=2e-3 * float(want_rows.abs().max()))
    torch.testing.assert_close(d_weight, want_weight, rtol=2e-3, atol=2e-3 * float(want_weight.abs().max()))
    only_rows, none = k.proj_backward_gemms(dl, w, None, want_weight=False)
    assert none is None
    torch.testing.assert_close(only_rows, d_rows, rtol=1e-5, atol=1e-5 * float(want_rows.abs().max()))
    assert ops.read_status(DEV) == 0


def test_projection_backward_gemms_with_no_rows(ops):
    """A batch without real nodes: d rows is empty and d weight exactly zero."""
    k = ops.get_pcfg_kernel()
    dl = torch.empty((0, 1024), dtype=torch.bfloat16, device=DEV)
    w = torch.ones((1024, 64), dtype=torch.bfloat16, device=DEV)
    rows = torch.empty((0, 64), dtype=torch.bfloat16, device=DEV)
    d_rows, d_weight = k.proj_backward_gemms(dl, w, rows)
    assert tuple(d_rows.shape) == (0, 64) and tuple(d_weight.shape) == (1024, 64)
    assert float(d_weight.abs().sum()) == 0.0
    with pytest.raises(RuntimeError, match="unsupported"):
        k.proj_backward_gemms(torch.zeros((8, 1001), dtype=torch.bfloat16, device=DEV),
                              torch.zeros((1001, 64), dtype=torch.bfloat16, device=DEV), None, want_weight=False)


def test_copy_real_rows_sends_the_real_nodes_only(ops):
    """pcfgnat_copy_real_rows: rows l < length arrive, the others keep what they held; lengths beyond the tensor
    and below zero are clamped; full sentences next to each other go as one copy; a sentence range."""
    k = ops.get_pcfg_kernel()
    g = torch.Generator().manual_seed(3)
    B, L, H = 7, 12, 40
    src = torch.randn(B, L, H, generator=g).half().pin_memory()
    lengths = torch.tensor([3, 12, 12, 0, 20, -4, 5])
    dst = torch.full((B, L, H), 7.0, dtype=torch.float16, device=DEV)
    assert k.copy_real_rows(dst, src, lengths) == 3 + 12 + 12 + 12 + 5
    torch.cuda.synchronize()
    m = lengths.clamp(0, L)
    for b in range(B):
        assert torch.equal(dst[b, :m[b]].cpu(), src[b, :m[b]])
        assert (dst[b, m[b]:] == 7).all()
    # at most 2 copies: runs are rows [0,3), [12,36), [48,60), [72,77); the gaps of 9 and 12 rows are closed first
    dst.fill_(7.0)
    sent = k.copy_real_rows(dst, src, lengths, max_copies=2)
    torch.cuda.synchronize()
    flat_d, flat_s = dst.view(B * L, H).cpu(), src.view(B * L, H)
    assert sent == 60 + 5 and torch.equal(flat_d[:60], flat_s[:60]) and torch.equal(flat_d[72:77], flat_s[72:77])
    assert (flat_d[60:72] == 7).all() and (flat_d[77:] == 7).all()
    dst.fill_(7.0)
    k.copy_real_rows(dst, src, lengths, 1, 3)
    torch.cuda.synchronize()
    assert torch.equal(dst[1:3].cpu(), src[1:3]) and (dst[0] == 7).all() and (dst[3:] == 7).all()
    with pytest.raises(RuntimeError, match="host"):
        k.copy_real_rows(dst, src, lengths.to(DEV))


def test_fused_projection_flags_bad_targets(ops):
    g = torch.Generator().manual_seed(0)
    hidden = torch.randn(1, 16, 64, generator=g).half().to(DEV)
    weight = torch.randn(300, 64, generator=g).half().to(DEV)
    targets = torch.tensor([[5, 300, 7, -1]], device=DEV)
    ops.read_status(DEV)
    out = ops.proj_logsoftmax_gather(hidden, weight, targets)
    m = out["match"]
    assert torch.isnan(m[0, :, 1]).all() and torch.isnan(m[0, :, 3]).all()
    assert torch.isfinite(m[0, :, 0]).all() and torch.isfinite(m[0, :, 2]).all()
    assert ops.read_status(DEV) & 4
    with pytest.raises(RuntimeError, match="multiple of 64"):
        ops.proj_logsoftmax_gather(hidden[:, :, :48].contiguous(), weight[:, :48].contiguous(), targets)


# ---- the fixed-shape step object (CUDA-graph replay) ---------------------------------------------------------------

def test_loss_step_graph_replay_matches_eager(pkg, ops, syn):
    import importlib

    runtime = importlib.import_module("pcfg_nat_b200.runtime")
    w = syn.Workload("step", batch=6, vocab=3000, hidden=128, src_min=5, src_max=20, hidden_std=1.0)
    b1, b2 = syn.make_batch(w, seed=1), syn.make_batch(w, seed=2)
    L, T = max(b1.L, b2.L), max(b1.T, b2.T)

    def padded(b):
        hid = torch.zeros(b.B, L, w.hidden, dtype=torch.float16)
        hid[:, :b.L] = b.hidden
        lk = torch.full((b.B, L, 2, L), float("-inf"))
        lk[:, :b.L, :, :b.L] = b.links
        tg = torch.ones(b.B, T, dtype=torch.long)
        tg[:, :b.T] = b.targets
        return hid, lk, b.output_length, tg, b.target_length  # LossStep.load order

    weight = b1.weight.to(DEV)
    eager = runtime.LossStep(weight, w.batch, L, T, DEV, use_graph=False)
    graphed = runtime.LossStep(weight, w.batch, L, T, DEV, use_graph=True)
    # the graphs are captured on the first batch and replayed on the others; the last two loads go over the
    # copy stream, transitions last, each stage waiting for its own inputs only
    for b, overlap in ((b1, False), (b2, False), (b1, True), (b2, True)):
        args = padded(b)
        eager.load(*args)
        graphed.load(*[t.pin_memory() for t in args], overlap=overlap)
        se, mge, lge, le = [t.clone() for t in eager.run()]
        sg, mgg, lgg, lg_ = graphed.run()
        torch.cuda.synchronize()
        assert torch.isfinite(le).all()
        assert torch.equal(lg_, le) and torch.equal(sg, se)
        assert torch.equal(mgg, mge) and torch.equal(lgg, lge)
        # and against the torch reference of the projection feeding the oracle
        hid, lk, ol, tg, tl = args
        lp = torch.log_softmax(hid.float() @ b1.weight.float().t(), -1)  # the step objects hold b1's projection matrix
        match = lp.gather(2, tg[:, None, :].expand(-1, L, -1)).contiguous()
        syn.eos_mask_(match, ol, tl)
        So, _ = oracle.pcfg_loss(match.numpy(), lk.numpy(), ol.numpy(), tl.numpy())
        np.testing.assert_allclose(le.cpu().numpy(), So[:, 0, 0], rtol=1e-4)
        want = -(torch.from_numpy(So[:, 0, 0]) / tl).sum()
        assert abs(float(-se[0]) - float(want)) < 1e-3 * abs(float(want)) and int(se[1]) == w.batch


def test_empty_and_minimal_inputs(ops, syn):
    k = ops.get_pcfg_kernel()
    L, T = 8, 3
    ma = torch.zeros(0, L, T, device=DEV)
    lk = torch.zeros(0, L, 2, L, device=DEV)
    n0 = torch.zeros(0, dtype=torch.long, device=DEV)
    # no sentences at all: every operator returns empty outputs without launching anything harmful
    S, C = k.pcfg_loss(ma, lk, n0, n0, 1)
    assert S.shape[0] == 0 and C.shape[0] == 0
    loss, mg, lg = k.pcfg_loss_fwd_bwd(ma, lk, n0, n0)
    assert loss.numel() == 0 and mg.shape == ma.shape and lg.shape == lk.shape
    assert k.pcfg_best_tree(S, None, ma, lk, n0, n0, 1).shape == (0, L)
    Sv, R, Lt, Mt = k.pcfg_viterbi(torch.zeros(0, L, device=DEV), lk, n0, 1)
    assert Sv.shape == (0, L, L // 4)
    tok, cnt = k.viterbi_decoding_device(n0, n0, Lt, R, Mt, torch.zeros(0, L, dtype=torch.long, device=DEV),
                                         torch.zeros(L, L, dtype=torch.long, device=DEV), 1)
    assert tok.shape == (0, L) and cnt.numel() == 0
    em = k.proj_logsoftmax_gather(torch.zeros(0, L, 64, dtype=torch.float16, device=DEV),
                                  torch.zeros(100, 64, dtype=torch.float16, device=DEV),
                                  torch.zeros(0, T, dtype=torch.long, device=DEV), n0, n0, want_max=True)
    assert em["match"].shape == (0, L, T) and em["argmax"].shape == (0, L)
    assert k.loss_stats(loss, n0).cpu().tolist() == [0.0, 0.0, 0.0]
    torch.cuda.synchronize()
    # the smallest sentence the grammar admits: two graph nodes... and the smallest table the decoder admits
    b = syn.make_batch(syn.Workload("min", batch=3, vocab=30, hidden=8, src_min=1, src_max=2, emissions="logits"),
                       seed=3)
    ma2 = syn.reference_match_all(b)
    S2, C2 = k.pcfg_loss(ma2.to(DEV), b.links.to(DEV), b.output_length.to(DEV), b.target_length.to(DEV), 1)
    So, Co = oracle.pcfg_loss(ma2.numpy(), b.links.numpy(), b.output_length.numpy(), b.target_length.numpy())
    _rel_close(S2.cpu().numpy(), So, 1e-5, 1e-5)
    tree = k.pcfg_best_tree(S2, None, ma2.to(DEV), b.links.to(DEV), b.output_length.to(DEV), b.target_length.to(DEV), 1)
    want = oracle.pcfg_best_tree(S2.cpu().numpy(), Co, ma2.numpy(), b.links.numpy(), b.output_length.numpy(),
                                 b.target_length.numpy())
    np.testing.assert_array_equal(tree.cpu().numpy(), want)
    assert ops.read_status(DEV) == 0


@pytest.mark.parametrize("L", [12, 9])
def test_copy_links_main_rows(ops, L):
    k = ops.get_pcfg_kernel()
    g = torch.Generator().manual_seed(L)
    src = torch.randn(3, L, 2, L, generator=g)
    for s_ in (src.pin_memory(), src.to(DEV)):
        dst = torch.full((3, L, 2, L), -7.0, device=DEV)
        k.copy_links_main_rows(dst, s_)
        torch.cuda.synchronize()
        assert torch.equal(dst[:, 1::2].cpu(), src[:, 1::2])  # main-chain nodes
        assert (dst[:, 0::2] == -7.0).all()  # rows no kernel reads keep their contents


def test_loss_stats_and_glance_select(ops):
    k = ops.get_pcfg_kernel()
    g = torch.Generator().manual_seed(11)
    loss = -torch.rand(37, generator=g) * 50
    loss[3], loss[20], loss[21] = float("-inf"), float("nan"), float("inf")
    tl = torch.randint(1, 40, (37,), generator=g)
    tl[5] = 0  # clamped to 1
    stats = k.loss_stats(loss.to(DEV), tl.to(DEV)).cpu()
    ok = torch.isfinite(loss)
    want = (loss[ok].double() / tl[ok].clamp(min=1).double()).sum()
    assert abs(float(stats[0]) - float(want)) < 1e-5 * abs(float(want))
    assert stats[1] == 37 and stats[2] == 3
    assert k.loss_stats(loss[:0].to(DEV), tl[:0].to(DEV)).cpu().tolist() == [0.0, 0.0, 0.0]

    for B, L, T, p, seed in ((5, 40, 12, 0.5, 0), (3, 300, 90, 0.3, 1), (2, 16, 5, 1.0, 2), (4, 24, 7, 0.0, 3)):
        g = torch.Generator().manual_seed(seed)
        tlen = torch.randint(2, T + 1, (B,), generator=g)
        path = torch.randint(-1, T + 2, (B, L), generator=g)  # also positions past the target (dropped from the mask)
        path[torch.rand(B, L, generator=g) < 0.4] = -1
        tgt = torch.randint(4, 50, (B, T), generator=g)
        pred = torch.randint(4, 50, (B, L), generator=g)
        pred = torch.where(torch.rand(B, L, generator=g) < 0.5, tgt.gather(-1, path.clip(0, T - 1)), pred)
        prev = torch.randint(1, 4, (B, L), generator=g)
        noise = torch.randn(B, L, generator=g)
        noise[0, : L // 2] = noise[0, 0]  # ties at the threshold
        got = k.glance_select(path.to(DEV), pred.to(DEV), tgt.to(DEV), prev.to(DEV), tlen.to(DEV), noise.to(DEV), p)
        want = pyref.glance_select(path, pred, tgt, prev, tlen, noise, p)
        for key, val in want.items():
            assert torch.equal(got[key].cpu(), val), (key, B, L, T)


@pytest.mark.parametrize("case", ["small", "mid"])
def test_extract_links_against_reference_model(ops, case):
    """links from the projected link features against the reference model's own extract_links (run on the CPU
    by tests/golden/make_golden_links.py)."""
    g = np.load(golden_path("host_extract_links.npz"))
    heads = int(g[f"{case}_heads"])
    q, kl, kr = (torch.from_numpy(g[f"{case}_{n}"]) for n in ("q", "kl", "kr"))
    B, L, E = q.shape
    shape = (B, L, heads, E // heads)
    links = ops.get_pcfg_kernel().extract_links(
        q.view(shape).to(DEV), kl.view(shape).to(DEV), kr.view(shape).to(DEV), torch.from_numpy(g[f"{case}_gates"]).to(DEV),
        torch.from_numpy(g[f"{case}_prev"]).to(DEV), 1, torch.from_numpy(g[f"{case}_left_mask"]),
        torch.from_numpy(g[f"{case}_right_mask"]), torch.from_numpy(g[f"{case}_main_chain"]))
    want = g[f"{case}_links"]
    got = links.cpu().numpy()
    assert got.shape == want.shape
    assert np.array_equal(np.isfinite(got), np.isfinite(want))
    fin = np.isfinite(want)
    assert fin.sum() > 20
    np.testing.assert_allclose(got[fin], want[fin], rtol=1e-4, atol=1e-5)
    # the rows of a node are a distribution over (left option, right child)
    rows = np.isfinite(want).any(axis=(2, 3))
    mass = np.exp(got[rows].reshape(rows.sum(), -1).astype(np.float64)).sum(-1)
    np.testing.assert_allclose(mass, 1.0, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("case", ["small", "mid"])
def test_extract_links_backward_against_reference_autograd(ops, case, dtype):
    """The hand-written backward of extract_links against the reference model's own function differentiated by
    autograd (tests/golden/make_golden_links.py): gradient of sum(links * G) over the finite entries with respect to
    the three link feature tensors and the gate logits."""
    g = np.load(golden_path("host_extract_links.npz"))
    heads = int(g[f"{case}_heads"])
    t = lambda n: torch.from_numpy(g[f"{case}_{n}"])
    B, L, E = t("q").shape
    shape = (B, L, heads, E // heads)
    leaves = [t(n).view(shape).to(DEV, dtype).requires_grad_(True) for n in ("q", "kl", "kr")]
    gates = t("gates").to(DEV).requires_grad_(True)
    links = ops.get_pcfg_kernel().extract_links(*leaves, gates, t("prev").to(DEV), 1, t("left_mask"), t("right_mask"),
                                                t("main_chain"))
    assert links.requires_grad
    fin = torch.isfinite(links)
    (torch.where(fin, links, torch.zeros_like(links)) * t("G").to(DEV)).sum().backward()
    tol = dict(rtol=1e-3, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)  # f16 inputs are rounded
    for leaf, name in zip(leaves, ("dq", "dkl", "dkr")):
        assert leaf.grad.dtype == dtype
        np.testing.assert_allclose(leaf.grad.float().cpu().numpy().reshape(B, L, E), g[f"{case}_{name}"], **tol)
    np.testing.assert_allclose(gates.grad.cpu().numpy(), g[f"{case}_dgates"], **tol)
    if dtype == torch.float32:  # and through the loss: d loss / d link features, against float64 torch autograd
        import importlib

        match = torch.randn(B, L, 5, device=DEV).log_softmax(0)
        ol = t("prev").ne(1).sum(1).to(DEV)
        tl = torch.full((B,), 5, device=DEV)
        for x in leaves + [gates]:
            x.grad = None
        links = ops.get_pcfg_kernel().extract_links(*leaves, gates, t("prev").to(DEV), 1, t("left_mask"), t("right_mask"),
                                                    t("main_chain"))
        loss = ops.cuda_pcfg_loss(match, links, ol, tl)
        ok = torch.isfinite(loss)
        assert ok.any()
        loss[ok].sum().backward()
        assert all(torch.isfinite(x.grad).all() for x in leaves + [gates]) and leaves[0].grad.abs().sum() > 0


def test_decode_step_from_link_features(pkg, ops, syn):
    """DecodeStep fed with the projected link features gives what extract_links + the transition-fed step give."""
    import importlib

    runtime = importlib.import_module("pcfg_nat_b200.runtime")
    support_tree = importlib.import_module("pcfg_nat_b200.support_tree")
    w = syn.Workload("decf", batch=4, vocab=500, hidden=64, src_min=4, src_max=12, kind="viterbi")
    b = syn.make_batch(w, seed=8)
    heads, dim = 8, 16
    g = torch.Generator().manual_seed(3)
    q, kl, kr = (torch.randn(b.B, b.L, heads, dim, generator=g).half() for _ in range(3))
    gates = torch.randn(b.B, b.L, heads, generator=g)
    prev = torch.where(torch.arange(b.L)[None, :] < b.output_length[:, None], 3, 1)
    lm, rm, mc = support_tree.get_mask(b.L, 1)
    k = ops.get_pcfg_kernel()
    links = k.extract_links(q.to(DEV), kl.to(DEV), kr.to(DEV), gates.to(DEV), prev.to(DEV), 1, lm, rm, mc)
    want = pyref.extract_links(q, kl, kr, gates, prev, 1, lm, rm, mc)
    assert torch.equal(torch.isfinite(links).cpu(), torch.isfinite(want))
    fin = torch.isfinite(want)
    torch.testing.assert_close(links.cpu()[fin], want[fin], rtol=1e-4, atol=1e-5)
    weight = b.weight.to(DEV)
    plain = runtime.DecodeStep(weight, b.B, b.L, lm, DEV)
    plain.load(b.hidden.pin_memory(), links, b.output_length.pin_memory())
    feat = runtime.DecodeStep(weight, b.B, b.L, lm, DEV, link_features=(heads, dim), right_tree_mask=rm, main_chain=mc)
    feat.load(b.hidden.pin_memory(), q.pin_memory(), kl.pin_memory(), kr.pin_memory(), gates.pin_memory(),
              prev.pin_memory(), b.output_length.pin_memory(), overlap=True)
    for _ in range(2):
        t1, c1, p1 = [t.clone() for t in plain.run()]
        t2, c2, p2 = [t.clone() for t in feat.run()]
    assert torch.equal(t1, t2) and torch.equal(c1, c2) and torch.equal(p1, p2)
    assert int(c1.min()) >= 1


def test_loss_stats_exchange_bounded_wait(ops):
    """The in-kernel exchange of the loss statistics with a peer that never arrives: the wait runs out, the
    status word says so, the statistics are NaN (never a short sum that could pass for a loss), the host-side
    check raises, and the context stays usable."""
    k = ops.get_pcfg_kernel()
    bufs = [torch.zeros(64, dtype=torch.float32, device=DEV) for _ in range(2)]  # >= PCFGNAT_EXCHANGE_BYTES(2)
    peers = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=DEV)
    loss = torch.tensor([-4.0, -9.0, float("-inf")], device=DEV)
    tl = torch.tensor([2, 3, 5], device=DEV)
    ops.read_status(DEV)
    stats = k.loss_stats_exchange(loss, tl, peers, 0, 2).cpu()
    assert torch.isnan(stats).all()
    assert ops.read_status(DEV) & 8  # PCFGNAT_STATUS_TIMEOUT
    import importlib

    sharding = importlib.import_module("pcfg_nat_b200.sharding")
    with pytest.raises(RuntimeError, match="did not arrive"):
        sharding.check_exchanged_stats(stats)
    assert sharding.check_exchanged_stats(torch.tensor([-5.0, 3.0, 1.0])) is None
    # a world of one rank needs nobody else
    one = torch.zeros(64, dtype=torch.float32, device=DEV)
    stats = k.loss_stats_exchange(loss, tl, torch.tensor([one.data_ptr()], dtype=torch.int64, device=DEV), 0, 1).cpu()
    assert stats.tolist() == [-5.0, 3.0, 1.0] and ops.read_status(DEV) == 0


def test_decode_and_glance_steps_match_operator_chain(pkg, ops, syn):
    """The graph-replayed decode / glancing steps give what the individual operators give."""
    import importlib

    runtime = importlib.import_module("pcfg_nat_b200.runtime")
    w = syn.Workload("dec", batch=5, vocab=2000, hidden=64, src_min=6, src_max=24, kind="viterbi")
    b = syn.make_batch(w, seed=4)
    weight = b.weight.to(DEV)
    dec = runtime.DecodeStep(weight, b.B, b.L, b.left_tree_mask, DEV, beta=1.0, pad_index=1)
    dec.load(b.hidden.pin_memory(), b.links.pin_memory(), b.output_length.pin_memory())
    for _ in range(2):  # capture, then replay
        tokens, count, pred = [t.clone() for t in dec.run()]
    torch.cuda.synchronize()
    # reference chain on the CPU: fp32 projection -> log-softmax max -> oracle Viterbi -> oracle back-trace
    lp = torch.log_softmax(b.hidden.float() @ b.weight.float().t(), -1)
    ob, tok = lp.max(-1)
    out = ops.proj_logsoftmax_gather(b.hidden.to(DEV), weight, None, b.output_length.to(DEV), None, want_max=True)
    real = torch.arange(b.L)[None, :] < b.output_length[:, None]
    torch.testing.assert_close(out["max_lprob"].cpu()[real], ob[real], rtol=0, atol=2e-3)
    # Viterbi on the kernel's own emissions (bit-exact path), compared with the oracle on the same numbers
    ob_k, tok_k = out["max_lprob"].cpu(), out["argmax"].cpu()
    So, Ro, Lo, Mo = oracle.pcfg_viterbi(ob_k.numpy(), b.links.numpy(), b.output_length.numpy())
    sc = torch.from_numpy(So[:, 1, :]) / torch.arange(b.L // 4).unsqueeze(0)
    sc = torch.where(torch.isnan(sc), torch.full_like(sc, float("-inf")), sc)
    want_pred = sc[:, 1:].max(-1)[1] + 1
    assert torch.equal(pred.cpu(), want_pred)
    want = oracle.viterbi_decoding_lists(want_pred.numpy(), b.output_length.numpy(), Lo, Ro, Mo, tok_k.numpy(),
                                         b.left_tree_mask.long().numpy(), 1)
    for i, row in enumerate(want):
        assert tokens[i, :int(count[i])].cpu().tolist() == row
        assert (tokens[i, int(count[i]):] == 1).all()

    wg = syn.Workload("gl", batch=4, vocab=2000, hidden=64, src_min=6, src_max=20, kind="glance")
    g = syn.make_batch(wg, seed=5)
    gs = runtime.GlanceStep(g.weight.to(DEV), g.B, g.L, g.T, DEV, context_p=0.5)
    prev = torch.where(torch.arange(g.L)[None, :] < g.output_length[:, None], 3, 1)
    gs.load(g.hidden.pin_memory(), g.links.pin_memory(), g.output_length.pin_memory(), g.targets.pin_memory(),
            g.target_length.pin_memory(), prev.pin_memory())
    for _ in range(2):
        tree, ll, am, glance = gs.run()
        tree, ll, am = tree.clone(), ll.clone(), am.clone()
    noise = gs.noise.cpu()
    assert noise.std() > 0.5  # drawn inside the replayed graph
    want = pyref.glance_select(tree.cpu(), am.cpu(), g.targets, prev, g.target_length, noise, 0.5)
    for key, val in want.items():
        assert torch.equal(glance[key].cpu(), val), key
    em = ops.proj_logsoftmax_gather(g.hidden.to(DEV), g.weight.to(DEV), g.targets.to(DEV), g.output_length.to(DEV),
                                    g.target_length.to(DEV), want_max=True)
    tree2, ll2 = ops.cuda_pcfg_best_tree(em["match"], g.links.to(DEV), g.output_length.to(DEV), g.target_length.to(DEV))
    assert torch.equal(tree, tree2) and torch.equal(ll, ll2) and torch.equal(am, em["argmax"])
    So, Co = oracle.pcfg_loss(em["match"].cpu().numpy(), g.links.numpy(), g.output_length.numpy(), g.target_length.numpy())
    want_tree = oracle.pcfg_best_tree(So, Co, em["match"].cpu().numpy(), g.links.numpy(), g.output_length.numpy(),
                                      g.target_length.numpy())
    # same emissions; the tables differ from the oracle's only in the last ulp of expf/logf
    assert (tree.cpu().numpy() == want_tree).mean() > 0.99


# ---- criterion glue against the reference criterion's own code (tests/golden/host_criterion.npz) -----------------

@pytest.mark.parametrize("tag,strategy", [("none", None), ("number_random", "number-random"), ("cmlm", "cmlm")])
def test_glance_select_against_reference_criterion(ops, tag, strategy):
    g = _g("host_criterion.npz")
    t = lambda key: torch.from_numpy(g[key]).to(DEV)
    B, L = g["path"].shape
    noise, uniform = pyref.criterion_draws(strategy, int(g[f"{tag}_seed"]), B, L)
    k = ops.get_pcfg_kernel()
    pred = t("logits").argmax(-1)
    got = k.glance_select(t("path"), pred, t("tgt"), t("prev"), t("tgt_len"),
                          None if noise is None else noise.to(DEV), 0.5, strategy,
                          None if uniform is None else uniform.to(DEV))
    assert torch.equal(got["matchmask"], t(f"{tag}_matchmask"))
    assert torch.equal(got["keep_word_mask"], t(f"{tag}_keep"))
    assert torch.equal(got["glat_prev_output_tokens"], t(f"{tag}_glat_prev"))
    accu = float(got["same_num"].sum() / t("tgt_len").sum())
    assert abs(accu - float(g[f"{tag}_glat_accu"])) < 1e-6
    want = pyref.glance_select(t("path").cpu(), pred.cpu(), t("tgt").cpu(), t("prev").cpu(), t("tgt_len").cpu(), noise,
                               0.5, strategy, uniform)
    for key, val in want.items():
        assert torch.equal(got[key].cpu(), val), key


def test_force_emit_against_reference_criterion(pkg, ops, syn):
    g = _g("host_criterion.npz")
    t = lambda key: torch.from_numpy(g[key]).to(DEV)
    eos = syn.eos_mask_(t("match_plain").clone(), t("out_len"), t("tgt_len"))
    assert torch.equal(eos, t("plain_loss_match"))
    ma = eos.clone().requires_grad_(True)
    out = ops.force_emit_mask(ma, t("number_random_matchmask"), t("number_random_keep"))
    assert torch.equal(out.detach(), t("force_loss_match"))
    # the same recording loss as the fixture's: linear with weights loss_w on the finite entries
    n = t("tgt_len").float()
    fin = torch.isfinite(out)
    sent = (torch.where(fin, out, torch.zeros_like(out)) * t("loss_w")).sum((1, 2))
    valid = torch.tensor([True, True, False, True, True], device=DEV)
    (-(torch.where(valid, sent, torch.zeros_like(sent)) / n).mean()).backward()
    torch.testing.assert_close(ma.grad, t("force_match_grad"), rtol=1e-6, atol=0)
    # in place, as the step object uses it
    k = ops.get_pcfg_kernel()
    buf = eos.clone()
    k.force_emit(buf, t("number_random_matchmask"), t("number_random_keep"), out=buf)
    assert torch.equal(buf, t("force_loss_match"))


def test_loss_step_with_force_emit_matches_operator_chain(pkg, ops, syn):
    """GlanceStep -> LossStep(force_emit=True), as a GLAT training step chains them, against the operators one by
    one with autograd and against the oracle fed the masked emissions."""
    import importlib

    runtime = importlib.import_module("pcfg_nat_b200.runtime")
    w = syn.Workload("fe", batch=5, vocab=2000, hidden=64, src_min=6, src_max=20, kind="glance")
    b = syn.make_batch(w, seed=6)
    weight = b.weight.to(DEV)
    prev = torch.where(torch.arange(b.L)[None, :] < b.output_length[:, None], 3, 1)
    gs = runtime.GlanceStep(weight, b.B, b.L, b.T, DEV, context_p=0.5)
    gs.load(b.hidden, b.links, b.output_length, b.targets, b.target_length, prev)
    tree, ll, am, glance = gs.run()
    assert glance["keep_word_mask"].any()
    ls = runtime.LossStep(weight, b.B, b.L, b.T, DEV, force_emit=True)
    ls.load(b.hidden, b.links, b.output_length, b.targets, b.target_length, glance["matchmask"], glance["keep_word_mask"])
    for _ in range(2):  # capture, replay
        stats, mg, lg, loss = [x.clone() for x in ls.run()]
    em = ops.proj_logsoftmax_gather(b.hidden.to(DEV), weight, b.targets.to(DEV), b.output_length.to(DEV),
                                    b.target_length.to(DEV))["match"].requires_grad_(True)
    lk = b.links.to(DEV).requires_grad_(True)
    masked = ops.force_emit_mask(em, glance["matchmask"], glance["keep_word_mask"])
    loss2 = ops.cuda_pcfg_loss(masked, lk, b.output_length.to(DEV), b.target_length.to(DEV))
    loss2.sum().backward()
    assert torch.isfinite(loss2).all()
    assert torch.equal(loss, loss2.detach()) and torch.equal(mg, em.grad) and torch.equal(lg, lk.grad)
    assert (mg[glance["keep_word_mask"]] == 0).all()
    m_np = masked.detach().cpu().numpy()
    So, Co = oracle.pcfg_loss(m_np, b.links.numpy(), b.output_length.numpy(), b.target_length.numpy())
    np.testing.assert_allclose(loss.cpu().numpy(), So[:, 0, 0], rtol=1e-4)
    mgo, lgo = oracle.pcfg_loss_backward(np.ones(b.B, np.float32), So, Co, m_np, b.links.numpy(),
                                         b.output_length.numpy(), b.target_length.numpy())
    mgo[glance["keep_word_mask"].cpu().numpy()] = 0
    np.testing.assert_allclose(mg.cpu().numpy(), mgo, rtol=1e-3, atol=2e-6)
    np.testing.assert_allclose(lg.cpu().numpy(), lgo, rtol=1e-3, atol=2e-6)


# ---- linear-space loss forward + backward (the default of the fused entry point) ---------------------------------

def _fused(ops, ma, lk, ol, tl):
    k = ops.get_pcfg_kernel()
    loss, mg, lg = k.pcfg_loss_fwd_bwd(ma, lk, ol, tl)
    torch.cuda.synchronize()
    return loss, mg, lg


@pytest.mark.parametrize("peak", [1.0, 8.0, 25.0])
@pytest.mark.parametrize("shape", [dict(batch=5, src_min=4, src_max=30), dict(batch=3, fixed_graph=384, fixed_target=90),
                                   dict(batch=70, src_min=6, src_max=20)])
def test_linear_space_loss_against_oracle_peaked_inputs(ops, syn, monkeypatch, peak, shape):
    """Emissions and transitions sharpened by `peak` (a trained model is far from the near-uniform synthetic
    inputs): columns then span many e-folds, which is what the per-column scaling has to absorb; whatever it
    cannot is recomputed in log space.  Either way the results hold the parity tolerances."""
    monkeypatch.delenv("PCFGNAT_DP_KERNEL", raising=False)
    w = syn.Workload("lin", vocab=50, hidden=8, emissions="logits", **shape)
    b = syn.make_batch(w, seed=31)
    b.logits.mul_(peak)
    ma = syn.reference_match_all(b)
    lk = torch.log_softmax((b.links * peak).view(b.B, b.L, -1), -1).view_as(b.links)
    lk = torch.where(torch.isfinite(b.links), lk, b.links).contiguous()
    lk = torch.where(torch.isnan(lk), torch.full_like(lk, float("-inf")), lk)
    ol, tl = b.output_length.numpy(), b.target_length.numpy()
    So, Co = oracle.pcfg_loss(ma.numpy(), lk.numpy(), ol, tl)
    mgo, lgo = oracle.pcfg_loss_backward(np.ones(b.B, np.float32), So, Co, ma.numpy(), lk.numpy(), ol, tl)
    ops.read_status(DEV)
    loss, mg, lg = _fused(ops, ma.to(DEV), lk.to(DEV), b.output_length.to(DEV), b.target_length.to(DEV))
    recomputed = bool(ops.read_status(DEV) & 16)  # PCFGNAT_STATUS_RECOMPUTED
    assert peak > 1.0 or not recomputed  # ordinary inputs stay in linear space
    assert np.isfinite(So[:, 0, 0]).all()
    np.testing.assert_allclose(loss.cpu().numpy(), So[:, 0, 0], rtol=1e-4)
    np.testing.assert_allclose(mg.cpu().numpy(), mgo, rtol=1e-3, atol=2e-6)
    np.testing.assert_allclose(lg.cpu().numpy(), lgo, rtol=1e-3, atol=2e-6)
    # and against the log-space kernels of the same library
    monkeypatch.setenv("PCFGNAT_LINEAR_DP", "0")
    loss2, mg2, lg2 = _fused(ops, ma.to(DEV), lk.to(DEV), b.output_length.to(DEV), b.target_length.to(DEV))
    torch.testing.assert_close(loss, loss2, rtol=1e-5, atol=0)
    torch.testing.assert_close(mg, mg2, rtol=1e-3, atol=2e-6)
    torch.testing.assert_close(lg, lg2, rtol=1e-3, atol=2e-6)


def test_linear_space_loss_hands_unusual_sentences_to_the_log_space_kernels(ops, syn, monkeypatch):
    """One batch with everything the linear-space kernels do not take themselves: an emission far beyond the range of
    exp() relative to its token's maximum, an out-of-range length, an odd graph length, a single target token, an infeasible sentence (more tokens
    than the graph can emit), next to ordinary sentences.  Every sentence must come out as the log-space kernels
    alone give it, and output buffers that were dirty must be fully overwritten."""
    monkeypatch.delenv("PCFGNAT_DP_KERNEL", raising=False)
    w = syn.Workload("lin2", batch=8, vocab=50, hidden=8, src_min=5, src_max=12, emissions="logits")
    b = syn.make_batch(w, seed=32)
    ma = syn.reference_match_all(b)
    ol, tl = b.output_length.clone(), b.target_length.clone()
    ma[0, 2, 0] = 200.0           # a leaf emission far above the main chain's: exp() overflows
    ol[1] = b.L + 4               # out of range
    ol[2] = ol[2] - 1             # odd graph length
    tl[3] = 1                     # one target token
    tl[4] = min(int(ol[4]) - 1, b.T)  # infeasible: n > m - 2
    k = ops.get_pcfg_kernel()
    args = (ma.to(DEV), b.links.to(DEV), ol.to(DEV), tl.to(DEV))
    ops.read_status(DEV)
    loss, mg, lg = _fused(ops, *args)
    st = ops.read_status(DEV)
    assert st & 1 and st & 16  # a bad length was seen; sentences were recomputed in log space
    monkeypatch.setenv("PCFGNAT_DP_KERNEL", "rows")  # the kernels that pick up the marked sentences, on their own
    loss2, mg2, lg2 = _fused(ops, *args)
    ops.read_status(DEV)
    assert torch.equal(torch.isfinite(loss), torch.isfinite(loss2))
    fin = torch.isfinite(loss2)
    assert fin[5:].all() and not fin[1] and not fin[4]
    torch.testing.assert_close(loss[fin], loss2[fin], rtol=1e-5, atol=0)
    torch.testing.assert_close(mg, mg2, rtol=1e-3, atol=2e-6, equal_nan=True)
    torch.testing.assert_close(lg, lg2, rtol=1e-3, atol=2e-6, equal_nan=True)
    for i in (0, 1, 2, 3, 4):  # handed over: bit for bit what the log-space kernels give
        assert torch.equal(mg[i].nan_to_num(7.0), mg2[i].nan_to_num(7.0)) and torch.equal(lg[i].nan_to_num(7.0), lg2[i].nan_to_num(7.0))


def test_pipelined_steps_overlap_copies_without_mixing_batches(pkg, ops, syn):
    """Two step objects in turn (copies of the next batch while the current one is computed): different batches
    through the pipeline come out exactly as through a single step object, in order."""
    import importlib

    runtime = importlib.import_module("pcfg_nat_b200.runtime")
    w = syn.Workload("pipe", batch=6, vocab=3000, hidden=128, fixed_graph=40, fixed_target=9, hidden_std=1.0)
    batches = [syn.make_batch(w, seed=40 + i) for i in range(5)]
    weight = batches[0].weight.to(DEV)
    B, L, T = batches[0].B, batches[0].L, batches[0].T
    host = [[t.contiguous().pin_memory() for t in (b.hidden, b.links, b.output_length, b.targets, b.target_length)]
            for b in batches]
    single = runtime.LossStep(weight, B, L, T, DEV)
    want = []
    for h in host:
        single.load(*h)
        want.append([t.clone() for t in single.run()])
    pipe = runtime.PipelinedStep(lambda: runtime.LossStep(weight, B, L, T, DEV))
    got = []
    for h in host:
        pipe.load(*h)
        out = pipe.run()
        got.append([t.clone() for t in out])  # cloned on the run's stream, before the run after next reuses the buffers
    torch.cuda.synchronize()
    for a, b in zip(got, want):
        for x, y in zip(a, b):
            assert torch.equal(x, y)
    assert not torch.equal(want[0][3], want[1][3])


# ---- lookahead / greedy decoding ---------------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["look_b1_a", "look_b1_b", "greedy_b4", "greedy_b1"])
def test_lookahead_decode_against_reference_model(ops, name):
    g = _g("host_lookahead.npz")
    t = lambda key: torch.from_numpy(g[f"{name}_{key}"]).to(DEV)
    strategy = "lookahead" if int(g[f"{name}_lookahead"]) else "greedy"
    k = ops.get_pcfg_kernel()
    ops.read_status(DEV)
    out, cnt = k.lookahead_decode_device(t("links"), t("ob"), t("tok"), t("out_len"), t("mask"), 1,
                                         float(g[f"{name}_beta"]), strategy)
    want = g[f"{name}_result"]
    assert int(cnt.max()) == want.shape[1]
    assert np.array_equal(out[:, :want.shape[1]].cpu().numpy(), want)
    assert (out[:, want.shape[1]:] == 1).all() and ops.read_status(DEV) == 0


@pytest.mark.parametrize("strategy", ["lookahead", "greedy"])
def test_lookahead_decode_step_against_restatement(pkg, ops, syn, strategy):
    """DecodeStep with the two host-loop strategies of the model, on a ragged batch, against the restatement fed the
    kernel's own emissions (arg-max decoding on identical numbers: exact)."""
    import importlib

    runtime = importlib.import_module("pcfg_nat_b200.runtime")
    w = syn.Workload("la", batch=9, vocab=2000, hidden=64, src_min=4, src_max=40, kind="viterbi")
    b = syn.make_batch(w, seed=8)
    weight = b.weight.to(DEV)
    step = runtime.DecodeStep(weight, b.B, b.L, b.left_tree_mask, DEV, strategy=strategy, decode_beta=0.7)
    step.load(b.hidden, b.links, b.output_length)
    for _ in range(2):
        tokens, count = [x.clone() for x in step.run()]
    em = ops.proj_logsoftmax_gather(b.hidden.to(DEV), weight, None, b.output_length.to(DEV), None, want_max=True)
    rows = pyref.lookahead_decode(b.links, em["max_lprob"].cpu(), em["argmax"].cpu(), b.output_length,
                                  b.left_tree_mask.bool(), 1, 0.7, strategy == "lookahead")
    assert min(len(r) for r in rows) >= 2
    for i, r in enumerate(rows):
        assert int(count[i]) == len(r) and tokens[i, :len(r)].cpu().tolist() == r
        assert (tokens[i, len(r):] == 1).all()


def test_loss_step_from_link_features_matches_autograd_chain(pkg, ops, syn):
    """LossStep fed with the projected link features (transitions formed and differentiated inside the step) against
    the operators chained by autograd: extract_links -> cuda_pcfg_loss -> backward."""
    import importlib

    runtime = importlib.import_module("pcfg_nat_b200.runtime")
    support = importlib.import_module("pcfg_nat_b200.support_tree")
    w = syn.Workload("lf", batch=5, vocab=2000, hidden=64, src_min=5, src_max=14)
    b = syn.make_batch(w, seed=9)
    heads, dim = 4, 16
    g = torch.Generator().manual_seed(3)
    q, kl, kr = (torch.randn(b.B, b.L, heads, dim, generator=g).half() for _ in range(3))
    gates = torch.randn(b.B, b.L, heads, generator=g)
    prev = torch.where(torch.arange(b.L)[None, :] < b.output_length[:, None], 3, 1)
    lm, rm, mc = support.get_mask(b.L, 1)
    weight = b.weight.to(DEV)
    step = runtime.LossStep(weight, b.B, b.L, b.T, DEV, link_features=(heads, dim), left_tree_mask=lm, right_tree_mask=rm,
                            main_chain=mc)
    step.load(b.hidden, q, kl, kr, gates, prev, b.output_length, b.targets, b.target_length)
    for _ in range(2):  # capture, replay
        stats, mg, (dq, dkl, dkr, dgates), loss = step.run()
    torch.cuda.synchronize()
    leaves = [x.to(DEV).requires_grad_(True) for x in (q, kl, kr)]
    gt = gates.to(DEV).requires_grad_(True)
    links = ops.get_pcfg_kernel().extract_links(*leaves, gt, prev.to(DEV), 1, lm, rm, mc)
    em = ops.proj_logsoftmax_gather(b.hidden.to(DEV), weight, b.targets.to(DEV), b.output_length.to(DEV),
                                    b.target_length.to(DEV))["match"]
    loss2 = ops.cuda_pcfg_loss(em, links, b.output_length.to(DEV), b.target_length.to(DEV))
    assert torch.isfinite(loss2).all()
    loss2.sum().backward()
    assert torch.equal(loss, loss2.detach())
    for got, leaf in zip((dq, dkl, dkr), leaves):
        torch.testing.assert_close(got, leaf.grad.float(), rtol=1e-3, atol=1e-3)  # the chain rounds its gradients to f16
    torch.testing.assert_close(dgates, gt.grad, rtol=1e-5, atol=1e-6)
    assert dq.abs().sum() > 0 and dkr.abs().sum() > 0


@pytest.mark.parametrize("mode", ["links", "all"])
def test_overlapped_load_fetching_from_host_buffers(pkg, ops, syn, mode):
    """An overlapped load whose large inputs are fetched by the kernel that reads the pinned host buffers itself
    (only the real nodes' states / only the transitions the tree masks leave finite) gives the step exactly what the
    plain copies give it, batch after batch (shorter sentences after longer ones: nothing stale is read)."""
    import importlib

    runtime = importlib.import_module("pcfg_nat_b200.runtime")
    w = syn.Workload("fh", batch=6, vocab=3000, hidden=128, src_min=3, src_max=12, hidden_std=1.0)
    batches = [syn.make_batch(w, seed=50 + i) for i in range(4)]
    L, T = max(b.L for b in batches), max(b.T for b in batches)

    def padded(b):
        hid = torch.randn(b.B, L, w.hidden).half()  # garbage beyond the real nodes: it must not matter
        hid[:, :b.L] = b.hidden
        lk = torch.full((b.B, L, 2, L), float("-inf"))
        lk[:, :b.L, :, :b.L] = b.links
        tg = torch.ones(b.B, T, dtype=torch.long)
        tg[:, :b.T] = b.targets
        return [t.contiguous().pin_memory() for t in (hid, lk, b.output_length, tg, b.target_length)]

    weight = batches[0].weight.to(DEV)
    plain = runtime.LossStep(weight, w.batch, L, T, DEV)
    fetched = runtime.LossStep(weight, w.batch, L, T, DEV)
    fetched.fetch_from_host = mode
    for b in batches:
        args = padded(b)
        plain.load(*args)
        want = [t.clone() for t in plain.run()]
        fetched.load(*args, overlap=True)
        got = fetched.run()
        torch.cuda.synchronize()
        for x, y in zip(got, want):
            assert torch.equal(x, y)
        assert fetched.input_bytes() < plain.input_bytes()
        kernel_links = fetched.links.cpu()
        assert torch.equal(kernel_links, args[1])  # the model's masks leave nothing finite outside what was fetched


def test_smoke_with_dependent_launches_and_ranges_switched_on():
    """PCFGNAT_PDL=1 (programmatic dependent launch along the kernel chain) and PCFGNAT_NVTX=1 are read once per
    process: a fresh interpreter runs the package's smoke check, which compares a step with the oracle, with both on."""
    import subprocess
    import sys

    from conftest import ROOT

    env = dict(os.environ, PCFGNAT_PDL="1", PCFGNAT_NVTX="1")
    r = subprocess.run([sys.executable, "-c", "import __graft_entry__ as g; g.smoke()"], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "smoke ok" in r.stdout
