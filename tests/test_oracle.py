"""CPU tests of the oracle: against independent restatements (brute-force enumeration of
derivations, float64 autograd), against structural invariants, and against golden outputs
of the reference itself (tests/golden/)."""
import os

import numpy as np
import pytest
import torch

import oracle
from _pyref import loss_bruteforce, loss_two_term
from conftest import golden_path


def _small_batch(syn, seed, batch=4, smin=2, smax=5):
    w = syn.Workload("t", batch=batch, vocab=50, hidden=8, src_min=smin, src_max=smax, emissions="logits")
    b = syn.make_batch(w, seed=seed)
    return b, syn.reference_match_all(b)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_loss_matches_bruteforce_and_two_term(syn, seed):
    b, ma = _small_batch(syn, seed)
    S, C = oracle.pcfg_loss(ma.numpy(), b.links.numpy(), b.output_length.numpy(), b.target_length.numpy())
    for i in range(b.B):
        m, n = int(b.output_length[i]), int(b.target_length[i])
        bf = loss_bruteforce(ma[i].double(), b.links[i].double(), m, n)
        tt = loss_two_term(ma[i].double(), b.links[i].double(), m, n).item()
        assert abs(S[i, 0, 0] - bf) <= 1e-4 * max(1.0, abs(bf))
        assert abs(S[i, 0, 0] - tt) <= 1e-4 * max(1.0, abs(tt))


def test_feasibility_boundary(syn):
    # at left_tree_layer 1 a sentence is derivable iff 2 <= n <= m - 2
    b, ma = _small_batch(syn, 5, batch=1, smin=4, smax=4)
    m = int(b.output_length[0])
    lp = torch.log_softmax(torch.randn(1, b.L, 50, generator=torch.Generator().manual_seed(1)), -1)
    for n in (1, 2, m - 2, m - 1):
        tgt = torch.randint(4, 50, (1, n), generator=torch.Generator().manual_seed(n))
        mm = lp.gather(2, tgt[:, None, :].expand(-1, b.L, -1)).contiguous()
        syn.eos_mask_(mm, b.output_length, torch.tensor([n]))
        S, _ = oracle.pcfg_loss(mm.numpy(), b.links.numpy(), b.output_length.numpy(), np.array([n]))
        assert np.isfinite(S[0, 0, 0]) == (2 <= n <= m - 2), n


@pytest.mark.parametrize("seed", [0, 3])
def test_backward_matches_float64_autograd(syn, seed):
    b, ma = _small_batch(syn, seed)
    ol, tl = b.output_length.numpy(), b.target_length.numpy()
    S, C = oracle.pcfg_loss(ma.numpy(), b.links.numpy(), ol, tl)
    mg, lg = oracle.pcfg_loss_backward(np.ones(b.B, np.float32), S, C, ma.numpy(), b.links.numpy(), ol, tl)
    for i in range(b.B):
        mt = ma[i].double().clone().requires_grad_(True)
        lt = b.links[i].double().clone().requires_grad_(True)
        loss_two_term(mt, lt, int(ol[i]), int(tl[i])).backward()
        gm = torch.nan_to_num(mt.grad, nan=0.0).numpy()
        gl = torch.nan_to_num(lt.grad, nan=0.0).numpy()
        assert np.abs(gm - mg[i]).max() < 1e-4
        assert np.abs(gl - lg[i]).max() < 1e-4
        # posterior marginals: every target position is emitted by exactly one node
        n = int(tl[i])
        np.testing.assert_allclose(mg[i].sum(0)[:n], 1.0, atol=1e-4)
        assert np.abs(mg[i][:, n:]).max(initial=0.0) == 0.0


def test_backward_rejects_other_tree_depths():
    ma = np.zeros((1, 10, 3), np.float32)
    lk = np.zeros((1, 10, 4, 10), np.float32)
    S, C = oracle.pcfg_loss(ma, lk, np.array([10]), np.array([3]))
    with pytest.raises(RuntimeError):
        oracle.pcfg_loss_backward(np.ones(1, np.float32), S, C, ma, lk, np.array([10]), np.array([3]))


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_best_tree_invariants(syn, seed):
    b, ma = _small_batch(syn, seed, batch=5, smin=3, smax=9)
    ol, tl = b.output_length.numpy(), b.target_length.numpy()
    S, C = oracle.pcfg_loss(ma.numpy(), b.links.numpy(), ol, tl)
    tree = oracle.pcfg_best_tree(S, C, ma.numpy(), b.links.numpy(), ol, tl)
    for i in range(b.B):
        m, n = int(ol[i]), int(tl[i])
        used = [(a, int(t)) for a, t in enumerate(tree[i]) if t >= 0]
        assert [t for _, t in used] == list(range(n))  # in-order = target order, each position once
        assert used[0] == (1, 0) and used[-1] == (m - 1, n - 1)
        for a, t in used:
            if a % 2 == 0:  # a leaf is used only together with its parent
                assert tree[i, a + 1] == t + 1
        assert (tree[i, m:] == -1).all()


@pytest.mark.parametrize("seed", [0, 1])
def test_viterbi_and_backtrace_invariants(syn, seed):
    w = syn.Workload("v", batch=4, vocab=60, hidden=8, src_min=5, src_max=15, emissions="logits", kind="viterbi")
    b = syn.make_batch(w, seed=seed)
    ob, tok = torch.log_softmax(b.logits, -1).max(-1)
    tok = torch.arange(b.L)[None, :].expand(b.B, -1).contiguous() + 100  # distinct tokens: no collapsing
    S, R, Lt, Mt = oracle.pcfg_viterbi(ob.numpy(), b.links.numpy(), b.output_length.numpy())
    for i in range(b.B):
        m = int(b.output_length[i])
        root = S[i, 1]
        finite = np.nonzero(np.isfinite(root))[0]
        assert set(finite.tolist()) <= set(range(2, m // 4))  # root scores exist only for lengths 2..m/4-1
        for ln in finite:
            out = oracle.viterbi_decoding_lists(np.array([ln]), b.output_length[i:i + 1].numpy(), Lt[i:i + 1],
                                                R[i:i + 1], Mt[i:i + 1], tok[i:i + 1].numpy(),
                                                b.left_tree_mask.long().numpy(), 1)[0]
            assert len(out) == ln and out[0] == 101 and out[-1] == 100 + m - 1
            assert out == sorted(out)
            # the score of the walked derivation equals the table entry
            nodes = [t - 100 for t in out]
            sc, k = 0.0, 0
            mains = [a for a in nodes if a % 2 == 1]
            for idx, a in enumerate(mains):
                sc += float(ob[i, a])
                leaf = a - 1 in nodes and a >= 3
                if leaf:
                    sc += float(ob[i, a - 1])
                if idx + 1 < len(mains):
                    sc += float(b.links[i, a, 1 if leaf else 0, mains[idx + 1]])
            assert abs(sc - root[ln]) < 1e-3


def test_backtrace_matches_reference_host_function():
    g = np.load(golden_path("host_viterbi_decoding.npz"))
    rows = oracle.viterbi_decoding_lists(g["pred_length"], g["output_length"], g["L"], g["R"], g["M"], g["tokens"],
                                         g["left_tree_mask"].astype(np.int64), 1)
    for i, r in enumerate(rows):
        assert r == g["decoded"][i, :g["decoded_len"][i]].tolist()
    padded = oracle.viterbi_decoding(g["pred_length"], g["output_length"], g["L"], g["R"], g["M"], g["tokens"],
                                     g["left_tree_mask"].astype(np.int64), 1)
    assert padded.dtype == np.float32
    np.testing.assert_array_equal(padded.astype(np.int64), g["decoded"])


def test_logsoftmax_gather_against_torch():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 5, 97, generator=g) * 4
    idx = torch.randint(0, 97, (2, 7), generator=g)
    sel, probs = oracle.logsoftmax_gather(x.numpy(), idx[:, None, :].expand(-1, 5, -1).numpy(), True)
    ref = torch.log_softmax(x.double(), -1).gather(2, idx[:, None, :].expand(-1, 5, -1))
    np.testing.assert_allclose(sel, ref.numpy(), atol=2e-5)
    np.testing.assert_allclose(probs, torch.softmax(x.double(), -1).numpy(), atol=1e-6)


# ---- golden outputs of the reference CUDA kernels (recorded on a B200) ---------------------------------------

LOSS_GOLDEN = ["ref_loss_tiny.npz", "ref_loss_ragged.npz", "ref_loss_mid.npz"]


def _load(name):
    p = golden_path(name)
    if not os.path.isfile(p):
        pytest.skip(f"{name} not recorded yet")
    return np.load(p)


def _close_tables(a, b, rtol):
    assert np.array_equal(np.isinf(a), np.isinf(b))
    fin = np.isfinite(a)
    np.testing.assert_allclose(a[fin], b[fin], rtol=rtol, atol=rtol)


@pytest.mark.parametrize("name", LOSS_GOLDEN)
def test_oracle_loss_against_reference_kernels(name):
    g = _load(name)
    S, C = oracle.pcfg_loss(g["match_all"], g["links"], g["output_length"], g["target_length"])
    _close_tables(S, g["S"], 1e-5)
    assert np.array_equal(C, g["C"])  # copies of inputs and constants: bit-exact
    mg, lg = oracle.pcfg_loss_backward(np.ones(len(S), np.float32), g["S"], g["C"], g["match_all"], g["links"],
                                       g["output_length"], g["target_length"])
    np.testing.assert_allclose(mg, g["match_all_grad"], rtol=1e-3, atol=1e-5)
    np.testing.assert_allclose(lg, g["links_grad"], rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("name", LOSS_GOLDEN)
def test_oracle_best_tree_against_reference_kernels(name):
    g = _load(name)
    # fed with the reference's own tables the arg-max trace must agree index for index
    tree = oracle.pcfg_best_tree(g["S"], g["C"], g["match_all"], g["links"], g["output_length"], g["target_length"])
    np.testing.assert_array_equal(tree, g["tree"])


@pytest.mark.parametrize("name", ["ref_viterbi_ragged.npz", "ref_viterbi_mid.npz"])
def test_oracle_viterbi_against_reference_kernels(name):
    g = _load(name)
    S, R, Lt, Mt = oracle.pcfg_viterbi(g["ob_lprob"], g["links"], g["output_length"])
    assert np.array_equal(S.view(np.int32), g["S"].view(np.int32))  # max-plus: bit-exact
    np.testing.assert_array_equal(R, g["R"])
    np.testing.assert_array_equal(Lt, g["L"])
    np.testing.assert_array_equal(Mt, g["M"])


def test_oracle_logsoftmax_gather_against_reference_kernel():
    g = _load("ref_logsoftmax_gather.npz")
    sel_idx = np.broadcast_to(g["targets"][:, None, :], (2, 8, 10))
    sel, probs = oracle.logsoftmax_gather(g["logits"], sel_idx, True)
    np.testing.assert_allclose(sel, g["selected_f32_0"], atol=1e-4)
    np.testing.assert_allclose(sel, g["selected_f32_1"], atol=1e-4)
    np.testing.assert_allclose(probs, g["probs_f32"], atol=1e-6, rtol=1e-4)
    half = g["logits"].astype(np.float16).astype(np.float32)
    sel16, probs16 = oracle.logsoftmax_gather(half, sel_idx, True)
    np.testing.assert_allclose(sel16, g["selected_f16_0"], atol=1e-4)
    np.testing.assert_allclose(probs16, g["probs_f16"], atol=1e-3)


@pytest.mark.parametrize("case", ["small", "mid"])
def test_links_restatement_against_reference_model(case):
    """The torch restatement of extract_links (tests/_pyref.py) against the reference model's own function, whose
    output tests/golden/make_golden_links.py recorded."""
    import _pyref

    g = np.load(golden_path("host_extract_links.npz"))
    heads = int(g[f"{case}_heads"])
    q, kl, kr = (torch.from_numpy(g[f"{case}_{n}"]) for n in ("q", "kl", "kr"))
    B, L, E = q.shape
    shape = (B, L, heads, E // heads)
    got = _pyref.extract_links(q.view(shape), kl.view(shape), kr.view(shape), torch.from_numpy(g[f"{case}_gates"]),
                               torch.from_numpy(g[f"{case}_prev"]), 1, torch.from_numpy(g[f"{case}_left_mask"]),
                               torch.from_numpy(g[f"{case}_right_mask"]), torch.from_numpy(g[f"{case}_main_chain"])).numpy()
    want = g[f"{case}_links"]
    assert np.array_equal(np.isfinite(got), np.isfinite(want))
    fin = np.isfinite(want)
    np.testing.assert_allclose(got[fin], want[fin], rtol=1e-5, atol=1e-6)


# ---- criterion glue: the restatements in _pyref.py against the reference criterion's own code --------------------

@pytest.mark.parametrize("tag,strategy", [("none", None), ("number_random", "number-random"), ("cmlm", "cmlm")])
def test_glance_select_restatement_against_reference_criterion(tag, strategy):
    """tests/golden/make_golden_criterion.py ran the reference's glat_function (nat_pcfg_loss.py:193-269) with a
    seeded alignment; the restatement must give the same masks and tokens from the same draws."""
    import _pyref as pyref

    g = np.load(golden_path("host_criterion.npz"))
    t = lambda k: torch.from_numpy(g[k])
    B, L = g["path"].shape
    noise, uniform = pyref.criterion_draws(strategy, int(g[f"{tag}_seed"]), B, L)
    pred = t("logits").argmax(-1)
    got = pyref.glance_select(t("path"), pred, t("tgt"), t("prev"), t("tgt_len"), noise, 0.5, strategy, uniform)
    assert torch.equal(got["matchmask"], t(f"{tag}_matchmask"))
    assert torch.equal(got["keep_word_mask"], t(f"{tag}_keep"))
    assert torch.equal(got["glat_prev_output_tokens"], t(f"{tag}_glat_prev"))
    accu = float(got["same_num"].sum() / t("tgt_len").sum())
    assert abs(accu - float(g[f"{tag}_glat_accu"])) < 1e-6
    assert got["keep_word_mask"].any()
    # the emissions the best-tree operator was handed: EOS column masked except at the last graph node
    lp = torch.log_softmax(t("logits"), -1).gather(-1, t("tgt").unsqueeze(1).expand(-1, L, -1))
    import __graft_entry__ as entry

    syn = entry.load_package().synthetic
    assert torch.equal(syn.eos_mask_(lp.clone(), t("out_len"), t("tgt_len")), t("glance_match"))


def test_force_emit_and_loss_scalar_against_reference_criterion():
    """The reference's _compute_pfcg_loss (nat_pcfg_loss.py:98-145) with a recording loss operator: emissions it
    hands to the loss (EOS + force-emit masks), which entries carry a gradient, the scalar and the invalid count."""
    import _pyref as pyref
    import __graft_entry__ as entry

    pkg = entry.load_package()
    syn = pkg.synthetic
    g = np.load(golden_path("host_criterion.npz"))
    t = lambda k: torch.from_numpy(g[k])
    eos = syn.eos_mask_(t("match_plain").clone(), t("out_len"), t("tgt_len"))
    assert torch.equal(eos, t("plain_loss_match"))
    out, live = pyref.force_emit(eos, t("number_random_matchmask"), t("number_random_keep"))
    assert torch.equal(out, t("force_loss_match"))
    # gradient of -mean_b(loss_b / n_b) over valid sentences w.r.t. the gathered emissions; loss_b is linear with
    # weights loss_w on finite entries
    n = t("tgt_len").float()
    valid = torch.tensor([True, True, False, True, True])
    for tag, masked, alive in (("plain", eos, torch.ones_like(live)), ("force", out, live)):
        want = -(t("loss_w") / n[:, None, None]) / len(n)
        want = want * torch.isfinite(masked) * alive * valid[:, None, None]
        torch.testing.assert_close(t(f"{tag}_match_grad"), want, rtol=1e-6, atol=0)
        # the scalar: invalid sentences zeroed and counted, the others divided by their length, batch mean
        fin = torch.isfinite(masked)
        sent = (torch.where(fin, masked, torch.zeros_like(masked)) * t("loss_w")).sum((1, 2))
        sent[2] = float("-inf")
        import importlib

        sharding = importlib.import_module("pcfg_nat_b200.sharding")
        stats = sharding.local_loss_stats(sent, t("tgt_len"))
        assert abs(float(-stats[0] / stats[1]) - float(g[f"{tag}_loss"])) < 1e-5 * abs(float(g[f"{tag}_loss"]))
        assert int(stats[2]) == int(g[f"{tag}_invalid"]) == 1


@pytest.mark.parametrize("name", ["look_b1_a", "look_b1_b", "greedy_b4", "greedy_b1"])
def test_lookahead_restatement_against_reference_model(name):
    """tests/golden/make_golden_lookahead.py executed the reference's own decoding block
    (models/glat_decomposed_with_link_two_hands_tri_pcfg.py:419-482); the restatement must give the same tokens."""
    import _pyref as pyref

    g = np.load(golden_path("host_lookahead.npz"))
    t = lambda k: torch.from_numpy(g[f"{name}_{k}"])
    rows = pyref.lookahead_decode(t("links"), t("ob"), t("tok"), t("out_len"), t("mask").bool(), 1,
                                  float(g[f"{name}_beta"]), bool(g[f"{name}_lookahead"]))
    want = t("result")
    assert max(len(r) for r in rows) == want.shape[1]
    for r, w in zip(rows, want.tolist()):
        assert r + [1] * (len(w) - len(r)) == w
