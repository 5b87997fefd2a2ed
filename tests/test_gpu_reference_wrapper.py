"""The extension-level contract: the reference's own, UNMODIFIED Python wrapper
(fs_plugins/custom_ops/pcfg_loss.py) running on top of this package's extension object.

The wrapper keeps its extension in the module global ``pcfg_kernel`` (pcfg_loss.py:15-23) and only compiles
when that is None; setting it to ``get_pcfg_kernel()`` of this package is the whole integration.  The five
public operators of the wrapper are then run and compared with the CPU oracle.  The wrapper file is loaded
from the byte-for-byte copy that oracle/build_ref.py stages beside the built reference extension (a
git-ignored build product), or from the reference checkout where that is mounted.
"""
import importlib.util
import os

import numpy as np
import pytest
import torch

import oracle
from oracle import build_ref

DEV = "cuda:0"


def _wrapper_file():
    p = build_ref.ref_wrapper_path()
    if os.path.isfile(p):
        return p
    root = build_ref.find_reference()
    if root is not None:
        return os.path.join(root, "fs_plugins", "custom_ops", "pcfg_loss.py")
    return None


def test_staged_wrapper_is_the_reference_file():
    root, staged = build_ref.find_reference(), build_ref.ref_wrapper_path()
    if root is None or not os.path.isfile(staged):
        pytest.skip("needs the reference checkout and the staged copy")
    with open(os.path.join(root, "fs_plugins", "custom_ops", "pcfg_loss.py"), "rb") as f, open(staged, "rb") as g:
        assert f.read() == g.read()


@pytest.fixture(scope="module")
def ref_wrapper(ops):
    path = _wrapper_file()
    if path is None:
        pytest.skip("reference wrapper not available")
    spec = importlib.util.spec_from_file_location("reference_pcfg_loss_wrapper", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.pcfg_kernel = ops.get_pcfg_kernel()  # the wrapper's loader returns it as is (pcfg_loss.py:22-23)
    return mod


@pytest.mark.gpu
def test_unmodified_wrapper_loss_and_backward(ref_wrapper, ops, syn):
    w = syn.Workload("wrap", batch=7, vocab=100, hidden=8, src_min=2, src_max=21, emissions="logits")
    b = syn.make_batch(w, seed=1)
    ma = syn.reference_match_all(b)
    ol, tl = b.output_length.numpy(), b.target_length.numpy()
    So, Co = oracle.pcfg_loss(ma.numpy(), b.links.numpy(), ol, tl)
    go = np.linspace(0.5, 2.0, b.B).astype(np.float32)
    mgo, lgo = oracle.pcfg_loss_backward(go, So, Co, ma.numpy(), b.links.numpy(), ol, tl)
    mat = ma.to(DEV).requires_grad_(True)
    lkt = b.links.to(DEV).requires_grad_(True)
    loss = ref_wrapper.cuda_pcfg_loss(mat, lkt, b.output_length.to(DEV), b.target_length.to(DEV))
    np.testing.assert_allclose(loss.detach().cpu().numpy(), So[:, 0, 0], rtol=1e-4)
    (loss * torch.as_tensor(go, device=DEV)).sum().backward()
    np.testing.assert_allclose(mat.grad.cpu().numpy(), mgo, rtol=1e-3, atol=2e-6)
    np.testing.assert_allclose(lkt.grad.cpu().numpy(), lgo, rtol=1e-3, atol=2e-6)
    # without a gradient the wrapper only runs the inside pass
    loss2 = ref_wrapper.cuda_pcfg_loss(ma.to(DEV), b.links.to(DEV), b.output_length.to(DEV), b.target_length.to(DEV))
    assert torch.equal(loss2, loss.detach())


@pytest.mark.gpu
def test_unmodified_wrapper_best_tree(ref_wrapper, ops, syn):
    w = syn.Workload("wrap", batch=4, vocab=100, hidden=8, src_min=30, src_max=40, emissions="logits")
    b = syn.make_batch(w, seed=2)
    ma = syn.reference_match_all(b)
    ol, tl = b.output_length.numpy(), b.target_length.numpy()
    tree, ll = ref_wrapper.cuda_pcfg_best_tree(ma.to(DEV), b.links.to(DEV), b.output_length.to(DEV),
                                               b.target_length.to(DEV))
    So, Co = oracle.pcfg_loss(ma.numpy(), b.links.numpy(), ol, tl)
    np.testing.assert_allclose(ll.cpu().numpy(), So[:, 0, 0], rtol=1e-4)
    # arg-max over sums of the table: walk the table the kernels built (equal to the oracle's to 1e-5)
    S, _ = ops.get_pcfg_kernel().pcfg_loss(ma.to(DEV), b.links.to(DEV), b.output_length.to(DEV), b.target_length.to(DEV), 1)
    want = oracle.pcfg_best_tree(S.cpu().numpy(), Co, ma.numpy(), b.links.numpy(), ol, tl)
    assert np.array_equal(tree.cpu().numpy(), want)
    assert tree.dtype == torch.int64


@pytest.mark.gpu
def test_unmodified_wrapper_viterbi_and_decoding(ref_wrapper, ops, syn):
    w = syn.Workload("wrapv", batch=1, vocab=200, hidden=8, src_min=12, src_max=12, emissions="logits", kind="viterbi")
    b = syn.make_batch(w, seed=3)
    ob, tok = torch.log_softmax(b.logits, -1).max(-1)
    scores, R, Lt, Mt = ref_wrapper.cuda_pcfg_viterbi(ob.to(DEV), b.links.to(DEV), b.output_length.to(DEV))
    So, Ro, Lo, Mo = oracle.pcfg_viterbi(ob.numpy(), b.links.numpy(), b.output_length.numpy())
    assert np.array_equal(scores.cpu().numpy().view(np.int32), So[:, 1, :].view(np.int32))
    assert np.array_equal(R.cpu().numpy(), Ro) and np.array_equal(Lt.cpu().numpy(), Lo)
    assert np.array_equal(Mt.cpu().numpy(), Mo)
    sc = scores / torch.arange(b.L // 4, device=DEV).unsqueeze(0)
    sc.masked_fill_(sc.isnan(), float("-inf"))
    pred = sc[:, 1:].max(-1)[1] + 1
    # the model moves the traces to the host first (models/glat_decomposed_with_link_two_hands_tri_pcfg.py:500)
    out = ref_wrapper.viterbi_decoding(pred.long(), b.output_length.to(DEV), Lt.cpu().long(), R.cpu().long(),
                                       Mt.cpu().long(), tok.to(DEV).long(), b.left_tree_mask.long(), 1)
    want = oracle.viterbi_decoding(pred.cpu().numpy(), b.output_length.numpy(), Lo, Ro, Mo, tok.numpy(),
                                   b.left_tree_mask.long().numpy(), 1)
    assert out.dtype == torch.float32
    assert np.array_equal(out.cpu().numpy(), want)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_unmodified_wrapper_logsoftmax_gather(ref_wrapper, ops, dtype):
    g = torch.Generator().manual_seed(7)
    B, L, V, T = 3, 10, 1000, 6
    logits = torch.randn(B, L, V, generator=g).to(dtype)
    tgt = torch.randint(0, V, (B, T), generator=g)
    sel = tgt[:, None, :].expand(-1, L, -1)
    want, probs = oracle.logsoftmax_gather(logits.float().numpy(), sel.numpy(), True)
    x = logits.to(DEV).requires_grad_(True)
    y = x * 1  # a non-leaf the operator may overwrite
    out, selected = ref_wrapper.dag_logsoftmax_gather_inplace(y, sel.to(DEV))
    tol = 2e-5 if dtype == torch.float32 else 2e-3
    np.testing.assert_allclose(selected.detach().cpu().numpy(), want, rtol=0, atol=tol)
    np.testing.assert_allclose(out.detach().float().cpu().numpy(), probs, rtol=0, atol=2e-3 if dtype == torch.float16 else 1e-6)
    gsel = torch.randn(B, L, T, generator=g)
    selected.backward(gsel.to(DEV))
    p = torch.from_numpy(probs)
    want_grad = -p * gsel.sum(-1, keepdim=True)
    want_grad.scatter_add_(-1, sel.contiguous(), gsel)
    np.testing.assert_allclose(x.grad.float().cpu().numpy(), want_grad.numpy(), rtol=0,
                               atol=1e-5 if dtype == torch.float32 else 5e-3)
