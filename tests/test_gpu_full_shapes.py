"""Parity at the full shapes of the benchmark's workloads, through the step objects the benchmark times.

Every case builds the workload with ``synthetic.make_batch`` at the benchmark's seed, makes the step exactly
as ``bench.make_step`` does (CUDA-graph replay; the second load goes over the copy stream with
``overlap=True``) and compares with the CPU oracle:

* emissions of the fused projection against a float32 torch projection of the same fp16 inputs: 2e-3 abs;
* per-sentence loss against the oracle fed the float32 torch emissions: 1e-4 relative;
* both gradients against the oracle on the kernel's own emissions (identical fp32 DP inputs): 1e-3 relative;
* best tree, Viterbi token ids, counts and predicted lengths: exact (max-plus / arg-max on identical inputs);
  the best tree compares sums of the inside table, so the oracle walks the table the kernels built (which a
  second test holds bit-identical to the reference kernels' table).

Where the build of the unmodified reference kernels travelled along, the shapes with at most 128 main-chain
nodes are also compared with those kernels live.
"""
import importlib
import os

import numpy as np
import pytest
import torch

import bench
import oracle
import _pyref as pyref

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _runtime():
    return importlib.import_module("pcfg_nat_b200.runtime")


def _torch_log_probs(batch):
    """float32 log-softmax of the float32 projection of the fp16 inputs, [B, L, V] on the device."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        h = batch.hidden.to(DEV).float().view(-1, batch.hidden.shape[-1])
        w = batch.weight.to(DEV).float()
        return torch.log_softmax(h @ w.t(), -1).view(batch.B, batch.L, -1)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def _real_rows(batch):
    return (torch.arange(batch.L)[None, :] < batch.output_length[:, None]).to(DEV)


def _clone(out):
    if isinstance(out, dict):
        return {k: v.clone() for k, v in out.items()}
    if isinstance(out, (tuple, list)):
        return type(out)(_clone(o) for o in out)
    return out.clone()


def _run_twice(step, host):
    """Capture + replay as the benchmark does: a plain load (one projection graph), then an overlapped load from
    pinned memory (the sentences projected in two groups).  Returns both results.  The two differ in the last
    ulp of the emissions: the tile schedule of a group merges the softmax partials of a row in another order."""
    outs = []
    for overlap in (False, True):
        step.load(*host, overlap=overlap)
        out = step.run()
        torch.cuda.synchronize()
        outs.append(_clone(out))
    return outs


def _rel_close(a, b, rtol, atol=0.0):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    assert np.array_equal(np.isfinite(a), np.isfinite(b))
    fin = np.isfinite(a)
    err = np.abs(a[fin] - b[fin])
    assert (err <= atol + rtol * np.abs(b[fin])).all(), float(err.max())


@pytest.mark.parametrize("wname", ["train_batch", "long_seq", "train_batch_model_graph"])
def test_loss_step_full_shape_against_oracle(pkg, ops, syn, wname):
    batch = syn.make_batch(wname, seed=0)
    weight = batch.weight.to(DEV)
    step, host = bench.make_step(_runtime(), batch, weight, DEV, True, 2)
    first = None
    for overlap in (False, True):
        step.load(*host, overlap=overlap)
        stats, mg, lg, loss = step.run()
        torch.cuda.synchronize()
        if first is None:
            first = [t.clone() for t in (stats, mg, lg, loss)]
    # replay after the overlapped load against the capture run: the overlapped load projects the sentences in two
    # groups, whose tile schedule merges the softmax partials of a row in another order (last-ulp differences)
    for a, b in zip(first, (stats, mg, lg, loss)):
        torch.testing.assert_close(b, a, rtol=1e-3, atol=2e-5)
    torch.testing.assert_close(loss, first[3], rtol=1e-6, atol=0)
    assert ops.read_status(DEV) == 0
    ol, tl = batch.output_length.numpy(), batch.target_length.numpy()
    lk = batch.links.numpy()

    # emissions: fused projection against the float32 torch projection
    lp = _torch_log_probs(batch)
    want = lp.gather(2, batch.targets.to(DEV)[:, None, :].expand(-1, batch.L, -1)).contiguous()
    del lp
    syn.eos_mask_(want, batch.output_length, batch.target_length)
    em = ops.proj_logsoftmax_gather(step.hidden, weight, step.targets, step.output_length, step.target_length)["match"]
    real = _real_rows(batch)
    assert torch.equal(torch.isfinite(em[real]), torch.isfinite(want[real]))
    fin = torch.isfinite(want) & real[:, :, None]
    assert float((em[fin] - want[fin]).abs().max()) < 2e-3

    # loss against the oracle fed the torch emissions
    So, _ = oracle.pcfg_loss(want.cpu().numpy(), lk, ol, tl)
    assert np.isfinite(So[:, 0, 0]).all()
    np.testing.assert_allclose(loss.cpu().numpy(), So[:, 0, 0], rtol=1e-4)
    want_stat = float((torch.from_numpy(So[:, 0, 0]).double() / batch.target_length).sum())
    assert abs(float(stats[0]) - want_stat) <= 1e-4 * abs(want_stat)
    assert int(stats[1]) == batch.B and int(stats[2]) == 0

    # gradients against the oracle on the kernel's own emissions
    em_np = em.cpu().numpy()
    Sk, Ck = oracle.pcfg_loss(em_np, lk, ol, tl)
    mgo, lgo = oracle.pcfg_loss_backward(np.ones(batch.B, np.float32), Sk, Ck, em_np, lk, ol, tl)
    np.testing.assert_allclose(mg.cpu().numpy(), mgo, rtol=1e-3, atol=2e-6)
    np.testing.assert_allclose(lg.cpu().numpy(), lgo, rtol=1e-3, atol=2e-6)


@pytest.mark.parametrize("wname", ["glance", "glance_train"])
def test_glance_step_full_shape_against_oracle(pkg, ops, syn, wname):
    batch = syn.make_batch(wname, seed=0)
    weight = batch.weight.to(DEV)
    step, host = bench.make_step(_runtime(), batch, weight, DEV, True, 2)
    (tree, ll, am, glance), (tree2, ll2, am2, _) = _run_twice(step, host)
    noise = step.noise.cpu()  # the draws of the last run; the sampler is checked on that run's outputs below
    assert ops.read_status(DEV) == 0
    torch.testing.assert_close(ll2, ll, rtol=1e-6, atol=0)
    assert (tree2 == tree).float().mean() > 0.999 and (am2 == am).float().mean() > 0.999
    ol, tl = batch.output_length.numpy(), batch.target_length.numpy()
    lk = batch.links.numpy()
    k = ops.get_pcfg_kernel()
    real = _real_rows(batch)

    lp = _torch_log_probs(batch)
    want = lp.gather(2, batch.targets.to(DEV)[:, None, :].expand(-1, batch.L, -1)).contiguous()
    # arg-max token: the kernel's choice is a maximum of the float32 row to within the projection's tolerance
    at_choice = lp.gather(2, am[:, :, None]).squeeze(-1)
    assert float((lp.max(-1)[0] - at_choice)[real].max()) < 2e-3
    del lp
    syn.eos_mask_(want, batch.output_length, batch.target_length)
    em = ops.proj_logsoftmax_gather(step.hidden, weight, step.targets, step.output_length, step.target_length,
                                    want_max=True)
    assert torch.equal(em["argmax"], am)
    fin = torch.isfinite(want) & real[:, :, None]
    assert float((em["match"][fin] - want[fin]).abs().max()) < 2e-3

    # sentence log-likelihood against the oracle fed the torch emissions
    So, _ = oracle.pcfg_loss(want.cpu().numpy(), lk, ol, tl)
    np.testing.assert_allclose(ll.cpu().numpy(), So[:, 0, 0], rtol=1e-4)

    # inside table on the kernel's emissions: 1e-5 against the oracle's; the tree exact on that table
    em_np = em["match"].cpu().numpy()
    S, _ = k.pcfg_loss(em["match"], step.links, step.output_length, step.target_length, 1)
    assert torch.equal(S[:, 0, 0], ll)
    Sk, Ck = oracle.pcfg_loss(em_np, lk, ol, tl)
    _rel_close(S.cpu().numpy(), Sk, 1e-5, 1e-5)
    want_tree = oracle.pcfg_best_tree(S.cpu().numpy(), Ck, em_np, lk, ol, tl)
    assert np.array_equal(tree.cpu().numpy(), want_tree)

    # the sampler on the step's own draws
    prev = host[-1]
    glance2 = step.out[3]
    want_g = pyref.glance_select(tree2.cpu(), am2.cpu(), batch.targets, prev, batch.target_length, noise, step.context_p)
    for key, val in want_g.items():
        assert torch.equal(glance2[key].cpu(), val), key


@pytest.mark.parametrize("wname", ["viterbi_b64", "viterbi_b1"])
def test_decode_step_full_shape_against_oracle(pkg, ops, syn, wname):
    batch = syn.make_batch(wname, seed=0)
    weight = batch.weight.to(DEV)
    step, host = bench.make_step(_runtime(), batch, weight, DEV, True, 2)
    (tokens, count, pred), (tokens2, count2, pred2) = _run_twice(step, host)
    assert ops.read_status(DEV) == 0
    assert (pred2 == pred).float().mean() > 0.95 and (count2 == count).float().mean() > 0.95
    ol = batch.output_length.numpy()
    real = _real_rows(batch)

    lp = _torch_log_probs(batch)
    ob_t = lp.max(-1)[0]
    em = ops.proj_logsoftmax_gather(step.hidden, weight, None, step.output_length, None, want_max=True)
    assert float((em["max_lprob"] - ob_t)[real].abs().max()) < 2e-3
    at_choice = lp.gather(2, em["argmax"][:, :, None]).squeeze(-1)
    assert float((ob_t - at_choice)[real].max()) < 2e-3
    del lp

    # Viterbi is max-plus: on the kernel's own emissions everything downstream is exact
    ob_k, tok_k = em["max_lprob"].cpu(), em["argmax"].cpu()
    So, Ro, Lo, Mo = oracle.pcfg_viterbi(ob_k.numpy(), batch.links.numpy(), ol)
    sc = torch.from_numpy(So[:, 1, :]) / torch.arange(batch.L // 4).unsqueeze(0)
    sc = torch.where(torch.isnan(sc), torch.full_like(sc, float("-inf")), sc)
    want_pred = sc[:, 1:].max(-1)[1] + 1
    assert torch.equal(pred.cpu(), want_pred)
    want = oracle.viterbi_decoding_lists(want_pred.numpy(), ol, Lo, Ro, Mo, tok_k.numpy(),
                                         batch.left_tree_mask.long().numpy(), 1)
    for i, row in enumerate(want):
        assert int(count[i]) == len(row)
        assert tokens[i, :len(row)].cpu().tolist() == row
        assert (tokens[i, len(row):] == 1).all()
    k = ops.get_pcfg_kernel()
    S, R, Lt, Mt = k.pcfg_viterbi(em["max_lprob"], step.links, step.output_length, 1)
    assert np.array_equal(S.cpu().numpy().view(np.int32), So.view(np.int32))
    assert np.array_equal(R.cpu().numpy(), Ro) and np.array_equal(Lt.cpu().numpy(), Lo)
    assert np.array_equal(Mt.cpu().numpy(), Mo)


@pytest.mark.parametrize("wname", ["train_batch", "glance", "viterbi_b64"])
def test_full_shape_live_against_reference_kernels(pkg, ops, syn, wname):
    """The benchmark's shapes with at most 128 main-chain nodes per sentence (one row segment per sentence in
    every reference launch, so none of its inter-block waits depends on another block) against the unmodified
    reference kernels on the same device tensors."""
    from oracle.build_ref import load_ref, ref_so_path

    if not os.path.isfile(ref_so_path()):
        pytest.skip("reference extension not built")
    ref = load_ref()
    batch = syn.make_batch(wname, seed=0)
    assert batch.L <= 256
    k = ops.get_pcfg_kernel()
    weight = batch.weight.to(DEV)
    hid, lk = batch.hidden.to(DEV), batch.links.to(DEV)
    ol = batch.output_length.to(DEV)
    if batch.workload.kind == "viterbi":
        em = ops.proj_logsoftmax_gather(hid, weight, None, ol, None, want_max=True)
        for x, y in zip(k.pcfg_viterbi(em["max_lprob"], lk, ol, 1), ref.pcfg_viterbi(em["max_lprob"], lk, ol, 1)):
            assert torch.equal(x.view(torch.int32) if x.dtype == torch.float32 else x,
                               y.view(torch.int32) if y.dtype == torch.float32 else y)
        return
    tl, tg = batch.target_length.to(DEV), batch.targets.to(DEV)
    ma = ops.proj_logsoftmax_gather(hid, weight, tg, ol, tl)["match"]
    Sr, Cr = ref.pcfg_loss(ma, lk, ol, tl, 1)
    S, C = k.pcfg_loss(ma, lk, ol, tl, 1)
    assert torch.equal(S.view(torch.int32), Sr.view(torch.int32))
    assert torch.equal(C.view(torch.int32), Cr.view(torch.int32))
    assert torch.equal(k.pcfg_best_tree(S, C, ma, lk, ol, tl, 1), ref.pcfg_best_tree(Sr, Cr, ma, lk, ol, tl, 1))
    mgr, lgr = ref.pcfg_loss_backward(torch.ones(batch.B, device=DEV), Sr, Cr, ma, lk, ol, tl, 1)
    loss, mg, lg = k.pcfg_loss_fwd_bwd(ma, lk, ol, tl)
    torch.testing.assert_close(loss, Sr[:, 0, 0], rtol=1e-5, atol=0)
    torch.testing.assert_close(mg, mgr, rtol=1e-3, atol=2e-6)
    torch.testing.assert_close(lg, lgr, rtol=1e-3, atol=2e-6)


def test_projection_backward_full_shape_against_float32_autograd(pkg, ops, syn):
    """train_batch through LossStep(proj_backward=True): d-logits of the 10 804 real nodes, then the two tensor-core
    products, against float32 autograd of log_softmax(hidden @ weight.T) fed the step's own emission gradient
    (1.5e-2 of the Frobenius norm: bf16 d-logits and operands); padding rows of d hidden exactly zero."""
    batch = syn.make_batch("train_batch", seed=0)
    weight = batch.weight.to(DEV)
    step = _runtime().LossStep(weight, batch.B, batch.L, batch.T, DEV, use_graph=True, proj_backward=True)
    step.load(batch.hidden, batch.links, batch.output_length, batch.targets, batch.target_length)
    stats, mg, lg, loss, d_hidden, d_weight = step.run()
    torch.cuda.synchronize()
    assert ops.read_status(DEV) == 0 and torch.isfinite(loss).all()
    rows = _real_rows(batch)
    assert float(d_hidden[~rows].abs().sum()) == 0.0
    h32 = batch.hidden.float().to(DEV).requires_grad_(True)
    w32 = batch.weight.float().to(DEV).requires_grad_(True)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        lp = torch.log_softmax(h32 @ w32.t(), -1)
        ref = lp.gather(2, batch.targets.to(DEV)[:, None, :].expand(-1, batch.L, -1))
        g = torch.where(torch.isfinite(mg) & rows[:, :, None], mg, torch.zeros_like(mg))
        # entries the forward masked (EOS) or did not project get no gradient
        syn.eos_mask_(ref, batch.output_length.to(DEV), batch.target_length.to(DEV))
        g = torch.where(torch.isfinite(ref), g, torch.zeros_like(g))
        (torch.where(torch.isfinite(ref), ref, torch.zeros_like(ref)) * g).sum().backward()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    for got, want in ((d_hidden.float(), h32.grad), (d_weight.float(), w32.grad)):
        assert float((got - want).norm() / want.norm()) < 1.5e-2
