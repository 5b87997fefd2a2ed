"""CPU tests of the host side: the C-ABI library loads and exports every declared symbol, the
drop-in operators refuse to run without CUDA (no fallback), support-tree masks equal the
reference's, sentence sharding and the scalar reduction work across gloo ranks."""
import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, golden_path


def test_library_exports_every_declared_symbol(pkg):
    import importlib

    build = importlib.import_module("pcfg_nat_b200.build")
    cabi = importlib.import_module("pcfg_nat_b200._cabi")
    path = build.build()
    header = open(os.path.join(ROOT, "include", "pcfgnat.h")).read()
    declared = set(re.findall(r"\b(pcfgnat_[a-z_0-9]+)\s*\(", header))
    assert declared and declared == set(cabi.SIGNATURES)
    lib = ctypes.CDLL(path)
    for name in declared:
        assert hasattr(lib, name), name
    l = cabi.lib()
    assert l.pcfgnat_version() >= 100
    assert b"max_left" in l.pcfgnat_error_string(-2)
    # argument checks run before any CUDA call, so they can be exercised without a GPU
    assert l.pcfgnat_loss_fwd(None, None, None, None, 1, 32, 10, 3, None, None, None, None) == -2
    assert l.pcfgnat_loss_fwd(None, None, None, None, 1, 32, 10, 1, None, None, None, None) == -1
    assert l.pcfgnat_viterbi(None, None, None, 1, 4, 1, None, None, None, None, None, None) == -1
    assert l.pcfgnat_loss_workspace_bytes(2, 32, 10, 1) >= 2 * 2 * 16 * 12 * 4
    assert l.pcfgnat_loss_fwd_bwd(1, 1, 1, 1, 1, 32, 10, 1, 1, 8, 1, 1, 1, None, None) == -4


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_operators_refuse_to_run_without_cuda(ops):
    with pytest.raises(RuntimeError, match="You need GPU"):
        ops.get_pcfg_kernel()
    ma, lk = torch.zeros(1, 8, 3), torch.zeros(1, 8, 2, 8)
    with pytest.raises(RuntimeError, match="You need GPU"):
        ops.cuda_pcfg_loss(ma, lk, torch.tensor([8]), torch.tensor([3]))
    with pytest.raises(RuntimeError, match="You need GPU"):
        ops.viterbi_decoding(*([torch.zeros(1, dtype=torch.long)] * 7), 1)


def test_public_names_match_the_reference_wrapper(pkg):
    import importlib

    co = importlib.import_module("pcfg_nat_b200.custom_ops")
    for name in ("cuda_pcfg_loss", "cuda_pcfg_best_tree", "cuda_pcfg_viterbi", "dag_logsoftmax_gather_inplace",
                 "viterbi_decoding", "get_pcfg_kernel"):
        assert callable(getattr(co, name))
    k = importlib.import_module("pcfg_nat_b200.custom_ops.pcfg_loss")._Kernel
    for name in ("pcfg_loss", "pcfg_loss_backward", "pcfg_best_tree", "pcfg_viterbi", "logsoftmax_gather",
                 "viterbi_decoding"):
        assert callable(getattr(k, name))


def test_support_tree_masks_equal_reference(pkg):
    g = np.load(golden_path("host_support_tree.npz"))
    for key in g.files:
        kind, ltl, dim = key.split("_")
        if kind != "left":
            continue
        l, r, mc = pkg.support_tree.get_mask(int(dim), int(ltl), 4.0)
        np.testing.assert_array_equal(l.numpy().astype(np.uint8), g[f"left_{ltl}_{dim}"])
        np.testing.assert_array_equal(r.numpy().astype(np.uint8), g[f"right_{ltl}_{dim}"])
        np.testing.assert_array_equal(mc.numpy().astype(np.uint8), g[f"main_{ltl}_{dim}"])
    assert pkg.support_tree.graph_length(20, 4.0, 1) == 162  # 8 * src + 2


def test_synthetic_links_are_normalised_and_masked(syn):
    b = syn.make_batch("tiny_loss")
    lk = b.links
    assert lk.shape == (2, 32, 2, 32)
    rows = torch.logsumexp(lk.reshape(2, 32, -1), -1)
    live = torch.isfinite(rows)
    assert live[:, 1:31:2].all() and not live[:, 0::2].any() and not live[:, 31].any()
    torch.testing.assert_close(rows[live], torch.zeros(int(live.sum())), atol=1e-5, rtol=0)
    assert torch.isinf(lk[:, :, :, 0::2]).all()  # right children are main-chain (odd) nodes only
    a = syn.make_batch("tiny_loss")
    assert torch.equal(a.links, lk) and torch.equal(a.targets, b.targets)  # seeded
    for name in ("train_batch", "viterbi_b64"):
        w = syn.WORKLOADS[name]
        t = syn.make_batch(syn.Workload(name, batch=w.batch, vocab=50, hidden=4, src_min=w.src_min, src_max=w.src_max,
                                        emissions="logits", kind=w.kind), seed=0)
        assert ((t.target_length >= 2) & (t.target_length <= t.output_length - 2)).all()
        assert (t.output_length % 2 == 0).all() and int(t.output_length.max()) == t.L


def test_shard_sentences_partitions_and_balances(pkg):
    sh = pkg.sharding
    costs = [float((i * 37) % 23 + 1) for i in range(90)]
    for ws in (1, 2, 4, 8):
        shards = sh.shard_sentences(costs, ws)
        flat = sorted(i for s in shards for i in s)
        assert flat == list(range(90))
        loads = [sum(costs[i] for i in s) for s in shards]
        assert max(loads) - min(loads) <= max(costs)
    assert sh.shard_sentences([1.0], 4) == [[0], [], [], []]


def test_local_loss_stats_mirror_the_criterion(pkg):
    loss = torch.tensor([-10.0, float("-inf"), -6.0, float("nan")])
    tl = torch.tensor([5, 3, 2, 4])
    s = pkg.sharding.local_loss_stats(loss, tl)
    assert s.tolist() == [-5.0, 4.0, 2.0]
    # the criterion: invalid -> 0, then -(loss / n).mean()
    l2 = loss.clone()
    l2[torch.isinf(l2) | torch.isnan(l2)] = 0
    want = -(l2 / tl).mean()
    got, nsent, ninv = pkg.sharding.reduce_loss(loss, tl)
    assert float(got) == float(want) and int(nsent) == 4 and int(ninv) == 2


_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
import __graft_entry__ as entry
pkg = entry.load_package()
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}", rank=int(sys.argv[3]), world_size=2)
rank = dist.get_rank()
g = torch.Generator().manual_seed(0)
loss = -torch.rand(11, generator=g) * 30
loss[4] = float("-inf")
tl = torch.randint(2, 9, (11,), generator=g)
shards = pkg.sharding.shard_sentences(pkg.sharding.sentence_cost(tl * 8, tl), 2)
mine = torch.tensor(shards[rank])
got, nsent, ninv = pkg.sharding.reduce_loss(loss[mine], tl[mine])
full, _, _ = pkg.sharding.local_loss_stats(loss, tl)
want = -full / 11
assert abs(float(got) - float(want)) < 1e-5, (float(got), float(want))
assert int(nsent) == 11 and int(ninv) == 1
dist.destroy_process_group()
print("ok", rank)
"""


def test_reduce_loss_across_two_gloo_ranks(tmp_path):
    import socket

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, str(port), str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    for p in procs:
        out, _ = p.communicate(timeout=180)
        assert p.returncode == 0 and "ok" in out, out


def _plan(l, lengths, b0, b1, L, max_copies):
    lengths = np.ascontiguousarray(lengths, dtype=np.int64)
    runs = np.zeros((max(b1 - b0, 1), 2), dtype=np.int64)
    n = l.pcfgnat_plan_real_rows(lengths.ctypes.data, b0, b1, L, max_copies, runs.ctypes.data, runs.shape[0])
    assert n >= 0, n
    return [(int(a), int(c)) for a, c in runs[:n]]


def test_plan_of_the_real_row_copies(pkg):
    """pcfgnat_plan_real_rows (the host arithmetic behind pcfgnat_copy_real_rows): every real row is covered exactly
    once, runs are disjoint and ascending, at most max_copies of them, and joining costs no more padding rows than
    the cheapest choice of gaps."""
    import importlib

    l = importlib.import_module("pcfg_nat_b200._cabi").lib()
    # a worked case: runs [0,3) [12,36) [48,60) [72,77); two copies close the gaps of 9 and one of the 12s
    lengths = [3, 12, 12, 0, 20, -4, 5]
    assert _plan(l, lengths, 0, 7, 12, 0) == [(0, 3), (12, 24), (48, 12), (72, 5)]
    assert _plan(l, lengths, 0, 7, 12, 2) == [(0, 60), (72, 5)]
    assert _plan(l, lengths, 1, 3, 12, 0) == [(12, 24)]
    assert _plan(l, [0, 0, 0], 0, 3, 8, 4) == []
    assert l.pcfgnat_plan_real_rows(None, 0, 2, 8, 0, None, 0) == -1
    rng = np.random.default_rng(0)
    for _ in range(200):
        B, L = int(rng.integers(1, 40)), int(rng.integers(1, 30))
        lengths = rng.integers(-2, L + 3, size=B)
        k = int(rng.integers(0, 12))
        free = _plan(l, lengths, 0, B, L, 0)
        runs = _plan(l, lengths, 0, B, L, k)
        real = np.zeros(B * L, dtype=bool)
        for b in range(B):
            real[b * L: b * L + int(np.clip(lengths[b], 0, L))] = True
        sent = np.zeros(B * L, dtype=int)
        for first, rows in runs:
            assert rows > 0
            sent[first: first + rows] += 1
        assert sent.max(initial=0) <= 1 and (sent[real] == 1).all()
        assert all(runs[i][0] + runs[i][1] < runs[i + 1][0] for i in range(len(runs) - 1))
        assert len(runs) <= len(free) and (k == 0 or len(runs) <= max(k, 0) or len(free) <= k)
        if k and len(free) > k:  # the joined gaps are the smallest ones
            gaps = sorted(free[i + 1][0] - (free[i][0] + free[i][1]) for i in range(len(free) - 1))
            assert len(runs) == k and int(sent.sum() - real.sum()) == sum(gaps[: len(free) - k])
        else:
            assert runs == free
