"""The allocation-free loss entry point (pcfgnat_loss_fwd_bwd_static) against the regular one.

Some hosts of this library cannot supply a workspace: an FFI caller that merely forwards device
pointers it received from another framework, or a process that owns all device memory through
its own arena and forbids cudaMalloc in libraries.  For them the two DP tables sit in a fixed
array inside the library.  The test calls the entry point through the C ABI twice in a row on
different batches (the array still holds the first call's tables during the second) and checks
each result against pcfgnat_loss_fwd_bwd with a caller-supplied workspace.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import importlib

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _call_both(cabi, syn, workload, seed):
    b = syn.make_batch(workload, seed=seed)
    ma = syn.reference_match_all(b).to(DEV).contiguous()
    lk = b.links.to(DEV).contiguous()
    ol, tl = b.output_length.to(DEV), b.target_length.to(DEV)
    B, L, T = ma.shape
    lib = cabi.lib()
    stream = torch.cuda.current_stream(DEV).cuda_stream

    def outputs():
        return (torch.empty(B, device=DEV), torch.empty_like(ma), torch.empty_like(lk))

    loss_a, mg_a, lg_a = outputs()
    nbytes = lib.pcfgnat_loss_workspace_bytes(B, L, T, 1)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    rc = lib.pcfgnat_loss_fwd_bwd(ma.data_ptr(), lk.data_ptr(), ol.data_ptr(), tl.data_ptr(), B, L, T, 1, ws.data_ptr(),
                                  nbytes, loss_a.data_ptr(), mg_a.data_ptr(), lg_a.data_ptr(), None, stream)
    assert rc == 0
    loss_b, mg_b, lg_b = outputs()
    rc = lib.pcfgnat_loss_fwd_bwd_static(ma.data_ptr(), lk.data_ptr(), ol.data_ptr(), tl.data_ptr(), B, L, T, 1,
                                         loss_b.data_ptr(), mg_b.data_ptr(), lg_b.data_ptr(), None, stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.isfinite(loss_a).all()
    torch.testing.assert_close(loss_b, loss_a, rtol=1e-4, atol=0)   # loss tolerance of the parity tests
    torch.testing.assert_close(mg_b, mg_a, rtol=1e-3, atol=2e-6)    # gradient tolerance of the parity tests
    torch.testing.assert_close(lg_b, lg_a, rtol=1e-3, atol=2e-6)


def test_static_scratch_entry_point_matches_workspace_entry_point(pkg, syn):
    cabi = importlib.import_module("pcfg_nat_b200._cabi")
    first = syn.Workload("na1", batch=5, vocab=60, hidden=8, src_min=6, src_max=30, emissions="logits")
    second = syn.Workload("na2", batch=3, vocab=60, hidden=8, src_min=10, src_max=20, emissions="logits")
    _call_both(cabi, syn, first, seed=21)
    _call_both(cabi, syn, second, seed=22)  # the array still holds the (larger) tables of the first call
    # a problem whose tables exceed the fixed array is refused, nothing is allocated instead
    lib = cabi.lib()
    big = lib.pcfgnat_loss_fwd_bwd_static(1, 1, 1, 1, 4096, 512, 128, 1, 1, 1, 1, None, None)
    assert big == -5 and b"too large" in lib.pcfgnat_error_string(big)


def _static_call(lib, ma, lk, ol, tl, status=None):
    B, L, T = ma.shape
    loss, mg, lg = torch.full((B,), 7.0, device=DEV), torch.full_like(ma, 7.0), torch.full_like(lk, 7.0)
    rc = lib.pcfgnat_loss_fwd_bwd_static(ma.data_ptr(), lk.data_ptr(), ol.data_ptr(), tl.data_ptr(), B, L, T, 1,
                                         loss.data_ptr(), mg.data_ptr(), lg.data_ptr(),
                                         None if status is None else status.data_ptr(),
                                         torch.cuda.current_stream(DEV).cuda_stream)
    torch.cuda.synchronize()
    return rc, loss, mg, lg


@pytest.mark.parametrize("family", ["auto", "balanced", "rows"])
def test_static_entry_point_with_an_invalid_sentence_after_a_valid_batch(pkg, syn, monkeypatch, family):
    """The shared array holds the previous call's tables when a batch with an out-of-range length comes in: the
    skipped sentence must come back with -inf loss, exactly zero gradients and the status bit, on the kernel
    family the library picks and on a forced one; the other sentences as the workspace entry point gives them."""
    cabi = importlib.import_module("pcfg_nat_b200._cabi")
    lib = cabi.lib()
    if family != "auto":
        monkeypatch.setenv("PCFGNAT_DP_KERNEL", family)
    w = syn.Workload("na3", batch=4, vocab=60, hidden=8, src_min=6, src_max=24, emissions="logits")
    _call_both(cabi, syn, w, seed=23)  # leaves its tables in the array
    b = syn.make_batch(w, seed=24)
    ma = syn.reference_match_all(b).to(DEV).contiguous()
    lk = b.links.to(DEV).contiguous()
    ol, tl = b.output_length.clone(), b.target_length.clone()
    ol[1] = b.L + 2  # more graph nodes than the tensors hold
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc, loss, mg, lg = _static_call(lib, ma, lk, ol.to(DEV), tl.to(DEV), status)
    assert rc == 0
    assert int(status.item()) & 1  # PCFGNAT_STATUS_BAD_LENGTH
    assert loss[1] == float("-inf") and (mg[1] == 0).all() and (lg[1] == 0).all()
    good = [0, 2, 3]
    sub = b.select(good)
    rc2, loss2, mg2, lg2 = _static_call(lib, ma[good].contiguous(), lk[good].contiguous(), sub.output_length.to(DEV),
                                        sub.target_length.to(DEV))
    assert rc2 == 0
    torch.testing.assert_close(loss[good], loss2, rtol=1e-5, atol=0)
    torch.testing.assert_close(mg[good], mg2, rtol=1e-4, atol=1e-7)
    torch.testing.assert_close(lg[good], lg2, rtol=1e-4, atol=1e-7)


def test_static_entry_point_accepts_an_empty_batch(pkg):
    cabi = importlib.import_module("pcfg_nat_b200._cabi")
    rc = cabi.lib().pcfgnat_loss_fwd_bwd_static(None, None, None, None, 0, 16, 4, 1, None, None, None, None,
                                                torch.cuda.current_stream(DEV).cuda_stream)
    assert rc == 0
