"""Device-side failure reporting and robustness of the step before routing.  Needs a B200.

* A bounded wait inside the tcgen05 GEMM that runs out is reported through the per-device status word, the kernel
  returns, the next entry point refuses with HEXA_ERR_DEVICE until the word is cleared, and the device keeps
  working.  The wait is made to run out without any fault: the kernel's producer is told (hexa_set_tc_debug bit 2)
  to neither load nor signal, and the limit is lowered to a few milliseconds.  The reference's answer to a device
  error is printf + exit(1) (hexa_moe_cuda/hexa_moe/kernels/esmm_half.cu:27-36).
* The fused gate step gives valid ids for rows of NaN / inf logits (the reference chain F.softmax -> torch.topk
  survives such rows too, cascaded_moe.py:568-598) and is bit-identical from run to run.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from hexa_moe_b200 import ops as _ops
    return _ops


def _case(ops, n_out):
    from hexa_moe_b200 import _lib as L
    T, k, E, d = 1024, 2, 4, 256
    g = torch.Generator().manual_seed(n_out)
    ids = torch.topk(torch.randn(T, E, generator=g), k, dim=1).indices.to(torch.int32).cuda()
    r = ops.route(ids, E)
    xs = ops.gather_rows(torch.randn(T, d, generator=g).bfloat16().cuda(), r)
    w = (torch.randn(E, n_out, d, generator=g) / 16).bfloat16().cuda()
    return L, r, xs, w


@pytest.mark.parametrize("n_out", [128, 512])          # single-CTA tiles and CTA-pair tiles
def test_a_wait_that_runs_out_is_reported_and_the_device_keeps_working(ops, n_out):
    L, r, xs, w = _case(ops, n_out)
    lib = L.lib()
    good = ops.esmm(xs, w, L.B_NK, r, engine=L.ENGINE_TCGEN05)
    torch.cuda.synchronize()
    assert L.device_status() == 0
    try:
        assert lib.hexa_set_wait_limit_ns(5_000_000) == 0
        assert lib.hexa_set_tc_debug(4) == 0
        t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        # the launch itself succeeds; the failure happens on the device (checked below, not by the wrapper)
        assert lib.hexa_esmm(xs.data_ptr(), xs.stride(0), w.data_ptr(), L.B_NK, w.stride(1), w.stride(0), None, 0, None, 0,
                             torch.empty_like(good).data_ptr(), good.stride(0), r.tile_expert.data_ptr(),
                             r.pad_offsets.data_ptr(), r.row_token.data_ptr(), r.pair_block.data_ptr(), r.num_experts,
                             r.row_capacity, n_out, xs.shape[1], L.BF16, L.EPI_LINEAR, L.ACT_NONE, L.ENGINE_TCGEN05,
                             torch.cuda.current_stream().cuda_stream) == 0
        t1.record()
        torch.cuda.synchronize()                      # returns: the kernel gave up instead of spinning
        assert t0.elapsed_time(t1) < 1000.0           # a few ms of limit plus the drain, nowhere near the 2 s default
    finally:
        lib.hexa_set_tc_debug(0)
        lib.hexa_set_wait_limit_ns(2_000_000_000)
    code = L.device_status()
    assert code in (1, 2, 3, 4), code
    assert lib.hexa_pending_device_status() == code
    with pytest.raises(L.HexaError, match="bounded wait"):          # the entry point refuses: HEXA_ERR_DEVICE
        ops.esmm(xs, w, L.B_NK, r, engine=L.ENGINE_TCGEN05)
    assert lib.hexa_esmm(xs.data_ptr(), xs.stride(0), w.data_ptr(), L.B_NK, w.stride(1), w.stride(0), None, 0, None, 0,
                         good.data_ptr(), good.stride(0), r.tile_expert.data_ptr(), r.pad_offsets.data_ptr(),
                         r.row_token.data_ptr(), r.pair_block.data_ptr(), r.num_experts, r.row_capacity, n_out, xs.shape[1],
                         L.BF16, L.EPI_LINEAR, L.ACT_NONE, L.ENGINE_TCGEN05, torch.cuda.current_stream().cuda_stream) == L.ERR_DEVICE
    L.clear_device_status()
    again = ops.esmm(xs, w, L.B_NK, r, engine=L.ENGINE_TCGEN05)     # same context, same answer as before
    torch.cuda.synchronize()
    n_pad = int(r.pad_offsets[-1])                                  # rows beyond the last segment are never written
    assert torch.equal(again[:n_pad], good[:n_pad]) and L.device_status() == 0


def test_status_word_is_shared_by_host_threads(ops):
    """Backward runs on the autograd engine's thread: the word installed from the main thread must be the one a
    kernel launched from another thread reports to."""
    import threading
    from hexa_moe_b200 import _lib as L
    L.ensure_status_word(torch.cuda.current_device())
    seen = {}

    def other():
        torch.cuda.set_device(0)
        seen["code"] = L.lib().hexa_pending_device_status()
        seen["word"] = L._status_words[0].data_ptr()
    th = threading.Thread(target=other); th.start(); th.join()
    assert seen["code"] == 0 and seen["word"] == L._status_words[0].data_ptr()


def test_gate_rows_of_nan_and_inf_get_valid_ids(ops):
    T, E, k = 300, 40, 3
    g = torch.Generator().manual_seed(0)
    logits = torch.randn(T, E, generator=g)
    bad = {7: float("nan"), 50: float("inf"), 120: float("-inf")}
    for t, v in bad.items():
        logits[t] = v
    logits[200, 5] = float("inf")                     # one overflowed logit: softmax of the row is NaN everywhere
    logits[201, 9] = float("nan")
    ids, loss, first_count, mass = ops.gate_topk(logits.cuda(), k)
    torch.cuda.synchronize()
    got = ids.cpu().t()                               # [T, k]
    assert int(got.min()) >= 0 and int(got.max()) < E
    for t in range(T):
        assert len(set(got[t].tolist())) == k
    for t in list(bad) + [200, 201]:
        assert got[t].tolist() == [0, 1, 2]           # the lowest free ids, by definition of this library
    healthy = torch.ones(T, dtype=torch.bool)
    healthy[list(bad) + [200, 201]] = False
    want = torch.topk(torch.softmax(logits[healthy], 1), k, dim=1).indices
    assert torch.equal(got[healthy].long(), want)
    assert int(first_count.sum()) == T
    assert torch.isnan(loss).item()                   # the loss carries the NaN, as in the reference chain
    # and routing accepts the ids
    r = ops.route(ids, E, route_major=True)
    assert int(r.counts.sum()) == T * k


def test_gate_outputs_are_bit_identical_from_run_to_run(ops):
    T, E, k = 70000, 64, 2
    logits = torch.randn(T, E, generator=torch.Generator().manual_seed(1)).cuda()
    first = ops.gate_topk(logits, k)
    for _ in range(4):
        again = ops.gate_topk(logits, k)
        for a, b in zip(first, again):
            assert torch.equal(a, b)
