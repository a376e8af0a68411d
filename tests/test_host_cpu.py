"""Host-side logic that needs no GPU: the C ABI loads and exports what the header declares, the
module mirrors the reference's constructor / parameter names / sharding rule, activation
recognition, and loud failure where there is no CUDA device."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build():
    from hexa_moe_b200 import build
    return build.build()


def test_library_exports_every_declared_symbol():
    lib_path = _build()
    hdr = open(os.path.join(ROOT, "include", "hexa_moe_b200.h")).read()
    hdr = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)
    declared = sorted(set(re.findall(r"\b(hexa_[a-z0-9_]+)\s*\(", hdr)))
    assert len(declared) >= 12
    lib = ctypes.CDLL(lib_path)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/hexa_moe_b200.h but not exported"
    from hexa_moe_b200 import _lib
    assert set(_lib.SIGNATURES) == set(declared)
    # pure host entry points can be called without a GPU
    h = _lib.lib()
    assert h.hexa_version() >= 100
    assert h.hexa_route_row_capacity(1000, 2, 8, 128) == (2000 + 8 * 127 + 127) // 128 * 128
    assert h.hexa_route_workspace_bytes(1000, 2, 8) == (4 * 8 + 8 + 1) * 4
    assert h.hexa_route_pair_capacity(1000, 2, 8) == h.hexa_route_row_capacity(1000, 2, 8, 128) // 256 + 8 + 1
    assert h.hexa_ess_workspace_bytes(1024, 100) == 8 * 100 * 4
    assert h.hexa_route_row_capacity(10, 0, 8, 128) == -1


def test_argument_errors_come_back_as_status_codes():
    from hexa_moe_b200 import _lib
    h = _lib.lib()
    rc = h.hexa_route(None, 10, 1, 1, 10, 4, 128, None, None, None, None, None, None, None, None, 0, None)
    assert rc == -1 and b"null" in h.hexa_last_error_string()
    rc = h.hexa_esmm(None, 0, None, 0, 0, 0, None, 0, None, 0, None, 0, None, None, None, None, 4, 128, 8, 8, 2, 0, 0, 0, None)
    assert rc == -1
    # the gate step: expert count beyond the kernel's limit, top_k beyond the expert count (checked before any CUDA call)
    assert h.hexa_gate_max_experts() == 512 and h.hexa_gate_workspace_bytes() >= 4
    rc = h.hexa_gate_topk(None, 0, 16, 513, 1, None, None, None, None, None, 0, None)
    assert rc == -1 and b"experts" in h.hexa_last_error_string()
    rc = h.hexa_gate_topk(None, 0, 16, 8, 9, None, None, None, None, None, 0, None)
    assert rc == -1 and b"top_k" in h.hexa_last_error_string()
    rc = h.hexa_gate_loss_grad(None, 0, 16, 0, None, None, None, 0, None)
    assert rc == -1
    # the scatter form of ESTMM: no destination list
    rc = h.hexa_estmm_scatter(None, 0, None, 0, None, 4, 128, 64, 64, None, 2, 64, 64 * 32, 32, 2, 2, None)
    assert rc == -1 and b"null" in h.hexa_last_error_string()


def _toy(**kw):
    from hexa_moe import moe as hmoe
    args = dict(gate_type={'type': 'top', 'k': 1, 'gate_noise': 1.0, 'fp32_gate': True}, model_dim_list=[32] * 4,
                moe_idx_list=[2, 3], mlp_ratio=4, mlp_proportion=None, num_global_experts=4, total_depth=4,
                data_centric=True, mlp_fc1_bias=True, mlp_fc2_bias=True, activation_fn=lambda t: F.gelu(t))
    args.update(kw)
    return hmoe.MoE_Cascaded(**args)


def test_module_parameters_match_reference_state_dict(golden_dir):
    z = np.load(os.path.join(golden_dir, "module.npz"))
    ref = {n.split("param/")[1]: z[n] for n in z.files if n.startswith("top1/param/")}
    m = _toy()
    mine = {n: tuple(p.shape) for n, p in m.state_dict().items()}
    assert mine == {n: v.shape for n, v in ref.items()}
    m.load_state_dict({n: torch.from_numpy(v) for n, v in ref.items()})
    # dense depths are plain PyTorch and match the reference's activations on CPU
    x = torch.from_numpy(z["top1/x"])
    y0, l0 = m(0, x)
    np.testing.assert_allclose(y0.detach().numpy(), z["top1/y0"], rtol=2e-5, atol=2e-5)
    assert l0 == 0
    y1, _ = m(1, torch.from_numpy(z["top1/y0"]))
    np.testing.assert_allclose(y1.detach().numpy(), z["top1/y1"], rtol=2e-5, atol=2e-5)


def test_moe_depth_fails_loudly_without_cuda():
    from hexa_moe_b200._lib import HexaError
    m = _toy()
    with pytest.raises(HexaError, match="CUDA tensors only"):
        m(2, torch.randn(2, 8, 32))


def test_init_and_options():
    m = _toy(mlp_fc1_bias=False, gate_type=[{'type': 'top', 'k': 2}, {'type': 'cosine_top', 'k': 1, 'proj_dim': 16}])
    assert m.batched_fc1_bias[0] is None and m.mlp_fc1_b[0] is None
    assert len(m.gates) == 4 and m.gate_len == 2
    assert type(m.gates[1]).__name__ == "CosineTopKGate" and type(m.gates[3]).__name__ == "CosineTopKGate"
    assert abs(float(m.batched_fc1_w[0].detach().std()) - 0.005) < 5e-4 and float(m.batched_fc2_bias[0].detach().abs().max()) == 0
    with pytest.raises(Exception, match="Unrecognized gate_type"):
        _toy(gate_type={'type': 'nope', 'k': 1})
    with pytest.raises(Exception, match="Unrecognized argument"):
        _toy(gate_type={'type': 'top', 'k': 1, 'bogus': 3})
    m2 = _toy(gate_type="Top2Gate")
    assert m2.gates[0].top_k == 2
    os.environ["SKIP_MOE"] = "1"
    try:
        m3 = _toy()
        x = torch.randn(2, 4, 32)
        y, l = m3(2, x)
        assert y is x and l is None
    finally:
        del os.environ["SKIP_MOE"]


def test_split_hidden_rule():
    from hexa_moe_b200.impls.cascaded_moe import split_hidden
    from oracle import hexa_oracle as O
    for H, prop in ((8192, [0.2, 0.2, 0.15, 0.15, 0.1, 0.1, 0.05, 0.05]), (512, [0.5, 0.5]), (100, [1 / 3] * 3), (64, [1.0])):
        assert split_hidden(H, prop) == O.dim_split(H, prop)
    assert split_hidden(8192, [0.2, 0.2, 0.15, 0.15, 0.1, 0.1, 0.05, 0.05]) == [1639, 1639, 1229, 1229, 819, 819, 409, 409]


def test_activation_recognition():
    from hexa_moe_b200 import _lib as L
    from hexa_moe_b200.impls.activations import classify
    assert classify(lambda t: F.gelu(t)) == L.ACT_GELU
    assert classify(F.relu) == L.ACT_RELU
    assert classify(torch.nn.GELU(approximate="tanh")) == L.ACT_GELU_TANH
    assert classify(torch.nn.SiLU()) == L.ACT_SILU
    assert classify(lambda t: t) == L.ACT_NONE
    assert classify(lambda t: torch.sigmoid(t)) == -1
    assert classify(lambda t: t.cuda_only_thing()) == -1


def test_checkpoint_buffer_roundtrip_single_rank():
    from hexa_moe import moe as hmoe
    m = _toy()
    buf = hmoe.MoE_Buffer([32, 32], 4, 2, 4, None, True, True)
    with torch.no_grad():
        for p in m.parameters():
            p.normal_()
    m.save_ckpt(buf)
    m2 = _toy()
    m2.load_ckpt(buf)
    for i in range(2):
        assert torch.equal(m2.batched_fc1_w[i], m.batched_fc1_w[i]) and torch.equal(m2.batched_fc2_bias[i], m.batched_fc2_bias[i])
        assert torch.equal(m2.batched_fc1_bias[i], m.batched_fc1_bias[i])


def test_split_terms_reproduce_fp32_exactly():
    """The fp32 gate weight is fed to the tensor cores as three bf16 terms; their sum must be the fp32 value itself
    (24 mantissa bits = 3 x 8), otherwise the 'fp32 gate' would silently lose precision."""
    from hexa_moe_b200.impls.gating import _split_terms
    g = torch.Generator().manual_seed(0)
    w = torch.randn(64, 300, generator=g) * torch.logspace(-6, 3, 300)
    terms = _split_terms(w, torch.bfloat16, 3)
    assert all(t.dtype == torch.bfloat16 for t in terms)
    total = (terms[0].double() + terms[1].double()) + terms[2].double()
    assert torch.equal(total.float(), w)
    two = terms[0].double() + terms[1].double()                 # two terms are not enough: that is why there are three
    assert not torch.equal(two.float(), w)


def test_fused_gate_step_declines_what_it_cannot_do():
    """CPU logits, half-precision logits and a missing backend fall through to the PyTorch chain (None)."""
    from hexa_moe_b200.impls.gating import fused_topk_gshard
    from hexa_moe_b200 import ops
    logits = torch.randn(16, 8)
    assert fused_topk_gshard(logits, 2, ops) is None
    assert fused_topk_gshard(logits.to(torch.bfloat16), 2, ops) is None
    assert fused_topk_gshard(logits, 2, None) is None


def test_barrier_watchdog_releases_and_reports_after_its_deadline():
    """Host logic of the bounded rank barrier, with a fake clock and fake probes (no GPU, no sleeping): a probe that
    completes is forgotten; one that stays unfinished past the deadline trips the watchdog exactly once, the release
    action runs, and the cache raises at its next use instead of waiting for a rank that is gone."""
    from hexa_moe_b200._lib import HexaError
    from hexa_moe_b200.impls.param_cache import BarrierWatchdog, PipelineSharedCache
    now = [0.0]
    released = []
    wd = BarrierWatchdog(timeout_s=5.0, release=lambda: released.append(now[0]), clock=lambda: now[0], poll_s=3600.0)
    state = {"a": False}
    wd.watch(lambda: state["a"], "barrier A")
    wd.watch(lambda: False, "barrier B (its peer never arrives)")
    assert wd.pending() == 2 and not wd.poll_once()
    now[0] = 4.0
    state["a"] = True
    assert not wd.poll_once() and wd.pending() == 1          # A done; B still inside its deadline
    now[0] = 5.5
    assert wd.poll_once() and released == [5.5]
    assert "barrier B" in wd.failed and wd.pending() == 0
    assert wd.poll_once() and released == [5.5]              # trips once
    wd.stop()

    class Owner:           # the few attributes the cache reads before it would touch a device
        world_size, total_depth_moe = 2, 1
    cache = PipelineSharedCache(Owner())
    cache._watchdog = wd
    with pytest.raises(HexaError, match="HEXA_BARRIER_TIMEOUT_S"):
        cache.prefetch(0)
    with pytest.raises(HexaError, match="peer has failed or left"):
        cache.reduce_deferred(0, "fc1", None, None, [1, 1], 0)
    cache.close()                                            # does not block on anything after a failure


def test_barrier_watchdog_thread_trips_on_a_real_clock():
    import time
    from hexa_moe_b200.impls.param_cache import BarrierWatchdog
    hit = []
    wd = BarrierWatchdog(timeout_s=0.2, release=lambda: hit.append(1), poll_s=0.02)
    wd.watch(lambda: False, "barrier whose peer left between steps")
    t0 = time.monotonic()
    while not hit and time.monotonic() - t0 < 5.0:
        time.sleep(0.02)
    assert hit == [1] and "left between steps" in wd.failed and time.monotonic() - t0 < 5.0
    wd.stop()


def test_installing_the_status_word_in_a_fresh_process_does_not_deadlock():
    """The first operator call of a process installs the device status word; that path loads the library under the
    same lock it is about to take.  Run in a fresh interpreter (the library not loaded yet) with the two CUDA-only
    steps replaced: the call must get as far as the C entry point (which, without a device, answers with an error)."""
    import subprocess
    import sys
    code = r'''
import sys, threading, contextlib
sys.path.insert(0, %r)
import torch
from hexa_moe_b200 import _lib as L
torch.Tensor.pin_memory = lambda self: self
torch.cuda.device = lambda idx: contextlib.nullcontext()
out = []
def run():
    try:
        L.ensure_status_word(0)
        out.append("installed")
    except L.HexaError as e:
        out.append("entry point reached: " + str(e)[:60])
t = threading.Thread(target=run, daemon=True); t.start(); t.join(60)
print("DEADLOCK" if t.is_alive() else out[0])
''' % ROOT
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=180)
    assert "DEADLOCK" not in res.stdout and ("installed" in res.stdout or "entry point reached" in res.stdout), res.stdout + res.stderr


def test_load_importance_loss_of_the_module_equals_the_oracle_restatement():
    """impls/losses.py:load_importance_loss (what the PyTorch-op path of the module evaluates, reference
    hexa_moe/impls/losses.py:21-43) against the oracle's float64 restatement, value and gradient."""
    from hexa_moe_b200.impls import losses
    from oracle import hexa_oracle as O
    g = torch.Generator().manual_seed(4)
    T, E, k, noise = 500, 16, 2, 1.0
    logits = (torch.randn(T, E, generator=g) * 0.05).requires_grad_(True)
    noisy = logits + noise * torch.randn(T, E, generator=g) / E
    ids = torch.topk(F.softmax(noisy, dim=1), k, dim=1).indices
    got = losses.load_importance_loss(F.softmax(logits, dim=1), noisy.gather(1, ids), E, noise)
    ref = logits.detach().double().requires_grad_(True)
    noisy_ref = ref + (noisy.detach().double() - logits.detach().double())
    want = O.load_importance_loss(F.softmax(ref, dim=1), noisy_ref.gather(1, ids), E, noise)
    assert abs(float(got) - float(want)) <= 1e-5 * abs(float(want))
    got.backward(); want.backward()
    assert float((logits.grad.double() - ref.grad).abs().max()) <= 2e-3 * float(ref.grad.abs().max())      # fp32 chain vs float64


def test_bench_arms_describe_the_same_configuration():
    """bench.py prints the same `config` object for this library's arm and for the reference arm, and the heterogeneous
    split of config 5 merges neighbouring shares for fewer than eight ranks."""
    import argparse
    import bench
    for world, want in ((8, [0.2, 0.2, 0.15, 0.15, 0.1, 0.1, 0.05, 0.05]), (4, [0.4, 0.3, 0.2, 0.1]), (2, [0.7, 0.3]), (1, [1.0])):
        args = argparse.Namespace(hetero=True, mode="data", workload="c5", tokens=0, gpus=world)
        split, _ = bench.hetero_proportion(args, world)
        assert split == want and abs(sum(split) - 1) < 1e-9 and args.mode == "model"
        cfg = bench.layer_config(args, 2048, 8192, 64, 2, 2, 131072 // world, split)
        assert cfg["mode"] == "model-centric" and cfg["hidden_split"] == want and cfg["tokens_per_gpu"] == 131072 // world
    args = argparse.Namespace(hetero=False, mode="data", workload="c5", tokens=0, gpus=1)
    assert bench.hetero_proportion(args, 1) == (None, None) and args.mode == "data"
    assert bench.cpu_sample_text(2, 64).startswith("16384 tokens (seed 0) top-2 over 8 of the 64 experts")
    assert set(bench.TRAFFIC_RATIO) == {"esmm:fc1_forward_act", "esmm:fc2_forward", "estmm:dw2", "esmm:fc2_dgrad_dact",
                                        "estmm:dw1", "esmm:fc1_dgrad"}


def test_token_chunks_are_the_same_count_on_every_rank(monkeypatch):
    from hexa_moe_b200.impls.layers import token_chunks
    monkeypatch.setenv("HEXA_MC_CHUNKS", "4")
    monkeypatch.setenv("HEXA_MC_MIN_CHUNK_TOKENS", "10")
    assert token_chunks([100]) == [[0, 100]]                               # one rank: nothing to overlap
    cuts = token_chunks([100, 41])
    assert cuts == [[0, 25, 50, 75, 100], [0, 10, 20, 30, 41]]             # 41 // 10 = 4 chunks fit the smallest rank
    assert token_chunks([100, 25]) == [[0, 50, 100], [0, 12, 25]]          # only two chunks of >= 10 tokens fit
    assert token_chunks([100, 0]) == [[0, 100], [0, 0]]                    # a rank without tokens: no cutting
    monkeypatch.delenv("HEXA_MC_CHUNKS"); monkeypatch.delenv("HEXA_MC_MIN_CHUNK_TOKENS")
    assert token_chunks([16384] * 8)[0] == [0, 16384]                      # default: one chunk
    monkeypatch.setenv("HEXA_MC_CHUNKS", "2")
    assert token_chunks([16384] * 8)[0] == [0, 8192, 16384]
    assert token_chunks([384] * 2)[0] == [0, 384]                          # too few tokens to cut
