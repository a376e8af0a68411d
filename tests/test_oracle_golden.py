"""The CPU oracle against the fixtures produced by the reference's own kernels
(tests/golden/make_golden.py).  CPU only."""
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import hexa_oracle as O


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def _cases(z):
    return sorted({k.split("/")[0] for k in z.files})


def test_counter_matches_reference(golden_dir):
    z = _load(golden_dir, "counter.npz")
    for c in _cases(z):
        r = torch.from_numpy(z[c + "/routing"]); E = int(z[c + "/E"])
        n, starts, tok, exp = O.counter(r, E)
        assert n == int(z[c + "/n"]), c
        assert np.array_equal(starts.numpy(), z[c + "/starts"]), c
        assert np.array_equal(exp.numpy(), z[c + "/exp_ids"]), c
        # the reference's order inside a segment is unspecified on a GPU: compare as sets per
        # segment, and additionally exactly (the interpreter run that made the fixture is sequential)
        ref_tok = z[c + "/tok_ids"]
        for e in range(E):
            a, b = int(starts[e]), int(starts[e + 1])
            assert sorted(tok.numpy()[a:b].tolist()) == sorted(ref_tok[a:b].tolist()), (c, e)
        assert np.array_equal(tok.numpy(), ref_tok), c


def test_route_merged_is_per_route_counter(golden_dir):
    z = _load(golden_dir, "counter.npz")
    for c in _cases(z):
        r = torch.from_numpy(z[c + "/routing"]); E = int(z[c + "/E"])
        m = O.route(r.view(-1, 1), E, align=16)
        assert np.array_equal(m["pad_offsets"].numpy(), z[c + "/starts"]), c
        assert np.array_equal(m["row_token"].numpy(), z[c + "/tok_ids"]), c
        assert np.array_equal(m["tile_expert"].numpy(), z[c + "/exp_ids"]), c
    # k = 2: each expert's rows are route 0's tokens ascending, then route 1's
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 5, (40, 2), generator=g, dtype=torch.int32)
    m = O.route(ids, 5, align=8)
    for e in range(5):
        a = int(m["pad_offsets"][e]); cnt = int(m["counts"][e])
        want = []
        for j in range(2):
            _, st, tok, _ = O.counter(ids[:, j], 5)
            seg = tok[int(st[e]): int(st[e + 1])]
            want += seg[seg >= 0].tolist()
        assert m["row_token"][a: a + cnt].tolist() == want
        assert (m["row_token"][a + cnt: int(m["pad_offsets"][e + 1])] == -1).all()
    tr = m["token_row"].view(40, 2)
    for t in range(40):
        for j in range(2):
            assert int(m["row_token"][tr[t, j]]) == t


def test_esmm_and_dgrad_match_reference(golden_dir):
    z = _load(golden_dir, "esmm.npz")
    for c in _cases(z):
        x, w, b, dy = (torch.from_numpy(z[f"{c}/{k}"]) for k in ("x", "w", "b", "dy"))
        r = torch.from_numpy(z[c + "/routing"])
        # the reference rounds both operands to fp16 and accumulates in fp32 (kernels/esmm.py:133-134)
        for got, want in ((O.esmm(x, w, b, r, torch.float16), z[c + "/y_bias"]),
                          (O.esmm(x, w, None, r, torch.float16), z[c + "/y_nobias"]),
                          (O.esmm_dgrad(dy, w, r, torch.float16), z[c + "/dx"])):
            np.testing.assert_allclose(got.numpy(), want, rtol=0, atol=5e-6)
        # and the operand rounding is what separates it from exact math
        assert np.abs(O.esmm(x, w, b, r).numpy() - z[c + "/y_bias"]).max() > 1e-5


def test_estmm_ess_match_reference_where_it_is_correct(golden_dir):
    z = _load(golden_dir, "estmm_ess.npz")
    for c in _cases(z):
        x, w, dy = (torch.from_numpy(z[f"{c}/{k}"]) for k in ("x", "w", "dy"))
        r = torch.from_numpy(z[c + "/routing"]); E = int(z[c + "/E"])
        counts = np.bincount(r.numpy(), minlength=E)
        ess_ref, dw_ref = z[c + "/ess"], z[c + "/estmm"]
        # experts after the last non-empty one are never written by the reference (NaN pre-fill survives)
        written = ~np.isnan(ess_ref).any(axis=1)
        assert written[counts > 0].all()
        got_ess = O.ess(dy, r, E).numpy(); got_dw = O.estmm(dy, x, r, E, torch.float16).numpy()
        np.testing.assert_allclose(got_ess[written], ess_ref[written], rtol=0, atol=5e-6)
        np.testing.assert_allclose(got_dw[written], dw_ref[written], rtol=0, atol=2e-5)
        assert (got_ess[counts == 0] == 0).all() and (got_dw[counts == 0] == 0).all()


def test_layer_and_gate_match_reference_module(golden_dir):
    z = _load(golden_dir, "module.npz")
    for tag, k in (("top1", 1), ("top2", 2)):
        P = {n.split("param/")[1]: torch.from_numpy(z[n]) for n in z.files if n.startswith(tag + "/param/")}
        x = torch.from_numpy(z[tag + "/x"]).requires_grad_(True)
        h = x; laux = 0
        for d in range(4):
            flat = h.reshape(-1, h.shape[-1])
            if d in (2, 3):
                i = d - 2
                ids, l, _ = O.gate_topk(flat, P[f"gates.{i}.wg.weight"], k)
                # forward value from the oracle (operands rounded to fp16 as the reference kernels do)
                res = O.moe_layer(flat.detach(), ids, P[f"batched_fc1_w.{i}"], P[f"batched_fc2_w.{i}"],
                                  P[f"batched_fc1_bias.{i}"], P[f"batched_fc2_bias.{i}"], F.gelu,
                                  operand_dtype=torch.float16)
                np.testing.assert_allclose(res["y"].numpy().reshape(h.shape), z[f"{tag}/y{d}"], rtol=5e-5, atol=2e-3)  # fp16 re-rounding of the hidden can flip an ulp
                assert abs(float(l.detach()) - float(z[f"{tag}/l_aux{d}"])) < 1e-6
                h = torch.from_numpy(z[f"{tag}/y{d}"])          # continue from the reference activations
            else:
                j = d
                y1 = flat @ P[f"mlp_fc1_w.{j}"].T + P[f"mlp_fc1_b.{j}"]
                y = F.gelu(y1) @ P[f"mlp_fc2_w.{j}"] + P[f"mlp_fc2_b.{j}"]
                h = y.reshape(h.shape)
                np.testing.assert_allclose(h.detach().numpy(), z[f"{tag}/y{d}"], rtol=2e-5, atol=2e-5)


def test_moe_layer_backward_is_autograd_of_forward():
    """The oracle's hand-written backward equals autograd through a dense restatement."""
    torch.manual_seed(5)
    T, k, E, d, H = 37, 2, 5, 12, 20
    x = torch.randn(T, d, dtype=torch.float64, requires_grad=True)
    ids = torch.stack([torch.randperm(E)[:k] for _ in range(T)]).to(torch.int32)
    w1 = torch.randn(E, H, d, dtype=torch.float64, requires_grad=True)
    w2 = torch.randn(E, H, d, dtype=torch.float64, requires_grad=True)
    b1 = torch.randn(E, H, dtype=torch.float64, requires_grad=True)
    b2 = torch.randn(E, d, dtype=torch.float64, requires_grad=True)
    dy = torch.randn(T, d, dtype=torch.float64)
    y = 0
    for j in range(k):
        e = ids[:, j].long()
        y1 = torch.einsum("td,thd->th", x, w1[e]) + b1[e]
        y = y + torch.einsum("th,tho->to", F.gelu(y1), w2[e]) + b2[e]
    y.backward(dy)
    res = O.moe_layer(x.detach(), ids, w1.detach(), w2.detach(), b1.detach(), b2.detach(), F.gelu, dy)
    for got, want in ((res["y"], y.detach()), (res["dx"], x.grad), (res["dw1"], w1.grad), (res["dw2"], w2.grad),
                      (res["db1"], b1.grad), (res["db2"], b2.grad)):
        torch.testing.assert_close(got, want, rtol=1e-10, atol=1e-10)
    fast = O.moe_layer_fast(x.detach().float(), ids, w1.detach().float(), w2.detach().float(), b1.detach().float(),
                            b2.detach().float(), dy.float())
    for kk in ("y", "dx", "dw1", "dw2", "db1", "db2"):
        torch.testing.assert_close(fast[kk].double(), res[kk], rtol=1e-4, atol=1e-4)


def test_dim_split_matches_reference_rule():
    assert O.dim_split(8192, [0.2, 0.2, 0.15, 0.15, 0.1, 0.1, 0.05, 0.05]) == [1639, 1639, 1229, 1229, 819, 819, 409, 409]
    assert O.dim_split(512, [0.25] * 4) == [128] * 4
    assert sum(O.dim_split(4096, [1 / 3] * 3)) == 4096
