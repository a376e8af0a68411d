"""The two small configurations of the benchmark list at their own sizes, against the CPU oracle.  Needs a B200.

* the README toy: total_depth 4, model dim 128 everywhere, MoE at depths 2 and 3 (dense FFN at 0 and 1), 8 experts,
  top-1 gate with gate_noise 1.0 and an fp32 gate, mlp_ratio 4, GELU, both biases, fp32, input [8, 512, 128];
  forward and backward of sum(outputs) + l_aux (reference README.md:28-40, impls/cascaded_moe.py:527-621);
* the operator sweep: 16384 tokens, d=768, hidden 3072, E=8 and E=32, top-2, bf16: ESMM forward, ESMM input
  gradient, ESTMM and ESS each checked on sampled rows / experts against float64 (the whole layer at this size
  takes the float64 oracle minutes; sampled rows take seconds).
Tolerances: fp32 1e-5, bf16 2e-2, relative to the largest magnitude of the expected tensor; indices exact.
"""
import pytest
import torch
import torch.nn.functional as F

from oracle import hexa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


def rel_err(got, want):
    got = got.detach().double().cpu(); want = want.detach().double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def test_readme_toy_at_its_own_size():
    from hexa_moe import moe as hmoe
    torch.manual_seed(0)
    d, E = 128, 8
    m = hmoe.MoE_Cascaded(gate_type={'type': 'top', 'k': 1, 'gate_noise': 1.0, 'fp32_gate': True}, model_dim_list=[d] * 4,
                          moe_idx_list=[2, 3], mlp_ratio=4, mlp_proportion=None, num_global_experts=E, total_depth=4,
                          data_centric=True, mlp_fc1_bias=True, mlp_fc2_bias=True, activation_fn=lambda t: F.gelu(t))
    with torch.no_grad():          # the module's own init (std 0.005, zero biases) gives outputs ~1e-4: scale up so that
        for n_, p in m.named_parameters():      # every term of the comparison is well away from zero
            p.normal_(0, 0.5 if "gates" in n_ else 0.08)
    m = m.cuda().train()           # training mode: the gate noise is drawn
    x = torch.randn(8, 512, d)
    xg = x.cuda().requires_grad_(True)
    torch.manual_seed(123)         # the two noise draws of the forward pass are replayed below from the same seed
    h, aux, acts, ids_used, l_used = xg, 0, [], [], []
    for depth in range(4):
        acts.append(h)
        h, l = m(depth, h)
        if depth in (2, 3):
            ids_used.append(torch.stack([i.cpu() for i in m.dispatch_params.indices_], dim=1))
            l_used.append(float(l))
        aux = aux + l
    assert h.shape == (8, 512, d) and h.dtype == torch.float32
    for a in acts[1:]:
        a.retain_grad()
    (h.sum() + aux).backward()
    torch.manual_seed(123)
    noise = [torch.randn(4096, E, device="cuda").cpu(), torch.randn(4096, E, device="cuda").cpu()]
    P = {n_: p.detach().cpu().double() for n_, p in m.named_parameters()}
    G = {n_: p.grad.detach().cpu() for n_, p in m.named_parameters() if p.grad is not None}
    # float64 replay of the two dense depths
    t = x.double().reshape(-1, d)
    for i in range(2):
        t = F.gelu(t @ P[f"mlp_fc1_w.{i}"].t() + P[f"mlp_fc1_b.{i}"]) @ P[f"mlp_fc2_w.{i}"] + P[f"mlp_fc2_b.{i}"]
    dense_out = t
    assert rel_err(acts[2].reshape(-1, d), dense_out) < 1e-5
    # gate of both MoE depths: the oracle's ids (same noise) and auxiliary loss
    ins = [acts[2].detach().cpu().reshape(-1, d), acts[3].detach().cpu().reshape(-1, d)]
    for i in range(2):
        ids_exp, l_exp, _ = O.gate_topk(ins[i], P[f"gates.{i}.wg.weight"], 1, noise=noise[i], gate_noise=1.0)
        assert (ids_exp == ids_used[i]).float().mean() > 0.999          # a near-tie may resolve differently
        assert int(ids_used[i].min()) >= 0 and int(ids_used[i].max()) < E
        assert abs(l_used[i] - float(l_exp)) < 1e-4 * abs(float(l_exp))
    # MoE depths through the oracle's layer with the module's routing decisions
    y2 = O.moe_layer(dense_out, ids_used[0], P["batched_fc1_w.0"], P["batched_fc2_w.0"], P["batched_fc1_bias.0"],
                     P["batched_fc2_bias.0"], F.gelu, None)["y"]
    res3 = O.moe_layer(y2, ids_used[1], P["batched_fc1_w.1"], P["batched_fc2_w.1"], P["batched_fc1_bias.1"],
                       P["batched_fc2_bias.1"], F.gelu, torch.ones_like(y2))
    assert rel_err(acts[3].reshape(-1, d), y2) < 1e-5
    assert rel_err(h.reshape(-1, d), res3["y"]) < 1e-5
    for name, key in (("batched_fc1_w.1", "dw1"), ("batched_fc2_w.1", "dw2"), ("batched_fc1_bias.1", "db1"),
                      ("batched_fc2_bias.1", "db2")):
        assert rel_err(G[name], res3[key]) < 1e-5, name
    # input gradient of the last depth = the expert path (oracle) + the auxiliary loss's path through the gate (float64
    # autograd of the reference formulation with the same noise and ids)
    a3 = y2.clone().requires_grad_(True)
    scores = F.softmax(a3 @ P["gates.1.wg.weight"].t() + noise[1].double() / E, dim=1)
    (g_gate,) = torch.autograd.grad(O.gshard_loss(scores, ids_used[1].long()), a3)
    assert rel_err(acts[3].grad.reshape(-1, d), res3["dx"] + g_gate) < 1e-5
    assert float(aux) > 0 and torch.isfinite(xg.grad).all()
    for n_ in ("mlp_fc1_w.0", "mlp_fc2_w.1", "gates.0.wg.weight", "batched_fc1_w.0"):
        assert n_ in G and torch.isfinite(G[n_]).all() and float(G[n_].abs().max()) > 0


@pytest.mark.parametrize("E", [8, 32])
def test_operator_sweep_config_on_sampled_rows(E):
    from hexa_moe_b200 import _lib as L, ops
    T, d, H, k = 16384, 768, 3072, 2
    g = torch.Generator().manual_seed(E)
    ids = torch.topk(torch.randn(T, E, generator=g), k, dim=1).indices.to(torch.int32)
    x = torch.randn(T, d, generator=g).bfloat16()
    dy = torch.randn(T, d, generator=g).bfloat16()
    w1 = (torch.randn(E, H, d, generator=g) / d ** 0.5).bfloat16()
    w2 = (torch.randn(E, H, d, generator=g) / H ** 0.5).bfloat16()
    b1 = torch.randn(E, H, generator=g) * 0.1
    b2 = torch.randn(E, d, generator=g) * 0.1
    y, st = ops.moe_forward(x.cuda(), ids.cuda(), w1.cuda(), w2.cuda(), b1.cuda(), b2.cuda(), L.ACT_GELU, engine=L.ENGINE_TCGEN05)
    dx, dw1, dw2, db1, db2 = ops.moe_backward(st, dy.cuda(), w1.cuda(), w2.cuda(), L.ACT_GELU, grad_dtype=torch.float32,
                                              engine=L.ENGINE_TCGEN05)
    r = st.routing
    want_r = O.route(ids, E, 128)
    assert torch.equal(r.row_token.cpu()[: want_r["n_pad"]], want_r["row_token"])         # routing: bit-exact at this size
    assert torch.equal(r.token_row.cpu(), want_r["token_row"])
    W1, W2, B1, B2 = w1.double(), w2.double(), b1.double(), b2.double()
    X, DY = x.double(), dy.double()
    # forward and input gradient on 64 sampled tokens
    toks = torch.randperm(T, generator=g)[:64]
    for t in toks.tolist():
        yt = torch.zeros(d, dtype=torch.float64); dxt = torch.zeros(d, dtype=torch.float64)
        for j in range(k):
            e = int(ids[t, j])
            y1 = W1[e] @ X[t] + B1[e]
            y1v = y1.clone().requires_grad_(True)
            hh = F.gelu(y1v)
            yt += W2[e].t() @ hh.detach() + B2[e]
            dh = W2[e] @ DY[t]
            (gact,) = torch.autograd.grad(hh.sum(), y1v)
            dxt += W1[e].t() @ (dh * gact)
        assert float((y[t].double().cpu() - yt).abs().max() / yt.abs().max()) < 2e-2
        assert float((dx[t].double().cpu() - dxt).abs().max() / dxt.abs().max()) < 2e-2
    # ESS and ESTMM on two sampled experts, whole segments, float64
    for e in torch.randperm(E, generator=g)[:2].tolist():
        rows = [(t, j) for j in range(k) for t in torch.nonzero(ids[:, j] == e).flatten().tolist()]
        tt = torch.tensor([t for t, _ in rows])
        Y1 = X[tt] @ W1[e].t() + B1[e]
        Y1v = Y1.clone().requires_grad_(True)
        Hh = F.gelu(Y1v)
        (Gact,) = torch.autograd.grad(Hh.sum(), Y1v)
        DH = (DY[tt] @ W2[e].t()) * Gact
        want_db2, want_db1 = DY[tt].sum(0), DH.sum(0)
        want_dw2 = Hh.detach().t() @ DY[tt]              # [H, d]
        want_dw1 = DH.t() @ X[tt]                        # [H, d]
        assert rel_err(db2[e], want_db2) < 2e-2 and rel_err(db1[e], want_db1) < 2e-2
        assert rel_err(dw2[e], want_dw2) < 2e-2 and rel_err(dw1[e], want_dw1) < 2e-2
