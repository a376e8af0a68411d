"""softmax + top-k + GShard loss kernels (hexa_gate_topk / hexa_gate_loss_grad) against the CPU oracle's restatement
of the reference chain F.softmax -> torch.topk -> gshard_loss (cascaded_moe.py:568-598, layers.py:480-489,
losses.py:12-19).  Index work is bit-exact; the float outputs are held to 1e-5 of their scale (fp32 summation order)."""
import pytest
import torch
import torch.nn.functional as F

from oracle import hexa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


CASES = [(1000, 64, 2), (257, 7, 1), (4096, 8, 4), (33, 300, 3), (5, 512, 8), (16, 1, 1), (1, 4, 4), (70000, 32, 1)]


@pytest.mark.parametrize("T,E,k", CASES)
def test_ids_loss_and_counts_match_the_oracle(T, E, k):
    from hexa_moe_b200 import ops
    g = torch.Generator().manual_seed(T * 31 + E)
    logits = torch.randn(T, E, generator=g) * 2.0
    ids, loss, first_count, mass = ops.gate_topk(logits.cuda(), k)
    scores = F.softmax(logits, dim=1)
    want = torch.topk(scores, k, dim=1)
    got = ids.cpu().t().long()                                   # [T, k]
    assert got.shape == (T, k) and ids.dtype == torch.int32
    same = got == want.indices
    if not bool(same.all()):
        # two scores within an ulp of each other may swap; nothing else may differ
        picked = scores.gather(1, got)
        assert torch.allclose(picked, want.values, rtol=1e-6, atol=0)
        assert float(same.float().mean()) > 0.999
    for t in range(0, T, max(T // 50, 1)):                       # k distinct experts per token
        assert len(set(got[t].tolist())) == k
    assert torch.equal(first_count.cpu().long(), torch.bincount(got[:, 0], minlength=E))
    assert torch.allclose(mass.cpu(), scores.sum(0), rtol=1e-5, atol=1e-6)
    want_loss = O.gshard_loss(scores.double(), got)
    assert abs(float(loss) - float(want_loss)) <= 1e-5 * abs(float(want_loss))


def test_equal_scores_go_to_the_lowest_expert_ids():
    from hexa_moe_b200 import ops
    logits = torch.zeros(64, 40, device="cuda")
    logits[:, 17] = 1.0                                         # one clear winner, everything else tied
    ids, _, first_count, _ = ops.gate_topk(logits, 3)
    assert ids.cpu().tolist() == [[17] * 64, [0] * 64, [1] * 64]
    assert int(first_count[17]) == 64 and int(first_count.sum()) == 64


@pytest.mark.parametrize("T,E,k", [(1000, 64, 2), (33, 300, 3), (4096, 8, 1)])
def test_loss_gradient_matches_autograd_of_the_reference_formulation(T, E, k):
    from hexa_moe_b200 import ops
    g = torch.Generator().manual_seed(7 + T)
    logits = torch.randn(T, E, generator=g)
    ref = logits.double().requires_grad_(True)
    scores = F.softmax(ref, dim=1)
    top = torch.topk(scores, k, dim=1).indices
    loss = O.gshard_loss(scores, top)
    (loss * 3.0).backward()
    dev = logits.cuda()
    _, _, first_count, _ = ops.gate_topk(dev, k)
    got = ops.gate_loss_grad(dev, first_count, torch.tensor(3.0, device="cuda"))
    scale = float(ref.grad.abs().max())
    assert float((got.cpu().double() - ref.grad).abs().max()) <= 1e-5 * scale


def test_module_routes_through_the_fused_gate_and_matches_the_pytorch_chain():
    """Same layer, same input: the fused gate step and the PyTorch-op chain give the same output, auxiliary loss and
    input gradient (2e-2, the bf16 tolerance of the layer; the gate itself is fp32 either way)."""
    import os
    from hexa_moe import moe as hmoe
    from hexa_moe_b200 import ops
    torch.manual_seed(11)
    m = hmoe.MoE_Cascaded(gate_type={'type': 'top', 'k': 2, 'fp32_gate': True}, model_dim_list=[64], moe_idx_list=[0],
                          mlp_ratio=4, num_global_experts=8, total_depth=1, data_centric=True,
                          activation_fn=lambda t: F.gelu(t))
    with torch.no_grad():
        for n_, p in m.named_parameters():
            p.normal_(0, 0.3 if "gates" in n_ else 0.1)
    m = m.to(torch.bfloat16).cuda().train()
    x = torch.randn(300, 64, device="cuda").bfloat16()

    def run():
        xi = x.clone().requires_grad_(True)
        y, aux = m(0, xi)
        (y.float().sum() + 5.0 * aux).backward()
        return y.detach().float(), float(aux), xi.grad.float(), m.gates[0].wg.weight.grad.clone()

    m.zero_grad()
    before = ops.LAUNCHES
    fused = run()
    n_fused = ops.LAUNCHES - before
    os.environ["HEXA_FUSED_GATE"] = "0"
    try:
        m.zero_grad()
        before = ops.LAUNCHES
        plain = run()
        n_plain = ops.LAUNCHES - before
    finally:
        del os.environ["HEXA_FUSED_GATE"]
    assert n_fused == n_plain + 2                                # one gate kernel each way
    assert abs(fused[1] - plain[1]) <= 1e-5 * abs(plain[1])
    for a, b in ((fused[0], plain[0]), (fused[2], plain[2]), (fused[3], plain[3])):
        assert float((a - b).abs().max()) <= 2e-2 * float(b.abs().max())


@pytest.mark.parametrize("T,E,k", [(1000, 64, 2), (257, 7, 1), (4096, 8, 4), (33, 300, 3), (70000, 32, 2)])
def test_load_importance_ids_loss_and_gradient_match_the_oracle(T, E, k):
    """The other auxiliary loss of the reference (is_gshard_loss=False, impls/losses.py:21-43): ids of the noisy logits
    bit-exact, loss and its gradient against float64 autograd of the oracle's restatement (1e-5 of their scale), and
    bit-identical outputs from run to run."""
    from hexa_moe_b200 import ops
    g = torch.Generator().manual_seed(T + E)
    logits = torch.randn(T, E, generator=g) * 0.05
    gate_noise = 1.0
    noisy = logits + gate_noise * torch.randn(T, E, generator=g) / E
    ids, loss, importance, load = ops.gate_topk_load_importance(logits.cuda(), noisy.cuda(), k, gate_noise / E)
    got = ids.cpu().t().long()
    assert torch.equal(got, torch.topk(noisy, k, dim=1).indices)          # the kernel ranks the noisy logits themselves
    # the reference ranks softmax(noisy) in fp32, where two different logits can round to the same score: the picks may
    # differ there, and only there (the picked scores agree to an ulp)
    scores = F.softmax(noisy, dim=1)
    ref_pick = torch.topk(scores, k, dim=1)
    assert torch.allclose(scores.gather(1, got), ref_pick.values, rtol=1e-6, atol=0)
    assert float((got == ref_pick.indices).float().mean()) > 0.99
    ref = logits.double().requires_grad_(True)
    noisy_ref = ref + (noisy.double() - logits.double())
    want = O.load_importance_loss(F.softmax(ref, dim=1), noisy_ref.gather(1, got), E, gate_noise)
    # the loss is a variance of nearly equal column sums over their squared mean: fp32 sums (1e-6 relative) are amplified
    # by mean / spread; the reference evaluates it in fp32 as well
    assert abs(float(loss) - float(want)) <= 2e-3 * abs(float(want)), (float(loss), float(want))
    assert torch.allclose(importance.cpu().double(), F.softmax(ref, dim=1).sum(0).detach(), rtol=1e-5, atol=1e-6)
    z = (F.softmax(ref, dim=1).detach() - noisy.double().gather(1, got)[:, -1:]) / (gate_noise / E)
    assert torch.allclose(load.cpu().double(), (0.5 * (1 + torch.erf(z / 2 ** 0.5))).sum(0), rtol=1e-4, atol=1e-5)
    (want * 3.0).backward()
    grad = ops.gate_load_importance_grad(logits.cuda(), noisy.cuda(), k, gate_noise / E, importance, load,
                                         torch.tensor(3.0, device="cuda"))
    scale = float(ref.grad.abs().max())
    # fp32 kernel against float64: the gradient factors of var / mean^2 are differences of nearly equal column sums
    assert float((grad.cpu().double() - ref.grad).abs().max()) <= 5e-3 * scale
    again = ops.gate_topk_load_importance(logits.cuda(), noisy.cuda(), k, gate_noise / E)
    for a, b in zip((ids, loss, importance, load), again):
        assert torch.equal(a, b)


def test_module_with_the_load_importance_loss_takes_the_fused_gate():
    """is_gshard_loss=False in training mode: the fused kernels and the PyTorch chain (HEXA_FUSED_GATE=0) see the same
    noise (same seed) and give the same output, auxiliary loss and gradients."""
    import os
    from hexa_moe import moe as hmoe
    from hexa_moe_b200 import ops
    torch.manual_seed(12)
    m = hmoe.MoE_Cascaded(gate_type={'type': 'top', 'k': 2, 'fp32_gate': True, 'gate_noise': 1.0}, model_dim_list=[64],
                          moe_idx_list=[0], mlp_ratio=4, num_global_experts=8, total_depth=1, data_centric=True,
                          is_gshard_loss=False, activation_fn=lambda t: F.gelu(t))
    with torch.no_grad():
        for n_, p in m.named_parameters():
            p.normal_(0, 0.02 if "gates" in n_ else 0.1)
    m = m.to(torch.bfloat16).cuda().train()
    x = torch.randn(300, 64, device="cuda").bfloat16()

    def run():
        torch.manual_seed(99)                        # the same noise draw both times
        xi = x.clone().requires_grad_(True)
        y, aux = m(0, xi)
        (y.float().sum() + 5.0 * aux).backward()
        return y.detach().float(), float(aux), xi.grad.float(), m.gates[0].wg.weight.grad.clone()

    m.zero_grad()
    before = ops.LAUNCHES
    fused = run()
    n_fused = ops.LAUNCHES - before
    os.environ["HEXA_FUSED_GATE"] = "0"
    try:
        m.zero_grad()
        before = ops.LAUNCHES
        plain = run()
        n_plain = ops.LAUNCHES - before
    finally:
        del os.environ["HEXA_FUSED_GATE"]
    assert n_fused == n_plain + 2                                # one gate kernel each way
    assert abs(fused[1] - plain[1]) <= 1e-4 * abs(plain[1])
    for a, b in ((fused[0], plain[0]), (fused[2], plain[2]), (fused[3], plain[3])):
        assert float((a - b).abs().max()) <= 2e-2 * float(b.abs().max())
