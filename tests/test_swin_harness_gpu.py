"""The Swin-MoE-like harness on a B200: every MoE depth of a two-image batch against the CPU oracle (fp32, 1e-5),
and one bf16 training step reaching every parameter.  The attention blocks are stock PyTorch; what is checked is that
the shared MoE_Cascaded serves the depths of a real network shape (changing token counts and model dims, no fc1
bias, top-1) with the kernels of this library."""
import pytest
import torch
import torch.nn.functional as F

from oracle import hexa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


def _small(**kw):
    from swin_moe_harness import SwinMoEHarness
    args = dict(img_size=96, patch=4, dims=(32, 64, 128, 256), depths=(2, 2, 4, 2), heads=(2, 2, 4, 8), window=3,
                num_experts=4, top_k=1, num_classes=10)
    args.update(kw)
    return SwinMoEHarness(**args)


def test_moe_depths_of_the_harness_equal_the_oracle():
    from hexa_moe_b200 import ops
    torch.manual_seed(0)
    m = _small()
    with torch.no_grad():
        for n, p in m.cascaded_moe.named_parameters():
            p.normal_(0, 0.5 if "gates" in n else 0.1)
    m = m.cuda().eval()
    moe = m.cascaded_moe
    seen = []
    inner = moe.forward

    def recording(depth, x, *a, **kw):
        y, aux = inner(depth, x, *a, **kw)
        if depth in m.moe_idx:
            ids = torch.stack([i.cpu() for i in moe.dispatch_params.indices_], dim=1)
            seen.append((depth, x.detach().cpu(), y.detach().cpu(), ids))
        return y, aux
    moe.forward = recording
    before = ops.LAUNCHES
    with torch.no_grad():
        logits, _ = m(torch.randn(2, 3, 96, 96, device="cuda"))
    assert ops.LAUNCHES > before and torch.isfinite(logits).all()
    assert [s[0] for s in seen] == m.moe_idx == [5, 7, 9]
    P = {n: p.detach().cpu() for n, p in moe.named_parameters()}
    for i, (depth, x, y, ids) in enumerate(seen):
        d = x.shape[-1]
        want = O.moe_layer(x.reshape(-1, d), ids, P[f"batched_fc1_w.{i}"], P[f"batched_fc2_w.{i}"], None,
                           P[f"batched_fc2_bias.{i}"], F.gelu, None)["y"]
        err = float((y.reshape(-1, d).double() - want).abs().max() / want.abs().max())
        assert err < 1e-5, (depth, err)


def test_bf16_training_step_reaches_every_parameter():
    torch.manual_seed(1)
    m = _small().to(torch.bfloat16).cuda().train()
    logits, l_aux = m(torch.randn(2, 3, 96, 96, device="cuda").bfloat16())
    (F.cross_entropy(logits.float(), torch.tensor([1, 2], device="cuda")) + 0.01 * l_aux).backward()
    missing = [n for n, p in m.named_parameters() if p.grad is None or not torch.isfinite(p.grad).all()]
    assert not missing, missing
