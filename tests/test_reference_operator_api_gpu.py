"""The reference's operator-level API (`counter`, `ESMM`, `es_fused`: same names, arguments and return values) on
the CUDA kernels, checked against the golden outputs of the reference's own Triton kernels (tests/golden/*.npz)."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _need_cuda():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")


def _cases(z):
    return sorted({k.split("/")[0] for k in z.files})


def test_counter_equals_reference_lists(golden_dir):
    from hexa_moe_b200.kernels.basics import counter
    z = np.load(os.path.join(golden_dir, "counter.npz"))
    for c in _cases(z):
        n, starts, tok, exp = counter(torch.from_numpy(z[c + "/routing"]).cuda(), int(z[c + "/E"]))
        assert n == int(z[c + "/n"])
        assert np.array_equal(starts.cpu().numpy(), z[c + "/starts"])
        assert np.array_equal(tok.cpu().numpy(), z[c + "/tok_ids"])       # ascending inside a segment = stable sort
        assert np.array_equal(exp.cpu().numpy(), z[c + "/exp_ids"])


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-3), (torch.float16, 2e-3)])
def test_esmm_and_fused_dx_equal_reference_outputs(golden_dir, dtype, tol):
    """The reference rounds both operands to fp16 and accumulates in fp32.  fp16 inputs here reproduce that rounding
    (the result differs only by the fp16 rounding of the output); fp32 inputs are NOT rounded by this library, so the
    distance to the golden values is the reference's own operand-rounding error (~1e-3)."""
    from hexa_moe_b200.kernels.basics import counter
    from hexa_moe_b200.kernels.esmm import ESMM
    from hexa_moe_b200.kernels.fused import es_fused
    z = np.load(os.path.join(golden_dir, "esmm.npz"))
    for c in _cases(z):
        x, w, b, dy = (torch.from_numpy(z[f"{c}/{k}"]).cuda() for k in ("x", "w", "b", "dy"))
        routing = torch.from_numpy(z[c + "/routing"]).cuda()
        E = int(z[c + "/E"])
        n, starts, tok, exp = counter(routing, E)
        y_b = ESMM(x.to(dtype), w.to(dtype), b, (tok + 1).contiguous(), exp)
        y_nb = ESMM(x.to(dtype), w.to(dtype), torch.empty(0, device="cuda"), (tok + 1).contiguous(), exp)
        wt = w.permute(0, 2, 1).contiguous()                    # es_fused takes [E, out, in] (reference layers.py:407)
        r_ess, dx, r_dw = es_fused(dy.to(dtype), x.to(dtype), wt.to(dtype), (tok + 1).contiguous(), exp, starts, E, bias=True)
        for got, key in ((y_b, "y_bias"), (y_nb, "y_nobias"), (dx, "dx")):
            want = torch.from_numpy(z[f"{c}/{key}"])
            err = float((got.float().cpu() - want).abs().max() / want.abs().max())
            assert err < tol, (c, key, err)
        assert y_b.dtype == dtype and y_b.shape == (x.shape[0], w.shape[2])


def test_fused_ess_estmm_equal_reference_where_it_is_correct(golden_dir):
    from hexa_moe_b200.kernels.basics import counter
    from hexa_moe_b200.kernels.fused import es_fused
    z = np.load(os.path.join(golden_dir, "estmm_ess.npz"))
    for c in _cases(z):
        x, w, dy = (torch.from_numpy(z[f"{c}/{k}"]).cuda() for k in ("x", "w", "dy"))
        routing = torch.from_numpy(z[c + "/routing"]).cuda()
        E = int(z[c + "/E"])
        n, starts, tok, exp = counter(routing, E)
        wt = w.permute(0, 2, 1).contiguous().half()
        r_ess, dx, r_dw = es_fused(dy.half(), x.half(), wt, (tok + 1).contiguous(), exp, starts, E, bias=True)
        ess_ref, dw_ref = z[c + "/ess"], z[c + "/estmm"]
        written = ~np.isnan(ess_ref).any(axis=1)              # the reference never writes trailing empty experts
        got_ess, got_dw = r_ess.float().cpu().numpy(), r_dw.float().cpu().numpy()
        assert np.abs(got_ess[written] - ess_ref[written]).max() / np.abs(ess_ref[written]).max() < 2e-3
        assert np.abs(got_dw[written] - dw_ref[written]).max() / np.abs(dw_ref[written]).max() < 2e-3
        counts = np.bincount(routing.cpu().numpy(), minlength=E)
        assert (got_ess[counts == 0] == 0).all() and (got_dw[counts == 0] == 0).all()
