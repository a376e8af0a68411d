"""Generate the golden fixtures in this directory from the UNMODIFIED reference sources.

Run once, on a machine that has a checkout of the reference (UNITES-Lab/HEXA-MoE) and triton:

    python tests/golden/make_golden.py --ref <path to the HEXA-MoE checkout>

The reference's Triton kernels are executed on CPU tensors with TRITON_INTERPRET=1.  Three tiny
import shims (an empty `constant` namespace, an attribute-dict `easydict.EasyDict`, and
`timm.models.layers.trunc_normal_` forwarded to torch) are written to a temporary directory so
the package imports; the autotuner is bypassed by calling the wrapped jit function with one fixed
tile configuration, because autotuning needs a GPU driver.  No reference source is copied.

Outputs (small .npz files, committed):
  counter.npz   routing lists of kernels/basics.py:counter for several id vectors
  esmm.npz      ESMM forward (bias / no bias) and the ESMM-dX part of es_fused
  estmm_ess.npz ESTMM and ESS of es_fused on inputs where every expert has <= 16 rows (the only
                regime in which the reference kernels implement the operator definition)
  module.npz    MoE_Cascaded toy network: parameters, input, per-depth outputs, l_aux, input grad
"""
import argparse
import os
import sys
import tempfile

os.environ["TRITON_INTERPRET"] = "1"
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
os.environ.setdefault("MASTER_PORT", "29577")
os.environ.setdefault("RANK", "0")
os.environ.setdefault("WORLD_SIZE", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
CFG = dict(BLOCK_SIZE_M=16, BLOCK_SIZE_N=32, BLOCK_SIZE_K=32, GROUP_SIZE_M=8)


def write_shims(d):
    os.makedirs(os.path.join(d, "timm", "models"), exist_ok=True)
    open(os.path.join(d, "constant.py"), "w").write("MAX_TOKEN_CHUNK = 16\n")
    open(os.path.join(d, "easydict.py"), "w").write(
        "class EasyDict(dict):\n"
        "    def __getattr__(self, k):\n"
        "        try:\n            return self[k]\n        except KeyError:\n            raise AttributeError(k)\n"
        "    def __setattr__(self, k, v):\n        self[k] = v\n")
    open(os.path.join(d, "timm", "__init__.py"), "w").write("")
    open(os.path.join(d, "timm", "models", "__init__.py"), "w").write("")
    open(os.path.join(d, "timm", "models", "layers.py"), "w").write("from torch.nn.init import trunc_normal_\n")


def routing_cases():
    g = torch.Generator().manual_seed(1234)
    cases = {}
    cases["uniform_T100_E4"] = (torch.randint(0, 4, (100,), generator=g, dtype=torch.int32), 4)
    cases["uniform_T257_E7"] = (torch.randint(0, 7, (257,), generator=g, dtype=torch.int32), 7)
    r = torch.randint(0, 8, (64,), generator=g, dtype=torch.int32)
    r[r == 3] = 5; r[r == 0] = 1                       # experts 0 and 3 empty
    cases["empty_experts_T64_E8"] = (r, 8)
    cases["one_expert_T50_E5"] = (torch.full((50,), 2, dtype=torch.int32), 5)
    cases["exact16_T32_E2"] = (torch.tensor([0] * 16 + [1] * 16, dtype=torch.int32), 2)
    cases["single_token_E3"] = (torch.tensor([1], dtype=torch.int32), 3)
    return cases


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("HEXA_MOE_REFERENCE", "reference"),
                    help="path of the HEXA-MoE checkout (or set HEXA_MOE_REFERENCE)")
    args = ap.parse_args()
    shim = tempfile.mkdtemp(prefix="hexa_shims_")
    write_shims(shim)
    sys.path.insert(0, shim)
    sys.path.insert(0, os.path.join(args.ref, "hexa_moe_triton"))
    import triton
    from hexa_moe.kernels.basics import counter
    from hexa_moe.kernels import esmm as M, fused as Fz

    # ---------------- counter ----------------
    out = {}
    for name, (r, E) in routing_cases().items():
        n, starts, tok, exp = counter(r, E)
        out[name + "/routing"] = r.numpy(); out[name + "/E"] = np.int64(E); out[name + "/n"] = np.int64(n)
        out[name + "/starts"] = starts.numpy(); out[name + "/tok_ids"] = tok.numpy(); out[name + "/exp_ids"] = exp.numpy()
    np.savez_compressed(os.path.join(HERE, "counter.npz"), **out)

    # ---------------- ESMM fwd + dX ----------------
    def run_esmm(x, w, b, tok_ids, exp_ids, n):
        T, din = x.shape; E, _, dout = w.shape
        xp = torch.cat([torch.zeros(1, din), x]).contiguous()
        w2 = w.reshape(E * din, dout).contiguous()
        tid = (tok_ids + 1).contiguous()
        c = torch.zeros(T, dout)
        grid = (triton.cdiv(n, 16) * triton.cdiv(dout, 32),)
        if b is not None:
            M.esmm_kernel_bias.fn[grid](c, xp, w2, b, tid, exp_ids, n, din, dout, xp.stride(0), xp.stride(1),
                                        w2.stride(0), w2.stride(1), b.stride(0), b.stride(1), c.stride(0), c.stride(1), **CFG)
        else:
            M.esmm_kernel_no_bias.fn[grid](c, xp, w2, tid, exp_ids, n, din, dout, xp.stride(0), xp.stride(1),
                                           w2.stride(0), w2.stride(1), c.stride(0), c.stride(1), **CFG)
        return c

    def run_fused(dy, x, w, tok_ids, exp_ids, starts, n):
        """w [E,din,dout] as ESMM takes it; es_fused wants its transpose [E,dout,din] (impls/layers.py:407)."""
        T, din = x.shape; E, _, dout = w.shape
        wt = w.permute(0, 2, 1).contiguous().reshape(E * dout, din).contiguous()
        dyp = torch.cat([torch.zeros(1, dout), dy]).contiguous()
        xp = torch.cat([torch.zeros(1, din), x]).contiguous()
        tid = (tok_ids + 1).contiguous()
        r_ess = torch.full((E, dout), float("nan")); r_dx = torch.full((T, din), float("nan"))
        r_dw = torch.full((E * dout, din), float("nan"))
        g = (E * triton.cdiv(dout, 32) + triton.cdiv(n, 16) * triton.cdiv(din, 32) + E * triton.cdiv(dout, 32) * triton.cdiv(din, 32),)
        Fz.fused_kernel_bias.fn[g](r_ess, r_dx, r_dw, dyp, xp, wt, tid, exp_ids, starts, n, T, E, din, dout,
                                   dyp.stride(0), dyp.stride(1), xp.stride(0), xp.stride(1), wt.stride(0), wt.stride(1),
                                   r_ess.stride(0), r_ess.stride(1), r_dx.stride(0), r_dx.stride(1),
                                   r_dw.stride(0), r_dw.stride(1), **CFG)
        return r_ess, r_dx, r_dw.reshape(E, dout, din)

    out = {}
    torch.manual_seed(7)
    for name, (T, E, din, dout) in {"a": (100, 4, 32, 48), "b": (77, 5, 40, 24)}.items():
        routing = torch.randint(0, E, (T,), dtype=torch.int32)
        n, starts, tok, exp = counter(routing, E)
        x = torch.randn(T, din); w = torch.randn(E, din, dout) * 0.1; b = torch.randn(E, dout); dy = torch.randn(T, dout)
        y_b = run_esmm(x, w, b, tok, exp, n)
        y_nb = run_esmm(x, w, None, tok, exp, n)
        _, dx, _ = run_fused(dy, x, w, tok, exp, starts, n)
        for k_, v in dict(routing=routing, x=x, w=w, b=b, dy=dy, y_bias=y_b, y_nobias=y_nb, dx=dx).items():
            out[f"{name}/{k_}"] = v.numpy()
        out[f"{name}/E"] = np.int64(E)
    np.savez_compressed(os.path.join(HERE, "esmm.npz"), **out)

    # ---------------- ESTMM + ESS where they are correct (<= 16 rows per expert) ----------------
    out = {}
    torch.manual_seed(11)
    for name, (T, E, din, dout) in {"a": (40, 6, 32, 48), "b": (16, 1, 24, 40), "c": (30, 8, 40, 32)}.items():
        while True:
            routing = torch.randint(0, E, (T,), dtype=torch.int32)
            if name == "c":
                routing[routing == 2] = 4                      # an empty expert in the middle
            if torch.bincount(routing.long(), minlength=E).max() <= 16:
                break
        n, starts, tok, exp = counter(routing, E)
        x = torch.randn(T, din); w = torch.randn(E, din, dout) * 0.1; dy = torch.randn(T, dout)
        r_ess, dx, r_dw = run_fused(dy, x, w, tok, exp, starts, n)
        for k_, v in dict(routing=routing, x=x, w=w, dy=dy, ess=r_ess, dx=dx, estmm=r_dw).items():
            out[f"{name}/{k_}"] = v.numpy()
        out[f"{name}/E"] = np.int64(E)
    np.savez_compressed(os.path.join(HERE, "estmm_ess.npz"), **out)

    # ---------------- module level ----------------
    import torch.distributed as dist
    import torch.nn.functional as F
    from triton.runtime.autotuner import Autotuner

    def _run(self, *a, **kw):
        return self.fn.run(*a, **kw, **self.configs[2].all_kwargs())
    Autotuner.run = _run
    dist.init_process_group("gloo")
    _ar = dist.all_reduce

    class _Done:
        def wait(self):
            pass

    def all_reduce(t, op=dist.ReduceOp.SUM, group=None, async_op=False):
        if op == dist.ReduceOp.AVG:                      # gloo has no AVG
            _ar(t, op=dist.ReduceOp.SUM, group=group); t.div_(dist.get_world_size()); return _Done()
        return _ar(t, op=op, group=group, async_op=async_op)
    dist.all_reduce = all_reduce
    from hexa_moe import moe as hmoe

    out = {}
    for tag, k in (("top1", 1), ("top2", 2)):
        torch.manual_seed(0)
        m = hmoe.MoE_Cascaded(gate_type={'type': 'top', 'k': k, 'gate_noise': 1.0, 'fp32_gate': True},
                              model_dim_list=[32] * 4, moe_idx_list=[2, 3], mlp_ratio=4, mlp_proportion=None,
                              num_global_experts=4, total_depth=4, data_centric=True, mlp_fc1_bias=True,
                              mlp_fc2_bias=True, activation_fn=lambda t: F.gelu(t))
        with torch.no_grad():                              # the module's own init is tiny (std 0.005); widen it
            for n_, p in m.named_parameters():
                if "bias" in n_ or n_.startswith("mlp_fc1_b") or n_.startswith("mlp_fc2_b"):
                    p.normal_(0, 0.1)
                elif "gates" in n_:
                    p.normal_(0, 0.5)
                else:
                    p.normal_(0, 0.2)
        m.eval()                                           # no gate noise: the RNG stream is not part of the contract
        x = torch.randn(2, 48, 32, requires_grad=True)
        h = x; laux = 0
        for d in range(4):
            h, l = m(d, h)
            laux = laux + l
            out[f"{tag}/y{d}"] = h.detach().numpy()
            out[f"{tag}/l_aux{d}"] = np.float64(float(l))
        (h.sum() + laux).backward()
        out[f"{tag}/x"] = x.detach().numpy(); out[f"{tag}/x_grad"] = x.grad.numpy()
        for n_, p in m.state_dict().items():
            out[f"{tag}/param/{n_}"] = p.numpy()
    np.savez_compressed(os.path.join(HERE, "module.npz"), **out)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
