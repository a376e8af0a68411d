"""`es_fused`: the reference's backward operator, same arguments and result tuple
(hexa_moe_triton/hexa_moe/kernels/fused.py:382-450): ESS, the ESMM input gradient and ESTMM of one route.

ESS and ESTMM follow the operator definition; the reference's kernels agree with it only while every expert has at
most 16 rows (they consume the first 16-row chunk twice and never the last one, fused.py:123-134, 199-221) and
leave experts behind the last non-empty one uninitialised."""
import torch

from .. import _lib as L
from .. import ops
from .esmm import ids_from_lists


def es_fused(tok1, tok2, w, tok_ids_list, exp_ids_list, exp_start_list, num_exps, bias=True):
    """tok1 [T, out] (the incoming gradient), tok2 [T, in] (the layer input), w [E, out, in].
    Returns (r_ess [E, out] if bias, r_esmm [T, in] = tok1[t] @ w[e(t)], r_estmm [E, out, in] = sum_t tok1[t]^T tok2[t])."""
    assert tok1.dtype == tok2.dtype and tok1.shape[0] == tok2.shape[0]
    assert tok2.shape[1] == w.shape[2] and num_exps == w.shape[0] and tok1.shape[1] == w.shape[1]
    assert exp_start_list.shape[0] == 1 + num_exps
    assert tok1.is_contiguous() and tok2.is_contiguous()
    ids = ids_from_lists(tok1.shape[0], tok_ids_list, exp_ids_list)
    r = ops.route(ids.view(-1, 1), num_exps)
    g = ops.gather_rows(tok1, r)
    x = ops.gather_rows(tok2, r)
    r_esmm = ops.combine_rows(ops.esmm(g, w.to(tok1.dtype).contiguous(), L.B_KN, r), r)
    r_estmm = ops.estmm(g, x, r, out_dtype=torch.float32 if w.dtype == torch.float32 else tok1.dtype).to(w.dtype)
    if bias:
        return ops.ess(g, r).to(w.dtype), r_esmm, r_estmm
    return r_esmm, r_estmm
