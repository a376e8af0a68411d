"""`ESMM`: the reference's forward operator, same arguments and result
(hexa_moe_triton/hexa_moe/kernels/esmm.py:249-295).  The reference's lists (16-row chunks, token ids shifted by
one with 0 meaning "pad") are turned back into one expert id per token, which then takes the regular path of this
library: 128-row segmentation, row gather, grouped GEMM, scatter back to token order."""
import torch

from .. import _lib as L
from .. import ops
from .basics import MAX_TOKEN_CHUNK


def ids_from_lists(num_toks, tok_ids_list, exp_ids_list):
    """Expert id per token (-1: token not in any segment) from the reference's (tok_ids + 1, exp_ids) lists."""
    assert tok_ids_list.shape[0] == MAX_TOKEN_CHUNK * exp_ids_list.shape[0]
    ids = torch.full((num_toks + 1,), -1, dtype=torch.int32, device=tok_ids_list.device)
    ids[tok_ids_list.long()] = exp_ids_list.repeat_interleave(MAX_TOKEN_CHUNK).to(torch.int32)
    return ids[1:].contiguous()          # slot 0 collected the pad entries


def ESMM(toks, w, b, tok_ids_list, exp_ids_list):
    """toks [T, in]; w [E, in, out]; b [E, out] or an empty tensor; tok_ids_list = counter's list + 1;
    exp_ids_list per 16 rows.  Returns c [T, out] in toks' dtype: c[t] = toks[t] @ w[e(t)] (+ b[e(t)]), zero rows
    for tokens that are in no segment."""
    assert toks.is_contiguous() and w.is_contiguous() and toks.shape[1] == w.shape[1], "Matrix A must be contiguous"
    num_toks = toks.shape[0]
    num_exps, _, num_out_dims = w.shape
    ids = ids_from_lists(num_toks, tok_ids_list, exp_ids_list)
    r = ops.route(ids.view(-1, 1), num_exps)
    xs = ops.gather_rows(toks, r)
    bias = None
    if b is not None and b.numel():
        assert num_out_dims == b.shape[1] and num_exps == b.shape[0]
        bias = b.to(torch.float32).contiguous()
    ys = ops.esmm(xs, w.to(toks.dtype), L.B_KN, r, bias)
    return ops.combine_rows(ys, r)
