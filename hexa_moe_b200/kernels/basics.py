"""`counter`: the reference's routing entry point, same arguments and return values
(hexa_moe_triton/hexa_moe/kernels/basics.py:89-118), on the hexa_route kernel with 16-row alignment."""
import torch

from .. import ops

MAX_TOKEN_CHUNK = 16    # constant.MAX_TOKEN_CHUNK in the reference


def counter(routing, num_exps):
    """routing: int32 [T] expert id per token.  Returns (num_expanded_toks: int, exp_start_list int32 [E+1],
    tok_ids_list int32 [num_expanded] with -1 in the pad slots, exp_ids_list int32 [num_expanded / 16]).
    Returning a Python int forces one host synchronisation, as in the reference (its `.item()` calls)."""
    assert routing.dim() == 1
    r = ops.route(routing.contiguous().view(-1, 1), num_exps, MAX_TOKEN_CHUNK)
    n = int(r.pad_offsets[-1])
    return n, r.pad_offsets, r.row_token[:n].contiguous(), r.tile_expert[: n // MAX_TOKEN_CHUNK].contiguous()
