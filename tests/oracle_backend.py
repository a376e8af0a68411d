"""Test double for `config.backend`: the CPU oracle behind the interface of hexa_moe_b200.ops.

Only tests use it - to exercise the multi-rank host logic (sharding, gathers, reductions) on
CPU `gloo` ranks, where the CUDA kernels cannot run.  The product never imports this file.
"""
import torch

from oracle import hexa_oracle as O


class _State:
    pass


def moe_forward(x, ids, w1, w2, b1, b2, act_id, act_fn=None, route_major=False, engine=0, need_state=True, before_fc2=None):
    if before_fc2 is not None:
        before_fc2()
    ids_tk = ids.t().contiguous() if route_major else ids
    st = _State()
    st.x, st.ids, st.w1, st.w2, st.b1, st.b2, st.act = x, ids_tk, w1, w2, b1, b2, act_fn
    res = O.moe_layer(x, ids_tk, w1, w2, b1, b2, act_fn)
    return res["y"].to(x.dtype), st


def _full(st, dy):
    if not hasattr(st, "res"):
        b2 = st.b2 if st.b2 is not None else torch.zeros(st.w2.shape[0], st.w2.shape[2])
        b1 = st.b1 if st.b1 is not None else torch.zeros(st.w1.shape[0], st.w1.shape[1])
        st.res = O.moe_layer(st.x, st.ids, st.w1, st.w2, b1, b2, st.act, dy)
    return st.res


def moe_backward_fc2(st, dy, w2, act_id, has_b2=True, grad_dtype=None, engine=0, ranks=1, want_db1=False):
    r = _full(st, dy)
    gd = grad_dtype or dy.dtype
    return None, r["dw2"].to(gd), (r["db2"].float() if has_b2 else None)


def moe_backward_fc1(st, dh, w1, has_b1=True, grad_dtype=None, engine=0, ranks=1, after_dw=None):
    r = st.res
    gd = grad_dtype or st.x.dtype
    dw1, db1 = r["dw1"].to(gd), (r["db1"].float() if has_b1 else None)
    if after_dw is not None:
        after_dw(dw1, db1)
    return r["dx"].to(st.x.dtype), dw1, db1


def moe_backward_inputs(st, dy, w1, w2, act_id, engine=0, want_db1=False):
    r = _full(st, dy)
    return r["dx"].to(st.x.dtype), (st, dy)


def moe_backward_params(st, kept, has_b1=True, has_b2=True, grad_dtype=None, engine=0, into=None):
    r = st.res
    gd = grad_dtype or st.x.dtype
    new = (r["dw1"].to(gd), r["dw2"].to(gd), r["db1"].float() if has_b1 else None, r["db2"].float() if has_b2 else None)
    if into is None:
        return new
    for acc, g in zip(into, new):
        if g is not None:
            acc += g
    return into
