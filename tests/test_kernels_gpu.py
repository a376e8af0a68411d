"""Parity of every CUDA operator with the CPU oracle, called through the C ABI.  Needs a B200.

Tolerances (stated by the task): routing and indices bit-exact; fp32 within 1e-5 relative;
16-bit within 2e-2 relative.  "Relative" is measured against the largest magnitude of the
expected tensor (norm-wise), the usual meaning for accumulated dot products.
"""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import hexa_oracle as O

pytestmark = pytest.mark.gpu

REL = {torch.float32: 1e-5, torch.float16: 2e-2, torch.bfloat16: 2e-2}


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from hexa_moe_b200 import ops as _ops
    return _ops


def L():
    from hexa_moe_b200 import _lib
    return _lib


def rel_err(got, want):
    got = got.detach().double().cpu(); want = want.detach().double().cpu()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def make_ids(T, k, E, seed, skew=False, empty=()):
    g = torch.Generator().manual_seed(seed)
    if skew:
        p = torch.arange(1, E + 1, dtype=torch.float64) ** -1.2
    else:
        p = torch.ones(E, dtype=torch.float64)
    for e in empty:
        p[e] = 0
    ids = torch.multinomial(p.expand(T, E), k, replacement=False, generator=g)
    return ids.to(torch.int32)


# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("T,k,E,align", [(100, 1, 4, 16), (1000, 2, 8, 128), (4097, 2, 64, 128), (513, 4, 7, 128),
                                         (64, 1, 3, 128), (1, 1, 5, 128), (3000, 2, 300, 16)])
def test_route_bit_exact(ops, T, k, E, align):
    ids = make_ids(T, k, E, seed=T + k, skew=(E > 4), empty=(1,) if E > 2 else ())
    if T > 50:
        ids[5, 0] = -1          # out-of-range ids are skipped, as in the reference kernels
        ids[7, k - 1] = E
    r = ops.route(ids.cuda(), E, align)
    want = O.route(ids, E, align)
    n_pad = want["n_pad"]
    assert torch.equal(r.counts.cpu(), want["counts"])
    assert torch.equal(r.seg_offsets.cpu(), want["seg_offsets"])
    assert torch.equal(r.pad_offsets.cpu(), want["pad_offsets"])
    assert torch.equal(r.row_token.cpu()[:n_pad], want["row_token"])
    assert torch.equal(r.token_row.cpu()[: T * k], want["token_row"])
    te = r.tile_expert.cpu()
    assert torch.equal(te[: n_pad // align], want["tile_expert"])
    assert (te[n_pad // align: r.row_capacity // align] == -1).all()
    if align == 128:
        pb = r.pair_block.cpu()
        n_pairs = want["pair_block"].numel()
        assert torch.equal(pb[:n_pairs], want["pair_block"]) and (pb[n_pairs:] == -1).all() and pb.numel() > n_pairs
    else:
        assert r.pair_block is None
    # route-major ids ([k, T]) give the same answer
    r2 = ops.route(ids.t().contiguous().cuda(), E, align, route_major=True)
    assert torch.equal(r2.row_token.cpu()[:n_pad], want["row_token"])
    assert torch.equal(r2.token_row.cpu()[: T * k], want["token_row"])


def test_route_matches_reference_counter(ops, golden_dir):
    """align=16 reproduces the reference's own lists (golden fixture from kernels/basics.py:counter)."""
    import os
    z = np.load(os.path.join(golden_dir, "counter.npz"))
    for c in sorted({k.split("/")[0] for k in z.files}):
        routing = torch.from_numpy(z[c + "/routing"]); E = int(z[c + "/E"])
        r = ops.route(routing.view(-1, 1).cuda(), E, 16)
        n = int(z[c + "/n"])
        assert int(r.pad_offsets[-1]) == n
        assert np.array_equal(r.pad_offsets.cpu().numpy(), z[c + "/starts"])
        assert np.array_equal(r.row_token.cpu().numpy()[:n], z[c + "/tok_ids"])
        assert np.array_equal(r.tile_expert.cpu().numpy()[: n // 16], z[c + "/exp_ids"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cols", [64, 200, 3])
def test_gather_combine(ops, dtype, cols):
    T, k, E = 777, 2, 6
    ids = make_ids(T, k, E, 3, empty=(2,))
    r = ops.route(ids.cuda(), E)
    want = O.route(ids, E, 128)
    x = torch.randn(T, cols).to(dtype)
    xs = ops.gather_rows(x.cuda(), r).cpu()
    rt = want["row_token"].long()
    exp = torch.where((rt >= 0).unsqueeze(1), x[rt.clamp_min(0)], torch.zeros((), dtype=dtype))
    assert torch.equal(xs[: want["n_pad"]], exp)
    y = ops.combine_rows(xs.cuda(), r).cpu()
    exp_y = (x.double() * k).to(dtype) if dtype == torch.float32 else None
    # combine of gathered rows = k * x (each token appears once per route), fp32 accumulation then one rounding
    torch.testing.assert_close(y.double(), (x.double() * k).to(dtype).double(), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ess(ops, dtype):
    T, k, E, n = 3000, 2, 16, 328
    ids = make_ids(T, k, E, 5, skew=True, empty=(3, 15))
    r = ops.route(ids.cuda(), E)
    dy = torch.randn(T, n).to(dtype)
    dys = ops.gather_rows(dy.cuda(), r)
    got = ops.ess(dys, r).cpu()
    want = sum(O.ess(dy, ids[:, j], E) for j in range(k))
    assert rel_err(got, want) < 1e-5          # fp32 accumulation for every input dtype
    assert (got[3] == 0).all() and (got[15] == 0).all()
    got2 = ops.ess(dys, r).cpu()
    assert torch.equal(got, got2)             # deterministic


def _esmm_case(ops, dtype, engine, T, k, E, K, N, b_layout, epilogue, act, seed=0, bias=True):
    Lb = L()
    ids = make_ids(T, k, E, seed, skew=True, empty=(1,))
    r = ops.route(ids.cuda(), E)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, K, generator=g).to(dtype)
    w = (torch.randn(E, K, N, generator=g) / K ** 0.5).to(dtype)          # [E, K, N]
    b = torch.randn(E, N, generator=g) if bias else None
    wdev = (w.transpose(1, 2).contiguous() if b_layout == Lb.B_NK else w).cuda()
    xs = ops.gather_rows(x.cuda(), r)
    bdev = None if b is None else ops._f32(b.cuda())            # rows padded to whole 16-byte chunks when N % 4 != 0
    aux_pre = None
    if epilogue == Lb.EPI_DACT:
        pre = torch.randn(T, N, generator=g).to(dtype)
        aux_pre = ops.gather_rows(pre.cuda(), r)
        out = ops.esmm(xs, wdev, b_layout, r, bdev, epilogue, act, aux=aux_pre, engine=engine)
    elif epilogue == Lb.EPI_ACT:
        aux_pre = ops.sorted_buffer(r.row_capacity, N, dtype, "cuda")
        out = ops.esmm(xs, wdev, b_layout, r, bdev, epilogue, act, aux=aux_pre, engine=engine)
    else:
        out = ops.esmm(xs, wdev, b_layout, r, bdev, epilogue, act, engine=engine)
    torch_act = {Lb.ACT_NONE: lambda t: t, Lb.ACT_RELU: F.relu, Lb.ACT_GELU: F.gelu,
                 Lb.ACT_GELU_TANH: lambda t: F.gelu(t, approximate="tanh"), Lb.ACT_SILU: F.silu}[act]
    n_pad = int(r.pad_offsets[-1])
    tol = REL[dtype]
    for j in range(k):
        lin = O.esmm(x, w, b, ids[:, j])                                   # float64, token order
        rows = r.token_row.view(T, k)[:, j].cpu().long()
        got = out.cpu()[rows]
        if epilogue == Lb.EPI_LINEAR:
            want = lin
        elif epilogue == Lb.EPI_ACT:
            want = torch_act(lin)
            assert rel_err(aux_pre.cpu()[rows], lin) < tol
        else:
            _, gr = O.act_and_grad(torch_act, pre.double())
            want = lin * gr
        assert rel_err(got, want) < tol, (j, rel_err(got, want))
    # pad rows are zeros
    pad = (r.row_token[:n_pad] < 0).cpu()
    assert (out.cpu()[:n_pad][pad] == 0).all()
    return out


@pytest.mark.parametrize("b_layout", [0, 1])
@pytest.mark.parametrize("epilogue,act", [(0, 0), (1, 2), (2, 2), (1, 1), (2, 4), (1, 3)])
def test_esmm_simt_fp32(ops, b_layout, epilogue, act):
    _esmm_case(ops, torch.float32, L().ENGINE_SIMT, T=500, k=2, E=5, K=72, N=100, b_layout=b_layout, epilogue=epilogue, act=act)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b_layout", [0, 1])
def test_esmm_tcgen05_linear(ops, dtype, b_layout):
    _esmm_case(ops, dtype, L().ENGINE_TCGEN05, T=1500, k=2, E=6, K=256, N=512, b_layout=b_layout, epilogue=0, act=0)


@pytest.mark.parametrize("b_layout,K,N", [(0, 200, 328), (1, 200, 328), (0, 64, 128), (1, 1024, 64), (0, 776, 2048)])
def test_esmm_tcgen05_ragged_dims(ops, b_layout, K, N):
    """K not a multiple of 64 (TMA zero fill), N not a multiple of the tile, both tile widths."""
    _esmm_case(ops, torch.bfloat16, L().ENGINE_TCGEN05, T=900, k=2, E=4, K=K, N=N, b_layout=b_layout, epilogue=0, act=0, seed=2)


@pytest.mark.parametrize("b_layout,K,N,epilogue", [(0, 128, 203, 0), (0, 128, 203, 1), (0, 256, 1639, 2), (1, 203, 128, 0),
                                                   (1, 1639, 256, 0), (0, 64, 1229, 1)])
def test_esmm_tcgen05_odd_widths(ops, b_layout, K, N, epilogue):
    """Output widths and contraction lengths that are not multiples of 8: a rank's slice of an unevenly split hidden
    dimension (8192 x 0.2 = 1639 columns).  The buffers keep a 16-byte row pitch, the tensor cores do the work."""
    _esmm_case(ops, torch.bfloat16, L().ENGINE_TCGEN05, T=700, k=2, E=3, K=K, N=N, b_layout=b_layout, epilogue=epilogue,
               act=2 if epilogue else 0, seed=6)


@pytest.mark.parametrize("epilogue,act", [(1, 2), (2, 2), (1, 1), (2, 1), (1, 4), (2, 3)])
def test_esmm_tcgen05_epilogues(ops, epilogue, act):
    _esmm_case(ops, torch.bfloat16, L().ENGINE_TCGEN05, T=700, k=1, E=3, K=128, N=384, b_layout=0, epilogue=epilogue, act=act, seed=4)


def test_esmm_tcgen05_equals_simt_many_tiles(ops):
    """More tiles than SMs so every CTA loops over several tiles and both accumulators are reused."""
    Lb = L()
    T, k, E, K, N = 12000, 2, 8, 192, 1024
    ids = make_ids(T, k, E, 9, skew=True)
    r = ops.route(ids.cuda(), E)
    x = torch.randn(T, K).bfloat16().cuda()
    w = (torch.randn(E, N, K) / K ** 0.5).bfloat16().cuda()
    b = torch.randn(E, N).cuda()
    xs = ops.gather_rows(x, r)
    a = ops.esmm(xs, w, Lb.B_NK, r, b, engine=Lb.ENGINE_TCGEN05)
    s = ops.esmm(xs, w, Lb.B_NK, r, b, engine=Lb.ENGINE_SIMT)
    n_pad = int(r.pad_offsets[-1])
    assert rel_err(a[:n_pad], s[:n_pad]) < 1e-2
    a2 = ops.esmm(xs, w, Lb.B_NK, r, b, engine=Lb.ENGINE_TCGEN05)
    assert torch.equal(a[:n_pad], a2[:n_pad])


def _estmm_case(ops, dtype, engine, T, k, E, M, N, out_dtype, seed=0):
    ids = make_ids(T, k, E, seed, skew=True, empty=(0, E - 1))
    r = ops.route(ids.cuda(), E)
    g = torch.Generator().manual_seed(seed)
    p = torch.randn(T, M, generator=g).to(dtype); q = torch.randn(T, N, generator=g).to(dtype)
    # every route sees its own p rows in the layer; here the same token rows are used for all routes
    ps = ops.gather_rows(p.cuda(), r); qs = ops.gather_rows(q.cuda(), r)
    got = ops.estmm(ps, qs, r, out_dtype=out_dtype, engine=engine)
    want = sum(O.estmm(p, q, ids[:, j], E) for j in range(k))            # [E, M, N]
    tol = REL[out_dtype] if out_dtype != torch.float32 else REL[dtype] if dtype != torch.float32 else 1e-5
    # 16-bit inputs are exact in the oracle, so an fp32 output must be accurate to fp32 accumulation
    if out_dtype == torch.float32:
        tol = 2e-5
    assert rel_err(got, want) < tol, rel_err(got, want)
    assert (got[0] == 0).all() and (got[E - 1] == 0).all()                 # empty experts are written as zeros
    got_b = ops.estmm(ps, qs, r, out=got.clone(), beta=1, engine=engine)
    assert rel_err(got_b, 2 * want) < max(tol, 1e-2 if out_dtype != torch.float32 else tol)
    return got


@pytest.mark.parametrize("dtype,engine", [(torch.bfloat16, 1), (torch.float32, 2)])
def test_estmm_rank_grouped_layout_and_copy_2d(ops, dtype, engine):
    """ranks=W writes the gradient as [W, E, m/W, n] (what a reduce-scatter over the hidden dimension reads);
    copy_2d moves hidden slices between that layout and [E, m, n]."""
    T, k, E, M, N, W = 1500, 2, 5, 512, 256, 4
    ids = make_ids(T, k, E, 8, skew=True)
    r = ops.route(ids.cuda(), E)
    p = ops.gather_rows(torch.randn(T, M).to(dtype).cuda(), r); q = ops.gather_rows(torch.randn(T, N).to(dtype).cuda(), r)
    plain = ops.estmm(p, q, r, out_dtype=torch.float32, engine=engine)
    grouped = ops.estmm(p, q, r, out_dtype=torch.float32, engine=engine, ranks=W)
    assert grouped.shape == (W, E, M // W, N)
    assert torch.equal(grouped.permute(1, 0, 2, 3).reshape(E, M, N), plain)
    back = torch.empty_like(plain)
    for w in range(W):
        ops.copy_2d(back[:, w * (M // W):(w + 1) * (M // W)], back.stride(0), grouped[w], grouped.stride(1), (M // W) * N, E)
    assert torch.equal(back, plain)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,W", [(512, 4), (768, 2), (1024, 8)])
def test_estmm_scatter_to_per_owner_buffers(ops, out_dtype, M, W):
    """A list of W outputs: slice w of the hidden dimension is stored straight into out[w] ([E, M/W, N]).
    Bit-identical to the rank-grouped single-buffer layout, and nothing outside the slices is touched."""
    T, k, E, N = 1500, 2, 5, 256
    ids = make_ids(T, k, E, 8, skew=True)
    r = ops.route(ids.cuda(), E)
    p = ops.gather_rows(torch.randn(T, M).bfloat16().cuda(), r); q = ops.gather_rows(torch.randn(T, N).bfloat16().cuda(), r)
    grouped = ops.estmm(p, q, r, out_dtype=out_dtype, ranks=W)
    arena = torch.full((W, 2, E, M // W, N), 7.0, dtype=out_dtype, device="cuda")      # slot 1 of every owner is the target
    outs = [arena[w, 1] for w in range(W)]
    back = ops.estmm(p, q, r, ranks=W, out=outs)
    assert back is outs
    for w in range(W):
        assert torch.equal(outs[w], grouped[w])
        assert (arena[w, 0] == 7.0).all()
    with pytest.raises(L().HexaError):
        ops.estmm(p, q, r, ranks=W, out=outs[:-1])


def test_estmm_simt_fp32(ops):
    _estmm_case(ops, torch.float32, L().ENGINE_SIMT, T=900, k=2, E=6, M=100, N=72, out_dtype=torch.float32)


@pytest.mark.parametrize("dtype,out_dtype", [(torch.bfloat16, torch.float32), (torch.bfloat16, torch.bfloat16),
                                             (torch.float16, torch.float32)])
@pytest.mark.parametrize("M,N", [(256, 512), (200, 328), (128, 64), (1000, 136)])
def test_estmm_tcgen05(ops, dtype, out_dtype, M, N):
    _estmm_case(ops, dtype, L().ENGINE_TCGEN05, T=2500, k=2, E=7, M=M, N=N, out_dtype=out_dtype, seed=M)


@pytest.mark.parametrize("E,M,N,out_dtype,ranks", [(1, 256, 512, torch.float32, 1), (1, 512, 128, torch.bfloat16, 1),
                                                    (3, 256, 256, torch.float32, 2), (2, 200, 136, torch.bfloat16, 1)])
def test_estmm_split_segments(ops, E, M, N, out_dtype, ranks):
    """Few output tiles and long segments (the dense FFN's weight gradient is the E = 1 case): with scratch the kernel
    cuts every segment into chunks and adds the fp32 partial results in chunk order.  Same answer as the oracle and as
    the unsplit kernel, bit-identical from run to run, beta and the rank-grouped layout honoured, an expert without
    rows written as zeros."""
    Lb = L()
    T, k = 6000, 1
    g = torch.Generator().manual_seed(E * 100 + M)
    ids = torch.randint(0, max(E - 1, 1), (T, k), generator=g).to(torch.int32)          # the last of several experts stays empty
    r = ops.route(ids.cuda(), E)
    p = torch.randn(T, M, generator=g).bfloat16(); q = torch.randn(T, N, generator=g).bfloat16()
    ps, qs = ops.gather_rows(p.cuda(), r), ops.gather_rows(q.cuda(), r)
    lib = Lb.lib()
    need = lib.hexa_estmm_workspace_bytes(E, r.row_capacity, M, N, Lb.BF16)
    assert need > 0, "this shape is meant to take the split path"
    got = ops.estmm(ps, qs, r, out_dtype=out_dtype, engine=Lb.ENGINE_TCGEN05, ranks=ranks)
    flat = got.permute(1, 0, 2, 3).reshape(E, M, N) if ranks > 1 else got
    want = O.estmm(p, q, ids[:, 0], E)
    tol = 2e-5 if out_dtype == torch.float32 else 2e-2
    assert rel_err(flat, want) < tol, rel_err(flat, want)
    if E > 1:
        assert (flat[E - 1] == 0).all()
    for _ in range(3):
        assert torch.equal(ops.estmm(ps, qs, r, out_dtype=out_dtype, engine=Lb.ENGINE_TCGEN05, ranks=ranks), got)
    # the unsplit kernel (no scratch offered) on the same inputs
    plain = torch.empty(E, M, N, dtype=out_dtype, device="cuda")
    Lb.check(lib.hexa_estmm(ps.data_ptr(), ps.stride(0), qs.data_ptr(), qs.stride(0), r.pad_offsets.data_ptr(), E, r.row_capacity,
                            M, N, plain.data_ptr(), plain.stride(1), plain.stride(0), 0, 0, Lb.BF16, Lb.dt(plain), 0,
                            Lb.ENGINE_TCGEN05, None, 0, torch.cuda.current_stream().cuda_stream), "hexa_estmm")
    assert rel_err(flat, plain) < (2e-5 if out_dtype == torch.float32 else 1e-2)     # fp32: another summation order
    if ranks == 1:
        twice = ops.estmm(ps, qs, r, out=got.clone(), beta=1, engine=Lb.ENGINE_TCGEN05)
        assert rel_err(twice, 2 * want) < max(tol, 1e-2 if out_dtype != torch.float32 else tol)


@pytest.mark.parametrize("dtype,E,k,d,H,act", [(torch.float32, 8, 1, 128, 512, "gelu"), (torch.bfloat16, 8, 2, 256, 1024, "gelu"),
                                               (torch.float16, 5, 2, 128, 320, "relu"), (torch.bfloat16, 4, 2, 128, 256, "generic"),
                                               (torch.bfloat16, 4, 2, 128, 203, "gelu"), (torch.bfloat16, 3, 1, 256, 1639, "gelu"),
                                               (torch.bfloat16, 4, 2, 128, 203, "generic")])
def test_layer_forward_backward(ops, dtype, E, k, d, H, act):
    Lb = L()
    T = 1200
    ids = make_ids(T, k, E, 21, skew=True, empty=(2,))
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, d, generator=g).to(dtype)
    w1 = (torch.randn(E, H, d, generator=g) / d ** 0.5).to(dtype)
    w2 = (torch.randn(E, H, d, generator=g) / H ** 0.5).to(dtype)
    b1 = (torch.randn(E, H, generator=g) * 0.1).to(dtype); b2 = (torch.randn(E, d, generator=g) * 0.1).to(dtype)
    dy = torch.randn(T, d, generator=g).to(dtype)
    fn = {"gelu": F.gelu, "relu": F.relu, "generic": lambda t: torch.sigmoid(t) * t * 1.5}[act]
    act_id = {"gelu": Lb.ACT_GELU, "relu": Lb.ACT_RELU, "generic": -1}[act]
    # 16-bit data must run on the tensor-core kernels whatever the hidden width (no silent CUDA-core fallback)
    engine = Lb.ENGINE_TCGEN05 if dtype != torch.float32 else Lb.ENGINE_AUTO
    y, st = ops.moe_forward(x.cuda(), ids.cuda(), w1.cuda(), w2.cuda(), b1.cuda(), b2.cuda(), act_id, act_fn=fn, engine=engine)
    dx, dw1, dw2, db1, db2 = ops.moe_backward(st, dy.cuda(), w1.cuda(), w2.cuda(), act_id, grad_dtype=torch.float32,
                                              engine=engine)
    want = O.moe_layer(x, ids, w1, w2, b1, b2, fn, dy)
    tol = REL[dtype]
    for name, got, exp in (("y", y, want["y"]), ("dx", dx, want["dx"]), ("dw1", dw1, want["dw1"]), ("dw2", dw2, want["dw2"]),
                           ("db1", db1, want["db1"]), ("db2", db2, want["db2"])):
        e = rel_err(got, exp)
        assert e < tol, (name, e)


@pytest.mark.parametrize("dtype,n_out", [(torch.bfloat16, 512), (torch.bfloat16, 128), (torch.float32, 96)])
def test_esmm_by_expert_groups_equals_one_launch(ops, dtype, n_out):
    """hexa_esmm_experts: launching the operator once per group of experts (any order) writes exactly what one launch
    over all experts writes, and a group's launch leaves the rows of other experts untouched."""
    Lb = L()
    T, k, E, d = 3000, 2, 7, 256
    ids = make_ids(T, k, E, 4, skew=True, empty=(3,))
    r = ops.route(ids.cuda(), E)
    g = torch.Generator().manual_seed(n_out)
    xs = ops.gather_rows(torch.randn(T, d, generator=g).to(dtype).cuda(), r)
    w = (torch.randn(E, n_out, d, generator=g) / 16).to(dtype).cuda()
    b = (torch.randn(E, n_out, generator=g) * 0.1).cuda()
    n_pad = int(r.pad_offsets[-1])
    full_aux = torch.zeros(r.row_capacity, n_out, dtype=dtype, device="cuda")
    full = ops.esmm(xs, w, Lb.B_NK, r, b, Lb.EPI_ACT, Lb.ACT_GELU, aux=full_aux)
    out = torch.full((r.row_capacity, n_out), 7.0, dtype=dtype, device="cuda")
    aux = torch.full_like(out, 7.0)
    ops.esmm(xs, w, Lb.B_NK, r, b, Lb.EPI_ACT, Lb.ACT_GELU, aux=aux, out=out, experts=(4, 7))
    lo = int(r.pad_offsets[4])
    assert (out[:lo] == 7.0).all() and (aux[:lo] == 7.0).all()                    # experts 0..3 untouched
    assert torch.equal(out[lo:n_pad], full[lo:n_pad]) and torch.equal(aux[lo:n_pad], full_aux[lo:n_pad])
    for e0, e1 in ((2, 4), (0, 2)):                                              # the remaining groups, out of order
        ops.esmm(xs, w, Lb.B_NK, r, b, Lb.EPI_ACT, Lb.ACT_GELU, aux=aux, out=out, experts=(e0, e1))
    assert torch.equal(out[:n_pad], full[:n_pad]) and torch.equal(aux[:n_pad], full_aux[:n_pad])
    ops.esmm(xs, w, Lb.B_NK, r, b, out=out, experts=(3, 3))                        # an empty range launches nothing
    with pytest.raises(Lb.HexaError):
        ops.esmm(xs, w, Lb.B_NK, r, b, out=out, experts=(5, 9))


@pytest.mark.parametrize("dtype,K,N,epilogue,b_layout", [(torch.bfloat16, 256, 512, 2, 0), (torch.float16, 256, 512, 2, 0),
                                                          (torch.bfloat16, 512, 328, 0, 1), (torch.bfloat16, 128, 64, 1, 0),
                                                          (torch.bfloat16, 256, 1639, 2, 0), (torch.float32, 64, 96, 0, 0)])
def test_esmm_with_fused_column_sums(ops, dtype, K, N, epilogue, b_layout):
    """hexa_esmm_ess: the output is bit-identical to hexa_esmm's and the sums are ESS of that output - on the tcgen05
    engine from the epilogue's staging tile (ragged column tiles, an empty expert, both 16-bit types, all epilogues),
    on the other engine (fp32, odd pitches) as the two-pass fallback.  Deterministic."""
    Lb = L()
    T, k, E = 2500, 2, 7
    ids = make_ids(T, k, E, 11, skew=True, empty=(2,))
    r = ops.route(ids.cuda(), E)
    g = torch.Generator().manual_seed(3)
    xs = ops.gather_rows(torch.randn(T, K, generator=g).to(dtype).cuda(), r)
    w = (torch.randn(E, K, N, generator=g) / K ** 0.5).to(dtype)
    wdev = (w.transpose(1, 2).contiguous() if b_layout == Lb.B_NK else w).cuda()
    bias = ops._f32(torch.randn(E, N, generator=g).cuda()) if epilogue != Lb.EPI_DACT else None
    aux = None
    if epilogue == Lb.EPI_DACT:
        aux = ops.gather_rows(torch.randn(T, N, generator=g).to(dtype).cuda(), r)
    elif epilogue == Lb.EPI_ACT:
        aux = ops.sorted_buffer(r.row_capacity, N, dtype, xs.device)
    act = Lb.ACT_GELU if epilogue != Lb.EPI_LINEAR else Lb.ACT_NONE
    plain = ops.esmm(xs, wdev, b_layout, r, bias, epilogue, act, aux=aux)
    sums = torch.full((E, N), float("nan"), dtype=torch.float32, device="cuda")
    fused = ops.esmm(xs, wdev, b_layout, r, bias, epilogue, act, aux=aux, sums=sums)
    n_pad = int(r.pad_offsets[-1])
    assert torch.equal(fused[:n_pad], plain[:n_pad])
    want = ops.ess(plain, r)
    assert torch.isfinite(sums).all()
    assert rel_err(sums, want) < 1e-5
    assert (sums[2] == 0).all()                                   # the empty expert
    sums2 = torch.empty_like(sums)
    ops.esmm(xs, wdev, b_layout, r, bias, epilogue, act, aux=aux, sums=sums2)
    assert torch.equal(sums, sums2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("n_recv", [0, 1, 2, 3, 5, 7])
def test_mean_slices(ops, dtype, n_recv):
    """The reduction step of the peer-copy reduce-scatter: out = (local + received slices) / world with fp32
    accumulation in slice order, for slice counts with and without an unrolled variant and sizes that leave a tail."""
    world = n_recv + 1
    for elems in (8 * 1000, 8 * 128 * 8 * 37 + 8 * 5, 1 << 22):
        g = torch.Generator().manual_seed(elems % 1000 + n_recv)
        local = torch.randn(elems, generator=g).to(dtype).cuda()
        recv = torch.randn(max(n_recv, 1), elems, generator=g).to(dtype).cuda()
        out = torch.empty_like(local)
        ops.mean_slices(local, recv, n_recv, world, out)
        acc = local.float()
        for s_ in range(n_recv):
            acc = acc + recv[s_].float()
        want = (acc * (1.0 / world)).to(dtype)
        assert torch.equal(out, want), (elems, float((out.float() - want.float()).abs().max()))


def test_errors_are_reported_not_fatal(ops):
    Lb = L()
    ids = make_ids(64, 1, 4, 0)
    r = ops.route(ids.cuda(), 4)
    a = torch.zeros(r.row_capacity, 20, dtype=torch.bfloat16, device="cuda")      # lda = 20: not a multiple of 8
    b = torch.zeros(4, 16, 20, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(Lb.HexaError, match="tcgen05"):
        ops.esmm(a, b, Lb.B_NK, r, engine=Lb.ENGINE_TCGEN05)
    out = ops.esmm(a, b, Lb.B_NK, r)                # AUTO falls back to the CUDA-core kernel
    assert out.shape == (r.row_capacity, 16)
    with pytest.raises(Lb.HexaError):
        ops.route(ids.cuda().long(), 4)
    with pytest.raises(Lb.HexaError, match="CUDA tensors only"):
        ops.route(ids, 4)
