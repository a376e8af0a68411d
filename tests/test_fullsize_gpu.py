"""BASELINE-sized runs checked through size-independent properties (the CPU oracle cannot finish these sizes in
seconds): permutation / sortedness of the routing, sampled rows of ESMM against float64, column-sum identities for
ESS and ESTMM, and agreement of the tensor-core path with the fp32 CUDA-core path on sampled experts.

Sizes: the skewed-routing stress (65536 tokens, d=1024, hidden 4096, 64 experts, top-2, Zipf(1.2) with four experts
receiving nothing) and the large layer (131072 tokens, d=2048, hidden 8192, 64 experts, top-2)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from hexa_moe_b200 import ops as _ops
    return _ops


def zipf_ids(T, k, E, n_empty, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    perm = torch.randperm(E, generator=torch.Generator().manual_seed(seed))
    p = torch.arange(1, E + 1, dtype=torch.float64) ** -1.2
    p[E - n_empty:] = 0                       # the least likely experts get nothing
    p = p[torch.argsort(perm)]                # seeded relabelling of the experts
    ids = torch.multinomial(p.cuda().expand(T, E), k, replacement=False, generator=g)
    return ids.to(torch.int32), p


def check_routing(r, ids, E):
    T, k = ids.shape
    n_pad = int(r.pad_offsets[-1])
    counts = torch.bincount(ids.flatten().long(), minlength=E).int()
    assert torch.equal(r.counts, counts)
    assert (r.pad_offsets % 128 == 0).all() and n_pad <= r.row_capacity
    rt = r.row_token[:n_pad].long()
    live = rt >= 0
    assert int(live.sum()) == T * k
    # token_row is the inverse of row_token and every routed row sits inside its expert's segment
    tr = r.token_row.view(T, k).long()
    assert torch.equal(rt[tr.flatten()], torch.arange(T, device="cuda").repeat_interleave(k))
    seg_of_row = torch.bucketize(tr, r.pad_offsets.long(), right=True) - 1
    assert torch.equal(seg_of_row, ids.long())
    # stable: inside a segment rows are ordered by (route, token)
    key = torch.full((n_pad,), -1, dtype=torch.int64, device="cuda")
    j = torch.arange(k, device="cuda").view(1, k).expand(T, k)
    t = torch.arange(T, device="cuda").view(T, 1).expand(T, k)
    key[tr.flatten()] = (j * T + t).flatten()
    for e in torch.randperm(E)[:16].tolist():
        a, c = int(r.pad_offsets[e]), int(counts[e])
        seg = key[a: a + c]
        assert (seg[1:] > seg[:-1]).all()
        assert (key[a + c: int(r.pad_offsets[e + 1])] == -1).all()


@pytest.mark.parametrize("T,d,H,E,empty", [(65536, 1024, 4096, 64, 4), (131072, 2048, 8192, 64, 0)])
def test_full_size_layer_properties(ops, T, d, H, E, empty):
    from hexa_moe_b200 import _lib as L
    k = 2
    torch.manual_seed(0)
    ids, p = zipf_ids(T, k, E, empty, seed=7)
    r = ops.route(ids, E)
    check_routing(r, ids, E)
    if empty:
        assert int((r.counts == 0).sum()) == empty and float(r.counts.max()) / (T * k) > 0.15      # ragged for real
    x = torch.randn(T, d, device="cuda").bfloat16()
    w1 = (torch.randn(E, H, d, device="cuda") / d ** 0.5).bfloat16()
    b1 = torch.randn(E, H, device="cuda") * 0.1
    xs = ops.gather_rows(x, r)
    n_pad = int(r.pad_offsets[-1])
    y1 = torch.empty(r.row_capacity, H, device="cuda", dtype=torch.bfloat16)
    h = ops.esmm(xs, w1, L.B_NK, r, b1, L.EPI_ACT, L.ACT_GELU, aux=y1)
    # (1) sampled rows against float64 on the CPU
    rows = torch.randint(0, n_pad, (96,), device="cuda")
    rows = rows[r.row_token[rows] >= 0]
    e_of = (torch.bucketize(rows, r.pad_offsets.long(), right=True) - 1)
    for row, e in zip(rows.tolist()[:48], e_of.tolist()[:48]):
        want = xs[row].double().cpu() @ w1[e].double().cpu().T + b1[e].double().cpu()
        got = y1[row].double().cpu()
        assert float((got - want).abs().max() / want.abs().max()) < 2e-2
        gh = h[row].double().cpu()
        assert float((gh - F.gelu(want)).abs().max() / F.gelu(want).abs().max()) < 2e-2
    # (2) pad rows are zeros, so column sums over all rows equal column sums over routed rows
    pad = r.row_token[:n_pad] < 0
    assert (h[:n_pad][pad] == 0).all() and (y1[:n_pad][pad] == 0).all()
    # (3) ESS: the per-expert sums add up to the plain column sum (fp32 accumulation both ways)
    dy = torch.randn(T, d, device="cuda").bfloat16()
    dys = ops.gather_rows(dy, r)
    db = ops.ess(dys, r)
    total = dys[:n_pad].float().sum(0)
    assert float((db.sum(0) - total).abs().max() / total.abs().max()) < 1e-4
    assert (db[r.counts == 0] == 0).all()
    # (4) ESTMM: linear in q, and its sum over experts is the dense X^T dY of the sorted buffers
    dw = ops.estmm(h, dys, r, out_dtype=torch.float32)                     # [E, H, d]
    dense = h[:n_pad, :512].float().T @ dys[:n_pad].float()                # a 512-row slab is enough
    got = dw[:, :512].sum(0)
    assert float((got - dense).abs().max() / dense.abs().max()) < 2e-3
    dw2 = ops.estmm(h, (dys.float() * 2).bfloat16(), r, out_dtype=torch.float32)
    assert torch.equal(dw2, dw * 2)                                        # exact: scaling by 2 commutes with rounding
    assert (dw[r.counts == 0] == 0).all()
    # (5) tensor-core ESMM equals the fp32 CUDA-core ESMM on whole experts (the smallest non-empty ones, to stay quick)
    order = torch.argsort(torch.where(r.counts > 0, r.counts, torch.full_like(r.counts, 1 << 30)))
    for e in order[:2].tolist():
        a, b_ = int(r.pad_offsets[e]), int(r.pad_offsets[e + 1])
        ref = xs[a:b_].float() @ w1[e].float().T + b1[e]
        live = (r.row_token[a:b_] >= 0).unsqueeze(1)
        assert float(((y1[a:b_].float() - ref) * live).abs().max() / ref.abs().max()) < 2e-2
    # (6) combine of the gathered rows returns k * x
    back = ops.combine_rows(xs, r)
    assert torch.equal(back, (x.float() * k).bfloat16())


def test_degenerate_shapes(ops):
    """No tokens at all, one expert, every token to the same expert, more experts than tokens."""
    from hexa_moe_b200 import _lib as L
    dev = "cuda"
    # T = 0
    r = ops.route(torch.empty(0, 2, dtype=torch.int32, device=dev), 4)
    assert int(r.pad_offsets[-1]) == 0 and (r.counts == 0).all() and (r.pair_block == -1).all()
    xs = ops.gather_rows(torch.empty(0, 64, device=dev, dtype=torch.bfloat16), r)
    w = torch.randn(4, 128, 64, device=dev).bfloat16()
    out = ops.esmm(xs, w, L.B_NK, r)
    dw = ops.estmm(out, xs, r, out_dtype=torch.float32)
    assert dw.shape == (4, 128, 64) and (dw == 0).all()
    assert (ops.ess(out, r) == 0).all()
    assert ops.combine_rows(out, r).shape == (0, 128)
    # one expert / everything to expert 2 of 5 / E > T
    for T, E, ids in ((300, 1, torch.zeros(300, 1, dtype=torch.int32)), (513, 5, torch.full((513, 1), 2, dtype=torch.int32)),
                      (7, 40, torch.arange(7, dtype=torch.int32).view(7, 1) * 5)):
        ids = ids.to(dev)
        r = ops.route(ids, E)
        x = torch.randn(T, 64, device=dev).bfloat16()
        w = (torch.randn(E, 256, 64, device=dev) / 8).bfloat16()
        xs = ops.gather_rows(x, r)
        y = ops.combine_rows(ops.esmm(xs, w, L.B_NK, r), r)
        want = torch.einsum("td,tnd->tn", x.float(), w[ids[:, 0].long()].float())
        assert float((y.float() - want).abs().max() / want.abs().max()) < 2e-2
