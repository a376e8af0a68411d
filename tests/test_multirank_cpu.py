"""World-size-2 `gloo` runs of the two multi-device modes on CPU.

The expert math is supplied by the CPU oracle (tests/oracle_backend.py) so that what is tested is
the host logic around it: hidden-dimension sharding with uneven `mlp_proportion`, the
pipeline-shared cache's all-gather + unpack, reduce-scatter/average of the expert gradients,
the model-centric token all-gather and output / input-gradient reduce-scatter."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _full_params(E, d, H, n_layers, seed=0):
    g = torch.Generator().manual_seed(seed)
    P = []
    for _ in range(n_layers):
        P.append(dict(w1=torch.randn(E, H, d, generator=g) * 0.2, w2=torch.randn(E, H, d, generator=g) * 0.2,
                      b1=torch.randn(E, H, generator=g) * 0.1, b2=torch.randn(E, d, generator=g) * 0.1,
                      wg=torch.randn(E, d, generator=g) * 0.5))
    return P


def _worker(rank, world, port, data_centric, proportion, tokens_per_rank, q, defer_grads="1", env=None):
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), HEXA_DEFER_GRADS=defer_grads)
    os.environ.update(env or {})
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle_backend
        from hexa_moe import moe as hmoe
        from oracle import hexa_oracle as O
        E, d, H, k, L = 4, 16, 64, 2, 2
        m = hmoe.MoE_Cascaded(gate_type={'type': 'top', 'k': k, 'fp32_gate': True}, model_dim_list=[d] * L, moe_idx_list=[0, 1],
                              mlp_ratio=H // d, mlp_proportion=proportion, num_global_experts=E, total_depth=L,
                              data_centric=data_centric, activation_fn=lambda t: F.gelu(t))
        m.dispatch_params.backend = oracle_backend          # test double: CPU oracle instead of the CUDA kernels
        m.eval()
        P = _full_params(E, d, H, L)
        split = [m.local_dim_list_all[r][0] for r in range(world)]
        lo = sum(split[:rank]); n = split[rank]
        with torch.no_grad():
            for i in range(L):
                m.batched_fc1_w[i].zero_(); m.batched_fc2_w[i].zero_(); m.batched_fc1_bias[i].zero_()
                m.batched_fc1_w[i][:, :n] = P[i]["w1"][:, lo: lo + n]
                m.batched_fc2_w[i][:, :n] = P[i]["w2"][:, lo: lo + n]
                m.batched_fc1_bias[i][:, :n] = P[i]["b1"][:, lo: lo + n]
                m.batched_fc2_bias[i].copy_(P[i]["b2"]); m.gates[i].wg.weight.copy_(P[i]["wg"])
        xs = [torch.randn(tokens_per_rank[r], d, generator=torch.Generator().manual_seed(100 + r)) for r in range(world)]
        x = xs[rank].clone().requires_grad_(True)
        h, aux = x, 0
        for i in range(L):
            h, l = m(i, h)
            aux = aux + l
        if defer_grads == "0":
            # the reduced expert gradients come back through autograd itself: torch.autograd.grad sees them
            prms = [m.batched_fc1_w[0], m.batched_fc2_w[0], m.batched_fc1_bias[0], m.batched_fc2_bias[0],
                    m.batched_fc1_w[1], m.batched_fc2_w[1], m.batched_fc1_bias[1], m.batched_fc2_bias[1]]
            grads = torch.autograd.grad(h.sum(), [x] + prms)
            x.grad = grads[0]
            for p_, g_ in zip(prms, grads[1:]):
                assert g_ is not None and g_.shape == p_.shape
                p_.grad = g_
        else:
            h.sum().backward()

        # expectation from the oracle, layer by layer on every rank's tokens
        def run_rank(r):
            cur = xs[r].double().requires_grad_(False)
            saved = []
            for i in range(L):
                ids, _, _ = O.gate_topk(cur.float(), P[i]["wg"], k)
                res = O.moe_layer(cur, ids, P[i]["w1"], P[i]["w2"], P[i]["b1"], P[i]["b2"], F.gelu)
                saved.append((cur, ids)); cur = res["y"]
            y = cur
            g = torch.ones_like(y); grads = [None] * L
            for i in reversed(range(L)):
                cin, ids = saved[i]
                res = O.moe_layer(cin, ids, P[i]["w1"], P[i]["w2"], P[i]["b1"], P[i]["b2"], F.gelu, g)
                grads[i] = res; g = res["dx"]
            return y, g, grads
        outs = [run_rank(r) for r in range(world)]
        y_exp, dx_exp, _ = outs[rank]
        torch.testing.assert_close(h.detach().double(), y_exp, rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(x.grad.double(), dx_exp, rtol=1e-4, atol=1e-4)
        for i in range(L):
            if data_centric:   # data parallel over tokens: gradients are averaged over ranks
                comb = lambda key: sum(outs[r][2][i][key] for r in range(world)) / world
            else:              # every rank saw all tokens for its hidden slice: plain sum
                comb = lambda key: sum(outs[r][2][i][key] for r in range(world))
            torch.testing.assert_close(m.batched_fc1_w[i].grad[:, :n].double(), comb("dw1")[:, lo: lo + n], rtol=1e-4, atol=1e-4)
            torch.testing.assert_close(m.batched_fc2_w[i].grad[:, :n].double(), comb("dw2")[:, lo: lo + n], rtol=1e-4, atol=1e-4)
            torch.testing.assert_close(m.batched_fc1_bias[i].grad[:, :n].double(), comb("db1")[:, lo: lo + n], rtol=1e-4, atol=1e-4)
            torch.testing.assert_close(m.batched_fc2_bias[i].grad.double(), comb("db2"), rtol=1e-4, atol=1e-4)
            if n < m.batched_fc1_w[i].shape[1]:
                assert (m.batched_fc1_w[i].grad[:, n:] == 0).all()      # storage padding gets no gradient
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        import traceback
        q.put((rank, "FAIL: " + traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def _run(data_centric, proportion, tokens_per_rank, defer_grads="1", env=None):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, data_centric, proportion, tokens_per_rank, q, defer_grads, env))
             for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = [q.get(timeout=240) for _ in range(world)]
    finally:
        for p in procs:
            p.join(60)
            if p.is_alive():          # a rank that is stuck must not outlive the test
                p.kill()
    for rank, msg in res:
        assert msg == "ok", f"rank {rank}: {msg}"


@pytest.mark.parametrize("proportion", [None, [0.7, 0.3]])
def test_data_centric_two_ranks(proportion):
    _run(True, proportion, [40, 40])


@pytest.mark.parametrize("proportion,tokens", [(None, [32, 32]), ([0.3, 0.7], [24, 40])])
def test_model_centric_two_ranks(proportion, tokens):
    _run(False, proportion, tokens)


@pytest.mark.parametrize("proportion,tokens,chunks", [(None, [32, 32], 2), ([0.3, 0.7], [24, 40], 3), (None, [5, 2], 4)])
def test_model_centric_token_chunks(proportion, tokens, chunks):
    """The tokens of every rank cut into chunks whose transfers overlap the other chunks' GEMMs: same results; ragged
    chunks when the token counts differ or do not divide, fewer chunks than asked when a rank has too few tokens."""
    _run(False, proportion, tokens, env={"HEXA_MC_CHUNKS": str(chunks), "HEXA_MC_MIN_CHUNK_TOKENS": "1"})


@pytest.mark.parametrize("proportion", [None, [0.7, 0.3]])
def test_data_centric_gradients_through_autograd_when_not_deferred(proportion):
    """HEXA_DEFER_GRADS=0: backward returns the reduced slices like the reference does (impls/layers.py:431-474)
    instead of adding them to .grad from an end-of-backward callback."""
    _run(True, proportion, [40, 40], defer_grads="0")


def _ckpt_worker(rank, world, port, proportion, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from hexa_moe import moe as hmoe
        E, d, H, L = 4, 16, 64, 2
        mk = lambda: hmoe.MoE_Cascaded(gate_type={'type': 'top', 'k': 1}, model_dim_list=[d] * L, moe_idx_list=[0, 1],
                                       mlp_ratio=H // d, mlp_proportion=proportion, num_global_experts=E, total_depth=L,
                                       data_centric=True, activation_fn=lambda t: F.gelu(t))
        m = mk()
        P = _full_params(E, d, H, L, seed=3)
        src = hmoe.MoE_Buffer([d] * L, E, L, H // d, None, True, True)
        if rank == 0:                         # only the source rank holds the unsharded checkpoint
            with torch.no_grad():
                for i in range(L):
                    src.batched_fc1_w[i].copy_(P[i]["w1"]); src.batched_fc2_w[i].copy_(P[i]["w2"])
                    src.batched_fc1_bias[i].copy_(P[i]["b1"]); src.batched_fc2_bias[i].copy_(P[i]["b2"])
        m.load_ckpt(src, src_rank=0)
        split = [m.local_dim_list_all[r][0] for r in range(world)]
        lo, n = sum(split[:rank]), split[rank]
        for i in range(L):                    # every rank got exactly its slice of the hidden dimension
            assert torch.equal(m.batched_fc1_w[i].data[:, :n], P[i]["w1"][:, lo: lo + n])
            assert torch.equal(m.batched_fc2_w[i].data[:, :n], P[i]["w2"][:, lo: lo + n])
            assert torch.equal(m.batched_fc1_bias[i].data[:, :n], P[i]["b1"][:, lo: lo + n])
            assert torch.equal(m.batched_fc2_bias[i].data, P[i]["b2"])
        dst = hmoe.MoE_Buffer([d] * L, E, L, H // d, None, True, True)
        m.save_ckpt(dst, dst_rank=1)          # gathered back, unevenly sized slices in rank order
        if rank == 1:
            for i in range(L):
                assert torch.equal(dst.batched_fc1_w[i].data, P[i]["w1"])
                assert torch.equal(dst.batched_fc2_w[i].data, P[i]["w2"])
                assert torch.equal(dst.batched_fc1_bias[i].data, P[i]["b1"])
                assert torch.equal(dst.batched_fc2_bias[i].data, P[i]["b2"])
        q.put((rank, "ok"))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, "FAIL: " + traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("proportion", [None, [0.7, 0.3]])
def test_checkpoint_scatter_and_gather_two_ranks(proportion):
    """load_ckpt broadcasts an unsharded MoE_Buffer from one rank and keeps each rank's hidden slice; save_ckpt gathers
    the (uneven) slices back into an unsharded buffer on another rank (reference cascaded_moe.py:413-525)."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ckpt_worker, args=(r, world, port, proportion, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(60)
    for rank, msg in res:
        assert msg == "ok", f"rank {rank}: {msg}"


def _dense_worker(rank, world, port, defer, q):
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), HEXA_DEFER_GRADS=defer, HEXA_DENSE_BUCKET_MB="0.001")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle_backend
        from hexa_moe import moe as hmoe
        d, H = 16, 64
        torch.manual_seed(5)                 # same parameters on both ranks
        m = hmoe.MoE_Cascaded(gate_type={'type': 'top', 'k': 1}, model_dim_list=[d] * 3, moe_idx_list=[2], mlp_ratio=H // d,
                              num_global_experts=2, total_depth=3, data_centric=True, activation_fn=lambda t: F.gelu(t))
        m.dispatch_params.backend = oracle_backend
        with torch.no_grad():
            for n_, p in m.named_parameters():
                if n_.startswith("mlp_"):
                    p.normal_(0, 0.3)
        x = torch.randn(24, d, generator=torch.Generator().manual_seed(50 + rank))
        if defer == "1":
            # a backward pass that raises after the dense layers queued their gradients must not leak into the next step
            class _Boom(torch.autograd.Function):
                @staticmethod
                def forward(ctx, t):
                    return t.clone()

                @staticmethod
                def backward(ctx, g):
                    raise RuntimeError("boom")
            h = _Boom.apply(x.clone().requires_grad_(True))
            for depth in range(2):
                h, _ = m(depth, h)
            with pytest.raises(RuntimeError, match="boom"):
                h.pow(2).sum().backward()
            for p in m.parameters():
                p.grad = None
        h = x
        for depth in range(2):               # the two dense depths
            h, aux = m(depth, h)
            assert aux == 0
        h.pow(2).sum().backward()
        # expectation: plain autograd of the same FFNs, averaged over the ranks
        names = ["mlp_fc1_w", "mlp_fc2_w", "mlp_fc1_b", "mlp_fc2_b"]
        ref = [[getattr(m, n_)[i].detach().clone().requires_grad_(True) for n_ in names] for i in range(2)]
        t = x
        for w1, w2, b1, b2 in ref:
            t = F.gelu(t @ w1.t() + b1) @ w2 + b2
        t.pow(2).sum().backward()
        for i in range(2):
            for n_, r_ in zip(names, ref[i]):
                want = r_.grad.clone()
                dist.all_reduce(want)
                want /= world
                got = getattr(m, n_)[i].grad
                assert got is not None and got.shape == want.shape, (n_, i)
                torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-6)
        q.put((rank, "ok"))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, "FAIL: " + traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("defer", ["1", "0"])
def test_dense_ffn_gradients_are_averaged_over_ranks(defer):
    """Dense depths (reference impls/layers.py:18-88): parameter gradients are the mean over the data-parallel ranks,
    whether they travel in buckets on a side path and land in .grad at the end of backward (default; the tiny bucket
    size here forces several buckets) or are all-reduced inline and returned through autograd (HEXA_DEFER_GRADS=0)."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_dense_worker, args=(r, world, port, defer, q)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = [q.get(timeout=240) for _ in range(world)]
    finally:
        for p in procs:
            p.join(60)
            if p.is_alive():
                p.kill()
    for rank, msg in res:
        assert msg == "ok", f"rank {rank}: {msg}"


def test_model_centric_without_a_process_group():
    """A single process that never initialised torch.distributed runs the model-centric branch as well: the collectives
    pass their input through and nothing asks the (absent) process group for its backend."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_backend
    from hexa_moe import moe as hmoe
    assert not dist.is_initialized()
    E, d, H, k, L, T = 4, 16, 64, 2, 2, 24
    outs = []
    for data_centric in (True, False):
        torch.manual_seed(0)
        m = hmoe.MoE_Cascaded(gate_type={'type': 'top', 'k': k, 'fp32_gate': True}, model_dim_list=[d] * L, moe_idx_list=[0, 1],
                              mlp_ratio=H // d, mlp_proportion=None, num_global_experts=E, total_depth=L,
                              data_centric=data_centric, activation_fn=lambda t: F.gelu(t))
        m.dispatch_params.backend = oracle_backend
        m.eval()
        x = torch.randn(T, d, generator=torch.Generator().manual_seed(5)).requires_grad_(True)
        h = x
        for i in range(L):
            h, _ = m(i, h)
        h.sum().backward()
        outs.append((h.detach(), x.grad, m.batched_fc1_w[0].grad, m.batched_fc2_bias[1].grad))
    for a, b in zip(*outs):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
