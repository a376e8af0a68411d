"""Two-GPU NCCL runs of the data-centric and model-centric modes with the real kernels, checked
against the CPU oracle.  Skipped on boxes with fewer than two GPUs (the same host logic is covered
on CPU `gloo` ranks in test_multirank_cpu.py)."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, data_centric, proportion, dtype_name, q, env=None):
    import torch.distributed as dist
    import torch.nn.functional as F
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    os.environ.update(env or {})
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from hexa_moe import moe as hmoe
        from oracle import hexa_oracle as O
        dtype = getattr(torch, dtype_name)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        E, d, H, k, L, T = 6, 64, 256, 2, 2, 384
        m = hmoe.MoE_Cascaded(gate_type={'type': 'top', 'k': k, 'fp32_gate': True}, model_dim_list=[d] * L, moe_idx_list=[0, 1],
                              mlp_ratio=H // d, mlp_proportion=proportion, num_global_experts=E, total_depth=L,
                              data_centric=data_centric, activation_fn=lambda t: F.gelu(t))
        g = torch.Generator().manual_seed(0)
        P = [dict(w1=torch.randn(E, H, d, generator=g) * 0.15, w2=torch.randn(E, H, d, generator=g) * 0.1,
                  b1=torch.randn(E, H, generator=g) * 0.1, b2=torch.randn(E, d, generator=g) * 0.1,
                  wg=torch.randn(E, d, generator=g) * 0.5) for _ in range(L)]
        split = [m.local_dim_list_all[r][0] for r in range(world)]
        lo = sum(split[:rank]); n = split[rank]
        with torch.no_grad():
            for i in range(L):
                for prm in (m.batched_fc1_w[i], m.batched_fc2_w[i], m.batched_fc1_bias[i]):
                    prm.zero_()
                m.batched_fc1_w[i][:, :n] = P[i]["w1"][:, lo: lo + n]
                m.batched_fc2_w[i][:, :n] = P[i]["w2"][:, lo: lo + n]
                m.batched_fc1_bias[i][:, :n] = P[i]["b1"][:, lo: lo + n]
                m.batched_fc2_bias[i].copy_(P[i]["b2"]); m.gates[i].wg.weight.copy_(P[i]["wg"])
        m = m.to(dtype).cuda().eval()
        Pd = [{k_: v.to(dtype).float() for k_, v in p.items()} for p in P]      # what the module really holds
        xs = [torch.randn(T, d, generator=torch.Generator().manual_seed(100 + r)).to(dtype) for r in range(world)]
        x = xs[rank].cuda().requires_grad_(True)
        ids_used = []
        h = x
        for i in range(L):
            h, _ = m(i, h)
            ids_used.append(torch.stack([t.cpu() for t in m.dispatch_params.indices_], dim=1))
        h.float().sum().backward()
        torch.cuda.synchronize()
        # every rank needs every rank's routing decisions to build the expectation
        all_ids = [[None] * world for _ in range(L)]
        for i in range(L):
            dist.all_gather_object(all_ids[i], ids_used[i])

        def run_rank(r):
            cur = xs[r].double()
            saved = []
            for i in range(L):
                ids = all_ids[i][r]          # the module routes its local tokens in both modes
                res = O.moe_layer(cur, ids, Pd[i]["w1"], Pd[i]["w2"], Pd[i]["b1"], Pd[i]["b2"], F.gelu)
                saved.append((cur, ids)); cur = res["y"].to(dtype).double()
            gy = torch.ones_like(cur); grads = [None] * L
            for i in reversed(range(L)):
                cin, ids = saved[i]
                res = O.moe_layer(cin, ids, Pd[i]["w1"], Pd[i]["w2"], Pd[i]["b1"], Pd[i]["b2"], F.gelu, gy)
                grads[i] = res; gy = res["dx"].to(dtype).double()
            return cur, gy, grads
        outs = [run_rank(r) for r in range(world)]

        def err(a, b):
            a, b = a.detach().double().cpu(), b.double()
            return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))
        assert err(h, outs[rank][0]) < tol, ("y", err(h, outs[rank][0]))
        assert err(x.grad, outs[rank][1]) < tol, ("dx", err(x.grad, outs[rank][1]))
        for i in range(L):
            comb = (lambda key: sum(outs[r][2][i][key] for r in range(world)) / world) if data_centric else \
                   (lambda key: sum(outs[r][2][i][key] for r in range(world)))
            for name, prm, key, sl in (("dw1", m.batched_fc1_w[i], "dw1", True), ("dw2", m.batched_fc2_w[i], "dw2", True),
                                       ("db1", m.batched_fc1_bias[i], "db1", True), ("db2", m.batched_fc2_bias[i], "db2", False)):
                want = comb(key)[:, lo: lo + n] if sl else comb(key)
                got = prm.grad[:, :n] if sl else prm.grad
                assert err(got, want) < tol * 1.5, (i, name, err(got, want))
        if m.dispatch_params.cache is not None:
            dist.barrier(); m.dispatch_params.cache.close(); dist.barrier()
        q.put((rank, "ok"))
    except Exception:  # noqa: BLE001
        import traceback
        q.put((rank, "FAIL: " + traceback.format_exc()))
    finally:
        dist.destroy_process_group()


def _run(data_centric, proportion, dtype_name, env=None):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, data_centric, proportion, dtype_name, q, env)) for r in range(2)]
    for p in procs:
        p.start()
    try:
        res = [q.get(timeout=300) for _ in range(2)]
    finally:
        for p in procs:
            p.join(60)
            if p.is_alive():          # a rank that is stuck must not keep its GPU behind the test
                p.kill()
    for rank, msg in res:
        assert msg == "ok", f"rank {rank}: {msg}"


@pytest.mark.parametrize("proportion,dtype_name", [(None, "float32"), ([0.625, 0.375], "bfloat16"), (None, "bfloat16")])
def test_data_centric_two_gpus(proportion, dtype_name):
    _run(True, proportion, dtype_name)


@pytest.mark.parametrize("proportion,dtype_name", [(None, "float32"), ([0.375, 0.625], "bfloat16")])
def test_model_centric_two_gpus(proportion, dtype_name):
    _run(False, proportion, dtype_name)


@pytest.mark.parametrize("chunks", ["0", "3"])
def test_model_centric_two_gpus_token_chunks(chunks):
    """Tokens cut into three chunks per rank (collectives of one chunk beside the GEMMs of another, weight gradients
    accumulated over the chunks), and the in-line order with one chunk: same results."""
    _run(False, [0.375, 0.625], "bfloat16", env={"HEXA_MC_CHUNKS": chunks, "HEXA_MC_MIN_CHUNK_TOKENS": "64"})


def test_data_centric_two_gpus_gradients_returned_through_autograd():
    """HEXA_DEFER_GRADS=0 on real devices: backward waits for the side-stream reduction and returns the slices."""
    _run(True, None, "bfloat16", env={"HEXA_DEFER_GRADS": "0"})


def test_weight_gradient_stores_into_another_gpus_memory_are_refused():
    """hexa_estmm_scatter takes destinations in the calling GPU's memory only; a pointer into a peer's memory is
    refused before anything is launched (stores of that kernel into peer memory are not supported)."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    sys.path.insert(0, ROOT)
    from hexa_moe_b200 import _lib as L, ops
    torch.cuda.set_device(0)
    T, k, E, M, N = 600, 1, 2, 256, 128
    ids = torch.randint(0, E, (T, k), dtype=torch.int32, device="cuda:0")
    r = ops.route(ids, E)
    p = ops.gather_rows(torch.randn(T, M, device="cuda:0").bfloat16(), r)
    q = ops.gather_rows(torch.randn(T, N, device="cuda:0").bfloat16(), r)
    local = torch.zeros(E, M // 2, N, dtype=torch.bfloat16, device="cuda:0")
    remote = torch.zeros(E, M // 2, N, dtype=torch.bfloat16, device="cuda:1")
    with pytest.raises(L.HexaError, match="another GPU"):
        ops.estmm(p, q, r, ranks=2, out=[local, remote])
    torch.cuda.synchronize()
    assert (local == 0).all() and (remote == 0).all()          # refused before any launch
