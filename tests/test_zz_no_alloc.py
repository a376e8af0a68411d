"""hexa_ess_static: the ESS entry point that brings its own scratch memory.

Some callers cannot allocate device memory at the point where they need the bias gradient - code that
runs where the framework's caching allocator must not be touched, or a C host that only holds the
pointers it was given.  For them the library keeps ESS's partial-sum scratch in a fixed 32 MiB device
array.  This file checks, through the C ABI, that the variant returns exactly what hexa_ess returns,
twice in a row on different data (the array keeps the previous call's contents), that it allocates
nothing through torch, and that a request beyond the built-in capacity is refused with a clear error.
Collected last on purpose: a failure here cannot hide any other test behind `-x`."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_ess_static_matches_ess_twice_and_rejects_oversize():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from hexa_moe_b200 import _lib as L, ops
    lib = L.lib()
    cap_bytes = lib.hexa_ess_static_capacity_bytes()
    assert cap_bytes == 32 << 20
    stream = torch.cuda.current_stream().cuda_stream
    for call, (T, k, E, cols, dtype, seed) in enumerate([(5000, 2, 16, 520, torch.bfloat16, 1), (3000, 1, 7, 200, torch.float32, 2)]):
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32).cuda()
        r = ops.route(ids, E)
        src = ops.gather_rows(torch.randn(T, cols, generator=g).to(dtype).cuda(), r)
        want = ops.ess(src, r)                                   # existing entry point, caller-provided workspace
        got = torch.full((E, cols), float("nan"), device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = lib.hexa_ess_static(src.data_ptr(), src.stride(0), r.pad_offsets.data_ptr(), E, r.row_capacity, cols,
                                 got.data_ptr(), got.stride(0), L.dt(src), stream)
        assert rc == 0, lib.hexa_last_error_string().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before           # nothing was allocated on our behalf
        assert torch.equal(got, want), f"call {call}: max diff {(got - want).abs().max().item()}"   # same kernels, same order: bit-equal
    # beyond the built-in capacity: refused, nothing launched
    big_rows, big_cols = 128 * 4096, 4096                        # 4096 tiles * 4096 cols * 4 B = 64 MiB
    assert lib.hexa_ess_workspace_bytes(big_rows, big_cols) > cap_bytes
    rc = lib.hexa_ess_static(src.data_ptr(), big_cols, r.pad_offsets.data_ptr(), E, big_rows, big_cols, got.data_ptr(), big_cols,
                             L.dt(src), stream)
    assert rc == -4
    msg = lib.hexa_last_error_string().decode()
    assert "built-in buffer" in msg and "hexa_ess" in msg
