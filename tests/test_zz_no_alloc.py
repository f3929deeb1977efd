"""The allocation-free entry point, called through its exported C symbol.

``hs_attention_decode_noalloc`` is for hosts that must not allocate device memory while
they run (a loop with memory fixed at start-up, a process whose GPU memory is promised to
another allocator): it is the split-context decode attention with its scratch memory in a
static device array instead of buffers the caller allocates.  This test calls the symbol
with ``ctypes`` exactly as such a host would — raw pointers, no wrapper of the package — and
checks its output against the existing entry point's (scratch allocated by PyTorch) and
against the plain implementation in float64, twice in a row, since the second call finds the
array as the first one left it.

It is collected last (the file name sorts after every other test file), so a run that stops
at the first failure has already run everything else.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(H=16, D=64, PS=16, lens=(700, 333, 1024, 17, 64), seed=5):
    """Single-query tokens of several requests over shuffled pages (bfloat16)."""
    from hetero_serve_b200.kernels import AttentionGeometry
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    max_pages = max(-(-n // PS) for n in lens) + 1
    n_pages = sum(-(-n // PS) for n in lens) + 2
    perm = iter(torch.randperm(n_pages, generator=g).tolist())
    table = torch.full((R, max_pages), -1, dtype=torch.int32)
    pool = torch.full((n_pages, 2, H, PS, D), float("nan")).bfloat16()
    for r, n in enumerate(lens):
        for i in range(-(-n // PS)):
            table[r, i] = next(perm)
        vals = torch.randn(n, 2, H, D, generator=g).bfloat16()
        for p in range(n):
            pool[table[r, p // PS], :, :, p % PS, :] = vals[p]
    W = 3 * H * D
    geom = AttentionGeometry(H, H, D, PS, n_pages, max_pages, 0, H * D, 2 * H * D, W)
    qkv = torch.randn(R, W, generator=g).bfloat16()
    tok_pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    tok_req = torch.arange(R, dtype=torch.int32)
    host_batch = [(f"r{r}", r, n - 1, 1) for r, n in enumerate(lens)]
    return geom, qkv.to(DEV), pool.to(DEV), table.to(DEV), tok_pos.to(DEV), tok_req.to(DEV), host_batch


def _call_noalloc(lib, out, qkv, pool, table, tok_pos, tok_req, plan, g, scale, splits, status):
    fn = lib.hs_attention_decode_noalloc
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, P, P]
    fn.restype = I
    data = plan.data
    dec_info = data[4:]
    return fn(out.data_ptr(), qkv.data_ptr(), pool.data_ptr(), table.data_ptr(),
              tok_pos.data_ptr(), tok_req.data_ptr(), dec_info.data_ptr(), data.data_ptr(),
              plan.decode_cap, g.n_heads, g.n_kv_heads, g.head_dim, g.page_size, g.num_pages,
              g.max_pages, g.q_off, g.qkv_stride, g.window, scale, splits, status.data_ptr(),
              torch.cuda.current_stream().cuda_stream)


def test_no_alloc_entry_point_matches_the_allocating_one_twice_in_a_row():
    from hetero_serve_b200.kernels import CudaOps
    ops = CudaOps()
    lib = ops.lib
    geom, qkv, pool, table, tok_pos, tok_req, host_batch = _case()
    R = qkv.shape[0]
    plan = ops.make_plan(host_batch, R, geom.page_size)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 0.125
    # the existing entry point: the same kernel (hs_attention_decode_append) with its scratch
    # allocated by PyTorch; decode_mma off, or the wrapper would pick the tensor-core kernel
    ops.decode_mma = False
    want = torch.empty(R, geom.n_heads * geom.head_dim, device=DEV, dtype=torch.bfloat16)
    ops.attention(want, qkv, pool, table, tok_pos, tok_req, geom, scale, status, plan)
    # and the plain implementation in float64, so that a fault both entry points share shows
    import plain_ops
    plain = torch.empty(R, geom.n_heads * geom.head_dim, dtype=torch.float64)
    plain_ops.PlainOps().attention(plain, qkv.cpu(), pool.cpu(), table.cpu(), tok_pos.cpu(),
                                   tok_req.cpu(), geom, scale, None)
    assert (want.double().cpu() - plain).abs().max() < 2e-2
    splits = ops.decode_splits(plan.decode_cap, geom.n_heads, geom.max_pages * geom.page_size)
    assert splits > 1                                    # the scratch memory really is used
    lib.hs_attention_decode_noalloc_capacity.restype = ctypes.c_longlong
    cap = lib.hs_attention_decode_noalloc_capacity()
    assert R * geom.n_heads * (splits * (geom.head_dim + 2) + 1) <= cap
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for call in range(2):
        got = torch.full_like(want, float("nan"))
        code = _call_noalloc(lib, got, qkv, pool, table, tok_pos, tok_req, plan, geom, scale,
                             splits, status)
        assert code == 0, code
        torch.cuda.synchronize()
        assert status.item() == 0
        assert torch.isfinite(got).all()
        # the tolerance the attention tests use for bfloat16 outputs
        assert (got.float() - want.float()).abs().max() < 2e-2, call
        assert (got.double().cpu() - plain).abs().max() < 2e-2, call
    assert torch.cuda.mem_get_info()[0] == free_before   # nothing was allocated on the device


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    from hetero_serve_b200.kernels import CudaOps
    ops = CudaOps()
    geom, qkv, pool, table, tok_pos, tok_req, host_batch = _case(lens=(40, 50))
    plan = ops.make_plan(host_batch, 2, geom.page_size)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((2, geom.n_heads * geom.head_dim), 7.0, device=DEV, dtype=torch.bfloat16)
    fn = ops.lib.hs_attention_decode_noalloc
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, I, F, I, P, P]
    fn.restype = I
    # a token capacity far beyond the static array: refused with HS_ERR_TOO_LARGE, nothing runs
    code = fn(out.data_ptr(), qkv.data_ptr(), pool.data_ptr(), table.data_ptr(),
              tok_pos.data_ptr(), tok_req.data_ptr(), plan.data[4:].data_ptr(),
              plan.data.data_ptr(), 1 << 20, geom.n_heads, geom.n_kv_heads, geom.head_dim,
              geom.page_size, geom.num_pages, geom.max_pages, geom.q_off, geom.qkv_stride, 0,
              0.125, 8, status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert code == -3
    torch.cuda.synchronize()
    assert (out == 7.0).all()
