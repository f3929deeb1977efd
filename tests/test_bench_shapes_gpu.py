"""The kernels at the shapes the benchmark times, against float64 references.

The small kernel tests never make a persistent CTA take a second work item: the tcgen05
prefill attention walks 128-query tiles x heads with one CTA per SM (2 x 1,024 queries of 16
heads are 256 items for 148 CTAs), the tcgen05 linear's tiles outnumber its CTAs from 2,048
rows on (TMEM accumulator ping-pong and a shared-memory ring that wraps across items), and
the decode attention chooses its shape by batch x heads against the SM count.  Here those
paths run under a comparison.  The references are vectorised float64 PyTorch on the device
(per request: gather the pages through the table, scores, causal mask, softmax, values)."""

import pytest
import torch

from test_kernels_gpu import _attention_case, _host_batch, _status

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from hetero_serve_b200.kernels import CudaOps
    return CudaOps()


def _attention_reference(qkv, pool, table, lens, new, geom, scale):
    """float64 causal attention over the pages, request by request: [T, H*D]."""
    H, HK, D, PS = geom.n_heads, geom.n_kv_heads, geom.head_dim, geom.page_size
    pv = pool.view(geom.num_pages, 2, HK, PS, D)
    scale32 = float(torch.tensor(scale, dtype=torch.float32))
    out = []
    t = 0
    for r, (n, k) in enumerate(zip(lens, new)):
        pos = torch.arange(n, device=pool.device)
        pages = table[r, pos // PS].long()
        keys = pv[pages, 0, :, pos % PS, :].double()                  # [n, HK, D]
        vals = pv[pages, 1, :, pos % PS, :].double()
        q = qkv[t:t + k, geom.q_off:geom.q_off + H * D].view(k, H, D).double()
        keys = keys.repeat_interleave(H // HK, dim=1)
        vals = vals.repeat_interleave(H // HK, dim=1)
        s = torch.einsum("qhd,nhd->hqn", q, keys) * scale32
        qpos = torch.arange(n - k, n, device=pool.device)
        s = s.masked_fill((pos[None, :] > qpos[:, None])[None], float("-inf"))
        o = torch.einsum("hqn,nhd->qhd", torch.softmax(s, -1), vals)
        out.append(o.reshape(k, H * D))
        t += k
    return torch.cat(out)


PREFILL = [
    # H, D, lens, new: the bench's prefill, and a ragged one with portions starting mid-context
    (16, 64, [1024, 1024], [1024, 1024]),
    (16, 64, [1024, 700, 130, 1000], [600, 700, 2 * 64 + 2, 333]),
    (20, 64, [900, 1024, 517], [900, 1024, 517]),        # GPT-2 large's heads
    (16, 128, [1024, 1024], [1024, 1024]),               # head size 128: the mma.sync kernel
]


@pytest.mark.parametrize("case", PREFILL, ids=[f"H{c[0]}D{c[1]}n{len(c[2])}t{sum(c[3])}" for c in PREFILL])
def test_prefill_attention_with_more_work_items_than_ctas(ops, case):
    H, D, lens, new = case
    geom, qkv, pool, table, tok_pos, tok_req = _attention_case(H, H, D, 16, lens, new, 0,
                                                               torch.bfloat16, seed=H + D)
    st = _status()
    ops.kv_append(pool, qkv, table, tok_pos, tok_req, geom, st)
    T = qkv.shape[0]
    plan = ops.make_plan(_host_batch(lens, new), T, 16)
    assert plan.tile_cap * H > ops.sm_count            # some CTA takes a second item
    out = torch.full((T, H * D), float("nan"), device=DEV, dtype=torch.bfloat16)
    scale = 0.9 / D ** 0.5
    ops.attention(out, qkv, pool, table, tok_pos, tok_req, geom, scale, st, plan)
    ref = _attention_reference(qkv, pool, table, lens, new, geom, scale)
    assert st.item() == 0
    assert torch.isfinite(out).all()
    assert (out.double() - ref).abs().max() < 2e-2
    out2 = torch.empty_like(out)                        # launched again: same bits
    ops.attention(out2, qkv, pool, table, tok_pos, tok_req, geom, scale, st, plan)
    assert torch.equal(out, out2)


@pytest.mark.parametrize("lens", [[768 + (37 * i) % 256 for i in range(64)],
                                  [1024] * 64, [512 + 8 * i for i in range(64)]],
                         ids=["ragged", "full", "growing"])
@pytest.mark.parametrize("kernel", ["tensor_cores", "cuda_cores"])
def test_decode_attention_at_batch_64_and_long_contexts(ops, lens, kernel):
    H, D = 16, 64
    new = [1] * len(lens)
    geom, qkv, pool, table, tok_pos, tok_req = _attention_case(H, H, D, 16, lens, new, 0,
                                                               torch.bfloat16, seed=64)
    st = _status()
    plan = ops.make_plan(_host_batch(lens, new), len(lens), 16)
    out = torch.full((len(lens), H * D), float("nan"), device=DEV, dtype=torch.bfloat16)
    was = ops.decode_mma
    ops.decode_mma = kernel == "tensor_cores"
    try:
        ops.attention_append(out, qkv, pool, table, tok_pos, tok_req, geom, 0.125, st, plan, True)
    finally:
        ops.decode_mma = was
    ref = _attention_reference(qkv, pool, table, lens, new, geom, 0.125)   # pages now hold the new keys
    assert st.item() == 0
    assert torch.isfinite(out).all()
    assert (out.double() - ref).abs().max() < 2e-2


def test_decode_attention_falls_back_when_its_kernel_refuses_the_shape(ops):
    """Forcing narrow CTAs and a single slice makes the CUDA-core decode kernel refuse a long
    table (a slice spans at most 32 pages per warp): the general kernel serves the batch."""
    H, D, lens = 4, 64, [700, 33, 1024]
    new = [1] * len(lens)
    geom, qkv, pool, table, tok_pos, tok_req = _attention_case(H, H, D, 16, lens, new, 0,
                                                               torch.bfloat16, seed=9)
    st = _status()
    plan = ops.make_plan(_host_batch(lens, new), len(lens), 16)
    out = torch.full((len(lens), H * D), float("nan"), device=DEV, dtype=torch.bfloat16)
    saved = ops.decode_mma, ops.decode_force
    ops.decode_mma, ops.decode_force = False, (0, 1)    # 4 warps, one slice: 128 pages at most
    try:
        # a table of more than 128 pages: widen it
        wide = torch.full((len(lens), 160), -1, dtype=torch.int32, device=DEV)
        wide[:, :table.shape[1]] = table
        from dataclasses import replace
        g2 = replace(geom, max_pages=160)
        ops.attention_append(out, qkv, pool, wide, tok_pos, tok_req, g2, 0.125, st, plan, True)
    finally:
        ops.decode_mma, ops.decode_force = saved
    ref = _attention_reference(qkv, pool, table, lens, new, geom, 0.125)
    assert st.item() == 0
    assert (out.double() - ref).abs().max() < 2e-2


LINEAR = [(2048, 3072, 1024), (2048, 1024, 1024), (2048, 4096, 1024), (2048, 1024, 4096),
          (2048, 1280, 5120), (1536, 4800, 1600)]


@pytest.mark.parametrize("M,N,K", LINEAR)
@pytest.mark.parametrize("tile_n", [0, 128, 192, 256])
def test_tcgen05_linear_with_more_tiles_than_ctas(ops, M, N, K, tile_n):
    """Every epilogue at the prefill shapes of GPT-2 medium (and one each of large and XL), at
    the tile width the planner picks (0) and at each width forced."""
    torch.manual_seed(M + N + K + tile_n)
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) / K ** 0.5).bfloat16()
    bias = torch.randn(N, device=DEV)
    ref0 = a.double() @ w.double().T + bias.double()
    saved = ops.tile_n
    ops.tile_n = tile_n
    try:
        for act, out_dtype, with_res in (("none", torch.bfloat16, False),
                                         ("gelu_tanh", torch.bfloat16, False),
                                         ("gelu_erf", torch.bfloat16, False),
                                         ("none", torch.float32, True)):
            ref = ref0
            if act == "gelu_tanh":
                ref = torch.nn.functional.gelu(ref0, approximate="tanh")
            elif act == "gelu_erf":
                ref = torch.nn.functional.gelu(ref0)
            if with_res:
                res = torch.randn(M, N, device=DEV)
                out = res.clone()
                ops.linear(out, a, w, bias, act=act, residual=out)
                ref = ref + res.double()
            else:
                out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
                ops.linear(out, a, w, bias, act=act)
            tol = 3e-2 if out_dtype == torch.bfloat16 else 2e-3
            assert (out.double() - ref).abs().max() < tol, (act, out_dtype, with_res)
        assert ops.status.item() == 0
    finally:
        ops.tile_n = saved
