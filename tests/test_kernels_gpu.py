"""Each CUDA kernel alone against its plain PyTorch twin (tests/plain_ops.py, float64), at
sizes other than the tiny models': widths and vocabularies that are no power of two, head
sizes from 16 to 256, grouped heads, windows, pages of 16 and 32 tokens."""

import pytest
import torch

import plain_ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from hetero_serve_b200.kernels import CudaOps
    return CudaOps()


@pytest.fixture(scope="module")
def plain():
    return plain_ops.PlainOps()


def _status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ embedding, norm
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(ops, plain, dtype):
    torch.manual_seed(0)
    V, P, E, n = 777, 50, 200, 13
    wte = torch.randn(V, E, device=DEV).to(dtype)
    wpe = torch.randn(P, E, device=DEV).to(dtype)
    ids = torch.randint(0, V, (n,), device=DEV, dtype=torch.int32)
    pos = torch.randint(0, P, (n,), device=DEV, dtype=torch.int32)
    req = _i32([0, 0, 1, -1, 2, 2, 2, -1, 3, 3, 3, 3, 0])
    x = torch.full((n, E), 9.0, device=DEV)
    ref = torch.empty(n, E, device=DEV, dtype=torch.float64)
    st = _status()
    ops.embed(x, ids, pos, req, wte, wpe, st)
    plain.embed(ref, ids, pos, req, wte, wpe, st)
    assert (x.double() - ref).abs().max() < 1e-6
    assert x[3].abs().max() == 0 and st.item() == 0          # padding rows are zeroed
    ops.embed(x, ids, pos, req, wte, None, st)                # no position table
    plain.embed(ref, ids, pos, req, wte, None, st)
    assert (x.double() - ref).abs().max() < 1e-6


def test_embed_flags_bad_indices_instead_of_reading_them(ops):
    wte = torch.randn(10, 32, device=DEV)
    wpe = torch.randn(4, 32, device=DEV)
    x = torch.empty(3, 32, device=DEV)
    st = _status()
    ops.embed(x, _i32([1, 10, 2]), _i32([0, 1, 4]), _i32([0, 0, 0]), wte, wpe, st)
    assert st.item() == 1 | 2 and x[1].abs().max() == 0 and x[2].abs().max() == 0
    assert torch.allclose(x[0], wte[1] + wpe[0])


@pytest.mark.parametrize("width", [16, 100, 1600, 5000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layernorm(ops, plain, width, dtype):
    torch.manual_seed(width)
    x = torch.randn(19, width, device=DEV) * 7 + 3          # large mean: centring matters
    g, b = torch.randn(width, device=DEV), torch.randn(width, device=DEV)
    out = torch.empty(19, width, device=DEV, dtype=dtype)
    ref = torch.empty(19, width, device=DEV, dtype=torch.float64)
    ops.layernorm(out, x, g, b, 1e-6)
    plain.layernorm(ref, x, g, b, 1e-6)
    tol = 5e-6 if dtype == torch.float32 else 4e-2
    assert (out.double() - ref).abs().max() < tol
    rows = _i32([18, 0, 7])
    out2 = torch.empty(3, width, device=DEV, dtype=dtype)
    ops.layernorm(out2, x, g, b, 1e-6, rows)
    assert torch.equal(out2, out[rows.long()])               # a row's result is its own


def test_layernorm_refuses_rows_that_do_not_fit_shared_memory(ops):
    from hetero_serve_b200.kernels import KernelError
    w = 60000
    x = torch.zeros(1, w, device=DEV)
    with pytest.raises(KernelError, match="unsupported"):
        ops.layernorm(torch.empty(1, w, device=DEV), x, torch.ones(w, device=DEV),
                      torch.zeros(w, device=DEV), 1e-5)


# ------------------------------------------------------------------ linear
SHAPES = [(1, 50, 24), (7, 130, 100), (64, 192, 320), (200, 1000, 96), (33, 257, 515)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", ["none", "gelu_tanh", "gelu_erf"])
def test_linear(ops, plain, M, N, K, dtype, act):
    torch.manual_seed(M * N + K)
    a = torch.randn(M, K, device=DEV).to(dtype)
    w = (torch.randn(N, K, device=DEV) / K ** 0.5).to(dtype)
    bias = torch.randn(N, device=DEV)
    out = torch.empty(M, N, device=DEV, dtype=dtype)
    ref = torch.empty(M, N, device=DEV, dtype=torch.float64)
    ops.linear(out, a, w, bias, act=act)
    plain.linear(ref, a, w, bias, act=act)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (out.double() - ref).abs().max() < tol
    # accumulate into a float32 residual in place; no bias
    res = torch.randn(M, N, device=DEV)
    acc = res.clone()
    ops.linear(acc, a, w, None, act=act, residual=acc)
    plain.linear(ref, a, w, None, act=act, residual=res)
    assert (acc.double() - ref).abs().max() < (2e-5 if dtype == torch.float32 else 2e-3 * K ** 0.5)


TC_SHAPES = [(1, 1000, 96), (5, 50257, 64), (16, 192, 320), (17, 1024, 1024), (40, 288, 96),
             (64, 1024, 4096), (100, 3072, 1024), (128, 64, 64), (129, 257, 520), (300, 1000, 1600)]


@pytest.mark.parametrize("M,N,K", TC_SHAPES + [(256, 128, 64), (700, 1000, 1000), (1024, 3072, 1024)])
@pytest.mark.parametrize("path", ["few_rows", "tcgen05", "splits_through_scratch", "tiles_of_192",
                                  "cta_pairs"])
def test_bfloat16_linear_kernels_each_on_its_own(ops, plain, M, N, K, path):
    """The weight-streaming kernel (up to 64 rows, k a multiple of 32), the tcgen05 kernel
    (any rows; few rows take its split over k, whose shares travel inside a thread-block
    cluster or, once more, through scratch memory; once more with its 192-column tiles, which
    the shapes here would not choose) and its variant on pairs of CTAs (cta_group::2, 256-row
    tiles) forced one at a time, all epilogues."""
    if path == "few_rows" and (M > 64 or K % 32):
        pytest.skip("the few-row kernel takes up to 64 rows and k in multiples of 32")
    if path in ("few_rows", "tcgen05", "splits_through_scratch") and M > 300:
        pytest.skip("the larger shapes are there for the pairs and the 192-column tiles")
    if path == "tiles_of_192" and K % 8:
        pytest.skip("TMA needs rows of a multiple of 16 bytes")
    if path == "cta_pairs" and K % 8:
        pytest.skip("TMA needs rows of a multiple of 16 bytes")
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device=DEV).bfloat16()
    w = (torch.randn(N, K, device=DEV) / K ** 0.5).bfloat16()
    bias = torch.randn(N, device=DEV)
    saved = ops.skinny_max_rows, ops.cta_pairs, ops.tile_n, ops.split_clusters
    ops.skinny_max_rows = 64 if path == "few_rows" else 0
    ops.cta_pairs = 1 if path == "cta_pairs" else 0
    ops.tile_n = 192 if path == "tiles_of_192" else 0
    ops.split_clusters = path != "splits_through_scratch"
    try:
        for act, out_dtype, with_res in (("none", torch.bfloat16, False), ("gelu_tanh", torch.bfloat16, False),
                                         ("gelu_erf", torch.bfloat16, False), ("none", torch.float32, False),
                                         ("none", torch.float32, True)):
            ref = torch.empty(M, N, device=DEV, dtype=torch.float64)
            if with_res:
                res = torch.randn(M, N, device=DEV)
                out = res.clone()
                ops.linear(out, a, w, bias, act=act, residual=out)
                plain.linear(ref, a, w, bias, act=act, residual=res)
            else:
                out = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
                ops.linear(out, a, w, bias, act=act)
                plain.linear(ref, a, w, bias, act=act)
            tol = 3e-2 if out_dtype == torch.bfloat16 else 2e-3      # hardware tanh: 2^-11
            assert (out.double() - ref).abs().max() < tol, (act, out_dtype, with_res)
            # launched twice: scratch and counters of a split launch are left ready
            if with_res:
                out2 = res.clone()
                ops.linear(out2, a, w, bias, act=act, residual=out2)
                assert torch.equal(out, out2)
        assert ops.status.item() == 0
    finally:
        ops.skinny_max_rows, ops.cta_pairs, ops.tile_n, ops.split_clusters = saved


@pytest.mark.parametrize("M,N,K", [(1, 192, 64), (8, 3072, 1024), (16, 4096, 1024), (5, 288, 96),
                                   (16, 4800, 1600), (9, 1024, 4096), (30, 320, 2048),
                                   (200, 1000, 96)])
def test_layernorm_fused_into_the_linear(ops, plain, M, N, K):
    torch.manual_seed(M * K + N)
    x = torch.randn(M, K, device=DEV) * 4 + 2
    g, b = torch.randn(K, device=DEV), torch.randn(K, device=DEV)
    w = (torch.randn(N, K, device=DEV) / K ** 0.5).bfloat16()
    bias = torch.randn(N, device=DEV)
    out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    h = torch.empty(M, K, device=DEV, dtype=torch.bfloat16)
    ref = torch.empty(M, N, device=DEV, dtype=torch.float64)
    href = torch.empty(M, K, device=DEV, dtype=torch.bfloat16)
    before = ops.launches
    ops.norm_linear(out, h, x, g, b, 1e-6, w, bias, act="gelu_tanh")
    fused = ops.launches - before == 1
    assert fused == (M <= ops.skinny_max_rows and K % 32 == 0)
    plain.norm_linear(ref, href, x, g, b, 1e-6, w, bias, act="gelu_tanh")
    assert (out.double() - ref).abs().max() < 3e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_linear_rows_do_not_depend_on_the_batch(ops, dtype):
    torch.manual_seed(5)
    a = torch.randn(150, 96, device=DEV).to(dtype)
    w = torch.randn(1000, 96, device=DEV).to(dtype)
    full = torch.empty(150, 1000, device=DEV, dtype=dtype)
    ops.linear(full, a, w)
    for lo, hi in ((0, 1), (63, 66), (149, 150)):
        part = torch.empty(hi - lo, 1000, device=DEV, dtype=dtype)
        ops.linear(part, a[lo:hi].contiguous(), w)
        assert torch.equal(part, full[lo:hi])


def test_linear_checks_its_arguments(ops):
    from hetero_serve_b200.kernels import KernelError
    a = torch.randn(4, 8, device=DEV)
    w = torch.randn(6, 8, device=DEV)
    with pytest.raises(KernelError, match="do not fit"):
        ops.linear(torch.empty(4, 5, device=DEV), a, w)
    with pytest.raises(KernelError, match="dtype"):
        ops.linear(torch.empty(4, 6, device=DEV), a, w.bfloat16())
    with pytest.raises(KernelError, match="CUDA tensor"):
        ops.linear(torch.empty(4, 6), a.cpu(), w.cpu())
    with pytest.raises(KernelError, match="contiguous"):
        ops.linear(torch.empty(4, 6, device=DEV), a, torch.randn(8, 6, device=DEV).t())


# ------------------------------------------------------------------ cache and attention
def _attention_case(H, HK, D, PS, lens, new, window=0, dtype=torch.float32, seed=0, scramble=True):
    """Requests with ``lens[r]`` tokens after the step, of which the last ``new[r]`` are in
    the batch.  Earlier keys/values are laid into pages directly."""
    from hetero_serve_b200.kernels import AttentionGeometry
    g_ = torch.Generator(device="cpu").manual_seed(seed)
    R = len(lens)
    max_pages = max(-(-n // PS) for n in lens) + 1
    n_pages = sum(-(-n // PS) for n in lens) + 3
    perm = torch.randperm(n_pages, generator=g_).tolist() if scramble else list(range(n_pages))
    table = torch.full((R, max_pages), -1, dtype=torch.int32)
    it = iter(perm)
    for r, n in enumerate(lens):
        for i in range(-(-n // PS)):
            table[r, i] = next(it)
    W = (H + 2 * HK) * D
    geom = AttentionGeometry(H, HK, D, PS, n_pages, max_pages, 0, H * D, (H + HK) * D, W, window)
    T = sum(new)
    qkv = torch.randn(T, W, generator=g_).to(dtype)
    pool = torch.full((n_pages, 2, HK, PS, D), float("nan")).to(dtype)   # unwritten slots poison
    tok_pos, tok_req = [], []
    for r, (n, k) in enumerate(zip(lens, new)):
        past = torch.randn(n - k, 2, HK, D, generator=g_).to(dtype)
        for p in range(n - k):
            pool[table[r, p // PS], :, :, p % PS, :] = past[p]
        tok_pos += list(range(n - k, n))
        tok_req += [r] * k
    return (geom, qkv.to(DEV), pool.to(DEV), table.to(DEV), _i32(tok_pos), _i32(tok_req))


CASES = [
    # H, HK, D,  PS, lens,            new,           window
    (4, 4, 16, 16, [5, 17, 33], [5, 17, 33], 0),            # whole prompts
    (3, 3, 32, 16, [40, 16, 70, 1], [1, 1, 1, 1], 0),       # decode, a page edge (16), one token
    (6, 2, 64, 16, [50, 23], [7, 23], 0),                   # grouped heads, portion + prompt
    (2, 1, 128, 32, [100, 64], [3, 1], 0),                  # pages of 32
    (1, 1, 256, 16, [35], [2], 0),                          # the largest head
    (5, 5, 48, 16, [90, 31], [30, 1], 0),                   # head size 48, five heads
    (4, 2, 32, 16, [80, 40, 20], [10, 1, 20], 24),          # a window of 24
    (2, 2, 16, 16, [48], [48], 16),                         # window == page
]


@pytest.mark.parametrize("case", CASES, ids=[f"H{c[0]}k{c[1]}D{c[2]}P{c[3]}w{c[6]}" for c in CASES])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kv_append_and_attention(ops, plain, case, dtype):
    H, HK, D, PS, lens, new, window = case
    geom, qkv, pool, table, tok_pos, tok_req = _attention_case(H, HK, D, PS, lens, new, window,
                                                               dtype, seed=D + H)
    st = _status()
    pool_ref = pool.clone()
    ops.kv_append(pool, qkv, table, tok_pos, tok_req, geom, st)
    plain.kv_append(pool_ref, qkv, table, tok_pos, tok_req, geom, st)
    assert torch.equal(torch.nan_to_num(pool, nan=123.0), torch.nan_to_num(pool_ref, nan=123.0))
    T = qkv.shape[0]
    out = torch.empty(T, H * D, device=DEV, dtype=dtype)
    ref = torch.empty(T, H * D, device=DEV, dtype=torch.float64)
    scale = 0.37 / D ** 0.5
    ops.attention(out, qkv, pool, table, tok_pos, tok_req, geom, scale, st)
    plain.attention(ref, qkv, pool, table, tok_pos, tok_req, geom, scale, st)
    assert st.item() == 0
    assert torch.isfinite(out).all()           # no poisoned (unwritten or foreign) slot was read
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (out.double() - ref).abs().max() < tol


def _host_batch(lens, new):
    return [(f"r{r}", r, n - k, k) for r, (n, k) in enumerate(zip(lens, new))]


@pytest.fixture
def decode_kernel(request, ops):
    """Which kernel serves single-query tokens: the tensor-core one where the shape allows it
    (head sizes 32/64/128), or the CUDA-core one everywhere."""
    was = ops.decode_mma
    ops.decode_mma = {"tensor_cores": True, "cuda_cores": False}[request.param]
    yield request.param
    ops.decode_mma = was


DECODE_KERNELS = ["tensor_cores", "cuda_cores"]


FAST_CASES = [
    # H, HK, D, PS, lens, new     (bfloat16, no window: the specialised kernels)
    (4, 4, 16, 16, [5, 17, 33, 200], [5, 17, 33, 200]),          # prompts: tensor-core tiles
    (3, 3, 32, 16, [40, 16, 70, 1, 300], [1, 1, 1, 1, 1]),       # single queries: split contexts
    (16, 16, 64, 16, [1024, 700, 64, 65], [1, 1, 1, 2]),         # long contexts, many splits
    (6, 2, 64, 16, [150, 23, 90, 77], [70, 23, 3, 1]),           # grouped heads; both kernels
    (2, 1, 128, 32, [300, 64, 129], [130, 1, 129]),              # pages of 32, head size 128
    (5, 5, 32, 48, [100, 130], [100, 2]),                        # pages of 48
    (2, 2, 64, 16, [64, 63, 65, 128, 1, 300], [64, 63, 65, 64, 1, 129]),   # tile edges
    # head sizes that are no power of two: prompt portions only (the single-query kernels do not
    # take them; a batch that has such tokens goes to the general kernel whole)
    (3, 3, 48, 16, [70, 130, 9, 200], [70, 130, 9, 66]),
    (2, 1, 80, 16, [150, 64, 30], [150, 20, 30]),
    (4, 2, 96, 16, [129, 300, 40], [129, 65, 40]),
    (2, 2, 112, 32, [200, 65], [200, 5]),
]


@pytest.mark.parametrize("decode_kernel", DECODE_KERNELS, indirect=True)
@pytest.mark.parametrize("case", FAST_CASES,
                         ids=[f"H{c[0]}k{c[1]}D{c[2]}P{c[3]}n{len(c[4])}" for c in FAST_CASES])
def test_specialised_attention_kernels(ops, plain, case, decode_kernel):
    H, HK, D, PS, lens, new = case
    geom, qkv, pool, table, tok_pos, tok_req = _attention_case(H, HK, D, PS, lens, new, 0,
                                                               torch.bfloat16, seed=H * D)
    st = _status()
    ops.kv_append(pool, qkv, table, tok_pos, tok_req, geom, st)
    T = qkv.shape[0]
    plan = ops.make_plan(_host_batch(lens, new), T, PS)
    assert plan.decode_cap == sum(k for k in new if k <= 4)
    assert plan.tile_cap == sum(-(-k // 128) for k in new if k > 4)
    out = torch.full((T, H * D), float("nan"), device=DEV, dtype=torch.bfloat16)
    ref = torch.empty(T, H * D, device=DEV, dtype=torch.float64)
    scale = 0.9 / D ** 0.5
    before = ops.launches
    ops.attention(out, qkv, pool, table, tok_pos, tok_req, geom, scale, st, plan)
    assert ops.launches - before == (plan.decode_cap > 0) + (plan.tile_cap > 0)
    plain.attention(ref, qkv, pool, table, tok_pos, tok_req, geom, scale, st)
    assert st.item() == 0
    assert torch.isfinite(out).all()
    assert (out.double() - ref).abs().max() < 2e-2
    # a second launch reuses the scratch memory and its counters
    out2 = torch.empty_like(out)
    ops.attention(out2, qkv, pool, table, tok_pos, tok_req, geom, scale, st, plan)
    assert torch.equal(out, out2)
    # and agrees with the general kernel to rounding
    gen = torch.empty_like(out)
    ops.attention(gen, qkv, pool, table, tok_pos, tok_req, geom, scale, st, None)
    assert (out.float() - gen.float()).abs().max() < 2e-2


DECODE_ONLY = [
    # H, HK, D, PS, lens: every request brings one token -> append fused into the decode kernel
    (16, 16, 64, 16, [1024, 700, 64, 65, 1, 16, 17, 513]),       # wide CTAs, one slice
    (4, 2, 32, 16, [300]),                                         # few pairs: several slices
    (8, 8, 128, 32, [90] * 40),                                    # many pairs: narrow CTAs
    (2, 1, 16, 16, [33, 2]),
    (6, 2, 64, 16, [1, 2, 31, 32, 33, 64, 65, 500, 1000, 96, 97]),  # grouped heads, chunk edges
    (3, 3, 32, 48, [200, 49, 48, 47, 700]),                        # pages of 48, head size 32
    (20, 20, 64, 16, [600] * 16),                                  # 320 pairs: narrow CTAs
    (16, 16, 64, 16, [300, 31, 97] * 4),                           # 192 pairs: between the two
    (8, 8, 32, 16, [150, 33] * 12),                                # the same for head size 32
    (8, 8, 32, 16, [70] * 40),
    (16, 16, 64, 16, [90, 17, 160, 33] * 8),                       # 512 pairs: four CTAs an SM
    (16, 16, 64, 16, [5000, 2049, 100]),                           # beyond 2,048 keys: slices, merged
    (4, 2, 64, 16, [6000]),                                        # a long table, two pairs: many slices
    (2, 2, 128, 32, [4100, 33, 2048, 2047]),
]


@pytest.mark.parametrize("decode_kernel", DECODE_KERNELS, indirect=True)
@pytest.mark.parametrize("case", DECODE_ONLY, ids=[f"H{c[0]}D{c[2]}n{len(c[4])}" for c in DECODE_ONLY])
def test_decode_attention_with_the_append_fused_in(ops, plain, case, decode_kernel):
    H, HK, D, PS, lens = case
    new = [1] * len(lens)
    geom, qkv, pool, table, tok_pos, tok_req = _attention_case(H, HK, D, PS, lens, new, 0,
                                                               torch.bfloat16, seed=7 * D + H)
    st = _status()
    T = qkv.shape[0]
    plan = ops.make_plan(_host_batch(lens, new), T, PS)
    assert plan.single_new and plan.tile_cap == 0
    pool_ref = pool.clone()
    out = torch.full((T, H * D), float("nan"), device=DEV, dtype=torch.bfloat16)
    ref = torch.empty(T, H * D, device=DEV, dtype=torch.float64)
    before = ops.launches
    ops.attention_append(out, qkv, pool, table, tok_pos, tok_req, geom, 0.11, st, plan, True)
    assert ops.launches - before == 1                      # one kernel does both
    plain.attention_append(ref, qkv, pool_ref, table, tok_pos, tok_req, geom, 0.11, st, None, True)
    assert st.item() == 0
    # the pages hold the new keys and values, bit for bit
    assert torch.equal(torch.nan_to_num(pool, nan=9.0), torch.nan_to_num(pool_ref, nan=9.0))
    assert torch.isfinite(out).all()
    assert (out.double() - ref).abs().max() < 2e-2
    # a reader of somebody else's cache entry does not write
    pool2 = pool_ref.clone()
    ops.attention_append(out, qkv, pool2, table, tok_pos, tok_req, geom, 0.11, st, plan, False)
    assert torch.equal(torch.nan_to_num(pool2, nan=9.0), torch.nan_to_num(pool_ref, nan=9.0))


@pytest.mark.parametrize("far", [0, 700, 2047, 2048, 3500, 4999])
def test_far_key_in_every_slice_of_a_long_context(ops, far):
    """One request of 5,000 keys: its context is cut into slices between CTAs.  A planted key
    decides the output wherever it lies (a slice dropped, or merged with a wrong weight, shows)."""
    H, D, PS, n = 4, 64, 16, 5000
    geom, qkv, pool, table, tok_pos, tok_req = _attention_case(H, H, D, PS, [n], [1], 0,
                                                               torch.bfloat16, 5)
    st = _status()
    ops.kv_append(pool, qkv, table, tok_pos, tok_req, geom, st)
    pv = pool.view(geom.num_pages, 2, H, PS, D)
    q = qkv[-1, :H * D].view(H, D).float()
    page, slot = int(table[0, far // PS]), far % PS
    pv[page, 0, :, slot, :] = (q / q.norm(dim=-1, keepdim=True) * 40).to(torch.bfloat16)
    out = torch.empty(1, H * D, device=DEV, dtype=torch.bfloat16)
    plan = ops.make_plan(_host_batch([n], [1]), 1, PS)
    ops.attention(out, qkv, pool, table, tok_pos, tok_req, geom, 1.0, st, plan)
    want = pv[page, 1, :, slot, :].reshape(H * D).float()
    assert st.item() == 0
    assert (out[-1].float() - want).abs().max() < 2e-2


@pytest.mark.parametrize("far", [0, 63, 64, 500, 1000])
@pytest.mark.parametrize("new", [1, 100])
def test_far_key_with_the_specialised_kernels(ops, far, new):
    H, D, PS, n = 4, 64, 16, 1024
    geom, qkv, pool, table, tok_pos, tok_req = _attention_case(H, H, D, PS, [n], [new], 0,
                                                               torch.bfloat16, 3)
    st = _status()
    ops.kv_append(pool, qkv, table, tok_pos, tok_req, geom, st)
    far = min(far, n - new)                      # a key every query of the portion can see
    pv = pool.view(geom.num_pages, 2, H, PS, D)
    q = qkv[-1, :H * D].view(H, D).float()       # the last query
    page, slot = int(table[0, far // PS]), far % PS
    pv[page, 0, :, slot, :] = (q / q.norm(dim=-1, keepdim=True) * 40).to(torch.bfloat16)
    out = torch.empty(new, H * D, device=DEV, dtype=torch.bfloat16)
    plan = ops.make_plan(_host_batch([n], [new]), new, PS)
    ops.attention(out, qkv, pool, table, tok_pos, tok_req, geom, 1.0, st, plan)
    want = pv[page, 1, :, slot, :].reshape(H * D).float()
    assert (out[-1].float() - want).abs().max() < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("far", [0, 15, 16, 255, 256, 511, 600])
def test_one_far_key_among_hundreds_decides_the_output(ops, dtype, far):
    """Random scores are nearly uniform, which hides a key that is dropped or misplaced.
    Here one key's score stands out, so the output must be that key's value row."""
    H, D, PS, n = 2, 64, 16, 640
    geom, qkv, pool, table, tok_pos, tok_req = _attention_case(H, H, D, PS, [n], [1], 0, dtype, 3)
    st = _status()
    ops.kv_append(pool, qkv, table, tok_pos, tok_req, geom, st)
    pv = pool.view(geom.num_pages, 2, H, PS, D)
    q = qkv[0, :H * D].view(H, D).float()
    page, slot = int(table[0, far // PS]), far % PS
    pv[page, 0, :, slot, :] = (q / q.norm(dim=-1, keepdim=True) * 40).to(dtype)  # score ~ 40*|q|
    out = torch.empty(1, H * D, device=DEV, dtype=dtype)
    ops.attention(out, qkv, pool, table, tok_pos, tok_req, geom, 1.0, st)
    want = pv[page, 1, :, slot, :].reshape(1, H * D).float()
    assert (out.float() - want).abs().max() < (1e-4 if dtype == torch.float32 else 2e-2)


def test_window_edge_is_exact(ops):
    """With a window w the key at p - w is out and the key at p - w + 1 is in."""
    H, D, PS, n, w = 1, 16, 16, 50, 20
    geom, qkv, pool, table, tok_pos, tok_req = _attention_case(H, H, D, PS, [n], [1], w,
                                                               torch.float32, 4)
    st = _status()
    ops.kv_append(pool, qkv, table, tok_pos, tok_req, geom, st)
    pv = pool.view(geom.num_pages, 2, H, PS, D)
    q = qkv[0, :D].float()
    big = q / q.norm() * 60
    out = torch.empty(1, D, device=DEV)
    p = n - 1
    for key, inside in ((p - w, False), (p - w + 1, True)):
        page, slot = int(table[0, key // PS]), key % PS
        saved = pv[page, 0, 0, slot].clone()
        pv[page, 0, 0, slot] = big
        ops.attention(out, qkv, pool, table, tok_pos, tok_req, geom, 1.0, st)
        hit = (out[0] - pv[page, 1, 0, slot]).abs().max() < 1e-4
        assert bool(hit) == inside
        pv[page, 0, 0, slot] = saved


def test_attention_flags_a_bad_page(ops):
    geom, qkv, pool, table, tok_pos, tok_req = _attention_case(2, 2, 16, 16, [20], [1])
    table[0, 0] = geom.num_pages + 5
    st = _status()
    out = torch.empty(1, 32, device=DEV)
    ops.attention(out, qkv, pool, table, tok_pos, tok_req, geom, 1.0, st)
    assert st.item() & 4


def test_attention_refuses_head_sizes_it_does_not_take(ops):
    from hetero_serve_b200.kernels import AttentionGeometry, KernelError
    for D in (24, 272):
        g = AttentionGeometry(1, 1, D, 16, 2, 2, 0, D, 2 * D, 3 * D)
        qkv = torch.zeros(1, 3 * D, device=DEV)
        pool = torch.zeros(2, 2, 1, 16, D, device=DEV)
        with pytest.raises(KernelError, match="unsupported"):
            ops.attention(torch.empty(1, D, device=DEV), qkv, pool,
                          torch.zeros(1, 2, dtype=torch.int32, device=DEV), _i32([0]), _i32([0]),
                          g, 1.0, _status())


# ------------------------------------------------------------------ sampling
@pytest.mark.parametrize("vocab", [17, 1000, 50257])
def test_argmax_lowest_index_on_ties(ops, vocab):
    torch.manual_seed(vocab)
    lg = torch.randn(5, vocab, device=DEV)
    lg[1, vocab - 1] = lg[1, 3] = 50.0
    lg[2, :] = 1.0
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax(out, lg)
    want = [int(torch.argmax(lg[0])), 3, 0, int(torch.argmax(lg[3])), int(torch.argmax(lg[4]))]
    assert out.tolist() == want


@pytest.mark.parametrize("M,N,K", [(1, 50257, 1024), (8, 50257, 1024), (16, 50257, 1600),
                                   (3, 517, 64), (8, 1000, 128), (13, 40000, 768), (5, 17, 32)])
def test_head_with_the_greedy_choice_fused_in(ops, M, N, K):
    """linear_argmax: the logits equal those of `linear`, the tokens are the lowest index of
    each row's maximum (ties planted across feature blocks and CTAs, and a row whose values
    are all equal), the status word follows the tokens, feedback slots receive their tokens
    and slots below zero are skipped; a second launch finds the counter at zero again."""
    torch.manual_seed(M * N + K)
    a = (torch.randn(M, K, device=DEV) * 0.5).bfloat16()
    w = (torch.randn(N, K, device=DEV) * 0.5).bfloat16()
    if N > 600:                                 # equal rows of the table give equal logits
        w[N - 1] = w[3]
        w[N // 2] = w[3]
    a[M - 1] = 0 if M > 1 else a[M - 1]          # a row of zeros: every logit equal -> token 0
    plain_out = torch.empty(M, N, device=DEV)
    ops.linear(plain_out, a, w)
    for _ in range(2):
        out = torch.full((M, N), float("nan"), device=DEV)
        tokens = torch.full((M + 1,), -7, dtype=torch.int32, device=DEV)
        feedback = torch.full((M + 2,), -1, dtype=torch.int32, device=DEV)
        slot = torch.arange(M, dtype=torch.int32, device=DEV) + 1
        slot[0] = -1
        status = torch.tensor([1234], dtype=torch.int32, device=DEV)
        assert ops.linear_argmax(out, a, w, tokens, feedback=feedback, feedback_slot=slot,
                                 status_word=status)
        assert torch.equal(out, plain_out)
        ref = out.double()
        want = [int((ref[m] == ref[m].max()).nonzero()[0]) for m in range(M)]
        assert tokens[:M].tolist() == want
        assert int(tokens[M]) == 1234
        assert feedback[0].item() == -1 and feedback[1].item() == -1     # slot -1 and no row for 1
        assert feedback[2:M + 1].tolist() == want[1:]
    if M > 1:
        assert want[M - 1] == 0


def test_head_with_the_greedy_choice_refuses_what_it_does_not_take(ops):
    a = torch.randn(40, 64, device=DEV).bfloat16()
    w = torch.randn(100, 64, device=DEV).bfloat16()
    out = torch.empty(40, 100, device=DEV)
    tokens = torch.zeros(41, dtype=torch.int32, device=DEV)
    assert ops.linear_argmax(out, a, w, tokens) is False                 # too many rows
    assert ops.linear_argmax(out[:4].float(), a[:4].float(), w.float(), tokens) is False


@pytest.mark.parametrize("vocab,top_k", [(1000, 0), (1000, 1), (1000, 40), (50257, 0),
                                         (50257, 50), (37, 36), (37, 100), (50257, 50256),
                                         (1025, 7), (60001, 0), (60001, 300)])   # 60001: too long for shared memory
def test_sample_matches_the_plain_sampler(ops, plain, vocab, top_k):
    torch.manual_seed(vocab + top_k)
    rows = 8
    lg = torch.randn(rows, vocab, device=DEV) * 2.5
    lg[5, 7] = lg[5, 2] = lg[5].max() + 1                   # a tie at the top
    temp = torch.tensor([0.8, 0.0, 1.7, 0.3, 1.0, 1.0, 0.05, 3.0], device=DEV)
    k = torch.full((rows,), top_k, dtype=torch.int32, device=DEV)
    lo = torch.arange(rows, dtype=torch.int32, device=DEV) * 1000003
    hi = torch.arange(rows, dtype=torch.int32, device=DEV)
    mism = 0
    for pos in range(6):
        p = torch.full((rows,), pos + 11, dtype=torch.int32, device=DEV)
        out = torch.empty(rows, dtype=torch.int32, device=DEV)
        ref = torch.empty(rows, dtype=torch.int32)
        ops.sample(out, lg, temp, k, lo, hi, p)
        plain.sample(ref, lg.cpu(), temp.cpu(), k.cpu(), lo.cpu(), hi.cpu(), p.cpu())
        mism += sum(int(a != b) for a, b in zip(out.tolist(), ref.tolist()))
    # float32 against float64 cumulative sums may disagree when u lands within rounding of a
    # boundary; with 48 draws that is not expected at all
    assert mism == 0


def test_sample_distribution(ops):
    """Over many positions the draws follow softmax(logits / T) restricted to the top k."""
    vocab, n = 12, 4000
    lg = torch.tensor([[0.1, 2.0, -1.0, 0.5, 1.5, 1.5, -3.0, 0.0, 0.7, 1.1, -0.4, 0.9]], device=DEV)
    lgs = lg.expand(n, vocab).contiguous()
    temp = torch.full((n,), 0.7, device=DEV)
    k = torch.full((n,), 5, dtype=torch.int32, device=DEV)
    z = torch.zeros(n, dtype=torch.int32, device=DEV)
    pos = torch.arange(n, dtype=torch.int32, device=DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(out, lgs, temp, k, z + 5, z, pos)
    keep = torch.topk(lg[0], 5).indices
    p = torch.zeros(vocab, device=DEV)
    p[keep] = torch.softmax(lg[0, keep] / 0.7, 0)
    freq = torch.bincount(out.long(), minlength=vocab).float() / n
    assert (freq - p).abs().max() < 0.03
    assert freq[p == 0].sum() == 0


def test_tokens_kept_on_the_device_feed_the_next_embedding(ops, plain):
    """Sampling leaves a row's token in ``feedback[slot]`` (slots below zero are skipped); the
    embedding takes ``feedback[s]`` for an id ``-(s + 1)`` and checks it like any other id."""
    torch.manual_seed(3)
    V, E = 300, 48
    lg = torch.randn(5, V, device=DEV)
    temp = torch.tensor([0.0, 0.9, 0.0, 1.2, 0.0], device=DEV)
    k = _i32([0, 0, 0, 7, 0])
    z = torch.zeros(5, dtype=torch.int32, device=DEV)
    pos = _i32([4, 9, 1, 30, 2])
    slots = _i32([3, -1, 0, 6, -1])
    fb = torch.full((8,), 77, dtype=torch.int32, device=DEV)
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.sample(out, lg, temp, k, z + 11, z, pos, feedback=fb, feedback_slot=slots)
    plain_out = torch.empty(5, dtype=torch.int32)
    plain.sample(plain_out, lg.cpu(), temp.cpu(), k.cpu(), (z + 11).cpu(), z.cpu(), pos.cpu())
    assert out.cpu().tolist() == plain_out.tolist()
    want = [77] * 8
    want[3], want[0], want[6] = int(out[0]), int(out[2]), int(out[3])
    assert fb.cpu().tolist() == want
    # the embedding of ids given directly and through the device copy agree bit for bit
    wte = torch.randn(V, E, device=DEV)
    wpe = torch.randn(40, E, device=DEV)
    st = _status()
    direct = torch.empty(4, E, device=DEV)
    via = torch.empty(4, E, device=DEV)
    p4, r4 = _i32([5, 10, 2, 31]), _i32([0, 1, 2, 3])
    ops.embed(direct, _i32([want[3], 12, want[0], want[6]]), p4, r4, wte, wpe, st)
    ops.embed(via, _i32([-(3 + 1), 12, -(0 + 1), -(6 + 1)]), p4, r4, wte, wpe, st, feedback=fb)
    assert st.item() == 0 and torch.equal(direct, via)
    # a slot outside the table, a negative id without a table, a kept token outside the vocabulary
    ops.embed(via, _i32([-9, 1, 1, 1]), p4, r4, wte, wpe, st, feedback=fb)
    assert st.item() == 1 and via[0].abs().max() == 0
    st.zero_()
    ops.embed(via, _i32([-1, 1, 1, 1]), p4, r4, wte, wpe, st)
    assert st.item() == 1
    st.zero_()
    fb[2] = V
    ops.embed(via, _i32([-3, 1, 1, 1]), p4, r4, wte, wpe, st, feedback=fb)
    assert st.item() == 1 and via[0].abs().max() == 0
