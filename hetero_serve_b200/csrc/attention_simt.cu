// Paged key/value append and a general causal attention over the paged cache on the CUDA cores.
//
// Cache layout of one cache entry (one layer's keys and values):
//     pool[page][kv][kv_head][slot][d]      kv: 0 = keys, 1 = values
// so the `page_size x head_dim` tile of one (page, head) is contiguous.  The reference keeps
// [page][slot][head][d] (heteroserve/kv/blocks.py:8-11); the layout is private to the cache
// and these kernels.  A request's token at position p lives in page table[p / page_size],
// slot p % page_size (heteroserve/model/torch_engine.py:292-294, kv/torch_blocks.py:68-73).
//
// Order inside a layer, as in the reference (torch_engine.py:306-314): the new keys and values
// are written first, then attention reads positions 0..p from the pages, the new ones included.
//
// attention_simt_kernel: one warp per (token, head).  Keys are taken 32 at a time in position
// order, one key per lane; scores = (q . k) * scale with the multiply after the dot product
// (torch_engine.py:135); the running maximum, the running sum and the output accumulators are
// float32 (online softmax, as heteroserve/model/paged_attn_v2.py:124-156).  The order of every
// sum depends only on the key positions, never on the batch.
#include "common.cuh"

namespace hs {

struct AttnGeom {
  int n_heads, n_kv_heads, head_dim, page_size, num_pages, max_pages;
  int q_off, k_off, v_off, qkv_stride;  // columns of q | k | v in a row of the fused buffer
  int window;                           // 0: all keys; w: keys p-w+1 .. p
};

template <typename T>
__global__ void kv_append_kernel(T* __restrict__ pool, const T* __restrict__ qkv,
                                 const int* __restrict__ table, const int* __restrict__ tok_pos,
                                 const int* __restrict__ tok_req, AttnGeom g, int* status) {
  pdl_trigger();
  const int t = blockIdx.x;
  const int r = tok_req[t];
  const int p = tok_pos[t];
  const bool pos_ok = r >= 0 && p >= 0 && p / g.page_size < g.max_pages;
  const int page = pos_ok ? table[(size_t)r * g.max_pages + p / g.page_size] : -1;
  pdl_wait();           // the rows of `qkv` are what the previous kernel wrote
  if (r < 0) return;
  if (!pos_ok) {
    if (threadIdx.x == 0) atomicOr(status, HS_STATUS_BAD_POSITION);
    return;
  }
  if (page < 0 || page >= g.num_pages) {
    if (threadIdx.x == 0) atomicOr(status, HS_STATUS_BAD_PAGE);
    return;
  }
  const int slot = p % g.page_size;
  const int kvw = g.n_kv_heads * g.head_dim;
  const size_t tile = (size_t)g.page_size * g.head_dim;
  const T* src = qkv + (size_t)t * g.qkv_stride;
  T* pk = pool + (size_t)page * 2 * g.n_kv_heads * tile;
  T* pv = pk + (size_t)g.n_kv_heads * tile;
  // 16 bytes at a time (head sizes are multiples of 16 elements) when the columns are aligned
  constexpr int VEC = 16 / sizeof(T);
  if ((g.k_off % VEC == 0) && (g.v_off % VEC == 0) && (g.qkv_stride % VEC == 0)) {
    for (int e = threadIdx.x * VEC; e < kvw; e += blockDim.x * VEC) {
      const int hk = e / g.head_dim, d = e - hk * g.head_dim;
      const size_t dst = (size_t)hk * tile + (size_t)slot * g.head_dim + d;
      *(uint4*)(pk + dst) = *(const uint4*)(src + g.k_off + e);
      *(uint4*)(pv + dst) = *(const uint4*)(src + g.v_off + e);
    }
    return;
  }
  for (int e = threadIdx.x; e < kvw; e += blockDim.x) {
    const int hk = e / g.head_dim, d = e - hk * g.head_dim;
    const size_t dst = (size_t)hk * tile + (size_t)slot * g.head_dim + d;
    pk[dst] = src[g.k_off + e];
    pv[dst] = src[g.v_off + e];
  }
}

constexpr int AS_WARPS = 4;
constexpr int AS_MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(AS_WARPS * 32)
attention_simt_kernel(T* __restrict__ out, const T* __restrict__ qkv, const T* __restrict__ pool,
                      const int* __restrict__ table, const int* __restrict__ tok_pos,
                      const int* __restrict__ tok_req, AttnGeom g, float scale, int* status) {
  extern __shared__ float sq_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int h = blockIdx.y * AS_WARPS + warp;
  if (h >= g.n_heads) return;
  const int D = g.head_dim;
  float* sq = sq_all + warp * D;
  T* orow = out + (size_t)t * g.n_heads * D + (size_t)h * D;
  const int r = tok_req[t];
  const int p = tok_pos[t];
  if (r < 0 || p < 0 || p / g.page_size >= g.max_pages) {
    for (int d = lane; d < D; d += 32) orow[d] = from_f<T>(0.f);
    return;
  }
  const int hk = h / (g.n_heads / g.n_kv_heads);
  const T* qrow = qkv + (size_t)t * g.qkv_stride + g.q_off + (size_t)h * D;
  for (int d = lane; d < D; d += 32) sq[d] = to_f(qrow[d]);
  __syncwarp();

  const size_t tile = (size_t)g.page_size * D;
  const size_t page_stride = 2 * (size_t)g.n_kv_heads * tile;
  const int* trow = table + (size_t)r * g.max_pages;
  const int lo = (g.window > 0 && p - g.window + 1 > 0) ? p - g.window + 1 : 0;

  float m = -INFINITY, l = 0.f;
  float acc[AS_MAX_D / 32];
#pragma unroll
  for (int i = 0; i < AS_MAX_D / 32; ++i) acc[i] = 0.f;

  for (int j0 = lo; j0 <= p; j0 += 32) {
    const int j = j0 + lane;
    const bool valid = j <= p;
    float s = -INFINITY;
    long long voff = -1;
    if (valid) {
      const int page = trow[j / g.page_size];
      if (page < 0 || page >= g.num_pages) {
        atomicOr(status, HS_STATUS_BAD_PAGE);
      } else {
        const size_t koff = (size_t)page * page_stride + (size_t)hk * tile +
                            (size_t)(j % g.page_size) * D;
        voff = (long long)(koff + (size_t)g.n_kv_heads * tile);
        const T* krow = pool + koff;
        float dot = 0.f;
        for (int d = 0; d < D; ++d) dot = fmaf(sq[d], to_f(krow[d]), dot);
        s = dot * scale;
      }
    }
    const float cm = warp_max(s);
    const float m_new = fmaxf(m, cm);
    // a chunk whose pages were all refused leaves m_new at -inf: skip it
    if (m_new == -INFINITY) continue;
    const float pj = (s == -INFINITY) ? 0.f : expf(s - m_new);
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(pj);
#pragma unroll
    for (int i = 0; i < AS_MAX_D / 32; ++i) acc[i] *= corr;
    const int cnt = (p - j0 + 1) < 32 ? (p - j0 + 1) : 32;
    for (int jj = 0; jj < cnt; ++jj) {
      const float pv = __shfl_sync(0xffffffffu, pj, jj);
      const long long vo = __shfl_sync(0xffffffffu, voff, jj);
      if (vo < 0) continue;
      const T* vrow = pool + vo;
#pragma unroll
      for (int i = 0; i < AS_MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) acc[i] = fmaf(pv, to_f(vrow[d]), acc[i]);
      }
    }
    m = m_new;
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int i = 0; i < AS_MAX_D / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < D) orow[d] = from_f<T>(acc[i] * inv);
  }
}

}  // namespace hs

static int check_geom(const hs::AttnGeom& g) {
  if (g.head_dim <= 0 || g.head_dim % 16 || g.head_dim > hs::AS_MAX_D) return HS_ERR_UNSUPPORTED;
  if (g.n_heads <= 0 || g.n_kv_heads <= 0 || g.n_heads % g.n_kv_heads) return HS_ERR_UNSUPPORTED;
  if (g.page_size <= 0 || g.num_pages <= 0 || g.max_pages <= 0) return HS_ERR_ARGUMENT;
  if (g.window < 0) return HS_ERR_ARGUMENT;
  return HS_OK;
}

HS_EXPORT int hs_kv_append(void* pool, const void* qkv, const int* table, const int* tok_pos,
                           const int* tok_req, int n_tokens, int n_heads, int n_kv_heads,
                           int head_dim, int page_size, int num_pages, int max_pages, int q_off,
                           int k_off, int v_off, int qkv_stride, int dtype, int* status,
                           void* stream) {
  if (!pool || !qkv || !table || !tok_pos || !tok_req || !status) return HS_ERR_ARGUMENT;
  hs::AttnGeom g{n_heads, n_kv_heads, head_dim, page_size, num_pages, max_pages,
                 q_off,   k_off,      v_off,    qkv_stride, 0};
  if (int e = check_geom(g)) return e;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  int threads = n_kv_heads * head_dim >= 1024 ? 128 : 64;
  cudaError_t le;
  if (dtype == HS_DT_F32)
    le = hs_launch(hs::kv_append_kernel<float>, dim3(n_tokens), dim3(threads), 0, st,
                   hs_pdl_enabled(), (float*)pool, (const float*)qkv, table, tok_pos, tok_req, g,
                   status);
  else if (dtype == HS_DT_BF16)
    le = hs_launch(hs::kv_append_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, st,
                   hs_pdl_enabled(), (__nv_bfloat16*)pool, (const __nv_bfloat16*)qkv, table,
                   tok_pos, tok_req, g, status);
  else
    return HS_ERR_UNSUPPORTED;
  if (le != cudaSuccess) return (int)le;
  HS_LAUNCH_CHECK();
  return HS_OK;
}

HS_EXPORT int hs_attention_simt(void* out, const void* qkv, const void* pool, const int* table,
                                const int* tok_pos, const int* tok_req, int n_tokens, int n_heads,
                                int n_kv_heads, int head_dim, int page_size, int num_pages,
                                int max_pages, int q_off, int k_off, int v_off, int qkv_stride,
                                int window, float scale, int dtype, int* status, void* stream) {
  if (!out || !pool || !qkv || !table || !tok_pos || !tok_req || !status) return HS_ERR_ARGUMENT;
  hs::AttnGeom g{n_heads, n_kv_heads, head_dim, page_size, num_pages, max_pages,
                 q_off,   k_off,      v_off,    qkv_stride, window};
  if (int e = check_geom(g)) return e;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(n_tokens, (n_heads + hs::AS_WARPS - 1) / hs::AS_WARPS);
  size_t smem = (size_t)hs::AS_WARPS * head_dim * sizeof(float);
  if (dtype == HS_DT_F32)
    hs::attention_simt_kernel<float><<<grid, hs::AS_WARPS * 32, smem, st>>>(
        (float*)out, (const float*)qkv, (const float*)pool, table, tok_pos, tok_req, g, scale,
        status);
  else if (dtype == HS_DT_BF16)
    hs::attention_simt_kernel<__nv_bfloat16><<<grid, hs::AS_WARPS * 32, smem, st>>>(
        (__nv_bfloat16*)out, (const __nv_bfloat16*)qkv, (const __nv_bfloat16*)pool, table,
        tok_pos, tok_req, g, scale, status);
  else
    return HS_ERR_UNSUPPORTED;
  HS_LAUNCH_CHECK();
  return HS_OK;
}
