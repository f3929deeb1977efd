// Split-context paged attention for tokens that bring one query each (decoding), bfloat16.
//
// The successor of the reference's split-K decode kernels (heteroserve/model/paged_attn_v3.py:
// split kernel :75-165, merge kernel :170-208, split heuristic :212-232): the keys 0..p of a
// query are cut into `splits` slices; one CTA streams one slice of one (token, head) with an
// online softmax in float32 (running maximum m, running sum l, un-normalised accumulator),
// writes its partial (acc, m, l) to scratch memory, and the LAST CTA of a (token, head) to
// finish — found with a counter in scratch — merges the partials in slice order:
//     m_g = max_s m_s;  l_g = sum_s l_s * exp(m_s - m_g);  out = sum_s acc_s * exp(m_s - m_g) / l_g
// (paged_attn_v3.py:170-208), so no second launch is needed.  The slice length is read from
// device memory (the batch's longest context / splits, rounded up to whole pages), which keeps a
// captured CUDA graph valid while contexts grow.
//
// Inside a CTA each warp takes every 4th page of the slice; the next group of keys is loaded
// while the current one is used.  A key row of D bfloat16 is read by
// D/8 adjacent lanes with one 16-byte load each, so a warp covers 256/D keys per load and the
// loads of a page (keys and values) are all in flight before the first is used.  Scores are
// (q . k) * scale with the multiply after the dot product (heteroserve/model/torch_engine.py:135).
//
// Scratch layout (float32 unless noted), T = token capacity, H = heads, S = splits:
//     acc  [T][H][S][D]      ml [T][H][S][2]      counters [T][H] (int32, zero between launches)
#include "common.cuh"
#include "no_alloc.h"

#include <mutex>

namespace hs {

constexpr int AD_WARPS = 4;          // warps per CTA of the narrow variant (the wide one has 16)

struct DecodeParams {
  const __nv_bfloat16* qkv;
  const __nv_bfloat16* pool;
  __nv_bfloat16* out;
  const int* table;
  const int* tok_pos;
  const int* tok_req;
  const int* dec_info;     // per served token: flat index, request row, position
  const int* plan_head;    // [0] = number of tokens in tok_list, [2] = longest context among them
  float* acc;
  float* ml;
  int* counters;
  int* status;
  int n_heads, n_kv_heads, page_size, num_pages, max_pages;
  int q_off, qkv_stride, splits, window;
  int k_off, v_off, fuse_append;   // fuse_append: take and store the token's own key/value
  float scale;
};

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <int D, int NW>
__global__ void __launch_bounds__(NW * 32)
attention_decode_kernel(const DecodeParams p) {
  constexpr int LPK = D / 8;          // lanes per key row
  constexpr int KPW = 32 / LPK;       // keys per warp-wide load
  static_assert(D == 16 || D == 32 || D == 64 || D == 128 || D == 256, "head size");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = blockIdx.x;                       // index into tok_list
  const int h = blockIdx.y, split = blockIdx.z;
  const int n_served = p.plan_head[0];
  const int t = p.dec_info[3 * slot], r = p.dec_info[3 * slot + 1], pos = p.dec_info[3 * slot + 2];
  if (slot >= n_served) return;
  __nv_bfloat16* orow = p.out + ((size_t)t * p.n_heads + h) * D;
  if (r < 0 || pos < 0 || pos / p.page_size >= p.max_pages) {
    if (split == 0)
      for (int d = threadIdx.x; d < D; d += blockDim.x) orow[d] = __float2bfloat16_rn(0.f);
    return;
  }
  const int hk = h / (p.n_heads / p.n_kv_heads);
  const int PS = p.page_size;
  const int lo_all = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
  // slice boundaries in whole pages, from the batch's longest context
  const int max_ctx = p.plan_head[2];
  int chunk = (max_ctx + p.splits - 1) / p.splits;
  chunk = (chunk + PS - 1) / PS * PS;
  const int k_begin = max(split * chunk, lo_all);
  // With the append fused in, the token's own key (position pos) is not in the pages yet: the
  // slice that contains pos takes it from the projection's output row and writes it to its page.
  const bool own_here = p.fuse_append && pos >= split * chunk && pos < (split + 1) * chunk;
  const int k_end = min((split + 1) * chunk, p.fuse_append ? pos : pos + 1);   // exclusive

  // the query, 8 elements per lane (the same 8 its key lanes read).  It is the first thing the
  // previous kernel wrote that this one needs: the work lists, the block table and the keys and
  // values of earlier positions are fetched before the dependency wait.
  const int part = lane % LPK, sub = lane / LPK;
  float q[8];
  auto wait_and_load_query = [&]() {
    pdl_trigger();
    pdl_wait();
    const uint4 qu = *(const uint4*)(p.qkv + (size_t)t * p.qkv_stride + p.q_off + (size_t)h * D +
                                     part * 8);
    unpack8(qu, q);
  };
  float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;

  const size_t tile = (size_t)PS * D;
  const size_t page_stride = 2 * (size_t)p.n_kv_heads * tile;
  const int* trow = p.table + (size_t)r * p.max_pages;

  if (k_begin < k_end) {
    const int pg_first = k_begin / PS, pg_last = (k_end - 1) / PS;
    // This warp's pages: pg_first + warp, + NW, ...  Their page numbers are fetched at
    // once, one per lane (the host keeps a slice within 32 pages per warp), so that no key
    // load waits for a table lookup.
    const int my_pg = pg_first + warp + NW * lane;
    const int my_page = my_pg <= pg_last ? trow[my_pg] : -1;
    const int n_pages = (pg_last - pg_first - warp + NW) / NW;   // may be <= 0
    constexpr int UNIT = 4 * KPW;                        // keys per unit of work
    const int upp = (PS + UNIT - 1) / UNIT;              // units per page
    const int n_units = n_pages > 0 ? n_pages * upp : 0;

    struct Unit {
      uint4 k[4], v[4];
      int j0;                                            // position of the unit's first key
      int g0;
    };
    auto load_unit = [&](int u, Unit& un) {
      const int it = u / upp;
      un.g0 = (u - it * upp) * UNIT;
      const int pg = pg_first + warp + NW * it;
      const int page = __shfl_sync(0xffffffffu, my_page, it & 31);
      un.j0 = pg * PS;
      const bool page_ok = page >= 0 && page < p.num_pages;
      if (!page_ok && lane == 0) atomicOr(p.status, HS_STATUS_BAD_PAGE);
      const __nv_bfloat16* kbase = p.pool + (size_t)(page_ok ? page : 0) * page_stride +
                                   (size_t)hk * tile;
      const __nv_bfloat16* vbase = kbase + (size_t)p.n_kv_heads * tile;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int sip = un.g0 + i * KPW + sub;
        const int j = un.j0 + sip;
        if (page_ok && sip < PS && j >= k_begin && j < k_end) {
          un.k[i] = *(const uint4*)(kbase + (size_t)sip * D + part * 8);
          un.v[i] = *(const uint4*)(vbase + (size_t)sip * D + part * 8);
        } else {
          un.k[i] = make_uint4(0, 0, 0, 0);
          un.v[i] = make_uint4(0, 0, 0, 0);
          if (!page_ok) un.j0 = -(1 << 30);              // every key of it fails the range test
        }
      }
    };
    Unit cur, nxt;
    // Keys and values of earlier positions were written by earlier steps, so with the append
    // fused in (nothing else writes this layer's pages during the step) the first group is
    // requested before the dependency wait.  Without fusion the previous kernel may be the one
    // that appends this step's keys: wait first.
    if (!p.fuse_append) wait_and_load_query();
    if (n_units > 0) load_unit(0, cur);
    if (n_units > 1) load_unit(1, nxt);
    if (p.fuse_append) wait_and_load_query();
    for (int u = 0; u < n_units; ++u) {
      float s[4];
      float bm = -INFINITY;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float kf[8];
        unpack8(cur.k[i], kf);
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) dot = fmaf(q[e], kf[e], dot);
#pragma unroll
        for (int o = 1; o < LPK; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const int sip = cur.g0 + i * KPW + sub;
        const int j = cur.j0 + sip;
        const bool valid = sip < PS && j >= k_begin && j < k_end;
        s[i] = valid ? dot * p.scale : -INFINITY;
        bm = fmaxf(bm, s[i]);
      }
      // maximum over the key groups of the warp (lanes with the same `part`)
#pragma unroll
      for (int o = LPK; o < 32; o <<= 1) bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, o));
      if (bm != -INFINITY) {
        const float m_new = fmaxf(m, bm);
        const float corr = __expf(m - m_new);
        l *= corr;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] *= corr;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float pr = (s[i] == -INFINITY) ? 0.f : __expf(s[i] - m_new);
          l += pr;
          float vf[8];
          unpack8(cur.v[i], vf);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = fmaf(pr, vf[e], acc[e]);
        }
        m = m_new;
      }
      cur = nxt;
      if (u + 2 < n_units) load_unit(u + 2, nxt);        // two groups ahead of the one in use
    }
  } else {
    wait_and_load_query();
  }
  if (own_here && warp == NW - 1) {
    // the new key and value: lanes of key group 0 hold 8 elements each
    const __nv_bfloat16* row = p.qkv + (size_t)t * p.qkv_stride;
    uint4 ku = make_uint4(0, 0, 0, 0), vu = make_uint4(0, 0, 0, 0);
    if (sub == 0) {
      ku = *(const uint4*)(row + p.k_off + (size_t)hk * D + part * 8);
      vu = *(const uint4*)(row + p.v_off + (size_t)hk * D + part * 8);
      if (h % (p.n_heads / p.n_kv_heads) == 0) {          // one writer per key/value head
        const int page = trow[pos / PS];
        if (page < 0 || page >= p.num_pages) {
          if (part == 0) atomicOr(p.status, HS_STATUS_BAD_PAGE);
        } else {
          __nv_bfloat16* kdst = const_cast<__nv_bfloat16*>(p.pool) + (size_t)page * page_stride +
                                (size_t)hk * tile + (size_t)(pos % PS) * D + part * 8;
          *(uint4*)kdst = ku;
          *(uint4*)(kdst + (size_t)p.n_kv_heads * tile) = vu;
        }
      }
    }
    float kf[8];
    unpack8(ku, kf);
    float dot = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) dot = fmaf(q[e], kf[e], dot);
#pragma unroll
    for (int o = 1; o < LPK; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float sc = __shfl_sync(0xffffffffu, dot, 0) * p.scale;      // group 0's score, to all
    const float m_new = fmaxf(m, sc);
    const float corr = __expf(m - m_new);
    const float pr = (sub == 0) ? __expf(sc - m_new) : 0.f;
    l = l * corr + pr;
    float vf[8];
    unpack8(vu, vf);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = fmaf(pr, vf[e], acc[e] * corr);
    m = m_new;
  }
  // ---- combine the key groups of a warp, then the warps of the CTA (all share m per warp)
  // every lane of a warp holds the same m; l and acc are per key group: sum over groups
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1) {
    l += __shfl_xor_sync(0xffffffffu, l, o);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], o);
  }
  // l was added once per lane of a key group: every lane of a group holds the same l, fine
  __shared__ float s_m[NW], s_l[NW], s_acc[NW][D];
  if (sub == 0) {
#pragma unroll
    for (int e = 0; e < 8; ++e) s_acc[warp][part * 8 + e] = acc[e];
  }
  if (lane == 0) {
    s_m[warp] = m;
    s_l[warp] = l;
  }
  __syncthreads();
  const size_t pidx = ((size_t)slot * p.n_heads + h) * p.splits + split;
  float* pacc = p.acc + pidx * D;
  float cm = -INFINITY;
#pragma unroll
  for (int w = 0; w < NW; ++w) cm = fmaxf(cm, s_m[w]);
  float cl = 0.f;
  float wscale[NW];
#pragma unroll
  for (int w = 0; w < NW; ++w) {
    wscale[w] = (s_m[w] == -INFINITY) ? 0.f : __expf(s_m[w] - cm);
    cl += s_l[w] * wscale[w];
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) a += s_acc[w][d] * wscale[w];
    if (p.splits == 1) {
      orow[d] = __float2bfloat16_rn(cl > 0.f ? a / cl : 0.f);
    } else {
      pacc[d] = a;
    }
  }
  if (p.splits == 1) return;
  if (threadIdx.x == 0) {
    p.ml[pidx * 2] = cm;
    p.ml[pidx * 2 + 1] = cl;
  }
  // ---- the last CTA of this (token, head) merges
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(&p.counters[slot * p.n_heads + h], 1);
    s_last = (done == p.splits - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const size_t base = ((size_t)slot * p.n_heads + h) * p.splits;
  float gm = -INFINITY;
  for (int s2 = 0; s2 < p.splits; ++s2) gm = fmaxf(gm, __ldcg(&p.ml[(base + s2) * 2]));
  float gl = 0.f;
  for (int s2 = 0; s2 < p.splits; ++s2) {
    const float ms = __ldcg(&p.ml[(base + s2) * 2]);
    if (ms != -INFINITY) gl += __ldcg(&p.ml[(base + s2) * 2 + 1]) * __expf(ms - gm);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f;
    for (int s2 = 0; s2 < p.splits; ++s2) {
      const float ms = __ldcg(&p.ml[(base + s2) * 2]);
      if (ms != -INFINITY) a += __ldcg(&p.acc[(base + s2) * D + d]) * __expf(ms - gm);
    }
    orow[d] = __float2bfloat16_rn(gl > 0.f ? a / gl : 0.f);
  }
  if (threadIdx.x == 0) p.counters[slot * p.n_heads + h] = 0;     // ready for the next launch
}

}  // namespace hs

// fuse_append != 0: every served token is the only new token of its request; its key and value
// (columns k_off / v_off of its row in `qkv`) are used from there and written to its page by the
// kernel, so no separate append pass is needed.  wide: 0 = 4 warps per CTA, 1 = 8, 2 = 16 (for
// batches whose token x head count alone does not fill the GPU).
HS_EXPORT int hs_attention_decode_append(void* out, const void* qkv, void* pool, const int* table,
                                         const int* tok_pos, const int* tok_req,
                                         const int* dec_info, const int* plan_head, int token_cap,
                                         int n_heads, int n_kv_heads, int head_dim, int page_size,
                                         int num_pages, int max_pages, int q_off, int k_off,
                                         int v_off, int qkv_stride, int window, float scale,
                                         int splits, int fuse_append, int wide, int pdl,
                                         float* scratch_acc, float* scratch_ml, int* counters,
                                         int* status, void* stream) {
  using namespace hs;
  if (!out || !qkv || !pool || !table || !tok_pos || !tok_req || !dec_info || !plan_head ||
      !status)
    return HS_ERR_ARGUMENT;
  if (token_cap <= 0) return HS_OK;
  if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return HS_ERR_UNSUPPORTED;
  if (page_size <= 0 || page_size % 16 || splits < 1 || splits > 65535) return HS_ERR_UNSUPPORTED;
  if (n_heads > 65535) return HS_ERR_UNSUPPORTED;
  if (splits > 1 && (!scratch_acc || !scratch_ml || !counters)) return HS_ERR_ARGUMENT;
  if ((qkv_stride % 8) || (q_off % 8) || (k_off % 8) || (v_off % 8))
    return HS_ERR_UNSUPPORTED;   // 16-byte loads of the query, key and value rows
  const int nw = wide == 2 ? 16 : (wide == 1 ? 8 : AD_WARPS);
  // a slice may span at most 32 pages per warp
  if ((long long)splits * 32 * nw < max_pages) return HS_ERR_UNSUPPORTED;
  DecodeParams p;
  p.qkv = (const __nv_bfloat16*)qkv;
  p.pool = (const __nv_bfloat16*)pool;
  p.out = (__nv_bfloat16*)out;
  p.table = table; p.tok_pos = tok_pos; p.tok_req = tok_req; p.dec_info = dec_info;
  p.plan_head = plan_head; p.acc = scratch_acc; p.ml = scratch_ml; p.counters = counters;
  p.status = status;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
  p.num_pages = num_pages; p.max_pages = max_pages; p.q_off = q_off; p.qkv_stride = qkv_stride;
  p.splits = splits; p.window = window; p.scale = scale;
  p.k_off = k_off; p.v_off = v_off; p.fuse_append = fuse_append;
  dim3 grid(token_cap, n_heads, splits);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t le = cudaSuccess;
#define HS_AD(DD)                                                                             \
  if (wide == 2) le = hs_launch(attention_decode_kernel<DD, 16>, grid, dim3(16 * 32), 0, st, pdl != 0, p); \
  else if (wide == 1) le = hs_launch(attention_decode_kernel<DD, 8>, grid, dim3(8 * 32), 0, st, pdl != 0, p); \
  else le = hs_launch(attention_decode_kernel<DD, AD_WARPS>, grid, dim3(AD_WARPS * 32), 0, st, pdl != 0, p)
  switch (head_dim) {
    case 16: HS_AD(16); break;
    case 32: HS_AD(32); break;
    case 64: HS_AD(64); break;
    case 128: HS_AD(128); break;
    case 256: HS_AD(256); break;
    default: return HS_ERR_UNSUPPORTED;
  }
#undef HS_AD
  if (le != cudaSuccess) return (int)le;
  HS_LAUNCH_CHECK();
  return HS_OK;
}

// Bytes of scratch one launch needs (acc + ml + counters), for a token capacity.
HS_EXPORT long long hs_attention_decode_scratch_floats(int token_cap, int n_heads, int head_dim,
                                                       int splits) {
  return (long long)token_cap * n_heads * splits * (head_dim + 2);
}

HS_EXPORT int hs_attention_decode(void* out, const void* qkv, const void* pool, const int* table,
                                  const int* tok_pos, const int* tok_req, const int* dec_info,
                                  const int* plan_head, int token_cap, int n_heads,
                                  int n_kv_heads, int head_dim, int page_size, int num_pages,
                                  int max_pages, int q_off, int qkv_stride, int window,
                                  float scale, int splits, float* scratch_acc, float* scratch_ml,
                                  int* counters, int* status, void* stream) {
  return hs_attention_decode_append(out, qkv, const_cast<void*>(pool), table, tok_pos, tok_req, dec_info, plan_head,
                                    token_cap, n_heads, n_kv_heads, head_dim, page_size,
                                    num_pages, max_pages, q_off, 0, 0, qkv_stride, window, scale,
                                    splits, 0, 0, 0, scratch_acc, scratch_ml, counters, status,
                                    stream);
}

// ------------------------------------------------------------------------------------------
// The same kernel for callers that must not allocate (declared in no_alloc.h).
//
// The partial sums, their (max, sum) pairs and the arrival counters live in one file-scope
// device array instead of caller-provided scratch.  Host code cannot use the array's name as
// an address (on the host it is only a stand-in for the symbol), so the device address is
// looked up with cudaGetSymbolAddress once per device, with that device current, and kept.
namespace hs {

static __device__ __align__(256) float noalloc_scratch[HS_NOALLOC_SCRATCH_FLOATS];

static std::mutex noalloc_mutex;
static float* noalloc_address[HS_NOALLOC_MAX_DEVICES];     // per device, null until looked up

// Device address of the static scratch on the current device (first call per device does the
// look-up; it is not a stream operation and should not happen inside a stream capture).
static int noalloc_scratch_address(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= HS_NOALLOC_MAX_DEVICES) return HS_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(noalloc_mutex);
  if (noalloc_address[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (ptr == nullptr) return HS_ERR_ARGUMENT;
    noalloc_address[dev] = ptr;
  }
  *out = noalloc_address[dev];
  return HS_OK;
}

}  // namespace hs

HS_EXPORT long long hs_attention_decode_noalloc_capacity(void) {
  return (long long)HS_NOALLOC_SCRATCH_FLOATS;
}

HS_EXPORT int hs_attention_decode_noalloc(void* out, const void* qkv, const void* pool,
                                          const int* table, const int* tok_pos,
                                          const int* tok_req, const int* dec_info,
                                          const int* plan_head, int token_cap, int n_heads,
                                          int n_kv_heads, int head_dim, int page_size,
                                          int num_pages, int max_pages, int q_off, int qkv_stride,
                                          int window, float scale, int splits, int* status,
                                          void* stream) {
  using namespace hs;
  if (token_cap <= 0) return HS_OK;
  if (splits < 1 || n_heads <= 0 || head_dim <= 0) return HS_ERR_ARGUMENT;
  if (splits == 1)      // one slice per (token, head): the kernel touches no scratch at all
    return hs_attention_decode(out, qkv, pool, table, tok_pos, tok_req, dec_info, plan_head,
                               token_cap, n_heads, n_kv_heads, head_dim, page_size, num_pages,
                               max_pages, q_off, qkv_stride, window, scale, 1, nullptr, nullptr,
                               nullptr, status, stream);
  // layout inside the static array: acc [rows][D] | ml [rows][2] | counters [token_cap * heads]
  const long long rows = (long long)token_cap * n_heads * splits;
  const long long pairs = (long long)token_cap * n_heads;
  const long long need = rows * head_dim + rows * 2 + pairs;
  if (need > (long long)HS_NOALLOC_SCRATCH_FLOATS) return HS_ERR_TOO_LARGE;
  float* base = nullptr;
  if (int e = noalloc_scratch_address(&base)) return e;
  float* acc = base;
  float* ml = acc + rows * head_dim;
  int* counters = (int*)(ml + rows * 2);
  // The array keeps whatever the last call (or an aborted one) left.  Only the counters must
  // start at zero; partial sums are fully written before they are read.
  cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)pairs * sizeof(int), (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return hs_attention_decode(out, qkv, pool, table, tok_pos, tok_req, dec_info, plan_head,
                             token_cap, n_heads, n_kv_heads, head_dim, page_size, num_pages,
                             max_pages, q_off, qkv_stride, window, scale, splits, acc, ml, counters,
                             status, stream);
}
