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
// attention_simt_kernel: one CTA of four warps per (token, head).  Keys are taken 32 at a time
// in position order, one key per lane; chunk c of a token's keys belongs to stream c mod 4, and
// warp s walks stream s with an online softmax (running maximum, running sum and output
// accumulators in float32, as heteroserve/model/paged_attn_v2.py:124-156); the four streams are
// then folded in stream order.  scores = (q . k) * scale with the multiply after the dot
// product (torch_engine.py:135).  The order of every sum depends only on the key positions,
// never on the batch, the cut of the prompt or the pages.
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

constexpr int AS_MAX_D = 256;
constexpr int AS_CHUNK = 32;          // keys per step: one per lane

__device__ __forceinline__ void as_copy16(void* smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void as_copies_done() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
// dot += q[e..] . k[e..] over the elements of one 16-byte piece, in index order
__device__ __forceinline__ float as_dot_piece(const float* q, uint4 raw, float dot, float) {
  dot = fmaf(q[0], __uint_as_float(raw.x), dot);
  dot = fmaf(q[1], __uint_as_float(raw.y), dot);
  dot = fmaf(q[2], __uint_as_float(raw.z), dot);
  return fmaf(q[3], __uint_as_float(raw.w), dot);
}
__device__ __forceinline__ float as_dot_piece(const float* q, uint4 raw, float dot, __nv_bfloat16) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    dot = fmaf(q[2 * i], __uint_as_float(w[i] << 16), dot);
    dot = fmaf(q[2 * i + 1], __uint_as_float(w[i] & 0xffff0000u), dot);
  }
  return dot;
}

constexpr int AS_STREAMS = 4;         // warps per CTA; chunk c of a token belongs to stream c % 4

// A step of 32 keys: every lane looks up its own key's page; the warp copies the 32 key rows
// and the 32 value rows into its shared memory with 16-byte cp.async copies (all in flight
// together: with a lane reading its key's row straight from the pool, and the value rows
// fetched one after the other behind a shuffle, a step was 32 dependent trips to the L2),
// 16-byte pieces swizzled by the key's index so that lane-per-key reads are free of bank
// conflicts; then lane j forms key j's score as one chain of fused multiply-adds over
// d = 0..D-1, the chunk joins the stream's running softmax, and lane d accumulates the values
// of dimension d, d+32, ... key by key.  `both` false (large heads): keys and values take
// turns in one buffer.
//
// G > 1 (prompt portions): a CTA serves G tokens.  When they are consecutive positions of one
// request (and there is no window) a staged chunk serves all of them, each with its own mask,
// running softmax and accumulators - the arithmetic of a token is the same as alone, so its
// result does not depend on its company; otherwise the CTA takes its tokens one after the other.
template <typename T, int G>
__global__ void __launch_bounds__(AS_STREAMS * 32)
attention_simt_kernel(T* __restrict__ out, const T* __restrict__ qkv, const T* __restrict__ pool,
                      const int* __restrict__ table, const int* __restrict__ tok_pos,
                      const int* __restrict__ tok_req, int n_tokens, AttnGeom g, float scale,
                      int both, int* status) {
  extern __shared__ __align__(16) uint8_t as_smem[];
  constexpr int VEC = 16 / (int)sizeof(T);             // elements per 16-byte piece
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  const int D = g.head_dim;
  const int pieces = D / VEC;                          // 16-byte pieces per row: 2 .. 64
  // pieces are permuted inside groups of 8, or of the largest power of two that divides a row
  int swz = 8;
  while (pieces % swz) swz >>= 1;
  swz -= 1;
  // this warp's shared memory: G queries as float [G][D] | keys [32][D] T | values (if `both`)
  const size_t rows_bytes = (size_t)AS_CHUNK * D * sizeof(T);
  const size_t q_bytes = (size_t)G * D * sizeof(float);
  const size_t per_warp = q_bytes + (both ? 2 : 1) * rows_bytes;
  uint8_t* base = as_smem + (size_t)warp * per_warp;
  float* sq = (float*)base;
  T* sk = (T*)(base + q_bytes);
  T* sv = both ? sk + (size_t)AS_CHUNK * D : sk;
  const int hk = h / (g.n_heads / g.n_kv_heads);
  const size_t tile = (size_t)g.page_size * D;
  const size_t page_stride = 2 * (size_t)g.n_kv_heads * tile;
  const long long v_off = (long long)g.n_kv_heads * (long long)tile;
  // piece i = lane + 32 * trip of a chunk: key i / pieces, piece i % pieces of its row
  const int key0 = lane / pieces, pc0 = lane - key0 * pieces;
  const int dkey = 32 / pieces, dpc = 32 - dkey * pieces;

  // the CTA's tokens: one run of consecutive positions of a request, or one by one
  const int t_first = blockIdx.x * G;
  const int n_here = min(G, n_tokens - t_first);
  bool run = G > 1 && n_here > 1 && g.window == 0;
  if (run) {
    const int r0 = tok_req[t_first], p0 = tok_pos[t_first];
    run = r0 >= 0 && p0 >= 0;
    for (int i = 1; i < n_here && run; ++i)
      run = tok_req[t_first + i] == r0 && tok_pos[t_first + i] == p0 + i;
  }
  const int n_groups = run ? 1 : n_here;                // groups of n_q tokens each
  const int n_q = run ? n_here : 1;

  for (int grp = 0; grp < n_groups; ++grp) {
    const int t0 = t_first + grp * n_q;
    const int r = tok_req[t0];
    const int p0 = tok_pos[t0];
    const int p_last = p0 + n_q - 1;
    if (grp > 0) __syncthreads();                      // the group before is done with shared memory
    if (r < 0 || p0 < 0 || p_last / g.page_size >= g.max_pages) {   // the same for the whole CTA
      for (int i = 0; i < n_q; ++i) {
        T* orow = out + (size_t)(t0 + i) * g.n_heads * D + (size_t)h * D;
        for (int d = threadIdx.x; d < D; d += blockDim.x) orow[d] = from_f<T>(0.f);
      }
      continue;
    }
    for (int i = 0; i < n_q; ++i) {
      const T* qrow = qkv + (size_t)(t0 + i) * g.qkv_stride + g.q_off + (size_t)h * D;
      for (int d = lane; d < D; d += 32) sq[i * D + d] = to_f(qrow[d]);
    }
    const int* trow = table + (size_t)r * g.max_pages;
    const int lo = (g.window > 0 && p0 - g.window + 1 > 0) ? p0 - g.window + 1 : 0;   // n_q == 1

    float m[G], l[G];
    float acc[G][AS_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < G; ++i) {
      m[i] = -INFINITY;
      l[i] = 0.f;
#pragma unroll
      for (int c = 0; c < AS_MAX_D / 32; ++c) acc[i][c] = 0.f;
    }

    for (int j0 = lo + warp * AS_CHUNK; j0 <= p_last; j0 += AS_STREAMS * AS_CHUNK) {
      const int j = j0 + lane;
      long long koff = -1;                               // this lane's key row in the pool
      if (j <= p_last) {
        const int page = trow[j / g.page_size];
        if (page < 0 || page >= g.num_pages)
          atomicOr(status, HS_STATUS_BAD_PAGE);
        else
          koff = (long long)((size_t)page * page_stride + (size_t)hk * tile +
                             (size_t)(j % g.page_size) * D);
      }
      const int cnt = (p_last - j0 + 1) < AS_CHUNK ? (p_last - j0 + 1) : AS_CHUNK;
      const unsigned live = __ballot_sync(0xffffffffu, koff >= 0);
      __syncwarp();                                      // the step before is done with sk / sv
      auto stage = [&](T* dst_rows, long long extra) {
        int key = key0, pc = pc0;
        for (int i0 = 0; i0 < cnt * pieces; i0 += 32) {  // the same trips for every lane
          const long long ko = __shfl_sync(0xffffffffu, koff, key & 31);
          if (key < cnt && ko >= 0)
            as_copy16(dst_rows + key * D + ((pc & ~swz) | ((pc ^ key) & swz)) * VEC,
                      pool + ko + extra + pc * VEC);
          key += dkey;
          pc += dpc;
          if (pc >= pieces) { pc -= pieces; ++key; }
        }
      };
      stage(sk, 0);
      if (both) stage(sv, v_off);
      as_copies_done();
      __syncwarp();
      if constexpr (G == 1) {
        // one query: score, running softmax, values (the loops of the grouped form below cost
        // a lone query half as much again)
        float s1 = -INFINITY;
        if (koff >= 0) {
          float dot = 0.f;
          const uint4* krow = (const uint4*)(sk + (size_t)lane * D);
          for (int pc = 0; pc < pieces; ++pc)
            dot = as_dot_piece(sq + pc * VEC, krow[(pc & ~swz) | ((pc ^ lane) & swz)], dot, T());
          s1 = dot * scale;
        }
        if (!both) {                                     // the values take the keys' place
          __syncwarp();
          stage(sv, v_off);
          as_copies_done();
          __syncwarp();
        }
        const float cm = warp_max(s1);
        const float m_new = fmaxf(m[0], cm);
        // a chunk whose pages were all refused leaves m_new at -inf: skip it
        if (m_new == -INFINITY) continue;
        const float pj1 = (s1 == -INFINITY) ? 0.f : expf(s1 - m_new);
        const float corr = expf(m[0] - m_new);
        l[0] = l[0] * corr + warp_sum(pj1);
#pragma unroll
        for (int c = 0; c < AS_MAX_D / 32; ++c) acc[0][c] *= corr;
        for (int jj = 0; jj < cnt; ++jj) {
          const float pv = __shfl_sync(0xffffffffu, pj1, jj);
          if (!((live >> jj) & 1u)) continue;
          const T* vrow = sv + (size_t)jj * D;
#pragma unroll
          for (int c = 0; c < AS_MAX_D / 32; ++c) {
            const int d = lane + 32 * c;
            if (d < D) {
              const int pc = d / VEC;
              acc[0][c] = fmaf(pv, to_f(vrow[((pc & ~swz) | ((pc ^ jj) & swz)) * VEC + (d - pc * VEC)]),
                               acc[0][c]);
            }
          }
        }
        m[0] = m_new;
      } else {
      // scores of the chunk's key `lane` for every query of the group: the queries' chains of
      // fused multiply-adds run side by side on one read of the key's pieces
      float s[G];
      bool sees[G];
#pragma unroll
      for (int i = 0; i < G; ++i) {
        sees[i] = i < n_q && koff >= 0 && j <= p0 + i;     // key j is visible to query i
        s[i] = 0.f;
      }
      if (koff >= 0) {
        const uint4* krow = (const uint4*)(sk + (size_t)lane * D);
        for (int pc = 0; pc < pieces; ++pc) {
          const uint4 kp = krow[(pc & ~swz) | ((pc ^ lane) & swz)];
#pragma unroll
          for (int i = 0; i < G; ++i)
            if (i < n_q) s[i] = as_dot_piece(sq + i * D + pc * VEC, kp, s[i], T());
        }
      }
#pragma unroll
      for (int i = 0; i < G; ++i) s[i] = sees[i] ? s[i] * scale : -INFINITY;
      if (!both) {                                       // the values take the keys' place
        __syncwarp();
        stage(sv, v_off);
        as_copies_done();
        __syncwarp();
      }
      // each query's running softmax takes the chunk in; then the values, read once per key,
      // go into every query that sees the key
      float pj[G];
      int cnt_q[G];
#pragma unroll
      for (int i = 0; i < G; ++i) {
        pj[i] = 0.f;
        cnt_q[i] = 0;
        if (i >= n_q || j0 > p0 + i) continue;           // (the same for the whole warp)
        const float cm = warp_max(s[i]);
        const float m_new = fmaxf(m[i], cm);
        // a chunk whose pages were all refused leaves m_new at -inf: skip it
        if (m_new == -INFINITY) continue;
        pj[i] = (s[i] == -INFINITY) ? 0.f : expf(s[i] - m_new);
        const float corr = expf(m[i] - m_new);
        l[i] = l[i] * corr + warp_sum(pj[i]);
#pragma unroll
        for (int c = 0; c < AS_MAX_D / 32; ++c) acc[i][c] *= corr;
        cnt_q[i] = (p0 + i - j0 + 1) < AS_CHUNK ? (p0 + i - j0 + 1) : AS_CHUNK;
        m[i] = m_new;
      }
      for (int jj = 0; jj < cnt; ++jj) {
        float pv[G];
#pragma unroll
        for (int i = 0; i < G; ++i) pv[i] = __shfl_sync(0xffffffffu, pj[i], jj);
        if (!((live >> jj) & 1u)) continue;
        const T* vrow = sv + (size_t)jj * D;
#pragma unroll
        for (int c = 0; c < AS_MAX_D / 32; ++c) {
          const int d = lane + 32 * c;
          if (d < D) {
            const int pc = d / VEC;
            const float v = to_f(vrow[((pc & ~swz) | ((pc ^ jj) & swz)) * VEC + (d - pc * VEC)]);
#pragma unroll
            for (int i = 0; i < G; ++i)
              if (jj < cnt_q[i]) acc[i][c] = fmaf(pv[i], v, acc[i][c]);
          }
        }
      }
      }
    }

    // fold the streams in stream order: each warp leaves (m, l, acc) of every query in its own
    // shared memory (the key rows' place: 32 rows of D against G x (2 + D) floats)
    __syncwarp();
    float* st = (float*)(base + q_bytes);
#pragma unroll
    for (int i = 0; i < G; ++i) {
      if (i >= n_q) continue;
      float* sti = st + (size_t)i * (2 + D);
      if (lane == 0) { sti[0] = m[i]; sti[1] = l[i]; }
#pragma unroll
      for (int c = 0; c < AS_MAX_D / 32; ++c) {
        const int d = lane + 32 * c;
        if (d < D) sti[2 + d] = acc[i][c];
      }
    }
    __syncthreads();
    // warp w folds query w, w + 4, ...
    for (int i = warp; i < n_q; i += AS_STREAMS) {
      float M = -INFINITY, L = 0.f;
      float o[AS_MAX_D / 32];
#pragma unroll
      for (int c = 0; c < AS_MAX_D / 32; ++c) o[c] = 0.f;
      for (int sidx = 0; sidx < AS_STREAMS; ++sidx) {
        const float* ss = (const float*)(as_smem + (size_t)sidx * per_warp + q_bytes) +
                          (size_t)i * (2 + D);
        const float ms = ss[0];
        if (ms == -INFINITY) continue;                   // a stream without keys
        const float m_new = fmaxf(M, ms);
        const float c0 = expf(M - m_new), c1 = expf(ms - m_new);
        L = L * c0 + ss[1] * c1;
#pragma unroll
        for (int c = 0; c < AS_MAX_D / 32; ++c) {
          const int d = lane + 32 * c;
          if (d < D) o[c] = fmaf(ss[2 + d], c1, o[c] * c0);
        }
        M = m_new;
      }
      const float inv = L > 0.f ? 1.0f / L : 0.f;
      T* orow = out + (size_t)(t0 + i) * g.n_heads * D + (size_t)h * D;
#pragma unroll
      for (int c = 0; c < AS_MAX_D / 32; ++c) {
        const int d = lane + 32 * c;
        if (d < D) orow[d] = from_f<T>(o[c] * inv);
      }
    }
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

// group: tokens per CTA (1, or 4 for steps of prompt portions, where neighbours in the batch
// are consecutive positions of one request and share the staged keys).
template <typename T, int G>
static int launch_attention_simt(void* out, const void* qkv, const void* pool, const int* table,
                                 const int* tok_pos, const int* tok_req, int n_tokens,
                                 const hs::AttnGeom& g, float scale, size_t esz, int* status,
                                 cudaStream_t st) {
  // keys and values side by side in shared memory while four warps of them fit in 160 KB
  const size_t rows_bytes = (size_t)hs::AS_CHUNK * g.head_dim * esz;
  const size_t q_bytes = (size_t)G * g.head_dim * 4;
  const int both = hs::AS_STREAMS * (q_bytes + 2 * rows_bytes) <= 160 * 1024 ? 1 : 0;
  const size_t smem = hs::AS_STREAMS * (q_bytes + (both ? 2 : 1) * rows_bytes);
  dim3 grid((n_tokens + G - 1) / G, g.n_heads);
  auto* k = hs::attention_simt_kernel<T, G>;
  static cudaError_t state = cudaErrorUnknown;
  if (state != cudaSuccess)
    state = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 164 * 1024);
  if (state != cudaSuccess) return (int)state;
  k<<<grid, hs::AS_STREAMS * 32, smem, st>>>((T*)out, (const T*)qkv, (const T*)pool, table,
                                              tok_pos, tok_req, n_tokens, g, scale, both, status);
  HS_LAUNCH_CHECK();
  return HS_OK;
}

HS_EXPORT int hs_attention_simt_grouped(void* out, const void* qkv, const void* pool,
                                        const int* table, const int* tok_pos, const int* tok_req,
                                        int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                        int page_size, int num_pages, int max_pages, int q_off,
                                        int k_off, int v_off, int qkv_stride, int window,
                                        float scale, int dtype, int group, int* status,
                                        void* stream) {
  if (!out || !pool || !qkv || !table || !tok_pos || !tok_req || !status) return HS_ERR_ARGUMENT;
  hs::AttnGeom g{n_heads, n_kv_heads, head_dim, page_size, num_pages, max_pages,
                 q_off,   k_off,      v_off,    qkv_stride, window};
  if (int e = check_geom(g)) return e;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if ((uintptr_t)pool & 15) return HS_ERR_UNSUPPORTED;   // rows are copied 16 bytes at a time
  if (n_heads > 65535) return HS_ERR_UNSUPPORTED;
  if (group != 1 && group != 4) return HS_ERR_ARGUMENT;
  using bf16 = __nv_bfloat16;
  if (dtype == HS_DT_F32)
    return group == 4 ? launch_attention_simt<float, 4>(out, qkv, pool, table, tok_pos, tok_req,
                                                         n_tokens, g, scale, 4, status, st)
                      : launch_attention_simt<float, 1>(out, qkv, pool, table, tok_pos, tok_req,
                                                         n_tokens, g, scale, 4, status, st);
  if (dtype == HS_DT_BF16)
    return group == 4 ? launch_attention_simt<bf16, 4>(out, qkv, pool, table, tok_pos, tok_req,
                                                        n_tokens, g, scale, 2, status, st)
                      : launch_attention_simt<bf16, 1>(out, qkv, pool, table, tok_pos, tok_req,
                                                        n_tokens, g, scale, 2, status, st);
  return HS_ERR_UNSUPPORTED;
}

HS_EXPORT int hs_attention_simt(void* out, const void* qkv, const void* pool, const int* table,
                                const int* tok_pos, const int* tok_req, int n_tokens, int n_heads,
                                int n_kv_heads, int head_dim, int page_size, int num_pages,
                                int max_pages, int q_off, int k_off, int v_off, int qkv_stride,
                                int window, float scale, int dtype, int* status, void* stream) {
  return hs_attention_simt_grouped(out, qkv, pool, table, tok_pos, tok_req, n_tokens, n_heads,
                                   n_kv_heads, head_dim, page_size, num_pages, max_pages, q_off,
                                   k_off, v_off, qkv_stride, window, scale, dtype, 1, status,
                                   stream);
}
