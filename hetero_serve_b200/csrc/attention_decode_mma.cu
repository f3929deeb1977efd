// Paged attention for single-query tokens on the tensor cores (mma.sync), bfloat16: the decode
// kernel for head sizes 32, 64 and 128 at every batch size.
//
// Same work as attention_decode.cu (the successor of the reference's split-K decode kernels,
// heteroserve/model/paged_attn_v3.py:75-232), arranged for streaming:
//   * one CTA serves one (token, key/value head, slice): the G = n_heads / n_kv_heads query
//     heads that share those keys are the rows of one 16-row MMA tile (GPT-2 has G = 1; the
//     other rows are zero), so grouped heads read their keys once;
//   * each of the NW (4 or 8) warps takes every NW-th chunk of 32 keys and owns a ring of chunk
//     buffers in shared memory, filled by cp.async 16 bytes at a time through the block table
//     (a chunk is two 16-position blocks, each inside one page) and never touched by another
//     warp: no block-wide barrier in the loop, one to three chunks in flight per warp;
//   * S = Q K^T and O += P V are mma.sync m16n8k16 (bf16 in, float32 accumulate) on fragments
//     fetched with ldmatrix from XOR-swizzled tiles; scores are multiplied by the scale after
//     the dot product (heteroserve/model/torch_engine.py:135); running maximum, sum and O are
//     float32;
//   * chunks of earlier positions are requested before the dependency wait; the chunk that
//     holds the token's own position comes after it, and with the append fused in its row is
//     copied from the projection's output row (and stored to the page by warp 0);
//   * the warps' partial (m, l, O) are merged through the ring memory; with slices the CTA
//     writes its partial to scratch and the last CTA of the (token, head) merges them in slice
//     order, exactly as in attention_decode.cu (same scratch layout).
// A bandwidth kernel: per 32 keys a warp issues about 150 instructions instead of the 450 of
// the CUDA-core loop, and 8-24 KB per warp are in flight without holding registers.
#include "common.cuh"

namespace hs {

constexpr int DM_WARPS = 4;             // fewest warps per CTA (the launcher picks 4 or 8)
constexpr int DM_CHUNK = 32;            // keys per chunk

struct DecodeMmaParams {
  const __nv_bfloat16* qkv;
  const __nv_bfloat16* pool;
  __nv_bfloat16* out;
  const int* table;
  const int* dec_info;     // per served token: flat index, request row, position
  const int* plan_head;    // [0] = number of served tokens, [2] = longest context among them
  float* acc;              // [tokens][heads][splits][D]
  float* ml;               // [tokens][heads][splits][2]
  int* counters;           // [tokens][heads], zero between launches
  int* status;
  int n_heads, n_kv_heads, page_size, num_pages, max_pages;
  int q_off, k_off, v_off, qkv_stride, splits, fuse_append;
  float scale;
};

template <int D>
__device__ __forceinline__ int dm_swz(int row, int chunk) {
  constexpr int CPR = D / 8;                       // 16-byte pieces per row
  constexpr int RPL = CPR >= 8 ? 1 : 8 / CPR;      // rows per 128-byte line
  constexpr int MASK = (CPR >= 8 ? 8 : CPR) - 1;
  return row * CPR + (chunk ^ ((row / RPL) & MASK));
}
__device__ __forceinline__ void dm_cp16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void dm_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void dm_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void dm_ldsm(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void dm_ldsm_t(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void dm_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float dm_ex2(float x) {      // 2^x, hardware approximation; -inf -> 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t dm_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}

template <int D, int STAGES_, int NW_ = DM_WARPS>
struct DmShape {
  static constexpr int CPR = D / 8;
  static constexpr int STAGES = STAGES_;
  static constexpr int CHUNK_PIECES = DM_CHUNK * CPR;            // uint4 per chunk of keys
  static constexpr int WARP_PIECES = STAGES * 2 * CHUNK_PIECES;  // keys and values
  static constexpr size_t SMEM = (size_t)NW_ * WARP_PIECES * 16;
};

template <int D, int STAGES_, int NW>
__global__ void __launch_bounds__(NW * 32)
attention_decode_mma_kernel(const DecodeMmaParams p) {
  using SH = DmShape<D, STAGES_, NW>;
  constexpr int CPR = SH::CPR, STAGES = SH::STAGES;
  constexpr int KSTEPS = D / 16;       // k-steps of Q K^T
  constexpr int DT = D / 8;            // 8-wide tiles of the output
  extern __shared__ __align__(128) uint8_t dm_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  uint4* ring = (uint4*)dm_smem + (size_t)warp * SH::WARP_PIECES;

  pdl_trigger();
  const int slot = blockIdx.x, hk = blockIdx.y, split = blockIdx.z;
  if (slot >= p.plan_head[0]) return;
  const int tok = p.dec_info[3 * slot], r = p.dec_info[3 * slot + 1], pos = p.dec_info[3 * slot + 2];
  const int G = p.n_heads / p.n_kv_heads;              // query heads on these keys (<= 16)
  const int PS = p.page_size;
  if (r < 0 || pos < 0 || pos / PS >= p.max_pages) {
    if (split == 0)
      for (int e = threadIdx.x; e < G * D; e += blockDim.x)
        p.out[((size_t)tok * p.n_heads + hk * G) * D + e] = __float2bfloat16_rn(0.f);
    return;
  }
  // the slice of this CTA, in whole chunks
  const int max_ctx = p.plan_head[2];
  int span = (max_ctx + p.splits - 1) / p.splits;
  span = (span + DM_CHUNK - 1) / DM_CHUNK * DM_CHUNK;
  const int k_begin = split * span;
  const int k_end = min((split + 1) * span, pos + 1);           // exclusive; pos itself included
  const int n_chunks = k_end > k_begin ? (k_end - k_begin + DM_CHUNK - 1) / DM_CHUNK : 0;
  const int own_chunk = (pos >= k_begin && pos < k_end) ? (pos - k_begin) / DM_CHUNK : -1;

  const size_t ptile = (size_t)PS * D;
  const size_t page_stride = 2 * (size_t)p.n_kv_heads * ptile;
  const int* trow = p.table + (size_t)r * p.max_pages;
  const __nv_bfloat16* own_row = p.qkv + (size_t)tok * p.qkv_stride;

  // This warp's chunks are warp, warp + NW, ...; lane i keeps the page of the warp's i-th
  // 16-position block (two a chunk), so that no copy waits for a table lookup.
  const int my_chunks = n_chunks > warp ? (n_chunks - warp + NW - 1) / NW : 0;
  int my_page = -1;
  {
    const int ci = lane >> 1, b = lane & 1;
    if (ci < my_chunks) {
      const int j0 = k_begin + (warp + ci * NW) * DM_CHUNK + b * 16;
      if (j0 < k_end) {
        my_page = trow[j0 / PS];
        if (my_page < 0 || my_page >= p.num_pages) {
          atomicOr(p.status, HS_STATUS_BAD_PAGE);
          my_page = -1;
        }
      }
    }
  }
  if (my_chunks > 16) atomicOr(p.status, HS_STATUS_BAD_POSITION);   // the host keeps slices shorter

  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  // A lane always copies the same 16-byte piece `ch` of rows lrow, lrow + 32 / CPR, ...: what
  // does not depend on the chunk is formed once.
  constexpr int RPI = 32 / CPR;                  // rows a warp instruction covers
  const int ch = lane % CPR, lrow = lane / CPR;
  const size_t head_off = (size_t)hk * ptile + (size_t)ch * 8;
  const size_t v_off_pool = (size_t)p.n_kv_heads * ptile;
  const __nv_bfloat16* own_k = own_row + p.k_off + (size_t)hk * D + ch * 8;
  const __nv_bfloat16* own_v = own_row + p.v_off + (size_t)hk * D + ch * 8;
  auto load_chunk = [&](int ci) {             // ci: index among this warp's chunks
    uint4* dK = ring + (size_t)(ci % STAGES) * 2 * SH::CHUNK_PIECES;
    uint4* dV = dK + SH::CHUNK_PIECES;
    const int c0 = k_begin + (warp + ci * NW) * DM_CHUNK;      // first key of the chunk
    const int page_a = __shfl_sync(0xffffffffu, my_page, (2 * ci) & 31);
    const int page_b = __shfl_sync(0xffffffffu, my_page, (2 * ci + 1) & 31);
    // the two 16-position blocks of the chunk: where they start inside their pages
    const __nv_bfloat16* blk_a = p.pool + (size_t)(page_a < 0 ? 0 : page_a) * page_stride +
                                 (size_t)(c0 % PS) * D + head_off;
    const __nv_bfloat16* blk_b = p.pool + (size_t)(page_b < 0 ? 0 : page_b) * page_stride +
                                 (size_t)((c0 + 16) % PS) * D + head_off;
#pragma unroll
    for (int i = 0; i < CPR; ++i) {           // 32 rows x CPR pieces; a warp instruction covers
      const int row = i * RPI + lrow;         // 512 contiguous bytes of a page
      const int j = c0 + row;
      const bool second = row >= 16;
      const int page = second ? page_b : page_a;
      const int dst = dm_swz<D>(row, ch);
      if (j < k_end && p.fuse_append && j == pos) {
        dm_cp16(&dK[dst], own_k);
        dm_cp16(&dV[dst], own_v);
      } else if (j < k_end && page >= 0) {
        const __nv_bfloat16* kp = (second ? blk_b : blk_a) + (size_t)(row & 15) * D;
        dm_cp16(&dK[dst], kp);
        dm_cp16(&dV[dst], kp + v_off_pool);
      } else {                                 // past the slice (or a refused page): zeros
        dK[dst] = zero4;
        dV[dst] = zero4;
      }
    }
  };
  // Chunks of earlier positions do not change during the step: with the append fused in they
  // are requested before the dependency wait.  The chunk that holds `pos` (the warp's last, if
  // it is this warp's) takes a row from the projection's output, so it comes after the wait.
  // Without fusion the previous kernel may be the one that appends this step's keys (up to
  // four positions of a request): nothing is requested before the wait.
  const int own_ci = (own_chunk >= 0 && own_chunk % NW == warp) ? own_chunk / NW : -1;
  const int first_fill = min(STAGES, my_chunks);                  // chunks of the first ring fill
  int n_pre = first_fill;
  if (!p.fuse_append) n_pre = 0;
  else if (own_ci >= 0 && own_ci < first_fill) n_pre = own_ci;    // the own chunk is the last one
#pragma unroll
  for (int s = 0; s < STAGES; ++s) {
    if (s < n_pre) {
      load_chunk(s);
      dm_commit();
    }
  }
  pdl_wait();
  // the rest of the first ring fill; then empty groups, so that group i is chunk i from here on
#pragma unroll
  for (int s = 0; s < STAGES; ++s) {
    if (s >= n_pre) {
      if (s < first_fill) load_chunk(s);
      dm_commit();
    }
  }
  // the queries: A fragments of the G heads' rows (row g and g + 8), straight from global memory
  uint32_t qf[KSTEPS][4];
  {
    const __nv_bfloat16* qb = own_row + p.q_off + (size_t)hk * G * D;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
      const int c = ks * 16 + t * 2;
      qf[ks][0] = g < G ? *(const uint32_t*)(qb + (size_t)g * D + c) : 0u;
      qf[ks][1] = g + 8 < G ? *(const uint32_t*)(qb + (size_t)(g + 8) * D + c) : 0u;
      qf[ks][2] = g < G ? *(const uint32_t*)(qb + (size_t)g * D + c + 8) : 0u;
      qf[ks][3] = g + 8 < G ? *(const uint32_t*)(qb + (size_t)(g + 8) * D + c + 8) : 0u;
    }
  }
  // with the append fused in, warp 0 of the slice that holds `pos` stores the new key and value
  if (p.fuse_append && own_chunk >= 0 && warp == 0) {
    const int page = trow[pos / PS];
    if (page < 0 || page >= p.num_pages) {
      if (lane == 0) atomicOr(p.status, HS_STATUS_BAD_PAGE);
    } else if (lane < 2 * CPR) {
      const int is_v = lane >= CPR, ch = lane % CPR;
      const uint4 v = *(const uint4*)(own_row + (is_v ? p.v_off : p.k_off) + (size_t)hk * D + ch * 8);
      __nv_bfloat16* dst = const_cast<__nv_bfloat16*>(p.pool) + (size_t)page * page_stride +
                           ((size_t)is_v * p.n_kv_heads + hk) * ptile + (size_t)(pos % PS) * D +
                           ch * 8;
      *(uint4*)dst = v;
    }
  }

  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  const float sl2 = p.scale * 1.4426950408889634f;       // scores in units of log2(e)

  for (int ci = 0; ci < my_chunks; ++ci) {
    // all groups but the newest STAGES - 1 have landed: chunk ci is in its buffer
    dm_wait<STAGES - 1>();
    __syncwarp();
    const uint4* tK = ring + (size_t)(ci % STAGES) * 2 * SH::CHUNK_PIECES;
    const uint4* tV = tK + SH::CHUNK_PIECES;
    const int c0 = k_begin + (warp + ci * NW) * DM_CHUNK;
    float s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int np = 0; np < 2; ++np) {            // pairs of 8-key tiles
        uint32_t b[4];
        const int mi = lane >> 3;
        const int key = np * 16 + (mi >> 1) * 8 + (lane & 7);
        dm_ldsm(b, &tK[dm_swz<D>(key, ks * 2 + (mi & 1))]);
        dm_mma(s[np * 2], qf[ks], b[0], b[1]);
        dm_mma(s[np * 2 + 1], qf[ks], b[2], b[3]);
      }
    }
    // mask the keys past the slice (only the last chunk has any), running maximum
    const bool ragged = c0 + DM_CHUNK > k_end;
    float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      if (ragged) {
        const int j = c0 + nt * 8 + t * 2;
        if (j >= k_end) s[nt][0] = s[nt][2] = -INFINITY;
        if (j + 1 >= k_end) s[nt][1] = s[nt][3] = -INFINITY;
      }
      mx_a = fmaxf(mx_a, fmaxf(s[nt][0], s[nt][1]));
      mx_b = fmaxf(mx_b, fmaxf(s[nt][2], s[nt][3]));
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float mn_a = fmaxf(m_a, mx_a * sl2), mn_b = fmaxf(m_b, mx_b * sl2);
    const float ca = (mn_a == -INFINITY) ? 1.f : dm_ex2(m_a - mn_a);
    const float cb = (mn_b == -INFINITY) ? 1.f : dm_ex2(m_b - mn_b);
    const float base_a = (mn_a == -INFINITY) ? 0.f : mn_a;
    const float base_b = (mn_b == -INFINITY) ? 0.f : mn_b;
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      s[nt][0] = dm_ex2(fmaf(s[nt][0], sl2, -base_a));
      s[nt][1] = dm_ex2(fmaf(s[nt][1], sl2, -base_a));
      s[nt][2] = dm_ex2(fmaf(s[nt][2], sl2, -base_b));
      s[nt][3] = dm_ex2(fmaf(s[nt][3], sl2, -base_b));
      sum_a += s[nt][0] + s[nt][1];
      sum_b += s[nt][2] + s[nt][3];
    }
    l_a = l_a * ca + sum_a;
    l_b = l_b * cb + sum_b;
    m_a = mn_a;
    m_b = mn_b;
#pragma unroll
    for (int i = 0; i < DT; ++i) {
      o[i][0] *= ca; o[i][1] *= ca; o[i][2] *= cb; o[i][3] *= cb;
    }
    // O += P V, 16 keys per k-step
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      uint32_t a[4];
      a[0] = dm_pack(s[2 * kk][0], s[2 * kk][1]);
      a[1] = dm_pack(s[2 * kk][2], s[2 * kk][3]);
      a[2] = dm_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = dm_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < DT / 2; ++dp) {
        uint32_t b[4];
        const int mi = lane >> 3;
        const int key = kk * 16 + (mi & 1) * 8 + (lane & 7);
        dm_ldsm_t(b, &tV[dm_swz<D>(key, dp * 2 + (mi >> 1))]);
        dm_mma(o[dp * 2], a, b[0], b[1]);
        dm_mma(o[dp * 2 + 1], a, b[2], b[3]);
      }
    }
    // the buffer of this chunk is free: the chunk STAGES further on goes into it
    __syncwarp();
    if (ci + STAGES < my_chunks) load_chunk(ci + STAGES);
    dm_commit();
  }
  dm_wait<0>();

  // ---- merge the warps' partial results through the ring memory (all copies have landed)
  __syncthreads();
  float* s_m = (float*)dm_smem;                       // [NW][16]
  float* s_l = s_m + NW * 16;                   // [NW][16]
  float* s_o = s_l + NW * 16;                   // [NW][16][D]
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  if (t == 0) {
    s_m[warp * 16 + g] = m_a; s_m[warp * 16 + g + 8] = m_b;
    s_l[warp * 16 + g] = l_a; s_l[warp * 16 + g + 8] = l_b;
  }
#pragma unroll
  for (int i = 0; i < DT; ++i) {
    const int d = i * 8 + t * 2;
    float* oa = s_o + ((size_t)warp * 16 + g) * D + d;
    float* ob = s_o + ((size_t)warp * 16 + g + 8) * D + d;
    oa[0] = o[i][0]; oa[1] = o[i][1];
    ob[0] = o[i][2]; ob[1] = o[i][3];
  }
  __syncthreads();
  __shared__ int s_last[16];
  for (int e = threadIdx.x; e < G * D; e += blockDim.x) {
    const int row = e / D, d = e - row * D;
    float cm = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) cm = fmaxf(cm, s_m[w * 16 + row]);
    float cl = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float mw = s_m[w * 16 + row];
      const float ws = (mw == -INFINITY) ? 0.f : dm_ex2(mw - cm);
      cl += s_l[w * 16 + row] * ws;
      a += s_o[((size_t)w * 16 + row) * D + d] * ws;
    }
    const int h = hk * G + row;
    if (p.splits == 1) {
      p.out[((size_t)tok * p.n_heads + h) * D + d] = __float2bfloat16_rn(cl > 0.f ? a / cl : 0.f);
    } else {
      const size_t pidx = ((size_t)slot * p.n_heads + h) * p.splits + split;
      p.acc[pidx * D + d] = a;
      if (d == 0) {
        // the maxima are kept in units of log2(e) here; the merge below uses exp2 as well
        p.ml[pidx * 2] = cm;
        p.ml[pidx * 2 + 1] = cl;
      }
    }
  }
  if (p.splits == 1) return;
  // ---- the last CTA of a (token, head) to arrive merges the slices in slice order
  __threadfence();
  __syncthreads();
  if (threadIdx.x < G) {
    const int h = hk * G + threadIdx.x;
    s_last[threadIdx.x] = atomicAdd(&p.counters[slot * p.n_heads + h], 1) == p.splits - 1;
  }
  __syncthreads();
  __threadfence();
  for (int e = threadIdx.x; e < G * D; e += blockDim.x) {
    const int row = e / D, d = e - row * D;
    if (!s_last[row]) continue;
    const int h = hk * G + row;
    const size_t base = ((size_t)slot * p.n_heads + h) * p.splits;
    float gm = -INFINITY;
    for (int s2 = 0; s2 < p.splits; ++s2) gm = fmaxf(gm, __ldcg(&p.ml[(base + s2) * 2]));
    float gl = 0.f, a = 0.f;
    for (int s2 = 0; s2 < p.splits; ++s2) {
      const float ms = __ldcg(&p.ml[(base + s2) * 2]);
      if (ms == -INFINITY) continue;
      const float w = dm_ex2(ms - gm);
      gl += __ldcg(&p.ml[(base + s2) * 2 + 1]) * w;
      a += __ldcg(&p.acc[(base + s2) * D + d]) * w;
    }
    p.out[((size_t)tok * p.n_heads + h) * D + d] = __float2bfloat16_rn(gl > 0.f ? a / gl : 0.f);
  }
  __syncthreads();
  if (threadIdx.x < G && s_last[threadIdx.x])
    p.counters[slot * p.n_heads + hk * G + threadIdx.x] = 0;        // ready for the next launch
}

template <int D, int STAGES_, int NW>
static cudaError_t dm_configure() {
  static cudaError_t state = cudaErrorUnknown;
  if (state != cudaSuccess)
    state = cudaFuncSetAttribute(attention_decode_mma_kernel<D, STAGES_, NW>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)DmShape<D, STAGES_, NW>::SMEM);
  return state;
}

// CTAs of this shape that share an SM (0: could not be asked)
template <int D, int STAGES_, int NW>
static int dm_occupancy() {
  static int occ = -1;
  if (occ < 0) {
    int n = 0;
    if (dm_configure<D, STAGES_, NW>() != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(
            &n, attention_decode_mma_kernel<D, STAGES_, NW>, NW * 32,
            DmShape<D, STAGES_, NW>::SMEM) != cudaSuccess)
      return 0;
    occ = n;
  }
  return occ;
}

template <int D, int STAGES_, int NW = DM_WARPS>
static cudaError_t dm_launch(const DecodeMmaParams& p, dim3 grid, cudaStream_t st, bool pdl) {
  if (cudaError_t e = dm_configure<D, STAGES_, NW>()) return e;
  return hs_launch(attention_decode_mma_kernel<D, STAGES_, NW>, grid, dim3(NW * 32),
                   DmShape<D, STAGES_, NW>::SMEM, st, pdl, p);
}

}  // namespace hs

// Single-query attention on the tensor cores.  Every served token brings one query per head at
// position `pos` (the work list's third entry); keys 0..pos are used.  fuse_append != 0: the
// key and value of `pos` are taken from the token's row of `qkv` (columns k_off / v_off) and
// stored to its page by the kernel; otherwise they are already in the pages.  Slices: keys per
// slice = ceil(longest context / splits) rounded up to 32, at most 2,048 (16 chunks a warp).
// Refuses (HS_ERR_UNSUPPORTED) head sizes other than 32, 64, 128, more than 16 query heads per
// key/value head, and slices that would be too long.
HS_EXPORT int hs_attention_decode_mma(void* out, const void* qkv, void* pool, const int* table,
                                      const int* dec_info, const int* plan_head, int token_cap,
                                      int n_heads, int n_kv_heads, int head_dim, int page_size,
                                      int num_pages, int max_pages, int q_off, int k_off,
                                      int v_off, int qkv_stride, float scale, int splits,
                                      int fuse_append, int pdl, float* scratch_acc,
                                      float* scratch_ml, int* counters, int* status,
                                      void* stream) {
  using namespace hs;
  if (!out || !qkv || !pool || !table || !dec_info || !plan_head || !status)
    return HS_ERR_ARGUMENT;
  if (token_cap <= 0) return HS_OK;
  if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return HS_ERR_UNSUPPORTED;
  if (n_heads / n_kv_heads > 16) return HS_ERR_UNSUPPORTED;
  if (page_size <= 0 || page_size % 16 || splits < 1 || splits > 65535) return HS_ERR_UNSUPPORTED;
  if (n_kv_heads > 65535 || token_cap > 2147483647 / 4) return HS_ERR_UNSUPPORTED;
  if (splits > 1 && (!scratch_acc || !scratch_ml || !counters)) return HS_ERR_ARGUMENT;
  if ((qkv_stride % 8) || (q_off % 8) || (k_off % 8) || (v_off % 8)) return HS_ERR_UNSUPPORTED;
  if (((uintptr_t)qkv & 15) || ((uintptr_t)pool & 15)) return HS_ERR_UNSUPPORTED;
  // a slice of at most 16 chunks per warp
  const long long max_ctx = (long long)max_pages * page_size;
  long long span = (max_ctx + splits - 1) / splits;
  span = (span + DM_CHUNK - 1) / DM_CHUNK * DM_CHUNK;
  if (span > 16LL * DM_WARPS * DM_CHUNK) return HS_ERR_UNSUPPORTED;
  DecodeMmaParams p;
  p.qkv = (const __nv_bfloat16*)qkv; p.pool = (const __nv_bfloat16*)pool;
  p.out = (__nv_bfloat16*)out; p.table = table; p.dec_info = dec_info; p.plan_head = plan_head;
  p.acc = scratch_acc; p.ml = scratch_ml; p.counters = counters; p.status = status;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
  p.num_pages = num_pages; p.max_pages = max_pages; p.q_off = q_off; p.k_off = k_off;
  p.v_off = v_off; p.qkv_stride = qkv_stride; p.splits = splits; p.fuse_append = fuse_append;
  p.scale = scale;
  dim3 grid(token_cap, n_kv_heads, splits);
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t le;
  // Shape by the number of CTAs against the SMs (measured with 16 heads of 64 at contexts of
  // 200 and 760): up to one CTA per SM, 8 warps with two chunks in flight each (128 KB); up to
  // two per SM, 8 warps with one chunk each (64 KB, so that two or three CTAs share an SM);
  // beyond that 4 warps with two chunks, and a third CTA per SM covers the fixed parts of the
  // others.  Head size 128 has chunks twice as large: one chunk in flight per warp (with 32 heads
  // over 8 key/value heads at batch 64: 49 us against 74 with two).
  int sms = 148;
  sms = hs_sm_count();
  const long long ctas = (long long)token_cap * n_kv_heads * splits;
  const int load = ctas <= sms ? 0 : (ctas <= 2LL * sms ? 1 : 2);
  const bool dep = pdl != 0;
  switch (head_dim) {
    case 32:
      le = load == 0   ? dm_launch<32, 3, 8>(p, grid, st, dep)
           : load == 1 ? dm_launch<32, 2, 8>(p, grid, st, dep)
                       : dm_launch<32, 2, 4>(p, grid, st, dep);
      break;
    case 64:
      if (load == 2) {
        // One chunk in flight per warp lets a fourth CTA share an SM: taken when that leaves
        // fewer empty places in the last round of CTAs (1,024 CTAs: 2 rounds of 592 places
        // instead of 3 of 444; 768 CTAs: 2 of 444 instead of 2 of 592).
        const long long two = (long long)dm_occupancy<64, 2, 4>() * sms;
        const long long one = (long long)dm_occupancy<64, 1, 4>() * sms;
        if (two <= 0 || one <= 0) return HS_ERR_UNSUPPORTED;
        const bool shallow = (ctas + one - 1) / one * one < (ctas + two - 1) / two * two;
        le = shallow ? dm_launch<64, 1, 4>(p, grid, st, dep) : dm_launch<64, 2, 4>(p, grid, st, dep);
        break;
      }
      le = load == 0 ? dm_launch<64, 2, 8>(p, grid, st, dep) : dm_launch<64, 1, 8>(p, grid, st, dep);
      break;
    case 128:
      le = load == 0 ? dm_launch<128, 1, 8>(p, grid, st, dep) : dm_launch<128, 1, 4>(p, grid, st, dep);
      break;
    default: return HS_ERR_UNSUPPORTED;
  }
  if (le != cudaSuccess) return (int)le;
  HS_LAUNCH_CHECK();
  return HS_OK;
}
