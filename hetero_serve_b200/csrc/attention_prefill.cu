// Causal attention of prompt portions over the paged cache on the tensor cores, bfloat16.
//
// The successor of the reference's WMMA prefill kernel (heteroserve/model/paged_attn_wmma.py:
// 80-254: FlashAttention tiling, one 16-token page = one key tile, 16-query tiles) and of its
// scalar one (heteroserve/model/paged_attn_prefill.py:72-157: query s of a portion sits at
// absolute position ctx_len - S + s and sees keys 0..that position; the mask is the loop bound).
//
// A work item = up to 128 consecutive queries of one request x one head, 8 warps of 16 queries.
// CTAs are persistent: each takes the next item from a counter in device memory, and the host
// lists the items with the most keys first, so the causal triangle's uneven tiles spread evenly
// over the SMs.  Keys and
// values are taken 64 positions at a time: each 16-position block of a tile lies inside one page
// (page sizes are multiples of 16), is found through the block table and copied to shared memory
// with cp.async (a ring of three tiles: two in flight while one is used).  S = Q K^T and O += P V run on mma.sync m16n8k16 (this is the kernel for head sizes 16, 32 and 128; head size 64 runs on
// tcgen05, attention_prefill_tc.cu)
// (bf16 in, f32 accumulate), fragments fetched with ldmatrix from XOR-swizzled tiles; the scores
// are multiplied by `scale` after the dot product (heteroserve/model/torch_engine.py:135); the
// running maximum, the running sum and O are float32 (online softmax).  The new tokens' own keys
// are already in the pages (they are appended first, torch_engine.py:306-308), so a portion needs
// no special case.  Tiles past a warp's last query are skipped.
//
// Work list (device memory, written by the host per step): plan_head[1] = number of tiles;
// tile_info[4 i ..] = flat index of the tile's first query, its number of queries (<= 128), its
// request's row in the block table, the position of its first query.
#include "common.cuh"

namespace hs {

constexpr int AP_BQ = 128, AP_BKV = 64, AP_WARPS = 8, AP_STAGES = 3;

struct PrefillParams {
  const __nv_bfloat16* qkv;
  const __nv_bfloat16* pool;
  __nv_bfloat16* out;
  const int* table;
  const int* tok_pos;
  const int* tok_req;
  const int* tile_info;    // per tile: first query's flat index, queries, request row, first position
  const int* plan_head;
  int* status;
  int* work_counter;       // next work item; zero at launch
  int n_heads, n_kv_heads, page_size, num_pages, max_pages;
  int q_off, qkv_stride;
  int ps_log2;             // log2(page_size) when it is a power of two, else -1
  float scale;
};

template <int D>
__device__ __forceinline__ int swz(int row, int chunk) {
  constexpr int CPR = D / 8;                       // 16-byte chunks per row
  constexpr int RPL = CPR >= 8 ? 1 : (8 / CPR > 0 ? 8 / CPR : 1);   // rows per 128-byte line
  // chunks are permuted inside groups of 8, or of the largest power of two that divides a row
  // (head sizes 48, 80, 96, 112: groups of 2 or 4, some bank conflicts, the same result)
  constexpr int GROUP = CPR % 8 == 0 ? 8 : (CPR % 4 == 0 ? 4 : (CPR % 2 == 0 ? 2 : 1));
  return row * CPR + (chunk ^ ((row / RPL) & (GROUP - 1)));
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* smem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}

template <int D>
__global__ void __launch_bounds__(AP_WARPS * 32, (D <= 64 ? 2 : 1))
attention_prefill_kernel(const PrefillParams p) {
  constexpr int CPR = D / 8;
  constexpr int KSTEPS = D / 16;       // k-steps of Q K^T
  constexpr int DT = D / 8;            // n-tiles of the output
  extern __shared__ __align__(128) uint8_t smem_raw[];
  uint4* sQ = (uint4*)smem_raw;                          // [64][CPR]
  uint4* sK = sQ + AP_BQ * CPR;                          // [AP_STAGES][64][CPR]
  uint4* sV = sK + AP_STAGES * AP_BKV * CPR;             // [AP_STAGES][64][CPR]

  __shared__ int s_item;
  const int n_items = p.plan_head[1] * p.n_heads;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  while (true) {
  __syncthreads();            // the previous item's shared memory has been consumed
  if (threadIdx.x == 0) s_item = atomicAdd(p.work_counter, 1);
  __syncthreads();
  const int item = s_item;
  if (item >= n_items) break;
  const int tile = item / p.n_heads, h = item - tile * p.n_heads;
  const int4 ti = *(const int4*)(p.tile_info + 4 * tile);
  const int tok0 = ti.x, nq = ti.y, r = ti.z, pos0 = ti.w;
  if (r < 0 || nq <= 0 || pos0 < 0) continue;
  const int pos_last = pos0 + nq - 1;
  if (pos_last / p.page_size >= p.max_pages) {
    if (threadIdx.x == 0) atomicOr(p.status, HS_STATUS_BAD_POSITION);
    continue;
  }
  const int hk = h / (p.n_heads / p.n_kv_heads);
  const int PS = p.page_size;
  const size_t ptile = (size_t)PS * D;
  const size_t page_stride = 2 * (size_t)p.n_kv_heads * ptile;
  const int* trow = p.table + (size_t)r * p.max_pages;
  const uint4 zero4 = make_uint4(0, 0, 0, 0);

  // ---- Q tile -> shared memory (rows past nq are zero)
  for (int c = threadIdx.x; c < AP_BQ * CPR; c += blockDim.x) {
    const int row = c / CPR, ch = c % CPR;
    uint4 v = zero4;
    if (row < nq)
      v = *(const uint4*)(p.qkv + (size_t)(tok0 + row) * p.qkv_stride + p.q_off + (size_t)h * D +
                          ch * 8);
    sQ[swz<D>(row, ch)] = v;
  }

  const int n_tiles = pos_last / AP_BKV + 1;
  auto load_tile = [&](int kt, int stage) {
    uint4* dK = sK + stage * AP_BKV * CPR;
    uint4* dV = sV + stage * AP_BKV * CPR;
    for (int c = threadIdx.x; c < AP_BKV * CPR; c += blockDim.x) {
      const int row = c / CPR, ch = c % CPR;
      const int j = kt * AP_BKV + row;
      const int dst = swz<D>(row, ch);
      bool ok = j <= pos_last;
      int page = 0;
      int slot_in_page = 0;
      if (ok) {
        const int pg = p.ps_log2 >= 0 ? (j >> p.ps_log2) : (j / PS);
        slot_in_page = j - pg * PS;
        page = trow[pg];
        if (page < 0 || page >= p.num_pages) {
          atomicOr(p.status, HS_STATUS_BAD_PAGE);
          ok = false;
        }
      }
      if (ok) {
        const __nv_bfloat16* kp = p.pool + (size_t)page * page_stride + (size_t)hk * ptile +
                                  (size_t)slot_in_page * D + ch * 8;
        cp_async16(&dK[dst], kp);
        cp_async16(&dV[dst], kp + (size_t)p.n_kv_heads * ptile);
      } else {
        dK[dst] = zero4;
        dV[dst] = zero4;
      }
    }
  };

  // tiles 0 .. AP_STAGES-2 are requested up front; one commit group per tile (empty ones too)
#pragma unroll
  for (int st = 0; st < AP_STAGES - 1; ++st) {
    if (st < n_tiles) load_tile(st, st);
    cp_async_commit();
  }
  __syncthreads();          // Q is in shared memory

  // ---- Q fragments stay in registers
  uint32_t qf[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks)
    ldsm_x4(qf[ks], &sQ[swz<D>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4))]);

  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  const int row_a = warp * 16 + g, row_b = row_a + 8;
  const int pos_a = min(pos0 + row_a, pos_last), pos_b = min(pos0 + row_b, pos_last);
  // last position any query of this warp sees; a warp whose rows are all past nq sees nothing
  const int warp_last = (warp * 16 < nq) ? min(pos0 + warp * 16 + 15, pos_last) : -1;
  const int warp_first = pos0 + warp * 16;               // position of the warp's first query
  const float sl2 = p.scale * 1.4426950408889634f;       // scores in units of log2(e)

  for (int kt = 0; kt < n_tiles; ++kt) {
    const int stage = kt % AP_STAGES;
    cp_async_wait<AP_STAGES - 2>();     // tile kt has landed (for this thread's copies)
    __syncthreads();                    // ... for everyone's; and tile kt-1 has been consumed
    if (kt + AP_STAGES - 1 < n_tiles)
      load_tile(kt + AP_STAGES - 1, (kt + AP_STAGES - 1) % AP_STAGES);
    cp_async_commit();
    if (kt * AP_BKV <= warp_last) {
      const uint4* tK = sK + stage * AP_BKV * CPR;
      const uint4* tV = sV + stage * AP_BKV * CPR;
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int np = 0; np < 4; ++np) {           // pairs of 8-key tiles
          uint32_t b[4];
          const int mi = lane >> 3;
          const int key = np * 16 + (mi >> 1) * 8 + (lane & 7);
          ldsm_x4(b, &tK[swz<D>(key, ks * 2 + (mi & 1))]);
          mma_bf16(s[np * 2], qf[ks], b[0], b[1]);
          mma_bf16(s[np * 2 + 1], qf[ks], b[2], b[3]);
        }
      }
      // scale (folded into the exponent: p = 2^(s * scale * log2 e - m)), mask, running maximum.
      // Only tiles that reach past the warp's first query need the mask.
      const bool diagonal = kt * AP_BKV + AP_BKV - 1 > warp_first;
      float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (diagonal) {
          const int j = kt * AP_BKV + nt * 8 + t * 2;
          if (j > pos_a) s[nt][0] = -INFINITY;
          if (j + 1 > pos_a) s[nt][1] = -INFINITY;
          if (j > pos_b) s[nt][2] = -INFINITY;
          if (j + 1 > pos_b) s[nt][3] = -INFINITY;
        }
        mx_a = fmaxf(mx_a, fmaxf(s[nt][0], s[nt][1]));
        mx_b = fmaxf(mx_b, fmaxf(s[nt][2], s[nt][3]));
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      // running maxima are kept in scaled units (m = max(s) * sl2; the scale is positive)
      const float mn_a = fmaxf(m_a, mx_a * sl2), mn_b = fmaxf(m_b, mx_b * sl2);
      // a row whose keys of this tile are all masked keeps its state (mn == m); a row with
      // no key at all yet (mn == -inf) contributes zeros
      const float ca = (mn_a == -INFINITY) ? 1.f : exp2f(m_a - mn_a);
      const float cb = (mn_b == -INFINITY) ? 1.f : exp2f(m_b - mn_b);
      const float base_a = (mn_a == -INFINITY) ? 0.f : mn_a;
      const float base_b = (mn_b == -INFINITY) ? 0.f : mn_b;
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = exp2f(fmaf(s[nt][0], sl2, -base_a));
        s[nt][1] = exp2f(fmaf(s[nt][1], sl2, -base_a));
        s[nt][2] = exp2f(fmaf(s[nt][2], sl2, -base_b));
        s[nt][3] = exp2f(fmaf(s[nt][3], sl2, -base_b));
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
      for (int kk = 0; kk < 4; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dp = 0; dp < DT / 2; ++dp) {      // pairs of 8-wide output tiles
          uint32_t b[4];
          const int mi = lane >> 3;
          const int key = kk * 16 + (mi & 1) * 8 + (lane & 7);
          ldsm_x4_t(b, &tV[swz<D>(key, dp * 2 + (mi >> 1))]);
          mma_bf16(o[dp * 2], a, b[0], b[1]);
          mma_bf16(o[dp * 2 + 1], a, b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  // ---- finish: the per-thread sums cover 2 of a row's 8 columns per tile; add the quad
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const float ia = l_a > 0.f ? 1.f / l_a : 0.f, ib = l_b > 0.f ? 1.f / l_b : 0.f;
  __nv_bfloat16* oa = p.out + ((size_t)(tok0 + row_a) * p.n_heads + h) * D;
  __nv_bfloat16* ob = p.out + ((size_t)(tok0 + row_b) * p.n_heads + h) * D;
#pragma unroll
  for (int i = 0; i < DT; ++i) {
    const int d = i * 8 + t * 2;
    if (row_a < nq) *(uint32_t*)(oa + d) = pack_bf16(o[i][0] * ia, o[i][1] * ia);
    if (row_b < nq) *(uint32_t*)(ob + d) = pack_bf16(o[i][2] * ib, o[i][3] * ib);
  }
  }   // next work item
}

template <int D>
static int launch_prefill(const PrefillParams& p, cudaStream_t st) {
  auto kern = attention_prefill_kernel<D>;
  constexpr int smem = (AP_BQ + 2 * AP_STAGES * AP_BKV) * D * 2;
  static int ctas = 0;                 // persistent CTAs: as many as are resident at once
  if (ctas == 0) {
    if (smem > 40 * 1024) {      // with the kernel's static shared memory: beyond the default 48 KB
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return (int)e;
    }
    int per_sm = 0, sms = 148;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, AP_WARPS * 32,
                                                                  smem);
    if (e != cudaSuccess) return (int)e;
    sms = hs_sm_count();
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 2) per_sm = 2;
    ctas = per_sm * sms;
  }
  cudaError_t e = cudaMemsetAsync(p.work_counter, 0, sizeof(int), st);
  if (e != cudaSuccess) return (int)e;
  kern<<<ctas, AP_WARPS * 32, smem, st>>>(p);
  HS_LAUNCH_CHECK();
  return HS_OK;
}

}  // namespace hs

HS_EXPORT int hs_attention_prefill(void* out, const void* qkv, const void* pool, const int* table,
                                   const int* tok_pos, const int* tok_req, const int* tile_info,
                                   const int* plan_head, int tile_cap,
                                   int* work_counter, int n_heads, int n_kv_heads, int head_dim, int page_size,
                                   int num_pages, int max_pages, int q_off, int qkv_stride,
                                   float scale, int* status, void* stream) {
  using namespace hs;
  if (!out || !qkv || !pool || !table || !tok_pos || !tok_req || !tile_info ||
      !plan_head || !status || !work_counter)
    return HS_ERR_ARGUMENT;
  if (tile_cap <= 0) return HS_OK;
  if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads || n_heads > 65535)
    return HS_ERR_UNSUPPORTED;
  if (page_size <= 0 || page_size % 16) return HS_ERR_UNSUPPORTED;
  if ((qkv_stride % 8) || (q_off % 8)) return HS_ERR_UNSUPPORTED;
  if (!(scale > 0.f)) return HS_ERR_UNSUPPORTED;     // maxima are tracked in scaled units
  PrefillParams p;
  p.qkv = (const __nv_bfloat16*)qkv; p.pool = (const __nv_bfloat16*)pool;
  p.out = (__nv_bfloat16*)out; p.table = table; p.tok_pos = tok_pos; p.tok_req = tok_req;
  p.tile_info = tile_info; p.plan_head = plan_head; p.status = status;
  p.work_counter = work_counter;
  p.ps_log2 = (page_size & (page_size - 1)) == 0 ? __builtin_ctz(page_size) : -1;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
  p.num_pages = num_pages; p.max_pages = max_pages; p.q_off = q_off; p.qkv_stride = qkv_stride;
  p.scale = scale;
  cudaStream_t st = (cudaStream_t)stream;
  switch (head_dim) {
    case 16: return launch_prefill<16>(p, st);
    case 32: return launch_prefill<32>(p, st);
    case 48: return launch_prefill<48>(p, st);
    case 64: return launch_prefill<64>(p, st);
    case 80: return launch_prefill<80>(p, st);
    case 96: return launch_prefill<96>(p, st);
    case 112: return launch_prefill<112>(p, st);
    case 128: return launch_prefill<128>(p, st);
    default: return HS_ERR_UNSUPPORTED;
  }
}
