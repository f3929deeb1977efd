// bfloat16 linear layer on the 5th-generation tensor cores (tcgen05) of sm_100a.
//
//   out[m, n] = act( sum_k a[m, k] * w[n, k] + bias[n] ) (+ residual[m, n])
//
// a [M, K] and w [N, K] are bfloat16 with K contiguous ("K-major" for both operands), the
// accumulator is float32 in tensor memory (TMEM), out is bfloat16 or float32.  It replaces the
// library matrix products of the reference (`h @ attn_w + attn_b`, `gelu(x @ fc_w + fc_b)`,
// `x + (... @ proj_w + proj_b)`, `ln_f(x) @ wte.T`: heteroserve/model/torch_engine.py:77-87,122,139)
// with the bias, the activation and the float32 residual sum fused into the epilogue.
//
// A persistent CTA (one per SM) walks over 128 x BN output tiles (n fastest, so that CTAs running
// together share rows of `a`):
//   warp 0       TMA producer: cp.async.bulk.tensor loads of a [128 x 64] tile of `a` and a
//                [BN x 64] tile of `w` per stage, 128-byte swizzle, completion on an mbarrier;
//   warp 1       allocates TMEM (two accumulators), then one elected thread issues tcgen05.mma
//                (M=128, N=BN, K=16, kind::f16, bf16 inputs, f32 accumulate), four per stage, and
//                commits each stage's completion to the stage's "empty" barrier and each tile's
//                to its accumulator's "full" barrier;
//   warps 4..11  epilogue: tcgen05.ld of the accumulator (lane = row, 32 columns at a time, two
//                warps per lane quarter), bias / activation / residual in float32, stores; it
//                runs while the MMAs of the next tile fill the other accumulator.
// Rows and columns beyond M, N and K are zero-filled by TMA and never stored.  With few rows
// (one row tile and few column tiles) the k range is also split between CTAs: each writes its
// share to scratch memory and the last to arrive (a counter per tile) adds them in split order.
//
// Every wait on an mbarrier is bounded: after HS_SPIN_LIMIT failed polls the thread sets
// HS_STATUS_PIPELINE_TIMEOUT in the status word and leaves the loop; the kernel then runs to
// its end (no store of that tile is trusted; the host raises on the status bit), frees its
// TMEM and returns.  Nothing can spin forever.
//
// The k-blocks of a tile are accumulated in index order by one MMA chain, whatever M is, so an
// output row does not depend on which other rows share its tile.
#include "tcgen05.cuh"

namespace hs {

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;          // 64 bf16 = 128 bytes = one swizzle row
constexpr int TC_UMMA_K = 16;

template <int BN, int STAGES>
struct TcSmem {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;  // + alignment slack
};

constexpr int TC_THREADS = 384;       // warp 0 TMA, warp 1 MMA, warps 4..11 epilogue
constexpr int TC_EPI_WARPS = 8;

struct TcParams {
  void* out;
  const float* bias;
  const float* residual;
  float* partial;        // [splits][M][N] float32 (splits > 1)
  int* counters;         // one per output tile, zero between launches (splits > 1)
  int* status;
  int M, N, K, act;
  int tiles_m, tiles_n;
  int splits, kb_per_split;   // k blocks (of 64) per split
};

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// The activation of the bfloat16 tensor-core path: the hardware tanh (relative error 2^-11,
// below bfloat16's 2^-9) for the tanh GELU; erff for the exact one.
__device__ __forceinline__ float act_tc(float u, int act) {
  if (act == HS_ACT_GELU_TANH) {
    const float inner = 0.7978845608028654f * (u + 0.044715f * u * u * u);
    return 0.5f * u * (1.0f + tanh_fast(inner));
  }
  if (act == HS_ACT_GELU_ERF) return gelu_erf(u);
  return u;
}
__device__ __forceinline__ void epi_bar_sync() {   // the 8 epilogue warps only
  asm volatile("bar.sync 1, 256;" ::: "memory");
}

// Stores 32 consecutive columns of one row: v[j] final values.
template <typename TO>
__device__ __forceinline__ void store_row32(TO* out, size_t off, const float (&f)[32], int nvalid,
                                            bool vec) {
  if (vec && nvalid == 32) {
    if constexpr (sizeof(TO) == 4) {
      float4* o4 = (float4*)((float*)out + off);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        o4[j] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
    } else {
      uint4* o4 = (uint4*)((__nv_bfloat16*)out + off);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 p0 = __floats2bfloat162_rn(f[8 * j], f[8 * j + 1]);
        __nv_bfloat162 p1 = __floats2bfloat162_rn(f[8 * j + 2], f[8 * j + 3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(f[8 * j + 4], f[8 * j + 5]);
        __nv_bfloat162 p3 = __floats2bfloat162_rn(f[8 * j + 6], f[8 * j + 7]);
        uint4 u;
        u.x = *(uint32_t*)&p0; u.y = *(uint32_t*)&p1; u.z = *(uint32_t*)&p2; u.w = *(uint32_t*)&p3;
        o4[j] = u;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < nvalid) out[off + j] = from_f<TO>(f[j]);
  }
}

// The epilogue of 32 consecutive columns of one row: bias, activation, float32 residual, store.
template <typename TO>
__device__ __forceinline__ void finish_row32(const TcParams& p, const uint32_t (&v)[32], int row,
                                             int nbase, int nvalid, bool vec) {
  TO* out = (TO*)p.out;
  float f[32];
  if (p.bias != nullptr && nvalid == 32 && (p.N % 4 == 0)) {
    const float4* b4 = (const float4*)(p.bias + nbase);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 b = __ldg(b4 + j);
      f[4 * j] = __uint_as_float(v[4 * j]) + b.x;
      f[4 * j + 1] = __uint_as_float(v[4 * j + 1]) + b.y;
      f[4 * j + 2] = __uint_as_float(v[4 * j + 2]) + b.z;
      f[4 * j + 3] = __uint_as_float(v[4 * j + 3]) + b.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      f[j] = __uint_as_float(v[j]) + ((p.bias && j < nvalid) ? p.bias[nbase + j] : 0.f);
  }
  if (p.act != HS_ACT_NONE) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = act_tc(f[j], p.act);
  }
  const size_t off = (size_t)row * p.N + nbase;
  if (p.residual) {
    if (nvalid == 32 && (p.N % 4 == 0)) {
      const float4* r4 = (const float4*)(p.residual + off);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 r = r4[j];
        f[4 * j] += r.x; f[4 * j + 1] += r.y; f[4 * j + 2] += r.z; f[4 * j + 3] += r.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < nvalid) f[j] += p.residual[off + j];
    }
  }
  store_row32<TO>(out, off, f, nvalid, vec);
}

// Persistent: each CTA takes work items (output tile x k split) blockIdx.x, + gridDim.x, ...
// Tiles are numbered with n fastest, so CTAs running together share the rows of `a`.
// Two accumulators in TMEM: the epilogue of one work item overlaps the MMAs of the next.
template <int BN, int STAGES, typename TO>
__global__ void __launch_bounds__(TC_THREADS, 1)
linear_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                      const __grid_constant__ CUtensorMap map_w, const TcParams p) {
  using S = TcSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzled tiles need 1024-byte alignment
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;       // [2] MMA -> epilogue
  uint64_t* acc_empty = acc_full + 2;            // [2] epilogue -> MMA
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  __shared__ int s_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (p.K + TC_BK - 1) / TC_BK;
  const int n_items = p.tiles_m * p.tiles_n * p.splits;
  constexpr uint32_t ACC_COLS = BN < 32 ? 32 : BN;
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;          // 64 .. 512, a power of two

  pdl_trigger();       // the next kernel may set itself up while this one runs
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], TC_EPI_WARPS);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above (barriers, tensor memory) touches nothing an earlier kernel writes; from
  // here on activations, the residual stream and the split-k scratch are read.
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer
      uint32_t it = 0;                          // k blocks issued so far (over all work items)
      bool ok = true;
      for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x) {
        const int tile = w / p.splits, split = w - tile * p.splits;
        const int m0 = (tile / p.tiles_n) * TC_BM, n0 = (tile % p.tiles_n) * BN;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, num_kb);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t round = it / STAGES;
          if (round > 0) ok = mbar_wait(&empty_bar[s], (round - 1) & 1, p.status);
          if (!ok) break;
          uint8_t* a_dst = smem + s * S::STAGE_BYTES;
          uint8_t* b_dst = a_dst + S::A_BYTES;
          mbar_expect_tx(&full_bar[s], S::STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, &full_bar[s], kb * TC_BK, m0);
          tma_load_2d(b_dst, &map_w, &full_bar[s], kb * TC_BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer
      constexpr uint32_t idesc = make_idesc(TC_BM, BN);
      uint32_t it = 0, wi = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < n_items && ok; w += gridDim.x, ++wi) {
        const int split = w % p.splits;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(kb0 + p.kb_per_split, num_kb);
        const uint32_t acc = wi & 1, acc_round = wi >> 1;
        if (acc_round > 0) ok = mbar_wait(&acc_empty[acc], (acc_round - 1) & 1, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * ACC_COLS;
        for (int kb = kb0; kb < kb1 && ok; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t round = it / STAGES;
          ok = mbar_wait(&full_bar[s], round & 1, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * S::STAGE_BYTES);
          const uint32_t b_addr = a_addr + S::A_BYTES;
          const uint64_t adesc = make_smem_desc(a_addr);
          const uint64_t bdesc = make_smem_desc(b_addr);
#pragma unroll
          for (int k = 0; k < TC_BK / TC_UMMA_K; ++k) {
            // advance 16 elements = 32 bytes along K inside the swizzled row: +2 in 16-byte units
            umma_bf16(tmem_d, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc,
                      (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);     // the stage may be refilled once these MMAs are done
        }
        umma_commit(&acc_full[acc]);      // this accumulator is complete (or the pipeline gave up)
      }
    }
  } else if (warp >= 4) {
    // ---------------- epilogue: 8 warps; warp (w % 4) owns TMEM lanes 32*(w%4) .. +31, the two
    // groups of four take the two halves of the columns
    const int q = warp & 3, half = (warp - 4) >> 2;
    constexpr int HALF_COLS = BN / 2;
    TO* out = (TO*)p.out;
    const bool vec = (p.N % 8 == 0);
    uint32_t wi = 0;
    for (int w = blockIdx.x; w < n_items; w += gridDim.x, ++wi) {
      const int tile = w / p.splits, split = w - tile * p.splits;
      const int m0 = (tile / p.tiles_n) * TC_BM, n0 = (tile % p.tiles_n) * BN;
      const uint32_t acc = wi & 1, acc_round = wi >> 1;
      const bool ok = mbar_wait(&acc_full[acc], acc_round & 1, p.status);
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t t_addr = tmem_base + acc * ACC_COLS + ((uint32_t)(q * 32) << 16);
      if (ok) {
#pragma unroll 1
        for (int c0 = half * HALF_COLS; c0 < (half + 1) * HALF_COLS; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(t_addr + (uint32_t)c0, v);
          tmem_ld_wait();
          const int nbase = n0 + c0;
          if (row >= p.M || nbase >= p.N) continue;
          const int nvalid = min(32, p.N - nbase);
          if (p.splits > 1) {
            // raw partial sums to scratch; the last split to arrive finishes the tile below
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
            store_row32<float>(p.partial, ((size_t)split * p.M + row) * p.N + nbase, f, nvalid,
                               p.N % 4 == 0);
            continue;
          }
          finish_row32<TO>(p, v, row, nbase, nvalid, vec);
        }
      }
      // the accumulator may be overwritten by the MMAs of the work item after next
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);

      if (p.splits > 1) {
        // ---- the last split of this tile to arrive adds the shares in split order
        __threadfence();
        epi_bar_sync();
        if (threadIdx.x == 4 * 32) s_last = atomicAdd(&p.counters[tile], 1) == p.splits - 1;
        epi_bar_sync();
        if (s_last) {
          __threadfence();
          // 256 threads sweep the tile in float4 pieces, rows of the tile x BN/4 pieces a row;
          // the loads of all shares of a piece are issued together, then added in split order
          const int et = threadIdx.x - 4 * 32;                   // 0..255
          constexpr int PIECES = BN / 4;
          const int rows_here = min(TC_BM, p.M - m0);
          const bool vec4 = (p.N % 4 == 0);
          for (int e = et; e < rows_here * PIECES; e += TC_EPI_WARPS * 32) {
            const int r = e / PIECES, c = (e % PIECES) * 4;
            const int n = n0 + c;
            if (n >= p.N) continue;
            const size_t off = (size_t)(m0 + r) * p.N + n;
            float4 acc4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (vec4) {
              float4 sh[16];
#pragma unroll
              for (int sp = 0; sp < 16; ++sp)
                if (sp < p.splits)
                  sh[sp] = __ldcg((const float4*)(p.partial + (size_t)sp * p.M * p.N + off));
#pragma unroll
              for (int sp = 0; sp < 16; ++sp)
                if (sp < p.splits) {
                  acc4.x += sh[sp].x; acc4.y += sh[sp].y; acc4.z += sh[sp].z; acc4.w += sh[sp].w;
                }
            } else {
              float* a = (float*)&acc4;
              for (int sp = 0; sp < p.splits; ++sp)
                for (int j = 0; j < 4; ++j)
                  if (n + j < p.N) a[j] += __ldcg(p.partial + (size_t)sp * p.M * p.N + off + j);
            }
            float vals[4] = {acc4.x, acc4.y, acc4.z, acc4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (n + j < p.N) {
                float x = vals[j] + (p.bias ? p.bias[n + j] : 0.f);
                x = act_tc(x, p.act);
                if (p.residual) x += p.residual[off + j];
                out[off + j] = from_f<TO>(x);
              }
            }
          }
          epi_bar_sync();
          if (threadIdx.x == 4 * 32) p.counters[tile] = 0;       // ready for the next launch
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------- pairs of CTAs
// The same linear layer with cta_group::2: a cluster of two CTAs on neighbouring SMs works on
// one 256 x BN output tile.  CTA r of the pair loads rows m0 + 128 r .. of `a` and rows
// n0 + BN/2 r .. of `w` into its own shared memory (BN/2 instead of BN rows of the weight a
// stage: a third less L2 traffic per FLOP than the single-CTA 128 x 256 tile, which is what
// bounds the main loop at these sizes); the even CTA's elected thread issues
// tcgen05.mma.cta_group::2 (M = 256), which reads both CTAs' tiles and accumulates each CTA's
// 128 rows into that CTA's tensor memory; each CTA's epilogue warps store their own rows.
// Barriers: "full" lives in the even CTA (its producer announces the bytes of both CTAs, both
// CTAs' TMA loads complete on it); "empty" and "accumulator full" are signalled in both CTAs at
// once by tcgen05.commit with a CTA mask; "accumulator empty" lives in the even CTA and counts
// the epilogue warps of both.  No split over k (used only when there are many rows).
template <int BN, int STAGES>
struct PairSmem {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = (BN / 2) * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;
};

template <int BN, int STAGES, typename TO>
__global__ void __launch_bounds__(TC_THREADS, 1)
linear_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a,
                           const __grid_constant__ CUtensorMap map_w, const TcParams p) {
  using S = PairSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();              // 0: issues the MMAs
  const int num_kb = (p.K + TC_BK - 1) / TC_BK;
  const int n_items = p.tiles_m * p.tiles_n;            // tiles of 256 x BN
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  constexpr uint32_t ACC_COLS = BN;
  constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 2 * TC_EPI_WARPS);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();          // both CTAs' barriers exist before either signals the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer (one per CTA)
      uint32_t it = 0;
      bool ok = true;
      for (int w = pair; w < n_items && ok; w += n_pairs) {
        const int m0 = (w / p.tiles_n) * (2 * TC_BM) + (int)rank * TC_BM;
        const int n0 = (w % p.tiles_n) * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t round = it / STAGES;
          if (round > 0) ok = mbar_wait(&empty_bar[s], (round - 1) & 1, p.status);
          if (!ok) break;
          uint8_t* a_dst = smem + s * S::STAGE_BYTES;
          uint8_t* b_dst = a_dst + S::A_BYTES;
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * S::STAGE_BYTES);
          const uint32_t bar = cluster_map(&full_bar[s], 0);
          tma_load_2d_pair(a_dst, &map_a, bar, kb * TC_BK, m0);
          tma_load_2d_pair(b_dst, &map_w, bar, kb * TC_BK, n0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ---------------- MMA issuer (the even CTA only)
      constexpr uint32_t idesc = make_idesc(2 * TC_BM, BN);
      uint32_t it = 0, wi = 0;
      bool ok = true;
      for (int w = pair; w < n_items && ok; w += n_pairs, ++wi) {
        const uint32_t acc = wi & 1, acc_round = wi >> 1;
        if (acc_round > 0) ok = mbar_wait(&acc_empty[acc], (acc_round - 1) & 1, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * ACC_COLS;
        for (int kb = 0; kb < num_kb && ok; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t round = it / STAGES;
          ok = mbar_wait(&full_bar[s], round & 1, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * S::STAGE_BYTES);
          const uint32_t b_addr = a_addr + S::A_BYTES;
          const uint64_t adesc = make_smem_desc(a_addr);
          const uint64_t bdesc = make_smem_desc(b_addr);
#pragma unroll
          for (int k = 0; k < TC_BK / TC_UMMA_K; ++k)
            umma_bf16_pair(tmem_d, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc,
                           (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty_bar[s], 3);       // both CTAs may refill the stage
        }
        umma_commit_pair(&acc_full[acc], 3);        // both CTAs' epilogues may read
      }
    }
  } else if (warp >= 4) {
    // ---------------- epilogue: this CTA's 128 rows of the tile
    const int q = warp & 3, half = (warp - 4) >> 2;
    constexpr int HALF_COLS = BN / 2;
    const bool vec = (p.N % 8 == 0);
    const uint32_t acc_empty_leader0 = cluster_map(&acc_empty[0], 0);
    const uint32_t acc_empty_leader1 = cluster_map(&acc_empty[1], 0);
    uint32_t wi = 0;
    for (int w = pair; w < n_items; w += n_pairs, ++wi) {
      const int m0 = (w / p.tiles_n) * (2 * TC_BM) + (int)rank * TC_BM;
      const int n0 = (w % p.tiles_n) * BN;
      const uint32_t acc = wi & 1, acc_round = wi >> 1;
      const bool ok = mbar_wait(&acc_full[acc], acc_round & 1, p.status);
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t t_addr = tmem_base + acc * ACC_COLS + ((uint32_t)(q * 32) << 16);
      if (ok) {
#pragma unroll 1
        for (int c0 = half * HALF_COLS; c0 < (half + 1) * HALF_COLS; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(t_addr + (uint32_t)c0, v);
          tmem_ld_wait();
          const int nbase = n0 + c0;
          if (row >= p.M || nbase >= p.N) continue;
          finish_row32<TO>(p, v, row, nbase, min(32, p.N - nbase), vec);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(acc ? acc_empty_leader1 : acc_empty_leader0);
    }
  }
  // Neither CTA may leave (or free its tensor memory) while the other can still signal its
  // barriers or the MMAs can still touch its memories.
  tc_fence_before();
  __syncthreads();
  cluster_sync();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// A [rows, K] bfloat16 matrix with K contiguous, fetched in boxes of [box_rows x 64].
static int make_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return HS_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                   strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? HS_OK : HS_ERR_ARGUMENT;
}

template <int BN, int STAGES, typename TO>
static int launch(const CUtensorMap& ma, const CUtensorMap& mw, const TcParams& p, int grid,
                  cudaStream_t st) {
  auto kern = linear_tcgen05_kernel<BN, STAGES, TO>;
  constexpr int smem = TcSmem<BN, STAGES>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaError_t le = hs_launch(kern, dim3(grid), dim3(TC_THREADS), (size_t)smem, st,
                             hs_pdl_enabled(), ma, mw, p);
  if (le != cudaSuccess) return (int)le;
  HS_LAUNCH_CHECK();
  return HS_OK;
}

template <int BN, int STAGES, typename TO>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mw, const TcParams& p, int grid,
                       cudaStream_t st) {
  auto kern = linear_tcgen05_pair_kernel<BN, STAGES, TO>;
  constexpr int smem = PairSmem<BN, STAGES>::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = hs_pdl_enabled() ? 2 : 1;
  cudaError_t le = cudaLaunchKernelEx(&cfg, kern, ma, mw, p);
  if (le != cudaSuccess) return (int)le;
  HS_LAUNCH_CHECK();
  return HS_OK;
}

struct TcPlan {
  int bn, splits, kb_per_split, tiles_m, tiles_n, grid;
  bool pair;
};

// pair: -1 = decide here, 0 = single CTAs, 1 = pairs of CTAs (256-row tiles)
static bool plan_tc(int M, int N, int K, int tile_n, int pair, TcPlan& pl) {
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  const int mt = (M + TC_BM - 1) / TC_BM;
  const int num_kb = (K + TC_BK - 1) / TC_BK;
  // measured on B200: pairs gain 5-9 % from 4,096 rows on (4096^3, 8192^3) and nothing at 2,048
  pl.pair = pair == 1 || (pair < 0 && M >= 4096);
  if (pl.pair) {
    // 256 x BN tiles over sms / 2 pairs; a CTA loads 128 + BN/2 rows per k-block
    const int pairs = sms / 2 > 0 ? sms / 2 : 1;
    const int mt2 = (M + 2 * TC_BM - 1) / (2 * TC_BM);
    int bn = tile_n;
    if (bn == 0) {
      long best = -1;
      for (int cand : {256, 128}) {
        if (cand / 2 >= N && cand > 128) continue;
        const long tiles = (long)mt2 * ((N + cand - 1) / cand);
        const long cost = ((tiles + pairs - 1) / pairs) * (cand / 2 + 128 + 64);
        if (best < 0 || cost < best) {
          best = cost;
          bn = cand;
        }
      }
    }
    if (bn != 128 && bn != 256) return false;
    pl.bn = bn;
    pl.tiles_m = mt2;
    pl.tiles_n = (N + bn - 1) / bn;
    pl.splits = 1;
    pl.kb_per_split = num_kb;
    const int tiles = pl.tiles_m * pl.tiles_n;
    pl.grid = 2 * (tiles < pairs ? tiles : pairs);
    return true;
  }
  int bn = tile_n;
  if (bn == 0) {
    // A tile's time grows with the bytes it loads per k-block (128 + width rows) plus a fixed
    // part; pick the width for which rounds over the SMs x that is smallest.
    long best = -1;
    for (int cand : {256, 128, 64}) {
      if (cand > 64 && cand / 2 >= N) continue;
      const long tiles = (long)mt * ((N + cand - 1) / cand);
      const long cost = ((tiles + sms - 1) / sms) * (cand + 128 + 64);
      if (best < 0 || cost < best) {
        best = cost;
        bn = cand;
      }
    }
    if (mt == 1) bn = 64;     // few rows: narrow tiles (more CTAs stream the weights) and splits
  }
  if (bn != 64 && bn != 128 && bn != 256) return false;
  pl.bn = bn;
  pl.tiles_m = mt;
  pl.tiles_n = (N + bn - 1) / bn;
  const int tiles = pl.tiles_m * pl.tiles_n;
  // splits over k only while the tiles alone leave most SMs idle (few rows), each split at
  // least 2 k blocks deep
  int splits = 1;
  if (tiles * 2 <= sms) {
    splits = sms / tiles;
    if (splits > num_kb / 2) splits = num_kb / 2;
    if (splits < 1) splits = 1;
    if (splits > 16) splits = 16;
  }
  pl.kb_per_split = (num_kb + splits - 1) / splits;
  pl.splits = (num_kb + pl.kb_per_split - 1) / pl.kb_per_split;
  const int items = tiles * pl.splits;
  pl.grid = items < sms ? items : sms;
  return true;
}

}  // namespace hs

// Scratch a launch needs when it is split over k: floats for the shares, ints for the counters
// (both zero when it is not split).
HS_EXPORT int hs_linear_tcgen05_scratch(int M, int N, int K, int tile_n, int pair,
                                        long long* floats, int* counters) {
  hs::TcPlan pl;
  if (M <= 0 || N <= 0 || K <= 0 || !hs::plan_tc(M, N, K, tile_n, pair, pl))
    return HS_ERR_UNSUPPORTED;
  *floats = pl.splits > 1 ? (long long)pl.splits * M * N : 0;
  *counters = pl.splits > 1 ? pl.tiles_m * pl.tiles_n : 0;
  return HS_OK;
}

// Returns HS_ERR_UNSUPPORTED for shapes the TMA path cannot take (K not a multiple of 8:
// row strides must be multiples of 16 bytes; pointers not 16-byte aligned); the caller falls
// back to the CUDA-core kernel.
HS_EXPORT int hs_linear_tcgen05(void* out, const void* a, const void* w, const float* bias,
                                const float* residual, int M, int N, int K, int act,
                                int out_dtype, int tile_n, int pair, float* scratch,
                                int* counters, int* status, void* stream) {
  using namespace hs;
  if (!out || !a || !w || !status) return HS_ERR_ARGUMENT;
  if (M <= 0 || N <= 0) return HS_OK;
  if (K <= 0) return HS_ERR_ARGUMENT;
  if (K % 8 != 0) return HS_ERR_UNSUPPORTED;
  if (((uintptr_t)a & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15)) return HS_ERR_UNSUPPORTED;
  if (residual && ((uintptr_t)residual & 15)) return HS_ERR_UNSUPPORTED;
  if (bias && ((uintptr_t)bias & 15)) return HS_ERR_UNSUPPORTED;
  if (act < HS_ACT_NONE || act > HS_ACT_GELU_ERF) return HS_ERR_UNSUPPORTED;
  if (out_dtype != HS_DT_F32 && out_dtype != HS_DT_BF16) return HS_ERR_UNSUPPORTED;
  TcPlan pl;
  if (!plan_tc(M, N, K, tile_n, pair, pl)) return HS_ERR_UNSUPPORTED;
  if (pl.splits > 1 && (!scratch || !counters)) return HS_ERR_ARGUMENT;
  CUtensorMap ma, mw;
  if (int e = make_map(&ma, a, M, K, TC_BM)) return e;
  if (int e = make_map(&mw, w, N, K, pl.pair ? pl.bn / 2 : pl.bn)) return e;
  TcParams p;
  p.out = out; p.bias = bias; p.residual = residual; p.partial = scratch; p.counters = counters;
  p.status = status; p.M = M; p.N = N; p.K = K; p.act = act;
  p.tiles_m = pl.tiles_m; p.tiles_n = pl.tiles_n; p.splits = pl.splits;
  p.kb_per_split = pl.kb_per_split;
  cudaStream_t st = (cudaStream_t)stream;
  using bf16 = __nv_bfloat16;
#define HS_TC(BN, ST)                                                        \
  (out_dtype == HS_DT_F32 ? launch<BN, ST, float>(ma, mw, p, pl.grid, st)    \
                          : launch<BN, ST, bf16>(ma, mw, p, pl.grid, st))
  if (pl.pair) {
    if (pl.bn == 256)
      return out_dtype == HS_DT_F32 ? launch_pair<256, 6, float>(ma, mw, p, pl.grid, st)
                                    : launch_pair<256, 6, bf16>(ma, mw, p, pl.grid, st);
    return out_dtype == HS_DT_F32 ? launch_pair<128, 8, float>(ma, mw, p, pl.grid, st)
                                  : launch_pair<128, 8, bf16>(ma, mw, p, pl.grid, st);
  }
  switch (pl.bn) {
    case 256: return HS_TC(256, 4);
    case 128: return HS_TC(128, 6);
    default: return HS_TC(64, 8);
  }
#undef HS_TC
}
