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

constexpr int TC_THREADS = 384;       // warp 0 TMA, warp 1 MMA, warps 4..11 epilogue
constexpr int TC_EPI_WARPS = 8;
constexpr int TC_PATCH_BYTES = 32 * 64;   // per epilogue warp: 32 rows x 64 bytes

template <int BN, int STAGES>
struct TcSmem {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int PATCH_OFFSET = STAGES * STAGE_BYTES;          // epilogue staging
  static constexpr int BIAS_OFFSET = PATCH_OFFSET + TC_EPI_WARPS * TC_PATCH_BYTES;
  static constexpr int BAR_OFFSET = BIAS_OFFSET + 2 * 256 * 4;      // bias of two tiles
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16 + 1024;  // + alignment slack
};

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
  // one branch per chunk, not per element (the compiler must not evaluate both forms)
  if (p.act == HS_ACT_GELU_TANH) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = act_tc(f[j], HS_ACT_GELU_TANH);
  } else if (p.act == HS_ACT_GELU_ERF) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = act_tc(f[j], HS_ACT_GELU_ERF);
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

// Bias and activation of a full chunk of 32 columns, in registers.  `bias_s`: the chunk's 32
// bias values in shared memory (staged by the epilogue warps before the accumulator is ready:
// a global load here would cost an L2 round trip per chunk), or null.
__device__ __forceinline__ void bias_act32(const TcParams& p, const uint32_t (&v)[32],
                                           const float* bias_s, float (&f)[32]) {
  if (bias_s != nullptr) {
    const float4* b4 = (const float4*)bias_s;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 b = b4[j];
      f[4 * j] = __uint_as_float(v[4 * j]) + b.x;
      f[4 * j + 1] = __uint_as_float(v[4 * j + 1]) + b.y;
      f[4 * j + 2] = __uint_as_float(v[4 * j + 2]) + b.z;
      f[4 * j + 3] = __uint_as_float(v[4 * j + 3]) + b.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]) + 0.f;
  }
  // one branch per chunk, not per element (the compiler must not evaluate both forms)
  if (p.act == HS_ACT_GELU_TANH) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = act_tc(f[j], HS_ACT_GELU_TANH);
  } else if (p.act == HS_ACT_GELU_ERF) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = act_tc(f[j], HS_ACT_GELU_ERF);
  }
}

// Storing a full chunk (32 valid columns, N a multiple of 8) with coalesced global
// accesses.  A lane owns one ROW of the accumulator, so storing its values directly makes every
// warp instruction touch 32 different cache lines (the epilogue was bound by exactly that).
// Instead the finished values go through a 32 x 64-byte patch of shared memory (pieces of 16
// bytes, XOR-swizzled: no bank conflicts either way) and leave it with 4 lanes per row: a warp
// instruction then covers 8 rows x 64 contiguous bytes.  The float32 residual is read with the
// same coalesced pattern.  The arithmetic and its order are those of finish_row32.
// The residual of a chunk in the layout the staged store uses: piece (h, i) is the float4 of row
// 8 i + lane / 4 at columns 16 h + 4 (lane % 4) .. of the chunk.
struct ResChunk {
  float4 r[2][4];
};
__device__ __forceinline__ void load_residual_chunk(const TcParams& p, ResChunk& rc, int lane,
                                                    int row0, int nbase) {
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = i * 8 + (lane >> 2);
      const size_t off = (size_t)(row0 + r) * p.N + nbase + h * 16 + (lane & 3) * 4;
      rc.r[h][i] = (row0 + r < p.M) ? *(const float4*)(p.residual + off)
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

template <typename TO>
__device__ __forceinline__ void store_chunk_staged(const TcParams& p, const float (&f)[32],
                                                   const ResChunk* rc, uint8_t* patch, int lane,
                                                   int row0, int nbase) {
  constexpr int PER = 64 / (int)sizeof(TO);          // columns per 64-byte piece of a row
  TO* out = (TO*)p.out;
  const int sw_w = (lane >> 1) & 3;                   // swizzle of the row this lane writes
#pragma unroll
  for (int h = 0; h < 32 / PER; ++h) {
#pragma unroll
    for (int pc = 0; pc < 4; ++pc) {
      uint4 u;
      if constexpr (sizeof(TO) == 4) {
        const int c = h * PER + pc * 4;
        u.x = __float_as_uint(f[c]); u.y = __float_as_uint(f[c + 1]);
        u.z = __float_as_uint(f[c + 2]); u.w = __float_as_uint(f[c + 3]);
      } else {
        const int c = h * PER + pc * 8;
        __nv_bfloat162 p0 = __floats2bfloat162_rn(f[c], f[c + 1]);
        __nv_bfloat162 p1 = __floats2bfloat162_rn(f[c + 2], f[c + 3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(f[c + 4], f[c + 5]);
        __nv_bfloat162 p3 = __floats2bfloat162_rn(f[c + 6], f[c + 7]);
        u.x = *(uint32_t*)&p0; u.y = *(uint32_t*)&p1; u.z = *(uint32_t*)&p2; u.w = *(uint32_t*)&p3;
      }
      *(uint4*)(patch + lane * 64 + ((pc ^ sw_w) << 4)) = u;
    }
    __syncwarp();
    const int pc = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = i * 8 + (lane >> 2);
      const uint4 u = *(const uint4*)(patch + r * 64 + ((pc ^ ((r >> 1) & 3)) << 4));
      if (row0 + r >= p.M) continue;
      if constexpr (sizeof(TO) == 4) {
        const size_t off = (size_t)(row0 + r) * p.N + nbase + h * PER + pc * 4;
        float4 o = make_float4(__uint_as_float(u.x), __uint_as_float(u.y), __uint_as_float(u.z),
                               __uint_as_float(u.w));
        if (rc != nullptr) {
          const float4 q = rc->r[h][i];
          o.x += q.x; o.y += q.y; o.z += q.z; o.w += q.w;
        }
        *(float4*)((float*)out + off) = o;
      } else {
        const size_t off = (size_t)(row0 + r) * p.N + nbase + h * PER + pc * 8;
        *(uint4*)((__nv_bfloat16*)out + off) = u;
      }
    }
    __syncwarp();
  }
}

// One epilogue warp's share of a tile: NCHUNK chunks of 32 columns from c_begin on, of the 32
// rows it owns in tensor memory.  Before it waits for the accumulator it has the residual of
// its first two chunks on the way (the main loop hides the loads); afterwards the tcgen05.ld of
// the next chunk and the residual two chunks ahead are in flight while a chunk is finished and
// stored.  `bias_s`: this tile's bias in shared memory (index = column inside the tile) or null.
// Returns false if the wait ran out.
template <typename TO, int NCHUNK, bool SPLIT>
__device__ __forceinline__ bool epilogue_columns(const TcParams& p, uint64_t* acc_bar,
                                                 uint32_t parity, uint32_t t_addr, int c_begin,
                                                 int row0, int n0, int lane, uint8_t* patch,
                                                 const float* bias_s, int split) {
  const int row = row0 + lane;
  const bool vec = (p.N % 8 == 0);
  const bool staged_ok = !SPLIT && vec && !(sizeof(TO) == 2 && p.residual != nullptr);
  const bool res_ahead = !SPLIT && sizeof(TO) == 4 && staged_ok && p.residual != nullptr;
  auto full_chunk = [&](int c) { return n0 + c_begin + 32 * c + 32 <= p.N; };
  ResChunk rc[2];
  if constexpr (!SPLIT) if (res_ahead) {
#pragma unroll
    for (int c = 0; c < 2 && c < NCHUNK; ++c)
      if (full_chunk(c)) load_residual_chunk(p, rc[c], lane, row0, n0 + c_begin + 32 * c);
  }
  const bool ok = mbar_wait(acc_bar, parity, p.status);
  tc_fence_after();
  if (!ok) return false;
  uint32_t v[32];
  tmem_ld32(t_addr + (uint32_t)c_begin, v);
#pragma unroll
  for (int c = 0; c < NCHUNK; ++c) {
    const int c0 = c_begin + 32 * c;
    tmem_ld_wait();
    const int nbase = n0 + c0;
    const int nvalid = min(32, p.N - nbase);
    if (!SPLIT && staged_ok && nvalid == 32) {
      float f[32];
      bias_act32(p, v, bias_s ? bias_s + c0 : nullptr, f);
      if (c + 1 < NCHUNK) tmem_ld32(t_addr + (uint32_t)(c0 + 32), v);
      store_chunk_staged<TO>(p, f, res_ahead ? &rc[c & 1] : nullptr, patch, lane, row0, nbase);
      if (res_ahead && c + 2 < NCHUNK && full_chunk(c + 2))
        load_residual_chunk(p, rc[c & 1], lane, row0, nbase + 64);
      continue;
    }
    if constexpr (SPLIT) {
      // raw partial sums to this split's share of the scratch; the last split to arrive
      // finishes the tile.  Whole chunks leave through the staging patch (coalesced).
      float f[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
      if (c + 1 < NCHUNK) tmem_ld32(t_addr + (uint32_t)(c0 + 32), v);
      if (vec && nvalid == 32) {
        TcParams share = p;
        share.out = p.partial + (size_t)split * p.M * p.N;
        store_chunk_staged<float>(share, f, nullptr, patch, lane, row0, nbase);
      } else if (row < p.M && nbase < p.N) {
        store_row32<float>(p.partial, ((size_t)split * p.M + row) * p.N + nbase, f, nvalid,
                           p.N % 4 == 0);
      }
      continue;
    }
    if (row < p.M && nbase < p.N) finish_row32<TO>(p, v, row, nbase, nvalid, vec);
    if (c + 1 < NCHUNK) tmem_ld32(t_addr + (uint32_t)(c0 + 32), v);
  }
  return true;
}

// The epilogue warps (256 threads) put the bias of the tile at columns n0 .. n0 + BN into
// `dst` (zeros past N) and meet at their own barrier.
template <int BN>
__device__ __forceinline__ void stage_bias(const TcParams& p, float* dst, int n0) {
  const int e = threadIdx.x - 4 * 32;
  if (e < BN) dst[e] = (n0 + e < p.N) ? __ldg(p.bias + n0 + e) : 0.f;
  epi_bar_sync();
}

// Persistent: each CTA takes work items (output tile x k split) blockIdx.x, + gridDim.x, ...
// Tiles are numbered with n fastest, so CTAs running together share the rows of `a`.
// Two accumulators in TMEM: the epilogue of one work item overlaps the MMAs of the next.
template <int BN, int STAGES, typename TO, bool SPLIT>
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
  // columns from one accumulator to the other: a power of two (192-wide tiles sit 256 apart)
  constexpr uint32_t ACC_COLS = BN < 32 ? 32 : (BN == 192 ? 256 : BN);
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
  // Everything above (barriers, tensor memory) touches nothing an earlier kernel writes, and
  // neither do the weights: the weight tiles of the first work item's first stages are
  // requested here, before the dependency wait, so that their way from DRAM overlaps the
  // kernel before; the activations of those stages follow after the wait.  From there on
  // activations, the residual stream and the split-k scratch are read.
  int pre = 0;                                  // stages whose weight tile is already requested
  if (threadIdx.x == 0 && (int)blockIdx.x < n_items) {
    const int tile = blockIdx.x / p.splits, split = blockIdx.x - tile * p.splits;
    const int n0 = (tile % p.tiles_n) * BN;
    const int kb0 = split * p.kb_per_split;
    pre = min(STAGES, min(kb0 + p.kb_per_split, num_kb) - kb0);
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(&full_bar[i], S::STAGE_BYTES);
      tma_load_2d(smem + i * S::STAGE_BYTES + S::A_BYTES, &map_w, &full_bar[i],
                  (kb0 + i) * TC_BK, n0);
    }
  }
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
          if ((int)it >= pre) {
            mbar_expect_tx(&full_bar[s], S::STAGE_BYTES);
            tma_load_2d(b_dst, &map_w, &full_bar[s], kb * TC_BK, n0);
          }
          tma_load_2d(a_dst, &map_a, &full_bar[s], kb * TC_BK, m0);
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
    uint8_t* patch = smem + S::PATCH_OFFSET + (warp - 4) * TC_PATCH_BYTES;
    uint32_t wi = 0;
    for (int w = blockIdx.x; w < n_items; w += gridDim.x, ++wi) {
      const int tile = w / p.splits, split = w - tile * p.splits;
      const int m0 = (tile / p.tiles_n) * TC_BM, n0 = (tile % p.tiles_n) * BN;
      const uint32_t acc = wi & 1, acc_round = wi >> 1;
      // the tile's bias goes to shared memory while the MMAs still run (two buffers: a warp
      // can be one tile ahead of the slowest at most, because of the barrier inside)
      float* bias_s = nullptr;
      if (!SPLIT && p.bias != nullptr) {
        bias_s = (float*)(smem + S::BIAS_OFFSET) + (wi & 1) * 256;
        stage_bias<BN>(p, bias_s, n0);
      }
      const uint32_t t_addr = tmem_base + acc * ACC_COLS + ((uint32_t)(q * 32) << 16);
      epilogue_columns<TO, HALF_COLS / 32, SPLIT>(p, &acc_full[acc], acc_round & 1, t_addr,
                                                  half * HALF_COLS, m0 + q * 32, n0, lane, patch,
                                                  bias_s, split);
      // the accumulator may be overwritten by the MMAs of the work item after next
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);

      if constexpr (SPLIT) {
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
          const int n_pieces = rows_here * PIECES;
          if (vec4 && p.splits <= 8) {
            // every load of a piece (shares, bias, residual) is on its way before the first sum
#pragma unroll 1
            for (int e = et; e < n_pieces; e += TC_EPI_WARPS * 32) {
              const int r = e / PIECES, n = n0 + (e % PIECES) * 4;
              if (n >= p.N) continue;
              const size_t off = (size_t)(m0 + r) * p.N + n;
              float4 sh[8];
#pragma unroll
              for (int sp = 0; sp < 8; ++sp)
                if (sp < p.splits)
                  sh[sp] = __ldcg((const float4*)(p.partial + (size_t)sp * p.M * p.N + off));
              float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f), r4 = b4;
              if (p.bias) b4 = __ldg((const float4*)(p.bias + n));
              if (p.residual) r4 = *(const float4*)(p.residual + off);
              float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
              for (int sp = 0; sp < 8; ++sp)
                if (sp < p.splits) {
                  a.x += sh[sp].x; a.y += sh[sp].y; a.z += sh[sp].z; a.w += sh[sp].w;
                }
              float x[4] = {a.x + b4.x, a.y + b4.y, a.z + b4.z, a.w + b4.w};
              if (p.act == HS_ACT_GELU_TANH) {
#pragma unroll
                for (int j = 0; j < 4; ++j) x[j] = act_tc(x[j], HS_ACT_GELU_TANH);
              } else if (p.act == HS_ACT_GELU_ERF) {
#pragma unroll
                for (int j = 0; j < 4; ++j) x[j] = act_tc(x[j], HS_ACT_GELU_ERF);
              }
              if (p.residual) {
                x[0] += r4.x; x[1] += r4.y; x[2] += r4.z; x[3] += r4.w;
              }
              if constexpr (sizeof(TO) == 4) {
                *(float4*)((float*)out + off) = make_float4(x[0], x[1], x[2], x[3]);
              } else {
                __nv_bfloat162 p0 = __floats2bfloat162_rn(x[0], x[1]);
                __nv_bfloat162 p1 = __floats2bfloat162_rn(x[2], x[3]);
                uint2 o;
                o.x = *(uint32_t*)&p0; o.y = *(uint32_t*)&p1;
                *(uint2*)((__nv_bfloat16*)out + off) = o;
              }
            }
          } else
          for (int e = et; e < n_pieces; e += TC_EPI_WARPS * 32) {
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
  static constexpr int PATCH_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BIAS_OFFSET = PATCH_OFFSET + TC_EPI_WARPS * TC_PATCH_BYTES;
  static constexpr int BAR_OFFSET = BIAS_OFFSET + 2 * 256 * 4;
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
    uint8_t* patch = smem + S::PATCH_OFFSET + (warp - 4) * TC_PATCH_BYTES;
    const uint32_t acc_empty_leader0 = cluster_map(&acc_empty[0], 0);
    const uint32_t acc_empty_leader1 = cluster_map(&acc_empty[1], 0);
    uint32_t wi = 0;
    for (int w = pair; w < n_items; w += n_pairs, ++wi) {
      const int m0 = (w / p.tiles_n) * (2 * TC_BM) + (int)rank * TC_BM;
      const int n0 = (w % p.tiles_n) * BN;
      const uint32_t acc = wi & 1, acc_round = wi >> 1;
      float* bias_s = nullptr;
      if (p.bias != nullptr) {
        bias_s = (float*)(smem + S::BIAS_OFFSET) + (wi & 1) * 256;
        stage_bias<BN>(p, bias_s, n0);
      }
      const uint32_t t_addr = tmem_base + acc * ACC_COLS + ((uint32_t)(q * 32) << 16);
      epilogue_columns<TO, HALF_COLS / 32, false>(p, &acc_full[acc], acc_round & 1, t_addr,
                                                  half * HALF_COLS, m0 + q * 32, n0, lane, patch,
                                                  bias_s, 0);
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
// ---------------------------------------------------------------------------------------------
// Few rows, deep layer: the k splits of a tile as a thread-block cluster.
//
// Tiles of 64 columns (few rows), 2..8 splits over k.  The CTAs of a cluster are
// the splits of one tile: each runs its k range into tensor memory as above, then the partial
// tiles are exchanged through distributed shared memory instead of scratch in global memory:
// the tile's rows are dealt to the CTAs of the cluster, every CTA sends each row of its partial
// to the row's owner (st.shared::cluster), one hardware cluster barrier follows, and each owner
// adds the shares of its rows in split order and applies bias, activation and residual.  No
// counters, no fences, and the last step is spread over all CTAs of the cluster (with scratch
// and a counter the last CTA to arrive swept the whole tile alone: 3.5 us of a 9.4 us launch
// at 64 x 3072 x 1024).
constexpr int CL_BN = 64, CL_STAGES = 6, CL_MAX_SPLITS = 8;

struct ClSmem {
  static constexpr int A_BYTES = TC_BM * TC_BK * 2;
  static constexpr int B_BYTES = CL_BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int RED_OFFSET = CL_STAGES * STAGE_BYTES;
  // [splits][rows per owner][64] floats; splits * rows per owner < 128 + splits
  static constexpr int RED_BYTES = (TC_BM + CL_MAX_SPLITS) * CL_BN * 4;
  static constexpr int BAR_OFFSET = RED_OFFSET + RED_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + (2 * CL_STAGES + 1) * 8 + 16 + 1024;
};

__device__ __forceinline__ void st_cluster_f4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                              uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b),
               "r"(c), "r"(d)
               : "memory");
}

template <typename TO>
__global__ void __launch_bounds__(TC_THREADS, 1)
linear_tcgen05_cluster_kernel(const __grid_constant__ CUtensorMap map_a,
                              const __grid_constant__ CUtensorMap map_w, const TcParams p) {
  using S = ClSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* red = (float*)(smem + S::RED_OFFSET);
  uint64_t* full_bar = (uint64_t*)(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + CL_STAGES;
  uint64_t* acc_full = empty_bar + CL_STAGES;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int splits = p.splits;                       // = the cluster's size
  const int rank = (int)cluster_ctarank();           // = this CTA's split
  const int tile = blockIdx.x / splits;
  const int m0 = (tile / p.tiles_n) * TC_BM, n0 = (tile % p.tiles_n) * CL_BN;
  const int num_kb = (p.K + TC_BK - 1) / TC_BK;
  const int kb0 = rank * p.kb_per_split;
  const int kb1 = min(kb0 + p.kb_per_split, num_kb);
  constexpr uint32_t TMEM_COLS = CL_BN;

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < CL_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
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
  // the weights do not change during a step: the first stages' weight tiles are requested
  // before the dependency wait
  int pre = 0;
  if (threadIdx.x == 0) {
    pre = min(CL_STAGES, kb1 - kb0);
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(&full_bar[i], S::STAGE_BYTES);
      tma_load_2d(smem + i * S::STAGE_BYTES + S::A_BYTES, &map_w, &full_bar[i],
                  (kb0 + i) * TC_BK, n0);
    }
  }
  // every CTA of the cluster has started: its shared memory may be written by the others
  __syncwarp();
  cluster_sync();
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer
      bool ok = true;
      for (int kb = kb0, it = 0; kb < kb1 && ok; ++kb, ++it) {
        const int s = it % CL_STAGES;
        const int round = it / CL_STAGES;
        if (round > 0) ok = mbar_wait(&empty_bar[s], (round - 1) & 1, p.status);
        if (!ok) break;
        uint8_t* a_dst = smem + s * S::STAGE_BYTES;
        if (it >= pre) {
          mbar_expect_tx(&full_bar[s], S::STAGE_BYTES);
          tma_load_2d(a_dst + S::A_BYTES, &map_w, &full_bar[s], kb * TC_BK, n0);
        }
        tma_load_2d(a_dst, &map_a, &full_bar[s], kb * TC_BK, m0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer
      constexpr uint32_t idesc = make_idesc(TC_BM, CL_BN);
      bool ok = true;
      for (int kb = kb0, it = 0; kb < kb1 && ok; ++kb, ++it) {
        const int s = it % CL_STAGES;
        ok = mbar_wait(&full_bar[s], (it / CL_STAGES) & 1, p.status);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * S::STAGE_BYTES);
        const uint64_t adesc = make_smem_desc(a_addr);
        const uint64_t bdesc = make_smem_desc(a_addr + S::A_BYTES);
#pragma unroll
        for (int k = 0; k < TC_BK / TC_UMMA_K; ++k)
          umma_bf16(tmem_base, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc,
                    (kb > kb0 || k > 0) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      umma_commit(acc_full);            // the partial tile is complete (or the pipeline gave up)
    }
  }

  // rows of the tile that exist, dealt to the CTAs of the cluster in blocks of `rpo`
  const int rows_here = min(TC_BM, p.M - m0);
  const int rpo = (rows_here + splits - 1) / splits;
  const int et = threadIdx.x - 4 * 32;                   // 0..255 among the epilogue threads
  // What this thread's first two output pieces need besides the sums - bias and residual - is
  // requested now, while the MMAs run: behind the cluster's barrier it would be a trip to the
  // L2 on the launch's critical path.
  constexpr int CL_PIECES = CL_BN / 4;
  constexpr int CL_EARLY = 2;
  const int cl_first = rank * rpo;
  const int cl_rows = max(0, min(rpo, rows_here - cl_first));
  const bool cl_vec4 = (p.N % 4 == 0);
  float4 early_b[CL_EARLY], early_r[CL_EARLY];
#pragma unroll
  for (int i = 0; i < CL_EARLY; ++i) {
    early_b[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    early_r[i] = early_b[i];
    const int e = et + i * TC_EPI_WARPS * 32;
    if (warp >= 4 && cl_vec4 && e < cl_rows * CL_PIECES) {
      const int lr = e / CL_PIECES, n = n0 + (e % CL_PIECES) * 4;
      if (n < p.N) {
        if (p.bias) early_b[i] = __ldg((const float4*)(p.bias + n));
        if (p.residual)
          early_r[i] = *(const float4*)(p.residual + (size_t)(m0 + cl_first + lr) * p.N + n);
      }
    }
  }
  if (warp >= 4) {
    // ---------------- send: warp (w % 4) owns TMEM lanes 32*(w%4) .. +31 = rows of the tile,
    // the two groups of four warps take the two halves of the 64 columns
    const int q = warp & 3, half = (warp - 4) >> 2;
    const int row = q * 32 + lane;
    if (mbar_wait(acc_full, 0, p.status)) {
      tc_fence_after();
      uint32_t v[32];
      tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + half * 32, v);
      tmem_ld_wait();
      if (row < rows_here) {
        const int owner = row / rpo, lr = row - owner * rpo;
        const uint32_t dst =
            cluster_map(red + ((size_t)(rank * rpo + lr) * CL_BN + half * 32), (uint32_t)owner);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          st_cluster_f4(dst + 16 * j, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      }
    }
    tc_fence_before();
  }
  // all shares have arrived everywhere (every thread of every CTA comes here, also after a
  // time-out, whose status bit tells the host that the result is not to be used)
  __syncwarp();
  cluster_sync();

  if (warp >= 4) {
    // ---------------- this CTA's rows: shares added in split order, then the epilogue
    const int my_first = cl_first;
    const int my_rows = cl_rows;
    TO* out = (TO*)p.out;
    const bool vec4 = cl_vec4;
    constexpr int PIECES = CL_PIECES;
    int it = 0;
    for (int e = et; e < my_rows * PIECES; e += TC_EPI_WARPS * 32, ++it) {
      const int lr = e / PIECES, c = (e % PIECES) * 4;
      const int n = n0 + c;
      if (n >= p.N) continue;
      const size_t off = (size_t)(m0 + my_first + lr) * p.N + n;
      float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f), r4 = b4;
      if (vec4) {
        if (it == 0) {
          b4 = early_b[0]; r4 = early_r[0];
        } else if (it == 1) {
          b4 = early_b[1]; r4 = early_r[1];
        } else {
          if (p.bias) b4 = __ldg((const float4*)(p.bias + n));
          if (p.residual) r4 = *(const float4*)(p.residual + off);
        }
      } else {
        float* bb = (float*)&b4;
        float* rr = (float*)&r4;
        for (int j = 0; j < 4; ++j)
          if (n + j < p.N) {
            if (p.bias) bb[j] = p.bias[n + j];
            if (p.residual) rr[j] = p.residual[off + j];
          }
      }
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int sp = 0; sp < splits; ++sp) {
        const float4 sh = *(const float4*)(red + ((size_t)(sp * rpo + lr) * CL_BN + c));
        a.x += sh.x; a.y += sh.y; a.z += sh.z; a.w += sh.w;
      }
      float x[4] = {a.x + b4.x, a.y + b4.y, a.z + b4.z, a.w + b4.w};
      if (p.act == HS_ACT_GELU_TANH) {
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = act_tc(x[j], HS_ACT_GELU_TANH);
      } else if (p.act == HS_ACT_GELU_ERF) {
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = act_tc(x[j], HS_ACT_GELU_ERF);
      }
      x[0] += r4.x; x[1] += r4.y; x[2] += r4.z; x[3] += r4.w;
      if (vec4) {
        if constexpr (sizeof(TO) == 4) {
          *(float4*)((float*)out + off) = make_float4(x[0], x[1], x[2], x[3]);
        } else {
          __nv_bfloat162 p0 = __floats2bfloat162_rn(x[0], x[1]);
          __nv_bfloat162 p1 = __floats2bfloat162_rn(x[2], x[3]);
          uint2 o;
          o.x = *(uint32_t*)&p0; o.y = *(uint32_t*)&p1;
          *(uint2*)((__nv_bfloat16*)out + off) = o;
        }
      } else {
        for (int j = 0; j < 4; ++j)
          if (n + j < p.N) out[off + j] = from_f<TO>(x[j]);
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

template <int BN, int STAGES, typename TO, bool SPLIT>
static int launch(const CUtensorMap& ma, const CUtensorMap& mw, const TcParams& p, int grid,
                  cudaStream_t st) {
  auto kern = linear_tcgen05_kernel<BN, STAGES, TO, SPLIT>;
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

template <typename TO>
static int launch_cluster(const CUtensorMap& ma, const CUtensorMap& mw, const TcParams& p,
                          int tiles, cudaStream_t st) {
  auto kern = linear_tcgen05_cluster_kernel<TO>;
  constexpr int smem = ClSmem::TOTAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * p.splits);
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.splits;
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
  bool cluster;      // the splits of a tile exchange their shares inside a cluster: no scratch
};

static bool g_split_clusters = true;


// How many clusters of `size` CTAs of the cluster kernel the device holds at once (asked once
// per size; 0: the question could not be asked).
static int cluster_capacity(int size) {
  static int cached[CL_MAX_SPLITS + 1] = {0};
  static bool asked[CL_MAX_SPLITS + 1] = {false};
  if (size < 1 || size > CL_MAX_SPLITS) return 0;
  if (asked[size]) return cached[size];
  asked[size] = true;
  auto kern = linear_tcgen05_cluster_kernel<float>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ClSmem::TOTAL) !=
      cudaSuccess)
    return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(size * 64);
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = ClSmem::TOTAL;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = size;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) n = 0;
  cached[size] = n;
  return n;
}

// pair: -1 = decide here, 0 = single CTAs, 1 = pairs of CTAs (256-row tiles)
static bool plan_tc(int M, int N, int K, int tile_n, int pair, TcPlan& pl) {
  int sms = 148;
  sms = hs_sm_count();
  const int mt = (M + TC_BM - 1) / TC_BM;
  const int num_kb = (K + TC_BK - 1) / TC_BK;
  // measured on B200: pairs gain 5-9 % from 4,096 rows on (4096^3, 8192^3) and nothing at 2,048
  pl.pair = pair == 1 || (pair < 0 && M >= 4096);
  pl.cluster = false;
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
    for (int cand : {256, 192, 128, 64}) {
      if (cand > 64 && cand / 2 >= N) continue;
      const long tiles = (long)mt * ((N + cand - 1) / cand);
      const long cost = ((tiles + sms - 1) / sms) * (cand + 128 + 64);
      if (best < 0 || cost < best) {
        best = cost;
        bn = cand;
      }
    }
    // few rows: narrow tiles (more CTAs stream the weights) and splits; a very wide layer (the
    // vocabulary) has tiles enough and reads the activations less often with 128 columns
    if (mt == 1) bn = ((N + 63) / 64 >= 2 * sms) ? 128 : 64;
  }
  if (bn != 64 && bn != 128 && bn != 192 && bn != 256) return false;
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
    // 64-column tiles split over k: the splits of a tile form a cluster, as many as the device
    // holds at once for all tiles.  A cluster that has to wait for the next round costs more than
    // its splits save: of this kernel 74 clusters of two fit, 45 of three, 33 of four, 22 of
    // six, 15 of eight, so 48 tiles take two splits and 16 tiles six.  Measured in a decode
    // step of GPT-2 medium at batch 32: 1.23 ms, against 1.53 ms with the shares going through
    // scratch memory (3, 8, 2 and 8 splits).
    if (g_split_clusters && bn == CL_BN) {
      int pick = 0;
      for (int cand = 2; cand <= splits && cand <= CL_MAX_SPLITS; ++cand)
        if (cluster_capacity(cand) >= tiles) pick = cand;
      if (pick) {
        pl.cluster = true;
        splits = pick;
      }
    }
  }
  pl.kb_per_split = (num_kb + splits - 1) / splits;
  pl.splits = (num_kb + pl.kb_per_split - 1) / pl.kb_per_split;
  if (pl.splits < 2) pl.cluster = false;
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
  const bool scratch = pl.splits > 1 && !pl.cluster;
  *floats = scratch ? (long long)pl.splits * M * N : 0;
  *counters = scratch ? pl.tiles_m * pl.tiles_n : 0;
  return HS_OK;
}

// Few rows split over k: the splits of a tile as a thread-block cluster that exchanges the
// shares through distributed shared memory (on, the default), or through scratch memory and a
// counter.  Scratch sizes depend on it: ask hs_linear_tcgen05_scratch again after a change.
HS_EXPORT void hs_set_split_clusters(int on) { hs::g_split_clusters = on != 0; }

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
  if (pl.splits > 1 && !pl.cluster && (!scratch || !counters)) return HS_ERR_ARGUMENT;
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
#define HS_TC(BN, ST)                                                                      \
  (pl.splits > 1                                                                           \
       ? (out_dtype == HS_DT_F32 ? launch<BN, ST, float, true>(ma, mw, p, pl.grid, st)     \
                                 : launch<BN, ST, bf16, true>(ma, mw, p, pl.grid, st))     \
       : (out_dtype == HS_DT_F32 ? launch<BN, ST, float, false>(ma, mw, p, pl.grid, st)    \
                                 : launch<BN, ST, bf16, false>(ma, mw, p, pl.grid, st)))
  if (pl.cluster)
    return out_dtype == HS_DT_F32
               ? launch_cluster<float>(ma, mw, p, pl.tiles_m * pl.tiles_n, st)
               : launch_cluster<bf16>(ma, mw, p, pl.tiles_m * pl.tiles_n, st);
  if (pl.pair) {
    if (pl.bn == 256)
      return out_dtype == HS_DT_F32 ? launch_pair<256, 6, float>(ma, mw, p, pl.grid, st)
                                    : launch_pair<256, 6, bf16>(ma, mw, p, pl.grid, st);
    return out_dtype == HS_DT_F32 ? launch_pair<128, 8, float>(ma, mw, p, pl.grid, st)
                                  : launch_pair<128, 8, bf16>(ma, mw, p, pl.grid, st);
  }
  switch (pl.bn) {
    case 256: return HS_TC(256, 4);
    case 192: return HS_TC(192, 5);
    case 128: return HS_TC(128, 6);
    default: return HS_TC(64, 8);
  }
#undef HS_TC
}
