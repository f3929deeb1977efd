// bfloat16 linear layer for few rows (M <= 64: decoding), bound by streaming the weights.
//
//   out[m, n] = act( sum_k a[m, k] * w[n, k] + bias[n] ) (+ residual[m, n])
//   a = the bfloat16 input, or LayerNorm(x) of a float32 input computed on the fly.
//
// With M this small a 128-row tensor-core tile would be nearly empty and only N/128 CTAs would
// stream the weights.  Here the roles are swapped: a warp owns 16 output features, the weights
// are the row operand of mma.sync m16n8k16 and the (few) tokens are the 8-wide column operand.
// Each lane loads 16 bytes (8 consecutive k) of two weight rows straight from global memory into
// the registers of two MMA k-steps — the k order inside a 32-wide block is permuted the same way
// for both operands, which a dot product allows — so the weights are read once, fully coalesced,
// with no shared-memory round trip.  The activations (M_pad x K, bfloat16) sit in shared memory,
// padded so that the 16-byte fragment reads are conflict-free.  A CTA = 8 warps owns 16 features
// (up to 128 for a wide layer such as the vocabulary head, so that the activations are staged
// less often); its warps take the 32-wide k blocks round-robin and their partial tiles are added
// in warp order.  Narrow, deep layers are also split over k between CTAs: each writes its share
// to scratch memory and the last to arrive (a counter in scratch) adds the shares in split
// order.  Every order is fixed, there are no floating-point atomics; then bias, activation
// and the float32 residual are applied.
//
// Optional fused LayerNorm (the reference's `F.layer_norm` before each projection,
// heteroserve/model/torch_engine.py:74-75,121,140): every CTA normalises the M rows itself
// (statistics in float32: mean, then centred variance) while it stages them.
#include "common.cuh"

namespace hs {

constexpr int SK_FEATS = 16;

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct SkinnyParams {
  const __nv_bfloat16* a;      // [M, K] bf16, or null when x is given
  const float* x;              // [M, K] f32 to be normalised, or null
  const float* gamma;
  const float* beta;
  const __nv_bfloat16* w;      // [N, K]
  const float* bias;
  const float* residual;
  void* out;
  float* partial;              // [ksplit][MP][N] float32 scratch (ksplit > 1)
  int* counters;               // one per feature block, zero between launches (ksplit > 1)
  int M, N, K, act, out_f32;
  int kper, stride;            // k per CTA (multiple of 32); smem row stride in elements
  int red_offset;              // bytes from the start of shared memory to the reduction tiles
  int ng;                      // feature groups (of 16) per feature block: 1, 2, 4 or 8
  float eps;
  unsigned long long* timing;  // null, or the tuning buffer (see mark_time)
};

// What the kernels with the greedy choice fused in (ARGMAX) take besides: every CTA leaves its
// best (value, index) per row, the last one to arrive picks each row's token (lowest index on
// ties).  The other kernels' parameters stay as they are.
struct SkinnyArgmaxParams : SkinnyParams {
  int* tokens;                 // [M] chosen tokens, then one word for the status
  int* feedback;               // or null: row m's token also goes to feedback[feedback_slot[m]]
  const int* feedback_slot;
  const int* status_word;      // or null: its value is stored to tokens[M]
  float* am_val;               // [grid][MP] scratch
  int* am_idx;                 // [grid][MP] scratch
  int* am_counter;             // zero between launches
};
template <bool ARGMAX> struct SkinnyParamsOf { using type = SkinnyParams; };
template <> struct SkinnyParamsOf<true> { using type = SkinnyArgmaxParams; };

struct WBatch {
  uint4 a[4], b[4];
};

// A warp's partial tile in shared memory: [row of the batch][feature], 17 floats a row, so that
// the epilogue's threads (consecutive features of one row) read consecutive words and the
// writers' lanes spread over the banks.  (As [feature][row] a read of 16-row tiles hit two banks:
// 1 us of a 7.5 us launch at 16 rows.)
constexpr int SK_RED_ROW = 17;
constexpr int SK_LN_ROW_F4 = 8;       // a row of up to 8 * 128 = 1024 floats is normalised from registers
                                      // two rows at a time, up to 2048 floats one row at a time;
                                      // longer rows take the three-pass route

// LayerNorm from registers: a warp reads a whole row once (F4 float4 per lane: rows of up to
// F4 * 128 floats), forms the mean and the centred variance, and writes the normalised k range
// of this CTA to shared memory.  A warp takes rows warp, warp + NW, ...; the loads of TOGETHER
// rows are in flight at once.
template <int MP, int NW, int F4, int TOGETHER>
__device__ __forceinline__ void ln_rows_from_registers(const float* __restrict__ x, int K, int M,
                                                       int stride, float eps, __nv_bfloat16* sx,
                                                       const float* sgb, int k0, int kn, int warp,
                                                       int lane) {
  constexpr int RPW = (MP + NW - 1) / NW;                // rows per warp
  const int nf4 = K / 4;
#pragma unroll
  for (int r0 = 0; r0 < RPW; r0 += TOGETHER) {
    float4 xr[TOGETHER][F4];
    int rows[TOGETHER];
#pragma unroll
    for (int j = 0; j < TOGETHER; ++j) {
      rows[j] = warp + (r0 + j) * NW;
      const bool live = (r0 + j) < RPW && rows[j] < M;
      const float4* src = (const float4*)(x + (size_t)(live ? rows[j] : 0) * K);
#pragma unroll
      for (int i = 0; i < F4; ++i)
        xr[j][i] = (live && lane + 32 * i < nf4) ? src[lane + 32 * i]
                                                 : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < TOGETHER; ++j) {
      const int m = rows[j];
      if ((r0 + j) >= RPW || m >= MP) continue;
      if (m < M) {
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < F4; ++i)
          sum += (xr[j][i].x + xr[j][i].y) + (xr[j][i].z + xr[j][i].w);
        const float mu = warp_sum(sum) / (float)K;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < F4; ++i) {
          if (lane + 32 * i < nf4) {
            const float c0 = xr[j][i].x - mu, c1 = xr[j][i].y - mu, c2 = xr[j][i].z - mu,
                        c3 = xr[j][i].w - mu;
            q += (c0 * c0 + c1 * c1) + (c2 * c2 + c3 * c3);
          }
        }
        const float rs = 1.0f / sqrtf(warp_sum(q) / (float)K + eps);
#pragma unroll
        for (int i = 0; i < F4; ++i) {
          const int kk = (lane + 32 * i) * 4 - k0;        // column inside this CTA's k range
          if (lane + 32 * i < nf4 && kk >= 0 && kk < kn) {
            const float4 ga = *(const float4*)(sgb + kk), be = *(const float4*)(sgb + kn + kk);
            __nv_bfloat162 o0 = __floats2bfloat162_rn((xr[j][i].x - mu) * rs * ga.x + be.x,
                                                      (xr[j][i].y - mu) * rs * ga.y + be.y);
            __nv_bfloat162 o1 = __floats2bfloat162_rn((xr[j][i].z - mu) * rs * ga.z + be.z,
                                                      (xr[j][i].w - mu) * rs * ga.w + be.w);
            uint2 v;
            v.x = *(uint32_t*)&o0; v.y = *(uint32_t*)&o1;
            *(uint2*)(sx + (size_t)m * stride + kk) = v;
          }
        }
      } else {
        for (int kk = lane * 4; kk < kn; kk += 128)
          *(uint2*)(sx + (size_t)m * stride + kk) = make_uint2(0, 0);
      }
    }
  }
}

struct SkBest {
  float v;
  int i;
};
__device__ __forceinline__ SkBest sk_better(SkBest a, SkBest b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ SkBest sk_warp_best(SkBest b) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    SkBest other{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
    b = sk_better(b, other);
  }
  return b;
}

// NW warps per CTA: 8, or 16 for deep layers (more 32-wide k blocks in flight per feature group).
// The kernel is compiled once per way it is used, because a launch of a few microseconds
// begins with cold instruction caches: code of paths a launch does not take, lying between the
// blocks it runs, measured 0.3 us per launch (one more inlined LayerNorm route made a decode
// step of 96 such launches 1 % slower).
//   LOOP:  a CTA may walk several feature blocks (the partial tiles then lie beside the
//          activations instead of over them).
//   LN:    0 bfloat16 activations, no norm; 1 / 2 LayerNorm of rows up to 1024 / 2048 floats
//          from registers; 3 longer rows, three passes; -1 decided when it runs.
//   SPLIT: 0 never split over k between CTAs; -1 decided when it runs.
template <int MT, int NW, bool LOOP, bool ARGMAX = false, int LN = -1, int SPLIT = -1>
__global__ void __launch_bounds__(NW * 32)
linear_skinny_kernel(const typename SkinnyParamsOf<ARGMAX>::type p) {
  constexpr int MP = MT * 8;
  constexpr int THREADS = NW * 32;
  extern __shared__ __align__(16) uint8_t sk_smem[];
  __nv_bfloat16* sx = (__nv_bfloat16*)sk_smem;             // [MP][stride]
  float* sgb = (float*)(sk_smem + (size_t)MP * p.stride * 2);   // gamma | beta of the k range
  __shared__ float s_mu[MP], s_rs[MP];
  __shared__ int s_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  // warp -> (feature group, k group): ng groups of 16 features, NW / ng warps share each
  const int fg = warp % p.ng, kg = warp / p.ng, n_kg = NW / p.ng;
  const int K = p.K, M = p.M;
  const int ksplit = SPLIT == 0 ? 1 : (int)gridDim.y;
  const bool has_norm = LN < 0 ? p.x != nullptr : LN > 0;
  const int k0 = blockIdx.y * p.kper;
  const int kn = min(p.kper, K - k0);                       // may be <= 0 for the last splits
  const int nblk = kn > 0 ? kn / 32 : 0;
  const int feats = 16 * p.ng;
  // A CTA walks the feature blocks blockIdx.x, blockIdx.x + gridDim.x, ... (more than one only
  // when the layer has more blocks than CTAs fit the GPU at once: the activations are staged
  // and normalised once, and the last blocks do not wait for a second round of CTAs).
  const int n_fblocks = (p.N + feats - 1) / feats;
  int fb = blockIdx.x;
  const __nv_bfloat16 *wa, *wb;
  auto point_at = [&](int block) {
    const int n0 = (block * p.ng + fg) * SK_FEATS;
    const int row_a = min(n0 + g, p.N - 1), row_b = min(n0 + g + 8, p.N - 1);   // clamped: never stored
    wa = p.w + (size_t)row_a * K + k0 + t * 8;
    wb = p.w + (size_t)row_b * K + k0 + t * 8;
  };
  point_at(fb);
  auto load_batch = [&](int b, WBatch& wbt) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int blk = b + u * n_kg;
      if (blk < nblk) {
        wbt.a[u] = ld_stream16(wa + blk * 32);
        wbt.b[u] = ld_stream16(wb + blk * 32);
      }
    }
  };
  // ---- before the previous kernel is waited for: everything that only reads parameters.
  // The first weight fragments, the bias of this thread's output element, the norm's scale and
  // shift for this CTA's k range.
  const int cta_id = blockIdx.y * gridDim.x + blockIdx.x;
  mark_time(p.timing, cta_id, 0);
  WBatch cur;
  load_batch(kg, cur);
  const int my_e = threadIdx.x;                              // first epilogue element of this thread
  const int my_n = blockIdx.x * feats + (my_e % feats);
  float my_bias = 0.f;
  if (p.bias && my_e < feats * MP && my_n < p.N) my_bias = p.bias[my_n];
  if (has_norm && kn > 0) {
    for (int i = threadIdx.x; i < kn / 4; i += THREADS) {
      ((float4*)sgb)[i] = ((const float4*)(p.gamma + k0))[i];
      ((float4*)(sgb + kn))[i] = ((const float4*)(p.beta + k0))[i];
    }
  }
  pdl_trigger();      // the next kernel may begin its own parameter fetch
  pdl_wait();         // from here on what the previous kernels wrote is read
  mark_time(p.timing, cta_id, 1);

  // the residual element of this thread, requested early so that the epilogue does not wait
  float my_res = 0.f;
  const int my_m = my_e / feats;
  if (p.residual && my_e < feats * MP && my_m < M && my_n < p.N && ksplit == 1)
    my_res = p.residual[(size_t)my_m * p.N + my_n];

  if (has_norm) {
    const int ln_route =
        LN > 0 ? LN : (K <= SK_LN_ROW_F4 * 128 ? 1 : (K <= 2 * SK_LN_ROW_F4 * 128 ? 2 : 3));
    if (ln_route == 1) {
      __syncthreads();                                       // gamma/beta are in shared memory
      ln_rows_from_registers<MP, NW, SK_LN_ROW_F4, 2>(p.x, K, M, p.stride, p.eps, sx, sgb, k0, kn,
                                                      warp, lane);
    } else if (ln_route == 2) {
      __syncthreads();
      ln_rows_from_registers<MP, NW, 2 * SK_LN_ROW_F4, 1>(p.x, K, M, p.stride, p.eps, sx, sgb, k0,
                                                          kn, warp, lane);
    } else {
      // long rows: statistics in two passes over global memory, then staging
      for (int m = warp; m < MP; m += NW) {
        float mu = 0.f, rs = 0.f;
        if (m < M) {
          const float4* xr = (const float4*)(p.x + (size_t)m * K);
          float sum = 0.f;
#pragma unroll 8
          for (int k = lane; k < K / 4; k += 32) {
            const float4 v = xr[k];
            sum += (v.x + v.y) + (v.z + v.w);
          }
          mu = warp_sum(sum) / (float)K;
          float q = 0.f;
#pragma unroll 8
          for (int k = lane; k < K / 4; k += 32) {
            const float4 v = xr[k];
            const float c0 = v.x - mu, c1 = v.y - mu, c2 = v.z - mu, c3 = v.w - mu;
            q += (c0 * c0 + c1 * c1) + (c2 * c2 + c3 * c3);
          }
          rs = 1.0f / sqrtf(warp_sum(q) / (float)K + p.eps);
        }
        if (lane == 0) {
          s_mu[m] = mu;
          s_rs[m] = rs;
        }
      }
      __syncthreads();
      if (kn > 0) {
#pragma unroll 4
        for (int i = threadIdx.x; i < MP * (kn / 4); i += THREADS) {
          const int m = i / (kn / 4), kk = (i % (kn / 4)) * 4;
          uint2 v = make_uint2(0, 0);
          if (m < M) {
            const float4 x0 = *(const float4*)(p.x + (size_t)m * K + k0 + kk);
            const float4 ga = *(const float4*)(sgb + kk), be = *(const float4*)(sgb + kn + kk);
            const float mu = s_mu[m], rs = s_rs[m];
            __nv_bfloat162 o0 = __floats2bfloat162_rn((x0.x - mu) * rs * ga.x + be.x,
                                                      (x0.y - mu) * rs * ga.y + be.y);
            __nv_bfloat162 o1 = __floats2bfloat162_rn((x0.z - mu) * rs * ga.z + be.z,
                                                      (x0.w - mu) * rs * ga.w + be.w);
            v.x = *(uint32_t*)&o0; v.y = *(uint32_t*)&o1;
          }
          *(uint2*)(sx + (size_t)m * p.stride + kk) = v;
        }
      }
    }
  } else if (kn > 0) {
    // ---- stage this CTA's k range of the bfloat16 activations [MP][kn] (rows past M are zero)
    // by 16-byte cp.async copies, all in flight together (through registers, four at a time,
    // 16 rows of a 4,096-wide layer were four trips to the L2: 3.0 us; eight rows 1.3 us)
    for (int i = threadIdx.x; i < MP * (kn / 8); i += THREADS) {
      const int m = i / (kn / 8), kk = (i % (kn / 8)) * 8;
      __nv_bfloat16* dst = sx + (size_t)m * p.stride + kk;
      if (m < M) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                         (uint32_t)__cvta_generic_to_shared(dst)),
                     "l"(p.a + (size_t)m * K + k0 + kk)
                     : "memory");
      } else {
        *(uint4*)dst = make_uint4(0, 0, 0, 0);
      }
    }
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
  }
  __syncthreads();
  mark_time(p.timing, cta_id, 2);

  float* red = (float*)(sk_smem + (LOOP ? p.red_offset : 0));   // [NW][MP][SK_RED_ROW]
  // output elements of a feature block per thread: up to 128 features x MP rows over the CTA
  constexpr int SLOTS = (128 * MP + THREADS - 1) / THREADS;
  float best_v[ARGMAX ? SLOTS : 1];
  int best_i[ARGMAX ? SLOTS : 1];
#pragma unroll
  for (int j = 0; j < (ARGMAX ? SLOTS : 1); ++j) {
    best_v[j] = -INFINITY;
    best_i[j] = 0x7fffffff;
  }
  for (;;) {
  float c[MT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
  // ---- this warp's 32-wide k blocks, four per batch, the next batch in flight meanwhile
  for (int b = kg; b < nblk; b += n_kg * 4) {
    WBatch nxt;
    load_batch(b + n_kg * 4, nxt);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int blk = b + u * n_kg;
      if (blk < nblk) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint4 xb = *(const uint4*)(sx + (size_t)(mt * 8 + g) * p.stride + blk * 32 + t * 8);
          mma16816(c[mt], cur.a[u].x, cur.b[u].x, cur.a[u].y, cur.b[u].y, xb.x, xb.y);
          mma16816(c[mt], cur.a[u].z, cur.b[u].z, cur.a[u].w, cur.b[u].w, xb.z, xb.w);
        }
      }
    }
    cur = nxt;
  }
  // the next feature block's first weights are requested before this block's sums are formed
  const int this_fb = fb;
  fb += gridDim.x;
  const bool more = LOOP && fb < n_fblocks;
  if (more) {
    point_at(fb);
    load_batch(kg, cur);
  }
  // ---- add the warps' partial tiles in warp order
  __syncthreads();                 // (also: the block before is done reading `red`)
  mark_time(p.timing, cta_id, 3);
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int m = mt * 8 + t * 2;
    red[(warp * MP + m) * SK_RED_ROW + g] = c[mt][0];
    red[(warp * MP + m + 1) * SK_RED_ROW + g] = c[mt][1];
    red[(warp * MP + m) * SK_RED_ROW + g + 8] = c[mt][2];
    red[(warp * MP + m + 1) * SK_RED_ROW + g + 8] = c[mt][3];
  }
  __syncthreads();
  if (ksplit > 1) {
    // this CTA's share goes to scratch; the last CTA of the feature block to arrive adds the
    // shares in split order
    float* mine = p.partial + (size_t)blockIdx.y * MP * p.N;
    for (int i = threadIdx.x; i < feats * MP; i += THREADS) {
      const int m = i / feats, ff = i % feats;
      const int n = this_fb * feats + ff;
      if (n >= p.N) continue;
      const int grp = ff / 16, f = ff % 16;
      float v = 0.f;
      for (int k8 = 0; k8 < n_kg; ++k8) v += red[((k8 * p.ng + grp) * MP + m) * SK_RED_ROW + f];
      mine[(size_t)m * p.N + n] = v;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&p.counters[this_fb], 1) == ksplit - 1;
    __syncthreads();
    if (!s_last) return;           // split launches have one feature block per CTA
    __threadfence();
  }
  const bool first_fb = this_fb == (int)blockIdx.x;
  if constexpr (!ARGMAX) {
  for (int i = threadIdx.x; i < feats * MP; i += THREADS) {
    const int m = i / feats, ff = i % feats;             // consecutive threads -> consecutive n
    const int n = this_fb * feats + ff;
    if (m >= M || n >= p.N) continue;
    float v = 0.f;
    if (ksplit > 1) {
      for (int ks = 0; ks < ksplit; ++ks)
        v += __ldcg(p.partial + ((size_t)ks * MP + m) * p.N + n);
    } else {
      const int grp = ff / 16, f = ff % 16;
      for (int k8 = 0; k8 < n_kg; ++k8) v += red[((k8 * p.ng + grp) * MP + m) * SK_RED_ROW + f];
    }
    const bool first = first_fb && i == my_e;            // bias (and residual) already in registers
    if (p.bias) v += first ? my_bias : p.bias[n];
    v = apply_act(v, p.act);
    if (p.residual) v += (first && ksplit == 1) ? my_res : p.residual[(size_t)m * p.N + n];
    if (p.out_f32) ((float*)p.out)[(size_t)m * p.N + n] = v;
    else ((__nv_bfloat16*)p.out)[(size_t)m * p.N + n] = __float2bfloat16_rn(v);
  }
  } else {
    // the head with the greedy choice: no split, bias, activation or residual.  Slot j of this
    // thread is the same row in every feature block, and n only rises from block to block:
    // the first seen wins ties
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
      const int i = threadIdx.x + j * THREADS;
      const int m = i / feats, ff = i % feats;
      const int n = this_fb * feats + ff;
      if (i < feats * MP && m < M && n < p.N) {
        const int grp = ff / 16, f = ff % 16;
        float v = 0.f;
        for (int k8 = 0; k8 < n_kg; ++k8) v += red[((k8 * p.ng + grp) * MP + m) * SK_RED_ROW + f];
        ((float*)p.out)[(size_t)m * p.N + n] = v;
        if (v > best_v[j] || best_i[j] == 0x7fffffff) {
          best_v[j] = v;
          best_i[j] = n;
        }
      }
    }
  }
  if (ksplit > 1 && threadIdx.x == 0) p.counters[this_fb] = 0;   // ready for the next launch
  if (!more) break;
  }
  if constexpr (ARGMAX) {
    // the CTA's best per row, through the partial tiles' place: [feats * MP] values | indices
    __syncthreads();
    float* cv = red;
    int* ci = (int*)(red + feats * MP);
#pragma unroll
    for (int j = 0; j < SLOTS; ++j) {
      const int i = threadIdx.x + j * THREADS;
      if (i < feats * MP) {
        cv[i] = best_v[j];
        ci[i] = best_i[j];
      }
    }
    __syncthreads();
    for (int m = warp; m < M; m += NW) {
      SkBest b{-INFINITY, 0x7fffffff};
      for (int ff = lane; ff < feats; ff += 32) b = sk_better(b, SkBest{cv[m * feats + ff], ci[m * feats + ff]});
      b = sk_warp_best(b);
      if (lane == 0) {
        p.am_val[(size_t)blockIdx.x * MP + m] = b.v;
        p.am_idx[(size_t)blockIdx.x * MP + m] = b.i;
      }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(p.am_counter, 1) == (int)gridDim.x - 1;
    __syncthreads();
    if (s_last) {
      __threadfence();
      for (int m = warp; m < M; m += NW) {
        SkBest b{-INFINITY, 0x7fffffff};
        // eight candidates per lane requested together, then folded
        for (int c0 = 0; c0 < (int)gridDim.x; c0 += 32 * 8) {
          float cvv[8];
          int cii[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int cta = c0 + u * 32 + lane;
            const bool ok = cta < (int)gridDim.x;
            cvv[u] = ok ? __ldcg(p.am_val + (size_t)cta * MP + m) : -INFINITY;
            cii[u] = ok ? __ldcg(p.am_idx + (size_t)cta * MP + m) : 0x7fffffff;
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) b = sk_better(b, SkBest{cvv[u], cii[u]});
        }
        b = sk_warp_best(b);
        if (lane == 0) {
          const int tok = b.i == 0x7fffffff ? 0 : b.i;
          p.tokens[m] = tok;
          const int fbk = (p.feedback && p.feedback_slot) ? p.feedback_slot[m] : -1;
          if (fbk >= 0) p.feedback[fbk] = tok;
        }
      }
      if (threadIdx.x == 0) {
        if (p.status_word) p.tokens[M] = *p.status_word;
        *p.am_counter = 0;                               // ready for the next launch
      }
    }
  }
  mark_time(p.timing, cta_id, 4);
}

template <int MT, int NW, bool LOOP, bool ARGMAX = false, int LN = -1, int SPLIT = -1>
static int launch_skinny_as(const typename SkinnyParamsOf<ARGMAX>::type& p, int grid_x, int ksplit,
                            size_t smem, cudaStream_t st, bool pdl) {
  auto kern = linear_skinny_kernel<MT, NW, LOOP, ARGMAX, LN, SPLIT>;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  dim3 grid(grid_x, ksplit);
  cudaError_t le = hs_launch(kern, grid, dim3(NW * 32), smem, st, pdl, p);
  if (le != cudaSuccess) return (int)le;
  HS_LAUNCH_CHECK();
  return HS_OK;
}

// One feature block per CTA (split over k or not), or CTAs that walk several.
template <int MT, int NW, int LN>
static int launch_skinny_mode(const SkinnyParams& p, int grid_x, int blocks, int ksplit,
                              size_t smem, size_t smem_loop, cudaStream_t st, bool pdl) {
  if (grid_x < blocks)
    return launch_skinny_as<MT, NW, true, false, LN, 0>(p, grid_x, 1, smem_loop, st, pdl);
  if constexpr (NW == 8) {          // the 16-warp shapes are never split
    if (ksplit > 1)
      return launch_skinny_as<MT, NW, false, false, LN, -1>(p, grid_x, ksplit, smem, st, pdl);
  }
  return launch_skinny_as<MT, NW, false, false, LN, 0>(p, grid_x, 1, smem, st, pdl);
}

// Up to 16 rows (decode): a kernel per norm route.  More rows: one kernel that decides as it runs.
template <int MT, int NW>
static int launch_skinny(const SkinnyParams& p, int grid_x, int blocks, int ksplit, size_t smem,
                         size_t smem_loop, cudaStream_t st, bool pdl) {
  if constexpr (MT > 2) {
    return launch_skinny_mode<MT, NW, -1>(p, grid_x, blocks, ksplit, smem, smem_loop, st, pdl);
  } else {
    const int route =
        !p.x ? 0 : (p.K <= SK_LN_ROW_F4 * 128 ? 1 : (p.K <= 2 * SK_LN_ROW_F4 * 128 ? 2 : 3));
    switch (route) {
      case 0: return launch_skinny_mode<MT, NW, 0>(p, grid_x, blocks, ksplit, smem, smem_loop, st, pdl);
      case 1: return launch_skinny_mode<MT, NW, 1>(p, grid_x, blocks, ksplit, smem, smem_loop, st, pdl);
      case 2: return launch_skinny_mode<MT, NW, 2>(p, grid_x, blocks, ksplit, smem, smem_loop, st, pdl);
      default: return launch_skinny_mode<MT, NW, 3>(p, grid_x, blocks, ksplit, smem, smem_loop, st, pdl);
    }
  }
}

struct SkinnyPlan {
  int mt, mp, ng, nw, ksplit, kper, stride, blocks, red_offset;
  int grid_x;            // CTAs along the features: the blocks, or as many as fit the GPU at once
  size_t smem;           // activations (+ norm parameters), the partial tiles over them
  size_t smem_loop;      // the partial tiles beside them (grid_x < blocks)
};

// How a shape is cut: features per CTA, warps per CTA, splits over k, shared memory.  Returns
// false for shapes the kernel does not take.
static bool plan_skinny(int M, int N, int K, bool with_norm, SkinnyPlan& pl) {
  if (M <= 0 || M > 64 || K <= 0 || K % 32) return false;
  pl.mt = M <= 8 ? 1 : (M <= 16 ? 2 : (M <= 32 ? 4 : 8));
  pl.mp = pl.mt * 8;
  int sms = 148;
  sms = hs_sm_count();
  // more features per feature block (fewer reductions and barriers per weight byte) while
  // every CTA of a full GPU (two per SM) still walks five blocks or more, so that the last
  // round of blocks is a small part of a CTA's work
  pl.ng = 1;
  while (pl.ng < 8 && (N + 32 * pl.ng - 1) / (32 * pl.ng) >= 5 * sms) pl.ng *= 2;
  pl.blocks = (N + 16 * pl.ng - 1) / (16 * pl.ng);
  auto smem_for = [&](int kper, int& stride) {
    stride = kper + ((32 - kper % 64) + 64) % 64;             // stride % 64 == 32
    if (stride % 64 != 32) stride += 32;
    // activations | the norm's scale and shift; the warps' partial tiles (up to 16 warps) over
    // them, or behind them when a CTA walks several feature blocks
    size_t sm = (size_t)pl.mp * stride * 2 + (with_norm ? (size_t)kper * 8 : 0);
    sm = (sm + 15) / 16 * 16;
    const size_t red = (size_t)16 * SK_RED_ROW * pl.mp * 4;
    pl.red_offset = (int)sm;
    pl.smem_loop = sm + red;
    return sm > red ? sm : red;
  };
  // Deep layers (k >= 2048) whose feature blocks alone leave SMs idle: 16 warps per CTA and
  // the whole k range in one CTA if its activations fit shared memory - no scratch round trip.
  pl.nw = 8;
  // CTAs along the features: every block its own CTA while they all fit the GPU at once (two
  // CTAs of 8 warps per SM by registers, fewer by shared memory; one of 16 warps), else that
  // many CTAs, each walking several blocks.  Split launches keep a CTA per block.
  auto finish = [&]() {
    int per_sm = pl.nw == 16 ? 1 : 2;
    const int by_smem = (int)((227 * 1024) / (pl.smem_loop + 1024));
    if (by_smem < per_sm) per_sm = by_smem < 1 ? 1 : by_smem;
    const int slots = per_sm * sms;
    pl.grid_x = (pl.ksplit > 1 || pl.blocks <= slots) ? pl.blocks : slots;
    return true;
  };
  int stride = 0;
  if (K >= 2048 && pl.ng == 1 && pl.mt <= 2 && smem_for(K, stride) <= 200 * 1024) {
    pl.nw = 16;
    pl.ksplit = 1;
    pl.kper = K;
    pl.stride = stride;
    pl.smem = smem_for(K, stride);
    return finish();
  }
  // 9-16 rows with the LayerNorm fused in, more feature blocks than SMs: 16 warps per CTA and
  // two feature groups, so that a warp normalises one row instead of two and one round of CTAs
  // covers the layer (a decode step at batch 16: 0.92 ms against 0.97).
  if (pl.mt == 2 && with_norm && pl.ng == 1 && K <= SK_LN_ROW_F4 * 128 && pl.blocks > sms) {
    pl.ng = 2;
    pl.blocks = (N + 31) / 32;
    pl.nw = 16;
    pl.ksplit = 1;
    pl.kper = K;
    pl.smem = smem_for(K, pl.stride);
    return finish();
  }
  // otherwise: k per CTA at most what fits ~96 KB of shared memory, at least 1024 (four blocks
  // a warp), and few enough splits that about two CTAs per SM are in flight
  const size_t budget = 96 * 1024;
  int kc = (int)(budget / (2 * (size_t)pl.mp + (with_norm ? 8 : 0))) - 64;
  kc = kc / 32 * 32;
  if (kc < 256) return false;
  int want = (2 * sms + pl.blocks - 1) / pl.blocks;
  int by_size = K / 1024 > 0 ? K / 1024 : 1;
  int ksplit = want < by_size ? want : by_size;
  const int need = (K + kc - 1) / kc;
  if (ksplit < need) ksplit = need;
  if (ksplit < 1) ksplit = 1;
  pl.kper = ((K / 32 + ksplit - 1) / ksplit) * 32;
  pl.ksplit = (K + pl.kper - 1) / pl.kper;
  pl.smem = smem_for(pl.kper, pl.stride);
  return finish();
}

}  // namespace hs

// Scratch a launch needs: floats for the partial sums and ints for the counters (both zero for
// shapes that are not split over k).  Negative: the shape is not taken.
HS_EXPORT int hs_linear_skinny_scratch(int M, int N, int K, int with_norm, long long* floats,
                                       int* counters) {
  hs::SkinnyPlan pl;
  if (!hs::plan_skinny(M, N, K, with_norm != 0, pl)) return HS_ERR_UNSUPPORTED;
  *floats = pl.ksplit > 1 ? (long long)pl.ksplit * pl.mp * N : 0;
  *counters = pl.ksplit > 1 ? pl.blocks : 0;
  return HS_OK;
}

// pdl != 0: launched with programmatic stream serialization (the weight fetch overlaps the
// previous kernel of the stream).
// Refuses (HS_ERR_UNSUPPORTED) M > 64, K not a multiple of 32, and unaligned pointers; the
// caller then uses another kernel.
HS_EXPORT int hs_linear_skinny(void* out, const void* a, const float* x, const float* gamma,
                               const float* beta, float eps, const void* w, const float* bias,
                               const float* residual, int M, int N, int K, int act, int out_dtype,
                               float* scratch, int* counters, int pdl, void* stream) {
  using namespace hs;
  if (!out || !w || (!a && !x)) return HS_ERR_ARGUMENT;
  if (x && (!gamma || !beta)) return HS_ERR_ARGUMENT;
  if (M <= 0 || N <= 0) return HS_OK;
  SkinnyPlan pl;
  if (!plan_skinny(M, N, K, x != nullptr, pl)) return HS_ERR_UNSUPPORTED;
  if (((uintptr_t)w & 15) || (a && ((uintptr_t)a & 15)) || (x && ((uintptr_t)x & 15)) ||
      (gamma && ((uintptr_t)gamma & 15)) || (beta && ((uintptr_t)beta & 15)))
    return HS_ERR_UNSUPPORTED;
  if (act < HS_ACT_NONE || act > HS_ACT_GELU_ERF) return HS_ERR_UNSUPPORTED;
  if (out_dtype != HS_DT_F32 && out_dtype != HS_DT_BF16) return HS_ERR_UNSUPPORTED;
  if (pl.ksplit > 1 && (!scratch || !counters)) return HS_ERR_ARGUMENT;
  SkinnyParams p;
  p.a = (const __nv_bfloat16*)a; p.x = x; p.gamma = gamma; p.beta = beta;
  p.w = (const __nv_bfloat16*)w; p.bias = bias; p.residual = residual; p.out = out;
  p.partial = scratch; p.counters = counters;
  p.M = M; p.N = N; p.K = K; p.act = act; p.out_f32 = out_dtype == HS_DT_F32;
  p.kper = pl.kper; p.stride = pl.stride; p.ng = pl.ng; p.eps = eps;
  p.red_offset = pl.red_offset;
  p.timing = hs_timing_buffer();
  cudaStream_t st = (cudaStream_t)stream;
  if (pl.nw == 16) {
    if (pl.mt == 1) return launch_skinny<1, 16>(p, pl.grid_x, pl.blocks, pl.ksplit, pl.smem, pl.smem_loop, st, pdl != 0);
    return launch_skinny<2, 16>(p, pl.grid_x, pl.blocks, pl.ksplit, pl.smem, pl.smem_loop, st, pdl != 0);
  }
  switch (pl.mt) {
    case 1: return launch_skinny<1, 8>(p, pl.grid_x, pl.blocks, pl.ksplit, pl.smem, pl.smem_loop, st, pdl != 0);
    case 2: return launch_skinny<2, 8>(p, pl.grid_x, pl.blocks, pl.ksplit, pl.smem, pl.smem_loop, st, pdl != 0);
    case 4: return launch_skinny<4, 8>(p, pl.grid_x, pl.blocks, pl.ksplit, pl.smem, pl.smem_loop, st, pdl != 0);
    default: return launch_skinny<8, 8>(p, pl.grid_x, pl.blocks, pl.ksplit, pl.smem, pl.smem_loop, st, pdl != 0);
  }
}

// The same product with the greedy choice fused in (the vocabulary head of a decode step whose
// rows all take the argmax): `out` receives the logits as above, `tokens[m]` the index of row
// m's largest value (lowest index on ties), `tokens[M]` the value of `status_word` (when not
// null), and `feedback[feedback_slot[m]]` the token too (slots below zero are skipped).  Every
// CTA leaves its best per row in `am_val` / `am_idx` ([entries] each, entries from
// hs_linear_skinny_argmax_scratch); `am_counter` is one int, zero between launches.  Takes
// bfloat16 activations without a norm, M <= 16, float32 logits, shapes that are not split
// over k; HS_ERR_UNSUPPORTED otherwise.
HS_EXPORT int hs_linear_skinny_argmax_scratch(int M, int N, int K, int* entries) {
  hs::SkinnyPlan pl;
  if (!hs::plan_skinny(M, N, K, false, pl) || pl.ksplit != 1 || pl.nw != 8 || pl.mt > 2)
    return HS_ERR_UNSUPPORTED;
  *entries = pl.grid_x * pl.mp;
  return HS_OK;
}

HS_EXPORT int hs_linear_skinny_argmax(float* out, const void* a, const void* w, int M, int N, int K,
                                      int* tokens, int* feedback, const int* feedback_slot,
                                      const int* status_word, float* am_val, int* am_idx,
                                      int* am_counter, int pdl, void* stream) {
  using namespace hs;
  if (!out || !a || !w || !tokens || !am_val || !am_idx || !am_counter) return HS_ERR_ARGUMENT;
  if ((feedback == nullptr) != (feedback_slot == nullptr)) return HS_ERR_ARGUMENT;
  if (M <= 0 || N <= 0) return HS_ERR_ARGUMENT;
  SkinnyPlan pl;
  if (!plan_skinny(M, N, K, false, pl) || pl.ksplit != 1 || pl.nw != 8 || pl.mt > 2)
    return HS_ERR_UNSUPPORTED;
  if (((uintptr_t)w & 15) || ((uintptr_t)a & 15)) return HS_ERR_UNSUPPORTED;
  SkinnyArgmaxParams p;
  p.a = (const __nv_bfloat16*)a; p.x = nullptr; p.gamma = nullptr; p.beta = nullptr;
  p.w = (const __nv_bfloat16*)w; p.bias = nullptr; p.residual = nullptr; p.out = out;
  p.partial = nullptr; p.counters = nullptr;
  p.M = M; p.N = N; p.K = K; p.act = HS_ACT_NONE; p.out_f32 = 1;
  p.kper = pl.kper; p.stride = pl.stride; p.ng = pl.ng; p.eps = 0.f;
  p.red_offset = pl.red_offset;
  p.tokens = tokens; p.feedback = feedback; p.feedback_slot = feedback_slot;
  p.status_word = status_word; p.am_val = am_val; p.am_idx = am_idx; p.am_counter = am_counter;
  p.timing = hs_timing_buffer();
  cudaStream_t st = (cudaStream_t)stream;
  if (pl.mt == 1)
    return launch_skinny_as<1, 8, true, true, 0, 0>(p, pl.grid_x, 1, pl.smem_loop, st, pdl != 0);
  return launch_skinny_as<2, 8, true, true, 0, 0>(p, pl.grid_x, 1, pl.smem_loop, st, pdl != 0);
}
