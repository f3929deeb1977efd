// A float32-accumulating linear layer on the CUDA cores (FFMA), for the true 32-bit path and
// as the fallback for shapes the tensor-core kernel refuses.
//
//   out[m, n] = act( sum_k a[m, k] * w[n, k] + bias[n] ) (+ residual[m, n])
//
// `w` is [N, K] with K contiguous (Conv1D weights, stored [in, out], are transposed once when
// they are bound; the tied head uses the token table as it is).  Reference call sites:
// `h @ attn_w + attn_b`, `x + (attn @ proj_w + proj_b)`, `gelu(x @ fc_w + fc_b) @ fcp_w + fcp_b`,
// `ln_f(x) @ wte.T` (heteroserve/model/torch_engine.py:77-79,86-87,122,139).
//
// Every output element is one chain of fused multiply-adds over k = 0..K-1 in index order,
// whatever M is and wherever the row sits in its tile: a row's result does not depend on
// the batch it is computed in.  No tensor cores, no TF32, no split over K.
#include "common.cuh"

namespace hs {

constexpr int LS_BM = 64, LS_BN = 64, LS_BK = 16, LS_THREADS = 256;

// four consecutive elements of a row in one load (the rows are 16-byte / 8-byte aligned there)
__device__ __forceinline__ void lb_load4(const float* p, float (&v)[4]) {
  const float4 x = *(const float4*)p;
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
__device__ __forceinline__ void lb_load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 x = *(const uint2*)p;
  v[0] = __uint_as_float(x.x << 16); v[1] = __uint_as_float(x.x & 0xffff0000u);
  v[2] = __uint_as_float(x.y << 16); v[3] = __uint_as_float(x.y & 0xffff0000u);
}


// VEC: K is a multiple of 4 and both matrices start on a 16-byte boundary: a thread's four k
// of a row come in one load.
template <typename TI, typename TO, bool VEC>
__global__ void __launch_bounds__(LS_THREADS)
linear_simt_kernel(TO* out, const TI* __restrict__ a, const TI* __restrict__ w,
                   const float* __restrict__ bias, const float* residual, int M, int N, int K,
                   int act) {
  __shared__ float As[LS_BK][LS_BM + 4];
  __shared__ float Ws[LS_BK][LS_BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * LS_BM, n0 = blockIdx.x * LS_BN;
  // loader mapping: thread -> (row 0..63, 4 consecutive k)
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += LS_BK) {
    {
      const int gm = m0 + lr, gn = n0 + lr;
      if (VEC) {
        float ra[4] = {0.f, 0.f, 0.f, 0.f}, rw[4] = {0.f, 0.f, 0.f, 0.f};
        const int gk = k0 + lk;                           // K % 4 == 0: all four or none
        if (gm < M && gk < K) lb_load4(a + (size_t)gm * K + gk, ra);
        if (gn < N && gk < K) lb_load4(w + (size_t)gn * K + gk, rw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          As[lk + j][lr] = ra[j];
          Ws[lk + j][lr] = rw[j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int gk = k0 + lk + j;
          As[lk + j][lr] = (gm < M && gk < K) ? to_f(a[(size_t)gm * K + gk]) : 0.f;
          Ws[lk + j][lr] = (gn < N && gk < K) ? to_f(w[(size_t)gn * K + gk]) : 0.f;
        }
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < LS_BK; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      v = apply_act(v, act);
      if (residual) v += residual[(size_t)gm * N + gn];
      out[(size_t)gm * N + gn] = from_f<TO>(v);
    }
  }
}

// ---- many rows (prompts): 128 x 128 tiles, an 8 x 8 patch of outputs per thread ---------------
// The same chains again (every output one fmaf chain over k = 0..K-1 in index order), with
// twice the outputs per shared-memory word read: a thread's 64 outputs take 16 words per k.
// Tiles of both operands arrive k-major ([k][row]) through registers, two buffers.
constexpr int LB_BM = 128, LB_BN = 128, LB_BK = 8, LB_THREADS = 256;

// VEC: K is a multiple of 4 and both matrices start on a 16-byte boundary, so a thread's four
// k of a row come in one load (with one 4-byte load per element the load pipe, 16 sectors an
// instruction, took as long as the products).
template <typename TI, typename TO, bool VEC>
__global__ void __launch_bounds__(LB_THREADS)
linear_simt_big_kernel(TO* out, const TI* __restrict__ a, const TI* __restrict__ w,
                       const float* __restrict__ bias, const float* residual, int M, int N, int K,
                       int act) {
  __shared__ __align__(16) float As[2][LB_BK][LB_BM];
  __shared__ __align__(16) float Ws[2][LB_BK][LB_BN];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;                 // 16 x 16 threads, 8 x 8 outputs each
  const int m0 = blockIdx.y * LB_BM, n0 = blockIdx.x * LB_BN;
  // loader: thread -> (row 0..127, 4 consecutive k of the 8)
  const int lr = tid >> 1, lk = (tid & 1) * 4;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  float ra[4], rw[4];
  auto fetch = [&](int k0) {
    const int gm = m0 + lr, gn = n0 + lr;
    if (VEC) {
      const int gk = k0 + lk;                             // K % 4 == 0: all four or none
#pragma unroll
      for (int j = 0; j < 4; ++j) ra[j] = rw[j] = 0.f;
      if (gm < M && gk < K) lb_load4(a + (size_t)gm * K + gk, ra);
      if (gn < N && gk < K) lb_load4(w + (size_t)gn * K + gk, rw);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gk = k0 + lk + j;
        ra[j] = (gm < M && gk < K) ? to_f(a[(size_t)gm * K + gk]) : 0.f;
        rw[j] = (gn < N && gk < K) ? to_f(w[(size_t)gn * K + gk]) : 0.f;
      }
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      As[buf][lk + j][lr] = ra[j];
      Ws[buf][lk + j][lr] = rw[j];
    }
  };
  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += LB_BK) {
    const bool more = k0 + LB_BK < K;
    if (more) fetch(k0 + LB_BK);                          // in flight during the products below
#pragma unroll
    for (int kk = 0; kk < LB_BK; ++kk) {
      // rows ty*4..+3 and 64+ty*4..+3, columns tx*4..+3 and 64+tx*4..+3: 16-byte reads, no
      // bank conflicts
      const float4 a0 = *(const float4*)&As[buf][kk][ty * 4];
      const float4 a1 = *(const float4*)&As[buf][kk][64 + ty * 4];
      const float4 w0 = *(const float4*)&Ws[buf][kk][tx * 4];
      const float4 w1 = *(const float4*)&Ws[buf][kk][64 + tx * 4];
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    if (more) {
      stash(buf ^ 1);
      __syncthreads();
      buf ^= 1;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
      if (gn >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[gn];
      v = apply_act(v, act);
      if (residual) v += residual[(size_t)gm * N + gn];
      out[(size_t)gm * N + gn] = from_f<TO>(v);
    }
  }
}

// ---- few rows (decode): the same chains, laid out for a weight stream -------------------------
// With M <= 16 the tile kernel above leaves most of the machine idle (N / 64 CTAs, each walking
// all of K behind two barriers per 16 columns).  Here a CTA owns 16 output features and all
// rows; thread (feature f, row group g) runs the chains of rows g and g + 8 for feature f over
// k = 0..K-1 in index order - the same chain of fused multiply-adds, so the same bits, as the
// tile kernel gives that element.  The weight rows and the activation rows arrive through a
// ring of four 128-column stages of 16-byte cp.async copies.  RPT rows per thread: 2 for up to
// 16 rows, 8 for up to 64 (rows g, g + 8, ..., g + 56).
constexpr int LF_BN = 16, LF_BK = 128, LF_THREADS = 128, LF_STAGES = 4;

template <typename TI, int RPT>
struct LfShape {
  static constexpr int MAX_M = 8 * RPT;
  static constexpr int VEC = 16 / (int)sizeof(TI);           // elements per 16-byte copy
  static constexpr int WS = LF_BK + VEC;                     // weight row stride: no bank conflicts
  static constexpr int STAGE = LF_BN * WS + MAX_M * LF_BK;   // elements per stage
  static constexpr size_t SMEM = (size_t)LF_STAGES * STAGE * sizeof(TI);
};

__device__ __forceinline__ void lf_copy16(void* smem_dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;                              // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src),
               "r"(n)
               : "memory");
}
__device__ __forceinline__ void lf_load4(const float* p, float (&v)[4]) {
  const float4 x = *(const float4*)p;
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
__device__ __forceinline__ void lf_load4(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 x = *(const uint2*)p;
  v[0] = __uint_as_float(x.x << 16); v[1] = __uint_as_float(x.x & 0xffff0000u);
  v[2] = __uint_as_float(x.y << 16); v[3] = __uint_as_float(x.y & 0xffff0000u);
}

template <typename TI, typename TO, int RPT>
__global__ void __launch_bounds__(LF_THREADS)
linear_simt_few_rows_kernel(TO* out, const TI* __restrict__ a, const TI* __restrict__ w,
                            const float* __restrict__ bias, const float* residual, int M, int N,
                            int K, int act) {
  using S = LfShape<TI, RPT>;
  extern __shared__ __align__(16) uint8_t lf_smem[];
  TI* ring = (TI*)lf_smem;
  const int tid = threadIdx.x;
  const int f = tid & 15, grp = tid >> 4;                    // rows grp, grp + 8, ...
  const int n0 = blockIdx.x * LF_BN;
  const int num_kt = (K + LF_BK - 1) / LF_BK;
  constexpr int CPR = LF_BK / S::VEC;                        // copies per row of a stage

  auto issue = [&](int kt) {
    if (kt < num_kt) {
      TI* sw = ring + (size_t)(kt % LF_STAGES) * S::STAGE;
      TI* sa = sw + LF_BN * S::WS;
      for (int c = tid; c < LF_BN * CPR; c += LF_THREADS) {
        const int row = c / CPR, kc = (c - row * CPR) * S::VEC;
        const int gk = kt * LF_BK + kc, gn = n0 + row;
        const bool ok = gn < N && gk < K;
        lf_copy16(sw + row * S::WS + kc, ok ? w + (size_t)gn * K + gk : w, ok);
      }
      for (int c = tid; c < S::MAX_M * CPR; c += LF_THREADS) {
        const int row = c / CPR, kc = (c - row * CPR) * S::VEC;
        const int gk = kt * LF_BK + kc;
        const bool ok = row < M && gk < K;
        lf_copy16(sa + row * LF_BK + kc, ok ? a + (size_t)row * K + gk : a, ok);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");   // one group per call, empty or not
  };

  for (int s = 0; s < LF_STAGES - 1; ++s) issue(s);
  float acc[RPT];
#pragma unroll
  for (int r = 0; r < RPT; ++r) acc[r] = 0.f;
  for (int kt = 0; kt < num_kt; ++kt) {
    asm volatile("cp.async.wait_group %0;" ::"n"(LF_STAGES - 2) : "memory");
    __syncthreads();                 // stage kt has landed; stage kt - 1 is free for every thread
    issue(kt + LF_STAGES - 1);
    const TI* sw = ring + (size_t)(kt % LF_STAGES) * S::STAGE + f * S::WS;
    const TI* sa = ring + (size_t)(kt % LF_STAGES) * S::STAGE + LF_BN * S::WS + grp * LF_BK;
    const int kmax = min(LF_BK, K - kt * LF_BK);             // a multiple of 4
#pragma unroll 4
    for (int k = 0; k < kmax; k += 4) {
      float wv[4];
      lf_load4(sw + k, wv);
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        float x[4];
        lf_load4(sa + r * 8 * LF_BK + k, x);
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[r] = fmaf(x[i], wv[i], acc[r]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  const int gn = n0 + f;
  if (gn >= N) return;
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int gm = grp + 8 * r;
    if (gm >= M) continue;
    float v = acc[r];
    if (bias) v += bias[gn];
    v = apply_act(v, act);
    if (residual) v += residual[(size_t)gm * N + gn];
    out[(size_t)gm * N + gn] = from_f<TO>(v);
  }
}

template <typename TI, typename TO, int RPT>
static int launch_few_rows_as(void* out, const void* a, const void* w, const float* bias,
                              const float* residual, int M, int N, int K, int act,
                              cudaStream_t st) {
  auto* k = linear_simt_few_rows_kernel<TI, TO, RPT>;
  static cudaError_t state = cudaErrorUnknown;
  if (state != cudaSuccess)
    state = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)LfShape<TI, RPT>::SMEM);
  if (state != cudaSuccess) return (int)state;
  k<<<(N + LF_BN - 1) / LF_BN, LF_THREADS, LfShape<TI, RPT>::SMEM, st>>>(
      (TO*)out, (const TI*)a, (const TI*)w, bias, residual, M, N, K, act);
  return HS_OK;
}

template <typename TI, typename TO>
static int launch_few_rows(void* out, const void* a, const void* w, const float* bias,
                           const float* residual, int M, int N, int K, int act, cudaStream_t st) {
  if (M <= 16) return launch_few_rows_as<TI, TO, 2>(out, a, w, bias, residual, M, N, K, act, st);
  return launch_few_rows_as<TI, TO, 8>(out, a, w, bias, residual, M, N, K, act, st);
}

}  // namespace hs

HS_EXPORT int hs_linear_simt(void* out, const void* a, const void* w, const float* bias,
                             const float* residual, int M, int N, int K, int act, int in_dtype,
                             int out_dtype, void* stream) {
  if (!out || !a || !w) return HS_ERR_ARGUMENT;
  if (M <= 0 || N <= 0) return HS_OK;
  if (K <= 0) return HS_ERR_ARGUMENT;
  if (act < HS_ACT_NONE || act > HS_ACT_GELU_ERF) return HS_ERR_UNSUPPORTED;
  dim3 grid((N + hs::LS_BN - 1) / hs::LS_BN, (M + hs::LS_BM - 1) / hs::LS_BM);
  if (grid.y > 65535) return HS_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  using bf16 = __nv_bfloat16;
  // few rows: the weight-stream kernel (rows and pointers that 16-byte copies can take)
  const int vec = in_dtype == HS_DT_F32 ? 4 : 8;
  // (17-64 rows: while the layer's feature blocks are a few per SM; a wide layer such as the
  // vocabulary head keeps more in flight with the tile kernel: 233 us against 599 at 64 rows)
  const bool few = M <= 16 || (M <= 64 && (N + hs::LF_BN - 1) / hs::LF_BN <= 4 * hs_sm_count());
  if (few && K % vec == 0 && !((uintptr_t)a & 15) && !((uintptr_t)w & 15)) {
    int rc = HS_ERR_UNSUPPORTED;
    if (in_dtype == HS_DT_F32 && out_dtype == HS_DT_F32)
      rc = hs::launch_few_rows<float, float>(out, a, w, bias, residual, M, N, K, act, st);
    else if (in_dtype == HS_DT_BF16 && out_dtype == HS_DT_BF16)
      rc = hs::launch_few_rows<bf16, bf16>(out, a, w, bias, residual, M, N, K, act, st);
    else if (in_dtype == HS_DT_BF16 && out_dtype == HS_DT_F32)
      rc = hs::launch_few_rows<bf16, float>(out, a, w, bias, residual, M, N, K, act, st);
    if (rc != HS_OK) return rc;
    HS_LAUNCH_CHECK();
    return HS_OK;
  }
  if (M >= 256) {                    // prompts: the larger tile
    dim3 big((N + hs::LB_BN - 1) / hs::LB_BN, (M + hs::LB_BM - 1) / hs::LB_BM);
    if (big.y > 65535) return HS_ERR_UNSUPPORTED;
    const bool vec4 = K % 4 == 0 && !((uintptr_t)a & 15) && !((uintptr_t)w & 15);
#define HS_LB_LAUNCH(TI, TO)                                                                   \
  do {                                                                                         \
    if (vec4)                                                                                  \
      hs::linear_simt_big_kernel<TI, TO, true><<<big, hs::LB_THREADS, 0, st>>>(                \
          (TO*)out, (const TI*)a, (const TI*)w, bias, residual, M, N, K, act);                 \
    else                                                                                       \
      hs::linear_simt_big_kernel<TI, TO, false><<<big, hs::LB_THREADS, 0, st>>>(               \
          (TO*)out, (const TI*)a, (const TI*)w, bias, residual, M, N, K, act);                 \
  } while (0)
    if (in_dtype == HS_DT_F32 && out_dtype == HS_DT_F32) HS_LB_LAUNCH(float, float);
    else if (in_dtype == HS_DT_BF16 && out_dtype == HS_DT_BF16) HS_LB_LAUNCH(bf16, bf16);
    else if (in_dtype == HS_DT_BF16 && out_dtype == HS_DT_F32) HS_LB_LAUNCH(bf16, float);
    else return HS_ERR_UNSUPPORTED;
#undef HS_LB_LAUNCH
    HS_LAUNCH_CHECK();
    return HS_OK;
  }
  const bool ls_vec = K % 4 == 0 && !((uintptr_t)a & 15) && !((uintptr_t)w & 15);
#define HS_LS_LAUNCH(TI, TO)                                                                  \
  do {                                                                                        \
    if (ls_vec)                                                                               \
      hs::linear_simt_kernel<TI, TO, true><<<grid, hs::LS_THREADS, 0, st>>>(                  \
          (TO*)out, (const TI*)a, (const TI*)w, bias, residual, M, N, K, act);                \
    else                                                                                      \
      hs::linear_simt_kernel<TI, TO, false><<<grid, hs::LS_THREADS, 0, st>>>(                 \
          (TO*)out, (const TI*)a, (const TI*)w, bias, residual, M, N, K, act);                \
  } while (0)
  if (in_dtype == HS_DT_F32 && out_dtype == HS_DT_F32) HS_LS_LAUNCH(float, float);
  else if (in_dtype == HS_DT_BF16 && out_dtype == HS_DT_BF16) HS_LS_LAUNCH(bf16, bf16);
  else if (in_dtype == HS_DT_BF16 && out_dtype == HS_DT_F32) HS_LS_LAUNCH(bf16, float);
  else return HS_ERR_UNSUPPORTED;
#undef HS_LS_LAUNCH
  HS_LAUNCH_CHECK();
  return HS_OK;
}
