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

template <typename TI, typename TO>
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
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int gk = k0 + lk + j;
        As[lk + j][lr] = (gm < M && gk < K) ? to_f(a[(size_t)gm * K + gk]) : 0.f;
        Ws[lk + j][lr] = (gn < N && gk < K) ? to_f(w[(size_t)gn * K + gk]) : 0.f;
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
#define HS_LS_LAUNCH(TI, TO)                                                                  \
  hs::linear_simt_kernel<TI, TO><<<grid, hs::LS_THREADS, 0, st>>>(                             \
      (TO*)out, (const TI*)a, (const TI*)w, bias, residual, M, N, K, act)
  if (in_dtype == HS_DT_F32 && out_dtype == HS_DT_F32) HS_LS_LAUNCH(float, float);
  else if (in_dtype == HS_DT_BF16 && out_dtype == HS_DT_BF16) HS_LS_LAUNCH(bf16, bf16);
  else if (in_dtype == HS_DT_BF16 && out_dtype == HS_DT_F32) HS_LS_LAUNCH(bf16, float);
  else return HS_ERR_UNSUPPORTED;
#undef HS_LS_LAUNCH
  HS_LAUNCH_CHECK();
  return HS_OK;
}
