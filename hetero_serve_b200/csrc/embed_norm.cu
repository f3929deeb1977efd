// Embedding gather (token table + optional learned position table) and LayerNorm.
//
// Reference formulas: x[t] = wte[ids[t]] + wpe[pos[t]] (heteroserve/model/torch_engine.py:89-90);
// mu = mean(x), var = mean((x-mu)^2), y = (x-mu)/sqrt(var+eps)*g + b
// (heteroserve/model/numpy_engine.py:26-30).  The sum and the statistics are float32.
#include "common.cuh"

namespace hs {

template <typename T>
__global__ void embed_kernel(float* __restrict__ x, const int* __restrict__ ids,
                             const int* __restrict__ pos, const int* __restrict__ req,
                             const T* __restrict__ wte, const T* __restrict__ wpe, int width,
                             int vocab, int n_pos, const int* __restrict__ feedback,
                             int n_feedback, int* status) {
  pdl_trigger();
  const int t = blockIdx.x;
  float* row = x + (size_t)t * width;
  const int r = req[t];
  int id = ids[t];
  const int p = pos[t];
  bool ok = r >= 0;
  // id = -(s + 1): the token that the latest sampling step left in feedback[s]
  if (ok && id < 0 && feedback != nullptr && -(id + 1) < n_feedback) id = feedback[-(id + 1)];
  if (ok && (id < 0 || id >= vocab)) {
    if (threadIdx.x == 0) atomicOr(status, HS_STATUS_BAD_TOKEN);
    ok = false;
  }
  if (ok && wpe != nullptr && (p < 0 || p >= n_pos)) {
    if (threadIdx.x == 0) atomicOr(status, HS_STATUS_BAD_POSITION);
    ok = false;
  }
  if (!ok) {  // padding rows of a bucket, or a refused index: a defined, finite row
    for (int e = threadIdx.x; e < width; e += blockDim.x) row[e] = 0.f;
    return;
  }
  const T* a = wte + (size_t)id * width;
  if (wpe != nullptr) {
    const T* b = wpe + (size_t)p * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x) row[e] = to_f(a[e]) + to_f(b[e]);
  } else {
    for (int e = threadIdx.x; e < width; e += blockDim.x) row[e] = to_f(a[e]);
  }
}

// One block per output row.  The row is staged in shared memory as float32; the mean and
// the centred variance are two block reductions whose tree depends on `width` and the
// block size only, so a row's result never depends on the batch around it.
template <typename TO, int THREADS>
__global__ void layernorm_kernel(TO* __restrict__ out, const float* __restrict__ x,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 const int* __restrict__ rows, int width, float eps) {
  extern __shared__ float srow[];
  __shared__ float red[THREADS / 32];
  __shared__ float bcast;
  pdl_trigger();
  const int o = blockIdx.x;
  const int src = rows ? rows[o] : o;
  const float* xr = x + (size_t)src * width;
  pdl_wait();
  float s = 0.f;
  for (int e = threadIdx.x; e < width; e += THREADS) {
    float v = xr[e];
    srow[e] = v;
    s += v;
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < THREADS / 32; ++i) t += red[i];
    bcast = t / (float)width;
  }
  __syncthreads();
  const float mu = bcast;
  float q = 0.f;
  for (int e = threadIdx.x; e < width; e += THREADS) {
    float c = srow[e] - mu;
    q += c * c;
  }
  q = warp_sum(q);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = q;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int i = 0; i < THREADS / 32; ++i) t += red[i];
    bcast = 1.0f / sqrtf(t / (float)width + eps);
  }
  __syncthreads();
  const float rstd = bcast;
  TO* orow = out + (size_t)o * width;
  for (int e = threadIdx.x; e < width; e += THREADS)
    orow[e] = from_f<TO>((srow[e] - mu) * rstd * gamma[e] + beta[e]);
}

// One warp per row, the row held in registers (up to 32 * 4 * LN_F4 floats): no shared memory,
// no block barrier.  The mean and the centred variance are two warp reductions (a fixed
// butterfly), so a row's result does not depend on the batch here either.
constexpr int LN_F4 = 16;           // rows of up to 2048 floats
constexpr int LN_ROWS_PER_CTA = 8;

template <typename TO>
__global__ void __launch_bounds__(LN_ROWS_PER_CTA * 32)
layernorm_warp_kernel(TO* __restrict__ out, const float* __restrict__ x,
                      const float* __restrict__ gamma, const float* __restrict__ beta,
                      const int* __restrict__ rows, int n_rows, int width, float eps) {
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int o = blockIdx.x * LN_ROWS_PER_CTA + warp;
  const int nf4 = width / 4;
  // weight and bias of the norm do not change during a step: they are brought into shared
  // memory before the dependency wait, off the critical path
  extern __shared__ float4 s_gb[];                       // [nf4] weight, [nf4] bias
  for (int i = threadIdx.x; i < nf4; i += blockDim.x) {
    s_gb[i] = ((const float4*)gamma)[i];
    s_gb[nf4 + i] = ((const float4*)beta)[i];
  }
  __syncthreads();
  if (o >= n_rows) return;
  const int src = rows ? rows[o] : o;
  const float4* xr = (const float4*)(x + (size_t)src * width);
  pdl_wait();                      // x is what the previous kernel wrote
  float4 v[LN_F4];
#pragma unroll
  for (int i = 0; i < LN_F4; ++i)
    v[i] = (lane + 32 * i < nf4) ? xr[lane + 32 * i] : make_float4(0.f, 0.f, 0.f, 0.f);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < LN_F4; ++i) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  const float mu = warp_sum(s) / (float)width;
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < LN_F4; ++i) {
    if (lane + 32 * i < nf4) {
      const float c0 = v[i].x - mu, c1 = v[i].y - mu, c2 = v[i].z - mu, c3 = v[i].w - mu;
      q += (c0 * c0 + c1 * c1) + (c2 * c2 + c3 * c3);
    }
  }
  const float rstd = 1.0f / sqrtf(warp_sum(q) / (float)width + eps);
  TO* orow = out + (size_t)o * width;
#pragma unroll
  for (int i = 0; i < LN_F4; ++i) {
    const int e = (lane + 32 * i) * 4;
    if (lane + 32 * i < nf4) {
      const float4 g = s_gb[lane + 32 * i], b = s_gb[nf4 + lane + 32 * i];
      const float y0 = (v[i].x - mu) * rstd * g.x + b.x, y1 = (v[i].y - mu) * rstd * g.y + b.y;
      const float y2 = (v[i].z - mu) * rstd * g.z + b.z, y3 = (v[i].w - mu) * rstd * g.w + b.w;
      if constexpr (sizeof(TO) == 4) {
        *(float4*)((float*)orow + e) = make_float4(y0, y1, y2, y3);
      } else {
        __nv_bfloat162 p0 = __floats2bfloat162_rn(y0, y1), p1 = __floats2bfloat162_rn(y2, y3);
        uint2 u;
        u.x = *(uint32_t*)&p0; u.y = *(uint32_t*)&p1;
        *(uint2*)((__nv_bfloat16*)orow + e) = u;
      }
    }
  }
}

}  // namespace hs

// feedback (may be null): `n_feedback` token ids kept on the device; a negative id -(s + 1) in
// `ids` stands for feedback[s], so that a step can start before the host has seen the token the
// previous step sampled.
HS_EXPORT int hs_embed(float* x, const int* ids, const int* pos, const int* req, const void* wte,
                       const void* wpe, int n_tokens, int width, int vocab, int n_pos,
                       int table_dtype, const int* feedback, int n_feedback, int* status,
                       void* stream) {
  if (!x || !ids || !pos || !req || !wte || !status) return HS_ERR_ARGUMENT;
  if (n_tokens <= 0) return HS_OK;
  cudaStream_t st = (cudaStream_t)stream;
  int threads = width >= 1024 ? 256 : 128;
  if (table_dtype == HS_DT_F32)
    hs::embed_kernel<float><<<n_tokens, threads, 0, st>>>(
        x, ids, pos, req, (const float*)wte, (const float*)wpe, width, vocab, n_pos, feedback,
        n_feedback, status);
  else if (table_dtype == HS_DT_BF16)
    hs::embed_kernel<__nv_bfloat16><<<n_tokens, threads, 0, st>>>(
        x, ids, pos, req, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, width, vocab,
        n_pos, feedback, n_feedback, status);
  else
    return HS_ERR_UNSUPPORTED;
  HS_LAUNCH_CHECK();
  return HS_OK;
}

HS_EXPORT int hs_layernorm(void* out, const float* x, const float* gamma, const float* beta,
                           const int* rows, int n_rows, int width, float eps, int out_dtype,
                           void* stream) {
  if (!out || !x || !gamma || !beta) return HS_ERR_ARGUMENT;
  if (n_rows <= 0) return HS_OK;
  cudaStream_t st0 = (cudaStream_t)stream;
  // rows of up to 2048 floats (a multiple of 4, 16-byte aligned): one warp per row
  if (width % 4 == 0 && width <= hs::LN_F4 * 128 && !((uintptr_t)x & 15) && !((uintptr_t)out & 15) &&
      !((uintptr_t)gamma & 15) && !((uintptr_t)beta & 15)) {
    const int grid = (n_rows + hs::LN_ROWS_PER_CTA - 1) / hs::LN_ROWS_PER_CTA;
    cudaError_t le;
    const bool pdl = hs_pdl_enabled();
    if (out_dtype == HS_DT_F32)
      le = hs_launch(hs::layernorm_warp_kernel<float>, dim3(grid), dim3(hs::LN_ROWS_PER_CTA * 32),
                     (size_t)width * 8, st0, pdl, (float*)out, x, gamma, beta, rows, n_rows, width,
                     eps);
    else if (out_dtype == HS_DT_BF16)
      le = hs_launch(hs::layernorm_warp_kernel<__nv_bfloat16>, dim3(grid),
                     dim3(hs::LN_ROWS_PER_CTA * 32), (size_t)width * 8, st0, pdl,
                     (__nv_bfloat16*)out, x, gamma, beta, rows, n_rows, width, eps);
    else
      return HS_ERR_UNSUPPORTED;
    if (le != cudaSuccess) return (int)le;
    HS_LAUNCH_CHECK();
    return HS_OK;
  }
  constexpr int THREADS = 256;
  size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return HS_ERR_UNSUPPORTED;  // a row must fit shared memory
  cudaStream_t st = (cudaStream_t)stream;
  if (out_dtype == HS_DT_F32) {
    auto k = hs::layernorm_kernel<float, THREADS>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t le = hs_launch(k, dim3(n_rows), dim3(THREADS), smem, st, hs_pdl_enabled(),
                               (float*)out, x, gamma, beta, rows, width, eps);
    if (le != cudaSuccess) return (int)le;
  } else if (out_dtype == HS_DT_BF16) {
    auto k = hs::layernorm_kernel<__nv_bfloat16, THREADS>;
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t le = hs_launch(k, dim3(n_rows), dim3(THREADS), smem, st, hs_pdl_enabled(),
                               (__nv_bfloat16*)out, x, gamma, beta, rows, width, eps);
    if (le != cudaSuccess) return (int)le;
  } else {
    return HS_ERR_UNSUPPORTED;
  }
  HS_LAUNCH_CHECK();
  return HS_OK;
}

// Tuning aid: a device buffer of 8 x uint64 per CTA that instrumented kernels fill with
// nanosecond timestamps (see mark_time in common.cuh); null switches it off.
static unsigned long long* g_timing_buffer = nullptr;
HS_EXPORT void hs_set_timing_buffer(unsigned long long* buf) { g_timing_buffer = buf; }
unsigned long long* hs_timing_buffer() { return g_timing_buffer; }

// Programmatic dependent launch for the kernels that take no `pdl` argument of their own
// (LayerNorm, the tcgen05 linear, the cache append, the prompt attention, sampling): each of
// them waits (griddepcontrol.wait) before it first reads what an earlier kernel wrote, so with
// the switch on they are launched with the programmatic-serialization attribute and their
// prologue overlaps the tail of the kernel before them.  Off by default.
static bool g_pdl = false;
HS_EXPORT void hs_set_pdl(int on) { g_pdl = on != 0; }
bool hs_pdl_enabled() { return g_pdl; }
