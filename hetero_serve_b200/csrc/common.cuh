// Shared helpers for the sm_100a kernels of hetero_serve_b200.
//
// Conventions used by every entry point in this directory:
//  * entry points are extern "C", take raw device pointers, sizes and the CUDA stream,
//    allocate nothing and return 0 or a negative HS_ERR_* code (sizes refused) or a
//    positive cudaError_t (launch failed);
//  * `dtype` arguments: 0 = float32, 1 = bfloat16;
//  * the residual stream, normalisation statistics, softmax state, accumulators, biases
//    and norm parameters are float32 in both precisions;
//  * `status` is one device int the engine owns.  A kernel that meets an index outside
//    its table (token id, position, page) skips the access and ORs a bit into it; the
//    host reads it with the step's results.  Nothing traps.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define HS_OK 0
#define HS_ERR_UNSUPPORTED (-1)   // a size or option this kernel does not take
#define HS_ERR_ARGUMENT (-2)      // null pointer / inconsistent arguments
#define HS_ERR_TOO_LARGE (-3)     // beyond a fixed capacity of the entry point

#define HS_STATUS_BAD_TOKEN 1
#define HS_STATUS_BAD_POSITION 2
#define HS_STATUS_BAD_PAGE 4
#define HS_STATUS_PIPELINE_TIMEOUT 8

#define HS_DT_F32 0
#define HS_DT_BF16 1

#define HS_ACT_NONE 0
#define HS_ACT_GELU_TANH 1
#define HS_ACT_GELU_ERF 2

#define HS_EXPORT extern "C" __attribute__((visibility("default")))

unsigned long long* hs_timing_buffer();   // embed_norm.cu
bool hs_pdl_enabled();                    // embed_norm.cu: programmatic dependent launch on?

// SM count of the device that is current when an entry point is called (the device of the
// stream the caller passes; the engine makes its own device current around every step).
static inline int hs_sm_count() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

#define HS_LAUNCH_CHECK()                      \
  do {                                         \
    cudaError_t e__ = cudaGetLastError();      \
    if (e__ != cudaSuccess) return (int)e__;   \
  } while (0)

namespace hs {

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// 0.5*u*(1+tanh(sqrt(2/pi)*(u+0.044715 u^3))) and 0.5*u*(1+erf(u/sqrt(2))), both with the
// accurate libm-grade device functions (this library is never built with fast-math).
__device__ __forceinline__ float gelu_tanh(float u) {
  const float k = 0.7978845608028654f;
  float inner = k * (u + 0.044715f * u * u * u);
  return 0.5f * u * (1.0f + tanhf(inner));
}
__device__ __forceinline__ float gelu_erf(float u) {
  return 0.5f * u * (1.0f + erff(u * 0.70710678118654752440f));
}
__device__ __forceinline__ float apply_act(float u, int act) {
  if (act == HS_ACT_GELU_TANH) return gelu_tanh(u);
  if (act == HS_ACT_GELU_ERF) return gelu_erf(u);
  return u;
}

// Phase timing for tuning builds only: compiled in with -DHS_PHASE_MARKS (the build script adds
// it when HETERO_SERVE_PHASE_MARKS=1 is set).  Then, once a buffer has been set with
// hs_set_timing_buffer, thread 0 of every CTA of the instrumented kernels stores the global
// nanosecond timer at a few marks: buffer[(cta * 8) + mark].  The product build has none of it.
__device__ __forceinline__ void mark_time(unsigned long long* buf, int cta, int mark) {
#ifdef HS_PHASE_MARKS
  if (buf != nullptr && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    buf[(size_t)cta * 8 + mark] = t;
  }
#else
  (void)buf; (void)cta; (void)mark;
#endif
}

// Programmatic dependent launch: a kernel launched with the programmatic-serialization
// attribute may start while its predecessor in the stream still runs.  `pdl_wait` blocks until
// the predecessor has completed and its writes are visible (a no-op for a normal launch);
// `pdl_trigger` lets the successor start.  What a kernel does before `pdl_wait` must not read
// anything an earlier kernel of the step writes (weights, block tables and work lists are safe).
// The decode attention kernels also fetch cache pages of EARLIER positions before the wait.
// Those were written by a kernel of an earlier step, and that is safe only because steps are
// separated on the stream by something that is not a programmatic edge between kernels: the
// upload of the step's metadata (a copy; a programmatic launch overlaps its predecessor
// kernel, never a copy) when steps are launched kernel by kernel, the boundary between two
// graph launches when a step is a CUDA graph (its first kernel node has no kernel before it
// in the graph, and a graph starts after all earlier work of its stream).  A caller that
// chains steps inside ONE graph or stream of kernels without such a boundary must launch
// these kernels without the attribute (`pdl` = 0).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

}  // namespace hs

// Launch with the programmatic-serialization attribute when `pdl` is set.
template <typename... KArgs, typename... Args>
static inline cudaError_t hs_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, bool pdl, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}
