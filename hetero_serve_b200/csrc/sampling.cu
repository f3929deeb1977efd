// Token selection on the device: argmax, and temperature / top-k sampling by inverse CDF.
//
// The reference samples on the host (heteroserve/worker/worker.py:38-50): temperature <= 0
// takes the argmax; otherwise softmax(logits / temperature) over all tokens or, for
// 0 < top_k < V, over the top_k largest, and one draw from it.  Here the draw is one uniform
// number u in [0, 1) from Philox-4x32-10 keyed by the request's seed with the position of the
// new token as counter, so that (like the reference's reseeding with seed + n_kv,
// worker.py:647,694) a sampled token does not depend on how requests were batched.  The token
// is the first, in index order, whose cumulative unnormalised probability exceeds u * total.
// Ties in argmax and at the top-k threshold go to the lower index.  All arithmetic is float32.
#include "common.cuh"

namespace hs {

constexpr int SM_THREADS = 1024;

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t (&k)[2]) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
  const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k[0], n1 = lo1, n2 = hi0 ^ c[3] ^ k[1], n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
  k[0] += 0x9E3779B9u;
  k[1] += 0xBB67AE85u;
}

__device__ __forceinline__ float philox_uniform(uint32_t seed_lo, uint32_t seed_hi,
                                                uint32_t position) {
  uint32_t c[4] = {position, 0u, 0u, 0u};
  uint32_t k[2] = {seed_lo, seed_hi};
#pragma unroll
  for (int i = 0; i < 10; ++i) philox_round(c, k);
  return (float)(c[0] >> 8) * (1.0f / 16777216.0f);
}

__device__ __forceinline__ uint32_t order_key(float v) {
  uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

// block-wide argmax of one row; every thread returns the result
__device__ ArgMax block_argmax(const float* row, int vocab) {
  __shared__ ArgMax sh[SM_THREADS / 32];
  __shared__ ArgMax result;
  ArgMax best{-INFINITY, 0x7fffffff};
  // 32 loads in flight per thread (a row of 50k logits is two rounds for 1,024 threads); within
  // a thread indices rise, so the first seen wins ties
  constexpr int INFLIGHT = 32;
  for (int base = threadIdx.x; base < vocab; base += INFLIGHT * blockDim.x) {
    float v[INFLIGHT];
#pragma unroll
    for (int j = 0; j < INFLIGHT; ++j) {
      const int i = base + j * blockDim.x;
      v[j] = i < vocab ? row[i] : -INFINITY;
    }
#pragma unroll
    for (int j = 0; j < INFLIGHT; ++j) {
      const int i = base + j * blockDim.x;
      if (i < vocab && (v[j] > best.v || best.i == 0x7fffffff)) best = ArgMax{v[j], i};
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    ArgMax b = sh[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) b = better(b, sh[w]);
    if (b.i == 0x7fffffff) b.i = 0;
    result = b;
  }
  __syncthreads();
  ArgMax r = result;
  __syncthreads();
  return r;
}

__device__ int block_sum_int(int v) {
  __shared__ int sh[SM_THREADS / 32];
  __shared__ int total;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += sh[w];
    total = t;
  }
  __syncthreads();
  int r = total;
  __syncthreads();
  return r;
}

// Inclusive scan over the block in thread order of a float and an int at once.
// Returns the block totals through `tot_f`, `tot_i`.
__device__ void block_scan(float& f, int& n, float& tot_f, int& tot_i) {
  __shared__ float wf[SM_THREADS / 32];
  __shared__ int wn[SM_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float uf = __shfl_up_sync(0xffffffffu, f, o);
    const int un = __shfl_up_sync(0xffffffffu, n, o);
    if (lane >= o) {
      f += uf;
      n += un;
    }
  }
  if (lane == 31) {
    wf[warp] = f;
    wn[warp] = n;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    float a = lane < nw ? wf[lane] : 0.f;
    int b = lane < nw ? wn[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float ua = __shfl_up_sync(0xffffffffu, a, o);
      const int ub = __shfl_up_sync(0xffffffffu, b, o);
      if (lane >= o) {
        a += ua;
        b += ub;
      }
    }
    if (lane < nw) {
      wf[lane] = a;
      wn[lane] = b;
    }
  }
  __syncthreads();
  if (warp > 0) {
    f += wf[warp - 1];
    n += wn[warp - 1];
  }
  tot_f = wf[(blockDim.x >> 5) - 1];
  tot_i = wn[(blockDim.x >> 5) - 1];
  __syncthreads();
}

__global__ void __launch_bounds__(SM_THREADS)
argmax_kernel(int* __restrict__ out, const float* __restrict__ logits, int vocab) {
  const float* row = logits + (size_t)blockIdx.x * vocab;
  ArgMax r = block_argmax(row, vocab);
  if (threadIdx.x == 0) out[blockIdx.x] = r.i;
}

__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(int* __restrict__ out, const float* __restrict__ logits,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const int* __restrict__ seed_lo, const int* __restrict__ seed_hi,
              const int* __restrict__ position, int vocab, int* __restrict__ feedback,
              const int* __restrict__ feedback_slot, const int* __restrict__ status_word) {
  const int rowi = blockIdx.x;
  const float* row = logits + (size_t)rowi * vocab;
  const float temp = temperature[rowi];
  pdl_wait();                       // the logits are what the previous kernel wrote
  // the engine's status word rides behind the tokens, so that one copy brings both to the host
  if (status_word != nullptr && rowi == 0 && threadIdx.x == 0) out[gridDim.x] = *status_word;
  const ArgMax top = block_argmax(row, vocab);
  // a row with a feedback slot also leaves its token there, for the next step's embedding
  const int fb = (feedback != nullptr && feedback_slot != nullptr) ? feedback_slot[rowi] : -1;
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) {
      out[rowi] = top.i;
      if (fb >= 0) feedback[fb] = top.i;
    }
    return;
  }
  const float mx = top.v / temp;
  int k = top_k[rowi];
  uint32_t thr = 0;   // order key of the k-th largest logit; 0 keeps everything
  int need_eq = 0;    // how many entries equal to the threshold are kept (lowest indices)
  const bool use_k = k > 0 && k < vocab;
  if (use_k) {
    for (int b = 31; b >= 0; --b) {
      const uint32_t cand = thr | (1u << b);
      int c = 0;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) c += order_key(row[i]) >= cand;
      if (block_sum_int(c) >= k) thr = cand;
    }
    int c = 0;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) c += order_key(row[i]) > thr;
    need_eq = k - block_sum_int(c);
  }
  const float u = philox_uniform((uint32_t)seed_lo[rowi], (uint32_t)seed_hi[rowi],
                                 (uint32_t)position[rowi]);
  __shared__ int found;
  if (threadIdx.x == 0) found = 0x7fffffff;
  float target = 0.f;
  int last_kept = 0;
  for (int pass = 0; pass < 2; ++pass) {
    float run = 0.f;
    int run_eq = 0;
    for (int base = 0; base < vocab; base += blockDim.x) {
      const int i = base + threadIdx.x;
      float e = 0.f;
      int eq = 0;
      uint32_t key = 0;
      if (i < vocab) {
        key = order_key(row[i]);
        eq = use_k && key == thr;
      }
      float sf = 0.f;
      int sn = eq;
      // the rank of an entry among those equal to the threshold needs the scan of `eq`
      // before its own probability is known, so scan the flags first
      float tf;
      int tn;
      block_scan(sf, sn, tf, tn);
      bool kept = false;
      if (i < vocab) {
        if (!use_k) kept = true;
        else if (key > thr) kept = true;
        else if (eq) kept = (run_eq + sn - 1) < need_eq;
        if (kept) e = expf(row[i] / temp - mx);
      }
      run_eq += tn;
      float cf = e;
      int dummy = kept ? 1 : 0;
      float chunk_total;
      int chunk_kept;
      block_scan(cf, dummy, chunk_total, chunk_kept);
      if (pass == 1) {
        if (kept && run + cf > target) atomicMin(&found, i);
        if (kept) last_kept = i;
        __syncthreads();
        if (found != 0x7fffffff) break;
      }
      run += chunk_total;
    }
    if (pass == 0) target = u * run;
  }
  __syncthreads();
  if (found == 0x7fffffff) {
    // u * total rounded up to the total itself: the last kept token
    __shared__ int lastk;
    if (threadIdx.x == 0) lastk = 0;
    __syncthreads();
    atomicMax(&lastk, last_kept);
    __syncthreads();
    if (threadIdx.x == 0) {
      out[rowi] = lastk;
      if (fb >= 0) feedback[fb] = lastk;
    }
  } else if (threadIdx.x == 0) {
    out[rowi] = found;
    if (fb >= 0) feedback[fb] = found;
  }
}

// ---- the same rule with the row held in shared memory ------------------------------------------
// A row of up to ~55k logits fits a CTA's shared memory.  It is read from global memory once;
// thread t owns the positions [t*C, (t+1)*C) (C odd: its walks are free of bank conflicts), so
// sums over threads in thread order are sums in index order.  The k-th largest logit is found
// by a radix select of four 8-bit digits over a 256-bin histogram (not 32 one-bit passes over
// the row), the kept entries' weights exp(x/T - max/T) replace the logits in place, one scan
// over the threads gives every thread the weight before its range, and the thread that holds
// the crossing of u * total finds the token.  Streaming the row from global memory for every
// pass (the kernel above, which stays for longer rows) took 90 us without top-k and 240-270 us
// with it at 50,257 logits.
constexpr int SS_THREADS = 1024;

__device__ float block_max_f(float v) {
  __shared__ float sh[SS_THREADS / 32];
  __shared__ float res;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float w = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : -INFINITY;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) w = fmaxf(w, __shfl_xor_sync(0xffffffffu, w, o));
    if (threadIdx.x == 0) res = w;
  }
  __syncthreads();
  const float r = res;
  __syncthreads();
  return r;
}

// Exclusive scan over the block in thread order of a float and an int; totals through tot_*.
__device__ void block_exclusive_scan(float& f, int& n, float& tot_f, int& tot_i) {
  __shared__ float wf[SS_THREADS / 32];
  __shared__ int wn[SS_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float fi = f;
  int ni = n;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float uf = __shfl_up_sync(0xffffffffu, fi, o);
    const int un = __shfl_up_sync(0xffffffffu, ni, o);
    if (lane >= o) {
      fi += uf;
      ni += un;
    }
  }
  if (lane == 31) {
    wf[warp] = fi;
    wn[warp] = ni;
  }
  float fe = __shfl_up_sync(0xffffffffu, fi, 1);      // the warp's sum before this lane
  int ne = __shfl_up_sync(0xffffffffu, ni, 1);
  if (lane == 0) {
    fe = 0.f;
    ne = 0;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    float a = lane < nw ? wf[lane] : 0.f;
    int b = lane < nw ? wn[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float ua = __shfl_up_sync(0xffffffffu, a, o);
      const int ub = __shfl_up_sync(0xffffffffu, b, o);
      if (lane >= o) {
        a += ua;
        b += ub;
      }
    }
    if (lane < nw) {
      wf[lane] = a;          // inclusive over the warps
      wn[lane] = b;
    }
  }
  __syncthreads();
  f = (warp > 0 ? wf[warp - 1] : 0.f) + fe;
  n = (warp > 0 ? wn[warp - 1] : 0) + ne;
  tot_f = wf[(blockDim.x >> 5) - 1];
  tot_i = wn[(blockDim.x >> 5) - 1];
  __syncthreads();
}

__global__ void __launch_bounds__(SS_THREADS)
sample_smem_kernel(int* __restrict__ out, const float* __restrict__ logits,
                   const float* __restrict__ temperature, const int* __restrict__ top_k,
                   const int* __restrict__ seed_lo, const int* __restrict__ seed_hi,
                   const int* __restrict__ position, int vocab, int* __restrict__ feedback,
                   const int* __restrict__ feedback_slot, const int* __restrict__ status_word) {
  extern __shared__ float s_row[];                  // [vocab]: logits, then weights (-1: dropped)
  __shared__ int hist[256];
  __shared__ int s_digit, s_above, s_found, s_last;
  const int rowi = blockIdx.x;
  const float* row = logits + (size_t)rowi * vocab;
  const float temp = temperature[rowi];
  pdl_wait();                       // the logits are what the previous kernel wrote
  if (status_word != nullptr && rowi == 0 && threadIdx.x == 0) out[gridDim.x] = *status_word;
  const int fb = (feedback != nullptr && feedback_slot != nullptr) ? feedback_slot[rowi] : -1;
  if (!(temp > 0.f)) {
    const ArgMax top = block_argmax(row, vocab);
    if (threadIdx.x == 0) {
      out[rowi] = top.i;
      if (fb >= 0) feedback[fb] = top.i;
    }
    return;
  }
  float m = -INFINITY;                              // the maximum needs no order: taken on the way in
#pragma unroll 8
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    s_row[i] = v;
    m = fmaxf(m, v);
  }
  if (threadIdx.x == 0) {
    s_found = 0x7fffffff;
    s_last = 0;
  }
  const float mx = block_max_f(m) / temp;           // (its barriers also publish the row)
  int C = (vocab + blockDim.x - 1) / blockDim.x;
  C |= 1;                                           // odd
  const int lo = min(vocab, (int)threadIdx.x * C), hi = min(vocab, lo + C);

  const int k = top_k[rowi];
  const bool use_k = k > 0 && k < vocab;
  uint32_t thr = 0;     // order key of the k-th largest logit; 0 keeps everything
  int need_eq = 0;      // how many entries equal to the threshold are kept (lowest indices)
  if (use_k) {
    uint32_t prefix = 0;
    int remaining = k;  // the k-th largest is the remaining-th largest among keys with the prefix
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (threadIdx.x < 256) hist[threadIdx.x] = 0;
      __syncthreads();
      const uint32_t above_mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      // (one atomic per entry: shared-memory atomics to the few digits most logits share
      // measured 4 us a pass; adding once per warp and digit through __match_any_sync 9 us)
      for (int i = lo; i < hi; ++i) {
        const uint32_t key = order_key(s_row[i]);
        if ((key & above_mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1);
      }
      __syncthreads();
      if (threadIdx.x < 32) {
        // lane l owns digits 8l .. 8l+7; digits are taken from the largest down
        const int lane = threadIdx.x;
        int c[8], grp = 0;
#pragma unroll
        for (int b = 0; b < 8; ++b) {
          c[b] = hist[8 * lane + b];
          grp += c[b];
        }
        int incl = grp;             // inclusive sum over lanes lane .. 31
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int u = __shfl_down_sync(0xffffffffu, incl, o);
          if (lane + o < 32) incl += u;
        }
        int run = incl - grp;       // keys with a digit above this lane's
        if (run < remaining && remaining <= incl) {
#pragma unroll
          for (int b = 7; b >= 0; --b) {
            if (run < remaining && remaining <= run + c[b]) {
              s_digit = 8 * lane + b;
              s_above = run;
            }
            run += c[b];
          }
        }
      }
      __syncthreads();
      prefix |= (uint32_t)s_digit << shift;
      remaining -= s_above;
    }
    thr = prefix;
    need_eq = remaining;
  }

  // entries equal to the threshold are kept in index order until k are reached
  int eq = 0;
  if (use_k) {                                      // the same for the whole CTA
    for (int i = lo; i < hi; ++i) eq += order_key(s_row[i]) == thr;
    float unused = 0.f, tf;
    int tn;
    block_exclusive_scan(unused, eq, tf, tn);       // eq: equal entries before this range
  }
  float sum = 0.f;
  for (int i = lo; i < hi; ++i) {
    const float v = s_row[i];
    bool kept = true;
    if (use_k) {
      const uint32_t key = order_key(v);
      kept = key > thr || (key == thr && eq++ < need_eq);
    }
    const float e = kept ? expf(v / temp - mx) : -1.f;
    s_row[i] = e;
    if (kept) sum += e;
  }
  float before = sum, total;
  int nz = 0, tnz;
  block_exclusive_scan(before, nz, total, tnz);     // before: weight of all kept entries below lo
  const float u = philox_uniform((uint32_t)seed_lo[rowi], (uint32_t)seed_hi[rowi],
                                 (uint32_t)position[rowi]);
  const float target = u * total;
  int cand = 0x7fffffff, last_kept = -1;
  float run = before;
  for (int i = lo; i < hi; ++i) {
    const float e = s_row[i];
    if (e >= 0.f) {
      run += e;
      if (cand == 0x7fffffff && run > target) cand = i;
      last_kept = i;
    }
  }
  if (cand != 0x7fffffff) atomicMin(&s_found, cand);
  if (last_kept >= 0) atomicMax(&s_last, last_kept);
  __syncthreads();
  if (threadIdx.x == 0) {
    // u * total rounded up to the total itself: the last kept token
    const int tok = s_found != 0x7fffffff ? s_found : s_last;
    out[rowi] = tok;
    if (fb >= 0) feedback[fb] = tok;
  }
}

}  // namespace hs

HS_EXPORT int hs_argmax(int* out, const float* logits, int rows, int vocab, void* stream) {
  if (!out || !logits) return HS_ERR_ARGUMENT;
  if (rows <= 0) return HS_OK;
  if (vocab <= 0) return HS_ERR_ARGUMENT;
  hs::argmax_kernel<<<rows, hs::SM_THREADS, 0, (cudaStream_t)stream>>>(out, logits, vocab);
  HS_LAUNCH_CHECK();
  return HS_OK;
}

// feedback / feedback_slot (both may be null): row i also stores its token to
// feedback[feedback_slot[i]] when that slot is not negative.  status_word (may be null): its
// value is stored to out[rows].
HS_EXPORT int hs_sample(int* out, const float* logits, const float* temperature, const int* top_k,
                        const int* seed_lo, const int* seed_hi, const int* position, int rows,
                        int vocab, int* feedback, const int* feedback_slot,
                        const int* status_word, void* stream) {
  if (!out || !logits || !temperature || !top_k || !seed_lo || !seed_hi || !position)
    return HS_ERR_ARGUMENT;
  if (rows <= 0) return HS_OK;
  if (vocab <= 0) return HS_ERR_ARGUMENT;
  // a row that fits shared memory (beside the kernel's own few KB) is read once
  const size_t row_bytes = (size_t)vocab * sizeof(float);
  cudaError_t le;
  if (row_bytes <= 220 * 1024) {
    static cudaError_t state = cudaErrorUnknown;
    if (state != cudaSuccess)
      state = cudaFuncSetAttribute(hs::sample_smem_kernel,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (state != cudaSuccess) return (int)state;
    le = hs_launch(hs::sample_smem_kernel, dim3(rows), dim3(hs::SS_THREADS), row_bytes,
                   (cudaStream_t)stream, hs_pdl_enabled(), out, logits, temperature, top_k,
                   seed_lo, seed_hi, position, vocab, feedback, feedback_slot, status_word);
  } else {
    le = hs_launch(hs::sample_kernel, dim3(rows), dim3(hs::SM_THREADS), 0, (cudaStream_t)stream,
                   hs_pdl_enabled(), out, logits, temperature, top_k, seed_lo, seed_hi, position,
                   vocab, feedback, feedback_slot, status_word);
  }
  if (le != cudaSuccess) return (int)le;
  HS_LAUNCH_CHECK();
  return HS_OK;
}
