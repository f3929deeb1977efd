// A whole decode step in ONE persistent kernel (bfloat16 serving path, up to 16 single-query
// tokens, heads of 64, 16-token pages, pre-norm layers of LayerNorm / attention / dense
// feed-forward, learned positions, linear head).
//
// Why.  Layer by layer a decode step is five dependent kernels per layer (LayerNorm+QKV,
// attention, attention out, LayerNorm+fc, MLP out).  Each moves a few megabytes and lasts 4-8 us
// of which about one is the transfer: the rest is launch, ramp-up, the wait for the kernel
// before, and the tail.  Here the step is one cooperative launch of one CTA per SM:
//
//   * a PRODUCER warp per CTA streams everything that does not depend on this step's
//     arithmetic - the CTA's share of every weight matrix of every layer, the head, and the
//     cache pages of earlier positions - through a ring of 16 KB shared-memory slots (one
//     mbarrier pair per slot), in the order the CTA will use it, as far ahead as the ring
//     allows.  Weights come from a copy packed for this kernel when the model is bound: every
//     [16 features x 512 k] unit is 16 contiguous kilobytes, already in the XOR-swizzled
//     layout ldmatrix wants, so a unit is ONE bulk copy (cp.async.bulk) of a contiguous run -
//     with the matrices as stored, [features, k], the same unit is 128 pieces of 128 bytes
//     2 KB apart, which HBM served at under a third of its rate.  Cache pages come through a
//     tensor map (cp.async.bulk.tensor, 128-byte swizzle), 2 KB a box.  The stream never stops
//     at a phase boundary: HBM stays busy while the CTAs synchronise;
//   * eight CONSUMER warps per CTA walk the phases.  A phase's work is cut into items of 16
//     output features (linear phases: the weight tile is the 16-row operand of mma.sync
//     m16n8k16, the tokens are its 8- or 16-wide operand; the eight warps split k and add
//     their parts in warp order through shared memory) or of one (token, head, context
//     slice) (attention: online softmax in float32 over pages of 16 keys, the token's own key
//     and value row patched into the tile and appended to the page);
//   * between phases the CTAs meet at a grid-wide barrier (one counter in global memory).
//     Every wait - ring slots and grid barrier - is bounded: when one runs out the kernel sets
//     HS_STATUS_PIPELINE_TIMEOUT, raises an abort word that ends all other waits, runs to its
//     end without touching anything out of bounds, and returns.
//
// Sums are formed in float32 in an order that depends on the element alone (k in order within a
// warp, warps in order), so a token's result does not depend on the batch around it.  The
// float32 residual stream is updated in place by the CTA that owns the feature tile.
//
// What the reference does for the same step: heteroserve/model/torch_engine.py:195-253
// (decode_batch_paged: one library call per operation and layer) with
// heteroserve/model/paged_attn_v3.py:75-232 for the attention.
#include "tcgen05.cuh"

#include <string.h>

namespace hs {

constexpr int PD_CW = 8;                          // consumer warps
constexpr int PD_THREADS = (PD_CW + 1) * 32;      // + the producer warp
constexpr int PD_SLOTS = 8;
constexpr int PD_SLOT_BYTES = 16384;              // 8 boxes
constexpr int PD_BOX_BYTES = 2048;                // 16 rows x 64 bf16, 128-byte swizzle
constexpr int PD_MT = 16;                         // token rows of an activation tile
constexpr int PD_CK = 512;                        // k per unit (one ring slot) and per chunk
constexpr int PD_AROW = PD_CK * 2 + 16;           // bytes per token row of a chunk (padded)
constexpr int PD_ACHUNK = PD_MT * PD_AROW;        // 16,640
constexpr int PD_ACHUNKS = 4;                     // a row of up to 2,048 stays resident
constexpr int PD_RED_TILE = 16 * 17;              // floats of one warp's partial tile (padded rows)
constexpr int PD_RED_BYTES = PD_CW * PD_RED_TILE * 4;
constexpr int PD_MAX_E = PD_ACHUNKS * PD_CK;      // widest row a norm takes here
constexpr int PD_BIAS_ITEMS = 8;                  // tiles per phase whose bias is staged
constexpr int PD_PAR_BYTES = (2 * PD_MAX_E + 4 * PD_BIAS_ITEMS * 16) * 4;
constexpr int PD_D = 64;                          // head size
constexpr int PD_PS = 16;                         // page size
constexpr int PD_KV_PAGES = 4;                    // pages (keys and values) per ring slot
constexpr uint32_t PD_GRID_SPIN = 1u << 22;

constexpr int PD_OFF_ACT = PD_SLOTS * PD_SLOT_BYTES;
constexpr int PD_OFF_RED = PD_OFF_ACT + PD_ACHUNKS * PD_ACHUNK;
constexpr int PD_OFF_BAR = PD_OFF_RED + PD_RED_BYTES;
constexpr int PD_OFF_PAR = PD_OFF_BAR + 256;      // staged norm parameters and biases
constexpr int PD_SMEM = PD_OFF_PAR + PD_PAR_BYTES + 1024;   // + slack to align the base

struct alignas(64) PdLayer {
  const __nv_bfloat16* w_qkv;                     // packed: [tile of 16 features][k / 64][16][64]
  const __nv_bfloat16* w_out;
  const __nv_bfloat16* w_fc;
  const __nv_bfloat16* w_mlp;
  const float* b_qkv;
  const float* b_out;
  const float* b_fc;
  const float* b_mlp;
  const float* ln1_g;
  const float* ln1_b;
  const float* ln2_g;
  const float* ln2_b;
  float scale, eps1, eps2;
  int act;
  long long kv_row0;                              // first row of this layer's cache entry in the kv map
  int pad[2];
};
static_assert(sizeof(PdLayer) % 64 == 0, "PdLayer must keep its tensor maps 64-byte aligned");

struct alignas(64) PdTables {
  CUtensorMap kv;                                 // every cache entry: [rows, 64], boxes of 16 x 64
  const __nv_bfloat16* w_head;                    // packed like the layers' matrices
  long long pad[7];
};

struct PdParams {
  const PdLayer* layers;
  const PdTables* tables;
  const __nv_bfloat16* wte;
  const __nv_bfloat16* wpe;
  const float* lnf_g;
  const float* lnf_b;
  float eps_f;
  int n_layers, E, I, V, H, n_pos;
  __nv_bfloat16* pool;                            // the cache group's storage (for the append)
  int num_pages, max_pages;
  // buffers of the step
  float* x;                                       // [MT, E] residual stream
  __nv_bfloat16* qkv;                             // [M, 3E]
  __nv_bfloat16* att;                             // [M, E]
  __nv_bfloat16* u;                               // [M, I]
  float* logits;                                  // [W, V]
  float* att_acc;                                 // [M, H, S, 64]   (S > 1)
  float* att_ml;                                  // [M, H, S, 2]
  float* amax_val;                                // [grid, 16]
  int* amax_idx;                                  // [grid, 16]
  int* tokens_out;                                // [Wcap + 1]: tokens, then the status word
  int* feedback;                                  // token each request sampled last, by slot
  // metadata of the step (device)
  const int* tok_ids;
  const int* tok_pos;
  const int* tok_req;
  const int* table;                               // [requests, max_pages]
  const int* logit_rows;                          // [W]
  const int* samp_slot;                           // [W]
  const int* plan_head;                           // [2]: the longest context among the tokens
  int n_feedback;
  int M, W, Wcap, S;
  unsigned* sync;                                 // [0] barrier arrivals, [1] abort
  int* status;
  int stop_after;                                 // > 0: leave after that many grid barriers (tests)
  unsigned long long* timing;                     // tuning builds: see PdMarks
};

// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void pd_ldsm4(uint32_t (&r)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
__device__ __forceinline__ void pd_ldsm4_t(uint32_t (&r)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(saddr));
}
__device__ __forceinline__ void pd_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                       uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float pd_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pd_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}
__device__ __forceinline__ void pd_bar_consumers() {        // the eight consumer warps
  asm volatile("bar.sync 1, 256;" ::: "memory");
}
__device__ __forceinline__ unsigned pd_ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float gelu_tanh_fast(float u) {   // hardware tanh, as the other bf16 epilogues
  const float k = 0.7978845608028654f;
  float inner = k * (u + 0.044715f * u * u * u), t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(inner));
  return 0.5f * u * (1.0f + t);
}

// Tuning builds (-DHS_PHASE_MARKS): lane 0 of the producer and thread 0 of the consumers of the
// every 21st CTA store the nanosecond timer with a tag: buffer[(cta / 21 * 2 + role) * 512 + n].
struct PdMarks {
#ifdef HS_PHASE_MARKS
  unsigned long long* buf;
  int n = 0;
  __device__ __forceinline__ PdMarks(unsigned long long* b, int role)
      : buf(b && blockIdx.x % 21 == 0 ? b + ((size_t)(blockIdx.x / 21) * 2 + role) * 512 : nullptr) {}
  __device__ __forceinline__ void operator()(int tag) {
    if (buf && n < 511) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      buf[n++] = (t << 8) | (unsigned)(tag & 255);
      buf[511] = n;
    }
  }
#else
  __device__ __forceinline__ PdMarks(unsigned long long*, int) {}
  __device__ __forceinline__ void operator()(int) {}
#endif
};

// Contiguous global -> shared copy whose bytes are counted on an mbarrier (16-byte aligned
// addresses, a multiple of 16 bytes).
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes,
                                          uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void pd_cp16(void* smem_dst, const void* gsrc) {     // 16-byte cp.async
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc)
               : "memory");
}
__device__ __forceinline__ void pd_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void pd_cp_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

struct PdShared {
  uint8_t* base;          // 1024-byte aligned
  uint64_t* full;         // [PD_SLOTS]
  uint64_t* empty;        // [PD_SLOTS]
  volatile int* abort;    // CTA-local copy of the abort word
};

// Waits on a ring barrier.  After an abort every wait returns at once.
__device__ __forceinline__ void pd_wait(const PdShared& sh, uint64_t* bar, uint32_t parity,
                                        const PdParams& p) {
  if (*sh.abort) return;
  if (!mbar_wait(bar, parity, p.status, 1u << 21)) {
    *sh.abort = 1;
    atomicExch(p.sync + 1, 1u);
  }
}

// Grid-wide barrier of the consumer warps of all CTAs.  `n` counts the barriers passed.
__device__ __noinline__ void pd_grid_sync(const PdShared sh, const PdParams& p, int& n) {
  pd_bar_consumers();
  if (threadIdx.x == 0 && !*sh.abort) {
    __threadfence();
    atomicAdd(p.sync, 1u);
    const unsigned target = (unsigned)(n + 1) * gridDim.x;
    uint32_t spin = 0;
    while (pd_ld_acquire(p.sync) < target) {
      if (++spin >= PD_GRID_SPIN || ((spin & 255u) == 0 && pd_ld_acquire(p.sync + 1))) {
        if (spin >= PD_GRID_SPIN) {
          atomicOr(p.status, HS_STATUS_PIPELINE_TIMEOUT);
          atomicExch(p.sync + 1, 1u);
        }
        *sh.abort = 1;
        break;
      }
    }
    __threadfence();
  }
  ++n;
  pd_bar_consumers();
}

// Tiles of a phase are dealt round-robin, starting at CTA `rot`: the first tile of this CTA.
__device__ __forceinline__ int pd_first_tile(int rot) {
  const int G = gridDim.x;
  return ((int)blockIdx.x - rot % G + G) % G;
}

// ------------------------------------------------------------------------------------------
// The producer: one lane walks the same schedule as the consumers and keeps the ring full.
struct PdProducer {
  const PdShared& sh;
  const PdParams& p;
  uint32_t fill = 0;

  __device__ __forceinline__ PdProducer(const PdShared& s, const PdParams& q) : sh(s), p(q) {}

  __device__ __forceinline__ uint8_t* open_slot(int boxes) {
    const int s = fill % PD_SLOTS;
    pd_wait(sh, &sh.empty[s], ((fill / PD_SLOTS) & 1) ^ 1, p);
    mbar_expect_tx(&sh.full[s], (uint32_t)boxes * PD_BOX_BYTES);
    return sh.base + (size_t)s * PD_SLOT_BYTES;
  }
  // the units of one 16-feature tile: k in steps of 512, each one contiguous run of the packed copy
  __device__ __forceinline__ void weight_tile(const __nv_bfloat16* packed, int tile, int K) {
    const __nv_bfloat16* src = packed + (size_t)tile * (K / 64) * (PD_BOX_BYTES / 2);
    for (int k0 = 0; k0 < K && !*sh.abort; k0 += PD_CK) {
      const int boxes = min(8, (K - k0) / 64);
      uint8_t* dst = open_slot(boxes);
      if (*sh.abort) return;
      bulk_load(dst, src + (size_t)(k0 / 64) * (PD_BOX_BYTES / 2), boxes * PD_BOX_BYTES,
                &sh.full[fill % PD_SLOTS]);
      ++fill;
    }
  }
  __device__ __forceinline__ void weight_phase(const __nv_bfloat16* packed, int n_tiles, int rot,
                                               int K) {
    for (int j = pd_first_tile(rot); j < n_tiles && !*sh.abort; j += gridDim.x)
      weight_tile(packed, j, K);
  }
};

// ------------------------------------------------------------------------------------------
// Consumer side of the ring.
struct PdConsumer {
  const PdShared& sh;
  const PdParams& p;
  uint32_t take = 0;

  __device__ __forceinline__ PdConsumer(const PdShared& s, const PdParams& q) : sh(s), p(q) {}
  __device__ __forceinline__ const uint8_t* wait_slot() {
    const int s = take % PD_SLOTS;
    pd_wait(sh, &sh.full[s], (take / PD_SLOTS) & 1, p);
    return sh.base + (size_t)s * PD_SLOT_BYTES;
  }
  __device__ __forceinline__ void release_slot() {       // every consumer warp, once per slot
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(&sh.empty[take % PD_SLOTS]);
    ++take;
  }
};

// One unit (up to 8 boxes of 64 k) of a 16-feature tile: warp w multiplies box w with the
// tokens' activations of the same k range.  `act` points at the chunk that holds k0.
__device__ __forceinline__ void pd_unit_mma(float (&acc)[2][4], const uint8_t* slot, int boxes,
                                            uint32_t act_chunk, bool two, int warp, int lane) {
  if (warp >= boxes) return;
  const uint32_t box = smem_u32(slot) + warp * PD_BOX_BYTES;
  const int mi = lane >> 3, r8 = lane & 7;
  const int a_row = r8 + (mi & 1) * 8;                          // A: rows 0-7 / 8-15, k halves
  const uint32_t a_base = box + a_row * 128;
  // B: tokens r8 (+8 for matrices 2,3), k halves by mi & 1
  const uint32_t b_base = act_chunk + (r8 + (mi >> 1) * 8) * PD_AROW + warp * 128 + (mi & 1) * 16;
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    uint32_t a[4], b[4];
    pd_ldsm4(a, a_base + (((ks * 2 + (mi >> 1)) ^ (a_row & 7)) << 4));
    pd_ldsm4(b, b_base + ks * 32);
    pd_mma(acc[0], a, b[0], b[1]);
    if (two) pd_mma(acc[1], a, b[2], b[3]);
  }
}

// The eight warps' partial 16 x 16 tiles are added in warp order; thread (feature f = tid % 16,
// token t = tid / 16) returns the sum for its element.  Tiles lie token-major with a row of 17
// floats, so that neither the stores nor the loads meet in a bank.
__device__ __forceinline__ float pd_reduce_tile(const float (&acc)[2][4], float* red, int warp,
                                                int lane, int boxes_max) {
  const int g = lane >> 2, t4 = lane & 3;
  float* mine = red + warp * PD_RED_TILE;
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    const int col = nt * 8 + t4 * 2;
    mine[col * 17 + g] = acc[nt][0];
    mine[(col + 1) * 17 + g] = acc[nt][1];
    mine[col * 17 + g + 8] = acc[nt][2];
    mine[(col + 1) * 17 + g + 8] = acc[nt][3];
  }
  pd_bar_consumers();
  const int f = threadIdx.x & 15, t = threadIdx.x >> 4;
  float sum = 0.f;
  const int nw = boxes_max < PD_CW ? boxes_max : PD_CW;
  for (int w = 0; w < nw; ++w) sum += red[w * PD_RED_TILE + t * 17 + f];
  pd_bar_consumers();
  return sum;
}

// ---- vectors staged in shared memory ahead of the phase that uses them (cp.async: the copies
// fly while the CTA waits at the grid barrier).  After the barrier: pd_cp_wait + CTA barrier.
__device__ __forceinline__ float* pd_par_g(const PdShared& sh) { return (float*)(sh.base + PD_OFF_PAR); }
__device__ __forceinline__ float* pd_par_b(const PdShared& sh) { return pd_par_g(sh) + PD_MAX_E; }
__device__ __forceinline__ float* pd_par_bias(const PdShared& sh, int which) {
  return pd_par_b(sh) + PD_MAX_E + which * (PD_BIAS_ITEMS * 16);
}
__device__ __forceinline__ void pd_stage_norm(const PdShared& sh, const float* g, const float* b,
                                              int E) {
  for (int i = threadIdx.x; i < E / 4; i += PD_CW * 32) {
    pd_cp16(pd_par_g(sh) + 4 * i, g + 4 * i);
    pd_cp16(pd_par_b(sh) + 4 * i, b + 4 * i);
  }
}
// the bias of this CTA's first PD_BIAS_ITEMS tiles of a phase (zeros when there is no bias)
__device__ __forceinline__ void pd_stage_bias(const PdShared& sh, int which, const float* bias,
                                              int n_tiles, int rot) {
  const int q = threadIdx.x >> 2, piece = threadIdx.x & 3;
  if (q >= PD_BIAS_ITEMS) return;
  const int tile = pd_first_tile(rot) + q * (int)gridDim.x;
  float* dst = pd_par_bias(sh, which) + q * 16 + piece * 4;
  if (tile < n_tiles && bias) pd_cp16(dst, bias + (size_t)tile * 16 + piece * 4);
  else *(float4*)dst = make_float4(0.f, 0.f, 0.f, 0.f);
}

// LayerNorm of the step's rows into the activation chunks (bf16; rows past n_rows are zero).
// Warp w takes rows w and w + 8.  The norm's weight and bias are staged in shared memory.
// `rows` (may be null) picks the source rows; `embed` forms the source from the token and
// position tables instead of reading x, and CTA r % grid stores row r of the stream.
__device__ __noinline__ void pd_layernorm_rows(const PdShared sh, const PdParams& p, float eps, const int* rows,
                                  int n_rows, bool embed, int rows_alloc, int warp, int lane) {
  const int E = p.E;
  uint8_t* act = sh.base + PD_OFF_ACT;
  const size_t cstride = (size_t)rows_alloc * PD_AROW;
  const float* sg = pd_par_g(sh);
  const float* sb = pd_par_b(sh);
  for (int r = warp; r < rows_alloc; r += PD_CW) {
    bool live = r < n_rows;
    int src = r;
    if (live && rows) src = rows[r];
    if (live && !embed && (src < 0 || src >= p.M)) live = false;
    int tok = 0, pos = 0;
    if (live && embed) {
      if (p.tok_req[r] < 0) live = false;
      tok = p.tok_ids[r];
      pos = p.tok_pos[r];
      if (live && tok < 0) {                          // the token the device sampled last
        const int s = -tok - 1;
        tok = s < p.n_feedback ? p.feedback[s] : -1;
      }
      if (live && (tok < 0 || tok >= p.V)) {
        if (lane == 0) atomicOr(p.status, HS_STATUS_BAD_TOKEN);
        live = false;
      }
      if (live && (pos < 0 || pos >= p.n_pos)) {
        if (lane == 0) atomicOr(p.status, HS_STATUS_BAD_POSITION);
        live = false;
      }
    }
    float4 v[16];                                     // E <= 2048: 16 float4 per lane
    // every load of the row is in flight before the first is used
    if (embed) {
      uint2 a[16], w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int c = i * 128 + lane * 4;
        a[i] = w[i] = make_uint2(0u, 0u);
        if (live && c < E) {
          a[i] = *(const uint2*)(p.wte + (size_t)tok * E + c);
          w[i] = *(const uint2*)(p.wpe + (size_t)pos * E + c);
        }
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const __nv_bfloat162 a0 = *(const __nv_bfloat162*)&a[i].x, a1 = *(const __nv_bfloat162*)&a[i].y;
        const __nv_bfloat162 w0 = *(const __nv_bfloat162*)&w[i].x, w1 = *(const __nv_bfloat162*)&w[i].y;
        v[i] = make_float4(__low2float(a0) + __low2float(w0), __high2float(a0) + __high2float(w0),
                           __low2float(a1) + __low2float(w1), __high2float(a1) + __high2float(w1));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int c = i * 128 + lane * 4;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live && c < E) v[i] = __ldcg((const float4*)(p.x + (size_t)src * E + c));
      }
    }
    if (embed && r < p.M && (int)blockIdx.x == r % (int)gridDim.x) {
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int c = i * 128 + lane * 4;
        if (c < E) *(float4*)(p.x + (size_t)r * E + c) = v[i];
      }
    }
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) sum += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    const float mean = warp_sum(sum) / E;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (i * 128 + lane * 4 < E) {
        const float d0 = v[i].x - mean, d1 = v[i].y - mean, d2 = v[i].z - mean, d3 = v[i].w - mean;
        sq += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
      }
    }
    const float inv = rsqrtf(warp_sum(sq) / E + eps);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int c = i * 128 + lane * 4;
      if (c < E) {
        uint2 o = make_uint2(0u, 0u);
        if (live) {
          const float4 gg = *(const float4*)(sg + c), bb = *(const float4*)(sb + c);
          o.x = pd_pack((v[i].x - mean) * inv * gg.x + bb.x, (v[i].y - mean) * inv * gg.y + bb.y);
          o.y = pd_pack((v[i].z - mean) * inv * gg.z + bb.z, (v[i].w - mean) * inv * gg.w + bb.w);
        }
        *(uint2*)(act + (size_t)(c / PD_CK) * cstride + (size_t)r * PD_AROW + (c % PD_CK) * 2) = o;
      }
    }
  }
}

// A [M, K] bf16 matrix of the step into the activation chunks (K up to what the chunks of
// `rows_alloc` rows hold), zero rows past M.
__device__ __noinline__ void pd_load_rows(const PdShared sh, const __nv_bfloat16* src, int M, int K, int ld,
                             int rows_alloc) {
  uint8_t* act = sh.base + PD_OFF_ACT;
  const size_t cstride = (size_t)rows_alloc * PD_AROW;
  const int pieces = K / 8;                         // 16-byte pieces per row
  for (int e = threadIdx.x; e < rows_alloc * pieces; e += PD_CW * 32) {
    const int r = e / pieces, c = (e - r * pieces) * 8;
    uint4 q = make_uint4(0, 0, 0, 0);
    if (r < M) q = __ldcg((const uint4*)(src + (size_t)r * ld + c));
    *(uint4*)(act + (size_t)(c / PD_CK) * cstride + (size_t)r * PD_AROW + (c % PD_CK) * 2) = q;
  }
}

// The attention output rows from the slices' partial results (S > 1): for every live (token,
// head) the slices are merged in slice order.  Thread (row, head, 16 dims).
__device__ __noinline__ void pd_load_merged_attention(const PdShared sh, const PdParams& p, int rows_alloc) {
  uint8_t* act = sh.base + PD_OFF_ACT;
  const size_t cstride = (size_t)rows_alloc * PD_AROW;
  const int E = p.E, S = p.S;
  const int per_row = E / 16;                       // 16-dim groups per row
  for (int e = threadIdx.x; e < rows_alloc * per_row; e += PD_CW * 32) {
    const int r = e / per_row, c = (e - r * per_row) * 16;
    float out[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) out[j] = 0.f;
    if (r < p.M && p.tok_req[r] >= 0) {
      const int h = c / PD_D, d = c % PD_D;
      const size_t base = ((size_t)r * p.H + h) * S;
      float ms[8], ls[8];
      float gm = -INFINITY;
#pragma unroll
      for (int s2 = 0; s2 < 8; ++s2) {
        ms[s2] = -INFINITY;
        ls[s2] = 0.f;
        if (s2 < S) {
          const float2 ml = __ldcg((const float2*)&p.att_ml[(base + s2) * 2]);
          ms[s2] = ml.x;
          ls[s2] = ml.y;
        }
        gm = fmaxf(gm, ms[s2]);
      }
      float gl = 0.f;
#pragma unroll
      for (int s2 = 0; s2 < 8; ++s2) {
        ms[s2] = (ms[s2] == -INFINITY) ? 0.f : pd_ex2(ms[s2] - gm);      // now the weight
        gl += ls[s2] * ms[s2];
      }
      const float inv = gl > 0.f ? 1.f / gl : 0.f;
#pragma unroll
      for (int s2 = 0; s2 < 8; ++s2) {
        if (s2 < S && ms[s2] > 0.f) {
          const float4* a = (const float4*)&p.att_acc[(base + s2) * PD_D + d];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 q = __ldcg(a + j);
            out[4 * j] += q.x * ms[s2]; out[4 * j + 1] += q.y * ms[s2];
            out[4 * j + 2] += q.z * ms[s2]; out[4 * j + 3] += q.w * ms[s2];
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) out[j] *= inv;
    }
    uint4 lo, hi;
    lo.x = pd_pack(out[0], out[1]); lo.y = pd_pack(out[2], out[3]);
    lo.z = pd_pack(out[4], out[5]); lo.w = pd_pack(out[6], out[7]);
    hi.x = pd_pack(out[8], out[9]); hi.y = pd_pack(out[10], out[11]);
    hi.z = pd_pack(out[12], out[13]); hi.w = pd_pack(out[14], out[15]);
    uint8_t* dst = act + (size_t)(c / PD_CK) * cstride + (size_t)r * PD_AROW + (c % PD_CK) * 2;
    *(uint4*)dst = lo;
    *(uint4*)(dst + 16) = hi;
  }
}

enum { PD_EPI_QKV = 0, PD_EPI_RESIDUAL = 1, PD_EPI_ACT = 2, PD_EPI_LOGITS = 3 };

struct PdBest {
  float val = -INFINITY;
  int idx = 0x7fffffff;
};

// The items of a linear phase whose activations are resident in the chunks.  `bias_s` is the
// staged bias of this CTA's first PD_BIAS_ITEMS tiles (null: none); `bias` the whole vector.
__device__ __noinline__ uint32_t pd_linear_resident(const PdShared sh, const PdParams& p, uint32_t take,
                                   int n_features, int rot, int K, const float* bias,
                                   const float* bias_s, int epi, int act_kind, int rows_out,
                                   int rows_alloc, PdBest* best, int warp, int lane) {
  PdConsumer ring(sh, p);
  ring.take = take;
  const bool two = rows_out > 8;
  const uint32_t act0 = smem_u32(sh.base + PD_OFF_ACT);
  const uint32_t cstride = (uint32_t)rows_alloc * PD_AROW;
  float* red = (float*)(sh.base + PD_OFF_RED);
  const int n_tiles = (n_features + 15) / 16;
  int q = 0;
  for (int j = pd_first_tile(rot); j < n_tiles; j += gridDim.x, ++q) {
    const int f = j * 16 + (threadIdx.x & 15), t = threadIdx.x >> 4;
    const bool mine = f < n_features && t < rows_out;
    // what the epilogue needs from global memory is asked for before the multiplications
    float xold = 0.f, bv = 0.f;
    if (mine && epi == PD_EPI_RESIDUAL) xold = __ldcg(p.x + (size_t)t * p.E + f);
    if (mine && bias) bv = (bias_s && q < PD_BIAS_ITEMS) ? bias_s[q * 16 + (threadIdx.x & 15)] : bias[f];
    float acc[2][4] = {};
    int boxes_max = 0;
    for (int k0 = 0; k0 < K; k0 += PD_CK) {
      const int boxes = min(8, (K - k0) / 64);
      boxes_max = max(boxes_max, boxes);
      const uint8_t* slot = ring.wait_slot();
      pd_unit_mma(acc, slot, boxes, act0 + (k0 / PD_CK) * cstride, two, warp, lane);
      ring.release_slot();
    }
    const float sum = pd_reduce_tile(acc, red, warp, lane, boxes_max);
    if (mine) {
      float v = sum + bv;
      if (epi == PD_EPI_QKV) {
        p.qkv[(size_t)t * 3 * p.E + f] = __float2bfloat16_rn(v);
      } else if (epi == PD_EPI_RESIDUAL) {
        p.x[(size_t)t * p.E + f] = xold + v;
      } else if (epi == PD_EPI_ACT) {
        v = act_kind == HS_ACT_GELU_TANH ? gelu_tanh_fast(v) : apply_act(v, act_kind);
        p.u[(size_t)t * p.I + f] = __float2bfloat16_rn(v);
      } else {
        p.logits[(size_t)t * p.V + f] = v;
        if (v > best->val || (v == best->val && f < best->idx)) {
          best->val = v;
          best->idx = f;
        }
      }
    }
  }
  return ring.take;
}

// The MLP's second matrix when k = I exceeds what stays resident: the activations of a tile are
// streamed through four chunk buffers, three chunks ahead of the unit being multiplied.
__device__ __noinline__ uint32_t pd_linear_streamed(const PdShared sh, const PdParams& p, uint32_t take,
                                   int n_features, int rot, int K, const float* bias,
                                   const float* bias_s, int rows_out, int warp, int lane) {
  PdConsumer ring(sh, p);
  ring.take = take;
  const bool two = rows_out > 8;
  uint8_t* act = sh.base + PD_OFF_ACT;
  const uint32_t act0 = smem_u32(act);
  float* red = (float*)(sh.base + PD_OFF_RED);
  const int n_tiles = (n_features + 15) / 16;
  const int units = (K + PD_CK - 1) / PD_CK;
  // thread -> 16-byte pieces of a chunk: 16 rows x 64 pieces = 1024 pieces, 4 per thread
  auto fetch = [&](int unit, uint4 (&q)[4]) {
    const int k0 = unit * PD_CK, kw = min(PD_CK, K - k0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = threadIdx.x + i * 256, r = e >> 6, c = (e & 63) * 8;
      q[i] = make_uint4(0, 0, 0, 0);
      if (r < p.M && c < kw) q[i] = __ldcg((const uint4*)(p.u + (size_t)r * p.I + k0 + c));
    }
  };
  auto stash = [&](int unit, const uint4 (&q)[4]) {
    uint8_t* dst = act + (size_t)(unit % PD_ACHUNKS) * PD_ACHUNK;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = threadIdx.x + i * 256, r = e >> 6, c = (e & 63) * 8;
      *(uint4*)(dst + (size_t)r * PD_AROW + c * 2) = q[i];
    }
  };
  int qi = 0;
  for (int j = pd_first_tile(rot); j < n_tiles; j += gridDim.x, ++qi) {
    const int f = j * 16 + (threadIdx.x & 15), t = threadIdx.x >> 4;
    const bool mine = f < n_features && t < rows_out;
    float xold = 0.f, bv = 0.f;
    if (mine) xold = __ldcg(p.x + (size_t)t * p.E + f);
    if (mine && bias) bv = (bias_s && qi < PD_BIAS_ITEMS) ? bias_s[qi * 16 + (threadIdx.x & 15)] : bias[f];
    float acc[2][4] = {};
    uint4 q[4];
    for (int un = 0; un < 3 && un < units; ++un) {
      fetch(un, q);
      stash(un, q);
    }
    pd_bar_consumers();
    for (int un = 0; un < units; ++un) {
      const bool more = un + 3 < units;
      if (more) fetch(un + 3, q);
      const int boxes = min(8, (K - un * PD_CK) / 64);
      const uint8_t* slot = ring.wait_slot();
      pd_unit_mma(acc, slot, boxes, act0 + (un % PD_ACHUNKS) * PD_ACHUNK, two, warp, lane);
      ring.release_slot();
      if (more) stash(un + 3, q);          // the buffer of unit un - 1: every warp is past it
      pd_bar_consumers();
    }
    const float sum = pd_reduce_tile(acc, red, warp, lane, 8);
    if (mine) p.x[(size_t)t * p.E + f] = xold + sum + bv;
  }
  return ring.take;
}

// Geometry of an attention item, the same on the producer and the consumer side.
struct PdAttItem {
  int t, h, s, pos, req, k_begin, k_end, units;
};
__device__ __forceinline__ bool pd_att_item(const PdParams& p, int span, int i, PdAttItem& it) {
  it.s = i % p.S;
  it.h = (i / p.S) % p.H;
  it.t = i / (p.S * p.H);
  it.req = p.tok_req[it.t];
  it.pos = p.tok_pos[it.t];
  it.units = 0;
  it.k_begin = it.k_end = 0;
  if (it.req < 0 || it.pos < 0 || it.pos / PD_PS >= p.max_pages) return false;
  it.k_begin = it.s * span;
  it.k_end = min((it.s + 1) * span, it.pos + 1);
  if (it.k_end > it.k_begin) it.units = (it.k_end - it.k_begin + 63) / 64;
  return true;
}
__device__ __forceinline__ int pd_att_first() {      // attention items start at the last CTA
  return (int)gridDim.x - 1 - (int)blockIdx.x;
}

// The attention phase of one layer for this CTA: its (token, head, slice) items one after
// the other.  Returns the ring position.
__device__ __noinline__ uint32_t pd_attention_phase(const PdShared sh, const PdParams& p,
                                                    uint32_t take, const PdLayer* L, int span,
                                                    int n_att, int warp, int lane) {
  PdConsumer ring(sh, p);
  ring.take = take;
  const int E = p.E, H = p.H, M = p.M, G = gridDim.x;
  float* red = (float*)(sh.base + PD_OFF_RED);
  for (int i = pd_att_first(); i < n_att; i += G) {
    PdAttItem it;
    const bool ok = pd_att_item(p, span, i, it);
    const __nv_bfloat16* own = p.qkv + (size_t)it.t * 3 * E;
    // the query of this head: row 0 of the 16-row operand
    uint32_t qf[4][4];
    {
      const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        const int c = ks * 16 + t4 * 2;
        qf[ks][0] = (ok && g == 0) ? __ldcg((const unsigned*)(own + it.h * PD_D + c)) : 0u;
        qf[ks][2] = (ok && g == 0) ? __ldcg((const unsigned*)(own + it.h * PD_D + c + 8)) : 0u;
        qf[ks][1] = qf[ks][3] = 0u;
      }
    }
    float o[8][4];
#pragma unroll
    for (int d = 0; d < 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const float sl2 = L->scale * 1.4426950408889634f;
    const bool holds_own = ok && it.pos >= it.k_begin && it.pos < it.k_end;
    int page_own = -1;
    if (holds_own) {
      page_own = p.table[(size_t)it.req * p.max_pages + it.pos / PD_PS];
      if (page_own < 0 || page_own >= p.num_pages) {
        if (threadIdx.x == 0) atomicOr(p.status, HS_STATUS_BAD_PAGE);
        page_own = -1;
      }
    }
    for (int un = 0; un < it.units; ++un) {
      const uint8_t* slot = ring.wait_slot();
      const int page_in_unit = warp & 3;
      const int key0 = it.k_begin + un * 64 + page_in_unit * PD_PS;     // first key of my page
      const bool mine = ((un & 1) == (warp >> 2)) && key0 < it.k_end;
      if (mine) {
        uint8_t* kt = const_cast<uint8_t*>(slot) + (2 * page_in_unit) * PD_BOX_BYTES;
        uint8_t* vt = kt + PD_BOX_BYTES;
        if (holds_own && it.pos >= key0 && it.pos < key0 + PD_PS) {
          // the token's own row: from the projection's output into the tile and the page
          const int row = it.pos - key0;
          if (lane < 16) {
            const bool is_v = lane >= 8;
            const int ch = lane & 7;
            const uint4 val = __ldcg((const uint4*)(own + (is_v ? 2 : 1) * E + it.h * PD_D + ch * 8));
            *(uint4*)((is_v ? vt : kt) + row * 128 + ((ch ^ (row & 7)) << 4)) = val;
            if (page_own >= 0) {
              __nv_bfloat16* dst = p.pool + (size_t)(L->kv_row0 +
                  (((long long)page_own * 2 + (is_v ? 1 : 0)) * H + it.h) * PD_PS + row) * PD_D + ch * 8;
              *(uint4*)dst = val;
            }
          }
          fence_proxy_async();
          __syncwarp();
        }
        float s[2][4] = {};
        const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          uint32_t b[4];
          const int key = (mi >> 1) * 8 + r8;
          pd_ldsm4(b, smem_u32(kt) + key * 128 + (((ks * 2 + (mi & 1)) ^ (key & 7)) << 4));
          pd_mma(s[0], qf[ks], b[0], b[1]);
          pd_mma(s[1], qf[ks], b[2], b[3]);
        }
        const int t4 = lane & 3;
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int j = key0 + nt * 8 + t4 * 2;
          if (j >= it.k_end) s[nt][0] = -INFINITY;
          if (j + 1 >= it.k_end) s[nt][1] = -INFINITY;
          mx = fmaxf(mx, fmaxf(s[nt][0], s[nt][1]));
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float mn = fmaxf(m_run, mx * sl2);
        const float corr = (mn == -INFINITY) ? 1.f : pd_ex2(m_run - mn);
        const float basev = (mn == -INFINITY) ? 0.f : mn;
        float ps = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          s[nt][0] = pd_ex2(fmaf(s[nt][0], sl2, -basev));
          s[nt][1] = pd_ex2(fmaf(s[nt][1], sl2, -basev));
          ps += s[nt][0] + s[nt][1];
        }
        l_run = l_run * corr + ps;
        m_run = mn;
#pragma unroll
        for (int d = 0; d < 8; ++d) { o[d][0] *= corr; o[d][1] *= corr; }
        uint32_t a[4];
        a[0] = pd_pack(s[0][0], s[0][1]);
        a[1] = 0u;
        a[2] = pd_pack(s[1][0], s[1][1]);
        a[3] = 0u;
#pragma unroll
        for (int dp = 0; dp < 4; ++dp) {
          uint32_t b[4];
          const int key = (mi & 1) * 8 + r8;
          pd_ldsm4_t(b, smem_u32(vt) + key * 128 + (((dp * 2 + (mi >> 1)) ^ (key & 7)) << 4));
          pd_mma(o[dp * 2], a, b[0], b[1]);
          pd_mma(o[dp * 2 + 1], a, b[2], b[3]);
        }
      }
      ring.release_slot();
    }
    // ---- merge the warps' (m, l, o) of row 0, in warp order
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    float* s_m = red;                // [8]
    float* s_l = red + 8;            // [8]
    float* s_o = red + 16;           // [8][64]
    if (lane < 4) {
      if (lane == 0) { s_m[warp] = m_run; s_l[warp] = l_run; }
#pragma unroll
      for (int d = 0; d < 8; ++d) {
        s_o[warp * 64 + d * 8 + lane * 2] = o[d][0];
        s_o[warp * 64 + d * 8 + lane * 2 + 1] = o[d][1];
      }
    }
    pd_bar_consumers();
    if (threadIdx.x < PD_D && it.t < M) {
      const int d = threadIdx.x;
      float cm = -INFINITY;
#pragma unroll
      for (int w = 0; w < PD_CW; ++w) cm = fmaxf(cm, s_m[w]);
      float cl = 0.f, a = 0.f;
#pragma unroll
      for (int w = 0; w < PD_CW; ++w) {
        const float ws = (s_m[w] == -INFINITY) ? 0.f : pd_ex2(s_m[w] - cm);
        cl += s_l[w] * ws;
        a += s_o[w * 64 + d] * ws;
      }
      if (p.S == 1) {
        p.att[(size_t)it.t * E + it.h * PD_D + d] = __float2bfloat16_rn(cl > 0.f ? a / cl : 0.f);
      } else {
        const size_t pidx = ((size_t)it.t * H + it.h) * p.S + it.s;
        p.att_acc[pidx * PD_D + d] = a;
        if (d == 0) {
          p.att_ml[pidx * 2] = cm;
          p.att_ml[pidx * 2 + 1] = cl;
        }
      }
    }
    pd_bar_consumers();
  }
  return ring.take;
}

// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(PD_THREADS, 1)
decode_persistent_kernel(const __grid_constant__ PdParams p) {
  extern __shared__ uint8_t pd_raw[];
  __shared__ int s_abort;
  PdShared sh;
  sh.base = (uint8_t*)(((uintptr_t)pd_raw + 1023) & ~(uintptr_t)1023);
  sh.full = (uint64_t*)(sh.base + PD_OFF_BAR);
  sh.empty = sh.full + PD_SLOTS;
  sh.abort = &s_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < PD_SLOTS; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], PD_CW);
    }
    fence_barrier_init();
  }
  __syncthreads();
  const int E = p.E, I = p.I, H = p.H, M = p.M, G = gridDim.x;
  const int n_att = M * H * p.S;
  // the slices of a context: equal spans of whole 64-key units that cover the longest context
  int span = (p.plan_head[2] + p.S - 1) / p.S;
  span = max(64, (span + 63) / 64 * 64);
  const PdLayer* layers = p.layers;
  const int rot_out = G / 3, rot_fc = (2 * G) / 3;

  if (warp == PD_CW) {
    // ================================ producer ================================
    PdProducer pr(sh, p);
    PdMarks mark(lane == 0 ? p.timing : nullptr, 0);
    mark(0);
    int phases = 0;
    // asked by all 32 lanes together, so that the warp never splits over the answer
    auto stop = [&]() {
      return __any_sync(0xffffffffu, (p.stop_after > 0 && phases >= p.stop_after) || *sh.abort) != 0;
    };
    for (int l = 0; l < p.n_layers && !stop(); ++l) {
      const PdLayer* L = layers + l;
      if (lane == 0) pr.weight_phase(L->w_qkv, 3 * E / 16, 0, E);
      mark(1);
      ++phases;
      if (stop()) break;
      // cache pages of earlier positions; lane i holds the i-th and (i+32)-th page of the item
      for (int i = pd_att_first(); i < n_att; i += G) {
        if (__shfl_sync(0xffffffffu, (int)*sh.abort, 0)) break;      // the same answer on every lane
        PdAttItem it;
        if (!pd_att_item(p, span, i, it) || it.units == 0) continue;
        const int* trow = p.table + (size_t)it.req * p.max_pages;
        const int first_page = it.k_begin / PD_PS;
        const int n_pages = (it.k_end - it.k_begin + PD_PS - 1) / PD_PS;
        for (int base = 0; base < n_pages; base += 32) {
          int page = 0;
          if (base + lane < n_pages) {
            page = trow[first_page + base + lane];
            if (page < 0 || page >= p.num_pages) {
              atomicOr(p.status, HS_STATUS_BAD_PAGE);
              page = 0;
            }
          }
          const int todo = min(32, n_pages - base);
          for (int u0 = 0; u0 < todo; u0 += PD_KV_PAGES) {
            const int np = min(PD_KV_PAGES, todo - u0);
            uint8_t* dst = nullptr;
            if (lane == 0) dst = pr.open_slot(2 * np);
            const int s = pr.fill % PD_SLOTS;
            for (int q = 0; q < np; ++q) {
              const int pg = __shfl_sync(0xffffffffu, page, u0 + q);
              if (lane == 0 && !*sh.abort) {
                const long long row = L->kv_row0 + (((long long)pg * 2) * H + it.h) * PD_PS;
                tma_load_2d(dst + (2 * q) * PD_BOX_BYTES, &p.tables->kv, &sh.full[s], 0, (int)row);
                tma_load_2d(dst + (2 * q + 1) * PD_BOX_BYTES, &p.tables->kv, &sh.full[s], 0,
                            (int)(row + (long long)H * PD_PS));
              }
            }
            if (lane == 0) ++pr.fill;
            pr.fill = __shfl_sync(0xffffffffu, pr.fill, 0);
          }
        }
      }
      mark(2);
      ++phases;
      if (stop()) break;
      if (lane == 0) pr.weight_phase(L->w_out, E / 16, rot_out, E);
      mark(3);
      ++phases;
      if (stop()) break;
      if (lane == 0) pr.weight_phase(L->w_fc, I / 16, rot_fc, E);
      mark(4);
      ++phases;
      if (stop()) break;
      if (lane == 0) pr.weight_phase(L->w_mlp, E / 16, G - 1 - (E / 16 - 1) % G, I);
      mark(5);
      ++phases;
      __syncwarp();
    }
    const bool stopped = stop();
    if (lane == 0 && !stopped && p.W > 0) pr.weight_phase(p.tables->w_head, (p.V + 15) / 16, 0, E);
    // Leave only when every copy this warp issued has landed: a slot still in flight was
    // either consumed (its full barrier completed) or is waited for here, bounded.
    if (lane == 0 && *sh.abort) {
      for (uint32_t f = pr.fill > PD_SLOTS ? pr.fill - PD_SLOTS : 0; f < pr.fill; ++f)
        mbar_wait(&sh.full[f % PD_SLOTS], (f / PD_SLOTS) & 1, p.status, 1u << 20);
    }
    return;
  }

  // ================================== consumers ==================================
  PdConsumer ring(sh, p);
  PdMarks mark(threadIdx.x == 0 ? p.timing : nullptr, 1);
  mark(0);
  int passed = 0;                                   // grid barriers passed
  auto done = [&]() { return p.stop_after > 0 && passed >= p.stop_after; };
  float* red = (float*)(sh.base + PD_OFF_RED);
  // activation rows kept per chunk: 8 when the step has at most 8 tokens (twice the chunks)
  const int RA = M > 8 ? 16 : 8;
  const int resident_k = (PD_ACHUNKS * PD_ACHUNK) / (RA * PD_AROW) * PD_CK;
  const int rot_mlp = G - 1 - (E / 16 - 1) % G;
  enum { B_QKV = 0, B_OUT = 1, B_FC = 2, B_MLP = 3 };
  // Vectors are staged one phase ahead (cp.async before the grid barrier, awaited after it):
  // the first layer's before anything else.
  pd_stage_norm(sh, layers[0].ln1_g, layers[0].ln1_b, E);
  pd_stage_bias(sh, B_QKV, layers[0].b_qkv, 3 * E / 16, 0);
  pd_cp_commit();
  pd_cp_wait();
  pd_bar_consumers();

  for (int l = 0; l < p.n_layers; ++l) {
    const PdLayer* L = layers + l;
    const bool last = l + 1 == p.n_layers;
    // ---- 1. LayerNorm + QKV projection -----------------------------------------------
    {
      const bool has = pd_first_tile(0) < 3 * E / 16;
      if (has || (l == 0 && (int)blockIdx.x < M))
        pd_layernorm_rows(sh, p, L->eps1, nullptr, M, l == 0, RA, warp, lane);
      pd_bar_consumers();
      mark(10);
      ring.take = pd_linear_resident(sh, p, ring.take, 3 * E, 0, E, L->b_qkv, pd_par_bias(sh, B_QKV), PD_EPI_QKV, 0,
                         M, RA, nullptr, warp, lane);
      mark(11);
    }
    pd_stage_bias(sh, B_OUT, L->b_out, E / 16, rot_out);
    pd_cp_commit();
    pd_grid_sync(sh, p, passed);
    mark(12);
    if (done()) return;
    // ---- 2. attention over the pages, the token's own key and value appended -----------
    ring.take = pd_attention_phase(sh, p, ring.take, L, span, n_att, warp, lane);
    mark(21);
    pd_stage_norm(sh, L->ln2_g, L->ln2_b, E);
    pd_stage_bias(sh, B_FC, L->b_fc, I / 16, rot_fc);
    pd_cp_commit();
    pd_grid_sync(sh, p, passed);
    pd_cp_wait();
    mark(22);
    if (done()) return;
    // ---- 3. attention output projection, added to the stream ---------------------------
    if (pd_first_tile(rot_out) < E / 16) {
      if (p.S == 1) pd_load_rows(sh, p.att, M, E, E, RA);
      else pd_load_merged_attention(sh, p, RA);
    }
    pd_bar_consumers();
    mark(30);
    ring.take = pd_linear_resident(sh, p, ring.take, E, rot_out, E, L->b_out, pd_par_bias(sh, B_OUT),
                       PD_EPI_RESIDUAL, 0, M, RA, nullptr, warp, lane);
    mark(31);
    pd_stage_bias(sh, B_MLP, L->b_mlp, E / 16, rot_mlp);
    pd_cp_commit();
    pd_grid_sync(sh, p, passed);
    pd_cp_wait();
    mark(32);
    if (done()) return;
    // ---- 4. LayerNorm + first MLP matrix + activation ----------------------------------
    if (pd_first_tile(rot_fc) < I / 16)
      pd_layernorm_rows(sh, p, L->eps2, nullptr, M, false, RA, warp, lane);
    pd_bar_consumers();
    mark(40);
    ring.take = pd_linear_resident(sh, p, ring.take, I, rot_fc, E, L->b_fc, pd_par_bias(sh, B_FC), PD_EPI_ACT,
                       L->act, M, RA, nullptr, warp, lane);
    mark(41);
    // the next norm's vectors (the norm of this phase has been applied by every warp)
    if (!last) {
      pd_stage_norm(sh, layers[l + 1].ln1_g, layers[l + 1].ln1_b, E);
      pd_stage_bias(sh, B_QKV, layers[l + 1].b_qkv, 3 * E / 16, 0);
    } else {
      pd_stage_norm(sh, p.lnf_g, p.lnf_b, E);
    }
    pd_cp_commit();
    pd_grid_sync(sh, p, passed);
    pd_cp_wait();
    mark(42);
    if (done()) return;
    // ---- 5. second MLP matrix, added to the stream -------------------------------------
    if (I <= resident_k) {
      if (pd_first_tile(rot_mlp) < E / 16) pd_load_rows(sh, p.u, M, I, I, RA);
      pd_bar_consumers();
      ring.take = pd_linear_resident(sh, p, ring.take, E, rot_mlp, I, L->b_mlp, pd_par_bias(sh, B_MLP),
                         PD_EPI_RESIDUAL, 0, M, RA, nullptr, warp, lane);
    } else {
      ring.take = pd_linear_streamed(sh, p, ring.take, E, rot_mlp, I, L->b_mlp, pd_par_bias(sh, B_MLP), M, warp, lane);
    }
    mark(51);
    pd_grid_sync(sh, p, passed);
    mark(52);
    if (done()) return;
  }
  if (p.W <= 0) return;
  // ---- final LayerNorm of the wanted rows, head, greedy choice -------------------------
  PdBest best;
  if (pd_first_tile(0) < (p.V + 15) / 16)
    pd_layernorm_rows(sh, p, p.eps_f, p.logit_rows, p.W, false, RA, warp, lane);
  pd_bar_consumers();
  ring.take = pd_linear_resident(sh, p, ring.take, p.V, 0, E, nullptr, nullptr, PD_EPI_LOGITS, 0, p.W, RA, &best,
                     warp, lane);
  {
    // the 16 feature lanes of a token -> one candidate per token and CTA (lowest index on ties)
    float* bv = red;
    int* bi = (int*)(red + 256);
    bv[threadIdx.x] = best.val;
    bi[threadIdx.x] = best.idx;
    pd_bar_consumers();
    if (threadIdx.x < PD_MT) {
      const int t = threadIdx.x;
      float v = -INFINITY;
      int ix = 0x7fffffff;
      for (int f = 0; f < 16; ++f) {
        const float cv = bv[t * 16 + f];
        const int ci = bi[t * 16 + f];
        if (cv > v || (cv == v && ci < ix)) { v = cv; ix = ci; }
      }
      p.amax_val[blockIdx.x * PD_MT + t] = v;
      p.amax_idx[blockIdx.x * PD_MT + t] = ix;
    }
  }
  pd_grid_sync(sh, p, passed);
  if (blockIdx.x == 0 && threadIdx.x < PD_MT) {
    const int t = threadIdx.x;
    if (t < p.W) {
      float v = -INFINITY;
      int ix = 0x7fffffff;
      for (int c = 0; c < G; ++c) {
        const float cv = __ldcg(&p.amax_val[c * PD_MT + t]);
        const int ci = __ldcg(&p.amax_idx[c * PD_MT + t]);
        if (cv > v || (cv == v && ci < ix)) { v = cv; ix = ci; }
      }
      if (ix == 0x7fffffff) ix = 0;
      p.tokens_out[t] = ix;
      const int slot = p.samp_slot[t];
      if (slot >= 0 && slot < p.n_feedback) p.feedback[slot] = ix;
    }
    if (t == 0) p.tokens_out[p.Wcap] = *(volatile int*)p.status;
  }
}

// ------------------------------------------------------------------------------------------
typedef CUresult (*PdEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                               const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PdEncodeFn pd_encode() {
  static PdEncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (PdEncodeFn)ptr;
  }
  return fn;
}

// [rows, cols] bfloat16 (cols contiguous), boxes of 16 rows x 64 columns, 128-byte swizzle,
// zeros outside.
static int pd_map(CUtensorMap* map, const void* base, long long rows, long long cols) {
  PdEncodeFn enc = pd_encode();
  if (!enc) return HS_ERR_UNSUPPORTED;
  if (((uintptr_t)base & 15) || cols % 8) return HS_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64u, 16u};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                   strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? HS_OK : HS_ERR_ARGUMENT;
}

}  // namespace hs

// Sizes of the descriptor records the caller allocates (host memory, then copied to the device).
HS_EXPORT int hs_decode_persistent_layer_bytes() { return (int)sizeof(hs::PdLayer); }
HS_EXPORT int hs_decode_persistent_tables_bytes() { return (int)sizeof(hs::PdTables); }
HS_EXPORT int hs_decode_persistent_max_tokens() { return hs::PD_MT; }

// Whether a model of these sizes is served by the kernel at all.
HS_EXPORT int hs_decode_persistent_supports(int E, int I, int H, int head_dim, int n_kv_heads,
                                            int page_size, int window) {
  if (head_dim != hs::PD_D || n_kv_heads != H || H * head_dim != E) return 0;
  if (page_size != hs::PD_PS || window != 0) return 0;
  if (E % 64 || I % 64 || E > hs::PD_ACHUNKS * hs::PD_CK || E < 64 || I < 64) return 0;
  return 1;
}

// Fills one layer record (host memory).  The matrices are the PACKED copies: for a matrix
// [features, k] (k contiguous, features padded with zero rows to a multiple of 16), tile j holds
// rows 16 j .. 16 j + 15 as k / 64 boxes of [16 rows x 64 k] one behind the other, and inside a
// box the 16-byte piece c of row r lies at piece c ^ (r & 7) of that row (the 128-byte XOR
// swizzle ldmatrix reads without bank conflicts).
HS_EXPORT int hs_decode_persistent_layer(void* record, const void* w_qkv, const void* w_out,
                                         const void* w_fc, const void* w_mlp, const float* b_qkv,
                                         const float* b_out, const float* b_fc, const float* b_mlp,
                                         const float* ln1_g, const float* ln1_b, const float* ln2_g,
                                         const float* ln2_b, float eps1, float eps2, float scale,
                                         int act, int E, int I, long long kv_row0) {
  using namespace hs;
  (void)E; (void)I;
  if (!record || !w_qkv || !w_out || !w_fc || !w_mlp || !ln1_g || !ln1_b || !ln2_g || !ln2_b)
    return HS_ERR_ARGUMENT;
  if (((uintptr_t)w_qkv | (uintptr_t)w_out | (uintptr_t)w_fc | (uintptr_t)w_mlp) & 15)
    return HS_ERR_UNSUPPORTED;
  if (!(scale > 0.f)) return HS_ERR_UNSUPPORTED;
  PdLayer L;
  memset(&L, 0, sizeof(L));
  L.w_qkv = (const __nv_bfloat16*)w_qkv; L.w_out = (const __nv_bfloat16*)w_out;
  L.w_fc = (const __nv_bfloat16*)w_fc; L.w_mlp = (const __nv_bfloat16*)w_mlp;
  L.b_qkv = b_qkv; L.b_out = b_out; L.b_fc = b_fc; L.b_mlp = b_mlp;
  L.ln1_g = ln1_g; L.ln1_b = ln1_b; L.ln2_g = ln2_g; L.ln2_b = ln2_b;
  L.scale = scale; L.eps1 = eps1; L.eps2 = eps2; L.act = act; L.kv_row0 = kv_row0;
  memcpy(record, &L, sizeof(L));
  return HS_OK;
}

// Fills the record of the head (packed like the layers' matrices) and of the cache storage
// (host memory).  `pool` is the storage of the whole page group: [entries, pages, 2, heads, 16,
// 64] bfloat16.
HS_EXPORT int hs_decode_persistent_tables(void* record, const void* w_head, int V, int E,
                                          const void* pool, long long pool_rows) {
  using namespace hs;
  (void)V; (void)E;
  if (!record || !w_head || !pool) return HS_ERR_ARGUMENT;
  if ((uintptr_t)w_head & 15) return HS_ERR_UNSUPPORTED;
  if (pool_rows <= 0 || pool_rows > 0x7fffffffLL) return HS_ERR_UNSUPPORTED;
  PdTables T;
  memset(&T, 0, sizeof(T));
  int rc;
  if ((rc = pd_map(&T.kv, pool, pool_rows, PD_D)) != HS_OK) return rc;
  T.w_head = (const __nv_bfloat16*)w_head;
  memcpy(record, &T, sizeof(T));
  return HS_OK;
}

// Floats / ints of scratch a launch needs besides the step's buffers: the slices' partial
// attention results, and one greedy candidate per CTA and token.
HS_EXPORT int hs_decode_persistent_grid() {
  static int grid = 0;
  if (grid) return grid;
  if (cudaFuncSetAttribute(hs::decode_persistent_kernel,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, hs::PD_SMEM) != cudaSuccess)
    return 0;
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, hs::decode_persistent_kernel,
                                                    hs::PD_THREADS, hs::PD_SMEM) != cudaSuccess)
    return 0;
  if (per_sm < 1) return 0;
  grid = hs_sm_count();                 // one CTA per SM; all of them are resident at once
  return grid;
}

// The slices of a token's context for a batch of M tokens: so many that tokens x heads x
// slices fills the GPU once, at most 8.  (The span of a slice follows the longest context of
// the step, on the device; a slice past a token's context is empty.)
HS_EXPORT int hs_decode_persistent_slices(int M, int H) {
  const int grid = hs_decode_persistent_grid();
  if (grid <= 0 || M <= 0 || H <= 0) return 1;
  int s = grid / (M * H);
  if (s > 8) s = 8;
  return s < 1 ? 1 : s;
}

HS_EXPORT int hs_decode_persistent(
    const void* layers_dev, const void* tables_dev, int n_layers, const void* wte, const void* wpe,
    const float* lnf_g, const float* lnf_b, float eps_f, int E, int I, int V, int H, int n_pos,
    void* pool, int num_pages, int max_pages, float* x, void* qkv, void* att, void* u,
    float* logits, float* att_acc, float* att_ml, float* amax_val, int* amax_idx, int* tokens_out,
    int* feedback, int n_feedback, const int* tok_ids, const int* tok_pos, const int* tok_req,
    const int* table, const int* logit_rows, const int* samp_slot, const int* plan_head, int M,
    int W, int Wcap, int slices, unsigned* sync, int* status, int stop_after, void* stream) {
  using namespace hs;
  if (!layers_dev || !tables_dev || !wte || !wpe || !lnf_g || !lnf_b || !pool || !x || !qkv ||
      !att || !u || !tokens_out || !feedback || !tok_ids || !tok_pos || !tok_req || !table ||
      !sync || !status || !amax_val || !amax_idx || !plan_head)
    return HS_ERR_ARGUMENT;
  if (M <= 0 || M > PD_MT || W < 0 || W > PD_MT || Wcap < W || n_layers <= 0)
    return HS_ERR_UNSUPPORTED;
  if (W > 0 && (!logits || !logit_rows || !samp_slot)) return HS_ERR_ARGUMENT;
  if (!hs_decode_persistent_supports(E, I, H, E / (H > 0 ? H : 1), H, PD_PS, 0))
    return HS_ERR_UNSUPPORTED;
  if (slices < 1 || slices > 8 || (slices > 1 && (!att_acc || !att_ml))) return HS_ERR_ARGUMENT;
  const int grid = hs_decode_persistent_grid();
  if (grid <= 0) return HS_ERR_UNSUPPORTED;
  PdParams p;
  memset(&p, 0, sizeof(p));
  p.layers = (const PdLayer*)layers_dev;
  p.tables = (const PdTables*)tables_dev;
  p.wte = (const __nv_bfloat16*)wte; p.wpe = (const __nv_bfloat16*)wpe;
  p.lnf_g = lnf_g; p.lnf_b = lnf_b; p.eps_f = eps_f;
  p.n_layers = n_layers; p.E = E; p.I = I; p.V = V; p.H = H; p.n_pos = n_pos;
  p.pool = (__nv_bfloat16*)pool; p.num_pages = num_pages; p.max_pages = max_pages;
  p.x = x; p.qkv = (__nv_bfloat16*)qkv; p.att = (__nv_bfloat16*)att; p.u = (__nv_bfloat16*)u;
  p.logits = logits; p.att_acc = att_acc; p.att_ml = att_ml; p.amax_val = amax_val;
  p.amax_idx = amax_idx; p.tokens_out = tokens_out; p.feedback = feedback;
  p.n_feedback = n_feedback;
  p.tok_ids = tok_ids; p.tok_pos = tok_pos; p.tok_req = tok_req; p.table = table;
  p.logit_rows = logit_rows; p.samp_slot = samp_slot; p.plan_head = plan_head;
  p.M = M; p.W = W; p.Wcap = Wcap; p.S = slices;
  p.sync = sync; p.status = status; p.stop_after = stop_after;
  p.timing = hs_timing_buffer();
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(sync, 0, 2 * sizeof(unsigned), st);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(PD_THREADS);
  cfg.dynamicSmemBytes = PD_SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;     // all CTAs resident: the grid barrier is safe
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, decode_persistent_kernel, p);
  if (e != cudaSuccess) return (int)e;
  HS_LAUNCH_CHECK();
  return HS_OK;
}
