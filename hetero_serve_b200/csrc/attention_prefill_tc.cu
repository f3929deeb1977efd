// Causal attention of prompt portions over the paged cache on tcgen05 tensor cores (sm_100a),
// bfloat16, head size 64.
//
// What the reference does with WMMA fragments (heteroserve/model/paged_attn_wmma.py:80-254:
// FlashAttention tiling over 16-token pages, online softmax, query s of a portion at absolute
// position ctx_len - S + s, heteroserve/model/paged_attn_prefill.py:93-104) is laid out here for
// Blackwell: S = Q K^T and O_tile = P V are tcgen05.mma instructions with their accumulators in
// tensor memory, the operands are staged by TMA, and the softmax runs with ONE THREAD PER QUERY
// ROW (a TMEM lane is a row), so row maxima and sums need no shuffles.
//
// A work item is up to 128 consecutive queries of one request x one head.  CTAs are persistent;
// the host lists the items with the most keys first and CTA b walks b, 2G-1-b, 2G+b, ... (a snake
// over the sorted list, G CTAs), so every role knows its sequence and runs ahead on its own.
//   warp 0      TMA producer, all 32 lanes: the Q tile [128 x 64] once per item (two buffers, so
//               the next item's queries are fetched while this item's MMAs still run); per
//               128-key tile, one [16 x 64] box of K and of V per 16-position block, found
//               through the block table (a page holds whole blocks), into a four-stage ring:
//               lanes 0..7 look the eight blocks up and copy the keys, lanes 8..15 the values,
//               lane 0 waits for the ring slot and announces the bytes (with one lane doing
//               all of it the producer barely kept ahead: the softmax threads waited 30 % of
//               their time for S, now 18 %);
//   warp 1      one thread issues  S[b] = Q K^T  (M=128, N=128, 4 k-steps) into one of two TMEM
//               buffers, and  O_tile = P V  (M=128, N=64, 8 k-steps, V as the N-contiguous
//               operand) once the softmax warps have written P;
//   warps 2..9  softmax, two threads per query row (one per 64-key half; the halves exchange
//               their maxima through shared memory): tcgen05.ld of the row, maximum, exponentials,
//               scores * scale folded into the exponent (2^(s*scale*log2e - m)), causal mask by
//               position, P written to shared memory as bfloat16 in the swizzled operand layout,
//               O_tile added into the row's float32 accumulator in registers with the usual
//               rescale.  S(t+1) is computed while the softmax of tile t runs.
// Rows of K/V past the item's last position are never loaded; their (stale) rows of V are
// zeroed in shared memory before P V so that 0 * garbage cannot make a NaN.
//
// Every mbarrier wait is bounded (tcgen05.cuh); on a time-out the status word is set and the
// CTA leaves its loops, frees its TMEM and returns.
#include "tcgen05.cuh"

namespace hs {

constexpr int TA_BQ = 128, TA_BKV = 128, TA_D = 64;
constexpr int TA_THREADS = 320;          // warp 0 TMA, warp 1 MMA, warps 2..9 softmax
constexpr int TA_SOFTMAX_WARPS = 8;
constexpr int TA_KV_STAGES = 4;
constexpr int TA_Q_BYTES = TA_BQ * TA_D * 2;             // 16 KB
constexpr int TA_KV_BYTES = TA_BKV * TA_D * 2;           // 16 KB per K or V tile
constexpr int TA_P_BYTES = TA_BQ * TA_BKV * 2;           // 32 KB: two 64-key k-blocks
// padded beyond half of an SM's shared memory: two of these CTAs must never share an SM, since
// each allocates all 512 TMEM columns
constexpr int TA_SMEM = 2 * TA_Q_BYTES + 2 * TA_KV_STAGES * TA_KV_BYTES + TA_P_BYTES + 256 + 1024 + 4096;

struct PrefillTcParams {
  __nv_bfloat16* out;
  const int* table;
  const int* tile_info;
  const int* plan_head;
  int* status;
  int* work_counter;
  int n_heads, n_kv_heads, page_size, num_pages, max_pages, q_off, ps_log2;
  float scale;
  unsigned long long* timing;   // tuning builds (-DHS_PHASE_MARKS) only: null, or 8 x uint64 per
                                // CTA, cycles of one softmax thread per phase (0 wait for S,
                                // 1 maximum, 2 exponentials, 3 wait for P V and add O, 4 write P,
                                // 5 loop, 6 last O, 7 wait for an item's first S)
};

// barriers, in this order in shared memory
enum { B_Q_FULL = 0, B_KV_FULL = 2, B_KV_EMPTY = 2 + TA_KV_STAGES, B_S_FULL = 2 + 2 * TA_KV_STAGES,
       B_S_EMPTY = B_S_FULL + 2, B_P_FULL = B_S_EMPTY + 2, B_P_EMPTY = B_P_FULL + 1,
       B_O_FULL = B_P_EMPTY + 1, B_O_EMPTY = B_O_FULL + 1, B_Q_EMPTY = B_O_EMPTY + 1,
       B_COUNT = B_Q_EMPTY + 2 };

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(TA_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                            const __grid_constant__ CUtensorMap map_kv,
                            const PrefillTcParams p) {
  pdl_trigger();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                                     // [2 items][128 queries][128 B]
  uint8_t* sK = sQ + 2 * TA_Q_BYTES;                      // [stages][128 keys][128 B]
  uint8_t* sV = sK + TA_KV_STAGES * TA_KV_BYTES;
  uint8_t* sP = sV + TA_KV_STAGES * TA_KV_BYTES;          // [2 k-blocks][128 rows][128 B]
  uint64_t* bars = (uint64_t*)(sP + TA_P_BYTES);
  uint32_t* tmem_slot = (uint32_t*)(bars + B_COUNT);
  __shared__ float s_max2[2][2][TA_BQ];  // [tile parity][half][row]: row maxima of the halves
  __shared__ float s_l[2][TA_BQ];        // [half][row]: the halves' shares of the row sum

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_items = p.plan_head[1] * p.n_heads;
  const int PS = p.page_size;
  constexpr uint32_t S_COLS = TA_BKV;                     // 128 columns per S buffer
  constexpr uint32_t O_COL = 2 * S_COLS;                  // O_tile after the two S buffers
  constexpr uint32_t TMEM_COLS = 512;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[B_Q_FULL + i], 1);
      mbar_init(&bars[B_Q_EMPTY + i], 1);
    }
    for (int i = 0; i < TA_KV_STAGES; ++i) {
      mbar_init(&bars[B_KV_FULL + i], 1);
      mbar_init(&bars[B_KV_EMPTY + i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[B_S_FULL + i], 1);
      mbar_init(&bars[B_S_EMPTY + i], TA_SOFTMAX_WARPS);
    }
    mbar_init(&bars[B_P_FULL], TA_SOFTMAX_WARPS);
    mbar_init(&bars[B_P_EMPTY], 1);
    mbar_init(&bars[B_O_FULL], 1);
    mbar_init(&bars[B_O_EMPTY], TA_SOFTMAX_WARPS);
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
  pdl_wait();          // queries and this step's keys and values come from earlier kernels

  // running counts of completed phases, kept identically by every role
  uint32_t n_item = 0;        // items processed by this CTA
  uint32_t n_tile = 0;        // key tiles processed by this CTA (over all items)
  bool ok = true;

  // Items are listed heaviest first; CTA b takes b, 2G-1-b, 2G+b, 4G-1-b, ... (G CTAs): a
  // snake over the sorted list, so heavy and light items alternate per CTA.  Every role walks
  // the same sequence on its own: no CTA-wide synchronisation between items.
  const int G = gridDim.x;
  for (int round = 0; ok; ++round) {
    const int item = round * G + ((round & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x);
    if (round * G >= n_items) break;
    if (item >= n_items) continue;
    const int tile = item / p.n_heads, h = item - tile * p.n_heads;
    const int4 ti = *(const int4*)(p.tile_info + 4 * tile);
    const int tok0 = ti.x, nq = ti.y, r = ti.z, pos0 = ti.w;
    if (r < 0 || nq <= 0 || pos0 < 0) continue;
    const int pos_last = pos0 + nq - 1;
    if (pos_last / PS >= p.max_pages) {
      if (threadIdx.x == 0) atomicOr(p.status, HS_STATUS_BAD_POSITION);
      continue;
    }
    const int hk = h / (p.n_heads / p.n_kv_heads);
    const int n_kv = pos_last / TA_BKV + 1;               // key tiles of this item
    const int* trow = p.table + (size_t)r * p.max_pages;

    if (warp == 0) {
      // ---------------- TMA producer: the whole warp.  Lane 0 waits and announces the bytes;
      // lanes 0..7 look up the pages of the tile's eight 16-position blocks and copy their keys,
      // lanes 8..15 the values, so that a tile costs one table round trip and one issue slot
      // per lane.  Q has two buffers: the next item's queries never wait for this item's MMAs.
      const int qb = n_item & 1;
      if (lane == 0) {
        if (n_item >= 2)
          ok = mbar_wait(&bars[B_Q_EMPTY + qb], ((n_item >> 1) - 1) & 1, p.status);
        if (ok) {
          mbar_expect_tx(&bars[B_Q_FULL + qb], TA_Q_BYTES);
          tma_load_2d(sQ + qb * TA_Q_BYTES, &map_q, &bars[B_Q_FULL + qb], p.q_off + h * TA_D,
                      tok0);
        }
      }
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      const int v_rows = p.n_kv_heads * PS;                // from a page's keys to its values
      for (int kt = 0; kt < n_kv && ok; ++kt) {
        const uint32_t it = n_tile + kt;
        const int st = it % TA_KV_STAGES;
        // blocks of 16 positions up to the item's last one; the lookup needs only the table,
        // so it comes before the wait for the ring slot
        const int first = kt * TA_BKV;
        const int n_blocks = min(TA_BKV / 16, (pos_last - first) / 16 + 1);
        const int b = lane & 7;
        int src_row = -1;          // row of the block's first position in the [rows, 64] view
        if (lane < 16 && b < n_blocks) {
          const int j = first + b * 16;
          const int pg = p.ps_log2 >= 0 ? (j >> p.ps_log2) : (j / PS);
          const int page = trow[pg];
          if (page < 0 || page >= p.num_pages) {
            if (lane < 8) atomicOr(p.status, HS_STATUS_BAD_PAGE);
          } else {
            src_row = ((page * 2) * p.n_kv_heads + hk) * PS + (j - pg * PS) +
                      (lane >= 8 ? v_rows : 0);
          }
        }
        const unsigned good = __ballot_sync(0xffffffffu, src_row >= 0) & 0xffu;   // key blocks
        if (lane == 0) {
          if (it >= TA_KV_STAGES)
            ok = mbar_wait(&bars[B_KV_EMPTY + st], ((it / TA_KV_STAGES) - 1) & 1, p.status);
          if (ok) mbar_expect_tx(&bars[B_KV_FULL + st], __popc(good) * 2 * 16 * TA_D * 2);
        }
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) break;
        if (src_row >= 0)
          tma_load_2d((lane >= 8 ? sV : sK) + st * TA_KV_BYTES + b * 2048, &map_kv,
                      &bars[B_KV_FULL + st], 0, src_row);
      }
    } else if (warp == 1) {
      if (lane == 0) {
        // ---------------- MMA issuer
        constexpr uint32_t idesc_s = make_idesc(TA_BQ, TA_BKV, false);
        constexpr uint32_t idesc_o = make_idesc(TA_BQ, TA_D, true);
        const int qb = n_item & 1;
        const uint32_t q_addr = smem_u32(sQ + qb * TA_Q_BYTES);
        ok = mbar_wait(&bars[B_Q_FULL + qb], (n_item >> 1) & 1, p.status);
        auto issue_s = [&](int kt) -> bool {
          const uint32_t it = n_tile + kt;
          const int st = it % TA_KV_STAGES, sb = it & 1;
          if (!mbar_wait(&bars[B_KV_FULL + st], (it / TA_KV_STAGES) & 1, p.status)) return false;
          if (it >= 2 && !mbar_wait(&bars[B_S_EMPTY + sb], ((it >> 1) - 1) & 1, p.status))
            return false;
          tc_fence_after();
          const uint64_t qd = make_smem_desc(q_addr);
          const uint64_t kd = make_smem_desc(smem_u32(sK + st * TA_KV_BYTES));
#pragma unroll
          for (int k = 0; k < TA_D / 16; ++k)
            umma_bf16(tmem_base + sb * S_COLS, qd + (uint64_t)(k * 2), kd + (uint64_t)(k * 2),
                      idesc_s, k > 0 ? 1u : 0u);
          umma_commit(&bars[B_S_FULL + sb]);
          // the item's last S: once it has completed, Q may be replaced by the next item's
          if (kt == n_kv - 1) umma_commit(&bars[B_Q_EMPTY + qb]);
          return true;
        };
        if (ok) ok = issue_s(0);
        for (int kt = 0; kt < n_kv && ok; ++kt) {
          const uint32_t it = n_tile + kt;
          const int st = it % TA_KV_STAGES;
          if (kt + 1 < n_kv) ok = issue_s(kt + 1);      // overlaps the softmax of tile kt
          if (!ok) break;
          ok = mbar_wait(&bars[B_P_FULL], it & 1, p.status);
          if (ok && it >= 1) ok = mbar_wait(&bars[B_O_EMPTY], (it - 1) & 1, p.status);
          if (!ok) break;
          tc_fence_after();
          const uint32_t p_addr = smem_u32(sP);
          const uint32_t v_addr = smem_u32(sV + st * TA_KV_BYTES);
#pragma unroll
          for (int k = 0; k < TA_BKV / 16; ++k) {
            // P: k-block (k / 4) of 64 keys, 32 bytes per k-step inside its 128-byte rows;
            // V: 16 keys = 16 rows of 128 bytes further
            const uint64_t pd = make_smem_desc(p_addr + (k >> 2) * 16384) + (uint64_t)((k & 3) * 2);
            const uint64_t vd = make_smem_desc(v_addr + k * 2048);
            umma_bf16(tmem_base + O_COL, pd, vd, idesc_o, k > 0 ? 1u : 0u);
          }
          umma_commit(&bars[B_O_FULL]);
          umma_commit(&bars[B_P_EMPTY]);
          umma_commit(&bars[B_KV_EMPTY + st]);
        }
      }
    } else {
      // ---------------- softmax and output: two threads per query row, one per half of the
      // tile's 128 keys (and per half of the 64 output columns)
      const int q = warp & 3;                               // TMEM lane quarter of this warp
      const int half = (warp - 2) >> 2;                     // 0: keys 0..63, 1: keys 64..127
      const int row = q * 32 + lane;
      const int pos_r = min(pos0 + row, pos_last);          // rows past nq: finite, never stored
      const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
      const float sl2 = p.scale * 1.4426950408889634f;
      float m = -INFINITY, l = 0.f, corr_pending = 1.f;
#ifdef HS_PHASE_MARKS
      long long t_mark = clock64();
      auto lap = [&](int phase) {
        if (p.timing != nullptr && threadIdx.x == 64) {
          const long long now = clock64();
          p.timing[(size_t)blockIdx.x * 8 + phase] += (unsigned long long)(now - t_mark);
          t_mark = now;
        }
      };
#else
      auto lap = [](int) {};
#endif
      constexpr int OC = TA_D / 2;                          // output columns of this thread
      float o[OC];
#pragma unroll
      for (int d = 0; d < OC; ++d) o[d] = 0.f;

      auto accumulate_o = [&](uint32_t it) -> bool {
        if (!mbar_wait(&bars[B_O_FULL], it & 1, p.status)) return false;
        tc_fence_after();
        uint32_t v[32];
        tmem_ld32(lane_addr + O_COL + half * OC, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < OC; ++j) o[j] = fmaf(o[j], corr_pending, __uint_as_float(v[j]));
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[B_O_EMPTY]);
        return true;
      };

      for (int kt = 0; kt < n_kv && ok; ++kt) {
        const uint32_t it = n_tile + kt;
        const int sb = it & 1, st = it % TA_KV_STAGES;
        lap(5);
        ok = mbar_wait(&bars[B_S_FULL + sb], (it >> 1) & 1, p.status);
        if (!ok) break;
        tc_fence_after();
        lap(kt == 0 ? 7 : 0);
        const int j0 = kt * TA_BKV + half * 64;             // first key of this thread's half
        const bool diagonal = kt * TA_BKV + TA_BKV - 1 > pos0;   // some row needs the mask
        const uint32_t s_addr = lane_addr + sb * S_COLS + half * 64;
        // pass 1: the maximum over this half of the row (raw score units; the scale is positive);
        // the second chunk's TMEM load is in flight while the first is reduced
        uint32_t va[32], vb[32];
        tmem_ld32(s_addr, va);
        tmem_ld_wait();
        tmem_ld32(s_addr + 32, vb);
        float mx = -INFINITY;
        if (diagonal) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j0 + j <= pos_r) mx = fmaxf(mx, __uint_as_float(va[j]));
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j0 + 32 + j <= pos_r) mx = fmaxf(mx, __uint_as_float(vb[j]));
        } else {
          float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            m0 = fmaxf(m0, __uint_as_float(va[j]));
            m1 = fmaxf(m1, __uint_as_float(va[j + 1]));
            m2 = fmaxf(m2, __uint_as_float(va[j + 2]));
            m3 = fmaxf(m3, __uint_as_float(va[j + 3]));
          }
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            m0 = fmaxf(m0, __uint_as_float(vb[j]));
            m1 = fmaxf(m1, __uint_as_float(vb[j + 1]));
            m2 = fmaxf(m2, __uint_as_float(vb[j + 2]));
            m3 = fmaxf(m3, __uint_as_float(vb[j + 3]));
          }
          mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        }
        // the other half's maximum, through shared memory (buffers alternate by tile parity)
        s_max2[it & 1][half][row] = mx;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory");   // the two warps of this quarter
        mx = fmaxf(mx, s_max2[it & 1][half ^ 1][row]);
        lap(1);
        const float m_new = fmaxf(m, mx * sl2);
        const float corr = (m_new == -INFINITY) ? 1.f : ex2_fast(m - m_new);
        const float base = (m_new == -INFINITY) ? 0.f : m_new;
        // pass 2: exponentials of this half, packed to bfloat16 (32 registers)
        uint32_t pk[32];
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float e0 = ex2_fast(fmaf(__uint_as_float(va[j]), sl2, -base));
          float e1 = ex2_fast(fmaf(__uint_as_float(va[j + 1]), sl2, -base));
          if (diagonal) {
            if (j0 + j > pos_r) e0 = 0.f;
            if (j0 + j + 1 > pos_r) e1 = 0.f;
          }
          sum += e0 + e1;
          __nv_bfloat162 bq = __floats2bfloat162_rn(e0, e1);
          pk[j >> 1] = *(uint32_t*)&bq;
        }
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float e0 = ex2_fast(fmaf(__uint_as_float(vb[j]), sl2, -base));
          float e1 = ex2_fast(fmaf(__uint_as_float(vb[j + 1]), sl2, -base));
          if (diagonal) {
            if (j0 + 32 + j > pos_r) e0 = 0.f;
            if (j0 + 32 + j + 1 > pos_r) e1 = 0.f;
          }
          sum += e0 + e1;
          __nv_bfloat162 bq = __floats2bfloat162_rn(e0, e1);
          pk[16 + (j >> 1)] = *(uint32_t*)&bq;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[B_S_EMPTY + sb]);   // S[sb] may be overwritten
        l = l * corr + sum;                                  // this half's share of the row sum
        m = m_new;
        lap(2);
        // the previous tile's P V has finished (P is free) and its O_tile is ready
        if (it >= 1) {
          ok = mbar_wait(&bars[B_P_EMPTY], (it - 1) & 1, p.status);
          if (!ok) break;
          if (kt >= 1) {
            ok = accumulate_o(it - 1);
            if (!ok) break;
          }
        }
        corr_pending = corr;
        lap(3);
        // write this half-row of P: k-block `half`, 8 chunks of 8 keys; chunk c at
        //   half * 16 KB + (row / 8) * 1 KB + (row % 8) * 128 B + ((c ^ (row % 8)) * 16 B)
        uint8_t* prow = sP + half * 16384 + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint4 u = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
          *(uint4*)(prow + ((c ^ (row & 7)) << 4)) = u;
        }
        // rows of V past the item's last position were not loaded: zero them (the row index
        // doubles as a key index of the tile; each half clears half of the 128-byte row)
        if (kt * TA_BKV + row > pos_last) {
          uint4* vrow = (uint4*)(sV + st * TA_KV_BYTES + row * 128) + half * 4;
#pragma unroll
          for (int c = 0; c < 4; ++c) vrow[c] = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars[B_P_FULL]);
        lap(4);
      }
      if (ok) ok = accumulate_o(n_tile + n_kv - 1);
      lap(6);
      // the row sum is the two halves' shares together (the next write of s_l comes after
      // at least one more barrier of these warps, so one barrier is enough)
      s_l[half][row] = l;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory");
      const float l_all = l + s_l[half ^ 1][row];
      if (ok && row < nq) {
        const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
        __nv_bfloat16* orow = p.out + ((size_t)(tok0 + row) * p.n_heads + h) * TA_D + half * OC;
#pragma unroll
        for (int c = 0; c < OC; c += 8) {
          __nv_bfloat162 a0 = __floats2bfloat162_rn(o[c] * inv, o[c + 1] * inv);
          __nv_bfloat162 a1 = __floats2bfloat162_rn(o[c + 2] * inv, o[c + 3] * inv);
          __nv_bfloat162 a2 = __floats2bfloat162_rn(o[c + 4] * inv, o[c + 5] * inv);
          __nv_bfloat162 a3 = __floats2bfloat162_rn(o[c + 6] * inv, o[c + 7] * inv);
          uint4 u;
          u.x = *(uint32_t*)&a0; u.y = *(uint32_t*)&a1; u.z = *(uint32_t*)&a2; u.w = *(uint32_t*)&a3;
          *(uint4*)(orow + c) = u;
        }
      }
    }
    n_item += 1;
    n_tile += n_kv;
    // a role that gave up tells the others through the status word; they time out in turn
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

typedef CUresult (*EncodeTiledFnA)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFnA get_encode_a() {
  static EncodeTiledFnA fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFnA)ptr;
  }
  return fn;
}

// [rows, cols] bfloat16, row stride `stride_elems`, boxes of [box_rows x 64], 128-byte swizzle.
static int make_map_2d(CUtensorMap* map, const void* base, long long rows, int cols,
                       long long stride_elems, int box_rows) {
  EncodeTiledFnA enc = get_encode_a();
  if (!enc) return HS_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)stride_elems * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                   strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? HS_OK : HS_ERR_ARGUMENT;
}

}  // namespace hs

// Takes head size 64, bfloat16, no window, positive scale, 16-byte aligned buffers; anything else
// is refused with HS_ERR_UNSUPPORTED and the caller uses another kernel.  `n_tokens` is the
// number of rows of `qkv`; tiles bring up to 128 queries each.
HS_EXPORT int hs_attention_prefill_tc(void* out, const void* qkv, const void* pool,
                                      const int* table, const int* tile_info,
                                      const int* plan_head, int tile_cap, int* work_counter,
                                      int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                      int page_size, int num_pages, int max_pages, int q_off,
                                      int qkv_stride, float scale, int* status, void* stream) {
  using namespace hs;
  (void)work_counter;      // items are assigned statically here; the argument is kept for symmetry
  if (!out || !qkv || !pool || !table || !tile_info || !plan_head || !status)
    return HS_ERR_ARGUMENT;
  if (tile_cap <= 0) return HS_OK;
  if (head_dim != TA_D) return HS_ERR_UNSUPPORTED;
  if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads) return HS_ERR_UNSUPPORTED;
  if (page_size <= 0 || page_size % 16) return HS_ERR_UNSUPPORTED;
  if ((qkv_stride % 8) || (q_off % 8) || ((uintptr_t)qkv & 15) || ((uintptr_t)pool & 15) ||
      ((uintptr_t)out & 15))
    return HS_ERR_UNSUPPORTED;
  if (!(scale > 0.f)) return HS_ERR_UNSUPPORTED;
  const long long pool_rows = (long long)num_pages * 2 * n_kv_heads * page_size;
  if (pool_rows >= (1ll << 31)) return HS_ERR_UNSUPPORTED;
  CUtensorMap mq, mkv;
  if (int e = make_map_2d(&mq, qkv, n_tokens, qkv_stride, qkv_stride, TA_BQ)) return e;
  if (int e = make_map_2d(&mkv, pool, pool_rows, TA_D, TA_D, 16)) return e;
  PrefillTcParams p;
  p.out = (__nv_bfloat16*)out; p.table = table; p.tile_info = tile_info; p.plan_head = plan_head;
  p.status = status; p.work_counter = work_counter;
  p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.page_size = page_size;
  p.num_pages = num_pages; p.max_pages = max_pages; p.q_off = q_off;
  p.ps_log2 = (page_size & (page_size - 1)) == 0 ? __builtin_ctz(page_size) : -1;
  p.scale = scale;
  p.timing = hs_timing_buffer();
  static bool ready[64] = {};            // per device: the shared-memory attribute is set
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return HS_ERR_UNSUPPORTED;
  if (!ready[dev]) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, TA_SMEM);
    if (e != cudaSuccess) return (int)e;
    ready[dev] = true;
  }
  const int sms = hs_sm_count();
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t le = hs_launch(attention_prefill_tc_kernel, dim3(sms), dim3(TA_THREADS),
                             (size_t)TA_SMEM, st, hs_pdl_enabled(), mq, mkv, p);
  if (le != cudaSuccess) return (int)le;
  HS_LAUNCH_CHECK();
  return HS_OK;
}
