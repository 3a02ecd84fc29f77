// Full (and general banded) varlen attention on the sm_100a tensor cores, built so that
// TWO CTAs share each SM.
//
// The softmax of a 128 x 128 score tile costs 16384 exp2 on a unit that retires 16 per clock
// per SM: 1024 clocks in which the other pipes idle, followed by a stretch (tensor-memory
// loads, row maxima, barrier round trips, the P V product) in which the exp2 unit idles.
// Warps that work on the same tile move through those phases together, so one CTA per SM can
// never overlap them.  Two independent CTAs per SM - each a complete pipeline over its own
// work items - drift out of phase and fill each other's gaps.  To fit twice, a CTA is cut to
// 192 threads (168 registers), 113 KB of shared memory and 256 tensor-memory columns:
//   warps 0..3 : softmax - thread t owns query row t: one tcgen05.ld pass brings its 128
//                scores into registers (S is released at once, so the next Q K^T overlaps the
//                exp2 work), exp2 against an inherited reference exponent, row sum - and no row
//                maximum: the sum says when the reference has to move; P goes back to TENSOR
//                MEMORY as bf16 pairs (tcgen05.st), never through shared memory
//   warp 4     : TMA producer - Q (single buffer), K and V in separate three-deep rings (K is
//                free as soon as Q K^T retires, so it runs ahead of V)
//   warp 5     : tensor-memory owner and MMA issuer - S = Q K^T (both operands from shared
//                memory) into one 128-column buffer; O += P V with P read from tensor memory
//                (the A operand of tcgen05.mma may live there) and V from shared memory,
//                ACCUMULATED in 64 columns over the whole item
// Shared memory then carries only Q, K and V: with P there as well, its 128 bytes per clock
// (operand reads of both products, P written and read back, the TMA fills) were as loaded as
// the exp2 unit.
// The output accumulator is rescaled in tensor memory only when a tile's row sum has reached
// 2^16 against the reference it was exponentiated to (P is bf16 and the sums fp32: both keep
// their relative precision at any scale, and 2^60 is far from overflow); after the first tile
// or two of an item that almost never happens, so the per-tile loop has no accumulator traffic
// at all.  A row sum that shows overflow or underflow sends the warp through an exact by-hand
// path for that tile (g_tile_by_hand).
//
// Rows of a K/V tile outside the sequence (or the band) are whatever TMA fetched and are
// masked to -inf before the softmax, so P is exactly 0 there.  Query rows past the end of a
// sequence are computed on whatever was fetched and never stored.  Every mbarrier wait is
// bounded and reports through the status word.
#include "pe_host.h"
#include "pe_ptx.cuh"
#include "attn_tmem.cuh"

namespace pe {

constexpr int G_BM = 128;
constexpr int G_BN = 128;
constexpr int G_THREADS = 192;
constexpr int G_TILE_BYTES = 128 * 64 * 2;  // one 128 x 64 bf16 tile (Q, K, V, half of P)
constexpr int G_PREFETCH_ITEMS = 3;         // how many items ahead the producer warms L2
constexpr int G_STAGES = 3;                 // depth of the K ring and of the V ring
// Q, K[3], V[3] = 7 tiles, then the barriers.  No alignment slack: the kernel checks that
// the dynamic shared memory starts on a 1024-byte boundary.
constexpr int G_SMEM = (1 + 2 * G_STAGES) * G_TILE_BYTES + 256;
constexpr uint32_t G_TMEM_COLS = 256;
constexpr uint32_t G_S_COL = 0;    // S: columns 0..127
constexpr uint32_t G_O_COL = 128;  // O: columns 128..191
constexpr uint32_t G_P_COL = 192;  // P: bf16 pairs, keys 2c and 2c + 1 in column 192 + c
// How many 16-key groups of P a softmax thread holds in registers before it needs the P buffer.
constexpr int G_HOLD = 4;
constexpr int G_RESCALE_LOG2_SUM = 16;   // a tile's row sum of 2^16 or more moves the reference
constexpr float G_SUM_MAX = 1.152921504606846976e18f;   // 2^60: above it (or not finite) the tile is redone
constexpr float G_SUM_MIN = 8.673617379884035e-19f;     // 2^-60: an item's first tile below it is redone

enum {
  GB_Q_FULL = 0,
  GB_Q_EMPTY = 1,
  GB_K_FULL = 2,    // G_STAGES
  GB_K_EMPTY = 5,   // G_STAGES
  GB_V_FULL = 8,    // G_STAGES
  GB_V_EMPTY = 11,  // G_STAGES
  GB_S_FULL = 14,
  GB_S_EMPTY = 15,
  GB_P_FULL = 16,
  GB_O_FULL = 17,
  GB_COUNT = 18
};

struct GItem {
  int seq_begin, len, q0, head;
  int kv_start, n_kv;
};

__device__ __forceinline__ GItem g_make_item(const int4 info, int item, int nh, int half_window) {
  GItem it;
  it.seq_begin = info.x;
  it.len = info.y;
  it.q0 = info.z;
  it.head = item % nh;
  // key tile j covers keys [kv_start + 128 j, kv_start + 128 j + 128) of the sequence
  it.kv_start = 0;
  it.n_kv = (it.len + G_BN - 1) / G_BN;
  if (half_window >= 0) {
    it.kv_start = it.q0 - half_window;  // may be negative: those keys are masked
    const int kv_end = min(it.len, it.q0 + G_BM + half_window);
    it.n_kv = (kv_end - it.kv_start + G_BN - 1) / G_BN;
  }
  return it;
}

// A cursor over the flat sequence of key tiles of this CTA's items.
struct GCursor {
  int item, j;
  GItem it;
  __device__ __forceinline__ void open(const int4* tile_info, int first, int total, int nh, int hw) {
    item = first;
    j = 0;
    if (item < total) it = g_make_item(__ldg(tile_info + item / nh), item, nh, hw);
  }
  __device__ __forceinline__ void advance(const int4* tile_info, int stride, int total, int nh, int hw) {
    if (++j == it.n_kv) {
      j = 0;
      item += stride;
      if (item < total) it = g_make_item(__ldg(tile_info + item / nh), item, nh, hw);
    }
  }
};

// Rare path of the softmax warps, kept out of line so that its registers do not add to the
// 128 live scores of the caller: scale this thread's accumulator row by alpha in tensor memory.
__device__ __noinline__ void g_rescale_accumulator(uint32_t o_addr, float alpha) {
  for (int h = 0; h < 8; ++h) {
    uint32_t ov[8];
    g_tmem_ld8(o_addr + h * 8, ov);
    tmem_ld_wait();
#pragma unroll
    for (int d = 0; d < 8; ++d) ov[d] = __float_as_uint(__uint_as_float(ov[d]) * alpha);
    g_tmem_st8(o_addr + h * 8, ov);
  }
  g_tmem_st_wait();
}

// Rare path of the softmax warps (out of line, with registers of its own): the scores of one
// query row against the 128 keys of a tile by hand - fp32 dot products of the bf16 inputs in
// global memory.  Pass 0 takes the row maximum, pass 1 exponentiates against it and writes P
// one column (two keys) at a time.  Taken only when a tile's row sum shows that P overflowed or
// vanished against the inherited reference, which needs scores 2^60 apart within a row; every
// lane of the warp comes here together, lanes that are not `bad` keep their reference.
struct GByHand {
  float m_ref, l_run, sum;
};
__device__ __noinline__ GByHand g_tile_by_hand(const __nv_bfloat16* qrow, const __nv_bfloat16* k0, int64_t ld, int len,
                                               int col0, int c_lo, int c_hi, uint32_t lane_addr, float m_ref,
                                               float l_run, bool bad, bool have_acc) {
  const float scale_log2 = 0.125f * 1.4426950408889634f;
  uint4 qv[8];  // the row of q as packed bf16 pairs
#pragma unroll
  for (int i = 0; i < 8; ++i) qv[i] = __ldg(reinterpret_cast<const uint4*>(qrow) + i);
  float m = -INFINITY, sum = 0.f;
#pragma unroll 1
  for (int step = 0; step < 128; ++step) {
    const int cp = step & 63, c = 2 * cp;
    if (step == 64) {  // between the passes: the new reference, the accumulator moved to it
      const float m_new = m * scale_log2;
      const bool move = bad && m > -INFINITY;
      const float alpha = (move && have_acc) ? g_ex2(m_ref - m_new) : 1.0f;
      if (have_acc) {
        g_rescale_accumulator(lane_addr + G_O_COL, alpha);
        l_run *= alpha;
      }
      if (move) m_ref = m_new;
    }
    float s01[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int key = min(max(col0 + c + h, 0), len - 1);  // for the address only; validity below
      const uint4* krow = reinterpret_cast<const uint4*>(k0 + key * ld);
      float2 acc[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 u = __ldg(krow + i);
        acc[0] = __ffma2_rn(bf16x2_to_float2(qv[i].x), bf16x2_to_float2(u.x), acc[0]);
        acc[1] = __ffma2_rn(bf16x2_to_float2(qv[i].y), bf16x2_to_float2(u.y), acc[1]);
        acc[2] = __ffma2_rn(bf16x2_to_float2(qv[i].z), bf16x2_to_float2(u.z), acc[2]);
        acc[3] = __ffma2_rn(bf16x2_to_float2(qv[i].w), bf16x2_to_float2(u.w), acc[3]);
      }
      const float sc = ((acc[0].x + acc[0].y) + (acc[1].x + acc[1].y)) + ((acc[2].x + acc[2].y) + (acc[3].x + acc[3].y));
      s01[h] = (c + h >= c_lo && c + h <= c_hi) ? sc : -INFINITY;
    }
    if (step < 64) {
      m = fmax3(m, s01[0], s01[1]);
    } else {
      const float p0 = g_ex2(fmaf(s01[0], scale_log2, -m_ref));
      const float p1 = g_ex2(fmaf(s01[1], scale_log2, -m_ref));
      sum += p0 + p1;
      g_tmem_st1(lane_addr + G_P_COL + cp, pack_bf16(p0, p1));
    }
  }
  return GByHand{m_ref, l_run, sum};
}

__global__ void __launch_bounds__(G_THREADS, 2)
attn_global_tc_kernel(const __grid_constant__ CUtensorMap tm_qkv, const int4* __restrict__ tile_info,
                      const int32_t* __restrict__ total_tiles_ptr, int nh, int half_window,
                      const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ out, int* status) {
  const int total_items = *total_tiles_ptr * nh;
  if (int(blockIdx.x) >= total_items) return;  // whole CTA leaves before any barrier or allocation

  extern __shared__ __align__(1024) uint8_t g_smem[];
  const uint32_t base = smem_u32(g_smem);
  if (base & 1023u) {  // the swizzled tiles need it; nothing has been allocated yet
    if (threadIdx.x == 0) set_status(status, ST_ATTN_SMEM_MISALIGNED);
    return;
  }
  const uint32_t sQ = base;
  const uint32_t sK = sQ + G_TILE_BYTES;       // K[s] at + s * 16 KB
  const uint32_t sV = sK + G_STAGES * G_TILE_BYTES;  // V[s] at + s * 16 KB
  const uint32_t bar_base = sV + G_STAGES * G_TILE_BYTES;
  auto bar = [&](int i) { return bar_base + 8u * i; };
  const uint32_t tmem_slot = bar_base + 8u * GB_COUNT;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int H = nh * 64;
  const int stride_items = gridDim.x;

  if (threadIdx.x == 0) {
    mbar_init(bar(GB_Q_FULL), 1);
    mbar_init(bar(GB_Q_EMPTY), 1);
    for (int s = 0; s < G_STAGES; ++s) {
      mbar_init(bar(GB_K_FULL + s), 1);
      mbar_init(bar(GB_K_EMPTY + s), 1);
      mbar_init(bar(GB_V_FULL + s), 1);
      mbar_init(bar(GB_V_EMPTY + s), 1);
    }
    mbar_init(bar(GB_S_FULL), 1);
    mbar_init(bar(GB_S_EMPTY), 4);  // one arrival per softmax warp
    mbar_init(bar(GB_P_FULL), 4);
    mbar_init(bar(GB_O_FULL), 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_qkv);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, G_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  if (warp == 4) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      GCursor kc, vc;
      kc.open(tile_info, blockIdx.x, total_items, nh, half_window);
      vc = kc;
      uint32_t gk = 0, gv = 0, nq = 0;  // K tiles, V tiles, Q tiles loaded so far
      bool ok = true;
      while (ok && vc.item < total_items) {
        while (ok && kc.item < total_items && gk <= gv + 1) {  // K runs one tile ahead of V
          if (kc.j == 0) {
            // warm L2 with the first tiles of an item a few steps ahead
            const int ahead = kc.item + G_PREFETCH_ITEMS * stride_items;
            if (ahead < total_items) {
              const GItem nx = g_make_item(__ldg(tile_info + ahead / nh), ahead, nh, half_window);
              const int c = nx.head * 64;
              tma_prefetch_l2_2d(&tm_qkv, c, nx.seq_begin + nx.q0);
              for (int j = 0; j < min(nx.n_kv, 2); ++j) {
                const int r = nx.seq_begin + nx.kv_start + j * G_BN;
                tma_prefetch_l2_2d(&tm_qkv, H + c, r);
                tma_prefetch_l2_2d(&tm_qkv, 2 * H + c, r);
              }
            }
            ok = mbar_wait(bar(GB_Q_EMPTY), (nq & 1) ^ 1u, status, ST_ATTN_TIMEOUT);
            if (!ok) break;
            mbar_expect_tx(bar(GB_Q_FULL), G_TILE_BYTES);
            tma_load_2d(sQ, &tm_qkv, bar(GB_Q_FULL), kc.it.head * 64, kc.it.seq_begin + kc.it.q0);
            ++nq;
          }
          const uint32_t s = gk % G_STAGES;
          ok = mbar_wait(bar(GB_K_EMPTY + s), ((gk / G_STAGES) & 1) ^ 1u, status, ST_ATTN_TIMEOUT);
          if (!ok) break;
          mbar_expect_tx(bar(GB_K_FULL + s), G_TILE_BYTES);
          tma_load_2d(sK + s * G_TILE_BYTES, &tm_qkv, bar(GB_K_FULL + s), H + kc.it.head * 64,
                      kc.it.seq_begin + kc.it.kv_start + kc.j * G_BN);
          ++gk;
          kc.advance(tile_info, stride_items, total_items, nh, half_window);
        }
        if (!ok) break;
        const uint32_t s = gv % G_STAGES;
        ok = mbar_wait(bar(GB_V_EMPTY + s), ((gv / G_STAGES) & 1) ^ 1u, status, ST_ATTN_TIMEOUT);
        if (!ok) break;
        mbar_expect_tx(bar(GB_V_FULL + s), G_TILE_BYTES);
        tma_load_2d(sV + s * G_TILE_BYTES, &tm_qkv, bar(GB_V_FULL + s), 2 * H + vc.it.head * 64,
                    vc.it.seq_begin + vc.it.kv_start + vc.j * G_BN);
        ++gv;
        vc.advance(tile_info, stride_items, total_items, nh, half_window);
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 64, 1);  // B (= V) is MN-major
      GCursor qc, pc;
      qc.open(tile_info, blockIdx.x, total_items, nh, half_window);
      pc = qc;
      uint32_t gq = 0, gp = 0, nq = 0;  // Q K^T tiles issued, P V tiles issued, items begun
      bool ok = true;
      // S = Q K^T for the tile under the q cursor; the caller has made sure S is free.
      auto issue_qk = [&]() {
        const uint32_t s = gq % G_STAGES;
        if (qc.j == 0) ok = mbar_wait(bar(GB_Q_FULL), nq & 1, status, ST_ATTN_MMA_TIMEOUT);
        ok = ok && mbar_wait(bar(GB_K_FULL + s), (gq / G_STAGES) & 1, status, ST_ATTN_MMA_TIMEOUT);
        if (!ok) return;
        tc_fence_after();
        const uint64_t qdesc = umma_smem_desc_sw128(sQ, 1024);
        const uint64_t kdesc = umma_smem_desc_sw128(sK + s * G_TILE_BYTES, 1024);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(tmem_base + G_S_COL, qdesc + 2u * kk, kdesc + 2u * kk, idesc_qk, kk != 0 ? 1u : 0u);
        umma_commit(bar(GB_S_FULL));
        umma_commit(bar(GB_K_EMPTY + s));
        ++gq;
        if (qc.j + 1 == qc.it.n_kv) {  // last key tile of the item: Q is free once these retire
          umma_commit(bar(GB_Q_EMPTY));
          ++nq;
        }
        qc.advance(tile_info, stride_items, total_items, nh, half_window);
      };
      if (qc.item < total_items) issue_qk();
      while (ok && pc.item < total_items) {
        // The softmax warps release S as soon as tile gp is in their registers: the next
        // Q K^T then runs under their exp2 work.  Across an item boundary the next Q may still
        // be in flight; then P V goes first so the item's epilogue is not held up.
        bool qk_pending = qc.item < total_items;
        if (qk_pending && (qc.j != 0 || mbar_try_wait(bar(GB_Q_FULL), nq & 1))) {
          ok = mbar_wait(bar(GB_S_EMPTY), gp & 1, status, ST_ATTN_MMA_TIMEOUT);
          if (!ok) break;
          issue_qk();
          if (!ok) break;
          qk_pending = false;
        }
        {
          const uint32_t s = gp % G_STAGES;
          ok = mbar_wait(bar(GB_P_FULL), gp & 1, status, ST_ATTN_MMA_TIMEOUT) &&
               mbar_wait(bar(GB_V_FULL + s), (gp / G_STAGES) & 1, status, ST_ATTN_MMA_TIMEOUT);
          if (!ok) break;
          tc_fence_after();
          const uint32_t vbase = sV + s * G_TILE_BYTES;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            // A: keys [16 kk, 16 kk + 16) of P, straight from tensor memory: 8 columns of pairs
            // B: V rows [16 kk, 16 kk + 16), 128 bytes per row
            const uint64_t vdesc = umma_smem_desc_sw128(vbase + kk * 2048, 1024);
            g_umma_ts(tmem_base + G_O_COL, tmem_base + G_P_COL + kk * 8, vdesc, idesc_pv,
                      (pc.j | kk) != 0 ? 1u : 0u);
          }
          umma_commit(bar(GB_O_FULL));
          umma_commit(bar(GB_V_EMPTY + s));
          ++gp;
          pc.advance(tile_info, stride_items, total_items, nh, half_window);
        }
        if (qk_pending) {  // S was released before P was complete, so no wait on S_EMPTY is needed
          issue_qk();
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax warps
    const int row = threadIdx.x;  // query row within the tile = tensor-memory lane
    const uint32_t lane_addr = tmem_base + (uint32_t(warp * 32) << 16);
    const float scale_log2 = 0.125f * 1.4426950408889634f;  // 1/sqrt(64) * log2(e)
    bool ok = true;
    // After a bounded wait has given up, `ok` is false: waits are skipped but the loops still
    // run to the end (on garbage), so the CTA reaches its final barrier and frees tensor memory.
    auto wait = [&](uint32_t barrier, uint32_t parity) {
      if (ok && !mbar_wait(barrier, parity, status, ST_ATTN_SOFTMAX_TIMEOUT)) ok = false;
    };
    uint32_t g = 0;  // key tiles consumed so far
    for (int item = blockIdx.x; item < total_items; item += stride_items) {
      // Only what the tile loop needs stays in registers beside the 128 scores; the epilogue
      // re-reads the item's descriptor.
      int n_kv, col0, key_lo, key_hi;  // key tiles; key of column 0; valid keys of this row
      {
        const GItem it = g_make_item(__ldg(tile_info + item / nh), item, nh, half_window);
        const int qi = it.q0 + row;
        n_kv = it.n_kv;
        col0 = it.kv_start;
        key_lo = 0;
        key_hi = it.len - 1;
        if (half_window >= 0) {
          key_lo = max(0, qi - half_window);
          key_hi = min(it.len - 1, qi + half_window);
        }
        // Rows past the end of the sequence are computed like the others (on whatever TMA
        // fetched) and never stored: masking them would only make their warps diverge.
      }
      // P and the accumulator are scaled to 2^m_ref.  m_ref need not be the running maximum:
      // fp32 and bf16 carry 8 exponent bits, so any reference within about 2^60 of the maximum
      // gives the same relative precision.  No maximum is taken at all: a tile is exponentiated
      // against the reference it inherits, and its row sum - which the softmax needs anyway -
      // bounds its maximum from both sides (max <= sum <= 128 max).  A sum of 2^16 or more moves
      // the reference up by that power of two at the next tile (pending; the factor is exact).
      // A sum beyond 2^60, or not finite, or, for an item's first tile, below 2^-60, means that
      // P has overflowed or vanished: then, and only then, the tile's scores are recomputed by
      // hand from q and k in global memory and exponentiated against their true maximum.
      float m_ref = 0.f;
      float l_run = 0.f;
      int k_pend = 0;
      bool pend = false;
      for (int j = 0; j < n_kv; ++j, ++g, col0 += G_BN) {
        wait(bar(GB_S_FULL), g & 1);
        tc_fence_after();
        uint32_t sv[128];
        g_tmem_ld32(lane_addr + G_S_COL, sv);
        g_tmem_ld32(lane_addr + G_S_COL + 32, sv + 32);
        g_tmem_ld32(lane_addr + G_S_COL + 64, sv + 64);
        g_tmem_ld32(lane_addr + G_S_COL + 96, sv + 96);
        const int c_lo = key_lo - col0, c_hi = key_hi - col0;  // valid columns [c_lo, c_hi]
        // warp-uniform, so a warp never runs both branches
        const bool full = __all_sync(0xffffffffu, c_lo <= 0 && c_hi >= G_BN - 1);
        if (__builtin_expect(__any_sync(0xffffffffu, pend), 0)) {  // rare: move the reference up by 2^k_pend
          wait(bar(GB_O_FULL), (g - 1) & 1);  // the last tile's P V has retired (pend is never set when j == 0)
          tc_fence_after();
          const float alpha = pend ? __int_as_float((127 - k_pend) << 23) : 1.0f;
          g_rescale_accumulator(lane_addr + G_O_COL, alpha);
          l_run *= alpha;
          if (pend) m_ref += float(k_pend);
        }
        tmem_ld_wait();
        // All 128 scores are in registers and S is not read again: the next Q K^T may overwrite it.
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(GB_S_EMPTY));
        // A tile that is not valid for every row of the warp (the last one of a sequence, every
        // one of a band) first has its invalid scores replaced by -inf, in one block of its own;
        // the exponentials below are then the same code for every tile.  (Separate unrolled
        // variants per 16-column group were 1 % faster on bands and cost more than that on full
        // attention by crowding the instruction cache.)
        if (__builtin_expect(!full, 0)) {
#pragma unroll
          for (int c = 0; c < 128; ++c) sv[c] = (c >= c_lo && c <= c_hi) ? sv[c] : 0xff800000u;  // -inf
        }
        // Two scores at a time through the packed fp32 instructions of sm_100 (one FFMA2 for
        // the scale-and-shift, one FADD2 for the row sums): the softmax is bound by instruction
        // issue.
        float2 sum2[4] = {{0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}, {0.f, 0.f}};
        const float2 scale2 = make_float2(scale_log2, scale_log2);
        const float2 shift2 = make_float2(-m_ref, -m_ref);
        auto exp16 = [&](int c16, uint32_t* pk) {  // 16 keys -> 8 bf16 pairs
#pragma unroll
          for (int e = 0; e < 16; e += 2) {
            const float2 x = __ffma2_rn(make_float2(__uint_as_float(sv[c16 * 16 + e]),
                                                    __uint_as_float(sv[c16 * 16 + e + 1])), scale2, shift2);
            const float2 p = make_float2(g_ex2(x.x), g_ex2(x.y));
            sum2[(e >> 1) & 3] = __fadd2_rn(sum2[(e >> 1) & 3], p);
            pk[e >> 1] = pack_bf16(p.x, p.y);
          }
        };
        uint32_t pkh[G_HOLD][8];  // P of the first 16 * G_HOLD keys, held until the P buffer is free
#pragma unroll
        for (int c16 = 0; c16 < G_HOLD; ++c16) exp16(c16, pkh[c16]);
        if (j > 0) {
          // P is a single buffer: the previous tile's P V must have retired before P is
          // overwritten.  Holding the first groups of P in registers (which the scores they
          // were made from no longer need) puts this wait where it no longer waits.
          wait(bar(GB_O_FULL), (g - 1) & 1);
          tc_fence_after();
        }
#pragma unroll
        for (int c16 = 0; c16 < G_HOLD; ++c16) g_tmem_st8(lane_addr + G_P_COL + c16 * 8, pkh[c16]);
#pragma unroll
        for (int c16 = G_HOLD; c16 < 8; ++c16) {
          uint32_t pk[8];
          exp16(c16, pk);
          g_tmem_st8(lane_addr + G_P_COL + c16 * 8, pk);
        }
        float sum_tile = ((sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y)) + ((sum2[2].x + sum2[2].y) + (sum2[3].x + sum2[3].y));
        const bool has_key = full || (c_hi >= 0 && c_lo <= G_BN - 1 && c_hi >= c_lo);
        const bool bad = !(sum_tile <= G_SUM_MAX) || (j == 0 && has_key && sum_tile < G_SUM_MIN);
        if (__builtin_expect(__any_sync(0xffffffffu, bad), 0)) {
          g_tmem_st_wait();
          const int64_t ld = 3 * int64_t(H);
          const GItem it = g_make_item(__ldg(tile_info + item / nh), item, nh, half_window);
          const GByHand r = g_tile_by_hand(qkv + (int64_t(it.seq_begin) + min(it.q0 + row, it.len - 1)) * ld + it.head * 64,
                                           qkv + int64_t(it.seq_begin) * ld + H + it.head * 64, ld, it.len, col0,
                                           full ? 0 : c_lo, full ? G_BN - 1 : c_hi, lane_addr, m_ref, l_run, bad, j > 0);
          m_ref = r.m_ref;
          l_run = r.l_run;
          sum_tile = r.sum;
        }
        g_tmem_st_wait();
        l_run += sum_tile;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(GB_P_FULL));
        // floor(log2(sum)) from the exponent field; a sum of 0 gives -127
        k_pend = (__float_as_int(sum_tile) >> 23) - 127;
        pend = k_pend >= G_RESCALE_LOG2_SUM && k_pend <= 127;
      }
      {  // the item's accumulator: normalise and store this row
        const GItem it = g_make_item(__ldg(tile_info + item / nh), item, nh, half_window);
        const int qi = it.q0 + row;
        wait(bar(GB_O_FULL), (g - 1) & 1);
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* orow = out + (int64_t(it.seq_begin) + qi) * H + it.head * 64;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t ov[32];
          g_tmem_ld32(lane_addr + G_O_COL + h * 32, ov);
          tmem_ld_wait();
          if (ok && qi < it.len) {
#pragma unroll
            for (int d8 = 0; d8 < 4; ++d8) {
              uint4 w;
              w.x = pack_bf16(__uint_as_float(ov[d8 * 8 + 0]) * inv, __uint_as_float(ov[d8 * 8 + 1]) * inv);
              w.y = pack_bf16(__uint_as_float(ov[d8 * 8 + 2]) * inv, __uint_as_float(ov[d8 * 8 + 3]) * inv);
              w.z = pack_bf16(__uint_as_float(ov[d8 * 8 + 4]) * inv, __uint_as_float(ov[d8 * 8 + 5]) * inv);
              w.w = pack_bf16(__uint_as_float(ov[d8 * 8 + 6]) * inv, __uint_as_float(ov[d8 * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + h * 32 + d8 * 8) = w;
            }
          }
        }
        // The next item's first P V overwrites O; it waits for this warp's next P_FULL arrival,
        // which follows these loads in program order.
        tc_fence_before();
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, G_TMEM_COLS);
  }
}

int attn_run_global_tc(const void* qkv, const int4* tile_info, const int32_t* total_tiles,
                       int64_t max_tiles, int64_t T, int nh, int half_window, void* out,
                       int32_t* status, cudaStream_t st) {
  int rc = set_max_dynamic_smem(reinterpret_cast<const void*>(attn_global_tc_kernel), G_SMEM, true);
  if (rc != PE_OK) return rc;
  CUtensorMap tm;
  rc = make_tmap_bf16_2d(&tm, qkv, (uint64_t)T, (uint64_t)(3 * nh * 64), (uint64_t)(3 * nh * 64),
                             128);
  if (rc != PE_OK) return rc;
  const int64_t max_items = max_tiles * nh;
  const int64_t slots = 2 * (int64_t)sm_count();  // two resident CTAs per SM
  const int grid = (int)(max_items < slots ? max_items : slots);
  attn_global_tc_kernel<<<grid, G_THREADS, G_SMEM, st>>>(tm, tile_info, total_tiles, nh, half_window,
                                                        static_cast<const __nv_bfloat16*>(qkv),
                                                        static_cast<__nv_bfloat16*>(out), status);
  PE_LAUNCH_CHECK("attn_global_tc_kernel");
  return PE_OK;
}

}  // namespace pe
