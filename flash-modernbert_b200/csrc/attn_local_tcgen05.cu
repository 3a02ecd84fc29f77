// Sliding-window (|i - j| <= 64) varlen attention on the sm_100a tensor cores, two CTAs per SM.
//
// A 128-query tile attends a window of at most 256 keys (64 before its first query to 64 after
// its last), so an item (query tile, head) is ONE pass: S = Q K^T for both 128-key tiles, a
// reference exponent per row (the row maximum, or a cheaper bound within 2^60 above it),
// P = exp2(S - reference), O = P V.  There is no running maximum to maintain and nothing to
// rescale.  What limits such a kernel is latency: one softmax warp per scheduler
// executes a long dependent instruction stream per item, and each item is a chain of TMA ->
// MMA -> softmax -> MMA -> store.  So a CTA is kept small enough for two to share an SM
// (192 threads, 113 KB of shared memory, 256 tensor-memory columns) and otherwise simple: a
// CTA works through its items strictly one after the other, and the second CTA fills the gaps.
//
// Tensor memory of a CTA (256 columns), reused in place within an item:
//   columns   0..255 : S (key tile j at 128 j), written by 8 MMAs
//   columns   0..127 : P as bf16 pairs, written by the softmax threads over scores they have
//                      already consumed: the 32-column chunk c of S becomes the 16 columns at
//                      16 c, which never reaches past a chunk that is still unread (lanes are
//                      private to their thread, so only the thread's own order matters)
//   columns 128..191 : O, written by P V (16 MMAs with P as the tensor-memory A operand) after
//                      every thread has turned its S into P
// Shared memory: Q (16 KB), K of this item and of the next (2 x 32 KB), V of this item (32 KB,
// fetched while the scores are being computed and exponentiated; once P V has retired the same
// buffer stages the output rows for coalesced stores).
//   warps 0..3 : softmax - thread t owns query row t.  Of the eight 32-column chunks a warp
//                needs five (its rows' windows start between columns 32 w and 32 w + 31): chunks
//                are classified per warp as valid / masked / mixed; masked chunks are never
//                read, their P is written as zeros.  Two passes over tensor memory (maxima,
//                then exponentials), each fetching three chunks and then two per round trip.
//   warp 4     : TMA producer, warp 5 : tensor-memory owner and MMA issuer
// Every mbarrier wait is bounded and reports through the status word.
#include "pe_host.h"
#include "pe_ptx.cuh"
#include "attn_tmem.cuh"

namespace pe {

constexpr int LW_THREADS = 192;
constexpr int LW_TILE_BYTES = 128 * 64 * 2;  // one 128 x 64 bf16 tile
// Q, K[2 items][2 tiles], V[2 tiles] = 7 tiles, then the barriers.  No alignment slack: the
// kernel checks that the dynamic shared memory starts on a 1024-byte boundary.
constexpr int LW_SMEM = 7 * LW_TILE_BYTES + 256;
constexpr uint32_t LW_TMEM_COLS = 256;
constexpr uint32_t LW_O_COL = 128;
constexpr int LW_HALF_WINDOW = 64;

enum {
  LB_Q_FULL = 0,
  LB_Q_EMPTY = 1,
  LB_K_FULL = 2,   // 2 (item parity)
  LB_K_EMPTY = 4,  // 2
  LB_V_FULL = 6,
  LB_V_EMPTY = 7,
  LB_S_FULL = 8,
  LB_P_FULL = 9,   // 4 arrivals: every softmax warp has turned its S into P
  LB_O_FULL = 10,
  LB_S_FREE = 11,  // 4 arrivals: every softmax warp has read its rows of O
  LB_COUNT = 12
};

struct LwItem {
  int seq_begin, len, q0, head;
};

__device__ __forceinline__ LwItem lw_item(const int4* __restrict__ tile_info, int item, int nh) {
  const int4 info = __ldg(tile_info + item / nh);
  LwItem it;
  it.seq_begin = info.x;
  it.len = info.y;
  it.q0 = info.z;
  it.head = item % nh;
  return it;
}

__global__ void __launch_bounds__(LW_THREADS, 2)
attn_local_tc2_kernel(const __grid_constant__ CUtensorMap tm_qkv, const int4* __restrict__ tile_info,
                      const int32_t* __restrict__ total_tiles_ptr, int nh,
                      __nv_bfloat16* __restrict__ out, int* status) {
  const int total_items = *total_tiles_ptr * nh;
  if (int(blockIdx.x) >= total_items) return;  // whole CTA leaves before any barrier or allocation

  extern __shared__ __align__(1024) uint8_t lw_smem[];
  const uint32_t base = smem_u32(lw_smem);
  if (base & 1023u) {  // the swizzled tiles need it; nothing has been allocated yet
    if (threadIdx.x == 0) set_status(status, ST_ATTN_SMEM_MISALIGNED);
    return;
  }
  const uint32_t sQ = base;
  const uint32_t sK = sQ + LW_TILE_BYTES;      // K[item parity][tile] at + (2 parity + tile) * 16 KB
  const uint32_t sV = sK + 4 * LW_TILE_BYTES;  // V[tile] at + tile * 16 KB
  const uint32_t bar_base = sV + 2 * LW_TILE_BYTES;
  auto bar = [&](int i) { return bar_base + 8u * i; };
  const uint32_t tmem_slot = bar_base + 8u * LB_COUNT;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int H = nh * 64;
  const int stride_items = gridDim.x;

  if (threadIdx.x == 0) {
    mbar_init(bar(LB_Q_FULL), 1);
    mbar_init(bar(LB_Q_EMPTY), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(LB_K_FULL + s), 1);
      mbar_init(bar(LB_K_EMPTY + s), 1);
    }
    mbar_init(bar(LB_V_FULL), 1);
    mbar_init(bar(LB_V_EMPTY), 4);  // the softmax warps release it: V's buffer doubles as their output staging
    mbar_init(bar(LB_S_FULL), 1);
    mbar_init(bar(LB_P_FULL), 4);
    mbar_init(bar(LB_O_FULL), 1);
    mbar_init(bar(LB_S_FREE), 4);
    mbar_fence_init();
    tma_prefetch_desc(&tm_qkv);
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, LW_TMEM_COLS);
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
      // Item n needs Q(n) and K(n) before its Q K^T and V(n) before its P V.  In the order the
      // buffers come free: K(n + 1) once Q K^T of item n - 1 has retired (other parity), V(n)
      // once P V of item n - 1 has retired, Q(n + 1) once Q K^T of item n has retired.
      auto load_q = [&](const LwItem& it) {
        mbar_expect_tx(bar(LB_Q_FULL), LW_TILE_BYTES);
        tma_load_2d(sQ, &tm_qkv, bar(LB_Q_FULL), it.head * 64, it.seq_begin + it.q0);
      };
      auto load_k = [&](const LwItem& it, uint32_t par) {
        const int row = it.seq_begin + it.q0 - LW_HALF_WINDOW;  // may be negative: filled, then masked
        mbar_expect_tx(bar(LB_K_FULL + par), 2 * LW_TILE_BYTES);
        tma_load_2d(sK + (2 * par) * LW_TILE_BYTES, &tm_qkv, bar(LB_K_FULL + par), H + it.head * 64, row);
        tma_load_2d(sK + (2 * par + 1) * LW_TILE_BYTES, &tm_qkv, bar(LB_K_FULL + par), H + it.head * 64,
                    row + 128);
      };
      auto load_v = [&](const LwItem& it) {
        const int row = it.seq_begin + it.q0 - LW_HALF_WINDOW;
        mbar_expect_tx(bar(LB_V_FULL), 2 * LW_TILE_BYTES);
        tma_load_2d(sV, &tm_qkv, bar(LB_V_FULL), 2 * H + it.head * 64, row);
        tma_load_2d(sV + LW_TILE_BYTES, &tm_qkv, bar(LB_V_FULL), 2 * H + it.head * 64, row + 128);
      };
      LwItem cur = lw_item(tile_info, blockIdx.x, nh);
      load_q(cur);
      load_k(cur, 0);
      uint32_t n = 0;
      for (int item = blockIdx.x; item < total_items; item += stride_items, ++n) {
        const int next = item + stride_items;
        LwItem nx = cur;
        if (next < total_items) {
          nx = lw_item(tile_info, next, nh);
          const uint32_t par = (n + 1) & 1;
          if (!mbar_wait(bar(LB_K_EMPTY + par), (((n + 1) >> 1) & 1) ^ 1u, status, ST_ATTN_TIMEOUT)) break;
          load_k(nx, par);
        }
        if (!mbar_wait(bar(LB_V_EMPTY), (n & 1) ^ 1u, status, ST_ATTN_TIMEOUT)) break;
        load_v(cur);
        if (next < total_items) {
          if (!mbar_wait(bar(LB_Q_EMPTY), n & 1, status, ST_ATTN_TIMEOUT)) break;
          load_q(nx);
        }
        cur = nx;
      }
    }
    __syncwarp();
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 64, 1);  // B (= V) is MN-major
      uint32_t n = 0;
      for (int item = blockIdx.x; item < total_items; item += stride_items, ++n) {
        const uint32_t par = n & 1;
        bool ok = mbar_wait(bar(LB_Q_FULL), n & 1, status, ST_ATTN_MMA_TIMEOUT) &&
                  mbar_wait(bar(LB_K_FULL + par), (n >> 1) & 1, status, ST_ATTN_MMA_TIMEOUT);
        // S, P and O share the 256 columns: the previous item's output must have been read
        if (ok && n > 0) ok = mbar_wait(bar(LB_S_FREE), (n - 1) & 1, status, ST_ATTN_MMA_TIMEOUT);
        if (!ok) break;
        tc_fence_after();
        const uint64_t qdesc = umma_smem_desc_sw128(sQ, 1024);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint64_t kdesc = umma_smem_desc_sw128(sK + (2 * par + j) * LW_TILE_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tmem_base + j * 128, qdesc + 2u * kk, kdesc + 2u * kk, idesc_qk, kk != 0 ? 1u : 0u);
        }
        umma_commit(bar(LB_S_FULL));
        umma_commit(bar(LB_K_EMPTY + par));
        umma_commit(bar(LB_Q_EMPTY));

        ok = mbar_wait(bar(LB_P_FULL), n & 1, status, ST_ATTN_MMA_TIMEOUT) &&
             mbar_wait(bar(LB_V_FULL), n & 1, status, ST_ATTN_MMA_TIMEOUT);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
          // A: keys [16 k, 16 k + 16) of P = 8 columns of pairs at 8 k.
          // B: V rows [16 k, 16 k + 16) of the window: tile k / 8, 128 bytes per row
          const uint64_t vdesc = umma_smem_desc_sw128(sV + (k >> 3) * LW_TILE_BYTES + (k & 7) * 2048, 1024);
          g_umma_ts(tmem_base + LW_O_COL, tmem_base + k * 8, vdesc, idesc_pv, k != 0 ? 1u : 0u);
        }
        umma_commit(bar(LB_O_FULL));
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax warps
    const int row = threadIdx.x;  // query row within the tile = tensor-memory lane
    const uint32_t lane_addr = tmem_base + (uint32_t(warp * 32) << 16);
    const float scale_log2 = 0.125f * 1.4426950408889634f;  // 1/sqrt(64) * log2(e)
    const uint32_t stage = sV + warp * 4096;  // this warp's 32 x 128-byte output staging (V is dead by then)
    bool ok = true;
    // After a bounded wait has given up, `ok` is false: waits are skipped but the loop still
    // runs to the end (on garbage), so the CTA reaches its final barrier and frees tensor memory.
    auto wait = [&](uint32_t barrier, uint32_t parity) {
      if (ok && !mbar_wait(barrier, parity, status, ST_ATTN_SOFTMAX_TIMEOUT)) ok = false;
    };
    // Rows 32 w .. 32 w + 31 see window columns [32 w, 32 w + 159] at most: the warp needs the
    // five 32-column chunks w .. w + 4 and writes P = 0 for the other three.
    const int c_first = warp;
    uint32_t n = 0;
    // (query tile, head) of the item, advanced by the stride without a division per item
    int tile = blockIdx.x / nh, head = blockIdx.x % nh;
    const int stride_tiles = stride_items / nh, stride_heads = stride_items % nh;
    int4 info = __ldg(tile_info + tile);
    for (int item = blockIdx.x; item < total_items; item += stride_items, ++n) {
      const int seq_begin = info.x, len = info.y, q0 = info.z;
      const int this_head = head;
      tile += stride_tiles;
      head += stride_heads;
      if (head >= nh) {
        head -= nh;
        ++tile;
      }
      if (item + stride_items < total_items)  // next item's descriptor, in flight during this one
        info = __ldg(tile_info + tile);
      const int qi = q0 + row;  // position in the sequence
      // valid columns [c_lo, c_hi] of the 256-key window that starts at key q0 - 64
      const int c_lo = max(0, qi - LW_HALF_WINDOW) - (q0 - LW_HALF_WINDOW);
      const int c_hi = min(len - 1, qi + LW_HALF_WINDOW) - (q0 - LW_HALF_WINDOW);
      // the five chunks, classified for the whole warp: bit k set = chunk c_first + k
      uint32_t masked = 0, mixed = 0x11u;  // away from the ends of a sequence: chunks 0 and 4 are mixed
      if (q0 < LW_HALF_WINDOW || q0 + 128 + LW_HALF_WINDOW > len) {  // the window leaves the sequence
        mixed = 0;
#pragma unroll
        for (int k = 0; k < 5; ++k) {
          const int lo = (c_first + k) * 32, hi = lo + 31;
          if (__all_sync(0xffffffffu, c_hi < lo || c_lo > hi)) masked |= 1u << k;
          else if (!__all_sync(0xffffffffu, c_lo <= lo && c_hi >= hi)) mixed |= 1u << k;
        }
      }
      const uint32_t s_addr = lane_addr + c_first * 32;  // chunk k of this warp at + 32 k

      wait(bar(LB_S_FULL), n & 1);
      tc_fence_after();

      // Tensor-memory loads cost a round trip of a few hundred clocks each: both passes fetch
      // three chunks, then two, per wait.
      uint32_t va[32], vb[32], vc[32];
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains, not one
      // pass 1: the row maximum - or any reference within 2^60 above it, which serves as well
      // (P keeps its relative precision in bf16, the sums are fp32).  When chunks 1..3 are valid
      // for every row of the warp, the unmasked maximum over all five chunks is such a reference
      // unless chunk 0 or 4 holds an out-of-window score more than 2^60 above everything in
      // chunks 1..3: then, and at the ends of a sequence, the exact masked maximum is taken.
      bool have_m = false;
      if (masked == 0 && (mixed & 0xeu) == 0) {
        float e4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        auto raw = [&](const uint32_t* v, float* chain) {
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            chain[(i >> 1) & 3] = fmax3(chain[(i >> 1) & 3], __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
        };
        g_tmem_ld32(s_addr, va);
        g_tmem_ld32(s_addr + 32, vb);
        g_tmem_ld32(s_addr + 64, vc);
        tmem_ld_wait();
        raw(va, e4);
        g_tmem_ld32(s_addr + 96, va);
        raw(vb, mx4);
        g_tmem_ld32(s_addr + 128, vb);
        raw(vc, mx4);
        tmem_ld_wait();
        raw(va, mx4);
        raw(vb, e4);
        const float m_in = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const float m_edge = fmaxf(fmaxf(e4[0], e4[1]), fmaxf(e4[2], e4[3]));
        have_m = __all_sync(0xffffffffu, (m_edge - m_in) * scale_log2 <= 60.0f);
        mx4[0] = fmaxf(m_in, m_edge);
        if (!have_m) mx4[0] = mx4[1] = mx4[2] = mx4[3] = -INFINITY;
      }
      if (__builtin_expect(!have_m, 0)) {
        // Exact masked maximum: one copy of the code, rolled over the five chunks (a tensor-memory
        // round trip each).  Unrolled variants of every rarely-taken path would push the hot loops
        // out of the instruction cache.
#pragma unroll 1
        for (int k = 0; k < 5; ++k) {
          if (masked & (1u << k)) continue;
          g_tmem_ld32(s_addr + k * 32, va);
          tmem_ld_wait();
          const int lo = c_lo - (c_first + k) * 32, hi = c_hi - (c_first + k) * 32;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            mx4[i & 3] = fmaxf(mx4[i & 3], (i >= lo && i <= hi) ? __uint_as_float(va[i]) : -INFINITY);
        }
      }
      const float m = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
      const float m_safe = (m == -INFINITY) ? 0.f : m;  // a row with no valid key: P = 0 throughout

      // pass 2: P = exp2(S * scale - m) as bf16 pairs, chunk c of S into the 16 columns at 16 c
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      // Chunks 0 and 4 of a warp are where its rows' windows begin and end: they are always
      // masked with the two-sided column test; chunks 1..3 only where a sequence ends inside them.
      // The masking is a block of its own in front of one common exponentiation block.
      auto emit = [&](uint32_t* v, int k) {
        uint32_t pk[16];
        if (masked & (1u << k)) {
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[i] = 0u;
        } else {
          if (k == 0 || k == 4 || (mixed & (1u << k)) != 0) {
            const int lo = c_lo - (c_first + k) * 32, hi = c_hi - (c_first + k) * 32;
#pragma unroll
            for (int i = 0; i < 32; ++i)
              v[i] = (i >= lo && i <= hi) ? v[i] : 0xff800000u;  // -inf
          }
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = g_ex2(fmaf(__uint_as_float(v[i]), scale_log2, -m_safe));
            const float p1 = g_ex2(fmaf(__uint_as_float(v[i + 1]), scale_log2, -m_safe));
            sum4[(i >> 1) & 3] += p0 + p1;
            pk[i >> 1] = pack_bf16(p0, p1);
          }
        }
        g_tmem_st16(lane_addr + (c_first + k) * 16, pk);
      };
      g_tmem_ld32(s_addr, va);
      g_tmem_ld32(s_addr + 32, vb);
      g_tmem_ld32(s_addr + 64, vc);
      {  // chunks below the warp's first: columns [0, 16 c_first), none of which it still needs
        uint32_t z[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) z[i] = 0u;
        for (int c = 0; c < c_first; ++c) g_tmem_st16(lane_addr + c * 16, z);
      }
      tmem_ld_wait();
      emit(va, 0);
      g_tmem_ld32(s_addr + 96, va);
      emit(vb, 1);
      g_tmem_ld32(s_addr + 128, vb);
      emit(vc, 2);
      tmem_ld_wait();
      emit(va, 3);
      emit(vb, 4);
      {  // chunks above the warp's last: their columns held scores the warp needed until now
        uint32_t z[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) z[i] = 0u;
        for (int c = c_first + 5; c < 8; ++c) g_tmem_st16(lane_addr + c * 16, z);
      }
      g_tmem_st_wait();
      const float l = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(LB_P_FULL));

      // O = P V: normalise, turn the warp's 32 x 64 block from row-per-thread into row-major
      // through shared memory (V's buffer, dead once P V has retired) and store it coalesced:
      // four full 128-byte rows per instruction instead of 32 scattered 16-byte pieces.
      wait(bar(LB_O_FULL), n & 1);
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint32_t o0[32], o1[32];
      g_tmem_ld32(lane_addr + LW_O_COL, o0);
      g_tmem_ld32(lane_addr + LW_O_COL + 32, o1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(LB_S_FREE));  // the next item's Q K^T may overwrite the columns
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t* src = j < 4 ? o0 : o1;
        const int e = (j & 3) * 8;
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(stage + lane * 128 + ((j ^ (lane & 7)) << 4)),
                     "r"(pack_bf16(__uint_as_float(src[e + 0]) * inv, __uint_as_float(src[e + 1]) * inv)),
                     "r"(pack_bf16(__uint_as_float(src[e + 2]) * inv, __uint_as_float(src[e + 3]) * inv)),
                     "r"(pack_bf16(__uint_as_float(src[e + 4]) * inv, __uint_as_float(src[e + 5]) * inv)),
                     "r"(pack_bf16(__uint_as_float(src[e + 6]) * inv, __uint_as_float(src[e + 7]) * inv))
                     : "memory");
      }
      __syncwarp();
      {
        const int rows_valid = len - (q0 + warp * 32);  // rows of this warp inside the sequence
        __nv_bfloat16* obase = out + (int64_t(seq_begin) + q0 + warp * 32) * H + this_head * 64 + (lane & 7) * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = i * 4 + (lane >> 3);
          uint4 w;
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                       : "r"(stage + r * 128 + (((lane & 7) ^ (r & 7)) << 4)));
          if (ok && r < rows_valid) *reinterpret_cast<uint4*>(obase + int64_t(r) * H) = w;
        }
      }
      fence_proxy_async_smem();  // these generic-proxy accesses come before the TMA write that follows the release
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(LB_V_EMPTY));  // the staging area may take the next item's V
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, LW_TMEM_COLS);
  }
}

int attn_run_local_tc2(const void* qkv, const int4* tile_info, const int32_t* total_tiles,
                       int64_t max_tiles, int64_t T, int nh, void* out, int32_t* status,
                       cudaStream_t st) {
  int rc = set_max_dynamic_smem(reinterpret_cast<const void*>(attn_local_tc2_kernel), LW_SMEM, true);
  if (rc != PE_OK) return rc;
  CUtensorMap tm;
  rc = make_tmap_bf16_2d(&tm, qkv, (uint64_t)T, (uint64_t)(3 * nh * 64), (uint64_t)(3 * nh * 64),
                             128);
  if (rc != PE_OK) return rc;
  const int64_t max_items = max_tiles * nh;
  const int64_t slots = 2 * (int64_t)sm_count();  // two resident CTAs per SM
  const int grid = (int)(max_items < slots ? max_items : slots);
  attn_local_tc2_kernel<<<grid, LW_THREADS, LW_SMEM, st>>>(tm, tile_info, total_tiles, nh,
                                                          static_cast<__nv_bfloat16*>(out), status);
  PE_LAUNCH_CHECK("attn_local_tc2_kernel");
  return PE_OK;
}

}  // namespace pe
