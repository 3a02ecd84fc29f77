// The one-CTA-per-SM varlen attention kernels: the first tensor-core generation of this
// library, kept selectable (pe_set_option keys 5 and 6) as a cross-check for the two-CTA kernels
// in attn_global_tcgen05.cu and attn_local_tcgen05.cu, which the forward uses by default.
//
// Varlen attention for sequences longer than one short tile, on the sm_100a tensor
// cores: S = Q K^T and O = P V run as tcgen05.mma with S and O in tensor memory,
// Q / K / V tiles arrive by TMA straight from the fused qkv [T, 3*nh*64].
//
// Persistent CTAs (one per SM) walk work items (128-query tile, head) round-robin;
// each item walks 128-key tiles.  The three roles keep their own cursors over the
// same item sequence, so the pipeline never drains between items:
//   warps 0..3 : softmax - thread t owns query row t (tensor-memory lane t): reads its
//                128 scores with tcgen05.ld, online softmax in the exp2 domain, writes
//                P (bf16) into shared memory in the 128-byte-swizzled K-major layout
//                tcgen05.mma reads, then folds the previous tile's P V into its fp32
//                output row held in registers; stores the row at the end of the item
//   warp 4     : TMA producer - Q into a double buffer, K_j and V_j into a 3-stage ring,
//                running ahead across items as far as the buffers allow
//   warp 5     : tensor-memory owner and MMA issuer - S = Q K^T runs up to two key tiles
//                ahead (across item boundaries) into a double-buffered S; O_j = P_j V_j
//                goes to a double-buffered 64-column scratch that the softmax warps drain
// Keeping the running output in registers (rather than rescaling an accumulator in
// tensor memory) means P V never needs a correction pass over tensor memory.
//
// Rows of a K/V tile that lie outside the sequence (or outside the sliding window)
// are whatever TMA fetched - the neighbouring sequence or zero fill - and are masked
// to -inf before the softmax, so P is exactly 0 there.  Every mbarrier wait is
// bounded and reports through the status word.
#include "pe_host.h"
#include "pe_ptx.cuh"

namespace pe {

constexpr int TC_BM = 128;
constexpr int TC_BN = 128;
constexpr int TC_STAGES = 4;
constexpr int TC_PREFETCH_ITEMS = 3;  // how many items ahead the producer warms L2
constexpr int TC_TILE_BYTES = 128 * 64 * 2;          // one 128 x 64 bf16 tile (Q, K or V)
constexpr int TC_P_BYTES = 128 * 128 * 2;            // one P buffer: two 128 x 64 halves
constexpr int TC_THREADS = 192;         // single-pass kernel: 4 softmax warps + producer + MMA
constexpr int TC_THREADS_ONLINE = 320;  // online-softmax kernel: 8 softmax warps + producer + MMA
constexpr int TC_SMEM = TC_TILE_BYTES * (2 + 2 * TC_STAGES) + 2 * TC_P_BYTES + 1024 /*align*/ +
                        256 /*barriers*/ + 1024 /*row-sum mailbox*/;
constexpr uint32_t TC_TMEM_COLS = 512;
constexpr uint32_t TC_S_COL = 0;    // S[b] at columns b * 128
constexpr uint32_t TC_O_COL = 256;  // O[b] at columns 256 + b * 64

// barrier slots
enum {
  TCB_Q_FULL = 0,     // 2
  TCB_Q_EMPTY = 2,    // 2
  TCB_KV_FULL = 4,    // 4
  TCB_KV_EMPTY = 8,   // 4
  TCB_S_FULL = 12,    // 2
  TCB_S_EMPTY = 14,   // 2
  TCB_P_FULL = 16,    // 2
  TCB_O_FULL = 18,    // 2
  TCB_COUNT = 20
};

// One work item: a 128-query tile of one sequence, for one head.
struct TcItem {
  int seq_begin, len, q0, head;
  int kv_start, n_kv;
};

__device__ __forceinline__ TcItem tc_make_item(const int4 info, int item, int nh, int half_window) {
  TcItem it;
  it.seq_begin = info.x;
  it.len = info.y;
  it.q0 = info.z;
  it.head = item % nh;
  // key tile j covers keys [kv_start + 128 j, kv_start + 128 j + 128) of the sequence
  it.kv_start = 0;
  it.n_kv = (it.len + TC_BN - 1) / TC_BN;
  if (half_window >= 0) {
    it.kv_start = it.q0 - half_window;  // may be negative: those keys are masked
    const int kv_end = min(it.len, it.q0 + TC_BM + half_window);
    it.n_kv = (kv_end - it.kv_start + TC_BN - 1) / TC_BN;
  }
  return it;
}

__device__ __forceinline__ TcItem tc_load_item(const int4* __restrict__ tile_info, int item, int nh,
                                               int half_window) {
  return tc_make_item(__ldg(tile_info + item / nh), item, nh, half_window);
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void tmem_ld_32x32_nowait(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]),
        "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]),
        "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

template <bool LOCAL>
__global__ void __launch_bounds__(LOCAL ? TC_THREADS : TC_THREADS_ONLINE, 1)
attn_varlen_tc_kernel(const __grid_constant__ CUtensorMap tm_qkv, const int4* __restrict__ tile_info,
                      const int32_t* __restrict__ total_tiles_ptr, int nh, int half_window,
                      __nv_bfloat16* __restrict__ out, int* status) {
  const int total_items = *total_tiles_ptr * nh;
  if (int(blockIdx.x) >= total_items) return;  // whole CTA leaves before any barrier or allocation

  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base;                                      // Q[qb] at + qb * 16 KB
  const uint32_t sKV = sQ + 2 * TC_TILE_BYTES;                   // stage s: K at +0, V at +16 KB
  const uint32_t sP = sKV + 2 * TC_STAGES * TC_TILE_BYTES;       // P[b] at + b * 32 KB
  const uint32_t bar_base = sP + 2 * TC_P_BYTES;
  auto bar = [&](int i) { return bar_base + 8u * i; };
  const uint32_t tmem_slot = bar_base + 8u * TCB_COUNT;

  constexpr int NSW = LOCAL ? 4 : 8;  // softmax warps; then one producer warp, one MMA warp
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int H = nh * 64;
  const int stride_items = gridDim.x;

  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(TCB_Q_FULL + b), 1);
      mbar_init(bar(TCB_Q_EMPTY + b), 1);
      mbar_init(bar(TCB_S_FULL + b), 1);
      mbar_init(bar(TCB_S_EMPTY + b), NSW);
      mbar_init(bar(TCB_P_FULL + b), NSW);  // one arrival per softmax warp: per-thread arrivals
                                            // on one mbarrier serialise and cost microseconds
      mbar_init(bar(TCB_O_FULL + b), 1);
    }
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(bar(TCB_KV_FULL + s), 1);
      mbar_init(bar(TCB_KV_EMPTY + s), 1);
    }
    mbar_fence_init();
    tma_prefetch_desc(&tm_qkv);
  }
  if (warp == NSW + 1) {
    tmem_alloc(tmem_slot, TC_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  if (warp == NSW) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      uint32_t g = 0;  // key tiles loaded so far (ring position)
      uint32_t n = 0;  // items started so far (Q buffer position)
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += stride_items, ++n) {
        const TcItem it = tc_load_item(tile_info, item, nh, half_window);
        const int qcol = it.head * 64, kcol = H + qcol, vcol = 2 * H + qcol;
        const uint32_t qb = n & 1;
        {  // warm L2 with the first tiles of an item a few steps ahead: its loads then miss no DRAM
          const int ahead = item + TC_PREFETCH_ITEMS * stride_items;
          if (ahead < total_items) {
            const TcItem nx = tc_load_item(tile_info, ahead, nh, half_window);
            const int c = nx.head * 64;
            tma_prefetch_l2_2d(&tm_qkv, c, nx.seq_begin + nx.q0);
            for (int j = 0; j < min(nx.n_kv, 2); ++j) {
              const int r = nx.seq_begin + nx.kv_start + j * TC_BN;
              tma_prefetch_l2_2d(&tm_qkv, H + c, r);
              tma_prefetch_l2_2d(&tm_qkv, 2 * H + c, r);
            }
          }
        }
        if (!mbar_wait(bar(TCB_Q_EMPTY + qb), ((n >> 1) & 1) ^ 1u, status, ST_ATTN_TIMEOUT)) break;
        mbar_expect_tx(bar(TCB_Q_FULL + qb), TC_TILE_BYTES);
        tma_load_2d(sQ + qb * TC_TILE_BYTES, &tm_qkv, bar(TCB_Q_FULL + qb), qcol, it.seq_begin + it.q0);
        for (int j = 0; j < it.n_kv; ++j, ++g) {
          const uint32_t s = g % TC_STAGES;
          if (!mbar_wait(bar(TCB_KV_EMPTY + s), ((g / TC_STAGES) & 1) ^ 1u, status, ST_ATTN_TIMEOUT)) {
            ok = false;
            break;
          }
          const uint32_t dst = sKV + s * 2 * TC_TILE_BYTES;
          const int row = it.seq_begin + it.kv_start + j * TC_BN;
          mbar_expect_tx(bar(TCB_KV_FULL + s), 2 * TC_TILE_BYTES);
          tma_load_2d(dst, &tm_qkv, bar(TCB_KV_FULL + s), kcol, row);
          tma_load_2d(dst + TC_TILE_BYTES, &tm_qkv, bar(TCB_KV_FULL + s), vcol, row);
        }
      }
    }
    __syncwarp();
  } else if (warp == NSW + 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      if constexpr (LOCAL) {
        // One item = at most two key tiles = one softmax pass.  S of item n goes to region
        // n & 1 (256 columns) one item ahead of the softmax; O of item n is accumulated over its
        // tiles into the first 64 columns of the same region once its P is complete.
        constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0);
        constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 64, 1);
        uint32_t gq = 0, gp = 0, nq = 0, np = 0;
        int q_item = blockIdx.x;
        bool ok = true;
        auto issue_qk_item = [&]() {
          const TcItem it = tc_load_item(tile_info, q_item, nh, half_window);
          const uint32_t r = nq & 1;
          ok = mbar_wait(bar(TCB_S_EMPTY + r), ((nq >> 1) & 1) ^ 1u, status, ST_ATTN_MMA_TIMEOUT) &&
               mbar_wait(bar(TCB_Q_FULL + r), (nq >> 1) & 1, status, ST_ATTN_MMA_TIMEOUT);
          const uint64_t qdesc = umma_smem_desc_sw128(sQ + r * TC_TILE_BYTES, 1024);
          for (int j = 0; ok && j < it.n_kv; ++j, ++gq) {
            const uint32_t s = gq % TC_STAGES;
            ok = mbar_wait(bar(TCB_KV_FULL + s), (gq / TC_STAGES) & 1, status, ST_ATTN_MMA_TIMEOUT);
            if (!ok) break;
            tc_fence_after();
            const uint64_t kdesc = umma_smem_desc_sw128(sKV + s * 2 * TC_TILE_BYTES, 1024);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_ss(tmem_base + r * 256 + j * 128, qdesc + 2u * kk, kdesc + 2u * kk, idesc_qk,
                      kk != 0 ? 1u : 0u);
          }
          umma_commit(bar(TCB_S_FULL + r));
          umma_commit(bar(TCB_Q_EMPTY + r));
          ++nq;
          q_item += stride_items;
        };
        if (q_item < total_items) issue_qk_item();
        for (int p_item = blockIdx.x; ok && p_item < total_items; p_item += stride_items, ++np) {
          if (q_item < total_items) issue_qk_item();  // next item's S while this item's softmax runs
          if (!ok) break;
          const TcItem it = tc_load_item(tile_info, p_item, nh, half_window);
          const uint32_t r = np & 1;
          if (!mbar_wait(bar(TCB_P_FULL), np & 1, status, ST_ATTN_MMA_TIMEOUT)) break;
          tc_fence_after();
          for (int j = 0; j < it.n_kv; ++j, ++gp) {
            const uint32_t s = gp % TC_STAGES;
            const uint32_t pbase = sP + j * TC_P_BYTES;
            const uint32_t vbase = sKV + s * 2 * TC_TILE_BYTES + TC_TILE_BYTES;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const uint64_t pdesc =
                  umma_smem_desc_sw128(pbase + (kk >> 2) * TC_TILE_BYTES, 1024) + 2u * (kk & 3);
              const uint64_t vdesc = umma_smem_desc_sw128(vbase + kk * 2048, 1024);
              umma_ss(tmem_base + r * 256, pdesc, vdesc, idesc_pv, (j | kk) != 0 ? 1u : 0u);
            }
            umma_commit(bar(TCB_KV_EMPTY + s));
          }
          umma_commit(bar(TCB_O_FULL + r));
        }
      } else {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 64, 1);  // B (= V) is MN-major
      // Two cursors over the same flat sequence of key tiles: `q` issues S = Q K^T,
      // `p` issues O = P V; q runs at most two tiles ahead of p.
      int q_item = blockIdx.x, q_j = 0, q_nkv = 0;
      int p_item = blockIdx.x, p_j = 0, p_nkv = 0;
      uint32_t gq = 0, gp = 0, nq = 0;  // tiles issued by q / by p, items begun by q
      if (q_item < total_items) q_nkv = tc_load_item(tile_info, q_item, nh, half_window).n_kv;
      p_nkv = q_nkv;
      bool ok = true;
      while (ok && p_item < total_items) {
        while (ok && gq < gp + 2 && q_item < total_items) {
          const uint32_t s = gq % TC_STAGES, b = gq & 1, qb = nq & 1;
          if (q_j == 0) ok = mbar_wait(bar(TCB_Q_FULL + qb), (nq >> 1) & 1, status, ST_ATTN_MMA_TIMEOUT);
          ok = ok && mbar_wait(bar(TCB_KV_FULL + s), (gq / TC_STAGES) & 1, status, ST_ATTN_MMA_TIMEOUT);
          ok = ok && mbar_wait(bar(TCB_S_EMPTY + b), ((gq >> 1) & 1) ^ 1u, status, ST_ATTN_MMA_TIMEOUT);
          if (!ok) break;
          tc_fence_after();
          const uint64_t qdesc = umma_smem_desc_sw128(sQ + qb * TC_TILE_BYTES, 1024);
          const uint64_t kdesc = umma_smem_desc_sw128(sKV + s * 2 * TC_TILE_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(tmem_base + TC_S_COL + b * 128, qdesc + 2u * kk, kdesc + 2u * kk, idesc_qk,
                    kk != 0 ? 1u : 0u);
          umma_commit(bar(TCB_S_FULL + b));
          ++gq;
          if (++q_j == q_nkv) {  // last key tile of the item: its Q buffer is free once these MMAs retire
            umma_commit(bar(TCB_Q_EMPTY + qb));
            ++nq;
            q_item += stride_items;
            q_j = 0;
            if (q_item < total_items) q_nkv = tc_load_item(tile_info, q_item, nh, half_window).n_kv;
          }
        }
        if (!ok) break;
        {
          const uint32_t s = gp % TC_STAGES, b = gp & 1;
          if (!mbar_wait(bar(TCB_P_FULL + b), (gp >> 1) & 1, status, ST_ATTN_MMA_TIMEOUT)) break;
          tc_fence_after();
          const uint32_t pbase = sP + b * TC_P_BYTES;
          const uint32_t vbase = sKV + s * 2 * TC_TILE_BYTES + TC_TILE_BYTES;
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            // A: keys [16 kk, 16 kk + 16) of P = half kk / 4, 32-byte step kk % 4 inside the atom
            const uint64_t pdesc =
                umma_smem_desc_sw128(pbase + (kk >> 2) * TC_TILE_BYTES, 1024) + 2u * (kk & 3);
            // B: V rows [16 kk, 16 kk + 16), 128 bytes per row
            const uint64_t vdesc = umma_smem_desc_sw128(vbase + kk * 2048, 1024);
            umma_ss(tmem_base + TC_O_COL + b * 64, pdesc, vdesc, idesc_pv, kk != 0 ? 1u : 0u);
          }
          umma_commit(bar(TCB_O_FULL + b));
          umma_commit(bar(TCB_KV_EMPTY + s));
          ++gp;
          if (++p_j == p_nkv) {
            p_item += stride_items;
            p_j = 0;
            if (p_item < total_items) p_nkv = tc_load_item(tile_info, p_item, nh, half_window).n_kv;
          }
        }
      }
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax warps
    const int wq = warp & 3;                // tensor-memory lane quarter of this warp
    const int row = wq * 32 + lane;         // query row in the tile == tensor-memory lane
    const uint32_t lane_addr = tmem_base + (uint32_t(wq * 32) << 16);
    const float scale_log2 = 0.125f * 1.4426950408889634f;
    uint32_t g = 0;  // key tiles consumed so far
    bool ok = true;
    if constexpr (LOCAL) {
      // Sliding-window layers (|i - j| <= 64): an item has at most two key tiles, both fully
      // masked bands, so the whole item is one softmax pass.  Row r of the tile can only see
      // columns [r, r + 128] of the 256 fetched keys; warp w therefore reads 32-column chunks
      // w..3 of tile 0 and 0..w of tile 1 (five of eight) and writes zeros into the rest of P.
      // S of the item sits in tensor-memory region n & 1 (256 columns); once every row is in
      // registers, O = P V is accumulated into the first 64 columns of the same region.
      int4 info = __ldg(tile_info + blockIdx.x / nh);
      uint32_t n = 0;
      // The output row of item n - 1 is drained while item n is in flight: its P V runs during
      // item n's S load and masking, so the wait below does not stall, and handing region
      // (n - 1) & 1 back before item n's exp2 phase lets the MMA warp compute S of item n + 1
      // under it.
      bool prev_valid = false;
      uint32_t prev_r = 0, prev_phase = 0;
      float prev_inv = 0.f;
      __nv_bfloat16* prev_orow = nullptr;  // nullptr: row past the end of its sequence
      auto drain_prev = [&]() -> bool {
        if (!mbar_wait(bar(TCB_O_FULL + prev_r), prev_phase, status, ST_ATTN_SOFTMAX_TIMEOUT)) return false;
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t ov[32];
          tmem_ld_32x32_nowait(lane_addr + prev_r * 256 + h * 32, ov);
          tmem_ld_wait();
          if (prev_orow != nullptr) {
#pragma unroll
            for (int d8 = 0; d8 < 4; ++d8) {
              uint4 w4;
              w4.x = pack_bf16(__uint_as_float(ov[d8 * 8 + 0]) * prev_inv, __uint_as_float(ov[d8 * 8 + 1]) * prev_inv);
              w4.y = pack_bf16(__uint_as_float(ov[d8 * 8 + 2]) * prev_inv, __uint_as_float(ov[d8 * 8 + 3]) * prev_inv);
              w4.z = pack_bf16(__uint_as_float(ov[d8 * 8 + 4]) * prev_inv, __uint_as_float(ov[d8 * 8 + 5]) * prev_inv);
              w4.w = pack_bf16(__uint_as_float(ov[d8 * 8 + 6]) * prev_inv, __uint_as_float(ov[d8 * 8 + 7]) * prev_inv);
              *reinterpret_cast<uint4*>(prev_orow + h * 32 + d8 * 8) = w4;
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(TCB_S_EMPTY + prev_r));  // the region may take the next S
        return true;
      };
      for (int item = blockIdx.x; item < total_items; item += stride_items, ++n) {
        const TcItem it = tc_make_item(info, item, nh, half_window);
        if (item + stride_items < total_items) info = __ldg(tile_info + (item + stride_items) / nh);
        const uint32_t r = n & 1;
        const int qi = it.q0 + row;
        const int key_lo = max(0, qi - half_window);
        const int key_hi = qi < it.len ? min(it.len - 1, qi + half_window) : -1;
        if (!mbar_wait(bar(TCB_S_FULL + r), (n >> 1) & 1, status, ST_ATTN_SOFTMAX_TIMEOUT)) break;
        tc_fence_after();
        const int n0 = 4 - warp;                       // chunks taken from tile 0
        const int n1 = it.n_kv > 1 ? warp + 1 : 0;     // chunks taken from tile 1
        const uint32_t region = lane_addr + r * 256;
        uint32_t sv[5][32];
#pragma unroll
        for (int k = 0; k < 5; ++k) {
          if (k < n0 + n1) {
            const int tile = k < n0 ? 0 : 1;
            const int chunk = k < n0 ? warp + k : k - n0;
            tmem_ld_32x32_nowait(region + tile * 128 + chunk * 32, sv[k]);
          }
        }
        tmem_ld_wait();
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains, not one
        // Interior item: all 256 fetched keys and all 128 query rows lie inside the sequence, so
        // the band alone decides.  Then only the warp's first chunk (keys >= row: column e >= lane)
        // and last chunk (keys <= row + 128: column e <= lane) need a per-element test.
        const bool interior = it.kv_start >= 0 && it.kv_start + 2 * TC_BN <= it.len;
        if (interior) {
#pragma unroll
          for (int k = 0; k < 5; ++k) {
            if (k == 0 || k == 4) {
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const bool ok_e = (k == 0) ? (e >= lane) : (e <= lane);
                const float v = ok_e ? __uint_as_float(sv[k][e]) : -INFINITY;
                sv[k][e] = __float_as_uint(v);
                mx4[e & 3] = fmaxf(mx4[e & 3], v);
              }
            } else {
#pragma unroll
              for (int e = 0; e < 32; e += 2)
                mx4[(e >> 1) & 3] = fmax3(mx4[(e >> 1) & 3], __uint_as_float(sv[k][e]), __uint_as_float(sv[k][e + 1]));
            }
          }
        } else {
#pragma unroll
          for (int k = 0; k < 5; ++k) {
            if (k < n0 + n1) {
              const int tile = k < n0 ? 0 : 1;
              const int chunk = k < n0 ? warp + k : k - n0;
              const int key0 = it.kv_start + tile * 128 + chunk * 32;
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const int key = key0 + e;
                const float v = (key >= key_lo && key <= key_hi) ? __uint_as_float(sv[k][e]) : -INFINITY;
                sv[k][e] = __float_as_uint(v);
                mx4[e & 3] = fmaxf(mx4[e & 3], v);
              }
            }
          }
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const float m_safe = (mx == -INFINITY) ? 0.f : mx * scale_log2;
        if (prev_valid && !drain_prev()) break;  // also guarantees P V of item n - 1 is done with P
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        const uint32_t prow = sP + row * 128;
        const uint32_t sw = row & 7;
#pragma unroll
        for (int k = 0; k < 5; ++k) {
          if (k < n0 + n1) {
            const int tile = k < n0 ? 0 : 1;
            const int chunk = k < n0 ? warp + k : k - n0;
            const uint32_t pbase = prow + tile * TC_P_BYTES + (chunk >> 1) * TC_TILE_BYTES;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float pv[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                pv[e] = ex2(fmaf(__uint_as_float(sv[k][i * 8 + e]), scale_log2, -m_safe));
                sum4[e & 3] += pv[e];
              }
              const uint32_t addr = pbase + (((((chunk & 1) << 2) + i) ^ sw) << 4);
              asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                           "r"(pack_bf16(pv[0], pv[1])), "r"(pack_bf16(pv[2], pv[3])),
                           "r"(pack_bf16(pv[4], pv[5])), "r"(pack_bf16(pv[6], pv[7]))
                           : "memory");
            }
          }
        }
        // zero the chunks this warp's rows cannot see: tile 0 chunks 0..w-1, tile 1 chunks w+1..3
        for (int tile = 0; tile < it.n_kv; ++tile) {
          const int c_begin = tile == 0 ? 0 : warp + 1;
          const int c_end = tile == 0 ? warp : 4;
          for (int chunk = c_begin; chunk < c_end; ++chunk) {
            const uint32_t pbase = prow + tile * TC_P_BYTES + (chunk >> 1) * TC_TILE_BYTES;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint32_t addr = pbase + (((((chunk & 1) << 2) + i) ^ sw) << 4);
              asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
            }
          }
        }
        const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(TCB_P_FULL));

        prev_valid = true;
        prev_r = r;
        prev_phase = (n >> 1) & 1;
        prev_inv = sum > 0.f ? 1.f / sum : 0.f;
        prev_orow = qi < it.len ? out + (int64_t(it.seq_begin) + qi) * H + it.head * 64 : nullptr;
      }
      if (prev_valid) drain_prev();
    } else {
      // Full attention (and any band other than 64): online softmax over the key tiles.  Eight
      // softmax warps: warps w and w + 4 own the same 32 query rows (same tensor-memory lanes) and
      // split each row between them - warpgroup `hf` takes score columns [64 hf, 64 hf + 64) of
      // every tile, writes that half of P, and keeps output dims [32 hf, 32 hf + 32).  Two warps
      // per scheduler hide each other's exp2 / tensor-memory / dependency latencies and each
      // thread's instruction stream is half as long.  The two halves of a row swap their tile
      // maxima through shared memory (the tile's K buffer is dead once S is complete) and meet at
      // a 64-thread named barrier; their partial row sums are combined once per item.
      // After a bounded wait has given up, `ok` is false: waits are skipped but the loops and
      // the named barriers still run to the end, so no warp is left alone at a barrier.
      const uint32_t hf = warp >> 2;
      const uint32_t pair_bar = 1 + wq;  // named barrier of warps wq and wq + 4
      const uint32_t lbox = bar_base + 256;  // float[2][128]: per-item exchange of partial row sums
      auto wait = [&](uint32_t barrier, uint32_t parity) {
        if (ok && !mbar_wait(barrier, parity, status, ST_ATTN_SOFTMAX_TIMEOUT)) ok = false;
      };
      int4 info = __ldg(tile_info + blockIdx.x / nh);
      uint32_t g = 0;  // key tiles consumed so far
      for (int item = blockIdx.x; item < total_items; item += stride_items) {
        const TcItem it = tc_make_item(info, item, nh, half_window);
        if (item + stride_items < total_items)  // next item's descriptor, in flight during this one
          info = __ldg(tile_info + (item + stride_items) / nh);
        const int qi = it.q0 + row;  // position in the sequence
        float acc[32];
#pragma unroll
        for (int d = 0; d < 32; ++d) acc[d] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;
        int key_lo = 0, key_hi = it.len - 1;  // valid keys of this row (empty for rows past the end)
        if (half_window >= 0) {
          key_lo = max(0, qi - half_window);
          key_hi = min(it.len - 1, qi + half_window);
        }
        if (qi >= it.len) key_hi = -1;

        for (int j = 0; j < it.n_kv; ++j, ++g) {
          const uint32_t b = g & 1;
          wait(bar(TCB_S_FULL + b), (g >> 1) & 1);
          tc_fence_after();
          uint32_t sv[64];
          const uint32_t s_addr = lane_addr + TC_S_COL + b * 128 + hf * 64;
          tmem_ld_32x32_nowait(s_addr, sv);
          tmem_ld_32x32_nowait(s_addr + 32, sv + 32);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(TCB_S_EMPTY + b));

          const int col0 = it.kv_start + j * TC_BN + int(hf) * 64;       // key of this thread's column 0
          const int c_lo = key_lo - col0, c_hi = key_hi - col0;          // valid columns [c_lo, c_hi]
          const bool full = (c_lo <= 0) && (c_hi >= 63);
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains, not one
          if (full) {
#pragma unroll
            for (int c = 0; c < 64; c += 2)
              mx4[(c >> 1) & 3] = fmax3(mx4[(c >> 1) & 3], __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]));
          } else {
#pragma unroll
            for (int c = 0; c < 64; ++c) {
              const float v = (c >= c_lo && c <= c_hi) ? __uint_as_float(sv[c]) : -INFINITY;
              sv[c] = __float_as_uint(v);
              mx4[c & 3] = fmaxf(mx4[c & 3], v);
            }
          }
          float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
          // swap the half-row maxima: mailbox = first KB of this tile's (dead) K buffer
          const uint32_t mbox = sKV + (g % TC_STAGES) * 2 * TC_TILE_BYTES;
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(mbox + (hf * 128 + row) * 4), "f"(mx) : "memory");
          asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
          float other;
          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(other) : "r"(mbox + ((hf ^ 1) * 128 + row) * 4) : "memory");
          mx = fmaxf(mx, other);
          const float m_new = fmaxf(m_run, mx * scale_log2);
          const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
          const float alpha = ex2(m_run - m_safe);
          float sum4[4] = {0.f, 0.f, 0.f, 0.f};
          const uint32_t prow = sP + b * TC_P_BYTES + hf * TC_TILE_BYTES + row * 128;
#pragma unroll
          for (int c8 = 0; c8 < 8; ++c8) {  // 8 chunks of 8 keys = 16 bytes of bf16
            float p[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              p[e] = ex2(fmaf(__uint_as_float(sv[c8 * 8 + e]), scale_log2, -m_safe));
              sum4[e & 3] += p[e];
            }
            const uint32_t addr = prow + ((c8 ^ (row & 7)) << 4);
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr),
                         "r"(pack_bf16(p[0], p[1])), "r"(pack_bf16(p[2], p[3])),
                         "r"(pack_bf16(p[4], p[5])), "r"(pack_bf16(p[6], p[7]))
                         : "memory");
          }
          fence_proxy_async_smem();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(TCB_P_FULL + b));

          if (j > 0) {  // fold in the previous tile's P V, then move to the new running maximum
            const uint32_t pb = b ^ 1;
            wait(bar(TCB_O_FULL + pb), ((g - 1) >> 1) & 1);
            tc_fence_after();
            uint32_t ov[32];
            tmem_ld_32x32_nowait(lane_addr + TC_O_COL + pb * 64 + hf * 32, ov);
            tmem_ld_wait();
            if (__all_sync(0xffffffffu, alpha == 1.0f)) {  // common once the row maxima have settled
#pragma unroll
              for (int d = 0; d < 32; ++d) acc[d] += __uint_as_float(ov[d]);
            } else {
#pragma unroll
              for (int d = 0; d < 32; ++d) acc[d] = (acc[d] + __uint_as_float(ov[d])) * alpha;
            }
          }
          l_run = l_run * alpha + ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
          m_run = m_new;
        }
        {  // last tile's P V, the other half's row sum, normalise, store this half of the row
          const uint32_t pb = (g - 1) & 1;
          wait(bar(TCB_O_FULL + pb), ((g - 1) >> 1) & 1);
          tc_fence_after();
          uint32_t ov[32];
          tmem_ld_32x32_nowait(lane_addr + TC_O_COL + pb * 64 + hf * 32, ov);
          tmem_ld_wait();
          tc_fence_before();
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(lbox + (hf * 128 + row) * 4), "f"(l_run) : "memory");
          asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
          float l_other;
          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(l_other) : "r"(lbox + ((hf ^ 1) * 128 + row) * 4) : "memory");
          const float l_all = l_run + l_other;  // both halves use the same running maximum
          if (ok && qi < it.len) {
            const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
            __nv_bfloat16* orow = out + (int64_t(it.seq_begin) + qi) * H + it.head * 64 + hf * 32;
#pragma unroll
            for (int d8 = 0; d8 < 4; ++d8) {
              float o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] = (acc[d8 * 8 + e] + __uint_as_float(ov[d8 * 8 + e])) * inv;
              uint4 w;
              w.x = pack_bf16(o[0], o[1]);
              w.y = pack_bf16(o[2], o[3]);
              w.z = pack_bf16(o[4], o[5]);
              w.w = pack_bf16(o[6], o[7]);
              *reinterpret_cast<uint4*>(orow + d8 * 8) = w;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == NSW + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TC_TMEM_COLS);
  }
}

int attn_run_tc(const void* qkv, const int4* tile_info, const int32_t* total_tiles, int64_t max_tiles,
                int64_t T, int nh, int half_window, void* out, int32_t* status, cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set) {
    PE_CUDA(cudaFuncSetAttribute(attn_varlen_tc_kernel<false>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM));
    PE_CUDA(cudaFuncSetAttribute(attn_varlen_tc_kernel<true>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM));
    attr_set = true;
  }
  CUtensorMap tm;
  int rc = make_tmap_bf16_2d(&tm, qkv, (uint64_t)T, (uint64_t)(3 * nh * 64), (uint64_t)(3 * nh * 64),
                             128);
  if (rc != PE_OK) return rc;
  const int64_t max_items = max_tiles * nh;
  const int grid = (int)(max_items < sm_count() ? max_items : sm_count());
  if (half_window == TC_BN / 2 && get_option(OPT_LOCAL_ATTN_TWO_CTA))
    return attn_run_local_tc2(qkv, tile_info, total_tiles, max_tiles, T, nh, out, status, st);
  // The single-pass kernel relies on the band being exactly one key tile wide.
  if (half_window == TC_BN / 2 && get_option(OPT_LOCAL_ATTN_SINGLE_PASS))
    attn_varlen_tc_kernel<true><<<grid, TC_THREADS, TC_SMEM, st>>>(
        tm, tile_info, total_tiles, nh, half_window, static_cast<__nv_bfloat16*>(out), status);
  else if (get_option(OPT_ATTN_TWO_CTA))
    return attn_run_global_tc(qkv, tile_info, total_tiles, max_tiles, T, nh, half_window, out, status, st);
  else
    attn_varlen_tc_kernel<false><<<grid, TC_THREADS_ONLINE, TC_SMEM, st>>>(
        tm, tile_info, total_tiles, nh, half_window, static_cast<__nv_bfloat16*>(out), status);
  PE_LAUNCH_CHECK("attn_varlen_tc_kernel");
  return PE_OK;
}

}  // namespace pe
