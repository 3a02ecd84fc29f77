// bf16 "TN" GEMM for the four ModernBERT projections, C[M, N] = A[M, K] * W[N, K]^T,
// written for sm_100a: TMA-fed shared-memory pipeline, tcgen05.mma with the
// fp32 accumulator in tensor memory, persistent CTAs.
//
// Two forms of one kernel template.
// PAIR (the default for all but tiny M): the two CTAs of a cluster of 2 share output tiles of
// 256 rows x 256 accumulator columns (tcgen05 cta_group::2).  Each CTA stages its own 128 rows of
// A and its own 128 rows of W per k block (32 KB instead of 48 KB per 128 x 256 x 64 block of
// work), owns 128 lanes x 256 columns of the accumulator in its tensor memory and runs the
// epilogue for its own 128 rows; one thread of the even CTA issues the MMAs for both.  Every CTA
// fetches its own operands with plain per-CTA TMA loads; the two CTAs meet only in mbarriers.
// Single CTA (M <= 256, or pe_set_option(PE_OPT_GEMM_PAIR, 0)): one CTA per SM, 128 x 256 tiles.
//   warp 0      : TMA producer (one elected lane)
//   warp 1      : allocates tensor memory, issues tcgen05.mma (one elected lane; in a pair only
//                 the even CTA's)
//   warps 2..5  : epilogue - tcgen05.ld the accumulator, round to bf16, transform, store
//                 (GEGLU mode: warps 2..9, two per tensor-memory lane quarter, each taking one
//                 64-column half of the tile's output; with four warps that epilogue, a GELU per
//                 element, ran about as long as a 768-deep main loop and lost 4 % on pairs)
// Tensor memory holds two 256-column accumulators, so the epilogue of tile i
// overlaps the main loop of tile i+1.  The k loop runs over 64-wide blocks through
// a ring of stage buffers guarded by full/empty mbarriers.
//
// GEGLU mode computes the first half of the MLP in one pass: the 256 accumulator
// columns of a tile are 128 columns of the gelu input (rows n0.. of Wi) and the
// matching 128 gate columns (rows I + n0.. of Wi; in a pair, the odd CTA's half of B); the
// epilogue rounds both to bf16, as the unfused path materialises them, and writes gelu(a) * gate.
//
// RESIDUAL mode never reads X: it is the plain epilogue with TMA reduce-adds in place of TMA
// stores, so the memory system adds the rounded product to what C holds (C is X; out of place the
// host copies X to C first).
//
// Every mbarrier wait is bounded; a wait that gives up records a code in the
// status word and the CTA unwinds through the common exit, which frees its
// tensor memory.
#include <algorithm>
#include <atomic>

#include "pe_host.h"
#include "pe_ptx.cuh"

namespace pe {

constexpr int BM = 128;   // rows per CTA
constexpr int BN = 256;   // accumulator columns per tile
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int OUT_STAGE_BYTES = 32 * 128;  // one warp's 32 rows x 64 bf16 columns
constexpr uint32_t TMEM_COLS = 512;

// GEMM_RESIDUAL: the plain epilogue, its TMA stores replaced by TMA reduce-adds (C += bf16(A W^T)).
enum GemmMode : int { GEMM_PLAIN = 0, GEMM_GEGLU = 1, GEMM_QKV_ROPE = 2, GEMM_RESIDUAL = 3, GEMM_L2NORM = 4 };

template <int MODE, bool PAIR>
struct GemmCfg {
  static constexpr int B_ROWS = PAIR ? 128 : 256;              // rows of W one CTA stages per k block
  static constexpr int B_BYTES = B_ROWS * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = PAIR ? 6 : 4;
  // WIDE epilogue (GEGLU mode, whose epilogue is the longest: a GELU per output element): eight
  // warps, two per tensor-memory lane quarter, each owning one 64-column half of the tile's
  // output.  A warp pulls its 128 accumulator columns into registers in one go and hands the
  // accumulator back to the MMA thread at once, before it rounds, transforms and stores anything.
  // Measured at 306,851 x 2304 x 768: 0.758 ms against 0.785 ms with the accumulator held through
  // the epilogue (and 0.826 ms before the GELU went to packed fp32 instructions).  The same form
  // was tried for the other modes and was no faster (plain, RoPE) or slower (reduce-add: 0.303
  // against 0.285 ms), so they keep four warps that walk the tile in 64-column chunks and release
  // the accumulator after the last chunk's tensor-memory load.
  static constexpr bool WIDE = MODE == GEMM_GEGLU;
  static constexpr int EPI_WARPS = WIDE ? 8 : 4;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int OUT_BUFS = EPI_WARPS == 8 ? 1 : 2;  // staging buffers per epilogue warp
  static constexpr int OUT_BYTES = EPI_WARPS * OUT_BUFS * OUT_STAGE_BYTES;
  // barrier slots (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then
  // the tensor-memory base address
  static constexpr int BAR_FULL = 0, BAR_EMPTY = STAGES, BAR_TFULL = 2 * STAGES, BAR_TEMPTY = 2 * STAGES + 2,
                       BAR_COUNT = 2 * STAGES + 4;
  static constexpr int SMEM = STAGES * STAGE_BYTES + OUT_BYTES + 1024 /*align*/ + 8 * BAR_COUNT + 16;
};

__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// Extra operands of the Wqkv + RoPE epilogue.
struct RopeArgs {
  const int64_t* pos;            // [M] position of each row
  const __nv_bfloat16* table;    // [max_positions, 64]: cos of the 32 frequencies, then sin
  int rope_cols;                 // columns [0, rope_cols) are q and k heads, the rest is v
  int max_positions;
};

template <int MODE, bool PAIR>
__global__ void __launch_bounds__((GemmCfg<MODE, PAIR>::THREADS), 1)
gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC,
                    int M, int n_out, int K, int gate_row0, int num_m, int num_n, RopeArgs rope,
                    int* status) {
  using Cfg = GemmCfg<MODE, PAIR>;
  constexpr bool GEGLU = MODE == GEMM_GEGLU;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int STAGE_BYTES = Cfg::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t out_base = base + STAGES * STAGE_BYTES;
  const uint32_t bar_base = out_base + Cfg::OUT_BYTES;
  auto bar = [&](int i) { return bar_base + 8u * i; };
  const uint32_t tmem_slot = bar_base + 8u * Cfg::BAR_COUNT;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (K + BK - 1) / BK;
  const int num_tiles = num_m * num_n;
  // In a pair both CTAs walk the same tiles; the odd CTA owns rows 128..255 of each.
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;
  const int first_tile = PAIR ? int(blockIdx.x >> 1) : int(blockIdx.x);
  const int tile_stride = PAIR ? int(gridDim.x >> 1) : int(gridDim.x);
  constexpr int TILE_ROWS = PAIR ? 2 * BM : BM;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(bar(Cfg::BAR_FULL + i), 1);
      mbar_init(bar(Cfg::BAR_EMPTY + i), 1);
    }
    mbar_init(bar(Cfg::BAR_TFULL), 1);
    mbar_init(bar(Cfg::BAR_TFULL + 1), 1);
    mbar_init(bar(Cfg::BAR_TEMPTY), (PAIR ? 2 : 1) * Cfg::EPI_WARPS);  // one arrival per epilogue warp (of both CTAs)
    mbar_init(bar(Cfg::BAR_TEMPTY + 1), (PAIR ? 2 : 1) * Cfg::EPI_WARPS);
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_slot, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if (PAIR) cluster_sync_all(); else __syncthreads();  // the peer's barriers are initialised too
  tc_fence_after();
  uint32_t tmem_base;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

  if (warp == 0) {
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_stride) {
        const int m0 = (tile / num_n) * TILE_ROWS + int(cta_rank) * BM;
        const int nt = tile % num_n;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar(Cfg::BAR_EMPTY + stage), phase ^ 1u, status, ST_GEMM_PRODUCER_TIMEOUT)) {
            ok = false;
            break;
          }
          const uint32_t sa = base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          if (PAIR) {
            // Both CTAs' bytes are counted on the leader's barrier: its MMA thread waits for the
            // whole 256-row stage.  The odd CTA's half of B: rows 128..255 of the tile's 256 W rows,
            // or the gate rows in GEGLU mode.
            const uint32_t full = cta_rank == 0 ? bar(Cfg::BAR_FULL + stage)
                                                : cluster_map(bar(Cfg::BAR_FULL + stage), 0);
            const int brow = GEGLU ? (cta_rank == 0 ? nt * 128 : gate_row0 + nt * 128)
                                   : nt * BN + int(cta_rank) * 128;
            if (cta_rank == 0) mbar_expect_tx(full, 2 * STAGE_BYTES);
            tma_load_2d_pair(sa, &tmA, full, kb * BK, m0);
            tma_load_2d_pair(sb, &tmB, full, kb * BK, brow);
          } else {
            const int brow0 = GEGLU ? nt * 128 : nt * BN;
            const int brow1 = GEGLU ? gate_row0 + nt * 128 : nt * BN + 128;
            mbar_expect_tx(bar(Cfg::BAR_FULL + stage), STAGE_BYTES);
            tma_load_2d(sa, &tmA, bar(Cfg::BAR_FULL + stage), kb * BK, m0);
            tma_load_2d(sb, &tmB, bar(Cfg::BAR_FULL + stage), kb * BK, brow0);
            tma_load_2d(sb + Cfg::B_BYTES / 2, &tmB, bar(Cfg::BAR_FULL + stage), kb * BK, brow1);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (cta_rank == 0 && elect_one()) {
      constexpr uint32_t idesc = umma_idesc_bf16(TILE_ROWS, BN, 0);
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_stride) {
        if (!mbar_wait(bar(Cfg::BAR_TEMPTY + acc), acc_phase ^ 1u, status, ST_GEMM_MMA_TIMEOUT)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar(Cfg::BAR_FULL + stage), phase, status, ST_GEMM_MMA_TIMEOUT)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = base + stage * STAGE_BYTES;
          const uint64_t adesc = umma_smem_desc_sw128(sa, 1024);
          const uint64_t bdesc = umma_smem_desc_sw128(sa + A_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            // 16 bf16 along K = 32 bytes = 2 descriptor address units inside the swizzle atom
            if (PAIR) umma_ss_pair(d_tmem, adesc + 2u * kk, bdesc + 2u * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
            else umma_ss(d_tmem, adesc + 2u * kk, bdesc + 2u * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          if (PAIR) umma_commit_pair(bar(Cfg::BAR_EMPTY + stage));  // frees the stage in both CTAs
          else umma_commit(bar(Cfg::BAR_EMPTY + stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (PAIR) umma_commit_pair(bar(Cfg::BAR_TFULL + acc));
        else umma_commit(bar(Cfg::BAR_TFULL + acc));
        acc ^= 1u;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else {
    // Epilogue: 64 accumulator columns at a time - tcgen05.ld, round (and transform) in
    // registers, write the warp's 32 x 64 block into its own 128-byte-swizzled staging buffer,
    // and let TMA store it.  Row-per-thread global stores would cost one cache line per lane
    // per instruction; the TMA store keeps the load/store unit out of the way and clips rows
    // and columns that fall outside C.
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    const uint32_t stage0 = out_base + (warp - 2) * Cfg::OUT_BUFS * OUT_STAGE_BYTES;
    uint32_t ob = 0;  // staging buffer in use
    auto emit64 = [&](const uint32_t (&lo)[32], const uint32_t (&hi)[32], int col, int row0) {
      if (lane == 0) tma_store_wait_read<Cfg::OUT_BUFS - 1>();  // the buffer about to be written is free again
      __syncwarp();
      const uint32_t dst = stage0 + ob * OUT_STAGE_BYTES + lane * 128;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst + ((j ^ (lane & 7)) << 4)),
                     "r"(pack_bf16(__uint_as_float(lo[j * 8 + 0]), __uint_as_float(lo[j * 8 + 1]))),
                     "r"(pack_bf16(__uint_as_float(lo[j * 8 + 2]), __uint_as_float(lo[j * 8 + 3]))),
                     "r"(pack_bf16(__uint_as_float(lo[j * 8 + 4]), __uint_as_float(lo[j * 8 + 5]))),
                     "r"(pack_bf16(__uint_as_float(lo[j * 8 + 6]), __uint_as_float(lo[j * 8 + 7])))
                     : "memory");
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst + (((4 + j) ^ (lane & 7)) << 4)),
                     "r"(pack_bf16(__uint_as_float(hi[j * 8 + 0]), __uint_as_float(hi[j * 8 + 1]))),
                     "r"(pack_bf16(__uint_as_float(hi[j * 8 + 2]), __uint_as_float(hi[j * 8 + 3]))),
                     "r"(pack_bf16(__uint_as_float(hi[j * 8 + 4]), __uint_as_float(hi[j * 8 + 5]))),
                     "r"(pack_bf16(__uint_as_float(hi[j * 8 + 6]), __uint_as_float(hi[j * 8 + 7])))
                     : "memory");
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        if constexpr (MODE == GEMM_RESIDUAL) tma_reduce_add_2d(&tmC, stage0 + ob * OUT_STAGE_BYTES, col, row0);
        else tma_store_2d(&tmC, stage0 + ob * OUT_STAGE_BYTES, col, row0);
        tma_store_commit();
      }
      ob = (ob + 1u) % Cfg::OUT_BUFS;
    };
    uint32_t acc = 0, acc_phase = 0;
    for (int tile = first_tile; tile < num_tiles; tile += tile_stride) {
      const int m0 = (tile / num_n) * TILE_ROWS + int(cta_rank) * BM;
      const int nt = tile % num_n;
      if (!mbar_wait(bar(Cfg::BAR_TFULL + acc), acc_phase, status, ST_GEMM_EPILOGUE_TIMEOUT)) break;
      tc_fence_after();
      const int row0 = m0 + q * 32;
      const int row = row0 + lane;
      const uint32_t t_addr = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      // Hands the accumulator back to the MMA thread: as soon as a warp has read all it needs of it.
      auto release_acc = [&]() {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {  // the accumulator is free again: tell the (leader's) MMA thread
          if (cta_rank == 0) mbar_arrive(bar(Cfg::BAR_TEMPTY + acc));
          else mbar_arrive_cluster(cluster_map(bar(Cfg::BAR_TEMPTY + acc), 0));
        }
      };
      const int half = (warp - 2) >> 2;  // WIDE (GEGLU) mode: which 64 output columns this warp owns
      if constexpr (MODE == GEMM_QKV_ROPE) {
        // One 64-column head at a time: rotate the (j, j + 32) pairs of q and k heads by the
        // row's position, on values rounded to bf16 first (as the unfused path stores them).
        const int col0 = nt * BN;
        // cos[0..31] and sin[0..31] of this row's position, widened to fp32 once per tile (its four
        // heads share them).  The epilogue's instruction count shows in this kernel's time
        // (skipping the rotation saves 0.06 of 0.85 ms at 306,851 rows), so the rotation below
        // works on two pairs at a time with the packed fp32 instructions of sm_100.
        float2 cf[16], sf[16];
        if (col0 < rope.rope_cols) {
          int64_t p = row < M ? rope.pos[row] : 0;
          if (p < 0 || p >= rope.max_positions) {
            set_status(status, ST_BAD_POSITION);
            p = 0;
          }
          const uint4* trow = reinterpret_cast<const uint4*>(rope.table + p * 64);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 cw = __ldg(trow + i), sw = __ldg(trow + 4 + i);
            const uint32_t c4[4] = {cw.x, cw.y, cw.z, cw.w}, s4[4] = {sw.x, sw.y, sw.z, sw.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {  // a 32-bit word holds the values of pairs 8i + 2e and 8i + 2e + 1
              cf[i * 4 + e] = make_float2(__uint_as_float(c4[e] << 16), __uint_as_float(c4[e] & 0xffff0000u));
              sf[i * 4 + e] = make_float2(__uint_as_float(s4[e] << 16), __uint_as_float(s4[e] & 0xffff0000u));
            }
          }
        }
#pragma unroll 1
        for (int hp = 0; hp < BN / 64; ++hp) {
          const int col = col0 + hp * 64;
          if (col >= n_out) break;
          uint32_t lo[32], hi[32];
          tmem_ld_32x32(t_addr + hp * 64, lo);
          tmem_ld_32x32(t_addr + hp * 64 + 32, hi);
          tmem_ld_wait();
          if (hp == BN / 64 - 1 || col + 64 >= n_out) release_acc();  // the whole accumulator has been read
          if (col < rope.rope_cols) {
            // Pairs (i, i + 1) of (dim j, dim j + 32): both values rounded to bf16 first (as the
            // unfused path stores the projection), then exactly rope_pair()'s arithmetic:
            // lo' = fma(lo, c, -(hi * s)), hi' = fma(hi, c, lo * s), each product and sum rounded once.
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const uint32_t lw = pack_bf16(__uint_as_float(lo[i]), __uint_as_float(lo[i + 1]));
              const uint32_t hw = pack_bf16(__uint_as_float(hi[i]), __uint_as_float(hi[i + 1]));
              const float2 l2 = make_float2(__uint_as_float(lw << 16), __uint_as_float(lw & 0xffff0000u));
              const float2 h2 = make_float2(__uint_as_float(hw << 16), __uint_as_float(hw & 0xffff0000u));
              const float2 c2 = cf[i >> 1], s2 = sf[i >> 1];
              const float2 ns2 = make_float2(-s2.x, -s2.y);
              const float2 ol = __ffma2_rn(l2, c2, __fmul2_rn(h2, ns2));
              const float2 oh = __ffma2_rn(h2, c2, __fmul2_rn(l2, s2));
              lo[i] = __float_as_uint(ol.x);
              lo[i + 1] = __float_as_uint(ol.y);
              hi[i] = __float_as_uint(oh.x);
              hi[i + 1] = __float_as_uint(oh.y);
            }
          }
          emit64(lo, hi, col, row0);
        }
      } else if constexpr (MODE == GEMM_L2NORM) {
        // Projection head: at most 256 output columns, so the tile holds whole rows and each
        // thread can L2-normalise its own.  Two passes over the accumulator: the norm of the
        // bf16-rounded row (rounded to bf16 itself, as a bf16 F.normalize produces it), then
        // row / norm.
        float ss = 0.f;
        for (int c = 0; c * 64 < n_out; ++c) {
          uint32_t lo[32], hi[32];
          tmem_ld_32x32(t_addr + c * 64, lo);
          tmem_ld_32x32(t_addr + c * 64 + 32, hi);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float a = round_bf16(__uint_as_float(lo[i])), b = round_bf16(__uint_as_float(hi[i]));
            ss = fmaf(a, a, ss);
            ss = fmaf(b, b, ss);
          }
        }
        const float norm = fmaxf(round_bf16(sqrtf(ss)), 1e-12f);
        for (int c = 0; c * 64 < n_out; ++c) {
          uint32_t lo[32], hi[32];
          tmem_ld_32x32(t_addr + c * 64, lo);
          tmem_ld_32x32(t_addr + c * 64 + 32, hi);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            lo[i] = __float_as_uint(round_bf16(__uint_as_float(lo[i])) / norm);
            hi[i] = __float_as_uint(round_bf16(__uint_as_float(hi[i])) / norm);
          }
          emit64(lo, hi, c * 64, row0);
        }
      } else if constexpr (!GEGLU) {
        const int col0 = nt * BN;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          const int col = col0 + c * 64;
          if (col >= n_out) break;
          uint32_t lo[32], hi[32];
          tmem_ld_32x32(t_addr + c * 64, lo);
          tmem_ld_32x32(t_addr + c * 64 + 32, hi);
          tmem_ld_wait();
          if (c == BN / 64 - 1 || col + 64 >= n_out) release_acc();  // the whole accumulator has been read
          emit64(lo, hi, col, row0);
        }
      } else {
        // this warp's 64 output columns: gelu input columns [64 half, 64 half + 64) and the gate
        // columns 128 further on
        const int col = nt * 128 + half * 64;
        uint32_t va[2][32], vg[2][32];
        tmem_ld_32x32(t_addr + half * 64, va[0]);
        tmem_ld_32x32(t_addr + half * 64 + 32, va[1]);
        tmem_ld_32x32(t_addr + 128 + half * 64, vg[0]);
        tmem_ld_32x32(t_addr + 128 + half * 64 + 32, vg[1]);
        tmem_ld_wait();
        release_acc();
        if (col < n_out) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int e = 0; e < 32; e += 2) {  // two elements at a time: packed roundings and packed GELU
              const uint32_t aw = pack_bf16(__uint_as_float(va[h][e]), __uint_as_float(va[h][e + 1]));
              const uint32_t gw = pack_bf16(__uint_as_float(vg[h][e]), __uint_as_float(vg[h][e + 1]));
              const float2 a2 = make_float2(__uint_as_float(aw << 16), __uint_as_float(aw & 0xffff0000u));
              const float2 g2 = make_float2(__uint_as_float(gw << 16), __uint_as_float(gw & 0xffff0000u));
              const float2 o2 = __fmul2_rn(gelu_erf2(a2), g2);
              va[h][e] = __float_as_uint(o2.x);
              va[h][e + 1] = __float_as_uint(o2.y);
            }
          }
          emit64(va[0], va[1], col, row0);
        }
      }
      if constexpr (MODE == GEMM_L2NORM) release_acc();
      acc ^= 1u;
      if (acc == 0) acc_phase ^= 1u;
    }
    if (lane == 0) tma_store_wait_all<0>();  // staging memory must outlive the stores that read it
    __syncwarp();
  }

  // Common exit: every role arrives here (each of its waits is bounded).  In a pair both CTAs
  // must be done before either frees tensor memory that the leader's MMAs write.
  tc_fence_before();
  if (PAIR) cluster_sync_all(); else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

static std::atomic<int> g_gemm_pair{1};
void set_gemm_pair(int on) { g_gemm_pair.store(on, std::memory_order_relaxed); }

template <int MODE, bool PAIR>
static int launch_gemm_as(const void* A, const void* W, void* C, int64_t M, int n_out, int K,
                          int w_rows, int gate_row0, RopeArgs rope, int32_t* status,
                          cudaStream_t stream) {
  using Cfg = GemmCfg<MODE, PAIR>;
  constexpr bool GEGLU = MODE == GEMM_GEGLU;
  auto kern = gemm_bf16_tn_kernel<MODE, PAIR>;
  int rc = set_max_dynamic_smem(reinterpret_cast<const void*>(kern), Cfg::SMEM, false);
  if (rc != PE_OK) return rc;
  CUtensorMap tmA, tmB;
  rc = make_tmap_bf16_2d(&tmA, A, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM);
  if (rc != PE_OK) return rc;
  rc = make_tmap_bf16_2d(&tmB, W, (uint64_t)w_rows, (uint64_t)K, (uint64_t)K, 128);
  if (rc != PE_OK) return rc;
  CUtensorMap tmC;  // output, stored in 32-row x 64-column boxes
  rc = make_tmap_bf16_2d(&tmC, C, (uint64_t)M, (uint64_t)n_out, (uint64_t)n_out, 32);
  if (rc != PE_OK) return rc;
  const int tile_rows = PAIR ? 2 * BM : BM;
  const int num_m = int((M + tile_rows - 1) / tile_rows);
  const int cols_per_tile = GEGLU ? 128 : BN;
  const int num_n = (n_out + cols_per_tile - 1) / cols_per_tile;
  const long long tiles = (long long)num_m * num_n;
  if (PAIR) {
    const long long pairs = std::min<long long>(tiles, sm_count() / 2);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * pairs));
    cfg.blockDim = dim3(Cfg::THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PE_CUDA(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, (int)M, n_out, K, gate_row0, num_m, num_n,
                               rope, (int*)status));
  } else {
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    kern<<<grid, Cfg::THREADS, Cfg::SMEM, stream>>>(tmA, tmB, tmC, (int)M, n_out, K, gate_row0,
                                                    num_m, num_n, rope, status);
  }
  PE_LAUNCH_CHECK("gemm_bf16_tn_kernel");
  return PE_OK;
}

template <int MODE>
static int launch_gemm(const void* A, const void* W, void* C, int64_t M, int n_out, int K,
                       int w_rows, int gate_row0, RopeArgs rope, int32_t* status,
                       cudaStream_t stream) {
  // A pair needs more than one CTA's worth of rows to be worth its second CTA.
  if (M > 2 * BM && g_gemm_pair.load(std::memory_order_relaxed) != 0)
    return launch_gemm_as<MODE, true>(A, W, C, M, n_out, K, w_rows, gate_row0, rope, status, stream);
  return launch_gemm_as<MODE, false>(A, W, C, M, n_out, K, w_rows, gate_row0, rope, status, stream);
}

static int check_gemm_args(const void* A, const void* W, const void* C, int64_t M, int n, int K,
                           const char* who) {
  PE_REQUIRE(A && W && C, "%s: null pointer", who);
  PE_REQUIRE(M >= 0 && M < (1ll << 31) - 256, "%s: M=%lld out of range", who, (long long)M);
  PE_REQUIRE(n > 0 && n % 8 == 0, "%s: output columns %d must be a positive multiple of 8", who, n);
  PE_REQUIRE(K > 0 && K % 8 == 0, "%s: K=%d must be a positive multiple of 8", who, K);
  PE_REQUIRE(((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0 && ((uintptr_t)C & 15) == 0,
             "%s: pointers must be 16-byte aligned", who);
  return PE_OK;
}

}  // namespace pe

extern "C" int pe_gemm_bf16_tn(const void* A, const void* W, void* C, int64_t M, int Nout, int K,
                               int32_t* status, void* stream) {
  if (M == 0) return PE_OK;
  int rc = pe::check_gemm_args(A, W, C, M, Nout, K, "pe_gemm_bf16_tn");
  if (rc != PE_OK) return rc;
  return pe::launch_gemm<pe::GEMM_PLAIN>(A, W, C, M, Nout, K, Nout, 0, pe::RopeArgs{}, status,
                                         static_cast<cudaStream_t>(stream));
}

extern "C" int pe_gemm_qkv_rope_bf16(const void* A, const void* Wqkv, void* qkv, int64_t M, int nh,
                                     int K, const int64_t* position_ids, const void* table,
                                     int max_positions, int32_t* status, void* stream) {
  if (M == 0) return PE_OK;
  PE_REQUIRE(nh > 0 && position_ids && table && max_positions > 0,
             "pe_gemm_qkv_rope_bf16: bad RoPE arguments");
  const int n_out = 3 * nh * 64;
  int rc = pe::check_gemm_args(A, Wqkv, qkv, M, n_out, K, "pe_gemm_qkv_rope_bf16");
  if (rc != PE_OK) return rc;
  pe::RopeArgs rope{position_ids, static_cast<const __nv_bfloat16*>(table), 2 * nh * 64, max_positions};
  return pe::launch_gemm<pe::GEMM_QKV_ROPE>(A, Wqkv, qkv, M, n_out, K, n_out, 0, rope, status,
                                            static_cast<cudaStream_t>(stream));
}

extern "C" int pe_gemm_geglu_bf16(const void* A, const void* Wi, void* out, int64_t M, int I, int K,
                                  int32_t* status, void* stream) {
  if (M == 0) return PE_OK;
  int rc = pe::check_gemm_args(A, Wi, out, M, I, K, "pe_gemm_geglu_bf16");
  if (rc != PE_OK) return rc;
  return pe::launch_gemm<pe::GEMM_GEGLU>(A, Wi, out, M, I, K, 2 * I, I, pe::RopeArgs{}, status,
                                         static_cast<cudaStream_t>(stream));
}

extern "C" int pe_gemm_residual_bf16(const void* A, const void* W, const void* X, void* C, int64_t M,
                                     int Nout, int K, int32_t* status, void* stream) {
  if (M == 0) return PE_OK;
  int rc = pe::check_gemm_args(A, W, C, M, Nout, K, "pe_gemm_residual_bf16");
  if (rc != PE_OK) return rc;
  PE_REQUIRE(X != nullptr && ((uintptr_t)X & 15) == 0, "pe_gemm_residual_bf16: X is NULL or unaligned");
  // Nothing has to read X: the rounded product is ADDED to what C holds by TMA reduce-adds, one
  // bf16 add with one rounding per element, exactly the sum above.  Out of place, C first
  // receives a copy of X on the same stream.
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (X != C)
    PE_CUDA(cudaMemcpyAsync(C, X, size_t(M) * size_t(Nout) * 2, cudaMemcpyDeviceToDevice, st));
  return pe::launch_gemm<pe::GEMM_RESIDUAL>(A, W, C, M, Nout, K, Nout, 0, pe::RopeArgs{}, status, st);
}

extern "C" int pe_gemm_l2norm_bf16(const void* A, const void* W, void* C, int64_t M, int Nout, int K,
                                   int32_t* status, void* stream) {
  if (M == 0) return PE_OK;
  int rc = pe::check_gemm_args(A, W, C, M, Nout, K, "pe_gemm_l2norm_bf16");
  if (rc != PE_OK) return rc;
  PE_REQUIRE(Nout <= pe::BN, "pe_gemm_l2norm_bf16: at most %d output columns (one tile holds whole rows), got %d",
             pe::BN, Nout);
  return pe::launch_gemm<pe::GEMM_L2NORM>(A, W, C, M, Nout, K, Nout, 0, pe::RopeArgs{}, status,
                                          static_cast<cudaStream_t>(stream));
}
