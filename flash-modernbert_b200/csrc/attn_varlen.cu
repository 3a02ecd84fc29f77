// Varlen (cu_seqlens-confined) non-causal self-attention for head dim 64 on the
// fused, already-rotated qkv [T, 3*nh*64]: full attention for global layers and a
// |i-j| <= half_window band for local layers, one kernel family.
//
// A small scheduling kernel turns cu_seqlens into a table of query tiles
// (prefix sum of ceil(len / BM)), so the attention grid depends only on the token
// and sequence capacities and can be captured in a CUDA graph while the real
// boundaries stay in device memory.
//
// This file holds the register-tiled kernel for batches whose longest sequence is at most 64
// tokens (one key tile): NWARPS warps per CTA, 16 query rows per warp, mma.sync m16n8k16, online
// softmax in fp32 in the exp2 domain, P rounded to bf16 for the P*V product.  NWARPS is chosen
// from max_seqlen, which gives the short-query tiles that ~30-token sequences want (one 32-row
// CTA covers a whole sequence).  A CTA serves its query tile for four heads; the next head's
// Q / K / V tiles arrive by cp.async while the current one is computed.  Longer batches take the
// tensor-memory kernels (attn_global_tcgen05.cu, attn_local_tcgen05.cu).
#include <algorithm>
#include <mutex>

#include "pe_host.h"
#include "pe_ptx.cuh"

namespace pe {

constexpr int ATT_BN = 64;  // keys per tile
constexpr int ATT_D = 64;

// One pass over cu_seqlens builds the query-tile tables every attention launch of a forward reads.
// Sequences longer than `short_max` go to the main table in tiles of `bm` rows:
//   tile_start[n] = number of such tiles of sequences 0..n-1, tile_start[n_seqs] = their total,
//   tile_info[t]  = {first token of the sequence, sequence length, first query row of the tile, sequence}.
// Sequences of at most `short_max` tokens (short_max = 0: none) get one entry each in a second
// table, short_info, counted by short_start[] in the same way: in a window that mixes ~30-token
// queries with documents they are served by the register-tiled kernel below instead of paying for a
// 128-row tensor-memory tile per query and head.
// The boundaries are never trusted: a begin or end outside [0, T] or an end before its begin is
// clamped into range and reported as ST_BAD_CU_SEQLENS, and no more than `cap_long` main tiles are
// written, so that neither this kernel nor the ones that follow the descriptors can leave the
// caller's buffers.
__global__ void attn_schedule_kernel(const int32_t* __restrict__ cu_seqlens, int n_seqs, int T, int bm,
                                     int short_max, int cap_long, int32_t* __restrict__ tile_start,
                                     int32_t* __restrict__ short_start, int4* __restrict__ tile_info,
                                     int4* __restrict__ short_info, int* status) {
  __shared__ unsigned long long warp_sums[32];
  __shared__ unsigned long long carry_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    carry_s = 0ull;
    tile_start[0] = 0;
    short_start[0] = 0;
  }
  __syncthreads();
  for (int base = 0; base < n_seqs; base += blockDim.x) {
    const int i = base + threadIdx.x;
    int begin = 0, len = 0;
    unsigned long long v = 0ull;  // low half: main-table tiles of this sequence; high half: short entries
    if (i < n_seqs) {
      const int b_raw = cu_seqlens[i], e_raw = cu_seqlens[i + 1];
      begin = min(max(b_raw, 0), T);
      const int end = min(max(e_raw, begin), T);
      if (b_raw != begin || e_raw != end) set_status(status, ST_BAD_CU_SEQLENS);
      len = end - begin;
      if (len > 0) v = (len <= short_max) ? (1ull << 32) : (unsigned long long)((len + bm - 1) / bm);
    }
    unsigned long long incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      unsigned long long w = (lane < (blockDim.x >> 5)) ? warp_sums[lane] : 0ull;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long n = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += n;
      }
      warp_sums[lane] = w;
    }
    __syncthreads();
    const unsigned long long after = carry_s + (warp == 0 ? 0ull : warp_sums[warp - 1]) + incl;
    if (i < n_seqs) {
      const unsigned long long before = after - v;
      const int long_hi = (int)min((unsigned long long)cap_long, after & 0xffffffffull);
      const int long_lo = (int)min((unsigned long long)cap_long, before & 0xffffffffull);
      if ((after & 0xffffffffull) > (unsigned long long)cap_long) set_status(status, ST_BAD_CU_SEQLENS);
      tile_start[i + 1] = long_hi;
      short_start[i + 1] = (int)(after >> 32);
      for (int t = long_lo; t < long_hi; ++t) tile_info[t] = make_int4(begin, len, (t - long_lo) * bm, i);
      if ((v >> 32) != 0ull) short_info[(int)(before >> 32)] = make_int4(begin, len, 0, i);
    }
    __syncthreads();
    if (threadIdx.x == 0) carry_s += warp_sums[(blockDim.x >> 5) - 1];
    __syncthreads();
  }
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                          uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Byte offset of the 16-byte chunk `chunk` (0..7) of row `row` in a [rows][64] bf16
// tile whose chunks are XOR-swizzled by the row so ldmatrix reads are conflict free.
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return uint32_t(row * 128 + ((chunk ^ (row & 7)) << 4));
}

// Loads `rows` rows x 64 bf16 from global (row stride `stride` elements) into a
// swizzled tile; rows at or beyond `valid_rows` are zero-filled.
template <int THREADS>
__device__ __forceinline__ void load_tile_async(uint32_t smem_tile, const __nv_bfloat16* gbase,
                                                int64_t stride, int rows, int valid_rows) {
  constexpr int RPP = THREADS / 8;  // rows per pass of the CTA
  if constexpr (RPP % 8 == 0) {
    // a thread keeps its 16-byte column and its row modulo 8 from pass to pass: the swizzle term
    // is fixed and both addresses advance by constants
    const int r0 = threadIdx.x >> 3, c = threadIdx.x & 7;
    uint32_t dst = smem_tile + tile_off(r0, c);
    const __nv_bfloat16* src = gbase + int64_t(r0) * stride + c * 8;
    for (int r = r0; r < rows; r += RPP, dst += RPP * 128, src += RPP * stride) {
      const bool ok = r < valid_rows;
      cp_async16(dst, ok ? src : gbase, ok ? 16 : 0);
    }
  } else {
    for (int i = threadIdx.x; i < rows * 8; i += THREADS) {
      const int r = i >> 3, c = i & 7;
      const bool ok = r < valid_rows;
      const __nv_bfloat16* src = gbase + (ok ? int64_t(r) * stride : 0) + c * 8;
      cp_async16(smem_tile + tile_off(r, c), src, ok ? 16 : 0);
    }
  }
}

template <int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32, 16 / NWARPS)  // 16 warps per SM: 128 registers
attn_varlen_mma_kernel(const __nv_bfloat16* __restrict__ qkv, const int4* __restrict__ tile_info,
                       const int32_t* __restrict__ total_tiles_ptr, int nh, int half_window,
                       __nv_bfloat16* __restrict__ out) {
  constexpr int BM = NWARPS * 16;
  constexpr int THREADS = NWARPS * 32;
  // One CTA serves a query tile for several heads (blockIdx.y, blockIdx.y + gridDim.y, ...), with
  // two shared-memory stages of (Q, one K tile, one V tile): the loads of the next head are in
  // flight while this head is computed.  The kernel is latency bound - one short global round
  // trip and a few hundred MMAs per (tile, head) - so what counts is never waiting for that
  // round trip with nothing else to do.  The sequences it serves (at most 64 tokens) have a
  // single key tile; the shortest of them share their tile among several heads (below).
  constexpr int STAGE_BYTES_ = BM * 128 + 2 * ATT_BN * 128;
  __shared__ __align__(128) uint8_t smem[2 * STAGE_BYTES_];
  const uint32_t smem0 = smem_u32(smem);

  const int tile = blockIdx.x;
  if (tile >= *total_tiles_ptr) return;
  const int4 info = tile_info[tile];
  const int seq_begin = info.x;
  const int len = info.y;
  const int q0 = info.z;
  const int H = nh * ATT_D;
  const int64_t stride = 3 * int64_t(H);

  int kv_lo = 0, kv_hi = len;
  if (half_window >= 0) {
    kv_lo = max(0, q0 - half_window);
    kv_hi = min(len, q0 + BM + half_window);
  }
  const int n_kv = (kv_hi - kv_lo + ATT_BN - 1) / ATT_BN;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float scale_log2 = 0.125f * 1.4426950408889634f;
  const int row_in_warp = lane >> 2;           // rows r and r + 8 of this warp's 16
  // A sequence of at most BM / 2 tokens leaves half of the tile's rows - and warps - without
  // work.  Such a tile is shared by several heads instead: with R = 16 or 32 rows per head, rows
  // [R hs, R hs + R) of the Q, K and V tiles belong to head slot hs, and a step of the CTA serves
  // BM / R of its heads at once (same loads, same shared memory, a quarter or half of the steps).
  int R = BM;
  if (q0 == 0 && n_kv == 1) R = len <= 16 ? 16 : (len <= 32 ? min(32, BM) : BM);
  const int hps = BM / R;                                // heads per step
  const int hs = (warp * 16) / R, rb = (warp * 16) % R;  // this warp's head slot and first row in it
  const int qrow0 = q0 + rb + row_in_warp;               // position in sequence of row r
  const int my_heads = (nh - int(blockIdx.y) + int(gridDim.y) - 1) / int(gridDim.y);  // heads of this CTA
  auto head_of = [&](int i) { return int(blockIdx.y) + i * int(gridDim.y); };           // the i-th of them

  auto load_step = [&](int t, int stage) {
    const uint32_t sQ_ = smem0 + stage * STAGE_BYTES_;
    for (int s_ = 0; s_ < hps; ++s_) {
      const bool hv = t * hps + s_ < my_heads;  // slots past the CTA's last head are zero-filled
      const __nv_bfloat16* qg_ = qkv + int64_t(seq_begin) * stride + (hv ? head_of(t * hps + s_) : 0) * ATT_D;
      const uint32_t sub = uint32_t(s_ * R) * 128u;
      load_tile_async<THREADS>(sQ_ + sub, qg_ + int64_t(q0) * stride, stride, R, hv ? len - q0 : 0);
      load_tile_async<THREADS>(sQ_ + BM * 128 + sub, qg_ + H + int64_t(kv_lo) * stride, stride,
                               hps == 1 ? ATT_BN : R, hv ? kv_hi - kv_lo : 0);
      load_tile_async<THREADS>(sQ_ + BM * 128 + ATT_BN * 128 + sub, qg_ + 2 * H + int64_t(kv_lo) * stride, stride,
                               hps == 1 ? ATT_BN : R, hv ? kv_hi - kv_lo : 0);
    }
    cp_async_commit();
  };
  load_step(0, 0);

  int stage = 0;
  for (int t = 0; t * hps < my_heads; ++t, stage ^= 1) {
  const uint32_t sQ = smem0 + stage * STAGE_BYTES_;
  const uint32_t sK = sQ + BM * 128;
  const uint32_t sV = sK + ATT_BN * 128;
  const bool head_valid = t * hps + hs < my_heads;
  const int head = head_of(head_valid ? t * hps + hs : 0);
  // Warps whose 16 rows lie past the end of the sequence (or whose slot holds no head) only take
  // part in the loads and barriers.
  const bool active = head_valid && q0 + rb < len;
  const __nv_bfloat16* kg = qkv + int64_t(seq_begin) * stride + head * ATT_D + H;
  const __nv_bfloat16* vg = kg + H;
  const bool more = (t + 1) * hps < my_heads;
  if (more) load_step(t + 1, stage ^ 1);  // the other stage was released by the barrier below

  float o_acc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[j][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  uint32_t qf[4][4];

  for (int it = 0; it < n_kv; ++it) {
    if (it > 0) {  // a longer sequence (not selected by the dispatcher): reload this stage's K / V
      __syncthreads();
      const int k0n = kv_lo + it * ATT_BN;
      load_tile_async<THREADS>(sK, kg + int64_t(k0n) * stride, stride, ATT_BN, kv_hi - k0n);
      load_tile_async<THREADS>(sV, vg + int64_t(k0n) * stride, stride, ATT_BN, kv_hi - k0n);
      cp_async_commit();
      cp_async_wait<0>();
    } else if (more) {
      cp_async_wait<1>();  // this head's tiles have landed; the next head's are still in flight
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (!active) continue;
    if (it == 0) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = kk * 2 + (lane >> 4);
        ldsm_x4(sQ + tile_off(r, c), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
      }
    }
    const uint32_t kt = sK;
    const uint32_t vt = sV;
    const int k0 = kv_lo + it * ATT_BN;
    // 16-key blocks of this tile that hold any key of the sequence: the MMAs of the others are
    // skipped (their scores are masked to -inf below, their P is 0).  mma.sync is the scarce
    // resource of this kernel, and a 30-token query fills two of a tile's four blocks.
    const int nkb = min(4, (kv_hi - k0 + 15) >> 4);

    // S = Q K^T for this warp's 16 rows x 64 keys.  Everything from here to P V touches only the
    // nkb 16-key blocks in use (s[2 jp], s[2 jp + 1] for jp < nkb): the rest of a short sequence's
    // tile would be scaled, masked to -inf, exponentiated to 0 and added, instruction by instruction.
    float s[8][4];
#pragma unroll
    for (int jp = 0; jp < 4; ++jp) {
      if (jp >= nkb) break;
#pragma unroll
      for (int e = 0; e < 4; ++e) s[2 * jp][e] = s[2 * jp + 1][e] = 0.f;
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {
        if (jp >= nkb) break;
        const int mid = lane >> 3;
        const int r = hs * R + (jp * 2 + (mid >> 1)) * 8 + (lane & 7);
        const int c = kk * 2 + (mid & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(kt + tile_off(r, c), b0, b1, b2, b3);
        mma_bf16_16816(s[jp * 2], qf[kk], b0, b1);
        mma_bf16_16816(s[jp * 2 + 1], qf[kk], b2, b3);
      }
    }

    // scale into the exp2 domain and mask.  A band as wide as the sequence excludes nothing.
    const bool band = half_window >= 0 && half_window < len - 1;
    const bool need_mask = band || (k0 + ATT_BN > kv_hi);
    const int lim = kv_hi - k0 - (lane & 3) * 2;  // column 8 j + (e & 1) of this lane is a key of the sequence iff < lim
#pragma unroll
    for (int jp = 0; jp < 4; ++jp) {
      if (jp >= nkb) break;
#pragma unroll
      for (int j = 2 * jp; j < 2 * jp + 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float v = s[j][e] * scale_log2;
          if (need_mask) {
            bool ok = j * 8 + (e & 1) < lim;
            if (band) {
              const int key = k0 + j * 8 + (lane & 3) * 2 + (e & 1);
              const int qi = qrow0 + (e >> 1) * 8;
              ok = ok && (abs(qi - key) <= half_window);
            }
            if (!ok) v = -INFINITY;
          }
          s[j][e] = v;
        }
      }
    }
    // online softmax for rows r (e = 0,1) and r + 8 (e = 2,3)
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2) {
      float mx = -INFINITY;
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {
        if (jp >= nkb) break;
        mx = fmaxf(mx, fmaxf(fmaxf(s[2 * jp][h2 * 2], s[2 * jp][h2 * 2 + 1]),
                             fmaxf(s[2 * jp + 1][h2 * 2], s[2 * jp + 1][h2 * 2 + 1])));
      }
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_run[h2], mx);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      float sum = 0.f;
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {
        if (jp >= nkb) break;
#pragma unroll
        for (int j = 2 * jp; j < 2 * jp + 2; ++j) {
          const float p0 = fast_exp2(s[j][h2 * 2] - m_safe);
          const float p1 = fast_exp2(s[j][h2 * 2 + 1] - m_safe);
          s[j][h2 * 2] = p0;
          s[j][h2 * 2 + 1] = p1;
          sum += p0 + p1;
        }
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if (it > 0) {  // a first tile has nothing to rescale
        const float alpha = fast_exp2(m_run[h2] - m_safe);
        l_run[h2] *= alpha;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o_acc[j][h2 * 2] *= alpha;
          o_acc[j][h2 * 2 + 1] *= alpha;
        }
      }
      l_run[h2] += sum;
      m_run[h2] = m_new;
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      if (kk >= nkb) break;
      uint32_t pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) {
        const int mid = lane >> 3;
        const int r = hs * R + kk * 16 + (mid & 1) * 8 + (lane & 7);
        const int c = jp * 2 + (mid >> 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(vt + tile_off(r, c), b0, b1, b2, b3);
        mma_bf16_16816(o_acc[jp * 2], pa, b0, b1);
        mma_bf16_16816(o_acc[jp * 2 + 1], pa, b2, b3);
      }
    }
  }

  // normalise, stage this warp's 16 x 64 outputs in its own rows of the Q tile, store 16 B wide
  const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f;
  const float inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int r0 = warp * 16 + row_in_warp;
    const uint32_t w0 = pack_bf16(o_acc[j][0] * inv0, o_acc[j][1] * inv0);
    const uint32_t w1 = pack_bf16(o_acc[j][2] * inv1, o_acc[j][3] * inv1);
    const uint32_t a0 = sQ + tile_off(r0, j) + (lane & 3) * 4;
    const uint32_t a1 = sQ + tile_off(r0 + 8, j) + (lane & 3) * 4;
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(a0), "r"(w0) : "memory");
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(a1), "r"(w1) : "memory");
  }
  __syncwarp();
  __nv_bfloat16* og = out + int64_t(seq_begin) * H + head * ATT_D;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = i * 32 + lane;
    const int r = warp * 16 + (idx >> 3), c = idx & 7;  // row of the tile; rb + (idx >> 3) within the head slot
    if (active && q0 + rb + (idx >> 3) < len) {
      uint4 v;
      asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                   : "r"(sQ + tile_off(r, c)));
      *reinterpret_cast<uint4*>(og + int64_t(q0 + rb + (idx >> 3)) * H + c * 8) = v;
    }
  }
  __syncthreads();  // every warp is done with this stage before the head after next is loaded into it
  }  // heads
}

int attn_pick_bm(int max_seqlen) {
  if (max_seqlen <= 16) return 16;
  if (max_seqlen <= 32) return 32;
  if (max_seqlen <= 64) return 64;
  return 128;  // tensor-memory kernels, with the sequences of at most 64 tokens on the register kernel
}

// Sequences of at most this many tokens form the short class of a batch scheduled with 128-row tiles.
constexpr int ATT_SHORT_MAX = 64;

// Scratch layout: tile_start int32[n_seqs + 1], short_start int32[n_seqs + 1], padded to 16 bytes,
// then tile_info int4[T / bm + n_seqs] and short_info int4[n_seqs].  The size is taken for the
// smallest tile height (16), which bounds every other.
constexpr size_t info_offset_c(int n_seqs) { return (size_t(2 * n_seqs + 2) * sizeof(int32_t) + 15) & ~size_t(15); }
constexpr size_t scratch_bytes_c(int64_t T, int n_seqs) {
  return info_offset_c(n_seqs) + size_t(T / 16 + 2 * int64_t(n_seqs) + 2) * sizeof(int4);
}
size_t attn_info_offset(int n_seqs) { return info_offset_c(n_seqs); }
size_t attn_scratch_bytes(int64_t T, int n_seqs) { return scratch_bytes_c(T, n_seqs); }

struct TileTables {
  int32_t* tile_start;
  int32_t* short_start;
  int4* tile_info;
  int4* short_info;
  int cap_long;
};
static TileTables tile_tables(void* scratch, int n_seqs, int64_t T, int bm) {
  TileTables t;
  t.tile_start = static_cast<int32_t*>(scratch);
  t.short_start = t.tile_start + n_seqs + 1;
  t.tile_info = reinterpret_cast<int4*>(static_cast<uint8_t*>(scratch) + info_offset_c(n_seqs));
  t.cap_long = int(T / bm + n_seqs);
  t.short_info = t.tile_info + t.cap_long;
  return t;
}

int attn_schedule(const int32_t* cu_seqlens, int n_seqs, int64_t T, int bm, bool split_short,
                  void* scratch, int32_t* status, cudaStream_t st) {
  PE_REQUIRE(T >= 0 && T < (1ll << 31) - 256 && n_seqs > 0 && T / bm + n_seqs < (1ll << 31),
             "attention schedule: %lld tokens / %d sequences out of range", (long long)T, n_seqs);
  const TileTables t = tile_tables(scratch, n_seqs, T, bm);
  attn_schedule_kernel<<<1, 1024, 0, st>>>(cu_seqlens, n_seqs, (int)T, bm,
                                           split_short ? ATT_SHORT_MAX : 0, t.cap_long, t.tile_start,
                                           t.short_start, t.tile_info, t.short_info, status);
  PE_LAUNCH_CHECK("attn_schedule_kernel");
  return PE_OK;
}

static int launch_short(const __nv_bfloat16* q, const int4* info, const int32_t* total, int64_t max_tiles,
                        int bm, int nh, int half_window, int heads_per_cta, __nv_bfloat16* o,
                        cudaStream_t st) {
  dim3 grid((unsigned)max_tiles, (unsigned)((nh + heads_per_cta - 1) / heads_per_cta));
  switch (bm) {
    case 16:
      attn_varlen_mma_kernel<1><<<grid, 32, 0, st>>>(q, info, total, nh, half_window, o);
      break;
    case 32:
      attn_varlen_mma_kernel<2><<<grid, 64, 0, st>>>(q, info, total, nh, half_window, o);
      break;
    case 64:
      attn_varlen_mma_kernel<4><<<grid, 128, 0, st>>>(q, info, total, nh, half_window, o);
      break;
    default:
      set_last_error("attention: unsupported query tile %d", bm);
      return PE_ERR_ARG;
  }
  PE_LAUNCH_CHECK("attn_varlen_mma_kernel");
  return PE_OK;
}

int attn_run(const void* qkv, const void* scratch, int n_seqs, int64_t T, int nh, int half_window,
             int bm, void* out, int32_t* status, cudaStream_t st) {
  const TileTables t = tile_tables(const_cast<void*>(scratch), n_seqs, T, bm);
  const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(qkv);
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(out);
  // A batch of short sequences only: four heads per CTA (see the kernel) - enough CTAs to fill the
  // GPU, few enough that each hides its own load latency.
  if (bm != 128) return launch_short(q, t.tile_info, t.tile_start + n_seqs, t.cap_long, bm, nh, half_window, 4, o, st);
  // Long batch: the tensor-memory kernels take the sequences of more than 64 tokens (at most
  // T / 128 + T / 65 tiles of them exist), the register kernel with 64-row tiles the rest.
  const int64_t max_long = std::min<int64_t>(t.cap_long, T / 128 + T / (ATT_SHORT_MAX + 1) + 1);
  int rc = (half_window == 64)
               ? attn_run_local_tc2(qkv, t.tile_info, t.tile_start + n_seqs, max_long, T, nh, out, status, st)
               : attn_run_global_tc(qkv, t.tile_info, t.tile_start + n_seqs, max_long, T, nh, half_window,
                                    out, status, st);
  if (rc != PE_OK) return rc;
  // Usually few sequences are short here, so this launch is a latency chain, not a throughput
  // problem: one head per CTA keeps the chain at a quarter of the four-head form's.
  const int64_t max_short = std::min<int64_t>(n_seqs, T);
  return launch_short(q, t.short_info, t.short_start + n_seqs, max_short, 64, nh, half_window, 1, o, st);
}

// ---- scratch that needs no allocation -------------------------------------------------
// pe_attn_varlen_static keeps its tile table in this array instead of caller memory.  Every
// GPU that loads the library carries the array from load until the process exits.
constexpr int STATIC_MAX_SEQS = 4096;
constexpr int64_t STATIC_MAX_TOKENS = 1 << 20;
constexpr size_t STATIC_SCRATCH_BYTES = scratch_bytes_c(STATIC_MAX_TOKENS, STATIC_MAX_SEQS);
static __device__ __align__(256) unsigned char g_attn_static_scratch[STATIC_SCRATCH_BYTES];

// Device address of the array on the current device.  In host code the symbol's name is only
// a handle, so the address is asked of the runtime, once per device, with that device current.
static int static_scratch_ptr(void** out) {
  static std::mutex lock;
  static void* ptrs[64] = {nullptr};
  int dev = 0;
  PE_CUDA(cudaGetDevice(&dev));
  PE_REQUIRE(dev >= 0 && dev < 64, "pe_attn_varlen_static: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> guard(lock);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    PE_CUDA(cudaGetSymbolAddress(&p, g_attn_static_scratch));
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return PE_OK;
}

}  // namespace pe

extern "C" int pe_attn_varlen_static(const void* qkv, const int32_t* cu_seqlens, int n_seqs, int64_t T,
                                     int nh, int half_window, int max_seqlen, void* out,
                                     int32_t* status, void* stream) {
  using namespace pe;
  PE_REQUIRE(qkv && cu_seqlens && out, "pe_attn_varlen_static: null pointer");
  PE_REQUIRE(n_seqs > 0 && T >= 0 && nh > 0 && nh <= 65535 && max_seqlen > 0,
             "pe_attn_varlen_static: bad sizes");
  if (n_seqs > STATIC_MAX_SEQS || T > STATIC_MAX_TOKENS) {
    set_last_error("pe_attn_varlen_static: %d sequences / %lld tokens exceed the built-in scratch "
                   "(at most %d sequences and %lld tokens); use pe_attn_varlen with caller scratch",
                   n_seqs, (long long)T, STATIC_MAX_SEQS, (long long)STATIC_MAX_TOKENS);
    return PE_ERR_WORKSPACE;
  }
  if (T == 0) return PE_OK;
  void* scratch = nullptr;
  int rc = static_scratch_ptr(&scratch);
  if (rc != PE_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int bm = attn_pick_bm(max_seqlen);
  // The scheduling kernel rewrites every table entry this call reads, so nothing left by an
  // earlier call is used and nothing has to be cleared first.
  rc = attn_schedule(cu_seqlens, n_seqs, T, bm, bm == 128, scratch, status, st);
  if (rc != PE_OK) return rc;
  return attn_run(qkv, scratch, n_seqs, T, nh, half_window, bm, out, status, st);
}

extern "C" size_t pe_attn_workspace_bytes(int64_t T, int n_seqs) {
  if (T < 0 || n_seqs < 0) return 0;
  return pe::attn_scratch_bytes(T, n_seqs);
}

extern "C" int pe_attn_varlen(const void* qkv, const int32_t* cu_seqlens, int n_seqs, int64_t T,
                              int nh, int half_window, int max_seqlen, void* out, void* workspace,
                              size_t workspace_bytes, int32_t* status, void* stream) {
  using namespace pe;
  PE_REQUIRE(qkv && cu_seqlens && out && workspace, "pe_attn_varlen: null pointer");
  PE_REQUIRE(n_seqs > 0 && T >= 0 && nh > 0 && nh <= 65535, "pe_attn_varlen: bad sizes");
  PE_REQUIRE(max_seqlen > 0, "pe_attn_varlen: max_seqlen must be positive");
  PE_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0,
             "pe_attn_varlen: workspace must be 16-byte aligned");
  if (workspace_bytes < pe_attn_workspace_bytes(T, n_seqs)) {
    set_last_error("pe_attn_varlen: workspace %zu < %zu bytes", workspace_bytes,
                   pe_attn_workspace_bytes(T, n_seqs));
    return PE_ERR_WORKSPACE;
  }
  if (T == 0) return PE_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int bm = attn_pick_bm(max_seqlen);
  int rc = attn_schedule(cu_seqlens, n_seqs, T, bm, bm == 128, workspace, status, st);
  if (rc != PE_OK) return rc;
  return attn_run(qkv, workspace, n_seqs, T, nh, half_window, bm, out, status, st);
}
