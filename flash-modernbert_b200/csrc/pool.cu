// Pooling head on the packed output: what every caller of packed_forward in the reference does
// next (benchmarks/showcases/inference.py:193-206 - fp32 segment sums by index_add_, divide by
// the length, F.normalize(p=2), cast back; or the first token of each sequence).  Turns the
// [T, H] last hidden state into [N, H] sentence embeddings, which is also what a multi-GPU run
// has to gather instead of [T, H].
//
// HBM-bound: the hidden state is read once.  Two launches, no atomics, fixed summation order:
//   pool_partial_kernel : one CTA per 128-row tile of one sequence (the attention tile
//                         schedule) -> fp32 column sums of the tile
//   pool_finish_kernel  : one CTA per sequence: adds its tiles' sums in order, divides by the
//                         length, L2-normalises, rounds to bf16
#include <algorithm>

#include "pe_host.h"
#include "pe_ptx.cuh"
#include "pe_vec.cuh"

namespace pe {

constexpr int POOL_THREADS = 256;          // finish kernel: up to 8 columns per thread
constexpr int POOL_PARTIAL_THREADS = 512;  // partial sums: as many row groups in flight as fit
constexpr int POOL_ROWS = 128;  // rows per partial sum = rows per scheduler tile

static size_t pool_align(size_t v) { return (v + 255) & ~size_t(255); }

__global__ void __launch_bounds__(POOL_PARTIAL_THREADS)
pool_partial_kernel(const __nv_bfloat16* __restrict__ hidden, const int4* __restrict__ tile_info,
                    const int32_t* __restrict__ total_tiles, int H, float* __restrict__ partial) {
  extern __shared__ float pool_smem[];  // [row groups - 1][H]
  const int tile = blockIdx.x;
  if (tile >= *total_tiles) return;
  const int4 info = __ldg(tile_info + tile);  // {first token of the sequence, length, first row, sequence}
  const int rows = min(POOL_ROWS, info.y - info.z);
  const int cols8 = H >> 3;                      // 16-byte column groups
  const int groups = POOL_PARTIAL_THREADS / cols8;  // row groups that fit in the block
  const int cg = threadIdx.x % cols8, rg = threadIdx.x / cols8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (rg < groups) {
    const __nv_bfloat16* src = hidden + (size_t(info.x) + info.z) * H + cg * 8;
#pragma unroll 4
    for (int r = rg; r < rows; r += groups) {
      uint4 v;
      asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                   : "l"(src + size_t(r) * H));
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(p[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
    if (rg > 0) {
#pragma unroll
      for (int e = 0; e < 8; ++e) pool_smem[(rg - 1) * H + cg * 8 + e] = acc[e];
    }
  }
  __syncthreads();
  if (rg == 0) {
    for (int g = 1; g < groups; ++g) {  // fixed order
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] += pool_smem[(g - 1) * H + cg * 8 + e];
    }
    float4* dst = reinterpret_cast<float4*>(partial + size_t(tile) * H + cg * 8);
    dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
  }
}

// mode 0: first token; mode 1: mean over the sequence.
__global__ void __launch_bounds__(POOL_THREADS)
pool_finish_kernel(const __nv_bfloat16* __restrict__ hidden, const int32_t* __restrict__ cu_seqlens,
                   const int32_t* __restrict__ tile_start, const float* __restrict__ partial, int T,
                   int H, int mode, int normalize, __nv_bfloat16* __restrict__ out) {
  __shared__ float red[POOL_THREADS / 32];
  __shared__ float inv_s;
  const int seq = blockIdx.x;
  // boundaries clamped into [0, T] exactly as the tile schedule clamps them
  const int begin = min(max(cu_seqlens[seq], 0), T);
  const int len = min(max(cu_seqlens[seq + 1], begin), T) - begin;
  constexpr int MAXV = 8;  // columns per thread: H <= 2048
  float v[MAXV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = threadIdx.x + i * POOL_THREADS;
    v[i] = 0.f;
    if (c < H && len > 0) {
      if (mode == 0) {
        v[i] = __bfloat162float(hidden[size_t(begin) * H + c]);
      } else {
        float s = 0.f;
        for (int t = tile_start[seq]; t < tile_start[seq + 1]; ++t) s += partial[size_t(t) * H + c];
        v[i] = s / float(len);
      }
    }
    ss += v[i] * v[i];
  }
  float inv = 1.f;
  if (normalize) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float total = 0.f;
      for (int w = 0; w < POOL_THREADS / 32; ++w) total += red[w];
      inv_s = 1.f / fmaxf(sqrtf(total), 1e-12f);  // F.normalize's eps
    }
    __syncthreads();
    inv = inv_s;
  }
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = threadIdx.x + i * POOL_THREADS;
    if (c < H) out[size_t(seq) * H + c] = __float2bfloat16(v[i] * inv);
  }
}

// ---- the final LayerNorm fused with the pooling head -----------------------------------------
// The last step of a forward whose caller wants sentence embeddings: y = LayerNorm(x) * w is
// computed row by row as in ln_rows_kernel and, in the same pass, summed per 128-row tile of its
// sequence, so the [T, H] hidden state is never read back (and not even written when the caller
// does not ask for it).  Sums are taken over the bf16-rounded y, as a caller pooling the
// materialised hidden state would see it.

// One LayerNorm row held by a warp: VPL 16-byte vectors per lane.  Returns y rounded to bf16.
template <int VPL>
__device__ __forceinline__ void ln_row_to_bf16(const __nv_bfloat16* __restrict__ xrow,
                                               const __nv_bfloat16* __restrict__ w, float eps, int H,
                                               int lane, uint4 (&yq)[VPL]) {
  const int nvec = H >> 3;
  float v[VPL][8];
  float sum = 0.f, sq = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      unpack8(ld_stream(reinterpret_cast<const uint4*>(xrow) + c), v[i]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        sum += v[i][e];
        sq += v[i][e] * v[i][e];
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
    sq += __shfl_xor_sync(0xffffffffu, sq, o);
  }
  const float mean = sum / float(H);
  const float var = sq / float(H) - mean * mean;
  const float rstd = rsqrtf(var + eps);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + 32 * i;
    yq[i] = make_uint4(0u, 0u, 0u, 0u);
    if (c < nvec) {
      float wv[8], o[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(w) + c), wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[i][e] - mean) * rstd * wv[e];
      yq[i] = pack8(o);
    }
  }
}

constexpr int LNP_WARPS = 8;

template <int VPL>
__global__ void __launch_bounds__(LNP_WARPS * 32)
ln_pool_partial_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, float eps,
                       const int4* __restrict__ tile_info, const int32_t* __restrict__ total_tiles, int H,
                       __nv_bfloat16* __restrict__ y, float* __restrict__ partial) {
  extern __shared__ float pool_smem[];  // [LNP_WARPS - 1][H]
  const int tile = blockIdx.x;
  if (tile >= *total_tiles) return;
  const int4 info = __ldg(tile_info + tile);
  const int rows = min(POOL_ROWS, info.y - info.z);
  const size_t row0 = size_t(info.x) + info.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = H >> 3;
  float acc[VPL][8];
#pragma unroll
  for (int i = 0; i < VPL; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
  for (int r = warp; r < rows; r += LNP_WARPS) {
    uint4 yq[VPL];
    ln_row_to_bf16<VPL>(x + (row0 + r) * H, w, eps, H, lane, yq);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        if (y != nullptr) reinterpret_cast<uint4*>(y + (row0 + r) * H)[c] = yq[i];
        float f[8];
        unpack8(yq[i], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[i][e] += f[e];
      }
    }
  }
  if (warp > 0) {
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
#pragma unroll
        for (int e = 0; e < 8; ++e) pool_smem[(warp - 1) * H + c * 8 + e] = acc[i][e];
      }
    }
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        for (int g = 1; g < LNP_WARPS; ++g) {  // fixed order: repeated calls give the same bits
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[i][e] += pool_smem[(g - 1) * H + c * 8 + e];
        }
        float4* dst = reinterpret_cast<float4*>(partial + size_t(tile) * H + c * 8);
        dst[0] = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        dst[1] = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
      }
    }
  }
}

// First-token pooling without the hidden state: the final LayerNorm runs on one row per
// sequence only.  One warp per sequence.
template <int VPL>
__global__ void __launch_bounds__(256)
ln_first_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, float eps,
                     const int32_t* __restrict__ cu_seqlens, int n_seqs, int T, int H, int normalize,
                     __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int seq = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (seq >= n_seqs) return;
  const int nvec = H >> 3;
  const int begin = min(max(cu_seqlens[seq], 0), T);
  const int len = min(max(cu_seqlens[seq + 1], begin), T) - begin;
  uint4 yq[VPL];
  if (len > 0) {
    ln_row_to_bf16<VPL>(x + size_t(begin) * H, w, eps, H, lane, yq);
  } else {
#pragma unroll
    for (int i = 0; i < VPL; ++i) yq[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  float inv = 1.f;
  if (normalize) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      float f[8];
      unpack8(yq[i], f);  // lanes beyond the row hold zeros
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    inv = 1.f / fmaxf(sqrtf(ss), 1e-12f);
  }
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      float f[8];
      unpack8(yq[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] *= inv;
      reinterpret_cast<uint4*>(out + size_t(seq) * H)[c] = pack8(f);
    }
  }
}

int final_ln_pool(const void* x, const void* w, float eps, const int32_t* cu_seqlens, int n_seqs,
                  int64_t T, int H, int mode, int normalize, void* hidden_out, void* pooled_out,
                  void* workspace, size_t workspace_bytes, cudaStream_t st) {
  PE_REQUIRE(x && w && cu_seqlens && pooled_out, "final norm + pooling: null pointer");
  PE_REQUIRE(mode == 0 || mode == 1, "final norm + pooling: mode %d (0 = first token, 1 = mean)", mode);
  PE_REQUIRE(H > 0 && H % 8 == 0 && H <= 2048, "final norm + pooling: H=%d must be a multiple of 8, <= 2048", H);
  PE_REQUIRE(n_seqs > 0 && T > 0 && T < (1ll << 31) - 256, "final norm + pooling: bad sizes");
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(w);
  __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(hidden_out);
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(pooled_out);
  const int vpl = (H / 8 + 31) / 32;
  if (mode == 0) {
    if (hidden_out != nullptr) {  // the caller wants both: plain final norm, then pick the first rows
      int rc = pe_add_ln(x, nullptr, w, eps, T, H, nullptr, hidden_out, st);
      if (rc != PE_OK) return rc;
      return pe_pool_packed(hidden_out, cu_seqlens, n_seqs, T, H, 0, normalize, pooled_out, nullptr, 0, st);
    }
    const unsigned blocks = (unsigned)((int64_t(n_seqs) * 32 + 255) / 256);
#define PE_FIRST_CASE(V)                                                                          \
  case V:                                                                                         \
    ln_first_rows_kernel<V><<<blocks, 256, 0, st>>>(xp, wp, eps, cu_seqlens, n_seqs, (int)T, H,   \
                                                    normalize, op);                               \
    break;
    switch (vpl) {
      PE_FIRST_CASE(1) PE_FIRST_CASE(2) PE_FIRST_CASE(3) PE_FIRST_CASE(4) PE_FIRST_CASE(5)
      PE_FIRST_CASE(6) PE_FIRST_CASE(7) PE_FIRST_CASE(8)
      default:
        set_last_error("final norm + pooling: unsupported H=%d", H);
        return PE_ERR_ARG;
    }
#undef PE_FIRST_CASE
    PE_LAUNCH_CHECK("ln_first_rows_kernel");
    return PE_OK;
  }
  PE_REQUIRE(workspace != nullptr, "final norm + pooling: mean pooling needs a workspace");
  if (workspace_bytes < pe_pool_workspace_bytes(T, n_seqs, H)) {
    set_last_error("final norm + pooling: workspace of %zu bytes, %zu needed", workspace_bytes,
                   pe_pool_workspace_bytes(T, n_seqs, H));
    return PE_ERR_WORKSPACE;
  }
  int rc = attn_schedule(cu_seqlens, n_seqs, T, POOL_ROWS, false, workspace, nullptr, st);
  if (rc != PE_OK) return rc;
  const int32_t* tile_start = static_cast<const int32_t*>(workspace);
  const int4* tile_info =
      reinterpret_cast<const int4*>(static_cast<const uint8_t*>(workspace) + attn_info_offset(n_seqs));
  float* part = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + pool_align(attn_scratch_bytes(T, n_seqs)));
  const int64_t max_tiles = T / POOL_ROWS + n_seqs;
  const size_t smem = size_t(LNP_WARPS - 1) * H * sizeof(float);
#define PE_LNP_CASE(V)                                                                                 \
  case V:                                                                                              \
    rc = set_max_dynamic_smem(reinterpret_cast<const void*>(ln_pool_partial_kernel<V>), (int)smem, false); \
    if (rc != PE_OK) return rc;                                                                        \
    ln_pool_partial_kernel<V><<<(unsigned)max_tiles, LNP_WARPS * 32, smem, st>>>(                      \
        xp, wp, eps, tile_info, tile_start + n_seqs, H, yp, part);                                     \
    break;
  switch (vpl) {
    PE_LNP_CASE(1) PE_LNP_CASE(2) PE_LNP_CASE(3) PE_LNP_CASE(4) PE_LNP_CASE(5) PE_LNP_CASE(6)
    PE_LNP_CASE(7) PE_LNP_CASE(8)
    default:
      set_last_error("final norm + pooling: unsupported H=%d", H);
      return PE_ERR_ARG;
  }
#undef PE_LNP_CASE
  PE_LAUNCH_CHECK("ln_pool_partial_kernel");
  pool_finish_kernel<<<(unsigned)n_seqs, POOL_THREADS, 0, st>>>(nullptr, cu_seqlens, tile_start, part, (int)T,
                                                               H, 1, normalize, op);
  PE_LAUNCH_CHECK("pool_finish_kernel");
  return PE_OK;
}

}  // namespace pe

extern "C" size_t pe_pool_workspace_bytes(int64_t T, int n_seqs, int H) {
  if (T < 0 || n_seqs < 0 || H <= 0) return 0;
  return pe::pool_align(pe::attn_scratch_bytes(T, n_seqs)) +
         pe::pool_align(size_t(T / pe::POOL_ROWS + n_seqs + 1) * size_t(H) * sizeof(float));
}

extern "C" int pe_pool_packed(const void* hidden, const int32_t* cu_seqlens, int n_seqs, int64_t T,
                              int H, int mode, int normalize, void* out, void* workspace,
                              size_t workspace_bytes, void* stream) {
  using namespace pe;
  PE_REQUIRE(hidden && cu_seqlens && out, "pe_pool_packed: null pointer");
  PE_REQUIRE(mode == 0 || mode == 1, "pe_pool_packed: mode %d (0 = first token, 1 = mean)", mode);
  PE_REQUIRE(H > 0 && H % 8 == 0 && H <= 2048, "pe_pool_packed: H=%d must be a multiple of 8, at most 2048", H);
  PE_REQUIRE(n_seqs >= 0 && T >= 0 && T < (1ll << 31) - 256, "pe_pool_packed: bad sizes");
  if (n_seqs == 0) return PE_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int32_t* tile_start = nullptr;
  const float* partial = nullptr;
  if (mode == 1) {
    PE_REQUIRE(workspace != nullptr, "pe_pool_packed: mean pooling needs a workspace");
    if (workspace_bytes < pe_pool_workspace_bytes(T, n_seqs, H)) {
      set_last_error("pe_pool_packed: workspace of %zu bytes, %zu needed", workspace_bytes,
                     pe_pool_workspace_bytes(T, n_seqs, H));
      return PE_ERR_WORKSPACE;
    }
    int rc = attn_schedule(cu_seqlens, n_seqs, T, POOL_ROWS, false, workspace, nullptr, st);
    if (rc != PE_OK) return rc;
    tile_start = static_cast<const int32_t*>(workspace);
    const int4* tile_info = reinterpret_cast<const int4*>(static_cast<const uint8_t*>(workspace) +
                                                          attn_info_offset(n_seqs));
    float* part = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) +
                                           pool_align(attn_scratch_bytes(T, n_seqs)));
    partial = part;
    const int64_t max_tiles = T / POOL_ROWS + n_seqs;
    PE_REQUIRE(max_tiles < (1ll << 31), "pe_pool_packed: too many tiles");
    const int groups = POOL_PARTIAL_THREADS / (H / 8);
    const size_t smem = size_t(groups > 1 ? groups - 1 : 0) * H * sizeof(float);
    if (max_tiles > 0) {
      pool_partial_kernel<<<(unsigned)max_tiles, POOL_PARTIAL_THREADS, smem, st>>>(
          static_cast<const __nv_bfloat16*>(hidden), tile_info, tile_start + n_seqs, H, part);
      PE_LAUNCH_CHECK("pool_partial_kernel");
    }
  }
  pool_finish_kernel<<<(unsigned)n_seqs, POOL_THREADS, 0, st>>>(
      static_cast<const __nv_bfloat16*>(hidden), cu_seqlens, tile_start, partial, (int)T, H, mode, normalize,
      static_cast<__nv_bfloat16*>(out));
  PE_LAUNCH_CHECK("pool_finish_kernel");
  return PE_OK;
}
