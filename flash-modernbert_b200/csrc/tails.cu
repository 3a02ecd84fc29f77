// Memory-bound pieces of the packed ModernBERT forward for sm_100a: the padding
// boundary (mask -> cu_seqlens / indices / position_ids, row gather, re-pad
// scatter), embedding-gather + LayerNorm, residual-add + LayerNorm, RoPE on the
// fused qkv, GeGLU and the RoPE table.  All are 128-bit vectorised, one warp per
// row where a row reduction is needed, and sized to keep HBM busy rather than
// the SMs.
#include <algorithm>

#include "pe_host.h"
#include "pe_ptx.cuh"
#include "pe_vec.cuh"

namespace pe {

// ------------------------------------------------------------------------------
// unpad: mask [B, S] -> seqlens, cu_seqlens, indices, position_ids, {T, max_seqlen}
// ------------------------------------------------------------------------------
template <typename MaskT>
__global__ void unpad_count_kernel(const MaskT* __restrict__ mask, int B, int S,
                                   int32_t* __restrict__ seqlens) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= B) return;
  const MaskT* row = mask + size_t(warp) * S;
  int cnt = 0;
  for (int s = lane; s < S; s += 32) cnt += (row[s] != 0) ? 1 : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if (lane == 0) seqlens[warp] = cnt;
}

// One block: exclusive scan of seqlens into cu_seqlens[0..B], totals = {sum, max}.
__global__ void unpad_scan_kernel(const int32_t* __restrict__ seqlens, int B,
                                  int32_t* __restrict__ cu_seqlens, int32_t* __restrict__ totals) {
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  __shared__ int max_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    carry_s = 0;
    max_s = 0;
    cu_seqlens[0] = 0;
  }
  __syncthreads();
  int local_max = 0;
  for (int base = 0; base < B; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const int v = (i < B) ? seqlens[i] : 0;
    local_max = max(local_max, v);
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = (lane < (blockDim.x >> 5)) ? warp_sums[lane] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += n;
      }
      warp_sums[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const int warp_off = (warp == 0) ? 0 : warp_sums[warp - 1];
    const int carry = carry_s;
    if (i < B) cu_seqlens[i + 1] = carry + warp_off + incl;
    __syncthreads();
    if (threadIdx.x == 0) carry_s = carry + warp_sums[(blockDim.x >> 5) - 1];
    __syncthreads();
  }
  atomicMax(&max_s, local_max);
  __syncthreads();
  if (threadIdx.x == 0) {
    totals[0] = carry_s;
    totals[1] = max_s;
  }
}

template <typename MaskT>
__global__ void unpad_fill_kernel(const MaskT* __restrict__ mask, int B, int S,
                                  const int32_t* __restrict__ cu_seqlens,
                                  int64_t* __restrict__ indices,
                                  int64_t* __restrict__ position_ids) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= B) return;
  const MaskT* row = mask + size_t(warp) * S;
  int64_t out = cu_seqlens[warp];
  for (int s0 = 0; s0 < S; s0 += 32) {
    const int s = s0 + lane;
    const bool m = (s < S) && (row[s] != 0);
    const unsigned bal = __ballot_sync(0xffffffffu, m);
    if (m) {
      const int64_t o = out + __popc(bal & ((1u << lane) - 1u));
      indices[o] = int64_t(warp) * S + s;
      position_ids[o] = s;
    }
    out += __popc(bal);
  }
}

template <typename MaskT>
static int unpad_launch(const void* mask, int B, int S, int32_t* seqlens, int32_t* cu,
                        int64_t* indices, int64_t* pos, int32_t* totals, cudaStream_t st) {
  const int threads = 128;
  const int blocks = (B * 32 + threads - 1) / threads;
  unpad_count_kernel<MaskT><<<blocks, threads, 0, st>>>(static_cast<const MaskT*>(mask), B, S,
                                                        seqlens);
  PE_LAUNCH_CHECK("unpad_count_kernel");
  unpad_scan_kernel<<<1, 1024, 0, st>>>(seqlens, B, cu, totals);
  PE_LAUNCH_CHECK("unpad_scan_kernel");
  unpad_fill_kernel<MaskT><<<blocks, threads, 0, st>>>(static_cast<const MaskT*>(mask), B, S, cu,
                                                       indices, pos);
  PE_LAUNCH_CHECK("unpad_fill_kernel");
  return PE_OK;
}

// ------------------------------------------------------------------------------
// row gather / re-pad scatter
// ------------------------------------------------------------------------------
// count_dev (may be NULL): the real number of packed rows, read on the device and clamped to T;
// rows at or beyond it are written as zeros and their indices are not read.
template <typename V>
__global__ void gather_rows_kernel(const V* __restrict__ src, const int64_t* __restrict__ indices,
                                   int64_t T, const int32_t* __restrict__ count_dev, int vec_per_row,
                                   V* __restrict__ dst) {
  const int64_t total = T * vec_per_row;
  const int64_t real = count_dev ? min(max(int64_t(*count_dev), int64_t(0)), T) : T;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t t = i / vec_per_row;
    const int c = int(i - t * vec_per_row);
    V v;
    memset(&v, 0, sizeof(V));
    if (t < real) v = src[indices[t] * vec_per_row + c];
    dst[i] = v;
  }
}

// Each output row r looks itself up in the ascending `indices` (binary search):
// found at t -> copy packed row t, else write zeros.  No memset pass.
template <typename V>
__global__ void repad_kernel(const V* __restrict__ packed, const int64_t* __restrict__ indices,
                             int64_t T_cap, const int32_t* __restrict__ count_dev, int64_t rows_out,
                             int vec_per_row, V* __restrict__ out) {
  const int64_t T = count_dev ? min(max(int64_t(*count_dev), int64_t(0)), T_cap) : T_cap;
  const int lanes_per_row = min(vec_per_row, 32);
  const int rows_per_block = blockDim.x / lanes_per_row;
  const int sub = threadIdx.x / lanes_per_row;
  const int l = threadIdx.x % lanes_per_row;
  if (sub >= rows_per_block) return;
  for (int64_t r = int64_t(blockIdx.x) * rows_per_block + sub; r < rows_out;
       r += int64_t(gridDim.x) * rows_per_block) {
    int64_t lo = 0, hi = T;  // first t with indices[t] >= r
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if (indices[mid] < r) lo = mid + 1; else hi = mid;
    }
    const bool hit = (lo < T) && (indices[lo] == r);
    V zero;
    memset(&zero, 0, sizeof(V));
    for (int c = l; c < vec_per_row; c += lanes_per_row)
      out[r * vec_per_row + c] = hit ? packed[lo * vec_per_row + c] : zero;
  }
}

static int pick_vec_bytes(const void* a, const void* b, int64_t row_bytes) {
  const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                         static_cast<uintptr_t>(row_bytes);
  if ((bits & 15) == 0) return 16;
  if ((bits & 7) == 0) return 8;
  if ((bits & 3) == 0) return 4;
  if ((bits & 1) == 0) return 2;
  return 1;
}

// ------------------------------------------------------------------------------
// LayerNorm family: one warp per row, row kept in registers between the
// statistics pass and the normalise pass.  VPL = 16-byte vectors per lane.
// ------------------------------------------------------------------------------
// MODE 0: y = LN(x).  MODE 1: x_new = bf16(x + res), y = LN(x_new).
// MODE 2: x = tok_emb[ids[row]], y = LN(x).
template <int VPL, int MODE>
__global__ void __launch_bounds__(256)
ln_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
               const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ w, float eps,
               int64_t T, int H, int vocab, __nv_bfloat16* __restrict__ x_out,
               __nv_bfloat16* __restrict__ y, int* status) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (row >= T) return;
  const int nvec = H >> 3;
  int64_t src_row = row;
  if (MODE == 2) {
    int64_t id = ids[row];
    if (id < 0 || id >= vocab) {
      if (lane == 0) set_status(status, ST_BAD_TOKEN_ID);
      id = 0;
    }
    src_row = id;
  }
  const uint4* xr = reinterpret_cast<const uint4*>(x + src_row * H);
  const uint4* rr = (MODE == 1) ? reinterpret_cast<const uint4*>(res + row * H) : nullptr;
  float v[VPL][8];
  float sum = 0.f, sq = 0.f;
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      unpack8(MODE == 2 ? __ldg(xr + c) : ld_stream(xr + c), v[i]);
      if (MODE == 1) {
        float r[8];
        unpack8(ld_stream(rr + c), r);
#pragma unroll
        for (int e = 0; e < 8; ++e)
          v[i][e] = __bfloat162float(__float2bfloat16_rn(v[i][e] + r[e]));
        if (x_out != nullptr) reinterpret_cast<uint4*>(x_out + row * H)[c] = pack8(v[i]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        sum += v[i][e];
        sq += v[i][e] * v[i][e];
      }
    }
  }
  if (y == nullptr) return;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
    sq += __shfl_xor_sync(0xffffffffu, sq, o);
  }
  const float mean = sum / float(H);
  const float var = sq / float(H) - mean * mean;
  const float rstd = rsqrtf(var + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      float wv[8], o[8];
      unpack8(__ldg(wr + c), wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = (v[i][e] - mean) * rstd * wv[e];
      reinterpret_cast<uint4*>(y + row * H)[c] = pack8(o);
    }
  }
}

// Plain LayerNorm with two rows per warp: a row of H = 768 is only 1.5 KB, and with one row per
// warp too few bytes are in flight per SM to cover the DRAM latency (72 % of the copy bandwidth);
// loading both rows before reducing either doubles the bytes in flight.  Same arithmetic per row
// as ln_rows_kernel.
template <int VPL>
__global__ void __launch_bounds__(256)
ln2_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, float eps,
                int64_t T, int H, __nv_bfloat16* __restrict__ y) {
  const int lane = threadIdx.x & 31;
  const int64_t row0 = ((int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5) * 2;
  if (row0 >= T) return;
  const int nvec = H >> 3;
  const bool two = row0 + 1 < T;
  uint4 raw[2][VPL];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (row0 + ((r == 1 && two) ? 1 : 0)) * H);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) raw[r][i] = ld_stream(xr + c);
    }
  }
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (r == 1 && !two) break;
    float v[VPL][8];
    float sum = 0.f, sq = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = lane + 32 * i;
      if (c < nvec) {
        unpack8(raw[r][i], v[i]);
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
      if (c < nvec) {
        float wv[8], o[8];
        unpack8(__ldg(wr + c), wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (v[i][e] - mean) * rstd * wv[e];
        reinterpret_cast<uint4*>(y + (row0 + r) * H)[c] = pack8(o);
      }
    }
  }
}

template <int MODE>
static int ln_launch(const void* x, const void* res, const int64_t* ids, const void* w, float eps,
                     int64_t T, int H, int vocab, void* x_out, void* y, int* status,
                     cudaStream_t st) {
  PE_REQUIRE(H > 0 && H % 8 == 0 && H <= 2048, "layer norm: H=%d must be a multiple of 8, <= 2048",
             H);
  if (T == 0) return PE_OK;
  const int threads = 256;  // 8 rows per block
  const int64_t blocks = (T * 32 + threads - 1) / threads;
  const int vpl = (H / 8 + 31) / 32;
  if (MODE == 0 && vpl <= 4) {  // plain LayerNorm of a narrow row: two rows per warp
    const int64_t blocks2 = ((T + 1) / 2 * 32 + threads - 1) / threads;
    const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
    const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(w);
    __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y);
    switch (vpl) {
      case 1: ln2_rows_kernel<1><<<(unsigned)blocks2, threads, 0, st>>>(xp, wp, eps, T, H, yp); break;
      case 2: ln2_rows_kernel<2><<<(unsigned)blocks2, threads, 0, st>>>(xp, wp, eps, T, H, yp); break;
      case 3: ln2_rows_kernel<3><<<(unsigned)blocks2, threads, 0, st>>>(xp, wp, eps, T, H, yp); break;
      default: ln2_rows_kernel<4><<<(unsigned)blocks2, threads, 0, st>>>(xp, wp, eps, T, H, yp); break;
    }
    PE_LAUNCH_CHECK("ln2_rows_kernel");
    return PE_OK;
  }
#define PE_LN_CASE(V)                                                                         \
  case V:                                                                                     \
    ln_rows_kernel<V, MODE><<<(unsigned)blocks, threads, 0, st>>>(                            \
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(res), ids,    \
        static_cast<const __nv_bfloat16*>(w), eps, T, H, vocab,                               \
        static_cast<__nv_bfloat16*>(x_out), static_cast<__nv_bfloat16*>(y), status);          \
    break;
  switch (vpl) {
    PE_LN_CASE(1) PE_LN_CASE(2) PE_LN_CASE(3) PE_LN_CASE(4) PE_LN_CASE(5) PE_LN_CASE(6)
    PE_LN_CASE(7) PE_LN_CASE(8)
    default:
      set_last_error("layer norm: unsupported H=%d", H);
      return PE_ERR_ARG;
  }
#undef PE_LN_CASE
  PE_LAUNCH_CHECK("ln_rows_kernel");
  return PE_OK;
}

// ------------------------------------------------------------------------------
// RoPE table and in-place rotation of q, k inside the fused qkv
// ------------------------------------------------------------------------------
__global__ void rope_table_kernel(float theta, int max_positions, __nv_bfloat16* __restrict__ t) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= max_positions * 32) return;
  const int p = i >> 5, f = i & 31;
  const float inv_freq = 1.0f / powf(theta, float(2 * f) / 64.0f);
  const float ang = float(p) * inv_freq;
  t[size_t(p) * 64 + f] = __float2bfloat16_rn(cosf(ang));
  t[size_t(p) * 64 + 32 + f] = __float2bfloat16_rn(sinf(ang));
}

// One thread rotates 8 (low, high) pairs of one head: dims [8c, 8c+8) and [32+8c, 40+8c).
__global__ void __launch_bounds__(256)
rope_qk_kernel(__nv_bfloat16* __restrict__ qkv, const int64_t* __restrict__ pos,
               const __nv_bfloat16* __restrict__ table, int max_positions, int64_t T, int nh,
               int* status) {
  const int items_per_tok = nh * 8;  // (q|k) x head x 4 chunks
  const int64_t total = T * items_per_tok;
  const int64_t gid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= total) return;
  const int64_t t = gid / items_per_tok;
  const int r = int(gid - t * items_per_tok);
  const int qk = r / (nh * 4);
  const int head = (r >> 2) % nh;
  const int chunk = r & 3;
  int64_t p = pos[t];
  if (p < 0 || p >= max_positions) {
    set_status(status, ST_BAD_POSITION);
    p = 0;
  }
  const int H = nh * 64;
  __nv_bfloat16* base = qkv + t * (3 * int64_t(H)) + qk * H + head * 64 + chunk * 8;
  float lo[8], hi[8], c[8], s[8];
  unpack8(*reinterpret_cast<const uint4*>(base), lo);
  unpack8(*reinterpret_cast<const uint4*>(base + 32), hi);
  const __nv_bfloat16* trow = table + p * 64 + chunk * 8;
  unpack8(__ldg(reinterpret_cast<const uint4*>(trow)), c);
  unpack8(__ldg(reinterpret_cast<const uint4*>(trow + 32)), s);
  float olo[8], ohi[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) rope_pair(lo[e], hi[e], c[e], s[e], olo[e], ohi[e]);
  *reinterpret_cast<uint4*>(base) = pack8(olo);
  *reinterpret_cast<uint4*>(base + 32) = pack8(ohi);
}

// ------------------------------------------------------------------------------
// GeGLU
// ------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
geglu_kernel(const __nv_bfloat16* __restrict__ proj, int64_t T, int I,
             __nv_bfloat16* __restrict__ out) {
  const int vec_per_row = I >> 3;
  const int64_t total = T * vec_per_row;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t t = i / vec_per_row;
    const int c = int(i - t * vec_per_row);
    const uint4* row = reinterpret_cast<const uint4*>(proj + t * 2 * int64_t(I));
    float a[8], g[8], o[8];
    unpack8(ld_stream(row + c), a);
    unpack8(ld_stream(row + vec_per_row + c), g);
#pragma unroll
    for (int e = 0; e < 8; ++e)
      o[e] = gelu_erf(a[e]) * g[e];
    reinterpret_cast<uint4*>(out)[i] = pack8(o);
  }
}

}  // namespace pe

// =============================== C ABI ===========================================
using namespace pe;

extern "C" int pe_unpad_build(const void* mask, int mask_elt_bytes, int B, int S,
                              int32_t* seqlens, int32_t* cu_seqlens, int64_t* indices,
                              int64_t* position_ids, int32_t* totals_dev, int32_t* totals_host,
                              void* stream) {
  PE_REQUIRE(mask && seqlens && cu_seqlens && indices && position_ids && totals_dev,
             "pe_unpad_build: null pointer");
  PE_REQUIRE(B > 0 && S > 0 && int64_t(B) * S < (1ll << 31), "pe_unpad_build: bad B=%d S=%d", B, S);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc;
  switch (mask_elt_bytes) {
    case 1: rc = unpad_launch<uint8_t>(mask, B, S, seqlens, cu_seqlens, indices, position_ids, totals_dev, st); break;
    case 4: rc = unpad_launch<int32_t>(mask, B, S, seqlens, cu_seqlens, indices, position_ids, totals_dev, st); break;
    case 8: rc = unpad_launch<int64_t>(mask, B, S, seqlens, cu_seqlens, indices, position_ids, totals_dev, st); break;
    default:
      set_last_error("pe_unpad_build: mask element width %d not in {1,4,8}", mask_elt_bytes);
      return PE_ERR_ARG;
  }
  if (rc != PE_OK) return rc;
  if (totals_host != nullptr) {
    PE_CUDA(cudaMemcpyAsync(totals_host, totals_dev, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    PE_CUDA(cudaStreamSynchronize(st));
  }
  return PE_OK;
}

static int gather_rows_launch(const void* src, const int64_t* indices, int64_t T,
                              const int32_t* count_dev, int64_t row_bytes, void* dst, void* stream,
                              const char* who) {
  PE_REQUIRE(src && indices && dst, "%s: null pointer", who);
  PE_REQUIRE(T >= 0 && row_bytes > 0, "%s: bad sizes", who);
  if (T == 0) return PE_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int vb = pick_vec_bytes(src, dst, row_bytes);
  const int64_t vpr = row_bytes / vb;
  PE_REQUIRE(vpr < (1ll << 30), "%s: row too wide", who);
  const int64_t total = T * vpr;
  const int threads = 256;
  const unsigned blocks = (unsigned)std::min<int64_t>((total + threads - 1) / threads, (int64_t)sm_count() * 32);
  switch (vb) {
    case 16: gather_rows_kernel<uint4><<<blocks, threads, 0, st>>>((const uint4*)src, indices, T, count_dev, (int)vpr, (uint4*)dst); break;
    case 8: gather_rows_kernel<uint2><<<blocks, threads, 0, st>>>((const uint2*)src, indices, T, count_dev, (int)vpr, (uint2*)dst); break;
    case 4: gather_rows_kernel<uint32_t><<<blocks, threads, 0, st>>>((const uint32_t*)src, indices, T, count_dev, (int)vpr, (uint32_t*)dst); break;
    case 2: gather_rows_kernel<uint16_t><<<blocks, threads, 0, st>>>((const uint16_t*)src, indices, T, count_dev, (int)vpr, (uint16_t*)dst); break;
    default: gather_rows_kernel<uint8_t><<<blocks, threads, 0, st>>>((const uint8_t*)src, indices, T, count_dev, (int)vpr, (uint8_t*)dst); break;
  }
  PE_LAUNCH_CHECK("gather_rows_kernel");
  return PE_OK;
}

static int repad_launch(const void* packed, const int64_t* indices, int64_t T, const int32_t* count_dev,
                        int64_t rows_out, int64_t row_bytes, void* out, void* stream, const char* who) {
  PE_REQUIRE(out && (T == 0 || (packed && indices)), "%s: null pointer", who);
  PE_REQUIRE(T >= 0 && rows_out >= 0 && row_bytes > 0, "%s: bad sizes", who);
  if (rows_out == 0) return PE_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int vb = pick_vec_bytes(packed ? packed : out, out, row_bytes);
  const int64_t vpr = row_bytes / vb;
  PE_REQUIRE(vpr < (1ll << 30), "%s: row too wide", who);
  const int threads = 256;
  const int lanes = (int)std::min<int64_t>(vpr, 32);
  const int rows_per_block = threads / lanes;
  const unsigned blocks =
      (unsigned)std::min<int64_t>((rows_out + rows_per_block - 1) / rows_per_block, (int64_t)sm_count() * 64);
  switch (vb) {
    case 16: repad_kernel<uint4><<<blocks, threads, 0, st>>>((const uint4*)packed, indices, T, count_dev, rows_out, (int)vpr, (uint4*)out); break;
    case 8: repad_kernel<uint2><<<blocks, threads, 0, st>>>((const uint2*)packed, indices, T, count_dev, rows_out, (int)vpr, (uint2*)out); break;
    case 4: repad_kernel<uint32_t><<<blocks, threads, 0, st>>>((const uint32_t*)packed, indices, T, count_dev, rows_out, (int)vpr, (uint32_t*)out); break;
    case 2: repad_kernel<uint16_t><<<blocks, threads, 0, st>>>((const uint16_t*)packed, indices, T, count_dev, rows_out, (int)vpr, (uint16_t*)out); break;
    default: repad_kernel<uint8_t><<<blocks, threads, 0, st>>>((const uint8_t*)packed, indices, T, count_dev, rows_out, (int)vpr, (uint8_t*)out); break;
  }
  PE_LAUNCH_CHECK("repad_kernel");
  return PE_OK;
}

extern "C" int pe_gather_rows(const void* src, const int64_t* indices, int64_t T, int64_t row_bytes,
                              void* dst, void* stream) {
  return gather_rows_launch(src, indices, T, nullptr, row_bytes, dst, stream, "pe_gather_rows");
}

extern "C" int pe_gather_rows_counted(const void* src, const int64_t* indices, const int32_t* count_dev,
                                      int64_t capacity, int64_t row_bytes, void* dst, void* stream) {
  PE_REQUIRE(count_dev != nullptr, "pe_gather_rows_counted: count_dev is NULL");
  return gather_rows_launch(src, indices, capacity, count_dev, row_bytes, dst, stream,
                            "pe_gather_rows_counted");
}

extern "C" int pe_repad_scatter(const void* packed, const int64_t* indices, int64_t T,
                                int64_t rows_out, int64_t row_bytes, void* out, void* stream) {
  return repad_launch(packed, indices, T, nullptr, rows_out, row_bytes, out, stream, "pe_repad_scatter");
}

extern "C" int pe_repad_scatter_counted(const void* packed, const int64_t* indices,
                                        const int32_t* count_dev, int64_t capacity, int64_t rows_out,
                                        int64_t row_bytes, void* out, void* stream) {
  PE_REQUIRE(count_dev != nullptr, "pe_repad_scatter_counted: count_dev is NULL");
  return repad_launch(packed, indices, capacity, count_dev, rows_out, row_bytes, out, stream,
                      "pe_repad_scatter_counted");
}

extern "C" int pe_rope_table(float theta, int max_positions, void* table, void* stream) {
  PE_REQUIRE(table && max_positions > 0 && theta > 0.f, "pe_rope_table: bad argument");
  const int total = max_positions * 32;
  rope_table_kernel<<<(total + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      theta, max_positions, static_cast<__nv_bfloat16*>(table));
  PE_LAUNCH_CHECK("rope_table_kernel");
  return PE_OK;
}

extern "C" int pe_embed_ln(const int64_t* ids, const void* tok_emb, const void* w, float eps,
                           int64_t T, int H, int vocab, void* out, int32_t* status, void* stream) {
  PE_REQUIRE(ids && tok_emb && w && out, "pe_embed_ln: null pointer");
  return ln_launch<2>(tok_emb, nullptr, ids, w, eps, T, H, vocab, nullptr, out, status,
                      static_cast<cudaStream_t>(stream));
}

extern "C" int pe_add_ln(const void* x, const void* res, const void* w, float eps, int64_t T, int H,
                         void* x_out, void* y, void* stream) {
  PE_REQUIRE(x && (y || x_out), "pe_add_ln: null pointer");
  PE_REQUIRE(y == nullptr || w != nullptr, "pe_add_ln: weight is NULL");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (res == nullptr)
    return ln_launch<0>(x, nullptr, nullptr, w, eps, T, H, 0, nullptr, y, nullptr, st);
  return ln_launch<1>(x, res, nullptr, w, eps, T, H, 0, x_out, y, nullptr, st);
}

extern "C" int pe_rope_qk_inplace(void* qkv, const int64_t* position_ids, const void* table,
                                  int max_positions, int64_t T, int nh, int32_t* status,
                                  void* stream) {
  PE_REQUIRE(qkv && position_ids && table, "pe_rope_qk_inplace: null pointer");
  PE_REQUIRE(nh > 0 && max_positions > 0, "pe_rope_qk_inplace: bad sizes");
  if (T == 0) return PE_OK;
  const int64_t total = T * nh * 8;
  const int threads = 256;
  rope_qk_kernel<<<(unsigned)((total + threads - 1) / threads), threads, 0,
                   static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(qkv), position_ids, static_cast<const __nv_bfloat16*>(table),
      max_positions, T, nh, status);
  PE_LAUNCH_CHECK("rope_qk_kernel");
  return PE_OK;
}

extern "C" int pe_geglu(const void* proj, int64_t T, int I, void* out, void* stream) {
  PE_REQUIRE(proj && out, "pe_geglu: null pointer");
  PE_REQUIRE(I > 0 && I % 8 == 0, "pe_geglu: I=%d must be a multiple of 8", I);
  if (T == 0) return PE_OK;
  const int64_t total = T * (I / 8);
  const int threads = 256;
  const unsigned blocks = (unsigned)std::min<int64_t>((total + threads - 1) / threads, (int64_t)sm_count() * 64);
  geglu_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(proj), T, I, static_cast<__nv_bfloat16*>(out));
  PE_LAUNCH_CHECK("geglu_kernel");
  return PE_OK;
}
