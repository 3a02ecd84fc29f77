// Host-side helpers shared by the translation units of libpe_b200.so: error
// recording for the C ABI, launch checks, and TMA descriptor construction.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/pe_b200.h"

namespace pe {

void set_last_error(const char* fmt, ...);

// Returns PE_OK or records the CUDA error text and returns PE_ERR_CUDA.
int check_cuda(cudaError_t e, const char* what);

#define PE_CUDA(call)                                  \
  do {                                                 \
    int _rc = ::pe::check_cuda((call), #call);         \
    if (_rc != PE_OK) return _rc;                      \
  } while (0)

#define PE_LAUNCH_CHECK(name) PE_CUDA(cudaGetLastError())

#define PE_REQUIRE(cond, ...)                          \
  do {                                                 \
    if (!(cond)) {                                     \
      ::pe::set_last_error(__VA_ARGS__);               \
      return PE_ERR_ARG;                               \
    }                                                  \
  } while (0)

// Number of SMs of the current device (cached per device).
int sm_count();

// Raises the dynamic shared-memory limit of kernel `func` to `bytes` on the CURRENT device (the
// attribute is per device), once per (kernel, device); `max_carveout` also asks for the largest
// shared-memory carve-out, for kernels that keep two CTAs per SM.
int set_max_dynamic_smem(const void* func, int bytes, bool max_carveout);

// Encodes a 2-D bf16 tensor map: global tensor [rows, cols] with `row_stride_elts`
// between rows, box [box_rows, 64 columns], 128-byte swizzle, zero fill outside.
int make_tmap_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                      uint64_t row_stride_elts, uint32_t box_rows);

// Attention in two steps so that a forward builds the query-tile table once and
// reuses it for every layer (attn_varlen.cu).  `scratch` holds pe_attn_workspace_bytes.
int attn_pick_bm(int max_seqlen);
size_t attn_scratch_bytes(int64_t T, int n_seqs);
// Byte offset of the int4 tile descriptors inside that scratch (tile_start int32[n_seqs + 1] comes first).
size_t attn_info_offset(int n_seqs);
// Boundaries outside [0, T] or running backwards are clamped (never followed) and reported as
// ST_BAD_CU_SEQLENS in `status` (may be NULL); at most T / bm + n_seqs tiles are written.
// `split_short` (attention with bm = 128 only) lists sequences of at most 64 tokens in the second
// table, for the register-tiled kernel; attn_run expects the tables of an attention forward built so.
int attn_schedule(const int32_t* cu_seqlens, int n_seqs, int64_t T, int bm, bool split_short,
                  void* scratch, int32_t* status, cudaStream_t st);
int attn_run(const void* qkv, const void* scratch, int n_seqs, int64_t T, int nh, int half_window,
             int bm, void* out, int32_t* status, cudaStream_t st);
// Full / banded attention with two CTAs per SM and the accumulator in tensor memory.
int attn_run_global_tc(const void* qkv, const int4* tile_info, const int32_t* total_tiles,
                       int64_t max_tiles, int64_t T, int nh, int half_window, void* out,
                       int32_t* status, cudaStream_t st);
// Sliding-window (half window 64) attention with two CTAs per SM, S / P / O in place in tensor memory.
int attn_run_local_tc2(const void* qkv, const int4* tile_info, const int32_t* total_tiles,
                       int64_t max_tiles, int64_t T, int nh, void* out, int32_t* status,
                       cudaStream_t st);

// The final LayerNorm of a forward fused with the pooling head (pool.cu): pooled_out [n_seqs, H] =
// first-token (mode 0) or mean (mode 1) of LayerNorm(x) * w per sequence, optionally L2-normalised;
// hidden_out (may be NULL) also receives the [T, H] normalised rows.  `workspace` as pe_pool_packed.
int final_ln_pool(const void* x, const void* w, float eps, const int32_t* cu_seqlens, int n_seqs,
                  int64_t T, int H, int mode, int normalize, void* hidden_out, void* pooled_out,
                  void* workspace, size_t workspace_bytes, cudaStream_t st);

// Process-wide switches (pe_set_option).
enum Option : int { OPT_FUSED_GEGLU = 1, OPT_FUSED_ROPE = 2, OPT_GEMM_PAIR = 3, OPT_FUSED_RESIDUAL = 4, OPT_COUNT = 5 };
void set_gemm_pair(int on);  // gemm_tcgen05.cu: CTA-pair tiles on (default) or off
int get_option(int key);

}  // namespace pe
