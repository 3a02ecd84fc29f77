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
int attn_schedule(const int32_t* cu_seqlens, int n_seqs, int bm, void* scratch, cudaStream_t st);
int attn_run(const void* qkv, const void* scratch, int n_seqs, int64_t T, int nh, int half_window,
             int bm, void* out, int32_t* status, cudaStream_t st);
// The persistent 128-row tensor-memory kernel (attn_tcgen05.cu); tiles built with bm = 128.
int attn_run_tc(const void* qkv, const int4* tile_info, const int32_t* total_tiles, int64_t max_tiles,
                int64_t T, int nh, int half_window, void* out, int32_t* status, cudaStream_t st);
// Full / banded attention with two CTAs per SM and the accumulator in tensor memory.
int attn_run_global_tc(const void* qkv, const int4* tile_info, const int32_t* total_tiles,
                       int64_t max_tiles, int64_t T, int nh, int half_window, void* out,
                       int32_t* status, cudaStream_t st);
// Sliding-window (half window 64) attention with two CTAs per SM, S / P / O in place in tensor memory.
int attn_run_local_tc2(const void* qkv, const int4* tile_info, const int32_t* total_tiles,
                       int64_t max_tiles, int64_t T, int nh, void* out, int32_t* status,
                       cudaStream_t st);

// Process-wide switches (pe_set_option).
enum Option : int { OPT_FUSED_GEGLU = 1, OPT_FUSED_ROPE = 2, OPT_LOCAL_ATTN_SINGLE_PASS = 3,
                    OPT_FUSED_RESIDUAL = 4, OPT_ATTN_TWO_CTA = 5, OPT_LOCAL_ATTN_TWO_CTA = 6,
                    OPT_COUNT };
int get_option(int key);

}  // namespace pe
