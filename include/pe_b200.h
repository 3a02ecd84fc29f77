/*
 * pe_b200.h -- C ABI of the B200 (sm_100a) packed ModernBERT inference forward.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed
 * as void*, a cudaStream_t), returns 0 on success or a negative PE_ERR_* code,
 * never throws, never allocates device memory (scratch is passed in by the
 * caller) and never synchronises the stream, except pe_unpad_build when asked
 * for a host read-back and pe_read_status.  All kernels are enqueued on the
 * stream given, so a caller that is capturing that stream into a CUDA graph
 * captures them.
 *
 * Each declaration names the function of pau-mensa/flash-modernbert
 * (package `packed_encoders`) whose work it takes over, as file:line.
 *
 * Device status word (the `status` arguments): a kernel that has to give up writes the first
 * such code there and carries on without touching memory it should not; 0 means none did.
 * 101-103: a bounded wait inside a GEMM ran out; 201-204: inside an attention kernel;
 * 301: token id outside the vocabulary (row 0 was used); 302: position outside the RoPE table
 * (position 0 was used); 303: a cu_seqlens entry outside [0, T] or smaller than its predecessor
 * (clamped into range: no kernel follows a boundary outside the caller's buffers).
 *
 * Inputs are expected to be finite.  The attention kernels fetch whole key/value tiles and mask
 * the scores of keys outside a sequence to zero probability, so a NaN or Inf in one sequence's
 * values can reach the rows of the sequences packed next to it (0 * NaN).  pe_forward_packed
 * keeps the padding rows of a graph bucket finite by itself.
 *
 * Tensors are row-major and contiguous unless a stride is named.  "bf16" is
 * __nv_bfloat16.  T = packed tokens, N = sequences, H = hidden size,
 * nh = heads, D = head dim (64 only), I = GeGLU intermediate size.
 */
#ifndef PE_B200_H
#define PE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PE_OK 0
#define PE_ERR_ARG (-1)        /* bad argument (null pointer, unsupported size) */
#define PE_ERR_CUDA (-2)       /* a CUDA runtime/driver call failed; see pe_last_error */
#define PE_ERR_WORKSPACE (-3)  /* workspace too small */
#define PE_ERR_DEVICE (-4)     /* a kernel recorded a fault in the status word */
#define PE_ERR_UNSUPPORTED (-5)/* not an sm_100 device, or shape outside the kernels' envelope */

/* Per-layer weights, HF ModernBERT layout, all bf16, never copied or re-laid out
 * (packed_encoders/pack.py:3-6).  attn_norm_w is NULL where the layer's attn_norm
 * is nn.Identity (layer 0, packed_encoders/forward.py:178-183). */
typedef struct pe_layer_weights {
  const void* attn_norm_w; /* [H] or NULL */
  const void* wqkv;        /* [3H, H]  rows q|k|v, each nh x D */
  const void* wo;          /* [H, H] */
  const void* mlp_norm_w;  /* [H] */
  const void* wi;          /* [2I, H]  rows 0..I-1 gelu input, I..2I-1 gate */
  const void* wo_mlp;      /* [H, I] */
  int32_t is_global;       /* 1: full attention + global RoPE table; 0: sliding window + local table */
  int32_t reserved;
} pe_layer_weights;

/* The slice of the model the forward reads (packed_encoders/config.py:17-67). */
typedef struct pe_model {
  int32_t hidden;        /* H, multiple of 64, <= 2048 */
  int32_t n_heads;       /* nh, H == nh * 64 */
  int32_t head_dim;      /* 64 */
  int32_t intermediate;  /* I, multiple of 8 */
  int32_t n_layers;
  int32_t vocab;
  int32_t half_window;   /* local_attention / 2 (64) */
  int32_t max_positions; /* rows of the two RoPE tables */
  float eps;
  float reserved;
  const void* tok_emb;      /* bf16 [vocab, H] */
  const void* emb_norm_w;   /* bf16 [H] */
  const void* final_norm_w; /* bf16 [H] */
  const void* rope_global;  /* bf16 [max_positions, 64] from pe_rope_table(theta_global) */
  const void* rope_local;   /* bf16 [max_positions, 64] from pe_rope_table(theta_local) */
  const pe_layer_weights* layers; /* host array of n_layers entries */
} pe_model;

/* Library version (major*10000 + minor*100 + patch). */
int pe_version(void);
/* Text of the most recent PE_ERR_CUDA / PE_ERR_ARG on the calling thread. */
const char* pe_last_error(void);
/* 0 if the current device is sm_100 and the TMA descriptor entry point resolves. */
int pe_device_check(void);
/* Process-wide switch. key 1 (PE_OPT_FUSED_GEGLU, default 1): pe_forward_packed runs Wi and
 * GeGLU as one kernel (1) or as pe_gemm_bf16_tn followed by pe_geglu (0). */
#define PE_OPT_FUSED_GEGLU 1
/* key 2 (PE_OPT_FUSED_ROPE, default 1): Wqkv and RoPE as one kernel (1) or as pe_gemm_bf16_tn
 * followed by pe_rope_qk_inplace (0). */
#define PE_OPT_FUSED_ROPE 2
/* key 3 (PE_OPT_GEMM_PAIR, default 1): every GEMM with more than 256 rows runs on pairs of CTAs
 * sharing 256 x 256 tiles (1), or on single CTAs with 128 x 256 tiles (0).  Same results. */
#define PE_OPT_GEMM_PAIR 3
/* key 4 (PE_OPT_FUSED_RESIDUAL, default 1): Wo and the MLP's Wo add their result to the residual
 * stream in the GEMM epilogue and the norms run as plain LayerNorms (1), or the projections are
 * materialised and pe_add_ln adds them (0). */
#define PE_OPT_FUSED_RESIDUAL 4
/* A forward reads the switches once, when it starts to enqueue its kernels. */
int pe_set_option(int key, int value);

/* ---- padding boundary ------------------------------------------------------ */

/* packed_encoders/forward.py:384-403 (_unpad) and benchmarks/helpers/packed_collator.py:68-96.
 * mask: [B, S] of mask_elt_bytes-wide integers (1, 4 or 8), non-zero = real token.
 * Writes seqlens int32[B], cu_seqlens int32[B+1], indices int64[T] (row-major flat
 * positions of the non-zero mask entries, ascending), position_ids int64[T]
 * (= indices % S) and totals_dev int32[2] = {T, max_seqlen}.  indices/position_ids
 * must have room for B*S entries.  If totals_host is non-NULL the call copies
 * totals_dev there and synchronises the stream (the reference's int(seqlens.max())
 * host sync). */
int pe_unpad_build(const void* mask, int mask_elt_bytes, int B, int S,
                   int32_t* seqlens, int32_t* cu_seqlens, int64_t* indices,
                   int64_t* position_ids, int32_t* totals_dev, int32_t* totals_host,
                   void* stream);

/* x.reshape(B*S, -1).index_select(0, indices) of packed_encoders/forward.py:401:
 * dst[t, :] = src[indices[t], :], rows of row_bytes bytes. */
int pe_gather_rows(const void* src, const int64_t* indices, int64_t T, int64_t row_bytes,
                   void* dst, void* stream);

/* packed_encoders/forward.py:406-412 (_repad): out[B*S rows] = 0 except
 * out[indices[t]] = packed[t].  indices must be ascending (as pe_unpad_build
 * writes them); every output row is written exactly once. */
int pe_repad_scatter(const void* packed, const int64_t* indices, int64_t T, int64_t rows_out,
                     int64_t row_bytes, void* out, void* stream);

/* pe_gather_rows and pe_repad_scatter for a caller that has not read the row count back to the
 * host: the padded API inside a captured CUDA graph, where pe_unpad_build (totals_host = NULL)
 * leaves T in totals_dev[0] and the synchronising read of packed_encoders/forward.py:397-402
 * (int(seqlens.max())) would end the capture.  The count is read on the device from *count_dev
 * and clamped to `capacity` (the rows the buffers hold).  Gather: rows at or beyond the count are
 * written as zeros, their indices are not read.  Scatter: only indices[0 .. count) are searched. */
int pe_gather_rows_counted(const void* src, const int64_t* indices, const int32_t* count_dev,
                           int64_t capacity, int64_t row_bytes, void* dst, void* stream);
int pe_repad_scatter_counted(const void* packed, const int64_t* indices, const int32_t* count_dev,
                             int64_t capacity, int64_t rows_out, int64_t row_bytes, void* out,
                             void* stream);

/* ---- tails (memory-bound) -------------------------------------------------- */

/* packed_encoders/forward.py:40-51 (_rope_tables): row p of table holds
 * bf16(cos(p * f_i)) for i in 0..31 then bf16(sin(p * f_i)), f_i = theta^(-2i/64),
 * angles and cos/sin in fp32. table: bf16 [max_positions, 64]. */
int pe_rope_table(float theta, int max_positions, void* table, void* stream);

/* packed_encoders/forward.py:472-476: out[t] = LayerNorm(tok_emb[ids[t]]) * w
 * (no bias, fp32 statistics with var = E[x^2] - mean^2, bf16 out). */
int pe_embed_ln(const int64_t* ids, const void* tok_emb, const void* w, float eps,
                int64_t T, int H, int vocab, void* out, int32_t* status, void* stream);

/* packed_encoders/ops.py:303-314 and 191-208, kernel
 * packed_encoders/_kernels/triton_layer_norm.py:26-59.
 * x_new = bf16(x + res); y = LayerNorm(x_new) * w.  res == NULL: plain LayerNorm of x.
 * x_out may be NULL (x_new not kept) or alias x (in place).  y may be NULL only if
 * x_out is not. */
int pe_add_ln(const void* x, const void* res, const void* w, float eps, int64_t T, int H,
              void* x_out, void* y, void* stream);

/* packed_encoders/_kernels/rope.py:142-218 (BSHD RoPE on the fused qkv), in place:
 * rotates the q and k thirds of qkv [T, 3*nh*64] by the table row position_ids[t];
 * v is untouched.  Split-half pairing (j, j+32), fp32 math on bf16 inputs. */
int pe_rope_qk_inplace(void* qkv, const int64_t* position_ids, const void* table,
                       int max_positions, int64_t T, int nh, int32_t* status, void* stream);

/* packed_encoders/ops.py:275-280, kernel packed_encoders/_kernels/triton_layer_norm.py:62-79:
 * out[t, i] = gelu_erf(proj[t, i]) * proj[t, I + i]. */
int pe_geglu(const void* proj, int64_t T, int I, void* out, void* stream);

/* ---- GEMM (tensor-bound) --------------------------------------------------- */

/* packed_encoders/ops.py:290-300 (_linear -> cuBLAS on sm_100): C = A * W^T with
 * A bf16 [M, K], W bf16 [Nout, K] (nn.Linear.weight), C bf16 [M, Nout], fp32
 * accumulation in tensor memory.  K % 8 == 0, Nout % 8 == 0, pointers 16-byte aligned. */
int pe_gemm_bf16_tn(const void* A, const void* W, void* C, int64_t M, int Nout, int K,
                    int32_t* status, void* stream);

/* geglu_mlp's first half (packed_encoders/ops.py:317-319) in one kernel:
 * out[t, i] = gelu_erf(bf16(A W_a^T)[t, i]) * bf16(A W_g^T)[t, i], W_a = Wi[0:I], W_g = Wi[I:2I].
 * The [T, 2I] projection is rounded to bf16 as the reference materialises it, but
 * never written to memory. */
int pe_gemm_geglu_bf16(const void* A, const void* Wi, void* out, int64_t M, int I, int K,
                       int32_t* status, void* stream);

/* The Wqkv projection (packed_encoders/forward.py:191) and the RoPE that follows it
 * (packed_encoders/ops.py:496) in one kernel: qkv = A Wqkv^T rounded to bf16, then the q and k
 * heads rotated by table[position_ids[row]] in the epilogue; v columns are stored as they are.
 * qkv: bf16 [M, 3*nh*64]. Same bits as pe_gemm_bf16_tn followed by pe_rope_qk_inplace. */
int pe_gemm_qkv_rope_bf16(const void* A, const void* Wqkv, void* qkv, int64_t M, int nh, int K,
                          const int64_t* position_ids, const void* table, int max_positions,
                          int32_t* status, void* stream);

/* A projection and the residual add that follows it in one kernel:
 * C = bf16(X + bf16(A W^T)), the value packed_encoders/ops.py:303-314 computes as x_new from the
 * materialised projection (packed_encoders/forward.py:216-220 and the deferred MLP residual,
 * 221-225).  X, C: bf16 [M, Nout]; C may be X (in place: the kernel then never reads X, it adds
 * its rounded product to it with TMA reduce-adds; out of place X is first copied to C on the
 * stream). */
int pe_gemm_residual_bf16(const void* A, const void* W, const void* X, void* C, int64_t M, int Nout,
                          int K, int32_t* status, void* stream);

/* Projection head with per-token L2 normalisation, in one kernel
 * (benchmarks/helpers/packed_index.py:182-186 of the reference: the ColBERT Dense projection of
 * the token embeddings followed by F.normalize(p=2, dim=-1)):
 * C[m, :] = y / max(bf16(||y||_2), 1e-12) with y = bf16(A[m, :] W^T), rounded to bf16.
 * A: bf16 [M, K]; W: bf16 [Nout, K] (nn.Linear layout, no bias); C: bf16 [M, Nout];
 * Nout <= 256 (a tile then holds whole rows), Nout and K multiples of 8. */
int pe_gemm_l2norm_bf16(const void* A, const void* W, void* C, int64_t M, int Nout, int K,
                        int32_t* status, void* stream);

/* ---- pooling head on the packed output ---------------------------------------- */

/* Bytes of workspace pe_pool_packed needs for mean pooling (mode 1); mode 0 needs none. */
size_t pe_pool_workspace_bytes(int64_t T, int n_seqs, int H);

/* benchmarks/showcases/inference.py:193-206 (what the reference's callers do with the output of
 * packed_forward): per sequence, the fp32 sum of its token rows divided by its length (mode 1)
 * or its first token's row (mode 0); normalize != 0 divides by max(||x||_2, 1e-12) as
 * F.normalize does; the result is rounded to bf16 last.
 * hidden: bf16 [T, H]; cu_seqlens: int32 [n_seqs + 1]; out: bf16 [n_seqs, H]; zero-length
 * sequences give zero rows.  H a multiple of 8, at most 2048.  Summation order is fixed
 * (no atomics): repeated calls are bit-identical. */
int pe_pool_packed(const void* hidden, const int32_t* cu_seqlens, int n_seqs, int64_t T, int H,
                   int mode, int normalize, void* out, void* workspace, size_t workspace_bytes,
                   void* stream);

/* ---- attention -------------------------------------------------------------- */

/* Bytes of scratch pe_attn_varlen needs for n_seqs sequences and T tokens. */
size_t pe_attn_workspace_bytes(int64_t T, int n_seqs);

/* packed_encoders/ops.py:485-532 (flash_attn_varlen_func call) and
 * packed_encoders/_kernels/triton_packed_attention.py:45-143: per sequence and head,
 * softmax(q k^T / 8 + mask) v, non-causal, no attention across cu_seqlens
 * boundaries.  half_window < 0: full attention; else keys with |i-j| <= half_window.
 * qkv: bf16 [T, 3*nh*64] with q and k already rotated; out: bf16 [T, nh*64].
 * n_seqs may include trailing zero-length sequences (cu_seqlens repeats T). */
int pe_attn_varlen(const void* qkv, const int32_t* cu_seqlens, int n_seqs, int64_t T, int nh,
                   int half_window, int max_seqlen, void* out, void* workspace,
                   size_t workspace_bytes, int32_t* status, void* stream);

/* pe_attn_varlen for callers that must not allocate device memory and have none to lend: a
 * plug-in hosted by a process whose own allocator already holds the whole GPU, or a serving
 * thread with a frozen memory budget that may not call cudaMalloc (which can stall the device)
 * on its request path.  No counterpart in the reference.  The tile table lives in a 1.2 MB
 * array inside the library (every GPU that loads the library holds it until exit), so the
 * call takes no workspace and calls no allocator.  Limits: n_seqs <= 4096 and T <= 1,048,576,
 * beyond which it returns PE_ERR_WORKSPACE.  The first call on each device looks the array's
 * address up once; make that call outside any stream capture.  All calls share the one array:
 * each call rebuilds the part it reads, so nothing needs clearing, but two calls whose kernels
 * may overlap on the GPU (different streams) race on it - keep them on one stream. */
int pe_attn_varlen_static(const void* qkv, const int32_t* cu_seqlens, int n_seqs, int64_t T,
                          int nh, int half_window, int max_seqlen, void* out, int32_t* status,
                          void* stream);

/* ---- whole forward ---------------------------------------------------------- */

/* Scratch bytes for pe_forward_packed at a capacity of T tokens and n_seqs sequences. */
size_t pe_forward_workspace_bytes(const pe_model* model, int64_t T, int n_seqs);

/* packed_encoders/forward.py:415-516 (packed_forward) with core 229-277 and
 * _encoder_layer 161-226: ids int64[T], cu_seqlens int32[n_seqs+1], position_ids
 * int64[T] -> out bf16 [T, H] (last hidden state after final_norm).  Tokens at or
 * beyond cu_seqlens[n_seqs] (graph-bucket padding) run through the GEMMs and
 * tails but attend to nothing, as in packed_encoders/graph.py:244-248.
 * status: device int32, must be zero on entry; a kernel that gives up on a bounded
 * wait or meets an out-of-range id / position / boundary writes a non-zero code there. */
int pe_forward_packed(const pe_model* model, const int64_t* ids, const int32_t* cu_seqlens,
                      const int64_t* position_ids, int64_t T, int n_seqs, int max_seqlen,
                      void* workspace, size_t workspace_bytes, void* out, int32_t* status,
                      void* stream);

/* pe_forward_packed with the pooling head fused into the final LayerNorm, for callers that turn
 * the hidden state into one embedding per sequence right away
 * (benchmarks/showcases/inference.py:193-209 of the reference: packed_forward, fp32 segment mean
 * by index_add_, F.normalize).  pooled_out: bf16 [n_seqs, H] = per sequence the first token's row
 * (pool_mode 0) or the fp32 mean of its rows (pool_mode 1) of the bf16 last hidden state, divided
 * by max(||.||_2, 1e-12) if normalize != 0, rounded to bf16 last; zero-length sequences give zero
 * rows.  hidden_out: bf16 [T, H] or NULL; with NULL the hidden state is never written (and with
 * pool_mode 0 the final LayerNorm runs on one row per sequence only).  Same workspace size as
 * pe_forward_packed.  Fixed summation order: repeated calls are bit-identical. */
int pe_forward_packed_pooled(const pe_model* model, const int64_t* ids, const int32_t* cu_seqlens,
                             const int64_t* position_ids, int64_t T, int n_seqs, int max_seqlen,
                             void* workspace, size_t workspace_bytes, int pool_mode, int normalize,
                             void* hidden_out, void* pooled_out, int32_t* status, void* stream);

/* Copies the device status word to the host and synchronises the stream.
 * Returns PE_OK if it is zero, else PE_ERR_DEVICE with *code_out = the word. */
int pe_read_status(const int32_t* status, int32_t* code_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PE_B200_H */
