// The whole packed forward as one host call: embedding + LayerNorm, then per layer
// add+LN -> Wqkv -> RoPE -> varlen attention -> Wo -> add+LN -> Wi(+GeGLU) -> Wo_mlp,
// with the MLP residual deferred into the next layer's add+LN, and the final norm.
// All launches go to the caller's stream; the caller owns every buffer.
#include <atomic>

#include "pe_host.h"

namespace pe {

// Read once at the top of a forward, so a switch flipped by another thread never changes the
// op list of a forward that is already being enqueued.
static std::atomic<int> g_options[OPT_COUNT] = {{0}, /*OPT_FUSED_GEGLU*/ {1}, /*OPT_FUSED_ROPE*/ {1},
                                                /*OPT_GEMM_PAIR*/ {1}, /*OPT_FUSED_RESIDUAL*/ {1}};

static bool known_option(int key) {
  return key == OPT_FUSED_GEGLU || key == OPT_FUSED_ROPE || key == OPT_GEMM_PAIR || key == OPT_FUSED_RESIDUAL;
}

int get_option(int key) { return known_option(key) ? g_options[key].load(std::memory_order_relaxed) : 0; }

// Zeroes the rows of `buf` ([T, row_bytes]) at or beyond *first_row_ptr (read on the device, so
// the launch is the same whatever the real token count: graph-safe).
__global__ void zero_tail_rows_kernel(uint8_t* __restrict__ buf, const int32_t* __restrict__ first_row_ptr,
                                      int T, int row_bytes) {
  const int first = min(max(*first_row_ptr, 0), T);
  const size_t begin = size_t(first) * row_bytes, end = size_t(T) * row_bytes;  // multiples of 16
  for (size_t i = begin + (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * 16; i < end;
       i += size_t(gridDim.x) * blockDim.x * 16)
    *reinterpret_cast<uint4*>(buf + i) = make_uint4(0u, 0u, 0u, 0u);
}

static size_t align_up(size_t v) { return (v + 255) & ~size_t(255); }

struct Workspace {
  size_t x, normed, qkv, ctx, tmp, act, proj, tiles, pool, total;
};

static Workspace plan(const pe_model* m, int64_t T, int n_seqs) {
  Workspace w;
  const size_t H = (size_t)m->hidden, I = (size_t)m->intermediate;
  const size_t rows = (size_t)(T > 0 ? T : 1);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off += align_up(bytes);
    return o;
  };
  w.x = take(rows * H * 2);
  w.normed = take(rows * H * 2);
  w.qkv = take(rows * 3 * H * 2);
  w.ctx = take(rows * H * 2);
  w.tmp = take(rows * H * 2);
  w.act = take(rows * I * 2);
  w.proj = take(rows * 2 * I * 2);  // used only when the fused Wi+GeGLU kernel is switched off
  w.tiles = take(pe_attn_workspace_bytes(T, n_seqs));
  w.pool = take(pe_pool_workspace_bytes(T, n_seqs, m->hidden));  // fused final norm + mean pooling
  w.total = off;
  return w;
}

static int check_model(const pe_model* m) {
  PE_REQUIRE(m != nullptr, "model is NULL");
  PE_REQUIRE(m->head_dim == 64, "head_dim=%d: only 64 is supported", m->head_dim);
  PE_REQUIRE(m->hidden > 0 && m->hidden == m->n_heads * 64 && m->hidden <= 2048,
             "hidden=%d must equal n_heads*64 and be <= 2048", m->hidden);
  PE_REQUIRE(m->intermediate > 0 && m->intermediate % 8 == 0, "intermediate=%d must be a multiple of 8",
             m->intermediate);
  PE_REQUIRE(m->n_layers > 0 && m->layers != nullptr, "model has no layers");
  PE_REQUIRE(m->tok_emb && m->emb_norm_w && m->final_norm_w && m->rope_global && m->rope_local,
             "model has a NULL weight or RoPE table");
  PE_REQUIRE(m->max_positions > 0 && m->vocab > 0, "bad max_positions/vocab");
  for (int l = 0; l < m->n_layers; ++l) {
    const pe_layer_weights& L = m->layers[l];
    PE_REQUIRE(L.wqkv && L.wo && L.mlp_norm_w && L.wi && L.wo_mlp, "layer %d has a NULL weight", l);
  }
  return PE_OK;
}

}  // namespace pe

extern "C" int pe_set_option(int key, int value) {
  if (!pe::known_option(key)) {
    pe::set_last_error("pe_set_option: unknown key %d", key);
    return PE_ERR_ARG;
  }
  pe::g_options[key].store(value, std::memory_order_relaxed);
  if (key == pe::OPT_GEMM_PAIR) pe::set_gemm_pair(value);
  return PE_OK;
}

extern "C" size_t pe_forward_workspace_bytes(const pe_model* model, int64_t T, int n_seqs) {
  if (model == nullptr || T < 0 || n_seqs < 0) return 0;
  return pe::plan(model, T, n_seqs).total;
}

namespace pe {

// hidden_out and pooled_out: at least one is given.  pool_mode / normalize as pe_pool_packed.
static int forward_impl(const pe_model* model, const int64_t* ids, const int32_t* cu_seqlens,
                        const int64_t* position_ids, int64_t T, int n_seqs, int max_seqlen,
                        void* workspace, size_t workspace_bytes, void* hidden_out, void* pooled_out,
                        int pool_mode, int normalize, int32_t* status, void* stream, const char* who) {
  int rc = check_model(model);
  if (rc != PE_OK) return rc;
  PE_REQUIRE(ids && cu_seqlens && position_ids && workspace && (hidden_out || pooled_out) && status,
             "%s: null pointer", who);
  PE_REQUIRE(T >= 0 && T < (1ll << 31) - 256 && n_seqs > 0 && max_seqlen > 0, "%s: bad sizes", who);
  PE_REQUIRE(max_seqlen <= model->max_positions, "%s: max_seqlen %d exceeds the RoPE table (%d rows)", who,
             max_seqlen, model->max_positions);
  const Workspace w = plan(model, T, n_seqs);
  if (workspace_bytes < w.total) {
    set_last_error("%s: workspace %zu < %zu bytes", who, workspace_bytes, w.total);
    return PE_ERR_WORKSPACE;
  }
  if (T == 0) return PE_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  void* x = ws + w.x;
  void* normed = ws + w.normed;
  void* qkv = ws + w.qkv;
  void* ctx = ws + w.ctx;
  void* tmp = ws + w.tmp;
  void* act = ws + w.act;
  void* proj = ws + w.proj;
  void* tiles = ws + w.tiles;
  const int H = model->hidden, I = model->intermediate, nh = model->n_heads;
  const float eps = model->eps;
  const bool fuse_rope = get_option(OPT_FUSED_ROPE) != 0;
  const bool fuse_geglu = get_option(OPT_FUSED_GEGLU) != 0;
  const bool fuse_res = get_option(OPT_FUSED_RESIDUAL) != 0;

#define PE_TRY(call)            \
  do {                          \
    rc = (call);                \
    if (rc != PE_OK) return rc; \
  } while (0)

  PE_TRY(pe_embed_ln(ids, model->tok_emb, model->emb_norm_w, eps, T, H, model->vocab, x, status, st));
  const int bm = attn_pick_bm(max_seqlen);
  PE_TRY(attn_schedule(cu_seqlens, n_seqs, T, bm, bm == 128, tiles, status, st));
  // Rows at or beyond cu_seqlens[n_seqs] (the padding of a graph bucket) are never written by
  // attention.  Left as the arena's previous contents they would flow through Wo into the residual
  // stream and from there into the V rows that the last real sequence's final key tile fetches,
  // where a non-finite bit pattern times P = 0 is NaN.  Zeroed once, they stay finite.
  zero_tail_rows_kernel<<<sm_count(), 256, 0, st>>>(static_cast<uint8_t*>(ctx), cu_seqlens + n_seqs, (int)T,
                                                   H * 2);
  PE_LAUNCH_CHECK("zero_tail_rows_kernel");

  bool pending = false;  // tmp holds the previous layer's MLP output, not yet added to x
  for (int l = 0; l < model->n_layers; ++l) {
    const pe_layer_weights& L = model->layers[l];
    const void* attn_in = normed;
    if (L.attn_norm_w != nullptr) {
      PE_TRY(pe_add_ln(x, pending ? tmp : nullptr, L.attn_norm_w, eps, T, H, pending ? x : nullptr,
                       normed, st));
    } else {
      if (pending) PE_TRY(pe_add_ln(x, tmp, nullptr, eps, T, H, x, nullptr, st));
      attn_in = x;
    }
    pending = false;
    const void* rope_table = L.is_global ? model->rope_global : model->rope_local;
    if (fuse_rope) {
      PE_TRY(pe_gemm_qkv_rope_bf16(attn_in, L.wqkv, qkv, T, nh, H, position_ids, rope_table,
                                   model->max_positions, status, st));
    } else {
      PE_TRY(pe_gemm_bf16_tn(attn_in, L.wqkv, qkv, T, 3 * H, H, status, st));
      PE_TRY(pe_rope_qk_inplace(qkv, position_ids, rope_table, model->max_positions, T, nh, status, st));
    }
    PE_TRY(attn_run(qkv, tiles, n_seqs, T, nh, L.is_global ? -1 : model->half_window, bm, ctx, status,
                    st));
    if (fuse_res) {  // x += Wo ctx in the GEMM epilogue, then a plain LayerNorm
      PE_TRY(pe_gemm_residual_bf16(ctx, L.wo, x, x, T, H, H, status, st));
      PE_TRY(pe_add_ln(x, nullptr, L.mlp_norm_w, eps, T, H, nullptr, normed, st));
    } else {
      PE_TRY(pe_gemm_bf16_tn(ctx, L.wo, tmp, T, H, H, status, st));
      PE_TRY(pe_add_ln(x, tmp, L.mlp_norm_w, eps, T, H, x, normed, st));
    }
    if (fuse_geglu) {
      PE_TRY(pe_gemm_geglu_bf16(normed, L.wi, act, T, I, H, status, st));
    } else {
      PE_TRY(pe_gemm_bf16_tn(normed, L.wi, proj, T, 2 * I, H, status, st));
      PE_TRY(pe_geglu(proj, T, I, act, st));
    }
    if (fuse_res) {  // the MLP residual lands in x right away instead of waiting for the next norm
      PE_TRY(pe_gemm_residual_bf16(act, L.wo_mlp, x, x, T, H, I, status, st));
    } else {
      PE_TRY(pe_gemm_bf16_tn(act, L.wo_mlp, tmp, T, H, I, status, st));
      pending = true;
    }
  }
  if (pooled_out == nullptr) {
    PE_TRY(pe_add_ln(x, pending ? tmp : nullptr, model->final_norm_w, eps, T, H, nullptr, hidden_out, st));
  } else {
    if (pending) PE_TRY(pe_add_ln(x, tmp, nullptr, eps, T, H, x, nullptr, st));
    PE_TRY(final_ln_pool(x, model->final_norm_w, eps, cu_seqlens, n_seqs, T, H, pool_mode, normalize,
                         hidden_out, pooled_out, ws + w.pool, w.total - w.pool, st));
  }
#undef PE_TRY
  return PE_OK;
}

}  // namespace pe

extern "C" int pe_forward_packed(const pe_model* model, const int64_t* ids,
                                 const int32_t* cu_seqlens, const int64_t* position_ids, int64_t T,
                                 int n_seqs, int max_seqlen, void* workspace, size_t workspace_bytes,
                                 void* out, int32_t* status, void* stream) {
  if (out == nullptr) {
    pe::set_last_error("pe_forward_packed: out is NULL");
    return PE_ERR_ARG;
  }
  return pe::forward_impl(model, ids, cu_seqlens, position_ids, T, n_seqs, max_seqlen, workspace,
                          workspace_bytes, out, nullptr, 0, 0, status, stream, "pe_forward_packed");
}

extern "C" int pe_forward_packed_pooled(const pe_model* model, const int64_t* ids,
                                        const int32_t* cu_seqlens, const int64_t* position_ids,
                                        int64_t T, int n_seqs, int max_seqlen, void* workspace,
                                        size_t workspace_bytes, int pool_mode, int normalize,
                                        void* hidden_out, void* pooled_out, int32_t* status,
                                        void* stream) {
  if (pooled_out == nullptr || (pool_mode != 0 && pool_mode != 1)) {
    pe::set_last_error("pe_forward_packed_pooled: pooled_out is NULL or pool_mode %d is not 0 / 1", pool_mode);
    return PE_ERR_ARG;
  }
  return pe::forward_impl(model, ids, cu_seqlens, position_ids, T, n_seqs, max_seqlen, workspace,
                          workspace_bytes, hidden_out, pooled_out, pool_mode, normalize, status, stream,
                          "pe_forward_packed_pooled");
}
