// Python bindings of the sm_100a kernels.  The kernels live in .cu files that know nothing about
// PyTorch (raw pointers + a stream); this file checks tensors and forwards to their C launchers.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstring>
#include <vector>

using torch::Tensor;
using OptTensor = c10::optional<Tensor>;

// ---- argument blocks shared with the .cu files ------------------------------------------------------------------
struct CltExchangeArgs {
  int world;
  int rank;
  void* data[8];
  void* flags[8];
  int slot_elems;
  unsigned int seq;
};
struct CltSelectArgs {
  const void* x;
  const float* mean;
  const float* rstd;
  int L, B, F;
  int stat_pitch;
  long long ld, layer_stride;
  int col_pitch;
  int feat_offset;
  long long full_F;
  long long k_total;
  unsigned int key_lo;
  int shift;
  unsigned int* hist;
  long long* ctl;
  int* ent_tok; int* ent_col; float* ent_val; long long ent_cap;
  unsigned int* cand_key; int* cand_tok; int* cand_col; float* cand_val; long long cand_cap;
  int* status;
  long long* sel_state;
  unsigned int* pool_key; int* pool_tok; int* pool_col; float* pool_val; long long pool_cap;
};
struct CltThetaGradArgs {
  const void* gs; const void* w[32]; const void* preact;
  long long ldx, layer_stride_x;
  const float* theta; int stat_pitch; float bandwidth;
  float* S1; float* S2;
  int L, B, F, d;
  int* status;
  int tying;            // 0 untied ([F, L - s, d] per source), 1 per_source, 2 per_target ([F, 1, d] per layer)
  const void* gs_cum;   // per_source: suffix sums of the gradient seed over the layers
};
struct CltCsrArgs {
  const int* ent_tok; const int* ent_col; const float* ent_val; long long ent_cap;
  const long long* ctl;
  int num_tokens; int num_cols;
  int* tok_cnt; int* feat_cnt;
  int* tok_off; int* feat_off;
  int* tok_cursor; int* feat_cursor;
  int* tcsr_col; float* tcsr_val; int* fcsr_tok; float* fcsr_val;
  unsigned char* fired;
  int sort_segments;
  int col_pitch;
};
struct CltDecodeArgs {
  const void* w[32];
  int rows[32];
  int L, B, d, col_pitch, tying;
  const int* tok_off; const int* tcsr_col; const float* tcsr_val;
  const float* feat_offset; const float* feat_scale;
  float* yhat_partial;
  const float* bias_sum; const float* addend; const void* target; const float* sigma;
  void* gs; float* yhat_out; double* sq_err;
  void* stage_peers[8];
  int rows_per_rank, rank, world;
  int mode;
  int* status;
  float* ctl;
  int rows_limit;
};
struct CltPeerTable {
  int world;
  int rank;
  void* ptr[8];
};
struct CltAdamHyper {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;
  int decoupled;
  float grad_scale;
  unsigned int sr_seed;
  unsigned int moment_seed;
};
struct CltDecAdamArgs {
  void* w[32]; float* m[32]; float* v[32]; int rows[32];
  int ntensors, L, B, d, F_pitch, tying, weights_bf16;
  const int* feat_off; const int* fcsr_tok; const float* fcsr_val;
  const void* gs; float* grad_a; const float* pen_coef; float* norm2_out;
  const float* feat_offset; const float* feat_scale;
  const float* dgrad_row0;
  CltAdamHyper h;
  int* status;
  int moments_bf16;
  const int* extra_idx; const float* extra_rows;
  float* ctl;
  int norm_only;
  float* d_feat_offset; float* d_feat_scale;
};
struct CltEncAdamArgs {
  void* w; float* m; float* v; void* bias; float* bias_m; float* bias_v;
  int L, B, d, F_pitch, weights_bf16;
  const int* feat_off; const int* fcsr_tok; const float* delta; const void* x;
  const float* dense_grad; const float* dense_bias_grad;
  CltAdamHyper h;
  int* status;
  int moments_bf16;
  const int* extra_idx; const float* extra_rows; const float* extra_bias;
  float* ctl;
  int norm_only;
};
struct CltStepControlArgs {
  float* ctl; const int* status; double* sq_err; int L; double* scalars; int n_scalars; float* losses; double inv_bd;
  int phase, dynamic_scale, growth_interval; float max_norm; int round;
};
struct CltThetaAdamArgs {
  void* log_theta; float* m; float* v; float* theta; const float* S1; const float* S2; const float* norm2;
  const int* feat_off; const float* fcsr_val;
  int L, pitch, tying, weights_16;
  float c_g, lambda, c, bandwidth;
  CltAdamHyper h;
  float* ctl;
  float norm_weight;
  float* grad_out;
};

extern "C" {
// type-independent entry points (compiled once)
int clt_colstats_from_tiles(const float* tile_stats, float* mean, float* rstd, int L, int B, int F, cudaStream_t st);
int clt_build_csr(const CltCsrArgs* a, cudaStream_t st);
int clt_dead_counter_update(long long* counter, unsigned char* fired, int n, cudaStream_t st);
int clt_peer_barrier(const CltPeerTable* flags, int slot, unsigned int seq, int* status, long long timeout_cycles, cudaStream_t st);
int clt_sparsity_penalty(const int* feat_off, const float* fcsr_val, const float* norm2, int ncols, float lambda, float c,
                         float* grad_a, float* pen_coef, double* penalty_out, cudaStream_t st);
int clt_step_control(const CltStepControlArgs* a, const CltExchangeArgs* exa, cudaStream_t st);
struct CltTopkTpArgs {
  const int* cand_col; const float* cand_val;
  unsigned long long* cand_key;
  const float* mean; const float* rstd; int stat_pitch;
  int col_pitch, feat_offset; long long full_F;
  int B, k, world, rank, rows_per_rank;
  void* stage[8];
  void* cut[8];
  long long* ctl;
  int* ent_tok; int* ent_col; float* ent_val; long long ent_cap;
  int* status;
};
int clt_token_topk_tp(const CltTopkTpArgs* a, int phase, cudaStream_t st);
int clt_aux_compact(const long long* dead_counter, long long window, int L, int F_pitch, int F_valid, int nd_cap, int* dead_cols, int* nd,
                    int* nd_all, int* extra_idx, cudaStream_t st);
int clt_scatter_add_rows(float* dst, float* dst_bias, const float* src, const float* src_bias, const int* extra_idx, long long n_dst_rows, int d,
                         cudaStream_t st);
int clt_unscale(float* buf, long long n, const float* ctl, cudaStream_t st);
struct CltAuxRowsArgs {
  const void* w[32];
  int rows[32];
};
// entry points that exist once per 16-bit storage type: name (bf16) and name_h (fp16)
#define CLT_API(name) name
#include "clt_api.inc"
#undef CLT_API
#define CLT_API(name) name##_h
#include "clt_api.inc"
#undef CLT_API
}

// picks the fp16 or the bf16 build of an entry point
#define CLT_PICK(half, name) ((half) ? name##_h : name)

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int num_sms() {
  static int n = 0;
  if (n == 0) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return n;
}

void check(int rc, const char* what) {
  TORCH_CHECK(rc == 0, what, " failed with code ", rc);
}
void need(const Tensor& t, c10::ScalarType ty, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == ty, name, " has dtype ", t.scalar_type(), ", expected ", ty);
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
// 16-bit storage type of a tensor: true for fp16, false for bf16 (anything else is refused)
bool is_half(const Tensor& t, const char* name) {
  TORCH_CHECK(t.scalar_type() == at::kHalf || t.scalar_type() == at::kBFloat16, name, " must be bf16 or fp16, got ", t.scalar_type());
  return t.scalar_type() == at::kHalf;
}
c10::ScalarType t16_of(bool half) { return half ? at::kHalf : at::kBFloat16; }
template <typename T>
T* opt_ptr(const OptTensor& t) {
  return t.has_value() && t->defined() ? static_cast<T*>(t->data_ptr()) : nullptr;
}
float* ctl_ptr(const OptTensor& ctl) {
  if (!ctl.has_value() || !ctl->defined()) return nullptr;
  TORCH_CHECK(ctl->is_cuda() && ctl->scalar_type() == at::kFloat && ctl->numel() >= 16 && ctl->is_contiguous(), "ctl: contiguous fp32 CUDA tensor of 16 words");
  return ctl->data_ptr<float>();
}

CltAdamHyper hyper_from(const std::vector<double>& h) {
  TORCH_CHECK(h.size() == 10 || h.size() == 11, "hyper expects 10 values (+ the moment rounding seed)");
  CltAdamHyper c;
  c.lr = float(h[0]); c.beta1 = float(h[1]); c.beta2 = float(h[2]); c.eps = float(h[3]); c.weight_decay = float(h[4]);
  c.bc1 = float(h[5]); c.bc2 = float(h[6]); c.decoupled = int(h[7]); c.grad_scale = float(h[8]); c.sr_seed = static_cast<unsigned int>(h[9]);
  c.moment_seed = h.size() > 10 ? static_cast<unsigned int>(h[10]) : 0x1234567u;
  return c;
}

// ----------------------------------------------------------------------------------------------
// tile_stats (optional, fp32 [L, ceil(M / 128), N, 2]): per 128-row block sums / sums of squares of the stored outputs.
void encoder_gemm(const Tensor& x, const Tensor& w, const OptTensor& bias, Tensor& out, Tensor& status, const OptTensor& tile_stats) {
  const bool half = is_half(x, "x");
  const auto ty = t16_of(half);
  need(x, ty, "x"); need(w, ty, "w"); need(out, ty, "out"); need(status, at::kInt, "status");
  TORCH_CHECK(x.dim() == 3 && w.dim() == 3 && out.dim() == 3, "expected [L, M, K], [L, N, K], [L, M, N]");
  const int L = x.size(0), M = x.size(1), K = x.size(2), N = w.size(1);
  TORCH_CHECK(w.size(0) == L && w.size(2) == K && out.size(0) == L && out.size(1) == M && out.size(2) == N, "shape mismatch");
  if (bias.has_value() && bias->defined()) { need(*bias, ty, "bias"); TORCH_CHECK(bias->numel() == 1LL * L * N, "bias must be [L, N]"); }
  float* ts = nullptr;
  if (tile_stats.has_value() && tile_stats->defined()) {
    need(*tile_stats, at::kFloat, "tile_stats");
    TORCH_CHECK(tile_stats->numel() == 2LL * L * ((M + 127) / 128) * N, "tile_stats must be [L, ceil(M / 128), N, 2]");
    ts = tile_stats->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(x.device());
  check(CLT_PICK(half, clt_encoder_gemm)(x.data_ptr(), w.data_ptr(), opt_ptr<void>(bias), out.data_ptr(), L, M, N, K, N, 1LL * M * N,
                                         status.data_ptr<int>(), ts, num_sms(), cur_stream()), "encoder_gemm");
}

// mean / rstd [L, F] from the per-block sums written by encoder_gemm (B rows per column).
void colstats_from_tiles(const Tensor& tile_stats, Tensor& mean, Tensor& rstd, int64_t B) {
  need(tile_stats, at::kFloat, "tile_stats"); need(mean, at::kFloat, "mean"); need(rstd, at::kFloat, "rstd");
  TORCH_CHECK(tile_stats.dim() == 4 && tile_stats.size(3) == 2 && tile_stats.size(1) == (B + 127) / 128, "tile_stats must be [L, ceil(B / 128), F, 2]");
  const int L = tile_stats.size(0), F = tile_stats.size(2);
  TORCH_CHECK(mean.numel() == 1LL * L * F && rstd.numel() == 1LL * L * F, "mean/rstd must be [L, F]");
  c10::cuda::CUDAGuard guard(tile_stats.device());
  check(clt_colstats_from_tiles(tile_stats.data_ptr<float>(), mean.data_ptr<float>(), rstd.data_ptr<float>(), L, int(B), F, cur_stream()), "colstats_from_tiles");
}

void colstats(const Tensor& x, Tensor& mean, Tensor& rstd) {
  const bool half = is_half(x, "x");
  need(x, t16_of(half), "x"); need(mean, at::kFloat, "mean"); need(rstd, at::kFloat, "rstd");
  const int L = x.size(0), B = x.size(1), F = x.size(2);
  TORCH_CHECK(mean.numel() == 1LL * L * F && rstd.numel() == 1LL * L * F, "mean/rstd must be [L, F]");
  c10::cuda::CUDAGuard guard(x.device());
  check(CLT_PICK(half, clt_colstats)(x.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), L, B, F, F, 1LL * B * F, cur_stream()), "colstats");
}

// exchange: (world, rank, data_ptrs[world], flag_ptrs[world], slot_elems, seq) or empty for a single rank
bool fill_exchange(CltExchangeArgs& ex, int64_t world, int64_t rank, const std::vector<int64_t>& data, const std::vector<int64_t>& flags,
                   int64_t slot_elems, int64_t seq) {
  if (world <= 1) return false;
  TORCH_CHECK(world <= 8 && int64_t(data.size()) == world && int64_t(flags.size()) == world, "exchange expects `world` pointers");
  std::memset(&ex, 0, sizeof(ex));
  ex.world = int(world); ex.rank = int(rank); ex.slot_elems = int(slot_elems); ex.seq = static_cast<unsigned int>(seq);
  for (int i = 0; i < world; ++i) { ex.data[i] = reinterpret_cast<void*>(data[i]); ex.flags[i] = reinterpret_cast<void*>(flags[i]); }
  return true;
}

void batchtopk_select(const Tensor& x, const Tensor& mean, const Tensor& rstd, int64_t f_valid, int64_t col_pitch, int64_t feat_offset,
                      int64_t full_F, int64_t k_total, int64_t key_lo, int64_t shift, Tensor& hist, Tensor& ctl, Tensor& ent_tok,
                      Tensor& ent_col, Tensor& ent_val, Tensor& cand_key, Tensor& cand_tok, Tensor& cand_col, Tensor& cand_val,
                      Tensor& status, int64_t world, int64_t rank, const std::vector<int64_t>& ex_data,
                      const std::vector<int64_t>& ex_flags, int64_t slot_elems, int64_t seq, const OptTensor& sel_state,
                      const OptTensor& pool) {
  const bool half = is_half(x, "x");
  need(x, t16_of(half), "x"); need(mean, at::kFloat, "mean"); need(rstd, at::kFloat, "rstd");
  need(hist, at::kInt, "hist"); need(ctl, at::kLong, "ctl"); need(status, at::kInt, "status");
  need(ent_tok, at::kInt, "ent_tok"); need(ent_col, at::kInt, "ent_col"); need(ent_val, at::kFloat, "ent_val");
  need(cand_key, at::kInt, "cand_key"); need(cand_tok, at::kInt, "cand_tok"); need(cand_col, at::kInt, "cand_col"); need(cand_val, at::kFloat, "cand_val");
  TORCH_CHECK(hist.numel() >= 2 * 8192 + 32 && ctl.numel() >= 16, "hist needs 2 * 8192 + 32 and ctl 16 elements");
  CltSelectArgs a;
  a.x = x.data_ptr(); a.mean = mean.data_ptr<float>(); a.rstd = rstd.data_ptr<float>();
  a.L = x.size(0); a.B = x.size(1); a.F = int(f_valid); a.stat_pitch = int(mean.size(-1));
  a.ld = x.size(2); a.layer_stride = 1LL * x.size(1) * x.size(2);
  a.col_pitch = int(col_pitch); a.feat_offset = int(feat_offset); a.full_F = full_F; a.k_total = k_total;
  a.key_lo = static_cast<unsigned int>(key_lo); a.shift = int(shift);
  a.hist = reinterpret_cast<unsigned int*>(hist.data_ptr<int>()); a.ctl = reinterpret_cast<long long*>(ctl.data_ptr<int64_t>());
  a.ent_tok = ent_tok.data_ptr<int>(); a.ent_col = ent_col.data_ptr<int>(); a.ent_val = ent_val.data_ptr<float>(); a.ent_cap = ent_tok.numel();
  a.cand_key = reinterpret_cast<unsigned int*>(cand_key.data_ptr<int>()); a.cand_tok = cand_tok.data_ptr<int>();
  a.cand_col = cand_col.data_ptr<int>(); a.cand_val = cand_val.data_ptr<float>(); a.cand_cap = cand_key.numel();
  a.status = status.data_ptr<int>();
  a.sel_state = nullptr; a.pool_key = nullptr; a.pool_tok = nullptr; a.pool_col = nullptr; a.pool_val = nullptr; a.pool_cap = 0;
  if (sel_state.has_value() && sel_state->defined()) {
    // tracked range: {key_lo, shift} on the device plus the pool [4, cap] (key, token, column, value bits)
    need(*sel_state, at::kLong, "sel_state");
    TORCH_CHECK(pool.has_value() && pool->defined(), "sel_state needs a pool");
    need(*pool, at::kInt, "pool");
    TORCH_CHECK(sel_state->numel() >= 2 && pool->dim() == 2 && pool->size(0) == 4, "sel_state needs 2 elements and pool the shape [4, cap]");
    a.sel_state = reinterpret_cast<long long*>(sel_state->data_ptr<int64_t>());
    a.pool_cap = pool->size(1);
    int* pb = pool->data_ptr<int>();
    a.pool_key = reinterpret_cast<unsigned int*>(pb); a.pool_tok = pb + a.pool_cap; a.pool_col = pb + 2 * a.pool_cap;
    a.pool_val = reinterpret_cast<float*>(pb + 3 * a.pool_cap);
  }
  CltExchangeArgs ex;
  const bool multi = fill_exchange(ex, world, rank, ex_data, ex_flags, slot_elems, seq);
  c10::cuda::CUDAGuard guard(x.device());
  check(CLT_PICK(half, clt_batchtopk_select)(&a, multi ? &ex : nullptr, cur_stream()), "batchtopk_select");
}

// Entries with x >= theta[l, f] (JumpReLU; ReLU with theta = smallest positive value) as a (token, column, value) list.
void threshold_select(const Tensor& x, const Tensor& theta, int64_t f_valid, int64_t col_pitch, Tensor& ctl, Tensor& ent_tok,
                      Tensor& ent_col, Tensor& ent_val, Tensor& status) {
  const bool half = is_half(x, "x");
  need(x, t16_of(half), "x"); need(theta, at::kFloat, "theta"); need(ctl, at::kLong, "ctl"); need(status, at::kInt, "status");
  need(ent_tok, at::kInt, "ent_tok"); need(ent_col, at::kInt, "ent_col"); need(ent_val, at::kFloat, "ent_val");
  TORCH_CHECK(x.dim() == 3 && theta.dim() == 2 && theta.size(0) == x.size(0) && theta.size(1) >= f_valid, "theta must be [L, >= F]");
  TORCH_CHECK(ctl.numel() >= 16, "ctl needs 16 elements");
  CltSelectArgs a;
  std::memset(&a, 0, sizeof(a));
  a.x = x.data_ptr(); a.rstd = theta.data_ptr<float>();
  a.L = x.size(0); a.B = x.size(1); a.F = int(f_valid); a.stat_pitch = int(theta.size(1));
  a.ld = x.size(2); a.layer_stride = 1LL * x.size(1) * x.size(2);
  a.col_pitch = int(col_pitch);
  a.ctl = reinterpret_cast<long long*>(ctl.data_ptr<int64_t>());
  a.ent_tok = ent_tok.data_ptr<int>(); a.ent_col = ent_col.data_ptr<int>(); a.ent_val = ent_val.data_ptr<float>(); a.ent_cap = ent_tok.numel();
  a.status = status.data_ptr<int>();
  c10::cuda::CUDAGuard guard(x.device());
  check(CLT_PICK(half, clt_threshold_select)(&a, cur_stream()), "threshold_select");
}

// Per-token top-k of the batch z-scores: exactly k entries per token at [token * k, token * k + k) of the entry list.
void token_topk_select(const Tensor& x, const Tensor& mean, const Tensor& rstd, int64_t col_pitch, int64_t k, Tensor& ctl, Tensor& ent_tok,
                       Tensor& ent_col, Tensor& ent_val, Tensor& status, int64_t f_valid) {
  const bool half = is_half(x, "x");
  need(x, t16_of(half), "x"); need(mean, at::kFloat, "mean"); need(rstd, at::kFloat, "rstd"); need(ctl, at::kLong, "ctl");
  need(status, at::kInt, "status"); need(ent_tok, at::kInt, "ent_tok"); need(ent_col, at::kInt, "ent_col"); need(ent_val, at::kFloat, "ent_val");
  TORCH_CHECK(x.dim() == 3 && mean.dim() == 2 && mean.size(0) == x.size(0) && mean.size(1) == x.size(2), "mean / rstd must be [L, F]");
  TORCH_CHECK(ctl.numel() >= 16 && ent_tok.numel() >= x.size(1) * k, "entry list needs B * k elements");
  CltSelectArgs a;
  std::memset(&a, 0, sizeof(a));
  a.x = x.data_ptr(); a.mean = mean.data_ptr<float>(); a.rstd = rstd.data_ptr<float>();
  a.L = x.size(0); a.B = x.size(1); a.F = x.size(2); a.stat_pitch = int(mean.size(1));
  a.ld = x.size(2); a.layer_stride = 1LL * x.size(1) * x.size(2);
  a.col_pitch = int(col_pitch); a.k_total = k;
  a.feat_offset = int(f_valid);  // valid columns per layer (0: all of them)
  a.ctl = reinterpret_cast<long long*>(ctl.data_ptr<int64_t>());
  a.ent_tok = ent_tok.data_ptr<int>(); a.ent_col = ent_col.data_ptr<int>(); a.ent_val = ent_val.data_ptr<float>(); a.ent_cap = ent_tok.numel();
  a.status = status.data_ptr<int>();
  c10::cuda::CUDAGuard guard(x.device());
  check(CLT_PICK(half, clt_token_topk_select)(&a, cur_stream()), "token_topk_select");
}

// One phase of the TokenTopK selection across feature shards (0: push the local candidates' keys to the token owners,
// 1: owners find the cut of their tokens and publish it, 2: keep the candidates at or above the cut).  The caller separates
// the phases with peer barriers.  cand_* [B * k]: the local top k of every token (token_topk_select into scratch lists).
void token_topk_tp(int64_t phase, const Tensor& cand_col, const Tensor& cand_val, Tensor& cand_key, const Tensor& mean, const Tensor& rstd,
                   int64_t col_pitch, int64_t feat_offset, int64_t full_F, int64_t B, int64_t k, int64_t rank, int64_t rows_per_rank,
                   const std::vector<int64_t>& stage_ptrs, const std::vector<int64_t>& cut_ptrs, Tensor& ctl, Tensor& ent_tok, Tensor& ent_col,
                   Tensor& ent_val, Tensor& status) {
  need(cand_col, at::kInt, "cand_col"); need(cand_val, at::kFloat, "cand_val"); need(cand_key, at::kLong, "cand_key");
  need(mean, at::kFloat, "mean"); need(rstd, at::kFloat, "rstd"); need(ctl, at::kLong, "ctl"); need(status, at::kInt, "status");
  need(ent_tok, at::kInt, "ent_tok"); need(ent_col, at::kInt, "ent_col"); need(ent_val, at::kFloat, "ent_val");
  TORCH_CHECK(cand_col.numel() >= B * k && cand_val.numel() >= B * k && cand_key.numel() >= B * k, "candidate lists hold B * k elements");
  TORCH_CHECK(stage_ptrs.size() == cut_ptrs.size() && !stage_ptrs.empty() && stage_ptrs.size() <= 8, "one staging and one cut pointer per rank");
  CltTopkTpArgs a;
  std::memset(&a, 0, sizeof(a));
  a.cand_col = cand_col.data_ptr<int>(); a.cand_val = cand_val.data_ptr<float>();
  a.cand_key = reinterpret_cast<unsigned long long*>(cand_key.data_ptr<int64_t>());
  a.mean = mean.data_ptr<float>(); a.rstd = rstd.data_ptr<float>(); a.stat_pitch = int(mean.size(1));
  a.col_pitch = int(col_pitch); a.feat_offset = int(feat_offset); a.full_F = full_F;
  a.B = int(B); a.k = int(k); a.world = int(stage_ptrs.size()); a.rank = int(rank); a.rows_per_rank = int(rows_per_rank);
  for (size_t i = 0; i < stage_ptrs.size(); ++i) { a.stage[i] = reinterpret_cast<void*>(stage_ptrs[i]); a.cut[i] = reinterpret_cast<void*>(cut_ptrs[i]); }
  a.ctl = reinterpret_cast<long long*>(ctl.data_ptr<int64_t>());
  a.ent_tok = ent_tok.data_ptr<int>(); a.ent_col = ent_col.data_ptr<int>(); a.ent_val = ent_val.data_ptr<float>(); a.ent_cap = ent_tok.numel();
  a.status = status.data_ptr<int>();
  c10::cuda::CUDAGuard guard(cand_col.device());
  check(clt_token_topk_tp(&a, int(phase), cur_stream()), "token_topk_tp");
}

// JumpReLU threshold gradient sums: S1[l, f] += sum_b window * x * (gs . W_dec rows), S2[l, f] += sum_b window * x.
// tying: 0 untied (decoder tensor s is [F, L - s, d]), 1 per_source, 2 per_target (tensors [F, 1, d]); per_source needs
// gs_cum, the suffix sums of the gradient seed over the layers (gs_suffix_sum).
void theta_grad_gemm(const Tensor& gs, const std::vector<Tensor>& dec_w, const Tensor& preact, const Tensor& theta, double bandwidth,
                     Tensor& S1, Tensor& S2, Tensor& status, int64_t tying, const OptTensor& gs_cum) {
  const bool half = is_half(gs, "gs");
  const auto ty = t16_of(half);
  need(gs, ty, "gs"); need(preact, ty, "preact"); need(theta, at::kFloat, "theta");
  need(S1, at::kFloat, "S1"); need(S2, at::kFloat, "S2"); need(status, at::kInt, "status");
  const int L = gs.size(0), B = gs.size(1), d = gs.size(2), F = preact.size(2);
  TORCH_CHECK(int(dec_w.size()) == L && L <= 32, "one decoder tensor per layer (at most 32)");
  TORCH_CHECK(preact.size(0) == L && preact.size(1) == B && theta.size(0) == L && theta.size(1) >= F, "shape mismatch");
  TORCH_CHECK(S1.sizes() == theta.sizes() && S2.sizes() == theta.sizes(), "S1 / S2 must have theta's shape");
  TORCH_CHECK(tying >= 0 && tying <= 2, "tying must be 0, 1 or 2");
  CltThetaGradArgs a;
  std::memset(&a, 0, sizeof(a));
  a.gs = gs.data_ptr(); a.preact = preact.data_ptr(); a.ldx = preact.size(2); a.layer_stride_x = 1LL * B * preact.size(2);
  for (int s = 0; s < L; ++s) {
    need(dec_w[s], ty, "decoder weight");
    const int rows = tying == 0 ? L - s : 1;
    TORCH_CHECK(dec_w[s].dim() == 3 && dec_w[s].size(0) == F && dec_w[s].size(1) == rows && dec_w[s].size(2) == d, "decoder tensor must be [F, rows, d]");
    a.w[s] = dec_w[s].data_ptr();
  }
  a.theta = theta.data_ptr<float>(); a.stat_pitch = int(theta.size(1)); a.bandwidth = float(bandwidth);
  a.S1 = S1.data_ptr<float>(); a.S2 = S2.data_ptr<float>();
  a.L = L; a.B = B; a.F = F; a.d = d; a.status = status.data_ptr<int>();
  a.tying = int(tying);
  if (tying == 1) {
    TORCH_CHECK(gs_cum.has_value() && gs_cum->defined(), "per_source tying needs gs_cum");
    need(*gs_cum, ty, "gs_cum");
    TORCH_CHECK(gs_cum->sizes() == gs.sizes(), "gs_cum must have the shape of gs");
    a.gs_cum = gs_cum->data_ptr();
  }
  c10::cuda::CUDAGuard guard(gs.device());
  check(CLT_PICK(half, clt_theta_grad_gemm)(&a, num_sms(), cur_stream()), "theta_grad_gemm");
}

void build_csr(const Tensor& ent_tok, const Tensor& ent_col, const Tensor& ent_val, const Tensor& ctl, int64_t num_tokens, int64_t num_cols,
               Tensor& tok_cnt, Tensor& feat_cnt, Tensor& tok_off, Tensor& feat_off, Tensor& tok_cursor, Tensor& feat_cursor,
               Tensor& tcsr_col, Tensor& tcsr_val, Tensor& fcsr_tok, Tensor& fcsr_val, const OptTensor& fired, int64_t sort_segments,
               int64_t col_pitch) {
  need(ent_tok, at::kInt, "ent_tok"); need(ctl, at::kLong, "ctl");
  need(tok_cnt, at::kInt, "tok_cnt"); need(feat_cnt, at::kInt, "feat_cnt"); need(tok_off, at::kInt, "tok_off"); need(feat_off, at::kInt, "feat_off");
  TORCH_CHECK(tok_off.numel() >= num_tokens + 1 && feat_off.numel() >= num_cols + 1, "offset arrays too small");
  TORCH_CHECK(tok_cnt.numel() >= num_tokens && feat_cnt.numel() >= num_cols && tok_cursor.numel() >= num_tokens && feat_cursor.numel() >= num_cols, "count arrays too small");
  CltCsrArgs a;
  a.ent_tok = ent_tok.data_ptr<int>(); a.ent_col = ent_col.data_ptr<int>(); a.ent_val = ent_val.data_ptr<float>(); a.ent_cap = ent_tok.numel();
  a.ctl = reinterpret_cast<const long long*>(ctl.data_ptr<int64_t>());
  a.num_tokens = int(num_tokens); a.num_cols = int(num_cols);
  a.tok_cnt = tok_cnt.data_ptr<int>(); a.feat_cnt = feat_cnt.data_ptr<int>(); a.tok_off = tok_off.data_ptr<int>(); a.feat_off = feat_off.data_ptr<int>();
  a.tok_cursor = tok_cursor.data_ptr<int>(); a.feat_cursor = feat_cursor.data_ptr<int>();
  a.tcsr_col = tcsr_col.data_ptr<int>(); a.tcsr_val = tcsr_val.data_ptr<float>(); a.fcsr_tok = fcsr_tok.data_ptr<int>(); a.fcsr_val = fcsr_val.data_ptr<float>();
  a.fired = fired.has_value() && fired->defined() ? fired->data_ptr<uint8_t>() : nullptr;
  a.sort_segments = int(sort_segments);
  a.col_pitch = int(col_pitch);
  TORCH_CHECK(col_pitch > 0 && col_pitch < (1 << 24), "col_pitch must be in (0, 2^24)");
  c10::cuda::CUDAGuard guard(ent_tok.device());
  check(clt_build_csr(&a, cur_stream()), "build_csr");
}

void dead_counter_update(Tensor& counter, Tensor& fired) {
  need(counter, at::kLong, "counter"); need(fired, at::kByte, "fired");
  TORCH_CHECK(counter.numel() == fired.numel(), "counter / fired size mismatch");
  c10::cuda::CUDAGuard guard(counter.device());
  check(clt_dead_counter_update(reinterpret_cast<long long*>(counter.data_ptr<int64_t>()), fired.data_ptr<uint8_t>(), int(counter.numel()), cur_stream()),
        "dead_counter_update");
}

// ctl (optional): step control block; the gradient seed is multiplied by its loss scale and a seed outside the 16-bit range
// raises its found-inf flag.  rows_limit > 0: only the first rows_limit target rows of every feature are decoded.
void sparse_decode(const std::vector<Tensor>& dec_w, int64_t L, int64_t B, int64_t d, int64_t col_pitch, int64_t tying, const Tensor& tok_off,
                   const Tensor& tcsr_col, const Tensor& tcsr_val, const OptTensor& feat_offset, const OptTensor& feat_scale,
                   const OptTensor& yhat_partial, const OptTensor& bias_sum, const OptTensor& addend, const OptTensor& target,
                   const OptTensor& sigma, const OptTensor& gs, const OptTensor& yhat_out, const OptTensor& sq_err, int64_t mode,
                   const std::vector<int64_t>& stage_peers, int64_t rows_per_rank, int64_t rank, const OptTensor& status,
                   const OptTensor& ctl, int64_t rows_limit) {
  TORCH_CHECK(dec_w.size() >= 1 && dec_w.size() <= 32, "1..32 decoder tensors");
  const bool half = is_half(dec_w[0], "dec_w");
  const auto ty = t16_of(half);
  CltDecodeArgs a;
  std::memset(&a, 0, sizeof(a));
  for (size_t i = 0; i < dec_w.size(); ++i) {
    need(dec_w[i], ty, "dec_w");
    a.w[i] = dec_w[i].data_ptr();
    a.rows[i] = int(dec_w[i].size(1));
  }
  a.L = int(L); a.B = int(B); a.d = int(d); a.col_pitch = int(col_pitch); a.tying = int(tying);
  a.tok_off = tok_off.data_ptr<int>(); a.tcsr_col = tcsr_col.data_ptr<int>(); a.tcsr_val = tcsr_val.data_ptr<float>();
  a.feat_offset = opt_ptr<const float>(feat_offset); a.feat_scale = opt_ptr<const float>(feat_scale);
  a.yhat_partial = opt_ptr<float>(yhat_partial); a.bias_sum = opt_ptr<const float>(bias_sum); a.addend = opt_ptr<const float>(addend);
  if (target.has_value() && target->defined()) need(*target, ty, "target");
  if (gs.has_value() && gs->defined()) need(*gs, ty, "gs");
  a.target = opt_ptr<const void>(target); a.sigma = opt_ptr<const float>(sigma); a.gs = opt_ptr<void>(gs);
  a.yhat_out = opt_ptr<float>(yhat_out); a.sq_err = opt_ptr<double>(sq_err); a.mode = int(mode);
  if (status.has_value()) TORCH_CHECK(status->scalar_type() == at::kInt && status->numel() >= 4, "status: int32 tensor of at least 4 words (word 0 holds the code)");
  a.status = opt_ptr<int>(status);
  a.ctl = ctl_ptr(ctl);
  a.rows_limit = int(rows_limit);
  if (mode == 2) {
    TORCH_CHECK(stage_peers.size() >= 1 && stage_peers.size() <= 8 && rows_per_rank > 0, "mode 2 needs the peers' staging pointers");
    for (size_t i = 0; i < stage_peers.size(); ++i) a.stage_peers[i] = reinterpret_cast<void*>(stage_peers[i]);
    a.rows_per_rank = int(rows_per_rank); a.rank = int(rank); a.world = int(stage_peers.size());
  } else if (mode == 0) {
    TORCH_CHECK(a.yhat_partial != nullptr, "mode 0 needs yhat_partial");
  } else {
    TORCH_CHECK(a.bias_sum && a.target && a.gs && a.sq_err, "mode 1 needs bias_sum, target, gs, sq_err");
  }
  c10::cuda::CUDAGuard guard(tok_off.device());
  check(CLT_PICK(half, clt_sparse_decode)(&a, cur_stream()), "sparse_decode");
}

void recon_epilogue(const Tensor& yhat_sum, const Tensor& bias_sum, const OptTensor& addend, const Tensor& target, const OptTensor& sigma,
                    Tensor& gs, const OptTensor& yhat_out, Tensor& sq_err, int64_t row0, int64_t nrows, const OptTensor& ctl) {
  const bool half = is_half(target, "target");
  need(yhat_sum, at::kFloat, "yhat_sum"); need(bias_sum, at::kFloat, "bias_sum"); need(target, t16_of(half), "target");
  need(gs, t16_of(half), "gs"); need(sq_err, at::kDouble, "sq_err");
  const int L = yhat_sum.size(0), B = yhat_sum.size(1), d = yhat_sum.size(2);
  c10::cuda::CUDAGuard guard(yhat_sum.device());
  check(CLT_PICK(half, clt_recon_epilogue)(yhat_sum.data_ptr<float>(), bias_sum.data_ptr<float>(), opt_ptr<const float>(addend), target.data_ptr(),
                                           opt_ptr<const float>(sigma), gs.data_ptr(), opt_ptr<float>(yhat_out), sq_err.data_ptr<double>(), L, B, d,
                                           int(row0), int(nrows), ctl_ptr(ctl), cur_stream()), "recon_epilogue");
}

CltPeerTable make_table(const std::vector<int64_t>& ptrs, int64_t rank) {
  TORCH_CHECK(ptrs.size() >= 1 && ptrs.size() <= 8, "peer table holds 1..8 pointers");
  CltPeerTable t;
  std::memset(&t, 0, sizeof(t));
  t.world = int(ptrs.size()); t.rank = int(rank);
  for (size_t i = 0; i < ptrs.size(); ++i) t.ptr[i] = reinterpret_cast<void*>(ptrs[i]);
  return t;
}

// timeout_s <= 0: the default bound of every device-side wait (about a second)
void peer_barrier(const std::vector<int64_t>& flag_ptrs, int64_t rank, int64_t slot, int64_t seq, Tensor& status, double timeout_s) {
  need(status, at::kInt, "status");
  const CltPeerTable t = make_table(flag_ptrs, rank);
  c10::cuda::CUDAGuard guard(status.device());
  const long long cycles = timeout_s > 0 ? static_cast<long long>(timeout_s * 2.0e9) : 0;  // SM clock <= 2 GHz
  check(clt_peer_barrier(&t, int(slot), static_cast<unsigned int>(seq), status.data_ptr<int>(), cycles, cur_stream()), "peer_barrier");
}

// One strided copy on the current stream through the copy engines: `height` rows of `width` bytes, source and
// destination pitches in bytes.  Either side may be pinned host memory, local device memory or a peer's
// memory that is mapped into this process (the driver picks the direction from the pointers).
void memcpy_2d(int64_t dst, int64_t dst_pitch, int64_t src, int64_t src_pitch, int64_t width, int64_t height) {
  TORCH_CHECK(dst != 0 && src != 0 && width > 0 && height > 0 && dst_pitch >= width && src_pitch >= width, "memcpy_2d: bad geometry");
  const cudaError_t err = cudaMemcpy2DAsync(reinterpret_cast<void*>(dst), size_t(dst_pitch), reinterpret_cast<const void*>(src),
                                            size_t(src_pitch), size_t(width), size_t(height), cudaMemcpyDefault, cur_stream());
  TORCH_CHECK(err == cudaSuccess, "memcpy_2d: ", cudaGetErrorString(err));
}

void owner_reduce_loss(const Tensor& stage, const std::vector<int64_t>& gs_ptrs, int64_t rank, const Tensor& bias_sum, const OptTensor& addend,
                       const Tensor& target, const OptTensor& sigma, const OptTensor& yhat_out, Tensor& sq_err, int64_t rows_per_rank,
                       const OptTensor& ctl) {
  const bool half = is_half(target, "target");
  need(stage, at::kFloat, "stage"); need(bias_sum, at::kFloat, "bias_sum"); need(target, t16_of(half), "target"); need(sq_err, at::kDouble, "sq_err");
  const int L = target.size(0), B = target.size(1), d = target.size(2);
  const CltPeerTable t = make_table(gs_ptrs, rank);
  TORCH_CHECK(stage.numel() >= 1LL * t.world * L * rows_per_rank * d, "staging area too small");
  c10::cuda::CUDAGuard guard(stage.device());
  check(CLT_PICK(half, clt_owner_reduce_loss)(stage.data_ptr<float>(), &t, bias_sum.data_ptr<float>(), opt_ptr<const float>(addend), target.data_ptr(),
                                              opt_ptr<const float>(sigma), opt_ptr<float>(yhat_out), sq_err.data_ptr<double>(), L, B, d, int(rows_per_rank),
                                              ctl_ptr(ctl), cur_stream()), "owner_reduce_loss");
}

void gs_colsum(const Tensor& gs, Tensor& out) {
  const bool half = is_half(gs, "gs");
  need(gs, t16_of(half), "gs"); need(out, at::kFloat, "out");
  c10::cuda::CUDAGuard guard(gs.device());
  check(CLT_PICK(half, clt_gs_colsum)(gs.data_ptr(), out.data_ptr<float>(), int(gs.size(0)), int(gs.size(1)), int(gs.size(2)), cur_stream()), "gs_colsum");
}

// out[s] = sum over t >= s of gs[t] (same shape and type)
void gs_suffix_sum(const Tensor& gs, Tensor& out) {
  const bool half = is_half(gs, "gs");
  need(gs, t16_of(half), "gs"); need(out, t16_of(half), "out");
  TORCH_CHECK(gs.dim() == 3 && out.sizes() == gs.sizes(), "gs / out must be [L, B, d]");
  c10::cuda::CUDAGuard guard(gs.device());
  check(CLT_PICK(half, clt_gs_suffix_sum)(gs.data_ptr(), out.data_ptr(), int(gs.size(0)), int(gs.size(1)), int(gs.size(2)), cur_stream()), "gs_suffix_sum");
}

// extra_idx / extra_rows: compact extra gradient rows for the features' first rows (extra_idx[col] = row or -1);
// ctl: step control block (skip flag, 1 / loss scale, clip coefficient); norm_only: gradient-norm pre-pass.
void decoder_rows_adam(std::vector<Tensor>& w, std::vector<Tensor>& m, std::vector<Tensor>& v, int64_t L, int64_t B, int64_t d,
                       int64_t F_pitch, int64_t tying, const Tensor& feat_off, const Tensor& fcsr_tok, const Tensor& fcsr_val,
                       const Tensor& gs, const OptTensor& grad_a, const OptTensor& pen_coef, const OptTensor& norm2_out,
                       const OptTensor& feat_offset, const OptTensor& feat_scale, const OptTensor& dgrad_row0,
                       const std::vector<double>& hyper, const OptTensor& status, const OptTensor& extra_idx, const OptTensor& extra_rows,
                       const OptTensor& ctl, bool norm_only, const OptTensor& d_feat_offset, const OptTensor& d_feat_scale) {
  TORCH_CHECK(w.size() >= 1 && w.size() <= 32 && w.size() == m.size() && w.size() == v.size(), "bad tensor lists");
  CltDecAdamArgs a;
  std::memset(&a, 0, sizeof(a));
  const bool half = is_half(gs, "gs");
  const bool w16 = w[0].scalar_type() != at::kFloat;
  for (size_t i = 0; i < w.size(); ++i) {
    need(w[i], w16 ? t16_of(half) : at::kFloat, "w");
    need(m[i], m[0].scalar_type(), "m"); need(v[i], m[0].scalar_type(), "v");
    TORCH_CHECK(m[0].scalar_type() == at::kFloat || m[0].scalar_type() == at::kBFloat16, "moments must be fp32 or bf16");
    TORCH_CHECK(w[i].dim() == 3 && w[i].size(0) == F_pitch && w[i].size(2) == d, "decoder tensor must be [F, R, d]");
    a.w[i] = w[i].data_ptr(); a.m[i] = static_cast<float*>(m[i].data_ptr()); a.v[i] = static_cast<float*>(v[i].data_ptr()); a.rows[i] = int(w[i].size(1));
  }
  a.ntensors = int(w.size()); a.L = int(L); a.B = int(B); a.d = int(d); a.F_pitch = int(F_pitch); a.tying = int(tying); a.weights_bf16 = w16;
  a.feat_off = feat_off.data_ptr<int>(); a.fcsr_tok = fcsr_tok.data_ptr<int>(); a.fcsr_val = fcsr_val.data_ptr<float>();
  need(gs, t16_of(half), "gs");
  a.gs = gs.data_ptr(); a.grad_a = opt_ptr<float>(grad_a); a.pen_coef = opt_ptr<const float>(pen_coef); a.norm2_out = opt_ptr<float>(norm2_out);
  a.feat_offset = opt_ptr<const float>(feat_offset); a.feat_scale = opt_ptr<const float>(feat_scale);
  a.dgrad_row0 = opt_ptr<const float>(dgrad_row0);
  if (a.dgrad_row0) TORCH_CHECK(dgrad_row0->scalar_type() == at::kFloat && dgrad_row0->numel() == int64_t(w.size()) * F_pitch * d, "dgrad_row0 must be fp32 [ntensors, F, d]");
  a.extra_idx = opt_ptr<const int>(extra_idx); a.extra_rows = opt_ptr<const float>(extra_rows);
  if (a.extra_idx) {
    TORCH_CHECK(extra_idx->scalar_type() == at::kInt && extra_idx->numel() >= int64_t(w.size()) * F_pitch && a.extra_rows != nullptr && extra_rows->scalar_type() == at::kFloat,
                "extra_idx: int32 [ntensors * F]; extra_rows: fp32 [n, d]");
  }
  a.h = hyper_from(hyper);
  a.status = opt_ptr<int>(status);
  a.moments_bf16 = m[0].scalar_type() == at::kBFloat16 ? 1 : 0;
  a.ctl = ctl_ptr(ctl);
  a.norm_only = norm_only ? 1 : 0;
  a.d_feat_offset = opt_ptr<float>(d_feat_offset); a.d_feat_scale = opt_ptr<float>(d_feat_scale);
  for (const OptTensor* t : {&d_feat_offset, &d_feat_scale})
    if (t->has_value() && (*t)->defined())
      TORCH_CHECK((*t)->is_cuda() && (*t)->scalar_type() == at::kFloat && (*t)->is_contiguous() && (*t)->numel() >= L * F_pitch, "affine gradient accumulators: fp32 [L, F]");
  c10::cuda::CUDAGuard guard(gs.device());
  check(CLT_PICK(half, clt_decoder_rows_adam)(&a, num_sms(), cur_stream()), "decoder_rows_adam");
}

void encoder_rows_adam(Tensor& w, Tensor& m, Tensor& v, Tensor& bias, Tensor& bias_m, Tensor& bias_v, const Tensor& feat_off,
                       const Tensor& fcsr_tok, const Tensor& delta, const Tensor& x, const OptTensor& dense_grad,
                       const OptTensor& dense_bias_grad, const std::vector<double>& hyper, const OptTensor& status,
                       const OptTensor& extra_idx, const OptTensor& extra_rows, const OptTensor& extra_bias, const OptTensor& ctl, bool norm_only) {
  const bool half = is_half(x, "x");
  const bool w16 = w.scalar_type() != at::kFloat;
  const bool mbf16 = m.scalar_type() == at::kBFloat16;
  need(w, w16 ? t16_of(half) : at::kFloat, "w"); need(m, mbf16 ? at::kBFloat16 : at::kFloat, "m"); need(v, mbf16 ? at::kBFloat16 : at::kFloat, "v");
  need(bias, w16 ? t16_of(half) : at::kFloat, "bias"); need(bias_m, at::kFloat, "bias_m"); need(bias_v, at::kFloat, "bias_v");
  need(x, t16_of(half), "x"); need(delta, at::kFloat, "delta");
  CltEncAdamArgs a;
  std::memset(&a, 0, sizeof(a));
  a.w = w.data_ptr(); a.m = static_cast<float*>(m.data_ptr()); a.v = static_cast<float*>(v.data_ptr());
  a.moments_bf16 = mbf16 ? 1 : 0;
  a.bias = bias.data_ptr(); a.bias_m = bias_m.data_ptr<float>(); a.bias_v = bias_v.data_ptr<float>();
  a.L = int(w.size(0)); a.F_pitch = int(w.size(1)); a.d = int(w.size(2)); a.B = int(x.size(1)); a.weights_bf16 = w16;
  a.feat_off = feat_off.data_ptr<int>(); a.fcsr_tok = fcsr_tok.data_ptr<int>(); a.delta = delta.data_ptr<float>(); a.x = x.data_ptr();
  a.dense_grad = opt_ptr<const float>(dense_grad); a.dense_bias_grad = opt_ptr<const float>(dense_bias_grad);
  a.extra_idx = opt_ptr<const int>(extra_idx); a.extra_rows = opt_ptr<const float>(extra_rows); a.extra_bias = opt_ptr<const float>(extra_bias);
  a.h = hyper_from(hyper);
  a.status = opt_ptr<int>(status);
  a.ctl = ctl_ptr(ctl);
  a.norm_only = norm_only ? 1 : 0;
  c10::cuda::CUDAGuard guard(w.device());
  check(CLT_PICK(half, clt_encoder_rows_adam)(&a, num_sms(), cur_stream()), "encoder_rows_adam");
}

// seed_scaled: the gradient carries the loss scale; norm_weight > 0: norm-only pass (adds norm_weight * |g|^2 to the control block)
void dense_adam(Tensor& w, Tensor& m, Tensor& v, const Tensor& grad, const std::vector<double>& hyper, const OptTensor& ctl, bool seed_scaled,
                double norm_weight) {
  const bool w16 = w.scalar_type() != at::kFloat;
  const bool half = w16 && is_half(w, "w");
  need(w, w16 ? t16_of(half) : at::kFloat, "w"); need(m, at::kFloat, "m"); need(v, at::kFloat, "v"); need(grad, at::kFloat, "grad");
  TORCH_CHECK(w.numel() == m.numel() && w.numel() == v.numel() && w.numel() == grad.numel(), "size mismatch");
  const CltAdamHyper h = hyper_from(hyper);
  c10::cuda::CUDAGuard guard(w.device());
  check(CLT_PICK(half, clt_dense_adam)(w.data_ptr(), m.data_ptr<float>(), v.data_ptr<float>(), grad.data_ptr<float>(), w.numel(), w16, &h,
                                       ctl_ptr(ctl), seed_scaled ? 1 : 0, float(norm_weight), cur_stream()), "dense_adam");
}

void decoder_norm2(const Tensor& w, Tensor& out) {
  const bool w16 = w.scalar_type() != at::kFloat;
  const bool half = w16 && is_half(w, "w");
  need(w, w16 ? t16_of(half) : at::kFloat, "w"); need(out, at::kFloat, "out");
  TORCH_CHECK(w.dim() == 3 && out.numel() >= w.size(0), "w must be [F, R, d], out [F]");
  c10::cuda::CUDAGuard guard(w.device());
  check(CLT_PICK(half, clt_decoder_norm2)(w.data_ptr(), out.data_ptr<float>(), int(w.size(0)), int(w.size(1)), int(w.size(2)), w16, cur_stream()), "decoder_norm2");
}

void sparsity_penalty(const Tensor& feat_off, const Tensor& fcsr_val, const Tensor& norm2, double lambda, double c, Tensor& grad_a,
                      Tensor& pen_coef, Tensor& penalty_out) {
  need(feat_off, at::kInt, "feat_off"); need(fcsr_val, at::kFloat, "fcsr_val"); need(norm2, at::kFloat, "norm2");
  need(grad_a, at::kFloat, "grad_a"); need(pen_coef, at::kFloat, "pen_coef"); need(penalty_out, at::kDouble, "penalty_out");
  const int ncols = int(norm2.numel());
  TORCH_CHECK(feat_off.numel() >= ncols + 1 && pen_coef.numel() >= ncols, "size mismatch");
  c10::cuda::CUDAGuard guard(norm2.device());
  check(clt_sparsity_penalty(feat_off.data_ptr<int>(), fcsr_val.data_ptr<float>(), norm2.data_ptr<float>(), ncols, float(lambda), float(c),
                             grad_a.data_ptr<float>(), pen_coef.data_ptr<float>(), penalty_out.data_ptr<double>(), cur_stream()),
        "sparsity_penalty");
}

// Device-side decision of a step (see step.cu): phase 0 after the loss kernels, phase 1 after the gradient-norm pre-pass.
// scalars: fp64 [n] further loss sums (penalty, pre-activation, auxiliary); losses: fp32 [8] out.
void step_control(Tensor& ctl, const OptTensor& status, Tensor& sq_err, const OptTensor& scalars, Tensor& losses, double inv_bd, int64_t phase,
                  bool dynamic_scale, int64_t growth_interval, double max_norm, int64_t world, int64_t rank,
                  const std::vector<int64_t>& ex_data, const std::vector<int64_t>& ex_flags, int64_t slot_elems, int64_t seq, int64_t round) {
  need(sq_err, at::kDouble, "sq_err"); need(losses, at::kFloat, "losses");
  TORCH_CHECK(losses.numel() >= 8, "losses needs 8 elements");
  CltStepControlArgs a;
  std::memset(&a, 0, sizeof(a));
  a.ctl = ctl_ptr(ctl);
  TORCH_CHECK(a.ctl != nullptr, "ctl is required");
  a.status = opt_ptr<const int>(status);
  a.sq_err = sq_err.data_ptr<double>(); a.L = int(sq_err.numel());
  if (scalars.has_value() && scalars->defined()) { need(*scalars, at::kDouble, "scalars"); a.scalars = scalars->data_ptr<double>(); a.n_scalars = int(scalars->numel()); }
  a.losses = losses.data_ptr<float>(); a.inv_bd = inv_bd; a.phase = int(phase); a.dynamic_scale = dynamic_scale ? 1 : 0;
  a.growth_interval = int(growth_interval); a.max_norm = float(max_norm); a.round = int(round);
  CltExchangeArgs ex;
  const bool multi = fill_exchange(ex, world, rank, ex_data, ex_flags, slot_elems, seq);
  c10::cuda::CUDAGuard guard(sq_err.device());
  check(clt_step_control(&a, multi ? &ex : nullptr, cur_stream()), "step_control");
}

// Decoder-bias gradient from the column sums of the gradient seed (sel [L, n_bias]: which targets a bias feeds) + AdamW.
void decoder_bias_adam(Tensor& bias, Tensor& m, Tensor& v, const Tensor& sel, const Tensor& gs_sum, const OptTensor& extra,
                       const std::vector<double>& hyper, const OptTensor& ctl, double norm_weight) {
  const bool w16 = bias.scalar_type() != at::kFloat;
  const bool half = w16 && is_half(bias, "bias");
  need(bias, w16 ? t16_of(half) : at::kFloat, "bias"); need(m, at::kFloat, "m"); need(v, at::kFloat, "v");
  need(sel, at::kFloat, "sel"); need(gs_sum, at::kFloat, "gs_sum");
  const int n_bias = bias.size(0), d = bias.size(1), L = gs_sum.size(0);
  TORCH_CHECK(sel.dim() == 2 && sel.size(0) == L && sel.size(1) == n_bias && gs_sum.size(1) == d && m.numel() == bias.numel() && v.numel() == bias.numel(), "shape mismatch");
  if (extra.has_value() && extra->defined()) { need(*extra, at::kFloat, "extra"); TORCH_CHECK(extra->numel() == bias.numel(), "extra must have the shape of bias"); }
  const CltAdamHyper h = hyper_from(hyper);
  c10::cuda::CUDAGuard guard(bias.device());
  check(CLT_PICK(half, clt_decoder_bias_adam)(bias.data_ptr(), m.data_ptr<float>(), v.data_ptr<float>(), sel.data_ptr<float>(), gs_sum.data_ptr<float>(),
                                              opt_ptr<const float>(extra), n_bias, L, d, w16, &h, ctl_ptr(ctl), float(norm_weight), cur_stream()),
        "decoder_bias_adam");
}

// End of a step: dead-feature counters (optional) and bias_sum[t] = sum_p sel[t, p] bias[p] (optional).
void step_finish(const OptTensor& counter, const OptTensor& fired, const OptTensor& bias, const OptTensor& sel, const OptTensor& bias_sum) {
  long long* cnt = nullptr; unsigned char* frd = nullptr; int ncols = 0;
  if (counter.has_value() && counter->defined()) {
    need(*counter, at::kLong, "counter"); TORCH_CHECK(fired.has_value() && fired->defined(), "counter needs fired"); need(*fired, at::kByte, "fired");
    TORCH_CHECK(counter->numel() == fired->numel(), "counter / fired size mismatch");
    cnt = reinterpret_cast<long long*>(counter->data_ptr<int64_t>()); frd = fired->data_ptr<uint8_t>(); ncols = int(counter->numel());
  }
  const void* bp = nullptr; const float* sp = nullptr; float* bs = nullptr; int n_bias = 0, L = 0, d = 0; bool w16 = false, half = false;
  at::Device dev = counter.has_value() && counter->defined() ? counter->device() : bias->device();
  if (bias_sum.has_value() && bias_sum->defined()) {
    TORCH_CHECK(bias.has_value() && sel.has_value(), "bias_sum needs bias and sel");
    w16 = bias->scalar_type() != at::kFloat; half = w16 && is_half(*bias, "bias");
    need(*bias, w16 ? t16_of(half) : at::kFloat, "bias"); need(*sel, at::kFloat, "sel"); need(*bias_sum, at::kFloat, "bias_sum");
    n_bias = bias->size(0); d = bias->size(1); L = sel->size(0);
    TORCH_CHECK(sel->size(1) == n_bias && bias_sum->numel() == 1LL * L * d, "shape mismatch");
    bp = bias->data_ptr(); sp = sel->data_ptr<float>(); bs = bias_sum->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(dev);
  check(CLT_PICK(half, clt_step_finish)(cnt, frd, ncols, bp, sp, bs, n_bias, L, d, w16, cur_stream()), "step_finish");
}

// JumpReLU threshold update from the window sums (see step.cu); theta holds exp(log_theta) and is refreshed.
void theta_adam(Tensor& log_theta, Tensor& m, Tensor& v, Tensor& theta, const Tensor& S1, const Tensor& S2, const Tensor& norm2,
                const Tensor& feat_off, const Tensor& fcsr_val, int64_t tying, double c_g, double lambda, double c, double bandwidth,
                const std::vector<double>& hyper, const OptTensor& ctl, double norm_weight, const OptTensor& grad_out) {
  const bool w16 = log_theta.scalar_type() != at::kFloat;
  const bool half = w16 && is_half(log_theta, "log_theta");
  need(log_theta, w16 ? t16_of(half) : at::kFloat, "log_theta"); need(m, at::kFloat, "m"); need(v, at::kFloat, "v"); need(theta, at::kFloat, "theta");
  need(S1, at::kFloat, "S1"); need(S2, at::kFloat, "S2"); need(norm2, at::kFloat, "norm2"); need(feat_off, at::kInt, "feat_off"); need(fcsr_val, at::kFloat, "fcsr_val");
  TORCH_CHECK(log_theta.dim() == 2 && theta.sizes() == log_theta.sizes() && S1.sizes() == log_theta.sizes() && S2.sizes() == log_theta.sizes() &&
              m.sizes() == log_theta.sizes() && v.sizes() == log_theta.sizes() && norm2.numel() >= log_theta.numel() && feat_off.numel() >= log_theta.numel() + 1,
              "shape mismatch");
  CltThetaAdamArgs a;
  std::memset(&a, 0, sizeof(a));
  a.log_theta = log_theta.data_ptr(); a.m = m.data_ptr<float>(); a.v = v.data_ptr<float>(); a.theta = theta.data_ptr<float>();
  a.S1 = S1.data_ptr<float>(); a.S2 = S2.data_ptr<float>(); a.norm2 = norm2.data_ptr<float>();
  a.feat_off = feat_off.data_ptr<int>(); a.fcsr_val = fcsr_val.data_ptr<float>();
  a.L = int(log_theta.size(0)); a.pitch = int(log_theta.size(1)); a.tying = int(tying); a.weights_16 = w16;
  a.c_g = float(c_g); a.lambda = float(lambda); a.c = float(c); a.bandwidth = float(bandwidth);
  a.h = hyper_from(hyper); a.ctl = ctl_ptr(ctl); a.norm_weight = float(norm_weight); a.grad_out = opt_ptr<float>(grad_out);
  c10::cuda::CUDAGuard guard(log_theta.device());
  check(CLT_PICK(half, clt_theta_adam)(&a, cur_stream()), "theta_adam");
}

void theta_exp(const Tensor& log_theta, Tensor& theta) {
  const bool w16 = log_theta.scalar_type() != at::kFloat;
  const bool half = w16 && is_half(log_theta, "log_theta");
  need(log_theta, w16 ? t16_of(half) : at::kFloat, "log_theta"); need(theta, at::kFloat, "theta");
  TORCH_CHECK(theta.numel() == log_theta.numel(), "size mismatch");
  c10::cuda::CUDAGuard guard(log_theta.device());
  check(CLT_PICK(half, clt_theta_exp)(log_theta.data_ptr(), theta.data_ptr<float>(), log_theta.numel(), w16, cur_stream()), "theta_exp");
}

// out = ((in - mean) * inv_std) * mul cast to out's 16-bit type; in: [..., rows, d] fp32 / bf16 / fp16, mean / inv_std (optional):
// one row of d statistics per rows_per_stat consecutive rows.
void normalize_cast(const Tensor& in, Tensor& out, const OptTensor& mean, const OptTensor& inv_std, int64_t rows_per_stat, double mul) {
  const bool half = is_half(out, "out");
  need(out, t16_of(half), "out");
  TORCH_CHECK(in.is_cuda() && in.is_contiguous() && in.numel() == out.numel() && in.dim() >= 2, "in / out: contiguous CUDA tensors of one shape");
  const int in_type = in.scalar_type() == at::kFloat ? 0 : in.scalar_type() == at::kBFloat16 ? 1 : in.scalar_type() == at::kHalf ? 2 : -1;
  TORCH_CHECK(in_type >= 0, "in must be fp32, bf16 or fp16");
  const int d = int(in.size(-1));
  const long long rows = in.numel() / d;
  const float* mp = nullptr; const float* sp = nullptr;
  if (mean.has_value() && mean->defined()) {
    need(*mean, at::kFloat, "mean"); TORCH_CHECK(inv_std.has_value() && inv_std->defined(), "mean needs inv_std"); need(*inv_std, at::kFloat, "inv_std");
    TORCH_CHECK(rows_per_stat > 0 && rows % rows_per_stat == 0 && mean->numel() == (rows / rows_per_stat) * d && inv_std->numel() == mean->numel(),
                "statistics must be [rows / rows_per_stat, d]");
    mp = mean->data_ptr<float>(); sp = inv_std->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(in.device());
  check(CLT_PICK(half, clt_normalize_cast)(in.data_ptr(), in_type, out.data_ptr(), mp, sp, rows, int(rows_per_stat > 0 ? rows_per_stat : rows), d, float(mul),
                                           cur_stream()), "normalize_cast");
}

// hist[k] (int64 [n_scales + 1], zeroed here) = number of elements of x [B, F] whose ratio x / theta[f] satisfies exactly the
// first k of the ascending `scales`: L0(scales[j]) = sum_{k > j} hist[k] / B.
void scale_histogram(const Tensor& x, const Tensor& theta, const Tensor& scales, Tensor& hist) {
  const bool half = is_half(x, "x");
  need(x, t16_of(half), "x"); need(theta, at::kFloat, "theta"); need(scales, at::kFloat, "scales"); need(hist, at::kLong, "hist");
  TORCH_CHECK(x.dim() == 2 && theta.numel() >= x.size(1) && hist.numel() == scales.numel() + 1, "x [B, F], theta [F], hist [n_scales + 1]");
  c10::cuda::CUDAGuard guard(x.device());
  hist.zero_();
  check(CLT_PICK(half, clt_scale_histogram)(x.data_ptr(), theta.data_ptr<float>(), scales.data_ptr<float>(), int(scales.numel()),
                                            reinterpret_cast<unsigned long long*>(hist.data_ptr<int64_t>()), int(x.size(0)), int(x.size(1)), x.size(1),
                                            cur_stream()), "scale_histogram");
}

// C[g] = alpha * sum over the segments (a, b) of group g of A[a] @ B[b]^T.  A [LA, M, K], B [LB, N, K] (16-bit, contiguous),
// C [G, M, N] fp32 or 16-bit; group_off int32 [G + 1], segs int32 [n_segs, 2] on the device.
void dense_gemm(const Tensor& A, const Tensor& B, Tensor& C, const Tensor& group_off, const Tensor& segs, double alpha, Tensor& status) {
  const bool half = is_half(A, "A");
  need(A, t16_of(half), "A"); need(B, t16_of(half), "B"); need(group_off, at::kInt, "group_off"); need(segs, at::kInt, "segs"); need(status, at::kInt, "status");
  TORCH_CHECK(A.dim() == 3 && B.dim() == 3 && C.dim() == 3 && A.size(2) == B.size(2) && C.size(1) == A.size(1) && C.size(2) == B.size(1), "A [LA, M, K], B [LB, N, K], C [G, M, N]");
  const bool out_f32 = C.scalar_type() == at::kFloat;
  need(C, out_f32 ? at::kFloat : t16_of(half), "C");
  const int G = int(C.size(0));
  TORCH_CHECK(group_off.numel() == G + 1 && segs.dim() == 2 && segs.size(1) == 2, "group_off [G + 1], segs [n, 2]");
  c10::cuda::CUDAGuard guard(A.device());
  check(CLT_PICK(half, clt_dense_gemm)(A.data_ptr(), int(A.size(0)), A.size(2), A.size(1) * A.size(2), B.data_ptr(), int(B.size(0)), B.size(2),
                                       B.size(1) * B.size(2), C.data_ptr(), out_f32 ? 1 : 0, group_off.data_ptr<int>(), segs.data_ptr<int>(), G,
                                       int(A.size(1)), int(B.size(1)), int(A.size(2)), float(alpha), status.data_ptr<int>(), num_sms(), cur_stream()),
        "dense_gemm");
}

// out[l] = in[l]^T for 16-bit [L, R, C] tensors; with `mask` (shape of `in`) the elements whose mask value is zero become zero
void transpose16(const Tensor& in, Tensor& out, const OptTensor& mask) {
  const bool half = is_half(in, "in");
  need(in, t16_of(half), "in"); need(out, t16_of(half), "out");
  if (mask.has_value() && mask->defined()) {
    need(*mask, t16_of(half), "mask");
    TORCH_CHECK(mask->sizes() == in.sizes(), "mask: the shape of in");
  }
  TORCH_CHECK(in.dim() == 3 && out.dim() == 3 && out.size(0) == in.size(0) && out.size(1) == in.size(2) && out.size(2) == in.size(1), "in [L, R, C], out [L, C, R]");
  c10::cuda::CUDAGuard guard(in.device());
  check(CLT_PICK(half, clt_transpose16)(in.data_ptr(), out.data_ptr(), int(in.size(0)), int(in.size(1)), int(in.size(2)), in.size(2),
                                        in.size(1) * in.size(2), opt_ptr<const void>(mask), cur_stream()), "transpose16");
}

// ind[l][f, b] = 1[pre[l][b, f] < 0]; bias_grad[l, f] -= c * count; loss[0] += c * sum relu(-pre)   (c = coef / numel)
void negative_indicator(const Tensor& pre, Tensor& ind, Tensor& bias_grad, Tensor& loss, int64_t f_valid, double coef_over_numel) {
  const bool half = is_half(pre, "pre");
  need(pre, t16_of(half), "pre"); need(ind, t16_of(half), "ind"); need(bias_grad, at::kFloat, "bias_grad"); need(loss, at::kDouble, "loss");
  TORCH_CHECK(pre.dim() == 3 && ind.dim() == 3 && ind.size(0) == pre.size(0) && ind.size(1) == pre.size(2) && ind.size(2) == pre.size(1) &&
              bias_grad.numel() == pre.size(0) * pre.size(2) && loss.numel() >= 1, "pre [L, B, F], ind [L, F, B], bias_grad [L, F]");
  c10::cuda::CUDAGuard guard(pre.device());
  check(CLT_PICK(half, clt_negative_indicator)(pre.data_ptr(), ind.data_ptr(), bias_grad.data_ptr<float>(), loss.data_ptr<double>(), int(pre.size(0)),
                                               int(pre.size(1)), int(pre.size(2)), int(f_valid), pre.size(2), float(coef_over_numel), cur_stream()),
        "negative_indicator");
}

// ---- auxiliary loss on dead features (aux.cu)
// dead_cols [L, nd_cap], nd / nd_all [L], extra_idx [L * F_pitch] from the counters: feature f of layer l is dead when counter > window
void aux_compact(const Tensor& counter, int64_t window, int64_t L, int64_t f_valid, Tensor& dead_cols, Tensor& nd, Tensor& nd_all, Tensor& extra_idx) {
  need(counter, at::kLong, "counter"); need(dead_cols, at::kInt, "dead_cols"); need(nd, at::kInt, "nd"); need(nd_all, at::kInt, "nd_all");
  need(extra_idx, at::kInt, "extra_idx");
  TORCH_CHECK(counter.numel() % L == 0 && dead_cols.dim() == 2 && dead_cols.size(0) == L && nd.numel() == L && nd_all.numel() == L &&
              extra_idx.numel() == counter.numel(), "counter [L * F], dead_cols [L, nd_cap], nd [L], nd_all [L], extra_idx [L * F]");
  c10::cuda::CUDAGuard guard(counter.device());
  check(clt_aux_compact(reinterpret_cast<const long long*>(counter.data_ptr<int64_t>()), window, int(L), int(counter.numel() / L), int(f_valid),
                        int(dead_cols.size(1)), dead_cols.data_ptr<int>(), nd.data_ptr<int>(), nd_all.data_ptr<int>(), extra_idx.data_ptr<int>(),
                        cur_stream()), "aux_compact");
}

// A [L, B, nd_cap]: per token the top k_aux dead pre-activations of the layer (the others zero).  Either `pre` [L, B, F] (the
// stored pre-activations, gathered at the dead columns) or `enc_bias` [L, F] (A already holds x W_dead^T; the bias is added and
// A is rewritten in place).
void aux_gather_select(const OptTensor& pre, const OptTensor& enc_bias, const Tensor& dead_cols, const Tensor& nd, const Tensor& nd_all,
                       int64_t k_aux_max, Tensor& A, const OptTensor& bias_scratch) {
  const bool half = is_half(A, "A");
  need(A, t16_of(half), "A"); need(dead_cols, at::kInt, "dead_cols"); need(nd, at::kInt, "nd"); need(nd_all, at::kInt, "nd_all");
  const bool from_pre = pre.has_value() && pre->defined();
  TORCH_CHECK(from_pre != (enc_bias.has_value() && enc_bias->defined()), "either pre or enc_bias");
  TORCH_CHECK(A.dim() == 3 && A.size(2) == dead_cols.size(1) && dead_cols.size(0) == A.size(0), "A [L, B, nd_cap], dead_cols [L, nd_cap]");
  const void* pre_p = nullptr; const void* bias_p = nullptr;
  int64_t ld = 0, stride = 0, f_pitch = 0; int bias16 = 0;
  if (from_pre) {
    need(*pre, t16_of(half), "pre");
    TORCH_CHECK(pre->dim() == 3 && pre->size(0) == A.size(0) && pre->size(1) == A.size(1), "pre [L, B, F]");
    pre_p = pre->data_ptr(); ld = pre->size(2); stride = pre->size(1) * pre->size(2);
  } else {
    TORCH_CHECK(enc_bias->is_cuda() && enc_bias->is_contiguous() && enc_bias->dim() == 2 && enc_bias->size(0) == A.size(0) &&
                (enc_bias->scalar_type() == at::kFloat || enc_bias->scalar_type() == t16_of(half)), "enc_bias [L, F], fp32 or the 16-bit type");
    bias_p = enc_bias->data_ptr(); f_pitch = enc_bias->size(1); bias16 = enc_bias->scalar_type() == at::kFloat ? 0 : 1;
    TORCH_CHECK(bias_scratch.has_value() && bias_scratch->defined() && bias_scratch->is_cuda() && bias_scratch->scalar_type() == at::kFloat &&
                bias_scratch->is_contiguous() && bias_scratch->numel() >= A.size(0) * A.size(2), "bias_scratch: fp32 [L, nd_cap]");
  }
  c10::cuda::CUDAGuard guard(A.device());
  check(CLT_PICK(half, clt_aux_gather_select)(pre_p, ld, stride, bias_p, bias16, int(f_pitch), opt_ptr<float>(bias_scratch), dead_cols.data_ptr<int>(), nd.data_ptr<int>(),
                                              nd_all.data_ptr<int>(), int(A.size(2)), int(k_aux_max), int(A.size(0)), int(A.size(1)), A.data_ptr(),
                                              cur_stream()), "aux_gather_select");
}

// W0 [L, nd_cap, d]: first row (the layer's own target) of every dead feature's decoder block
void aux_gather_rows(const std::vector<Tensor>& dec_w, const Tensor& dead_cols, const Tensor& nd, Tensor& W0) {
  TORCH_CHECK(!dec_w.empty() && dec_w.size() <= 32 && W0.dim() == 3 && int64_t(dec_w.size()) == W0.size(0), "one decoder tensor per layer (at most 32)");
  const bool half = is_half(W0, "W0");
  CltAuxRowsArgs a{};
  for (size_t i = 0; i < dec_w.size(); ++i) {
    need(dec_w[i], t16_of(half), "dec_w");
    TORCH_CHECK(dec_w[i].dim() == 3 && dec_w[i].size(2) == W0.size(2), "dec_w[l] [F, R, d]");
    a.w[i] = dec_w[i].data_ptr(); a.rows[i] = int(dec_w[i].size(1));
  }
  c10::cuda::CUDAGuard guard(W0.device());
  check(CLT_PICK(half, clt_aux_gather_rows)(&a, dead_cols.data_ptr<int>(), nd.data_ptr<int>(), int(W0.size(1)), int(W0.size(0)), int(W0.size(2)),
                                            W0.data_ptr(), cur_stream()), "aux_gather_rows");
}

// r = recon + bias[bias_row[l]] - residual(gs); loss[0] += factor mean r^2; g = dL/d recon (16-bit); gs += the term's gradient through the residual
void aux_residual(const Tensor& recon, const Tensor& bias, const Tensor& bias_row, const c10::optional<Tensor>& sigma, Tensor& gs, Tensor& g_out,
                  Tensor& loss, const Tensor& nd, const c10::optional<Tensor>& ctl, double factor, bool scale_g) {
  const bool half = is_half(gs, "gs");
  need(recon, at::kFloat, "recon"); need(gs, t16_of(half), "gs"); need(g_out, t16_of(half), "g_out"); need(loss, at::kDouble, "loss");
  need(bias_row, at::kInt, "bias_row"); need(nd, at::kInt, "nd");
  TORCH_CHECK(bias.is_cuda() && bias.is_contiguous() && (bias.scalar_type() == at::kFloat || bias.scalar_type() == t16_of(half)), "bias: fp32 or the 16-bit type");
  TORCH_CHECK(recon.dim() == 3 && gs.sizes() == recon.sizes() && g_out.sizes() == recon.sizes(), "recon, gs, g_out [L, B, d]");
  c10::cuda::CUDAGuard guard(gs.device());
  check(CLT_PICK(half, clt_aux_residual)(recon.data_ptr<float>(), bias.data_ptr(), bias.scalar_type() == at::kFloat ? 0 : 1, bias_row.data_ptr<int>(),
                                         opt_ptr<float>(sigma), gs.data_ptr(), g_out.data_ptr(), loss.data_ptr<double>(), nd.data_ptr<int>(),
                                         ctl_ptr(ctl), int(recon.size(0)), int(recon.size(1)), int(recon.size(2)), float(factor), scale_g ? 1 : 0, cur_stream()),
        "aux_residual");
}

// buf *= 1 / loss scale (read from the step control block on the device)
void unscale(Tensor& buf, const Tensor& ctl) {
  need(buf, at::kFloat, "buf");
  c10::cuda::CUDAGuard guard(buf.device());
  check(clt_unscale(buf.data_ptr<float>(), buf.numel(), ctl_ptr(ctl), cur_stream()), "unscale");
}

// out[r] = sum of row r of the 16-bit matrix in [rows, n]
void rowsum16(const Tensor& in, Tensor& out) {
  const bool half = is_half(in, "in");
  need(in, t16_of(half), "in"); need(out, at::kFloat, "out");
  const int64_t n = in.size(-1);
  TORCH_CHECK(out.numel() * n == in.numel(), "out: one value per row");
  c10::cuda::CUDAGuard guard(in.device());
  check(CLT_PICK(half, clt_rowsum16)(in.data_ptr(), out.data_ptr<float>(), out.numel(), int(n), cur_stream()), "rowsum16");
}

// dst[r, :] += src[extra_idx[r], :] (and dst_bias[r] += src_bias[extra_idx[r]]) for the rows with extra_idx >= 0
void scatter_add_rows(Tensor& dst, const c10::optional<Tensor>& dst_bias, const Tensor& src, const c10::optional<Tensor>& src_bias, const Tensor& extra_idx) {
  need(dst, at::kFloat, "dst"); need(src, at::kFloat, "src"); need(extra_idx, at::kInt, "extra_idx");
  const int64_t d = dst.size(-1);
  TORCH_CHECK(src.size(-1) == d && dst.numel() == extra_idx.numel() * d, "dst [rows, d], src [n, d], extra_idx [rows]");
  TORCH_CHECK(dst_bias.has_value() == src_bias.has_value(), "both bias tensors or none");
  c10::cuda::CUDAGuard guard(dst.device());
  check(clt_scatter_add_rows(dst.data_ptr<float>(), opt_ptr<float>(dst_bias), src.data_ptr<float>(), opt_ptr<float>(src_bias), extra_idx.data_ptr<int>(),
                             extra_idx.numel(), int(d), cur_stream()), "scatter_add_rows");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  const auto none = py::none();
  m.def("encoder_gemm", &encoder_gemm);
  m.def("colstats", &colstats);
  m.def("colstats_from_tiles", &colstats_from_tiles);
  m.def("batchtopk_select", &batchtopk_select);
  m.def("threshold_select", &threshold_select);
  m.def("token_topk_select", &token_topk_select, py::arg("x"), py::arg("mean"), py::arg("rstd"), py::arg("col_pitch"), py::arg("k"), py::arg("ctl"),
        py::arg("ent_tok"), py::arg("ent_col"), py::arg("ent_val"), py::arg("status"), py::arg("f_valid") = 0);
  m.def("token_topk_tp", &token_topk_tp);
  m.def("theta_grad_gemm", &theta_grad_gemm, py::arg("gs"), py::arg("dec_w"), py::arg("preact"), py::arg("theta"), py::arg("bandwidth"),
        py::arg("S1"), py::arg("S2"), py::arg("status"), py::arg("tying") = 0, py::arg("gs_cum") = none);
  m.def("build_csr", &build_csr);
  m.def("dead_counter_update", &dead_counter_update);
  m.def("sparse_decode", &sparse_decode, py::arg("dec_w"), py::arg("L"), py::arg("B"), py::arg("d"), py::arg("col_pitch"), py::arg("tying"),
        py::arg("tok_off"), py::arg("tcsr_col"), py::arg("tcsr_val"), py::arg("feat_offset"), py::arg("feat_scale"), py::arg("yhat_partial"),
        py::arg("bias_sum"), py::arg("addend"), py::arg("target"), py::arg("sigma"), py::arg("gs"), py::arg("yhat_out"), py::arg("sq_err"),
        py::arg("mode"), py::arg("stage_peers"), py::arg("rows_per_rank"), py::arg("rank"), py::arg("status"), py::arg("ctl") = none,
        py::arg("rows_limit") = 0);
  m.def("recon_epilogue", &recon_epilogue, py::arg("yhat_sum"), py::arg("bias_sum"), py::arg("addend"), py::arg("target"), py::arg("sigma"),
        py::arg("gs"), py::arg("yhat_out"), py::arg("sq_err"), py::arg("row0"), py::arg("nrows"), py::arg("ctl") = none);
  m.def("gs_colsum", &gs_colsum);
  m.def("gs_suffix_sum", &gs_suffix_sum);
  m.def("peer_barrier", &peer_barrier, py::arg("flag_ptrs"), py::arg("rank"), py::arg("slot"), py::arg("seq"), py::arg("status"),
        py::arg("timeout_s") = 0.0);
  m.def("memcpy_2d", &memcpy_2d);
  m.def("owner_reduce_loss", &owner_reduce_loss, py::arg("stage"), py::arg("gs_ptrs"), py::arg("rank"), py::arg("bias_sum"), py::arg("addend"),
        py::arg("target"), py::arg("sigma"), py::arg("yhat_out"), py::arg("sq_err"), py::arg("rows_per_rank"), py::arg("ctl") = none);
  m.def("decoder_rows_adam", &decoder_rows_adam, py::arg("w"), py::arg("m"), py::arg("v"), py::arg("L"), py::arg("B"), py::arg("d"),
        py::arg("F_pitch"), py::arg("tying"), py::arg("feat_off"), py::arg("fcsr_tok"), py::arg("fcsr_val"), py::arg("gs"), py::arg("grad_a"),
        py::arg("pen_coef"), py::arg("norm2_out"), py::arg("feat_offset"), py::arg("feat_scale"), py::arg("dgrad_row0"), py::arg("hyper"),
        py::arg("status"), py::arg("extra_idx") = none, py::arg("extra_rows") = none, py::arg("ctl") = none, py::arg("norm_only") = false,
        py::arg("d_feat_offset") = none, py::arg("d_feat_scale") = none);
  m.def("encoder_rows_adam", &encoder_rows_adam, py::arg("w"), py::arg("m"), py::arg("v"), py::arg("bias"), py::arg("bias_m"), py::arg("bias_v"),
        py::arg("feat_off"), py::arg("fcsr_tok"), py::arg("delta"), py::arg("x"), py::arg("dense_grad"), py::arg("dense_bias_grad"),
        py::arg("hyper"), py::arg("status"), py::arg("extra_idx") = none, py::arg("extra_rows") = none, py::arg("extra_bias") = none,
        py::arg("ctl") = none, py::arg("norm_only") = false);
  m.def("dense_adam", &dense_adam, py::arg("w"), py::arg("m"), py::arg("v"), py::arg("grad"), py::arg("hyper"), py::arg("ctl") = none,
        py::arg("seed_scaled") = false, py::arg("norm_weight") = 0.0);
  m.def("decoder_norm2", &decoder_norm2);
  m.def("sparsity_penalty", &sparsity_penalty);
  m.def("step_control", &step_control, py::arg("ctl"), py::arg("status"), py::arg("sq_err"), py::arg("scalars"), py::arg("losses"),
        py::arg("inv_bd"), py::arg("phase") = 0, py::arg("dynamic_scale") = false, py::arg("growth_interval") = 2000, py::arg("max_norm") = 0.0,
        py::arg("world") = 1, py::arg("rank") = 0, py::arg("ex_data") = std::vector<int64_t>(), py::arg("ex_flags") = std::vector<int64_t>(),
        py::arg("slot_elems") = 0, py::arg("seq") = 0, py::arg("round") = 14);
  m.def("decoder_bias_adam", &decoder_bias_adam, py::arg("bias"), py::arg("m"), py::arg("v"), py::arg("sel"), py::arg("gs_sum"), py::arg("extra"),
        py::arg("hyper"), py::arg("ctl") = none, py::arg("norm_weight") = 0.0);
  m.def("step_finish", &step_finish, py::arg("counter") = none, py::arg("fired") = none, py::arg("bias") = none, py::arg("sel") = none,
        py::arg("bias_sum") = none);
  m.def("theta_adam", &theta_adam, py::arg("log_theta"), py::arg("m"), py::arg("v"), py::arg("theta"), py::arg("S1"), py::arg("S2"),
        py::arg("norm2"), py::arg("feat_off"), py::arg("fcsr_val"), py::arg("tying"), py::arg("c_g"), py::arg("lambda_"), py::arg("c"),
        py::arg("bandwidth"), py::arg("hyper"), py::arg("ctl") = none, py::arg("norm_weight") = 0.0, py::arg("grad_out") = none);
  m.def("theta_exp", &theta_exp);
  m.def("dense_gemm", &dense_gemm);
  m.def("transpose16", &transpose16, py::arg("inp"), py::arg("out"), py::arg("mask") = none);
  m.def("negative_indicator", &negative_indicator);
  m.def("scale_histogram", &scale_histogram);
  m.def("aux_compact", &aux_compact);
  m.def("aux_gather_select", &aux_gather_select, py::arg("pre"), py::arg("enc_bias"), py::arg("dead_cols"), py::arg("nd"), py::arg("nd_all"),
        py::arg("k_aux_max"), py::arg("A"), py::arg("bias_scratch") = none);
  m.def("aux_gather_rows", &aux_gather_rows);
  m.def("aux_residual", &aux_residual, py::arg("recon"), py::arg("bias"), py::arg("bias_row"), py::arg("sigma"), py::arg("gs"), py::arg("g_out"),
        py::arg("loss"), py::arg("nd"), py::arg("ctl"), py::arg("factor"), py::arg("scale_g") = false);
  m.def("unscale", &unscale);
  m.def("rowsum16", &rowsum16);
  m.def("scatter_add_rows", &scatter_add_rows);
  m.def("normalize_cast", &normalize_cast, py::arg("inp"), py::arg("out"), py::arg("mean") = none, py::arg("inv_std") = none,
        py::arg("rows_per_stat") = 0, py::arg("mul") = 1.0);
}
