// Python bindings of the sm_100a kernels.  The kernels live in .cu files that know nothing about
// PyTorch (raw pointers + a stream); this file checks tensors and forwards to their C launchers.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstring>
#include <vector>

using torch::Tensor;
using OptTensor = c10::optional<Tensor>;

extern "C" {
int clt_encoder_gemm(const void* A, const void* B, const void* bias, void* C, int L, int M, int N, int K, long long ldc,
                     long long layer_stride_c, int* status, float* tile_stats, int num_sms, cudaStream_t stream);
int clt_colstats_from_tiles(const float* tile_stats, float* mean, float* rstd, int L, int B, int F, cudaStream_t st);
int clt_colstats(const void* x, float* mean, float* rstd, int L, int B, int F, long long ld, long long layer_stride, cudaStream_t st);

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
int clt_batchtopk_select(const CltSelectArgs* a, const CltExchangeArgs* exa, cudaStream_t st);
int clt_threshold_select(const CltSelectArgs* a, cudaStream_t st);
int clt_token_topk_select(const CltSelectArgs* a, cudaStream_t st);

struct CltThetaGradArgs {
  const void* gs; const void* w[32]; const void* preact;
  long long ldx, layer_stride_x;
  const float* theta; int stat_pitch; float bandwidth;
  float* S1; float* S2;
  int L, B, F, d;
  int* status;
};
int clt_theta_grad_gemm(const CltThetaGradArgs* a, int num_sms, cudaStream_t st);

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
int clt_build_csr(const CltCsrArgs* a, cudaStream_t st);
int clt_dead_counter_update(long long* counter, unsigned char* fired, int n, cudaStream_t st);

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
};
struct CltPeerTable {
  int world;
  int rank;
  void* ptr[8];
};
int clt_peer_barrier(const CltPeerTable* flags, int slot, unsigned int seq, int* status, long long timeout_cycles, cudaStream_t st);
int clt_owner_reduce_loss(const float* stage, const CltPeerTable* gs_peers, const float* bias_sum, const float* addend, const void* target,
                          const float* sigma, float* yhat_out, double* sq_err, int L, int B, int d, int rows_per_rank, cudaStream_t st);
int clt_sparse_decode(const CltDecodeArgs* a, cudaStream_t st);
int clt_recon_epilogue(const float* yhat_sum, const float* bias_sum, const float* addend, const void* target, const float* sigma,
                       void* gs, float* yhat_out, double* sq_err, int L, int B, int d, int row0, int nrows, cudaStream_t st);
int clt_gs_colsum(const void* gs, float* out, int L, int B, int d, cudaStream_t st);

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
};
int clt_decoder_rows_adam(const CltDecAdamArgs* a, int num_sms, cudaStream_t st);
struct CltEncAdamArgs {
  void* w; float* m; float* v; void* bias; float* bias_m; float* bias_v;
  int L, B, d, F_pitch, weights_bf16;
  const int* feat_off; const int* fcsr_tok; const float* delta; const void* x;
  const float* dense_grad; const float* dense_bias_grad;
  CltAdamHyper h;
  int* status;
  int moments_bf16;
};
int clt_encoder_rows_adam(const CltEncAdamArgs* a, int num_sms, cudaStream_t st);
int clt_dense_adam(void* w, float* m, float* v, const float* grad, long long n, int weights_bf16, const CltAdamHyper* h, cudaStream_t st);
int clt_decoder_norm2(const void* w, float* out, int F, int R, int d, int weights_bf16, cudaStream_t st);
int clt_sparsity_penalty(const int* feat_off, const float* fcsr_val, const float* norm2, int ncols, float lambda, float c,
                         float* grad_a, float* pen_coef, double* penalty_out, cudaStream_t st);
}

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
template <typename T>
T* opt_ptr(const OptTensor& t) {
  return t.has_value() && t->defined() ? static_cast<T*>(t->data_ptr()) : nullptr;
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
  need(x, at::kBFloat16, "x"); need(w, at::kBFloat16, "w"); need(out, at::kBFloat16, "out"); need(status, at::kInt, "status");
  TORCH_CHECK(x.dim() == 3 && w.dim() == 3 && out.dim() == 3, "expected [L, M, K], [L, N, K], [L, M, N]");
  const int L = x.size(0), M = x.size(1), K = x.size(2), N = w.size(1);
  TORCH_CHECK(w.size(0) == L && w.size(2) == K && out.size(0) == L && out.size(1) == M && out.size(2) == N, "shape mismatch");
  if (bias.has_value() && bias->defined()) { need(*bias, at::kBFloat16, "bias"); TORCH_CHECK(bias->numel() == 1LL * L * N, "bias must be [L, N]"); }
  float* ts = nullptr;
  if (tile_stats.has_value() && tile_stats->defined()) {
    need(*tile_stats, at::kFloat, "tile_stats");
    TORCH_CHECK(tile_stats->numel() == 2LL * L * ((M + 127) / 128) * N, "tile_stats must be [L, ceil(M / 128), N, 2]");
    ts = tile_stats->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(x.device());
  check(clt_encoder_gemm(x.data_ptr(), w.data_ptr(), opt_ptr<void>(bias), out.data_ptr(), L, M, N, K, N, 1LL * M * N,
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
  need(x, at::kBFloat16, "x"); need(mean, at::kFloat, "mean"); need(rstd, at::kFloat, "rstd");
  const int L = x.size(0), B = x.size(1), F = x.size(2);
  TORCH_CHECK(mean.numel() == 1LL * L * F && rstd.numel() == 1LL * L * F, "mean/rstd must be [L, F]");
  c10::cuda::CUDAGuard guard(x.device());
  check(clt_colstats(x.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), L, B, F, F, 1LL * B * F, cur_stream()), "colstats");
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
  need(x, at::kBFloat16, "x"); need(mean, at::kFloat, "mean"); need(rstd, at::kFloat, "rstd");
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
  check(clt_batchtopk_select(&a, multi ? &ex : nullptr, cur_stream()), "batchtopk_select");
}

// Entries with x >= theta[l, f] (JumpReLU; ReLU with theta = smallest positive bf16) as a (token, column, value) list.
void threshold_select(const Tensor& x, const Tensor& theta, int64_t f_valid, int64_t col_pitch, Tensor& ctl, Tensor& ent_tok,
                      Tensor& ent_col, Tensor& ent_val, Tensor& status) {
  need(x, at::kBFloat16, "x"); need(theta, at::kFloat, "theta"); need(ctl, at::kLong, "ctl"); need(status, at::kInt, "status");
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
  check(clt_threshold_select(&a, cur_stream()), "threshold_select");
}

// Per-token top-k of the batch z-scores: exactly k entries per token at [token * k, token * k + k) of the entry list.
void token_topk_select(const Tensor& x, const Tensor& mean, const Tensor& rstd, int64_t col_pitch, int64_t k, Tensor& ctl, Tensor& ent_tok,
                       Tensor& ent_col, Tensor& ent_val, Tensor& status) {
  need(x, at::kBFloat16, "x"); need(mean, at::kFloat, "mean"); need(rstd, at::kFloat, "rstd"); need(ctl, at::kLong, "ctl");
  need(status, at::kInt, "status"); need(ent_tok, at::kInt, "ent_tok"); need(ent_col, at::kInt, "ent_col"); need(ent_val, at::kFloat, "ent_val");
  TORCH_CHECK(x.dim() == 3 && mean.dim() == 2 && mean.size(0) == x.size(0) && mean.size(1) == x.size(2), "mean / rstd must be [L, F]");
  TORCH_CHECK(ctl.numel() >= 16 && ent_tok.numel() >= x.size(1) * k, "entry list needs B * k elements");
  CltSelectArgs a;
  std::memset(&a, 0, sizeof(a));
  a.x = x.data_ptr(); a.mean = mean.data_ptr<float>(); a.rstd = rstd.data_ptr<float>();
  a.L = x.size(0); a.B = x.size(1); a.F = x.size(2); a.stat_pitch = int(mean.size(1));
  a.ld = x.size(2); a.layer_stride = 1LL * x.size(1) * x.size(2);
  a.col_pitch = int(col_pitch); a.k_total = k;
  a.ctl = reinterpret_cast<long long*>(ctl.data_ptr<int64_t>());
  a.ent_tok = ent_tok.data_ptr<int>(); a.ent_col = ent_col.data_ptr<int>(); a.ent_val = ent_val.data_ptr<float>(); a.ent_cap = ent_tok.numel();
  a.status = status.data_ptr<int>();
  c10::cuda::CUDAGuard guard(x.device());
  check(clt_token_topk_select(&a, cur_stream()), "token_topk_select");
}

// JumpReLU threshold gradient sums: S1[l, f] += sum_b window * x * (gs . W_dec rows), S2[l, f] += sum_b window * x.
void theta_grad_gemm(const Tensor& gs, const std::vector<Tensor>& dec_w, const Tensor& preact, const Tensor& theta, double bandwidth,
                     Tensor& S1, Tensor& S2, Tensor& status) {
  need(gs, at::kBFloat16, "gs"); need(preact, at::kBFloat16, "preact"); need(theta, at::kFloat, "theta");
  need(S1, at::kFloat, "S1"); need(S2, at::kFloat, "S2"); need(status, at::kInt, "status");
  const int L = gs.size(0), B = gs.size(1), d = gs.size(2), F = preact.size(2);
  TORCH_CHECK(int(dec_w.size()) == L && L <= 32, "one untied decoder tensor per layer (at most 32)");
  TORCH_CHECK(preact.size(0) == L && preact.size(1) == B && theta.size(0) == L && theta.size(1) >= F, "shape mismatch");
  TORCH_CHECK(S1.sizes() == theta.sizes() && S2.sizes() == theta.sizes(), "S1 / S2 must have theta's shape");
  CltThetaGradArgs a;
  std::memset(&a, 0, sizeof(a));
  a.gs = gs.data_ptr(); a.preact = preact.data_ptr(); a.ldx = preact.size(2); a.layer_stride_x = 1LL * B * preact.size(2);
  for (int s = 0; s < L; ++s) {
    need(dec_w[s], at::kBFloat16, "decoder weight");
    TORCH_CHECK(dec_w[s].dim() == 3 && dec_w[s].size(0) == F && dec_w[s].size(1) == L - s && dec_w[s].size(2) == d, "decoder tensor must be [F, L - s, d]");
    a.w[s] = dec_w[s].data_ptr();
  }
  a.theta = theta.data_ptr<float>(); a.stat_pitch = int(theta.size(1)); a.bandwidth = float(bandwidth);
  a.S1 = S1.data_ptr<float>(); a.S2 = S2.data_ptr<float>();
  a.L = L; a.B = B; a.F = F; a.d = d; a.status = status.data_ptr<int>();
  c10::cuda::CUDAGuard guard(gs.device());
  check(clt_theta_grad_gemm(&a, num_sms(), cur_stream()), "theta_grad_gemm");
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

void sparse_decode(const std::vector<Tensor>& dec_w, int64_t L, int64_t B, int64_t d, int64_t col_pitch, int64_t tying, const Tensor& tok_off,
                   const Tensor& tcsr_col, const Tensor& tcsr_val, const OptTensor& feat_offset, const OptTensor& feat_scale,
                   const OptTensor& yhat_partial, const OptTensor& bias_sum, const OptTensor& addend, const OptTensor& target,
                   const OptTensor& sigma, const OptTensor& gs, const OptTensor& yhat_out, const OptTensor& sq_err, int64_t mode,
                   const std::vector<int64_t>& stage_peers, int64_t rows_per_rank, int64_t rank, const OptTensor& status) {
  TORCH_CHECK(dec_w.size() <= 32, "at most 32 decoder tensors");
  CltDecodeArgs a;
  std::memset(&a, 0, sizeof(a));
  for (size_t i = 0; i < dec_w.size(); ++i) {
    need(dec_w[i], at::kBFloat16, "dec_w");
    a.w[i] = dec_w[i].data_ptr();
    a.rows[i] = int(dec_w[i].size(1));
  }
  a.L = int(L); a.B = int(B); a.d = int(d); a.col_pitch = int(col_pitch); a.tying = int(tying);
  a.tok_off = tok_off.data_ptr<int>(); a.tcsr_col = tcsr_col.data_ptr<int>(); a.tcsr_val = tcsr_val.data_ptr<float>();
  a.feat_offset = opt_ptr<const float>(feat_offset); a.feat_scale = opt_ptr<const float>(feat_scale);
  a.yhat_partial = opt_ptr<float>(yhat_partial); a.bias_sum = opt_ptr<const float>(bias_sum); a.addend = opt_ptr<const float>(addend);
  a.target = opt_ptr<const void>(target); a.sigma = opt_ptr<const float>(sigma); a.gs = opt_ptr<void>(gs);
  a.yhat_out = opt_ptr<float>(yhat_out); a.sq_err = opt_ptr<double>(sq_err); a.mode = int(mode);
  if (status.has_value()) TORCH_CHECK(status->scalar_type() == at::kInt && status->numel() >= 4, "status: int32 tensor of at least 4 words (word 0 holds the code)");
  a.status = opt_ptr<int>(status);
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
  check(clt_sparse_decode(&a, cur_stream()), "sparse_decode");
}

void recon_epilogue(const Tensor& yhat_sum, const Tensor& bias_sum, const OptTensor& addend, const Tensor& target, const OptTensor& sigma,
                    Tensor& gs, const OptTensor& yhat_out, Tensor& sq_err, int64_t row0, int64_t nrows) {
  need(yhat_sum, at::kFloat, "yhat_sum"); need(bias_sum, at::kFloat, "bias_sum"); need(target, at::kBFloat16, "target");
  need(gs, at::kBFloat16, "gs"); need(sq_err, at::kDouble, "sq_err");
  const int L = yhat_sum.size(0), B = yhat_sum.size(1), d = yhat_sum.size(2);
  c10::cuda::CUDAGuard guard(yhat_sum.device());
  check(clt_recon_epilogue(yhat_sum.data_ptr<float>(), bias_sum.data_ptr<float>(), opt_ptr<const float>(addend), target.data_ptr(),
                           opt_ptr<const float>(sigma), gs.data_ptr(), opt_ptr<float>(yhat_out), sq_err.data_ptr<double>(), L, B, d,
                           int(row0), int(nrows), cur_stream()), "recon_epilogue");
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
                       const Tensor& target, const OptTensor& sigma, const OptTensor& yhat_out, Tensor& sq_err, int64_t rows_per_rank) {
  need(stage, at::kFloat, "stage"); need(bias_sum, at::kFloat, "bias_sum"); need(target, at::kBFloat16, "target"); need(sq_err, at::kDouble, "sq_err");
  const int L = target.size(0), B = target.size(1), d = target.size(2);
  const CltPeerTable t = make_table(gs_ptrs, rank);
  TORCH_CHECK(stage.numel() >= 1LL * t.world * L * rows_per_rank * d, "staging area too small");
  c10::cuda::CUDAGuard guard(stage.device());
  check(clt_owner_reduce_loss(stage.data_ptr<float>(), &t, bias_sum.data_ptr<float>(), opt_ptr<const float>(addend), target.data_ptr(),
                              opt_ptr<const float>(sigma), opt_ptr<float>(yhat_out), sq_err.data_ptr<double>(), L, B, d, int(rows_per_rank),
                              cur_stream()), "owner_reduce_loss");
}

void gs_colsum(const Tensor& gs, Tensor& out) {
  need(gs, at::kBFloat16, "gs"); need(out, at::kFloat, "out");
  c10::cuda::CUDAGuard guard(gs.device());
  check(clt_gs_colsum(gs.data_ptr(), out.data_ptr<float>(), int(gs.size(0)), int(gs.size(1)), int(gs.size(2)), cur_stream()), "gs_colsum");
}

void decoder_rows_adam(std::vector<Tensor>& w, std::vector<Tensor>& m, std::vector<Tensor>& v, int64_t L, int64_t B, int64_t d,
                       int64_t F_pitch, int64_t tying, const Tensor& feat_off, const Tensor& fcsr_tok, const Tensor& fcsr_val,
                       const Tensor& gs, const OptTensor& grad_a, const OptTensor& pen_coef, const OptTensor& norm2_out,
                       const OptTensor& feat_offset, const OptTensor& feat_scale, const OptTensor& dgrad_row0,
                       const std::vector<double>& hyper, const OptTensor& status) {
  TORCH_CHECK(w.size() <= 32 && w.size() == m.size() && w.size() == v.size(), "bad tensor lists");
  CltDecAdamArgs a;
  std::memset(&a, 0, sizeof(a));
  const bool bf16 = w[0].scalar_type() == at::kBFloat16;
  for (size_t i = 0; i < w.size(); ++i) {
    need(w[i], bf16 ? at::kBFloat16 : at::kFloat, "w");
    need(m[i], m[0].scalar_type(), "m"); need(v[i], m[0].scalar_type(), "v");
    TORCH_CHECK(m[0].scalar_type() == at::kFloat || m[0].scalar_type() == at::kBFloat16, "moments must be fp32 or bf16");
    TORCH_CHECK(w[i].dim() == 3 && w[i].size(0) == F_pitch && w[i].size(2) == d, "decoder tensor must be [F, R, d]");
    a.w[i] = w[i].data_ptr(); a.m[i] = static_cast<float*>(m[i].data_ptr()); a.v[i] = static_cast<float*>(v[i].data_ptr()); a.rows[i] = int(w[i].size(1));
  }
  a.ntensors = int(w.size()); a.L = int(L); a.B = int(B); a.d = int(d); a.F_pitch = int(F_pitch); a.tying = int(tying); a.weights_bf16 = bf16;
  a.feat_off = feat_off.data_ptr<int>(); a.fcsr_tok = fcsr_tok.data_ptr<int>(); a.fcsr_val = fcsr_val.data_ptr<float>();
  need(gs, at::kBFloat16, "gs");
  a.gs = gs.data_ptr(); a.grad_a = opt_ptr<float>(grad_a); a.pen_coef = opt_ptr<const float>(pen_coef); a.norm2_out = opt_ptr<float>(norm2_out);
  a.feat_offset = opt_ptr<const float>(feat_offset); a.feat_scale = opt_ptr<const float>(feat_scale);
  a.dgrad_row0 = opt_ptr<const float>(dgrad_row0);
  if (a.dgrad_row0) TORCH_CHECK(dgrad_row0->scalar_type() == at::kFloat && dgrad_row0->numel() == int64_t(w.size()) * F_pitch * d, "dgrad_row0 must be fp32 [ntensors, F, d]");
  a.h = hyper_from(hyper);
  a.status = opt_ptr<int>(status);
  a.moments_bf16 = m[0].scalar_type() == at::kBFloat16 ? 1 : 0;
  c10::cuda::CUDAGuard guard(gs.device());
  check(clt_decoder_rows_adam(&a, num_sms(), cur_stream()), "decoder_rows_adam");
}

void encoder_rows_adam(Tensor& w, Tensor& m, Tensor& v, Tensor& bias, Tensor& bias_m, Tensor& bias_v, const Tensor& feat_off,
                       const Tensor& fcsr_tok, const Tensor& delta, const Tensor& x, const OptTensor& dense_grad,
                       const OptTensor& dense_bias_grad, const std::vector<double>& hyper, const OptTensor& status) {
  const bool bf16 = w.scalar_type() == at::kBFloat16;
  const bool mbf16 = m.scalar_type() == at::kBFloat16;
  need(w, bf16 ? at::kBFloat16 : at::kFloat, "w"); need(m, mbf16 ? at::kBFloat16 : at::kFloat, "m"); need(v, mbf16 ? at::kBFloat16 : at::kFloat, "v");
  need(bias, bf16 ? at::kBFloat16 : at::kFloat, "bias"); need(bias_m, at::kFloat, "bias_m"); need(bias_v, at::kFloat, "bias_v");
  need(x, at::kBFloat16, "x"); need(delta, at::kFloat, "delta");
  CltEncAdamArgs a;
  std::memset(&a, 0, sizeof(a));
  a.w = w.data_ptr(); a.m = static_cast<float*>(m.data_ptr()); a.v = static_cast<float*>(v.data_ptr());
  a.moments_bf16 = mbf16 ? 1 : 0;
  a.bias = bias.data_ptr(); a.bias_m = bias_m.data_ptr<float>(); a.bias_v = bias_v.data_ptr<float>();
  a.L = int(w.size(0)); a.F_pitch = int(w.size(1)); a.d = int(w.size(2)); a.B = int(x.size(1)); a.weights_bf16 = bf16;
  a.feat_off = feat_off.data_ptr<int>(); a.fcsr_tok = fcsr_tok.data_ptr<int>(); a.delta = delta.data_ptr<float>(); a.x = x.data_ptr();
  a.dense_grad = opt_ptr<const float>(dense_grad); a.dense_bias_grad = opt_ptr<const float>(dense_bias_grad);
  a.h = hyper_from(hyper);
  a.status = opt_ptr<int>(status);
  c10::cuda::CUDAGuard guard(w.device());
  check(clt_encoder_rows_adam(&a, num_sms(), cur_stream()), "encoder_rows_adam");
}

void dense_adam(Tensor& w, Tensor& m, Tensor& v, const Tensor& grad, const std::vector<double>& hyper) {
  const bool bf16 = w.scalar_type() == at::kBFloat16;
  need(w, bf16 ? at::kBFloat16 : at::kFloat, "w"); need(m, at::kFloat, "m"); need(v, at::kFloat, "v"); need(grad, at::kFloat, "grad");
  TORCH_CHECK(w.numel() == m.numel() && w.numel() == v.numel() && w.numel() == grad.numel(), "size mismatch");
  const CltAdamHyper h = hyper_from(hyper);
  c10::cuda::CUDAGuard guard(w.device());
  check(clt_dense_adam(w.data_ptr(), m.data_ptr<float>(), v.data_ptr<float>(), grad.data_ptr<float>(), w.numel(), bf16, &h, cur_stream()), "dense_adam");
}

void decoder_norm2(const Tensor& w, Tensor& out) {
  const bool bf16 = w.scalar_type() == at::kBFloat16;
  need(w, bf16 ? at::kBFloat16 : at::kFloat, "w"); need(out, at::kFloat, "out");
  TORCH_CHECK(w.dim() == 3 && out.numel() >= w.size(0), "w must be [F, R, d], out [F]");
  c10::cuda::CUDAGuard guard(w.device());
  check(clt_decoder_norm2(w.data_ptr(), out.data_ptr<float>(), int(w.size(0)), int(w.size(1)), int(w.size(2)), bf16, cur_stream()), "decoder_norm2");
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

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("encoder_gemm", &encoder_gemm);
  m.def("colstats", &colstats);
  m.def("colstats_from_tiles", &colstats_from_tiles);
  m.def("batchtopk_select", &batchtopk_select);
  m.def("threshold_select", &threshold_select);
  m.def("token_topk_select", &token_topk_select);
  m.def("theta_grad_gemm", &theta_grad_gemm);
  m.def("build_csr", &build_csr);
  m.def("dead_counter_update", &dead_counter_update);
  m.def("sparse_decode", &sparse_decode);
  m.def("recon_epilogue", &recon_epilogue);
  m.def("gs_colsum", &gs_colsum);
  m.def("peer_barrier", &peer_barrier, py::arg("flag_ptrs"), py::arg("rank"), py::arg("slot"), py::arg("seq"), py::arg("status"),
        py::arg("timeout_s") = 0.0);
  m.def("memcpy_2d", &memcpy_2d);
  m.def("owner_reduce_loss", &owner_reduce_loss);
  m.def("decoder_rows_adam", &decoder_rows_adam);
  m.def("encoder_rows_adam", &encoder_rows_adam);
  m.def("dense_adam", &dense_adam);
  m.def("decoder_norm2", &decoder_norm2);
  m.def("sparsity_penalty", &sparsity_penalty);
}
