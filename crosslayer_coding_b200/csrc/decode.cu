// Sparse cross-layer decode and the reconstruction loss (sm_100a).
//
// The reference decodes with one dense GEMM per (source, target) pair over activations that are more
// than 99 % zeros, each followed by an all-reduce (clt/models/decoder.py:289-295, clt/models/parallel.py:363-383),
// and then computes the MSE in separate passes (clt/training/losses.py:76-90).  Here one CTA per token walks
// that token's active (layer, feature, value) entries, reads each feature's contiguous block of decoder rows
// (feature-major layout [F, R, d]) and accumulates every target layer's reconstruction in registers
// (the targets are split over four warp groups to keep the register footprint small).
// The epilogue either writes the fp32 partial reconstruction (tensor parallel: summed across ranks before
// the loss) or, single rank, finishes in place: bias, optional dense addend (skip connection), residual,
// per-layer squared-error sum in de-normalised units and the bf16 gradient seed  gs = (y_hat - y) * sigma^2.
#include "common.cuh"

namespace clt {

constexpr int kMaxLayers = 32;

struct DecodeParams {
  const t16* w[kMaxLayers];  // decoder tensor i: [F_pitch, rows_i, d]
  int rows[kMaxLayers];                // rows per feature of tensor i
  int L, B, d;
  int col_pitch;                       // entries encode column = layer * col_pitch + feature
  int tying;                           // 0 untied, 1 per_source, 2 per_target
  const int* tok_off;                  // [B+1]
  const int* tcsr_col;                 // (layer << 24) | feature
  const float* tcsr_val;
  const float* feat_offset;            // optional [L, col_pitch]  (tied decoders)
  const float* feat_scale;             // optional [L, col_pitch]
  // outputs / epilogue
  float* yhat_partial;                 // mode 0: [L, B, d] fp32 partial sums
  const float* bias_sum;               // mode 1: [L, d] summed decoder biases per target
  const float* addend;                 // mode 1: optional [L, B, d] fp32 (skip term)
  const t16* target;         // mode 1: [L, B, d]
  const float* sigma;                  // mode 1: optional [L, d] de-normalisation scale of the targets
  t16* gs;                   // mode 1: [L, B, d] (y_hat - y) * sigma^2
  float* yhat_out;                     // mode 1: optional [L, B, d] fp32 reconstruction
  double* sq_err;                      // mode 1: [L] sum of ((y_hat - y) * sigma)^2
  // mode 2 (tensor parallel): partial sums are pushed into the staging area of the rank that owns the token.
  // stage_peers[o] = rank o's staging area [world][L][rows_per_rank][d] fp32; this rank writes slot `rank`.
  float* stage_peers[8];
  int rows_per_rank, rank, world;
  int mode;
  // optional step control block: the gradient seed is multiplied by ctl[SC_LOSS_SCALE] (fp16 loss scaling) and a
  // seed that leaves the 16-bit range or is NaN raises ctl[SC_FOUND_INF] (the step is then skipped)
  float* ctl;
  int rows_limit;  // > 0: only the first rows_limit target rows of a feature are decoded (auxiliary loss: same layer only)
  int* dbg_status; // status words for the index checks of the debug build (may be null)
};

__device__ __forceinline__ void fma8(float (&acc)[8], float a, const uint4& v) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    acc[2 * j] = fmaf(a, t16_lo(u[j]), acc[2 * j]);
    acc[2 * j + 1] = fmaf(a, t16_hi(u[j]), acc[2 * j + 1]);
  }
}

// Output of one (token, target, 8-element slice): partial sums (mode 0), peer push (mode 2) or the finished
// loss epilogue (mode 1).  Returns the slice's squared error (mode 1, else 0); the callers sum it in registers and
// across the warp: a shared-memory atomic per thread on the L per-target sums costs tens of thousands of cycles
// per token (32 lanes on one address, floating-point add as a compare-and-swap loop).
__device__ __forceinline__ float decode_epilogue(const DecodeParams& p, int tok, int t, int e0, const float (&a)[8], float loss_scale) {
  const long long off = (1LL * t * p.B + tok) * p.d + e0;
  if (p.mode == 0) {
    float4* dst = reinterpret_cast<float4*>(p.yhat_partial + off);
    dst[0] = make_float4(a[0], a[1], a[2], a[3]);
    dst[1] = make_float4(a[4], a[5], a[6], a[7]);
    return 0.f;
  } else if (p.mode == 2) {
    // reduce-scatter by push: peer store into the owner's slot for this rank (NVLink posted writes)
    const int owner = tok / p.rows_per_rank;
    const int lrow = tok - owner * p.rows_per_rank;
    if (!clt_in_bounds(owner, p.world, p.dbg_status, 105)) return 0.f;  // peer rank derived from the token index
    float4* dst = reinterpret_cast<float4*>(p.stage_peers[owner] + ((1LL * p.rank * p.L + t) * p.rows_per_rank + lrow) * p.d + e0);
    dst[0] = make_float4(a[0], a[1], a[2], a[3]);
    dst[1] = make_float4(a[4], a[5], a[6], a[7]);
    return 0.f;
  } else {
    float y[8], out[8];
    const uint4 tv = *reinterpret_cast<const uint4*>(p.target + off);
    const uint32_t u[4] = {tv.x, tv.y, tv.z, tv.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { y[2 * i] = t16_lo(u[i]); y[2 * i + 1] = t16_hi(u[i]); }
    float sq = 0.f;
    bool bad = false;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float v = a[i] + p.bias_sum[1LL * t * p.d + e0 + i];
      if (p.addend) v += p.addend[off + i];
      const float sg = p.sigma ? p.sigma[1LL * t * p.d + e0 + i] : 1.f;
      out[i] = v;
      const float r = (v - y[i]) * sg;
      sq = fmaf(r, r, sq);
      y[i] = r * sg * loss_scale;  // gradient seed
      bad |= !(fabsf(y[i]) <= kT16Max);
    }
    if (bad && p.ctl != nullptr) atomicOr(reinterpret_cast<int*>(p.ctl) + SC_FOUND_INF, 1);
    uint4 gv;
    gv.x = pack_t16x2(y[0], y[1]); gv.y = pack_t16x2(y[2], y[3]);
    gv.z = pack_t16x2(y[4], y[5]); gv.w = pack_t16x2(y[6], y[7]);
    *reinterpret_cast<uint4*>(p.gs + off) = gv;
    if (p.yhat_out) {
      float4* dst = reinterpret_cast<float4*>(p.yhat_out + off);
      dst[0] = make_float4(out[0], out[1], out[2], out[3]);
      dst[1] = make_float4(out[4], out[5], out[6], out[7]);
    }
    return sq;
  }
}

constexpr int kGroups = 4;  // warp groups per token; group g owns targets t with t % kGroups == g

// One CTA per token.  The CTA is split into kGroups warp groups of `gthreads` threads; every group walks
// all entries of the token but only accumulates its own targets (t = g, g + kGroups, ...), so a thread
// holds TPG x 8 accumulators instead of L x 8 and many more warps fit on an SM (more than 16 layers:
// blockIdx.y selects the next 16 targets).  Each thread covers 8
// consecutive elements of d (one 16-byte load per decoder row).
template <int TPG>
__global__ void __launch_bounds__(1024) decode_kernel(const DecodeParams p, int gthreads) {
  // Tensor-parallel push: rank r starts with the tokens owned by rank r + 1, so that at any moment the ranks
  // store into different owners instead of all into the same one.
  const int tok = p.mode == 2 ? int((blockIdx.x + 1LL * ((p.rank + 1) % p.world) * p.rows_per_rank) % p.B) : int(blockIdx.x);
  const int g = threadIdx.x / gthreads;
  const int gt = threadIdx.x - g * gthreads;
  const int e0 = gt * 8;
  const bool active = e0 < p.d;
  float acc[TPG][8];
#pragma unroll
  for (int j = 0; j < TPG; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
  __shared__ float sq_s[kMaxLayers];
  __shared__ const t16* w_s[kMaxLayers];  // parameter tables in shared memory: indexed per entry
  __shared__ int rows_s[kMaxLayers];
  if (threadIdx.x < kMaxLayers) {
    sq_s[threadIdx.x] = 0.f;
    w_s[threadIdx.x] = p.w[threadIdx.x];
    rows_s[threadIdx.x] = p.rows[threadIdx.x];
  }
  __syncthreads();
  const int L = p.L, d = p.d, tying = p.tying;
  const float loss_scale = p.ctl != nullptr ? p.ctl[SC_LOSS_SCALE] : 1.f;
  const int t_span = p.rows_limit > 0 ? p.rows_limit : kMaxLayers;  // targets s .. s + t_span - 1 of a source layer s

  const int b = p.tok_off[tok], e = p.tok_off[tok + 1];
  if (active) {
    for (int i = b; i < e; ++i) {
      const int col = __ldg(p.tcsr_col + i);  // packed by the CSR build: (layer << 24) | feature
      const float a = __ldg(p.tcsr_val + i);
      const int s = col >> 24;
      const int f = col & 0xFFFFFF;
      if (a == 0.f) continue;
      if (!clt_in_bounds(s, L, p.dbg_status, 101) || !clt_in_bounds(f, p.col_pitch, p.dbg_status, 102)) continue;
      if (tying == 0) {
        // row (t - s) of feature f; rows of one feature are contiguous
        const t16* base = w_s[s] + (1LL * f * rows_s[s] - s) * d + e0;
#pragma unroll
        for (int j = 0; j < TPG; ++j) {
          const int t = g + (blockIdx.y * TPG + j) * kGroups;
          if (t < L && t >= s && t - s < t_span) fma8(acc[j], a, __ldg(reinterpret_cast<const uint4*>(base + 1LL * t * d)));
        }
      } else if (tying == 1) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(w_s[s] + 1LL * f * d + e0));
#pragma unroll
        for (int j = 0; j < TPG; ++j) {
          const int t = g + (blockIdx.y * TPG + j) * kGroups;
          if (t < p.L && t >= s && t - s < t_span) {
            float av = a;
            if (p.feat_offset) av += p.feat_offset[1LL * t * p.col_pitch + f];
            if (p.feat_scale) av *= p.feat_scale[1LL * t * p.col_pitch + f];
            fma8(acc[j], av, v);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < TPG; ++j) {
          const int t = g + (blockIdx.y * TPG + j) * kGroups;
          if (t < p.L && t >= s && t - s < t_span) {
            float av = a;
            if (p.feat_offset) av += p.feat_offset[1LL * t * p.col_pitch + f];
            if (p.feat_scale) av *= p.feat_scale[1LL * t * p.col_pitch + f];
            fma8(acc[j], av, __ldg(reinterpret_cast<const uint4*>(w_s[t] + 1LL * f * d + e0)));
          }
        }
      }
    }
  }

#pragma unroll
  for (int j = 0; j < TPG; ++j) {
    const int t = g + (blockIdx.y * TPG + j) * kGroups;  // the same for all lanes of a warp (gthreads is a multiple of 32)
    if (t >= p.L) continue;
    float sq = active ? decode_epilogue(p, tok, t, e0, acc[j], loss_scale) : 0.f;
    if (p.mode == 1) {
      sq = warp_sum(sq);
      if ((threadIdx.x & 31) == 0) atomicAdd(&sq_s[t], sq);
    }
  }
  if (p.mode == 1) {
    __syncthreads();
    if (threadIdx.x < p.L && sq_s[threadIdx.x] != 0.f) atomicAdd(&p.sq_err[threadIdx.x], double(sq_s[threadIdx.x]));
  }
}

// Untied decoders, the flagship path: the rows of one active feature for all its targets are one contiguous
// block of (L - s) * d bf16.  A producer warp streams these blocks into a shared-memory ring with 1-D bulk
// copies (cp.async.bulk + mbarrier, no multicast); the four consumer groups take their targets' rows from
// shared memory.  Large contiguous reads and a ring that is always full keep HBM busy, where the per-row
// register loads of decode_kernel wait on a dependent load chain.  Every mbarrier wait is bounded.
constexpr int kDecodeStages = 16;  // at most; the launcher picks the depth so that the ring holds a few tens of KB

struct DecodeBulkShared {
  uint64_t full[kDecodeStages];
  uint64_t empty[kDecodeStages];
  float sq_s[kMaxLayers];
  const t16* w_s[kMaxLayers];
  int rows_s[kMaxLayers];
  int abort_flag;
  int ent_sl[kDecodeStages];    // source layer and activation of the entry in each stage, written by the producer
  float ent_a[kDecodeStages];
};

// V: 8-element column chunks per thread (1 for d <= 1024, 2 up to d = 2048: chunk v of thread gt covers columns
// (v * gthreads + gt) * 8 ...), so that the CTA stays at four groups of at most 128 threads plus the producer warp.
template <int TPG, int V>
__global__ void __launch_bounds__(544) decode_bulk_kernel(const DecodeParams p, int gthreads, int stage_bytes, int nstages, int* status) {
  extern __shared__ __align__(128) uint8_t smem_raw_dec[];  // bulk copies need 16-byte alignment only
  uint8_t* ring = smem_raw_dec;
  DecodeBulkShared* sh = reinterpret_cast<DecodeBulkShared*>(ring + size_t(nstages) * stage_bytes);
  // per-source tied decoders: one row per feature that serves every target >= its source layer
  const bool shared_row = p.tying == 1;
  // Tensor-parallel push: rank r starts with the tokens owned by rank r + 1, so that at any moment the ranks
  // store into different owners instead of all into the same one.
  const int tok = p.mode == 2 ? int((blockIdx.x + 1LL * ((p.rank + 1) % p.world) * p.rows_per_rank) % p.B) : int(blockIdx.x);
  const int nconsumer = kGroups * gthreads;
  const bool is_producer = int(threadIdx.x) >= nconsumer;
  const int L = p.L, d = p.d;
  if (threadIdx.x < kMaxLayers) {
    sh->sq_s[threadIdx.x] = 0.f;
    sh->w_s[threadIdx.x] = p.w[threadIdx.x];
    sh->rows_s[threadIdx.x] = p.rows[threadIdx.x];
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < nstages; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], nconsumer / 32);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  volatile int* abort_flag = &sh->abort_flag;
  const int b = p.tok_off[tok], e = p.tok_off[tok + 1];
  const float loss_scale = p.ctl != nullptr ? p.ctl[SC_LOSS_SCALE] : 1.f;

  if (is_producer) {
    if (threadIdx.x == nconsumer) {
      int issued = 0;
      int col_next = b < e ? __ldg(p.tcsr_col + b) : 0;
      float a_next = b < e ? __ldg(p.tcsr_val + b) : 0.f;
      for (int i = b; i < e; ++i, ++issued) {
        const int st = issued % nstages;
        const uint32_t ph = (issued / nstages) & 1;
        const int col = col_next;
        float a = a_next;
        if (i + 1 < e) {  // the next entry's index is in flight while this stage is waited for
          col_next = __ldg(p.tcsr_col + i + 1);
          a_next = __ldg(p.tcsr_val + i + 1);
        }
        if (!mbar_wait(&sh->empty[st], ph ^ 1, abort_flag)) break;
        int sl = col >> 24, f = col & 0xFFFFFF;
        if (!clt_in_bounds(sl, L, p.dbg_status, 103) || !clt_in_bounds(f, p.col_pitch, p.dbg_status, 104)) { sl = 0; f = 0; a = 0.f; }  // decode a harmless row with weight zero
        const int R = sh->rows_s[sl];
        const int r_eff = (p.rows_limit > 0 && p.rows_limit < R) ? p.rows_limit : R;
        const uint32_t bytes = uint32_t(r_eff) * uint32_t(d) * 2u;
        sh->ent_sl[st] = sl;
        sh->ent_a[st] = a;
        mbar_expect_tx(&sh->full[st], bytes);  // release: the two words above are visible to whoever sees the phase
        bulk_load_1d(ring + size_t(st) * stage_bytes, sh->w_s[sl] + 1LL * f * R * d, bytes, &sh->full[st]);
      }
      if (*abort_flag) {
        // give copies already issued a bounded chance to land before the CTA retires
        const int first = issued > nstages ? issued - nstages : 0;
        for (int j = first; j < issued; ++j) {
          const long long start = clock64();
          while (!mbar_try_wait(&sh->full[j % nstages], (j / nstages) & 1))
            if (clock64() - start > kWaitTimeoutCycles) break;
        }
      }
    }
  } else {
    const int g = threadIdx.x / gthreads;
    const int gt = threadIdx.x - g * gthreads;
    const int lane = threadIdx.x & 31;
    int e0[V];
    bool active[V];
#pragma unroll
    for (int v = 0; v < V; ++v) { e0[v] = (v * gthreads + gt) * 8; active[v] = e0[v] < d; }
    float acc[TPG][V][8];
#pragma unroll
    for (int j = 0; j < TPG; ++j)
#pragma unroll
      for (int v = 0; v < V; ++v)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[j][v][i] = 0.f;
    int it = 0;
    bool ok = true;
    const int t_span = p.rows_limit > 0 ? p.rows_limit : kMaxLayers;
    for (int i = b; i < e; ++i, ++it) {
      const int st = it % nstages;
      const uint32_t ph = (it / nstages) & 1;
      if (!mbar_wait(&sh->full[st], ph, abort_flag)) { ok = false; break; }
      const int sl = sh->ent_sl[st];
      const float a = sh->ent_a[st];
      if (a != 0.f) {
        const t16* rows = reinterpret_cast<const t16*>(ring + size_t(st) * stage_bytes);
#pragma unroll
        for (int j = 0; j < TPG; ++j) {
          const int t = g + (blockIdx.y * TPG + j) * kGroups;
          if (t < L && t >= sl && t - sl < t_span) {
            const t16* row = rows + (shared_row ? 0 : (t - sl) * d);
#pragma unroll
            for (int v = 0; v < V; ++v)
              if (active[v]) fma8(acc[j][v], a, *reinterpret_cast<const uint4*>(row + e0[v]));
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->empty[st]);  // this warp is done with the stage
    }
    // one warp-level sum and one shared atomic per warp and target (the lanes of a warp share their targets)
#pragma unroll
    for (int j = 0; j < TPG; ++j) {
      const int t = g + (blockIdx.y * TPG + j) * kGroups;
      if (t >= L) continue;
      float sq = 0.f;
#pragma unroll
      for (int v = 0; v < V; ++v)
        if (ok && active[v]) sq += decode_epilogue(p, tok, t, e0[v], acc[j][v], loss_scale);
      if (p.mode == 1) {
        sq = warp_sum(sq);
        if (lane == 0) atomicAdd(&sh->sq_s[t], sq);
      }
    }
  }
  __syncthreads();
  if (p.mode == 1 && threadIdx.x < L && sh->sq_s[threadIdx.x] != 0.f) atomicAdd(&p.sq_err[threadIdx.x], double(sh->sq_s[threadIdx.x]));
  if (threadIdx.x == 0 && sh->abort_flag && status != nullptr) atomicCAS(status, STATUS_OK, STATUS_WAIT_TIMEOUT);
}

// Epilogue for the tensor-parallel path, run after the partial reconstructions were summed across ranks:
// bias, addend, residual, loss sum and gradient seed for rows [row0, row0 + nrows) of every layer.
__global__ void __launch_bounds__(256) recon_epilogue_kernel(const float* __restrict__ yhat_sum, const float* __restrict__ bias_sum,
                                                               const float* __restrict__ addend, const t16* __restrict__ target,
                                                               const float* __restrict__ sigma, t16* __restrict__ gs,
                                                               float* __restrict__ yhat_out, double* __restrict__ sq_err, int L, int B,
                                                               int d, int row0, int nrows, float* __restrict__ ctl) {
  const int t = blockIdx.y;
  const float loss_scale = ctl != nullptr ? ctl[SC_LOSS_SCALE] : 1.f;
  bool bad = false;
  const int vec_per_row = d / 8;
  const long long nvec = 1LL * nrows * vec_per_row;
  float sq = 0.f;
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < nvec; i += 1LL * gridDim.x * blockDim.x) {
    const int row = row0 + int(i / vec_per_row);
    const int e0 = int(i % vec_per_row) * 8;
    const long long off = (1LL * t * B + row) * d + e0;
    const float4 a0 = *reinterpret_cast<const float4*>(yhat_sum + off), a1 = *reinterpret_cast<const float4*>(yhat_sum + off + 4);
    float v[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    const uint4 tv = *reinterpret_cast<const uint4*>(target + off);
    const uint32_t u[4] = {tv.x, tv.y, tv.z, tv.w};
    float g[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] += bias_sum[1LL * t * d + e0 + j];
      if (addend) v[j] += addend[off + j];
      const float y = (j & 1) ? t16_hi(u[j >> 1]) : t16_lo(u[j >> 1]);
      const float sg = sigma ? sigma[1LL * t * d + e0 + j] : 1.f;
      const float r = (v[j] - y) * sg;
      sq = fmaf(r, r, sq);
      g[j] = r * sg * loss_scale;
      bad |= !(fabsf(g[j]) <= kT16Max);
    }
    uint4 gv;
    gv.x = pack_t16x2(g[0], g[1]); gv.y = pack_t16x2(g[2], g[3]); gv.z = pack_t16x2(g[4], g[5]); gv.w = pack_t16x2(g[6], g[7]);
    *reinterpret_cast<uint4*>(gs + off) = gv;
    if (yhat_out) {
      float4* dst = reinterpret_cast<float4*>(yhat_out + off);
      dst[0] = make_float4(v[0], v[1], v[2], v[3]);
      dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
  }
  __shared__ float red[8];
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) tot += red[w];
    atomicAdd(&sq_err[t], double(tot));
  }
  if (bad && ctl != nullptr) atomicOr(reinterpret_cast<int*>(ctl) + SC_FOUND_INF, 1);
}

// Column sums of the gradient seed: out[t, :] += sum_b gs[t, b, :]  (decoder-bias gradient up to a constant).
// blockDim = (d / 8 rounded up to 32, up to 8 row lanes): a thread owns 8 adjacent columns (one 16-byte load per row), the
// threadIdx.y lanes of a block walk the block's row range, shared memory folds them, one atomic per column and block.
__global__ void __launch_bounds__(1024) gs_colsum_kernel(const t16* __restrict__ gs, float* __restrict__ out, int B, int d,
                                                          int rows_per_block) {
  const int t = blockIdx.z;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(B, r0 + rows_per_block);
  float s[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = 0.f;
  if (c0 < d) {
    for (int r = r0 + threadIdx.y; r < r1; r += blockDim.y) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(gs + (1LL * t * B + r) * d + c0));
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { s[2 * j] += t16_lo(u[j]); s[2 * j + 1] += t16_hi(u[j]); }
    }
  }
  __shared__ float red[1024][9];
  const int lin = threadIdx.y * blockDim.x + threadIdx.x;
#pragma unroll
  for (int j = 0; j < 8; ++j) red[lin][j] = s[j];
  __syncthreads();
  if (threadIdx.y == 0 && c0 < d) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float tot = 0.f;
      for (int y = 0; y < int(blockDim.y); ++y) tot += red[y * blockDim.x + threadIdx.x][j];
      atomicAdd(&out[1LL * t * d + c0 + j], tot);
    }
  }
}

// Suffix sums of the gradient seed over the layers: out[s] = sum over t >= s of gs[t]  (per_source tied decoders:
// the threshold-gradient GEMM of source layer s needs the seed of all its targets added up).  fp32 accumulation.
__global__ void __launch_bounds__(256) gs_suffix_sum_kernel(const t16* __restrict__ gs, t16* __restrict__ out, int L, long long per_layer) {
  for (long long i = (blockIdx.x * 1LL * blockDim.x + threadIdx.x) * 8; i < per_layer; i += 1LL * gridDim.x * blockDim.x * 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int t = L - 1; t >= 0; --t) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(gs + t * per_layer + i));
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) { acc[2 * j] += t16_lo(u[j]); acc[2 * j + 1] += t16_hi(u[j]); }
      uint4 o;
      o.x = pack_t16x2(acc[0], acc[1]); o.y = pack_t16x2(acc[2], acc[3]); o.z = pack_t16x2(acc[4], acc[5]); o.w = pack_t16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out + t * per_layer + i) = o;
    }
  }
}

}  // namespace clt

using namespace clt;

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
  int* status;  // when given, untied decoders use the bulk-copy pipeline (its bounded waits report here)
  float* ctl;   // optional step control block (loss scale in, found-inf flag out)
  int rows_limit;
};

extern "C" int CLT_FN(clt_sparse_decode)(const CltDecodeArgs* a, cudaStream_t st) {
  if (a->d % 8 != 0 || a->L > kMaxLayers || a->d > 2048) return -1;
  DecodeParams p;
  for (int i = 0; i < kMaxLayers; ++i) { p.w[i] = static_cast<const t16*>(a->w[i]); p.rows[i] = a->rows[i]; }
  p.L = a->L; p.B = a->B; p.d = a->d; p.col_pitch = a->col_pitch; p.tying = a->tying;
  p.tok_off = a->tok_off; p.tcsr_col = a->tcsr_col; p.tcsr_val = a->tcsr_val;
  p.feat_offset = a->feat_offset; p.feat_scale = a->feat_scale;
  p.yhat_partial = a->yhat_partial; p.bias_sum = a->bias_sum; p.addend = a->addend;
  p.target = static_cast<const t16*>(a->target); p.sigma = a->sigma;
  p.gs = static_cast<t16*>(a->gs); p.yhat_out = a->yhat_out; p.sq_err = a->sq_err; p.mode = a->mode;
  for (int i = 0; i < 8; ++i) p.stage_peers[i] = static_cast<float*>(a->stage_peers[i]);
  p.rows_per_rank = a->rows_per_rank; p.rank = a->rank; p.world = a->world;
  p.ctl = a->ctl; p.rows_limit = a->rows_limit; p.dbg_status = a->status;
  int gthreads = ((a->d / 8 + 31) / 32) * 32;
  int threads = gthreads * kGroups;
  if (threads > 1024) return -1;
  const int tpg = (a->L + kGroups - 1) / kGroups;  // targets per warp group
  int max_rows = 0;
  for (int i = 0; i < a->L; ++i) max_rows = a->rows[i] > max_rows ? a->rows[i] : max_rows;
  if (a->rows_limit > 0 && a->rows_limit < max_rows) max_rows = a->rows_limit;
  const int stage_bytes = ((max_rows * a->d * 2 + 127) / 128) * 128;
  // ring depth: four stages for the long rows of untied decoders, more for short rows so that the copies in flight per
  // CTA stay in the tens of kilobytes
  int nstages = 4;
  while (nstages < kDecodeStages && nstages * stage_bytes < 24 * 1024) nstages *= 2;
  // long rows (d_model 2048 with many target layers): fewer, larger stages; two column chunks per thread
  while (nstages > 2 && size_t(nstages) * stage_bytes + sizeof(DecodeBulkShared) + 256 > 200 * 1024) --nstages;
  const size_t smem = size_t(nstages) * stage_bytes + sizeof(DecodeBulkShared) + 256;
  const bool plain_tied = a->tying == 1 && a->feat_offset == nullptr && a->feat_scale == nullptr;
  const int vchunks = a->d > 1024 ? 2 : 1;
  const int bulk_gthreads = vchunks == 2 ? ((a->d / 16 + 31) / 32) * 32 : gthreads;
  const bool bulk = (a->tying == 0 || plain_tied) && a->status != nullptr && tpg <= 4 && smem <= 200 * 1024 && bulk_gthreads * kGroups + 32 <= 544;
  if (bulk) {
    gthreads = bulk_gthreads;
    threads = gthreads * kGroups;
    static size_t attr_set[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    auto launch = [&](auto kern) -> int {
      size_t& have = attr_set[tpg + 5 * (vchunks - 1)];
      if (have < smem) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return -4;
        have = smem;
      }
      kern<<<dim3(a->B, 1), threads + 32, smem, st>>>(p, gthreads, stage_bytes, nstages, a->status);
      return 0;
    };
    int rc = 0;
    if (vchunks == 1) {
      if (tpg <= 1) rc = launch(decode_bulk_kernel<1, 1>);
      else if (tpg == 2) rc = launch(decode_bulk_kernel<2, 1>);
      else if (tpg == 3) rc = launch(decode_bulk_kernel<3, 1>);
      else rc = launch(decode_bulk_kernel<4, 1>);
    } else {
      if (tpg <= 1) rc = launch(decode_bulk_kernel<1, 2>);
      else if (tpg == 2) rc = launch(decode_bulk_kernel<2, 2>);
      else if (tpg == 3) rc = launch(decode_bulk_kernel<3, 2>);
      else rc = launch(decode_bulk_kernel<4, 2>);
    }
    if (rc != 0) return rc;
  } else if (tpg <= 1) decode_kernel<1><<<dim3(a->B, 1), threads, 0, st>>>(p, gthreads);
  else if (tpg == 2) decode_kernel<2><<<dim3(a->B, 1), threads, 0, st>>>(p, gthreads);
  else if (tpg == 3) decode_kernel<3><<<dim3(a->B, 1), threads, 0, st>>>(p, gthreads);
  else decode_kernel<4><<<dim3(a->B, (tpg + 3) / 4), threads, 0, st>>>(p, gthreads);  // 16 targets per pass
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int CLT_FN(clt_recon_epilogue)(const float* yhat_sum, const float* bias_sum, const float* addend, const void* target,
                                  const float* sigma, void* gs, float* yhat_out, double* sq_err, int L, int B, int d, int row0,
                                  int nrows, float* ctl, cudaStream_t st) {
  if (d % 8 != 0) return -1;
  if (nrows <= 0) return 0;
  dim3 grid(148, L);
  recon_epilogue_kernel<<<grid, 256, 0, st>>>(yhat_sum, bias_sum, addend, static_cast<const t16*>(target), sigma,
                                              static_cast<t16*>(gs), yhat_out, sq_err, L, B, d, row0, nrows, ctl);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int CLT_FN(clt_gs_colsum)(const void* gs, float* out, int L, int B, int d, cudaStream_t st) {
  if (d % 8 != 0) return -1;
  const int tx = d / 8 >= 128 ? 128 : ((d / 8 + 31) / 32) * 32;
  const int ty = 1024 / tx < 8 ? 1024 / tx : 8;
  const int rpb = 128;
  dim3 grid((d / 8 + tx - 1) / tx, (B + rpb - 1) / rpb, L), block(tx, ty);
  gs_colsum_kernel<<<grid, block, 0, st>>>(static_cast<const t16*>(gs), out, B, d, rpb);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int CLT_FN(clt_gs_suffix_sum)(const void* gs, void* out, int L, int B, int d, cudaStream_t st) {
  const long long per_layer = 1LL * B * d;
  if (per_layer % 8 != 0) return -1;
  const long long nvec = per_layer / 8;
  const int grid = int(nvec / 256 + 1 < 1184 ? nvec / 256 + 1 : 1184);
  gs_suffix_sum_kernel<<<grid, 256, 0, st>>>(static_cast<const t16*>(gs), static_cast<t16*>(out), L, per_layer);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
