// Global BatchTopK without a dense [B, L*F] ranking tensor (sm_100a).
//
// The reference concatenates every layer's batch-z-scored pre-activations and calls torch.topk on the
// flattened tensor (clt/models/activations.py:27-32, 281-357).  Here the same selection is a threshold
// search over the bf16 pre-activations written by the encoder GEMM:
//
//   1. colstats      per-feature batch mean and 1/(std+1e-6) (unbiased std, shifted sums)
//   2. zhist         8192-bin histogram of the order-preserving key of z = (x-mean)*rstd, keys >= key_lo
//   3. find_bin      bin that contains the k_total-th largest key (after the ranks' histograms were summed)
//   4. compact       entries above the bin go to the output list, entries inside it to a candidate list
//   5. refine        exact key cut inside the bin by radix passes; ties resolved by lowest flat index
//                    b*(L*F) + l*F + f so the result does not depend on the tensor-parallel world size
//   6. finalize      candidates on the keep side of the cut are appended to the output list
//   7. csr           token-major and feature-major CSR views of the list for the decoder / backward
//
// Under tensor parallelism every rank runs 1-2 and 4-7 on its feature shard; only histograms cross GPUs
// (the 8192-bin one and the 512-bin refinement rounds), written straight into the peers' exchange
// buffers by the kernels below with bounded flag waits.
#include "common.cuh"

namespace clt {

constexpr int kHistBins = 8192;
constexpr int kRefineBins = 512;

// Control block shared by the selection kernels (device memory, int64 slots).
enum SelCtl : int {
  CTL_BIN = 0,          // threshold bin
  CTL_ABOVE = 1,        // number of keys in bins above it (global over ranks)
  CTL_NEED = 2,         // how many the threshold bin has to contribute (global)
  CTL_NUM_ENTRIES = 3,  // length of the output list (this rank)
  CTL_NUM_CAND = 4,     // length of the candidate list (this rank)
  CTL_CUT_KEY = 5,      // exact key cut T
  CTL_TIE_MODE = 6,     // 0: keep every key == T; 1: keep ties with flat index <= CTL_CUT_FLAT
  CTL_CUT_FLAT = 7,
  CTL_KEY_LO = 8,       // histogram range actually used: keys >= key_lo, bin = (key - key_lo) >> shift
  CTL_SHIFT = 9,
  CTL_RETRY = 10,       // 1: the narrow histogram did not contain the cut, the full-range pass runs
  CTL_SIZE = 16,
};

// Sum `n` uint32 counters over all ranks, in place in shared memory `vals` (one CTA).  Every rank stores
// its vector into slot [round][rank] of every peer, raises flag [round][rank] there, then waits (bounded)
// for the flags of all peers in its own area and adds the slots up.  Returns false on a timeout.
__device__ bool exchange_sum(const Exchange& ex, int round, uint32_t* vals, int n, int* timeout_flag_smem) {
  if (ex.world <= 1) return true;
  if (!exchange_gather(ex, round, vals, n, timeout_flag_smem)) return false;
  const uint32_t* mine = exchange_slot(ex, round, 0);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    uint32_t s = 0;
    for (int p = 0; p < ex.world; ++p) s += mine[size_t(p) * ex.slot_elems + i];
    vals[i] = s;
  }
  __syncthreads();
  return true;
}

// ------------------------------------------------------------------ 1. column statistics
// x: [L, B, ld] bf16.  Each thread owns 8 adjacent columns; blockDim = (32, 8): 8 row groups.
// With gridDim.z > 1 (narrow shards, where one CTA per column block would leave SMs idle) the rows are split
// over blockIdx.z: the shifted sums are additive because every chunk shifts by the column's first row, so the
// chunks add them into mean / rstd (zeroed by the launcher) and colstats_finalize_kernel converts in place.
__global__ void __launch_bounds__(256) colstats_kernel(const t16* __restrict__ x, float* __restrict__ mean,
                                                         float* __restrict__ rstd, int B, int F, long long ld,
                                                         long long layer_stride) {
  const int l = blockIdx.y;
  const int rows_per_z = (((B + int(gridDim.z) - 1) / int(gridDim.z)) + 31) / 32 * 32;
  const int row_lo = int(blockIdx.z) * rows_per_z;
  const int row_hi = min(B, row_lo + rows_per_z);
  const int cg = blockIdx.x * 32 + threadIdx.x;  // column group of 8
  const int c0 = cg * 8;
  __shared__ float red[8][32][17];
  float s[8], q[8], shift[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s[j] = q[j] = shift[j] = 0.f;
  const bool active = c0 < F;
  const t16* base = x + 1LL * l * layer_stride + c0;
  if (active) {
    uint4 v0 = *reinterpret_cast<const uint4*>(base);
    const uint32_t w[4] = {v0.x, v0.y, v0.z, v0.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) { shift[2 * j] = t16_lo(w[j]); shift[2 * j + 1] = t16_hi(w[j]); }
    for (int r0 = row_lo + threadIdx.y; r0 < row_hi; r0 += 32) {
      uint4 v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {  // four independent loads in flight
        const int r = r0 + 8 * k;
        v[k] = r < row_hi ? __ldcs(reinterpret_cast<const uint4*>(base + 1LL * r * ld)) : v0;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (r0 + 8 * k >= row_hi) break;
        const uint32_t u[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = t16_lo(u[j]) - shift[2 * j], b = t16_hi(u[j]) - shift[2 * j + 1];
          s[2 * j] += a; q[2 * j] += a * a;
          s[2 * j + 1] += b; q[2 * j + 1] += b * b;
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) { red[threadIdx.y][threadIdx.x][j] = s[j]; red[threadIdx.y][threadIdx.x][8 + j] = q[j]; }
  __syncthreads();
  if (threadIdx.y == 0 && active) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float ss = 0.f, qq = 0.f;
      for (int y = 0; y < 8; ++y) { ss += red[y][threadIdx.x][j]; qq += red[y][threadIdx.x][8 + j]; }
      if (c0 + j < F && gridDim.z > 1) {
        atomicAdd(&mean[1LL * l * F + c0 + j], ss);
        atomicAdd(&rstd[1LL * l * F + c0 + j], qq);
      } else if (c0 + j < F) {
        const float mu = ss / float(B);
        float var = B > 1 ? (qq - ss * mu) / float(B - 1) : 0.f;
        var = fmaxf(var, 0.f);
        mean[1LL * l * F + c0 + j] = shift[j] + mu;
        rstd[1LL * l * F + c0 + j] = 1.f / (sqrtf(var) + 1e-6f);
      }
    }
  }
}

// Column statistics from the per-block sums that the encoder GEMM's epilogue leaves behind:
// tile_stats [L][row_blocks][F][2] = (sum, sum of squares) over the rows of one 128-row block.  The blocks are merged
// with the pairwise update of Chan et al. (block means first), which keeps the variance accurate when the mean is
// large against the spread.
__global__ void __launch_bounds__(256) colstats_from_tiles_kernel(const float* __restrict__ tile_stats, float* __restrict__ mean,
                                                                    float* __restrict__ rstd, int B, int F, int row_blocks, long long n) {
  const long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int l = int(i / F), c = int(i - 1LL * l * F);
  const float2* src = reinterpret_cast<const float2*>(tile_stats) + (1LL * l * row_blocks) * F + c;
  float cnt = 0.f, mu = 0.f, m2 = 0.f;
  for (int rb = 0; rb < row_blocks; ++rb) {
    const float2 sq = src[1LL * rb * F];
    const float nb = float(min(128, B - rb * 128));
    const float mb = sq.x / nb;
    const float m2b = fmaxf(sq.y - sq.x * mb, 0.f);
    const float tot = cnt + nb;
    const float delta = mb - mu;
    m2 += m2b + delta * delta * (cnt * nb / tot);
    mu += delta * (nb / tot);
    cnt = tot;
  }
  const float var = B > 1 ? fmaxf(m2 / float(B - 1), 0.f) : 0.f;
  mean[i] = mu;
  rstd[i] = 1.f / (sqrtf(var) + 1e-6f);
}

// mean / rstd hold the shifted sum and sum of squares (shift = the column's first row); convert in place.
__global__ void __launch_bounds__(256) colstats_finalize_kernel(const t16* __restrict__ x, float* __restrict__ mean,
                                                                  float* __restrict__ rstd, int B, int F, long long layer_stride,
                                                                  long long n) {
  const long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int l = int(i / F), c = int(i - 1LL * l * F);
  const float shift = t16_to_float(x[1LL * l * layer_stride + c]);
  const float ss = mean[i], qq = rstd[i];
  const float mu = ss / float(B);
  float var = B > 1 ? (qq - ss * mu) / float(B - 1) : 0.f;
  var = fmaxf(var, 0.f);
  mean[i] = shift + mu;
  rstd[i] = 1.f / (sqrtf(var) + 1e-6f);
}

// ------------------------------------------------------------------ 2. histogram of z keys
struct ScanGeom {
  int B, F, L;           // F = valid local columns per layer
  int sp;                // pitch of the mean / rstd rows (>= F)
  long long ld;          // row pitch of x (elements)
  long long layer_stride;
  int rows_per_block;
};

__device__ __forceinline__ void load_cols8(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}

// `only_if_retry`: the full-range pass; it runs only when the narrow pass asked for it.
__global__ void __launch_bounds__(256) zhist_kernel(const t16* __restrict__ x, const float* __restrict__ mean,
                                                      const float* __restrict__ rstd, ScanGeom g, uint32_t key_lo, int shift,
                                                      unsigned int* __restrict__ hist, const long long* __restrict__ ctl,
                                                      int only_if_retry) {
  if (only_if_retry && ctl[CTL_RETRY] == 0) return;
  const float z_lo = key_lo == 0u ? -INFINITY : key_to_float(key_lo);
  __shared__ unsigned int sh[kHistBins];
  for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const int l = blockIdx.z;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c0 < g.F) {
    float mu[8], rs[8];
    if (c0 + 8 <= g.F) {
      load_cols8(mean + 1LL * l * g.sp + c0, mu);
      load_cols8(rstd + 1LL * l * g.sp + c0, rs);
    } else {
      for (int j = 0; j < 8; ++j) {
        const bool in = c0 + j < g.F;
        mu[j] = in ? mean[1LL * l * g.sp + c0 + j] : 0.f;
        rs[j] = in ? rstd[1LL * l * g.sp + c0 + j] : 0.f;
      }
    }
    const int nvalid = min(8, g.F - c0);
    const int r0 = blockIdx.y * g.rows_per_block;
    const int r1 = min(g.B, r0 + g.rows_per_block);
    const t16* base = x + 1LL * l * g.layer_stride + c0;
    for (int rb = r0; rb < r1; rb += 4) {
      uint4 v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        v[k] = (rb + k < r1) ? __ldg(reinterpret_cast<const uint4*>(base + 1LL * (rb + k) * g.ld)) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (rb + k >= r1) break;
        const uint32_t u[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xv = (j & 1) ? t16_hi(u[j >> 1]) : t16_lo(u[j >> 1]);
          const float z = (xv - mu[j]) * rs[j];
          if (z >= z_lo && j < nvalid) {  // one float compare for the bulk; keys only for the tail that counts
            const uint32_t key = float_to_key(z);
            atomicAdd(&sh[min((key - key_lo) >> shift, uint32_t(kHistBins - 1))], 1u);
          }
        }
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) {
    const unsigned int c = sh[i];
    if (c) atomicAdd(&hist[i], c);
  }
}

// ------------------------------------------------------------------ 2b. histogram + pool in one pass
// The range of the narrow histogram lives in device memory (`sel_state`: key_lo, shift) and follows the
// cut from step to step (find_bin_kernel moves it).  Every element inside the range is also appended to a
// pool (key, token, column, value), so that the later stages read a list of a few k_total elements instead
// of the whole pre-activation matrix a second time.
struct Pool {
  uint32_t* key;
  int* tok;
  int* col;
  float* val;
  long long cap;
  unsigned int* count;  // zeroed by the caller together with the histograms
};
constexpr int kPoolStage = 512;   // histogram + queue + staging stay inside the 48 KB of static shared memory
constexpr int kHitQueue = 1024;   // 16-byte groups per CTA that passed the coarse filter
constexpr int kHistExtra = 32;    // words after the two histograms: [0] = pool counter

// Phase A streams the matrix with a coarse filter in the input's own format (one packed compare per two
// elements) and only queues the 16-byte groups that may hold an element of the range; phase B runs the exact
// test on the queued groups, one element per thread.  The hot loop stays a few instructions per group.
__global__ void __launch_bounds__(256) zhist_collect_kernel(const t16* __restrict__ x, const float* __restrict__ mean,
                                                              const float* __restrict__ rstd, ScanGeom g, int col_pitch,
                                                              const long long* __restrict__ sel_state,
                                                              unsigned int* __restrict__ hist, Pool pool) {
  const uint32_t key_lo = uint32_t(sel_state[0]);
  const int shift = int(sel_state[1]);
  const float z_lo = key_to_float(key_lo);
  __shared__ unsigned int sh[kHistBins];
  __shared__ uint32_t s_queue[kHitQueue];
  __shared__ uint32_t s_key[kPoolStage];
  __shared__ int s_tok[kPoolStage];
  __shared__ int s_col[kPoolStage];
  __shared__ float s_val[kPoolStage];
  __shared__ int s_q, s_n;
  __shared__ unsigned int s_base;
  for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) sh[i] = 0;
  if (threadIdx.x == 0) { s_q = 0; s_n = 0; }
  __syncthreads();
  const int l = blockIdx.z;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  const int r0 = blockIdx.y * g.rows_per_block;
  const int r1 = min(g.B, r0 + g.rows_per_block);
  if (c0 < g.F) {
    // thr_j = mean_j + z_lo / rstd_j, lowered by a margin for the fp32 rounding of the exact test and rounded
    // down to bf16: x >= thr_j is implied by z_j >= z_lo
    uint32_t thr2[4];
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      float t[2];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const bool in = c0 + j + q < g.F;
        const float mu = in ? __ldg(mean + 1LL * l * g.sp + c0 + j + q) : 0.f;
        const float rs = in ? __ldg(rstd + 1LL * l * g.sp + c0 + j + q) : 0.f;
        const float span = z_lo / rs;
        t[q] = (in && rs > 0.f) ? mu + span - 1e-5f * (fabsf(mu) + fabsf(span)) - 1e-30f : INFINITY;
      }
      const t16x2 pk = make_t16x2(float_to_t16_rd(t[0]), float_to_t16_rd(t[1]));
      thr2[j >> 1] = *reinterpret_cast<const uint32_t*>(&pk);
    }
    const t16* base = x + 1LL * l * g.layer_stride + c0;
    for (int rb = r0; rb < r1; rb += 8) {
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int r = min(rb + k, r1 - 1);
        v[k] = __ldcs(reinterpret_cast<const uint4*>(base + 1LL * r * g.ld));
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t hit = t16x2_ge_mask(v[k].x, thr2[0]) | t16x2_ge_mask(v[k].y, thr2[1]) |
                             t16x2_ge_mask(v[k].z, thr2[2]) | t16x2_ge_mask(v[k].w, thr2[3]);
        if (hit != 0 && rb + k < r1) {
          const int slot = atomicAdd(&s_q, 1);
          if (slot < kHitQueue) s_queue[slot] = (uint32_t(rb + k - r0) << 8) | threadIdx.x;
        }
      }
    }
  }
  __syncthreads();
  // ---- phase B: exact test, histogram and pool staging, one element per thread
  const int nq_all = s_q;
  if (nq_all > kHitQueue && threadIdx.x == 0) atomicOr(pool.count, 0x80000000u);  // lost groups: force the full-range pass
  const int nq = min(nq_all, kHitQueue);
  for (int e = threadIdx.x; e < nq * 8; e += blockDim.x) {
    const uint32_t item = s_queue[e >> 3];
    const int r = r0 + int(item >> 8);
    const int c = (blockIdx.x * blockDim.x + int(item & 255u)) * 8 + (e & 7);
    if (c >= g.F) continue;
    const float xv = t16_to_float(x[1LL * l * g.layer_stride + 1LL * r * g.ld + c]);
    const float z = (xv - __ldg(mean + 1LL * l * g.sp + c)) * __ldg(rstd + 1LL * l * g.sp + c);
    if (!(z >= z_lo)) continue;
    const uint32_t key = float_to_key(z);
    atomicAdd(&sh[min((key - key_lo) >> shift, uint32_t(kHistBins - 1))], 1u);
    const int slot = atomicAdd(&s_n, 1);
    if (slot < kPoolStage) {
      s_key[slot] = key; s_tok[slot] = r; s_col[slot] = l * col_pitch + c; s_val[slot] = xv;
    } else {  // staging full: append directly
      const unsigned int q = atomicAdd(pool.count, 1u);
      if ((long long)q < pool.cap) { pool.key[q] = key; pool.tok[q] = r; pool.col[q] = l * col_pitch + c; pool.val[q] = xv; }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kHistBins; i += blockDim.x) {
    const unsigned int c = sh[i];
    if (c) atomicAdd(&hist[i], c);
  }
  const int staged = min(s_n, kPoolStage);
  if (staged == 0) return;
  if (threadIdx.x == 0) s_base = atomicAdd(pool.count, (unsigned int)staged);
  __syncthreads();
  for (int i = threadIdx.x; i < staged; i += blockDim.x) {
    const long long q = (long long)s_base + i;
    if (q < pool.cap) { pool.key[q] = s_key[i]; pool.tok[q] = s_tok[i]; pool.col[q] = s_col[i]; pool.val[q] = s_val[i]; }
  }
}

// ------------------------------------------------------------------ 3. threshold bin (one CTA, 1024 threads)
// pass 0: narrow histogram; when it does not contain the cut it only raises CTL_RETRY.
// pass 1: full-range histogram, runs only on retry; a miss there is a real error.
struct Lists {
  int* ent_tok;    // token index
  int* ent_col;    // l * F_local_pitch + f_local
  float* ent_val;  // original pre-activation
  long long ent_cap;
  uint32_t* cand_key;
  int* cand_tok;
  int* cand_col;
  float* cand_val;
  long long cand_cap;
};

// `sel_state` (optional): the tracked range.  Pass 0 reads the range from it; the pass that finds the cut
// moves the range for the next step so that about kPoolFactor * k_total elements fall inside it.
constexpr double kPoolFactor = 1.75;

// Bin width for a tracked range that starts at key_lo: the bins resolve z in [z_lo, max(2 z_lo, z_lo + 4)];
// everything above lands in the top bin (kernels clamp the bin index), which is therefore never accepted as
// the threshold bin.  Finer bins leave fewer candidates for the exact cut.
__device__ __forceinline__ int shift_for(uint32_t key_lo) {
  const float z_lo = key_to_float(key_lo);
  const uint32_t key_hi = float_to_key(fmaxf(2.f * z_lo, z_lo + 4.f));
  const uint32_t span = key_hi > key_lo ? key_hi - key_lo : 0xFFFFFFFFu - key_lo;
  int sh = 0;
  while ((span >> sh) >= uint32_t(kHistBins - 1)) ++sh;
  return sh;
}

__global__ void __launch_bounds__(1024) find_bin_kernel(const unsigned int* __restrict__ hist, long long k_total,
                                                          long long* __restrict__ ctl, Exchange ex, uint32_t key_lo_arg,
                                                          int shift_arg, int pass, int exchange_round,
                                                          long long* __restrict__ sel_state,
                                                          const unsigned int* __restrict__ pool_count, long long pool_cap,
                                                          int* __restrict__ status) {
  __shared__ uint32_t vals[kHistBins + kHistExtra];
  __shared__ unsigned long long part[1024];
  __shared__ int timeout;
  __shared__ int found;
  const int tid = threadIdx.x;
  if (pass == 1 && ctl[CTL_RETRY] == 0) return;
  const bool tracked = sel_state != nullptr;
  const uint32_t key_lo = (pass == 0 && tracked) ? uint32_t(sel_state[0]) : key_lo_arg;
  const int shift = (pass == 0 && tracked) ? int(sel_state[1]) : shift_arg;
  if (tid == 0) { timeout = 0; found = 0; }
  for (int i = tid; i < kHistBins; i += 1024) vals[i] = hist[i];
  if (tid < kHistExtra) vals[kHistBins + tid] = 0;
  __syncthreads();
  // a rank whose pool overflowed makes every rank take the full-range path
  if (tid == 0 && pass == 0 && pool_count != nullptr && (long long)(*pool_count) > pool_cap) vals[kHistBins] = 1;
  __syncthreads();
  if (!exchange_sum(ex, exchange_round, vals, kHistBins + 1, &timeout)) {
    if (tid == 0) atomicCAS(status, STATUS_OK, STATUS_WAIT_TIMEOUT);
    return;
  }
  const bool overflow = vals[kHistBins] != 0;
  // thread t owns bins [8t, 8t+8); part[t] = number of keys in the bins of all threads above t (suffix scan:
  // shuffles inside a warp, then over the 32 warp totals)
  unsigned long long mine = 0;
  for (int j = 0; j < 8; ++j) mine += vals[tid * 8 + j];
  {
    __shared__ unsigned long long warp_tot[32], warp_above[32];
    const int lane = tid & 31, warp = tid >> 5;
    unsigned long long incl = mine;  // sum over lanes >= this lane
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const unsigned long long t = __shfl_down_sync(0xFFFFFFFFu, incl, o);
      if (lane + o < 32) incl += t;
    }
    if (lane == 0) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      unsigned long long w = warp_tot[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long t = __shfl_down_sync(0xFFFFFFFFu, w, o);
        if (lane + o < 32) w += t;
      }
      warp_above[lane] = w - warp_tot[lane];
    }
    __syncthreads();
    part[tid] = (incl - mine) + warp_above[warp];
  }
  __syncthreads();
  unsigned long long total = 0;
  if (tid == 0) {
    const unsigned long long run = part[0] + mine;
    total = run;
    // tracked ranges clamp large keys into the top bin: a cut inside it cannot be refined, take the full pass
    const bool top_bin_cut = tracked && pass == 0 && (unsigned long long)vals[kHistBins - 1] >= (unsigned long long)k_total;
    const bool in_range = run >= (unsigned long long)k_total;
    found = (in_range && !overflow && !top_bin_cut) ? 1 : 0;
    if (!found) {
      if (pass == 0) ctl[CTL_RETRY] = 1;
      else atomicCAS(status, STATUS_OK, STATUS_SELECT_RANGE);
    } else if (pass == 0) {
      ctl[CTL_RETRY] = 0;
    }
    if (pass == 0 || found) {
      ctl[CTL_NUM_ENTRIES] = 0;
      ctl[CTL_NUM_CAND] = 0;
    }
    if (tracked && pass == 0 && !in_range) {
      // the range starts above the cut: lower it (the full-range pass of this step refines the guess)
      const float z = fmaxf(key_to_float(key_lo) - 0.1f, 0.f);
      const uint32_t nk = float_to_key(z);
      sel_state[0] = (long long)nk;
      sel_state[1] = shift_for(nk);
    }
  }
  __syncthreads();
  const unsigned long long target = (unsigned long long)(kPoolFactor * double(k_total));
  unsigned long long above = part[tid];  // keys in bins above this thread's group
  for (int j = 7; j >= 0; --j) {
    const unsigned long long c = vals[tid * 8 + j];
    if (found && above < (unsigned long long)k_total && above + c >= (unsigned long long)k_total) {
      ctl[CTL_BIN] = tid * 8 + j;
      ctl[CTL_ABOVE] = (long long)above;
      ctl[CTL_NEED] = k_total - (long long)above;
      ctl[CTL_KEY_LO] = (long long)key_lo;
      ctl[CTL_SHIFT] = shift;
    }
    if (tracked && above < target && above + c >= target) {
      // next step's range starts at the bin that holds the target-th largest key (never below z = 0)
      const unsigned long long nk64 = (unsigned long long)key_lo + ((unsigned long long)(tid * 8 + j) << shift);
      uint32_t nk = nk64 > 0xFFFFFFFFULL ? 0xFFFFFFFFu : uint32_t(nk64);
      if (nk < 0x80000000u) nk = 0x80000000u;
      sel_state[0] = (long long)nk;
      sel_state[1] = shift_for(nk);
    }
    above += c;
  }
  if (tracked && tid == 0 && found && total < target) {
    // fewer elements in range than wanted: widen a little for the next step
    const float z = fmaxf(key_to_float(key_lo) - 0.1f, 0.f);
    const uint32_t nk = float_to_key(z);
    sel_state[0] = (long long)nk;
    sel_state[1] = shift_for(nk);
  }
}

// ------------------------------------------------------------------ 2c. per-feature threshold selection
// JumpReLU (x >= theta_f) and ReLU (theta = smallest positive bf16) as a sparse selection: the same two-phase
// scan as above with the feature's own threshold as the filter; emits the (token, column, value) list that the
// CSR build and the sparse decode consume.  Meant for sparse activations: when a CTA queues more groups than
// its queue holds, or the list does not fit, the status word reports STATUS_CAPACITY and the caller falls back
// to the dense path.
__global__ void __launch_bounds__(256) threshold_collect_kernel(const t16* __restrict__ x, const float* __restrict__ theta,
                                                                  ScanGeom g, int col_pitch, long long* __restrict__ ctl,
                                                                  Lists o, int* __restrict__ status) {
  __shared__ uint32_t s_queue[4 * kHitQueue];
  __shared__ int s_tok[2 * kPoolStage];
  __shared__ int s_col[2 * kPoolStage];
  __shared__ float s_val[2 * kPoolStage];
  __shared__ int s_q, s_n;
  __shared__ unsigned long long s_base;
  constexpr int kQueue = 4 * kHitQueue, kStage = 2 * kPoolStage;
  if (threadIdx.x == 0) { s_q = 0; s_n = 0; }
  __syncthreads();
  const int l = blockIdx.z;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  const int r0 = blockIdx.y * g.rows_per_block;
  const int r1 = min(g.B, r0 + g.rows_per_block);
  unsigned long long* n_ent = reinterpret_cast<unsigned long long*>(ctl + CTL_NUM_ENTRIES);
  if (c0 < g.F) {
    uint32_t thr2[4];
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      float t[2];
#pragma unroll
      for (int q = 0; q < 2; ++q) t[q] = c0 + j + q < g.F ? __ldg(theta + 1LL * l * g.sp + c0 + j + q) : INFINITY;
      const t16x2 pk = make_t16x2(float_to_t16_rd(t[0]), float_to_t16_rd(t[1]));
      thr2[j >> 1] = *reinterpret_cast<const uint32_t*>(&pk);
    }
    const t16* base = x + 1LL * l * g.layer_stride + c0;
    for (int rb = r0; rb < r1; rb += 8) {
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int r = min(rb + k, r1 - 1);
        v[k] = __ldcs(reinterpret_cast<const uint4*>(base + 1LL * r * g.ld));
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t hit = t16x2_ge_mask(v[k].x, thr2[0]) | t16x2_ge_mask(v[k].y, thr2[1]) |
                             t16x2_ge_mask(v[k].z, thr2[2]) | t16x2_ge_mask(v[k].w, thr2[3]);
        if (hit != 0 && rb + k < r1) {
          const int slot = atomicAdd(&s_q, 1);
          if (slot < kQueue) s_queue[slot] = (uint32_t(rb + k - r0) << 8) | threadIdx.x;
        }
      }
    }
  }
  __syncthreads();
  const int nq_all = s_q;
  if (nq_all > kQueue && threadIdx.x == 0) atomicCAS(status, STATUS_OK, STATUS_CAPACITY);  // too dense for this path
  const int nq = min(nq_all, kQueue);
  for (int e0 = 0; e0 < nq * 8; e0 += kStage) {
    // exact test, staged in rounds so that any number of queued groups fits the staging arrays
    const int e1 = min(nq * 8, e0 + kStage);
    for (int e = e0 + threadIdx.x; e < e1; e += blockDim.x) {
      const uint32_t item = s_queue[e >> 3];
      const int r = r0 + int(item >> 8);
      const int c = (blockIdx.x * blockDim.x + int(item & 255u)) * 8 + (e & 7);
      if (c >= g.F) continue;
      const float xv = t16_to_float(x[1LL * l * g.layer_stride + 1LL * r * g.ld + c]);
      if (!(xv >= __ldg(theta + 1LL * l * g.sp + c))) continue;
      const int slot = atomicAdd(&s_n, 1);
      s_tok[slot] = r; s_col[slot] = l * col_pitch + c; s_val[slot] = xv;
    }
    __syncthreads();
    const int staged = s_n;
    if (threadIdx.x == 0) s_base = staged ? atomicAdd(n_ent, (unsigned long long)staged) : 0ULL;
    __syncthreads();
    for (int i = threadIdx.x; i < staged; i += blockDim.x) {
      const long long q = (long long)s_base + i;
      if (q < o.ent_cap) { o.ent_tok[q] = s_tok[i]; o.ent_col[q] = s_col[i]; o.ent_val[q] = s_val[i]; }
      else atomicCAS(status, STATUS_OK, STATUS_CAPACITY);
    }
    __syncthreads();
    if (threadIdx.x == 0) s_n = 0;
    __syncthreads();
  }
}

// ------------------------------------------------------------------ 2d. per-token top-k (TokenTopK)
// Every token keeps its k largest z-scores over all layers' features (reference: torch.topk(dim=-1) + scatter_,
// clt/models/activations.py:121-124, ranking on the per-feature batch z-scores).  One CTA handles four tokens (so
// that the per-column statistics are loaded once for four rows) and finds each token's k-th largest key exactly
// with a three-round radix select over the 32-bit keys (11 + 11 + 10 bits, histograms in shared memory), then
// emits the entries above the cut and the lowest-index ties at the cut.  Output: exactly k entries per token at
// [token * k, token * k + k) of the entry list.
constexpr int kTokPerCta = 4;
constexpr int kTokBins = 2048;
constexpr int kTieCap = 256;

struct TokenTopkShared {
  uint32_t hist[kTokPerCta][kTokBins];
  uint32_t prefix[kTokPerCta], mask[kTokPerCta];
  unsigned int need[kTokPerCta];
  int emitted[kTokPerCta];
  int nties[kTokPerCta];
  int tie_col[kTokPerCta][kTieCap];
  float tie_val[kTokPerCta][kTieCap];
};

template <typename Fn>
__device__ __forceinline__ void token_rows_scan(const t16* __restrict__ x, const float* __restrict__ mean,
                                                const float* __restrict__ rstd, const ScanGeom& g, int tok0, int ntok, Fn fn) {
  for (int l = 0; l < g.L; ++l) {
    for (int c0 = threadIdx.x * 8; c0 < g.F; c0 += blockDim.x * 8) {
      float mu[8], rs[8];
      load_cols8(mean + 1LL * l * g.sp + c0, mu);
      load_cols8(rstd + 1LL * l * g.sp + c0, rs);
      uint4 v[kTokPerCta];
#pragma unroll
      for (int t = 0; t < kTokPerCta; ++t)
        v[t] = t < ntok ? __ldg(reinterpret_cast<const uint4*>(x + 1LL * l * g.layer_stride + 1LL * (tok0 + t) * g.ld + c0)) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int t = 0; t < kTokPerCta; ++t) {
        if (t >= ntok) break;
        const uint32_t u[4] = {v[t].x, v[t].y, v[t].z, v[t].w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xv = (j & 1) ? t16_hi(u[j >> 1]) : t16_lo(u[j >> 1]);
          fn(t, l, c0 + j, xv, float_to_key((xv - mu[j]) * rs[j]));
        }
      }
    }
  }
}

__global__ void __launch_bounds__(256) token_topk_kernel(const t16* __restrict__ x, const float* __restrict__ mean,
                                                           const float* __restrict__ rstd, ScanGeom g, int col_pitch, int f_valid, int k,
                                                           long long* __restrict__ ctl, Lists o, int* __restrict__ status) {
  extern __shared__ uint8_t tk_smem[];
  TokenTopkShared* sh = reinterpret_cast<TokenTopkShared*>(tk_smem);
  const int tok0 = blockIdx.x * kTokPerCta;
  const int ntok = min(kTokPerCta, g.B - tok0);
  const int tid = threadIdx.x;
  if (tid < kTokPerCta) { sh->prefix[tid] = 0; sh->mask[tid] = 0; sh->need[tid] = (unsigned int)k; sh->emitted[tid] = 0; sh->nties[tid] = 0; }
  if (blockIdx.x == 0 && tid == 0) ctl[CTL_NUM_ENTRIES] = 1LL * g.B * k;
  // ---- exact k-th largest key per token: radix select, most significant digits first
  const int shifts[3] = {21, 10, 0};
  const int widths[3] = {11, 11, 10};
  for (int round = 0; round < 3; ++round) {
    const int shift = shifts[round];
    const uint32_t nb = 1u << widths[round];
    for (int i = tid; i < kTokPerCta * kTokBins; i += blockDim.x) (&sh->hist[0][0])[i] = 0;
    __syncthreads();
    token_rows_scan(x, mean, rstd, g, tok0, ntok, [&](int t, int, int c, float, uint32_t key) {
      if (c < f_valid && (key & sh->mask[t]) == sh->prefix[t]) atomicAdd(&sh->hist[t][(key >> shift) & (nb - 1u)], 1u);
    });
    __syncthreads();
    if (tid < ntok) {
      // digit that holds the need-th largest remaining key (counting from the top)
      unsigned int run = 0, need = sh->need[tid];
      int digit = 0;
      for (int b = int(nb) - 1; b >= 0; --b) {
        const unsigned int c = sh->hist[tid][b];
        if (run + c >= need) { digit = b; break; }
        run += c;
      }
      sh->need[tid] = need - run;
      sh->prefix[tid] |= uint32_t(digit) << shift;
      sh->mask[tid] |= (nb - 1u) << shift;
    }
    __syncthreads();
  }
  // prefix[t] is now the cut key T of token t, need[t] the number of keys equal to T that are kept
  token_rows_scan(x, mean, rstd, g, tok0, ntok, [&](int t, int l, int c, float xv, uint32_t key) {
    const uint32_t T = sh->prefix[t];
    if (c >= f_valid) return;  // padding columns of a shard take no part
    if (key > T) {
      const int slot = atomicAdd(&sh->emitted[t], 1);
      if (slot < k) {
        const long long q = 1LL * (tok0 + t) * k + slot;
        o.ent_tok[q] = tok0 + t; o.ent_col[q] = l * col_pitch + c; o.ent_val[q] = xv;
      }
    } else if (key == T) {
      const int i = atomicAdd(&sh->nties[t], 1);
      if (i < kTieCap) { sh->tie_col[t][i] = l * col_pitch + c; sh->tie_val[t][i] = xv; }
    }
  });
  __syncthreads();
  // ---- ties at the cut: the lowest flat indices first (l * col_pitch + c grows with the reference's column order)
  for (int t = 0; t < ntok; ++t) {
    const int n = sh->nties[t];
    const int need = int(sh->need[t]);
    const int above = sh->emitted[t];
    if (n > kTieCap && need < n) {
      if (tid == 0) atomicCAS(status, STATUS_OK, STATUS_TIE_OVERFLOW);
      continue;
    }
    if (tid == 0 && above + need != k) atomicCAS(status, STATUS_OK, STATUS_SELECT_RANGE);
    for (int i = tid; i < min(n, kTieCap); i += blockDim.x) {
      const int ci = sh->tie_col[t][i];
      int rank = 0;
      for (int j = 0; j < min(n, kTieCap); ++j) rank += sh->tie_col[t][j] < ci;
      if (rank < need && above + rank < k) {
        const long long q = 1LL * (tok0 + t) * k + above + rank;
        o.ent_tok[q] = tok0 + t; o.ent_col[q] = ci; o.ent_val[q] = sh->tie_val[t][i];
      }
    }
  }
}

// ------------------------------------------------------------------ 3b. split the pool at the threshold bin
// Runs instead of the full compaction pass when the tracked range contained the cut.
__global__ void __launch_bounds__(256) classify_pool_kernel(Pool pool, long long* __restrict__ ctl, Lists o,
                                                              int* __restrict__ status) {
  if (ctl[CTL_RETRY] != 0) return;
  const uint32_t tbin = uint32_t(ctl[CTL_BIN]);
  const uint32_t key_lo = uint32_t(ctl[CTL_KEY_LO]);
  const int shift = int(ctl[CTL_SHIFT]);
  unsigned long long* n_ent = reinterpret_cast<unsigned long long*>(ctl + CTL_NUM_ENTRIES);
  unsigned long long* n_cand = reinterpret_cast<unsigned long long*>(ctl + CTL_NUM_CAND);
  const long long n = min((long long)(*pool.count), pool.cap);
  // every CTA owns one contiguous slice of the pool: count, reserve once per list, then place
  const long long per_cta = (n + gridDim.x - 1) / gridDim.x;
  const long long lo = blockIdx.x * per_cta, hi = min(n, lo + per_cta);
  __shared__ int cnt[2];
  __shared__ unsigned long long base[2];
  if (threadIdx.x < 2) cnt[threadIdx.x] = 0;
  __syncthreads();
  int my_ent = 0, my_cand = 0;
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const uint32_t bin = min((pool.key[i] - key_lo) >> shift, uint32_t(kHistBins - 1));
    my_ent += bin > tbin;
    my_cand += bin == tbin;
  }
  if (my_ent) atomicAdd(&cnt[0], my_ent);
  if (my_cand) atomicAdd(&cnt[1], my_cand);
  __syncthreads();
  if (threadIdx.x == 0) {
    base[0] = cnt[0] ? atomicAdd(n_ent, (unsigned long long)cnt[0]) : 0ULL;
    base[1] = cnt[1] ? atomicAdd(n_cand, (unsigned long long)cnt[1]) : 0ULL;
    cnt[0] = 0; cnt[1] = 0;
  }
  __syncthreads();
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const uint32_t key = pool.key[i];
    const uint32_t bin = min((key - key_lo) >> shift, uint32_t(kHistBins - 1));
    if (bin > tbin) {
      const long long q = (long long)base[0] + atomicAdd(&cnt[0], 1);
      if (q < o.ent_cap) { o.ent_tok[q] = pool.tok[i]; o.ent_col[q] = pool.col[i]; o.ent_val[q] = pool.val[i]; }
      else atomicCAS(status, STATUS_OK, STATUS_CAPACITY);
    } else if (bin == tbin) {
      const long long q = (long long)base[1] + atomicAdd(&cnt[1], 1);
      if (q < o.cand_cap) { o.cand_key[q] = key; o.cand_tok[q] = pool.tok[i]; o.cand_col[q] = pool.col[i]; o.cand_val[q] = pool.val[i]; }
      else atomicCAS(status, STATUS_OK, STATUS_CAPACITY);
    }
  }
}

// ------------------------------------------------------------------ 4. compaction

// Selected elements are staged in shared memory and appended with one global reservation per CTA and
// list: a single counter cannot absorb one atomic per selected element (hundreds of thousands per step).
constexpr int kStageCap = 1024;

__global__ void __launch_bounds__(256) compact_kernel(const t16* __restrict__ x, const float* __restrict__ mean,
                                                        const float* __restrict__ rstd, ScanGeom g, int col_pitch,
                                                        long long* __restrict__ ctl, Lists o, int* __restrict__ status,
                                                        int only_if_retry) {
  if (only_if_retry && ctl[CTL_RETRY] == 0) return;
  __shared__ int s_tok[kStageCap];
  __shared__ int s_col[kStageCap];
  __shared__ float s_val[kStageCap];
  __shared__ uint32_t s_key[kStageCap];  // 0 marks a definite entry, otherwise the candidate's key (never 0 here)
  __shared__ int s_n;
  __shared__ unsigned long long s_base_ent, s_base_cand;
  __shared__ int s_cnt_ent, s_cnt_cand;
  if (threadIdx.x == 0) { s_n = 0; s_cnt_ent = 0; s_cnt_cand = 0; }
  __syncthreads();
  const int l = blockIdx.z;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  const uint32_t tbin = uint32_t(ctl[CTL_BIN]);
  const uint32_t key_lo = uint32_t(ctl[CTL_KEY_LO]);
  const int shift = int(ctl[CTL_SHIFT]);
  // smallest key that can matter: everything below the threshold bin is dropped with one compare
  const unsigned long long lo64 = (unsigned long long)key_lo + ((unsigned long long)tbin << shift);
  const uint32_t key_min = lo64 > 0xFFFFFFFFULL ? 0xFFFFFFFFu : uint32_t(lo64);
  const float z_min = key_min == 0u ? -INFINITY : key_to_float(key_min);
  unsigned long long* n_ent = reinterpret_cast<unsigned long long*>(ctl + CTL_NUM_ENTRIES);
  unsigned long long* n_cand = reinterpret_cast<unsigned long long*>(ctl + CTL_NUM_CAND);
  if (c0 < g.F) {
    float mu[8], rs[8];
    if (c0 + 8 <= g.F) {
      load_cols8(mean + 1LL * l * g.sp + c0, mu);
      load_cols8(rstd + 1LL * l * g.sp + c0, rs);
    } else {
      for (int j = 0; j < 8; ++j) {
        const bool in = c0 + j < g.F;
        mu[j] = in ? mean[1LL * l * g.sp + c0 + j] : 0.f;
        rs[j] = in ? rstd[1LL * l * g.sp + c0 + j] : 0.f;
      }
    }
    const int nvalid = min(8, g.F - c0);
    const int r0 = blockIdx.y * g.rows_per_block;
    const int r1 = min(g.B, r0 + g.rows_per_block);
    const t16* base = x + 1LL * l * g.layer_stride + c0;
    for (int rb = r0; rb < r1; rb += 4) {
      uint4 v[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int r = min(rb + k, r1 - 1);
        v[k] = __ldcs(reinterpret_cast<const uint4*>(base + 1LL * r * g.ld));
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int r = rb + k;
        const uint32_t u[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xv = (j & 1) ? t16_hi(u[j >> 1]) : t16_lo(u[j >> 1]);
          const float z = (xv - mu[j]) * rs[j];
          if (!(z >= z_min) || j >= nvalid || r >= r1) continue;
          const uint32_t key = float_to_key(z);
          const uint32_t bin = min((key - key_lo) >> shift, uint32_t(kHistBins - 1));
          if (bin < tbin) continue;
          const bool is_ent = bin > tbin;
          const int slot = atomicAdd(&s_n, 1);
          if (slot < kStageCap) {
            s_tok[slot] = r; s_col[slot] = l * col_pitch + c0 + j; s_val[slot] = xv; s_key[slot] = is_ent ? 0u : key;
            atomicAdd(is_ent ? &s_cnt_ent : &s_cnt_cand, 1);
          } else if (is_ent) {  // staging full: append directly
            const unsigned long long p = atomicAdd(n_ent, 1ULL);
            if ((long long)p < o.ent_cap) { o.ent_tok[p] = r; o.ent_col[p] = l * col_pitch + c0 + j; o.ent_val[p] = xv; }
            else atomicCAS(status, STATUS_OK, STATUS_CAPACITY);
          } else {
            const unsigned long long p = atomicAdd(n_cand, 1ULL);
            if ((long long)p < o.cand_cap) { o.cand_key[p] = key; o.cand_tok[p] = r; o.cand_col[p] = l * col_pitch + c0 + j; o.cand_val[p] = xv; }
            else atomicCAS(status, STATUS_OK, STATUS_CAPACITY);
          }
        }
      }
    }
  }
  __syncthreads();
  const int staged = min(s_n, kStageCap);
  if (staged == 0) return;
  if (threadIdx.x == 0) {
    s_base_ent = s_cnt_ent ? atomicAdd(n_ent, (unsigned long long)s_cnt_ent) : 0ULL;
    s_base_cand = s_cnt_cand ? atomicAdd(n_cand, (unsigned long long)s_cnt_cand) : 0ULL;
    s_cnt_ent = 0; s_cnt_cand = 0;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < staged; i += blockDim.x) {
    const uint32_t key = s_key[i];
    if (key == 0u) {
      const unsigned long long p = s_base_ent + (unsigned long long)atomicAdd(&s_cnt_ent, 1);
      if ((long long)p < o.ent_cap) { o.ent_tok[p] = s_tok[i]; o.ent_col[p] = s_col[i]; o.ent_val[p] = s_val[i]; }
      else atomicCAS(status, STATUS_OK, STATUS_CAPACITY);
    } else {
      const unsigned long long p = s_base_cand + (unsigned long long)atomicAdd(&s_cnt_cand, 1);
      if ((long long)p < o.cand_cap) { o.cand_key[p] = key; o.cand_tok[p] = s_tok[i]; o.cand_col[p] = s_col[i]; o.cand_val[p] = s_val[i]; }
      else atomicCAS(status, STATUS_OK, STATUS_CAPACITY);
    }
  }
}

// ------------------------------------------------------------------ 5. exact cut inside the bin (one CTA)
constexpr int kGatherCap = 4096;   // candidates (all ranks together) that the one-round exact cut handles
constexpr int kGatherSlot = 4096;  // ... and per rank: 2 + 2 * 4096 words fit one exchange slot (8224 words)
struct FlatGeom {
  int col_pitch;        // local column pitch used in ent_col / cand_col
  int feat_offset;      // first global feature of this shard
  long long full_F;     // un-sharded features per layer
  long long row_width;  // L * full_F
};
__device__ __forceinline__ unsigned long long flat_index(const FlatGeom& fg, int tok, int col) {
  const int l = col / fg.col_pitch, f = col - l * fg.col_pitch;
  return (unsigned long long)tok * (unsigned long long)fg.row_width + (unsigned long long)l * fg.full_F + (unsigned long long)(fg.feat_offset + f);
}

// Picks the digit whose bucket contains the `need`-th element counting from the top (descending=true)
// or from the bottom (descending=false).  Writes the digit and the remaining need.
__device__ void pick_digit(const uint32_t* hist, int nb, bool descending, unsigned long long need, int* digit_out,
                           unsigned long long* need_out) {
  if (threadIdx.x == 0) {
    unsigned long long run = 0;
    int d = descending ? nb - 1 : 0;
    for (int i = 0; i < nb; ++i) {
      const int b = descending ? nb - 1 - i : i;
      const unsigned long long c = hist[b];
      if (run + c >= need) { d = b; break; }
      run += c;
      d = b;
    }
    *digit_out = d;
    *need_out = need - run;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(1024) refine_kernel(const uint32_t* __restrict__ cand_key, const int* __restrict__ cand_tok,
                                                        const int* __restrict__ cand_col, long long cand_cap,
                                                        FlatGeom fg, long long* __restrict__ ctl, Exchange ex,
                                                        int* __restrict__ status) {
  const int shift = int(ctl[CTL_SHIFT]);
  const uint32_t key_lo = uint32_t(ctl[CTL_KEY_LO]);  // bins are over (key - key_lo): refine on the same offset
  __shared__ uint32_t hist[kRefineBins];
  __shared__ int digit;
  __shared__ unsigned long long need;
  __shared__ int timeout;
  const int tid = threadIdx.x;
  long long n = ctl[CTL_NUM_CAND];
  if (n > cand_cap) n = cand_cap;
  if (tid == 0) { timeout = 0; need = (unsigned long long)ctl[CTL_NEED]; }
  __syncthreads();
  const uint32_t low_mask = shift >= 32 ? 0xFFFFFFFFu : ((1u << shift) - 1u);
  // ---- fast path: one all-gather of the candidates of the threshold bin, exact cut found locally.
  // A candidate travels as one 64-bit word: (low key bits << 45) | (2^45 - 1 - flat index), so that a larger word
  // ranks first and, among equal keys, the lowest flat index does.  Every rank sorts out the same cut from the
  // same words.  Bins with more candidates than the gather holds (heavy ties) take the radix rounds below.
  {
    __shared__ unsigned long long comp[kGatherCap];
    __shared__ int total_s, fits_s;
    constexpr unsigned long long kFlatMask = (1ULL << 45) - 1ULL;
    const bool local_fits = n <= kGatherSlot && shift <= 19;
    const int world = ex.world <= 1 ? 1 : ex.world;
    // own candidates -> comp[0 .. n) (single rank) or through the exchange area
    if (world == 1) {
      if (tid == 0) { total_s = int(n); fits_s = (local_fits && n <= kGatherCap) ? 1 : 0; }
      __syncthreads();
      if (fits_s)
        for (long long i = tid; i < n; i += 1024)
          comp[i] = ((unsigned long long)((cand_key[i] - key_lo) & low_mask) << 45) | (kFlatMask - flat_index(fg, cand_tok[i], cand_col[i]));
    } else {
      // message: word 0 = count (0xFFFFFFFF: does not fit), then the 64-bit words
      uint32_t* msg = reinterpret_cast<uint32_t*>(comp);
      if (tid == 0) { msg[0] = local_fits ? uint32_t(n) : 0xFFFFFFFFu; msg[1] = 0; }
      if (local_fits)
        for (long long i = tid; i < n; i += 1024)
          comp[1 + i] = ((unsigned long long)((cand_key[i] - key_lo) & low_mask) << 45) | (kFlatMask - flat_index(fg, cand_tok[i], cand_col[i]));
      __syncthreads();
      if (!exchange_gather(ex, 2, msg, local_fits ? 2 + 2 * int(n) : 2, &timeout)) {
        if (tid == 0) atomicCAS(status, STATUS_OK, STATUS_WAIT_TIMEOUT);
        return;
      }
      if (tid == 0) {
        long long tot = 0;
        bool ok = true;
        for (int q = 0; q < world; ++q) {
          const uint32_t c = exchange_slot(ex, 2, q)[0];
          if (c == 0xFFFFFFFFu) ok = false; else tot += c;
        }
        fits_s = (ok && tot <= kGatherCap) ? 1 : 0;
        total_s = int(tot < kGatherCap ? tot : kGatherCap);
      }
      __syncthreads();
      if (fits_s) {
        int base = 0;
        for (int q = 0; q < world; ++q) {
          const uint32_t* slot = exchange_slot(ex, 2, q);
          const int c = int(slot[0]);
          const unsigned long long* src = reinterpret_cast<const unsigned long long*>(slot) + 1;
          for (int i = tid; i < c; i += 1024) comp[base + i] = src[i];
          base += c;
        }
      }
    }
    __syncthreads();
    if (fits_s) {
      const int G = total_s;
      const unsigned long long want = need;  // the want-th largest word is the cut
      // bitonic sort of the words in shared memory, descending (the words are distinct; zero pads the power of two)
      int P = 1;
      while (P < G) P <<= 1;
      for (int i = G + tid; i < P; i += 1024) comp[i] = 0ULL;
      __syncthreads();
      for (int size = 2; size <= P; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
          for (int t = tid; t < P / 2; t += 1024) {
            const int lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
            const unsigned long long a = comp[lo], b = comp[hi];
            const bool descending = (lo & size) == 0;
            if (descending ? a < b : a > b) { comp[lo] = b; comp[hi] = a; }
          }
          __syncthreads();
        }
      }
      if (tid == 0) {
        if (want == 0 || want > (unsigned long long)G) {
          atomicCAS(status, STATUS_OK, STATUS_SELECT_RANGE);
        } else {
          const unsigned long long cutw = comp[want - 1];
          ctl[CTL_CUT_KEY] = (long long)(cutw >> 45);
          ctl[CTL_TIE_MODE] = 1;
          ctl[CTL_CUT_FLAT] = (long long)(kFlatMask - (cutw & kFlatMask));
        }
      }
      return;
    }
  }
  // ---- key cut: radix passes over the low `shift` bits, 9 bits at a time, most significant first.
  uint32_t prefix = 0, prefix_mask = 0;
  int round = 3;  // rounds 0 and 1 belong to the two histogram passes, round 2 to the candidate gather

  for (int hi = shift; hi > 0; hi -= 9, ++round) {
    const int lo = max(hi - 9, 0);
    const int nb = 1 << (hi - lo);
    for (int i = tid; i < kRefineBins; i += 1024) hist[i] = 0;
    __syncthreads();
    for (long long i = tid; i < n; i += 1024) {
      const uint32_t k = (cand_key[i] - key_lo) & low_mask;
      if ((k & prefix_mask) == prefix) atomicAdd(&hist[(k >> lo) & (nb - 1)], 1u);
    }
    __syncthreads();
    if (!exchange_sum(ex, round, hist, kRefineBins, &timeout)) {
      if (tid == 0) atomicCAS(status, STATUS_OK, STATUS_WAIT_TIMEOUT);
      return;
    }
    unsigned long long cur = need;
    __syncthreads();
    pick_digit(hist, nb, true, cur, &digit, &need);
    prefix |= uint32_t(digit) << lo;
    prefix_mask |= uint32_t(nb - 1) << lo;
    __syncthreads();
  }
  // All candidates share the bits above `shift`; recover them from the bin.  `prefix` now holds the low
  // bits of the cut key T and `need` how many keys equal to T must be kept.
  // ---- ties: count keys == T (global), then cut by flat index if only part of them is kept.
  for (int i = tid; i < kRefineBins; i += 1024) hist[i] = 0;
  __syncthreads();
  unsigned int local_ties = 0;
  for (long long i = tid; i < n; i += 1024) local_ties += (((cand_key[i] - key_lo) & low_mask) == prefix) ? 1u : 0u;
  if (local_ties) atomicAdd(&hist[0], local_ties);
  __syncthreads();
  if (!exchange_sum(ex, round++, hist, kRefineBins, &timeout)) {
    if (tid == 0) atomicCAS(status, STATUS_OK, STATUS_WAIT_TIMEOUT);
    return;
  }
  const unsigned long long ties = hist[0];
  __syncthreads();
  unsigned long long flat_prefix = 0, flat_mask = 0;
  const bool partial = need < ties;
  if (partial) {
    // the `need` smallest flat indices among the ties: radix passes over 45 bits, 9 at a time
    for (int hi = 45; hi > 0; hi -= 9, ++round) {
      const int lo = hi - 9;
      for (int i = tid; i < kRefineBins; i += 1024) hist[i] = 0;
      __syncthreads();
      for (long long i = tid; i < n; i += 1024) {
        if (((cand_key[i] - key_lo) & low_mask) != prefix) continue;
        const unsigned long long fl = flat_index(fg, cand_tok[i], cand_col[i]);
        if ((fl & flat_mask) == flat_prefix) atomicAdd(&hist[(fl >> lo) & 511ULL], 1u);
      }
      __syncthreads();
      if (!exchange_sum(ex, round, hist, kRefineBins, &timeout)) {
        if (tid == 0) atomicCAS(status, STATUS_OK, STATUS_WAIT_TIMEOUT);
        return;
      }
      unsigned long long cur = need;
      __syncthreads();
      pick_digit(hist, 512, false, cur, &digit, &need);
      flat_prefix |= (unsigned long long)digit << lo;
      flat_mask |= 511ULL << lo;
      __syncthreads();
    }
  }
  if (tid == 0) {
    ctl[CTL_CUT_KEY] = (long long)prefix;  // low bits; compared under low_mask
    ctl[CTL_TIE_MODE] = partial ? 1 : 0;
    ctl[CTL_CUT_FLAT] = (long long)flat_prefix;
  }
}

// ------------------------------------------------------------------ 6. append the kept candidates
__global__ void __launch_bounds__(256) finalize_kernel(Lists o, FlatGeom fg, long long* __restrict__ ctl,
                                                         int* __restrict__ status) {
  const int shift = int(ctl[CTL_SHIFT]);
  const uint32_t key_lo = uint32_t(ctl[CTL_KEY_LO]);
  long long n = ctl[CTL_NUM_CAND];
  if (n > o.cand_cap) n = o.cand_cap;
  const uint32_t low_mask = shift >= 32 ? 0xFFFFFFFFu : ((1u << shift) - 1u);
  const uint32_t cut = uint32_t(ctl[CTL_CUT_KEY]);
  const bool tie_cut = ctl[CTL_TIE_MODE] != 0;
  const unsigned long long cut_flat = (unsigned long long)ctl[CTL_CUT_FLAT];
  unsigned long long* n_ent = reinterpret_cast<unsigned long long*>(ctl + CTL_NUM_ENTRIES);
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < n; i += 1LL * gridDim.x * blockDim.x) {
    const uint32_t k = (o.cand_key[i] - key_lo) & low_mask;
    bool keep = k > cut;
    if (k == cut) keep = !tie_cut || flat_index(fg, o.cand_tok[i], o.cand_col[i]) <= cut_flat;
    if (keep) {
      const unsigned long long p = atomicAdd(n_ent, 1ULL);
      if ((long long)p < o.ent_cap) {
        o.ent_tok[p] = o.cand_tok[i]; o.ent_col[p] = o.cand_col[i]; o.ent_val[p] = o.cand_val[i];
      } else {
        atomicCAS(status, STATUS_OK, STATUS_CAPACITY);
      }
    }
  }
}

// ------------------------------------------------------------------ 7. CSR views
__global__ void __launch_bounds__(256) csr_count_kernel(const int* __restrict__ ent_tok, const int* __restrict__ ent_col,
                                                          const float* __restrict__ ent_val, long long cap,
                                                          const long long* __restrict__ ctl, int* __restrict__ tok_cnt,
                                                          int* __restrict__ feat_cnt, unsigned char* __restrict__ fired,
                                                          int num_tokens, int num_cols) {
  long long n = ctl[CTL_NUM_ENTRIES];
  if (n > cap) n = cap;
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < n; i += 1LL * gridDim.x * blockDim.x) {
    const int t = ent_tok[i];
    const int c = ent_col[i];
    // an entry outside the problem (a stale count, a wrong pitch on the caller's side) is left out of both views
    // instead of being counted into a neighbouring region
    if (t < 0 || t >= num_tokens || c < 0 || c >= num_cols) continue;
    atomicAdd(&tok_cnt[t], 1);
    atomicAdd(&feat_cnt[c], 1);
    if (fired != nullptr && ent_val[i] > 1e-6f) fired[c] = 1;  // c was range-checked above
  }
}

// Exclusive scan of `n` ints by one CTA (1024 threads) over coalesced tiles of 4096 elements; out has n+1
// entries.  cursor (optional) gets a copy of the offsets for the scatter pass.
__global__ void __launch_bounds__(1024) exclusive_scan_kernel(const int* __restrict__ in, int* __restrict__ out,
                                                                int* __restrict__ cursor, int n) {
  __shared__ int warp_tot[32];
  __shared__ int carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < n; base += 4096) {
    const int i0 = base + tid * 4;
    int v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = (i0 + k < n) ? in[i0 + k] : 0;
    const int mine = v[0] + v[1] + v[2] + v[3];
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = warp_tot[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xFFFFFFFFu, w, o);
        if (lane >= o) w += t;
      }
      warp_tot[lane] = w;  // inclusive over warps
    }
    __syncthreads();
    const int carry = carry_s;
    int run = carry + (warp > 0 ? warp_tot[warp - 1] : 0) + incl - mine;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      if (i0 + k < n) {
        out[i0 + k] = run;
        if (cursor != nullptr) cursor[i0 + k] = run;
      }
      run += v[k];
    }
    __syncthreads();
    if (tid == 1023) carry_s = carry + warp_tot[31];
    __syncthreads();
  }
  if (tid == 0) out[n] = carry_s;
}

// Multi-CTA variant without scratch memory: CTA t owns elements [4096 t, 4096 (t + 1)).  It first adds up
// everything in front of its tile (the counts are small and stay in L2, so the repeated reads are cheaper
// than a second launch or a look-back protocol), then scans its own tile.
__global__ void __launch_bounds__(1024) exclusive_scan_tiles_kernel(const int* __restrict__ in, int* __restrict__ out,
                                                                      int* __restrict__ cursor, int n) {
  __shared__ int warp_tot[32];
  __shared__ int carry_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int base = blockIdx.x * 4096;
  int front = 0;
  {
    const int4* in4 = reinterpret_cast<const int4*>(in);  // base is a multiple of 4
    for (int i = tid; i < base / 4; i += 1024) {
      const int4 q = __ldg(in4 + i);
      front += q.x + q.y + q.z + q.w;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) front += __shfl_xor_sync(0xFFFFFFFFu, front, o);
    if (lane == 0) warp_tot[warp] = front;
    __syncthreads();
    if (tid == 0) {
      int c = 0;
      for (int w = 0; w < 32; ++w) c += warp_tot[w];
      carry_s = c;
    }
    __syncthreads();
  }
  const int carry = carry_s;
  __syncthreads();
  const int i0 = base + tid * 4;
  int v[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) v[k] = (i0 + k < n) ? in[i0 + k] : 0;
  const int mine = v[0] + v[1] + v[2] + v[3];
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_tot[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xFFFFFFFFu, w, o);
      if (lane >= o) w += t;
    }
    warp_tot[lane] = w;
  }
  __syncthreads();
  int run = carry + (warp > 0 ? warp_tot[warp - 1] : 0) + incl - mine;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if (i0 + k < n) {
      out[i0 + k] = run;
      if (cursor != nullptr) cursor[i0 + k] = run;
    }
    run += v[k];
  }
  if (blockIdx.x == gridDim.x - 1 && tid == 1023) out[n] = carry + warp_tot[31];
}

static void launch_exclusive_scan(const int* in, int* out, int* cursor, int n, cudaStream_t st) {
  const int ntiles = (n + 4095) / 4096;
  const bool aligned = (reinterpret_cast<uintptr_t>(in) & 15) == 0;
  if (ntiles >= 2 && ntiles <= 512 && aligned) exclusive_scan_tiles_kernel<<<ntiles, 1024, 0, st>>>(in, out, cursor, n);
  else exclusive_scan_kernel<<<1, 1024, 0, st>>>(in, out, cursor, n);
}

__global__ void __launch_bounds__(256) csr_scatter_kernel(const int* __restrict__ ent_tok, const int* __restrict__ ent_col,
                                                            const float* __restrict__ ent_val, long long cap,
                                                            const long long* __restrict__ ctl, int* __restrict__ tok_cursor,
                                                            int* __restrict__ feat_cursor, int* __restrict__ tcsr_col,
                                                            float* __restrict__ tcsr_val, int* __restrict__ fcsr_tok,
                                                            float* __restrict__ fcsr_val, int col_pitch, int num_tokens, int num_cols) {
  long long n = ctl[CTL_NUM_ENTRIES];
  if (n > cap) n = cap;
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < n; i += 1LL * gridDim.x * blockDim.x) {
    const int t = ent_tok[i], c = ent_col[i];
    if (t < 0 || t >= num_tokens || c < 0 || c >= num_cols) continue;  // the same entries that the count pass left out
    const float v = ent_val[i];
    const int p = atomicAdd(&tok_cursor[t], 1);
    const int layer = c / col_pitch;  // token-major view stores (layer << 24) | feature for the decoder
    if (p >= 0 && p < cap) { tcsr_col[p] = (layer << 24) | (c - layer * col_pitch); tcsr_val[p] = v; }
    const int q = atomicAdd(&feat_cursor[c], 1);
    if (q >= 0 && q < cap) { fcsr_tok[q] = t; fcsr_val[q] = v; }
  }
}

// Sort every CSR segment by its integer key (segments are short: insertion sort by one thread), so the
// order of the entries - and with it every floating-point sum over a segment - is reproducible.
constexpr int kShortSegment = 32;  // longer segments are sorted by a whole CTA (csr_sort_long_segments_kernel)

__global__ void __launch_bounds__(256) csr_sort_segments_kernel(const int* __restrict__ off, int nseg, int* __restrict__ key,
                                                                  float* __restrict__ val) {
  for (int sidx = blockIdx.x * blockDim.x + threadIdx.x; sidx < nseg; sidx += gridDim.x * blockDim.x) {
    const int b = off[sidx], e = off[sidx + 1];
    if (e - b > kShortSegment) continue;
    for (int i = b + 1; i < e; ++i) {
      const int k = key[i];
      const float v = val[i];
      int j = i - 1;
      while (j >= b && key[j] > k) { key[j + 1] = key[j]; val[j + 1] = val[j]; --j; }
      key[j + 1] = k; val[j + 1] = v;
    }
  }
}

// Long segments (a feature that fires on most tokens of the batch, a token with a thousand active features): an insertion
// sort by one thread would take O(n^2) dependent global-memory moves.  Here a CTA walks the segments, skips the short
// ones and sorts a long one cooperatively with a bitonic network in place (keys inside a segment are distinct, so no
// stability is needed); out-of-range partners of the virtual power-of-two padding are skipped.
__global__ void __launch_bounds__(256) csr_sort_long_segments_kernel(const int* __restrict__ off, int nseg, int* __restrict__ key,
                                                                       float* __restrict__ val) {
  __shared__ int long_list[256];
  __shared__ int long_count;
  // every thread looks at one segment of a block of 256; the few long ones are then sorted one after the other by the CTA
  for (int base = blockIdx.x * 256; base < nseg; base += gridDim.x * 256) {
    if (threadIdx.x == 0) long_count = 0;
    __syncthreads();
    const int mine = base + threadIdx.x;
    if (mine < nseg && off[mine + 1] - off[mine] > kShortSegment) long_list[atomicAdd(&long_count, 1)] = mine;
    __syncthreads();
    const int nlong = long_count;
    for (int q = 0; q < nlong; ++q) {
      const int sidx = long_list[q];
      const int b = off[sidx], n = off[sidx + 1] - b;
      int* k = key + b;
      float* v = val + b;
      int p2 = 1;
      while (p2 < n) p2 <<= 1;
      // every comparator puts the smaller key at the lower index (the first step of a merge pairs mirrored positions), so
      // the virtual padding, which stands for +infinity at the end of the array, never has to move
      for (int size = 2; size <= p2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
          __syncthreads();
          for (int i = threadIdx.x; i < p2 / 2; i += blockDim.x) {
            int lo, hi;
            if (stride == (size >> 1)) {
              const int blk = i / stride, j = i - blk * stride;
              lo = blk * size + j;
              hi = blk * size + size - 1 - j;
            } else {
              lo = 2 * i - (i & (stride - 1));
              hi = lo + stride;
            }
            if (hi >= n) continue;
            const int ka = k[lo], kb = k[hi];
            if (ka > kb) {
              k[lo] = kb; k[hi] = ka;
              const float t = v[lo]; v[lo] = v[hi]; v[hi] = t;
            }
          }
        }
      }
      __syncthreads();
    }
    __syncthreads();
  }
}

// Dead-feature counters: +1 per step, reset where the feature fired (reference trainer.py:693-712).
__global__ void __launch_bounds__(256) dead_counter_kernel(long long* __restrict__ counter, unsigned char* __restrict__ fired, int n) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    counter[i] = fired[i] ? 0 : counter[i] + 1;
    fired[i] = 0;
  }
}

}  // namespace clt

// ====================================================================== C launchers
using namespace clt;

extern "C" int CLT_FN(clt_colstats)(const void* x, float* mean, float* rstd, int L, int B, int F, long long ld, long long layer_stride,
                            cudaStream_t st) {
  if (F % 8 != 0 || ld % 8 != 0 || layer_stride % 8 != 0) return -1;
  const int col_blocks = (F / 8 + 31) / 32;
  int zsplit = 1;
  while (1LL * col_blocks * L * zsplit < 592 && zsplit < 16 && B / (zsplit * 2) >= 128) zsplit *= 2;
  dim3 grid(col_blocks, L, zsplit), block(32, 8);
  const t16* xp = static_cast<const t16*>(x);
  if (zsplit > 1) {
    if (cudaMemsetAsync(mean, 0, sizeof(float) * size_t(L) * F, st) != cudaSuccess) return -5;
    if (cudaMemsetAsync(rstd, 0, sizeof(float) * size_t(L) * F, st) != cudaSuccess) return -5;
  }
  colstats_kernel<<<grid, block, 0, st>>>(xp, mean, rstd, B, F, ld, layer_stride);
  if (zsplit > 1) {
    const long long n = 1LL * L * F;
    colstats_finalize_kernel<<<int((n + 255) / 256), 256, 0, st>>>(xp, mean, rstd, B, F, layer_stride, n);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

#if !CLT_T16_IS_HALF
extern "C" int clt_colstats_from_tiles(const float* tile_stats, float* mean, float* rstd, int L, int B, int F, cudaStream_t st) {
  const long long n = 1LL * L * F;
  if (n == 0) return 0;
  colstats_from_tiles_kernel<<<int((n + 255) / 256), 256, 0, st>>>(tile_stats, mean, rstd, B, F, (B + 127) / 128, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

#endif

struct CltExchangeArgs {
  int world;
  int rank;
  void* data[8];
  void* flags[8];
  int slot_elems;
  unsigned int seq;
};

static Exchange to_exchange(const CltExchangeArgs* a) {
  Exchange ex;
  ex.world = a ? a->world : 1;
  ex.rank = a ? a->rank : 0;
  ex.slot_elems = a ? a->slot_elems : 0;
  ex.seq = a ? a->seq : 0;
  for (int i = 0; i < kMaxPeers; ++i) {
    ex.peers[i] = a ? static_cast<uint32_t*>(a->data[i]) : nullptr;
    ex.flags[i] = a ? static_cast<uint32_t*>(a->flags[i]) : nullptr;
  }
  return ex;
}

struct CltSelectArgs {
  const void* x;  // [L, B, ld] bf16 pre-activations
  const float* mean;
  const float* rstd;
  int L, B, F;  // F: valid local features per layer
  int stat_pitch;  // row pitch of mean / rstd
  long long ld, layer_stride;
  int col_pitch;       // pitch used to encode columns (l * col_pitch + f)
  int feat_offset;     // first global feature of the shard
  long long full_F;    // un-sharded feature count
  long long k_total;   // global number of entries to keep
  unsigned int key_lo; // histogram covers keys >= key_lo
  int shift;           // bin = (key - key_lo) >> shift
  unsigned int* hist;  // [2 * 8192 + 32], zeroed by the caller
  long long* ctl;      // [CTL_SIZE]
  int* ent_tok; int* ent_col; float* ent_val; long long ent_cap;
  unsigned int* cand_key; int* cand_tok; int* cand_col; float* cand_val; long long cand_cap;
  int* status;
  // Optional tracked range: sel_state = {key_lo, shift} in device memory, moved by the kernels every step,
  // and the pool that the single pass over the matrix fills.  Null sel_state: fixed range from key_lo / shift.
  long long* sel_state;
  unsigned int* pool_key; int* pool_tok; int* pool_col; float* pool_val; long long pool_cap;
};

static ScanGeom scan_geom(const CltSelectArgs* a) {
  ScanGeom g;
  g.B = a->B; g.F = a->F; g.L = a->L; g.sp = a->stat_pitch; g.ld = a->ld; g.layer_stride = a->layer_stride;
  g.rows_per_block = 64;
  return g;
}
static Lists lists_of(const CltSelectArgs* a) {
  Lists o;
  o.ent_tok = a->ent_tok; o.ent_col = a->ent_col; o.ent_val = a->ent_val; o.ent_cap = a->ent_cap;
  o.cand_key = a->cand_key; o.cand_tok = a->cand_tok; o.cand_col = a->cand_col; o.cand_val = a->cand_val; o.cand_cap = a->cand_cap;
  return o;
}
static FlatGeom flat_geom(const CltSelectArgs* a) {
  FlatGeom fg;
  fg.col_pitch = a->col_pitch; fg.feat_offset = a->feat_offset; fg.full_F = a->full_F; fg.row_width = a->full_F * a->L;
  return fg;
}

// Steps 2-6.  `exa` may be null (single rank).  The histogram first covers keys >= key_lo only (the
// caller's guess of where the cut lies); if the cut is not inside, a full-range pass repeats it.
// `hist` holds two histograms of 8192 counters, zeroed by the caller.
extern "C" int CLT_FN(clt_batchtopk_select)(const CltSelectArgs* a, const CltExchangeArgs* exa, cudaStream_t st) {
  if (a->ld % 8 != 0 || a->layer_stride % 8 != 0 || a->stat_pitch % 4 != 0 || a->F > a->ld) return -1;
  const ScanGeom g = scan_geom(a);
  const Exchange ex = to_exchange(exa);
  dim3 grid(((a->F + 7) / 8 + 255) / 256, (a->B + g.rows_per_block - 1) / g.rows_per_block, a->L);
  const t16* x = static_cast<const t16*>(a->x);
  if (a->sel_state != nullptr && a->key_lo != 0) {
    Pool pool;
    pool.key = a->pool_key; pool.tok = a->pool_tok; pool.col = a->pool_col; pool.val = a->pool_val; pool.cap = a->pool_cap;
    pool.count = a->hist + 2 * kHistBins;
    zhist_collect_kernel<<<grid, 256, 0, st>>>(x, a->mean, a->rstd, g, a->col_pitch, a->sel_state, a->hist, pool);
    find_bin_kernel<<<1, 1024, 0, st>>>(a->hist, a->k_total, a->ctl, ex, 0u, 0, 0, 0, a->sel_state, pool.count, pool.cap, a->status);
    classify_pool_kernel<<<592, 256, 0, st>>>(pool, a->ctl, lists_of(a), a->status);
    // fallback, skipped inside the kernels unless the tracked range missed the cut or the pool overflowed
    zhist_kernel<<<grid, 256, 0, st>>>(x, a->mean, a->rstd, g, 0u, 19, a->hist + kHistBins, a->ctl, 1);
    find_bin_kernel<<<1, 1024, 0, st>>>(a->hist + kHistBins, a->k_total, a->ctl, ex, 0u, 19, 1, 1, a->sel_state, nullptr, 0, a->status);
    compact_kernel<<<grid, 256, 0, st>>>(x, a->mean, a->rstd, g, a->col_pitch, a->ctl, lists_of(a), a->status, 1);
  } else {
    zhist_kernel<<<grid, 256, 0, st>>>(x, a->mean, a->rstd, g, a->key_lo, a->shift, a->hist, a->ctl, 0);
    find_bin_kernel<<<1, 1024, 0, st>>>(a->hist, a->k_total, a->ctl, ex, a->key_lo, a->shift, 0, 0, nullptr, nullptr, 0, a->status);
    if (a->key_lo != 0) {
      zhist_kernel<<<grid, 256, 0, st>>>(x, a->mean, a->rstd, g, 0u, 19, a->hist + kHistBins, a->ctl, 1);
      find_bin_kernel<<<1, 1024, 0, st>>>(a->hist + kHistBins, a->k_total, a->ctl, ex, 0u, 19, 1, 1, nullptr, nullptr, 0, a->status);
    }
    compact_kernel<<<grid, 256, 0, st>>>(x, a->mean, a->rstd, g, a->col_pitch, a->ctl, lists_of(a), a->status, 0);
  }
  refine_kernel<<<1, 1024, 0, st>>>(a->cand_key, a->cand_tok, a->cand_col, a->cand_cap, flat_geom(a), a->ctl, ex, a->status);
  finalize_kernel<<<256, 256, 0, st>>>(lists_of(a), flat_geom(a), a->ctl, a->status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Per-feature threshold selection (JumpReLU / ReLU as a sparse list).  theta: [L, stat_pitch] fp32.  Uses of the
// argument block: x, rstd (= theta), L, B, F, stat_pitch, ld, layer_stride, col_pitch, ctl, ent_*, status.
extern "C" int CLT_FN(clt_threshold_select)(const CltSelectArgs* a, cudaStream_t st) {
  if (a->ld % 8 != 0 || a->layer_stride % 8 != 0 || a->F > a->ld) return -1;
  const ScanGeom g = scan_geom(a);
  dim3 grid(((a->F + 7) / 8 + 255) / 256, (a->B + g.rows_per_block - 1) / g.rows_per_block, a->L);
  if (cudaMemsetAsync(a->ctl + CTL_NUM_ENTRIES, 0, sizeof(long long), st) != cudaSuccess) return -5;
  threshold_collect_kernel<<<grid, 256, 0, st>>>(static_cast<const t16*>(a->x), a->rstd, g, a->col_pitch, a->ctl, lists_of(a), a->status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Per-token top-k of the batch z-scores (TokenTopK).  Uses x, mean, rstd, L, B, F, stat_pitch, ld, layer_stride,
// col_pitch, ctl, ent_* (capacity >= B * k), status of the argument block; k_total carries the per-token k and feat_offset
// (when positive) the number of valid columns per layer (the rest of F is shard padding).
extern "C" int CLT_FN(clt_token_topk_select)(const CltSelectArgs* a, cudaStream_t st) {
  if (a->ld % 8 != 0 || a->layer_stride % 8 != 0 || a->F % 8 != 0 || a->stat_pitch % 4 != 0 || a->F > a->ld) return -1;
  const long long k = a->k_total;
  const int f_valid = a->feat_offset > 0 && a->feat_offset <= a->F ? a->feat_offset : a->F;  // feat_offset carries the valid column count here
  if (k <= 0 || k > 1LL * a->L * f_valid || 1LL * a->B * k > a->ent_cap) return -1;
  const ScanGeom g = scan_geom(a);
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(token_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(TokenTopkShared))) != cudaSuccess) return -4;
    attr_set = true;
  }
  const int grid = (a->B + kTokPerCta - 1) / kTokPerCta;
  token_topk_kernel<<<grid, 256, sizeof(TokenTopkShared), st>>>(static_cast<const t16*>(a->x), a->mean, a->rstd, g, a->col_pitch,
                                                                 f_valid, int(k), a->ctl, lists_of(a), a->status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

#if !CLT_T16_IS_HALF
// ------------------------------------------------------------------ TokenTopK across feature shards
// Every rank holds a slice of the columns; a token keeps its k largest z-scores over all ranks' columns (reference:
// clt/models/activations.py:360-491, where the full pre-activations are gathered and the mask is broadcast).  Here each
// rank first takes the exact top k of its own columns (token_topk_kernel: a superset of what survives), then
//   1. token_topk_push:   composite keys (z key << 32 | inverted global flat index) of the local candidates go to the
//                         owner of the token (tokens are dealt to the ranks in blocks of rows_per_rank) by peer stores;
//   2. token_topk_cut:    the owner ranks the W * k keys of each of its tokens, takes the k-th largest as the cut and stores
//                         it into every rank's cut array;
//   3. token_topk_filter: every rank keeps its candidates at or above the cut and appends them to its entry list.
// The composite keys are distinct and their order does not depend on the number of ranks (larger z first, lower flat index
// first among equal z), so the selection equals the single-GPU one entry for entry.  Phase barriers (peer_barrier) separate
// the three kernels; nothing here waits.
struct CltTopkTpArgs {
  const int* cand_col; const float* cand_val;   // [B * k] local candidates (token t at t * k ...), from token_topk_select
  unsigned long long* cand_key;                 // [B * k] composite keys (written by push, read by filter)
  const float* mean; const float* rstd; int stat_pitch;
  int col_pitch, feat_offset; long long full_F;
  int B, k, world, rank, rows_per_rank;
  void* stage[8];                               // every rank's key staging [world][rows_per_rank][k] u64
  void* cut[8];                                 // every rank's cut array [B] u64
  long long* ctl;
  int* ent_tok; int* ent_col; float* ent_val; long long ent_cap;
  int* status;
};

__global__ void __launch_bounds__(256) token_topk_push_kernel(CltTopkTpArgs a) {
  if (blockIdx.x == 0 && threadIdx.x == 0) a.ctl[CTL_NUM_ENTRIES] = 0;  // refilled by the filter pass
  const long long n = 1LL * a.B * a.k;
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < n; i += 1LL * gridDim.x * blockDim.x) {
    const int t = int(i / a.k), j = int(i - 1LL * t * a.k);
    const int col = a.cand_col[i];
    const int l = col / a.col_pitch, c = col - l * a.col_pitch;
    const float z = (a.cand_val[i] - a.mean[1LL * l * a.stat_pitch + c]) * a.rstd[1LL * l * a.stat_pitch + c];
    const unsigned long long flat = (unsigned long long)l * (unsigned long long)a.full_F + (unsigned long long)(a.feat_offset + c);
    const unsigned long long key = ((unsigned long long)float_to_key(z) << 32) | (0xFFFFFFFFULL - flat);
    a.cand_key[i] = key;
    const int owner = t / a.rows_per_rank, lt = t - owner * a.rows_per_rank;
    static_cast<unsigned long long*>(a.stage[owner])[(1LL * a.rank * a.rows_per_rank + lt) * a.k + j] = key;
  }
}

// One CTA per owned token; dynamic shared memory world * k keys.
__global__ void __launch_bounds__(256) token_topk_cut_kernel(CltTopkTpArgs a) {
  extern __shared__ unsigned long long tk_keys[];
  const int lt = blockIdx.x;
  const int t = a.rank * a.rows_per_rank + lt;
  if (t >= a.B) return;
  const int n = a.world * a.k;
  const unsigned long long* mine = static_cast<const unsigned long long*>(a.stage[a.rank]);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int w = i / a.k, j = i - w * a.k;
    tk_keys[i] = mine[(1LL * w * a.rows_per_rank + lt) * a.k + j];
  }
  __syncthreads();
  // the key that exactly k - 1 keys exceed (the keys are distinct)
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const unsigned long long ki = tk_keys[i];
    int above = 0;
    for (int j = 0; j < n; ++j) above += tk_keys[j] > ki;
    if (above == a.k - 1) {
      for (int w = 0; w < a.world; ++w) static_cast<unsigned long long*>(a.cut[w])[t] = ki;
    }
  }
}

// One warp per token: candidates at or above the cut are appended to the entry list.
__global__ void __launch_bounds__(256) token_topk_filter_kernel(CltTopkTpArgs a) {
  const int lane = threadIdx.x & 31;
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (t >= a.B) return;
  const unsigned long long cut = static_cast<const unsigned long long*>(a.cut[a.rank])[t];
  unsigned long long* n_ent = reinterpret_cast<unsigned long long*>(a.ctl + CTL_NUM_ENTRIES);
  for (int j0 = 0; j0 < a.k; j0 += 32) {
    const int j = j0 + lane;
    const long long i = 1LL * t * a.k + j;
    const bool keep = j < a.k && a.cand_key[i] >= cut;
    const unsigned ball = __ballot_sync(0xFFFFFFFFu, keep);
    if (ball == 0u) continue;
    unsigned long long base = 0;
    if (lane == 0) base = atomicAdd(n_ent, (unsigned long long)__popc(ball));
    base = __shfl_sync(0xFFFFFFFFu, base, 0);
    if (keep) {
      const long long q = (long long)base + __popc(ball & ((1u << lane) - 1u));
      if (q < a.ent_cap) { a.ent_tok[q] = t; a.ent_col[q] = a.cand_col[i]; a.ent_val[q] = a.cand_val[i]; }
      else atomicCAS(a.status, STATUS_OK, STATUS_CAPACITY);
    }
  }
}

// phase: 0 push, 1 cut, 2 filter (the caller puts a phase barrier between them)
extern "C" int clt_token_topk_tp(const CltTopkTpArgs* a, int phase, cudaStream_t st) {
  if (a->world < 1 || a->world > 8 || a->k <= 0 || a->B <= 0 || a->rows_per_rank <= 0) return -1;
  if (1LL * a->world * a->rows_per_rank < a->B) return -1;
  const size_t smem = sizeof(unsigned long long) * size_t(a->world) * size_t(a->k);
  if (smem > 200 * 1024) return -2;
  if (phase == 0) {
    const long long n = 1LL * a->B * a->k;
    const int grid = int((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    token_topk_push_kernel<<<grid, 256, 0, st>>>(*a);
  } else if (phase == 1) {
    static size_t attr_smem = 0;
    if (smem > 48 * 1024 && smem > attr_smem) {
      if (cudaFuncSetAttribute(token_topk_cut_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return -4;
      attr_smem = smem;
    }
    token_topk_cut_kernel<<<a->rows_per_rank, 256, smem, st>>>(*a);
  } else {
    token_topk_filter_kernel<<<(a->B + 7) / 8, 256, 0, st>>>(*a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

struct CltCsrArgs {
  const int* ent_tok; const int* ent_col; const float* ent_val; long long ent_cap;
  const long long* ctl;
  int num_tokens; int num_cols;
  int* tok_cnt; int* feat_cnt;        // zeroed by the caller
  int* tok_off; int* feat_off;        // [num_tokens+1], [num_cols+1]
  int* tok_cursor; int* feat_cursor;  // scratch
  int* tcsr_col; float* tcsr_val; int* fcsr_tok; float* fcsr_val;
  unsigned char* fired;               // optional [num_cols]
  int sort_segments;                  // bit 0: token segments, bit 1: feature segments
  int col_pitch;                      // columns are layer * col_pitch + feature (feature < 2^24)
};

extern "C" int clt_build_csr(const CltCsrArgs* a, cudaStream_t st) {
  const int blocks = 592;
  csr_count_kernel<<<blocks, 256, 0, st>>>(a->ent_tok, a->ent_col, a->ent_val, a->ent_cap, a->ctl, a->tok_cnt, a->feat_cnt, a->fired,
                                           a->num_tokens, a->num_cols);
  launch_exclusive_scan(a->tok_cnt, a->tok_off, a->tok_cursor, a->num_tokens, st);
  launch_exclusive_scan(a->feat_cnt, a->feat_off, a->feat_cursor, a->num_cols, st);
  csr_scatter_kernel<<<blocks, 256, 0, st>>>(a->ent_tok, a->ent_col, a->ent_val, a->ent_cap, a->ctl, a->tok_cursor, a->feat_cursor,
                                             a->tcsr_col, a->tcsr_val, a->fcsr_tok, a->fcsr_val, a->col_pitch, a->num_tokens, a->num_cols);
  if (a->sort_segments & 1) {
    csr_sort_segments_kernel<<<(a->num_tokens + 255) / 256, 256, 0, st>>>(a->tok_off, a->num_tokens, a->tcsr_col, a->tcsr_val);
    csr_sort_long_segments_kernel<<<(a->num_tokens + 255) / 256 < 1184 ? (a->num_tokens + 255) / 256 : 1184, 256, 0, st>>>(a->tok_off, a->num_tokens, a->tcsr_col, a->tcsr_val);
  }
  if (a->sort_segments & 2) {
    csr_sort_segments_kernel<<<(a->num_cols + 255) / 256, 256, 0, st>>>(a->feat_off, a->num_cols, a->fcsr_tok, a->fcsr_val);
    csr_sort_long_segments_kernel<<<(a->num_cols + 255) / 256 < 1184 ? (a->num_cols + 255) / 256 : 1184, 256, 0, st>>>(a->feat_off, a->num_cols, a->fcsr_tok, a->fcsr_val);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int clt_dead_counter_update(long long* counter, unsigned char* fired, int n, cudaStream_t st) {
  dead_counter_kernel<<<(n + 255) / 256, 256, 0, st>>>(counter, fired, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// ====================================================================== allocation-free CSR build
#include <cstdio>
#include <mutex>

#include "csr_static.h"

// Scratch of clt_build_csr_static: [tok_cnt | feat_cnt | tok_cursor | feat_cursor], each region sized for the
// maximum problem.  One copy per GPU that loads this library; host code must not pass this name to a kernel
// (on the host it is only a stand-in) - the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) int csr_static_scratch[2 * (CLT_CSR_STATIC_MAX_TOKENS + CLT_CSR_STATIC_MAX_COLS)];

namespace {
constexpr int kMaxDevicesStatic = 64;
int* g_static_scratch_ptr[kMaxDevicesStatic] = {nullptr};
std::mutex g_static_scratch_mu;

// Device address of the scratch array on the current device; looked up once per device.
int* csr_static_scratch_address() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevicesStatic) return nullptr;
  std::lock_guard<std::mutex> lock(g_static_scratch_mu);
  if (g_static_scratch_ptr[dev] == nullptr) {
    int* p = nullptr;
    const cudaError_t rc = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), csr_static_scratch);
    if (rc != cudaSuccess || p == nullptr) {
      fprintf(stderr, "clt_build_csr_static: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(rc));
      return nullptr;
    }
    g_static_scratch_ptr[dev] = p;
  }
  return g_static_scratch_ptr[dev];
}
}  // namespace

extern "C" int clt_build_csr_static(const int* ent_tok, const int* ent_col, const float* ent_val, long long ent_cap,
                                    const long long* ctl, int num_tokens, int num_cols, int col_pitch, int* tok_off, int* feat_off,
                                    int* tcsr_col, float* tcsr_val, int* fcsr_tok, float* fcsr_val, int sort_segments,
                                    cudaStream_t stream) {
  if (!ent_tok || !ent_col || !ent_val || !ctl || !tok_off || !feat_off || !tcsr_col || !tcsr_val || !fcsr_tok || !fcsr_val ||
      ent_cap <= 0 || num_tokens <= 0 || num_cols <= 0 || col_pitch <= 0 || col_pitch >= (1 << 24)) {
    fprintf(stderr, "clt_build_csr_static: bad argument (null pointer, non-positive size or col_pitch outside (0, 2^24))\n");
    return -1;
  }
  if (num_tokens > CLT_CSR_STATIC_MAX_TOKENS || num_cols > CLT_CSR_STATIC_MAX_COLS) {
    fprintf(stderr, "clt_build_csr_static: num_tokens=%d / num_cols=%d exceed the built-in scratch (max %d tokens, %d columns); "
                    "use clt_build_csr with caller-provided scratch\n",
            num_tokens, num_cols, CLT_CSR_STATIC_MAX_TOKENS, CLT_CSR_STATIC_MAX_COLS);
    return -2;
  }
  int* scratch = csr_static_scratch_address();
  if (scratch == nullptr) return -3;
  int* tok_cnt = scratch;
  int* feat_cnt = tok_cnt + CLT_CSR_STATIC_MAX_TOKENS;
  int* tok_cursor = feat_cnt + CLT_CSR_STATIC_MAX_COLS;
  int* feat_cursor = tok_cursor + CLT_CSR_STATIC_MAX_TOKENS;
  // the array still holds the previous call's counters: clear the parts that must start at zero
  if (cudaMemsetAsync(tok_cnt, 0, sizeof(int) * size_t(num_tokens), stream) != cudaSuccess) return -5;
  if (cudaMemsetAsync(feat_cnt, 0, sizeof(int) * size_t(num_cols), stream) != cudaSuccess) return -5;
  const int blocks = 592;
  csr_count_kernel<<<blocks, 256, 0, stream>>>(ent_tok, ent_col, ent_val, ent_cap, ctl, tok_cnt, feat_cnt, nullptr, num_tokens, num_cols);
  exclusive_scan_kernel<<<1, 1024, 0, stream>>>(tok_cnt, tok_off, tok_cursor, num_tokens);
  exclusive_scan_kernel<<<1, 1024, 0, stream>>>(feat_cnt, feat_off, feat_cursor, num_cols);
  csr_scatter_kernel<<<blocks, 256, 0, stream>>>(ent_tok, ent_col, ent_val, ent_cap, ctl, tok_cursor, feat_cursor, tcsr_col, tcsr_val,
                                                 fcsr_tok, fcsr_val, col_pitch, num_tokens, num_cols);
  if (sort_segments & 1) {
    csr_sort_segments_kernel<<<(num_tokens + 255) / 256, 256, 0, stream>>>(tok_off, num_tokens, tcsr_col, tcsr_val);
    csr_sort_long_segments_kernel<<<num_tokens < 1184 ? num_tokens : 1184, 256, 0, stream>>>(tok_off, num_tokens, tcsr_col, tcsr_val);
  }
  if (sort_segments & 2) {
    csr_sort_segments_kernel<<<(num_cols + 255) / 256, 256, 0, stream>>>(feat_off, num_cols, fcsr_tok, fcsr_val);
    csr_sort_long_segments_kernel<<<num_cols < 1184 ? num_cols : 1184, 256, 0, stream>>>(feat_off, num_cols, fcsr_tok, fcsr_val);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
#endif  // !CLT_T16_IS_HALF
