// Auxiliary loss on dead features (AuxK), device side (sm_100a).
//
// Reference (clt/training/losses.py:263-329): per layer, the pre-activations of the dead features (those that have not
// fired for `dead_feature_window` steps) are ranked per token, the top k_aux = min(512, n_dead) of them are decoded to
// the same layer with the layer's own decoder rows and bias, and the result is matched to the residual of the main
// reconstruction.  The reference does this with a clone of the dense [B, F] pre-activations, torch.topk, scatter_ and a
// dense decoder GEMM per layer, after a host read of the dead count.
//
// Here the dead features of a layer are compacted into a short list (at most `nd_cap` per layer, chosen by the host from
// an occasional read of the counts), and the whole term becomes dense algebra on the compact set, [B, nd_cap] wide:
//
//   aux_compact        dead flags -> per-layer list of dead columns, counts, and the column -> compact-row index
//   aux_gather_rows    encoder rows of the dead features;  (grouped GEMM)  A = x W_dead^T
//   aux_gather_select  adds the encoder bias and keeps the token's top k_aux dead values of A, 0 elsewhere (exact radix
//                      selection on the 16-bit keys, ties by lowest feature index); it can also gather the values from the
//                      stored pre-activations instead
//   aux_gather_rows    W0[l][i, :] = same-layer decoder row of dead feature i
//   (grouped tensor-core GEMM, dense_gemm.cu)   recon = A W0
//   aux_residual       r = recon + bias - residual, loss, g = dL/d recon, and the term's gradient through the residual
//                      added to the gradient seed
//   (grouped GEMM)     G = g W0^T,  masked to the kept positions (straight-through) while it is transposed;
//                      dW0 = A^T g;  dW_enc = G^T x
//
// The gradients reach the optimizer kernels as compact extra rows (adam.cu: extra_idx / extra_rows).
#include "common.cuh"

namespace clt {

constexpr int kAuxMaxCap = 4096;  // compact dead features per layer that one CTA ranks in shared memory

// ------------------------------------------------------------------ compaction of the dead features
// One CTA (1024 threads) per layer.  dead_cols [L, nd_cap], nd [L] (clamped to nd_cap), nd_all [L] (unclamped),
// extra_idx [L * F_pitch] = l * nd_cap + i for dead column i of layer l, -1 for everything else.
__global__ void __launch_bounds__(1024) aux_compact_kernel(const long long* __restrict__ dead_counter, long long window, int F_pitch, int F_valid,
                                                            int nd_cap, int* __restrict__ dead_cols, int* __restrict__ nd, int* __restrict__ nd_all,
                                                            int* __restrict__ extra_idx) {
  __shared__ int warp_tot[32];
  __shared__ int carry_s;
  const int l = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < F_pitch; base += 1024) {
    const int f = base + tid;
    const bool dead = f < F_valid && dead_counter[1LL * l * F_pitch + f] > window;
    const unsigned ball = __ballot_sync(0xFFFFFFFFu, dead);
    const int before = __popc(ball & ((1u << lane) - 1u));
    if (lane == 0) warp_tot[warp] = __popc(ball);
    __syncthreads();
    if (warp == 0) {
      int w = warp_tot[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xFFFFFFFFu, w, o);
        if (lane >= o) w += t;
      }
      warp_tot[lane] = w;  // inclusive
    }
    __syncthreads();
    const int pos = carry_s + (warp > 0 ? warp_tot[warp - 1] : 0) + before;
    if (f < F_pitch) {
      int idx = -1;
      if (dead && pos < nd_cap) { dead_cols[1LL * l * nd_cap + pos] = f; idx = l * nd_cap + pos; }
      extra_idx[1LL * l * F_pitch + f] = idx;
    }
    __syncthreads();
    if (tid == 0) carry_s += warp_tot[31];
    __syncthreads();
  }
  if (tid == 0) { nd_all[l] = carry_s; nd[l] = min(carry_s, nd_cap); }
}

__device__ __forceinline__ uint32_t key16(uint32_t bits) { return (bits & 0x8000u) ? (~bits & 0xFFFFu) : (bits | 0x8000u); }

// ------------------------------------------------------------------ per-token selection
// Largest bin (from the top) at which the running count reaches `need`; executed by one warp on a 256-bin histogram.
// Returns the bin; *need_out = how many of that bin's values are still wanted.
__device__ __forceinline__ int warp_find_bin_from_top(const unsigned int* hist, int need, int lane, int* need_out) {
  // lane i owns bins [255 - 8 i - 7, 255 - 8 i] (lane 0 the top eight)
  const int hi = 255 - 8 * lane;
  int own = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) own += int(hist[hi - j]);
  int incl = own;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
    if (lane >= o) incl += t;
  }
  const unsigned reach = __ballot_sync(0xFFFFFFFFu, incl >= need);
  const int owner = reach != 0u ? __ffs(reach) - 1 : 31;
  int bin = 0, left = 0;
  if (lane == owner) {
    int run = incl - own;
    bin = hi - 7;
    left = need - run;
    for (int j = 0; j < 8; ++j) {
      const int c = int(hist[hi - j]);
      if (run + c >= need) { bin = hi - j; left = need - run; break; }
      run += c;
    }
  }
  bin = __shfl_sync(0xFFFFFFFFu, bin, owner);
  *need_out = __shfl_sync(0xFFFFFFFFu, left, owner);
  return bin;
}

// bias_c[l][i] = encoder bias of dead column i of layer l (0 beyond nd[l]): gathered once per step, so that the selection
// below reads it coalesced instead of chasing column index -> bias for every token.
__global__ void __launch_bounds__(256) aux_gather_bias_kernel(const void* __restrict__ enc_bias, int bias_is_16, int F_pitch,
                                                                const int* __restrict__ dead_cols, const int* __restrict__ nd, int nd_cap,
                                                                float* __restrict__ bias_c) {
  const int l = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nd_cap) return;
  float v = 0.f;
  if (i < nd[l]) {
    const long long bi = 1LL * l * F_pitch + __ldg(dead_cols + 1LL * l * nd_cap + i);
    v = bias_is_16 ? t16_to_float(static_cast<const t16*>(enc_bias)[bi]) : static_cast<const float*>(enc_bias)[bi];
  }
  bias_c[1LL * l * nd_cap + i] = v;
}

// One warp per (token, layer), eight of them per CTA, each with its own key array and histogram in shared memory (no CTA-wide
// barrier anywhere).  A [L, B, nd_cap] 16-bit: the token's dead pre-activations, the top k_aux of them
// (k_aux = min(k_aux_max, nd_all[l])) kept, the rest zero; columns >= nd[l] are zero.  Two sources:
//   enc_bias == nullptr: the values are gathered from the stored pre-activations `pre` [L, B, ld] at the dead columns;
//   bias_c != nullptr:   A already holds x W_dead^T (the encoder rows of the dead features, one GEMM for all layers); the
//                        compact encoder bias bias_c [L, nd_cap] is added here and A is rewritten in place.
// Dynamic shared memory: 8 * (nd_cap * 2 + 1024) bytes.
__global__ void __launch_bounds__(256) aux_gather_select_kernel(const t16* __restrict__ pre, long long ld, long long layer_stride,
                                                                  const float* __restrict__ bias_c,
                                                                  const int* __restrict__ dead_cols, const int* __restrict__ nd,
                                                                  const int* __restrict__ nd_all, int nd_cap, int k_aux_max, int B,
                                                                  t16* __restrict__ A) {
  extern __shared__ __align__(16) uint8_t aux_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tok = blockIdx.x * 8 + warp, l = blockIdx.y;
  if (tok >= B) return;  // whole warp
  unsigned short* keys = reinterpret_cast<unsigned short*>(aux_smem + size_t(warp) * (size_t(nd_cap) * 2 + 1024));
  unsigned int* hist = reinterpret_cast<unsigned int*>(reinterpret_cast<uint8_t*>(keys) + size_t(nd_cap) * 2);
  const int n = nd[l];
  const int k_aux = min(k_aux_max, nd_all[l]);
  t16* out = A + (1LL * l * B + tok) * nd_cap;
  unsigned short* obits = reinterpret_cast<unsigned short*>(out);
  const int* cols = dead_cols + 1LL * l * nd_cap;
  if (bias_c == nullptr) {
    const unsigned short* rbits = reinterpret_cast<const unsigned short*>(pre + 1LL * l * layer_stride + 1LL * tok * ld);
    for (int i = lane; i < nd_cap; i += 32) keys[i] = i < n ? rbits[__ldg(cols + i)] : (unsigned short)0;
  } else {
    // eight values per lane and step: one 16-byte load of the products, two of the bias
    const float* bl = bias_c + 1LL * l * nd_cap;
    for (int i8 = lane; i8 < nd_cap / 8; i8 += 32) {
      const int i = i8 * 8;
      uint4 q = make_uint4(0, 0, 0, 0);
      if (i < n) {
        const uint4 pv = *reinterpret_cast<const uint4*>(out + i);
        const float4 b0 = __ldg(reinterpret_cast<const float4*>(bl + i)), b1 = __ldg(reinterpret_cast<const float4*>(bl + i + 4));
        const uint32_t pu[4] = {pv.x, pv.y, pv.z, pv.w};
        const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        uint32_t r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // columns at or beyond n hold zero products and zero bias: they stay zero
          const float lo = i + 2 * j < n ? t16_lo(pu[j]) + bb[2 * j] : 0.f, hi = i + 2 * j + 1 < n ? t16_hi(pu[j]) + bb[2 * j + 1] : 0.f;
          r[j] = pack_t16x2(lo, hi);
        }
        q = make_uint4(r[0], r[1], r[2], r[3]);
      }
      *reinterpret_cast<uint4*>(keys + i) = q;
    }
  }
  __syncwarp();
  if (n > k_aux) {
    // exact k_aux-th largest of the n values: two radix rounds over the monotone 16-bit key
    uint32_t prefix = 0;
    int need = k_aux;
    for (int round = 0; round < 2; ++round) {
      const int shift = round == 0 ? 8 : 0;
      for (int i = lane; i < 256; i += 32) hist[i] = 0;
      __syncwarp();
      for (int i = lane; i < n; i += 32) {
        const uint32_t k = key16(keys[i]);
        if (round == 0 || (k >> 8) == prefix) atomicAdd(&hist[(k >> shift) & 255u], 1u);
      }
      __syncwarp();
      int left;
      const int bin = warp_find_bin_from_top(hist, need, lane, &left);
      prefix = round == 0 ? uint32_t(bin) : ((prefix << 8) | uint32_t(bin));
      need = left;
      __syncwarp();
    }
    const uint32_t T = prefix;  // cut key; `need` of the values equal to it are kept, lowest index first
    // ties: every lane owns a contiguous chunk of indices; exclusive scan of the per-chunk tie counts
    const int chunk = (n + 31) / 32;
    const int i0 = min(n, lane * chunk), i1 = min(n, i0 + chunk);
    int ties = 0;
    for (int i = i0; i < i1; ++i) ties += key16(keys[i]) == T;
    int incl = ties;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
      if (lane >= o) incl += t;
    }
    int tie_rank = incl - ties;
    for (int i = i0; i < i1; ++i) {
      const uint32_t k = key16(keys[i]);
      bool keep = k > T;
      if (k == T) { keep = tie_rank < need; ++tie_rank; }
      if (!keep) keys[i] = 0;
    }
    __syncwarp();
  }
  // one coalesced pass writes the row (16 bytes per lane and step; nd_cap is a multiple of 8)
  const uint4* k4 = reinterpret_cast<const uint4*>(keys);
  uint4* o4 = reinterpret_cast<uint4*>(obits);
  for (int i = lane; i < nd_cap / 8; i += 32) o4[i] = k4[i];
}

// ------------------------------------------------------------------ same-layer decoder rows of the dead features
// W0 [L, nd_cap, d]: row i of layer l = row 0 of feature dead_cols[l][i] in decoder tensor l (zero for i >= nd[l]).
struct AuxRowsParams {
  const t16* w[32];
  int rows[32];
};
__global__ void __launch_bounds__(256) aux_gather_rows_kernel(AuxRowsParams p, const int* __restrict__ dead_cols, const int* __restrict__ nd,
                                                                int nd_cap, int d, t16* __restrict__ W0) {
  const int l = blockIdx.y;
  const int vec = d / 8;
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < 1LL * nd_cap * vec; i += 1LL * gridDim.x * blockDim.x) {
    const int r = int(i / vec), e0 = int(i - 1LL * r * vec) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < nd[l]) {
      const int f = __ldg(dead_cols + 1LL * l * nd_cap + r);
      v = __ldg(reinterpret_cast<const uint4*>(p.w[l] + 1LL * f * p.rows[l] * d + e0));
    }
    *reinterpret_cast<uint4*>(W0 + (1LL * l * nd_cap + r) * d + e0) = v;
  }
}

// ------------------------------------------------------------------ residual, loss and gradients of the auxiliary decode
// recon [L, B, d] fp32 (A W0); bias [n_bias, d] with the same-layer bias of layer l at row bias_row[l]; gs [L, B, d] holds
// (y_hat - y) sigma^2 scale.  residual = (y - y_hat) sigma = -gs / (scale sigma);  r = recon + bias - residual;
// loss += factor * mean(r^2);  g = 2 factor / (B d) r  (16-bit);  gs += factor * r * sigma * scale  (the term's gradient
// with respect to the main reconstruction, in the seed's units: the optimizer multiplies the seed by 2 / (B d)).
__global__ void __launch_bounds__(256) aux_residual_kernel(const float* __restrict__ recon, const void* __restrict__ bias, int bias_is_16,
                                                             const int* __restrict__ bias_row, const float* __restrict__ sigma,
                                                             t16* __restrict__ gs, t16* __restrict__ g_out, double* __restrict__ loss,
                                                             const int* __restrict__ nd, const float* __restrict__ ctl, int L, int B, int d,
                                                             float factor, int scale_g) {
  const int l = blockIdx.y;
  const bool live = nd[l] > 0;  // a layer without dead features has no auxiliary term
  const float scale = ctl != nullptr ? ctl[SC_LOSS_SCALE] : 1.f;
  const float inv_scale = 1.f / scale;
  // dL/d recon is of the order 1e-8 per element at training sizes: below the smallest fp16 value.  With scale_g it is kept
  // times the loss scale (like the main gradient seed) and the fp32 products are unscaled afterwards (unscale_kernel).
  const float gcoef = 2.f * factor / (float(B) * float(d)) * (scale_g ? scale : 1.f);
  const int vec = d / 8;
  float sq = 0.f;
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < 1LL * B * vec; i += 1LL * gridDim.x * blockDim.x) {
    const int b = int(i / vec), e0 = int(i - 1LL * b * vec) * 8;
    const long long off = (1LL * l * B + b) * d + e0;
    uint4 gq = make_uint4(0, 0, 0, 0);
    if (live) {
      const float4 r0 = *reinterpret_cast<const float4*>(recon + off), r1 = *reinterpret_cast<const float4*>(recon + off + 4);
      const float rc[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
      uint4 sv = *reinterpret_cast<const uint4*>(gs + off);
      uint32_t su[4] = {sv.x, sv.y, sv.z, sv.w};
      float g[8], ns[8];
      const long long boff = 1LL * bias_row[l] * d + e0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sg = sigma != nullptr ? sigma[1LL * l * d + e0 + j] : 1.f;
        const float bj = bias_is_16 ? t16_to_float(static_cast<const t16*>(bias)[boff + j]) : static_cast<const float*>(bias)[boff + j];
        const float seed = (j & 1) ? t16_hi(su[j >> 1]) : t16_lo(su[j >> 1]);
        const float residual = -seed * inv_scale / sg;
        const float r = rc[j] + bj - residual;
        sq = fmaf(r, r, sq);
        g[j] = gcoef * r;
        ns[j] = seed + factor * r * sg * scale;
      }
      gq.x = pack_t16x2(g[0], g[1]); gq.y = pack_t16x2(g[2], g[3]); gq.z = pack_t16x2(g[4], g[5]); gq.w = pack_t16x2(g[6], g[7]);
      sv.x = pack_t16x2(ns[0], ns[1]); sv.y = pack_t16x2(ns[2], ns[3]); sv.z = pack_t16x2(ns[4], ns[5]); sv.w = pack_t16x2(ns[6], ns[7]);
      *reinterpret_cast<uint4*>(gs + off) = sv;
    }
    *reinterpret_cast<uint4*>(g_out + off) = gq;
  }
  __shared__ float red[8];
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < 8; ++w) tot += red[w];
    if (tot != 0.f) atomicAdd(loss, double(tot) * double(factor) / (double(B) * double(d)));
  }
}

// buf *= 1 / loss scale (gradients that were formed from a scaled 16-bit factor)
__global__ void __launch_bounds__(256) unscale_kernel(float* __restrict__ buf, long long n, const float* __restrict__ ctl) {
  const float inv = ctl[SC_INV_SCALE];
  for (long long i = (blockIdx.x * 1LL * blockDim.x + threadIdx.x) * 4; i < n; i += 1LL * gridDim.x * blockDim.x * 4) {
    if (i + 4 <= n) {
      float4 v = *reinterpret_cast<float4*>(buf + i);
      v.x *= inv; v.y *= inv; v.z *= inv; v.w *= inv;
      *reinterpret_cast<float4*>(buf + i) = v;
    } else {
      for (long long j = i; j < n; ++j) buf[j] *= inv;
    }
  }
}

// out[r] = sum of the 16-bit row r of in [rows, n]  (encoder-bias gradient of the dead features: row sums of G^T)
__global__ void __launch_bounds__(256) rowsum16_kernel(const t16* __restrict__ in, float* __restrict__ out, long long rows, int n) {
  const int lane = threadIdx.x & 31;
  const long long warp_global = (blockIdx.x * 1LL * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (gridDim.x * 1LL * blockDim.x) >> 5;
  for (long long r = warp_global; r < rows; r += nwarps) {
    const t16* p = in + r * n;
    float s = 0.f;
    for (int i = lane * 8; i < n; i += 256) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(p + i));
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) s += t16_lo(u[j]) + t16_hi(u[j]);
    }
    s = warp_sum(s);
    if (lane == 0) out[r] = s;
  }
}

// dst[idx[r], :] += src[r, :] for the rows with idx >= 0 (compact extra rows added into a dense [rows_dst, d] gradient)
__global__ void __launch_bounds__(256) scatter_add_rows_kernel(float* __restrict__ dst, float* __restrict__ dst_bias, const float* __restrict__ src,
                                                                 const float* __restrict__ src_bias, const int* __restrict__ extra_idx,
                                                                 long long n_dst_rows, int d) {
  const int vec = d / 4;
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < n_dst_rows * vec; i += 1LL * gridDim.x * blockDim.x) {
    const long long row = i / vec;
    const int e0 = int(i - row * vec) * 4;
    const int x = __ldg(extra_idx + row);
    if (x < 0) continue;
    float4 a = *reinterpret_cast<float4*>(dst + row * d + e0);
    const float4 b = *reinterpret_cast<const float4*>(src + 1LL * x * d + e0);
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    *reinterpret_cast<float4*>(dst + row * d + e0) = a;
    if (e0 == 0 && dst_bias != nullptr) dst_bias[row] += src_bias[x];
  }
}

}  // namespace clt

using namespace clt;

#if !CLT_T16_IS_HALF
extern "C" int clt_aux_compact(const long long* dead_counter, long long window, int L, int F_pitch, int F_valid, int nd_cap, int* dead_cols,
                               int* nd, int* nd_all, int* extra_idx, cudaStream_t st) {
  if (L <= 0 || nd_cap <= 0) return -1;
  aux_compact_kernel<<<L, 1024, 0, st>>>(dead_counter, window, F_pitch, F_valid, nd_cap, dead_cols, nd, nd_all, extra_idx);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int clt_unscale(float* buf, long long n, const float* ctl, cudaStream_t st) {
  if (n <= 0) return 0;
  if (ctl == nullptr || (reinterpret_cast<uintptr_t>(buf) & 15) != 0) return -1;
  const long long nv = (n + 3) / 4;
  const int grid = int((nv + 255) / 256 < 148 * 16 ? (nv + 255) / 256 : 148 * 16);
  unscale_kernel<<<grid, 256, 0, st>>>(buf, n, ctl);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int clt_scatter_add_rows(float* dst, float* dst_bias, const float* src, const float* src_bias, const int* extra_idx,
                                    long long n_dst_rows, int d, cudaStream_t st) {
  if (d % 4 != 0) return -1;
  const long long n = n_dst_rows * (d / 4);
  const int grid = int((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  scatter_add_rows_kernel<<<grid, 256, 0, st>>>(dst, dst_bias, src, src_bias, extra_idx, n_dst_rows, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
#endif

extern "C" int CLT_FN(clt_aux_gather_select)(const void* pre, long long ld, long long layer_stride, const void* enc_bias, int bias_is_16,
                                             int F_pitch, float* bias_c, const int* dead_cols, const int* nd, const int* nd_all, int nd_cap,
                                             int k_aux_max, int L, int B, void* A, cudaStream_t st) {
  if (nd_cap > kAuxMaxCap || nd_cap % 8 != 0 || (pre == nullptr) == (enc_bias == nullptr)) return -1;
  if (enc_bias != nullptr) {
    if (bias_c == nullptr) return -1;  // scratch [L, nd_cap] fp32 for the compact bias
    aux_gather_bias_kernel<<<dim3((nd_cap + 255) / 256, L), 256, 0, st>>>(enc_bias, bias_is_16, F_pitch, dead_cols, nd, nd_cap, bias_c);
  }
  const size_t smem = 8 * (size_t(nd_cap) * 2 + 1024);
  static size_t attr_smem = 0;
  if (smem > 48 * 1024 && smem > attr_smem) {
    if (cudaFuncSetAttribute(aux_gather_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return -4;
    attr_smem = smem;
  }
  aux_gather_select_kernel<<<dim3((B + 7) / 8, L), 256, smem, st>>>(static_cast<const t16*>(pre), ld, layer_stride, enc_bias != nullptr ? bias_c : nullptr, dead_cols,
                                                        nd, nd_all, nd_cap, k_aux_max, B, static_cast<t16*>(A));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

struct CltAuxRowsArgs {
  const void* w[32];
  int rows[32];
};
extern "C" int CLT_FN(clt_aux_gather_rows)(const CltAuxRowsArgs* a, const int* dead_cols, const int* nd, int nd_cap, int L, int d, void* W0,
                                           cudaStream_t st) {
  if (d % 8 != 0 || L > 32) return -1;
  AuxRowsParams p;
  for (int i = 0; i < 32; ++i) { p.w[i] = static_cast<const t16*>(a->w[i]); p.rows[i] = a->rows[i]; }
  const long long n = 1LL * nd_cap * (d / 8);
  const int gx = int((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
  aux_gather_rows_kernel<<<dim3(gx, L), 256, 0, st>>>(p, dead_cols, nd, nd_cap, d, static_cast<t16*>(W0));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int CLT_FN(clt_aux_residual)(const float* recon, const void* bias, int bias_is_16, const int* bias_row, const float* sigma, void* gs,
                                        void* g_out, double* loss, const int* nd, const float* ctl, int L, int B, int d, float factor,
                                        int scale_g, cudaStream_t st) {
  if (d % 8 != 0) return -1;
  const long long n = 1LL * B * (d / 8);
  const int gx = int((n + 255) / 256 < 592 ? (n + 255) / 256 : 592);
  aux_residual_kernel<<<dim3(gx, L), 256, 0, st>>>(recon, bias, bias_is_16, bias_row, sigma, static_cast<t16*>(gs), static_cast<t16*>(g_out), loss,
                                                   nd, ctl, L, B, d, factor, scale_g);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int CLT_FN(clt_rowsum16)(const void* in, float* out, long long rows, int n, cudaStream_t st) {
  if (n % 8 != 0) return -1;
  const int grid = int((rows + 7) / 8 < 1184 ? (rows + 7) / 8 : 1184);
  rowsum16_kernel<<<grid, 256, 0, st>>>(static_cast<const t16*>(in), out, rows, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
