// Grouped dense GEMM on the tensor cores for the loss terms that are not sparse (sm_100a).
//
//   C[g][m, n] = alpha * sum over the segments (a, b) of group g of  sum_k A[a][m, k] * B[b][n, k]
//
// A = [LA, M, K], B = [LB, N, K], both K-major 16-bit; C = [G, M, N] fp32 or 16-bit.  A group names which layers of A
// and B are multiplied and accumulates several (A layer, B layer) pairs into one output - the K dimension runs over the
// segments, the accumulator stays in tensor memory.  Users:
//
//   * skip connection forward (reference clt/models/decoder.py:298-338): group = target layer t, segments = sources
//     s <= t with A = layer inputs x[s] [B, d], B = W_skip[s -> t] [d_out, d_in]; tied: one segment per layer;
//   * skip connection backward: group = pair (s, t), A = gs[t]^T [d, B], B = x[s]^T [d, B]  ->  dW_skip [d_out, d_in];
//   * pre-activation loss (reference clt/training/losses.py:203-261): group = layer, A = 1[pre < 0]^T [F, B],
//     B = x^T [d, B]  ->  dense encoder gradient [F, d];
//   * auxiliary loss on dead features (losses.py:263-329): the four products between the gathered dead decoder rows,
//     the masked dead pre-activations, the residual gradient and the layer inputs.
//
// Structure: the persistent single-CTA pipeline of encoder_gemm.cu: warp 0 feeds a four-stage ring with TMA tile
// loads (no multicast), warp 1 issues tcgen05.mma 128x256x16 into one of two TMEM accumulators, warps 2-5 drain the
// other one through a swizzled staging tile and TMA stores.  Every mbarrier wait is bounded.
#include "common.cuh"

namespace clt {

namespace dg {
constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr uint32_t A_BYTES = BM * BK * 2;
constexpr uint32_t B_BYTES = BN * BK * 2;
constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr size_t SMEM_BYTES = size_t(STAGES) * STAGE_BYTES + 4 * 4096 + 1024 + 2048;
}  // namespace dg

struct DenseGemmShared {
  uint64_t full[dg::STAGES];
  uint64_t empty[dg::STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int epi_ok;
};

// One 32-row slab of the accumulator (lane = row) -> staging tile -> TMA store, 32 fp32 columns (or 64 16-bit columns)
// at a time.  `stage` is this warp's 4 KB buffer (1024-byte aligned): 32 rows of 128 bytes, 16-byte chunks swizzled
// with the row index like the tensor map expects.
template <bool OUT_F32>
__device__ __forceinline__ void dense_epilogue_slab(uint32_t taddr, const CUtensorMap* map_c, uint8_t* stage, int bn, int n_base, int m_base,
                                                    int g, int lane, float alpha) {
  constexpr int kCols = OUT_F32 ? 32 : 64;
  for (int c = 0; c < bn / kCols; ++c) {
    uint32_t r0[32], r1[32];
    tmem_ld_32x32(taddr + c * kCols, r0);
    if (!OUT_F32) tmem_ld_32x32(taddr + c * kCols + 32, r1);
    if (lane == 0) bulk_wait_read<0>();  // the previous store has read the staging tile
    __syncwarp();
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 8; ++j) {  // 16-byte chunk j of this lane's row
      uint4 q;
      if (OUT_F32) {
        q.x = __float_as_uint(__uint_as_float(r0[4 * j]) * alpha); q.y = __float_as_uint(__uint_as_float(r0[4 * j + 1]) * alpha);
        q.z = __float_as_uint(__uint_as_float(r0[4 * j + 2]) * alpha); q.w = __float_as_uint(__uint_as_float(r0[4 * j + 3]) * alpha);
      } else {
        const uint32_t* r = j < 4 ? &r0[8 * j] : &r1[8 * (j - 4)];
        q.x = pack_t16x2(__uint_as_float(r[0]) * alpha, __uint_as_float(r[1]) * alpha);
        q.y = pack_t16x2(__uint_as_float(r[2]) * alpha, __uint_as_float(r[3]) * alpha);
        q.z = pack_t16x2(__uint_as_float(r[4]) * alpha, __uint_as_float(r[5]) * alpha);
        q.w = pack_t16x2(__uint_as_float(r[6]) * alpha, __uint_as_float(r[7]) * alpha);
      }
      *reinterpret_cast<uint4*>(stage + lane * 128 + ((j ^ (lane & 7)) << 4)) = q;
    }
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      tma_store_3d(map_c, stage, n_base + c * kCols, m_base, g);
      bulk_commit();
    }
  }
}

// group_off [G + 1]: first segment of every group; segs [n_segs]: (A layer, B layer) per segment.
template <bool OUT_F32>
__global__ void __launch_bounds__(dg::NUM_THREADS, 1)
dense_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_c, const int* __restrict__ group_off, const int2* __restrict__ segs,
                  int G, int M, int N, int K, float alpha, int* __restrict__ status) {
  using namespace dg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = tiles + size_t(STAGES) * STAGE_BYTES;
  DenseGemmShared* sh = reinterpret_cast<DenseGemmShared*>(epi_stage + 4 * 4096);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_kb = (K + BK - 1) / BK;
  const long long tiles_per_group = 1LL * tiles_m * tiles_n;
  const long long total_tiles = 1LL * G * tiles_per_group;
  volatile int* abort_flag = &sh->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->tmem_full[b], 1);
      mbar_init(&sh->tmem_empty[b], 4);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      uint32_t it = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int g = int(t / tiles_per_group);
        const long long rem = t - 1LL * g * tiles_per_group;
        const int mt = int(rem % tiles_m), nt = int(rem / tiles_m);
        const int s0 = __ldg(group_off + g), s1 = __ldg(group_off + g + 1);
        for (int sg = s0; sg < s1 && ok; ++sg) {
          const int2 ab = __ldg(segs + sg);
          for (int kb = 0; kb < num_kb; ++kb, ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            if (!mbar_wait(&sh->empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
            mbar_expect_tx(&sh->full[s], STAGE_BYTES);
            uint8_t* a_dst = tiles + size_t(s) * STAGE_BYTES;
            tma_load_3d(a_dst, &map_a, &sh->full[s], kb * BK, mt * BM, ab.x);
            tma_load_3d(a_dst + A_BYTES, &map_b, &sh->full[s], kb * BK, nt * BN, ab.y);
          }
        }
      }
      if (!ok) {
        // give the copies already issued a bounded chance to land before the CTA retires
        const uint32_t issued = it;
        const uint32_t first = issued > STAGES ? issued - STAGES : 0;
        for (uint32_t j = first; j < issued; ++j) {
          const long long start = clock64();
          while (!mbar_try_wait(&sh->full[j % STAGES], (j / STAGES) & 1)) {
            if (clock64() - start > kWaitTimeoutCycles) break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local_tile) {
        const int g = int(t / tiles_per_group);
        const int nseg = __ldg(group_off + g + 1) - __ldg(group_off + g);
        const uint32_t buf = local_tile & 1;
        const uint32_t tph = (local_tile >> 1) & 1;
        if (!mbar_wait(&sh->tmem_empty[buf], tph ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        const int steps = nseg * num_kb;
        for (int kb = 0; kb < steps; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&sh->full[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(tiles + size_t(s) * STAGE_BYTES);
          const uint64_t a_desc = umma_desc_kmajor_sw128(a_addr);
          const uint64_t b_desc = umma_desc_kmajor_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16_ss(d_tmem, a_desc + uint64_t(k * 2), b_desc + uint64_t(k * 2), idesc, (kb | k) != 0);
          tc_commit(&sh->empty[s]);
        }
        if (ok) tc_commit(&sh->tmem_full[buf]);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;
    const int etid = (warp - 2) * 32 + lane;
    uint32_t local_tile = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local_tile) {
      const int g = int(t / tiles_per_group);
      const long long rem = t - 1LL * g * tiles_per_group;
      const int mt = int(rem % tiles_m), nt = int(rem / tiles_m);
      const uint32_t buf = local_tile & 1;
      const uint32_t tph = (local_tile >> 1) & 1;
      // one thread performs the bounded wait and publishes the outcome: the four warps take the same branch
      if (etid == 0) sh->epi_ok = mbar_wait(&sh->tmem_full[buf], tph, abort_flag) ? 1 : 0;
      named_barrier_sync(1, 128);
      const bool good = sh->epi_ok != 0;
      named_barrier_sync(1, 128);  // everybody has read the flag before the next tile overwrites it
      if (!good) { ok = false; break; }
      tc_fence_after();
      const int m_base = mt * BM + quarter * 32;
      const uint32_t taddr = tmem_base + buf * BN + (uint32_t(quarter * 32) << 16);
      constexpr int kCols = OUT_F32 ? 32 : 64;
      const int bn = min(BN, ((N - nt * BN + kCols - 1) / kCols) * kCols);
      if (m_base < M) dense_epilogue_slab<OUT_F32>(taddr, &map_c, epi_stage + (warp - 2) * 4096, bn, nt * BN, m_base, g, lane, alpha);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->tmem_empty[buf]);
    }
  }

  if (warp >= 2 && lane == 0) bulk_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && sh->abort_flag && status != nullptr) atomicCAS(status, STATUS_OK, STATUS_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------ transposes and the pre-activation indicator
// out[l][c, r] = in[l][r, c] for 16-bit elements, 64 x 64 tiles through shared memory.
__global__ void __launch_bounds__(256) transpose16_kernel(const t16* __restrict__ in, t16* __restrict__ out, int R, int C, long long ld_in,
                                                            long long layer_stride_in) {
  __shared__ t16 tile[64][66];
  const int l = blockIdx.z;
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const t16* src = in + 1LL * l * layer_stride_in;
  t16* dst = out + 1LL * l * R * C;
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int r = i >> 6, c = i & 63;
    tile[r][c] = (r0 + r < R && c0 + c < C) ? src[1LL * (r0 + r) * ld_in + c0 + c] : float_to_t16(0.f);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int c = i >> 6, r = i & 63;
    if (c0 + c < C && r0 + r < R) dst[1LL * (c0 + c) * R + r0 + r] = tile[r][c];
  }
}

// The same for shapes and addresses that allow 16-byte accesses on both sides (R, C, ld_in multiples of 8).  With `mask`
// (same layout as `in`) the elements whose mask value is zero are written as zero: the straight-through gradient of a
// selection, applied while the gradient is transposed for the GEMM that consumes it.
__global__ void __launch_bounds__(256) transpose16_vec_kernel(const t16* __restrict__ in, const t16* __restrict__ mask, t16* __restrict__ out, int R,
                                                                int C, long long ld_in, long long layer_stride_in) {
  __shared__ uint32_t tile[64][33];  // 64 rows x 64 elements, two per word
  const int l = blockIdx.z;
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const t16* src = in + 1LL * l * layer_stride_in;
  const t16* msk = mask != nullptr ? mask + 1LL * l * layer_stride_in : nullptr;
  t16* dst = out + 1LL * l * R * C;
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int r = (threadIdx.x >> 3) + 32 * it, v = threadIdx.x & 7;
    uint4 q = make_uint4(0, 0, 0, 0);
    if (r0 + r < R && c0 + 8 * v < C) {
      q = __ldg(reinterpret_cast<const uint4*>(src + 1LL * (r0 + r) * ld_in + c0 + 8 * v));
      if (msk != nullptr) {
        const uint4 k = __ldg(reinterpret_cast<const uint4*>(msk + 1LL * (r0 + r) * ld_in + c0 + 8 * v));
        const uint32_t ku[4] = {k.x, k.y, k.z, k.w};
        uint32_t qu[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if ((ku[j] & 0x7FFFu) == 0u) qu[j] &= 0xFFFF0000u;
          if ((ku[j] & 0x7FFF0000u) == 0u) qu[j] &= 0x0000FFFFu;
        }
        q = make_uint4(qu[0], qu[1], qu[2], qu[3]);
      }
    }
    tile[r][4 * v + 0] = q.x; tile[r][4 * v + 1] = q.y; tile[r][4 * v + 2] = q.z; tile[r][4 * v + 3] = q.w;
  }
  __syncthreads();
  const unsigned short* t16s = reinterpret_cast<const unsigned short*>(&tile[0][0]);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int c = 8 * warp + (lane & 7), rg = 4 * it + (lane >> 3);  // output row c, elements 8 rg .. 8 rg + 7
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t lo = t16s[(8 * rg + 2 * j) * 66 + c], hi = t16s[(8 * rg + 2 * j + 1) * 66 + c];
      w[j] = lo | (hi << 16);
    }
    if (c0 + c < C && r0 + 8 * rg < R) *reinterpret_cast<uint4*>(dst + 1LL * (c0 + c) * R + r0 + 8 * rg) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// Pre-activation loss, first half: ind[l][f, b] = 1 where pre[l][b, f] < 0 (transposed, as the A operand of the gradient
// GEMM), loss[0] += coef / numel * sum relu(-pre), bias_grad[l, f] = -(coef / numel) * #{b : pre < 0}.
__global__ void __launch_bounds__(256) negative_indicator_kernel(const t16* __restrict__ pre, t16* __restrict__ ind, float* __restrict__ bias_grad,
                                                                   double* __restrict__ loss, int B, int F, int F_valid, long long ld,
                                                                   float coef_over_numel) {
  __shared__ t16 tile[64][66];
  __shared__ float colsum[64];
  __shared__ float red[8];
  const int l = blockIdx.z;
  const int b0 = blockIdx.y * 64, f0 = blockIdx.x * 64;
  if (threadIdx.x < 64) colsum[threadIdx.x] = 0.f;
  __syncthreads();
  const t16* src = pre + 1LL * l * B * ld;
  float part = 0.f;
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int r = i >> 6, c = i & 63;
    float v = 0.f;
    if (b0 + r < B && f0 + c < F_valid) v = t16_to_float(src[1LL * (b0 + r) * ld + f0 + c]);
    const bool neg = v < 0.f;
    tile[r][c] = float_to_t16(neg ? 1.f : 0.f);
    if (neg) { part -= v; atomicAdd(&colsum[c], 1.f); }
  }
  __syncthreads();
  t16* dst = ind + 1LL * l * F * B;
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int c = i >> 6, r = i & 63;
    if (f0 + c < F && b0 + r < B) dst[1LL * (f0 + c) * B + b0 + r] = tile[r][c];
  }
  if (threadIdx.x < 64 && f0 + threadIdx.x < F && colsum[threadIdx.x] != 0.f)
    atomicAdd(&bias_grad[1LL * l * F + f0 + threadIdx.x], -coef_over_numel * colsum[threadIdx.x]);
  part = warp_sum(part);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < 8; ++w) tot += red[w];
    if (tot != 0.f) atomicAdd(loss, double(tot) * double(coef_over_numel));
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFnD)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFnD dg_encode_fn() {
  static EncodeTiledFnD fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFnD>(p);
  }
  return fn;
}

// [layers, rows, cols], cols contiguous; box = [1, box_rows, box_cols] with the 128-byte swizzle (box_cols * elem = 128 bytes).
static bool dg_make_map(CUtensorMap* map, const void* base, CUtensorMapDataType dt, int elem_bytes, int layers, int rows, long long cols,
                        long long row_stride_elems, long long layer_stride_elems, int box_rows, int box_cols) {
  EncodeTiledFnD enc = dg_encode_fn();
  if (enc == nullptr) return false;
  cuuint64_t dims[3] = {cuuint64_t(cols), cuuint64_t(rows), cuuint64_t(layers)};
  cuuint64_t strides[2] = {cuuint64_t(row_stride_elems) * elem_bytes, cuuint64_t(layer_stride_elems) * elem_bytes};
  cuuint32_t box[3] = {cuuint32_t(box_cols), cuuint32_t(box_rows), 1};
  cuuint32_t elem[3] = {1, 1, 1};
  return enc(map, dt, 3, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace clt

using namespace clt;

// A [LA, M, K] (row stride lda, layer stride a_layer_stride, in elements), B [LB, N, K], C [G, M, N] contiguous (fp32 when
// out_f32, else 16-bit).  group_off [G + 1] and segs [n_segs][2] live in device memory.
extern "C" int CLT_FN(clt_dense_gemm)(const void* A, int LA, long long lda, long long a_layer_stride, const void* B, int LB, long long ldb,
                                      long long b_layer_stride, void* C, int out_f32, const int* group_off, const int* segs, int G, int M,
                                      int N, int K, float alpha, int* status, int num_sms, cudaStream_t stream) {
  if (K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0 || a_layer_stride % 8 != 0 || b_layer_stride % 8 != 0) return -1;
  if (N % (out_f32 ? 4 : 8) != 0) return -1;  // 16-byte output rows
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -2;
  if (G <= 0 || M <= 0 || N <= 0) return 0;
  const CUtensorMapDataType t16dt = CLT_T16_IS_HALF ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap map_a, map_b, map_c;
  if (!dg_make_map(&map_a, A, t16dt, 2, LA, M, K, lda, a_layer_stride, dg::BM, dg::BK)) return -3;
  if (!dg_make_map(&map_b, B, t16dt, 2, LB, N, K, ldb, b_layer_stride, dg::BN, dg::BK)) return -3;
  if (out_f32) {
    if (!dg_make_map(&map_c, C, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, G, M, N, N, 1LL * M * N, 32, 32)) return -3;
  } else {
    if (!dg_make_map(&map_c, C, t16dt, 2, G, M, N, N, 1LL * M * N, 32, 64)) return -3;
  }
  static bool attr_set[2] = {false, false};
  if (!attr_set[out_f32 ? 1 : 0]) {
    const cudaError_t rc = out_f32 ? cudaFuncSetAttribute(dense_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dg::SMEM_BYTES))
                                   : cudaFuncSetAttribute(dense_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(dg::SMEM_BYTES));
    if (rc != cudaSuccess) return -4;
    attr_set[out_f32 ? 1 : 0] = true;
  }
  const long long tiles = 1LL * G * ((M + dg::BM - 1) / dg::BM) * ((N + dg::BN - 1) / dg::BN);
  const int grid = int(tiles < num_sms ? tiles : num_sms);
  const int2* sp = reinterpret_cast<const int2*>(segs);
  if (out_f32) dense_gemm_kernel<true><<<grid, dg::NUM_THREADS, dg::SMEM_BYTES, stream>>>(map_a, map_b, map_c, group_off, sp, G, M, N, K, alpha, status);
  else dense_gemm_kernel<false><<<grid, dg::NUM_THREADS, dg::SMEM_BYTES, stream>>>(map_a, map_b, map_c, group_off, sp, G, M, N, K, alpha, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int CLT_FN(clt_transpose16)(const void* in, void* out, int L, int R, int C, long long ld_in, long long layer_stride_in,
                                       const void* mask, cudaStream_t st) {
  if (L <= 0 || R <= 0 || C <= 0) return 0;
  dim3 grid((C + 63) / 64, (R + 63) / 64, L);
  const bool vec = R % 8 == 0 && C % 8 == 0 && ld_in % 8 == 0 && layer_stride_in % 8 == 0 &&
                   ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(mask)) & 15) == 0;
  if (vec) {
    transpose16_vec_kernel<<<grid, 256, 0, st>>>(static_cast<const t16*>(in), static_cast<const t16*>(mask), static_cast<t16*>(out), R, C, ld_in,
                                                 layer_stride_in);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
  }
  if (mask != nullptr) return -1;  // the masked form needs the 16-byte layout
  transpose16_kernel<<<grid, 256, 0, st>>>(static_cast<const t16*>(in), static_cast<t16*>(out), R, C, ld_in, layer_stride_in);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int CLT_FN(clt_negative_indicator)(const void* pre, void* ind, float* bias_grad, double* loss, int L, int B, int F, int F_valid,
                                              long long ld, float coef_over_numel, cudaStream_t st) {
  if (L <= 0 || B <= 0 || F <= 0) return 0;
  dim3 grid((F + 63) / 64, (B + 63) / 64, L);
  negative_indicator_kernel<<<grid, 256, 0, st>>>(static_cast<const t16*>(pre), static_cast<t16*>(ind), bias_grad, loss, B, F, F_valid, ld,
                                                  coef_over_numel);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
