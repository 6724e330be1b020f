// Threshold gradient of JumpReLU as one tcgen05 GEMM per source layer with a reducing epilogue (sm_100a).
//
// The straight-through estimator of the reference gives every feature's threshold the gradient
//     d loss / d theta[f] = -(1 / bw) * sum_b  1[|x[b,f] - theta[f]| <= bw / 2] * x[b,f] * G[b,f]
// (clt/models/activations.py:196-220), where G = d loss / d activation is needed at every position inside the
// window, active or not.  With bw = 1 the window holds most positions, so G is a dense quantity:
//     G[b, f] = sum over targets t >= s of  gs[t][b, :] . W_dec[s -> t][f, :]   (+ the sparsity-penalty term)
// For source layer s this is a GEMM  [B, (L - s) d] x [(L - s) d, F]  whose K dimension runs over the target
// layers: A = the gradient seed of layers s..L-1 side by side, B = the packed decoder tensor of layer s,
// which is already K-major ([F, (L - s), d]).  The [B, F] product is never written: the epilogue multiplies it
// with window * x and reduces over the 128 token rows of the tile,
//     S1[s, f] += sum_b window * x * G_recon        S2[s, f] += sum_b window * x
// (S2 carries the penalty term, whose G is a per-feature constant outside the active entries).
// The autograd path computes the same through P dense GEMM pairs and a dense [B, F] backward per layer.
//
// Structure: the persistent single-CTA pipeline of encoder_gemm.cu (TMA ring, one MMA thread, two TMEM
// accumulators, four epilogue warps).  No multicast loads.  Every mbarrier wait is bounded.
#include "common.cuh"

namespace clt {

namespace tg {
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
constexpr size_t SMEM_BYTES = size_t(STAGES) * STAGE_BYTES + 1024 + 4096;
constexpr int kMaxLayers = 32;
}  // namespace tg

struct ThetaGradMaps {
  CUtensorMap b[tg::kMaxLayers];  // decoder tensor of source layer s viewed as [F, (L - s) * d]
};

struct ThetaGradShared {
  uint64_t full[tg::STAGES];
  uint64_t empty[tg::STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  int epi_ok;
  alignas(16) float theta[tg::BN];
  float acc1[tg::BN];
  float acc2[tg::BN];
};

// v[0..31] of every lane -> lane j holds the sum over the warp's lanes of v[j].
__device__ __forceinline__ float warp_transpose_sum(float (&v)[32], int lane) {
#pragma unroll
  for (int off = 16, n = 32; off >= 1; off >>= 1, n >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < n / 2; ++i) {
      const float send = upper ? v[i] : v[i + n / 2];
      const float keep = upper ? v[i + n / 2] : v[i];
      v[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, off);
    }
  }
  return v[0];
}

__global__ void __launch_bounds__(tg::NUM_THREADS, 1)
theta_grad_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a_cum,
                       const __grid_constant__ ThetaGradMaps maps_b, int tying,
                       const t16* __restrict__ preact, long long ldx, long long layer_stride_x,
                       const float* __restrict__ theta, int stat_pitch, float half_bw, float* __restrict__ S1,
                       float* __restrict__ S2, int L, int M, int N, int d, int* __restrict__ status) {
  using namespace tg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  ThetaGradShared* sh = reinterpret_cast<ThetaGradShared*>(tiles + size_t(STAGES) * STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int kb_per_layer = (d + BK - 1) / BK;
  const long long tiles_per_layer = 1LL * tiles_m * tiles_n;
  const long long total_tiles = 1LL * L * tiles_per_layer;  // source layers in ascending order: longest K first
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
  for (int j = threadIdx.x; j < BN; j += NUM_THREADS) { sh->acc1[j] = 0.f; sh->acc2[j] = 0.f; }
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
      uint32_t it = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const int src = int(t / tiles_per_layer);
        const long long rem = t - 1LL * src * tiles_per_layer;
        const int mt = int(rem % tiles_m);
        const int nt = int(rem / tiles_m);
        // K runs over the target layers t >= src (untied: rows of the packed tensor of layer src; per_target: the
        // tensors of the layers t); per_source has one decoder row per feature, its A operand is the seed summed over t
        const int num_kb = (tying == 1 ? 1 : L - src) * kb_per_layer;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const int tl = kb / kb_per_layer, kk = kb - tl * kb_per_layer;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&sh->empty[s], ph ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&sh->full[s], STAGE_BYTES);
          uint8_t* a_dst = tiles + size_t(s) * STAGE_BYTES;
          if (tying == 1) tma_load_3d(a_dst, &map_a_cum, &sh->full[s], kk * BK, mt * BM, src);
          else tma_load_3d(a_dst, &map_a, &sh->full[s], kk * BK, mt * BM, src + tl);
          if (tying == 0) tma_load_3d(a_dst + A_BYTES, &maps_b.b[src], &sh->full[s], tl * d + kk * BK, nt * BN, 0);
          else tma_load_3d(a_dst + A_BYTES, &maps_b.b[tying == 2 ? src + tl : src], &sh->full[s], kk * BK, nt * BN, 0);
        }
      }
      if (!ok) {
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
      uint32_t it = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local_tile) {
        const int src = int(t / tiles_per_layer);
        const int num_kb = (tying == 1 ? 1 : L - src) * kb_per_layer;
        const uint32_t buf = local_tile & 1;
        const uint32_t tph = (local_tile >> 1) & 1;
        if (!mbar_wait(&sh->tmem_empty[buf], tph ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
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
    // ---------------------------------------------------------------- reducing epilogue
    const int quarter = warp & 3;
    const int etid = (warp - 2) * 32 + lane;
    uint32_t local_tile = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++local_tile) {
      const int src = int(t / tiles_per_layer);
      const long long rem = t - 1LL * src * tiles_per_layer;
      const int mt = int(rem % tiles_m);
      const int nt = int(rem / tiles_m);
      const uint32_t buf = local_tile & 1;
      const uint32_t tph = (local_tile >> 1) & 1;
      named_barrier_sync(1, 128);  // accumulators of the previous tile were flushed and cleared
      for (int j = etid; j < BN; j += 128) {
        const int n = nt * BN + j;
        sh->theta[j] = n < N ? theta[1LL * src * stat_pitch + n] : INFINITY;
      }
      if (etid == 0) sh->epi_ok = mbar_wait(&sh->tmem_full[buf], tph, abort_flag) ? 1 : 0;
      named_barrier_sync(1, 128);
      if (!sh->epi_ok) { ok = false; break; }
      tc_fence_after();
      const int m = mt * BM + quarter * 32 + lane;
      const bool row_ok = m < M;
      const t16* xrow = preact + 1LL * src * layer_stride_x + 1LL * (row_ok ? m : 0) * ldx + 1LL * nt * BN;
      const uint32_t taddr = tmem_base + buf * BN + (uint32_t(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        float wx[32];
        const int n0 = nt * BN + c * 32;
        if (row_ok && n0 + 32 <= N) {
          const uint4* xp = reinterpret_cast<const uint4*>(xrow + c * 32);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 u = __ldg(xp + q);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) { wx[q * 8 + 2 * j] = t16_lo(w[j]); wx[q * 8 + 2 * j + 1] = t16_hi(w[j]); }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) wx[j] = (row_ok && n0 + j < N) ? t16_to_float(xrow[c * 32 + j]) : INFINITY;
        }
        tmem_ld_wait();
        float p[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const bool in = fabsf(wx[j] - sh->theta[c * 32 + j]) <= half_bw;  // false for the INFINITY fillers
          wx[j] = in ? wx[j] : 0.f;
          p[j] = wx[j] * __uint_as_float(r[j]);
        }
        const float s1 = warp_transpose_sum(p, lane);
        const float s2 = warp_transpose_sum(wx, lane);
        if (s1 != 0.f) atomicAdd(&sh->acc1[c * 32 + lane], s1);
        if (s2 != 0.f) atomicAdd(&sh->acc2[c * 32 + lane], s2);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->tmem_empty[buf]);
      named_barrier_sync(1, 128);  // all four warps added their rows
      for (int j = etid; j < BN; j += 128) {
        const int n = nt * BN + j;
        const float a1 = sh->acc1[j], a2 = sh->acc2[j];
        if (n < N) {
          if (a1 != 0.f) atomicAdd(&S1[1LL * src * stat_pitch + n], a1);
          if (a2 != 0.f) atomicAdd(&S2[1LL * src * stat_pitch + n], a2);
        }
        sh->acc1[j] = 0.f;
        sh->acc2[j] = 0.f;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && sh->abort_flag && status != nullptr) atomicCAS(status, STATUS_OK, STATUS_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFnT)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFnT tg_encode_fn() {
  static EncodeTiledFnT fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFnT>(p);
  }
  return fn;
}

static bool tg_make_map(CUtensorMap* map, const void* base, int layers, int rows, long long K, long long row_stride_elems,
                        long long layer_stride_elems, int box_rows) {
  EncodeTiledFnT enc = tg_encode_fn();
  if (enc == nullptr) return false;
  cuuint64_t dims[3] = {cuuint64_t(K), cuuint64_t(rows), cuuint64_t(layers)};
  cuuint64_t strides[2] = {cuuint64_t(row_stride_elems) * 2, cuuint64_t(layer_stride_elems) * 2};
  cuuint32_t box[3] = {cuuint32_t(tg::BK), cuuint32_t(box_rows), 1};
  cuuint32_t elem[3] = {1, 1, 1};
  return enc(map, (CLT_T16_IS_HALF ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16), 3, const_cast<void*>(base), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace clt

struct CltThetaGradArgs {
  const void* gs;          // [L, B, d] bf16 gradient seed
  const void* w[32];       // untied decoder tensors, layer s: [F, L - s, d] bf16
  const void* preact;      // [L, B, ldx] bf16
  long long ldx, layer_stride_x;
  const float* theta;      // [L, stat_pitch]
  int stat_pitch;
  float bandwidth;
  float* S1;               // [L, stat_pitch], zeroed by the caller
  float* S2;
  int L, B, F, d;
  int* status;
  int tying;               // 0 untied ([F, L - s, d]), 1 per_source, 2 per_target (tensors [F, 1, d])
  const void* gs_cum;      // per_source: [L, B, d] suffix sums of gs over the layers
};

// Returns 0 on success, a negative value when the arguments cannot be handled (the caller raises).
extern "C" int CLT_FN(clt_theta_grad_gemm)(const CltThetaGradArgs* a, int num_sms, cudaStream_t stream) {
  using namespace clt;
  if (a->d % 8 != 0 || a->ldx % 8 != 0 || a->layer_stride_x % 8 != 0 || a->L > tg::kMaxLayers || a->L < 1) return -1;
  CUtensorMap map_a, map_a_cum;
  ThetaGradMaps maps;
  if (a->tying < 0 || a->tying > 2 || (a->tying == 1 && a->gs_cum == nullptr)) return -1;
  if (!tg_make_map(&map_a, a->gs, a->L, a->B, a->d, a->d, 1LL * a->B * a->d, tg::BM)) return -3;
  if (!tg_make_map(&map_a_cum, a->tying == 1 ? a->gs_cum : a->gs, a->L, a->B, a->d, a->d, 1LL * a->B * a->d, tg::BM)) return -3;
  for (int s = 0; s < tg::kMaxLayers; ++s) {
    const int src = s < a->L ? s : a->L - 1;
    const long long K = a->tying == 0 ? 1LL * (a->L - src) * a->d : a->d;
    if ((reinterpret_cast<uintptr_t>(a->w[src]) & 15) != 0) return -2;
    if (!tg_make_map(&maps.b[s], a->w[src], 1, a->F, K, K, 1LL * a->F * K, tg::BN)) return -3;
  }
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(theta_grad_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(tg::SMEM_BYTES)) != cudaSuccess) return -4;
    attr_set = true;
  }
  const long long tiles = 1LL * a->L * ((a->B + tg::BM - 1) / tg::BM) * ((a->F + tg::BN - 1) / tg::BN);
  if (tiles == 0) return 0;
  const int grid = int(tiles < num_sms ? tiles : num_sms);
  theta_grad_gemm_kernel<<<grid, tg::NUM_THREADS, tg::SMEM_BYTES, stream>>>(
      map_a, map_a_cum, maps, a->tying, static_cast<const t16*>(a->preact), a->ldx, a->layer_stride_x, a->theta, a->stat_pitch,
      0.5f * a->bandwidth, a->S1, a->S2, a->L, a->B, a->F, a->d, a->status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
