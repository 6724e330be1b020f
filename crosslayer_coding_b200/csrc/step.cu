// Step control and the small per-step kernels of the fused training step (sm_100a).
//
// The reference decides on the host whether a step is applied: GradScaler.unscale_/step/update with an inf check
// (clt/training/trainer.py:751-783), clip_grad_norm_ with a host-side norm (:769-772), a NaN-loss skip (:740-747),
// five .item() reads for the loss terms (clt/training/losses.py:402-406).  Here one single-CTA kernel does all of it
// on the device after the loss kernels:
//
//   step_control_kernel   sums the loss terms (across ranks through the exchange area, which also serves as the
//                         phase barrier behind the gradient-seed all-gather), decides skip / no skip, keeps the fp16
//                         loss scale (grow / back off) and, in a second call after the norm pre-pass, the clip
//                         coefficient.  The optimizer kernels read the result from the step control block.
//   decoder_bias_adam     gradient of every decoder bias from the column sums of the gradient seed + AdamW.
//   theta_adam            JumpReLU: threshold gradient from the window sums of theta_grad_gemm, the sparsity-penalty
//                         correction at the active entries, AdamW on log_threshold, next step's thresholds.
//   step_finish           dead-feature counters and the per-target bias sums of the next step's loss epilogue.
#include "common.cuh"

namespace clt {

struct AdamHyperS {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;
  int decoupled;
  float grad_scale;
  unsigned int sr_seed;
  unsigned int moment_seed;
};

__device__ __forceinline__ void adam_scalar(float& w, float& m, float& v, float g, const AdamHyperS& h) {
  if (h.decoupled) w *= (1.f - h.lr * h.weight_decay);
  else g = fmaf(h.weight_decay, w, g);
  m = fmaf(h.beta1, m, (1.f - h.beta1) * g);
  v = fmaf(h.beta2, v, (1.f - h.beta2) * g * g);
  w -= (h.lr / h.bc1) * (m / (sqrtf(v) * rsqrtf(h.bc2) + h.eps));
}

template <typename WT>
__device__ __forceinline__ float load_w(const WT* p);
template <>
__device__ __forceinline__ float load_w<t16>(const t16* p) { return t16_to_float(*p); }
template <>
__device__ __forceinline__ float load_w<float>(const float* p) { return *p; }
template <typename WT>
__device__ __forceinline__ void store_w(WT* p, float v);
template <>
__device__ __forceinline__ void store_w<t16>(t16* p, float v) { *p = float_to_t16(v); }
template <>
__device__ __forceinline__ void store_w<float>(float* p, float v) { *p = v; }

// ---------------------------------------------------------------------------------------- step control
constexpr int kMaxScalars = 8;
constexpr int kCtlMaxLayers = 32;

struct StepControlParams {
  float* ctl;           // [SC_SIZE] step control block
  const int* status;    // kernel status word of the step (non-zero: skip)
  double* sq_err;       // [L] squared-error sums: this rank's part in, the sum over ranks out
  int L;
  double* scalars;      // [n_scalars] further loss sums (penalty, pre-activation, auxiliary): part in, total out
  int n_scalars;
  float* losses;        // [8] out: total, reconstruction, sparsity, pre-activation, auxiliary, gradient norm, skipped steps, loss scale
  double inv_bd;        // 1 / (tokens * d_model)
  int phase;            // 0: after the loss kernels; 1: after the gradient-norm pre-pass
  int dynamic_scale;    // fp16: keep the loss scale (halve on overflow, double after growth_interval good steps)
  int growth_interval;
  float max_norm;       // phase 1: clip to this global gradient norm
  Exchange ex;
  int round;
};

__global__ void __launch_bounds__(64) step_control_kernel(const StepControlParams p) {
  __shared__ double vals[kCtlMaxLayers + kMaxScalars + 2];
  __shared__ int timeout;
  const int tid = threadIdx.x;
  const int n = p.phase == 0 ? p.L + p.n_scalars + 1 : 1;
  if (tid == 0) timeout = 0;
  if (p.phase == 0) {
    if (tid < p.L) vals[tid] = p.sq_err[tid];
    else if (tid < p.L + p.n_scalars) vals[tid] = p.scalars[tid - p.L];
    else if (tid == p.L + p.n_scalars)
      vals[tid] = (__float_as_int(p.ctl[SC_FOUND_INF]) != 0 || (p.status != nullptr && *p.status != 0)) ? 1.0 : 0.0;
  } else if (tid == 0) {
    vals[0] = double(p.ctl[SC_GRAD_NORM_SQ]);
  }
  __syncthreads();
  if (p.ex.world > 1) {
    if (!exchange_gather(p.ex, p.round, reinterpret_cast<const uint32_t*>(vals), 2 * n, &timeout)) {
      // a peer did not arrive: this step must not be applied
      if (tid == 0) { p.ctl[SC_SKIP] = __int_as_float(1); p.ctl[SC_CLIP] = 1.f; }
      return;
    }
    if (tid < n) {
      double s = 0.0;
      for (int q = 0; q < p.ex.world; ++q) s += reinterpret_cast<const double*>(exchange_slot(p.ex, p.round, q))[tid];
      vals[tid] = s;
    }
    __syncthreads();
  }
  if (p.phase == 0) {
    if (tid < p.L) p.sq_err[tid] = vals[tid];
    else if (tid < p.L + p.n_scalars) p.scalars[tid - p.L] = vals[tid];
    if (tid != 0) return;
    double sq = 0.0;
    for (int l = 0; l < p.L; ++l) sq += vals[l];
    const float recon = float(sq * p.inv_bd);
    const float sparsity = p.n_scalars > 0 ? float(vals[p.L]) : 0.f;
    const float preact = p.n_scalars > 1 ? float(vals[p.L + 1]) : 0.f;
    const float aux = p.n_scalars > 2 ? float(vals[p.L + 2]) : 0.f;
    const float total = recon + sparsity + preact + aux;
    const bool found = vals[p.L + p.n_scalars] > 0.0 || !(fabsf(total) <= 3.0e38f);
    float scale = p.ctl[SC_LOSS_SCALE];
    if (!(scale > 0.f)) scale = 1.f;
    int skipped = __float_as_int(p.ctl[SC_SKIPPED]);
    if (found) ++skipped;
    p.ctl[SC_SKIP] = __int_as_float(found ? 1 : 0);
    p.ctl[SC_INV_SCALE] = 1.f / scale;
    p.ctl[SC_CLIP] = 1.f;
    p.ctl[SC_GRAD_NORM_SQ] = 0.f;
    p.ctl[SC_FOUND_INF] = __int_as_float(0);
    p.ctl[SC_SKIPPED] = __int_as_float(skipped);
    p.losses[0] = total; p.losses[1] = recon; p.losses[2] = sparsity; p.losses[3] = preact; p.losses[4] = aux;
    p.losses[5] = 0.f; p.losses[6] = float(skipped); p.losses[7] = scale;
    if (p.dynamic_scale) {
      // same policy as torch.amp.GradScaler: back off by 2 on overflow, double after growth_interval clean steps
      int growth = __float_as_int(p.ctl[SC_GROWTH]);
      if (found) { scale *= 0.5f; growth = 0; }
      else if (++growth >= p.growth_interval) { scale *= 2.f; growth = 0; }
      scale = fminf(fmaxf(scale, 1.0f / 65536.f), 1.0e30f);
      p.ctl[SC_LOSS_SCALE] = scale;  // the next step's gradient seed is multiplied with it
      p.ctl[SC_GROWTH] = __int_as_float(growth);
    }
  } else {
    if (tid != 0) return;
    const float norm = sqrtf(float(vals[0]));
    float clip = 1.f;
    if (!(norm <= 3.0e38f)) {  // inf / NaN gradient norm: skip the step
      p.ctl[SC_SKIP] = __int_as_float(1);
      p.ctl[SC_SKIPPED] = __int_as_float(__float_as_int(p.ctl[SC_SKIPPED]) + 1);
    } else if (p.max_norm > 0.f) {
      clip = fminf(1.f, p.max_norm / (norm + 1e-6f));
    }
    p.ctl[SC_CLIP] = clip;
    p.losses[5] = norm;
  }
}

// ---------------------------------------------------------------------------------------- decoder biases
// grad[p, e] = grad_scale / loss_scale * sum_t sel[t, p] * gs_sum[t, e]  (+ extra[p, e]);  one thread per element.
template <typename WT>
__global__ void __launch_bounds__(256) decoder_bias_adam_kernel(WT* __restrict__ bias, float* __restrict__ m, float* __restrict__ v,
                                                                  const float* __restrict__ sel, const float* __restrict__ gs_sum,
                                                                  const float* __restrict__ extra, int n_bias, int L, int d,
                                                                  AdamHyperS h, float* __restrict__ ctl, float norm_weight) {
  const StepScales sc = read_step_ctl(ctl);
  if (sc.skip) return;
  const long long n = 1LL * n_bias * d;
  float nsq = 0.f;
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < n; i += 1LL * gridDim.x * blockDim.x) {
    const int pidx = int(i / d), e = int(i - 1LL * pidx * d);
    float g = 0.f;
    for (int t = 0; t < L; ++t) {
      const float w = __ldg(sel + 1LL * t * n_bias + pidx);
      if (w != 0.f) g = fmaf(w, __ldg(gs_sum + 1LL * t * d + e), g);
    }
    g *= h.grad_scale * sc.inv_scale;
    if (extra != nullptr) g += extra[i];
    if (norm_weight > 0.f) { nsq = fmaf(g, g, nsq); continue; }
    float wv = load_w<WT>(bias + i), mm = m[i], vv = v[i];
    adam_scalar(wv, mm, vv, g * sc.clip, h);
    m[i] = mm; v[i] = vv;
    store_w<WT>(bias + i, wv);
  }
  if (norm_weight > 0.f) {
    __shared__ float red[8];
    nsq = warp_sum(nsq);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = nsq;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int w = 0; w < 8; ++w) tot += red[w];
      if (tot != 0.f && ctl != nullptr) atomicAdd(ctl + SC_GRAD_NORM_SQ, tot * norm_weight);
    }
  }
}

// End of a step: dead-feature counters (+1 per step, reset where the feature fired; reference trainer.py:693-712; not
// subject to the skip flag, the reference counts before its NaN check too) and bias_sum[t, :] = sum_p sel[t, p] bias[p, :]
// for the next step's loss epilogue.  Either part may be left out (null pointers).
template <typename WT>
__global__ void __launch_bounds__(256) step_finish_kernel(long long* __restrict__ counter, unsigned char* __restrict__ fired, int ncols,
                                                            const WT* __restrict__ bias, const float* __restrict__ sel,
                                                            float* __restrict__ bias_sum, int n_bias, int L, int d) {
  const long long stride = 1LL * gridDim.x * blockDim.x;
  const long long tid = blockIdx.x * 1LL * blockDim.x + threadIdx.x;
  if (counter != nullptr)
    for (long long i = tid; i < ncols; i += stride) {
      counter[i] = fired[i] ? 0 : counter[i] + 1;
      fired[i] = 0;
    }
  if (bias_sum != nullptr)
    for (long long i = tid; i < 1LL * L * d; i += stride) {
      const int t = int(i / d), e = int(i - 1LL * t * d);
      float s = 0.f;
      for (int pidx = 0; pidx < n_bias; ++pidx) {
        const float w = __ldg(sel + 1LL * t * n_bias + pidx);
        if (w != 0.f) s = fmaf(w, load_w<WT>(bias + 1LL * pidx * d + e), s);
      }
      bias_sum[i] = s;
    }
}

// ---------------------------------------------------------------------------------------- JumpReLU thresholds
struct ThetaAdamParams {
  void* log_theta;       // [L, pitch] parameter (16-bit or fp32)
  float* m; float* v;    // fp32 moments
  float* theta;          // [L, pitch] fp32: exp(log_theta) of this step in, of the next step out
  const float* S1;       // [L, pitch] window sums of x * G_recon (carry the loss scale)
  const float* S2;       // [L, pitch] window sums of x
  const float* norm2;    // squared decoder norms per decoder-tensor column at this step (before the update)
  const int* feat_off; const float* fcsr_val;  // feature-major CSR of the active entries (values = pre-activations)
  int L, pitch, tying;
  float c_g;             // 2 / (B d)
  float lambda, c, bandwidth;
  AdamHyperS h;
  float* ctl;
  float norm_weight;     // > 0: norm-only pass
  float* grad_out;       // optional [L, pitch]: gradient with respect to log_theta (diagnostics / tests)
};

template <typename WT>
__global__ void __launch_bounds__(256) theta_adam_kernel(const ThetaAdamParams p) {
  const StepScales sc = read_step_ctl(p.ctl);
  if (sc.skip) return;
  const long long n = 1LL * p.L * p.pitch;
  float nsq = 0.f;
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < n; i += 1LL * gridDim.x * blockDim.x) {
    const int l = int(i / p.pitch), f = int(i - 1LL * l * p.pitch);
    const float theta = p.theta[i];
    float g = p.c_g * sc.inv_scale * p.S1[i];
    if (p.lambda > 0.f) {
      // decoder norm of feature (l, f); with per-target tying the feature uses the decoders of all targets >= l
      float n2 = 0.f;
      if (p.tying == 2) { for (int t = l; t < p.L; ++t) n2 += p.norm2[1LL * t * p.pitch + f]; }
      else n2 = p.norm2[i];
      const float nf = sqrtf(fmaxf(n2, 0.f));
      // d penalty / d a = lambda c n sech^2(c n a): constant lambda c n outside the active entries (a = 0), corrected
      // at the active ones that lie inside the window
      float corr = 0.f;
      const int b = __ldg(p.feat_off + i), e = __ldg(p.feat_off + i + 1);
      for (int j = b; j < e; ++j) {
        const float x = __ldg(p.fcsr_val + j);
        if (fabsf(x - theta) <= 0.5f * p.bandwidth) {
          const float th = tanhf(p.c * nf * x);
          corr = fmaf(x, th * th, corr);
        }
      }
      g = fmaf(p.lambda * p.c * nf, p.S2[i] - corr, g);
    }
    const float grad_log = -g / p.bandwidth * theta;  // d / d log(theta) = theta * d / d theta
    if (p.grad_out != nullptr) p.grad_out[i] = grad_log;
    if (p.norm_weight > 0.f) { nsq = fmaf(grad_log, grad_log, nsq); continue; }
    WT* wp = static_cast<WT*>(p.log_theta) + i;
    float wv = load_w<WT>(wp), mm = p.m[i], vv = p.v[i];
    adam_scalar(wv, mm, vv, grad_log * sc.clip, p.h);
    p.m[i] = mm; p.v[i] = vv;
    store_w<WT>(wp, wv);
    p.theta[i] = __expf(load_w<WT>(wp));  // from the stored (rounded) parameter
  }
  if (p.norm_weight > 0.f) {
    __shared__ float red[8];
    nsq = warp_sum(nsq);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = nsq;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int w = 0; w < 8; ++w) tot += red[w];
      if (tot != 0.f && p.ctl != nullptr) atomicAdd(p.ctl + SC_GRAD_NORM_SQ, tot * p.norm_weight);
    }
  }
}

// ---------------------------------------------------------------------------------------- batch normalisation
// Activation batches arrive on the device as stored ([2, L, B, d]: inputs and targets of every layer, bf16 / fp16 /
// fp32); the store's normalisation (x - mean) / std with per-(side, layer, element) statistics, or x * mul, and the
// cast to the training type run as one pass (reference: three eager passes in fp32,
// clt/training/data/manifest_activation_store.py:906-934).  One thread per 8 elements; d % 8 == 0.
template <typename IT>
__device__ __forceinline__ void load8_in(const IT* p, float (&o)[8]);
template <>
__device__ __forceinline__ void load8_in<float>(const float* p, float (&o)[8]) {
  const float4 a = __ldcs(reinterpret_cast<const float4*>(p)), b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <>
__device__ __forceinline__ void load8_in<__nv_bfloat16>(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 q = __ldcs(reinterpret_cast<const uint4*>(p));
  const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) { o[2 * j] = bf16_lo(u[j]); o[2 * j + 1] = bf16_hi(u[j]); }
}
template <>
__device__ __forceinline__ void load8_in<__half>(const __half* p, float (&o)[8]) {
  const uint4 q = __ldcs(reinterpret_cast<const uint4*>(p));
  const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
  for (int j = 0; j < 4; ++j) { const float2 f = __half22float2(h[j]); o[2 * j] = f.x; o[2 * j + 1] = f.y; }
}

template <typename IT>
__global__ void __launch_bounds__(256) normalize_cast_kernel(const IT* __restrict__ in, t16* __restrict__ out, const float* __restrict__ mean,
                                                               const float* __restrict__ inv_std, long long rows, int rows_per_stat, int d, float mul) {
  const int vec_per_row = d / 8;
  const long long nvec = rows * vec_per_row;
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < nvec; i += 1LL * gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int e0 = int(i - r * vec_per_row) * 8;
    float x[8];
    load8_in<IT>(in + r * d + e0, x);
    if (mean != nullptr) {
      const long long so = (r / rows_per_stat) * d + e0;
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = (x[j] - __ldg(mean + so + j)) * __ldg(inv_std + so + j);
    }
    uint4 q;
    q.x = pack_t16x2(x[0] * mul, x[1] * mul); q.y = pack_t16x2(x[2] * mul, x[3] * mul);
    q.z = pack_t16x2(x[4] * mul, x[5] * mul); q.w = pack_t16x2(x[6] * mul, x[7] * mul);
    *reinterpret_cast<uint4*>(out + r * d + e0) = q;
  }
}

// ---------------------------------------------------------------------------------------- L0 calibration histogram
// Layer-wise L0 calibration scales a layer's thresholds by s until the layer's L0 matches a target (reference: a 15-step
// binary search that re-encodes per probe, scripts/convert_batchtopk_to_jumprelu.py:649-763).  L0(s) = #{x >= s * theta}
// for every candidate s comes from one pass: an element with ratio r = x / theta satisfies the first k scales of the
// ascending vector `scales` (k = number of scales <= r); hist[k] counts them.  Most elements lie below scales[0] and
// cost one compare; the others do a binary search in shared memory.
constexpr int kMaxScales = 1024;
__global__ void __launch_bounds__(256) scale_histogram_kernel(const t16* __restrict__ x, const float* __restrict__ theta,
                                                                const float* __restrict__ scales, int n_scales,
                                                                unsigned long long* __restrict__ hist, int B, int F, long long ld) {
  __shared__ float sc[kMaxScales];
  __shared__ unsigned int sh[kMaxScales + 1];
  for (int i = threadIdx.x; i < n_scales; i += blockDim.x) sc[i] = scales[i];
  for (int i = threadIdx.x; i <= n_scales; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const float s0 = sc[0];
  const long long n = 1LL * B * F;
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < n; i += 1LL * gridDim.x * blockDim.x) {
    const int b = int(i / F), f = int(i - 1LL * b * F);
    const float r = __fdiv_rn(t16_to_float(x[1LL * b * ld + f]), fmaxf(__ldg(theta + f), 1e-30f));
    if (!(r >= s0)) continue;
    int lo = 0, hi = n_scales;  // number of scales <= r, in [1, n_scales]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (sc[mid] <= r) lo = mid; else hi = mid;
    }
    atomicAdd(&sh[lo + 1], 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i <= n_scales; i += blockDim.x)
    if (sh[i]) atomicAdd(&hist[i], (unsigned long long)sh[i]);
}

// theta = exp(log_theta) (set-up, after a checkpoint load)
template <typename WT>
__global__ void __launch_bounds__(256) theta_exp_kernel(const WT* __restrict__ log_theta, float* __restrict__ theta, long long n) {
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < n; i += 1LL * gridDim.x * blockDim.x)
    theta[i] = __expf(load_w<WT>(log_theta + i));
}

}  // namespace clt

using namespace clt;

struct CltAdamHyper {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;
  int decoupled;
  float grad_scale;
  unsigned int sr_seed;
  unsigned int moment_seed;
};
static AdamHyperS to_hyper_s(const CltAdamHyper& c) {
  AdamHyperS h;
  h.lr = c.lr; h.beta1 = c.beta1; h.beta2 = c.beta2; h.eps = c.eps; h.weight_decay = c.weight_decay;
  h.bc1 = c.bc1; h.bc2 = c.bc2; h.decoupled = c.decoupled; h.grad_scale = c.grad_scale; h.sr_seed = c.sr_seed; h.moment_seed = c.moment_seed;
  return h;
}

struct CltExchangeArgs {
  int world;
  int rank;
  void* data[8];
  void* flags[8];
  int slot_elems;
  unsigned int seq;
};

#if !CLT_T16_IS_HALF
struct CltStepControlArgs {
  float* ctl; const int* status; double* sq_err; int L; double* scalars; int n_scalars; float* losses; double inv_bd;
  int phase, dynamic_scale, growth_interval; float max_norm; int round;
};

extern "C" int clt_step_control(const CltStepControlArgs* a, const CltExchangeArgs* exa, cudaStream_t st) {
  if (a->L > kCtlMaxLayers || a->n_scalars > kMaxScalars || a->ctl == nullptr || a->losses == nullptr) return -1;
  StepControlParams p;
  p.ctl = a->ctl; p.status = a->status; p.sq_err = a->sq_err; p.L = a->L; p.scalars = a->scalars; p.n_scalars = a->n_scalars;
  p.losses = a->losses; p.inv_bd = a->inv_bd; p.phase = a->phase; p.dynamic_scale = a->dynamic_scale;
  p.growth_interval = a->growth_interval; p.max_norm = a->max_norm; p.round = a->round;
  p.ex.world = exa ? exa->world : 1; p.ex.rank = exa ? exa->rank : 0; p.ex.slot_elems = exa ? exa->slot_elems : 0; p.ex.seq = exa ? exa->seq : 0;
  for (int i = 0; i < kMaxPeers; ++i) {
    p.ex.peers[i] = exa ? static_cast<uint32_t*>(exa->data[i]) : nullptr;
    p.ex.flags[i] = exa ? static_cast<uint32_t*>(exa->flags[i]) : nullptr;
  }
  if (exa && 2 * (a->L + a->n_scalars + 1) > exa->slot_elems) return -1;
  step_control_kernel<<<1, 64, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
#endif

extern "C" int CLT_FN(clt_decoder_bias_adam)(void* bias, float* m, float* v, const float* sel, const float* gs_sum, const float* extra,
                                             int n_bias, int L, int d, int weights_16, const CltAdamHyper* h, float* ctl,
                                             float norm_weight, cudaStream_t st) {
  const long long n = 1LL * n_bias * d;
  if (n <= 0) return 0;
  const int grid = int((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
  if (weights_16) decoder_bias_adam_kernel<t16><<<grid, 256, 0, st>>>(static_cast<t16*>(bias), m, v, sel, gs_sum, extra, n_bias, L, d, to_hyper_s(*h), ctl, norm_weight);
  else decoder_bias_adam_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(bias), m, v, sel, gs_sum, extra, n_bias, L, d, to_hyper_s(*h), ctl, norm_weight);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int CLT_FN(clt_step_finish)(long long* counter, unsigned char* fired, int ncols, const void* bias, const float* sel,
                                       float* bias_sum, int n_bias, int L, int d, int weights_16, cudaStream_t st) {
  long long work = counter != nullptr ? ncols : 0;
  if (bias_sum != nullptr && 1LL * L * d > work) work = 1LL * L * d;
  if (work <= 0) return 0;
  const int grid = int((work + 255) / 256 < 1184 ? (work + 255) / 256 : 1184);
  if (weights_16) step_finish_kernel<t16><<<grid, 256, 0, st>>>(counter, fired, ncols, static_cast<const t16*>(bias), sel, bias_sum, n_bias, L, d);
  else step_finish_kernel<float><<<grid, 256, 0, st>>>(counter, fired, ncols, static_cast<const float*>(bias), sel, bias_sum, n_bias, L, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

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

extern "C" int CLT_FN(clt_theta_adam)(const CltThetaAdamArgs* a, cudaStream_t st) {
  ThetaAdamParams p;
  p.log_theta = a->log_theta; p.m = a->m; p.v = a->v; p.theta = a->theta; p.S1 = a->S1; p.S2 = a->S2; p.norm2 = a->norm2;
  p.feat_off = a->feat_off; p.fcsr_val = a->fcsr_val; p.L = a->L; p.pitch = a->pitch; p.tying = a->tying;
  p.c_g = a->c_g; p.lambda = a->lambda; p.c = a->c; p.bandwidth = a->bandwidth; p.h = to_hyper_s(a->h); p.ctl = a->ctl;
  p.norm_weight = a->norm_weight; p.grad_out = a->grad_out;
  const long long n = 1LL * a->L * a->pitch;
  if (n <= 0) return 0;
  const int grid = int((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
  if (a->weights_16) theta_adam_kernel<t16><<<grid, 256, 0, st>>>(p);
  else theta_adam_kernel<float><<<grid, 256, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int CLT_FN(clt_theta_exp)(const void* log_theta, float* theta, long long n, int weights_16, cudaStream_t st) {
  if (n <= 0) return 0;
  const int grid = int((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
  if (weights_16) theta_exp_kernel<t16><<<grid, 256, 0, st>>>(static_cast<const t16*>(log_theta), theta, n);
  else theta_exp_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(log_theta), theta, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// in_type: 0 fp32, 1 bf16, 2 fp16.  mean / inv_std: [rows / rows_per_stat, d] or null (only the multiplier applies).
extern "C" int CLT_FN(clt_normalize_cast)(const void* in, int in_type, void* out, const float* mean, const float* inv_std, long long rows,
                                          int rows_per_stat, int d, float mul, cudaStream_t st) {
  if (d % 8 != 0 || rows <= 0 || rows_per_stat <= 0) return -1;
  const long long nvec = rows * (d / 8);
  const int grid = int((nvec + 255) / 256 < 148 * 16 ? (nvec + 255) / 256 : 148 * 16);
  t16* o = static_cast<t16*>(out);
  if (in_type == 0) normalize_cast_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(in), o, mean, inv_std, rows, rows_per_stat, d, mul);
  else if (in_type == 1) normalize_cast_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in), o, mean, inv_std, rows, rows_per_stat, d, mul);
  else if (in_type == 2) normalize_cast_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(in), o, mean, inv_std, rows, rows_per_stat, d, mul);
  else return -1;
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// hist: [n_scales + 1] uint64, zeroed by the caller; hist[k] = number of elements that satisfy exactly the first k scales.
extern "C" int CLT_FN(clt_scale_histogram)(const void* x, const float* theta, const float* scales, int n_scales, unsigned long long* hist,
                                           int B, int F, long long ld, cudaStream_t st) {
  if (n_scales < 1 || n_scales > kMaxScales || B <= 0 || F <= 0) return -1;
  const long long n = 1LL * B * F;
  const int grid = int((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  scale_histogram_kernel<<<grid, 256, 0, st>>>(static_cast<const t16*>(x), theta, scales, n_scales, hist, B, F, ld);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
