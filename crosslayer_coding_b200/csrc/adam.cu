// Backward + optimizer in one pass over the parameters (sm_100a).
//
// The reference materialises dense gradients for every decoder and encoder matrix with autograd GEMMs and
// then runs torch.optim.Adam/AdamW over them (clt/training/trainer.py:751-783).  With a (Batch)TopK or
// JumpReLU code the gradients are row-sparse sums over the active (token, feature) entries, so this file
// never writes a gradient tensor: one warp per parameter row gathers the few rows of the gradient seed
// (decoder) or of the layer input (encoder) that touch its feature, forms the row gradient in registers,
// and applies the Adam update to (w, m, v) in the same pass.  The decoder pass also produces
//   * dL/da for every entry (dot of the seed row with the *old* weight row), consumed by the encoder pass,
//   * the squared decoder norm of every feature after the update (used by the sparsity penalty next step).
//
// Row layout: decoder tensor s is [F, R_s, d] (feature-major), encoder is [L, F, d]; bf16 weights with
// fp32 moments (or fp32 weights).  d must be a multiple of 8.
#include "common.cuh"

namespace clt {

constexpr int kMaxLayersA = 32;

struct AdamHyper {
  float lr, beta1, beta2, eps, weight_decay;
  float bc1, bc2;        // 1 - beta^step
  int decoupled;         // 1: AdamW, 0: Adam (decay folded into the gradient)
  float grad_scale;      // multiplies the gathered gradient (e.g. 2/(B*d), 1/loss_scale, clip factor)
  unsigned int sr_seed;  // stochastic rounding seed; 0 = round to nearest
  unsigned int moment_seed;  // seed for the stochastic rounding of bf16 moments (changes every step)
};

__device__ __forceinline__ uint32_t hash32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}
// fp32 -> 16-bit weight; a non-zero seed asks for stochastic rounding (bf16 builds; fp16 rounds to nearest)
__device__ __forceinline__ t16 to_bf16(float v, unsigned int seed, unsigned long long idx) {
#if CLT_T16_IS_HALF
  return float_to_t16(v);
#else
  if (seed == 0) return float_to_t16(v);
  const uint32_t u = __float_as_uint(v);
  if ((u & 0x7F800000u) == 0x7F800000u) return float_to_t16(v);
  const uint32_t r = hash32(uint32_t(idx) ^ hash32(seed + uint32_t(idx >> 32))) & 0xFFFFu;
  const uint32_t t = (u + r) & 0xFFFF0000u;
  return float_to_t16(__uint_as_float(t));
#endif
}

// Hyper-parameters pre-combined once per thread so the per-element update is 11 instructions.
struct HyperRegs {
  float decay;   // 1 - lr * wd (AdamW) or 1
  float wd_l2;   // wd folded into the gradient (Adam) or 0
  float omb1, omb2;
  float step;    // lr / (1 - beta1^t)
  float isb2;    // 1 / sqrt(1 - beta2^t)
  float eps;
  float gscale;
};
__device__ __forceinline__ HyperRegs make_regs(const AdamHyper& h) {
  HyperRegs r;
  r.decay = h.decoupled ? 1.f - h.lr * h.weight_decay : 1.f;
  r.wd_l2 = h.decoupled ? 0.f : h.weight_decay;
  r.omb1 = 1.f - h.beta1;
  r.omb2 = 1.f - h.beta2;
  r.step = h.lr / h.bc1;
  r.isb2 = rsqrtf(h.bc2);
  r.eps = h.eps;
  r.gscale = h.grad_scale;
  return r;
}
// m <- m + (1-b1)(g - m);  v <- v + (1-b2)(g^2 - v);  w <- decay*w - step * m / (sqrt(v)/sqrt(bc2) + eps)
__device__ __forceinline__ void adam1(float& w, float& m, float& v, float g, const HyperRegs& r) {
  g = fmaf(r.wd_l2, w, g);
  w *= r.decay;
  m = fmaf(r.omb1, g - m, m);
  v = fmaf(r.omb2, fmaf(g, g, -v), v);
  const float denom = fmaf(sqrtf(v), r.isb2, r.eps);
  w = fmaf(-r.step, __fdividef(m, denom), w);
}
__device__ __forceinline__ void adam_update8(float (&w)[8], float (&m)[8], float (&v)[8], const float (&g)[8], const AdamHyper& h) {
  const HyperRegs r = make_regs(h);
#pragma unroll
  for (int i = 0; i < 8; ++i) adam1(w[i], m[i], v[i], g[i], r);
}
// 8 fp32 -> 8 bf16 (one 16-byte vector); SR selects stochastic rounding with a counter-based hash.
template <bool SR>
__device__ __forceinline__ uint4 pack8_bf16(const float (&o)[8], unsigned int seed, unsigned int idx) {
  uint4 q;
  if (!SR || CLT_T16_IS_HALF) {
    q.x = pack_t16x2(o[0], o[1]); q.y = pack_t16x2(o[2], o[3]);
    q.z = pack_t16x2(o[4], o[5]); q.w = pack_t16x2(o[6], o[7]);
  } else {
    uint32_t h[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t u = __float_as_uint(o[k]);
      const uint32_t rnd = hash32((idx + k) ^ seed) & 0xFFFFu;
      h[k] = ((u & 0x7F800000u) == 0x7F800000u) ? (u >> 16) : ((u + rnd) >> 16);
    }
    q.x = h[0] | (h[1] << 16); q.y = h[2] | (h[3] << 16); q.z = h[4] | (h[5] << 16); q.w = h[6] | (h[7] << 16);
  }
  return q;
}

__device__ __forceinline__ void unpack8(const uint4& q, float (&o)[8]) {
  const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) { o[2 * j] = t16_lo(u[j]); o[2 * j + 1] = t16_hi(u[j]); }
}
__device__ __forceinline__ void load8f(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void store8f(float* p, const float (&o)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(o[4], o[5], o[6], o[7]);
}

template <typename WT>
__device__ __forceinline__ void load_w8(const WT* p, float (&o)[8]);
template <>
__device__ __forceinline__ void load_w8<t16>(const t16* p, float (&o)[8]) {
  unpack8(*reinterpret_cast<const uint4*>(p), o);
}
template <>
__device__ __forceinline__ void load_w8<float>(const float* p, float (&o)[8]) { load8f(p, o); }

template <typename WT>
__device__ __forceinline__ void store_w8(WT* p, const float (&o)[8], unsigned int seed, unsigned long long idx);
template <>
__device__ __forceinline__ void store_w8<t16>(t16* p, const float (&o)[8], unsigned int seed, unsigned long long idx) {
  t16 b[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) b[i] = to_bf16(o[i], seed, idx + i);
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(b);
}
template <>
__device__ __forceinline__ void store_w8<float>(float* p, const float (&o)[8], unsigned int, unsigned long long) { store8f(p, o); }

// ------------------------------------------------------------------ decoder rows
struct DecAdamParams {
  void* w[kMaxLayersA];        // tensor i: [F_pitch, rows_i, d]
  float* m[kMaxLayersA];
  float* v[kMaxLayersA];
  long long row_start[kMaxLayersA + 1];  // prefix of F_pitch * rows_i over tensors
  int rows[kMaxLayersA];
  int ntensors;
  int L, B, d, F_pitch, tying;
  const int* feat_off;         // [L * F_pitch + 1] feature-major CSR
  const int* fcsr_tok;
  const float* fcsr_val;
  const t16* gs;     // [L, B, d] gradient seed
  float* grad_a;               // [nnz] dL/da per CSR slot (atomicAdd; zeroed by the caller); may be null
  const float* pen_coef;       // optional [L * F_pitch]: coefficient of w in the row gradient (sparsity penalty via norms)
  float* norm2_out;            // optional [L * F_pitch]: sum of squares of the updated rows (atomicAdd; zeroed by caller)
  const float* feat_offset;    // tied decoders: optional [L, F_pitch] affine applied to the activation
  const float* feat_scale;
  float* d_feat_offset;        // optional [L, F_pitch] gradient accumulators of the affine terms (zeroed by the caller); filled in
  float* d_feat_scale;         // the pass that also writes grad_a
  int moments_bf16;            // bulk pipeline only: m / v hold bf16 (stochastically rounded) instead of fp32
  const float* dgrad_row0;     // optional [ntensors, F_pitch, d] fp32: extra gradient of every feature's first row
  // optional compact extras (auxiliary loss on dead features): extra_idx[col] = row of extra_rows, or -1
  const int* extra_idx;
  const float* extra_rows;     // [n_extra, d] fp32, added to the feature's first row
  const float* ctl;            // optional step control block (skip flag, 1 / loss scale, clip coefficient)
  int use_inv_scale;           // the "gradient seed" operand carries the loss scale (decoder: yes; encoder inputs: no)
  float* norm_sq_out;          // norm-only pass: squared norm of all row gradients is added here
  AdamHyper h;
};

// Extra gradient of a feature's first row (dense buffer or compact rows through an index), or null.
__device__ __forceinline__ const float* extra_row_ptr(const DecAdamParams& p, int col) {
  if (p.dgrad_row0 != nullptr) return p.dgrad_row0 + 1LL * col * p.d;
  if (p.extra_idx != nullptr) {
    const int i = __ldg(p.extra_idx + col);
    if (i >= 0) return p.extra_rows + 1LL * i * p.d;
  }
  return nullptr;
}
// Block-wide sum of `v` added to *out (one atomic per CTA); every thread of the CTA calls it.
__device__ __forceinline__ void block_add(float v, float* out) {
  __shared__ float red_s[32];
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red_s[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < int((blockDim.x + 31) >> 5); ++w) tot += red_s[w];
    if (tot != 0.f && out != nullptr) atomicAdd(out, tot);
  }
}

__device__ __forceinline__ void f4x2_to8(const float4& a, const float4& b, float (&o)[8]) {
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void stream_store8f(float* p, const float (&o)[8]) {
  __stcs(reinterpret_cast<float4*>(p), make_float4(o[0], o[1], o[2], o[3]));
  __stcs(reinterpret_cast<float4*>(p) + 1, make_float4(o[4], o[5], o[6], o[7]));
}
template <typename WT>
struct WVec;
template <>
struct WVec<t16> {
  uint4 q;
  __device__ __forceinline__ void load(const t16* p) { q = __ldcs(reinterpret_cast<const uint4*>(p)); }
  __device__ __forceinline__ void get(float (&o)[8]) const { unpack8(q, o); }
};
template <>
struct WVec<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = __ldcs(reinterpret_cast<const float4*>(p));
    b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
  }
  __device__ __forceinline__ void get(float (&o)[8]) const { f4x2_to8(a, b, o); }
};

template <typename WT>
struct RowRegs {
  WVec<WT> w;
  float4 m0, m1, v0, v1;
  __device__ __forceinline__ void load(const WT* wp, const float* mp, const float* vp) {
    w.load(wp);
    m0 = __ldcs(reinterpret_cast<const float4*>(mp)); m1 = __ldcs(reinterpret_cast<const float4*>(mp) + 1);
    v0 = __ldcs(reinterpret_cast<const float4*>(vp)); v1 = __ldcs(reinterpret_cast<const float4*>(vp) + 1);
  }
};

// Untied decoders, the flagship path.  Work item = (source feature, 256-element segment): one warp, 8
// elements per lane, walking the feature's R = L - s target rows with the next row's (w, m, v) already in
// flight.  The first four entries of the feature stay in registers: their activation, token and the
// partial dot products for dL/da, which are reduced once per item instead of once per row.
// NORM_ONLY: the gradient-norm pre-pass of gradient clipping.  Nothing is updated: features without entries (and
// without an extra row) are skipped, the row gradients of the others are formed as in the update, their squares
// are summed into p.norm_sq_out and dL/da is written to p.grad_a.
template <typename WT, bool SR, bool NORM_ONLY>
__global__ void __launch_bounds__(256, 2) decoder_rows_adam_untied_kernel(const DecAdamParams p) {
  const int lane = threadIdx.x & 31;
  const int warp_global = int((blockIdx.x * 1LL * blockDim.x + threadIdx.x) >> 5);
  const int nwarps = int((gridDim.x * 1LL * blockDim.x) >> 5);
  const HyperRegs hr = make_regs(p.h);
  const StepScales sc = read_step_ctl(p.ctl);
  if (sc.skip) return;
  const float gsc = hr.gscale * (p.use_inv_scale ? sc.inv_scale : 1.f);
  float nsq = 0.f;
  const int d = p.d, B = p.B, Fp = p.F_pitch;
  const int nseg = (d + 255) / 256;
  const int per_tensor = Fp * nseg;
  const int total_items = per_tensor * p.ntensors;
  const t16* __restrict__ gs = p.gs;
  for (int item = warp_global; item < total_items; item += nwarps) {
    const int ti = item / per_tensor;
    const int rem = item - ti * per_tensor;
    const int f = rem / nseg;
    const int seg = rem - f * nseg;
    const int R = p.rows[ti];
    const int e0 = seg * 256 + lane * 8;
    const bool act = e0 < d;
    const long long row0 = 1LL * f * R;
    WT* wbase = static_cast<WT*>(p.w[ti]) + row0 * d + e0;
    float* mbase = p.m[ti] + row0 * d + e0;
    float* vbase = p.v[ti] + row0 * d + e0;
    const int col = ti * Fp + f;
    const int b = __ldg(p.feat_off + col), e = __ldg(p.feat_off + col + 1);
    const int ne = e - b;
    const float* xrow = extra_row_ptr(p, col);
    if (NORM_ONLY && ne == 0 && xrow == nullptr) continue;
    RowRegs<WT> cur, nxt;
    if (act) { if (NORM_ONLY) cur.w.load(wbase); else cur.load(wbase, mbase, vbase); }
    int tok4[4];
    float a4[4], dacc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      tok4[j] = j < ne ? __ldg(p.fcsr_tok + b + j) : 0;
      a4[j] = j < ne ? __ldg(p.fcsr_val + b + j) : 0.f;
      dacc[j] = 0.f;
    }
    const float pc = p.pen_coef ? p.pen_coef[col] : 0.f;
    float norm2 = 0.f;
    const unsigned int idx_base = (unsigned int)((p.row_start[ti] + row0) * d + e0);
    for (int r = 0; r < R; ++r) {
      const long long roff = 1LL * r * d;
      if (act && r + 1 < R) { if (NORM_ONLY) nxt.w.load(wbase + roff + d); else nxt.load(wbase + roff + d, mbase + roff + d, vbase + roff + d); }
      float w[8], g[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) { g[i] = 0.f; w[i] = 0.f; }
      if (act) {
        cur.w.get(w);
        const t16* gs_t = gs + 1LL * (ti + r) * B * d + e0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j < ne) {
            float gv[8];
            unpack8(__ldg(reinterpret_cast<const uint4*>(gs_t + 1LL * tok4[j] * d)), gv);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              g[k] = fmaf(a4[j], gv[k], g[k]);
              dacc[j] = fmaf(gv[k], w[k], dacc[j]);
            }
          }
        }
      }
      for (int i = b + 4; i < e; ++i) {  // rare: features with more than four entries
        float dot = 0.f;
        if (act) {
          const float a = __ldg(p.fcsr_val + i);
          float gv[8];
          unpack8(__ldg(reinterpret_cast<const uint4*>(gs + (1LL * (ti + r) * B + __ldg(p.fcsr_tok + i)) * d + e0)), gv);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            g[k] = fmaf(a, gv[k], g[k]);
            dot = fmaf(gv[k], w[k], dot);
          }
        }
        if (p.grad_a != nullptr) {
          dot = warp_sum(dot);
          if (lane == 0 && dot != 0.f) atomicAdd(&p.grad_a[i], dot * gsc);
        }
      }
      if (act) {
        float dg0[8];
        const bool extra = r == 0 && xrow != nullptr;
        if (extra) load8f(xrow + e0, dg0);
        if (NORM_ONLY) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            float gk = fmaf(pc, w[k], g[k] * gsc);
            if (extra) gk += dg0[k];
            nsq = fmaf(gk, gk, nsq);
          }
        } else {
          float m[8], v[8];
          f4x2_to8(cur.m0, cur.m1, m);
          f4x2_to8(cur.v0, cur.v1, v);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            float gk = fmaf(pc, w[k], g[k] * gsc);
            if (extra) gk += dg0[k];
            adam1(w[k], m[k], v[k], gk * sc.clip, hr);
            norm2 = fmaf(w[k], w[k], norm2);
          }
          stream_store8f(mbase + roff, m);
          stream_store8f(vbase + roff, v);
          if (sizeof(WT) == 2) __stcs(reinterpret_cast<uint4*>(wbase + roff), pack8_bf16<SR>(w, p.h.sr_seed, idx_base + (unsigned int)roff));
          else stream_store8f(reinterpret_cast<float*>(wbase + roff), w);
        }
      }
      cur = nxt;
    }
    if (p.grad_a != nullptr) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j < ne) {
          const float sdot = warp_sum(dacc[j]);
          if (lane == 0 && sdot != 0.f) atomicAdd(&p.grad_a[b + j], sdot * gsc);
        }
      }
    }
    if (!NORM_ONLY && p.norm2_out != nullptr) {
      norm2 = warp_sum(norm2);
      if (lane == 0) atomicAdd(&p.norm2_out[col], norm2);
    }
  }
  if (NORM_ONLY) block_add(nsq, p.norm_sq_out);
}

// ---------------------------------------------------------------- untied decoders, bulk-copy pipeline
// The update streams every decoder row once: (w, m, v) in, (w, m, v) out, 20 bytes per element with bf16
// weights, so the kernel is a copy with some arithmetic in the middle.  A producer thread per CTA moves
// whole rows between global and shared memory with 1-D bulk copies (cp.async.bulk, no multicast): row in
// (w, m, v and the gradient-seed rows of the feature's first four entries) -> consumers update the row in
// place in shared memory -> row out.  The ring keeps several rows per CTA in flight in both directions and
// the consumers never wait on a global load, except for the rare feature with more than four entries.
// Every mbarrier wait is bounded; a timeout sets the status word and drains the copies in flight.
constexpr int kAdamStages = 4;  // at most; rows above 24 KB per stage run with three so that two CTAs fit an SM
constexpr int kAdamSlots = 4;  // gradient-seed rows per stage

struct AdamStageHdr {  // 64 bytes in front of every stage, written by the producer before it arms the barrier
  int ne;      // entries of the feature
  int b;       // start of the feature in the CSR arrays
  int col;     // ti * F_pitch + f
  int ti;
  int r;       // row inside the feature
  int R;
  long long elem_off;  // element offset of the row inside its tensor
  float a[kAdamSlots];
  int pad[4];
};
static_assert(sizeof(AdamStageHdr) == 64, "stage header is 64 bytes");

struct AdamBulkShared {
  uint64_t full[kAdamStages];
  uint64_t done[kAdamStages];
  int abort_flag;
};

struct FeatMeta {
  int b, e;
  int tok[kAdamSlots];
  float a[kAdamSlots];
};

// Vector access to EPT (4 or 8) consecutive elements of a row held in shared memory.
template <int EPT>
__device__ __forceinline__ void ldf(const float* p, float (&o)[EPT]) {
#pragma unroll
  for (int i = 0; i < EPT; i += 4) {
    const float4 a = *reinterpret_cast<const float4*>(p + i);
    o[i] = a.x; o[i + 1] = a.y; o[i + 2] = a.z; o[i + 3] = a.w;
  }
}
template <int EPT>
__device__ __forceinline__ void stf(float* p, const float (&o)[EPT]) {
#pragma unroll
  for (int i = 0; i < EPT; i += 4) *reinterpret_cast<float4*>(p + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
}
template <int EPT>
__device__ __forceinline__ void ldbf(const t16* p, float (&o)[EPT]) {
#pragma unroll
  for (int i = 0; i < EPT; i += 4) {
    const uint2 q = *reinterpret_cast<const uint2*>(p + i);
    o[i] = t16_lo(q.x); o[i + 1] = t16_hi(q.x); o[i + 2] = t16_lo(q.y); o[i + 3] = t16_hi(q.y);
  }
}
template <int EPT>
__device__ __forceinline__ void ldbf_global(const t16* p, float (&o)[EPT]) {
#pragma unroll
  for (int i = 0; i < EPT; i += 4) {
    const uint2 q = __ldg(reinterpret_cast<const uint2*>(p + i));
    o[i] = t16_lo(q.x); o[i + 1] = t16_hi(q.x); o[i + 2] = t16_lo(q.y); o[i + 3] = t16_hi(q.y);
  }
}
template <int EPT, bool SR>
__device__ __forceinline__ void stbf(t16* p, const float (&o)[EPT], unsigned int seed, unsigned int idx) {
#pragma unroll
  for (int i = 0; i < EPT; i += 4) {
    uint2 q;
    if (!SR || CLT_T16_IS_HALF) {
      q.x = pack_t16x2(o[i], o[i + 1]); q.y = pack_t16x2(o[i + 2], o[i + 3]);
    } else {
      uint32_t h[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t u = __float_as_uint(o[i + k]);
        const uint32_t rnd = hash32((idx + i + k) ^ seed) & 0xFFFFu;
        h[k] = ((u & 0x7F800000u) == 0x7F800000u) ? (u >> 16) : ((u + rnd) >> 16);
      }
      q.x = h[0] | (h[1] << 16); q.y = h[2] | (h[3] << 16);
    }
    *reinterpret_cast<uint2*>(p + i) = q;
  }
}

template <typename WT, bool SR, int EPT, typename MT>
__global__ void __launch_bounds__(288) decoder_rows_adam_bulk_kernel(const DecAdamParams p, int gthreads, int stage_bytes, int ns, int* status) {
  extern __shared__ __align__(128) uint8_t smem_raw_adam[];  // bulk copies need 16-byte alignment only
  uint8_t* ring = smem_raw_adam;
  AdamBulkShared* sh = reinterpret_cast<AdamBulkShared*>(ring + size_t(ns) * stage_bytes);
  const int d = p.d, B = p.B, Fp = p.F_pitch;
  const int nconsumer = gthreads;
  const int tid = threadIdx.x;
  const StepScales sc = read_step_ctl(p.ctl);
  if (sc.skip) return;  // the whole grid sees the same flag: a skipped step touches nothing
  const int nf = (Fp - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x);  // features of this CTA per tensor
  long long n_rows = 0;
  for (int ti = 0; ti < p.ntensors; ++ti) n_rows += 1LL * (nf > 0 ? nf : 0) * p.rows[ti];
  const int n = int(n_rows);
  const uint32_t w_bytes = uint32_t(d) * sizeof(WT), mv_bytes = uint32_t(d) * sizeof(MT), gs_bytes = uint32_t(d) * 2u;
  const uint32_t off_w = 64, off_m = off_w + w_bytes, off_v = off_m + mv_bytes, off_gs = off_v + mv_bytes;
  if (tid == 0) {
    for (int s = 0; s < ns; ++s) {
      mbar_init(&sh->full[s], 1);
      mbar_init(&sh->done[s], nconsumer / 32);
    }
    sh->abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  volatile int* abort_flag = &sh->abort_flag;

  if (tid == nconsumer) {
    // ------------------------------------------------------------------ producer / store issuer
    const int n_feat = nf * p.ntensors;
    auto col_of = [&](int k) { const int ti = k / nf; return ti * Fp + int(blockIdx.x) + (k - ti * nf) * int(gridDim.x); };
    auto load_offsets = [&](int k, FeatMeta& mt) {
      if (k < n_feat) { const int c = col_of(k); mt.b = __ldg(p.feat_off + c); mt.e = __ldg(p.feat_off + c + 1); }
      else { mt.b = 0; mt.e = 0; }
    };
    auto load_entries = [&](FeatMeta& mt) {
#pragma unroll
      for (int j = 0; j < kAdamSlots; ++j) {
        const bool in = mt.b + j < mt.e;
        mt.tok[j] = in ? __ldg(p.fcsr_tok + mt.b + j) : 0;
        mt.a[j] = in ? __ldg(p.fcsr_val + mt.b + j) : 0.f;
        if (!clt_in_bounds(mt.tok[j], B, status, 201)) { mt.tok[j] = 0; mt.a[j] = 0.f; }  // debug build: token index from the CSR
      }
    };
    // rows are touched once per step, the gradient seed is re-read by every feature: keep the latter in L2
    const uint64_t pol_stream = l2_policy_evict_first();
    const uint64_t pol_keep = l2_policy_evict_last();
    FeatMeta cur, nxt, nn;
    load_offsets(0, cur); load_entries(cur);
    load_offsets(1, nxt);
    int k = 0, r = 0;             // feature / row whose loads are issued next
    int ti = 0, R = n_feat > 0 ? p.rows[0] : 0;
    int f = int(blockIdx.x);
    bool fresh = true;            // first row of a feature: start the prefetch of the following ones
    auto issue_loads = [&](int i) {
      if (fresh) {
        load_entries(nxt);        // offsets of k + 1 were requested one feature ago
        load_offsets(k + 2, nn);
        fresh = false;
      }
      const int st = i % ns;
      uint8_t* stage = ring + size_t(st) * stage_bytes;
      AdamStageHdr* h = reinterpret_cast<AdamStageHdr*>(stage);
      const int ne = cur.e - cur.b;
      const long long elem_off = (1LL * f * R + r) * d;
      h->ne = ne; h->b = cur.b; h->col = ti * Fp + f; h->ti = ti; h->r = r; h->R = R; h->elem_off = elem_off;
#pragma unroll
      for (int j = 0; j < kAdamSlots; ++j) h->a[j] = cur.a[j];
      const int nslot = ne < kAdamSlots ? ne : kAdamSlots;
      mbar_expect_tx(&sh->full[st], w_bytes + 2u * mv_bytes + uint32_t(nslot) * gs_bytes);
      bulk_load_1d_hint(stage + off_w, static_cast<const WT*>(p.w[ti]) + elem_off, w_bytes, &sh->full[st], pol_stream);
      bulk_load_1d_hint(stage + off_m, reinterpret_cast<const MT*>(p.m[ti]) + elem_off, mv_bytes, &sh->full[st], pol_stream);
      bulk_load_1d_hint(stage + off_v, reinterpret_cast<const MT*>(p.v[ti]) + elem_off, mv_bytes, &sh->full[st], pol_stream);
      const t16* gs_t = p.gs + 1LL * (ti + r) * B * d;
#pragma unroll
      for (int j = 0; j < kAdamSlots; ++j)
        if (j < nslot) bulk_load_1d_hint(stage + off_gs + j * gs_bytes, gs_t + 1LL * cur.tok[j] * d, gs_bytes, &sh->full[st], pol_keep);
      // advance to the next row
      if (++r == R) {
        r = 0; ++k;
        cur = nxt; nxt.b = nn.b; nxt.e = nn.e;
        fresh = true;
        if (k < n_feat) {
          const int nti = k / nf;
          if (nti != ti) { ti = nti; R = p.rows[ti]; }
          f = int(blockIdx.x) + (k - ti * nf) * int(gridDim.x);
        }
      }
    };
    int issued = 0;
    for (; issued < n && issued < ns; ++issued) issue_loads(issued);
    int i = 0;
    for (; i < n; ++i) {
      const int st = i % ns;
      if (!mbar_wait(&sh->done[st], (i / ns) & 1, abort_flag)) break;
      uint8_t* stage = ring + size_t(st) * stage_bytes;
      const AdamStageHdr* h = reinterpret_cast<const AdamStageHdr*>(stage);
      const int sti = h->ti;
      const long long eo = h->elem_off;
      bulk_store_1d_hint(static_cast<WT*>(p.w[sti]) + eo, stage + off_w, w_bytes, pol_stream);
      bulk_store_1d_hint(reinterpret_cast<MT*>(p.m[sti]) + eo, stage + off_m, mv_bytes, pol_stream);
      bulk_store_1d_hint(reinterpret_cast<MT*>(p.v[sti]) + eo, stage + off_v, mv_bytes, pol_stream);
      bulk_commit();
      if (i >= 1 && issued < n) {
        bulk_wait_read<1>();  // the stores of row i - 1 have read their stage: it can be refilled
        issue_loads(issued);
        ++issued;
      }
    }
    bulk_wait_all();
    if (*abort_flag) {
      // rows whose loads were issued but never consumed: give them a bounded chance to land
      for (int j = i; j < issued; ++j) {
        const long long start = clock64();
        while (!mbar_try_wait(&sh->full[j % ns], (j / ns) & 1))
          if (clock64() - start > kWaitTimeoutCycles) break;
      }
    }
  } else if (tid < nconsumer) {
// ------------------------------------------------------------------ consumers: one row per stage
    const int lane = tid & 31;
    const int e0 = tid * EPT;
    const bool act = e0 < d;
    const HyperRegs hr = make_regs(p.h);
    const float gsc = hr.gscale * (p.use_inv_scale ? sc.inv_scale : 1.f);
    float dacc[kAdamSlots] = {0.f, 0.f, 0.f, 0.f};
    float norm2 = 0.f, pc = 0.f;
    for (int i = 0; i < n; ++i) {
      const int st = i % ns;
      if (!mbar_wait(&sh->full[st], (i / ns) & 1, abort_flag)) break;
      uint8_t* stage = ring + size_t(st) * stage_bytes;
      const AdamStageHdr* h = reinterpret_cast<const AdamStageHdr*>(stage);
      const int ne = h->ne, r = h->r, R = h->R, col = h->col, ti = h->ti, b = h->b;
      if (r == 0) {
#pragma unroll
        for (int j = 0; j < kAdamSlots; ++j) dacc[j] = 0.f;
        norm2 = 0.f;
        pc = p.pen_coef ? __ldg(p.pen_coef + col) : 0.f;
      }
      float w[EPT], m[EPT], v[EPT], g[EPT];
#pragma unroll
      for (int q = 0; q < EPT; ++q) { g[q] = 0.f; w[q] = 0.f; }
      WT* w_s = reinterpret_cast<WT*>(stage + off_w) + e0;
      MT* m_s = reinterpret_cast<MT*>(stage + off_m) + e0;
      MT* v_s = reinterpret_cast<MT*>(stage + off_v) + e0;
      if (act) {
        if (sizeof(WT) == 2) ldbf<EPT>(reinterpret_cast<const t16*>(w_s), w);
        else ldf<EPT>(reinterpret_cast<const float*>(w_s), w);
        if (sizeof(MT) == 2) {
          ldbf<EPT>(reinterpret_cast<const t16*>(m_s), m);
          ldbf<EPT>(reinterpret_cast<const t16*>(v_s), v);
        } else {
          ldf<EPT>(reinterpret_cast<const float*>(m_s), m);
          ldf<EPT>(reinterpret_cast<const float*>(v_s), v);
        }
        const t16* gs_s = reinterpret_cast<const t16*>(stage + off_gs) + e0;
#pragma unroll
        for (int j = 0; j < kAdamSlots; ++j) {
          if (j < ne) {
            const float a = h->a[j];
            float gv[EPT];
            ldbf<EPT>(gs_s + j * d, gv);
#pragma unroll
            for (int q = 0; q < EPT; ++q) {
              g[q] = fmaf(a, gv[q], g[q]);
              dacc[j] = fmaf(gv[q], w[q], dacc[j]);
            }
          }
        }
      }
      for (int x = b + kAdamSlots; x < b + ne; ++x) {  // rare: features with more entries than slots
        float dot = 0.f;
        if (act) {
          const float a = __ldg(p.fcsr_val + x);
          float gv[EPT];
          ldbf_global<EPT>(p.gs + (1LL * (ti + r) * B + __ldg(p.fcsr_tok + x)) * d + e0, gv);
#pragma unroll
          for (int q = 0; q < EPT; ++q) {
            g[q] = fmaf(a, gv[q], g[q]);
            dot = fmaf(gv[q], w[q], dot);
          }
        }
        if (p.grad_a != nullptr) {
          dot = warp_sum(dot);
          if (lane == 0 && dot != 0.f) atomicAdd(&p.grad_a[x], dot * gsc);
        }
      }
      if (act) {
        float dg0[EPT];
        const float* xrow = r == 0 ? extra_row_ptr(p, col) : nullptr;
        const bool extra = xrow != nullptr;
        if (extra) {
#pragma unroll
          for (int q = 0; q < EPT; q += 4) {
            const float4 t4 = __ldg(reinterpret_cast<const float4*>(xrow + e0 + q));
            dg0[q] = t4.x; dg0[q + 1] = t4.y; dg0[q + 2] = t4.z; dg0[q + 3] = t4.w;
          }
        }
#pragma unroll
        for (int q = 0; q < EPT; ++q) {
          float gq = fmaf(pc, w[q], g[q] * gsc);
          if (extra) gq += dg0[q];
          adam1(w[q], m[q], v[q], gq * sc.clip, hr);
          norm2 = fmaf(w[q], w[q], norm2);
        }
        const unsigned long long gidx = (unsigned long long)(p.row_start[ti] * d + h->elem_off + e0);
        if (sizeof(WT) == 2) stbf<EPT, SR>(reinterpret_cast<t16*>(w_s), w, p.h.sr_seed, (unsigned int)gidx);
        else stf<EPT>(reinterpret_cast<float*>(w_s), w);
        if (sizeof(MT) == 2) {
          // bf16 moments are always rounded stochastically: with beta2 = 0.999 a nearest rounding would freeze v
          // one hash per thread and row seeds a linear congruential stream: two 16-bit dither values per element
          uint32_t rng = hash32((unsigned int)gidx ^ p.h.moment_seed);
          t16* mo = reinterpret_cast<t16*>(m_s);
          t16* vo = reinterpret_cast<t16*>(v_s);
#pragma unroll
          for (int q = 0; q < EPT; q += 2) {
            uint32_t hm[2], hv[2];
#pragma unroll
            for (int z = 0; z < 2; ++z) {
              rng = rng * 1664525u + 1013904223u;
              const uint32_t um = __float_as_uint(m[q + z]), uv = __float_as_uint(v[q + z]);
              hm[z] = ((um & 0x7F800000u) == 0x7F800000u) ? (um >> 16) : ((um + (rng >> 16)) >> 16);
              hv[z] = ((uv & 0x7F800000u) == 0x7F800000u) ? (uv >> 16) : ((uv + ((rng * 0x9E3779B1u) >> 16)) >> 16);
            }
            *reinterpret_cast<uint32_t*>(mo + q) = hm[0] | (hm[1] << 16);
            *reinterpret_cast<uint32_t*>(vo + q) = hv[0] | (hv[1] << 16);
          }
        } else {
          stf<EPT>(reinterpret_cast<float*>(m_s), m);
          stf<EPT>(reinterpret_cast<float*>(v_s), v);
        }
      }
      if (r == R - 1) {
        if (p.grad_a != nullptr) {
          const int nslot = ne < kAdamSlots ? ne : kAdamSlots;
#pragma unroll
          for (int j = 0; j < kAdamSlots; ++j) {
            if (j < nslot) {
              const float sdot = warp_sum(dacc[j]);
              if (lane == 0 && sdot != 0.f) atomicAdd(&p.grad_a[b + j], sdot * gsc);
            }
          }
        }
        if (p.norm2_out != nullptr) {
          const float sn = warp_sum(norm2);
          if (lane == 0) atomicAdd(&p.norm2_out[col], sn);
        }
      }
      fence_proxy_async();  // the row written above is read next by the bulk store (async proxy)
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh->done[st]);
    }
  }
  __syncthreads();
  if (tid == 0 && sh->abort_flag && status != nullptr) atomicCAS(status, STATUS_OK, STATUS_WAIT_TIMEOUT);
}

// Tied decoders (per_source / per_target): same structure without the register-resident entries.
// Work item = (feature of one decoder tensor, 256-element segment): one warp, 8 elements per lane, walking
// the feature's R rows with the next row's (w, m, v) already in flight while the current row is updated.
// Row r of tensor i (source layer i, or target layer i with per_target tying); its gradient is
//   grad_scale * sum over contributing (entry, target) pairs of  a' * gs[target][tok, :]  (+ pen_coef * w).
template <typename WT, bool NORM_ONLY>
__global__ void __launch_bounds__(256) decoder_rows_adam_kernel(const DecAdamParams p) {
  const int lane = threadIdx.x & 31;
  const long long warp_global = (blockIdx.x * 1LL * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (gridDim.x * 1LL * blockDim.x) >> 5;
  const StepScales sc = read_step_ctl(p.ctl);
  if (sc.skip) return;
  const float gsc = p.h.grad_scale * (p.use_inv_scale ? sc.inv_scale : 1.f);
  float nsq = 0.f;
  const int nseg = (p.d + 255) / 256;
  const long long per_tensor = 1LL * p.F_pitch * nseg;
  const long long total_items = per_tensor * p.ntensors;
  const bool affine_grads = p.tying != 0 && p.grad_a != nullptr && (p.d_feat_offset != nullptr || p.d_feat_scale != nullptr);
  for (long long item = warp_global; item < total_items; item += nwarps) {
    const int ti = int(item / per_tensor);
    const long long rem = item - ti * per_tensor;
    const int f = int(rem / nseg);
    const int seg = int(rem - 1LL * f * nseg);
    const int R = p.rows[ti];
    const int e0 = seg * 256 + lane * 8;
    const bool act = e0 < p.d;
    const long long row0 = 1LL * f * R;
    WT* wbase = static_cast<WT*>(p.w[ti]) + row0 * p.d + e0;
    float* mbase = p.m[ti] + row0 * p.d + e0;
    float* vbase = p.v[ti] + row0 * p.d + e0;
    // contributing source layers of this tensor's rows
    const int s_lo = p.tying == 2 ? 0 : ti;
    const int s_hi = ti;
    // d/dw of the norm-weighted sparsity penalty: coefficient of feature (ti, f); with per-target tying
    // the row belongs to the norm of every source feature (s <= ti, f).
    float pc = 0.f;
    if (p.pen_coef) {
      if (p.tying == 2) { for (int s = 0; s <= ti; ++s) pc += p.pen_coef[s * p.F_pitch + f]; }
      else pc = p.pen_coef[ti * p.F_pitch + f];
    }
    const float* xrow = extra_row_ptr(p, ti * p.F_pitch + f);
    if (NORM_ONLY && xrow == nullptr) {
      bool any = false;
      for (int s = s_lo; s <= s_hi; ++s) any |= __ldg(p.feat_off + s * p.F_pitch + f + 1) > __ldg(p.feat_off + s * p.F_pitch + f);
      if (!any) continue;
    }
    RowRegs<WT> cur, nxt;
    if (act) { if (NORM_ONLY) cur.w.load(wbase); else cur.load(wbase, mbase, vbase); }
    float norm2 = 0.f;
    for (int r = 0; r < R; ++r) {
      if (act && r + 1 < R) {
        if (NORM_ONLY) nxt.w.load(wbase + 1LL * (r + 1) * p.d);
        else nxt.load(wbase + 1LL * (r + 1) * p.d, mbase + 1LL * (r + 1) * p.d, vbase + 1LL * (r + 1) * p.d);
      }
      const int t_fixed = p.tying == 0 ? ti + r : (p.tying == 2 ? ti : -1);
      float w[8], g[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) { g[i] = 0.f; w[i] = 0.f; }
      if (act) cur.w.get(w);
      for (int s = s_lo; s <= s_hi; ++s) {
        const int col = s * p.F_pitch + f;
        const int b = __ldg(p.feat_off + col), e = __ldg(p.feat_off + col + 1);
        for (int i = b; i < e; ++i) {
          const int tok = __ldg(p.fcsr_tok + i);
          const float a = __ldg(p.fcsr_val + i);
          const int t_begin = t_fixed >= 0 ? t_fixed : s;
          const int t_end = t_fixed >= 0 ? t_fixed : p.L - 1;
          float dot = 0.f;
          for (int t = t_begin; t <= t_end; ++t) {
            float av = a, dscale = 1.f, shifted = a;
            if (p.tying != 0 && a != 0.f) {
              if (p.feat_offset) av += p.feat_offset[1LL * t * p.F_pitch + f];
              shifted = av;
              if (p.feat_scale) { const float fsc = p.feat_scale[1LL * t * p.F_pitch + f]; av *= fsc; dscale = fsc; }
            }
            float dot_t = 0.f;
            if (act) {
              float gv[8];
              unpack8(__ldg(reinterpret_cast<const uint4*>(p.gs + (1LL * t * p.B + tok) * p.d + e0)), gv);
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                g[k] = fmaf(av, gv[k], g[k]);
                dot_t = fmaf(gv[k], w[k], dot_t);
              }
            }
            dot = fmaf(dot_t, dscale, dot);
            // gradients of the affine terms of target t: d/d offset = scale * (gs_t . w), d/d scale = (a + offset) * (gs_t . w)
            if (affine_grads && a != 0.f) {
              const float ds = warp_sum(dot_t) * gsc;
              if (lane == 0 && ds != 0.f) {
                if (p.d_feat_offset != nullptr) atomicAdd(&p.d_feat_offset[1LL * t * p.F_pitch + f], ds * dscale);
                if (p.d_feat_scale != nullptr) atomicAdd(&p.d_feat_scale[1LL * t * p.F_pitch + f], ds * shifted);
              }
            }
          }
          if (p.grad_a != nullptr) {
            dot = warp_sum(dot);
            if (lane == 0 && dot != 0.f) atomicAdd(&p.grad_a[i], dot * gsc);
          }
        }
      }
      if (act) {
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] = fmaf(pc, w[k], g[k] * gsc);
        if (r == 0 && xrow != nullptr) {
          float dg0[8];
          load8f(xrow + e0, dg0);
#pragma unroll
          for (int k = 0; k < 8; ++k) g[k] += dg0[k];
        }
        if (NORM_ONLY) {
#pragma unroll
          for (int k = 0; k < 8; ++k) nsq = fmaf(g[k], g[k], nsq);
          cur = nxt;
          continue;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] *= sc.clip;
        float m[8], v[8];
        f4x2_to8(cur.m0, cur.m1, m);
        f4x2_to8(cur.v0, cur.v1, v);
        adam_update8(w, m, v, g, p.h);
        WT* wrow = wbase + 1LL * r * p.d;
        stream_store8f(mbase + 1LL * r * p.d, m);
        stream_store8f(vbase + 1LL * r * p.d, v);
        if (sizeof(WT) == 2) {
          t16 bq[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            bq[k] = to_bf16(w[k], p.h.sr_seed, (unsigned long long)((p.row_start[ti] + row0 + r) * p.d + e0 + k));
            const float wr = t16_to_float(bq[k]);  // norms are taken of the stored (rounded) weights
            norm2 = fmaf(wr, wr, norm2);
          }
          __stcs(reinterpret_cast<uint4*>(wrow), *reinterpret_cast<const uint4*>(bq));
        } else {
          stream_store8f(reinterpret_cast<float*>(wrow), w);
#pragma unroll
          for (int k = 0; k < 8; ++k) norm2 = fmaf(w[k], w[k], norm2);
        }
      }
      cur = nxt;
    }
    if (!NORM_ONLY && p.norm2_out != nullptr) {
      norm2 = warp_sum(norm2);
      if (lane == 0) atomicAdd(&p.norm2_out[ti * p.F_pitch + f], norm2);
    }
  }
  if (NORM_ONLY) block_add(nsq, p.norm_sq_out);
}

// ------------------------------------------------------------------ encoder rows
struct EncAdamParams {
  void* w;            // [L, F_pitch, d]
  float* m;
  float* v;
  void* bias;         // [L, F_pitch] (same dtype as w), updated here too
  float* bias_m;
  float* bias_v;
  int L, B, d, F_pitch;
  const int* feat_off;
  const int* fcsr_tok;
  const float* delta;           // [nnz] dL/d(pre-activation) per CSR slot (already scaled)
  const t16* x;       // [L, B, d] layer inputs
  const float* dense_grad;      // optional [L, F_pitch, d] fp32 gradient added to the sparse one (e.g. pre-activation loss)
  const float* dense_bias_grad; // optional [L, F_pitch]
  const int* extra_idx;         // optional compact extras (auxiliary loss): extra_idx[row] = row of extra_rows / extra_bias, or -1
  const float* extra_rows;      // [n_extra, d]
  const float* extra_bias;      // [n_extra]
  const float* ctl;             // optional step control block
  float* norm_sq_out;           // norm-only pass
  int norm_only;                // bias kernel: 1 = only add the squared bias gradients to norm_sq_out
  AdamHyper h;                  // grad_scale applies to the sparse part
};
__device__ __forceinline__ int enc_extra_index(const EncAdamParams& p, long long row) {
  return p.extra_idx != nullptr ? __ldg(p.extra_idx + row) : -1;
}

template <typename WT, bool NORM_ONLY>
__global__ void __launch_bounds__(256) encoder_rows_adam_kernel(const EncAdamParams p) {
  const int lane = threadIdx.x & 31;
  const long long warp_global = (blockIdx.x * 1LL * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (gridDim.x * 1LL * blockDim.x) >> 5;
  const StepScales sc = read_step_ctl(p.ctl);
  if (sc.skip) return;
  float nsq = 0.f;
  const int nseg = (p.d + 255) / 256;
  const long long total_items = 1LL * p.L * p.F_pitch * nseg;
  for (long long item = warp_global; item < total_items; item += nwarps) {
    const long long row = item / nseg;
    const int seg = int(item - row * nseg);
    const int l = int(row / p.F_pitch);
    const int e0 = seg * 256 + lane * 8;
    const bool act = e0 < p.d;
    const int b = __ldg(p.feat_off + row), e = __ldg(p.feat_off + row + 1);
    const int xi = enc_extra_index(p, row);
    if (NORM_ONLY && e == b && xi < 0 && p.dense_grad == nullptr) continue;
    WT* wrow = static_cast<WT*>(p.w) + row * p.d + e0;
    float* mrow = p.m + row * p.d + e0;
    float* vrow = p.v + row * p.d + e0;
    WVec<WT> wq;
    float4 m0, m1, v0, v1;
    if (act && !NORM_ONLY) {
      wq.load(wrow);
      m0 = __ldcs(reinterpret_cast<const float4*>(mrow)); m1 = __ldcs(reinterpret_cast<const float4*>(mrow) + 1);
      v0 = __ldcs(reinterpret_cast<const float4*>(vrow)); v1 = __ldcs(reinterpret_cast<const float4*>(vrow) + 1);
    }
    if (act) {
      float w[8], g[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) g[i] = 0.f;
      for (int i = b; i < e; ++i) {
        const float dl = __ldg(p.delta + i);
        float xv[8];
        unpack8(__ldg(reinterpret_cast<const uint4*>(p.x + (1LL * l * p.B + __ldg(p.fcsr_tok + i)) * p.d + e0)), xv);
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] = fmaf(dl, xv[k], g[k]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] *= p.h.grad_scale;
      if (p.dense_grad) {
        float dg[8];
        load8f(p.dense_grad + row * p.d + e0, dg);
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] += dg[k];
      }
      if (xi >= 0) {
        float dg[8];
        load8f(p.extra_rows + 1LL * xi * p.d + e0, dg);
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] += dg[k];
      }
      if (NORM_ONLY) {
#pragma unroll
        for (int k = 0; k < 8; ++k) nsq = fmaf(g[k], g[k], nsq);
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] *= sc.clip;
        float m[8], v[8];
        wq.get(w);
        f4x2_to8(m0, m1, m);
        f4x2_to8(v0, v1, v);
        adam_update8(w, m, v, g, p.h);
        stream_store8f(mrow, m);
        stream_store8f(vrow, v);
        store_w8<WT>(wrow, w, p.h.sr_seed, (unsigned long long)(row * p.d + e0));
      }
    }
    if (seg == 0 && lane == 0 && p.bias != nullptr) {
      float gb = 0.f;
      for (int i = b; i < e; ++i) gb += p.delta[i];
      gb *= p.h.grad_scale;
      if (p.dense_bias_grad) gb += p.dense_bias_grad[row];
      if (xi >= 0 && p.extra_bias != nullptr) gb += p.extra_bias[xi];
      if (NORM_ONLY) { nsq = fmaf(gb, gb, nsq); continue; }
      gb *= sc.clip;
      WT* bp = static_cast<WT*>(p.bias) + row;
      float wv = sizeof(WT) == 2 ? t16_to_float(*reinterpret_cast<t16*>(bp)) : *reinterpret_cast<float*>(bp);
      float mm = p.bias_m[row], vv = p.bias_v[row];
      if (p.h.decoupled) wv *= (1.f - p.h.lr * p.h.weight_decay);
      else gb = fmaf(p.h.weight_decay, wv, gb);
      mm = fmaf(p.h.beta1, mm, (1.f - p.h.beta1) * gb);
      vv = fmaf(p.h.beta2, vv, (1.f - p.h.beta2) * gb * gb);
      wv -= (p.h.lr / p.h.bc1) * (mm / (sqrtf(vv) * rsqrtf(p.h.bc2) + p.h.eps));
      p.bias_m[row] = mm; p.bias_v[row] = vv;
      if (sizeof(WT) == 2) *reinterpret_cast<t16*>(bp) = to_bf16(wv, p.h.sr_seed, 0x9000000000ULL + row);
      else *reinterpret_cast<float*>(bp) = wv;
    }
  }
  if (NORM_ONLY) block_add(nsq, p.norm_sq_out);
}

// Encoder bias update on its own (used with the bulk-copy row pipeline, which handles the weight rows).
template <typename WT>
__global__ void __launch_bounds__(256) encoder_bias_adam_kernel(const EncAdamParams p) {
  const long long rows = 1LL * p.L * p.F_pitch;
  const StepScales sc = read_step_ctl(p.ctl);
  if (sc.skip) return;
  float nsq = 0.f;
  for (long long row = blockIdx.x * 1LL * blockDim.x + threadIdx.x; row < rows; row += 1LL * gridDim.x * blockDim.x) {
    const int b = __ldg(p.feat_off + row), e = __ldg(p.feat_off + row + 1);
    float gb = 0.f;
    for (int i = b; i < e; ++i) gb += p.delta[i];
    gb *= p.h.grad_scale;
    if (p.dense_bias_grad) gb += p.dense_bias_grad[row];
    const int xi = enc_extra_index(p, row);
    if (xi >= 0 && p.extra_bias != nullptr) gb += p.extra_bias[xi];
    if (p.norm_only) { nsq = fmaf(gb, gb, nsq); continue; }
    gb *= sc.clip;
    WT* bp = static_cast<WT*>(p.bias) + row;
    float wv = sizeof(WT) == 2 ? t16_to_float(*reinterpret_cast<t16*>(bp)) : *reinterpret_cast<float*>(bp);
    float mm = p.bias_m[row], vv = p.bias_v[row];
    if (p.h.decoupled) wv *= (1.f - p.h.lr * p.h.weight_decay);
    else gb = fmaf(p.h.weight_decay, wv, gb);
    mm = fmaf(p.h.beta1, mm, (1.f - p.h.beta1) * gb);
    vv = fmaf(p.h.beta2, vv, (1.f - p.h.beta2) * gb * gb);
    wv -= (p.h.lr / p.h.bc1) * (mm / (sqrtf(vv) * rsqrtf(p.h.bc2) + p.h.eps));
    p.bias_m[row] = mm; p.bias_v[row] = vv;
    if (sizeof(WT) == 2) *reinterpret_cast<t16*>(bp) = to_bf16(wv, p.h.sr_seed, 0x9000000000ULL + row);
    else *reinterpret_cast<float*>(bp) = wv;
  }
  if (p.norm_only) block_add(nsq, p.norm_sq_out);
}

// ------------------------------------------------------------------ dense Adam for the small tensors
// `ctl` (optional): skip flag and clip coefficient; `seed_scaled`: the gradient carries the loss scale (times 1 / scale);
// `norm_weight` > 0: norm-only pass, norm_weight * sum g^2 is added to ctl[SC_GRAD_NORM_SQ] and nothing is updated.
template <typename WT>
__global__ void __launch_bounds__(256) dense_adam_kernel(WT* __restrict__ w, float* __restrict__ m, float* __restrict__ v,
                                                           const float* __restrict__ grad, long long n, AdamHyper h,
                                                           float* __restrict__ ctl, int seed_scaled, float norm_weight) {
  const StepScales sc = read_step_ctl(ctl);
  if (sc.skip) return;
  const float gmul = h.grad_scale * (seed_scaled ? sc.inv_scale : 1.f);
  if (norm_weight > 0.f) {
    float nsq = 0.f;
    for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < n; i += 1LL * gridDim.x * blockDim.x) {
      const float g = grad[i] * gmul;
      nsq = fmaf(g, g, nsq);
    }
    block_add(nsq * norm_weight, ctl != nullptr ? ctl + SC_GRAD_NORM_SQ : nullptr);
    return;
  }
  for (long long i = blockIdx.x * 1LL * blockDim.x + threadIdx.x; i < n; i += 1LL * gridDim.x * blockDim.x) {
    float wv = sizeof(WT) == 2 ? t16_to_float(*reinterpret_cast<const t16*>(w + i)) : *reinterpret_cast<const float*>(w + i);
    float g = grad[i] * gmul * sc.clip;
    if (h.decoupled) wv *= (1.f - h.lr * h.weight_decay);
    else g = fmaf(h.weight_decay, wv, g);
    const float mm = fmaf(h.beta1, m[i], (1.f - h.beta1) * g);
    const float vv = fmaf(h.beta2, v[i], (1.f - h.beta2) * g * g);
    wv -= (h.lr / h.bc1) * (mm / (sqrtf(vv) * rsqrtf(h.bc2) + h.eps));
    m[i] = mm; v[i] = vv;
    if (sizeof(WT) == 2) *reinterpret_cast<t16*>(w + i) = to_bf16(wv, h.sr_seed, 0xA000000000ULL + i);
    else *reinterpret_cast<float*>(w + i) = wv;
  }
}

// Squared decoder norms per feature: out[ti * F_pitch + f] = sum over the feature's rows and d of w^2.
template <typename WT>
__global__ void __launch_bounds__(256) decoder_norm2_kernel(const WT* __restrict__ w, float* __restrict__ out, int F, int R, int d) {
  const int lane = threadIdx.x & 31;
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const long long per_feat = 1LL * R * d;
  for (int f = warp_global; f < F; f += nwarps) {
    const WT* base = w + per_feat * f;
    float s = 0.f;
    for (long long i = lane * 8; i < per_feat; i += 256) {
      float x[8];
      load_w8<WT>(base + i, x);
#pragma unroll
      for (int k = 0; k < 8; ++k) s = fmaf(x[k], x[k], s);
    }
    s = warp_sum(s);
    if (lane == 0) out[f] = s;
  }
}

// Norm-weighted tanh sparsity penalty on the active entries (reference clt/training/losses.py:143-195):
//   penalty = lambda * sum tanh(c * n_f * a),  n_f = decoder norm of the entry's feature.
// One thread per feature column walks its CSR segment and writes
//   grad_a[i]   = lambda * c * n * sech^2(c n a)                (assignment: runs before the decoder pass)
//   pen_coef[f] = lambda * c * sum_i a_i sech^2(c n a_i) / n    (coefficient of w in dL/dw through the norm)
// and adds the penalty value to *penalty_out.
__global__ void __launch_bounds__(256) sparsity_penalty_kernel(const int* __restrict__ feat_off, const float* __restrict__ fcsr_val,
                                                                 const float* __restrict__ norm2, int ncols, float lambda, float c,
                                                                 float* __restrict__ grad_a, float* __restrict__ pen_coef,
                                                                 double* __restrict__ penalty_out) {
  float local = 0.f;
  for (int col = blockIdx.x * blockDim.x + threadIdx.x; col < ncols; col += gridDim.x * blockDim.x) {
    const int b = feat_off[col], e = feat_off[col + 1];
    float coef = 0.f;
    if (e > b) {
      const float n = sqrtf(norm2[col]);
      float acc = 0.f;
      for (int i = b; i < e; ++i) {
        const float a = fcsr_val[i];
        const float th = tanhf(c * n * a);
        const float sech2 = 1.f - th * th;
        local += th;
        grad_a[i] = lambda * c * n * sech2;
        acc = fmaf(a, sech2, acc);
      }
      coef = n > 0.f ? lambda * c * acc / n : 0.f;
    }
    pen_coef[col] = coef;
  }
  __shared__ float red[8];
  local = warp_sum(local);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int w = 0; w < 8; ++w) tot += red[w];
    if (tot != 0.f) atomicAdd(penalty_out, double(tot) * double(lambda));
  }
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
static AdamHyper to_hyper(const CltAdamHyper& c) {
  AdamHyper h;
  h.lr = c.lr; h.beta1 = c.beta1; h.beta2 = c.beta2; h.eps = c.eps; h.weight_decay = c.weight_decay;
  h.bc1 = c.bc1; h.bc2 = c.bc2; h.decoupled = c.decoupled; h.grad_scale = c.grad_scale; h.sr_seed = c.sr_seed; h.moment_seed = c.moment_seed;
  return h;
}

struct CltDecAdamArgs {
  void* w[32]; float* m[32]; float* v[32]; int rows[32];
  int ntensors, L, B, d, F_pitch, tying, weights_bf16;
  const int* feat_off; const int* fcsr_tok; const float* fcsr_val;
  const void* gs; float* grad_a; const float* pen_coef; float* norm2_out;
  const float* feat_offset; const float* feat_scale;
  const float* dgrad_row0;
  CltAdamHyper h;
  int* status;  // when given, untied decoders use the bulk-copy pipeline (its bounded waits report here)
  int moments_bf16;  // m / v are bf16 tensors (bulk pipeline with bf16 weights only)
  const int* extra_idx; const float* extra_rows;  // compact extra gradient rows (auxiliary loss), see DecAdamParams
  float* ctl;        // step control block (skip flag, 1 / loss scale, clip coefficient); may be null
  int norm_only;     // 1: gradient-norm pre-pass (adds to ctl[SC_GRAD_NORM_SQ], writes grad_a, updates nothing)
  float* d_feat_offset; float* d_feat_scale;  // tied decoders: gradient accumulators of the affine terms, see DecAdamParams
};

// Launch geometry of the bulk-copy row pipeline (shared by the decoder and the encoder update).
static int bulk_rows_adam_geometry(int d, bool weights_bf16, bool moments_bf16, int* ept_out, int* gthreads_out, int* stage_bytes_out, size_t* smem_out,
                                   int* nstages_out = nullptr) {
  const int ept = d <= 1024 ? 4 : 8;  // elements per consumer thread: more, shorter threads where the row allows
  const int gthreads = ((d / ept + 31) / 32) * 32;
  const size_t wsz = weights_bf16 ? 2 : 4;
  const size_t msz = moments_bf16 ? 2 : 4;
  const int stage_bytes = int(((64 + size_t(d) * (wsz + 2 * msz + 2 * kAdamSlots)) + 127) / 128 * 128);
  const int nstages = stage_bytes > 24 * 1024 ? 3 : kAdamStages;
  if (nstages_out) *nstages_out = nstages;
  const size_t smem = size_t(nstages) * stage_bytes + sizeof(AdamBulkShared) + 256;
  *ept_out = ept; *gthreads_out = gthreads; *stage_bytes_out = stage_bytes; *smem_out = smem;
  return (d % 8 == 0 && gthreads <= 256 && smem <= 200 * 1024) ? 1 : 0;
}
static bool bulk_rows_adam_fits(int d, int weights_bf16) {
  int ept, gthreads, stage_bytes;
  size_t smem;
  return bulk_rows_adam_geometry(d, weights_bf16 != 0, false, &ept, &gthreads, &stage_bytes, &smem) != 0;
}
static int launch_rows_adam_bulk(const DecAdamParams& p, bool weights_bf16, bool sr, int num_sms, int* status, cudaStream_t st) {
  int ept, gthreads, stage_bytes;
  size_t smem;
  const bool mb = p.moments_bf16 != 0;
  if (mb && !weights_bf16) return -1;  // bf16 moments go with bf16 weights
  int nstages = kAdamStages;
  if (!bulk_rows_adam_geometry(p.d, weights_bf16, mb, &ept, &gthreads, &stage_bytes, &smem, &nstages)) return -1;
  int per_sm = int((227 * 1024) / (smem + 1024));
  const int by_threads = 2048 / (gthreads + 32);
  per_sm = per_sm > by_threads ? by_threads : per_sm;
  per_sm = per_sm < 1 ? 1 : (per_sm > 6 ? 6 : per_sm);
  int bgrid = num_sms * per_sm;
  if (bgrid > p.F_pitch) bgrid = p.F_pitch;
  {
    // CTA b owns the features b, b + grid, ... of every tensor: pick the grid (between half of the resident slots and all
    // of them) that splits the features most evenly, so that no CTA still streams rows when the others are done.  On a
    // narrow shard (3072 features, 888 slots) the naive grid leaves CTAs with 3 and with 4 features per tensor.
    int best = bgrid;
    double best_waste = double((p.F_pitch + bgrid - 1) / bgrid) * bgrid / double(p.F_pitch) - 0.03;  // a few per cent do not pay for fewer CTAs
    for (int g = bgrid - 1; g >= (3 * bgrid) / 4 && g >= 1; --g) {
      const int per = (p.F_pitch + g - 1) / g;
      const double waste = double(per) * g / double(p.F_pitch);
      if (waste < best_waste - 1e-9) { best_waste = waste; best = g; }
    }
    bgrid = best;
  }
  auto launch = [&](auto kern, int which) -> int {
    static size_t attr_set[10] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
    if (attr_set[which] < smem) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)) != cudaSuccess) return -4;
      attr_set[which] = smem;
    }
    kern<<<bgrid, gthreads + 32, smem, st>>>(p, gthreads, stage_bytes, nstages, status);
    return 0;
  };
  using bf = t16;
  if (mb) {
#if CLT_T16_IS_HALF
    return -6;  // bf16 moments go with bf16 weights
#else
    if (ept == 4) return sr ? launch(decoder_rows_adam_bulk_kernel<bf, true, 4, bf>, 6) : launch(decoder_rows_adam_bulk_kernel<bf, false, 4, bf>, 7);
    return sr ? launch(decoder_rows_adam_bulk_kernel<bf, true, 8, bf>, 8) : launch(decoder_rows_adam_bulk_kernel<bf, false, 8, bf>, 9);
#endif
  }
  if (ept == 4) {
    if (weights_bf16) return sr ? launch(decoder_rows_adam_bulk_kernel<bf, true, 4, float>, 0) : launch(decoder_rows_adam_bulk_kernel<bf, false, 4, float>, 1);
    return launch(decoder_rows_adam_bulk_kernel<float, false, 4, float>, 2);
  }
  if (weights_bf16) return sr ? launch(decoder_rows_adam_bulk_kernel<bf, true, 8, float>, 3) : launch(decoder_rows_adam_bulk_kernel<bf, false, 8, float>, 4);
  return launch(decoder_rows_adam_bulk_kernel<float, false, 8, float>, 5);
}

extern "C" int CLT_FN(clt_decoder_rows_adam)(const CltDecAdamArgs* a, int num_sms, cudaStream_t st) {
  if (a->d % 8 != 0 || a->ntensors > kMaxLayersA) return -1;
  DecAdamParams p;
  long long acc = 0;
  for (int i = 0; i < kMaxLayersA; ++i) {
    p.w[i] = a->w[i]; p.m[i] = a->m[i]; p.v[i] = a->v[i]; p.rows[i] = a->rows[i];
    p.row_start[i] = acc;
    if (i < a->ntensors) acc += 1LL * a->F_pitch * a->rows[i];
  }
  p.row_start[kMaxLayersA] = acc;
  for (int i = a->ntensors; i <= kMaxLayersA; ++i) p.row_start[i] = acc;
  p.ntensors = a->ntensors; p.L = a->L; p.B = a->B; p.d = a->d; p.F_pitch = a->F_pitch; p.tying = a->tying;
  p.feat_off = a->feat_off; p.fcsr_tok = a->fcsr_tok; p.fcsr_val = a->fcsr_val;
  p.gs = static_cast<const t16*>(a->gs); p.grad_a = a->grad_a; p.pen_coef = a->pen_coef; p.norm2_out = a->norm2_out;
  p.feat_offset = a->feat_offset; p.feat_scale = a->feat_scale; p.dgrad_row0 = a->dgrad_row0; p.h = to_hyper(a->h);
  p.d_feat_offset = a->d_feat_offset; p.d_feat_scale = a->d_feat_scale;
  p.moments_bf16 = a->moments_bf16;
  p.extra_idx = a->extra_idx; p.extra_rows = a->extra_rows; p.ctl = a->ctl; p.use_inv_scale = 1;
  p.norm_sq_out = a->ctl != nullptr ? a->ctl + SC_GRAD_NORM_SQ : nullptr;
  if (a->moments_bf16 && !(a->tying == 0 && a->status != nullptr && a->weights_bf16)) return -6;  // only the bulk pipeline handles bf16 moments
  if (acc == 0) return 0;
  const int grid = num_sms * 8;
  if (a->norm_only) {
    if (a->ctl == nullptr) return -1;
    if (a->tying == 0) {
      if (a->weights_bf16) decoder_rows_adam_untied_kernel<t16, false, true><<<grid, 256, 0, st>>>(p);
      else decoder_rows_adam_untied_kernel<float, false, true><<<grid, 256, 0, st>>>(p);
    } else if (a->weights_bf16) {
      decoder_rows_adam_kernel<t16, true><<<grid, 256, 0, st>>>(p);
    } else {
      decoder_rows_adam_kernel<float, true><<<grid, 256, 0, st>>>(p);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
  }
  if (a->tying == 0 && a->status != nullptr && bulk_rows_adam_fits(a->d, a->weights_bf16) && acc * a->d < (1LL << 62)) {
    const int rc = launch_rows_adam_bulk(p, a->weights_bf16 != 0, a->h.sr_seed != 0, num_sms, a->status, st);
    if (rc != 0) return rc;
  } else if (a->tying == 0) {
    const bool sr = a->h.sr_seed != 0;
    if (a->weights_bf16) {
      if (sr) decoder_rows_adam_untied_kernel<t16, true, false><<<grid, 256, 0, st>>>(p);
      else decoder_rows_adam_untied_kernel<t16, false, false><<<grid, 256, 0, st>>>(p);
    } else {
      decoder_rows_adam_untied_kernel<float, false, false><<<grid, 256, 0, st>>>(p);
    }
  } else if (a->weights_bf16) {
    decoder_rows_adam_kernel<t16, false><<<grid, 256, 0, st>>>(p);
  } else {
    decoder_rows_adam_kernel<float, false><<<grid, 256, 0, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

struct CltEncAdamArgs {
  void* w; float* m; float* v; void* bias; float* bias_m; float* bias_v;
  int L, B, d, F_pitch, weights_bf16;
  const int* feat_off; const int* fcsr_tok; const float* delta; const void* x;
  const float* dense_grad; const float* dense_bias_grad;
  CltAdamHyper h;
  int* status;  // when given, the weight rows go through the bulk-copy pipeline
  int moments_bf16;
  const int* extra_idx; const float* extra_rows; const float* extra_bias;  // compact extras, see EncAdamParams
  float* ctl;
  int norm_only;
};

extern "C" int CLT_FN(clt_encoder_rows_adam)(const CltEncAdamArgs* a, int num_sms, cudaStream_t st) {
  if (a->d % 8 != 0) return -1;
  EncAdamParams p;
  p.w = a->w; p.m = a->m; p.v = a->v; p.bias = a->bias; p.bias_m = a->bias_m; p.bias_v = a->bias_v;
  p.L = a->L; p.B = a->B; p.d = a->d; p.F_pitch = a->F_pitch;
  p.feat_off = a->feat_off; p.fcsr_tok = a->fcsr_tok; p.delta = a->delta; p.x = static_cast<const t16*>(a->x);
  p.dense_grad = a->dense_grad; p.dense_bias_grad = a->dense_bias_grad; p.h = to_hyper(a->h);
  p.extra_idx = a->extra_idx; p.extra_rows = a->extra_rows; p.extra_bias = a->extra_bias; p.ctl = a->ctl;
  p.norm_sq_out = a->ctl != nullptr ? a->ctl + SC_GRAD_NORM_SQ : nullptr; p.norm_only = a->norm_only;
  const int grid = num_sms * 8;
  if (a->norm_only) {
    if (a->ctl == nullptr) return -1;
    if (a->weights_bf16) encoder_rows_adam_kernel<t16, true><<<grid, 256, 0, st>>>(p);
    else encoder_rows_adam_kernel<float, true><<<grid, 256, 0, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
  }
  if (a->status != nullptr && a->L <= kMaxLayersA && bulk_rows_adam_fits(a->d, a->weights_bf16)) {
    // the encoder is the one-row-per-feature case of the row pipeline: layer l is "tensor" l with R = 1, the
    // layer inputs play the gradient seed and delta the activation
    DecAdamParams q;
    const size_t wsz = a->weights_bf16 ? 2 : 4;
    const long long per_layer = 1LL * a->F_pitch * a->d;
    for (int i = 0; i < kMaxLayersA; ++i) {
      const int l = i < a->L ? i : 0;
      q.w[i] = static_cast<char*>(a->w) + size_t(l) * per_layer * wsz;
      const size_t msz = a->moments_bf16 ? 2 : 4;
      q.m[i] = reinterpret_cast<float*>(reinterpret_cast<char*>(a->m) + size_t(l) * per_layer * msz);
      q.v[i] = reinterpret_cast<float*>(reinterpret_cast<char*>(a->v) + size_t(l) * per_layer * msz);
      q.rows[i] = 1;
      q.row_start[i] = 1LL * (i < a->L ? i : a->L) * a->F_pitch;
    }
    q.row_start[kMaxLayersA] = 1LL * a->L * a->F_pitch;
    q.ntensors = a->L; q.L = a->L; q.B = a->B; q.d = a->d; q.F_pitch = a->F_pitch; q.tying = 0;
    q.feat_off = a->feat_off; q.fcsr_tok = a->fcsr_tok; q.fcsr_val = a->delta; q.gs = p.x;
    q.grad_a = nullptr; q.pen_coef = nullptr; q.norm2_out = nullptr; q.feat_offset = nullptr; q.feat_scale = nullptr;
    q.d_feat_offset = nullptr; q.d_feat_scale = nullptr;
    q.dgrad_row0 = a->dense_grad; q.h = p.h;
    q.moments_bf16 = a->moments_bf16;
    q.extra_idx = a->dense_grad == nullptr ? a->extra_idx : nullptr; q.extra_rows = a->extra_rows;
    q.ctl = a->ctl; q.use_inv_scale = 0; q.norm_sq_out = nullptr;
    if (a->dense_grad != nullptr && a->extra_idx != nullptr) return -7;  // the row pipeline takes one kind of extra rows
    const int rc = launch_rows_adam_bulk(q, a->weights_bf16 != 0, a->h.sr_seed != 0, num_sms, a->status, st);
    if (rc != 0) return rc;
    if (p.bias != nullptr) {
      const int bgrid = int((1LL * a->L * a->F_pitch + 255) / 256);
      if (a->weights_bf16) encoder_bias_adam_kernel<t16><<<bgrid, 256, 0, st>>>(p);
      else encoder_bias_adam_kernel<float><<<bgrid, 256, 0, st>>>(p);
    }
  } else if (a->moments_bf16) {
    return -6;  // only the bulk pipeline handles bf16 moments
  } else if (a->weights_bf16) encoder_rows_adam_kernel<t16, false><<<grid, 256, 0, st>>>(p);
  else encoder_rows_adam_kernel<float, false><<<grid, 256, 0, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int CLT_FN(clt_dense_adam)(void* w, float* m, float* v, const float* grad, long long n, int weights_bf16, const CltAdamHyper* h,
                                      float* ctl, int seed_scaled, float norm_weight, cudaStream_t st) {
  if (n <= 0) return 0;
  const int grid = int((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
  if (weights_bf16) dense_adam_kernel<t16><<<grid, 256, 0, st>>>(static_cast<t16*>(w), m, v, grad, n, to_hyper(*h), ctl, seed_scaled, norm_weight);
  else dense_adam_kernel<float><<<grid, 256, 0, st>>>(static_cast<float*>(w), m, v, grad, n, to_hyper(*h), ctl, seed_scaled, norm_weight);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int CLT_FN(clt_decoder_norm2)(const void* w, float* out, int F, int R, int d, int weights_bf16, cudaStream_t st) {
  if ((1LL * R * d) % 8 != 0) return -1;
  const int grid = (F + 7) / 8 < 1184 ? (F + 7) / 8 : 1184;
  if (grid == 0) return 0;
  if (weights_bf16) decoder_norm2_kernel<t16><<<grid, 256, 0, st>>>(static_cast<const t16*>(w), out, F, R, d);
  else decoder_norm2_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(w), out, F, R, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

#if !CLT_T16_IS_HALF
extern "C" int clt_sparsity_penalty(const int* feat_off, const float* fcsr_val, const float* norm2, int ncols, float lambda, float c,
                                    float* grad_a, float* pen_coef, double* penalty_out, cudaStream_t st) {
  if (ncols <= 0) return 0;
  const int grid = (ncols + 255) / 256 < 1184 ? (ncols + 255) / 256 : 1184;
  sparsity_penalty_kernel<<<grid, 256, 0, st>>>(feat_off, fcsr_val, norm2, ncols, lambda, c, grad_a, pen_coef, penalty_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
#endif
