// Row-reduction class: RMSNorm, softmax, LayerNorm (+ fused cast to fp16).
//
// Counterpart of the reference's "general reduction" schedule
// (python/dtas/schedule/tir_reduction.py:36-105): one thread group per row, the row
// cached on chip between the reduction and the normalising epilogue, fp32 arithmetic,
// launch shape picked per m-bucket (python/dtas/policy/reduction_config_emiter.py:77-158).
//
// Design: a row is owned by TPR threads (a power of two, 32..1024).  Each thread loads
// its 16-byte chunks (8 fp16, or 2 x 16 B for fp32 input) with all loads in flight at
// once, keeps the row in registers as loaded, reduces with warp shuffles (+ one shared
// memory hop when TPR > 32) and writes 16-byte fp16 vectors.  HBM sees each element
// once in and once out: algorithmic bytes 4*n_cols per row for fp16 in/out
// (+ 2*n_cols once for the RMSNorm weight).  Bound: HBM bandwidth.
#include "common.cuh"

namespace dtas {
namespace {

constexpr int kCtaThreads = 256;

__device__ __forceinline__ float2 h2f(uint32_t v) {
  return __half22float2(*reinterpret_cast<__half2*>(&v));
}
__device__ __forceinline__ uint32_t f2h(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// A chunk is 8 consecutive elements of a row.  Between the reduction and the epilogue a
// thread keeps its chunks as loaded (16 bytes for fp16 input, 32 bytes for fp32 input) and
// unpacks to fp32 at each use: half the registers of holding fp32 for the common fp16 case,
// which is what lets one warp own a whole 4096-element row with every load in flight.
template <typename InT>
struct RawChunk;
template <>
struct RawChunk<__half> {
  uint4 r;
  __device__ __forceinline__ void load(const __half* row, int c) {
    r = __ldcs(reinterpret_cast<const uint4*>(row) + c);
  }
  __device__ __forceinline__ void unpack(float* v) const {
    float2 a = h2f(r.x), b = h2f(r.y), d = h2f(r.z), e = h2f(r.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    v[4] = d.x; v[5] = d.y; v[6] = e.x; v[7] = e.y;
  }
  __device__ __forceinline__ void fill(float f) {
    const uint32_t h = f2h(f, f);
    r = make_uint4(h, h, h, h);
  }
};
template <>
struct RawChunk<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* row, int c) {
    a = __ldcs(reinterpret_cast<const float4*>(row) + 2 * c);
    b = __ldcs(reinterpret_cast<const float4*>(row) + 2 * c + 1);
  }
  __device__ __forceinline__ void unpack(float* v) const {
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
  __device__ __forceinline__ void fill(float f) {
    a = make_float4(f, f, f, f);
    b = a;
  }
};

__device__ __forceinline__ void store_chunk(__half* row, int c, const float* v) {
  uint4 w;
  w.x = f2h(v[0], v[1]);
  w.y = f2h(v[2], v[3]);
  w.z = f2h(v[4], v[5]);
  w.w = f2h(v[6], v[7]);
  __stcs(reinterpret_cast<uint4*>(row) + c, w);
}

// exp(x) for x <= 0 as 2^(x * log2 e) on the special-function unit.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct SumOp {
  __device__ __forceinline__ float operator()(float a, float b) const { return a + b; }
};
struct MaxOp {
  __device__ __forceinline__ float operator()(float a, float b) const { return fmaxf(a, b); }
};

// All-reduce of `v` over the TPR threads that own one row.  `scratch` holds one float
// per warp of the CTA and must not be reused before the next __syncthreads().
template <int TPR, typename F>
__device__ __forceinline__ float group_allreduce(float v, F f, float* scratch) {
  constexpr int kShfl = TPR < 32 ? TPR : 32;
#pragma unroll
  for (int o = kShfl / 2; o > 0; o >>= 1) v = f(v, __shfl_xor_sync(0xffffffffu, v, o));
  if constexpr (TPR > 32) {
    constexpr int kWarpsPerRow = TPR / 32;
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) scratch[warp] = v;
    __syncthreads();
    const int first = (warp / kWarpsPerRow) * kWarpsPerRow;
    float r = scratch[first];
#pragma unroll
    for (int i = 1; i < kWarpsPerRow; ++i) r = f(r, scratch[first + i]);
    v = r;
  }
  return v;
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kNegHuge = -3.4028234663852886e+38f;

// One row per TPR threads, up to MAXCH chunks per thread held in registers.
template <int OP, typename InT, int TPR, int MAXCH>
__global__ void __launch_bounds__(TPR > kCtaThreads ? TPR : kCtaThreads)
    row_regs_kernel(const InT* __restrict__ x, const void* __restrict__ p0,
                    const void* __restrict__ p1, __half* __restrict__ y, int64_t m, int n_cols,
                    float eps) {
  constexpr int kThreads = TPR > kCtaThreads ? TPR : kCtaThreads;
  constexpr int kRowsPerCta = kThreads / TPR;
  __shared__ float scratch_a[kThreads / 32];
  __shared__ float scratch_b[kThreads / 32];

  const int t = threadIdx.x % TPR;
  const int64_t row = (int64_t)blockIdx.x * kRowsPerCta + threadIdx.x / TPR;
  const bool live = row < m;
  const int n_chunks = n_cols >> 3;
  const InT* xr = x + (live ? row : 0) * (int64_t)n_cols;
  __half* yr = y + (live ? row : 0) * (int64_t)n_cols;

  pdl_wait();
  pdl_launch_dependents();
  RawChunk<InT> raw[MAXCH];
#pragma unroll
  for (int c = 0; c < MAXCH; ++c) {
    const int ch = c * TPR + t;
    if (live && ch < n_chunks)
      raw[c].load(xr, ch);
    else
      raw[c].fill(OP == ROW_SOFTMAX ? -65504.f : 0.f);   // neutral for max (fp16 lowest) / sums
  }

  if constexpr (OP == ROW_RMSNORM) {
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < MAXCH; ++c) {
      float v[8];
      raw[c].unpack(v);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
    }
    ss = group_allreduce<TPR>(ss, SumOp(), scratch_a);
    const float r = 1.0f / sqrtf(ss * (1.0f / (float)n_cols) + eps);
    const __half* w = static_cast<const __half*>(p0);
#pragma unroll
    for (int c = 0; c < MAXCH; ++c) {
      const int ch = c * TPR + t;
      if (live && ch < n_chunks) {
        float v[8], wv[8], o[8];
        raw[c].unpack(v);
        RawChunk<__half> wr;
        wr.r = __ldg(reinterpret_cast<const uint4*>(w) + ch);
        wr.unpack(wv);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __fmul_rn(__fmul_rn(v[i], r), wv[i]);
        store_chunk(yr, ch, o);
      }
    }
  } else if constexpr (OP == ROW_SOFTMAX) {
    float mx = kNegHuge;
#pragma unroll
    for (int c = 0; c < MAXCH; ++c) {
      const bool on = (c * TPR + t) < n_chunks;
      float v[8];
      raw[c].unpack(v);
#pragma unroll
      for (int i = 0; i < 8; ++i) mx = on ? fmaxf(mx, v[i]) : mx;
    }
    mx = group_allreduce<TPR>(mx, MaxOp(), scratch_a);
    // exp(x - mx) = 2^((x - mx) * log2e); the subtraction comes first so that rows with
    // large |x| keep full precision in the exponent.  With at most 4 chunks per thread the
    // 32 exponentials are parked in registers between the sum and the output; with more
    // they are evaluated twice (a second MUFU pass costs less than the registers).
    constexpr bool kKeep = MAXCH <= 4;
    float e[kKeep ? MAXCH : 1][8];
    float sum = 0.f;
#pragma unroll
    for (int c = 0; c < MAXCH; ++c) {
      const bool on = (c * TPR + t) < n_chunks;
      float v[8];
      raw[c].unpack(v);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float ev = on ? fast_exp2((v[i] - mx) * kLog2e) : 0.f;
        if constexpr (kKeep) e[c][i] = ev;
        sum += ev;
      }
    }
    sum = group_allreduce<TPR>(sum, SumOp(), scratch_b);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int c = 0; c < MAXCH; ++c) {
      const int ch = c * TPR + t;
      if (live && ch < n_chunks) {
        float o[8];
        if constexpr (kKeep) {
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = e[c][i] * inv;
        } else {
          float v[8];
          raw[c].unpack(v);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = fast_exp2((v[i] - mx) * kLog2e) * inv;
        }
        store_chunk(yr, ch, o);
      }
    }
  } else {  // ROW_LAYERNORM
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int c = 0; c < MAXCH; ++c) {
      float v[8];
      raw[c].unpack(v);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        s1 += v[i];
        s2 = fmaf(v[i], v[i], s2);
      }
    }
    s1 = group_allreduce<TPR>(s1, SumOp(), scratch_a);
    s2 = group_allreduce<TPR>(s2, SumOp(), scratch_b);
    const float inv_n = 1.0f / (float)n_cols;
    const float mean = s1 * inv_n;
    const float r = 1.0f / sqrtf(__fadd_rn(__fsub_rn(s2 * inv_n, __fmul_rn(mean, mean)), eps));
    const float* g = static_cast<const float*>(p0);
    const float* be = static_cast<const float*>(p1);
#pragma unroll
    for (int c = 0; c < MAXCH; ++c) {
      const int ch = c * TPR + t;
      if (live && ch < n_chunks) {
        float v[8], gv[8], bv[8], o[8];
        raw[c].unpack(v);
        RawChunk<float> gr, br;
        gr.a = __ldg(reinterpret_cast<const float4*>(g) + 2 * ch);
        gr.b = __ldg(reinterpret_cast<const float4*>(g) + 2 * ch + 1);
        br.a = __ldg(reinterpret_cast<const float4*>(be) + 2 * ch);
        br.b = __ldg(reinterpret_cast<const float4*>(be) + 2 * ch + 1);
        gr.unpack(gv);
        br.unpack(bv);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          o[i] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(v[i], mean), r), gv[i]), bv[i]);
        store_chunk(yr, ch, o);
      }
    }
  }
}

// Any n_cols / any alignment: one CTA per row, scalar accesses, the row re-read from
// global memory (L2) for each pass.  Only used when the vector path does not apply and the row
// is longer than row_elems_kernel holds in registers (4096 columns).
__device__ __forceinline__ float ld_as_f32(const __half* p, int64_t i) { return __half2float(p[i]); }
__device__ __forceinline__ float ld_as_f32(const float* p, int64_t i) { return p[i]; }

template <typename F>
__device__ __forceinline__ float cta_allreduce(float v, F f, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = f(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5;
  __syncthreads();  // scratch may still be read by the previous reduction
  if ((threadIdx.x & 31) == 0) scratch[warp] = v;
  __syncthreads();
  float r = scratch[0];
  for (int i = 1; i < kCtaThreads / 32; ++i) r = f(r, scratch[i]);
  return r;
}

template <int OP, typename InT>
__global__ void __launch_bounds__(kCtaThreads)
    row_generic_kernel(const InT* __restrict__ x, const void* __restrict__ p0,
                       const void* __restrict__ p1, __half* __restrict__ y, int64_t m,
                       int64_t n_cols, float eps) {
  __shared__ float scratch[kCtaThreads / 32];
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t row = blockIdx.x; row < m; row += gridDim.x) {
    const InT* xr = x + row * n_cols;
    __half* yr = y + row * n_cols;
    if constexpr (OP == ROW_RMSNORM) {
      float ss = 0.f;
      for (int64_t i = threadIdx.x; i < n_cols; i += kCtaThreads) {
        float a = ld_as_f32(xr, i);
        ss = fmaf(a, a, ss);
      }
      ss = cta_allreduce(ss, SumOp(), scratch);
      const float r = 1.0f / sqrtf(ss * (1.0f / (float)n_cols) + eps);
      const __half* w = static_cast<const __half*>(p0);
      for (int64_t i = threadIdx.x; i < n_cols; i += kCtaThreads)
        yr[i] = __float2half_rn(__fmul_rn(__fmul_rn(ld_as_f32(xr, i), r), __half2float(w[i])));
    } else if constexpr (OP == ROW_SOFTMAX) {
      float mx = -3.4028234663852886e+38f;
      for (int64_t i = threadIdx.x; i < n_cols; i += kCtaThreads) mx = fmaxf(mx, ld_as_f32(xr, i));
      mx = cta_allreduce(mx, MaxOp(), scratch);
      float sum = 0.f;
      for (int64_t i = threadIdx.x; i < n_cols; i += kCtaThreads)
        sum += __expf(ld_as_f32(xr, i) - mx);
      sum = cta_allreduce(sum, SumOp(), scratch);
      const float inv = 1.0f / sum;
      for (int64_t i = threadIdx.x; i < n_cols; i += kCtaThreads)
        yr[i] = __float2half_rn(__expf(ld_as_f32(xr, i) - mx) * inv);
    } else {
      float s1 = 0.f, s2 = 0.f;
      for (int64_t i = threadIdx.x; i < n_cols; i += kCtaThreads) {
        float a = ld_as_f32(xr, i);
        s1 += a;
        s2 = fmaf(a, a, s2);
      }
      s1 = cta_allreduce(s1, SumOp(), scratch);
      s2 = cta_allreduce(s2, SumOp(), scratch);
      const float inv_n = 1.0f / (float)n_cols;
      const float mean = s1 * inv_n;
      const float r = 1.0f / sqrtf(__fadd_rn(__fsub_rn(s2 * inv_n, __fmul_rn(mean, mean)), eps));
      const float* g = static_cast<const float*>(p0);
      const float* be = static_cast<const float*>(p1);
      for (int64_t i = threadIdx.x; i < n_cols; i += kCtaThreads)
        yr[i] = __float2half_rn(
            __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(ld_as_f32(xr, i), mean), r), g[i]), be[i]));
    }
  }
}

// Rows whose length or alignment rules out 16-byte vectors (n_cols not a multiple of 8: the
// reference sweeps softmax over reduction lengths such as 17, 1025 and 2049,
// experiment/dtas_tuned/general_reduction/softmax/profile_dlight.py:8-52), up to 4096 columns:
// the same one-read design with scalar accesses.  A row is owned by TPR threads, thread t holds
// elements t, t + TPR, ... (up to MAXE of them) in registers, so a warp's loads and stores are
// contiguous, HBM sees every element once in and once out, and short rows share a CTA (8 rows of
// up to 256 columns, 2 of up to 1024) instead of taking one each.  Measured on 12800 rows of
// fp32: 17 columns 15.5 -> 3.2 us, 1025 columns 36 -> 25 us against one CTA per row.
template <int OP, typename InT, int TPR, int MAXE>
__global__ void __launch_bounds__(kCtaThreads)
    row_elems_kernel(const InT* __restrict__ x, const void* __restrict__ p0,
                     const void* __restrict__ p1, __half* __restrict__ y, int64_t m, int n_cols,
                     float eps) {
  constexpr int kRowsPerCta = kCtaThreads / TPR;
  __shared__ float scratch_a[kCtaThreads / 32];
  __shared__ float scratch_b[kCtaThreads / 32];
  const int t = threadIdx.x % TPR;
  const int64_t row = (int64_t)blockIdx.x * kRowsPerCta + threadIdx.x / TPR;
  const bool live = row < m;
  const InT* xr = x + (live ? row : 0) * (int64_t)n_cols;
  __half* yr = y + (live ? row : 0) * (int64_t)n_cols;

  pdl_wait();
  pdl_launch_dependents();
  float v[MAXE];
#pragma unroll
  for (int j = 0; j < MAXE; ++j) {
    const int e = j * TPR + t;
    v[j] = (live && e < n_cols) ? ld_as_f32(xr, e) : 0.f;
  }

  if constexpr (OP == ROW_RMSNORM) {
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < MAXE; ++j) ss = fmaf(v[j], v[j], ss);
    ss = group_allreduce<TPR>(ss, SumOp(), scratch_a);
    const float r = 1.0f / sqrtf(ss * (1.0f / (float)n_cols) + eps);
    const __half* w = static_cast<const __half*>(p0);
#pragma unroll
    for (int j = 0; j < MAXE; ++j) {
      const int e = j * TPR + t;
      if (live && e < n_cols) yr[e] = __float2half_rn(__fmul_rn(__fmul_rn(v[j], r), __half2float(w[e])));
    }
  } else if constexpr (OP == ROW_SOFTMAX) {
    float mx = kNegHuge;
#pragma unroll
    for (int j = 0; j < MAXE; ++j) mx = (j * TPR + t) < n_cols ? fmaxf(mx, v[j]) : mx;
    mx = group_allreduce<TPR>(mx, MaxOp(), scratch_a);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < MAXE; ++j) {
      v[j] = (j * TPR + t) < n_cols ? fast_exp2((v[j] - mx) * kLog2e) : 0.f;
      sum += v[j];
    }
    sum = group_allreduce<TPR>(sum, SumOp(), scratch_b);
    const float inv = 1.0f / sum;
#pragma unroll
    for (int j = 0; j < MAXE; ++j) {
      const int e = j * TPR + t;
      if (live && e < n_cols) yr[e] = __float2half_rn(v[j] * inv);
    }
  } else {  // ROW_LAYERNORM
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < MAXE; ++j) {
      s1 += v[j];
      s2 = fmaf(v[j], v[j], s2);
    }
    s1 = group_allreduce<TPR>(s1, SumOp(), scratch_a);
    s2 = group_allreduce<TPR>(s2, SumOp(), scratch_b);
    const float inv_n = 1.0f / (float)n_cols;
    const float mean = s1 * inv_n;
    const float r = 1.0f / sqrtf(__fadd_rn(__fsub_rn(s2 * inv_n, __fmul_rn(mean, mean)), eps));
    const float* g = static_cast<const float*>(p0);
    const float* be = static_cast<const float*>(p1);
#pragma unroll
    for (int j = 0; j < MAXE; ++j) {
      const int e = j * TPR + t;
      if (live && e < n_cols)
        yr[e] = __float2half_rn(__fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(v[j], mean), r), g[e]), be[e]));
    }
  }
}

// ---- dispatch ------------------------------------------------------------------
// Threads per row (TPR) and chunks per thread (MAXCH), per m-bucket.  From a sweep on B200
// at 4096 columns (TPR 32..512, m = 33..8192): 256 threads per row up to m = 1024 (short
// dependent chains, the latency-bound regime: 2.0 us at m = 33 vs 6.0 us with one warp per
// row), 128 beyond (5.5 TB/s RMSNorm at m = 4096, 6.2 TB/s at m = 8192; one warp per row
// reaches 3.4 TB/s, 512 threads 3.5 TB/s).  TPR is raised when a row would not fit the
// register budget (16 chunks of fp16, 8 of fp32 per thread).
struct RowCfg {
  int tpr;
  int maxch;     // 2, 4, 8 or 16
  bool generic;
  int elems_tpr;  // generic rows of up to 4096 columns: threads per row of row_elems_kernel (0 = not used)
  int elems_max;  // ... and elements per thread (8 or 16)
};
std::atomic<int> g_row_tpr{0};

inline int pow2_ceil(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

inline RowCfg row_cfg(int64_t m, int64_t n_cols, bool vec_ok, int in_dtype) {
  RowCfg c{0, 0, false, 0, 0};
  if (!vec_ok || n_cols > 65536) {
    c.generic = true;
    // scalar loads put only 4 bytes per thread in flight, so long rows take a whole CTA each:
    // 128 threads x 32 elements ran a 2049-column softmax in 181 us, 256 x 16 in 44 us
    if (n_cols <= 256) { c.elems_tpr = 32; c.elems_max = 8; }
    else if (n_cols <= 1024) { c.elems_tpr = 128; c.elems_max = 8; }
    else if (n_cols <= 2048) { c.elems_tpr = 256; c.elems_max = 8; }
    else if (n_cols <= 4096) { c.elems_tpr = 256; c.elems_max = 16; }
    return c;
  }
  const int n_chunks = (int)(n_cols >> 3);
  const int bucket = bucket_of(m);
  // chunks a thread may hold without spilling: 16 of fp16 / 8 of fp32, half that in a
  // 1024-thread CTA (64 registers per thread)
  auto cap_for = [&](int tpr) {
    const int base = in_dtype == DTAS_F16 ? 16 : 8;
    return tpr >= 1024 ? base / 2 : base;
  };
  int max_tpr = pow2_ceil(n_chunks);
  if (max_tpr < 32) max_tpr = 32;
  if (max_tpr > 1024) max_tpr = 1024;
  int tpr = bucket <= 3 ? 256 : 128;
  const int forced = g_row_tpr.load();
  if (forced >= 32 && forced <= 1024 && (forced & (forced - 1)) == 0) tpr = forced;
  if (tpr > max_tpr) tpr = max_tpr;
  // from 512 rows up, at least two chunks per thread where the row has them: rows of 2-4 KB ran
  // 15-35 % faster with 32-64 threads than with 128 (12800 x 1024 fp16 softmax: 9.5 us against
  // 15.0); below that the launch is latency-bound and more threads per row are faster
  // (256 x 2560 fp32 layer norm: 2.2 us with 256 threads, 2.7 us with 128)
  if (forced == 0 && m >= 512) {
    int by_chunks = pow2_ceil(n_chunks / 2 + 1) / 2;   // largest power of two <= n_chunks / 2
    if (by_chunks < 32) by_chunks = 32;
    if (tpr > by_chunks) tpr = by_chunks;
  }
  while (tpr <= 1024 && (n_chunks + tpr - 1) / tpr > cap_for(tpr)) tpr *= 2;
  if (tpr > 1024) {
    c.generic = true;
    return c;
  }
  c.tpr = tpr;
  const int need = (n_chunks + tpr - 1) / tpr;
  c.maxch = need <= 2 ? 2 : (need <= 4 ? 4 : (need <= 8 ? 8 : 16));
  return c;
}

template <int OP, typename InT, int TPR, int MAXCH>
int launch_regs(const InT* x, const void* p0, const void* p1, __half* y, int64_t m, int n_cols,
                float eps, cudaStream_t st) {
  constexpr int kThreads = TPR > kCtaThreads ? TPR : kCtaThreads;
  constexpr int kRowsPerCta = kThreads / TPR;
  const int64_t grid = (m + kRowsPerCta - 1) / kRowsPerCta;
  if (grid > 0x7fffffffLL) DTAS_FAIL(DTAS_EINVAL, "row op: too many rows (%lld)", (long long)m);
  launch_kernel(row_regs_kernel<OP, InT, TPR, MAXCH>, (unsigned)grid, kThreads, 0, st, x, p0, p1, y, m, n_cols, eps);
  return after_launch("row_regs_kernel");
}

template <int OP, typename InT, int MAXCH>
int launch_tpr(int tpr, const InT* x, const void* p0, const void* p1, __half* y, int64_t m,
               int n_cols, float eps, cudaStream_t st) {
  switch (tpr) {
    case 32: return launch_regs<OP, InT, 32, MAXCH>(x, p0, p1, y, m, n_cols, eps, st);
    case 64: return launch_regs<OP, InT, 64, MAXCH>(x, p0, p1, y, m, n_cols, eps, st);
    case 128: return launch_regs<OP, InT, 128, MAXCH>(x, p0, p1, y, m, n_cols, eps, st);
    case 256: return launch_regs<OP, InT, 256, MAXCH>(x, p0, p1, y, m, n_cols, eps, st);
    case 512: return launch_regs<OP, InT, 512, MAXCH>(x, p0, p1, y, m, n_cols, eps, st);
    case 1024: return launch_regs<OP, InT, 1024, MAXCH>(x, p0, p1, y, m, n_cols, eps, st);
  }
  DTAS_FAIL(DTAS_EINVAL, "row op: bad threads-per-row %d", tpr);
}

template <int OP, typename InT>
int launch_typed(const RowCfg& c, const InT* x, const void* p0, const void* p1, __half* y,
                 int64_t m, int64_t n_cols, float eps, const DeviceCtx* ctx, cudaStream_t st) {
  if (c.generic && c.elems_tpr > 0) {
    const int64_t rows_per_cta = kCtaThreads / c.elems_tpr;
    const int64_t grid = (m + rows_per_cta - 1) / rows_per_cta;
    if (grid > 0x7fffffffLL) DTAS_FAIL(DTAS_EINVAL, "row op: too many rows (%lld)", (long long)m);
    const int nc = (int)n_cols;
    if (c.elems_tpr == 32)
      launch_kernel(row_elems_kernel<OP, InT, 32, 8>, (unsigned)grid, kCtaThreads, 0, st, x, p0, p1, y, m, nc, eps);
    else if (c.elems_tpr == 128)
      launch_kernel(row_elems_kernel<OP, InT, 128, 8>, (unsigned)grid, kCtaThreads, 0, st, x, p0, p1, y, m, nc, eps);
    else if (c.elems_max == 8)
      launch_kernel(row_elems_kernel<OP, InT, 256, 8>, (unsigned)grid, kCtaThreads, 0, st, x, p0, p1, y, m, nc, eps);
    else
      launch_kernel(row_elems_kernel<OP, InT, 256, 16>, (unsigned)grid, kCtaThreads, 0, st, x, p0, p1, y, m, nc, eps);
    return after_launch("row_elems_kernel");
  }
  if (c.generic) {
    int64_t grid = m < (int64_t)ctx->sm_count * 8 ? m : (int64_t)ctx->sm_count * 8;
    launch_kernel(row_generic_kernel<OP, InT>, (unsigned)grid, kCtaThreads, 0, st, x, p0, p1, y, m, n_cols, eps);
    return after_launch("row_generic_kernel");
  }
  switch (c.maxch) {
    case 2: return launch_tpr<OP, InT, 2>(c.tpr, x, p0, p1, y, m, (int)n_cols, eps, st);
    case 4: return launch_tpr<OP, InT, 4>(c.tpr, x, p0, p1, y, m, (int)n_cols, eps, st);
    case 8: return launch_tpr<OP, InT, 8>(c.tpr, x, p0, p1, y, m, (int)n_cols, eps, st);
    default:
      if constexpr (sizeof(InT) == 2)
        return launch_tpr<OP, InT, 16>(c.tpr, x, p0, p1, y, m, (int)n_cols, eps, st);
      else
        DTAS_FAIL(DTAS_EINVAL, "row op: 16 chunks per thread is an fp16-only configuration");
  }
}

template <int OP>
int launch_op(const RowCfg& c, const void* x, const void* p0, const void* p1, void* y, int64_t m,
              int64_t n_cols, float eps, int in_dtype, const DeviceCtx* ctx, cudaStream_t st) {
  if (in_dtype == DTAS_F16)
    return launch_typed<OP, __half>(c, (const __half*)x, p0, p1, (__half*)y, m, n_cols, eps, ctx, st);
  if (in_dtype == DTAS_F32)
    return launch_typed<OP, float>(c, (const float*)x, p0, p1, (__half*)y, m, n_cols, eps, ctx, st);
  DTAS_FAIL(DTAS_EUNSUPPORTED, "row op: unsupported input dtype %d", in_dtype);
}

bool row_vec_ok(RowOp op, const void* x, const void* p0, const void* p1, const void* y,
                int64_t n_cols, int in_dtype) {
  (void)in_dtype;
  bool ok = (n_cols % 8 == 0) && aligned16(x) && aligned16(y);
  if (op == ROW_RMSNORM) ok = ok && aligned16(p0);
  if (op == ROW_LAYERNORM) ok = ok && aligned16(p0) && aligned16(p1);
  return ok;
}

}  // namespace

int launch_row_op(RowOp op, const void* x, const void* p0, const void* p1, void* y, int64_t m,
                  int64_t n_cols, float eps, int in_dtype, const DeviceCtx* ctx, cudaStream_t st) {
  const RowCfg c = row_cfg(m, n_cols, row_vec_ok(op, x, p0, p1, y, n_cols, in_dtype), in_dtype);
  switch (op) {
    case ROW_RMSNORM: return launch_op<ROW_RMSNORM>(c, x, p0, p1, y, m, n_cols, eps, in_dtype, ctx, st);
    case ROW_SOFTMAX: return launch_op<ROW_SOFTMAX>(c, x, p0, p1, y, m, n_cols, eps, in_dtype, ctx, st);
    case ROW_LAYERNORM: return launch_op<ROW_LAYERNORM>(c, x, p0, p1, y, m, n_cols, eps, in_dtype, ctx, st);
  }
  DTAS_FAIL(DTAS_EINVAL, "row op: unknown op %d", (int)op);
}

void row_set_override(int tpr) { g_row_tpr.store(tpr); }

void row_variant_name(RowOp op, int64_t m, int64_t n_cols, char* buf, int len) {
  static const char* names[] = {"rms_norm", "softmax", "layer_norm"};
  const RowCfg c = row_cfg(m, n_cols, n_cols % 8 == 0, DTAS_F16);
  if (c.generic && c.elems_tpr > 0)
    snprintf(buf, len, "%s_generic_elems_tpr%d_e%d", names[op], c.elems_tpr, c.elems_max);
  else if (c.generic)
    snprintf(buf, len, "%s_generic_cta256", names[op]);
  else
    snprintf(buf, len, "%s_regs_tpr%d_ch%d", names[op], c.tpr, c.maxch);
}

}  // namespace dtas
