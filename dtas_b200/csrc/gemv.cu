// Decode-time GEMV: y[n] = sum_k W[n,k] * x[k] (+ bias[n]), fp16 in/out, fp32 accumulate.
//
// Counterpart of the reference GEMV template (python/dtas/schedule/tir_gemv.py:33-249):
// W rows streamed with 16-byte vector loads, the reduction over K split over the lanes
// of a warp (and over several warps for short N) and combined with shuffles.
//
// Design: the kernel is a pure stream over W (2*N*K bytes; x and y are noise), so the
// only goal is enough 16-byte loads in flight on every SM.  A row is owned by WPR warps
// (1, 2, 4 or 8) of a 256-thread CTA; each lane issues UNROLL independent 16-byte loads
// of W per step with the matching x chunks read through L1 (x is 8-22 KB and hot in
// L1/L2), accumulates 8 products per chunk in fp32, and the partials meet through warp
// shuffles and one shared-memory hop.  WPR is chosen from K alone (pick_wpr).
// Algorithmic bytes: 2*N*K + 2*K + 2*N.  Bound: HBM bandwidth.
#include "common.cuh"

namespace dtas {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ float dot8(uint4 w, uint4 x, float acc) {
  const __half2* wh = reinterpret_cast<const __half2*>(&w);
  const __half2* xh = reinterpret_cast<const __half2*>(&x);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 a = __half22float2(wh[i]);
    float2 b = __half22float2(xh[i]);
    acc = fmaf(a.x, b.x, acc);
    acc = fmaf(a.y, b.y, acc);
  }
  return acc;
}

template <int WPR, int UNROLL>
__global__ void __launch_bounds__(kThreads)
    gemv_f16_kernel(const __half* __restrict__ x, const __half* __restrict__ w, const Epilogue epi,
                    void* __restrict__ y, int n, int k) {
  constexpr int kRowsPerCta = kWarps / WPR;
  __shared__ float partial[kWarps];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kRowsPerCta + warp / WPR;
  const int part = warp % WPR;  // which K-slice of the row this warp owns
  const bool live = row < n;

  const int n_chunks = k >> 3;                       // 16-byte chunks per row
  const int per_part = (n_chunks + WPR - 1) / WPR;   // chunks per K-slice
  const int c0 = part * per_part;
  const int c1 = min(c0 + per_part, n_chunks);

  const uint4* wr = reinterpret_cast<const uint4*>(w + (int64_t)(live ? row : 0) * k);
  const uint4* xv = reinterpret_cast<const uint4*>(x);

  float acc[UNROLL];
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) acc[u] = 0.f;

  pdl_wait();
  pdl_launch_dependents();
  if (live) {
    int c = c0 + lane;
    // Full steps: UNROLL independent 16-byte loads of W per lane before any use.
    for (; c + (UNROLL - 1) * 32 < c1; c += UNROLL * 32) {
      uint4 wv[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) wv[u] = __ldcs(wr + c + u * 32);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) acc[u] = dot8(wv[u], __ldg(xv + c + u * 32), acc[u]);
    }
    for (; c < c1; c += 32) acc[0] = dot8(__ldcs(wr + c), __ldg(xv + c), acc[0]);
  }

  float s = 0.f;
#pragma unroll
  for (int u = 0; u < UNROLL; ++u) s += acc[u];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);

  if constexpr (WPR > 1) {
    if (lane == 0) partial[warp] = s;
    __syncthreads();
    if (part == 0 && lane == 0 && live) {
      float r = partial[warp];
#pragma unroll
      for (int i = 1; i < WPR; ++i) r += partial[warp + i];
      epi_store(epi, y, 0, 0, row, epi_value(epi, r, 0, row));
    }
  } else {
    if (lane == 0 && live) {
      epi_store(epi, y, 0, 0, row, epi_value(epi, s, 0, row));
    }
  }
}

// Any K / any alignment: one warp per row, scalar loads.
__global__ void __launch_bounds__(kThreads)
    gemv_f16_scalar_kernel(const __half* __restrict__ x, const __half* __restrict__ w, const Epilogue epi,
                           void* __restrict__ y, int n, int k) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarps + warp;
  float s = 0.f;
  pdl_wait();
  pdl_launch_dependents();
  if (row < n) {
    const __half* wr = w + (int64_t)row * k;
    for (int i = lane; i < k; i += 32) s = fmaf(__half2float(wr[i]), __half2float(x[i]), s);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0 && row < n) {
    epi_store(epi, y, 0, 0, row, epi_value(epi, s, 0, row));
  }
}

std::atomic<int> g_gemv_wpr{0}, g_gemv_unroll{0};

// Warps per row and loads in flight per lane.  Measured on B200 over the Llama-2-7B shapes
// and their 8-way column shards: the best point is always "one batch of four 16-byte loads
// per lane and done" - i.e. as many warps per row as it takes to bring a warp's K-slice
// down to 128 chunks (4 per lane), up to the 8 warps of a CTA.  Short-lived warps with
// short dependent chains beat fewer warps that loop (w4/u4 vs w1/u8 at 4096 x 4096:
// 8.0 us vs 9.6 us; at 32000 x 4096: 43.1 us vs 51.8 us).
inline int pick_wpr(int64_t n, int64_t k, int sm_count) {
  (void)n;
  (void)sm_count;
  const int forced = g_gemv_wpr.load();
  if (forced == 1 || forced == 2 || forced == 4 || forced == 8) return forced;
  const int64_t n_chunks = k >> 3;
  int wpr = 1;
  while (wpr < 8 && n_chunks / (wpr * 2) >= 128) wpr *= 2;
  return wpr;
}

inline int pick_unroll(int wpr) {
  (void)wpr;
  const int forced = g_gemv_unroll.load();
  if (forced == 4 || forced == 8) return forced;
  return 4;
}

}  // namespace

void gemv_set_override(int wpr, int unroll) {
  g_gemv_wpr.store(wpr);
  g_gemv_unroll.store(unroll);
}

int launch_gemv(const void* x, const void* w, const Epilogue& epi, void* y, int64_t n, int64_t k,
                const DeviceCtx* ctx, cudaStream_t st) {
  if (n > 0x7fffffffLL || k > 0x7fffffffLL) DTAS_FAIL(DTAS_EINVAL, "gemv: n or k too large");
  const __half* xp = (const __half*)x;
  const __half* wp = (const __half*)w;
  const bool vec_ok = (k % 8 == 0) && aligned16(x) && aligned16(w);
  if (!vec_ok) {
    const unsigned grid = (unsigned)((n + kWarps - 1) / kWarps);
    launch_kernel(gemv_f16_scalar_kernel, grid, kThreads, 0, st, xp, wp, epi, y, (int)n, (int)k);
    return after_launch("gemv_f16_scalar_kernel");
  }
  const int wpr = pick_wpr(n, k, ctx->sm_count);
  const int rows_per_cta = kWarps / wpr;
  const unsigned grid = (unsigned)((n + rows_per_cta - 1) / rows_per_cta);
  const int unroll = pick_unroll(wpr);
#define DTAS_GEMV_CASE(W, U)                                                                  \
  if (wpr == W && unroll == U) {                                                              \
    launch_kernel(gemv_f16_kernel<W, U>, grid, kThreads, 0, st, xp, wp, epi, y, (int)n, (int)k); \
    return after_launch("gemv_f16_kernel");                                                   \
  }
  DTAS_GEMV_CASE(1, 4) DTAS_GEMV_CASE(1, 8) DTAS_GEMV_CASE(2, 4) DTAS_GEMV_CASE(2, 8)
  DTAS_GEMV_CASE(4, 4) DTAS_GEMV_CASE(4, 8) DTAS_GEMV_CASE(8, 4) DTAS_GEMV_CASE(8, 8)
#undef DTAS_GEMV_CASE
  DTAS_FAIL(DTAS_EINVAL, "gemv: no kernel for wpr=%d unroll=%d", wpr, unroll);
}

void gemv_variant_name(int64_t n, int64_t k, const DeviceCtx* ctx, char* buf, int len) {
  if (k % 8 != 0) {
    snprintf(buf, len, "gemv_scalar_warp_per_row");
    return;
  }
  const int wpr = pick_wpr(n, k, ctx ? ctx->sm_count : 148);
  snprintf(buf, len, "gemv_vec16_wpr%d_unroll%d", wpr, pick_unroll(wpr));
}

}  // namespace dtas
