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
//
// Second kernel, for weights that do not fit the first kernel's two short waves well
// (gemv_f16_stream_kernel): one persistent CTA per SM owns a contiguous band of rows - a
// contiguous slab of W - and a producer thread streams it row by row into a shared-memory
// ring with bulk copies (one 8-22 KB copy per row, full DRAM pages, tens of KB in flight per
// SM without a register), while eight consumer warps take a row each from the ring and
// reduce it against x held in shared memory.  No second wave, no cross-CTA reduction.
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


// ---------------------------------------------------------------------------------------
// Streaming kernel: bulk copies into a ring of whole rows.
// ---------------------------------------------------------------------------------------
constexpr int kStreamConsumers = 8;                       // consumer warps
constexpr int kStreamThreads = 32 * (1 + kStreamConsumers);
constexpr int ERR_GEMV_PRODUCER = 0x201, ERR_GEMV_CONSUMER = 0x202;

__device__ __forceinline__ uint32_t sm_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void gv_mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void gv_mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void gv_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool gv_mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait (about a second): records `code` in the status word and returns false.
__device__ __noinline__ bool gv_mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  for (int i = 0; i < 64; ++i)
    if (gv_mbar_try_wait(bar, parity)) return true;
  uint64_t t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    for (int i = 0; i < 2048; ++i)
      if (gv_mbar_try_wait(bar, parity)) return true;
    uint64_t t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    if (t1 - t0 > 1000000000ull) {
      atomicExch(status, code);
      return false;
    }
  }
}
__device__ __forceinline__ void gv_bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Shared memory: x (k fp16), then STAGES buffers of `rps` consecutive rows each (one bulk copy:
// the rows of a band are contiguous in W), then the barriers.  Stage s is always consumed by
// consumer warp s % 8 (STAGES is a multiple of 8), which reduces its rows one after another.
template <int STAGES>
__global__ void __launch_bounds__(kStreamThreads, 1)
    gemv_f16_stream_kernel(const __half* __restrict__ x, const __half* __restrict__ w, const Epilogue epi,
                           void* __restrict__ y, int n, int k, int rps, int* status) {
  static_assert(STAGES % kStreamConsumers == 0, "stage -> warp mapping");
  extern __shared__ __align__(128) uint8_t gv_smem[];
  const uint32_t row_bytes = (uint32_t)k * 2u;
  const uint32_t stage_bytes = row_bytes * (uint32_t)rps;
  uint8_t* x_s = gv_smem;
  uint8_t* ring = gv_smem + row_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ring + (size_t)STAGES * stage_bytes);
  const uint32_t bar0 = sm_u32(bars);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (STAGES + s); };
  const uint32_t x_bar = bar0 + 8u * (2 * STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // this CTA's band of rows
  const int r0 = (int)(((int64_t)blockIdx.x * n) / gridDim.x);
  const int r1 = (int)(((int64_t)(blockIdx.x + 1) * n) / gridDim.x);
  const int rows = r1 - r0;
  const int items = (rows + rps - 1) / rps;       // stage fills: rps rows each, the last one maybe fewer

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      gv_mbar_init(full_bar(s), 1);
      gv_mbar_init(empty_bar(s), 1);
    }
    gv_mbar_init(x_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      gv_mbar_expect_tx(x_bar, row_bytes);
      gv_bulk_load(sm_u32(x_s), x, row_bytes, x_bar);
    }
    if (lane == 0) {                                // one thread: lanes that spin side by side slow each other
      bool ok = true;
      for (int i = 0; i < items && ok; ++i) {
        const int s = i % STAGES;
        const uint32_t parity = (uint32_t)(i / STAGES) & 1u;
        if (!gv_mbar_wait(empty_bar(s), parity ^ 1u, status, ERR_GEMV_PRODUCER)) { ok = false; break; }
        const uint32_t bytes = (uint32_t)min(rps, rows - i * rps) * row_bytes;
        gv_mbar_expect_tx(full_bar(s), bytes);
        gv_bulk_load(sm_u32(ring + (size_t)s * stage_bytes), w + (int64_t)(r0 + i * rps) * k, bytes, full_bar(s));
      }
    }
  } else {
    const int cw = warp - 1;
    const int n_chunks = k >> 3;
    const uint4* xv = reinterpret_cast<const uint4*>(x_s);
    bool ok = gv_mbar_wait(x_bar, 0u, status, ERR_GEMV_CONSUMER);
    for (int i = cw; i < items && ok; i += kStreamConsumers) {
      const int s = i % STAGES;
      const uint32_t parity = (uint32_t)(i / STAGES) & 1u;
      if (!gv_mbar_wait(full_bar(s), parity, status, ERR_GEMV_CONSUMER)) { ok = false; break; }
      const int nrows = min(rps, rows - i * rps);
      float mine = 0.f;                              // lane rr keeps the dot product of row rr of the stage
      for (int rr = 0; rr < nrows; ++rr) {
        const uint4* wv = reinterpret_cast<const uint4*>(ring + (size_t)s * stage_bytes + (size_t)rr * row_bytes);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        int c = lane;
        for (; c + 96 < n_chunks; c += 128) {
#pragma unroll
          for (int u = 0; u < 4; ++u) acc[u] = dot8(wv[c + 32 * u], xv[c + 32 * u], acc[u]);
        }
        for (; c < n_chunks; c += 32) acc[0] = dot8(wv[c], xv[c], acc[0]);
        float sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (lane == rr) mine = sum;
      }
      __syncwarp();                                   // every lane has read the stage
      if (lane == 0) gv_mbar_arrive(empty_bar(s));    // hand the stage back before the stores
      if (lane < nrows) {
        const int row = r0 + i * rps + lane;
        epi_store(epi, y, 0, 0, row, epi_value(epi, mine, 0, row));
      }
    }
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

// Ring depth of the streaming kernel for this shape, 0 = use the per-row kernel.  A row must fit a
// stage (16 stages up to K = 5632, 8 up to K = 11264 in ~200 KB of shared memory).  Override code
// 16 (dtas_gemv_set_override) forces the streaming kernel where it fits, 1/2/4/8 the per-row kernel.
constexpr int kStreamSmemMax = 200 * 1024;
// Measured on B200 against the per-row kernel (us): W[4096,4096] 7.4 vs 7.9, [11008,4096] 15.8 vs 17.1,
// [4096,11008] 16.1 vs 20.1, [32000,4096] 41.3 vs 44.0, [2048,4096] 4.9 vs 5.2; [1024,4096] 3.8 vs 3.2.
constexpr bool kStreamByDefault = true;
constexpr int64_t kStreamMinBytes = 16ll << 20;   // below that the per-row kernel's single wave is as good
constexpr int kStreamStageBytes16 = 11264, kStreamStageBytes8 = 22528;   // stage capacity at 16 / 8 stages
struct StreamPlan {
  int stages = 0;   // 0: use the per-row kernel
  int rps = 1;      // rows per stage
};
inline StreamPlan pick_stream(int64_t n, int64_t k, int sm_count) {
  (void)sm_count;
  StreamPlan p;
  const int forced = g_gemv_wpr.load();
  if (forced == 1 || forced == 2 || forced == 4 || forced == 8) return p;
  const int64_t row_bytes = 2 * k;
  // One thread issues a copy in ~0.2 us and an SM has to take in ~45 KB per us, so a copy should carry
  // two rows of 8 KB where the band of a CTA is long enough to still give every consumer warp two stage
  // fills (W[32000,4096]: 41.3 us with two rows per copy, 43.9 with one); short bands keep one row per
  // copy and the deeper ring (W[4096,4096]: 7.4-7.7 us against 8.1).  Rows under 5.5 KB always travel
  // several to a copy (W[4096,2560]: 6.2 us against 7.1; W[50280,2560]: 39.7 against 62.2).
  if (row_bytes > kStreamStageBytes8 || n < kStreamConsumers) return p;
  if (forced != 16 && !(kStreamByDefault && 2 * n * k >= kStreamMinBytes)) return p;
  const int64_t band = (n + sm_count - 1) / (sm_count > 0 ? sm_count : 1);
  const int64_t fit16 = kStreamStageBytes16 / row_bytes, fit8 = kStreamStageBytes8 / row_bytes;
  if (fit16 >= 2) {                    // short rows: as many as fill an 11 KB stage
    p.stages = 16;
    p.rps = (int)(fit16 < 32 ? fit16 : 32);        // one lane per row of a stage keeps its result
  } else if (fit8 >= 2 && band >= 2 * kStreamConsumers * fit8) {
    p.stages = 8;                      // 5.5-11 KB rows in a long band: two per copy, 8 deep stages
    p.rps = (int)fit8;
  } else {
    p.stages = fit16 >= 1 ? 16 : 8;
    p.rps = 1;
  }
  return p;
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
  const StreamPlan sp = pick_stream(n, k, ctx->sm_count);
  const int stream_stages = sp.stages;
  if (stream_stages > 0) {
    const size_t smem = (size_t)(1 + stream_stages * sp.rps) * (size_t)k * 2 + (size_t)(2 * stream_stages + 1) * 8 + 8;
    const int64_t bands = (n + kStreamConsumers - 1) / kStreamConsumers;      // at least a row per consumer warp
    const unsigned grid = (unsigned)(bands < ctx->sm_count ? bands : ctx->sm_count);
    int dev = 0;
    DTAS_CUDA(cudaGetDevice(&dev));
    static bool attr_set[2][64] = {{false}};
    if (stream_stages == 16) {
      if (dev < 64 && !attr_set[0][dev]) {
        DTAS_CUDA(cudaFuncSetAttribute(gemv_f16_stream_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmemMax));
        attr_set[0][dev] = true;
      }
      launch_kernel(gemv_f16_stream_kernel<16>, grid, kStreamThreads, smem, st, xp, wp, epi, y, (int)n, (int)k, sp.rps, ctx->status);
    } else {
      if (dev < 64 && !attr_set[1][dev]) {
        DTAS_CUDA(cudaFuncSetAttribute(gemv_f16_stream_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStreamSmemMax));
        attr_set[1][dev] = true;
      }
      launch_kernel(gemv_f16_stream_kernel<8>, grid, kStreamThreads, smem, st, xp, wp, epi, y, (int)n, (int)k, sp.rps, ctx->status);
    }
    return after_launch("gemv_f16_stream_kernel");
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
  const StreamPlan sp = pick_stream(n, k, ctx ? ctx->sm_count : 148);
  if (sp.stages > 0) {
    snprintf(buf, len, "gemv_stream_s%d_rows%d", sp.stages, sp.rps);
    return;
  }
  const int wpr = pick_wpr(n, k, ctx ? ctx->sm_count : 148);
  snprintf(buf, len, "gemv_vec16_wpr%d_unroll%d", wpr, pick_unroll(wpr));
}

}  // namespace dtas
