// Elementwise class: cast, add, copy.
//
// Counterpart of the kernels the reference generates from TIRElementwiseScheduler
// (python/dtas/schedule/tir_elementwise.py:22-47): the flat index space is cut into
// [grid, iterations, 256 threads, vector], with the vector width capped at 128 bits
// (python/dtas/policy/elementwise_config_emiter.py:9-33).  Here that is one
// grid-stride kernel template: every thread moves UNROLL 16-byte vectors per
// iteration (all loads issued before the first store, so a thread keeps
// UNROLL x 16..32 bytes in flight); by default the grid covers the data once (one tile
// per CTA), and the ragged tail and unaligned buffers take a scalar path.
//
// Algorithmic HBM bytes per element: cast f32->f16 6, cast f16->f32 6, add 3*size,
// copy 2*size.  The kernels are pure streams: their roofline is HBM bandwidth.
#include "common.cuh"

#include <type_traits>

namespace dtas {
namespace {

constexpr int kThreads = 256;

// H = true: evict-first streaming accesses (ld.global.cs / st.global.cs); H = false: plain.
template <bool H, typename V>
__device__ __forceinline__ V ld_stream(const V* p) {
  if constexpr (H) return __ldcs(p);
  else return *p;
}
template <bool H, typename V>
__device__ __forceinline__ void st_stream(V* p, V v) {
  if constexpr (H) __stcs(p, v);
  else *p = v;
}

__device__ __forceinline__ uint32_t pack_half2_rn(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);  // round-to-nearest-even, like a C cast
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_half2(uint32_t v) {
  return __half22float2(*reinterpret_cast<__half2*>(&v));
}
__device__ __forceinline__ uint32_t hadd2_bits(uint32_t a, uint32_t b) {
  __half2 r = __hadd2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

// Each Op describes one vector of work: Reg = registers held between load and store,
// kVec = elements per vector, scalar() = the one-element fallback.
struct CastF32F16 {
  static constexpr int kLoads = 2;   // 16-byte loads per vector
  static constexpr int kVec = 8;
  const float* a;
  __half* o;
  struct Reg { float4 lo, hi; };
  template <bool H>
  __device__ __forceinline__ void load(Reg& r, int64_t v) const {
    const float4* p = reinterpret_cast<const float4*>(a) + 2 * v;
    r.lo = ld_stream<H>(p);
    r.hi = ld_stream<H>(p + 1);
  }
  template <bool H>
  __device__ __forceinline__ void store(const Reg& r, int64_t v) const {
    uint4 w;
    w.x = pack_half2_rn(r.lo.x, r.lo.y);
    w.y = pack_half2_rn(r.lo.z, r.lo.w);
    w.z = pack_half2_rn(r.hi.x, r.hi.y);
    w.w = pack_half2_rn(r.hi.z, r.hi.w);
    st_stream<H>(reinterpret_cast<uint4*>(o) + v, w);
  }
  __device__ __forceinline__ void scalar(int64_t i) const { o[i] = __float2half_rn(a[i]); }
};

// A vector here is 4 elements (8 bytes in, 16 bytes out) so that a warp's stores are contiguous:
// with 8 elements per thread every thread writes 32 bytes as two 16-byte halves, each store
// instruction fills only half of every 32-byte sector it touches, and the kernel ran at
// 4.7 TB/s where the 4-element form reaches the add kernel's rate.
struct CastF16F32 {
  static constexpr int kLoads = 1;
  static constexpr int kVec = 4;
  static constexpr int kUnrollMul = 2;   // half the bytes per vector: twice the vectors in flight
  const __half* a;
  float* o;
  struct Reg { uint2 v; };
  template <bool H>
  __device__ __forceinline__ void load(Reg& r, int64_t v) const {
    r.v = ld_stream<H>(reinterpret_cast<const uint2*>(a) + v);
  }
  template <bool H>
  __device__ __forceinline__ void store(const Reg& r, int64_t v) const {
    float2 f0 = unpack_half2(r.v.x), f1 = unpack_half2(r.v.y);
    st_stream<H>(reinterpret_cast<float4*>(o) + v, make_float4(f0.x, f0.y, f1.x, f1.y));
  }
  __device__ __forceinline__ void scalar(int64_t i) const { o[i] = __half2float(a[i]); }
};

struct AddF16 {
  static constexpr int kLoads = 2;   // 16-byte loads per vector
  static constexpr int kVec = 8;
  const __half *a, *b;
  __half* o;
  struct Reg { uint4 x, y; };
  template <bool H>
  __device__ __forceinline__ void load(Reg& r, int64_t v) const {
    r.x = ld_stream<H>(reinterpret_cast<const uint4*>(a) + v);
    r.y = ld_stream<H>(reinterpret_cast<const uint4*>(b) + v);
  }
  template <bool H>
  __device__ __forceinline__ void store(const Reg& r, int64_t v) const {
    uint4 w;
    w.x = hadd2_bits(r.x.x, r.y.x);
    w.y = hadd2_bits(r.x.y, r.y.y);
    w.z = hadd2_bits(r.x.z, r.y.z);
    w.w = hadd2_bits(r.x.w, r.y.w);
    st_stream<H>(reinterpret_cast<uint4*>(o) + v, w);
  }
  __device__ __forceinline__ void scalar(int64_t i) const { o[i] = __hadd(a[i], b[i]); }
};

// out = a + b (+ c), summed in fp32 and rounded once: the residual adds behind a large GEMM when
// they run as their own pass (launch_add_residuals).  `out` may be `a`.
struct AddResF16 {
  static constexpr int kLoads = 3;
  static constexpr int kVec = 8;
  const __half *a, *b, *c;   // c may be null
  __half* o;
  struct Reg { uint4 x, y, z; };
  template <bool H>
  __device__ __forceinline__ void load(Reg& r, int64_t v) const {
    r.x = ld_stream<H>(reinterpret_cast<const uint4*>(a) + v);
    r.y = ld_stream<H>(reinterpret_cast<const uint4*>(b) + v);
    r.z = c != nullptr ? ld_stream<H>(reinterpret_cast<const uint4*>(c) + v) : make_uint4(0u, 0u, 0u, 0u);
  }
  static __device__ __forceinline__ uint32_t add3(uint32_t p, uint32_t q, uint32_t t) {
    const float2 fp = unpack_half2(p), fq = unpack_half2(q), ft = unpack_half2(t);
    return pack_half2_rn(fp.x + fq.x + ft.x, fp.y + fq.y + ft.y);
  }
  template <bool H>
  __device__ __forceinline__ void store(const Reg& r, int64_t v) const {
    uint4 w;
    w.x = add3(r.x.x, r.y.x, r.z.x);
    w.y = add3(r.x.y, r.y.y, r.z.y);
    w.z = add3(r.x.z, r.y.z, r.z.z);
    w.w = add3(r.x.w, r.y.w, r.z.w);
    st_stream<H>(reinterpret_cast<uint4*>(o) + v, w);
  }
  __device__ __forceinline__ void scalar(int64_t i) const {
    o[i] = __float2half_rn(__half2float(a[i]) + __half2float(b[i]) + (c != nullptr ? __half2float(c[i]) : 0.f));
  }
};

struct AddF32 {
  static constexpr int kLoads = 2;   // 16-byte loads per vector
  static constexpr int kVec = 4;
  const float *a, *b;
  float* o;
  struct Reg { float4 x, y; };
  template <bool H>
  __device__ __forceinline__ void load(Reg& r, int64_t v) const {
    r.x = ld_stream<H>(reinterpret_cast<const float4*>(a) + v);
    r.y = ld_stream<H>(reinterpret_cast<const float4*>(b) + v);
  }
  template <bool H>
  __device__ __forceinline__ void store(const Reg& r, int64_t v) const {
    st_stream<H>(reinterpret_cast<float4*>(o) + v,
              make_float4(__fadd_rn(r.x.x, r.y.x), __fadd_rn(r.x.y, r.y.y),
                          __fadd_rn(r.x.z, r.y.z), __fadd_rn(r.x.w, r.y.w)));
  }
  __device__ __forceinline__ void scalar(int64_t i) const { o[i] = __fadd_rn(a[i], b[i]); }
};

struct AddI8 {  // two's-complement wrap-around per byte, like the int8 PrimFunc
  static constexpr int kLoads = 2;   // 16-byte loads per vector
  static constexpr int kVec = 16;
  const int8_t *a, *b;
  int8_t* o;
  struct Reg { uint4 x, y; };
  template <bool H>
  __device__ __forceinline__ void load(Reg& r, int64_t v) const {
    r.x = ld_stream<H>(reinterpret_cast<const uint4*>(a) + v);
    r.y = ld_stream<H>(reinterpret_cast<const uint4*>(b) + v);
  }
  template <bool H>
  __device__ __forceinline__ void store(const Reg& r, int64_t v) const {
    uint4 w;
    w.x = __vadd4(r.x.x, r.y.x);
    w.y = __vadd4(r.x.y, r.y.y);
    w.z = __vadd4(r.x.z, r.y.z);
    w.w = __vadd4(r.x.w, r.y.w);
    st_stream<H>(reinterpret_cast<uint4*>(o) + v, w);
  }
  __device__ __forceinline__ void scalar(int64_t i) const {
    o[i] = (int8_t)((uint8_t)a[i] + (uint8_t)b[i]);
  }
};

struct CopyBytes {
  static constexpr int kLoads = 1;   // 16-byte loads per vector
  static constexpr int kVec = 16;
  const uint8_t* a;
  uint8_t* o;
  struct Reg { uint4 v; };
  template <bool H>
  __device__ __forceinline__ void load(Reg& r, int64_t v) const {
    r.v = ld_stream<H>(reinterpret_cast<const uint4*>(a) + v);
  }
  template <bool H>
  __device__ __forceinline__ void store(const Reg& r, int64_t v) const {
    st_stream<H>(reinterpret_cast<uint4*>(o) + v, r.v);
  }
  __device__ __forceinline__ void scalar(int64_t i) const { o[i] = a[i]; }
};

// Vector path: n_vec full vectors, then (n_elem - n_vec*kVec) tail elements handled
// by the first threads of block 0.
template <typename Op, int UNROLL, bool HINT>
__global__ void __launch_bounds__(kThreads) ew_vec_kernel(const Op op, int64_t n_vec,
                                                          int64_t n_elem) {
  constexpr int64_t kTile = (int64_t)kThreads * UNROLL;
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t base = (int64_t)blockIdx.x * kTile; base < n_vec;
       base += (int64_t)gridDim.x * kTile) {
    typename Op::Reg r[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      int64_t v = base + (int64_t)u * kThreads + threadIdx.x;
      if (v < n_vec) op.template load<HINT>(r[u], v);
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      int64_t v = base + (int64_t)u * kThreads + threadIdx.x;
      if (v < n_vec) op.template store<HINT>(r[u], v);
    }
  }
  if (blockIdx.x == 0) {
    int64_t i = n_vec * Op::kVec + threadIdx.x;
    if (i < n_elem) op.scalar(i);  // tail is shorter than one vector (< 256 elements)
  }
}

// Scalar path for buffers that are not 16-byte aligned.
template <typename Op>
__global__ void __launch_bounds__(kThreads) ew_scalar_kernel(const Op op, int64_t n_elem) {
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n_elem;
       i += (int64_t)gridDim.x * kThreads)
    op.scalar(i);
}

// Per-bucket launch shape, the static counterpart of the reference's per-range best
// ElementwiseConfig (python/dtas/common/config.py:407-429).  Small buckets spread the
// few vectors over as many CTAs as possible (latency-bound); large buckets use deeper
// per-thread unrolling and a grid capped at a multiple of the SM count.
struct EwCfg {
  int unroll;        // 1, 2, 4 or 8 vectors in flight per thread
  int ctas_per_sm;   // grid cap as a multiple of the SM count; <= 0: one tile per CTA, no cap
  bool hints;        // streaming cache hints
};
std::atomic<int> g_ew_unroll{0}, g_ew_ctas{0}, g_ew_hints{-1};

// Defaults, from a sweep on B200 (unroll 1/2/4/8 x grid cap 4/8/16 CTAs per SM or none x
// hints on/off, at m = 64 ... 8192): one tile per CTA with no cap on the grid beats every
// capped, looping grid (copy [8192,11008]: 6.69 TB/s uncapped vs 5.8-6.4 capped), two
// 16-byte loads in flight per thread are enough (copy: two vectors; add and cast already
// load two per vector), streaming hints are worth 0-2 %.  The grid-stride loop stays: it is
// what makes a capped grid (override, or a grid beyond 2^31 tiles) correct.
inline EwCfg ew_cfg(int bucket, int loads_per_vec) {
  EwCfg c{loads_per_vec >= 2 ? 1 : 2, -1, true};
  if (bucket <= 0 && loads_per_vec < 2) c.unroll = 1;   // a few KB: spread over as many CTAs as possible
  const int u = g_ew_unroll.load(), g = g_ew_ctas.load(), h = g_ew_hints.load();
  if (u == 1 || u == 2 || u == 4 || u == 8) c.unroll = u;
  if (g != 0) c.ctas_per_sm = g;
  if (h >= 0) c.hints = h != 0;
  return c;
}

template <typename Op, int UNROLL>
void launch_vec(const Op& op, int64_t n_vec, int64_t n_elem, unsigned blocks, bool hints, cudaStream_t st) {
  if (hints)
    launch_kernel(ew_vec_kernel<Op, UNROLL, true>, blocks, kThreads, 0, st, op, n_vec, n_elem);
  else
    launch_kernel(ew_vec_kernel<Op, UNROLL, false>, blocks, kThreads, 0, st, op, n_vec, n_elem);
}

// Ops whose vector is narrower than 16 bytes on one side ask for more vectors per thread.
template <typename Op, typename = void>
struct UnrollMul { static constexpr int v = 1; };
template <typename Op>
struct UnrollMul<Op, std::void_t<decltype(Op::kUnrollMul)>> { static constexpr int v = Op::kUnrollMul; };

template <typename Op>
int launch_ew(const Op& op, int64_t n_elem, bool aligned, const DeviceCtx* ctx, cudaStream_t st,
              int bucket, const char* name) {
  if (!aligned) {
    int64_t blocks = (n_elem + kThreads - 1) / kThreads;
    int64_t cap = (int64_t)ctx->sm_count * 8;
    launch_kernel(ew_scalar_kernel<Op>, (unsigned)(blocks < cap ? blocks : cap), kThreads, 0, st, op, n_elem);
    return after_launch(name);
  }
  const int64_t n_vec = n_elem / Op::kVec;
  EwCfg cfg = ew_cfg(bucket, Op::kLoads);
  if (UnrollMul<Op>::v > 1 && g_ew_unroll.load() == 0)
    cfg.unroll = cfg.unroll * UnrollMul<Op>::v > 8 ? 8 : cfg.unroll * UnrollMul<Op>::v;
  const int64_t tile = (int64_t)kThreads * cfg.unroll;
  int64_t blocks = (n_vec + tile - 1) / tile;
  if (cfg.ctas_per_sm > 0) {
    const int64_t cap = (int64_t)ctx->sm_count * cfg.ctas_per_sm;
    if (blocks > cap) blocks = cap;
  }
  if (blocks > 0x7fffffffLL) blocks = 0x7fffffffLL;
  if (blocks < 1) blocks = 1;
  switch (cfg.unroll) {
    case 1: launch_vec<Op, 1>(op, n_vec, n_elem, (unsigned)blocks, cfg.hints, st); break;
    case 2: launch_vec<Op, 2>(op, n_vec, n_elem, (unsigned)blocks, cfg.hints, st); break;
    case 4: launch_vec<Op, 4>(op, n_vec, n_elem, (unsigned)blocks, cfg.hints, st); break;
    default: launch_vec<Op, 8>(op, n_vec, n_elem, (unsigned)blocks, cfg.hints, st); break;
  }
  return after_launch(name);
}

}  // namespace

int launch_cast(const void* a, void* out, int64_t n, int src, int dst, const DeviceCtx* ctx,
                cudaStream_t st, int bucket) {
  const bool al = aligned16(a) && aligned16(out);
  if (src == DTAS_F32 && dst == DTAS_F16)
    return launch_ew(CastF32F16{(const float*)a, (__half*)out}, n, al, ctx, st, bucket,
                     "cast_f32_f16");
  if (src == DTAS_F16 && dst == DTAS_F32)
    return launch_ew(CastF16F32{(const __half*)a, (float*)out}, n, al, ctx, st, bucket,
                     "cast_f16_f32");
  DTAS_FAIL(DTAS_EUNSUPPORTED, "cast: unsupported dtype pair %d -> %d", src, dst);
}

int launch_add(const void* a, const void* b, void* out, int64_t n, int dt, const DeviceCtx* ctx,
               cudaStream_t st, int bucket) {
  const bool al = aligned16(a) && aligned16(b) && aligned16(out);
  switch (dt) {
    case DTAS_F16:
      return launch_ew(AddF16{(const __half*)a, (const __half*)b, (__half*)out}, n, al, ctx, st,
                       bucket, "add_f16");
    case DTAS_F32:
      return launch_ew(AddF32{(const float*)a, (const float*)b, (float*)out}, n, al, ctx, st,
                       bucket, "add_f32");
    case DTAS_I8:
      return launch_ew(AddI8{(const int8_t*)a, (const int8_t*)b, (int8_t*)out}, n, al, ctx, st,
                       bucket, "add_i8");
  }
  DTAS_FAIL(DTAS_EUNSUPPORTED, "add: unsupported dtype %d", dt);
}

int launch_add_residuals(void* y, const void* res1, const void* res2, int64_t n, const DeviceCtx* ctx,
                         cudaStream_t st, int bucket) {
  const bool al = aligned16(y) && aligned16(res1) && (res2 == nullptr || aligned16(res2));
  return launch_ew(AddResF16{(const __half*)y, (const __half*)res1, (const __half*)res2, (__half*)y}, n, al, ctx, st,
                   bucket, "add_residuals_f16");
}

int launch_copy(const void* a, void* out, int64_t nbytes, const DeviceCtx* ctx, cudaStream_t st,
                int bucket) {
  const bool al = aligned16(a) && aligned16(out);
  return launch_ew(CopyBytes{(const uint8_t*)a, (uint8_t*)out}, nbytes, al, ctx, st, bucket,
                   "copy");
}

const char* ew_variant_name(const char* op, int64_t m, int64_t, const DeviceCtx*) {
  const int loads = (op != nullptr && strcmp(op, "copy") == 0) ? 1 : 2;
  switch (ew_cfg(bucket_of(m), loads).unroll) {
    case 1: return "ew_vec16_unroll1";
    case 2: return "ew_vec16_unroll2";
    case 4: return "ew_vec16_unroll4";
    default: return "ew_vec16_unroll8";
  }
}

void ew_set_override(int unroll, int ctas_per_sm, int hints) {
  g_ew_unroll.store(unroll);
  g_ew_ctas.store(ctas_per_sm);
  g_ew_hints.store(hints);
}

}  // namespace dtas
