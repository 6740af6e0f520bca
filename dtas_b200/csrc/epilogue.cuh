// What happens to a GEMM / GEMV accumulator before it is stored: the fused tails of the
// reference's real workloads
//   fused_NT_matmul_add                  y = mm + bias
//   fused_NT_matmul3_add2_gelu           y = gelu(mm + bias)
//   fused_NT_matmul2_add1_add3_add3      y = (res1 + (mm + bias)) + res2
//   fused_NT_matmul2_add1_add3_add3_cast the same, widened to fp32
// (experiment/ModelIR/dolly-v2-3b-q0f16/before_dl.py:552-573, 248-318, 163-200, 202-246; the
// decode-time GEMV forms at :96-114, 408-440, 442-481, 483-550).  The reference rounds every
// intermediate to fp16; here the chain is evaluated in fp32 on the fp32 accumulator and rounded
// to fp16 once, which is the closer of the two to exact arithmetic.  An fp32 output holds that
// fp16 value widened, as the reference's trailing cast does.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/dtas_b200.h"

namespace dtas {

struct Epilogue {
  const __half* bias = nullptr;   // [n], optional
  const __half* res1 = nullptr;   // [m, n], rows ldr elements apart, optional
  const __half* res2 = nullptr;   // [m, n], same stride, optional
  int64_t ldr = 0;
  int act = DTAS_ACT_NONE;
  int out_f32 = 0;                // 0: Y is fp16, 1: Y is fp32
  int vec_res = 0;                // 16-byte loads from residual rows are aligned (set by the launcher)
};

// Further copies of Y: base pointers of buffers with Y's layout (same row stride, same dtype) in which
// every stored vector is stored again.  With the output columns of a GEMM sharded over g GPUs these are
// the places of this rank's slab in the other ranks' gather buffers (peer memory mapped into this
// process), so the gather rides on the epilogue of the GEMM tile by tile instead of following it.
// `mc`, when set, is the address of the same slab in a multicast mapping that covers this GPU's buffer
// and every peer's (an NVLink SHARP multicast object): one multimem.st there lands in all of them, the
// switch doing the fan-out, so whole staged blocks leave as one store per vector instead of 1 + n.
struct PeerOut {
  void* y[DTAS_MAX_PEERS] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  int n = 0;
  void* mc = nullptr;
};

// Host and device: true when finishing an element costs more than a bias add and a store.
inline __host__ __device__ bool epi_has_work(const Epilogue& e) { return e.act != DTAS_ACT_NONE || e.res1 != nullptr; }

#ifdef __CUDACC__
// GELU, erf form: x * (0.5 + 0.5 * erf(x / sqrt(2))), as the reference's workload spells it
// (before_dl.py:272-318).  erf by the rational approximation 7.1.26 of Abramowitz & Stegun,
//   erf(z) = 1 - (a1 t + ... + a5 t^5) exp(-z^2),  t = 1 / (1 + p z),  z >= 0,
// |error| <= 1.5e-7 in exact arithmetic and ~5e-7 here: three orders of magnitude under the fp16
// rounding of the result.  It is branch-free, and it is written for N elements side by side,
// stage by stage: the four epilogue warps of a CTA have a scheduler each, so nothing but
// instruction-level parallelism hides the ~100-cycle dependent chain of one element (with a
// per-element erff the epilogue of a 256 x 256 tile took longer than its main loop at K = 2560).
__device__ __forceinline__ float epi_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float epi_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <int N>
__device__ __forceinline__ void gelu_erf_n(float* v) {
  float z[N], t[N], e[N], p[N];
#pragma unroll
  for (int j = 0; j < N; ++j) z[j] = fabsf(v[j]) * 0.70710678118654757f;
#pragma unroll
  for (int j = 0; j < N; ++j) t[j] = epi_rcp(fmaf(0.3275911f, z[j], 1.0f));
#pragma unroll
  for (int j = 0; j < N; ++j) e[j] = epi_ex2(-1.4426950408889634f * z[j] * z[j]);
#pragma unroll
  for (int j = 0; j < N; ++j) p[j] = fmaf(1.061405429f, t[j], -1.453152027f);
#pragma unroll
  for (int j = 0; j < N; ++j) p[j] = fmaf(p[j], t[j], 1.421413741f);
#pragma unroll
  for (int j = 0; j < N; ++j) p[j] = fmaf(p[j], t[j], -0.284496736f);
#pragma unroll
  for (int j = 0; j < N; ++j) p[j] = fmaf(p[j], t[j], 0.254829592f);
#pragma unroll
  for (int j = 0; j < N; ++j) {
    const float erf_abs = fmaf(-p[j] * t[j], e[j], 1.0f);            // erf(|x| / sqrt(2))
    v[j] = v[j] * fmaf(0.5f, copysignf(erf_abs, v[j]), 0.5f);
  }
}
__device__ __forceinline__ float gelu_erf(float x) {
  gelu_erf_n<1>(&x);
  return x;
}

// What follows the bias: activation, then the residuals.
__device__ __forceinline__ float epi_tail(const Epilogue& e, float t, int64_t row, int col) {
  if (e.act == DTAS_ACT_GELU) t = gelu_erf(t);
  if (e.res1 != nullptr) t += __half2float(e.res1[row * e.ldr + col]);
  if (e.res2 != nullptr) t += __half2float(e.res2[row * e.ldr + col]);
  return t;
}
// Value of one output element from its fp32 dot product.
__device__ __forceinline__ float epi_value(const Epilogue& e, float acc, int64_t row, int col) {
  if (e.bias != nullptr) acc += __half2float(e.bias[col]);
  return epi_tail(e, acc, row, col);
}

__device__ __forceinline__ void epi_store(const Epilogue& e, void* y, int64_t ldy, int64_t row, int col, float v) {
  const __half h = __float2half_rn(v);
  if (e.out_f32) static_cast<float*>(y)[row * ldy + col] = __half2float(h);
  else static_cast<__half*>(y)[row * ldy + col] = h;
}

// COUNT consecutive rows row0, row0+1, ... of one output column; v[] holds dot product + bias.
template <int COUNT>
__device__ __forceinline__ void epi_store_column(const Epilogue& e, void* y, int64_t ldy, int row0, int m, int col,
                                                 const float* v) {
  if (e.act == DTAS_ACT_NONE && e.res1 == nullptr && !e.out_f32) {   // plain fp16 result: nothing but the store
    __half* yc = static_cast<__half*>(y) + col;
#pragma unroll
    for (int j = 0; j < COUNT; ++j)
      if (row0 + j < m) yc[(int64_t)(row0 + j) * ldy] = __float2half_rn(v[j]);
  } else {
    // all residual values first, then the stores: a store in between would make every row wait for
    // its own loads (the compiler cannot move loads over stores that might alias)
    float r1[COUNT], r2[COUNT];
#pragma unroll
    for (int j = 0; j < COUNT; ++j) {
      const bool on = row0 + j < m;
      r1[j] = (on && e.res1 != nullptr) ? __half2float(e.res1[(int64_t)(row0 + j) * e.ldr + col]) : 0.f;
      r2[j] = (on && e.res2 != nullptr) ? __half2float(e.res2[(int64_t)(row0 + j) * e.ldr + col]) : 0.f;
    }
    float t[COUNT];
#pragma unroll
    for (int j = 0; j < COUNT; ++j) t[j] = v[j];
    if (e.act == DTAS_ACT_GELU) {
      constexpr int kGroup = COUNT % 8 == 0 ? 8 : COUNT;
#pragma unroll
      for (int g = 0; g < COUNT; g += kGroup) gelu_erf_n<kGroup>(t + g);
    }
#pragma unroll
    for (int j = 0; j < COUNT; ++j)
      if (row0 + j < m) epi_store(e, y, ldy, row0 + j, col, (t[j] + r1[j]) + r2[j]);
  }
}

// Residual values of one 32-column chunk of one row, fetched ahead of use: 4 x 16 bytes per residual.
struct ResChunk {
  uint4 v[2][4];
};
// Whether chunk col0 .. col0+31 of a row can be fetched with 16-byte loads (else it is read in place).
__device__ __forceinline__ bool epi_can_prefetch(const Epilogue& e, int col0, int n) {
  return e.res1 != nullptr && e.vec_res && col0 + 32 <= n;
}
__device__ __forceinline__ void epi_prefetch_res32(const Epilogue& e, int64_t row, int col0, ResChunk& r) {
  const uint4* s1 = reinterpret_cast<const uint4*>(e.res1 + row * e.ldr + col0);
#pragma unroll
  for (int q = 0; q < 4; ++q) r.v[0][q] = s1[q];
  if (e.res2 != nullptr) {
    const uint4* s2 = reinterpret_cast<const uint4*>(e.res2 + row * e.ldr + col0);
#pragma unroll
    for (int q = 0; q < 4; ++q) r.v[1][q] = s2[q];
  }
}
__device__ __forceinline__ void epi_add_vec32(const uint4* v, float* acc32) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const __half2* h = reinterpret_cast<const __half2*>(&v[q]);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      acc32[8 * q + 2 * i] += f.x;
      acc32[8 * q + 2 * i + 1] += f.y;
    }
  }
}

// bias[col0 .. col0 + 31] added to 32 fp32 values of one row.  Every lane reads the same addresses;
// a whole chunk of an aligned bias comes in four 16-byte loads instead of 32 two-byte ones.
__device__ __forceinline__ void epi_add_bias32(const __half* bias, int col0, int n, float* acc32) {
  if (col0 + 32 <= n && (reinterpret_cast<uintptr_t>(bias + col0) & 15) == 0) {
    const uint4* src = reinterpret_cast<const uint4*>(bias + col0);
    uint4 v[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) v[q] = __ldg(src + q);
    epi_add_vec32(v, acc32);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < n) acc32[j] += __half2float(bias[col0 + j]);
  }
}

__device__ __forceinline__ void epi_add_res32(const __half* res, int64_t off, int col0, int n, int vec, float* acc32) {
  if (vec && col0 + 32 <= n) {
    const uint4* src = reinterpret_cast<const uint4*>(res + off + col0);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint4 v = src[q];
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        acc32[8 * q + 2 * i] += f.x;
        acc32[8 * q + 2 * i + 1] += f.y;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < n) acc32[j] += __half2float(res[off + col0 + j]);
  }
}

// True when the tail is nothing but an optional bias and an fp16 store: the path every plain GEMM
// takes, kept free of the machinery below.
__device__ __forceinline__ bool epi_is_plain(const Epilogue& e) {
  return e.res1 == nullptr && e.act == DTAS_ACT_NONE && !e.out_f32;
}
// The plain tail for 32 consecutive columns of one row, from the raw accumulator words.
__device__ __forceinline__ void epi_store_row32_plain(const __half* bias, __half* yrow, int vec_store, int col0, int n,
                                                      uint32_t* r, const PeerOut* peers = nullptr, int64_t row_off = 0) {
  if (bias != nullptr) epi_add_bias32(bias, col0, n, reinterpret_cast<float*>(r));
  const int n_peers = peers != nullptr ? peers->n : 0;
  if (vec_store && col0 + 32 <= n) {
    uint4 v[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      __half2 h0 = __floats2half2_rn(__uint_as_float(r[8 * q + 0]), __uint_as_float(r[8 * q + 1]));
      __half2 h1 = __floats2half2_rn(__uint_as_float(r[8 * q + 2]), __uint_as_float(r[8 * q + 3]));
      __half2 h2 = __floats2half2_rn(__uint_as_float(r[8 * q + 4]), __uint_as_float(r[8 * q + 5]));
      __half2 h3 = __floats2half2_rn(__uint_as_float(r[8 * q + 6]), __uint_as_float(r[8 * q + 7]));
      v[q].x = *reinterpret_cast<uint32_t*>(&h0);
      v[q].y = *reinterpret_cast<uint32_t*>(&h1);
      v[q].z = *reinterpret_cast<uint32_t*>(&h2);
      v[q].w = *reinterpret_cast<uint32_t*>(&h3);
    }
    uint4* dst = reinterpret_cast<uint4*>(yrow + col0);
#pragma unroll
    for (int q = 0; q < 4; ++q) dst[q] = v[q];
    for (int p = 0; p < n_peers; ++p) {
      uint4* pd = reinterpret_cast<uint4*>(static_cast<__half*>(peers->y[p]) + row_off + col0);
#pragma unroll
      for (int q = 0; q < 4; ++q) pd[q] = v[q];
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < n) {
        const __half h = __float2half_rn(__uint_as_float(r[j]));
        yrow[col0 + j] = h;
        for (int p = 0; p < n_peers; ++p) static_cast<__half*>(peers->y[p])[row_off + col0 + j] = h;
      }
  }
}

// The arithmetic of the tail on 32 consecutive columns of one row, in place: bias, activation,
// residuals.  `pre`, when given, holds the residual values of this chunk fetched earlier.
__device__ __forceinline__ void epi_apply_row32(const Epilogue& e, int64_t row, int col0, int n, float* acc32,
                                                const ResChunk* pre = nullptr) {
  if (e.bias != nullptr) epi_add_bias32(e.bias, col0, n, acc32);
  if (e.act == DTAS_ACT_GELU) {
#pragma unroll
    for (int g = 0; g < 32; g += 8) gelu_erf_n<8>(acc32 + g);   // groups of 4 time the same, of 16 slower
  }
  if (pre != nullptr) {
    epi_add_vec32(pre->v[0], acc32);
    if (e.res2 != nullptr) epi_add_vec32(pre->v[1], acc32);
  } else {
    if (e.res1 != nullptr) epi_add_res32(e.res1, row * e.ldr, col0, n, e.vec_res, acc32);
    if (e.res2 != nullptr) epi_add_res32(e.res2, row * e.ldr, col0, n, e.vec_res, acc32);
  }
}
// 16 bytes (eight fp16 values) to a multicast address: stored into every buffer the mapping covers.
__device__ __forceinline__ void epi_multimem_st16(void* addr, const uint4& v) {
  asm volatile("multimem.st.weak.global.v4.f16x2 [%0], {%1, %2, %3, %4};"
               :
               : "l"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// Eight fp32 values -> one 16-byte vector of fp16.
__device__ __forceinline__ uint4 epi_pack8(const float* f) {
  uint4 v;
  __half2 h0 = __floats2half2_rn(f[0], f[1]);
  __half2 h1 = __floats2half2_rn(f[2], f[3]);
  __half2 h2 = __floats2half2_rn(f[4], f[5]);
  __half2 h3 = __floats2half2_rn(f[6], f[7]);
  v.x = *reinterpret_cast<uint32_t*>(&h0);
  v.y = *reinterpret_cast<uint32_t*>(&h1);
  v.z = *reinterpret_cast<uint32_t*>(&h2);
  v.w = *reinterpret_cast<uint32_t*>(&h3);
  return v;
}
// Row-contiguous stores of a block of 32 rows x (8 * CPR) fp16 columns that the 32 lanes of a warp
// (lane = row) have parked in shared memory as 16-byte vectors at stage[row * CPR + (chunk ^ (row & 7))]:
// every store instruction of the warp now writes 32 / CPR whole rows of 16 * CPR contiguous bytes (full
// 128-byte lines), to Y and to every further copy of Y.  Both the parking writes (a quarter warp = 8
// rows, one chunk) and these reads (a quarter warp = 8 chunks of a row) cover all 32 banks.
template <int CPR>
__device__ __forceinline__ void epi_store_staged_block(const uint4* stage, int lane, int64_t row_base, int m, void* y,
                                                       int64_t ldy, int col0, const PeerOut& peers) {
  constexpr int kRowsPerInstr = 32 / CPR;
  const int ch = lane % CPR;
#pragma unroll 4
  for (int it = 0; it < CPR; ++it) {
    const int rl = kRowsPerInstr * it + lane / CPR;
    const int64_t grow = row_base + rl;
    if (grow < m) {
      const uint4 v = stage[rl * CPR + (ch ^ (rl & 7))];
      const int64_t off = grow * ldy + col0 + ch * 8;
      if (peers.mc != nullptr) {
        epi_multimem_st16(static_cast<__half*>(peers.mc) + off, v);     // this GPU's copy included
      } else {
        *reinterpret_cast<uint4*>(static_cast<__half*>(y) + off) = v;
        for (int p = 0; p < peers.n; ++p) *reinterpret_cast<uint4*>(static_cast<__half*>(peers.y[p]) + off) = v;
      }
    }
  }
}

// Finishes 32 consecutive output columns col0 .. col0+31 of one row held in acc32 (fp32 dot
// products) and stores them.  vec_store: 16-byte stores into Y rows are aligned.  `pre`, when
// given, holds the residual values of this chunk fetched earlier (epi_prefetch_res32).
__device__ __forceinline__ void epi_store_row32(const Epilogue& e, void* y, int64_t ldy, int vec_store, int64_t row,
                                                int col0, int n, float* acc32, const ResChunk* pre = nullptr,
                                                const PeerOut* peers = nullptr) {
  const int n_peers = peers != nullptr ? peers->n : 0;
  epi_apply_row32(e, row, col0, n, acc32, pre);
  const bool full = vec_store && col0 + 32 <= n;
  if (!e.out_f32) {
    __half* yrow = static_cast<__half*>(y) + row * ldy;
    if (full) {
      uint4* dst = reinterpret_cast<uint4*>(yrow + col0);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 v;
        __half2 h0 = __floats2half2_rn(acc32[8 * q + 0], acc32[8 * q + 1]);
        __half2 h1 = __floats2half2_rn(acc32[8 * q + 2], acc32[8 * q + 3]);
        __half2 h2 = __floats2half2_rn(acc32[8 * q + 4], acc32[8 * q + 5]);
        __half2 h3 = __floats2half2_rn(acc32[8 * q + 6], acc32[8 * q + 7]);
        v.x = *reinterpret_cast<uint32_t*>(&h0);
        v.y = *reinterpret_cast<uint32_t*>(&h1);
        v.z = *reinterpret_cast<uint32_t*>(&h2);
        v.w = *reinterpret_cast<uint32_t*>(&h3);
        dst[q] = v;
        for (int p = 0; p < n_peers; ++p)
          reinterpret_cast<uint4*>(static_cast<__half*>(peers->y[p]) + row * ldy + col0)[q] = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < n) {
          const __half h = __float2half_rn(acc32[j]);
          yrow[col0 + j] = h;
          for (int p = 0; p < n_peers; ++p) static_cast<__half*>(peers->y[p])[row * ldy + col0 + j] = h;
        }
    }
  } else {
    float* yrow = static_cast<float*>(y) + row * ldy;
    if (full) {
      float4* dst = reinterpret_cast<float4*>(yrow + col0);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 v = make_float4(__half2float(__float2half_rn(acc32[4 * q + 0])), __half2float(__float2half_rn(acc32[4 * q + 1])),
                                     __half2float(__float2half_rn(acc32[4 * q + 2])), __half2float(__float2half_rn(acc32[4 * q + 3])));
        dst[q] = v;
        for (int p = 0; p < n_peers; ++p)
          reinterpret_cast<float4*>(static_cast<float*>(peers->y[p]) + row * ldy + col0)[q] = v;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < n) {
          const float v = __half2float(__float2half_rn(acc32[j]));
          yrow[col0 + j] = v;
          for (int p = 0; p < n_peers; ++p) static_cast<float*>(peers->y[p])[row * ldy + col0 + j] = v;
        }
    }
  }
}
#endif  // __CUDACC__

}  // namespace dtas
