// Shared host/device helpers of the dtas_b200 kernel library (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <string.h>
#include <atomic>

#include "../../include/dtas_b200.h"
#include "epilogue.cuh"

namespace dtas {

constexpr int kNumBuckets = 32;        // 32 buckets of 256 rows: m = 1 .. 8192, clamped above
constexpr int kBucketWidth = 256;      // the reference's range_div_factor (engine/tuner.py:53-58)

// ---- error reporting -------------------------------------------------------
void set_error(const char* fmt, ...);
extern std::atomic<int64_t> g_launches;

#define DTAS_FAIL(code, ...)        \
  do {                              \
    ::dtas::set_error(__VA_ARGS__); \
    return (code);                  \
  } while (0)

#define DTAS_CUDA(expr)                                                          \
  do {                                                                           \
    cudaError_t _e = (expr);                                                     \
    if (_e != cudaSuccess) {                                                     \
      ::dtas::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),  \
                        __FILE__, __LINE__);                                     \
      return DTAS_ECUDA;                                                         \
    }                                                                            \
  } while (0)

// Counts the launch and turns a launch error into DTAS_ECUDA.
inline int after_launch(const char* what) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("launch of %s failed: %s", what, cudaGetErrorString(e));
    return DTAS_ECUDA;
  }
  return DTAS_OK;
}

// ---- programmatic dependent launch ---------------------------------------------
// Every kernel of the library is launched with the programmatic-stream-serialization attribute
// and runs pdl_wait() before its first access to global memory.  The wait returns once the
// kernel launched before it on the stream has finished and its writes are visible, so stream
// order is what the caller sees; what comes before the wait (barrier and tensor-memory set-up,
// descriptor prefetch, index arithmetic) overlaps the tail of the previous kernel.
// pdl_launch_dependents() right after the wait lets the next kernel start its own preamble.
// A kernel that has no predecessor, or whose predecessor is not a kernel, passes the wait at
// once.  DTAS_B200_PDL=0 in the environment launches without the attribute.
bool pdl_enabled();
int pdl_mode();
int set_pdl_mode(int mode);

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// ---- per-device context ------------------------------------------------------
// Split-K scratch of the GEMM: fp32 partial tiles + one arrival counter per output tile.  A call takes
// the set that belongs to its stream, so calls on different streams of one device never share
// partial sums or counters and may overlap freely.  Calls made while their stream is being captured
// into a CUDA graph take one more set, shared by all captured work of the device (a stream that
// exists only for a capture should not pin a set for the life of the process).
constexpr int kSplitKSlots = 8;
struct SplitKScratch {
  bool used = false;
  cudaStream_t stream = nullptr;   // the stream whose calls own this set
  float* ws = nullptr;
  int* counters = nullptr;
  uint64_t last_use = 0;
};
struct DeviceCtx {
  bool ready = false;
  int sm_count = 0;
  SplitKScratch splitk[kSplitKSlots];
  SplitKScratch splitk_capture;     // the set of calls that are being captured into a CUDA graph
  uint64_t splitk_clock = 0;
  int* status = nullptr;  // device status word written by bounded waits that gave up
};
int get_ctx(int device, DeviceCtx** out);           // creates on first use (device must be current)
// The split-K scratch set of `st` (created on the stream's first split-K call; cudaMalloc).
int acquire_splitk_scratch(DeviceCtx* ctx, cudaStream_t st, float** ws, int** counters);
int reset_splitk_counters(DeviceCtx* ctx);          // after a timeout: every set's counters back to zero
void free_splitk_scratch(DeviceCtx* ctx);
// Built-in scratch of dtas_gemm_nt_static_scratch: reads and clears its status word (0 when never used).
int static_scratch_poll(int device, int* code);

// Makes `device` current for the scope and restores the previous device.
struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  int enter(int device) {
    DTAS_CUDA(cudaGetDevice(&prev));
    if (prev != device) {
      DTAS_CUDA(cudaSetDevice(device));
      switched = true;
    }
    return DTAS_OK;
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

inline int bucket_of(int64_t m) {
  if (m <= 0) return -1;
  int64_t b = (m - 1) / kBucketWidth;
  return (int)(b >= kNumBuckets ? kNumBuckets - 1 : b);
}

inline int dtype_size(int dt) {
  switch (dt) {
    case DTAS_F16: return 2;
    case DTAS_F32: return 4;
    case DTAS_I8: return 1;
    default: return 0;
  }
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- launchers implemented by the per-class translation units --------------------
int launch_cast(const void* a, void* out, int64_t n, int src, int dst, const DeviceCtx* ctx,
                cudaStream_t st, int bucket);
int launch_add(const void* a, const void* b, void* out, int64_t n, int dt, const DeviceCtx* ctx,
               cudaStream_t st, int bucket);
int launch_add_residuals(void* y, const void* res1, const void* res2, int64_t n, const DeviceCtx* ctx,
                         cudaStream_t st, int bucket);   // y += res1 (+ res2), fp16, in place
int launch_copy(const void* a, void* out, int64_t nbytes, const DeviceCtx* ctx, cudaStream_t st,
                int bucket);
int launch_peer_push(const void* src, void* const* dsts, int n_dsts, int64_t bytes, const DeviceCtx* ctx,
                     cudaStream_t st);
const char* ew_variant_name(const char* op, int64_t m, int64_t n_cols, const DeviceCtx* ctx);
void ew_set_override(int unroll, int ctas_per_sm, int hints);

enum RowOp { ROW_RMSNORM = 0, ROW_SOFTMAX = 1, ROW_LAYERNORM = 2 };
int launch_row_op(RowOp op, const void* x, const void* p0, const void* p1, void* y, int64_t m,
                  int64_t n_cols, float eps, int in_dtype, const DeviceCtx* ctx, cudaStream_t st);
void row_variant_name(RowOp op, int64_t m, int64_t n_cols, char* buf, int len);
void row_set_override(int tpr);

int launch_gemv(const void* x, const void* w, const Epilogue& epi, void* y, int64_t n, int64_t k,
                const DeviceCtx* ctx, cudaStream_t st);
void gemv_variant_name(int64_t n, int64_t k, const DeviceCtx* ctx, char* buf, int len);
void gemv_set_override(int wpr, int unroll);

int launch_gemm(const void* x, const void* w, const Epilogue& epi, void* y, int64_t m, int64_t n,
                int64_t k, int64_t ldy, DeviceCtx* ctx, cudaStream_t st, const PeerOut* peers = nullptr);
void gemm_variant_name(int64_t m, int64_t n, int64_t k, const DeviceCtx* ctx, char* buf, int len);
void gemm_set_override(int bn, int split_k);
int gemm_table_set(int64_t n, int64_t k, int64_t m_lo, int64_t m_hi, int bn, int split_k);
void gemm_table_clear();

}  // namespace dtas
