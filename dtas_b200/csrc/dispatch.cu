// C ABI of the library: argument checks, device / stream handling, m-bucket lookup and
// the call into the per-class launcher.
//
// This file is the hand-written counterpart of the host code the reference generates per
// PrimFunc (python/dtas/codegen/code_gen.py:242-405, an instance being
// experiment/dtas_tuned/elementwise/cast/top10_256/host.cc:42-131): unpack arguments,
// select the device, index = min(n/256, last), info = call_table[index_table[index]],
// launch.  The bucket -> kernel-variant tables live next to the kernels they select
// (ew_cfg, row_cfg, pick_wpr, plan_gemm).
#include <mutex>
#include <stdlib.h>

#include "common.cuh"

namespace dtas {

static thread_local char tl_error[512] = {0};
std::atomic<int64_t> g_launches{0};

// 0 = plain launches, 1 = programmatic dependent launch.  Initialised from DTAS_B200_PDL (default 1).
static std::atomic<int> g_pdl_mode{-1};
int pdl_mode() {
  int m = g_pdl_mode.load(std::memory_order_relaxed);
  if (m < 0) {
    const char* e = getenv("DTAS_B200_PDL");
    m = (e && e[0] == '0') ? 0 : 1;
    g_pdl_mode.store(m, std::memory_order_relaxed);
  }
  return m;
}
bool pdl_enabled() { return pdl_mode() != 0; }
int set_pdl_mode(int mode) {
  const int prev = pdl_mode();
  g_pdl_mode.store(mode, std::memory_order_relaxed);
  return prev;
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
  va_end(ap);
}

static constexpr int kMaxDevices = 64;
static DeviceCtx g_ctx[kMaxDevices];
static std::mutex g_ctx_mutex;

int get_ctx(int device, DeviceCtx** out) {
  if (device < 0 || device >= kMaxDevices) DTAS_FAIL(DTAS_EINVAL, "device ordinal %d out of range", device);
  DeviceCtx* c = &g_ctx[device];
  if (!c->ready) {
    std::lock_guard<std::mutex> lock(g_ctx_mutex);
    if (!c->ready) {
      cudaDeviceProp prop;
      DTAS_CUDA(cudaGetDeviceProperties(&prop, device));
      if (prop.major != 10)
        DTAS_FAIL(DTAS_EUNSUPPORTED, "device %d is sm_%d%d; this library only carries sm_100a code", device,
                  prop.major, prop.minor);
      c->sm_count = prop.multiProcessorCount;
      DTAS_CUDA(cudaMalloc(&c->status, sizeof(int)));
      DTAS_CUDA(cudaMemset(c->status, 0, sizeof(int)));
      c->ready = true;
    }
  }
  *out = c;
  return DTAS_OK;
}

namespace {

struct Call {
  DeviceGuard guard;
  DeviceCtx* ctx = nullptr;
  cudaStream_t stream = nullptr;
  int begin(int device, void* stream_handle) {
    int rc = guard.enter(device);
    if (rc != DTAS_OK) return rc;
    stream = static_cast<cudaStream_t>(stream_handle);
    return get_ctx(device, &ctx);
  }
};

int check_rows_cols(const char* op, int64_t m, int64_t n_cols) {
  if (m <= 0) DTAS_FAIL(DTAS_EINVAL, "%s: dynamic dim m must be > 0, got %lld", op, (long long)m);
  if (n_cols <= 0) DTAS_FAIL(DTAS_EINVAL, "%s: n_cols must be > 0, got %lld", op, (long long)n_cols);
  if (n_cols > ((int64_t)1 << 30) || m > ((int64_t)1 << 40) / n_cols)
    DTAS_FAIL(DTAS_EINVAL, "%s: shape [%lld, %lld] too large", op, (long long)m, (long long)n_cols);
  return DTAS_OK;
}

int op_index(const char* op) {
  static const char* names[] = {"cast", "add", "copy", "rms_norm", "softmax", "layer_norm", "gemv", "gemm"};
  if (op == nullptr) return -1;
  for (int i = 0; i < 8; ++i)
    if (strcmp(op, names[i]) == 0) return i;
  return -1;
}

}  // namespace
}  // namespace dtas

using namespace dtas;

#define DTAS_NONNULL(op, p) \
  if ((p) == nullptr) DTAS_FAIL(DTAS_EINVAL, "%s: argument %s is NULL", op, #p)

extern "C" {

int dtas_cast(const void* a, void* out, int64_t m, int64_t n_cols, int src_dtype, int dst_dtype,
              int device, void* stream) {
  DTAS_NONNULL("cast", a);
  DTAS_NONNULL("cast", out);
  int rc = check_rows_cols("cast", m, n_cols);
  if (rc) return rc;
  Call c;
  if ((rc = c.begin(device, stream))) return rc;
  return launch_cast(a, out, m * n_cols, src_dtype, dst_dtype, c.ctx, c.stream, bucket_of(m));
}

int dtas_add(const void* a, const void* b, void* out, int64_t m, int64_t n_cols, int dtype, int device,
             void* stream) {
  DTAS_NONNULL("add", a);
  DTAS_NONNULL("add", b);
  DTAS_NONNULL("add", out);
  int rc = check_rows_cols("add", m, n_cols);
  if (rc) return rc;
  Call c;
  if ((rc = c.begin(device, stream))) return rc;
  return launch_add(a, b, out, m * n_cols, dtype, c.ctx, c.stream, bucket_of(m));
}

int dtas_copy(const void* a, void* out, int64_t m, int64_t n_cols, int dtype, int device, void* stream) {
  DTAS_NONNULL("copy", a);
  DTAS_NONNULL("copy", out);
  int rc = check_rows_cols("copy", m, n_cols);
  if (rc) return rc;
  const int es = dtype_size(dtype);
  if (es == 0) DTAS_FAIL(DTAS_EUNSUPPORTED, "copy: unknown dtype %d", dtype);
  Call c;
  if ((rc = c.begin(device, stream))) return rc;
  return launch_copy(a, out, m * n_cols * es, c.ctx, c.stream, bucket_of(m));
}

int dtas_peer_push(const void* src, void* const* dsts, int n_dsts, int64_t bytes, int device, void* stream) {
  DTAS_NONNULL("peer_push", src);
  DTAS_NONNULL("peer_push", dsts);
  if (n_dsts < 1 || n_dsts > DTAS_MAX_PEERS)
    DTAS_FAIL(DTAS_EINVAL, "peer_push: n_dsts = %d is not in 1..%d", n_dsts, DTAS_MAX_PEERS);
  if (bytes < 1) DTAS_FAIL(DTAS_EINVAL, "peer_push: bytes = %lld must be >= 1", (long long)bytes);
  if (!aligned16(src)) DTAS_FAIL(DTAS_EALIGN, "peer_push: src is not 16-byte aligned");
  for (int j = 0; j < n_dsts; ++j) {
    if (dsts[j] == nullptr) DTAS_FAIL(DTAS_EINVAL, "peer_push: dsts[%d] is null", j);
    if (!aligned16(dsts[j])) DTAS_FAIL(DTAS_EALIGN, "peer_push: dsts[%d] is not 16-byte aligned", j);
    if (dsts[j] == src) DTAS_FAIL(DTAS_EINVAL, "peer_push: dsts[%d] is the source", j);
  }
  Call c;
  int rc = c.begin(device, stream);
  if (rc) return rc;
  return launch_peer_push(src, dsts, n_dsts, bytes, c.ctx, c.stream);
}

int dtas_rms_norm(const void* x, const void* weight, void* y, int64_t m, int64_t n_cols, float eps,
                  int in_dtype, int device, void* stream) {
  DTAS_NONNULL("rms_norm", x);
  DTAS_NONNULL("rms_norm", weight);
  DTAS_NONNULL("rms_norm", y);
  int rc = check_rows_cols("rms_norm", m, n_cols);
  if (rc) return rc;
  Call c;
  if ((rc = c.begin(device, stream))) return rc;
  return launch_row_op(ROW_RMSNORM, x, weight, nullptr, y, m, n_cols, eps, in_dtype, c.ctx, c.stream);
}

int dtas_softmax(const void* x, void* y, int64_t m, int64_t n_cols, int in_dtype, int device, void* stream) {
  DTAS_NONNULL("softmax", x);
  DTAS_NONNULL("softmax", y);
  int rc = check_rows_cols("softmax", m, n_cols);
  if (rc) return rc;
  Call c;
  if ((rc = c.begin(device, stream))) return rc;
  return launch_row_op(ROW_SOFTMAX, x, nullptr, nullptr, y, m, n_cols, 0.f, in_dtype, c.ctx, c.stream);
}

int dtas_layer_norm(const void* x, const void* gamma, const void* beta, void* y, int64_t m, int64_t n_cols,
                    float eps, int in_dtype, int device, void* stream) {
  DTAS_NONNULL("layer_norm", x);
  DTAS_NONNULL("layer_norm", gamma);
  DTAS_NONNULL("layer_norm", beta);
  DTAS_NONNULL("layer_norm", y);
  int rc = check_rows_cols("layer_norm", m, n_cols);
  if (rc) return rc;
  Call c;
  if ((rc = c.begin(device, stream))) return rc;
  return launch_row_op(ROW_LAYERNORM, x, gamma, beta, y, m, n_cols, eps, in_dtype, c.ctx, c.stream);
}

int dtas_gemv(const void* x, const void* w, const void* bias, void* y, int64_t n, int64_t k, int dtype,
              int device, void* stream) {
  DTAS_NONNULL("gemv", x);
  DTAS_NONNULL("gemv", w);
  DTAS_NONNULL("gemv", y);
  if (n <= 0 || k <= 0) DTAS_FAIL(DTAS_EINVAL, "gemv: n and k must be > 0, got n=%lld k=%lld", (long long)n, (long long)k);
  if (dtype != DTAS_F16) DTAS_FAIL(DTAS_EUNSUPPORTED, "gemv: only fp16 is implemented (dtype %d)", dtype);
  Call c;
  int rc;
  if ((rc = c.begin(device, stream))) return rc;
  Epilogue epi;
  epi.bias = static_cast<const __half*>(bias);
  return launch_gemv(x, w, epi, y, n, k, c.ctx, c.stream);
}

constexpr int64_t kResidualPassMinRows = 2048;

static int check_epilogue(const char* what, int act, int out_dtype) {
  if (act != DTAS_ACT_NONE && act != DTAS_ACT_GELU) DTAS_FAIL(DTAS_EINVAL, "%s: unknown activation %d", what, act);
  if (out_dtype != DTAS_F16 && out_dtype != DTAS_F32)
    DTAS_FAIL(DTAS_EUNSUPPORTED, "%s: the output is fp16 or fp32 (dtype %d)", what, out_dtype);
  return DTAS_OK;
}

int dtas_gemv_fused(const void* x, const void* w, const void* bias, const void* res1, const void* res2, void* y,
                    int64_t n, int64_t k, int act, int out_dtype, int dtype, int device, void* stream) {
  DTAS_NONNULL("gemv_fused", x);
  DTAS_NONNULL("gemv_fused", w);
  DTAS_NONNULL("gemv_fused", y);
  if (n <= 0 || k <= 0)
    DTAS_FAIL(DTAS_EINVAL, "gemv_fused: n and k must be > 0, got n=%lld k=%lld", (long long)n, (long long)k);
  if (dtype != DTAS_F16) DTAS_FAIL(DTAS_EUNSUPPORTED, "gemv_fused: only fp16 operands are implemented (dtype %d)", dtype);
  int rc;
  if ((rc = check_epilogue("gemv_fused", act, out_dtype))) return rc;
  if (res1 == nullptr && res2 != nullptr) DTAS_FAIL(DTAS_EINVAL, "gemv_fused: res2 without res1");
  Call c;
  if ((rc = c.begin(device, stream))) return rc;
  Epilogue epi;
  epi.bias = static_cast<const __half*>(bias);
  epi.res1 = static_cast<const __half*>(res1);
  epi.res2 = static_cast<const __half*>(res2);
  epi.ldr = 0;
  epi.act = act;
  epi.out_f32 = out_dtype == DTAS_F32 ? 1 : 0;
  return launch_gemv(x, w, epi, y, n, k, c.ctx, c.stream);
}

int dtas_gemm_nt(const void* x, const void* w, const void* bias, void* y, int64_t m, int64_t n, int64_t k,
                 int64_t ldy, int dtype, int device, void* stream) {
  DTAS_NONNULL("gemm", x);
  DTAS_NONNULL("gemm", w);
  DTAS_NONNULL("gemm", y);
  if (m <= 0) DTAS_FAIL(DTAS_EINVAL, "gemm: dynamic dim m must be > 0, got %lld", (long long)m);
  if (n <= 0 || k <= 0) DTAS_FAIL(DTAS_EINVAL, "gemm: n and k must be > 0, got n=%lld k=%lld", (long long)n, (long long)k);
  if (ldy < n) DTAS_FAIL(DTAS_EINVAL, "gemm: ldy (%lld) must be >= n (%lld)", (long long)ldy, (long long)n);
  if (dtype != DTAS_F16) DTAS_FAIL(DTAS_EUNSUPPORTED, "gemm: only fp16 is implemented (dtype %d)", dtype);
  Call c;
  int rc;
  if ((rc = c.begin(device, stream))) return rc;
  Epilogue epi;
  epi.bias = static_cast<const __half*>(bias);
  return launch_gemm(x, w, epi, y, m, n, k, ldy, c.ctx, c.stream);
}

int dtas_gemm_nt_fused(const void* x, const void* w, const void* bias, const void* res1, const void* res2, void* y,
                       int64_t m, int64_t n, int64_t k, int64_t ldy, int64_t ldr, int act, int out_dtype, int dtype,
                       int device, void* stream) {
  DTAS_NONNULL("gemm_fused", x);
  DTAS_NONNULL("gemm_fused", w);
  DTAS_NONNULL("gemm_fused", y);
  if (m <= 0) DTAS_FAIL(DTAS_EINVAL, "gemm_fused: dynamic dim m must be > 0, got %lld", (long long)m);
  if (n <= 0 || k <= 0)
    DTAS_FAIL(DTAS_EINVAL, "gemm_fused: n and k must be > 0, got n=%lld k=%lld", (long long)n, (long long)k);
  if (ldy < n) DTAS_FAIL(DTAS_EINVAL, "gemm_fused: ldy (%lld) must be >= n (%lld)", (long long)ldy, (long long)n);
  if (dtype != DTAS_F16) DTAS_FAIL(DTAS_EUNSUPPORTED, "gemm_fused: only fp16 operands are implemented (dtype %d)", dtype);
  int rc;
  if ((rc = check_epilogue("gemm_fused", act, out_dtype))) return rc;
  if (res1 == nullptr && res2 != nullptr) DTAS_FAIL(DTAS_EINVAL, "gemm_fused: res2 without res1");
  if (res1 != nullptr && ldr < n)
    DTAS_FAIL(DTAS_EINVAL, "gemm_fused: ldr (%lld) must be >= n (%lld)", (long long)ldr, (long long)n);
  Call c;
  if ((rc = c.begin(device, stream))) return rc;
  Epilogue epi;
  epi.bias = static_cast<const __half*>(bias);
  epi.act = act;
  epi.out_f32 = out_dtype == DTAS_F32 ? 1 : 0;
  // Behind a large GEMM the residual rows cost less as one streaming pass over Y (every thread of the
  // GEMM epilogue owns a row, so its residual loads touch 32 rows per instruction): measured at
  // m = 4096, N = K = 2560, two residuals: 76 us in the epilogue, 70 us as GEMM + two adds.
  const bool own_pass = res1 != nullptr && !epi.out_f32 && m >= kResidualPassMinRows && ldy == n && ldr == n;
  if (!own_pass) {
    epi.res1 = static_cast<const __half*>(res1);
    epi.res2 = static_cast<const __half*>(res2);
    epi.ldr = res1 != nullptr ? ldr : 0;
  }
  rc = launch_gemm(x, w, epi, y, m, n, k, ldy, c.ctx, c.stream);
  if (rc != DTAS_OK || !own_pass) return rc;
  return launch_add_residuals(y, res1, res2, m * n, c.ctx, c.stream, bucket_of(m));
}

int dtas_gemm_nt_scatter(const void* x, const void* w, const void* bias, void* y, void* const* peer_ys, int n_peers,
                         int64_t m, int64_t n, int64_t k, int64_t ldy, int dtype, int device, void* stream) {
  return dtas_gemm_nt_scatter_multicast(x, w, bias, y, peer_ys, n_peers, nullptr, m, n, k, ldy, dtype, device, stream);
}

int dtas_gemm_nt_scatter_multicast(const void* x, const void* w, const void* bias, void* y, void* const* peer_ys,
                                   int n_peers, void* y_multicast, int64_t m, int64_t n, int64_t k, int64_t ldy,
                                   int dtype, int device, void* stream) {
  DTAS_NONNULL("gemm_scatter", x);
  DTAS_NONNULL("gemm_scatter", w);
  DTAS_NONNULL("gemm_scatter", y);
  DTAS_NONNULL("gemm_scatter", peer_ys);
  if (n_peers < 1 || n_peers > DTAS_MAX_PEERS)
    DTAS_FAIL(DTAS_EINVAL, "gemm_scatter: n_peers = %d is not in 1..%d", n_peers, DTAS_MAX_PEERS);
  if (m <= 0) DTAS_FAIL(DTAS_EINVAL, "gemm_scatter: dynamic dim m must be > 0, got %lld", (long long)m);
  if (n <= 0 || k <= 0) DTAS_FAIL(DTAS_EINVAL, "gemm_scatter: n and k must be > 0");
  if (ldy < n) DTAS_FAIL(DTAS_EINVAL, "gemm_scatter: ldy (%lld) must be >= n (%lld)", (long long)ldy, (long long)n);
  if (dtype != DTAS_F16) DTAS_FAIL(DTAS_EUNSUPPORTED, "gemm_scatter: only fp16 is implemented (dtype %d)", dtype);
  PeerOut peers;
  peers.n = n_peers;
  for (int j = 0; j < n_peers; ++j) {
    if (peer_ys[j] == nullptr) DTAS_FAIL(DTAS_EINVAL, "gemm_scatter: peer_ys[%d] is null", j);
    if (peer_ys[j] == y) DTAS_FAIL(DTAS_EINVAL, "gemm_scatter: peer_ys[%d] is y itself", j);
    peers.y[j] = peer_ys[j];
  }
  if (y_multicast != nullptr) {
    if ((reinterpret_cast<uintptr_t>(y_multicast) & 15) != 0 || (reinterpret_cast<uintptr_t>(y) & 15) != 0 || (ldy & 7) != 0)
      DTAS_FAIL(DTAS_EALIGN, "gemm_scatter: the multicast address, y and its row stride must be 16-byte aligned");
    if (y_multicast == y) DTAS_FAIL(DTAS_EINVAL, "gemm_scatter: y_multicast is y itself");
    peers.mc = y_multicast;
  }
  Call c;
  int rc;
  if ((rc = c.begin(device, stream))) return rc;
  Epilogue epi;
  epi.bias = static_cast<const __half*>(bias);
  return launch_gemm(x, w, epi, y, m, n, k, ldy, c.ctx, c.stream, &peers);
}

int dtas_bucket_of(const char* op, int64_t m) {
  if (op_index(op) < 0) return -1;
  return bucket_of(m);
}

int dtas_bucket_count(const char* op) { return op_index(op) < 0 ? -1 : kNumBuckets; }

int dtas_variant_of(const char* op, int64_t m, int64_t n, int64_t k, int device, char* buf, int buf_len) {
  if (buf == nullptr || buf_len <= 0) DTAS_FAIL(DTAS_EINVAL, "variant_of: no buffer");
  const int idx = op_index(op);
  if (idx < 0) DTAS_FAIL(DTAS_EINVAL, "variant_of: unknown op '%s'", op ? op : "(null)");
  if (m <= 0 || n <= 0) DTAS_FAIL(DTAS_EINVAL, "variant_of: m and n must be > 0");
  // The SM count only matters for the grid caps; without a device the B200 count is assumed.
  DeviceCtx fake;
  fake.sm_count = 148;
  const DeviceCtx* ctx = &fake;
  if (device >= 0 && device < kMaxDevices && g_ctx[device].ready) ctx = &g_ctx[device];
  switch (idx) {
    case 0: case 1: case 2:
      snprintf(buf, buf_len, "%s", ew_variant_name(op, m, n, ctx));
      break;
    case 3: row_variant_name(ROW_RMSNORM, m, n, buf, buf_len); break;
    case 4: row_variant_name(ROW_SOFTMAX, m, n, buf, buf_len); break;
    case 5: row_variant_name(ROW_LAYERNORM, m, n, buf, buf_len); break;
    case 6: gemv_variant_name(n, k, ctx, buf, buf_len); break;
    default: gemm_variant_name(m, n, k, ctx, buf, buf_len); break;
  }
  return DTAS_OK;
}

int dtas_gemm_set_override(int bn, int split_k) {
  if (!(bn == 0 || bn == 64 || bn == 128 || bn == 256 || bn == 512 || bn == 513 || bn == 1024 || bn == 2048 || bn == 4160 || bn == 4224 || bn == 4352 || bn == 8256 || bn == 8320 || (bn >= 16386 && bn <= 16388)))
    DTAS_FAIL(DTAS_EINVAL, "gemm override: bn must be 0, 64, 128, 256, 512 (two-CTA 256 x 256 tile) 1024 (swapped operands, m <= 256), 2048 (the same with stream-K) or 4096 + 64/128/256 (single-CTA tiles with stream-K)");
  if (split_k < 0 || split_k > 64) DTAS_FAIL(DTAS_EINVAL, "gemm override: split_k must be in [0, 64]");
  gemm_set_override(bn, split_k);
  return DTAS_OK;
}

int dtas_gemm_table_set(int64_t n, int64_t k, int64_t m_lo, int64_t m_hi, int bn, int split_k) {
  if (n <= 0 || k <= 0 || m_lo < 1 || m_hi < m_lo) DTAS_FAIL(DTAS_EINVAL, "gemm table: bad key n=%lld k=%lld m=[%lld,%lld]", (long long)n, (long long)k, (long long)m_lo, (long long)m_hi);
  if (!(bn == 0 || bn == 64 || bn == 128 || bn == 256 || bn == 512 || bn == 513 || bn == 1024 || bn == 2048 || bn == 4160 || bn == 4224 || bn == 4352 || bn == 8256 || bn == 8320 || (bn >= 16386 && bn <= 16388))) DTAS_FAIL(DTAS_EINVAL, "gemm table: bad tile code %d", bn);
  if (split_k < 0 || split_k > 64) DTAS_FAIL(DTAS_EINVAL, "gemm table: split_k must be in [0, 64]");
  return gemm_table_set(n, k, m_lo, m_hi, bn, split_k);
}

int dtas_gemm_table_clear(void) {
  gemm_table_clear();
  return DTAS_OK;
}

int dtas_ew_set_override(int unroll, int ctas_per_sm, int stream_hints) {
  if (!(unroll == 0 || unroll == 1 || unroll == 2 || unroll == 4 || unroll == 8))
    DTAS_FAIL(DTAS_EINVAL, "elementwise override: unroll must be 0, 1, 2, 4 or 8");
  ew_set_override(unroll, ctas_per_sm, stream_hints);
  return DTAS_OK;
}

int dtas_row_set_override(int threads_per_row) {
  if (threads_per_row != 0 && (threads_per_row < 32 || threads_per_row > 1024 || (threads_per_row & (threads_per_row - 1))))
    DTAS_FAIL(DTAS_EINVAL, "row override: threads per row must be 0 or a power of two in [32, 1024]");
  row_set_override(threads_per_row);
  return DTAS_OK;
}

int dtas_gemv_set_override(int warps_per_row, int unroll) {
  if (!(warps_per_row == 0 || warps_per_row == 1 || warps_per_row == 2 || warps_per_row == 4 || warps_per_row == 8 ||
        warps_per_row == 16))
    DTAS_FAIL(DTAS_EINVAL, "gemv override: warps per row must be 0, 1, 2, 4, 8, or 16 for the streaming kernel");
  if (!(unroll == 0 || unroll == 4 || unroll == 8)) DTAS_FAIL(DTAS_EINVAL, "gemv override: unroll must be 0, 4 or 8");
  gemv_set_override(warps_per_row, unroll);
  return DTAS_OK;
}

const char* dtas_last_error(void) { return tl_error; }

int dtas_set_pdl(int mode) {
  if (mode < 0 || mode > 1) DTAS_FAIL(-1, "dtas_set_pdl: mode %d is not 0 or 1", mode);
  return set_pdl_mode(mode);
}

int64_t dtas_launch_count(void) { return g_launches.load(); }

int dtas_poll_status(int device) {
  if (device < 0 || device >= kMaxDevices) return DTAS_OK;
  // the built-in scratch of dtas_gemm_nt_static_scratch carries a status word of its own
  int static_code = 0;
  int rc = static_scratch_poll(device, &static_code);
  if (rc) return rc;
  int host = 0;
  if (g_ctx[device].ready) {
    DeviceGuard g;
    if ((rc = g.enter(device))) return rc;
    DTAS_CUDA(cudaDeviceSynchronize());
    DTAS_CUDA(cudaMemcpy(&host, g_ctx[device].status, sizeof(int), cudaMemcpyDeviceToHost));
    if (host != 0) {
      DTAS_CUDA(cudaMemset(g_ctx[device].status, 0, sizeof(int)));
      // a kernel that gave up may have left arrival counters of shared tiles behind
      if ((rc = reset_splitk_counters(&g_ctx[device]))) return rc;
    }
  }
  if (host == 0) host = static_code;
  if (host != 0) DTAS_FAIL(DTAS_ETIMEOUT, "a bounded device-side wait gave up (code 0x%x)", host);
  return DTAS_OK;
}

int dtas_shutdown(void) {
  std::lock_guard<std::mutex> lock(g_ctx_mutex);
  for (int d = 0; d < kMaxDevices; ++d) {
    DeviceCtx& c = g_ctx[d];
    if (!c.ready) continue;
    DeviceGuard g;
    if (g.enter(d) != DTAS_OK) continue;
    free_splitk_scratch(&c);
    if (c.status) cudaFree(c.status);
    c = DeviceCtx();
  }
  return DTAS_OK;
}

const char* dtas_version(void) { return "dtas_b200 0.1.0 sm_100a"; }

}  // extern "C"
