// Peer push: one rank's column slab of a sharded GEMM / GEMV result, written into the same
// place of every other rank's gather buffer with plain stores over NVLink.
//
// The reference is single-GPU (python/dtas/arch/RTX3090.py:6-7 opens one device); with the
// output columns sharded over g GPUs a caller that needs the whole Y on every rank would
// otherwise run an all-gather behind the kernel.  Here the rank that produced a block of rows
// pushes it: the source is read once (it is still in L2 behind the GEMM that wrote it) and every
// 16-byte vector is stored to up to seven destinations, which are device pointers to the peers'
// buffers mapped into this process.  The kernel waits on nothing and signals nothing: the
// caller orders it behind the producing kernel on the stream and runs a barrier across ranks
// after the last push.  Each destination receives (g-1)/g of Y in total, so the bound is the
// NVLink ingress of one GPU.  Measured on two B200s: plain peer stores sustain about 13 GB/s per
// CTA of 256 threads (16 KB in flight per CTA over a ~1.2 us round trip), so the grid covers every
// SM; beside a GEMM that holds every SM the copy engines move the same block faster, and
// dtas_b200.dist uses them by default for large blocks.
#include "common.cuh"

#include <cstdlib>

namespace dtas {
namespace {

constexpr int kPushThreads = 256;
constexpr int kPushUnroll = 4;

struct PushDsts {
  uint4* p[DTAS_MAX_PEERS];
  int n;
};

__global__ void __launch_bounds__(kPushThreads)
peer_push_kernel(const uint4* __restrict__ src, PushDsts d, int64_t n_vec, int64_t tail_bytes) {
  pdl_wait();
  pdl_launch_dependents();
  const int64_t stride = (int64_t)gridDim.x * kPushThreads;
  int64_t v = (int64_t)blockIdx.x * kPushThreads + threadIdx.x;
  for (; v + (kPushUnroll - 1) * stride < n_vec; v += kPushUnroll * stride) {
    uint4 r[kPushUnroll];
#pragma unroll
    for (int u = 0; u < kPushUnroll; ++u) r[u] = src[v + u * stride];
    for (int j = 0; j < d.n; ++j) {
#pragma unroll
      for (int u = 0; u < kPushUnroll; ++u) d.p[j][v + u * stride] = r[u];
    }
  }
  for (; v < n_vec; v += stride) {
    const uint4 r = src[v];
    for (int j = 0; j < d.n; ++j) d.p[j][v] = r;
  }
  if (tail_bytes > 0 && blockIdx.x == 0 && threadIdx.x < tail_bytes) {
    const uint8_t b = reinterpret_cast<const uint8_t*>(src + n_vec)[threadIdx.x];
    for (int j = 0; j < d.n; ++j) reinterpret_cast<uint8_t*>(d.p[j] + n_vec)[threadIdx.x] = b;
  }
}

}  // namespace

int launch_peer_push(const void* src, void* const* dsts, int n_dsts, int64_t bytes, const DeviceCtx* ctx,
                     cudaStream_t st) {
  PushDsts d;
  d.n = n_dsts;
  for (int j = 0; j < DTAS_MAX_PEERS; ++j) d.p[j] = j < n_dsts ? reinterpret_cast<uint4*>(dsts[j]) : nullptr;
  const int64_t n_vec = bytes / 16;
  const int64_t tail = bytes - n_vec * 16;
  const int64_t per_cta = (int64_t)kPushThreads * kPushUnroll;
  int64_t blocks = (n_vec + per_cta - 1) / per_cta;
  // One CTA per SM at most (8 CTAs: 106 GB/s, 148: NVLink-bound).  DTAS_B200_PUSH_CTAS overrides
  // the grid limit (read once).
  static const int env_cap = [] {
    const char* e = getenv("DTAS_B200_PUSH_CTAS");
    return e != nullptr ? atoi(e) : 0;
  }();
  const int64_t cap = env_cap > 0 ? env_cap : (ctx->sm_count > 0 ? ctx->sm_count : 1);
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  launch_kernel(peer_push_kernel, (unsigned)blocks, kPushThreads, 0, st, (const uint4*)src, d, n_vec, tail);
  return after_launch("peer_push");
}

}  // namespace dtas
