// Stand-alone probe, not part of the library: what one SM moves between itself and L2-resident
// data, by plain 16-byte loads / stores with a varying number of threads and loads in flight, and
// by 1-D bulk copies into / out of shared memory.  It is what the design of the split-K
// reduction rests on (few warps of plain loads: ~22 GB/s per SM; bulk copy: 100-150 GB/s;
// writes ~40 GB/s either way).  Every wait is bounded.
// Build and run:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o l2_probe dtas_b200/csrc/l2_probe.cu && ./l2_probe
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <algorithm>
#include <vector>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); exit(1); } } while (0)

constexpr int kRegion = 128 * 1024;          // bytes per CTA
constexpr int kVec = kRegion / 16;           // float4 per region

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- plain loads: THREADS threads, INFL float4 loads in flight per thread
template <int INFL>
__global__ void read_lsu(const float4* __restrict__ buf, float* sink, long long* stamps, int shift, int bytes) {
  const int g = gridDim.x;
  const float4* src = buf + (size_t)((blockIdx.x + shift) % g) * kVec;
  const int nvec = bytes / 16;
  __syncthreads();
  long long t0 = clock64();
  float acc = 0.f;
  for (int base = 0; base < nvec; base += blockDim.x * INFL) {
    float4 v[INFL];
#pragma unroll
    for (int u = 0; u < INFL; ++u) {
      int i = base + u * blockDim.x + threadIdx.x;
      v[u] = i < nvec ? __ldcg(src + i) : make_float4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < INFL; ++u) acc += v[u].x + v[u].y + v[u].z + v[u].w;
  }
  if (acc == 123.456f) sink[0] = acc;
  __syncthreads();
  long long t1 = clock64();
  if (threadIdx.x == 0) stamps[blockIdx.x] = t1 - t0;
}

// ---- plain stores + fence
__global__ void write_lsu(float4* __restrict__ buf, long long* stamps, int shift, int bytes, float val) {
  const int g = gridDim.x;
  float4* dst = buf + (size_t)((blockIdx.x + shift) % g) * kVec;
  const int nvec = bytes / 16;
  __syncthreads();
  long long t0 = clock64();
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) dst[i] = make_float4(val, val + 1, val + 2, val + 3);
  __threadfence();
  __syncthreads();
  long long t1 = clock64();
  if (threadIdx.x == 0) stamps[blockIdx.x] = t1 - t0;
}

// ---- bulk loads into shared memory: `pieces` copies of bytes/pieces each, issued by distinct threads
__global__ void read_bulk(const float4* __restrict__ buf, float* sink, long long* stamps, int shift, int bytes, int pieces) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t bar;
  const int g = gridDim.x;
  const uint8_t* src = reinterpret_cast<const uint8_t*>(buf + (size_t)((blockIdx.x + shift) % g) * kVec);
  const uint32_t b = smem_u32(&bar), s0 = smem_u32(smem);
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  long long t0 = clock64();
  if (threadIdx.x == 0)
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(bytes) : "memory");
  __syncthreads();
  const int piece = bytes / pieces;
  for (int p = threadIdx.x; p < pieces; p += blockDim.x)
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(s0 + p * piece), "l"(src + (size_t)p * piece), "r"(piece), "r"(b) : "memory");
  uint32_t done = 0;
  for (int spin = 0; spin < (1 << 24) && !done; ++spin)
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(b) : "memory");
  long long t1 = clock64();
  float acc = reinterpret_cast<float*>(smem)[threadIdx.x];
  if (acc == 123.456f) sink[0] = acc;
  if (threadIdx.x == 0) stamps[blockIdx.x] = done ? t1 - t0 : -1;
}

// ---- smem -> global bulk stores
__global__ void write_bulk(float4* __restrict__ buf, long long* stamps, int shift, int bytes, int pieces) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int g = gridDim.x;
  uint8_t* dst = reinterpret_cast<uint8_t*>(buf + (size_t)((blockIdx.x + shift) % g) * kVec);
  for (int i = threadIdx.x; i < bytes / 16; i += blockDim.x) reinterpret_cast<float4*>(smem)[i] = make_float4(1, 2, 3, 4);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  long long t0 = clock64();
  const int piece = bytes / pieces;
  const uint32_t s0 = smem_u32(smem);
  for (int p = threadIdx.x; p < pieces; p += blockDim.x)
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst + (size_t)p * piece), "r"(s0 + p * piece), "r"(piece) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  __threadfence();
  __syncthreads();
  long long t1 = clock64();
  if (threadIdx.x == 0) stamps[blockIdx.x] = t1 - t0;
}

static void report(const char* name, long long* d_stamps, int grid, int bytes) {
  std::vector<long long> h(grid);
  CK(cudaMemcpy(h.data(), d_stamps, grid * sizeof(long long), cudaMemcpyDeviceToHost));
  std::sort(h.begin(), h.end());
  const double ghz = 1.965;
  double med = h[grid / 2] / (ghz * 1e3), mn = h[0] / (ghz * 1e3), mx = h[grid - 1] / (ghz * 1e3);
  printf("%-44s grid %3d  %3d KB/CTA: med %6.2f us (%6.1f GB/s per SM)  min %6.2f  max %6.2f\n", name, grid, bytes / 1024, med,
         bytes / med / 1e3, mn, mx);
}

int main() {
  const int G = 148;
  float4* buf;
  float* sink;
  long long* stamps;
  CK(cudaMalloc(&buf, (size_t)G * kRegion));
  CK(cudaMalloc(&sink, 16));
  CK(cudaMalloc(&stamps, G * sizeof(long long)));
  CK(cudaMemset(buf, 0, (size_t)G * kRegion));
  CK(cudaFuncSetAttribute(read_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, kRegion + 1024));
  CK(cudaFuncSetAttribute(write_bulk, cudaFuncAttributeMaxDynamicSharedMemorySize, kRegion + 1024));
  for (int grid : {32, 64, 128, 148}) {
    for (int bytes : {65536, 131072}) {
      for (int shift : {0, 1, 37}) {
        char nm[128];
        // fresh data written by CTA (b - shift): with shift 0 the reader is (most likely) the writer's SM
        write_lsu<<<grid, 128>>>(buf, stamps, 0, kRegion, 1.f);
        CK(cudaDeviceSynchronize());
        read_lsu<32><<<grid, 128>>>(buf, sink, stamps, shift, bytes);
        CK(cudaDeviceSynchronize());
        snprintf(nm, sizeof nm, "read lsu 128thr x32 infl, shift %d", shift);
        report(nm, stamps, grid, bytes);
      }
      write_lsu<<<grid, 128>>>(buf, stamps, 0, kRegion, 1.f);
      read_lsu<8><<<grid, 128>>>(buf, sink, stamps, 1, bytes);
      CK(cudaDeviceSynchronize());
      report("read lsu 128thr x8 infl, shift 1", stamps, grid, bytes);
      read_lsu<8><<<grid, 512>>>(buf, sink, stamps, 1, bytes);
      CK(cudaDeviceSynchronize());
      report("read lsu 512thr x8 infl, shift 1", stamps, grid, bytes);
      read_lsu<16><<<grid, 1024>>>(buf, sink, stamps, 1, bytes);
      CK(cudaDeviceSynchronize());
      report("read lsu 1024thr x16 infl, shift 1", stamps, grid, bytes);
      for (int pieces : {1, 8, 64}) {
        char nm[128];
        read_bulk<<<grid, 128, kRegion + 1024>>>(buf, sink, stamps, 1, bytes, pieces);
        CK(cudaDeviceSynchronize());
        snprintf(nm, sizeof nm, "read bulk, %d pieces, shift 1", pieces);
        report(nm, stamps, grid, bytes);
      }
      write_lsu<<<grid, 128>>>(buf, stamps, 1, bytes, 2.f);
      CK(cudaDeviceSynchronize());
      report("write lsu 128thr + fence", stamps, grid, bytes);
      write_lsu<<<grid, 512>>>(buf, stamps, 1, bytes, 2.f);
      CK(cudaDeviceSynchronize());
      report("write lsu 512thr + fence", stamps, grid, bytes);
      for (int pieces : {1, 32}) {
        char nm[128];
        write_bulk<<<grid, 128, kRegion + 1024>>>(buf, stamps, 1, bytes, pieces);
        CK(cudaDeviceSynchronize());
        snprintf(nm, sizeof nm, "write bulk, %d pieces + fence", pieces);
        report(nm, stamps, grid, bytes);
      }
    }
  }
  printf("done\n");
  return 0;
}
