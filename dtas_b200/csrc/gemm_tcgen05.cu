// Dynamic-m NT GEMM on the 5th-generation tensor cores:
//   Y[m,n] = X[m,k] * W[n,k]^T (+ bias[n]),  fp16 operands, fp32 accumulation in TMEM, fp16 out.
//
// Counterpart of the reference's tensor-core GEMM schedule
// (python/dtas/schedule/tir_wmma.py:20-222: block tile, shared-memory double buffering of
// both operands, software pipeline, L2-friendly block swizzle, accumulator written back
// through a fused epilogue; tile choice per m-range by the roofline/wave model of
// python/dtas/policy/wmma_config_emiter.py:148-353).  Nothing of nvcuda::wmma survives:
//
//   * operands arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle) into a ring of
//     shared-memory stages guarded by mbarriers; rows >= m and columns >= k are
//     zero-filled by the TMA unit, so no padding pass over X is needed for ragged m;
//   * one elected thread issues tcgen05.mma (M=128, N=BN, K=16, kind::f16) with both
//     operands read from shared memory through matrix descriptors; the 128 x BN fp32
//     accumulator lives in tensor memory, double-buffered so the epilogue of one tile
//     overlaps the main loop of the next;
//   * four epilogue warps pull the accumulator out with tcgen05.ld (lane = row,
//     32 columns per instruction), add the bias, round to fp16 and store;
//   * the kernel is persistent: at most one CTA per SM walks a list of
//     (m-tile, n-tile, k-split) work items ordered so that CTAs running at the same time
//     share X and W tiles in L2;
//   * tall-skinny m is HBM-bound on W, so small-m buckets cut K into `splits` slices to
//     put every SM to work: each slice stores its fp32 partial tile to a workspace, and
//     the last CTA to arrive at a tile (atomic ticket, no spinning) sums the slices in
//     slice order - deterministic - and writes fp16.
//
// No TMA multicast is used anywhere: every CTA loads its own operand tiles.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocator + MMA issuer,
// warps 2..5 = epilogue (warp w owns TMEM lanes 32*(w%4) .. +31).
//
// Every mbarrier wait is bounded: after about a second without progress the waiting role
// records a code in the device status word and leaves its loop; the CTA then drains,
// frees its tensor memory and exits.
//
// Work per launch: 2*m*n*k flop; bytes 2*(m*k + n*k + m*n).  Bound: tensor pipe for
// m >= ~1024, HBM (W stream) for small m.
#include <cuda.h>

#include <mutex>
#include <vector>

#include "common.cuh"

namespace dtas {
namespace {

constexpr int BM = 128;         // rows of X per tile = MMA M
constexpr int BK = 64;          // k elements per stage = one 128-byte swizzle row of fp16
constexpr int UMMA_K = 16;      // k per tcgen05.mma for 16-bit operands
constexpr int kGemmThreads = 192;
constexpr int kEpilogueThreads = 128;
constexpr int kStageBudget = 192 * 1024;   // bytes of operand ring per CTA
constexpr int kGroupM = 16;     // m-tiles per rasterisation band

constexpr int ERR_PRODUCER = 0x101, ERR_MMA_FULL = 0x102, ERR_MMA_TMEM = 0x103, ERR_EPILOGUE = 0x104;

// ---------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
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
// Bounded wait: gives up after `limit_ns` (~1 s by default) of wall time, records `code` and returns false.
constexpr uint64_t kWaitLimitNs = 1000000000ull;
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, int* status, int code,
                                            uint64_t limit_ns = kWaitLimitNs) {
  const uint64_t t0 = global_timer_ns();
  for (;;) {
    for (int i = 0; i < 2048; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > limit_ns) {
      atomicExch(status, code);
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  for (int i = 0; i < 64; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, status, code);
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; accumulate == 0 overwrites D.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has retired.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// After a wait: makes later uses of the loaded registers depend on the wait.  Where a load is issued well
// before its wait (to be in flight during other work), nothing else keeps arithmetic on its
// destination registers from being scheduled ahead of the wait.
__device__ __forceinline__ void tmem_ld_landed(uint32_t* r) {
  asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                    "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]));
  asm volatile("" : "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]),
                    "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]),
                    "+r"(r[30]), "+r"(r[31]));
}
__device__ __forceinline__ void epilogue_bar_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 fp16)
// laid out by TMA with the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride
// byte offset), the leading byte offset is unused for swizzled K-major layouts,
// descriptor version 1 (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor for kind::f16: D fp32, A and B fp16, both K-major, M=128, N=BN.
__host__ __device__ constexpr uint32_t make_idesc_f16_f32(int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

struct GemmArgs {
  void* y;            // fp16, or fp32 when epi.out_f32
  Epilogue epi;       // bias, activation, residuals, output dtype
  float* ws;          // partial tiles of shared output tiles (layout: see the epilogues)
  int* counters;      // one arrival counter per output tile (zero between launches)
  int* status;
  int64_t ldy;
  int m, n, k;
  int m_tiles, n_tiles, splits, kb_per_split, num_kb;
  int vec_store;      // 1 when 16-byte stores into Y are aligned
  int sk_per = 0;     // > 0: stream-K, every CTA owns sk_per consecutive (tile, k-block) units
  int sk_first = 0;   // two-CTA kernel, stream-K: first tile of the region that is cut into runs of units
  int slots_cap = 0;  // partial-tile slots reserved per output tile in the workspace
  PeerOut peers;      // two-CTA kernel: further buffers that receive every stored vector of Y
};

template <int BN>
struct Cfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = kStageBudget / kStageBytes;
  static constexpr int kTmemCols = 2 * BN;  // two accumulators
  static constexpr int kBarBytes = (2 * kStages + 4) * 8 + 16;
  // per epilogue warp 32 rows x min(BN, 128) fp16 columns, staged for row-contiguous stores
  static constexpr int kStoreCpr = BN >= 128 ? 16 : 8;            // 16-byte chunks per staged row
  static constexpr int kStoreStage = 4 * 32 * kStoreCpr * 16;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kStoreStage + kBarBytes;
  static_assert(kTmemCols >= 32 && kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "tmem");
  static_assert(kSmemBytes <= 227 * 1024, "smem");
};

// Tile index -> (m_tile, n_tile).  Tiles are visited band by band (kGroupM m-tiles per band);
// inside a band the m index runs fastest, so CTAs that run side by side read the same W tile
// and a small set of X tiles.
__device__ __forceinline__ void decode_tile(const GemmArgs& a, int tile, int& mt, int& nt) {
  const int band_tiles = kGroupM * a.n_tiles;
  const int band = tile / band_tiles;
  const int in_band = tile - band * band_tiles;
  const int band_rows = min(kGroupM, a.m_tiles - band * kGroupM);
  mt = band * kGroupM + in_band % band_rows;
  nt = in_band / band_rows;
}

// The work of a CTA as a sequence of segments: k-blocks [kb0, kb1) of output tile (mt, nt),
// being contribution `slot` of `count` to that tile.
//   * fixed split (a.sk_per == 0): items (tile, split) dealt round-robin to the CTAs;
//   * stream-K (a.sk_per > 0): the (tile, k-block) units are numbered tile-major and CTA c owns
//     units [c*per, (c+1)*per), so all CTAs stream the same number of k-blocks whatever the
//     tile count; a tile whose units fall to several CTAs is finished through the workspace.
// Producer, MMA issuer and epilogue each walk the same sequence with their own iterator.
struct TileSeg {
  int mt, nt, tile, kb0, kb1, slot, count;
  int first;   // stream-K: the CTA that holds contribution 0 of this tile
};
struct TileIter {
  int pos, end;
  __device__ __forceinline__ void init(const GemmArgs& a) {
    if (a.sk_per > 0) {
      const int total = a.m_tiles * a.n_tiles * a.num_kb;
      pos = min((int)blockIdx.x * a.sk_per, total);
      end = min(pos + a.sk_per, total);
    } else {
      pos = blockIdx.x;
      end = a.m_tiles * a.n_tiles * a.splits;
    }
  }
  __device__ __forceinline__ bool next(const GemmArgs& a, TileSeg& s) {
    if (pos >= end) return false;
    if (a.sk_per > 0) {
      s.tile = pos / a.num_kb;
      s.kb0 = pos - s.tile * a.num_kb;
      s.kb1 = min(a.num_kb, s.kb0 + (end - pos));
      const int u0 = s.tile * a.num_kb;
      const int first = u0 / a.sk_per, last = (u0 + a.num_kb - 1) / a.sk_per;
      s.count = last - first + 1;
      s.slot = (int)blockIdx.x - first;
      s.first = first;
      pos += s.kb1 - s.kb0;
    } else {
      s.first = 0;
      s.tile = pos / a.splits;
      s.slot = pos - s.tile * a.splits;
      s.count = a.splits;
      s.kb0 = s.slot * a.kb_per_split;
      s.kb1 = min(s.kb0 + a.kb_per_split, a.num_kb);
      pos += gridDim.x;
    }
    decode_tile(a, s.tile, s.mt, s.nt);
    return true;
  }
};

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_f16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x,
                            const __grid_constant__ CUtensorMap tmap_w, const GemmArgs a) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;   // swizzle atoms need 1024 B
  const uint32_t store_stage = base + C::kStages * C::kStageBytes;
  const uint32_t bars = store_stage + C::kStoreStage;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };
  auto tfull_bar = [&](int i) { return bars + 8u * (2 * C::kStages + i); };
  auto tempty_bar = [&](int i) { return bars + 8u * (2 * C::kStages + 2 + i); };
  const uint32_t tmem_slot = bars + 8u * (2 * C::kStages + 4);
  const uint32_t last_flag = tmem_slot + 4;
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(gen_base + C::kStages * C::kStageBytes + C::kStoreStage + 8 * (2 * C::kStages + 4));
  volatile uint32_t* last_flag_ptr = tmem_slot_ptr + 1;
  (void)last_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    // descriptor fetch overlaps the set-up below and the wait for the previous kernel
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_x)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_w)) : "memory");
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull_bar(i), 1);
      mbar_init(tempty_bar(i), kEpilogueThreads / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  pdl_wait();                 // the previous kernel on the stream is complete from here on
  pdl_launch_dependents();    // the next one may run its own set-up while this one works

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      TileIter it;
      TileSeg sg;
      it.init(a);
      while (ok && it.next(a, sg)) {
        const int mt = sg.mt, nt = sg.nt;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, a.status, ERR_PRODUCER)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), C::kStageBytes);
          const uint32_t sa = base + stage * C::kStageBytes;
          tma_load_2d(sa, &tmap_x, kb * BK, mt * BM, full_bar(stage));
          tma_load_2d(sa + C::kABytes, &tmap_w, kb * BK, nt * BN, full_bar(stage));
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16_f32(BN);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      TileIter it;
      TileSeg sg;
      it.init(a);
      for (; ok && it.next(a, sg); ++iter) {
        const int kb0 = sg.kb0, kb1 = sg.kb1;
        const int acc = iter & 1;
        const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, a.status, ERR_MMA_TMEM)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, a.status, ERR_MMA_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * C::kStageBytes;
          const uint64_t da = make_kmajor_sw128_desc(sa);
          const uint64_t db = make_kmajor_sw128_desc(sa + C::kABytes);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            // advancing 16 fp16 along K inside the swizzle row = +32 bytes = +2 in the address field
            umma_f16(d_tmem, da + 2u * kk, db + 2u * kk, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));   // stage reusable once these MMAs have read it
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(acc));  // accumulator complete
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quarter = warp & 3;                 // TMEM lanes 32*quarter .. +31
    const int epi_tid = threadIdx.x - 64;
    int iter = 0;
    bool ok = true;
    TileIter it;
    TileSeg sg;
    it.init(a);
    for (; ok && it.next(a, sg); ++iter) {
      const int mt = sg.mt, nt = sg.nt, sp = sg.slot, n_parts = sg.count;
      const int acc = iter & 1;
      const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
      if (!mbar_wait(tfull_bar(acc), acc_phase, a.status, ERR_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      const int row = mt * BM + quarter * 32 + lane;
      const bool row_ok = row < a.m;
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
      const int col_base = nt * BN;

      if (n_parts == 1) {
        if (epi_is_plain(a.epi)) {
          __half* yrow = static_cast<__half*>(a.y) + (int64_t)row * a.ldy;
          // blocks of 8 * kStoreCpr columns go through shared memory and leave as whole rows of 128 or 256
          // contiguous bytes (see epi_store_staged_block); ragged edges and unaligned Y from the registers
          constexpr int kCpr = C::kStoreCpr, kBlk = kCpr / 4;          // 32-column chunks per staged block
          uint4* stage = reinterpret_cast<uint4*>(gen_base + (store_stage - base)) + (warp - 2) * (32 * kCpr);
          const PeerOut no_peers;
#pragma unroll 1
          for (int c = 0; c < BN / 32; c += kBlk) {
            const int colb = col_base + c * 32;
            if (!(a.vec_store && colb + 8 * kCpr <= a.n)) {
#pragma unroll 1
              for (int cc = c; cc < c + kBlk; ++cc) {
                uint32_t r[32];
                tmem_ld32(t_addr + cc * 32, r);
                tmem_ld_wait();
                const int col0 = col_base + cc * 32;
                if (row_ok && col0 < a.n) epi_store_row32_plain(a.epi.bias, yrow, a.vec_store, col0, a.n, r);
              }
              continue;
            }
#pragma unroll 1
            for (int cc = 0; cc < kBlk; ++cc) {
              uint32_t r[32];
              tmem_ld32(t_addr + (c + cc) * 32, r);
              tmem_ld_wait();
              float f[32];
#pragma unroll
              for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
              if (a.epi.bias != nullptr) epi_add_bias32(a.epi.bias, colb + cc * 32, a.n, f);
#pragma unroll
              for (int q = 0; q < 4; ++q) stage[lane * kCpr + ((cc * 4 + q) ^ (lane & 7))] = epi_pack8(f + 8 * q);
            }
            __syncwarp();
            epi_store_staged_block<kCpr>(stage, lane, mt * BM + quarter * 32, a.m, a.y, a.ldy, colb, no_peers);
            __syncwarp();
          }
        } else {
        // Residual rows are fetched two chunks ahead of their use, so that their latency is not
        // paid once per chunk.
        ResChunk r_next, r_after;
        if (row_ok && epi_can_prefetch(a.epi, col_base, a.n)) epi_prefetch_res32(a.epi, row, col_base, r_next);
        if (row_ok && BN > 32 && epi_can_prefetch(a.epi, col_base + 32, a.n)) epi_prefetch_res32(a.epi, row, col_base + 32, r_after);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_addr + c * 32, r);
          const int col0 = col_base + c * 32;
          const ResChunk r_now = r_next;
          r_next = r_after;
          if (row_ok && c + 2 < BN / 32 && epi_can_prefetch(a.epi, col0 + 64, a.n)) epi_prefetch_res32(a.epi, row, col0 + 64, r_after);
          tmem_ld_wait();
          if (row_ok && col0 < a.n) {
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
            epi_store_row32(a.epi, a.y, a.ldy, a.vec_store, row, col0, a.n, f,
                            epi_can_prefetch(a.epi, col0, a.n) ? &r_now : nullptr);
          }
        }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
      } else {
        // Shared tile: park the fp32 partial, then the last contributor to arrive reduces.
        // Partials are float4s of four consecutive columns, laid out
        // [n tile][slot][column group][row]: the 32 lanes of a warp (32 consecutive rows) write
        // and read 512 contiguous bytes; rows at or beyond m are never touched.
        // Stream-K: a CTA's range of units cuts at most two tiles (the one it starts in and the one it
        // ends in), so its partials go to two tile-sized areas of its own, [CTA][first or last
        // segment][column group][row in tile]: the workspace does not grow with m or n.  Contribution
        // `slot` of a tile lives with CTA first + slot; it is that CTA's first segment unless the CTA
        // began before the tile did.
        const bool compact = a.sk_per > 0;
        const int r_in_tile = quarter * 32 + lane;
        const int64_t tile_u0 = (int64_t)sg.tile * a.num_kb;
        float4* ws4 = compact ? reinterpret_cast<float4*>(a.ws) + r_in_tile
                              : reinterpret_cast<float4*>(a.ws) + (int64_t)nt * a.slots_cap * (BN / 4) * a.m + row;
        auto ws_off = [&](int slot, int c4) -> int64_t {
          if (compact) {
            const int cta = sg.first + slot;
            const int which = ((int64_t)cta * a.sk_per >= tile_u0) ? 0 : 1;
            return ((int64_t)(cta * 2 + which) * (BN / 4) + c4) * BM;
          }
          return ((int64_t)slot * (BN / 4) + c4) * a.m;
        };
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_addr + c * 32, r);
          tmem_ld_wait();
          if (row_ok && col_base + c * 32 < a.n) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              ws4[ws_off(sp, c * 8 + q)] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                       __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));   // TMEM no longer needed for this tile

        __threadfence();
        epilogue_bar_sync();
        if (epi_tid == 0) {
          const int old = atomicAdd(&a.counters[sg.tile], 1);
          const uint32_t last = (old == n_parts - 1) ? 1u : 0u;
          if (last) a.counters[sg.tile] = 0;   // every contributor has arrived: re-arm for the next launch
          *last_flag_ptr = last;
        }
        epilogue_bar_sync();
        const bool is_last = *last_flag_ptr != 0;
        epilogue_bar_sync();                 // flag consumed before a later tile rewrites it
        if (is_last) {
          __threadfence();
          if (row_ok) {
            // 32 columns and two slots per batch: 16 independent 16-byte loads in flight per
            // thread (twice that measured no faster and costs 64 registers); slots are added in
            // slot order = K order, whatever the arrival order
            constexpr int W = 32;
            const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
            for (int c = 0; c < BN / W; ++c) {
              const int col0 = col_base + c * W;
              if (col0 >= a.n) break;
              const int live4 = min(W / 4, (a.n - col0 + 3) >> 2);   // column groups holding data
              float acc[W];
#pragma unroll
              for (int j = 0; j < W; ++j) acc[j] = 0.f;
#pragma unroll 1
              for (int sb = 0; sb < n_parts; sb += 2) {
                float4 v0[W / 4], v1[W / 4];
                const bool two = sb + 1 < n_parts;
#pragma unroll
                for (int q = 0; q < W / 4; ++q) {
                  const bool on = q < live4;
                  v0[q] = on ? __ldcg(ws4 + ws_off(sb, c * (W / 4) + q)) : zero4;
                  v1[q] = (on && two) ? __ldcg(ws4 + ws_off(sb + 1, c * (W / 4) + q)) : zero4;
                }
#pragma unroll
                for (int q = 0; q < W / 4; ++q) {
                  acc[4 * q] += v0[q].x; acc[4 * q + 1] += v0[q].y; acc[4 * q + 2] += v0[q].z; acc[4 * q + 3] += v0[q].w;
                }
#pragma unroll
                for (int q = 0; q < W / 4; ++q) {
                  acc[4 * q] += v1[q].x; acc[4 * q + 1] += v1[q].y; acc[4 * q + 2] += v1[q].z; acc[4 * q + 3] += v1[q].w;
                }
              }
              epi_store_row32(a.epi, a.y, a.ldy, a.vec_store, row, col0, a.n, acc);
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------
// Small-m variant (m <= 256): the operands trade places.
//
// With few rows the GEMM is a stream over W, and what limits a CTA is how many bytes of W it
// keeps in flight.  In the kernel above a stage always carries a 128-row X tile (16 KB, mostly
// zero fill when m is small) next to the W tile, so at BN = 64 only a third of the ring is W.
// Here the MMA computes Y^T: the 128 rows of the A operand are 128 rows of W (output columns),
// the B operand is the X tile with MN = m rounded up to 16/32/64/128/256 rows.  A stage is
// 16 KB of W plus MN*128 bytes of X, so at m = 16 the ring holds ten 16 KB W tiles.  The
// accumulator is 128 (n) x MN (m) in tensor memory: an epilogue thread owns one output column
// n and writes it row by row, so that a warp's store covers 32 consecutive columns of Y.
//
// K is cut either into a fixed number of slices per tile, or stream-K fashion: the (tile,
// k-block) units are dealt out in equal consecutive runs, so the CTAs finish together even
// when the tile count is no multiple of the SM count.  Partial tiles are float4s of four
// consecutive rows, laid out [tile][slot][row group][column], so that warps write and read
// 512 contiguous bytes; the last CTA to arrive at a tile sums the slots in K order with
// 16-32 independent loads in flight per thread.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

template <int MN>
struct SwapCfg {
  static constexpr int kWBytes = BM * BK * 2;            // 128 rows of W
  static constexpr int kXBytes = MN * BK * 2;            // MN rows of X
  static constexpr int kXPad = (kXBytes + 1023) / 1024 * 1024;
  static constexpr int kStageBytes = kWBytes + kXPad;
  static constexpr int kStages = kStageBudget / kStageBytes > 12 ? 12 : kStageBudget / kStageBytes;
  static constexpr int kTmemCols = 2 * MN < 32 ? 32 : 2 * MN;
  static constexpr int kBarBytes = (2 * kStages + 4) * 8 + 16;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kBarBytes;
  static_assert(kSmemBytes <= 227 * 1024, "smem");
  static_assert((kTmemCols & (kTmemCols - 1)) == 0 && kTmemCols <= 512, "tmem");
};

// The work of a CTA of the swapped-operand kernel as a sequence of segments: k-blocks
// [kb0, kb1) of output tile nt, being contribution `slot` of `count` to that tile.
//   * fixed split (a.sk_per == 0): items w = (tile, split) dealt round-robin to the CTAs;
//   * stream-K (a.sk_per > 0): the (tile, k-block) units are numbered tile-major and CTA c owns
//     units [c*per, (c+1)*per); a tile is finished by whichever CTAs its units fall to, so every
//     CTA streams the same number of k-blocks whatever the tile count.
// The three roles walk the same sequence, each with its own copy of the iterator.
struct SwapSeg {
  int nt, kb0, kb1, slot, count;
};
struct SwapIter {
  int pos, end;
  __device__ __forceinline__ void init(const GemmArgs& a) {
    if (a.sk_per > 0) {
      const int total = a.n_tiles * a.num_kb;
      pos = min((int)blockIdx.x * a.sk_per, total);
      end = min(pos + a.sk_per, total);
    } else {
      pos = blockIdx.x;
      end = a.n_tiles * a.splits;
    }
  }
  __device__ __forceinline__ bool next(const GemmArgs& a, SwapSeg& s) {
    if (pos >= end) return false;
    if (a.sk_per > 0) {
      s.nt = pos / a.num_kb;
      s.kb0 = pos - s.nt * a.num_kb;
      s.kb1 = min(a.num_kb, s.kb0 + (end - pos));
      const int u0 = s.nt * a.num_kb;
      const int first = u0 / a.sk_per, last = (u0 + a.num_kb - 1) / a.sk_per;
      s.count = last - first + 1;
      s.slot = (int)blockIdx.x - first;
      pos += s.kb1 - s.kb0;
    } else {
      s.nt = pos / a.splits;
      s.slot = pos - s.nt * a.splits;
      s.count = a.splits;
      s.kb0 = s.slot * a.kb_per_split;
      s.kb1 = min(s.kb0 + a.kb_per_split, a.num_kb);
      pos += gridDim.x;
    }
    return true;
  }
};

// a.n_tiles counts 128-column tiles of Y (128-row tiles of W); a.m_tiles is 1.
template <int MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_f16_tcgen05_swap_kernel(const __grid_constant__ CUtensorMap tmap_w,
                                 const __grid_constant__ CUtensorMap tmap_x, const GemmArgs a) {
  using C = SwapCfg<MN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + C::kStages * C::kStageBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };
  auto tfull_bar = [&](int i) { return bars + 8u * (2 * C::kStages + i); };
  auto tempty_bar = [&](int i) { return bars + 8u * (2 * C::kStages + 2 + i); };
  const uint32_t tmem_slot = bars + 8u * (2 * C::kStages + 4);
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(gen_base + C::kStages * C::kStageBytes + 8 * (2 * C::kStages + 4));
  volatile uint32_t* last_flag_ptr = tmem_slot_ptr + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    // descriptor fetch overlaps the set-up below and the wait for the previous kernel
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_x)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_w)) : "memory");
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull_bar(i), 1);
      mbar_init(tempty_bar(i), kEpilogueThreads / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  pdl_wait();                 // the previous kernel on the stream is complete from here on
  pdl_launch_dependents();    // the next one may run its own set-up while this one works

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      SwapIter it;
      SwapSeg sg;
      it.init(a);
      while (ok && it.next(a, sg)) {
        const int nt = sg.nt;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, a.status, ERR_PRODUCER)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), C::kWBytes + C::kXBytes);
          const uint32_t sa = base + stage * C::kStageBytes;
          tma_load_2d(sa, &tmap_w, kb * BK, nt * BM, full_bar(stage));
          tma_load_2d(sa + C::kWBytes, &tmap_x, kb * BK, 0, full_bar(stage));
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16_f32(MN);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      SwapIter it;
      SwapSeg sg;
      it.init(a);
      for (; ok && it.next(a, sg); ++iter) {
        const int kb0 = sg.kb0, kb1 = sg.kb1;
        const int acc = iter & 1;
        const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, a.status, ERR_MMA_TMEM)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * MN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, a.status, ERR_MMA_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * C::kStageBytes;
          const uint64_t da = make_kmajor_sw128_desc(sa);                // W rows: the M side
          const uint64_t db = make_kmajor_sw128_desc(sa + C::kWBytes);   // X rows: the N side
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            umma_f16(d_tmem, da + 2u * kk, db + 2u * kk, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
          umma_commit(empty_bar(stage));
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(acc));
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int epi_tid = threadIdx.x - 64;
    constexpr int kChunk = MN < 32 ? 16 : 32;     // columns per tcgen05.ld
    int iter = 0;
    bool ok = true;
    SwapIter it;
    SwapSeg sg;
    it.init(a);
    for (; ok && it.next(a, sg); ++iter) {
      const int nt = sg.nt, sp = sg.slot, n_parts = sg.count;
      const int acc = iter & 1;
      const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
      if (!mbar_wait(tfull_bar(acc), acc_phase, a.status, ERR_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      const int col = nt * BM + quarter * 32 + lane;        // output column owned by this thread
      const bool col_ok = col < a.n;
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * MN);

      if (n_parts == 1) {
        const float bias = (a.epi.bias != nullptr && col_ok) ? __half2float(a.epi.bias[col]) : 0.f;
#pragma unroll 1
        for (int c = 0; c < MN / kChunk; ++c) {
          uint32_t r[kChunk];
          if constexpr (kChunk == 16) tmem_ld16(t_addr + c * kChunk, r);
          else tmem_ld32(t_addr + c * kChunk, r);
          tmem_ld_wait();
          if (col_ok) {
            float f[kChunk];
#pragma unroll
            for (int j = 0; j < kChunk; ++j) f[j] = __uint_as_float(r[j]) + bias;
            epi_store_column<kChunk>(a.epi, a.y, a.ldy, c * kChunk, a.m, col, f);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
      } else {
        // Partials as float4 = four consecutive rows (m) of one output column, laid out
        // [tile][slot][row group][column in tile]: a warp's store covers 32 consecutive columns
        // (512 B).  Row groups at or beyond m are never written or read.
        const int groups = (a.m + 3) >> 2;                   // live row groups
        float4* ws4 = reinterpret_cast<float4*>(a.ws) + (int64_t)nt * a.slots_cap * (MN / 4) * BM + (quarter * 32 + lane);
        auto ws_off = [&](int slot, int g) { return ((int64_t)slot * (MN / 4) + g) * BM; };
#pragma unroll 1
        for (int c = 0; c < MN / kChunk; ++c) {
          uint32_t r[kChunk];
          if constexpr (kChunk == 16) tmem_ld16(t_addr + c * kChunk, r);
          else tmem_ld32(t_addr + c * kChunk, r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < kChunk / 4; ++q) {
            const int g = c * (kChunk / 4) + q;
            if (g < groups) {
              const float4 v = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                           __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
              ws4[ws_off(sp, g)] = v;
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));

        __threadfence();
        epilogue_bar_sync();
        if (epi_tid == 0) {
          const int old = atomicAdd(&a.counters[nt], 1);
          const uint32_t last = (old == n_parts - 1) ? 1u : 0u;
          if (last) a.counters[nt] = 0;
          *last_flag_ptr = last;
        }
        epilogue_bar_sync();
        const bool is_last = *last_flag_ptr != 0;
        epilogue_bar_sync();
        if (is_last) {
          __threadfence();
          const float bias = (a.epi.bias != nullptr && col_ok) ? __half2float(a.epi.bias[col]) : 0.f;
          // Up to eight row groups and four slots per batch: 16-32 independent 16-byte loads in
          // flight per thread, so that a tile of up to 32 rows costs one L2 round trip per four
          // slots.  Slots are summed in slot order = K order, whatever the arrival order.
          constexpr int G = MN / 4 < 8 ? MN / 4 : 8;
          const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
          for (int g0 = 0; g0 < groups; g0 += G) {
            float4 sum4[G];
#pragma unroll
            for (int j = 0; j < G; ++j) sum4[j] = zero4;
#pragma unroll 1
            for (int sb = 0; sb < n_parts; sb += 4) {
              float4 v[4][G];
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const bool on = sb + u < n_parts;
                const float4* src = ws4 + ws_off(on ? sb + u : 0, g0);
#pragma unroll
                for (int j = 0; j < G; ++j)
                  v[u][j] = (on && g0 + j < groups) ? __ldcg(src + (int64_t)j * BM) : zero4;
              }
#pragma unroll
              for (int u = 0; u < 4; ++u) {     // fixed split order: deterministic
#pragma unroll
                for (int j = 0; j < G; ++j) {
                  sum4[j].x += v[u][j].x; sum4[j].y += v[u][j].y; sum4[j].z += v[u][j].z; sum4[j].w += v[u][j].w;
                }
              }
            }
            if (col_ok) {
              float o[4 * G];
#pragma unroll
              for (int j = 0; j < G; ++j) {
                o[4 * j] = sum4[j].x + bias; o[4 * j + 1] = sum4[j].y + bias;
                o[4 * j + 2] = sum4[j].z + bias; o[4 * j + 3] = sum4[j].w + bias;
              }
              epi_store_column<4 * G>(a.epi, a.y, a.ldy, g0 * 4, a.m, col, o);
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------
// Two-CTA variant for large m: a cluster of two CTAs (the two SMs of a TPC) computes one
// 256 x 256 tile with tcgen05.mma.cta_group::2.
//
// Each CTA loads only its own halves - 128 rows of X and 128 rows of W per k-block, 32 KB
// per stage instead of 48 KB - so the ring is 7 stages deep (against 4), shared memory
// feeds the tensor pipe at 2/3 of the single-CTA rate per flop, and L2 sees 2/3 of the
// operand requests.  The MMA reads X rows from each CTA's own shared memory for that CTA's
// 128 accumulator rows, and the W rows of both CTAs as the 256 columns of B.
//
// Protocol (rank 0 of the pair is the leader):
//   * every CTA's producer waits on its own empty[s], then issues its two TMA loads with
//     cta_group::2 so that the bytes are counted on the LEADER's full[s]; only the leader
//     arms full[s], with the byte count of both CTAs;
//   * the leader's MMA thread waits full[s], issues the MMAs, and commits with a multicast
//     arrive to empty[s] of both CTAs; after the last k-block it commits to tmem_full[acc]
//     of both CTAs;
//   * the epilogue warps of both CTAs drain their own 128 accumulator rows and arrive on the
//     leader's tmem_empty[acc] (8 arrivals: 4 warps x 2 CTAs; the peer arrives remotely);
//   * before leaving, producers wait until every stage's last empty arrival has landed, and
//     all threads of the pair meet at a cluster barrier, so nobody signals shared memory of
//     a CTA that has exited; then both CTAs free their tensor memory.
// No TMA multicast is involved: cta_group::2 only redirects the completion bytes.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                                 uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this offset in every CTA of `cta_mask` once the MMAs issued so far retire.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(cta_mask)
      : "memory");
}
// Arrive on the barrier at the same offset in CTA `cta` of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar, uint32_t cta) {
  asm volatile(
      "{\n\t"
      ".reg .b32 remote;\n\t"
      "mapa.shared::cluster.u32 remote, %0, %1;\n\t"
      "mbarrier.arrive.release.cluster.shared::cluster.b64 _, [remote];\n\t"
      "}" ::"r"(bar),
      "r"(cta)
      : "memory");
}

constexpr int kPairBN = 256;                 // columns of the pair's tile
constexpr int kPairHalfBytes = BM * BK * 2;  // one 128 x 64 fp16 operand half: 16 KB
constexpr int kPairStageBytes = 2 * kPairHalfBytes;
#ifndef DTAS_PAIR_STAGED_STORE
#define DTAS_PAIR_STAGED_STORE 1      // 0: one more operand stage instead of the store staging area (for A/B timing)
#endif
constexpr int kPairStages = DTAS_PAIR_STAGED_STORE ? 6 : 7;
// per epilogue warp 32 rows x 128 fp16 columns, staged for row-contiguous stores
constexpr int kPairStoreStage = DTAS_PAIR_STAGED_STORE ? 4 * 32 * 256 : 0;
constexpr int kPairTmemCols = 2 * kPairBN;
constexpr int kPairBarBytes = (2 * kPairStages + 4) * 8 + 16;
constexpr int kPairSmemBytes = 1024 + kPairStages * kPairStageBytes + kPairStoreStage + kPairBarBytes;
static_assert(kPairSmemBytes <= 227 * 1024, "smem");
constexpr int kPairGroupM = 16;              // 256-row tiles per rasterisation band (8: W re-read twice as often, 1-3 % slower; 32: 5-8 % slower)
constexpr int ERR_PAIR_TAIL = 0x105;

__device__ __forceinline__ void decode_pair_work(int w, int m_tiles, int n_tiles, int& mt, int& nt) {
  const int band_tiles = kPairGroupM * n_tiles;
  const int band = w / band_tiles;
  const int in_band = w - band * band_tiles;
  const int band_rows = min(kPairGroupM, m_tiles - band * kPairGroupM);
  mt = band * kPairGroupM + in_band % band_rows;
  nt = in_band / band_rows;
}

// a.m_tiles / a.n_tiles count 256 x 256 tiles here; a.splits must be 1.
// The work of a CTA pair as a sequence of segments: k-blocks [kb0, kb1) of tile `tile`, being
// contribution `slot` of `count` to it.  Whole tiles are dealt round-robin to the pairs; with stream-K
// (a.sk_per > 0) the tiles from a.sk_first on - the last, partial wave - are instead cut, as
// (tile, k-block) units in tile-major order, into equal consecutive runs of a.sk_per units, one per
// pair, so that the wave ends for all pairs together whatever the tile count (32 tiles on 74 pairs: 28
// k-blocks each instead of 64 on fewer than half the pairs).  A tile whose units fall to several pairs
// is finished through the workspace.  (Taking the whole wave before the last into the region as well,
// so that a run is longer than a tile and a tile has two contributors instead of up to six, was
// measured: 57 against 67 us at m = 255, N = 22016 - still behind the 55 us of whole tiles - and 1-4 %
// slower from m = 1024 up, where more tiles then pay for the workspace.)
struct PairSeg {
  int mt, nt, tile, kb0, kb1, slot, count, first;
};
struct PairIter {
  int pos, end;        // whole tiles: next tile, one past the last whole-tile index
  int spos, send;      // stream-K tail: next unit and end of this pair's run of (tile, k-block) units
  int tail_first;      // first tile of the tail
  __device__ __forceinline__ void init(const GemmArgs& a, int pair, int n_pairs) {
    const int tiles = a.m_tiles * a.n_tiles;
    pos = pair;
    end = tiles;
    spos = send = 0;
    tail_first = tiles;
    if (a.sk_per > 0) {
      // whole waves of tiles are dealt round-robin (pairs running side by side share X and W tiles in
      // L2); the tiles from a.sk_first on are cut into equal runs of k-blocks
      end = tail_first = a.sk_first;
      const int units = (tiles - tail_first) * a.num_kb;
      spos = min(pair * a.sk_per, units);
      send = min(spos + a.sk_per, units);
    }
  }
  __device__ __forceinline__ bool next(const GemmArgs& a, int pair, int n_pairs, PairSeg& s) {
    if (pos < end) {
      s.tile = pos;
      s.kb0 = 0;
      s.kb1 = a.num_kb;
      s.first = pair;
      s.count = 1;
      s.slot = 0;
      pos += n_pairs;
    } else if (spos < send) {
      const int t = spos / a.num_kb;              // tile within the tail
      s.tile = tail_first + t;
      s.kb0 = spos - t * a.num_kb;
      s.kb1 = min(a.num_kb, s.kb0 + (send - spos));
      const int u0 = t * a.num_kb;
      s.first = u0 / a.sk_per;
      s.count = (u0 + a.num_kb - 1) / a.sk_per - s.first + 1;
      s.slot = pair - s.first;
      spos += s.kb1 - s.kb0;
    } else {
      return false;
    }
    decode_pair_work(s.tile, a.m_tiles, a.n_tiles, s.mt, s.nt);
    return true;
  }
};
// Named barrier over the epilogue warps of a CTA (4 or 8 of them).
__device__ __forceinline__ void epilogue_bar_sync_n(int threads) {
  asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

constexpr int kPairMaxThreads = 32 * (2 + 8);   // producer, MMA issuer and up to eight epilogue warps

// Launched with four epilogue warps (192 threads), or with eight (320 threads) when the epilogue has an
// activation or residuals to work through: of the two warps that share a quarter of the tensor-memory
// lanes one then finishes columns 0..127 of the tile and the other columns 128..255, so the tail of a
// 256 x 256 tile is spread over twice the issue slots and hides behind a shorter main loop.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairMaxThreads, 1)
    gemm_f16_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_x,
                                 const __grid_constant__ CUtensorMap tmap_w, const GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t store_stage = base + kPairStages * kPairStageBytes;
  const uint32_t bars = store_stage + kPairStoreStage;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (kPairStages + s); };
  auto tfull_bar = [&](int i) { return bars + 8u * (2 * kPairStages + i); };
  auto tempty_bar = [&](int i) { return bars + 8u * (2 * kPairStages + 2 + i); };
  const uint32_t tmem_slot = bars + 8u * (2 * kPairStages + 4);
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(
      gen_base + kPairStages * kPairStageBytes + kPairStoreStage + 8 * (2 * kPairStages + 4));
  volatile uint32_t* last_flag_ptr = tmem_slot_ptr + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  constexpr uint32_t kPeerMask = 0xFEFFFFFFu;       // clears the CTA-rank bit of a shared::cluster address

  if (threadIdx.x == 0) {
    // descriptor fetch overlaps the set-up below and the wait for the previous kernel
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_x)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_w)) : "memory");
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tfull_bar(i), 1);
      mbar_init(tempty_bar(i), 2 * ((blockDim.x >> 5) - 2));   // every epilogue warp of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kPairTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();      // barriers of both CTAs are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  pdl_wait();                 // the previous kernel on the stream is complete from here on
  pdl_launch_dependents();    // the next one may run its own set-up while this one works

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      PairIter it;
      PairSeg sg;
      it.init(a, pair, n_pairs);
      while (ok && it.next(a, pair, n_pairs, sg)) {
        const int row0 = sg.mt * 2 * BM + (int)rank * BM;          // this CTA's 128 rows of X
        const int col0 = sg.nt * kPairBN + (int)rank * (kPairBN / 2);  // this CTA's 128 rows of W
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, a.status, ERR_PRODUCER)) { ok = false; break; }
          if (leader) mbar_expect_tx(full_bar(stage), 2 * kPairStageBytes);
          const uint32_t sa = base + stage * kPairStageBytes;
          const uint32_t lbar = full_bar(stage) & kPeerMask;
          tma_load_2d_pair(sa, &tmap_x, kb * BK, row0, lbar);
          tma_load_2d_pair(sa + kPairHalfBytes, &tmap_w, kb * BK, col0, lbar);
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
      // Tail: every stage's last release by the leader's MMA thread must have landed here
      // before this CTA may exit.
      for (int s = 0; s < kPairStages && ok; ++s) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, a.status, ERR_PAIR_TAIL)) ok = false;
        if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(kPairBN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      PairIter it;
      PairSeg sg;
      it.init(a, pair, n_pairs);
      for (; ok && it.next(a, pair, n_pairs, sg); ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, a.status, ERR_MMA_TMEM)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * kPairBN);
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, a.status, ERR_MMA_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * kPairStageBytes;
          const uint64_t da = make_kmajor_sw128_desc(sa);
          const uint64_t db = make_kmajor_sw128_desc(sa + kPairHalfBytes);
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk)
            umma_f16_pair(d_tmem, da + 2u * kk, db + 2u * kk, idesc, (kb > sg.kb0 || kk > 0) ? 1u : 0u);
          umma_commit_pair(empty_bar(stage), 0x3);
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(tfull_bar(acc), 0x3);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int quarter = warp & 3;
    const int chunks = (kPairBN / 32) / (((int)blockDim.x >> 5) - 2 > 4 ? 2 : 1);   // 32-column chunks per warp
    const int c_begin = ((warp - 2) >> 2) * chunks, c_end = c_begin + chunks;
    const int n_epi_threads = (int)blockDim.x - 64;
    const int epi_tid = (int)threadIdx.x - 64;
    int iter = 0;
    bool ok = true;
    PairIter it;
    PairSeg sg;
    it.init(a, pair, n_pairs);
    for (; ok && it.next(a, pair, n_pairs, sg); ++iter) {
      const int mt = sg.mt, nt = sg.nt;
      const int acc = iter & 1;
      const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
      if (!mbar_wait(tfull_bar(acc), acc_phase, a.status, ERR_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      const int r_in_tile = quarter * 32 + lane;
      const int row = mt * 2 * BM + (int)rank * BM + r_in_tile;
      const bool row_ok = row < a.m;
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * kPairBN);
      const int col_base = nt * kPairBN;
      if (sg.count > 1) {
        // Shared tile (stream-K): park this CTA's 128 x 256 partial, then the last CTA of this rank to
        // arrive at the tile sums the contributions in slot order = K order and runs the epilogue.
        // A pair's range cuts at most two tiles, so its partials live in two areas of its own,
        // [pair][first or last segment][rank][column group][row]: a warp writes and reads 512
        // contiguous bytes.  The two CTAs of a pair count arrivals separately (one counter per tile
        // and rank): neither waits for the other, and nobody spins.
        constexpr int kArea = (kPairBN / 4) * BM;                      // float4s of one CTA's partial tile
        const int64_t tile_u0 = (int64_t)(sg.tile - it.tail_first) * a.num_kb;   // units are counted within the tail
        auto area_of = [&](int q) -> int64_t {
          const int which = ((int64_t)q * a.sk_per >= tile_u0) ? 0 : 1;
          return (int64_t)((q * 2 + which) * 2 + (int)rank) * kArea + r_in_tile;
        };
        float4* ws4 = reinterpret_cast<float4*>(a.ws);
        float4* mine = ws4 + area_of(pair);
#pragma unroll 1
        for (int c = c_begin; c < c_end; ++c) {
          uint32_t r[32];
          tmem_ld32(t_addr + c * 32, r);
          tmem_ld_wait();
          if (row_ok && col_base + c * 32 < a.n) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
              mine[(c * 8 + q) * BM] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                   __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
          }
        }
        __threadfence();
        epilogue_bar_sync_n(n_epi_threads);
        if (epi_tid == 0) {
          int* counter = a.counters + (sg.tile * 2 + (int)rank);
          const int old = atomicAdd(counter, 1);
          const uint32_t last = (old == sg.count - 1) ? 1u : 0u;
          if (last) *counter = 0;          // every contributor has arrived: re-arm for the next launch
          *last_flag_ptr = last;
        }
        epilogue_bar_sync_n(n_epi_threads);
        const bool is_last = *last_flag_ptr != 0;
        epilogue_bar_sync_n(n_epi_threads);     // flag consumed before a later tile rewrites it
        if (is_last) {
          // The other contributions come back from the workspace; this CTA's own is still in tensor
          // memory and is added from there at its place in the K order (the same values and the same
          // sequence of additions whichever contributor happens to arrive last).
          __threadfence();
          const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
          for (int c = c_begin; c < c_end; ++c) {
            const int col0 = col_base + c * 32;
            if (col0 >= a.n) break;
            const int live4 = row_ok ? min(8, (a.n - col0 + 3) >> 2) : 0;
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = 0.f;
#pragma unroll 1
            for (int sb = 0; sb < sg.count; sb += 2) {
              const bool two = sb + 1 < sg.count;
              const bool own0 = sb == sg.slot, own1 = two && sb + 1 == sg.slot;
              const float4* s0 = ws4 + area_of(sg.first + sb) + (int64_t)c * 8 * BM;
              const float4* s1 = ws4 + area_of(sg.first + (two ? sb + 1 : sb)) + (int64_t)c * 8 * BM;
              uint32_t v0[32], v1[32];
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const bool on = q < live4;
                const float4 t0 = (on && !own0) ? __ldcg(s0 + q * BM) : zero4;
                const float4 t1 = (on && two && !own1) ? __ldcg(s1 + q * BM) : zero4;
                v0[4 * q] = __float_as_uint(t0.x); v0[4 * q + 1] = __float_as_uint(t0.y);
                v0[4 * q + 2] = __float_as_uint(t0.z); v0[4 * q + 3] = __float_as_uint(t0.w);
                v1[4 * q] = __float_as_uint(t1.x); v1[4 * q + 1] = __float_as_uint(t1.y);
                v1[4 * q + 2] = __float_as_uint(t1.z); v1[4 * q + 3] = __float_as_uint(t1.w);
              }
              if (own0) {                    // the same for the whole warp
                tmem_ld32(t_addr + c * 32, v0);
                tmem_ld_wait();
              } else if (own1) {
                tmem_ld32(t_addr + c * 32, v1);
                tmem_ld_wait();
              }
#pragma unroll
              for (int j = 0; j < 32; ++j) f[j] += __uint_as_float(v0[j]);
              if (two) {
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] += __uint_as_float(v1[j]);
              }
            }
            if (row_ok) epi_store_row32(a.epi, a.y, a.ldy, a.vec_store, row, col0, a.n, f, nullptr, &a.peers);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(tempty_bar(acc), 0);   // tensor memory no longer needed for this tile
        continue;
      }
      if (epi_is_plain(a.epi)) {
        __half* yrow = static_cast<__half*>(a.y) + (int64_t)row * a.ldy;
        // Four warps (the plain launch): 128 columns at a time go through shared memory, so that a warp
        // stores two whole rows of 256 contiguous bytes per instruction instead of 16 bytes of each of
        // its 32 rows - full lines for the local Y and, where the result is also stored to other GPUs,
        // for NVLink.  Thread = row writes its 16-byte vectors at chunk ^ (row & 7): both the writes (a
        // quarter warp = 8 rows, one chunk) and the reads (a quarter warp = 8 chunks of one row) then
        // cover all 32 banks.
        const bool staged = DTAS_PAIR_STAGED_STORE && a.vec_store && warp < 6;
        uint4* stage = reinterpret_cast<uint4*>(gen_base + (store_stage - base)) + (warp - 2) * (32 * 16);
        const int row_base = mt * 2 * BM + (int)rank * BM + quarter * 32;
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 4) {
          const int colb = col_base + c * 32;
          if (!(staged && c + 4 <= c_end && colb + 128 <= a.n)) {
#pragma unroll 1
            for (int cc = c; cc < min(c + 4, c_end); ++cc) {
              uint32_t r[32];
              tmem_ld32(t_addr + cc * 32, r);
              tmem_ld_wait();
              const int col0 = col_base + cc * 32;
              if (row_ok && col0 < a.n) epi_store_row32_plain(a.epi.bias, yrow, a.vec_store, col0, a.n, r, &a.peers, (int64_t)row * a.ldy);
            }
            continue;
          }
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t r[32];
            tmem_ld32(t_addr + (c + cc) * 32, r);
            tmem_ld_wait();
            if (a.epi.bias != nullptr) epi_add_bias32(a.epi.bias, colb + cc * 32, a.n, reinterpret_cast<float*>(r));
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
#pragma unroll
            for (int q = 0; q < 4; ++q) stage[lane * 16 + ((cc * 4 + q) ^ (lane & 7))] = epi_pack8(f + 8 * q);
          }
          __syncwarp();
          epi_store_staged_block<16>(stage, lane, row_base, a.m, a.y, a.ldy, colb, a.peers);
          __syncwarp();
        }
      } else {
      uint4* stage_f = reinterpret_cast<uint4*>(gen_base + (store_stage - base)) + (warp - 2) * (32 * 8);
      // One chunk of 32 columns: the tail's arithmetic, then - fp16 results - through shared memory in
      // blocks of 64 columns (two chunks), which leave as whole 128-byte rows; an fp32 output, ragged
      // edges and unaligned buffers are stored from the registers.
      auto finish_chunk = [&](int c, const uint32_t* r, const ResChunk* res) {
        const int col0 = col_base + c * 32;
        const int blk0 = col_base + (c & ~1) * 32;
        const bool staged_f = DTAS_PAIR_STAGED_STORE && a.vec_store && !a.epi.out_f32 && blk0 + 64 <= a.n && (c | 1) < c_end;
        float f[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
        if (staged_f) {
          if (row_ok) epi_apply_row32(a.epi, row, col0, a.n, f, res);
#pragma unroll
          for (int q = 0; q < 4; ++q) stage_f[lane * 8 + (((c & 1) * 4 + q) ^ (lane & 7))] = epi_pack8(f + 8 * q);
          if (c & 1) {
            __syncwarp();
            epi_store_staged_block<8>(stage_f, lane, mt * 2 * BM + (int)rank * BM + quarter * 32, a.m, a.y, a.ldy, blk0, a.peers);
            __syncwarp();
          }
        } else if (row_ok && col0 < a.n) {
          epi_store_row32(a.epi, a.y, a.ldy, a.vec_store, row, col0, a.n, f, res, &a.peers);
        }
      };
      if (a.epi.res1 == nullptr) {
        // Activation without residuals: the accumulator words of the next chunk are on their way from
        // tensor memory while the current chunk is worked on (two sets of registers in turn).
        uint32_t ra[32], rb[32];
        tmem_ld32(t_addr + c_begin * 32, ra);
        tmem_ld_wait();
        tmem_ld_landed(ra);
#pragma unroll 1
        for (int c = c_begin; c < c_end; c += 2) {        // c_begin is even: a pair of chunks is a staged block
          const bool second = c + 1 < c_end;
          if (second) tmem_ld32(t_addr + (c + 1) * 32, rb);
          finish_chunk(c, ra, nullptr);
          tmem_ld_wait();
          tmem_ld_landed(rb);
          if (second) {
            if (c + 2 < c_end) tmem_ld32(t_addr + (c + 2) * 32, ra);
            finish_chunk(c + 1, rb, nullptr);
            tmem_ld_wait();
            tmem_ld_landed(ra);
          }
        }
      } else {
        // Residual rows are fetched two chunks ahead of their use.
        ResChunk r_next, r_after;
        const int colb = col_base + c_begin * 32;
        if (row_ok && epi_can_prefetch(a.epi, colb, a.n)) epi_prefetch_res32(a.epi, row, colb, r_next);
        if (row_ok && epi_can_prefetch(a.epi, colb + 32, a.n)) epi_prefetch_res32(a.epi, row, colb + 32, r_after);
#pragma unroll 1
        for (int c = c_begin; c < c_end; ++c) {
          uint32_t r[32];
          tmem_ld32(t_addr + c * 32, r);
          const int col0 = col_base + c * 32;
          const ResChunk r_now = r_next;
          r_next = r_after;
          if (row_ok && c + 2 < c_end && epi_can_prefetch(a.epi, col0 + 64, a.n)) epi_prefetch_res32(a.epi, row, col0 + 64, r_after);
          tmem_ld_wait();
          finish_chunk(c, r, epi_can_prefetch(a.epi, col0, a.n) ? &r_now : nullptr);
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_bar(acc), 0);   // the leader's barrier, from either CTA
    }
  }

  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kPairTmemCols);
  }
}

// ---------------------------------------------------------------------------------------
// K cut in two inside a cluster: the hand-over of the second half goes through shared memory.
//
// For 128 < m <= ~512 at N ~ 4096 the output has too few 128 x 128 tiles to fill the SMs, and a
// tile finished through the global workspace pays ~6 us for it at m = 255 (park the partial,
// fence, ticket, read both partials back with four warps).  Here the two K halves of a tile are
// the two CTAs of a cluster: each runs the usual TMA / MMA pipeline on its half; CTA 1 then moves
// its accumulator (TMEM -> registers -> its own shared memory) into a staging area of CTA 0 with
// one bulk copy through distributed shared memory, and CTA 0 adds its own accumulator and runs the
// epilogue.  No workspace, no ticket, no fence; the sum is own half + other half: deterministic.
// One tile per cluster (the regime is a single wave).  BN = 64 or 128 (the staging tile has to fit
// beside the ring).
// ---------------------------------------------------------------------------------------
template <int BN>
struct K2Cfg {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStagingBytes = BM * BN * 4;                 // one fp32 accumulator tile
  static constexpr int kStages = (224 * 1024 - kStagingBytes) / kStageBytes;
  static constexpr int kTmemCols = BN < 32 ? 32 : BN;
  static constexpr int kBarBytes = (2 * kStages + 2) * 8 + 16;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kStagingBytes + kBarBytes;
  static_assert(kSmemBytes <= 227 * 1024 && kStages >= 3, "smem");
};
constexpr int ERR_K2_DATA = 0x106;

__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
  return r;
}
// Bulk copy from this CTA's shared memory into a peer's (both addresses 16-byte aligned, size a
// multiple of 16); completion is counted on the peer's mbarrier.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster, uint32_t src_cta, uint32_t bytes,
                                                  uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :
               : "r"(dst_cluster), "r"(src_cta), "r"(bytes), "r"(bar_cluster)
               : "memory");
}

// a.m_tiles x a.n_tiles tiles of 128 x BN; grid = 2 x tiles; a.num_kb >= 2; a.splits is not used.
template <int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    gemm_f16_tcgen05_k2_kernel(const __grid_constant__ CUtensorMap tmap_x,
                               const __grid_constant__ CUtensorMap tmap_w, const GemmArgs a) {
  using C = K2Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t staging = base + C::kStages * C::kStageBytes;           // [column group][128 rows] float4
  const uint32_t bars = staging + C::kStagingBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };
  const uint32_t tfull_bar = bars + 8u * (2 * C::kStages);
  const uint32_t data_bar = bars + 8u * (2 * C::kStages + 1);            // CTA 0: the peer's tile has landed
  const uint32_t tmem_slot = bars + 8u * (2 * C::kStages + 2);
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  float4* staging4 = reinterpret_cast<float4*>(gen_base + C::kStages * C::kStageBytes);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(
      gen_base + C::kStages * C::kStageBytes + C::kStagingBytes + 8 * (2 * C::kStages + 2));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int tile = blockIdx.x >> 1;
  int mt, nt;
  decode_tile(a, tile, mt, nt);
  const int half = (a.num_kb + 1) >> 1;
  const int kb0 = rank == 0 ? 0 : half, kb1 = rank == 0 ? half : a.num_kb;

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_x)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_w)) : "memory");
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    mbar_init(data_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (rank == 0) mbar_expect_tx(data_bar, C::kStagingBytes);    // armed before the peer can send
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  cluster_sync_all();          // both CTAs' barriers exist before anything crosses
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, a.status, ERR_PRODUCER)) break;
        mbar_expect_tx(full_bar(stage), C::kStageBytes);
        const uint32_t sa = base + stage * C::kStageBytes;
        tma_load_2d(sa, &tmap_x, kb * BK, mt * BM, full_bar(stage));
        tma_load_2d(sa + C::kABytes, &tmap_w, kb * BK, nt * BN, full_bar(stage));
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16_f32(BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(full_bar(stage), phase, a.status, ERR_MMA_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = base + stage * C::kStageBytes;
        const uint64_t da = make_kmajor_sw128_desc(sa);
        const uint64_t db = make_kmajor_sw128_desc(sa + C::kABytes);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk)
          umma_f16(tmem_base, da + 2u * kk, db + 2u * kk, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
        umma_commit(empty_bar(stage));
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
      if (ok) umma_commit(tfull_bar);
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int epi_tid = threadIdx.x - 64;
    const int r_in_tile = quarter * 32 + lane;
    const int row = mt * BM + r_in_tile;
    const bool row_ok = row < a.m;
    const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int col_base = nt * BN;
    bool ok = mbar_wait(tfull_bar, 0u, a.status, ERR_EPILOGUE);
    tc_fence_after();
    if (rank == 1) {
      // accumulator -> own staging area -> one bulk copy into CTA 0's staging area
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 8; ++q)
            staging4[(c * 8 + q) * BM + r_in_tile] =
                make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                            __uint_as_float(r[4 * q + 3]));
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the copy reads what the threads wrote
      epilogue_bar_sync();
      if (epi_tid == 0 && ok) bulk_copy_to_peer(mapa_u32(staging, 0), staging, C::kStagingBytes, mapa_u32(data_bar, 0));
    } else {
      if (ok) ok = mbar_wait(data_bar, 0u, a.status, ERR_K2_DATA);
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_addr + c * 32, r);
          tmem_ld_wait();
          const int col0 = col_base + c * 32;
          if (row_ok && col0 < a.n) {
            float f[32];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 v = staging4[(c * 8 + q) * BM + r_in_tile];
              f[4 * q] = __uint_as_float(r[4 * q]) + v.x;
              f[4 * q + 1] = __uint_as_float(r[4 * q + 1]) + v.y;
              f[4 * q + 2] = __uint_as_float(r[4 * q + 2]) + v.z;
              f[4 * q + 3] = __uint_as_float(r[4 * q + 3]) + v.w;
            }
            epi_store_row32(a.epi, a.y, a.ldy, a.vec_store, row, col0, a.n, f);
          }
        }
      }
    }
  }

  // CTA 1 may not leave while its copy is still reading its shared memory: CTA 0 comes here only
  // after the data barrier (or after giving up on it).
  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------
// The same hand-over for the swapped-operand kernel at m <= 64: K cut in S = 2, 3 or 4 slices, the
// S CTAs of a cluster.  CTAs 1 .. S-1 send their MN x 128 accumulators (8 - 32 KB) into slots of
// CTA 0's staging area with one bulk copy each; CTA 0 adds them to its own in rank order = K order.
// One 128-column tile of Y per cluster; single wave.
// ---------------------------------------------------------------------------------------
template <int MN>
struct SwapKcCfg {
  static constexpr int kWBytes = BM * BK * 2;
  static constexpr int kXBytes = MN * BK * 2;
  static constexpr int kXPad = (kXBytes + 1023) / 1024 * 1024;
  static constexpr int kStageBytes = kWBytes + kXPad;
  static constexpr int kSlotBytes = MN * BM * 4;                    // one accumulator tile: [row group][column] float4
  static constexpr int kStagingBytes = 3 * kSlotBytes;              // up to three peers
  static constexpr int kStages = (224 * 1024 - kStagingBytes) / kStageBytes > 12 ? 12 : (224 * 1024 - kStagingBytes) / kStageBytes;
  static constexpr int kTmemCols = MN < 32 ? 32 : MN;
  static constexpr int kBarBytes = (2 * kStages + 2) * 8 + 16;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kStagingBytes + kBarBytes;
  static_assert(kSmemBytes <= 227 * 1024 && kStages >= 4, "smem");
};

// a.n_tiles 128-column tiles; grid = S x a.n_tiles; a.num_kb >= S.
template <int MN, int S>
__global__ void __cluster_dims__(S, 1, 1) __launch_bounds__(kGemmThreads, 1)
    gemm_f16_tcgen05_swap_kc_kernel(const __grid_constant__ CUtensorMap tmap_w,
                                    const __grid_constant__ CUtensorMap tmap_x, const GemmArgs a) {
  using C = SwapKcCfg<MN>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t staging = base + C::kStages * C::kStageBytes;
  const uint32_t bars = staging + C::kStagingBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (C::kStages + s); };
  const uint32_t tfull_bar = bars + 8u * (2 * C::kStages);
  const uint32_t data_bar = bars + 8u * (2 * C::kStages + 1);
  const uint32_t tmem_slot = bars + 8u * (2 * C::kStages + 2);
  uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
  float4* staging4 = reinterpret_cast<float4*>(gen_base + C::kStages * C::kStageBytes);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(
      gen_base + C::kStages * C::kStageBytes + C::kStagingBytes + 8 * (2 * C::kStages + 2));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int nt = blockIdx.x / S;
  const int per = (a.num_kb + S - 1) / S;
  const int kb0 = min((int)rank * per, a.num_kb), kb1 = min(kb0 + per, a.num_kb);   // the last slices may be short or empty

  if (threadIdx.x == 0) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_w)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmap_x)) : "memory");
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(tfull_bar, 1);
    mbar_init(data_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (rank == 0) mbar_expect_tx(data_bar, (S - 1) * C::kSlotBytes);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(empty_bar(stage), phase ^ 1u, a.status, ERR_PRODUCER)) break;
        mbar_expect_tx(full_bar(stage), C::kWBytes + C::kXBytes);
        const uint32_t sa = base + stage * C::kStageBytes;
        tma_load_2d(sa, &tmap_w, kb * BK, nt * BM, full_bar(stage));
        tma_load_2d(sa + C::kWBytes, &tmap_x, kb * BK, 0, full_bar(stage));
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16_f32(MN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(full_bar(stage), phase, a.status, ERR_MMA_FULL)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = base + stage * C::kStageBytes;
        const uint64_t da = make_kmajor_sw128_desc(sa);
        const uint64_t db = make_kmajor_sw128_desc(sa + C::kWBytes);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk)
          umma_f16(tmem_base, da + 2u * kk, db + 2u * kk, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
        umma_commit(empty_bar(stage));
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
      }
      if (ok) umma_commit(tfull_bar);     // with an empty slice this arrives at once
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int epi_tid = threadIdx.x - 64;
    const int c_in_tile = quarter * 32 + lane;
    const int col = nt * BM + c_in_tile;
    const bool col_ok = col < a.n;
    const bool mine_empty = kb1 <= kb0;                 // nothing accumulated: this CTA contributes zeros
    const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    constexpr int kChunk = MN < 32 ? 16 : 32;
    bool ok = mbar_wait(tfull_bar, 0u, a.status, ERR_EPILOGUE);
    tc_fence_after();
    if (rank != 0) {
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < MN / kChunk; ++c) {
          uint32_t r[kChunk];
          if constexpr (kChunk == 16) tmem_ld16(t_addr + c * kChunk, r);
          else tmem_ld32(t_addr + c * kChunk, r);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < kChunk / 4; ++q) {
            const int g = c * (kChunk / 4) + q;
            staging4[g * BM + c_in_tile] =
                mine_empty ? make_float4(0.f, 0.f, 0.f, 0.f)
                           : make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                         __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
          }
        }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      epilogue_bar_sync();
      if (epi_tid == 0 && ok)
        bulk_copy_to_peer(mapa_u32(staging + (rank - 1) * C::kSlotBytes, 0), staging, C::kSlotBytes, mapa_u32(data_bar, 0));
    } else {
      if (ok) ok = mbar_wait(data_bar, 0u, a.status, ERR_K2_DATA);
      if (ok) {
        const float bias = (a.epi.bias != nullptr && col_ok) ? __half2float(a.epi.bias[col]) : 0.f;
#pragma unroll 1
        for (int c = 0; c < MN / kChunk; ++c) {
          uint32_t r[kChunk];
          if constexpr (kChunk == 16) tmem_ld16(t_addr + c * kChunk, r);
          else tmem_ld32(t_addr + c * kChunk, r);
          tmem_ld_wait();
          if (col_ok) {
            float f[kChunk];
#pragma unroll
            for (int j = 0; j < kChunk; ++j) f[j] = __uint_as_float(r[j]);
#pragma unroll
            for (int p = 0; p < S - 1; ++p) {          // rank order = K order
#pragma unroll
              for (int q = 0; q < kChunk / 4; ++q) {
                const float4 v = staging4[(p * (MN / 4) + c * (kChunk / 4) + q) * BM + c_in_tile];
                f[4 * q] += v.x; f[4 * q + 1] += v.y; f[4 * q + 2] += v.z; f[4 * q + 3] += v.w;
              }
            }
#pragma unroll
            for (int j = 0; j < kChunk; ++j) f[j] += bias;
            epi_store_column<kChunk>(a.epi, a.y, a.ldy, c * kChunk, a.m, col, f);
          }
        }
      }
    }
  }

  tc_fence_before();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---------------------------------------------------------------------------------------
// SIMT fallback for shapes TMA cannot describe (k % 8 != 0 or unaligned bases): one thread
// per output element, fp32 accumulation.  Correct for every shape, not a performance path.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
    gemm_f16_simt_kernel(const __half* __restrict__ x, const __half* __restrict__ w, const Epilogue epi,
                         void* __restrict__ y, int m, int n, int k, int64_t ldy) {
  const int col = blockIdx.x * 16 + (threadIdx.x & 15);
  const int row = blockIdx.y * 16 + (threadIdx.x >> 4);
  pdl_wait();
  pdl_launch_dependents();
  if (row >= m || col >= n) return;
  const __half* xr = x + (int64_t)row * k;
  const __half* wr = w + (int64_t)col * k;
  float acc = 0.f;
  for (int i = 0; i < k; ++i) acc = fmaf(__half2float(xr[i]), __half2float(wr[i]), acc);
  epi_store(epi, y, ldy, row, col, epi_value(epi, acc, row, col));
}

// ---------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D fp16 row-major [rows, cols] tensor, box = [box_rows, 64 cols], 128-byte swizzle,
// out-of-bounds elements read as zero.  Encoding costs a driver call; a descriptor depends
// only on (base, rows, cols, box rows), so each host thread keeps its last few.
struct TmapKey {
  const void* ptr;
  int64_t rows, cols;
  int box_rows;
};
struct TmapSlot {
  TmapKey key{nullptr, 0, 0, 0};
  CUtensorMap map;
};
constexpr int kTmapCacheSlots = 16;
thread_local TmapSlot tl_tmap_cache[kTmapCacheSlots];
thread_local int tl_tmap_next = 0;

int make_tmap(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int box_rows) {
  for (int i = 0; i < kTmapCacheSlots; ++i) {
    const TmapKey& k = tl_tmap_cache[i].key;
    if (k.ptr == ptr && k.rows == rows && k.cols == cols && k.box_rows == box_rows) {
      *map = tl_tmap_cache[i].map;
      return DTAS_OK;
    }
  }
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) DTAS_FAIL(DTAS_ECUDA, "gemm: cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), gdim, gstride, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) DTAS_FAIL(DTAS_ECUDA, "gemm: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  TmapSlot& slot = tl_tmap_cache[tl_tmap_next];
  tl_tmap_next = (tl_tmap_next + 1) % kTmapCacheSlots;
  slot.key = TmapKey{ptr, rows, cols, box_rows};
  slot.map = *map;
  return DTAS_OK;
}

struct GemmPlan {
  int bn;
  int splits;
  int kb_per_split;
  bool simt;
  bool pair = false;   // two-CTA 256 x 256 tiles (gemm_f16_tcgen05_pair_kernel)
  bool pair_sk = false;  //   ... with stream-K work distribution over the CTA pairs
  bool k2 = false;     // K cut in two inside a cluster of two CTAs (gemm_f16_tcgen05_k2_kernel<bn>), bn = 64 or 128
  int kc = 0;          // > 0: swapped operands, K cut in kc = 2..4 slices inside a cluster (m <= 64)
  int swap_mn = 0;     // > 0: swapped-operand kernel with the X tile padded to this many rows
  int sk_per = 0;      // swapped kernel, stream-K: (tile, k-block) units per CTA (0 = fixed split)
  int sk_grid = 0;     //   CTAs launched
  int slots_cap = 0;   //   partial slots reserved per tile
};

std::atomic<int> g_override_bn{0};
std::atomic<int> g_override_split{0};

// Measured dispatch table: (n, k, [m_lo, m_hi]) -> (tile code, split).  This is the counterpart of
// the reference's per-range best configs (python/dtas/engine/tuner.py:103-133): Engine.tune_module
// with search=True times the candidates on the device and installs the winners here; without
// entries the cost model below decides.
struct TableEntry {
  int64_t n, k, m_lo, m_hi;
  int bn, split;
};
std::vector<TableEntry> g_table;
std::mutex g_table_mutex;

bool table_lookup(int64_t m, int64_t n, int64_t k, int* bn, int* split) {
  std::lock_guard<std::mutex> lock(g_table_mutex);
  for (const TableEntry& e : g_table)
    if (e.n == n && e.k == k && m >= e.m_lo && m <= e.m_hi) {
      *bn = e.bn;
      *split = e.split;
      return true;
    }
  return false;
}

// Global override first, then the table, else 0 / 0 (cost model).
void effective_choice(int64_t m, int64_t n, int64_t k, int* bn, int* split) {
  *bn = g_override_bn.load();
  *split = g_override_split.load();
  if (*bn == 0 && *split == 0) {
    int tb = 0, ts = 0;
    if (table_lookup(m, n, k, &tb, &ts)) {
      *bn = tb;
      *split = ts;
    }
  }
  if ((*bn == 1024 || *bn == 2048) && m > 256) *bn = 0;   // the swapped kernel only exists for m <= 256
}

constexpr bool kStreamKByDefault = true; // stream-K candidates of the tiled kernel for mid m
constexpr int kStreamKMaxM = 1024;
constexpr bool kSwapByDefault = true;    // swapped-operand kernel for small m
constexpr int kSwapMaxM = 64;            // beyond that the X tile crowds W out of the ring
constexpr bool kPairByDefault = true;    // consider two-CTA tiles
constexpr int kScatterMinM = 129;        // dtas_gemm_nt_scatter: rows from which a 256-row tile is at least half full
constexpr int kPairMinM = 257;           // the cost model considers two-CTA tiles from here; a tuned table may choose them from m = 129
constexpr bool kK2ByDefault = true;      // consider the cluster K-split kernel where it fits one wave
constexpr bool kSwapKcByDefault = true;  // the same for the swapped-operand kernel
constexpr int kSwapKcMaxM = 64;          //   up to this m (the X tile of larger m leaves too little room for the slots)
constexpr size_t kSplitKWorkspaceBytes = 64ull << 20;
constexpr int kTileCounters = 16384;

// Tile width and split factor for a call shape: the idea of the reference's policy
// (python/dtas/policy/wmma_config_emiter.py:148-259 - score every candidate tile with a
// wave-quantised roofline model and keep the best), restated for one persistent CTA per
// SM.  For each (BN, splits) candidate the model charges per k-block the larger of
//   * the tensor/shared-memory time: max(2*BN MMA clocks, operand bytes / 128 B per clock),
//   * the HBM time of the distinct X and W tiles that the CTAs running side by side touch
//     (tiles shared inside a rasterisation band come from L2),
// adds a fixed fill/drain cost per work item, multiplies by the number of rounds
// ceil(work / SMs), and adds the partial-sum traffic of a split.  Larger BN wins ties.
// `lim` narrows the search for callers with their own scratch: no override / table, only the tiled
// single-CTA kernel with a fixed split, partial sums and counters within the given sizes.
struct PlanLimits {
  bool use_overrides = true;
  bool tiled_fixed_only = false;
  int64_t ws_bytes = (int64_t)kSplitKWorkspaceBytes;
  int64_t counters = kTileCounters;
};

GemmPlan plan_gemm(int64_t m, int64_t n, int64_t k, int sm_count, bool tma_ok, const PlanLimits& lim = PlanLimits()) {
  GemmPlan p{256, 1, 0, !tma_ok};
  const int num_kb = (int)((k + BK - 1) / BK);
  p.kb_per_split = num_kb;
  if (p.simt) return p;
  int obn0 = 0, osp0 = 0;
  if (lim.use_overrides) effective_choice(m, n, k, &obn0, &osp0);
  if ((obn0 == 8192 + 64 || obn0 == 8192 + 128) && num_kb >= 2) {   // tile codes 8256 / 8320
    p.bn = obn0 - 8192;
    p.splits = 1;
    p.k2 = true;
    return p;
  }
  if (obn0 >= 16384 + 2 && obn0 <= 16384 + 4 && m <= 64 && num_kb >= obn0 - 16384) {   // tile codes 16386 .. 16388
    p.swap_mn = m <= 16 ? 16 : (m <= 32 ? 32 : 64);
    p.bn = BM;
    p.splits = 1;
    p.kc = obn0 - 16384;
    return p;
  }
  if (obn0 >= 8192) obn0 = 0;      // not applicable to this shape: plan as usual
  if (!lim.tiled_fixed_only &&
      ((m <= 256 && (obn0 == 1024 || obn0 == 2048)) || (m <= kSwapMaxM && obn0 == 0 && kSwapByDefault))) {
    // Swapped-operand kernel: 128-row W tiles, split K until the work items fill the SMs.
    const int mn = m <= 16 ? 16 : (m <= 32 ? 32 : (m <= 64 ? 64 : (m <= 128 ? 128 : 256)));
    const int stage_bytes = BM * BK * 2 + ((mn * BK * 2 + 1023) / 1024) * 1024;
    int stages = kStageBudget / stage_bytes;
    if (stages > 12) stages = 12;
    const int64_t t = (n + BM - 1) / BM;
    constexpr double kClock = 1.7, kHbm = 6500.0;
    double best_cost = 1e30;
    int best_s = 1;
    for (int want = 1; want <= 32; ++want) {
      const int kb_per = (num_kb + want - 1) / want;
      const int sp = (num_kb + kb_per - 1) / kb_per;
      if (sp != want) continue;
      if (want > 1 && (kb_per < 2 || t > kTileCounters || (int64_t)sp * (t * BM) * mn * 4 > (int64_t)kSplitKWorkspaceBytes)) continue;
      if (osp0 > 0 && want != osp0 && !(want == 1 && osp0 > num_kb)) continue;
      const int64_t work = t * sp;
      const int64_t rounds = (work + sm_count - 1) / sm_count;
      const double active = (double)(work < sm_count ? work : sm_count);
      const double smem_clk = (double)stage_bytes / 128.0, mma_clk = 2.0 * mn;
      const double t_core = (mma_clk > smem_clk ? mma_clk : smem_clk) / kClock;
      const double t_hbm = (active * BM * BK * 2 + mn * BK * 2) / kHbm;
      // A CTA alone pulls one stage per (ring round trip / stages); the round trip measured
      // 2.6 us on B200 (TMA issue -> data -> MMA -> commit -> producer wake-up).
      const double t_lat = 2600.0 / stages;
      double t_kb = t_core > t_hbm ? t_core : t_hbm;
      if (t_lat > t_kb) t_kb = t_lat;
      double cost = (double)rounds * (kb_per * t_kb + 3000.0);
      // the last CTA of a tile sums the partials in batches of 2 row groups x 4 splits, one L2
      // round trip (~0.7 us) per batch
      if (sp > 1) cost += 1500.0 + 700.0 * (double)((((m + 3) / 4) + 1) / 2) * (double)((sp + 3) / 4);
      if (cost < best_cost * 0.999) {
        best_cost = cost;
        best_s = sp;
      }
    }
    p.swap_mn = mn;
    p.bn = BM;
    p.splits = best_s;
    p.kb_per_split = (num_kb + best_s - 1) / best_s;
    p.slots_cap = best_s;
    // Stream-K: every CTA streams the same number of k-blocks whatever the tile count; only
    // tiles that straddle two CTAs' ranges go through the workspace.
    if (obn0 == 2048 || (obn0 == 0 && osp0 == 0)) {
      const int64_t total = t * num_kb;
      int64_t grid = total / 2 < sm_count ? total / 2 : sm_count;
      if (grid < 1) grid = 1;
      const int64_t per = (total + grid - 1) / grid;
      grid = (total + per - 1) / per;
      const int slots = (int)((num_kb - 1) / per) + 2;
      const bool fits = t <= kTileCounters && t * slots * (int64_t)mn * BM * 4 <= (int64_t)kSplitKWorkspaceBytes;
      if (fits && total < 0x7fffffffLL) {
        const double smem_clk = (double)stage_bytes / 128.0, mma_clk = 2.0 * mn;
        const double t_core = (mma_clk > smem_clk ? mma_clk : smem_clk) / kClock;
        const double t_hbm = ((double)grid * BM * BK * 2 + mn * BK * 2) / kHbm;
        const double t_lat = 2600.0 / stages;
        double t_kb = t_core > t_hbm ? t_core : t_hbm;
        if (t_lat > t_kb) t_kb = t_lat;
        double cost = (double)per * t_kb + 3000.0;
        if (per % num_kb != 0)   // some tile is shared between CTAs
          cost += 1500.0 + 700.0 * (double)((((m + 3) / 4) + 1) / 2) * (double)((slots + 3) / 4);
        if (obn0 == 2048 || cost < best_cost) {
          p.sk_per = (int)per;
          p.sk_grid = (int)grid;
          p.slots_cap = slots;
          p.splits = 1;
          p.kb_per_split = num_kb;
        }
      }
    }
    // Fixed split of 2..4 in one wave at m <= 32: the slices are the CTAs of a cluster and hand over through
    // shared memory instead of the workspace.
    if (kSwapKcByDefault && obn0 == 0 && osp0 == 0 && p.sk_per == 0 && m <= kSwapKcMaxM && p.splits >= 2 && p.splits <= 4 &&
        t * p.splits <= sm_count - (p.splits >= 3 ? 16 : 4)) {   // clusters do not pack every SM of every GPC
      p.kc = p.splits;
      p.splits = 1;
    }
    return p;
  }
  const int64_t m_tiles = (m + BM - 1) / BM;
  auto tiles = [&](int bn) { return m_tiles * ((n + bn - 1) / bn); };
  auto ws_ok = [&](int bn, int slots) {   // partial tiles: [n tile][slot][BN/4][m] float4
    const int64_t n_pad = ((n + bn - 1) / bn) * bn;
    return tiles(bn) <= lim.counters && (int64_t)slots * m * n_pad * 4 <= lim.ws_bytes;
  };

  constexpr double kClockGHz = 1.7, kHbmGBs = 6500.0, kItemFixedNs = 1500.0;
  static const int kBn[3] = {256, 128, 64};
  static const int kSplits[10] = {1, 2, 3, 4, 5, 6, 8, 10, 12, 16};
  double best = 1e30;
  int best_bn = 256, best_splits = 1;
  double k2_cost = 1e30;     // K cut in two inside a cluster (single wave only): no workspace tail
  int k2_bn = 0;
  for (int bi = 0; bi < 3; ++bi) {
    const int bn = kBn[bi];
    const int64_t n_tiles = (n + bn - 1) / bn;
    const int64_t t = m_tiles * n_tiles;
    for (int si = 0; si < 10; ++si) {
      const int want = kSplits[si];
      if (want > 1 && (m > 512 || !ws_ok(bn, want))) continue;
      const int kb_per = (num_kb + want - 1) / want;
      const int s = (num_kb + kb_per - 1) / kb_per;
      if (s != want || (want > 1 && kb_per < 2)) continue;
      const int64_t work = t * s;
      const int64_t rounds = (work + sm_count - 1) / sm_count;
      const double active = (double)(work < sm_count ? work : sm_count);
      const double smem_clk = (double)(BM * BK * 2 + bn * BK * 2) / 128.0;
      const double mma_clk = 2.0 * bn;
      // Narrow tiles re-read the X tile from shared memory per MMA and ran at 0.7x / 0.45x
      // the per-flop rate of BN = 256 when measured on B200.
      const double narrow = bn == 256 ? 1.0 : (bn == 128 ? 1.4 : 2.2);
      const double t_core = narrow * (mma_clk > smem_clk ? mma_clk : smem_clk) / kClockGHz;
      // HBM bytes per k-block over the whole machine: the CTAs running side by side cover
      // am m-tiles x an n-tiles of one band and share those X and W tiles through L2.
      const double rows_x = (double)(m < BM ? m : BM);
      const double am = (double)(m_tiles < kGroupM ? m_tiles : kGroupM);
      const double an = active / am < 1.0 ? 1.0 : active / am;
      const double t_hbm = 128.0 * (an * bn + am * rows_x) / kHbmGBs;
      double cost = (double)rounds * (kb_per * (t_core > t_hbm ? t_core : t_hbm) + kItemFixedNs);
      if (s == 2 && bn <= 128 && work <= sm_count - 4 && kK2ByDefault && !lim.tiled_fixed_only) {
        // the same main loop, the second half handed over through shared memory (~1.5 us measured
        // against ~4.5 us through the workspace at m = 255)
        const double c2 = cost + 1500.0;
        if (c2 < k2_cost * 0.999) {
          k2_cost = c2;
          k2_bn = bn;
        }
      }
      // split-K tail: partial traffic, plus the last CTA summing chunk by chunk and split by
      // split, one L2 round trip (~0.7 us) each
      if (s > 1) cost += 2.0 * s * (double)m * (double)n * 4.0 / kHbmGBs + 1500.0 + 700.0 * (bn / 32) * ((s + 1) / 2);
      if (cost < best * 0.999) {
        best = cost;
        best_bn = bn;
        best_splits = s;
      }
    }
  }
  // Stream-K candidates (tile codes 4096 + BN): the (tile, k-block) units are dealt out in equal
  // consecutive runs, one per CTA; tiles shared between CTAs are finished through the workspace.
  struct SkPlan {
    int per = 0, grid = 0, slots = 0;
    double cost = 1e30;
  };
  auto sk_plan = [&](int bn) {
    SkPlan q;
    const int64_t n_tiles = (n + bn - 1) / bn;
    const int64_t total = m_tiles * n_tiles * num_kb;
    if (total >= 0x7fffffffLL) return q;
    int64_t grid = total / 2 < sm_count ? total / 2 : sm_count;
    if (grid < 1) grid = 1;
    const int64_t per = (total + grid - 1) / grid;
    grid = (total + per - 1) / per;
    const int slots = (int)((num_kb - 1) / per) + 2;
    // partials: two tile-sized areas per CTA, whatever m and n; counters: one per tile
    if (m_tiles * n_tiles > lim.counters || grid * 2 * (int64_t)BM * bn * 4 > lim.ws_bytes) return q;
    const double smem_clk = (double)(BM * BK * 2 + bn * BK * 2) / 128.0, mma_clk = 2.0 * bn;
    const double narrow = bn == 256 ? 1.0 : (bn == 128 ? 1.4 : 2.2);
    const double t_core = narrow * (mma_clk > smem_clk ? mma_clk : smem_clk) / kClockGHz;
    const double rows_x = (double)(m < BM ? m : BM);
    const double am = (double)(m_tiles < kGroupM ? m_tiles : kGroupM);
    const double an = (double)grid / am < 1.0 ? 1.0 : (double)grid / am;
    const double t_hbm = 128.0 * (an * bn + am * rows_x) / kHbmGBs;
    q.cost = (double)per * (t_core > t_hbm ? t_core : t_hbm) + 2.0 * kItemFixedNs;
    if (per % num_kb != 0)
      q.cost += 2.0 * (double)grid * BM * bn * 4.0 * 2.0 / kHbmGBs / 4.0 + 1500.0 + 700.0 * (bn / 32) * ((slots + 1) / 2);
    q.per = (int)per;
    q.grid = (int)grid;
    q.slots = slots;
    return q;
  };
  SkPlan sk;
  int sk_bn = 0;
  if (obn0 >= 4096) {
    sk_bn = obn0 - 4096;
    sk = sk_plan(sk_bn);
    if (sk.per == 0) sk_bn = 0;   // does not fit the workspace: fall through to the fixed plan
  } else if (obn0 == 0 && osp0 == 0 && kStreamKByDefault && m <= kStreamKMaxM && !lim.tiled_fixed_only) {
    for (int bi = 0; bi < 3; ++bi) {
      const SkPlan q = sk_plan(kBn[bi]);
      if (q.per > 0 && q.cost < sk.cost * 0.999) {
        sk = q;
        sk_bn = kBn[bi];
      }
    }
    if (!(sk.cost < best)) sk_bn = 0;
    else best = sk.cost;
  }
  int bn = best_bn, splits = best_splits;
  const int obn = obn0 >= 4096 ? 0 : obn0, osp = osp0;
  // The two-CTA kernel as one more candidate: 256 x 256 tiles on SM pairs.  Measured per
  // k-block it runs at about 0.9x the time of two single-CTA 128 x 256 tiles (1.40-1.50
  // PFLOP/s against 1.30-1.33 at m >= 4096), and its ring is deeper.
  bool pair = false;
  if (kPairByDefault && m >= kPairMinM && !lim.tiled_fixed_only) {
    const int64_t pm = (m + 2 * BM - 1) / (2 * BM), pn = (n + kPairBN - 1) / kPairBN;
    const int64_t work = pm * pn, slots = sm_count / 2 > 0 ? sm_count / 2 : 1;
    const int64_t rounds = (work + slots - 1) / slots;
    const double active = (double)(work < slots ? work : slots);
    const double t_core = 0.9 * 512.0 / kClockGHz;
    const double am = (double)(pm < kPairGroupM ? pm : kPairGroupM);
    const double an = active / am < 1.0 ? 1.0 : active / am;
    const double t_hbm = 128.0 * (an * kPairBN + am * 2 * BM) / kHbmGBs;
    const double cost = (double)rounds * (num_kb * (t_core > t_hbm ? t_core : t_hbm) + kItemFixedNs);
    pair = cost < (k2_cost < best ? k2_cost : best);
  }
  if (obn == 512 || obn == 513) pair = true;
  if (obn == 64 || obn == 128 || obn == 256) pair = false;
  if (pair && obn0 < 4096) {
    p.bn = 256;
    p.splits = 1;
    p.kb_per_split = num_kb;
    p.pair = true;
    // Stream-K over the pairs only on request (tile code 513, from a tuned table): parking a 128 x 256
    // fp32 partial per CTA and reading the others back with four warps (~40 GB/s) costs more than an
    // empty half wave saves on the shapes measured so far (m = 4096, N = 512: 38.6 us against 25.4).
    const int64_t pm = (m + 2 * BM - 1) / (2 * BM), pn = (n + kPairBN - 1) / kPairBN;
    const int64_t tiles = pm * pn, slots = sm_count / 2 > 0 ? sm_count / 2 : 1;
    const bool fits = tiles * 2 <= lim.counters && slots * 4 * (int64_t)BM * kPairBN * 4 <= lim.ws_bytes &&
                      tiles * num_kb < 0x7fffffffLL;
    p.pair_sk = fits && !lim.tiled_fixed_only && obn == 513;
    return p;
  }
  if (k2_bn > 0 && k2_cost < best && obn == 0 && osp == 0 && obn0 < 4096) {
    p.bn = k2_bn;
    p.splits = 1;
    p.k2 = true;
    return p;
  }
  if (sk_bn > 0) {
    p.bn = sk_bn;
    p.splits = 1;
    p.kb_per_split = num_kb;
    p.sk_per = sk.per;
    p.sk_grid = sk.grid;
    p.slots_cap = sk.slots;
    return p;
  }
  if (obn == 64 || obn == 128 || obn == 256) {
    bn = obn;
    if (osp <= 0 && !ws_ok(bn, splits)) splits = 1;
  }
  if (osp > 0) {
    splits = osp > num_kb ? num_kb : osp;
    if (splits > 1 && !ws_ok(bn, splits)) splits = 1;
  }
  const int kb_per = (num_kb + splits - 1) / splits;
  splits = (num_kb + kb_per - 1) / kb_per;   // no empty slice
  p.bn = bn;
  p.splits = splits;
  p.kb_per_split = kb_per;
  p.slots_cap = splits;
  return p;
}

template <int BN>
int launch_tc(const CUtensorMap& tx, const CUtensorMap& tw, const GemmArgs& a, int sm_count,
              cudaStream_t st) {
  using C = Cfg<BN>;
  static std::atomic<bool> attr_set[64];   // zero-initialised; set after the attribute call returned
  int dev = 0;
  DTAS_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
    DTAS_CUDA(cudaFuncSetAttribute(gemm_f16_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   C::kSmemBytes));
    attr_set[dev].store(true, std::memory_order_release);
  }
  const int total = a.m_tiles * a.n_tiles * a.splits;
  int grid = total < sm_count ? total : sm_count;
  if (a.sk_per > 0) grid = (a.m_tiles * a.n_tiles * a.num_kb + a.sk_per - 1) / a.sk_per;
  launch_kernel(gemm_f16_tcgen05_kernel<BN>, grid, kGemmThreads, C::kSmemBytes, st, tx, tw, a);
  return after_launch("gemm_f16_tcgen05_kernel");
}

int launch_pair(const CUtensorMap& tx, const CUtensorMap& tw, const GemmArgs& a, int sm_count, cudaStream_t st, bool stream_k) {
  static std::atomic<bool> attr_set[64];   // zero-initialised; set after the attribute call returned
  static int max_pairs[64] = {0};
  int dev = 0;
  DTAS_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
    DTAS_CUDA(cudaFuncSetAttribute(gemm_f16_tcgen05_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   kPairSmemBytes));
    // how many CTA pairs the device can hold at once (one CTA per SM, pairs share a TPC)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (unsigned)(sm_count / 2));
    cfg.blockDim = dim3(kPairMaxThreads);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_f16_tcgen05_pair_kernel, &cfg) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = sm_count / 2;
    }
    max_pairs[dev] = n;
    attr_set[dev].store(true, std::memory_order_release);
  }
  const int total = a.m_tiles * a.n_tiles;
  int pairs = dev < 64 ? max_pairs[dev] : sm_count / 2;
  GemmArgs ap = a;
  ap.sk_per = 0;
  ap.sk_first = total;
  const int tail = total % pairs;       // tiles of the last, partial wave
  if (stream_k && tail > 0) {
    const int region = tail;
    const int64_t units = (int64_t)region * a.num_kb;
    ap.sk_first = total - region;
    ap.sk_per = (int)((units + pairs - 1) / pairs);     // every pair takes part: the grid stays at `pairs`
  } else if (pairs > total) {
    pairs = total;
  }
  // twice the epilogue warps when there is an activation or a residual to work through per element, or
  // partial tiles to read back (the read rate of a CTA grows with the warps that issue the loads)
  const int threads = (epi_has_work(a.epi) || ap.sk_per > 0) ? kPairMaxThreads : kGemmThreads;
  launch_kernel(gemm_f16_tcgen05_pair_kernel, 2 * pairs, threads, kPairSmemBytes, st, tx, tw, ap);
  return after_launch("gemm_f16_tcgen05_pair_kernel");
}

template <int BN>
int launch_k2(const CUtensorMap& tx, const CUtensorMap& tw, const GemmArgs& a, cudaStream_t st) {
  using C = K2Cfg<BN>;
  static std::atomic<bool> attr_set[64];   // zero-initialised; set after the attribute call returned
  int dev = 0;
  DTAS_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
    DTAS_CUDA(cudaFuncSetAttribute(gemm_f16_tcgen05_k2_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   C::kSmemBytes));
    attr_set[dev].store(true, std::memory_order_release);
  }
  const int64_t grid = 2ll * a.m_tiles * a.n_tiles;
  if (grid > 0x7fffffffLL) DTAS_FAIL(DTAS_EINVAL, "gemm: too many tiles");
  launch_kernel(gemm_f16_tcgen05_k2_kernel<BN>, (unsigned)grid, kGemmThreads, C::kSmemBytes, st, tx, tw, a);
  return after_launch("gemm_f16_tcgen05_k2_kernel");
}

template <int MN, int S>
int launch_swap_kc(const CUtensorMap& tw, const CUtensorMap& tx, const GemmArgs& a, cudaStream_t st) {
  using C = SwapKcCfg<MN>;
  static std::atomic<bool> attr_set[64];   // zero-initialised; set after the attribute call returned
  int dev = 0;
  DTAS_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
    DTAS_CUDA(cudaFuncSetAttribute((gemm_f16_tcgen05_swap_kc_kernel<MN, S>), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   C::kSmemBytes));
    attr_set[dev].store(true, std::memory_order_release);
  }
  const int64_t grid = (int64_t)S * a.n_tiles;
  if (grid > 0x7fffffffLL) DTAS_FAIL(DTAS_EINVAL, "gemm: too many tiles");
  launch_kernel(gemm_f16_tcgen05_swap_kc_kernel<MN, S>, (unsigned)grid, kGemmThreads, C::kSmemBytes, st, tw, tx, a);
  return after_launch("gemm_f16_tcgen05_swap_kc_kernel");
}

template <int MN>
int launch_swap(const CUtensorMap& tw, const CUtensorMap& tx, const GemmArgs& a, int sm_count, cudaStream_t st) {
  using C = SwapCfg<MN>;
  static std::atomic<bool> attr_set[64];   // zero-initialised; set after the attribute call returned
  int dev = 0;
  DTAS_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev].load(std::memory_order_acquire)) {
    DTAS_CUDA(cudaFuncSetAttribute(gemm_f16_tcgen05_swap_kernel<MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   C::kSmemBytes));
    attr_set[dev].store(true, std::memory_order_release);
  }
  const int total = a.n_tiles * a.splits;
  int grid = total < sm_count ? total : sm_count;
  if (a.sk_per > 0) grid = (a.n_tiles * a.num_kb + a.sk_per - 1) / a.sk_per;
  launch_kernel(gemm_f16_tcgen05_swap_kernel<MN>, grid, kGemmThreads, C::kSmemBytes, st, tw, tx, a);
  return after_launch("gemm_f16_tcgen05_swap_kernel");
}

bool gemm_tma_ok(const void* x, const void* w, int64_t k) {
  return (k % 8 == 0) && aligned16(x) && aligned16(w);
}

}  // namespace

// A new range replaces whatever the table held for the same (n, k) inside [m_lo, m_hi]: entries that
// overlap it are trimmed to the part outside (an entry that straddles it is cut in two), so that the
// latest measurement always wins, whatever ranges an earlier table used.
int gemm_table_set(int64_t n, int64_t k, int64_t m_lo, int64_t m_hi, int bn, int split_k) {
  std::lock_guard<std::mutex> lock(g_table_mutex);
  std::vector<TableEntry> kept;
  kept.reserve(g_table.size() + 2);
  for (const TableEntry& e : g_table) {
    if (e.n != n || e.k != k || e.m_hi < m_lo || e.m_lo > m_hi) {
      kept.push_back(e);
      continue;
    }
    if (e.m_lo < m_lo) kept.push_back(TableEntry{n, k, e.m_lo, m_lo - 1, e.bn, e.split});
    if (e.m_hi > m_hi) kept.push_back(TableEntry{n, k, m_hi + 1, e.m_hi, e.bn, e.split});
  }
  kept.push_back(TableEntry{n, k, m_lo, m_hi, bn, split_k});
  g_table.swap(kept);
  return DTAS_OK;
}

void gemm_table_clear() {
  std::lock_guard<std::mutex> lock(g_table_mutex);
  g_table.clear();
}

void gemm_set_override(int bn, int split_k) {
  g_override_bn.store(bn);
  g_override_split.store(split_k);
}

static std::mutex g_splitk_mutex;

// Creates one scratch set.  May run while a stream of this thread is being captured: the capture mode
// is relaxed for the duration (as allocators that serve captured work do), and the counters are
// zeroed through a private stream that is waited for, so the set is ready before any launch.
static int create_splitk_set(SplitKScratch* s) {
  cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
  DTAS_CUDA(cudaThreadExchangeStreamCaptureMode(&mode));
  float* w = nullptr;
  int* c = nullptr;
  cudaStream_t tmp = nullptr;
  cudaError_t e = cudaMalloc(&w, kSplitKWorkspaceBytes);
  if (e == cudaSuccess) e = cudaMalloc(&c, kTileCounters * sizeof(int));
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&tmp, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaMemsetAsync(c, 0, kTileCounters * sizeof(int), tmp);
  if (e == cudaSuccess) e = cudaStreamSynchronize(tmp);
  if (tmp != nullptr) cudaStreamDestroy(tmp);
  cudaThreadExchangeStreamCaptureMode(&mode);
  if (e != cudaSuccess) {
    if (w != nullptr) cudaFree(w);
    if (c != nullptr) cudaFree(c);
    (void)cudaGetLastError();
    DTAS_FAIL(DTAS_ECUDA, "gemm: creating the split-K scratch failed: %s", cudaGetErrorString(e));
  }
  s->ws = w;          // published last, under the caller's lock: nobody sees half a set
  s->counters = c;
  s->used = true;
  return DTAS_OK;
}

// Split-K calls are re-entrant across streams: the partial tiles and arrival counters a call uses
// belong to its stream.  A stream gets its set on its first split-K call (two cudaMallocs), up to
// kSplitKSlots sets per device.  When more streams than that issue split-K calls, the least recently
// used set moves to the new stream, ordered behind everything submitted so far to its previous owner
// by an event, so the two never overlap on it.  Calls that are being captured into a CUDA graph use
// one further set of their own, shared by all graphs of the device: replays on one stream are
// ordered; graphs holding split-K calls must not be replayed at the same time on different streams.
int acquire_splitk_scratch(DeviceCtx* ctx, cudaStream_t st, float** ws, int** counters) {
  std::lock_guard<std::mutex> lock(g_splitk_mutex);
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) {
    (void)cudaGetLastError();
    cap = cudaStreamCaptureStatusNone;
  }
  if (cap != cudaStreamCaptureStatusNone) {
    SplitKScratch* s = &ctx->splitk_capture;
    if (!s->used) {
      int rc = create_splitk_set(s);
      if (rc != DTAS_OK) return rc;
    }
    *ws = s->ws;
    *counters = s->counters;
    return DTAS_OK;
  }
  const uint64_t now = ++ctx->splitk_clock;
  SplitKScratch* unused = nullptr;
  SplitKScratch* lru = nullptr;
  for (SplitKScratch& s : ctx->splitk) {
    if (s.used && s.stream == st) {
      s.last_use = now;
      *ws = s.ws;
      *counters = s.counters;
      return DTAS_OK;
    }
    if (!s.used) {
      if (unused == nullptr) unused = &s;
    } else if (lru == nullptr || s.last_use < lru->last_use) {
      lru = &s;
    }
  }
  if (unused != nullptr) {
    unused->stream = st;
    unused->last_use = now;
    int rc = create_splitk_set(unused);
    if (rc != DTAS_OK) return rc;
    *ws = unused->ws;
    *counters = unused->counters;
    return DTAS_OK;
  }
  cudaEvent_t ev = nullptr;
  bool ordered = false;
  if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) == cudaSuccess) {
    if (cudaEventRecord(ev, lru->stream) == cudaSuccess && cudaStreamWaitEvent(st, ev, 0) == cudaSuccess) ordered = true;
    cudaEventDestroy(ev);
  }
  if (!ordered) {           // the previous owner no longer exists as a stream: wait for the whole device once
    (void)cudaGetLastError();
    DTAS_CUDA(cudaDeviceSynchronize());
  }
  lru->stream = st;
  lru->last_use = now;
  *ws = lru->ws;
  *counters = lru->counters;
  return DTAS_OK;
}

// A kernel that gave up on a bounded wait may leave arrival counters of its tiles non-zero; every
// later split-K launch on that set would then misjudge who arrives last.  Called with the device idle.
int reset_splitk_counters(DeviceCtx* ctx) {
  std::lock_guard<std::mutex> lock(g_splitk_mutex);
  for (SplitKScratch& s : ctx->splitk)
    if (s.used) DTAS_CUDA(cudaMemset(s.counters, 0, kTileCounters * sizeof(int)));
  if (ctx->splitk_capture.used) DTAS_CUDA(cudaMemset(ctx->splitk_capture.counters, 0, kTileCounters * sizeof(int)));
  DTAS_CUDA(cudaDeviceSynchronize());
  return DTAS_OK;
}

void free_splitk_scratch(DeviceCtx* ctx) {
  std::lock_guard<std::mutex> lock(g_splitk_mutex);
  for (SplitKScratch& s : ctx->splitk) {
    if (!s.used) continue;
    cudaFree(s.ws);
    cudaFree(s.counters);
    s = SplitKScratch();
  }
  if (ctx->splitk_capture.used) {
    cudaFree(ctx->splitk_capture.ws);
    cudaFree(ctx->splitk_capture.counters);
    ctx->splitk_capture = SplitKScratch();
  }
}

// Fills the launcher-owned fields of the epilogue and says whether 16-byte stores into Y rows are aligned.
static int finish_epilogue(Epilogue& e, const void* y, int64_t ldy) {
  e.vec_res = ((e.res1 == nullptr || aligned16(e.res1)) && (e.res2 == nullptr || aligned16(e.res2)) &&
               e.ldr % 8 == 0) ? 1 : 0;
  return (aligned16(y) && ldy % (e.out_f32 ? 4 : 8) == 0) ? 1 : 0;
}

int launch_gemm(const void* x, const void* w, const Epilogue& epi, void* y, int64_t m, int64_t n,
                int64_t k, int64_t ldy, DeviceCtx* ctx, cudaStream_t st, const PeerOut* peers) {
  if (m > 0x7fffffffLL / 2 || n > 0x7fffffffLL / 2 || k > 0x7fffffffLL / 2)
    DTAS_FAIL(DTAS_EINVAL, "gemm: dimension too large");
  GemmPlan p = plan_gemm(m, n, k, ctx->sm_count, gemm_tma_ok(x, w, k));
  const bool scatter = peers != nullptr && peers->n > 0;
  if (scatter && !p.pair) {
    // only the two-CTA kernel stores to further buffers; it serves any m, at a loss below ~128 rows
    if (p.simt || m < kScatterMinM)
      DTAS_FAIL(DTAS_EUNSUPPORTED, "gemm (scatter): needs m >= %d, 16-byte aligned operands and k a multiple of 8", kScatterMinM);
    p = GemmPlan{256, 1, (int)((k + BK - 1) / BK), false};
    p.pair = true;
  }
  if (p.simt) {
    dim3 grid((unsigned)((n + 15) / 16), (unsigned)((m + 15) / 16));
    if (grid.y > 65535) DTAS_FAIL(DTAS_EUNSUPPORTED, "gemm: unaligned operands with m > 1048560");
    launch_kernel(gemm_f16_simt_kernel, grid, 256, 0, st, (const __half*)x, (const __half*)w, epi, y, (int)m,
                  (int)n, (int)k, ldy);
    return after_launch("gemm_f16_simt_kernel");
  }
  float* ws = nullptr;
  int* counters = nullptr;
  if (p.splits > 1 || p.sk_per > 0 || p.pair_sk) {
    int rc = acquire_splitk_scratch(ctx, st, &ws, &counters);
    if (rc != DTAS_OK) return rc;
  }
  CUtensorMap tx, tw;
  int rc = make_tmap(&tx, x, m, k, p.swap_mn > 0 ? p.swap_mn : BM);
  if (rc != DTAS_OK) return rc;
  rc = make_tmap(&tw, w, n, k, p.pair ? kPairBN / 2 : p.bn);
  if (rc != DTAS_OK) return rc;

  GemmArgs a;
  a.y = y;
  a.epi = epi;
  a.ws = ws;
  a.counters = counters;
  a.status = ctx->status;
  a.ldy = ldy;
  a.m = (int)m;
  a.n = (int)n;
  a.k = (int)k;
  a.m_tiles = (int)((m + BM - 1) / BM);
  a.n_tiles = (int)((n + p.bn - 1) / p.bn);
  a.splits = p.splits;
  a.sk_per = p.swap_mn > 0 ? 0 : p.sk_per;
  a.slots_cap = p.slots_cap > 0 ? p.slots_cap : p.splits;
  a.kb_per_split = p.kb_per_split;
  a.num_kb = (int)((k + BK - 1) / BK);
  a.vec_store = finish_epilogue(a.epi, y, ldy);
  if (scatter) {
    a.peers = *peers;
    for (int j = 0; j < peers->n; ++j)
      if (!aligned16(peers->y[j])) a.vec_store = 0;      // scalar stores everywhere rather than a fault
  }
  if ((int64_t)a.m_tiles * a.n_tiles * a.splits > 0x7fffffffLL)
    DTAS_FAIL(DTAS_EINVAL, "gemm: too many tiles");
  if (p.k2) return p.bn == 128 ? launch_k2<128>(tx, tw, a, st) : launch_k2<64>(tx, tw, a, st);
  if (p.pair) {
    a.m_tiles = (int)((m + 2 * BM - 1) / (2 * BM));
    a.n_tiles = (int)((n + kPairBN - 1) / kPairBN);
    return launch_pair(tx, tw, a, ctx->sm_count, st, p.pair_sk);
  }
  if (p.swap_mn > 0) {
    a.m_tiles = 1;
    a.n_tiles = (int)((n + BM - 1) / BM);
    a.sk_per = p.sk_per;
    a.slots_cap = p.slots_cap;
    if (p.kc > 0) {
      const int code = (p.swap_mn == 16 ? 0 : (p.swap_mn == 32 ? 10 : 20)) + p.kc;
      switch (code) {
        case 2: return launch_swap_kc<16, 2>(tw, tx, a, st);
        case 3: return launch_swap_kc<16, 3>(tw, tx, a, st);
        case 4: return launch_swap_kc<16, 4>(tw, tx, a, st);
        case 12: return launch_swap_kc<32, 2>(tw, tx, a, st);
        case 13: return launch_swap_kc<32, 3>(tw, tx, a, st);
        case 14: return launch_swap_kc<32, 4>(tw, tx, a, st);
        case 22: return launch_swap_kc<64, 2>(tw, tx, a, st);
        case 23: return launch_swap_kc<64, 3>(tw, tx, a, st);
        default: return launch_swap_kc<64, 4>(tw, tx, a, st);
      }
    }
    switch (p.swap_mn) {
      case 16: return launch_swap<16>(tw, tx, a, ctx->sm_count, st);
      case 32: return launch_swap<32>(tw, tx, a, ctx->sm_count, st);
      case 64: return launch_swap<64>(tw, tx, a, ctx->sm_count, st);
      case 128: return launch_swap<128>(tw, tx, a, ctx->sm_count, st);
      default: return launch_swap<256>(tw, tx, a, ctx->sm_count, st);
    }
  }
  switch (p.bn) {
    case 256: return launch_tc<256>(tx, tw, a, ctx->sm_count, st);
    case 128: return launch_tc<128>(tx, tw, a, ctx->sm_count, st);
    default: return launch_tc<64>(tx, tw, a, ctx->sm_count, st);
  }
}

void gemm_variant_name(int64_t m, int64_t n, int64_t k, const DeviceCtx* ctx, char* buf, int len) {
  const GemmPlan p = plan_gemm(m, n, k, ctx ? ctx->sm_count : 148, k % 8 == 0);
  if (p.simt) {
    snprintf(buf, len, "gemm_simt_fallback");
    return;
  }
  if (p.pair) {
    snprintf(buf, len, "gemm_tcgen05_2cta_bm256_bn256_bk64_s%d%s", kPairStages, p.pair_sk ? "_streamk" : "");
    return;
  }
  if (p.k2) {
    snprintf(buf, len, "gemm_tcgen05_bm128_bn%d_bk64_s%d_k2cluster", p.bn, p.bn == 128 ? K2Cfg<128>::kStages : K2Cfg<64>::kStages);
    return;
  }
  if (p.swap_mn > 0 && p.kc > 0) {
    snprintf(buf, len, "gemm_tcgen05_swap_n128_m%d_bk64_k%dcluster", p.swap_mn, p.kc);
    return;
  }
  if (p.swap_mn > 0) {
    if (p.sk_per > 0)
      snprintf(buf, len, "gemm_tcgen05_swap_n128_m%d_bk64_streamk%d", p.swap_mn, p.sk_grid);
    else
      snprintf(buf, len, "gemm_tcgen05_swap_n128_m%d_bk64_splitk%d", p.swap_mn, p.splits);
    return;
  }
  if (p.sk_per > 0) {
    snprintf(buf, len, "gemm_tcgen05_bm128_bn%d_bk64_streamk%d", p.bn, p.sk_grid);
    return;
  }
  const int stages = p.bn == 256 ? Cfg<256>::kStages : (p.bn == 128 ? Cfg<128>::kStages : Cfg<64>::kStages);
  snprintf(buf, len, "gemm_tcgen05_bm128_bn%d_bk64_s%d_splitk%d", p.bn, stages, p.splits);
}


// ---------------------------------------------------------------------------------------
// Split-K GEMM on scratch that lives inside the library image
// ---------------------------------------------------------------------------------------
// Some hosts of this library cannot create device memory at the moment they call it: an
// inference runtime that handed the whole device to its own pool at start-up (a later
// cudaMalloc fails or eats into what the pool left), or a process under a fixed memory
// budget that is checked when the library is loaded, not while it runs.  For them the partial sums and the
// arrival counters of the split-K reduction live in this file-scope array, which is part of
// the module image: every GPU that loads the library holds these bytes from load to exit,
// and nothing is ever allocated or freed by the entry point below.
constexpr size_t kStaticPartialBytes = 8ull << 20;    // fp32 partial tiles: splits * m * n * 4 <= 8 MiB
constexpr int kStaticTileCounters = 1024;             // one arrival counter per output tile
constexpr size_t kStaticCounterBytes = kStaticTileCounters * sizeof(int);
constexpr size_t kStaticTailBytes = kStaticCounterBytes + 256;   // counters + status word (padded)
static __device__ __align__(256) unsigned char g_gemm_static_scratch[kStaticPartialBytes + kStaticTailBytes];

namespace {

struct StaticDev {
  bool ready = false;
  unsigned char* base = nullptr;   // device address of g_gemm_static_scratch on this device
  int sm_count = 0;
};
StaticDev g_static_dev[64];
std::mutex g_static_mutex;

// One-time set-up per device, with that device current.  In host code the array's name is
// only a handle for the runtime; the address kernels can use comes from cudaGetSymbolAddress.
int static_scratch_setup(int device, StaticDev** out) {
  if (device < 0 || device >= 64) DTAS_FAIL(DTAS_EINVAL, "gemm (static scratch): device ordinal %d out of range", device);
  StaticDev* d = &g_static_dev[device];
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (!d->ready) {
    int major = 0, sms = 0;
    DTAS_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10)
      DTAS_FAIL(DTAS_EUNSUPPORTED, "device %d is not sm_100; this library only carries sm_100a code", device);
    DTAS_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    void* ptr = nullptr;
    DTAS_CUDA(cudaGetSymbolAddress(&ptr, g_gemm_static_scratch));
    if (ptr == nullptr) DTAS_FAIL(DTAS_ECUDA, "gemm (static scratch): cudaGetSymbolAddress returned a null address");
    d->base = static_cast<unsigned char*>(ptr);
    d->sm_count = sms;
    d->ready = true;
  }
  *out = d;
  return DTAS_OK;
}

// Tile width and split of a call on the built-in scratch.  The choice never reads the global override
// or the measured table (those tune dtas_gemm_nt), and it only considers the tiled kernel with a fixed
// split whose partial sums fit the array.  A split asked for by the caller is kept when it fits and
// refused otherwise; split_k = 0 always yields a plan that fits, down to one slice.
struct StaticPlan {
  int bn, splits, kb_per;
  int64_t m_tiles, n_tiles;
};
int static_plan(int64_t m, int64_t n, int64_t k, int split_k, StaticPlan* out) {
  PlanLimits lim;
  lim.use_overrides = false;
  lim.tiled_fixed_only = true;
  lim.ws_bytes = (int64_t)kStaticPartialBytes;
  lim.counters = kStaticTileCounters;
  const GemmPlan p = plan_gemm(m, n, k, 148, true, lim);
  const int num_kb = (int)((k + BK - 1) / BK);
  StaticPlan sp;
  sp.bn = p.bn;
  sp.m_tiles = (m + BM - 1) / BM;
  sp.n_tiles = (n + p.bn - 1) / p.bn;
  auto normalise = [&](int want) {
    sp.kb_per = (num_kb + want - 1) / want;
    sp.splits = (num_kb + sp.kb_per - 1) / sp.kb_per;     // no empty slice
  };
  auto fits = [&]() {
    return sp.splits == 1 || ((int64_t)sp.splits * m * (sp.n_tiles * sp.bn) * 4 <= (int64_t)kStaticPartialBytes &&
                              sp.m_tiles * sp.n_tiles <= kStaticTileCounters);
  };
  if (split_k > 0) {
    normalise(split_k > num_kb ? num_kb : split_k);
    if (!fits())
      DTAS_FAIL(DTAS_EINVAL,
                "gemm (static scratch): split_k=%d at m=%lld n=%lld needs %lld bytes of partial sums and %lld tile "
                "counters; the built-in scratch holds %lld bytes and %d counters (use dtas_gemm_nt, a smaller split, "
                "or split_k=0)",
                sp.splits, (long long)m, (long long)n, (long long)((int64_t)sp.splits * m * (sp.n_tiles * sp.bn) * 4),
                (long long)(sp.m_tiles * sp.n_tiles), (long long)kStaticPartialBytes, kStaticTileCounters);
  } else {
    for (int want = p.splits; want >= 1; --want) {          // the planner's split, lowered until it fits
      normalise(want);
      if (fits()) break;
    }
  }
  if (sp.m_tiles * sp.n_tiles * sp.splits > 0x7fffffffLL) DTAS_FAIL(DTAS_EINVAL, "gemm (static scratch): too many tiles");
  *out = sp;
  return DTAS_OK;
}

int static_args_check(const void* x, const void* w, int64_t m, int64_t n, int64_t k, int split_k, int dtype) {
  if (m <= 0) DTAS_FAIL(DTAS_EINVAL, "gemm (static scratch): dynamic dim m must be > 0, got %lld", (long long)m);
  if (n <= 0 || k <= 0) DTAS_FAIL(DTAS_EINVAL, "gemm (static scratch): n and k must be > 0");
  if (dtype != DTAS_F16) DTAS_FAIL(DTAS_EUNSUPPORTED, "gemm (static scratch): only fp16 is implemented");
  if (split_k < 0 || split_k > 64) DTAS_FAIL(DTAS_EINVAL, "gemm (static scratch): split_k must be in [0, 64]");
  if (m > 0x3fffffffLL || n > 0x3fffffffLL || k > 0x3fffffffLL) DTAS_FAIL(DTAS_EINVAL, "gemm (static scratch): dimension too large");
  if (!gemm_tma_ok(x, w, k))
    DTAS_FAIL(DTAS_EALIGN, "gemm (static scratch): x and w must be 16-byte aligned and k a multiple of 8");
  return DTAS_OK;
}

}  // namespace

// Status word of the built-in scratch on `device`: read, and cleared when set.  0 when the entry point
// was never called on that device.  Synchronises the device.
int static_scratch_poll(int device, int* code) {
  *code = 0;
  if (device < 0 || device >= 64) return DTAS_OK;
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_dev[device].ready) return DTAS_OK;
    base = g_static_dev[device].base;
  }
  DeviceGuard g;
  int rc = g.enter(device);
  if (rc) return rc;
  int* word = reinterpret_cast<int*>(base + kStaticPartialBytes + kStaticCounterBytes);
  DTAS_CUDA(cudaDeviceSynchronize());
  DTAS_CUDA(cudaMemcpy(code, word, sizeof(int), cudaMemcpyDeviceToHost));
  if (*code != 0) DTAS_CUDA(cudaMemset(word, 0, sizeof(int)));
  return DTAS_OK;
}

}  // namespace dtas

extern "C" int dtas_gemm_nt_static_scratch_plan(int64_t m, int64_t n, int64_t k, int split_k, int* tile_n,
                                                int* splits) {
  using namespace dtas;
  int rc = static_args_check(nullptr, nullptr, m, n, k, split_k, DTAS_F16);
  if (rc != DTAS_OK) return rc;
  StaticPlan sp;
  if ((rc = static_plan(m, n, k, split_k, &sp)) != DTAS_OK) return rc;
  if (tile_n != nullptr) *tile_n = sp.bn;
  if (splits != nullptr) *splits = sp.splits;
  return DTAS_OK;
}

extern "C" int dtas_gemm_nt_static_scratch(const void* x, const void* w, const void* bias, void* y, int64_t m,
                                           int64_t n, int64_t k, int64_t ldy, int split_k, int dtype,
                                           int device, void* stream, void* status_word) {
  using namespace dtas;
  if (x == nullptr || w == nullptr || y == nullptr) DTAS_FAIL(DTAS_EINVAL, "gemm (static scratch): NULL operand");
  int rc = static_args_check(x, w, m, n, k, split_k, dtype);
  if (rc != DTAS_OK) return rc;
  if (ldy < n) DTAS_FAIL(DTAS_EINVAL, "gemm (static scratch): ldy (%lld) must be >= n (%lld)", (long long)ldy, (long long)n);
  StaticPlan sp;
  if ((rc = static_plan(m, n, k, split_k, &sp)) != DTAS_OK) return rc;

  DeviceGuard guard;
  if ((rc = guard.enter(device)) != DTAS_OK) return rc;
  StaticDev* sd = nullptr;
  if ((rc = static_scratch_setup(device, &sd)) != DTAS_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left: the arrival counters must start at zero.  The
  // status word behind them is left alone: it holds a code until dtas_poll_status has reported it.
  if (sp.splits > 1) DTAS_CUDA(cudaMemsetAsync(sd->base + kStaticPartialBytes, 0, kStaticCounterBytes, st));

  CUtensorMap tx, tw;
  if ((rc = make_tmap(&tx, x, m, k, BM)) != DTAS_OK) return rc;
  if ((rc = make_tmap(&tw, w, n, k, sp.bn)) != DTAS_OK) return rc;
  GemmArgs a;
  a.y = y;
  a.epi.bias = (const __half*)bias;
  a.ws = reinterpret_cast<float*>(sd->base);
  a.counters = reinterpret_cast<int*>(sd->base + kStaticPartialBytes);
  a.status = status_word != nullptr ? static_cast<int*>(status_word)
                                    : reinterpret_cast<int*>(sd->base + kStaticPartialBytes + kStaticCounterBytes);
  a.ldy = ldy;
  a.m = (int)m;
  a.n = (int)n;
  a.k = (int)k;
  a.m_tiles = (int)sp.m_tiles;
  a.n_tiles = (int)sp.n_tiles;
  a.splits = sp.splits;
  a.slots_cap = sp.splits;
  a.kb_per_split = sp.kb_per;
  a.num_kb = (int)((k + BK - 1) / BK);
  a.vec_store = finish_epilogue(a.epi, y, ldy);
  switch (sp.bn) {
    case 256: return launch_tc<256>(tx, tw, a, sd->sm_count, st);
    case 128: return launch_tc<128>(tx, tw, a, sd->sm_count, st);
    default: return launch_tc<64>(tx, tw, a, sd->sm_count, st);
  }
}

// ---------------------------------------------------------------------------------------
// Self-test of the bounded waits.  One warp initialises an mbarrier that nothing ever arrives on and
// waits for it with the limit given by the caller; when the limit runs out the wait records its code
// in the device status word and the kernel returns normally, exactly as a stuck role of a GEMM
// kernel would.  Nothing traps or spins without bound; dtas_poll_status then reports DTAS_ETIMEOUT.
// ---------------------------------------------------------------------------------------
namespace dtas {
namespace {
constexpr int ERR_SELFTEST = 0x1ff;
__global__ void __launch_bounds__(32) wait_selftest_kernel(int* status, uint64_t limit_ns) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x == 0) (void)mbar_wait_slow(b, 0u, status, ERR_SELFTEST, limit_ns);
  __syncwarp();
}
}  // namespace
}  // namespace dtas

extern "C" int dtas_selftest_wait_timeout(int device, void* stream, int64_t limit_ns) {
  using namespace dtas;
  if (limit_ns < 1000 || limit_ns > 100000000)
    DTAS_FAIL(DTAS_EINVAL, "selftest: the wait limit must be between 1 us and 100 ms, got %lld ns", (long long)limit_ns);
  DeviceGuard guard;
  int rc = guard.enter(device);
  if (rc != DTAS_OK) return rc;
  DeviceCtx* ctx = nullptr;
  if ((rc = get_ctx(device, &ctx)) != DTAS_OK) return rc;
  launch_kernel(wait_selftest_kernel, 1, 32, 0, static_cast<cudaStream_t>(stream), ctx->status, (uint64_t)limit_ns);
  return after_launch("wait_selftest_kernel");
}
