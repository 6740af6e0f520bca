/*
 * dtas_b200 — C ABI of the sm_100a kernel library that stands in for the
 * packed functions DTAS generates with TVM.
 *
 * In the reference every tuned PrimFunc becomes one generated host function
 *   extern "C" int32_t <name>(void* args, int32_t* arg_type_ids, int32_t num_args,
 *                             void* out_ret_value, int32_t* out_ret_tcode, void* resource_handle)
 * (experiment/dtas_tuned/elementwise/cast/top10_256/host.cc:38-42) that unpacks
 * DLTensor arguments, reads the symbolic dim from the tensor shape, looks up
 * call_table[index_table[min(n/256, last)]] and launches one kernel of the cubin
 * (host.cc:92-131; generator: python/dtas/codegen/code_gen.py:242-405).
 *
 * Here the same thing is a plain C entry point per operator class: raw device
 * pointers, the runtime row count m, the static dims, a dtype code, the device
 * ordinal and the CUDA stream.  Calling convention is destination-passing like
 * the reference (inputs first, pre-allocated output last among the pointers).
 *
 * Every entry point
 *   - returns DTAS_OK (0) or a positive DTAS_E* code; the message is available
 *     from dtas_last_error() (thread-local), like TVM's last-error string;
 *   - rejects m <= 0 (the reference asserts dynamic dims > 0,
 *     python/dtas/IRpass/add_assert.py:36-37);
 *   - launches on the given stream of the given device and restores the
 *     caller's current device; never synchronises;
 *   - allocates nothing per call.  The split-K GEMM keeps one workspace per
 *     device that is created on the first call that needs it.
 */
#ifndef DTAS_B200_H_
#define DTAS_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
#define DTAS_OK            0
#define DTAS_EINVAL        1  /* bad argument: null pointer, m <= 0, bad dim, unknown dtype */
#define DTAS_EALIGN        2  /* pointer / leading dimension alignment the kernel cannot honour */
#define DTAS_ECUDA         3  /* a CUDA runtime / driver call failed                       */
#define DTAS_ETIMEOUT      4  /* a bounded device-side wait gave up (reported by dtas_poll_status) */
#define DTAS_EUNSUPPORTED  5  /* dtype / shape combination without a kernel                 */

/* ---- dtype codes ------------------------------------------------------- */
#define DTAS_F16  0
#define DTAS_F32  1
#define DTAS_I8   2

/* ---- elementwise class --------------------------------------------------
 * Replaces the generated `cast`, `add`, `copy` packed functions
 * (tuning_test/tune_cast.py:10-21, tune_ele_add.py:10-22, tune_ele_copy.py:10-21;
 *  kernels experiment/dtas_tuned/elementwise/{cast,add,copy}/...).
 * Tensors are row-major contiguous [m, n_cols] (the reference's [1, n, H]).   */
int dtas_cast(const void* a, void* out, int64_t m, int64_t n_cols,
              int src_dtype, int dst_dtype, int device, void* stream);
int dtas_add(const void* a, const void* b, void* out, int64_t m, int64_t n_cols,
             int dtype, int device, void* stream);
int dtas_copy(const void* a, void* out, int64_t m, int64_t n_cols,
              int dtype, int device, void* stream);

/* ---- row-reduction class -------------------------------------------------
 * Replaces the "general reduction" packed functions
 * (fused_layer_norm_cast / fused_softmax_cast,
 *  experiment/dtas_tuned/general_reduction/{layernorm,softmax}/profile_dlight.py;
 *  scheduler python/dtas/schedule/tir_reduction.py:36-105).
 * x is [m, n_cols] of in_dtype (DTAS_F16 or DTAS_F32); the result is fp16;
 * all arithmetic is fp32.
 *   rms_norm  : y = x * rsqrt(mean(x^2) + eps) * weight      (weight fp16 [n_cols])
 *   softmax   : y = exp(x - max) / sum(exp(x - max)) over the last dim
 *   layer_norm: y = (x - mean) * rsqrt(E[x^2] - mean^2 + eps) * gamma + beta
 *               (gamma, beta fp32 [n_cols], as in the reference workload)      */
int dtas_rms_norm(const void* x, const void* weight, void* y, int64_t m, int64_t n_cols,
                  float eps, int in_dtype, int device, void* stream);
int dtas_softmax(const void* x, void* y, int64_t m, int64_t n_cols,
                 int in_dtype, int device, void* stream);
int dtas_layer_norm(const void* x, const void* gamma, const void* beta, void* y,
                    int64_t m, int64_t n_cols, float eps, int in_dtype, int device, void* stream);

/* ---- GEMV ----------------------------------------------------------------
 * y[n] = sum_k W[n,k] * x[k] (+ bias[n]); fp16 in/out, fp32 accumulation.
 * Replaces the NT_matmul(+add) GEMV packed function
 * (experiment/testIR/GEMV/m1n2560k10240/dlight_gemv.py:8-27,
 *  python/dtas/schedule/tir_gemv.py:33-249).  bias may be NULL.               */
int dtas_gemv(const void* x, const void* w, const void* bias, void* y,
              int64_t n, int64_t k, int dtype, int device, void* stream);

/* ---- GEMM ----------------------------------------------------------------
 * Y[m,n] = X[m,k] * W[n,k]^T (+ bias[n]); fp16 in/out, fp32 accumulation on
 * the tcgen05 tensor cores.  Replaces fused_NT_matmul*_add*
 * (experiment/testIR/GEMM/dlight.py:30-50, python/dtas/schedule/tir_wmma.py:20-222).
 * X and W are row-major contiguous; Y has row stride ldy elements (ldy >= n), so
 * a column-sharded rank can write its slab straight into a wider buffer.
 * bias may be NULL.                                                            */
int dtas_gemm_nt(const void* x, const void* w, const void* bias, void* y,
                 int64_t m, int64_t n, int64_t k, int64_t ldy,
                 int dtype, int device, void* stream);

/* ---- GEMM / GEMV with a fused tail -----------------------------------------
 * The forms the reference's model workloads take after operator fusion
 * (experiment/ModelIR/dolly-v2-3b-q0f16/before_dl.py):
 *   fused_NT_matmul_add                   (:552)  y = x.W^T + bias
 *   fused_NT_matmul3_add2_gelu            (:248)  y = gelu(x.W^T + bias)
 *   fused_NT_matmul2_add1_add3_add3       (:163)  y = (res1 + (x.W^T + bias)) + res2
 *   fused_NT_matmul2_add1_add3_add3_cast  (:202)  the same, written as fp32
 * and their decode-time GEMV forms (:96, :408, :442, :483).  One call computes
 *   y = act(x.W^T + bias) + res1 + res2
 * on the fp32 accumulator, rounds to fp16 once, and stores fp16 or (out_dtype DTAS_F32) that
 * fp16 value widened to fp32.  bias [n], res1 and res2 [m, n] (row stride ldr elements; [n] for
 * the GEMV) are fp16 and optional (NULL); res2 needs res1.  act is DTAS_ACT_NONE or
 * DTAS_ACT_GELU = t * (0.5 + 0.5 * erf(t / sqrt(2))), the erf form of the reference's workload.
 * The reference rounds every intermediate to fp16; results agree within the GEMM tolerance.   */
#define DTAS_ACT_NONE 0
#define DTAS_ACT_GELU 1
int dtas_gemm_nt_fused(const void* x, const void* w, const void* bias, const void* res1, const void* res2,
                       void* y, int64_t m, int64_t n, int64_t k, int64_t ldy, int64_t ldr, int act,
                       int out_dtype, int dtype, int device, void* stream);
int dtas_gemv_fused(const void* x, const void* w, const void* bias, const void* res1, const void* res2,
                    void* y, int64_t n, int64_t k, int act, int out_dtype, int dtype, int device, void* stream);

/* ---- GEMM without any allocation ------------------------------------------
 * No counterpart in the reference.  Same operation and operands as dtas_gemm_nt, for callers
 * that must not create device memory when they call: runtimes that gave the whole device to
 * their own pool at start-up (a later cudaMalloc fails or eats into what the pool left), and
 * processes under a fixed memory budget that is checked when the library is loaded, not while
 * it runs.  dtas_gemm_nt keeps its split-K partial sums in a
 * workspace it cudaMallocs on first use; this entry point keeps them in an array that is part
 * of the library image (8 MiB of fp32 partials + 1024 tile counters per GPU that loads the
 * library, held until the process exits) and calls no allocating routine at all.
 *   split_k     : K slices per output tile.  0 lets the library choose: it starts from the split its
 *                 cost model prefers and lowers it until the partial sums fit, so split_k = 0 is never
 *                 refused for size.  A split the caller asks for is refused with DTAS_EINVAL when
 *                 split_k * m * n * 4 bytes (n rounded up to the tile width) exceed 8 MiB or the output
 *                 has more than 1024 tiles; with one slice no scratch is used and any size is accepted.
 *                 x and w must be 16-byte aligned and k a multiple of 8 (DTAS_EALIGN otherwise).
 *                 The tile width and split come from the shape alone: dtas_gemm_set_override and
 *                 dtas_gemm_table_set, which tune dtas_gemm_nt, do not apply here.
 *   status_word : optional device int32 that receives a non-zero code if a bounded wait inside
 *                 the kernel gives up; NULL keeps the code in a word of the library's own array,
 *                 which dtas_poll_status reads and clears like the status word of the other calls.
 * The first call on a device looks up the array's device address; make that call before any
 * stream capture.  Every call on a device uses the same array: the call clears the counters it
 * needs on the given stream, and two calls that overlap on the GPU (different streams) race.
 * dtas_gemm_nt_static_scratch_plan reports the tile width and split a call of that shape would
 * use (same argument checks, no device needed); either output pointer may be NULL.            */
int dtas_gemm_nt_static_scratch(const void* x, const void* w, const void* bias, void* y,
                                int64_t m, int64_t n, int64_t k, int64_t ldy, int split_k,
                                int dtype, int device, void* stream, void* status_word);
int dtas_gemm_nt_static_scratch_plan(int64_t m, int64_t n, int64_t k, int split_k, int* tile_n, int* splits);

/* ---- dispatch introspection ---------------------------------------------
 * dtas_bucket_of: index of the m-bucket the op dispatches on, the counterpart of
 * the generated `index = (n/256) > L ? L : n/256` statement
 * (python/dtas/engine/tuner.py:156-209) with the off-by-one at multiples of the
 * width removed: bucket = min((m-1)/256, last).  op is one of "cast", "add",
 * "copy", "rms_norm", "softmax", "layer_norm", "gemv", "gemm".  Returns -1 for
 * an unknown op or m <= 0.
 * dtas_variant_of: writes the name of the kernel variant that the given call
 * shape would launch (e.g. "gemm_tc_bn256_s4_splitk1") into buf; returns DTAS_OK. */
int dtas_bucket_of(const char* op, int64_t m);
int dtas_bucket_count(const char* op);
int dtas_variant_of(const char* op, int64_t m, int64_t n, int64_t k, int device,
                    char* buf, int buf_len);

/* Overrides the GEMM dispatch for testing and offline re-tuning: block-tile
 * width bn in {64,128,256} (0 = automatic; 512 = the two-CTA kernel with 256 x 256 tiles dealt out whole,
 * 513 = the same kernel with stream-K work distribution over the CTA pairs;
 * 1024 = the swapped-operand kernel, which applies to m <= 256; 2048 = the same kernel with
 * stream-K work distribution; 4096 + 64/128/256 = single-CTA tiles of that width with stream-K;
 * 8192 + 64/128 = tiles of that width with K cut in two inside a two-CTA cluster, the second half
 * handed over through shared memory; 16384 + 2/3/4 = the swapped-operand kernel (m <= 64) with K cut
 * in that many slices inside a cluster; split_k is ignored by the stream-K and cluster codes) and
 * split-K factor (0 = automatic). */
int dtas_gemm_set_override(int bn, int split_k);

/* Measured dispatch table for the GEMM: for weight shape (n, k) and row counts m_lo..m_hi use
 * tile code bn (as in dtas_gemm_set_override) and split_k.  The counterpart of the per-range
 * best configs the reference's search records (python/dtas/engine/tuner.py:103-133,211-299);
 * Engine.tune_module(..., search=True) fills it from on-device timings.  Calls whose shape has
 * no entry are planned by the built-in cost model.  dtas_gemm_set_override wins over the table. */
int dtas_gemm_table_set(int64_t n, int64_t k, int64_t m_lo, int64_t m_hi, int bn, int split_k);
int dtas_gemm_table_clear(void);

/* Same for the elementwise class: vectors in flight per thread (0 = per-bucket default, else
 * 1, 2, 4 or 8), grid cap in CTAs per SM (0 = default, < 0 = one tile per CTA without a cap)
 * and streaming cache hints (-1 = default, 0 = off, 1 = on).                                 */
int dtas_ew_set_override(int unroll, int ctas_per_sm, int stream_hints);

/* Row reductions: threads that own one row (0 = per-bucket default, else a power of two in
 * [32, 1024]; raised automatically when a row would not fit the register budget).
 * GEMV: warps per output row (0 = automatic, else 1, 2, 4, 8; 16 = the streaming kernel, one
 * persistent CTA per SM fed by bulk copies, wherever a row fits its ring) and 16-byte loads in
 * flight per lane (0 = automatic, else 4 or 8).                                               */
int dtas_row_set_override(int threads_per_row);
int dtas_gemv_set_override(int warps_per_row, int unroll);

/* Launch mode of every kernel of the library.  No counterpart in the reference.
 *   1 (default): programmatic dependent launch - a kernel may be scheduled, and run the set-up it
 *      does before touching global memory, while the kernel before it on the stream drains; it
 *      waits for that kernel's results before its first global access, so callers see plain
 *      stream order;
 *   0: plain launches.
 * The initial mode comes from the environment variable DTAS_B200_PDL (0 or 1).  Returns the
 * previous mode, or -1 for any other value.                                                  */
int dtas_set_pdl(int mode);

/* ---- multi-GPU: pushing a column slab to the other ranks -------------------
 * No counterpart in the reference, which opens one device (python/dtas/arch/RTX3090.py:6-7).
 * With Y's columns sharded over g GPUs, dtas_peer_push copies `bytes` bytes at `src` (this rank's
 * slab, or a block of its rows) to each of the n_dsts addresses in `dsts`: device pointers, valid
 * in this process, to the same place in the other ranks' gather buffers (peer memory mapped
 * through CUDA IPC or a symmetric-memory allocation).  `dsts` is a host array, read during the
 * call.  One launch on `stream`: it reads the source once and stores over NVLink; it waits on no
 * other rank and signals none, so the caller runs a barrier across ranks behind the last push
 * before anyone reads a gathered buffer.  src and every destination must be 16-byte aligned
 * (DTAS_EALIGN), 1 <= n_dsts <= DTAS_MAX_PEERS, bytes >= 1.  This replaces the all-gather a
 * caller would run behind dtas_gemm_nt / dtas_gemv; Python: dtas_b200.dist.PeerGatherBuffer.
 * The environment variable DTAS_B200_PUSH_CTAS limits its grid (default: one CTA per SM).     */
#define DTAS_MAX_PEERS 7
int dtas_peer_push(const void* src, void* const* dsts, int n_dsts, int64_t bytes, int device, void* stream);

/* The same gather fused into the GEMM (no counterpart in the reference).  dtas_gemm_nt_scatter computes
 * Y = X.W^T (+ bias) exactly like dtas_gemm_nt and stores every finished 16-byte vector of Y a second
 * time into each of the n_peers buffers in `peer_ys` (host array of device pointers, read during the
 * call): buffers with Y's layout and row stride ldy - with Y's columns sharded over g GPUs, the place of
 * this rank's slab in the other ranks' gather buffers, mapped into this process.  The stores leave from
 * the epilogue of the two-CTA tcgen05 kernel, tile by tile, with plain st.global over NVLink, so the
 * transfer is spread over the whole GEMM and over every SM instead of following the kernel; nothing
 * waits on another rank or signals one, so the caller still runs one barrier across ranks before a
 * gathered buffer is read.  Needs m >= 129, 16-byte aligned x and w and k a multiple of 8
 * (DTAS_EUNSUPPORTED otherwise: use dtas_gemm_nt and dtas_peer_push); peer buffers that are not 16-byte
 * aligned are written with scalar stores.  1 <= n_peers <= DTAS_MAX_PEERS.                          */
int dtas_gemm_nt_scatter(const void* x, const void* w, const void* bias, void* y, void* const* peer_ys,
                         int n_peers, int64_t m, int64_t n, int64_t k, int64_t ldy, int dtype, int device,
                         void* stream);

/* dtas_gemm_nt_scatter with the fan-out done by the NVLink switch (no counterpart in the reference).
 * `y_multicast` is the address of Y's slab in a multicast mapping that covers this GPU's gather buffer and
 * every peer's at the same offset (CUDA multicast object / NVLink SHARP; in PyTorch the multicast_ptr of
 * a symmetric-memory allocation plus the slab's offset).  Whole 32-row blocks of the output then leave as
 * one multimem.st per 16-byte vector, which the switch stores into every buffer of the mapping - this
 * GPU's own included - instead of one local and n_peers peer stores; ragged edges still go through
 * `y` and `peer_ys`, which must be given as for dtas_gemm_nt_scatter.  y_multicast == NULL is
 * dtas_gemm_nt_scatter.  y, y_multicast and ldy * 2 bytes must be multiples of 16 (DTAS_EALIGN).  The
 * caller's barrier across ranks before the gathered buffer is read stands.                              */
int dtas_gemm_nt_scatter_multicast(const void* x, const void* w, const void* bias, void* y, void* const* peer_ys,
                                   int n_peers, void* y_multicast, int64_t m, int64_t n, int64_t k, int64_t ldy,
                                   int dtype, int device, void* stream);

/* ---- bookkeeping ---------------------------------------------------------
 * dtas_last_error : message of the last failing call on this thread ("" if none).
 * dtas_launch_count: kernels launched by this library since load (all threads).
 * dtas_poll_status : reads the device-side status word of `device` (written by a
 *                    kernel whose bounded wait gave up); synchronises the device.
 *                    Returns DTAS_OK or DTAS_ETIMEOUT, clears the word and re-arms the
 *                    split-K arrival counters a kernel that gave up may have left behind.
 * dtas_selftest_wait_timeout: launches one warp that waits, with a limit of limit_ns
 *                    (1 us .. 100 ms), on a barrier nothing arrives on, so that the bounded-wait
 *                    path can be exercised: the kernel returns normally once the limit has run
 *                    out and the next dtas_poll_status reports DTAS_ETIMEOUT.  No counterpart
 *                    in the reference.
 * dtas_shutdown    : frees per-device workspaces.
 * dtas_version     : "dtas_b200 <semver> sm_100a".                              */
const char* dtas_last_error(void);
int64_t dtas_launch_count(void);
int dtas_poll_status(int device);
int dtas_selftest_wait_timeout(int device, void* stream, int64_t limit_ns);
int dtas_shutdown(void);
const char* dtas_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DTAS_B200_H_ */
