/*
 * TEST INFRASTRUCTURE - not part of the product.  Only tests/, __graft_entry__.smoke()
 * and the cpu_baseline / --impl reference legs of bench.py may build, load or call this.
 *
 * CPU restatement, in plain C, of the arithmetic of the DTAS workload PrimFuncs.  DTAS
 * itself contains no arithmetic: its workloads are TVMScript PrimFuncs whose semantics are
 * those of Apache TVM (not vendored, not pinned by the reference).  Each function below
 * follows the loop nest and expression order of one PrimFunc, exactly as TVM's C backend
 * emits it (sequential loops, fp32 temporaries, `1.0f / sqrtf(x)` for T.rsqrt, `expf` for
 * T.exp, C casts for T.Cast), so that it can be pinned bit-for-bit against a TVM build of
 * the same PrimFunc (tests/golden/make_golden.py does that; tests/test_oracle.py checks it).
 *
 * Parity status: the reference ships no golden vectors or known-answer tests for this path,
 * so the oracle is pinned against outputs of the reference's workload definitions built by
 * the TVM available in this image (tilelang's TVM 0.23.dev0 fork, target "c", g++ -O2),
 * committed as tests/golden/*.npz.
 *
 * Rows are independent in every PrimFunc; the outer row loop carries an OpenMP pragma so the
 * CPU baseline can use all host cores (oracle_set_threads).  Arithmetic inside a row is
 * strictly sequential, so results do not depend on the thread count.
 *
 * Build: gcc -O2 -mf16c -fopenmp -shared -fPIC (-mf16c only makes the exact fp16<->fp32
 * conversions use hardware; no -ffast-math, no -mfma: keeps FMA contraction
 * off, as in TVM's own g++ -O2 build).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 f16;

void oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* tuning_test/tune_cast.py:10-21 (`compute[...] = T.Cast(dtype, A[...])`), fp32 -> fp16:
 * a C cast, i.e. round-to-nearest-even. */
void oracle_cast_f32_f16(const float* a, f16* out, int64_t m, int64_t h) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r)
    for (int64_t c = 0; c < h; ++c) out[r * h + c] = (f16)a[r * h + c];
}

/* tuning_test/tune_cast.py:10-21 as written in the reference: fp16 -> fp32 (exact). */
void oracle_cast_f16_f32(const f16* a, float* out, int64_t m, int64_t h) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r)
    for (int64_t c = 0; c < h; ++c) out[r * h + c] = (float)a[r * h + c];
}

/* tuning_test/tune_ele_add.py:10-22 (`T_add = A + B`) for fp16: TVM's C backend emits
 * `half + half`; with half = _Float16 that is an fp32 add rounded once to fp16. */
void oracle_add_f16(const f16* a, const f16* b, f16* out, int64_t m, int64_t h) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r)
    for (int64_t c = 0; c < h; ++c) out[r * h + c] = (f16)((float)a[r * h + c] + (float)b[r * h + c]);
}

void oracle_add_f32(const float* a, const float* b, float* out, int64_t m, int64_t h) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r)
    for (int64_t c = 0; c < h; ++c) out[r * h + c] = a[r * h + c] + b[r * h + c];
}

/* int8 as in tuning_test/tune_ele_add.py:2,13-16: two's-complement wrap-around. */
void oracle_add_i8(const int8_t* a, const int8_t* b, int8_t* out, int64_t m, int64_t h) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r)
    for (int64_t c = 0; c < h; ++c)
      out[r * h + c] = (int8_t)(uint8_t)((uint8_t)a[r * h + c] + (uint8_t)b[r * h + c]);
}

/* tuning_test/tune_ele_copy.py:10-21 (`B = A`), any dtype: bytes. */
void oracle_copy(const void* a, void* out, int64_t m, int64_t h, int64_t elem_size) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r)
    memcpy((char*)out + r * h * elem_size, (const char*)a + r * h * elem_size, (size_t)(h * elem_size));
}

/* RMSNorm has no counterpart in the reference; the PrimFunc (dtas_b200/workloads/tir_defs.py,
 * rms_norm) is modelled on the block structure of fused_layer_norm_cast
 * (experiment/dtas_tuned/general_reduction/layernorm/profile_dlight.py:8-40): one "SSR"
 * reduction block accumulating x*x in fp32 in k order, one injective block
 *   y = (f16)( ((float)x * (1/sqrtf(ss * (1/H) + eps))) * (float)w ). */
void oracle_rms_norm_f16(const f16* x, const f16* w, f16* y, int64_t m, int64_t h, float eps) {
  const float inv_h = (float)(1.0 / (double)h);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r) {
    float ss = 0.0f;
    for (int64_t k = 0; k < h; ++k) ss = ss + ((float)x[r * h + k]) * ((float)x[r * h + k]);
    for (int64_t c = 0; c < h; ++c)
      y[r * h + c] = (f16)((((float)x[r * h + c]) * (1.0f / sqrtf((ss * inv_h) + eps))) * ((float)w[c]));
  }
}

/* experiment/dtas_tuned/general_reduction/softmax/profile_dlight.py:8-52
 * (T_softmax_maxelem, T_softmax_exp, T_softmax_expsum, T_softmax_norm, compute):
 * max over the row from -FLT_MAX, exp(x - max), sum in k order, divide, cast to fp16.
 * `in_f16` selects the fp16-input variant (a T.Cast("float32", .) on every read). */
static void softmax_row(const float* x, f16* y, int64_t h, float* tmp) {
  float mx = -3.4028234663852886e+38f;
  for (int64_t k = 0; k < h; ++k) mx = mx > x[k] ? mx : x[k];
  for (int64_t k = 0; k < h; ++k) tmp[k] = expf(x[k] - mx);
  float sum = 0.0f;
  for (int64_t k = 0; k < h; ++k) sum = sum + tmp[k];
  for (int64_t k = 0; k < h; ++k) y[k] = (f16)(tmp[k] / sum);
}

void oracle_softmax(const void* x, f16* y, int64_t m, int64_t h, int in_f16, float* scratch /* 2*h floats per thread */) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r) {
#ifdef _OPENMP
    float* tmp = scratch + (int64_t)omp_get_thread_num() * 2 * h;
#else
    float* tmp = scratch;
#endif
    const float* xr;
    if (in_f16) {
      float* conv = tmp + h;
      const f16* src = (const f16*)x + r * h;
      for (int64_t k = 0; k < h; ++k) conv[k] = (float)src[k];
      xr = conv;
    } else {
      xr = (const float*)x + r * h;
    }
    softmax_row(xr, y + r * h, h, tmp);
  }
}

/* experiment/dtas_tuned/general_reduction/layernorm/profile_dlight.py:8-40
 * (A_red_temp: sum and sum of squares in k order; T_layer_norm:
 *  (x - s1*c) * rsqrt(s2*c - (s1*c)*(s1*c) + eps) * gamma + beta; compute: cast to fp16),
 * with c = 1/H as an fp32 constant.  fp32 or fp16 input, fp32 gamma/beta. */
void oracle_layer_norm(const void* x, const float* gamma, const float* beta, f16* y, int64_t m, int64_t h,
                       float eps, int in_f16) {
  const float c = (float)(1.0 / (double)h);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < m; ++r) {
    float s1 = 0.0f, s2 = 0.0f;
    for (int64_t k = 0; k < h; ++k) {
      float v = in_f16 ? (float)((const f16*)x)[r * h + k] : ((const float*)x)[r * h + k];
      s1 = s1 + v;
      s2 = s2 + v * v;
    }
    for (int64_t k = 0; k < h; ++k) {
      float v = in_f16 ? (float)((const f16*)x)[r * h + k] : ((const float*)x)[r * h + k];
      float o = (((v - (s1 * c)) * (1.0f / sqrtf(((s2 * c) - ((s1 * c) * (s1 * c))) + eps))) * gamma[k]) + beta[k];
      y[r * h + k] = (f16)o;
    }
  }
}

/* GEMM: experiment/testIR/GEMM/dlight.py:30-50 (block "NT_matmul":
 * acc[i, j] += X[i, k] * W[j, k] in k order) with the accumulator widened to fp32 and the
 * result cast to fp16 once, which is the configuration the build's parity rule names
 * ("fp32-accumulated reference").  Optional bias is added in fp32 before the cast.
 * Rows [row0, row1) and columns [col0, col1) are computed, so large shapes can be sampled. */
void oracle_gemm_nt_f16(const f16* x, const f16* w, const f16* bias, f16* y, int64_t m, int64_t n, int64_t k,
                        int64_t ldy, int64_t row0, int64_t row1, int64_t col0, int64_t col1) {
  (void)m;
  (void)n;
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t i = row0; i < row1; ++i) {
    for (int64_t j = col0; j < col1; ++j) {
      float acc = 0.0f;
      const f16* xr = x + i * k;
      const f16* wr = w + j * k;
      for (int64_t kk = 0; kk < k; ++kk) acc = acc + ((float)xr[kk]) * ((float)wr[kk]);
      if (bias) acc = acc + (float)bias[j];
      y[i * ldy + j] = (f16)acc;
    }
  }
}

/* GEMV: experiment/testIR/GEMV/m1n2560k10240/dlight_gemv.py:8-27 with an fp32
 * accumulator: y[j] = (f16)(sum_k x[k] * W[j, k] (+ bias[j])). */
void oracle_gemv_f16(const f16* x, const f16* w, const f16* bias, f16* y, int64_t n, int64_t k) {
#pragma omp parallel for schedule(static)
  for (int64_t j = 0; j < n; ++j) {
    float acc = 0.0f;
    const f16* wr = w + j * k;
    for (int64_t kk = 0; kk < k; ++kk) acc = acc + ((float)x[kk]) * ((float)wr[kk]);
    if (bias) acc = acc + (float)bias[j];
    y[j] = (f16)acc;
  }
}

/* The same two PrimFuncs exactly as the reference's files state them: the accumulator is an fp16
 * buffer (experiment/testIR/GEMM/dlight.py:35-44, `var_NT_matmul_intermediate` is "float16" and the
 * update is `acc = acc + x * w`; experiment/testIR/GEMV/m1n2560k10240/dlight_gemv.py:13-22), and the
 * bias is added by a second block that rounds to fp16 again (dlight.py:45-50).  TVM's C backend emits
 * `half + half * half`; with half = _Float16 on x86 that is evaluated in fp32 and rounded once per
 * update (the product of two fp16 numbers is exact in fp32), which the TVM build of the reference text
 * confirms bit for bit (tests/golden/make_ref_golden.py).  Rows [row0, row1) are computed. */
void oracle_gemm_nt_f16acc(const f16* x, const f16* w, const f16* bias, f16* y, int64_t n, int64_t k,
                           int64_t row0, int64_t row1) {
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t i = row0; i < row1; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      f16 acc = (f16)0.0f;
      const f16* xr = x + i * k;
      const f16* wr = w + j * k;
      for (int64_t kk = 0; kk < k; ++kk) acc = (f16)((float)acc + ((float)xr[kk]) * ((float)wr[kk]));
      if (bias) acc = (f16)((float)acc + (float)bias[j]);
      y[i * n + j] = acc;
    }
  }
}

/* Fused matmul tails of the model workloads, stage by stage as the reference's TIR stores them
 * (experiment/ModelIR/dolly-v2-3b-q0f16/before_dl.py:163-200 add/add/add, :202-246 + cast,
 * :248-318 add + gelu; decode-time forms :96-114, :408-550): every stage after the matmul is a
 * separate block writing an fp16 buffer, so every stage rounds to fp16.
 *   T_add        t = mm + bias
 *   T_multiply   u = t * (half)0.70710678118654757      gelu, erf form
 *   compute      c = (float)u;  compute_1  e = erff(c);  compute_2  h = (half)e
 *   T_multiply_1 h = h * (half)0.5;  T_add_1  s = (half)0.5 + h;  T_multiply_2  t = t * s
 *   T_add_1      t = res1 + t;   T_add_2  t = t + res2
 *   compute      y = (float)t                            the _cast variants
 * The matmul itself is the fp32-accumulated one above, rounded to fp16 once. */
static inline f16 fused_tail(f16 mm, const f16* bias, const f16* res1, const f16* res2, int64_t j, int64_t roff,
                             int act) {
  f16 t = mm;
  if (bias) t = (f16)((float)t + (float)bias[j]);
  if (act == 1) {
    const f16 u = (f16)((float)t * (float)(f16)0.70710678118654757f);
    const float e = erff((float)u);
    f16 h = (f16)e;
    h = (f16)((float)h * 0.5f);
    const f16 sgm = (f16)(0.5f + (float)h);
    t = (f16)((float)t * (float)sgm);
  }
  if (res1) t = (f16)((float)res1[roff + j] + (float)t);
  if (res2) t = (f16)((float)t + (float)res2[roff + j]);
  return t;
}

void oracle_gemm_nt_fused_f16(const f16* x, const f16* w, const f16* bias, const f16* res1, const f16* res2, void* y,
                              int64_t m, int64_t n, int64_t k, int64_t ldy, int64_t ldr, int act, int out_f32,
                              int64_t row0, int64_t row1, int64_t col0, int64_t col1) {
  (void)m;
  (void)n;
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t i = row0; i < row1; ++i) {
    for (int64_t j = col0; j < col1; ++j) {
      float acc = 0.0f;
      const f16* xr = x + i * k;
      const f16* wr = w + j * k;
      for (int64_t kk = 0; kk < k; ++kk) acc = acc + ((float)xr[kk]) * ((float)wr[kk]);
      const f16 t = fused_tail((f16)acc, bias, res1, res2, j, i * ldr, act);
      if (out_f32) ((float*)y)[i * ldy + j] = (float)t;
      else ((f16*)y)[i * ldy + j] = t;
    }
  }
}

void oracle_gemv_fused_f16(const f16* x, const f16* w, const f16* bias, const f16* res1, const f16* res2, void* y,
                           int64_t n, int64_t k, int act, int out_f32) {
  oracle_gemm_nt_fused_f16(x, w, bias, res1, res2, y, 1, n, k, n, n, act, out_f32, 0, 1, 0, n);
}
