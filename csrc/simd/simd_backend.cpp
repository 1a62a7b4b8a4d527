// Host vector kernels: the C++ counterpart of the reference's `simd` module (crates/runtime/src/simd/mod.rs:103-201,
// the `SimdBackend` trait: q4_gemv, q4_gemm, rms_norm, fused_swiglu, apply_rope, softmax, silu, mul, add, dot) with
// the same run-time dispatch idea (`CpuFeatures::detect`, :29-97): AVX2+FMA when the CPU has it, portable code
// otherwise.  They serve the CPU oracle path and the host side of the engine; the GPU never calls them.
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "../quant/quant_blocks.h"

#if defined(__x86_64__) || defined(__i386__)
#include <immintrin.h>
#define UBS_X86 1
#else
#define UBS_X86 0
#endif

namespace {

int g_level = -1;  // 0 scalar, 1 avx2+fma, 2 avx512 (runs the avx2 code, like the reference's AVX-512 backend)

int detect() {
#if UBS_X86
  __builtin_cpu_init();
  if (__builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) return 2;
  if (__builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma")) return 1;
#endif
  return 0;
}

inline int level() {
  if (g_level < 0) g_level = detect();
  return g_level;
}

#if UBS_X86
__attribute__((target("avx2,fma"))) float dot_avx2(const float* a, const float* b, int64_t n) {
  __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
  int64_t i = 0;
  for (; i + 16 <= n; i += 16) {
    acc0 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), acc0);
    acc1 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 8), _mm256_loadu_ps(b + i + 8), acc1);
  }
  acc0 = _mm256_add_ps(acc0, acc1);
  __m128 lo = _mm_add_ps(_mm256_castps256_ps128(acc0), _mm256_extractf128_ps(acc0, 1));
  lo = _mm_add_ps(lo, _mm_movehl_ps(lo, lo));
  lo = _mm_add_ss(lo, _mm_shuffle_ps(lo, lo, 1));
  float s = _mm_cvtss_f32(lo);
  for (; i < n; ++i) s += a[i] * b[i];
  return s;
}

__attribute__((target("avx2,fma"))) void axpby_avx2(float* out, const float* a, const float* b, int64_t n, int op) {
  int64_t i = 0;
  for (; i + 8 <= n; i += 8) {
    const __m256 x = _mm256_loadu_ps(a + i), y = _mm256_loadu_ps(b + i);
    _mm256_storeu_ps(out + i, op == 0 ? _mm256_add_ps(x, y) : _mm256_mul_ps(x, y));
  }
  for (; i < n; ++i) out[i] = op == 0 ? a[i] + b[i] : a[i] * b[i];
}

__attribute__((target("avx2,fma"))) void scale_mul_avx2(float* out, const float* x, const float* w, float s, int64_t n) {
  const __m256 vs = _mm256_set1_ps(s);
  int64_t i = 0;
  for (; i + 8 <= n; i += 8)
    _mm256_storeu_ps(out + i, _mm256_mul_ps(_mm256_mul_ps(_mm256_loadu_ps(x + i), vs), _mm256_loadu_ps(w + i)));
  for (; i < n; ++i) out[i] = x[i] * s * w[i];
}
#endif

float dot_any(const float* a, const float* b, int64_t n) {
#if UBS_X86
  if (level() >= 1) return dot_avx2(a, b, n);
#endif
  float s = 0.f;
  for (int64_t i = 0; i < n; ++i) s += a[i] * b[i];
  return s;
}

inline float silu1(float v) { return v / (1.f + expf(-v)); }

}  // namespace

extern "C" {

// 0 scalar, 1 AVX2+FMA, 2 AVX-512 present (AVX2 code paths).
int ubs_backend_level() { return level(); }
const char* ubs_backend_name() {
  switch (level()) {
    case 2: return "avx512 (avx2 kernels)";
    case 1: return "avx2+fma";
    default: return "scalar";
  }
}
// Tests use this to run both code paths on one machine; level is clamped to what the CPU supports.
void ubs_force_level(int lvl) {
  const int hw = detect();
  g_level = lvl < 0 ? hw : (lvl > hw ? hw : lvl);
}

float ubs_dot(const float* a, const float* b, int64_t n) { return dot_any(a, b, n); }

void ubs_add(float* out, const float* a, const float* b, int64_t n) {
#if UBS_X86
  if (level() >= 1) return axpby_avx2(out, a, b, n, 0);
#endif
  for (int64_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}

void ubs_mul(float* out, const float* a, const float* b, int64_t n) {
#if UBS_X86
  if (level() >= 1) return axpby_avx2(out, a, b, n, 1);
#endif
  for (int64_t i = 0; i < n; ++i) out[i] = a[i] * b[i];
}

void ubs_silu(float* out, const float* x, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = silu1(x[i]);
}

void ubs_fused_swiglu(float* out, const float* gate, const float* up, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = silu1(gate[i]) * up[i];
}

// rows x dim, out may alias x.
void ubs_rms_norm(float* out, const float* x, const float* w, int64_t rows, int64_t dim, float eps) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * dim;
    const float inv = 1.f / sqrtf(dot_any(xr, xr, dim) / (float)dim + eps);
#if UBS_X86
    if (level() >= 1) { scale_mul_avx2(out + r * dim, xr, w, inv, dim); continue; }
#endif
    for (int64_t i = 0; i < dim; ++i) out[r * dim + i] = xr[i] * inv * w[i];
  }
}

void ubs_softmax(float* out, const float* x, int64_t rows, int64_t dim) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * dim;
    float* o = out + r * dim;
    float mx = xr[0];
    for (int64_t i = 1; i < dim; ++i) mx = xr[i] > mx ? xr[i] : mx;
    float s = 0.f;
    for (int64_t i = 0; i < dim; ++i) { o[i] = expf(xr[i] - mx); s += o[i]; }
    const float inv = 1.f / s;
    for (int64_t i = 0; i < dim; ++i) o[i] *= inv;
  }
}

// In-place rotary embedding of x [tokens, heads, head_dim]; pairs (i, i + rot/2) rotate by pos * theta^(-2i/rot).
void ubs_apply_rope(float* x, const int32_t* positions, int64_t tokens, int heads, int head_dim, int rot_dim, float theta) {
  const int half = rot_dim / 2;
  for (int64_t t = 0; t < tokens; ++t) {
    for (int i = 0; i < half; ++i) {
      const float ang = (float)positions[t] * powf(theta, -2.f * (float)i / (float)rot_dim);
      const float c = cosf(ang), s = sinf(ang);
      for (int h = 0; h < heads; ++h) {
        float* p = x + (t * heads + h) * head_dim;
        const float a = p[i], b = p[i + half];
        p[i] = a * c - b * s;
        p[i + half] = b * c + a * s;
      }
    }
  }
}

// out[m, n] = x[m, :] . dequant(w[n, :]);  one dequantised row is reused for all M activations.
int ubs_q_gemm(const uint8_t* w, const float* x, float* out, int M, int N, int K, int qtype) {
  const int be = ubq_block_elems(qtype), bb = ubq_block_bytes(qtype);
  if (bb == 0 || K % be != 0) return -1;
  const int64_t row_bytes = (int64_t)(K / be) * bb;
  float buf[4096];
  for (int n = 0; n < N; ++n) {
    for (int m = 0; m < M; ++m) out[(int64_t)m * N + n] = 0.f;
    for (int k0 = 0; k0 < K; k0 += 4096) {
      const int len = K - k0 < 4096 ? K - k0 : 4096;
      for (int k = 0; k < len; k += 8)
        ubq_decode8(w + n * row_bytes + (int64_t)((k0 + k) / be) * bb, qtype, (k0 + k) % be, buf + k);
      for (int m = 0; m < M; ++m) out[(int64_t)m * N + n] += dot_any(buf, x + (int64_t)m * K + k0, len);
    }
  }
  return 0;
}

int ubs_q_gemv(const uint8_t* w, const float* x, float* out, int N, int K, int qtype) {
  return ubs_q_gemm(w, x, out, 1, N, K, qtype);
}

}  // extern "C"
