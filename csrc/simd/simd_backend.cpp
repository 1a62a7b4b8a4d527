// Host vector kernels: the C++ counterpart of the reference's `simd` module (crates/runtime/src/simd/mod.rs:103-201,
// the `SimdBackend` trait: q4_gemv, q4_gemm, rms_norm, fused_swiglu, apply_rope, softmax, silu, mul, add, dot) with
// the same run-time dispatch idea (`CpuFeatures::detect`, :29-97): AVX2+FMA when the CPU has it, portable code
// otherwise.  They serve the CPU oracle path and the host side of the engine; the GPU never calls them.
//
// What is vectorised at level >= 1 (AVX2+FMA): dot / add / mul, RMSNorm, SiLU and SwiGLU (a polynomial exp in 8
// lanes; the reference's AVX2 code calls scalar expf per lane, simd/arch/avx2.rs:204-243), softmax (vector max, exp
// and sum), rotary embedding (8 pair columns at a time) and the Q4_0 / Q4_K / Q8_0 row dot products (nibbles unpacked
// to 8 float lanes, simd/arch/avx2.rs:59-107).  The quantised GEMM is tiled over (rows of w) x (rows of x) and the
// row tiles are spread over threads (simd/matmul/gemm.rs:107-155 uses rayon over 64 x 64 x 256 tiles).
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <thread>
#include <vector>

#include "../quant/quant_blocks.h"

#if defined(__x86_64__) || defined(__i386__)
#include <immintrin.h>
#define UBS_X86 1
#else
#define UBS_X86 0
#endif

namespace {

int g_level = -1;  // 0 scalar, 1 avx2+fma, 2 avx512 (runs the avx2 code, like the reference's AVX-512 backend)
int g_threads = 0; // 0 = hardware concurrency (capped)

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

inline float silu1(float v) { return v / (1.f + expf(-v)); }

#if UBS_X86
#define AVX2 __attribute__((target("avx2,fma,f16c")))

AVX2 inline float hsum(__m256 v) {
  __m128 lo = _mm_add_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
  lo = _mm_add_ps(lo, _mm_movehl_ps(lo, lo));
  lo = _mm_add_ss(lo, _mm_shuffle_ps(lo, lo, 1));
  return _mm_cvtss_f32(lo);
}
AVX2 inline float hmax(__m256 v) {
  __m128 lo = _mm_max_ps(_mm256_castps256_ps128(v), _mm256_extractf128_ps(v, 1));
  lo = _mm_max_ps(lo, _mm_movehl_ps(lo, lo));
  lo = _mm_max_ss(lo, _mm_shuffle_ps(lo, lo, 1));
  return _mm_cvtss_f32(lo);
}

// exp(x) in 8 lanes: x = n ln2 + r, |r| <= ln2 / 2, degree-6 polynomial for exp(r), exponent stitched in by bits.
// Relative error about 2e-7 over the clamped range [-87.3, 88.3].
AVX2 inline __m256 exp8(__m256 x) {
  x = _mm256_min_ps(_mm256_max_ps(x, _mm256_set1_ps(-87.3f)), _mm256_set1_ps(88.3f));
  const __m256 n = _mm256_round_ps(_mm256_mul_ps(x, _mm256_set1_ps(1.44269504088896341f)), _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
  __m256 r = _mm256_fnmadd_ps(n, _mm256_set1_ps(0.693359375f), x);
  r = _mm256_fnmadd_ps(n, _mm256_set1_ps(-2.12194440e-4f), r);
  __m256 p = _mm256_set1_ps(1.0f / 720.0f);
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(1.0f / 120.0f));
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(1.0f / 24.0f));
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(1.0f / 6.0f));
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(0.5f));
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(1.0f));
  p = _mm256_fmadd_ps(p, r, _mm256_set1_ps(1.0f));
  const __m256i e = _mm256_slli_epi32(_mm256_add_epi32(_mm256_cvtps_epi32(n), _mm256_set1_epi32(127)), 23);
  return _mm256_mul_ps(p, _mm256_castsi256_ps(e));
}

AVX2 float dot_avx2(const float* a, const float* b, int64_t n) {
  __m256 acc0 = _mm256_setzero_ps(), acc1 = _mm256_setzero_ps();
  int64_t i = 0;
  for (; i + 16 <= n; i += 16) {
    acc0 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), acc0);
    acc1 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 8), _mm256_loadu_ps(b + i + 8), acc1);
  }
  float s = hsum(_mm256_add_ps(acc0, acc1));
  for (; i < n; ++i) s += a[i] * b[i];
  return s;
}

AVX2 void axpby_avx2(float* out, const float* a, const float* b, int64_t n, int op) {
  int64_t i = 0;
  for (; i + 8 <= n; i += 8) {
    const __m256 x = _mm256_loadu_ps(a + i), y = _mm256_loadu_ps(b + i);
    _mm256_storeu_ps(out + i, op == 0 ? _mm256_add_ps(x, y) : _mm256_mul_ps(x, y));
  }
  for (; i < n; ++i) out[i] = op == 0 ? a[i] + b[i] : a[i] * b[i];
}

AVX2 void scale_mul_avx2(float* out, const float* x, const float* w, float s, int64_t n) {
  const __m256 vs = _mm256_set1_ps(s);
  int64_t i = 0;
  for (; i + 8 <= n; i += 8)
    _mm256_storeu_ps(out + i, _mm256_mul_ps(_mm256_mul_ps(_mm256_loadu_ps(x + i), vs), _mm256_loadu_ps(w + i)));
  for (; i < n; ++i) out[i] = x[i] * s * w[i];
}

// out = silu(g) (* up when up != nullptr)
AVX2 void silu_avx2(float* out, const float* g, const float* up, int64_t n) {
  const __m256 one = _mm256_set1_ps(1.f);
  int64_t i = 0;
  for (; i + 8 <= n; i += 8) {
    const __m256 v = _mm256_loadu_ps(g + i);
    const __m256 e = exp8(_mm256_sub_ps(_mm256_setzero_ps(), v));
    __m256 y = _mm256_div_ps(v, _mm256_add_ps(one, e));
    if (up != nullptr) y = _mm256_mul_ps(y, _mm256_loadu_ps(up + i));
    _mm256_storeu_ps(out + i, y);
  }
  for (; i < n; ++i) out[i] = silu1(g[i]) * (up != nullptr ? up[i] : 1.f);
}

AVX2 void softmax_row_avx2(float* o, const float* x, int64_t n) {
  __m256 vm = _mm256_set1_ps(-INFINITY);
  int64_t i = 0;
  for (; i + 8 <= n; i += 8) vm = _mm256_max_ps(vm, _mm256_loadu_ps(x + i));
  float mx = hmax(vm);
  for (; i < n; ++i) mx = x[i] > mx ? x[i] : mx;
  const __m256 vmx = _mm256_set1_ps(mx);
  __m256 vs = _mm256_setzero_ps();
  for (i = 0; i + 8 <= n; i += 8) {
    const __m256 e = exp8(_mm256_sub_ps(_mm256_loadu_ps(x + i), vmx));
    _mm256_storeu_ps(o + i, e);
    vs = _mm256_add_ps(vs, e);
  }
  float s = hsum(vs);
  for (; i < n; ++i) { o[i] = expf(x[i] - mx); s += o[i]; }
  const __m256 inv = _mm256_set1_ps(1.f / s);
  for (i = 0; i + 8 <= n; i += 8) _mm256_storeu_ps(o + i, _mm256_mul_ps(_mm256_loadu_ps(o + i), inv));
  for (; i < n; ++i) o[i] *= 1.f / s;
}

// rotate the pair columns of one head, 8 at a time: (a, b) -> (a c - b s, b c + a s); returns the columns done
AVX2 int rope_head_avx2(float* p, int half, const float* cs, const float* sn) {
  int i = 0;
  for (; i + 8 <= half; i += 8) {
    const __m256 c = _mm256_loadu_ps(cs + i), s = _mm256_loadu_ps(sn + i);
    const __m256 a = _mm256_loadu_ps(p + i), b = _mm256_loadu_ps(p + i + half);
    _mm256_storeu_ps(p + i, _mm256_fmsub_ps(a, c, _mm256_mul_ps(b, s)));
    _mm256_storeu_ps(p + i + half, _mm256_fmadd_ps(b, c, _mm256_mul_ps(a, s)));
  }
  return i;
}

// 16 packed nibbles (low or high half of 16 bytes) -> two float vectors of 8
AVX2 inline void nib16(const uint8_t* q, int shift, __m256& lo8, __m256& hi8) {
  __m128i b = _mm_loadu_si128(reinterpret_cast<const __m128i*>(q));
  if (shift) b = _mm_srli_epi16(b, 4);
  b = _mm_and_si128(b, _mm_set1_epi8(0x0F));
  lo8 = _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(b));
  hi8 = _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(_mm_srli_si128(b, 8)));
}

// dot of one Q4_0 row with x: per 32-value block d * sum((q - 8) x)
AVX2 float q4_0_dot_avx2(const uint8_t* row, const float* x, int K) {
  __m256 acc = _mm256_setzero_ps();
  const __m256 eight = _mm256_set1_ps(8.f);
  for (int b = 0; b < K / 32; ++b) {
    const uint8_t* blk = row + (int64_t)b * 18;
    const float d = ubq_f16(blk);
    const float* xb = x + b * 32;
    __m256 s = _mm256_setzero_ps(), q0, q1;
    nib16(blk + 2, 0, q0, q1);            // values 0..15
    s = _mm256_fmadd_ps(_mm256_sub_ps(q0, eight), _mm256_loadu_ps(xb), s);
    s = _mm256_fmadd_ps(_mm256_sub_ps(q1, eight), _mm256_loadu_ps(xb + 8), s);
    nib16(blk + 2, 1, q0, q1);            // values 16..31
    s = _mm256_fmadd_ps(_mm256_sub_ps(q0, eight), _mm256_loadu_ps(xb + 16), s);
    s = _mm256_fmadd_ps(_mm256_sub_ps(q1, eight), _mm256_loadu_ps(xb + 24), s);
    acc = _mm256_fmadd_ps(s, _mm256_set1_ps(d), acc);
  }
  return hsum(acc);
}

AVX2 float q8_0_dot_avx2(const uint8_t* row, const float* x, int K) {
  __m256 acc = _mm256_setzero_ps();
  for (int b = 0; b < K / 32; ++b) {
    const uint8_t* blk = row + (int64_t)b * 34;
    const float d = ubq_f16(blk);
    const float* xb = x + b * 32;
    __m256 s = _mm256_setzero_ps();
    for (int j = 0; j < 4; ++j) {
      const __m128i q = _mm_loadl_epi64(reinterpret_cast<const __m128i*>(blk + 2 + 8 * j));
      s = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(q)), _mm256_loadu_ps(xb + 8 * j), s);
    }
    acc = _mm256_fmadd_ps(s, _mm256_set1_ps(d), acc);
  }
  return hsum(acc);
}

// dot of one Q4_K row with x: per 32-value sub-block d*s * sum(q x) - dmin*m * sum(x)
AVX2 float q4_k_dot_avx2(const uint8_t* row, const float* x, int K) {
  float total = 0.f;
  for (int b = 0; b < K / 256; ++b) {
    const uint8_t* blk = row + (int64_t)b * 144;
    const float d = ubq_f16(blk), dmin = ubq_f16(blk + 2);
    const uint8_t* sc = blk + 4;
    const float* xb = x + b * 256;
    for (int g = 0; g < 4; ++g) {
      for (int e = 0; e < 2; ++e) {
        const int j = 2 * g + e;
        int s, m;
        if (j < 4) { s = sc[j] & 63; m = sc[j + 4] & 63; }
        else { s = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4); m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
        const uint8_t* qs = blk + 16 + g * 32;
        const float* xs = xb + g * 64 + e * 32;
        __m256 qa = _mm256_setzero_ps(), xa = _mm256_setzero_ps(), q0, q1;
        for (int h = 0; h < 2; ++h) {
          nib16(qs + 16 * h, e, q0, q1);
          const __m256 x0 = _mm256_loadu_ps(xs + 16 * h), x1 = _mm256_loadu_ps(xs + 16 * h + 8);
          qa = _mm256_fmadd_ps(q0, x0, qa);
          qa = _mm256_fmadd_ps(q1, x1, qa);
          xa = _mm256_add_ps(xa, _mm256_add_ps(x0, x1));
        }
        total += d * (float)s * hsum(qa) - dmin * (float)m * hsum(xa);
      }
    }
  }
  return total;
}
#endif  // UBS_X86

float dot_any(const float* a, const float* b, int64_t n) {
#if UBS_X86
  if (level() >= 1) return dot_avx2(a, b, n);
#endif
  float s = 0.f;
  for (int64_t i = 0; i < n; ++i) s += a[i] * b[i];
  return s;
}

// dot of one quantised row with x; `buf` (K floats) is scratch for the formats without a dedicated kernel
float qrow_dot(const uint8_t* row, const float* x, int K, int qtype, float* buf) {
#if UBS_X86
  if (level() >= 1) {
    if (qtype == UBQ_Q4_0) return q4_0_dot_avx2(row, x, K);
    if (qtype == UBQ_Q8_0) return q8_0_dot_avx2(row, x, K);
    if (qtype == UBQ_Q4_K) return q4_k_dot_avx2(row, x, K);
  }
#endif
  const int be = ubq_block_elems(qtype), bb = ubq_block_bytes(qtype);
  for (int k = 0; k < K; k += 8) ubq_decode8(row + (int64_t)(k / be) * bb, qtype, k % be, buf + k);
  return dot_any(buf, x, K);
}

int worker_count(int64_t work_items) {
  int n = g_threads > 0 ? g_threads : (int)std::thread::hardware_concurrency();
  if (n <= 0) n = 1;
  if (n > 16) n = 16;
  if ((int64_t)n > work_items) n = (int)work_items;
  return n < 1 ? 1 : n;
}

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
// Threads of the tiled quantised GEMM: 0 = all hardware threads (at most 16).
void ubs_set_threads(int n) { g_threads = n < 0 ? 0 : n; }

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
#if UBS_X86
  if (level() >= 1) return silu_avx2(out, x, nullptr, n);
#endif
  for (int64_t i = 0; i < n; ++i) out[i] = silu1(x[i]);
}

void ubs_fused_swiglu(float* out, const float* gate, const float* up, int64_t n) {
#if UBS_X86
  if (level() >= 1) return silu_avx2(out, gate, up, n);
#endif
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
#if UBS_X86
    if (level() >= 1) { softmax_row_avx2(o, xr, dim); continue; }
#endif
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
  std::vector<float> inv_freq(half), cs(half), sn(half);
  for (int i = 0; i < half; ++i) inv_freq[i] = powf(theta, -2.f * (float)i / (float)rot_dim);
  for (int64_t t = 0; t < tokens; ++t) {
    for (int i = 0; i < half; ++i) {
      const float ang = (float)positions[t] * inv_freq[i];
      cs[i] = cosf(ang);
      sn[i] = sinf(ang);
    }
    for (int h = 0; h < heads; ++h) {
      float* p = x + (t * heads + h) * head_dim;
      int i = 0;
#if UBS_X86
      if (level() >= 1) i = rope_head_avx2(p, half, cs.data(), sn.data());
#endif
      for (; i < half; ++i) {
        const float a = p[i], b = p[i + half];
        p[i] = a * cs[i] - b * sn[i];
        p[i + half] = b * cs[i] + a * sn[i];
      }
    }
  }
}

// out[m, n] = x[m, :] . dequant(w[n, :]).  Tiled: a tile of 64 weight rows is walked by one thread against blocks of 8
// activation rows (the 8 activation rows stay in cache while the 64 quantised rows stream by); tiles are handed to
// the worker threads through a shared counter.  Disjoint output columns per tile: no synchronisation on `out`.
int ubs_q_gemm(const uint8_t* w, const float* x, float* out, int M, int N, int K, int qtype) {
  const int be = ubq_block_elems(qtype), bb = ubq_block_bytes(qtype);
  if (bb == 0 || K % be != 0 || K % 8 != 0) return -1;
  if (M <= 0 || N <= 0) return 0;
  const int64_t row_bytes = (int64_t)(K / be) * bb;
  constexpr int TN = 64, TM = 8;
  const int n_tiles = (N + TN - 1) / TN;
  std::atomic<int> next(0);
  auto work = [&]() {
    std::vector<float> buf((size_t)K);
    for (;;) {
      const int t = next.fetch_add(1);
      if (t >= n_tiles) return;
      const int n0 = t * TN, n1 = std::min(N, n0 + TN);
      for (int m0 = 0; m0 < M; m0 += TM) {
        const int m1 = std::min(M, m0 + TM);
        for (int n = n0; n < n1; ++n) {
          const uint8_t* row = w + n * row_bytes;
          for (int m = m0; m < m1; ++m) out[(int64_t)m * N + n] = qrow_dot(row, x + (int64_t)m * K, K, qtype, buf.data());
        }
      }
    }
  };
  // small problems are not worth a thread start (the reference switches at m >= 8 and n >= 64, gemm.rs:19-25)
  const int nt = ((int64_t)M * N * K < (1 << 22)) ? 1 : worker_count(n_tiles);
  if (nt <= 1) {
    work();
    return 0;
  }
  std::vector<std::thread> th;
  th.reserve(nt - 1);
  for (int i = 1; i < nt; ++i) th.emplace_back(work);
  work();
  for (auto& t : th) t.join();
  return 0;
}

int ubs_q_gemv(const uint8_t* w, const float* x, float* out, int N, int K, int qtype) {
  return ubs_q_gemm(w, x, out, 1, N, K, qtype);
}

}  // extern "C"
