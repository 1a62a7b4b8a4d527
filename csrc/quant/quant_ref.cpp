// Host oracle for the block-quantised formats: scalar dequantisation and a quantised GEMV.  Exported with C linkage
// from the host runtime library; the CUDA kernels in quant.cu are tested against it and against the NumPy reader.
#include <stdint.h>

#include "quant_blocks.h"

extern "C" {

// out[n] = dequantised elements; n must be a multiple of the block size.  Returns 0, or -1 for an unknown type.
int ubq_dequantize(const uint8_t* blocks, float* out, int64_t n, int qtype) {
  const int be = ubq_block_elems(qtype), bb = ubq_block_bytes(qtype);
  if (bb == 0 || n % be != 0) return -1;
  for (int64_t b = 0; b < n / be; ++b)
    for (int i = 0; i < be; i += 8) ubq_decode8(blocks + b * bb, qtype, i, out + b * be + i);
  return 0;
}

// out[m, n] = sum_k x[m, k] * dequant(w)[n, k];  w holds N rows of K/block_elems blocks each.
int ubq_gemv(const uint8_t* w, const float* x, float* out, int M, int N, int K, int qtype) {
  const int be = ubq_block_elems(qtype), bb = ubq_block_bytes(qtype);
  if (bb == 0 || K % be != 0) return -1;
  const int64_t row_bytes = (int64_t)(K / be) * bb;
  for (int n = 0; n < N; ++n) {
    const uint8_t* row = w + n * row_bytes;
    for (int m = 0; m < M; ++m) out[(int64_t)m * N + n] = 0.f;
    for (int k = 0; k < K; k += 8) {
      float v[8];
      ubq_decode8(row + (int64_t)(k / be) * bb, qtype, k % be, v);
      for (int m = 0; m < M; ++m) {
        const float* xr = x + (int64_t)m * K + k;
        float acc = 0.f;
        for (int j = 0; j < 8; ++j) acc += v[j] * xr[j];
        out[(int64_t)m * N + n] += acc;
      }
    }
  }
  return 0;
}

}  // extern "C"
