// Block layouts of the ggml quantisation formats this framework reads, and an 8-element decoder shared by the host
// oracle (quant_ref.cpp) and the CUDA kernels (quant.cu).  The layouts follow ggml (low nibbles are the first half
// of a block); the reference's own SIMD blocks interleave nibbles and pad Q4_0 blocks to 32 bytes
// (crates/runtime/src/simd/quant/block.rs:27-61), which cannot read real GGUF files.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define UBQ_HD __host__ __device__ __forceinline__
#else
#define UBQ_HD inline
#endif

enum UbqType { UBQ_Q4_0 = 2, UBQ_Q4_1 = 3, UBQ_Q5_0 = 6, UBQ_Q8_0 = 8, UBQ_Q4_K = 12, UBQ_Q6_K = 14 };

UBQ_HD int ubq_block_elems(int t) { return (t == UBQ_Q4_K || t == UBQ_Q6_K) ? 256 : 32; }
UBQ_HD int ubq_block_bytes(int t) {
  switch (t) {
    case UBQ_Q4_0: return 18;
    case UBQ_Q4_1: return 20;
    case UBQ_Q5_0: return 22;
    case UBQ_Q8_0: return 34;
    case UBQ_Q4_K: return 144;
    case UBQ_Q6_K: return 210;
    default: return 0;
  }
}

// IEEE half -> float without relying on a half type (works on host and device).
UBQ_HD float ubq_f16(const uint8_t* p) {
  const uint32_t h = (uint32_t)p[0] | ((uint32_t)p[1] << 8);
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal: renormalise
      int e = -1;
      do { ++e; man <<= 1; } while ((man & 0x400u) == 0);
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  union { uint32_t u; float f; } cv;
  cv.u = bits;
  return cv.f;
}

// Elements [i, i+8) of one block (i a multiple of 8, inside the block) as floats.
UBQ_HD void ubq_decode8(const uint8_t* blk, int t, int i, float* out) {
  switch (t) {
    case UBQ_Q4_0: {
      const float d = ubq_f16(blk);
      const uint8_t* qs = blk + 2 + (i & 15);
      const int sh = i < 16 ? 0 : 4;
      for (int j = 0; j < 8; ++j) out[j] = d * (float)(((qs[j] >> sh) & 0xF) - 8);
      return;
    }
    case UBQ_Q4_1: {
      const float d = ubq_f16(blk), m = ubq_f16(blk + 2);
      const uint8_t* qs = blk + 4 + (i & 15);
      const int sh = i < 16 ? 0 : 4;
      for (int j = 0; j < 8; ++j) out[j] = d * (float)((qs[j] >> sh) & 0xF) + m;
      return;
    }
    case UBQ_Q5_0: {
      const float d = ubq_f16(blk);
      const uint32_t qh = (uint32_t)blk[2] | ((uint32_t)blk[3] << 8) | ((uint32_t)blk[4] << 16) | ((uint32_t)blk[5] << 24);
      const uint8_t* qs = blk + 6 + (i & 15);
      const int sh = i < 16 ? 0 : 4;
      for (int j = 0; j < 8; ++j) {
        const int q = ((qs[j] >> sh) & 0xF) | (int)(((qh >> (i + j)) & 1u) << 4);
        out[j] = d * (float)(q - 16);
      }
      return;
    }
    case UBQ_Q8_0: {
      const float d = ubq_f16(blk);
      const int8_t* qs = reinterpret_cast<const int8_t*>(blk + 2) + i;
      for (int j = 0; j < 8; ++j) out[j] = d * (float)qs[j];
      return;
    }
    case UBQ_Q4_K: {
      const float d = ubq_f16(blk), dmin = ubq_f16(blk + 2);
      const uint8_t* sc = blk + 4;
      const int g = i >> 6, r = i & 63, hi = r >= 32;
      const int j = 2 * g + hi;
      int s, m;
      if (j < 4) { s = sc[j] & 63; m = sc[j + 4] & 63; }
      else { s = (sc[j + 4] & 0x0F) | ((sc[j - 4] >> 6) << 4); m = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4); }
      const uint8_t* qs = blk + 16 + g * 32 + (r & 31);
      const float ds = d * (float)s, dm = dmin * (float)m;
      const int sh = hi ? 4 : 0;
      for (int k = 0; k < 8; ++k) out[k] = ds * (float)((qs[k] >> sh) & 0xF) - dm;
      return;
    }
    case UBQ_Q6_K: {
      const float d = ubq_f16(blk + 208);
      const int half = i >> 7, r = i & 127, qd = r >> 5, pos = r & 31;
      const uint8_t* ql = blk + half * 64 + ((qd & 1) ? 32 : 0) + pos;
      const uint8_t* qh = blk + 128 + half * 32 + pos;
      const int8_t* scs = reinterpret_cast<const int8_t*>(blk + 192) + half * 8 + 2 * qd;
      const int lsh = qd >= 2 ? 4 : 0, hsh = 2 * qd;
      for (int k = 0; k < 8; ++k) {
        const int q = ((ql[k] >> lsh) & 0xF) | (((qh[k] >> hsh) & 3) << 4);
        out[k] = d * (float)scs[(pos + k) >> 4] * (float)(q - 32);
      }
      return;
    }
    default:
      for (int j = 0; j < 8; ++j) out[j] = 0.f;
  }
}
