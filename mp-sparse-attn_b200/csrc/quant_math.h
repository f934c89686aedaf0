// Element / scale arithmetic of the MX block quantizers, shared by the CUDA kernels and by a
// host-side unit test (the functions are __host__ __device__ and have no CUDA-only dependency
// besides <cuda_fp8.h>, whose conversions also have host implementations).
//
// Follows ours/quant_mxint8.py of the reference:
//   shared exponent  floor(log2(amax)) - emax            (:303-304 fp4, :191-192 fp8)
//   scale code       clamp(floor(log2(scale)) + 127, 0, 254)                 (:347-351)
//   fp4 element rule thresholds 1/2/4 for the exponent, mantissa bit iff the value
//                    normalised by 2^(exp-1) is > 1.25 (> 0.25 when exp == 0)  (:315-331)
//   fp8 element rule clamp to +-57344, round-to-nearest-even cast to E5M2     (:203-205)
#pragma once
#include <cstdint>
#include <cmath>
#include <cuda_fp8.h>

#if defined(__CUDACC__)
#define MPSA_HD __host__ __device__ __forceinline__
#else
#define MPSA_HD inline
#endif

namespace mpsa {

enum ElemFmt : int { FMT_FP4 = 0, FMT_FP8_E5M2 = 1, FMT_FP8_E4M3 = 2 };

MPSA_HD float bits_to_float(uint32_t b) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(b);
#else
  union { uint32_t u; float f; } c; c.u = b; return c.f;
#endif
}

MPSA_HD uint32_t float_to_bits_early(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  union { uint32_t u; float f; } c; c.f = f; return c.u;
#endif
}

// Result of the shared-exponent step for one block.
struct BlockScale {
  float inv_scale;   // 2^-shared_exp (exact); elements are multiplied by it
  uint8_t code;      // E8M0 code stored for the block
  bool zero;         // amax == 0 (the reference produces 0/0 here)
};

// emax: 3 for E2M1 and 7 for the reference's fp8 path (ours/quant_mxint8.py:303, :191);
// 8 for the E4M3 variant, which the reference does not have.
MPSA_HD BlockScale mx_block_scale(float amax, int emax) {
  BlockScale r;
  if (!(amax > 0.0f)) {          // 0 (or NaN): log2 -> -inf, code clamps to 0
    r.inv_scale = 0.0f; r.code = 0; r.zero = true;
    return r;
  }
  // floor(log2f(amax)) with the accurate library log2f, as the reference's tl.log2 does.  This is
  // the exponent field of amax except for the one or two largest mantissa codes below a power of
  // two, where the correctly rounded logarithm already equals the next integer.
  // The library call is only needed for those codes (and for subnormals); elsewhere the exponent
  // field is the answer.
  const uint32_t ab = float_to_bits_early(amax);
  const uint32_t ef = ab >> 23, mant = ab & 0x007fffffu;
  int e = (ef == 0 || ef == 255 || mant >= 0x007fff00u) ? (int)floorf(log2f(amax)) : (int)ef - 127;
  int sh = e - emax;
  if (sh < -126) sh = -126;
  if (sh > 126) sh = 126;
  r.inv_scale = bits_to_float((uint32_t)(127 - sh) << 23);
  int c = sh + 127;
  r.code = (uint8_t)(c < 0 ? 0 : (c > 254 ? 254 : c));
  r.zero = false;
  return r;
}

// E2M1 code of y (already divided by the block scale) under the reference's rule.
// Equivalent closed form of ours/quant_mxint8.py:315-331:
//   |y| <= 0.125 -> 0 ; (0.125,1) -> 0.5 ; [1,1.25] -> 1 ; (1.25,2) -> 1.5 ; [2,2.5] -> 2 ;
//   (2.5,4) -> 3 ; [4,5] -> 4 ; > 5 -> 6 ; sign bit = !(y >= 0).
MPSA_HD uint32_t fp4_code_ref(float y) {
  float a = fabsf(y);
  uint32_t m = (uint32_t)(a > 0.125f) + (uint32_t)(a >= 1.0f) + (uint32_t)(a > 1.25f) +
               (uint32_t)(a >= 2.0f) + (uint32_t)(a > 2.5f) + (uint32_t)(a >= 4.0f) +
               (uint32_t)(a > 5.0f);
  uint32_t s = (y >= 0.0f) ? 0u : 8u;
  return s | m;
}

MPSA_HD uint32_t float_to_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  union { uint32_t u; float f; } c; c.f = f; return c.u;
#endif
}

// The reference's E2M1 rule as a snap to the grid: returns the (signed) E2M1-representable value whose
// code fp4_code_ref(y) would produce, so that ANY exact float -> E2M1 converter (the hardware cvt on the
// device, fp4_code_rne on the host) yields the reference's code.  |y| >= 1: keep the exponent, mantissa
// becomes .5 iff it exceeded .25 (ours/quant_mxint8.py:326-328); |y| < 1: 0.5 iff |y| > 0.125 (:328 with
// exp == 0); sign bit iff y < 0 (the reference tests y >= 0, so -0.0 counts as positive, :318).
MPSA_HD float fp4_snap_ref(float y) {
  y = y + 0.0f;                                   // -0.0 -> +0.0
  const uint32_t u = float_to_bits(y);
  const uint32_t s = u & 0x80000000u, au = u & 0x7fffffffu;
  uint32_t r;
  if (au >= 0x3f800000u) r = (au & 0x7f800000u) | (((au & 0x007fffffu) > 0x00200000u) ? 0x00400000u : 0u);
  else r = (au > 0x3e000000u) ? 0x3f000000u : 0u;
  return bits_to_float(s | r);
}

// E2M1 round-to-nearest-even, saturating (OCP MX rule; ours/mxfp.py:84-170).  Used where no
// reference quantizer exists (NVFP4, P and V operands).
MPSA_HD uint32_t fp4_code_rne(float y) {
  float a = fabsf(y);
  uint32_t m = (uint32_t)(a > 0.25f) + (uint32_t)(a >= 0.75f) + (uint32_t)(a > 1.25f) +
               (uint32_t)(a >= 1.75f) + (uint32_t)(a > 2.5f) + (uint32_t)(a >= 3.5f) +
               (uint32_t)(a > 5.0f);
  uint32_t s = (y < 0.0f || (y == 0.0f && std::signbit(y))) ? 8u : 0u;
  return s | m;
}

MPSA_HD uint32_t fp8_code(float y, int fmt) {
  if (fmt == FMT_FP8_E5M2) {
    y = fminf(fmaxf(y, -57344.0f), 57344.0f);
    return (uint32_t)__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E5M2);
  }
  y = fminf(fmaxf(y, -448.0f), 448.0f);
  return (uint32_t)__nv_cvt_float_to_fp8(y, __NV_SATFINITE, __NV_E4M3);
}

// int8 rule of ours/quant_mxint8.py:46-52: scale = amax/127 + 1e-7, y = x/scale,
// add 0.5*sign(y), truncate toward zero.
MPSA_HD int8_t int8_code_ref(float x, float scale) {
  float y = x / scale;
  y += (y >= 0.0f) ? 0.5f : -0.5f;
  return (int8_t)(int)y;
}

}  // namespace mpsa
