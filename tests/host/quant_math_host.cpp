// Host build of the quantizer arithmetic (csrc/quant_math.h) so that the exact code the CUDA
// kernels run per element can be compared with the golden vectors without a GPU.
#include "quant_math.h"

#include <cstring>

using namespace mpsa;

static float bf16_to_float(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// x: bf16 bits [rows, d]; outputs: fp4 codes (one per byte), fp8 codes, scale codes [rows, d/32]
extern "C" void host_quant_mx(const uint16_t* x, long long rows, int d, float s, int fp8_fmt, uint8_t* fp4,
                              uint8_t* fp4_scale, uint8_t* fp8, uint8_t* fp8_scale) {
  for (long long r = 0; r < rows; ++r)
    for (int kb = 0; kb < d / 32; ++kb) {
      float v[32], amax = 0.0f;
      for (int i = 0; i < 32; ++i) {
        v[i] = bf16_to_float(x[r * d + kb * 32 + i]) * s;
        amax = fmaxf(amax, fabsf(v[i]));
      }
      BlockScale b4 = mx_block_scale(amax, 3);
      BlockScale b8 = mx_block_scale(amax, fp8_fmt == FMT_FP8_E4M3 ? 8 : 7);
      fp4_scale[r * (d / 32) + kb] = b4.code;
      fp8_scale[r * (d / 32) + kb] = b8.code;
      for (int i = 0; i < 32; ++i) {
        float y4 = fminf(fmaxf(v[i] * b4.inv_scale, -6.0f), 6.0f);
        const uint8_t direct = (uint8_t)fp4_code_ref(y4);
        // the kernels snap to the grid and convert with the hardware; both routes must agree
        const uint8_t snapped = (uint8_t)fp4_code_rne(fp4_snap_ref(v[i] * b4.inv_scale));
        fp4[r * d + kb * 32 + i] = b4.zero ? 8 : (direct == snapped ? direct : 0xEE);
        fp8[r * d + kb * 32 + i] = b8.zero ? 0 : (uint8_t)fp8_code(v[i] * b8.inv_scale, fp8_fmt);
      }
    }
}

extern "C" void host_quant_int8(const uint16_t* x, long long rows, int d, float s, int8_t* codes, float* scales) {
  for (long long r = 0; r < rows; ++r)
    for (int kb = 0; kb < d / 32; ++kb) {
      float v[32], amax = 0.0f;
      for (int i = 0; i < 32; ++i) {
        v[i] = bf16_to_float(x[r * d + kb * 32 + i]) * s;
        amax = fmaxf(amax, fabsf(v[i]));
      }
      float scale = amax / 127.0f + 0.0000001f;
      for (int i = 0; i < 32; ++i) codes[r * d + kb * 32 + i] = int8_code_ref(v[i], scale);
      __nv_fp8_storage_t s8 = __nv_cvt_float_to_fp8(scale, __NV_SATFINITE, __NV_E5M2);
      __half_raw hr = __nv_cvt_fp8_to_halfraw(s8, __NV_E5M2);
      scales[r * (d / 32) + kb] = __half2float(__half(hr));
    }
}

extern "C" void host_fp4_rne(const float* x, long long n, uint8_t* codes) {
  for (long long i = 0; i < n; ++i) codes[i] = (uint8_t)fp4_code_rne(x[i]);
}
