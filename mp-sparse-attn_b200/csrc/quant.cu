// MX block quantizers (bf16/fp16/fp32 -> MXFP8 / MXFP4 with E8M0 scales per 32 elements, and the
// per-32 int8 variant) for sm_100a.
//
// One CTA handles a tile of 128 rows x 128 columns of one (batch, head).  Each thread owns runs of
// 16 consecutive elements (128-bit loads), two neighbouring lanes own one 32-element block and
// combine their amax with a single warp shuffle.  One pass over the input can emit, at once,
//   * MXFP8 codes (E5M2 as in the reference, or E4M3), one byte per element,
//   * MXFP4 codes packed two per byte (low nibble first) and/or one per byte (the reference's
//     output format, ours/quant_mxint8.py:454),
//   * the scales row-major [.., L, D/32] (reference format) and/or as 512-byte 128x4 tiles
//     [.., ceil(L/128), ceil(D/128), 32, 4, 4] - the layout tcgen05.cp moves into TMEM unchanged
//     (ours/mxfp_attn_kernel.py:56-57 builds the same layout with a separate permute+copy).
// The kernel is HBM-bound: algorithmic bytes per element are 2 (bf16 in) + 1 (fp8) + 1/32, or
// 2 + 1/2 + 1/32 for packed fp4.
#include "api_internal.h"
#include "quant_math.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <mutex>

namespace mpsa {

struct QuantParams {
  const void* x;
  int in_dtype;               // 0 bf16, 1 fp16, 2 fp32
  int B, H, L, D;
  long long xs_b, xs_h, xs_l;  // input strides in elements (inner stride 1)
  float s;                     // fp32 scalar multiplied into x before quantisation
  const float* center;         // optional [B,H,D]: subtracted from every row first (result rounded to the input dtype)
  const float* rope_cos;       // ROPE kernels: cos / sin of the rotation angles, fp32 [.., L, D/2], batch stride rope_sb
  const float* rope_sin;       // (0 = shared by the batch), shared by the heads
  long long rope_sb;
  int fp8_fmt;                 // FMT_FP8_E5M2 or FMT_FP8_E4M3
  // reference-format outputs (strided like the input tensor's logical shape)
  uint8_t* fp8_codes;  long long o8_b, o8_h, o8_l;
  uint8_t* fp4_codes_unpacked;  long long o4_b, o4_h, o4_l;
  uint8_t* fp8_scales_rm;      // [B,H,L,D/32]
  uint8_t* fp4_scales_rm;
  // kernel-format outputs (dense [B,H,L,*])
  uint8_t* fp4_codes_packed;   // [B,H,L,D/2]
  uint8_t* fp8_scales_tiled;   // [B,H,ceil(L/128),ceil(D/128),512]
  uint8_t* fp4_scales_tiled;
};

template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&v)[16]);

template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[16]) {
  uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
  uint4 b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void load16<__half>(const __half* p, float (&v)[16]) {
  uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
  uint4 b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
  uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    __half2 h = *reinterpret_cast<__half2*>(&w[i]);
    float2 f = __half22float2(h);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load16<float>(const float* p, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float4 a = __ldg(reinterpret_cast<const float4*>(p) + i);
    v[4 * i] = a.x; v[4 * i + 1] = a.y; v[4 * i + 2] = a.z; v[4 * i + 3] = a.w;
  }
}

// x rounded to the storage type T (what an elementwise torch op on a T tensor returns)
template <typename T> __device__ __forceinline__ float round_as(float x);
template <> __device__ __forceinline__ float round_as<__nv_bfloat16>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
template <> __device__ __forceinline__ float round_as<__half>(float x) { return __half2float(__float2half_rn(x)); }
template <> __device__ __forceinline__ float round_as<float>(float x) { return x; }

constexpr int kQuantThreads = 256;
constexpr int kRunsPerThread = 4;   // 256 threads * 4 runs * 16 elements = 128 x 128 tile (int8 / NVFP4 kernels)
constexpr int kMxThreads = 512;     // MX kernel: 512 threads * 2 runs * 16 elements
constexpr int kMxRuns = 2;

// 8 floats -> 8 E2M1 codes in one word (element 0 in the low nibble); the inputs are already on the
// E2M1 grid (fp4_snap_ref), so the conversion is exact.
__device__ __forceinline__ uint32_t cvt_e2m1x8_regs(float y0, float y1, float y2, float y3, float y4, float y5,
                                                    float y6, float y7) {
  uint32_t r;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(r)
      : "f"(y0), "f"(y1), "f"(y2), "f"(y3), "f"(y4), "f"(y5), "f"(y6), "f"(y7));
  return r;
}
// 4 floats -> 4 fp8 codes in one word (round to nearest even; satfinite clamps to +-57344 / +-448, which
// is the clamp of ours/quant_mxint8.py:203).
template <bool E4M3>
__device__ __forceinline__ uint32_t cvt_fp8x4_regs(float y0, float y1, float y2, float y3) {
  uint32_t r;
  if (E4M3) {
    asm("{\n\t.reg .b16 lo, hi;\n\tcvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\tcvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
        "mov.b32 %0, {lo, hi};\n\t}" : "=r"(r) : "f"(y0), "f"(y1), "f"(y2), "f"(y3));
  } else {
    asm("{\n\t.reg .b16 lo, hi;\n\tcvt.rn.satfinite.e5m2x2.f32 lo, %2, %1;\n\tcvt.rn.satfinite.e5m2x2.f32 hi, %4, %3;\n\t"
        "mov.b32 %0, {lo, hi};\n\t}" : "=r"(r) : "f"(y0), "f"(y1), "f"(y2), "f"(y3));
  }
  return r;
}

// ROPE: the rotary embedding is applied on the way in (rotate-half convention: y1 = x1 cos - x2 sin, y2 = x2 cos + x1 sin
// with x1 / x2 the two halves of a row; fp32 products and sum, the result rounded to the input dtype, i.e. the tensor an
// unfused pipeline would have stored).  A thread then holds a 16-element run of the first half and its partner run of
// the second half of the same row; D <= 128.
// W8 / W4: which formats this instance can produce (a caller that wants one format gets a kernel without the other's
// arithmetic and registers; more CTAs then fit an SM, i.e. more loads in flight).
// 16 elements as they arrive from memory (two or four 16-byte pieces), unpacked to fp32 when their tile's turn comes:
// a CTA asks for all its tiles' elements up front and holds them packed (8 registers per run of bf16 / fp16).
template <typename T> struct Raw16 { uint4 q[sizeof(T) == 4 ? 4 : 2]; };
template <typename T> __device__ __forceinline__ void load_raw(const T* p, Raw16<T>& r) {
#pragma unroll
  for (int j = 0; j < (sizeof(T) == 4 ? 4 : 2); ++j) r.q[j] = __ldg(reinterpret_cast<const uint4*>(p) + j);
}
__device__ __forceinline__ void unpack16(const Raw16<__nv_bfloat16>& r, float (&v)[16]) {
  const uint32_t w[8] = {r.q[0].x, r.q[0].y, r.q[0].z, r.q[0].w, r.q[1].x, r.q[1].y, r.q[1].z, r.q[1].w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void unpack16(const Raw16<__half>& r, float (&v)[16]) {
  uint32_t w[8] = {r.q[0].x, r.q[0].y, r.q[0].z, r.q[0].w, r.q[1].x, r.q[1].y, r.q[1].z, r.q[1].w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<__half2*>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void unpack16(const Raw16<float>& r, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[4 * i] = __uint_as_float(r.q[i].x); v[4 * i + 1] = __uint_as_float(r.q[i].y);
    v[4 * i + 2] = __uint_as_float(r.q[i].z); v[4 * i + 3] = __uint_as_float(r.q[i].w);
  }
}
// tiles along L per CTA: twice the loads in flight per SM, half the CTA turn-overs (one tile where the registers are
// needed otherwise: fp32 input, whose packed runs are twice as large, and the rotary variant, which unpacks two runs at once)
template <typename T, bool ROPE> __host__ __device__ constexpr int mx_tiles_per_cta() { return (sizeof(T) == 4 || ROPE) ? 1 : 2; }

template <typename T, bool ROPE, bool W8, bool W4>
__global__ void __launch_bounds__(kMxThreads, 2) quant_mx_kernel(const QuantParams p) {
  constexpr int TPC = mx_tiles_per_cta<T, ROPE>();
  __shared__ __align__(16) uint8_t sf8s[TPC][512];
  __shared__ __align__(16) uint8_t sf4s[TPC][512];
  __shared__ __align__(16) uint8_t rm8s[TPC][512];  // row-major scale codes of the tile: [row][k-block & 3]
  __shared__ __align__(16) uint8_t rm4s[TPC][512];
  const int tile_d = blockIdx.y, bh = blockIdx.z;
  const int b = bh / p.H, h = bh % p.H;
  const int col0 = tile_d * 128;
  const int tid = threadIdx.x;
  const bool want8 = W8 && (p.fp8_codes || p.fp8_scales_rm || p.fp8_scales_tiled);
  const bool want4 = W4 && (p.fp4_codes_unpacked || p.fp4_codes_packed || p.fp4_scales_rm || p.fp4_scales_tiled);

  const T* xb = reinterpret_cast<const T*>(p.x) + (long long)b * p.xs_b + (long long)h * p.xs_h;
  int rls[kMxRuns], cols[kMxRuns];              // row inside the tile and first column of each run
#pragma unroll
  for (int i = 0; i < kMxRuns; ++i) {
    if (ROPE) {
      const int cpr = p.D >> 5;                 // 16-element runs per half row
      rls[i] = tid / cpr;
      cols[i] = (tid % cpr) * 16 + i * (p.D >> 1);
    } else {
      const int g = tid + i * kMxThreads;       // run index inside the tile
      rls[i] = g >> 3;
      cols[i] = col0 + (g & 7) * 16;
    }
  }
  // every load of the CTA goes out before any arithmetic
  Raw16<T> raw[TPC][kMxRuns];
#pragma unroll
  for (int tt = 0; tt < TPC; ++tt) {
#pragma unroll
    for (int i = 0; i < kMxRuns; ++i) {
      const int r = (blockIdx.x * TPC + tt) * 128 + rls[i];
      if ((rls[i] < 128) && (r < p.L) && (cols[i] < p.D)) load_raw<T>(xb + (long long)r * p.xs_l + cols[i], raw[tt][i]);
    }
  }
  // padding of the scale tiles: rows beyond L and k-blocks beyond D carry E8M0 1.0
  for (int i = tid; i < TPC * 256; i += kMxThreads) {
    reinterpret_cast<uint16_t*>(&sf8s[0][0])[i] = 0x7f7f;
    reinterpret_cast<uint16_t*>(&sf4s[0][0])[i] = 0x7f7f;
  }
  __syncthreads();
  const int nblk = p.D >> 5;
  const bool scaled = (p.s != 1.0f);
#pragma unroll
  for (int tt = 0; tt < TPC; ++tt) {
  const int tile_l = blockIdx.x * TPC + tt;
  const int row0 = tile_l * 128;
  if (row0 >= p.L) break;
  uint8_t* sf8 = sf8s[tt]; uint8_t* sf4 = sf4s[tt]; uint8_t* rm8 = rm8s[tt]; uint8_t* rm4 = rm4s[tt];
  float v[kMxRuns][16];
  bool live[kMxRuns];
#pragma unroll
  for (int i = 0; i < kMxRuns; ++i) {
    const int r = row0 + rls[i], c = cols[i];
    live[i] = (rls[i] < 128) && (r < p.L) && (c < p.D);
    if (live[i]) {
      unpack16(raw[tt][i], v[i]);
      if (p.center) {
        // "smooth K": k - mean over the sequence (ours/mxfp_attn_kernel.py:33-34), an elementwise op in the input dtype
        const float4* cen = reinterpret_cast<const float4*>(p.center + ((long long)b * p.H + h) * p.D + c);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 m = __ldg(cen + j);
          v[i][4 * j] = round_as<T>(v[i][4 * j] - m.x);
          v[i][4 * j + 1] = round_as<T>(v[i][4 * j + 1] - m.y);
          v[i][4 * j + 2] = round_as<T>(v[i][4 * j + 2] - m.z);
          v[i][4 * j + 3] = round_as<T>(v[i][4 * j + 3] - m.w);
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[i][j] = 0.0f;
    }
  }
  if (ROPE && live[0]) {
    const long long ang = (long long)b * p.rope_sb + (long long)(row0 + rls[0]) * (p.D >> 1) + cols[0];
    const float4* cs4 = reinterpret_cast<const float4*>(p.rope_cos + ang);
    const float4* sn4 = reinterpret_cast<const float4*>(p.rope_sin + ang);
#pragma unroll
    for (int j4 = 0; j4 < 4; ++j4) {
      const float4 c4 = __ldg(cs4 + j4), s4 = __ldg(sn4 + j4);
      const float co[4] = {c4.x, c4.y, c4.z, c4.w}, si[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int j = 4 * j4 + jj;
        const float x1 = v[0][j], x2 = v[1][j];
        v[0][j] = round_as<T>(__fsub_rn(__fmul_rn(x1, co[jj]), __fmul_rn(x2, si[jj])));
        v[1][j] = round_as<T>(__fadd_rn(__fmul_rn(x2, co[jj]), __fmul_rn(x1, si[jj])));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kMxRuns; ++i) {
    const int rl = rls[i];                  // row inside the tile
    const int r = row0 + rl, c = cols[i];
    float amax = 0.0f;
    if (scaled) {
#pragma unroll
      for (int j = 0; j < 16; ++j) v[i][j] = __fmul_rn(v[i][j], p.s);
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    if (!live[i]) continue;
    const int kb = c >> 5;                  // 32-element block index along D
    const int sf_off = (rl & 31) * 16 + (rl >> 5) * 4 + (kb & 3);
    const bool writer = (tid & 1) == 0;
    const long long row_lin = ((long long)b * p.H + h) * p.L + r;
    if (want8) {
      const BlockScale bs = mx_block_scale(amax, p.fp8_fmt == FMT_FP8_E4M3 ? 8 : 7);
      uint32_t w[4];
      if (bs.zero) {
        w[0] = w[1] = w[2] = w[3] = 0;        // the reference stores the NaN pattern of 0/0 here
      } else if (p.fp8_fmt == FMT_FP8_E4M3) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          w[j] = cvt_fp8x4_regs<true>(v[i][4 * j] * bs.inv_scale, v[i][4 * j + 1] * bs.inv_scale,
                                      v[i][4 * j + 2] * bs.inv_scale, v[i][4 * j + 3] * bs.inv_scale);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          w[j] = cvt_fp8x4_regs<false>(v[i][4 * j] * bs.inv_scale, v[i][4 * j + 1] * bs.inv_scale,
                                       v[i][4 * j + 2] * bs.inv_scale, v[i][4 * j + 3] * bs.inv_scale);
      }
      if (p.fp8_codes) {
        uint8_t* o = p.fp8_codes + (long long)b * p.o8_b + (long long)h * p.o8_h + (long long)r * p.o8_l + c;
        *reinterpret_cast<uint4*>(o) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      if (writer) {
        sf8[sf_off] = bs.code;
        rm8[rl * 4 + (kb & 3)] = bs.code;
      }
    }
    if (want4) {
      const BlockScale bs = mx_block_scale(amax, 3);
      uint32_t lo, hi;                         // 8 nibbles each, element 0 in the low nibble
      if (bs.zero) {
        lo = hi = 0x88888888u;                 // 0/0 in the reference: sign 1, exponent 0, mantissa 0
      } else {
        float y[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) y[j] = fp4_snap_ref(v[i][j] * bs.inv_scale);
        lo = cvt_e2m1x8_regs(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7]);
        hi = cvt_e2m1x8_regs(y[8], y[9], y[10], y[11], y[12], y[13], y[14], y[15]);
      }
      if (p.fp4_codes_unpacked) {
        const uint32_t le = lo & 0x0f0f0f0fu, lod = (lo >> 4) & 0x0f0f0f0fu;
        const uint32_t he = hi & 0x0f0f0f0fu, hod = (hi >> 4) & 0x0f0f0f0fu;
        uint8_t* o = p.fp4_codes_unpacked + (long long)b * p.o4_b + (long long)h * p.o4_h +
                     (long long)r * p.o4_l + c;
        *reinterpret_cast<uint4*>(o) = make_uint4(__byte_perm(le, lod, 0x5140), __byte_perm(le, lod, 0x7362),
                                                  __byte_perm(he, hod, 0x5140), __byte_perm(he, hod, 0x7362));
      }
      if (p.fp4_codes_packed) {
        uint8_t* o = p.fp4_codes_packed + row_lin * (p.D >> 1) + (c >> 1);
        *reinterpret_cast<uint2*>(o) = make_uint2(lo, hi);
      }
      if (writer) {
        sf4[sf_off] = bs.code;
        rm4[rl * 4 + (kb & 3)] = bs.code;
      }
    }
  }
  }  // tiles of the CTA
  __syncthreads();
  // one coalesced 512-byte store per scale tile
  for (int tt = 0; tt < TPC; ++tt) {
  const int tile_l = blockIdx.x * TPC + tt, row0 = tile_l * 128;
  if (row0 >= p.L) break;
  uint8_t* sf8 = sf8s[tt]; uint8_t* sf4 = sf4s[tt]; uint8_t* rm8 = rm8s[tt]; uint8_t* rm4 = rm4s[tt];
  const long long ntl = (p.L + 127) >> 7, ntd = (p.D + 127) >> 7;
  const long long tile_lin = (((long long)b * p.H + h) * ntl + tile_l) * ntd + tile_d;
  if (tid < 32) {
    if (p.fp8_scales_tiled && want8)
      reinterpret_cast<uint4*>(p.fp8_scales_tiled + tile_lin * 512)[tid] = reinterpret_cast<uint4*>(sf8)[tid];
  } else if (tid < 64) {
    if (p.fp4_scales_tiled && want4)
      reinterpret_cast<uint4*>(p.fp4_scales_tiled + tile_lin * 512)[tid - 32] =
          reinterpret_cast<uint4*>(sf4)[tid - 32];
  } else if (tid >= 128 && tid < 384) {
    // row-major scales (the reference's output format): one row of the tile per thread, its up to four codes in one store
    const bool f8 = tid < 256;
    const int rl = tid & 127, r = row0 + rl;
    uint8_t* dst = f8 ? p.fp8_scales_rm : p.fp4_scales_rm;
    if (dst && (f8 ? want8 : want4) && r < p.L) {
      const uint8_t* src = (f8 ? rm8 : rm4) + rl * 4;
      const int kb0 = tile_d * 4, n = min(4, nblk - kb0);
      uint8_t* o = dst + (((long long)b * p.H + h) * p.L + r) * nblk + kb0;
      if (n == 4 && (nblk & 3) == 0) {
        *reinterpret_cast<uint32_t*>(o) = *reinterpret_cast<const uint32_t*>(src);
      } else {
        for (int i = 0; i < n; ++i) o[i] = src[i];
      }
    }
  }
  }  // tiles of the CTA
}

// MXFP8 alone from 16-bit input, no rotary embedding, no centring: the case that has to run at memory speed.  Nothing is
// unpacked to fp32 ahead of its use - the block maximum is taken on the packed 16-bit patterns (for non-negative
// values their order as unsigned integers is their order as numbers, in bf16 and in fp16 alike), which leaves
// registers for THREE tiles of packed loads in flight per CTA.  Same results as quant_mx_kernel: the maximum of the
// rounded products |x|*s is the rounded product of the maximum (rounding is monotonic, s > 0).
template <typename T> __device__ __forceinline__ float pattern_to_float(uint32_t h);
template <> __device__ __forceinline__ float pattern_to_float<__nv_bfloat16>(uint32_t h) { return __uint_as_float(h << 16); }
template <> __device__ __forceinline__ float pattern_to_float<__half>(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)h)); }
template <typename T> __device__ __forceinline__ void unpack2(uint32_t w, float& lo, float& hi);
template <> __device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t w, float& lo, float& hi) {
  lo = __uint_as_float(w << 16);
  hi = __uint_as_float(w & 0xffff0000u);
}
template <> __device__ __forceinline__ void unpack2<__half>(uint32_t w, float& lo, float& hi) {
  const float2 f = __half22float2(*reinterpret_cast<__half2*>(&w));
  lo = f.x;
  hi = f.y;
}
constexpr int kMx8Tiles = 3;

template <typename T>
__global__ void __launch_bounds__(kMxThreads, 2) quant_mx8_kernel(const QuantParams p) {
  constexpr int TPC = kMx8Tiles;
  __shared__ __align__(16) uint8_t sf8s[TPC][512];
  __shared__ __align__(16) uint8_t rm8s[TPC][512];
  const int tile_d = blockIdx.y, bh = blockIdx.z;
  const int b = bh / p.H, h = bh % p.H;
  const int tid = threadIdx.x;
  const int rl0 = tid >> 3;                      // rows rl0 and rl0 + 64 of a tile, 16 columns from c
  const int c = tile_d * 128 + (tid & 7) * 16;
  const T* xb = reinterpret_cast<const T*>(p.x) + (long long)b * p.xs_b + (long long)h * p.xs_h;
  Raw16<T> raw[TPC][2];
#pragma unroll
  for (int tt = 0; tt < TPC; ++tt) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = (blockIdx.x * TPC + tt) * 128 + rl0 + 64 * i;
      if (r < p.L && c < p.D) load_raw<T>(xb + (long long)r * p.xs_l + c, raw[tt][i]);
    }
  }
  for (int i = tid; i < TPC * 256; i += kMxThreads) reinterpret_cast<uint16_t*>(&sf8s[0][0])[i] = 0x7f7f;   // padding: E8M0 1.0
  __syncthreads();
  const int nblk = p.D >> 5;
  const bool scaled = (p.s != 1.0f);
  const bool e4m3 = p.fp8_fmt == FMT_FP8_E4M3;
#pragma unroll
  for (int tt = 0; tt < TPC; ++tt) {
    const int row0 = (blockIdx.x * TPC + tt) * 128;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int rl = rl0 + 64 * i, r = row0 + rl;
      const bool live = r < p.L && c < p.D;
      const uint4 qa = raw[tt][i].q[0], qb = raw[tt][i].q[1];
      const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
      uint32_t m = 0;
      if (live) {
#pragma unroll
        for (int j = 0; j < 8; ++j) m = __vmaxu2(m, w[j] & 0x7fff7fffu);
      }
      m = max(m & 0xffffu, m >> 16);
      float amax = pattern_to_float<T>(m);
      if (scaled) amax = __fmul_rn(amax, p.s);
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      if (!live) continue;
      const BlockScale bs = mx_block_scale(amax, e4m3 ? 8 : 7);
      uint32_t o[4];
      if (bs.zero) {
        o[0] = o[1] = o[2] = o[3] = 0;            // the reference stores the NaN pattern of 0/0 here
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float x0, x1, x2, x3;
          unpack2<T>(w[2 * j], x0, x1);
          unpack2<T>(w[2 * j + 1], x2, x3);
          if (scaled) { x0 = __fmul_rn(x0, p.s); x1 = __fmul_rn(x1, p.s); x2 = __fmul_rn(x2, p.s); x3 = __fmul_rn(x3, p.s); }
          o[j] = e4m3 ? cvt_fp8x4_regs<true>(x0 * bs.inv_scale, x1 * bs.inv_scale, x2 * bs.inv_scale, x3 * bs.inv_scale)
                      : cvt_fp8x4_regs<false>(x0 * bs.inv_scale, x1 * bs.inv_scale, x2 * bs.inv_scale, x3 * bs.inv_scale);
        }
      }
      if (p.fp8_codes) {
        uint8_t* dst = p.fp8_codes + (long long)b * p.o8_b + (long long)h * p.o8_h + (long long)r * p.o8_l + c;
        *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
      }
      if ((tid & 1) == 0) {
        const int kb = c >> 5;
        sf8s[tt][(rl & 31) * 16 + (rl >> 5) * 4 + (kb & 3)] = bs.code;
        rm8s[tt][rl * 4 + (kb & 3)] = bs.code;
      }
    }
  }
  __syncthreads();
  const long long ntl = (p.L + 127) >> 7, ntd = (p.D + 127) >> 7;
  for (int tt = 0; tt < TPC; ++tt) {
    const int tile_l = blockIdx.x * TPC + tt, row0 = tile_l * 128;
    if (row0 >= p.L) break;
    if (tid < 32) {
      if (p.fp8_scales_tiled) {
        const long long tile_lin = (((long long)b * p.H + h) * ntl + tile_l) * ntd + tile_d;
        reinterpret_cast<uint4*>(p.fp8_scales_tiled + tile_lin * 512)[tid] = reinterpret_cast<uint4*>(sf8s[tt])[tid];
      }
    } else if (tid >= 128 && tid < 256) {
      // row-major scales (the reference's output format): one row of the tile per thread, its up to four codes in one store
      const int rl = tid & 127, r = row0 + rl;
      if (p.fp8_scales_rm && r < p.L) {
        const uint8_t* src = rm8s[tt] + rl * 4;
        const int kb0 = tile_d * 4, n = min(4, nblk - kb0);
        uint8_t* dst = p.fp8_scales_rm + (((long long)b * p.H + h) * p.L + r) * nblk + kb0;
        if (n == 4 && (nblk & 3) == 0) {
          *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(src);
        } else {
          for (int j = 0; j < n; ++j) dst[j] = src[j];
        }
      }
    }
  }
}

// ---- per-32 int8 quantizer (ours/quant_mxint8.py:21-58) ------------------------------------
struct QuantI8Params {
  const void* x; int in_dtype; int B, H, L, D;
  long long xs_b, xs_h, xs_l; float s;
  int8_t* codes; long long o_b, o_h, o_l;
  float* scales;   // [B,H,L,D/32]
};

template <typename T>
__global__ void __launch_bounds__(kQuantThreads) quant_i8_kernel(const QuantI8Params p) {
  const int tile_l = blockIdx.x, tile_d = blockIdx.y, bh = blockIdx.z;
  const int b = bh / p.H, h = bh % p.H;
  const int tid = threadIdx.x;
  const T* xb = reinterpret_cast<const T*>(p.x) + (long long)b * p.xs_b + (long long)h * p.xs_h;
#pragma unroll
  for (int i = 0; i < kRunsPerThread; ++i) {
    const int g = tid + i * kQuantThreads;
    const int r = tile_l * 128 + (g >> 3), c = tile_d * 128 + (g & 7) * 16;
    const bool live = (r < p.L) && (c < p.D);
    float v[16];
    if (live) load16<T>(xb + (long long)r * p.xs_l + c, v);
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      v[j] = live ? __fmul_rn(v[j], p.s) : 0.0f;
      amax = fmaxf(amax, fabsf(v[j]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    if (!live) continue;
    const float scale = __fadd_rn(__fdiv_rn(amax, 127.0f), 0.0000001f);
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t q0 = (uint8_t)int8_code_ref(v[4 * j + 0], scale), q1 = (uint8_t)int8_code_ref(v[4 * j + 1], scale);
      uint32_t q2 = (uint8_t)int8_code_ref(v[4 * j + 2], scale), q3 = (uint8_t)int8_code_ref(v[4 * j + 3], scale);
      w[j] = q0 | (q1 << 8) | (q2 << 16) | (q3 << 24);
    }
    int8_t* o = p.codes + (long long)b * p.o_b + (long long)h * p.o_h + (long long)r * p.o_l + c;
    *reinterpret_cast<uint4*>(o) = make_uint4(w[0], w[1], w[2], w[3]);
    if ((tid & 1) == 0) {
      // stored scale goes through an E5M2 round trip (ours/quant_mxint8.py:57)
      __nv_fp8_storage_t s8 = __nv_cvt_float_to_fp8(scale, __NV_SATFINITE, __NV_E5M2);
      __half_raw hr = __nv_cvt_fp8_to_halfraw(s8, __NV_E5M2);
      const long long row_lin = ((long long)b * p.H + h) * p.L + r;
      p.scales[row_lin * (p.D >> 5) + (c >> 5)] = __half2float(__half(hr));
    }
  }
}


// ---- V operand of P.V: 32-key blocks along the SEQUENCE axis, transposed output -------------------
// V [B,H,Skv,D] -> V^T codes [B,H,D,Skv_pad] (MXFP8) and/or [B,H,D,Skv_pad/2] (MXFP4 packed), scale tiles
// [B,H,ceil(Skv/128),512] with rows = head-dim index and columns = the four 32-key blocks of a
// 128-key tile.  Elements are rounded to nearest even (OCP MX rule: shared exponent
// floor(log2(amax)) - emax, emax = 2 for E2M1; the fp8 rule is the same as in quant_mx_kernel).
// The reference has no such quantizer: it keeps V in fp16 (ours/mxfp_attn_kernel.py:29-31).
struct QuantVParams {
  const void* v; int B, H, Skv, D, Skv_pad;
  long long vs_b, vs_h, vs_l;
  int fp8_fmt;
  uint8_t* vt8; uint8_t* vt4; uint8_t* sf8; uint8_t* sf4;
};

__device__ __forceinline__ uint32_t cvt_e2m1x8(const float* y) {
  uint32_t r;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(r)
      : "f"(y[0]), "f"(y[1]), "f"(y[2]), "f"(y[3]), "f"(y[4]), "f"(y[5]), "f"(y[6]), "f"(y[7]));
  return r;
}

template <typename T>
__global__ void __launch_bounds__(256) quant_v_seq_kernel(const QuantVParams p) {
  __shared__ float tile[64][129];                  // [key][d] half tile, padded against bank conflicts
  __shared__ __align__(16) uint8_t s8[512];
  __shared__ __align__(16) uint8_t s4[512];
  const int kt = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int tid = threadIdx.x;
  reinterpret_cast<uint16_t*>(s8)[tid] = 0x7f7f;
  reinterpret_cast<uint16_t*>(s4)[tid] = 0x7f7f;
  const T* src = reinterpret_cast<const T*>(p.v) + (long long)b * p.vs_b + (long long)h * p.vs_h;
  for (int half = 0; half < 2; ++half) {
    const int key0 = kt * 128 + half * 64;
    __syncthreads();
    for (int i = tid; i < 64 * p.D; i += 256) {
      const int kl = i / p.D, d = i % p.D;
      tile[kl][d] = (key0 + kl < p.Skv) ? (float)src[(long long)(key0 + kl) * p.vs_l + d] : 0.0f;
    }
    __syncthreads();
    // one unit = (head-dim index d, 32-key block)
    for (int u = tid; u < p.D * 2; u += 256) {
      const int d = u % p.D, bl = u / p.D, blk = half * 2 + bl;
      float v[32], amax = 0.0f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        v[i] = tile[bl * 32 + i][d];
        amax = fmaxf(amax, fabsf(v[i]));
      }
      const long long row = ((long long)bh * p.D + d);
      const int sf_off = (d & 31) * 16 + (d >> 5) * 4 + blk;
      if (p.vt8) {
        BlockScale bs = mx_block_scale(amax, p.fp8_fmt == FMT_FP8_E4M3 ? 8 : 7);
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint32_t c[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) c[e] = bs.zero ? 0u : fp8_code(v[4 * j + e] * bs.inv_scale, p.fp8_fmt);
          w[j] = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
        }
        uint4* o = reinterpret_cast<uint4*>(p.vt8 + row * p.Skv_pad + key0 + bl * 32);
        o[0] = make_uint4(w[0], w[1], w[2], w[3]);
        o[1] = make_uint4(w[4], w[5], w[6], w[7]);
        s8[sf_off] = bs.code;
      }
      if (p.vt4) {
        BlockScale bs = mx_block_scale(amax, 2);
        float y[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) y[i] = bs.zero ? 0.0f : v[i] * bs.inv_scale;
        uint4 o4 = make_uint4(cvt_e2m1x8(y), cvt_e2m1x8(y + 8), cvt_e2m1x8(y + 16), cvt_e2m1x8(y + 24));
        *reinterpret_cast<uint4*>(p.vt4 + row * (p.Skv_pad >> 1) + ((key0 + bl * 32) >> 1)) = o4;
        s4[sf_off] = bs.code;
      }
    }
  }
  __syncthreads();
  const long long nkt = p.Skv_pad >> 7;
  const long long tile_lin = (long long)bh * nkt + kt;
  if (tid < 32) {
    if (p.sf8) reinterpret_cast<uint4*>(p.sf8 + tile_lin * 512)[tid] = reinterpret_cast<uint4*>(s8)[tid];
  } else if (tid < 64) {
    if (p.sf4) reinterpret_cast<uint4*>(p.sf4 + tile_lin * 512)[tid - 32] = reinterpret_cast<uint4*>(s4)[tid - 32];
  }
}


// The same quantizer for 16-bit input whose rows are 16-byte aligned (the usual case): the whole 128-key tile goes
// through shared memory in the input type with 16-byte loads, all issued up front; a unit of work is (head-dim index d,
// 32-key block) with the block index fastest, so the four lanes of one d write 128 (MXFP8) or 64 (MXFP4) consecutive
// bytes of a V^T row.  Rows of a 32-key block are skewed by 16 bytes per block in shared memory, which keeps the
// column reads of the four blocks in different banks.  Same arithmetic, same results as quant_v_seq_kernel.
template <typename T>
__global__ void __launch_bounds__(256) quant_v_seq_vec_kernel(const QuantVParams p) {
  constexpr int MAXD = 128;
  constexpr int PITCH = MAXD * 2 + 16;             // bytes per key row
  __shared__ __align__(16) uint8_t tile[128 * PITCH + 3 * 16];
  __shared__ __align__(16) uint8_t s8[512];
  __shared__ __align__(16) uint8_t s4[512];
  const int kt = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
  const int tid = threadIdx.x;
  const int key0 = kt * 128;
  const uint8_t* src = reinterpret_cast<const uint8_t*>(p.v) + ((long long)b * p.vs_b + (long long)h * p.vs_h) * 2;
  const int vpr = p.D >> 3;                        // 16-byte vectors per key row
  const int nvec = 128 * vpr;                      // 2048 (D=128) or 1024 (D=64): 8 or 4 per thread
  uint4 ld[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int i = tid + j * 256;
    ld[j] = make_uint4(0, 0, 0, 0);
    if (i < nvec) {
      const int kl = i / vpr, vc = i % vpr;
      if (key0 + kl < p.Skv) ld[j] = __ldg(reinterpret_cast<const uint4*>(src + (long long)(key0 + kl) * p.vs_l * 2) + vc);
    }
  }
  reinterpret_cast<uint16_t*>(s8)[tid] = 0x7f7f;
  reinterpret_cast<uint16_t*>(s4)[tid] = 0x7f7f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int i = tid + j * 256;
    if (i < nvec) {
      const int kl = i / vpr, vc = i % vpr;
      *reinterpret_cast<uint4*>(tile + kl * PITCH + (kl >> 5) * 16 + vc * 16) = ld[j];
    }
  }
  __syncthreads();
  // one unit = (head-dim index d, 32-key block), block index fastest
  for (int u = tid; u < p.D * 4; u += 256) {
    const int blk = u & 3, d = u >> 2;
    float v[32], amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const int kl = blk * 32 + i;
      const T e = *reinterpret_cast<const T*>(tile + kl * PITCH + blk * 16 + d * 2);
      v[i] = (float)e;
      amax = fmaxf(amax, fabsf(v[i]));
    }
    const long long row = ((long long)bh * p.D + d);
    const int sf_off = (d & 31) * 16 + (d >> 5) * 4 + blk;
    if (p.vt8) {
      BlockScale bs = mx_block_scale(amax, p.fp8_fmt == FMT_FP8_E4M3 ? 8 : 7);
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (bs.zero) w[j] = 0;
        else if (p.fp8_fmt == FMT_FP8_E4M3)
          w[j] = cvt_fp8x4_regs<true>(v[4 * j] * bs.inv_scale, v[4 * j + 1] * bs.inv_scale, v[4 * j + 2] * bs.inv_scale, v[4 * j + 3] * bs.inv_scale);
        else
          w[j] = cvt_fp8x4_regs<false>(v[4 * j] * bs.inv_scale, v[4 * j + 1] * bs.inv_scale, v[4 * j + 2] * bs.inv_scale, v[4 * j + 3] * bs.inv_scale);
      }
      uint4* o = reinterpret_cast<uint4*>(p.vt8 + row * p.Skv_pad + key0 + blk * 32);
      o[0] = make_uint4(w[0], w[1], w[2], w[3]);
      o[1] = make_uint4(w[4], w[5], w[6], w[7]);
      s8[sf_off] = bs.code;
    }
    if (p.vt4) {
      BlockScale bs = mx_block_scale(amax, 2);
      float y[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) y[i] = bs.zero ? 0.0f : v[i] * bs.inv_scale;
      uint4 o4 = make_uint4(cvt_e2m1x8(y), cvt_e2m1x8(y + 8), cvt_e2m1x8(y + 16), cvt_e2m1x8(y + 24));
      *reinterpret_cast<uint4*>(p.vt4 + row * (p.Skv_pad >> 1) + ((key0 + blk * 32) >> 1)) = o4;
      s4[sf_off] = bs.code;
    }
  }
  __syncthreads();
  const long long nkt = p.Skv_pad >> 7;
  const long long tile_lin = (long long)bh * nkt + kt;
  if (tid < 32) {
    if (p.sf8) reinterpret_cast<uint4*>(p.sf8 + tile_lin * 512)[tid] = reinterpret_cast<uint4*>(s8)[tid];
  } else if (tid < 64) {
    if (p.sf4) reinterpret_cast<uint4*>(p.sf4 + tile_lin * 512)[tid - 32] = reinterpret_cast<uint4*>(s4)[tid - 32];
  }
}

// ---- NVFP4: 16-element blocks, E4M3 block scales, one fp32 tensor scale ------------------------------
// The reference only has the GEMM mode string for this format (ours/block_scaled_matmul.py:321-324), no
// quantizer.  Definition used here: ts = amax(tensor) / (6 * 448); block scale = e4m3_rne(amax(block) /
// (6 * ts)); element = e2m1_rne(x / (scale * ts)).  Two launches: stage 1 leaves one partial amax per CTA
// in a scratch array (no atomics, nothing to zero), stage 2 reduces the partials and quantises.
struct QuantNvParams {
  const void* x; int rows, cols; long long ld; float s;
  int H; long long xs_b, xs_h;              // batch (blockIdx.z = b * H + h): input strides in elements; 2-D: H = 1, strides 0
  float* scratch; int n_partials;
  uint8_t* codes; long long ldc_bytes;      // [batch, rows, cols/2]
  uint8_t* scales;                          // [batch, ceil(rows/128), cols/64, 512] E4M3 bytes
  float* tensor_scale;
};

template <typename T>
__global__ void __launch_bounds__(kQuantThreads) nvfp4_amax_kernel(const QuantNvParams p) {
  __shared__ float red[kQuantThreads / 32];
  const int tid = threadIdx.x;
  const T* xb = reinterpret_cast<const T*>(p.x) + (blockIdx.z / p.H) * p.xs_b + (blockIdx.z % p.H) * p.xs_h;
  float amax = 0.0f;
  // CTA tile: 128 rows x 512 columns, 16 elements per step and thread
  for (int i = tid; i < 128 * 32; i += kQuantThreads) {
    const int r = blockIdx.x * 128 + (i >> 5), c = blockIdx.y * 512 + (i & 31) * 16;
    if (r < p.rows && c < p.cols) {
      float v[16];
      load16<T>(xb + (long long)r * p.ld + c, v);
#pragma unroll
      for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(__fmul_rn(v[j], p.s)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((tid & 31) == 0) red[tid >> 5] = amax;
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < kQuantThreads / 32; ++w) amax = fmaxf(amax, red[w]);
    p.scratch[(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x] = amax;
  }
}

template <typename T>
__global__ void __launch_bounds__(kQuantThreads) nvfp4_quant_kernel(const QuantNvParams p) {
  __shared__ __align__(16) uint8_t sf[2][512];
  __shared__ float red[kQuantThreads / 32];
  __shared__ float ts_s;
  const int tid = threadIdx.x;
  // tensor amax = max of the partials
  float amax = 0.0f;
  for (int i = tid; i < p.n_partials; i += kQuantThreads) amax = fmaxf(amax, p.scratch[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((tid & 31) == 0) red[tid >> 5] = amax;
  reinterpret_cast<uint32_t*>(&sf[0][0])[tid] = 0;   // 1024 bytes: padding rows carry scale 0
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < kQuantThreads / 32; ++w) amax = fmaxf(amax, red[w]);
    float ts = __fdiv_rn(amax, 2688.0f);              // 6 * 448
    if (ts == 0.0f) ts = 1.0f;
    ts_s = ts;
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) *p.tensor_scale = ts;
  }
  __syncthreads();
  const float ts = ts_s;
  const float denom = __fmul_rn(6.0f, ts);
  const T* xb = reinterpret_cast<const T*>(p.x) + (blockIdx.z / p.H) * p.xs_b + (blockIdx.z % p.H) * p.xs_h;
  uint8_t* codes = p.codes + (long long)blockIdx.z * p.rows * p.ldc_bytes;
  const int row0 = blockIdx.x * 128, col0 = blockIdx.y * 128;
#pragma unroll
  for (int i = 0; i < kRunsPerThread; ++i) {
    const int g = tid + i * kQuantThreads;          // 16-element block index inside the 128x128 tile
    const int rl = g >> 3, r = row0 + rl, c = col0 + (g & 7) * 16;
    if (r >= p.rows || c >= p.cols) continue;
    float v[16], bmax = 0.0f;
    load16<T>(xb + (long long)r * p.ld + c, v);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      v[j] = __fmul_rn(v[j], p.s);
      bmax = fmaxf(bmax, fabsf(v[j]));
    }
    const float ratio = fminf(__fdiv_rn(bmax, denom), 448.0f);
    const __nv_fp8_storage_t s8 = __nv_cvt_float_to_fp8(ratio, __NV_SATFINITE, __NV_E4M3);
    const float sdec = __half2float(__half(__nv_cvt_fp8_to_halfraw(s8, __NV_E4M3)));
    const float scf = __fmul_rn(sdec, ts);
    float y[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) y[j] = (scf == 0.0f) ? 0.0f : __fdiv_rn(v[j], scf);
    *reinterpret_cast<uint2*>(codes + (long long)r * p.ldc_bytes + (c >> 1)) = make_uint2(cvt_e2m1x8(y), cvt_e2m1x8(y + 8));
    const int blk = (g & 7);                        // block inside the tile: chunk blk / 4, column blk % 4
    sf[blk >> 2][(rl & 31) * 16 + (rl >> 5) * 4 + (blk & 3)] = (uint8_t)s8;
  }
  __syncthreads();
  const long long nchunks = p.cols >> 6;
  if (tid < 64) {
    const int ch = tid >> 5;
    const long long chunk = (long long)blockIdx.y * 2 + ch;
    if (chunk < nchunks)
      reinterpret_cast<uint4*>(p.scales + (((long long)blockIdx.z * gridDim.x + blockIdx.x) * nchunks + chunk) * 512)[tid & 31] =
          reinterpret_cast<uint4*>(sf[ch])[tid & 31];
  }
}

}  // namespace mpsa

namespace mpsa {
// ---- mean over the sequence per (batch, head, depth index): the vector "smooth K" subtracts ------------------
// Two launches, fixed summation order: partial column sums of kMeanRows rows per CTA, then their sum / L rounded to
// the input dtype (torch's mean of a 16-bit tensor accumulates in fp32 and returns the input dtype).
constexpr int kMeanRows = 512;
template <typename T>
__global__ void __launch_bounds__(128) col_sum_kernel(const T* x, float* part, int H, int L, int D, long long xs_b,
                                                      long long xs_h, long long xs_l, int nchunk) {
  __shared__ float acc_s[16][128];
  const int chunk = blockIdx.x, col0 = blockIdx.y * 128, bh = blockIdx.z;
  const int b = bh / H, h = bh % H;
  const int c16 = threadIdx.x & 7, rg = threadIdx.x >> 3;      // 8 threads x 16 columns per row, 16 rows per pass
  const int c = col0 + c16 * 16;
  const T* xb = x + (long long)b * xs_b + (long long)h * xs_h;
  float acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
  const int r_end = min(L, (chunk + 1) * kMeanRows);
  if (c < D) {
    for (int r = chunk * kMeanRows + rg; r < r_end; r += 16) {
      float v[16];
      load16<T>(xb + (long long)r * xs_l + c, v);
#pragma unroll
      for (int j = 0; j < 16; ++j) acc[j] += v[j];
    }
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) acc_s[rg][c16 * 16 + j] = acc[j];
  __syncthreads();
  const int col = col0 + threadIdx.x;
  if (col < D) {
    float t = 0.0f;
#pragma unroll
    for (int g = 0; g < 16; ++g) t += acc_s[g][threadIdx.x];
    part[((long long)bh * nchunk + chunk) * D + col] = t;
  }
}

template <typename T>
__global__ void col_mean_finish_kernel(const float* part, float* mean, int L, int D, int nchunk) {
  const int bh = blockIdx.x;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float t = 0.0f;
    for (int ch = 0; ch < nchunk; ++ch) t += part[((long long)bh * nchunk + ch) * D + d];
    mean[(long long)bh * D + d] = round_as<T>(__fdiv_rn(t, (float)L));
  }
}
}  // namespace mpsa

using namespace mpsa;

static int quant_mx_launch(const void* x, int in_dtype, int B, int H, int L, int D, long long xs_b,
                           long long xs_h, long long xs_l, float s, const void* center, const void* rope_cos,
                           const void* rope_sin, long long rope_sb, int fp8_fmt, void* fp8_codes,
                           long long o8_b, long long o8_h, long long o8_l, void* fp4_codes_unpacked,
                           long long o4_b, long long o4_h, long long o4_l, void* fp8_scales_rm,
                           void* fp4_scales_rm, void* fp4_codes_packed, void* fp8_scales_tiled,
                           void* fp4_scales_tiled, void* stream) {
  if (center && ((uintptr_t)center % 16)) return set_error(MPSA_ERR_BAD_ARG, "quant_mx: center must be 16-byte aligned");
  if (rope_cos) {
    if (!rope_sin || center) return set_error(MPSA_ERR_BAD_ARG, "rope_quant_mx: cos and sin go together, and not with a center");
    if (D != 64 && D != 128) return set_error(MPSA_ERR_UNSUPPORTED, "rope_quant_mx: head_dim must be 64 or 128");
    if (((uintptr_t)rope_cos % 16) || ((uintptr_t)rope_sin % 16) || (rope_sb % 4))
      return set_error(MPSA_ERR_BAD_ARG, "rope_quant_mx: cos / sin must be 16-byte aligned");
  }
  if (!x || B <= 0 || H <= 0 || L <= 0 || D <= 0) return set_error(MPSA_ERR_BAD_ARG, "quant_mx: null input or non-positive shape");
  if (D % 32 != 0) return set_error(MPSA_ERR_UNSUPPORTED, "quant_mx: head_dim must be a multiple of 32");
  if (in_dtype < 0 || in_dtype > 2) return set_error(MPSA_ERR_BAD_ARG, "quant_mx: in_dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)");
  if (fp8_fmt != FMT_FP8_E5M2 && fp8_fmt != FMT_FP8_E4M3) return set_error(MPSA_ERR_BAD_ARG, "quant_mx: fp8_fmt must be 1 (E5M2) or 2 (E4M3)");
  const int esz = in_dtype == 2 ? 4 : 2;
  if (((uintptr_t)x % 16) || ((xs_b * esz) % 16) || ((xs_h * esz) % 16) || ((xs_l * esz) % 16))
    return set_error(MPSA_ERR_BAD_ARG, "quant_mx: input base and strides must be 16-byte aligned");
  if ((fp8_codes && (((uintptr_t)fp8_codes | o8_b | o8_h | o8_l) % 16)) ||
      (fp4_codes_unpacked && (((uintptr_t)fp4_codes_unpacked | o4_b | o4_h | o4_l) % 16)) ||
      (fp4_codes_packed && ((uintptr_t)fp4_codes_packed % 16)) ||
      (fp8_scales_tiled && ((uintptr_t)fp8_scales_tiled % 16)) ||
      (fp4_scales_tiled && ((uintptr_t)fp4_scales_tiled % 16)))
    return set_error(MPSA_ERR_BAD_ARG, "quant_mx: output pointers and strides must be 16-byte aligned");
  QuantParams p;
  p.x = x; p.in_dtype = in_dtype; p.B = B; p.H = H; p.L = L; p.D = D;
  p.xs_b = xs_b; p.xs_h = xs_h; p.xs_l = xs_l; p.s = s; p.fp8_fmt = fp8_fmt; p.center = (const float*)center;
  p.rope_cos = (const float*)rope_cos; p.rope_sin = (const float*)rope_sin; p.rope_sb = rope_sb;
  p.fp8_codes = (uint8_t*)fp8_codes; p.o8_b = o8_b; p.o8_h = o8_h; p.o8_l = o8_l;
  p.fp4_codes_unpacked = (uint8_t*)fp4_codes_unpacked; p.o4_b = o4_b; p.o4_h = o4_h; p.o4_l = o4_l;
  p.fp8_scales_rm = (uint8_t*)fp8_scales_rm; p.fp4_scales_rm = (uint8_t*)fp4_scales_rm;
  p.fp4_codes_packed = (uint8_t*)fp4_codes_packed;
  p.fp8_scales_tiled = (uint8_t*)fp8_scales_tiled; p.fp4_scales_tiled = (uint8_t*)fp4_scales_tiled;
  const int tpc = (in_dtype == 2 || rope_cos) ? 1 : 2;     // mx_tiles_per_cta of the instance launched below
  dim3 grid(((L + 127) / 128 + tpc - 1) / tpc, (D + 127) / 128, B * H);
  if (grid.y > 65535 || grid.z > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "quant_mx: B*H and D/128 must be below 65536");
  cudaStream_t st = (cudaStream_t)stream;
  const bool w8 = p.fp8_codes || p.fp8_scales_rm || p.fp8_scales_tiled;
  const bool w4 = p.fp4_codes_unpacked || p.fp4_codes_packed || p.fp4_scales_rm || p.fp4_scales_tiled;
  if (!w8 && !w4) return set_error(MPSA_ERR_BAD_ARG, "quant_mx: no output requested");
  if (w8 && !w4 && !p.rope_cos && !p.center && in_dtype != 2) {
    // MXFP8 alone from bf16 / fp16: the memory-speed kernel, three tiles per CTA
    const dim3 g8(((L + 127) / 128 + kMx8Tiles - 1) / kMx8Tiles, (D + 127) / 128, B * H);
    if (in_dtype == 0) quant_mx8_kernel<__nv_bfloat16><<<g8, kMxThreads, 0, st>>>(p);
    else quant_mx8_kernel<__half><<<g8, kMxThreads, 0, st>>>(p);
    return check_launch("quant_mx");
  }
#define MPSA_QMX(T, ROPE)                                                                       \
  do {                                                                                          \
    if (w8 && w4) quant_mx_kernel<T, ROPE, true, true><<<grid, kMxThreads, 0, st>>>(p);         \
    else if (w8) quant_mx_kernel<T, ROPE, true, false><<<grid, kMxThreads, 0, st>>>(p);         \
    else quant_mx_kernel<T, ROPE, false, true><<<grid, kMxThreads, 0, st>>>(p);                 \
  } while (0)
  if (p.rope_cos) {
    if (in_dtype == 0) MPSA_QMX(__nv_bfloat16, true);
    else if (in_dtype == 1) MPSA_QMX(__half, true);
    else MPSA_QMX(float, true);
  } else {
    if (in_dtype == 0) MPSA_QMX(__nv_bfloat16, false);
    else if (in_dtype == 1) MPSA_QMX(__half, false);
    else MPSA_QMX(float, false);
  }
#undef MPSA_QMX
  return check_launch("quant_mx");
}

extern "C" int mpsa_quant_mx(const void* x, int in_dtype, int B, int H, int L, int D, long long xs_b,
                             long long xs_h, long long xs_l, float s, int fp8_fmt, void* fp8_codes,
                             long long o8_b, long long o8_h, long long o8_l, void* fp4_codes_unpacked,
                             long long o4_b, long long o4_h, long long o4_l, void* fp8_scales_rm,
                             void* fp4_scales_rm, void* fp4_codes_packed, void* fp8_scales_tiled,
                             void* fp4_scales_tiled, void* stream) {
  return quant_mx_launch(x, in_dtype, B, H, L, D, xs_b, xs_h, xs_l, s, nullptr, nullptr, nullptr, 0, fp8_fmt, fp8_codes, o8_b, o8_h, o8_l,
                         fp4_codes_unpacked, o4_b, o4_h, o4_l, fp8_scales_rm, fp4_scales_rm, fp4_codes_packed,
                         fp8_scales_tiled, fp4_scales_tiled, stream);
}

extern "C" int mpsa_quant_mx_centered(const void* x, int in_dtype, int B, int H, int L, int D, long long xs_b,
                                      long long xs_h, long long xs_l, float s, const void* center, int fp8_fmt,
                                      void* fp8_codes, long long o8_b, long long o8_h, long long o8_l,
                                      void* fp4_codes_unpacked, long long o4_b, long long o4_h, long long o4_l,
                                      void* fp8_scales_rm, void* fp4_scales_rm, void* fp4_codes_packed,
                                      void* fp8_scales_tiled, void* fp4_scales_tiled, void* stream) {
  if (!center) return set_error(MPSA_ERR_BAD_ARG, "quant_mx_centered: center is null");
  return quant_mx_launch(x, in_dtype, B, H, L, D, xs_b, xs_h, xs_l, s, center, nullptr, nullptr, 0, fp8_fmt, fp8_codes, o8_b, o8_h, o8_l,
                         fp4_codes_unpacked, o4_b, o4_h, o4_l, fp8_scales_rm, fp4_scales_rm, fp4_codes_packed,
                         fp8_scales_tiled, fp4_scales_tiled, stream);
}

extern "C" int mpsa_rope_quant_mx(const void* x, int in_dtype, int B, int H, int L, int D, long long xs_b,
                                  long long xs_h, long long xs_l, const void* cos, const void* sin, long long rope_sb,
                                  float s, int fp8_fmt, void* fp8_codes, long long o8_b, long long o8_h, long long o8_l,
                                  void* fp4_codes_unpacked, long long o4_b, long long o4_h, long long o4_l,
                                  void* fp8_scales_rm, void* fp4_scales_rm, void* fp4_codes_packed,
                                  void* fp8_scales_tiled, void* fp4_scales_tiled, void* stream) {
  if (!cos || !sin) return set_error(MPSA_ERR_BAD_ARG, "rope_quant_mx: cos or sin is null");
  return quant_mx_launch(x, in_dtype, B, H, L, D, xs_b, xs_h, xs_l, s, nullptr, cos, sin, rope_sb, fp8_fmt, fp8_codes, o8_b,
                         o8_h, o8_l, fp4_codes_unpacked, o4_b, o4_h, o4_l, fp8_scales_rm, fp4_scales_rm, fp4_codes_packed,
                         fp8_scales_tiled, fp4_scales_tiled, stream);
}

extern "C" long long mpsa_col_mean_scratch_floats(int B, int H, int L, int D) {
  return (long long)B * H * ((L + kMeanRows - 1) / kMeanRows) * D;
}

extern "C" int mpsa_col_mean(const void* x, int in_dtype, int B, int H, int L, int D, long long xs_b, long long xs_h,
                             long long xs_l, void* mean, void* scratch, long long scratch_floats, void* stream) {
  if (!x || !mean || !scratch || B <= 0 || H <= 0 || L <= 0 || D <= 0) return set_error(MPSA_ERR_BAD_ARG, "col_mean: null pointer or non-positive shape");
  if (D % 16 != 0) return set_error(MPSA_ERR_UNSUPPORTED, "col_mean: depth must be a multiple of 16");
  if (in_dtype < 0 || in_dtype > 2) return set_error(MPSA_ERR_BAD_ARG, "col_mean: in_dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)");
  const int esz = in_dtype == 2 ? 4 : 2;
  if (((uintptr_t)x % 16) || ((xs_b * esz) % 16) || ((xs_h * esz) % 16) || ((xs_l * esz) % 16))
    return set_error(MPSA_ERR_BAD_ARG, "col_mean: input base and strides must be 16-byte aligned");
  if (scratch_floats < mpsa_col_mean_scratch_floats(B, H, L, D)) return set_error(MPSA_ERR_BAD_ARG, "col_mean: scratch too small");
  const int nchunk = (L + kMeanRows - 1) / kMeanRows;
  dim3 grid(nchunk, (D + 127) / 128, B * H);
  if (grid.y > 65535 || grid.z > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "col_mean: B*H and D/128 must be below 65536");
  cudaStream_t st = (cudaStream_t)stream;
  float* part = (float*)scratch;
  float* m = (float*)mean;
  if (in_dtype == 0) {
    col_sum_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, part, H, L, D, xs_b, xs_h, xs_l, nchunk);
    col_mean_finish_kernel<__nv_bfloat16><<<B * H, 128, 0, st>>>(part, m, L, D, nchunk);
  } else if (in_dtype == 1) {
    col_sum_kernel<__half><<<grid, 128, 0, st>>>((const __half*)x, part, H, L, D, xs_b, xs_h, xs_l, nchunk);
    col_mean_finish_kernel<__half><<<B * H, 128, 0, st>>>(part, m, L, D, nchunk);
  } else {
    col_sum_kernel<float><<<grid, 128, 0, st>>>((const float*)x, part, H, L, D, xs_b, xs_h, xs_l, nchunk);
    col_mean_finish_kernel<float><<<B * H, 128, 0, st>>>(part, m, L, D, nchunk);
  }
  return check_launch("col_mean");
}

extern "C" int mpsa_quant_int8(const void* x, int in_dtype, int B, int H, int L, int D, long long xs_b,
                               long long xs_h, long long xs_l, float s, void* codes, long long o_b,
                               long long o_h, long long o_l, void* scales, void* stream) {
  if (!x || !codes || !scales || B <= 0 || H <= 0 || L <= 0 || D <= 0)
    return set_error(MPSA_ERR_BAD_ARG, "quant_int8: null pointer or non-positive shape");
  if (D % 32 != 0) return set_error(MPSA_ERR_UNSUPPORTED, "quant_int8: head_dim must be a multiple of 32");
  if (in_dtype < 0 || in_dtype > 2) return set_error(MPSA_ERR_BAD_ARG, "quant_int8: bad in_dtype");
  const int esz = in_dtype == 2 ? 4 : 2;
  if (((uintptr_t)x % 16) || ((xs_b * esz) % 16) || ((xs_h * esz) % 16) || ((xs_l * esz) % 16) ||
      (((uintptr_t)codes | o_b | o_h | o_l) % 16))
    return set_error(MPSA_ERR_BAD_ARG, "quant_int8: pointers and strides must be 16-byte aligned");
  QuantI8Params p;
  p.x = x; p.in_dtype = in_dtype; p.B = B; p.H = H; p.L = L; p.D = D;
  p.xs_b = xs_b; p.xs_h = xs_h; p.xs_l = xs_l; p.s = s;
  p.codes = (int8_t*)codes; p.o_b = o_b; p.o_h = o_h; p.o_l = o_l; p.scales = (float*)scales;
  dim3 grid((L + 127) / 128, (D + 127) / 128, B * H);
  if (grid.y > 65535 || grid.z > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "quant_int8: B*H and D/128 must be below 65536");
  cudaStream_t st = (cudaStream_t)stream;
  if (in_dtype == 0) quant_i8_kernel<__nv_bfloat16><<<grid, kQuantThreads, 0, st>>>(p);
  else if (in_dtype == 1) quant_i8_kernel<__half><<<grid, kQuantThreads, 0, st>>>(p);
  else quant_i8_kernel<float><<<grid, kQuantThreads, 0, st>>>(p);
  return check_launch("quant_int8");
}

extern "C" int mpsa_quant_v_seq(const void* v, int in_dtype, int B, int H, int Skv, int D, int Skv_pad, long long vs_b,
                                long long vs_h, long long vs_l, int fp8_fmt, void* vt8, void* v8_sf, void* vt4,
                                void* v4_sf, void* stream) {
  if (!v || B <= 0 || H <= 0 || Skv <= 0) return set_error(MPSA_ERR_BAD_ARG, "quant_v_seq: null input or non-positive shape");
  if (D != 64 && D != 128) return set_error(MPSA_ERR_UNSUPPORTED, "quant_v_seq: head_dim must be 64 or 128");
  if (Skv_pad < Skv || Skv_pad % 128) return set_error(MPSA_ERR_BAD_ARG, "quant_v_seq: Skv_pad must be a multiple of 128, at least Skv");
  if (in_dtype < 0 || in_dtype > 2) return set_error(MPSA_ERR_BAD_ARG, "quant_v_seq: bad in_dtype");
  if (fp8_fmt != FMT_FP8_E5M2 && fp8_fmt != FMT_FP8_E4M3) return set_error(MPSA_ERR_BAD_ARG, "quant_v_seq: fp8_fmt must be 1 (E5M2) or 2 (E4M3)");
  if ((vt8 && !v8_sf) || (vt4 && !v4_sf) || (!vt8 && !vt4)) return set_error(MPSA_ERR_BAD_ARG, "quant_v_seq: codes and scales go together");
  if (((uintptr_t)vt8 | (uintptr_t)vt4 | (uintptr_t)v8_sf | (uintptr_t)v4_sf) % 16)
    return set_error(MPSA_ERR_BAD_ARG, "quant_v_seq: outputs must be 16-byte aligned");
  if (B * H > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "quant_v_seq: B*H must be below 65536");
  QuantVParams p;
  p.v = v; p.B = B; p.H = H; p.Skv = Skv; p.D = D; p.Skv_pad = Skv_pad; p.vs_b = vs_b; p.vs_h = vs_h; p.vs_l = vs_l;
  p.fp8_fmt = fp8_fmt; p.vt8 = (uint8_t*)vt8; p.vt4 = (uint8_t*)vt4; p.sf8 = (uint8_t*)v8_sf; p.sf4 = (uint8_t*)v4_sf;
  dim3 grid(Skv_pad / 128, B * H);
  cudaStream_t st = (cudaStream_t)stream;
  const bool vec = in_dtype != 2 && !((uintptr_t)v % 16) && !((vs_b * 2) % 16) && !((vs_h * 2) % 16) && !((vs_l * 2) % 16);
  if (vec && in_dtype == 0) quant_v_seq_vec_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p);
  else if (vec) quant_v_seq_vec_kernel<__half><<<grid, 256, 0, st>>>(p);
  else if (in_dtype == 0) quant_v_seq_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p);
  else if (in_dtype == 1) quant_v_seq_kernel<__half><<<grid, 256, 0, st>>>(p);
  else quant_v_seq_kernel<float><<<grid, 256, 0, st>>>(p);
  return check_launch("quant_v_seq");
}

static int launch_nvfp4(const void* x, int in_dtype, int rows, int cols, long long ld, float s, float* scratch,
                        long long scratch_floats, void* codes, long long ldc_bytes, void* scales, float* tensor_scale,
                        cudaStream_t st, const char* who, int B = 1, int H = 1, long long xs_b = 0, long long xs_h = 0) {
  if (!x || !codes || !scales || !tensor_scale || !scratch || rows <= 0 || cols <= 0)
    return set_error(MPSA_ERR_BAD_ARG, "%s: null pointer or non-positive shape", who);
  if (cols % 64) return set_error(MPSA_ERR_UNSUPPORTED, "%s: the quantised axis must be a multiple of 64", who);
  if (in_dtype < 0 || in_dtype > 2) return set_error(MPSA_ERR_BAD_ARG, "%s: bad in_dtype", who);
  const int esz = in_dtype == 2 ? 4 : 2;
  if (((uintptr_t)x % 16) || ((ld * esz) % 16) || ((uintptr_t)codes % 8) || (ldc_bytes % 8) || ldc_bytes < cols / 2 ||
      ((uintptr_t)scales % 16))
    return set_error(MPSA_ERR_BAD_ARG, "%s: misaligned pointer or pitch", who);
  if (B <= 0 || H <= 0 || (long long)B * H > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "%s: batch x heads must be in [1, 65535]", who);
  if (((xs_b * esz) % 16) || ((xs_h * esz) % 16)) return set_error(MPSA_ERR_BAD_ARG, "%s: misaligned batch stride", who);
  dim3 g1((rows + 127) / 128, (cols + 511) / 512, B * H), g2((rows + 127) / 128, (cols + 127) / 128, B * H);
  const long long n_partials = (long long)g1.x * g1.y * g1.z;
  if (n_partials > 0x7fffffff) return set_error(MPSA_ERR_UNSUPPORTED, "%s: operand too large", who);
  if (n_partials > scratch_floats)
    return set_error(MPSA_ERR_UNSUPPORTED, "%s: needs %lld floats of scratch, %lld available", who, n_partials, scratch_floats);
  if (g1.y > 65535 || g2.y > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "%s: too many columns", who);
  QuantNvParams p;
  p.x = x; p.rows = rows; p.cols = cols; p.ld = ld; p.s = s; p.scratch = scratch; p.n_partials = (int)n_partials;
  p.codes = (uint8_t*)codes; p.ldc_bytes = ldc_bytes; p.scales = (uint8_t*)scales; p.tensor_scale = tensor_scale;
  p.H = H; p.xs_b = xs_b; p.xs_h = xs_h;
  if (in_dtype == 0) { nvfp4_amax_kernel<__nv_bfloat16><<<g1, kQuantThreads, 0, st>>>(p); nvfp4_quant_kernel<__nv_bfloat16><<<g2, kQuantThreads, 0, st>>>(p); }
  else if (in_dtype == 1) { nvfp4_amax_kernel<__half><<<g1, kQuantThreads, 0, st>>>(p); nvfp4_quant_kernel<__half><<<g2, kQuantThreads, 0, st>>>(p); }
  else { nvfp4_amax_kernel<float><<<g1, kQuantThreads, 0, st>>>(p); nvfp4_quant_kernel<float><<<g2, kQuantThreads, 0, st>>>(p); }
  return check_launch(who);
}

extern "C" int mpsa_quant_nvfp4_scratch_floats(int rows, int cols) {
  const long long n = (long long)((rows + 127) / 128) * ((cols + 511) / 512);
  return n > 0x7fffffff ? -2 : (int)n;
}

extern "C" int mpsa_quant_nvfp4(const void* x, int in_dtype, int rows, int cols, long long ld, float s, void* scratch,
                                long long scratch_floats, void* codes, long long ldc_bytes, void* scales,
                                void* tensor_scale, void* stream) {
  return launch_nvfp4(x, in_dtype, rows, cols, ld, s, (float*)scratch, scratch_floats, codes, ldc_bytes, scales,
                      (float*)tensor_scale, (cudaStream_t)stream, "quant_nvfp4");
}

extern "C" int mpsa_quant_nvfp4_bh(const void* x, int in_dtype, int B, int H, int L, int D, long long xs_b, long long xs_h,
                                   long long xs_l, float s, void* scratch, long long scratch_floats, void* codes,
                                   void* scales, void* tensor_scale, void* stream) {
  if (L <= 0 || D <= 0) return set_error(MPSA_ERR_BAD_ARG, "quant_nvfp4_bh: non-positive shape");
  return launch_nvfp4(x, in_dtype, L, D, xs_l, s, (float*)scratch, scratch_floats, codes, D / 2, scales,
                      (float*)tensor_scale, (cudaStream_t)stream, "quant_nvfp4_bh", B, H, xs_b, xs_h);
}

// ---- NVFP4 quantizer for callers that must not allocate ------------------------------------------------
// Some hosts of this library cannot obtain the scratch array the two-stage NVFP4 quantizer needs: a
// serving process that gave its whole memory budget to its own pool at start-up, a plugin that is not
// allowed to call the CUDA allocator on the request path, a C host with no allocator wrapper at all.
// For them the partial maxima live in a fixed array inside this library's device image.  Every GPU that
// loads the library carries these 64 KB until the process exits.
constexpr int kStaticScratchFloats = 16384;            // one partial per 128x512 input tile
static __device__ __align__(256) float g_nvfp4_scratch[kStaticScratchFloats];

extern "C" int mpsa_quant_nvfp4_static(const void* x, int in_dtype, int rows, int cols, long long ld, float s,
                                       void* codes, long long ldc_bytes, void* scales, void* tensor_scale,
                                       void* stream) {
  // In host code the array's name only stands for the symbol; its device address has to be asked for,
  // once per device, with that device current.  The first call on a device does it.
  constexpr int kMaxDevices = 64;
  static float* scratch_of[kMaxDevices] = {};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return set_error(MPSA_ERR_LAUNCH, "quant_nvfp4_static: cannot identify the current device");
  float* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!scratch_of[dev]) {
      float* ptr = nullptr;
      const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_nvfp4_scratch);
      if (e != cudaSuccess || !ptr)
        return set_error(MPSA_ERR_LAUNCH, "quant_nvfp4_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      scratch_of[dev] = ptr;
    }
    scratch = scratch_of[dev];
  }
  if (rows > 0 && cols > 0) {
    const long long need = (long long)((rows + 127) / 128) * ((cols + 511) / 512);
    if (need > kStaticScratchFloats)
      return set_error(MPSA_ERR_UNSUPPORTED,
                       "quant_nvfp4_static: a %d x %d operand needs %lld partial maxima, the built-in scratch holds %d "
                       "(about 1e9 elements); use mpsa_quant_nvfp4 with caller-provided scratch",
                       rows, cols, need, kStaticScratchFloats);
  }
  return launch_nvfp4(x, in_dtype, rows, cols, ld, s, scratch, kStaticScratchFloats, codes, ldc_bytes, scales,
                      (float*)tensor_scale, (cudaStream_t)stream, "quant_nvfp4_static");
}
