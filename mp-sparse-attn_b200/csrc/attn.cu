// Fused diagonal-tiled mixed-precision attention forward for sm_100a.
//
// Counterpart of block_scaled_batched_attn_kernel (ours/mxfp_attn_kernel.py:103-359) with the parts
// the reference leaves out: causal masking and GQA (taken from its INT8 sibling,
// ours/online_routing.py:68-77, :113-118, :160) and a per-tile precision map.
//
// One CTA owns one 128-row query tile of one (batch, q-head) and walks the 128-key tiles the
// precision map enables for it:
//   S = Q.K^T   tcgen05.mma block-scaled: kind::mxf8f6f4 (MXFP8 x MXFP8, 4 x K=32) on FP8 tiles,
//               kind::mxf4 (MXFP4 x MXFP4, 2 x K=64) on FP4 tiles; Q is resident in shared memory
//               in both formats, K tiles arrive by TMA in the format the map asks for; E8M0 scale
//               tiles go to TMEM with tcgen05.cp.  The softmax scale * log2(e) is already folded
//               into Q by the quantizer (ours/quant_mxint8.py:494), so S is in the log2 domain.
//   softmax     one thread per query row reads its S row from TMEM (tcgen05.ld), keeps running
//               max / sum (ours/mxfp_attn_kernel.py:320-328), writes P as fp16 back into TMEM over S
//               (:339).  The accumulator is rescaled only when the running max grows by more than
//               2^8, which leaves the result O = sum(P.V) / sum(P) unchanged.
//   O += P.V    pv_mode 0 (the reference's precision): tcgen05.mma kind::f16 with P (fp16) read from
//               TMEM and V^T (fp16, [D, keys]) from shared memory, fp32 accumulation in TMEM (:340
//               accumulates each tile in fp16 first).  pv_mode 1: P is re-quantised to the tile's
//               format (MXFP8 or MXFP4, one E8M0 scale per 32 keys, written by the softmax threads)
//               and multiplied with V quantised along the sequence, as block-scaled MMAs with P in
//               TMEM (its own columns, so that Q.K^T of tile t+2 can be issued before P.V of tile t); the
//               row reference is kept integral so that the codes do not depend on it.  By default the
//               reference is fixed after the first key tile (template parameter LAZY, see the kernel).
// Roles: warp 0 TMA loads (Q once, then a K ring and a V ring), warp 1 Q.K^T issuer, warp 2 P.V issuer (quantised
// P.V; with fp16 P.V warp 1 issues both products, in order, because P then overwrites S), warp 3 router (ROUTE
// kernels), warps 4.. softmax / correction / epilogue (a warp reaches the TMEM lane quarter warp % 4, so any four
// consecutive warps cover the 128 rows).  Every role walks the CTA's visit list - the non-skipped cells of its map row,
// compacted once into shared memory; in ROUTE kernels the router appends the tiles it promotes, as MXFP8 tiles, and the
// roles walk those in a second phase once the router has been through the row.  The issuing threads' loops hold nothing but their waits, the scale copies, the
// MMAs and the commits (measured: 64 cycles per MXFP4 MMA, ~48 per scale copy, ~44 per commit; a loop that also
// searched the map and derived ring slots by division took ~2000 cycles per tile and bound the whole kernel).  S is
// double-buffered in TMEM so that Q.K^T of tile t+2 overlaps the softmax of tile t.  NWG softmax
// warpgroups take the key tiles in turn (warpgroup w owns tiles t = w mod NWG), so that the
// exponentials of one tile (MUFU) overlap the max / pack / TMEM traffic of the next; the running
// row maximum is handed from the owner of tile t to the owner of tile t+1 through shared memory.
// Inside a warpgroup the 128 keys of a tile can further be split over NSPLIT threads per query row,
// which exchange partial row maxima.  Every thread keeps a partial row sum; the epilogue adds them.
// TMEM columns: S0/P0 [0,128) S1/P1 [128,256) O [256,384) Q scales [384,392) K scales [392,400)
// P scales [400,408) V scales [408,416); with NVFP4 score tiles: Q scales [416,424) K scales [424,440);
// quantised P [448,512) (two buffers; fp16 P overwrites S in place instead).
#include "api_internal.h"
#include "common.cuh"
#include "tma_host.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstdlib>
#include <mutex>

namespace mpsa {

constexpr int ATT_BM = 128, ATT_BN = 128, ATT_DQK = 128;
constexpr int ATT_KSTAGES = 4;                        // K ring
constexpr int ATT_VSLOTS_MAX = 4;                     // V ring: 2 slots of 32 KB (fp16 V^T) or 4 of 16 KB (quantised V^T)
constexpr int ATT_Q8_BYTES = ATT_BM * 128, ATT_Q4_BYTES = ATT_BM * 64;
constexpr int ATT_K_BYTES = ATT_BN * 128;             // slot sized for the FP8 tile; FP4 uses half
constexpr int ATT_V_BYTES = 128 * ATT_BN * 2;         // V^T tile, up to D=128 rows of 128 fp16
constexpr int ATT_OFF_Q8 = 0;
constexpr int ATT_OFF_Q4 = ATT_OFF_Q8 + ATT_Q8_BYTES;
constexpr int ATT_OFF_K = ATT_OFF_Q4 + ATT_Q4_BYTES;
constexpr int ATT_OFF_V = ATT_OFF_K + ATT_KSTAGES * ATT_K_BYTES;
constexpr int ATT_OFF_SF = ATT_OFF_V + 2 * ATT_V_BYTES;   // scale tiles: Q8 (512 B), Q4 (1024), K[stages] (1024 each;
                                                                    // an NVFP4 operand has two 128x4 tiles per 128 rows)
constexpr int ATT_MAX_SPLIT = 4, ATT_MAX_WG = 2;
constexpr int ATT_SERVICE_THREADS = 128;              // warp 0 TMA loads, warp 1 Q.K^T issuer, warp 2 P.V issuer, warp 3 router
constexpr int ATT_OFF_PSF = ATT_OFF_SF + (3 + 2 * ATT_KSTAGES) * 512;    // P scale tiles [2], V scale tiles [VSTAGES]
constexpr int ATT_OFF_XMAX = ATT_OFF_PSF + (2 + ATT_VSLOTS_MAX) * 512;   // float [WG][2][SPLIT][128] partial row maxima
constexpr int ATT_OFF_XSUM = ATT_OFF_XMAX + ATT_MAX_WG * 2 * ATT_MAX_SPLIT * 128 * 4;   // float [WG*SPLIT][128] partial sums
constexpr int ATT_OFF_MROW = ATT_OFF_XSUM + ATT_MAX_WG * ATT_MAX_SPLIT * 128 * 4;       // float [3][128] running row max: per tile parity, and an unsynchronised hint
constexpr int ATT_OFF_RMAX = ATT_OFF_MROW + 3 * 128 * 4;               // float [2 buffers][MAX_SPLIT][128]: slice maxima for the router
constexpr int ATT_OFF_BAR = ATT_OFF_RMAX + 2 * ATT_MAX_SPLIT * 128 * 4;
constexpr int ATT_BAR_BYTES = 1024;                                   // mbarriers, then the TMEM slot, the visit count and the router's words
constexpr int ATT_NUM_BARS = 1 + 2 * ATT_KSTAGES + 2 * ATT_VSLOTS_MAX + 6 + ATT_MAX_WG * 8 + 8 + 4 + 6;
static_assert(ATT_NUM_BARS * 8 + 4 + 4 + 16 + 8 <= ATT_BAR_BYTES, "the barrier block does not fit its share of shared memory");
constexpr int ATT_OFF_MAP = ATT_OFF_BAR + ATT_BAR_BYTES;              // this CTA's row of the precision map
constexpr int ATT_MAP_SMEM = 8192;                                    // longest row: 8192 key tiles (1M keys)
constexpr int ATT_OFF_VLIST = ATT_OFF_MAP + ATT_MAP_SMEM;             // uint16 per visited tile
constexpr int ATT_SMEM = ATT_OFF_VLIST + 2 * ATT_MAP_SMEM + 1024;
static_assert(ATT_SMEM <= 232448, "more shared memory than a CTA can have");
constexpr uint32_t ATT_TMEM_COLS = 512;
constexpr uint32_t ATT_COL_S = 0, ATT_COL_O = 256, ATT_COL_SFQ8 = 384, ATT_COL_SFQ4 = 388, ATT_COL_SFK = 392;
constexpr uint32_t ATT_COL_SFP = 400, ATT_COL_SFV = 408;
constexpr uint32_t ATT_COL_SFQN = 416, ATT_COL_SFKN = 424;        // NVFP4 scales: Q 8 columns, K 2 x 8
constexpr uint32_t ATT_COL_P = 448;                              // quantised P: 2 buffers of 32 columns (128 keys x 1 byte)
constexpr float ATT_RESCALE_LOG2 = 8.0f;
#ifndef ATT_POLY_PER_BLOCK
#define ATT_POLY_PER_BLOCK 4                          // of the 32 exponentials of a block (fixed-reference kernel, MXFP4 tiles)
#endif
constexpr float ATT_LAZY_HEADROOM = 64.0f;            // log2: P up to 2^64 relative to the fixed reference stays far from fp32 overflow

constexpr int TILE_SKIP = 0, TILE_FP8 = 1, TILE_FP4 = 2;

struct AttnParams {
  int B, Hq, Hkv, S, Skv, D;        // D = value head dim (64 or 128); Q/K depth is padded to 128
  int causal;
  int fp8_fmt;                       // descriptor format field: 0 E4M3, 1 E5M2
  const uint8_t* q8_sf; const uint8_t* q4_sf;   // [B,Hq,nq,512]
  const uint8_t* k8_sf; const uint8_t* k4_sf;   // [B,Hkv,nk,512]
  const uint8_t* v8_sf; const uint8_t* v4_sf;   // [B,Hkv,nk,512] (pv_mode 1)
  int pv_mode;                       // 0: P and V in fp16; 1: P and V in the tile's MX format
  int v_tiles;                       // 128-key scale tiles per head in v8_sf / v4_sf (= Skv_pad / 128)
  float fp4_scale;                   // NVFP4 score tiles: product of the tensor scales of Q and K
  const uint8_t* map; long long map_sb, map_sh; // [.., nq, nk], strides may be 0 (broadcast)
  void* out; int out_dtype;          // [B,Hq,S,D] contiguous; 0 f32, 1 f16, 2 bf16
  float* lse;                        // optional [B,Hq,S]: log2 of the softmax denominator (incl. the row reference)
  const void* acc_in;                // optional [B,Hq,S,D] (acc_dtype) + lse_in [B,Hq,S]: an earlier partial result over OTHER keys;
  const float* lse_in;               // the kernel then writes the merged result (lse is required); may alias out / lse: each
  int acc_dtype;                     // thread reads its own elements before it writes them.  acc_dtype: 0 f32, 1 f16, 2 bf16
  // router inside the forward (ROUTE kernels): an MXFP4 tile whose statistic reaches tau x that of the row's first key
  // tile gets no P.V and no share of the row sum; it is marked TILE_FP8 in map_rw, appended to the CTA's visit list and
  // done again in MXFP8 after the row's own tiles.
  float tau;
  uint8_t* map_rw;                   // the map again, writable (same buffer and strides as `map`)
  float* stat_out;                   // optional [B,Hq,nq,nk]: the statistic of every MXFP4 tile visited
  int* range_flag;                   // LAZY kernels: set to 1 when a score leaves the fixed reference's headroom
  const int* run_if;                 // when given: the kernel does nothing unless this word is non-zero
  int* status;
};

__device__ __forceinline__ void tmem_ld32p(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32p(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16p(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ void tmem_st8p(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
               "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st4p(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]),
               "r"(r[2]), "r"(r[3])
               : "memory");
}
// Block-scaled MMAs with the A operand (P) in TMEM.
__device__ __forceinline__ void mma_mxf8f6f4_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t sfa,
                                                uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.scale_vec::1X [%0], [%1], %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_mxf4_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t sfa,
                                            uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], [%1], %2, %3, [%4], [%5], p;\n\t}"
      ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}
// 8 floats -> 8 E2M1 codes (round to nearest even, saturating), element 0 in the low nibble.
__device__ __forceinline__ uint32_t pack_e2m1x8(float y0, float y1, float y2, float y3, float y4, float y5, float y6,
                                                float y7) {
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
// 4 floats -> 4 fp8 codes (E5M2 or E4M3, round to nearest even, saturating), element 0 in the low byte.
template <bool E4M3>
__device__ __forceinline__ uint32_t pack_fp8x4(float y0, float y1, float y2, float y3) {
  uint32_t r;
  if (E4M3) {
    asm("{\n\t.reg .b16 lo, hi;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
        "mov.b32 %0, {lo, hi};\n\t}"
        : "=r"(r) : "f"(y0), "f"(y1), "f"(y2), "f"(y3));
  } else {
    asm("{\n\t.reg .b16 lo, hi;\n\t"
        "cvt.rn.satfinite.e5m2x2.f32 lo, %2, %1;\n\t"
        "cvt.rn.satfinite.e5m2x2.f32 hi, %4, %3;\n\t"
        "mov.b32 %0, {lo, hi};\n\t}"
        : "=r"(r) : "f"(y0), "f"(y1), "f"(y2), "f"(y3));
  }
  return r;
}

// Maximum of 32 scores with the three-input max: 16 instructions in four independent chains.
__device__ __forceinline__ float max3f(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float block_max32(const uint32_t* sc) {
  float b0 = __uint_as_float(sc[0]), b1 = __uint_as_float(sc[1]), b2 = __uint_as_float(sc[2]), b3 = __uint_as_float(sc[3]);
#pragma unroll
  for (int i = 4; i < 28; i += 8) {
    b0 = max3f(b0, __uint_as_float(sc[i]), __uint_as_float(sc[i + 1]));
    b1 = max3f(b1, __uint_as_float(sc[i + 2]), __uint_as_float(sc[i + 3]));
    b2 = max3f(b2, __uint_as_float(sc[i + 4]), __uint_as_float(sc[i + 5]));
    b3 = max3f(b3, __uint_as_float(sc[i + 6]), __uint_as_float(sc[i + 7]));
  }
  b0 = max3f(b0, __uint_as_float(sc[28]), __uint_as_float(sc[29]));
  b1 = max3f(b1, __uint_as_float(sc[30]), __uint_as_float(sc[31]));
  return fmaxf(max3f(b0, b1, b2), b3);
}

// Packed fp32 pairs (one instruction for two lanes of arithmetic): (a, b) += (c, d) and (a, b) = (c, d) - (e, e).
__device__ __forceinline__ void add2(float& a, float& b, float c, float d) {
  asm("{\n\t.reg .b64 x, y;\n\tmov.b64 x, {%0, %1};\n\tmov.b64 y, {%2, %3};\n\tadd.rn.f32x2 x, x, y;\n\tmov.b64 {%0, %1}, x;\n\t}"
      : "+f"(a), "+f"(b) : "f"(c), "f"(d));
}
__device__ __forceinline__ void sub2(float& a, float& b, float c, float d, float neg_e) {
  asm("{\n\t.reg .b64 x, y;\n\tmov.b64 x, {%2, %3};\n\tmov.b64 y, {%4, %4};\n\tadd.rn.f32x2 x, x, y;\n\tmov.b64 {%0, %1}, x;\n\t}"
      : "=f"(a), "=f"(b) : "f"(c), "f"(d), "f"(neg_e));
}

// One 32-key block of one query row: P = exp2(S - m) in the precision the P.V product uses.
//   PMODE 0: fp16 pairs (16 words).  PMODE 1/2: MXFP8 E5M2/E4M3 (8 words), PMODE 3: MXFP4 (4 words), with the
//   block's E8M0 scale code returned: shared exponent floor(log2(amax P)) - emax = floor(bmax - m) - emax,
//   folded into the exponent so that exp2 delivers P / scale directly (power-of-two scaling is exact).
//   `lsum` accumulates the unrounded P (the reference sums P before rounding it, ours/mxfp_attn_kernel.py:325).
template <int PMODE>
__device__ __forceinline__ uint32_t softmax_block(const uint32_t* sc, float mref, float bmax, uint32_t* pk,
                                                  float& lsum0, float& lsum1) {
  if (PMODE == 0) {
    const float nm = -mref;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float x0, x1;
      sub2(x0, x1, __uint_as_float(sc[2 * i]), __uint_as_float(sc[2 * i + 1]), nm);
      const float p0 = ex2(x0);
      const float p1 = ex2(x1);
      add2(lsum0, lsum1, p0, p1);
      pk[i] = pack_f16x2(p0, p1);
    }
    return 0;
  } else {
    constexpr int EMAX = (PMODE == 3) ? 2 : ((PMODE == 2) ? 8 : 7);
    if (bmax == -INFINITY) {                      // nothing visible in this block
      constexpr int NW = (PMODE == 3) ? 4 : 8;
#pragma unroll
      for (int i = 0; i < NW; ++i) pk[i] = 0;
      return 0;
    }
    int sh = (int)floorf(bmax - mref) - EMAX;
    sh = max(sh, -126);
    const float cb = mref + (float)sh;            // exact: mref is integral in this mode
    float y[32];
    float a0 = 0.0f, a1 = 0.0f;
    const float ncb = -cb;
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float x0, x1;
      sub2(x0, x1, __uint_as_float(sc[i]), __uint_as_float(sc[i + 1]), ncb);
      y[i] = ex2(x0);
      y[i + 1] = ex2(x1);
      add2(a0, a1, y[i], y[i + 1]);
    }
    const float two_sh = __uint_as_float((uint32_t)(sh + 127) << 23);
    lsum0 = fmaf(a0, two_sh, lsum0);
    lsum1 = fmaf(a1, two_sh, lsum1);
    if (PMODE == 3) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        pk[i] = pack_e2m1x8(y[8 * i], y[8 * i + 1], y[8 * i + 2], y[8 * i + 3], y[8 * i + 4], y[8 * i + 5], y[8 * i + 6], y[8 * i + 7]);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) pk[i] = pack_fp8x4<PMODE == 2>(y[4 * i], y[4 * i + 1], y[4 * i + 2], y[4 * i + 3]);
    }
    return (uint32_t)(sh + 127);
  }
}

// 2^x for a pair of values on the FMA pipe, for the share of the exponentials taken off the special-function unit:
// x = n + f with n = round(x) (adding 1.5 * 2^23 leaves n in the low mantissa bits), 2^f on [-0.5, 0.5] by a degree-4
// polynomial (relative error 8e-6, far below half a step of any P format), 2^n by adding n to the exponent field.
// x is clamped at -125: anything smaller is zero in every P format.
__device__ __forceinline__ void fma2(float& a, float& b, float c, float d, float e) {   // (a, b) = (a, b) * (c, d) + (e, e)
  asm("{\n\t.reg .b64 x, y, z;\n\tmov.b64 x, {%0, %1};\n\tmov.b64 y, {%2, %3};\n\tmov.b64 z, {%4, %4};\n\t"
      "fma.rn.f32x2 x, x, y, z;\n\tmov.b64 {%0, %1}, x;\n\t}"
      : "+f"(a), "+f"(b) : "f"(c), "f"(d), "f"(e));
}
__device__ __forceinline__ void ex2_poly2(float& y0, float& y1, float x0, float x1) {
  x0 = fmaxf(x0, -125.0f);
  x1 = fmaxf(x1, -125.0f);
  float t0, t1, n0, n1;
  sub2(t0, t1, x0, x1, 12582912.0f);              // t = x + 1.5 * 2^23
  sub2(n0, n1, t0, t1, -12582912.0f);             // n = round(x), as a float
  float f0 = x0 - n0, f1 = x1 - n1;
  float p0 = 0.009278289f, p1 = 0.009278289f;
  fma2(p0, p1, f0, f1, 0.055865023f);
  fma2(p0, p1, f0, f1, 0.240308955f);
  fma2(p0, p1, f0, f1, 0.693129539f);
  fma2(p0, p1, f0, f1, 0.999997854f);
  y0 = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  y1 = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

// Bounded wait for a tagged word in shared memory: returns the word once its tag (bits 1..) equals `tag`, or -1 after
// the limit (status set) or when another role has already recorded a failure.  The status word and the clock are looked
// at every 1024 probes only.
__device__ __forceinline__ int poll_tag(volatile int* word, int tag, int* status) {
  int w = *word;
  if ((w >> 1) == tag) return w;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    w = *word;
    if ((w >> 1) == tag) return w;
    if ((++spins & 0x3ff) == 0) {
      if (*(volatile int*)status != KS_OK) return -1;
      if (clock64() - t0 > kWaitLimitCycles) { atomicCAS(status, KS_OK, KS_TIMEOUT_PIPE); return -1; }
    }
  }
}

// floor(d) - emax as an integer and as a float, without conversion instructions (which share the exponential's
// pipe): d + 1.5 * 2^23 rounded DOWN holds floor(d) in its low mantissa bits (|d| < 2^22).
__device__ __forceinline__ int block_shift(float d, int emax, float& sh_f) {
  const float t = __fadd_rd(fmaxf(d, -1024.0f), 12582912.0f);
  const int sh = max(__float_as_int(t) - 0x4b400000 - emax, -126);
  sh_f = fmaxf(t - 12582912.0f - (float)emax, -126.0f);
  return sh;
}

// One 32-key block of a query row for the quantised P.V (the fixed-reference kernel's form of softmax_block<1..3>:
// same arithmetic, no conversion instructions for the block exponent).
template <int PMODE>
__device__ __forceinline__ uint32_t softmax_block_q(const uint32_t* sc, float mref, float bmax, uint32_t* pk,
                                                    float& lsum0, float& lsum1) {
  constexpr int EMAX = (PMODE == 3) ? 2 : ((PMODE == 2) ? 8 : 7);
  constexpr int NW = (PMODE == 3) ? 4 : 8;
  if (bmax == -INFINITY) {                        // nothing visible in this block
#pragma unroll
    for (int i = 0; i < NW; ++i) pk[i] = 0;
    return 0;
  }
  float sh_f;
  const int sh = block_shift(bmax - mref, EMAX, sh_f);
  const float ncb = -(mref + sh_f);               // exact: mref is integral in this mode
  // Three passes over the block, each of independent instructions (the values are rewritten in place): all
  // subtractions, then all exponentials back to back - a warp then keeps its share of the exponential unit busy
  // without waiting for results - then the sums and the packing.
  float y[32];
#pragma unroll
  for (int i = 0; i < 32; i += 2) sub2(y[i], y[i + 1], __uint_as_float(sc[i]), __uint_as_float(sc[i + 1]), ncb);
  // MXFP4 tiles (nearly all of them): a few of the exponentials are computed on the FMA pipe instead (measured
  // at S=32768: 4 of 32 is the best split; 8 or more lose to the extra instructions)
  constexpr int NPOLY = (PMODE == 3) ? ATT_POLY_PER_BLOCK : 0;
#pragma unroll
  for (int i = 0; i < 32 - NPOLY; ++i) y[i] = ex2(y[i]);
#pragma unroll
  for (int i = 32 - NPOLY; i < 32; i += 2) ex2_poly2(y[i], y[i + 1], y[i], y[i + 1]);
  float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    add2(a0, a1, y[i], y[i + 1]);
    add2(b0, b1, y[i + 2], y[i + 3]);
  }
  a0 += b0;
  a1 += b1;
#pragma unroll
  for (int w = 0; w < NW; ++w) {
    constexpr int E = 32 / NW;                    // elements per word
    if (PMODE == 3) pk[w] = pack_e2m1x8(y[w * E], y[w * E + 1], y[w * E + 2], y[w * E + 3], y[w * E + (E > 4 ? 4 : 0)], y[w * E + (E > 4 ? 5 : 1)],
                                        y[w * E + (E > 4 ? 6 : 2)], y[w * E + (E > 4 ? 7 : 3)]);
    else pk[w] = pack_fp8x4<PMODE == 2>(y[w * E], y[w * E + 1], y[w * E + 2], y[w * E + 3]);
  }
  const float two_sh = __uint_as_float((uint32_t)(sh + 127) << 23);
  lsum0 = fmaf(a0, two_sh, lsum0);
  lsum1 = fmaf(a1, two_sh, lsum1);
  return (uint32_t)(sh + 127);
}


// NVF4: the FP4 tiles of Q.K^T are NVFP4 (16-element blocks, E4M3 scales, kind::mxf4nvf4) instead of MXFP4; their
// scores are multiplied by the product of the two tensor scales before the softmax.
// LAZY (quantised P.V only): the row reference is fixed after the first key tile.  Block-scaled P carries its
// magnitude in E8M0 scale codes, so P, O and the row sums may exceed 1 by up to 2^ATT_LAZY_HEADROOM without loss; then
// no tile after the first needs the row maximum agreed between threads, the reference handed over between
// warpgroups, a second look at S or a rescale of O, and S is released as soon as it has been read.  A score beyond
// the headroom sets *range_flag; the launcher then re-runs the exact kernel, which is launched behind this one with
// run_if = range_flag.
// ROUTE (fixed-reference kernel, two warpgroups, MXFP4 operands): the online router runs inside the forward.  The
// softmax threads publish the maximum of their slice of every MXFP4 tile; the P.V-issuing warp reduces them to the
// tile's statistic - mean over the query rows of the row maximum, in the very order of the stand-alone statistic
// kernel, so the two agree bit for bit - compares it with tau x the statistic of the row's first key tile and either
// issues P.V or leaves the tile's MXFP4 result out and appends the tile to the CTA's visit list as an MXFP8 tile, which
// the same pipeline does after the row's own tiles (same accumulator, same row reference).
template <int NWG, int NSPLIT, int PVQ, int NVF4, int LAZY, int ROUTE = 0>
__global__ void __launch_bounds__(ATT_SERVICE_THREADS + 128 * NWG * NSPLIT, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q8, const __grid_constant__ CUtensorMap tm_q4,
                const __grid_constant__ CUtensorMap tm_k8, const __grid_constant__ CUtensorMap tm_k4,
                const __grid_constant__ CUtensorMap tm_vt, const __grid_constant__ CUtensorMap tm_vt8,
                const __grid_constant__ CUtensorMap tm_vt4, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  if (p.run_if && *(volatile const int*)p.run_if == 0) return;     // conditional re-run: nothing to do
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024 - (raw & 1023)) & 1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ATT_OFF_BAR);
  uint64_t* q_full = bars;                         // 1
  uint64_t* k_full = bars + 1;                     // KSTAGES
  uint64_t* k_empty = k_full + ATT_KSTAGES;        // KSTAGES
  uint64_t* v_full = k_empty + ATT_KSTAGES;        // VSLOTS_MAX
  uint64_t* v_empty = v_full + ATT_VSLOTS_MAX;     // VSLOTS_MAX
  uint64_t* s_full = v_empty + ATT_VSLOTS_MAX;     // 2
  uint64_t* p_ready = s_full + 2;                  // 2
  uint64_t* pv_done = p_ready + 2;                 // 2
  uint64_t* x_bar = pv_done + 2;                   // [WG][2][4] partial-max exchange inside a warpgroup
  uint64_t* m_bar = x_bar + ATT_MAX_WG * 8;        // [2][4] running-max hand-over, per tile parity and row quarter
  uint64_t* l_bar = m_bar + 8;                     // [4] partial-sum exchange in the epilogue
  uint64_t* s_free = l_bar + 4;                    // 2: quantised P.V only - every softmax thread is done with the S buffer
  uint64_t* st_bar = s_free + 2;                   // 2: ROUTE - the owners of the tile have published their slice maxima
  uint64_t* dec_bar = st_bar + 2;                  // [0] = list_bar, ROUTE: the router has been through the row and the visit list is final
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dec_bar + 2);
  int* n_visit = reinterpret_cast<int*>(tmem_slot + 1);
  volatile int* dec = n_visit + 1;                 // [4], slot tile & 3: (tile << 1 | keep) once the router has decided on the tile
  volatile int* n_total = dec + 4;                 // ROUTE: final length of the visit list, valid once list_bar has completed
  float* xmax = reinterpret_cast<float*>(smem + ATT_OFF_XMAX);
  float* xsum = reinterpret_cast<float*>(smem + ATT_OFF_XSUM);
  float* mrow = reinterpret_cast<float*>(smem + ATT_OFF_MROW);
  // the tiles this CTA visits, in order: key-tile index, bit 15 set on MXFP8 tiles.  Every role walks this list, so
  // skipped cells of the map (above a causal diagonal, the unused end of a longer key buffer, dropped tiles) cost nothing.
  const uint16_t* vlist = reinterpret_cast<const uint16_t*>(smem + ATT_OFF_VLIST);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (p.S + ATT_BM - 1) / ATT_BM, nk = (p.Skv + ATT_BN - 1) / ATT_BN;
  const int qi = nq - 1 - (int)blockIdx.x;          // heavy (late) causal rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const uint8_t* map_glob = p.map + (long long)b * p.map_sb + (long long)h * p.map_sh + (long long)qi * nk;
  const void* const acc_in = p.acc_in;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) smem[ATT_OFF_MAP + i] = map_glob[i];     // nk <= ATT_MAP_SMEM (host check)
  if (threadIdx.x < 128) reinterpret_cast<float*>(smem + ATT_OFF_MROW)[2 * 128 + threadIdx.x] = -INFINITY;   // reference hint
  if (threadIdx.x < 4) dec[threadIdx.x] = -1;       // no tile decided yet
  const int off = p.Skv - p.S;                      // queries are aligned to the end of the keys

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < ATT_KSTAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < ATT_VSLOTS_MAX; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&p_ready[s], 128 * NSPLIT); mbar_init(&pv_done[s], 1); mbar_init(&s_free[s], 128 * NSPLIT); }
    for (int s = 0; s < 2; ++s) { mbar_init(&st_bar[s], 128 * NSPLIT); mbar_init(&dec_bar[s], 1); }
    for (int s = 0; s < ATT_MAX_WG * 8; ++s) mbar_init(&x_bar[s], NSPLIT);
    for (int s = 0; s < 8; ++s) mbar_init(&m_bar[s], NSPLIT);
    for (int s = 0; s < 4; ++s) mbar_init(&l_bar[s], NSPLIT * NWG);
    fence_mbar_init();
    // The Q tile does not depend on the visit list: the thread that has just initialised q_full requests it now, so
    // that it travels while the CTA builds its list (this thread is also the loader of the K and V rings below).
    tma_prefetch_desc(&tm_q8); tma_prefetch_desc(&tm_q4); tma_prefetch_desc(&tm_k8); tma_prefetch_desc(&tm_k4);
    tma_prefetch_desc(&tm_vt); tma_prefetch_desc(&tm_vt8); tma_prefetch_desc(&tm_vt4);
    constexpr int SF4Q = NVF4 ? 1024 : 512;           // bytes of FP4 scales per 128 rows
    const int q_row = (b * p.Hq + h) * p.S + qi * ATT_BM;
    const long long qsf = ((long long)(b * p.Hq + h) * nq + qi) * 512;
    uint8_t* sSFq = smem + ATT_OFF_SF;
    mbar_arrive_expect_tx(q_full, ATT_Q8_BYTES + ATT_Q4_BYTES + 512 + SF4Q);
    tma_load_2d(smem + ATT_OFF_Q8, &tm_q8, q_full, 0, q_row);
    tma_load_2d(smem + ATT_OFF_Q4, &tm_q4, q_full, 0, q_row);
    bulk_load(sSFq, p.q8_sf + qsf, 512, q_full);
    bulk_load(sSFq + 512, p.q4_sf + (NVF4 ? 2 * qsf : qsf), SF4Q, q_full);
  }
  if (warp == 1) tmem_alloc(tmem_slot, ATT_TMEM_COLS);
  __syncthreads();
  if (warp == 2) {
    // ordered compaction of the map row, 32 cells at a time
    uint16_t* vl = reinterpret_cast<uint16_t*>(smem + ATT_OFF_VLIST);
    int base = 0;
    for (int i0 = 0; i0 < nk; i0 += 32) {
      const int i = i0 + lane;
      const uint8_t c = i < nk ? smem[ATT_OFF_MAP + i] : (uint8_t)TILE_SKIP;
      const bool visit = c != TILE_SKIP;
      const uint32_t vis = __ballot_sync(0xffffffffu, visit);
      if (visit) {
        vl[base + __popc(vis & ((1u << lane) - 1u))] = (uint16_t)(i | (c == TILE_FP8 ? 0x8000 : 0));
      }
      base += __popc(vis);
    }
    if (lane == 0) *n_visit = base;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int nv = *n_visit;                          // number of tiles to visit (0: the row has none)
  // ROUTE: a tile the router promotes is appended to the visit list as an MXFP8 tile and done by the same pipeline after
  // the row's own tiles (same O accumulator, same row reference, no second launch).  Every role therefore walks the list
  // in two phases: the row's own tiles [0, nv), then - after list_bar, which the router completes when it has been
  // through the row - the appended ones [nv, *n_total).  The phases share one loop body; its bounds stay loop-invariant
  // (a list polled inside the hot loops cost 0.3 - 0.45 ms per role at cfg3 S=32768, however the poll was written).
  uint64_t* list_bar = dec_bar;
  constexpr int PHASES = ROUTE ? 2 : 1;
  auto list_end = [&](int ph, bool& ok) -> int {     // upper bound of phase ph (waits for the router before phase 1)
    if (ph == 0) return nv;
    ok = mbar_wait(list_bar, 0, p.status, KS_TIMEOUT_PIPE);
    return ok ? (int)*n_total : nv;
  };

  uint8_t* sQ8 = smem + ATT_OFF_Q8;
  uint8_t* sQ4 = smem + ATT_OFF_Q4;
  uint8_t* sK = smem + ATT_OFF_K;
  uint8_t* sV = smem + ATT_OFF_V;
  uint8_t* sSF = smem + ATT_OFF_SF;                 // [0] Q8, [1] Q4, [2+s] K stage s
  uint8_t* sPSF = smem + ATT_OFF_PSF;               // [0..1] P scale tiles per S buffer, [2+s] V stage s
  const int v_half_bytes = p.D * 128;               // one 64-key half of a V^T tile
  constexpr int SF4 = NVF4 ? 1024 : 512;            // bytes of FP4 scales per 128 rows
  constexpr int VSTAGES = PVQ ? 4 : 2;              // V ring depth, and the bytes of one slot
  constexpr int VSLOT = PVQ ? ATT_V_BYTES / 2 : ATT_V_BYTES;

  if (warp == 0) {
    // ------------------------------ Q, K and V loads ---------------------------
    if (lane == 0) {
      const int k_row0 = (b * p.Hkv + hk) * p.Skv;
      const uint8_t* k8sf = p.k8_sf + (long long)(b * p.Hkv + hk) * nk * 512;
      const uint8_t* k4sf = p.k4_sf + (long long)(b * p.Hkv + hk) * nk * SF4;
      const long long vsf0 = (long long)(b * p.Hkv + hk) * p.v_tiles * 512;
      const int v_row = (b * p.Hkv + hk) * p.D;
      bool ok = true;
      int sk = 0, sv = 0;                          // ring slots, and the parity of the `empty` phase to wait for
      uint32_t pk_par = 0, pv_par = 0;
      auto issue_k = [&](int t) {
        const uint32_t e = vlist[t];
        const int j = e & 0x7fff;
        const bool f8 = (e & 0x8000) != 0;
        if (t >= ATT_KSTAGES) ok = mbar_wait(&k_empty[sk], pk_par, p.status, KS_TIMEOUT_PIPE);
        if (!ok) return;
        mbar_arrive_expect_tx(&k_full[sk], (f8 ? ATT_K_BYTES + 512 : ATT_K_BYTES / 2 + SF4));
        tma_load_2d(sK + sk * ATT_K_BYTES, f8 ? &tm_k8 : &tm_k4, &k_full[sk], 0, k_row0 + j * ATT_BN);
        if (f8) bulk_load(sSF + (3 + 2 * sk) * 512, k8sf + (long long)j * 512, 512, &k_full[sk]);
        else bulk_load(sSF + (3 + 2 * sk) * 512, k4sf + (long long)j * SF4, SF4, &k_full[sk]);
        if (++sk == ATT_KSTAGES) { sk = 0; if (t >= ATT_KSTAGES) pk_par ^= 1; }
      };
      auto issue_v = [&](int t) {
        const uint32_t e = vlist[t];
        const int j = e & 0x7fff;
        if (t >= VSTAGES) ok = mbar_wait(&v_empty[sv], pv_par, p.status, KS_TIMEOUT_PIPE);
        if (!ok) return;
        if (PVQ == 0) {
          mbar_arrive_expect_tx(&v_full[sv], 2 * v_half_bytes);
          tma_load_2d(sV + sv * VSLOT, &tm_vt, &v_full[sv], j * ATT_BN, v_row);
          tma_load_2d(sV + sv * VSLOT + v_half_bytes, &tm_vt, &v_full[sv], j * ATT_BN + 64, v_row);
        } else {
          // V^T tile in the tile's format: D rows of 128 (MXFP8) or 64 (MXFP4) bytes, and its scale tile
          const bool f8 = (e & 0x8000) != 0;
          mbar_arrive_expect_tx(&v_full[sv], (f8 ? v_half_bytes : v_half_bytes / 2) + 512);
          tma_load_2d(sV + sv * VSLOT, f8 ? &tm_vt8 : &tm_vt4, &v_full[sv], f8 ? j * ATT_BN : j * (ATT_BN / 2), v_row);
          bulk_load(sPSF + (2 + sv) * 512, (f8 ? p.v8_sf : p.v4_sf) + vsf0 + (long long)j * 512, 512, &v_full[sv]);
        }
        if (++sv == VSTAGES) { sv = 0; if (t >= VSTAGES) pv_par ^= 1; }
      };
      // consumption order: K0, K1, (V0, K2), (V1, K3), ...; with rings this deep neither wait below holds the other
      // ring up for long
      int tk = 0, tv = 0;                          // tiles issued on each ring
      _Pragma("unroll 1") for (int ph = 0; ph < PHASES && ok; ++ph) {
        const int hi = list_end(ph, ok);
        if (!ok) break;
        if (tk == 0 && hi > 0) { issue_k(0); tk = 1; }
        while (ok && tk < hi) {
          issue_k(tk);
          if (!ok) break;
          ++tk;
          issue_v(tv);
          if (ok) ++tv;
        }
        while (ok && tv < tk) { issue_v(tv); if (ok) ++tv; }
      }
      if (!ok) {
        // unwind: give copies in flight a chance to land before shared memory is released
        mbar_wait(q_full, 0, p.status, KS_TIMEOUT_TMA);
        for (int u = max(0, tk - ATT_KSTAGES); u < tk; ++u)
          mbar_wait(&k_full[u % ATT_KSTAGES], (u / ATT_KSTAGES) & 1, p.status, KS_TIMEOUT_TMA);
        for (int u = max(0, tv - VSTAGES); u < tv; ++u)
          mbar_wait(&v_full[u % VSTAGES], (u / VSTAGES) & 1, p.status, KS_TIMEOUT_TMA);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ Q.K^T issuer ------------------------------
    // S(t) goes to accumulator t & 1 as soon as its K tile has landed and the softmax threads have read S(t - 2).
    // One thread issues; its loop holds nothing but the waits, one scale copy, the MMAs and two commits: the tensor
    // pipe takes ~64 cycles per MXFP4 MMA and the loop must stay well below the softmax time of a tile.
    if (lane == 0) {
      uint32_t id8[4], id4[2];
#pragma unroll
      for (int j = 0; j < 4; ++j) id8[j] = idesc_with_sf_id(idesc_block_scaled(p.fp8_fmt, p.fp8_fmt, ATT_BM, ATT_BN, 1), j, j);
#pragma unroll
      for (int j = 0; j < 2; ++j) id4[j] = idesc_with_sf_id(idesc_block_scaled(1, 1, ATT_BM, ATT_BN, 1), 2 * j, 2 * j);
      const uint32_t idn = idesc_block_scaled(1, 1, ATT_BM, ATT_BN, 0);   // NVFP4: E4M3 scales, four per instruction
      const uint64_t q8d = sdesc_kmajor_sw128(smem_u32(sQ8));
      const uint64_t q4d = sdesc_kmajor_sw64(smem_u32(sQ4));
      const uint64_t k8d0 = sdesc_kmajor_sw128(smem_u32(sK));
      const uint64_t k4d0 = sdesc_kmajor_sw64(smem_u32(sK));
      const uint64_t sfk0 = sdesc_sf_tile(smem_u32(sSF + 3 * 512));
      bool ok = mbar_wait(q_full, 0, p.status, KS_TIMEOUT_TMA);
      if (ok) {
        tc_fence_after();
        tc_cp_32x128b_warpx4(tmem + ATT_COL_SFQ8, sdesc_sf_tile(smem_u32(sSF)));
        if (NVF4) {
          tc_cp_32x128b_warpx4(tmem + ATT_COL_SFQN, sdesc_sf_tile(smem_u32(sSF + 512)));
          tc_cp_32x128b_warpx4(tmem + ATT_COL_SFQN + 4, sdesc_sf_tile(smem_u32(sSF + 1024)));
        } else {
          tc_cp_32x128b_warpx4(tmem + ATT_COL_SFQ4, sdesc_sf_tile(smem_u32(sSF + 512)));
        }
      }
      int sk = 0;                                   // K ring slot of the next Q.K^T
      uint32_t k_par = 0;                           // phase parity of k_full[sk]
      // S(t) = Q.K(t)^T into accumulator t & 1; the caller has waited for the accumulator to be free
      auto issue_qk = [&](int t, uint32_t e) {
        ok = mbar_wait(&k_full[sk], k_par, p.status, KS_TIMEOUT_TMA);
        if (!ok) return;
        tc_fence_after();
        const int bsel = t & 1;
        const bool f8 = (e & 0x8000) != 0;
        const uint32_t d = tmem + ATT_COL_S + bsel * 128;
        const uint32_t sfk = tmem + ATT_COL_SFK + bsel * 4;
        const uint64_t ksf = sfk0 + (uint64_t)(sk * (1024 >> 4));
        if (NVF4 && !f8) {
          const uint32_t sfkn = tmem + ATT_COL_SFKN + bsel * 8;
          tc_cp_32x128b_warpx4(sfkn, ksf);
          tc_cp_32x128b_warpx4(sfkn + 4, ksf + (512 >> 4));
          const uint64_t kd = k4d0 + (uint64_t)(sk * (ATT_K_BYTES >> 4));
#pragma unroll
          for (int j = 0; j < 2; ++j) mma_nvf4(d, q4d + 2 * j, kd + 2 * j, idn, tmem + ATT_COL_SFQN + 4 * j, sfkn + 4 * j, j > 0);
        } else if (f8) {
          tc_cp_32x128b_warpx4(sfk, ksf);
          const uint64_t kd = k8d0 + (uint64_t)(sk * (ATT_K_BYTES >> 4));
#pragma unroll
          for (int j = 0; j < 4; ++j) mma_mxf8f6f4(d, q8d + 2 * j, kd + 2 * j, id8[j], tmem + ATT_COL_SFQ8, sfk, j > 0);
        } else {
          tc_cp_32x128b_warpx4(sfk, ksf);
          const uint64_t kd = k4d0 + (uint64_t)(sk * (ATT_K_BYTES >> 4));
#pragma unroll
          for (int j = 0; j < 2; ++j) mma_mxf4(d, q4d + 2 * j, kd + 2 * j, id4[j], tmem + ATT_COL_SFQ4, sfk, j > 0);
        }
        tc_commit(&k_empty[sk]);
        tc_commit(&s_full[bsel]);
        if (++sk == ATT_KSTAGES) { sk = 0; k_par ^= 1; }
      };
      if (PVQ) {
        // Quantised P lives in its own TMEM columns, so an accumulator is free as soon as the softmax threads have
        // read it: this warp issues nothing but Q.K^T, two tiles ahead of the softmax; P.V has its own issuer.
        uint32_t f_par = 0;                         // phase parity of s_free[t & 1] (the release of tile t - 2)
        int t = 0;
        _Pragma("unroll 1") for (int ph = 0; ph < PHASES && ok; ++ph) {
          const int hi = list_end(ph, ok);
          if (!ok) break;
          uint32_t e = t < hi ? vlist[t] : 0;
          for (; t < hi && ok; ++t) {
            const uint32_t e_next = t + 1 < hi ? vlist[t + 1] : 0;    // fetched a tile ahead of its use
            if (t >= 2) {
              ok = mbar_wait(&s_free[t & 1], f_par, p.status, KS_TIMEOUT_PIPE);
              if (t & 1) f_par ^= 1;
              if (!ok) break;
            }
            issue_qk(t, e);
            e = e_next;
          }
        }
      } else {
        // fp16 P overwrites S in place, so Q.K^T of tile t + 2 must stay behind P.V of tile t: one thread issues both,
        // in that order (the tensor pipe executes a thread's instructions in order).
        const uint32_t idesc_pv = idesc_f16(0, 0, ATT_BM, p.D);
        const uint64_t vd0 = sdesc_kmajor_sw128(smem_u32(sV));      // + slot * (VSLOT >> 4)
        const uint32_t v_half16 = (uint32_t)v_half_bytes >> 4;
        constexpr int PW = 128 / NSPLIT;                            // keys per softmax column split
        if (ok && nv > 0) issue_qk(0, vlist[0]);
        if (ok && nv > 1) issue_qk(1, vlist[1]);
        int sv = 0;
        uint32_t v_par = 0, r_par = 0;              // phase parities: v_full[sv]; p_ready[t & 1]
        for (int t = 0; t < nv && ok; ++t) {
          const int bsel = t & 1;
          const uint32_t e2 = t + 2 < nv ? vlist[t + 2] : 0;
          ok = mbar_wait(&v_full[sv], v_par, p.status, KS_TIMEOUT_TMA);
          if (ok) ok = mbar_wait(&p_ready[bsel], r_par, p.status, KS_TIMEOUT_PIPE);
          if (bsel) r_par ^= 1;
          if (!ok) break;
          tc_fence_after();
          const uint32_t ptm = tmem + ATT_COL_S + bsel * 128;
          const uint64_t vd = vd0 + (uint64_t)(sv * (VSLOT >> 4));
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t pcol = ((ks * 16) / PW) * PW + ((ks * 16) % PW) / 2;
            mma_f16_ts(tmem + ATT_COL_O, ptm + pcol, vd + (uint64_t)((ks >> 2) * v_half16 + 2 * (ks & 3)), idesc_pv,
                       ks > 0 ? 1u : (t > 0 ? 1u : 0u));
          }
          tc_commit(&v_empty[sv]);
          tc_commit(&pv_done[bsel]);
          if (++sv == VSTAGES) { sv = 0; v_par ^= 1; }
          if (t + 2 < nv) issue_qk(t + 2, e2);
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------ P.V issuer (quantised P.V) ----------------
    // O += P(t).V(t) as soon as V has landed and every softmax thread of the tile has stored its part of P.  ROUTE: an
    // MXFP4 tile the router leaves out gets no MMA (the commits still go out: the loader and the softmax carry on).
    if (PVQ && lane == 0) {
      const uint64_t vd0 = sdesc_kmajor_sw128(smem_u32(sV));        // + slot * (VSLOT >> 4)
      const uint64_t v4d0 = sdesc_kmajor_sw64(smem_u32(sV));        // MXFP4 V^T tile (64-byte rows)
      const uint64_t sfp0 = sdesc_sf_tile(smem_u32(sPSF));          // P scale tiles [2], then V scale tiles per stage
      uint32_t idp8[4], idp4[2];                                    // P.V block-scaled: M=128, N=D
#pragma unroll
      for (int j = 0; j < 4; ++j) idp8[j] = idesc_with_sf_id(idesc_block_scaled(p.fp8_fmt, p.fp8_fmt, ATT_BM, p.D, 1), j, j);
#pragma unroll
      for (int j = 0; j < 2; ++j) idp4[j] = idesc_with_sf_id(idesc_block_scaled(1, 1, ATT_BM, p.D, 1), 2 * j, 2 * j);
      bool ok = true;
      int sv = 0;
      uint32_t v_par = 0, r_par = 0;                // phase parities: v_full[sv]; p_ready[t & 1]
      uint32_t acc_any = 0;                         // 1 once an MMA has written O
      int t = 0;
      _Pragma("unroll 1") for (int ph = 0; ph < PHASES && ok; ++ph) {
      const int hi = list_end(ph, ok);
      if (!ok) break;
      uint32_t e = t < hi ? vlist[t] : 0;
      for (; t < hi && ok; ++t) {
        const uint32_t e_next = t + 1 < hi ? vlist[t + 1] : 0;
        const int bsel = t & 1;
        bool keep = true;
        ok = mbar_wait(&v_full[sv], v_par, p.status, KS_TIMEOUT_TMA);
        if (ROUTE && ok && !(e & 0x8000)) {
          // the router's word for this tile (it was written while P was being stored, as a rule)
          const int w = poll_tag(&dec[t & 3], t, p.status);
          if (w < 0) ok = false;
          keep = (w & 1) != 0;
        }
        if (ok) ok = mbar_wait(&p_ready[bsel], r_par, p.status, KS_TIMEOUT_PIPE);
        if (bsel) r_par ^= 1;
        if (!ok) break;
        if (keep) {
          tc_fence_after();
          const uint32_t ptm = tmem + ATT_COL_P + bsel * 32;          // quantised P has its own columns
          const uint32_t sfp = tmem + ATT_COL_SFP + bsel * 4, sfv = tmem + ATT_COL_SFV + bsel * 4;
          tc_cp_32x128b_warpx4(sfp, sfp0 + (uint64_t)(bsel * (512 >> 4)));
          tc_cp_32x128b_warpx4(sfv, sfp0 + (uint64_t)((2 + sv) * (512 >> 4)));
          if (e & 0x8000) {
            const uint64_t vd = vd0 + (uint64_t)(sv * (VSLOT >> 4));
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)                             // 32 keys per instruction, 8 TMEM columns of P
              mma_mxf8f6f4_ts(tmem + ATT_COL_O, ptm + ks * 8, vd + 2 * ks, idp8[ks], sfp, sfv, ks > 0 ? 1u : acc_any);
          } else {
            const uint64_t vd = v4d0 + (uint64_t)(sv * (VSLOT >> 4));
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)                             // 64 keys per instruction, 8 TMEM columns of P
              mma_mxf4_ts(tmem + ATT_COL_O, ptm + ks * 8, vd + 2 * ks, idp4[ks], sfp, sfv, ks > 0 ? 1u : acc_any);
          }
          acc_any = 1;
        }
        tc_commit(&v_empty[sv]);
        tc_commit(&pv_done[bsel]);
        if (++sv == VSTAGES) { sv = 0; v_par ^= 1; }
        e = e_next;
      }
      }  // phases of the visit list
    }
  } else if (warp == 3) {
    if (ROUTE) {
    // ------------------------------ router -------------------------------------
    // Statistic of every MXFP4 tile: mean over the query rows of the row maximum.  Lane l takes rows l, 32 + l, 64 + l,
    // 96 + l of the published slice maxima; the four 32-row sums are formed by the same butterfly and added in the same
    // order as in route_stat_kernel / route_stat_finish_kernel, so the statistic is the same bit for bit.
    bool ok = true;
    uint32_t st_par0 = 0, st_par1 = 0;              // phase parity of st_bar[0], st_bar[1]
    float sink = 0.0f;                              // statistic of the row's first key tile (0 until it has been seen)
    const float inv_rows = 1.0f / (float)min(ATT_BM, p.S - qi * ATT_BM);
    int appended = 0;                               // promoted tiles appended to the visit list so far
    uint16_t* vl_w = reinterpret_cast<uint16_t*>(smem + ATT_OFF_VLIST);
    for (int t = 0; t < nv && ok; ++t) {
      const uint32_t e = vlist[t];
      if (e & 0x8000) continue;                     // MXFP8 by the band rule: nothing to decide
      const int bsel = t & 1;
      ok = __all_sync(0xffffffffu, mbar_wait<false>(&st_bar[bsel], bsel ? st_par1 : st_par0, p.status, KS_TIMEOUT_PIPE));
      if (bsel) st_par1 ^= 1; else st_par0 ^= 1;
      if (!ok) break;
      const float* rm = reinterpret_cast<const float*>(smem + ATT_OFF_RMAX) + bsel * ATT_MAX_SPLIT * 128;
      float pq[4];
#pragma unroll
      for (int qq = 0; qq < 4; ++qq) {
        const int r = qq * 32 + lane;
        float mxr = rm[r];
#pragma unroll
        for (int gg = 1; gg < NSPLIT; ++gg) mxr = fmaxf(mxr, rm[gg * 128 + r]);
        float v = (qi * ATT_BM + r < p.S && mxr != -INFINITY) ? mxr * inv_rows : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        pq[qq] = v;
      }
      const float stat = ((pq[0] + pq[1]) + pq[2]) + pq[3];
      const int j = e & 0x7fff;
      if (j == 0) sink = stat;
      const bool keep = !(stat >= sink * p.tau);
      if (lane == 0) {
        if (!keep) {
          // promoted: the MXFP4 result of this tile is left out; the tile is done again in MXFP8 after the row's own tiles
          p.map_rw[(long long)b * p.map_sb + (long long)h * p.map_sh + (long long)qi * nk + j] = TILE_FP8;
          vl_w[nv + appended] = (uint16_t)(j | 0x8000);
        }
        if (p.stat_out) p.stat_out[(((long long)b * p.Hq + h) * nq + qi) * nk + j] = stat;
        dec[t & 3] = (t << 1) | (keep ? 1 : 0);     // one word: readers poll it, nothing else to publish
      }
      if (!keep) ++appended;
      __syncwarp();
    }
    if (lane == 0) {
      *n_total = nv + appended;                     // the list is complete (also after a failure: the others see the status word)
      __threadfence_block();
      mbar_arrive(list_bar);                        // release: the appended entries and the count are visible to who waits
    }
    }
  } else {
    // ------------------------------ softmax / correction / epilogue -----------
    // Per tile and thread: ONE pass over the S slice computes P = exp2(S - m) with the row reference
    // m known so far, the slice maximum and the partial row sum; P stays in registers.  Afterwards
    // the row maximum is assembled (partial maxima of the column splits), the reference decided by
    // the previous tile's owner is taken over, and only if the reference has to move (the maximum
    // grew by more than 2^8, or another warpgroup moved it meanwhile; always on the first tile) the
    // tile is redone from S, which is still intact in TMEM.  P is written over S only then.
    constexpr int W = 128 / NSPLIT;                 // keys of a tile owned by this thread
    constexpr int NCH = W / 32;                     // 32-column chunks of the slice
    const int sw = warp - ATT_SERVICE_THREADS / 32; // warps 0-3 are the service warps
    const int q = warp & 3;                         // TMEM lane quarter this warp may access
    const int g = (sw >> 2) % NSPLIT;               // column split owned by this warp
    const int wg = (sw >> 2) / NSPLIT;              // warpgroup: owns tiles t with t % NWG == wg
    const int part = wg * NSPLIT + g;               // index among the threads that share a row
    const int r_in = q * 32 + lane;                 // row inside the tile == TMEM lane
    const int m_glob = qi * ATT_BM + r_in;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    float* mhint = mrow + 2 * 128;
    float m_seen = -INFINITY;                       // row reference this thread's partial sum refers to
    [[maybe_unused]] float m_fix = -INFINITY;       // LAZY: the row reference fixed by the first tile
    [[maybe_unused]] bool have_ref = false;
    float l_run = 0.0f;                             // partial row sum over this thread's tiles / columns
    bool ok = true;
    static_assert(!ROUTE || (NWG == 2 && PVQ && LAZY && !NVF4), "the router runs in the fixed-reference MXFP4 kernel with two warpgroups");
    int t_own = wg;                                 // next tile of this warpgroup
    int n_tiles = nv;                               // tiles of the CTA, appended ones included once they are known
    _Pragma("unroll 1") for (int ph = 0; ph < PHASES && ok; ++ph) {
    if (ph == 1) {
      ok = __all_sync(0xffffffffu, mbar_wait(list_bar, 0, p.status, KS_TIMEOUT_PIPE));
      if (!ok) break;
      n_tiles = *n_total;
    }
    for (int t = t_own; t < n_tiles && ok; t += NWG, t_own = t) {   // t: index in the visit list; this warpgroup owns every NWG-th tile
      const uint32_t entry = vlist[t];
      const int j = entry & 0x7fff;                 // key tile
      const bool tile_f8 = (entry & 0x8000) != 0;
      const int bsel = t & 1, lt = t / NWG;         // S buffer; count of tiles this warpgroup has done
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[bsel], (t >> 1) & 1, p.status, KS_TIMEOUT_MMA));
      if (!ok) break;
      tc_fence_after();
      const uint32_t slice_addr = tmem + lane_base + ATT_COL_S + bsel * 128 + g * W;
      const int n0 = j * ATT_BN + g * W;            // first key of this thread's slice
      const bool need_mask = (p.causal && (j * ATT_BN + ATT_BN - 1 > qi * ATT_BM + off)) || (j * ATT_BN + ATT_BN > p.Skv);
      const int lim = p.causal ? min(p.Skv - 1, m_glob + off) : (p.Skv - 1);   // last visible key
      [[maybe_unused]] const bool nv_tile = NVF4 && !tile_f8;                   // scores still lack the tensor scales
      // all chunk loads go out up front when the slice and its packed P fit in the register budget
      constexpr int REG_BUDGET = ((16384 / 32) / (1 + NWG * NSPLIT)) >= 255 ? 255 : (((16384 / 32) / (1 + NWG * NSPLIT)) & ~7);
      constexpr bool ALL_UP = (W + W / 2 + 40 <= REG_BUDGET);
      uint32_t sr[ALL_UP ? W : 32];
      uint32_t pk[W / 2];
      float mx0 = -INFINITY;
      float lsum0 = 0.0f, lsum1 = 0.0f;
      uint32_t psc = 0;                             // E8M0 codes of this thread's P blocks (pv_mode 1)
      // precision of P for this tile: 0 fp16; 1 MXFP8 E5M2; 2 MXFP8 E4M3; 3 MXFP4
      const int pmode = (PVQ == 0) ? 0 : (tile_f8 ? (p.fp8_fmt == 0 ? 2 : 1) : 3);
      // reference to start with: this thread's own on one warpgroup, else the latest published hint
      const bool lazy_tile = PVQ && LAZY && t > 0;
      if (lazy_tile && !have_ref) {                  // the first tile's owner has fixed the reference
        if (NWG > 1) {
          ok = __all_sync(0xffffffffu, mbar_wait(&m_bar[q], 0, p.status, KS_TIMEOUT_PIPE));
          if (!ok) break;
        }
        m_fix = mrow[r_in];
        m_seen = m_fix;
        have_ref = true;
      }
      const float m0 = (t == 0) ? -INFINITY : (lazy_tile ? m_fix : ((NWG > 1) ? mhint[r_in] : m_seen));
      const float mref0 = (m0 == -INFINITY) ? 0.0f : m0;
      if (!lazy_tile) {
      // ---- the pass ----
      if (ALL_UP) {
#pragma unroll
        for (int c = 0; c < NCH; ++c) tmem_ld32p(slice_addr + c * 32, sr + c * 32);
      } else {
        tmem_ld32p(slice_addr, sr);
      }
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        uint32_t* sc = ALL_UP ? (sr + c * 32) : sr;
        if (!ALL_UP || c == 0) tmem_ld_wait();
        if (NVF4 && nv_tile) {
#pragma unroll
          for (int i = 0; i < 32; ++i) sc[i] = __float_as_uint(__uint_as_float(sc[i]) * p.fp4_scale);
        }
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (n0 + c * 32 + i > lim) sc[i] = 0xff800000u;      // -inf
        }
        const float bm = block_max32(sc);                          // maximum of this 32-key block
        mx0 = fmaxf(mx0, bm);
        if (t > 0) {
          uint32_t code = 0;
          if (pmode == 0) code = softmax_block<0>(sc, mref0, bm, pk + c * 16, lsum0, lsum1);
          else if (pmode == 3) code = softmax_block<3>(sc, mref0, bm, pk + c * 4, lsum0, lsum1);
          else if (pmode == 1) code = softmax_block<1>(sc, mref0, bm, pk + c * 8, lsum0, lsum1);
          else code = softmax_block<2>(sc, mref0, bm, pk + c * 8, lsum0, lsum1);
          psc |= code << (8 * c);
        }
        if (!ALL_UP && c + 1 < NCH) tmem_ld32p(slice_addr + (c + 1) * 32, sr);
      }
      }
      [[maybe_unused]] float mx = mx0;
      if (lazy_tile) {
        // Fixed reference: nothing to agree on between the threads of a row.
        // 32 columns at a time (few live registers, so the arithmetic of a block interleaves freely); the S buffer is
        // released as soon as the last block has been read, before its arithmetic.
        uint32_t sl[32];
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          uint32_t* sc = sl;
          tmem_ld32p(slice_addr + c * 32, sl);
          tmem_ld_wait();
          if (c == NCH - 1) {
            tc_fence_before();
            mbar_arrive(&s_free[bsel]);
          }
          if (NVF4 && nv_tile) {
#pragma unroll
            for (int i = 0; i < 32; ++i) sc[i] = __float_as_uint(__uint_as_float(sc[i]) * p.fp4_scale);
          }
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (n0 + c * 32 + i > lim) sc[i] = 0xff800000u;      // -inf
          }
          const float bm = block_max32(sc);
          mx0 = fmaxf(mx0, bm);
          if (ROUTE && !tile_f8 && c == NCH - 1) {
            // the slice maximum is complete: publish it now, so that the router decides while this thread still
            // does the arithmetic of its last block
            reinterpret_cast<float*>(smem + ATT_OFF_RMAX)[(bsel * ATT_MAX_SPLIT + g) * 128 + r_in] = mx0;
            mbar_arrive(&st_bar[bsel]);
          }
          uint32_t code;
          if (pmode == 3) code = softmax_block_q<3>(sc, mref0, bm, pk + c * 4, lsum0, lsum1);
          else if (pmode == 1) code = softmax_block_q<1>(sc, mref0, bm, pk + c * 8, lsum0, lsum1);
          else code = softmax_block_q<2>(sc, mref0, bm, pk + c * 8, lsum0, lsum1);
          psc |= code << (8 * c);
        }
        if (m_glob < p.S && mx0 > mref0 + ATT_LAZY_HEADROOM) *p.range_flag = 1;   // rows of the ragged tail hold no data
      } else {
      if (NSPLIT > 1) {
        // full-row maximum = max over the NSPLIT partial maxima of this row
        float* xm = xmax + ((wg * 2 + (lt & 1)) * ATT_MAX_SPLIT) * 128;
        xm[g * 128 + r_in] = mx;
        __syncwarp();
        uint64_t* xb = &x_bar[(wg * 2 + (lt & 1)) * 4 + q];
        if (lane == 0) mbar_arrive(xb);
        ok = __all_sync(0xffffffffu, mbar_wait(xb, (lt >> 1) & 1, p.status, KS_TIMEOUT_PIPE));
        if (!ok) break;
#pragma unroll
        for (int gg = 0; gg < NSPLIT; ++gg) mx = fmaxf(mx, xm[gg * 128 + r_in]);
      }
      // ---- reference decided by the owner of the previous tile ----
      float m1 = m_seen;
      if (NWG > 1 && t > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&m_bar[((t - 1) & 1) * 4 + q], ((t - 1) >> 1) & 1, p.status, KS_TIMEOUT_PIPE));
        if (!ok) break;
        m1 = mrow[((t - 1) & 1) * 128 + r_in];
      }
      // the reference moves only when the maximum grew by more than 2^8 (every thread of a row takes
      // the same decision: it sees the same maximum and the same previous reference)
      const bool grow = (t == 0) || (mx > m1 + ATT_RESCALE_LOG2);
      // with quantised P the reference is kept integral: a power-of-two change of P then changes block
      // scale codes only, never element codes
      const float m_used = grow ? (PVQ ? ceilf(fmaxf(m1, mx)) : fmaxf(m1, mx)) : m1;
      if (m_seen != m_used) {                       // bring this thread's partial sum to the reference
        l_run = (m_seen == -INFINITY) ? 0.0f : l_run * ex2(m_seen - m_used);
        m_seen = m_used;
      }
      if (NWG > 1) {                                // publish the decision; the next tile's owner waits for it
        if (g == 0) { mrow[(t & 1) * 128 + r_in] = m_used; mhint[r_in] = m_used; }
        __syncwarp();
        if (lane == 0) mbar_arrive(&m_bar[(t & 1) * 4 + q]);
      }
      const bool redo = (t == 0) || (m_used != m0);  // P of the pass used another reference (or none)
      if (__any_sync(0xffffffffu, redo)) {
        if (t > 0 && __any_sync(0xffffffffu, grow)) {
          // rescale the accumulator; it must be quiescent: P.V of the previous tile finished
          ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(t - 1) & 1], ((t - 1) >> 1) & 1, p.status, KS_TIMEOUT_MMA));
          if (!ok) break;
          tc_fence_after();
          const float alpha = grow ? ex2(m1 - m_used) : 1.0f;
          for (int c = g; c < p.D / 32; c += NSPLIT) {          // this split's share of the O columns
            uint32_t o[32];
            tmem_ld32p(tmem + lane_base + ATT_COL_O + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32p(tmem + lane_base + ATT_COL_O + c * 32, o);
          }
          tmem_st_wait();
        }
        // redo the pass from S with the final reference
        const float mref = (m_used == -INFINITY) ? 0.0f : m_used;   // row with no visible key so far
        lsum0 = 0.0f;
        lsum1 = 0.0f;
        psc = 0;
        tmem_ld32p(slice_addr, sr);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          tmem_ld_wait();
          if (NVF4 && nv_tile) {
#pragma unroll
            for (int i = 0; i < 32; ++i) sr[i] = __float_as_uint(__uint_as_float(sr[i]) * p.fp4_scale);
          }
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (n0 + c * 32 + i > lim) sr[i] = 0xff800000u;
          }
          const float bm = block_max32(sr);
          uint32_t code = 0;
          if (pmode == 0) code = softmax_block<0>(sr, mref, bm, pk + c * 16, lsum0, lsum1);
          else if (pmode == 3) code = softmax_block<3>(sr, mref, bm, pk + c * 4, lsum0, lsum1);
          else if (pmode == 1) code = softmax_block<1>(sr, mref, bm, pk + c * 8, lsum0, lsum1);
          else code = softmax_block<2>(sr, mref, bm, pk + c * 8, lsum0, lsum1);
          psc |= code << (8 * c);
          if (c + 1 < NCH) tmem_ld32p(slice_addr + (c + 1) * 32, sr);
        }
      }
      if (PVQ && LAZY && t == 0) { m_fix = m_used; have_ref = true; }
      }  // !lazy_tile
      if (ROUTE && !tile_f8) {
        if (!lazy_tile) {                           // the first tile went through the exact path and knows the row's maximum
          reinterpret_cast<float*>(smem + ATT_OFF_RMAX)[(bsel * ATT_MAX_SPLIT + g) * 128 + r_in] = mx;
          mbar_arrive(&st_bar[bsel]);
        }
        // the tile's sum counts only if the router keeps the tile (its word is there by now, as a rule)
        const int w = poll_tag(&dec[t & 3], t, p.status);
        if (w < 0) { ok = false; break; }
        if (w & 1) l_run += lsum0 + lsum1;
      } else {
        l_run += lsum0 + lsum1;
      }
      if (PVQ) {
        if (!lazy_tile) {
          tc_fence_before();
          mbar_arrive(&s_free[bsel]);               // this thread will not read the S buffer again
        }
        if (t >= 2) {                               // the P buffer and its scale tile: P.V of tile t-2 has read them
          ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[bsel], ((t - 2) >> 1) & 1, p.status, KS_TIMEOUT_MMA));
          if (!ok) break;
          tc_fence_after();
        }
      }
      // fp16 P overwrites S inside this thread's own slice: key k of the tile sits in column
      // (k / W) * W + (k % W) / e with e = 2 (fp16), 4 (MXFP8) or 8 (MXFP4) elements per 32-bit column
      if (pmode == 0) {
#pragma unroll
        for (int c = 0; c < NCH; ++c) tmem_st16p(slice_addr + c * 16, pk + c * 16);
      } else {
        // quantised P has its own buffer: key k of the tile in column k / 4 (MXFP8) or k / 8 (MXFP4)
        const uint32_t p_addr = tmem + lane_base + ATT_COL_P + bsel * 32;
        if (pmode == 3) {
#pragma unroll
          for (int c = 0; c < NCH; ++c) tmem_st4p(p_addr + g * (W / 8) + c * 4, pk + c * 4);
        } else {
#pragma unroll
          for (int c = 0; c < NCH; ++c) tmem_st8p(p_addr + g * (W / 4) + c * 8, pk + c * 8);
        }
        // this row's block scales go into the 128x4 scale tile of the S buffer, which the MMA warp
        // copies to TMEM: row r, block k at byte (r % 32) * 16 + (r / 32) * 4 + k
        uint8_t* dst = sPSF + bsel * 512 + lane * 16 + q * 4 + g * NCH;
        if (NCH == 4) *reinterpret_cast<uint32_t*>(dst) = psc;
        else if (NCH == 2) *reinterpret_cast<uint16_t*>(dst) = (uint16_t)psc;
        else *dst = (uint8_t)psc;
        fence_proxy_async_smem();                   // make the tile visible to tcgen05.cp
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_ready[bsel]);
    }
    }  // phases of the visit list
    const int t = n_tiles;                          // tiles visited by the CTA (whoever owned them)
    // ---- epilogue: bring every partial sum to the final reference, add them, O / l ----
    float l_tot = l_run;
    float m_final = m_seen;                         // reference the partial sums end up referring to
    if (NWG * NSPLIT > 1 && ok) {
      if (PVQ && LAZY) {
        if (t > 0 && !have_ref) {                   // this thread owned no tile: all sums refer to the first tile's reference
          if (NWG > 1) ok = __all_sync(0xffffffffu, mbar_wait(&m_bar[q], 0, p.status, KS_TIMEOUT_PIPE));
          if (ok) m_fix = mrow[r_in];
        }
        if (t > 0) m_final = m_fix;
      } else if (NWG > 1 && t > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&m_bar[((t - 1) & 1) * 4 + q], ((t - 1) >> 1) & 1, p.status, KS_TIMEOUT_PIPE));
        if (ok) {
          const float m_fin = mrow[((t - 1) & 1) * 128 + r_in];
          if (m_fin != m_seen) l_run = (m_seen == -INFINITY) ? 0.0f : l_run * ex2(m_seen - m_fin);
          m_final = m_fin;
        }
      }
      if (ok) {
        xsum[part * 128 + r_in] = l_run;
        __syncwarp();
        if (lane == 0) mbar_arrive(&l_bar[q]);
        ok = __all_sync(0xffffffffu, mbar_wait(&l_bar[q], 0, p.status, KS_TIMEOUT_PIPE));
      }
      if (ok) {
        l_tot = 0.0f;
#pragma unroll
        for (int gg = 0; gg < NWG * NSPLIT; ++gg) l_tot += xsum[gg * 128 + r_in];
      }
    }
    if (ok && t > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(t - 1) & 1], ((t - 1) >> 1) & 1, p.status, KS_TIMEOUT_MMA));
      tc_fence_after();
    }
    if (ok) {
      float inv_l = (t > 0 && l_tot > 0.0f) ? 1.0f / l_tot : 0.0f;
      const long long o_off = ((long long)(b * p.Hq + h) * p.S + m_glob) * p.D;
      float lse_row = (t > 0 && l_tot > 0.0f) ? m_final + log2f(l_tot) : -INFINITY;
      float w_prev = 0.0f;                          // weight of the earlier partial result (merge mode)
      if (acc_in && m_glob < p.S) {
        // two normalised partial results over disjoint key sets combine with weights 2^(lse_i - lse),
        // lse = log2(2^lse_a + 2^lse_b); every thread of a row computes the same numbers
        const float la = p.lse_in[(long long)(b * p.Hq + h) * p.S + m_glob];
        const float lm = fmaxf(la, lse_row);
        if (lm != -INFINITY) {
          const float ea = exp2f(la - lm), eb = exp2f(lse_row - lm);
          const float inv = 1.0f / (ea + eb);
          w_prev = ea * inv;
          inv_l *= eb * inv;
          lse_row = lm + log2f(ea + eb);
        }
      }
      if (p.lse && part == 0 && m_glob < p.S)       // log2(sum_k exp2(S_k)): lets partial results be merged
        p.lse[(long long)(b * p.Hq + h) * p.S + m_glob] = lse_row;
      for (int c = part; c < p.D / 32; c += NWG * NSPLIT) {
        uint32_t o[32];
        if (t > 0) {
          tmem_ld32p(tmem + lane_base + ATT_COL_O + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0;
        }
        if (m_glob < p.S) {
          float val[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) val[i] = __uint_as_float(o[i]) * inv_l;
          if (acc_in) {
            // the earlier partial result of the same elements (it may be the very buffer written below)
            if (p.acc_dtype == 0) {
              const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(acc_in) + o_off + c * 32);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 a = src[i];
                val[4 * i] = fmaf(a.x, w_prev, val[4 * i]);
                val[4 * i + 1] = fmaf(a.y, w_prev, val[4 * i + 1]);
                val[4 * i + 2] = fmaf(a.z, w_prev, val[4 * i + 2]);
                val[4 * i + 3] = fmaf(a.w, w_prev, val[4 * i + 3]);
              }
            } else {
              const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(acc_in) + o_off + c * 32);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const uint4 a = src[i];
                const uint32_t w4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  float2 f;
                  if (p.acc_dtype == 1) f = __half22float2(*reinterpret_cast<const __half2*>(&w4[k]));
                  else f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[k]));
                  val[8 * i + 2 * k] = fmaf(f.x, w_prev, val[8 * i + 2 * k]);
                  val[8 * i + 2 * k + 1] = fmaf(f.y, w_prev, val[8 * i + 2 * k + 1]);
                }
              }
            }
          }
          if (p.out_dtype == 0) {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + o_off + c * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_float4(val[4 * i], val[4 * i + 1], val[4 * i + 2], val[4 * i + 3]);
          } else {
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              if (p.out_dtype == 1) {
                w[i] = pack_f16x2(val[2 * i], val[2 * i + 1]);
              } else {
                __nv_bfloat162 hb = __floats2bfloat162_rn(val[2 * i], val[2 * i + 1]);
                w[i] = *reinterpret_cast<uint32_t*>(&hb);
              }
            }
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) + o_off + c * 32);
#pragma unroll
            for (int i = 0; i < 4; ++i) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, ATT_TMEM_COLS);
}

// ---- merging partial attention results -----------------------------------------------------------
// Two softmax-normalised partial outputs over disjoint key sets, with their log2 denominators, combine to
// the result over the union: w_i = 2^(lse_i - lse), lse = log2(2^lse_a + 2^lse_b).  acc (fp32) and
// lse_acc are updated in place; one thread per 4 output elements.
__global__ void __launch_bounds__(256) attn_merge_kernel(float* acc, float* lse_acc, const void* part, int part_dtype,
                                                         const float* lse_part, long long rows, int D) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;     // index of a 4-element group
  const long long per_row = D / 4;
  if (i >= rows * per_row) return;
  const long long r = i / per_row;
  const float la = lse_acc[r], lb = lse_part[r];
  const float lm = fmaxf(la, lb);
  float wa = 0.0f, wb = 0.0f, lnew = -INFINITY;
  if (lm != -INFINITY) {
    const float ea = exp2f(la - lm), eb = exp2f(lb - lm);
    const float inv = 1.0f / (ea + eb);
    wa = ea * inv;
    wb = eb * inv;
    lnew = lm + log2f(ea + eb);
  }
  float4 a = reinterpret_cast<float4*>(acc)[i];
  float4 bv;
  if (part_dtype == 0) {
    bv = reinterpret_cast<const float4*>(part)[i];
  } else {
    const uint2 raw = reinterpret_cast<const uint2*>(part)[i];
    if (part_dtype == 1) {
      const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
      const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
      bv = make_float4(f0.x, f0.y, f1.x, f1.y);
    } else {
      const float2 f0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
      const float2 f1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      bv = make_float4(f0.x, f0.y, f1.x, f1.y);
    }
  }
  a.x = (wa == 0.0f ? 0.0f : a.x * wa) + (wb == 0.0f ? 0.0f : bv.x * wb);
  a.y = (wa == 0.0f ? 0.0f : a.y * wa) + (wb == 0.0f ? 0.0f : bv.y * wb);
  a.z = (wa == 0.0f ? 0.0f : a.z * wa) + (wb == 0.0f ? 0.0f : bv.z * wb);
  a.w = (wa == 0.0f ? 0.0f : a.w * wa) + (wb == 0.0f ? 0.0f : bv.w * wb);
  reinterpret_cast<float4*>(acc)[i] = a;
  __syncwarp();
  if (i % per_row == 0) lse_acc[r] = lnew;
}

// ---- V^T preparation: V [B,Hkv,Skv,D] (any 16-bit/32-bit float, strided) -> fp16 [B,Hkv,D,Skv_pad],
// keys beyond Skv zero-filled.  The reference casts V to fp16 on the host (ours/mxfp_attn_kernel.py:29-31);
// the transpose makes V the K-major B operand of P.V.
template <typename T>
__global__ void __launch_bounds__(256) prepare_vt_kernel(const T* v, __half* vt, int H, int Skv, int D, int Skv_pad,
                                                         long long vs_b, long long vs_h, long long vs_l) {
  __shared__ float tile[64][65];
  const int bh = blockIdx.z, b = bh / H, h = bh % H;
  const int s0 = blockIdx.x * 64, d0 = blockIdx.y * 64;
  const T* src = v + (long long)b * vs_b + (long long)h * vs_h;
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int sl = i >> 6, dl = i & 63;
    const int s = s0 + sl, d = d0 + dl;
    tile[sl][dl] = (s < Skv && d < D) ? (float)src[(long long)s * vs_l + d] : 0.0f;
  }
  __syncthreads();
  __half* dst = vt + (long long)bh * D * Skv_pad;
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int dl = i >> 6, sl = i & 63;
    const int s = s0 + sl, d = d0 + dl;
    if (d < D && s < Skv_pad) dst[(long long)d * Skv_pad + s] = __float2half_rn(tile[sl][dl]);
  }
}

// ---- band-rule precision map: FP8 iff |i + off/T - j| < band, else FP4; causal => tiles entirely above
// the diagonal are SKIP.  Tiles are T x T; `off` = Skv - S aligns queries to the end of the keys.
__global__ void route_band_kernel(uint8_t* map, int nq, int nk, int T, int causal, int band, int off, int S) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x, i = blockIdx.y;
  if (j >= nk) return;
  map += (long long)blockIdx.z * nq * nk;             // one copy of the map per (batch, head) when launched with grid.z > 1
  uint8_t v = (abs(i + off / T - j) < band) ? TILE_FP8 : TILE_FP4;
  if (causal) {
    const int last_q = min(S - 1, i * T + T - 1);       // last query row of the tile
    if (j * T > last_q + off) v = TILE_SKIP;
  }
  map[(long long)i * nk + j] = v;
}

}  // namespace mpsa

using namespace mpsa;

extern "C" int mpsa_route_band(void* map, int nq, int nk, int tile, int causal, int band, int S, int Skv, void* stream) {
  if (!map || nq <= 0 || nk <= 0 || tile <= 0 || band < 0) return set_error(MPSA_ERR_BAD_ARG, "route_band: bad argument");
  if (nq > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "route_band: more than 65535 query tiles");
  dim3 grid((nk + 127) / 128, nq);
  route_band_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((uint8_t*)map, nq, nk, tile, causal, band, Skv - S, S);
  return check_launch("route_band");
}

extern "C" int mpsa_attn_merge(void* acc, void* lse_acc, const void* part, int part_dtype, const void* lse_part,
                               long long rows, int D, void* stream) {
  if (!acc || !lse_acc || !part || !lse_part || rows <= 0)
    return set_error(MPSA_ERR_BAD_ARG, "attn_merge: null pointer or bad shape");
  if (D != 32 && D != 64 && D != 128)      // a row's threads must sit in one warp (in-place update of lse_acc)
    return set_error(MPSA_ERR_UNSUPPORTED, "attn_merge: head_dim must be 32, 64 or 128");
  if (part_dtype < 0 || part_dtype > 2) return set_error(MPSA_ERR_BAD_ARG, "attn_merge: part_dtype must be 0 (f32), 1 (f16) or 2 (bf16)");
  if (((uintptr_t)acc % 16) || ((uintptr_t)part % 16)) return set_error(MPSA_ERR_BAD_ARG, "attn_merge: 16-byte aligned buffers needed");
  const long long groups = rows * (D / 4);
  const long long blocks = (groups + 255) / 256;
  if (blocks > 0x7fffffffll) return set_error(MPSA_ERR_UNSUPPORTED, "attn_merge: too many rows");
  attn_merge_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>((float*)acc, (float*)lse_acc, part, part_dtype,
                                                                     (const float*)lse_part, rows, D);
  return check_launch("attn_merge");
}

extern "C" int mpsa_prepare_vt(const void* v, int in_dtype, void* vt, int B, int H, int Skv, int D, int Skv_pad,
                               long long vs_b, long long vs_h, long long vs_l, void* stream) {
  if (!v || !vt || B <= 0 || H <= 0 || Skv <= 0 || D <= 0) return set_error(MPSA_ERR_BAD_ARG, "prepare_vt: bad argument");
  if (Skv_pad < Skv || Skv_pad % 8) return set_error(MPSA_ERR_BAD_ARG, "prepare_vt: Skv_pad must be >= Skv and a multiple of 8");
  if (B * H > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "prepare_vt: B*H must be below 65536");
  dim3 grid((Skv_pad + 63) / 64, (D + 63) / 64, B * H);
  cudaStream_t st = (cudaStream_t)stream;
  if (in_dtype == 0) prepare_vt_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)v, (__half*)vt, H, Skv, D, Skv_pad, vs_b, vs_h, vs_l);
  else if (in_dtype == 1) prepare_vt_kernel<__half><<<grid, 256, 0, st>>>((const __half*)v, (__half*)vt, H, Skv, D, Skv_pad, vs_b, vs_h, vs_l);
  else if (in_dtype == 2) prepare_vt_kernel<float><<<grid, 256, 0, st>>>((const float*)v, (__half*)vt, H, Skv, D, Skv_pad, vs_b, vs_h, vs_l);
  else return set_error(MPSA_ERR_BAD_ARG, "prepare_vt: in_dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)");
  return check_launch("prepare_vt");
}

namespace {
struct AttnMaps { const CUtensorMap *q8, *q4, *k8, *k4, *vt, *vt8, *vt4; };

// One launch of one organisation of the forward.  The opt-in for more than 48 KB of dynamic shared memory is a
// per-device attribute of the kernel: it is set before every launch (a host-side table write), so that any device and
// any thread may make the first call.
template <int NWG, int NSPLIT, int PVQ, int NVF4, int LAZY, int ROUTE = 0>
int launch_attn(dim3 grid, cudaStream_t st, const AttnMaps& m, const AttnParams& p) {
  auto kern = attn_fwd_kernel<NWG, NSPLIT, PVQ, NVF4, (PVQ ? LAZY : 0), ROUTE>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_SMEM) != cudaSuccess) {
    cudaGetLastError();
    return set_error(MPSA_ERR_LAUNCH, "attn_fwd: cannot reserve %d bytes of shared memory", ATT_SMEM);
  }
  kern<<<grid, ATT_SERVICE_THREADS + 128 * NWG * NSPLIT, ATT_SMEM, st>>>(*m.q8, *m.q4, *m.k8, *m.k4, *m.vt, *m.vt8, *m.vt4, p);
  return check_launch("attn_fwd");
}
}  // namespace

namespace {
struct AttnLaunch {
  CUtensorMap tq8, tq4, tk8, tk4, tvt, tvt8, tvt4;
  AttnParams p;
};

// argument checks, tensor maps and the parameter block shared by the forward entry points
int prepare_attn(AttnLaunch& L, const void* q8, const void* q8_sf, const void* q4, const void* q4_sf, const void* k8,
                             const void* k8_sf, const void* k4, const void* k4_sf, const void* vt, const void* vt8,
                             const void* v8_sf, const void* vt4, const void* v4_sf, int pv_mode, const void* map,
                             long long map_sb, long long map_sh, void* out, int out_dtype, void* lse, int B, int Hq,
                             int Hkv, int S, int Skv, int D, int Skv_pad, int causal, int fp8_fmt, int fp4_kind,
                             float fp4_scale, const void* acc_in, const void* lse_in, int acc_dtype, int* status) {
  if (!q8 || !q8_sf || !q4 || !q4_sf || !k8 || !k8_sf || !k4 || !k4_sf || !map || !out || !status)
    return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: null pointer");
  if (pv_mode != 0 && pv_mode != 1) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: pv_mode must be 0 (fp16 P.V) or 1 (quantised P.V)");
  if (pv_mode == 0 && !vt) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: pv_mode 0 needs vt");
  if (pv_mode == 1 && (!vt8 || !v8_sf || !vt4 || !v4_sf)) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: pv_mode 1 needs vt8, v8_sf, vt4, v4_sf");
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || S <= 0 || Skv <= 0) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: non-positive shape");
  if (Hq % Hkv) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: Hq must be a multiple of Hkv");
  if (D != 64 && D != 128) return set_error(MPSA_ERR_UNSUPPORTED, "attn_fwd: head_dim must be 64 or 128");
  if (out_dtype < 0 || out_dtype > 2) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: out_dtype must be 0 (f32), 1 (f16) or 2 (bf16)");
  if (fp8_fmt != 0 && fp8_fmt != 1) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: fp8_fmt must be 0 (E4M3) or 1 (E5M2)");
  if (fp4_kind != 0 && fp4_kind != 1) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: fp4_kind must be 0 (MXFP4) or 1 (NVFP4)");
  if ((acc_in != nullptr) != (lse_in != nullptr)) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: acc_in and lse_in go together");
  if (acc_in && (acc_dtype < 0 || acc_dtype > 2 || lse_in == lse || ((uintptr_t)acc_in % 16)))
    return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: merging needs a 16-byte aligned acc_in of dtype 0..2 and an lse output distinct from lse_in");
  if (fp4_kind == 1 && !(fp4_scale > 0.0f)) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: NVFP4 needs a positive fp4_scale");
  if (causal && Skv < S) return set_error(MPSA_ERR_UNSUPPORTED, "attn_fwd: causal needs Skv >= S");
  if ((Skv + ATT_BN - 1) / ATT_BN > ATT_MAP_SMEM) return set_error(MPSA_ERR_UNSUPPORTED, "attn_fwd: at most %d keys", ATT_MAP_SMEM * ATT_BN);
  if (Skv_pad < Skv || Skv_pad % 128) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: Skv_pad must be a multiple of 128, at least Skv");
  const void* ptrs[] = {q8, q8_sf, q4, q4_sf, k8, k8_sf, k4, k4_sf, vt, vt8, v8_sf, vt4, v4_sf, out};
  for (const void* ptr : ptrs)
    if ((uintptr_t)ptr % 16) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: every tensor base must be 16-byte aligned");
  if ((long long)B * Hq * S >= (1ll << 31) || (long long)B * Hkv * Skv >= (1ll << 31))
    return set_error(MPSA_ERR_UNSUPPORTED, "attn_fwd: B*H*S must fit in 31 bits");
  CUtensorMap &tq8 = L.tq8, &tq4 = L.tq4, &tk8 = L.tk8, &tk4 = L.tk4, &tvt = L.tvt, &tvt8 = L.tvt8, &tvt4 = L.tvt4;
  const uint64_t qrows = (uint64_t)B * Hq * S, krows = (uint64_t)B * Hkv * Skv;
  if (make_tmap_2d_bytes(&tq8, q8, ATT_DQK, qrows, ATT_DQK, 128, ATT_BM, CU_TENSOR_MAP_SWIZZLE_128B) ||
      make_tmap_2d_bytes(&tq4, q4, ATT_DQK / 2, qrows, ATT_DQK / 2, 64, ATT_BM, CU_TENSOR_MAP_SWIZZLE_64B) ||
      make_tmap_2d_bytes(&tk8, k8, ATT_DQK, krows, ATT_DQK, 128, ATT_BN, CU_TENSOR_MAP_SWIZZLE_128B) ||
      make_tmap_2d_bytes(&tk4, k4, ATT_DQK / 2, krows, ATT_DQK / 2, 64, ATT_BN, CU_TENSOR_MAP_SWIZZLE_64B) ||
      false)
    return set_error(MPSA_ERR_LAUNCH, "attn_fwd: cuTensorMapEncodeTiled failed");
  const uint64_t vrows = (uint64_t)B * Hkv * D;
  if (pv_mode == 0) {
    if (make_tmap_2d_b16(&tvt, vt, Skv_pad, vrows, (uint64_t)Skv_pad * 2, 64, D, CU_TENSOR_MAP_SWIZZLE_128B))
      return set_error(MPSA_ERR_LAUNCH, "attn_fwd: cuTensorMapEncodeTiled failed");
    tvt8 = tvt; tvt4 = tvt;      // not dereferenced in this mode
  } else {
    if (make_tmap_2d_bytes(&tvt8, vt8, Skv_pad, vrows, Skv_pad, 128, D, CU_TENSOR_MAP_SWIZZLE_128B) ||
        make_tmap_2d_bytes(&tvt4, vt4, Skv_pad / 2, vrows, Skv_pad / 2, 64, D, CU_TENSOR_MAP_SWIZZLE_64B))
      return set_error(MPSA_ERR_LAUNCH, "attn_fwd: cuTensorMapEncodeTiled failed");
    tvt = tvt8;                  // not dereferenced in this mode
  }
  AttnParams& p = L.p;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.S = S; p.Skv = Skv; p.D = D; p.causal = causal; p.fp8_fmt = fp8_fmt;
  p.q8_sf = (const uint8_t*)q8_sf; p.q4_sf = (const uint8_t*)q4_sf;
  p.k8_sf = (const uint8_t*)k8_sf; p.k4_sf = (const uint8_t*)k4_sf;
  p.v8_sf = (const uint8_t*)v8_sf; p.v4_sf = (const uint8_t*)v4_sf; p.pv_mode = pv_mode; p.v_tiles = Skv_pad / 128;
  p.fp4_scale = fp4_scale;
  p.map = (const uint8_t*)map; p.map_sb = map_sb; p.map_sh = map_sh;
  p.out = out; p.out_dtype = out_dtype; p.lse = (float*)lse; p.status = status;
  p.range_flag = nullptr; p.run_if = nullptr;
  p.acc_in = acc_in; p.lse_in = (const float*)lse_in; p.acc_dtype = acc_dtype;
  p.tau = 0.0f; p.map_rw = nullptr; p.stat_out = nullptr;
  if (Hq > 65535 || B > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "attn_fwd: Hq and B must be below 65536");
  return MPSA_OK;
}
}  // namespace

extern "C" int mpsa_attn_fwd(const void* q8, const void* q8_sf, const void* q4, const void* q4_sf, const void* k8,
                             const void* k8_sf, const void* k4, const void* k4_sf, const void* vt, const void* vt8,
                             const void* v8_sf, const void* vt4, const void* v4_sf, int pv_mode, const void* map,
                             long long map_sb, long long map_sh, void* out, int out_dtype, void* lse, int B, int Hq,
                             int Hkv, int S, int Skv, int D, int Skv_pad, int causal, int fp8_fmt, int fp4_kind,
                             float fp4_scale, int* range_flag, const void* acc_in, const void* lse_in, int* status,
                             void* stream) {
  if (acc_in && (out_dtype != 0 || !lse || acc_in == out))
    return set_error(MPSA_ERR_BAD_ARG, "attn_fwd: merging needs fp32 out, lse, and an output distinct from acc_in");
  AttnLaunch L;
  if (int rc = prepare_attn(L, q8, q8_sf, q4, q4_sf, k8, k8_sf, k4, k4_sf, vt, vt8, v8_sf, vt4, v4_sf, pv_mode, map, map_sb, map_sh,
                            out, out_dtype, lse, B, Hq, Hkv, S, Skv, D, Skv_pad, causal, fp8_fmt, fp4_kind, fp4_scale, acc_in, lse_in,
                            0, status))
    return rc;
  AttnParams& p = L.p;
  CUtensorMap &tq8 = L.tq8, &tq4 = L.tq4, &tk8 = L.tk8, &tk4 = L.tk4, &tvt = L.tvt, &tvt8 = L.tvt8, &tvt4 = L.tvt4;
  // Softmax organisation: warpgroups taking tiles in turn (1 or 2) x threads per query row inside a
  // warpgroup (1, 2 or 4).  MPSA_ATTN_WG / MPSA_ATTN_SPLIT override the defaults (read once per process):
  // fp16 P.V 2 warpgroups x 1, quantised P.V 2 x 2.
  static std::once_flag cfg_once;
  static int cfg_of[2];
  std::call_once(cfg_once, [] {
    const char* e1 = getenv("MPSA_ATTN_WG");
    const char* e2 = getenv("MPSA_ATTN_SPLIT");
    for (int m = 0; m < 2; ++m) {
      int nwg = e1 ? atoi(e1) : 2, ns = e2 ? atoi(e2) : (m == 0 ? 1 : 2);
      if (nwg != 1 && nwg != 2) nwg = 2;
      if (ns != 1 && ns != 2 && ns != 4) ns = 1;
      if (nwg == 2 && ns == 4) ns = 2;
      cfg_of[m] = nwg * 10 + ns;
    }
  });
  const int cfg = cfg_of[pv_mode];
  const int nq = (S + ATT_BM - 1) / ATT_BM;
  const dim3 grid(nq, Hq, B);
  cudaStream_t st = (cudaStream_t)stream;
  const AttnMaps maps{&tq8, &tq4, &tk8, &tk4, &tvt, &tvt8, &tvt4};
  // quantised P.V with a range word: the fixed-reference kernel first, the exact kernel behind it runs only if a
  // score left the headroom (its CTAs return at once otherwise)
  const bool lazy_first = pv_mode == 1 && range_flag != nullptr;
#define MPSA_GO(A, B, PV, NV)                                                              \
  do {                                                                                     \
    if (lazy_first) {                                                                      \
      p.range_flag = range_flag;                                                           \
      if (int rc = launch_attn<A, B, PV, NV, PV>(grid, st, maps, p)) return rc;            \
      p.range_flag = nullptr;                                                              \
      p.run_if = range_flag;                                                               \
    }                                                                                      \
    return launch_attn<A, B, PV, NV, 0>(grid, st, maps, p);                                \
  } while (0)
  if (fp4_kind == 1) {               // NVFP4 score tiles: the default organisation of each P.V mode only
    if (pv_mode == 0) MPSA_GO(2, 1, 0, 1);
    MPSA_GO(2, 2, 1, 1);
  }
  if (pv_mode == 0) {
    switch (cfg) {
      case 11: MPSA_GO(1, 1, 0, 0);
      case 12: MPSA_GO(1, 2, 0, 0);
      case 14: MPSA_GO(1, 4, 0, 0);
      case 22: MPSA_GO(2, 2, 0, 0);
      default: MPSA_GO(2, 1, 0, 0);
    }
  }
  switch (cfg) {
    case 11: MPSA_GO(1, 1, 1, 0);
    case 12: MPSA_GO(1, 2, 1, 0);
    case 14: MPSA_GO(1, 4, 1, 0);
    case 21: MPSA_GO(2, 1, 1, 0);
    default: MPSA_GO(2, 2, 1, 0);
  }
#undef MPSA_GO
}

// The forward with the online router inside (no stand-alone statistic pass): MXFP8 inside the diagonal band, MXFP4
// elsewhere unless the MXFP4 statistic of a tile reaches tau x that of the row's first key tile, in which case the tile is
// done in MXFP8.  Quantised P.V, causal.  Three launches:
//   1. the band map for every (batch, head) into `map`;
//   2. the fixed-reference forward with the router (ROUTE): a promoted tile is marked TILE_FP8 in `map` (which ends up as
//      mpsa_route_online would have written it) and done again in MXFP8 by the same CTA after the row's own tiles;
//   3. the exact forward over the final map, conditional on *range_flag: it runs only if a score left the fixed
//      reference's headroom in (2) - then (2)'s output is void, its map is not - and its CTAs return at once otherwise.
extern "C" int mpsa_attn_fwd_routed(const void* q8, const void* q8_sf, const void* q4, const void* q4_sf, const void* k8,
                                    const void* k8_sf, const void* k4, const void* k4_sf, const void* vt8, const void* v8_sf,
                                    const void* vt4, const void* v4_sf, void* map, int band, float tau, void* out,
                                    int out_dtype, void* lse, void* lse_final, void* stat, void* stat_scratch, int B, int Hq,
                                    int Hkv, int S, int Skv, int D, int Skv_pad, int fp8_fmt, int stages, int* range_flag,
                                    int* status, void* stream) {
  if (!map || !lse || !range_flag) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd_routed: null pointer");
  (void)stat_scratch;
  if (stages < 1 || stages > 15) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd_routed: stages is a mask of 1 (band map), 2 (forward), 8 (conditional exact forward)");
  if (band < 1) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd_routed: band must be at least 1");
  if (lse_final == lse) return set_error(MPSA_ERR_BAD_ARG, "attn_fwd_routed: lse_final must be another buffer than lse (or null)");
  const int nq = (S + ATT_BM - 1) / ATT_BM, nk = (Skv + ATT_BN - 1) / ATT_BN;
  const long long msh = (long long)nq * nk, msb = msh * Hq;
  AttnLaunch L;
  if (int rc = prepare_attn(L, q8, q8_sf, q4, q4_sf, k8, k8_sf, k4, k4_sf, nullptr, vt8, v8_sf, vt4, v4_sf, 1, map, msb, msh, out,
                            out_dtype, lse, B, Hq, Hkv, S, Skv, D, Skv_pad, 1, fp8_fmt, 0, 0.0f, nullptr, nullptr, 0, status))
    return rc;
  if (nq > 65535 || (long long)B * Hq > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "attn_fwd_routed: too many tiles or heads");
  if (nk > ATT_MAP_SMEM / 2)                        // the visit list holds the row's own tiles and as many promoted ones
    return set_error(MPSA_ERR_UNSUPPORTED, "attn_fwd_routed: at most %d key tiles", ATT_MAP_SMEM / 2);
  cudaStream_t st = (cudaStream_t)stream;
  const AttnMaps maps{&L.tq8, &L.tq4, &L.tk8, &L.tk4, &L.tvt, &L.tvt8, &L.tvt4};
  const dim3 grid(nq, Hq, B);
  // 1. band map, one copy per (batch, head)
  if (stages & 1) {
    route_band_kernel<<<dim3((nk + 127) / 128, nq, B * Hq), 128, 0, st>>>((uint8_t*)map, nq, nk, 128, 1, band, Skv - S, S);
    if (int rc = check_launch("route_band")) return rc;
  }
  // 2. the forward, router inside: a promoted tile's MXFP4 result is left out and the tile is done again in MXFP8 by the
  // same CTA after the row's own tiles
  float* lse_out = lse_final ? (float*)lse_final : (float*)lse;
  if (stages & 2) {
    AttnParams pa = L.p;
    pa.tau = tau; pa.map_rw = (uint8_t*)map; pa.stat_out = (float*)stat; pa.range_flag = range_flag; pa.lse = lse_out;
    if (int rc = launch_attn<2, 2, 1, 0, 1, 1>(grid, st, maps, pa)) return rc;
  }
  // 3. only if the forward raised *range_flag (a score left the fixed reference's 2^64 headroom: its output is void, its
  // map is not - a slice maximum does not depend on the reference): the exact kernel over the final map.  Its CTAs
  // return at once otherwise.  (stages bit 4 is unused.)
  if (!(stages & 8)) return MPSA_OK;
  AttnParams pf = L.p;
  pf.run_if = range_flag; pf.lse = lse_out;
  return launch_attn<2, 2, 1, 0, 0>(grid, st, maps, pf);
}

