// Standalone block-scaled GEMM  C[M,N] = alpha * (A . sa) (B . sb)^T  for sm_100a.
//
// Counterpart of block_scaled_matmul_kernel (ours/block_scaled_matmul.py:154-267): A is [M, K] and
// B is [N, K], both K-major, quantised along K; the scales arrive as 512-byte 128x4 tiles
// [rows/128, K/vec/4, 32, 4, 4] (:45-66, :382-384).
//
// Design: one CTA per 128x256 output tile.  A TMA producer warp streams 128-byte-wide K slabs of
// A and B into a 4-stage shared-memory ring (128-byte swizzle) together with the scale tiles
// (untiled bulk copies); the scale tiles are moved into TMEM with tcgen05.cp - by the MMA thread
// itself in MXFP8 mode, by copier threads of their own in the FP4 modes, where a K step has 6 or
// 12 of them - and one thread of the MMA warp issues tcgen05.mma block-scaled instructions that
// accumulate 128x256 fp32 in TMEM; four epilogue warps read the accumulator back with tcgen05.ld,
// apply alpha, convert and store.  All hand-offs go through mbarriers with bounded waits.
//
//   mode 0  MXFP8  kind::mxf8f6f4  K=32 per instruction, one E8M0 scale per 32 elements
//   mode 1  MXFP4  kind::mxf4      K=64 per instruction, two E8M0 scales
//   mode 2  NVFP4  kind::mxf4nvf4  K=64 per instruction, four E4M3 scales (16-element blocks)
#include "api_internal.h"
#include "common.cuh"
#include "tma_host.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace mpsa {

constexpr int GEMM_BM = 128, GEMM_BN = 256, GEMM_STAGES = 4;
constexpr int GEMM_SLAB = 128;                       // bytes of K per stage and row
constexpr int GEMM_A_BYTES = GEMM_BM * GEMM_SLAB;    // 16 KB
constexpr int GEMM_B_BYTES = GEMM_BN * GEMM_SLAB;    // 32 KB
constexpr int GEMM_SFA_BYTES = 4 * 512;              // up to 4 scale tiles per stage
constexpr int GEMM_SFB_BYTES = 2 * 4 * 512;
constexpr int GEMM_STAGE_BYTES = GEMM_A_BYTES + GEMM_B_BYTES + GEMM_SFA_BYTES + GEMM_SFB_BYTES;
constexpr int GEMM_SMEM = GEMM_STAGES * GEMM_STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int GEMM_COPIERS = 4;                      // warps set aside for scale-tile copies (a mode uses 0, 1 or all of them)
constexpr int GEMM_THREADS = 192 + 32 * GEMM_COPIERS;  // producer, MMA issuer, 4 epilogue warps, scale copiers
constexpr uint32_t GEMM_TMEM_COLS = 512;
constexpr uint32_t GEMM_SF_COL0 = 256;               // scale sets live behind the accumulator
constexpr uint32_t GEMM_SF_SET_STRIDE = 64;          // one set per stage: 256 + 4 x 64 = 512 columns
static_assert(GEMM_SF_COL0 + GEMM_STAGES * GEMM_SF_SET_STRIDE <= GEMM_TMEM_COLS, "scale sets do not fit");

struct GemmParams {
  int M, N, K;            // elements
  int mode;               // 0 mxfp8, 1 mxfp4, 2 nvfp4
  int a_fmt, b_fmt;       // element format field of the instruction descriptor
  const uint8_t* sfa;     // [ceil(M/128), nchunks, 512]
  const uint8_t* sfb;     // [ceil(N/128), nchunks, 512]
  int nchunks;            // scale tiles along K
  void* c; long long ldc; int out_dtype;   // 0 f32, 1 f16, 2 bf16, 3 fp8 e5m2
  float alpha;
  int* status;
};

__device__ __forceinline__ void store_row32(void* c, long long off, int out_dtype, const float (&v)[32], int nvalid) {
  if (out_dtype == 0) {
    float* o = reinterpret_cast<float*>(c) + off;
    if (nvalid == 32 && ((uintptr_t)o % 16 == 0)) {
#pragma unroll
      for (int i = 0; i < 8; ++i) reinterpret_cast<float4*>(o)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
      for (int i = 0; i < nvalid; ++i) o[i] = v[i];
    }
  } else if (out_dtype == 1 || out_dtype == 2) {
    uint16_t* o = reinterpret_cast<uint16_t*>(c) + off;
    uint32_t w[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (out_dtype == 1) {
        __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
      } else {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
      }
    }
    if (nvalid == 32 && ((uintptr_t)o % 16 == 0)) {
#pragma unroll
      for (int i = 0; i < 4; ++i) reinterpret_cast<uint4*>(o)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    } else {
      for (int i = 0; i < nvalid; ++i) o[i] = (uint16_t)(w[i >> 1] >> ((i & 1) * 16));
    }
  } else {
    uint8_t* o = reinterpret_cast<uint8_t*>(c) + off;
    for (int i = 0; i < nvalid; ++i) o[i] = (uint8_t)__nv_cvt_float_to_fp8(v[i], __NV_SATFINITE, __NV_E5M2);
  }
}

template <int MODE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_block_scaled_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024 - (raw & 1023)) & 1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + GEMM_STAGES * GEMM_STAGE_BYTES);
  uint64_t* full = bars;                       // [STAGES]
  uint64_t* empty = bars + GEMM_STAGES;        // [STAGES]
  uint64_t* accum_full = bars + 2 * GEMM_STAGES;
  uint64_t* sf_ready = accum_full + 1;         // [STAGES] the stage's scale tiles are in TMEM
  uint64_t* sf_full = sf_ready + GEMM_STAGES;  // [STAGES] the stage's scale tiles are in shared memory (FP4 modes)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sf_full + GEMM_STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * GEMM_BM, n0 = blockIdx.y * GEMM_BN;
  // per-mode geometry, all compile-time: the two single-thread loops below must stay short (an MXFP8 K step is 512
  // tensor-pipe cycles; a loop with run-time mode switches and divisions took ~1200)
  constexpr int EPB = MODE == 0 ? 1 : 2;                 // elements per byte
  constexpr int K_STAGE = GEMM_SLAB * EPB;               // elements of K per stage
  constexpr int CHUNK = MODE == 2 ? 64 : 128;            // K elements covered by one scale tile
  constexpr int NC = K_STAGE / CHUNK;                    // scale tiles per stage and row tile: 1, 2, 4
  constexpr int MPC = 4 / NC;                            // instructions per scale tile (4 instructions per stage)
  // FP4 modes: the scale-tile copies are issued by threads of their own (see the MMA issuer); MXFP8 has one scale tile
  // per stage and row tile and keeps its three copies in the issuing thread (a hop less per stage: 2186 against 2140 TFLOP/s)
  constexpr bool SPLIT = MODE != 0;
  constexpr int NCOP = MODE == 2 ? 4 : (MODE == 1 ? 2 : 0);   // copying threads: one per scale tile of a stage
  const int KT = (p.K + K_STAGE - 1) / K_STAGE;
  const int n_row_tiles = (p.N + 127) / 128;
  const bool two_b = n_row_tiles - (int)blockIdx.y * 2 >= 2;   // the CTA's second 128-row tile of B exists

  if (threadIdx.x == 0) {
    for (int s = 0; s < GEMM_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); mbar_init(&sf_ready[s], NCOP > 0 ? NCOP : 1); mbar_init(&sf_full[s], 1); }
    mbar_init(accum_full, 1);
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, GEMM_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      // batched launch (blockIdx.z): operands, scale tiles and C of the batches lie one after the other
      const uint8_t* sfa_g = p.sfa + ((long long)blockIdx.z * ((p.M + 127) / 128) + blockIdx.x) * p.nchunks * 512;
      const uint8_t* sfb_g = p.sfb + ((long long)blockIdx.z * n_row_tiles + blockIdx.y * 2) * p.nchunks * 512;
      const long long sfb_tile1 = (long long)p.nchunks * 512;           // the second B row tile's scale tiles
      const int ya = (int)blockIdx.z * p.M + m0, yb = (int)blockIdx.z * p.N + n0;
      int issued = 0, s = 0, left = p.nchunks;      // left: scale tiles along K not yet requested
      uint32_t e_par = 1;                           // parity that a never-used barrier already satisfies
      bool ok = true;
      for (int kt = 0; kt < KT; ++kt) {
        if (kt >= GEMM_STAGES) {
          ok = mbar_wait(&empty[s], e_par, p.status, KS_TIMEOUT_PIPE);
          if (!ok) break;
        }
        uint8_t* st = smem + s * GEMM_STAGE_BYTES;
        const int ncv = left < NC ? left : NC;                  // valid scale tiles in this stage (fewer only in the last)
        // FP4 modes: the scale tiles go first and have a barrier of their own, so that their copies to TMEM (by the
        // copier threads) run while the operand slabs are still on their way
        uint64_t* sf_bar = SPLIT ? &sf_full[s] : &full[s];
        if (SPLIT) {
          mbar_arrive_expect_tx(sf_bar, (uint32_t)ncv * (two_b ? 1536u : 1024u));
          mbar_arrive_expect_tx(&full[s], GEMM_A_BYTES + GEMM_B_BYTES);
        } else {
          mbar_arrive_expect_tx(&full[s], GEMM_A_BYTES + GEMM_B_BYTES + (uint32_t)ncv * (two_b ? 1536u : 1024u));
        }
        bulk_load(st + GEMM_A_BYTES + GEMM_B_BYTES, sfa_g, ncv * 512, sf_bar);
        bulk_load(st + GEMM_A_BYTES + GEMM_B_BYTES + GEMM_SFA_BYTES, sfb_g, ncv * 512, sf_bar);
        if (two_b) bulk_load(st + GEMM_A_BYTES + GEMM_B_BYTES + GEMM_SFA_BYTES + NC * 512, sfb_g + sfb_tile1, ncv * 512, sf_bar);
        tma_load_2d(st, &tmap_a, &full[s], kt * GEMM_SLAB, ya);
        tma_load_2d(st + GEMM_A_BYTES, &tmap_b, &full[s], kt * GEMM_SLAB, yb);
        sfa_g += NC * 512;
        sfb_g += NC * 512;
        left -= NC;
        issued = kt + 1;
        if (++s == GEMM_STAGES) { s = 0; e_par ^= 1; }
      }
      if (!ok) {
        // unwind: let the copies already in flight land before the CTA's shared memory goes away
        for (int kt = max(0, issued - GEMM_STAGES); kt < issued; ++kt) {
          mbar_wait(&full[kt % GEMM_STAGES], (kt / GEMM_STAGES) & 1, p.status, KS_TIMEOUT_TMA);
          if (SPLIT) mbar_wait(&sf_full[kt % GEMM_STAGES], (kt / GEMM_STAGES) & 1, p.status, KS_TIMEOUT_TMA);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    // Issuing a tcgen05 instruction costs its thread ~75 cycles; a stage is 4 MMAs and 3 (MXFP8), 6 (MXFP4) or 12
    // (NVFP4) scale-tile copies, against ~710 cycles of tensor time.  The copies therefore have a thread of their own
    // (warps 6..), which signal through sf_ready[stage].
    if (lane == 0) {
      uint32_t idj[4];                              // instruction descriptors of the four instructions of a stage
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (MODE == 0) idj[j] = idesc_with_sf_id(idesc_block_scaled(p.a_fmt, p.b_fmt, GEMM_BM, GEMM_BN, 1), j, j);
        else if (MODE == 1) idj[j] = idesc_with_sf_id(idesc_block_scaled(1, 1, GEMM_BM, GEMM_BN, 1), (j & 1) * 2, (j & 1) * 2);
        else idj[j] = idesc_block_scaled(1, 1, GEMM_BM, GEMM_BN, 0);
      }
      // descriptors of stage 0; a stage further on adds its byte offset >> 4 to the address field
      const uint64_t adesc0 = sdesc_kmajor_sw128(smem_u32(smem)), bdesc0 = sdesc_kmajor_sw128(smem_u32(smem + GEMM_A_BYTES));
      constexpr uint64_t STAGE_STEP = GEMM_STAGE_BYTES >> 4;
      bool ok = true;
      int s = 0, left = p.nchunks;
      uint32_t f_par = 0;
      for (int kt = 0; kt < KT; ++kt) {
        ok = mbar_wait(&full[s], f_par, p.status, KS_TIMEOUT_TMA);
        if (SPLIT && ok) ok = mbar_wait(&sf_ready[s], f_par, p.status, KS_TIMEOUT_TMA);
        if (!ok) break;
        tc_fence_after();
        const uint64_t ad = adesc0 + (uint64_t)s * STAGE_STEP, bd = bdesc0 + (uint64_t)s * STAGE_STEP;
        const uint32_t sfa_t = tmem + GEMM_SF_COL0 + (uint32_t)s * GEMM_SF_SET_STRIDE, sfb_t = sfa_t + 16;
        if (!SPLIT) {                               // NC == 1: the stage's scale tiles, A, B and B's second row tile
          const uint64_t sfa_d = sdesc_sf_tile(smem_u32(smem + GEMM_A_BYTES + GEMM_B_BYTES)) + (uint64_t)s * STAGE_STEP;
          const uint64_t sfb_d = sfa_d + (GEMM_SFA_BYTES >> 4);
          tc_cp_32x128b_warpx4(sfa_t, sfa_d);
          tc_cp_32x128b_warpx4(sfb_t, sfb_d);
          if (two_b) tc_cp_32x128b_warpx4(sfb_t + 4, sfb_d + (NC * 512 >> 4));
        }
        if (left >= NC) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t acc = (kt > 0 || j > 0) ? 1u : 0u;
            const int c = j / MPC;                  // scale tile of this instruction
            if (MODE == 0) mma_mxf8f6f4(tmem, ad + 2 * j, bd + 2 * j, idj[j], sfa_t, sfb_t, acc);
            else if (MODE == 1) mma_mxf4(tmem, ad + 2 * j, bd + 2 * j, idj[j], sfa_t + 4 * c, sfb_t + 8 * c, acc);
            else mma_nvf4(tmem, ad + 2 * j, bd + 2 * j, idj[j], sfa_t + 4 * c, sfb_t + 8 * c, acc);
          }
        } else {
          // the last stage of a K that is not a multiple of the stage: fewer scale tiles, fewer instructions
          for (int j = 0; j < left * MPC; ++j) {
            const uint32_t acc = (kt > 0 || j > 0) ? 1u : 0u;
            const int c = j / MPC;
            if (MODE == 0) mma_mxf8f6f4(tmem, ad + 2 * j, bd + 2 * j, idj[j & 3], sfa_t, sfb_t, acc);
            else if (MODE == 1) mma_mxf4(tmem, ad + 2 * j, bd + 2 * j, idj[j & 3], sfa_t + 4 * c, sfb_t + 8 * c, acc);
            else mma_nvf4(tmem, ad + 2 * j, bd + 2 * j, idj[j & 3], sfa_t + 4 * c, sfb_t + 8 * c, acc);
          }
        }
        tc_commit(&empty[s]);
        left -= NC;
        if (++s == GEMM_STAGES) { s = 0; f_par ^= 1; }
      }
      if (ok) tc_commit(accum_full);
    }
  } else if (warp >= 6) {
    // ------------------------------ scale-tile copiers -------------------------
    // copier ci takes the scale tiles c with c * NCOP / NC == ci of every stage; each commits once per stage
    const int ci = warp - 6;
    if (SPLIT && ci < NCOP && lane == 0) {
      const uint64_t sfdesc0 = sdesc_sf_tile(smem_u32(smem + GEMM_A_BYTES + GEMM_B_BYTES));
      constexpr uint64_t STAGE_STEP = GEMM_STAGE_BYTES >> 4, SFB_STEP = GEMM_SFA_BYTES >> 4, TILE_STEP = 512 >> 4;
      bool ok = true;
      int s = 0, left = p.nchunks;
      uint32_t f_par = 0;
      for (int kt = 0; kt < KT; ++kt) {
        // the producer requests a stage's tiles only after it has seen empty[s]: the MMAs that read this stage's scale
        // set the last time round are done
        ok = mbar_wait(&sf_full[s], f_par, p.status, KS_TIMEOUT_TMA);
        if (!ok) break;
        tc_fence_after();
        const uint64_t sfa_d = sfdesc0 + (uint64_t)s * STAGE_STEP, sfb_d = sfa_d + SFB_STEP;
        const uint32_t sfa_t = tmem + GEMM_SF_COL0 + (uint32_t)s * GEMM_SF_SET_STRIDE, sfb_t = sfa_t + 16;
        const int nc = left < NC ? left : NC;        // scale tiles of this stage (fewer only in the last)
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          if (c * NCOP / NC != ci || c >= nc) continue;
          tc_cp_32x128b_warpx4(sfa_t + 4 * c, sfa_d + c * TILE_STEP);
          tc_cp_32x128b_warpx4(sfb_t + 8 * c, sfb_d + c * TILE_STEP);
          if (two_b) tc_cp_32x128b_warpx4(sfb_t + 8 * c + 4, sfb_d + (NC + c) * TILE_STEP);
        }
        tc_commit(&sf_ready[s]);
        left -= NC;
        if (++s == GEMM_STAGES) { s = 0; f_par ^= 1; }
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    // A thread holds 32 consecutive columns of ONE row, so storing from registers sends 16-byte pieces to 32 different
    // rows per instruction (measured: 6.3k of a CTA's 58k cycles at 8192^3 with bf16 output).  The operand stages are
    // idle by now (every MMA has completed), so a warp parks its 32 rows there and writes whole rows instead.
    const int q = warp & 3;                       // TMEM lane quarter this warp may touch
    const bool ok = __all_sync(0xffffffffu, mbar_wait(accum_full, 0, p.status, KS_TIMEOUT_MMA));
    tc_fence_after();
    if (ok) {
      const int esz = p.out_dtype == 0 ? 4 : (p.out_dtype == 3 ? 1 : 2);
      const int row0 = m0 + q * 32;
      const int rows_valid = min(32, p.M - row0);
      uint8_t* cbase = reinterpret_cast<uint8_t*>(p.c) + (((long long)blockIdx.z * p.M + row0) * p.ldc + n0) * esz;
      const long long row_bytes = p.ldc * esz;
      const bool whole_rows = (n0 + GEMM_BN <= p.N) && ((uintptr_t)cbase % 16 == 0) && (row_bytes % 16 == 0);
      if (whole_rows) {
        const int pitch = GEMM_BN * esz + 16;     // 16 bytes of padding: the 16-byte pieces of 8 lanes fall into 32 banks
        uint8_t* stg = smem + (size_t)q * 32 * pitch;
        for (int ch = 0; ch < GEMM_BN / 32; ++ch) {
          uint32_t r[32];
          tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + ch * 32, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
          store_row32(stg + (size_t)lane * pitch, ch * 32, p.out_dtype, v, 32);
        }
        __syncwarp();
        const int line = GEMM_BN * esz;           // bytes of a row of the tile
        for (int r = 0; r < rows_valid; ++r) {
          const uint8_t* src = stg + (size_t)r * pitch;
          uint8_t* dst = cbase + r * row_bytes;
          for (int o = lane * 16; o < line; o += 512) *reinterpret_cast<uint4*>(dst + o) = *reinterpret_cast<const uint4*>(src + o);
        }
      } else {
        const int row = row0 + lane;
        for (int ch = 0; ch < GEMM_BN / 32; ++ch) {
          uint32_t r[32];
          tmem_ld32(tmem + ((uint32_t)(q * 32) << 16) + ch * 32, r);
          tmem_ld_wait();
          const int col = n0 + ch * 32;
          if (row < p.M && col < p.N) {
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * p.alpha;
            store_row32(p.c, ((long long)blockIdx.z * p.M + row) * p.ldc + col, p.out_dtype, v, min(32, p.N - col));
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, GEMM_TMEM_COLS);
}

}  // namespace mpsa

using namespace mpsa;

static int launch_gemm(const void* a, const void* a_scale, const void* b, const void* b_scale, void* c, int batch, int M,
                       int N, int K, long long lda_bytes, long long ldb_bytes, long long ldc, int mode, int a_fmt, int b_fmt,
                       int out_dtype, float alpha, int* status, void* stream) {
  if (!a || !b || !a_scale || !b_scale || !c || !status)
    return set_error(MPSA_ERR_BAD_ARG, "gemm_block_scaled: null pointer");
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return set_error(MPSA_ERR_BAD_ARG, "gemm_block_scaled: non-positive shape");
  if (batch > 65535 || (long long)batch * M >= (1ll << 31) || (long long)batch * N >= (1ll << 31))
    return set_error(MPSA_ERR_UNSUPPORTED, "gemm_block_scaled: batch too large");
  if (mode < 0 || mode > 2) return set_error(MPSA_ERR_BAD_ARG, "gemm_block_scaled: mode must be 0 (mxfp8), 1 (mxfp4) or 2 (nvfp4)");
  if (out_dtype < 0 || out_dtype > 3) return set_error(MPSA_ERR_BAD_ARG, "gemm_block_scaled: out_dtype must be 0..3");
  const int chunk = mode == 2 ? 64 : 128;
  if (K % chunk != 0) return set_error(MPSA_ERR_UNSUPPORTED, "gemm_block_scaled: K must be a multiple of %d for this mode", chunk);
  if (mode == 0 && !((a_fmt == 0 || a_fmt == 1) && (b_fmt == 0 || b_fmt == 1)))
    return set_error(MPSA_ERR_BAD_ARG, "gemm_block_scaled: mxfp8 element formats are 0 (E4M3) or 1 (E5M2)");
  const int epb = mode == 0 ? 1 : 2;
  const long long kbytes = K / epb;
  if (((uintptr_t)a % 16) || ((uintptr_t)b % 16) || (lda_bytes % 16) || (ldb_bytes % 16) || lda_bytes < kbytes ||
      ldb_bytes < kbytes || ((uintptr_t)a_scale % 16) || ((uintptr_t)b_scale % 16))
    return set_error(MPSA_ERR_BAD_ARG, "gemm_block_scaled: operands need 16-byte aligned bases and row pitches >= K bytes");
  if (ldc < N) return set_error(MPSA_ERR_BAD_ARG, "gemm_block_scaled: ldc < N");
  CUtensorMap ta, tb;
  if (make_tmap_2d_bytes(&ta, a, kbytes, (uint64_t)batch * M, lda_bytes, GEMM_SLAB, GEMM_BM, CU_TENSOR_MAP_SWIZZLE_128B) ||
      make_tmap_2d_bytes(&tb, b, kbytes, (uint64_t)batch * N, ldb_bytes, GEMM_SLAB, GEMM_BN, CU_TENSOR_MAP_SWIZZLE_128B))
    return set_error(MPSA_ERR_LAUNCH, "gemm_block_scaled: cuTensorMapEncodeTiled failed");
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.mode = mode; p.a_fmt = a_fmt; p.b_fmt = b_fmt;
  p.sfa = (const uint8_t*)a_scale; p.sfb = (const uint8_t*)b_scale; p.nchunks = K / chunk;
  p.c = c; p.ldc = ldc; p.out_dtype = out_dtype; p.alpha = alpha; p.status = status;
  // per-device attribute of the kernel: set before every launch, so that any device and any thread may call first
  auto kernel = mode == 0 ? gemm_block_scaled_kernel<0> : (mode == 1 ? gemm_block_scaled_kernel<1> : gemm_block_scaled_kernel<2>);
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM) != cudaSuccess) {
    cudaGetLastError();
    return set_error(MPSA_ERR_LAUNCH, "gemm_block_scaled: cannot reserve %d bytes of shared memory", GEMM_SMEM);
  }
  dim3 grid((M + GEMM_BM - 1) / GEMM_BM, (N + GEMM_BN - 1) / GEMM_BN, batch);
  if (grid.y > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "gemm_block_scaled: N too large");
  kernel<<<grid, GEMM_THREADS, GEMM_SMEM, (cudaStream_t)stream>>>(ta, tb, p);
  return check_launch("gemm_block_scaled");
}

extern "C" int mpsa_gemm_block_scaled(const void* a, const void* a_scale, const void* b, const void* b_scale,
                                      void* c, int M, int N, int K, long long lda_bytes, long long ldb_bytes,
                                      long long ldc, int mode, int a_fmt, int b_fmt, int out_dtype, float alpha,
                                      int* status, void* stream) {
  return launch_gemm(a, a_scale, b, b_scale, c, 1, M, N, K, lda_bytes, ldb_bytes, ldc, mode, a_fmt, b_fmt, out_dtype, alpha,
                     status, stream);
}

extern "C" int mpsa_gemm_block_scaled_batched(const void* a, const void* a_scale, const void* b, const void* b_scale,
                                              void* c, int batch, int M, int N, int K, int mode, int a_fmt, int b_fmt,
                                              int out_dtype, float alpha, int* status, void* stream) {
  const long long kbytes = K / (mode == 0 ? 1 : 2);
  return launch_gemm(a, a_scale, b, b_scale, c, batch, M, N, K, kbytes, kbytes, N, mode, a_fmt, b_fmt, out_dtype, alpha,
                     status, stream);
}
