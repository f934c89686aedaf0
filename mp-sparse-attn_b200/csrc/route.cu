// Online tile-precision router for sm_100a.
//
// The reference's router statistic of a score tile is the mean over the query rows of the row maximum,
// and the first key tile of a query tile is its "sink" reference (ours/mxfp_attn_kernel.py:272-280, same
// in ours/online_routing.py:87-112); there it decides whether a tile is processed at all.  Here the same
// statistic, computed from the MXFP4 product, decides the PRECISION of a tile: tiles within the diagonal
// band are MXFP8 anyway; any other visible tile is promoted from MXFP4 to MXFP8 iff
// stat(tile) >= stat(first tile) * tau.
//
// route_stat_kernel: one CTA per (128 query rows, q-head, batch); warp 0 streams the MXFP4 K tiles by
// TMA, warp 1 issues the Q.K^T block-scaled MMAs (kind::mxf4) into a double-buffered TMEM accumulator,
// warps 4-7 reduce every S tile to its statistic.  route_online_kernel then writes the map.
#include "api_internal.h"
#include "common.cuh"
#include "tma_host.h"

namespace mpsa {

// 12 K stages: deep prefetch, and more than half of an SM's shared memory, so that one CTA (which takes all 512
// TMEM columns) runs per SM.
constexpr int RT_BM = 128, RT_BN = 128, RT_KSTAGES = 12, RT_MAXH = 2, RT_SBUF = 3;
constexpr int RT_Q_BYTES = RT_BM * 64, RT_K_BYTES = RT_BN * 64;
constexpr int RT_OFF_Q = 0;                                         // Q tiles of the CTA's heads
constexpr int RT_OFF_K = RT_OFF_Q + RT_MAXH * RT_Q_BYTES;
constexpr int RT_OFF_SF = RT_OFF_K + RT_KSTAGES * RT_K_BYTES;       // Q scale tile per head, then K scale tile per stage
constexpr int RT_OFF_BAR = RT_OFF_SF + (RT_MAXH + RT_KSTAGES) * 512;
constexpr int RT_SMEM = RT_OFF_BAR + 512 + 1024;
constexpr int RT_THREADS = 128 + RT_SBUF * 128;                     // 4 service warps + one reducing warpgroup per accumulator
// TMEM: three S accumulators (128 columns each), then the scale columns: Q per head, K per issuer x 2
constexpr uint32_t RT_TMEM_COLS = 512, RT_COL_SFQ = 384, RT_COL_SFK = 392;

struct RouteParams {
  int B, Hq, Hkv, S, Skv, causal, nh;   // nh: q-heads per CTA (1 or 2; 2 needs an even GQA group)
  const uint8_t* q4_sf; const uint8_t* k4_sf;
  float* part;            // [B,Hq,nq,nk,4] per-warp partial means; cells of tiles above the causal diagonal are not written
  int* status;
  const int* run_if;      // when given: the kernel does nothing unless this word is non-zero
};

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Work of a CTA is a stream of units u = key tile * nh + head.  Unit u uses S accumulator u % 3, which belongs to
// reducing warpgroup u % 3 (warps 4-7 / 8-11 / 12-15); with two heads per CTA a K tile is fetched once for both, and
// each head has its own issuing thread.  A unit's chain (wait, tcgen05.mma, commit, wait, tcgen05.ld, maxima,
// shuffles) is several times longer than its MMAs (2 x 64 cycles), hence three units in flight.  The issuing loops
// hold nothing but two waits, the scale copy, the MMAs and the commits.
__global__ void __launch_bounds__(RT_THREADS, 1)
route_stat_kernel(const __grid_constant__ CUtensorMap tm_q4, const __grid_constant__ CUtensorMap tm_k4,
                  const RouteParams p) {
  extern __shared__ uint8_t smem_raw[];
  if (p.run_if && *(volatile const int*)p.run_if == 0) return;
  uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + RT_OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + RT_KSTAGES;
  uint64_t* s_full = k_empty + RT_KSTAGES;       // RT_SBUF: the unit's MMAs are complete
  uint64_t* s_free = s_full + RT_SBUF;           // RT_SBUF: the four warps of the group have read the accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + RT_SBUF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (p.S + RT_BM - 1) / RT_BM, nk = (p.Skv + RT_BN - 1) / RT_BN;
  const int nh = p.nh;
  const int qi = nq - 1 - (int)blockIdx.x, h0 = blockIdx.y * nh, b = blockIdx.z;
  const int hk = h0 / (p.Hq / p.Hkv);
  const int off = p.Skv - p.S;
  // key tiles visible to this query tile (all of them without causality)
  const int last_q = min(p.S - 1, qi * RT_BM + RT_BM - 1);
  const int n_tiles = p.causal ? min(nk, (last_q + off) / RT_BN + 1) : nk;
  const int n_units = n_tiles * nh;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < RT_KSTAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], nh); }
    for (int s = 0; s < RT_SBUF; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_free[s], 4); }
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, RT_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  uint8_t* sQ = smem + RT_OFF_Q;
  uint8_t* sK = smem + RT_OFF_K;
  uint8_t* sSF = smem + RT_OFF_SF;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q4); tma_prefetch_desc(&tm_k4);
      mbar_arrive_expect_tx(q_full, nh * (RT_Q_BYTES + 512));
      for (int j = 0; j < nh; ++j) {
        tma_load_2d(sQ + j * RT_Q_BYTES, &tm_q4, q_full, 0, (b * p.Hq + h0 + j) * p.S + qi * RT_BM);
        bulk_load(sSF + j * 512, p.q4_sf + ((long long)(b * p.Hq + h0 + j) * nq + qi) * 512, 512, q_full);
      }
      const int k_row0 = (b * p.Hkv + hk) * p.Skv;
      const uint8_t* ksf = p.k4_sf + (long long)(b * p.Hkv + hk) * nk * 512;
      bool ok = true;
      int issued = 0, s = 0;
      uint32_t par = 0;
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (t >= RT_KSTAGES) ok = mbar_wait(&k_empty[s], par, p.status, KS_TIMEOUT_PIPE);
        if (!ok) break;
        mbar_arrive_expect_tx(&k_full[s], RT_K_BYTES + 512);
        tma_load_2d(sK + s * RT_K_BYTES, &tm_k4, &k_full[s], 0, k_row0 + t * RT_BN);
        bulk_load(sSF + (RT_MAXH + s) * 512, ksf + (long long)t * 512, 512, &k_full[s]);
        issued = t + 1;
        if (++s == RT_KSTAGES) { s = 0; if (t >= RT_KSTAGES) par ^= 1; }
      }
      if (!ok) {                                 // unwind: let the copies in flight land before the CTA exits
        mbar_wait(q_full, 0, p.status, KS_TIMEOUT_TMA);
        for (int t = max(0, issued - RT_KSTAGES); t < issued; ++t)
          mbar_wait(&k_full[t % RT_KSTAGES], (t / RT_KSTAGES) & 1, p.status, KS_TIMEOUT_TMA);
      }
    }
  } else if (warp == 1 || (warp == 2 && nh == 2)) {
    // MMA issuer of head j (one thread)
    if (lane == 0) {
      const int j = warp - 1;
      const uint32_t id0 = idesc_with_sf_id(idesc_block_scaled(1, 1, RT_BM, RT_BN, 1), 0, 0);
      const uint32_t id1 = idesc_with_sf_id(idesc_block_scaled(1, 1, RT_BM, RT_BN, 1), 2, 2);
      const uint64_t qd = sdesc_kmajor_sw64(smem_u32(sQ + j * RT_Q_BYTES));
      const uint64_t kd0 = sdesc_kmajor_sw64(smem_u32(sK));
      const uint64_t ksf0 = sdesc_sf_tile(smem_u32(sSF + RT_MAXH * 512));
      const uint32_t sfq = tmem + RT_COL_SFQ + j * 4;
      bool ok = mbar_wait(q_full, 0, p.status, KS_TIMEOUT_TMA);
      if (ok) {
        tc_fence_after();
        tc_cp_32x128b_warpx4(sfq, sdesc_sf_tile(smem_u32(sSF + j * 512)));
      }
      int s = 0, u = j;                          // K ring slot of tile t; unit index
      uint32_t k_par = 0;
      for (int t = 0; t < n_tiles && ok; ++t, u += nh) {
        const int cnt = u / RT_SBUF, bsel = u - cnt * RT_SBUF;       // uses of the accumulator before this one
        ok = mbar_wait<false>(&k_full[s], k_par, p.status, KS_TIMEOUT_TMA);
        if (ok && cnt > 0) ok = mbar_wait<false>(&s_free[bsel], (uint32_t)(cnt - 1) & 1u, p.status, KS_TIMEOUT_PIPE);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sfk = tmem + RT_COL_SFK + j * 8 + (t & 1) * 4;
        tc_cp_32x128b_warpx4(sfk, ksf0 + (uint64_t)(s * (512 >> 4)));
        const uint64_t kd = kd0 + (uint64_t)(s * (RT_K_BYTES >> 4));
        const uint32_t d = tmem + bsel * 128;
        mma_mxf4(d, qd, kd, id0, sfq, sfk, 0);
        mma_mxf4(d, qd + 2, kd + 2, id1, sfq, sfk, 1);
        tc_commit(&s_full[bsel]);
        tc_commit(&k_empty[s]);
        if (++s == RT_KSTAGES) { s = 0; k_par ^= 1; }
      }
    }
  } else if (warp >= 4) {
    const int q = warp & 3, g = (warp - 4) >> 2;           // TMEM lane quarter; warpgroup = accumulator it owns
    const int m_glob = qi * RT_BM + q * 32 + lane;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const float inv_rows = 1.0f / (float)min(RT_BM, p.S - qi * RT_BM);
    const bool row_ok = m_glob < p.S;
    const int lim = p.causal ? min(p.Skv - 1, m_glob + off) : (p.Skv - 1);      // last visible key of this row
    const int lim_all = p.causal ? min(p.Skv - 1, qi * RT_BM + off) : (p.Skv - 1);  // ... of every row of the tile
    float* part_row = p.part + (((long long)(b * p.Hq + h0) * nq + qi) * nk) * 4 + q;
    const long long head_stride = (long long)nq * nk * 4;
    bool ok = true;
    uint32_t par = 0;
    for (int u = g; u < n_units && ok; u += RT_SBUF, par ^= 1) {
      const int t = u / nh, hh = u - t * nh;
      ok = __all_sync(0xffffffffu, mbar_wait<false>(&s_full[g], par, p.status, KS_TIMEOUT_MMA));
      if (!ok) break;
      tc_fence_after();
      const int n0 = t * RT_BN;
      // the row of the tile goes through registers in two halves of 64 columns; the accumulator is released as soon
      // as the second half has been read, before its arithmetic
      float m[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) m[i] = -INFINITY;
      // the reference's statistic knows no mask; keys beyond the sequence end (zero padding) and, on
      // the tiles the causal diagonal crosses, keys above the query are left out here
      const bool full_tile = n0 + RT_BN - 1 <= lim_all;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r[2][32];
#pragma unroll
        for (int c = 0; c < 2; ++c) tmem_ld32(tmem + lane_base + g * 128 + (half * 2 + c) * 32, r[c]);
        tmem_ld_wait();
        if (half == 1) {
          tc_fence_before();
          if (lane == 0) mbar_arrive(&s_free[g]);    // count 4: one per warp of the group
        }
        if (full_tile) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const int k = (half * 2 + c) * 2 + ((i >> 1) & 1);
              m[k] = max3(m[k], __uint_as_float(r[c][i]), __uint_as_float(r[c][i + 1]));
            }
        } else {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (n0 + (half * 2 + c) * 32 + i <= lim) m[half * 2 + c] = fmaxf(m[half * 2 + c], __uint_as_float(r[c][i]));
        }
      }
      const float mx = fmaxf(fmaxf(max3(m[0], m[1], m[2]), max3(m[3], m[4], m[5])), fmaxf(m[6], m[7]));
      float v = (row_ok && mx != -INFINITY) ? mx * inv_rows : 0.0f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) part_row[hh * head_stride + (long long)t * 4] = v;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, RT_TMEM_COLS);
}

// stat = ((p0 + p1) + p2) + p3: the four per-warp partial means of a tile, added in a fixed order
__global__ void route_stat_finish_kernel(const float4* part, float* stat, long long n, const int* run_if) {
  if (run_if && *(volatile const int*)run_if == 0) return;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float4 v = part[i];
    stat[i] = ((v.x + v.y) + v.z) + v.w;
  }
}

// map[b,h,i,j]: SKIP above the causal diagonal, FP8 inside the band, else FP8 iff stat >= sink * tau, else FP4;
// with use_skip, tiles outside the band whose statistic is below sink * skip_tau are SKIP as well.
__global__ void route_online_kernel(uint8_t* map, const float* stat, int nq, int nk, int tile, int causal, int band,
                                    float tau, float skip_tau, int use_skip, int S, int Skv, const int* run_if) {
  if (run_if && *(volatile const int*)run_if == 0) return;
  const int j = blockIdx.x * blockDim.x + threadIdx.x, i = blockIdx.y;
  const long long bh = blockIdx.z;
  if (j >= nk) return;
  const int off = Skv - S;
  const long long row = (bh * nq + i) * nk;
  uint8_t v;
  const int last_q = min(S - 1, i * tile + tile - 1);
  if (causal && j * tile > last_q + off) {
    v = 0;
  } else if (abs(i + off / tile - j) < band) {
    v = 1;
  } else {
    const float st = stat[row + j], sink = stat[row];
    v = (st >= sink * tau) ? 1 : 2;
    // the reference's own use of the statistic: a tile is processed iff it is the row's first one or
    // stat >= sink * skip_thresh (ours/mxfp_attn_kernel.py:276-280); the band is always processed
    if (use_skip && j > 0 && !(st >= sink * skip_tau)) v = 0;
  }
  map[row + j] = v;
}

}  // namespace mpsa

using namespace mpsa;

int mpsa::launch_route_stat(const void* q4, const void* q4_sf, const void* k4, const void* k4_sf, void* stat, void* scratch, int B,
                            int Hq, int Hkv, int S, int Skv, int causal, int* status, const int* run_if, void* stream) {
  if (!q4 || !q4_sf || !k4 || !k4_sf || !stat || !scratch || !status) return set_error(MPSA_ERR_BAD_ARG, "route_stat: null pointer");
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || S <= 0 || Skv <= 0 || Hq % Hkv) return set_error(MPSA_ERR_BAD_ARG, "route_stat: bad shape");
  if (causal && Skv < S) return set_error(MPSA_ERR_UNSUPPORTED, "route_stat: causal needs Skv >= S");
  const void* ptrs[] = {q4, q4_sf, k4, k4_sf, scratch};
  for (const void* ptr : ptrs)
    if ((uintptr_t)ptr % 16) return set_error(MPSA_ERR_BAD_ARG, "route_stat: tensors must be 16-byte aligned");
  if ((long long)B * Hq * S >= (1ll << 31) || (long long)B * Hkv * Skv >= (1ll << 31))
    return set_error(MPSA_ERR_UNSUPPORTED, "route_stat: B*H*S must fit in 31 bits");
  CUtensorMap tq, tk;
  if (make_tmap_2d_bytes(&tq, q4, 64, (uint64_t)B * Hq * S, 64, 64, RT_BM, CU_TENSOR_MAP_SWIZZLE_64B) ||
      make_tmap_2d_bytes(&tk, k4, 64, (uint64_t)B * Hkv * Skv, 64, 64, RT_BN, CU_TENSOR_MAP_SWIZZLE_64B))
    return set_error(MPSA_ERR_LAUNCH, "route_stat: cuTensorMapEncodeTiled failed");
  RouteParams p;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.S = S; p.Skv = Skv; p.causal = causal;
  p.nh = ((Hq / Hkv) % 2 == 0) ? 2 : 1;
  p.q4_sf = (const uint8_t*)q4_sf; p.k4_sf = (const uint8_t*)k4_sf; p.part = (float*)scratch; p.status = status;
  p.run_if = run_if;
  // per-device attribute of the kernel: set before every launch, so that any device and any thread may call first
  if (cudaFuncSetAttribute(route_stat_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_SMEM) != cudaSuccess) {
    cudaGetLastError();
    return set_error(MPSA_ERR_LAUNCH, "route_stat: cannot reserve shared memory");
  }
  if (Hq > 65535 || B > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "route_stat: Hq and B must be below 65536");
  const int nq = (S + RT_BM - 1) / RT_BM, nk = (Skv + RT_BN - 1) / RT_BN;
  const long long cells = (long long)B * Hq * nq * nk;
  // tiles above the causal diagonal are never visited: their cells read 0
  if (cudaMemsetAsync(scratch, 0, cells * 16, (cudaStream_t)stream) != cudaSuccess)
    return set_error(MPSA_ERR_LAUNCH, "route_stat: memset failed");
  dim3 grid(nq, Hq / p.nh, B);
  route_stat_kernel<<<grid, RT_THREADS, RT_SMEM, (cudaStream_t)stream>>>(tq, tk, p);
  if (int rc = check_launch("route_stat")) return rc;
  route_stat_finish_kernel<<<(unsigned)((cells + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const float4*)scratch, (float*)stat, cells, run_if);
  return check_launch("route_stat_finish");
}

extern "C" int mpsa_route_stat(const void* q4, const void* q4_sf, const void* k4, const void* k4_sf, void* stat,
                               void* scratch, int B, int Hq, int Hkv, int S, int Skv, int causal, int* status, void* stream) {
  return mpsa::launch_route_stat(q4, q4_sf, k4, k4_sf, stat, scratch, B, Hq, Hkv, S, Skv, causal, status, nullptr, stream);
}

int mpsa::launch_route_online(void* map, const void* stat, int B, int Hq, int S, int Skv, int causal, int band, float tau,
                              float skip_tau, int use_skip, const int* run_if, void* stream) {
  if (!map || !stat || B <= 0 || Hq <= 0 || S <= 0 || Skv <= 0 || band < 0) return set_error(MPSA_ERR_BAD_ARG, "route_online: bad argument");
  const int nq = (S + 127) / 128, nk = (Skv + 127) / 128;
  if (nq > 65535 || (long long)B * Hq > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "route_online: too many tiles or heads");
  dim3 grid((nk + 127) / 128, nq, B * Hq);
  route_online_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((uint8_t*)map, (const float*)stat, nq, nk, 128, causal, band,
                                                             tau, skip_tau, use_skip, S, Skv, run_if);
  return check_launch("route_online");
}

extern "C" int mpsa_route_online(void* map, const void* stat, int B, int Hq, int S, int Skv, int causal, int band,
                                 float tau, float skip_tau, int use_skip, void* stream) {
  return mpsa::launch_route_online(map, stat, B, Hq, S, Skv, causal, band, tau, skip_tau, use_skip, nullptr, stream);
}
