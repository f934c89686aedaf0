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

// 14 K stages: deep prefetch, and more than half of an SM's shared memory, so that one CTA (which takes all 512
// TMEM columns) runs per SM.
constexpr int RT_BM = 128, RT_BN = 128, RT_KSTAGES = 14;
constexpr int RT_Q_BYTES = RT_BM * 64, RT_K_BYTES = RT_BN * 64;
constexpr int RT_OFF_Q = 0;
constexpr int RT_OFF_K = RT_OFF_Q + RT_Q_BYTES;
constexpr int RT_OFF_SF = RT_OFF_K + RT_KSTAGES * RT_K_BYTES;      // Q scale tile, then K scale tile per stage
constexpr int RT_OFF_RED = RT_OFF_SF + (1 + RT_KSTAGES) * 512;     // float [4][4] per-warp partial sums of the last four tiles
constexpr int RT_OFF_BAR = RT_OFF_RED + 64;
constexpr int RT_SMEM = RT_OFF_BAR + 512 + 1024;
constexpr uint32_t RT_TMEM_COLS = 512, RT_COL_SFQ = 256, RT_COL_SFK = 260;

struct RouteParams {
  int B, Hq, Hkv, S, Skv, causal;
  const uint8_t* q4_sf; const uint8_t* k4_sf;
  float* stat;            // [B,Hq,nq,nk]; cells of tiles entirely above the causal diagonal are not written
  int* status;
};

__global__ void __launch_bounds__(256, 1)
route_stat_kernel(const __grid_constant__ CUtensorMap tm_q4, const __grid_constant__ CUtensorMap tm_k4,
                  const RouteParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + RT_OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + RT_KSTAGES;
  uint64_t* s_full = k_empty + RT_KSTAGES;       // 2
  uint64_t* s_free = s_full + 2;                 // 2: the statistic warps have read the S buffer
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_free + 2);
  float* red = reinterpret_cast<float*>(smem + RT_OFF_RED);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = (p.S + RT_BM - 1) / RT_BM, nk = (p.Skv + RT_BN - 1) / RT_BN;
  const int qi = nq - 1 - (int)blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);
  const int off = p.Skv - p.S;
  // key tiles visible to this query tile (all of them without causality)
  const int last_q = min(p.S - 1, qi * RT_BM + RT_BM - 1);
  const int n_tiles = p.causal ? min(nk, (last_q + off) / RT_BN + 1) : nk;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < RT_KSTAGES; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&s_free[s], 4); }
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
      mbar_arrive_expect_tx(q_full, RT_Q_BYTES + 512);
      tma_load_2d(sQ, &tm_q4, q_full, 0, (b * p.Hq + h) * p.S + qi * RT_BM);
      bulk_load(sSF, p.q4_sf + ((long long)(b * p.Hq + h) * nq + qi) * 512, 512, q_full);
      const int k_row0 = (b * p.Hkv + hk) * p.Skv;
      const long long ksf0 = (long long)(b * p.Hkv + hk) * nk * 512;
      bool ok = true;
      int issued = 0;
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int s = t % RT_KSTAGES;
        if (t >= RT_KSTAGES) ok = mbar_wait(&k_empty[s], ((t / RT_KSTAGES) - 1) & 1, p.status, KS_TIMEOUT_PIPE);
        if (!ok) break;
        mbar_arrive_expect_tx(&k_full[s], RT_K_BYTES + 512);
        tma_load_2d(sK + s * RT_K_BYTES, &tm_k4, &k_full[s], 0, k_row0 + t * RT_BN);
        bulk_load(sSF + (1 + s) * 512, p.k4_sf + ksf0 + (long long)t * 512, 512, &k_full[s]);
        issued = t + 1;
      }
      if (!ok) {
        mbar_wait(q_full, 0, p.status, KS_TIMEOUT_TMA);
        for (int t = max(0, issued - RT_KSTAGES); t < issued; ++t)
          mbar_wait(&k_full[t % RT_KSTAGES], (t / RT_KSTAGES) & 1, p.status, KS_TIMEOUT_TMA);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t id0 = idesc_with_sf_id(idesc_block_scaled(1, 1, RT_BM, RT_BN, 1), 0, 0);
      const uint32_t id1 = idesc_with_sf_id(idesc_block_scaled(1, 1, RT_BM, RT_BN, 1), 2, 2);
      const uint64_t qd = sdesc_kmajor_sw64(smem_u32(sQ));
      bool ok = mbar_wait(q_full, 0, p.status, KS_TIMEOUT_TMA);
      if (ok) {
        tc_fence_after();
        tc_cp_32x128b_warpx4(tmem + RT_COL_SFQ, sdesc_sf_tile(smem_u32(sSF)));
      }
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int s = t % RT_KSTAGES, bsel = t & 1;
        ok = mbar_wait(&k_full[s], (t / RT_KSTAGES) & 1, p.status, KS_TIMEOUT_TMA);
        if (ok && t >= 2) ok = mbar_wait(&s_free[bsel], ((t >> 1) - 1) & 1, p.status, KS_TIMEOUT_PIPE);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sfk = tmem + RT_COL_SFK + bsel * 4;
        tc_cp_32x128b_warpx4(sfk, sdesc_sf_tile(smem_u32(sSF + (1 + s) * 512)));
        const uint64_t kd = sdesc_kmajor_sw64(smem_u32(sK + s * RT_K_BYTES));
        const uint32_t d = tmem + bsel * 128;
        mma_mxf4(d, qd, kd, id0, tmem + RT_COL_SFQ, sfk, 0);
        mma_mxf4(d, qd + 2, kd + 2, id1, tmem + RT_COL_SFQ, sfk, 1);
        tc_commit(&k_empty[s]);
        tc_commit(&s_full[bsel]);
      }
    }
  } else if (warp >= 4) {
    const int q = warp & 3;
    const int m_glob = qi * RT_BM + q * 32 + lane;
    const uint32_t lane_base = (uint32_t)(q * 32) << 16;
    const int valid_rows = min(RT_BM, p.S - qi * RT_BM);
    float* out = p.stat + ((long long)(b * p.Hq + h) * nq + qi) * nk;
    bool ok = true;
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int bsel = t & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[bsel], (t >> 1) & 1, p.status, KS_TIMEOUT_MMA));
      if (!ok) break;
      tc_fence_after();
      float mx = -INFINITY;
      const int n0 = t * RT_BN;
      // the reference's statistic knows no mask; keys beyond the sequence end (zero padding) and, on
      // the tiles the causal diagonal crosses, keys above the query are left out here
      const int lim = p.causal ? min(p.Skv - 1, m_glob + off) : (p.Skv - 1);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem + lane_base + bsel * 128 + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (n0 + c * 32 + i <= lim) mx = fmaxf(mx, __uint_as_float(r[i]));
      }
      tc_fence_before();
      float v = (m_glob < p.S && mx != -INFINITY) ? mx : 0.0f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) {
        red[(t & 3) * 4 + q] = v;
        mbar_arrive(&s_free[bsel]);              // S buffer consumed (count 4: one per warp)
      }
      // warp 4 (q == 0) adds the four partial sums once all of them are there
      if (q == 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&s_free[bsel], (t >> 1) & 1, p.status, KS_TIMEOUT_PIPE));
        if (!ok) break;
        if (lane == 0) out[t] = (red[(t & 3) * 4] + red[(t & 3) * 4 + 1] + red[(t & 3) * 4 + 2] + red[(t & 3) * 4 + 3]) / (float)valid_rows;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, RT_TMEM_COLS);
}

// map[b,h,i,j]: SKIP above the causal diagonal, FP8 inside the band, else FP8 iff stat >= sink * tau, else FP4.
__global__ void route_online_kernel(uint8_t* map, const float* stat, int nq, int nk, int tile, int causal, int band,
                                    float tau, int S, int Skv) {
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
    v = (stat[row + j] >= stat[row] * tau) ? 1 : 2;
  }
  map[row + j] = v;
}

}  // namespace mpsa

using namespace mpsa;

extern "C" int mpsa_route_stat(const void* q4, const void* q4_sf, const void* k4, const void* k4_sf, void* stat, int B,
                               int Hq, int Hkv, int S, int Skv, int causal, int* status, void* stream) {
  if (!q4 || !q4_sf || !k4 || !k4_sf || !stat || !status) return set_error(MPSA_ERR_BAD_ARG, "route_stat: null pointer");
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || S <= 0 || Skv <= 0 || Hq % Hkv) return set_error(MPSA_ERR_BAD_ARG, "route_stat: bad shape");
  if (causal && Skv < S) return set_error(MPSA_ERR_UNSUPPORTED, "route_stat: causal needs Skv >= S");
  const void* ptrs[] = {q4, q4_sf, k4, k4_sf};
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
  p.q4_sf = (const uint8_t*)q4_sf; p.k4_sf = (const uint8_t*)k4_sf; p.stat = (float*)stat; p.status = status;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(route_stat_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_SMEM) != cudaSuccess)
      return set_error(MPSA_ERR_LAUNCH, "route_stat: cannot reserve shared memory");
    attr_set = true;
  }
  if (Hq > 65535 || B > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "route_stat: Hq and B must be below 65536");
  dim3 grid((S + RT_BM - 1) / RT_BM, Hq, B);
  route_stat_kernel<<<grid, 256, RT_SMEM, (cudaStream_t)stream>>>(tq, tk, p);
  return check_launch("route_stat");
}

extern "C" int mpsa_route_online(void* map, const void* stat, int B, int Hq, int S, int Skv, int causal, int band,
                                 float tau, void* stream) {
  if (!map || !stat || B <= 0 || Hq <= 0 || S <= 0 || Skv <= 0 || band < 0) return set_error(MPSA_ERR_BAD_ARG, "route_online: bad argument");
  const int nq = (S + 127) / 128, nk = (Skv + 127) / 128;
  if (nq > 65535 || (long long)B * Hq > 65535) return set_error(MPSA_ERR_UNSUPPORTED, "route_online: too many tiles or heads");
  dim3 grid((nk + 127) / 128, nq, B * Hq);
  route_online_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>((uint8_t*)map, (const float*)stat, nq, nk, 128, causal, band,
                                                             tau, S, Skv);
  return check_launch("route_online");
}
