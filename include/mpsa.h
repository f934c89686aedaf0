/* C-ABI of libmpsa.so: B200 (sm_100a) kernels for the diagonal-tiled mixed-precision attention
 * path.  Plain pointers and sizes only; every pointer is a DEVICE pointer unless stated
 * otherwise; nothing here allocates or frees device memory; every call is asynchronous on
 * `stream` (a cudaStream_t passed as void*).  Return value: 0 on success, negative on error
 * (MPSA_ERR_*); the message is available from mpsa_last_error() on the calling thread.
 *
 * Each entry names the reference function it replaces (paths relative to the reference
 * project root).
 */
#ifndef MPSA_H_
#define MPSA_H_

#ifdef __cplusplus
extern "C" {
#endif

#define MPSA_OK 0
#define MPSA_ERR_BAD_ARG (-1)
#define MPSA_ERR_UNSUPPORTED (-2)
#define MPSA_ERR_LAUNCH (-3)
#define MPSA_ERR_TIMEOUT (-4)

/* input dtypes: 0 bf16, 1 fp16, 2 fp32.  output dtypes: 0 fp32, 1 fp16, 2 bf16, 3 fp8 e5m2 (GEMM only) */
/* fp8 element formats of the quantizer: 1 E5M2 (the reference's), 2 E4M3 */
/* precision-map cells: 0 skip, 1 FP8 tile, 2 FP4 tile */

int mpsa_version(void);

/* Copies the calling thread's last error message (NUL terminated) into buf[0..n). HOST pointer. */
int mpsa_last_error(char* buf, unsigned long long n);

/* Self-test of the failure path every kernel here shares.  No counterpart in the reference (its kernels have no waits
 * of their own).  Launches one thread that waits, with the library's bounded wait, on a barrier that nothing ever
 * arrives at: after `limit_cycles` SM clock cycles (1 .. 2e9) the wait gives up, writes `code` (1 TMA, 2 tensor-core
 * commit, 3 pipeline hand-off) into the device word *status if that word is still 0, and the kernel returns normally.
 * The context stays usable; the host learns of the failure by reading *status, as after any other kernel. */
int mpsa_selftest_wait_timeout(int* status, long long limit_cycles, int code, void* stream);

/* MX block quantizer, one side (Q or K) per call.
 * Replaces quant_mxfp4 / quant_mxfp8e5 and their Triton kernels (ours/quant_mxint8.py:276-351,
 * :453-512 and :164-272) and the scale relayout (ours/mxfp_attn_kernel.py:56-57).
 *   x                [B,H,L,D] logical shape, element strides xs_b/xs_h/xs_l, inner stride 1
 *   s                fp32 scalar multiplied in before quantising (softmax scale * log2e for Q, 1 for K)
 *   Any output pointer may be NULL (that output is not produced).
 *   fp8_codes            one byte per element, byte strides o8_*   (reference output format)
 *   fp4_codes_unpacked   one E2M1 code per byte, byte strides o4_* (reference output format)
 *   fp8_scales_rm / fp4_scales_rm   E8M0 [B,H,L,D/32]              (reference output format)
 *   fp4_codes_packed     [B,H,L,D/2], two codes per byte, low nibble first
 *   fp8_scales_tiled / fp4_scales_tiled   [B,H,ceil(L/128),ceil(D/128),512]: 128x4 scale tiles,
 *                        element (row r, block c) at byte (r%32)*16 + (r/32)*4 + c%4, padding = 127
 */
int mpsa_quant_mx(const void* x, int in_dtype, int B, int H, int L, int D, long long xs_b, long long xs_h,
                  long long xs_l, float s, int fp8_fmt, void* fp8_codes, long long o8_b, long long o8_h,
                  long long o8_l, void* fp4_codes_unpacked, long long o4_b, long long o4_h, long long o4_l,
                  void* fp8_scales_rm, void* fp4_scales_rm, void* fp4_codes_packed, void* fp8_scales_tiled,
                  void* fp4_scales_tiled, void* stream);

/* "Smooth K": the reference subtracts the mean over the sequence from K before quantising it
 * (ours/mxfp_attn_kernel.py:33-34: km = k.mean(dim=-2, keepdim=True); k = k - km).  mpsa_col_mean leaves that mean,
 * fp32 [B,H,D] holding values rounded to the input dtype (fp32 sums in a fixed order, divided by L), and
 * mpsa_quant_mx_centered is mpsa_quant_mx with `center` subtracted from every row first, the difference rounded to
 * the input dtype as the elementwise torch op does, so K is read once instead of three times.
 *   scratch  fp32, at least mpsa_col_mean_scratch_floats(B,H,L,D) elements; center 16-byte aligned. */
long long mpsa_col_mean_scratch_floats(int B, int H, int L, int D);
int mpsa_col_mean(const void* x, int in_dtype, int B, int H, int L, int D, long long xs_b, long long xs_h,
                  long long xs_l, void* mean, void* scratch, long long scratch_floats, void* stream);
int mpsa_quant_mx_centered(const void* x, int in_dtype, int B, int H, int L, int D, long long xs_b, long long xs_h,
                           long long xs_l, float s, const void* center, int fp8_fmt, void* fp8_codes, long long o8_b,
                           long long o8_h, long long o8_l, void* fp4_codes_unpacked, long long o4_b, long long o4_h,
                           long long o4_l, void* fp8_scales_rm, void* fp4_scales_rm, void* fp4_codes_packed,
                           void* fp8_scales_tiled, void* fp4_scales_tiled, void* stream);

/* Rotary embedding fused into the MX quantizer (the step in front of the path: Q and K come out of the QKV projection,
 * are rotated and then quantised by quant_mxfp4 / quant_mxfp8e5, ours/mxfp_attn_kernel.py:41-55; fusing the rotation
 * removes one read and one write of the 16-bit tensor).  Rotate-half convention, as evaluate/llama applies it through
 * transformers: with x1 / x2 the two halves of a row, y1 = x1 cos - x2 sin, y2 = x2 cos + x1 sin; fp32 products and sum,
 * the result rounded to the input dtype (the tensor an unfused pipeline stores), then mpsa_quant_mx's arithmetic.
 *   cos, sin  fp32 [.., L, D/2], 16-byte aligned, shared by the heads; rope_sb = batch stride in floats (0: shared)
 *   D         64 or 128; the other arguments as mpsa_quant_mx. */
int mpsa_rope_quant_mx(const void* x, int in_dtype, int B, int H, int L, int D, long long xs_b, long long xs_h,
                       long long xs_l, const void* cos, const void* sin, long long rope_sb, float s, int fp8_fmt,
                       void* fp8_codes, long long o8_b, long long o8_h, long long o8_l, void* fp4_codes_unpacked,
                       long long o4_b, long long o4_h, long long o4_l, void* fp8_scales_rm, void* fp4_scales_rm,
                       void* fp4_codes_packed, void* fp8_scales_tiled, void* fp4_scales_tiled, void* stream);

/* Per-32 int8 quantizer, one side per call.  Replaces quant_fpxint8 (ours/quant_mxint8.py:21-114).
 *   codes int8 with byte strides o_*; scales fp32 [B,H,L,D/32]. */
int mpsa_quant_int8(const void* x, int in_dtype, int B, int H, int L, int D, long long xs_b, long long xs_h,
                    long long xs_l, float s, void* codes, long long o_b, long long o_h, long long o_l,
                    void* scales, void* stream);

/* V [B,H,Skv,D] (strided) -> fp16 V^T [B,H,D,Skv_pad], keys >= Skv zero.  Replaces the host-side
 * v.to(float16) of the wrapper (ours/mxfp_attn_kernel.py:27-31) and makes V the K-major operand of P.V. */
int mpsa_prepare_vt(const void* v, int in_dtype, void* vt, int B, int H, int Skv, int D, int Skv_pad,
                    long long vs_b, long long vs_h, long long vs_l, void* stream);

/* NVFP4 quantizer of a 2-D operand [rows, cols] (row pitch ld elements) along its columns: 16-element
 * blocks, E4M3 block scales, one fp32 tensor scale: ts = amax/(6*448), block scale = e4m3(amax_blk/(6*ts)),
 * element = e2m1_rne(x/(scale*ts)).  The reference has the GEMM mode only (ours/block_scaled_matmul.py:321-324),
 * no quantizer.  codes [rows, cols/2] (pitch ldc_bytes), scales [ceil(rows/128), cols/64, 512] (128x4 tiles of
 * E4M3 bytes), tensor_scale: one float.  `scratch` holds one partial amax per 128x512 input tile:
 * mpsa_quant_nvfp4_scratch_floats(rows, cols) floats; it needs no initialisation. */
int mpsa_quant_nvfp4_scratch_floats(int rows, int cols);
int mpsa_quant_nvfp4(const void* x, int in_dtype, int rows, int cols, long long ld, float s, void* scratch,
                     long long scratch_floats, void* codes, long long ldc_bytes, void* scales, void* tensor_scale,
                     void* stream);

/* The same quantizer for an attention operand [B,H,L,D] (strides in elements, innermost contiguous), blocks
 * along D, ONE tensor scale for the whole operand: codes [B,H,L,D/2], scales [B,H,ceil(L/128),D/64,512] (the
 * 128-row tiles restart at every head, as mpsa_attn_fwd expects them).  D must be a multiple of 64;
 * scratch: B*H*ceil(L/128)*ceil(D/512) floats.  No counterpart in the reference. */
int mpsa_quant_nvfp4_bh(const void* x, int in_dtype, int B, int H, int L, int D, long long xs_b, long long xs_h,
                        long long xs_l, float s, void* scratch, long long scratch_floats, void* codes, void* scales,
                        void* tensor_scale, void* stream);

/* The same quantizer for callers that cannot allocate device memory (a process whose memory was handed to
 * its own pool at start-up, a plugin barred from the CUDA allocator on its request path, a bare C host):
 * the partial maxima are kept in a 64 KB array built into the library's device image instead of a
 * caller-provided scratch.  This entry has no counterpart in the reference.  It calls no allocator.
 *   - Limit: ceil(rows/128) * ceil(cols/512) <= 16384 partials (about 1e9 elements); larger operands are
 *     refused with MPSA_ERR_UNSUPPORTED and a message naming the limit.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current); make that first call before any stream capture begins.
 *   - All calls on a device share the one array (each call overwrites the part it uses; nothing needs
 *     clearing), so two calls that overlap in time on the GPU race: keep them on one stream or order them.
 *   - Inputs and outputs are the caller's, as in mpsa_quant_nvfp4; results are identical to it. */
int mpsa_quant_nvfp4_static(const void* x, int in_dtype, int rows, int cols, long long ld, float s, void* codes,
                            long long ldc_bytes, void* scales, void* tensor_scale, void* stream);

/* V operand of a quantised P.V: 32-key MX blocks along the SEQUENCE axis, transposed.  V [B,H,Skv,D]
 * (strided) -> vt8 [B,H,D,Skv_pad] MXFP8 codes and/or vt4 [B,H,D,Skv_pad/2] MXFP4 codes (two per byte),
 * scale tiles v8_sf / v4_sf [B,H,Skv_pad/128,512] (rows = head-dim index, columns = the four 32-key
 * blocks of a 128-key tile).  Round-to-nearest-even elements (OCP MX rule).  No counterpart in the
 * reference, which keeps V in fp16 (ours/mxfp_attn_kernel.py:29-31).  fp8_fmt: 1 E5M2, 2 E4M3. */
int mpsa_quant_v_seq(const void* v, int in_dtype, int B, int H, int Skv, int D, int Skv_pad, long long vs_b,
                     long long vs_h, long long vs_l, int fp8_fmt, void* vt8, void* v8_sf, void* vt4, void* v4_sf,
                     void* stream);

/* Band-rule precision map uint8 [nq, nk] over tile x tile cells: FP8 iff the cell is within
 * `band` tiles of the (end-aligned) diagonal, else FP4; causal cells entirely above the diagonal
 * are SKIP.  The reference has no per-tile precision selection; the causal tile range follows
 * ours/online_routing.py:68-77. */
int mpsa_route_band(void* map, int nq, int nk, int tile, int causal, int band, int S, int Skv, void* stream);

/* Router statistic of every visible 128 x 128 score tile, computed from the MXFP4 operands:
 * stat[b,h,i,j] = mean over the query rows of the row maximum of S = Q4.K4^T (log2 domain, the softmax
 * scale is already folded into Q by the quantizer).  This is the quantity the reference's kernels compute
 * per tile as `sum(max(qk, 1)) / BLOCK_M` (ours/mxfp_attn_kernel.py:272-280, ours/online_routing.py:87-112).
 * Keys beyond Skv and, with causal != 0, keys above the query are left out of the row maximum; a row with no
 * visible key in the tile counts as 0.
 *   q4,k4 packed MXFP4 codes [B,H,L,64]; q4_sf,k4_sf tiled scales [B,H,ceil(L/128),512] (from mpsa_quant_mx)
 *   stat     float32 [B,Hq,ceil(S/128),ceil(Skv/128)], every cell written (0 above the causal diagonal)
 *   scratch  4 floats per cell of stat (16-byte aligned): the per-warp partial means, added in a fixed order
 *   status   device int32, stays 0 unless a wait expired. */
int mpsa_route_stat(const void* q4, const void* q4_sf, const void* k4, const void* k4_sf, void* stat, void* scratch,
                    int B, int Hq, int Hkv, int S, int Skv, int causal, int* status, void* stream);

/* Online precision map uint8 [B,Hq,nq,nk] (128 x 128 cells) from the statistic above: SKIP above the causal
 * diagonal, FP8 within `band` tiles of the diagonal, and elsewhere FP8 iff stat[i,j] >= stat[i,0] * tau, else
 * FP4.  The first key tile is the reference row statistic ("sink"), as in ours/mxfp_attn_kernel.py:272-276.
 * With use_skip != 0 the reference's own rule is applied on top: a tile outside the band is processed only if
 * it is the row's first one or stat[i,j] >= stat[i,0] * skip_tau (:276-297), otherwise it is SKIP. */
int mpsa_route_online(void* map, const void* stat, int B, int Hq, int S, int Skv, int causal, int band, float tau,
                      float skip_tau, int use_skip, void* stream);

/* Fused attention forward.  Replaces block_scaled_batched_attn (ours/mxfp_attn_kernel.py:362-423)
 * and its kernel (:103-359).
 *   q8/q4, k8/k4   codes from mpsa_quant_mx with D padded to 128: fp8 [B,H,L,128], fp4 packed [B,H,L,64]
 *   *_sf           tiled scales [B,H,ceil(L/128),512]
 *   pv_mode 0      P and V in fp16 (the reference's P.V precision): vt from mpsa_prepare_vt
 *   pv_mode 1      P re-quantised to the tile's format, V from mpsa_quant_v_seq (vt8, v8_sf, vt4, v4_sf)
 *   Skv_pad        keys per row of the V^T buffers (the value given to mpsa_prepare_vt / mpsa_quant_v_seq): any multiple
 *                  of 128 that is at least Skv
 *   map            uint8 [.., ceil(S/128), ceil(Skv/128)] with batch / head strides map_sb / map_sh (0 = shared)
 *                  (0 skip, 1 MXFP8, 2 FP4; a CTA walks only from the first to the last non-skipped tile of its row)
 *   out            [B,Hq,S,D] contiguous
 *   lse            optional fp32 [B,Hq,S]: log2 of each row's softmax denominator (for merging partial results)
 *   fp8_fmt        descriptor format of the fp8 codes: 0 E4M3, 1 E5M2
 *   fp4_kind       0: the FP4 operands of Q.K^T are MXFP4 (above).  1: NVFP4 from mpsa_quant_nvfp4_bh (q4/k4 the same
 *                  packed codes, q4_sf/k4_sf [B,H,ceil(L/128),2,512] E4M3 scale tiles); fp4_scale is then the product
 *                  of the two tensor scales, applied to the scores of the FP4 tiles.  P.V keeps the MX formats.
 *   range_flag     optional (pv_mode 1): one int32, 0 on entry, private to this call.  When given, the forward runs
 *                  with the row reference fixed after the first key tile (block-scaled P carries its magnitude in
 *                  the scale codes, so nothing has to be rescaled while scores stay within 2^64 of that reference);
 *                  a score beyond that sets the word, and the exact kernel, launched behind the first one, then
 *                  recomputes the output.  Results are the same either way.  NULL: the exact kernel only.
 *   acc_in, lse_in optional, together: an earlier partial result (fp32 [B,Hq,S,D], log2 denominators [B,Hq,S]) over OTHER keys;
 *                  out (fp32) and lse then receive the merged result (buffers distinct from the inputs), which saves
 *                  the separate mpsa_attn_merge pass
 *   status         one int32, must be 0 on entry; a kernel whose bounded waits expire stores a
 *                  non-zero code here (1 TMA, 2 MMA, 3 pipeline) and unwinds
 */
int mpsa_attn_fwd(const void* q8, const void* q8_sf, const void* q4, const void* q4_sf, const void* k8,
                  const void* k8_sf, const void* k4, const void* k4_sf, const void* vt, const void* vt8,
                  const void* v8_sf, const void* vt4, const void* v4_sf, int pv_mode, const void* map,
                  long long map_sb, long long map_sh, void* out, int out_dtype, void* lse, int B, int Hq, int Hkv,
                  int S, int Skv, int D, int Skv_pad, int causal, int fp8_fmt, int fp4_kind,
                  float fp4_scale, int* range_flag,
                  const void* acc_in, const void* lse_in, int* status, void* stream);

/* The fused forward with the online router inside it: what mpsa_route_stat + mpsa_route_online + mpsa_attn_fwd do together
 * for a causal problem with quantised P.V and MXFP4 operands, without the stand-alone statistic pass.  Replaces the same
 * reference code as mpsa_attn_fwd, with the tile router of ours/mxfp_attn_kernel.py:272-297 deciding precision.
 *   map           uint8 [B,Hq,nq,nk], OUTPUT: the precision map used (as mpsa_route_online with this band and tau writes it)
 *   band, tau     MXFP8 within `band` tiles of the diagonal; elsewhere MXFP8 iff statistic >= tau x the row's first tile's
 *   out           [B,Hq,S,D] of out_dtype
 *   lse, lse_final  fp32 [B,Hq,S]: log2 denominators of the result go to lse_final when it is given (another buffer than
 *                 lse), else to lse
 *   stat          optional fp32 [B,Hq,nq,nk], OUTPUT: the router statistic of every tile outside the band (the
 *                 other cells are left as they are); stat_scratch: unused, may be NULL
 *   range_flag    device int, zero on entry.  The forward runs with the row reference fixed after the first key tile; if a
 *                 score leaves its 2^64 headroom the word is set and the exact kernel, launched behind it, recomputes the
 *                 output over the final map (which does not depend on the reference) - same results either way.
 * Three launches: band map; the forward (a promoted tile's MXFP4 result is left out and the tile is done again in MXFP8 by
 * the same CTA after the row's own tiles); the conditional exact forward, whose CTAs return at once unless the word is set.
 * At most 4096 key tiles (512K keys).  Skv_pad, fp8_fmt, the operand pointers: as in mpsa_attn_fwd.
 *   stages        which of these to launch, a mask of 1 (band map), 2 (forward), 8 (conditional exact forward) (4 is
 *                 accepted and ignored); 15 for the operation itself, a subset for timing one stage alone. */
int mpsa_attn_fwd_routed(const void* q8, const void* q8_sf, const void* q4, const void* q4_sf, const void* k8,
                         const void* k8_sf, const void* k4, const void* k4_sf, const void* vt8, const void* v8_sf,
                         const void* vt4, const void* v4_sf, void* map, int band, float tau, void* out, int out_dtype,
                         void* lse, void* lse_final, void* stat, void* stat_scratch, int B, int Hq, int Hkv, int S, int Skv,
                         int D, int Skv_pad, int fp8_fmt, int stages, int* range_flag, int* status, void* stream);

/* Merges a partial attention result into an accumulator: acc fp32 [rows, D] and lse_acc fp32 [rows] are
 * updated in place with part [rows, D] (part_dtype 0 f32, 1 f16, 2 bf16) and lse_part, where every lse is
 * log2 of the softmax denominator of its (disjoint) key set as written by mpsa_attn_fwd; rows with
 * lse = -inf carry no keys.  Used by the sequence-parallel ring, which has no counterpart in the
 * reference (its kernel sees all keys in one launch, ours/mxfp_attn_kernel.py:245). */
int mpsa_attn_merge(void* acc, void* lse_acc, const void* part, int part_dtype, const void* lse_part, long long rows,
                    int D, void* stream);

/* C[M,N] = alpha * (A . sa)(B . sb)^T.  Replaces block_scaled_matmul (ours/block_scaled_matmul.py:271-296)
 * and its kernel (:154-267).
 *   a [M, K/epb] and b [N, K/epb] bytes with row pitches lda_bytes / ldb_bytes (K-major)
 *   a_scale [ceil(M/128), K/vec/4, 32,4,4], b_scale [ceil(N/128), K/vec/4, 32,4,4]
 *   mode 0 MXFP8 (a_fmt/b_fmt: 0 E4M3, 1 E5M2; vec 32, E8M0), 1 MXFP4 (vec 32, E8M0),
 *        2 NVFP4 (vec 16, E4M3 scales; pass the product of the two tensor scales as alpha)
 *   c [M, ldc] of out_dtype;  status as in mpsa_attn_fwd */
int mpsa_gemm_block_scaled(const void* a, const void* a_scale, const void* b, const void* b_scale, void* c, int M,
                           int N, int K, long long lda_bytes, long long ldb_bytes, long long ldc, int mode,
                           int a_fmt, int b_fmt, int out_dtype, float alpha, int* status, void* stream);

/* The same product for `batch` independent problems laid out one after the other, all contiguous:
 * a [batch,M,K/epb], b [batch,N,K/epb], scale tiles [batch,ceil(rows/128),K/vec/4,512], c [batch,M,N].
 * Replaces block_scaled_batched_matmul (ours/batched_block_scaled_matmul.py:183-236) with batch = B*H. */
int mpsa_gemm_block_scaled_batched(const void* a, const void* a_scale, const void* b, const void* b_scale, void* c,
                                   int batch, int M, int N, int K, int mode, int a_fmt, int b_fmt, int out_dtype,
                                   float alpha, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MPSA_H_ */
