"""Benchmark of the diagonal-tiled mixed-precision attention forward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--seq 32768]

Workload (N=1): causal prefill attention shaped like a Llama-3-8B layer - B=1, Hq=32, Hkv=8,
D=128, S=32768, bf16 inputs N(0,1) with 5 of the 128 K channels scaled x20, diagonal tiles in
MXFP8 and the rest in MXFP4 unless the online router promotes them (statistic of the MXFP4 score tile >=
TAU x that of the row's first key tile), P re-quantised to the tile's format before P.V (V quantised along
the sequence).  One step = quantise Q and K (both formats, one pass each), quantise V and run the fused forward
with the router inside it (band map, the forward - a promoted tile is done again in MXFP8 at the end of its row - and
the exact forward behind it as its conditional fallback, whose CTAs return at once).  Metric: effective attention TFLOP/s =
4*B*Hq*S^2*D/2 / time.  With N > 1 every rank runs the same workload on its own batch element
(batch x head sharding, no collective; weak scaling) and the value is the sum over ranks divided by
the slowest rank's time.

`--impl reference` times the CPU restatement of the reference's algorithm (the oracle) on the host
cores, on a bounded sample of the same workload.

Other workloads (their own JSON line, not the headline): `--workload ring [--layout zigzag|contiguous]
[--exchange gather|ring]` - one causal sequence of 131072 tokens sharded over the ranks (strong scaling);
`--workload gemm [--size 8192]` - the stand-alone block-scaled GEMM in MXFP8, MXFP4 and NVFP4 (the default line carries
the same figures in its `gemm` object);
`--workload refcmp --reference-dir DIR` - the reference's own Triton kernels (imported unmodified from DIR, a
checkout of the reference project) timed beside this library's on the same GPU and the same operands.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "mp-sparse-attn_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

HQ, HKV, D = 32, 8, 128
OUTLIERS = 5
LAUNCHES_PER_STEP = 6      # quant Q, quant K, quant V, band map, forward, conditional exact forward (returns at once)
TAU = 1.1                  # online router: a tile is promoted to MXFP8 iff its statistic >= TAU x the first key tile's
# DRAM bytes (read + written) of one launch of the fused forward at S=8192, from an ncu capture; every term of it
# (Q, K, V codes and scales, the output) grows linearly with S
ATTN_TRAFFIC_BYTES_S8192 = 107_451_904


def attn_flops(B, Hq, S, Dh, causal=True):
    return 4.0 * B * Hq * S * S * Dh * (0.5 if causal else 1.0)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_inputs(seed, S, device, outliers=OUTLIERS, hq=HQ, hkv=HKV):
    """The workload's seeded tensors: a CPU generator draws fp32 N(0,1) Q, K, V in that order, then the indices of the
    outlier K channels (scaled x20); everything is cast to bf16 and copied to the device.  The parity tests draw the same
    bits, so a slice of this very workload can be handed to the CPU oracle."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(1, hq, S, D, generator=g)
    k = torch.randn(1, hkv, S, D, generator=g)
    v = torch.randn(1, hkv, S, D, generator=g)
    if outliers:
        idx = torch.randperm(D, generator=g)[:outliers]
        k[..., idx] *= 20.0
    return tuple(t.to(torch.bfloat16).to(device) for t in (q, k, v))


def run_ours(args):
    import mpsa
    from ours.mxfp_attn_kernel import mxfp_attn_kernel
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    S, K, W = args.seq or 32768, args.steps, args.warmup
    q, k, v = make_inputs(2 + rank, S, dev)

    def step():
        return mpsa.attention_forward(q, k, v, causal=True, out_dtype=torch.bfloat16, pv_mode="requant",
                                      router="online", tau=TAU)

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.5)            # let nvidia-smi come up so that its samples cover the timed region
    for _ in range(W):
        out = step()
    mpsa.check_status(dev)
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        out = step()
    e1.record()
    sync_all()
    ms = e0.elapsed_time(e1)
    mpsa.check_status(dev)

    # ---- dominant kernel alone (fused forward), operands already quantised -------------
    sq = mpsa.ops.q_side_scale(D)
    qq, kq = mpsa.quantize_mx(q, sq), mpsa.quantize_mx(k, 1.0)
    stat = mpsa.router_statistic(qq, kq, 1, HQ, HKV, S, S, causal=True)
    pm = mpsa.precision_map_online(stat, S, S, causal=True, band=1, tau=TAU)
    n_fp8 = int((pm == mpsa.TILE_FP8).sum())
    n_fp4 = int((pm == mpsa.TILE_FP4).sum())

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(K):
            fn()
        a1.record()
        torch.cuda.synchronize()
        return a0.elapsed_time(a1) / K

    route_ms = timed(lambda: mpsa.precision_map_online(mpsa.router_statistic(qq, kq, 1, HQ, HKV, S, S, causal=True),
                                                       S, S, causal=True, band=1, tau=TAU))
    del stat

    def time_forward(vt):
        for _ in range(2):
            mpsa.attention_forward_quantized(qq, kq, vt, 1, HQ, HKV, S, S, D, causal=True, prec_map=pm)
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(K):
            mpsa.attention_forward_quantized(qq, kq, vt, 1, HQ, HKV, S, S, D, causal=True, prec_map=pm)
        a1.record()
        torch.cuda.synchronize()
        return a0.elapsed_time(a1) / K

    vt = mpsa.quantize_v_seq(v)
    plain_ms = time_forward(vt)                  # one launch over the final map (no router inside)
    # the dominant kernel of the step: the routed forward (router inside; the band-map launch before it
    # takes a few microseconds and is inside the bracket), and the whole routed forward
    attn_ms = timed(lambda: mpsa.attention_forward_routed(qq, kq, vt, 1, HQ, HKV, S, S, D, band=1, tau=TAU, stages=3))
    routed_ms = timed(lambda: mpsa.attention_forward_routed(qq, kq, vt, 1, HQ, HKV, S, S, D, band=1, tau=TAU))
    band = mpsa.precision_map_band(S, S, True, 1, 128, dev)
    n_band = int((band == mpsa.TILE_FP8).sum()) * HQ
    n_promoted = n_fp8 - n_band
    vt = mpsa.prepare_vt(v)
    attn_fp16_ms = time_forward(vt)              # the reference's P.V precision (P and V in fp16)
    # quantizer alone (Q operand, both formats): HBM-bound leg
    torch.cuda.synchronize()
    b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    b0.record()
    for _ in range(K):
        mpsa.quantize_mx(q, sq)
    b1.record()
    torch.cuda.synchronize()
    quant_ms = b0.elapsed_time(b1) / K
    del qq, kq, vt
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end through the reference-facing call, host buffers ---------------------
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    hout = torch.empty((1, HQ, S, D), dtype=torch.bfloat16).pin_memory()
    del q, k, v, out

    def e2e_step():
        # host tensors in, host tensor out: the call streams the (batch, KV group) chunks through the GPU
        mxfp_attn_kernel(hq, hk, hv, is_causal=True, block_scale_type="online_requant", promote_thresh=TAU,
                         output_dtype=torch.bfloat16, out=hout)

    for _ in range(max(1, min(W, 2))):
        e2e_step()
    sync_all()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    for _ in range(K):
        e2e_step()
    c1.record()
    sync_all()
    e2e_ms = c0.elapsed_time(c1)
    mpsa.check_status(dev)

    if dist is not None:
        t = torch.tensor([ms, e2e_ms, attn_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, attn_ms = (float(x) for x in t.tolist())
    seq_par = None
    if dist is not None:
        del hq, hk, hv, hout
        torch.cuda.empty_cache()
        seq_par = seq_parallel_leg(dist, dev, rank, world, K)
    flops_rank = attn_flops(1, HQ, S, D)
    value = world * flops_rank * K / (ms * 1e-3) / 1e12
    e2e_value = world * flops_rank * K / (e2e_ms * 1e-3) / 1e12
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return
    pk = measured_peaks()
    # blended tensor peak: both products of a diagonal tile at the MXFP8 rate (2x the measured bf16
    # rate), both products of an off-diagonal tile at the MXFP4 rate (4x)
    # work the forward executes: both products of the band tiles and of the promoted tiles (MXFP8 rate), both products
    # of the MXFP4 tiles it keeps and the score product of the promoted ones, whose MXFP4 result is left out (MXFP4 rate)
    f_tile = 2.0 * 128 * 128 * D
    executed = (n_band + n_promoted + n_fp4) * 2 * f_tile + n_promoted * f_tile

    def blended(base_tflops):
        t_peak = (n_band + n_promoted) * 2 * f_tile / (2 * base_tflops * 1e12) + (n_fp4 * 2 + n_promoted) * f_tile / (4 * base_tflops * 1e12)
        return executed / t_peak / 1e12
    # the forward is timed alone, back to back: the burst figure is its denominator; the sustained one is given beside it
    peak_tflops, peak_sustained = blended(pk["bf16"]), blended(pk["bf16_sustained"])
    achieved = executed / (attn_ms * 1e-3) / 1e12
    line = {
        "metric": "effective attn TFLOPS, Llama-3-8B shape causal", "value": round(value, 3), "unit": "TFLOP/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "mxfp8/mxfp4 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": f"cfg3 causal prefill B=1 Hq=32 Hkv=8 D=128 S={S} per GPU, diag MXFP8 / off-diag MXFP4 with online "
                               f"promotion to MXFP8 (tau={TAU}), P re-quantised to the tile's format before P.V", "seq_len": S,
                   "router": {"kind": "online, inside the forward", "tau": TAU, "fp8_tiles": n_fp8, "fp4_tiles": n_fp4,
                              "stand_alone_statistic_pass_ms": round(route_ms, 4)}, "l2": "inputs (403 MB per step) larger than L2",
                   "sharding": "batch x head replicas, no collective"},
        "roofline": {"bound": "tensor", "kernel": "attn_fwd_kernel (the routed forward: router inside, promoted tiles done again in MXFP8 at the end of their row)", "achieved": round(achieved, 2),
                     "peak": round(peak_tflops, 1), "unit": "TFLOP/s", "frac": round(achieved / peak_tflops, 4),
                     "traffic": ATTN_TRAFFIC_BYTES_S8192 * S // 8192, "ms": round(attn_ms, 4),
                     "peak_source": pk["source"] + " bf16 burst x2 (MXFP8 tiles) / x4 (MXFP4 tiles), blended by executed tiles",
                     "frac_of_sustained_peak": round(achieved / peak_sustained, 4), "peak_sustained": round(peak_sustained, 1),
                     "routed_forward_ms": round(routed_ms, 4), "promoted_tiles": n_promoted,
                     "single_launch_over_final_map_ms": round(plain_ms, 4),
                     "effective_tflops": round(flops_rank / (routed_ms * 1e-3) / 1e12, 2),
                     "fp16_pv_variant": {"ms": round(attn_fp16_ms, 4), "effective_tflops": round(flops_rank / (attn_fp16_ms * 1e-3) / 1e12, 2)},
                     "quantizer": {"bound": "hbm", "achieved": round(HQ * S * D * (2 + 1 + 0.5 + 2 / 32) / (quant_ms * 1e-3) / 1e9, 1),
                                   "peak": pk["hbm_gbs"], "unit": "GB/s", "ms": round(quant_ms, 4)}},
        "e2e": {"value": round(e2e_value, 3), "unit": "TFLOP/s", "ms_per_step": round(e2e_ms / K, 3),
                "h2d_bytes_per_step": (HQ + 2 * HKV) * S * D * 2, "d2h_bytes_per_step": HQ * S * D * 2},
        "gpu_launches": LAUNCHES_PER_STEP * K,
        "clocks": clocks,
    }
    if seq_par is not None:
        line["seq_parallel"] = seq_par
    # the stand-alone block-scaled GEMM (cfg2, M=N=K=8192) beside the headline: 20 launches per variant after 3 warm-up
    # launches, outside every timed region above; fractions are of 2x (MXFP8) / 4x (FP4) the measured bf16 burst peak
    gres, _ = gemm_variants(dev, 8192, 20, 3)
    line["gemm"] = {"workload": "cfg2 GEMM M=N=K=8192, operands quantised along K, bf16 out", "variants": gres}
    line["cpu_baseline"] = cpu_baseline(steps=1, warmup=0, budget_s=20.0)
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def seq_parallel_leg(dist, dev, rank, world, steps, S=131072):
    """The long-context configuration inside the headline run (N > 1 only): one causal sequence of S tokens, B=1 Hq=32
    Hkv=8 D=128, sharded over the ranks in the balanced zigzag layout; every rank quantises its slice once and the MXFP4
    K/V payloads are exchanged over NCCL, (a) by send/recv round the ring with the next block in flight while the current
    one is consumed, (b) by one all-gather behind the diagonal launches.  Times are the maximum over ranks; the
    denominator of the strong-scaling efficiency is measured in the same run: rank 0 alone does the whole sequence."""
    import mpsa
    from mpsa.ring import ring_attention
    s_local = S // world
    g = torch.Generator(device=dev).manual_seed(4 + rank)
    q = torch.randn(1, HQ, s_local, D, generator=g, device=dev).to(torch.bfloat16)
    k = torch.randn(1, HKV, s_local, D, generator=g, device=dev).to(torch.bfloat16)
    v = torch.randn(1, HKV, s_local, D, generator=g, device=dev).to(torch.bfloat16)

    def sync_all():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        for _ in range(2):
            fn()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        sync_all()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    n = max(2, min(steps, 5))
    res = {"S": S, "layout": "zigzag", "steps": n}
    for exchange in ("ring", "gather"):
        res[exchange + "_ms"] = round(timed(lambda: ring_attention(q, k, v, causal=True, layout="zigzag", exchange=exchange), n), 3)
    mpsa.check_status(dev)
    del q, k, v
    # the same sequence on ONE GPU (rank 0; the others wait at the barrier): the strong-scaling denominator
    solo = dist.new_group([0])
    n1 = torch.zeros(1, device=dev)
    if rank == 0:
        g = torch.Generator(device=dev).manual_seed(4)
        q = torch.randn(1, HQ, S, D, generator=g, device=dev).to(torch.bfloat16)
        k = torch.randn(1, HKV, S, D, generator=g, device=dev).to(torch.bfloat16)
        v = torch.randn(1, HKV, S, D, generator=g, device=dev).to(torch.bfloat16)
        f = lambda: ring_attention(q, k, v, causal=True, layout="zigzag", exchange="ring", group=solo)
        f()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(2):
            f()
        e1.record()
        torch.cuda.synchronize()
        n1[0] = e0.elapsed_time(e1) / 2
        del q, k, v
    dist.broadcast(n1, 0)
    sync_all()
    res["n1_ms"] = round(float(n1.item()), 3)
    best = min(res["ring_ms"], res["gather_ms"])
    res["strong_efficiency"] = {"ring": round(res["n1_ms"] / (world * res["ring_ms"]), 4),
                                "gather": round(res["n1_ms"] / (world * res["gather_ms"]), 4)}
    res["tflops"] = round(attn_flops(1, HQ, S, D) / (best * 1e-3) / 1e12, 1)
    return res


def run_ring(args):
    """Long-context causal attention, B=1 Hq=32 Hkv=8 D=128 S=131072, sequence-sharded over the GPUs: every
    rank quantises its slice once and the MXFP4 K/V blocks are exchanged over NCCL, by one all-gather (default) or
    by send/recv round a ring (strong scaling)."""
    import torch.distributed as dist
    import mpsa
    from mpsa.ring import RingSchedule, ring_attention
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    else:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    S = args.seq or 131072
    sched = RingSchedule(world, rank, args.layout, True)
    s_local = S // world
    g = torch.Generator(device=dev).manual_seed(4 + rank)
    q = torch.randn(1, HQ, s_local, D, generator=g, device=dev).to(torch.bfloat16)
    k = torch.randn(1, HKV, s_local, D, generator=g, device=dev).to(torch.bfloat16)
    v = torch.randn(1, HKV, s_local, D, generator=g, device=dev).to(torch.bfloat16)
    K, W = args.steps, args.warmup

    def sync_all():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    for _ in range(W):
        ring_attention(q, k, v, causal=True, layout=args.layout, exchange=args.exchange)
    mpsa.check_status(dev)
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        ring_attention(q, k, v, causal=True, layout=args.layout, exchange=args.exchange)
    e1.record()
    sync_all()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    mpsa.check_status(dev)
    if rank == 0:
        flops = attn_flops(1, HQ, S, D)
        print(json.dumps({
            "metric": "effective attn TFLOPS, Llama-3-8B shape causal, sequence-parallel ring", "value": round(flops * K / (ms * 1e-3) / 1e12, 3),
            "unit": "TFLOP/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(ms / K, 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "mxfp8/mxfp4 (fp32 accumulate)",
            "data": "synthetic", "config": {"workload": f"cfg5 causal B=1 Hq=32 Hkv=8 D=128 S={S} sequence-sharded, "
                                                        f"{args.layout} ownership, MXFP4 K/V " + ("ring (send/recv)" if args.exchange == "ring" else "all-gather") + " over NCCL",
                                            "work_units_per_rank": sched.work_units()}}))
    dist.destroy_process_group()


def cpu_baseline(steps=1, warmup=0, budget_s=25.0):
    """The oracle (CPU restatement of the reference's algorithm, PyTorch on all host cores) doing what one step of the
    GPU arm does on a bounded sample of the workload: quantise Q and K, router statistic from the MXFP4 product, online
    precision map, both products emulated tile by tile, softmax, P re-quantised, P.V.  The sample (sequence length
    2048..8192, 1..8 KV groups of the workload's head layout, 4 or 1 query heads per group) is the largest one whose
    predicted time - scaled from a small calibration pass by S^2 x heads - fits budget_s / (steps + warmup)."""
    from oracle import mx_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)

    def one_pass(q, k, v):
        S = q.shape[2]
        stat = O.router_statistic_map(q, k, causal=True)
        pm = O.precision_map_online(stat, S, S, causal=True, band=1, tau=TAU)
        return O.attention_mxfp(q, k, v, causal=True, prec_map=pm, pv_mode="requant")

    S0 = 2048
    q, k, v = O.make_qkv(2, 1, 4, 1, S0, D, outliers=OUTLIERS)
    t0 = time.perf_counter()
    one_pass(q, k, v)
    t_cal = time.perf_counter() - t0                 # 4 query heads, 1 KV group, S0
    per_pass = budget_s / max(1, steps + warmup)
    S, groups, hq = S0, 1, 1
    found = False
    for s_ in (8192, 4096, 2048):
        for g_ in (8, 4, 2, 1):
            for h_ in (4, 1):
                if not found and t_cal * (s_ / S0) ** 2 * g_ * (h_ / 4.0) <= per_pass:
                    S, groups, hq, found = s_, g_, h_, True
    q, k, v = O.make_qkv(2, 1, HQ, HKV, S, D, outliers=OUTLIERS)
    q = torch.cat([q[:, 4 * g:4 * g + hq] for g in range(groups)], dim=1)
    k, v = k[:, :groups], v[:, :groups]
    for _ in range(warmup):
        one_pass(q, k, v)
    t0 = time.perf_counter()
    for _ in range(steps):
        one_pass(q, k, v)
    dt = (time.perf_counter() - t0) / steps
    val = attn_flops(1, hq * groups, S, D) / dt / 1e12
    return {"value": round(val, 5), "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"B=1 Hq={hq * groups} Hkv={groups} D={D} S={S} causal (of the workload's 32 query heads in 8 KV groups at "
                      f"S=32768), online router tau={TAU}, re-quantised P.V, {dt:.2f} s per pass", "seconds": round(dt, 3)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = cpu_baseline(steps=max(1, args.steps), warmup=min(args.warmup, 1), budget_s=120.0)
    line = {
        "impl": "reference", "metric": "effective attn TFLOPS, Llama-3-8B shape causal", "value": base["value"],
        "unit": "TFLOP/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(base["seconds"] * 1e3, 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "mxfp8/mxfp4 emulated in fp32", "data": "synthetic",
        "config": {"workload": f"cfg3 causal prefill B=1 Hq=32 Hkv=8 D=128 S={args.seq or 32768} (bounded sample, see cpu_baseline.sample)"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def gemm_variants(dev, n, K, W):
    """The three block-scaled GEMM variants and the library bf16 GEMM at M = N = K = n: bf16 N(0,1) operands from seed 1
    quantised along K, K timed launches each after max(W, 3) warm-up launches, CUDA events."""
    import mpsa
    g = torch.Generator(device=dev).manual_seed(1)
    a = torch.randn(n, n, generator=g, device=dev).to(torch.bfloat16)
    b = torch.randn(n, n, generator=g, device=dev).to(torch.bfloat16)
    qa, qb = mpsa.quantize_mx(a.view(1, 1, n, n), 1.0), mpsa.quantize_mx(b.view(1, 1, n, n), 1.0)
    na, sa, tsa = mpsa.quantize_nvfp4(a)
    nb, sb, tsb = mpsa.quantize_nvfp4(b)
    alpha = float(tsa.item()) * float(tsb.item())

    def timed(fn):
        for _ in range(max(W, 3)):
            fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / K

    variants = {
        "mxfp8": lambda: mpsa.gemm_block_scaled(qa.fp8.view(n, n), qa.fp8_sf, qb.fp8.view(n, n), qb.fp8_sf, torch.bfloat16, n, n, n, "mxfp8"),
        "mxfp4": lambda: mpsa.gemm_block_scaled(qa.fp4.view(n, n // 2), qa.fp4_sf, qb.fp4.view(n, n // 2), qb.fp4_sf, torch.bfloat16, n, n, n, "mxfp4"),
        "nvfp4": lambda: mpsa.gemm_block_scaled(na, sa, nb, sb, torch.bfloat16, n, n, n, "nvfp4", alpha=alpha),
    }
    pk = measured_peaks()
    flops = 2.0 * n * n * n
    res = {}
    for name, fn in variants.items():
        ms = timed(fn)
        mult = 2.0 if name == "mxfp8" else 4.0
        res[name] = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
                     "frac_of_peak": round(flops / ms / 1e9 / (mult * pk["bf16"]), 4)}
    mpsa.check_status(dev)
    ms = timed(lambda: a @ b.T)
    res["library_bf16"] = {"ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1)}
    return res, pk


def run_gemm(args):
    """Standalone block-scaled GEMM C[M,N] = A[M,K] . B[N,K]^T, M = N = K = --size (default 8192); prints one JSON
    line with the three variants and the library bf16 GEMM of the same shape beside them."""
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    n = args.size
    K, W = args.steps, args.warmup
    res, pk = gemm_variants(dev, n, K, W)
    print(json.dumps({"metric": "block-scaled GEMM TFLOPS", "unit": "TFLOP/s", "value": res["mxfp8"]["tflops"], "n_gpus": 1,
                      "steps": K, "warmup": max(W, 3), "higher_is_better": True, "dtype": "mxfp8 / mxfp4 / nvfp4 (fp32 accumulate)",
                      "data": "synthetic", "config": {"workload": f"cfg2 GEMM M=N=K={n}, operands quantised along K, bf16 out"},
                      "variants": res, "peak": {"bf16_burst_tflops": pk["bf16"], "mxfp8": "2x", "fp4": "4x", "source": pk["source"]},
                      "gpu_launches": 3 * K}))


def run_refcmp(args):
    """The reference's Triton kernels beside this library's, same process, same operands, CUDA events:
    block_scaled_matmul "mxfp8" at M=N=K=--size (ours/block_scaled_matmul.py:271-296); the fused attention in its
    "mxfp8" mode, non-causal, equal head counts, D=128 - the one shape family the reference kernel handles
    (ours/mxfp_attn_kernel.py:19-74, :362-423) - kernel alone and whole wrapper; quant_mxfp4 / quant_mxfp8e5 on the
    Llama-shaped Q and K (ours/quant_mxint8.py:453-512, :223-272).  The reference's MXFP4 attention mode packs the
    wrong axis and reads out of bounds, and its "nvfp4" GEMM mode does not compile: neither is run."""
    ref_dir = args.reference_dir or os.environ.get("MPSA_REFERENCE_DIR")
    if not ref_dir or not os.path.isdir(os.path.join(ref_dir, "ours")):
        raise SystemExit("--workload refcmp needs --reference-dir (or MPSA_REFERENCE_DIR): a checkout of the reference project")
    import importlib
    import torch._dynamo  # noqa: F401  (the reference's decorators pull it in; it must be imported before `ours` is swapped)
    import mpsa
    import ours.quant_mxint8 as our_quant
    from ours.mxfp_attn_kernel import mxfp_attn_kernel as our_attn
    # The reference's package is a directory `ours` without __init__.py and this library's mirror has the same name:
    # import the reference modules with only the reference checkout on the path, then put everything back.
    saved = {n: m for n, m in sys.modules.items() if n == "ours" or n.startswith("ours.")}
    for n in saved:
        del sys.modules[n]
    saved_path = list(sys.path)
    sys.path[:] = [ref_dir] + [p for p in saved_path if not os.path.isdir(os.path.join(p or ".", "ours"))]
    try:
        ref_quant = importlib.import_module("ours.quant_mxint8")
        ref_attn = importlib.import_module("ours.mxfp_attn_kernel")
        ref_gemm = importlib.import_module("ours.block_scaled_matmul")
    finally:
        sys.path[:] = saved_path
        for n in [n for n in sys.modules if n == "ours" or n.startswith("ours.")]:
            del sys.modules[n]
        sys.modules.update(saved)
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    K, W = args.steps, max(args.warmup, 3)
    sampler = ClockSampler(0)
    sampler.start()

    def timed(fn, steps=K):
        for _ in range(W):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    res = {}
    # ---- GEMM, mxfp8 ----
    n = args.size
    g = torch.Generator(device=dev).manual_seed(1)
    a = torch.randn(n, n, generator=g, device=dev).to(torch.bfloat16)
    b = torch.randn(n, n, generator=g, device=dev).to(torch.bfloat16)
    qa, qb = mpsa.quantize_mx(a.view(1, 1, n, n), 1.0, want_fp4=False), mpsa.quantize_mx(b.view(1, 1, n, n), 1.0, want_fp4=False)
    a8, b8 = qa.fp8.view(n, n).view(torch.float8_e5m2), qb.fp8.view(n, n).view(torch.float8_e5m2)
    sa, sb = qa.fp8_sf.view(n // 128, n // 128, 32, 4, 4), qb.fp8_sf.view(n // 128, n // 128, 32, 4, 4)
    cfg = {"BLOCK_SIZE_M": 128, "BLOCK_SIZE_N": 256, "BLOCK_SIZE_K": 128, "num_stages": 4, "ELEM_PER_BYTE_A": 1,
           "ELEM_PER_BYTE_B": 1, "VEC_SIZE": 32}
    c_ref = ref_gemm.block_scaled_matmul(a8, sa, b8, sb, torch.float16, n, n, n, cfg)
    c_our = mpsa.gemm_block_scaled(a8, sa, b8, sb, torch.float16, n, n, n, "mxfp8")
    flops = 2.0 * n ** 3
    t_ref = timed(lambda: ref_gemm.block_scaled_matmul(a8, sa, b8, sb, torch.float16, n, n, n, cfg))
    t_our = timed(lambda: mpsa.gemm_block_scaled(a8, sa, b8, sb, torch.float16, n, n, n, "mxfp8"))
    d = (c_ref.float() - c_our.float())
    res["gemm_mxfp8"] = {"shape": f"M=N=K={n}", "reference_ms": round(t_ref, 4), "ours_ms": round(t_our, 4),
                         "reference_tflops": round(flops / t_ref / 1e9, 1), "ours_tflops": round(flops / t_our / 1e9, 1),
                         "rel_l2_between": float(d.norm() / c_ref.float().norm())}
    del a, b, qa, qb, a8, b8, sa, sb, c_ref, c_our, d
    # ---- attention, mxfp8 mode, non-causal, equal head counts ----
    for S in args.refcmp_seq:
        H = 32
        g = torch.Generator(device=dev).manual_seed(2)
        q = torch.randn(1, H, S, D, generator=g, device=dev).to(torch.float16)
        k = torch.randn(1, H, S, D, generator=g, device=dev).to(torch.float16)
        v = torch.randn(1, H, S, D, generator=g, device=dev).to(torch.float16)
        o_ref = ref_attn.mxfp_attn_kernel(q, k, v, is_causal=False, block_scale_type="mxfp8", skip_thresh=-1e9)
        o_our = our_attn(q, k, v, is_causal=False, block_scale_type="mxfp8", output_dtype=torch.float16)
        dd = o_ref.float() - o_our.float()
        cos = float((o_ref.float().flatten() @ o_our.float().flatten()) / (o_ref.float().norm() * o_our.float().norm()))
        steps = max(2, min(K, 10))
        t_ref = timed(lambda: ref_attn.mxfp_attn_kernel(q, k, v, is_causal=False, block_scale_type="mxfp8", skip_thresh=-1e9), steps)
        t_our = timed(lambda: our_attn(q, k, v, is_causal=False, block_scale_type="mxfp8", output_dtype=torch.float16), steps)
        # the fused kernels alone, operands already quantised
        a8r, sar, b8r, sbr = ref_quant.quant_mxfp8e5(q, k)
        sar = sar.reshape(1, H, S // 128, 4, 32, 1, 4).permute(0, 1, 2, 5, 4, 3, 6).contiguous()
        sbr = sbr.reshape(1, H, S // 128, 4, 32, 1, 4).permute(0, 1, 2, 5, 4, 3, 6).contiguous()
        rcfg = {"BLOCK_SIZE_M": 128, "BLOCK_SIZE_N": 128, "BLOCK_SIZE_K": 128, "num_stages": 1, "ELEM_PER_BYTE_A": 1,
                "ELEM_PER_BYTE_B": 1, "VEC_SIZE": 32}
        tk_ref = timed(lambda: ref_attn.block_scaled_batched_attn(a8r, sar, b8r, sbr, v, torch.float16, 1, H, S, S, D, rcfg, skip_thresh=-1e9), steps)
        del a8r, sar, b8r, sbr
        qq = mpsa.quantize_mx(q, mpsa.ops.q_side_scale(D), want_fp4=False)
        kq = mpsa.quantize_mx(k, 1.0, want_fp4=False)
        vt = mpsa.prepare_vt(v)
        tk_our = timed(lambda: mpsa.attention_forward_quantized(qq, kq, vt, 1, H, H, S, S, D, causal=False, uniform="fp8",
                                                                out_dtype=torch.float16), steps)
        fl = attn_flops(1, H, S, D, causal=False)
        res[f"attn_mxfp8_S{S}"] = {
            "shape": f"B=1 H={H} S={S} D={D} non-causal, fp16 P.V", "reference_ms": round(t_ref, 3), "ours_ms": round(t_our, 3),
            "reference_kernel_ms": round(tk_ref, 3), "ours_kernel_ms": round(tk_our, 3),
            "reference_kernel_tflops": round(fl / tk_ref / 1e9, 1), "ours_kernel_tflops": round(fl / tk_our / 1e9, 1),
            "cos_between": cos, "rel_l2_between": float(dd.norm() / o_ref.float().norm())}
        del q, k, v, o_ref, o_our, dd, qq, kq, vt
    # ---- quantizers on the Llama-shaped operands ----
    S = args.seq or 32768
    g = torch.Generator(device=dev).manual_seed(2)
    q = torch.randn(1, HQ, S, D, generator=g, device=dev).to(torch.bfloat16)
    k = torch.randn(1, HKV, S, D, generator=g, device=dev).to(torch.bfloat16)
    elems = (HQ + HKV) * S * D
    for name in ("quant_mxfp4", "quant_mxfp8e5"):
        rf, of = getattr(ref_quant, name), getattr(our_quant, name)
        r, o = rf(q, k), of(q, k)
        same = all(bool(torch.equal(x.view(torch.uint8), y.view(torch.uint8))) for x, y in zip(r, o))
        t_ref, t_our = timed(lambda: rf(q, k)), timed(lambda: of(q, k))
        by = elems * (2 + 1 + 1 / 32)              # 16-bit in, one byte per element out, one scale byte per 32
        res[name] = {"shape": f"Q [1,{HQ},{S},{D}] + K [1,{HKV},{S},{D}] bf16, reference output format",
                     "reference_ms": round(t_ref, 4), "ours_ms": round(t_our, 4), "reference_gbs": round(by / t_ref / 1e6, 1),
                     "ours_gbs": round(by / t_our / 1e6, 1), "bit_identical": same}
        del r, o
    mpsa.check_status(dev)
    print(json.dumps({"workload": "reference Triton kernels beside this library, one B200", "steps": K, "warmup": W,
                      "results": res, "clocks": sampler.stop(), "peaks": measured_peaks()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seq", type=int, default=None, help="sequence length (default 32768; 131072 for --workload ring)")
    ap.add_argument("--workload", default="prefill", choices=["prefill", "ring", "gemm", "refcmp"],
                    help="prefill: the headline single-GPU workload replicated per GPU; ring: S=131072 causal, "
                         "sequence-sharded over the GPUs (strong scaling); gemm: the standalone block-scaled GEMM (1 GPU)")
    ap.add_argument("--size", type=int, default=8192, help="M = N = K of --workload gemm")
    ap.add_argument("--reference-dir", default=None, help="refcmp: checkout of the reference project (default $MPSA_REFERENCE_DIR)")
    ap.add_argument("--refcmp-seq", type=int, nargs="+", default=[8192], help="refcmp: sequence lengths of the attention comparison")
    ap.add_argument("--layout", default="zigzag", choices=["contiguous", "zigzag"])
    ap.add_argument("--exchange", default="gather", choices=["ring", "gather"],
                    help="ring workload: K/V blocks by send/recv round the ring, or one all-gather")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    if args.workload == "ring":
        run_ring(args)
    elif args.workload == "gemm":
        run_gemm(args)
    elif args.workload == "refcmp":
        run_refcmp(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
