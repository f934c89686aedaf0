"""Sequence-parallel ring on real GPUs (one process per GPU, NCCL): each rank's output slice must equal the
single-GPU fused forward on the whole sequence.  Needs at least two GPUs."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, layout, exchange, lengths, ret):
    for p in (ROOT, os.path.join(ROOT, "mp-sparse-attn_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    import torch.distributed as dist
    import mpsa
    from mpsa.ring import RingSchedule, ring_attention
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        worst = 0.0
        for S in lengths:                          # several lengths in one process: per-length state must not leak
            g = torch.Generator().manual_seed(4)
            B, Hq, Hkv, D = 1, 8, 2, 128
            q = torch.randn(B, Hq, S, D, generator=g).to(torch.bfloat16).cuda()
            k = torch.randn(B, Hkv, S, D, generator=g).to(torch.bfloat16).cuda()
            v = torch.randn(B, Hkv, S, D, generator=g).to(torch.bfloat16).cuda()
            full = mpsa.attention_forward(q, k, v, causal=True, pv_mode="requant", out_dtype=torch.float32, check=True)
            sched = RingSchedule(world, rank, layout, True)
            rows = S // sched.n_blocks
            take = lambda t: torch.cat([t[:, :, b * rows:(b + 1) * rows] for b in sched.my_blocks], dim=2).contiguous()
            out = ring_attention(take(q), take(k), take(v), causal=True, layout=layout, out_dtype=torch.float32, exchange=exchange)
            mpsa.check_status()
            ref = take(full)
            worst = max(worst, float((out - ref).norm() / ref.norm()))
        ret[rank] = worst
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["ring", "gather"])
@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
def test_ring_equals_single_gpu(layout, exchange):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    ret = mp.get_context("spawn").Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), layout, exchange, (2048, 1024), ret), nprocs=world, join=True)
    assert len(ret) == world and max(ret.values()) < 1e-4, dict(ret)


def test_one_process_drives_two_devices():
    """The kernels' per-device attributes (more than 48 KB of dynamic shared memory) are set on whatever device a call
    runs on: forward, router statistic and GEMM on cuda:0 and then on cuda:1 from the same process."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import mpsa
    from oracle import mx_oracle as O
    q, k, v = O.make_qkv(3, 1, 4, 2, 512, 128, outliers=3)
    ref = O.attention_mxfp(q, k, v, causal=True, pv_mode="requant")
    outs = []
    for d in (0, 1):
        dev = torch.device("cuda", d)
        with torch.cuda.device(dev):
            o = mpsa.attention_forward(q.to(dev), k.to(dev), v.to(dev), causal=True, pv_mode="requant", router="online", tau=1e9,
                                       out_dtype=torch.float32, check=True)
            qa = mpsa.quantize_mx(q.to(dev).reshape(1, 1, -1, 128), 1.0, want_fp4=False)
            c = mpsa.gemm_block_scaled(qa.fp8.view(-1, 128), qa.fp8_sf, qa.fp8.view(-1, 128), qa.fp8_sf, torch.float32,
                                       qa.fp8.shape[2], qa.fp8.shape[2], 128, "mxfp8", check=True)
        m = O.parity_metrics(o.cpu(), ref)
        assert m["cos"] >= 0.9999 and m["rel_l2"] <= 1e-2, (d, m)
        outs.append((o.cpu(), c.cpu()))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
