"""Host-side logic of the sequence-parallel ring on CPU: the schedule, and the ring loop itself run as
gloo ranks with a reference backend (plain fp32 attention per block pair) in place of the CUDA kernels."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mpsa.ring import DIAG, FULL, RingSchedule, ring_attention

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_schedule_covers_the_causal_triangle_once(world, layout):
    seen = {}
    units = []
    for r in range(world):
        s = RingSchedule(world, r, layout, True)
        assert s.source_at(0) == r and sorted(s.source_at(i) for i in range(world)) == list(range(world))
        for step in range(world):
            src = s.source_at(step)
            for qi, ki, kind in s.pairs_at(step):
                qb, kb = s.my_blocks[qi], s.blocks_of(src)[ki]
                assert (qb, kb) not in seen
                seen[(qb, kb)] = kind
                assert (kind == DIAG) == (qb == kb) and kb <= qb
        units.append(s.work_units())
    n = RingSchedule(world, 0, layout, True).n_blocks
    assert len(seen) == n * (n + 1) // 2
    if layout == "zigzag":
        assert max(units) == min(units)              # balanced
    else:
        assert units == [r + 0.5 for r in range(world)]
    # non-causal: every pair, all of kind FULL
    s = RingSchedule(world, 0, layout, False)
    assert all(kind == FULL for step in range(world) for _, _, kind in s.pairs_at(step))


class RefBackend:
    """fp32 attention per (query block, key block) with the log2 denominator, and the merge in torch."""

    def __init__(self, rows, D):
        self.rows, self.D = rows, D

    def prepare_q(self, qb):
        return qb.float() * (self.D ** -0.5 * 1.4426950408889634)

    def prepare_kv(self, kb, vb):
        pay = torch.cat([kb.float().reshape(-1), vb.float().reshape(-1)])
        return (kb.float(), vb.float()), pay

    def split_payload(self, payload, n):
        return list(payload.chunk(n))

    def partial(self, qq, local_kv, payload, kind):
        half = payload.numel() // 2
        B, H = qq.shape[:2]
        k = payload[:half].view(B, H, self.rows, self.D)
        v = payload[half:].view(B, H, self.rows, self.D)
        s = qq @ k.transpose(-1, -2)
        if kind == DIAG:
            s = s.masked_fill(torch.triu(torch.ones(self.rows, self.rows, dtype=torch.bool), 1), float("-inf"))
        m = s.amax(-1, keepdim=True)
        p = torch.exp2(s - m)
        l = p.sum(-1, keepdim=True)
        return (p @ v) / l, (m + torch.log2(l)).squeeze(-1)

    def assemble(self, gathered, order):
        return torch.stack([gathered[i] for i in order])

    def partial_prefix(self, qq, gkv, n_key_blocks):
        B, H = qq.shape[:2]
        half = gkv.shape[1] // 2
        k = torch.cat([gkv[g, :half].view(B, H, self.rows, self.D) for g in range(n_key_blocks)], dim=2)
        v = torch.cat([gkv[g, half:].view(B, H, self.rows, self.D) for g in range(n_key_blocks)], dim=2)
        s = qq @ k.transpose(-1, -2)
        m = s.amax(-1, keepdim=True)
        p = torch.exp2(s - m)
        l = p.sum(-1, keepdim=True)
        return (p @ v) / l, (m + torch.log2(l)).squeeze(-1)

    def new_accumulator(self):
        return None, None

    def merge(self, acc, lse_acc, o, lse):
        raise NotImplementedError


class MergingRefBackend(RefBackend):
    def __init__(self, rows, D, B, H):
        super().__init__(rows, D)
        self.B, self.H = B, H

    def new_accumulator(self):
        return (torch.zeros(self.B, self.H, self.rows, self.D), torch.full((self.B, self.H, self.rows), float("-inf")))

    def merge(self, acc, lse_acc, o, lse):
        lm = torch.maximum(lse_acc, lse)
        wa, wb = torch.exp2(lse_acc - lm), torch.exp2(lse - lm)
        wa, wb = torch.nan_to_num(wa), torch.nan_to_num(wb)
        tot = wa + wb
        acc.copy_(acc * (wa / tot).unsqueeze(-1) + o * (wb / tot).unsqueeze(-1))
        lse_acc.copy_(lm + torch.log2(tot))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, layout, causal, exchange, q, k, v, ref, ret):
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "mp-sparse-attn_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sched = RingSchedule(world, rank, layout, causal)
        S = q.shape[2]
        rows = S // sched.n_blocks
        take = lambda t: torch.cat([t[:, :, b * rows:(b + 1) * rows] for b in sched.my_blocks], dim=2)
        out = ring_attention(take(q), take(k), take(v), causal=causal, layout=layout,
                             backend=MergingRefBackend(rows, q.shape[-1], q.shape[0], q.shape[1]), out_dtype=torch.float32,
                             exchange=exchange)
        err = float((out - take(ref)).abs().max())
        ret[rank] = err
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["ring", "gather"])
@pytest.mark.parametrize("world,layout,causal", [(2, "contiguous", True), (2, "zigzag", True), (4, "zigzag", True),
                                                 (3, "contiguous", False)])
def test_ring_matches_single_process_attention(world, layout, causal, exchange):
    g = torch.Generator().manual_seed(3)
    B, H, D = 1, 2, 16
    S = 24 * world
    q, k, v = (torch.randn(B, H, S, D, generator=g) for _ in range(3))
    s = (q @ k.transpose(-1, -2)) * D ** -0.5
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), float("-inf"))
    ref = torch.softmax(s, -1) @ v
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), layout, causal, exchange, q, k, v, ref, ret), nprocs=world, join=True)
    assert len(ret) == world and max(ret.values()) < 1e-5, dict(ret)


def test_assemble_lays_the_gathered_blocks_out_in_sequence_order():
    """exchange="gather": the per-block payloads (arrival order) become one K operand and one V^T operand whose rows
    run over the whole sequence; checked byte for byte on the host with the CUDA backend's own code (it only moves
    bytes; the kernels are not involved)."""
    from mpsa import ops, ring

    class Ops:
        v_pitch = staticmethod(ops.v_pitch)
        TILE_FP4 = ops.TILE_FP4

        class QuantizedOperand:
            def __init__(self, **kw):
                self.__dict__.update(kw)

        class QuantizedV:
            def __init__(self, vt8, v8_sf, vt4, v4_sf, fp8_elem):
                self.vt8, self.v8_sf, self.vt4, self.v4_sf = vt8, v8_sf, vt4, v4_sf

    B, Hkv, D, rows, G = 1, 2, 128, 256, 4
    be = ring.CudaRingBackend.__new__(ring.CudaRingBackend)
    be.ops, be.B, be.Hkv, be.D, be.rows, be.device, be.fp8_elem, be._zeros = Ops, B, Hkv, D, rows, "cpu", "e5m2", {}
    be.nt, be.pad = rows // 128, ops.v_pitch(rows)
    nt, pad = be.nt, be.pad
    be.sizes = (B * Hkv * rows * 64, B * Hkv * nt * 512, B * Hkv * D * pad // 2, B * Hkv * (pad // 128) * 512)
    g = torch.Generator().manual_seed(7)
    gathered = torch.randint(0, 256, (G, sum(be.sizes)), dtype=torch.uint8, generator=g)
    order = [2, 0, 3, 1]                           # order[g] = arrival row of sequence block g
    kq, vq, n = be.assemble(gathered, order)
    assert n == G and kq.fp4.shape == (B, Hkv, G * rows, 64) and vq.vt4.shape[-1] * 2 >= G * rows
    for blk in range(G):
        row, o = gathered[order[blk]], 0
        k4 = row[o:o + be.sizes[0]].view(B, Hkv, rows, 64); o += be.sizes[0]
        k4s = row[o:o + be.sizes[1]].view(B, Hkv, nt, 1, 512); o += be.sizes[1]
        v4 = row[o:o + be.sizes[2]].view(B, Hkv, D, pad // 2); o += be.sizes[2]
        v4s = row[o:o + be.sizes[3]].view(B, Hkv, pad // 128, 512)
        assert torch.equal(kq.fp4[:, :, blk * rows:(blk + 1) * rows], k4)
        assert torch.equal(kq.fp4_sf[:, :, blk * nt:(blk + 1) * nt], k4s)
        assert torch.equal(vq.vt4[..., blk * rows // 2:(blk + 1) * rows // 2], v4[..., :rows // 2])
        assert torch.equal(vq.v4_sf[:, :, blk * nt:(blk + 1) * nt], v4s[:, :, :nt])
    with pytest.raises(ValueError):
        be.rows = 200
        be.assemble(gathered, order)


class _FailingBackend(MergingRefBackend):
    """Raises on the rank `bad` at its first block pair: the exchange of step 0 is posted, that of step 1 never is."""

    def __init__(self, rows, D, B, H, fail):
        super().__init__(rows, D, B, H)
        self.fail, self.calls = fail, 0

    def partial(self, qq, local_kv, payload, kind):
        self.calls += 1
        if self.fail and self.calls == 1:
            raise RuntimeError("injected failure on this rank")
        return super().partial(qq, local_kv, payload, kind)


def _failing_worker(rank, world, port, bad, ret):
    import datetime
    import time
    sys.path.insert(0, os.path.join(os.path.dirname(HERE), "mp-sparse-attn_b200"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=10))
    t0 = time.time()
    g = torch.Generator().manual_seed(rank)
    q, k, v = (torch.randn(1, 2, 24, 16, generator=g) for _ in range(3))
    try:
        ring_attention(q, k, v, causal=True, layout="contiguous", backend=_FailingBackend(24, 16, 1, 2, rank == bad),
                       out_dtype=torch.float32, exchange="ring")
        ret[rank] = ("finished", time.time() - t0)
    except Exception as e:  # noqa: BLE001  (the point of the test: which exception, and how soon)
        ret[rank] = (type(e).__name__ + ": " + str(e)[:80], time.time() - t0)
    # no destroy_process_group: the failed rank leaves as a crashed process would


def test_a_failing_rank_ends_the_ring_with_an_error_not_a_hang():
    """Failure detection on the host: one rank raises during the first ring step and leaves.  The rank downstream of it
    never gets its next block: its receive must end with an exception (peer gone, or the process group's 10 s timeout)
    instead of waiting for ever; the rank upstream either finishes (it needed nothing from the failed rank) or gets an
    error from its send.  No rank may hang.  (CPU ranks over gloo: nothing here touches a GPU.)"""
    world, bad = 3, 1
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, bad, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=90)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.kill()                                    # exactly the processes started above
    assert not hung, "a rank was still waiting after 90 s"
    assert set(ret.keys()) == set(range(world)), dict(ret)
    assert ret[bad][0].startswith("RuntimeError: injected failure")
    what, secs = ret[(bad + 1) % world]
    assert what != "finished" and secs < 60, (what, secs)       # the downstream rank saw the failure
    assert all(v[1] < 60 for v in ret.values()), dict(ret)
