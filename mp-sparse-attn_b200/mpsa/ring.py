"""Sequence-parallel attention over a ring of GPUs (one process per GPU, torch.distributed).

Every rank owns a slice of the sequence: its query rows, and the matching keys / values, which it
quantises ONCE.  The diagonal (MXFP8 band) tiles only ever involve a rank's own keys, so what travels
round the ring is the MXFP4 form of K and V (codes + E8M0 scale tiles, about 0.53 byte per element):
at step s a rank computes the partial attention of its queries against the block that started s hops
upstream while the next block is already in flight (NCCL send/recv on NVLink), and merges the partial
result into its accumulator with the log-sum-exp weights the forward kernel reports.

The reference has no multi-GPU path (its kernel sees all keys in one launch,
ours/mxfp_attn_kernel.py:245); this module is new functionality on top of the same kernels.

Ownership layouts
  "contiguous"  rank r owns sequence block r of n.  Causal work is unbalanced (rank r has r+1 blocks
                of keys to visit), which caps the efficiency at (n+1)/(2n).
  "zigzag"      the sequence is cut into 2n blocks and rank r owns blocks r and 2n-1-r: every rank then
                visits 2n+1 (query block, key block) pairs, so causal work is balanced.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch

FULL, DIAG, SKIP = "full", "diag", "skip"


# --------------------------------------------------------------------------------------------------
# schedule (pure host logic)
# --------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class RingSchedule:
    world: int
    rank: int
    layout: str = "contiguous"
    causal: bool = True

    def __post_init__(self):
        if self.layout not in ("contiguous", "zigzag"):
            raise ValueError(f"unknown layout {self.layout!r}")
        if not (0 <= self.rank < self.world):
            raise ValueError("rank out of range")

    @property
    def n_blocks(self) -> int:
        return self.world if self.layout == "contiguous" else 2 * self.world

    def blocks_of(self, rank: int) -> Tuple[int, ...]:
        """Global sequence blocks a rank owns, in the order its local tensors hold them."""
        if self.layout == "contiguous":
            return (rank,)
        return (rank, 2 * self.world - 1 - rank)

    @property
    def my_blocks(self) -> Tuple[int, ...]:
        return self.blocks_of(self.rank)

    @property
    def send_to(self) -> int:
        return (self.rank + 1) % self.world

    @property
    def recv_from(self) -> int:
        return (self.rank - 1) % self.world

    def source_at(self, step: int) -> int:
        """Rank whose K/V this rank holds at ring step `step` (step 0 = its own)."""
        return (self.rank - step) % self.world

    def pair_kind(self, q_block: int, k_block: int) -> str:
        if not self.causal:
            return FULL
        if k_block == q_block:
            return DIAG
        return FULL if k_block < q_block else SKIP

    def pairs_at(self, step: int) -> List[Tuple[int, int, str]]:
        """(local query block index, local key block index of the source rank, kind) to compute at `step`."""
        src = self.source_at(step)
        out = []
        for qi, qb in enumerate(self.my_blocks):
            for ki, kb in enumerate(self.blocks_of(src)):
                kind = self.pair_kind(qb, kb)
                if kind != SKIP:
                    out.append((qi, ki, kind))
        return out

    def work_units(self) -> float:
        """Visited pairs (a diagonal pair counts one half): the load-balance figure of a layout."""
        return sum(0.5 if kind == DIAG else 1.0 for s in range(self.world) for _, _, kind in self.pairs_at(s))


# --------------------------------------------------------------------------------------------------
# backends
# --------------------------------------------------------------------------------------------------
class CudaRingBackend:
    """Quantisation, partial attention and merging with the sm_100a kernels (quantised P.V)."""

    def __init__(self, B, Hq, Hkv, D, block_rows, device, sm_scale=None, fp8_elem="e5m2", out_dtype=torch.bfloat16):
        from . import ops
        self.ops = ops
        self.B, self.Hq, self.Hkv, self.D, self.rows = B, Hq, Hkv, D, block_rows
        self.device, self.fp8_elem, self.out_dtype = device, fp8_elem, out_dtype
        self.sq = ops.q_side_scale(D, sm_scale)
        nt = -(-block_rows // 128)
        self.pad = nt * 128
        # byte sizes of the four pieces of one key/value block in MXFP4 form
        self.sizes = (B * Hkv * block_rows * 64, B * Hkv * nt * 512, B * Hkv * D * self.pad // 2, B * Hkv * nt * 512)
        self.payload_bytes = sum(self.sizes)
        self._zeros = {}

    def prepare_q(self, q_block):
        return self.ops.quantize_mx(self.ops._pad_depth_128(q_block), self.sq, fp8_elem=self.fp8_elem)

    def prepare_kv(self, k_block, v_block):
        """-> (local operands in both formats for the diagonal pair, MXFP4 payload to send)."""
        kq = self.ops.quantize_mx(self.ops._pad_depth_128(k_block), 1.0, fp8_elem=self.fp8_elem)
        vq = self.ops.quantize_v_seq(v_block, self.fp8_elem)
        payload = torch.empty(self.payload_bytes, dtype=torch.uint8, device=self.device)
        o = 0
        for t, n in zip((kq.fp4, kq.fp4_sf, vq.vt4, vq.v4_sf), self.sizes):
            payload[o:o + n].copy_(t.reshape(-1))
            o += n
        return (kq, vq), payload

    def _zero(self, shape):
        if shape not in self._zeros:
            self._zeros[shape] = torch.zeros(shape, dtype=torch.uint8, device=self.device)
        return self._zeros[shape]

    def _unpack(self, payload):
        B, Hkv, D, rows, pad = self.B, self.Hkv, self.D, self.rows, self.pad
        views, o = [], 0
        for n in self.sizes:
            views.append(payload[o:o + n])
            o += n
        k4 = views[0].view(B, Hkv, rows, 64)
        k4s = views[1].view(B, Hkv, pad // 128, 1, 512)
        kq = self.ops.QuantizedOperand(fp4=k4, fp4_sf=k4s, fp8_elem=self.fp8_elem)
        vq = self.ops.QuantizedV(self._zero((B, Hkv, D, pad)), self._zero((B, Hkv, pad // 128, 512)),
                                 views[2].view(B, Hkv, D, pad // 2), views[3].view(B, Hkv, pad // 128, 512), self.fp8_elem)
        return kq, vq

    def partial(self, qq, local_kv, payload, kind, merge_with=None):
        """Attention of one query block against one key block -> (normalised output, log2 denominator); with
        merge_with = (acc, lse) the result is already merged with that earlier partial result."""
        rows = self.rows
        if kind == DIAG:
            kq, vq = local_kv
            return self.ops.attention_forward_quantized(qq, kq, vq, self.B, self.Hq, self.Hkv, rows, rows, self.D,
                                                        causal=True, out_dtype=torch.float32, return_lse=True,
                                                        merge_with=merge_with)
        kq, vq = self._unpack(payload)
        return self.ops.attention_forward_quantized(qq, kq, vq, self.B, self.Hq, self.Hkv, rows, rows, self.D,
                                                    causal=False, uniform="fp4", out_dtype=torch.float32,
                                                    return_lse=True, merge_with=merge_with)

    fused_merge = True                             # partial() can merge in its epilogue

    def new_accumulator(self):
        acc = torch.zeros((self.B, self.Hq, self.rows, self.D), dtype=torch.float32, device=self.device)
        lse = torch.full((self.B, self.Hq, self.rows), float("-inf"), dtype=torch.float32, device=self.device)
        return acc, lse

    def merge(self, acc, lse_acc, o, lse):
        self.ops.attention_merge(acc, lse_acc, o, lse)

    def split_payload(self, payload, n_blocks):
        return [payload[i * self.payload_bytes:(i + 1) * self.payload_bytes] for i in range(n_blocks)]


# --------------------------------------------------------------------------------------------------
# the ring
# --------------------------------------------------------------------------------------------------
def _exchange(dist, group, send_buf, recv_buf, send_to, recv_from):
    ops = [dist.P2POp(dist.isend, send_buf, send_to, group), dist.P2POp(dist.irecv, recv_buf, recv_from, group)]
    return dist.batch_isend_irecv(ops)


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = True, group=None,
                   layout: str = "contiguous", backend=None, sm_scale: Optional[float] = None,
                   out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """q [B,Hq,S_local,D], k/v [B,Hkv,S_local,D]: this rank's slice (its blocks concatenated in the order
    of RingSchedule.blocks_of).  Returns this rank's slice of the output, [B,Hq,S_local,D]."""
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    sched = RingSchedule(world, rank, layout, causal)
    nb = len(sched.my_blocks)
    B, Hq, S_local, D = q.shape
    Hkv = k.shape[1]
    if S_local % nb:
        raise ValueError("local sequence length must divide into the rank's blocks")
    rows = S_local // nb
    if backend is None:
        backend = CudaRingBackend(B, Hq, Hkv, D, rows, q.device, sm_scale, out_dtype=out_dtype)

    qqs = [backend.prepare_q(q[:, :, i * rows:(i + 1) * rows]) for i in range(nb)]
    local, payloads = [], []
    for i in range(nb):
        kv, pay = backend.prepare_kv(k[:, :, i * rows:(i + 1) * rows], v[:, :, i * rows:(i + 1) * rows])
        local.append(kv)
        payloads.append(pay)
    cur = torch.cat(payloads) if nb > 1 else payloads[0]
    nxt = torch.empty_like(cur)
    accs = [backend.new_accumulator() for _ in range(nb)]

    for step in range(world):
        works = None
        if step + 1 < world:
            # the block received at this step is forwarded while it is being consumed
            works = _exchange(dist, group, cur, nxt, sched.send_to, sched.recv_from)
        blocks = backend.split_payload(cur, nb)
        for qi, ki, kind in sched.pairs_at(step):
            if getattr(backend, "fused_merge", False):
                # the forward's epilogue merges with what has been accumulated so far (fresh output buffers each time)
                accs[qi] = backend.partial(qqs[qi], local[ki] if step == 0 else None, blocks[ki], kind, merge_with=accs[qi])
            else:
                o, lse = backend.partial(qqs[qi], local[ki] if step == 0 else None, blocks[ki], kind)
                backend.merge(accs[qi][0], accs[qi][1], o, lse)
        if works is not None:
            for w in works:
                w.wait()
            cur, nxt = nxt, cur
    out = torch.cat([a for a, _ in accs], dim=2) if nb > 1 else accs[0][0]
    return out.to(out_dtype)
