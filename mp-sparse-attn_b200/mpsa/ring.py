"""Sequence-parallel attention over a ring of GPUs (one process per GPU, torch.distributed).

Every rank owns a slice of the sequence: its query rows, and the matching keys / values, which it
quantises ONCE.  The diagonal (MXFP8 band) tiles only ever involve a rank's own keys, so what travels
round the ring is the MXFP4 form of K and V (codes + E8M0 scale tiles, about 0.53 byte per element):
at step s a rank computes the partial attention of its queries against the block that started s hops
upstream while the next block is already in flight (NCCL send/recv on NVLink), and merges the partial
result into its accumulator with the log-sum-exp weights the forward kernel reports.

exchange="gather" is the alternative for sequences whose MXFP4 K/V fit every GPU (0.53 byte per element:
128K tokens of 8 KV heads x 128 are 140 MB): the payloads are all-gathered once, behind the diagonal pairs,
which need local data only, and each query block then visits ALL its earlier keys in one launch that merges with
the diagonal result in its epilogue.  A launch costs every CTA a fixed prologue and epilogue, so one long
launch per query block instead of one per ring step is what keeps short per-rank blocks efficient.

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
_ZERO_CACHE = {}


class CudaRingBackend:
    """Quantisation, partial attention and merging with the sm_100a kernels (quantised P.V)."""

    def __init__(self, B, Hq, Hkv, D, block_rows, device, sm_scale=None, fp8_elem="e5m2", out_dtype=torch.bfloat16):
        from . import ops
        self.ops = ops
        self.B, self.Hq, self.Hkv, self.D, self.rows = B, Hq, Hkv, D, block_rows
        self.device, self.fp8_elem, self.out_dtype = device, fp8_elem, out_dtype
        self.sq = ops.q_side_scale(D, sm_scale)
        self.nt = nt = -(-block_rows // 128)          # 128-key tiles of a block
        self.pad = ops.v_pitch(block_rows)              # keys per V^T row of a block (a multiple of 128, >= the rows)
        # byte sizes of the four pieces of one key/value block in MXFP4 form
        self.sizes = (B * Hkv * block_rows * 64, B * Hkv * nt * 512, B * Hkv * D * self.pad // 2,
                      B * Hkv * (self.pad // 128) * 512)
        self.payload_bytes = sum(self.sizes)
        self._zeros = _ZERO_CACHE.setdefault(str(device), {})       # placeholders and maps, kept across calls

    def prepare_q(self, q_block):
        return self.ops.quantize_mx(self.ops._pad_depth_128(q_block), self.sq, fp8_elem=self.fp8_elem)

    def prepare_kv(self, k_block, v_block):
        """-> (local operands in both formats for the diagonal pair, MXFP4 payload to send)."""
        kq = self.ops.quantize_mx(self.ops._pad_depth_128(k_block), 1.0, fp8_elem=self.fp8_elem)
        vq = self.ops.quantize_v_seq(v_block, self.fp8_elem, pad=self.pad)
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
        k4s = views[1].view(B, Hkv, self.nt, 1, 512)
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

    # ---- exchange="gather": all blocks of the sequence side by side ----
    def assemble(self, gathered, order):
        """gathered: uint8 [n_blocks, payload_bytes] in arrival order; order[g] = row of global block g.
        -> the MXFP4 K and V of the whole sequence laid out as one operand (blocks in sequence order)."""
        B, Hkv, D, rows, pad = self.B, self.Hkv, self.D, self.rows, self.pad
        if rows % 128:
            raise ValueError("exchange='gather' needs block lengths that are multiples of 128")
        G, nt = gathered.shape[0], self.nt
        gp = self.ops.v_pitch(G * rows)                 # keys per row of the assembled V^T
        # copies go through 8-byte words (every piece is a multiple of 512 bytes): byte-wise strided copies are slow
        W = torch.int64
        k4 = torch.empty((B, Hkv, G, rows, 64), dtype=torch.uint8, device=self.device)
        k4s = torch.empty((B, Hkv, G, nt, 512), dtype=torch.uint8, device=self.device)
        v4 = torch.empty((B, Hkv, D, gp // 2), dtype=torch.uint8, device=self.device)
        v4s = torch.empty((B, Hkv, gp // 128, 512), dtype=torch.uint8, device=self.device)
        k4w, k4sw, v4w, v4sw = k4.view(W), k4s.view(W), v4.view(W), v4s.view(W)
        for g in range(G):
            row, o, parts = gathered[order[g]], 0, []
            for n in self.sizes:
                parts.append(row[o:o + n].view(W))
                o += n
            k4w[:, :, g].copy_(parts[0].view(B, Hkv, rows, 8))
            k4sw[:, :, g].copy_(parts[1].view(B, Hkv, nt, 64))
            v4w[:, :, :, g * rows // 16:(g + 1) * rows // 16].copy_(parts[2].view(B, Hkv, D, pad // 16)[..., :rows // 16])
            v4sw[:, :, g * nt:(g + 1) * nt].copy_(parts[3].view(B, Hkv, pad // 128, 64)[:, :, :nt])
        # the MXFP8 forms are never selected by the maps below; the kernel's tensor maps still need buffers that size
        kq = self.ops.QuantizedOperand(fp8=self._zero((B * Hkv * G * rows, 128)), fp4=k4.view(B, Hkv, G * rows, 64),
                                       fp4_sf=k4s.view(B, Hkv, G * nt, 1, 512), fp8_elem=self.fp8_elem)
        vq = self.ops.QuantizedV(self._zero((B, Hkv, D, gp)), self._zero((B, Hkv, gp // 128, 512)), v4, v4s, self.fp8_elem)
        return kq, vq, G

    def partial_prefix(self, qq, gkv, n_key_blocks, merge_with=None):
        """Attention of one query block against sequence blocks [0, n_key_blocks), all tiles MXFP4, no mask."""
        kq, vq, G = gkv
        nt = self.nt
        key = ("map", nt, G, n_key_blocks)       # the map is [nt, G * nt]: every length gets its own
        if key not in self._zeros:
            m = torch.zeros((nt, G * nt), dtype=torch.uint8, device=self.device)      # 0 = skip
            m[:, :n_key_blocks * nt] = self.ops.TILE_FP4
            self._zeros[key] = m
        return self.ops.attention_forward_quantized(qq, kq, vq, self.B, self.Hq, self.Hkv, self.rows, G * self.rows,
                                                    self.D, causal=False, prec_map=self._zeros[key], uniform="fp4",
                                                    out_dtype=torch.float32, return_lse=True, merge_with=merge_with)


# --------------------------------------------------------------------------------------------------
# the ring
# --------------------------------------------------------------------------------------------------
def _exchange(dist, group, send_buf, recv_buf, send_to, recv_from):
    ops = [dist.P2POp(dist.isend, send_buf, send_to, group), dist.P2POp(dist.irecv, recv_buf, recv_from, group)]
    return dist.batch_isend_irecv(ops)


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = True, group=None,
                   layout: str = "contiguous", backend=None, sm_scale: Optional[float] = None,
                   out_dtype: torch.dtype = torch.bfloat16, exchange: str = "ring") -> torch.Tensor:
    """q [B,Hq,S_local,D], k/v [B,Hkv,S_local,D]: this rank's slice (its blocks concatenated in the order
    of RingSchedule.blocks_of).  Returns this rank's slice of the output, [B,Hq,S_local,D].
    exchange: "ring" (send/recv, one block pair per launch) or "gather" (one all-gather, one launch per query block)."""
    if exchange not in ("ring", "gather"):
        raise ValueError(f"unknown exchange {exchange!r}")
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
    fused = getattr(backend, "fused_merge", False)

    if exchange == "gather" and world > 1:
        gathered = torch.empty((world,) + tuple(cur.shape), dtype=cur.dtype, device=cur.device)
        work = dist.all_gather_into_tensor(gathered.view(-1), cur.reshape(-1), group=group, async_op=True)
        accs = [None] * nb
        if causal:                                   # the diagonal pairs need local data only: they cover the gather
            blocks = backend.split_payload(cur, nb)
            for qi in range(nb):
                accs[qi] = backend.partial(qqs[qi], local[qi], blocks[qi], DIAG)
        work.wait()
        arrival = [b for r in range(world) for b in sched.blocks_of(r)]
        order = [arrival.index(g) for g in range(sched.n_blocks)]
        gkv = backend.assemble(gathered.view(world * nb, -1), order)
        # longest first: the short launch then fills the tail of the long one
        for qi in sorted(range(nb), key=lambda i: -sched.my_blocks[i]):
            n_keys = sched.my_blocks[qi] if causal else sched.n_blocks
            if n_keys == 0:
                continue
            if accs[qi] is None:
                accs[qi] = backend.partial_prefix(qqs[qi], gkv, n_keys)
            elif fused:
                accs[qi] = backend.partial_prefix(qqs[qi], gkv, n_keys, merge_with=accs[qi])
            else:
                o, lse = backend.partial_prefix(qqs[qi], gkv, n_keys)
                acc = tuple(t.clone() for t in accs[qi])
                backend.merge(acc[0], acc[1], o, lse)
                accs[qi] = acc
        out = torch.cat([a for a, _ in accs], dim=2) if nb > 1 else accs[0][0]
        return out.to(out_dtype)

    nxt = torch.empty_like(cur)
    accs = [backend.new_accumulator() for _ in range(nb)]

    for step in range(world):
        works = None
        if step + 1 < world:
            # the block received at this step is forwarded while it is being consumed
            works = _exchange(dist, group, cur, nxt, sched.send_to, sched.recv_from)
        blocks = backend.split_payload(cur, nb)
        for qi, ki, kind in sched.pairs_at(step):
            if fused:
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
