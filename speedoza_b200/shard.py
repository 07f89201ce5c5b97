"""Multi-GPU partitioning of the hot path (one process per GPU, torch.distributed).

The reference is single-GPU; these are the natural shards of its path:
  * NVFP4 linear layers: output rows split in 128-row blocks (block-scale tiles stay whole),
    activations replicated, all-gather of the bf16 output slices;
  * lm_head: vocab rows split, each rank runs the fused GEMV+argmax on its slice with
    ``row_offset`` = first row, all-gather of (value, index) pairs, lowest index wins ties;
  * int8 KV decode attention: contiguous token ranges per rank, each rank produces one (m, l, o)
    partial per q head, all-gather, log-sum-exp merge.
The collectives move a few bytes to a few hundred KB; they are there because the path has a real
exchange step, nothing else is communicated.  Works with any backend of torch.distributed (NCCL on
GPUs; gloo on CPU tensors for the host-side logic tests).
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


def shard_rows(n: int, rank: int, world: int, block: int = 128) -> Tuple[int, int]:
    """Rows [lo, hi) of rank: whole `block`-row blocks, ceil-split, the tail goes to the last rank."""
    blocks = n // block
    per = (blocks + world - 1) // world
    lo = min(blocks, per * rank) * block
    hi = min(blocks, per * (rank + 1)) * block
    if rank == world - 1:
        hi = n
    return lo, hi


def shard_tokens(tokens: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous token range of rank (KV appends stay local to the owner of the tail)."""
    per = (tokens + world - 1) // world
    return min(tokens, per * rank), min(tokens, per * (rank + 1))


def arena_layout(vectors: dict, bytes_per_value: int = 4, align: int = 256):
    """Byte offsets of the activation vectors of a tensor-parallel GEMV chain inside a rank's arena
    ({name: (offset, length)}, total bytes).  Flagged cells take 4 bytes per value (two bf16 values +
    the call number per 8 bytes); every vector starts on an `align`-byte boundary.  The same on every
    rank, since a rank stores into its peers' arenas at the offsets of its own."""
    offsets, at = {}, 0
    for name, n in vectors.items():
        offsets[name] = (at, n)
        at += (bytes_per_value * n + align - 1) // align * align
    return offsets, at


def tp_slices(shapes, rank: int, world: int):
    """Row slice [lo, hi) of every matrix of a tensor-parallel chain for `rank`: whole 128-row blocks,
    so that the scale tiles of a slice stay whole.  shapes = [(name, rows, cols), ...]."""
    return {name: shard_rows(rows, rank, world) for name, rows, _ in shapes}


def all_gather_rows(local: torch.Tensor, n_full: int, world: int, out: torch.Tensor = None) -> torch.Tensor:
    """Gathers 1-D row slices produced by shard_rows() back into the full vector."""
    per = ((n_full // 128 + world - 1) // world) * 128
    if per * world == n_full and local.numel() == per:
        if out is None:
            out = torch.empty(n_full, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local)
        return out
    pad = torch.zeros(per, dtype=local.dtype, device=local.device)
    pad[: local.numel()] = local
    buf = torch.empty(per * world, dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, pad)
    pieces, r = [], 0
    for rank in range(world):
        lo, hi = shard_rows(n_full, rank, world)
        pieces.append(buf[rank * per: rank * per + (hi - lo)])
    full = torch.cat(pieces)
    if out is not None:
        out.copy_(full)
        return out
    return full


def combine_argmax(values: torch.Tensor, indices: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """values/indices [world, tokens]: per-rank winners -> global winner per token.  Greedy rule of
    the reference (kernels-cuda/ops.cu:19-23): strictly greater wins, equal values keep the lower
    index, NaN never wins, the scan starts from (-inf, 0)."""
    world, tokens = values.shape
    best_v = torch.full((tokens,), float("-inf"), dtype=values.dtype, device=values.device)
    best_i = torch.zeros(tokens, dtype=torch.int64, device=values.device)
    for r in range(world):
        v, i = values[r], indices[r].to(torch.int64)
        better = (v > best_v) | ((v == best_v) & (i < best_i))
        best_v = torch.where(better, v, best_v)
        best_i = torch.where(better, i, best_i)
    return best_v, best_i


def gather_argmax(value: torch.Tensor, index: torch.Tensor, world: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """All-gather of this rank's (value [tokens] f32, index [tokens] i32) and the global combine."""
    pair = torch.stack([value.to(torch.float32), index.to(torch.int32).view(torch.float32)])   # [2, tokens]
    buf = torch.empty((world * 2, pair.shape[1]), dtype=torch.float32, device=pair.device)   # concatenated on dim 0
    dist.all_gather_into_tensor(buf, pair)
    buf = buf.view(world, 2, -1)
    return combine_argmax(buf[:, 0].contiguous(), buf[:, 1].contiguous().view(torch.int32))


def gather_partials(part_m: torch.Tensor, part_l: torch.Tensor, part_o: torch.Tensor, world: int):
    """All-gather of one (m [H], l [H], o [H, D]) partial per rank into the [H, world(, D)] layout
    that qwen36_attention_merge_partials consumes."""
    h, d = part_o.shape
    packed = torch.cat([part_o, part_m[:, None], part_l[:, None]], dim=1).contiguous()       # [H, D+2]
    buf = torch.empty((world * h, d + 2), dtype=packed.dtype, device=packed.device)          # concatenated on dim 0
    dist.all_gather_into_tensor(buf, packed)
    buf = buf.view(world, h, d + 2).permute(1, 0, 2).contiguous()                             # [H, world, D+2]
    return buf[:, :, d].contiguous(), buf[:, :, d + 1].contiguous(), buf[:, :, :d].contiguous()


class ShardedLmHead:
    """Vocab-sharded FP8 lm_head with fused greedy argmax.  combine = "peer": the per-rank winners are
    pushed into the peers' memory over NVLink by one kernel (speedoza_b200.peer, ranks of one node);
    "collective": all-gather through torch.distributed plus a combine on every rank."""

    def __init__(self, backend, w_e4m3_full_rows: int, w_local, scales_local, row_lo: int, world: int,
                 max_tokens: int, combine: str = "collective"):
        self.b, self.w, self.s, self.row_lo, self.world = backend, w_local, scales_local, row_lo, world
        self.ws = backend.lm_head_argmax_workspace(w_local.shape[0], max_tokens, w_local.device)
        self.peer = None
        if combine == "peer" and world > 1:
            from .peer import ArgmaxPeerCombine
            self.peer = ArgmaxPeerCombine(backend, max_tokens, w_local.device)
            self.tok = torch.empty(max_tokens, dtype=torch.int32, device=w_local.device)
            self.best = torch.empty(max_tokens, dtype=torch.float32, device=w_local.device)
            self.out = torch.empty(max_tokens, dtype=torch.int32, device=w_local.device)

    def argmax(self, x_bf16):
        if self.peer is not None:
            n = x_bf16.shape[0]
            self.b.lm_head_fp8_gemv_argmax(self.w, self.s, x_bf16, self.ws, row_offset=self.row_lo,
                                           out_tokens=self.tok[:n], out_best=self.best[:n])
            return self.peer(self.best[:n], self.tok[:n], self.out[:n])
        tok, best = self.b.lm_head_fp8_gemv_argmax(self.w, self.s, x_bf16, self.ws, row_offset=self.row_lo)
        if self.world == 1:
            return tok.to(torch.int64)
        return gather_argmax(best, tok, self.world)[1]


class ShardedKvAttention:
    """KV-range-sharded int8 decode attention: this rank holds cache rows [t_lo, t_hi).  combine as in
    ShardedLmHead: "peer" merges the ranks' (m, l, o) partials through NVLink peer memory."""

    def __init__(self, backend, kq_local, vq_local, meta_local, t_lo: int, world: int, q_heads: int, head_dim: int,
                 combine: str = "collective"):
        self.b, self.kq, self.vq, self.meta, self.t_lo, self.world = backend, kq_local, vq_local, meta_local, t_lo, world
        self.ws = backend.attention_workspace(q_heads, head_dim, kq_local.device)
        self.peer = None
        if combine == "peer" and world > 1:
            from .peer import AttentionPeerMerge
            dev = kq_local.device
            self.peer = AttentionPeerMerge(backend, q_heads, head_dim, dev)
            self.out = torch.empty((q_heads, head_dim), dtype=torch.bfloat16, device=dev)

    def attend(self, q_bf16, position: int):
        local_end = max(0, min(self.kq.shape[0], position + 1 - self.t_lo))
        if self.peer is not None:
            return self.peer.attend(q_bf16, self.kq, self.vq, self.meta, 0, local_end, self.ws, self.out)
        m, l, o = self.b.turboquant_attention_partial(q_bf16, self.kq, self.vq, self.meta, 0, local_end, self.ws)
        if self.world == 1:
            return self.b.attention_merge_partials(m[:, None].contiguous(), l[:, None].contiguous(),
                                                   o[:, None, :].contiguous())
        pm, pl, po = gather_partials(m, l, o, self.world)
        return self.b.attention_merge_partials(pm, pl, po)
