"""Peer-memory exchange between the ranks of one node (one process per GPU).

Every rank owns an inbox and a flag array allocated through the C ABI, exports them as CUDA IPC
handles, and maps the other ranks' ones; the combine kernels of the library then push a rank's piece
straight into every peer's inbox over NVLink (see include/qwen36_fp4_b200.h, "Multi-GPU combine").
torch.distributed is used once, at construction, to pass the 64-byte handles around; the data path
after that has no collective.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import abi
from .backend import KernelError, _check, _dp


class PeerExchange:
    """Inbox + flags of this rank, the peers' mappings, and the device pointer tables."""

    def __init__(self, backend, inbox_bytes: int, flags_per_rank: int, device, group=None):
        self.lib = backend.lib
        self._dist = dist.is_available() and dist.is_initialized()      # a lone process is a world of one
        self.world = dist.get_world_size(group) if self._dist else 1
        self.rank = dist.get_rank(group) if self._dist else 0
        self.device = torch.device(device)
        self._opened, self._owned = [], []
        flag_bytes = 4 * self.world * flags_per_rank
        with torch.cuda.device(self.device):
            inbox = self._malloc(inbox_bytes)
            flags = self._malloc(flag_bytes)
            torch.cuda.synchronize()
            try:
                mine = (self._export(inbox), self._export(flags))
            except KernelError:
                mine = None
            everyone = [mine]
            if self._dist:
                everyone = [None] * self.world
                dist.all_gather_object(everyone, mine, group=group)
            inbox_ptrs, flag_ptrs, mapped = [], [], all(h is not None for h in everyone)
            try:
                for r, handles in enumerate(everyone if mapped else []):
                    if r == self.rank:
                        inbox_ptrs.append(inbox)
                        flag_ptrs.append(flags)
                    else:
                        inbox_ptrs.append(self._open(handles[0]))
                        flag_ptrs.append(self._open(handles[1]))
            except KernelError:
                mapped = False
            if self._dist:                  # all ranks take the same way out
                verdicts = [None] * self.world
                dist.all_gather_object(verdicts, mapped, group=group)
                mapped = all(verdicts)
            if not mapped:
                self._release()
                raise KernelError("peer_exchange (CUDA IPC mapping of a peer's buffers)", abi.CUDA_ERROR)
        self.inbox_table = torch.tensor(inbox_ptrs, dtype=torch.int64, device=self.device)
        self.flag_table = torch.tensor(flag_ptrs, dtype=torch.int64, device=self.device)
        self.state = torch.zeros(4, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        if self._dist:
            dist.barrier(group=group)       # every inbox is mapped and zeroed before anybody pushes

    def _malloc(self, nbytes: int) -> int:
        alloc = abi.DeviceAllocation()
        _check("cuda_malloc", self.lib.qwen36_cuda_malloc(C.byref(alloc), max(256, nbytes)))
        _check("cuda_memset", self.lib.qwen36_cuda_memset(alloc.ptr, 0, max(256, nbytes)))
        self._owned.append(alloc.ptr.ptr)
        return alloc.ptr.ptr

    def _export(self, ptr: int) -> bytes:
        buf = C.create_string_buffer(64)
        _check("ipc_get_handle", self.lib.qwen36_ipc_get_handle(abi.DevicePtr(ptr), buf))
        return buf.raw

    def _open(self, handle: bytes) -> int:
        out = abi.DevicePtr()
        _check("ipc_open_handle", self.lib.qwen36_ipc_open_handle(C.create_string_buffer(handle, 64), C.byref(out)))
        self._opened.append(out.ptr)
        return out.ptr

    def failed(self) -> bool:
        """True once a combine kernel of this process gave up waiting for a peer."""
        return int(self.lib.qwen36_peer_last_error()) != 0

    def failed_call(self) -> int:
        """Number of the first call on THIS exchange whose wait ran out (0 = none): state[2], which the
        kernel writes beside the poisoned output.  After a failure the exchange must be rebuilt on
        every rank (re-zeroed state, flags and inbox under a barrier) before it is used again."""
        return int(self.state[2].item())

    def close(self, group=None) -> None:
        torch.cuda.synchronize(self.device)
        if self._dist:
            dist.barrier(group=group)       # nobody still pushes into a buffer that is about to go
        self._release()

    def _release(self) -> None:
        with torch.cuda.device(self.device):
            for p in self._opened:
                self.lib.qwen36_ipc_close_handle(abi.DevicePtr(p))
            for p in self._owned:
                self.lib.qwen36_cuda_free(abi.DevicePtr(p))
        self._opened, self._owned = [], []


class AttentionPeerMerge:
    """Cross-rank merge of (m, l, o) partials: qwen36_attention_peer_merge."""

    def __init__(self, backend, q_heads: int, head_dim: int, device, group=None):
        self.lib, self.q_heads, self.head_dim = backend.lib, q_heads, head_dim
        world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        nbytes = int(self.lib.qwen36_attention_peer_inbox_bytes(world, q_heads, head_dim))
        self.ex = PeerExchange(backend, nbytes, q_heads, device, group)

    def __call__(self, part_m, part_l, part_o, out=None) -> torch.Tensor:
        if out is None:
            out = torch.empty((self.q_heads, self.head_dim), dtype=torch.bfloat16, device=part_o.device)
        spec = abi.AttentionPeerMergeSpec(self.ex.world, self.ex.rank, self.q_heads, self.head_dim,
                                          _dp(part_o), _dp(part_m), _dp(part_l), _dp(self.ex.inbox_table),
                                          _dp(self.ex.flag_table), _dp(self.ex.state), _dp(out))
        _check("attention_peer_merge", self.lib.qwen36_attention_peer_merge(C.byref(spec)))
        return out


    def attend(self, q_bf16, kq, vq, meta, t_begin: int, t_end: int, workspace, out=None) -> torch.Tensor:
        """Attention over rows [t_begin, t_end) of this rank's cache and the cross-rank merge, two
        launches: qwen36_turboquant_attention_peer."""
        if out is None:
            out = torch.empty((self.q_heads, self.head_dim), dtype=torch.bfloat16, device=q_bf16.device)
        shape = abi.AttentionShape(self.q_heads, kq.shape[1], self.head_dim, 0)
        spec = abi.TurboquantAttentionPeerSpec(t_begin, t_end, _dp(q_bf16), _dp(kq), _dp(vq), _dp(meta),
                                               _dp(workspace), workspace.numel(), shape, self.ex.world,
                                               self.ex.rank, _dp(self.ex.inbox_table), _dp(self.ex.flag_table),
                                               _dp(self.ex.state), _dp(out))
        _check("turboquant_attention_peer", self.lib.qwen36_turboquant_attention_peer(C.byref(spec)))
        return out


class ArgmaxPeerCombine:
    """Cross-rank greedy argmax of per-rank (value, index) winners: qwen36_argmax_peer_combine.
    Every rank must pass the same number of tokens in a given call."""

    def __init__(self, backend, max_tokens: int, device, group=None):
        self.lib, self.max_tokens = backend.lib, max_tokens
        world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        nbytes = int(self.lib.qwen36_argmax_peer_inbox_bytes(world, max_tokens))
        self.ex = PeerExchange(backend, nbytes, 1, device, group)

    def __call__(self, best_value_f32, best_index_i32, out=None) -> torch.Tensor:
        n = best_value_f32.numel()
        if n > self.max_tokens:
            raise KernelError("argmax_peer_combine", abi.INVALID_ARGUMENT)
        if out is None:
            out = torch.empty(n, dtype=torch.int32, device=best_value_f32.device)
        spec = abi.ArgmaxPeerCombineSpec(self.ex.world, self.ex.rank, n, _dp(best_value_f32), _dp(best_index_i32),
                                         _dp(self.ex.inbox_table), _dp(self.ex.flag_table), _dp(self.ex.state),
                                         _dp(out))
        _check("argmax_peer_combine", self.lib.qwen36_argmax_peer_combine(C.byref(spec)))
        return out


class TensorParallelGemv:
    """Chain of row-split W4A16 GEMVs whose outputs meet in every rank's arena over NVLink:
    qwen36_nvfp4_matvec_peer.  `vectors` = {name: length}: the activation vectors of the chain; each
    rank keeps one full copy of every one of them in its arena, as flagged cells (8 bytes per two
    values: bf16 pair + number of the call that wrote them).  A call names the slot (call counter)
    its output travels under; the call that consumes the output names the same slot as its input
    slot.  Every rank must make the same sequence of calls."""

    def __init__(self, backend, vectors: dict, slots: int, device, group=None):
        self.lib = backend.lib
        from .shard import arena_layout
        self.offsets, at = arena_layout(vectors)
        self.slots = slots
        self.ex = PeerExchange(backend, at, 1, device, group)
        self.state = torch.zeros(4 * slots, dtype=torch.int32, device=self.ex.device)
        self._arena = int(self.ex.inbox_table[self.ex.rank].item())

    def _spec(self, out_names, row_offsets, out_slot: int, in_slot):
        offs = (abi.size_t * 4)(*([self.offsets[n][0] for n in out_names] + [0] * (4 - len(out_names))))
        rows = (abi.size_t * 4)(*(list(row_offsets) + [0] * (4 - len(row_offsets))))
        return abi.Nvfp4MatvecPeerSpec(self.ex.world, self.ex.rank, _dp(self.ex.inbox_table), _dp(self.state),
                                       self.slots, out_slot, abi.PEER_INPUT_LOCAL if in_slot is None else in_slot,
                                       offs, rows)

    def gemv(self, x, mats, out_slot: int, in_slot=None) -> None:
        """`x`: a local bf16 tensor (in_slot None), or (vector name, length) for the first `length`
        values of a vector of the arena that the call of slot `in_slot` produced.  `mats`: up to four
        (weight_u8 [local rows, K/2], sf_tiled, tensor_scale, output vector name, first row of the
        slice) that share `x`."""
        if isinstance(x, tuple):
            x_ptr, k = abi.DevicePtr(self._arena + self.offsets[x[0]][0]), x[1]
        else:
            x_ptr, k = _dp(x), x.numel()
        specs = (abi.Nvfp4MatvecSpec * len(mats))()
        for i, (weight_u8, sf_tiled, tensor_scale, _, _) in enumerate(mats):
            specs[i] = abi.Nvfp4MatvecSpec(weight_u8.shape[0], k, x_ptr, _dp(weight_u8), _dp(sf_tiled),
                                           _dp(tensor_scale), abi.DevicePtr(0))
        peer = self._spec([m[3] for m in mats], [m[4] for m in mats], out_slot, in_slot)
        _check("nvfp4_matvec_peer", self.lib.qwen36_nvfp4_matvec_peer(specs, len(mats), C.byref(peer)))

    def collect(self, name: str, slot: int, out=None, n=None) -> torch.Tensor:
        """The vector `name`, produced by the call of `slot`, as a plain bf16 tensor (waits, bounded,
        for every rank's part)."""
        off, full = self.offsets[name]
        n = full if n is None else n
        if out is None:
            out = torch.empty(n, dtype=torch.bfloat16, device=self.ex.device)
        peer = self._spec([], [], 0, None)
        _check("nvfp4_matvec_peer_collect",
               self.lib.qwen36_nvfp4_matvec_peer_collect(C.byref(peer), slot, abi.DevicePtr(self._arena + off), n, _dp(out)))
        return out

    def failed_call(self) -> int:
        """Number of the first call, on any slot, that went out poisoned or whose wait ran out (0 = none)."""
        bad = self.state.view(-1, 4)[:, 2]
        bad = bad[bad != 0]
        return int(bad.min().item()) if bad.numel() else 0

    def close(self, group=None) -> None:
        self.ex.close(group)
