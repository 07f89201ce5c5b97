"""Tensor-parallel W4A16 GEMV (qwen36_nvfp4_matvec_peer) on one GPU: a world of one (the rank stores
into its own arena), and rank 0 of a world of two whose peer is played by the host (the peer's cells
are written before the launch, so no kernel waits for another kernel).  Results must equal the
bytes of the single-GPU entry on the same matrices."""
import ctypes as C

import pytest
import torch

from speedoza_b200 import abi, synth
from speedoza_b200.peer import TensorParallelGemv

pytestmark = pytest.mark.gpu


def weights(backend, gen, n, k):
    packed, sf_rm = synth.nvfp4_weight_device(gen, n, k, "cuda")
    ts = torch.tensor([synth.WEIGHT_GLOBAL_SCALE * 2688.0 / (14.0 * k ** 0.5)], device="cuda")
    return packed, backend.nvfp4_retile_scales(sf_rm), ts


def test_world_of_one_chain_matches_single_gpu_entry(backend):
    gen = torch.Generator(device="cuda").manual_seed(91)
    k0, n1, n2a, n2b = 1024, 2048, 512, 256
    w1 = weights(backend, gen, n1, k0)
    w2a, w2b = weights(backend, gen, n2a, n1), weights(backend, gen, n2b, n1)
    x = torch.randn(k0, generator=gen, device="cuda").to(torch.bfloat16)
    tp = TensorParallelGemv(backend, {"h": n1, "a": n2a, "b": n2b}, 2, "cuda")
    try:
        for _ in range(3):                       # call numbers advance, vectors are overwritten
            tp.gemv(x, [(w1[0], w1[1], w1[2], "h", 0)], out_slot=0)
            tp.gemv(("h", n1), [(w2a[0], w2a[1], w2a[2], "a", 0), (w2b[0], w2b[1], w2b[2], "b", 0)], out_slot=1,
                    in_slot=0)
        got_h, got_a, got_b = tp.collect("h", 0), tp.collect("a", 1), tp.collect("b", 1)
        torch.cuda.synchronize()
        h = backend.nvfp4_matvec(x, *w1)
        assert torch.equal(got_h.view(torch.int16), h.view(torch.int16))
        assert torch.equal(got_a.view(torch.int16), backend.nvfp4_matvec(h, *w2a).view(torch.int16))
        assert torch.equal(got_b.view(torch.int16), backend.nvfp4_matvec(h, *w2b).view(torch.int16))
        assert tp.failed_call() == 0 and backend.lib.qwen36_nvfp4_gemv_mma_last_error() == 0
        assert tp.state.view(-1, 4)[:, :3].tolist() == [[3, 0, 0], [3, 0, 0]]
    finally:
        tp.close()


def cells_of(values_bf16, call):
    """Flagged cells of a bf16 vector: int32 [n / 2, 2] = (pair of values, call number)."""
    pairs = values_bf16.contiguous().view(torch.int32)
    return torch.stack([pairs, torch.full_like(pairs, call)], dim=1).contiguous()


class HostPlayedWorld:
    """Rank 0 of a world of two on one GPU: the second arena is a plain local buffer."""

    def __init__(self, vectors, slots):
        self.offsets, at = {}, 0
        for name, n in vectors.items():
            self.offsets[name] = at
            at += (4 * n + 255) // 256 * 256
        self.slots = slots
        self.arena = [torch.zeros(at // 4, dtype=torch.int32, device="cuda") for _ in range(2)]
        self.arena_table = torch.tensor([a.data_ptr() for a in self.arena], dtype=torch.int64, device="cuda")
        self.state = torch.zeros(4 * slots, dtype=torch.int32, device="cuda")

    def cells(self, rank, name, n):
        """int32 view [n / 2, 2] of a vector's cells in `rank`'s arena."""
        return self.arena[rank][self.offsets[name] // 4: self.offsets[name] // 4 + n].view(-1, 2)

    def values(self, rank, name, n):
        return self.cells(rank, name, n)[:, 0].contiguous().view(torch.bfloat16)

    def spec(self, out_names, row_offsets, out_slot, in_slot):
        dp = lambda t: abi.DevicePtr(t.data_ptr())
        offs = (abi.size_t * 4)(*([self.offsets[n] for n in out_names] + [0] * (4 - len(out_names))))
        rows = (abi.size_t * 4)(*(list(row_offsets) + [0] * (4 - len(row_offsets))))
        return abi.Nvfp4MatvecPeerSpec(2, 0, dp(self.arena_table), dp(self.state), self.slots, out_slot,
                                       abi.PEER_INPUT_LOCAL if in_slot is None else in_slot, offs, rows)


def call_peer(backend, x_ptr, k, mats, peer):
    dp = lambda t: abi.DevicePtr(t.data_ptr())
    specs = (abi.Nvfp4MatvecSpec * len(mats))()
    for i, (w, sf, ts) in enumerate(mats):
        specs[i] = abi.Nvfp4MatvecSpec(w.shape[0], k, abi.DevicePtr(x_ptr), dp(w), dp(sf), dp(ts), abi.DevicePtr(0))
    return backend.lib.qwen36_nvfp4_matvec_peer(specs, len(mats), C.byref(peer))


def test_rank0_of_two_with_host_played_peer(backend):
    gen = torch.Generator(device="cuda").manual_seed(92)
    k0, n1, n2 = 512, 1024, 768
    w1, w2 = weights(backend, gen, n1, k0), weights(backend, gen, n2, n1)
    x = torch.randn(k0, generator=gen, device="cuda").to(torch.bfloat16)
    h_full = backend.nvfp4_matvec(x, *w1)                     # what the two ranks produce together
    y_full = backend.nvfp4_matvec(h_full, *w2)
    world = HostPlayedWorld({"h": n1, "y": n2}, 2)
    half1, half2 = n1 // 2, 384
    # the peer (rank 1) has delivered its half of h under call number 1
    world.cells(0, "h", n1)[half1 // 2:] = cells_of(h_full[half1:], 1)
    torch.cuda.synchronize()
    assert call_peer(backend, x.data_ptr(), k0, [(w1[0][:half1], w1[1][: half1 // 128 * (k0 // 64) * 512], w1[2])],
                     world.spec(["h"], [0], 0, None)) == abi.SUCCESS
    # second call: consumes h (slot 0), produces rows [0, 384) of y into both arenas
    sf2_bytes = half2 // 128 * (n1 // 64) * 512
    h_cells = world.arena[0].data_ptr() + world.offsets["h"]
    assert call_peer(backend, h_cells, n1, [(w2[0][:half2], w2[1][:sf2_bytes], w2[2])],
                     world.spec(["y"], [0], 1, 0)) == abi.SUCCESS
    torch.cuda.synchronize()
    assert backend.lib.qwen36_nvfp4_gemv_mma_last_error() == 0
    for rank in (0, 1):                                      # both arenas received rank 0's rows, flagged with call 1
        assert torch.equal(world.values(rank, "h", n1)[:half1].view(torch.int16), h_full[:half1].view(torch.int16))
        assert torch.equal(world.values(rank, "y", n2)[:half2].view(torch.int16), y_full[:half2].view(torch.int16))
        assert (world.cells(rank, "y", n2)[: half2 // 2, 1] == 1).all()
    assert torch.count_nonzero(world.cells(1, "y", n2)[half2 // 2:]) == 0          # nothing outside the slice
    assert world.state.view(-1, 4)[:, :3].tolist() == [[1, 0, 0], [1, 0, 0]]
    # the unpacking entry on the complete vector h of arena 0
    out = torch.empty(n1, dtype=torch.bfloat16, device="cuda")
    peer = world.spec([], [], 0, None)
    assert backend.lib.qwen36_nvfp4_matvec_peer_collect(C.byref(peer), 0, abi.DevicePtr(h_cells), n1,
                                                        abi.DevicePtr(out.data_ptr())) == abi.SUCCESS
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), h_full.view(torch.int16))


def test_missing_peer_poisons_the_rows_and_records_the_call(backend):
    gen = torch.Generator(device="cuda").manual_seed(93)
    k0, n1 = 512, 256
    w1 = weights(backend, gen, n1, k0)
    x = torch.randn(k0, generator=gen, device="cuda").to(torch.bfloat16)
    world = HostPlayedWorld({"x": k0, "y": n1}, 2)
    world.state[0] = 1                                      # this rank's producer of slot 0 has completed call 1
    world.cells(0, "x", k0)[: k0 // 4] = cells_of(x[: k0 // 2], 1)     # its own half is there; the peer's never comes
    torch.cuda.synchronize()
    x_cells = world.arena[0].data_ptr() + world.offsets["x"]
    assert call_peer(backend, x_cells, k0, [(w1[0][:128], w1[1][: (k0 // 64) * 512], w1[2])],
                     world.spec(["y"], [0], 1, 0)) == abi.SUCCESS
    torch.cuda.synchronize()
    try:
        assert backend.lib.qwen36_nvfp4_gemv_mma_last_error() == 2
        for rank in (0, 1):
            assert torch.isnan(world.values(rank, "y", n1)[:128].float()).all()
            assert (world.cells(rank, "y", n1)[:64, 1] == 1).all()          # the poison travels under the call's number
        assert world.state.view(-1, 4)[1, :3].tolist() == [1, 0, 1]         # call 1 of slot 1 went out poisoned
    finally:
        assert backend.lib.qwen36_nvfp4_gemv_mma_reset_error() == 0


def test_argument_checks(backend):
    world = HostPlayedWorld({"x": 512, "y": 256}, 2)
    gen = torch.Generator(device="cuda").manual_seed(94)
    w1 = weights(backend, gen, 256, 512)
    mats = [(w1[0][:128], w1[1][: 8 * 512], w1[2])]
    x = torch.zeros(512, dtype=torch.bfloat16, device="cuda")
    bad = world.spec(["y"], [4], 1, None)                   # row offset not a multiple of 8
    assert call_peer(backend, x.data_ptr(), 512, mats, bad) == abi.INVALID_ARGUMENT
    bad = world.spec(["y"], [0], 2, None)                   # slot out of range
    assert call_peer(backend, x.data_ptr(), 512, mats, bad) == abi.INVALID_ARGUMENT
    ok = world.spec(["y"], [0], 1, None)
    assert backend.lib.qwen36_nvfp4_matvec_peer(None, 1, C.byref(ok)) == abi.NULL_POINTER
    odd = [(w1[0][:64], w1[1][: 8 * 512], w1[2])]           # 64 rows: not a whole scale-tile block
    assert call_peer(backend, x.data_ptr(), 512, odd, ok) == abi.NOT_IMPLEMENTED
    assert backend.lib.qwen36_nvfp4_matvec_peer_collect(C.byref(ok), 0, abi.DevicePtr(x.data_ptr()), 6,
                                                        abi.DevicePtr(x.data_ptr())) == abi.INVALID_ARGUMENT
