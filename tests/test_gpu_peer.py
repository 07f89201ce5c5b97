"""Cross-rank combine kernels over peer memory (speedoza_b200/csrc/peer_combine.cu).

On one GPU the second rank is played by the host: its piece and its flag are written into the inbox
before the kernel starts, so nothing waits.  The real two-process run over NVLink needs two GPUs and
is skipped otherwise."""
import ctypes as C
import os
import subprocess
import sys

import pytest
import torch

from speedoza_b200 import abi

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def backend():
    from speedoza_b200.backend import CudaBackend
    return CudaBackend()


def _tables(*tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device="cuda")


def _partials(gen, world, heads, dim):
    m = torch.randn((world, heads), generator=gen, device="cuda") * 3
    l = torch.rand((world, heads), generator=gen, device="cuda") * 50 + 1
    o = torch.randn((world, heads, dim), generator=gen, device="cuda") * l[:, :, None]
    return m, l, o


def test_lone_rank_merge_is_the_local_merge_and_survives_many_calls(backend):
    from speedoza_b200.peer import ArgmaxPeerCombine, AttentionPeerMerge
    gen = torch.Generator(device="cuda").manual_seed(5)
    merge = AttentionPeerMerge(backend, 24, 256, "cuda")
    for call in range(5):                                       # both slots, growing call numbers
        m, l, o = _partials(gen, 1, 24, 256)
        got = merge(m[0].contiguous(), l[0].contiguous(), o[0].contiguous())
        want = backend.attention_merge_partials(m[0][:, None].contiguous(), l[0][:, None].contiguous(),
                                                o[0][:, None, :].contiguous())
        assert torch.equal(got, want), call
    assert int(merge.ex.state[0]) == 5 and int(merge.ex.state[1]) == 0
    pick = ArgmaxPeerCombine(backend, 8, "cuda")
    for n in (1, 4, 8):
        v = torch.randn(n, generator=gen, device="cuda")
        i = torch.randint(0, 248320, (n,), generator=gen, device="cuda", dtype=torch.int32)
        assert torch.equal(pick(v, i), i)
    assert not merge.ex.failed()
    merge.ex.close()
    pick.ex.close()


@pytest.mark.parametrize("tokens", [1, 300, 5000])
def test_lone_rank_fused_attention_equals_the_single_gpu_call(backend, tokens):
    from speedoza_b200.peer import AttentionPeerMerge
    gen = torch.Generator(device="cuda").manual_seed(tokens)
    k = torch.randn((tokens, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
    v = torch.randn((tokens, 4, 256), generator=gen, device="cuda").to(torch.bfloat16)
    q = torch.randn((24, 256), generator=gen, device="cuda").to(torch.bfloat16)
    kq = torch.empty((tokens, 4, 256), dtype=torch.int8, device="cuda"); vq = torch.empty_like(kq)
    meta = torch.empty((tokens, 4, 2), dtype=torch.float32, device="cuda")
    backend.turboquant_encode_kv_rows(k, v, kq, vq, meta, 0)
    ws = backend.attention_workspace(24, 256, "cuda")
    merge = AttentionPeerMerge(backend, 24, 256, "cuda")
    for _ in range(3):
        got = merge.attend(q, kq, vq, meta, 0, tokens, ws)
        assert torch.equal(got, backend.turboquant_attention(q, kq, vq, meta, tokens - 1, ws))
    assert not merge.ex.failed()
    merge.ex.close()


@pytest.mark.parametrize("world,rank", [(2, 0), (2, 1), (8, 3)])
def test_merge_with_host_played_peers_equals_merge_partials(backend, world, rank):
    heads, dim = 24, 256
    gen = torch.Generator(device="cuda").manual_seed(world * 10 + rank)
    m, l, o = _partials(gen, world, heads, dim)
    m[world - 1, 3] = float("-inf"); l[world - 1, 3] = 0; o[world - 1, 3] = 0      # an empty shard
    row = (dim + 2 + 3) // 4 * 4              # rows are padded to 16 bytes
    inbox = torch.zeros((2, world, heads, row), dtype=torch.float32, device="cuda")
    flags = torch.zeros((world, heads), dtype=torch.int32, device="cuda")
    sink = [torch.zeros_like(inbox) for _ in range(world)]      # where the pushes to the "peers" land
    sink_flags = [torch.zeros_like(flags) for _ in range(world)]
    # call number 1 -> slot 1; the peers' rows and flags are already there
    for p in range(world):
        if p != rank:
            inbox[1, p, :, :dim] = o[p]; inbox[1, p, :, dim] = m[p]; inbox[1, p, :, dim + 1] = l[p]
            flags[p, :] = 1
    boxes = [inbox if p == rank else sink[p] for p in range(world)]
    flgs = [flags if p == rank else sink_flags[p] for p in range(world)]
    t_in, t_fl = _tables(*boxes), _tables(*flgs)
    state = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.zeros((heads, dim), dtype=torch.bfloat16, device="cuda")
    dp = lambda t: abi.DevicePtr(t.data_ptr())
    po, pm, pl = o[rank].contiguous(), m[rank].contiguous(), l[rank].contiguous()
    spec = abi.AttentionPeerMergeSpec(world, rank, heads, dim, dp(po), dp(pm), dp(pl), dp(t_in), dp(t_fl), dp(state),
                                      dp(out))
    assert backend.lib.qwen36_attention_peer_merge(C.byref(spec)) == abi.SUCCESS
    torch.cuda.synchronize()
    want = backend.attention_merge_partials(m.t().contiguous(), l.t().contiguous(), o.permute(1, 0, 2).contiguous())
    assert torch.equal(out, want)
    assert int(state[0]) == 1 and int(backend.lib.qwen36_peer_last_error()) == 0
    for p in range(world):                                      # every peer got this rank's rows and flags
        if p != rank:
            assert torch.equal(sink[p][1, rank, :, :dim], po) and torch.equal(sink[p][1, rank, :, dim], pm)
            assert torch.equal(sink[p][1, rank, :, dim + 1], pl)
            assert bool((sink_flags[p][rank] == 1).all()) and int(sink[p][0].abs().sum()) == 0


def test_argmax_with_host_played_peers_follows_the_greedy_rule(backend):
    from speedoza_b200 import shard
    world, rank, n = 4, 2, 8
    gen = torch.Generator(device="cuda").manual_seed(9)
    v = torch.randn((world, n), generator=gen, device="cuda")
    i = torch.randint(0, 248320, (world, n), generator=gen, device="cuda", dtype=torch.int32)
    v[:, 1] = 0.5                                               # a four-way tie: lowest index wins
    v[0, 2] = float("nan")                                      # NaN never wins
    v[:, 3] = float("-inf"); i[:, 3] = torch.tensor([7, 5, 9, 6], dtype=torch.int32, device="cuda")
    inbox = torch.zeros((2, world, 2, n), dtype=torch.int32, device="cuda")
    flags = torch.zeros(world, dtype=torch.int32, device="cuda")
    sink = [torch.zeros_like(inbox) for _ in range(world)]
    sink_flags = [torch.zeros_like(flags) for _ in range(world)]
    for p in range(world):
        if p != rank:
            inbox[1, p, 0] = v[p].view(torch.int32); inbox[1, p, 1] = i[p]; flags[p] = 1
    t_in = _tables(*[inbox if p == rank else sink[p] for p in range(world)])
    t_fl = _tables(*[flags if p == rank else sink_flags[p] for p in range(world)])
    state = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.full((n,), -1, dtype=torch.int32, device="cuda")
    dp = lambda t: abi.DevicePtr(t.data_ptr())
    mv, mi = v[rank].contiguous(), i[rank].contiguous()
    spec = abi.ArgmaxPeerCombineSpec(world, rank, n, dp(mv), dp(mi), dp(t_in), dp(t_fl), dp(state), dp(out))
    assert backend.lib.qwen36_argmax_peer_combine(C.byref(spec)) == abi.SUCCESS
    torch.cuda.synchronize()
    want = shard.combine_argmax(v, i)[1]
    assert torch.equal(out.to(torch.int64), want)
    assert int(out[3]) == 0                                     # nothing beats the (-inf, 0) start


def test_a_peer_that_never_answers_ends_in_an_error_status_not_a_hang(backend):
    """The flag of rank 1 is never raised: the wait runs out, the output is poisoned (token 0xFFFFFFFF),
    state[2] names the failed call (both readable without a synchronising query), the sticky status
    says so too, and the context is still usable afterwards."""
    world, rank, n = 2, 0, 4
    inbox = [torch.zeros((2, world, 2, n), dtype=torch.int32, device="cuda") for _ in range(world)]
    flags = [torch.zeros(world, dtype=torch.int32, device="cuda") for _ in range(world)]
    t_in, t_fl = _tables(*inbox), _tables(*flags)
    state = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.full((n,), 7, dtype=torch.int32, device="cuda")
    v = torch.ones(n, device="cuda"); i = torch.arange(n, dtype=torch.int32, device="cuda")
    dp = lambda t: abi.DevicePtr(t.data_ptr())
    spec = abi.ArgmaxPeerCombineSpec(world, rank, n, dp(v), dp(i), dp(t_in), dp(t_fl), dp(state), dp(out))
    assert backend.lib.qwen36_peer_reset_error() == abi.SUCCESS
    assert backend.lib.qwen36_argmax_peer_combine(C.byref(spec)) == abi.SUCCESS
    torch.cuda.synchronize()
    assert int(backend.lib.qwen36_peer_last_error()) == 1
    assert bool((out == -1).all())                              # 0xFFFFFFFF: no vocabulary has this token
    assert state.tolist() == [1, 0, 1, 0]                       # call 1 completed, and call 1 is the failed one
    # the attention merge poisons its rows the same way
    heads, dim, row = 2, 64, 68
    a_inbox = [torch.zeros((2, world, heads, row), device="cuda") for _ in range(world)]
    a_flags = [torch.zeros((world, heads), dtype=torch.int32, device="cuda") for _ in range(world)]
    a_state = torch.zeros(4, dtype=torch.int32, device="cuda")
    a_out = torch.zeros((heads, dim), dtype=torch.bfloat16, device="cuda")
    po = torch.ones((heads, dim), device="cuda"); pm = torch.zeros(heads, device="cuda"); pl = torch.ones(heads, device="cuda")
    a_spec = abi.AttentionPeerMergeSpec(world, rank, heads, dim, dp(po), dp(pm), dp(pl), dp(_tables(*a_inbox)),
                                        dp(_tables(*a_flags)), dp(a_state), dp(a_out))
    assert backend.lib.qwen36_attention_peer_merge(C.byref(a_spec)) == abi.SUCCESS
    torch.cuda.synchronize()
    assert bool(torch.isnan(a_out.float()).all()) and int(a_state[2]) == 1
    assert backend.lib.qwen36_peer_reset_error() == abi.SUCCESS
    assert int(backend.lib.qwen36_peer_last_error()) == 0
    assert int((torch.ones(4, device="cuda") * 2).sum()) == 8


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs of one node")
def test_two_processes_over_nvlink_agree_with_the_collective_combine():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29641", os.path.join(ROOT, "tests", "peer_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    assert "PEER_OK" in res.stdout
