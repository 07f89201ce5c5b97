"""One rank of the two-GPU check of the peer-memory combines (started by test_gpu_peer.py through
torch.distributed.run): every call is compared with the all-gather route, eagerly and as a replayed
CUDA graph."""
import os
import sys

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    from speedoza_b200 import shard
    from speedoza_b200.backend import CudaBackend
    from speedoza_b200.peer import ArgmaxPeerCombine, AttentionPeerMerge
    b = CudaBackend()
    heads, dim, n = 24, 256, 4
    merge = AttentionPeerMerge(b, heads, dim, "cuda")
    pick = ArgmaxPeerCombine(b, n, "cuda")
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    for call in range(12):
        m = torch.randn(heads, generator=gen, device="cuda") * 3
        l = torch.rand(heads, generator=gen, device="cuda") * 50 + 1
        o = torch.randn((heads, dim), generator=gen, device="cuda") * l[:, None]
        if call == 3 and rank == 1:
            m[:] = float("-inf"); l[:] = 0; o[:] = 0            # a rank with no tokens
        got = merge(m, l, o).clone()
        pm, pl, po = shard.gather_partials(m, l, o, world)
        assert torch.equal(got, b.attention_merge_partials(pm, pl, po)), ("merge", call)
        v = torch.randn(n, generator=gen, device="cuda")
        i = torch.randint(0, 248320, (n,), generator=gen, device="cuda", dtype=torch.int32)
        if call == 5:
            v[:] = 1.0                                          # ties across ranks
        assert torch.equal(pick(v, i).to(torch.int64), shard.gather_argmax(v, i, world)[1]), ("argmax", call)
    # fused route: attention over this rank's rows + cross-rank merge in two launches
    tokens = 3000 + 500 * rank
    k = torch.randn((tokens, 4, dim), generator=gen, device="cuda").to(torch.bfloat16)
    v = torch.randn((tokens, 4, dim), generator=gen, device="cuda").to(torch.bfloat16)
    q = torch.randn((heads, dim), device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)).to(torch.bfloat16)
    kq = torch.empty((tokens, 4, dim), dtype=torch.int8, device="cuda"); vq = torch.empty_like(kq)
    meta = torch.empty((tokens, 4, 2), dtype=torch.float32, device="cuda")
    b.turboquant_encode_kv_rows(k, v, kq, vq, meta, 0)
    ws = b.attention_workspace(heads, dim, "cuda")
    for t_end in (tokens, 0 if rank == 1 else 77):
        got = merge.attend(q, kq, vq, meta, 0, t_end, ws).clone()
        pm, pl, po = shard.gather_partials(*b.turboquant_attention_partial(q, kq, vq, meta, 0, t_end, ws), world)
        assert torch.equal(got, b.attention_merge_partials(pm, pl, po)), ("fused", t_end)
    # replayed graph: the call number advances on the device
    m = torch.randn(heads, generator=gen, device="cuda"); l = torch.rand(heads, generator=gen, device="cuda") + 1
    o = torch.randn((heads, dim), generator=gen, device="cuda")
    out = torch.empty((heads, dim), dtype=torch.bfloat16, device="cuda")
    pm, pl, po = shard.gather_partials(m, l, o, world)
    want = b.attention_merge_partials(pm, pl, po)
    torch.cuda.synchronize(); dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, capture_error_mode="thread_local"):
        b.sync_stream()
        merge(m, l, o, out)
    b.sync_stream()
    for replay in range(7):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want), ("graph", replay)
    assert not merge.ex.failed()
    del graph
    merge.ex.close()
    pick.ex.close()
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print("PEER_OK", flush=True)
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
