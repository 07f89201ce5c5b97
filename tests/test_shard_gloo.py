"""Host-side logic of the multi-GPU path on CPU: two gloo ranks partition, gather and combine.
The device kernels are replaced by the CPU oracle here (test infrastructure); what is under test
is speedoza_b200/shard.py: row/token partition, padded all-gather, argmax tie rule across ranks,
(m, l, o) gather layout."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, case, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle as orc
        from speedoza_b200 import shard, synth
        rng = np.random.default_rng(5)                   # same data on every rank
        if case == "rows":
            for n in (1024, 5120, 640, 200):
                full = torch.arange(n, dtype=torch.float32)
                lo, hi = shard.shard_rows(n, rank, world)
                got = shard.all_gather_rows(full[lo:hi].clone(), n, world)
                assert torch.equal(got, full), n
        elif case == "argmax":
            rows, cols, n = 1024, 256, 3
            w, s = synth.lm_head_weight(rng, rows, cols)
            w[700] = w[100]; s[700] = s[100]              # identical rows on different ranks -> exact tie
            x = synth.activations(rng, n, cols)
            logits = orc.lm_head_fp8_gemv(w, s, x)
            # make that tie the maximum of token 0
            lo, hi = shard.shard_rows(rows, rank, world)
            lf = synth.bf16_bits_to_f32(logits).copy()
            lf[0, 100] = lf[0, 700] = lf[0].max() + 1.0
            local = lf[:, lo:hi]
            loc_idx = orc.argmax_rows(synth.f32_to_bf16_bits(local))
            val = torch.from_numpy(np.take_along_axis(local, loc_idx[:, None].astype(np.int64), 1)[:, 0].copy())
            idx = torch.from_numpy((loc_idx + lo).astype(np.int32))
            _, win = shard.gather_argmax(val, idx, world)
            want = orc.argmax_rows(synth.f32_to_bf16_bits(lf))
            assert win.tolist() == want.tolist() and win[0].item() == 100
            # NaN / -inf ranks never win
            v = torch.tensor([[float("nan"), -float("inf")], [1.0, -float("inf")]])
            i = torch.tensor([[5, 7], [9, 3]], dtype=torch.int32)
            bv, bi = shard.combine_argmax(v, i)
            assert bi.tolist() == [9, 0]
        elif case == "attention":
            T, H, KV, D = 301, 6, 2, 64
            q, k, v = synth.qkv(rng, T, H, KV, D)
            kq = np.zeros((T, KV, D), np.int8); vq = np.zeros_like(kq); meta = np.zeros((T, KV, 2), np.float32)
            orc.kv_encode(k, v, 0, kq, vq, meta)
            for position in (T - 1, 120, 0):
                lo, hi = shard.shard_tokens(T, rank, world)
                end = max(lo, min(hi, position + 1))
                m, l, o = orc.kv_attention_partial(q, kq, vq, meta, lo, end)
                pm, pl, po = shard.gather_partials(torch.from_numpy(m), torch.from_numpy(l), torch.from_numpy(o), world)
                assert pm.shape == (H, world) and po.shape == (H, world, D)
                got = synth.bf16_bits_to_f32(orc.merge_partials(pm.numpy(), pl.numpy(), po.numpy()))
                want = synth.bf16_bits_to_f32(orc.kv_attention(q, kq, vq, meta, position))
                err = np.linalg.norm(got - want) / np.linalg.norm(want)
                assert err < 1e-2, (position, err)
        elif case == "tp_chain":
            # the data flow of the tensor-parallel GEMV chain: every rank computes its row slices, the
            # slices meet in every rank's full vector (an all-gather stands in for the peer stores),
            # the next GEMV consumes the full vector; two chained layers must equal the unsplit chain
            shapes = [("a", 512, 256), ("b", 256, 512)]
            mats = {}
            for name, n, k in shapes:
                packed, sf_rm = synth.nvfp4_weight(rng, n, k)
                mats[name] = (packed, sf_rm, n, k)
            x0 = synth.activations(rng, 1, 256)[0]
            gain = synth.WEIGHT_GLOBAL_SCALE * 40.0
            full = x0
            for _ in range(2):
                for name, n, k in shapes:
                    full = orc.nvfp4_matvec(full, mats[name][0], orc.retile_scales(mats[name][1]), gain, k)
            mine = x0
            slices = shard.tp_slices(shapes, rank, world)
            offsets, total = shard.arena_layout({name: n for name, n, _ in shapes})
            assert total % 256 == 0 and all(off % 256 == 0 for off, _ in offsets.values())
            assert offsets["b"][0] >= 4 * 512                 # vectors do not overlap
            for _ in range(2):
                for name, n, k in shapes:
                    lo, hi = slices[name]
                    assert lo % 128 == 0 and (hi - lo) % 128 == 0
                    part = orc.nvfp4_matvec(mine, mats[name][0][lo:hi].copy(), orc.retile_scales(mats[name][1][lo:hi].copy()),
                                            gain, k)
                    got = shard.all_gather_rows(torch.from_numpy(synth.bf16_bits_to_f32(part).copy()), n, world)
                    mine = synth.f32_to_bf16_bits(got.numpy())        # bf16 values travel as float32: exact both ways
            assert np.array_equal(mine, full)
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", ["rows", "argmax", "attention", "tp_chain"])
def test_two_rank_gloo(case):
    world = 2
    port = 29500 + (os.getpid() % 2000) + {"rows": 0, "argmax": 1, "attention": 2, "tp_chain": 3}[case]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, case, ret), nprocs=world, join=True)
    assert dict(ret) == {0: "ok", 1: "ok"}


def test_partitions_cover_everything():
    sys.path.insert(0, ROOT)
    from speedoza_b200 import shard
    for n in (1024, 5120, 12288, 34816, 248320, 200, 129):
        for world in (1, 2, 4, 8):
            spans = [shard.shard_rows(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(lo % 128 == 0 for lo, _ in spans)
    for t in (1, 8192, 131072, 1000):
        for world in (1, 2, 4, 8):
            spans = [shard.shard_tokens(t, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == t and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
