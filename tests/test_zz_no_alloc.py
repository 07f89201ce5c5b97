"""The allocation-free attention entry point, for callers that cannot provide scratch memory
(no cudaMalloc allowed where they run): it must give what the workspace-based entry point
gives.  Called through the C ABI, twice in a row, with different inputs, because the built-in
scratch buffer keeps the previous call's contents."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import oracle as orc
from speedoza_b200 import abi, synth
from conftest import bf16_host, to_dev

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    a = a.float().cpu().numpy().astype(np.float64); b = b.float().cpu().numpy().astype(np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def make_cache(backend, rng, tokens):
    q, k, v = synth.qkv(rng, tokens)
    kq = torch.zeros((tokens, 4, 256), dtype=torch.int8, device="cuda"); vq = torch.zeros_like(kq)
    meta = torch.zeros((tokens, 4, 2), dtype=torch.float32, device="cuda")
    backend.turboquant_encode_kv_rows(to_dev(k), to_dev(v), kq, vq, meta, 0)
    return to_dev(q), kq, vq, meta, q


def test_static_scratch_attention_matches_workspace_entry(backend):
    rng = np.random.default_rng(123)
    lib = backend.lib
    ws = backend.attention_workspace(24, 256, "cuda")
    shape = abi.AttentionShape(24, 4, 256, 0)
    # long context first, short second: the second call must not see the first call's partials
    for tokens in (5000, 130):
        q, kq, vq, meta, q_host = make_cache(backend, rng, tokens)
        want = torch.empty((24, 256), dtype=torch.bfloat16, device="cuda")
        got = torch.full((24, 256), float("nan"), dtype=torch.bfloat16, device="cuda")
        dp = lambda t: abi.DevicePtr(t.data_ptr())
        spec_ws = abi.TurboquantAttentionSpec(0, tokens - 1, dp(q), dp(kq), dp(vq), dp(meta), dp(want), dp(ws),
                                              ws.numel(), shape, 0)
        spec_static = abi.TurboquantAttentionSpec(0, tokens - 1, dp(q), dp(kq), dp(vq), dp(meta), dp(got),
                                                  abi.DevicePtr(0), 0, shape, 0)
        assert lib.qwen36_turboquant_attention(C.byref(spec_ws)) == abi.SUCCESS
        torch.cuda.synchronize()
        # the entry point itself must allocate nothing: neither through the library's allocator (its call
        # counter stays put) nor behind its back (the device's free memory stays put)
        before, free_before = abi.CudaCounters(), torch.cuda.mem_get_info()[0]
        assert lib.qwen36_cuda_counters_read(C.byref(before)) == abi.SUCCESS
        assert lib.qwen36_turboquant_attention_static(C.byref(spec_static)) == abi.SUCCESS
        torch.cuda.synchronize()
        after = abi.CudaCounters()
        assert lib.qwen36_cuda_counters_read(C.byref(after)) == abi.SUCCESS
        assert (after.malloc_calls, after.free_calls) == (before.malloc_calls, before.free_calls)
        assert torch.cuda.mem_get_info()[0] == free_before
        assert rel_l2(got, want) <= 1e-2          # the tolerance of the attention parity tests
        assert torch.equal(got, want)              # same kernels, same order: in fact identical
        # and against the CPU restatement of the reference's attention over the same cache bytes
        oracle_out = orc.kv_attention(q_host, kq.cpu().numpy(), vq.cpu().numpy(), meta.cpu().numpy(), tokens - 1)
        a = synth.bf16_bits_to_f32(bf16_host(got)).astype(np.float64)
        b = synth.bf16_bits_to_f32(oracle_out).astype(np.float64)
        assert np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30) <= 1e-2


def test_static_scratch_rejects_shapes_beyond_its_size(backend):
    lib = backend.lib
    lib.qwen36_turboquant_attention_static_max_head_floats.restype = C.c_size_t
    cap = lib.qwen36_turboquant_attention_static_max_head_floats()
    assert cap == 32 * 258
    q_heads = 64                                   # 64 * 258 floats per split: over the limit
    assert q_heads * 258 > cap
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    p = abi.DevicePtr(buf.data_ptr())
    spec = abi.TurboquantAttentionSpec(0, 3, p, p, p, p, p, abi.DevicePtr(0), 0, abi.AttentionShape(q_heads, 4, 256, 0), 0)
    assert lib.qwen36_turboquant_attention_static(C.byref(spec)) == abi.INVALID_ARGUMENT
    assert lib.qwen36_turboquant_attention_static(None) == abi.NULL_POINTER
