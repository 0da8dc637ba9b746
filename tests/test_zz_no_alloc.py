"""The allocation-free routing entry point, called through its exported C symbol.

Some hosts cannot call cudaMalloc while they use this library (a server that owns the whole device
through its own pool, a latency-critical thread that must not take allocator locks). For them
`fastb_route_topk_noalloc` keeps its intermediate tables in a fixed array inside the library. This
test calls it with ctypes, twice in a row with different inputs, and compares with the regular
routing entry point and with a plain PyTorch top-k. It is collected last so that a failure here cannot hide other results.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from fast_b200 import runtime

    lib = ctypes.CDLL(runtime.ext().__file__)
    fn = lib.fastb_route_topk_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                   ctypes.c_void_p]
    lib.fastb_noalloc_last_error.restype = ctypes.c_char_p
    return lib, fn


def _regular(logits, bias, K):
    from fast_b200 import runtime

    C = runtime.ext()
    T, E = logits.shape
    nb = (T + C.ROUTE_TOKENS_PER_BLOCK - 1) // C.ROUTE_TOKENS_PER_BLOCK
    idx = torch.empty(T, K, dtype=torch.int32, device="cuda")
    w = torch.empty(T, K, dtype=torch.float32, device="cuda")
    slot = torch.zeros(nb * C.ROUTE_TOKENS_PER_BLOCK, K, dtype=torch.int32, device="cuda")
    cnt = torch.zeros(nb, E, dtype=torch.int32, device="cuda")
    C.route_topk(logits, bias, K, idx, w, slot, cnt)
    return idx, w, cnt.sum(0).to(torch.int32)


def test_no_alloc_route_matches_regular_twice():
    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for seed, (T, E, K) in enumerate([(5000, 256, 8), (777, 8, 2)]):  # second call is smaller: stale scratch must not leak in
        g = torch.Generator(device="cuda").manual_seed(40 + seed)
        logits = torch.randn(T, E, generator=g, device="cuda")
        bias = torch.randn(E, generator=g, device="cuda")
        idx = torch.full((T, K), -7, dtype=torch.int32, device="cuda")
        w = torch.zeros(T, K, dtype=torch.float32, device="cuda")
        counts = torch.full((E,), -1, dtype=torch.int32, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = fn(logits.data_ptr(), bias.data_ptr(), T, E, K, idx.data_ptr(), w.data_ptr(), counts.data_ptr(), stream)
        assert rc == 0, lib.fastb_noalloc_last_error()
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        ridx, rw, rcounts = _regular(logits, bias, K)
        assert torch.equal(idx, ridx)
        assert torch.allclose(w, rw, atol=1e-6, rtol=0)
        assert torch.equal(counts, rcounts)
        assert int(counts.sum()) == T * K
        # Independent of this library: top-k of (logits + bias) in PyTorch, softmax of the raw logits over it.
        ref = (logits + bias).topk(K, dim=-1).indices
        assert torch.equal(idx.long(), ref)
        assert torch.allclose(w, torch.softmax(logits.gather(1, ref), dim=-1), atol=1e-5, rtol=0)
        assert torch.equal(counts.long(), torch.bincount(ref.reshape(-1), minlength=E))


def test_no_alloc_route_rejects_oversize():
    lib, fn = _lib()
    mt, me, mk = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    lib.fastb_route_topk_noalloc_limits(ctypes.byref(mt), ctypes.byref(me), ctypes.byref(mk))
    assert (mt.value, me.value, mk.value) == (16384, 256, 8)
    x = torch.zeros(8, device="cuda")
    rc = fn(x.data_ptr(), None, mt.value + 1, 8, 2, x.data_ptr(), x.data_ptr(), x.data_ptr(), None)
    assert rc != 0 and b"exceed" in lib.fastb_noalloc_last_error()
    rc = fn(x.data_ptr(), None, 16, me.value + 1, 2, x.data_ptr(), x.data_ptr(), x.data_ptr(), None)
    assert rc != 0 and b"experts" in lib.fastb_noalloc_last_error()
