"""glqb_trellis_linear_noalloc against the ordinary (plan + caller workspace) entry point.

The entry point under test serves callers that must not allocate device memory where they run a
layer (memory fixed at start-up, code running inside another allocator's callback, programs without
an allocator): it keeps its scratch in a fixed array inside the library.  All calls share that array,
so the test makes two calls in a row with different layers and inputs and checks each against the
plan-based result.  This file sorts last on purpose: a run that stops at the first failure has then
already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-3      # same bound as the other layer-output tests (max |err| / max |ref|)


def _layer(rng, m, n, K):
    packed = rng.integers(0, 65536, size=((m // 16) * (n // 16), 16 * K), dtype=np.uint16).view(np.int16)
    su = (rng.integers(0, 2, size=m) * 2 - 1).astype(np.float16)
    sv = (rng.integers(0, 2, size=n) * 2 - 1).astype(np.float16)
    x = rng.standard_normal((1, n)).astype(np.float32)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return dev(packed), dev(su), dev(sv), dev(x)


def _blocks(n):
    out = []
    while n:
        p = 1 << (n.bit_length() - 1)
        out.append(p)
        n -= p
    return out


def _noalloc(lib, x, packed, su, sv, wscale, m, n, K):
    y = torch.empty(1, m, dtype=torch.float32, device="cuda")
    bn, bm = _blocks(n), _blocks(m)
    rc = lib.glqb_trellis_linear_noalloc(x.data_ptr(), 2, y.data_ptr(), 2, packed.data_ptr(), K, su.data_ptr(),
                                         sv.data_ptr(), C.c_float(wscale), m, n, (C.c_int32 * len(bn))(*bn), len(bn),
                                         (C.c_int32 * len(bm))(*bm), len(bm),
                                         torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.glqb_last_error()
    return y


def test_two_calls_in_a_row_match_the_plan_entry_point():
    from glq_b200 import _lib, ops
    lib = _lib.load()
    assert lib.glqb_noalloc_scratch_bytes() == 4 << 20
    rng = np.random.default_rng(2024)
    cases = [(352, 576, 4, 0.031), (2048, 2048, 4, 0.017), (96, 128, 2, 0.05)]
    layers = [(_layer(rng, m, n, K), m, n, K, ws) for (m, n, K, ws) in cases]
    # back-to-back calls on one stream: each reuses the scratch the previous one left behind
    got = [_noalloc(lib, x, packed, su, sv, ws, m, n, K) for ((packed, su, sv, x), m, n, K, ws) in layers]
    got2 = [_noalloc(lib, x, packed, su, sv, ws, m, n, K) for ((packed, su, sv, x), m, n, K, ws) in layers]
    torch.cuda.synchronize()
    from oracle import c_oracle as CO
    from oracle import glq_oracle as O
    for ((packed, su, sv, x), m, n, K, ws), y, y2 in zip(layers, got, got2):
        ref = ops.fused_linear_trellis_3inst(x, sv, su, packed, None, None, None, None, ws, n, m, n, m,
                                             out_dtype=torch.float32)
        err = (y - ref).abs().max().item() / ref.abs().max().item()
        assert err <= TOL, (m, n, K, err)
        assert torch.equal(y, y2)          # same call, same scratch, same bits
        # and against the CPU oracle directly, not only against the other CUDA entry point
        W = CO.trellis_decode(packed.cpu().numpy(), m, n, K).astype(np.float32)
        oracle = O.linear_forward(x.cpu().numpy(), W, su.cpu().numpy(), sv.cpu().numpy(), ws)
        assert np.abs(y.cpu().numpy() - oracle).max() / np.abs(oracle).max() <= TOL, (m, n, K)


def test_sizes_beyond_the_built_in_scratch_are_refused():
    from glq_b200 import _lib
    lib = _lib.load()
    t = torch.zeros(64, dtype=torch.float32, device="cuda")
    one = (C.c_int32 * 1)(65536)
    rc = lib.glqb_trellis_linear_noalloc(t.data_ptr(), 2, t.data_ptr(), 2, t.data_ptr(), 4, t.data_ptr(),
                                         t.data_ptr(), C.c_float(1.0), 65536, 65536, one, 1, one, 1, None)
    assert rc == -1 and b"exceeds the built-in scratch" in lib.glqb_last_error()
