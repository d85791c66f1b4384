"""ctypes view of libglq_oracle.so (oracle/glq_oracle.c).  TEST INFRASTRUCTURE ONLY."""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def load():
    global _LIB
    if _LIB is None:
        path = os.path.join(HERE, "libglq_oracle.so")
        src = os.path.join(HERE, "glq_oracle.c")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            subprocess.run(["make", "-C", HERE, "-s"], check=True)
        _LIB = C.CDLL(path)
        _LIB.glqo_decode_3inst.restype = C.c_uint16
        _LIB.glqo_decode_3inst.argtypes = [C.c_uint32]
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def decode_3inst_table():
    lib = load()
    return np.array([lib.glqo_decode_3inst(s) for s in range(65536)], dtype=np.uint16).view(np.float16)


def trellis_decode(packed, m, n, K):
    out = np.empty((m, n), dtype=np.uint16)
    load().glqo_trellis_decode(_p(np.ascontiguousarray(packed)), C.c_int(m), C.c_int(n), C.c_int(K), _p(out))
    return out.view(np.float16)


def trellis_decode_f32(p1, K1, p2, K2, s2, m, n):
    out = np.empty((m, n), dtype=np.float32)
    p1 = np.ascontiguousarray(p1)
    p2c = np.ascontiguousarray(p2) if p2 is not None else None
    load().glqo_trellis_decode_f32(_p(p1), C.c_int(K1), _p(p2c) if p2c is not None else None, C.c_int(K2),
                                   C.c_float(s2), C.c_int(m), C.c_int(n), _p(out))
    return out


def e8_decode(qs, tables_packed, scales, m, n):
    ns = len(qs)
    qs = [np.ascontiguousarray(q).view(np.uint16) for q in qs]
    tbs = [np.ascontiguousarray(t, dtype=np.uint32) for t in tables_packed]
    qa = (C.c_void_p * ns)(*[q.ctypes.data for q in qs])
    ta = (C.c_void_p * ns)(*[t.ctypes.data for t in tbs])
    ent = (C.c_int * ns)(*[t.size for t in tbs])
    sc = (C.c_float * ns)(1.0, *[float(s) for s in scales])
    out = np.empty((m, n), dtype=np.float32)
    load().glqo_e8_decode(qa, ta, ent, sc, C.c_int(ns), C.c_int(m), C.c_int(n), _p(out))
    return out


def fht(x):
    x = np.array(x, dtype=np.float32, copy=True)
    flat = x.reshape(-1, x.shape[-1])
    for r in flat:
        load().glqo_fht(_p(r), C.c_int(r.size))
    return flat.reshape(x.shape)


def trellis_linear(x, p1, K1, p2, K2, s2, m, n, su, sv, wscale, blocks_n, blocks_m):
    x = np.ascontiguousarray(x, dtype=np.float32)
    B = x.shape[0]
    y = np.empty((B, m), dtype=np.float32)
    bn = (C.c_int * len(blocks_n))(*blocks_n)
    bm = (C.c_int * len(blocks_m))(*blocks_m)
    p1 = np.ascontiguousarray(p1)
    p2c = np.ascontiguousarray(p2) if p2 is not None else None
    su = np.ascontiguousarray(su, dtype=np.float16)
    sv = np.ascontiguousarray(sv, dtype=np.float16)
    load().glqo_trellis_linear(_p(x), C.c_int(B), _p(p1), C.c_int(K1), _p(p2c) if p2c is not None else None,
                               C.c_int(K2), C.c_float(s2), C.c_int(m), C.c_int(n), _p(su), _p(sv),
                               C.c_float(wscale), bn, C.c_int(len(blocks_n)), bm, C.c_int(len(blocks_m)), _p(y))
    return y


def e8_linear(x, qs, tables_packed, scales, m, n, su, sv, wscale, blocks_n, blocks_m, out_f):
    x = np.ascontiguousarray(x, dtype=np.float32)
    B, in_f = x.shape
    ns = len(qs)
    qs = [np.ascontiguousarray(q).view(np.uint16) for q in qs]
    tbs = [np.ascontiguousarray(t, dtype=np.uint32) for t in tables_packed]
    qa = (C.c_void_p * ns)(*[q.ctypes.data for q in qs])
    ta = (C.c_void_p * ns)(*[t.ctypes.data for t in tbs])
    ent = (C.c_int * ns)(*[t.size for t in tbs])
    sc = (C.c_float * ns)(1.0, *[float(s) for s in scales])
    bn = (C.c_int * len(blocks_n))(*blocks_n)
    bm = (C.c_int * len(blocks_m))(*blocks_m)
    su = np.ascontiguousarray(su, dtype=np.float16)
    sv = np.ascontiguousarray(sv, dtype=np.float16)
    y = np.empty((B, out_f), dtype=np.float32)
    load().glqo_e8_linear(_p(x), C.c_int(B), C.c_int(in_f), qa, ta, ent, sc, C.c_int(ns), C.c_int(m), C.c_int(n),
                          _p(su), _p(sv), C.c_float(wscale), bn, C.c_int(len(blocks_n)), bm,
                          C.c_int(len(blocks_m)), C.c_int(out_f), _p(y))
    return y
