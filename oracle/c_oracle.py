"""ctypes loader for the C restatement of the oracle (oracle/kvq_oracle.c).
Test infrastructure only; see the header of kvq_oracle.c."""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "libkvq_oracle.so")
_LIB = None


def load(build_if_missing=True):
    global _LIB
    if _LIB is None:
        if not os.path.exists(SO) and build_if_missing:
            subprocess.run(["make", "-s", "-C", HERE], check=True)
        _LIB = C.CDLL(SO)
        _LIB.kvq_oracle_num_threads.restype = C.c_int
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def num_threads():
    return int(load().kvq_oracle_num_threads())


def decode_attn(fmt, q, k, v, ks, vs, ctx, sm_scale, inv_tau=None, kz=None, vz=None,
                kside=None, vside=None, outlier_idx=None):
    """fmt 0 fp16 / 1 int8 / 2 packed int4.  numpy arrays, contiguous; returns fp16 [B,Hq,D]."""
    q = np.ascontiguousarray(q, np.float16)
    B, Hq, D = q.shape
    Hkv, S = k.shape[1], k.shape[2]
    G = 1 if ks is None else ks.shape[-1]
    arrs = [None if a is None else np.ascontiguousarray(a) for a in (k, v, ks, vs, kz, vz, kside, vside)]
    k, v, ks, vs, kz, vz, kside, vside = arrs
    tau = None if inv_tau is None else np.ascontiguousarray(inv_tau, np.float32)
    oidx = None if outlier_idx is None else np.ascontiguousarray(outlier_idx, np.int16)
    n_out = 0 if oidx is None else oidx.shape[1]
    ctx = np.ascontiguousarray(ctx, np.int32)
    out = np.empty((B, Hq, D), np.float16)
    load().kvq_oracle_decode_attn(
        C.c_int(fmt), _p(q), _p(tau), _p(k), _p(v), _p(ks), _p(vs), _p(kz), _p(vz), _p(kside), _p(vside),
        _p(oidx), C.c_int(n_out), _p(ctx), C.c_int(B), C.c_int(Hq), C.c_int(Hkv), C.c_int(S), C.c_int(D),
        C.c_int(G), C.c_float(sm_scale), _p(out))
    return out


def quant_int8_static(x, table, gs):
    x = np.ascontiguousarray(x, np.float16)
    B, H, T, D = x.shape
    table = np.ascontiguousarray(table, np.float16)
    codes = np.empty(x.shape, np.int8)
    scale = np.empty((B, H, T, D // gs), np.float16)
    load().kvq_oracle_quant_int8_static(_p(x), _p(table), C.c_long(B * H * T), C.c_int(H), C.c_int(T),
                                        C.c_int(D), C.c_int(gs), _p(codes), _p(scale))
    return codes, scale


def quant_int4_static(x, table, gs):
    x = np.ascontiguousarray(x, np.float16)
    B, H, T, D = x.shape
    table = np.ascontiguousarray(table, np.float32)
    packed = np.empty((B, H, T, D // 2), np.uint8)
    scale = np.empty((B, H, T, D // gs), np.float16)
    load().kvq_oracle_quant_int4_static(_p(x), _p(table), C.c_long(B * H * T), C.c_int(H), C.c_int(T),
                                        C.c_int(D), C.c_int(gs), _p(packed), _p(scale))
    return packed.view(np.int8), scale


def quant_int4_asym(x, gs):
    x = np.ascontiguousarray(x, np.float16)
    B, H, T, D = x.shape
    packed = np.empty((B, H, T, D // 2), np.uint8)
    scale = np.empty((B, H, T, D // gs), np.float16)
    zp = np.empty((B, H, T, D // gs), np.float16)
    load().kvq_oracle_quant_int4_asym(_p(x), C.c_long(B * H * T), C.c_int(D), C.c_int(gs), _p(packed),
                                      _p(scale), _p(zp))
    return packed.view(np.int8), scale, zp
