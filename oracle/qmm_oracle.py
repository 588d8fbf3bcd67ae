"""CPU oracle for the quantized-matmul path -- TEST INFRASTRUCTURE ONLY.

Two layers:
  * `C`: ctypes binding of qmm_oracle.c, the scalar restatement of the reference's loops
    (metal/src/ops/conv.mm:612-732, cuda/src/ops/matmul.cu:153-189,327-352,733-747).
  * `*_fast`: numpy/BLAS versions of the same arithmetic for sizes the scalar loops cannot
    finish in seconds.  tests/test_oracle.py checks each one against the C restatement.

Only tests/, the smoke test and the bench's cpu_baseline / reference legs may import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "libqmm_oracle.so")

MXK_E4M3, MXK_E5M2, MXK_E2M1 = 0, 1, 2


def build():
    """Compile the C restatement next to its source (gcc, a second or two)."""
    subprocess.check_call(["make", "-s", "-C", _HERE])


def _load():
    if not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(os.path.join(_HERE, "qmm_oracle.c")):
        build()
    lib = ctypes.CDLL(_LIB)
    P, I64, I32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    lib.oracle_wqbmm.argtypes = [P, P, I32, P, P, P, I64, I64, I64, I64, P]
    lib.oracle_qmm_acc.argtypes = [P, P, I64, I64, I64, P]
    lib.oracle_qmm_epilogue.argtypes = [P, P, P, P, I64, I64, P]
    lib.oracle_mx_matmul.argtypes = [P, I32, P, P, I32, P, I64, I64, I64, P]
    lib.oracle_int4_pack.argtypes = [P, I64, P]
    lib.oracle_scale_swizzle_index.argtypes = [I64, I64, I64]
    lib.oracle_scale_swizzle_index.restype = I64
    for name in ("oracle_e2m1_decode", "oracle_e4m3_decode", "oracle_e5m2_decode"):
        getattr(lib, name).argtypes = [ctypes.c_uint8]
        getattr(lib, name).restype = ctypes.c_float
    for name in ("oracle_e2m1_encode", "oracle_e4m3_encode"):
        getattr(lib, name).argtypes = [ctypes.c_float]
        getattr(lib, name).restype = ctypes.c_uint8
    return lib


_lib = None


def C():
    global _lib
    if _lib is None:
        _lib = _load()
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dt):
    return None if a is None else np.ascontiguousarray(a, dtype=dt)


# ------------------------------------------------------------------ 16-bit float bit helpers
def f32_to_bf16_bits(a):
    """float32 -> bf16 bit pattern, round-to-nearest-even (what __float2bfloat16_rn does)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_f16_bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).astype(np.float16).view(np.uint16)


def f16_bits_to_f32(b):
    return np.ascontiguousarray(b, dtype=np.uint16).view(np.float16).astype(np.float32)


# ------------------------------------------------------------------ table codecs (vectorised)
def _table(fn):
    return np.array([fn(i) for i in range(256)], dtype=np.float32)


_tabs = {}


def decode_table(kind):
    """256-entry (16 for e2m1) decode table taken from the C restatement."""
    if kind not in _tabs:
        lib = C()
        if kind == MXK_E4M3:
            _tabs[kind] = _table(lib.oracle_e4m3_decode)
        elif kind == MXK_E5M2:
            _tabs[kind] = _table(lib.oracle_e5m2_decode)
        else:
            _tabs[kind] = np.array([lib.oracle_e2m1_decode(i) for i in range(16)], dtype=np.float32)
    return _tabs[kind]


def unpack_nibbles(packed, count):
    """Packed sub-byte buffer -> one code per element (element 0 = low nibble)."""
    p = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)
    out = np.empty(p.size * 2, dtype=np.uint8)
    out[0::2] = p & 0xF
    out[1::2] = p >> 4
    return out[:count]


def pack_nibbles(codes):
    c = np.ascontiguousarray(codes, dtype=np.uint8).reshape(-1) & 0xF
    if c.size & 1:
        c = np.concatenate([c, np.zeros(1, np.uint8)])
    return (c[0::2] | (c[1::2] << 4)).astype(np.uint8)


def int4_unpack(packed, count):
    u = unpack_nibbles(packed, count).astype(np.int16)
    return np.where(u >= 8, u - 16, u).astype(np.int8)


def mx_decode(buf, kind, rows, cols):
    """MX operand bytes -> float32 element values [rows, cols] (no scale applied)."""
    if kind == MXK_E2M1:
        codes = unpack_nibbles(buf, rows * cols)
    else:
        codes = np.ascontiguousarray(buf, dtype=np.uint8).reshape(-1)[: rows * cols]
    return decode_table(kind)[codes].reshape(rows, cols)


def e4m3_encode(a):
    lib = C()
    flat = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    return np.fromiter((lib.oracle_e4m3_encode(float(v)) for v in flat), dtype=np.uint8, count=flat.size)


def e4m3_encode_fast(a):
    """Vectorised round-to-nearest-even e4m3 encoder (saturating); checked against the C one."""
    x = np.ascontiguousarray(a, dtype=np.float32)
    s = (np.signbit(x).astype(np.uint8) << 7)
    ax = np.abs(x).astype(np.float64)
    out = np.zeros(x.shape, dtype=np.uint8)
    sub = ax < 2.0 ** -6
    q = np.rint(ax * 512.0)
    out = np.where(sub, np.minimum(q, 8).astype(np.uint8), out)
    fr, e = np.frexp(ax)
    ue = e - 1
    qn = np.rint(fr * 16.0)
    bump = qn >= 16
    qn = np.where(bump, 8, qn)
    ue = np.where(bump, ue + 1, ue)
    code = ((ue + 7).astype(np.int64) << 3) | (qn.astype(np.int64) - 8)
    code = np.clip(code, 0, 0x7E)
    out = np.where(~sub, code.astype(np.uint8), out)
    out = np.where(ax >= 464.0, np.uint8(0x7E), out)
    out = np.where(np.isnan(x), np.uint8(0x7F), out)
    return (out | s).astype(np.uint8)


def e2m1_encode_fast(a):
    """Vectorised fp4 e2m1 encoder with the reference's boundaries (cuda/src/ops/subfp.cuh:44)."""
    x = np.ascontiguousarray(a, dtype=np.float32)
    bounds = np.array([0.4375, 0.875, 1.25000012, 1.75, 2.50000024, 3.5, 5.00000048], dtype=np.float32)
    c = np.searchsorted(bounds, np.abs(x), side="right").astype(np.uint8)
    c = np.where(np.isnan(x), np.uint8(0), c | (np.signbit(x).astype(np.uint8) << 3))
    return c.astype(np.uint8)


# ------------------------------------------------------------------ scalar (C) operators
def wqbmm(x, w, is_int4, scale, offset, bias, M, K, N, group=0):
    out = np.empty((M, N), dtype=np.float64)
    x, scale, offset, bias = _c(x, np.float32), _c(scale, np.float32), _c(offset, np.float32), _c(bias, np.float32)
    w = _c(w, np.uint8)
    C().oracle_wqbmm(_p(x), _p(w), int(is_int4), _p(scale), _p(offset), _p(bias), M, K, N, group, _p(out))
    return out


def qmm_acc(x, w, M, K, N):
    acc = np.empty((M, N), dtype=np.int32)
    x, w = _c(x, np.int8), _c(w, np.int8)
    C().oracle_qmm_acc(_p(x), _p(w), M, K, N, _p(acc))
    return acc


def qmm_epilogue(acc, scale, pertoken=None, bias=None):
    M, N = acc.shape
    out = np.empty((M, N), dtype=np.float32)
    acc, scale = _c(acc, np.int32), _c(scale, np.float32)
    pertoken, bias = _c(pertoken, np.float32), _c(bias, np.int32)
    C().oracle_qmm_epilogue(_p(acc), _p(scale), _p(pertoken), _p(bias), M, N, _p(out))
    return out


def mx_matmul(a, a_kind, sa, b, b_kind, sb, M, K, N):
    out = np.empty((M, N), dtype=np.float64)
    a, sa, b, sb = _c(a, np.uint8), _c(sa, np.uint8), _c(b, np.uint8), _c(sb, np.uint8)
    C().oracle_mx_matmul(_p(a), a_kind, _p(sa), _p(b), b_kind, _p(sb), M, K, N, _p(out))
    return out


def int4_pack(vals):
    vals = _c(vals, np.int8).reshape(-1)
    out = np.empty(vals.size // 2, dtype=np.uint8)
    C().oracle_int4_pack(_p(vals), out.size, _p(out))
    return out


def scale_swizzle_index(r, b, nb):
    return C().oracle_scale_swizzle_index(r, b, nb)


# ------------------------------------------------------------------ BLAS-backed versions
def wq_dequant_fast(w, is_int4, scale, offset, K, N, group=0):
    """(w - offset) * scale as float64 [K,N]."""
    g = group if group > 0 else K
    wv = (int4_unpack(w, K * N) if is_int4 else np.ascontiguousarray(w).view(np.int8).reshape(-1)[: K * N])
    wf = wv.reshape(K, N).astype(np.float64)
    sc = np.asarray(scale, dtype=np.float64).reshape(-1, N)
    rep = g if sc.shape[0] > 1 else K
    if offset is not None:
        wf -= np.repeat(np.asarray(offset, dtype=np.float64).reshape(-1, N), rep, axis=0)[:K]
    wf *= np.repeat(sc, rep, axis=0)[:K]
    return wf


def wqbmm_fast(x, w, is_int4, scale, offset, bias, M, K, N, group=0, weight_round=None):
    """weight_round = "bf16" | "f16": the reference's large-M form, which rounds each dequantised weight
    (computed in fp32) once to the activation type before the GEMM (cuda/src/ops/matmul.cu:733-747,
    790-795: deq_wq8 / deq_wq4 into a half buffer, then gemm_half)."""
    wf = wq_dequant_fast(w, is_int4, scale, offset, K, N, group)
    if weight_round is not None:
        g = group if group > 0 else K
        wv = (int4_unpack(w, K * N) if is_int4 else np.ascontiguousarray(w).view(np.int8).reshape(-1)[: K * N])
        w32 = wv.reshape(K, N).astype(np.float32)
        sc = np.asarray(scale, dtype=np.float32).reshape(-1, N)
        rep = g if sc.shape[0] > 1 else K
        if offset is not None:
            w32 = w32 - np.repeat(np.asarray(offset, dtype=np.float32).reshape(-1, N), rep, axis=0)[:K]
        w32 = w32 * np.repeat(sc, rep, axis=0)[:K]
        if weight_round == "bf16":
            wf = bf16_bits_to_f32(f32_to_bf16_bits(w32)).astype(np.float64)
        else:
            wf = f16_bits_to_f32(f32_to_f16_bits(w32)).astype(np.float64)
    out = np.asarray(x, dtype=np.float64).reshape(M, K) @ wf
    if bias is not None:
        out = out + np.asarray(bias, dtype=np.float64).reshape(1, N)
    return out


def qmm_acc_fast(x, w, M, K, N):
    """Exact int32 accumulators through float64 BLAS (every partial sum is < 2^53)."""
    assert K * 128 * 128 < 2 ** 53
    a = np.ascontiguousarray(x).view(np.int8).reshape(M, K).astype(np.float64)
    b = np.ascontiguousarray(w).view(np.int8).reshape(K, N).astype(np.float64)
    return np.rint(a @ b).astype(np.int64).astype(np.int32)


def qmm_epilogue_fast(acc, scale, pertoken=None, bias=None):
    a = acc.astype(np.int32)
    if bias is not None:
        a = a + np.asarray(bias, dtype=np.int32).reshape(1, -1)
    v = a.astype(np.float32) * np.asarray(scale, dtype=np.float32).reshape(1, -1)
    if pertoken is not None:
        v = v * np.asarray(pertoken, dtype=np.float32).reshape(-1, 1)
    return v.astype(np.float32)


def mx_dequant_fast(buf, kind, scales, rows, cols, scale_along_cols):
    """element * 2^(scale-127) as float64.  scale_along_cols: scales are [rows, cols/32] (operand A);
    otherwise [rows/32, cols] (operand B)."""
    v = mx_decode(buf, kind, rows, cols).astype(np.float64)
    s = np.ldexp(1.0, np.ascontiguousarray(scales, dtype=np.uint8).astype(np.int32) - 127)
    if scale_along_cols:
        v *= np.repeat(s.reshape(rows, cols // 32), 32, axis=1)
    else:
        v *= np.repeat(s.reshape(rows // 32, cols), 32, axis=0)
    return v


def mx_matmul_fast(a, a_kind, sa, b, b_kind, sb, M, K, N):
    return mx_dequant_fast(a, a_kind, sa, M, K, True) @ mx_dequant_fast(b, b_kind, sb, K, N, False)


def dynamic_quant(x):
    """Per-token dynamic int8 quantiser, restating cuda/src/ops/quant.cu:37-49 of the reference in fp32:
    scale = max|x| / 127 per row (1 for an all-zero row), q = clamp(rint(x * (1 / scale)), -128, 127)
    with the quotient formed as x * (1.f / scale) and rint rounding half to even.
    x: float array [..., D] (already widened to fp32 exactly).  Returns (int8 [..., D], float32 [...])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    amax = np.abs(x).max(axis=-1) if x.shape[-1] else np.zeros(x.shape[:-1], np.float32)
    scale = np.where(amax == 0, np.float32(1), amax / np.float32(127)).astype(np.float32)
    inv = (np.float32(1) / scale).astype(np.float32)
    q = np.rint((x * inv[..., None]).astype(np.float32))
    return np.clip(q, -128, 127).astype(np.int8), scale


def add_rmsnorm(x, residual, gamma, eps, kind):
    """Residual add + RMS norm, restating cuda/src/ops/norm_ext.cu:123-139: v = x + residual in fp32,
    residual_sum = T(v), y = T(float(residual_sum) * rsqrt(mean(v^2) + eps) * gamma) per row, with T the
    tensors' type (`kind`: "f32", "f16" or "bf16").  The mean is summed in float64 here (the device sums
    in fp32 in its own order), so y agrees to rounding, not bitwise.  Returns (y, residual_sum) as float32
    arrays holding T-representable values."""
    def rt(v):
        if kind == "f32":
            return v.astype(np.float32)
        if kind == "f16":
            return v.astype(np.float16).astype(np.float32)
        return bf16_bits_to_f32(f32_to_bf16_bits(v.astype(np.float32)))
    v = (np.asarray(x, np.float32) + np.asarray(residual, np.float32)).astype(np.float32)
    ysum = rt(v)
    ms = (v.astype(np.float64) ** 2).mean(axis=-1, keepdims=True)
    inv = (1.0 / np.sqrt(ms + eps)).astype(np.float32)
    g = np.float32(1) if gamma is None else np.asarray(gamma, np.float32)
    return rt((ysum * inv).astype(np.float32) * g), ysum


def swiglu_quant(x, dequant_scale=None):
    """SwiGLU fused with the per-token int8 quantiser, restating cuda/src/ops/glu_ext.cu:89-103 in fp32:
    x [..., 2D] = [a | b]; g = a / (1 + exp(-a)) * b; scale = max|g| / 127 per row (1 for a zero row);
    q = clamp(rint(g * (1 / scale)), -127, 127).  exp here is numpy's float32 exp, the device uses
    CUDA's expf (both within a couple of ulp of the true value), so a code may differ by one where
    g / scale falls next to a rounding boundary.  Returns (int8 [..., D], float32 [...])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if dequant_scale is not None:   # DequantSwigluQuant (cuda/src/ops/norm_ext.cu:1354-1369): x * dq[row] first
        x = (x * np.asarray(dequant_scale, np.float32)[..., None]).astype(np.float32)
    D = x.shape[-1] // 2
    a, b = x[..., :D], x[..., D:]
    with np.errstate(over="ignore"):
        g = ((a / (np.float32(1) + np.exp(-a, dtype=np.float32))).astype(np.float32) * b).astype(np.float32)
    amax = np.abs(g).max(axis=-1) if D else np.zeros(x.shape[:-1], np.float32)
    scale = np.where(amax > 0, amax / np.float32(127), np.float32(1)).astype(np.float32)
    inv = (np.float32(1) / scale).astype(np.float32)
    q = np.rint((g * inv[..., None]).astype(np.float32))
    return np.clip(q, -127, 127).astype(np.int8), scale


def dynamic_mx_quant(x, block):
    """Block-wise int8 quantiser with power-of-two scales, restating cuda/src/ops/quant.cu:380-389 in fp32:
    per block of `block` consecutive elements scale = 2^ceil(log2(max|x| / 127)) (1 for a zero block),
    q = clamp(rint(x * (1 / scale)), -128, 127).  Returns (int8 of x's shape, float32 [numel / block])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    b = x.reshape(-1, block)
    amax = np.abs(b).max(axis=1)
    with np.errstate(divide="ignore"):
        e = np.ceil(np.log2((amax / np.float32(127)).astype(np.float32)).astype(np.float32))
    scale = np.where(amax > 0, np.exp2(e).astype(np.float32), np.float32(1)).astype(np.float32)
    inv = (np.float32(1) / scale).astype(np.float32)
    q = np.clip(np.rint((b * inv[:, None]).astype(np.float32)), -128, 127).astype(np.int8)
    return q.reshape(x.shape), scale


# ------------------------------------------------------------------ PyTorch-CPU form (all host cores)
def wqbmm_torch(x, w, is_int4, scale, offset, bias, M, K, N, group=0):
    """The same weight-only matmul written with PyTorch CPU ops: dequantise in fp32, then torch.matmul
    (the shape of the reference's torch oracles, tools/torch_common.py:20-40 -- which hold no
    quant-matmul case of their own).  Multi-threaded; used as the timed CPU baseline."""
    import torch
    g = group if group > 0 else K
    wt = torch.from_numpy(np.ascontiguousarray(w).view(np.uint8).reshape(-1))
    if is_int4:
        lo = (wt & 0xF).to(torch.int8)
        hi = (wt >> 4).to(torch.int8)
        v = torch.stack([lo, hi], dim=1).reshape(-1)[: K * N]
        v = torch.where(v >= 8, v - 16, v)
    else:
        v = wt.view(torch.int8)[: K * N]
    wf = v.reshape(K, N).to(torch.float32)
    sc = torch.from_numpy(np.asarray(scale, dtype=np.float32)).reshape(-1, N)
    rep = g if sc.shape[0] > 1 else K
    if offset is not None:
        wf = wf - torch.from_numpy(np.asarray(offset, dtype=np.float32)).reshape(-1, N).repeat_interleave(rep, dim=0)[:K]
    wf = wf * sc.repeat_interleave(rep, dim=0)[:K]
    out = torch.from_numpy(np.asarray(x, dtype=np.float32)).reshape(M, K) @ wf
    if bias is not None:
        out = out + torch.from_numpy(np.asarray(bias, dtype=np.float32)).reshape(1, N)
    return out.numpy()
