"""ctypes view of the quantized-matmul library's C ABI, for the Python tests and the bench.

The product is `lib/libascendcl.so` (C++/CUDA, sm_100a).  This module only loads it and wraps the
two-phase aclnn call protocol around torch device buffers; it contains no compute and no fallback:
if the library is missing, `load()` raises.
"""
import ctypes
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libascendcl.so")
HCCL_PATH = os.path.join(_HERE, "lib", "libhccl.so")

# aclDataType values (include/acl/acl.h)
ACL_FLOAT, ACL_FLOAT16, ACL_INT8, ACL_INT32, ACL_UINT8 = 0, 1, 2, 3, 4
ACL_INT64, ACL_BF16, ACL_INT4 = 9, 27, 29
ACL_FLOAT8_E5M2, ACL_FLOAT8_E4M3FN, ACL_FLOAT8_E8M0, ACL_FLOAT4_E2M1 = 35, 36, 37, 40
ACL_FORMAT_ND = 2
ACL_FORMAT_FRACTAL_NZ = 29

ACLNN_SUCCESS = 0
ACLNN_ERR_PARAM_NULLPTR = 161001
ACLNN_ERR_PARAM_INVALID = 161002
ACLNN_ERR_RUNTIME_ERROR = 361001


def build(verbose=False):
    """Compile the library in-tree (nvcc, sm_100a)."""
    cmd = ["make", "-C", _HERE, "-j8"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or r.returncode != 0:
        print(r.stdout)
    if r.returncode != 0:
        raise RuntimeError("building libascendcl.so failed")


_lib = None
_libs = {}


def load(path=None):
    """The loaded C library (default: this package's libascendcl.so).  Raises if it is missing.
    Another library exporting the same C ABI can be loaded by path; `use_library` switches to it."""
    global _lib
    if path is None and _lib is not None:
        return _lib
    if path is None:
        path = LIB_PATH
    if path not in _libs:
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: run __graft_entry__.build() (there is no fallback path)")
        lib = ctypes.CDLL(path)
        lib.aclCreateTensor.restype = ctypes.c_void_p
        lib.aclCreateTensor.argtypes = [ctypes.POINTER(ctypes.c_int64), ctypes.c_uint64, ctypes.c_int,
                                        ctypes.POINTER(ctypes.c_int64), ctypes.c_int64, ctypes.c_int,
                                        ctypes.POINTER(ctypes.c_int64), ctypes.c_uint64, ctypes.c_void_p]
        lib.aclDestroyTensor.argtypes = [ctypes.c_void_p]
        lib.aclCreateIntArray.restype = ctypes.c_void_p
        lib.aclCreateIntArray.argtypes = [ctypes.POINTER(ctypes.c_int64), ctypes.c_uint64]
        lib.aclDestroyIntArray.argtypes = [ctypes.c_void_p]
        _libs[path] = lib
    if _lib is None and path == LIB_PATH:
        _lib = _libs[path]
    return _libs[path]


class use_library:
    """Context manager: route AclTensor/call through another library with the same C ABI (the tests
    use it to drive the reference's own backend when that has been built)."""

    def __init__(self, path):
        self.lib = load(path)

    def __enter__(self):
        global _lib
        load()
        self.prev, _lib = _lib, self.lib
        return self.lib

    def __exit__(self, *a):
        global _lib
        _lib = self.prev


def torch_acl_dtype(t):
    import torch
    return {torch.float32: ACL_FLOAT, torch.float16: ACL_FLOAT16, torch.bfloat16: ACL_BF16, torch.int8: ACL_INT8,
            torch.uint8: ACL_UINT8, torch.int32: ACL_INT32, torch.int64: ACL_INT64}[t.dtype]


class AclTensor:
    """An aclTensor handle over a torch tensor's storage (kept alive by this object)."""

    def __init__(self, t, dtype=None, shape=None, fmt=ACL_FORMAT_ND, storage=None):
        self.t = t
        self.dtype = torch_acl_dtype(t) if dtype is None else dtype
        dims = list(t.shape) if shape is None else list(shape)
        arr = (ctypes.c_int64 * max(1, len(dims)))(*dims)
        sdims = dims if storage is None else list(storage)
        sarr = (ctypes.c_int64 * max(1, len(sdims)))(*sdims)
        self.lib = load()
        self.h = self.lib.aclCreateTensor(arr, len(dims), self.dtype, None, 0, fmt, sarr, len(sdims),
                                        ctypes.c_void_p(t.data_ptr()))
        if not self.h:
            raise RuntimeError("aclCreateTensor failed")

    def __del__(self):
        try:
            if self.h:
                self.lib.aclDestroyTensor(ctypes.c_void_p(self.h))
                self.h = None
        except Exception:
            pass


def _h(x):
    return ctypes.c_void_p(x.h) if isinstance(x, AclTensor) else (None if x is None else x)


class Workspace:
    """A reusable device scratch buffer (grown on demand, never shrunk)."""

    def __init__(self):
        self.buf = None

    def get(self, nbytes, device):
        import torch
        if nbytes == 0:
            return None, 0
        if self.buf is None or self.buf.numel() < nbytes or self.buf.device != device:
            self.buf = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
        return self.buf, self.buf.numel()


_default_ws = Workspace()


def call(name, *args, stream=None, workspace=None, device=None, return_status=False):
    """Run the two-phase operator `name` with the phase-1 argument list `args` (AclTensor, None or
    ctypes scalars) on `stream` (default: torch's current stream)."""
    import torch
    lib = load()
    ws_size = ctypes.c_uint64(0)
    ex = ctypes.c_void_p(0)
    cargs = [_h(a) for a in args] + [ctypes.byref(ws_size), ctypes.byref(ex)]
    st = getattr(lib, name + "GetWorkspaceSize")(*cargs)
    if st != ACLNN_SUCCESS:
        if return_status:
            return st
        raise RuntimeError(f"{name}GetWorkspaceSize -> {st}")
    if device is None:
        device = next(a.t.device for a in args if isinstance(a, AclTensor))
    ws = workspace if workspace is not None else _default_ws
    buf, nbytes = ws.get(ws_size.value, device)
    s = torch.cuda.current_stream(device).cuda_stream if stream is None else stream
    st = getattr(lib, name)(ctypes.c_void_p(buf.data_ptr() if buf is not None else 0), ctypes.c_uint64(nbytes), ex,
                            ctypes.c_void_p(s))
    if return_status:
        return st
    if st != ACLNN_SUCCESS:
        raise RuntimeError(f"{name} -> {st}")
    return ws_size.value


# ---------------------------------------------------------------- operator wrappers (device tensors in, device tensor out)
def pack_weight_nz(w, K, N):
    """One-time re-layout of packed int4 weights [K,N] (bytes, two per byte) into the tile-packed on-device
    format: aclnnCalculateMatmulWeightSizeV2 for the size, aclnnTransMatmulWeight into an
    ACL_FORMAT_FRACTAL_NZ tensor.  Returns the packed buffer (uint8)."""
    import torch
    lib = load()
    shp = (ctypes.c_int64 * 2)(K, N)
    ia = ctypes.c_void_p(lib.aclCreateIntArray(shp, 2))
    n_out = torch.zeros(1, dtype=torch.int64, device=w.device)
    call("aclnnCalculateMatmulWeightSizeV2", ia, ctypes.c_int64(ACL_INT4), AclTensor(n_out), device=w.device)
    lib.aclDestroyIntArray(ia)
    elems = int(n_out.item())
    packed = torch.empty(elems // 2, dtype=torch.uint8, device=w.device)
    call("aclnnTransMatmulWeight", AclTensor(w, ACL_INT4, (K, N)),
         AclTensor(packed, ACL_INT4, (K, N), fmt=ACL_FORMAT_FRACTAL_NZ, storage=(elems,)))
    return packed


def weight_quant_matmul(x, w, scale, offset=None, bias=None, int4=False, group=0, name="aclnnWeightQuantBatchMatmulV2Ex",
                        out=None, nz=False, **kw):
    """x [M,K] f16/bf16/f32; w int8 [K,N] or packed int4 bytes [K*N/2]; scale/offset [N] or [G,N].
    nz: w is the tile-packed buffer pack_weight_nz returned (int4 only)."""
    import torch
    M, K = x.shape
    N = scale.shape[-1]
    if out is None:
        out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    if nz:
        tw = AclTensor(w, ACL_INT4, (K, N), fmt=ACL_FORMAT_FRACTAL_NZ, storage=(w.numel() * 2,))
    else:
        tw = AclTensor(w, ACL_INT4 if int4 else ACL_INT8, (K, N))
    targs = [AclTensor(x), tw, AclTensor(scale), AclTensor(offset) if offset is not None else None]
    if name.endswith("Ex"):
        targs += [AclTensor(bias) if bias is not None else None, ctypes.c_int64(group)]
    elif bias is not None:
        raise ValueError("bias needs the Ex entry point")
    call(name, *targs, AclTensor(out), **kw)
    return out


def quant_matmul(x, w, scale, pertoken=None, bias=None, out_dtype=None, name="aclnnQuantMatmulV4Ex", out=None, **kw):
    """x int8 [M,K], w int8 [K,N]; scale [N] or None (raw int32 accumulators)."""
    import torch
    M, N = x.shape[-2], (w.shape[-2] if name == "aclnnTransposeQuantBatchMatMul" else w.shape[-1])
    if out is None:
        odt = torch.int32 if scale is None else (out_dtype or torch.bfloat16)
        out = torch.empty(tuple(x.shape[:-2]) + (M, N), dtype=odt, device=x.device)
    if name.endswith("Ex"):
        targs = [AclTensor(x), AclTensor(w), AclTensor(scale) if scale is not None else None, None,
                 AclTensor(pertoken) if pertoken is not None else None, AclTensor(bias) if bias is not None else None]
    else:
        targs = [AclTensor(x), AclTensor(w), AclTensor(scale)]
    call(name, *targs, AclTensor(out), **kw)
    return out


def widen_fp4_weight(b, K, N):
    """One-time re-layout of an fp4 (e2m1, two per byte) weight [K,N] of a block-scaled matmul into its on-device
    format, one fp8 e4m3 byte per element: aclnnCalculateMatmulWeightSizeV2 for the size, aclnnTransMatmulWeight
    into an ACL_FORMAT_FRACTAL_NZ tensor.  Returns the widened buffer (uint8, K * N bytes)."""
    import torch
    lib = load()
    shp = (ctypes.c_int64 * 2)(K, N)
    ia = ctypes.c_void_p(lib.aclCreateIntArray(shp, 2))
    n_out = torch.zeros(1, dtype=torch.int64, device=b.device)
    call("aclnnCalculateMatmulWeightSizeV2", ia, ctypes.c_int64(ACL_FLOAT4_E2M1), AclTensor(n_out), device=b.device)
    lib.aclDestroyIntArray(ia)
    elems = int(n_out.item())
    wide = torch.empty(elems // 2, dtype=torch.uint8, device=b.device)
    call("aclnnTransMatmulWeight", AclTensor(b, ACL_FLOAT4_E2M1, (K, N)),
         AclTensor(wide, ACL_FLOAT4_E2M1, (K, N), fmt=ACL_FORMAT_FRACTAL_NZ, storage=(elems,)))
    return wide


def mx_matmul(a, a_kind, sa, b, b_kind, sb, M, K, N, out_dtype=None, name="aclnnMatmulMxFp8", b_widened=False, **kw):
    """a/b: uint8 buffers of MX elements (fp8: one byte each; fp4: two per byte); sa [M,K/32], sb [K/32,N] e8m0.
    b_widened: b is the buffer widen_fp4_weight returned."""
    import torch
    out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=a.device)
    tb = (AclTensor(b, b_kind, (K, N), fmt=ACL_FORMAT_FRACTAL_NZ, storage=(b.numel() * 2,)) if b_widened
          else AclTensor(b, b_kind, (K, N)))
    call(name, AclTensor(a, a_kind, (M, K)), AclTensor(sa, ACL_FLOAT8_E8M0, (M, K // 32)),
         tb, AclTensor(sb, ACL_FLOAT8_E8M0, (K // 32, N)), AclTensor(out), **kw)
    return out


def dynamic_quant(x, name="aclnnDynamicQuant", **kw):
    """x [..., D] f32/f16/bf16 -> (int8 [..., D], fp32 per-row scales [...])."""
    import torch
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    scale = torch.empty(x.shape[:-1] if x.dim() > 1 else (1,), dtype=torch.float32, device=x.device)
    call(name, AclTensor(x), AclTensor(q), AclTensor(scale), **kw)
    return q, scale



def swiglu_quant(x, name="aclnnSwiGluQuant", dequant_scale=None, **kw):
    """x [..., 2D] f32/f16/bf16 -> (int8 [..., D] of silu(x[..., :D]) * x[..., D:], fp32 per-row scales [...]).
    With the aclnnDequantSwigluQuant names, `dequant_scale` (fp32 per row, or None) multiplies x first."""
    import torch
    D = x.shape[-1] // 2
    q = torch.empty(tuple(x.shape[:-1]) + (D,), dtype=torch.int8, device=x.device)
    scale = torch.empty(x.shape[:-1] if x.dim() > 1 else (1,), dtype=torch.float32, device=x.device)
    if "Dequant" in name:
        call(name, AclTensor(x), AclTensor(dequant_scale) if dequant_scale is not None else None, AclTensor(q), AclTensor(scale), **kw)
    else:
        call(name, AclTensor(x), AclTensor(q), AclTensor(scale), **kw)
    return q, scale

def dynamic_mx_quant(x, block, name="aclnnDynamicMxQuant", **kw):
    """x (numel a multiple of block) f32/f16/bf16 -> (int8 of x's shape, fp32 power-of-two scale per block)."""
    import torch
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    scale = torch.empty((x.numel() // block,), dtype=torch.float32, device=x.device)
    call(name, AclTensor(x), ctypes.c_int64(block), AclTensor(q), AclTensor(scale), **kw)
    return q, scale


def cast(src, src_kind, dst_kind, n, **kw):
    """aclnnCast over flat buffers; returns the destination buffer (uint8 for fp8/fp4 kinds)."""
    import torch
    td = {ACL_FLOAT: torch.float32, ACL_FLOAT16: torch.float16, ACL_BF16: torch.bfloat16, ACL_INT8: torch.int8,
          ACL_INT32: torch.int32}
    if dst_kind == ACL_FLOAT4_E2M1:
        dst = torch.empty((n + 1) // 2, dtype=torch.uint8, device=src.device)
    elif dst_kind in td:
        dst = torch.empty(n, dtype=td[dst_kind], device=src.device)
    else:
        dst = torch.empty(n, dtype=torch.uint8, device=src.device)
    call("aclnnCast", AclTensor(src, src_kind, (n,)), ctypes.c_int(dst_kind), AclTensor(dst, dst_kind, (n,)), **kw)
    return dst
