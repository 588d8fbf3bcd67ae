"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the headers declare,
and phase 1 (host-only) validates arguments with the reference's status codes.  No kernel runs."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include")


def declared_symbols():
    names = set()
    qm = open(os.path.join(INC, "aclnnop", "aclnn_quant_matmul.h")).read()
    body = qm.split('extern "C"', 1)[1]
    for m in re.finditer(r"^B200_ACLNN_(?:WQBMM|QMM|MX|QMM_GROUPED|QMM_COMM|QPARAM|DYNQUANT|DEQSWIGLUQUANT|MXQUANT)\((\w+)\)", body, re.M):
        names.update({m.group(1), m.group(1) + "GetWorkspaceSize"})
    for m in re.finditer(r"^B200_ACLNN_RUN\((\w+)\)", body, re.M):
        names.add(m.group(1))
    for m in re.finditer(r"aclnnStatus (\w+GetWorkspaceSize)\(", body):
        if "##" not in m.group(0) and m.group(1) != "GetWorkspaceSize":
            names.add(m.group(1))
    for m in re.finditer(r"^ACL_FUNC_VISIBILITY [\w \*]*?(\w+)\(", body, re.M):   # the library's own entry points
        names.add(m.group(1))
    for h in ("acl/acl.h", "aclnn/acl_meta.h"):
        for m in re.finditer(r"^ACL_FUNC_VISIBILITY\s+[\w ]+?\*?\s*\*?(\w+)\(", open(os.path.join(INC, h)).read(), re.M):
            names.add(m.group(1))
    return sorted(names)


def test_library_exports_every_declared_symbol(pkg):
    lib = ctypes.CDLL(pkg.LIB_PATH)
    names = declared_symbols()
    assert len(names) > 80
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_c_client_library_loads(pkg):
    """The plain C client of the ABI (the benchmark's end-to-end loop) links against the library
    and exports its one entry point."""
    path = os.path.join(os.path.dirname(pkg.LIB_PATH), "libqmm_client.so")
    assert os.path.exists(path), "run __graft_entry__.build()"
    ctypes.CDLL(pkg.LIB_PATH)
    client = ctypes.CDLL(path)
    assert hasattr(client, "qmmClientWeightQuantPass") and hasattr(client, "qmmClientWeightQuantStep")


def test_hccl_library_exports(pkg):
    if not os.path.exists(pkg.HCCL_PATH):
        pytest.skip("libhccl.so not built (nccl.h absent)")
    try:
        lib = ctypes.CDLL(pkg.HCCL_PATH)
    except OSError as e:
        pytest.skip(f"libhccl.so not loadable here: {e}")
    for m in re.finditer(r"HcclResult (\w+)\(", open(os.path.join(INC, "hccl", "hccl.h")).read()):
        assert hasattr(lib, m.group(1)), m.group(1)


class FakeTensor:
    """aclTensor over a made-up device address: phase 1 never dereferences data pointers."""

    def __init__(self, pkg, dims, dtype, addr=0x7F0000000000):
        arr = (ctypes.c_int64 * max(1, len(dims)))(*dims)
        self.lib = pkg.load()
        self.h = self.lib.aclCreateTensor(arr, len(dims), dtype, None, 0, pkg.ACL_FORMAT_ND, arr, len(dims),
                                          ctypes.c_void_p(addr))
        assert self.h

    def __del__(self):
        self.lib.aclDestroyTensor(ctypes.c_void_p(self.h))


def phase1(pkg, name, *args):
    lib = pkg.load()
    ws, ex = ctypes.c_uint64(123), ctypes.c_void_p(0)
    cargs = [ctypes.c_void_p(a.h) if isinstance(a, FakeTensor) else a for a in args]
    st = getattr(lib, name + "GetWorkspaceSize")(*cargs, ctypes.byref(ws), ctypes.byref(ex))
    if st == 0:
        lib.aclDestroyAclOpExecutor(ex)
    return st, ws.value


def test_hccl_library_exports_allreduce_matmuls(pkg):
    path = os.path.join(os.path.dirname(pkg.LIB_PATH), "libhccl.so")
    if not os.path.exists(path):
        pytest.skip("libhccl.so not built (nccl.h absent)")
    ctypes.CDLL(pkg.LIB_PATH)
    try:
        lib = ctypes.CDLL(path)
    except OSError as e:
        pytest.skip(f"libhccl.so not loadable here: {e}")
    hdr = open(os.path.join(INC, "aclnnop", "aclnn_quant_matmul_mc2.h")).read()
    names = set(re.findall(r"^B200_ACLNN_QMM_ALLREDUCE\((\w+)\)", hdr, re.M)) | {"aclnnWeightQuantMatmulAllReduce",
                                                                                     "aclnnQuantMatmulAllReduceAddRmsNorm"}
    assert len(names) == 6
    names.add("aclnnB200WeightQuantMatmulAllGather")
    for n in names:
        assert hasattr(lib, n) and hasattr(lib, n + "GetWorkspaceSize"), n
    for n in ("aclnnB200FusedGatherCount", "aclnnB200FusedAllReduceCount", "HcclB200P2pStatus", "HcclB200TestReceiverTimeout"):
        assert hasattr(lib, n), n


def test_wqbmm_phase1_validation(pkg):
    T = lambda d, t: FakeTensor(pkg, d, t)
    M, K, N = 4, 256, 64
    x, w, sc, off, out = T([M, K], pkg.ACL_FLOAT16), T([K, N], pkg.ACL_INT8), T([N], pkg.ACL_FLOAT16), \
        T([N], pkg.ACL_FLOAT16), T([M, N], pkg.ACL_FLOAT16)
    for name in ("aclnnWeightQuantBatchMatmul", "aclnnWeightQuantBatchMatmulV2", "aclnnWeightQuantBatchMatmulV3",
                 "aclnnWeightQuantBatchMatmulNz"):
        assert phase1(pkg, name, x, w, sc, off, out)[0] == 0
        assert phase1(pkg, name, x, w, sc, None, out)[0] == 0          # offset is optional
        assert phase1(pkg, name, None, w, sc, off, out)[0] == 161001
        assert phase1(pkg, name, x, w, None, off, out)[0] == 161001
    # wrong dtypes / shapes -> 161002 (reference: cuda/src/ops/matmul.cu:761-767)
    assert phase1(pkg, "aclnnWeightQuantBatchMatmul", x, T([K, N], pkg.ACL_FLOAT16), sc, off, out)[0] == 161002
    assert phase1(pkg, "aclnnWeightQuantBatchMatmul", x, T([K + 1, N], pkg.ACL_INT8), sc, off, out)[0] == 161002
    assert phase1(pkg, "aclnnWeightQuantBatchMatmul", x, w, T([N + 1], pkg.ACL_FLOAT16), None, out)[0] == 161002
    assert phase1(pkg, "aclnnWeightQuantBatchMatmul", x, w, sc, off, T([M, N], pkg.ACL_FLOAT))[0] == 161002
    # widened acceptance: bf16, group-wise [G,N] scales, int4, bias through the Ex name
    xb, ob = T([M, K], pkg.ACL_BF16), T([M, N], pkg.ACL_BF16)
    sg, og, bias = T([2, N], pkg.ACL_BF16), T([2, N], pkg.ACL_BF16), T([N], pkg.ACL_BF16)
    w4 = T([K, N], pkg.ACL_INT4)
    assert phase1(pkg, "aclnnWeightQuantBatchMatmulV2", xb, w4, sg, og, ob)[0] == 0
    i64 = ctypes.c_int64
    assert phase1(pkg, "aclnnWeightQuantBatchMatmulV2Ex", xb, w4, sg, og, bias, i64(128), ob)[0] == 0
    assert phase1(pkg, "aclnnWeightQuantBatchMatmulV2Ex", xb, w4, sg, og, bias, i64(0), ob)[0] == 0
    assert phase1(pkg, "aclnnWeightQuantBatchMatmulV2Ex", xb, w4, sg, og, bias, i64(64), ob)[0] == 161002
    assert phase1(pkg, "aclnnWeightQuantBatchMatmulV2Ex", xb, w4, T([3, N], pkg.ACL_BF16), None, None, i64(0), ob)[0] == 161002
    assert phase1(pkg, "aclnnWeightQuantBatchMatmulV2Ex", xb, w4, sg, og, T([N], pkg.ACL_FLOAT16), i64(0), ob)[0] == 161002


def test_qmm_phase1_validation(pkg):
    T = lambda d, t: FakeTensor(pkg, d, t)
    M, K, N = 8, 64, 32
    x, w, sc, out = T([M, K], pkg.ACL_INT8), T([K, N], pkg.ACL_INT8), T([N], pkg.ACL_FLOAT16), T([M, N], pkg.ACL_FLOAT16)
    names = ["aclnnQuantMatmul", "aclnnQuantMatmulV2", "aclnnQuantMatmulV3", "aclnnQuantMatmulV4", "aclnnQuantMatmulV5",
             "aclnnQuantMatmulDequant", "aclnnQuantMatmulWeightNz", "aclnnFusedQuantMatmul", "aclnnFusedQuantMatmulWeightNz",
             "aclnnMatmulCompressDequant", "aclnnSparse4to2QuantMatmulWeightNz", "aclnnDualLevelQuantMatmulWeightNz",
             "aclnnQuantBatchMatmulInplaceAdd"]
    for name in names:
        assert phase1(pkg, name, x, w, sc, out)[0] == 0, name
        assert phase1(pkg, name, x, w, None, out)[0] == 161001, name
        assert phase1(pkg, name, x, T([K, N], pkg.ACL_FLOAT16), sc, out)[0] == 161002, name
    assert phase1(pkg, "aclnnTransposeQuantBatchMatMul", x, T([N, K], pkg.ACL_INT8), sc, out)[0] == 0
    assert phase1(pkg, "aclnnTransposeQuantBatchMatMul", x, T([N, K + 1], pkg.ACL_INT8), sc, out)[0] == 161002
    B = 3
    assert phase1(pkg, "aclnnBatchMatmulQuant", T([B, M, K], pkg.ACL_INT8), T([B, K, N], pkg.ACL_INT8),
                  T([N], pkg.ACL_FLOAT), T([B, M, N], pkg.ACL_FLOAT))[0] == 0
    # extended form
    pt, bias, ob = T([M], pkg.ACL_FLOAT), T([N], pkg.ACL_INT32), T([M, N], pkg.ACL_BF16)
    scf = T([N], pkg.ACL_FLOAT)
    assert phase1(pkg, "aclnnQuantMatmulV4Ex", x, w, scf, None, pt, bias, ob)[0] == 0
    assert phase1(pkg, "aclnnQuantMatmulV4Ex", x, w, scf, None, T([M + 1], pkg.ACL_FLOAT), bias, ob)[0] == 161002
    assert phase1(pkg, "aclnnQuantMatmulV4Ex", x, w, scf, None, pt, T([N], pkg.ACL_FLOAT), ob)[0] == 161002
    assert phase1(pkg, "aclnnQuantMatmulV4Ex", x, w, None, None, None, None, T([M, N], pkg.ACL_INT32))[0] == 0
    assert phase1(pkg, "aclnnQuantMatmulV4Ex", x, w, None, None, None, None, ob)[0] == 161001


def test_mx_phase1_validation(pkg):
    T = lambda d, t: FakeTensor(pkg, d, t)
    M, K, N = 16, 64, 32
    a8, b8, b4 = T([M, K], pkg.ACL_FLOAT8_E4M3FN), T([K, N], pkg.ACL_FLOAT8_E4M3FN), T([K, N], pkg.ACL_FLOAT4_E2M1)
    sa, sb = T([M, K // 32], pkg.ACL_FLOAT8_E8M0), T([K // 32, N], pkg.ACL_FLOAT8_E8M0)
    for name in ("aclnnMatmulMxFp8", "aclnnMatmulMxFp8Hw", "aclnnMatmulMxFp4", "aclnnMatmulMxFp4Hw"):
        for out_t in (pkg.ACL_FLOAT, pkg.ACL_FLOAT16, pkg.ACL_BF16):
            assert phase1(pkg, name, a8, sa, b8, sb, T([M, N], out_t))[0] == 0
        assert phase1(pkg, name, a8, sa, b4, sb, T([M, N], pkg.ACL_BF16))[0] == 0     # mixed fp8 x fp4
        assert phase1(pkg, name, a8, None, b8, sb, T([M, N], pkg.ACL_FLOAT))[0] == 161001
        assert phase1(pkg, name, a8, T([M, 1], pkg.ACL_FLOAT8_E8M0), b8, sb, T([M, N], pkg.ACL_FLOAT))[0] == 161002
        assert phase1(pkg, name, a8, T([M, K // 32], pkg.ACL_UINT8), b8, sb, T([M, N], pkg.ACL_FLOAT))[0] == 161002
    # K must be a multiple of 32 (reference: cuda/src/ops/matmul.cu:445)
    assert phase1(pkg, "aclnnMatmulMxFp8", T([M, 48], pkg.ACL_FLOAT8_E4M3FN), T([M, 1], pkg.ACL_FLOAT8_E8M0),
                  T([48, N], pkg.ACL_FLOAT8_E4M3FN), T([1, N], pkg.ACL_FLOAT8_E8M0), T([M, N], pkg.ACL_FLOAT))[0] == 161002


def test_workspace_is_reported_and_checked(pkg):
    """Phase 2 rejects an undersized workspace before launching anything (host-side check)."""
    T = lambda d, t: FakeTensor(pkg, d, t)
    lib = pkg.load()
    M, K, N = 1, 4096, 4096
    x, w = T([M, K], pkg.ACL_BF16), T([K, N], pkg.ACL_INT4)
    sg, out = T([32, N], pkg.ACL_BF16), T([M, N], pkg.ACL_BF16)
    ws, ex = ctypes.c_uint64(0), ctypes.c_void_p(0)
    st = lib.aclnnWeightQuantBatchMatmulV2GetWorkspaceSize(ctypes.c_void_p(x.h), ctypes.c_void_p(w.h), ctypes.c_void_p(sg.h),
                                                           None, ctypes.c_void_p(out.h), ctypes.byref(ws), ctypes.byref(ex))
    assert st == 0
    if ws.value > 0:
        st = lib.aclnnWeightQuantBatchMatmulV2(None, ctypes.c_uint64(0), ex, None)
        assert st == 161002
    else:
        lib.aclDestroyAclOpExecutor(ex)


def test_meta_objects_round_trip(pkg):
    lib = pkg.load()
    t = FakeTensor(pkg, [3, 5], pkg.ACL_BF16, addr=0x1000)
    dims, num, dt, addr = ctypes.POINTER(ctypes.c_int64)(), ctypes.c_uint64(0), ctypes.c_int(0), ctypes.c_void_p(0)
    assert lib.aclGetViewShape(ctypes.c_void_p(t.h), ctypes.byref(dims), ctypes.byref(num)) == 0
    assert num.value == 2 and dims[0] == 3 and dims[1] == 5
    assert lib.aclGetDataType(ctypes.c_void_p(t.h), ctypes.byref(dt)) == 0 and dt.value == pkg.ACL_BF16
    assert lib.aclGetRawTensorAddr(ctypes.c_void_p(t.h), ctypes.byref(addr)) == 0 and addr.value == 0x1000
    assert lib.aclGetViewShape(None, ctypes.byref(dims), ctypes.byref(num)) == 161001
    lib.aclDataTypeSize.restype = ctypes.c_size_t
    assert lib.aclDataTypeSize(pkg.ACL_BF16) == 2 and lib.aclDataTypeSize(pkg.ACL_INT4) == 1


def test_gathering_matmul_phase1(pkg):
    """Phase 1 of the column-shard matmul with the fused gather, without a communicator (one rank: gathered is [1][M][N]):
    argument checks, a workspace that serves both forms of the decode kernel, and a plan that can be abandoned."""
    if not os.path.exists(pkg.HCCL_PATH):
        pytest.skip("libhccl.so not built (nccl.h absent)")
    try:
        hccl = ctypes.CDLL(pkg.HCCL_PATH)
    except OSError as e:
        pytest.skip(f"libhccl.so not loadable here: {e}")
    lib = pkg.load()
    M, K, N = 2, 1024, 512
    x, w = FakeTensor(pkg, (M, K), pkg.ACL_BF16), FakeTensor(pkg, (K, N), pkg.ACL_INT4)
    sc, g = FakeTensor(pkg, (K // 128, N), pkg.ACL_BF16), FakeTensor(pkg, (1, M, N), pkg.ACL_BF16)
    fn = hccl.aclnnB200WeightQuantMatmulAllGatherGetWorkspaceSize

    def plan(xt, wt, st, gt):
        ws, ex = ctypes.c_uint64(0), ctypes.c_void_p(0)
        r = fn(ctypes.c_void_p(xt.h) if xt else None, ctypes.c_void_p(wt.h), ctypes.c_void_p(st.h), None, None, ctypes.c_int64(128), None,
               ctypes.c_void_p(gt.h) if gt else None, ctypes.byref(ws), ctypes.byref(ex))
        return r, ws.value, ex
    r, need, ex = plan(x, w, sc, g)
    assert r == 0 and ex.value and need > 0
    plain = phase1(pkg, "aclnnWeightQuantBatchMatmulV2Ex", x, w, sc, None, None, ctypes.c_int64(128), FakeTensor(pkg, (M, N), pkg.ACL_BF16))
    assert plain[0] == 0 and need >= plain[1]
    assert lib.aclDestroyAclOpExecutor(ex) == 0
    assert plan(None, w, sc, g)[0] == 161001 and plan(x, w, sc, None)[0] == 161001
    assert plan(x, w, sc, FakeTensor(pkg, (M, N), pkg.ACL_BF16))[0] == 161002            # gathered must be [ranks][M][N/ranks]
    assert plan(x, w, sc, FakeTensor(pkg, (2, M, N), pkg.ACL_BF16))[0] == 161002         # two slots, one rank
    assert plan(x, w, sc, FakeTensor(pkg, (1, M, N), pkg.ACL_FLOAT))[0] == 161002        # 16-bit outputs only


def test_abandoned_collective_plan_is_released(pkg):
    """A caller may give up after phase 1.  The plans of the all-reduce matmuls (libhccl.so) are real
    executors that own their state, so aclDestroyAclOpExecutor releases them like any other plan, and a
    plain execute entry refuses them instead of reading them as a matmul plan."""
    if not os.path.exists(pkg.HCCL_PATH):
        pytest.skip("libhccl.so not built (nccl.h absent)")
    try:
        hccl = ctypes.CDLL(pkg.HCCL_PATH)
    except OSError as e:
        pytest.skip(f"libhccl.so not loadable here: {e}")
    lib = pkg.load()
    x, w = FakeTensor(pkg, (8, 64), pkg.ACL_INT8), FakeTensor(pkg, (64, 32), pkg.ACL_INT8)
    sc, out = FakeTensor(pkg, (32,), pkg.ACL_FLOAT16), FakeTensor(pkg, (8, 32), pkg.ACL_FLOAT16)
    lib.aclnnB200WrapperPayload.restype = ctypes.c_void_p
    lib.aclnnB200WrapperPayload.argtypes = [ctypes.c_void_p, ctypes.c_int]
    for _ in range(3):
        ws, ex = ctypes.c_uint64(0), ctypes.c_void_p(0)
        st = hccl.aclnnQuantMatmulAllReduceGetWorkspaceSize(ctypes.c_void_p(x.h), ctypes.c_void_p(w.h), ctypes.c_void_p(sc.h), None,
                                                            ctypes.c_void_p(out.h), ctypes.byref(ws), ctypes.byref(ex))
        assert st == 0 and ex.value
        assert lib.aclnnB200WrapperPayload(ex, 0)            # it is a wrapper plan ...
        assert lib.aclDestroyAclOpExecutor(ex) == 0          # ... and destroying it releases the inner plan too
    ws, ex = ctypes.c_uint64(0), ctypes.c_void_p(0)
    assert hccl.aclnnQuantMatmulAllReduceGetWorkspaceSize(ctypes.c_void_p(x.h), ctypes.c_void_p(w.h), ctypes.c_void_p(sc.h), None,
                                                          ctypes.c_void_p(out.h), ctypes.byref(ws), ctypes.byref(ex)) == 0
    # handed to a non-collective execute entry: refused (and consumed) before anything is launched
    assert lib.aclnnQuantMatmul(None, ctypes.c_uint64(0), ex, None) == 161002
    # an ordinary plan is not a wrapper
    ws, ex = ctypes.c_uint64(0), ctypes.c_void_p(0)
    assert lib.aclnnQuantMatmulGetWorkspaceSize(ctypes.c_void_p(x.h), ctypes.c_void_p(w.h), ctypes.c_void_p(sc.h),
                                                ctypes.c_void_p(out.h), ctypes.byref(ws), ctypes.byref(ex)) == 0
    assert not lib.aclnnB200WrapperPayload(ex, 0)
    assert lib.aclDestroyAclOpExecutor(ex) == 0


def test_phase1_does_not_depend_on_data_pointers(pkg):
    """Workspace size and kernel choice come from presence, types and shapes only: the same call with
    null, odd and aligned data pointers reports the same workspace."""
    lib = pkg.load()
    sizes = set()
    for addr in (0, 0x7F0000000002, 0x7F0000000100):
        x, w = FakeTensor(pkg, (40, 1024), pkg.ACL_BF16, addr), FakeTensor(pkg, (1024, 512), pkg.ACL_INT4, addr)
        sc, of = FakeTensor(pkg, (8, 512), pkg.ACL_BF16, addr), FakeTensor(pkg, (8, 512), pkg.ACL_BF16, addr)
        out = FakeTensor(pkg, (40, 512), pkg.ACL_BF16, addr)
        ws, ex = ctypes.c_uint64(0), ctypes.c_void_p(0)
        assert lib.aclnnWeightQuantBatchMatmulV2GetWorkspaceSize(ctypes.c_void_p(x.h), ctypes.c_void_p(w.h), ctypes.c_void_p(sc.h),
                                                                 ctypes.c_void_p(of.h), ctypes.c_void_p(out.h), ctypes.byref(ws),
                                                                 ctypes.byref(ex)) == 0
        sizes.add(ws.value)
        lib.aclDestroyAclOpExecutor(ex)
    assert len(sizes) == 1


def test_operator_archive_holds_the_operators(pkg):
    """lib/libascendcl_qmm.a (what the reference-side build links in the interposed configuration) defines the
    operator entry points and leaves the runtime / meta objects to the host library."""
    import subprocess
    path = os.path.join(os.path.dirname(pkg.LIB_PATH), "libascendcl_qmm.a")
    assert os.path.exists(path), "run __graft_entry__.build()"
    out = subprocess.run(["nm", "-g", "--defined-only", path], stdout=subprocess.PIPE, text=True, check=True).stdout
    defined = {ln.split()[-1] for ln in out.splitlines() if len(ln.split()) >= 3}
    for name in ("aclnnWeightQuantBatchMatmulV2GetWorkspaceSize", "aclnnWeightQuantBatchMatmulV2", "aclnnQuantMatmulV4",
                 "aclnnMatmulMxFp8Hw", "aclnnTransMatmulWeight", "aclnnDynamicQuant", "aclnnQuantGroupedMatmulDequant"):
        assert name in defined, name
    assert "aclrtMalloc" not in defined and "aclCreateTensor" not in defined
