"""GPU test of the entry point that takes no workspace and allocates nothing.

Some programs built around the reference give the decode path no scratch buffer (the reference
asks for 0 bytes there) and cannot allocate one where they run, so the library keeps the split-K
partial sums in a fixed array of its own.  The array is shared by all calls and never cleared:
the test calls the entry point twice in a row, with different inputs, and checks each result
against the ordinary workspace-taking entry point.  Collected last on purpose (zz), so a run that
stops at the first failure has already run everything else; it also passes alone in a fresh process.
"""
import ctypes

import pytest
import torch

from util import assert_close, to_np

pytestmark = pytest.mark.gpu


def _call(pkg, d, dev, group, int4):
    lib = pkg.load()
    fn = lib.aclnnB200WeightQuantMatmulNoAlloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int64] * 4 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    x, w, sc = d["x"].to(dev), d["w"].to(dev), d["scale"].to(dev)
    of = d["offset"].to(dev) if d["offset"] is not None else None
    b = d["bias"].to(dev) if d["bias"] is not None else None
    out = torch.empty((d["M"], d["N"]), dtype=x.dtype, device=dev)
    ptr = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    st = fn(ptr(x), ptr(w), ptr(sc), ptr(of), ptr(b), ptr(out), d["M"], d["K"], d["N"], group,
            pkg.torch_acl_dtype(x), pkg.ACL_INT4 if int4 else pkg.ACL_INT8, ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    return st, out


def test_no_alloc_entry_point_twice_in_a_row(pkg, workloads, dev):
    cases = [workloads.w4a16(M=1, K=4096, N=4096, group=128, seed=7001),            # 8 x 1 x 4096 partial sums
             workloads.w4a16(M=4, K=2048, N=1024, group=128, seed=7002, with_bias=False),
             workloads.w8a16(M=2, K=1024, N=3072, dtype=torch.float16, seed=7003, with_offset=True),
             workloads.w4a16(M=3, K=1024, N=512, group=128, seed=7005),                 # the 3..4-row form of the kernel
             workloads.w4a16(M=1, K=128, N=256, group=128, seed=7006),                  # one K slice: no partial sums at all
             workloads.w8a16(M=2, K=512, N=256, dtype=torch.float32, seed=7007, with_offset=True)]   # fp32 activations
    for d in cases:  # back to back on one stream: each call reuses the array the previous one left dirty
        st, got = _call(pkg, d, dev, d["group"], d["int4"])
        assert st == 0
        want = pkg.weight_quant_matmul(d["x"].to(dev), d["w"].to(dev), d["scale"].to(dev),
                                       d["offset"].to(dev) if d["offset"] is not None else None,
                                       d["bias"].to(dev) if d["bias"] is not None else None, int4=d["int4"], group=d["group"])
        torch.cuda.synchronize()
        assert_close(to_np(got), to_np(want), "no-alloc entry point vs aclnnWeightQuantBatchMatmulV2Ex")
    # and the first case again, after the others have overwritten the array
    st, again = _call(pkg, cases[0], dev, 128, True)
    first = pkg.weight_quant_matmul(cases[0]["x"].to(dev), cases[0]["w"].to(dev), cases[0]["scale"].to(dev),
                                    cases[0]["offset"].to(dev), cases[0]["bias"].to(dev), int4=True, group=128)
    torch.cuda.synchronize()
    assert st == 0
    assert_close(to_np(again), to_np(first), "second call on the same problem")


def test_no_alloc_entry_point_rejects_what_does_not_fit(pkg, workloads, dev):
    # M above the decode limit, and a problem whose partial sums exceed the built-in 2 MiB
    d = workloads.w4a16(M=8, K=256, N=64, group=128, seed=7004)
    assert _call(pkg, d, dev, 128, True)[0] == 161002
    big = dict(M=4, K=8192, N=65536, int4=True, group=128, bias=None, offset=None,
               x=torch.zeros((4, 8192), dtype=torch.bfloat16), w=torch.zeros(8192 * 65536 // 2, dtype=torch.uint8),
               scale=torch.ones((64, 65536), dtype=torch.bfloat16))
    assert _call(pkg, big, dev, 128, True)[0] == 161002
    torch.cuda.synchronize()
