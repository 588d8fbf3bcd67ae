"""GPU parity tests: every operator of the family, through the C ABI, against the CPU checker on
identical seeded inputs -- bit-exact for integer work, within the stated tolerance for fp outputs."""
import ctypes
import os

import numpy as np
import pytest
import torch

from util import assert_close, dev_or_none, errors, f32, nz_layout_model, to_np

pytestmark = pytest.mark.gpu


class forced_path:
    """Pin the kernel family (generic | gemv | tc) for the calls inside the block."""

    def __init__(self, path):
        self.path = path

    def __enter__(self):
        self.prev = os.environ.get("B200_QMM_PATH")
        if self.path:
            os.environ["B200_QMM_PATH"] = self.path
        elif self.prev is not None:
            del os.environ["B200_QMM_PATH"]

    def __exit__(self, *a):
        if self.prev is None:
            os.environ.pop("B200_QMM_PATH", None)
        else:
            os.environ["B200_QMM_PATH"] = self.prev


class env_set:
    """Set one environment knob of the library for the calls inside the block."""

    def __init__(self, name, value):
        self.name, self.value = name, value

    def __enter__(self):
        self.prev = os.environ.get(self.name)
        os.environ[self.name] = self.value

    def __exit__(self, *a):
        if self.prev is None:
            os.environ.pop(self.name, None)
        else:
            os.environ[self.name] = self.prev


def run_wq(pkg, d, dev, name="aclnnWeightQuantBatchMatmulV2Ex"):
    out = pkg.weight_quant_matmul(d["x"].to(dev), d["w"].to(dev), d["scale"].to(dev), dev_or_none(d["offset"], dev),
                                  dev_or_none(d["bias"], dev), int4=d["int4"], group=d["group"], name=name)
    torch.cuda.synchronize()
    return out


def ref_wq(oracle, d):
    return oracle.wqbmm_fast(f32(d["x"]), d["w"].numpy(), d["int4"], f32(d["scale"]), f32(d["offset"]), f32(d["bias"]),
                             d["M"], d["K"], d["N"], d["group"])


def assert_close_wq(oracle, out, d, what):
    """Every path is held to the family's bounds against the exact (unrounded) product.  fp16 problems with
    more than 32 rows of group-wise int4, or more than 128 rows, round the dequantised weights to fp16 as
    the reference does (cuda/src/ops/matmul.cu:734-747,790-795); bf16 problems keep them exact in the
    streaming kernels and carry them in fp16 on the expand-then-dense path."""
    assert_close(out, ref_wq(oracle, d), what)


# ------------------------------------------------------------------ weight-only quantized matmul
@pytest.mark.parametrize("path", ["generic", "gemv", "tc", None])
@pytest.mark.parametrize("M", [1, 2, 3, 4, 16, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_w4a16_groupwise(pkg, oracle, workloads, dev, path, M, dtype):
    d = workloads.w4a16(M=M, K=1024, N=512, group=128, dtype=dtype, seed=3000 + M)
    with forced_path(path):
        out = run_wq(pkg, d, dev)
    if path == "generic":   # the generic kernel keeps the weights exact at every M
        assert_close(to_np(out), ref_wq(oracle, d), f"W4A16 g128 M={M} {dtype} path={path}")
    else:
        assert_close_wq(oracle, to_np(out), d, f"W4A16 g128 M={M} {dtype} path={path}")


@pytest.mark.parametrize("path", ["generic", "gemv", "tc", None])
@pytest.mark.parametrize("int4", [False, True])
@pytest.mark.parametrize("M", [1, 4, 128])
def test_wqmm_reference_test_shapes(pkg, oracle, workloads, dev, path, int4, M):
    """The reference's t_wqmm cases (tests/test_matmul_conv.cpp:621-640,971-974): fp16, per-channel scale
    0.02+0.01*(n%5), offset (n%3)-1, K=256, N=64; its tolerance is 2e-2, ours is tighter."""
    K, N = 256, 64
    d = (workloads.w4a16(M=M, K=K, N=N, dtype=torch.float16, per_channel=True, with_bias=False, seed=11) if int4
         else workloads.w8a16(M=M, K=K, N=N, dtype=torch.float16, with_offset=True, seed=11))
    n = torch.arange(N)
    d["scale"] = (0.02 + 0.01 * (n % 5)).to(torch.float16)
    d["offset"] = ((n % 3) - 1).to(torch.float16)
    with forced_path(path):
        out = run_wq(pkg, d, dev, name="aclnnWeightQuantBatchMatmul")
    assert_close(to_np(out), ref_wq(oracle, d), f"t_wqmm int4={int4} M={M} path={path}")


def test_config0_w8a16_full_size(pkg, oracle, workloads, dev):
    d = workloads.w8a16()  # M=1, K=1024, N=3072, fp16, per-channel
    for name in ("aclnnWeightQuantBatchMatmul", "aclnnWeightQuantBatchMatmulV2", "aclnnWeightQuantBatchMatmulV3",
                 "aclnnWeightQuantBatchMatmulNz"):
        out = run_wq(pkg, d, dev, name=name)
        assert_close(to_np(out), ref_wq(oracle, d), name)


@pytest.mark.parametrize("M", [1, 16, 128])
def test_config1_w4a16_full_size(pkg, oracle, workloads, dev, M):
    d = workloads.w4a16(M=M)  # K=4096, N=4096, g128, bf16, offset + bias
    out = run_wq(pkg, d, dev)
    assert_close_wq(oracle, to_np(out), d, f"config1 M={M}")
    # without the optional arguments
    d2 = workloads.w4a16(M=M, with_offset=False, with_bias=False)
    assert_close_wq(oracle, to_np(run_wq(pkg, d2, dev)), d2, f"config1 no offset/bias M={M}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K,N,group", [(33, 1024, 512, 128), (64, 2048, 1056, 256), (100, 1024, 4096, 128),
                                         (128, 4096, 20000 // 32 * 32, 128), (70, 2048, 20000 // 32 * 32, 256)])
def test_w4a16_groupwise_mid_m(pkg, oracle, workloads, dev, dtype, M, K, N, group):
    """33..128 rows of group-wise int4: the streaming kernel's converters apply scale and offset
    themselves.  Covers a ragged last column tile (N % 128 = 32), two row tiles, two super-blocks per
    scale group, and more tiles than SMs (shares cut tiles anywhere); the two largest cases run one
    128-row tile per column block, the others 64-row tiles."""
    d = workloads.w4a16(M=M, K=K, N=N, group=group, dtype=dtype, seed=5200 + M)
    assert_close_wq(oracle, to_np(run_wq(pkg, d, dev)), d, f"W4A16 g{group} M={M} K={K} N={N} {dtype}")
    d2 = workloads.w4a16(M=M, K=K, N=N, group=group, dtype=dtype, with_offset=False, with_bias=False, seed=5300 + M)
    assert_close_wq(oracle, to_np(run_wq(pkg, d2, dev)), d2, f"W4A16 g{group} M={M} no offset/bias {dtype}")
    with env_set("B200_QMM_WQ_PRESCALE", "0"):   # the exact per-group fold stays available
        assert_close(to_np(run_wq(pkg, d, dev)), ref_wq(oracle, d), f"W4A16 g{group} M={M} exact fold {dtype}")


@pytest.mark.parametrize("int4", [True, False])
@pytest.mark.parametrize("M", [1, 40])
def test_wq_per_channel_long_k(pkg, oracle, workloads, dev, int4, M):
    """Per-channel scales over a long K: one scale fold covers dozens of super-blocks of the streaming
    kernel (shape of the Llama-70B projections the reference can run: fp16, [N] scales, offset)."""
    K, N = (8192, 1536) if M > 1 else (8192, 28672)   # the second has more tiles than SMs: shares cut tiles anywhere
    d = (workloads.w4a16(M=M, K=K, N=N, dtype=torch.float16, per_channel=True, with_bias=False, seed=31) if int4
         else workloads.w8a16(M=M, K=K, N=N, dtype=torch.float16, with_offset=True, seed=31))
    out = run_wq(pkg, d, dev, name="aclnnWeightQuantBatchMatmul")
    assert_close(to_np(out), ref_wq(oracle, d), f"per-channel long K int4={int4} M={M}")
    lib = pkg.load()
    lib.aclnnB200DeviceStatus.restype = ctypes.c_uint32
    assert lib.aclnnB200DeviceStatus() == 0


@pytest.mark.parametrize("shape", [(1, 1056, 160), (17, 200, 96), (70, 1160, 416), (300, 392, 224)])
@pytest.mark.parametrize("int4", [True, False])
def test_wq_tensor_core_tails(pkg, oracle, workloads, dev, shape, int4):
    """Shapes that are not multiples of any tile: K tails are zero-filled by TMA, M and N tails are
    masked in the epilogue.  Per-channel scales with offset and bias, through the tensor-core paths."""
    M, K, N = shape
    d = (workloads.w4a16(M=M, K=K, N=N, dtype=torch.bfloat16, per_channel=True, seed=41) if int4
         else workloads.w8a16(M=M, K=K, N=N, dtype=torch.bfloat16, with_offset=True, seed=41))
    if d["bias"] is None:
        d["bias"] = (torch.randn(N, generator=torch.Generator().manual_seed(42)) * 0.02).to(torch.bfloat16)
    with forced_path("tc"):
        out = run_wq(pkg, d, dev)
    assert_close(to_np(out), ref_wq(oracle, d), f"tails {shape} int4={int4}")


@pytest.mark.parametrize("shape", [(1, 16, 16), (5, 48, 80), (100, 528, 400), (300, 1040, 272), (513, 144, 1040)])
def test_w8a8_tensor_core_tails(pkg, oracle, workloads, dev, shape):
    M, K, N = shape
    d = workloads.w8a8(M=M, K=K, N=N, seed=43)
    with forced_path("tc"):
        acc = pkg.quant_matmul(d["x"].to(dev), d["w"].to(dev), None)
        out = pkg.quant_matmul(d["x"].to(dev), d["w"].to(dev), d["scale"].to(dev), d["pertoken"].to(dev), d["bias"].to(dev),
                               out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    ref_acc, ref_out = ref_qmm(oracle, d, torch.bfloat16)
    assert np.array_equal(acc.cpu().numpy(), ref_acc)
    assert torch.equal(out.cpu(), ref_out)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(129, 256, 264), (300, 1040, 520), (600, 2048, 8200), (1000, 144, 40000)])
def test_w8a8_row_tile_kernel_equals_column_kernel(pkg, oracle, workloads, dev, shape, out_dtype):
    """More than 128 rows run the row-tile dense kernel (rows on the accumulator lanes); with
    B200_QMM_DENSE_ROWTILE=0 the column-per-lane kernel takes the same call.  Accumulators and outputs
    must be the same bits for ragged M, N (multiples of 8 only) and K, for more tiles than SMs with a
    K-split tail, with and without per-token scales and bias; the small shapes also against the oracle."""
    M, K, N = shape
    d = workloads.w8a8(M=M, K=K, N=N, seed=47)
    x, w, sc, pt, bi = (d[k].to(dev) for k in ("x", "w", "scale", "pertoken", "bias"))
    def run():
        with forced_path("tc"):
            r = [pkg.quant_matmul(x, w, None), pkg.quant_matmul(x, w, sc, pt, bi, out_dtype=out_dtype),
                 pkg.quant_matmul(x, w, sc, None, None, out_dtype=out_dtype)]
        torch.cuda.synchronize()
        return r
    got = run()
    with env_set("B200_QMM_DENSE_ROWTILE", "0"):
        want = run()
    for g_, w_ in zip(got, want):
        assert torch.equal(g_, w_)
    if M * K * N <= 300 * 1040 * 520:
        ref_acc, ref_out = ref_qmm(oracle, d, out_dtype)
        assert np.array_equal(got[0].cpu().numpy(), ref_acc)
        assert torch.equal(got[1].cpu(), ref_out)


@pytest.mark.parametrize("shape", [(1, 32, 16), (33, 96, 48), (200, 544, 400)])
@pytest.mark.parametrize("kinds", [(False, True), (True, False)])
def test_mx_tensor_core_tails(pkg, oracle, workloads, dev, shape, kinds):
    M, K, N = shape
    d = workloads.mx(M=M, K=K, N=N, a_fp4=kinds[0], b_fp4=kinds[1], seed=44)
    with forced_path("tc"):
        out = run_mx(pkg, d, dev, torch.float32, "aclnnMatmulMxFp8")
    assert_close(to_np(out), ref_mx(oracle, d), f"mx tails {shape} {kinds}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M", [1, 2, 3, 5, 8, 9, 13, 16])
def test_w4a16_decode_kernel_rows(pkg, oracle, workloads, dev, M, dtype):
    """The decode kernel (register dequant + mma.sync, M <= 16): every row count on both sides of its
    one- and two-fragment forms, with group scales, offsets and bias, over several tiles and K shares."""
    d = workloads.w4a16(M=M, K=2048, N=1536, group=128, dtype=dtype, seed=5100 + M)
    assert_close(to_np(run_wq(pkg, d, dev)), ref_wq(oracle, d), f"decode M={M} {dtype}")


@pytest.mark.parametrize("case", [
    dict(K=1024, N=512, group=256),                      # two super-blocks per scale group
    dict(K=1024, N=512, group=128, with_offset=False),   # no offset: only the dequant constant is folded
    dict(K=1024, N=512, group=128, with_bias=False),
    dict(K=2176, N=800, per_channel=True),               # K and N off every tile size, per-channel scales
    dict(K=136, N=32, per_channel=True),                 # smallest shape the tensor-core family takes
    dict(K=8192, N=256, group=128),                      # one tile cut into many K shares
    dict(K=128, N=8192, group=128),                      # one quantum per tile, more tiles than SMs
])
@pytest.mark.parametrize("M", [1, 7, 16])
def test_w4a16_decode_kernel_shapes(pkg, oracle, workloads, dev, case, M):
    d = workloads.w4a16(M=M, dtype=torch.bfloat16, seed=5200 + M, **case)
    assert_close(to_np(run_wq(pkg, d, dev)), ref_wq(oracle, d), f"decode M={M} {case}")


@pytest.mark.parametrize("M", [1, 16])
def test_w4a16_decode_kernel_agrees_with_tcgen05_kernel(pkg, oracle, workloads, dev, M):
    """The same call through the decode kernel and, with it switched off, through the stream-K
    tcgen05 kernel that serves M > 16: both within the bounds of the oracle and of each other."""
    d = workloads.w4a16(M=M, K=4096, N=1024, group=128, dtype=torch.bfloat16, seed=5300 + M)
    ref = ref_wq(oracle, d)
    a = to_np(run_wq(pkg, d, dev))
    with env_set("B200_QMM_WQ_MMA", "0"):
        b = to_np(run_wq(pkg, d, dev))
    assert_close(a, ref, "decode kernel")
    assert_close(b, ref, "tcgen05 stream-K kernel")
    assert_close(a, b, "decode vs tcgen05")


def test_w4a16_decode_kernel_repeatable(pkg, workloads, dev):
    """Partial tiles are summed in a fixed order: two calls give identical bits."""
    d = workloads.w4a16(M=4, K=4096, N=2048, group=128, dtype=torch.bfloat16, seed=5400)
    a = run_wq(pkg, d, dev).clone()
    b = run_wq(pkg, d, dev)
    assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M", [1, 4, 8, 11, 16])
@pytest.mark.parametrize("shape", [(1024, 3072), (2176, 272), (4096, 1024)])
def test_w8a16_decode_kernel(pkg, oracle, workloads, dev, M, dtype, shape):
    """int8 weights through the decode kernel: each byte is split into an unsigned low and a signed
    high nibble that share one mma and are recombined in the fold.  Includes the extreme values
    -128 and 127, per-channel offsets and a group-wise case."""
    K, N = shape
    d = workloads.w8a16(M=M, K=K, N=N, dtype=dtype, with_offset=True, seed=5500 + M)
    d["w"][0, :] = -128
    d["w"][1, :] = 127
    d["w"][2, ::2] = -1
    assert_close(to_np(run_wq(pkg, d, dev)), ref_wq(oracle, d), f"W8A16 decode M={M} {shape} {dtype}")
    if K % 256 == 0:
        g = torch.Generator().manual_seed(5600 + M)
        d["group"] = 256
        d["scale"] = (torch.rand((K // 256, N), generator=g) * 0.015 + 0.005).to(dtype)
        d["offset"] = (torch.rand((K // 256, N), generator=g) * 2 - 1).to(dtype)
        d["bias"] = (torch.randn(N, generator=g) * 0.02).to(dtype)
        assert_close(to_np(run_wq(pkg, d, dev)), ref_wq(oracle, d), f"W8A16 g256 decode M={M} {shape} {dtype}")


def test_large_m_weight_only_prefill(pkg, oracle, workloads, dev):
    """M above the switch to the expand-then-dense path.  fp16: the weights are rounded once to fp16, the
    reference's own large-M form (cuda/src/ops/matmul.cu:733-747,790-795), checked against that form and
    against the exact product.  bf16 (which the reference cannot run): the product runs in fp16 with a
    power-of-two scale per activation row, so the weights keep 11 significant bits; checked against the
    exact product at the family's bounds, with and without offset and bias, including rows of very
    different magnitude, a zero row, and the bf16-weight form behind its switch."""
    def ref_rounded(d, kind):
        return oracle.wqbmm_fast(f32(d["x"]), d["w"].numpy(), d["int4"], f32(d["scale"]), f32(d["offset"]), f32(d["bias"]),
                                 d["M"], d["K"], d["N"], d["group"], weight_round=kind)
    d = workloads.w4a16(M=384, K=2048, N=1024, group=128, seed=45)
    d["x"][3] *= 2.0 ** 40     # rows far apart in magnitude: each row has its own power-of-two scale
    d["x"][4] *= 2.0 ** -60
    d["x"][5] = 0
    out = to_np(run_wq(pkg, d, dev))
    ref = ref_wq(oracle, d)
    mx, mean = assert_close(out, ref, "W4A16 g128 M=384 bf16 vs exact")
    print(f"[parity] W4A16 g128 M=384 bf16 (fp16 product): max_rel={mx:.3e} mean_rel={mean:.3e}")
    for r in (3, 4, 6):        # per row: the huge row must not hide the others in the pooled figure
        assert_close(out[r], ref[r], f"row {r}", max_rel=2e-2, mean_rel=3e-3)
    assert np.array_equal(out[5], to_np(d["bias"].to(torch.bfloat16)))   # zero row: bias only
    d2 = workloads.w4a16(M=200, K=1024, N=512, group=128, seed=46, with_offset=False, with_bias=False)
    assert_close(to_np(run_wq(pkg, d2, dev)), ref_wq(oracle, d2), "W4A16 g128 M=200 bf16, no offset/bias, vs exact")
    with env_set("B200_QMM_WQ_BF16_VIA_F16", "0"):
        out = to_np(run_wq(pkg, d2, dev))
    assert_close(out, ref_rounded(d2, "bf16"), "W4A16 g128 M=200 bf16 weights vs that form")
    d = workloads.w8a16(M=260, K=1024, N=512, dtype=torch.float16, with_offset=True, seed=46)
    out = to_np(run_wq(pkg, d, dev, name="aclnnWeightQuantBatchMatmulV2"))
    assert_close(out, ref_rounded(d, "f16"), "W8A16 M=260 vs reference large-M form")
    assert_close(out, ref_wq(oracle, d), "W8A16 M=260 vs exact")
    d = workloads.w8a16(M=300, K=2048, N=768, dtype=torch.bfloat16, with_offset=True, seed=47)
    assert_close(to_np(run_wq(pkg, d, dev, name="aclnnWeightQuantBatchMatmulV2")), ref_wq(oracle, d), "W8A16 M=300 bf16 vs exact")


def test_pointers_handed_over_between_the_phases(pkg, oracle, workloads, dev):
    """Phase 1 with every data pointer still null, then aclSetRawTensorAddr, then phase 2 (the executor
    reads the pointers when it runs): W4A16 with offset at 1, 40 and 200 rows must report a workspace that
    phase 2 accepts and give the ordinary result."""
    lib = pkg.load()
    for M in (1, 40, 200):
        d = workloads.w4a16(M=M, K=1024, N=512, group=128, seed=8100 + M)
        real = {k: d[k].to(dev) for k in ("x", "w", "scale", "offset", "bias")}
        out = torch.empty((M, 512), dtype=torch.bfloat16, device=dev)
        tens = {"x": pkg.AclTensor(real["x"]), "w": pkg.AclTensor(real["w"], pkg.ACL_INT4, (1024, 512)),
                "scale": pkg.AclTensor(real["scale"]), "offset": pkg.AclTensor(real["offset"]), "bias": pkg.AclTensor(real["bias"]),
                "out": pkg.AclTensor(out)}
        for t in tens.values():
            assert lib.aclSetRawTensorAddr(ctypes.c_void_p(t.h), None) == 0
        ws, ex = ctypes.c_uint64(0), ctypes.c_void_p(0)
        st = lib.aclnnWeightQuantBatchMatmulV2ExGetWorkspaceSize(
            ctypes.c_void_p(tens["x"].h), ctypes.c_void_p(tens["w"].h), ctypes.c_void_p(tens["scale"].h),
            ctypes.c_void_p(tens["offset"].h), ctypes.c_void_p(tens["bias"].h), ctypes.c_int64(128), ctypes.c_void_p(tens["out"].h),
            ctypes.byref(ws), ctypes.byref(ex))
        assert st == 0
        for k, t in tens.items():
            buf = out if k == "out" else real[k]
            assert lib.aclSetRawTensorAddr(ctypes.c_void_p(t.h), ctypes.c_void_p(buf.data_ptr())) == 0
        wsbuf = torch.empty(max(1, ws.value), dtype=torch.uint8, device=dev)
        st = lib.aclnnWeightQuantBatchMatmulV2Ex(ctypes.c_void_p(wsbuf.data_ptr()), ctypes.c_uint64(ws.value), ex,
                                                 ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        assert st == 0, (M, st)
        torch.cuda.synchronize()
        assert_close(to_np(out), ref_wq(oracle, d), f"pointers set between the phases, M={M}")


def test_misaligned_pointers_fall_back_to_the_generic_kernel(pkg, oracle, workloads, dev):
    """The fast kernels need 16-byte aligned operands.  A view that starts 2 or 8 bytes into a buffer is
    refused by their launchers before anything runs and the call is served by the bounds-checked generic
    kernel: same result, no device fault, status word still 0."""
    lib = pkg.load()
    lib.aclnnB200DeviceStatus.restype = ctypes.c_uint32
    for M in (1, 40, 200):
        d = workloads.w4a16(M=M, K=1024, N=512, group=128, seed=8200 + M)
        xbuf = torch.empty(M * 1024 + 8, dtype=torch.bfloat16, device=dev)
        x = xbuf[1:1 + M * 1024].view(M, 1024)          # 2 bytes off
        x.copy_(d["x"])
        obuf = torch.empty(M * 512 + 8, dtype=torch.bfloat16, device=dev)
        out = obuf[4:4 + M * 512].view(M, 512)          # 8 bytes off
        got = pkg.weight_quant_matmul(x, d["w"].to(dev), d["scale"].to(dev), d["offset"].to(dev), d["bias"].to(dev), int4=True,
                                      group=128, out=out)
        torch.cuda.synchronize()
        assert_close(to_np(got), ref_wq(oracle, d), f"misaligned x and out, M={M}")
    q = workloads.w8a8(M=200, K=512, N=256, seed=8300)
    obuf = torch.empty(200 * 256 + 8, dtype=torch.bfloat16, device=dev)
    out = obuf[1:1 + 200 * 256].view(200, 256)
    got = pkg.quant_matmul(q["x"].to(dev), q["w"].to(dev), q["scale"].to(dev), q["pertoken"].to(dev), q["bias"].to(dev), out=out)
    torch.cuda.synchronize()
    _, want = ref_qmm(oracle, q, torch.bfloat16)
    assert torch.equal(got.cpu(), want)
    assert lib.aclnnB200DeviceStatus() == 0


def test_wq_fp32_and_ragged_shapes(pkg, oracle, workloads, dev):
    """fp32 activations (tests/test_quant_parity.cpp:405-413, tol 1e-4) and shapes off every tile size."""
    for (M, K, N) in [(5, 8, 6), (3, 40, 50), (17, 72, 34)]:
        d = workloads.w8a16(M=M, K=K, N=N, dtype=torch.float32, with_offset=True, seed=5)
        out = run_wq(pkg, d, dev, name="aclnnWeightQuantBatchMatmulV2")
        mx, _ = errors(to_np(out), ref_wq(oracle, d))
        assert mx <= 1e-4, (M, K, N, mx)
    d = workloads.w4a16(M=3, K=40, N=50, group=8, dtype=torch.float16, seed=6)
    assert_close(to_np(run_wq(pkg, d, dev)), ref_wq(oracle, d), "ragged int4 g8")


def test_empty_m(pkg, dev):
    x = torch.empty((0, 64), dtype=torch.float16, device=dev)
    w = torch.zeros((64, 32), dtype=torch.int8, device=dev)
    sc = torch.ones(32, dtype=torch.float16, device=dev)
    out = pkg.weight_quant_matmul(x, w, sc, name="aclnnWeightQuantBatchMatmul")
    torch.cuda.synchronize()
    assert out.shape == (0, 32)


# ------------------------------------------------------------------ W8A8
def ref_qmm(oracle, d, out_dtype):
    acc = oracle.qmm_acc_fast(d["x"].numpy(), d["w"].numpy(), d["M"], d["K"], d["N"])
    v = oracle.qmm_epilogue_fast(acc, f32(d["scale"]), f32(d["pertoken"]),
                                 None if d["bias"] is None else d["bias"].numpy())
    return acc, torch.from_numpy(v).to(out_dtype)


@pytest.mark.parametrize("path", ["generic", "tc", None])
@pytest.mark.parametrize("M", [1, 8, 100, 256])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_w8a8_bit_exact(pkg, oracle, workloads, dev, path, M, out_dtype):
    d = workloads.w8a8(M=M, K=512, N=384, seed=4000 + M, out_dtype=out_dtype)
    x, w = d["x"].to(dev), d["w"].to(dev)
    with forced_path(path):
        acc = pkg.quant_matmul(x, w, None)
        out = pkg.quant_matmul(x, w, d["scale"].to(dev), d["pertoken"].to(dev), d["bias"].to(dev), out_dtype=out_dtype)
    torch.cuda.synchronize()
    ref_acc, ref_out = ref_qmm(oracle, d, out_dtype)
    assert np.array_equal(acc.cpu().numpy(), ref_acc), "int32 accumulators must be bit-exact"
    assert torch.equal(out.cpu(), ref_out), "epilogue is a fixed fp32 sequence: output must be bit-exact"


def test_w8a8_aliases_and_reference_test_case(pkg, oracle, workloads, dev):
    """t_qmm / t_qmm_v of the reference (tests/test_matmul_conv.cpp:641-673): M128 K256 N64, fp16 scale
    0.001*(1+n%7), fp16 out; plus the parity-test shape M8 K16 N8 with fp32 out through every alias name
    (tests/test_quant_parity.cpp:362-370,540-552)."""
    names = ["aclnnQuantMatmul", "aclnnQuantMatmulV2", "aclnnQuantMatmulV3", "aclnnQuantMatmulV4", "aclnnQuantMatmulV5",
             "aclnnQuantMatmulDequant", "aclnnQuantMatmulWeightNz", "aclnnFusedQuantMatmul", "aclnnFusedQuantMatmulWeightNz",
             "aclnnMatmulCompressDequant", "aclnnSparse4to2QuantMatmulWeightNz", "aclnnDualLevelQuantMatmulWeightNz"]
    for (M, K, N, odt) in [(128, 256, 64, torch.float16), (8, 16, 8, torch.float32)]:
        d = workloads.w8a8(M=M, K=K, N=N, seed=11, with_pertoken=False, with_bias=False)
        d["scale"] = (0.001 * (1 + torch.arange(N) % 7)).to(torch.float16)
        _, ref_out = ref_qmm(oracle, d, odt)
        for name in names:
            out = pkg.quant_matmul(d["x"].to(dev), d["w"].to(dev), d["scale"].to(dev), out_dtype=odt, name=name)
            torch.cuda.synchronize()
            assert torch.equal(out.cpu(), ref_out), name


def test_w8a8_wrappers(pkg, oracle, workloads, dev):
    # out += dequant(x @ w): the product is rounded to the output type before the add, like the
    # reference's temp buffer (cuda/src/ops/quant.cu:286-297); t_qmm_iadd shape 64x128x48.
    d = workloads.w8a8(M=64, K=128, N=48, seed=12, with_pertoken=False, with_bias=False, scale_dtype=torch.float16)
    _, prod = ref_qmm(oracle, d, torch.float16)
    acc0 = (0.5 * ((torch.arange(64 * 48) % 11) - 5)).to(torch.float16).reshape(64, 48)
    out = acc0.clone().to(dev)
    pkg.quant_matmul(d["x"].to(dev), d["w"].to(dev), d["scale"].to(dev), name="aclnnQuantBatchMatmulInplaceAdd", out=out)
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), (acc0.float() + prod.float()).to(torch.float16))
    # weight stored [N,K] (cuda/src/ops/quant.cu:303-326; test 32x64x48)
    d = workloads.w8a8(M=32, K=64, N=48, seed=13, with_pertoken=False, with_bias=False, scale_dtype=torch.float16)
    _, want = ref_qmm(oracle, d, torch.float16)
    wt = d["w"].t().contiguous()
    out = pkg.quant_matmul(d["x"].to(dev), wt.to(dev), d["scale"].to(dev), out_dtype=torch.float16,
                           name="aclnnTransposeQuantBatchMatMul")
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), want)
    # batched (tests/test_matmul_conv.cpp:1034-1043: 2x3x4x5, fp32 scale and output)
    B, M, K, N = 2, 3, 4, 5
    g = torch.Generator(); g.manual_seed(14)
    a = torch.randint(-127, 128, (B, M, K), generator=g, dtype=torch.int8)
    b = torch.randint(-127, 128, (B, K, N), generator=g, dtype=torch.int8)
    sc = torch.rand(N, generator=g) * 0.01
    out = pkg.quant_matmul(a.to(dev), b.to(dev), sc.to(dev), out_dtype=torch.float32, name="aclnnBatchMatmulQuant")
    torch.cuda.synchronize()
    want = torch.stack([torch.from_numpy(oracle.qmm_epilogue_fast(
        oracle.qmm_acc_fast(a[i].numpy(), b[i].numpy(), M, K, N), sc.numpy())) for i in range(B)])
    assert torch.equal(out.cpu(), want)


def test_config2_w8a8_full_size(pkg, oracle, workloads, dev):
    """M=2048, K=4096, N=14336 with per-token scale, per-channel scale and int32 bias, bf16 out."""
    d = workloads.w8a8()
    x, w = d["x"].to(dev), d["w"].to(dev)
    acc = pkg.quant_matmul(x, w, None)
    out = pkg.quant_matmul(x, w, d["scale"].to(dev), d["pertoken"].to(dev), d["bias"].to(dev), out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    # the CPU checker on a seeded sample of 96 rows (the full product is 240 GFLOP in float64)
    g = torch.Generator(); g.manual_seed(1)
    rows = torch.randperm(d["M"], generator=g)[:96].sort().values
    sub = dict(d, x=d["x"][rows], pertoken=d["pertoken"][rows], M=96)
    ref_acc, ref_out = ref_qmm(oracle, sub, torch.bfloat16)
    assert np.array_equal(acc[rows.to(dev)].cpu().numpy(), ref_acc)
    assert torch.equal(out[rows.to(dev)].cpu(), ref_out)
    # size-independent property over the whole output: column sums of the exact accumulators
    colsum = acc.to(torch.int64).sum(dim=0).cpu().numpy()
    want = d["x"].to(torch.float64).sum(dim=0).numpy() @ d["w"].to(torch.float64).numpy()
    assert np.array_equal(colsum, np.rint(want).astype(np.int64))


# ------------------------------------------------------------------ MX
def run_mx(pkg, d, dev, out_dtype, name):
    ak = pkg.ACL_FLOAT4_E2M1 if d["a_fp4"] else pkg.ACL_FLOAT8_E4M3FN
    bk = pkg.ACL_FLOAT4_E2M1 if d["b_fp4"] else pkg.ACL_FLOAT8_E4M3FN
    out = pkg.mx_matmul(d["a"].reshape(-1).to(dev), ak, d["sa"].to(dev), d["b"].reshape(-1).to(dev), bk, d["sb"].to(dev),
                        d["M"], d["K"], d["N"], out_dtype=out_dtype, name=name)
    torch.cuda.synchronize()
    return out


def ref_mx(oracle, d, rows=None):
    ak = oracle.MXK_E2M1 if d["a_fp4"] else oracle.MXK_E4M3
    bk = oracle.MXK_E2M1 if d["b_fp4"] else oracle.MXK_E4M3
    return oracle.mx_matmul_fast(d["a"].numpy(), ak, d["sa"].numpy(), d["b"].numpy(), bk, d["sb"].numpy(),
                                 d["M"], d["K"], d["N"])


@pytest.mark.parametrize("path", ["generic", "tc", None])
@pytest.mark.parametrize("kinds", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("shape", [(128, 256, 64), (64, 512, 128), (256, 256, 128)])
def test_mx_matmul(pkg, oracle, workloads, dev, path, kinds, shape):
    """Shapes of the reference's MX tests (tests/test_matmul_conv.cpp:965-970,994-995); its tolerances are
    5e-2 / 8e-2, ours are the family's 1e-2 / 2e-3."""
    M, K, N = shape
    d = workloads.mx(M=M, K=K, N=N, a_fp4=kinds[0], b_fp4=kinds[1], seed=5000 + M + K)
    want = ref_mx(oracle, d)
    for name in ("aclnnMatmulMxFp8", "aclnnMatmulMxFp8Hw", "aclnnMatmulMxFp4", "aclnnMatmulMxFp4Hw"):
        for odt in (torch.float32, torch.bfloat16):
            with forced_path(path):
                out = run_mx(pkg, d, dev, odt, name)
            assert_close(to_np(out), want, f"{name} {kinds} {shape} {odt} path={path}")


@pytest.mark.parametrize("kinds", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("shape", [(300, 1024, 800), (1, 128, 32), (129, 2048, 288), (520, 384, 1056)])
def test_mx_native_block_scaled_kernel(pkg, oracle, workloads, dev, kinds, shape):
    """The native block-scaled kernel (tcgen05.mma kind::mxf8f6f4.block_scale, e8m0 scales in tensor memory) on
    shapes with ragged M and N (zero-filled tiles, padded scale groups), every fp8 / fp4 operand mix, fp32 and bf16
    outputs, scale exponents over the whole benchmark range and beyond: against the oracle, and against the
    expand-then-bf16 path (B200_QMM_MX_NATIVE=0), which multiplies the same exact operand values."""
    M, K, N = shape
    d = workloads.mx(M=M, K=K, N=N, a_fp4=kinds[0], b_fp4=kinds[1], seed=5400 + M)
    g = torch.Generator().manual_seed(5401)
    d["sa"] = torch.randint(127 - 20, 127 + 21, d["sa"].shape, generator=g, dtype=torch.int32).to(torch.uint8)   # 2^-20 .. 2^20
    want = ref_mx(oracle, d)
    for odt in (torch.float32, torch.bfloat16):
        got = run_mx(pkg, d, dev, odt, "aclnnMatmulMxFp8Hw")
        assert_close(to_np(got), want, f"native MX {kinds} {shape} {odt}")
        with env_set("B200_QMM_MX_NATIVE", "0"):
            other = run_mx(pkg, d, dev, odt, "aclnnMatmulMxFp8Hw")
        assert_close(to_np(got), to_np(other), f"native vs expanded {kinds} {shape} {odt}", max_rel=2e-3 if odt == torch.float32 else 1e-2,
                     mean_rel=1e-5 if odt == torch.float32 else 2e-3)


def test_mx_native_tile_widths_agree(pkg, oracle, workloads, dev):
    """The native kernel's tile width is a launch parameter (256 columns and one accumulator by default; up to 240
    columns two accumulators fit and a tile's epilogue overlaps the next tile's MMAs).  Every form accumulates an output
    element in the same order, so they must agree bit for bit; the shape gives every CTA three tiles and more (both
    accumulators are reused), ragged M and N."""
    M, K, N = 1700, 256, 8000
    d = workloads.mx(M=M, K=K, N=N, a_fp4=False, b_fp4=True, seed=5470)
    outs = {}
    for width in ("240", "192", "256"):
        with env_set("B200_QMM_MX_TILE", width), env_set("B200_QMM_MX_ROWS", "128"):
            outs[width] = run_mx(pkg, d, dev, torch.float32, "aclnnMatmulMxFp8")
    torch.cuda.synchronize()
    assert torch.equal(outs["240"], outs["256"]) and torch.equal(outs["192"], outs["256"])
    # 256-row tiles (two accumulators over one weight tile, the default above 256 rows), at two widths
    for width in ("224", "160"):
        with env_set("B200_QMM_MX_TILE", width), env_set("B200_QMM_MX_ROWS", "256"):
            outs["rows256_" + width] = run_mx(pkg, d, dev, torch.float32, "aclnnMatmulMxFp8")
    torch.cuda.synchronize()
    assert torch.equal(outs["rows256_224"], outs["256"]) and torch.equal(outs["rows256_160"], outs["256"])
    assert torch.equal(run_mx(pkg, d, dev, torch.float32, "aclnnMatmulMxFp8"), outs["256"])      # the default choice
    rows = np.random.default_rng(5471).choice(M, size=96, replace=False)
    assert_close(to_np(outs["240"])[rows], ref_mx(oracle, d)[rows], "MX 1700x256x8000, 240-column tiles")
    small = workloads.mx(M=130, K=128, N=288, a_fp4=True, b_fp4=False, seed=5472)    # two tiles of 240: 240 + 48 columns
    for width, rows in (("240", "128"), ("256", "256")):     # (the 256-row form takes 240 columns where 256 are asked for)
        with env_set("B200_QMM_MX_TILE", width), env_set("B200_QMM_MX_ROWS", rows):
            outs[width] = run_mx(pkg, small, dev, torch.bfloat16, "aclnnMatmulMxFp4")
    torch.cuda.synchronize()
    assert torch.equal(outs["240"], outs["256"])
    assert_close(to_np(outs["240"]), ref_mx(oracle, small), "MX 130x128x288, 240-column tiles")


def test_mx_fp4_weight_widened_at_load_time(pkg, oracle, workloads, dev):
    """aclnnTransMatmulWeight of an fp4 weight into an ACL_FORMAT_FRACTAL_NZ tensor stores one e4m3 byte per element
    (every e2m1 value is exact in e4m3); the block-scaled matmul on it gives the bits of the call on the packed
    weight, without the per-call widening pass.  A shape the native kernel does not take is refused."""
    M, K, N = 300, 1024, 800
    d = workloads.mx(M=M, K=K, N=N, a_fp4=False, b_fp4=True, seed=5450)
    b = d["b"].reshape(-1).to(dev)
    wide = pkg.widen_fp4_weight(b, K, N)
    torch.cuda.synchronize()
    assert wide.numel() == K * N
    codes = oracle.unpack_nibbles(d["b"].numpy(), K * N)
    vals = oracle.decode_table(oracle.MXK_E2M1)[codes]
    assert np.array_equal(oracle.decode_table(oracle.MXK_E4M3)[wide.cpu().numpy()], vals)
    a, sa, sb = d["a"].reshape(-1).to(dev), d["sa"].to(dev), d["sb"].to(dev)
    plain = pkg.mx_matmul(a, pkg.ACL_FLOAT8_E4M3FN, sa, b, pkg.ACL_FLOAT4_E2M1, sb, M, K, N, out_dtype=torch.float32)
    pre = pkg.mx_matmul(a, pkg.ACL_FLOAT8_E4M3FN, sa, wide, pkg.ACL_FLOAT4_E2M1, sb, M, K, N, out_dtype=torch.float32, b_widened=True)
    torch.cuda.synchronize()
    assert torch.equal(plain, pre)
    assert_close(to_np(pre), ref_mx(oracle, d), "widened fp4 weight")
    d2 = workloads.mx(M=8, K=96, N=64, a_fp4=False, b_fp4=True, seed=5451)      # K not a multiple of 128
    w2 = pkg.widen_fp4_weight(d2["b"].reshape(-1).to(dev), 96, 64)
    out = torch.empty((8, 64), dtype=torch.float32, device=dev)
    st = pkg.call("aclnnMatmulMxFp8", pkg.AclTensor(d2["a"].reshape(-1).to(dev), pkg.ACL_FLOAT8_E4M3FN, (8, 96)),
                  pkg.AclTensor(d2["sa"].to(dev), pkg.ACL_FLOAT8_E8M0, (8, 3)),
                  pkg.AclTensor(w2, pkg.ACL_FLOAT4_E2M1, (96, 64), fmt=pkg.ACL_FORMAT_FRACTAL_NZ, storage=(w2.numel() * 2,)),
                  pkg.AclTensor(d2["sb"].to(dev), pkg.ACL_FLOAT8_E8M0, (3, 64)), pkg.AclTensor(out), return_status=True)
    assert st == 161002


def test_mx_native_e5m2_operand(pkg, oracle, dev):
    """fp8 e5m2 elements (the reference's other fp8 kind, cuda/src/ops/matmul.cu:437) through the native kernel."""
    M, K, N = 200, 512, 320
    g = torch.Generator().manual_seed(5500)
    a = torch.randn((M, K), generator=g).to(torch.float8_e5m2).view(torch.uint8)
    b = torch.randn((K, N), generator=g).to(torch.float8_e4m3fn).view(torch.uint8)
    sa = torch.randint(123, 132, (M, K // 32), generator=g, dtype=torch.int32).to(torch.uint8)
    sb = torch.randint(123, 132, (K // 32, N), generator=g, dtype=torch.int32).to(torch.uint8)
    want = oracle.mx_matmul_fast(a.numpy(), oracle.MXK_E5M2, sa.numpy(), b.numpy(), oracle.MXK_E4M3, sb.numpy(), M, K, N)
    out = pkg.mx_matmul(a.reshape(-1).to(dev), pkg.ACL_FLOAT8_E5M2, sa.to(dev), b.reshape(-1).to(dev), pkg.ACL_FLOAT8_E4M3FN, sb.to(dev),
                        M, K, N, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert_close(to_np(out), want, "MX e5m2 x e4m3")


# ------------------------------------------------------------------ the tile-packed weight layout
@pytest.mark.parametrize("shape", [(128, 256), (1024, 512), (1160, 800), (264, 32)])
def test_weight_pack_layout_and_round_trip(pkg, workloads, dev, shape):
    """aclnnCalculateMatmulWeightSizeV2 + aclnnTransMatmulWeight into an ACL_FORMAT_FRACTAL_NZ tensor:
    the packed bytes equal the layout's definition word for word (ragged K and N are zero-padded), and a
    matmul with more rows than the decode kernel takes -- which lays the weights back into [K,N] first --
    gives the same bits as the call on the original weights."""
    K, N = shape
    d = workloads.w4a16(M=40, K=K, N=N, per_channel=True, dtype=torch.float16, seed=8400 + K)
    w = d["w"].to(dev)
    packed = pkg.pack_weight_nz(w, K, N)
    torch.cuda.synchronize()
    tiles, num_sb = (N + 255) // 256, (K + 127) // 128
    assert packed.numel() == tiles * num_sb * 16384
    want = nz_layout_model(d["w_vals"].numpy())
    assert np.array_equal(packed.cpu().numpy().view(np.uint32), want)
    x, sc, of, bi = (d[k].to(dev) for k in ("x", "scale", "offset", "bias"))
    a = pkg.weight_quant_matmul(x, w, sc, of, bi, int4=True)
    b = pkg.weight_quant_matmul(x, packed, sc, of, bi, int4=True, nz=True)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    # an identity copy for everything else, as before: int8 weights, or an ND destination
    o = torch.empty_like(w)
    pkg.call("aclnnTransMatmulWeight", pkg.AclTensor(w, pkg.ACL_INT4, (K, N)), pkg.AclTensor(o, pkg.ACL_INT4, (K, N)))
    torch.cuda.synchronize()
    assert torch.equal(o, w)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M", [1, 2, 5, 8, 9, 16])
@pytest.mark.parametrize("case", [
    dict(K=1024, N=512, group=128),
    dict(K=2048, N=1536, group=256, with_offset=False),
    dict(K=1160, N=800, per_channel=True),               # K and N off every tile size: zero padding
    dict(K=8192, N=256, group=128, with_bias=False),     # one tile cut into many K shares
    dict(K=128, N=8192, group=128),                      # one stage per tile, more tiles than SMs
])
def test_w4a16_decode_kernel_packed_weights(pkg, oracle, workloads, dev, case, M, dtype):
    """The decode kernel on tile-packed weights (contiguous 16 KB copies, one 16-byte shared-memory load per
    step) against the oracle, and bit for bit against the same call on the caller's layout: both feed the
    tensor core the same fragments in the same order."""
    d = workloads.w4a16(M=M, dtype=dtype, seed=8500 + M, **case)
    K, N = d["K"], d["N"]
    w = d["w"].to(dev)
    packed = pkg.pack_weight_nz(w, K, N)
    args = (d["x"].to(dev),)
    rest = (d["scale"].to(dev), dev_or_none(d["offset"], dev), dev_or_none(d["bias"], dev))
    got = pkg.weight_quant_matmul(args[0], packed, *rest, int4=True, group=d["group"], nz=True)
    plain = pkg.weight_quant_matmul(args[0], w, *rest, int4=True, group=d["group"])
    torch.cuda.synchronize()
    assert_close(to_np(got), ref_wq(oracle, d), f"packed weights M={M} {case} {dtype}")
    if M <= 2:
        assert torch.equal(got, plain)       # the same kernel on both layouts
    else:
        # three and more rows on the caller's layout run the kernel that keeps the activations in their own type
        assert_close(to_np(got), to_np(plain), f"packed vs caller layout M={M}")
        with env_set("B200_QMM_WQ_ROWS", "0"):   # the same kernel on both layouts: same bits
            same = pkg.weight_quant_matmul(args[0], w, *rest, int4=True, group=d["group"])
        torch.cuda.synchronize()
        assert torch.equal(got, same)


def test_decode_kernel_unequal_shares(pkg, oracle, workloads, dev):
    """The decode kernel cuts the (tile, stage) space into one contiguous share per CTA from a table; with
    B200_QMM_WQ_STAGGER the shares of CTAs that lie inside one tile are shorter than the others.  Any table must give
    the oracle's result (the summation order over K changes, so not the same bits), on both weight layouts, and the
    tiles shared by two and three CTAs must all be finished (every output written)."""
    d = workloads.w4a16(M=2, K=8192, N=16384, group=128, seed=8700, with_offset=False)
    K, N = d["K"], d["N"]
    w, x, sc, bi = d["w"].to(dev), d["x"].to(dev), d["scale"].to(dev), d["bias"].to(dev)
    packed = pkg.pack_weight_nz(w, K, N)
    ref = ref_wq(oracle, d)
    for stagger in ("0", "6", "3.5"):
        with env_set("B200_QMM_WQ_STAGGER", stagger):
            a = pkg.weight_quant_matmul(x, packed, sc, None, bi, int4=True, group=128, nz=True)
            b = pkg.weight_quant_matmul(x, w, sc, None, bi, int4=True, group=128)
        torch.cuda.synchronize()
        assert torch.equal(a, b), stagger
        assert_close(to_np(a), ref, f"decode kernel, interior shares {stagger} stages shorter")


def test_packed_weights_large_m_and_rejections(pkg, oracle, workloads, dev):
    """More rows than the decode kernel takes: the weights are laid back into [K,N] in the workspace and the
    usual kernels run (17..128 rows: streaming kernel; more: expansion + dense).  int8 weights have no packed
    form (the format tag is ignored, identity copy), and a packed tensor whose storage is too small is refused."""
    for M in (17, 100, 300):
        d = workloads.w4a16(M=M, K=1024, N=1024, group=128, seed=8600 + M)
        packed = pkg.pack_weight_nz(d["w"].to(dev), 1024, 1024)
        got = pkg.weight_quant_matmul(d["x"].to(dev), packed, d["scale"].to(dev), d["offset"].to(dev), d["bias"].to(dev), int4=True,
                                      group=128, nz=True)
        torch.cuda.synchronize()
        assert_close(to_np(got), ref_wq(oracle, d), f"packed weights, M={M}")
    w = torch.zeros(256 * 256 // 2, dtype=torch.uint8, device=dev)
    small = torch.zeros(100, dtype=torch.uint8, device=dev)
    st = pkg.call("aclnnTransMatmulWeight", pkg.AclTensor(w, pkg.ACL_INT4, (256, 256)),
                  pkg.AclTensor(small, pkg.ACL_INT4, (256, 256), fmt=pkg.ACL_FORMAT_FRACTAL_NZ, storage=(200,)), return_status=True)
    assert st == 161002


# ------------------------------------------------------------------ benchmark configurations at full size
def wq_columns(d, lo, hi):
    """Columns lo..hi (even bounds) of a weight-only problem, as a problem of its own for the checker."""
    K, N = d["K"], d["N"]
    out = dict(d, N=hi - lo)
    if d["int4"]:
        out["w"] = d["w"].reshape(K, N // 2)[:, lo // 2:hi // 2].contiguous().reshape(-1)
    else:
        out["w"] = d["w"][:, lo:hi].contiguous()
    for k in ("scale", "offset", "bias"):
        if d.get(k) is not None:
            out[k] = d[k][..., lo:hi].contiguous()
    out.pop("w_vals", None)
    return out


def column_blocks(N, count, width, seed):
    """`count` blocks of `width` columns: the first, the last and seeded others, sorted."""
    rng = np.random.default_rng(seed)
    nb = N // width
    mid = rng.choice(np.arange(1, nb - 1), size=count - 2, replace=False)
    return [int(b) * width for b in sorted([0, nb - 1] + mid.tolist())]


_DEQUANT_CACHE = {}


def dequantised_weights(oracle, d, key):
    """(w - offset) * scale of a whole problem as float32 [K,N] (exact here: a 4-bit integer times a
    bf16 scale has at most 12 significant bits), built by the oracle in column chunks and kept for the
    next test on the same weights."""
    if _DEQUANT_CACHE.get("key") != key:
        _DEQUANT_CACHE.clear()
        wf = np.empty((d["K"], d["N"]), dtype=np.float32)
        for lo in range(0, d["N"], 2048):
            hi = min(d["N"], lo + 2048)
            sub = wq_columns(d, lo, hi)
            wf[:, lo:hi] = oracle.wq_dequant_fast(sub["w"].numpy(), sub["int4"], f32(sub["scale"]), f32(sub["offset"]),
                                                  sub["K"], sub["N"], sub["group"])
        _DEQUANT_CACHE.update(key=key, wf=wf)
    return _DEQUANT_CACHE["wf"]


def check_wq_sampled(oracle, out, d, what, key, col_blocks=(), width=128, rows=None, mean_rel=2e-3):
    """Compare a full-size weight-only result (no offset, no bias) with the exact product on whole column
    blocks (all rows) and, if `rows` is given, on those rows over every column.  Returns and prints
    (max_rel, mean_rel) pooled over everything compared."""
    assert d["offset"] is None and d["bias"] is None
    wf = dequantised_weights(oracle, d, key)
    x = d["x"].double().numpy()
    got_parts, ref_parts = [], []
    for lo in col_blocks:
        ref_parts.append((x @ wf[:, lo:lo + width].astype(np.float64)).reshape(-1))
        got_parts.append(to_np(out[:, lo:lo + width]).reshape(-1))
    if rows is not None:
        for lo in range(0, d["N"], 4096):
            ref_parts.append((x[rows] @ wf[:, lo:lo + 4096].astype(np.float64)).reshape(-1))
            got_parts.append(to_np(out[rows][:, lo:lo + 4096]).reshape(-1))
    got, ref = np.concatenate(got_parts), np.concatenate(ref_parts)
    mx, mean = errors(got, ref)
    print(f"[parity] {what}: {got.size} outputs vs exact oracle: max_rel={mx:.3e} mean_rel={mean:.3e}")
    assert mx <= 1e-2 and mean <= mean_rel, f"{what}: max_rel={mx:.3e}, mean_rel={mean:.3e} (<= {mean_rel})"
    return mx, mean


def test_bench_call_w4a16_llama_gate_up_m1(pkg, oracle, workloads, dev):
    """Exactly the call bench.py times: x bf16 [1,8192] @ int4 [8192,28672], bf16 scales per 128 rows, no
    offset, no bias, group 128, first weight set of its ring (seed 1004) -- every output column against
    the exact oracle."""
    d = workloads.w4a16(M=1, K=8192, N=28672, group=128, seed=1004, with_offset=False, with_bias=False)
    out = run_wq(pkg, d, dev)
    check_wq_sampled(oracle, out.cpu(), d, "bench call W4A16 g128 M=1 8192x28672", key="bench", rows=[0])


# 96 rows: beyond BASELINE's row counts, the streaming kernel's pre-scaled mode on the fp16 product
@pytest.mark.parametrize("which,M", [(w, m) for w in ("gate_up", "down") for m in (1, 32, 96, 512, 4096)])
def test_config4_llama70b_full_size(pkg, oracle, workloads, dev, which, M):
    """Llama-70B-shaped W4A16 group-128 projections (K=8192 N=28672 and K=28672 N=8192), bf16, at every row
    count of the configuration: all rows on eight whole 128-column blocks (first, last, seeded others), and
    eight seeded rows over every column.  Bounds: the family's 1e-2 / 2e-3 against the exact (unrounded)
    product."""
    d = workloads.llama70b_shard(M, which)
    out = run_wq(pkg, d, dev).cpu()
    blocks = column_blocks(d["N"], 8, 128, seed=M)
    rows = [0] if M == 1 else sorted(np.random.default_rng(M).choice(M, 8, replace=False).tolist())
    check_wq_sampled(oracle, out, d, f"config4 {which} M={M}", key=which, col_blocks=blocks, rows=rows)
    lib = pkg.load()
    lib.aclnnB200DeviceStatus.restype = ctypes.c_uint32
    assert lib.aclnnB200DeviceStatus() == 0


def test_config3_mx_full_size(pkg, oracle, workloads, dev):
    """MXFP8 e4m3 [4096,8192] x MXFP4 e2m1 [8192,8192], e8m0 scales per 32 along K, bf16 out, through
    aclnnMatmulMxFp8: 48 seeded rows over every column and all rows over 256 columns, against the product of
    the dequantised operands in float64."""
    d = workloads.mx()
    M, K, N = d["M"], d["K"], d["N"]
    out = run_mx(pkg, d, dev, torch.bfloat16, "aclnnMatmulMxFp8").cpu()
    a = oracle.mx_dequant_fast(d["a"].numpy(), oracle.MXK_E4M3, d["sa"].numpy(), M, K, True)
    rng = np.random.default_rng(7)
    rows = np.sort(rng.choice(M, 48, replace=False))
    got_parts, ref_parts = [], []
    b_bytes, sb = d["b"].numpy().reshape(K, N // 2), d["sb"].numpy()
    for lo in range(0, N, 2048):
        bb = oracle.mx_dequant_fast(np.ascontiguousarray(b_bytes[:, lo // 2:(lo + 2048) // 2]), oracle.MXK_E2M1,
                                    np.ascontiguousarray(sb[:, lo:lo + 2048]), K, 2048, False)
        ref_parts.append((a[rows] @ bb).reshape(-1))
        got_parts.append(to_np(out[rows][:, lo:lo + 2048]).reshape(-1))
        if lo in (0, 6144):   # all rows on the first and last 128 columns of this chunk
            for c in (0, 1920):
                ref_parts.append((a @ bb[:, c:c + 128]).reshape(-1))
                got_parts.append(to_np(out[:, lo + c:lo + c + 128]).reshape(-1))
    got, ref = np.concatenate(got_parts), np.concatenate(ref_parts)
    mx, mean = errors(got, ref)
    print(f"[parity] config3 MXFP8xMXFP4 4096x8192x8192 bf16: {got.size} outputs: max_rel={mx:.3e} mean_rel={mean:.3e}")
    assert mx <= 1e-2 and mean <= 2e-3, (mx, mean)


# ------------------------------------------------------------------ helpers of the family
def test_int4_pack_known_answer_and_bulk(pkg, oracle, dev):
    vals = torch.tensor([1, 2, -3, 7, -8, 0, 5, -1], dtype=torch.int8, device=dev)
    out = torch.empty(4, dtype=torch.int8, device=dev)
    pkg.call("aclnnConvertWeightToINT4Pack", pkg.AclTensor(vals), pkg.AclTensor(out))
    torch.cuda.synchronize()
    assert (out.cpu().numpy().view(np.uint8)).tolist() == [33, 125, 8, 245]
    g = torch.Generator(); g.manual_seed(3)
    for n in (2, 6, 10, 4098, 1 << 16):
        v = torch.randint(-8, 8, (n,), generator=g, dtype=torch.int8)
        o = torch.empty(n // 2, dtype=torch.uint8, device=dev)
        pkg.call("aclnnConvertWeightToINT4Pack", pkg.AclTensor(v.to(dev)), pkg.AclTensor(o))
        torch.cuda.synchronize()
        assert np.array_equal(o.cpu().numpy(), oracle.int4_pack(v.numpy()))


def test_cast_codecs(pkg, oracle, dev):
    import cases
    x = cases.cast_input()
    got = pkg.cast(x.to(dev), pkg.ACL_FLOAT, pkg.ACL_FLOAT4_E2M1, x.numel())
    torch.cuda.synchronize()
    want_codes = oracle.e2m1_encode_fast(x.numpy())
    assert np.array_equal(got.cpu().numpy(), oracle.pack_nibbles(want_codes))
    back = pkg.cast(got, pkg.ACL_FLOAT4_E2M1, pkg.ACL_FLOAT, x.numel())
    torch.cuda.synchronize()
    assert np.array_equal(back.cpu().numpy(), oracle.decode_table(oracle.MXK_E2M1)[want_codes])
    got8 = pkg.cast((x * 64).to(dev), pkg.ACL_FLOAT, pkg.ACL_FLOAT8_E4M3FN, x.numel())
    torch.cuda.synchronize()
    assert np.array_equal(got8.cpu().numpy(), oracle.e4m3_encode_fast((x * 64).numpy()))
    back8 = pkg.cast(got8, pkg.ACL_FLOAT8_E4M3FN, pkg.ACL_FLOAT, x.numel())
    torch.cuda.synchronize()
    assert np.array_equal(back8.cpu().numpy(), oracle.decode_table(oracle.MXK_E4M3)[got8.cpu().numpy()])


def test_weight_size_and_copy(pkg, dev):
    lib = pkg.load()
    shp = (ctypes.c_int64 * 2)(4096, 14336)
    ia = lib.aclCreateIntArray(shp, 2)
    out = torch.zeros(1, dtype=torch.int64, device=dev)
    pkg.call("aclnnCalculateMatmulWeightSize", ctypes.c_void_p(ia), pkg.AclTensor(out), device=dev)
    torch.cuda.synchronize()
    assert out.item() == 4096 * 14336
    lib.aclDestroyIntArray(ctypes.c_void_p(ia))
    w = torch.randint(-128, 128, (64, 48), dtype=torch.int8, device=dev)
    o = torch.empty_like(w)
    pkg.call("aclnnTransMatmulWeight", pkg.AclTensor(w), pkg.AclTensor(o))
    torch.cuda.synchronize()
    assert torch.equal(w, o)


# ------------------------------------------------------------------ against the reference's recorded outputs
def test_against_reference_backend_outputs(pkg, oracle, workloads, dev):
    """This library's kernels against outputs the reference's own CUDA backend produced on a B200 for
    the same seeded inputs (tests/golden/ref_b200_outputs.npz)."""
    import cases
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_b200_outputs.npz")
    if not os.path.exists(path):
        pytest.skip("reference outputs not recorded yet")
    ref = np.load(path)
    for name, (gen, kw) in cases.WQ_CASES.items():
        d = getattr(workloads, gen)(**kw)
        out = run_wq(pkg, d, dev, name="aclnnWeightQuantBatchMatmul")
        want = oracle.f16_bits_to_f32(ref[name]).reshape(d["M"], d["N"])
        assert_close(to_np(out), want, name)
    for name, kw in cases.QMM_CASES.items():
        d = workloads.w8a8(**kw)
        acc = pkg.quant_matmul(d["x"].to(dev), d["w"].to(dev), None)
        out = pkg.quant_matmul(d["x"].to(dev), d["w"].to(dev), d["scale"].to(dev), out_dtype=kw["out_dtype"],
                               name="aclnnQuantMatmulV4")
        torch.cuda.synchronize()
        assert np.array_equal(acc.cpu().numpy(), ref[name + "_acc"]), name
        got = out.cpu()
        got_bits = got.view(torch.int16).numpy().view(np.uint16) if got.dtype == torch.float16 else got.numpy().view(np.uint32)
        want_bits = ref[name] if got.dtype == torch.float16 else ref[name].view(np.uint32)
        assert np.array_equal(got_bits, want_bits.reshape(got_bits.shape)), name
    for name, (entry, kw) in cases.MX_CASES.items():
        d = workloads.mx(**kw)
        out = run_mx(pkg, d, dev, torch.float32, entry)
        assert_close(to_np(out), ref[name].astype(np.float64), name)


def test_grouped_and_collective_signature_forwards(pkg, oracle, workloads, dev):
    """Names that the reference forwards to the W8A8 matmul: the grouped forms (group list ignored,
    cuda/src/ops/matmul.cu:1195-1202,1402-1413) and the collective-signature forms that ignore
    their communicator (matmul.cu:1294-1302).  Same bits as aclnnQuantMatmul."""
    d = workloads.w8a8(M=40, K=256, N=96, seed=21, with_pertoken=False, with_bias=False, scale_dtype=torch.float16)
    _, want = ref_qmm(oracle, d, torch.float16)
    x, w, sc = d["x"].to(dev), d["w"].to(dev), d["scale"].to(dev)
    arr = (ctypes.c_int64 * 1)(40)
    lib = pkg.load()
    glist = ctypes.c_void_p(lib.aclCreateIntArray(arr, 1))
    for name in ("aclnnQuantGroupedMatmulDequant", "aclnnQuantGroupedMatmulDequantWeightNZ"):
        out = torch.empty((40, 96), dtype=torch.float16, device=dev)
        pkg.call(name, pkg.AclTensor(x), pkg.AclTensor(w), pkg.AclTensor(sc), glist, pkg.AclTensor(out))
        torch.cuda.synchronize()
        assert torch.equal(out.cpu(), want), name
    acc0 = torch.full((40, 96), 0.25, dtype=torch.float16)
    out = acc0.clone().to(dev)
    pkg.call("aclnnQuantGroupedMatmulInplaceAdd", pkg.AclTensor(x), pkg.AclTensor(w), pkg.AclTensor(sc), glist, pkg.AclTensor(out))
    torch.cuda.synchronize()
    assert torch.equal(out.cpu(), (acc0.float() + want.float()).to(torch.float16))
    lib.aclDestroyIntArray(glist)
    for name in ("aclnnAlltoAllQuantMatmul", "aclnnQuantMatmulAlltoAll", "aclnnAlltoAllvQuantGroupedMatMul",
                 "aclnnQuantGroupedMatMulAlltoAllv", "aclnnQuantReduceScatter", "aclnnQuantMatmulReduceSumWeightNz"):
        out = torch.empty((40, 96), dtype=torch.float16, device=dev)
        pkg.call(name, pkg.AclTensor(x), pkg.AclTensor(w), pkg.AclTensor(sc), ctypes.c_void_p(None), pkg.AclTensor(out))
        torch.cuda.synchronize()
        assert torch.equal(out.cpu(), want), name


def test_grouped_matmul_honours_the_group_list(pkg, oracle, workloads, dev):
    """Mixture-of-experts form: weight [E,K,N], scale [E,N], group list as rows per group or as running totals
    (one empty group among them): the rows of group g times weight[g], bit for bit the per-group W8A8 matmul of
    the oracle.  The reference's own form (2-D weight, list ignored, cuda/src/ops/matmul.cu:1195-1202) is covered by
    test_grouped_and_collective_signature_forwards."""
    E, K, N = 4, 256, 192
    counts = [40, 0, 130, 7]
    M = sum(counts)
    g = torch.Generator().manual_seed(8800)
    x = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    w = torch.randint(-127, 128, (E, K, N), generator=g, dtype=torch.int8)
    sc = (torch.rand((E, N), generator=g) * 0.009 + 0.001).to(torch.float16)
    want = torch.empty((M, N), dtype=torch.float16)
    r0 = 0
    for e, c in enumerate(counts):
        if c:
            acc = oracle.qmm_acc_fast(x[r0:r0 + c].numpy(), w[e].numpy(), c, K, N)
            want[r0:r0 + c] = torch.from_numpy(oracle.qmm_epilogue_fast(acc, f32(sc[e]))).to(torch.float16)
        r0 += c
    lib = pkg.load()
    xd, wd, sd = x.to(dev), w.to(dev), sc.to(dev)
    totals = [sum(counts[:i + 1]) for i in range(E)]
    for lst in (counts, totals):
        arr = (ctypes.c_int64 * E)(*lst)
        gl = ctypes.c_void_p(lib.aclCreateIntArray(arr, E))
        for name in ("aclnnQuantGroupedMatmulDequant", "aclnnQuantGroupedMatmulDequantWeightNZ"):
            out = torch.zeros((M, N), dtype=torch.float16, device=dev)
            pkg.call(name, pkg.AclTensor(xd), pkg.AclTensor(wd), pkg.AclTensor(sd), gl, pkg.AclTensor(out))
            torch.cuda.synchronize()
            assert torch.equal(out.cpu(), want), (name, lst)
        acc0 = torch.full((M, N), 0.5, dtype=torch.float16)
        out = acc0.clone().to(dev)
        pkg.call("aclnnQuantGroupedMatmulInplaceAdd", pkg.AclTensor(xd), pkg.AclTensor(wd), pkg.AclTensor(sd), gl, pkg.AclTensor(out))
        torch.cuda.synchronize()
        assert torch.equal(out.cpu(), (acc0.float() + want.float()).to(torch.float16))
        lib.aclDestroyIntArray(gl)
    bad = (ctypes.c_int64 * E)(40, 0, 130, 8)     # neither counts nor totals of M rows
    gl = ctypes.c_void_p(lib.aclCreateIntArray(bad, E))
    out = torch.zeros((M, N), dtype=torch.float16, device=dev)
    assert pkg.call("aclnnQuantGroupedMatmulDequant", pkg.AclTensor(xd), pkg.AclTensor(wd), pkg.AclTensor(sd), gl, pkg.AclTensor(out),
                    return_status=True) == 161002
    lib.aclDestroyIntArray(gl)


def test_trans_quant_param_known_answers(pkg, dev):
    """fp32 scale (+ offset) -> int64 word: low half the scale's bits, high half the offset rounded
    to the nearest int32 (cuda/src/ops/quant.cu:572-576)."""
    scale = torch.tensor([1.0, 0.5, 3.25e-3, 1e10], dtype=torch.float32)
    offset = torch.tensor([0.0, -1.4, 2.5, 7.6], dtype=torch.float32)
    bits = scale.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    for name in ("aclnnTransQuantParam", "aclnnTransQuantParamV2", "aclnnTransQuantParamV3"):
        out = torch.zeros(4, dtype=torch.int64, device=dev)
        pkg.call(name, pkg.AclTensor(scale.to(dev)), pkg.AclTensor(offset.to(dev)), pkg.AclTensor(out))
        torch.cuda.synchronize()
        hi = torch.tensor([0, -1, 2, 8], dtype=torch.int64)   # round half to even: 2.5 -> 2
        assert torch.equal(out.cpu(), ((hi & 0xFFFFFFFF) << 32) | bits), name
        out = torch.zeros(4, dtype=torch.int64, device=dev)
        pkg.call(name, pkg.AclTensor(scale.to(dev)), None, pkg.AclTensor(out))
        torch.cuda.synchronize()
        assert torch.equal(out.cpu(), bits), name
    bad = torch.zeros(4, dtype=torch.int32, device=dev)
    assert pkg.call("aclnnTransQuantParam", pkg.AclTensor(scale.to(dev)), None, pkg.AclTensor(bad), return_status=True) == 161002


def test_allreduce_matmuls_without_communicator(pkg, oracle, workloads, dev):
    """The all-reduce forms with comm == NULL give the local result (the reference's one-rank case,
    cuda/src/ops/matmul.cu:1304-1319); they live in libhccl.so and run the operators of libascendcl.so."""
    hccl = os.path.join(os.path.dirname(pkg.LIB_PATH), "libhccl.so")
    if not os.path.exists(hccl):
        pytest.skip("libhccl.so not built")
    d = workloads.w8a8(M=24, K=128, N=64, seed=22, with_pertoken=False, with_bias=False, scale_dtype=torch.float16)
    _, want = ref_qmm(oracle, d, torch.float16)
    x, w, sc = pkg.AclTensor(d["x"].to(dev)), pkg.AclTensor(d["w"].to(dev)), pkg.AclTensor(d["scale"].to(dev))
    dw = workloads.w8a16(M=4, K=256, N=128, dtype=torch.float16, with_offset=True, seed=23)
    wx, ww = pkg.AclTensor(dw["x"].to(dev)), pkg.AclTensor(dw["w"].to(dev))
    ws_, wo = pkg.AclTensor(dw["scale"].to(dev)), pkg.AclTensor(dw["offset"].to(dev))
    with pkg.use_library(hccl):
        for name in ("aclnnQuantMatmulAllReduce", "aclnnQuantMatmulAllReduceV2", "aclnnQuantMatmulAllReduceV3",
                     "aclnnQuantMatmulAllReduceV4"):
            out = torch.empty((24, 64), dtype=torch.float16, device=dev)
            pkg.call(name, x, w, sc, ctypes.c_void_p(None), pkg.AclTensor(out))
            torch.cuda.synchronize()
            assert torch.equal(out.cpu(), want), name
        out = torch.empty((4, 128), dtype=torch.float16, device=dev)
        pkg.call("aclnnWeightQuantMatmulAllReduce", wx, ww, ws_, wo, ctypes.c_void_p(None), pkg.AclTensor(out))
        torch.cuda.synchronize()
    assert_close(to_np(out), ref_wq(oracle, dw), "aclnnWeightQuantMatmulAllReduce, one rank")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_add_rmsnorm_and_the_allreduce_norm_matmul(pkg, oracle, workloads, dev, dtype):
    """aclnnAddRmsNorm (cuda/src/ops/norm_ext.cu:123-139,233-247) against the oracle, with and without
    gamma and with residualSum written over residual; then aclnnQuantMatmulAllReduceAddRmsNorm
    with comm == NULL (the reference's one-rank case, cuda/src/ops/matmul.cu:1222-1233,
    1344-1370): matmul -> residual add -> RMS norm, the partial output kept in the workspace."""
    kind = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}[dtype]
    g = torch.Generator().manual_seed(6600)
    rows, D, eps = 37, 1000, 1e-5
    x, res = torch.randn((rows, D), generator=g).to(dtype), torch.randn((rows, D), generator=g).to(dtype)
    gamma = (torch.rand(D, generator=g) + 0.5).to(dtype)
    for gm in (gamma, None):
        want_y, want_sum = oracle.add_rmsnorm(f32(x), f32(res), None if gm is None else f32(gm), eps, kind)
        y = torch.empty_like(x, device=dev)
        rs = res.to(dev).clone()   # residualSum aliases residual
        pkg.call("aclnnAddRmsNorm", pkg.AclTensor(x.to(dev)), pkg.AclTensor(rs), pkg.AclTensor(gm.to(dev)) if gm is not None else None,
                 ctypes.c_double(eps), pkg.AclTensor(y), pkg.AclTensor(rs))
        torch.cuda.synchronize()
        assert np.array_equal(rs.float().cpu().numpy(), want_sum)
        assert_close(to_np(y), want_y.astype(np.float64), f"aclnnAddRmsNorm {dtype} gamma={gm is not None}")
    bad = torch.empty((rows, D + 1), dtype=dtype, device=dev)
    assert pkg.call("aclnnAddRmsNorm", pkg.AclTensor(x.to(dev)), pkg.AclTensor(res.to(dev)), None, ctypes.c_double(eps),
                    pkg.AclTensor(bad), pkg.AclTensor(res.to(dev)), return_status=True) == 161002

    hccl = os.path.join(os.path.dirname(pkg.LIB_PATH), "libhccl.so")
    if not os.path.exists(hccl) or dtype == torch.float32:
        return
    M, K, N = 24, 128, 128
    d = workloads.w8a8(M=M, K=K, N=N, seed=6601, with_pertoken=False, with_bias=False, scale_dtype=torch.float16)
    acc = oracle.qmm_acc_fast(d["x"].numpy(), d["w"].numpy(), M, K, N)
    mm = torch.from_numpy(oracle.qmm_epilogue_fast(acc, f32(d["scale"]))).to(dtype)   # the partial output, rounded to its type
    res2, gamma2 = torch.randn((M, N), generator=g).to(dtype), (torch.rand(N, generator=g) + 0.5).to(dtype)
    want_y, want_sum = oracle.add_rmsnorm(f32(mm), f32(res2), f32(gamma2), eps, kind)
    tx, tw, tsc = pkg.AclTensor(d["x"].to(dev)), pkg.AclTensor(d["w"].to(dev)), pkg.AclTensor(d["scale"].to(dev))
    y, rs = torch.empty((M, N), dtype=dtype, device=dev), torch.empty((M, N), dtype=dtype, device=dev)
    with pkg.use_library(hccl):
        need = pkg.call("aclnnQuantMatmulAllReduceAddRmsNorm", tx, tw, tsc, pkg.AclTensor(res2.to(dev)), pkg.AclTensor(gamma2.to(dev)),
                        ctypes.c_double(eps), ctypes.c_void_p(None), pkg.AclTensor(y), pkg.AclTensor(rs))
        torch.cuda.synchronize()
    assert need >= M * N * 2
    assert np.array_equal(rs.float().cpu().numpy(), want_sum)
    assert_close(to_np(y), want_y.astype(np.float64), f"aclnnQuantMatmulAllReduceAddRmsNorm {dtype}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 1024), (8, 4096), (300, 8192), (5, 100), (3, 7, 520), (2, 16384), (2, 20000)])
def test_dynamic_quant_bit_exact(pkg, oracle, dev, shape, dtype):
    """Per-token int8 quantiser (cuda/src/ops/quant.cu:37-49,99-111): int8 codes and fp32 scales are
    bit-identical to the oracle for every input type, row length (register-resident, vectorised and
    generic forms) and for all-zero rows; all four names."""
    g = torch.Generator().manual_seed(6000 + shape[-1])
    x = (torch.randn(shape, generator=g) * 3).to(dtype)
    x.view(-1, shape[-1])[0, :] = 0
    want_q, want_s = oracle.dynamic_quant(x.float().numpy())
    for name in ("aclnnDynamicQuant", "aclnnDynamicQuantV2", "aclnnDynamicQuantV3", "aclnnDynamicQuantV4"):
        q, sc = pkg.dynamic_quant(x.to(dev), name=name)
        torch.cuda.synchronize()
        assert np.array_equal(sc.cpu().numpy().reshape(want_s.shape), want_s), name
        assert np.array_equal(q.cpu().numpy(), want_q), name


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("case", [((64, 4096), 32), ((7, 512), 64), ((3, 1024), 128), ((2, 2048), 256), ((5, 96), 48), ((4, 1000), 1000)])
def test_dynamic_mx_quant_bit_exact(pkg, oracle, dev, case, dtype):
    """Block-wise int8 quantiser with power-of-two scales (cuda/src/ops/quant.cu:380-389,496-514): codes and
    scales identical to the oracle for the vectorised block sizes, odd block sizes, zero blocks and blocks
    whose maximum is an exact power of two times 127; both names."""
    shape, block = case
    g = torch.Generator().manual_seed(6200 + block)
    x = (torch.randn(shape, generator=g) * 2).to(dtype)
    flat = x.view(-1, block)
    flat[0, :] = 0
    flat[1, :] = 0.25
    flat[1, 0] = 127.0 * 0.5      # max / 127 = 2^-1 exactly
    want_q, want_s = oracle.dynamic_mx_quant(x.float().numpy(), block)
    for name in ("aclnnDynamicMxQuant", "aclnnDynamicMxQuantV2"):
        q, sc = pkg.dynamic_mx_quant(x.to(dev), block, name=name)
        torch.cuda.synchronize()
        assert np.array_equal(sc.cpu().numpy(), want_s), name
        assert np.array_equal(q.cpu().numpy(), want_q), name
    assert want_s[0] == 1 and want_s[1] == 0.5


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(8, 32), (5, 200), (64, 4096), (3, 2, 8192), (4, 28672), (2, 40000)])
def test_swiglu_quant(pkg, oracle, dev, shape, dtype):
    """SwiGLU fused with the per-token quantiser (cuda/src/ops/glu_ext.cu:89-141), both names, the
    register-resident and the generic form, a zero row.  Scales agree to fp32 rounding of expf; codes are
    equal except where g / scale sits on a rounding boundary (at most 1 apart, under 1 in 1000), and the
    reference's own dequantisation check (tests/test_norm.cpp:152-161) holds."""
    g = torch.Generator().manual_seed(6400 + shape[-1])
    x = (torch.rand(shape, generator=g) * 4 - 2).to(dtype)
    x.view(-1, shape[-1])[0, :] = 0
    want_q, want_s = oracle.swiglu_quant(x.float().numpy())
    D = shape[-1] // 2
    a, b = x.double()[..., :D].numpy(), x.double()[..., D:].numpy()
    gd = a / (1.0 + np.exp(-a)) * b
    for name in ("aclnnSwiGluQuant", "aclnnSwiGluQuantV2"):
        q, sc = pkg.swiglu_quant(x.to(dev), name=name)
        torch.cuda.synchronize()
        q, sc = q.cpu().numpy(), sc.cpu().numpy().reshape(want_s.shape)
        assert np.allclose(sc, want_s, rtol=2e-6, atol=0), name
        diff = np.abs(q.astype(int) - want_q.astype(int))
        assert diff.max() <= 1 and (diff != 0).mean() < 1e-3, (name, diff.max(), (diff != 0).mean())
        assert np.abs(q * sc[..., None].astype(np.float64) - gd).max() / np.abs(gd).max() <= 1e-2, name
        assert (q.reshape(-1, D)[0] == 0).all() and sc.reshape(-1)[0] == 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dequant_swiglu_quant(pkg, oracle, dev, dtype):
    """aclnnDequantSwigluQuant[V2] (cuda/src/ops/norm_ext.cu:1354-1369,1416-1432): a per-row dequant scale
    in front of the SwiGLU quantiser; without the scale it is the plain SwiGLU quantiser, bit for bit."""
    g = torch.Generator().manual_seed(6450)
    x = (torch.rand((33, 2 * 1536), generator=g) * 40 - 20).to(dtype)
    dq = (torch.rand(33, generator=g) * 0.2 + 0.01).float()
    want_q, want_s = oracle.swiglu_quant(x.float().numpy(), dq.numpy())
    for name in ("aclnnDequantSwigluQuant", "aclnnDequantSwigluQuantV2"):
        q, sc = pkg.swiglu_quant(x.to(dev), name=name, dequant_scale=dq.to(dev))
        torch.cuda.synchronize()
        q, sc = q.cpu().numpy(), sc.cpu().numpy()
        assert np.allclose(sc, want_s, rtol=2e-6, atol=0), name
        diff = np.abs(q.astype(int) - want_q.astype(int))
        assert diff.max() <= 1 and (diff != 0).mean() < 1e-3, (name, diff.max(), (diff != 0).mean())
    q0, s0 = pkg.swiglu_quant(x.to(dev), name="aclnnDequantSwigluQuant", dequant_scale=None)
    q1, s1 = pkg.swiglu_quant(x.to(dev))
    torch.cuda.synchronize()
    assert torch.equal(q0, q1) and torch.equal(s0, s1)
    bad = torch.ones(32, dtype=torch.float32, device=dev)
    qb, sb = torch.empty((33, 1536), dtype=torch.int8, device=dev), torch.empty(33, dtype=torch.float32, device=dev)
    assert pkg.call("aclnnDequantSwigluQuant", pkg.AclTensor(x.to(dev)), pkg.AclTensor(bad), pkg.AclTensor(qb), pkg.AclTensor(sb),
                    return_status=True) == 161002


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,with_dq", [((600, 4096), False), ((300, 28672), False), ((320, 2192), True), ((1030, 32768), True)])
def test_swiglu_quant_many_long_rows(pkg, oracle, dev, shape, with_dq, dtype):
    """With at least two rows per SM and D >= 1024 the SwiGLU quantiser runs as persistent CTAs that stage rows
    through shared memory.  Same arithmetic as the one-row-per-CTA form, so the whole call equals, bit for bit, the
    same rows quantised in slices too short for the staged form; and the oracle's tolerance holds.  D = 1096 leaves
    idle lanes in the last warp, D = 16384 is the longest row the staged form takes, a zero row gets scale 1."""
    g = torch.Generator().manual_seed(6600 + shape[0])
    rows, D = shape[0], shape[1] // 2
    x = (torch.rand(shape, generator=g) * 6 - 3).to(dtype)
    x[7, :] = 0
    dq = (torch.rand(rows, generator=g) * 0.5 + 0.25).float() if with_dq else None
    name = "aclnnDequantSwigluQuant" if with_dq else "aclnnSwiGluQuant"
    xd = x.to(dev)
    q, sc = pkg.swiglu_quant(xd, name=name, dequant_scale=dq.to(dev) if with_dq else None)
    for r0 in range(0, rows, 100):
        qs, ss = pkg.swiglu_quant(xd[r0:r0 + 100].contiguous(), name=name, dequant_scale=dq[r0:r0 + 100].to(dev) if with_dq else None)
        assert torch.equal(q[r0:r0 + 100], qs) and torch.equal(sc.reshape(-1)[r0:r0 + 100], ss.reshape(-1)), r0
    torch.cuda.synchronize()
    lib = pkg.load()
    lib.aclnnB200DeviceStatus.restype = ctypes.c_uint32
    assert lib.aclnnB200DeviceStatus() == 0
    take = slice(0, 64)
    want_q, want_s = oracle.swiglu_quant(x[take].float().numpy(), dq[take].numpy() if with_dq else None)
    qh, sh = q[take].cpu().numpy(), sc.reshape(-1)[take].cpu().numpy()
    assert np.allclose(sh, want_s.reshape(-1), rtol=2e-6, atol=0)
    diff = np.abs(qh.astype(int) - want_q.astype(int))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3
    assert (qh[7] == 0).all() and sh[7] == 1


def test_swiglu_quant_feeds_the_w8a8_matmul(pkg, oracle, workloads, dev):
    """gate/up output -> SwiGluQuant -> aclnnQuantMatmulV4 with the scales as pertokenScale: the matmul's
    result is bit-exact for the codes and scales the quantiser produced."""
    g = torch.Generator().manual_seed(6500)
    M, K, N = 40, 1024, 256
    x = torch.randn((M, 2 * K), generator=g).to(torch.bfloat16)
    d = workloads.w8a8(M=M, K=K, N=N, seed=6501, with_pertoken=False)
    q, sc = pkg.swiglu_quant(x.to(dev))
    out = pkg.quant_matmul(q, d["w"].to(dev), d["scale"].to(dev), sc, d["bias"].to(dev), out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    acc = oracle.qmm_acc_fast(q.cpu().numpy(), d["w"].numpy(), M, K, N)
    want = torch.from_numpy(oracle.qmm_epilogue_fast(acc, f32(d["scale"]), sc.cpu().numpy(), d["bias"].numpy())).to(torch.bfloat16)
    assert torch.equal(out.cpu(), want)


def test_dynamic_quant_feeds_the_w8a8_matmul(pkg, oracle, workloads, dev):
    """The chain a W8A8 layer runs: quantise the activations per token, then aclnnQuantMatmulV4 with
    the scales as pertokenScale.  Accumulators and output bit-exact against the oracle's chain."""
    g = torch.Generator().manual_seed(6100)
    M, K, N = 48, 1024, 256
    x = torch.randn((M, K), generator=g).to(torch.bfloat16)
    d = workloads.w8a8(M=M, K=K, N=N, seed=6101, with_pertoken=False)
    q, sc = pkg.dynamic_quant(x.to(dev))
    out = pkg.quant_matmul(q, d["w"].to(dev), d["scale"].to(dev), sc, d["bias"].to(dev), out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    want_q, want_s = oracle.dynamic_quant(x.float().numpy())
    acc = oracle.qmm_acc_fast(want_q, d["w"].numpy(), M, K, N)
    want = torch.from_numpy(oracle.qmm_epilogue_fast(acc, f32(d["scale"]), want_s, d["bias"].numpy())).to(torch.bfloat16)
    assert torch.equal(out.cpu(), want)


def test_c_client_pipelined_pass(pkg, oracle, workloads, dev):
    """The compiled C client the benchmark's end-to-end leg uses (csrc/acl_client.c): copy-in, both phases
    and copy-out per call, overlapped over three streams with two activation and two output buffers.
    After a pass of n calls the host buffer holds call n-1's result: every n from 1 to 5 must give the
    bits of the plain call on that set."""
    path = os.path.join(os.path.dirname(pkg.LIB_PATH), "libqmm_client.so")
    client = ctypes.CDLL(path)
    client.qmmClientWeightQuantPass.restype = ctypes.c_int
    M, K, N, G = 2, 1024, 768, 128
    sets = [workloads.w4a16(M=M, K=K, N=N, group=G, seed=7000 + i, with_offset=False, with_bias=False) for i in range(5)]
    VP = ctypes.c_void_p
    hx = [d["x"].pin_memory() for d in sets]
    hout = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    dxs = [torch.empty((M, K), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    douts = [torch.empty((M, N), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    tdx, tdo = [pkg.AclTensor(t) for t in dxs], [pkg.AclTensor(t) for t in douts]
    w = [d["w"].to(dev) for d in sets]
    sc = [d["scale"].to(dev) for d in sets]
    tw = [pkg.AclTensor(t, pkg.ACL_INT4, (K, N)) for t in w]
    ts = [pkg.AclTensor(t) for t in sc]
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    own_stream = torch.cuda.Stream(dev)   # the legacy default stream cannot be captured
    stream = VP(own_stream.cuda_stream)
    want = [pkg.weight_quant_matmul(d["x"].to(dev), w[i], sc[i], int4=True, group=G).cpu() for i, d in enumerate(sets)]
    torch.cuda.synchronize()
    for n in range(1, 6):
        hout.zero_()
        st = client.qmmClientWeightQuantPass(
            ctypes.c_int(n), (VP * n)(*[VP(h.data_ptr()) for h in hx[:n]]), ctypes.c_size_t(M * K * 2),
            (VP * 2)(*[VP(t.data_ptr()) for t in dxs]), (VP * 2)(*[VP(t.h) for t in tdx]),
            (VP * n)(*[VP(t.h) for t in tw[:n]]), (VP * n)(*[VP(t.h) for t in ts[:n]]), None, None, ctypes.c_int64(G),
            (VP * 2)(*[VP(t.h) for t in tdo]), (VP * 2)(*[VP(t.data_ptr()) for t in douts]), VP(hout.data_ptr()),
            ctypes.c_size_t(M * N * 2), VP(ws.data_ptr()), ctypes.c_uint64(ws.numel()), stream)
        assert st == 0
        assert torch.equal(hout, want[n - 1]), n
    # the same pass captured into a model and replayed: new activations in the same host buffers must
    # come through (the copies are part of the model), three replays give the same bits
    client.qmmClientWeightQuantCapture.restype = ctypes.c_int
    client.qmmClientReplay.restype = ctypes.c_int
    for n in (1, 2, 5):
        model = VP()
        st = client.qmmClientWeightQuantCapture(
            ctypes.c_int(n), (VP * n)(*[VP(h.data_ptr()) for h in hx[:n]]), ctypes.c_size_t(M * K * 2),
            (VP * 2)(*[VP(t.data_ptr()) for t in dxs]), (VP * 2)(*[VP(t.h) for t in tdx]),
            (VP * n)(*[VP(t.h) for t in tw[:n]]), (VP * n)(*[VP(t.h) for t in ts[:n]]), None, None, ctypes.c_int64(G),
            (VP * 2)(*[VP(t.h) for t in tdo]), (VP * 2)(*[VP(t.data_ptr()) for t in douts]), VP(hout.data_ptr()),
            ctypes.c_size_t(M * N * 2), VP(ws.data_ptr()), ctypes.c_uint64(ws.numel()), stream, ctypes.byref(model))
        assert st == 0 and model.value
        for rep in range(3):
            hout.zero_()
            assert client.qmmClientReplay(model, stream) == 0
            assert torch.equal(hout, want[n - 1]), (n, rep)
        saved = hx[n - 1].clone()
        hx[n - 1].copy_(sets[(n + 1) % 5]["x"])   # other activations, same buffer
        want2 = pkg.weight_quant_matmul(hx[n - 1].to(dev), w[n - 1], sc[n - 1], int4=True, group=G).cpu()
        torch.cuda.synchronize()
        assert client.qmmClientReplay(model, stream) == 0
        assert torch.equal(hout, want2), n
        hx[n - 1].copy_(saved)
        assert pkg.load().aclmdlRIDestroy(model) == 0


def test_c_client_step_of_many_calls(pkg, oracle, workloads, dev):
    """The step form of the compiled client (the benchmark's end-to-end leg): n calls, each with its own activation and
    output slice of contiguous host and device blocks, copies in groups on two copy streams beside the matmuls.  Every
    call's result must come back with the bits of the plain call, for group sizes that divide n, do not divide it, and
    exceed it; directly and from a captured model replayed with new activations in the same host block."""
    path = os.path.join(os.path.dirname(pkg.LIB_PATH), "libqmm_client.so")
    client = ctypes.CDLL(path)
    client.qmmClientWeightQuantStep.restype = ctypes.c_int
    client.qmmClientWeightQuantStepCapture.restype = ctypes.c_int
    client.qmmClientReplay.restype = ctypes.c_int
    M, K, N, G, n = 1, 1024, 768, 128, 7
    sets = [workloads.w4a16(M=M, K=K, N=N, group=G, seed=7100 + i, with_offset=False, with_bias=False) for i in range(3)]
    VP = ctypes.c_void_p
    g = torch.Generator().manual_seed(7110)
    hx = torch.randn((n, M, K), generator=g).to(torch.bfloat16).pin_memory()
    hout = torch.empty((n, M, N), dtype=torch.bfloat16).pin_memory()
    dx = torch.empty((n, M, K), dtype=torch.bfloat16, device=dev)
    dout = torch.empty((n, M, N), dtype=torch.bfloat16, device=dev)
    tdx, tdo = [pkg.AclTensor(dx[i]) for i in range(n)], [pkg.AclTensor(dout[i]) for i in range(n)]
    w = [d["w"].to(dev) for d in sets]
    sc = [d["scale"].to(dev) for d in sets]
    tw = [pkg.AclTensor(t, pkg.ACL_INT4, (K, N)) for t in w]
    ts = [pkg.AclTensor(t) for t in sc]
    ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    own_stream = torch.cuda.Stream(dev)
    stream = VP(own_stream.cuda_stream)

    def wanted():
        out = torch.stack([pkg.weight_quant_matmul(hx[i].to(dev), w[i % 3], sc[i % 3], int4=True, group=G) for i in range(n)]).cpu()
        torch.cuda.synchronize()
        return out

    def args(per_group):
        return (ctypes.c_int(n), ctypes.c_int(per_group), VP(hx.data_ptr()), ctypes.c_size_t(M * K * 2), VP(dx.data_ptr()),
                (VP * n)(*[VP(t.h) for t in tdx]), (VP * n)(*[VP(tw[i % 3].h) for i in range(n)]),
                (VP * n)(*[VP(ts[i % 3].h) for i in range(n)]), None, None, ctypes.c_int64(G), (VP * n)(*[VP(t.h) for t in tdo]),
                VP(dout.data_ptr()), VP(hout.data_ptr()), ctypes.c_size_t(M * N * 2), VP(ws.data_ptr()), ctypes.c_uint64(ws.numel()), stream)
    want = wanted()
    for per_group in (1, 3, 7, 50):
        hout.zero_()
        assert client.qmmClientWeightQuantStep(*args(per_group)) == 0
        assert torch.equal(hout, want), per_group
    assert client.qmmClientWeightQuantStep(*((ctypes.c_int(n), ctypes.c_int(0)) + args(1)[2:])) == 161002   # no group size
    model = VP()
    assert client.qmmClientWeightQuantStepCapture(*args(3), ctypes.byref(model)) == 0 and model.value
    for rep in range(2):
        hout.zero_()
        assert client.qmmClientReplay(model, stream) == 0
        assert torch.equal(hout, want), rep
    hx.copy_(torch.randn((n, M, K), generator=g).to(torch.bfloat16))   # other activations in the same host block
    want = wanted()
    assert client.qmmClientReplay(model, stream) == 0
    assert torch.equal(hout, want)
    assert pkg.load().aclmdlRIDestroy(model) == 0


def test_fused_gather_receiver_gives_up_on_a_silent_peer(pkg, dev):
    """The receiver kernel of the fused gather polls the peers' packets with a time limit.  On one GPU, with a window whose
    peer never sends, the poll runs out: the kernel returns, the status word names the peer (0x500 + rank 1), and the
    device keeps working (nothing faulted, nothing hangs)."""
    path = os.path.join(os.path.dirname(pkg.LIB_PATH), "libhccl.so")
    if not os.path.exists(path):
        pytest.skip("libhccl.so not built")
    pkg.load()
    hccl = ctypes.CDLL(path)
    hccl.HcclB200TestReceiverTimeout.restype = ctypes.c_uint32
    hccl.HcclB200P2pStatus.restype = ctypes.c_uint32
    assert hccl.HcclB200TestReceiverTimeout(ctypes.c_uint64(200000)) == 0x501      # 200 us
    assert hccl.HcclB200P2pStatus() == 0                                               # cleared again
    a = torch.arange(1024, device=dev).float().sum().item()                            # the context is alive
    assert a == 1023 * 1024 / 2


def test_capture_replay_of_the_two_phase_call(pkg, oracle, workloads, dev):
    """aclmdlRICaptureBegin / End / ExecuteAsync around quantized matmuls, used like the reference's
    tests/test_graph.cpp:30-78: warm up, capture calls that share a caller-owned workspace (phase 1 runs
    at capture time only), destroy the tensors, replay three times; every replay equals the direct call.
    Covers the decode kernel (two launches), the W8A8 dense kernel and the capture status query."""
    lib = pkg.load()
    VP = ctypes.c_void_p
    own_stream = torch.cuda.Stream(dev)   # the legacy default stream cannot be captured
    stream = VP(own_stream.cuda_stream)
    d = workloads.w4a16(M=4, K=1024, N=512, group=128, seed=7300)
    q = workloads.w8a8(M=200, K=512, N=256, seed=7301)
    dd = {k: v.to(dev) for k, v in d.items() if isinstance(v, torch.Tensor)}
    qd = {k: v.to(dev) for k, v in q.items() if isinstance(v, torch.Tensor)}
    out_wq = torch.empty((4, 512), dtype=torch.bfloat16, device=dev)
    out_q = torch.empty((200, 256), dtype=torch.bfloat16, device=dev)

    def both():   # device tensors only, no allocation, no synchronisation: legal inside a capture
        pkg.weight_quant_matmul(dd["x"], dd["w"], dd["scale"], dd.get("offset"), dd.get("bias"), int4=True, group=128, out=out_wq,
                                stream=own_stream.cuda_stream)
        pkg.quant_matmul(qd["x"], qd["w"], qd["scale"], qd["pertoken"], qd["bias"], out=out_q, stream=own_stream.cuda_stream)

    both()   # warm-up: sizes the shared workspace, sets kernel attributes
    torch.cuda.synchronize()
    direct_wq, direct_q = out_wq.clone(), out_q.clone()
    assert_close(to_np(direct_wq), ref_wq(oracle, d), "captured W4A16 case, direct")
    status = ctypes.c_int(-1)
    assert lib.aclmdlRICaptureGetInfo(stream, ctypes.byref(status), None) == 0 and status.value == 0
    assert lib.aclmdlRICaptureBegin(stream, ctypes.c_int(2)) == 0
    assert lib.aclmdlRICaptureGetInfo(stream, ctypes.byref(status), None) == 0 and status.value == 1
    both()
    model = VP()
    assert lib.aclmdlRICaptureEnd(stream, ctypes.byref(model)) == 0 and model.value
    assert lib.aclmdlRICaptureEnd(stream, None) == 161001
    for _ in range(3):
        out_wq.zero_(); out_q.zero_()
        torch.cuda.synchronize()   # the zeroing ran on another stream
        assert lib.aclmdlRIExecuteAsync(model, stream) == 0
        torch.cuda.synchronize()
        assert torch.equal(out_wq, direct_wq) and torch.equal(out_q, direct_q)
    assert lib.aclmdlRIExecuteAsync(None, stream) == 161001
    assert lib.aclmdlRIDestroy(model) == 0


def test_seeded_random_shapes_default_path_against_generic_kernel(pkg, workloads, dev):
    """Seeded random shapes through whatever kernel the library picks (decode kernel with its whole-tile
    and share-aligned schedules, streaming kernel in both modes and tile heights, expansion + dense,
    row-tile dense) against the bounds-checked generic kernel on the same device: W8A8 bit for bit,
    weight-only within the output bounds (the two sum in different orders)."""
    rng = np.random.default_rng(20240607)
    for case in range(36):
        kind = ("w4g", "w4c", "w8c", "i8")[case % 4]
        M = int(rng.choice([1, 3, 8, 13, 16, 17, 31, 40, 64, 77, 128, 130, 200, 333]))
        K = int(rng.integers(1, 17)) * 128 * (2 if kind == "w4g" else 1)
        N = int(rng.integers(1, 40)) * 32 * int(rng.choice([1, 1, 1, 9]))
        if kind == "i8":
            d = workloads.w8a8(M=M, K=K, N=N, seed=9000 + case)
            args = [d[k].to(dev) for k in ("x", "w", "scale", "pertoken", "bias")]
            got = pkg.quant_matmul(*args, out_dtype=torch.bfloat16)
            with forced_path("generic"):
                want = pkg.quant_matmul(*args, out_dtype=torch.bfloat16)
            torch.cuda.synchronize()
            assert torch.equal(got, want), (case, kind, M, K, N)
            continue
        dtype = torch.bfloat16 if case % 8 < 4 else torch.float16
        if kind == "w4g":
            d = workloads.w4a16(M=M, K=K, N=N, group=int(rng.choice([128, 256])), dtype=dtype, seed=9000 + case,
                                with_offset=bool(case & 1), with_bias=bool(case & 2))
        elif kind == "w4c":
            d = workloads.w4a16(M=M, K=K, N=N, dtype=dtype, per_channel=True, seed=9000 + case, with_bias=bool(case & 2))
        else:
            d = workloads.w8a16(M=M, K=K, N=N, dtype=dtype, with_offset=bool(case & 1), seed=9000 + case)
        got = run_wq(pkg, d, dev)
        with forced_path("generic"):
            want = run_wq(pkg, d, dev)
        assert_close(to_np(got), to_np(want).astype(np.float64), f"case {case} {kind} M={M} K={K} N={N} {dtype}")


def test_a_wait_that_runs_out_is_reported_and_latched(pkg, oracle, workloads, dev):
    """Failure detection without a fault: a test hook makes one CTA of the decode kernel leave out the copy of its
    first stage, so its consumers wait for a barrier that nothing completes; with the wait limit set to 200 us (a
    second test hook) the wait runs out, the kernel comes back by itself, the context stays usable,
    aclnnB200DeviceStatus() names the wait, and from then on matmul calls are refused with 361001 until
    aclnnB200ResetDeviceStatus(); after the reset the same call gives the right result."""
    lib = pkg.load()
    lib.aclnnB200DeviceStatus.restype = ctypes.c_uint32
    lib.aclnnB200ResetDeviceStatus.restype = None
    d = workloads.w4a16(M=2, K=4096, N=1024, group=128, seed=8700)
    args = (d["x"].to(dev), d["w"].to(dev), d["scale"].to(dev), d["offset"].to(dev), d["bias"].to(dev))
    torch.cuda.synchronize()
    assert lib.aclnnB200DeviceStatus() == 0
    try:
        with env_set("B200_QMM_TEST_WAIT_LIMIT_NS", "200000"), env_set("B200_QMM_TEST_DROP_STAGE", "1"):
            pkg.weight_quant_matmul(*args, int4=True, group=128)     # launches; CTA 0's wait for its first stage runs out
        torch.cuda.synchronize()                                     # the kernel returned by itself
        code = lib.aclnnB200DeviceStatus()
        assert 0x300 <= code < 0x400, hex(code)                      # a wait of the decode kernel
        out = torch.empty((2, 1024), dtype=torch.bfloat16, device=dev)
        st = pkg.call("aclnnWeightQuantBatchMatmulV2Ex", pkg.AclTensor(args[0]), pkg.AclTensor(args[1], pkg.ACL_INT4, (4096, 1024)),
                      pkg.AclTensor(args[2]), pkg.AclTensor(args[3]), pkg.AclTensor(args[4]), ctypes.c_int64(128), pkg.AclTensor(out),
                      return_status=True)
        assert st == 361001
        q = workloads.w8a8(M=8, K=64, N=32, seed=8701)
        assert pkg.call("aclnnQuantMatmulV4", pkg.AclTensor(q["x"].to(dev)), pkg.AclTensor(q["w"].to(dev)), pkg.AclTensor(q["scale"].to(dev)),
                        pkg.AclTensor(torch.empty((8, 32), dtype=torch.bfloat16, device=dev)), return_status=True) == 361001
    finally:
        lib.aclnnB200ResetDeviceStatus()
    assert lib.aclnnB200DeviceStatus() == 0
    got = pkg.weight_quant_matmul(*args, int4=True, group=128)
    torch.cuda.synchronize()
    assert_close(to_np(got), ref_wq(oracle, d), "after the reset")


def test_zz_no_bounded_wait_gave_up(pkg, dev):
    """Every spin inside the tensor-core kernels is bounded and records a code when it gives up;
    after the whole suite the device status word must still be 0."""
    lib = pkg.load()
    lib.aclnnB200DeviceStatus.restype = ctypes.c_uint32
    torch.cuda.synchronize()
    assert lib.aclnnB200DeviceStatus() == 0
