"""Cases the reference's own CUDA backend accepts on this path, shared by the script that records
its outputs on a B200 (make_ref_fixtures.py) and by the tests that replay them.

The reference takes fp16 activations, per-channel [N] scales, fp16/fp32 outputs and same-kind MX
operands only (cuda/src/ops/matmul.cu:761-767,802-807,437,491), so these are the closest runnable
forms of the benchmark configurations; inputs are regenerated from the seeds in workloads.py.
"""
import torch

WQ_CASES = {
    # name: (generator, kwargs)
    "wq8_cfg0_m1": ("w8a16", dict(M=1, K=1024, N=3072, dtype=torch.float16, seed=1000)),
    "wq8_m4_off": ("w8a16", dict(M=4, K=256, N=64, dtype=torch.float16, seed=2001, with_offset=True)),
    "wq8_m128_off": ("w8a16", dict(M=128, K=256, N=64, dtype=torch.float16, seed=2002, with_offset=True)),
    "wq4_m1": ("w4a16", dict(M=1, K=512, N=256, dtype=torch.float16, seed=2003, per_channel=True, with_bias=False)),
    "wq4_m16": ("w4a16", dict(M=16, K=512, N=256, dtype=torch.float16, seed=2004, per_channel=True, with_bias=False)),
    "wq4_m128": ("w4a16", dict(M=128, K=512, N=256, dtype=torch.float16, seed=2005, per_channel=True, with_bias=False)),
}
QMM_CASES = {
    "qmm_f16": dict(M=128, K=256, N=64, seed=2010, out_dtype=torch.float16, with_pertoken=False, with_bias=False,
                    scale_dtype=torch.float16),
    "qmm_f32": dict(M=96, K=512, N=128, seed=2011, out_dtype=torch.float32, with_pertoken=False, with_bias=False,
                    scale_dtype=torch.float16),
}
MX_CASES = {
    # name: (entry point, kwargs)
    "mxfp8_fn": ("aclnnMatmulMxFp8", dict(M=128, K=256, N=64, a_fp4=False, b_fp4=False, seed=2020)),
    "mxfp8_hw": ("aclnnMatmulMxFp8Hw", dict(M=256, K=256, N=128, a_fp4=False, b_fp4=False, seed=2021)),
    "mxfp4_fn": ("aclnnMatmulMxFp4", dict(M=64, K=128, N=64, a_fp4=True, b_fp4=True, seed=2022)),
}
CAST_N = 4096
CAST_SEED = 2030


def cast_input():
    g = torch.Generator()
    g.manual_seed(CAST_SEED)
    return (torch.rand(CAST_N, generator=g) * 14 - 7).float()
