"""Shared helpers of the GPU parity tests."""
import numpy as np

# Tolerances of the floating-point outputs (fp16 / bf16 / fp32), as stated for this path:
# normalised max error max|err|/max|ref| <= 1e-2 (the reference's own metric, tests/harness.h:49-53)
# and mean|err|/mean|ref| <= 2e-3.
MAX_REL = 1e-2
MEAN_REL = 2e-3


def errors(got, ref):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    d = np.abs(got - ref)
    return d.max() / (np.abs(ref).max() + 1e-30), d.mean() / (np.abs(ref).mean() + 1e-30)


def assert_close(got, ref, what="", max_rel=MAX_REL, mean_rel=MEAN_REL):
    mx, mean = errors(got, ref)
    assert mx <= max_rel and mean <= mean_rel, f"{what}: max_rel={mx:.3e} (<= {max_rel}), mean_rel={mean:.3e} (<= {mean_rel})"
    return mx, mean


def to_np(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def f32(t):
    return None if t is None else t.float().numpy()


def dev_or_none(t, dev):
    return None if t is None else t.to(dev)
