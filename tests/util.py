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


def nz_layout_model(w_vals):
    """The tile-packed int4 layout as plain index arithmetic: int values [K,N] in -8..7 -> uint32 words.
    Blocks of 4096 words per (tile of 256 columns, stage of 128 rows), tile-major; inside a block
    [wq = 64 columns][st = 16 rows][lane = 4 g + t][r]; word r of lane (g, t) holds columns
    c + 2r, c + 2r + 1 (c = 256 tile + 64 wq + 8 g) at rows k + 2t + {0, 1, 8, 9} (k = 128 stage + 16 st):
    nibble 0 / 4 = column 2r at rows 2t / 2t+1, 1 / 5 = column 2r+1, 2 / 6 and 3 / 7 the same 8 rows on."""
    K, N = w_vals.shape
    tiles, num_sb = (N + 255) // 256, (K + 127) // 128
    pad = np.zeros((num_sb * 128, tiles * 256), dtype=np.uint32)
    pad[:K, :N] = w_vals.astype(np.int64) & 0xF
    v = pad.reshape(num_sb, 8, 2, 4, 2, tiles, 4, 8, 4, 2)   # [sb][st][half8][t][j] x [tile][wq][g][r][dc]
    words = np.zeros((tiles, num_sb, 4, 8, 8, 4, 4), dtype=np.uint32)   # [tile][sb][wq][st][g][t][r]
    for nib in range(8):
        dc, j, half = nib & 1, (nib >> 2) & 1, (nib >> 1) & 1
        src = v[:, :, half, :, j, :, :, :, :, dc]          # [sb][st][t][tile][wq][g][r]
        words |= src.transpose(3, 0, 4, 1, 5, 2, 6) << np.uint32(4 * nib)
    return words.reshape(-1)
