"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

No dataset or model weight is involved: the configurations name layer shapes only (Qwen3-0.6B MLP
up-projection, Llama-70B gate/up/down projections).  Every generator draws from
torch.Generator().manual_seed(1000 + config index [+ variant]) on the CPU, so the device path and
the CPU checker read identical bytes.
"""
import torch


def _gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def _uniform(g, shape, lo, hi, dtype):
    return (torch.rand(shape, generator=g) * (hi - lo) + lo).to(dtype)


def pack_int4(vals):
    """int8 values in [-8,7], any shape -> packed bytes, two per byte, even linear index = low nibble."""
    v = (vals.reshape(-1).to(torch.int16) & 0xF).to(torch.uint8)
    return (v[0::2] | (v[1::2] << 4)).contiguous()


def w8a16(M=1, K=1024, N=3072, dtype=torch.float16, seed=1000, with_offset=False):
    """Config 0: W8A16 per-channel, Qwen3-0.6B MLP up-projection shape."""
    g = _gen(seed)
    d = {"M": M, "K": K, "N": N, "int4": False, "group": 0}
    d["x"] = torch.randn((M, K), generator=g).to(dtype)
    d["w"] = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8)
    d["scale"] = _uniform(g, (N,), 0.005, 0.02, dtype)
    d["offset"] = _uniform(g, (N,), -1, 1, dtype) if with_offset else None
    d["bias"] = None
    return d


def w4a16(M=16, K=4096, N=4096, group=128, dtype=torch.bfloat16, seed=1001, with_offset=True, with_bias=True,
          per_channel=False):
    """Config 1 (and, with other K/N, config 4): W4A16 group-wise."""
    g = _gen(seed)
    d = {"M": M, "K": K, "N": N, "int4": True, "group": 0 if per_channel else group}
    d["x"] = torch.randn((M, K), generator=g).to(dtype)
    vals = torch.randint(-8, 8, (K, N), generator=g, dtype=torch.int8)
    d["w_vals"] = vals
    d["w"] = pack_int4(vals)
    sshape = (N,) if per_channel else (K // group, N)
    d["scale"] = _uniform(g, sshape, 0.002, 0.01, dtype)
    d["offset"] = _uniform(g, sshape, -1, 1, dtype) if with_offset else None
    d["bias"] = (torch.randn((N,), generator=g) * 0.02).to(dtype) if with_bias else None
    return d


def w8a8(M=2048, K=4096, N=14336, seed=1002, out_dtype=torch.bfloat16, with_pertoken=True, with_bias=True,
         scale_dtype=torch.float32):
    """Config 2: W8A8 with per-token x per-channel dequant epilogue and int32 bias."""
    g = _gen(seed)
    d = {"M": M, "K": K, "N": N, "out_dtype": out_dtype}
    d["x"] = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    d["w"] = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8)
    d["pertoken"] = _uniform(g, (M,), 0.001, 0.01, torch.float32) if with_pertoken else None
    d["scale"] = _uniform(g, (N,), 0.001, 0.01, scale_dtype)
    d["bias"] = torch.randint(-1000, 1001, (N,), generator=g, dtype=torch.int32) if with_bias else None
    return d


_E2M1_BOUNDS = torch.tensor([0.4375, 0.875, 1.25000012, 1.75, 2.50000024, 3.5, 5.00000048], dtype=torch.float32)


def encode_e2m1(v):
    """fp32 -> fp4 e2m1 codes (uint8, one per element) with the reference's boundaries
    (cuda/src/ops/subfp.cuh:44 of the reference); saturates to +-6."""
    c = torch.bucketize(v.abs().contiguous(), _E2M1_BOUNDS, right=True).to(torch.uint8)
    return c | ((v < 0) | ((v == 0) & torch.signbit(v))).to(torch.uint8) << 3


def mx(M=4096, K=8192, N=8192, a_fp4=False, b_fp4=True, seed=1003):
    """Config 3: MXFP8 e4m3 A x MXFP4 e2m1 B, e8m0 scales per 32 K-elements with exponents uniform in
    [-4,4]; values N(0,1) divided by the block scale and then quantised."""
    g = _gen(seed)
    d = {"M": M, "K": K, "N": N, "a_fp4": a_fp4, "b_fp4": b_fp4}
    a = torch.randn((M, K), generator=g)
    b = torch.randn((K, N), generator=g)
    ea = torch.randint(-4, 5, (M, K // 32), generator=g)
    eb = torch.randint(-4, 5, (K // 32, N), generator=g)
    d["sa"] = (ea + 127).to(torch.uint8)
    d["sb"] = (eb + 127).to(torch.uint8)
    a_scaled = a / torch.exp2(ea.float()).repeat_interleave(32, dim=1)
    b_scaled = b / torch.exp2(eb.float()).repeat_interleave(32, dim=0)

    def enc(v, fp4):
        if fp4:
            codes = encode_e2m1(v).reshape(-1)
            return (codes[0::2] | (codes[1::2] << 4)).contiguous()
        return v.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()

    d["a"] = enc(a_scaled, a_fp4)
    d["b"] = enc(b_scaled, b_fp4)
    return d


def llama70b_shard(M, which, n_shards=1, shard=0, dtype=torch.bfloat16, seed=1004):
    """Config 4: one column shard of a Llama-70B-shaped W4A16 group-128 projection.
    which = "gate_up" (K=8192, N=28672) or "down" (K=28672, N=8192); N is split in equal contiguous
    column blocks, the activations are replicated."""
    K, N = (8192, 28672) if which == "gate_up" else (28672, 8192)
    assert N % n_shards == 0 and (N // n_shards) % 2 == 0
    Ns = N // n_shards
    # x is the same on every rank; the weight shard has its own stream of the generator and does not
    # depend on M (the shard is drawn as an M = 1 problem, then given its activations).
    d = w4a16(M=1, K=K, N=Ns, group=128, dtype=dtype, seed=seed * 100 + shard, with_offset=False, with_bias=False)
    d["M"] = M
    d["x"] = torch.randn((M, K), generator=_gen(seed)).to(dtype)
    d["N_total"] = N
    return d


def shard_columns(d, n_shards, shard):
    """Column shard `shard` of `n_shards` of a weight-only problem: rank r owns
    weight[:, r*N/g:(r+1)*N/g] with the matching scale / offset / bias slices as separate contiguous
    tensors; activations are replicated.  Shard boundaries fall on even columns so a packed int4 byte
    never straddles two ranks."""
    K, N = d["K"], d["N"]
    assert N % n_shards == 0 and (N // n_shards) % 2 == 0
    ns = N // n_shards
    lo, hi = shard * ns, (shard + 1) * ns
    out = dict(d, N=ns)
    if d["int4"]:
        out["w"] = d["w"].reshape(K, N // 2)[:, lo // 2:hi // 2].contiguous().reshape(-1)
        if "w_vals" in d:
            out["w_vals"] = d["w_vals"][:, lo:hi].contiguous()
    else:
        out["w"] = d["w"][:, lo:hi].contiguous()
    for k in ("scale", "offset", "bias"):
        if d.get(k) is not None:
            out[k] = d[k][..., lo:hi].contiguous()
    return out


def interleave_gathered(gathered, n_shards, M, N):
    """An all-gather returns the shards rank-major, [g][M][N/g]; the [M,N] matrix is their interleave
    along columns (identical only for M = 1)."""
    return gathered.reshape(n_shards, M, N // n_shards).permute(1, 0, 2).reshape(M, N).contiguous()
