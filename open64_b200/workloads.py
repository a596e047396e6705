"""Seeded synthetic inputs for the five benchmark configurations (all data is synthetic; no
dataset or checkpoint is involved).  Tensors are drawn on the CPU with a fixed generator so
that every host and every rank sees identical values, then moved by the caller.

  C1  fp32 fused linear  Y = ReLU(A B + bias), 512^3, A,B ~ U(-1,1), bias ~ U(-0.1,0.1)   seed 1001
  C2  bf16 NT GEMM       8192^3, N(0,1) rounded to bf16                                    seed 1002
  C3  SwiGLU MLP         x [4096,4096] N(0,1); Wg, Wu [4096,14336], Wd [14336,4096] N(0,0.02)   seed 1003
  C4  fp8 e4m3 scaled    M=4096, N=K=8192; per-row / per-output-channel scale = amax/448   seed 1004
  C5  int8 W8A8          M=16384, N=K=8192, uniform integers in [-127,127]                 seed 1005
"""
import torch

SEEDS = {"c1": 1001, "c2": 1002, "c3": 1003, "c4": 1004, "c5": 1005}


def _gen(seed):
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def c1_linear_f32(M=512, N=512, K=512, seed=SEEDS["c1"]):
    g = _gen(seed)
    A = torch.rand((M, K), generator=g) * 2 - 1
    B = torch.rand((K, N), generator=g) * 2 - 1
    bias = (torch.rand((N,), generator=g) * 2 - 1) * 0.1
    return A, B, bias


def c2_gemm_bf16(M=8192, N=8192, K=8192, seed=SEEDS["c2"]):
    g = _gen(seed)
    A = torch.randn((M, K), generator=g).to(torch.bfloat16)
    B = torch.randn((N, K), generator=g).to(torch.bfloat16)
    return A, B


def c3_swiglu(T=4096, D=4096, F=14336, seed=SEEDS["c3"]):
    g = _gen(seed)
    x = torch.randn((T, D), generator=g).to(torch.bfloat16)
    Wg = (torch.randn((D, F), generator=g) * 0.02).to(torch.bfloat16)
    Wu = (torch.randn((D, F), generator=g) * 0.02).to(torch.bfloat16)
    Wd = (torch.randn((F, D), generator=g) * 0.02).to(torch.bfloat16)
    return x, Wg, Wu, Wd


def quantize_e4m3_rows(x):
    """Per-row scale = amax/448; q = clamp(x/scale, +-448) rounded to e4m3 (saturating)."""
    amax = x.abs().amax(dim=1).clamp_min(1e-12)
    scale = (amax / 448.0).to(torch.float32)
    q = (x / scale[:, None]).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    return q, scale


def c4_fp8(M=4096, N=8192, K=8192, seed=SEEDS["c4"]):
    g = _gen(seed)
    A = torch.randn((M, K), generator=g)
    W = torch.randn((N, K), generator=g)
    bias = (torch.rand((N,), generator=g) * 2 - 1) * 0.1
    A8, sA = quantize_e4m3_rows(A)
    W8, sB = quantize_e4m3_rows(W)
    return A8, W8, sA, sB, bias


def c5_int8(M=16384, N=8192, K=8192, seed=SEEDS["c5"]):
    g = _gen(seed)
    A = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    B = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    return A, B


def shard_rows(B, rank, world):
    """The [N/g, K] slab of a [N,K] weight that rank `rank` of `world` owns."""
    N = B.shape[0]
    if N % world:
        raise ValueError("N must divide by the number of ranks")
    ns = N // world
    return B[rank * ns:(rank + 1) * ns]


# algorithmic work per call: flops = 2 M N K; bytes = each operand read once + result written once
def work(M, N, K, in_bytes, out_bytes, extra_bytes=0):
    return 2 * M * N * K, (M * K + N * K) * in_bytes + M * N * out_bytes + extra_bytes
