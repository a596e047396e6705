"""Generates tests/golden/gemm_golden.npz: small seeded inputs for every operator of the GEMM
path with expected results computed independently of the C oracle (numpy float64 / exact
integer arithmetic, torch's own bf16 and float8_e4m3fn conversions).

The reference (open64-compiler/open64) ships no golden vectors for a matrix product, so these
fixtures pin the oracle against an independent computation, not against the reference.

    python tests/golden/make_golden.py
"""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits16(t):
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def main():
    g = torch.Generator().manual_seed(20240607)
    out = {}

    # C1-mini: fp32 fused linear, ReLU
    A = torch.rand(48, 56, generator=g) * 2 - 1
    B = torch.rand(56, 40, generator=g) * 2 - 1
    bias = (torch.rand(40, generator=g) * 2 - 1) * 0.1
    out["c1_A"], out["c1_B"], out["c1_bias"] = A.numpy(), B.numpy(), bias.numpy()
    out["c1_Y"] = np.maximum(A.double().numpy() @ B.double().numpy() + bias.double().numpy(), 0.0)

    # C2-mini: bf16 NT
    A = torch.randn(64, 96, generator=g).to(torch.bfloat16)
    B = torch.randn(48, 96, generator=g).to(torch.bfloat16)
    out["c2_A"], out["c2_B"] = bits16(A), bits16(B)
    out["c2_C"] = A.double().numpy() @ B.double().numpy().T

    # C3-mini: SwiGLU
    X = torch.randn(32, 64, generator=g).to(torch.bfloat16)
    Wg = (torch.randn(64, 48, generator=g) * 0.2).to(torch.bfloat16)
    Wu = (torch.randn(64, 48, generator=g) * 0.2).to(torch.bfloat16)
    gd = X.double() @ Wg.double()
    ud = X.double() @ Wu.double()
    out["c3_X"], out["c3_Wg"], out["c3_Wu"] = bits16(X), bits16(Wg), bits16(Wu)
    out["c3_H"] = (gd / (1 + torch.exp(-gd)) * ud).numpy()

    # C4-mini: fp8 e4m3 scaled
    Af = torch.randn(40, 64, generator=g)
    Wf = torch.randn(24, 64, generator=g)
    sA = (Af.abs().amax(1) / 448).float()
    sB = (Wf.abs().amax(1) / 448).float()
    A8 = (Af / sA[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    W8 = (Wf / sB[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    b4 = (torch.rand(24, generator=g) * 2 - 1) * 0.1
    out["c4_A8"] = A8.view(torch.uint8).numpy().copy()
    out["c4_B8"] = W8.view(torch.uint8).numpy().copy()
    out["c4_sA"], out["c4_sB"], out["c4_bias"] = sA.numpy(), sB.numpy(), b4.numpy()
    out["c4_C"] = ((A8.double() * sA.double()[:, None]) @ (W8.double() * sB.double()[:, None]).T
                   + b4.double()).numpy()

    # C5-mini: int8 -> int32, exact
    A = torch.randint(-127, 128, (40, 200), generator=g, dtype=torch.int8)
    B = torch.randint(-127, 128, (56, 200), generator=g, dtype=torch.int8)
    out["c5_A"], out["c5_B"] = A.numpy(), B.numpy()
    out["c5_C"] = (A.to(torch.int64) @ B.to(torch.int64).T).to(torch.int32).numpy()

    # strided alpha/beta kernel: column-major A (m x k), transposed B passed by swapped
    # increments, row-major C
    m, n, k = 19, 13, 17
    a = torch.randn(m * k, generator=g)          # A(i,l) = a[i + l*m]
    b = torch.randn(n * k, generator=g)          # B(l,j) = b[j*k + l]   (inc1b=1, inc2b=k)
    c = torch.randn(m * n, generator=g)          # C(i,j) = c[i*n + j]   (inc1c=n, inc2c=1)
    Am = a.view(k, m).t().double()
    Bm = b.view(n, k).t().double()
    Cm = c.view(m, n).double()
    out["x_a"], out["x_b"], out["x_c"] = a.numpy(), b.numpy(), c.numpy()
    out["x_mnk"] = np.array([m, n, k], np.int32)
    out["x_alpha_beta"] = np.array([1.25, -0.5], np.float32)
    out["x_C"] = (1.25 * Am @ Bm - 0.5 * Cm).numpy()
    xv = torch.randn(k, generator=g)
    yv = torch.randn(m, generator=g)
    out["v_x"], out["v_y"] = xv.numpy(), yv.numpy()
    out["v_Y"] = (0.75 * Am @ xv.double() + 2.0 * yv.double()).numpy()

    # known answers for the element codecs
    codes = torch.arange(256, dtype=torch.uint8)
    out["e4m3_decode"] = codes.view(torch.float8_e4m3fn).float().numpy()
    probe = torch.tensor([0.0, -0.0, 1.0, -1.0, 448.0, 460.0, 1e9, -1e9, 2.0 ** -9, 2.0 ** -10,
                          1.5 * 2.0 ** -10, 0.0009765625, 0.017, 0.3, 1.0625, 1.1875, 240.0, 232.0,
                          3.1415926, -7.77], dtype=torch.float32)
    out["e4m3_probe"] = probe.numpy()
    out["e4m3_encode"] = probe.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy().copy()
    ties = torch.tensor([1.0, 1.00390625, 1.01171875, 1.0 + 2.0 ** -9, 3.3895314e38, -2.5, 1e-40,
                         65504.0, 0.1, -0.3], dtype=torch.float32)
    out["bf16_probe"] = ties.numpy()
    out["bf16_encode"] = bits16(ties.to(torch.bfloat16))

    np.savez_compressed(os.path.join(HERE, "gemm_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "gemm_golden.npz"), sum(v.nbytes for v in out.values()), "bytes raw")


if __name__ == "__main__":
    main()
