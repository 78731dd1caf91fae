"""Generates tests/golden/*.npz: seeded inputs and the oracle's outputs for small cases.

The reference ships no golden vectors (its tests draw unseeded inputs and compare with torch),
and it cannot be executed where this repository is developed, so these vectors come from
oracle/pure_oracle.py, whose agreement with the reference's own comparators is what
tests/test_oracle_pins.py checks. Run from the repository root:

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import pure_oracle as po  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def rng(seed):
    return np.random.default_rng(seed)


def save(name, **arrays):
    np.savez_compressed(os.path.join(OUT, name + ".npz"),
                        **{k: np.asarray(v, dtype=np.float32) if not isinstance(v, (int, np.integer)) else v
                           for k, v in arrays.items()})


def main():
    torch.set_num_threads(1)  # bit-reproducible accumulation order
    r = rng(0)
    # Softmax / LogSoftmax: the reference's test shape [2,4,10], N(0, 10^2), axis 0 and -1,
    # plus rows that exercise the vector, scalar and CTA-per-row kernels.
    for tag, shape, axis, scale in [("t2x4x10_ax0", (2, 4, 10), 0, 10.0), ("t2x4x10_axm1", (2, 4, 10), -1, 10.0),
                                    ("r7x512", (7, 512), -1, 2.0), ("r5x1000", (5, 1000), -1, 2.0),
                                    ("r3x3", (3, 3), -1, 2.0), ("r2x1", (2, 1), -1, 2.0),
                                    ("r3x4100", (3, 4100), -1, 2.0), ("t3x5x4_ax1", (3, 5, 4), 1, 2.0)]:
        x = (r.standard_normal(shape) * scale).astype(np.float32)
        save("softmax_" + tag, x=x, axis=axis, y=po.Softmax(x, axis).numpy(), ylog=po.LogSoftmax(x, axis).numpy())
    # LayerNorm chain: BERT eps, widths 768 / 1024 / odd.
    for tag, shape in [("r9x768", (9, 768)), ("r4x1024", (4, 1024)), ("r5x10", (5, 10)), ("r3x1000", (3, 1000)),
                       ("r2x3x100", (2, 3, 100))]:
        x = r.standard_normal(shape).astype(np.float32)
        g = (1 + 0.1 * r.standard_normal(shape[-1])).astype(np.float32)
        b = (0.1 * r.standard_normal(shape[-1])).astype(np.float32)
        save("layernorm_" + tag, x=x, gamma=g, beta=b, eps=np.float32(1e-12),
             y=po.LayerNormChain(x, g, b, np.float32(1e-12)).numpy(),
             mean=po.ReduceMean(x, [-1], 1).numpy())
    # MatMul / Gemm: the reference's [2,4]@[4,3]; batched broadcasting; tile-tail shapes.
    for tag, sa, sb in [("2x4_4x3", (2, 4), (4, 3)), ("b3_5x8_8x6", (3, 5, 8), (3, 8, 6)),
                        ("bcast_2x3x7x16_16x12", (2, 3, 7, 16), (16, 12)), ("130x72_72x260", (130, 72), (72, 260)),
                        ("bh_2x2x40x64_64x40", (2, 2, 40, 64), (2, 2, 64, 40))]:
        a = r.random(sa).astype(np.float32)
        b = r.random(sb).astype(np.float32)
        save("matmul_" + tag, A=a, B=b, Y=po.MatMul(a, b).numpy())
    for tag, m, k, n in [("c1_l1", 33, 784, 120), ("c1_l2", 33, 120, 32), ("c1_l3", 33, 32, 10), ("k36", 140, 36, 72)]:
        a = r.standard_normal((m, k)).astype(np.float32)
        w = (r.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32)
        c = r.standard_normal(n).astype(np.float32)
        save("gemm_" + tag, A=a, B=w, C=c, Y=po.Gemm(a, w, c).numpy())
    # Conv: the reference's (Cin, k, Cout, bias) cases on 32x32 (batch reduced to 2), and pad 1.
    for tag, cin, k, cout, bias, pad, hw in [("1_3_8_b", 1, 3, 8, True, 0, 32), ("8_3_3", 8, 3, 3, False, 0, 32),
                                             ("8_5_3_b", 8, 5, 3, True, 0, 32), ("8_4_3", 8, 4, 3, False, 0, 32),
                                             ("64_3_64_b_p1", 64, 3, 64, True, 1, 16),
                                             ("32_3_16_b_p1", 32, 3, 16, True, 1, 11)]:
        x = r.random((2, cin, hw, hw)).astype(np.float32)
        w = ((r.random((cout, cin, k, k)) * 2 - 1) / np.sqrt(cin * k * k)).astype(np.float32)
        b = ((r.random(cout) * 2 - 1) / np.sqrt(cin * k * k)).astype(np.float32) if bias else None
        y = po.Conv(x, w, b, pads=(pad,) * 4).numpy()
        kw = dict(X=x, W=w, Y=y, pad=pad)
        if bias:
            kw["B"] = b
        save("conv_" + tag, **kw)
    # Elementwise + chains.
    x = r.standard_normal((6, 40)).astype(np.float32)
    row = r.standard_normal(40).astype(np.float32)
    col = r.standard_normal((6, 1)).astype(np.float32)
    pos = (r.random((6, 40)) + 0.1).astype(np.float32)
    save("eltwise", x=x, row=row, col=col, pos=pos, add_row=po.Add(x, row).numpy(), sub_col=po.Sub(x, col).numpy(),
         mul_full=po.Mul(x, pos).numpy(), div_full=po.Div(x, pos).numpy(), pow2=po.Pow(x, 2.0).numpy(),
         pow_full=po.Pow(pos, x).numpy(), sqrt=po.Sqrt(pos).numpy(), erf=po.Erf(x).numpy(), relu=po.Relu(x).numpy(),
         gelu=po.GeluChain(x).numpy(), add_scalar=po.Add(col, np.float32(1e-12)).numpy())
    # One small BERT layer (hidden 64, 4 heads, ffn 128) end to end.
    p = po.make_bert_layer_params(64, 128, seed=3, std=0.05)
    xb = torch.randn(2, 16, 64, generator=torch.Generator().manual_seed(4))
    save("bert_layer_small", x=xb.numpy(), y=po.bert_layer_forward(xb, p, heads=4).numpy(),
         **{k: v.numpy() for k, v in p.items()})
    print("wrote", len([f for f in os.listdir(OUT) if f.endswith(".npz")]), "fixtures to", OUT)


if __name__ == "__main__":
    main()
