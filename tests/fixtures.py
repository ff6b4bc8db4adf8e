"""Deterministic known-answer inputs of the reference's own kernel tests, restated.

Each builder reproduces the input formulas of one reference test and the expected
values the way that test computes them on the host (double or float loops), so the
oracle and the CUDA kernels can be held to the reference's own thresholds:

* mxfp4_block17   src/test_mxfp4.cu:10-25     max_rel < 2e-4 (denominator + 1e-6)
* mxfp4_mlx       src/bench_mxfp4_mlx.cu:7    max_rel <= 3e-4 (denominator + 1e-5)
* deltanet        src/test_deltanet.cu:7      max_rel < 3e-3 (denominator + 1e-5)
* attention       src/test_attention.cu:7     max_abs < 2e-5
* rmsnorm         src/test_ops.cu:7           max_abs < 2e-6
"""
import numpy as np

LUT = np.array([0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6], np.float32)


def x_vector(cols=4096):
    i = np.arange(cols)
    return (((i * 17) % 31 - 15) / 16.0).astype(np.float32)


def mxfp4_block17(rows=257, cols=4096):
    blocks = cols // 32
    r = np.arange(rows)[:, None, None]
    b = np.arange(blocks)[None, :, None]
    j = np.arange(16)[None, None, :]
    scale = (124 + ((r + b) % 7)).astype(np.uint8)[:, :, 0]
    q = (((r + b + j * 3) & 15) | (((r * 5 + b + j * 7) & 15) << 4)).astype(np.uint8)
    raw = np.concatenate([scale[:, :, None], q], axis=2)  # [rows][blocks][17]
    x = x_vector(cols)
    codes = np.concatenate([q & 15, q >> 4], axis=2)  # lane<16 low nibble, lane>=16 high nibble
    sc = (scale.astype(np.uint32) << 23).view(np.float32)
    w = (LUT[codes] * sc[:, :, None]).astype(np.float32)  # the test multiplies in float, sums in double
    expected = (w.astype(np.float64) * x.reshape(blocks, 32)[None]).sum(axis=(1, 2)).astype(np.float32)
    return np.ascontiguousarray(raw).reshape(-1), x, expected


def mxfp4_mlx(rows=4096, cols=4096):
    groups = cols // 32
    r = np.arange(rows)[:, None, None]
    g = np.arange(groups)[None, :, None]
    lane = np.arange(32)[None, None, :]
    scales = (124 + (r + g) % 7).astype(np.uint8)[:, :, 0]
    codes = ((r * 5 + g + lane * 7) & 15).astype(np.uint32)  # [rows][groups][32]
    c = codes.reshape(rows, groups * 4, 8)
    weight = np.zeros((rows, groups * 4), np.uint32)
    for jj in range(8):
        weight |= c[:, :, jj] << np.uint32(4 * jj)
    x = x_vector(cols)
    sc = (scales.astype(np.uint32) << 23).view(np.float32)
    w = (LUT[codes] * sc[:, :, None]).astype(np.float32)
    expected = (w.astype(np.float64) * x.reshape(groups, 32)[None]).sum(axis=(1, 2)).astype(np.float32)
    return weight, scales, x, expected


def deltanet():
    H, K, V, KH = 32, 128, 128, 16
    i = np.arange(H * K * V, dtype=np.int64)
    s = ((i * 13 % 37 - 18) * np.float32(1e-3)).astype(np.float32)
    i = np.arange(KH * K, dtype=np.int64)
    q = ((i * 7 % 29 - 14).astype(np.float32) * np.float32(.03)).astype(np.float32)
    k = ((i * 11 % 31 - 15).astype(np.float32) * np.float32(.02)).astype(np.float32)
    i = np.arange(H * V, dtype=np.int64)
    v = ((i * 5 % 23 - 11).astype(np.float32) * np.float32(.04)).astype(np.float32)
    h = np.arange(H)
    g = (np.float32(-.01) * (1 + h % 7)).astype(np.float32)
    b = (np.float32(.1) + np.float32(.02) * (h % 11)).astype(np.float32)
    # float32 host loop of the test, vectorised over v (the sums over i run in the same order)
    S = s.reshape(H, K, V).copy()
    ref = np.zeros((H, V), np.float32)
    for hh in range(H):
        kh = hh // 2
        qq, kk = q[kh * K:(kh + 1) * K], k[kh * K:(kh + 1) * K]
        qn, kn = np.float32(1e-6), np.float32(1e-6)
        for t in range(K):
            qn = np.float32(qn + qq[t] * qq[t])
            kn = np.float32(kn + kk[t] * kk[t])
        qn = np.float32(np.float32(1) / np.sqrt(qn) / np.sqrt(np.float32(K)))
        kn = np.float32(np.float32(1) / np.sqrt(kn))
        d = np.float32(np.exp(g[hh]))
        mem = np.zeros(V, np.float32)
        for t in range(K):
            mem = (mem + S[hh, t] * d * kk[t] * kn).astype(np.float32)
        delta = ((v[hh * V:(hh + 1) * V] - mem) * b[hh]).astype(np.float32)
        z = np.zeros(V, np.float32)
        for t in range(K):
            S[hh, t] = (S[hh, t] * d + kk[t] * kn * delta).astype(np.float32)
            z = (z + S[hh, t] * qq[t] * qn).astype(np.float32)
        ref[hh] = z
    return s, q, k, v, g, b, ref.reshape(-1), S.reshape(-1)


def attention(T=257):
    H, KV, D = 16, 4, 256
    i = np.arange(H * D, dtype=np.int64)
    q = ((i * 7 % 31 - 15).astype(np.float32) * np.float32(.02)).astype(np.float32)
    i = np.arange(T * KV * D, dtype=np.int64)
    k = ((i * 11 % 37 - 18).astype(np.float32) * np.float32(.015)).astype(np.float32)
    v = ((i * 5 % 29 - 14).astype(np.float32) * np.float32(.03)).astype(np.float32)
    kk = k.reshape(T, KV, D).astype(np.float64)
    vv = v.reshape(T, KV, D).astype(np.float64)
    ref = np.zeros((H, D), np.float32)
    for h in range(H):
        s = kk[:, h // 4, :] @ q[h * D:(h + 1) * D].astype(np.float64) / 16
        p = np.exp(s - s.max())
        ref[h] = ((p / p.sum())[:, None] * vv[:, h // 4, :]).sum(0).astype(np.float32)
    return q, k, v, ref.reshape(-1)


def rmsnorm(R=3, C=4096):
    i = np.arange(R * C, dtype=np.int64)
    x = ((i * 13 % 43 - 21).astype(np.float32) * np.float32(.03)).astype(np.float32).reshape(R, C)
    i = np.arange(C, dtype=np.int64)
    w = ((i * 5 % 17 - 8).astype(np.float32) * np.float32(.01)).astype(np.float32)
    ss = (x.astype(np.float64) ** 2).sum(1)
    inv = (np.float32(1) / np.sqrt((ss / C).astype(np.float32) + np.float32(1e-6))).astype(np.float32)
    ref = (x * inv[:, None] * (1 + w)[None]).astype(np.float32)
    return x, w, ref


def max_rel(actual, expected, eps):
    return float(np.max(np.abs(actual - expected) / (np.abs(expected) + eps)))
