"""Index arithmetic of the f64 tensor-core router (csrc/router_dmma.cu), modelled on the CPU.

mma.sync.m8n8k4.f64 is emulated at warp level from its documented fragment layout (lane l holds
A[l/4][l%4], B[l%4][l/4], D[l/4][2(l%4)+{0,1}]); warps, k-slices, shared-memory rows and the final fold
are indexed exactly as the kernel indexes them.  The result must equal x @ W^T in f64."""
import numpy as np
import pytest

KDW, TOK, KC = 8, 32, 32


def model(x, w, E_T):
    T, d = x.shape
    E = w.shape[0]
    NT = E_T // 8
    NW_N = min(NT, KDW)
    NW_K = KDW // NW_N
    NTW = NT // NW_N
    acc = np.zeros((KDW, 32, 4, NTW, 2))
    for k0 in range(0, d, KC):
        xs = np.zeros((TOK, KC))
        ws = np.zeros((E_T, KC))
        kc = min(KC, d - k0)
        xs[:T, :kc] = x[:, k0:k0 + kc]
        ws[:E, :kc] = w[:, k0:k0 + kc]
        for warp in range(KDW):
            ngrp, kslice = warp % NW_N, warp // NW_N
            for i in range(KC // 4 // NW_K):
                step = kslice + i * NW_K
                for j in range(NTW):
                    for mt in range(4):
                        A = np.zeros((8, 4))
                        B = np.zeros((4, 8))
                        for lane in range(32):
                            frow, fcol = lane >> 2, lane & 3
                            kk = step * 4 + fcol
                            A[frow, fcol] = xs[mt * 8 + frow, kk]
                            B[fcol, frow] = ws[(ngrp * NTW + j) * 8 + frow, kk]
                        D = A @ B
                        for lane in range(32):
                            frow, fcol = lane >> 2, lane & 3
                            acc[warp, lane, mt, j, 0] += D[frow, fcol * 2]
                            acc[warp, lane, mt, j, 1] += D[frow, fcol * 2 + 1]
    out = np.zeros((TOK, E_T + 1))
    for ksl in range(NW_K):
        for warp in range(KDW):
            ngrp, kslice = warp % NW_N, warp // NW_N
            if kslice != ksl:
                continue
            for lane in range(32):
                frow, fcol = lane >> 2, lane & 3
                for mt in range(4):
                    for j in range(NTW):
                        for i in range(2):
                            t, e = mt * 8 + frow, (ngrp * NTW + j) * 8 + fcol * 2 + i
                            if e < E:
                                out[t, e] = (0.0 if ksl == 0 else out[t, e]) + acc[warp, lane, mt, j, i]
    return out[:T, :E]


@pytest.mark.parametrize("E,E_T,T,d", [(8, 8, 32, 64), (4, 8, 5, 48), (16, 16, 32, 32), (32, 32, 17, 80),
                                        (60, 64, 32, 64), (64, 64, 9, 96), (128, 128, 32, 48), (100, 128, 3, 32)])
def test_fragment_indexing_reproduces_the_product(E, E_T, T, d):
    rng = np.random.default_rng(E * 7 + T)
    x = rng.standard_normal((T, d))
    w = rng.standard_normal((E, d))
    np.testing.assert_allclose(model(x, w, E_T), x @ w.T, rtol=1e-12, atol=1e-12)
