"""Expert-parallel exchange plan for 2, 4 and 8 ranks, simulated in one process: every rank's plan
comes from the library's atenia_moe_ep_plan; rows are moved as the device path moves them (send slice
p of the dispatch-ordered rows to rank p, place what rank p sent at recv_off[p]) and must arrive
grouped by (source rank, local expert) in the order the grouped GEMM walks, then travel back to their
original positions."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc


def _plan(lib, counts_all, world, E, rank):
    El = E // world
    so, sc, ro, rc = (np.zeros(world, dtype=np.int64) for _ in range(4))
    go = np.zeros(world * El + 1, dtype=np.int64)
    tot = C.c_int64()
    p = lambda a: C.c_void_p(a.ctypes.data)
    assert lib.atenia_moe_ep_plan(p(counts_all), world, E, rank, p(so), p(sc), p(ro), p(rc), p(go), C.byref(tot)) == 0
    return so, sc, ro, rc, go, tot.value


@pytest.mark.parametrize("world,E,k", [(2, 8, 2), (4, 8, 2), (8, 8, 2), (4, 64, 6), (8, 64, 6), (2, 60, 4), (4, 60, 4)])
def test_exchange_simulation(world, E, k):
    import __graft_entry__ as ge
    ge.build()
    from ateniaengine_b200 import _lib
    lib = _lib.lib()
    rng = np.random.default_rng(world * 1000 + E)
    El = E // world
    # skewed routing and ragged token counts, one rank with no tokens at all
    pop = rng.dirichlet(np.full(E, 0.3))
    tokens = [0 if r == world - 1 and world > 2 else int(rng.integers(1, 200)) for r in range(world)]
    rows, counts = [], []
    for r in range(world):
        idx = np.stack([np.sort(rng.choice(E, size=k, replace=False, p=pop)) for _ in range(tokens[r])]).astype(
            np.int32) if tokens[r] else np.zeros((0, k), np.int32)
        off, perm, _ = orc.dispatch_permutation(idx, E)
        counts.append(np.diff(off).astype(np.int32))
        # a row remembers (source rank, flat entry, expert)
        rows.append(np.stack([np.full(tokens[r] * k, r), perm, idx.ravel()[perm]], axis=1).astype(np.int64)
                    if tokens[r] else np.zeros((0, 3), np.int64))
    counts_all = np.ascontiguousarray(np.stack(counts))
    plans = [_plan(lib, counts_all, world, E, r) for r in range(world)]
    recv = [np.full((plans[r][5], 3), -1, dtype=np.int64) for r in range(world)]
    for src in range(world):
        so, sc = plans[src][0], plans[src][1]
        assert sc.sum() == tokens[src] * k
        for dst in range(world):
            ro, rc = plans[dst][2], plans[dst][3]
            assert sc[dst] == rc[src], "both sides agree on the size of every message"
            recv[dst][ro[src]:ro[src] + rc[src]] = rows[src][so[dst]:so[dst] + sc[dst]]
    for r in range(world):
        go = plans[r][4]
        assert (recv[r] >= 0).all()
        for p in range(world):
            for j in range(El):
                g = recv[r][go[p * El + j]:go[p * El + j + 1]]
                assert (g[:, 0] == p).all() and (g[:, 2] == r * El + j).all()
                assert (np.diff(g[:, 1]) > 0).all()
        assert go[-1] == plans[r][5]
    # way back
    back = [np.full_like(rows[r], -1) for r in range(world)]
    for owner in range(world):
        ro, rc = plans[owner][2], plans[owner][3]
        for src in range(world):
            so, sc = plans[src][0], plans[src][1]
            back[src][so[owner]:so[owner] + sc[owner]] = recv[owner][ro[src]:ro[src] + rc[src]]
    for r in range(world):
        np.testing.assert_array_equal(back[r], rows[r])
