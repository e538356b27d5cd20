"""Row placement of the direct (peer-store) expert-parallel exchange, simulated for 2, 4 and 8 ranks.

atenia_moe_ep_plan_direct is the host form of the function the device runs.  Every rank scatters its
dispatch-ordered rows to dst_base[e] + (i - expert_offsets[e]) of the owner's receive buffer; the
buffers must come out grouped [local expert][source rank] exactly as gemm_offsets and sub_offsets say,
never collide, and src_base must send every row back to where it came from."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc


def _plan(lib, counts_all, world, E, rank):
    dst = np.zeros(E, dtype=np.int32)
    src = np.zeros(E, dtype=np.int32)
    sub = np.zeros(E + 1, dtype=np.int32)
    gemm = np.zeros(E // world + 1, dtype=np.int32)
    p = lambda a: C.c_void_p(a.ctypes.data)
    assert lib.atenia_moe_ep_plan_direct(p(counts_all), world, E, rank, p(dst), p(src), p(sub), p(gemm)) == 0
    return dst, src, sub, gemm


@pytest.mark.parametrize("world,E,k", [(2, 8, 2), (4, 8, 2), (8, 8, 2), (2, 64, 6), (8, 64, 6), (4, 60, 4)])
def test_scatter_and_return_are_consistent(world, E, k):
    import __graft_entry__ as ge
    ge.build()
    from ateniaengine_b200 import _lib
    lib = _lib.lib()
    rng = np.random.default_rng(world * 100 + E)
    El = E // world
    pop = rng.dirichlet(np.full(E, 0.3))
    tokens = [0 if (r == 1 and world > 2) else int(rng.integers(1, 150)) for r in range(world)]
    idxs, offs, perms = [], [], []
    for r in range(world):
        idx = (np.stack([np.sort(rng.choice(E, size=k, replace=False, p=pop)) for _ in range(tokens[r])]).astype(np.int32)
               if tokens[r] else np.zeros((0, k), np.int32))
        off, perm, _ = orc.dispatch_permutation(idx, E)
        idxs.append(idx)
        offs.append(off)
        perms.append(perm)
    counts_all = np.ascontiguousarray(np.stack([np.diff(o) for o in offs]).astype(np.int32))
    plans = [_plan(lib, counts_all, world, E, r) for r in range(world)]
    totals = [int(plans[r][2][E]) for r in range(world)]  # sub_offsets[E] = rows received
    recv = [np.full((totals[r], 3), -1, dtype=np.int64) for r in range(world)]  # (source, dispatch row, expert)
    # scatter, as ep_scatter_kernel places rows
    for src in range(world):
        dst_base = plans[src][0]
        flat_e = idxs[src].ravel()
        for i in range(tokens[src] * k):
            e = int(flat_e[perms[src][i]])
            owner = e // El
            row = int(dst_base[e]) + (i - int(offs[src][e]))
            assert 0 <= row < totals[owner]
            assert recv[owner][row, 0] == -1, "two rows stored to one slot"
            recv[owner][row] = (src, i, e)
    for r in range(world):
        _, src_base, go, gemm = plans[r]
        assert (recv[r][:, 0] >= 0).all(), "a slot of the receive buffer was never written"
        assert gemm[El] == totals[r]
        back = {}
        for j in range(El):
            # all rows of one local expert are contiguous: one GEMM group
            assert (recv[r][gemm[j]:gemm[j + 1], 2] == r * El + j).all()
            assert gemm[j] == go[j * world] and gemm[j + 1] == go[(j + 1) * world]
            for p in range(world):
                g = j * world + p
                rows = recv[r][go[g]:go[g + 1]]
                assert (rows[:, 0] == p).all() and (rows[:, 2] == r * El + j).all()
                assert (np.diff(rows[:, 1]) == 1).all(), "rows of a slice keep the source's order, contiguously"
                # return, as ep_return_kernel places rows
                for i in range(go[g], go[g + 1]):
                    back_row = int(src_base[g]) + (i - int(go[g]))
                    assert back_row == recv[r][i, 1], "a result row goes back to the slot its input came from"
                    back[(p, back_row)] = True
        assert len(back) == totals[r]


def test_argument_checks():
    import __graft_entry__ as ge
    ge.build()
    from ateniaengine_b200 import _lib
    lib = _lib.lib()
    a = np.zeros(16, dtype=np.int32)
    p = C.c_void_p(a.ctypes.data)
    assert lib.atenia_moe_ep_plan_direct(None, 2, 8, 0, p, p, p, p) == -1
    assert lib.atenia_moe_ep_plan_direct(p, 3, 8, 0, p, p, p, p) == -2
    assert lib.atenia_moe_ep_plan_direct(p, 2, 8, 2, p, p, p, p) == -2
