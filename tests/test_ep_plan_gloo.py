"""Expert-parallel host logic on CPU: two gloo ranks route their own tokens, exchange rows according
to atenia_moe_ep_plan (the library's own partition arithmetic, called through the C ABI) and check
that every row reaches the rank that owns its expert, grouped as the device path expects, and comes
back to its original place."""
import ctypes as C
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as orc


def _plan(lib, counts_all, world, E, rank):
    El = E // world
    so, sc, ro, rc = (np.zeros(world, dtype=np.int64) for _ in range(4))
    go = np.zeros(world * El + 1, dtype=np.int64)
    tot = C.c_int64()
    p = lambda a: C.c_void_p(a.ctypes.data)
    st = lib.atenia_moe_ep_plan(p(counts_all), world, E, rank, p(so), p(sc), p(ro), p(rc), p(go), C.byref(tot))
    assert st == 0
    return so, sc, ro, rc, go, tot.value


def _worker(rank, world, port, E, k, T):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ateniaengine_b200 import _lib
        lib = _lib.lib()
        rng = np.random.default_rng(100 + rank)
        Tl = T + 3 * rank  # ragged token counts per rank
        idx = np.stack([np.sort(rng.choice(E, size=k, replace=False)) for _ in range(Tl)]).astype(np.int32)
        off, perm, inv = orc.dispatch_permutation(idx, E)
        counts = np.diff(off).astype(np.int32)
        gathered = [torch.zeros(E, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(counts))
        counts_all = np.ascontiguousarray(torch.stack(gathered).numpy())
        so, sc, ro, rc, go, total = _plan(lib, counts_all, world, E, rank)
        El = E // world
        # rows carry (source rank, flat entry id, expert) so their journey can be checked
        rows = np.stack([np.full(Tl * k, rank), perm, idx.ravel()[perm]], axis=1).astype(np.int64)
        assert sc.sum() == Tl * k and so[0] == 0
        out_lists = [None] * world
        dist.all_gather_object(out_lists, [rows[so[p]:so[p] + sc[p]] for p in range(world)])
        recv = np.concatenate([out_lists[p][rank] for p in range(world)]) if total else np.zeros((0, 3), np.int64)
        assert recv.shape[0] == total == rc.sum()
        for p in range(world):
            assert np.array_equal(recv[ro[p]:ro[p] + rc[p]], out_lists[p][rank])
            for j in range(El):
                g = recv[go[p * El + j]:go[p * El + j + 1]]
                assert (g[:, 0] == p).all() and (g[:, 2] == rank * El + j).all()
                assert (np.diff(g[:, 1]) > 0).all()  # the source's dispatch order is kept
        # way back: results return to the sender's dispatch order
        back = [None] * world
        dist.all_gather_object(back, [recv[ro[p]:ro[p] + rc[p]] for p in range(world)])
        y = np.concatenate([back[p][rank] for p in range(world)])
        assert np.array_equal(y, rows)
        # plans of the two sides agree
        plans = [None] * world
        dist.all_gather_object(plans, (sc.tolist(), rc.tolist()))
        for p in range(world):
            assert plans[p][1][rank] == sc[p] and plans[p][0][rank] == rc[p]
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("E,k", [(8, 2), (64, 6)])
def test_ep_plan_two_ranks_gloo(E, k):
    import __graft_entry__ as ge
    ge.build()
    port = 29500 + (os.getpid() % 1000) + E
    mp.spawn(_worker, args=(2, port, E, k, 57), nprocs=2, join=True)


def test_ep_plan_rejects_bad_arguments():
    from ateniaengine_b200 import _lib
    lib = _lib.lib()
    a = np.zeros(16, dtype=np.int64)
    c = np.zeros((2, 8), dtype=np.int32)
    p = lambda x: C.c_void_p(x.ctypes.data)
    assert lib.atenia_moe_ep_plan(None, 2, 8, 0, p(a), p(a), p(a), p(a), None, None) == -1
    assert lib.atenia_moe_ep_plan(p(c), 3, 8, 0, p(a), p(a), p(a), p(a), None, None) == -2
    assert lib.atenia_moe_ep_plan(p(c), 2, 8, 2, p(a), p(a), p(a), p(a), None, None) == -2
