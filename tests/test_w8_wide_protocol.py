"""Discrete-event model of the barrier protocol of the wide INT8 kernel (csrc/w8_gemm_wide.cu).

The four roles of a CTA (TMA producer, MMA issuer, two widening groups, epilogue) are written here
exactly as the kernel orders their waits, arrivals and asynchronous operations, with mbarrier phase
semantics, random latencies and versioned buffers.  The model fails on a deadlock, on a buffer that is
overwritten before its readers are done, and on a read of data that has not landed: it checks ring
indices, parities and arrival counts for any number of tiles and k-blocks, without a GPU."""
import heapq
import random

import pytest

S_STAGES, T_STAGES = 6, 4


class Bar:
    def __init__(self, count):
        self.count, self.pending, self.phase, self.tx = count, count, 0, 0

    def _maybe_flip(self):
        if self.pending == 0 and self.tx == 0:
            self.phase ^= 1
            self.pending = self.count

    def arrive(self, tx=0):
        assert self.pending > 0, "more arrivals than the barrier expects in one phase"
        self.pending -= 1
        self.tx += tx
        self._maybe_flip()

    def complete_tx(self, n):
        self.tx -= n
        self._maybe_flip()

    def done(self, parity):  # mbarrier.try_wait.parity
        return self.phase != parity


class Sim:
    acc_bufs = 2  # 1 models w8_gemm.cu: same widening protocol, single accumulator buffer

    def __init__(self, tiles, seed):
        self.rng = random.Random(seed)
        self.tiles = tiles  # list of (num_kb, nbox)
        self.t = 0.0
        self.events = []  # (time, seq, fn)
        self.seq = 0
        self.full = [Bar(1) for _ in range(S_STAGES)]
        self.empty = [Bar(5) for _ in range(S_STAGES)]
        self.a_full = [Bar(4) for _ in range(T_STAGES)]
        self.a_empty = [Bar(1) for _ in range(T_STAGES)]
        self.acc_full = [Bar(1), Bar(1)]
        self.acc_empty = [Bar(8), Bar(8)]
        # versioned buffers: which k-block (or tile) they hold and who is done with it
        self.smem = [dict(idx=None, landed=False, widen_reads=0, mma_read=False) for _ in range(S_STAGES)]
        self.ring = [dict(idx=None, stored=0, mma_read=True) for _ in range(T_STAGES)]
        self.acc = [dict(tile=None, mma_done=False, drained=8) for _ in range(2)]
        self.mma_queue_done = 0.0  # completion time of the last MMA issued (they complete in order)
        self.finished = 0

    def at(self, dt, fn):
        self.seq += 1
        heapq.heappush(self.events, (self.t + dt, self.seq, fn))

    def lat(self, lo, hi):
        return self.rng.uniform(lo, hi)

    # ---- roles (generators yield ("wait", bar, parity) or ("delay", dt)) ----
    def producer(self):
        idx = 0
        for num_kb, nbox in self.tiles:
            for kb in range(num_kb):
                stage, phase = idx % S_STAGES, (idx // S_STAGES) & 1
                yield ("wait", self.empty[stage], phase ^ 1)
                b = self.smem[stage]
                assert b["idx"] is None or (b["widen_reads"] == 4 and b["mma_read"]), "stage overwritten while in use"
                b.update(idx=idx, landed=False, widen_reads=0, mma_read=False)
                nbytes = 2 + nbox
                self.full[stage].arrive(tx=nbytes)
                for _ in range(nbytes):
                    def land(stage=stage, idx=idx):
                        self.full[stage].complete_tx(1)
                        if self.full[stage].tx == 0:
                            self.smem[stage]["landed"] = True
                    self.at(self.lat(50, 900), land)
                yield ("delay", self.lat(1, 10))
                idx += 1
        self.finished += 1

    def mma(self):
        idx, acc, acc_phase = 0, 0, [0, 0]
        for tile_no, (num_kb, nbox) in enumerate(self.tiles):
            yield ("wait", self.acc_empty[acc], acc_phase[acc] ^ 1)
            a = self.acc[acc]
            assert a["drained"] == 8, "accumulator reused before the epilogue drained it"
            a.update(tile=tile_no, mma_done=False, drained=0)
            for kb in range(num_kb):
                stage, tstage = idx % S_STAGES, idx % T_STAGES
                phase, tphase = (idx // S_STAGES) & 1, (idx // T_STAGES) & 1
                yield ("wait", self.full[stage], phase)
                yield ("wait", self.a_full[tstage], tphase)
                assert self.smem[stage]["idx"] == idx and self.smem[stage]["landed"], "MMA read tokens that had not landed"
                r = self.ring[tstage]
                assert r["idx"] == idx and r["stored"] == 4, "MMA read a widened tile that was not complete"
                # MMAs complete in issue order, some time after they are issued
                self.mma_queue_done = max(self.mma_queue_done, self.t) + self.lat(100, 400)
                done_in = self.mma_queue_done - self.t

                def finish(stage=stage, tstage=tstage, idx=idx):
                    assert self.smem[stage]["idx"] == idx and self.ring[tstage]["idx"] == idx, "operand replaced under a running MMA"
                    self.smem[stage]["mma_read"] = True
                    self.ring[tstage]["mma_read"] = True
                    self.empty[stage].arrive()     # tcgen05.commit -> empty[stage]
                    self.a_empty[tstage].arrive()  # tcgen05.commit -> a_empty[tstage]
                self.at(done_in, finish)
                yield ("delay", self.lat(1, 8))
                idx += 1

            def tile_done(acc=acc, tile_no=tile_no):
                assert self.acc[acc]["tile"] == tile_no
                self.acc[acc]["mma_done"] = True
                self.acc_full[acc].arrive()
            self.at(max(self.mma_queue_done - self.t, 0.0) + 1e-6, tile_done)
            acc_phase[acc] ^= 1
            acc = (acc + 1) % self.acc_bufs
        self.finished += 1

    def widen(self, group, quarter):
        idx = 0
        pend = None

        def retire():
            nonlocal pend
            if pend is None:
                return
            stage, tstage, pidx = pend
            assert self.ring[tstage]["idx"] == pidx
            self.ring[tstage]["stored"] += 1   # tcgen05.wait::st returned: this warp's rows are in TMEM
            self.a_full[tstage].arrive()
            self.empty[stage].arrive()
            pend = None

        for num_kb, nbox in self.tiles:
            for kb in range(num_kb):
                if (idx & 1) != group:
                    idx += 1
                    continue
                stage, tstage = idx % S_STAGES, idx % T_STAGES
                phase, tphase = (idx // S_STAGES) & 1, (idx // T_STAGES) & 1
                yield ("wait", self.full[stage], phase)
                b = self.smem[stage]
                assert b["idx"] == idx and b["landed"], "widening read codes that had not landed"
                yield ("delay", self.lat(20, 300))  # ld.shared + widen
                b["widen_reads"] += 1
                retire()
                yield ("wait", self.a_empty[tstage], tphase ^ 1)
                r = self.ring[tstage]
                if r["idx"] != idx:
                    assert r["mma_read"], "TMEM stage overwritten before its MMAs finished"
                    r.update(idx=idx, stored=0, mma_read=False)
                yield ("delay", self.lat(5, 150))   # tcgen05.st in flight
                pend = (stage, tstage, idx)
                idx += 1
        retire()
        self.finished += 1

    def epilogue(self, w):
        acc, acc_phase = 0, [0, 0]
        for tile_no, _ in enumerate(self.tiles):
            yield ("wait", self.acc_full[acc], acc_phase[acc])
            acc_phase[acc] ^= 1
            a = self.acc[acc]
            assert a["tile"] == tile_no and a["mma_done"], "epilogue read an unfinished accumulator"
            yield ("delay", self.lat(50, 2500))
            assert a["tile"] == tile_no, "accumulator overwritten while the epilogue was reading it"
            a["drained"] += 1
            self.acc_empty[acc].arrive()
            acc = (acc + 1) % self.acc_bufs
        self.finished += 1

    def run(self):
        procs = [self.producer(), self.mma()] + [self.widen(g, q) for g in range(2) for q in range(4)] + [
            self.epilogue(w) for w in range(8)]
        state = {}  # proc -> pending wait or None

        def step(p):
            while True:
                w = state.get(p)
                if w is not None:
                    if not w[0].done(w[1]):
                        return
                    state[p] = None
                try:
                    op = next(p)
                except StopIteration:
                    state[p] = "end"
                    return
                if op[0] == "wait":
                    state[p] = (op[1], op[2])
                else:
                    state[p] = ("sleep",)
                    self.at(op[1], lambda p=p: (state.__setitem__(p, None), step(p)))
                    return

        for p in procs:
            state[p] = None
            step(p)
        guard = 0
        while self.finished < len(procs):
            guard += 1
            assert guard < 5_000_000
            if not self.events:
                blocked = [i for i, p in enumerate(procs) if state[p] not in ("end",)]
                raise AssertionError(f"deadlock: roles {blocked} wait and nothing is in flight")
            self.t, _, fn = heapq.heappop(self.events)
            fn()
            for p in procs:
                if isinstance(state[p], tuple) and len(state[p]) == 2:
                    step(p)
        assert all(a["drained"] == 8 for a in self.acc if a["tile"] is not None)


@pytest.mark.parametrize("tiles", [
    [(1, 1)], [(2, 3)], [(3, 2), (1, 1)], [(64, 3)] * 3, [(5, 1), (7, 3), (1, 2), (12, 3)],
    [(1, 3)] * 9, [(6, 3), (6, 3)], [(13, 2)] * 5,
])
def test_protocol_has_no_deadlock_or_hazard(tiles):
    for seed in range(12):
        Sim(tiles, seed).run()


@pytest.mark.parametrize("tiles", [[(1, 1)], [(7, 1), (3, 1)], [(64, 1)] * 2, [(2, 1)] * 7, [(224, 1)]])
def test_alternating_groups_with_a_single_accumulator(tiles):
    """The decode variant (w8_gemm.cu): stream-K pieces of any length, one accumulator buffer."""
    class Single(Sim):
        acc_bufs = 1
    for seed in range(8):
        Single(tiles, seed).run()


def test_model_detects_a_wrong_arrival_count():
    """The model is only worth something if it fails on a broken protocol: with the shared-memory
    stage released by four arrivals instead of five, the producer overwrites a stage the MMA still
    reads (or a barrier sees more arrivals than it expects)."""
    class Broken(Sim):
        def __init__(self, tiles, seed):
            super().__init__(tiles, seed)
            self.empty = [Bar(4) for _ in range(S_STAGES)]
    failures = 0
    for seed in range(12):
        try:
            Broken([(40, 3)] * 2, seed).run()
        except AssertionError:
            failures += 1
    assert failures > 0


def test_lane_mapping_covers_every_output_once():
    """kSwiGLU tile of the wide kernel: TMEM lane 32q + l holds the row that widening thread (q, l)
    read from shared memory; the epilogue pairs lane l with lane l ^ 16 and the two share the token
    columns.  Every (token, feature) of the 64-feature tile must be stored exactly once, from a gate
    row and an up row of the same feature."""
    rows = 181  # tokens in the tile (ragged)
    written = {}
    for q in range(4):
        for half in range(2):
            for lane in range(32):
                upper = lane >> 4
                srow = (q * 16 + lane) if lane < 16 else 64 + q * 16 + (lane - 16)
                partner = lane ^ 16
                prow = (q * 16 + partner) if partner < 16 else 64 + q * 16 + (partner - 16)
                feature = q * 16 + (lane & 15)
                # my row and my partner's row are the gate and up rows of `feature`
                gate_row, up_row = (prow, srow) if upper else (srow, prow)
                assert gate_row == feature and up_row == 64 + feature
                c = half * 16
                while c < rows:
                    for j in range(16):
                        if (j & 1) == upper and c + j < rows:
                            key = (c + j, feature)
                            assert key not in written
                            written[key] = (q, half, lane)
                    c += 32
    assert len(written) == rows * 64
