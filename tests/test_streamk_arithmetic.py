"""The stream-K bookkeeping of the INT8 decode GEMM (ateniaengine_b200/csrc/w8_gemm.cu), restated in
Python and checked exhaustively on small cases: the spans the CTAs walk (PieceIter) and the pieces the
reduce kernel adds up (w8_splitk_reduce_kernel) must describe the same decomposition -- every k-block
of every tile covered exactly once, partial pieces found again under the (CTA, slot) they were written
to, whole tiles skipped by the reduce."""
import itertools


def cta_pieces(c, num_ctas, total_tiles, num_kb):
    """PieceIter in stream-K mode for CTA c: list of (tile, kb0, nkb, slot)."""
    total = total_tiles * num_kb
    span = (total + num_ctas - 1) // num_ctas
    g0 = c * span
    g_end = min(g0 + span, total)
    out = []
    g = g0
    while g < g_end:
        t = g // num_kb
        kb0 = g - t * num_kb
        nkb = min(num_kb - kb0, g_end - g)
        slot = -1 if nkb == num_kb else (0 if g == g0 else 1)
        out.append((t, kb0, nkb, slot))
        g += nkb
    return out


def reduce_pieces(t, num_ctas, total_tiles, num_kb):
    """What the reduce kernel reads for tile t: None for a whole tile, else [(cta, slot), ...]."""
    total = total_tiles * num_kb
    span = (total + num_ctas - 1) // num_ctas
    c0 = (t * num_kb) // span
    c1 = ((t + 1) * num_kb - 1) // span
    if c0 == c1:
        return None
    return [(c, 0 if t == (c * span) // num_kb else 1) for c in range(c0, c1 + 1)]


def test_streamk_decomposition_is_consistent():
    for num_ctas, total_tiles, num_kb in itertools.product((1, 2, 3, 7, 16, 148), (1, 2, 5, 32, 64, 224, 300),
                                                           (1, 3, 8, 22, 64, 224)):
        covered = {}
        written = {}
        for c in range(num_ctas):
            pieces = cta_pieces(c, num_ctas, total_tiles, num_kb)
            slots = [p[3] for p in pieces if p[3] >= 0]
            assert len(slots) == len(set(slots)) <= 2, "a CTA owns two workspace slots"
            for (t, kb0, nkb, slot) in pieces:
                for kb in range(kb0, kb0 + nkb):
                    assert (t, kb) not in covered
                    covered[(t, kb)] = c
                if slot >= 0:
                    written.setdefault(t, []).append((c, slot))
        assert len(covered) == total_tiles * num_kb
        for t in range(total_tiles):
            rp = reduce_pieces(t, num_ctas, total_tiles, num_kb)
            if rp is None:
                assert t not in written, "a whole tile leaves nothing in the workspace"
            else:
                assert rp == written[t], (num_ctas, total_tiles, num_kb, t)
