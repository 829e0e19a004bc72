"""The layout contract of the peer-memory expert-parallel exchange (include/axm_moe.h:
axm_ep_dispatch / axm_ep_segments), restated in numpy and checked for the properties the
kernels and the grouped GEMMs rely on: every row lands exactly once, a receive buffer is
expert-major with sources in rank order inside an expert, the return map points back at the
source's own permuted row, and one expert's rows form one run (one GEMM segment).

This is the arithmetic of csrc/ep_exchange.cu on the host; the kernels themselves are
compared bit for bit with the single-GPU layer in tests/test_expert_parallel_gpu.py."""
import numpy as np
import pytest


def dispatch_rows(cnt, El):
    """cnt[s][e] = rows source s holds for global expert e.  Returns per owner a dict
    {row in its receive buffer: (source, expert, source's permuted row)}."""
    G, E = cnt.shape
    recv = [dict() for _ in range(G)]
    for src in range(G):
        offs = np.concatenate([[0], np.cumsum(cnt[src])])
        for e in range(E):
            first = (e // El) * El
            base = sum(int(cnt[s, first:e].sum()) + (int(cnt[s, e]) if s < src else 0) for s in range(G))
            for r in range(offs[e], offs[e + 1]):
                d = base + (r - offs[e])
                assert d not in recv[e // El]
                recv[e // El][d] = (src, e, r)
    return recv


def segment_tables(cnt, El, rank):
    """ret_segments and merged GEMM segments of `rank`, entry j * G + s."""
    G, _ = cnt.shape
    n = G * El
    rows = [int(cnt[i % G, rank * El + i // G]) for i in range(n)]
    start = np.concatenate([[0], np.cumsum(rows)])
    ret = [(int(cnt[i % G, :rank * El + i // G].sum()), int(start[i]), rows[i], i % G) for i in range(n)]
    seg = []
    for i in range(n):
        j, s = divmod(i, G)
        first = j * G
        end = int(start[first + G]) if j + 1 < El else int(start[n - 1]) + rows[n - 1]
        seg.append((int(start[first]), int(start[first]), end - int(start[first]) if s == 0 else 0, j))
    return ret, seg, int(start[-1])


@pytest.mark.parametrize("G,El", [(2, 4), (4, 2), (8, 1), (8, 8), (2, 1), (3, 5)])
def test_exchange_layout(G, El):
    rng = np.random.default_rng(G * 100 + El)
    E = G * El
    cnt = rng.integers(0, 40, size=(G, E))
    cnt[rng.random((G, E)) < 0.2] = 0
    recv = dispatch_rows(cnt, El)
    for rank in range(G):
        ret, seg, total = segment_tables(cnt, El, rank)
        assert sorted(recv[rank]) == list(range(total)), "rows land exactly once, without gaps"
        # expert-major, sources in rank order, rows in the source's own order
        order = [recv[rank][d] for d in range(total)]
        assert order == sorted(order, key=lambda t: (t[1], t[0], t[2]))
        for a_row0, out_row0, rows, src in ret:
            for q in range(rows):
                s, e, r = recv[rank][out_row0 + q]
                assert s == src and r == a_row0 + q
        # one run per local expert, the other entries of that expert empty
        for j in range(El):
            a_row0, out_row0, rows, expert = seg[j * G]
            assert expert == j and a_row0 == out_row0
            assert rows == int(cnt[:, rank * El + j].sum())
            assert all(recv[rank][a_row0 + q][1] == rank * El + j for q in range(rows))
            assert all(seg[j * G + s][2] == 0 for s in range(1, G))


def up(v, a):
    return (v + a - 1) // a * a


def dispatch_rows_aligned(cnt, El, align):
    """The training layout (AxmEpLayout.row_align = 64): as dispatch_rows, with every expert's run
    starting at a multiple of `align` rows of the owner's buffer."""
    G, E = cnt.shape
    recv = [dict() for _ in range(G)]
    for src in range(G):
        offs = np.concatenate([[0], np.cumsum(cnt[src])])
        for e in range(E):
            first = (e // El) * El
            base = sum(up(int(cnt[:, q].sum()), align) for q in range(first, e)) + int(cnt[:src, e].sum())
            for r in range(offs[e], offs[e + 1]):
                d = base + (r - offs[e])
                assert d not in recv[e // El]
                recv[e // El][d] = (src, e, r)
    return recv


@pytest.mark.parametrize("G,El,align", [(2, 4, 64), (4, 2, 64), (8, 1, 64), (2, 8, 64), (3, 5, 16)])
def test_exchange_layout_with_aligned_runs(G, El, align):
    rng = np.random.default_rng(G * 1000 + El)
    E = G * El
    cnt = rng.integers(0, 200, size=(G, E))
    cnt[rng.random((G, E)) < 0.2] = 0
    cnt[:, 0] = 0   # an expert nobody chose
    recv = dispatch_rows_aligned(cnt, El, align)
    slots = int(cnt.sum(axis=1).max())
    cap = slots * G + (align - 1) * El
    for rank in range(G):
        start = 0
        for j in range(El):
            e = rank * El + j
            tot = int(cnt[:, e].sum())
            assert start % align == 0
            run = [recv[rank][d] for d in range(start, start + tot)]       # no gaps inside a run
            assert run == sorted(run, key=lambda t: (t[0], t[2])) and all(t[1] == e for t in run)
            pad = range(start + tot, start + up(tot, align))
            assert all(d not in recv[rank] for d in pad), "padding rows stay free (the owner zeroes them)"
            # return map: source s's rows of this expert sit after the lower ranks' rows
            for s in range(G):
                a_row0 = int(cnt[s, :e].sum())
                out_row0 = start + int(cnt[:s, e].sum())
                for q in range(int(cnt[s, e])):
                    assert recv[rank][out_row0 + q] == (s, e, a_row0 + q)
            start += up(tot, align)
        assert start <= cap, "the padded runs fit the receive buffer the layer asks for"
        assert len(recv[rank]) == int(cnt[:, rank * El:(rank + 1) * El].sum())
