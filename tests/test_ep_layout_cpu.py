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
