"""The tile order of the dense kernel, evaluated on the host by the very function the kernel
calls (``decode_tile`` in csrc/sm100/gemm_dense.cuh, exported as ``fluxb_decode_tiles``): every
tile exactly once, segments entered in the promised order, raster bands of ``group_m`` tile rows
that may span two segments."""
import ctypes

import numpy as np
import pytest


def _decode(num_seg, seg_first, m_tiles_seg, n_tiles, group_m, seg_span, solo, bm=256, bn=256):
    from tempname_new_b200 import _native
    n = num_seg * m_tiles_seg * n_tiles
    out = np.zeros(3 * n, dtype=np.int32)
    rc = _native.lib().fluxb_decode_tiles(num_seg, seg_first, m_tiles_seg, n_tiles, group_m, seg_span, solo, bm, bn,
                                          out.ctypes.data_as(ctypes.c_void_p), n)
    _native.check(rc, "fluxb_decode_tiles")
    return out.reshape(n, 3)


@pytest.mark.parametrize("W,mts,nt,G,span,solo", [
    (8, 4, 24, 8, 2, 1),    # all-gather GEMM of the TP-MLP step at 8 ranks
    (8, 4, 48, 8, 2, 0),    # GEMM + reduce-scatter of the same step
    (4, 8, 12, 8, 1, 0), (3, 4, 5, 8, 2, 0), (8, 2, 6, 4, 2, 1), (5, 3, 7, 6, 2, 0), (1, 16, 16, 8, 1, 0),
    (2, 1, 3, 2, 1, 0),
])
def test_every_tile_once_and_segments_in_order(W, mts, nt, G, span, solo):
    first = 3 % W
    t = _decode(W, first, mts, nt, min(G, span * mts), span, solo)
    assert len({tuple(r) for r in t.tolist()}) == W * mts * nt
    assert t[:, 0].min() >= 0 and t[:, 0].max() < W
    assert t[:, 1].min() >= 0 and t[:, 1].max() < mts
    assert set(t[:, 2].tolist()) == {256 * j for j in range(nt)}
    order = []
    for seg in t[:, 0].tolist():
        if seg not in order:
            order.append(seg)
    assert order == [(first + i) % W for i in range(W)]


def test_bands_span_two_segments_but_the_own_shard_stays_alone():
    W, mts, nt, G = 8, 4, 24, 8
    t = _decode(W, 2, mts, nt, G, 2, 1)
    per_seg = mts * nt
    assert set(t[:per_seg, 0].tolist()) == {2}                 # first group: the own shard only
    band = t[per_seg:per_seg + G * nt]                          # first band of the next group
    assert set(band[:, 0].tolist()) == {3, 4}                   # eight tile rows = two segments
    assert band[:G, 2].tolist() == [0] * G                      # rows innermost: B tile reused
    # without pairing a band never leaves its segment
    t1 = _decode(W, 2, mts, nt, mts, 1, 0)
    for s in range(W):
        assert len(set(t1[s * per_seg:(s + 1) * per_seg, 0].tolist())) == 1


@pytest.mark.parametrize("W", [3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("rank", [0, 2])
def test_reduce_scatter_keeps_the_own_segment_in_a_group_of_its_own(W, rank):
    """The own segment's tiles wait for the peers' partial tiles. If a raster band mixed them with
    tiles of another segment, a CTA could wait there while a partial tile that a peer waits for is
    still behind it in its queue - on every rank at once. So with bands spanning two segments the own
    segment, visited last, must still be a group of its own."""
    from tempname_new_b200 import _native
    mts, nt, G = 4, 6, 8
    solo = _native.lib().fluxb_rs_solo_first(W)
    t = _decode(W, (rank + 1) % W, mts, nt, G, 2, solo)
    per_seg = mts * nt
    assert set(t[-per_seg:, 0].tolist()) == {rank}
    assert rank not in set(t[:-per_seg, 0].tolist())
    # and the pairing is still there for the others
    start = per_seg if solo else 0
    assert any(len(set(t[i:i + G * nt, 0].tolist())) == 2 for i in range(start, len(t) - per_seg, G * nt))


@pytest.mark.parametrize("mts,nt,slots,mode", [
    (32, 24, 74, 1),     # 8192 x 6144 on 256 x 256 pair tiles: 768 tiles, 28 left over -> halves
    (16, 24, 74, 1),     # the same on 512 x 256 tiles: 384 tiles, 14 left over -> quarters
    (16, 24, 74, 2),     # halves only
    (16, 48, 74, 1),     # 768 tiles: 28 left over
    (4, 4, 74, 1),       # smaller than one wave: every tile is "last wave"
    (37, 2, 74, 1),      # exactly one wave: nothing is cut
    (10, 7, 74, 0),      # switched off
])
def test_last_wave_is_cut_into_column_pieces(mts, nt, slots, mode):
    """The launcher's rule (``fluxb_tail_split``) and the kernel's decoding of the resulting work items
    (``decode_tile`` through ``fluxb_decode_work_items``): the pieces fit one wave, every tile is covered
    exactly once by whole items or by all of its pieces, and whole tiles keep their order."""
    from tempname_new_b200 import _native
    lib = _native.lib()
    tiles = mts * nt
    sf, sh = ctypes.c_int32(), ctypes.c_int32()
    _native.check(lib.fluxb_tail_split(ctypes.c_int64(tiles), ctypes.c_int64(slots), mode, ctypes.byref(sf),
                                       ctypes.byref(sh)), "fluxb_tail_split")
    sf, sh = sf.value, sh.value
    rest = tiles % slots
    if mode == 0 or rest == 0:
        assert (sf, sh) == (tiles, 0)
    else:
        assert sf == tiles - rest and (rest << sh) <= slots        # the pieces fit one wave
        assert sh <= (1 if mode == 2 else 2)
        assert sh == 2 or mode == 2 or (rest << (sh + 1)) > slots   # and are as narrow as that allows
    n = sf + ((tiles - sf) << sh)
    out = np.zeros(4 * n, dtype=np.int32)
    _native.check(lib.fluxb_decode_work_items(1, 0, mts, nt, min(8, mts), 1, 0, 512, 256, sf, sh,
                                              out.ctypes.data_as(ctypes.c_void_p), n), "fluxb_decode_work_items")
    items = out.reshape(n, 4)
    whole = _decode(1, 0, mts, nt, min(8, mts), 1, 0, bm=512, bn=256)
    assert np.array_equal(items[:sf, :3], whole[:sf]) and not items[:sf, 3].any()
    covered = {}
    for seg, mt, n0, shift in items[sf:].tolist():
        assert shift == sh
        width = 256 >> shift
        tile = (seg, mt, n0 // 256)
        covered.setdefault(tile, []).append(n0 % 256)
        assert n0 % width == 0
    assert set(covered) == {(s, m, c // 256) for s, m, c in whole[sf:].tolist()}
    for offs in covered.values():
        assert sorted(offs) == [i * (256 >> sh) for i in range(1 << sh)]


def test_decode_rejects_a_bad_grid():
    from tempname_new_b200 import _native
    out = np.zeros(3, dtype=np.int32)
    assert _native.lib().fluxb_decode_tiles(0, 0, 1, 1, 1, 1, 0, 256, 256, out.ctypes.data_as(ctypes.c_void_p), 1) != 0
