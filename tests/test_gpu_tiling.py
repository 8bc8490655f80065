"""GPU parity tests (through the C ABI): the GPU partitioning + conversion must be BIT-EXACT against the
checker (the C restatement pinned to upstream, and the golden digests made by upstream itself)."""
import hashlib
import json
import os

import numpy as np
import pytest

import _orc
import cases

pytestmark = pytest.mark.gpu

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "tiling_golden.json")))
CASES = cases.small_cases()


def h(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()[:16]


def digest(m):
    return {f"{_orc.CLASSES[c]}:{w}": h(m.array(c, w)) for c in range(3) for w in _orc.ARRAYS}


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("prec", [0, 1])
def test_tiling_bit_exact_vs_upstream_golden(name, prec):
    from tilespmm_b200 import api
    rp, ci, v, shape = CASES[name]
    m = api.TileMatrix(prec)
    for (g, d) in cases.GAMMA_DELTA:
        rec = GOLDEN["tiling"][f"{name}|{prec}|{g}|{d}"]
        m.convert_host(shape, rp, ci, v, g, d)
        assert m.info().tolist() == rec["info"], (name, prec, g, d)
        got = digest(m)
        if got != rec["arrays"]:   # show the first differing array element by element
            o = _orc.Orc(prec, shape, rp, ci, v, g, d)
            for c in range(3):
                for w in _orc.ARRAYS:
                    np.testing.assert_array_equal(m.array(c, w), o.array(c, w), err_msg=f"{name} prec={prec} g={g} d={d} cls={c} {w}")
        assert got == rec["arrays"]
        for cls in range(3):
            for TH in (8, 24, 64):
                rows, cs = m.schedule(cls, TH)
                if rec["info"][cls][3] == 0:
                    # upstream builds no schedule for a class without tiles (src/csr2tile.h:662) and relies on a
                    # cleared C; here such a class gets one empty task per panel, which writes the zeros
                    assert rows.size == rec["info"][cls][2] and not cs.any() and not (rows >> 31).any()
                    continue
                assert [int(rows.size), h(rows), h(cs)] == rec["sched"][f"{cls}:{TH}"], (name, prec, g, d, cls, TH)
    m.close()


@pytest.mark.parametrize("prec", [0, 1])
def test_threshold_candidates_match_cost_model(prec):
    """tsp_top4 against the checker's cost model fed with the resource rows and the atomic weight of THESE kernels."""
    from tilespmm_b200 import api
    import torch
    props = torch.cuda.get_device_properties(0)
    for name in ("rmat_s11", "stencil_g17", "banded_4099", "rand_wide_64x5000"):
        rp, ci, v, shape = CASES[name]
        for (g, d) in ((2.0, 1.2), (0.0, 1.5), (5.0, 0.0), (5.0, 3.0)):
            m = api.TileMatrix(prec).convert_host(shape, rp, ci, v, g, d)
            o = _orc.Orc(prec, shape, rp, ci, v, g, d)
            for cls in range(3):
                for cb in (32, 64, 128, 256):
                    k = m.kernel_info(cls, cb)
                    res = _orc.OrcResources(props.multi_processor_count, props.max_threads_per_multi_processor, 32,
                                            props.regs_per_multiprocessor, props.L2_cache_size, props.shared_memory_per_multiprocessor,
                                            int(k[0]), int(k[1]), int(k[3]), int(k[2]), int(k[4]), int(k[5]),
                                            api.atom_weight(prec, cls, cb))
                    assert m.top4(cls, cb).tolist() == o.top4(cls, cb, res).tolist(), (name, g, d, cls, cb)
            m.close()


@pytest.mark.parametrize("prec", [0, 1])
def test_larger_seeded_inputs_vs_checker(prec):
    """Benchmark-shaped inputs at sizes the CPU checker converts in seconds."""
    from tilespmm_b200 import api, synth
    inputs = [synth.stencil27(40, 1002), synth.rmat_symmetric(16, 16, 1003), synth.mixed_density(65536, 1004),
              synth.fixed_nnz_per_row(4096, 16, 1001)]
    m = api.TileMatrix(prec)
    for rp, ci, v, shape in inputs:
        for (g, d) in ((2.0, 1.2), (1.4, 1.5), (0.0, 1.5), (5.0, 0.0), (5.0, 3.0)):
            m.convert_host(shape, rp, ci, v, g, d)
            o = _orc.Orc(prec, shape, rp, ci, v, g, d)
            assert m.info().tolist() == o.info().tolist()
            assert digest(m) == o.digest(), (shape, g, d)
    m.close()


def test_shards_agree_with_unsharded_tiling():
    """Sharding cuts the global panel sequence: concatenating the shards' arrays gives the unsharded arrays."""
    from tilespmm_b200 import api, synth
    rp, ci, v, shape = synth.rmat_symmetric(14, 16, 77)
    for prec, (g, d) in ((0, (2.0, 1.2)), (1, (5.0, 3.0)), (0, (0.0, 1.5))):
        full = api.TileMatrix(prec).convert_host(shape, rp, ci, v, g, d)
        full.info()
        parts = [api.TileMatrix(prec).convert_host(shape, rp, ci, v, g, d, shard=(k, 3)) for k in range(3)]
        infos = [p.info() for p in parts]
        assert sum(i[:, 3] for i in infos).tolist() == full.info()[:, 3].tolist()
        assert sum(i[:, 0] for i in infos).tolist() == full.info()[:, 0].tolist()
        assert parts[0].row_range[0] == 0 and parts[-1].row_range[1] == shape[0]
        for a, b in zip(parts[:-1], parts[1:]):
            assert a.row_range[1] == b.row_range[0]
        for cls in range(3):
            for w in ("tile_colidx", "tile_val", "panel_row", "orig_row"):
                np.testing.assert_array_equal(np.concatenate([p.array(cls, w) for p in parts]), full.array(cls, w))


def test_shard_boundaries_follow_the_byte_balance_rule():
    """The library cuts the global panel sequence where tilespmm_b200.multi.shard_cuts says (same cost rule)."""
    from tilespmm_b200 import api, multi, synth
    rp, ci, v, shape = synth.rmat_symmetric(14, 16, 78)
    prec, (g, d), world = 0, (2.0, 1.2), 4
    full = api.TileMatrix(prec).convert_host(shape, rp, ci, v, g, d)
    full.info()
    panels = []
    for cls in range(3):
        rows, tp = full.array(cls, "panel_row"), full.array(cls, "tile_ptr")
        panels += [(int(r), cls, int(n)) for r, n in zip(rows, np.diff(tp))]
    panels.sort()
    costs = [multi.panel_cost(n, _orc.CLASSES[cls], _orc.BN(prec, cls), 2) for _, cls, n in panels]
    cuts = multi.shard_cuts(costs, world)
    for k in range(world):
        part = api.TileMatrix(prec).convert_host(shape, rp, ci, v, g, d, shard=(k, world))
        part.info()
        want_begin = panels[cuts[k]][0] if cuts[k] < len(panels) else shape[0]
        want_end = panels[cuts[k + 1]][0] if cuts[k + 1] < len(panels) else shape[0]
        assert part.row_range == (want_begin, want_end), (k, part.row_range, want_begin, want_end)


def test_tile_cache_round_trip(tmp_path):
    """tsp_save / tsp_load: a handle restored from the cache file exports the same arrays and multiplies the same."""
    import ctypes as C
    from tilespmm_b200 import api, synth
    rp, ci, v, shape = cases.banded_blocks(3001, 7000, 91)
    for prec in (0, 1):
        m = api.TileMatrix(prec).convert_host(shape, rp, ci, v, 2.0, 1.2, shard=(1, 2))
        m.info()
        path = str(tmp_path / f"tiles{prec}.bin").encode()
        m.L.tsp_save.argtypes = [C.c_void_p, C.c_char_p]
        m.L.tsp_load.argtypes = [C.c_void_p, C.c_char_p]
        assert m.L.tsp_save(m.h, path) == 0, m.L.tsp_last_error()
        r = api.TileMatrix(prec)
        assert r.L.tsp_load(r.h, path) == 0, r.L.tsp_last_error()
        r.shape = shape
        assert r.info().tolist() == m.info().tolist() and r.row_range == m.row_range
        for cls in range(3):
            for w in _orc.ARRAYS:
                np.testing.assert_array_equal(r.array(cls, w), m.array(cls, w))
        B = api.to_values(synth.dense_b(shape[1], 64, 3), prec).reshape(shape[1], 64)
        np.testing.assert_array_equal(r.spmm_host(B, 64), m.spmm_host(B, 64))
        other = api.TileMatrix(1 - prec)
        assert other.L.tsp_load(other.h, path) == 1 and b"holds" in other.L.tsp_last_error()
        bad = tmp_path / "junk.bin"
        bad.write_bytes(b"not a cache")
        assert r.L.tsp_load(r.h, str(bad).encode()) == 1


# ---------------------------------------------------------------- packed records of the 64-row class

def _frag16(prec, r, c):
    """Position of (r, c) of a 16-row block in mma.sync A-fragment order (upstream src/csr2tile.h:289-307)."""
    if prec == 0:
        return ((((r & 7) << 2) + ((c & 7) >> 1)) << 3) + ((c >> 3) << 2) + ((r >> 3) << 1) + (c & 1)
    return ((((r & 7) << 2) + (c & 3)) << 2) + ((c >> 2) << 1) + (r >> 3)


def _upstream64(prec, r, c):
    """Position of (r, c) inside a 64-row tile as upstream stores it (src/csr2tile.h:319-372)."""
    kw = 16 if prec == 0 else 8
    return ((r >> 4) * 2 + c // kw) * 16 * kw + _frag16(prec, r & 15, c % kw)


def _umma64(prec, r, k):
    """Position of (r, k) in the K-major core-matrix order tcgen05.mma reads (dense records)."""
    t = 8 if prec == 0 else 4
    return ((k // t) * 8 + (r >> 3)) * 8 * t + (r & 7) * t + (k % t)


def masks_from_csr(prec, shape, rp, ci, o):
    """Ground truth of the row masks, from the CSR and the checker's tiling alone: bit k of masks[tile, r] is set when
    the CSR stores an entry (whatever its value) at row panel_row + r in the column tile_colidx[tile, k] names."""
    bn = _orc.BN(prec, 0)
    rows, tp = o.array(0, "panel_row"), o.array(0, "tile_ptr")
    masks = np.zeros((int(tp[-1]) if tp.size else 0, 64), dtype=np.uint32)
    for p, r0 in enumerate(rows):
        r1 = min(int(r0) + 64, shape[0])
        cols = ci[rp[r0]:rp[r1]]
        rank = np.searchsorted(np.unique(cols), cols)
        rr = np.repeat(np.arange(r0, r1), np.diff(rp[r0:r1 + 1])) - r0
        np.bitwise_or.at(masks, (tp[p] + rank // bn, rr), (np.uint32(1) << (rank % bn).astype(np.uint32)))
    return masks


def dense_from_records(prec, masks, rec, records):
    """Upstream's dense 64-row tiles rebuilt on the CPU from the exported records (not through the library's own export).
    A packed record: n_pad = n rounded up to 8 positions (uint16, the element's index in the tcgen05 operand tile, 0xffff
    in the padding), then n_pad values, both in row-major order of the set mask bits.  A dense record: the 4 KB tile."""
    bn, vt = _orc.BN(prec, 0), (np.uint16 if prec == 0 else np.float32)
    vsz = 2 if prec == 0 else 4
    ntile = masks.shape[0]
    out = np.zeros((ntile, 64 * bn), dtype=vt)
    r_idx, k_idx = np.meshgrid(np.arange(64), np.arange(bn), indexing="ij")
    up = _upstream64(prec, r_idx, k_idx)
    um = _umma64(prec, r_idx, k_idx)
    for t in range(ntile):
        off, end = int(rec[t] & 0x7fffffff) * 16, int(rec[t + 1] & 0x7fffffff) * 16
        set_bits = ((masks[t][:, None] >> np.arange(bn, dtype=np.uint32)[None, :]) & 1).astype(bool)   # [64, bn], row-major
        n = int(set_bits.sum())
        if rec[t] >> 31:
            assert end - off == 4096 and n > (256 if prec == 0 else 128)
            tile = records[off:off + 4096].view(vt)
            out[t, up.ravel()] = tile[um.ravel()]
            continue
        n_pad = (n + 7) // 8 * 8
        assert n <= (256 if prec == 0 else 128) and end - off == n_pad * (2 + vsz)
        pos = records[off:off + 2 * n_pad].view(np.uint16)
        vals = records[off + 2 * n_pad:end].view(vt)
        np.testing.assert_array_equal(pos[:n], um[set_bits])                 # positions follow the masks, row-major
        assert (pos[n:] == 0xffff).all() and not vals[n:].any()               # padding
        out[t, up[set_bits]] = vals[:n]
    return out.ravel()


@pytest.mark.parametrize("prec", [0, 1])
def test_packed_records_of_the_64_row_class(prec):
    """Row masks against the CSR ground truth (an explicit zero sets its bit), record offsets and contents against
    upstream's dense tiles, for sparse tiles (packed records), fuller tiles (dense records) and repeated entries."""
    from tilespmm_b200 import api
    picks = [("stencil_g17", (0.0, 1.5)), ("mixed_4096", (0.0, 1.5)), ("banded_4099", (1.0, 1.0)), ("rand_dups_150", (0.0, 1.5)),
             ("rand_wide_64x5000", (0.0, 1.5)), ("rmat_s11", (1.4, 1.5)), ("rand_tiny_5", (0.0, 1.5))]
    m = api.TileMatrix(prec)
    kinds = set()
    for name, (g, d) in picks:
        rp, ci, v, shape = CASES[name]
        v = v.copy()
        v[::7] = 0.0                                            # stored zeros: present in the masks, absent from the values
        m.convert_host(shape, rp, ci, v, g, d)
        info = m.info()
        o = _orc.Orc(prec, shape, rp, ci, v, g, d)
        assert info.tolist() == o.info().tolist()
        if info[0, 3] == 0:
            assert m.array(0, "masks").size == 0 and m.array(0, "records").size == 0
            continue
        masks = m.array(0, "masks").reshape(-1, 64).astype(np.uint32)
        np.testing.assert_array_equal(masks, masks_from_csr(prec, shape, rp, ci, o), err_msg=name)
        rec, records = m.array(0, "rec"), m.array(0, "records")
        assert rec[0] & 0x7fffffff == 0 and int(rec[-1] & 0x7fffffff) * 16 == records.size
        kinds |= {bool(x >> 31) for x in rec[:-1]}
        want = o.array(0, "tile_val")
        np.testing.assert_array_equal(dense_from_records(prec, masks, rec, records), want, err_msg=name)
        np.testing.assert_array_equal(m.array(0, "tile_val"), want, err_msg=name)      # the library's own expansion
    assert kinds == {False, True}                               # both record kinds were exercised
    m.close()


def test_inconsistent_csr_and_damaged_cache_are_refused(tmp_path):
    """Bad input must come back as TSP_EINVAL before any kernel indexes with it."""
    import ctypes as C
    from tilespmm_b200 import api
    rp, ci, v, shape = CASES["banded_1500"]
    m = api.TileMatrix(1)
    for what in ("column", "negative", "rowptr_order", "rowptr_end"):
        rp2, ci2 = rp.copy(), ci.copy()
        if what == "column":
            ci2[ci2.size // 2] = shape[1]
        elif what == "negative":
            ci2[3] = -1
        elif what == "rowptr_order":
            rp2[10], rp2[11] = rp2[11] + 5, rp2[10]
        else:
            rp2[-1] -= 1
        with pytest.raises(api.TileSpMMError, match="inconsistent"):
            m.convert_host(shape, rp2, ci2, v, 2.0, 1.2)
    m.convert_host(shape, rp, ci, v, 0.0, 1.5)                  # the handle is still usable
    m.info()
    path = tmp_path / "tiles.bin"
    m.L.tsp_save.argtypes = [C.c_void_p, C.c_char_p]
    m.L.tsp_load.argtypes = [C.c_void_p, C.c_char_p]
    assert m.L.tsp_save(m.h, str(path).encode()) == 0
    good = path.read_bytes()
    hdr = 112                                                   # sizeof(FileHeader) in csrc/tile_cache.cu; tilem[0] sits at byte 52
    tilem = int(m.info()[0, 2])
    col_at = hdr + (tilem + 1) * 4 + tilem * 4 + (int(m.info()[0, 3]) + 1) * 4      # first column index of the 64-row class
    damaged = {
        "truncated": good[:len(good) // 2],
        "negative count": good[:52] + (-5).to_bytes(4, "little", signed=True) + good[56:],
        "column": good[:col_at] + (shape[1] + 7).to_bytes(4, "little") + good[col_at + 4:],
        "tile pointer": good[:hdr + 4] + (10 ** 6).to_bytes(4, "little") + good[hdr + 8:],
    }
    r = api.TileMatrix(1)
    for what, blob in damaged.items():
        bad = tmp_path / "bad.bin"
        bad.write_bytes(blob)
        assert r.L.tsp_load(r.h, str(bad).encode()) == 1, what
    assert r.L.tsp_load(r.h, str(path).encode()) == 0
    m.close(); r.close()
