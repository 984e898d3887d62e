"""Per-row correction of residual-PQ indices: the host utilities of the C ABI against the reference's own builder and
quantiser (src/index/row_correction/row_correction.cpp, src/quantization/row_correction/u16.h), compiled in place when the
reference checkout is there; format and round-trip checks otherwise."""
import os
import struct

import numpy as np
import pytest

import oracle
from paraselect_b200 import api

needs_ref = pytest.mark.skipif(not oracle.have_ref_rowcorr(), reason="reference row-correction code not compiled here")


def _index(seed, n=5000, nlist=17, m=8, k=16, dsub=4, scale=3.0):
    rng = np.random.default_rng(seed)
    cen = (rng.standard_normal((nlist, m * dsub)) * scale).astype(np.float32)
    cb = (rng.standard_normal((m, k, dsub)) * scale).astype(np.float32)
    sizes = rng.multinomial(n, np.ones(nlist) / nlist)
    sizes[min(3, nlist - 1)] = 0  # an empty list
    off = np.zeros(nlist + 1, np.int64); off[1:] = np.cumsum(sizes)
    codes = rng.integers(0, k, (int(off[-1]), m), dtype=np.uint8)
    return cen, off, codes, cb


def _values_numpy(cen, off, codes, cb):
    m = cb.shape[0]
    recon = np.concatenate([cb[j][codes[:, j]] for j in range(m)], axis=1).astype(np.float64)
    lists = np.repeat(np.arange(len(off) - 1), np.diff(off))
    c = cen[lists].astype(np.float64)
    return ((recon * recon).sum(1) + 2.0 * (c * recon).sum(1))


def test_values_are_recon_norm_plus_twice_centroid_dot():
    cen, off, codes, cb = _index(1)
    got = api.row_correction_compute(cen, off, codes, cb)
    want = _values_numpy(cen, off, codes, cb)
    assert np.allclose(got, want, rtol=1e-6, atol=1e-4)


def test_affine_u16_rounds_up_and_file_layout(tmp_path):
    cen, off, codes, cb = _index(2)
    v = api.row_correction_compute(cen, off, codes, cb)
    hdr, u = api.row_correction_quantize_u16(v)
    assert bytes(hdr.magic).ljust(8, b"\0") == b"ISRC16\0\0" and hdr.version == 2 and hdr.header_bytes == 32 and hdr.count == v.size
    assert hdr.offset == np.floor(v.min()) and u.max() <= 65534
    dec = np.float32(hdr.offset) + np.float32(hdr.scale) * u.astype(np.float32)
    assert np.all(dec.astype(np.float64) >= v.astype(np.float64) - 1e-3 * hdr.scale)   # rounded up: never undercuts (one fp32 rounding of slack)
    assert np.all(np.abs(dec - v) <= hdr.scale * 1.01)
    path = str(tmp_path / "row_correction.u16a")
    api.row_correction_write_u16(path, hdr, u)
    raw = open(path, "rb").read()
    assert len(raw) == 32 + 2 * v.size
    magic, version, hb, count, scale, offset = struct.unpack("<8sIIQff", raw[:32])
    assert (magic, version, hb, count) == (b"ISRC16\0\0", 2, 32, v.size) and scale == hdr.scale and offset == hdr.offset
    hdr2, u2 = api.row_correction_read_u16(path)
    assert hdr2.count == hdr.count and hdr2.scale == hdr.scale and np.array_equal(u, u2)


def test_read_refuses_foreign_and_truncated_files(tmp_path):
    bad = tmp_path / "bad.u16a"
    bad.write_bytes(b"NOTMAGIC" + bytes(24))
    with pytest.raises(api.PsbError):
        api.row_correction_read_u16(str(bad))
    hdr, u = api.row_correction_quantize_u16(np.arange(100, dtype=np.float32))
    good = tmp_path / "good.u16a"
    api.row_correction_write_u16(str(good), hdr, u)
    trunc = tmp_path / "trunc.u16a"
    trunc.write_bytes(good.read_bytes()[:-10])
    with pytest.raises(api.PsbError):
        api.row_correction_read_u16(str(trunc))


def test_quantiser_refuses_non_finite_values():
    v = np.array([1.0, np.inf, 2.0], np.float32)
    with pytest.raises(api.PsbError):
        api.row_correction_quantize_u16(v)
    # a constant array quantises with scale 1 (zero range)
    hdr, u = api.row_correction_quantize_u16(np.full(7, 3.0, np.float32))
    assert hdr.scale == 1.0 and hdr.offset == 3.0 and np.all(u == 0)


@needs_ref
@pytest.mark.parametrize("seed,shape", [(3, dict()), (4, dict(n=20000, nlist=64, m=16, k=256, dsub=8, scale=40.0)),
                                        (5, dict(n=300, nlist=2, m=2, k=3, dsub=1, scale=10.0))])
def test_payload_bytes_equal_the_reference_builders(tmp_path, seed, shape):
    cen, off, codes, cb = _index(seed, **shape)
    payload, audit = oracle.ref_rc_build_pq(str(tmp_path), cen, off, codes, cb)
    v = api.row_correction_compute(cen, off, codes, cb)
    assert np.array_equal(v.view(np.uint32), audit.view(np.uint32))     # the fp32 values, bit for bit
    hdr, u = api.row_correction_quantize_u16(v)
    mine = str(tmp_path / "mine.u16a")
    api.row_correction_write_u16(mine, hdr, u)
    assert open(mine, "rb").read() == payload                           # header and codes, byte for byte
    hdr2, u2 = api.row_correction_read_u16(os.path.join(str(tmp_path), "row_correction.u16a"))
    assert np.array_equal(u2, u) and hdr2.scale == hdr.scale and hdr2.offset == hdr.offset


@needs_ref
def test_fixed_model_quantiser_equals_the_reference():
    # the reference's own exhaustive toy model (tests/unit/quantization/test_row_correction_u16.cpp) ...
    centers = np.array([[3, -5], [-11, 7]], np.float32)
    words = np.array([[[-10], [2], [19]], [[-13], [4], [25]]], np.float32)
    sc, off = api.row_correction_model_u16(centers, words)
    assert (sc, off) == oracle.ref_rc_for_pq(centers, words)
    for c in range(2):
        for a in range(3):
            for b in range(3):
                v = oracle.ref_rc_pq_value(centers[c], words, [a, b])
                code = api.row_correction_encode_u16(np.array([v], np.float32), sc, off)[0]
                assert code == oracle.ref_rc_encode(sc, off, v) and code <= 65534
                assert abs(oracle.ref_rc_decode(sc, off, int(code)) - v) <= sc * 1.01
    # ... and random models at the reference test's dimensions
    rng = np.random.default_rng(12345)
    for dim in (16, 128, 160):
        m, k = 16, 8
        cen = rng.uniform(-1000, 1000, (3, dim)).astype(np.float32)
        cb = rng.uniform(-1000, 1000, (m, k, dim // m)).astype(np.float32)
        sc, off = api.row_correction_model_u16(cen, cb)
        assert (sc, off) == oracle.ref_rc_for_pq(cen, cb)
        codes = rng.integers(0, k, (2000, m), dtype=np.uint8)
        lists = np.arange(2000) % 3
        vals = np.array([oracle.ref_rc_pq_value(cen[lists[i]], cb, codes[i]) for i in range(2000)], np.float32)
        mine = api.row_correction_encode_u16(vals, sc, off)
        ref = np.array([oracle.ref_rc_encode(sc, off, float(x)) for x in vals], np.uint16)
        assert np.array_equal(mine, ref)
    for bad in (np.inf, np.nan, np.finfo(np.float32).max):
        with pytest.raises(api.PsbError):
            api.row_correction_model_u16(np.array([[bad]], np.float32), np.array([[[bad]]], np.float32))
        with pytest.raises(api.PsbError):
            api.row_correction_encode_u16(np.array([bad], np.float32), sc, off)
