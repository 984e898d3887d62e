"""CPU tests of the C-ABI boundary: the library loads without a GPU, exports every symbol the header
declares, validates arguments like the reference, and refuses to compute without a device (no CPU path)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from paraselect_b200 import api, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.ensure_built()
    return api.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "psb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(psb_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), "symbol %s declared in include/psb.h is not exported" % n
    assert sorted(api.EXPORTS) == names


def test_struct_layouts_match_reference_views():
    # same field order and sizes as the reference's views on LP64
    assert C.sizeof(api.CoarseIndexView) == 16
    assert C.sizeof(api.ListLayoutView) == 32
    assert C.sizeof(api.PQCodeStorageView) == 32
    assert C.sizeof(api.QueryBatchView) == 32
    assert C.sizeof(api.SearchParams) == 20
    assert C.sizeof(api.SearchOutputView) == 24


def _tiny_index():
    rng = np.random.default_rng(0)
    return dict(centroids=rng.standard_normal((4, 8)).astype(np.float32),
                offsets=np.array([0, 2, 4, 6, 8], np.int64), reordered_ids=np.arange(8, dtype=np.int64),
                codes=rng.integers(0, 256, (8, 2)).astype(np.uint8),
                codebook=rng.standard_normal((2, 256, 4)).astype(np.float32),
                vectors=rng.standard_normal((8, 8)).astype(np.float32))


@pytest.mark.parametrize("mutate,msg", [
    (lambda ix: ix.update(offsets=np.array([1, 2, 4, 6, 8], np.int64)), "start at zero"),
    (lambda ix: ix.update(offsets=np.array([0, 4, 2, 6, 8], np.int64)), "monotonic"),
    (lambda ix: ix.update(offsets=np.array([0, 2, 4, 6, 7], np.int64)), "terminal offset"),
    (lambda ix: ix.update(codebook=np.zeros((3, 256, 2), np.float32)), "divide dim"),
    (lambda ix: ix.update(vectors=np.zeros((7, 8), np.float32)), "exact storage shape"),
])
def test_index_validation_matches_reference_rules(lib, mutate, msg):
    ix = _tiny_index()
    mutate(ix)
    with pytest.raises(api.InvalidArgument) as e:
        api.Session(ix, n_rerank=4)
    assert msg in str(e.value)


def test_no_device_means_error_not_fallback(lib):
    if api.device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(api.PsbError) as e:
        api.Session(_tiny_index(), n_rerank=4)
    assert e.value.status == 5  # PSB_NO_DEVICE
    with pytest.raises(api.PsbError) as e:
        api.coarse_host(np.zeros((1, 8), np.float32), np.zeros((4, 8), np.float32), 2)
    assert e.value.status == 5
    with pytest.raises(api.PsbError) as e:
        api.rerank_host(np.zeros((4, 8), np.float32), np.zeros((1, 8), np.float32), np.zeros((1, 4), np.int32), 2)
    assert e.value.status == 5


def test_rerank_argument_validation(lib):
    base = np.zeros((4, 8), np.float32)
    q = np.zeros((1, 8), np.float32)
    cand = np.zeros((1, 4), np.int32)
    with pytest.raises(api.InvalidArgument):
        api.rerank_host(base, q, cand, 0)
    with pytest.raises(api.InvalidArgument):
        api.rerank_host(base, q, cand, 2, candidate_count=5)  # stride < count
    with pytest.raises(api.InvalidArgument):
        api.rerank_host(base, q, cand, 2, counts=np.array([9], np.int32))


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "paraselect_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp", ".hpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("the oracle", ""), "%s mentions the oracle" % f


def test_index_build_glue_layout_and_reorder():
    """Host-side glue of the index build: list layout from an assignment (rows by (list, id)) and the reordered copy of the rows."""
    import numpy as np
    from paraselect_b200 import api
    rng = np.random.default_rng(3)
    n, nlist = 5000, 37
    assign = rng.integers(0, nlist, n).astype(np.int32)
    assign[assign == 5] = 6                      # an empty list
    off, rid = api.ivf_layout_from_assignment(assign, nlist)
    assert off[0] == 0 and off[-1] == n and off[5] == off[6]
    order = np.lexsort((np.arange(n), assign))   # by list, then by id
    assert np.array_equal(rid, order)
    assert np.array_equal(np.diff(off), np.bincount(assign, minlength=nlist))
    rows = rng.standard_normal((n, 12)).astype(np.float32)
    assert np.array_equal(api.reorder_rows(rows, rid), rows[rid])
    codes = rng.integers(0, 256, (n, 6)).astype(np.uint8)
    assert np.array_equal(api.reorder_rows(codes, rid), codes[rid])
    with pytest.raises(api.InvalidArgument):
        api.ivf_layout_from_assignment(np.array([0, 37], np.int32), nlist)
    bad = rid.copy(); bad[0] = bad[1]
    with pytest.raises(api.InvalidArgument):
        api.reorder_rows(rows, bad)


def test_nvtx_variant_builds_and_exports_the_same_symbols(lib):
    """-DPSB_USE_NVTX=1: stage ranges compiled in (NVTX 3 is header-only, nothing to link); same C ABI."""
    path = build.build_nvtx_variant()
    nv = C.CDLL(path)
    nv.psb_version.restype = C.c_char_p
    assert b"nvtx" in nv.psb_version() and b"nvtx" not in lib.psb_version()
    for name in api.EXPORTS:
        assert hasattr(nv, name), name


def test_ctypes_structs_have_the_sizes_the_library_was_built_with(lib):
    lib.psb_sizeof.restype = C.c_size_t
    for which, struct in ((0, api.Options), (1, api.Stats), (2, api.IndexView), (3, api.FlatIndexView), (4, api.RowCorrectionHeader),
                          (5, api.SearchParams)):
        assert lib.psb_sizeof(which) == C.sizeof(struct), struct.__name__
    assert lib.psb_sizeof(99) == 0
