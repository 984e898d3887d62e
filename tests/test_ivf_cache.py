"""The on-disk cache layout (cluster and PQ assets with JSON manifests) against the reference's own cache classes compiled in
place: what this package writes the reference loads, what the reference writes this package loads, and directory names,
layout ids and manifest matching agree.  Without the reference checkout only the self round trips run."""
import json
import os

import numpy as np
import pytest

import oracle
import synth
from paraselect_b200 import ivf_cache

needs_ref = pytest.mark.skipif(not oracle.have_ref_cache(), reason="reference cache code not compiled here")
RECIPE = {"family": "kmeans", "strategy": "lloyd", "iters": 10, "operator": "gemm", "precision": "fp32", "cluster_only": False,
          "sample_ratio": 1.0, "sample_limit": 0}


def small_index(seed=5):
    return synth.make_index(3000, 32, 20, 8, seed=seed, zipf=True, empty_lists=(7,))


def test_round_trip_and_lookup(tmp_path):
    ix = small_index()
    root = str(tmp_path)
    entry, pq_entry = ivf_cache.save_index(root, "synthetic", ix, RECIPE, pq_iters=8, training_rows=1000)
    assert os.path.basename(entry).startswith("asset-") and os.path.exists(os.path.join(entry, "manifest.json"))
    got = ivf_cache.load_index(root, "synthetic", 3000, 20, 32, RECIPE, 8, 256, 8, training_rows=1000)
    for key in ("centroids", "offsets", "reordered_ids", "codes", "codebook"):
        assert np.array_equal(got[key], ix[key]), key
    # identity is the manifest's fields: another recipe, dataset or PQ shape is a miss, not a wrong hit
    assert ivf_cache.load_index(root, "synthetic", 3000, 20, 32, dict(RECIPE, iters=11), 8, 256, 8, training_rows=1000) is None
    assert ivf_cache.load_index(root, "other", 3000, 20, 32, RECIPE, 8, 256, 8, training_rows=1000) is None
    assert ivf_cache.load_index(root, "synthetic", 3000, 20, 32, RECIPE, 8, 256, 9, training_rows=1000) is None
    # a payload of the wrong size is a miss as well
    with open(os.path.join(pq_entry, "codes.u8bin"), "ab") as f:
        f.write(b"\0")
    assert ivf_cache.load_index(root, "synthetic", 3000, 20, 32, RECIPE, 8, 256, 8, training_rows=1000) is None


def test_manifest_matching_rules():
    m = dict(ivf_cache.identity("cluster", "d"), n_vectors=10, build={"a": 1, "b": 2.5}, extra="x")
    assert ivf_cache.matches(m, {"n_vectors": 10, "build": {"a": 1}})
    assert not ivf_cache.matches(m, {"n_vectors": 10.0})            # a float does not match an integer
    assert not ivf_cache.matches(m, {"n_vectors": "10"})
    assert not ivf_cache.matches(m, {"missing": 1})
    assert not ivf_cache.matches(m, {"build": {"a": 2}})
    assert not ivf_cache.matches([], {}) and ivf_cache.matches(m, {})


def test_invalid_requests_are_refused(tmp_path):
    with pytest.raises(ValueError):
        ivf_cache.pq_request("d", 100, 32, 4, 8, 256, "x", 8, training_rows=0)            # a sample needs its row count
    with pytest.raises(ValueError):
        ivf_cache.pq_request("d", 100, 32, 4, 8, 256, "x", 8, residual=True, training_rows=50)  # "full" means all rows
    with pytest.raises(ValueError):
        ivf_cache.pq_request("d", 100, 32, 4, 8, 256, "x", 8, trainer="opq-gpu-v1", training_rows=50)
    ix = small_index()
    with pytest.raises(ValueError):
        ivf_cache.save_cluster(str(tmp_path), "d", ix["centroids"], ix["reordered_ids"], ix["offsets"][:-1], RECIPE)


@needs_ref
def test_reference_loads_what_this_package_writes(tmp_path):
    ix = small_index(6)
    root = str(tmp_path)
    entry, layout = ivf_cache.save_cluster(root, "synthetic", ix["centroids"], ix["reordered_ids"], ix["offsets"], RECIPE)
    ref = oracle.ref_cluster_load(root, "synthetic", 3000, 20, 32, json.dumps(RECIPE))
    assert ref is not None and ref["entry"] == entry and ref["layout_id"] == layout
    assert np.array_equal(ref["centroids"], ix["centroids"]) and np.array_equal(ref["reordered_ids"], ix["reordered_ids"])
    assert np.array_equal(ref["offsets"], ix["offsets"]) and np.array_equal(ref["counts"], np.diff(ix["offsets"]))
    assert oracle.ref_cluster_load(root, "synthetic", 3000, 20, 32, json.dumps(dict(RECIPE, iters=3))) is None
    for residual, kw in ((False, dict(training_rows=1200)), (True, dict())):
        req = ivf_cache.pq_request("synthetic", 3000, 32, 20, 8, 256, layout, 8, residual=residual, **kw)
        pq_entry = ivf_cache.save_pq(root, req, ix["codebook"], ix["codes"])
        got = oracle.ref_pq_load(root, "synthetic", 3000, 32, 20, layout, 8, 256, 8, residual, kw.get("training_rows", 0))
        assert got is not None and got["entry"] == pq_entry
        assert np.array_equal(got["codebook"], ix["codebook"]) and np.array_equal(got["codes"], ix["codes"])


@needs_ref
def test_this_package_loads_what_the_reference_writes(tmp_path):
    ix = small_index(7)
    root = str(tmp_path)
    oracle.ref_cluster_save(root, "synthetic", ix["centroids"], ix["reordered_ids"], ix["offsets"], json.dumps(RECIPE))
    cl = ivf_cache.load_cluster(root, "synthetic", 3000, 20, 32, RECIPE)
    assert cl is not None and cl["layout_id"] == ivf_cache.cluster_layout_id(cl["entry"])
    assert os.path.basename(cl["entry"]) == ivf_cache.storage_id(json.load(open(os.path.join(cl["entry"], "manifest.json"))))
    assert np.array_equal(cl["centroids"], ix["centroids"]) and np.array_equal(cl["reordered_ids"], ix["reordered_ids"])
    assert np.array_equal(cl["offsets"], ix["offsets"])
    for residual, rows in ((False, 1500), (True, 0)):
        oracle.ref_pq_save(root, "synthetic", 3000, 32, 20, cl["layout_id"], ix["codebook"], ix["codes"], 8, residual, rows)
    got = ivf_cache.load_index(root, "synthetic", 3000, 20, 32, RECIPE, 8, 256, 8, training_rows=1500)
    assert got is not None and np.array_equal(got["codes"], ix["codes"]) and np.array_equal(got["codebook"], ix["codebook"])
    got_r = ivf_cache.load_index(root, "synthetic", 3000, 20, 32, RECIPE, 8, 256, 8, residual=True)
    assert got_r is not None and np.array_equal(got_r["codes"], ix["codes"])


@needs_ref
def test_directory_names_and_matching_equal_the_reference():
    manifests = [ivf_cache.cluster_request("sift-1m", 1000000, 1024, 128, RECIPE, layout_id="00ab"),
                 ivf_cache.pq_request("d", 5000, 96, 64, 48, 256, "feed", 25, training_rows=2000),
                 ivf_cache.pq_request("d", 5000, 96, 64, 48, 256, "feed", 25, residual=True),
                 ivf_cache.pq_request("d", 5000, 96, 64, 48, 256, "feed", 25, trainer="opq-gpu-v1", training_rows=2000,
                                      opq=dict(iters=4, training_rows=3000, seed=7)),
                 {"z": [1, 2, {"k": "v"}], "a": -3, "f": 0.25, "s": 'text with "quotes" and / slash', "b": True, "n": None}]
    for m in manifests:
        assert ivf_cache.storage_id(m) == oracle.ref_storage_id(json.dumps(m))
    a = dict(manifests[1], extra=1)
    for expected in (manifests[1], {"m": 48}, {"m": 48.0}, {"training": {"rows": 2000}}, {"training": {"rows": 2001}}, {"nope": 1},
                     {"trainer": "plain-pq-ooc-v2"}, {"dsub": "2"}):
        assert int(ivf_cache.matches(a, expected)) == oracle.ref_manifest_matches(json.dumps(a), json.dumps(expected)), expected


def test_opq_rotation_file_round_trip(tmp_path):
    rng = np.random.default_rng(3)
    rot = np.linalg.qr(rng.standard_normal((24, 24)))[0].astype(np.float32)
    key = ivf_cache.opq_cache_key("my data/set", 5000, 24, 2000, 8, 256, 4, 25, 12345)
    path = ivf_cache.save_opq_rotation(str(tmp_path), key, rot, 2000, 8, 256, 4, 25, 12345)
    assert os.path.basename(path) == "my_data_set__n5000__train2000__d24__M8__K256__opq4__pq25__seed12345.opq"
    assert os.path.getsize(path) == 36 + 24 * 24 * 4
    assert np.array_equal(ivf_cache.load_opq_rotation(str(tmp_path), key, 24), rot)
    assert ivf_cache.load_opq_rotation(str(tmp_path), key, 32) is None and ivf_cache.load_opq_rotation(str(tmp_path), "other", 24) is None


@pytest.mark.skipif(not oracle.have_ref_train(), reason="reference training code not compiled here")
def test_opq_rotation_file_against_the_reference(tmp_path):
    rng = np.random.default_rng(4)
    rot = rng.standard_normal((16, 16)).astype(np.float32)
    d1, d2 = str(tmp_path / "a"), str(tmp_path / "b")
    key = oracle.ref_opq_save(d1, "sift 1m", 9000, 3000, rot, 4, 256, 6, 20, 77)
    assert key == ivf_cache.opq_cache_key("sift 1m", 9000, 16, 3000, 4, 256, 6, 20, 77)
    assert np.array_equal(ivf_cache.load_opq_rotation(d1, key, 16), rot)
    mine = ivf_cache.save_opq_rotation(d2, key, rot, 3000, 4, 256, 6, 20, 77)
    theirs = os.path.join(d1, os.path.basename(mine))
    assert open(mine, "rb").read() == open(theirs, "rb").read()
    assert np.array_equal(oracle.ref_opq_load(d2, key, 16), rot)


def sign_asset(n=500, dim=128, seed=3):
    rng = np.random.default_rng(seed)
    return (rng.integers(0, 2 ** 32, (n, dim // 32), dtype=np.uint64).astype(np.uint32),
            rng.uniform(0.1, 3.0, n).astype(np.float32))


def test_sign_code_asset_round_trip(tmp_path):
    codes, scales = sign_asset()
    root = ivf_cache.sign_cache_root(str(tmp_path / "cluster-entry"))
    req = ivf_cache.sign_request("synthetic", 500, 128, 20, 17, "layout0")
    entry = ivf_cache.save_sign(root, req, codes, scales)
    assert os.path.dirname(entry) == root and sorted(os.listdir(entry)) == ["codes.u32bin", "manifest.json", "scales.f32bin"]
    got = ivf_cache.load_sign(root, req)
    assert got["entry"] == entry and np.array_equal(got["codes"], codes) and np.array_equal(got["scales"], scales)
    # every field that changes the encoded bytes is part of the identity
    for other in (ivf_cache.sign_request("synthetic", 500, 128, 20, 18, "layout0"),
                  ivf_cache.sign_request("synthetic", 500, 128, 20, 17, "layout1"),
                  ivf_cache.sign_request("synthetic", 500, 128, 21, 17, "layout0"),
                  ivf_cache.sign_request("synthetic", 500, 128, 20, 17, "layout0", builder="other")):
        assert ivf_cache.load_sign(root, other) is None
    with open(os.path.join(entry, "scales.f32bin"), "ab") as f:
        f.write(b"\0\0\0\0")
    assert ivf_cache.load_sign(root, req) is None   # a payload of the wrong size is a miss
    with pytest.raises(ValueError):
        ivf_cache.sign_request("synthetic", 500, 100, 20, 17, "layout0")


@needs_ref
def test_sign_code_asset_against_the_reference(tmp_path):
    codes, scales = sign_asset(seed=4)
    root = ivf_cache.sign_cache_root(str(tmp_path / "a"))
    req = ivf_cache.sign_request("synthetic", 500, 128, 20, 17, "layout0")
    entry = ivf_cache.save_sign(root, req, codes, scales)
    ref = oracle.ref_sign_cache_map(root, "synthetic", 500, 128, 20, 17, "layout0")
    assert ref is not None and ref["entry"] == entry
    assert np.array_equal(ref["codes"], codes) and np.array_equal(ref["scales"], scales)
    assert oracle.ref_sign_cache_map(root, "synthetic", 500, 128, 20, 18, "layout0") is None
    # the other way round: the reference publishes a staged build, this package finds and reads it
    root_b = ivf_cache.sign_cache_root(str(tmp_path / "b"))
    staged = os.path.join(root_b, ".building-1")
    os.makedirs(staged)
    oracle.ref_sign_cache_publish(root_b, "synthetic", staged, 500, 128, 20, 17, "layout0", codes, scales)
    got = ivf_cache.load_sign(root_b, req)
    assert got is not None and os.path.basename(got["entry"]) == os.path.basename(entry)   # the same directory name on both sides
    assert np.array_equal(got["codes"], codes) and np.array_equal(got["scales"], scales)
    assert json.load(open(os.path.join(got["entry"], "manifest.json"))) == json.load(open(os.path.join(entry, "manifest.json")))
