"""The reference's on-disk caches of build products, read and written in its own layout, so that an index built by the
reference's tools loads into a psb session and the other way round.

An asset is a directory holding a `manifest.json` (its identity: structured fields, never the directory name) and payload
files in the "binary with header" form: uint32 n, uint32 dim, then n * dim values.

    cluster asset    centroids.fbin [nlist][dim] f32, reordered_indices.ibin [n][1] i64, cluster_counts.ibin [nlist][1] i32,
                     cluster_offsets.ibin [nlist + 1][1] i64, meta.json          src/dataset/cache/cluster_cache.cpp:159-275
    PQ asset         codebook.fbin [M * K][dsub] f32, codes.u8bin [n][M] u8 (cluster-reordered), meta.json
                                                                                  src/dataset/cache/residual_pq_cache.cpp:20-275
    manifests        identity fields, matching, lookup, directory names           src/dataset/cache/cache_manifest.h:13-104

Files are committed the way the reference commits them: written under a temporary name, renamed into place, the manifest
last (src/index/ivf_cache/cache_file.h:18-36, cache_manifest.h:86-102).  Host-side only; nothing here touches a GPU.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np

SCHEMA = "paraselect.cache"
SCHEMA_VERSION = 2


# ---------------------------------------------------------------------------------------------- manifests
def identity(kind: str, dataset: str) -> dict:
    """The fields every manifest starts from (cache_manifest.h:32-35)."""
    return {"schema": SCHEMA, "schema_version": SCHEMA_VERSION, "asset_type": kind, "dataset": dataset}


def _kind(v):
    """JSON type of a value; all integers are one kind, as the reference's comparison treats signed and unsigned alike."""
    if isinstance(v, bool):
        return "bool"
    if isinstance(v, int):
        return "int"
    if isinstance(v, float):
        return "float"
    if isinstance(v, str):
        return "str"
    if isinstance(v, (list, tuple)):
        return "array"
    if isinstance(v, dict):
        return "object"
    return "null" if v is None else type(v).__name__


def matches(actual, expected) -> bool:
    """Every field of `expected` is in `actual` with the same type and value, objects compared field by field
    (cache_manifest.h:17-30): structured fields only, never formatting or directory names."""
    if not isinstance(actual, dict) or not isinstance(expected, dict):
        return False
    for key, want in expected.items():
        if key not in actual:
            return False
        have = actual[key]
        if isinstance(want, dict):
            if not matches(have, want):
                return False
        elif _kind(have) != _kind(want) or have != want:
            return False
    return True


def dump_compact(manifest) -> str:
    """The serialisation the directory name is hashed from: keys in sorted order, no white space."""
    return json.dumps(manifest, sort_keys=True, separators=(",", ":"), ensure_ascii=False)


def _fnv1a(data: bytes, h: int = 1469598103934665603) -> int:
    for b in data:
        h ^= b
        h = (h * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def storage_id(manifest) -> str:
    """asset-<FNV-1a of the compact manifest, 16 hex digits> (cache_manifest.h:64-76): a compact path name only."""
    return "asset-%016x" % _fnv1a(dump_compact(manifest).encode("utf-8"))


def canonical_entry(root: str, manifest) -> str:
    return os.path.join(root, storage_id(manifest))


def find(root: str, request) -> str:
    """The one directory under `root` whose manifest matches `request` ("" when none; ambiguity is an error)."""
    if not root or not os.path.exists(root):
        return ""
    match = ""
    for d, _, files in os.walk(root):
        if d == root or "manifest.json" not in files:
            continue
        path = os.path.join(d, "manifest.json")
        try:
            manifest = json.load(open(path))
        except ValueError as e:
            raise RuntimeError("invalid cache manifest %s: %s" % (path, e))
        if not matches(manifest, request):
            continue
        if match:
            raise RuntimeError("ambiguous cache assets: %s and %s" % (match, d))
        match = d
    return match


def publish(entry: str, manifest) -> None:
    """Writes manifest.json last, through a temporary name: an asset without it is not an asset."""
    target = os.path.join(entry, "manifest.json")
    tmp = "%s.tmp.%d" % (target, os.getpid())
    try:
        with open(tmp, "w") as f:
            f.write(json.dumps(manifest, sort_keys=True, indent=2, ensure_ascii=False) + "\n")
        os.rename(tmp, target)
    except BaseException:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise


# ---------------------------------------------------------------------------------------------- payload files
def write_binary(path: str, array, dim=None) -> None:
    """uint32 n, uint32 dim, data; committed by rename (cache_file.h:18-36)."""
    a = np.ascontiguousarray(array)
    if a.ndim == 1:
        n, d = a.shape[0], 1
    else:
        n, d = a.shape[0], int(np.prod(a.shape[1:]))
    if dim is not None:
        if (n * d) % dim:
            raise ValueError("array does not divide into rows of %d" % dim)
        n, d = n * d // dim, dim
    if n >= 1 << 32 or d >= 1 << 32:
        raise ValueError("binary header holds 32-bit shapes")
    tmp = path + ".tmp"
    try:
        with open(tmp, "wb") as f:
            f.write(struct.pack("<II", n, d))
            a.tofile(f)
        os.rename(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise


def read_binary(path: str, dtype, n: int, dim: int, mmap: bool = False):
    """The payload as [n][dim]; header or size other than expected is an error (mapped_array.h:55-78)."""
    size = os.path.getsize(path)
    if size < 8:
        raise RuntimeError("mapped binary header is truncated: " + path)
    with open(path, "rb") as f:
        hn, hd = struct.unpack("<II", f.read(8))
    if hn != n or hd != dim:
        raise RuntimeError("mapped binary shape mismatch: %s holds [%d][%d], expected [%d][%d]" % (path, hn, hd, n, dim))
    dt = np.dtype(dtype)
    if size != 8 + n * dim * dt.itemsize:
        raise RuntimeError("mapped binary size mismatch: " + path)
    if mmap:
        return np.memmap(path, dtype=dt, mode="r", offset=8, shape=(n, dim))
    return np.fromfile(path, dtype=dt, offset=8).reshape(n, dim)


# ---------------------------------------------------------------------------------------------- cluster asset
CLUSTER_FILES = ("centroids.fbin", "reordered_indices.ibin", "cluster_counts.ibin", "cluster_offsets.ibin")


def cluster_layout_id(entry: str) -> str:
    """Identity of a cluster layout: FNV-1a over, per payload file, its name, its size (8 bytes) and its first and last 4 KB
    (cluster_cache.cpp:57-103).  PQ assets name the layout they were encoded for by this id."""
    h = 1469598103934665603
    for name in CLUSTER_FILES:
        path = os.path.join(entry, name)
        if not os.path.exists(path) or os.path.getsize(path) <= 0:
            return ""
        size = os.path.getsize(path)
        h = _fnv1a(name.encode(), h)
        h = _fnv1a(struct.pack("<q", size), h)
        first = min(4096, size)
        with open(path, "rb") as f:
            h = _fnv1a(f.read(first), h)
            if size > first:
                f.seek(size - first)
                h = _fnv1a(f.read(first), h)
    return "%016x" % h


def _check_layout(n_vectors, counts, offsets):
    nlist = counts.shape[0]
    if nlist == 0 or offsets.shape[0] != nlist + 1 or offsets[0] != 0 or offsets[nlist] != n_vectors:
        return False
    return bool(np.all(np.diff(offsets) == counts) and np.all(counts >= 0))


def cluster_request(dataset, n_vectors, nlist, dim, build_recipe, layout_id=None) -> dict:
    req = identity("cluster", dataset)
    recipe = json.loads(build_recipe) if isinstance(build_recipe, str) else build_recipe
    req.update({"n_vectors": int(n_vectors), "nlist": int(nlist), "dim": int(dim), "build": recipe})
    if layout_id:
        req["cluster_layout_id"] = layout_id
    return req


def save_cluster(root, dataset, centroids, reordered_indices, cluster_offsets, build_recipe):
    """Writes a cluster asset (ClusterCache::save + publish_staged); returns (entry directory, layout id)."""
    cen = np.ascontiguousarray(centroids, np.float32)
    ids = np.ascontiguousarray(reordered_indices, np.int64)
    off = np.ascontiguousarray(cluster_offsets, np.int64)
    nlist, dim = cen.shape
    n = ids.shape[0]
    counts = np.diff(off).astype(np.int32)
    if not _check_layout(n, counts, off):
        raise ValueError("invalid cluster offsets/counts")
    recipe = json.loads(build_recipe) if isinstance(build_recipe, str) else build_recipe
    staging = os.path.join(root, ".building-%d" % os.getpid())
    os.makedirs(staging, exist_ok=True)
    with open(os.path.join(staging, "meta.json"), "w") as f:
        f.write(json.dumps({"dataset_name": dataset, "n_lists": nlist, "build": recipe, "n_vectors": n, "n_dim": dim,
                            "n_clusters_actual": nlist}, sort_keys=True, indent=2) + "\n")
    write_binary(os.path.join(staging, "centroids.fbin"), cen)
    write_binary(os.path.join(staging, "reordered_indices.ibin"), ids)
    write_binary(os.path.join(staging, "cluster_counts.ibin"), counts)
    write_binary(os.path.join(staging, "cluster_offsets.ibin"), off)
    layout = cluster_layout_id(staging)
    manifest = cluster_request(dataset, n, nlist, dim, recipe)
    manifest.update({"n_clusters_actual": nlist, "cluster_layout_id": layout})
    entry = canonical_entry(root, manifest)
    if entry != staging:
        if os.path.exists(entry):
            raise RuntimeError("cluster publication destination already exists: " + entry)
        os.rename(staging, entry)
    publish(entry, manifest)
    return entry, layout


def load_cluster(root, dataset, n_vectors, nlist, dim, build_recipe, layout_id=None, mmap=False):
    """ClusterCache::try_map: None on a miss, else dict(entry, layout_id, centroids, reordered_ids, counts, offsets)."""
    req = cluster_request(dataset, n_vectors, nlist, dim, build_recipe, layout_id)
    entry = find(root, req)
    if not entry:
        return None
    manifest = json.load(open(os.path.join(entry, "manifest.json")))
    if manifest.get("build") != req["build"]:
        return None
    try:
        cen = read_binary(os.path.join(entry, "centroids.fbin"), np.float32, nlist, dim, mmap)
        ids = read_binary(os.path.join(entry, "reordered_indices.ibin"), np.int64, n_vectors, 1, mmap).reshape(-1)
        counts = read_binary(os.path.join(entry, "cluster_counts.ibin"), np.int32, nlist, 1, mmap).reshape(-1)
        off = read_binary(os.path.join(entry, "cluster_offsets.ibin"), np.int64, nlist + 1, 1, mmap).reshape(-1)
    except (RuntimeError, OSError):
        return None
    layout = manifest.get("cluster_layout_id")
    if not _check_layout(n_vectors, counts, off) or not isinstance(layout, str) or not layout:
        return None
    return dict(entry=entry, layout_id=layout, centroids=cen, reordered_ids=ids, counts=counts, offsets=off)


# ---------------------------------------------------------------------------------------------- PQ asset
def pq_request(dataset, n_vectors, dim, nlist, m, k, cluster_layout_id_, pq_iters, residual=False, trainer=None,
               training_sampling=None, training_rows=0, codes_layout="cluster-reordered-[N,M]", opq=None) -> dict:
    """The identity of a PQ asset (manifest_identity, residual_pq_cache.cpp:20-45).  Defaults follow the reference's two
    request builders: residual = the residual trainer on all rows ("gpu-ooc", "full"); plain = "plain-pq-ooc-v2" on a sample
    of training_rows rows (plain_pq_cache.h:11-32).  opq: dict(iters, training_rows, seed) for an OPQ-rotated codebook."""
    pq_type = "residual" if residual else "plain"
    trainer = trainer or ("gpu-ooc" if residual else "plain-pq-ooc-v2")
    sampling = training_sampling or ("full" if residual else "sample")
    rows = int(training_rows) if training_rows > 0 else int(n_vectors)
    if sampling not in ("full", "prefix", "sample") or rows <= 0 or rows > n_vectors or (sampling == "full" and rows != n_vectors) \
            or (sampling != "full" and training_rows <= 0):
        raise ValueError("invalid PQ training recipe")
    if dim % m:
        raise ValueError("dim must be a multiple of m")
    req = identity("residual_pq" if residual else "pq", dataset)
    req.update({"n_vectors": int(n_vectors), "nlist": int(nlist), "dim": int(dim), "m": int(m), "k": int(k), "dsub": dim // m,
                "pq_type": pq_type, "pq_iters": int(pq_iters), "training": {"sampling": sampling, "rows": rows},
                "trainer": trainer, "cluster_layout_id": cluster_layout_id_, "codes_layout": codes_layout})
    if opq:
        if trainer != "opq-gpu-v1" or opq.get("training_rows", 0) <= 0:
            raise ValueError("invalid OPQ build recipe")
        req["transform"] = {"kind": "opq", "iters": int(opq["iters"]), "training_rows": int(opq["training_rows"]),
                            "seed": int(opq.get("seed", 0))}
    elif trainer == "opq-gpu-v1":
        raise ValueError("OPQ build recipe is missing")
    return req


def save_pq(root, request, codebook, codes):
    """Writes a PQ asset (ResidualPQCache::save); returns the entry directory.  codebook [M][K][dsub], codes [n][M]."""
    m, k, dsub, n = request["m"], request["k"], request["dsub"], request["n_vectors"]
    cb = np.ascontiguousarray(codebook, np.float32).reshape(m * k, dsub)
    cd = np.ascontiguousarray(codes, np.uint8).reshape(n, m)
    entry = canonical_entry(root, request)
    os.makedirs(entry, exist_ok=True)
    manifest_path = os.path.join(entry, "manifest.json")
    if os.path.exists(manifest_path):
        os.remove(manifest_path)   # unpublish before replacing any payload
    write_binary(os.path.join(entry, "codebook.fbin"), cb)
    meta = {"format": "paraselect-pq-cache", "dataset_name": request["dataset"], "n_vectors": n, "n_dim": request["dim"],
            "n_lists": request["nlist"], "cluster_layout_id": request["cluster_layout_id"], "pq_type": request["pq_type"],
            "pq_m": m, "pq_k": k, "pq_d_sub": dsub, "pq_iters": request["pq_iters"], "trainer": request["trainer"],
            "training": request["training"], "codebook_layout": "[M,K,dsub]", "codes_layout": request["codes_layout"]}
    if "transform" in request:
        meta["transform"] = request["transform"]
    with open(os.path.join(entry, "meta.json.tmp"), "w") as f:
        f.write(json.dumps(meta, sort_keys=True, indent=2) + "\n")
    os.rename(os.path.join(entry, "meta.json.tmp"), os.path.join(entry, "meta.json"))
    write_binary(os.path.join(entry, "codes.u8bin"), cd)
    publish(entry, request)
    return entry


def load_pq(root, request, mmap=False):
    """ResidualPQCache::try_map: None on a miss, else dict(entry, codebook [M][K][dsub], codes [n][M])."""
    entry = find(root, request)
    if not entry:
        return None
    m, k, dsub, n = request["m"], request["k"], request["dsub"], request["n_vectors"]
    try:
        cb = read_binary(os.path.join(entry, "codebook.fbin"), np.float32, m * k, dsub, mmap)
        cd = read_binary(os.path.join(entry, "codes.u8bin"), np.uint8, n, m, mmap)
    except (RuntimeError, OSError):
        return None
    return dict(entry=entry, codebook=cb.reshape(m, k, dsub), codes=cd)


# ---------------------------------------------------------------------------------------------- sign-code asset
def sign_request(dataset, n_vectors, dim, nlist, rotation_seed, cluster_layout_id_, builder="chunk-residual-l1-v1",
                 codes_layout="cluster-reordered-[N,words]-u32") -> dict:
    """The identity of a 1-bit sign-code asset (manifest_identity, src/dataset/cache/turboquant_cache.cpp:18-26): every field
    that changes the encoded bytes is part of it.  The reference stores such assets for 128-dimensional rows only
    (dim / 32 words per code); any multiple of 32 is accepted here."""
    if dim <= 0 or dim % 32 or n_vectors <= 0 or nlist <= 0 or rotation_seed < 0:
        raise ValueError("invalid sign-code cache request")
    req = identity("turboquant", dataset)
    req.update({"n_vectors": int(n_vectors), "dim": int(dim), "nlist": int(nlist), "words_per_code": dim // 32,
                "rotation_seed": int(rotation_seed), "builder": builder, "cluster_layout_id": cluster_layout_id_,
                "codes_layout": codes_layout})
    return req


def sign_cache_root(cluster_entry: str) -> str:
    """Sign-code assets live under the cluster asset they encode (src/index/ivf_cache/turboquant.cu:46)."""
    return os.path.join(cluster_entry, "tq")


def save_sign(root, request, codes, scales):
    """Writes a sign-code asset - codes.u32bin [n][words], scales.f32bin [n][1], manifest last
    (TurboQuantCache::publish_staged); returns the entry directory."""
    n, words = request["n_vectors"], request["words_per_code"]
    cd = np.ascontiguousarray(codes).view(np.uint32).reshape(n, words)
    sc = np.ascontiguousarray(scales, np.float32).reshape(n, 1)
    entry = canonical_entry(root, request)
    os.makedirs(entry, exist_ok=True)
    manifest_path = os.path.join(entry, "manifest.json")
    if os.path.exists(manifest_path):
        os.remove(manifest_path)   # unpublish before replacing any payload
    write_binary(os.path.join(entry, "codes.u32bin"), cd)
    write_binary(os.path.join(entry, "scales.f32bin"), sc)
    publish(entry, request)
    return entry


def load_sign(root, request, mmap=False):
    """TurboQuantCache::try_map: None on a miss or a payload that does not fit the request, else
    dict(entry, codes [n][words] uint32, scales [n] float32)."""
    entry = find(root, request)
    if not entry:
        return None
    n, words = request["n_vectors"], request["words_per_code"]
    try:
        cd = read_binary(os.path.join(entry, "codes.u32bin"), np.uint32, n, words, mmap)
        sc = read_binary(os.path.join(entry, "scales.f32bin"), np.float32, n, 1, mmap)
    except (RuntimeError, OSError):
        return None
    return dict(entry=entry, codes=cd, scales=sc.reshape(n))


# ---------------------------------------------------------------------------------------------- an index for api.Session
def load_index(root, dataset, n_vectors, nlist, dim, build_recipe, m, k, pq_iters, residual=False, vectors=None, mmap=False, **pq_kw):
    """The view arrays of a psb session from a cluster asset and the PQ asset encoded for its layout; None when either is
    missing.  vectors: the exact rows in LIST order (the caller's, as in the reference's views), or None."""
    cl = load_cluster(root, dataset, n_vectors, nlist, dim, build_recipe, mmap=mmap)
    if cl is None:
        return None
    pq = load_pq(root, pq_request(dataset, n_vectors, dim, nlist, m, k, cl["layout_id"], pq_iters, residual=residual, **pq_kw), mmap=mmap)
    if pq is None:
        return None
    return dict(centroids=cl["centroids"], offsets=cl["offsets"], reordered_ids=cl["reordered_ids"], codes=pq["codes"],
                codebook=pq["codebook"], vectors=vectors, nlist=nlist)


def save_index(root, dataset, index, build_recipe, pq_iters, residual=False, **pq_kw):
    """The other way round: a session's view arrays as a cluster asset and a PQ asset the reference's tools load."""
    cen = np.asarray(index["centroids"])
    n = np.asarray(index["codes"]).shape[0]
    cb = np.asarray(index["codebook"])
    entry, layout = save_cluster(root, dataset, cen, index["reordered_ids"], index["offsets"], build_recipe)
    req = pq_request(dataset, n, cen.shape[1], cen.shape[0], cb.shape[0], cb.shape[1], layout, pq_iters, residual=residual, **pq_kw)
    return entry, save_pq(root, req, cb, index["codes"])


# ---------------------------------------------------------------------------------------------- OPQ rotation file
OPQ_MAGIC, OPQ_VERSION = 0x3151504F, 1   # "OPQ1"


def opq_cache_key(dataset, n, dim, train_n, pq_m, pq_k, opq_iters, pq_iters, seed) -> str:
    """The file stem of a rotation (make_opq_cache_key, src/transform/opq_cache.cu:50-66)."""
    return "%s__n%d__train%d__d%d__M%d__K%d__opq%d__pq%d__seed%d" % (dataset, n, train_n, dim, pq_m, pq_k, opq_iters, pq_iters, seed)


def _opq_path(cache_dir, key):
    safe = "".join(c if (c.isascii() and (c.isalnum() or c in "_-.")) else "_" for c in key)
    return os.path.join(cache_dir, safe + ".opq")


def save_opq_rotation(cache_dir, key, rotation, train_n, pq_m, pq_k, opq_iters, pq_iters, seed) -> str:
    """36-byte header (magic, version, training rows, dim, M, K, OPQ iterations, PQ iterations, seed) + [dim][dim] f32, row-major
    [out][in] (src/transform/opq_cache.cu:11-24,98-124): the matrix psb_options.opq_matrix takes."""
    rot = np.ascontiguousarray(rotation, np.float32)
    if rot.ndim != 2 or rot.shape[0] != rot.shape[1]:
        raise ValueError("the rotation must be [dim][dim]")
    os.makedirs(cache_dir, exist_ok=True)
    path = _opq_path(cache_dir, key)
    with open(path, "wb") as f:
        f.write(struct.pack("<IIiiiiiiI", OPQ_MAGIC, OPQ_VERSION, train_n, rot.shape[0], pq_m, pq_k, opq_iters, pq_iters, seed))
        rot.tofile(f)
    return path


def load_opq_rotation(cache_dir, key, dim):
    """The rotation [dim][dim], or None (no file, another format or dimension, short file)."""
    path = _opq_path(cache_dir, key)
    if not os.path.exists(path):
        return None
    with open(path, "rb") as f:
        head = f.read(36)
        if len(head) != 36:
            return None
        magic, version, _, d = struct.unpack("<IIii", head[:16])
        if magic != OPQ_MAGIC or version != OPQ_VERSION or d != dim:
            return None
        rot = np.fromfile(f, np.float32, dim * dim)
    return rot.reshape(dim, dim) if rot.size == dim * dim else None
