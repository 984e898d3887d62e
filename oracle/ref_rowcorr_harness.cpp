// TEST INFRASTRUCTURE: C entry points around the reference's own row-correction code, compiled in place from the
// reference checkout (index/row_correction/row_correction.cpp, quantization/row_correction/{u16,pq}.h,
// common/row_correction.h).  Nothing of the product links this.
#include <cstdint>
#include <cstring>
#include <exception>
#include <fstream>
#include <string>

#include "dataset/cache/cache_manifest.h"
#include "index/row_correction/row_correction.h"
#include "quantization/row_correction/pq.h"
#include "quantization/row_correction/u16.h"

namespace rc = paraselect::row_correction;

extern "C" {

// Runs the reference's builder into entry_dir (which must exist); the payload lands in entry_dir/row_correction.u16a and
// the fp32 audit copy in entry_dir/row_correction.f32.  Returns 0, or 1 after an exception.
int ref_rc_build_pq(const char* entry_dir, int64_t rows, int dim, int nlist, int m, int k, const float* centroids,
                    const int64_t* offsets, const uint8_t* codes, const float* codebook) {
    try {
        using Json = paraselect::dataset::cache_manifest::Json;
        Json parent = paraselect::dataset::cache_manifest::identity("residual_pq", "synthetic");
        parent.update({{"n_vectors", (uint64_t)rows}, {"dim", dim}, {"nlist", nlist}, {"m", m}, {"k", k}, {"dsub", dim / m},
                       {"cluster_layout_id", "layout0"}, {"codes_layout", "row_major"}});
        rc::Manifest mf;
        mf.dataset_name = "synthetic"; mf.parent_manifest_json = parent.dump(); mf.cluster_layout_id = "layout0";
        mf.codec = "residual_pq"; mf.row_layout = "row_major"; mf.rows = (uint64_t)rows; mf.dim = dim; mf.nlist = nlist;
        mf.code_width = m; mf.codebook_size = k; mf.subvector_dim = dim / m;
        rc::PQBuildInput in;
        in.centroids = centroids; in.cluster_offsets = offsets; in.codes = codes; in.codebook = codebook;
        rc::build_pq(entry_dir, mf, in);
        // the parent manifest beside it, so Asset::open accepts the directory
        std::ofstream(std::string(entry_dir) + "/manifest.json") << parent.dump(2) << std::endl;
        rc::Asset asset = rc::Asset::open(entry_dir, mf);
        return asset.view().count == rows ? 0 : 2;
    } catch (const std::exception&) { return 1; }
}

float ref_rc_value(const float* centroid, const float* reconstruction, int dim) { return rc::value(centroid, reconstruction, dim); }
float ref_rc_pq_value(const float* centroid, const float* codebook, const uint8_t* code, int m, int k, int dsub) {
    return rc::pq_value(centroid, codebook, code, m, k, dsub);
}
// The fixed-model quantiser: range from the model alone.  Returns 0, or 1 after an exception.
int ref_rc_for_pq(const float* centers, int nlist, const float* codebook, int m, int k, int dsub, float* scale, float* offset) {
    try { const auto q = rc::U16Quantizer::for_pq(centers, nlist, codebook, m, k, dsub); *scale = q.scale; *offset = q.offset; return 0; }
    catch (const std::exception&) { return 1; }
}
int ref_rc_encode(float scale, float offset, float v, uint16_t* out) {
    try { rc::U16Quantizer q; q.scale = scale; q.offset = offset; *out = q.encode(v); return 0; } catch (const std::exception&) { return 1; }
}
float ref_rc_decode(float scale, float offset, uint16_t code) { rc::U16Quantizer q; q.scale = scale; q.offset = offset; return q.decode(code); }

}  // extern "C"
