// TEST INFRASTRUCTURE: C entry points around the host functions of the reference's 1-bit sign codec
// (quantization/turboquant/turboquant_1bit_format.h), compiled in place from the reference checkout.  Nothing of the
// product links this.
#include <cstdint>
#include <cstring>
#include <vector>

#include "quantization/turboquant/turboquant_1bit_format.h"

namespace tq = paraselect::search::turboquant;

extern "C" {

int ref_sign_words(int dim) { return (int)tq::packed_word_count((std::size_t)dim); }

void ref_sign_pack(const float* values, int dim, uint32_t* words) {
    const std::vector<std::uint32_t> w = tq::pack_signs(values, (std::size_t)dim);
    std::memcpy(words, w.data(), w.size() * sizeof(std::uint32_t));
}

int ref_sign_hamming(const uint32_t* a, const uint32_t* b, int dim) { return tq::hamming_distance(a, b, (std::size_t)dim); }

float ref_sign_scale_l2(const float* query, const uint32_t* code, int dim, float scale) {
    return tq::sign_scale_l2_distance(query, code, (std::size_t)dim, scale);
}

float ref_sign_binary_l2(const uint32_t* qcode, const uint32_t* code, int dim, float qn, float dn) {
    return tq::binary_l2_distance(qcode, code, (std::size_t)dim, qn, dn);
}

float ref_sign_mse(const float* query, const uint32_t* code, int dim, float centroid) {
    return tq::mse_distance(query, code, (std::size_t)dim, centroid);
}

}  // extern "C"
