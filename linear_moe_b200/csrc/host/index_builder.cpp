// Host-side dataset index builders (plain C ABI, loaded with ctypes).
//
// Counterpart of Megatron's pybind `helpers.cpp` (`build_sample_idx`, `build_blending_indices`) that
// the reference compiles at start-up through `_compile_dependencies` (linear_moe/initialize.py:14,82).
#include <cstdint>
#include <cstddef>

extern "C" {

// sample_idx: [(num_samples + 1) * 2] int64, filled with (index into doc_idx, token offset) pairs.
// Samples hold seq_length + 1 tokens and overlap by one token.
// Returns 0 on success, 1 if the documents run out before num_samples samples are formed.
int lmoe_build_sample_idx(const int32_t* sizes, const int64_t* doc_idx, int64_t num_docs_in_idx,
                          int64_t seq_length, int64_t num_samples, int64_t* sample_idx) {
    int64_t di = 0, off = 0;
    sample_idx[0] = 0;
    sample_idx[1] = 0;
    for (int64_t s = 1; s <= num_samples; ++s) {
        int64_t remaining = seq_length + 1;
        while (remaining != 0) {
            if (di >= num_docs_in_idx) return 1;
            int64_t dlen = (int64_t)sizes[doc_idx[di]] - off;
            remaining -= dlen;
            if (remaining <= 0) {
                off += remaining + dlen - 1;
                remaining = 0;
            } else {
                ++di;
                off = 0;
            }
        }
        sample_idx[2 * s] = di;
        sample_idx[2 * s + 1] = off;
    }
    return 0;
}

// Greedy blending: sample i goes to the dataset whose running count lags its weight the most.
void lmoe_build_blending_indices(uint8_t* ds_index, int64_t* ds_sample, const double* weights,
                                 int32_t num_datasets, int64_t size) {
    int64_t counts[256] = {0};
    for (int64_t i = 0; i < size; ++i) {
        double denom = i > 0 ? (double)i : 1.0;
        int best = 0;
        double best_err = weights[0] * denom - (double)counts[0];
        for (int d = 1; d < num_datasets; ++d) {
            double err = weights[d] * denom - (double)counts[d];
            if (err > best_err) { best_err = err; best = d; }
        }
        ds_index[i] = (uint8_t)best;
        ds_sample[i] = counts[best];
        counts[best] += 1;
    }
}

}  // extern "C"
