// Host-side dataset index builders (plain C ABI, loaded with ctypes).
//
// Counterpart of Megatron's pybind `helpers.cpp` (`build_sample_idx`, `build_blending_indices`) that
// the reference compiles at start-up through `_compile_dependencies` (linear_moe/initialize.py:14,82).
#include <cstdint>
#include <cstddef>
#include <cstring>
#include <algorithm>
#include <atomic>
#include <thread>
#include <vector>

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
// ds_index is one byte per sample, so at most 256 datasets; returns 1 beyond that (nothing is written).
int lmoe_build_blending_indices(uint8_t* ds_index, int64_t* ds_sample, const double* weights,
                                int32_t num_datasets, int64_t size) {
    if (num_datasets < 1 || num_datasets > 256) return 1;
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
    return 0;
}

}  // extern "C"

namespace {

// Token width of the `.bin` file by the index header's dtype code (integer token types only).
inline int token_bytes(int32_t code) {
    switch (code) {
        case 1: case 2: return 1;      // uint8, int8
        case 3: case 8: return 2;      // int16, uint16
        case 4: return 4;              // int32
        case 5: return 8;              // int64
        default: return 0;
    }
}

// Widen `n` tokens starting at byte `src` to int64 (memcpy per token: the mapping is not assumed aligned).
inline void widen(const uint8_t* src, int32_t code, int64_t n, int64_t* out) {
    switch (code) {
        case 1: for (int64_t i = 0; i < n; ++i) out[i] = src[i]; break;
        case 2: for (int64_t i = 0; i < n; ++i) out[i] = (int8_t)src[i]; break;
        case 3: for (int64_t i = 0; i < n; ++i) { int16_t t; std::memcpy(&t, src + 2 * i, 2); out[i] = t; } break;
        case 8: for (int64_t i = 0; i < n; ++i) { uint16_t t; std::memcpy(&t, src + 2 * i, 2); out[i] = t; } break;
        case 4: for (int64_t i = 0; i < n; ++i) { int32_t t; std::memcpy(&t, src + 4 * i, 4); out[i] = t; } break;
        case 5: std::memcpy(out, src, (size_t)n * 8); break;
        default: break;
    }
}

struct GatherJob {
    const uint8_t* data; int64_t data_bytes; int32_t code;
    const int32_t* sizes; const int64_t* pointers; int64_t n_seq;
    const int64_t* doc_idx; int64_t n_doc_idx;
    const int64_t* sample_idx; int64_t n_samples;
    const int64_t* indices; int64_t seq_length; int64_t* out;
};

// One sample: tokens [o0 of document d0 .. o1 of document d1] inclusive, seq_length + 1 of them.
int gather_one(const GatherJob& j, int64_t row) {
    const int64_t s = j.indices[row];
    if (s < 0 || s >= j.n_samples) return 2;
    const int64_t d0 = j.sample_idx[2 * s], o0 = j.sample_idx[2 * s + 1];
    const int64_t d1 = j.sample_idx[2 * s + 2], o1 = j.sample_idx[2 * s + 3];
    if (d0 < 0 || d1 < d0 || d1 >= j.n_doc_idx || o0 < 0 || o1 < 0) return 2;
    const int eb = token_bytes(j.code);
    const int64_t want = j.seq_length + 1;
    int64_t* dst = j.out + row * want;
    int64_t got = 0;
    for (int64_t d = d0; d <= d1; ++d) {
        const int64_t doc = j.doc_idx[d];
        if (doc < 0 || doc >= j.n_seq) return 2;
        const int64_t len = j.sizes[doc];
        const int64_t begin = d == d0 ? o0 : 0;
        const int64_t end = d == d1 ? o1 + 1 : len;           // exclusive
        if (begin > end || end > len) return 4;
        const int64_t n = end - begin;
        if (got + n > want) return 4;
        const int64_t byte0 = j.pointers[doc] + begin * eb;
        if (byte0 < 0 || byte0 + n * eb > j.data_bytes) return 3;
        widen(j.data + byte0, j.code, n, dst + got);
        got += n;
    }
    return got == want ? 0 : 4;
}

}  // namespace

extern "C" {

// Assemble `n` fixed-length training samples (seq_length + 1 tokens each, widened to int64) from a memory-mapped
// Megatron `.bin` file: the batched form of the per-sample Python walk over document boundaries, spread over
// `nthreads` host threads.  Every index is checked against the tables it indexes.
// Returns 0, or the first error met: 2 = an index outside its table, 3 = a token range outside the file,
// 4 = a sample that does not hold seq_length + 1 tokens, 5 = a token type that is not an integer type.
int lmoe_gather_gpt_samples(const uint8_t* data, int64_t data_bytes, int32_t dtype_code,
                            const int32_t* sizes, const int64_t* pointers, int64_t n_seq,
                            const int64_t* doc_idx, int64_t n_doc_idx,
                            const int64_t* sample_idx, int64_t n_samples,
                            const int64_t* indices, int64_t n, int64_t seq_length, int64_t* out, int32_t nthreads) {
    if (token_bytes(dtype_code) == 0) return 5;
    if (n <= 0) return 0;
    const GatherJob job{data, data_bytes, dtype_code, sizes, pointers, n_seq, doc_idx, n_doc_idx,
                        sample_idx, n_samples, indices, seq_length, out};
    const int64_t workers = std::max<int64_t>(1, std::min<int64_t>(nthreads, n));
    std::atomic<int> err{0};
    auto run = [&](int64_t lo, int64_t hi) {
        for (int64_t r = lo; r < hi && err.load(std::memory_order_relaxed) == 0; ++r) {
            const int rc = gather_one(job, r);
            if (rc != 0) { int zero = 0; err.compare_exchange_strong(zero, rc); }
        }
    };
    if (workers == 1) {
        run(0, n);
    } else {
        std::vector<std::thread> pool;
        const int64_t per = (n + workers - 1) / workers;
        for (int64_t w = 0; w < workers; ++w) {
            const int64_t lo = w * per, hi = std::min(n, lo + per);
            if (lo < hi) pool.emplace_back(run, lo, hi);
        }
        for (auto& t : pool) t.join();
    }
    return err.load();
}

}  // extern "C"
