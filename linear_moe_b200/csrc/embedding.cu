// Embedding backward: scatter-add of the output gradient rows into the table's gradient.
//
//   dW[ids[t], :] += dY[t, :]        for every token t with 0 <= ids[t] < vocab
//
// The usual framework path builds a dense [vocab, hidden] gradient (sort the ids, segment-reduce, write ~vocab x hidden
// elements) and then adds it to the fp32 accumulator in a second pass: for a 128k x 2048 table that is more than 1.5 GB
// of traffic for 16k tokens' worth of information.  Here each token row goes straight into the fp32 accumulator with
// red.global.add (atomics resolve repeated ids), 64 MB for 16k tokens.  Rows whose id falls outside [0, vocab) (other
// vocabulary shards under tensor parallelism, padding) are skipped.
// Reference counterpart: Megatron's VocabParallelEmbedding backward (index_add into main_grad).
#include "common.cuh"

namespace lmoe {

template <typename T>
__global__ void embedding_bwd_kernel(const T* __restrict__ dy, const int64_t* __restrict__ ids, float* __restrict__ dw,
                                     int64_t tokens, int hidden, int64_t vocab, int64_t id_offset) {
    constexpr int VN = Vec<T>::N;
    const int nvec = hidden / VN;
    for (int64_t t = blockIdx.x; t < tokens; t += gridDim.x) {
        const int64_t id = ids[t] - id_offset;
        if (id < 0 || id >= vocab) continue;
        float* row = dw + id * hidden;
        for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
            Vec<T> v;
            v.load(dy + t * hidden + i * VN);
#pragma unroll
            for (int e = 0; e < VN; ++e) atomicAdd(row + i * VN + e, v.get(e));
        }
    }
}

}  // namespace lmoe

using namespace lmoe;

// dy [tokens, hidden] (bf16: dtype 1, fp32: dtype 0), ids [tokens] int64, dw [vocab, hidden] fp32 (accumulated into).
LMOE_API int lmoe_embedding_bwd(const void* dy, const int64_t* ids, float* dw, int64_t tokens, int hidden, int64_t vocab,
                                int64_t id_offset, int dtype, cudaStream_t st) {
    if (tokens <= 0) return 0;
    const int vn = dtype == 1 ? 8 : 4;
    if (hidden % vn != 0) return -1;
    const int threads = hidden / vn >= 256 ? 256 : (hidden / vn >= 128 ? 128 : 64);
    const int blocks = (int)(tokens < 148 * 16 ? tokens : 148 * 16);
    if (dtype == 1) embedding_bwd_kernel<bf16><<<blocks, threads, 0, st>>>((const bf16*)dy, ids, dw, tokens, hidden, vocab, id_offset);
    else embedding_bwd_kernel<float><<<blocks, threads, 0, st>>>((const float*)dy, ids, dw, tokens, hidden, vocab, id_offset);
    return (int)cudaGetLastError();
}
