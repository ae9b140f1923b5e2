// out = a + s * sigmoid(g) with one gate logit per row: the shared expert of a Qwen2-MoE layer joining the routed
// experts' output (moe layer: shared_expert_gate).  As separate tensor operations this is a sigmoid, a broadcast
// multiply, an add and, backward, two more broadcast multiplies and a row reduction; here it is one pass forward and one
// pass backward (one warp per row: the row's gate gradient is the dot product it reduces anyway).
#include "common.cuh"

namespace lmoe {

template <typename T>
__global__ void gated_add_fwd_kernel(const T* __restrict__ a, const T* __restrict__ s, const T* __restrict__ g, T* __restrict__ out,
                                     int64_t rows, int N) {
    constexpr int V = Vec<T>::N;
    const int64_t nvec = rows * (N / V);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / (N / V);
        const float sig = sigmoid_f((float)g[r]);
        Vec<T> va, vs, vo;
        va.load(a + i * V);
        vs.load(s + i * V);
#pragma unroll
        for (int e = 0; e < V; ++e) vo.set(e, va.get(e) + vs.get(e) * sig);
        vo.store(out + i * V);
    }
}

// ds = d_out * sigmoid(g);  dg[row] = sigmoid'(g) * <d_out[row], s[row]>.  (The gradient of `a` is d_out itself.)
template <typename T>
__global__ void gated_add_bwd_kernel(const T* __restrict__ d_out, const T* __restrict__ s, const T* __restrict__ g,
                                     T* __restrict__ ds, T* __restrict__ dg, int64_t rows, int N) {
    constexpr int V = Vec<T>::N;
    const int wpb = blockDim.x >> 5, l = threadIdx.x & 31;
    for (int64_t r = (int64_t)blockIdx.x * wpb + (threadIdx.x >> 5); r < rows; r += (int64_t)gridDim.x * wpb) {
        const float sig = sigmoid_f((float)g[r]);
        float dot = 0.f;
        for (int c = l * V; c < N; c += 32 * V) {
            Vec<T> vd, vs, vo;
            vd.load(d_out + r * N + c);
            vs.load(s + r * N + c);
#pragma unroll
            for (int e = 0; e < V; ++e) {
                dot += vd.get(e) * vs.get(e);
                vo.set(e, vd.get(e) * sig);
            }
            vo.store(ds + r * N + c);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (l == 0) dg[r] = (T)(dot * sig * (1.f - sig));
    }
}

}  // namespace lmoe

using namespace lmoe;

#define DISPATCH_T(dtype, ...)                      \
    if ((dtype) == 1) { typedef bf16 T; __VA_ARGS__ } \
    else { typedef float T; __VA_ARGS__ }

static inline int grid_for(int64_t n, int threads, int cap = 148 * 16) {
    int64_t b = (n + threads - 1) / threads;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

// a, s, out: [rows, N]; g: [rows] gate logits.  dtype 0 = fp32, 1 = bf16; N a multiple of the 16-byte vector width.
LMOE_API int lmoe_gated_add_fwd(const void* a, const void* s, const void* g, void* out, int64_t rows, int N, int dtype,
                                cudaStream_t st) {
    if (rows <= 0) return 0;
    DISPATCH_T(dtype, {
        if (N % Vec<T>::N != 0) return -1;
        gated_add_fwd_kernel<T><<<grid_for(rows * (N / Vec<T>::N), 256), 256, 0, st>>>((const T*)a, (const T*)s, (const T*)g, (T*)out, rows, N);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_gated_add_bwd(const void* d_out, const void* s, const void* g, void* ds, void* dg, int64_t rows, int N, int dtype,
                                cudaStream_t st) {
    if (rows <= 0) return 0;
    DISPATCH_T(dtype, {
        if (N % Vec<T>::N != 0) return -1;
        const int64_t blocks = (rows + 7) / 8;
        gated_add_bwd_kernel<T><<<grid_for(blocks * 256, 256), 256, 0, st>>>((const T*)d_out, (const T*)s, (const T*)g, (T*)ds, (T*)dg, rows, N);
    })
    return (int)cudaGetLastError();
}
