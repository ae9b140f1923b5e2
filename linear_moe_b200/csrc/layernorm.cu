// LayerNorm forward / backward with an optional fused residual add, for the backbones whose launcher selects
// --normalization LayerNorm (Mixtral) and for the per-head GroupNorm of the linear-attention output
// (--la-output-norm groupnorm = LayerNorm over the head dimension with rows = tokens x heads).
//
//   r = x (+ res);   y = (r - mean(r)) * rsqrt(var(r) + eps) * w + b
//
// Same structure as the RMSNorm kernels of elementwise.cu: 16-byte vectors, the row stays in registers between the
// statistics and the write, fp32 arithmetic; the backward walks rows blockIdx.x, +gridDim.x, ... and keeps its dw / db
// partial sums in registers, written once per block to [P, 2N] (dw partials, then db partials) and summed by a second
// small kernel.  Replaces the reference's Triton LayerNorm (common_modules/layernorm.py:55-131,300-420).
#include "common.cuh"

namespace lmoe {

template <typename T, int MAXV>
__global__ void layer_norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ w,
                                      const T* __restrict__ b, T* __restrict__ y, T* __restrict__ res_out,
                                      float* __restrict__ mean_out, float* __restrict__ rstd_out, int N, float eps) {
    __shared__ float red[32];
    constexpr int VN = Vec<T>::N;
    const int64_t row = blockIdx.x;
    const int nvec = N / VN;
    pdl_trigger();
    Vec<T> v[MAXV];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nvec) {
            v[j].load(x + row * N + i * VN);
            if (res != nullptr) {
                Vec<T> r;
                r.load(res + row * N + i * VN);
#pragma unroll
                for (int e = 0; e < VN; ++e) v[j].set(e, v[j].get(e) + r.get(e));
            }
            if (res_out != nullptr) v[j].store(res_out + row * N + i * VN);
#pragma unroll
            for (int e = 0; e < VN; ++e) s += v[j].get(e);
        }
    }
    const float mean = block_sum(s, red) / (float)N;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nvec) {
#pragma unroll
            for (int e = 0; e < VN; ++e) { const float d = v[j].get(e) - mean; ss += d * d; }
        }
    }
    const float rstd = rsqrtf(block_sum(ss, red) / (float)N + eps);
    if (threadIdx.x == 0) { mean_out[row] = mean; rstd_out[row] = rstd; }
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nvec) {
            Vec<T> o, wv, bv;
            if (w != nullptr) wv.load(w + i * VN);
            if (b != nullptr) bv.load(b + i * VN);
#pragma unroll
            for (int e = 0; e < VN; ++e) {
                float t = (v[j].get(e) - mean) * rstd;
                if (w != nullptr) t *= wv.get(e);
                if (b != nullptr) t += bv.get(e);
                o.set(e, t);
            }
            o.store(y + row * N + i * VN);
        }
    }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)) (+ dres) with g = dy * w
template <typename T, int MAXV>
__global__ void layer_norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ xin, const T* __restrict__ w,
                                      const float* __restrict__ mean, const float* __restrict__ rstd,
                                      const T* __restrict__ dres, T* __restrict__ dx, float* __restrict__ partial,
                                      int rows, int N) {
    __shared__ float red[32];
    constexpr int VN = Vec<T>::N;
    const int nvec = N / VN;
    float dwacc[MAXV][VN], dbacc[MAXV][VN];
#pragma unroll
    for (int j = 0; j < MAXV; ++j)
#pragma unroll
        for (int e = 0; e < VN; ++e) dwacc[j][e] = dbacc[j][e] = 0.f;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float mu = mean[row], rs = rstd[row];
        Vec<T> g[MAXV], xv[MAXV];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < nvec) {
                g[j].load(dy + row * N + i * VN);
                xv[j].load(xin + row * N + i * VN);
                Vec<T> wv;
                if (w != nullptr) wv.load(w + i * VN);
#pragma unroll
                for (int e = 0; e < VN; ++e) {
                    const float xh = (xv[j].get(e) - mu) * rs;
                    const float gy = g[j].get(e);
                    dwacc[j][e] += gy * xh;
                    dbacc[j][e] += gy;
                    const float gw = w != nullptr ? gy * wv.get(e) : gy;
                    s1 += gw;
                    s2 += gw * xh;
                }
            }
        }
        s1 = block_sum(s1, red) / (float)N;
        s2 = block_sum(s2, red) / (float)N;
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < nvec) {
                Vec<T> wv, o, dr;
                if (w != nullptr) wv.load(w + i * VN);
                if (dres != nullptr) dr.load(dres + row * N + i * VN);
#pragma unroll
                for (int e = 0; e < VN; ++e) {
                    const float xh = (xv[j].get(e) - mu) * rs;
                    const float gw = w != nullptr ? g[j].get(e) * wv.get(e) : g[j].get(e);
                    float d = rs * (gw - s1 - xh * s2);
                    if (dres != nullptr) d += dr.get(e);
                    o.set(e, d);
                }
                o.store(dx + row * N + i * VN);
            }
        }
    }
    if (partial != nullptr) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            if (i < nvec) {
#pragma unroll
                for (int e = 0; e < VN; ++e) {
                    partial[(int64_t)blockIdx.x * 2 * N + i * VN + e] = dwacc[j][e];
                    partial[(int64_t)blockIdx.x * 2 * N + N + i * VN + e] = dbacc[j][e];
                }
            }
        }
    }
}

// out[c] = sum_p partial[p, c] over a [P, C] fp32 matrix (C = 2N: dw then db), fp32 result
__global__ void ln_reduce_partials_kernel(const float* __restrict__ partial, float* __restrict__ out, int P, int C) {
    __shared__ float sm[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + tx;
    float s = 0.f;
    if (c < C)
        for (int p = ty; p < P; p += 8) s += partial[(int64_t)p * C + c];
    sm[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && c < C) {
        float t = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) t += sm[j][tx];
        out[c] = t;
    }
}

static inline int ln_threads(int nvec) {
    int t = 32;
    while (t < nvec && t < 256) t <<= 1;
    return t;
}

}  // namespace lmoe

using namespace lmoe;

#define LN_DISPATCH_T(dtype, ...)                     \
    if ((dtype) == 1) { typedef bf16 T; __VA_ARGS__ } \
    else { typedef float T; __VA_ARGS__ }

#define LN_DISPATCH_V(KERNEL, GRID, ...)                                                           \
    if (nvec <= threads * 1) KERNEL<T, 1><<<GRID, threads, 0, st>>>(__VA_ARGS__);                  \
    else if (nvec <= threads * 2) KERNEL<T, 2><<<GRID, threads, 0, st>>>(__VA_ARGS__);             \
    else if (nvec <= threads * 4) KERNEL<T, 4><<<GRID, threads, 0, st>>>(__VA_ARGS__);             \
    else KERNEL<T, 8><<<GRID, threads, 0, st>>>(__VA_ARGS__);

// x, res (nullable), y, res_out (nullable): [rows, N]; w, b (nullable): [N]; mean, rstd: [rows] fp32.
LMOE_API int lmoe_layer_norm_fwd(const void* x, const void* res, const void* w, const void* b, void* y, void* res_out,
                                 float* mean, float* rstd, int64_t rows, int N, float eps, int dtype, cudaStream_t st) {
    if (rows <= 0) return 0;
    LN_DISPATCH_T(dtype, {
        constexpr int VN = Vec<T>::N;
        if (N % VN != 0) return -1;
        const int nvec = N / VN;
        const int threads = ln_threads(nvec);
        if (nvec > threads * 8) return -2;
        LN_DISPATCH_V(layer_norm_fwd_kernel, (unsigned)rows, (const T*)x, (const T*)res, (const T*)w, (const T*)b, (T*)y,
                      (T*)res_out, mean, rstd, N, eps)
    })
    return (int)cudaGetLastError();
}

// partial: [P, 2N] fp32 scratch (nullable when neither dw nor db is wanted); dwdb: [2N] fp32 = dw then db.
LMOE_API int lmoe_layer_norm_bwd(const void* dy, const void* xin, const void* w, const float* mean, const float* rstd,
                                 const void* dres, void* dx, float* partial, float* dwdb, int64_t rows, int N, int P,
                                 int dtype, cudaStream_t st) {
    if (rows <= 0) return 0;
    if (rows > 2147483647LL) return -3;
    LN_DISPATCH_T(dtype, {
        constexpr int VN = Vec<T>::N;
        if (N % VN != 0) return -1;
        const int nvec = N / VN;
        const int threads = ln_threads(nvec);
        if (nvec > threads * 8) return -2;
        const int blocks = (int)(rows < P ? rows : P);
        LN_DISPATCH_V(layer_norm_bwd_kernel, blocks, (const T*)dy, (const T*)xin, (const T*)w, mean, rstd, (const T*)dres,
                      (T*)dx, partial, (int)rows, N)
        if (dwdb != nullptr && partial != nullptr)
            ln_reduce_partials_kernel<<<(2 * N + 31) / 32, 256, 0, st>>>(partial, dwdb, blocks, 2 * N);
    })
    return (int)cudaGetLastError();
}
