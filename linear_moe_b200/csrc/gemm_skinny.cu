// y[M, N] = x[M, K] W[N, K]^T for M <= 16: the linears of one-token decode steps.
//
// With a handful of rows the product is bound by reading W once (2 N K bytes); a 256 x 256 tensor-core tile would spend
// its time on rows that do not exist.  Here a CTA owns 16 rows of W and its eight warps split K.  Every lane streams
// 16-byte pieces of two W rows and of one x row straight from global memory into mma.sync.m16n8k16 fragments: the sum
// over k does not care about the order of k, so the eight consecutive elements a lane loads are used as the k slots
// that lane owns in two MMA steps (the same assignment for the W and the x fragment), and no shared-memory staging or
// transposition is needed.  The eight partial tiles are added through shared memory.  No atomics: results are
// deterministic.
#include "common.cuh"
#include "mma_utils.cuh"

namespace lmoe {
namespace sk {

__device__ __forceinline__ uint4 ld_stream(const bf16* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }

template <int NTILES>   // 1: M <= 8, 2: M <= 16
__global__ void __launch_bounds__(256) gemm_skinny_kernel(const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ W,
                                                          long long ldw, bf16* __restrict__ y, long long ldy, int M, int N, int K) {
    __shared__ float red[8][NTILES][32][4];
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const int g = l >> 2, q = l & 3;
    const int row_lo = blockIdx.x * 16 + g, row_hi = row_lo + 8;
    const bool lo_ok = row_lo < N, hi_ok = row_hi < N;
    const bf16* w_lo = W + (long long)(lo_ok ? row_lo : 0) * ldw + q * 8;
    const bf16* w_hi = W + (long long)(hi_ok ? row_hi : 0) * ldw + q * 8;
    const bf16* xr[NTILES];
    bool x_ok[NTILES];
#pragma unroll
    for (int t = 0; t < NTILES; ++t) {
        x_ok[t] = g + 8 * t < M;
        xr[t] = x + (long long)(x_ok[t] ? g + 8 * t : 0) * ldx + q * 8;
    }
    float acc[NTILES][4];
#pragma unroll
    for (int t = 0; t < NTILES; ++t) acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.f;
    const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll 4
    for (int k0 = w * 32; k0 < K; k0 += 256) {
        const uint4 a_lo = lo_ok ? ld_stream(w_lo + k0) : zero;
        const uint4 a_hi = hi_ok ? ld_stream(w_hi + k0) : zero;
        const uint32_t f1[4] = {a_lo.x, a_hi.x, a_lo.y, a_hi.y};
        const uint32_t f2[4] = {a_lo.z, a_hi.z, a_lo.w, a_hi.w};
#pragma unroll
        for (int t = 0; t < NTILES; ++t) {
            const uint4 b = x_ok[t] ? __ldg(reinterpret_cast<const uint4*>(xr[t] + k0)) : zero;
            mma16816(acc[t], f1, b.x, b.y);
            mma16816(acc[t], f2, b.z, b.w);
        }
    }
#pragma unroll
    for (int t = 0; t < NTILES; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[w][t][l][e] = acc[t][e];
    __syncthreads();
    if (w < NTILES) {
        const int t = w;
        float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[e] += red[i][t][l][e];
        const int n0 = 8 * t + 2 * q;                                   // batch rows n0, n0 + 1
        if (n0 < M) {
            if (lo_ok) y[(long long)n0 * ldy + row_lo] = __float2bfloat16(s[0]);
            if (hi_ok) y[(long long)n0 * ldy + row_hi] = __float2bfloat16(s[2]);
        }
        if (n0 + 1 < M) {
            if (lo_ok) y[(long long)(n0 + 1) * ldy + row_lo] = __float2bfloat16(s[1]);
            if (hi_ok) y[(long long)(n0 + 1) * ldy + row_hi] = __float2bfloat16(s[3]);
        }
    }
}

}  // namespace sk
}  // namespace lmoe

// x [M, K] (row pitch ldx), W [N, K] (row pitch ldw), y [M, N] (row pitch ldy), all bf16; M <= 16, K a multiple of 32,
// pitches multiples of 8 elements and bases 16-byte aligned.  Returns -1 for shapes it does not take.
LMOE_API int lmoe_gemm_skinny(const void* x, long long ldx, const void* W, long long ldw, void* y, long long ldy, int M, int N,
                              int K, cudaStream_t st) {
    using namespace lmoe;
    if (M <= 0 || M > 16 || N <= 0 || K <= 0 || K % 32 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return -1;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(W)) & 15) return -1;
    const int grid = (N + 15) / 16;
    if (M <= 8)
        sk::gemm_skinny_kernel<1><<<grid, 256, 0, st>>>((const bf16*)x, ldx, (const bf16*)W, ldw, (bf16*)y, ldy, M, N, K);
    else
        sk::gemm_skinny_kernel<2><<<grid, 256, 0, st>>>((const bf16*)x, ldx, (const bf16*)W, ldw, (bf16*)y, ldy, M, N, K);
    return (int)cudaGetLastError();
}
