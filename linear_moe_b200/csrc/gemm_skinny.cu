// y[M, N] = x[M, K] W[N, K]^T for M <= 16: the linears of one-token decode steps.
//
// With a handful of rows the product is bound by reading W once (2 N K bytes); a 256 x 256 tensor-core tile would spend
// its time on rows that do not exist.  Here a CTA owns 16 rows of W and its eight warps split K.  Every lane streams
// 16-byte pieces of two W rows and of one x row straight from global memory into mma.sync.m16n8k16 fragments: the sum
// over k does not care about the order of k, so the eight consecutive elements a lane loads are used as the k slots
// that lane owns in two MMA steps (the same assignment for the W and the x fragment), and no shared-memory staging or
// transposition is needed.  The eight partial tiles are added through shared memory.  No atomics: results are
// deterministic.  The kernel is launched with programmatic stream serialization: its first eight steps of W are in
// flight before it waits for the kernel that produces x, so consecutive linears of a decode step keep HBM busy across
// the kernel boundaries (the small kernels in between call griddepcontrol.launch_dependents at their start).
#include <cstdlib>

#include "common.cuh"
#include "mma_utils.cuh"

namespace lmoe {
namespace sk {

__device__ __forceinline__ uint4 ld_stream(const bf16* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ uint32_t sk_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void sk_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// store a float into the shared memory of CTA `rank` of the cluster, at the address `p` has in this CTA
__device__ __forceinline__ void st_cluster_f32(float* p, uint32_t rank, float v) {
    uint32_t local = (uint32_t)__cvta_generic_to_shared(p), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" :: "r"(remote), "f"(v) : "memory");
}

// NTILES 1: M <= 8, 2: M <= 16.  KS: CTAs of a cluster that split K between them (for matrices with few rows, so that
// every SM streams a piece of W); their partial tiles meet in the shared memory of the cluster's first CTA.
template <int NTILES, int KS>
__global__ void __launch_bounds__(256) gemm_skinny_kernel(const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ W,
                                                          long long ldw, bf16* __restrict__ y, long long ldy, int M, int N, int K) {
    __shared__ float red[8][NTILES][32][4];
    __shared__ float cred[KS][NTILES][32][4];
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const int g = l >> 2, q = l & 3;
    const uint32_t crank = KS > 1 ? sk_cluster_rank() : 0;
    const int row_lo = (blockIdx.x / KS) * 16 + g, row_hi = row_lo + 8;
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
    const int kslice = K / KS;                                           // a multiple of 32 (checked by the launcher)
    const int k_beg = (int)crank * kslice + w * 32, k_end = (int)(crank + 1) * kslice;
    // The weights do not depend on the kernel before this one: the first PF steps of W are requested before waiting for
    // it (programmatic dependent launch), so the weight stream of one linear overlaps the tail of whatever produced x.
    constexpr int PF = 8;
    uint4 pa_lo[PF], pa_hi[PF];
#pragma unroll
    for (int i = 0; i < PF; ++i) {
        const int k0 = k_beg + i * 256;
        pa_lo[i] = (lo_ok && k0 < k_end) ? ld_stream(w_lo + k0) : zero;
        pa_hi[i] = (hi_ok && k0 < k_end) ? ld_stream(w_hi + k0) : zero;
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");     // the next kernel may start its own prefetch
    asm volatile("griddepcontrol.wait;" ::: "memory");                  // x is complete and visible from here on
#pragma unroll
    for (int i = 0; i < PF; ++i) {
        const int k0 = k_beg + i * 256;
        if (k0 < k_end) {
            const uint32_t f1[4] = {pa_lo[i].x, pa_hi[i].x, pa_lo[i].y, pa_hi[i].y};
            const uint32_t f2[4] = {pa_lo[i].z, pa_hi[i].z, pa_lo[i].w, pa_hi[i].w};
#pragma unroll
            for (int t = 0; t < NTILES; ++t) {
                const uint4 b = x_ok[t] ? *reinterpret_cast<const uint4*>(xr[t] + k0) : zero;
                mma16816(acc[t], f1, b.x, b.y);
                mma16816(acc[t], f2, b.z, b.w);
            }
        }
    }
#pragma unroll 4
    for (int k0 = k_beg + PF * 256; k0 < k_end; k0 += 256) {
        const uint4 a_lo = lo_ok ? ld_stream(w_lo + k0) : zero;
        const uint4 a_hi = hi_ok ? ld_stream(w_hi + k0) : zero;
        const uint32_t f1[4] = {a_lo.x, a_hi.x, a_lo.y, a_hi.y};
        const uint32_t f2[4] = {a_lo.z, a_hi.z, a_lo.w, a_hi.w};
#pragma unroll
        for (int t = 0; t < NTILES; ++t) {
            const uint4 b = x_ok[t] ? *reinterpret_cast<const uint4*>(xr[t] + k0) : zero;
            mma16816(acc[t], f1, b.x, b.y);
            mma16816(acc[t], f2, b.z, b.w);
        }
    }
#pragma unroll
    for (int t = 0; t < NTILES; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) red[w][t][l][e] = acc[t][e];
    __syncthreads();
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    if (w < NTILES) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[e] += red[i][w][l][e];
    }
    if (KS > 1) {
        // the CTA's partial tile goes to slot `crank` of the first CTA; it adds the slots in rank order (deterministic)
        if (w < NTILES) {
#pragma unroll
            for (int e = 0; e < 4; ++e) st_cluster_f32(&cred[crank][w][l][e], 0, s[e]);
        }
        sk_cluster_sync();
        if (crank != 0) return;
        if (w < NTILES) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[e] = 0.f;
#pragma unroll
                for (int i = 0; i < KS; ++i) s[e] += cred[i][w][l][e];
            }
        }
    }
    if (w < NTILES) {
        const int n0 = 8 * w + 2 * q;                                   // batch rows n0, n0 + 1
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

template <int NTILES, int KS>
static int launch_skinny(const bf16* x, long long ldx, const bf16* W, long long ldw, bf16* y, long long ldy, int M, int N, int K,
                         cudaStream_t st) {
    const int blocks = ((N + 15) / 16) * KS;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    int na = 0;
    // the kernel may start while its predecessor in the stream is still running; it waits (griddepcontrol.wait) before it
    // reads x
    static const bool pdl = [] { const char* e = getenv("LMOE_SKINNY_PDL"); return e == nullptr || e[0] != '0'; }();
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (KS > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = KS;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return (int)cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<NTILES, KS>, x, ldx, W, ldw, y, ldy, M, N, K);
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
    const bf16 *xb = (const bf16*)x, *Wb = (const bf16*)W;
    bf16* yb = (bf16*)y;
    // few row blocks: four CTAs of a cluster split K so that the whole GPU streams W
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms = 148;
    }
    const bool split = (N + 15) / 16 < 2 * sms && K % 128 == 0;
    if (M <= 8) return split ? sk::launch_skinny<1, 4>(xb, ldx, Wb, ldw, yb, ldy, M, N, K, st)
                             : sk::launch_skinny<1, 1>(xb, ldx, Wb, ldw, yb, ldy, M, N, K, st);
    return split ? sk::launch_skinny<2, 4>(xb, ldx, Wb, ldw, yb, ldy, M, N, K, st)
                 : sk::launch_skinny<2, 1>(xb, ldx, Wb, ldw, yb, ldy, M, N, K, st);
}
