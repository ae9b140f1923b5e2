// One decoding step of decayed linear attention, scalar decay per head (lightning / retention / basic / simple GLA /
// per-token decay) or one decay per key channel (GLA, HGRN2):
//   S' = e^{g} diag(e^{gk}) S + k^T v,   o = scale * q S'
// for one new token per sequence.  The chunked training kernels pad a single token to a whole chunk and run three
// launches; here the step is what it is at decode time: one read and one write of the [D x D] fp32 state per head.
// One CTA per (batch, head); thread (r, j) owns column j of the value dimension and every fourth key row, so state
// accesses are coalesced over j; the four partial outputs of a column meet in shared memory.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace lmoe {
namespace {

template <int D>
__global__ void __launch_bounds__(4 * D)
lsm_scalar_step_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                       const __nv_bfloat16* __restrict__ v, long long qs_b, long long qs_h, long long ks_b, long long ks_h,
                       long long vs_b, long long vs_h, const float* __restrict__ g, const float* __restrict__ gk,
                       const float* __restrict__ s_in, float* __restrict__ s_out, __nv_bfloat16* __restrict__ o, int H,
                       float scale) {
    __shared__ float qs[D], ks[D], dec[D], part[4][D];
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int j = threadIdx.x % D, r = threadIdx.x / D;
    if (threadIdx.x < D) {
        qs[threadIdx.x] = __bfloat162float(q[b * qs_b + h * qs_h + threadIdx.x]) * scale;
        ks[threadIdx.x] = __bfloat162float(k[b * ks_b + h * ks_h + threadIdx.x]);
        dec[threadIdx.x] = (g == nullptr ? 1.f : __expf(g[bh])) * (gk == nullptr ? 1.f : __expf(gk[(long long)bh * D + threadIdx.x]));
    }
    const float vj = __bfloat162float(v[b * vs_b + h * vs_h + j]);
    __syncthreads();
    const float* si = s_in == nullptr ? nullptr : s_in + (long long)bh * D * D;
    float* so = s_out + (long long)bh * D * D;
    float acc = 0.f;
    // all D/4 loads of a thread are issued before the first use: the step is one pass over the state, and with a few
    // loads in flight per thread it is bound by memory latency instead of bandwidth
    float st[D / 4];
#pragma unroll
    for (int t = 0; t < D / 4; ++t) st[t] = si == nullptr ? 0.f : __ldcs(si + (r + 4 * t) * D + j);
#pragma unroll
    for (int t = 0; t < D / 4; ++t) {
        const int i = r + 4 * t;
        const float s = st[t] * dec[i] + ks[i] * vj;
        so[i * D + j] = s;
        acc = fmaf(qs[i], s, acc);
    }
    part[r][j] = acc;
    __syncthreads();
    if (r == 0) o[(long long)bh * D + j] = __float2bfloat16(part[0][j] + part[1][j] + part[2][j] + part[3][j]);
}

// (Gated) delta rule: S <- e^{g} S;  u = beta (v - k S);  S' = S + k^T u;  o = scale q S'.  Same thread layout; the
// D/4 state entries of a thread stay in registers between the k S reduction and the update, so the state is still read
// and written once.
template <int D>
__global__ void __launch_bounds__(4 * D)
lsm_delta_step_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                      const __nv_bfloat16* __restrict__ v, long long qs_b, long long qs_h, long long ks_b, long long ks_h,
                      long long vs_b, long long vs_h, const float* __restrict__ g, const float* __restrict__ beta,
                      const float* __restrict__ s_in, float* __restrict__ s_out, __nv_bfloat16* __restrict__ o, int H,
                      float scale) {
    __shared__ float qs[D], ks[D], part[4][D];
    const int bh = blockIdx.x, b = bh / H, h = bh % H;
    const int j = threadIdx.x % D, r = threadIdx.x / D;
    if (threadIdx.x < D) {
        qs[threadIdx.x] = __bfloat162float(q[b * qs_b + h * qs_h + threadIdx.x]) * scale;
        ks[threadIdx.x] = __bfloat162float(k[b * ks_b + h * ks_h + threadIdx.x]);
    }
    const float vj = __bfloat162float(v[b * vs_b + h * vs_h + j]);
    const float decay = g == nullptr ? 1.f : __expf(g[bh]);
    __syncthreads();
    const float* si = s_in == nullptr ? nullptr : s_in + (long long)bh * D * D;
    float* so = s_out + (long long)bh * D * D;
    float sreg[D / 4];
    float ks_dot = 0.f;
#pragma unroll
    for (int t = 0; t < D / 4; ++t) {
        const int i = r + 4 * t;
        sreg[t] = si == nullptr ? 0.f : si[i * D + j] * decay;
        ks_dot = fmaf(ks[i], sreg[t], ks_dot);
    }
    part[r][j] = ks_dot;
    __syncthreads();
    const float u = (vj - (part[0][j] + part[1][j] + part[2][j] + part[3][j])) * beta[bh];
    __syncthreads();
    float acc = 0.f;
#pragma unroll
    for (int t = 0; t < D / 4; ++t) {
        const int i = r + 4 * t;
        const float s = fmaf(ks[i], u, sreg[t]);
        so[i * D + j] = s;
        acc = fmaf(qs[i], s, acc);
    }
    part[r][j] = acc;
    __syncthreads();
    if (r == 0) o[(long long)bh * D + j] = __float2bfloat16(part[0][j] + part[1][j] + part[2][j] + part[3][j]);
}

}  // namespace
}  // namespace lmoe

// q, k, v: bf16, one token per (batch, head), element strides over batch and head, contiguous over D.  g: [B*H] log
// decay of this token or null; gk: [B*H, D] log decay per key channel or null.  s_in: [B*H, D, D] fp32 or null (zero
// state); s_out is a different buffer.  o: [B*H, D] bf16.
LMOE_API int lmoe_lsm_scalar_step(const void* q, const void* k, const void* v, long long qs_b, long long qs_h, long long ks_b,
                                  long long ks_h, long long vs_b, long long vs_h, const float* g, const float* gk,
                                  const float* s_in, float* s_out, void* o, int B, int H, int D, float scale,
                                  cudaStream_t st) {
    using namespace lmoe;
    const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)k, *vv = (const __nv_bfloat16*)v;
    if (D == 128)
        lsm_scalar_step_kernel<128><<<B * H, 512, 0, st>>>(qq, kk, vv, qs_b, qs_h, ks_b, ks_h, vs_b, vs_h, g, gk, s_in, s_out,
                                                          (__nv_bfloat16*)o, H, scale);
    else if (D == 64)
        lsm_scalar_step_kernel<64><<<B * H, 256, 0, st>>>(qq, kk, vv, qs_b, qs_h, ks_b, ks_h, vs_b, vs_h, g, gk, s_in, s_out,
                                                         (__nv_bfloat16*)o, H, scale);
    else
        return -1;
    return (int)cudaGetLastError();
}

// Delta-rule step; beta: [B*H]; g: [B*H] log decay or null (plain DeltaNet).  Other arguments as above.
LMOE_API int lmoe_lsm_delta_step(const void* q, const void* k, const void* v, long long qs_b, long long qs_h, long long ks_b,
                                 long long ks_h, long long vs_b, long long vs_h, const float* g, const float* beta,
                                 const float* s_in, float* s_out, void* o, int B, int H, int D, float scale,
                                 cudaStream_t st) {
    using namespace lmoe;
    const __nv_bfloat16 *qq = (const __nv_bfloat16*)q, *kk = (const __nv_bfloat16*)k, *vv = (const __nv_bfloat16*)v;
    if (D == 128)
        lsm_delta_step_kernel<128><<<B * H, 512, 0, st>>>(qq, kk, vv, qs_b, qs_h, ks_b, ks_h, vs_b, vs_h, g, beta, s_in, s_out,
                                                         (__nv_bfloat16*)o, H, scale);
    else if (D == 64)
        lsm_delta_step_kernel<64><<<B * H, 256, 0, st>>>(qq, kk, vv, qs_b, qs_h, ks_b, ks_h, vs_b, vs_h, g, beta, s_in, s_out,
                                                        (__nv_bfloat16*)o, H, scale);
    else
        return -1;
    return (int)cudaGetLastError();
}
