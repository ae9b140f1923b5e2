// Chunked linear attention with a log decay per key channel (GLA, HGRN2), forward and backward, bf16 in / fp32 state.
//
//   S_t = diag(e^{g_t}) S_{t-1} + k_t^T v_t,   o_t = scale * q_t S_t,     g_t in R^{dk} (<= 0)
//
// Replaces fla's chunk_gla Triton kernels that the reference calls (gla/gla.py:94, hgrn2/hgrn2.py:76).  Same
// three-step structure as lsm_scalar.cu (group summaries -> combine -> sweep; no chunk state in HBM).
//
// Per chunk, with b_i the inclusive in-chunk cumulative log decay (a vector per token) and b_m its value at the
// middle token, the operands are rescaled around the middle so that neither factor can overflow:
//   q~_i = q_i e^{b_i - b_m},  k~_j = k_j e^{b_m - b_j}          (q~_i . k~_j = q_i . k_j e^{b_i - b_j} for j <= i)
//   O    = scale [ (q~ k~^T . mask) V + q~ (diag(e^{b_m}) S) ]
//   S   <- diag(e^{b_C - b_m}) [ diag(e^{b_m}) S + k~^T V ]
// The backward uses the same rescaled tiles:
//   dq = e^{b_i - b_m} . scale [ (dO V^T . mask) k~ + dO (diag(e^{b_m}) S)^T ]
//   dk = e^{b_m - b_j} . [ (scale dO V^T . mask)^T q~ + V (diag(e^{b_C - b_m}) dS)^T ]
//   dv = (scale q~ k~^T . mask)^T dO + k~ (diag(e^{b_C - b_m}) dS)
//   dS <- diag(e^{b_m}) [ diag(e^{b_C - b_m}) dS + scale q~^T dO ]
// The gate gradient is d g = reverse-cumsum_t (q . dq - k . dk) per channel, taken by the caller.
#include "mma_utils.cuh"

namespace lmoe {

constexpr int VCH = 64;
constexpr int VTHREADS = 256;

struct GlaArgs {
    const bf16 *q, *k, *v, *d_o;
    int64_t qs_b, qs_t, qs_h, ks_b, ks_t, ks_h, vs_b, vs_t, vs_h;
    bf16 *o, *dq, *dk, *dv;
    int64_t dqs_b, dqs_t, dqs_h, dks_b, dks_t, dks_h, dvs_b, dvs_t, dvs_h;
    const float* gk;               // [B,T,H,D] fp32 log decay
    float scale;
    int B, T, H, G, cpg;
    float* states;                 // [B,H,G,D,D]
    float* gdecay;                 // [B,H,G,D] total log decay of each group per channel
};

template <int D> struct VCfg {
    static constexpr int LD = D + 8;
    static constexpr int PLD = VCH + 8;
    static constexpr int S_RB = D / 16;
    static constexpr int S_NT = D * D / 1024;
    static constexpr int O_NT = D / 16;
};

// Load the chunk's gates, turn them into inclusive cumulative sums b[i][d] in shared memory (fp32, [VCH][D]).
template <int D>
__device__ __forceinline__ void load_cumsum(const GlaArgs& a, int b, int h, int c, float* bt) {
    const float* g = a.gk + (((int64_t)b * a.T + (int64_t)c * VCH) * a.H + h) * D;
    const int valid = a.T - c * VCH;
    for (int i = threadIdx.x; i < VCH * (D / 4); i += blockDim.x) {
        int r = i / (D / 4), cc = (i % (D / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < valid) v = *reinterpret_cast<const float4*>(g + (int64_t)r * a.H * D + cc);
        *reinterpret_cast<float4*>(bt + r * D + cc) = v;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float s = 0.f;
#pragma unroll 8
        for (int r = 0; r < VCH; ++r) { s += bt[r * D + d]; bt[r * D + d] = s; }
    }
    __syncthreads();
}

// tile[r][d] *= exp(sign * (bt[r][d] - ref[d])) * mul, ref[d] = bt[ref_row][d] (ref_row < 0: ref = 0)
template <int D, int LD>
__device__ __forceinline__ void rescale_tile(bf16* tile, const float* bt, int ref_row, float sign, float mul) {
    for (int i = threadIdx.x; i < VCH * (D / 2); i += blockDim.x) {
        int r = i / (D / 2), d = (i % (D / 2)) * 2;
        float r0 = ref_row >= 0 ? bt[ref_row * D + d] : 0.f, r1 = ref_row >= 0 ? bt[ref_row * D + d + 1] : 0.f;
        __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(tile + r * LD + d);
        float2 x = __bfloat1622float2(*p);
        x.x *= __expf(sign * (bt[r * D + d] - r0)) * mul;
        x.y *= __expf(sign * (bt[r * D + d + 1] - r1)) * mul;
        *p = __floats2bfloat162_rn(x.x, x.y);
    }
}

template <int NT>
__device__ __forceinline__ void rowscale_acc(float (&acc)[NT][4], float f0, float f1) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { acc[nt][0] *= f0; acc[nt][1] *= f0; acc[nt][2] *= f1; acc[nt][3] *= f1; }
}

// mask only (no decay): keep (row >= col) if LOWER else (row <= col); multiply by scale; store bf16
template <int LOWER>
__device__ __forceinline__ void mask_store_plain(const float (&acc)[4][4], bf16* P, int pld, int m0, int n0, float scale) {
    const int l = threadIdx.x & 31;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            int r = m0 + (l >> 2) + 8 * hh, c = n0 + nt * 8 + (l & 3) * 2;
            bool k0 = LOWER ? r >= c : r <= c, k1 = LOWER ? r >= c + 1 : r <= c + 1;
            *reinterpret_cast<__nv_bfloat162*>(P + r * pld + c) =
                __floats2bfloat162_rn(k0 ? acc[nt][2 * hh] * scale : 0.f, k1 ? acc[nt][2 * hh + 1] * scale : 0.f);
        }
}

template <int D, int LD>
__device__ __forceinline__ void vstore_tile(const bf16* smem, bf16* gmem, int64_t row_stride, int valid_rows) {
    constexpr int VPR = D / 8;
    for (int i = threadIdx.x; i < VCH * VPR; i += blockDim.x) {
        int r = i / VPR, c = (i % VPR) * 8;
        if (r < valid_rows)
            *reinterpret_cast<uint4*>(gmem + (int64_t)r * row_stride + c) = *reinterpret_cast<const uint4*>(smem + r * LD + c);
    }
}

// ---------------------------------------------------------------------------------------------
// 1. group summaries.  REV = 0: S <- diag(e^{b_C}) S + (K e^{b_C - b})^T V (ascending chunks)
//                      REV = 1: dS <- diag(e^{b_C}) dS + (Q e^{b} scale)^T dO (descending chunks)
// ---------------------------------------------------------------------------------------------
template <int D, int REV>
__global__ void __launch_bounds__(VTHREADS) gla_state_scan_kernel(GlaArgs a) {
    using C = VCfg<D>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Xs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ys = Xs + VCH * C::LD;
    float* bt = reinterpret_cast<float*>(Ys + VCH * C::LD);        // [VCH][D]
    const int grp = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int nchunks = (a.T + VCH - 1) / VCH;
    const int c_lo = grp * a.cpg, c_hi = min(nchunks, c_lo + a.cpg);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const int s_m0 = 16 * (w % C::S_RB), s_n0 = (w / C::S_RB) * (C::S_NT * 8);
    const bf16* xg = REV ? a.q + b * a.qs_b + h * a.qs_h : a.k + b * a.ks_b + h * a.ks_h;
    const int64_t xs_t = REV ? a.qs_t : a.ks_t;
    const bf16* yg = REV ? a.d_o + ((int64_t)b * a.T * a.H + h) * D : a.v + b * a.vs_b + h * a.vs_h;
    const int64_t ys_t = REV ? (int64_t)a.H * D : a.vs_t;
    float acc[C::S_NT][4];
    zero_acc<C::S_NT>(acc);
    float gs0 = 0.f, gs1 = 0.f;                                    // running group decay of rows r, r+8 (threads with l&3 == 0, s_n0 == 0)
    for (int i = 0; i < c_hi - c_lo; ++i) {
        const int c = REV ? c_hi - 1 - i : c_lo + i;
        load_tile_async<VCH, D, C::LD>(Xs, xg + (int64_t)c * VCH * xs_t, xs_t, a.T - c * VCH);
        load_tile_async<VCH, D, C::LD>(Ys, yg + (int64_t)c * VCH * ys_t, ys_t, a.T - c * VCH);
        cp_async_commit();
        load_cumsum<D>(a, b, h, c, bt);
        cp_async_wait<0>();
        __syncthreads();
        if (REV) rescale_tile<D, C::LD>(Xs, bt, -1, 1.f, a.scale);             // q e^{b} scale
        else rescale_tile<D, C::LD>(Xs, bt, VCH - 1, -1.f, 1.f);               // k e^{b_C - b}
        __syncthreads();
        const int r = s_m0 + (l >> 2);
        const float t0 = bt[(VCH - 1) * D + r], t1 = bt[(VCH - 1) * D + r + 8];
        rowscale_acc<C::S_NT>(acc, __expf(t0), __expf(t1));
        gs0 += t0; gs1 += t1;
        warp_gemm<C::S_NT, VCH, true, true>(acc, Xs, C::LD, s_m0, Ys, C::LD, s_n0);
        __syncthreads();
    }
    float* out = a.states + ((int64_t)bh * a.G + grp) * D * D;
    const int r = s_m0 + (l >> 2), cc = s_n0 + (l & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < C::S_NT; ++nt) {
        *reinterpret_cast<float2*>(out + (int64_t)r * D + cc + nt * 8) = make_float2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<float2*>(out + (int64_t)(r + 8) * D + cc + nt * 8) = make_float2(acc[nt][2], acc[nt][3]);
    }
    if (a.gdecay != nullptr && s_n0 == 0 && (l & 3) == 0) {
        float* gd = a.gdecay + ((int64_t)bh * a.G + grp) * D;
        gd[r] = gs0;
        gd[r + 8] = gs1;
    }
}

// 2. combine with a per-row (key channel) decay
template <int REV>
__global__ void gla_combine_kernel(float* __restrict__ states, const float* __restrict__ gdecay, const float* __restrict__ seed,
                                   float* __restrict__ final_out, int G, int D) {
    const int bh = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int DD = D * D;
    if (e >= DD) return;
    const int row = e / D;
    float carry = seed != nullptr ? seed[(int64_t)bh * DD + e] : 0.f;
    // batches of loads in flight together (a load per group that waits for the previous store is bound by memory latency)
    constexpr int NB = 8;
    for (int i0 = 0; i0 < G; i0 += NB) {
        float m[NB], dec[NB];
#pragma unroll
        for (int j = 0; j < NB; ++j)
            if (i0 + j < G) {
                const int g = REV ? G - 1 - (i0 + j) : i0 + j;
                m[j] = __ldcg(states + ((int64_t)bh * G + g) * DD + e);
                dec[j] = __expf(gdecay[((int64_t)bh * G + g) * D + row]);
            }
#pragma unroll
        for (int j = 0; j < NB; ++j)
            if (i0 + j < G) {
                const int g = REV ? G - 1 - (i0 + j) : i0 + j;
                states[((int64_t)bh * G + g) * DD + e] = carry;
                carry = dec[j] * carry + m[j];
            }
    }
    if (final_out != nullptr) final_out[(int64_t)bh * DD + e] = carry;
}

// Write diag(e^{f[row]}) * S (registers) as bf16 into Sb.
template <int D>
__device__ __forceinline__ void store_state_scaled(const float (&acc)[VCfg<D>::S_NT][4], bf16* Sb, int s_m0, int s_n0, float f0, float f1) {
    using C = VCfg<D>;
    const int l = threadIdx.x & 31;
    const int r = s_m0 + (l >> 2), c = s_n0 + (l & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < C::S_NT; ++nt) {
        *reinterpret_cast<__nv_bfloat162*>(Sb + r * C::LD + c + nt * 8) = __floats2bfloat162_rn(acc[nt][0] * f0, acc[nt][1] * f0);
        *reinterpret_cast<__nv_bfloat162*>(Sb + (r + 8) * C::LD + c + nt * 8) = __floats2bfloat162_rn(acc[nt][2] * f1, acc[nt][3] * f1);
    }
}

template <int D>
__device__ __forceinline__ void load_state_regs(const float* src, float (&acc)[VCfg<D>::S_NT][4], int s_m0, int s_n0) {
    using C = VCfg<D>;
    const int l = threadIdx.x & 31;
    const int r = s_m0 + (l >> 2), cc = s_n0 + (l & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < C::S_NT; ++nt) {
        float2 x = *reinterpret_cast<const float2*>(src + (int64_t)r * D + cc + nt * 8);
        float2 y = *reinterpret_cast<const float2*>(src + (int64_t)(r + 8) * D + cc + nt * 8);
        acc[nt][0] = x.x; acc[nt][1] = x.y; acc[nt][2] = y.x; acc[nt][3] = y.y;
    }
}

// ---------------------------------------------------------------------------------------------
// 3a. forward output (MODE 0) / backward dq (MODE 1): forward sweep carrying S.
// ---------------------------------------------------------------------------------------------
template <int D, int MODE>
__global__ void __launch_bounds__(VTHREADS) gla_fwd_sweep_kernel(GlaArgs a) {
    using C = VCfg<D>;
    constexpr int MID = VCH / 2 - 1;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Tq = reinterpret_cast<bf16*>(smem_raw);                  // q (mode 0) | dO (mode 1)
    bf16* Tk = Tq + VCH * C::LD;
    bf16* Tv = Tk + VCH * C::LD;
    bf16* Sb = Tv + VCH * C::LD;
    bf16* P = Sb + D * C::LD;
    float* bt = reinterpret_cast<float*>(P + VCH * C::PLD);
    const int grp = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int nchunks = (a.T + VCH - 1) / VCH;
    const int c_lo = grp * a.cpg, c_hi = min(nchunks, c_lo + a.cpg);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const int s_m0 = 16 * (w % C::S_RB), s_n0 = (w / C::S_RB) * (C::S_NT * 8);
    const int o_m0 = 16 * (w & 3), o_n0 = (w >> 2) * (D / 2);
    const int a_m0 = 16 * (w & 3), a_n0 = (w >> 2) * 32;
    const bf16* qg = MODE == 0 ? a.q + b * a.qs_b + h * a.qs_h : a.d_o + ((int64_t)b * a.T * a.H + h) * D;
    const int64_t qst = MODE == 0 ? a.qs_t : (int64_t)a.H * D;
    const bf16* kg = a.k + b * a.ks_b + h * a.ks_h;
    const bf16* vg = a.v + b * a.vs_b + h * a.vs_h;
    bf16* og; int64_t ost;
    if (MODE == 0) { og = a.o + ((int64_t)b * a.T * a.H + h) * D; ost = (int64_t)a.H * D; }
    else { og = a.dq + b * a.dqs_b + h * a.dqs_h; ost = a.dqs_t; }
    float acc_s[C::S_NT][4];
    load_state_regs<D>(a.states + ((int64_t)bh * a.G + grp) * D * D, acc_s, s_m0, s_n0);
    for (int c = c_lo; c < c_hi; ++c) {
        const int valid = a.T - c * VCH;
        load_tile_async<VCH, D, C::LD>(Tq, qg + (int64_t)c * VCH * qst, qst, valid);
        load_tile_async<VCH, D, C::LD>(Tk, kg + (int64_t)c * VCH * a.ks_t, a.ks_t, valid);
        load_tile_async<VCH, D, C::LD>(Tv, vg + (int64_t)c * VCH * a.vs_t, a.vs_t, valid);
        cp_async_commit();
        load_cumsum<D>(a, b, h, c, bt);
        cp_async_wait<0>();
        __syncthreads();
        if (MODE == 0) rescale_tile<D, C::LD>(Tq, bt, MID, 1.f, 1.f);          // q~ ; in mode 1 the tile is dO (unscaled)
        rescale_tile<D, C::LD>(Tk, bt, MID, -1.f, 1.f);                        // k~
        {
            const int r = s_m0 + (l >> 2);
            store_state_scaled<D>(acc_s, Sb, s_m0, s_n0, __expf(bt[MID * D + r]), __expf(bt[MID * D + r + 8]));
        }
        __syncthreads();
        float acc_o[C::O_NT][4], acc_a[4][4];
        zero_acc<C::O_NT>(acc_o);
        zero_acc<4>(acc_a);
        if (MODE == 0) {
            warp_gemm<C::O_NT, D, false, true>(acc_o, Tq, C::LD, o_m0, Sb, C::LD, o_n0);          // q~ (e^{b_m} S)
            warp_gemm<4, D, false, false>(acc_a, Tq, C::LD, a_m0, Tk, C::LD, a_n0);               // q~ k~^T
        } else {
            warp_gemm<C::O_NT, D, false, false>(acc_o, Tq, C::LD, o_m0, Sb, C::LD, o_n0);         // dO (e^{b_m} S)^T
            warp_gemm<4, D, false, false>(acc_a, Tq, C::LD, a_m0, Tv, C::LD, a_n0);               // dO V^T
        }
        rowscale_acc<C::O_NT>(acc_o, a.scale, a.scale);
        mask_store_plain<1>(acc_a, P, C::PLD, a_m0, a_n0, a.scale);
        __syncthreads();
        if (MODE == 0) warp_gemm<C::O_NT, VCH, false, true>(acc_o, P, C::PLD, o_m0, Tv, C::LD, o_n0);   // A V
        else warp_gemm<C::O_NT, VCH, false, true>(acc_o, P, C::PLD, o_m0, Tk, C::LD, o_n0);             // dA k~
        // state: S <- e^{b_C - b_m} [ e^{b_m} S + k~^T V ]
        {
            const int r = s_m0 + (l >> 2);
            const float m0 = bt[MID * D + r], m1 = bt[MID * D + r + 8];
            const float e0 = bt[(VCH - 1) * D + r], e1 = bt[(VCH - 1) * D + r + 8];
            rowscale_acc<C::S_NT>(acc_s, __expf(m0), __expf(m1));
            warp_gemm<C::S_NT, VCH, true, true>(acc_s, Tk, C::LD, s_m0, Tv, C::LD, s_n0);
            rowscale_acc<C::S_NT>(acc_s, __expf(e0 - m0), __expf(e1 - m1));
        }
        __syncthreads();                                            // Tq free (its last readers were before the previous barrier's gemms)
        store_acc_bf16<C::O_NT>(acc_o, Tq, C::LD, o_m0, o_n0);
        __syncthreads();
        if (MODE == 1) rescale_tile<D, C::LD>(Tq, bt, MID, 1.f, 1.f);          // dq = e^{b_i - b_m} . (...)
        __syncthreads();
        vstore_tile<D, C::LD>(Tq, og + (int64_t)c * VCH * ost, ost, valid);
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// 3b. backward dk, dv: reverse sweep carrying dS.
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(VTHREADS) gla_bwd_dkv_kernel(GlaArgs a) {
    using C = VCfg<D>;
    constexpr int MID = VCH / 2 - 1;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Tq = reinterpret_cast<bf16*>(smem_raw);
    bf16* Tk = Tq + VCH * C::LD;
    bf16* Tv = Tk + VCH * C::LD;
    bf16* Tg = Tv + VCH * C::LD;
    bf16* Sb = Tg + VCH * C::LD;                                    // diag(e^{b_C - b_m}) dS
    bf16* P1 = Sb + D * C::LD;
    bf16* P2 = P1 + VCH * C::PLD;
    float* bt = reinterpret_cast<float*>(P2 + VCH * C::PLD);
    const int grp = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int nchunks = (a.T + VCH - 1) / VCH;
    const int c_lo = grp * a.cpg, c_hi = min(nchunks, c_lo + a.cpg);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const int s_m0 = 16 * (w % C::S_RB), s_n0 = (w / C::S_RB) * (C::S_NT * 8);
    const int o_m0 = 16 * (w & 3), o_n0 = (w >> 2) * (D / 2);
    const int a_m0 = 16 * (w & 3), a_n0 = (w >> 2) * 32;
    const bf16* qg = a.q + b * a.qs_b + h * a.qs_h;
    const bf16* kg = a.k + b * a.ks_b + h * a.ks_h;
    const bf16* vg = a.v + b * a.vs_b + h * a.vs_h;
    const bf16* gg = a.d_o + ((int64_t)b * a.T * a.H + h) * D;
    const int64_t gst = (int64_t)a.H * D;
    bf16* dkg = a.dk + b * a.dks_b + h * a.dks_h;
    bf16* dvg = a.dv + b * a.dvs_b + h * a.dvs_h;
    float acc_s[C::S_NT][4];
    load_state_regs<D>(a.states + ((int64_t)bh * a.G + grp) * D * D, acc_s, s_m0, s_n0);
    for (int c = c_hi - 1; c >= c_lo; --c) {
        const int valid = a.T - c * VCH;
        load_tile_async<VCH, D, C::LD>(Tq, qg + (int64_t)c * VCH * a.qs_t, a.qs_t, valid);
        load_tile_async<VCH, D, C::LD>(Tk, kg + (int64_t)c * VCH * a.ks_t, a.ks_t, valid);
        load_tile_async<VCH, D, C::LD>(Tv, vg + (int64_t)c * VCH * a.vs_t, a.vs_t, valid);
        load_tile_async<VCH, D, C::LD>(Tg, gg + (int64_t)c * VCH * gst, gst, valid);
        cp_async_commit();
        load_cumsum<D>(a, b, h, c, bt);
        cp_async_wait<0>();
        __syncthreads();
        rescale_tile<D, C::LD>(Tq, bt, MID, 1.f, 1.f);
        rescale_tile<D, C::LD>(Tk, bt, MID, -1.f, 1.f);
        const int r = s_m0 + (l >> 2);
        const float m0 = bt[MID * D + r], m1 = bt[MID * D + r + 8];
        const float e0 = bt[(VCH - 1) * D + r], e1 = bt[(VCH - 1) * D + r + 8];
        store_state_scaled<D>(acc_s, Sb, s_m0, s_n0, __expf(e0 - m0), __expf(e1 - m1));
        __syncthreads();
        float acc_dv[C::O_NT][4], acc_dk[C::O_NT][4], acc_a[4][4], acc_b[4][4];
        zero_acc<C::O_NT>(acc_dv);
        zero_acc<C::O_NT>(acc_dk);
        zero_acc<4>(acc_a);
        zero_acc<4>(acc_b);
        warp_gemm<4, D, false, false>(acc_a, Tk, C::LD, a_m0, Tq, C::LD, a_n0);               // k~ q~^T
        warp_gemm<4, D, false, false>(acc_b, Tv, C::LD, a_m0, Tg, C::LD, a_n0);               // V dO^T
        warp_gemm<C::O_NT, D, false, true>(acc_dv, Tk, C::LD, o_m0, Sb, C::LD, o_n0);         // k~ (e^{b_C-b_m} dS)
        warp_gemm<C::O_NT, D, false, false>(acc_dk, Tv, C::LD, o_m0, Sb, C::LD, o_n0);        // V (e^{b_C-b_m} dS)^T
        mask_store_plain<0>(acc_a, P1, C::PLD, a_m0, a_n0, a.scale);
        mask_store_plain<0>(acc_b, P2, C::PLD, a_m0, a_n0, a.scale);
        __syncthreads();
        warp_gemm<C::O_NT, VCH, false, true>(acc_dv, P1, C::PLD, o_m0, Tg, C::LD, o_n0);      // Abar dO
        warp_gemm<C::O_NT, VCH, false, true>(acc_dk, P2, C::PLD, o_m0, Tq, C::LD, o_n0);      // Bbar q~
        // dS <- e^{b_m} [ e^{b_C - b_m} dS + scale q~^T dO ]: fold `scale` by scaling around the product
        rowscale_acc<C::S_NT>(acc_s, __expf(e0 - m0) / a.scale, __expf(e1 - m1) / a.scale);
        warp_gemm<C::S_NT, VCH, true, true>(acc_s, Tq, C::LD, s_m0, Tg, C::LD, s_n0);
        rowscale_acc<C::S_NT>(acc_s, __expf(m0) * a.scale, __expf(m1) * a.scale);
        __syncthreads();
        store_acc_bf16<C::O_NT>(acc_dv, Tv, C::LD, o_m0, o_n0);
        store_acc_bf16<C::O_NT>(acc_dk, Tk, C::LD, o_m0, o_n0);
        __syncthreads();
        rescale_tile<D, C::LD>(Tk, bt, MID, -1.f, 1.f);                        // dk = e^{b_m - b_j} . (...)
        __syncthreads();
        vstore_tile<D, C::LD>(Tv, dvg + (int64_t)c * VCH * a.dvs_t, a.dvs_t, valid);
        vstore_tile<D, C::LD>(Tk, dkg + (int64_t)c * VCH * a.dks_t, a.dks_t, valid);
        __syncthreads();
    }
}

template <int D> constexpr size_t gla_smem_scan() { return (size_t)2 * VCH * VCfg<D>::LD * 2 + (size_t)VCH * D * 4; }
template <int D> constexpr size_t gla_smem_sweep() {
    return (size_t)3 * VCH * VCfg<D>::LD * 2 + (size_t)D * VCfg<D>::LD * 2 + (size_t)VCH * VCfg<D>::PLD * 2 + (size_t)VCH * D * 4;
}
template <int D> constexpr size_t gla_smem_dkv() {
    return (size_t)4 * VCH * VCfg<D>::LD * 2 + (size_t)D * VCfg<D>::LD * 2 + (size_t)2 * VCH * VCfg<D>::PLD * 2 + (size_t)VCH * D * 4;
}

}  // namespace lmoe

using namespace lmoe;

// which: 0 forward state scan, 1 reverse state scan, 2 forward output, 3 backward dq, 4 backward dk/dv
LMOE_API int lmoe_gla_launch(int which, int D, const GlaArgs* ap, cudaStream_t st) {
    const GlaArgs a = *ap;
    dim3 grid(a.G, a.B * a.H);
#define GLAUNCH(KERNEL, SMEM)                                                                              \
    do {                                                                                                   \
        int rc = (int)cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(SMEM)); \
        if (rc) return rc;                                                                                 \
        KERNEL<<<grid, VTHREADS, SMEM, st>>>(a);                                                           \
    } while (0)
    if (D == 128) {
        if (which == 0) GLAUNCH((gla_state_scan_kernel<128, 0>), gla_smem_scan<128>());
        else if (which == 1) GLAUNCH((gla_state_scan_kernel<128, 1>), gla_smem_scan<128>());
        else if (which == 2) GLAUNCH((gla_fwd_sweep_kernel<128, 0>), gla_smem_sweep<128>());
        else if (which == 3) GLAUNCH((gla_fwd_sweep_kernel<128, 1>), gla_smem_sweep<128>());
        else if (which == 4) GLAUNCH((gla_bwd_dkv_kernel<128>), gla_smem_dkv<128>());
        else return -1;
    } else if (D == 64) {
        if (which == 0) GLAUNCH((gla_state_scan_kernel<64, 0>), gla_smem_scan<64>());
        else if (which == 1) GLAUNCH((gla_state_scan_kernel<64, 1>), gla_smem_scan<64>());
        else if (which == 2) GLAUNCH((gla_fwd_sweep_kernel<64, 0>), gla_smem_sweep<64>());
        else if (which == 3) GLAUNCH((gla_fwd_sweep_kernel<64, 1>), gla_smem_sweep<64>());
        else if (which == 4) GLAUNCH((gla_bwd_dkv_kernel<64>), gla_smem_dkv<64>());
        else return -1;
    } else return -2;
#undef GLAUNCH
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_gla_combine(int rev, float* states, const float* gdecay, const float* seed, float* final_out, int BH,
                              int G, int D, cudaStream_t st) {
    dim3 grid((D * D + 255) / 256, BH);
    if (rev) gla_combine_kernel<1><<<grid, 256, 0, st>>>(states, gdecay, seed, final_out, G, D);
    else gla_combine_kernel<0><<<grid, 256, 0, st>>>(states, gdecay, seed, final_out, G, D);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------------------
// Gradient of the vector log-gates: dg[b,t,h,d] = sum_{i >= t} (q . dq - k . dk)[b,i,h,d]  (reverse cumulative sum
// over time per channel).  Two launches over segments of 256 tokens: per-segment channel sums, then every segment
// walks its tokens backwards starting from the sum of the later segments.  20 bytes of traffic per element instead of
// the ~70 of the elementwise + transpose + cumsum formulation.
// ---------------------------------------------------------------------------------------------------------------
namespace lmoe {
constexpr int DG_SEG = 256;
struct DgArgs {
    const bf16 *q, *k, *dq, *dk;
    int64_t qs_b, qs_t, qs_h, ks_b, ks_t, ks_h, dqs_b, dqs_t, dqs_h, dks_b, dks_t, dks_h;
    float* dg;            // [B,T,H,D] contiguous
    float* segsum;        // [B*H, nseg, D]
    int B, T, H, D, nseg;
};
// q*dq - k*dk for eight consecutive channels of one token (16-byte loads; the pitches are multiples of 8 elements)
__device__ __forceinline__ void dg_term8(const DgArgs& a, int b, int t, int h, int d, float (&o)[8]) {
    const uint4 q4 = __ldg(reinterpret_cast<const uint4*>(a.q + b * a.qs_b + (int64_t)t * a.qs_t + h * a.qs_h + d));
    const uint4 k4 = __ldg(reinterpret_cast<const uint4*>(a.k + b * a.ks_b + (int64_t)t * a.ks_t + h * a.ks_h + d));
    const uint4 dq4 = __ldg(reinterpret_cast<const uint4*>(a.dq + b * a.dqs_b + (int64_t)t * a.dqs_t + h * a.dqs_h + d));
    const uint4 dk4 = __ldg(reinterpret_cast<const uint4*>(a.dk + b * a.dks_b + (int64_t)t * a.dks_t + h * a.dks_h + d));
    const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&q4);
    const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&k4);
    const __nv_bfloat162* dq2 = reinterpret_cast<const __nv_bfloat162*>(&dq4);
    const __nv_bfloat162* dk2 = reinterpret_cast<const __nv_bfloat162*>(&dk4);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 fq = __bfloat1622float2(q2[i]), fk = __bfloat1622float2(k2[i]);
        const float2 fdq = __bfloat1622float2(dq2[i]), fdk = __bfloat1622float2(dk2[i]);
        o[2 * i] = fq.x * fdq.x - fk.x * fdk.x;
        o[2 * i + 1] = fq.y * fdq.y - fk.y * fdk.y;
    }
}

// Both kernels: grid (nseg, B*H), 256 threads.  D / 8 threads cover the channels of one token with 16-byte accesses;
// the 256 / (D / 8) thread groups each own a contiguous run of DG_SEG / groups tokens of the segment.
// 1. per-segment sums of the terms
__global__ void __launch_bounds__(256) gla_dg_segsum_kernel(DgArgs a) {
    __shared__ float part[32][129];                                    // [group][channel], D <= 128
    const int seg = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int tpr = a.D / 8, groups = 256 / tpr, L = DG_SEG / groups;
    const int grp = threadIdx.x / tpr, d = (threadIdx.x % tpr) * 8;
    const int t0 = seg * DG_SEG + grp * L, t1 = min(a.T, t0 + L);
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
        float o[8];
        dg_term8(a, b, t, h, d, o);
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] += o[i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) part[grp][d + i] = s[i];
    __syncthreads();
    if (threadIdx.x < a.D) {
        float tot = 0.f;
        for (int g2 = 0; g2 < groups; ++g2) tot += part[g2][threadIdx.x];
        a.segsum[((int64_t)bh * a.nseg + seg) * a.D + threadIdx.x] = tot;
    }
}
// 2. running suffix sums: later segments from the table, later token runs of this segment through shared memory, then
//    the run's own tokens from last to first (re-read; they are in L2 from the first pass of this CTA)
__global__ void __launch_bounds__(256) gla_dg_scan_kernel(DgArgs a) {
    __shared__ float part[32][129];
    const int seg = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int tpr = a.D / 8, groups = 256 / tpr, L = DG_SEG / groups;
    const int grp = threadIdx.x / tpr, d = (threadIdx.x % tpr) * 8;
    const int t0 = seg * DG_SEG + grp * L, t1 = min(a.T, t0 + L);
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
        float o[8];
        dg_term8(a, b, t, h, d, o);
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] += o[i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) part[grp][d + i] = s[i];
    __syncthreads();
    float run[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float r = 0.f;
        for (int s2 = a.nseg - 1; s2 > seg; --s2) r += a.segsum[((int64_t)bh * a.nseg + s2) * a.D + d + i];
        for (int g2 = groups - 1; g2 > grp; --g2) r += part[g2][d + i];
        run[i] = r;
    }
    for (int t = t1 - 1; t >= t0; --t) {
        float o[8];
        dg_term8(a, b, t, h, d, o);
#pragma unroll
        for (int i = 0; i < 8; ++i) run[i] += o[i];
        float4* dst = reinterpret_cast<float4*>(a.dg + (((int64_t)b * a.T + t) * a.H + h) * a.D + d);
        dst[0] = make_float4(run[0], run[1], run[2], run[3]);
        dst[1] = make_float4(run[4], run[5], run[6], run[7]);
    }
}
}  // namespace lmoe

LMOE_API int lmoe_gla_dg(const lmoe::DgArgs* ap, cudaStream_t st) {
    lmoe::DgArgs a = *ap;
    if ((a.D != 64 && a.D != 128) || a.T <= 0) return -1;
    if ((a.qs_t | a.qs_h | a.qs_b | a.ks_t | a.ks_h | a.ks_b | a.dqs_t | a.dqs_h | a.dqs_b | a.dks_t | a.dks_h | a.dks_b) % 8) return -1;
    if (((uintptr_t)a.q | (uintptr_t)a.k | (uintptr_t)a.dq | (uintptr_t)a.dk) & 15) return -1;
    a.nseg = (a.T + lmoe::DG_SEG - 1) / lmoe::DG_SEG;
    dim3 grid(a.nseg, a.B * a.H);
    lmoe::gla_dg_segsum_kernel<<<grid, 256, 0, st>>>(a);
    lmoe::gla_dg_scan_kernel<<<grid, 256, 0, st>>>(a);
    return (int)cudaGetLastError();
}
