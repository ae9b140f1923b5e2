// (Gated) delta rule: the recurrence over chunks, forward and backward, as hand-written kernels.
//
//   S_t = e^{g_t} S_{t-1} + beta_t k_t^T (v_t - k_t e^{g_t} S_{t-1}),      o_t = scale * q_t S_t
//
// In the chunked (WY / UT-transform) form every chunk of C = 64 tokens is described by tiles that do not depend on
// the state (computed chunk-parallel before this kernel):
//   W  [C,dk]  pseudo keys      T (beta e^{b} K),        T = (I + tril(diag(beta) (K K^T . Gamma), -1))^{-1}
//   U  [C,dv]  pseudo values    T (beta V)
//   Qd [C,dk]  scale * e^{b_i} q_i           Kd [C,dk]  e^{b_C - b_j} k_j
//   A  [C,C]   scale * tril((Q K^T) . Gamma)  (diagonal included),   Gamma_ij = e^{b_i - b_j},   gamma = e^{b_C}
// and the state-dependent part is, per chunk with entering state S,
//   Vn = U - W S,        O = Qd S + A Vn,        S' = gamma S + Kd^T Vn.
// The columns of S are independent, so a (batch, head) sequence is split over dv / 32 CTAs (value slices) to fill the
// machine; a CTA walks the chunks in order with its [dk x 32] state slice in fp32 registers and a bf16 copy in shared
// memory as the B operand.  The forward kernel also writes Vn and the entering state of every chunk (bf16): with them
// the gradients of W, U, Qd, Kd, A and gamma are chunk-parallel products; only the state gradient
//   dVn = A^T dO + Kd dS',      dS = gamma dS' + Qd^T dO - W^T dVn
// is a recurrence, walked in reverse by the backward kernel, which writes dVn and the dS' of every chunk.
//
// Reference counterpart: fla.ops.gated_delta_rule / delta_rule chunk kernels called by
// sequence_modeling/gated_deltanet/gated_deltanet.py:99-116 and deltanet/deltanet.py:127-130.
#include "mma_utils.cuh"

namespace lmoe {
namespace dr {

constexpr int C = 64;            // chunk length
constexpr int DVS = 32;          // value columns per CTA
constexpr int NT = 128;          // threads

struct Args {
    const bf16 *W, *U, *Qd, *Kd, *A;   // [BH, N, C, dk] / [BH, N, C, dv] / [BH, N, C, C]
    const float* gamma;                // [BH, N]
    const float* S0;                   // [BH, dk, dv] or null
    const bf16* dO;                    // backward: [BH, N, C, dv]
    const float* dSfinal;              // backward: [BH, dk, dv] or null
    bf16* O;                           // forward: [BH, N, C, dv]
    bf16* Vn;                          // forward out / backward in: [BH, N, C, dv]
    bf16* Sn;                          // forward out: state entering chunk n, [BH, N, dk, dv]
    float* Sfinal;                     // forward out: [BH, dk, dv]
    bf16* dVn;                         // backward out: [BH, N, C, dv]
    bf16* dSn;                         // backward out: gradient of the state leaving chunk n, [BH, N, dk, dv]
    float* dS0;                        // backward out: [BH, dk, dv]
    int N, dv;
};

template <int DK> struct Cfg {
    static constexpr int LDK = DK + 8;
    static constexpr int LDC = C + 8;
    static constexpr int LDV = DVS + 8;
    static constexpr int RB = DK / 64;              // 16-row blocks of the state per warp (4 warps)
    // shared memory (bf16 elements): 2 x {W, Qd, Kd: C x LDK; A: C x LDC; X (U or dO): C x LDV} + Sb [DK x LDV] + Vb [C x LDV] (+ Gb)
    static constexpr int STAGE = 3 * C * LDK + C * LDC + C * LDV;
    static constexpr size_t SMEM = (size_t)(2 * STAGE + DK * LDV + 2 * C * LDV) * 2;
};

template <int DK>
__device__ __forceinline__ void issue_chunk(bf16* st, const Args& a, const bf16* xsrc, long long bh, int n, int col0) {
    using F = Cfg<DK>;
    const long long cn = bh * a.N + n;
    load_tile_async<C, DK, F::LDK>(st, a.W + cn * C * DK, DK, C);
    load_tile_async<C, DK, F::LDK>(st + C * F::LDK, a.Qd + cn * C * DK, DK, C);
    load_tile_async<C, DK, F::LDK>(st + 2 * C * F::LDK, a.Kd + cn * C * DK, DK, C);
    load_tile_async<C, C, F::LDC>(st + 3 * C * F::LDK, a.A + cn * C * C, C, C);
    load_tile_async<C, DVS, F::LDV>(st + 3 * C * F::LDK + C * F::LDC, xsrc + cn * C * a.dv + col0, a.dv, C);
}

// write a [rows x DVS] bf16 tile held in shared memory (row stride LDV) to global rows of stride `gld`
template <int LDV>
__device__ __forceinline__ void store_rows(const bf16* s, bf16* g, int rows, long long gld) {
    for (int i = threadIdx.x; i < rows * (DVS / 8); i += NT) {
        const int r = i / (DVS / 8), c = (i % (DVS / 8)) * 8;
        *reinterpret_cast<uint4*>(g + (long long)r * gld + c) = *reinterpret_cast<const uint4*>(s + r * LDV + c);
    }
}

template <int DK>
__global__ void __launch_bounds__(NT) delta_scan_fwd_kernel(Args a) {
    using F = Cfg<DK>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* stage = reinterpret_cast<bf16*>(smem_raw);
    bf16* Sb = stage + 2 * F::STAGE;                 // [DK][LDV]
    bf16* Vb = Sb + DK * F::LDV;                     // [C][LDV]  Vn of the chunk
    bf16* Ob = Vb + C * F::LDV;                      // [C][LDV]  output staging
    const int col0 = blockIdx.x * DVS;
    const long long bh = blockIdx.y;
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;

    // state slice: warp w owns rows [w*16*RB, +16*RB) x 32 columns
    float S[F::RB][4][4];
#pragma unroll
    for (int rb = 0; rb < F::RB; ++rb) {
        const int r = (w * F::RB + rb) * 16 + (l >> 2);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int c = col0 + nt * 8 + (l & 3) * 2;
            if (a.S0 != nullptr) {
                const float* p = a.S0 + (bh * DK + r) * a.dv + c;
                S[rb][nt][0] = p[0]; S[rb][nt][1] = p[1];
                S[rb][nt][2] = p[8 * a.dv]; S[rb][nt][3] = p[8 * a.dv + 1];
            } else {
                S[rb][nt][0] = S[rb][nt][1] = S[rb][nt][2] = S[rb][nt][3] = 0.f;
            }
        }
        store_acc_bf16<4>(S[rb], Sb, F::LDV, (w * F::RB + rb) * 16, 0);
    }
    if (a.N > 0) issue_chunk<DK>(stage, a, a.U, bh, 0, col0);
    cp_async_commit();
    for (int n = 0; n < a.N; ++n) {
        bf16* st = stage + (n & 1) * F::STAGE;
        if (n + 1 < a.N) issue_chunk<DK>(stage + ((n + 1) & 1) * F::STAGE, a, a.U, bh, n + 1, col0);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();                                           // tiles of chunk n and Sb visible
        const bf16* Wt = st;
        const bf16* Qt = st + C * F::LDK;
        const bf16* Kt = st + 2 * C * F::LDK;
        const bf16* At = st + 3 * C * F::LDK;
        const bf16* Ut = At + C * F::LDC;
        const float gamma = a.gamma[bh * a.N + n];
        // entering state of this chunk (bf16), for the backward pass
        store_rows<F::LDV>(Sb, a.Sn + ((bh * a.N + n) * DK) * a.dv + col0, DK, a.dv);
        // Vn = U - W S   (warp w: rows 16w .. 16w+15)
        float acc[4][4];
        zero_acc<4>(acc);
        warp_gemm<4, DK, false, true>(acc, Wt, F::LDK, 16 * w, Sb, F::LDV, 0);
        {
            const int r = 16 * w + (l >> 2);
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const int c = nt * 8 + (l & 3) * 2;
                const __nv_bfloat162 u0 = *reinterpret_cast<const __nv_bfloat162*>(Ut + r * F::LDV + c);
                const __nv_bfloat162 u1 = *reinterpret_cast<const __nv_bfloat162*>(Ut + (r + 8) * F::LDV + c);
                acc[nt][0] = __bfloat162float(u0.x) - acc[nt][0]; acc[nt][1] = __bfloat162float(u0.y) - acc[nt][1];
                acc[nt][2] = __bfloat162float(u1.x) - acc[nt][2]; acc[nt][3] = __bfloat162float(u1.y) - acc[nt][3];
            }
        }
        store_acc_bf16<4>(acc, Vb, F::LDV, 16 * w, 0);
        // O = Qd S (needs only Sb) ...
        float acc_o[4][4];
        zero_acc<4>(acc_o);
        warp_gemm<4, DK, false, true>(acc_o, Qt, F::LDK, 16 * w, Sb, F::LDV, 0);
        __syncthreads();                                           // Vb complete; every read of Sb done
        // ... + A Vn
        warp_gemm<4, C, false, true>(acc_o, At, F::LDC, 16 * w, Vb, F::LDV, 0);
        store_acc_bf16<4>(acc_o, Ob, F::LDV, 16 * w, 0);
        // S <- gamma S + Kd^T Vn
#pragma unroll
        for (int rb = 0; rb < F::RB; ++rb) {
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) S[rb][nt][e] *= gamma;
            warp_gemm<4, C, true, true>(S[rb], Kt, F::LDK, (w * F::RB + rb) * 16, Vb, F::LDV, 0);
            store_acc_bf16<4>(S[rb], Sb, F::LDV, (w * F::RB + rb) * 16, 0);
        }
        __syncthreads();                                           // Ob, Vb, new Sb complete
        store_rows<F::LDV>(Ob, a.O + ((bh * a.N + n) * C) * a.dv + col0, C, a.dv);
        store_rows<F::LDV>(Vb, a.Vn + ((bh * a.N + n) * C) * a.dv + col0, C, a.dv);
        __syncthreads();                                           // staging drained before the next chunk rewrites it
    }
#pragma unroll
    for (int rb = 0; rb < F::RB; ++rb) {
        const int r = (w * F::RB + rb) * 16 + (l >> 2);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int c = col0 + nt * 8 + (l & 3) * 2;
            float* p = a.Sfinal + (bh * DK + r) * a.dv + c;
            p[0] = S[rb][nt][0]; p[1] = S[rb][nt][1];
            p[8 * a.dv] = S[rb][nt][2]; p[8 * a.dv + 1] = S[rb][nt][3];
        }
    }
}

// Reverse walk: dS' enters from the right (gradient of the state leaving the chunk).
template <int DK>
__global__ void __launch_bounds__(NT) delta_scan_bwd_kernel(Args a) {
    using F = Cfg<DK>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* stage = reinterpret_cast<bf16*>(smem_raw);
    bf16* Sb = stage + 2 * F::STAGE;                 // [DK][LDV]  bf16 copy of dS'
    bf16* Vb = Sb + DK * F::LDV;                     // [C][LDV]   dVn of the chunk
    const int col0 = blockIdx.x * DVS;
    const long long bh = blockIdx.y;
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;

    float S[F::RB][4][4];
#pragma unroll
    for (int rb = 0; rb < F::RB; ++rb) {
        const int r = (w * F::RB + rb) * 16 + (l >> 2);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int c = col0 + nt * 8 + (l & 3) * 2;
            if (a.dSfinal != nullptr) {
                const float* p = a.dSfinal + (bh * DK + r) * a.dv + c;
                S[rb][nt][0] = p[0]; S[rb][nt][1] = p[1];
                S[rb][nt][2] = p[8 * a.dv]; S[rb][nt][3] = p[8 * a.dv + 1];
            } else {
                S[rb][nt][0] = S[rb][nt][1] = S[rb][nt][2] = S[rb][nt][3] = 0.f;
            }
        }
        store_acc_bf16<4>(S[rb], Sb, F::LDV, (w * F::RB + rb) * 16, 0);
    }
    if (a.N > 0) issue_chunk<DK>(stage, a, a.dO, bh, a.N - 1, col0);
    cp_async_commit();
    for (int i = 0; i < a.N; ++i) {
        const int n = a.N - 1 - i;
        bf16* st = stage + (i & 1) * F::STAGE;
        if (n > 0) issue_chunk<DK>(stage + ((i + 1) & 1) * F::STAGE, a, a.dO, bh, n - 1, col0);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* Wt = st;
        const bf16* Qt = st + C * F::LDK;
        const bf16* Kt = st + 2 * C * F::LDK;
        const bf16* At = st + 3 * C * F::LDK;
        const bf16* Gt = At + C * F::LDC;             // dO slice
        const float gamma = a.gamma[bh * a.N + n];
        store_rows<F::LDV>(Sb, a.dSn + ((bh * a.N + n) * DK) * a.dv + col0, DK, a.dv);
        // dVn = A^T dO + Kd dS'
        float acc[4][4];
        zero_acc<4>(acc);
        warp_gemm<4, C, true, true>(acc, At, F::LDC, 16 * w, Gt, F::LDV, 0);
        warp_gemm<4, DK, false, true>(acc, Kt, F::LDK, 16 * w, Sb, F::LDV, 0);
        store_acc_bf16<4>(acc, Vb, F::LDV, 16 * w, 0);
        __syncthreads();                                           // Vb complete; reads of Sb done
        // dS = gamma dS' + Qd^T dO - W^T dVn
#pragma unroll
        for (int rb = 0; rb < F::RB; ++rb) {
            float t[4][4];
            zero_acc<4>(t);
            warp_gemm<4, C, true, true>(t, Wt, F::LDK, (w * F::RB + rb) * 16, Vb, F::LDV, 0);
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) S[rb][nt][e] = S[rb][nt][e] * gamma - t[nt][e];
            warp_gemm<4, C, true, true>(S[rb], Qt, F::LDK, (w * F::RB + rb) * 16, Gt, F::LDV, 0);
            store_acc_bf16<4>(S[rb], Sb, F::LDV, (w * F::RB + rb) * 16, 0);
        }
        store_rows<F::LDV>(Vb, a.dVn + ((bh * a.N + n) * C) * a.dv + col0, C, a.dv);
        __syncthreads();
    }
#pragma unroll
    for (int rb = 0; rb < F::RB; ++rb) {
        const int r = (w * F::RB + rb) * 16 + (l >> 2);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int c = col0 + nt * 8 + (l & 3) * 2;
            float* p = a.dS0 + (bh * DK + r) * a.dv + c;
            p[0] = S[rb][nt][0]; p[1] = S[rb][nt][1];
            p[8 * a.dv] = S[rb][nt][2]; p[8 * a.dv + 1] = S[rb][nt][3];
        }
    }
}


// ---------------------------------------------------------------------------------------------------------------
// Chunk-parallel construction of the tiles (forward): one CTA per (batch, head, chunk).
//   b_i = inclusive cumulative log decay inside the chunk,  Gamma_ij = e^{b_i - b_j}
//   A   = strictly-lower(diag(beta) (K K^T . Gamma)),   T = (I + A)^{-1}   (column c of T lives in the registers of
//         thread c: row i needs only rows < i of the same column, so the substitution runs without any barrier)
//   W = T (beta e^{b} K),  U = T (beta V),  Aqk = scale tril((Q K^T) . Gamma),  Qd = scale e^{b} Q,  Kd = e^{b_C - b} K
// ---------------------------------------------------------------------------------------------------------------
struct PrepArgs {
    const bf16 *q, *k, *v;             // [B,T,H,D] with the strides below (elements)
    long long qs_b, qs_t, qs_h, ks_b, ks_t, ks_h, vs_b, vs_t, vs_h;
    const float* beta;                 // [B,T,H]
    const float* g;                    // [B,T,H] log decay, or null
    bf16 *W, *U, *Qd, *Kd, *A;         // outputs, [BH, N, C, D] / [BH, N, C, C]
    float* gamma;                      // [BH, N]
    int B, T, H, N;
    float scale;
};

template <int D>
__global__ void __launch_bounds__(NT) delta_prep_fwd_kernel(PrepArgs a) {
    constexpr int LD = D + 8, LDC = C + 8, LDA = C + 1;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Ks = reinterpret_cast<bf16*>(smem_raw);            // [C][LD]
    bf16* Vs = Ks + C * LD;                                  // [C][LD]  V, then beta V
    bf16* Qs = Vs + C * LD;                                  // [C][LD]
    bf16* Kb = Qs + C * LD;                                  // [C][LD]  beta e^b K
    bf16* Tb = Kb + C * LD;                                  // [C][LDC] T in bf16
    float* A32 = reinterpret_cast<float*>(Tb + C * LDC);     // [C][LDA] strictly lower A
    float* bcum = A32 + C * LDA;                             // [C]
    float* bet = bcum + C;                                   // [C]
    const int n = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const int t0 = n * C;
    const int valid = min(C, a.T - t0);
    const long long cn = (long long)bh * a.N + n;

    load_tile_async<C, D, LD>(Ks, a.k + b * a.ks_b + h * a.ks_h + (long long)t0 * a.ks_t, a.ks_t, valid);
    load_tile_async<C, D, LD>(Vs, a.v + b * a.vs_b + h * a.vs_h + (long long)t0 * a.vs_t, a.vs_t, valid);
    load_tile_async<C, D, LD>(Qs, a.q + b * a.qs_b + h * a.qs_h + (long long)t0 * a.qs_t, a.qs_t, valid);
    cp_async_commit();
    if (w == 0) {                                            // decay table: two tokens per lane, warp scan
        const int i0 = 2 * l, i1 = 2 * l + 1;
        float g0 = 0.f, g1 = 0.f, be0 = 0.f, be1 = 0.f;
        if (i0 < valid) {
            const long long o = ((long long)b * a.T + t0 + i0) * a.H + h;
            be0 = a.beta[o];
            if (a.g != nullptr) g0 = a.g[o];
        }
        if (i1 < valid) {
            const long long o = ((long long)b * a.T + t0 + i1) * a.H + h;
            be1 = a.beta[o];
            if (a.g != nullptr) g1 = a.g[o];
        }
        float s = g0 + g1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float x = __shfl_up_sync(0xffffffffu, s, o);
            if (l >= o) s += x;
        }
        bcum[i1] = s;
        bcum[i0] = s - g1;
        bet[i0] = be0;
        bet[i1] = be1;
    }
    cp_async_wait<0>();
    __syncthreads();
    const float btot = bcum[C - 1];
    // ---- K K^T -> A (fp32, strictly lower) and Q K^T -> Aqk (bf16, to global); warp w owns rows 16w .. 16w+15
    {
        float kk[8][4], qk[8][4];
        zero_acc<8>(kk);
        zero_acc<8>(qk);
        warp_gemm<8, D, false, false>(kk, Ks, LD, 16 * w, Ks, LD, 0);
        warp_gemm<8, D, false, false>(qk, Qs, LD, 16 * w, Ks, LD, 0);
        bf16* Ag = a.A + cn * C * C;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = 16 * w + (l >> 2) + 8 * hh;
                const int j = nt * 8 + (l & 3) * 2;
                const float bi = bcum[i], be = bet[i];
                const float d0 = __expf(bi - bcum[j]), d1 = __expf(bi - bcum[j + 1]);
                A32[i * LDA + j] = i > j ? be * d0 * kk[nt][2 * hh] : 0.f;
                A32[i * LDA + j + 1] = i > j + 1 ? be * d1 * kk[nt][2 * hh + 1] : 0.f;
                const float a0 = i >= j ? a.scale * d0 * qk[nt][2 * hh] : 0.f;
                const float a1 = i >= j + 1 ? a.scale * d1 * qk[nt][2 * hh + 1] : 0.f;
                *reinterpret_cast<__nv_bfloat162*>(Ag + i * C + j) = __floats2bfloat162_rn(a0, a1);
            }
    }
    __syncthreads();
    // ---- threads 0..63: column c of T = (I + A)^{-1} by forward substitution, entirely in registers;
    //      threads 64..127: the elementwise tiles (beta e^b K -> Kb, beta V in place, Qd and Kd to global)
    if (threadIdx.x < C) {
        const int c = threadIdx.x;
        float t[C];
#pragma unroll
        for (int i = 0; i < C; ++i) {
            float acc = (i == c) ? 1.f : 0.f;
#pragma unroll
            for (int j = 0; j < i; ++j) acc -= A32[i * LDA + j] * t[j];
            t[i] = acc;
        }
#pragma unroll
        for (int i = 0; i < C; ++i) Tb[i * LDC + c] = __float2bfloat16(t[i]);
    } else {
        const int tid = threadIdx.x - C;                      // 0..63: one row each
        const int i = tid;
        const float bi = bcum[i], be = bet[i];
        const float fk = be * __expf(bi), fq = a.scale * __expf(bi), fd = __expf(btot - bi);
        bf16* Qg = a.Qd + (cn * C + i) * D;
        bf16* Kg = a.Kd + (cn * C + i) * D;
#pragma unroll 4
        for (int c = 0; c < D; c += 8) {
            Vec<bf16> kx, vx, qx, o1, o2, o3, o4;
            kx.load(Ks + i * LD + c);
            vx.load(Vs + i * LD + c);
            qx.load(Qs + i * LD + c);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                o1.set(e, kx.get(e) * fk);
                o2.set(e, vx.get(e) * be);
                o3.set(e, qx.get(e) * fq);
                o4.set(e, kx.get(e) * fd);
            }
            o1.store(Kb + i * LD + c);
            o2.store(Vs + i * LD + c);
            o3.store(Qg + c);
            o4.store(Kg + c);
        }
        if (tid == 0) a.gamma[cn] = __expf(btot);
    }
    __syncthreads();
    // ---- W = T Kb, U = T (beta V): warp w -> rows 16w .. 16w+15, all D columns
    {
        float acc[D / 8][4];
        zero_acc<D / 8>(acc);
        warp_gemm<D / 8, C, false, true>(acc, Tb, LDC, 16 * w, Kb, LD, 0);
        bf16* Wg = a.W + cn * C * D;
        const int r = 16 * w + (l >> 2), cc = (l & 3) * 2;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) {
            *reinterpret_cast<__nv_bfloat162*>(Wg + r * D + cc + nt * 8) = __floats2bfloat162_rn(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<__nv_bfloat162*>(Wg + (r + 8) * D + cc + nt * 8) = __floats2bfloat162_rn(acc[nt][2], acc[nt][3]);
        }
        zero_acc<D / 8>(acc);
        warp_gemm<D / 8, C, false, true>(acc, Tb, LDC, 16 * w, Vs, LD, 0);
        bf16* Ug = a.U + cn * C * D;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) {
            *reinterpret_cast<__nv_bfloat162*>(Ug + r * D + cc + nt * 8) = __floats2bfloat162_rn(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<__nv_bfloat162*>(Ug + (r + 8) * D + cc + nt * 8) = __floats2bfloat162_rn(acc[nt][2], acc[nt][3]);
        }
    }
}


// ---------------------------------------------------------------------------------------------------------------
// Chunk-parallel backward of everything that is not the state recurrence: one CTA per (batch, head, chunk).
// Inputs: q, k, v, beta, g (to rebuild the tiles), the entering state S_n and the gradient dS'_n of the leaving state,
// Vn, dVn (= dU) and dO of the chunk (written by the two scan kernels).  The gradient of the chunk's total decay,
// dgamma_n = <dS'_n, S_n> (gated case), is formed here too: every thread keeps its share of S_n in registers while the
// state buffer is refilled with dS'_n.
//
//   through the scan equations      dW = -dVn S^T,  dQd = dO S^T,  dKd = Vn dS'^T,  dAqk = tril(dO Vn^T)
//   through W = T Kb, U = T Vb      dKb = T^T dW,  dVb = T^T dU,  dT = dW Kb^T + dU Vb^T,  dA = -strict_lower(T^T dT T^T)
//   through the tiles               dq = s e^b dQd + P K                         P = s Gamma . dAqk
//                                   dk = e^{b_C-b} dKd + P^T Q + beta e^b dKb + M K + M^T K          M = beta_i Gamma . dA
//                                   dv = beta dVb
//                                   dbeta_i = e^{b_i} <dKb_i, k_i> + <dVb_i, v_i> + sum_j dA_ij Gamma_ij (k_i.k_j)
//                                   db_i (gradient of the cumulative log decay) from every e^{b}: rows minus columns of
//                                   dAqk . Aqk and dA . A, +<dQd_i, Qd_i>, -<dKd_j, Kd_j> (and their sum on b_C),
//                                   +beta_i e^{b_i} <dKb_i, k_i>, + dgamma gamma on b_C;   dg_s = sum_{i >= s} db_i
// The products are mma.sync tiles on bf16 copies in shared memory with fp32 accumulation; dk accumulates in registers
// across the phases, every other output is finished inside one phase.
// ---------------------------------------------------------------------------------------------------------------
struct PrepBwdArgs {
    const bf16 *q, *k, *v;
    long long qs_b, qs_t, qs_h, ks_b, ks_t, ks_h, vs_b, vs_t, vs_h;
    const float* beta;
    const float* g;                    // or null
    const bf16 *Sn, *dSn;              // [BH, N, D, D]
    const bf16 *Vn, *dVn, *dO;         // [BH, N, C, D]
    bf16 *dq, *dk, *dv;                // contiguous [B, T, H, D]
    float *dbeta, *dg;                 // [B, T, H]
    int B, T, H, N;
    float scale;
};

// sum over the thread's columns of acc[row][col] * tile[row][col] for its two rows (r, r + 8), reduced over the quad
template <int NTL>
__device__ __forceinline__ void row_dot(const float (&acc)[NTL][4], const bf16* tile, int ld, int m0, float& lo, float& hi) {
    const int l = threadIdx.x & 31;
    const int r = m0 + (l >> 2), c = (l & 3) * 2;
    lo = 0.f; hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < NTL; ++nt) {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(tile + r * ld + c + nt * 8);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(tile + (r + 8) * ld + c + nt * 8);
        lo += acc[nt][0] * __bfloat162float(a.x) + acc[nt][1] * __bfloat162float(a.y);
        hi += acc[nt][2] * __bfloat162float(b.x) + acc[nt][3] * __bfloat162float(b.y);
    }
    lo += __shfl_xor_sync(0xffffffffu, lo, 1); lo += __shfl_xor_sync(0xffffffffu, lo, 2);
    hi += __shfl_xor_sync(0xffffffffu, hi, 1); hi += __shfl_xor_sync(0xffffffffu, hi, 2);
}

// write a warp's [16 x 8 NTL] accumulator rows to global rows (bf16), rows >= valid skipped
template <int NTL>
__device__ __forceinline__ void store_rows_global(const float (&acc)[NTL][4], bf16* g, long long row_stride, int m0, int valid) {
    const int l = threadIdx.x & 31;
    const int r = m0 + (l >> 2), c = (l & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < NTL; ++nt) {
        if (r < valid) *reinterpret_cast<__nv_bfloat162*>(g + r * row_stride + c + nt * 8) = __floats2bfloat162_rn(acc[nt][0], acc[nt][1]);
        if (r + 8 < valid) *reinterpret_cast<__nv_bfloat162*>(g + (r + 8) * row_stride + c + nt * 8) = __floats2bfloat162_rn(acc[nt][2], acc[nt][3]);
    }
}

// 256 threads: warp w works on rows 16 (w & 3) .. +15 and on column half (w >> 2) of every product, so that eight
// warps per SM hide each other's shared-memory and tensor-pipe latencies (the tiles allow one CTA per SM only).
constexpr int NTB = 256;

template <int D>
__global__ void __launch_bounds__(NTB) delta_prep_bwd_kernel(PrepBwdArgs a) {
    constexpr int LD = D + 8, LDC = C + 8, LDA = C + 1, NTH = D / 16, HD = D / 2;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Ks = reinterpret_cast<bf16*>(smem_raw);            // [C][LD]
    bf16* Qs = Ks + C * LD;                                  // [C][LD]
    bf16* Vs = Qs + C * LD;                                  // [C][LD]  V, later beta V
    bf16* Gs = Vs + C * LD;                                  // [C][LD]  dO, later dW
    bf16* Ns = Gs + C * LD;                                  // [C][LD]  Vn
    bf16* Us = Ns + C * LD;                                  // [C][LD]  dVn = dU
    bf16* Sb = Us + C * LD;                                  // [D][LD]  S_n, then dS'_n, then Kb (first C rows)
    bf16* Tb = Sb + D * LD;                                  // [C][LDC] T
    bf16* Ps = Tb + C * LDC;                                 // [C][LDC] P, later M
    bf16* X1 = Ps + C * LDC;                                 // [C][LDC] dT
    bf16* X2 = X1 + C * LDC;                                 // [C][LDC] T^T dT
    float* GK = reinterpret_cast<float*>(X2 + C * LDC);      // [C][LDA] Gamma_ij (k_i.k_j), strictly lower
    float* bcum = GK + C * LDA;                              // [C]
    float* bet = bcum + C;                                   // [C]
    float* db = bet + C;                                     // [C] gradient of the cumulative log decay
    float* dbe = db + C;                                     // [C] gradient of beta
    float* dgam = dbe + C;                                   // [1] <dS'_n, S_n>
    const int n = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const int t0 = n * C;
    const int valid = min(C, a.T - t0);
    const long long cn = (long long)bh * a.N + n;
    const int m0 = 16 * (w & 3), r0 = m0 + (l >> 2), c0 = (l & 3) * 2;
    const bool gated = a.g != nullptr;
    const int nd = (w >> 2) * HD;                            // first column of this warp's half of a D-wide product
    const int nc = (w >> 2) * (C / 2);                       // ... of a C-wide product

    load_tile_async<C, D, LD>(Ks, a.k + b * a.ks_b + h * a.ks_h + (long long)t0 * a.ks_t, a.ks_t, valid);
    load_tile_async<C, D, LD>(Qs, a.q + b * a.qs_b + h * a.qs_h + (long long)t0 * a.qs_t, a.qs_t, valid);
    load_tile_async<C, D, LD>(Vs, a.v + b * a.vs_b + h * a.vs_h + (long long)t0 * a.vs_t, a.vs_t, valid);
    load_tile_async<C, D, LD>(Gs, a.dO + cn * C * D, D, C);
    load_tile_async<C, D, LD>(Ns, a.Vn + cn * C * D, D, C);
    load_tile_async<C, D, LD>(Us, a.dVn + cn * C * D, D, C);
    load_tile_async<D, D, LD>(Sb, a.Sn + cn * D * D, D, D);
    cp_async_commit();
    if (w == 0) {
        const int i0 = 2 * l, i1 = 2 * l + 1;
        float g0 = 0.f, g1 = 0.f, be0 = 0.f, be1 = 0.f;
        if (i0 < valid) { const long long o = ((long long)b * a.T + t0 + i0) * a.H + h; be0 = a.beta[o]; if (a.g != nullptr) g0 = a.g[o]; }
        if (i1 < valid) { const long long o = ((long long)b * a.T + t0 + i1) * a.H + h; be1 = a.beta[o]; if (a.g != nullptr) g1 = a.g[o]; }
        float s = g0 + g1;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const float x = __shfl_up_sync(0xffffffffu, s, o); if (l >= o) s += x; }
        bcum[i1] = s; bcum[i0] = s - g1; bet[i0] = be0; bet[i1] = be1;
        db[i0] = db[i1] = 0.f; dbe[i0] = dbe[i1] = 0.f;
        if (l == 0) dgam[0] = 0.f;
    }
    cp_async_wait<0>();
    __syncthreads();
    const float btot = bcum[C - 1];
    const float b_lo = bcum[r0], b_hi = bcum[r0 + 8], be_lo = bet[r0], be_hi = bet[r0 + 8];

    // ---- (1) K K^T -> GK (fp32), T by substitution (threads 0..63) ---------------------------------------------
    {
        float kk[4][4];
        zero_acc<4>(kk);
        warp_gemm<4, D, false, false>(kk, Ks, LD, m0, Ks, LD, nc);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = r0 + 8 * hh, j = nc + nt * 8 + c0;
                const float bi = hh ? b_hi : b_lo;
                GK[i * LDA + j] = i > j ? __expf(bi - bcum[j]) * kk[nt][2 * hh] : 0.f;
                GK[i * LDA + j + 1] = i > j + 1 ? __expf(bi - bcum[j + 1]) * kk[nt][2 * hh + 1] : 0.f;
            }
    }
    __syncthreads();
    if (threadIdx.x < C) {
        const int c = threadIdx.x;
        float t[C];
#pragma unroll
        for (int i = 0; i < C; ++i) {
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < i; ++j) acc += GK[i * LDA + j] * t[j];
            t[i] = ((i == c) ? 1.f : 0.f) - bet[i] * acc;
        }
#pragma unroll
        for (int i = 0; i < C; ++i) Tb[i * LDC + c] = __float2bfloat16(t[i]);
    }
    // ---- (2) dAqk = tril(dO Vn^T), Q K^T again for Aqk; P = scale Gamma . dAqk; decay gradients of Aqk ---------------
    {
        float da[4][4], qk[4][4];
        zero_acc<4>(da);
        zero_acc<4>(qk);
        warp_gemm<4, D, false, false>(da, Gs, LD, m0, Ns, LD, nc);
        warp_gemm<4, D, false, false>(qk, Qs, LD, m0, Ks, LD, nc);
        float rs_lo = 0.f, rs_hi = 0.f;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            float pv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = r0 + 8 * (e >> 1), j = nc + nt * 8 + c0 + (e & 1);
                const float gam = i >= j ? a.scale * __expf((e >> 1 ? b_hi : b_lo) - bcum[j]) : 0.f;
                pv[e] = gam * da[nt][e];                              // P_ij
                const float t_ = pv[e] * qk[nt][e];                   // dAqk_ij Aqk_ij
                if (e >> 1) rs_hi += t_; else rs_lo += t_;
                if (i >= j) atomicAdd(&db[j], -t_);
            }
            *reinterpret_cast<__nv_bfloat162*>(Ps + r0 * LDC + nc + nt * 8 + c0) = __floats2bfloat162_rn(pv[0], pv[1]);
            *reinterpret_cast<__nv_bfloat162*>(Ps + (r0 + 8) * LDC + nc + nt * 8 + c0) = __floats2bfloat162_rn(pv[2], pv[3]);
        }
        rs_lo += __shfl_xor_sync(0xffffffffu, rs_lo, 1); rs_lo += __shfl_xor_sync(0xffffffffu, rs_lo, 2);
        rs_hi += __shfl_xor_sync(0xffffffffu, rs_hi, 1); rs_hi += __shfl_xor_sync(0xffffffffu, rs_hi, 2);
        if ((l & 3) == 0) { atomicAdd(&db[r0], rs_lo); atomicAdd(&db[r0 + 8], rs_hi); }
    }
    __syncthreads();                                                   // Ps, Tb complete
    // ---- (3) dq = scale e^b (dO S^T) + P K; its decay gradient <dQd_i, Qd_i> ----------------------------------------
    float acc_dk[NTH][4];
    zero_acc<NTH>(acc_dk);
    {
        float acc[NTH][4];
        zero_acc<NTH>(acc);
        warp_gemm<NTH, D, false, false>(acc, Gs, LD, m0, Sb, LD, nd); // dQd = dO S^T  (S stored [dk][dv] = [n][k])
        const float f_lo = a.scale * __expf(b_lo), f_hi = a.scale * __expf(b_hi);
#pragma unroll
        for (int nt = 0; nt < NTH; ++nt) { acc[nt][0] *= f_lo; acc[nt][1] *= f_lo; acc[nt][2] *= f_hi; acc[nt][3] *= f_hi; }
        float d_lo, d_hi;
        row_dot<NTH>(acc, Qs + nd, LD, m0, d_lo, d_hi);               // = <dQd_i, Qd_i> over this warp's columns
        if ((l & 3) == 0) { atomicAdd(&db[r0], d_lo); atomicAdd(&db[r0 + 8], d_hi); }
        warp_gemm<NTH, C, false, true>(acc, Ps, LDC, m0, Ks, LD, nd); // + P K
        store_rows_global<NTH>(acc, a.dq + (((long long)b * a.T + t0) * a.H + h) * D + nd, (long long)a.H * D, m0, valid);
        // dk += P^T Q
        warp_gemm<NTH, C, true, true>(acc_dk, Ps, LDC, m0, Qs, LD, nd);
    }
    // ---- (4) dW = -dVn S^T -> shared (in dO's buffer once every warp is done with dO) --------------------------------
    {
        float acc[NTH][4];
        zero_acc<NTH>(acc);
        warp_gemm<NTH, D, false, false>(acc, Us, LD, m0, Sb, LD, nd);
#pragma unroll
        for (int nt = 0; nt < NTH; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][e] = -acc[nt][e];
        __syncthreads();                                               // all reads of dO (Gs) and S_n (Sb) are done
        store_acc_bf16<NTH>(acc, Gs, LD, m0, nd);                      // Gs now holds dW
    }
    // ---- (5) dS'_n into the state buffer; dgamma = <dS'_n, S_n>; dKd = Vn dS'^T --------------------------------------
    constexpr int SPT = D * D / 8 / NTB;                               // 16-byte pieces of the state per thread
    uint4 keep[SPT];
    if (gated) {
#pragma unroll
        for (int i = 0; i < SPT; ++i) {
            const int idx = threadIdx.x + i * NTB;
            keep[i] = *reinterpret_cast<const uint4*>(Sb + (idx / (D / 8)) * LD + (idx % (D / 8)) * 8);
        }
        __syncthreads();                                               // every thread has its share before the refill
    }
    load_tile_async<D, D, LD>(Sb, a.dSn + cn * D * D, D, D);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    if (gated) {
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < SPT; ++i) {
            const int idx = threadIdx.x + i * NTB;
            const uint4 d = *reinterpret_cast<const uint4*>(Sb + (idx / (D / 8)) * LD + (idx % (D / 8)) * 8);
            const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&keep[i]);
            const __nv_bfloat162* y = reinterpret_cast<const __nv_bfloat162*>(&d);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 fx = __bfloat1622float2(x[e]), fy = __bfloat1622float2(y[e]);
                dot += fx.x * fy.x + fx.y * fy.y;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if (l == 0) atomicAdd(dgam, dot);
    }
    {
        float acc[NTH][4];
        zero_acc<NTH>(acc);
        warp_gemm<NTH, D, false, false>(acc, Ns, LD, m0, Sb, LD, nd); // dKd_j = Vn_j dS'^T
        const float f_lo = __expf(btot - b_lo), f_hi = __expf(btot - b_hi);
#pragma unroll
        for (int nt = 0; nt < NTH; ++nt) { acc[nt][0] *= f_lo; acc[nt][1] *= f_lo; acc[nt][2] *= f_hi; acc[nt][3] *= f_hi; }
        float d_lo, d_hi;
        row_dot<NTH>(acc, Ks + nd, LD, m0, d_lo, d_hi);               // <dKd_j, Kd_j>
        if ((l & 3) == 0) {
            atomicAdd(&db[r0], -d_lo); atomicAdd(&db[r0 + 8], -d_hi);
            atomicAdd(&db[C - 1], d_lo + d_hi);
        }
#pragma unroll
        for (int nt = 0; nt < NTH; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc_dk[nt][e] += acc[nt][e];
    }
    __syncthreads();                                                   // dS'_n no longer needed: Sb becomes Kb
    // ---- (6) dVb = T^T dU: dv, dbeta; then Kb = beta e^b K and Vb = beta V in shared -------------------------------
    {
        float acc[NTH][4];
        zero_acc<NTH>(acc);
        warp_gemm<NTH, C, true, true>(acc, Tb, LDC, m0, Us, LD, nd);
        float d_lo, d_hi;
        row_dot<NTH>(acc, Vs + nd, LD, m0, d_lo, d_hi);               // <dVb_i, v_i>
        if ((l & 3) == 0) { atomicAdd(&dbe[r0], d_lo); atomicAdd(&dbe[r0 + 8], d_hi); }
#pragma unroll
        for (int nt = 0; nt < NTH; ++nt) { acc[nt][0] *= be_lo; acc[nt][1] *= be_lo; acc[nt][2] *= be_hi; acc[nt][3] *= be_hi; }
        store_rows_global<NTH>(acc, a.dv + (((long long)b * a.T + t0) * a.H + h) * D + nd, (long long)a.H * D, m0, valid);
    }
    __syncthreads();                                                   // every warp has read raw V
    for (int i = threadIdx.x; i < C * (D / 8); i += NTB) {
        const int r = i / (D / 8), c = (i % (D / 8)) * 8;
        const float be = bet[r], fk = be * __expf(bcum[r]);
        Vec<bf16> kx, vx, o1, o2;
        kx.load(Ks + r * LD + c);
        vx.load(Vs + r * LD + c);
#pragma unroll
        for (int e = 0; e < 8; ++e) { o1.set(e, kx.get(e) * fk); o2.set(e, vx.get(e) * be); }
        o1.store(Sb + r * LD + c);                                     // Kb
        o2.store(Vs + r * LD + c);                                     // Vb
    }
    __syncthreads();
    // ---- (7) dKb = T^T dW: its part of dk, dbeta and db -------------------------------------------------------------
    {
        float acc[NTH][4];
        zero_acc<NTH>(acc);
        warp_gemm<NTH, C, true, true>(acc, Tb, LDC, m0, Gs, LD, nd);
        float d_lo, d_hi;
        row_dot<NTH>(acc, Ks + nd, LD, m0, d_lo, d_hi);               // <dKb_i, k_i>
        const float e_lo = __expf(b_lo), e_hi = __expf(b_hi);
        if ((l & 3) == 0) {
            atomicAdd(&dbe[r0], e_lo * d_lo); atomicAdd(&dbe[r0 + 8], e_hi * d_hi);
            atomicAdd(&db[r0], be_lo * e_lo * d_lo); atomicAdd(&db[r0 + 8], be_hi * e_hi * d_hi);
        }
#pragma unroll
        for (int nt = 0; nt < NTH; ++nt) {
            acc_dk[nt][0] += be_lo * e_lo * acc[nt][0]; acc_dk[nt][1] += be_lo * e_lo * acc[nt][1];
            acc_dk[nt][2] += be_hi * e_hi * acc[nt][2]; acc_dk[nt][3] += be_hi * e_hi * acc[nt][3];
        }
    }
    // ---- (8) dT = dW Kb^T + dU Vb^T -> X1;  X2 = T^T dT;  dA = -(X2 T^T), strictly lower ------------------------------
    {
        float acc[4][4];
        zero_acc<4>(acc);
        warp_gemm<4, D, false, false>(acc, Gs, LD, m0, Sb, LD, nc);
        warp_gemm<4, D, false, false>(acc, Us, LD, m0, Vs, LD, nc);
        store_acc_bf16<4>(acc, X1, LDC, m0, nc);
    }
    __syncthreads();
    {
        float acc[4][4];
        zero_acc<4>(acc);
        warp_gemm<4, C, true, true>(acc, Tb, LDC, m0, X1, LDC, nc);
        store_acc_bf16<4>(acc, X2, LDC, m0, nc);
    }
    __syncthreads();
    {
        float acc[4][4];
        zero_acc<4>(acc);
        warp_gemm<4, C, false, false>(acc, X2, LDC, m0, Tb, LDC, nc); // (X2 T^T)_ij = sum_k X2_ik T_jk
        float rb_lo = 0.f, rb_hi = 0.f, rd_lo = 0.f, rd_hi = 0.f;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            float mv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int i = r0 + 8 * (e >> 1), j = nc + nt * 8 + c0 + (e & 1);
                const float dA = i > j ? -acc[nt][e] : 0.f;
                const float gk = GK[i * LDA + j];                      // Gamma_ij (k_i.k_j), zero on and above the diagonal
                const float be = (e >> 1) ? be_hi : be_lo;
                const float t1 = dA * gk;                              // -> dbeta_i
                const float t2 = t1 * be;                              // dA_ij A_ij -> db_i, -db_j
                if (e >> 1) { rb_hi += t1; rd_hi += t2; } else { rb_lo += t1; rd_lo += t2; }
                if (i > j) atomicAdd(&db[j], -t2);
                mv[e] = i > j ? dA * be * __expf(((e >> 1) ? b_hi : b_lo) - bcum[j]) : 0.f;      // M_ij
            }
            *reinterpret_cast<__nv_bfloat162*>(Ps + r0 * LDC + nc + nt * 8 + c0) = __floats2bfloat162_rn(mv[0], mv[1]);
            *reinterpret_cast<__nv_bfloat162*>(Ps + (r0 + 8) * LDC + nc + nt * 8 + c0) = __floats2bfloat162_rn(mv[2], mv[3]);
        }
#pragma unroll
        for (int o = 1; o <= 2; o <<= 1) {
            rb_lo += __shfl_xor_sync(0xffffffffu, rb_lo, o); rb_hi += __shfl_xor_sync(0xffffffffu, rb_hi, o);
            rd_lo += __shfl_xor_sync(0xffffffffu, rd_lo, o); rd_hi += __shfl_xor_sync(0xffffffffu, rd_hi, o);
        }
        if ((l & 3) == 0) {
            atomicAdd(&dbe[r0], rb_lo); atomicAdd(&dbe[r0 + 8], rb_hi);
            atomicAdd(&db[r0], rd_lo); atomicAdd(&db[r0 + 8], rd_hi);
        }
    }
    __syncthreads();                                                   // Ps holds M
    // ---- (9) dk += M K + M^T K; store ---------------------------------------------------------------------------------
    warp_gemm<NTH, C, false, true>(acc_dk, Ps, LDC, m0, Ks, LD, nd);
    warp_gemm<NTH, C, true, true>(acc_dk, Ps, LDC, m0, Ks, LD, nd);
    store_rows_global<NTH>(acc_dk, a.dk + (((long long)b * a.T + t0) * a.H + h) * D + nd, (long long)a.H * D, m0, valid);
    __syncthreads();                                                   // all contributions to db / dbeta are in
    // ---- (10) dbeta; dg_s = sum_{i >= s} db_i (+ dgamma gamma on the last position) -----------------------------------
    if (w == 0) {
        const int i0 = 2 * l, i1 = 2 * l + 1;
        float x0 = db[i0], x1 = db[i1];
        if (gated && l == 31) x1 += dgam[0] * __expf(btot);             // gamma = e^{b_C}: d b_C += dgamma gamma
        float s = x0 + x1;                                             // suffix sums over lane pairs
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) { const float y = __shfl_down_sync(0xffffffffu, s, o); if (l + o < 32) s += y; }
        const long long o0 = ((long long)b * a.T + t0 + i0) * a.H + h, o1 = o0 + a.H;
        if (i0 < valid) { a.dbeta[o0] = dbe[i0]; if (a.dg != nullptr) a.dg[o0] = s; }
        if (i1 < valid) { a.dbeta[o1] = dbe[i1]; if (a.dg != nullptr) a.dg[o1] = s - x0; }
    }
}

template <int D> constexpr size_t prep_bwd_smem() {
    return (size_t)(6 * C * (D + 8) + D * (D + 8) + 4 * C * (C + 8)) * 2 + (size_t)(C * (C + 1) + 4 * C + 4) * 4;
}

template <int D> constexpr size_t prep_smem() {
    return (size_t)(4 * C * (D + 8) + C * (C + 8)) * 2 + (size_t)(C * (C + 1) + 2 * C) * 4;
}

}  // namespace dr
}  // namespace lmoe

using namespace lmoe;

// dir 0: forward, dir 1: backward.  dk in {64, 128}; dv a multiple of 32.  Grid = (dv / 32, B*H).
LMOE_API int lmoe_delta_scan(int dir, int dk, int BH, const dr::Args* ap, cudaStream_t st) {
    const dr::Args a = *ap;
    if (a.dv % dr::DVS || (dk != 64 && dk != 128) || BH <= 0) return -1;
    dim3 grid(a.dv / dr::DVS, BH);
#define LMOE_DR_LAUNCH(KERNEL, DK)                                                                                     \
    do {                                                                                                               \
        cudaError_t e = cudaFuncSetAttribute(KERNEL<DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dr::Cfg<DK>::SMEM); \
        if (e != cudaSuccess) return (int)e;                                                                           \
        KERNEL<DK><<<grid, dr::NT, dr::Cfg<DK>::SMEM, st>>>(a);                                                        \
    } while (0)
    if (dir == 0) { if (dk == 128) LMOE_DR_LAUNCH(dr::delta_scan_fwd_kernel, 128); else LMOE_DR_LAUNCH(dr::delta_scan_fwd_kernel, 64); }
    else { if (dk == 128) LMOE_DR_LAUNCH(dr::delta_scan_bwd_kernel, 128); else LMOE_DR_LAUNCH(dr::delta_scan_bwd_kernel, 64); }
#undef LMOE_DR_LAUNCH
    return (int)cudaGetLastError();
}

// Tiles of the chunked (gated) delta rule for every chunk of every (batch, head): grid (N, B*H).  dk = dv = D in {64, 128}.
LMOE_API int lmoe_delta_prepare(int D, const dr::PrepArgs* ap, cudaStream_t st) {
    const dr::PrepArgs a = *ap;
    if (a.N <= 0 || a.B * a.H <= 0) return -1;
    dim3 grid(a.N, a.B * a.H);
    if (D == 128) {
        cudaError_t e = cudaFuncSetAttribute(dr::delta_prep_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dr::prep_smem<128>());
        if (e != cudaSuccess) return (int)e;
        dr::delta_prep_fwd_kernel<128><<<grid, dr::NT, dr::prep_smem<128>(), st>>>(a);
    } else if (D == 64) {
        cudaError_t e = cudaFuncSetAttribute(dr::delta_prep_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dr::prep_smem<64>());
        if (e != cudaSuccess) return (int)e;
        dr::delta_prep_fwd_kernel<64><<<grid, dr::NT, dr::prep_smem<64>(), st>>>(a);
    } else return -2;
    return (int)cudaGetLastError();
}

// Chunk-parallel backward of the tile construction and of the chunk-local scan equations: grid (N, B*H).
LMOE_API int lmoe_delta_prepare_bwd(int D, const dr::PrepBwdArgs* ap, cudaStream_t st) {
    const dr::PrepBwdArgs a = *ap;
    if (a.N <= 0 || a.B * a.H <= 0) return -1;
    dim3 grid(a.N, a.B * a.H);
    if (D == 128) {
        cudaError_t e = cudaFuncSetAttribute(dr::delta_prep_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dr::prep_bwd_smem<128>());
        if (e != cudaSuccess) return (int)e;
        dr::delta_prep_bwd_kernel<128><<<grid, dr::NTB, dr::prep_bwd_smem<128>(), st>>>(a);
    } else if (D == 64) {
        cudaError_t e = cudaFuncSetAttribute(dr::delta_prep_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dr::prep_bwd_smem<64>());
        if (e != cudaSuccess) return (int)e;
        dr::delta_prep_bwd_kernel<64><<<grid, dr::NTB, dr::prep_bwd_smem<64>(), st>>>(a);
    } else return -2;
    return (int)cudaGetLastError();
}
