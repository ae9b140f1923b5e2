// Chunked linear attention with a scalar decay per head (constant: retention / lightning; per token:
// Mamba2-SSD / simple-GLA; none: basic linear attention), forward and backward, bf16 in / fp32 state.
//
//   S_t = e^{g_t} S_{t-1} + k_t^T v_t,   o_t = scale * q_t S_t
//
// Replaces the external Triton kernels the reference calls (fla linear_attn / retention / simple_gla,
// lightning_attn2, mamba_ssm SSD chunk scan: basic_linear_attention.py:133, retention.py:91,
// lightning_attention.py:123, mamba_mixer.py:244-260) and the in-tree LASP-2 Triton kernels
// (lasp2_without_mask_triton_op.py:11-468).
//
// Parallel structure.  A (batch, head) sequence of N chunks of 64 tokens is cut into G groups so that
// B*H*G CTAs fill the 148 SMs in one wave.  Three launches per direction:
//   1. state_scan:  each CTA scans its group's chunks from a zero state and writes the group summary
//                   M_g (fp32 D x D) and the group's total log decay.
//   2. combine:     per (b, h): exclusive scan over the G summaries, seeded with the initial state (or,
//                   under LASP-2, with the prefix folded from the other ranks' summaries); in place.
//   3. output:      each CTA re-scans its group with the correct entering state and emits outputs.
// No per-chunk state is ever written to HBM (the 5-kernel pipelines this replaces materialise all N).
// The same three-step structure run over (rank, group) pairs IS the LASP-2 schedule, which is why the
// multi-GPU exchange slots into step 2 (see lasp_comm.cu).
//
// Per chunk (C = 64, b_i = inclusive in-chunk cumulative log decay):
//   A   = (Q K^T) .* [i >= j] e^{b_i - b_j} * scale          (64 x 64)
//   O   = A V + scale * e^{b_i} (Q S)                          (64 x D)
//   S  <- e^{b_C} S + (K .* e^{b_C - b_j})^T V                 (D x D)
// Tensor-core work uses mma.sync m16n8k16 on ldmatrix fragments; the fp32 state lives in registers
// across the whole group, with a bf16 copy in shared memory as the B operand of Q S.
#include "mma_utils.cuh"

namespace lmoe {

constexpr int CH = 64;             // chunk length
constexpr int NTHREADS = 256;

struct LsmArgs {
    const bf16 *q, *k, *v, *d_o;   // d_o: contiguous [B,T,H,D] (backward only)
    int64_t qs_b, qs_t, qs_h, ks_b, ks_t, ks_h, vs_b, vs_t, vs_h;
    bf16 *o, *dq, *dk, *dv;        // outputs (o contiguous; dq/dk/dv with the strides below)
    int64_t dqs_b, dqs_t, dqs_h, dks_b, dks_t, dks_h, dvs_b, dvs_t, dvs_h;
    const float* g;                // gmode 1: [H]; gmode 2: [B,T,H]
    int gmode;
    float scale;
    int B, T, H, G, cpg;           // G groups of cpg chunks
    float* states;                 // [B,H,G,D,D]
    float* gdecay;                 // [B,H,G] total log decay per group (gmode 2)
};

template <int D> struct Cfg {
    static constexpr int LD = D + 8;               // padded row stride of D-wide tiles
    static constexpr int PLD = CH + 8;             // padded row stride of the 64x64 score tile
    static constexpr int S_RB = D / 16;            // row blocks of the state
    static constexpr int S_NT = D * D / 1024;      // n-tiles of the state per warp
    static constexpr int O_NT = D / 16;            // n-tiles of a 64 x D output per warp
};

// In-chunk decay tables for chunk `c` of (b, h), written by warp 0.
//   lb[i]   = b_i                      (fp32)
//   ktab[j] = e^{b_C - b_j}            (bf16, pairs)      key-side scale of the state update
//   qtab[i] = e^{b_i} * scale          (bf16, pairs)      query-side scale of the reverse state update
//   misc[0] = e^{b_C}, misc[1] = b_C
__device__ __forceinline__ void build_tables(const LsmArgs& a, int b, int h, int c, float* lb, bf16* ktab, bf16* qtab,
                                             float* misc) {
    if (threadIdx.x >= 32) return;
    const int l = threadIdx.x;
    const int t0 = c * CH + 2 * l;
    float g0 = 0.f, g1 = 0.f;
    if (a.gmode == 1) {
        float gh = a.g[h];
        g0 = t0 < a.T ? gh : 0.f;
        g1 = t0 + 1 < a.T ? gh : 0.f;
    } else if (a.gmode == 2) {
        if (t0 < a.T) g0 = a.g[((int64_t)b * a.T + t0) * a.H + h];
        if (t0 + 1 < a.T) g1 = a.g[((int64_t)b * a.T + t0 + 1) * a.H + h];
    }
    float s = g0 + g1;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        float n = __shfl_up_sync(0xffffffffu, s, o);
        if (l >= o) s += n;
    }
    float tot = __shfl_sync(0xffffffffu, s, 31);
    float b1 = s, b0 = s - g1;
    lb[2 * l] = b0;
    lb[2 * l + 1] = b1;
    ktab[2 * l] = __float2bfloat16(__expf(tot - b0));
    ktab[2 * l + 1] = __float2bfloat16(__expf(tot - b1));
    qtab[2 * l] = __float2bfloat16(__expf(b0) * a.scale);
    qtab[2 * l + 1] = __float2bfloat16(__expf(b1) * a.scale);
    if (l == 0) { misc[0] = __expf(tot); misc[1] = tot; }
}

// ---------------------------------------------------------------------------------------------
// 1. state_scan: acc <- gamma * acc + (X .* tab)^T Y over the chunks of one group.
//    forward (REV=0): X = K (ktab), Y = V, ascending chunks.  backward (REV=1): X = Q (qtab), Y = dO, descending.
// ---------------------------------------------------------------------------------------------
template <int D, int REV>
__global__ void __launch_bounds__(NTHREADS) state_scan_kernel(LsmArgs a) {
    using C = Cfg<D>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Xs = reinterpret_cast<bf16*>(smem_raw);                 // [2][CH][LD]
    bf16* Ys = Xs + 2 * CH * C::LD;                               // [2][CH][LD]
    float* lb = reinterpret_cast<float*>(Ys + 2 * CH * C::LD);    // [CH]
    float* misc = lb + CH;                                        // [4]
    bf16* ktab = reinterpret_cast<bf16*>(misc + 4);               // [CH]
    bf16* qtab = ktab + CH;                                       // [CH]

    const int grp = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int nchunks = (a.T + CH - 1) / CH;
    const int c_lo = grp * a.cpg, c_hi = min(nchunks, c_lo + a.cpg);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const int s_m0 = 16 * (w % C::S_RB), s_n0 = (w / C::S_RB) * (C::S_NT * 8);

    const bf16* xg = REV ? a.q + b * a.qs_b + h * a.qs_h : a.k + b * a.ks_b + h * a.ks_h;
    const int64_t xs_t = REV ? a.qs_t : a.ks_t;
    const bf16* yg = REV ? a.d_o + ((int64_t)b * a.T * a.H + h) * D : a.v + b * a.vs_b + h * a.vs_h;
    const int64_t ys_t = REV ? (int64_t)a.H * D : a.vs_t;

    float acc[C::S_NT][4];
    zero_acc<C::S_NT>(acc);
    float gsum = 0.f;
    const int n = c_hi - c_lo;
    auto chunk_at = [&](int i) { return REV ? c_hi - 1 - i : c_lo + i; };
    if (n > 0) {
        int c = chunk_at(0);
        load_tile_async<CH, D, C::LD>(Xs, xg + (int64_t)c * CH * xs_t, xs_t, a.T - c * CH);
        load_tile_async<CH, D, C::LD>(Ys, yg + (int64_t)c * CH * ys_t, ys_t, a.T - c * CH);
    }
    cp_async_commit();
    for (int i = 0; i < n; ++i) {
        const int c = chunk_at(i), buf = i & 1;
        if (i + 1 < n) {
            int cn = chunk_at(i + 1);
            load_tile_async<CH, D, C::LD>(Xs + (buf ^ 1) * CH * C::LD, xg + (int64_t)cn * CH * xs_t, xs_t, a.T - cn * CH);
            load_tile_async<CH, D, C::LD>(Ys + (buf ^ 1) * CH * C::LD, yg + (int64_t)cn * CH * ys_t, ys_t, a.T - cn * CH);
        }
        cp_async_commit();
        build_tables(a, b, h, c, lb, ktab, qtab, misc);
        cp_async_wait<1>();
        __syncthreads();
        const float gamma = misc[0];
        gsum += misc[1];
#pragma unroll
        for (int nt = 0; nt < C::S_NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][e] *= gamma;
        warp_gemm_at_kscaled<C::S_NT, CH, true>(acc, Xs + buf * CH * C::LD, C::LD, s_m0, Ys + buf * CH * C::LD, C::LD, s_n0,
                                                reinterpret_cast<const __nv_bfloat162*>(REV ? qtab : ktab));
        __syncthreads();
    }
    float* out = a.states + ((int64_t)bh * a.G + grp) * D * D;
    const int r = s_m0 + (l >> 2), cc = s_n0 + (l & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < C::S_NT; ++nt) {
        *reinterpret_cast<float2*>(out + (int64_t)r * D + cc + nt * 8) = make_float2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<float2*>(out + (int64_t)(r + 8) * D + cc + nt * 8) = make_float2(acc[nt][2], acc[nt][3]);
    }
    if (threadIdx.x == 0 && a.gdecay != nullptr) a.gdecay[(int64_t)bh * a.G + grp] = gsum;
}

// ---------------------------------------------------------------------------------------------
// 2. combine: exclusive scan of the group summaries, in place.  forward: slot g <- state entering group g,
//    `final` <- state after the last group.  reverse: slot g <- state gradient leaving group g (entering from the
//    right), `final` <- gradient wrt the initial state.  `seed` = initial state / final-state gradient (nullable).
// ---------------------------------------------------------------------------------------------
template <int REV>
__global__ void combine_kernel(float* __restrict__ states, const float* __restrict__ gdecay, const float* __restrict__ gconst,
                               const float* __restrict__ seed, float* __restrict__ final_out, int H, int G, int cpg, int T,
                               int DD) {
    const int bh = blockIdx.y, h = bh % H;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= DD) return;
    float carry = seed != nullptr ? seed[(int64_t)bh * DD + e] : 0.f;
    // the summaries of a batch of groups are loaded before any of them is overwritten, so that the loads of a thread are
    // in flight together (one dependent load per group would leave the kernel bound by memory latency)
    constexpr int NB = 8;
    for (int i0 = 0; i0 < G; i0 += NB) {
        float m[NB], dec[NB];
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int i = i0 + j;
            if (i < G) {
                const int g = REV ? G - 1 - i : i;
                m[j] = __ldcg(states + ((int64_t)bh * G + g) * DD + e);
                float a;
                if (gdecay != nullptr) a = gdecay[(int64_t)bh * G + g];
                else if (gconst != nullptr) {
                    int t_lo = g * cpg * CH, t_hi = min(T, (g + 1) * cpg * CH);
                    a = gconst[h] * (float)max(t_hi - t_lo, 0);
                } else a = 0.f;
                dec[j] = __expf(a);
            }
        }
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int i = i0 + j;
            if (i < G) {
                const int g = REV ? G - 1 - i : i;
                states[((int64_t)bh * G + g) * DD + e] = carry;
                carry = dec[j] * carry + m[j];
            }
        }
    }
    if (final_out != nullptr) final_out[(int64_t)bh * DD + e] = carry;
}

// Copy a staged [CH x D] bf16 tile from shared memory to global rows with stride `row_stride`.
template <int D, int LD>
__device__ __forceinline__ void store_tile(const bf16* smem, bf16* gmem, int64_t row_stride, int valid_rows) {
    constexpr int VPR = D / 8;
    for (int i = threadIdx.x; i < CH * VPR; i += blockDim.x) {
        int r = i / VPR, c = (i % VPR) * 8;
        if (r < valid_rows)
            *reinterpret_cast<uint4*>(gmem + (int64_t)r * row_stride + c) = *reinterpret_cast<const uint4*>(smem + r * LD + c);
    }
}

// Load the fp32 entering state of this CTA's group into accumulator registers and its bf16 copy into smem.
template <int D>
__device__ __forceinline__ void load_state(const float* src, float (&acc)[Cfg<D>::S_NT][4], bf16* Sb, int s_m0, int s_n0) {
    using C = Cfg<D>;
    const int l = threadIdx.x & 31;
    const int r = s_m0 + (l >> 2), cc = s_n0 + (l & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < C::S_NT; ++nt) {
        float2 x = *reinterpret_cast<const float2*>(src + (int64_t)r * D + cc + nt * 8);
        float2 y = *reinterpret_cast<const float2*>(src + (int64_t)(r + 8) * D + cc + nt * 8);
        acc[nt][0] = x.x; acc[nt][1] = x.y; acc[nt][2] = y.x; acc[nt][3] = y.y;
    }
    store_acc_bf16<C::S_NT>(acc, Sb, C::LD, s_m0, s_n0);
}

// Mask + decay a 16 x 32 score fragment and write it as bf16 into the P tile.
//   LOWER=1: keep i >= j with factor e^{lb[i]-lb[j]} (rows are queries i, cols keys j)
//   LOWER=0: keep j <= i where rows are keys j and cols are queries i: factor e^{lb[col]-lb[row]}
template <int LOWER>
__device__ __forceinline__ void mask_store(const float (&acc)[4][4], bf16* P, int pld, int m0, int n0, const float* lb,
                                           float scale) {
    const int l = threadIdx.x & 31;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            int r = m0 + (l >> 2) + 8 * hh;
            int c = n0 + nt * 8 + (l & 3) * 2;
            float v0, v1;
            if (LOWER) {
                v0 = r >= c ? acc[nt][2 * hh] * __expf(lb[r] - lb[c]) * scale : 0.f;
                v1 = r >= c + 1 ? acc[nt][2 * hh + 1] * __expf(lb[r] - lb[c + 1]) * scale : 0.f;
            } else {
                v0 = r <= c ? acc[nt][2 * hh] * __expf(lb[c] - lb[r]) * scale : 0.f;
                v1 = r <= c + 1 ? acc[nt][2 * hh + 1] * __expf(lb[c + 1] - lb[r]) * scale : 0.f;
            }
            *reinterpret_cast<__nv_bfloat162*>(P + r * pld + c) = __floats2bfloat162_rn(v0, v1);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// 3a. forward output (MODE 0) and backward dq (MODE 1): both sweep forward carrying S.
//   MODE 0: tiles X0=Q, X1=K, X2=V; out = scale*[(Q K^T . D) V + e^{b} (Q S)]
//   MODE 1: tiles X0=dO, X1=V(as keys), X2=K(as values); out = dQ = scale*[(dO V^T . D) K + e^{b} (dO S^T)];
//           the state update still uses K, V.
// ---------------------------------------------------------------------------------------------
template <int D, int MODE>
__global__ void __launch_bounds__(NTHREADS) fwd_sweep_kernel(LsmArgs a) {
    using C = Cfg<D>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* T0 = reinterpret_cast<bf16*>(smem_raw);                 // [2][CH][LD]  Q | dO
    bf16* T1 = T0 + 2 * CH * C::LD;                               // [2][CH][LD]  K | V
    bf16* T2 = T1 + 2 * CH * C::LD;                               // [2][CH][LD]  V | K
    bf16* Sb = T2 + 2 * CH * C::LD;                               // [D][LD] bf16 copy of the state
    bf16* P = Sb + D * C::LD;                                     // [CH][PLD]
    float* lb = reinterpret_cast<float*>(P + CH * C::PLD);        // [CH]
    float* misc = lb + CH;
    bf16* ktab = reinterpret_cast<bf16*>(misc + 4);
    bf16* qtab = ktab + CH;

    const int grp = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int nchunks = (a.T + CH - 1) / CH;
    const int c_lo = grp * a.cpg, c_hi = min(nchunks, c_lo + a.cpg);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const int s_m0 = 16 * (w % C::S_RB), s_n0 = (w / C::S_RB) * (C::S_NT * 8);
    const int o_m0 = 16 * (w & 3), o_n0 = (w >> 2) * (D / 2);
    const int a_m0 = 16 * (w & 3), a_n0 = (w >> 2) * 32;

    const bf16* g0; int64_t st0; const bf16* g1; int64_t st1; const bf16* g2; int64_t st2;
    if (MODE == 0) {
        g0 = a.q + b * a.qs_b + h * a.qs_h; st0 = a.qs_t;
        g1 = a.k + b * a.ks_b + h * a.ks_h; st1 = a.ks_t;
        g2 = a.v + b * a.vs_b + h * a.vs_h; st2 = a.vs_t;
    } else {
        g0 = a.d_o + ((int64_t)b * a.T * a.H + h) * D; st0 = (int64_t)a.H * D;
        g1 = a.v + b * a.vs_b + h * a.vs_h; st1 = a.vs_t;
        g2 = a.k + b * a.ks_b + h * a.ks_h; st2 = a.ks_t;
    }
    bf16* og; int64_t ost;
    if (MODE == 0) { og = a.o + ((int64_t)b * a.T * a.H + h) * D; ost = (int64_t)a.H * D; }
    else { og = a.dq + b * a.dqs_b + h * a.dqs_h; ost = a.dqs_t; }

    float acc_s[C::S_NT][4];
    load_state<D>(a.states + ((int64_t)bh * a.G + grp) * D * D, acc_s, Sb, s_m0, s_n0);

    auto issue = [&](int c, int buf) {
        int valid = a.T - c * CH;
        load_tile_async<CH, D, C::LD>(T0 + buf * CH * C::LD, g0 + (int64_t)c * CH * st0, st0, valid);
        load_tile_async<CH, D, C::LD>(T1 + buf * CH * C::LD, g1 + (int64_t)c * CH * st1, st1, valid);
        load_tile_async<CH, D, C::LD>(T2 + buf * CH * C::LD, g2 + (int64_t)c * CH * st2, st2, valid);
    };
    if (c_lo < c_hi) issue(c_lo, 0);
    cp_async_commit();
    for (int c = c_lo; c < c_hi; ++c) {
        const int buf = (c - c_lo) & 1;
        if (c + 1 < c_hi) issue(c + 1, buf ^ 1);
        cp_async_commit();
        build_tables(a, b, h, c, lb, ktab, qtab, misc);
        cp_async_wait<1>();
        __syncthreads();                                            // tiles, tables and Sb of this chunk visible
        const bf16* X0 = T0 + buf * CH * C::LD;
        const bf16* X1 = T1 + buf * CH * C::LD;
        const bf16* X2 = T2 + buf * CH * C::LD;
        float acc_o[C::O_NT][4], acc_a[4][4];
        zero_acc<C::O_NT>(acc_o);
        zero_acc<4>(acc_a);
        // inter-chunk term X0 * S (MODE 0) or X0 * S^T (MODE 1), and the scores X0 * X1^T
        if (MODE == 0) warp_gemm<C::O_NT, D, false, true>(acc_o, X0, C::LD, o_m0, Sb, C::LD, o_n0);
        else warp_gemm<C::O_NT, D, false, false>(acc_o, X0, C::LD, o_m0, Sb, C::LD, o_n0);
        warp_gemm<4, D, false, false>(acc_a, X0, C::LD, a_m0, X1, C::LD, a_n0);
        {
            const float f0 = __expf(lb[o_m0 + (l >> 2)]) * a.scale, f1 = __expf(lb[o_m0 + (l >> 2) + 8]) * a.scale;
#pragma unroll
            for (int nt = 0; nt < C::O_NT; ++nt) { acc_o[nt][0] *= f0; acc_o[nt][1] *= f0; acc_o[nt][2] *= f1; acc_o[nt][3] *= f1; }
        }
        mask_store<1>(acc_a, P, C::PLD, a_m0, a_n0, lb, a.scale);
        __syncthreads();                                            // P complete; everyone is done reading X0 and Sb
        warp_gemm<C::O_NT, CH, false, true>(acc_o, P, C::PLD, o_m0, X2, C::LD, o_n0);
        // state update with K, V
        const float gamma = misc[0];
#pragma unroll
        for (int nt = 0; nt < C::S_NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc_s[nt][e] *= gamma;
        warp_gemm_at_kscaled<C::S_NT, CH, true>(acc_s, MODE == 0 ? X1 : X2, C::LD, s_m0, MODE == 0 ? X2 : X1, C::LD, s_n0,
                                                reinterpret_cast<const __nv_bfloat162*>(ktab));
        // stage the output tile in X0's buffer, refresh the bf16 state copy
        bf16* stage = T0 + buf * CH * C::LD;
        store_acc_bf16<C::O_NT>(acc_o, stage, C::LD, o_m0, o_n0);
        __syncthreads();                                            // all state-update reads of Sb's consumers done? (Sb is
                                                                    // only read in the first phase) -> safe to overwrite
        store_acc_bf16<C::S_NT>(acc_s, Sb, C::LD, s_m0, s_n0);
        store_tile<D, C::LD>(stage, og + (int64_t)c * CH * ost, ost, a.T - c * CH);
        __syncthreads();                                            // stage drained before the next prefetch overwrites it
    }
}

// ---------------------------------------------------------------------------------------------
// 3b. backward dk, dv: reverse sweep carrying dS (gradient of the state leaving the chunk).
//   Abar[j,i] = scale (K_j.Q_i) e^{b_i-b_j} [j<=i];  Bbar[j,i] = scale (V_j.dO_i) e^{b_i-b_j} [j<=i]
//   dV = Abar dO + e^{b_C-b_j} (K dS);   dK = Bbar Q + e^{b_C-b_j} (V dS^T);   dS <- e^{b_C} dS + (Q e^{b} scale)^T dO
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(NTHREADS) bwd_dkv_kernel(LsmArgs a) {
    using C = Cfg<D>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Tq = reinterpret_cast<bf16*>(smem_raw);                 // [2][CH][LD]
    bf16* Tk = Tq + 2 * CH * C::LD;
    bf16* Tv = Tk + 2 * CH * C::LD;
    bf16* Tg = Tv + 2 * CH * C::LD;                               // dO
    bf16* Sb = Tg + 2 * CH * C::LD;                               // [D][LD] bf16 copy of dS
    bf16* P1 = Sb + D * C::LD;                                    // [CH][PLD]
    bf16* P2 = P1 + CH * C::PLD;
    float* lb = reinterpret_cast<float*>(P2 + CH * C::PLD);
    float* misc = lb + CH;
    bf16* ktab = reinterpret_cast<bf16*>(misc + 4);
    bf16* qtab = ktab + CH;

    const int grp = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
    const int nchunks = (a.T + CH - 1) / CH;
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
    load_state<D>(a.states + ((int64_t)bh * a.G + grp) * D * D, acc_s, Sb, s_m0, s_n0);

    auto issue = [&](int c, int buf) {
        int valid = a.T - c * CH;
        load_tile_async<CH, D, C::LD>(Tq + buf * CH * C::LD, qg + (int64_t)c * CH * a.qs_t, a.qs_t, valid);
        load_tile_async<CH, D, C::LD>(Tk + buf * CH * C::LD, kg + (int64_t)c * CH * a.ks_t, a.ks_t, valid);
        load_tile_async<CH, D, C::LD>(Tv + buf * CH * C::LD, vg + (int64_t)c * CH * a.vs_t, a.vs_t, valid);
        load_tile_async<CH, D, C::LD>(Tg + buf * CH * C::LD, gg + (int64_t)c * CH * gst, gst, valid);
    };
    if (c_lo < c_hi) issue(c_hi - 1, 0);
    cp_async_commit();
    for (int c = c_hi - 1; c >= c_lo; --c) {
        const int buf = (c_hi - 1 - c) & 1;
        if (c - 1 >= c_lo) issue(c - 1, buf ^ 1);
        cp_async_commit();
        build_tables(a, b, h, c, lb, ktab, qtab, misc);
        cp_async_wait<1>();
        __syncthreads();
        bf16* Q = Tq + buf * CH * C::LD;
        bf16* K = Tk + buf * CH * C::LD;
        bf16* V = Tv + buf * CH * C::LD;
        bf16* G = Tg + buf * CH * C::LD;
        float acc_dv[C::O_NT][4], acc_dk[C::O_NT][4], acc_a[4][4], acc_b[4][4];
        zero_acc<C::O_NT>(acc_dv);
        zero_acc<C::O_NT>(acc_dk);
        zero_acc<4>(acc_a);
        zero_acc<4>(acc_b);
        warp_gemm<4, D, false, false>(acc_a, K, C::LD, a_m0, Q, C::LD, a_n0);           // K Q^T
        warp_gemm<4, D, false, false>(acc_b, V, C::LD, a_m0, G, C::LD, a_n0);           // V dO^T
        warp_gemm<C::O_NT, D, false, true>(acc_dv, K, C::LD, o_m0, Sb, C::LD, o_n0);    // K dS
        warp_gemm<C::O_NT, D, false, false>(acc_dk, V, C::LD, o_m0, Sb, C::LD, o_n0);   // V dS^T
        {
            const float tot = misc[1];
            const float f0 = __expf(tot - lb[o_m0 + (l >> 2)]), f1 = __expf(tot - lb[o_m0 + (l >> 2) + 8]);
#pragma unroll
            for (int nt = 0; nt < C::O_NT; ++nt) {
                acc_dv[nt][0] *= f0; acc_dv[nt][1] *= f0; acc_dv[nt][2] *= f1; acc_dv[nt][3] *= f1;
                acc_dk[nt][0] *= f0; acc_dk[nt][1] *= f0; acc_dk[nt][2] *= f1; acc_dk[nt][3] *= f1;
            }
        }
        mask_store<0>(acc_a, P1, C::PLD, a_m0, a_n0, lb, a.scale);
        mask_store<0>(acc_b, P2, C::PLD, a_m0, a_n0, lb, a.scale);
        __syncthreads();
        warp_gemm<C::O_NT, CH, false, true>(acc_dv, P1, C::PLD, o_m0, G, C::LD, o_n0);  // Abar dO
        warp_gemm<C::O_NT, CH, false, true>(acc_dk, P2, C::PLD, o_m0, Q, C::LD, o_n0);  // Bbar Q
        const float gamma = misc[0];
#pragma unroll
        for (int nt = 0; nt < C::S_NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc_s[nt][e] *= gamma;
        warp_gemm_at_kscaled<C::S_NT, CH, true>(acc_s, Q, C::LD, s_m0, G, C::LD, s_n0,
                                                reinterpret_cast<const __nv_bfloat162*>(qtab));
        __syncthreads();                                            // all reads of K, V, Q, dO, Sb done
        store_acc_bf16<C::O_NT>(acc_dv, V, C::LD, o_m0, o_n0);      // stage dV in V's buffer, dK in K's
        store_acc_bf16<C::O_NT>(acc_dk, K, C::LD, o_m0, o_n0);
        store_acc_bf16<C::S_NT>(acc_s, Sb, C::LD, s_m0, s_n0);
        __syncthreads();
        store_tile<D, C::LD>(V, dvg + (int64_t)c * CH * a.dvs_t, a.dvs_t, a.T - c * CH);
        store_tile<D, C::LD>(K, dkg + (int64_t)c * CH * a.dks_t, a.dks_t, a.T - c * CH);
        __syncthreads();
    }
}

template <int D> constexpr size_t smem_scan() { return (size_t)4 * CH * Cfg<D>::LD * 2 + CH * 4 + 16 + CH * 4; }
template <int D> constexpr size_t smem_sweep() {
    return (size_t)6 * CH * Cfg<D>::LD * 2 + (size_t)D * Cfg<D>::LD * 2 + (size_t)CH * Cfg<D>::PLD * 2 + CH * 4 + 16 + CH * 4;
}
template <int D> constexpr size_t smem_dkv() {
    return (size_t)8 * CH * Cfg<D>::LD * 2 + (size_t)D * Cfg<D>::LD * 2 + (size_t)2 * CH * Cfg<D>::PLD * 2 + CH * 4 + 16 + CH * 4;
}

template <typename K> static int set_smem(K kernel, size_t bytes) {
    return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace lmoe

using namespace lmoe;

// which: 0 = forward state scan (K,V), 1 = reverse state scan (Q,dO), 2 = forward output, 3 = backward dq,
//        4 = backward dk/dv.  Launch grid is (G, B*H).
LMOE_API int lmoe_lsm_scalar_launch(int which, int D, const LsmArgs* ap, cudaStream_t st) {
    const LsmArgs a = *ap;
    dim3 grid(a.G, a.B * a.H);
    int rc = 0;
#define LAUNCH(KERNEL, SMEM)                                   \
    do {                                                       \
        rc = set_smem(KERNEL, SMEM);                           \
        if (rc) return rc;                                     \
        KERNEL<<<grid, NTHREADS, SMEM, st>>>(a);               \
    } while (0)
    if (D == 128) {
        if (which == 0) LAUNCH((state_scan_kernel<128, 0>), smem_scan<128>());
        else if (which == 1) LAUNCH((state_scan_kernel<128, 1>), smem_scan<128>());
        else if (which == 2) LAUNCH((fwd_sweep_kernel<128, 0>), smem_sweep<128>());
        else if (which == 3) LAUNCH((fwd_sweep_kernel<128, 1>), smem_sweep<128>());
        else if (which == 4) LAUNCH((bwd_dkv_kernel<128>), smem_dkv<128>());
        else return -1;
    } else if (D == 64) {
        if (which == 0) LAUNCH((state_scan_kernel<64, 0>), smem_scan<64>());
        else if (which == 1) LAUNCH((state_scan_kernel<64, 1>), smem_scan<64>());
        else if (which == 2) LAUNCH((fwd_sweep_kernel<64, 0>), smem_sweep<64>());
        else if (which == 3) LAUNCH((fwd_sweep_kernel<64, 1>), smem_sweep<64>());
        else if (which == 4) LAUNCH((bwd_dkv_kernel<64>), smem_dkv<64>());
        else return -1;
    } else return -2;
#undef LAUNCH
    return (int)cudaGetLastError();
}

// rev = 0: forward prefix (seed = initial state, final_out = final state); rev = 1: reverse suffix
// (seed = gradient of the final state, final_out = gradient of the initial state).
LMOE_API int lmoe_lsm_scalar_combine(int rev, float* states, const float* gdecay, const float* gconst, const float* seed,
                                     float* final_out, int BH, int H, int G, int cpg, int T, int D, cudaStream_t st) {
    int DD = D * D;
    dim3 grid((DD + 255) / 256, BH);
    if (rev) combine_kernel<1><<<grid, 256, 0, st>>>(states, gdecay, gconst, seed, final_out, H, G, cpg, T, DD);
    else combine_kernel<0><<<grid, 256, 0, st>>>(states, gdecay, gconst, seed, final_out, H, G, cpg, T, DD);
    return (int)cudaGetLastError();
}
