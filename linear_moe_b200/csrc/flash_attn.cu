// Causal softmax attention with grouped-query heads (flash attention), forward and backward, bf16, head dim 64/128.
//
// Replaces the reference's unfused baddbmm -> FusedScaleMaskSoftmax -> bmm core
// (sequence_modeling/attention/dot_product_attention.py:139-183, O(s^2) memory) and its optional flash_attn /
// TransformerEngine back ends (llama3/transformer_legacy.py:446-505, qwen2/layer_specs.py:64-66).
//
// Layout: q [B, Tq, Hq, D], k/v [B, Tk, Hkv, D] (unit stride in D, free token/head strides), o [B, Tq, Hq, D] contiguous.
// `q_offset` is the absolute position of q[0] relative to k[0]: key j is visible to query i iff j <= q_offset + i (and
// j > q_offset + i - window when a sliding window is set).  Sequence-parallel ranks pass their slice of the queries with
// the all-gathered keys (LASP-2H style), decoding passes the cache length.
//
// forward   one CTA = 64 queries of one head, 4 warps x 16 rows; K/V tiles of 64 keys stream through shared memory;
//           S = Q K^T and O += P V on tensor cores (mma.sync m16n8k16, P reused from the S accumulator registers);
//           online softmax in the exp2 domain; writes O and the row log-sum-exp.
// backward  delta = rowsum(dO . O) (small kernel), then one CTA = 64 keys of one KV head: for every query head of the
//           group and every visible query tile it recomputes P^T, accumulates dV += P^T dO and dK += dS^T Q in
//           registers and adds dS K to an fp32 dQ buffer with red.global.add.
#include "mma_utils.cuh"

namespace lmoe {

constexpr int FA_BM = 64, FA_BN = 64, FA_THREADS = 128;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

struct FaArgs {
    const bf16 *q, *k, *v, *o, *d_o;
    int64_t qs_b, qs_t, qs_h, ks_b, ks_t, ks_h, vs_b, vs_t, vs_h;
    bf16* out;                   // forward output [B,Tq,Hq,D]
    float* lse;                  // [B,Hq,Tq] natural-log sum-exp
    float* delta;                // [B,Hq,Tq]
    float* dq_acc;               // [B,Tq,Hq,D] fp32
    bf16 *dk, *dv;               // [B,Tk,Hkv,D] contiguous
    int B, Tq, Tk, Hq, Hkv;
    int q_offset, window;        // window <= 0: none
    float scale;
};

template <int D> struct FaCfg { static constexpr int LD = D + 8; static constexpr int KS = D / 16; static constexpr int O_NT = D / 8; };

__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

template <int D>
__global__ void __launch_bounds__(FA_THREADS) fa_fwd_kernel(FaArgs a) {
    using C = FaCfg<D>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ks = Qs + FA_BM * C::LD;                 // [2][FA_BN][LD]
    bf16* Vs = Ks + 2 * FA_BN * C::LD;             // [2][FA_BN][LD]
    const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (a.Hq / a.Hkv);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const int q0 = qb * FA_BM;
    const bf16* qg = a.q + b * a.qs_b + h * a.qs_h + (int64_t)q0 * a.qs_t;
    const bf16* kg = a.k + b * a.ks_b + hk * a.ks_h;
    const bf16* vg = a.v + b * a.vs_b + hk * a.vs_h;
    // visible key range of this query tile
    const int last_q = min(a.Tq, q0 + FA_BM) - 1;
    int k_hi = min(a.Tk, a.q_offset + last_q + 1);
    int k_lo = 0;
    if (a.window > 0) k_lo = max(0, a.q_offset + q0 - a.window + 1);
    const int nb_lo = k_lo / FA_BN, nb_hi = (k_hi + FA_BN - 1) / FA_BN;

    load_tile_async<FA_BM, D, C::LD>(Qs, qg, a.qs_t, a.Tq - q0);
    if (nb_lo < nb_hi) {
        load_tile_async<FA_BN, D, C::LD>(Ks, kg + (int64_t)nb_lo * FA_BN * a.ks_t, a.ks_t, a.Tk - nb_lo * FA_BN);
        load_tile_async<FA_BN, D, C::LD>(Vs, vg + (int64_t)nb_lo * FA_BN * a.vs_t, a.vs_t, a.Tk - nb_lo * FA_BN);
    }
    cp_async_commit();
    float acc_o[C::O_NT][4];
    zero_acc<C::O_NT>(acc_o);
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const float sc = a.scale * LOG2E;
    const int r0 = q0 + w * 16 + (l >> 2), r1 = r0 + 8;          // query rows of this thread
    uint32_t qf[C::KS][4];
    bool q_loaded = false;
    for (int nb = nb_lo; nb < nb_hi; ++nb) {
        const int buf = (nb - nb_lo) & 1;
        if (nb + 1 < nb_hi) {
            load_tile_async<FA_BN, D, C::LD>(Ks + (buf ^ 1) * FA_BN * C::LD, kg + (int64_t)(nb + 1) * FA_BN * a.ks_t, a.ks_t, a.Tk - (nb + 1) * FA_BN);
            load_tile_async<FA_BN, D, C::LD>(Vs + (buf ^ 1) * FA_BN * C::LD, vg + (int64_t)(nb + 1) * FA_BN * a.vs_t, a.vs_t, a.Tk - (nb + 1) * FA_BN);
        }
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (!q_loaded) {
#pragma unroll
            for (int ks = 0; ks < C::KS; ++ks) load_a(qf[ks], Qs, C::LD, w * 16, ks * 16);
            q_loaded = true;
        }
        const bf16* Kb = Ks + buf * FA_BN * C::LD;
        const bf16* Vb = Vs + buf * FA_BN * C::LD;
        float s[8][4];
        zero_acc<8>(s);
#pragma unroll
        for (int ks = 0; ks < C::KS; ++ks)
#pragma unroll
            for (int nt = 0; nt < 8; nt += 2) {
                uint32_t bfr[4];
                load_b2(bfr, Kb, C::LD, nt * 8, ks * 16);
                mma16816(s[nt], qf[ks], bfr[0], bfr[1]);
                mma16816(s[nt + 1], qf[ks], bfr[2], bfr[3]);
            }
        // scale, mask, online softmax
        float mx0 = m0, mx1 = m1;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int j = nb * FA_BN + nt * 8 + (l & 3) * 2 + (e & 1);
                const int qi = a.q_offset + ((e < 2) ? r0 : r1);
                bool ok = j <= qi && j < a.Tk && (a.window <= 0 || j > qi - a.window);
                float x = ok ? s[nt][e] * sc : -INFINITY;
                s[nt][e] = x;
                if (e < 2) mx0 = fmaxf(mx0, x); else mx1 = fmaxf(mx1, x);
            }
        mx0 = quad_max(mx0); mx1 = quad_max(mx1);
        const float c0 = (mx0 == -INFINITY) ? 1.f : exp2f(m0 - mx0), c1 = (mx1 == -INFINITY) ? 1.f : exp2f(m1 - mx1);
        const float b0 = (mx0 == -INFINITY) ? 0.f : mx0, b1 = (mx1 == -INFINITY) ? 0.f : mx1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            s[nt][0] = exp2f(s[nt][0] - b0); s[nt][1] = exp2f(s[nt][1] - b0);
            s[nt][2] = exp2f(s[nt][2] - b1); s[nt][3] = exp2f(s[nt][3] - b1);
            ps0 += s[nt][0] + s[nt][1]; ps1 += s[nt][2] + s[nt][3];
        }
        l0 = l0 * c0 + ps0; l1 = l1 * c1 + ps1;
        m0 = mx0; m1 = mx1;
#pragma unroll
        for (int nt = 0; nt < C::O_NT; ++nt) { acc_o[nt][0] *= c0; acc_o[nt][1] *= c0; acc_o[nt][2] *= c1; acc_o[nt][3] *= c1; }
        // O += P V  (P from the S accumulators)
#pragma unroll
        for (int ks = 0; ks < FA_BN / 16; ++ks) {
            uint32_t pa[4] = {pack2(s[2 * ks][0], s[2 * ks][1]), pack2(s[2 * ks][2], s[2 * ks][3]),
                              pack2(s[2 * ks + 1][0], s[2 * ks + 1][1]), pack2(s[2 * ks + 1][2], s[2 * ks + 1][3])};
#pragma unroll
            for (int nt = 0; nt < C::O_NT; nt += 2) {
                uint32_t bfr[4];
                load_b2_t(bfr, Vb, C::LD, nt * 8, ks * 16);
                mma16816(acc_o[nt], pa, bfr[0], bfr[1]);
                mma16816(acc_o[nt + 1], pa, bfr[2], bfr[3]);
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    l0 = quad_sum(l0); l1 = quad_sum(l1);
    const float i0 = l0 > 0.f ? 1.f / l0 : 0.f, i1 = l1 > 0.f ? 1.f / l1 : 0.f;
    bf16* og = a.out + (((int64_t)b * a.Tq) * a.Hq + h) * D;
    const int64_t ost = (int64_t)a.Hq * D;
#pragma unroll
    for (int nt = 0; nt < C::O_NT; ++nt) {
        const int c = nt * 8 + (l & 3) * 2;
        if (r0 < a.Tq) *reinterpret_cast<uint32_t*>(og + (int64_t)r0 * ost + c) = pack2(acc_o[nt][0] * i0, acc_o[nt][1] * i0);
        if (r1 < a.Tq) *reinterpret_cast<uint32_t*>(og + (int64_t)r1 * ost + c) = pack2(acc_o[nt][2] * i1, acc_o[nt][3] * i1);
    }
    if ((l & 3) == 0) {
        float* lg = a.lse + ((int64_t)b * a.Hq + h) * a.Tq;
        if (r0 < a.Tq) lg[r0] = l0 > 0.f ? (m0 + log2f(l0)) * LN2 : -INFINITY;
        if (r1 < a.Tq) lg[r1] = l1 > 0.f ? (m1 + log2f(l1)) * LN2 : -INFINITY;
    }
}

// delta[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]; one warp per (b,t,h)
template <int D>
__global__ void fa_delta_kernel(FaArgs a) {
    const int l = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t rows = (int64_t)a.B * a.Tq * a.Hq;
    if (row >= rows) return;
    const int h = row % a.Hq;
    const int64_t bt = row / a.Hq;
    const int t = bt % a.Tq, b = bt / a.Tq;
    float s = 0.f;
    for (int c = l * 2; c < D; c += 64) {
        float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a.o + row * D + c));
        float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a.d_o + row * D + c));
        s += x.x * y.x + x.y * y.y;
    }
    s = warp_sum(s);
    if (l == 0) a.delta[((int64_t)b * a.Hq + h) * a.Tq + t] = s;
}

// One CTA = 64 keys of one KV head; warp w owns keys [16w, 16w+16).
template <int D>
__global__ void __launch_bounds__(FA_THREADS) fa_bwd_kernel(FaArgs a) {
    using C = FaCfg<D>;
    constexpr int PLD = FA_BM + 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Ks = reinterpret_cast<bf16*>(smem_raw);
    bf16* Vs = Ks + FA_BN * C::LD;
    bf16* Qs = Vs + FA_BN * C::LD;
    bf16* Gs = Qs + FA_BM * C::LD;                 // dO
    bf16* dSs = Gs + FA_BM * C::LD;                // [FA_BN][PLD]  dS^T (keys x queries)
    float* lse2 = reinterpret_cast<float*>(dSs + FA_BN * PLD);   // [FA_BM] lse * log2(e)
    float* dlt = lse2 + FA_BM;                     // [FA_BM]
    const int nbk = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int rep = a.Hq / a.Hkv;
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    const int k0 = nbk * FA_BN;
    const bf16* kg = a.k + b * a.ks_b + hk * a.ks_h + (int64_t)k0 * a.ks_t;
    const bf16* vg = a.v + b * a.vs_b + hk * a.vs_h + (int64_t)k0 * a.vs_t;
    load_tile_async<FA_BN, D, C::LD>(Ks, kg, a.ks_t, a.Tk - k0);
    load_tile_async<FA_BN, D, C::LD>(Vs, vg, a.vs_t, a.Tk - k0);
    cp_async_commit();
    float acc_dk[C::O_NT][4], acc_dv[C::O_NT][4];
    zero_acc<C::O_NT>(acc_dk);
    zero_acc<C::O_NT>(acc_dv);
    const float sc = a.scale * LOG2E;
    // query tiles that can see any key of this block: i >= k0 - q_offset; with a window: i < k0 + 64 + window - q_offset - 1
    int qb_lo = max(0, k0 - a.q_offset) / FA_BM;
    int q_end = a.Tq;
    if (a.window > 0) q_end = min(a.Tq, max(0, k0 + FA_BN - 1 + a.window - a.q_offset));
    const int qb_hi = (q_end + FA_BM - 1) / FA_BM;
    const int j0 = k0 + w * 16 + (l >> 2), j1 = j0 + 8;          // key rows of this thread
    for (int hh = 0; hh < rep; ++hh) {
        const int h = hk * rep + hh;
        const bf16* qg = a.q + b * a.qs_b + h * a.qs_h;
        const bf16* gg = a.d_o + ((int64_t)b * a.Tq * a.Hq + h) * D;
        const int64_t gst = (int64_t)a.Hq * D;
        const float* lg = a.lse + ((int64_t)b * a.Hq + h) * a.Tq;
        const float* dg = a.delta + ((int64_t)b * a.Hq + h) * a.Tq;
        float* dqg = a.dq_acc + ((int64_t)b * a.Tq * a.Hq + h) * D;
        for (int qb = qb_lo; qb < qb_hi; ++qb) {
            const int q0 = qb * FA_BM;
            __syncthreads();                                     // previous tile's readers are done
            load_tile_async<FA_BM, D, C::LD>(Qs, qg + (int64_t)q0 * a.qs_t, a.qs_t, a.Tq - q0);
            load_tile_async<FA_BM, D, C::LD>(Gs, gg + (int64_t)q0 * gst, gst, a.Tq - q0);
            cp_async_commit();
            if (threadIdx.x < FA_BM) {
                const int i = q0 + threadIdx.x;
                lse2[threadIdx.x] = i < a.Tq ? lg[i] * LOG2E : INFINITY;     // +inf -> p = 0 for padded queries
                dlt[threadIdx.x] = i < a.Tq ? dg[i] : 0.f;
            }
            cp_async_wait<0>();
            __syncthreads();
            // S^T = K Q^T, dP^T = V dO^T   (16 keys x 64 queries per warp)
            float st[8][4], dpt[8][4];
            zero_acc<8>(st);
            zero_acc<8>(dpt);
            warp_gemm<8, D, false, false>(st, Ks, C::LD, w * 16, Qs, C::LD, 0);
            warp_gemm<8, D, false, false>(dpt, Vs, C::LD, w * 16, Gs, C::LD, 0);
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int ci = nt * 8 + (l & 3) * 2 + (e & 1);      // query column inside the tile
                    const int qi = a.q_offset + q0 + ci;
                    const int j = (e < 2) ? j0 : j1;
                    const bool ok = j <= qi && j < a.Tk && (a.window <= 0 || j > qi - a.window);
                    const float p = ok ? exp2f(st[nt][e] * sc - lse2[ci]) : 0.f;
                    st[nt][e] = p;
                    dpt[nt][e] = p * (dpt[nt][e] - dlt[ci]);            // dS^T (unscaled)
                }
            // dV += P^T dO ; dK += dS^T Q   (A operands straight from the accumulator registers)
#pragma unroll
            for (int ks = 0; ks < FA_BM / 16; ++ks) {
                uint32_t pa[4] = {pack2(st[2 * ks][0], st[2 * ks][1]), pack2(st[2 * ks][2], st[2 * ks][3]),
                                  pack2(st[2 * ks + 1][0], st[2 * ks + 1][1]), pack2(st[2 * ks + 1][2], st[2 * ks + 1][3])};
                uint32_t da[4] = {pack2(dpt[2 * ks][0], dpt[2 * ks][1]), pack2(dpt[2 * ks][2], dpt[2 * ks][3]),
                                  pack2(dpt[2 * ks + 1][0], dpt[2 * ks + 1][1]), pack2(dpt[2 * ks + 1][2], dpt[2 * ks + 1][3])};
#pragma unroll
                for (int nt = 0; nt < C::O_NT; nt += 2) {
                    uint32_t bg[4], bq[4];
                    load_b2_t(bg, Gs, C::LD, nt * 8, ks * 16);
                    load_b2_t(bq, Qs, C::LD, nt * 8, ks * 16);
                    mma16816(acc_dv[nt], pa, bg[0], bg[1]);
                    mma16816(acc_dv[nt + 1], pa, bg[2], bg[3]);
                    mma16816(acc_dk[nt], da, bq[0], bq[1]);
                    mma16816(acc_dk[nt + 1], da, bq[2], bq[3]);
                }
            }
            // dS^T -> shared memory (bf16), then dQ[16 queries per warp] += dS K
            store_acc_bf16<8>(dpt, dSs, PLD, w * 16, 0);
            __syncthreads();
            float acc_dq[C::O_NT][4];
            zero_acc<C::O_NT>(acc_dq);
            warp_gemm<C::O_NT, FA_BN, true, true>(acc_dq, dSs, PLD, w * 16, Ks, C::LD, 0);
            const int i0 = q0 + w * 16 + (l >> 2), i1 = i0 + 8;
#pragma unroll
            for (int nt = 0; nt < C::O_NT; ++nt) {
                const int c = nt * 8 + (l & 3) * 2;
                if (i0 < a.Tq) {
                    atomicAdd(dqg + (int64_t)i0 * gst + c, acc_dq[nt][0] * a.scale);
                    atomicAdd(dqg + (int64_t)i0 * gst + c + 1, acc_dq[nt][1] * a.scale);
                }
                if (i1 < a.Tq) {
                    atomicAdd(dqg + (int64_t)i1 * gst + c, acc_dq[nt][2] * a.scale);
                    atomicAdd(dqg + (int64_t)i1 * gst + c + 1, acc_dq[nt][3] * a.scale);
                }
            }
        }
    }
    cp_async_wait<0>();
    bf16* dkg = a.dk + (((int64_t)b * a.Tk) * a.Hkv + hk) * D;
    bf16* dvg = a.dv + (((int64_t)b * a.Tk) * a.Hkv + hk) * D;
    const int64_t kst = (int64_t)a.Hkv * D;
#pragma unroll
    for (int nt = 0; nt < C::O_NT; ++nt) {
        const int c = nt * 8 + (l & 3) * 2;
        if (j0 < a.Tk) {
            *reinterpret_cast<uint32_t*>(dkg + (int64_t)j0 * kst + c) = pack2(acc_dk[nt][0] * a.scale, acc_dk[nt][1] * a.scale);
            *reinterpret_cast<uint32_t*>(dvg + (int64_t)j0 * kst + c) = pack2(acc_dv[nt][0], acc_dv[nt][1]);
        }
        if (j1 < a.Tk) {
            *reinterpret_cast<uint32_t*>(dkg + (int64_t)j1 * kst + c) = pack2(acc_dk[nt][2] * a.scale, acc_dk[nt][3] * a.scale);
            *reinterpret_cast<uint32_t*>(dvg + (int64_t)j1 * kst + c) = pack2(acc_dv[nt][2], acc_dv[nt][3]);
        }
    }
}

template <int D> constexpr size_t fa_smem_fwd() { return (size_t)(FA_BM + 4 * FA_BN) * FaCfg<D>::LD * 2; }
template <int D> constexpr size_t fa_smem_bwd() {
    return (size_t)(2 * FA_BN + 2 * FA_BM) * FaCfg<D>::LD * 2 + (size_t)FA_BN * (FA_BM + 8) * 2 + 2 * FA_BM * 4;
}

}  // namespace lmoe

using namespace lmoe;

LMOE_API int lmoe_flash_attn_fwd(const FaArgs* ap, int D, cudaStream_t st) {
    const FaArgs a = *ap;
    dim3 grid((a.Tq + FA_BM - 1) / FA_BM, a.Hq, a.B);
    if (D == 128) {
        cudaFuncSetAttribute(fa_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_smem_fwd<128>());
        fa_fwd_kernel<128><<<grid, FA_THREADS, fa_smem_fwd<128>(), st>>>(a);
    } else if (D == 64) {
        cudaFuncSetAttribute(fa_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_smem_fwd<64>());
        fa_fwd_kernel<64><<<grid, FA_THREADS, fa_smem_fwd<64>(), st>>>(a);
    } else return -1;
    return (int)cudaGetLastError();
}

// Needs a.delta [B,Hq,Tq] scratch and a.dq_acc zero-initialised fp32 [B,Tq,Hq,D].
LMOE_API int lmoe_flash_attn_bwd(const FaArgs* ap, int D, cudaStream_t st) {
    const FaArgs a = *ap;
    const int64_t rows = (int64_t)a.B * a.Tq * a.Hq;
    dim3 grid((a.Tk + FA_BN - 1) / FA_BN, a.Hkv, a.B);
    if (D == 128) {
        fa_delta_kernel<128><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(a);
        cudaFuncSetAttribute(fa_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_smem_bwd<128>());
        fa_bwd_kernel<128><<<grid, FA_THREADS, fa_smem_bwd<128>(), st>>>(a);
    } else if (D == 64) {
        fa_delta_kernel<64><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(a);
        cudaFuncSetAttribute(fa_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fa_smem_bwd<64>());
        fa_bwd_kernel<64><<<grid, FA_THREADS, fa_smem_bwd<64>(), st>>>(a);
    } else return -1;
    return (int)cudaGetLastError();
}
