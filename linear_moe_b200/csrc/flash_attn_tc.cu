// Flash-attention forward on the 5th-generation tensor cores: S = Q K^T and O_j = P_j V_j are tcgen05.mma instructions
// with accumulators in tensor memory, operands staged by TMA (4-D tensor maps over [B, T, H, D], 128-byte swizzle).
//
// One CTA = 128 queries of one head.  128 + 128 * SPLIT threads (warps 0-1: TMA / MMA, warps 2-3 idle, warps 4.. softmax):
//   warp 0      TMA producer: Q once, then K_j / V_j tiles of 128 keys through two 2-stage rings
//   warp 1      MMA issuer:   S_{j+1} = Q K_{j+1}^T is issued before P_j V_j, so the tensor core works on the next
//               score tile while the softmax warps are busy with the current one
//   warps 4..   softmax: the SPLIT warps with equal (w & 3) own the 32 query rows of that TMEM lane quarter and split
//               the columns: one tensor-memory load of the scores, row max (exchanged between the parts through
//               shared memory and a named barrier), exp2 / sum / bf16 pack, P_j written to shared memory in
//               the K-major 128-byte-swizzle layout the MMA reads; O += P_j V_j is folded into registers
//               (o = o * corr + O_j) one iteration later, so that it overlaps the next tile's math.  SPLIT warps per
//               scheduler hide the tensor-memory latency; no tensor-memory stores, no shuffles.
// Tensor memory: 2 x 128 columns of scores + 2 x D columns of partial outputs.
// Masking (causal with a query offset, sliding window, key length) is applied only on tiles that cross a boundary.
// Every mbarrier wait is bounded (clock64 budget); on expiry the error word is set and the CTA drains and frees its
// tensor memory.  Writes O (bf16) and the natural-log row log-sum-exp, which the backward kernels of flash_attn.cu use.
//
// Replaces dot_product_attention.py:139-183 (baddbmm + softmax + bmm) and the flash_attn / TransformerEngine back ends
// of the reference (llama3/transformer_legacy.py:446-505).
#include "tcgen05_utils.cuh"

namespace lmoe {
namespace fatc {
using namespace lmoe::tc;

constexpr int BM = 128, BN = 128, SPLIT = 4, THREADS = 128 + 128 * SPLIT, UMMA_K = 16;
constexpr float LOG2E = 1.4426950408889634f;

struct Args {
    bf16* out;            // [B, Tq, Hq, D]
    float* lse;           // [B, Hq, Tq]
    int B, Tq, Tk, Hq, Hkv;
    int q_offset, window; // window <= 0: none
    float scale;
    int* err;
};

template <int D>
struct __align__(1024) Smem {
    uint8_t q[BM * D * 2];
    uint8_t k[2][BN * D * 2];
    uint8_t v[2][BN * D * 2];
    uint8_t p[BM * BN * 2];
    uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], o_full[2], p_ready;
    float mx[2][SPLIT][BM], ls[SPLIT][BM];
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 :: "r"(s32(dst)), "l"(map), "r"(s32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
template <bool B_MN, int N>
__host__ __device__ constexpr uint32_t idesc_bf16() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((B_MN ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&r)[64]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
                 "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
                   "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
                   "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
                   "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
                   "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&r)[N]) {
    static_assert(N == 16 || N == 32 || N == 64, "tensor-memory load width");
    if constexpr (N == 64) tmem_ld64(taddr, r);
    else if constexpr (N == 32) tmem_ld32(taddr, r);
    else tmem_ld16(taddr, r);
}
// o[i] = o[i] * corr + partial[i] for this thread's OW columns of the partial output in tensor memory
template <int OW>
__device__ __forceinline__ void fold_o(float (&o)[OW], uint32_t taddr, float corr) {
    uint32_t v[OW];
    tmem_ld<OW>(taddr, v);
    tmem_ld_wait();
    const float2 c2 = make_float2(corr, corr);
#pragma unroll
    for (int i = 0; i < OW; i += 2) {                            // packed fp32 FMAs: two columns per instruction
        const float2 r = __ffma2_rn(make_float2(o[i], o[i + 1]), c2, make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])));
        o[i] = r.x;
        o[i + 1] = r.y;
    }
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// Bounded wait that lets the hardware suspend the warp (try_wait with a time hint) instead of spinning on test_wait:
// the 16 softmax warps share 4 schedulers, a spinning warp takes issue slots from the others.
__device__ __forceinline__ bool mbar_wait_suspend(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
                     : "=r"(ok) : "r"(s32(bar)), "r"(parity), "r"(20000u) : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_CYCLES) break;
    }
    *abort_flag = 1;
    atomicCAS(err, 0, code);
    return false;
}

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
fa_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, Args a) {
    extern __shared__ uint8_t smem_raw[];
    Smem<D>& sm = *reinterpret_cast<Smem<D>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int DK = D / 64;                              // 64-element blocks along the head dimension
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t O_COL = 2 * BN;                      // partial outputs behind the two score buffers
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = gridDim.x - 1 - blockIdx.x;              // long (late) query tiles first
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (a.Hq / a.Hkv);
    const int q0 = qb * BM;
    volatile int* abort_flag = &sm.abort_flag;
    int* err = a.err;

    // visible key range of this query tile -> key tiles [nb_lo, nb_hi)
    const int last_q = min(a.Tq, q0 + BM) - 1;
    const int k_hi = min(a.Tk, a.q_offset + last_q + 1);
    const int k_lo = a.window > 0 ? max(0, a.q_offset + q0 - a.window + 1) : 0;
    const int nb_lo = k_lo / BN, nb_hi = (k_hi + BN - 1) / BN;
    const int n_it = max(nb_hi - nb_lo, 0);

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sm.k_full[s], 1); mbar_init(&sm.k_empty[s], 1);
            mbar_init(&sm.v_full[s], 1); mbar_init(&sm.v_empty[s], 1);
            mbar_init(&sm.s_full[s], 1); mbar_init(&sm.o_full[s], 1);
        }
        mbar_init(&sm.p_ready, 4 * SPLIT);
        sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(s32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sm.tmem_base;

    if (warp == 0) {
        if (lane == 0 && n_it > 0) {
            mbar_expect_tx(&sm.q_full, BM * D * 2);
#pragma unroll
            for (int kb = 0; kb < DK; ++kb) tma_load_4d(sm.q + kb * BM * 128, &tmQ, &sm.q_full, kb * 64, h, q0, b);
            for (int j = 0; j < n_it; ++j) {
                const int s = j & 1;
                const uint32_t ph = (j >> 1) & 1;
                const int key0 = (nb_lo + j) * BN;
                if (!mbar_wait_suspend(&sm.k_empty[s], ph ^ 1, abort_flag, err, 0x1100 | s)) break;
                mbar_expect_tx(&sm.k_full[s], BN * D * 2);
#pragma unroll
                for (int kb = 0; kb < DK; ++kb) tma_load_4d(sm.k[s] + kb * BN * 128, &tmK, &sm.k_full[s], kb * 64, hk, key0, b);
                if (!mbar_wait_suspend(&sm.v_empty[s], ph ^ 1, abort_flag, err, 0x1200 | s)) break;
                mbar_expect_tx(&sm.v_full[s], BN * D * 2);
                // MN-major operand: per 64 keys, D/64 boxes of {64 d, 64 keys} (8 KiB each)
#pragma unroll
                for (int kk = 0; kk < BN / 64; ++kk)
#pragma unroll
                    for (int nb = 0; nb < DK; ++nb)
                        tma_load_4d(sm.v[s] + (kk * DK + nb) * 8192, &tmV, &sm.v_full[s], nb * 64, hk, key0 + kk * 64, b);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && n_it > 0) {
            constexpr uint32_t idesc_s = idesc_bf16<false, BN>();
            constexpr uint32_t idesc_o = idesc_bf16<true, D>();
            bool ok = mbar_wait_suspend(&sm.q_full, 0, abort_flag, err, 0x2000);
            auto issue_s = [&](int j) -> bool {
                const int s = j & 1;
                if (!mbar_wait_suspend(&sm.k_full[s], (j >> 1) & 1, abort_flag, err, 0x2100 | s)) return false;
                tc_fence_after();
                const uint32_t qa = s32(sm.q), ka = s32(sm.k[s]);
#pragma unroll
                for (int kk = 0; kk < D / UMMA_K; ++kk) {
                    const uint32_t off = (kk / 4) * (BM * 128) + (kk % 4) * 32;
                    umma_f16(tmem_base + s * BN, make_desc<false>(qa + off), make_desc<false>(ka + off), idesc_s, kk > 0 ? 1u : 0u);
                }
                umma_commit(&sm.k_empty[s]);
                umma_commit(&sm.s_full[s]);
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int j = 0; ok && j < n_it; ++j) {
                if (j + 1 < n_it) { ok = issue_s(j + 1); if (!ok) break; }
                const int s = j & 1;
                if (!mbar_wait_suspend(&sm.v_full[s], (j >> 1) & 1, abort_flag, err, 0x2200 | s)) break;
                if (!mbar_wait_suspend(&sm.p_ready, j & 1, abort_flag, err, 0x2300)) break;
                tc_fence_after();
                const uint32_t pa = s32(sm.p), va = s32(sm.v[s]);
#pragma unroll
                for (int kk = 0; kk < BN / UMMA_K; ++kk) {
                    const uint32_t aoff = (kk / 4) * (BM * 128) + (kk % 4) * 32;
                    const uint32_t boff = (kk / 4) * (DK * 8192) + (kk % 4) * 2048;
                    umma_f16(tmem_base + O_COL + s * D, make_desc<false>(pa + aoff), make_desc<true>(va + boff), idesc_o, kk > 0 ? 1u : 0u);
                }
                umma_commit(&sm.v_empty[s]);
                umma_commit(&sm.o_full[s]);
            }
        }
    } else if (warp >= 4) {
        // 4*SPLIT softmax warps: the SPLIT warps with the same (warp & 3) own the 32 query rows of that TMEM lane
        // quarter and split the score / output columns between them
        const int qd = warp & 3;
        const int part = (warp - 4) >> 2;
        const int r = qd * 32 + lane;                         // query row inside the tile
        const int qi = a.q_offset + q0 + r;                   // absolute position of this query
        const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
        const float sc = a.scale * LOG2E;
        constexpr int CW = BN / SPLIT;                        // score columns of this thread
        constexpr int OW = D / SPLIT;                         // output columns of this thread
        float o[OW];
#pragma unroll
        for (int i = 0; i < OW; ++i) o[i] = 0.f;
        float m = -INFINITY, l = 0.f, corr_prev = 1.f;
        // CW keys = CW * 2 bytes inside the 128-byte row of key block (part * CW) / 64
        uint8_t* prow = sm.p + ((part * CW) >> 6) * (BM * 128) + (r >> 3) * 1024 + (r & 7) * 128;
        const int ch0 = ((part * CW) & 63) >> 3;
        bool alive = n_it > 0;
        for (int j = 0; alive && j < n_it; ++j) {
            const int s = j & 1;
            const int tile_key0 = (nb_lo + j) * BN;
            const int key0 = tile_key0 + part * CW;           // first key of this thread's columns
            if (!mbar_wait_suspend(&sm.s_full[s], (j >> 1) & 1, abort_flag, err, 0x3100 | s)) { alive = false; break; }
            tc_fence_after();
            const bool need_mask = (tile_key0 + BN - 1 > a.q_offset + q0) || (tile_key0 + BN > a.Tk) ||
                                   (a.window > 0 && tile_key0 <= a.q_offset + q0 + BM - 1 - a.window);
            // pass 1: row maximum, 16 columns at a time (keeps the live register set small)
            float mx4[4] = {m, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < CW; c += 16) {
                uint32_t v[16];
                tmem_ld16(lane_addr + s * BN + part * CW + c, v);
                tmem_ld_wait();
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int key = key0 + c + i;
                        const bool vis = key <= qi && key < a.Tk && (a.window <= 0 || key > qi - a.window);
                        if (!vis) v[i] = 0xff800000u;         // -inf
                    }
                }
#pragma unroll
                for (int e = 0; e < 4; ++e)                              // 3-input max: two scores per instruction
                    mx4[e] = max3(max3(mx4[e], __uint_as_float(v[e]), __uint_as_float(v[e + 4])), __uint_as_float(v[e + 8]),
                                  __uint_as_float(v[e + 12]));
            }
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // row maximum over the SPLIT parts (buffers alternate so that a fast thread cannot overwrite a value a slow
            // one still has to read)
            sm.mx[s][part][r] = mx;
            asm volatile("bar.sync %0, %1;" :: "r"(1 + qd), "n"(32 * SPLIT) : "memory");
#pragma unroll
            for (int q2 = 0; q2 < SPLIT; ++q2) mx = fmaxf(mx, sm.mx[s][q2][r]);
            const float corr = (m == -INFINITY) ? 1.f : exp2f((m - mx) * sc);
            const float msc = (mx == -INFINITY) ? 0.f : mx * sc;
            m = mx;
            // the P buffer and the partial output of the previous tile are free once P_{j-1} V_{j-1} has completed
            if (j > 0 && !mbar_wait_suspend(&sm.o_full[s ^ 1], ((j - 1) >> 1) & 1, abort_flag, err, 0x3200 | s)) { alive = false; break; }
            // pass 2: p = exp2(s * sc - m * sc), row sum, bf16 pack, swizzled 16-byte stores
            float ps4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < CW; c += 16) {
                uint32_t v[16];
                tmem_ld16(lane_addr + s * BN + part * CW + c, v);
                tmem_ld_wait();
                if (need_mask) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int key = key0 + c + i;
                        const bool vis = key <= qi && key < a.Tk && (a.window <= 0 || key > qi - a.window);
                        if (!vis) v[i] = 0xff800000u;
                    }
                }
#pragma unroll
                for (int i = 0; i < 16; i += 4) {
                    const float2 sc2 = make_float2(sc, sc), nm2 = make_float2(-msc, -msc);
                    const float2 x01 = __ffma2_rn(make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), sc2, nm2);
                    const float2 x23 = __ffma2_rn(make_float2(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])), sc2, nm2);
                    const float p0 = exp2f(x01.x), p1 = exp2f(x01.y), p2 = exp2f(x23.x), p3 = exp2f(x23.y);
                    const float2 s01 = __fadd2_rn(make_float2(ps4[0], ps4[1]), make_float2(p0, p1));
                    const float2 s23 = __fadd2_rn(make_float2(ps4[2], ps4[3]), make_float2(p2, p3));
                    ps4[0] = s01.x; ps4[1] = s01.y; ps4[2] = s23.x; ps4[3] = s23.y;
                    v[i >> 1] = pack_bf16(p0, p1);
                    v[(i >> 1) + 1] = pack_bf16(p2, p3);
                }
                const int ch = ch0 + (c >> 3);
                *reinterpret_cast<uint4*>(prow + ((ch ^ (r & 7)) << 4)) = make_uint4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<uint4*>(prow + (((ch + 1) ^ (r & 7)) << 4)) = make_uint4(v[4], v[5], v[6], v[7]);
            }
            l = l * corr + ((ps4[0] + ps4[1]) + (ps4[2] + ps4[3]));
            // hand P_j to the MMA warp
            tc_fence_before();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.p_ready);
            // fold the previous tile's partial output while the tensor core runs P_j V_j
            if (j > 0) {
                tc_fence_after();
                fold_o<OW>(o, lane_addr + O_COL + (s ^ 1) * D + part * OW, corr_prev);
            }
            corr_prev = corr;
        }
        if (alive && n_it > 0) {
            const int s = (n_it - 1) & 1;
            if (mbar_wait_suspend(&sm.o_full[s], ((n_it - 1) >> 1) & 1, abort_flag, err, 0x3300 | s)) {
                tc_fence_after();
                fold_o<OW>(o, lane_addr + O_COL + s * D + part * OW, corr_prev);
            }
        }
        // total row sum over the parts
        sm.ls[part][r] = l;
        asm volatile("bar.sync %0, %1;" :: "r"(1 + qd), "n"(32 * SPLIT) : "memory");
        l = 0.f;
#pragma unroll
        for (int q2 = 0; q2 < SPLIT; ++q2) l += sm.ls[q2][r];
        const int row = q0 + r;
        if (row < a.Tq) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* og = a.out + (((long long)b * a.Tq + row) * a.Hq + h) * D + part * OW;
#pragma unroll
            for (int c = 0; c < OW; c += 8) {
                uint4 w;
                w.x = pack_bf16(o[c] * inv, o[c + 1] * inv);
                w.y = pack_bf16(o[c + 2] * inv, o[c + 3] * inv);
                w.z = pack_bf16(o[c + 4] * inv, o[c + 5] * inv);
                w.w = pack_bf16(o[c + 6] * inv, o[c + 7] * inv);
                *reinterpret_cast<uint4*>(og + c) = w;
            }
            if (part == 0) a.lse[((long long)b * a.Hq + h) * a.Tq + row] = l > 0.f ? m * a.scale + logf(l) : -INFINITY;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// [B, T, H, D] bf16 with element strides (sb, st, sh), unit stride along D; box = {64, 1, box_t, 1}
static int make_map_4d(CUtensorMap* map, const void* ptr, int B, int T, int H, int D, long long sb, long long st, long long sh,
                       uint32_t box_t) {
    EncodeTiledFn enc = get_encode();
    if (enc == nullptr) return -10;
    cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)st * 2, (cuuint64_t)sb * 2};
    cuuint32_t box[4] = {64, 1, box_t, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -11;
}

}  // namespace fatc
}  // namespace lmoe

using namespace lmoe;
using namespace lmoe::fatc;

// q [B,Tq,Hq,D], k/v [B,Tk,Hkv,D] bf16 with element strides (batch, token, head); 16-byte aligned bases, strides % 8 == 0.
LMOE_API int lmoe_flash_attn_fwd_tc(const void* q, const long long* qs, const void* k, const long long* ks, const void* v,
                                    const long long* vs, const Args* ap, int D, cudaStream_t st) {
    const Args a = *ap;
    CUtensorMap mq, mk, mv;
    int rc = make_map_4d(&mq, q, a.B, a.Tq, a.Hq, D, qs[0], qs[1], qs[2], BM);
    if (rc) return rc;
    rc = make_map_4d(&mk, k, a.B, a.Tk, a.Hkv, D, ks[0], ks[1], ks[2], BN);
    if (rc) return rc;
    rc = make_map_4d(&mv, v, a.B, a.Tk, a.Hkv, D, vs[0], vs[1], vs[2], 64);
    if (rc) return rc;
    dim3 grid((a.Tq + BM - 1) / BM, a.Hq, a.B);
    if (D == 128) {
        const size_t smem = sizeof(Smem<128>) + 1024;
        cudaFuncSetAttribute(fa_fwd_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        fa_fwd_tc_kernel<128><<<grid, THREADS, smem, st>>>(mq, mk, mv, a);
    } else if (D == 64) {
        const size_t smem = sizeof(Smem<64>) + 1024;
        cudaFuncSetAttribute(fa_fwd_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        fa_fwd_tc_kernel<64><<<grid, THREADS, smem, st>>>(mq, mk, mv, a);
    } else return -1;
    return (int)cudaGetLastError();
}
