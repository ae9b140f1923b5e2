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
#include <cstdio>
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
// The MMA warp runs its loop with all 32 lanes converged and only predicates the tcgen05 instructions on one lane: inside a
// single-lane branch every operand lives in vector registers and each MMA pays for moving two 64-bit descriptors into
// uniform registers, which at 64-column tiles costs more cycles than the MMA keeps the tensor core busy.  Descriptors are
// built once per tile as a 32-bit low word (address / 16 and the leading-dimension offset); the high word is a constant and
// stepping along K inside the swizzled tile is an add to the low word.
constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);      // stride offset 1024 B, version 1, 128-byte swizzle
template <bool MN>
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr) {
    return ((saddr >> 4) & 0x3FFFu) | ((MN ? (8192u >> 4) : 1u) << 16);
}
__device__ __forceinline__ void umma_lo(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate, uint32_t issue) {
    asm volatile("{\n.reg .pred p, q;\n.reg .b64 da, db;\nsetp.ne.b32 p, %4, 0;\nsetp.ne.b32 q, %5, 0;\n"
                 "mov.b64 da, {%1, %6};\nmov.b64 db, {%2, %6};\n"
                 "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n}"
                 :: "r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(issue), "r"(DESC_HI) : "memory");
}
__device__ __forceinline__ void umma_commit_if(uint64_t* bar, uint32_t issue) {
    asm volatile("{\n.reg .pred q;\nsetp.ne.b32 q, %1, 0;\n"
                 "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}" :: "r"(s32(bar)), "r"(issue) : "memory");
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
        if (n_it > 0) {
            const uint32_t issue = lane == 0 ? 1u : 0u;
            constexpr uint32_t idesc_s = idesc_bf16<false, BN>();
            constexpr uint32_t idesc_o = idesc_bf16<true, D>();
            bool ok = mbar_wait_suspend(&sm.q_full, 0, abort_flag, err, 0x2000);
            auto issue_s = [&](int j) -> bool {
                const int s = j & 1;
                if (!mbar_wait_suspend(&sm.k_full[s], (j >> 1) & 1, abort_flag, err, 0x2100 | s)) return false;
                tc_fence_after();
                const uint32_t ql = desc_lo<false>(s32(sm.q)), kl = desc_lo<false>(s32(sm.k[s]));
#pragma unroll
                for (int kk = 0; kk < D / UMMA_K; ++kk) {
                    const uint32_t off = ((kk / 4) * (BM * 128) + (kk % 4) * 32) >> 4;
                    umma_lo(tmem_base + s * BN, ql + off, kl + off, idesc_s, kk > 0 ? 1u : 0u, issue);
                }
                umma_commit_if(&sm.k_empty[s], issue);
                umma_commit_if(&sm.s_full[s], issue);
                return true;
            };
            if (ok) ok = issue_s(0);
            for (int j = 0; ok && j < n_it; ++j) {
                if (j + 1 < n_it) { ok = issue_s(j + 1); if (!ok) break; }
                const int s = j & 1;
                if (!mbar_wait_suspend(&sm.v_full[s], (j >> 1) & 1, abort_flag, err, 0x2200 | s)) break;
                if (!mbar_wait_suspend(&sm.p_ready, j & 1, abort_flag, err, 0x2300)) break;
                tc_fence_after();
                const uint32_t pl = desc_lo<false>(s32(sm.p)), vl = desc_lo<true>(s32(sm.v[s]));
#pragma unroll
                for (int kk = 0; kk < BN / UMMA_K; ++kk) {
                    const uint32_t aoff = ((kk / 4) * (BM * 128) + (kk % 4) * 32) >> 4;
                    const uint32_t boff = ((kk / 4) * (DK * 8192) + (kk % 4) * 2048) >> 4;
                    umma_lo(tmem_base + O_COL + s * D, pl + aoff, vl + boff, idesc_o, kk > 0 ? 1u : 0u, issue);
                }
                umma_commit_if(&sm.v_empty[s], issue);
                umma_commit_if(&sm.o_full[s], issue);
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


// =====================================================================================================================
// Backward on tcgen05, two kernels that recompute the scores (7 GEMMs per tile pair instead of 5, no atomics):
//   fa_bwd_dq_tc_kernel    one CTA = 128 queries of one head; loops over tiles of 64 keys:
//                          S = Q K^T and dP = dO V^T into tensor memory -> dS = P (dP - delta) scale (softmax warps,
//                          thread = query row) -> shared memory -> dQ += dS K accumulated in tensor memory.
//   fa_bwd_dkv_tc_kernel   one CTA = 128 keys of one KV head; loops over the query heads of the group and tiles of 64
//                          queries: S^T = K Q^T and dP^T = V dO^T -> P^T, dS^T (thread = key row) -> shared memory ->
//                          dV += P^T dO and dK += dS^T Q accumulated in tensor memory.
// A [64 x D] tile loaded as D/64 boxes of {64 d, 64 rows} serves both as a K-major operand (rows = N) of the score GEMMs
// and as an MN-major operand (rows = K) of the gradient GEMMs.  Same warp roles, barriers and bounded waits as the forward.
// =====================================================================================================================
constexpr int BT = 64;                                       // tile of the looped dimension (keys for dQ, queries for dK/dV)
constexpr int NST = 3;                                       // TMA stages of the looped tiles: a stage is released only after the
                                                             // gradient MMAs of its iteration, so two stages would expose the load latency

struct BwdArgs {
    const float* lse;     // [B, Hq, Tq] natural-log sum-exp from the forward
    const float* delta;   // [B, Hq, Tq] rowsum(dO * O)
    bf16* dq;             // [B, Tq, Hq, D]
    bf16* dk;             // [B, Tk, Hkv, D]
    bf16* dv;             // [B, Tk, Hkv, D]
    int B, Tq, Tk, Hq, Hkv;
    int q_offset, window;
    float scale;
    int* err;
};

template <int D>
struct __align__(1024) SmemBwd {
    uint8_t big0[BM * D * 2];          // dQ kernel: Q tile      | dK/dV kernel: K tile
    uint8_t big1[BM * D * 2];          // dQ kernel: dO tile     | dK/dV kernel: V tile
    uint8_t st0[NST][BT * D * 2];        // dQ kernel: K stages    | dK/dV kernel: Q stages
    uint8_t st1[NST][BT * D * 2];        // dQ kernel: V stages    | dK/dV kernel: dO stages
    uint8_t p[BM * BT * 2];            // dS (dQ kernel) | P^T (dK/dV kernel), K-major, 128 rows x 128 bytes
    uint8_t ds[BM * BT * 2];           // dS^T (dK/dV kernel)
    uint64_t big_full, st_full[NST], st_empty[NST], s_full[2], p_ready, acc_done;
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ bool visible(int key, int qi, int Tk, int window) {
    return key <= qi && key < Tk && (window <= 0 || key > qi - window);
}

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
fa_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmG,
                    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, BwdArgs a) {
    extern __shared__ uint8_t smem_raw[];
    SmemBwd<D>& sm = *reinterpret_cast<SmemBwd<D>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int DK = D / 64;
    constexpr uint32_t TMEM_COLS = 512, ACC_COL = 256;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = gridDim.x - 1 - blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (a.Hq / a.Hkv);
    const int q0 = qb * BM;
    volatile int* abort_flag = &sm.abort_flag;
    int* err = a.err;
    const int last_q = min(a.Tq, q0 + BM) - 1;
    const int k_hi = min(a.Tk, a.q_offset + last_q + 1);
    const int k_lo = a.window > 0 ? max(0, a.q_offset + q0 - a.window + 1) : 0;
    const int nb_lo = k_lo / BT, nb_hi = (k_hi + BT - 1) / BT;
    const int n_it = max(nb_hi - nb_lo, 0);

    if (threadIdx.x == 0) {
        mbar_init(&sm.big_full, 1);
        for (int s = 0; s < NST; ++s) { mbar_init(&sm.st_full[s], 1); mbar_init(&sm.st_empty[s], 1); }
        for (int s = 0; s < 2; ++s) mbar_init(&sm.s_full[s], 1);
        mbar_init(&sm.p_ready, 4 * SPLIT);
        mbar_init(&sm.acc_done, 1);
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
            mbar_expect_tx(&sm.big_full, 2 * BM * D * 2);
#pragma unroll
            for (int kb = 0; kb < DK; ++kb) {
                tma_load_4d(sm.big0 + kb * BM * 128, &tmQ, &sm.big_full, kb * 64, h, q0, b);
                tma_load_4d(sm.big1 + kb * BM * 128, &tmG, &sm.big_full, kb * 64, h, q0, b);
            }
            for (int j = 0; j < n_it; ++j) {
                const int s = j % NST;
                const int key0 = (nb_lo + j) * BT;
                if (!mbar_wait_suspend(&sm.st_empty[s], ((j / NST) & 1) ^ 1, abort_flag, err, 0x4100 | s)) break;
                mbar_expect_tx(&sm.st_full[s], 2 * BT * D * 2);
#pragma unroll
                for (int kb = 0; kb < DK; ++kb) {
                    tma_load_4d(sm.st0[s] + kb * 8192, &tmK, &sm.st_full[s], kb * 64, hk, key0, b);
                    tma_load_4d(sm.st1[s] + kb * 8192, &tmV, &sm.st_full[s], kb * 64, hk, key0, b);
                }
            }
        }
    } else if (warp == 1) {
        if (n_it > 0) {
            const uint32_t issue = lane == 0 ? 1u : 0u;
            constexpr uint32_t idesc_s = idesc_bf16<false, BT>();       // [128 q] x [64 keys], both K-major
            constexpr uint32_t idesc_a = idesc_bf16<true, D>();         // dQ += dS K: B = K tile read MN-major
            bool ok = mbar_wait_suspend(&sm.big_full, 0, abort_flag, err, 0x4200);
            auto issue_sd = [&](int j) -> bool {
                const int s = j & 1, g = j % NST;                    // tensor-memory buffer, shared-memory stage
                if (!mbar_wait_suspend(&sm.st_full[g], (j / NST) & 1, abort_flag, err, 0x4300 | g)) return false;
                tc_fence_after();
                const uint32_t ql = desc_lo<false>(s32(sm.big0)), gl = desc_lo<false>(s32(sm.big1));
                const uint32_t kl = desc_lo<false>(s32(sm.st0[g])), vl = desc_lo<false>(s32(sm.st1[g]));
#pragma unroll
                for (int kk = 0; kk < D / UMMA_K; ++kk) {
                    const uint32_t ao = ((kk / 4) * (BM * 128) + (kk % 4) * 32) >> 4, bo = ((kk / 4) * 8192 + (kk % 4) * 32) >> 4;
                    umma_lo(tmem_base + s * 128, ql + ao, kl + bo, idesc_s, kk > 0 ? 1u : 0u, issue);
                }
#pragma unroll
                for (int kk = 0; kk < D / UMMA_K; ++kk) {
                    const uint32_t ao = ((kk / 4) * (BM * 128) + (kk % 4) * 32) >> 4, bo = ((kk / 4) * 8192 + (kk % 4) * 32) >> 4;
                    umma_lo(tmem_base + s * 128 + 64, gl + ao, vl + bo, idesc_s, kk > 0 ? 1u : 0u, issue);
                }
                umma_commit_if(&sm.s_full[s], issue);
                return true;
            };
            if (ok) ok = issue_sd(0);
            for (int j = 0; ok && j < n_it; ++j) {
                if (j + 1 < n_it) { ok = issue_sd(j + 1); if (!ok) break; }
                const int s = j % NST;
                if (!mbar_wait_suspend(&sm.p_ready, j & 1, abort_flag, err, 0x4400)) break;
                tc_fence_after();
                const uint32_t pl = desc_lo<false>(s32(sm.p)), kl = desc_lo<true>(s32(sm.st0[s]));
#pragma unroll
                for (int kk = 0; kk < BT / UMMA_K; ++kk)
                    umma_lo(tmem_base + ACC_COL, pl + kk * 2, kl + kk * 128, idesc_a, (j > 0 || kk > 0) ? 1u : 0u, issue);
                umma_commit_if(&sm.st_empty[s], issue);
                umma_commit_if(&sm.acc_done, issue);
            }
        }
    } else if (warp >= 4) {
        const int qd = warp & 3, part = (warp - 4) >> 2;
        const int r = qd * 32 + lane;
        const int row = q0 + r;
        const int qi = a.q_offset + row;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
        const float sc = a.scale * LOG2E;
        constexpr int CW = BT / SPLIT;                           // 16 keys per thread
        const long long stat = ((long long)b * a.Hq + h) * a.Tq + row;
        const float lse2 = row < a.Tq ? a.lse[stat] * LOG2E : INFINITY;
        const float dl = row < a.Tq ? a.delta[stat] : 0.f;
        uint8_t* prow = sm.p + (r >> 3) * 1024 + (r & 7) * 128;
        bool alive = n_it > 0;
        for (int j = 0; alive && j < n_it; ++j) {
            const int s = j & 1;
            const int key0 = (nb_lo + j) * BT + part * CW;
            if (!mbar_wait_suspend(&sm.s_full[s], (j >> 1) & 1, abort_flag, err, 0x4500 | s)) { alive = false; break; }
            tc_fence_after();
            uint32_t sv[CW], dv[CW];
            tmem_ld16(lane_addr + s * 128 + part * CW, sv);
            tmem_ld16(lane_addr + s * 128 + 64 + part * CW, dv);
            tmem_ld_wait();
            // masking is needed only on tiles that cross the causal diagonal, the window edge or the key length
            const int tile_key0 = (nb_lo + j) * BT;
            const bool need_mask = (tile_key0 + BT - 1 > a.q_offset + q0) || (tile_key0 + BT > a.Tk) ||
                                   (a.window > 0 && tile_key0 <= a.q_offset + q0 + BM - 1 - a.window);
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < CW; ++i)
                    if (!visible(key0 + i, qi, a.Tk, a.window)) sv[i] = 0xff800000u;      // -inf -> p = 0
            }
            uint32_t pk[CW / 2];
#pragma unroll
            for (int i = 0; i < CW; i += 2) {
                const float p0 = exp2f(fmaf(__uint_as_float(sv[i]), sc, -lse2)), p1 = exp2f(fmaf(__uint_as_float(sv[i + 1]), sc, -lse2));
                pk[i >> 1] = pack_bf16(p0 * (__uint_as_float(dv[i]) - dl), p1 * (__uint_as_float(dv[i + 1]) - dl));   // the softmax scale is applied to dQ at the end
            }
            if (j > 0 && !mbar_wait_suspend(&sm.acc_done, (j - 1) & 1, abort_flag, err, 0x4600)) { alive = false; break; }
            *reinterpret_cast<uint4*>(prow + (((part * 2) ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            *reinterpret_cast<uint4*>(prow + (((part * 2 + 1) ^ (r & 7)) << 4)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            tc_fence_before();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.p_ready);
        }
        constexpr int OW = D / SPLIT;
        uint32_t acc[OW];
#pragma unroll
        for (int i = 0; i < OW; ++i) acc[i] = 0u;
        if (alive && n_it > 0 && mbar_wait_suspend(&sm.acc_done, (n_it - 1) & 1, abort_flag, err, 0x4700)) {
            tc_fence_after();
            tmem_ld<OW>(lane_addr + ACC_COL + part * OW, acc);
            tmem_ld_wait();
        }
        if (row < a.Tq) {
            bf16* og = a.dq + (((long long)b * a.Tq + row) * a.Hq + h) * D + part * OW;
#pragma unroll
            for (int c = 0; c < OW; c += 8)
                *reinterpret_cast<uint4*>(og + c) = make_uint4(pack_bf16(a.scale * __uint_as_float(acc[c]), a.scale * __uint_as_float(acc[c + 1])),
                                                               pack_bf16(a.scale * __uint_as_float(acc[c + 2]), a.scale * __uint_as_float(acc[c + 3])),
                                                               pack_bf16(a.scale * __uint_as_float(acc[c + 4]), a.scale * __uint_as_float(acc[c + 5])),
                                                               pack_bf16(a.scale * __uint_as_float(acc[c + 6]), a.scale * __uint_as_float(acc[c + 7])));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}


template <int D>
__global__ void __launch_bounds__(THREADS, 1)
fa_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmG,
                     const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, BwdArgs a) {
    extern __shared__ uint8_t smem_raw[];
    SmemBwd<D>& sm = *reinterpret_cast<SmemBwd<D>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int DK = D / 64;
    constexpr uint32_t TMEM_COLS = 512, DV_COL = 256, DK_COL = 256 + D;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kb_tile = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
    const int rep = a.Hq / a.Hkv;
    const int k0 = kb_tile * BM;
    volatile int* abort_flag = &sm.abort_flag;
    int* err = a.err;
    // query tiles (of 64) that can see a key of this tile: q >= k0 - q_offset, and with a window q < k0 + 127 + window - q_offset
    const int i_lo = max(0, k0 - a.q_offset) / BT;
    int q_end = a.Tq;
    if (a.window > 0) q_end = min(a.Tq, max(0, k0 + BM - 1 + a.window - a.q_offset));
    const int i_hi = (q_end + BT - 1) / BT;
    const int ni = max(i_hi - i_lo, 0);
    const int n_it = ni * rep;

    if (threadIdx.x == 0) {
        mbar_init(&sm.big_full, 1);
        for (int s = 0; s < NST; ++s) { mbar_init(&sm.st_full[s], 1); mbar_init(&sm.st_empty[s], 1); }
        for (int s = 0; s < 2; ++s) mbar_init(&sm.s_full[s], 1);
        mbar_init(&sm.p_ready, 4 * SPLIT);
        mbar_init(&sm.acc_done, 1);
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
            mbar_expect_tx(&sm.big_full, 2 * BM * D * 2);
#pragma unroll
            for (int kb = 0; kb < DK; ++kb) {
                tma_load_4d(sm.big0 + kb * BM * 128, &tmK, &sm.big_full, kb * 64, hk, k0, b);
                tma_load_4d(sm.big1 + kb * BM * 128, &tmV, &sm.big_full, kb * 64, hk, k0, b);
            }
            for (int it = 0; it < n_it; ++it) {
                const int s = it % NST;
                const int h = hk * rep + it / ni, q0 = (i_lo + it % ni) * BT;
                if (!mbar_wait_suspend(&sm.st_empty[s], ((it / NST) & 1) ^ 1, abort_flag, err, 0x5100 | s)) break;
                mbar_expect_tx(&sm.st_full[s], 2 * BT * D * 2);
#pragma unroll
                for (int kb = 0; kb < DK; ++kb) {
                    tma_load_4d(sm.st0[s] + kb * 8192, &tmQ, &sm.st_full[s], kb * 64, h, q0, b);
                    tma_load_4d(sm.st1[s] + kb * 8192, &tmG, &sm.st_full[s], kb * 64, h, q0, b);
                }
            }
        }
    } else if (warp == 1) {
        if (n_it > 0) {
            const uint32_t issue = lane == 0 ? 1u : 0u;
            constexpr uint32_t idesc_s = idesc_bf16<false, BT>();       // [128 keys] x [64 queries], both K-major
            constexpr uint32_t idesc_a = idesc_bf16<true, D>();         // B = dO / Q tile read MN-major
            bool ok = mbar_wait_suspend(&sm.big_full, 0, abort_flag, err, 0x5200);
            auto issue_sd = [&](int it) -> bool {
                const int s = it & 1, g = it % NST;                  // tensor-memory buffer, shared-memory stage
                if (!mbar_wait_suspend(&sm.st_full[g], (it / NST) & 1, abort_flag, err, 0x5300 | g)) return false;
                tc_fence_after();
                const uint32_t kl = desc_lo<false>(s32(sm.big0)), vl = desc_lo<false>(s32(sm.big1));
                const uint32_t ql = desc_lo<false>(s32(sm.st0[g])), gl = desc_lo<false>(s32(sm.st1[g]));
#pragma unroll
                for (int kk = 0; kk < D / UMMA_K; ++kk) {
                    const uint32_t ao = ((kk / 4) * (BM * 128) + (kk % 4) * 32) >> 4, bo = ((kk / 4) * 8192 + (kk % 4) * 32) >> 4;
                    umma_lo(tmem_base + s * 128, kl + ao, ql + bo, idesc_s, kk > 0 ? 1u : 0u, issue);
                }
#pragma unroll
                for (int kk = 0; kk < D / UMMA_K; ++kk) {
                    const uint32_t ao = ((kk / 4) * (BM * 128) + (kk % 4) * 32) >> 4, bo = ((kk / 4) * 8192 + (kk % 4) * 32) >> 4;
                    umma_lo(tmem_base + s * 128 + 64, vl + ao, gl + bo, idesc_s, kk > 0 ? 1u : 0u, issue);
                }
                umma_commit_if(&sm.s_full[s], issue);
                return true;
            };
            if (ok) ok = issue_sd(0);
            for (int it = 0; ok && it < n_it; ++it) {
                if (it + 1 < n_it) { ok = issue_sd(it + 1); if (!ok) break; }
                const int s = it % NST;
                if (!mbar_wait_suspend(&sm.p_ready, it & 1, abort_flag, err, 0x5400)) break;
                tc_fence_after();
                const uint32_t pl = desc_lo<false>(s32(sm.p)), dl_ = desc_lo<false>(s32(sm.ds));
                const uint32_t ql = desc_lo<true>(s32(sm.st0[s])), gl = desc_lo<true>(s32(sm.st1[s]));
#pragma unroll
                for (int kk = 0; kk < BT / UMMA_K; ++kk)        // dV += P^T dO
                    umma_lo(tmem_base + DV_COL, pl + kk * 2, gl + kk * 128, idesc_a, (it > 0 || kk > 0) ? 1u : 0u, issue);
#pragma unroll
                for (int kk = 0; kk < BT / UMMA_K; ++kk)        // dK += dS^T Q
                    umma_lo(tmem_base + DK_COL, dl_ + kk * 2, ql + kk * 128, idesc_a, (it > 0 || kk > 0) ? 1u : 0u, issue);
                umma_commit_if(&sm.st_empty[s], issue);
                umma_commit_if(&sm.acc_done, issue);
            }
        }
    } else if (warp >= 4) {
        const int qd = warp & 3, part = (warp - 4) >> 2;
        const int r = qd * 32 + lane;                            // key row inside the tile
        const int key = k0 + r;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(qd * 32) << 16);
        const float sc = a.scale * LOG2E;
        constexpr int CW = BT / SPLIT;                           // 16 queries per thread
        uint8_t* prow = sm.p + (r >> 3) * 1024 + (r & 7) * 128;
        uint8_t* drow = sm.ds + (r >> 3) * 1024 + (r & 7) * 128;
        bool alive = n_it > 0;
        for (int it = 0; alive && it < n_it; ++it) {
            const int s = it & 1;
            const int h = hk * rep + it / ni;
            const int qbase = (i_lo + it % ni) * BT + part * CW;     // first query of this thread's columns
            const float* lse_p = a.lse + ((long long)b * a.Hq + h) * a.Tq;
            const float* del_p = a.delta + ((long long)b * a.Hq + h) * a.Tq;
            float l2[CW], dl[CW];
            if ((a.Tq & 3) == 0 && qbase + CW <= a.Tq) {          // 16-byte aligned rows of lse / delta: 4 + 4 vector loads
#pragma unroll
                for (int i = 0; i < CW; i += 4) {
                    const float4 x = __ldg(reinterpret_cast<const float4*>(lse_p + qbase + i));
                    const float4 y = __ldg(reinterpret_cast<const float4*>(del_p + qbase + i));
                    l2[i] = x.x * LOG2E; l2[i + 1] = x.y * LOG2E; l2[i + 2] = x.z * LOG2E; l2[i + 3] = x.w * LOG2E;
                    dl[i] = y.x; dl[i + 1] = y.y; dl[i + 2] = y.z; dl[i + 3] = y.w;
                }
            } else {
#pragma unroll
                for (int i = 0; i < CW; ++i) {
                    const int q = qbase + i;
                    l2[i] = q < a.Tq ? __ldg(lse_p + q) * LOG2E : INFINITY;
                    dl[i] = q < a.Tq ? __ldg(del_p + q) : 0.f;
                }
            }
            if (!mbar_wait_suspend(&sm.s_full[s], (it >> 1) & 1, abort_flag, err, 0x5500 | s)) { alive = false; break; }
            tc_fence_after();
            uint32_t sv[CW], dv[CW];
            tmem_ld16(lane_addr + s * 128 + part * CW, sv);
            tmem_ld16(lane_addr + s * 128 + 64 + part * CW, dv);
            tmem_ld_wait();
            const int tile_q0 = (i_lo + it % ni) * BT;
            const bool need_mask = (k0 + BM - 1 > a.q_offset + tile_q0) || (k0 + BM > a.Tk) ||
                                   (a.window > 0 && k0 <= a.q_offset + tile_q0 + BT - 1 - a.window);
            if (need_mask) {
#pragma unroll
                for (int i = 0; i < CW; ++i)
                    if (!visible(key, a.q_offset + qbase + i, a.Tk, a.window)) sv[i] = 0xff800000u;
            }
            uint32_t pk[CW / 2], dk2[CW / 2];
#pragma unroll
            for (int i = 0; i < CW; i += 2) {
                const float p0 = exp2f(fmaf(__uint_as_float(sv[i]), sc, -l2[i])), p1 = exp2f(fmaf(__uint_as_float(sv[i + 1]), sc, -l2[i + 1]));
                pk[i >> 1] = pack_bf16(p0, p1);
                dk2[i >> 1] = pack_bf16(p0 * (__uint_as_float(dv[i]) - dl[i]), p1 * (__uint_as_float(dv[i + 1]) - dl[i + 1]));   // scale applied to dK at the end
            }
            if (it > 0 && !mbar_wait_suspend(&sm.acc_done, (it - 1) & 1, abort_flag, err, 0x5600)) { alive = false; break; }
            const int c0 = ((part * 2) ^ (r & 7)) << 4, c1 = ((part * 2 + 1) ^ (r & 7)) << 4;
            *reinterpret_cast<uint4*>(prow + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            *reinterpret_cast<uint4*>(prow + c1) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            *reinterpret_cast<uint4*>(drow + c0) = make_uint4(dk2[0], dk2[1], dk2[2], dk2[3]);
            *reinterpret_cast<uint4*>(drow + c1) = make_uint4(dk2[4], dk2[5], dk2[6], dk2[7]);
            tc_fence_before();
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.p_ready);
        }
        constexpr int OW = D / SPLIT;
        uint32_t av[OW], ak[OW];
#pragma unroll
        for (int i = 0; i < OW; ++i) { av[i] = 0u; ak[i] = 0u; }
        if (alive && n_it > 0 && mbar_wait_suspend(&sm.acc_done, (n_it - 1) & 1, abort_flag, err, 0x5700)) {
            tc_fence_after();
            tmem_ld<OW>(lane_addr + DV_COL + part * OW, av);
            tmem_ld<OW>(lane_addr + DK_COL + part * OW, ak);
            tmem_ld_wait();
        }
        if (key < a.Tk) {
            const long long off = (((long long)b * a.Tk + key) * a.Hkv + hk) * D + part * OW;
#pragma unroll
            for (int c = 0; c < OW; c += 8) {
                *reinterpret_cast<uint4*>(a.dv + off + c) = make_uint4(pack_bf16(__uint_as_float(av[c]), __uint_as_float(av[c + 1])),
                                                                       pack_bf16(__uint_as_float(av[c + 2]), __uint_as_float(av[c + 3])),
                                                                       pack_bf16(__uint_as_float(av[c + 4]), __uint_as_float(av[c + 5])),
                                                                       pack_bf16(__uint_as_float(av[c + 6]), __uint_as_float(av[c + 7])));
                *reinterpret_cast<uint4*>(a.dk + off + c) = make_uint4(pack_bf16(a.scale * __uint_as_float(ak[c]), a.scale * __uint_as_float(ak[c + 1])),
                                                                       pack_bf16(a.scale * __uint_as_float(ak[c + 2]), a.scale * __uint_as_float(ak[c + 3])),
                                                                       pack_bf16(a.scale * __uint_as_float(ak[c + 4]), a.scale * __uint_as_float(ak[c + 5])),
                                                                       pack_bf16(a.scale * __uint_as_float(ak[c + 6]), a.scale * __uint_as_float(ak[c + 7])));
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// delta[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]; one warp per (b,t,h)
template <int D>
__global__ void fa_delta_tc_kernel(const bf16* __restrict__ o, const bf16* __restrict__ d_o, float* __restrict__ delta, int B, int Tq, int Hq) {
    const int l = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= (long long)B * Tq * Hq) return;
    const int h = row % Hq;
    const long long bt = row / Hq;
    const int t = bt % Tq, b = bt / Tq;
    float s = 0.f;
    for (int c = l * 2; c < D; c += 64) {
        const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + row * D + c));
        const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(d_o + row * D + c));
        s += x.x * y.x + x.y * y.y;
    }
    s = warp_sum(s);
    if (l == 0) delta[((long long)b * Hq + h) * Tq + t] = s;
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
    if (r != CUDA_SUCCESS)
        fprintf(stderr, "flash_attn_tc: tensor map rejected (CUresult %d): ptr %p dims {%d,%d,%d,%d} strides {%lld,%lld,%lld} box_t %u\n",
                (int)r, ptr, D, H, T, B, sh, st, sb, box_t);
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

template <int D>
static int launch_bwd_tc(const CUtensorMap& q128, const CUtensorMap& g128, const CUtensorMap& k64, const CUtensorMap& v64,
                         const CUtensorMap& q64, const CUtensorMap& g64, const CUtensorMap& k128, const CUtensorMap& v128,
                         const BwdArgs& a, const bf16* o, const bf16* d_o, float* delta, cudaStream_t st) {
    const long long rows = (long long)a.B * a.Tq * a.Hq;
    fa_delta_tc_kernel<D><<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(o, d_o, delta, a.B, a.Tq, a.Hq);
    const size_t smem = sizeof(SmemBwd<D>) + 1024;
    cudaFuncSetAttribute(fa_bwd_dq_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(fa_bwd_dkv_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    fa_bwd_dq_tc_kernel<D><<<dim3((a.Tq + BM - 1) / BM, a.Hq, a.B), THREADS, smem, st>>>(q128, g128, k64, v64, a);
    fa_bwd_dkv_tc_kernel<D><<<dim3((a.Tk + BM - 1) / BM, a.Hkv, a.B), THREADS, smem, st>>>(q64, g64, k128, v128, a);
    return (int)cudaGetLastError();
}

// Backward of lmoe_flash_attn_fwd_tc.  o, d_o: contiguous [B,Tq,Hq,D]; ap->delta is scratch [B,Hq,Tq]; writes dq, dk, dv.
LMOE_API int lmoe_flash_attn_bwd_tc(const void* q, const long long* qs, const void* k, const long long* ks, const void* v,
                                    const long long* vs, const void* o, const void* d_o, float* delta, const BwdArgs* ap, int D,
                                    cudaStream_t st) {
    BwdArgs a = *ap;
    a.delta = delta;
    const long long gs[3] = {(long long)a.Tq * a.Hq * D, (long long)a.Hq * D, (long long)D};
    CUtensorMap q128, g128, k64, v64, q64, g64, k128, v128;
    int rc = 0;
    rc |= make_map_4d(&q128, q, a.B, a.Tq, a.Hq, D, qs[0], qs[1], qs[2], BM);
    rc |= make_map_4d(&g128, d_o, a.B, a.Tq, a.Hq, D, gs[0], gs[1], gs[2], BM);
    rc |= make_map_4d(&k64, k, a.B, a.Tk, a.Hkv, D, ks[0], ks[1], ks[2], BT);
    rc |= make_map_4d(&v64, v, a.B, a.Tk, a.Hkv, D, vs[0], vs[1], vs[2], BT);
    rc |= make_map_4d(&q64, q, a.B, a.Tq, a.Hq, D, qs[0], qs[1], qs[2], BT);
    rc |= make_map_4d(&g64, d_o, a.B, a.Tq, a.Hq, D, gs[0], gs[1], gs[2], BT);
    rc |= make_map_4d(&k128, k, a.B, a.Tk, a.Hkv, D, ks[0], ks[1], ks[2], BM);
    rc |= make_map_4d(&v128, v, a.B, a.Tk, a.Hkv, D, vs[0], vs[1], vs[2], BM);
    if (rc) return -11;
    if (D == 128) return launch_bwd_tc<128>(q128, g128, k64, v64, q64, g64, k128, v128, a, (const bf16*)o, (const bf16*)d_o, delta, st);
    if (D == 64) return launch_bwd_tc<64>(q128, g128, k64, v64, q64, g64, k128, v128, a, (const bf16*)o, (const bf16*)d_o, delta, st);
    return -1;
}
