// Grouped (per-expert) bf16 GEMMs on tcgen05 / TMA / TMEM, with K-major or MN-major operands.
//
// Expert-sorted tokens live in one padded buffer: expert e owns rows [offs[e], offs[e+1]) and every offset is a
// multiple of 128, so no tile straddles two experts.  `offs` stays on the device: the tile list is decoded by the
// kernel, there is no host synchronisation (the reference's grouped path needs the per-expert counts on the host,
// qwen2/moe/token_dispatcher.py:363-386, and runs CUTLASS sm80 grouped GEMM through grouped_gemm.ops.gmm,
// qwen2/moe/experts.py:156-168).
//
//   mode 1 (grouped along M), B K-major :  C[rows_e, N] = A[rows_e, K] * W[e][N, K]^T      forward  (x W^T)
//   mode 1 (grouped along M), B MN-major:  C[rows_e, N] = A[rows_e, K] * W[e][K, N]        dgrad    (dy W)
//   mode 2 (grouped along K), A,B MN-major: C[e][M, N]  = A[rows_e, M]^T * B[rows_e, N]    wgrad    (dy^T x)
//   mode 0: one dense problem with the same operand layouts.
//
// Operand tiles in shared memory (128-byte swizzle, filled by non-multicast TMA):
//   K-major  tile [R rows x 64 k]: one box {64 k, R rows}; descriptor SBO = 1024 B, k-step of 16 = +32 B
//   MN-major tile [64 k x R mn]  : R/64 boxes {64 mn, 64 k} of 8 KiB each; descriptor LBO = 8192 B (next 64 mn),
//                                  SBO = 1024 B (next 8 k), k-step of 16 = +2048 B; instruction-descriptor major bit set
// Warp roles, pipeline and bounded waits are those of gemm_tcgen05.cu.
#include "tcgen05_utils.cuh"

namespace lmoe {
namespace gg {
using namespace lmoe::tc;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;

struct __align__(1024) Smem {
    uint8_t tiles[STAGES][STAGE_BYTES];
    uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

struct Params {
    int mode;                 // 0 dense, 1 grouped along M, 2 grouped along K
    int M, N, K;              // dense sizes; mode 1: N, K per expert (M from offs); mode 2: M, N per expert (K from offs)
    int ldc;
    int num_groups;
    const int* offs;          // [num_groups + 1] row offsets, multiples of 128
    long long c_group_stride; // mode 2: elements between consecutive experts' outputs
    int b_group_rows;         // mode 1: rows of the B map per expert (N if B is K-major, K if MN-major)
    int* err;
    int out_f32;              // pair kernel: C is fp32 (weight gradients straight into the fp32 accumulators)
    int accumulate;           // with out_f32: C += result instead of C = result
};


// One output tile of the (possibly grouped) problem.
struct Tile {
    int a_row;      // K-major A: first row of the A tile.  MN-major A: first mn column
    int b_row;      // K-major B: first row of the B tile (in the B map).  MN-major B: first mn column
    int a_k0, b_k0; // first k coordinate in the A / B maps
    int kblocks;
    long long c_off;  // element offset of C(tile row 0, tile col 0)
    int rows_valid, cols_valid;
};

// `bm` = rows of one output tile: 128 for one CTA, 256 for a CTA pair
__device__ __forceinline__ bool decode_tile(const Params& p, int t, Tile& o, const int bm = BM) {
    const int tiles_n = (p.N + BN - 1) / BN;
    if (p.mode == 0) {
        const int tiles_m = (p.M + bm - 1) / bm;
        if (t >= tiles_m * tiles_n) return false;
        const int tm = t % tiles_m, tn = t / tiles_m;
        o.a_row = tm * bm; o.b_row = tn * BN; o.a_k0 = 0; o.b_k0 = 0;
        o.kblocks = (p.K + BK - 1) / BK;
        o.c_off = (long long)tm * bm * p.ldc + (long long)tn * BN;
        o.rows_valid = p.M - tm * bm; o.cols_valid = p.N - tn * BN;
        return true;
    }
    if (p.mode == 1) {
        int base = 0;
        for (int e = 0; e < p.num_groups; ++e) {
            const int r0 = p.offs[e], r1 = p.offs[e + 1];
            const int tm_e = (r1 - r0) / bm;
            const int n_e = tm_e * tiles_n;
            if (t < base + n_e) {
                const int lt = t - base;
                const int tm = lt % tm_e, tn = lt / tm_e;
                o.a_row = r0 + tm * bm;
                o.a_k0 = 0;
                // B map: K-major -> rows [e*N + tn*BN), k from 0.  MN-major -> mn column tn*BN, k rows from e*K
                o.b_row = tn * BN;
                o.b_k0 = e * p.b_group_rows;              // used as a row offset (K-major: added to b_row) or k offset (MN-major)
                o.kblocks = (p.K + BK - 1) / BK;
                o.c_off = (long long)(r0 + tm * bm) * p.ldc + (long long)tn * BN;
                o.rows_valid = bm; o.cols_valid = p.N - tn * BN;
                return true;
            }
            base += n_e;
        }
        return false;
    }
    // mode 2: per expert an (M x N) output, K = the expert's rows
    const int tiles_m = (p.M + bm - 1) / bm;
    const int per = tiles_m * tiles_n;
    const int e = t / per;
    if (e >= p.num_groups) return false;
    const int lt = t - e * per;
    const int tm = lt % tiles_m, tn = lt / tiles_m;
    const int r0 = p.offs[e], r1 = p.offs[e + 1];
    o.a_row = tm * bm; o.b_row = tn * BN; o.a_k0 = r0; o.b_k0 = r0;
    o.kblocks = (r1 - r0) / BK;
    o.c_off = (long long)e * p.c_group_stride + (long long)tm * bm * p.ldc + (long long)tn * BN;
    o.rows_valid = p.M - tm * bm; o.cols_valid = p.N - tn * BN;
    return true;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, bf16* __restrict__ C, Params p) {
    extern __shared__ uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &sm.abort_flag;
    int* err = p.err;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sm.tmem_full[b], 1); mbar_init(&sm.tmem_empty[b], 4); }
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
        if (lane == 0) {
            int it = 0;
            Tile t;
            for (int tile = blockIdx.x; !*abort_flag && decode_tile(p, tile, t); tile += gridDim.x) {
                for (int kb = 0; kb < t.kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&sm.empty[s], ph ^ 1, abort_flag, err, 0x100 | s)) goto producer_done;
                    mbar_expect_tx(&sm.full[s], STAGE_BYTES);
                    uint8_t* sa = sm.tiles[s];
                    uint8_t* sb = sa + A_BYTES;
                    if (!A_MN) {
                        tma_load_2d(sa, &tmA, &sm.full[s], t.a_k0 + kb * BK, t.a_row);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j)
                            tma_load_2d(sa + j * 8192, &tmA, &sm.full[s], t.a_row + j * 64, t.a_k0 + kb * BK);
                    }
                    if (!B_MN) {
                        const int brow = t.b_row + (p.mode == 1 ? t.b_k0 : 0);
                        tma_load_2d(sb, &tmB, &sm.full[s], (p.mode == 1 ? 0 : t.b_k0) + kb * BK, brow);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(sb + j * 8192, &tmB, &sm.full[s], t.b_row + j * 64, t.b_k0 + kb * BK);
                    }
                }
            }
        }
    producer_done:;
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc<A_MN, B_MN, BM, BN>();
            int it = 0, lt = 0;
            Tile t;
            for (int tile = blockIdx.x; !*abort_flag && decode_tile(p, tile, t); tile += gridDim.x, ++lt) {
                const int buf = lt & 1;
                const uint32_t aph = (lt >> 1) & 1;
                if (!mbar_wait(&sm.tmem_empty[buf], aph ^ 1, abort_flag, err, 0x200 | buf)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                bool dead = false;
                for (int kb = 0; kb < t.kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&sm.full[s], ph, abort_flag, err, 0x300 | s)) { dead = true; break; }
                    tc_fence_after();
                    const uint32_t a_addr = s32(sm.tiles[s]), b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t ad = make_desc<A_MN>(a_addr + (A_MN ? k * 2048 : k * UMMA_K * 2));
                        const uint64_t bd = make_desc<B_MN>(b_addr + (B_MN ? k * 2048 : k * UMMA_K * 2));
                        umma_f16(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&sm.empty[s]);
                }
                if (dead) break;
                umma_commit(&sm.tmem_full[buf]);
            }
        }
    } else {
        const int q = warp & 3;
        int lt = 0;
        Tile t;
        for (int tile = blockIdx.x; decode_tile(p, tile, t); tile += gridDim.x, ++lt) {
            const int buf = lt & 1;
            const uint32_t aph = (lt >> 1) & 1;
            if (!mbar_wait(&sm.tmem_full[buf], aph, abort_flag, err, 0x400 | buf)) break;
            tc_fence_after();
            const int r = q * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            bf16* crow = C + t.c_off + (long long)r * p.ldc;
            const bool zero = t.kblocks == 0;            // an expert without tokens: its weight gradient is zero
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t v[32];
                tmem_ld32(taddr + c, v);
                tmem_ld_wait();
                if (r < t.rows_valid) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const int col = c + g * 8;
                        if (col + 8 <= t.cols_valid) {
                            uint4 o;
                            if (zero) o = make_uint4(0, 0, 0, 0);
                            else {
                                o.x = pack_bf16(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]));
                                o.y = pack_bf16(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
                                o.z = pack_bf16(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
                                o.w = pack_bf16(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
                            }
                            *reinterpret_cast<uint4*>(crow + col) = o;
                        } else {
                            for (int e = 0; e < 8; ++e)
                                if (col + e < t.cols_valid) crow[col + e] = __float2bfloat16(zero ? 0.f : __uint_as_float(v[g * 8 + e]));
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.tmem_empty[buf]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}


template <bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, bf16* C, const Params& p, int grid, cudaStream_t st) {
    const size_t smem = sizeof(Smem) + 1024;
    cudaFuncSetAttribute(gemm_grouped_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gemm_grouped_kernel<A_MN, B_MN><<<grid, THREADS, smem, st>>>(ma, mb, C, p);
    return (int)cudaGetLastError();
}


// ---------------------------------------------------------------------------------------------------------------
// CTA-pair variant: tcgen05.mma.cta_group::2 on 256-row tiles (expert offsets must then be multiples of 256).  Each
// CTA of the pair stages its own 128 rows (or 128 mn columns) of A and of B, the leader issues M = 256, N = 256 MMAs,
// both CTAs drain their half of the accumulator.  Same protocol as gemm_2cta.cu.
// ---------------------------------------------------------------------------------------------------------------
constexpr int P_STAGES = 6, P_A_BYTES = 128 * BK * 2, P_B_BYTES = 128 * BK * 2, P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
struct __align__(1024) SmemPair {
    uint8_t tiles[P_STAGES][P_STAGE_BYTES];
    uint8_t stage_out[4][32 * 128];            // epilogue staging, one per epilogue warp
    uint64_t full[P_STAGES], empty[P_STAGES], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_grouped_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, bf16* __restrict__ C, Params p) {
    extern __shared__ uint8_t smem_raw[];
    SmemPair& sm = *reinterpret_cast<SmemPair*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    volatile int* abort_flag = &sm.abort_flag;
    int* err = p.err;

    if (threadIdx.x == 0) {
        for (int s = 0; s < P_STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sm.tmem_full[b], 1); mbar_init(&sm.tmem_empty[b], 8); }
        sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(s32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    tc_fence_after();
    const uint32_t tmem_base = sm.tmem_base;
    const int half = (int)rank * 128;                        // this CTA's rows of A (M) and of B (N) inside the pair tile

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            Tile t;
            for (int tile = pair; !*abort_flag && decode_tile(p, tile, t, 256); tile += num_pairs) {
                for (int kb = 0; kb < t.kblocks; ++kb, ++it) {
                    const int s = it % P_STAGES;
                    const uint32_t ph = (it / P_STAGES) & 1;
                    if (!mbar_wait(&sm.empty[s], ph ^ 1, abort_flag, err, 0x6100 | s)) goto producer_done;
                    if (rank == 0) mbar_expect_tx(&sm.full[s], 2 * P_STAGE_BYTES);
                    const uint32_t fl = map_to_cta(&sm.full[s], 0);
                    uint8_t* sa = sm.tiles[s];
                    uint8_t* sb = sa + P_A_BYTES;
                    if (!A_MN) {
                        tma_load_2d_pair(sa, &tmA, fl, t.a_k0 + kb * BK, t.a_row + half);
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j) tma_load_2d_pair(sa + j * 8192, &tmA, fl, t.a_row + half + j * 64, t.a_k0 + kb * BK);
                    }
                    if (!B_MN) {
                        const int brow = t.b_row + half + (p.mode == 1 ? t.b_k0 : 0);
                        tma_load_2d_pair(sb, &tmB, fl, (p.mode == 1 ? 0 : t.b_k0) + kb * BK, brow);
                    } else {
#pragma unroll
                        for (int j = 0; j < 2; ++j) tma_load_2d_pair(sb + j * 8192, &tmB, fl, t.b_row + half + j * 64, t.b_k0 + kb * BK);
                    }
                }
            }
        }
    producer_done:;
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                                       ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            int it = 0, lt = 0;
            Tile t;
            for (int tile = pair; !*abort_flag && decode_tile(p, tile, t, 256); tile += num_pairs, ++lt) {
                const int buf = lt & 1;
                const uint32_t aph = (lt >> 1) & 1;
                if (!mbar_wait(&sm.tmem_empty[buf], aph ^ 1, abort_flag, err, 0x6200 | buf)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                bool dead = false;
                for (int kb = 0; kb < t.kblocks; ++kb, ++it) {
                    const int s = it % P_STAGES;
                    const uint32_t ph = (it / P_STAGES) & 1;
                    if (!mbar_wait(&sm.full[s], ph, abort_flag, err, 0x6300 | s)) { dead = true; break; }
                    tc_fence_after();
                    const uint32_t a_addr = s32(sm.tiles[s]), b_addr = a_addr + P_A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t ad = make_desc<A_MN>(a_addr + (A_MN ? k * 2048 : k * UMMA_K * 2));
                        const uint64_t bd = make_desc<B_MN>(b_addr + (B_MN ? k * 2048 : k * UMMA_K * 2));
                        umma_pair<false>(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(&sm.empty[s]);
                }
                if (dead) break;
                umma_commit_pair(&sm.tmem_full[buf]);              // also for kblocks == 0: completes at once
            }
        }
    } else {
        const int q = warp & 3;
        int lt = 0;
        Tile t;
        for (int tile = pair; decode_tile(p, tile, t, 256); tile += num_pairs, ++lt) {
            const int buf = lt & 1;
            const uint32_t aph = (lt >> 1) & 1;
            if (!mbar_wait(&sm.tmem_full[buf], aph, abort_flag, err, 0x6400 | buf)) break;
            tc_fence_after();
            const int r0 = half + q * 32;                            // first of this warp's 32 rows inside the 256-row tile
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            const bool zero = t.kblocks == 0;                        // an expert without tokens: its weight gradient is zero
            uint8_t* stg = sm.stage_out[warp - 2];                   // 32 rows x 128 bytes, 16-byte chunks xor-swizzled
            if (p.out_f32) {
                // fp32 output (optionally accumulating): 32 columns = 128 bytes per row and pass through the staging buffer
                float* C32 = reinterpret_cast<float*>(C);
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t v[32];
                    tmem_ld32(taddr + c, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        uint4 o = zero ? make_uint4(0, 0, 0, 0) : make_uint4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                        *reinterpret_cast<uint4*>(stg + lane * 128 + ((g ^ (lane & 7)) << 4)) = o;
                    }
                    __syncwarp();
                    const int chunk = lane & 7;
                    const int col = c + chunk * 4;
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int rr = it * 4 + (lane >> 3);
                        float4 o = *reinterpret_cast<const float4*>(stg + rr * 128 + ((chunk ^ (rr & 7)) << 4));
                        if (r0 + rr < t.rows_valid && col + 4 <= t.cols_valid) {
                            float4* dst = reinterpret_cast<float4*>(C32 + t.c_off + (long long)(r0 + rr) * p.ldc + col);
                            if (p.accumulate) { const float4 old = *dst; o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w; }
                            *dst = o;
                        }
                    }
                    __syncwarp();
                }
            } else
#pragma unroll 1
            for (int c = 0; c < BN; c += 64) {
#pragma unroll
                for (int hc = 0; hc < 2; ++hc) {
                    uint32_t v[32];
                    tmem_ld32(taddr + c + hc * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 o;
                        if (zero) o = make_uint4(0, 0, 0, 0);
                        else {
                            o.x = pack_bf16(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]));
                            o.y = pack_bf16(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
                            o.z = pack_bf16(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
                            o.w = pack_bf16(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
                        }
                        *reinterpret_cast<uint4*>(stg + lane * 128 + (((hc * 4 + g) ^ (lane & 7)) << 4)) = o;
                    }
                }
                __syncwarp();
                // 8 lanes write one row's 128 contiguous bytes: whole lines, 4 rows per instruction
                const int chunk = lane & 7;
                const int col = c + chunk * 8;
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int rr = it * 4 + (lane >> 3);
                    const uint4 o = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((chunk ^ (rr & 7)) << 4));
                    if (r0 + rr < t.rows_valid && col + 8 <= t.cols_valid)
                        *reinterpret_cast<uint4*>(C + t.c_off + (long long)(r0 + rr) * p.ldc + col) = o;
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(&sm.tmem_empty[buf], 0));
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <bool A_MN, bool B_MN>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, bf16* C, const Params& p, int grid, cudaStream_t st) {
    const size_t smem = sizeof(SmemPair) + 1024;
    cudaFuncSetAttribute(gemm_grouped_pair_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gemm_grouped_pair_kernel<A_MN, B_MN><<<grid & ~1, THREADS, smem, st>>>(ma, mb, C, p);
    return (int)cudaGetLastError();
}

}  // namespace gg
}  // namespace lmoe

using namespace lmoe;
using namespace lmoe::gg;

// A: [a_rows, a_cols] row-major (pitch lda); B: [b_rows, b_cols] row-major (pitch ldb).
//   a_mn = 0: A is [rows, K] (K-major).   a_mn = 1: A is [K rows, M cols] (MN-major).   Same for B with N.
// mode 0: dense (M, N, K).  mode 1: grouped along M by offs (A rows), B holds num_groups matrices stacked along its rows.
// mode 2: grouped along K by offs (rows of A and B), C holds num_groups outputs c_group_stride elements apart.
// pairs != 0: CTA-pair kernel (256-row tiles; in mode 1 every offset must be a multiple of 256).
LMOE_API int lmoe_gemm_grouped(const void* A, int a_rows, int a_cols, int lda, int a_mn, const void* B, int b_rows, int b_cols,
                               int ldb, int b_mn, void* C, int ldc, int mode, int M, int N, int K, int num_groups,
                               const int* offs, long long c_group_stride, int* err, int num_sms, int pairs, int out_f32, int accumulate,
                               cudaStream_t st) {
    if (lda % 8 || ldb % 8 || ldc % 8 || a_cols % 8 || b_cols % 8 || N % 8) return -1;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, (uint64_t)a_rows, (uint64_t)a_cols, (uint64_t)lda, a_mn ? 64 : BM);
    if (rc) return rc;
    rc = make_map(&mb, B, (uint64_t)b_rows, (uint64_t)b_cols, (uint64_t)ldb, b_mn ? 64 : (pairs ? 128 : BN));
    if (rc) return rc;
    Params p;
    p.mode = mode; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.num_groups = num_groups; p.offs = offs;
    p.c_group_stride = c_group_stride; p.b_group_rows = b_mn ? K : N; p.err = err;
    p.out_f32 = out_f32; p.accumulate = accumulate;
    if (out_f32 && !pairs) return -3;
    if (pairs) {
        if (!a_mn && !b_mn) return launch_pair<false, false>(ma, mb, (bf16*)C, p, num_sms, st);
        if (!a_mn && b_mn) return launch_pair<false, true>(ma, mb, (bf16*)C, p, num_sms, st);
        if (a_mn && b_mn) return launch_pair<true, true>(ma, mb, (bf16*)C, p, num_sms, st);
        return launch_pair<true, false>(ma, mb, (bf16*)C, p, num_sms, st);
    }
    if (!a_mn && !b_mn) return launch<false, false>(ma, mb, (bf16*)C, p, num_sms, st);
    if (!a_mn && b_mn) return launch<false, true>(ma, mb, (bf16*)C, p, num_sms, st);
    if (a_mn && b_mn) return launch<true, true>(ma, mb, (bf16*)C, p, num_sms, st);
    return launch<true, false>(ma, mb, (bf16*)C, p, num_sms, st);
}
