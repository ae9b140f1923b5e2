// bf16 GEMM C[M,N] = A[M,K] * B[N,K]^T on CTA pairs: tcgen05.mma.cta_group::2 computes a 256 x 256 tile per pair of
// SMs, each CTA staging only its own 128 rows of A and its own 128 rows of B.
//
// Why pairs: the single-CTA kernel (gemm_tcgen05.cu, 128 x 256 tile) moves 96 KiB through one SM's shared memory per
// 64-wide k-block (48 KiB written by TMA, 48 KiB read by the MMA) for 512 clk of tensor work, more than the ~128 B/clk
// the shared memory delivers, and stalls at ~68 % tensor-pipe activity.  In a pair each CTA writes 32 KiB and the MMA
// reads 32 KiB per CTA for the same 512 clk: 64 KiB per SM, inside the budget.
//
// Structure per CTA (192 threads, one CTA per SM, clusters of 2 along x):
//   warp 0   TMA producer: own A rows [tm*256 + rank*128, +128) and own B rows [tn*256 + rank*128, +128) of every
//            k-block into a 6-stage ring; the loads carry .cta_group::2 and complete on the LEADER CTA's `full`
//            barrier (no multicast: every CTA fetches only what it stages itself).
//   warp 1   (leader CTA only) MMA issuer: M=256, N=256, K=16 instructions on both CTAs' operands, accumulators in
//            both CTAs' tensor memory (each holds its 128 rows x 256 columns, double buffered); tcgen05.commit with a
//            2-CTA mask releases the stage in both CTAs and publishes the accumulator to both epilogues.
//   warps 2-5  epilogue: TMEM -> registers -> bf16 -> swizzled shared-memory staging -> global stores in which 8 lanes
//            write one row's 128 contiguous bytes (whole lines; the row-per-lane stores of the single-CTA kernel
//            write 32 partial lines per instruction), then an arrive on the leader's `tmem_empty` barrier (remote
//            arrive from the peer CTA).
// Every wait is bounded by a clock64 budget; on expiry the error word is set, the CTA leaves its loops, the pair meets
// at the final cluster barrier and tensor memory is released.
#include <cooperative_groups.h>
#include "tcgen05_utils.cuh"

namespace lmoe {
namespace g2 {
using namespace lmoe::tc;

constexpr int BM = 128, BN_HALF = 128, BN = 256, BK_BYTES = 128, STAGES = 6;     // 64 bf16 or 128 e4m3 per k-block
constexpr int A_BYTES = BM * BK_BYTES, B_BYTES = BN_HALF * BK_BYTES, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;

struct __align__(1024) Smem {
    uint8_t tiles[STAGES][STAGE_BYTES];
    uint8_t stage_out[4][32 * 128];            // epilogue staging, one per epilogue warp
    uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// FP8 = false: bf16 operands.  FP8 = true: e4m3 operands, C = diag(sa) acc diag(sb) (per-row scales of A and B).
template <bool FP8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_nt_2cta_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, bf16* __restrict__ C,
                    const float* __restrict__ sa, const float* __restrict__ sb, int M, int N, int K, int ldc, int* err) {
    constexpr int BK = FP8 ? 128 : 64;                       // elements per k-block
    constexpr int UMMA_K = FP8 ? 32 : 16;                    // 32 bytes of K per instruction
    extern __shared__ uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();                    // 0 = leader of the pair
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int kblocks = (K + BK - 1) / BK;
    volatile int* abort_flag = &sm.abort_flag;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sm.tmem_full[b], 1); mbar_init(&sm.tmem_empty[b], 8); }   // 4 warps x 2 CTAs
        sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(s32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                          // both CTAs' barriers are initialised before any remote use
    tc_fence_after();
    const uint32_t tmem_base = sm.tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int tile = pair; tile < num_tiles && !*abort_flag; tile += num_pairs) {
                const int tm = tile % tiles_m, tn = tile / tiles_m;
                const int a_row = tm * 2 * BM + (int)rank * BM, b_row = tn * BN + (int)rank * BN_HALF;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&sm.empty[s], ph ^ 1, abort_flag, err, 0x5100 | s)) goto producer_done;
                    if (rank == 0) mbar_expect_tx(&sm.full[s], 2 * STAGE_BYTES);       // both CTAs' loads land on this barrier
                    const uint32_t full_leader = map_to_cta(&sm.full[s], 0);
                    tma_load_2d_pair(sm.tiles[s], &tmA, full_leader, kb * BK, a_row);
                    tma_load_2d_pair(sm.tiles[s] + A_BYTES, &tmB, full_leader, kb * BK, b_row);
                }
            }
        }
    producer_done:;
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // M = 256 (128 per CTA), N = 256, bf16 x bf16 -> fp32, both operands K-major
            constexpr uint32_t idesc = (1u << 4) | (FP8 ? 0u : ((1u << 7) | (1u << 10))) | ((uint32_t)(BN >> 3) << 17) |
                                       ((uint32_t)((2 * BM) >> 4) << 24);
            int it = 0, lt = 0;
            for (int tile = pair; tile < num_tiles && !*abort_flag; tile += num_pairs, ++lt) {
                const int buf = lt & 1;
                const uint32_t aph = (lt >> 1) & 1;
                if (!mbar_wait(&sm.tmem_empty[buf], aph ^ 1, abort_flag, err, 0x5200 | buf)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                bool dead = false;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&sm.full[s], ph, abort_flag, err, 0x5300 | s)) { dead = true; break; }
                    tc_fence_after();
                    const uint32_t a_addr = s32(sm.tiles[s]), b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_pair<FP8>(d_tmem, make_desc<false>(a_addr + k * 32), make_desc<false>(b_addr + k * 32), idesc,
                                       (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&sm.empty[s]);
                }
                if (dead) break;
                umma_commit_pair(&sm.tmem_full[buf]);
            }
        }
    } else {
        const int q = warp & 3;
        int lt = 0;
        for (int tile = pair; tile < num_tiles; tile += num_pairs, ++lt) {
            const int tm = tile % tiles_m, tn = tile / tiles_m;
            const int buf = lt & 1;
            const uint32_t aph = (lt >> 1) & 1;
            if (!mbar_wait(&sm.tmem_full[buf], aph, abort_flag, err, 0x5400 | buf)) break;
            tc_fence_after();
            const int row0 = tm * 2 * BM + (int)rank * BM + q * 32;       // first of this warp's 32 rows
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            const int cols_valid = N - tn * BN;
            const float ra = (FP8 && row0 + lane < M) ? sa[row0 + lane] : 1.f;
            uint8_t* stg = sm.stage_out[warp - 2];                         // 32 rows x 128 bytes, 16-byte chunks xor-swizzled
#pragma unroll 1
            for (int c = 0; c < BN; c += 64) {
#pragma unroll
                for (int hc = 0; hc < 2; ++hc) {
                    const int cc = c + hc * 32;
                    float4 sc[8];
                    if (FP8) {
#pragma unroll
                        for (int g = 0; g < 8; ++g)
                            sc[g] = (cc + g * 4 + 4 <= cols_valid) ? __ldg(reinterpret_cast<const float4*>(sb + tn * BN + cc + g * 4))
                                                                    : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                    uint32_t v[32];
                    tmem_ld32(taddr + cc, v);
                    tmem_ld_wait();
                    if (FP8) {
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            v[g * 4 + 0] = __float_as_uint(__uint_as_float(v[g * 4 + 0]) * ra * sc[g].x);
                            v[g * 4 + 1] = __float_as_uint(__uint_as_float(v[g * 4 + 1]) * ra * sc[g].y);
                            v[g * 4 + 2] = __float_as_uint(__uint_as_float(v[g * 4 + 2]) * ra * sc[g].z);
                            v[g * 4 + 3] = __float_as_uint(__uint_as_float(v[g * 4 + 3]) * ra * sc[g].w);
                        }
                    }
                    // this lane's row: 32 columns = 4 chunks of 16 bytes
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 o;
                        o.x = pack_bf16(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]));
                        o.y = pack_bf16(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
                        o.z = pack_bf16(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
                        o.w = pack_bf16(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
                        *reinterpret_cast<uint4*>(stg + lane * 128 + (((hc * 4 + g) ^ (lane & 7)) << 4)) = o;
                    }
                }
                __syncwarp();
                // 8 lanes write one row's 128 contiguous bytes: 4 rows per instruction, whole lines only
                const int chunk = lane & 7;
                const int col = c + chunk * 8;
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int rr = it * 4 + (lane >> 3);
                    const uint4 o = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((chunk ^ (rr & 7)) << 4));
                    if (row0 + rr < M && col + 8 <= cols_valid)
                        *reinterpret_cast<uint4*>(C + (long long)(row0 + rr) * ldc + (long long)tn * BN + col) = o;
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
    cluster_sync();                                          // nobody leaves while the peer may still signal its barriers
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

}  // namespace g2
}  // namespace lmoe

using namespace lmoe;
using namespace lmoe::g2;

static int make_map_u8(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    EncodeTiledFn enc = get_encode();
    if (enc == nullptr) return -10;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -11;
}

template <bool FP8>
static int launch_2cta(const CUtensorMap& ma, const CUtensorMap& mb, void* C, const float* sa, const float* sb, int M, int N, int K,
                       int ldc, int* err, int num_sms, cudaStream_t st) {
    const size_t smem = sizeof(Smem) + 1024;
    cudaFuncSetAttribute(gemm_nt_2cta_kernel<FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
    int pairs = num_sms / 2;
    if (tiles < pairs) pairs = tiles;
    gemm_nt_2cta_kernel<FP8><<<2 * pairs, THREADS, smem, st>>>(ma, mb, (bf16*)C, sa, sb, M, N, K, ldc, err);
    return (int)cudaGetLastError();
}

// A [M,K], B [N,K] bf16 (pitches lda, ldb), C [M,N] bf16 (pitch ldc).  K % 8 == 0, N % 8 == 0.
LMOE_API int lmoe_gemm_bf16_nt_2cta(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int* err,
                                    int num_sms, cudaStream_t st) {
    if (K % 8 || N % 8 || lda % 8 || ldb % 8 || ldc % 8) return -1;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM);
    if (rc) return rc;
    rc = make_map(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, BN_HALF);
    if (rc) return rc;
    return launch_2cta<false>(ma, mb, C, nullptr, nullptr, M, N, K, ldc, err, num_sms, st);
}

// A8 [M,K], B8 [N,K] e4m3 contiguous, sa [M], sb [N] fp32 row scales, C [M,N] bf16.  K % 16 == 0, N % 8 == 0.
LMOE_API int lmoe_gemm_fp8_nt_2cta(const void* A, const void* B, void* C, const float* sa, const float* sb, int M, int N, int K,
                                   int ldc, int* err, int num_sms, cudaStream_t st) {
    if (K % 16 || N % 8 || ldc % 8) return -1;
    CUtensorMap ma, mb;
    int rc = make_map_u8(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM);
    if (rc) return rc;
    rc = make_map_u8(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)K, BN_HALF);
    if (rc) return rc;
    return launch_2cta<true>(ma, mb, C, sa, sb, M, N, K, ldc, err, num_sms, st);
}
