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
#include <cuda.h>
#include "common.cuh"

namespace lmoe {
namespace gg {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr long long WAIT_CYCLES = 2000LL * 1000 * 1000;

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
};

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(s32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(s32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(s32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(s32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
    const long long t0 = clock64();
    for (int i = 0;; ++i) {
        if (mbar_test(bar, parity)) return true;
        if ((i & 255) == 255) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_CYCLES) break;
        }
    }
    *abort_flag = 1;
    atomicCAS(err, 0, code);
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(s32(dst)), "l"(map), "r"(s32(bar)), "r"(c0), "r"(c1) : "memory");
}
// K-major: LBO unused (1), SBO 1024 B.  MN-major: LBO 8192 B between 64-wide mn blocks, SBO 1024 B between 8-row k groups.
template <bool MN>
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)(MN ? (8192 >> 4) : 1) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
template <bool A_MN, bool B_MN>
__host__ __device__ constexpr uint32_t make_idesc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
           ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// One output tile of the (possibly grouped) problem.
struct Tile {
    int a_row;      // K-major A: first row of the A tile.  MN-major A: first mn column
    int b_row;      // K-major B: first row of the B tile (in the B map).  MN-major B: first mn column
    int a_k0, b_k0; // first k coordinate in the A / B maps
    int kblocks;
    long long c_off;  // element offset of C(tile row 0, tile col 0)
    int rows_valid, cols_valid;
};

__device__ __forceinline__ bool decode_tile(const Params& p, int t, Tile& o) {
    const int tiles_n = (p.N + BN - 1) / BN;
    if (p.mode == 0) {
        const int tiles_m = (p.M + BM - 1) / BM;
        if (t >= tiles_m * tiles_n) return false;
        const int tm = t % tiles_m, tn = t / tiles_m;
        o.a_row = tm * BM; o.b_row = tn * BN; o.a_k0 = 0; o.b_k0 = 0;
        o.kblocks = (p.K + BK - 1) / BK;
        o.c_off = (long long)tm * BM * p.ldc + (long long)tn * BN;
        o.rows_valid = p.M - tm * BM; o.cols_valid = p.N - tn * BN;
        return true;
    }
    if (p.mode == 1) {
        int base = 0;
        for (int e = 0; e < p.num_groups; ++e) {
            const int r0 = p.offs[e], r1 = p.offs[e + 1];
            const int tm_e = (r1 - r0) / BM;
            const int n_e = tm_e * tiles_n;
            if (t < base + n_e) {
                const int lt = t - base;
                const int tm = lt % tm_e, tn = lt / tm_e;
                o.a_row = r0 + tm * BM;
                o.a_k0 = 0;
                // B map: K-major -> rows [e*N + tn*BN), k from 0.  MN-major -> mn column tn*BN, k rows from e*K
                o.b_row = tn * BN;
                o.b_k0 = e * p.b_group_rows;              // used as a row offset (K-major: added to b_row) or k offset (MN-major)
                o.kblocks = (p.K + BK - 1) / BK;
                o.c_off = (long long)(r0 + tm * BM) * p.ldc + (long long)tn * BN;
                o.rows_valid = BM; o.cols_valid = p.N - tn * BN;
                return true;
            }
            base += n_e;
        }
        return false;
    }
    // mode 2: per expert an (M x N) output, K = the expert's rows
    const int tiles_m = (p.M + BM - 1) / BM;
    const int per = tiles_m * tiles_n;
    const int e = t / per;
    if (e >= p.num_groups) return false;
    const int lt = t - e * per;
    const int tm = lt % tiles_m, tn = lt / tiles_m;
    const int r0 = p.offs[e], r1 = p.offs[e + 1];
    o.a_row = tm * BM; o.b_row = tn * BN; o.a_k0 = r0; o.b_k0 = r0;
    o.kblocks = (r1 - r0) / BK;
    o.c_off = (long long)e * p.c_group_stride + (long long)tm * BM * p.ldc + (long long)tn * BN;
    o.rows_valid = p.M - tm * BM; o.cols_valid = p.N - tn * BN;
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
            constexpr uint32_t idesc = make_idesc<A_MN, B_MN>();
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}
// Row-major bf16 [rows, cols] with pitch ld; box = {64 inner, box_rows}.
static int make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    EncodeTiledFn enc = get_encode();
    if (enc == nullptr) return -10;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -11;
}

template <bool A_MN, bool B_MN>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, bf16* C, const Params& p, int grid, cudaStream_t st) {
    const size_t smem = sizeof(Smem) + 1024;
    cudaFuncSetAttribute(gemm_grouped_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    gemm_grouped_kernel<A_MN, B_MN><<<grid, THREADS, smem, st>>>(ma, mb, C, p);
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
LMOE_API int lmoe_gemm_grouped(const void* A, int a_rows, int a_cols, int lda, int a_mn, const void* B, int b_rows, int b_cols,
                               int ldb, int b_mn, void* C, int ldc, int mode, int M, int N, int K, int num_groups,
                               const int* offs, long long c_group_stride, int* err, int num_sms, cudaStream_t st) {
    if (lda % 8 || ldb % 8 || ldc % 8 || a_cols % 8 || b_cols % 8) return -1;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, (uint64_t)a_rows, (uint64_t)a_cols, (uint64_t)lda, a_mn ? 64 : BM);
    if (rc) return rc;
    rc = make_map(&mb, B, (uint64_t)b_rows, (uint64_t)b_cols, (uint64_t)ldb, b_mn ? 64 : BN);
    if (rc) return rc;
    Params p;
    p.mode = mode; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.num_groups = num_groups; p.offs = offs;
    p.c_group_stride = c_group_stride; p.b_group_rows = b_mn ? K : N; p.err = err;
    if (!a_mn && !b_mn) return launch<false, false>(ma, mb, (bf16*)C, p, num_sms, st);
    if (!a_mn && b_mn) return launch<false, true>(ma, mb, (bf16*)C, p, num_sms, st);
    if (a_mn && b_mn) return launch<true, true>(ma, mb, (bf16*)C, p, num_sms, st);
    return launch<true, false>(ma, mb, (bf16*)C, p, num_sms, st);
}
