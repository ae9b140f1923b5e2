// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] * B[N,K]^T  (x W^T of a linear layer),
// fp32 accumulation in tensor memory, optional fused SwiGLU epilogue.
//
// This is the framework's own replacement for the cuBLAS call behind ColumnParallelLinear /
// RowParallelLinear / the expert GEMMs of the reference (qwen2/layer_specs.py:94-96,
// qwen2/moe/experts.py:156-168, which reach cuBLAS / CUTLASS-sm80 grouped GEMM through Megatron).
//
// Structure (one persistent CTA per SM, 192 threads, no clusters, no multicast):
//   warp 0     TMA producer: cp.async.bulk.tensor.2d loads of the A (128 x 64) and B (256 x 64) k-blocks into a
//              4-stage ring of 128B-swizzled shared-memory tiles, completion counted on `full` mbarriers
//   warp 1     MMA issuer: one elected thread issues tcgen05.mma (M=128, N=256, K=16, kind::f16) from shared-
//              memory descriptors into one of two 256-column TMEM accumulators; tcgen05.commit releases
//              ring stages (`empty`) and publishes finished accumulators (`tmem_full`)
//   warps 2-5  epilogue: tcgen05.ld of the warp's 32 TMEM lanes, fp32 -> bf16 (or silu(gate)*up), 16-byte
//              global stores; `tmem_empty` hands the accumulator back, so the epilogue of tile i overlaps
//              the main loop of tile i+1
// Every mbarrier wait is bounded: when a wait runs out the thread raises the CTA's abort flag and the error
// word in global memory, every role leaves its loops, TMEM is freed and the kernel returns.
#include <cuda.h>
#include "common.cuh"

namespace lmoe {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr long long WAIT_CYCLES = 2000LL * 1000 * 1000;    // clock64 budget of one wait (about a second)

struct __align__(1024) GemmSmem {
    uint8_t tiles[STAGES][STAGE_BYTES];
    uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
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
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(s32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (and raises the abort flag + error word) when the limit is hit or another role
// of this CTA has already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err, int code) {
    const long long t0 = clock64();
    for (int i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;      // non-blocking test_wait
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

// Shared-memory matrix descriptor of a K-major bf16 tile with 128-byte swizzle: rows are 128 bytes, groups of 8
// rows (1024 bytes) repeat with stride SBO = 1024 bytes; LBO is unused for swizzled K-major (encoded 1);
// bits 46-47 = descriptor version 1; bits 61-63 = 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// Instruction descriptor, kind::f16: D = fp32 (bits 4-5 = 1), A = B = bf16 (bits 7-9 = 1, 10-12 = 1), both K-major,
// N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
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

// EPI = 0: C[M,N] = acc.   EPI = 1 (SwiGLU): B rows are laid out per 256-row tile as [128 gate rows | 128 up rows];
// C[M, N/2] tile columns [t*128, t*128+128) = silu(acc[:, 0:128]) * acc[:, 128:256].
template <int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_nt_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, bf16* __restrict__ C,
                    int M, int N, int K, int ldc, int* err) {
    extern __shared__ uint8_t smem_raw[];
    GemmSmem& sm = *reinterpret_cast<GemmSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int kblocks = (K + BK - 1) / BK;
    volatile int* abort_flag = &sm.abort_flag;

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
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x) {
                const int tm = tile % tiles_m, tn = tile / tiles_m;       // consecutive CTAs share the B (weight) tile
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&sm.empty[s], ph ^ 1, abort_flag, err, 0x100 | s)) goto producer_done;
                    mbar_expect_tx(&sm.full[s], STAGE_BYTES);
                    tma_load_2d(sm.tiles[s], &tmA, &sm.full[s], kb * BK, tm * BM);
                    tma_load_2d(sm.tiles[s] + A_BYTES, &tmB, &sm.full[s], kb * BK, tn * BN);
                }
            }
        }
    producer_done:;
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN);
            int it = 0, lt = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x, ++lt) {
                const int buf = lt & 1;
                const uint32_t aph = (lt >> 1) & 1;
                if (!mbar_wait(&sm.tmem_empty[buf], aph ^ 1, abort_flag, err, 0x200 | buf)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                bool dead = false;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&sm.full[s], ph, abort_flag, err, 0x300 | s)) { dead = true; break; }
                    tc_fence_after();
                    const uint32_t a_addr = s32(sm.tiles[s]), b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t ad = make_desc(a_addr + k * UMMA_K * 2);
                        const uint64_t bd = make_desc(b_addr + k * UMMA_K * 2);
                        umma_f16(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&sm.empty[s]);            // stage reusable once these MMAs have read it
                }
                if (dead) break;
                umma_commit(&sm.tmem_full[buf]);          // accumulator complete
            }
        }
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        const int q = warp & 3;                           // TMEM lane quarter this warp may access
        int lt = 0;
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++lt) {
            const int tm = tile % tiles_m, tn = tile / tiles_m;
            const int buf = lt & 1;
            const uint32_t aph = (lt >> 1) & 1;
            if (!mbar_wait(&sm.tmem_full[buf], aph, abort_flag, err, 0x400 | buf)) break;
            tc_fence_after();
            const int row = tm * BM + q * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            if (EPI == 0) {
                bf16* crow = C + (size_t)row * ldc + (size_t)tn * BN;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(taddr + c, r);
                    tmem_ld_wait();
                    if (row < M) {
                        const int col0 = tn * BN + c;
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            if (col0 + v * 8 + 8 <= N) {
                                uint4 o;
                                o.x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                                o.y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                                o.z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                                o.w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                                *reinterpret_cast<uint4*>(crow + c + v * 8) = o;
                            } else {
                                for (int e = 0; e < 8; ++e)
                                    if (col0 + v * 8 + e < N) crow[c + v * 8 + e] = __float2bfloat16(__uint_as_float(r[v * 8 + e]));
                            }
                        }
                    }
                }
            } else {
                bf16* crow = C + (size_t)row * ldc + (size_t)tn * (BN / 2);
#pragma unroll 1
                for (int c = 0; c < BN / 2; c += 32) {
                    uint32_t g[32], u[32];
                    tmem_ld32(taddr + c, g);
                    tmem_ld32(taddr + BN / 2 + c, u);
                    tmem_ld_wait();
                    if (row < M) {
                        const int col0 = tn * (BN / 2) + c;
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            float y[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) y[e] = silu_f(__uint_as_float(g[v * 8 + e])) * __uint_as_float(u[v * 8 + e]);
                            if (col0 + v * 8 + 8 <= N / 2) {
                                uint4 o;
                                o.x = pack_bf16(y[0], y[1]); o.y = pack_bf16(y[2], y[3]);
                                o.z = pack_bf16(y[4], y[5]); o.w = pack_bf16(y[6], y[7]);
                                *reinterpret_cast<uint4*>(crow + c + v * 8) = o;
                            } else {
                                for (int e = 0; e < 8; ++e)
                                    if (col0 + v * 8 + e < N / 2) crow[c + v * 8 + e] = __float2bfloat16(y[e]);
                            }
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
    // the encoder is a driver call: it wants the primary context current on this thread (an autograd worker that has
    // made no runtime call yet has none)
    static thread_local bool bound = false;
    if (!bound) { cudaFree(0); bound = true; }
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

// 2-D bf16 row-major tensor [rows, cols] (row pitch ld elements) -> tensor map with a {64 x box_rows} box, 128B swizzle.
static int make_map(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
    EncodeTiledFn enc = get_encode();
    if (enc == nullptr) return -10;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -11;
}

}  // namespace lmoe

using namespace lmoe;

// C[M,N] (row pitch ldc) = A[M,K] (pitch lda) * B[N,K]^T (pitch ldb), bf16.  epi = 1: SwiGLU over 256-row B tiles laid
// out as [128 gate | 128 up]; C is then [M, N/2].  `err` is a device int the kernel sets when a bounded wait expires.
// Requirements: K % 8 == 0, lda/ldb % 8 == 0, 16-byte aligned base pointers, ldc % 8 == 0.
LMOE_API int lmoe_gemm_bf16_nt(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int epi,
                               int* err, int num_sms, cudaStream_t st) {
    if (K % 8 || lda % 8 || ldb % 8 || ldc % 8) return -1;
    if (epi == 1 && (N % 256)) return -2;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM);
    if (rc) return rc;
    rc = make_map(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, BN);
    if (rc) return rc;
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = tiles < num_sms ? tiles : num_sms;
    const size_t smem = sizeof(GemmSmem) + 1024;
    if (epi == 0) {
        cudaFuncSetAttribute(gemm_bf16_nt_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gemm_bf16_nt_kernel<0><<<grid, GEMM_THREADS, smem, st>>>(ma, mb, (bf16*)C, M, N, K, ldc, err);
    } else {
        cudaFuncSetAttribute(gemm_bf16_nt_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gemm_bf16_nt_kernel<1><<<grid, GEMM_THREADS, smem, st>>>(ma, mb, (bf16*)C, M, N, K, ldc, err);
    }
    return (int)cudaGetLastError();
}
