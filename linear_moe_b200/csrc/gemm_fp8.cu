// fp8 (e4m3) GEMM on tcgen05 (kind::f8f6f4, fp32 accumulation in tensor memory) with per-row scales of both
// operands applied in the epilogue, and the quantisation kernels that produce the operands.
//
//   C[M,N] (bf16) = diag(sa) * (A8[M,K] * B8[N,K]^T) * diag(sb)
//
// A8/B8 are K-major e4m3; sa[m] / sb[n] are the fp32 scales of the rows (amax / 448), so the scaling is exact rank-1
// and costs one multiply per output element.  The three GEMMs of a linear layer all take this form once their
// operands are quantised along the contracted dimension:
//   forward  y  = x W^T      A = rows(x)        B = rows(W)
//   dgrad    dx = dy W       A = rows(dy)       B = rows(W^T)   (quant_cols_t of W)
//   wgrad    dW = dy^T x     A = rows(dy^T)     B = rows(x^T)   (quant_cols_t of dy and of x)
// This is the fp8 training path of this framework; the reference gets fp8 from TransformerEngine's delayed-scaling
// recipe (hybrid_transformer_block.py:355-377).  Scales here are computed from the current tensor (no amax history).
//
// Tiles: 128 x 256 x 128 (128 bytes of K per shared-memory row = one 128-byte swizzle span), 4 stages of 48 KiB,
// one TMA producer thread, one MMA thread, 4 epilogue warps, double-buffered accumulators (2 x 256 TMEM columns).
#include <cuda_fp8.h>
#include "tcgen05_utils.cuh"

namespace lmoe {
namespace f8 {
using namespace lmoe::tc;

constexpr int BM = 128, BN = 256, BK = 128, STAGES = 4, UMMA_K = 32;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;

struct __align__(1024) Smem {
    uint8_t tiles[STAGES][STAGE_BYTES];
    uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// kind::f8f6f4 instruction descriptor: fp32 accumulator, e4m3 x e4m3, both K-major
__host__ __device__ constexpr uint32_t make_idesc_f8() {
    return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}"
                 :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_fp8_nt_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, bf16* __restrict__ C,
                   const float* __restrict__ sa, const float* __restrict__ sb, int M, int N, int K, int ldc, int* err) {
    extern __shared__ uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
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
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*abort_flag; tile += gridDim.x) {
                const int tm = tile % tiles_m, tn = tile / tiles_m;
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
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f8();
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
                        const uint64_t ad = make_desc<false>(a_addr + k * UMMA_K);        // 32 e4m3 = 32 bytes per step
                        const uint64_t bd = make_desc<false>(b_addr + k * UMMA_K);
                        umma_f8(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
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
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++lt) {
            const int tm = tile % tiles_m, tn = tile / tiles_m;
            const int buf = lt & 1;
            const uint32_t aph = (lt >> 1) & 1;
            if (!mbar_wait(&sm.tmem_full[buf], aph, abort_flag, err, 0x400 | buf)) break;
            tc_fence_after();
            const int r = q * 32 + lane;
            const int row = tm * BM + r;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            const float ra = row < M ? sa[row] : 0.f;
            bf16* crow = C + (long long)row * ldc + (long long)tn * BN;
            const int cols_valid = N - tn * BN;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                // column scales first, so that their latency overlaps the tensor-memory load
                float4 sc[8];
#pragma unroll
                for (int g = 0; g < 8; ++g)
                    sc[g] = (c + g * 4 + 4 <= cols_valid) ? __ldg(reinterpret_cast<const float4*>(sb + tn * BN + c + g * 4))
                                                           : make_float4(0.f, 0.f, 0.f, 0.f);
                uint32_t v[32];
                tmem_ld32(taddr + c, v);
                tmem_ld_wait();
                if (row < M) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const int col = c + g * 8;
                        if (col + 8 <= cols_valid) {
                            const float4 s0 = sc[2 * g], s1 = sc[2 * g + 1];
                            uint4 o;
                            o.x = pack_bf16(__uint_as_float(v[g * 8 + 0]) * ra * s0.x, __uint_as_float(v[g * 8 + 1]) * ra * s0.y);
                            o.y = pack_bf16(__uint_as_float(v[g * 8 + 2]) * ra * s0.z, __uint_as_float(v[g * 8 + 3]) * ra * s0.w);
                            o.z = pack_bf16(__uint_as_float(v[g * 8 + 4]) * ra * s1.x, __uint_as_float(v[g * 8 + 5]) * ra * s1.y);
                            o.w = pack_bf16(__uint_as_float(v[g * 8 + 6]) * ra * s1.z, __uint_as_float(v[g * 8 + 7]) * ra * s1.w);
                            *reinterpret_cast<uint4*>(crow + col) = o;
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

// Row-major e4m3 [rows, cols] with pitch ld bytes; box = {128 bytes of K, box_rows}.
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

__device__ __forceinline__ uint8_t to_e4m3(float x) {
    return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

// One CTA per row: scale[r] = amax(row) / 448, q = x / scale.  cols % 8 == 0.
__global__ void quant_rows_kernel(const bf16* __restrict__ x, long long ld, uint8_t* __restrict__ q, float* __restrict__ scale,
                                  int cols) {
    __shared__ float red[32];
    const long long r = blockIdx.x;
    const uint4* xr = reinterpret_cast<const uint4*>(x + r * ld);
    const int v8 = cols / 8;
    float amax = 0.f;
    for (int i = threadIdx.x; i < v8; i += blockDim.x) {
        uint4 v = xr[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(h[j]);
            amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
    }
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    if (threadIdx.x < 32) {
        float m = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
        m = warp_max(m);
        if (threadIdx.x == 0) red[0] = m;
    }
    __syncthreads();
    amax = red[0];
    const float sc = amax > 0.f ? amax / 448.f : 1.f;
    const float inv = 1.f / sc;
    if (threadIdx.x == 0) scale[r] = sc;
    uint2* qr = reinterpret_cast<uint2*>(q + r * cols);
    for (int i = threadIdx.x; i < v8; i += blockDim.x) {
        uint4 v = xr[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
        uint8_t o[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 f = __bfloat1622float2(h[j]);
            o[2 * j] = to_e4m3(f.x * inv);
            o[2 * j + 1] = to_e4m3(f.y * inv);
        }
        qr[i] = *reinterpret_cast<uint2*>(o);
    }
}

// amax over the rows of every column: grid (cols/64 column groups of 64, row chunks); 64 x 4 threads
__global__ void col_amax_kernel(const bf16* __restrict__ x, long long ld, int rows, int cols, int rows_per_cta,
                                unsigned int* __restrict__ amax_bits) {
    const int c = blockIdx.x * 64 + (threadIdx.x & 63);
    const int r0 = blockIdx.y * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
    float m = 0.f;
    if (c < cols)
        for (int r = r0 + (threadIdx.x >> 6); r < r1; r += blockDim.x >> 6) m = fmaxf(m, fabsf(__bfloat162float(x[(long long)r * ld + c])));
    if (c < cols && m > 0.f) atomicMax(amax_bits + c, __float_as_uint(m));      // non-negative floats order like their bits
}

// qT[c][r] = x[r][c] / scale[c] with scale[c] = amax[c] / 448 (also written out); 32 x 32 tiles through shared memory
__global__ void quant_cols_t_kernel(const bf16* __restrict__ x, long long ld, int rows, int cols,
                                    const unsigned int* __restrict__ amax_bits, uint8_t* __restrict__ qT, float* __restrict__ scale) {
    __shared__ float tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;           // 32 x 8
    for (int i = ty; i < 32; i += 8) {
        const int r = r0 + i, c = c0 + tx;
        tile[i][tx] = (r < rows && c < cols) ? __bfloat162float(x[(long long)r * ld + c]) : 0.f;
    }
    __syncthreads();
    for (int i = ty; i < 32; i += 8) {
        const int c = c0 + i, r = r0 + tx;
        if (c < cols && r < rows) {
            const float am = __uint_as_float(amax_bits[c]);
            const float sc = am > 0.f ? am / 448.f : 1.f;
            qT[(long long)c * rows + r] = to_e4m3(tile[tx][i] / sc);
            if (blockIdx.y == 0 && tx == 0) scale[c] = sc;
        }
    }
}

}  // namespace f8
}  // namespace lmoe

using namespace lmoe;
using namespace lmoe::f8;

// A8 [M,K], B8 [N,K] e4m3 contiguous, sa [M], sb [N] fp32, C [M,N] bf16 (pitch ldc).  K % 16 == 0, N % 8 == 0.
LMOE_API int lmoe_gemm_fp8_nt(const void* A, const void* B, void* C, const float* sa, const float* sb, int M, int N, int K,
                              int ldc, int* err, int num_sms, cudaStream_t st) {
    if (K % 16 || N % 8 || ldc % 8) return -1;
    CUtensorMap ma, mb;
    int rc = make_map_u8(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM);
    if (rc) return rc;
    rc = make_map_u8(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)K, BN);
    if (rc) return rc;
    const size_t smem = sizeof(Smem) + 1024;
    cudaFuncSetAttribute(gemm_fp8_nt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    gemm_fp8_nt_kernel<<<tiles < num_sms ? tiles : num_sms, THREADS, smem, st>>>(ma, mb, (bf16*)C, sa, sb, M, N, K, ldc, err);
    return (int)cudaGetLastError();
}

// x [rows, cols] bf16 (pitch ld) -> q [rows, cols] e4m3, scale [rows]
LMOE_API int lmoe_fp8_quant_rows(const void* x, long long ld, void* q, float* scale, int rows, int cols, cudaStream_t st) {
    if (cols % 8 || ld % 8) return -1;
    if (rows > 0) quant_rows_kernel<<<rows, 256, 0, st>>>((const bf16*)x, ld, (uint8_t*)q, scale, cols);
    return (int)cudaGetLastError();
}

// x [rows, cols] bf16 -> qT [cols, rows] e4m3, scale [cols]; amax_bits [cols] is scratch (zeroed here)
LMOE_API int lmoe_fp8_quant_cols_t(const void* x, long long ld, void* qT, float* scale, unsigned int* amax_bits, int rows, int cols,
                                   cudaStream_t st) {
    if (rows <= 0 || cols <= 0) return 0;
    cudaMemsetAsync(amax_bits, 0, sizeof(unsigned int) * cols, st);
    const int rows_per_cta = 256;
    col_amax_kernel<<<dim3((cols + 63) / 64, (rows + rows_per_cta - 1) / rows_per_cta), 256, 0, st>>>((const bf16*)x, ld, rows, cols,
                                                                                                   rows_per_cta, amax_bits);
    quant_cols_t_kernel<<<dim3((cols + 31) / 32, (rows + 31) / 32), 256, 0, st>>>((const bf16*)x, ld, rows, cols, amax_bits,
                                                                               (uint8_t*)qT, scale);
    return (int)cudaGetLastError();
}
