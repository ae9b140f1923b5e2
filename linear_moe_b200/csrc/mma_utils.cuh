// Warp-level bf16 tensor-core helpers (mma.sync m16n8k16 + ldmatrix) and cp.async tile loads, shared by
// the chunked sequence-model and attention kernels.  Tiles live in shared memory with a padded row stride
// (a multiple of 8 elements that is an odd multiple of 16 bytes) so that ldmatrix rows fall in distinct banks.
#pragma once
#include "common.cuh"

namespace lmoe {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A fragment (16 x 16) of a matrix stored row-major [m][k] with leading dimension ld (elements).
__device__ __forceinline__ void load_a(uint32_t (&a)[4], const bf16* tile, int ld, int m0, int k0) {
    int l = threadIdx.x & 31;
    ldsm_x4(a, tile + (m0 + (l & 7) + 8 * ((l >> 3) & 1)) * ld + k0 + 8 * (l >> 4));
}
// A fragment of a matrix whose transpose is stored: storage [k][m].
__device__ __forceinline__ void load_a_t(uint32_t (&a)[4], const bf16* tile, int ld, int m0, int k0) {
    int l = threadIdx.x & 31;
    ldsm_x4_t(a, tile + (k0 + (l & 7) + 8 * (l >> 4)) * ld + m0 + 8 * ((l >> 3) & 1));
}
// Two B fragments (k 16 x n 16 -> n-tiles n0 and n0+8) from storage [n][k]  ("K-major").
__device__ __forceinline__ void load_b2(uint32_t (&b)[4], const bf16* tile, int ld, int n0, int k0) {
    int l = threadIdx.x & 31;
    ldsm_x4(b, tile + (n0 + (l & 7) + 8 * (l >> 4)) * ld + k0 + 8 * ((l >> 3) & 1));
}
// Two B fragments from storage [k][n].
__device__ __forceinline__ void load_b2_t(uint32_t (&b)[4], const bf16* tile, int ld, int n0, int k0) {
    int l = threadIdx.x & 31;
    ldsm_x4_t(b, tile + (k0 + (l & 7) + 8 * ((l >> 3) & 1)) * ld + n0 + 8 * (l >> 4));
}

// acc[NT][4] (16 rows x 8*NT cols) += A[m0:m0+16, 0:K] * B[0:K, n0:n0+8*NT]
//   A_T: A stored [k][m]; B_T: B stored [k][n] (else [n][k]).
template <int NT, int K, bool A_T, bool B_T>
__device__ __forceinline__ void warp_gemm(float (&acc)[NT][4], const bf16* A, int lda, int m0, const bf16* B, int ldb,
                                          int n0) {
    static_assert(NT % 2 == 0, "n-tiles come in pairs");
#pragma unroll
    for (int k0 = 0; k0 < K; k0 += 16) {
        uint32_t a[4];
        if (A_T) load_a_t(a, A, lda, m0, k0); else load_a(a, A, lda, m0, k0);
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
            uint32_t b[4];
            if (B_T) load_b2_t(b, B, ldb, n0 + nt * 8, k0); else load_b2(b, B, ldb, n0 + nt * 8, k0);
            mma16816(acc[nt], a, b[0], b[1]);
            mma16816(acc[nt + 1], a, b[2], b[3]);
        }
    }
}

// Same, with the A fragment multiplied per k index by a bf16x2 table (tab2[k/2] holds the scales of k, k+1).
// Requires A_T storage, where one register holds two consecutive k of the same row.
template <int NT, int K, bool B_T>
__device__ __forceinline__ void warp_gemm_at_kscaled(float (&acc)[NT][4], const bf16* A, int lda, int m0, const bf16* B,
                                                     int ldb, int n0, const __nv_bfloat162* tab2) {
    const int l = threadIdx.x & 31;
#pragma unroll
    for (int k0 = 0; k0 < K; k0 += 16) {
        uint32_t a[4];
        load_a_t(a, A, lda, m0, k0);
        __nv_bfloat162 s0 = tab2[(k0 >> 1) + (l & 3)], s1 = tab2[(k0 >> 1) + 4 + (l & 3)];
        __nv_bfloat162* ah = reinterpret_cast<__nv_bfloat162*>(a);
        ah[0] = __hmul2(ah[0], s0); ah[1] = __hmul2(ah[1], s0);
        ah[2] = __hmul2(ah[2], s1); ah[3] = __hmul2(ah[3], s1);
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
            uint32_t b[4];
            if (B_T) load_b2_t(b, B, ldb, n0 + nt * 8, k0); else load_b2(b, B, ldb, n0 + nt * 8, k0);
            mma16816(acc[nt], a, b[0], b[1]);
            mma16816(acc[nt + 1], a, b[2], b[3]);
        }
    }
}

template <int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[NT][4]) {
#pragma unroll
    for (int i = 0; i < NT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
}

// Store a warp's accumulator tile (16 x 8*NT) as bf16 into shared memory [m][n].
template <int NT>
__device__ __forceinline__ void store_acc_bf16(const float (&acc)[NT][4], bf16* tile, int ld, int m0, int n0) {
    int l = threadIdx.x & 31;
    int r = m0 + (l >> 2), c = n0 + (l & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        *reinterpret_cast<__nv_bfloat162*>(tile + r * ld + c + nt * 8) = __floats2bfloat162_rn(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<__nv_bfloat162*>(tile + (r + 8) * ld + c + nt * 8) = __floats2bfloat162_rn(acc[nt][2], acc[nt][3]);
    }
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(smem_u32(smem)), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N)); }

// Load a [ROWS x D] bf16 tile whose rows are `row_stride` elements apart in global memory into padded
// shared memory; rows >= valid_rows are zero-filled.
template <int ROWS, int D, int LD>
__device__ __forceinline__ void load_tile_async(bf16* smem, const bf16* gmem, int64_t row_stride, int valid_rows) {
    constexpr int VPR = D / 8;                       // 16-byte vectors per row
    for (int i = threadIdx.x; i < ROWS * VPR; i += blockDim.x) {
        int r = i / VPR, c = (i % VPR) * 8;
        bool ok = r < valid_rows;
        cp_async16(smem + r * LD + c, gmem + (ok ? (int64_t)r * row_stride + c : 0), ok);
    }
}

}  // namespace lmoe
