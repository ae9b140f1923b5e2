// Dense bf16 GEMM for every plain linear layer: forward (x W^T), data gradient (dy W) and weight gradient (dy^T x)
// are the same kernel with K-major or MN-major operands.  One 256 x 256 output tile per CTA pair
// (tcgen05.mma.cta_group::2), accumulators double-buffered in tensor memory, operands staged by TMA into a 6-stage ring,
// results leaving through TMA stores (or TMA reduce-adds for fp32 accumulation into an optimizer's gradient buffer).
//
//   C[M,N] (+)= A * B      A: [M,K] row-major (K-major)  or [K,M] row-major (MN-major, a_mn)
//                          B: [N,K] row-major (K-major)  or [K,N] row-major (MN-major, b_mn)
//   out_mode 0: C bf16 = result      1: C fp32 = result      2: C fp32 += result (cp.reduce.async.bulk .add, done in L2)
//   epi 1 (K-major operands, bf16 out): B = [gate rows ; up rows] of a SwiGLU fc1 weight ([2F, K]).  CTA 0 of the pair
//          stages 128 gate rows, CTA 1 the matching 128 up rows, so accumulator columns [0,128) / [128,256) are gate / up
//          of the same 128 outputs; the epilogue writes silu(gate) * up to C [M,F] and, if Y != null, the
//          pre-activations to Y [M,2F] (what the backward pass needs).  No re-tiling of the weight.
//   epi 2 (A K-major, B MN-major, bf16 out): the data-gradient GEMM of fc2, dAct = dY W2, with the SwiGLU backward in
//          the epilogue: the tile of dAct never leaves the SM; the matching gate / up pre-activations are fetched by TMA
//          from Y [M,2F] into shared memory and C [M,2F] receives dGate = dAct * up * silu'(gate), dUp = dAct * silu(gate).
//
// Tile order: tiles are numbered band by band (a band = `band` consecutive tile rows of C), column by column inside a
// band, so the ~74 tiles in flight cover about band x (74 / band) tiles: both operands' working sets stay a few MB and
// are served by L2 (with one tile column per wave, the whole of A streamed from HBM once per wave).
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (leader CTA) and TMEM allocator, warps 2-5 =
// epilogue (TMEM -> registers -> swizzled shared staging -> TMA store; two staging buffers per warp so the store of one
// 64-column slab overlaps the conversion of the next).  Every wait is bounded; on expiry the error word is set, the
// CTA leaves its loops, the pair meets at the final cluster barrier and tensor memory is released.
// Reference counterpart: the cuBLAS / TransformerEngine GEMMs behind ColumnParallelLinear / RowParallelLinear
// (linear_moe/model/qwen2/layer_specs.py:94-96,128-147,200-203).
#include "tcgen05_utils.cuh"

namespace lmoe {
namespace gd {
using namespace lmoe::tc;

constexpr int BK = 64, UMMA_K = 16, STAGES = 6, THREADS = 192;
constexpr int HALF_BYTES = 128 * BK * 2, STAGE_BYTES = 2 * HALF_BYTES;      // per CTA: 128 rows of A + 128 rows of B
constexpr int OUT_BYTES = 32 * 128;                                          // one staging slab: 32 rows x 128 bytes
constexpr uint32_t TMEM_COLS = 512;

struct __align__(1024) Smem {
    uint8_t tiles[STAGES][STAGE_BYTES];
    uint8_t out[4][2][OUT_BYTES];
    uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2];
    uint64_t epi_bar[4];                         // epi 2: arrival of a warp's gate / up slabs
    uint32_t tmem_base;
    int abort_flag;
};

struct Params {
    int M, N, K;
    int band;          // tile rows per band of the tile order
    int f_half;        // epi 1: F (rows of the gate block of B)
    int* err;
    const bf16* bias;  // out mode 0 without epilogue function: [N] added to every row, or null
};

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"(map), "r"(s32(src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"(map), "r"(s32(src)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void decode(const Params& p, int t, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int per_band = p.band * tiles_n;
    const int b = t / per_band, r = t - b * per_band;
    const int gm = min(p.band, tiles_m - b * p.band);
    tm = b * p.band + r % gm;
    tn = r / gm;
}

// v[i] += bias[i] for 32 consecutive columns (the same 64 bytes for every lane: broadcast loads); columns >= n_left skipped
__device__ __forceinline__ void add_bias32(uint32_t (&v)[32], const bf16* bias, int n_left) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        if (g * 8 < n_left) {                                           // N is a multiple of 8
            const uint4 b = __ldg(reinterpret_cast<const uint4*>(bias) + g);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(b2[i]);
                v[g * 8 + 2 * i] = __float_as_uint(__uint_as_float(v[g * 8 + 2 * i]) + f.x);
                v[g * 8 + 2 * i + 1] = __float_as_uint(__uint_as_float(v[g * 8 + 2 * i + 1]) + f.y);
            }
        }
    }
}

// one lane's 32 fp32 values -> 64 bytes (bf16) of its row in a swizzled staging slab; `part` = which half of the 128-byte row
__device__ __forceinline__ void stage_bf16(uint8_t* stg, int lane, int part, const uint32_t (&v)[32]) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 o;
        o.x = pack_bf16(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]));
        o.y = pack_bf16(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
        o.z = pack_bf16(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
        o.w = pack_bf16(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
        *reinterpret_cast<uint4*>(stg + lane * 128 + (((part * 4 + g) ^ (lane & 7)) << 4)) = o;
    }
}

template <bool A_MN, bool B_MN, int OUT, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_dense_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmY, int has_y, Params p) {
    extern __shared__ uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    constexpr int TILE_N = EPI == 1 ? 128 : 256;                        // output columns per tile
    constexpr int NS = EPI == 2 ? STAGES - 1 : STAGES;                  // epi 2 uses the last ring slot for its input slabs
    const int tiles_m = (p.M + 255) / 256, tiles_n = (p.N + TILE_N - 1) / TILE_N;
    const int num_tiles = tiles_m * tiles_n;
    const int kblocks = (p.K + BK - 1) / BK;
    volatile int* abort_flag = &sm.abort_flag;
    int* err = p.err;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sm.tmem_full[b], 1); mbar_init(&sm.tmem_empty[b], 8); }   // 4 warps x 2 CTAs
        for (int b = 0; b < 4; ++b) mbar_init(&sm.epi_bar[b], 1);
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
    const int half = (int)rank * 128;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int tile = pair; tile < num_tiles && !*abort_flag; tile += num_pairs) {
                int tm, tn;
                decode(p, tile, tiles_m, tiles_n, tm, tn);
                const int a0 = tm * 256 + half;
                const int b0 = EPI == 1 ? (int)rank * p.f_half + tn * 128 : tn * 256 + half;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % NS;
                    const uint32_t ph = (it / NS) & 1;
                    if (!mbar_wait(&sm.empty[s], ph ^ 1, abort_flag, err, 0x7100 | s)) goto producer_done;
                    if (rank == 0) mbar_expect_tx(&sm.full[s], 2 * STAGE_BYTES);      // both CTAs' loads land on the leader's barrier
                    const uint32_t fl = map_to_cta(&sm.full[s], 0);
                    uint8_t* sa = sm.tiles[s];
                    uint8_t* sb = sa + HALF_BYTES;
                    if (!A_MN) tma_load_2d_pair(sa, &tmA, fl, kb * BK, a0);
                    else {
                        tma_load_2d_pair(sa, &tmA, fl, a0, kb * BK);
                        tma_load_2d_pair(sa + 8192, &tmA, fl, a0 + 64, kb * BK);
                    }
                    if (!B_MN) tma_load_2d_pair(sb, &tmB, fl, kb * BK, b0);
                    else {
                        tma_load_2d_pair(sb, &tmB, fl, b0, kb * BK);
                        tma_load_2d_pair(sb + 8192, &tmB, fl, b0 + 64, kb * BK);
                    }
                }
            }
        }
    producer_done:;
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                                       ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            int it = 0, lt = 0;
            for (int tile = pair; tile < num_tiles && !*abort_flag; tile += num_pairs, ++lt) {
                const int buf = lt & 1;
                const uint32_t aph = (lt >> 1) & 1;
                if (!mbar_wait(&sm.tmem_empty[buf], aph ^ 1, abort_flag, err, 0x7200 | buf)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * 256;
                bool dead = false;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % NS;
                    const uint32_t ph = (it / NS) & 1;
                    if (!mbar_wait(&sm.full[s], ph, abort_flag, err, 0x7300 | s)) { dead = true; break; }
                    tc_fence_after();
                    const uint32_t a_addr = s32(sm.tiles[s]), b_addr = a_addr + HALF_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t ad = make_desc<A_MN>(a_addr + (A_MN ? k * 2048 : k * UMMA_K * 2));
                        const uint64_t bd = make_desc<B_MN>(b_addr + (B_MN ? k * 2048 : k * UMMA_K * 2));
                        umma_pair<false>(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(&sm.empty[s]);
                }
                if (dead) break;
                umma_commit_pair(&sm.tmem_full[buf]);
            }
        }
    } else {
        const int q = warp & 3;                                   // TMEM lane quadrant this warp may read
        uint8_t* stg0 = sm.out[warp - 2][0];
        int lt = 0, nst = 0;                                      // nst: staging slabs used so far (ring of 2)
        int nload = 0, nepi = 0;                                  // epi 2: input-slab loads completed by this warp
        for (int tile = pair; tile < num_tiles; tile += num_pairs, ++lt) {
            int tm, tn;
            decode(p, tile, tiles_m, tiles_n, tm, tn);
            const int buf = lt & 1;
            const uint32_t aph = (lt >> 1) & 1;
            if (!mbar_wait(&sm.tmem_full[buf], aph, abort_flag, err, 0x7400 | buf)) break;
            tc_fence_after();
            const int row0 = tm * 256 + half + q * 32;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256;
            const bool live = row0 < p.M;
            if (EPI == 1) {
                const int col_base = tn * 128;
#pragma unroll 1
                for (int c = 0; c < 128; c += 64) {
                    uint32_t g0[32], g1[32], u0[32], u1[32];
                    tmem_ld32(taddr + c, g0);
                    tmem_ld32(taddr + c + 32, g1);
                    tmem_ld32(taddr + 128 + c, u0);
                    tmem_ld32(taddr + 128 + c + 32, u1);
                    tmem_ld_wait();
                    if (has_y) {
                        uint8_t* s = stg0 + (nst & 1) * OUT_BYTES;
                        if (lane == 0) bulk_wait_read<1>();
                        __syncwarp();
                        stage_bf16(s, lane, 0, g0); stage_bf16(s, lane, 1, g1);
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) { if (live && col_base + c < p.f_half) tma_store_2d(&tmY, s, col_base + c, row0); bulk_commit(); }
                        ++nst;
                        s = stg0 + (nst & 1) * OUT_BYTES;
                        if (lane == 0) bulk_wait_read<1>();
                        __syncwarp();
                        stage_bf16(s, lane, 0, u0); stage_bf16(s, lane, 1, u1);
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) { if (live && col_base + c < p.f_half) tma_store_2d(&tmY, s, p.f_half + col_base + c, row0); bulk_commit(); }
                        ++nst;
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        g0[i] = __float_as_uint(silu_f(__uint_as_float(g0[i])) * __uint_as_float(u0[i]));
                        g1[i] = __float_as_uint(silu_f(__uint_as_float(g1[i])) * __uint_as_float(u1[i]));
                    }
                    uint8_t* s = stg0 + (nst & 1) * OUT_BYTES;
                    if (lane == 0) bulk_wait_read<1>();
                    __syncwarp();
                    stage_bf16(s, lane, 0, g0); stage_bf16(s, lane, 1, g1);
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) { if (live && col_base + c < p.f_half) tma_store_2d(&tmC, s, col_base + c, row0); bulk_commit(); }
                    ++nst;
                }
            } else if (EPI == 2) {
                const int col_base = tn * 256;
                uint8_t* gin = sm.tiles[STAGES - 1] + (warp - 2) * 2 * OUT_BYTES;      // gate slab, then up slab
                uint64_t* ebar = &sm.epi_bar[warp - 2];
#pragma unroll 1
                for (int c = 0; c < 256; c += 64, ++nepi) {
                    const bool cols_live = col_base + c < p.N;
                    if (lane == 0 && live && cols_live) {
                        fence_async_smem();                                // the lanes' reads of the previous slabs are done
                        mbar_expect_tx(ebar, 2 * OUT_BYTES);
                        tma_load_2d(gin, &tmY, ebar, col_base + c, row0);
                        tma_load_2d(gin + OUT_BYTES, &tmY, ebar, p.N + col_base + c, row0);
                    }
                    uint32_t v0[32], v1[32];
                    tmem_ld32(taddr + c, v0);
                    tmem_ld32(taddr + c + 32, v1);
                    tmem_ld_wait();
                    bool ok = true;
                    if (live && cols_live) ok = mbar_wait(ebar, nload & 1, abort_flag, err, 0x7500 | (warp - 2));
                    if (live && cols_live) ++nload;
                    if (!ok) break;
                    // this lane's row of the gate / up slabs (16-byte chunks are xor-swizzled by the row)
                    uint32_t dg[32], du[32];
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch) {
                        uint4 g4 = make_uint4(0, 0, 0, 0), u4 = make_uint4(0, 0, 0, 0);
                        if (live && cols_live) {
                            g4 = *reinterpret_cast<const uint4*>(gin + lane * 128 + ((ch ^ (lane & 7)) << 4));
                            u4 = *reinterpret_cast<const uint4*>(gin + OUT_BYTES + lane * 128 + ((ch ^ (lane & 7)) << 4));
                        }
                        const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int col = ch * 8 + e * 2;                               // columns col, col + 1 of the slab
                            const __nv_bfloat162 gb = *reinterpret_cast<const __nv_bfloat162*>(&gw[e]);
                            const __nv_bfloat162 ub = *reinterpret_cast<const __nv_bfloat162*>(&uw[e]);
                            const float g0 = __bfloat162float(gb.x), g1 = __bfloat162float(gb.y);
                            const float u0 = __bfloat162float(ub.x), u1 = __bfloat162float(ub.y);
                            const float d0 = __uint_as_float(col < 32 ? v0[col & 31] : v1[col & 31]);
                            const float d1 = __uint_as_float(col + 1 < 32 ? v0[(col + 1) & 31] : v1[(col + 1) & 31]);
                            const float s0 = sigmoid_f(g0), s1 = sigmoid_f(g1);
                            dg[ch * 4 + e] = pack_bf16(d0 * u0 * s0 * (1.f + g0 * (1.f - s0)), d1 * u1 * s1 * (1.f + g1 * (1.f - s1)));
                            du[ch * 4 + e] = pack_bf16(d0 * g0 * s0, d1 * g1 * s1);
                        }
                    }
                    __syncwarp();                                          // every lane has read its input row
                    uint8_t* s = stg0 + (nst & 1) * OUT_BYTES;
                    if (lane == 0) bulk_wait_read<1>();
                    __syncwarp();
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch)
                        *reinterpret_cast<uint4*>(s + lane * 128 + ((ch ^ (lane & 7)) << 4)) =
                            make_uint4(dg[ch * 4], dg[ch * 4 + 1], dg[ch * 4 + 2], dg[ch * 4 + 3]);
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) { if (live && cols_live) tma_store_2d(&tmC, s, col_base + c, row0); bulk_commit(); }
                    ++nst;
                    s = stg0 + (nst & 1) * OUT_BYTES;
                    if (lane == 0) bulk_wait_read<1>();
                    __syncwarp();
#pragma unroll
                    for (int ch = 0; ch < 8; ++ch)
                        *reinterpret_cast<uint4*>(s + lane * 128 + ((ch ^ (lane & 7)) << 4)) =
                            make_uint4(du[ch * 4], du[ch * 4 + 1], du[ch * 4 + 2], du[ch * 4 + 3]);
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) { if (live && cols_live) tma_store_2d(&tmC, s, p.N + col_base + c, row0); bulk_commit(); }
                    ++nst;
                }
            } else if (OUT == 0) {
                const int col_base = tn * 256;
#pragma unroll 1
                for (int c = 0; c < 256; c += 64) {
                    uint32_t v0[32], v1[32];
                    tmem_ld32(taddr + c, v0);
                    tmem_ld32(taddr + c + 32, v1);
                    uint8_t* s = stg0 + (nst & 1) * OUT_BYTES;
                    if (lane == 0) bulk_wait_read<1>();           // the store that last used this slab has read it
                    __syncwarp();
                    tmem_ld_wait();
                    if (p.bias != nullptr) {
                        add_bias32(v0, p.bias + col_base + c, p.N - (col_base + c));
                        add_bias32(v1, p.bias + col_base + c + 32, p.N - (col_base + c + 32));
                    }
                    stage_bf16(s, lane, 0, v0); stage_bf16(s, lane, 1, v1);
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) { if (live && col_base + c < p.N) tma_store_2d(&tmC, s, col_base + c, row0); bulk_commit(); }
                    ++nst;
                }
            } else {
                const int col_base = tn * 256;
#pragma unroll 1
                for (int c = 0; c < 256; c += 32) {
                    uint32_t v[32];
                    tmem_ld32(taddr + c, v);
                    uint8_t* s = stg0 + (nst & 1) * OUT_BYTES;
                    if (lane == 0) bulk_wait_read<1>();
                    __syncwarp();
                    tmem_ld_wait();
#pragma unroll
                    for (int g = 0; g < 8; ++g)
                        *reinterpret_cast<uint4*>(s + lane * 128 + ((g ^ (lane & 7)) << 4)) = make_uint4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (live && col_base + c < p.N) {
                            if (OUT == 2) tma_reduce_add_2d(&tmC, s, col_base + c, row0);
                            else tma_store_2d(&tmC, s, col_base + c, row0);
                        }
                        bulk_commit();
                    }
                    ++nst;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(&sm.tmem_empty[buf], 0));
        }
        if (lane == 0) bulk_wait_all();                            // staged slabs are read and written out before the CTA exits
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();                                                // nobody leaves while the peer may still signal its barriers
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// row-major [rows, cols] of `esize`-byte elements with pitch ld (elements); box = {box_cols, box_rows}, 128-byte swizzle
static int make_map_any(CUtensorMap* map, const void* ptr, CUtensorMapDataType dt, int esize, uint64_t rows, uint64_t cols, uint64_t ld,
                        uint32_t box_cols, uint32_t box_rows) {
    EncodeTiledFn enc = get_encode();
    if (enc == nullptr) return -10;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * (uint64_t)esize};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -11;
}

template <bool A_MN, bool B_MN, int OUT, int EPI>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const CUtensorMap& my, int has_y, const Params& p,
                  int num_sms, cudaStream_t st) {
    const size_t smem = sizeof(Smem) + 1024;
    static bool configured = false;                                 // one flag per template instantiation
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_dense_kernel<A_MN, B_MN, OUT, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const int tile_n = EPI == 1 ? 128 : 256;
    const int tiles = ((p.M + 255) / 256) * ((p.N + tile_n - 1) / tile_n);
    int pairs = num_sms / 2;
    if (tiles < pairs) pairs = tiles;
    if (pairs < 1) return 0;
    gemm_dense_kernel<A_MN, B_MN, OUT, EPI><<<2 * pairs, THREADS, smem, st>>>(ma, mb, mc, my, has_y, p);
    return (int)cudaGetLastError();
}

}  // namespace gd
}  // namespace lmoe

using namespace lmoe;
using namespace lmoe::gd;

// C[M,N] (+)= A * B, bf16 operands, fp32 accumulation.
//   a_mn = 0: A is [M,K] with pitch lda;  a_mn = 1: A is [K,M] with pitch lda.   Same for B with N.
//   out_mode 0: C bf16;  1: C fp32 (overwrite);  2: C fp32 += (reduce-add performed by the memory system).
//   band: tile rows per band of the tile order (0 = default).
// Every pitch and the contiguous extent of every matrix must be a multiple of 8 elements (16-byte TMA rule).
static int gemm_dense_impl(const void* A, int lda, int a_mn, const void* B, int ldb, int b_mn, void* C, int ldc, int out_mode,
                           int M, int N, int K, int band, int* err, int num_sms, cudaStream_t st, const void* bias) {
    if (M <= 0 || N <= 0 || K <= 0) return -1;
    if (bias != nullptr && (out_mode != 0 || ((uintptr_t)bias & 15))) return -1;
    if (lda % 8 || ldb % 8 || (a_mn ? M : K) % 8 || (b_mn ? N : K) % 8) return -1;
    if (out_mode == 0 ? (ldc % 8 || N % 8) : (ldc % 4 || N % 4)) return -1;
    if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) return -2;
    CUtensorMap ma, mb, mc;
    int rc = a_mn ? make_map(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64) : make_map(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, 128);
    if (rc) return rc;
    rc = b_mn ? make_map(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64) : make_map(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, 128);
    if (rc) return rc;
    rc = out_mode == 0 ? make_map_any(&mc, C, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, N, ldc, 64, 32)
                       : make_map_any(&mc, C, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, M, N, ldc, 32, 32);
    if (rc) return rc;
    Params p;
    p.M = M; p.N = N; p.K = K; p.band = band > 0 ? band : 8; p.f_half = 0; p.err = err; p.bias = (const bf16*)bias;
#define LMOE_GD_OUT(AMN, BMN)                                                                          \
    (out_mode == 0 ? launch<AMN, BMN, 0, 0>(ma, mb, mc, mc, 0, p, num_sms, st)                         \
   : out_mode == 1 ? launch<AMN, BMN, 1, 0>(ma, mb, mc, mc, 0, p, num_sms, st)                         \
                   : launch<AMN, BMN, 2, 0>(ma, mb, mc, mc, 0, p, num_sms, st))
    if (!a_mn && !b_mn) return LMOE_GD_OUT(false, false);
    if (!a_mn && b_mn) return LMOE_GD_OUT(false, true);
    if (a_mn && b_mn) return LMOE_GD_OUT(true, true);
    return LMOE_GD_OUT(true, false);
#undef LMOE_GD_OUT
}

LMOE_API int lmoe_gemm_dense(const void* A, int lda, int a_mn, const void* B, int ldb, int b_mn, void* C, int ldc, int out_mode,
                             int M, int N, int K, int band, int* err, int num_sms, cudaStream_t st) {
    return gemm_dense_impl(A, lda, a_mn, B, ldb, b_mn, C, ldc, out_mode, M, N, K, band, err, num_sms, st, nullptr);
}

// C[M,N] (bf16) = A * B + bias[N] (bf16, 16-byte aligned), the bias added to the fp32 accumulator in the epilogue.
LMOE_API int lmoe_gemm_dense_bias(const void* A, int lda, int a_mn, const void* B, int ldb, int b_mn, void* C, int ldc,
                                  const void* bias, int M, int N, int K, int band, int* err, int num_sms, cudaStream_t st) {
    return gemm_dense_impl(A, lda, a_mn, B, ldb, b_mn, C, ldc, 0, M, N, K, band, err, num_sms, st, bias);
}

// act[M,F] = silu(x Wg^T) * (x Wu^T) with W = [Wg ; Wu] of shape [2F, K] (pitch ldw); if Y != null the pre-activations
// x W^T go to Y [M, 2F] (pitch ldy).  F % 8 == 0, K % 8 == 0.
LMOE_API int lmoe_gemm_dense_swiglu(const void* X, int ldx, const void* W, int ldw, void* act, int ldact, void* Y, int ldy,
                                    int M, int F, int K, int band, int* err, int num_sms, cudaStream_t st) {
    if (M <= 0 || F <= 0 || K <= 0) return -1;
    if (ldx % 8 || ldw % 8 || K % 8 || F % 8 || ldact % 8 || (Y != nullptr && ldy % 8)) return -1;
    if (((uintptr_t)X | (uintptr_t)W | (uintptr_t)act | (uintptr_t)Y) & 15) return -2;
    CUtensorMap ma, mb, mc, my;
    int rc = make_map(&ma, X, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, 128);
    if (rc) return rc;
    rc = make_map(&mb, W, (uint64_t)(2 * F), (uint64_t)K, (uint64_t)ldw, 128);
    if (rc) return rc;
    rc = make_map_any(&mc, act, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, F, ldact, 64, 32);
    if (rc) return rc;
    my = mc;
    if (Y != nullptr) {
        rc = make_map_any(&my, Y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, 2 * F, ldy, 64, 32);
        if (rc) return rc;
    }
    Params p;
    p.M = M; p.N = F; p.K = K; p.band = band > 0 ? band : 8; p.f_half = F; p.err = err; p.bias = nullptr;
    return launch<false, false, 0, 1>(ma, mb, mc, my, Y != nullptr ? 1 : 0, p, num_sms, st);
}

// dPre[M,2F] = SwiGLU'(Pre[M,2F]) applied to dAct = dY[M,H] * W2[H,F] (W2 as stored: [H, F] row-major, pitch ldw), with the
// activation gradient in the GEMM epilogue (dAct is never written).  F % 64 == 0, H % 8 == 0.
LMOE_API int lmoe_gemm_dense_dswiglu(const void* dY, int lddy, const void* W2, int ldw, const void* pre, int ldpre, void* dpre,
                                     int lddpre, int M, int F, int H, int band, int* err, int num_sms, cudaStream_t st) {
    if (M <= 0 || F <= 0 || H <= 0) return -1;
    if (lddy % 8 || ldw % 8 || H % 8 || F % 64 || ldpre % 8 || lddpre % 8) return -1;   // 64-column slabs must not straddle F
    if (((uintptr_t)dY | (uintptr_t)W2 | (uintptr_t)pre | (uintptr_t)dpre) & 15) return -2;
    CUtensorMap ma, mb, mc, my;
    int rc = make_map(&ma, dY, (uint64_t)M, (uint64_t)H, (uint64_t)lddy, 128);
    if (rc) return rc;
    rc = make_map(&mb, W2, (uint64_t)H, (uint64_t)F, (uint64_t)ldw, 64);                      // MN-major B: [K = H rows, N = F cols]
    if (rc) return rc;
    rc = make_map_any(&mc, dpre, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, 2 * F, lddpre, 64, 32);
    if (rc) return rc;
    rc = make_map_any(&my, pre, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, 2 * F, ldpre, 64, 32);
    if (rc) return rc;
    Params p;
    p.M = M; p.N = F; p.K = H; p.band = band > 0 ? band : 8; p.f_half = F; p.err = err; p.bias = nullptr;
    return launch<false, true, 0, 2>(ma, mb, mc, my, 1, p, num_sms, st);
}
