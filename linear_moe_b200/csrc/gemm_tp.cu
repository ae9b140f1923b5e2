// Tensor-parallel linear layers under sequence parallelism with the collective inside the GEMM kernel
// (tcgen05 / TMA / TMEM tiles, NVLink peer memory for the transfer).
//
//   mode 0  all-gather -> GEMM   C[M_full, N] = gather_r(A_r)[M_full, K] * B      (column-parallel forward: QKV / FC1 /
//           in_proj; row-parallel input gradient).  Every rank publishes its activation shard A_r [M_loc, K] in a
//           symmetric buffer and raises a flag on its peers.  The first `n_copy` CTAs of this kernel are copiers: after
//           a bounded acquire-wait on a peer's flag they pull that peer's shard over NVLink, 128 rows at a time, into
//           the local gathered matrix (each remote byte crosses the link once) and release a per-row-block flag.  The
//           other CTAs are GEMM workers: tiles of the local shard (read from the own symmetric buffer) are scheduled
//           first, so the remote shards arrive while the tensor cores work on local data; the TMA producer of a tile
//           on remote rows waits (bounded) for that row block's flag and reads it from local memory.  All CTAs of the
//           launch are co-resident (grid <= number of SMs, one CTA per SM).  The gathered matrix also serves the
//           weight-gradient GEMM of the backward pass.
//   mode 1  GEMM -> reduce-scatter   each rank holds a K-slice and computes the partial C[M_full, N]; the epilogue
//           stores every tile (bf16) into the owner rank's inbox slot [src = this rank] with 16-byte peer stores,
//           tiles of the other ranks first.  The last CTA raises a flag on every peer.  tp_reduce_kernel on the owner
//           waits (bounded) for all sources and sums the W partials in fp32.
// They replace gather_from_sequence_parallel_region + GEMM and GEMM + reduce_scatter_to_sequence_parallel_region of
// Megatron's Column/RowParallelLinear, which every layer spec of the reference uses (qwen2/layer_specs.py:94-96,
// linear_attention.py:66 'qkv', mlp.py:93 'fc1').
//
// Row order: activations are [batch, tokens, features] and the sequence is split along tokens, so gathered row
// b * (W * T_loc) + r * T_loc + t is row b * T_loc + t of rank r.  T_loc is a multiple of 128: a tile never straddles
// two ranks.
//
// B may be K-major ([N, K], y = x W^T) or MN-major ([K, N], dx = dy W).  Waits on mbarriers and flags are bounded by a
// clock64 budget; on expiry the error/status word is set, the CTA drains and frees its tensor memory, and the host
// raises after the step.
#include "tcgen05_utils.cuh"

namespace lmoe {
namespace tp {
using namespace lmoe::tc;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr int MAX_W = 8;

struct __align__(1024) Smem {
    uint8_t tiles[STAGES][STAGE_BYTES];
    uint8_t stage_out[4][32 * 128];            // epilogue staging, one per epilogue warp
    uint64_t full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    int last;
};

struct Maps { CUtensorMap m[MAX_W]; };

struct Params {
    int mode;                   // 0 all-gather -> GEMM, 1 GEMM -> reduce-scatter
    int rank, world;
    int M_loc, T_loc;           // rows of one rank's shard (batch * T_loc), tokens per batch entry of one rank
    int N, K;
    int ldc;
    bf16* C;                    // mode 0: local output [M_full, N]
    bf16* const* peer_inbox;    // mode 1: inbox base pointers of every rank
    long long inbox_off;        // mode 1: element offset of this call's slot: layout [W(src)][M_loc][N]
    int* const* peer_flags;     // flag arrays: [2][W(src)] (0: shard published, 1: partial tiles delivered)
    int epoch;
    unsigned int* done_ctr;
    int* status;                // fused-communication status word (bounded flag waits)
    int* err;                   // GEMM error word (bounded mbarrier waits)
    long long spin_cycles;
    // mode 0: gather by copier CTAs
    const bf16* const* peer_x;  // [W] published shards of this call ([M_loc, K] each)
    bf16* gathered;             // local [M_full, K]: remote rows are written here (the local rows too, by the host copy)
    int* ready;                 // [W * M_loc / 128] epoch per (source rank, row block) of `gathered`
    int n_copy;                 // number of copier CTAs (0 when world == 1)
};

__device__ __forceinline__ void st_rel_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;\n" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acq_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_rel_gpu(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;\n" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acq_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Copier CTA: pull 128-row blocks of the peers' shards into the local gathered matrix.  One thread drives bulk copies
// (peer global -> shared memory ring -> local global), which keeps 3 x 48 KiB in flight per CTA over NVLink without
// spending registers or issue slots; a row block is contiguous on both sides.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(s32(dst)), "l"(src), "r"(bytes), "r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" :: "l"(dst), "r"(s32(src)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <class SmemT>
__device__ __forceinline__ void copier_loop(const Params& p, int copier, SmemT& sm) {
    if (threadIdx.x != 0) return;
    volatile int* abort_flag = &sm.abort_flag;
    const int tpr = p.M_loc / BM;
    const long long block_bytes = (long long)BM * p.K * 2;
    unsigned ready_mask = 0;
    int it = 0;                                                 // pieces issued so far (ring position)
    for (int idx = copier; idx < (p.world - 1) * tpr; idx += p.n_copy) {
        const int s = idx / tpr + 1, j = idx - (s - 1) * tpr;
        const int src = (p.rank + s) % p.world;
        if (!((ready_mask >> src) & 1u)) {
            const int* f = p.peer_flags[p.rank] + src;
            const long long t0 = clock64();
            while (ld_acq_sys(f) < p.epoch) {
                if (clock64() - t0 > p.spin_cycles) { atomicCAS(p.status, 0, (10 << 24) | (src << 16) | 4); return; }
                __nanosleep(100);
            }
            asm volatile("fence.proxy.async.global;" ::: "memory");
            ready_mask |= 1u << src;
        }
        const int local_row = j * BM;
        const int b = local_row / p.T_loc, tt = local_row - b * p.T_loc;
        const long long full_row = (long long)b * p.world * p.T_loc + (long long)src * p.T_loc + tt;
        const uint8_t* in = reinterpret_cast<const uint8_t*>(p.peer_x[src]) + (long long)local_row * p.K * 2;
        uint8_t* out = reinterpret_cast<uint8_t*>(p.gathered) + full_row * p.K * 2;
        const int pieces = (int)((block_bytes + STAGE_BYTES - 1) / STAGE_BYTES);
        const int lag = STAGES - 1;
        const int it0 = it;
        for (int i = 0; i < pieces + lag; ++i) {
            if (i < pieces) {
                const int st = (it0 + i) % STAGES;
                // the store that last read this stage was committed in the previous iteration
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                const uint32_t bytes = (uint32_t)min((long long)STAGE_BYTES, block_bytes - (long long)i * STAGE_BYTES);
                mbar_expect_tx(&sm.full[st], bytes);
                bulk_g2s(sm.tiles[st], in + (long long)i * STAGE_BYTES, bytes, &sm.full[st]);
            }
            const int jj = i - lag;
            if (jj >= 0) {
                const int st = (it0 + jj) % STAGES;
                const uint32_t ph = ((it0 + jj) / STAGES) & 1;
                if (!mbar_wait(&sm.full[st], ph, abort_flag, p.err, 0x700 | st)) return;
                const uint32_t bytes = (uint32_t)min((long long)STAGE_BYTES, block_bytes - (long long)jj * STAGE_BYTES);
                bulk_s2g(out + (long long)jj * STAGE_BYTES, sm.tiles[st], bytes);
            }
        }
        it = it0 + pieces;
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the block is in local memory
        __threadfence();
        st_rel_gpu(p.ready + src * tpr + j, p.epoch);
    }
}

struct Tile {
    int peer;        // mode 0: source rank of the A tile; mode 1: owner rank of the C tile
    int local_row;   // first row inside that rank's shard
    int full_row;    // first row in gathered order
    int tn;
    int cols_valid;
};

__device__ __forceinline__ bool decode_tile(const Params& p, int t, Tile& o) {
    const int tpr = p.M_loc / BM, tiles_n = (p.N + BN - 1) / BN;
    const int per = tpr * tiles_n;
    if (t >= per * p.world) return false;
    const int s = t / per, rem = t - s * per;
    o.tn = rem / tpr;
    const int j = rem - o.tn * tpr;
    o.peer = (p.rank + (p.mode == 0 ? s : s + 1)) % p.world;
    o.local_row = j * BM;
    const int b = o.local_row / p.T_loc, tt = o.local_row - b * p.T_loc;
    o.full_row = b * p.world * p.T_loc + o.peer * p.T_loc + tt;
    o.cols_valid = p.N - o.tn * BN;
    return true;
}

template <bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tp_kernel(const __grid_constant__ Maps mapsA, const __grid_constant__ CUtensorMap tmB, Params p) {
    extern __shared__ uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = &sm.abort_flag;
    int* err = p.err;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sm.tmem_full[b], 1); mbar_init(&sm.tmem_empty[b], 4); }
        sm.abort_flag = 0;
        sm.last = 0;
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
    const int kblocks = (p.K + BK - 1) / BK;
    const int n_copy = p.mode == 0 ? p.n_copy : 0;
    const int worker = (int)blockIdx.x - n_copy, workers = (int)gridDim.x - n_copy;
    const int tpr = p.M_loc / BM;

    if (worker < 0) {
        // copier CTA (mode 0): no tensor-core work
        copier_loop(p, (int)blockIdx.x, sm);
    } else if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            Tile t;
            for (int tile = worker; !*abort_flag && decode_tile(p, tile, t); tile += workers) {
                const bool remote = p.mode == 0 && t.peer != p.rank;
                if (remote) {
                    const int* f = p.ready + t.peer * tpr + t.local_row / BM;
                    const long long t0 = clock64();
                    bool ok = true;
                    while (ld_acq_gpu(f) < p.epoch) {
                        if (clock64() - t0 > p.spin_cycles) { ok = false; break; }
                        __nanosleep(100);
                    }
                    if (!ok) {
                        atomicCAS(p.status, 0, (10 << 24) | (t.peer << 16) | 1);
                        *abort_flag = 1;
                        break;
                    }
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                }
                // mode 0: own rows from the own published shard (map 0), remote rows from the gathered matrix (map 1)
                const CUtensorMap* ma = remote ? &mapsA.m[1] : &mapsA.m[0];
                const int a_row = (p.mode == 0 && !remote) ? t.local_row : t.full_row;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!mbar_wait(&sm.empty[s], ph ^ 1, abort_flag, err, 0x100 | s)) goto producer_done;
                    mbar_expect_tx(&sm.full[s], STAGE_BYTES);
                    uint8_t* sa = sm.tiles[s];
                    uint8_t* sb = sa + A_BYTES;
                    tma_load_2d(sa, ma, &sm.full[s], kb * BK, a_row);
                    if (!B_MN) {
                        tma_load_2d(sb, &tmB, &sm.full[s], kb * BK, t.tn * BN);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_2d(sb + j * 8192, &tmB, &sm.full[s], t.tn * BN + j * 64, kb * BK);
                    }
                }
            }
        }
    producer_done:;
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc<false, B_MN, BM, BN>();
            int it = 0, lt = 0;
            Tile t;
            for (int tile = worker; !*abort_flag && decode_tile(p, tile, t); tile += workers, ++lt) {
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
                        const uint64_t ad = make_desc<false>(a_addr + k * UMMA_K * 2);
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
        for (int tile = worker; decode_tile(p, tile, t); tile += workers, ++lt) {
            const int buf = lt & 1;
            const uint32_t aph = (lt >> 1) & 1;
            if (!mbar_wait(&sm.tmem_full[buf], aph, abort_flag, err, 0x400 | buf)) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;
            // first of this warp's 32 output rows; mode 1 writes into the owner rank's inbox slot [src = this rank]
            bf16* cbase;
            long long ld;
            if (p.mode == 0) { cbase = p.C + (long long)(t.full_row + q * 32) * p.ldc + (long long)t.tn * BN; ld = p.ldc; }
            else { cbase = p.peer_inbox[t.peer] + p.inbox_off + ((long long)p.rank * p.M_loc + t.local_row + q * 32) * p.N + (long long)t.tn * BN; ld = p.N; }
            uint8_t* stg = sm.stage_out[warp - 2];                       // 32 rows x 128 bytes, 16-byte chunks xor-swizzled
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
                        o.x = pack_bf16(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]));
                        o.y = pack_bf16(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
                        o.z = pack_bf16(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
                        o.w = pack_bf16(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
                        *reinterpret_cast<uint4*>(stg + lane * 128 + (((hc * 4 + g) ^ (lane & 7)) << 4)) = o;
                    }
                }
                __syncwarp();
                // 8 lanes write one row's 128 contiguous bytes (whole lines, also over NVLink in mode 1)
                const int chunk = lane & 7;
                const int col = c + chunk * 8;
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int rr = it * 4 + (lane >> 3);
                    const uint4 o = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((chunk ^ (rr & 7)) << 4));
                    if (col + 8 <= t.cols_valid) *reinterpret_cast<uint4*>(cbase + (long long)rr * ld + col) = o;
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.tmem_empty[buf]);
        }
        if (p.mode == 1) __threadfence_system();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (p.mode == 1) {
        // the last CTA of the grid tells every peer that this rank's partial tiles are in its inbox
        if (threadIdx.x == 0) {
            __threadfence_system();
            sm.last = atomicAdd(p.done_ctr, 1u) == gridDim.x - 1;
        }
        __syncthreads();
        if (sm.last) {
            __threadfence_system();
            if ((int)threadIdx.x < p.world) st_rel_sys(p.peer_flags[threadIdx.x] + p.world + p.rank, p.epoch);
            if (threadIdx.x == 0) *p.done_ctr = 0;
        }
    }
}

struct CommArgs {
    int* const* peer_flags;
    bf16* const* peer_x;        // published shards
    bf16* const* peer_inbox;
    long long x_off, inbox_off;
    int* status;
    int rank, world, epoch;
    int M_loc, T_loc, cols;
    bf16* out;                  // reduce: [M_loc, cols]; gather: [M_full, cols]
    long long spin_limit;
};

__device__ __forceinline__ bool wait_flags(const CommArgs& a, int phase, int code) {
    __shared__ int fail;
    if (threadIdx.x == 0) fail = 0;
    __syncthreads();
    if ((int)threadIdx.x < a.world) {
        const int* f = a.peer_flags[a.rank] + phase * a.world + threadIdx.x;
        long long spins = 0;
        while (ld_acq_sys(f) < a.epoch) {
            if (++spins > a.spin_limit) {
                atomicCAS(a.status, 0, (10 << 24) | ((int)threadIdx.x << 16) | code);
                fail = 1;
                break;
            }
            __nanosleep(64);
        }
    }
    __syncthreads();
    return fail == 0;
}

// "my shard is published": flag phase 0 on every peer
__global__ void tp_signal_kernel(CommArgs a) {
    __threadfence_system();
    if ((int)threadIdx.x < a.world) st_rel_sys(a.peer_flags[threadIdx.x] + 0 * a.world + a.rank, a.epoch);
}

// out[r, c] = sum over sources of inbox[src][r, c]
__global__ void tp_reduce_kernel(CommArgs a) {
    wait_flags(a, 1, 2);
    const long long n8 = (long long)a.M_loc * a.cols / 8;
    const uint4* in = reinterpret_cast<const uint4*>(a.peer_inbox[a.rank] + a.inbox_off);
    uint4* out = reinterpret_cast<uint4*>(a.out);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < a.world; ++s) {
            uint4 v = __ldcg(in + (long long)s * n8 + i);
            const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = __bfloat1622float2(hv[j]);
                acc[2 * j] += f.x;
                acc[2 * j + 1] += f.y;
            }
        }
        uint4 o;
        __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) ho[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        out[i] = o;
    }
}

// out[gathered row, :] = shard row of its rank (16-byte peer loads); used for the weight gradients
__global__ void tp_gather_kernel(CommArgs a) {
    wait_flags(a, 0, 3);
    const int v8 = a.cols / 8;
    const long long rows = (long long)a.M_loc * a.world;
    const long long n8 = rows * v8;
    uint4* out = reinterpret_cast<uint4*>(a.out);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / v8;
        const int c = (int)(i - row * v8);
        const long long per_b = (long long)a.world * a.T_loc;
        const long long b = row / per_b, rem = row - b * per_b;
        const int src = (int)(rem / a.T_loc);
        const long long lr = b * a.T_loc + (rem - (long long)src * a.T_loc);
        out[i] = __ldcg(reinterpret_cast<const uint4*>(a.peer_x[src] + a.x_off) + lr * v8 + c);
    }
}

}  // namespace tp
}  // namespace lmoe

using namespace lmoe;
using namespace lmoe::tp;

// mode 0: a_ptrs[0] = this rank's published shard [M_loc, K], a_ptrs[1] = local gathered matrix [M_full, K] (scratch that the
//         copier CTAs fill; also pp->gathered), pp->peer_x = device array of the W published shards, pp->n_copy copier CTAs.
// mode 1: a_ptrs[0] = local A [M_full, K].
LMOE_API int lmoe_gemm_tp(int mode, const void* const* a_ptrs, const void* B, int b_rows, int b_cols, int b_mn,
                          const Params* pp, int num_sms, cudaStream_t st) {
    Params p = *pp;
    p.mode = mode;
    if (p.world > MAX_W || p.M_loc % BM || p.T_loc % BM || p.K % 8 || p.N % 8 || b_cols % 8) return -1;
    if (mode == 0 && p.world > 1 && (p.n_copy < 1 || p.n_copy >= num_sms)) return -2;
    if (mode != 0 || p.world == 1) p.n_copy = 0;
    Maps maps;
    const uint64_t m_full = (uint64_t)p.M_loc * p.world;
    int rc = make_map(&maps.m[0], a_ptrs[0], mode == 0 ? (uint64_t)p.M_loc : m_full, (uint64_t)p.K, (uint64_t)p.K, BM);
    if (rc) return rc;
    rc = make_map(&maps.m[1], a_ptrs[mode == 0 ? 1 : 0], m_full, (uint64_t)p.K, (uint64_t)p.K, BM);
    if (rc) return rc;
    for (int i = 2; i < MAX_W; ++i) maps.m[i] = maps.m[0];
    CUtensorMap mb;
    rc = make_map(&mb, B, (uint64_t)b_rows, (uint64_t)b_cols, (uint64_t)b_cols, b_mn ? 64 : BN);
    if (rc) return rc;
    const size_t smem = sizeof(Smem) + 1024;
    // one CTA per SM and grid <= number of SMs: every CTA of the launch is resident, which the copier / worker hand-off needs
    if (b_mn) {
        cudaFuncSetAttribute(gemm_tp_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gemm_tp_kernel<true><<<num_sms, THREADS, smem, st>>>(maps, mb, p);
    } else {
        cudaFuncSetAttribute(gemm_tp_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        gemm_tp_kernel<false><<<num_sms, THREADS, smem, st>>>(maps, mb, p);
    }
    return (int)cudaGetLastError();
}

// which: 0 signal (shard published), 1 reduce, 2 gather
LMOE_API int lmoe_tp_comm(int which, const CommArgs* ap, int num_sms, cudaStream_t st) {
    const CommArgs a = *ap;
    if (a.cols % 8 || a.world > 32) return -1;
    if (which == 0) tp_signal_kernel<<<1, 32, 0, st>>>(a);
    else if (which == 1) tp_reduce_kernel<<<num_sms * 4, 256, 0, st>>>(a);
    else if (which == 2) tp_gather_kernel<<<num_sms * 4, 256, 0, st>>>(a);
    else return -2;
    return (int)cudaGetLastError();
}
