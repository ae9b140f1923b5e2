// Expert-parallel token exchange of the MoE layer over NVLink peer memory: no NCCL all-to-all, no host sync.
//
// Replaces the reference's permute -> all_to_all -> permute ... unpermute -> all_to_all -> unpermute chain
// (moe/token_dispatcher.py:412-548, whose split sizes are read back by the host with .tolist()) with
//
//   moe_exchange_kernel   sums the chunk histograms; every rank stores its per-expert token counts into every peer's count matrix, releases a
//                         flag, waits (bounded) for the peers' rows and derives, on the device: the padded row
//                         offsets of its local experts in its receive buffer (the grouped GEMM's problem sizes) and,
//                         for every global expert, the row in the owner's receive buffer where THIS rank's tokens
//                         for that expert start.
//   moe_count_kernel      per-chunk histograms of the (token, slot) -> expert assignments (chunks of 4096 assignments).
//   moe_assign_kernel     destination (rank, row) of every (token, slot) pair: a counting sort that is stable in the
//                         assignment index (deterministic row order), without any library sort.
//   moe_push_kernel       dispatch: every (token, slot) row is written straight into the owner rank's receive buffer
//                         with 16-byte peer stores (optionally scaled, which is the backward of the combine); the
//                         last CTA to finish releases a flag on every peer and waits for theirs.
//   moe_zero_pads_kernel  clears the padding rows behind every expert segment so that the weight-gradient GEMMs,
//                         which contract over the padded rows, see zeros.
//   moe_signal_kernel     "my expert outputs are complete" flag to every peer.
//   moe_pull_kernel       combine: waits for the owners' flags, then every token gathers its k expert outputs from
//                         the owners' result buffers with 16-byte peer loads, weights them by the routing
//                         probabilities and sums them in fp32 (un-permute + weighted sum + all-to-all in one pass).
//
// Buffers are symmetric allocations shared by all MoE layers; a push/pull pair of one layer is ordered against the
// next layer's by the flags themselves (a rank starts its next push only after its pull, which waited for every owner's
// compute; an owner overwrites its result buffer only after every peer's next push).  Flags carry monotonically
// increasing epochs.  Every spin is bounded: on expiry the kernel records {kernel, peer} in the status word and goes
// on (results are then wrong but finite, every address stays in bounds) and the host raises after the step.
#include "common.cuh"

namespace lmoe {

__device__ __forceinline__ void moe_st_rel(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;\n" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int moe_ld_acq(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct MoeArgs {
    int* const* peer_cnt;       // [W] count matrices, int32 [W(src)][E]
    int* const* peer_flags;     // [W] flag arrays, int32 [3][W(src)]: counts ready / push done / outputs ready
    bf16* const* peer_x;        // [W] receive buffers [cap][h]
    bf16* const* peer_y;        // [W] result buffers [cap][h]
    int* status;
    unsigned int* done_ctr;
    int rank, world, E, El, cap, h;
    int epoch;
    long long spin_limit;
    // exchange
    int* offs;                  // [El+1] out: padded row offsets of the local experts
    int* real;                  // [El]   out: tokens received per local expert
    int* send_base;             // [E]    out: first row of this rank's tokens in the owner's buffer, -1 = do not send
    // count / assign
    const long long* idx;       // [n_assign] expert id of every (token, slot) pair, -1 = dropped
    int* blockhist;             // [nchunks][E] assignments per chunk and expert
    int* blockbase;             // [nchunks][E] exclusive prefix of blockhist over the chunks
    int nchunks;
    int* dest_rank;             // [n_assign]
    int* dest_row;              // [n_assign]
    // push / pull
    const bf16* src;            // [T][h]
    const float* w;             // [n_assign] or null
    bf16* out;                  // [T][h]
    bf16* rows;                 // [n_assign][h] or null: the gathered rows, unweighted
    int n_assign, k;
    int pad;                    // expert segments in the receive buffer start at multiples of `pad` rows
};

// wait until flags[phase][j] >= epoch for every peer j; one thread per peer.  Returns through smem `fail`.
__device__ __forceinline__ void moe_wait_all(const MoeArgs& a, int phase, int code, int* fail) {
    if ((int)threadIdx.x < a.world) {
        const int* f = a.peer_flags[a.rank] + phase * a.world + threadIdx.x;
        long long spins = 0;
        while (moe_ld_acq(f) < a.epoch) {
            if (++spins > a.spin_limit) {
                atomicCAS(a.status, 0, (9 << 24) | ((int)threadIdx.x << 16) | code);
                *fail = 1;
                break;
            }
            __nanosleep(64);
        }
    }
}

__global__ void moe_exchange_kernel(MoeArgs a) {
    extern __shared__ int sm[];
    int* tot = sm;                 // [E]
    int* prior = sm + a.E;         // [E]
    int* over = sm + 2 * a.E;      // [W]
    __shared__ int fail;
    if (threadIdx.x == 0) fail = 0;
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
        int c = 0;
        for (int ch = 0; ch < a.nchunks; ++ch) {                     // exclusive prefix over the chunks, total = this rank's count
            a.blockbase[ch * a.E + e] = c;
            c += a.blockhist[ch * a.E + e];
        }
        for (int j = 0; j < a.world; ++j) a.peer_cnt[j][a.rank * a.E + e] = c;
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < a.world) moe_st_rel(a.peer_flags[threadIdx.x] + 0 * a.world + a.rank, a.epoch);
    moe_wait_all(a, 0, 1, &fail);
    __syncthreads();
    const int* cnt = a.peer_cnt[a.rank];
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) {
        int t = 0, p = 0;
        for (int s = 0; s < a.world; ++s) {
            const int c = fail ? 0 : max(__ldcg(cnt + s * a.E + e), 0);
            if (s < a.rank) p += c;
            t += c;
        }
        tot[e] = t;
        prior[e] = p;
    }
    __syncthreads();
    if ((int)threadIdx.x < a.world) {
        const int d = threadIdx.x;
        long long run = 0;
        for (int el = 0; el < a.El; ++el) run += (tot[d * a.El + el] + a.pad - 1) / a.pad * a.pad;
        over[d] = run > a.cap;
        if (run > a.cap) atomicCAS(a.status, 0, (9 << 24) | (d << 16) | 7);        // receive buffer of rank d too small
    }
    __syncthreads();
    if ((int)threadIdx.x < a.world) {
        const int d = threadIdx.x;
        int run = 0;
        for (int el = 0; el < a.El; ++el) {
            const int e = d * a.El + el;
            a.send_base[e] = over[d] ? -1 : run + prior[e];
            if (d == a.rank) { a.offs[el] = over[d] ? 0 : run; a.real[el] = over[d] ? 0 : tot[e]; }
            run += (tot[e] + a.pad - 1) / a.pad * a.pad;
        }
        if (d == a.rank) a.offs[a.El] = over[d] ? 0 : run;
    }
}

constexpr int ASSIGN_CHUNK = 4096, ASSIGN_PER_THREAD = 16;          // 256 threads x 16 consecutive assignments

// grid = nchunks: histogram of one chunk of assignments
__global__ void moe_count_kernel(MoeArgs a) {
    extern __shared__ int hist[];
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const long long base = (long long)blockIdx.x * ASSIGN_CHUNK;
    for (int i = threadIdx.x; i < ASSIGN_CHUNK; i += blockDim.x) {
        const long long p = base + i;
        if (p < a.n_assign) {
            const long long e = a.idx[p];
            if (e >= 0 && e < a.E) atomicAdd(&hist[e], 1);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < a.E; e += blockDim.x) a.blockhist[blockIdx.x * a.E + e] = hist[e];
}

// grid = nchunks, 256 threads, dynamic smem 256 * E * 2 bytes: thread t owns assignments [16 t, 16 t + 16) of the chunk
__global__ void moe_assign_kernel(MoeArgs a) {
    extern __shared__ unsigned short cnt[];                          // [256][E] -> exclusive prefix over the threads
    const int t = threadIdx.x;
    unsigned short* mine = cnt + t * a.E;
    for (int e = 0; e < a.E; ++e) mine[e] = 0;
    const long long base = (long long)blockIdx.x * ASSIGN_CHUNK + (long long)t * ASSIGN_PER_THREAD;
    long long ev[ASSIGN_PER_THREAD];
#pragma unroll
    for (int i = 0; i < ASSIGN_PER_THREAD; ++i) {
        const long long p = base + i;
        long long e = p < a.n_assign ? a.idx[p] : -1;
        if (e >= a.E) e = -1;
        ev[i] = e;
        if (e >= 0) mine[e]++;
    }
    __syncthreads();
    for (int e = t; e < a.E; e += blockDim.x) {
        unsigned int run = 0;
        for (int r = 0; r < (int)blockDim.x; ++r) {
            const unsigned short c = cnt[r * a.E + e];
            cnt[r * a.E + e] = (unsigned short)run;
            run += c;
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < ASSIGN_PER_THREAD; ++i) {
        const long long p = base + i;
        if (p >= a.n_assign) break;
        const long long e = ev[i];
        int dr = -1, row = -1;
        if (e >= 0) {
            const int pos = mine[e]++;
            const int sb = a.send_base[e];
            if (sb >= 0) { dr = (int)e / a.El; row = sb + a.blockbase[blockIdx.x * a.E + e] + pos; }
            if (row >= a.cap) { dr = -1; row = -1; }
        }
        a.dest_rank[p] = dr;
        a.dest_row[p] = row;
    }
}

__global__ void moe_push_kernel(MoeArgs a) {
    __shared__ int fail, last;
    const int wpb = blockDim.x >> 5, l = threadIdx.x & 31;
    const int vecs = a.h / 8;
    for (long long as = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); as < a.n_assign; as += (long long)gridDim.x * wpb) {
        const int dr = a.dest_rank[as];
        if (dr < 0) continue;
        const uint4* s = reinterpret_cast<const uint4*>(a.src + (as / a.k) * a.h);
        uint4* d = reinterpret_cast<uint4*>(a.peer_x[dr] + (long long)a.dest_row[as] * a.h);
        if (a.w == nullptr) {
            for (int c = l; c < vecs; c += 32) d[c] = s[c];
        } else {
            const float wt = a.w[as];
            for (int c = l; c < vecs; c += 32) {
                uint4 v = s[c];
                __nv_bfloat162* hv = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float2 f = __bfloat1622float2(hv[i]);
                    hv[i] = __floats2bfloat162_rn(f.x * wt, f.y * wt);
                }
                d[c] = v;
            }
        }
    }
    // grid-wide completion -> flag to every peer -> wait for every peer's flag
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        fail = 0;
        last = atomicAdd(a.done_ctr, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!last) return;
    __threadfence_system();
    if ((int)threadIdx.x < a.world) moe_st_rel(a.peer_flags[threadIdx.x] + 1 * a.world + a.rank, a.epoch);
    moe_wait_all(a, 1, 2, &fail);
    if (threadIdx.x == 0) *a.done_ctr = 0;
}

// grid (El, chunks): zero rows [offs[el] + real[el], offs[el+1]) of the local receive buffer
__global__ void moe_zero_pads_kernel(MoeArgs a) {
    const int el = blockIdx.x;
    const int lo = a.offs[el] + a.real[el], hi = min(a.offs[el + 1], a.cap);
    const int vecs = a.h / 8;
    uint4* x = reinterpret_cast<uint4*>(a.peer_x[a.rank]);
    const long long n = (long long)max(hi - lo, 0) * vecs;
    for (long long i = (long long)blockIdx.y * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.y * blockDim.x)
        x[(long long)lo * vecs + i] = make_uint4(0, 0, 0, 0);
}

__global__ void moe_signal_kernel(MoeArgs a) {
    __threadfence_system();
    if ((int)threadIdx.x < a.world) moe_st_rel(a.peer_flags[threadIdx.x] + 2 * a.world + a.rank, a.epoch);
}

template <int KMAX>
__global__ void moe_pull_kernel(MoeArgs a) {
    __shared__ int fail;
    if (threadIdx.x == 0) fail = 0;
    __syncthreads();
    moe_wait_all(a, 2, 3, &fail);
    __syncthreads();
    const int wpb = blockDim.x >> 5, l = threadIdx.x & 31;
    const int vecs = a.h / 8;
    const int T = a.n_assign / a.k;
    for (long long t = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += (long long)gridDim.x * wpb) {
        const uint4* rp[KMAX];
        float wt[KMAX];
#pragma unroll
        for (int j = 0; j < KMAX; ++j) {
            rp[j] = nullptr;
            wt[j] = 0.f;
            if (j < a.k) {
                const int dr = a.dest_rank[t * a.k + j];
                if (dr >= 0) {
                    rp[j] = reinterpret_cast<const uint4*>(a.peer_y[dr] + (long long)a.dest_row[t * a.k + j] * a.h);
                    wt[j] = a.w != nullptr ? a.w[t * a.k + j] : 1.f;
                }
            }
        }
        for (int c = l; c < vecs; c += 32) {
            uint4 v[KMAX];
#pragma unroll
            for (int j = 0; j < KMAX; ++j) v[j] = rp[j] != nullptr ? __ldcg(rp[j] + c) : make_uint4(0, 0, 0, 0);
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < KMAX; ++j) {
                const __nv_bfloat162* hv = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float2 f = __bfloat1622float2(hv[i]);
                    acc[2 * i] += wt[j] * f.x;
                    acc[2 * i + 1] += wt[j] * f.y;
                }
                if (a.rows != nullptr && j < a.k)
                    reinterpret_cast<uint4*>(a.rows + (t * a.k + j) * a.h)[c] = v[j];
            }
            uint4 o;
            __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) ho[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
            reinterpret_cast<uint4*>(a.out + t * a.h)[c] = o;
        }
    }
}

// Gradient of the routing probabilities in the combine: d_probs[t, j] = <rows[t * k + j, :], d_out[t, :]> (zero for a
// dropped assignment).  One warp per token: the token's output gradient is read once per 256-element piece and reused
// for its k gathered rows.  (A batched matrix product with one output column per batch runs this at a fraction of the
// memory bandwidth.)
template <int KMAX>
__global__ void moe_dprobs_kernel(const bf16* __restrict__ rows, const bf16* __restrict__ d_out, const int* __restrict__ dest_rank,
                                  float* __restrict__ d_probs, int T, int k, int h) {
    const int wpb = blockDim.x >> 5, l = threadIdx.x & 31;
    for (long long t = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); t < T; t += (long long)gridDim.x * wpb) {
        float acc[KMAX];
#pragma unroll
        for (int j = 0; j < KMAX; ++j) acc[j] = 0.f;
        const uint4* dp = reinterpret_cast<const uint4*>(d_out + t * h);
        for (int c = l; c < h / 8; c += 32) {
            const uint4 dv = __ldg(dp + c);
            const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv);
            float2 df[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) df[i] = __bfloat1622float2(d2[i]);
#pragma unroll
            for (int j = 0; j < KMAX; ++j) {
                if (j < k) {
                    const uint4 rv = __ldcs(reinterpret_cast<const uint4*>(rows + (t * k + j) * h) + c);
                    const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 rf = __bfloat1622float2(r2[i]);
                        acc[j] += rf.x * df[i].x + rf.y * df[i].y;
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < KMAX; ++j) {
            if (j < k) {
                float v = acc[j];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (l == 0) d_probs[t * k + j] = dest_rank[t * k + j] >= 0 ? v : 0.f;
            }
        }
    }
}

}  // namespace lmoe

using namespace lmoe;

// which: 0 exchange, 1 assign, 2 push, 3 zero pads, 4 signal, 5 pull, 6 count
LMOE_API int lmoe_moe_comm(int which, const MoeArgs* ap, int num_sms, cudaStream_t st) {
    const MoeArgs a = *ap;
    if (a.h % 8 != 0 || a.world > 32) return -2;
    const int T = a.k > 0 ? a.n_assign / a.k : 0;
    switch (which) {
    case 0:
        moe_exchange_kernel<<<1, 256, (2 * a.E + a.world) * sizeof(int), st>>>(a);
        break;
    case 1:
        if (a.nchunks > 0) {
            const size_t sm = (size_t)256 * a.E * sizeof(unsigned short);
            if (sm > 200 * 1024) return -4;
            cudaFuncSetAttribute(moe_assign_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
            moe_assign_kernel<<<a.nchunks, 256, sm, st>>>(a);
        }
        break;
    case 6:
        if (a.nchunks > 0) moe_count_kernel<<<a.nchunks, 256, a.E * sizeof(int), st>>>(a);
        break;
    case 2: {
        int grid = (int)std::min<long long>(std::max<long long>((a.n_assign + 7) / 8, 1), (long long)num_sms * 8);
        moe_push_kernel<<<grid, 256, 0, st>>>(a);
        break;
    }
    case 3:
        moe_zero_pads_kernel<<<dim3(a.El, 8), 256, 0, st>>>(a);
        break;
    case 4:
        moe_signal_kernel<<<1, 32, 0, st>>>(a);
        break;
    case 5: {
        int grid = (int)std::min<long long>(std::max<long long>((T + 7) / 8, 1), (long long)num_sms * 8);
        if (a.k <= 2) moe_pull_kernel<2><<<grid, 256, 0, st>>>(a);
        else if (a.k <= 4) moe_pull_kernel<4><<<grid, 256, 0, st>>>(a);
        else if (a.k <= 8) moe_pull_kernel<8><<<grid, 256, 0, st>>>(a);
        else if (a.k <= 16) moe_pull_kernel<16><<<grid, 256, 0, st>>>(a);
        else return -3;
        break;
    }
    default:
        return -1;
    }
    return (int)cudaGetLastError();
}

// d_probs [T, k] fp32 from the gathered expert outputs rows [T * k, h] (bf16) and the combine's output gradient
// d_out [T, h] (bf16); h a multiple of 8, k <= 16.
LMOE_API int lmoe_moe_dprobs(const void* rows, const void* d_out, const int* dest_rank, float* d_probs, int T, int k, int h,
                             int num_sms, cudaStream_t st) {
    if (T <= 0) return 0;
    if (h % 8 != 0 || k <= 0 || k > 16) return -1;
    const int grid = (int)std::min<long long>(((long long)T + 7) / 8, (long long)num_sms * 8);
    const bf16* r = (const bf16*)rows;
    const bf16* d = (const bf16*)d_out;
    if (k <= 2) moe_dprobs_kernel<2><<<grid, 256, 0, st>>>(r, d, dest_rank, d_probs, T, k, h);
    else if (k <= 4) moe_dprobs_kernel<4><<<grid, 256, 0, st>>>(r, d, dest_rank, d_probs, T, k, h);
    else if (k <= 8) moe_dprobs_kernel<8><<<grid, 256, 0, st>>>(r, d, dest_rank, d_probs, T, k, h);
    else moe_dprobs_kernel<16><<<grid, 256, 0, st>>>(r, d, dest_rank, d_probs, T, k, h);
    return (int)cudaGetLastError();
}
