// LASP-2 state exchange fused into the combine step of the chunked scan, over NVLink peer memory.
//
// Every rank of the sequence-parallel group holds a contiguous slice of the sequence.  After the local
// state_scan (lsm_scalar.cu) a rank owns G group summaries per (batch, head).  This kernel, one launch per
// layer and direction, does in ONE pass per state element:
//   1. the local scan over the G summaries (zero seed), giving the rank summary T_r (nothing is written yet);
//   2. PUSH of T_r into slot [src = r] of every peer's symmetric buffer with plain peer stores, a system
//      fence, and a release store of the epoch number into the matching per-CTA flag on that peer;
//   3. a BOUNDED acquire-spin on the flags of the ranks this rank depends on (ranks < r forward, ranks > r
//      backward), then the decayed fold of their summaries into the entering state R;
//   4. the local exclusive scan again, seeded with R, which writes the state entering every group.
// It replaces the reference's all_gather_into_tensor + torch.sum between its Triton kernels
// (lasp2_without_mask_triton_op.py:692-708,730-746): no NCCL call, no extra kernel, and the exchange carries
// the decay, which the reference's LASP-2 does not support.
//
// Decay forms (`dmode`): 0 = none or a constant log decay per head (`gconst`, lightning attention / retention);
// 1 = data-dependent scalar decay, given as the summed log decay of every group `gdecay[BH][G]` (Mamba2 SSD, simple
// GLA with per-token gates); 2 = per key channel, `gdecay[BH][G][D]` (GLA, HGRN2, RWKV6).  In modes 1 and 2 a rank also
// publishes the summed log decay of its whole slice (one value per state row), which the ranks that fold its summary
// need; it travels in the same slot and under the same flag as the rows it belongs to.
//
// Deadlock freedom: a CTA pushes before it waits and only waits for ranks on one side, so the dependency
// graph over ranks is a chain (rank 0 / rank W-1 waits for nobody); no co-residency of CTAs is assumed.
// Every wait is bounded: on expiry the CTA records {kernel, peer, phase} in the status word, skips the fold
// (the result is then wrong but finite) and returns, so the context stays usable and the host raises.
#include "common.cuh"

namespace lmoe {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;\n" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

struct LaspArgs {
    float* states;            // [BH, G, DD] local group summaries -> entering states (in place)
    float* final_out;         // [BH, DD] state after this rank's slice (fwd) / gradient wrt entering state (bwd)
    const float* gconst;      // [H] constant log decay per head, or null (no decay); dmode 0
    const float* gdecay;      // dmode 1: [BH, G]; dmode 2: [BH, G, D] summed log decay of every group
    float* r_out;             // [BH, DD] or null: the folded remote state R (bwd: gradient wrt the state leaving this rank)
    float* const* peer_data;  // [W] base pointers of the symmetric data buffers
    int* const* peer_flags;   // [W] base pointers of the symmetric flag buffers
    int* status;              // device status word, 0 = ok
    long long data_off;       // element offset of this call's slot in every data buffer: slot layout [W(src)][BH*DD]
    long long dec_off;        // element offset of this call's decay area in every data buffer: [W(src)][BH*D]
    long long flag_off;       // int offset of this call's slot in every flag buffer: [W(src)][nctas]
    int epoch;
    int rank, world;
    int H, G, cpg, T;         // T = tokens on this rank (same on every rank)
    int DD, BH;
    int dmode, D;             // decay form; row length of the state (DD = rows x D, the decay of dmode 2 is per row)
    long long spin_limit;     // iterations of the bounded wait
};

// REV = 0: forward (depends on ranks < r); REV = 1: backward (depends on ranks > r).
template <int REV>
__global__ void lasp_combine_kernel(LaspArgs a) {
    const int bh = blockIdx.y, h = bh % a.H;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const int cta = blockIdx.y * gridDim.x + blockIdx.x;
    const int nctas = gridDim.x * gridDim.y;
    const bool active = e < a.DD;
    const float gh = a.gconst != nullptr ? a.gconst[h] : 0.f;
    const int row = active ? e / a.D : 0;
    __shared__ int failed_peer;
    if (threadIdx.x == 0) failed_peer = -1;

    // summed log decay of group g for this thread's state row
    auto group_decay = [&](int g) -> float {
        if (a.dmode == 1) return a.gdecay[(long long)bh * a.G + g];
        if (a.dmode == 2) return a.gdecay[((long long)bh * a.G + g) * a.D + row];
        const int t_lo = g * a.cpg * 64, t_hi = min(a.T, (g + 1) * a.cpg * 64);
        return gh * (float)max(t_hi - t_lo, 0);
    };

    // 1. rank summary: the local scan from a zero seed, reading the group summaries only (batches of loads in flight
    //    together; nothing is written yet, so the second pass below can redo the scan from the folded remote state)
    constexpr int NB = 8;
    float carry = 0.f, total = 0.f;
    if (active) {
        for (int i0 = 0; i0 < a.G; i0 += NB) {
            float m[NB], ld[NB];
#pragma unroll
            for (int j = 0; j < NB; ++j)
                if (i0 + j < a.G) {
                    const int g = REV ? a.G - 1 - (i0 + j) : i0 + j;
                    m[j] = __ldcg(a.states + ((long long)bh * a.G + g) * a.DD + e);
                    ld[j] = group_decay(g);
                }
#pragma unroll
            for (int j = 0; j < NB; ++j)
                if (i0 + j < a.G) {
                    carry = __expf(ld[j]) * carry + m[j];
                    total += ld[j];
                }
        }
        // 2. push the rank summary (and, for data-dependent decays, the slice's summed log decay per row) to the peers
        const long long off = a.data_off + (long long)a.rank * a.BH * a.DD + (long long)bh * a.DD + e;
        const long long doff = a.dec_off + (long long)a.rank * a.BH * a.D + (long long)bh * a.D + row;
        const bool push_decay = a.dmode != 0 && (e % a.D) == 0;
        for (int j = 0; j < a.world; ++j) {
            bool needed = REV ? (j < a.rank) : (j > a.rank);
            if (needed) {
                a.peer_data[j][off] = carry;
                if (push_decay) a.peer_data[j][doff] = total;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        for (int j = 0; j < a.world; ++j) {
            bool needed = REV ? (j < a.rank) : (j > a.rank);
            if (needed) st_release_sys(a.peer_flags[j] + a.flag_off + (long long)a.rank * nctas + cta, a.epoch);
        }
        // 3. bounded wait for the ranks this CTA depends on
        int* myflags = a.peer_flags[a.rank] + a.flag_off;
        for (int j = 0; j < a.world; ++j) {
            bool dep = REV ? (j > a.rank) : (j < a.rank);
            if (!dep) continue;
            long long spins = 0;
            while (ld_acquire_sys(myflags + (long long)j * nctas + cta) < a.epoch) {
                if (++spins > a.spin_limit) {
                    failed_peer = j;
                    atomicCAS(a.status, 0, (7 << 24) | (j << 16) | (REV ? 2 : 1));
                    break;
                }
                __nanosleep(64);
            }
            if (failed_peer >= 0) break;
        }
    }
    __syncthreads();
    if (!active) return;
    float R = 0.f;
    if (failed_peer < 0) {
        const float* mine = a.peer_data[a.rank] + a.data_off + (long long)bh * a.DD + e;
        const float* mdec = a.peer_data[a.rank] + a.dec_off + (long long)bh * a.D + row;
        const float dec_const = __expf(gh * (float)a.T);          // dmode 0: decay across one whole rank slice
        if (!REV) {
            for (int j = 0; j < a.rank; ++j) {
                const float d = a.dmode != 0 ? __expf(mdec[(long long)j * a.BH * a.D]) : dec_const;
                R = d * R + mine[(long long)j * a.BH * a.DD];
            }
        } else {
            for (int j = a.world - 1; j > a.rank; --j) {
                const float d = a.dmode != 0 ? __expf(mdec[(long long)j * a.BH * a.D]) : dec_const;
                R = d * R + mine[(long long)j * a.BH * a.DD];
            }
        }
    }
    // 4. the scan again, seeded with the folded remote state: slot g <- state entering group g (forward) / gradient of
    //    the state leaving group g (backward); the summaries are still in L2 from the first pass
    float st = R;
    for (int i0 = 0; i0 < a.G; i0 += NB) {
        float m[NB], dec[NB];
#pragma unroll
        for (int j = 0; j < NB; ++j)
            if (i0 + j < a.G) {
                const int g = REV ? a.G - 1 - (i0 + j) : i0 + j;
                m[j] = __ldcg(a.states + ((long long)bh * a.G + g) * a.DD + e);
                dec[j] = __expf(group_decay(g));
            }
#pragma unroll
        for (int j = 0; j < NB; ++j)
            if (i0 + j < a.G) {
                const int g = REV ? a.G - 1 - (i0 + j) : i0 + j;
                a.states[((long long)bh * a.G + g) * a.DD + e] = st;
                st = dec[j] * st + m[j];
            }
    }
    if (a.final_out != nullptr) a.final_out[(long long)bh * a.DD + e] = st;
    if (a.r_out != nullptr) a.r_out[(long long)bh * a.DD + e] = R;
}

}  // namespace lmoe

using namespace lmoe;

LMOE_API int lmoe_lasp_combine(int rev, const LaspArgs* ap, cudaStream_t st) {
    LaspArgs a = *ap;
    dim3 grid((a.DD + 255) / 256, a.BH);
    if (rev) lasp_combine_kernel<1><<<grid, 256, 0, st>>>(a);
    else lasp_combine_kernel<0><<<grid, 256, 0, st>>>(a);
    return (int)cudaGetLastError();
}

// Number of CTAs (= flags per source rank) of a combine launch.
LMOE_API int lmoe_lasp_num_ctas(int DD, int BH) { return ((DD + 255) / 256) * BH; }
