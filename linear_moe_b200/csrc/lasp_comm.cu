// LASP-2 state exchange fused into the combine step of the chunked scan, over NVLink peer memory.
//
// Every rank of the sequence-parallel group holds a contiguous slice of the sequence.  After the local
// state_scan (lsm_scalar.cu) a rank owns G group summaries per (batch, head).  This kernel, one launch per
// layer and direction, does in ONE pass per state element:
//   1. the local exclusive scan over the G summaries (zero seed), giving the rank summary T_r;
//   2. PUSH of T_r into slot [src = r] of every peer's symmetric buffer with plain peer stores, a system
//      fence, and a release store of the epoch number into the matching per-CTA flag on that peer;
//   3. a BOUNDED acquire-spin on the flags of the ranks this rank depends on (ranks < r forward, ranks > r
//      backward), then the decayed fold of their summaries into the entering state R;
//   4. the fix-up of the local prefix states, P_g = P_g(local) + e^{a * tokens_before_g} R.
// It replaces the reference's all_gather_into_tensor + torch.sum between its Triton kernels
// (lasp2_without_mask_triton_op.py:692-708,730-746): no NCCL call, no extra kernel, and the exchange carries
// the decay, which the reference's LASP-2 does not support.
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
    const float* gconst;      // [H] constant log decay per head, or null (no decay)
    float* const* peer_data;  // [W] base pointers of the symmetric data buffers
    int* const* peer_flags;   // [W] base pointers of the symmetric flag buffers
    int* status;              // device status word, 0 = ok
    long long data_off;       // element offset of this call's slot in every data buffer: slot layout [W(src)][BH*DD]
    long long flag_off;       // int offset of this call's slot in every flag buffer: [W(src)][nctas]
    int epoch;
    int rank, world;
    int H, G, cpg, T;         // T = tokens on this rank (same on every rank)
    int DD, BH;
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
    __shared__ int failed_peer;
    if (threadIdx.x == 0) failed_peer = -1;

    // 1. local scan (zero seed); prefix states stay in registers-free form in memory
    float carry = 0.f;
    if (active) {
        for (int i = 0; i < a.G; ++i) {
            const int g = REV ? a.G - 1 - i : i;
            int t_lo = g * a.cpg * 64, t_hi = min(a.T, (g + 1) * a.cpg * 64);
            float dec = __expf(gh * (float)max(t_hi - t_lo, 0));
            float* p = a.states + ((long long)bh * a.G + g) * a.DD + e;
            float m = *p;
            *p = carry;
            carry = dec * carry + m;
        }
        // 2. push the rank summary to every peer (and to the own slot)
        const long long off = a.data_off + (long long)a.rank * a.BH * a.DD + (long long)bh * a.DD + e;
        for (int j = 0; j < a.world; ++j) {
            bool needed = REV ? (j < a.rank) : (j > a.rank);
            if (needed) a.peer_data[j][off] = carry;
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
        const float dec_rank = __expf(gh * (float)a.T);          // decay across one whole rank slice
        if (!REV) {
            for (int j = 0; j < a.rank; ++j) R = dec_rank * R + mine[(long long)j * a.BH * a.DD];
        } else {
            for (int j = a.world - 1; j > a.rank; --j) R = dec_rank * R + mine[(long long)j * a.BH * a.DD];
        }
    }
    // 4. fix-up of the local entering states and the rank's outgoing state
    for (int g = 0; g < a.G; ++g) {
        int tokens_between;                                         // tokens between the rank boundary and group g
        if (!REV) tokens_between = min(a.T, g * a.cpg * 64);
        else tokens_between = max(a.T - min(a.T, (g + 1) * a.cpg * 64), 0);
        float* p = a.states + ((long long)bh * a.G + g) * a.DD + e;
        *p += __expf(gh * (float)tokens_between) * R;
    }
    if (a.final_out != nullptr) a.final_out[(long long)bh * a.DD + e] = carry + __expf(gh * (float)a.T) * R;
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
