// ZeRO-1 optimizer step fused with its collectives over NVSwitch multicast (NVLS) or plain peer pointers.
//
//   zero_reduce_kernel      barrier -> reduce-scatter: this rank's shard of the flat fp32 gradient buffer is summed
//                           over all ranks with multimem.ld_reduce (in-switch reduction), scaled, written back in
//                           place, and its sum of squares accumulated for the global gradient norm
//   zero_adam_bcast_kernel  AdamW on the fp32 master shard -> the bf16 parameters are written to EVERY rank's flat
//                           parameter buffer with multimem.st (the all-gather) -> barrier
// Together they replace Megatron's DDP bucket reduce-scatter, Apex FusedAdam and the parameter all-gather that
// the reference uses through `--use-distributed-optimizer` (training.py:278-298,343-351): no NCCL call.
//
// Barriers are flag exchanges in symmetric memory (release store to every peer, acquire spin on the own copy), with
// monotonically increasing epochs.  Every spin is bounded; on expiry the status word is set and the kernel goes on
// without the peer (the host raises after the step).
#include "common.cuh"

namespace lmoe {

__device__ __forceinline__ void st_rel_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;\n" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acq_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 mc_ld_reduce_f32x4(const float* mc) {
    float4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];\n"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
    return v;
}
__device__ __forceinline__ void mc_st_16B(void* mc, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};\n"
                 :: "l"(mc), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                    "f"(__uint_as_float(v.w)) : "memory");
}

struct ZeroArgs {
    float* grads;               // local flat gradient buffer (symmetric)
    const float* grads_mc;      // multicast address of the gradient buffers, or null
    float* const* peer_grads;   // [W] peer pointers (used when grads_mc is null)
    bf16* params;               // local flat parameter buffer (symmetric)
    bf16* params_mc;            // multicast address of the parameter buffers, or null
    bf16* const* peer_params;   // [W]
    int* const* peer_flags;     // [W] flag arrays: [2][W] ints (phase A: before reduce, phase B: after broadcast)
    int* status;
    float* sumsq;               // [1] accumulated sum of squares of the reduced shard
    unsigned int* done_ctr;     // [1] block counter for the end-of-kernel barrier
    float *master, *exp_avg, *exp_avg_sq;   // shard-sized fp32 state
    long long lo, hi;           // shard range in elements (multiples of 8)
    int rank, world, epoch;
    float grad_scale;
    float lr, b1, b2, eps, wd, bc1, bc2, gscale;
    long long spin_limit;
    int slot;                   // flag slot of this reduce launch (0 for the whole-shard reduce; one per bucket when the
                                // reduction is split into buckets that overlap the backward pass)
};

__device__ __forceinline__ bool wait_all(const ZeroArgs& a, int phase, int code) {
    // one thread per peer
    bool ok = true;
    if ((int)threadIdx.x < a.world) {
        const int* f = a.peer_flags[a.rank] + phase * a.world + threadIdx.x;
        long long spins = 0;
        while (ld_acq_sys(f) < a.epoch) {
            if (++spins > a.spin_limit) {
                atomicCAS(a.status, 0, (8 << 24) | ((int)threadIdx.x << 16) | code);
                ok = false;
                break;
            }
            __nanosleep(64);
        }
    }
    return ok;
}

__global__ void zero_reduce_kernel(ZeroArgs a) {
    __shared__ float red[32];
    // slot 0 = flags [0, W); slot 1 is the parameter barrier of zero_adam_bcast_kernel; bucket slots follow
    const int phase = a.slot == 0 ? 0 : a.slot + 1;
    if (blockIdx.x == 0 && (int)threadIdx.x < a.world) {
        __threadfence_system();
        st_rel_sys(a.peer_flags[threadIdx.x] + phase * a.world + a.rank, a.epoch);  // "my gradients (of this bucket) are complete"
    }
    const long long n4 = (a.hi - a.lo) / 4;
    if (n4 <= 0) return;                                   // nothing of this bucket in this rank's shard: signal only
    wait_all(a, phase, 1);
    __syncthreads();
    float ss = 0.f;
    // four independent 16-byte reductions in flight per thread: a bucket launched next to the backward pass runs on a
    // few dozen CTAs only, and the in-switch reduction has microseconds of latency
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < n4; i0 += 4 * stride) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long i = i0 + u * stride;
            if (i >= n4) { v[u] = make_float4(0.f, 0.f, 0.f, 0.f); continue; }
            const long long e = a.lo + i * 4;
            if (a.grads_mc != nullptr) {
                v[u] = mc_ld_reduce_f32x4(a.grads_mc + e);
            } else {
                v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int j = 0; j < a.world; ++j) {
                    float4 p = __ldcg(reinterpret_cast<const float4*>(a.peer_grads[j] + e));
                    v[u].x += p.x; v[u].y += p.y; v[u].z += p.z; v[u].w += p.w;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long i = i0 + u * stride;
            if (i >= n4) continue;
            const long long e = a.lo + i * 4;
            float4 x = v[u];
            x.x *= a.grad_scale; x.y *= a.grad_scale; x.z *= a.grad_scale; x.w *= a.grad_scale;
            *reinterpret_cast<float4*>(a.grads + e) = x;
            ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        }
    }
    ss = block_sum(ss, red);
    if (threadIdx.x == 0) atomicAdd(a.sumsq, ss);
}

__global__ void zero_adam_bcast_kernel(ZeroArgs a) {
    const long long n8 = (a.hi - a.lo) / 8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
        const long long s = i * 8;                       // offset inside the shard
        float w[8], g[8], m[8], v[8];
        *reinterpret_cast<float4*>(w) = *reinterpret_cast<const float4*>(a.master + s);
        *reinterpret_cast<float4*>(w + 4) = *reinterpret_cast<const float4*>(a.master + s + 4);
        *reinterpret_cast<float4*>(g) = *reinterpret_cast<const float4*>(a.grads + a.lo + s);
        *reinterpret_cast<float4*>(g + 4) = *reinterpret_cast<const float4*>(a.grads + a.lo + s + 4);
        *reinterpret_cast<float4*>(m) = *reinterpret_cast<const float4*>(a.exp_avg + s);
        *reinterpret_cast<float4*>(m + 4) = *reinterpret_cast<const float4*>(a.exp_avg + s + 4);
        *reinterpret_cast<float4*>(v) = *reinterpret_cast<const float4*>(a.exp_avg_sq + s);
        *reinterpret_cast<float4*>(v + 4) = *reinterpret_cast<const float4*>(a.exp_avg_sq + s + 4);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float gg = g[e] * a.gscale;
            m[e] = a.b1 * m[e] + (1.f - a.b1) * gg;
            v[e] = a.b2 * v[e] + (1.f - a.b2) * gg * gg;
            w[e] = w[e] * (1.f - a.lr * a.wd) - a.lr * (m[e] / a.bc1) / (sqrtf(v[e] / a.bc2) + a.eps);
        }
        *reinterpret_cast<float4*>(a.master + s) = *reinterpret_cast<float4*>(w);
        *reinterpret_cast<float4*>(a.master + s + 4) = *reinterpret_cast<float4*>(w + 4);
        *reinterpret_cast<float4*>(a.exp_avg + s) = *reinterpret_cast<float4*>(m);
        *reinterpret_cast<float4*>(a.exp_avg + s + 4) = *reinterpret_cast<float4*>(m + 4);
        *reinterpret_cast<float4*>(a.exp_avg_sq + s) = *reinterpret_cast<float4*>(v);
        *reinterpret_cast<float4*>(a.exp_avg_sq + s + 4) = *reinterpret_cast<float4*>(v + 4);
        uint4 o;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(w[0], w[1]), h1 = __floats2bfloat162_rn(w[2], w[3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(w[4], w[5]), h3 = __floats2bfloat162_rn(w[6], w[7]);
        o.x = *reinterpret_cast<uint32_t*>(&h0); o.y = *reinterpret_cast<uint32_t*>(&h1);
        o.z = *reinterpret_cast<uint32_t*>(&h2); o.w = *reinterpret_cast<uint32_t*>(&h3);
        if (a.params_mc != nullptr) {
            mc_st_16B(a.params_mc + a.lo + s, o);
        } else {
            for (int j = 0; j < a.world; ++j) *reinterpret_cast<uint4*>(a.peer_params[j] + a.lo + s) = o;
        }
    }
    // end-of-kernel barrier: the last block to finish signals the peers and waits for theirs
    __shared__ int is_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) is_last = (atomicAdd(a.done_ctr, 1u) == gridDim.x - 1);
    __syncthreads();
    if (is_last) {
        if ((int)threadIdx.x < a.world) {
            __threadfence_system();
            st_rel_sys(a.peer_flags[threadIdx.x] + 1 * a.world + a.rank, a.epoch);  // "my parameter shard is everywhere"
        }
        wait_all(a, 1, 2);
        if (threadIdx.x == 0) *a.done_ctr = 0;
    }
}

}  // namespace lmoe

using namespace lmoe;

LMOE_API int lmoe_zero_reduce(const ZeroArgs* ap, int blocks, cudaStream_t st) {
    zero_reduce_kernel<<<blocks, 256, 0, st>>>(*ap);
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_zero_adam_bcast(const ZeroArgs* ap, int blocks, cudaStream_t st) {
    zero_adam_bcast_kernel<<<blocks, 256, 0, st>>>(*ap);
    return (int)cudaGetLastError();
}
