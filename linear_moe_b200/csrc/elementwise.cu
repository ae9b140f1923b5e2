// Bandwidth-bound operators: RMSNorm (+residual add) fwd/bwd, per-head norm + swish gate fwd/bwd,
// gated RMSNorm (Mamba2) fwd/bwd, SwiGLU fwd/bwd, l2norm fwd/bwd, rotary fwd/bwd, softmax cross
// entropy fwd/bwd over a chunk of logits, depthwise causal conv1d (+SiLU) fwd/bwd, router
// softmax/top-k, fused Adam over flat buffers.
//
// They replace the reference's Triton norm / l2norm / logsigmoid kernels
// (common_modules/layernorm.py:55-300, l2norm.py:22-95), its jiterator swiglu/swish snippets
// (activations.py:304-329), the external causal_conv1d CUDA op (mamba_mixer.py:291-296), Megatron's
// fused cross entropy and Apex FusedAdam.  Every kernel moves 16-byte vectors, keeps the row in
// registers between the reduction and the write, and computes in fp32.
#include "common.cuh"

namespace lmoe {

static inline int pick_threads(int nvec) {
    int t = 32;
    while (t < nvec && t < 256) t <<= 1;
    return t;
}

// ---------------------------------------------------------------------------------------------
// RMSNorm forward: r = x (+ res); y = r * rsqrt(mean(r^2) + eps) * w.  One block per row.
// ---------------------------------------------------------------------------------------------
template <typename T, int MAXV>
__global__ void rms_norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ res, const T* __restrict__ w,
                                    T* __restrict__ y, T* __restrict__ res_out, float* __restrict__ rstd_out,
                                    int N, float eps) {
    __shared__ float red[32];
    constexpr int VN = Vec<T>::N;
    const int64_t row = blockIdx.x;
    const int nvec = N / VN;
    pdl_trigger();
    const T* xr = x + row * N;
    Vec<T> v[MAXV];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        int i = threadIdx.x + j * blockDim.x;
        if (i < nvec) {
            v[j].load(xr + i * VN);
            if (res != nullptr) {
                Vec<T> r;
                r.load(res + row * N + i * VN);
#pragma unroll
                for (int e = 0; e < VN; ++e) v[j].set(e, v[j].get(e) + r.get(e));
            }
            if (res_out != nullptr) v[j].store(res_out + row * N + i * VN);
#pragma unroll
            for (int e = 0; e < VN; ++e) { float f = v[j].get(e); ss += f * f; }
        }
    }
    ss = block_sum(ss, red);
    float rstd = rsqrtf(ss / (float)N + eps);
    if (threadIdx.x == 0 && rstd_out != nullptr) rstd_out[row] = rstd;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
        int i = threadIdx.x + j * blockDim.x;
        if (i < nvec) {
            Vec<T> o;
            if (w != nullptr) {
                Vec<T> wv;
                wv.load(w + i * VN);
#pragma unroll
                for (int e = 0; e < VN; ++e) o.set(e, v[j].get(e) * rstd * wv.get(e));
            } else {
#pragma unroll
                for (int e = 0; e < VN; ++e) o.set(e, v[j].get(e) * rstd);
            }
            o.store(y + row * N + i * VN);
        }
    }
}

// RMSNorm backward.  Each block walks rows blockIdx.x, +gridDim.x, ...; per row
// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)) (+ dres); dw partials stay in registers across rows and
// are written once per block to dw_partial[gridDim.x, N].
template <typename T, int MAXV>
__global__ void rms_norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ xin, const T* __restrict__ w,
                                    const float* __restrict__ rstd, const T* __restrict__ dres,
                                    T* __restrict__ dx, float* __restrict__ dw_partial, int rows, int N) {
    __shared__ float red[32];
    constexpr int VN = Vec<T>::N;
    const int nvec = N / VN;
    float dwacc[MAXV][VN];
#pragma unroll
    for (int j = 0; j < MAXV; ++j)
#pragma unroll
        for (int e = 0; e < VN; ++e) dwacc[j][e] = 0.f;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const float rs = rstd[row];
        Vec<T> g[MAXV], xv[MAXV];
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            int i = threadIdx.x + j * blockDim.x;
            if (i < nvec) {
                g[j].load(dy + row * N + i * VN);
                xv[j].load(xin + row * N + i * VN);
                Vec<T> wv;
                if (w != nullptr) wv.load(w + i * VN);
#pragma unroll
                for (int e = 0; e < VN; ++e) {
                    float xh = xv[j].get(e) * rs;
                    float gy = g[j].get(e);
                    dwacc[j][e] += gy * xh;
                    float gw = w != nullptr ? gy * wv.get(e) : gy;
                    dot += gw * xh;
                }
            }
        }
        dot = block_sum(dot, red) / (float)N;
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            int i = threadIdx.x + j * blockDim.x;
            if (i < nvec) {
                Vec<T> wv, o, dr;
                if (w != nullptr) wv.load(w + i * VN);
                if (dres != nullptr) dr.load(dres + row * N + i * VN);
#pragma unroll
                for (int e = 0; e < VN; ++e) {
                    float xh = xv[j].get(e) * rs;
                    float gw = w != nullptr ? g[j].get(e) * wv.get(e) : g[j].get(e);
                    float d = rs * (gw - xh * dot);
                    if (dres != nullptr) d += dr.get(e);
                    o.set(e, d);
                }
                o.store(dx + row * N + i * VN);
            }
        }
    }
    if (dw_partial != nullptr) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            int i = threadIdx.x + j * blockDim.x;
            if (i < nvec) {
#pragma unroll
                for (int e = 0; e < VN; ++e) dw_partial[(int64_t)blockIdx.x * N + i * VN + e] = dwacc[j][e];
            }
        }
    }
}

// out[c] = sum_p partial[p, c].  Block = 32 columns x 8 row-slices; the slices are summed through shared memory.
template <typename T>
__global__ void reduce_partials_kernel(const float* __restrict__ partial, T* __restrict__ out, int P, int N) {
    __shared__ float sm[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + tx;
    float s = 0.f;
    if (c < N)
        for (int p = ty; p < P; p += 8) s += partial[(int64_t)p * N + c];
    sm[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && c < N) {
        float t = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) t += sm[j][tx];
        out[c] = from_f<T>(t);
    }
}

// ---------------------------------------------------------------------------------------------
// Per-head RMSNorm + swish gate (LSM epilogue).  rows = B*T*H, D = head value dim, one warp per row.
//   y = (norm ? o * rstd * w : o) * silu(gate)
// ---------------------------------------------------------------------------------------------
// Lane l owns the 4 contiguous channels [4l + 128j, 4l + 128j + 4) of the row: one 8-byte (bf16) or 16-byte
// (fp32) access per lane and j.
template <typename T> struct Quad;
template <> struct Quad<bf16> {
    uint2 raw;
    __device__ __forceinline__ void load(const bf16* p) { raw = *reinterpret_cast<const uint2*>(p); }
    __device__ __forceinline__ void store(bf16* p) const { *reinterpret_cast<uint2*>(p) = raw; }
    __device__ __forceinline__ float get(int i) const { return __bfloat162float(reinterpret_cast<const bf16*>(&raw)[i]); }
    __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<bf16*>(&raw)[i] = __float2bfloat16(v); }
};
template <> struct Quad<float> {
    float4 raw;
    __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = raw; }
    __device__ __forceinline__ float get(int i) const { return reinterpret_cast<const float*>(&raw)[i]; }
    __device__ __forceinline__ void set(int i, float v) { reinterpret_cast<float*>(&raw)[i] = v; }
};

template <typename T, int DMAX>
__global__ void head_norm_gate_fwd_kernel(const T* __restrict__ o, const T* __restrict__ w, const T* __restrict__ gate,
                                          T* __restrict__ y, float* __restrict__ rstd_out, int64_t rows, int D,
                                          float eps, int do_norm) {
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    constexpr int PER = DMAX / 128;
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    float wv[PER][4];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        int c = lane * 4 + j * 128;
#pragma unroll
        for (int e = 0; e < 4; ++e) wv[j][e] = (do_norm && w != nullptr && c + e < D) ? to_f(w[c + e]) : 1.f;
    }
    for (int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += nwarps) {
        Quad<T> v[PER], g[PER];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            int c = lane * 4 + j * 128;
            if (c < D) {
                v[j].load(o + row * D + c);
                g[j].load(gate + row * D + c);
#pragma unroll
                for (int e = 0; e < 4; ++e) { float f = v[j].get(e); ss += f * f; }
            }
        }
        float rs = 1.f;
        if (do_norm) {
            ss = warp_sum(ss);
            rs = rsqrtf(ss / (float)D + eps);
            if (lane == 0) rstd_out[row] = rs;
        }
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            int c = lane * 4 + j * 128;
            if (c < D) {
                Quad<T> out;
#pragma unroll
                for (int e = 0; e < 4; ++e) out.set(e, v[j].get(e) * rs * wv[j][e] * silu_f(g[j].get(e)));
                out.store(y + row * D + c);
            }
        }
    }
}

template <typename T, int DMAX>
__global__ void head_norm_gate_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ o, const T* __restrict__ w,
                                          const T* __restrict__ gate, const float* __restrict__ rstd,
                                          T* __restrict__ d_o, T* __restrict__ dgate, float* __restrict__ dw_partial,
                                          int64_t rows, int D, int do_norm) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    constexpr int PER = DMAX / 128;
    float dwacc[PER][4], wv[PER][4];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        int c = lane * 4 + j * 128;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            dwacc[j][e] = 0.f;
            wv[j][e] = (do_norm && w != nullptr && c + e < D) ? to_f(w[c + e]) : 1.f;
        }
    }
    for (int64_t row = (int64_t)blockIdx.x * nw + wid; row < rows; row += (int64_t)gridDim.x * nw) {
        const float rs = do_norm ? rstd[row] : 1.f;
        Quad<T> ov[PER], gv[PER], gy[PER];
        float xh[PER][4], gn[PER][4];
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            int c = lane * 4 + j * 128;
            if (c < D) {
                ov[j].load(o + row * D + c);
                gv[j].load(gate + row * D + c);
                gy[j].load(dy + row * D + c);
                Quad<T> dg;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float gt = gv[j].get(e), g = gy[j].get(e);
                    xh[j][e] = ov[j].get(e) * rs;
                    dg.set(e, g * xh[j][e] * wv[j][e] * dsilu_f(gt));
                    float gnorm = g * silu_f(gt);
                    dwacc[j][e] += gnorm * xh[j][e];
                    gn[j][e] = gnorm * wv[j][e];
                    dot += gn[j][e] * xh[j][e];
                }
                dg.store(dgate + row * D + c);
            }
        }
        if (do_norm) dot = warp_sum(dot) / (float)D;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            int c = lane * 4 + j * 128;
            if (c < D) {
                Quad<T> out;
#pragma unroll
                for (int e = 0; e < 4; ++e) out.set(e, do_norm ? rs * (gn[j][e] - xh[j][e] * dot) : gn[j][e]);
                out.store(d_o + row * D + c);
            }
        }
    }
    if (dw_partial != nullptr) {
        extern __shared__ float sm[];                  // [nw, DMAX]
#pragma unroll
        for (int j = 0; j < PER; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) sm[wid * DMAX + lane * 4 + j * 128 + e] = dwacc[j][e];
        __syncthreads();
        for (int c = threadIdx.x; c < D; c += blockDim.x) {
            float s = 0.f;
            for (int q = 0; q < nw; ++q) s += sm[q * DMAX + c];
            dw_partial[(int64_t)blockIdx.x * D + c] = s;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Gated RMSNorm (Mamba2): y = rmsnorm_group(x * silu(z)) * w, groups of G channels; warp per (row, group).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void gated_rms_norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ z, const T* __restrict__ w,
                                          T* __restrict__ y, float* __restrict__ rstd_out, int64_t rows, int N, int G,
                                          float eps) {
    const int lane = threadIdx.x & 31;
    const int ng = N / G;
    const int64_t idx = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (idx >= rows * ng) return;
    const int64_t row = idx / ng;
    const int g = idx % ng;
    const int64_t base = row * N + (int64_t)g * G;
    float ss = 0.f;
    for (int c = lane; c < G; c += 32) {
        float u = to_f(x[base + c]) * silu_f(to_f(z[base + c]));
        ss += u * u;
    }
    ss = warp_sum(ss);
    float rs = rsqrtf(ss / (float)G + eps);
    if (lane == 0) rstd_out[idx] = rs;
    for (int c = lane; c < G; c += 32) {
        float u = to_f(x[base + c]) * silu_f(to_f(z[base + c]));
        y[base + c] = from_f<T>(u * rs * to_f(w[g * G + c]));
    }
}

template <typename T>
__global__ void gated_rms_norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ z,
                                          const T* __restrict__ w, const float* __restrict__ rstd, T* __restrict__ dx,
                                          T* __restrict__ dz, float* __restrict__ dw, int64_t rows, int N, int G) {
    const int lane = threadIdx.x & 31;
    const int ng = N / G;
    const int64_t nwarps = (int64_t)gridDim.x * (blockDim.x >> 5);
    for (int64_t idx = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); idx < rows * ng; idx += nwarps) {
        const int64_t row = idx / ng;
        const int g = idx % ng;
        const int64_t base = row * N + (int64_t)g * G;
        const float rs = rstd[idx];
        float dot = 0.f;
        for (int c = lane; c < G; c += 32) {
            float u = to_f(x[base + c]) * silu_f(to_f(z[base + c]));
            dot += to_f(dy[base + c]) * to_f(w[g * G + c]) * u * rs;
        }
        dot = warp_sum(dot) / (float)G;
        for (int c = lane; c < G; c += 32) {
            float xv = to_f(x[base + c]), zv = to_f(z[base + c]);
            float sz = silu_f(zv);
            float u = xv * sz, uh = u * rs;
            float gy = to_f(dy[base + c]);
            atomicAdd(&dw[g * G + c], gy * uh);
            float du = rs * (gy * to_f(w[g * G + c]) - uh * dot);
            dx[base + c] = from_f<T>(du * sz);
            dz[base + c] = from_f<T>(du * xv * dsilu_f(zv));
        }
    }
}

// ---------------------------------------------------------------------------------------------
// SwiGLU: y[r, c] = silu(x[r, c]) * x[r, F + c]
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int64_t rows, int F) {
    pdl_trigger();
    constexpr int VN = Vec<T>::N;
    const int64_t nvec = rows * (F / VN);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / (F / VN);
        int c = (i % (F / VN)) * VN;
        Vec<T> a, b, o;
        a.load(x + r * 2 * F + c);
        b.load(x + r * 2 * F + F + c);
#pragma unroll
        for (int e = 0; e < VN; ++e) o.set(e, silu_f(a.get(e)) * b.get(e));
        o.store(y + r * F + c);
    }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx, int64_t rows,
                                  int F) {
    constexpr int VN = Vec<T>::N;
    const int64_t nvec = rows * (F / VN);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / (F / VN);
        int c = (i % (F / VN)) * VN;
        Vec<T> a, b, g, da, db;
        a.load(x + r * 2 * F + c);
        b.load(x + r * 2 * F + F + c);
        g.load(dy + r * F + c);
#pragma unroll
        for (int e = 0; e < VN; ++e) {
            float av = a.get(e), gv = g.get(e);
            da.set(e, gv * b.get(e) * dsilu_f(av));
            db.set(e, gv * silu_f(av));
        }
        da.store(dx + r * 2 * F + c);
        db.store(dx + r * 2 * F + F + c);
    }
}

// ---------------------------------------------------------------------------------------------
// l2norm over the last dim (D <= 512), warp per row.
// ---------------------------------------------------------------------------------------------
template <typename T, int DMAX>
__global__ void l2norm_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, float* __restrict__ rstd, int64_t rows,
                                  int D, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    constexpr int PER = DMAX / 32;
    float v[PER];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        int c = lane + j * 32;
        v[j] = c < D ? to_f(x[row * D + c]) : 0.f;
        ss += v[j] * v[j];
    }
    ss = warp_sum(ss);
    float rs = rsqrtf(ss + eps);
    if (lane == 0) rstd[row] = rs;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        int c = lane + j * 32;
        if (c < D) y[row * D + c] = from_f<T>(v[j] * rs);
    }
}

// dx = rs * (dy - y * (dy . y))
template <typename T, int DMAX>
__global__ void l2norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ rstd,
                                  T* __restrict__ dx, int64_t rows, int D) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    constexpr int PER = DMAX / 32;
    const float rs = rstd[row];
    float yv[PER], g[PER];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        int c = lane + j * 32;
        yv[j] = c < D ? to_f(x[row * D + c]) * rs : 0.f;
        g[j] = c < D ? to_f(dy[row * D + c]) : 0.f;
        dot += yv[j] * g[j];
    }
    dot = warp_sum(dot);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        int c = lane + j * 32;
        if (c < D) dx[row * D + c] = from_f<T>(rs * (g[j] - yv[j] * dot));
    }
}

// ---------------------------------------------------------------------------------------------
// Rotary embedding on x [B, T, H, D]; cos/sin [T, R/2] fp32; `conj` applies the inverse rotation (backward).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                            T* __restrict__ y, int64_t BT, int Tlen, int H, int D, int R, int interleaved, int conj) {
    const int half = R / 2;
    const int64_t total = BT * H * (int64_t)(D - half);     // one thread per rotated pair or pass-through element
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int e = i % (D - half);
        int64_t bh = i / (D - half);                         // (b*T + t)*H + h
        int64_t bt = bh / H;
        int t = bt % Tlen;
        const T* xp = x + bh * D;
        T* yp = y + bh * D;
        if (e < half) {
            int i1 = interleaved ? 2 * e : e;
            int i2 = interleaved ? 2 * e + 1 : e + half;
            float c = cs[(int64_t)t * half + e], s = sn[(int64_t)t * half + e];
            if (conj) s = -s;
            float x1 = to_f(xp[i1]), x2 = to_f(xp[i2]);
            yp[i1] = from_f<T>(x1 * c - x2 * s);
            yp[i2] = from_f<T>(x2 * c + x1 * s);
        } else {
            int c = R + (e - half);
            yp[c] = xp[c];
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Softmax cross entropy over a chunk of logits [rows, V]; one block per row.
//   fwd: lse = logsumexp(row); loss = lse - row[label] (0 if label == ignore)
//   bwd: grad[row, c] = (exp(row[c] - lse) - [c == label]) * g[row]   (0 row if ignored)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void softmax_ce_fwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ labels,
                                      float* __restrict__ loss, float* __restrict__ lse_out, int V, int64_t ignore) {
    __shared__ float red[32];
    constexpr int VN = Vec<T>::N;
    const int64_t row = blockIdx.x;
    const T* lr = logits + row * V;
    float m = -INFINITY, s = 0.f;
    const int nvec = V / VN;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        Vec<T> v;
        v.load(lr + i * VN);
        float lm = -INFINITY;
#pragma unroll
        for (int e = 0; e < VN; ++e) lm = fmaxf(lm, v.get(e));
        if (lm > m) { s *= __expf(m - lm); m = lm; }
#pragma unroll
        for (int e = 0; e < VN; ++e) s += __expf(v.get(e) - m);
    }
    for (int c = nvec * VN + threadIdx.x; c < V; c += blockDim.x) {
        float f = to_f(lr[c]);
        if (f > m) { s *= __expf(m - f); m = f; }
        s += __expf(f - m);
    }
    float gm = block_max(m, red);
    s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
    s = block_sum(s, red);
    if (threadIdx.x == 0) {
        float lse = gm + logf(s);
        lse_out[row] = lse;
        int64_t lab = labels[row];
        loss[row] = (lab == ignore) ? 0.f : lse - to_f(lr[lab]);
    }
}

template <typename T>
__global__ void softmax_ce_bwd_kernel(const T* __restrict__ logits, const int64_t* __restrict__ labels,
                                      const float* __restrict__ lse, const float* __restrict__ gloss,
                                      T* __restrict__ grad, int V, int64_t ignore) {
    constexpr int VN = Vec<T>::N;
    const int64_t row = blockIdx.x;
    const T* lr = logits + row * V;
    T* gr = grad + row * V;
    const int64_t lab = labels[row];
    const float g = (lab == ignore) ? 0.f : gloss[row];
    const float l = lse[row];
    const int nvec = V / VN;
    for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
        Vec<T> v, o;
        v.load(lr + i * VN);
#pragma unroll
        for (int e = 0; e < VN; ++e) {
            float p = __expf(v.get(e) - l);
            if ((int64_t)(i * VN + e) == lab) p -= 1.f;
            o.set(e, p * g);
        }
        o.store(gr + i * VN);
    }
    for (int c = nvec * VN + threadIdx.x; c < V; c += blockDim.x) {
        float p = __expf(to_f(lr[c]) - l);
        if (c == lab) p -= 1.f;
        gr[c] = from_f<T>(p * g);
    }
}

// ---------------------------------------------------------------------------------------------
// Depthwise causal conv1d (+SiLU).  x [B, T, D]; w [D, K]; init [B, K-1, D] (tokens before x[0]) or null.
// ---------------------------------------------------------------------------------------------
template <typename T, int K>
__global__ void causal_conv1d_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
                                         const T* __restrict__ init, T* __restrict__ y, int B, int Tlen, int D,
                                         int act) {
    const int64_t total = (int64_t)B * Tlen * D;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int d = i % D;
        int64_t bt = i / D;
        int t = bt % Tlen;
        int b = bt / Tlen;
        float acc = bias != nullptr ? to_f(bias[d]) : 0.f;
#pragma unroll
        for (int k = 0; k < K; ++k) {
            int ts = t - (K - 1) + k;
            float xv;
            if (ts >= 0) xv = to_f(x[((int64_t)b * Tlen + ts) * D + d]);
            else xv = init != nullptr ? to_f(init[((int64_t)b * (K - 1) + (K - 1 + ts)) * D + d]) : 0.f;
            acc += xv * to_f(w[d * K + k]);
        }
        y[i] = from_f<T>(act ? silu_f(acc) : acc);
    }
}

// Vectorised forward: a thread owns VN consecutive channels (one 16-byte access per token) and walks a run of
// `trun` tokens with the last K-1 rows kept in registers, so every input row is read once per thread.
template <typename T, int K>
__global__ void causal_conv1d_fwd_vec_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
                                             const T* __restrict__ init, T* __restrict__ y, int B, int Tlen, int D,
                                             int act, int trun) {
    constexpr int VN = Vec<T>::N;
    const int dv = blockIdx.x * blockDim.x + threadIdx.x;
    if (dv * VN >= D) return;
    const int d0 = dv * VN, b = blockIdx.z;
    const int t0 = blockIdx.y * trun, t1 = min(Tlen, t0 + trun);
    float wk[VN][K], bv[VN];
#pragma unroll
    for (int e = 0; e < VN; ++e) {
        bv[e] = bias != nullptr ? to_f(bias[d0 + e]) : 0.f;
#pragma unroll
        for (int k = 0; k < K; ++k) wk[e][k] = to_f(w[(d0 + e) * K + k]);
    }
    float hist[K - 1][VN];                                   // rows t-(K-1) .. t-1
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
        const int ts = t0 - (K - 1) + j;
        Vec<T> v;
        bool have = false;
        if (ts >= 0) { v.load(x + ((int64_t)b * Tlen + ts) * D + d0); have = true; }
        else if (init != nullptr) { v.load(init + ((int64_t)b * (K - 1) + (K - 1 + ts)) * D + d0); have = true; }
#pragma unroll
        for (int e = 0; e < VN; ++e) hist[j][e] = have ? v.get(e) : 0.f;
    }
    // eight rows per pass, their loads issued together before the first use
    constexpr int U = 8;
    for (int tb = t0; tb < t1; tb += U) {
        Vec<T> curv[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (tb + u < t1) curv[u].load(x + ((int64_t)b * Tlen + tb + u) * D + d0);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int t = tb + u;
            if (t >= t1) break;
            Vec<T> out;
#pragma unroll
            for (int e = 0; e < VN; ++e) {
                float acc = bv[e] + curv[u].get(e) * wk[e][K - 1];
#pragma unroll
                for (int j = 0; j < K - 1; ++j) acc += hist[j][e] * wk[e][j];
                out.set(e, act ? silu_f(acc) : acc);
            }
            out.store(y + ((int64_t)b * Tlen + t) * D + d0);
#pragma unroll
            for (int j = 0; j + 1 < K - 1; ++j)
#pragma unroll
                for (int e = 0; e < VN; ++e) hist[j][e] = hist[j + 1][e];
#pragma unroll
            for (int e = 0; e < VN; ++e) hist[K - 2][e] = curv[u].get(e);
        }
    }
}

// Backward: dx[b,t,d] = sum_k dpre[b, t + (K-1-k), d] * w[d,k]; dw[d,k] = sum dpre[b,t,d] * x[b, t-(K-1)+k, d];
// dpre = dy * dsilu(pre) is recomputed.  Blocks tile (b, time-chunk) x channel; dw/dbias via atomics.
template <typename T, int K>
__global__ void causal_conv1d_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                         const T* __restrict__ bias, const T* __restrict__ init, T* __restrict__ dx,
                                         float* __restrict__ dw, float* __restrict__ dbias, T* __restrict__ dinit,
                                         int B, int Tlen, int D, int act, int tchunk) {
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= D) return;
    const int b = blockIdx.z;
    const int t0 = blockIdx.y * tchunk;
    const int t1 = min(Tlen, t0 + tchunk);
    float wk[K];
#pragma unroll
    for (int k = 0; k < K; ++k) wk[k] = to_f(w[d * K + k]);
    const float bv = bias != nullptr ? to_f(bias[d]) : 0.f;
    auto xat = [&](int ts) -> float {
        if (ts >= 0) return ts < Tlen ? to_f(x[((int64_t)b * Tlen + ts) * D + d]) : 0.f;
        return init != nullptr ? to_f(init[((int64_t)b * (K - 1) + (K - 1 + ts)) * D + d]) : 0.f;
    };
    auto dpre_at = [&](int t) -> float {
        if (t >= Tlen) return 0.f;
        float g = to_f(dy[((int64_t)b * Tlen + t) * D + d]);
        if (!act) return g;
        float pre = bv;
#pragma unroll
        for (int k = 0; k < K; ++k) pre += xat(t - (K - 1) + k) * wk[k];
        return g * dsilu_f(pre);
    };
    float dwacc[K];
#pragma unroll
    for (int k = 0; k < K; ++k) dwacc[k] = 0.f;
    float dbacc = 0.f;
    // sliding window of dpre for t .. t+K-1
    float win[K];
#pragma unroll
    for (int k = 0; k < K; ++k) win[k] = dpre_at(t0 + k);
    for (int t = t0; t < t1; ++t) {
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < K; ++k) acc += win[K - 1 - k] * wk[k];      // dpre[t + K-1-k] * w[k]
        dx[((int64_t)b * Tlen + t) * D + d] = from_f<T>(acc);
        float dp = win[0];
        dbacc += dp;
#pragma unroll
        for (int k = 0; k < K; ++k) dwacc[k] += dp * xat(t - (K - 1) + k);
#pragma unroll
        for (int k = 0; k + 1 < K; ++k) win[k] = win[k + 1];
        win[K - 1] = dpre_at(t + K);
    }
    if (dinit != nullptr && t0 == 0) {
        // gradient wrt the K-1 tokens before x[0]: dinit[j] = sum_k dpre[j - (K-1) + (K-1-k)] * w[k] for valid t
        for (int j = 0; j < K - 1; ++j) {
            float acc = 0.f;
            for (int k = 0; k < K; ++k) {
                int t = j - (K - 1) + (K - 1 - k);
                if (t >= 0) acc += dpre_at(t) * wk[k];
            }
            dinit[((int64_t)b * (K - 1) + j) * D + d] = from_f<T>(acc);
        }
    }
#pragma unroll
    for (int k = 0; k < K; ++k) atomicAdd(&dw[d * K + k], dwacc[k]);
    if (dbias != nullptr) atomicAdd(&dbias[d], dbacc);
}

// Vectorised backward: a thread owns VN channels and a run of tokens [t0, t1); it walks t0 .. t1+K-2 recomputing the
// pre-activation from a K-row window of x, keeps the last K values of dpre = dy * dsilu(pre), emits dx[t-(K-1)] as soon as
// its K contributions are known, and accumulates dw / dbias for its own tokens in registers (atomics once per thread).
template <typename T, int K>
__global__ void causal_conv1d_bwd_vec_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                             const T* __restrict__ bias, const T* __restrict__ init, T* __restrict__ dx,
                                             float* __restrict__ dw, float* __restrict__ dbias, T* __restrict__ dinit,
                                             int B, int Tlen, int D, int act, int trun) {
    constexpr int VN = Vec<T>::N;
    const int dvec = blockIdx.x * blockDim.x + threadIdx.x;
    if (dvec * VN >= D) return;
    const int d0 = dvec * VN, b = blockIdx.z;
    const int t0 = blockIdx.y * trun, t1 = min(Tlen, t0 + trun);
    float wk[VN][K], bv[VN], dwacc[VN][K], dbacc[VN];
#pragma unroll
    for (int e = 0; e < VN; ++e) {
        bv[e] = bias != nullptr ? to_f(bias[d0 + e]) : 0.f;
        dbacc[e] = 0.f;
#pragma unroll
        for (int k = 0; k < K; ++k) { wk[e][k] = to_f(w[(d0 + e) * K + k]); dwacc[e][k] = 0.f; }
    }
    float xw[K][VN];                                         // xw[k] = x[t-(K-1)+k]
    float dp[K][VN];                                         // dp[k] = dpre[t-(K-1)+k]
#pragma unroll
    for (int k = 0; k < K; ++k)
#pragma unroll
        for (int e = 0; e < VN; ++e) { xw[k][e] = 0.f; dp[k][e] = 0.f; }
    // preload the K-1 rows before t0 into xw[1..K-1] (they shift down by one at the first step)
#pragma unroll
    for (int j = 0; j < K - 1; ++j) {
        const int ts = t0 - (K - 1) + j;
        Vec<T> v;
        bool have = false;
        if (ts >= 0) { v.load(x + ((int64_t)b * Tlen + ts) * D + d0); have = true; }
        else if (init != nullptr) { v.load(init + ((int64_t)b * (K - 1) + (K - 1 + ts)) * D + d0); have = true; }
#pragma unroll
        for (int e = 0; e < VN; ++e) xw[j + 1][e] = have ? v.get(e) : 0.f;
    }
    float first_dp[K - 1][VN];                               // dpre[0..K-2] of the sequence (for dinit)
#pragma unroll
    for (int j = 0; j < K - 1; ++j)
#pragma unroll
        for (int e = 0; e < VN; ++e) first_dp[j][e] = 0.f;
    // four time steps per pass: their loads are issued together (one dependent load per step left the kernel bound by
    // memory latency), then the steps run in order on the register windows
    constexpr int U = 4;
    for (int tb = t0; tb < t1 + K - 1; tb += U) {
        Vec<T> curv[U], gvec[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int t = tb + u;
            if (t < t1 + K - 1 && t < Tlen) {
                curv[u].load(x + ((int64_t)b * Tlen + t) * D + d0);
                gvec[u].load(dy + ((int64_t)b * Tlen + t) * D + d0);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int t = tb + u;
            if (t >= t1 + K - 1) break;
            // shift windows
#pragma unroll
            for (int k = 0; k + 1 < K; ++k)
#pragma unroll
                for (int e = 0; e < VN; ++e) { xw[k][e] = xw[k + 1][e]; dp[k][e] = dp[k + 1][e]; }
            if (t < Tlen) {
#pragma unroll
                for (int e = 0; e < VN; ++e) {
                    xw[K - 1][e] = curv[u].get(e);
                    float gv = gvec[u].get(e);
                    if (act) {
                        float pre = bv[e];
#pragma unroll
                        for (int k = 0; k < K; ++k) pre += xw[k][e] * wk[e][k];
                        gv *= dsilu_f(pre);
                    }
                    dp[K - 1][e] = gv;
                    if (t < t1) {
                        dbacc[e] += gv;
#pragma unroll
                        for (int k = 0; k < K; ++k) dwacc[e][k] += gv * xw[k][e];
                    }
                }
            } else {
#pragma unroll
                for (int e = 0; e < VN; ++e) { xw[K - 1][e] = 0.f; dp[K - 1][e] = 0.f; }
            }
            if (t0 == 0 && t < K - 1) {
#pragma unroll
                for (int j = 0; j < K - 1; ++j)
                    if (j == t)
#pragma unroll
                        for (int e = 0; e < VN; ++e) first_dp[j][e] = dp[K - 1][e];
            }
            const int tout = t - (K - 1);
            if (tout >= t0 && tout < t1) {
                Vec<T> o;
#pragma unroll
                for (int e = 0; e < VN; ++e) {
                    float acc = 0.f;
#pragma unroll
                    for (int k = 0; k < K; ++k) acc += dp[K - 1 - k][e] * wk[e][k];       // dpre[tout + K-1-k] * w[k]
                    o.set(e, acc);
                }
                o.store(dx + ((int64_t)b * Tlen + tout) * D + d0);
            }
        }
    }
    if (dinit != nullptr && t0 == 0) {
#pragma unroll
        for (int j = 0; j < K - 1; ++j) {
            Vec<T> o;
#pragma unroll
            for (int e = 0; e < VN; ++e) {
                float acc = 0.f;
#pragma unroll
                for (int k = 0; k < K; ++k)
                    if (k <= j) acc += first_dp[j - k][e] * wk[e][k];
                o.set(e, acc);
            }
            o.store(dinit + ((int64_t)b * (K - 1) + j) * D + d0);
        }
    }
#pragma unroll
    for (int e = 0; e < VN; ++e) {
#pragma unroll
        for (int k = 0; k < K; ++k) atomicAdd(&dw[(d0 + e) * K + k], dwacc[e][k]);
        if (dbias != nullptr) atomicAdd(&dbias[d0 + e], dbacc[e]);
    }
}

// ---------------------------------------------------------------------------------------------
// Router: softmax over E experts + top-k.  logits [T, E] fp32, E <= 256, k <= 16.  Warp per token.
//   order 0: softmax over all then top-k of probabilities; order 1: top-k of logits then softmax over k.
// Also accumulates per-expert token counts (for the dispatcher and the aux loss) in counts[E].
// ---------------------------------------------------------------------------------------------
__global__ void router_topk_kernel(const float* __restrict__ logits, float* __restrict__ full, float* __restrict__ probs,
                                   int64_t* __restrict__ idx, int* __restrict__ counts, int64_t Ttok, int E, int k,
                                   int order) {
    const int lane = threadIdx.x & 31;
    const int64_t tok = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (tok >= Ttok) return;
    float v[8];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        int e = lane + j * 32;
        v[j] = e < E ? logits[tok * E + e] : -INFINITY;
        m = fmaxf(m, v[j]);
    }
    m = warp_max(m);
    float s = 0.f;
    float p[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { p[j] = (lane + j * 32 < E) ? __expf(v[j] - m) : 0.f; s += p[j]; }
    s = warp_sum(s);
    float inv = 1.f / s;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        p[j] *= inv;
        int e = lane + j * 32;
        if (e < E) full[tok * E + e] = p[j];
    }
    float sel_sum = 0.f, sel_val[16];
    int sel_idx[16];
    for (int r = 0; r < k; ++r) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int e = lane + j * 32;
            if (e < E && (v[j] > best || (v[j] == best && e < bi))) { best = v[j]; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ob = __shfl_xor_sync(0xffffffffu, best, o);
            int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        sel_idx[r] = bi;
        sel_val[r] = best;
        if ((bi & 31) == lane) v[bi >> 5] = -INFINITY;
    }
    if (lane == 0) {
        if (order == 1) {
            float mm = sel_val[0];
            for (int r = 0; r < k; ++r) sel_sum += __expf(sel_val[r] - mm);
            for (int r = 0; r < k; ++r) probs[tok * k + r] = __expf(sel_val[r] - mm) / sel_sum;
        } else {
            for (int r = 0; r < k; ++r) probs[tok * k + r] = __expf(sel_val[r] - m) * inv;
        }
        for (int r = 0; r < k; ++r) {
            idx[tok * k + r] = sel_idx[r];
            if (counts != nullptr) atomicAdd(&counts[sel_idx[r]], 1);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Fused AdamW over a flat shard: fp32 grad, fp32 moments, optional fp32 master; writes the model-dtype
// parameter in the same pass.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void fused_adam_kernel(T* __restrict__ p, float* __restrict__ master, const float* __restrict__ g,
                                  float* __restrict__ m, float* __restrict__ v, int64_t n, float lr, float b1, float b2,
                                  float eps, float wd, float bc1, float bc2, float gscale) {
    for (int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (int64_t)gridDim.x * blockDim.x * 4) {
        float4 gv = *reinterpret_cast<const float4*>(g + i);
        float4 mv = *reinterpret_cast<const float4*>(m + i);
        float4 vv = *reinterpret_cast<const float4*>(v + i);
        float4 wv;
        if (master != nullptr) wv = *reinterpret_cast<const float4*>(master + i);
        else { wv.x = to_f(p[i]); wv.y = to_f(p[i + 1]); wv.z = to_f(p[i + 2]); wv.w = to_f(p[i + 3]); }
        float* gp = &gv.x; float* mp = &mv.x; float* vp = &vv.x; float* wp = &wv.x;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float gg = gp[e] * gscale;
            mp[e] = b1 * mp[e] + (1.f - b1) * gg;
            vp[e] = b2 * vp[e] + (1.f - b2) * gg * gg;
            float denom = sqrtf(vp[e] / bc2) + eps;
            wp[e] = wp[e] * (1.f - lr * wd) - lr * (mp[e] / bc1) / denom;
        }
        *reinterpret_cast<float4*>(m + i) = mv;
        *reinterpret_cast<float4*>(v + i) = vv;
        if (master != nullptr) *reinterpret_cast<float4*>(master + i) = wv;
        p[i] = from_f<T>(wv.x); p[i + 1] = from_f<T>(wv.y); p[i + 2] = from_f<T>(wv.z); p[i + 3] = from_f<T>(wv.w);
    }
}

// main_grad (fp32) += grad (bf16/fp32): gradient accumulation into the flat buffer.
template <typename T>
__global__ void accumulate_grad_kernel(float* __restrict__ acc, const T* __restrict__ g, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        acc[i] += to_f(g[i]);
}

}  // namespace lmoe

using namespace lmoe;

#define DISPATCH_T(dtype, ...)                      \
    if ((dtype) == 1) { typedef bf16 T; __VA_ARGS__ } \
    else { typedef float T; __VA_ARGS__ }

static inline int grid_for(int64_t n, int threads, int cap = 148 * 16) {
    int64_t b = (n + threads - 1) / threads;
    return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

LMOE_API int lmoe_rms_norm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out, float* rstd,
                               int64_t rows, int N, float eps, int dtype, cudaStream_t st) {
    DISPATCH_T(dtype, {
        constexpr int VN = Vec<T>::N;
        if (N % VN != 0) return -1;
        int nvec = N / VN;
        int threads = pick_threads(nvec);
        if (nvec > threads * 8) return -2;
        if (nvec <= threads * 1)
            rms_norm_fwd_kernel<T, 1><<<rows, threads, 0, st>>>((const T*)x, (const T*)res, (const T*)w, (T*)y, (T*)res_out, rstd, N, eps);
        else if (nvec <= threads * 2)
            rms_norm_fwd_kernel<T, 2><<<rows, threads, 0, st>>>((const T*)x, (const T*)res, (const T*)w, (T*)y, (T*)res_out, rstd, N, eps);
        else if (nvec <= threads * 4)
            rms_norm_fwd_kernel<T, 4><<<rows, threads, 0, st>>>((const T*)x, (const T*)res, (const T*)w, (T*)y, (T*)res_out, rstd, N, eps);
        else
            rms_norm_fwd_kernel<T, 8><<<rows, threads, 0, st>>>((const T*)x, (const T*)res, (const T*)w, (T*)y, (T*)res_out, rstd, N, eps);
    })
    return (int)cudaGetLastError();
}

// dw_partial: [P, N] fp32 scratch with P = value returned through *P_out (<= max_blocks)
LMOE_API int lmoe_rms_norm_bwd(const void* dy, const void* xin, const void* w, const float* rstd, const void* dres,
                               void* dx, float* dw_partial, void* dw, int64_t rows, int N, int P, int dtype,
                               cudaStream_t st) {
    DISPATCH_T(dtype, {
        constexpr int VN = Vec<T>::N;
        if (N % VN != 0) return -1;
        int nvec = N / VN;
        int threads = pick_threads(nvec);
        if (nvec > threads * 8) return -2;
        int blocks = (int)(rows < P ? rows : P);
        if (nvec <= threads * 1)
            rms_norm_bwd_kernel<T, 1><<<blocks, threads, 0, st>>>((const T*)dy, (const T*)xin, (const T*)w, rstd, (const T*)dres, (T*)dx, dw_partial, (int)rows, N);
        else if (nvec <= threads * 2)
            rms_norm_bwd_kernel<T, 2><<<blocks, threads, 0, st>>>((const T*)dy, (const T*)xin, (const T*)w, rstd, (const T*)dres, (T*)dx, dw_partial, (int)rows, N);
        else if (nvec <= threads * 4)
            rms_norm_bwd_kernel<T, 4><<<blocks, threads, 0, st>>>((const T*)dy, (const T*)xin, (const T*)w, rstd, (const T*)dres, (T*)dx, dw_partial, (int)rows, N);
        else
            rms_norm_bwd_kernel<T, 8><<<blocks, threads, 0, st>>>((const T*)dy, (const T*)xin, (const T*)w, rstd, (const T*)dres, (T*)dx, dw_partial, (int)rows, N);
        if (dw != nullptr && dw_partial != nullptr)
            reduce_partials_kernel<T><<<(N + 31) / 32, 256, 0, st>>>(dw_partial, (T*)dw, blocks, N);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_head_norm_gate_fwd(const void* o, const void* w, const void* gate, void* y, float* rstd, int64_t rows,
                                     int D, float eps, int do_norm, int dtype, cudaStream_t st) {
    if (D > 512 || D % 4 != 0) return -1;
    const int wpb = 8;
    int64_t need = (rows + wpb - 1) / wpb;
    int blocks = (int)(need < 148 * 8 ? need : 148 * 8);
    DISPATCH_T(dtype, {
        if (D <= 128) head_norm_gate_fwd_kernel<T, 128><<<blocks, wpb * 32, 0, st>>>((const T*)o, (const T*)w, (const T*)gate, (T*)y, rstd, rows, D, eps, do_norm);
        else if (D <= 256) head_norm_gate_fwd_kernel<T, 256><<<blocks, wpb * 32, 0, st>>>((const T*)o, (const T*)w, (const T*)gate, (T*)y, rstd, rows, D, eps, do_norm);
        else head_norm_gate_fwd_kernel<T, 512><<<blocks, wpb * 32, 0, st>>>((const T*)o, (const T*)w, (const T*)gate, (T*)y, rstd, rows, D, eps, do_norm);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_head_norm_gate_bwd(const void* dy, const void* o, const void* w, const void* gate, const float* rstd,
                                     void* d_o, void* dgate, float* dw_partial, void* dw, int64_t rows, int D,
                                     int do_norm, int P, int dtype, cudaStream_t st) {
    if (D > 512 || D % 4 != 0) return -1;
    const int wpb = 8;
    int64_t need = (rows + wpb - 1) / wpb;
    int blocks = (int)(need < P ? need : P);
    DISPATCH_T(dtype, {
        if (D <= 128) head_norm_gate_bwd_kernel<T, 128><<<blocks, wpb * 32, wpb * 128 * 4, st>>>((const T*)dy, (const T*)o, (const T*)w, (const T*)gate, rstd, (T*)d_o, (T*)dgate, dw_partial, rows, D, do_norm);
        else if (D <= 256) head_norm_gate_bwd_kernel<T, 256><<<blocks, wpb * 32, wpb * 256 * 4, st>>>((const T*)dy, (const T*)o, (const T*)w, (const T*)gate, rstd, (T*)d_o, (T*)dgate, dw_partial, rows, D, do_norm);
        else head_norm_gate_bwd_kernel<T, 512><<<blocks, wpb * 32, wpb * 512 * 4, st>>>((const T*)dy, (const T*)o, (const T*)w, (const T*)gate, rstd, (T*)d_o, (T*)dgate, dw_partial, rows, D, do_norm);
        if (dw != nullptr && dw_partial != nullptr)
            reduce_partials_kernel<T><<<(D + 31) / 32, 256, 0, st>>>(dw_partial, (T*)dw, blocks, D);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_gated_rms_norm_fwd(const void* x, const void* z, const void* w, void* y, float* rstd, int64_t rows,
                                     int N, int G, float eps, int dtype, cudaStream_t st) {
    int64_t warps = rows * (N / G);
    int blocks = (int)((warps + 7) / 8);
    DISPATCH_T(dtype, {
        gated_rms_norm_fwd_kernel<T><<<blocks, 256, 0, st>>>((const T*)x, (const T*)z, (const T*)w, (T*)y, rstd, rows, N, G, eps);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_gated_rms_norm_bwd(const void* dy, const void* x, const void* z, const void* w, const float* rstd,
                                     void* dx, void* dz, float* dw, int64_t rows, int N, int G, int dtype,
                                     cudaStream_t st) {
    int64_t warps = rows * (N / G);
    int blocks = grid_for(warps * 32, 256, 148 * 8);
    DISPATCH_T(dtype, {
        gated_rms_norm_bwd_kernel<T><<<blocks, 256, 0, st>>>((const T*)dy, (const T*)x, (const T*)z, (const T*)w, rstd, (T*)dx, (T*)dz, dw, rows, N, G);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_swiglu_fwd(const void* x, void* y, int64_t rows, int F, int dtype, cudaStream_t st) {
    DISPATCH_T(dtype, {
        if (F % Vec<T>::N != 0) return -1;
        swiglu_fwd_kernel<T><<<grid_for(rows * (F / Vec<T>::N), 256), 256, 0, st>>>((const T*)x, (T*)y, rows, F);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_swiglu_bwd(const void* dy, const void* x, void* dx, int64_t rows, int F, int dtype, cudaStream_t st) {
    DISPATCH_T(dtype, {
        if (F % Vec<T>::N != 0) return -1;
        swiglu_bwd_kernel<T><<<grid_for(rows * (F / Vec<T>::N), 256), 256, 0, st>>>((const T*)dy, (const T*)x, (T*)dx, rows, F);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_l2norm_fwd(const void* x, void* y, float* rstd, int64_t rows, int D, float eps, int dtype,
                             cudaStream_t st) {
    if (D > 512) return -1;
    int blocks = (int)((rows + 7) / 8);
    DISPATCH_T(dtype, {
        if (D <= 128) l2norm_fwd_kernel<T, 128><<<blocks, 256, 0, st>>>((const T*)x, (T*)y, rstd, rows, D, eps);
        else if (D <= 256) l2norm_fwd_kernel<T, 256><<<blocks, 256, 0, st>>>((const T*)x, (T*)y, rstd, rows, D, eps);
        else l2norm_fwd_kernel<T, 512><<<blocks, 256, 0, st>>>((const T*)x, (T*)y, rstd, rows, D, eps);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_l2norm_bwd(const void* dy, const void* x, const float* rstd, void* dx, int64_t rows, int D, int dtype,
                             cudaStream_t st) {
    if (D > 512) return -1;
    int blocks = (int)((rows + 7) / 8);
    DISPATCH_T(dtype, {
        if (D <= 128) l2norm_bwd_kernel<T, 128><<<blocks, 256, 0, st>>>((const T*)dy, (const T*)x, rstd, (T*)dx, rows, D);
        else if (D <= 256) l2norm_bwd_kernel<T, 256><<<blocks, 256, 0, st>>>((const T*)dy, (const T*)x, rstd, (T*)dx, rows, D);
        else l2norm_bwd_kernel<T, 512><<<blocks, 256, 0, st>>>((const T*)dy, (const T*)x, rstd, (T*)dx, rows, D);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_rope(const void* x, const float* cs, const float* sn, void* y, int64_t BT, int Tlen, int H, int D,
                       int R, int interleaved, int conj, int dtype, cudaStream_t st) {
    int64_t total = BT * H * (int64_t)(D - R / 2);
    DISPATCH_T(dtype, {
        rope_kernel<T><<<grid_for(total, 256), 256, 0, st>>>((const T*)x, cs, sn, (T*)y, BT, Tlen, H, D, R, interleaved, conj);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_softmax_ce_fwd(const void* logits, const int64_t* labels, float* loss, float* lse, int64_t rows, int V,
                                 int64_t ignore, int dtype, cudaStream_t st) {
    DISPATCH_T(dtype, {
        if ((V * sizeof(T)) % 16 != 0) return -1;
        softmax_ce_fwd_kernel<T><<<rows, 512, 0, st>>>((const T*)logits, labels, loss, lse, V, ignore);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_softmax_ce_bwd(const void* logits, const int64_t* labels, const float* lse, const float* gloss,
                                 void* grad, int64_t rows, int V, int64_t ignore, int dtype, cudaStream_t st) {
    DISPATCH_T(dtype, {
        if ((V * sizeof(T)) % 16 != 0) return -1;
        softmax_ce_bwd_kernel<T><<<rows, 512, 0, st>>>((const T*)logits, labels, lse, gloss, (T*)grad, V, ignore);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_causal_conv1d_fwd(const void* x, const void* w, const void* bias, const void* init, void* y, int B,
                                    int Tlen, int D, int K, int act, int dtype, cudaStream_t st) {
    int64_t total = (int64_t)B * Tlen * D;
    DISPATCH_T(dtype, {
        constexpr int VN = Vec<T>::N;
        if (D % VN == 0 && K >= 2 && K <= 4) {
            const int trun = 32;
            dim3 vgrid((D / VN + 127) / 128, (Tlen + trun - 1) / trun, B);
            if (K == 4) causal_conv1d_fwd_vec_kernel<T, 4><<<vgrid, 128, 0, st>>>((const T*)x, (const T*)w, (const T*)bias, (const T*)init, (T*)y, B, Tlen, D, act, trun);
            else if (K == 3) causal_conv1d_fwd_vec_kernel<T, 3><<<vgrid, 128, 0, st>>>((const T*)x, (const T*)w, (const T*)bias, (const T*)init, (T*)y, B, Tlen, D, act, trun);
            else causal_conv1d_fwd_vec_kernel<T, 2><<<vgrid, 128, 0, st>>>((const T*)x, (const T*)w, (const T*)bias, (const T*)init, (T*)y, B, Tlen, D, act, trun);
            return (int)cudaGetLastError();
        }
        int g = grid_for(total, 256);
        if (K == 4) causal_conv1d_fwd_kernel<T, 4><<<g, 256, 0, st>>>((const T*)x, (const T*)w, (const T*)bias, (const T*)init, (T*)y, B, Tlen, D, act);
        else if (K == 3) causal_conv1d_fwd_kernel<T, 3><<<g, 256, 0, st>>>((const T*)x, (const T*)w, (const T*)bias, (const T*)init, (T*)y, B, Tlen, D, act);
        else if (K == 2) causal_conv1d_fwd_kernel<T, 2><<<g, 256, 0, st>>>((const T*)x, (const T*)w, (const T*)bias, (const T*)init, (T*)y, B, Tlen, D, act);
        else return -1;
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_causal_conv1d_bwd(const void* dy, const void* x, const void* w, const void* bias, const void* init,
                                    void* dx, float* dw, float* dbias, void* dinit, int B, int Tlen, int D, int K,
                                    int act, int dtype, cudaStream_t st) {
    const int tchunk = 128;
    dim3 grid((D + 127) / 128, (Tlen + tchunk - 1) / tchunk, B);
    DISPATCH_T(dtype, {
        constexpr int VN = Vec<T>::N;
        if (D % VN == 0 && K >= 2 && K <= 4) {
            const int trun = 64;
            dim3 vgrid((D / VN + 63) / 64, (Tlen + trun - 1) / trun, B);
            if (K == 4) causal_conv1d_bwd_vec_kernel<T, 4><<<vgrid, 64, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, (const T*)bias, (const T*)init, (T*)dx, dw, dbias, (T*)dinit, B, Tlen, D, act, trun);
            else if (K == 3) causal_conv1d_bwd_vec_kernel<T, 3><<<vgrid, 64, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, (const T*)bias, (const T*)init, (T*)dx, dw, dbias, (T*)dinit, B, Tlen, D, act, trun);
            else causal_conv1d_bwd_vec_kernel<T, 2><<<vgrid, 64, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, (const T*)bias, (const T*)init, (T*)dx, dw, dbias, (T*)dinit, B, Tlen, D, act, trun);
            return (int)cudaGetLastError();
        }
        if (K == 4) causal_conv1d_bwd_kernel<T, 4><<<grid, 128, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, (const T*)bias, (const T*)init, (T*)dx, dw, dbias, (T*)dinit, B, Tlen, D, act, tchunk);
        else if (K == 3) causal_conv1d_bwd_kernel<T, 3><<<grid, 128, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, (const T*)bias, (const T*)init, (T*)dx, dw, dbias, (T*)dinit, B, Tlen, D, act, tchunk);
        else if (K == 2) causal_conv1d_bwd_kernel<T, 2><<<grid, 128, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, (const T*)bias, (const T*)init, (T*)dx, dw, dbias, (T*)dinit, B, Tlen, D, act, tchunk);
        else return -1;
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_router_topk(const float* logits, float* full, float* probs, int64_t* idx, int* counts, int64_t Ttok,
                              int E, int k, int order, cudaStream_t st) {
    if (E > 256 || k > 16) return -1;
    int blocks = (int)((Ttok + 7) / 8);
    router_topk_kernel<<<blocks, 256, 0, st>>>(logits, full, probs, idx, counts, Ttok, E, k, order);
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_fused_adam(void* p, float* master, const float* g, float* m, float* v, int64_t n, float lr, float b1,
                             float b2, float eps, float wd, float bc1, float bc2, float gscale, int dtype,
                             cudaStream_t st) {
    if (n % 4 != 0) return -1;
    DISPATCH_T(dtype, {
        fused_adam_kernel<T><<<grid_for(n / 4, 256), 256, 0, st>>>((T*)p, master, g, m, v, n, lr, b1, b2, eps, wd, bc1, bc2, gscale);
    })
    return (int)cudaGetLastError();
}

LMOE_API int lmoe_accumulate_grad(float* acc, const void* g, int64_t n, int dtype, cudaStream_t st) {
    DISPATCH_T(dtype, {
        accumulate_grad_kernel<T><<<grid_for(n, 256), 256, 0, st>>>(acc, (const T*)g, n);
    })
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// RMSNorm backward without any allocation: the dw partials go to a fixed array in the library image.
// See lmoe_noalloc.h for the contract.
// ---------------------------------------------------------------------------------------------
#include "lmoe_noalloc.h"

static __device__ __align__(256) float g_noalloc_partials[LMOE_NOALLOC_MAX_BLOCKS * LMOE_NOALLOC_MAX_N];

// Device address of g_noalloc_partials per device ordinal.  In host code the array's name is only a handle for
// the runtime, not a device pointer: the address a kernel can use comes from cudaGetSymbolAddress, looked up
// once per device with that device current.
static float* g_noalloc_addr[64] = {nullptr};

static int noalloc_scratch(float** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return LMOE_NOALLOC_ERR_SETUP;
    if (g_noalloc_addr[dev] == nullptr) {
        float* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, g_noalloc_partials) != cudaSuccess || p == nullptr)
            return LMOE_NOALLOC_ERR_SETUP;
        g_noalloc_addr[dev] = p;
    }
    *out = g_noalloc_addr[dev];
    return 0;
}

LMOE_API const char* lmoe_noalloc_strerror(int code) {
    switch (code) {
        case 0: return "ok";
        case LMOE_NOALLOC_ERR_SIZE:
            return "lmoe_rms_norm_bwd_noalloc: N exceeds LMOE_NOALLOC_MAX_N (4096) or is not a multiple of the "
                   "vector width (8 for bf16, 4 for fp32), or rows exceeds 2^31 - 1";
        case LMOE_NOALLOC_ERR_SETUP:
            return "lmoe_rms_norm_bwd_noalloc: could not obtain the device address of the built-in scratch array";
        default: return "lmoe_rms_norm_bwd_noalloc: CUDA launch error (code is a cudaError_t)";
    }
}

LMOE_API int lmoe_rms_norm_bwd_noalloc(const void* dy, const void* xin, const void* w, const float* rstd,
                                       const void* dres, void* dx, void* dw, int64_t rows, int N, int dtype,
                                       cudaStream_t st) {
    const int vn = dtype == 1 ? 8 : 4;
    if (N <= 0 || N > LMOE_NOALLOC_MAX_N || N % vn != 0) return LMOE_NOALLOC_ERR_SIZE;
    if (rows < 0 || rows > 2147483647LL) return LMOE_NOALLOC_ERR_SIZE;      // the kernels take the row count as an int
    if (rows == 0) return 0;
    float* scratch = nullptr;
    int rc = noalloc_scratch(&scratch);
    if (rc != 0) return rc;
    // same kernels as lmoe_rms_norm_bwd, with the built-in array as the partials buffer
    rc = lmoe_rms_norm_bwd(dy, xin, w, rstd, dres, dx, w != nullptr ? scratch : nullptr, dw, rows, N,
                           LMOE_NOALLOC_MAX_BLOCKS, dtype, st);
    return rc < 0 ? LMOE_NOALLOC_ERR_SIZE : rc;        // the launcher's own size refusals (-1, -2) are size errors too
}
