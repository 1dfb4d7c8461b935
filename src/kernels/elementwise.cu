#include "elementwise.cuh"

#include <cuda_bf16.h>

#include "launch_count.h"

namespace mgk {
namespace ew {

namespace {

__device__ __forceinline__ float lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(256) sgd_bf16_kernel(uint4* __restrict__ w, const uint4* __restrict__ g,
                                                       float4* __restrict__ mom, uint64_t nvec,
                                                       __nv_bfloat16* w_tail, const __nv_bfloat16* g_tail,
                                                       float* m_tail, int ntail, float lr, float mu, float wd) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        uint4 wv = w[i];
        const uint4 gv = __ldcs(g + i);
        float wf[8] = {lo(wv.x), hi(wv.x), lo(wv.y), hi(wv.y), lo(wv.z), hi(wv.z), lo(wv.w), hi(wv.w)};
        float gf[8] = {lo(gv.x), hi(gv.x), lo(gv.y), hi(gv.y), lo(gv.z), hi(gv.z), lo(gv.w), hi(gv.w)};
        if (mom != nullptr) {
            float4 m0 = mom[2 * i], m1 = mom[2 * i + 1];
            float mf[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                mf[k] = mu * mf[k] + gf[k] + wd * wf[k];
                wf[k] -= lr * mf[k];
            }
            mom[2 * i] = make_float4(mf[0], mf[1], mf[2], mf[3]);
            mom[2 * i + 1] = make_float4(mf[4], mf[5], mf[6], mf[7]);
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k)
                wf[k] -= lr * (gf[k] + wd * wf[k]);
        }
        wv.x = pack(wf[0], wf[1]);
        wv.y = pack(wf[2], wf[3]);
        wv.z = pack(wf[4], wf[5]);
        wv.w = pack(wf[6], wf[7]);
        w[i] = wv;
    }
    if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < ntail) {
        const int k = threadIdx.x;
        float wf = __bfloat162float(w_tail[k]);
        float gf = __bfloat162float(g_tail[k]) + wd * wf;
        if (m_tail != nullptr) {
            m_tail[k] = mu * m_tail[k] + gf;
            gf = m_tail[k];
        }
        w_tail[k] = __float2bfloat16_rn(wf - lr * gf);
    }
}

__global__ void __launch_bounds__(256) mse_bf16_kernel(const __nv_bfloat16* __restrict__ y,
                                                       const __nv_bfloat16* __restrict__ t,
                                                       __nv_bfloat16* __restrict__ dy, float* loss, uint64_t n,
                                                       float scale, int vec_ok) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const uint64_t tid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    float acc = 0.f;
    // 16-byte body (two vectors in flight per thread), scalar tail
    const uint64_t nvec = vec_ok ? n / 8 : 0;
    const uint4* yv = reinterpret_cast<const uint4*>(y);
    const uint4* tv = reinterpret_cast<const uint4*>(t);
    uint4* dv = reinterpret_cast<uint4*>(dy);
    auto one = [&](const uint4& a, const uint4& b, uint64_t i) {
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
        const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float d0 = lo(aw[k]) - lo(bw[k]);
            const float d1 = hi(aw[k]) - hi(bw[k]);
            acc += d0 * d0 + d1 * d1;
            ow[k] = pack(2.f * d0 * scale, 2.f * d1 * scale);
        }
        if (dy != nullptr)
            dv[i] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    };
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    // four independent vectors per thread and iteration, all loads issued before the first use
    constexpr int U = 4;
    uint64_t i = tid;
    for (; i + (U - 1) * stride < nvec; i += U * stride) {
        uint4 av[U], bv[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            av[u] = __ldcs(yv + i + u * stride);
            bv[u] = t != nullptr ? __ldcs(tv + i + u * stride) : zero;
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
            one(av[u], bv[u], i + u * stride);
    }
    for (; i < nvec; i += stride)
        one(__ldcs(yv + i), t != nullptr ? __ldcs(tv + i) : zero, i);
    for (uint64_t k = nvec * 8 + tid; k < n; k += stride) {
        const float d = __bfloat162float(y[k]) - (t != nullptr ? __bfloat162float(t[k]) : 0.f);
        acc += d * d;
        if (dy != nullptr)
            dy[k] = __float2bfloat16_rn(2.f * d * scale);
    }
    for (int o = 16; o > 0; o >>= 1)
        acc += __shfl_xor_sync(0xffffffffu, acc, o);
    __shared__ float part[8];
    if ((threadIdx.x & 31) == 0)
        part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.f;
        for (int k = 0; k < 8; ++k)
            s += part[k];
        atomicAdd(loss, s * scale);
    }
}


// One CTA of 256 threads per row; each thread keeps its 8-element vectors in registers so
// the row is read once.
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 8;  // 256 threads * 8 vectors * 8 elements = 16384 columns

__device__ __forceinline__ float block_sum(float v, float* smem) {
    for (int o = 16; o > 0; o >>= 1)
        v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0)
        smem[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kNormThreads / 32; ++k)
        s += smem[k];
    __syncthreads();
    return s;
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = lo(v.x); f[1] = hi(v.x); f[2] = lo(v.y); f[3] = hi(v.y);
    f[4] = lo(v.z); f[5] = hi(v.z); f[6] = lo(v.w); f[7] = hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 v;
    v.x = pack(f[0], f[1]); v.y = pack(f[2], f[3]); v.z = pack(f[4], f[5]); v.w = pack(f[6], f[7]);
    return v;
}

// NV = 16-byte vectors per thread; the row stays in registers as packed bf16 (4 registers per
// vector), which keeps several CTAs resident per SM.
template <int NV>
__global__ void __launch_bounds__(kNormThreads, NV <= 4 ? 4 : 2)
        add_rmsnorm_kernel(const uint4* __restrict__ x, const uint4* __restrict__ y, uint4* __restrict__ x_out,
                           uint4* __restrict__ n_out, float* __restrict__ inv_rms, int cols, float eps) {
    __shared__ float red[kNormThreads / 32];
    const int nvec = cols / 8;
    const size_t row = blockIdx.x;
    const uint4* xr = x + row * nvec;
    const uint4* yr = y != nullptr ? y + row * nvec : nullptr;
    uint4 xs[NV], ys[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = threadIdx.x + v * kNormThreads;
        if (i < nvec) {
            xs[v] = xr[i];
            if (yr != nullptr)
                ys[v] = __ldcs(yr + i);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = threadIdx.x + v * kNormThreads;
        if (i < nvec) {
            float s[8];
            unpack8(xs[v], s);
            if (yr != nullptr) {
                float t[8];
                unpack8(ys[v], t);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    s[k] += t[k];
                // the sum is rounded to bf16 where it is stored; normalise what was stored
                xs[v] = pack8(s);
                unpack8(xs[v], s);
            }
            if (x_out != nullptr)
                x_out[row * nvec + i] = xs[v];
#pragma unroll
            for (int k = 0; k < 8; ++k)
                ss += s[k] * s[k];
        }
    }
    if (n_out == nullptr && inv_rms == nullptr)
        return;
    const float total = block_sum(ss, red);
    const float r = rsqrtf(total / static_cast<float>(cols) + eps);
    if (inv_rms != nullptr && threadIdx.x == 0)
        inv_rms[row] = r;
    if (n_out != nullptr) {
#pragma unroll
        for (int v = 0; v < NV; ++v) {
            const int i = threadIdx.x + v * kNormThreads;
            if (i < nvec) {
                float o[8];
                unpack8(xs[v], o);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    o[k] *= r;
                n_out[row * nvec + i] = pack8(o);
            }
        }
    }
}

template <int NV>
__global__ void __launch_bounds__(kNormThreads, NV <= 4 ? 4 : 2)
        rmsnorm_bwd_kernel(const uint4* __restrict__ dn, const uint4* __restrict__ n, const float* __restrict__ inv_rms,
                           const uint4* __restrict__ dres, uint4* __restrict__ dx, int cols) {
    __shared__ float red[kNormThreads / 32];
    const int nvec = cols / 8;
    const size_t row = blockIdx.x;
    uint4 gs[NV], ns[NV], ds[NV];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = threadIdx.x + v * kNormThreads;
        if (i < nvec) {
            gs[v] = __ldcs(dn + row * nvec + i);
            ns[v] = __ldcs(n + row * nvec + i);
            if (dres != nullptr)
                ds[v] = __ldcs(dres + row * nvec + i);
        }
    }
    float dot = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = threadIdx.x + v * kNormThreads;
        if (i < nvec) {
            float g[8], nn[8];
            unpack8(gs[v], g);
            unpack8(ns[v], nn);
#pragma unroll
            for (int k = 0; k < 8; ++k)
                dot += g[k] * nn[k];
        }
    }
    const float mean = block_sum(dot, red) / static_cast<float>(cols);
    const float r = inv_rms[row];
#pragma unroll
    for (int v = 0; v < NV; ++v) {
        const int i = threadIdx.x + v * kNormThreads;
        if (i < nvec) {
            float g[8], nn[8], o[8];
            unpack8(gs[v], g);
            unpack8(ns[v], nn);
#pragma unroll
            for (int k = 0; k < 8; ++k)
                o[k] = r * (g[k] - nn[k] * mean);
            if (dres != nullptr) {
                float d[8];
                unpack8(ds[v], d);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    o[k] += d[k];
            }
            dx[row * nvec + i] = pack8(o);
        }
    }
}

// Smallest vectors-per-thread count that covers the row.
inline int norm_nv(int cols) {
    const int need = (cols / 8 + kNormThreads - 1) / kNormThreads;
    return need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
}

}  // namespace

cudaError_t launch_sgd_bf16(void* w, const void* g, float* momentum, uint64_t n, float lr, float mu,
                            float weight_decay, cudaStream_t stream) {
    if (n == 0)
        return cudaSuccess;
    if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(g)) & 15)
        return cudaErrorInvalidValue;
    const uint64_t nvec = n / 8;
    const int ntail = static_cast<int>(n - nvec * 8);
    uint64_t blocks = (nvec + 255) / 256;
    if (blocks > 148 * 8)
        blocks = 148 * 8;
    if (blocks == 0)
        blocks = 1;
    auto* wb = static_cast<__nv_bfloat16*>(w);
    auto* gb = static_cast<const __nv_bfloat16*>(g);
    sgd_bf16_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
            static_cast<uint4*>(w), static_cast<const uint4*>(g), reinterpret_cast<float4*>(momentum), nvec,
            wb + nvec * 8, gb + nvec * 8, momentum != nullptr ? momentum + nvec * 8 : nullptr, ntail, lr, mu,
            weight_decay);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_mse_bf16(const void* y, const void* target, void* dy, float* loss_out, uint64_t n,
                            float scale, cudaStream_t stream) {
    if (n == 0)
        return cudaSuccess;
    uint64_t blocks = (n + 256 * 8 - 1) / (256 * 8);
    if (blocks > 148 * 8)
        blocks = 148 * 8;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(target) |
                           reinterpret_cast<uintptr_t>(dy);
    mse_bf16_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
            static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(target),
            static_cast<__nv_bfloat16*>(dy), loss_out, n, scale, (bits & 15) == 0 ? 1 : 0);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_add_rmsnorm_bf16(const void* x, const void* y, void* x_out, void* n_out, float* inv_rms,
                                    int rows, int cols, float eps, cudaStream_t stream) {
    if (rows <= 0)
        return cudaSuccess;
    if (cols <= 0 || cols % 8 || cols > kNormThreads * kNormMaxVec * 8)
        return cudaErrorInvalidValue;
    auto go = [&](auto kernel) {
        kernel<<<rows, kNormThreads, 0, stream>>>(static_cast<const uint4*>(x), static_cast<const uint4*>(y),
                                                  static_cast<uint4*>(x_out), static_cast<uint4*>(n_out), inv_rms,
                                                  cols, eps);
    };
    switch (norm_nv(cols)) {
        case 1: go(add_rmsnorm_kernel<1>); break;
        case 2: go(add_rmsnorm_kernel<2>); break;
        case 4: go(add_rmsnorm_kernel<4>); break;
        default: go(add_rmsnorm_kernel<8>); break;
    }
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_rmsnorm_bwd_bf16(const void* dn, const void* n, const float* inv_rms, const void* dres,
                                    void* dx, int rows, int cols, cudaStream_t stream) {
    if (rows <= 0)
        return cudaSuccess;
    if (cols <= 0 || cols % 8 || cols > kNormThreads * kNormMaxVec * 8)
        return cudaErrorInvalidValue;
    auto go = [&](auto kernel) {
        kernel<<<rows, kNormThreads, 0, stream>>>(static_cast<const uint4*>(dn), static_cast<const uint4*>(n),
                                                  inv_rms, static_cast<const uint4*>(dres),
                                                  static_cast<uint4*>(dx), cols);
    };
    switch (norm_nv(cols)) {
        case 1: go(rmsnorm_bwd_kernel<1>); break;
        case 2: go(rmsnorm_bwd_kernel<2>); break;
        case 4: go(rmsnorm_bwd_kernel<4>); break;
        default: go(rmsnorm_bwd_kernel<8>); break;
    }
    count_launch();
    return cudaGetLastError();
}

}  // namespace ew
}  // namespace mgk
