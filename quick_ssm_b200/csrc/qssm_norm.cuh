// RMS normalisation of the layer input, forward and backward.
//
// The layer that calls the scan normalises its input first (reference: quick_ssm/layers.py:9-17):
//     y[r, :] = x[r, :] * w / sqrt(mean(x[r, :]^2) + eps)
// In torch that is five element-wise kernels forward and a dozen backward.  Here one kernel per
// direction moves the minimum bytes: forward reads x, writes y (and one float per row, rstd, kept for
// the backward); backward reads x and dy, writes dx, and leaves per-warp partial sums of dw that a
// second small kernel adds up in a fixed order (no atomics: dw is deterministic).
//     r = 1 / sqrt(mean(x^2) + eps)
//     dx = r * (w*dy) - x * r^3 * mean(x * w*dy)          dw = sum over rows of dy * x * r
//
// One warp per row, persistent over rows.  A lane owns EPL consecutive elements of every chunk of
// 32*EPL elements: EPL = 4 (one 16-byte access of fp32, 8 bytes of 16-bit data) or, for 16-bit rows
// whose length and pitch are multiples of 8 elements, EPL = 8 (16 bytes: half the load and store
// instructions per element, which is what bounds these kernels on 16-bit data).  Rows of up to
// 32*EPL*NCH elements are held in registers between the reduction and the output; longer rows
// (NCH = 0) are read twice, the second time from L1/L2.  The forward also keeps the weight in
// registers across the rows a warp walks (it is read from L1 once per warp instead of once per row).
// No bulk copies: rows are short, contiguous and touched once; shared memory only for the dw partials.
#pragma once
#include <type_traits>

#include "qssm_tile.cuh"

namespace qssm {

constexpr int NORM_WARPS = 8;  // warps per CTA

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
}
template <> __device__ __forceinline__ void load4<__half>(const __half* p, float (&v)[4]) {
    const uint2 q = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&q.x));
    const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&q.y));
    v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 q = *reinterpret_cast<const uint2*>(p);
    v[0] = __uint_as_float(q.x << 16); v[1] = __uint_as_float(q.x & 0xffff0000u);
    v[2] = __uint_as_float(q.y << 16); v[3] = __uint_as_float(q.y & 0xffff0000u);
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store4<__half>(__half* p, const float (&v)[4]) {
    const __half2 lo = __floats2half2_rn(v[0], v[1]), hi = __floats2half2_rn(v[2], v[3]);
    uint2 q;
    q.x = *reinterpret_cast<const unsigned int*>(&lo);
    q.y = *reinterpret_cast<const unsigned int*>(&hi);
    *reinterpret_cast<uint2*>(p) = q;
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 q;
    q.x = *reinterpret_cast<const unsigned int*>(&lo);
    q.y = *reinterpret_cast<const unsigned int*>(&hi);
    *reinterpret_cast<uint2*>(p) = q;
}

// EPL elements per lane and access: 4 (16 bytes of fp32, 8 bytes of 16-bit data) or, for 16-bit data whose
// rows allow it, 8 (16 bytes): half the load/store instructions per element.
template <typename T, int EPL> __device__ __forceinline__ void loadv(const T* p, float (&v)[EPL]) {
    if constexpr (EPL == 4) {
        load4<T>(p, v);
    } else {
        static_assert(EPL == 8 && sizeof(T) == 2, "eight elements per access are for 16-bit data");
        const uint4 q = *reinterpret_cast<const uint4*>(p);
        const unsigned int w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if constexpr (std::is_same<T, __half>::value) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
                v[2 * i] = f.x;
                v[2 * i + 1] = f.y;
            } else {
                v[2 * i] = __uint_as_float(w[i] << 16);
                v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
        }
    }
}
template <typename T, int EPL> __device__ __forceinline__ void storev(T* p, const float (&v)[EPL]) {
    if constexpr (EPL == 4) {
        store4<T>(p, v);
    } else {
        unsigned int w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if constexpr (std::is_same<T, __half>::value) {
                const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<const unsigned int*>(&h);
            } else {
                const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<const unsigned int*>(&h);
            }
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}
template <int EPL> __device__ __forceinline__ void loadw(const float* p, float (&v)[EPL]) {
#pragma unroll
    for (int i = 0; i < EPL; i += 4) {
        const float4 q = *reinterpret_cast<const float4*>(p + i);
        v[i] = q.x; v[i + 1] = q.y; v[i + 2] = q.z; v[i + 3] = q.w;
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct NormParams {
    const void* x;
    const float* w;
    void* y;            // forward: y; backward: dx
    const void* dy;     // backward only
    float* rstd;        // [rows]; forward writes (may be NULL), backward reads
    float* dw_part;     // backward: partial sums of dw, [gridDim.x, H] (rows held in registers) or
                        // [gridDim.x * NORM_WARPS, H] (long rows)
    long long rows, x_stride, y_stride, dy_stride;
    int H;
    float eps;
};

template <typename T, int NCH, int EPL>
__global__ void __launch_bounds__(32 * NORM_WARPS) rmsnorm_fwd_kernel(const NormParams p) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
    const long long n_warps = (long long)gridDim.x * NORM_WARPS;
    const int H = p.H;
    const float inv_h = 1.f / (float)H;
    constexpr bool W_IN_REGS = NCH > 0 && NCH * EPL <= 32;  // up to 32 weights per lane stay in registers
    float wreg[W_IN_REGS ? NCH : 1][EPL];
    if (W_IN_REGS) {
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
            const int col = (c * 32 + lane) * EPL;
            if (col < H) loadw<EPL>(p.w + col, wreg[c]);
            else {
#pragma unroll
                for (int i = 0; i < EPL; ++i) wreg[c][i] = 0.f;
            }
        }
    }
    for (long long row = warp; row < p.rows; row += n_warps) {
        const T* xr = static_cast<const T*>(p.x) + row * p.x_stride;
        T* yr = static_cast<T*>(p.y) + row * p.y_stride;
        float ss = 0.f;
        if (NCH > 0) {
            float v[NCH > 0 ? NCH : 1][EPL];
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const int col = (c * 32 + lane) * EPL;
                if (col < H) loadv<T, EPL>(xr + col, v[c]);
                else {
#pragma unroll
                    for (int i = 0; i < EPL; ++i) v[c][i] = 0.f;
                }
            }
#pragma unroll
            for (int c = 0; c < NCH; ++c)
#pragma unroll
                for (int i = 0; i < EPL; ++i) ss = fmaf(v[c][i], v[c][i], ss);
            ss = warp_sum(ss);
            const float r = 1.f / sqrtf(ss * inv_h + p.eps);
            if (lane == 0 && p.rstd != nullptr) p.rstd[row] = r;
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const int col = (c * 32 + lane) * EPL;
                if (col < H) {
                    float w4[EPL], o[EPL];
                    if (W_IN_REGS) {
#pragma unroll
                        for (int i = 0; i < EPL; ++i) w4[i] = wreg[W_IN_REGS ? c : 0][i];
                    } else {
                        loadw<EPL>(p.w + col, w4);
                    }
#pragma unroll
                    for (int i = 0; i < EPL; ++i) o[i] = v[c][i] * (w4[i] * r);
                    storev<T, EPL>(yr + col, o);
                }
            }
        } else {
            for (int col = lane * EPL; col < H; col += 32 * EPL) {
                float v[EPL];
                loadv<T, EPL>(xr + col, v);
#pragma unroll
                for (int i = 0; i < EPL; ++i) ss = fmaf(v[i], v[i], ss);
            }
            ss = warp_sum(ss);
            const float r = 1.f / sqrtf(ss * inv_h + p.eps);
            if (lane == 0 && p.rstd != nullptr) p.rstd[row] = r;
            for (int col = lane * EPL; col < H; col += 32 * EPL) {
                float v[EPL], w4[EPL], o[EPL];
                loadv<T, EPL>(xr + col, v);
                loadw<EPL>(p.w + col, w4);
#pragma unroll
                for (int i = 0; i < EPL; ++i) o[i] = v[i] * (w4[i] * r);
                storev<T, EPL>(yr + col, o);
            }
        }
    }
}

template <typename T, int NCH, int EPL>
__global__ void __launch_bounds__(32 * NORM_WARPS) rmsnorm_bwd_kernel(const NormParams p) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
    const long long n_warps = (long long)gridDim.x * NORM_WARPS;
    const int H = p.H;
    const float inv_h = 1.f / (float)H;
    float* const part = p.dw_part + (NCH > 0 ? (long long)blockIdx.x : warp) * H;  // long rows: one per warp

    float acc[NCH > 0 ? NCH : 1][EPL];
    if (NCH > 0) {
#pragma unroll
        for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < EPL; ++i) acc[c][i] = 0.f;
    } else {
        for (int col = lane * EPL; col < H; col += 32 * EPL) {
#pragma unroll
            for (int i = 0; i < EPL; i += 4) *reinterpret_cast<float4*>(part + col + i) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }

    for (long long row = warp; row < p.rows; row += n_warps) {
        const T* xr = static_cast<const T*>(p.x) + row * p.x_stride;
        const T* gr = static_cast<const T*>(p.dy) + row * p.dy_stride;
        T* dr = static_cast<T*>(p.y) + row * p.y_stride;
        const float r = p.rstd[row];
        float dot = 0.f;
        if (NCH > 0) {
            // all loads of the row first (they are independent: the whole row is in flight at once), then
            // the arithmetic; wg holds dy on the way in and w*dy afterwards
            float v[NCH > 0 ? NCH : 1][EPL], wg[NCH > 0 ? NCH : 1][EPL];
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const int col = (c * 32 + lane) * EPL;
                if (col < H) {
                    loadv<T, EPL>(xr + col, v[c]);
                    loadv<T, EPL>(gr + col, wg[c]);
                } else {
#pragma unroll
                    for (int i = 0; i < EPL; ++i) v[c][i] = wg[c][i] = 0.f;
                }
            }
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const int col = (c * 32 + lane) * EPL;
                if (col < H) {
                    float w4[EPL];
                    loadw<EPL>(p.w + col, w4);
#pragma unroll
                    for (int i = 0; i < EPL; ++i) {
                        acc[c][i] = fmaf(wg[c][i] * r, v[c][i], acc[c][i]);
                        wg[c][i] *= w4[i];
                        dot = fmaf(v[c][i], wg[c][i], dot);
                    }
                }
            }
            dot = warp_sum(dot);
            const float k = dot * inv_h * r * r * r;
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                const int col = (c * 32 + lane) * EPL;
                if (col < H) {
                    float o[EPL];
#pragma unroll
                    for (int i = 0; i < EPL; ++i) o[i] = fmaf(-v[c][i], k, r * wg[c][i]);
                    storev<T, EPL>(dr + col, o);
                }
            }
        } else {
            for (int col = lane * EPL; col < H; col += 32 * EPL) {
                float v[EPL], g[EPL], w4[EPL], a4[EPL];
                loadv<T, EPL>(xr + col, v);
                loadv<T, EPL>(gr + col, g);
                loadw<EPL>(p.w + col, w4);
                loadw<EPL>(part + col, a4);
#pragma unroll
                for (int i = 0; i < EPL; ++i) {
                    a4[i] = fmaf(g[i] * r, v[i], a4[i]);
                    dot = fmaf(v[i], w4[i] * g[i], dot);
                }
                {
#pragma unroll
                    for (int i = 0; i < EPL; i += 4)
                        *reinterpret_cast<float4*>(part + col + i) = make_float4(a4[i], a4[i + 1], a4[i + 2], a4[i + 3]);
                }
            }
            dot = warp_sum(dot);
            const float k = dot * inv_h * r * r * r;
            for (int col = lane * EPL; col < H; col += 32 * EPL) {
                float v[EPL], g[EPL], w4[EPL], o[EPL];
                loadv<T, EPL>(xr + col, v);
                loadv<T, EPL>(gr + col, g);
                loadw<EPL>(p.w + col, w4);
#pragma unroll
                for (int i = 0; i < EPL; ++i) o[i] = fmaf(-v[i], k, r * (w4[i] * g[i]));
                storev<T, EPL>(dr + col, o);
            }
        }
    }
    if (NCH > 0) {  // add the eight warps' sums in warp order through shared memory: one partial row per CTA
        extern __shared__ __align__(16) float red[];
        for (int wv = 0; wv < NORM_WARPS; ++wv) {
            if ((int)(threadIdx.x >> 5) == wv) {
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    const int col = (c * 32 + lane) * EPL;
                    if (col < H) {
                        float t[EPL];
#pragma unroll
                        for (int i = 0; i < EPL; ++i) t[i] = 0.f;
                        if (wv > 0) loadw<EPL>(red + col, t);
#pragma unroll
                        for (int i = 0; i < EPL; ++i) t[i] += acc[c][i];
#pragma unroll
                        for (int i = 0; i < EPL; i += 4)
                            *reinterpret_cast<float4*>(red + col + i) = make_float4(t[i], t[i + 1], t[i + 2], t[i + 3]);
                    }
                }
            }
            __syncthreads();
        }
        for (int col = threadIdx.x * 4; col < H; col += 4 * 32 * NORM_WARPS)
            *reinterpret_cast<float4*>(part + col) = *reinterpret_cast<const float4*>(red + col);
    }
}

// dw[h] = sum over the partial rows: thread (tx, ty) adds rows ty, ty+8, ... of column h, then the eight
// sums of a column are added in ty order - a fixed order, so dw does not depend on scheduling.
__global__ void __launch_bounds__(256) rmsnorm_dw_kernel(const float* part, float* dw, long long n_part, int H) {
    __shared__ float red[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int h = blockIdx.x * 32 + tx;
    float s = 0.f;
    if (h < H)
        for (long long q = ty; q < n_part; q += 8) s += part[q * H + h];
    red[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && h < H) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += red[k][tx];
        dw[h] = t;
    }
}

}  // namespace qssm
