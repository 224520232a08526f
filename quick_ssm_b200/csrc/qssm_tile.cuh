// Element types, per-lane vectors, shared-memory tile access, kernel parameter blocks and the small
// bookkeeping structs shared by every scan kernel.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qssm.h"
#include "qssm_ptx.cuh"

namespace qssm {


constexpr int TS = QSSM_TILE_ROWS;  // rows scanned per register batch; granularity of tile_h
constexpr int MAX_STAGES = 16;

// ---------------------------------------------------------------------------------------------
// element helpers
// ---------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// V consecutive channels of one lane, moved with a single shared-memory access.
template <typename T, int V> struct alignas(sizeof(T) * V) Vec { T v[V]; };

// Row r of a tile whose rows hold 32 lanes x V elements of T.  Loads and the arithmetic on them
// are kept apart so that all shared-memory loads of a 16-row batch can be in flight together.
template <typename T, int V>
__device__ __forceinline__ Vec<T, V> tile_raw(const unsigned char* tile, int r, int lane) {
    return reinterpret_cast<const Vec<T, V>*>(tile)[r * 32 + lane];
}
template <typename T, int V>
__device__ __forceinline__ void tile_put(unsigned char* tile, int r, int lane, const Vec<T, V>& w) {
    reinterpret_cast<Vec<T, V>*>(tile)[r * 32 + lane] = w;
}
template <typename T, int V> __device__ __forceinline__ void unpack(const Vec<T, V>& w, float (&out)[V]) {
#pragma unroll
    for (int i = 0; i < V; ++i) out[i] = to_f<T>(w.v[i]);
}
template <typename T, int V> __device__ __forceinline__ Vec<T, V> pack(const float (&in)[V]) {
    Vec<T, V> w;
#pragma unroll
    for (int i = 0; i < V; ++i) w.v[i] = from_f<T>(in[i]);
    return w;
}
// two 16-bit channels: one packed conversion instead of two conversions and a merge
template <> __device__ __forceinline__ Vec<__nv_bfloat16, 2> pack<__nv_bfloat16, 2>(const float (&in)[2]) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(in[0], in[1]);
    Vec<__nv_bfloat16, 2> w;
    w.v[0] = p.x;
    w.v[1] = p.y;
    return w;
}
template <> __device__ __forceinline__ Vec<__half, 2> pack<__half, 2>(const float (&in)[2]) {
    const __half2 p = __floats2half2_rn(in[0], in[1]);
    Vec<__half, 2> w;
    w.v[0] = p.x;
    w.v[1] = p.y;
    return w;
}
template <> __device__ __forceinline__ void unpack<__half, 2>(const Vec<__half, 2>& w, float (&out)[2]) {
    const float2 f = __half22float2(__halves2half2(w.v[0], w.v[1]));
    out[0] = f.x;
    out[1] = f.y;
}

// ---------------------------------------------------------------------------------------------
// kernel parameters
// ---------------------------------------------------------------------------------------------
struct alignas(64) TensorDesc {
    CUtensorMap map;     // bulk-copy path
    void* ptr;           // guarded path
    long long stride_b;  // elements
    long long stride_l;  // elements
    long long reserved;
};

struct Geom {
    long long B, L, D;
    int n_dtiles;   // ceil(D / channels per warp)
    int n_seg;      // time segments
    int seg_rows;   // rows per segment, a multiple of the tile rows
    long long n_chains;  // B * n_seg * n_dtiles; CTAs take chains blockIdx.x, + gridDim.x, ...
    int n_stages;   // ring depth
    int use_tma;    // 0: guarded per-lane accesses
    int l2_hint;    // bit 0: loads evict-first, bit 1: stores evict-first
    int n_out;      // forward: output staging buffers in the ring (2..4)
    int* status;    // may be NULL
};

struct FwdParams {
    TensorDesc x, a, b, c, y, hs;
    float* tile_h;       // [B, ceil(L/TS), D] or NULL
    const float* h_in;   // [B, n_seg, D] or NULL
    float* h_last;       // [B, D] or NULL
    Geom g;
};

// Chained (single-pass) forward for launches with few chains: see scan_fwd_chained_kernel.
struct ChainedParams {
    FwdParams f;
    unsigned int* ticket;   // work counter, zero at launch
    float* desc;            // [n_chains][slots][3][32] float4 {tag, v0, v1, -}: aggregate A, aggregate H,
                            // inclusive end state; tag = chunk + 1, the whole area zero at launch
    int chunk_rows;         // rows per chunk, a multiple of TS
    int slots;              // descriptor slots per chain (power of two)
    int n_chunks;           // chunks per chain
    unsigned long long wait_ns;  // limit of a look-back wait
};

struct BwdParams;
struct ChainedBwdParams;

struct BwdParams {
    TensorDesc x, a, b, c, dy, hsrc;  // hsrc: tile_h (recompute) or h_saved
    TensorDesc dx, da, db, dc;
    const float* h_in;   // [B, D] or NULL (only read with h_saved, for da at t = 0)
    const float* g_in;   // [B, n_seg, D] or NULL
    float* g_first;      // [B, D] or NULL
    Geom g;
};

// Chained (single-pass) backward: see scan_bwd_chained_kernel.
struct ChainedBwdParams {
    BwdParams f;
    unsigned int* ticket;
    float* desc;
    int chunk_rows, slots, n_chunks;
    unsigned long long wait_ns;
};

struct AggParams {
    TensorDesc t0, t1, t2;  // forward: x, a, b; backward: a, c, dy
    float* A;               // [B, n_seg, D]
    float* H;               // [B, n_seg, D]
    Geom g;
};

__device__ __forceinline__ void report(int* status, int code) {
    if (status != nullptr) {
        *reinterpret_cast<volatile int*>(status) = code;
        __threadfence_system();
    }
}

// Guarded fill of `rows` rows starting at time t0 (this lane's V channels), zero padded.
template <typename T, int V>
__device__ __noinline__ void plain_fill(unsigned char* tile, const void* ptr, long long stride_b,
                                        long long stride_l, long long b, long long t0, int rows, long long t_lim,
                                        long long d_lane, long long D, int lane) {
    const T* base = reinterpret_cast<const T*>(ptr) + b * stride_b;
    for (int r = 0; r < rows; ++r) {
        Vec<T, V> w;
        const long long t = t0 + r;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const bool ok = (t >= 0) && (t < t_lim) && (d_lane + i < D);
            w.v[i] = ok ? base[t * stride_l + d_lane + i] : from_f<T>(0.f);
        }
        reinterpret_cast<Vec<T, V>*>(tile)[r * 32 + lane] = w;
    }
}
template <typename T, int V>
__device__ __forceinline__ void plain_fill(unsigned char* tile, const TensorDesc& td, long long b, long long t0,
                                           int rows, long long t_lim, long long d_lane, long long D, int lane) {
    plain_fill<T, V>(tile, td.ptr, td.stride_b, td.stride_l, b, t0, rows, t_lim, d_lane, D, lane);
}
// Guarded write-back of `rows` rows.
template <typename T, int V>
__device__ __noinline__ void plain_drain(const unsigned char* tile, void* ptr, long long stride_b,
                                         long long stride_l, long long b, long long t0, int rows, long long t_lim,
                                         long long d_lane, long long D, int lane) {
    T* base = reinterpret_cast<T*>(ptr) + b * stride_b;
    for (int r = 0; r < rows; ++r) {
        const Vec<T, V> w = reinterpret_cast<const Vec<T, V>*>(tile)[r * 32 + lane];
        const long long t = t0 + r;
#pragma unroll
        for (int i = 0; i < V; ++i)
            if (t < t_lim && d_lane + i < D) base[t * stride_l + d_lane + i] = w.v[i];
    }
}
template <typename T, int V>
__device__ __forceinline__ void plain_drain(const unsigned char* tile, const TensorDesc& td, long long b,
                                            long long t0, int rows, long long t_lim, long long d_lane, long long D,
                                            int lane) {
    plain_drain<T, V>(tile, td.ptr, td.stride_b, td.stride_l, b, t0, rows, t_lim, d_lane, D, lane);
}

// Chain coordinates of this warp.
struct Chain {
    long long b, d0, t_begin, t_end;
    int seg, n_tiles;
    bool empty;
};
__device__ __forceinline__ Chain chain_of(const Geom& g, long long id, int chans_per_warp, int tile_rows) {
    Chain c;
    const long long dt = id % g.n_dtiles;
    const long long rest = id / g.n_dtiles;
    c.seg = static_cast<int>(rest % g.n_seg);
    c.b = rest / g.n_seg;
    c.d0 = dt * chans_per_warp;
    c.t_begin = static_cast<long long>(c.seg) * g.seg_rows;
    c.t_end = c.t_begin + g.seg_rows;
    if (c.t_end > g.L) c.t_end = g.L;
    c.empty = c.t_begin >= c.t_end;
    c.n_tiles = c.empty ? 0 : static_cast<int>((c.t_end - c.t_begin + tile_rows - 1) / tile_rows);
    return c;
}

// Position in the ring of stages (stage index and barrier phase), advanced without divisions.
struct RingPos {
    int s;
    uint32_t phase;
    __device__ __forceinline__ void advance(int n_stages) {
        if (++s == n_stages) {
            s = 0;
            phase ^= 1u;
        }
    }
};

}  // namespace qssm
