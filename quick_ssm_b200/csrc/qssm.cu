// Gated linear scan for NVIDIA B200 (sm_100a):  h(t) = a(t) h(t-1) + b(t) x(t),  y(t) = c(t) h(t).
//
// Execution model
// ---------------
// The path is HBM-bound (about three fused multiply-adds per element, no
// contraction), so the kernels are built around keeping many bytes in flight
// with the bulk tensor copy engine (TMA) and touching every tensor once:
//
//  * one warp owns one "chain": a column strip of one batch entry (32 lanes x
//    V channels, V = 1 or 2) over a range of time steps, and walks it
//    sequentially in tiles of TB rows (TB = 16 or 32);
//  * lane 0 issues cp.async.bulk.tensor loads of the next tiles of every input
//    into a ring of shared-memory stages (completion on an mbarrier per
//    stage); the warp scans the current tile out of shared memory, 16 rows at
//    a time, with fp32 state in registers, writes results back to shared
//    memory and lane 0 issues the bulk tensor store.  One CTA == one warp, so
//    no CTA-wide barrier exists anywhere; many small CTAs per SM give the
//    latency hiding;
//  * the carry between tiles of a chain never leaves registers.  When B*D
//    alone gives too few chains to fill the GPU the time axis is cut into
//    segments: an aggregate kernel (reads only the tensors the carry depends
//    on) produces (prod a, local end state) per segment, a tiny kernel scans
//    those per channel, and the main kernel runs every segment seeded.  The
//    same aggregate/seed pair is what sequence shards on different GPUs
//    exchange.
//  * shapes the copy engine cannot address (row pitch or base not a multiple
//    of 16 bytes, e.g. D = 1) take the same kernels with guarded per-lane
//    loads and stores instead of bulk copies.
//
// Every wait on an mbarrier is bounded; on expiry the kernel records
// QSSM_S_TMA_TIMEOUT in the caller's status word and leaves.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <type_traits>

#include "../../include/qssm.h"

namespace {

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
// PTX wrappers: mbarrier, bulk tensor copies
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: gives up after about two seconds.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity) {
    const unsigned long long t0 = global_timer_ns();
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 16) __nanosleep(32);
        if ((it & 1023u) == 1023u && global_timer_ns() - t0 > 2000000000ull) return false;
        if (it > (1u << 28)) return false;
    }
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity);
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(src), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
// Same copies with an L2 eviction-priority hint (policy from createpolicy).
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                                 int c2, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4, %5}], [%2], %6;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "l"(pol)
        : "memory");
}
__device__ __forceinline__ void tma_store_3d_hint(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2,
                                                  uint64_t pol) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3, %4}], [%1], %5;" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(src), "r"(c0), "r"(c1), "r"(c2), "l"(pol)
                 : "memory");
}
__device__ __forceinline__ void tma_ld(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                       bool hint, uint64_t pol) {
    if (hint)
        tma_load_3d_hint(dst, map, bar, c0, c1, c2, pol);
    else
        tma_load_3d(dst, map, bar, c0, c1, c2);
}
__device__ __forceinline__ void tma_st(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, bool hint,
                                       uint64_t pol) {
    if (hint)
        tma_store_3d_hint(map, src, c0, c1, c2, pol);
    else
        tma_store_3d(map, src, c0, c1, c2);
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void tma_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void tma_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

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

// ---------------------------------------------------------------------------------------------
// forward:  y = c*h (HAS_C) or y = h; optional fp32 h, optional tile boundary states
// ---------------------------------------------------------------------------------------------
template <typename Tin, typename Tout, int V, bool HAS_C, bool SAVE_H, bool FULL>
__device__ __forceinline__ void fwd_batch(const unsigned char* sx, const unsigned char* sa, const unsigned char* sb,
                                          const unsigned char* sc, unsigned char* oy, unsigned char* oh, int lane,
                                          int nrows, float (&h)[V]) {
    Vec<Tin, V> xw[TS], aw[TS], bw[TS], cw[HAS_C ? TS : 1];
#pragma unroll
    for (int r = 0; r < TS; ++r) {
        xw[r] = tile_raw<Tin, V>(sx, r, lane);
        aw[r] = tile_raw<Tin, V>(sa, r, lane);
        bw[r] = tile_raw<Tin, V>(sb, r, lane);
        if (HAS_C) cw[r] = tile_raw<Tin, V>(sc, r, lane);
    }
    Vec<Tout, V> yw[TS];
    Vec<float, V> hw[SAVE_H ? TS : 1];
#pragma unroll
    for (int r = 0; r < TS; ++r) {
        float xv[V], av[V], bv[V], yv[V];
        unpack<Tin, V>(xw[r], xv);
        unpack<Tin, V>(aw[r], av);
        unpack<Tin, V>(bw[r], bv);
        if (FULL || r < nrows) {
#pragma unroll
            for (int i = 0; i < V; ++i) h[i] = fmaf(av[i], h[i], bv[i] * xv[i]);
        }
        if (HAS_C) {
            float cv[V];
            unpack<Tin, V>(cw[r], cv);
#pragma unroll
            for (int i = 0; i < V; ++i) yv[i] = cv[i] * h[i];
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) yv[i] = h[i];
        }
        yw[r] = pack<Tout, V>(yv);
        if (SAVE_H) hw[r] = pack<float, V>(h);
    }
#pragma unroll
    for (int r = 0; r < TS; ++r) {
        tile_put<Tout, V>(oy, r, lane, yw[r]);
        if (SAVE_H) tile_put<float, V>(oh, r, lane, hw[r]);
    }
}

template <typename Tin, typename Tout, int V, int TB, bool HAS_C, bool SAVE_H>
__global__ void __launch_bounds__(32) scan_fwd_kernel(const __grid_constant__ FwdParams p) {
    constexpr int DT = 32 * V;
    constexpr int NSUB = TB / TS;
    constexpr int NIN = HAS_C ? 4 : 3;
    constexpr int IN_ROW = 32 * V * (int)sizeof(Tin);
    constexpr int OUT_ROW = 32 * V * (int)sizeof(Tout);
    constexpr int H_ROW = 32 * V * 4;
    constexpr int IN_TILE = TB * IN_ROW;
    constexpr int OUT_TILE = TB * OUT_ROW;
    constexpr int HS_TILE = SAVE_H ? TB * H_ROW : 0;
    constexpr int STAGE = NIN * IN_TILE;
    constexpr int OUTBUF = OUT_TILE + HS_TILE;

    extern __shared__ __align__(128) unsigned char smem[];
    const Geom& g = p.g;
    const int NS = g.n_stages;
    unsigned char* const outbuf = smem + NS * STAGE;
    const int NOUT = g.n_out;
    const uint32_t bars = smem_u32(outbuf + NOUT * OUTBUF);
    const uint32_t smem_base = smem_u32(smem);

    const int lane = threadIdx.x;
    const bool tma = g.use_tma != 0;
    const bool ld_hint = (g.l2_hint & 1) != 0, st_hint = (g.l2_hint & 2) != 0;
    const uint64_t pol = l2_policy_evict_first();

    if (tma) {
        if (lane == 0) {
            for (int s = 0; s < NS; ++s) mbar_init(bars + 8 * s, 1);
            fence_barrier_init();
        }
        __syncwarp();
    }

    bool ok = true;
    RingPos pf{0, 0};   // next stage to fill
    RingPos cur{0, 0};  // stage being scanned
    // A CTA walks chains blockIdx.x, blockIdx.x + gridDim.x, ...: the grid bounds how many chains
    // stream at once, independently of how many there are.
    for (long long chain_id = blockIdx.x; chain_id < g.n_chains; chain_id += gridDim.x) {
    const Chain ch = chain_of(g, chain_id, DT, TB);
    if (ch.empty) continue;
    const long long d_lane = ch.d0 + (long long)lane * V;

    float h[V];
#pragma unroll
    for (int i = 0; i < V; ++i) h[i] = 0.f;
    if (p.h_in != nullptr) {
        const float* src = p.h_in + (ch.b * g.n_seg + ch.seg) * g.D;
#pragma unroll
        for (int i = 0; i < V; ++i)
            if (d_lane + i < g.D) h[i] = src[d_lane + i];
    }
    float* th_dst = nullptr;  // tile_h row of the next 16-row batch, this lane's channels
    if (p.tile_h != nullptr) th_dst = p.tile_h + (ch.b * ((g.L + TS - 1) / TS) + ch.t_begin / TS) * g.D + d_lane;

    const int c0 = (int)ch.d0, c2 = (int)ch.b;
    int pf_row = (int)ch.t_begin;
    int pf_left = ch.n_tiles;
    auto issue = [&]() {  // lane 0 only: loads of the next tile into stage pf.s
        const uint32_t st = smem_base + pf.s * STAGE;
        const uint32_t bar = bars + 8 * pf.s;
        fence_proxy_async();
        mbar_expect_tx(bar, STAGE);
        tma_ld(st + 0 * IN_TILE, &p.x.map, bar, c0, pf_row, c2, ld_hint, pol);
        tma_ld(st + 1 * IN_TILE, &p.a.map, bar, c0, pf_row, c2, ld_hint, pol);
        tma_ld(st + 2 * IN_TILE, &p.b.map, bar, c0, pf_row, c2, ld_hint, pol);
        if (HAS_C) tma_ld(st + 3 * IN_TILE, &p.c.map, bar, c0, pf_row, c2, ld_hint, pol);
        pf.advance(NS);
        pf_row += TB;
        --pf_left;
    };

    if (tma && lane == 0) {
        for (int k = 0; k < NS - 1 && pf_left > 0; ++k) issue();
    }

    long long t0 = ch.t_begin;
    int oslot = 0;
    for (int j = 0; j < ch.n_tiles; ++j, t0 += TB) {
        unsigned char* st = smem + cur.s * STAGE;
        unsigned char* ob = outbuf + oslot * OUTBUF;
        if (++oslot == NOUT) oslot = 0;
        const int nrows = (int)((ch.t_end - t0) < TB ? (ch.t_end - t0) : TB);

        if (tma) {
            if (lane == 0) {
                if (pf_left > 0) issue();
                // the store issued NOUT tiles ago has finished reading `ob`
                if (NOUT == 2) tma_wait_read<1>();
                else if (NOUT == 3) tma_wait_read<2>();
                else tma_wait_read<3>();
            }
            ok = mbar_wait_bounded(bars + 8 * cur.s, cur.phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
        } else {
            plain_fill<Tin, V>(st + 0 * IN_TILE, p.x, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            plain_fill<Tin, V>(st + 1 * IN_TILE, p.a, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            plain_fill<Tin, V>(st + 2 * IN_TILE, p.b, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            if (HAS_C) plain_fill<Tin, V>(st + 3 * IN_TILE, p.c, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
        }

#pragma unroll
        for (int sub = 0; sub < NSUB; ++sub) {
            const int left = nrows - sub * TS;
            if (left > 0) {
                if (th_dst != nullptr) {
#pragma unroll
                    for (int i = 0; i < V; ++i)
                        if (d_lane + i < g.D) th_dst[i] = h[i];
                    th_dst += g.D;
                }
                const unsigned char* sx = st + 0 * IN_TILE + sub * TS * IN_ROW;
                const unsigned char* sa = st + 1 * IN_TILE + sub * TS * IN_ROW;
                const unsigned char* sb = st + 2 * IN_TILE + sub * TS * IN_ROW;
                const unsigned char* sc = st + 3 * IN_TILE + sub * TS * IN_ROW;
                unsigned char* oy = ob + sub * TS * OUT_ROW;
                unsigned char* oh = ob + OUT_TILE + sub * TS * H_ROW;
                if (left >= TS)
                    fwd_batch<Tin, Tout, V, HAS_C, SAVE_H, true>(sx, sa, sb, sc, oy, oh, lane, TS, h);
                else
                    fwd_batch<Tin, Tout, V, HAS_C, SAVE_H, false>(sx, sa, sb, sc, oy, oh, lane, left, h);
            }
        }

        if (tma) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_st(&p.y.map, smem_u32(ob), c0, (int)t0, c2, st_hint, pol);
                if (SAVE_H) tma_st(&p.hs.map, smem_u32(ob + OUT_TILE), c0, (int)t0, c2, st_hint, pol);
                tma_commit();
            }
        } else {
            plain_drain<Tout, V>(ob, p.y, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            if (SAVE_H) plain_drain<float, V>(ob + OUT_TILE, p.hs, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
        }
        __syncwarp();
        cur.advance(NS);
    }

    if (!ok) break;
    if (p.h_last != nullptr && ch.seg == g.n_seg - 1) {
        float* dst = p.h_last + ch.b * g.D;
#pragma unroll
        for (int i = 0; i < V; ++i)
            if (d_lane + i < g.D) dst[d_lane + i] = h[i];
    }
    if (tma) {  // the stores of this chain have read their buffers before the next chain reuses them
        if (lane == 0) tma_wait_read<0>();
        __syncwarp();
    }
    }  // chains

    if (tma && lane == 0) tma_wait_all();
    if (!ok && lane == 0) report(g.status, QSSM_S_TMA_TIMEOUT);
}

// ---------------------------------------------------------------------------------------------
// Look-back over the chunk descriptors of one chain (chained kernels).
//
// Descriptor of chunk j (slot j mod slots): three arrays of 32 float4, one word per lane,
//   [0..31] {tag, A0, A1, -}   [32..63] {tag, H0, H1, -}   [64..95] {tag, e0, e1, -}
// with tag = j + 1 (zero = nothing yet); (A, H) is the chunk aggregate, e its inclusive end state.
// A 16-byte word is written and read with one access, so a word whose tag matches carries its
// values and no separate flag or fence is needed.
//
// Returns in `h` the state entering chunk k: the inclusive end state of the nearest predecessor
// that has one, pushed through the aggregates of the chunks between it and k ONE BY ONE in time
// order, h = fma(A_m, h, H_m) - the same expression each of those chunks evaluates for its own
// end state.  The result is therefore bit-identical whichever predecessors happened to be
// finished when the warp looked: the kernels stay deterministic although chunks run concurrently.
// Waits are bounded (about two seconds); false means a predecessor never published.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ bool chained_lookback(const float4* cdesc, int slots, long long k, int lane,
                                                 float (&h)[2]) {
    constexpr int WIN = 8;
    bool ok = true;
    long long js = -1;  // nearest predecessor whose inclusive end state is known
    for (long long top = k - 1; js < 0 && ok; top -= WIN) {
        float4 wi[WIN], wa[WIN], wh[WIN];
#pragma unroll
        for (int q = 0; q < WIN; ++q) {
            const long long j = top - q;
            if (j >= 0) {
                const float4* dj = cdesc + (size_t)(j & (slots - 1)) * 96;
                wi[q] = __ldcg(dj + 64 + lane);
                wa[q] = __ldcg(dj + lane);
                wh[q] = __ldcg(dj + 32 + lane);
            }
        }
#pragma unroll
        for (int q = 0; q < WIN; ++q) {
            const long long j = top - q;
            if (j < 0 || js >= 0 || !ok) continue;
            const unsigned int want = (unsigned int)(j + 1);
            const float4* dj = cdesc + (size_t)(j & (slots - 1)) * 96;
            bool inc = __all_sync(0xffffffffu, __float_as_uint(wi[q].x) == want);
            bool agg = __all_sync(0xffffffffu, __float_as_uint(wa[q].x) == want && __float_as_uint(wh[q].x) == want);
            if (!inc && !agg) {  // nothing published yet: poll this chunk
                const unsigned long long start = global_timer_ns();
                for (unsigned int it = 0; ok; ++it) {
                    wi[q] = __ldcg(dj + 64 + lane);
                    wa[q] = __ldcg(dj + lane);
                    wh[q] = __ldcg(dj + 32 + lane);
                    inc = __all_sync(0xffffffffu, __float_as_uint(wi[q].x) == want);
                    agg = __all_sync(0xffffffffu,
                                     __float_as_uint(wa[q].x) == want && __float_as_uint(wh[q].x) == want);
                    if (inc || agg) break;
                    __nanosleep(100);
                    if ((it & 255u) == 255u) {
                        const bool late = global_timer_ns() - start > 2000000000ull;
                        if (__any_sync(0xffffffffu, late)) ok = false;
                    }
                }
            }
            if (ok && inc) {
                h[0] = wi[q].y;
                h[1] = wi[q].z;
                js = j;
            }
        }
    }
    if (!ok) return false;
    // forward through the aggregates of chunks js+1 .. k-1 (all seen published above)
    for (long long base = js + 1; base < k; base += WIN) {
        float4 wa[WIN], wh[WIN];
#pragma unroll
        for (int q = 0; q < WIN; ++q) {
            const long long j = base + q;
            if (j < k) {
                const float4* dj = cdesc + (size_t)(j & (slots - 1)) * 96;
                wa[q] = __ldcg(dj + lane);
                wh[q] = __ldcg(dj + 32 + lane);
            }
        }
#pragma unroll
        for (int q = 0; q < WIN; ++q) {
            if (base + q < k) {
                h[0] = fmaf(wa[q].y, h[0], wh[q].y);
                h[1] = fmaf(wa[q].z, h[1], wh[q].z);
            }
        }
    }
    return true;
}

// ---------------------------------------------------------------------------------------------
// chained forward: one pass over HBM when batch x channels gives too few chains to fill the GPU.
//
// Each chain (full time range of one strip) is cut into chunks of `chunk_rows` rows.  Warps take
// chunks from a global ticket counter in time-major order (chunk k of every chain before chunk
// k+1 of any), so many chunks of the same chain are in progress at once.  Per chunk a warp
//   1. streams x, a, b and reduces them to the chunk aggregate (A, H) = (prod a, end state from 0),
//   2. publishes the aggregate, looks back over the preceding chunks' descriptors - folding
//      aggregates until it meets a chunk whose inclusive end state is known - to get its h_in,
//      and publishes its own inclusive end state A*h_in + H,
//   3. streams the chunk a second time (x, a, b now come from L2, where step 1 left them; only c
//      comes from HBM) and writes y.
// HBM traffic is therefore the minimum (each tensor once) as long as the chunks in flight fit L2.
// Forward progress: a warp waits only on chunks with smaller tickets, all of which are held by
// warps that are already running; every wait is bounded and a failure makes all warps leave.
// ---------------------------------------------------------------------------------------------
template <typename Tin, typename Tout, bool HAS_C>
__global__ void __launch_bounds__(32) scan_fwd_chained_kernel(const __grid_constant__ ChainedParams cp) {
    constexpr int V = 2;
    constexpr int DT = 32 * V;
    constexpr int TB = TS;
    constexpr int IN_ROW = 32 * V * (int)sizeof(Tin);
    constexpr int OUT_ROW = 32 * V * (int)sizeof(Tout);
    constexpr int IN_TILE = TB * IN_ROW;
    constexpr int OUT_TILE = TB * OUT_ROW;
    constexpr int STAGE = 4 * IN_TILE;

    extern __shared__ __align__(128) unsigned char smem[];
    const FwdParams& p = cp.f;
    const Geom& g = p.g;
    const int NS = g.n_stages;
    const int NOUT = g.n_out;
    unsigned char* const outbuf = smem + NS * STAGE;
    const uint32_t bars = smem_u32(outbuf + NOUT * OUT_TILE);
    const uint32_t smem_base = smem_u32(smem);
    const int lane = threadIdx.x;
    const uint64_t pol_keep = l2_policy_evict_last();
    const uint64_t pol_drop = l2_policy_evict_first();
    const bool hint = g.l2_hint != 0;

    if (lane == 0) {
        for (int s = 0; s < NS; ++s) mbar_init(bars + 8 * s, 1);
        fence_barrier_init();
    }
    __syncwarp();

    const long long n_chains = g.B * g.n_dtiles;
    const unsigned int total = (unsigned int)(n_chains * cp.n_chunks);
    const long long tiles_per_b = (g.L + TS - 1) / TS;
    RingPos pf{0, 0}, cur{0, 0};
    int oslot = 0;
    bool ok = true;

    while (ok) {
        unsigned int t = 0;
        if (lane == 0) t = atomicAdd(cp.ticket, 1u);
        t = __shfl_sync(0xffffffffu, t, 0);
        if (t >= total) break;
        const long long k = t / n_chains;        // chunk index in time
        const long long c = t % n_chains;        // chain
        const long long b = c / g.n_dtiles;
        const long long d0 = (c % g.n_dtiles) * DT;
        const long long d_lane = d0 + (long long)lane * V;
        const long long t_begin = k * cp.chunk_rows;
        long long t_end = t_begin + cp.chunk_rows;
        if (t_end > g.L) t_end = g.L;
        const int n_tiles = (int)((t_end - t_begin + TB - 1) / TB);
        const int c0 = (int)d0, c2 = (int)b;

        // the tile stream of this chunk: n_tiles tiles of pass 1 (x, a, b), then n_tiles of pass 2 (x, a, b, c)
        int pf_item = 0;
        const int n_items = 2 * n_tiles;
        auto issue = [&]() {  // lane 0 only
            const bool second = pf_item >= n_tiles;
            const int row = (int)(t_begin + (long long)(second ? pf_item - n_tiles : pf_item) * TB);
            const uint32_t st = smem_base + pf.s * STAGE;
            const uint32_t bar = bars + 8 * pf.s;
            const uint64_t pol = second ? pol_drop : pol_keep;
            fence_proxy_async();
            mbar_expect_tx(bar, (second && HAS_C) ? 4 * IN_TILE : 3 * IN_TILE);
            tma_ld(st + 0 * IN_TILE, &p.x.map, bar, c0, row, c2, hint, pol);
            tma_ld(st + 1 * IN_TILE, &p.a.map, bar, c0, row, c2, hint, pol);
            tma_ld(st + 2 * IN_TILE, &p.b.map, bar, c0, row, c2, hint, pol);
            if (second && HAS_C) tma_ld(st + 3 * IN_TILE, &p.c.map, bar, c0, row, c2, hint, pol_drop);
            pf.advance(NS);
            ++pf_item;
        };
        if (lane == 0) {
            for (int q = 0; q < NS - 1 && pf_item < n_items; ++q) issue();
        }

        // ---- pass 1: chunk aggregate ----
        float A[V], H[V];
#pragma unroll
        for (int i = 0; i < V; ++i) { A[i] = 1.f; H[i] = 0.f; }
        long long t0 = t_begin;
        for (int j = 0; j < n_tiles && ok; ++j, t0 += TB) {
            const unsigned char* st = smem + cur.s * STAGE;
            const int nrows = (int)((t_end - t0) < TB ? (t_end - t0) : TB);
            if (lane == 0 && pf_item < n_items) issue();
            ok = mbar_wait_bounded(bars + 8 * cur.s, cur.phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
#pragma unroll
            for (int r = 0; r < TB; ++r) {
                float xv[V], av[V], bv[V];
                unpack<Tin, V>(tile_raw<Tin, V>(st + 0 * IN_TILE, r, lane), xv);
                unpack<Tin, V>(tile_raw<Tin, V>(st + 1 * IN_TILE, r, lane), av);
                unpack<Tin, V>(tile_raw<Tin, V>(st + 2 * IN_TILE, r, lane), bv);
                if (r < nrows) {
#pragma unroll
                    for (int i = 0; i < V; ++i) { A[i] *= av[i]; H[i] = fmaf(av[i], H[i], bv[i] * xv[i]); }
                }
            }
            __syncwarp();
            cur.advance(NS);
        }
        if (!ok) break;

        // ---- carry: publish aggregate, look back, publish inclusive end state ----
        float4* const cdesc = reinterpret_cast<float4*>(cp.desc) + (size_t)c * cp.slots * 96;
        float4* const mydesc = cdesc + (size_t)(k & (cp.slots - 1)) * 96;
        const float mytag = __uint_as_float((unsigned int)(k + 1));
        float h[V];
        if (k == 0) {
#pragma unroll
            for (int i = 0; i < V; ++i)
                h[i] = (p.h_in != nullptr && d_lane + i < g.D) ? p.h_in[b * g.D + d_lane + i] : 0.f;
        } else {
            __stcg(mydesc + lane, make_float4(mytag, A[0], A[1], 0.f));
            __stcg(mydesc + 32 + lane, make_float4(mytag, H[0], H[1], 0.f));
            ok = chained_lookback(cdesc, cp.slots, k, lane, h);
            if (!ok) break;
        }
        {   // inclusive end state of this chunk
            const float e0 = fmaf(A[0], h[0], H[0]), e1 = fmaf(A[1], h[1], H[1]);
            __stcg(mydesc + 64 + lane, make_float4(mytag, e0, e1, 0.f));
            if (p.h_last != nullptr && k == cp.n_chunks - 1) {
                if (d_lane < g.D) p.h_last[b * g.D + d_lane] = e0;
                if (d_lane + 1 < g.D) p.h_last[b * g.D + d_lane + 1] = e1;
            }
        }

        // ---- pass 2: the scan proper, seeded ----
        float* th_dst = nullptr;
        if (p.tile_h != nullptr) th_dst = p.tile_h + (b * tiles_per_b + t_begin / TS) * g.D + d_lane;
        t0 = t_begin;
        for (int j = 0; j < n_tiles; ++j, t0 += TB) {
            const unsigned char* st = smem + cur.s * STAGE;
            unsigned char* ob = outbuf + oslot * OUT_TILE;
            if (++oslot == NOUT) oslot = 0;
            const int nrows = (int)((t_end - t0) < TB ? (t_end - t0) : TB);
            if (lane == 0) {
                if (pf_item < n_items) issue();
                if (NOUT == 2) tma_wait_read<1>();
                else if (NOUT == 3) tma_wait_read<2>();
                else tma_wait_read<3>();
            }
            ok = mbar_wait_bounded(bars + 8 * cur.s, cur.phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (th_dst != nullptr) {
#pragma unroll
                for (int i = 0; i < V; ++i)
                    if (d_lane + i < g.D) th_dst[i] = h[i];
                th_dst += g.D;
            }
            if (nrows >= TS)
                fwd_batch<Tin, Tout, V, HAS_C, false, true>(st, st + IN_TILE, st + 2 * IN_TILE, st + 3 * IN_TILE, ob,
                                                            ob, lane, TS, h);
            else
                fwd_batch<Tin, Tout, V, HAS_C, false, false>(st, st + IN_TILE, st + 2 * IN_TILE, st + 3 * IN_TILE, ob,
                                                             ob, lane, nrows, h);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_st(&p.y.map, smem_u32(ob), c0, (int)t0, c2, hint, pol_drop);
                tma_commit();
            }
            __syncwarp();
            cur.advance(NS);
        }
    }
    if (lane == 0) {
        tma_wait_all();
        if (!ok) report(g.status, QSSM_S_TMA_TIMEOUT);
    }
}

// ---------------------------------------------------------------------------------------------
// backward: reverse scan of dh with h rebuilt per 16-row batch (tile_h) or read (h_saved).
// The carry between batches is G(t) = a(t) * dh(t), so no halo row of `a` is needed.
// Gradients overwrite the shared-memory slots of x, a, b, c and are stored from there.
// ---------------------------------------------------------------------------------------------
// Results go to (ox, oa, ob, oc), tiles whose rows hold OSTRIDE lane-vectors; `ocol` is this warp's first
// column in such a row.  In-place operation passes the input tiles again with OSTRIDE = 32, ocol = 0.
template <typename Tin, typename Tdy, int V, bool SAVED_H, bool FULL, int OSTRIDE = 32>
__device__ __forceinline__ void bwd_batch(const unsigned char* sx, const unsigned char* sa, const unsigned char* sb,
                                          const unsigned char* sc, const unsigned char* sg, const unsigned char* sh,
                                          unsigned char* ox, unsigned char* oa, unsigned char* ob, unsigned char* oc,
                                          int ocol, int lane, int nrows, bool first_rows, const float* h_in_lane,
                                          long long d_lane, long long D, float (&G)[V]) {
    Vec<Tin, V> xw[TS], aw[TS], bw[TS], cw[TS];
    Vec<Tdy, V> gw[TS];
#pragma unroll
    for (int r = 0; r < TS; ++r) {
        xw[r] = tile_raw<Tin, V>(sx, r, lane);
        aw[r] = tile_raw<Tin, V>(sa, r, lane);
        bw[r] = tile_raw<Tin, V>(sb, r, lane);
    }
    // h(t0-1 .. t0+TS-1): entry 0 is the state before the batch
    float hreg[TS + 1][V];
    if (SAVED_H) {
#pragma unroll
        for (int r = 0; r <= TS; ++r) {
            const Vec<float, V> w = tile_raw<float, V>(sh, r, lane);
            unpack<float, V>(w, hreg[r]);
        }
        if (first_rows && h_in_lane != nullptr) {
#pragma unroll
            for (int i = 0; i < V; ++i) hreg[0][i] = (d_lane + i < D) ? h_in_lane[i] : 0.f;
        }
    } else {
        const Vec<float, V> w = tile_raw<float, V>(sh, 0, lane);
        unpack<float, V>(w, hreg[0]);
    }
#pragma unroll
    for (int r = 0; r < TS; ++r) {
        cw[r] = tile_raw<Tin, V>(sc, r, lane);
        gw[r] = tile_raw<Tdy, V>(sg, r, lane);
    }
    if (!SAVED_H) {
#pragma unroll
        for (int r = 0; r < TS; ++r) {
            float xv[V], av[V], bv[V];
            unpack<Tin, V>(xw[r], xv);
            unpack<Tin, V>(aw[r], av);
            unpack<Tin, V>(bw[r], bv);
#pragma unroll
            for (int i = 0; i < V; ++i) hreg[r + 1][i] = fmaf(av[i], hreg[r][i], bv[i] * xv[i]);
        }
    }
#pragma unroll
    for (int r = TS - 1; r >= 0; --r) {
        float xv[V], av[V], bv[V], cv[V], gy[V];
        unpack<Tin, V>(xw[r], xv);
        unpack<Tin, V>(aw[r], av);
        unpack<Tin, V>(bw[r], bv);
        unpack<Tin, V>(cw[r], cv);
        unpack<Tdy, V>(gw[r], gy);
        float dxv[V], dav[V], dbv[V], dcv[V];
        const bool live = FULL || r < nrows;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const float dh = fmaf(cv[i], gy[i], G[i]);
            dxv[i] = dh * bv[i];
            dbv[i] = dh * xv[i];
            dav[i] = dh * hreg[r][i];
            dcv[i] = gy[i] * hreg[r + 1][i];
            if (live) G[i] = av[i] * dh;
        }
        // reuse the input words for the gradients: x -> dx, a -> da, b -> db, c -> dc
        xw[r] = pack<Tin, V>(dxv);
        aw[r] = pack<Tin, V>(dav);
        bw[r] = pack<Tin, V>(dbv);
        cw[r] = pack<Tin, V>(dcv);
    }
#pragma unroll
    for (int r = 0; r < TS; ++r) {
        reinterpret_cast<Vec<Tin, V>*>(ox)[r * OSTRIDE + ocol + lane] = xw[r];
        reinterpret_cast<Vec<Tin, V>*>(oa)[r * OSTRIDE + ocol + lane] = aw[r];
        reinterpret_cast<Vec<Tin, V>*>(ob)[r * OSTRIDE + ocol + lane] = bw[r];
        reinterpret_cast<Vec<Tin, V>*>(oc)[r * OSTRIDE + ocol + lane] = cw[r];
    }
}

template <typename Tin, typename Tdy, int V, int TB, bool SAVED_H>
__global__ void __launch_bounds__(32) scan_bwd_kernel(const __grid_constant__ BwdParams p) {
    constexpr int DT = 32 * V;
    constexpr int NSUB = TB / TS;
    constexpr int IN_ROW = 32 * V * (int)sizeof(Tin);
    constexpr int DY_ROW = 32 * V * (int)sizeof(Tdy);
    constexpr int H_ROW = 32 * V * 4;
    constexpr int IN_TILE = TB * IN_ROW;
    constexpr int DY_TILE = TB * DY_ROW;
    constexpr int H_TILE = SAVED_H ? (TB + 1) * H_ROW : NSUB * H_ROW;  // rows t0-1 .. t0+TB-1, or boundary rows
    constexpr int H_SLOT = ((H_TILE + 127) / 128) * 128;
    constexpr int STAGE = 4 * IN_TILE + DY_TILE + H_SLOT;
    constexpr int OFF_DY = 4 * IN_TILE;
    constexpr int OFF_H = OFF_DY + DY_TILE;

    extern __shared__ __align__(128) unsigned char smem[];
    const Geom& g = p.g;
    const int NS = g.n_stages;
    const uint32_t bars = smem_u32(smem + NS * STAGE);
    const uint32_t smem_base = smem_u32(smem);

    const int lane = threadIdx.x;
    const bool tma = g.use_tma != 0;
    const bool ld_hint = (g.l2_hint & 1) != 0, st_hint = (g.l2_hint & 2) != 0;
    const uint64_t pol = l2_policy_evict_first();
    const long long tiles_per_b = (g.L + TS - 1) / TS;

    if (tma) {
        if (lane == 0) {
            for (int s = 0; s < NS; ++s) mbar_init(bars + 8 * s, 1);
            fence_barrier_init();
        }
        __syncwarp();
    }

    bool ok = true;
    RingPos pf{0, 0};
    RingPos cur{0, 0};
    for (long long chain_id = blockIdx.x; chain_id < g.n_chains; chain_id += gridDim.x) {
    const Chain ch = chain_of(g, chain_id, DT, TB);
    if (ch.empty) continue;
    const long long d_lane = ch.d0 + (long long)lane * V;

    float G[V];
#pragma unroll
    for (int i = 0; i < V; ++i) G[i] = 0.f;
    if (p.g_in != nullptr) {
        const float* src = p.g_in + (ch.b * g.n_seg + ch.seg) * g.D;
#pragma unroll
        for (int i = 0; i < V; ++i)
            if (d_lane + i < g.D) G[i] = src[d_lane + i];
    }
    const float* h_in_lane = (SAVED_H && p.h_in != nullptr) ? p.h_in + ch.b * g.D + d_lane : nullptr;

    const int c0 = (int)ch.d0, c2 = (int)ch.b;
    // tiles are walked from the last to the first
    int pf_row = (int)(ch.t_begin + (long long)(ch.n_tiles - 1) * TB);
    int pf_left = ch.n_tiles;
    auto issue = [&]() {
        const uint32_t st = smem_base + pf.s * STAGE;
        const uint32_t bar = bars + 8 * pf.s;
        fence_proxy_async();
        mbar_expect_tx(bar, 4 * IN_TILE + DY_TILE + H_TILE);
        tma_ld(st + 0 * IN_TILE, &p.x.map, bar, c0, pf_row, c2, ld_hint, pol);
        tma_ld(st + 1 * IN_TILE, &p.a.map, bar, c0, pf_row, c2, ld_hint, pol);
        tma_ld(st + 2 * IN_TILE, &p.b.map, bar, c0, pf_row, c2, ld_hint, pol);
        tma_ld(st + 3 * IN_TILE, &p.c.map, bar, c0, pf_row, c2, ld_hint, pol);
        tma_ld(st + OFF_DY, &p.dy.map, bar, c0, pf_row, c2, ld_hint, pol);
        if (SAVED_H)
            tma_ld(st + OFF_H, &p.hsrc.map, bar, c0, pf_row - 1, c2, ld_hint, pol);  // row -1 reads zero fill
        else
            tma_ld(st + OFF_H, &p.hsrc.map, bar, c0, pf_row / TS, c2, ld_hint, pol);
        pf.advance(NS);
        pf_row -= TB;
        --pf_left;
    };

    // Gradients are stored from the stage itself, so a stage can be refilled only after the store
    // issued from it has finished reading.  With three or more stages the tile fetched at step j
    // goes into the stage of tile j-2 (prefetch distance NS - 2, at most one store left pending);
    // with two stages it goes into the stage of tile j-1, whose store must have drained completely.
    const int PF = NS > 2 ? NS - 2 : 1;
    if (tma && lane == 0) {
        for (int k = 0; k < PF && pf_left > 0; ++k) issue();
    }

    long long t0 = ch.t_begin + (long long)(ch.n_tiles - 1) * TB;
    for (int j = 0; j < ch.n_tiles; ++j, t0 -= TB) {
        unsigned char* st = smem + cur.s * STAGE;
        const int nrows = (int)((ch.t_end - t0) < TB ? (ch.t_end - t0) : TB);

        if (tma) {
            if (lane == 0 && pf_left > 0) {
                if (NS > 2)
                    tma_wait_read<1>();  // the store of the tile before the previous one is done with its stage
                else
                    tma_wait_read<0>();
                issue();
            }
            ok = mbar_wait_bounded(bars + 8 * cur.s, cur.phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
        } else {
            plain_fill<Tin, V>(st + 0 * IN_TILE, p.x, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            plain_fill<Tin, V>(st + 1 * IN_TILE, p.a, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            plain_fill<Tin, V>(st + 2 * IN_TILE, p.b, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            plain_fill<Tin, V>(st + 3 * IN_TILE, p.c, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            plain_fill<Tdy, V>(st + OFF_DY, p.dy, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            if (SAVED_H)
                plain_fill<float, V>(st + OFF_H, p.hsrc, ch.b, t0 - 1, TB + 1, ch.t_end, d_lane, g.D, lane);
            else  // tile_h is [B, tiles_per_b, D]
                plain_fill<float, V>(st + OFF_H, p.hsrc.ptr, tiles_per_b * g.D, g.D, ch.b, t0 / TS, NSUB,
                                     tiles_per_b, d_lane, g.D, lane);
        }

#pragma unroll
        for (int sub = NSUB - 1; sub >= 0; --sub) {
            const int left = nrows - sub * TS;
            if (left > 0) {
                unsigned char* sx = st + 0 * IN_TILE + sub * TS * IN_ROW;
                unsigned char* sa = st + 1 * IN_TILE + sub * TS * IN_ROW;
                unsigned char* sb = st + 2 * IN_TILE + sub * TS * IN_ROW;
                unsigned char* sc = st + 3 * IN_TILE + sub * TS * IN_ROW;
                const unsigned char* sg = st + OFF_DY + sub * TS * DY_ROW;
                const unsigned char* sh = st + OFF_H + (SAVED_H ? sub * TS * H_ROW : sub * H_ROW);
                const bool first_rows = (t0 == 0 && sub == 0);
                if (left >= TS)
                    bwd_batch<Tin, Tdy, V, SAVED_H, true>(sx, sa, sb, sc, sg, sh, sx, sa, sb, sc, 0, lane, TS,
                                                          first_rows, h_in_lane, d_lane, g.D, G);
                else
                    bwd_batch<Tin, Tdy, V, SAVED_H, false>(sx, sa, sb, sc, sg, sh, sx, sa, sb, sc, 0, lane, left,
                                                           first_rows, h_in_lane, d_lane, g.D, G);
            }
        }

        if (tma) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                const uint32_t sst = smem_base + cur.s * STAGE;
                tma_st(&p.dx.map, sst + 0 * IN_TILE, c0, (int)t0, c2, st_hint, pol);
                tma_st(&p.da.map, sst + 1 * IN_TILE, c0, (int)t0, c2, st_hint, pol);
                tma_st(&p.db.map, sst + 2 * IN_TILE, c0, (int)t0, c2, st_hint, pol);
                tma_st(&p.dc.map, sst + 3 * IN_TILE, c0, (int)t0, c2, st_hint, pol);
                tma_commit();
            }
        } else {
            plain_drain<Tin, V>(st + 0 * IN_TILE, p.dx, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            plain_drain<Tin, V>(st + 1 * IN_TILE, p.da, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            plain_drain<Tin, V>(st + 2 * IN_TILE, p.db, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            plain_drain<Tin, V>(st + 3 * IN_TILE, p.dc, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
        }
        __syncwarp();
        cur.advance(NS);
    }

    if (!ok) break;
    if (p.g_first != nullptr && ch.seg == 0) {
        float* dst = p.g_first + ch.b * g.D;
#pragma unroll
        for (int i = 0; i < V; ++i)
            if (d_lane + i < g.D) dst[d_lane + i] = G[i];
    }
    if (tma) {  // the stores of this chain have read their stages before the next chain refills them
        if (lane == 0) tma_wait_read<0>();
        __syncwarp();
    }
    }  // chains

    if (tma && lane == 0) tma_wait_all();
    if (!ok && lane == 0) report(g.status, QSSM_S_TMA_TIMEOUT);
}

// ---------------------------------------------------------------------------------------------
// chained backward: the reverse-time twin of scan_fwd_chained_kernel.  Chunks are claimed from the
// last one to the first; per chunk: (1) a, c, dy -> aggregate (P, Q) = (prod a, a(t0) dh(t0) from a
// zero carry), (2) publish, look back over the chunks later in time, publish the inclusive carry,
// (3) second pass (a, c, dy now from L2; x, b, tile_h from HBM) with the real carry, gradients
// stored from the stage as in scan_bwd_kernel.  h is rebuilt from tile_h (checkpoint=True only).
// ---------------------------------------------------------------------------------------------
template <typename Tin, typename Tdy>
__global__ void __launch_bounds__(32) scan_bwd_chained_kernel(const __grid_constant__ ChainedBwdParams cp) {
    constexpr int V = 2;
    constexpr int DT = 32 * V;
    constexpr int TB = TS;
    constexpr int IN_ROW = 32 * V * (int)sizeof(Tin);
    constexpr int DY_ROW = 32 * V * (int)sizeof(Tdy);
    constexpr int H_ROW = 32 * V * 4;
    constexpr int IN_TILE = TB * IN_ROW;
    constexpr int DY_TILE = TB * DY_ROW;
    constexpr int H_SLOT = ((H_ROW + 127) / 128) * 128;
    constexpr int STAGE = 4 * IN_TILE + DY_TILE + H_SLOT;
    constexpr int OFF_DY = 4 * IN_TILE;
    constexpr int OFF_H = OFF_DY + DY_TILE;

    extern __shared__ __align__(128) unsigned char smem[];
    const BwdParams& p = cp.f;
    const Geom& g = p.g;
    const int NS = g.n_stages;
    const uint32_t bars = smem_u32(smem + NS * STAGE);
    const uint32_t smem_base = smem_u32(smem);
    const int lane = threadIdx.x;
    const uint64_t pol_keep = l2_policy_evict_last();
    const uint64_t pol_drop = l2_policy_evict_first();
    const bool hint = g.l2_hint != 0;

    if (lane == 0) {
        for (int s = 0; s < NS; ++s) mbar_init(bars + 8 * s, 1);
        fence_barrier_init();
    }
    __syncwarp();

    const long long n_chains = g.B * g.n_dtiles;
    const unsigned int total = (unsigned int)(n_chains * cp.n_chunks);
    RingPos pf{0, 0}, cur{0, 0};
    const int PF = NS > 2 ? NS - 2 : 1;
    bool ok = true;

    while (ok) {
        unsigned int t = 0;
        if (lane == 0) t = atomicAdd(cp.ticket, 1u);
        t = __shfl_sync(0xffffffffu, t, 0);
        if (t >= total) break;
        const long long kk = t / n_chains;             // position in processing order
        const long long k = cp.n_chunks - 1 - kk;      // chunk index in time
        const long long c = t % n_chains;
        const long long b = c / g.n_dtiles;
        const long long d0 = (c % g.n_dtiles) * DT;
        const long long d_lane = d0 + (long long)lane * V;
        const long long t_begin = k * cp.chunk_rows;
        long long t_end = t_begin + cp.chunk_rows;
        if (t_end > g.L) t_end = g.L;
        const int n_tiles = (int)((t_end - t_begin + TB - 1) / TB);
        const int c0 = (int)d0, c2 = (int)b;

        int pf_item = 0;
        const int n_items = 2 * n_tiles;
        auto issue = [&]() {  // lane 0 only; tiles of a pass run from the end of the chunk to its start
            const bool second = pf_item >= n_tiles;
            const int idx = second ? pf_item - n_tiles : pf_item;
            const int row = (int)(t_begin + (long long)(n_tiles - 1 - idx) * TB);
            const uint32_t st = smem_base + pf.s * STAGE;
            const uint32_t bar = bars + 8 * pf.s;
            fence_proxy_async();
            if (!second) {
                mbar_expect_tx(bar, 2 * IN_TILE + DY_TILE);
                tma_ld(st + 1 * IN_TILE, &p.a.map, bar, c0, row, c2, hint, pol_keep);
                tma_ld(st + 3 * IN_TILE, &p.c.map, bar, c0, row, c2, hint, pol_keep);
                tma_ld(st + OFF_DY, &p.dy.map, bar, c0, row, c2, hint, pol_keep);
            } else {
                mbar_expect_tx(bar, 4 * IN_TILE + DY_TILE + H_ROW);
                tma_ld(st + 0 * IN_TILE, &p.x.map, bar, c0, row, c2, hint, pol_drop);
                tma_ld(st + 1 * IN_TILE, &p.a.map, bar, c0, row, c2, hint, pol_drop);
                tma_ld(st + 2 * IN_TILE, &p.b.map, bar, c0, row, c2, hint, pol_drop);
                tma_ld(st + 3 * IN_TILE, &p.c.map, bar, c0, row, c2, hint, pol_drop);
                tma_ld(st + OFF_DY, &p.dy.map, bar, c0, row, c2, hint, pol_drop);
                tma_ld(st + OFF_H, &p.hsrc.map, bar, c0, row / TS, c2, hint, pol_drop);
            }
            pf.advance(NS);
            ++pf_item;
        };
        // a stage is refilled only when the gradient store issued from it (if any) has drained
        auto refill = [&]() {
            if (NS > 2) tma_wait_read<1>();
            else tma_wait_read<0>();
            issue();
        };
        if (lane == 0) {
            for (int q = 0; q < PF && pf_item < n_items; ++q) refill();
        }

        // ---- pass 1: chunk aggregate, rows from the end of the chunk to its start ----
        float P[V], Q[V];
#pragma unroll
        for (int i = 0; i < V; ++i) { P[i] = 1.f; Q[i] = 0.f; }
        long long t0 = t_begin + (long long)(n_tiles - 1) * TB;
        for (int j = 0; j < n_tiles; ++j, t0 -= TB) {
            const unsigned char* st = smem + cur.s * STAGE;
            const int nrows = (int)((t_end - t0) < TB ? (t_end - t0) : TB);
            if (lane == 0 && pf_item < n_items) refill();
            ok = mbar_wait_bounded(bars + 8 * cur.s, cur.phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
#pragma unroll
            for (int r = TB - 1; r >= 0; --r) {
                float av[V], cv[V], gy[V];
                unpack<Tin, V>(tile_raw<Tin, V>(st + 1 * IN_TILE, r, lane), av);
                unpack<Tin, V>(tile_raw<Tin, V>(st + 3 * IN_TILE, r, lane), cv);
                unpack<Tdy, V>(tile_raw<Tdy, V>(st + OFF_DY, r, lane), gy);
                if (r < nrows) {
#pragma unroll
                    for (int i = 0; i < V; ++i) { P[i] *= av[i]; Q[i] = av[i] * fmaf(cv[i], gy[i], Q[i]); }
                }
            }
            __syncwarp();
            cur.advance(NS);
        }
        if (!ok) break;

        // ---- carry: same descriptor protocol as the forward, in processing order kk ----
        float4* const cdesc = reinterpret_cast<float4*>(cp.desc) + (size_t)c * cp.slots * 96;
        float4* const mydesc = cdesc + (size_t)(kk & (cp.slots - 1)) * 96;
        const float mytag = __uint_as_float((unsigned int)(kk + 1));
        float G[V];
        if (kk == 0) {
#pragma unroll
            for (int i = 0; i < V; ++i)
                G[i] = (p.g_in != nullptr && d_lane + i < g.D) ? p.g_in[b * g.D + d_lane + i] : 0.f;
        } else {
            __stcg(mydesc + lane, make_float4(mytag, P[0], P[1], 0.f));
            __stcg(mydesc + 32 + lane, make_float4(mytag, Q[0], Q[1], 0.f));
            ok = chained_lookback(cdesc, cp.slots, kk, lane, G);
            if (!ok) break;
        }
        {
            const float e0 = fmaf(P[0], G[0], Q[0]), e1 = fmaf(P[1], G[1], Q[1]);
            __stcg(mydesc + 64 + lane, make_float4(mytag, e0, e1, 0.f));
            if (p.g_first != nullptr && k == 0) {
                if (d_lane < g.D) p.g_first[b * g.D + d_lane] = e0;
                if (d_lane + 1 < g.D) p.g_first[b * g.D + d_lane + 1] = e1;
            }
        }

        // ---- pass 2: gradients ----
        t0 = t_begin + (long long)(n_tiles - 1) * TB;
        for (int j = 0; j < n_tiles; ++j, t0 -= TB) {
            unsigned char* st = smem + cur.s * STAGE;
            const int nrows = (int)((t_end - t0) < TB ? (t_end - t0) : TB);
            if (lane == 0 && pf_item < n_items) refill();
            ok = mbar_wait_bounded(bars + 8 * cur.s, cur.phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            unsigned char* sx = st;
            unsigned char* sa = st + IN_TILE;
            unsigned char* sb = st + 2 * IN_TILE;
            unsigned char* sc = st + 3 * IN_TILE;
            if (nrows >= TS)
                bwd_batch<Tin, Tdy, V, false, true>(sx, sa, sb, sc, st + OFF_DY, st + OFF_H, sx, sa, sb, sc, 0, lane, TS,
                                                    false, nullptr, d_lane, g.D, G);
            else
                bwd_batch<Tin, Tdy, V, false, false>(sx, sa, sb, sc, st + OFF_DY, st + OFF_H, sx, sa, sb, sc, 0, lane,
                                                     nrows, false, nullptr, d_lane, g.D, G);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                const uint32_t sst = smem_base + cur.s * STAGE;
                tma_st(&p.dx.map, sst + 0 * IN_TILE, c0, (int)t0, c2, hint, pol_drop);
                tma_st(&p.da.map, sst + 1 * IN_TILE, c0, (int)t0, c2, hint, pol_drop);
                tma_st(&p.db.map, sst + 2 * IN_TILE, c0, (int)t0, c2, hint, pol_drop);
                tma_st(&p.dc.map, sst + 3 * IN_TILE, c0, (int)t0, c2, hint, pol_drop);
                tma_commit();
            }
            __syncwarp();
            cur.advance(NS);
        }
        if (!ok) break;
        // the stores of this chunk must have read their stages before the next chunk refills them
        if (lane == 0) tma_wait_read<0>();
        __syncwarp();
    }
    if (lane == 0) {
        tma_wait_all();
        if (!ok) report(g.status, QSSM_S_TMA_TIMEOUT);
    }
}

// ---------------------------------------------------------------------------------------------
// backward with combined stores: a CTA of W = 4 warps scans four adjacent channel strips of the
// same batch entry and time range.  Every warp keeps its own input ring (no coupling on the load
// side); the gradients of a tile go to a shared staging tile 4 strips wide and ONE bulk store per
// gradient tensor writes 512 contiguous bytes per row instead of four stores of 128 bytes from
// four unrelated CTAs.  Measured on B200 the write-heavy backward gains from that locality: with
// 128-byte-wide stores it moves 5.9 TB/s, with contiguous rows 6.3-6.45 TB/s.
// One __syncthreads per tile orders "all four strips written" before the store is issued.
// ---------------------------------------------------------------------------------------------
constexpr int WIDE_W = 4;

template <typename Tin, typename Tdy, int V, bool SAVED_H>
__global__ void __launch_bounds__(32 * WIDE_W) scan_bwd_wide_kernel(const __grid_constant__ BwdParams p) {
    constexpr int W = WIDE_W;
    constexpr int TB = TS;
    constexpr int DT = 32 * V;
    constexpr int IN_ROW = 32 * V * (int)sizeof(Tin);
    constexpr int DY_ROW = 32 * V * (int)sizeof(Tdy);
    constexpr int H_ROW = 32 * V * 4;
    constexpr int IN_TILE = TB * IN_ROW;
    constexpr int DY_TILE = TB * DY_ROW;
    constexpr int H_TILE = SAVED_H ? (TB + 1) * H_ROW : H_ROW;
    constexpr int H_SLOT = ((H_TILE + 127) / 128) * 128;
    constexpr int STAGE = 4 * IN_TILE + DY_TILE + H_SLOT;
    constexpr int OFF_DY = 4 * IN_TILE;
    constexpr int OFF_H = OFF_DY + DY_TILE;
    constexpr int OUT_TILE = TB * W * IN_ROW;  // one gradient tensor, four strips wide
    constexpr int OUTBUF = 4 * OUT_TILE;

    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_fail;
    const Geom& g = p.g;
    const int NS = g.n_stages;
    const int NOUT = g.n_out;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    unsigned char* const my_stages = smem + (size_t)warp * NS * STAGE;
    unsigned char* const outbuf = smem + (size_t)W * NS * STAGE;
    const uint32_t bars = smem_u32(outbuf + (size_t)NOUT * OUTBUF) + warp * MAX_STAGES * 8;
    const uint32_t my_base = smem_u32(my_stages);
    const bool ld_hint = (g.l2_hint & 1) != 0, st_hint = (g.l2_hint & 2) != 0;
    const uint64_t pol = l2_policy_evict_first();

    if (threadIdx.x == 0) s_fail = 0;
    if (lane == 0) {
        for (int s = 0; s < NS; ++s) mbar_init(bars + 8 * s, 1);
        fence_barrier_init();
    }
    __syncthreads();

    const int n_dgroups = (g.n_dtiles + W - 1) / W;
    const long long n_groups = g.B * g.n_seg * n_dgroups;
    RingPos pf{0, 0};
    RingPos cur{0, 0};
    int oslot = 0;
    bool failed = false;
    for (long long gid = blockIdx.x; gid < n_groups && !failed; gid += gridDim.x) {
        const long long dgroup = gid % n_dgroups;
        const long long rest = gid / n_dgroups;
        const int seg = (int)(rest % g.n_seg);
        const long long b = rest / g.n_seg;
        const long long d0 = (dgroup * W + warp) * DT;
        const bool active = d0 < g.D;  // the last group of a row may have fewer than four strips
        const long long t_begin = (long long)seg * g.seg_rows;
        long long t_end = t_begin + g.seg_rows;
        if (t_end > g.L) t_end = g.L;
        const int n_tiles = (int)((t_end - t_begin + TB - 1) / TB);
        const long long d_lane = d0 + (long long)lane * V;

        float G[V];
#pragma unroll
        for (int i = 0; i < V; ++i) G[i] = 0.f;
        if (active && p.g_in != nullptr) {
            const float* src = p.g_in + (b * g.n_seg + seg) * g.D;
#pragma unroll
            for (int i = 0; i < V; ++i)
                if (d_lane + i < g.D) G[i] = src[d_lane + i];
        }
        const float* h_in_lane = (SAVED_H && p.h_in != nullptr) ? p.h_in + b * g.D + d_lane : nullptr;

        const int c0 = (int)d0, c2 = (int)b, c0_wide = (int)(dgroup * W * DT);
        int pf_row = (int)(t_begin + (long long)(n_tiles - 1) * TB);
        int pf_left = active ? n_tiles : 0;
        auto issue = [&]() {
            const uint32_t st = my_base + pf.s * STAGE;
            const uint32_t bar = bars + 8 * pf.s;
            fence_proxy_async();
            mbar_expect_tx(bar, 4 * IN_TILE + DY_TILE + H_TILE);
            tma_ld(st + 0 * IN_TILE, &p.x.map, bar, c0, pf_row, c2, ld_hint, pol);
            tma_ld(st + 1 * IN_TILE, &p.a.map, bar, c0, pf_row, c2, ld_hint, pol);
            tma_ld(st + 2 * IN_TILE, &p.b.map, bar, c0, pf_row, c2, ld_hint, pol);
            tma_ld(st + 3 * IN_TILE, &p.c.map, bar, c0, pf_row, c2, ld_hint, pol);
            tma_ld(st + OFF_DY, &p.dy.map, bar, c0, pf_row, c2, ld_hint, pol);
            if (SAVED_H)
                tma_ld(st + OFF_H, &p.hsrc.map, bar, c0, pf_row - 1, c2, ld_hint, pol);  // row -1 reads zero fill
            else
                tma_ld(st + OFF_H, &p.hsrc.map, bar, c0, pf_row / TS, c2, ld_hint, pol);
            pf.advance(NS);
            pf_row -= TB;
            --pf_left;
        };
        if (lane == 0) {
            for (int k = 0; k < NS - 1 && pf_left > 0; ++k) issue();
        }

        long long t0 = t_begin + (long long)(n_tiles - 1) * TB;
        for (int j = 0; j < n_tiles; ++j, t0 -= TB) {
            unsigned char* ob = outbuf + (size_t)oslot * OUTBUF;
            if (active) {
                const unsigned char* st = my_stages + cur.s * STAGE;
                const int nrows = (int)((t_end - t0) < TB ? (t_end - t0) : TB);
                if (lane == 0 && pf_left > 0) issue();
                bool ok = mbar_wait_bounded(bars + 8 * cur.s, cur.phase);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    if (lane == 0) s_fail = 1;
                } else {
                    const bool first_rows = (t0 == 0);
                    if (nrows >= TS)
                        bwd_batch<Tin, Tdy, V, SAVED_H, true, 32 * W>(
                            st, st + IN_TILE, st + 2 * IN_TILE, st + 3 * IN_TILE, st + OFF_DY, st + OFF_H, ob,
                            ob + OUT_TILE, ob + 2 * OUT_TILE, ob + 3 * OUT_TILE, warp * 32, lane, TS, first_rows,
                            h_in_lane, d_lane, g.D, G);
                    else
                        bwd_batch<Tin, Tdy, V, SAVED_H, false, 32 * W>(
                            st, st + IN_TILE, st + 2 * IN_TILE, st + 3 * IN_TILE, st + OFF_DY, st + OFF_H, ob,
                            ob + OUT_TILE, ob + 2 * OUT_TILE, ob + 3 * OUT_TILE, warp * 32, lane, nrows, first_rows,
                            h_in_lane, d_lane, g.D, G);
                }
                cur.advance(NS);
            }
            fence_proxy_async();
            // the staging tile written NOUT - 1 tiles from now must be free: stores older than that have drained
            if (threadIdx.x == 0) {
                if (NOUT == 2) tma_wait_read<0>();
                else tma_wait_read<1>();
            }
            __syncthreads();
            if (s_fail != 0) {
                failed = true;
                break;
            }
            if (threadIdx.x == 0) {
                const uint32_t so = smem_u32(ob);
                tma_st(&p.dx.map, so + 0 * OUT_TILE, c0_wide, (int)t0, c2, st_hint, pol);
                tma_st(&p.da.map, so + 1 * OUT_TILE, c0_wide, (int)t0, c2, st_hint, pol);
                tma_st(&p.db.map, so + 2 * OUT_TILE, c0_wide, (int)t0, c2, st_hint, pol);
                tma_st(&p.dc.map, so + 3 * OUT_TILE, c0_wide, (int)t0, c2, st_hint, pol);
                tma_commit();
            }
            if (++oslot == NOUT) oslot = 0;
        }
        if (failed) break;
        if (active && p.g_first != nullptr && seg == 0) {
            float* dst = p.g_first + b * g.D;
#pragma unroll
            for (int i = 0; i < V; ++i)
                if (d_lane + i < g.D) dst[d_lane + i] = G[i];
        }
    }
    if (threadIdx.x == 0) {
        tma_wait_all();
        if (failed) report(g.status, QSSM_S_TMA_TIMEOUT);
    }
}

// ---------------------------------------------------------------------------------------------
// aggregates of a segment.  forward: (prod a, h_end from 0) from x, a, b
//                           backward: (prod a, a(t0) dh(t0) from 0) from a, c, dy
// ---------------------------------------------------------------------------------------------
template <typename Tin, typename Tdy, int V, int TB, bool REVERSE>
__global__ void __launch_bounds__(32) scan_agg_kernel(const __grid_constant__ AggParams p) {
    constexpr int DT = 32 * V;
    constexpr int IN_ROW = 32 * V * (int)sizeof(Tin);
    constexpr int IN_TILE = TB * IN_ROW;
    constexpr int T2_TILE = REVERSE ? TB * 32 * V * (int)sizeof(Tdy) : IN_TILE;
    constexpr int STAGE = 2 * IN_TILE + T2_TILE;

    extern __shared__ __align__(128) unsigned char smem[];
    const Geom& g = p.g;
    const int NS = g.n_stages;
    const uint32_t bars = smem_u32(smem + NS * STAGE);
    const uint32_t smem_base = smem_u32(smem);

    const int lane = threadIdx.x;
    const bool tma = g.use_tma != 0;
    const bool ld_hint = (g.l2_hint & 1) != 0;
    const uint64_t pol = l2_policy_evict_first();
    if (tma) {
        if (lane == 0) {
            for (int s = 0; s < NS; ++s) mbar_init(bars + 8 * s, 1);
            fence_barrier_init();
        }
        __syncwarp();
    }
    bool ok = true;
    RingPos pf{0, 0};
    RingPos cur{0, 0};
    for (long long chain_id = blockIdx.x; chain_id < g.n_chains; chain_id += gridDim.x) {
    const Chain ch = chain_of(g, chain_id, DT, TB);
    const long long d_lane = ch.d0 + (long long)lane * V;
    float* const outA = p.A + (ch.b * g.n_seg + ch.seg) * g.D;
    float* const outH = p.H + (ch.b * g.n_seg + ch.seg) * g.D;
    if (ch.empty) {  // identity
#pragma unroll
        for (int i = 0; i < V; ++i)
            if (d_lane + i < g.D) { outA[d_lane + i] = 1.f; outH[d_lane + i] = 0.f; }
        continue;
    }

    float A[V], H[V];
#pragma unroll
    for (int i = 0; i < V; ++i) { A[i] = 1.f; H[i] = 0.f; }

    const int c0 = (int)ch.d0, c2 = (int)ch.b;
    int pf_row = (int)(REVERSE ? ch.t_begin + (long long)(ch.n_tiles - 1) * TB : ch.t_begin);
    int pf_left = ch.n_tiles;
    auto issue = [&]() {
        const uint32_t st = smem_base + pf.s * STAGE;
        const uint32_t bar = bars + 8 * pf.s;
        fence_proxy_async();
        mbar_expect_tx(bar, STAGE);
        tma_ld(st + 0 * IN_TILE, &p.t0.map, bar, c0, pf_row, c2, ld_hint, pol);
        tma_ld(st + 1 * IN_TILE, &p.t1.map, bar, c0, pf_row, c2, ld_hint, pol);
        tma_ld(st + 2 * IN_TILE, &p.t2.map, bar, c0, pf_row, c2, ld_hint, pol);
        pf.advance(NS);
        pf_row += REVERSE ? -TB : TB;
        --pf_left;
    };
    if (tma && lane == 0) {
        for (int k = 0; k < NS - 1 && pf_left > 0; ++k) issue();
    }
    long long t0 = REVERSE ? ch.t_begin + (long long)(ch.n_tiles - 1) * TB : ch.t_begin;
    for (int j = 0; j < ch.n_tiles; ++j, t0 += (REVERSE ? -TB : TB)) {
        unsigned char* st = smem + cur.s * STAGE;
        const int nrows = (int)((ch.t_end - t0) < TB ? (ch.t_end - t0) : TB);
        if (tma) {
            if (lane == 0 && pf_left > 0) issue();
            ok = mbar_wait_bounded(bars + 8 * cur.s, cur.phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
        } else {
            plain_fill<Tin, V>(st + 0 * IN_TILE, p.t0, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            plain_fill<Tin, V>(st + 1 * IN_TILE, p.t1, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            if (REVERSE)
                plain_fill<Tdy, V>(st + 2 * IN_TILE, p.t2, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
            else
                plain_fill<Tin, V>(st + 2 * IN_TILE, p.t2, ch.b, t0, TB, ch.t_end, d_lane, g.D, lane);
        }
        if (!REVERSE) {
#pragma unroll
            for (int r = 0; r < TB; ++r) {
                float xv[V], av[V], bv[V];
                unpack<Tin, V>(tile_raw<Tin, V>(st + 0 * IN_TILE, r, lane), xv);
                unpack<Tin, V>(tile_raw<Tin, V>(st + 1 * IN_TILE, r, lane), av);
                unpack<Tin, V>(tile_raw<Tin, V>(st + 2 * IN_TILE, r, lane), bv);
                if (r < nrows) {
#pragma unroll
                    for (int i = 0; i < V; ++i) { A[i] *= av[i]; H[i] = fmaf(av[i], H[i], bv[i] * xv[i]); }
                }
            }
        } else {
#pragma unroll
            for (int r = TB - 1; r >= 0; --r) {
                float av[V], cv[V], gy[V];
                unpack<Tin, V>(tile_raw<Tin, V>(st + 0 * IN_TILE, r, lane), av);
                unpack<Tin, V>(tile_raw<Tin, V>(st + 1 * IN_TILE, r, lane), cv);
                unpack<Tdy, V>(tile_raw<Tdy, V>(st + 2 * IN_TILE, r, lane), gy);
                if (r < nrows) {
#pragma unroll
                    for (int i = 0; i < V; ++i) { A[i] *= av[i]; H[i] = av[i] * fmaf(cv[i], gy[i], H[i]); }
                }
            }
        }
        __syncwarp();
        cur.advance(NS);
    }
    if (!ok) break;
#pragma unroll
    for (int i = 0; i < V; ++i)
        if (d_lane + i < g.D) { outA[d_lane + i] = A[i]; outH[d_lane + i] = H[i]; }
    }  // chains
    if (!ok && lane == 0) report(g.status, QSSM_S_TMA_TIMEOUT);
}

// ---------------------------------------------------------------------------------------------
// per-channel scan of segment aggregates -> seeds of every segment (+ optional totals)
//   A, H: [B, n_seg, D];  seed: [B, D] or NULL;  out: [B, n_seg, D];  totA/totH: [B, D] or NULL
// ---------------------------------------------------------------------------------------------
__global__ void seg_carry_kernel(const float* __restrict__ A, const float* __restrict__ H,
                                 const float* __restrict__ seed, float* __restrict__ out,
                                 float* __restrict__ totA, float* __restrict__ totH, long long B, int n_seg,
                                 long long D, int reverse) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * D) return;
    const long long b = idx / D, d = idx % D;
    float run = seed != nullptr ? seed[idx] : 0.f;
    float pa = 1.f, ph = 0.f;
    for (int k = 0; k < n_seg; ++k) {
        const int s = reverse ? n_seg - 1 - k : k;
        const long long o = (b * n_seg + s) * D + d;
        const float av = A[o], hv = H[o];
        if (out != nullptr) out[o] = run;
        run = fmaf(av, run, hv);
        ph = fmaf(av, ph, hv);
        pa *= av;
    }
    if (totA != nullptr) totA[idx] = pa;
    if (totH != nullptr) totH[idx] = ph;
}

__global__ void carry_fold_kernel(const float* __restrict__ A, const float* __restrict__ H, long long n,
                                  long long stride_k, long long n_chan, long long upto, int reverse,
                                  const float* __restrict__ seed, float* __restrict__ carry) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_chan) return;
    float run = seed != nullptr ? seed[idx] : 0.f;
    if (!reverse) {
        for (long long k = 0; k < upto; ++k) run = fmaf(A[k * stride_k + idx], run, H[k * stride_k + idx]);
    } else {
        for (long long k = n - 1; k > upto; --k) run = fmaf(A[k * stride_k + idx], run, H[k * stride_k + idx]);
    }
    carry[idx] = run;
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Driver-API calls (tensor map encoding) need the primary context current on the calling thread;
// a thread that has only inherited a device ordinal (e.g. an autograd worker) may not have one yet.
void ensure_context() {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaSetDevice(dev);
}

int dtype_size(int dt) { return dt == QSSM_F32 ? 4 : (dt == QSSM_F16 || dt == QSSM_BF16) ? 2 : 0; }

CUtensorMapDataType tm_dtype(int dt) {
    return dt == QSSM_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                          : dt == QSSM_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
}

// Can the copy engine address a [B, L, D] view with these strides?
bool tma_ok(const void* ptr, long long B, long long L, long long D, long long sb, long long sl, int esize) {
    if (ptr == nullptr) return true;
    if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) return false;
    if ((sl * esize) % 16 != 0 || (B > 1 && (sb * esize) % 16 != 0)) return false;
    if (sl * esize >= (1ll << 40) || sb * esize >= (1ll << 40)) return false;
    if (D >= (1ll << 32) || L >= (1ll << 31) || B >= (1ll << 31)) return false;
    return true;
}

int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return (v != nullptr && *v != '\0') ? atoi(v) : dflt;
}

// dims (D, rows, B); box (box_d, box_rows, 1)
int fill_desc(TensorDesc& td, const void* ptr, int dt, long long B, long long rows, long long D, long long sb,
              long long sl, int box_d, int box_rows, bool use_tma) {
    memset(&td, 0, sizeof(td));
    td.ptr = const_cast<void*>(ptr);
    td.stride_b = sb;
    td.stride_l = sl;
    if (!use_tma || ptr == nullptr) return 0;
    static thread_local bool have_context = false;
    if (!have_context) {
        ensure_context();
        have_context = true;
    }
    EncodeTiledFn enc = encode_fn();
    if (enc == nullptr) return QSSM_E_DRIVER;
    const int es = dtype_size(dt);
    cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)rows, (cuuint64_t)B};
    long long sb_bytes = sb * es;
    if (B <= 1 || sb_bytes == 0) sb_bytes = ((rows * sl * es + 15) / 16) * 16;
    if (sb_bytes == 0) sb_bytes = 16;
    cuuint64_t strides[2] = {(cuuint64_t)(sl * es), (cuuint64_t)sb_bytes};
    cuuint32_t box[3] = {(cuuint32_t)box_d, (cuuint32_t)box_rows, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = enc(&td.map, tm_dtype(dt), 3, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS && env_int("QSSM_DEBUG", 0) != 0)
        fprintf(stderr,
                "qssm: cuTensorMapEncodeTiled failed (%d): ptr=%p dt=%d dims=(%llu,%llu,%llu) strides=(%llu,%llu) "
                "box=(%u,%u,%u)\n",
                (int)r, ptr, dt, (unsigned long long)dims[0], (unsigned long long)dims[1],
                (unsigned long long)dims[2], (unsigned long long)strides[0], (unsigned long long)strides[1], box[0],
                box[1], box[2]);
    return r == CUDA_SUCCESS ? 0 : QSSM_E_STRIDE;
}

int sm_count() {
    static int n = []() {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 148;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) return 148;
        return v;
    }();
    return n;
}

// Launch shape of one call: channels per lane (V), rows per tile (TB), segments, ring depth.
struct Plan {
    Geom g;
    int V, TB;
    long long chains;  // chains of the launch
    long long grid;    // CTAs (= chains streaming at the same time)
};

// How many chains stream at once.  Measured on B200 (bf16/fp16, 128-byte strips): throughput rises
// with the number of resident chains up to about 3.5 per SM (512 in all) and then falls again -
// at 7 per SM the backward moves 17 % and the forward 7 % fewer bytes per second; the read-mostly
// forward peaks at exactly four per SM (one warp on every scheduler).  Launches with more chains
// than that therefore run them in equal rounds on a grid near the sweet spot; a launch is cut
// into rounds only when every round still fills the GPU.
long long concurrent_chains(long long chains, bool write_heavy) {
    const long long forced_grid = env_int("QSSM_GRID", 0);
    if (forced_grid > 0) return forced_grid < chains ? forced_grid : chains;
    const double target = write_heavy ? 3.5 * sm_count() : 4.0 * sm_count();
    long long rounds = (long long)((double)chains / target + (write_heavy ? 0.2 : 0.3));
    if (rounds < 1) rounds = 1;
    return (chains + rounds - 1) / rounds;
}

// Channels per lane.  Two channels per lane halve the shared-memory and copy-engine instructions
// per element, so one warp moves twice the bytes; narrow strips (V = 1) are for channel counts
// that would leave half of a wide strip empty, or for launches with too few chains to give
// every SM two warps even after the time axis has been segmented.
int pick_v(long long B, long long D, int n_seg) {
    const int forced = env_int("QSSM_V", 0);
    if (forced == 1 || forced == 2) return forced;
    if (D <= 32) return 1;
    const long long chains_v2 = B * ((D + 63) / 64) * (n_seg < 1 ? 1 : n_seg);
    return chains_v2 >= 2ll * sm_count() ? 2 : 1;
}
int pick_tb() {
    const int forced = env_int("QSSM_TB", 0);
    return forced == 16 || forced == 32 ? forced : 16;
}


// Segment count.  Cutting the time axis costs an extra read of the tensors the carry depends on
// (8 instead of 5 tensor passes forward, 12 instead of 9 backward), so it pays only when batch x
// channels alone leaves most of the GPU idle: fewer than two wide chains per SM.
int auto_segments(long long B, long long L, long long D, int in_dtype) {
    if (B <= 0 || L <= 0 || D <= 0 || dtype_size(in_dtype) == 0) return 1;
    const long long chains = B * ((D + 63) / 64);
    const long long sms = sm_count();
    if (chains >= 2 * sms) return 1;
    long long want = (4 * sms + chains - 1) / chains;
    const long long max_by_len = L / 256;  // at least 256 rows per segment
    if (want > max_by_len) want = max_by_len;
    if (want < 2) want = 1;
    if (want > 4096) want = 4096;
    return (int)want;
}

size_t ws_bytes_for(long long B, long long D, int n_seg) {
    if (n_seg <= 1) return 0;
    return (size_t)3 * (size_t)B * (size_t)n_seg * (size_t)D * sizeof(float);
}

// Ring depth.  Measured on B200: these kernels move the most bytes per second when roughly 15 MB of
// loads and stores are outstanding over the whole GPU (about 28 KB per chain at 512 chains); with
// more in flight throughput falls again (a fourth backward stage costs 19 %).  So the ring is as
// deep as that budget allows, within the shared memory an SM can give each of its resident CTAs.
//   grid          CTAs of the launch (all resident at once)
//   stage_bytes   one input stage
//   store_bytes   bytes of stores that can be pending while the ring is full
//   fixed_bytes   shared memory besides the input stages
//   prefetch(ns)  input tiles in flight with ns stages
template <typename F>
int pick_stages(long long grid, int stage_bytes, int store_bytes, int fixed_bytes, int lo, int hi, F prefetch) {
    const int forced = env_int("QSSM_STAGES", 0);
    if (forced >= lo && forced <= MAX_STAGES &&
        (long long)forced * stage_bytes + fixed_bytes + MAX_STAGES * 8 <= 227 * 1024)
        return forced;
    const long long sms = sm_count();
    const long long per_sm = (grid + sms - 1) / sms;
    const long long smem_cap = (228 * 1024) / (per_sm < 1 ? 1 : per_sm) - 1024;
    const long long budget = (15ll << 20) / (grid < 1 ? 1 : grid);
    int best = lo;
    for (int ns = lo; ns <= hi; ++ns) {
        const long long smem = (long long)ns * stage_bytes + fixed_bytes + MAX_STAGES * 8;
        if (smem > smem_cap || smem > 227 * 1024) break;
        if ((long long)prefetch(ns) * stage_bytes + store_bytes > budget) break;
        best = ns;
    }
    return best;
}

int make_plan(Plan& pl, long long B, long long L, long long D, int n_seg, int* status) {
    if (n_seg < 1) n_seg = 1;
    long long seg_rows = (L + n_seg - 1) / n_seg;
    seg_rows = ((seg_rows + 31) / 32) * 32;  // whole tiles for either tile height
    n_seg = (int)((L + seg_rows - 1) / seg_rows);
    pl.V = pick_v(B, D, n_seg);
    pl.TB = pick_tb();
    const int chans = 32 * pl.V;
    Geom& g = pl.g;
    g.B = B; g.L = L; g.D = D;
    g.n_dtiles = (int)((D + chans - 1) / chans);
    g.n_seg = n_seg;
    g.seg_rows = (int)seg_rows;
    g.status = status;
    g.use_tma = 1;
    g.l2_hint = env_int("QSSM_L2HINT", 0);
    g.n_stages = 2;
    pl.chains = B * n_seg * g.n_dtiles;
    g.n_chains = pl.chains;
    pl.grid = concurrent_chains(pl.chains, false);
    return 0;
}

template <typename K, typename P>
int launch(K kernel, const P& params, long long grid, int smem_bytes, cudaStream_t stream, int threads = 32) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return (int)e;
    kernel<<<(unsigned)grid, threads, smem_bytes, stream>>>(params);
    e = cudaGetLastError();
    return (int)e;
}

int check_common(long long B, long long L, long long D, int in_dtype, int out_dtype) {
    if (B < 0 || L < 0 || D < 0) return QSSM_E_SHAPE;
    if (dtype_size(in_dtype) == 0 || dtype_size(out_dtype) == 0) return QSSM_E_DTYPE;
    if (!(out_dtype == in_dtype || out_dtype == QSSM_F32)) return QSSM_E_DTYPE;
    if (L >= (1ll << 31) - 64 || B >= (1ll << 31)) return QSSM_E_SHAPE;
    return 0;
}
int check_strides(long long L, long long D, long long sb, long long sl) {
    if (sl < D) return QSSM_E_STRIDE;
    if (sb < 0) return QSSM_E_STRIDE;
    (void)L;
    return 0;
}

template <int N> using Int = std::integral_constant<int, N>;

// Calls f(Tin{}, Tout{}, Int<V>{}, Int<TB>{}) for the run-time (dtype pair, V, TB).
template <typename F> int dispatch(int in_dt, int out_dt, int V, int TB, F&& f) {
    auto with_types = [&](auto tin, auto tout) -> int {
        if (V == 1 && TB == 16) return f(tin, tout, Int<1>{}, Int<16>{});
        if (V == 1) return f(tin, tout, Int<1>{}, Int<32>{});
        if (TB == 16) return f(tin, tout, Int<2>{}, Int<16>{});
        return f(tin, tout, Int<2>{}, Int<32>{});
    };
    if (in_dt == QSSM_F32) return with_types(float{}, float{});
    if (in_dt == QSSM_F16 && out_dt == QSSM_F16) return with_types(__half{}, __half{});
    if (in_dt == QSSM_F16) return with_types(__half{}, float{});
    if (in_dt == QSSM_BF16 && out_dt == QSSM_BF16) return with_types(__nv_bfloat16{}, __nv_bfloat16{});
    return with_types(__nv_bfloat16{}, float{});
}

// segment aggregates -> seeds.  A/H/seeds live in ws: three [B, n_seg, D] fp32 arrays.
struct SegScratch {
    float *A, *H, *seeds;
};
SegScratch carve(void* ws, long long B, int n_seg, long long D) {
    SegScratch s;
    const size_t n = (size_t)B * n_seg * D;
    s.A = reinterpret_cast<float*>(ws);
    s.H = s.A + n;
    s.seeds = s.H + n;
    return s;
}

int run_aggregate(bool reverse, const void* t0, const void* t1, const void* t2, float* A, float* H,
                  const Plan& pl, long long sb, long long sl, long long sb2, long long sl2, int in_dtype,
                  int dt2, cudaStream_t stream) {
    AggParams ap;
    memset(&ap, 0, sizeof(ap));
    ap.g = pl.g;
    const Geom& g = pl.g;
    const int chans = 32 * pl.V, TB = pl.TB;
    bool tma = tma_ok(t0, g.B, g.L, g.D, sb, sl, dtype_size(in_dtype)) &&
               tma_ok(t1, g.B, g.L, g.D, sb, sl, dtype_size(in_dtype)) &&
               tma_ok(t2, g.B, g.L, g.D, sb2, sl2, dtype_size(dt2)) && env_int("QSSM_NO_TMA", 0) == 0;
    ap.g.use_tma = tma ? 1 : 0;
    int rc;
    if ((rc = fill_desc(ap.t0, t0, in_dtype, g.B, g.L, g.D, sb, sl, chans, TB, tma))) return rc;
    if ((rc = fill_desc(ap.t1, t1, in_dtype, g.B, g.L, g.D, sb, sl, chans, TB, tma))) return rc;
    if ((rc = fill_desc(ap.t2, t2, dt2, g.B, g.L, g.D, sb2, sl2, chans, TB, tma))) return rc;
    ap.A = A;
    ap.H = H;
    const int stage = TB * chans * (2 * dtype_size(in_dtype) + dtype_size(dt2));
    ap.g.n_stages = pick_stages(pl.grid, stage, 0, 0, 2, 8, [](int ns) { return ns - 1; });
    const int smem = ap.g.n_stages * stage + MAX_STAGES * 8;
    const int out_dt = reverse ? dt2 : in_dtype;
    return dispatch(in_dtype, out_dt, pl.V, pl.TB, [&](auto tin, auto tout, auto v, auto tb) -> int {
        using Tin = decltype(tin);
        using Tout = decltype(tout);
        constexpr int V = decltype(v)::value, TBc = decltype(tb)::value;
        if (reverse) return launch(scan_agg_kernel<Tin, Tout, V, TBc, true>, ap, pl.grid, smem, stream);
        return launch(scan_agg_kernel<Tin, Tin, V, TBc, false>, ap, pl.grid, smem, stream);
    });
}

int resolve_segments(int n_seg_req, long long B, long long L, long long D, int in_dtype, const void* ws,
                     size_t ws_bytes, int* n_seg_out) {
    if (n_seg_req < 0) n_seg_req = -n_seg_req;  // "aggregates already in ws": same count, same layout
    int n_seg = n_seg_req > 0 ? n_seg_req : auto_segments(B, L, D, in_dtype);
    if (n_seg > 1) {
        // make_plan may lower the count after rounding segments to whole tiles; size for the request
        const size_t need = ws_bytes_for(B, D, n_seg);
        if (ws == nullptr || ws_bytes < need) {
            if (n_seg_req > 1) return QSSM_E_WS;
            n_seg = 1;
        }
    }
    *n_seg_out = n_seg;
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Built-in scratch for qssm_scan_fwd_static_ws: lives in the library's device image, so every
// GPU that loads the library holds these bytes until the process exits.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_ws[QSSM_STATIC_WS_BYTES];

constexpr int MAX_DEVICES = 64;
void* g_static_ws_addr[MAX_DEVICES];  // device address of g_static_ws on each device, once resolved

// Device address of the built-in scratch on the current device.  `g_static_ws` in host code is only
// a handle for the runtime, never a pointer a kernel could use, so the address is asked for once
// per device (with that device current) and cached.
int static_ws_address(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return QSSM_E_SHAPE;
    void* p = __atomic_load_n(&g_static_ws_addr[dev], __ATOMIC_ACQUIRE);
    if (p == nullptr) {
        e = cudaGetSymbolAddress(&p, g_static_ws);
        if (e != cudaSuccess) return (int)e;
        if (p == nullptr) return QSSM_E_NULL;
        __atomic_store_n(&g_static_ws_addr[dev], p, __ATOMIC_RELEASE);  // same value from every thread
    }
    *out = p;
    return 0;
}

// ---------------------------------------------------------------------------------------------
// chained forward: host side
// ---------------------------------------------------------------------------------------------
struct ChainedLayout {
    long long n_chains, grid;
    int slots, chunk_rows, n_chunks;
    size_t desc_off, bytes, zero_bytes;
};

// 0 = never, 1 = when the time axis would otherwise be segmented, 2 = whenever the shape allows (tests)
int chained_mode() { return env_int("QSSM_CHAINED", 1); }

// Chunks of 256 rows of 16-bit data (128 of fp32): with about a thousand chunks in flight the three
// tensors the first pass leaves in L2 for the second one take ~100 MB of the 126 MB L2; measured on
// B200 the second pass then reads them from L2 (DRAM reads = one pass), with 512 rows it does not.
ChainedLayout chained_layout(long long B, long long L, long long D, int elem_size) {
    ChainedLayout c;
    c.n_chains = B * ((D + 63) / 64);
    c.chunk_rows = env_int("QSSM_CHUNK_ROWS", elem_size == 2 ? 256 : 128);
    if (c.chunk_rows < TS) c.chunk_rows = TS;
    c.chunk_rows = (c.chunk_rows / TS) * TS;
    c.n_chunks = (int)((L + c.chunk_rows - 1) / c.chunk_rows);
    // two warps per scheduler: the two passes make a lone warp per scheduler compute-bound
    c.grid = env_int("QSSM_CHAINED_GRID", 0) > 0 ? env_int("QSSM_CHAINED_GRID", 0) : 8ll * sm_count();
    const long long total = c.n_chains * c.n_chunks;
    if (c.grid > total) c.grid = total;
    if (c.grid < 1) c.grid = 1;
    long long need = (c.grid + c.n_chains - 1) / c.n_chains + 2;  // chunks of one chain in flight, plus slack
    int slots = 4;
    while (slots < need) slots <<= 1;
    c.slots = slots;
    c.desc_off = 256;
    c.bytes = c.desc_off + (size_t)c.n_chains * slots * 96 * 16;
    c.zero_bytes = c.bytes;
    return c;
}

bool chained_shape_ok(long long B, long long L, long long D) {
    return B > 0 && L >= 4 * TS && D > 32 && B * ((D + 63) / 64) * ((L + TS - 1) / TS) < 0x7fffffffll;
}

size_t chained_ws_bytes(long long B, long long L, long long D, int in_dtype) {
    const int mode = chained_mode();
    if (mode == 0 || !chained_shape_ok(B, L, D)) return 0;
    // measured crossover: below about 2.75 chains per SM the chained kernels (~182 Gelem/s fwd+bwd on
    // 16-bit data whatever the chain count) beat one warp per chain (168 at 384 chains, 196 at 448)
    if (mode == 1 && 4 * B * ((D + 63) / 64) >= 11 * (long long)sm_count()) return 0;
    return chained_layout(B, L, D, dtype_size(in_dtype)).bytes;
}

template <typename K> long long resident_ctas(K kernel, int threads, int smem) {
    int per_sm = 0;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess) return 0;
    return (long long)per_sm * sm_count();
}

}  // namespace

// =============================================================================================
// C ABI
// =============================================================================================
extern "C" {

int qssm_version(void) { return 100; }

int qssm_tile_rows(void) { return TS; }

const char* qssm_status_string(int code) {
    switch (code) {
        case 0: return "ok";
        case QSSM_E_NULL: return "a required pointer is NULL";
        case QSSM_E_SHAPE: return "bad shape";
        case QSSM_E_DTYPE: return "unknown dtype or unsupported in/out dtype pair";
        case QSSM_E_STRIDE: return "bad stride";
        case QSSM_E_NEED_H: return "backward needs tile_h or h_saved";
        case QSSM_E_WS: return "workspace too small for the requested segment count";
        case QSSM_E_DRIVER: return "CUDA driver entry point cuTensorMapEncodeTiled unavailable";
        case QSSM_E_STATIC_WS:
            return "segment scratch for this shape exceeds QSSM_STATIC_WS_BYTES, the built-in maximum";
        case QSSM_S_TMA_TIMEOUT: return "device: bounded wait on a bulk-copy barrier expired";
        default: break;
    }
    if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
    return "unknown qssm error";
}

size_t qssm_workspace_bytes(int64_t B, int64_t L, int64_t D, int in_dtype) {
    const size_t seg = ws_bytes_for(B, D, auto_segments(B, L, D, in_dtype));
    const size_t chained = chained_ws_bytes(B, L, D, in_dtype);
    return seg > chained ? seg : chained;
}

int qssm_auto_segments(int64_t B, int64_t L, int64_t D, int in_dtype) { return auto_segments(B, L, D, in_dtype); }

int qssm_scan_fwd(const void* x, const void* a, const void* b, const void* c, void* y, float* h_saved,
                  float* tile_h, const float* h_in, float* h_last, void* ws, size_t ws_bytes, int64_t B,
                  int64_t L, int64_t D, int64_t in_stride_b, int64_t in_stride_l, int64_t out_stride_b,
                  int64_t out_stride_l, int in_dtype, int out_dtype, int n_seg_req, int* status_word,
                  void* stream_v) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    int rc = check_common(B, L, D, in_dtype, out_dtype);
    if (rc) return rc;
    if (B == 0 || L == 0 || D == 0) {
        if (h_last != nullptr && B > 0 && D > 0) {  // L == 0: the state passes through
            if (h_in != nullptr)
                return (int)cudaMemcpyAsync(h_last, h_in, (size_t)B * D * 4, cudaMemcpyDeviceToDevice, stream);
            return (int)cudaMemsetAsync(h_last, 0, (size_t)B * D * 4, stream);
        }
        return 0;
    }
    if (x == nullptr || a == nullptr || b == nullptr || y == nullptr) return QSSM_E_NULL;
    if ((rc = check_strides(L, D, in_stride_b, in_stride_l))) return rc;
    if ((rc = check_strides(L, D, out_stride_b, out_stride_l))) return rc;

    // Few chains, long sequence: single-pass chained kernel instead of aggregate + carry + scan.
    if (n_seg_req == 0 && h_saved == nullptr && ws != nullptr && env_int("QSSM_NO_TMA", 0) == 0) {
        const size_t need = chained_ws_bytes(B, L, D, in_dtype);
        const int es = dtype_size(in_dtype), eo = dtype_size(out_dtype);
        if (need > 0 && ws_bytes >= need && tma_ok(x, B, L, D, in_stride_b, in_stride_l, es) &&
            tma_ok(a, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(b, B, L, D, in_stride_b, in_stride_l, es) &&
            tma_ok(c, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(y, B, L, D, out_stride_b, out_stride_l, eo)) {
            const ChainedLayout lay = chained_layout(B, L, D, es);
            ChainedParams cp;
            memset(&cp, 0, sizeof(cp));
            Geom& g = cp.f.g;
            g.B = B; g.L = L; g.D = D;
            g.n_dtiles = (int)((D + 63) / 64);
            g.n_seg = 1;
            g.seg_rows = 0;
            g.use_tma = 1;
            g.l2_hint = env_int("QSSM_CHAINED_HINT", 1);
            g.status = status_word;
            g.n_chains = lay.n_chains;
            g.n_out = 3;
            g.n_stages = env_int("QSSM_STAGES", 0) >= 2 && env_int("QSSM_STAGES", 0) <= 8 ? env_int("QSSM_STAGES", 0) : 3;
            const int chans = 64;
            if ((rc = fill_desc(cp.f.x, x, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TS, true))) return rc;
            if ((rc = fill_desc(cp.f.a, a, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TS, true))) return rc;
            if ((rc = fill_desc(cp.f.b, b, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TS, true))) return rc;
            if ((rc = fill_desc(cp.f.c, c, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TS, true))) return rc;
            if ((rc = fill_desc(cp.f.y, y, out_dtype, B, L, D, out_stride_b, out_stride_l, chans, TS, true))) return rc;
            cp.f.tile_h = tile_h;
            cp.f.h_in = h_in;
            cp.f.h_last = h_last;
            unsigned char* base = static_cast<unsigned char*>(ws);
            cp.ticket = reinterpret_cast<unsigned int*>(base);
            cp.desc = reinterpret_cast<float*>(base + lay.desc_off);
            cp.chunk_rows = lay.chunk_rows;
            cp.slots = lay.slots;
            cp.n_chunks = lay.n_chunks;
            const int smem = g.n_stages * 4 * TS * chans * es + g.n_out * TS * chans * eo + MAX_STAGES * 8;
            const bool has_c = c != nullptr;
            return dispatch(in_dtype, out_dtype, 2, TS, [&](auto tin, auto tout, auto, auto) -> int {
                using Tin = decltype(tin);
                using Tout = decltype(tout);
                auto go = [&](auto kernel) -> int {
                    // every CTA must be resident: warps wait on chunks held by other running warps
                    long long grid = lay.grid;
                    const long long cap = resident_ctas(kernel, 32, smem);
                    if (cap < 1) return QSSM_E_SHAPE;
                    if (grid > cap) grid = cap;
                    cudaError_t e = cudaMemsetAsync(ws, 0, lay.zero_bytes, stream);
                    if (e != cudaSuccess) return (int)e;
                    return launch(kernel, cp, grid, smem, stream);
                };
                if (has_c) return go(scan_fwd_chained_kernel<Tin, Tout, true>);
                return go(scan_fwd_chained_kernel<Tin, Tout, false>);
            });
        }
    }

    int n_seg = 1;
    if ((rc = resolve_segments(n_seg_req, B, L, D, in_dtype, ws, ws_bytes, &n_seg))) return rc;
    Plan pl;
    if ((rc = make_plan(pl, B, L, D, n_seg, status_word))) return rc;
    n_seg = pl.g.n_seg;

    const float* seeds = h_in;
    if (n_seg > 1) {
        SegScratch sc = carve(ws, B, n_seg, D);
        if (n_seg_req >= 0) {  // negative: qssm_scan_aggregate_fwd has already left them in ws
            rc = run_aggregate(false, x, a, b, sc.A, sc.H, pl, in_stride_b, in_stride_l, in_stride_b, in_stride_l,
                               in_dtype, in_dtype, stream);
            if (rc) return rc;
        }
        const long long n = B * D;
        seg_carry_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(sc.A, sc.H, h_in, sc.seeds, nullptr,
                                                                          nullptr, B, n_seg, D, 0);
        if ((rc = (int)cudaGetLastError())) return rc;
        seeds = sc.seeds;
    }

    FwdParams fp;
    memset(&fp, 0, sizeof(fp));
    fp.g = pl.g;
    const int es = dtype_size(in_dtype), eo = dtype_size(out_dtype);
    const int chans = 32 * pl.V, TB = pl.TB;
    const long long hs_sb = L * D, hs_sl = D;
    bool tma = env_int("QSSM_NO_TMA", 0) == 0 && tma_ok(x, B, L, D, in_stride_b, in_stride_l, es) &&
               tma_ok(a, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(b, B, L, D, in_stride_b, in_stride_l, es) &&
               tma_ok(c, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(y, B, L, D, out_stride_b, out_stride_l, eo) &&
               tma_ok(h_saved, B, L, D, hs_sb, hs_sl, 4);
    fp.g.use_tma = tma ? 1 : 0;
    if ((rc = fill_desc(fp.x, x, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TB, tma))) return rc;
    if ((rc = fill_desc(fp.a, a, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TB, tma))) return rc;
    if ((rc = fill_desc(fp.b, b, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TB, tma))) return rc;
    if ((rc = fill_desc(fp.c, c, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TB, tma))) return rc;
    if ((rc = fill_desc(fp.y, y, out_dtype, B, L, D, out_stride_b, out_stride_l, chans, TB, tma))) return rc;
    if ((rc = fill_desc(fp.hs, h_saved, QSSM_F32, B, L, D, hs_sb, hs_sl, chans, TB, tma))) return rc;
    fp.tile_h = tile_h;
    fp.h_in = seeds;
    fp.h_last = h_last;

    const int nin = c != nullptr ? 4 : 3;
    const int stage = nin * TB * chans * es;
    const int outbuf = TB * chans * eo + (h_saved != nullptr ? TB * chans * 4 : 0);
    int n_out = env_int("QSSM_NOUT", 3);
    if (n_out < 2) n_out = 2;
    if (n_out > 4) n_out = 4;
    fp.g.n_out = n_out;
    fp.g.n_stages = pick_stages(pl.grid, stage, (n_out - 1) * outbuf, n_out * outbuf, 2, 8,
                                [](int ns) { return ns - 1; });
    const int smem = fp.g.n_stages * stage + n_out * outbuf + MAX_STAGES * 8;
    const bool has_c = c != nullptr, save_h = h_saved != nullptr;

    return dispatch(in_dtype, out_dtype, pl.V, pl.TB, [&](auto tin, auto tout, auto v, auto tb) -> int {
        using Tin = decltype(tin);
        using Tout = decltype(tout);
        constexpr int V = decltype(v)::value, TBc = decltype(tb)::value;
        if (has_c && save_h) return launch(scan_fwd_kernel<Tin, Tout, V, TBc, true, true>, fp, pl.grid, smem, stream);
        if (has_c) return launch(scan_fwd_kernel<Tin, Tout, V, TBc, true, false>, fp, pl.grid, smem, stream);
        if (save_h) return launch(scan_fwd_kernel<Tin, Tout, V, TBc, false, true>, fp, pl.grid, smem, stream);
        return launch(scan_fwd_kernel<Tin, Tout, V, TBc, false, false>, fp, pl.grid, smem, stream);
    });
}

int qssm_scan_fwd_static_ws(const void* x, const void* a, const void* b, const void* c, void* y, float* h_saved,
                            float* tile_h, const float* h_in, float* h_last, int64_t B, int64_t L, int64_t D,
                            int64_t in_stride_b, int64_t in_stride_l, int64_t out_stride_b, int64_t out_stride_l,
                            int in_dtype, int out_dtype, int n_seg_req, int* status_word, void* stream) {
    int rc = check_common(B, L, D, in_dtype, out_dtype);
    if (rc) return rc;
    // Scratch the segmented scan would need; refuse rather than quietly run unsegmented.
    const int n_seg = n_seg_req != 0 ? (n_seg_req < 0 ? -n_seg_req : n_seg_req) : auto_segments(B, L, D, in_dtype);
    const size_t need = ws_bytes_for(B, D, n_seg);
    if (need > (size_t)QSSM_STATIC_WS_BYTES) return QSSM_E_STATIC_WS;
    void* ws = nullptr;
    if ((rc = static_ws_address(&ws))) return rc;
    return qssm_scan_fwd(x, a, b, c, y, h_saved, tile_h, h_in, h_last, ws, (size_t)QSSM_STATIC_WS_BYTES, B, L, D,
                         in_stride_b, in_stride_l, out_stride_b, out_stride_l, in_dtype, out_dtype, n_seg_req,
                         status_word, stream);
}

int qssm_scan_bwd(const void* x, const void* a, const void* b, const void* c, const void* dy,
                  const float* h_saved, const float* tile_h, const float* h_in, const float* g_in,
                  float* g_first, void* dx, void* da, void* db, void* dc, void* ws, size_t ws_bytes, int64_t B,
                  int64_t L, int64_t D, int64_t in_stride_b, int64_t in_stride_l, int64_t dy_stride_b,
                  int64_t dy_stride_l, int in_dtype, int out_dtype, int n_seg_req, int* status_word,
                  void* stream_v) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    int rc = check_common(B, L, D, in_dtype, out_dtype);
    if (rc) return rc;
    if (B == 0 || L == 0 || D == 0) {
        if (g_first != nullptr && B > 0 && D > 0) {
            if (g_in != nullptr)
                return (int)cudaMemcpyAsync(g_first, g_in, (size_t)B * D * 4, cudaMemcpyDeviceToDevice, stream);
            return (int)cudaMemsetAsync(g_first, 0, (size_t)B * D * 4, stream);
        }
        return 0;
    }
    if (x == nullptr || a == nullptr || b == nullptr || c == nullptr || dy == nullptr || dx == nullptr ||
        da == nullptr || db == nullptr || dc == nullptr)
        return QSSM_E_NULL;
    if (h_saved == nullptr && tile_h == nullptr) return QSSM_E_NEED_H;
    if ((rc = check_strides(L, D, in_stride_b, in_stride_l))) return rc;
    if ((rc = check_strides(L, D, dy_stride_b, dy_stride_l))) return rc;

    // Few chains, long sequence: single-pass chained kernel (h rebuilt from tile_h only).
    if (n_seg_req == 0 && h_saved == nullptr && ws != nullptr && env_int("QSSM_NO_TMA", 0) == 0) {
        const size_t need = chained_ws_bytes(B, L, D, in_dtype);
        const int es = dtype_size(in_dtype), eo = dtype_size(out_dtype);
        const long long n_tiles_b = (L + TS - 1) / TS;
        const long long g_sb = L * D, g_sl = D;
        if (need > 0 && ws_bytes >= need && tma_ok(x, B, L, D, in_stride_b, in_stride_l, es) &&
            tma_ok(a, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(b, B, L, D, in_stride_b, in_stride_l, es) &&
            tma_ok(c, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(dy, B, L, D, dy_stride_b, dy_stride_l, eo) &&
            tma_ok(dx, B, L, D, g_sb, g_sl, es) && tma_ok(da, B, L, D, g_sb, g_sl, es) &&
            tma_ok(db, B, L, D, g_sb, g_sl, es) && tma_ok(dc, B, L, D, g_sb, g_sl, es) &&
            tma_ok(tile_h, B, n_tiles_b, D, n_tiles_b * D, D, 4)) {
            const ChainedLayout lay = chained_layout(B, L, D, es);
            ChainedBwdParams cp;
            memset(&cp, 0, sizeof(cp));
            Geom& g = cp.f.g;
            g.B = B; g.L = L; g.D = D;
            g.n_dtiles = (int)((D + 63) / 64);
            g.n_seg = 1;
            g.use_tma = 1;
            g.l2_hint = env_int("QSSM_CHAINED_HINT", 1);
            g.status = status_word;
            g.n_chains = lay.n_chains;
            g.n_stages = env_int("QSSM_STAGES", 0) >= 2 && env_int("QSSM_STAGES", 0) <= 8 ? env_int("QSSM_STAGES", 0) : 4;
            const int chans = 64;
            BwdParams& f = cp.f;
            if ((rc = fill_desc(f.x, x, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TS, true))) return rc;
            if ((rc = fill_desc(f.a, a, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TS, true))) return rc;
            if ((rc = fill_desc(f.b, b, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TS, true))) return rc;
            if ((rc = fill_desc(f.c, c, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TS, true))) return rc;
            if ((rc = fill_desc(f.dy, dy, out_dtype, B, L, D, dy_stride_b, dy_stride_l, chans, TS, true))) return rc;
            if ((rc = fill_desc(f.hsrc, tile_h, QSSM_F32, B, n_tiles_b, D, n_tiles_b * D, D, chans, 1, true))) return rc;
            if ((rc = fill_desc(f.dx, dx, in_dtype, B, L, D, g_sb, g_sl, chans, TS, true))) return rc;
            if ((rc = fill_desc(f.da, da, in_dtype, B, L, D, g_sb, g_sl, chans, TS, true))) return rc;
            if ((rc = fill_desc(f.db, db, in_dtype, B, L, D, g_sb, g_sl, chans, TS, true))) return rc;
            if ((rc = fill_desc(f.dc, dc, in_dtype, B, L, D, g_sb, g_sl, chans, TS, true))) return rc;
            f.g_in = g_in;
            f.g_first = g_first;
            unsigned char* base = static_cast<unsigned char*>(ws);
            cp.ticket = reinterpret_cast<unsigned int*>(base);
            cp.desc = reinterpret_cast<float*>(base + lay.desc_off);
            cp.chunk_rows = lay.chunk_rows;
            cp.slots = lay.slots;
            cp.n_chunks = lay.n_chunks;
            const int stage = 4 * TS * chans * es + TS * chans * eo + ((chans * 4 + 127) / 128) * 128;
            const int smem = g.n_stages * stage + MAX_STAGES * 8;
            return dispatch(in_dtype, out_dtype, 2, TS, [&](auto tin, auto tout, auto, auto) -> int {
                using Tin = decltype(tin);
                using Tout = decltype(tout);
                auto kernel = scan_bwd_chained_kernel<Tin, Tout>;
                long long grid = lay.grid;
                const long long cap = resident_ctas(kernel, 32, smem);  // every CTA must be resident
                if (cap < 1) return QSSM_E_SHAPE;
                if (grid > cap) grid = cap;
                cudaError_t e = cudaMemsetAsync(ws, 0, lay.zero_bytes, stream);
                if (e != cudaSuccess) return (int)e;
                return launch(kernel, cp, grid, smem, stream);
            });
        }
    }

    int n_seg = 1;
    if ((rc = resolve_segments(n_seg_req, B, L, D, in_dtype, ws, ws_bytes, &n_seg))) return rc;
    Plan pl;
    if ((rc = make_plan(pl, B, L, D, n_seg, status_word))) return rc;
    n_seg = pl.g.n_seg;

    const float* seeds = g_in;
    if (n_seg > 1) {
        SegScratch sc = carve(ws, B, n_seg, D);
        if (n_seg_req >= 0) {  // negative: qssm_scan_aggregate_bwd has already left them in ws
            rc = run_aggregate(true, a, c, dy, sc.A, sc.H, pl, in_stride_b, in_stride_l, dy_stride_b, dy_stride_l,
                               in_dtype, out_dtype, stream);
            if (rc) return rc;
        }
        const long long n = B * D;
        seg_carry_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(sc.A, sc.H, g_in, sc.seeds, nullptr,
                                                                          nullptr, B, n_seg, D, 1);
        if ((rc = (int)cudaGetLastError())) return rc;
        seeds = sc.seeds;
    }

    BwdParams bp;
    memset(&bp, 0, sizeof(bp));
    bp.g = pl.g;
    const int es = dtype_size(in_dtype), eo = dtype_size(out_dtype);
    const int chans = 32 * pl.V, TB = pl.TB;
    const bool saved = h_saved != nullptr;
    const long long n_tiles_b = (L + TS - 1) / TS;
    const long long g_sb = L * D, g_sl = D;  // gradients and h_saved are contiguous
    bool tma = env_int("QSSM_NO_TMA", 0) == 0 && tma_ok(x, B, L, D, in_stride_b, in_stride_l, es) &&
               tma_ok(a, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(b, B, L, D, in_stride_b, in_stride_l, es) &&
               tma_ok(c, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(dy, B, L, D, dy_stride_b, dy_stride_l, eo) &&
               tma_ok(dx, B, L, D, g_sb, g_sl, es) && tma_ok(da, B, L, D, g_sb, g_sl, es) &&
               tma_ok(db, B, L, D, g_sb, g_sl, es) && tma_ok(dc, B, L, D, g_sb, g_sl, es) &&
               (saved ? tma_ok(h_saved, B, L, D, g_sb, g_sl, 4) : tma_ok(tile_h, B, n_tiles_b, D, n_tiles_b * D, D, 4));
    bp.g.use_tma = tma ? 1 : 0;
    if ((rc = fill_desc(bp.x, x, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TB, tma))) return rc;
    if ((rc = fill_desc(bp.a, a, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TB, tma))) return rc;
    if ((rc = fill_desc(bp.b, b, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TB, tma))) return rc;
    if ((rc = fill_desc(bp.c, c, in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TB, tma))) return rc;
    if ((rc = fill_desc(bp.dy, dy, out_dtype, B, L, D, dy_stride_b, dy_stride_l, chans, TB, tma))) return rc;
    if (saved)
        rc = fill_desc(bp.hsrc, h_saved, QSSM_F32, B, L, D, g_sb, g_sl, chans, TB + 1, tma);
    else
        rc = fill_desc(bp.hsrc, tile_h, QSSM_F32, B, n_tiles_b, D, n_tiles_b * D, D, chans, TB / TS, tma);
    if (rc) return rc;
    // Four adjacent strips per CTA with one store per gradient tensor (16-bit storage, full-width rows).
    const bool wide = tma && env_int("QSSM_WIDE", 1) != 0 && es == 2 && pl.V == 2 && TB == TS &&
                      pl.g.n_dtiles >= WIDE_W;
    const int out_box = wide ? WIDE_W * chans : chans;
    if ((rc = fill_desc(bp.dx, dx, in_dtype, B, L, D, g_sb, g_sl, out_box, TB, tma))) return rc;
    if ((rc = fill_desc(bp.da, da, in_dtype, B, L, D, g_sb, g_sl, out_box, TB, tma))) return rc;
    if ((rc = fill_desc(bp.db, db, in_dtype, B, L, D, g_sb, g_sl, out_box, TB, tma))) return rc;
    if ((rc = fill_desc(bp.dc, dc, in_dtype, B, L, D, g_sb, g_sl, out_box, TB, tma))) return rc;
    bp.h_in = h_in;
    bp.g_in = seeds;
    bp.g_first = g_first;

    const int hrow = chans * 4;
    const int h_tile = saved ? (TB + 1) * hrow : (TB / TS) * hrow;
    const int stage = 4 * TB * chans * es + TB * chans * eo + ((h_tile + 127) / 128) * 128;
    const int grad_tile = 4 * TB * chans * es;  // the four gradient tiles of one strip
    if (wide) {
        const int n_dgroups = (pl.g.n_dtiles + WIDE_W - 1) / WIDE_W;
        const long long n_groups = B * n_seg * n_dgroups;
        long long ctas = (concurrent_chains(n_groups * WIDE_W, true) + WIDE_W - 1) / WIDE_W;
        if (ctas > n_groups) ctas = n_groups;
        int n_out = env_int("QSSM_NOUT_BWD", 2);
        if (n_out < 2) n_out = 2;
        if (n_out > 3) n_out = 3;
        bp.g.n_out = n_out;
        const int outbuf = WIDE_W * grad_tile;
        bp.g.n_stages = pick_stages(ctas, WIDE_W * stage, (n_out - 1) * outbuf,
                                    n_out * outbuf + WIDE_W * MAX_STAGES * 8, 2, 6, [](int ns) { return ns - 1; });
        const int smem = WIDE_W * bp.g.n_stages * stage + n_out * outbuf + WIDE_W * MAX_STAGES * 8;
        return dispatch(in_dtype, out_dtype, 2, TS, [&](auto tin, auto tout, auto, auto) -> int {
            using Tin = decltype(tin);
            using Tout = decltype(tout);
            if constexpr (sizeof(Tin) == 2) {
                if (saved)
                    return launch(scan_bwd_wide_kernel<Tin, Tout, 2, true>, bp, ctas, smem, stream, 32 * WIDE_W);
                return launch(scan_bwd_wide_kernel<Tin, Tout, 2, false>, bp, ctas, smem, stream, 32 * WIDE_W);
            } else {
                return QSSM_E_DTYPE;
            }
        });
    }
    pl.grid = concurrent_chains(pl.chains, true);
    // gradients are stored from the stages themselves: up to two tiles of them pending (one with two stages)
    bp.g.n_stages = pick_stages(pl.grid, stage, 2 * grad_tile, 0, 2, 6,
                                [](int ns) { return ns > 2 ? ns - 2 : 1; });
    const int smem = bp.g.n_stages * stage + MAX_STAGES * 8;
    return dispatch(in_dtype, out_dtype, pl.V, pl.TB, [&](auto tin, auto tout, auto v, auto tb) -> int {
        using Tin = decltype(tin);
        using Tout = decltype(tout);
        constexpr int V = decltype(v)::value, TBc = decltype(tb)::value;
        if (saved) return launch(scan_bwd_kernel<Tin, Tout, V, TBc, true>, bp, pl.grid, smem, stream);
        return launch(scan_bwd_kernel<Tin, Tout, V, TBc, false>, bp, pl.grid, smem, stream);
    });
}

static int aggregate_entry(bool reverse, const void* t0, const void* t1, const void* t2, float* A, float* H,
                           void* ws, size_t ws_bytes, int64_t B, int64_t L, int64_t D, int64_t sb, int64_t sl,
                           int64_t sb2, int64_t sl2, int in_dtype, int dt2, int n_seg_req, int* status_word,
                           cudaStream_t stream) {
    int rc = check_common(B, L, D, in_dtype, dt2);
    if (rc) return rc;
    if (B == 0 || D == 0) return 0;
    if (A == nullptr || H == nullptr) return QSSM_E_NULL;
    if (L == 0) {  // identity aggregate: prod over an empty range is 1, state 0
        const long long n = B * D;
        rc = (int)cudaMemsetAsync(H, 0, (size_t)n * 4, stream);
        if (rc) return rc;
        seg_carry_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(nullptr, nullptr, nullptr, nullptr, A,
                                                                          nullptr, B, 0, D, 0);
        return (int)cudaGetLastError();
    }
    if (t0 == nullptr || t1 == nullptr || t2 == nullptr) return QSSM_E_NULL;
    if ((rc = check_strides(L, D, sb, sl))) return rc;
    if ((rc = check_strides(L, D, sb2, sl2))) return rc;
    int n_seg = 1;
    if ((rc = resolve_segments(n_seg_req, B, L, D, in_dtype, ws, ws_bytes, &n_seg))) return rc;
    Plan pl;
    if ((rc = make_plan(pl, B, L, D, n_seg, status_word))) return rc;
    n_seg = pl.g.n_seg;
    if (n_seg == 1) return run_aggregate(reverse, t0, t1, t2, A, H, pl, sb, sl, sb2, sl2, in_dtype, dt2, stream);
    SegScratch sc = carve(ws, B, n_seg, D);
    rc = run_aggregate(reverse, t0, t1, t2, sc.A, sc.H, pl, sb, sl, sb2, sl2, in_dtype, dt2, stream);
    if (rc) return rc;
    const long long n = B * D;
    seg_carry_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(sc.A, sc.H, nullptr, nullptr, A, H, B, n_seg,
                                                                      D, reverse ? 1 : 0);
    return (int)cudaGetLastError();
}

int qssm_scan_aggregate_fwd(const void* x, const void* a, const void* b, float* A, float* H, void* ws,
                            size_t ws_bytes, int64_t B, int64_t L, int64_t D, int64_t in_stride_b,
                            int64_t in_stride_l, int in_dtype, int n_seg, int* status_word, void* stream) {
    return aggregate_entry(false, x, a, b, A, H, ws, ws_bytes, B, L, D, in_stride_b, in_stride_l, in_stride_b,
                           in_stride_l, in_dtype, in_dtype, n_seg, status_word, static_cast<cudaStream_t>(stream));
}

int qssm_scan_aggregate_bwd(const void* a, const void* c, const void* dy, float* P, float* Q, void* ws,
                            size_t ws_bytes, int64_t B, int64_t L, int64_t D, int64_t in_stride_b,
                            int64_t in_stride_l, int64_t dy_stride_b, int64_t dy_stride_l, int in_dtype,
                            int out_dtype, int n_seg, int* status_word, void* stream) {
    return aggregate_entry(true, a, c, dy, P, Q, ws, ws_bytes, B, L, D, in_stride_b, in_stride_l, dy_stride_b,
                           dy_stride_l, in_dtype, out_dtype, n_seg, status_word, static_cast<cudaStream_t>(stream));
}

int qssm_carry_fold(const float* A, const float* H, int64_t n, int64_t stride_k, int64_t n_chan, int64_t upto,
                    int reverse, const float* seed, float* carry, void* stream) {
    if (n_chan == 0) return 0;
    if (carry == nullptr || (n > 0 && (A == nullptr || H == nullptr))) return QSSM_E_NULL;
    if (n < 0 || n_chan < 0 || upto < 0 || upto > n || stride_k < n_chan) return QSSM_E_SHAPE;
    carry_fold_kernel<<<(unsigned)((n_chan + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        A, H, n, stride_k, n_chan, upto, reverse, seed, carry);
    return (int)cudaGetLastError();
}

}  // extern "C"
