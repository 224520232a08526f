// Forward kernels: one warp per chain (scan_fwd_kernel) and the chained single-pass variant for
// launches with few chains (scan_fwd_chained_kernel), plus the descriptor look-back both chained
// kernels share.
#pragma once
#include "qssm_tile.cuh"

namespace qssm {

// ---------------------------------------------------------------------------------------------
// forward:  y = c*h (HAS_C) or y = h; optional fp32 h, optional tile boundary states
// ---------------------------------------------------------------------------------------------
// Tiles have rows of STRIDE lane-vectors and this warp starts at column `col` of a row (32 and 0 when
// the tile belongs to the warp alone).
template <typename Tin, typename Tout, int V, bool HAS_C, bool SAVE_H, bool FULL, int STRIDE = 32>
__device__ __forceinline__ void fwd_batch(const unsigned char* sx, const unsigned char* sa, const unsigned char* sb,
                                          const unsigned char* sc, unsigned char* oy, unsigned char* oh, int lane,
                                          int nrows, float (&h)[V], int col = 0) {
    Vec<Tin, V> xw[TS], aw[TS], bw[TS], cw[HAS_C ? TS : 1];
    const int at = col + lane;
#pragma unroll
    for (int r = 0; r < TS; ++r) {
        xw[r] = reinterpret_cast<const Vec<Tin, V>*>(sx)[r * STRIDE + at];
        aw[r] = reinterpret_cast<const Vec<Tin, V>*>(sa)[r * STRIDE + at];
        bw[r] = reinterpret_cast<const Vec<Tin, V>*>(sb)[r * STRIDE + at];
        if (HAS_C) cw[r] = reinterpret_cast<const Vec<Tin, V>*>(sc)[r * STRIDE + at];
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
        reinterpret_cast<Vec<Tout, V>*>(oy)[r * STRIDE + at] = yw[r];
        if (SAVE_H) reinterpret_cast<Vec<float, V>*>(oh)[r * STRIDE + at] = hw[r];
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
// forward on shared 4-strip tiles (16-bit storage, D > 192, fp32 h stored): a CTA of W = 4 warps scans
// four adjacent channel strips of one batch entry and time range as ONE tile - one bulk copy of 16 rows
// x 512 bytes per input tensor, y and h staged 512 / 1024 bytes wide and stored with one bulk copy each.
// With fp32 h the forward writes 6 of its 14 bytes per element, and like the backward it gains from
// wider copies (B200, cfg1 shape, checkpoint=False: 5.61 TB/s with one warp per CTA, 6.72 TB/s here;
// the plain forward, 20 % writes, is at the copy rate with one warp per CTA and 6 % slower here).
// Thread 0 issues every copy.  Per tile: all warps write their columns of the staging tile, one
// __syncthreads, thread 0 stores.  Before that barrier thread 0 has waited until the store that last
// read the NEXT staging tile is done, so the warps may write it right after the barrier.
// ---------------------------------------------------------------------------------------------
constexpr int WIDE_W = 4;

template <typename Tin, typename Tout, bool HAS_C, bool SAVE_H>
__global__ void __launch_bounds__(32 * WIDE_W) scan_fwd_tile4_kernel(const __grid_constant__ FwdParams p) {
    constexpr int W = WIDE_W;
    constexpr int V = 2;
    constexpr int TB = TS;
    constexpr int DT = 32 * V;
    constexpr int LANES = 32 * W;  // lane-vectors per tile row
    constexpr int NIN = HAS_C ? 4 : 3;
    constexpr int IN_TILE = TB * LANES * V * (int)sizeof(Tin);
    constexpr int OUT_TILE = TB * LANES * V * (int)sizeof(Tout);
    constexpr int HS_TILE = SAVE_H ? TB * LANES * V * 4 : 0;
    constexpr int STAGE = NIN * IN_TILE;
    constexpr int OUTBUF = OUT_TILE + HS_TILE;

    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_fail;
    const Geom& g = p.g;
    const int NS = g.n_stages;
    const int NOUT = g.n_out;  // 2 or 3
    unsigned char* const outbuf = smem + (size_t)NS * STAGE;
    const uint32_t bars = smem_u32(outbuf + (size_t)NOUT * OUTBUF);
    const uint32_t smem_base = smem_u32(smem);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const bool ld_hint = (g.l2_hint & 1) != 0, st_hint = (g.l2_hint & 2) != 0;
    const uint64_t pol = l2_policy_evict_first();

    if (threadIdx.x == 0) {
        s_fail = 0;
        for (int s = 0; s < NS; ++s) mbar_init(bars + 8 * s, 1);
        fence_barrier_init();
    }
    __syncthreads();

    const int n_dgroups = (g.n_dtiles + W - 1) / W;
    const long long n_groups = g.B * g.n_seg * n_dgroups;
    const long long tiles_per_b = (g.L + TS - 1) / TS;
    RingPos pf{0, 0}, cur{0, 0};
    int oslot = 0;
    bool failed = false;
    for (long long gid = blockIdx.x; gid < n_groups && !failed; gid += gridDim.x) {
        const long long dgroup = gid % n_dgroups;
        const long long rest = gid / n_dgroups;
        const int seg = (int)(rest % g.n_seg);
        const long long b = rest / g.n_seg;
        const long long d0 = (dgroup * W + warp) * DT;
        const long long t_begin = (long long)seg * g.seg_rows;
        long long t_end = t_begin + g.seg_rows;
        if (t_end > g.L) t_end = g.L;
        const int n_tiles = t_end > t_begin ? (int)((t_end - t_begin + TB - 1) / TB) : 0;
        const long long d_lane = d0 + (long long)lane * V;

        float h[V];
#pragma unroll
        for (int i = 0; i < V; ++i) h[i] = 0.f;
        if (p.h_in != nullptr) {
            const float* src = p.h_in + (b * g.n_seg + seg) * g.D;
#pragma unroll
            for (int i = 0; i < V; ++i)
                if (d_lane + i < g.D) h[i] = src[d_lane + i];
        }
        float* th_dst = nullptr;
        if (p.tile_h != nullptr) th_dst = p.tile_h + (b * tiles_per_b + t_begin / TS) * g.D + d_lane;

        const int c0 = (int)(dgroup * W * DT), c2 = (int)b;
        int pf_row = (int)t_begin;
        int pf_left = n_tiles;
        auto issue = [&]() {  // thread 0 only; the stage was read by all warps before the last barrier
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
        if (threadIdx.x == 0) {
            for (int k = 0; k < NS - 1 && pf_left > 0; ++k) issue();
        }

        long long t0 = t_begin;
        for (int j = 0; j < n_tiles; ++j, t0 += TB) {
            const unsigned char* st = smem + cur.s * STAGE;
            unsigned char* ob = outbuf + oslot * OUTBUF;
            if (++oslot == NOUT) oslot = 0;
            const int nrows = (int)((t_end - t0) < TB ? (t_end - t0) : TB);
            if (threadIdx.x == 0 && pf_left > 0) issue();
            bool ok = mbar_wait_bounded(bars + 8 * cur.s, cur.phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) s_fail = 1;
            } else {
                if (th_dst != nullptr) {
#pragma unroll
                    for (int i = 0; i < V; ++i)
                        if (d_lane + i < g.D) th_dst[i] = h[i];
                    th_dst += g.D;
                }
                if (nrows >= TS)
                    fwd_batch<Tin, Tout, V, HAS_C, SAVE_H, true, LANES>(st, st + IN_TILE, st + 2 * IN_TILE,
                                                                        st + 3 * IN_TILE, ob, ob + OUT_TILE, lane, TS, h,
                                                                        warp * 32);
                else
                    fwd_batch<Tin, Tout, V, HAS_C, SAVE_H, false, LANES>(st, st + IN_TILE, st + 2 * IN_TILE,
                                                                         st + 3 * IN_TILE, ob, ob + OUT_TILE, lane,
                                                                         nrows, h, warp * 32);
            }
            fence_proxy_async();
            if (threadIdx.x == 0) {  // the staging tile of the next iteration is free once this returns
                if (NOUT == 2) tma_wait_read<0>();
                else tma_wait_read<1>();
            }
            __syncthreads();
            if (s_fail != 0) {
                failed = true;
                break;
            }
            if (threadIdx.x == 0) {
                tma_st(&p.y.map, smem_u32(ob), c0, (int)t0, c2, st_hint, pol);
                if (SAVE_H) tma_st(&p.hs.map, smem_u32(ob + OUT_TILE), c0, (int)t0, c2, st_hint, pol);
                tma_commit();
            }
            cur.advance(NS);
        }
        if (failed) break;
        if (p.h_last != nullptr && seg == g.n_seg - 1) {
            float* dst = p.h_last + b * g.D;
#pragma unroll
            for (int i = 0; i < V; ++i)
                if (d_lane + i < g.D) dst[d_lane + i] = h[i];
        }
    }
    if (threadIdx.x == 0) {
        tma_wait_all();
        if (failed) report(g.status, QSSM_S_TMA_TIMEOUT);
    }
}

// Before chunk k (processing order) writes its descriptor into slot k mod slots it makes sure the
// previous owner of that slot, chunk k - slots, is no longer needed: once chunk k - slots + 1 has
// published its inclusive state, every later chunk finds that state (or a nearer one) before it would
// look at chunk k - slots.  Almost always true at once; the wait is bounded like every other.
__device__ __forceinline__ bool chained_slot_free(const float4* cdesc, int slots, long long k, int lane,
                                                  unsigned long long wait_ns) {
    const long long j = k - slots + 1;
    if (j < 0) return true;
    const float4* dj = cdesc + (size_t)(j & (slots - 1)) * 96 + 64 + lane;
    const unsigned int want = (unsigned int)(j + 1);
    if (__all_sync(0xffffffffu, __float_as_uint(__ldcg(dj).x) == want)) return true;
    const unsigned long long start = global_timer_ns();
    for (unsigned int it = 0;; ++it) {
        if (__all_sync(0xffffffffu, __float_as_uint(__ldcg(dj).x) == want)) return true;
        __nanosleep(100);
        if ((it & 255u) == 255u && __any_sync(0xffffffffu, global_timer_ns() - start > wait_ns)) return false;
    }
}

// The same check split in two so that its round trip to L2 overlaps the first pass of the chunk: the word is
// asked for when the chunk starts and looked at when the aggregate is ready (it nearly always says "free").
__device__ __forceinline__ float chained_slot_peek(const float4* cdesc, int slots, long long k, int lane) {
    const long long j = k - slots + 1;
    if (j < 0) return 0.f;
    return __ldcg(cdesc + (size_t)(j & (slots - 1)) * 96 + 64 + lane).x;
}
__device__ __forceinline__ bool chained_slot_free_peeked(float peeked, const float4* cdesc, int slots, long long k,
                                                         int lane, unsigned long long wait_ns) {
    const long long j = k - slots + 1;
    if (j < 0) return true;
    if (__all_sync(0xffffffffu, __float_as_uint(peeked) == (unsigned int)(j + 1))) return true;
    return chained_slot_free(cdesc, slots, k, lane, wait_ns);
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
// Waits are bounded (`wait_ns`, two seconds by default); false means a predecessor never published.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ bool chained_lookback(const float4* cdesc, int slots, long long k, int lane,
                                                 unsigned long long wait_ns, float (&h)[2]) {
    constexpr int WIN = 8;
    bool ok = true;
    long long js = -1;      // nearest predecessor whose inclusive end state is known
    long long folded = 0;   // aggregates of chunks js+1 .. folded-1 are already applied to h
    // A slot whose tag is LARGER than the one wanted has been taken over by a later chunk of the chain.
    // That happens only after the old owner's successor has published its inclusive state
    // (chained_slot_free), so a nearer inclusive state exists by now: start over from k - 1 with fresh
    // loads instead of waiting for a tag that will never come back.  Every restart finds the chain further
    // along; the count is bounded all the same.
    int restarts = 0;
restart:
    js = -1;
    folded = 0;
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
        bool reused = false;
#pragma unroll
        for (int q = 0; q < WIN; ++q) {
            const long long j = top - q;
            if (j < 0 || js >= 0 || !ok || reused) continue;
            const unsigned int want = (unsigned int)(j + 1);
            const float4* dj = cdesc + (size_t)(j & (slots - 1)) * 96;
            bool inc = __all_sync(0xffffffffu, __float_as_uint(wi[q].x) == want);
            bool agg = __all_sync(0xffffffffu, __float_as_uint(wa[q].x) == want && __float_as_uint(wh[q].x) == want);
            if (!inc && !agg) {  // nothing published yet: poll this chunk
                const unsigned long long start = global_timer_ns();
                for (unsigned int it = 0; ok; ++it) {
                    if (__any_sync(0xffffffffu, __float_as_uint(wi[q].x) > want || __float_as_uint(wa[q].x) > want ||
                                                    __float_as_uint(wh[q].x) > want)) {
                        reused = true;
                        break;
                    }
                    wi[q] = __ldcg(dj + 64 + lane);
                    wa[q] = __ldcg(dj + lane);
                    wh[q] = __ldcg(dj + 32 + lane);
                    inc = __all_sync(0xffffffffu, __float_as_uint(wi[q].x) == want);
                    agg = __all_sync(0xffffffffu,
                                     __float_as_uint(wa[q].x) == want && __float_as_uint(wh[q].x) == want);
                    if (inc || agg) break;
                    __nanosleep(100);
                    if ((it & 255u) == 255u) {
                        const bool late = global_timer_ns() - start > wait_ns;
                        if (__any_sync(0xffffffffu, late)) ok = false;
                    }
                }
            }
            if (ok && !reused && inc) {
                h[0] = wi[q].y;
                h[1] = wi[q].z;
                js = j;
            }
        }
        if (reused) {
            if (++restarts > 64) return false;
            goto restart;
        }
        if (ok && js >= 0) {  // the aggregates of this window that lie after js are in registers: apply them now
            const int qf = (int)(top - js);
#pragma unroll
            for (int q = WIN - 1; q >= 0; --q) {
                if (q < qf) {
                    h[0] = fmaf(wa[q].y, h[0], wh[q].y);
                    h[1] = fmaf(wa[q].z, h[1], wh[q].z);
                }
            }
            folded = top + 1;
        }
    }
    if (!ok) return false;
    // forward through the aggregates of the nearer windows, chunks folded .. k-1 (all seen published above)
    for (long long base = folded; base < k; base += WIN) {
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
        // these chunks were seen published above, but a slot may have changed hands since: check the tags again
        bool stale = false;
#pragma unroll
        for (int q = 0; q < WIN; ++q) {
            if (base + q < k) {
                const unsigned int want = (unsigned int)(base + q + 1);
                stale = stale || __float_as_uint(wa[q].x) != want || __float_as_uint(wh[q].x) != want;
            }
        }
        if (__any_sync(0xffffffffu, stale)) {
            if (++restarts > 64) return false;
            goto restart;
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
        float4* const cdesc = reinterpret_cast<float4*>(cp.desc) + (size_t)c * cp.slots * 96;
        const float slot_word = chained_slot_peek(cdesc, cp.slots, k, lane);

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
        float4* const mydesc = cdesc + (size_t)(k & (cp.slots - 1)) * 96;
        const float mytag = __uint_as_float((unsigned int)(k + 1));
        float h[V];
        if (k == 0) {
#pragma unroll
            for (int i = 0; i < V; ++i)
                h[i] = (p.h_in != nullptr && d_lane + i < g.D) ? p.h_in[b * g.D + d_lane + i] : 0.f;
        } else {
            ok = chained_slot_free_peeked(slot_word, cdesc, cp.slots, k, lane, cp.wait_ns);
            if (!ok) break;
            __stcg(mydesc + lane, make_float4(mytag, A[0], A[1], 0.f));
            __stcg(mydesc + 32 + lane, make_float4(mytag, H[0], H[1], 0.f));
            ok = chained_lookback(cdesc, cp.slots, k, lane, cp.wait_ns, h);
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

}  // namespace qssm
