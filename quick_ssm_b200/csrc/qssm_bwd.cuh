// Backward kernels: one warp per chain with in-place gradient stores (scan_bwd_kernel), the chained
// single-pass variant (scan_bwd_chained_kernel) and four strips per CTA on shared 512-byte-wide
// tiles (scan_bwd_tile4_kernel).
#pragma once
#include "qssm_fwd.cuh"

namespace qssm {

// ---------------------------------------------------------------------------------------------
// backward: reverse scan of dh with h rebuilt per 16-row batch (tile_h) or read (h_saved).
// The carry between batches is G(t) = a(t) * dh(t), so no halo row of `a` is needed.
// Gradients overwrite the shared-memory slots of x, a, b, c and are stored from there.
// ---------------------------------------------------------------------------------------------
// Results go to (ox, oa, ob, oc), tiles whose rows hold OSTRIDE lane-vectors; `ocol` is this warp's first
// column in such a row.  In-place operation passes the input tiles again with OSTRIDE = 32, ocol = 0.
// Input tiles have rows of ISTRIDE lane-vectors and this warp starts at column `icol` of a row
// (32 and 0 when the tile belongs to the warp alone).
template <typename Tin, typename Tdy, int V, bool SAVED_H, bool FULL, int OSTRIDE = 32, int ISTRIDE = 32>
__device__ __forceinline__ void bwd_batch(const unsigned char* sx, const unsigned char* sa, const unsigned char* sb,
                                          const unsigned char* sc, const unsigned char* sg, const unsigned char* sh,
                                          unsigned char* ox, unsigned char* oa, unsigned char* ob, unsigned char* oc,
                                          int ocol, int lane, int nrows, bool first_rows, const float* h_in_lane,
                                          long long d_lane, long long D, float (&G)[V], int icol = 0) {
    Vec<Tin, V> xw[TS], aw[TS], bw[TS], cw[TS];
    Vec<Tdy, V> gw[TS];
#pragma unroll
    for (int r = 0; r < TS; ++r) {
        xw[r] = reinterpret_cast<const Vec<Tin, V>*>(sx)[(r) * ISTRIDE + icol + lane];
        aw[r] = reinterpret_cast<const Vec<Tin, V>*>(sa)[(r) * ISTRIDE + icol + lane];
        bw[r] = reinterpret_cast<const Vec<Tin, V>*>(sb)[(r) * ISTRIDE + icol + lane];
    }
    // h(t0-1 .. t0+TS-1): entry 0 is the state before the batch
    float hreg[TS + 1][V];
    if (SAVED_H) {
#pragma unroll
        for (int r = 0; r <= TS; ++r) {
            const Vec<float, V> w = reinterpret_cast<const Vec<float, V>*>(sh)[(r) * ISTRIDE + icol + lane];
            unpack<float, V>(w, hreg[r]);
        }
        if (first_rows && h_in_lane != nullptr) {
#pragma unroll
            for (int i = 0; i < V; ++i) hreg[0][i] = (d_lane + i < D) ? h_in_lane[i] : 0.f;
        }
    } else {
        const Vec<float, V> w = reinterpret_cast<const Vec<float, V>*>(sh)[(0) * ISTRIDE + icol + lane];
        unpack<float, V>(w, hreg[0]);
    }
#pragma unroll
    for (int r = 0; r < TS; ++r) {
        cw[r] = reinterpret_cast<const Vec<Tin, V>*>(sc)[(r) * ISTRIDE + icol + lane];
        gw[r] = reinterpret_cast<const Vec<Tdy, V>*>(sg)[(r) * ISTRIDE + icol + lane];
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
        float4* const cdesc = reinterpret_cast<float4*>(cp.desc) + (size_t)c * cp.slots * 96;
        const float slot_word = chained_slot_peek(cdesc, cp.slots, kk, lane);

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
        float4* const mydesc = cdesc + (size_t)(kk & (cp.slots - 1)) * 96;
        const float mytag = __uint_as_float((unsigned int)(kk + 1));
        float G[V];
        if (kk == 0) {
#pragma unroll
            for (int i = 0; i < V; ++i)
                G[i] = (p.g_in != nullptr && d_lane + i < g.D) ? p.g_in[b * g.D + d_lane + i] : 0.f;
        } else {
            ok = chained_slot_free_peeked(slot_word, cdesc, cp.slots, kk, lane, cp.wait_ns);
            if (!ok) break;
            __stcg(mydesc + lane, make_float4(mytag, P[0], P[1], 0.f));
            __stcg(mydesc + 32 + lane, make_float4(mytag, Q[0], Q[1], 0.f));
            ok = chained_lookback(cdesc, cp.slots, kk, lane, cp.wait_ns, G);
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
// backward on shared 4-strip tiles (16-bit storage, D > 192): a CTA of W = 4 warps scans four adjacent
// channel strips of the same batch entry and time range as ONE tile - one bulk copy of 16 rows x
// 512 bytes per tensor in, gradients written in place, one bulk copy per gradient tensor out.
// The write-heavy backward gains from that contiguity: on B200, cfg1, one warp per CTA with
// 128-byte-wide copies moves 5.9 TB/s, four strips with only the stores combined 6.17 TB/s, this
// kernel 6.41 TB/s (on a layout whose strips are contiguous in memory, D = 64, the narrow kernel also
// reaches 6.46 TB/s).  One ring of stages and one mbarrier per stage for the whole CTA; thread 0
// issues every copy; one __syncthreads per tile orders "four strips written" before the store.
// ---------------------------------------------------------------------------------------------
template <typename Tin, typename Tdy, bool SAVED_H>
__global__ void __launch_bounds__(32 * WIDE_W) scan_bwd_tile4_kernel(const __grid_constant__ BwdParams p) {
    constexpr int W = WIDE_W;
    constexpr int V = 2;
    constexpr int TB = TS;
    constexpr int DT = 32 * V;
    constexpr int LANES = 32 * W;  // lane-vectors per tile row
    constexpr int IN_TILE = TB * LANES * V * (int)sizeof(Tin);
    constexpr int DY_TILE = TB * LANES * V * (int)sizeof(Tdy);
    constexpr int H_ROW = LANES * V * 4;
    constexpr int H_TILE = SAVED_H ? (TB + 1) * H_ROW : H_ROW;
    constexpr int STAGE = 4 * IN_TILE + DY_TILE + H_TILE;
    constexpr int OFF_DY = 4 * IN_TILE;
    constexpr int OFF_H = OFF_DY + DY_TILE;

    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_fail;
    const Geom& g = p.g;
    const int NS = g.n_stages;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t bars = smem_u32(smem + (size_t)NS * STAGE);
    const uint32_t smem_base = smem_u32(smem);
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
    const int PF = NS > 2 ? NS - 2 : 1;
    RingPos pf{0, 0}, cur{0, 0};
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
        const int n_tiles = (int)((t_end - t_begin + TB - 1) / TB);
        const long long d_lane = d0 + (long long)lane * V;

        float G[V];
#pragma unroll
        for (int i = 0; i < V; ++i) G[i] = 0.f;
        if (p.g_in != nullptr) {
            const float* src = p.g_in + (b * g.n_seg + seg) * g.D;
#pragma unroll
            for (int i = 0; i < V; ++i)
                if (d_lane + i < g.D) G[i] = src[d_lane + i];
        }
        const float* h_in_lane = (SAVED_H && p.h_in != nullptr) ? p.h_in + b * g.D + d_lane : nullptr;

        const int c0 = (int)(dgroup * W * DT), c2 = (int)b;
        int pf_row = (int)(t_begin + (long long)(n_tiles - 1) * TB);
        int pf_left = n_tiles;
        auto issue = [&]() {  // thread 0 only
            const uint32_t st = smem_base + pf.s * STAGE;
            const uint32_t bar = bars + 8 * pf.s;
            // gradients are stored from the stage: it is refilled only when that store has drained
            if (NS > 2) tma_wait_read<1>();
            else tma_wait_read<0>();
            fence_proxy_async();
            mbar_expect_tx(bar, STAGE);
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
        if (threadIdx.x == 0) {
            for (int k = 0; k < PF && pf_left > 0; ++k) issue();
        }

        long long t0 = t_begin + (long long)(n_tiles - 1) * TB;
        for (int j = 0; j < n_tiles; ++j, t0 -= TB) {
            unsigned char* st = smem + cur.s * STAGE;
            const int nrows = (int)((t_end - t0) < TB ? (t_end - t0) : TB);
            if (threadIdx.x == 0 && pf_left > 0) issue();
            bool ok = mbar_wait_bounded(bars + 8 * cur.s, cur.phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) s_fail = 1;
            } else {
                unsigned char* sx = st;
                unsigned char* sa = st + IN_TILE;
                unsigned char* sb = st + 2 * IN_TILE;
                unsigned char* sc = st + 3 * IN_TILE;
                const bool first_rows = (t0 == 0);
                if (nrows >= TS)
                    bwd_batch<Tin, Tdy, V, SAVED_H, true, LANES, LANES>(sx, sa, sb, sc, st + OFF_DY, st + OFF_H, sx, sa,
                                                                        sb, sc, warp * 32, lane, TS, first_rows,
                                                                        h_in_lane, d_lane, g.D, G, warp * 32);
                else
                    bwd_batch<Tin, Tdy, V, SAVED_H, false, LANES, LANES>(sx, sa, sb, sc, st + OFF_DY, st + OFF_H, sx,
                                                                         sa, sb, sc, warp * 32, lane, nrows, first_rows,
                                                                         h_in_lane, d_lane, g.D, G, warp * 32);
            }
            fence_proxy_async();
            __syncthreads();
            if (s_fail != 0) {
                failed = true;
                break;
            }
            if (threadIdx.x == 0) {
                const uint32_t sst = smem_base + cur.s * STAGE;
                tma_st(&p.dx.map, sst + 0 * IN_TILE, c0, (int)t0, c2, st_hint, pol);
                tma_st(&p.da.map, sst + 1 * IN_TILE, c0, (int)t0, c2, st_hint, pol);
                tma_st(&p.db.map, sst + 2 * IN_TILE, c0, (int)t0, c2, st_hint, pol);
                tma_st(&p.dc.map, sst + 3 * IN_TILE, c0, (int)t0, c2, st_hint, pol);
                tma_commit();
            }
            cur.advance(NS);
        }
        if (failed) break;
        if (p.g_first != nullptr && seg == 0) {
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

}  // namespace qssm
