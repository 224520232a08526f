// Segment aggregates and the per-channel scans of aggregates (segment seeds, rank folds).
#pragma once
#include "qssm_tile.cuh"

namespace qssm {

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
static __global__ void seg_carry_kernel(const float* __restrict__ A, const float* __restrict__ H,
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

static __global__ void carry_fold_kernel(const float* __restrict__ A, const float* __restrict__ H, long long n,
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

}  // namespace qssm
