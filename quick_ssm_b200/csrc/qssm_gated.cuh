// Scan with the gate activations of the SSM layer fused into its loads and stores.
//
// The layer that calls the scan (reference: quick_ssm/layers.py:76-104) builds the four scan inputs
// from five projection outputs with element-wise kernels:
//     a = sigmoid(pa)            decay                 x = px               drive
//     b = sigmoid(pd)            input gate            c = silu(pc1) * pc2  output gate (SwiGLU)
// each rounded to the layer's compute dtype (.to(compute_dtype), layers.py:85-88).  Those kernels
// move several times the bytes of the scan itself.  Here the scan kernels read the five
// pre-activations directly, apply the activations and the rounding in registers, and the backward
// returns the gradients of the pre-activations:
//     d pa  = da * a(1-a)        d px = dx             d pd = db * b(1-b)
//     d pc1 = dc * pc2 * s(1 + pc1(1-s)),  s = sigmoid(pc1)          d pc2 = dc * silu(pc1)
// where (dx, da, db, dc) are the scan's gradients rounded to the compute dtype, as the unfused path
// rounds them (the scan returns them in the dtype of its inputs).
//
// One warp per chain, tiles of 16 rows, ring of TMA stages, persistent over chains - the structure
// of scan_fwd_kernel / scan_bwd_kernel.  The backward stores the five gradients from the stage in
// place of the five inputs.
#pragma once
#include "qssm_tile.cuh"

namespace qssm {

struct GatedFwdParams {
    TensorDesc pa, px, pc1, pc2, pd, y;
    float* tile_h;       // [B, ceil(L/TS), D] or NULL
    const float* h_in;   // [B, D] or NULL
    float* h_last;       // [B, D] or NULL
    Geom g;
};

struct GatedBwdParams {
    TensorDesc pa, px, pc1, pc2, pd, dy, th;
    TensorDesc dpa, dpx, dpc1, dpc2, dpd;
    const float* g_in;   // [B, D] or NULL
    float* g_first;      // [B, D] or NULL
    Geom g;
};

// Round-trip of a lane's V values through the layer's compute dtype (identity for float); two
// 16-bit values share one packed conversion.
template <typename Tg, int V> __device__ __forceinline__ void gate_round(float (&v)[V]) {
    const Vec<Tg, V> w = pack<Tg, V>(v);
    unpack<Tg, V>(w, v);
}
template <> __device__ __forceinline__ void gate_round<float, 1>(float (&)[1]) {}
template <> __device__ __forceinline__ void gate_round<float, 2>(float (&)[2]) {}

// sigmoid.  With 16-bit gates the result is rounded to 8 or 11 significant bits right away, so the
// hardware tanh approximation (relative error about 2^-11) is used: sigmoid(v) = 0.5 tanh(v/2) + 0.5,
// three instructions instead of an exponential and a division.  fp32 gates take the accurate form.
template <typename Tg> __device__ __forceinline__ float sigmoid_g(float v) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * v));
    return fmaf(0.5f, t, 0.5f);
}
template <> __device__ __forceinline__ float sigmoid_g<float>(float v) { return __frcp_rn(1.f + expf(-v)); }

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
template <typename Tin, typename Tg, typename Tout, int V>
__global__ void __launch_bounds__(32) gated_fwd_kernel(const __grid_constant__ GatedFwdParams p) {
    constexpr int DT = 32 * V;
    constexpr int TB = TS;
    constexpr int IN_ROW = 32 * V * (int)sizeof(Tin);
    constexpr int OUT_ROW = 32 * V * (int)sizeof(Tout);
    constexpr int IN_TILE = TB * IN_ROW;
    constexpr int OUT_TILE = TB * OUT_ROW;
    constexpr int STAGE = 5 * IN_TILE;

    extern __shared__ __align__(128) unsigned char smem[];
    const Geom& g = p.g;
    const int NS = g.n_stages;
    const int NOUT = g.n_out;
    unsigned char* const outbuf = smem + NS * STAGE;
    const uint32_t bars = smem_u32(outbuf + NOUT * OUT_TILE);
    const uint32_t smem_base = smem_u32(smem);
    const int lane = threadIdx.x;

    if (lane == 0) {
        for (int s = 0; s < NS; ++s) mbar_init(bars + 8 * s, 1);
        fence_barrier_init();
    }
    __syncwarp();

    bool ok = true;
    RingPos pf{0, 0}, cur{0, 0};
    int oslot = 0;
    for (long long chain_id = blockIdx.x; chain_id < g.n_chains && ok; chain_id += gridDim.x) {
        const Chain ch = chain_of(g, chain_id, DT, TB);
        if (ch.empty) continue;
        const long long d_lane = ch.d0 + (long long)lane * V;
        float h[V];
#pragma unroll
        for (int i = 0; i < V; ++i) h[i] = (p.h_in != nullptr && d_lane + i < g.D) ? p.h_in[ch.b * g.D + d_lane + i] : 0.f;
        float* th_dst = nullptr;
        if (p.tile_h != nullptr) th_dst = p.tile_h + (ch.b * ((g.L + TS - 1) / TS) + ch.t_begin / TS) * g.D + d_lane;

        const int c0 = (int)ch.d0, c2 = (int)ch.b;
        int pf_row = (int)ch.t_begin;
        int pf_left = ch.n_tiles;
        auto issue = [&]() {
            const uint32_t st = smem_base + pf.s * STAGE;
            const uint32_t bar = bars + 8 * pf.s;
            fence_proxy_async();
            mbar_expect_tx(bar, STAGE);
            tma_load_3d(st + 0 * IN_TILE, &p.pa.map, bar, c0, pf_row, c2);
            tma_load_3d(st + 1 * IN_TILE, &p.px.map, bar, c0, pf_row, c2);
            tma_load_3d(st + 2 * IN_TILE, &p.pc1.map, bar, c0, pf_row, c2);
            tma_load_3d(st + 3 * IN_TILE, &p.pc2.map, bar, c0, pf_row, c2);
            tma_load_3d(st + 4 * IN_TILE, &p.pd.map, bar, c0, pf_row, c2);
            pf.advance(NS);
            pf_row += TB;
            --pf_left;
        };
        if (lane == 0) {
            for (int k = 0; k < NS - 1 && pf_left > 0; ++k) issue();
        }

        long long t0 = ch.t_begin;
        for (int j = 0; j < ch.n_tiles; ++j, t0 += TB) {
            const unsigned char* st = smem + cur.s * STAGE;
            unsigned char* ob = outbuf + oslot * OUT_TILE;
            if (++oslot == NOUT) oslot = 0;
            const int nrows = (int)((ch.t_end - t0) < TB ? (ch.t_end - t0) : TB);
            if (lane == 0) {
                if (pf_left > 0) issue();
                if (NOUT == 2) tma_wait_read<1>();
                else tma_wait_read<2>();
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
            Vec<Tin, V> w0[TS], w1[TS], w2[TS], w3[TS], w4[TS];
#pragma unroll
            for (int r = 0; r < TS; ++r) {
                w0[r] = tile_raw<Tin, V>(st + 0 * IN_TILE, r, lane);
                w1[r] = tile_raw<Tin, V>(st + 1 * IN_TILE, r, lane);
                w2[r] = tile_raw<Tin, V>(st + 2 * IN_TILE, r, lane);
                w3[r] = tile_raw<Tin, V>(st + 3 * IN_TILE, r, lane);
                w4[r] = tile_raw<Tin, V>(st + 4 * IN_TILE, r, lane);
            }
            Vec<Tout, V> yw[TS];
#pragma unroll
            for (int r = 0; r < TS; ++r) {
                float fa[V], fx[V], f1[V], f2[V], fd[V], yv[V];
                unpack<Tin, V>(w0[r], fa);
                unpack<Tin, V>(w1[r], fx);
                unpack<Tin, V>(w2[r], f1);
                unpack<Tin, V>(w3[r], f2);
                unpack<Tin, V>(w4[r], fd);
                float a[V], b[V], c[V];
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    a[i] = sigmoid_g<Tg>(fa[i]);
                    b[i] = sigmoid_g<Tg>(fd[i]);
                    c[i] = f1[i] * sigmoid_g<Tg>(f1[i]) * f2[i];
                }
                gate_round<Tg, V>(a);
                gate_round<Tg, V>(b);
                gate_round<Tg, V>(c);
                gate_round<Tg, V>(fx);
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    if (r < nrows) h[i] = fmaf(a[i], h[i], b[i] * fx[i]);
                    yv[i] = c[i] * h[i];
                }
                yw[r] = pack<Tout, V>(yv);
            }
#pragma unroll
            for (int r = 0; r < TS; ++r) tile_put<Tout, V>(ob, r, lane, yw[r]);
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                tma_store_3d(&p.y.map, smem_u32(ob), c0, (int)t0, c2);
                tma_commit();
            }
            __syncwarp();
            cur.advance(NS);
        }
        if (!ok) break;
        if (p.h_last != nullptr) {
#pragma unroll
            for (int i = 0; i < V; ++i)
                if (d_lane + i < g.D) p.h_last[ch.b * g.D + d_lane + i] = h[i];
        }
        if (lane == 0) tma_wait_read<0>();
        __syncwarp();
    }
    if (lane == 0) {
        tma_wait_all();
        if (!ok) report(g.status, QSSM_S_TMA_TIMEOUT);
    }
}

// ---------------------------------------------------------------------------------------------
// backward (h rebuilt from tile_h; gradients of the five pre-activations stored from the stage)
// ---------------------------------------------------------------------------------------------
template <typename Tin, typename Tg, typename Tdy, int V>
__global__ void __launch_bounds__(32) gated_bwd_kernel(const __grid_constant__ GatedBwdParams p) {
    constexpr int DT = 32 * V;
    constexpr int TB = TS;
    constexpr int IN_ROW = 32 * V * (int)sizeof(Tin);
    constexpr int DY_ROW = 32 * V * (int)sizeof(Tdy);
    constexpr int H_ROW = 32 * V * 4;
    constexpr int IN_TILE = TB * IN_ROW;
    constexpr int DY_TILE = TB * DY_ROW;
    constexpr int H_SLOT = ((H_ROW + 127) / 128) * 128;
    constexpr int STAGE = 5 * IN_TILE + DY_TILE + H_SLOT;
    constexpr int OFF_DY = 5 * IN_TILE;
    constexpr int OFF_H = OFF_DY + DY_TILE;

    extern __shared__ __align__(128) unsigned char smem[];
    const Geom& g = p.g;
    const int NS = g.n_stages;
    const uint32_t bars = smem_u32(smem + NS * STAGE);
    const uint32_t smem_base = smem_u32(smem);
    const int lane = threadIdx.x;

    if (lane == 0) {
        for (int s = 0; s < NS; ++s) mbar_init(bars + 8 * s, 1);
        fence_barrier_init();
    }
    __syncwarp();

    bool ok = true;
    RingPos pf{0, 0}, cur{0, 0};
    const int PF = NS > 2 ? NS - 2 : 1;
    for (long long chain_id = blockIdx.x; chain_id < g.n_chains && ok; chain_id += gridDim.x) {
        const Chain ch = chain_of(g, chain_id, DT, TB);
        if (ch.empty) continue;
        const long long d_lane = ch.d0 + (long long)lane * V;
        float G[V];
#pragma unroll
        for (int i = 0; i < V; ++i) G[i] = (p.g_in != nullptr && d_lane + i < g.D) ? p.g_in[ch.b * g.D + d_lane + i] : 0.f;

        const int c0 = (int)ch.d0, c2 = (int)ch.b;
        int pf_row = (int)(ch.t_begin + (long long)(ch.n_tiles - 1) * TB);
        int pf_left = ch.n_tiles;
        auto issue = [&]() {
            const uint32_t st = smem_base + pf.s * STAGE;
            const uint32_t bar = bars + 8 * pf.s;
            if (NS > 2) tma_wait_read<1>();  // the gradient store issued from this stage has drained
            else tma_wait_read<0>();
            fence_proxy_async();
            mbar_expect_tx(bar, 5 * IN_TILE + DY_TILE + H_ROW);
            tma_load_3d(st + 0 * IN_TILE, &p.pa.map, bar, c0, pf_row, c2);
            tma_load_3d(st + 1 * IN_TILE, &p.px.map, bar, c0, pf_row, c2);
            tma_load_3d(st + 2 * IN_TILE, &p.pc1.map, bar, c0, pf_row, c2);
            tma_load_3d(st + 3 * IN_TILE, &p.pc2.map, bar, c0, pf_row, c2);
            tma_load_3d(st + 4 * IN_TILE, &p.pd.map, bar, c0, pf_row, c2);
            tma_load_3d(st + OFF_DY, &p.dy.map, bar, c0, pf_row, c2);
            tma_load_3d(st + OFF_H, &p.th.map, bar, c0, pf_row / TS, c2);
            pf.advance(NS);
            pf_row -= TB;
            --pf_left;
        };
        if (lane == 0) {
            for (int k = 0; k < PF && pf_left > 0; ++k) issue();
        }

        long long t0 = ch.t_begin + (long long)(ch.n_tiles - 1) * TB;
        for (int j = 0; j < ch.n_tiles; ++j, t0 -= TB) {
            unsigned char* st = smem + cur.s * STAGE;
            const int nrows = (int)((ch.t_end - t0) < TB ? (ch.t_end - t0) : TB);
            if (lane == 0 && pf_left > 0) issue();
            ok = mbar_wait_bounded(bars + 8 * cur.s, cur.phase);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;

            Vec<Tin, V> w0[TS], w1[TS], w2[TS], w3[TS], w4[TS];
            Vec<Tdy, V> gw[TS];
#pragma unroll
            for (int r = 0; r < TS; ++r) {
                w0[r] = tile_raw<Tin, V>(st + 0 * IN_TILE, r, lane);
                w1[r] = tile_raw<Tin, V>(st + 1 * IN_TILE, r, lane);
                w4[r] = tile_raw<Tin, V>(st + 4 * IN_TILE, r, lane);
            }
            // h(t0-1 .. t0+TS-1) rebuilt from the boundary state with the rounded gates; the sigmoids of
            // the decay and the input gate are kept for the second loop (unrounded: their derivatives)
            float hreg[TS + 1][V];
            float sa[TS][V], sd[TS][V];
            unpack<float, V>(tile_raw<float, V>(st + OFF_H, 0, lane), hreg[0]);
#pragma unroll
            for (int r = 0; r < TS; ++r) {
                float fa[V], fx[V], fd[V], a[V], b[V];
                unpack<Tin, V>(w0[r], fa);
                unpack<Tin, V>(w1[r], fx);
                unpack<Tin, V>(w4[r], fd);
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    sa[r][i] = a[i] = sigmoid_g<Tg>(fa[i]);
                    sd[r][i] = b[i] = sigmoid_g<Tg>(fd[i]);
                }
                gate_round<Tg, V>(a);
                gate_round<Tg, V>(b);
                gate_round<Tg, V>(fx);
#pragma unroll
                for (int i = 0; i < V; ++i) hreg[r + 1][i] = fmaf(a[i], hreg[r][i], b[i] * fx[i]);
            }
#pragma unroll
            for (int r = 0; r < TS; ++r) {
                w2[r] = tile_raw<Tin, V>(st + 2 * IN_TILE, r, lane);
                w3[r] = tile_raw<Tin, V>(st + 3 * IN_TILE, r, lane);
                gw[r] = tile_raw<Tdy, V>(st + OFF_DY, r, lane);
            }
#pragma unroll
            for (int r = TS - 1; r >= 0; --r) {
                float fx[V], f1[V], f2[V], gy[V];
                unpack<Tin, V>(w1[r], fx);
                unpack<Tin, V>(w2[r], f1);
                unpack<Tin, V>(w3[r], f2);
                unpack<Tdy, V>(gw[r], gy);
                float a[V], b[V], c[V], s1[V], silu[V];
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    a[i] = sa[r][i];
                    b[i] = sd[r][i];
                    s1[i] = sigmoid_g<Tg>(f1[i]);
                    silu[i] = f1[i] * s1[i];
                    c[i] = silu[i] * f2[i];
                }
                gate_round<Tg, V>(a);
                gate_round<Tg, V>(b);
                gate_round<Tg, V>(c);
                gate_round<Tg, V>(fx);
                // the scan's gradients, rounded as the unfused path returns them
                float dx[V], db[V], da[V], dc[V];
                const bool live = r < nrows;
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    const float dh = fmaf(c[i], gy[i], G[i]);
                    dx[i] = dh * b[i];
                    db[i] = dh * fx[i];
                    da[i] = dh * hreg[r][i];
                    dc[i] = gy[i] * hreg[r + 1][i];
                    if (live) G[i] = a[i] * dh;
                }
                gate_round<Tg, V>(dx);
                gate_round<Tg, V>(db);
                gate_round<Tg, V>(da);
                gate_round<Tg, V>(dc);
                float o0[V], o2[V], o3[V], o4[V];
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    o0[i] = da[i] * sa[r][i] * (1.f - sa[r][i]);
                    o2[i] = dc[i] * f2[i] * s1[i] * fmaf(f1[i], 1.f - s1[i], 1.f);
                    o3[i] = dc[i] * silu[i];
                    o4[i] = db[i] * sd[r][i] * (1.f - sd[r][i]);
                }
                w0[r] = pack<Tin, V>(o0);
                w1[r] = pack<Tin, V>(dx);
                w2[r] = pack<Tin, V>(o2);
                w3[r] = pack<Tin, V>(o3);
                w4[r] = pack<Tin, V>(o4);
            }
#pragma unroll
            for (int r = 0; r < TS; ++r) {
                tile_put<Tin, V>(st + 0 * IN_TILE, r, lane, w0[r]);
                tile_put<Tin, V>(st + 1 * IN_TILE, r, lane, w1[r]);
                tile_put<Tin, V>(st + 2 * IN_TILE, r, lane, w2[r]);
                tile_put<Tin, V>(st + 3 * IN_TILE, r, lane, w3[r]);
                tile_put<Tin, V>(st + 4 * IN_TILE, r, lane, w4[r]);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                const uint32_t sst = smem_base + cur.s * STAGE;
                tma_store_3d(&p.dpa.map, sst + 0 * IN_TILE, c0, (int)t0, c2);
                tma_store_3d(&p.dpx.map, sst + 1 * IN_TILE, c0, (int)t0, c2);
                tma_store_3d(&p.dpc1.map, sst + 2 * IN_TILE, c0, (int)t0, c2);
                tma_store_3d(&p.dpc2.map, sst + 3 * IN_TILE, c0, (int)t0, c2);
                tma_store_3d(&p.dpd.map, sst + 4 * IN_TILE, c0, (int)t0, c2);
                tma_commit();
            }
            __syncwarp();
            cur.advance(NS);
        }
        if (!ok) break;
        if (p.g_first != nullptr) {
#pragma unroll
            for (int i = 0; i < V; ++i)
                if (d_lane + i < g.D) p.g_first[ch.b * g.D + d_lane + i] = G[i];
        }
        if (lane == 0) tma_wait_read<0>();
        __syncwarp();
    }
    if (lane == 0) {
        tma_wait_all();
        if (!ok) report(g.status, QSSM_S_TMA_TIMEOUT);
    }
}

}  // namespace qssm
