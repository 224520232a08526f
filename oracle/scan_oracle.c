/*
 * CPU oracle for the gated linear scan.  TEST INFRASTRUCTURE ONLY: it is the
 * checker the CUDA kernels are compared with (tests, the smoke run and the
 * CPU-baseline leg of the benchmark); nothing on the product path may call it.
 *
 * It restates, as plain sequential C loops, the algorithm of the reference's
 * quick_ssm/naive_baseline.py:
 *   - forward recurrence   h(t) = a(t)*h(t-1) + b(t)*x(t), h(-1) = 0
 *                          (naive_forward_3d, naive_baseline.py:12-40)
 *   - output               y(t) = c(t)*h(t)
 *                          (naive_full_3d, naive_baseline.py:43-64)
 *   - backward for the loss sum(y*grad_y)
 *                          (naive_backward_3d, naive_baseline.py:67-137)
 * Tensors are [B, L, D] with D contiguous; one independent recurrence per
 * (b, d).  Two accumulation widths are provided: double (the ground truth)
 * and float (what the reference does for fp32 and, after up-casting, for
 * fp16/bf16 inputs).  The float versions are compiled with
 * -ffp-contract=off so that every multiply and add rounds separately, like
 * the reference's element-wise torch ops; on fp32 inputs they reproduce the
 * reference bit for bit (pinned by tests against fixtures generated from the
 * reference itself).
 *
 * Optional arguments extend the reference's loop to the seeded form used for
 * sequence sharding: h_in[B,D] replaces h(-1)=0, g_in[B,D] replaces the zero
 * upstream carry a(L)*dh(L).  NULL means the reference's zero.
 *
 * Parallelism: OpenMP over (b, d-block); each thread walks time sequentially.
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define DBLK 64

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

#define DEFINE_ORACLE(T, SUFFIX)                                                          \
/* forward: writes h and/or y (either may be NULL). naive_baseline.py:34-39, :62 */      \
void oracle_scan_fwd_##SUFFIX(const T* x, const T* a, const T* b, const T* c,            \
                              const T* h_in, T* h, T* y, T* h_last,                      \
                              int64_t B, int64_t L, int64_t D) {                         \
    int64_t nblk = (D + DBLK - 1) / DBLK;                                                \
    _Pragma("omp parallel for collapse(2) schedule(static)")                             \
    for (int64_t bb = 0; bb < B; ++bb) {                                                 \
        for (int64_t blk = 0; blk < nblk; ++blk) {                                       \
            int64_t d0 = blk * DBLK;                                                     \
            int64_t d1 = d0 + DBLK < D ? d0 + DBLK : D;                                  \
            T run[DBLK];                                                                 \
            for (int64_t d = d0; d < d1; ++d)                                            \
                run[d - d0] = h_in ? h_in[bb * D + d] : (T)0;                            \
            for (int64_t t = 0; t < L; ++t) {                                            \
                size_t off = ((size_t)bb * L + t) * D;                                   \
                for (int64_t d = d0; d < d1; ++d) {                                      \
                    T ah = a[off + d] * run[d - d0];                                     \
                    T bx = b[off + d] * x[off + d];                                      \
                    T hv = ah + bx;                                                      \
                    run[d - d0] = hv;                                                    \
                    if (h) h[off + d] = hv;                                              \
                    if (y) y[off + d] = c[off + d] * hv;                                 \
                }                                                                        \
            }                                                                            \
            if (h_last)                                                                  \
                for (int64_t d = d0; d < d1; ++d) h_last[bb * D + d] = run[d - d0];      \
        }                                                                                \
    }                                                                                    \
}                                                                                        \
                                                                                         \
/* backward given h (recomputed by the caller or saved). naive_baseline.py:108-135 */    \
void oracle_scan_bwd_##SUFFIX(const T* x, const T* a, const T* b, const T* c,            \
                              const T* h, const T* h_in, const T* dy, const T* g_in,     \
                              T* dx, T* da, T* db, T* dc, T* g_first,                    \
                              int64_t B, int64_t L, int64_t D) {                         \
    int64_t nblk = (D + DBLK - 1) / DBLK;                                                \
    _Pragma("omp parallel for collapse(2) schedule(static)")                             \
    for (int64_t bb = 0; bb < B; ++bb) {                                                 \
        for (int64_t blk = 0; blk < nblk; ++blk) {                                       \
            int64_t d0 = blk * DBLK;                                                     \
            int64_t d1 = d0 + DBLK < D ? d0 + DBLK : D;                                  \
            T nxt[DBLK]; /* a(t+1)*dh(t+1): "dh_next", naive_baseline.py:99-101,135 */   \
            for (int64_t d = d0; d < d1; ++d)                                            \
                nxt[d - d0] = g_in ? g_in[bb * D + d] : (T)0;                            \
            for (int64_t t = L - 1; t >= 0; --t) {                                       \
                size_t off = ((size_t)bb * L + t) * D;                                   \
                for (int64_t d = d0; d < d1; ++d) {                                      \
                    T loc = dy[off + d] * c[off + d];                                    \
                    T tot = loc + nxt[d - d0];                                           \
                    T hp = t > 0 ? h[off - D + d]                                        \
                                 : (h_in ? h_in[bb * D + d] : (T)0);                     \
                    dc[off + d] = dy[off + d] * h[off + d];                              \
                    db[off + d] = tot * x[off + d];                                      \
                    da[off + d] = tot * hp;                                              \
                    dx[off + d] = tot * b[off + d];                                      \
                    nxt[d - d0] = tot * a[off + d];                                      \
                }                                                                        \
            }                                                                            \
            if (g_first)                                                                 \
                for (int64_t d = d0; d < d1; ++d) g_first[bb * D + d] = nxt[d - d0];     \
        }                                                                                \
    }                                                                                    \
}                                                                                        \
                                                                                         \
/* forward + backward in one call, h held in a scratch buffer the caller passes */       \
void oracle_scan_fwd_bwd_##SUFFIX(const T* x, const T* a, const T* b, const T* c,        \
                                  const T* dy, T* h_scratch, T* y,                       \
                                  T* dx, T* da, T* db, T* dc,                            \
                                  int64_t B, int64_t L, int64_t D) {                     \
    oracle_scan_fwd_##SUFFIX(x, a, b, c, NULL, h_scratch, y, NULL, B, L, D);             \
    oracle_scan_bwd_##SUFFIX(x, a, b, c, h_scratch, NULL, dy, NULL,                      \
                             dx, da, db, dc, NULL, B, L, D);                             \
}

DEFINE_ORACLE(float, f32)
DEFINE_ORACLE(double, f64)

/*
 * Blockwise restatement (second, independent shape of the same algorithm):
 * local scans inside blocks of block_l steps, a sequential scan of the block
 * carries with the combine (aL,xL)+(aR,xR) = (aR*aL, aR*xL + xR), then the
 * fix-up h = a_loc*h_in + h_loc.  Follows the structure of the reference's
 * three-kernel block scan (triton_forwards.py:33-131) and its float64
 * blockwise helper (depth_diff.py:15-60).  Double precision only.
 */
void oracle_scan_fwd_blockwise_f64(const double* x, const double* a, const double* b,
                                   double* h, int64_t B, int64_t L, int64_t D,
                                   int64_t block_l) {
    if (block_l <= 0) block_l = 256;
    int64_t nblocks = (L + block_l - 1) / block_l;
    if (nblocks == 0) return;
    #pragma omp parallel for collapse(2) schedule(static)
    for (int64_t bb = 0; bb < B; ++bb) {
        for (int64_t d = 0; d < D; ++d) {
            double* ca = (double*)malloc(sizeof(double) * 2 * (size_t)nblocks);
            double* cx = ca + nblocks;
            double* la = (double*)malloc(sizeof(double) * 2 * (size_t)L);
            double* lx = la + L;
            for (int64_t k = 0; k < nblocks; ++k) {
                double ar = 1.0, xr = 0.0;
                int64_t t1 = (k + 1) * block_l < L ? (k + 1) * block_l : L;
                for (int64_t t = k * block_l; t < t1; ++t) {
                    size_t off = ((size_t)bb * L + t) * D + d;
                    double an = a[off] * ar;
                    double xn = a[off] * xr + b[off] * x[off];
                    la[t] = an; lx[t] = xn; ar = an; xr = xn;
                }
                ca[k] = ar; cx[k] = xr;
            }
            for (int64_t k = 1; k < nblocks; ++k) { /* inclusive carry scan */
                double na = ca[k] * ca[k - 1];
                double nx = ca[k] * cx[k - 1] + cx[k];
                ca[k] = na; cx[k] = nx;
            }
            for (int64_t t = 0; t < L; ++t) {
                int64_t k = t / block_l;
                double xp = k == 0 ? 0.0 : cx[k - 1];
                h[((size_t)bb * L + t) * D + d] = la[t] * xp + lx[t];
            }
            free(ca); free(la);
        }
    }
}
