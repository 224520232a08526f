/*
 * qssm.h - C ABI of the B200 (sm_100a) gated linear scan
 *
 *     h(t) = a(t) * h(t-1) + b(t) * x(t),   y(t) = c(t) * h(t),   h(-1) = h_in (default 0)
 *
 * over [B, L, D] tensors whose innermost (D) axis is contiguous; one
 * independent recurrence per (b, d).  Storage types are fp32, fp16 or bf16;
 * all arithmetic is fp32.
 *
 * Conventions shared by every entry point
 *   - every pointer is a DEVICE pointer unless the parameter says "host";
 *   - strides are in ELEMENTS (stride_b between batches, stride_l between time
 *     steps); the D stride is 1;
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream);
 *   - the library allocates no device memory, never synchronises and keeps no
 *     state between calls that a result depends on (it remembers, per host thread,
 *     the tensor-map encodings of the buffers it saw last and, per device, what it
 *     asked the runtime about its own kernels); scratch comes from the caller
 *     (`ws`, sized by qssm_workspace_bytes);
 *   - return value: 0 ok; < 0 bad argument (QSSM_E_*); > 0 a cudaError_t from
 *     a launch.  Errors found on the device while a kernel runs (a bounded
 *     wait that expired) are reported through `status_word`, an int the
 *     caller owns (device memory or pinned host memory reachable from the
 *     device; may be NULL): 0 = ok, otherwise a QSSM_S_* code.
 *
 * Each entry point names the interface of the reference implementation
 * (samblouir/quick_ssm, paths inside that project) it replaces.
 */
#ifndef QSSM_H
#define QSSM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* storage dtypes */
#define QSSM_F32 0
#define QSSM_F16 1
#define QSSM_BF16 2

/* argument errors (negative return values) */
#define QSSM_E_NULL (-1)      /* a required pointer is NULL */
#define QSSM_E_SHAPE (-2)     /* negative size, or a size beyond what the kernels index */
#define QSSM_E_DTYPE (-3)     /* unknown dtype or unsupported in/out dtype pair */
#define QSSM_E_STRIDE (-4)    /* stride smaller than the extent it must step over */
#define QSSM_E_NEED_H (-5)    /* backward needs tile_h or h_saved */
#define QSSM_E_WS (-6)        /* workspace too small for the requested segment count */
#define QSSM_E_DRIVER (-7)    /* the CUDA driver entry point for tensor maps is unavailable */
#define QSSM_E_STATIC_WS (-8) /* qssm_scan_fwd_static_ws: scratch needed exceeds QSSM_STATIC_WS_BYTES */

/* device-side status codes written to *status_word (kept apart from cudaError_t values) */
#define QSSM_S_OK 0
#define QSSM_S_TMA_TIMEOUT 10001  /* a bounded wait on a bulk-copy barrier expired */

/* Rows of time covered by one entry of the `tile_h` boundary-state array. */
#define QSSM_TILE_ROWS 16

/* Library version (major*10000 + minor*100 + patch). No reference counterpart. */
int qssm_version(void);

/*
 * Tuning knobs and the test hook.  No counterpart in the reference; production callers use neither.
 * Launch-shape choices (strip width "V", tile rows "TB", ring depth "STAGES", "NOUT", "GRID", "WIDE",
 * "FWD_TILE4", "NO_TMA", "L2HINT", the single-pass kernels "CHAINED", "CHUNK_ROWS", "CHAINED_GRID",
 * "CHAINED_HINT", "CHAINED_SLOTS", the limit of bounded waits "WAIT_MS", "DEBUG") take their values from the
 * environment variables QSSM_<NAME> once, when the library is first used; afterwards only these two
 * calls change them, process-wide.  No launch reads the environment.  "TEST_SKIP_FIRST_CHUNK" (no
 * environment form) makes the single-pass kernels skip the first chunk of every chain, so that their
 * bounded waits expire: the host-side way to exercise the device error path on a healthy GPU.
 * qssm_tune_set returns 0, or QSSM_E_SHAPE for an unknown name; qssm_tune_reset restores the start-up values.
 */
int qssm_tune_set(const char* name, int value);
void qssm_tune_reset(void);

/* Text for a return value of any entry point or for a QSSM_S_* status code. */
const char* qssm_status_string(int code);

/* Rows per tile_h entry (== QSSM_TILE_ROWS), for callers that cannot read the header. */
int qssm_tile_rows(void);

/*
 * Bytes of scratch (`ws`) that lets qssm_scan_fwd / qssm_scan_bwd /
 * qssm_scan_aggregate_* split the time axis into parallel segments when B*D
 * alone gives the GPU too few independent recurrences, or run such a shape with
 * the single-pass chained kernels (ticket counter and chunk descriptors; the
 * larger of the forward's and the backward's need).  0 means no scratch is
 * ever used for this shape.  Passing less (or NULL) is legal: the call then
 * runs unsegmented with one warp per strip.
 * Replaces the scratch the reference allocates on every call
 * (triton_forwards.py:152-162, triton_backwards.py:188-199).
 */
size_t qssm_workspace_bytes(int64_t B, int64_t L, int64_t D, int in_dtype);

/* Segment count the library would pick for this shape (1 = unsegmented). */
int qssm_auto_segments(int64_t B, int64_t L, int64_t D, int in_dtype);

/*
 * Forward scan.
 *   c != NULL: y = c * h                       (scan(), scan_interface.py:169-213;
 *              _TritonScanFunction.forward, :58-110; block_scan_forward_3d,
 *              triton_forwards.py:134-172 plus the torch epilogue :104-107)
 *   c == NULL: y = h in out_dtype              (forward_only.block_scan_forward_3d,
 *              forward_only.py:423-540)
 * Optional outputs
 *   h_saved [B,L,D] fp32 contiguous: every h(t) (checkpoint=False, scan_interface.py:86,:102)
 *   tile_h  [B, ceil(L/QSSM_TILE_ROWS), D] fp32 contiguous: h just before each
 *           tile of QSSM_TILE_ROWS steps; lets the backward rebuild h in-kernel
 *           (checkpoint=True, replaces the forward re-run of scan_interface.py:133-134)
 *   h_last  [B,D] fp32: h(L-1)
 * Optional input
 *   h_in    [B,D] fp32: state before t=0 (sequence shards, streaming)
 * n_seg: 0 = automatic, k > 0 = k time segments run in parallel (needs ws; results are identical
 *        within fp32 rounding for every value), -k = k segments whose aggregates are already in
 *        ws, left there by qssm_scan_aggregate_fwd called with the same shape, dtype and n_seg = k
 *        (sequence shards: the aggregate pass that feeds the exchange is not repeated).
 *        qssm_scan_bwd takes the same three forms, paired with qssm_scan_aggregate_bwd.
 */
int qssm_scan_fwd(const void* x, const void* a, const void* b, const void* c, void* y,
                  float* h_saved, float* tile_h, const float* h_in, float* h_last,
                  void* ws, size_t ws_bytes,
                  int64_t B, int64_t L, int64_t D,
                  int64_t in_stride_b, int64_t in_stride_l,
                  int64_t out_stride_b, int64_t out_stride_l,
                  int in_dtype, int out_dtype, int n_seg,
                  int* status_word, void* stream);

/*
 * Forward scan that brings its own scratch.  No counterpart in the reference.
 *
 * Same arguments, results and return codes as qssm_scan_fwd, minus `ws`/`ws_bytes`.  It is meant
 * for callers that must not, or cannot, allocate device memory around the call: a plugin inside
 * a host runtime whose memory pool has already reserved the device heap and hands out no
 * allocator (a raw cudaMalloc there fails or fragments the pool), a service with a "no
 * allocation after start-up" rule, a latency-critical loop where the implicit device-wide
 * synchronisation of cudaMalloc/cudaFree is not acceptable.  The segment aggregates and seeds that
 * qssm_scan_fwd keeps in `ws` live instead in a fixed array of QSSM_STATIC_WS_BYTES inside the
 * library's device image (each GPU that loads the library carries those bytes until the process
 * ends).  The call performs no cudaMalloc/cudaFree and calls no allocating library routine.
 *
 * Limits and rules
 *   - the scratch the shape needs, 3 * B * n_seg * D * 4 bytes with n_seg = the `n_seg` argument or,
 *     for 0, qssm_auto_segments(), must fit: otherwise QSSM_E_STATIC_WS is returned and nothing
 *     is launched (the call never silently runs unsegmented).  With n_seg = 0 and no h_saved the
 *     library may run a few-chain, long-sequence shape with its single-pass kernels; their ticket
 *     counter and chunk descriptors (qssm_workspace_bytes) then live in the array as well, must fit
 *     too, and are zeroed by a memset on `stream` at the start of the call;
 *   - n_seg < 0 ("aggregates already in ws") is refused with QSSM_E_SHAPE: no aggregate entry point
 *     writes the built-in array, so there is nothing to reuse;
 *   - the first call on each device looks up the device address of the array (a short host-side
 *     runtime query, done with that device current); make that first call outside any stream
 *     capture;
 *   - all calls on one GPU share the one array and it keeps whatever the previous call left in
 *     it.  The segment path needs nothing in it to start at zero (every entry is written by the
 *     aggregate and carry kernels of a call before the scan kernel of the same call reads it); the
 *     single-pass path clears what it needs itself, as said above.  Two calls whose
 *     kernels can overlap on the GPU (different streams, no ordering between them) race on it:
 *     order them, or use qssm_scan_fwd with separate `ws` buffers.
 */
#define QSSM_STATIC_WS_BYTES (4 * 1024 * 1024)
int qssm_scan_fwd_static_ws(const void* x, const void* a, const void* b, const void* c, void* y,
                            float* h_saved, float* tile_h, const float* h_in, float* h_last,
                            int64_t B, int64_t L, int64_t D,
                            int64_t in_stride_b, int64_t in_stride_l,
                            int64_t out_stride_b, int64_t out_stride_l,
                            int in_dtype, int out_dtype, int n_seg,
                            int* status_word, void* stream);

/*
 * Backward scan for upstream gradient dy (dtype out_dtype, strides dy_stride_*):
 *   dh(t) = c(t)*dy(t) + a(t+1)*dh(t+1);  dx = dh*b, db = dh*x, da = dh*h(t-1), dc = dy*h
 * Gradients are written in in_dtype into contiguous [B,L,D] buffers.
 * Replaces _TritonScanFunction.backward (scan_interface.py:113-158) and
 * block_scan_backward_3d (triton_backwards.py:168-209).
 *   tile_h  (from qssm_scan_fwd) : h is rebuilt tile by tile in the kernel, or
 *   h_saved [B,L,D] fp32         : h is read (then h_in, if the forward had one, is
 *                                  needed again for da at t = 0).
 *   g_in    [B,D] fp32 optional  : a(L)*dh(L) handed over by the next sequence shard
 *   g_first [B,D] fp32 optional  : a(0)*dh(0), the value to hand to the previous shard
 */
int qssm_scan_bwd(const void* x, const void* a, const void* b, const void* c, const void* dy,
                  const float* h_saved, const float* tile_h, const float* h_in,
                  const float* g_in, float* g_first,
                  void* dx, void* da, void* db, void* dc,
                  void* ws, size_t ws_bytes,
                  int64_t B, int64_t L, int64_t D,
                  int64_t in_stride_b, int64_t in_stride_l,
                  int64_t dy_stride_b, int64_t dy_stride_l,
                  int in_dtype, int out_dtype, int n_seg,
                  int* status_word, void* stream);

/*
 * Scan with the gate activations of the SSM layer fused into its loads and stores.
 * Inputs are the five projection outputs ("pre-activations") of the layer:
 *     a = sigmoid(pa)   x = px   c = silu(pc1) * pc2   b = sigmoid(pd)     y = c * h
 * each rounded to gate_dtype before use, as the layer rounds them to its compute dtype
 * (reference: SSM.forward, layers.py:76-104; the element-wise kernels between the projections and
 * scan() are what this replaces).  The backward returns the gradients of the five
 * pre-activations (contiguous [B,L,D], in_dtype).  Supported: in fp32 with gates fp32/bf16/fp16
 * and y, dy fp32; in bf16 (fp16) with gates bf16 (fp16) and y, dy bf16 (fp16) or fp32.
 * All five inputs share one layout that the bulk copy engine can address (16-byte aligned base
 * and pitches); otherwise QSSM_E_STRIDE is returned and the caller composes the gates itself.
 * tile_h / h_in / h_last / g_in / g_first as in qssm_scan_fwd / qssm_scan_bwd.
 */
int qssm_gated_scan_fwd(const void* pa, const void* px, const void* pc1, const void* pc2, const void* pd,
                        void* y, float* tile_h, const float* h_in, float* h_last,
                        int64_t B, int64_t L, int64_t D,
                        int64_t in_stride_b, int64_t in_stride_l,
                        int64_t out_stride_b, int64_t out_stride_l,
                        int in_dtype, int gate_dtype, int out_dtype,
                        int* status_word, void* stream);

int qssm_gated_scan_bwd(const void* pa, const void* px, const void* pc1, const void* pc2, const void* pd,
                        const void* dy, const float* tile_h, const float* g_in, float* g_first,
                        void* dpa, void* dpx, void* dpc1, void* dpc2, void* dpd,
                        int64_t B, int64_t L, int64_t D,
                        int64_t in_stride_b, int64_t in_stride_l,
                        int64_t dy_stride_b, int64_t dy_stride_l,
                        int in_dtype, int gate_dtype, int out_dtype,
                        int* status_word, void* stream);

/*
 * Aggregates of a whole [B,L,D] block, the values sequence shards exchange:
 *   forward : A[B,D] = prod_t a(t),  H[B,D] = h(L-1) computed from h(-1)=0,
 *             so that for any h_in  h(L-1) = A*h_in + H
 *             (the block carry of ssm_local_forward_kernel, triton_forwards.py:33-74)
 *   backward: P[B,D] = prod_t a(t),  Q[B,D] = a(0)*dh(0) computed from g_in=0,
 *             so that for any g_in  g_first = P*g_in + Q
 *             (the block carry of ssm_local_backward_kernel, triton_backwards.py:32-82)
 */
int qssm_scan_aggregate_fwd(const void* x, const void* a, const void* b,
                            float* A, float* H, void* ws, size_t ws_bytes,
                            int64_t B, int64_t L, int64_t D,
                            int64_t in_stride_b, int64_t in_stride_l,
                            int in_dtype, int n_seg, int* status_word, void* stream);

int qssm_scan_aggregate_bwd(const void* a, const void* c, const void* dy,
                            float* P, float* Q, void* ws, size_t ws_bytes,
                            int64_t B, int64_t L, int64_t D,
                            int64_t in_stride_b, int64_t in_stride_l,
                            int64_t dy_stride_b, int64_t dy_stride_l,
                            int in_dtype, int out_dtype, int n_seg,
                            int* status_word, void* stream);

/*
 * Fold a list of n aggregates (A_k, H_k), each n_chan floats, stored with a
 * stride of `stride_k` floats between consecutive k, with the scan's combine
 *   (aL,xL) + (aR,xR) = (aR*aL, aR*xL + xR),   identity (1,0)
 * (combine_fn, triton_forwards.py:26-30; aggregator_combine, triton_backwards.py:25-29).
 *   reverse == 0: carry[c] = state after applying k = 0 .. upto-1 in order to seed[c]
 *   reverse != 0: carry[c] = state after applying k = n-1 .. upto+1 (descending) to seed[c]
 * seed may be NULL (zero).  Used to turn all-gathered shard aggregates into the
 * h_in / g_in of shard `upto`.
 */
int qssm_carry_fold(const float* A, const float* H, int64_t n, int64_t stride_k,
                    int64_t n_chan, int64_t upto, int reverse,
                    const float* seed, float* carry, void* stream);

/*
 * Carry exchange between sequence shards through peer memory, in place of the all-gather followed
 * by qssm_carry_fold.  No counterpart in the reference (it runs on one GPU).
 *
 * Every rank owns, in its own device memory, an inbox of qssm_peer_inbox_bytes(world, n_chan) bytes,
 * zero before the first call: QSSM_PEER_SLOTS * world * 2 * n_chan floats of aggregate pairs, then
 * (at qssm_peer_flags_offset) QSSM_PEER_SLOTS * world ints of flags.  Every rank has the inboxes of
 * all ranks mapped so that its OWN device may store into them (a cuMemCreate allocation shared as a
 * handle and mapped with cuMemSetAccess for the storing device, e.g. torch's symmetric memory;
 * `peer_inbox[rank]` is the rank's own inbox).  Only plain loads and stores touch peer memory: no
 * bulk-copy engine, no multicast.
 *   qssm_carry_push     : copies this rank's pair (first, second), n_chan floats each, into slot
 *                         `slot` of every rank's inbox and then sets this rank's flag there to
 *                         `epoch`.  counters: `world` zeroed unsigned ints in local memory.
 *   qssm_carry_wait_fold: waits (at most wait_ms, then QSSM_S_TMA_TIMEOUT in *status_word and an
 *                         unchanged `carry`) until the flags of all ranks in slot `slot` of the local
 *                         inbox show `epoch`, then carry[c] = the pairs of the ranks before `rank`
 *                         (reverse != 0: after) folded in rank order onto seed[c] (seed NULL = 0)
 *                         with (aL,xL)+(aR,xR) = (aR*aL, aR*xL+xR), exactly as qssm_carry_fold does
 *                         on gathered pairs.
 * Callers use epoch = 1, 2, 3, ... per direction and slot = 2*direction + (epoch & 1); all ranks
 * make the same sequence of calls on one stream each.  world <= QSSM_MAX_PEERS.
 */
#define QSSM_MAX_PEERS 16
#define QSSM_PEER_SLOTS 4

size_t qssm_peer_inbox_bytes(int world, int64_t n_chan);
size_t qssm_peer_flags_offset(int world, int64_t n_chan);

int qssm_carry_push(const float* first, const float* second, int64_t n_chan,
                    void* const* peer_inbox, unsigned int* counters,
                    int rank, int world, int slot, int epoch, void* stream);

int qssm_carry_wait_fold(const void* inbox, int64_t n_chan,
                         int rank, int world, int slot, int epoch, int reverse,
                         const float* seed, float* carry, int wait_ms,
                         int* status_word, void* stream);

/*
 * RMS normalisation of the layer input, the step before the projections that feed the scan
 * (RMSNorm.forward, quick_ssm/layers.py:9-17):
 *     y[r, :] = x[r, :] * w / sqrt(mean(x[r, :]^2) + eps)          r = 0 .. rows-1
 * x, y, dy, dx: `rows` rows of H elements of `dtype`, row pitches in elements; w, dw: H floats.
 * forward : writes y and, if rstd != NULL, rstd[r] = 1/sqrt(mean(x^2)+eps) for the backward.
 * backward: dx = rstd*(w*dy) - x*rstd^3*mean(x*w*dy),  dw = sum_r dy*x*rstd  (fixed summation
 *           order, no atomics).  ws: at least qssm_rmsnorm_workspace_bytes(H) bytes of scratch.
 * Rows need H % 4 == 0 and 16-byte aligned bases and pitches (8 bytes for 16-bit data);
 * otherwise QSSM_E_STRIDE and nothing is launched.
 */
size_t qssm_rmsnorm_workspace_bytes(int64_t H);

int qssm_rmsnorm_fwd(const void* x, const float* w, void* y, float* rstd,
                     int64_t rows, int64_t H, int64_t x_stride, int64_t y_stride,
                     float eps, int dtype, void* stream);

int qssm_rmsnorm_bwd(const void* x, const float* w, const void* dy, const float* rstd,
                     void* dx, float* dw, void* ws, size_t ws_bytes,
                     int64_t rows, int64_t H, int64_t x_stride, int64_t dy_stride, int64_t dx_stride,
                     int dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* QSSM_H */
