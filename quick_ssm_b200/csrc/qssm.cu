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
//    memory and lane 0 issues the bulk tensor store.  One CTA == one warp:
//    many small CTAs per SM give the latency hiding;
//  * the write-heavy launches on 16-bit data (the backward; the forward that
//    also stores fp32 h) give four adjacent strips to a CTA of four warps,
//    which loads and stores them as one 512-byte-wide tile per tensor with
//    one __syncthreads per tile (scan_bwd_tile4_kernel, scan_fwd_tile4_kernel);
//  * with very few chains (long sequences of a few thousand channels) the
//    chained kernels cut every chain into chunks claimed from a ticket
//    counter and pass the carry between chunks through descriptors in
//    global memory (decoupled look-back, every wait bounded);
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
//
// Files: qssm_ptx.cuh (PTX wrappers), qssm_tile.cuh (element/tile helpers, parameter blocks),
// qssm_fwd.cuh, qssm_bwd.cuh, qssm_agg.cuh (scan kernels), qssm_gated.cuh (scan with the layer's gate
// activations fused in), qssm_norm.cuh (the layer's RMS norm), this file (launch planning and the C ABI).
#include <limits.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "qssm_agg.cuh"
#include "qssm_bwd.cuh"
#include "qssm_fwd.cuh"
#include "qssm_gated.cuh"
#include "qssm_norm.cuh"
#include "qssm_peer.cuh"

using namespace qssm;

namespace {

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

// ---------------------------------------------------------------------------------------------
// Tuning knobs.  Production callers set none of them.  Each knob is read from the environment
// variable QSSM_<NAME> once, when the library is first used, and can be changed afterwards only
// through qssm_tune_set (measurement scripts and tests); launches never call getenv.
// TEST_SKIP_FIRST_CHUNK is a test hook and has no environment form.
// ---------------------------------------------------------------------------------------------
enum Knob {
    K_GRID, K_V, K_TB, K_STAGES, K_NOUT, K_WIDE, K_FWD_TILE4, K_NO_TMA, K_L2HINT, K_CHAINED, K_CHUNK_ROWS,
    K_CHAINED_GRID, K_CHAINED_HINT, K_CHAINED_SLOTS, K_WAIT_MS, K_DEBUG, K_TEST_SKIP_FIRST_CHUNK, K_COUNT
};
const char* const kKnobNames[K_COUNT] = {"GRID", "V", "TB", "STAGES", "NOUT", "WIDE", "FWD_TILE4", "NO_TMA", "L2HINT",
                                         "CHAINED", "CHUNK_ROWS", "CHAINED_GRID", "CHAINED_HINT", "CHAINED_SLOTS", "WAIT_MS", "DEBUG",
                                         "TEST_SKIP_FIRST_CHUNK"};
constexpr int KNOB_UNSET = INT_MIN;

struct Knobs {
    int now[K_COUNT];    // current values (KNOB_UNSET = use the call site's default)
    int start[K_COUNT];  // values taken from the environment at first use
    Knobs() {
        for (int k = 0; k < K_COUNT; ++k) {
            start[k] = KNOB_UNSET;
            if (k != K_TEST_SKIP_FIRST_CHUNK) {
                char name[64];
                snprintf(name, sizeof(name), "QSSM_%s", kKnobNames[k]);
                const char* v = getenv(name);
                if (v != nullptr && *v != '\0') start[k] = atoi(v);
            }
            now[k] = start[k];
        }
    }
};
Knobs& knobs() {
    static Knobs k;
    return k;
}
inline int knob(Knob k, int dflt) {
    const int v = __atomic_load_n(&knobs().now[k], __ATOMIC_RELAXED);
    return v == KNOB_UNSET ? dflt : v;
}

// A tensor map is a pure function of (base, dtype, extents, pitches, box).  Training loops call with the
// same buffers step after step (a caching allocator hands the same addresses back), so each host thread
// keeps the maps it encoded last: a hit copies 128 bytes instead of calling into the driver.
struct MapKey {
    const void* ptr;
    long long B, rows, D, sb, sl;
    int dt, box_d, box_rows, pad;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && B == o.B && rows == o.rows && D == o.D && sb == o.sb && sl == o.sl && dt == o.dt &&
               box_d == o.box_d && box_rows == o.box_rows;
    }
};
struct MapCache {
    static constexpr int N = 64;  // direct mapped
    MapKey key[N];
    CUtensorMap map[N];
    bool used[N];
    MapCache() { memset(used, 0, sizeof(used)); }
    static unsigned slot_of(const MapKey& k) {
        unsigned long long h = (unsigned long long)reinterpret_cast<uintptr_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
        h ^= (unsigned long long)k.box_d * 0x85EBCA6Bull + (unsigned long long)k.box_rows * 0xC2B2AE35ull +
             (unsigned long long)k.rows * 0x27D4EB2Full + (unsigned long long)k.dt;
        return (unsigned)(h >> 40) % N;
    }
};

// dims (D, rows, B); box (box_d, box_rows, 1)
int fill_desc(TensorDesc& td, const void* ptr, int dt, long long B, long long rows, long long D, long long sb,
              long long sl, int box_d, int box_rows, bool use_tma) {
    memset(&td, 0, sizeof(td));
    td.ptr = const_cast<void*>(ptr);
    td.stride_b = sb;
    td.stride_l = sl;
    if (!use_tma || ptr == nullptr) return 0;
    static thread_local MapCache cache;
    const MapKey key{ptr, B, rows, D, sb, sl, dt, box_d, box_rows, 0};
    const unsigned slot = MapCache::slot_of(key);
    if (cache.used[slot] && cache.key[slot] == key) {
        td.map = cache.map[slot];
        return 0;
    }
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
    if (r != CUDA_SUCCESS && knob(K_DEBUG, 0) != 0)
        fprintf(stderr,
                "qssm: cuTensorMapEncodeTiled failed (%d): ptr=%p dt=%d dims=(%llu,%llu,%llu) strides=(%llu,%llu) "
                "box=(%u,%u,%u)\n",
                (int)r, ptr, dt, (unsigned long long)dims[0], (unsigned long long)dims[1],
                (unsigned long long)dims[2], (unsigned long long)strides[0], (unsigned long long)strides[1], box[0],
                box[1], box[2]);
    if (r != CUDA_SUCCESS) return QSSM_E_STRIDE;
    cache.key[slot] = key;
    cache.map[slot] = td.map;
    cache.used[slot] = true;
    return 0;
}

constexpr int MAX_DEVICES = 64;

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return 0;
    return dev;
}

// SM count of the current device (looked up once per device ordinal).
int sm_count() {
    static int cached[MAX_DEVICES];
    const int dev = current_device();
    int n = __atomic_load_n(&cached[dev], __ATOMIC_RELAXED);
    if (n <= 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        n = v;
        __atomic_store_n(&cached[dev], n, __ATOMIC_RELAXED);
    }
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
    const long long forced_grid = knob(K_GRID, 0);
    if (forced_grid > 0) return forced_grid < chains ? forced_grid : chains;
    const double target = write_heavy ? 3.5 * sm_count() : 4.0 * sm_count();
    long long rounds = (long long)((double)chains / target + (write_heavy ? 0.2 : 0.3));
    if (rounds < 1) rounds = 1;
    return (chains + rounds - 1) / rounds;
}

// The fused-gate kernels execute two to three times the instructions of the plain scan per element
// (activations and their derivatives) and are bound by instruction issue rather than by bytes in
// flight: they run fastest with every chain resident.  Measured on 16 x 4096 x 4096 (1024 chains),
// forward + backward: all chains at once 2.12 ms with bf16 and 2.89 ms with fp32 projection outputs,
// two rounds of 512 chains 2.73 / 3.16 ms.
long long concurrent_chains_gated(long long chains) {
    const long long forced_grid = knob(K_GRID, 0);
    if (forced_grid > 0) return forced_grid < chains ? forced_grid : chains;
    const long long cap = 8ll * sm_count();
    const long long rounds = (chains + cap - 1) / cap;
    return (chains + rounds - 1) / rounds;
}

// Channels per lane.  Two channels per lane halve the shared-memory and copy-engine instructions
// per element, so one warp moves twice the bytes; narrow strips (V = 1) are for channel counts
// that would leave half of a wide strip empty, or for launches with too few chains to give
// every SM two warps even after the time axis has been segmented.
int pick_v(long long B, long long D, int n_seg, int elem_size = 0) {
    const int forced = knob(K_V, 0);
    if (forced == 1 || forced == 2) return forced;
    if (D <= 32) return 1;
    const long long chains_v2 = B * ((D + 63) / 64) * (n_seg < 1 ? 1 : n_seg);
    // fp32 rows are twice as long, so a warp has twice the bytes in flight and wide strips pay from 1.2 chains
    // per SM on (192 wide chains on 148 SMs: 0.93 of the copy peak forward + backward against 0.89 narrow;
    // 160: 0.82 wide against 0.95 narrow)
    if (elem_size == 4 && n_seg <= 1) return 5 * chains_v2 >= 6ll * sm_count() ? 2 : 1;
    return chains_v2 >= 2ll * sm_count() ? 2 : 1;
}
int pick_tb() {
    const int forced = knob(K_TB, 0);
    return forced == 16 || forced == 32 ? forced : 16;
}
// Read-mostly kernels on 16-bit data move more bytes per second with tiles of 32 rows (4 KB bulk copies per
// tensor instead of 2 KB).  Measured on B200, 128-byte strips: aggregates 6.1 -> 7.1 TB/s (cfg1 and cfg4 shapes),
// forward with 16-bit output 6.45 -> 6.64 TB/s, h only 6.08 -> 6.52 TB/s; the forward with fp32 output and
// every backward lose (4.5 against 6.5 TB/s, 4.8 against 6.25), so they stay on 16 rows.
bool prefers_tall_tiles(int in_dtype, int V) { return knob(K_TB, 0) == 0 && dtype_size(in_dtype) == 2 && V == 2; }

// fp32 storage, one pass over an unsegmented time axis, h rebuilt from the tile states.  Tiles of 32 rows double
// the bytes a warp keeps in flight, which is what a launch with few chains lacks; with many chains they help the
// backward only (two 40 KB stages, two CTAs per SM).  Measured on B200 (148 SMs), D = 2048, 2^27 elements,
// forward / backward in GB/s of the 5 / 9 tensor passes, 16 against 32 rows:
//   narrow strips  128 wide-strip equivalents: 4029/5226 -> 5716/5666    160: 5006/5632 -> 6713/6012
//   wide strips    192: 5566/5500 -> 6274/6002    256: 6846/6216 -> 6783/5654    320: 6792/6084 -> 4821/4778
//                  512: 6846/5737 -> 6742/6103   1024: 6840/5731 -> 6748/6035
int f32_tile_rows(int V, long long chains, bool backward) {
    const long long sms = sm_count();
    if (V == 1) return 2 * chains < 5 * sms ? 32 : 16;
    if (2 * chains < 3 * sms) return 32;
    return backward && chains >= 3 * sms ? 32 : 16;
}

// fp32 storage: the forward runs at the copy rate with one warp per strip from one wide strip per SM on (160 strips
// on 148 SMs: 6.70 TB/s, the chained forward 5.82 at any count), below that the chained forward wins (128: 5.84
// against 5.71, 96: 5.85 against 4.30); segmenting the time axis never does (0.68 of the copy peak).
bool f32_one_pass(long long chains_v2, int elem_size) { return elem_size == 4 && chains_v2 >= (long long)sm_count(); }

// Segment count.  Cutting the time axis costs an extra read of the tensors the carry depends on
// (8 instead of 5 tensor passes forward, 12 instead of 9 backward), so it pays only when batch x
// channels alone leaves most of the GPU idle: fewer than two wide chains per SM.
int auto_segments(long long B, long long L, long long D, int in_dtype) {
    if (B <= 0 || L <= 0 || D <= 0 || dtype_size(in_dtype) == 0) return 1;
    const long long chains = B * ((D + 63) / 64);
    const long long sms = sm_count();
    if (chains >= 2 * sms || f32_one_pass(chains, dtype_size(in_dtype))) return 1;
    long long want = (4 * sms) / chains;  // rounded down: never more chains than four per SM hold at once
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
int pick_stages(long long grid, int stage_bytes, int store_bytes, int fixed_bytes, int lo, int hi, F prefetch,
                long long total_budget = 15ll << 20) {
    const int forced = knob(K_STAGES, 0);
    if (forced >= lo && forced <= MAX_STAGES &&
        (long long)forced * stage_bytes + fixed_bytes + MAX_STAGES * 8 <= 227 * 1024)
        return forced;
    const long long sms = sm_count();
    const long long per_sm = (grid + sms - 1) / sms;
    const long long smem_cap = (228 * 1024) / (per_sm < 1 ? 1 : per_sm) - 1024;
    const long long budget = total_budget / (grid < 1 ? 1 : grid);
    int best = lo;
    for (int ns = lo; ns <= hi; ++ns) {
        const long long smem = (long long)ns * stage_bytes + fixed_bytes + MAX_STAGES * 8;
        if (smem > smem_cap || smem > 227 * 1024) break;
        if ((long long)prefetch(ns) * stage_bytes + store_bytes > budget) break;
        best = ns;
    }
    return best;
}

int make_plan(Plan& pl, long long B, long long L, long long D, int n_seg, int* status, int force_v = 0,
              int elem_size = 0) {
    if (n_seg < 1) n_seg = 1;
    long long seg_rows = (L + n_seg - 1) / n_seg;
    seg_rows = ((seg_rows + 31) / 32) * 32;  // whole tiles for either tile height
    n_seg = (int)((L + seg_rows - 1) / seg_rows);
    pl.V = pick_v(B, D, n_seg, elem_size);
    if (force_v > 0 && knob(K_V, 0) == 0) pl.V = force_v;
    pl.TB = pick_tb();
    const int chans = 32 * pl.V;
    Geom& g = pl.g;
    g.B = B; g.L = L; g.D = D;
    g.n_dtiles = (int)((D + chans - 1) / chans);
    g.n_seg = n_seg;
    g.seg_rows = (int)seg_rows;
    g.status = status;
    g.use_tma = 1;
    g.l2_hint = knob(K_L2HINT, 0);
    g.n_stages = 2;
    pl.chains = B * n_seg * g.n_dtiles;
    g.n_chains = pl.chains;
    pl.grid = concurrent_chains(pl.chains, false);
    return 0;
}

// Per kernel instantiation and device: the largest dynamic shared-memory size the function has been
// opted into, and how many of its CTAs fit on an SM at a given size.  Both are asked of the runtime
// once, not on every launch.
struct KernelCache {
    std::mutex mu;
    std::unordered_map<unsigned long long, int> smem_set;   // (kernel, device) -> bytes
    std::unordered_map<unsigned long long, int> per_sm;     // (kernel, device, smem, threads) -> CTAs per SM
};
KernelCache& kernel_cache() {
    static KernelCache c;
    return c;
}
inline unsigned long long kernel_key(const void* fn, int dev) {
    return (unsigned long long)reinterpret_cast<uintptr_t>(fn) * 64ull + (unsigned long long)dev;
}

template <typename K> int ensure_smem(K kernel, int smem_bytes) {
    KernelCache& kc = kernel_cache();
    const unsigned long long key = kernel_key(reinterpret_cast<const void*>(kernel), current_device());
    std::lock_guard<std::mutex> lock(kc.mu);
    auto it = kc.smem_set.find(key);
    if (it != kc.smem_set.end() && it->second >= smem_bytes) return 0;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return (int)e;
    kc.smem_set[key] = smem_bytes;
    return 0;
}

template <typename K, typename P>
int launch(K kernel, const P& params, long long grid, int smem_bytes, cudaStream_t stream, int threads = 32) {
    const int rc = ensure_smem(kernel, smem_bytes);
    if (rc) return rc;
    kernel<<<(unsigned)grid, threads, smem_bytes, stream>>>(params);
    return (int)cudaGetLastError();
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
    const int chans = 32 * pl.V, TB = prefers_tall_tiles(in_dtype, pl.V) ? 32 : pl.TB;
    bool tma = tma_ok(t0, g.B, g.L, g.D, sb, sl, dtype_size(in_dtype)) &&
               tma_ok(t1, g.B, g.L, g.D, sb, sl, dtype_size(in_dtype)) &&
               tma_ok(t2, g.B, g.L, g.D, sb2, sl2, dtype_size(dt2)) && knob(K_NO_TMA, 0) == 0;
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
    return dispatch(in_dtype, out_dt, pl.V, TB, [&](auto tin, auto tout, auto v, auto tb) -> int {
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
int chained_mode() { return knob(K_CHAINED, 1); }

// Chunk length: with about a thousand chunks in flight, the tensors the first pass leaves in L2 for the
// second one (three of them, 128 bytes per row) have to fit in the 126 MB L2 next to the streaming
// traffic; shorter chunks mean more look-backs.  Measured on B200, 1 x 2^20 x 2048 fp16: the forward is
// fastest with 192-224 rows (3.67 ms; 256: 3.81, 160: 3.77, 128: 3.84), the backward with 128 rows and
// two stages, which lets nine CTAs share an SM (6.83 ms; 256 rows and four stages: 6.93); 512 rows
// overflow the L2 and the second pass reads HBM again.  fp32 rows are twice as long: two stages (five CTAs
// per SM instead of three forward, two backward) and chunks of 112 / 64 rows took 1 x 65536 x 2048 fp32 from
// 4.71 / 4.82 TB/s forward / backward (128 rows, three / four stages) to 5.87 / 6.44; forward 96: 5.85,
// 128: 5.84, 160: 5.63, 256: 4.66; backward 48: 6.33, 80: 6.36, 96: 6.26; eight CTAs' worth of grid, which
// residency cuts to five, loses 1-5 % in the backward to uneven last rounds.
ChainedLayout chained_layout(long long B, long long L, long long D, int elem_size, bool backward) {
    ChainedLayout c;
    c.n_chains = B * ((D + 63) / 64);
    c.chunk_rows = knob(K_CHUNK_ROWS, elem_size == 2 ? (backward ? 128 : 192) : (backward ? 64 : 112));
    if (c.chunk_rows < TS) c.chunk_rows = TS;
    c.chunk_rows = (c.chunk_rows / TS) * TS;
    c.n_chunks = (int)((L + c.chunk_rows - 1) / c.chunk_rows);
    // two warps per scheduler: the two passes make a lone warp per scheduler compute-bound
    c.grid = knob(K_CHAINED_GRID, 0) > 0 ? knob(K_CHAINED_GRID, 0)
                                                  : (elem_size == 2 ? (backward ? 9ll : 8ll) : 5ll) * sm_count();
    const long long total = c.n_chains * c.n_chunks;
    if (c.grid > total) c.grid = total;
    if (c.grid < 1) c.grid = 1;
    // chunks of one chain in flight, plus slack; the kernels check before they reuse a slot, so a ring
    // that is too small (one chain far behind the others) costs waiting, not correctness
    long long need = (c.grid + c.n_chains - 1) / c.n_chains + 8;
    int slots = 4;
    while (slots < need) slots <<= 1;
    // tests shrink the ring so that slots change hands while readers still look for the old owner
    const int forced_slots = knob(K_CHAINED_SLOTS, 0);
    if (forced_slots >= 2 && forced_slots < slots) {
        slots = 2;
        while (slots * 2 <= forced_slots) slots <<= 1;
    }
    c.slots = slots;
    c.desc_off = 256;
    c.bytes = c.desc_off + (size_t)c.n_chains * slots * 96 * 16;
    c.zero_bytes = c.bytes;
    return c;
}

bool chained_shape_ok(long long B, long long L, long long D) {
    return B > 0 && L >= 4 * TS && D > 32 && B * ((D + 63) / 64) * ((L + TS - 1) / TS) < 0x7fffffffll;
}

// Which launches take the chained kernels by themselves (mode 1).  16-bit storage: below about 2.75 strips
// per SM the chained kernels (~182 Gelem/s fwd+bwd whatever the strip count) beat one warp per strip (168 at
// 384 strips, 196 at 448); the forward with 16-bit output leaves them at two strips per SM already, where wide
// strips on 32-row tiles overtake them (2^28 elements, D = 2048, bf16, TB/s: 320 strips 5.67 against 5.32 chained,
// 352: 6.15 against 5.37, 384: 6.53 against 5.28; 288: 5.12 against 5.37; the backward gains at most 4 %).
// fp32 storage: the forward below one strip per SM (f32_one_pass); the backward up to
// five strips per SM, where it holds 6.1-6.4 TB/s at every strip count while one warp per strip swings between
// 5.6 and 6.5 with how evenly the strips fill the SMs (416: 6.13 against 5.70, 640: 6.14 against 5.70,
// 288: 6.24 against 6.50; level from 768 strips on).
bool chained_wanted(long long B, long long L, long long D, int in_dtype, int out_dtype, bool backward) {
    const int mode = chained_mode();
    if (mode == 0 || !chained_shape_ok(B, L, D)) return false;
    if (mode != 1) return true;
    const long long strips = B * ((D + 63) / 64), sms = sm_count();
    if (dtype_size(in_dtype) == 4) return backward ? strips < 5 * sms : !f32_one_pass(strips, 4);
    if (!backward && dtype_size(out_dtype) == 2 && knob(K_TB, 0) == 0) return strips < 2 * sms;
    return 4 * strips < 11 * sms;
}

// Workspace of the chained kernels for one direction, 0 when that direction does not take them.
size_t chained_ws_bytes(long long B, long long L, long long D, int in_dtype, int out_dtype, bool backward) {
    if (!chained_wanted(B, L, D, in_dtype, out_dtype, backward)) return 0;
    return chained_layout(B, L, D, dtype_size(in_dtype), backward).bytes;
}
// Either direction, whatever the type of y / dy.
size_t chained_ws_bytes_any(long long B, long long L, long long D, int in_dtype) {
    const size_t f = chained_ws_bytes(B, L, D, in_dtype, QSSM_F32, false);
    const size_t r = chained_ws_bytes(B, L, D, in_dtype, QSSM_F32, true);
    return f > r ? f : r;
}

unsigned long long lookback_wait_ns() {
    const int ms = knob(K_WAIT_MS, 2000);
    return (unsigned long long)(ms < 1 ? 1 : ms) * 1000000ull;
}

// Zero the ticket counter and the descriptors.  Test hook (QSSM_TEST_SKIP_FIRST_CHUNK=1): start the
// counter past the first chunk of every chain, so that nothing ever publishes those chunks and every
// look-back wait runs into its limit - the way to exercise the bounded-wait error path on a healthy GPU.
int prepare_chained_ws(void* ws, const ChainedLayout& lay, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(ws, 0, lay.zero_bytes, stream);
    if (e != cudaSuccess) return (int)e;
    if (knob(K_TEST_SKIP_FIRST_CHUNK, 0) != 0) {
        static unsigned int start[MAX_DEVICES];
        const int dev = current_device();
        start[dev] = (unsigned int)lay.n_chains;
        e = cudaMemcpyAsync(ws, &start[dev], sizeof(unsigned int), cudaMemcpyHostToDevice, stream);
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

template <typename K> long long resident_ctas(K kernel, int threads, int smem) {
    if (ensure_smem(kernel, smem) != 0) return 0;
    KernelCache& kc = kernel_cache();
    const unsigned long long key =
        (kernel_key(reinterpret_cast<const void*>(kernel), current_device()) * 1048576ull + (unsigned)smem) * 2048ull +
        (unsigned)threads;
    int per_sm = 0;
    {
        std::lock_guard<std::mutex> lock(kc.mu);
        auto it = kc.per_sm.find(key);
        if (it != kc.per_sm.end()) per_sm = it->second;
    }
    if (per_sm == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess) return 0;
        std::lock_guard<std::mutex> lock(kc.mu);
        kc.per_sm[key] = per_sm;
    }
    return (long long)per_sm * sm_count();
}

}  // namespace

// =============================================================================================
// C ABI
// =============================================================================================
extern "C" {

int qssm_version(void) { return 200; }

int qssm_tune_set(const char* name, int value) {
    if (name == nullptr) return QSSM_E_NULL;
    if (strncmp(name, "QSSM_", 5) == 0) name += 5;
    for (int k = 0; k < K_COUNT; ++k)
        if (strcmp(name, kKnobNames[k]) == 0) {
            __atomic_store_n(&knobs().now[k], value, __ATOMIC_RELAXED);
            return 0;
        }
    return QSSM_E_SHAPE;
}

void qssm_tune_reset(void) {
    Knobs& k = knobs();
    for (int i = 0; i < K_COUNT; ++i) __atomic_store_n(&k.now[i], k.start[i], __ATOMIC_RELAXED);
}

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
    const size_t chained = chained_ws_bytes_any(B, L, D, in_dtype);
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
    if (n_seg_req == 0 && h_saved == nullptr && ws != nullptr && knob(K_NO_TMA, 0) == 0) {
        const size_t need = chained_ws_bytes(B, L, D, in_dtype, out_dtype, false);
        const int es = dtype_size(in_dtype), eo = dtype_size(out_dtype);
        if (need > 0 && ws_bytes >= need && tma_ok(x, B, L, D, in_stride_b, in_stride_l, es) &&
            tma_ok(a, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(b, B, L, D, in_stride_b, in_stride_l, es) &&
            tma_ok(c, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(y, B, L, D, out_stride_b, out_stride_l, eo)) {
            const ChainedLayout lay = chained_layout(B, L, D, es, false);
            ChainedParams cp;
            memset(&cp, 0, sizeof(cp));
            Geom& g = cp.f.g;
            g.B = B; g.L = L; g.D = D;
            g.n_dtiles = (int)((D + 63) / 64);
            g.n_seg = 1;
            g.seg_rows = 0;
            g.use_tma = 1;
            g.l2_hint = knob(K_CHAINED_HINT, 1);
            g.status = status_word;
            g.n_chains = lay.n_chains;
            g.n_out = knob(K_NOUT, 0) == 2 ? 2 : 3;
            g.n_stages = knob(K_STAGES, 0) >= 2 && knob(K_STAGES, 0) <= 8 ? knob(K_STAGES, 0) : (es == 2 ? 3 : 2);
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
            cp.wait_ns = lookback_wait_ns();
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
                    const int prc = prepare_chained_ws(ws, lay, stream);
                    if (prc) return prc;
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
    if ((rc = make_plan(pl, B, L, D, n_seg, status_word, 0, dtype_size(in_dtype)))) return rc;
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
    if (prefers_tall_tiles(in_dtype, pl.V) && eo == 2 && h_saved == nullptr && knob(K_FWD_TILE4, 0) == 0) pl.TB = 32;
    if (es == 4 && pl.g.n_seg == 1 && h_saved == nullptr && knob(K_TB, 0) == 0)
        pl.TB = f32_tile_rows(pl.V, pl.chains, false);
    const int chans = 32 * pl.V, TB = pl.TB;
    const long long hs_sb = L * D, hs_sl = D;
    bool tma = knob(K_NO_TMA, 0) == 0 && tma_ok(x, B, L, D, in_stride_b, in_stride_l, es) &&
               tma_ok(a, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(b, B, L, D, in_stride_b, in_stride_l, es) &&
               tma_ok(c, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(y, B, L, D, out_stride_b, out_stride_l, eo) &&
               tma_ok(h_saved, B, L, D, hs_sb, hs_sl, 4);
    fp.g.use_tma = tma ? 1 : 0;
    fp.tile_h = tile_h;
    fp.h_in = seeds;
    fp.h_last = h_last;

    const int nin = c != nullptr ? 4 : 3;
    const bool has_c = c != nullptr, save_h = h_saved != nullptr;

    // Forward that also stores fp32 h (6 of its 14 bytes per element are writes): four adjacent strips per
    // CTA on 512-byte-wide tiles, under the same conditions as the four-strip backward.  The plain forward
    // (20 % writes) is at the copy rate with one warp per CTA and stays there.
    bool wide = tma && knob(K_WIDE, 1) != 0 && es == 2 && pl.V == 2 && TB == TS && pl.g.n_dtiles >= WIDE_W &&
                (save_h || knob(K_FWD_TILE4, 0) != 0);
    const long long groups = B * n_seg * ((pl.g.n_dtiles + WIDE_W - 1) / WIDE_W);
    const long long rounds = (groups + sm_count() - 1) / sm_count();
    if (wide && (double)groups / (double)(rounds * sm_count()) < 0.85) wide = false;

    // tensor maps, encoded once with the box of the kernel that will run
    {
        const int box = wide ? WIDE_W * chans : chans;
        if ((rc = fill_desc(fp.x, x, in_dtype, B, L, D, in_stride_b, in_stride_l, box, TB, tma))) return rc;
        if ((rc = fill_desc(fp.a, a, in_dtype, B, L, D, in_stride_b, in_stride_l, box, TB, tma))) return rc;
        if ((rc = fill_desc(fp.b, b, in_dtype, B, L, D, in_stride_b, in_stride_l, box, TB, tma))) return rc;
        if ((rc = fill_desc(fp.c, c, in_dtype, B, L, D, in_stride_b, in_stride_l, box, TB, tma))) return rc;
        if ((rc = fill_desc(fp.y, y, out_dtype, B, L, D, out_stride_b, out_stride_l, box, TB, tma))) return rc;
        if ((rc = fill_desc(fp.hs, h_saved, QSSM_F32, B, L, D, hs_sb, hs_sl, box, TB, tma))) return rc;
    }

    if (wide) {
        {
            const int box = WIDE_W * chans;
            const long long ctas = (groups + rounds - 1) / rounds;  // equal rounds, at most one CTA per SM
            const int stage4 = nin * TB * box * es;
            const int outbuf4 = TB * box * eo + (save_h ? TB * box * 4 : 0);
            const int n_out4 = knob(K_NOUT, 2) == 3 ? 3 : 2;
            fp.g.n_out = n_out4;
            // measured (bf16, h stored): 3 stages 0.559 ms on the cfg1 shape and 4.72 ms on cfg4, 4 stages
            // 0.613 / 4.95 ms, 2 stages 0.669 / 4.98 ms; two or three staging tiles make no difference
            fp.g.n_stages = pick_stages(ctas, stage4, (n_out4 - 1) * outbuf4, n_out4 * outbuf4, 2, 3,
                                        [](int ns) { return ns - 1; });
            const int smem4 = fp.g.n_stages * stage4 + n_out4 * outbuf4 + MAX_STAGES * 8;
            return dispatch(in_dtype, out_dtype, 2, TS, [&](auto tin, auto tout, auto, auto) -> int {
                using Tin = decltype(tin);
                using Tout = decltype(tout);
                if constexpr (sizeof(Tin) == 2) {
                    const int th = 32 * WIDE_W;
                    if (has_c && save_h)
                        return launch(scan_fwd_tile4_kernel<Tin, Tout, true, true>, fp, ctas, smem4, stream, th);
                    if (has_c) return launch(scan_fwd_tile4_kernel<Tin, Tout, true, false>, fp, ctas, smem4, stream, th);
                    if (save_h) return launch(scan_fwd_tile4_kernel<Tin, Tout, false, true>, fp, ctas, smem4, stream, th);
                    return launch(scan_fwd_tile4_kernel<Tin, Tout, false, false>, fp, ctas, smem4, stream, th);
                } else {
                    return QSSM_E_DTYPE;
                }
            });
        }
    }

    const int stage = nin * TB * chans * es;
    const int outbuf = TB * chans * eo + (h_saved != nullptr ? TB * chans * 4 : 0);
    int n_out = knob(K_NOUT, 3);
    if (n_out < 2) n_out = 2;
    if (n_out > 4) n_out = 4;
    fp.g.n_out = n_out;
    fp.g.n_stages = pick_stages(pl.grid, stage, (n_out - 1) * outbuf, n_out * outbuf, 2, 8,
                                [](int ns) { return ns - 1; });
    const int smem = fp.g.n_stages * stage + n_out * outbuf + MAX_STAGES * 8;

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
    // "aggregates already in ws" has no meaning here: no aggregate entry point writes the built-in array
    if (n_seg_req < 0) return QSSM_E_SHAPE;
    // Scratch the call would use; refuse rather than quietly run another way.  With n_seg = 0 the library
    // may pick the single-pass kernels for few-chain shapes, whose ticket and descriptor area then lives in
    // the array too (and is zeroed by a memset on the stream at the start of the call).
    const int n_seg = n_seg_req != 0 ? n_seg_req : auto_segments(B, L, D, in_dtype);
    size_t need = ws_bytes_for(B, D, n_seg);
    if (n_seg_req == 0 && h_saved == nullptr) {
        const size_t chained = chained_ws_bytes(B, L, D, in_dtype, out_dtype, false);
        if (chained > need) need = chained;
    }
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
    if (n_seg_req == 0 && h_saved == nullptr && ws != nullptr && knob(K_NO_TMA, 0) == 0) {
        const size_t need = chained_ws_bytes(B, L, D, in_dtype, out_dtype, true);
        const int es = dtype_size(in_dtype), eo = dtype_size(out_dtype);
        const long long n_tiles_b = (L + TS - 1) / TS;
        const long long g_sb = L * D, g_sl = D;
        if (need > 0 && ws_bytes >= need && tma_ok(x, B, L, D, in_stride_b, in_stride_l, es) &&
            tma_ok(a, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(b, B, L, D, in_stride_b, in_stride_l, es) &&
            tma_ok(c, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(dy, B, L, D, dy_stride_b, dy_stride_l, eo) &&
            tma_ok(dx, B, L, D, g_sb, g_sl, es) && tma_ok(da, B, L, D, g_sb, g_sl, es) &&
            tma_ok(db, B, L, D, g_sb, g_sl, es) && tma_ok(dc, B, L, D, g_sb, g_sl, es) &&
            tma_ok(tile_h, B, n_tiles_b, D, n_tiles_b * D, D, 4)) {
            const ChainedLayout lay = chained_layout(B, L, D, es, true);
            ChainedBwdParams cp;
            memset(&cp, 0, sizeof(cp));
            Geom& g = cp.f.g;
            g.B = B; g.L = L; g.D = D;
            g.n_dtiles = (int)((D + 63) / 64);
            g.n_seg = 1;
            g.use_tma = 1;
            g.l2_hint = knob(K_CHAINED_HINT, 1);
            g.status = status_word;
            g.n_chains = lay.n_chains;
            g.n_stages = knob(K_STAGES, 0) >= 2 && knob(K_STAGES, 0) <= 8 ? knob(K_STAGES, 0)
                                                                                          : 2;
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
            cp.wait_ns = lookback_wait_ns();
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
                const int prc = prepare_chained_ws(ws, lay, stream);
                if (prc) return prc;
                return launch(kernel, cp, grid, smem, stream);
            });
        }
    }

    int n_seg = 1;
    if ((rc = resolve_segments(n_seg_req, B, L, D, in_dtype, ws, ws_bytes, &n_seg))) return rc;
    Plan pl;
    if ((rc = make_plan(pl, B, L, D, n_seg, status_word, 0, dtype_size(in_dtype)))) return rc;
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
    const bool saved = h_saved != nullptr;
    if (es == 4 && pl.g.n_seg == 1 && !saved && knob(K_TB, 0) == 0) pl.TB = f32_tile_rows(pl.V, pl.chains, true);
    const int chans = 32 * pl.V, TB = pl.TB;
    const long long n_tiles_b = (L + TS - 1) / TS;
    const long long g_sb = L * D, g_sl = D;  // gradients and h_saved are contiguous
    bool tma = knob(K_NO_TMA, 0) == 0 && tma_ok(x, B, L, D, in_stride_b, in_stride_l, es) &&
               tma_ok(a, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(b, B, L, D, in_stride_b, in_stride_l, es) &&
               tma_ok(c, B, L, D, in_stride_b, in_stride_l, es) && tma_ok(dy, B, L, D, dy_stride_b, dy_stride_l, eo) &&
               tma_ok(dx, B, L, D, g_sb, g_sl, es) && tma_ok(da, B, L, D, g_sb, g_sl, es) &&
               tma_ok(db, B, L, D, g_sb, g_sl, es) && tma_ok(dc, B, L, D, g_sb, g_sl, es) &&
               (saved ? tma_ok(h_saved, B, L, D, g_sb, g_sl, 4) : tma_ok(tile_h, B, n_tiles_b, D, n_tiles_b * D, D, 4));
    bp.g.use_tma = tma ? 1 : 0;
    // Four adjacent strips per CTA, loaded and stored as one 512-byte-wide tile per tensor (16-bit storage).
    // One such CTA fits per SM, so the groups must fill whole rounds of SM-count CTAs reasonably well;
    // otherwise (e.g. 152 groups on 148 SMs) the one-warp-per-CTA kernel, which packs finer, is used.
    bool wide = tma && knob(K_WIDE, 1) != 0 && es == 2 && pl.V == 2 && TB == TS && pl.g.n_dtiles >= WIDE_W;
    if (wide) {
        const long long groups = B * n_seg * ((pl.g.n_dtiles + WIDE_W - 1) / WIDE_W);
        const long long rounds = (groups + sm_count() - 1) / sm_count();
        if ((double)groups / (double)(rounds * sm_count()) < 0.85) wide = false;
    }
    // tensor maps, encoded once with the box of the kernel that will run
    const int box = wide ? WIDE_W * chans : chans;
    if ((rc = fill_desc(bp.x, x, in_dtype, B, L, D, in_stride_b, in_stride_l, box, TB, tma))) return rc;
    if ((rc = fill_desc(bp.a, a, in_dtype, B, L, D, in_stride_b, in_stride_l, box, TB, tma))) return rc;
    if ((rc = fill_desc(bp.b, b, in_dtype, B, L, D, in_stride_b, in_stride_l, box, TB, tma))) return rc;
    if ((rc = fill_desc(bp.c, c, in_dtype, B, L, D, in_stride_b, in_stride_l, box, TB, tma))) return rc;
    if ((rc = fill_desc(bp.dy, dy, out_dtype, B, L, D, dy_stride_b, dy_stride_l, box, TB, tma))) return rc;
    if (saved)
        rc = fill_desc(bp.hsrc, h_saved, QSSM_F32, B, L, D, g_sb, g_sl, box, TB + 1, tma);
    else
        rc = fill_desc(bp.hsrc, tile_h, QSSM_F32, B, n_tiles_b, D, n_tiles_b * D, D, box, wide ? 1 : TB / TS, tma);
    if (rc) return rc;
    if ((rc = fill_desc(bp.dx, dx, in_dtype, B, L, D, g_sb, g_sl, box, TB, tma))) return rc;
    if ((rc = fill_desc(bp.da, da, in_dtype, B, L, D, g_sb, g_sl, box, TB, tma))) return rc;
    if ((rc = fill_desc(bp.db, db, in_dtype, B, L, D, g_sb, g_sl, box, TB, tma))) return rc;
    if ((rc = fill_desc(bp.dc, dc, in_dtype, B, L, D, g_sb, g_sl, box, TB, tma))) return rc;
    bp.h_in = h_in;
    bp.g_in = seeds;
    bp.g_first = g_first;

    const int hrow = chans * 4;
    const int h_tile = saved ? (TB + 1) * hrow : (TB / TS) * hrow;
    const int stage = 4 * TB * chans * es + TB * chans * eo + ((h_tile + 127) / 128) * 128;
    const int grad_tile = 4 * TB * chans * es;  // the four gradient tiles of one strip
    if (wide) {
        const long long n_groups = B * n_seg * ((pl.g.n_dtiles + WIDE_W - 1) / WIDE_W);
        const long long wide_rounds = (n_groups + sm_count() - 1) / sm_count();
        const long long ctas = (n_groups + wide_rounds - 1) / wide_rounds;  // equal rounds, at most one CTA per SM
        const int stage4 = WIDE_W * (4 * TB * chans * es + TB * chans * eo + h_tile);
        // measured: with CTA-wide tiles the best depth corresponds to about 20 MB in flight
        // (cfg1, 128 CTAs: 4 stages 0.755 ms, 3 stages 0.820 ms; cfg4, 147 CTAs: 3 stages 6.28 ms, 4 stages 6.59 ms)
        bp.g.n_stages = pick_stages(ctas, stage4, 2 * WIDE_W * grad_tile, 0, 2, 5,
                                    [](int ns) { return ns > 2 ? ns - 2 : 1; }, 20ll << 20);
        const int smem = bp.g.n_stages * stage4 + MAX_STAGES * 8;
        return dispatch(in_dtype, out_dtype, 2, TS, [&](auto tin, auto tout, auto, auto) -> int {
            using Tin = decltype(tin);
            using Tout = decltype(tout);
            if constexpr (sizeof(Tin) == 2) {
                if (saved) return launch(scan_bwd_tile4_kernel<Tin, Tout, true>, bp, ctas, smem, stream, 32 * WIDE_W);
                return launch(scan_bwd_tile4_kernel<Tin, Tout, false>, bp, ctas, smem, stream, 32 * WIDE_W);
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

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// scan with fused gate activations
// ---------------------------------------------------------------------------------------------
namespace {

// Calls f(Tin{}, Tgate{}, Tout{}, Int<V>{}); Tout is the dtype of y / dy.
template <typename F> int dispatch_gated(int in_dt, int gate_dt, int out_dt, int V, F&& f) {
    auto with_v = [&](auto tin, auto tg, auto tout) -> int {
        if (V == 1) return f(tin, tg, tout, Int<1>{});
        return f(tin, tg, tout, Int<2>{});
    };
    if (in_dt == QSSM_F32 && out_dt == QSSM_F32) {
        if (gate_dt == QSSM_F32) return with_v(float{}, float{}, float{});
        if (gate_dt == QSSM_BF16) return with_v(float{}, __nv_bfloat16{}, float{});
        if (gate_dt == QSSM_F16) return with_v(float{}, __half{}, float{});
    }
    if (in_dt == QSSM_BF16 && gate_dt == QSSM_BF16) {
        if (out_dt == QSSM_BF16) return with_v(__nv_bfloat16{}, __nv_bfloat16{}, __nv_bfloat16{});
        if (out_dt == QSSM_F32) return with_v(__nv_bfloat16{}, __nv_bfloat16{}, float{});
    }
    if (in_dt == QSSM_F16 && gate_dt == QSSM_F16) {
        if (out_dt == QSSM_F16) return with_v(__half{}, __half{}, __half{});
        if (out_dt == QSSM_F32) return with_v(__half{}, __half{}, float{});
    }
    return QSSM_E_DTYPE;
}

int check_gated(int64_t B, int64_t L, int64_t D, int in_dtype, int gate_dtype, int out_dtype) {
    if (B < 0 || L < 0 || D < 0 || L >= (1ll << 31) - 64 || B >= (1ll << 31)) return QSSM_E_SHAPE;
    if (dtype_size(in_dtype) == 0 || dtype_size(gate_dtype) == 0 || dtype_size(out_dtype) == 0) return QSSM_E_DTYPE;
    return 0;
}

}  // namespace

extern "C" {

int qssm_gated_scan_fwd(const void* pa, const void* px, const void* pc1, const void* pc2, const void* pd, void* y,
                        float* tile_h, const float* h_in, float* h_last, int64_t B, int64_t L, int64_t D,
                        int64_t in_stride_b, int64_t in_stride_l, int64_t out_stride_b, int64_t out_stride_l,
                        int in_dtype, int gate_dtype, int out_dtype, int* status_word, void* stream_v) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    int rc = check_gated(B, L, D, in_dtype, gate_dtype, out_dtype);
    if (rc) return rc;
    if (B == 0 || L == 0 || D == 0) return 0;
    if (pa == nullptr || px == nullptr || pc1 == nullptr || pc2 == nullptr || pd == nullptr || y == nullptr)
        return QSSM_E_NULL;
    if ((rc = check_strides(L, D, in_stride_b, in_stride_l))) return rc;
    if ((rc = check_strides(L, D, out_stride_b, out_stride_l))) return rc;
    const int es = dtype_size(in_dtype), eo = dtype_size(out_dtype);
    const void* ins[5] = {pa, px, pc1, pc2, pd};
    for (const void* t : ins)
        if (!tma_ok(t, B, L, D, in_stride_b, in_stride_l, es)) return QSSM_E_STRIDE;
    if (!tma_ok(y, B, L, D, out_stride_b, out_stride_l, eo)) return QSSM_E_STRIDE;

    // 16-bit projection outputs with fp32 y: twice as many warps on strips half as wide are faster (16 x 4096 x 4096,
    // forward 0.66 ms against 0.82 ms); with 16-bit y the wide strips win (0.50 against 0.69 ms), and with fp32
    // projection outputs too (0.95 ms either way)
    Plan pl;
    if ((rc = make_plan(pl, B, L, D, 1, status_word, es == 2 && eo == 4 ? 1 : 0))) return rc;
    pl.grid = concurrent_chains_gated(pl.chains);
    GatedFwdParams fp;
    memset(&fp, 0, sizeof(fp));
    fp.g = pl.g;
    const int chans = 32 * pl.V;
    TensorDesc* descs[5] = {&fp.pa, &fp.px, &fp.pc1, &fp.pc2, &fp.pd};
    for (int i = 0; i < 5; ++i)
        if ((rc = fill_desc(*descs[i], ins[i], in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TS, true))) return rc;
    if ((rc = fill_desc(fp.y, y, out_dtype, B, L, D, out_stride_b, out_stride_l, chans, TS, true))) return rc;
    fp.tile_h = tile_h;
    fp.h_in = h_in;
    fp.h_last = h_last;
    const int stage = 5 * TS * chans * es;
    const int outbuf = TS * chans * eo;
    fp.g.n_out = 3;
    fp.g.n_stages = pick_stages(pl.grid, stage, 2 * outbuf, 3 * outbuf, 2, 8, [](int ns) { return ns - 1; });
    const int smem = fp.g.n_stages * stage + 3 * outbuf + MAX_STAGES * 8;
    return dispatch_gated(in_dtype, gate_dtype, out_dtype, pl.V, [&](auto tin, auto tg, auto tout, auto v) -> int {
        return launch(gated_fwd_kernel<decltype(tin), decltype(tg), decltype(tout), decltype(v)::value>, fp, pl.grid,
                      smem, stream);
    });
}

int qssm_gated_scan_bwd(const void* pa, const void* px, const void* pc1, const void* pc2, const void* pd,
                        const void* dy, const float* tile_h, const float* g_in, float* g_first, void* dpa, void* dpx,
                        void* dpc1, void* dpc2, void* dpd, int64_t B, int64_t L, int64_t D, int64_t in_stride_b,
                        int64_t in_stride_l, int64_t dy_stride_b, int64_t dy_stride_l, int in_dtype, int gate_dtype,
                        int out_dtype, int* status_word, void* stream_v) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    int rc = check_gated(B, L, D, in_dtype, gate_dtype, out_dtype);
    if (rc) return rc;
    if (B == 0 || L == 0 || D == 0) return 0;
    const void* ins[5] = {pa, px, pc1, pc2, pd};
    void* outs[5] = {dpa, dpx, dpc1, dpc2, dpd};
    for (int i = 0; i < 5; ++i)
        if (ins[i] == nullptr || outs[i] == nullptr) return QSSM_E_NULL;
    if (dy == nullptr) return QSSM_E_NULL;
    if (tile_h == nullptr) return QSSM_E_NEED_H;
    if ((rc = check_strides(L, D, in_stride_b, in_stride_l))) return rc;
    if ((rc = check_strides(L, D, dy_stride_b, dy_stride_l))) return rc;
    const int es = dtype_size(in_dtype), eo = dtype_size(out_dtype);
    const long long g_sb = L * D, g_sl = D, n_tiles_b = (L + TS - 1) / TS;
    for (int i = 0; i < 5; ++i)
        if (!tma_ok(ins[i], B, L, D, in_stride_b, in_stride_l, es) || !tma_ok(outs[i], B, L, D, g_sb, g_sl, es))
            return QSSM_E_STRIDE;
    if (!tma_ok(dy, B, L, D, dy_stride_b, dy_stride_l, eo) || !tma_ok(tile_h, B, n_tiles_b, D, n_tiles_b * D, D, 4))
        return QSSM_E_STRIDE;

    // 16-bit projection outputs: twice as many warps on strips half as wide are faster (16 x 4096 x 4096, backward
    // 1.15 ms against 1.31 ms with fp32 dy, 1.13 against 1.19 with 16-bit dy); fp32 ones are not (2.00 against 2.41)
    Plan pl;
    if ((rc = make_plan(pl, B, L, D, 1, status_word, dtype_size(in_dtype) == 2 ? 1 : 0))) return rc;
    pl.grid = concurrent_chains_gated(pl.chains);
    GatedBwdParams bp;
    memset(&bp, 0, sizeof(bp));
    bp.g = pl.g;
    const int chans = 32 * pl.V;
    TensorDesc* din[5] = {&bp.pa, &bp.px, &bp.pc1, &bp.pc2, &bp.pd};
    TensorDesc* dout[5] = {&bp.dpa, &bp.dpx, &bp.dpc1, &bp.dpc2, &bp.dpd};
    for (int i = 0; i < 5; ++i) {
        if ((rc = fill_desc(*din[i], ins[i], in_dtype, B, L, D, in_stride_b, in_stride_l, chans, TS, true))) return rc;
        if ((rc = fill_desc(*dout[i], outs[i], in_dtype, B, L, D, g_sb, g_sl, chans, TS, true))) return rc;
    }
    if ((rc = fill_desc(bp.dy, dy, out_dtype, B, L, D, dy_stride_b, dy_stride_l, chans, TS, true))) return rc;
    if ((rc = fill_desc(bp.th, tile_h, QSSM_F32, B, n_tiles_b, D, n_tiles_b * D, D, chans, 1, true))) return rc;
    bp.g_in = g_in;
    bp.g_first = g_first;
    const int stage = 5 * TS * chans * es + TS * chans * eo + ((chans * 4 + 127) / 128) * 128;
    bp.g.n_stages = pick_stages(pl.grid, stage, 2 * 5 * TS * chans * es, 0, 2, 6,
                                [](int ns) { return ns > 2 ? ns - 2 : 1; });
    const int smem = bp.g.n_stages * stage + MAX_STAGES * 8;
    return dispatch_gated(in_dtype, gate_dtype, out_dtype, pl.V, [&](auto tin, auto tg, auto tout, auto v) -> int {
        return launch(gated_bwd_kernel<decltype(tin), decltype(tg), decltype(tout), decltype(v)::value>, bp, pl.grid,
                      smem, stream);
    });
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

// =============================================================================================
// RMS normalisation
// =============================================================================================
namespace {

constexpr int NORM_CTAS_PER_SM = 4;  // upper bound used to size the scratch
constexpr int NORM_FWD_ELEMS = 128;  // elements per lane held in registers: rows of up to 4096 in the forward,
constexpr int NORM_BWD_ELEMS = 64;   // 2048 in the backward (x, w*dy and the dw sums: three values per element)

int norm_check(const void* a, long long stride, long long H, int es) {
    const long long align = es == 4 ? 16 : 8;
    if (reinterpret_cast<uintptr_t>(a) % align != 0 || (stride * es) % align != 0 || stride < H) return QSSM_E_STRIDE;
    return 0;
}
// 16-bit rows that can be moved 16 bytes (eight elements) per lane and access
bool norm_wide_ok(const void* a, long long stride, long long H) {
    return H % 8 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0 && (stride * 2) % 16 == 0;
}

// calls f(T{}, Int<NCH>{}, Int<EPL>{}) for the element type, the number of 32*EPL-element chunks held in
// registers (0 = rows longer than the register budget of max_elems elements per lane: read twice) and the
// elements per lane and access (8 only for 16-bit rows with `wide`)
template <typename F> int norm_dispatch(int dtype, long long H, int max_elems, bool wide, F&& f) {
    auto with_type = [&](auto t, auto epl) -> int {
        constexpr int EPL = decltype(epl)::value;
        const long long n = (H + 32 * EPL - 1) / (32 * EPL);
        if (n * EPL > max_elems) return f(t, Int<0>{}, epl);
        if (n <= 1) return f(t, Int<1>{}, epl);
        if (n <= 2) return f(t, Int<2>{}, epl);
        if (n <= 4) return f(t, Int<4>{}, epl);
        if (n <= 8) return f(t, Int<8>{}, epl);
        if (n <= 16) return f(t, Int<16>{}, epl);
        return f(t, Int<32>{}, epl);
    };
    switch (dtype) {
        case QSSM_F32: return with_type(float{}, Int<4>{});
        case QSSM_F16: return wide ? with_type(__half{}, Int<8>{}) : with_type(__half{}, Int<4>{});
        case QSSM_BF16: return wide ? with_type(__nv_bfloat16{}, Int<8>{}) : with_type(__nv_bfloat16{}, Int<4>{});
        default: return QSSM_E_DTYPE;
    }
}

template <typename K> long long norm_grid(K kernel, long long rows, int smem) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 32 * NORM_WARPS, smem) != cudaSuccess) return 0;
    if (per_sm > NORM_CTAS_PER_SM) per_sm = NORM_CTAS_PER_SM;
    long long grid = (long long)per_sm * sm_count();
    const long long need = (rows + NORM_WARPS - 1) / NORM_WARPS;
    if (grid > need) grid = need;
    return grid;
}

}  // namespace

extern "C" {

size_t qssm_rmsnorm_workspace_bytes(int64_t H) {
    if (H <= 0) return 0;
    // one partial row of dw per CTA, or per warp when rows are too long for the backward's registers
    const size_t parts = (size_t)sm_count() * NORM_CTAS_PER_SM * (H > 32 * NORM_BWD_ELEMS ? NORM_WARPS : 1);
    return parts * (size_t)H * 4;
}

int qssm_rmsnorm_fwd(const void* x, const float* w, void* y, float* rstd, int64_t rows, int64_t H, int64_t x_stride,
                     int64_t y_stride, float eps, int dtype, void* stream_v) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int es = dtype_size(dtype);
    if (es == 0) return QSSM_E_DTYPE;
    if (rows < 0 || H < 0 || H >= (1ll << 30)) return QSSM_E_SHAPE;
    if (rows == 0 || H == 0) return 0;
    if (x == nullptr || w == nullptr || y == nullptr) return QSSM_E_NULL;
    int rc;
    if (H % 4 != 0) return QSSM_E_STRIDE;
    if ((rc = norm_check(x, x_stride, H, es)) || (rc = norm_check(y, y_stride, H, es)) || (rc = norm_check(w, H, H, 4)))
        return rc;
    NormParams p;
    memset(&p, 0, sizeof(p));
    p.x = x; p.w = w; p.y = y; p.rstd = rstd;
    p.rows = rows; p.x_stride = x_stride; p.y_stride = y_stride; p.H = (int)H; p.eps = eps;
    const bool wide = es == 2 && norm_wide_ok(x, x_stride, H) && norm_wide_ok(y, y_stride, H);
    return norm_dispatch(dtype, H, NORM_FWD_ELEMS, wide, [&](auto t, auto nch, auto epl) -> int {
        using T = decltype(t);
        auto kernel = rmsnorm_fwd_kernel<T, decltype(nch)::value, decltype(epl)::value>;
        const long long grid = norm_grid(kernel, rows, 0);
        if (grid < 1) return QSSM_E_SHAPE;
        kernel<<<(unsigned)grid, 32 * NORM_WARPS, 0, stream>>>(p);
        return (int)cudaGetLastError();
    });
}

int qssm_rmsnorm_bwd(const void* x, const float* w, const void* dy, const float* rstd, void* dx, float* dw, void* ws,
                     size_t ws_bytes, int64_t rows, int64_t H, int64_t x_stride, int64_t dy_stride, int64_t dx_stride,
                     int dtype, void* stream_v) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    const int es = dtype_size(dtype);
    if (es == 0) return QSSM_E_DTYPE;
    if (rows < 0 || H < 0 || H >= (1ll << 30)) return QSSM_E_SHAPE;
    if (H == 0) return 0;
    if (dw == nullptr) return QSSM_E_NULL;
    if (rows == 0) return (int)cudaMemsetAsync(dw, 0, (size_t)H * 4, stream);
    if (x == nullptr || w == nullptr || dy == nullptr || rstd == nullptr || dx == nullptr || ws == nullptr)
        return QSSM_E_NULL;
    int rc;
    if (H % 4 != 0) return QSSM_E_STRIDE;
    if ((rc = norm_check(x, x_stride, H, es)) || (rc = norm_check(dy, dy_stride, H, es)) ||
        (rc = norm_check(dx, dx_stride, H, es)) || (rc = norm_check(w, H, H, 4)) || (rc = norm_check(ws, H, H, 4)))
        return rc;
    if (ws_bytes < qssm_rmsnorm_workspace_bytes(H)) return QSSM_E_WS;
    NormParams p;
    memset(&p, 0, sizeof(p));
    p.x = x; p.w = w; p.y = dx; p.dy = dy; p.rstd = const_cast<float*>(rstd);
    p.dw_part = static_cast<float*>(ws);
    p.rows = rows; p.x_stride = x_stride; p.y_stride = dx_stride; p.dy_stride = dy_stride; p.H = (int)H;
    const bool wide = es == 2 && norm_wide_ok(x, x_stride, H) && norm_wide_ok(dy, dy_stride, H) &&
                      norm_wide_ok(dx, dx_stride, H);
    return norm_dispatch(dtype, H, NORM_BWD_ELEMS, wide, [&](auto t, auto nch, auto epl) -> int {
        using T = decltype(t);
        constexpr int NCH = decltype(nch)::value, EPL = decltype(epl)::value;
        if constexpr (NCH * EPL > NORM_BWD_ELEMS) {
            return QSSM_E_SHAPE;  // never dispatched: longer rows take NCH = 0
        } else {
            auto kernel = rmsnorm_bwd_kernel<T, NCH, EPL>;
            const int smem = NCH > 0 ? (int)H * 4 : 0;
            const long long grid = norm_grid(kernel, rows, smem);
            if (grid < 1) return QSSM_E_SHAPE;
            kernel<<<(unsigned)grid, 32 * NORM_WARPS, smem, stream>>>(p);
            const int e = (int)cudaGetLastError();
            if (e) return e;
            const long long parts = grid * (NCH > 0 ? 1 : NORM_WARPS);
            rmsnorm_dw_kernel<<<(unsigned)((H + 31) / 32), 256, 0, stream>>>(p.dw_part, dw, parts, (int)H);
            return (int)cudaGetLastError();
        }
    });
}

// ---------------------------------------------------------------------------------------------
// carry exchange through peer memory
// ---------------------------------------------------------------------------------------------
static_assert(QSSM_MAX_PEERS == MAX_PEERS && QSSM_PEER_SLOTS == PEER_SLOTS, "header and kernels disagree");

size_t qssm_peer_inbox_bytes(int world, int64_t n_chan) {
    if (world < 1 || n_chan < 0) return 0;
    const size_t data = (size_t)PEER_SLOTS * (size_t)world * 2 * (size_t)n_chan * sizeof(float);
    return ((data + 255) / 256) * 256 + (size_t)PEER_SLOTS * (size_t)world * sizeof(int);
}

size_t qssm_peer_flags_offset(int world, int64_t n_chan) {
    if (world < 1 || n_chan < 0) return 0;
    const size_t data = (size_t)PEER_SLOTS * (size_t)world * 2 * (size_t)n_chan * sizeof(float);
    return ((data + 255) / 256) * 256;
}

int qssm_carry_push(const float* first, const float* second, int64_t n_chan, void* const* peer_inbox,
                    unsigned int* counters, int rank, int world, int slot, int epoch, void* stream) {
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world || slot < 0 || slot >= PEER_SLOTS || n_chan < 0)
        return QSSM_E_SHAPE;
    if (n_chan == 0) return 0;
    if (first == nullptr || second == nullptr || peer_inbox == nullptr || counters == nullptr) return QSSM_E_NULL;
    PeerPushParams p;
    memset(&p, 0, sizeof(p));
    p.first = first; p.second = second; p.counters = counters; p.n_chan = n_chan;
    p.rank = rank; p.world = world; p.slot = slot; p.epoch = epoch;
    const size_t flags_off = qssm_peer_flags_offset(world, n_chan);
    for (int k = 0; k < world; ++k) {
        if (peer_inbox[k] == nullptr) return QSSM_E_NULL;
        p.inbox[k] = static_cast<float*>(peer_inbox[k]);
        p.flags[k] = reinterpret_cast<int*>(static_cast<unsigned char*>(peer_inbox[k]) + flags_off);
    }
    long long per_peer = (n_chan + 1023) / 1024;  // about four elements of each array per thread
    if (per_peer > 32) per_peer = 32;
    carry_push_kernel<<<dim3((unsigned)per_peer, (unsigned)world), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return (int)cudaGetLastError();
}

int qssm_carry_wait_fold(const void* inbox, int64_t n_chan, int rank, int world, int slot, int epoch, int reverse,
                         const float* seed, float* carry, int wait_ms, int* status_word, void* stream) {
    if (world < 1 || world > MAX_PEERS || rank < 0 || rank >= world || slot < 0 || slot >= PEER_SLOTS || n_chan < 0)
        return QSSM_E_SHAPE;
    if (n_chan == 0) return 0;
    if (inbox == nullptr || carry == nullptr) return QSSM_E_NULL;
    long long grid = (n_chan + 255) / 256;
    if (grid > 2ll * sm_count()) grid = 2ll * sm_count();
    const unsigned long long wait_ns = (unsigned long long)(wait_ms < 1 ? 1 : wait_ms) * 1000000ull;
    const int* flags = reinterpret_cast<const int*>(static_cast<const unsigned char*>(inbox) +
                                                    qssm_peer_flags_offset(world, n_chan));
    carry_wait_fold_kernel<<<(unsigned)grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float*>(inbox), flags, n_chan, rank, world, slot, epoch, reverse, seed, carry, wait_ns,
        status_word);
    return (int)cudaGetLastError();
}

}  // extern "C"
