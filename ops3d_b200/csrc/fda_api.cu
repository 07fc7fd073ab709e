// Host side of the C ABI declared in include/fda_b200.h: argument validation, dtype
// dispatch and kernel launches.  No torch types, no allocation, nothing but the CUDA runtime.
#include "../../include/fda_b200.h"

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <type_traits>
#include <utility>

#include "fda_backward.cuh"
#include "fda_backward_binned.cuh"
#include "fda_backward_sorted.cuh"
#include "fda_backward_touched.cuh"
#include "fda_config.h"
#include "fda_forward.cuh"

namespace {

thread_local int g_last_cuda_error = 0;

inline int cuda_fail(cudaError_t e) {
    g_last_cuda_error = (int)e;
    return FDA_ERR_CUDA;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int dtype_size(int dt) { return dt == FDA_DTYPE_F32 ? 4 : 2; }

struct Shape {
    int B, N, G, D, L, Q, K, vdt, pdt;
};

int validate(const Shape &s, int im2col_step) {
    if (s.vdt < 0 || s.vdt > 2 || s.pdt < 0 || s.pdt > 2) return FDA_ERR_BAD_DTYPE;
    if (!(s.pdt == s.vdt || (s.pdt == FDA_DTYPE_F32))) return FDA_ERR_BAD_DTYPE;
    if (s.B <= 0 || s.N <= 0 || s.G <= 0 || s.D <= 0 || s.Q <= 0) return FDA_ERR_BAD_SHAPE;
    if (s.L < 1 || s.L > fda::kMaxLevels) return FDA_ERR_BAD_LEVELS;
    if (s.K != 4 && s.K != 8) return FDA_ERR_BAD_POINTS;
    const int cpl = 16 / dtype_size(s.vdt);
    if (s.D % cpl != 0 || s.D / cpl > 32) return FDA_ERR_BAD_HEAD_DIM;
    // 32-bit element offsets inside one batch element; 32-bit row index; grid.y limit
    if ((int64_t)s.N * s.G * s.D >= (int64_t)1 << 31) return FDA_ERR_BAD_SHAPE;
    if ((int64_t)s.Q * s.G >= (int64_t)1 << 31) return FDA_ERR_BAD_SHAPE;
    if (s.B > 65535) return FDA_ERR_BAD_SHAPE;
    const int step = s.B < im2col_step ? s.B : im2col_step;
    if (step <= 0 || s.B % step != 0) return FDA_ERR_IM2COL_STEP;
    return FDA_OK;
}

fda::Config read_config() {
    fda::Config c;
    c.l2_keep_fraction = 0.7;
    c.binning = 1;
    c.bin_slab_mb = 4.0;   // image bytes per brick (value rows add half of that); 16 / 8 / 4 / 2 MB: 43.4 / 42.5 / 42.4 / 42.2 ms per backward
    c.bin_grid_x = 0;      // blocks striding over one slab's list; 0: sized from the entry count (launch_binned_slabs)
    c.pair_rows = 1;
    c.forced_variant = 0;
    c.peer_reduce_blocks = 32;
    c.fwd_head_groups = 1;
    c.sorted = 1;
    c.sort_seg = 32;
    c.sort_grid_x = 0;
    c.touched = 1;
    c.sort_ahead = 2;  // 2 / 3 / 4 with 3 / 2 / 2 resident blocks: 31.2 / 33.8 / 33.5 ms per full-size backward
    if (const char *e = std::getenv("FDA_L2_KEEP_FRACTION")) c.l2_keep_fraction = std::atof(e);
    if (c.l2_keep_fraction < 0) c.l2_keep_fraction = 0;
    if (const char *e = std::getenv("FDA_BINNING")) c.binning = std::atoi(e) != 0;
    if (const char *e = std::getenv("FDA_BIN_SLAB_MB")) c.bin_slab_mb = std::atof(e);
    if (const char *e = std::getenv("FDA_BIN_GRID_X")) c.bin_grid_x = std::atoi(e);
    if (c.bin_grid_x < 0) c.bin_grid_x = 0;
    if (const char *e = std::getenv("FDA_PAIR_ROWS")) c.pair_rows = std::atoi(e) != 0;
    if (const char *e = std::getenv("FDA_FORCE_VARIANT")) {
        if (!std::strcmp(e, "reg")) c.forced_variant = 1;
        if (!std::strcmp(e, "smem")) c.forced_variant = 2;
    }
    if (const char *e = std::getenv("FDA_PEER_REDUCE_BLOCKS")) c.peer_reduce_blocks = std::atoi(e);
    if (c.peer_reduce_blocks < 1) c.peer_reduce_blocks = 1;
    if (const char *e = std::getenv("FDA_FWD_HEAD_GROUPS")) c.fwd_head_groups = std::atoi(e);
    if (const char *e = std::getenv("FDA_BWD_SORT")) c.sorted = std::atoi(e);
    if (const char *e = std::getenv("FDA_SORT_SEGMENT")) c.sort_seg = std::atoi(e);
    c.sort_seg = (c.sort_seg + 3) & ~3;
    if (c.sort_seg < 4) c.sort_seg = 4;
    if (c.sort_seg > 256) c.sort_seg = 256;
    if (const char *e = std::getenv("FDA_SORT_GRID_X")) c.sort_grid_x = std::atoi(e);
    if (c.sort_grid_x < 0) c.sort_grid_x = 0;
    if (const char *e = std::getenv("FDA_SORT_AHEAD")) c.sort_ahead = std::atoi(e);
    if (c.sort_ahead < 2) c.sort_ahead = 2;
    if (c.sort_ahead > 4) c.sort_ahead = 4;
    if (const char *e = std::getenv("FDA_BWD_TOUCHED")) c.touched = std::atoi(e);
    return c;
}

fda::Config g_config = read_config();

// L2 size of the current device, looked up once per device.
constexpr int kMaxDevices = 64;
std::atomic<int> g_l2_bytes[kMaxDevices];

// Bytes of re-used data the kernels may mark "evict last": a fraction of the device's L2.
unsigned long long l2_keep_budget() {
    const double frac = g_config.l2_keep_fraction;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();  // no device (sizing queries on a build machine): B200's 126 MB
        return (unsigned long long)(frac * 126.0 * 1024 * 1024);
    }
    int l2 = g_l2_bytes[dev].load(std::memory_order_relaxed);
    if (l2 == 0) {
        if (cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev) != cudaSuccess || l2 <= 0) l2 = 1;
        g_l2_bytes[dev].store(l2, std::memory_order_relaxed);
    }
    return (unsigned long long)(frac * (double)l2);
}

// Multiprocessors of the current device, looked up once per device (148 when there is no device).
std::atomic<int> g_sm_count[kMaxDevices];
int sm_count() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();
        return 148;
    }
    int n = g_sm_count[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        g_sm_count[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

fda::Problem make_problem(const Shape &s) {
    fda::Problem p;
    std::memset(&p, 0, sizeof(p));
    p.B = s.B; p.N = s.N; p.G = s.G; p.D = s.D; p.L = s.L; p.K = s.K; p.Q = s.Q;
    p.LK = s.L * s.K;
    p.k_shift = s.K == 8 ? 1 : 0;
    p.lpg = s.D / (16 / dtype_size(s.vdt));
    int lg = 0;
    while ((1 << lg) < p.lpg) ++lg;
    p.gs_log2 = lg;
    p.rows_per_b = s.Q * s.G;
    p.GD = s.G * s.D;
    p.value_elem_bytes = dtype_size(s.vdt);
    p.l2_keep_bytes = l2_keep_budget();
    p.head_group = s.G;
    p.level_mask = (1 << s.L) - 1;
    p.finalize = 1;
    p.slab_part = 0;
    p.slab_parts = 1;
    return p;
}

// Row stride (floats) of a staged tile holding `floats_per_row` payload floats: a multiple of 4
// (16-byte vector access) whose quarter is odd, so that the rows of a warp start in different banks.
inline int padded_stride(int floats_per_row) {
    int s = (floats_per_row + 3) & ~3;
    if (((s >> 2) & 1) == 0) s += 4;
    return s;
}

// Opt in to > 48 KB of dynamic shared memory, once per (device, kernel).
int ensure_smem(const void *kernel, size_t bytes) {
    static std::mutex mu;
    static std::set<std::pair<int, const void *>> done;
    if (bytes + 1024 <= 48 * 1024) return FDA_OK;  // the kernels also have a little static shared memory
    if (bytes > 200 * 1024) return FDA_ERR_TOO_LARGE_STATIC;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e);
    std::lock_guard<std::mutex> lock(mu);
    if (done.count({dev, kernel})) return FDA_OK;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return cuda_fail(e);
    done.insert({dev, kernel});
    return FDA_OK;
}

// Threads per block: 256 unless the staged tile of 256 threads' rows would leave room for fewer
// than two blocks per SM; then halve (down to one warp).  Rows never straddle blocks.
inline int pick_threads(const fda::Problem &p, int row_stride) {
    int threads = fda::kThreads;
    while (threads > 32 && (size_t)(threads >> p.gs_log2) * row_stride * sizeof(float) > 96 * 1024) threads >>= 1;
    return threads;
}

inline dim3 row_grid(const fda::Problem &p, int threads) {
    const int rows_per_block = threads >> p.gs_log2;
    return dim3((unsigned)((p.rows_per_b + rows_per_block - 1) / rows_per_block), (unsigned)p.B, 1);
}

// Heads per group of the forward's row order: when one batch element's value volume exceeds the L2 budget and the call
// is large, the largest power-of-two divisor of G whose share of the volume fits; G (plain row order) otherwise.
int forward_head_group(const fda::Problem &p) {
    if (g_config.fwd_head_groups == 0) return p.G;
    const unsigned long long volume = (unsigned long long)p.N * p.GD * p.value_elem_bytes;
    if (g_config.fwd_head_groups == 1 && (volume <= p.l2_keep_bytes || (unsigned long long)p.rows_per_b * p.LK < (4ull << 20))) return p.G;
    int hg = p.G;
    while (hg > 1 && hg % 2 == 0 && volume / p.G * hg > p.l2_keep_bytes) hg /= 2;
    return hg;
}

// grid of a forward launch: blocks per head group x groups, batch elements
inline dim3 forward_grid(const fda::Problem &p, int threads) {
    const int rows_per_block = threads >> p.gs_log2;
    const int rows_per_group = p.Q * p.head_group;
    return dim3((unsigned)(((rows_per_group + rows_per_block - 1) / rows_per_block) * (p.G / p.head_group)), (unsigned)p.B, 1);
}

template <typename VT, typename PT>
int launch_forward(fda::Problem p, bool stage, cudaStream_t st) {
    p.head_group = forward_head_group(p);
    if (stage) {
        p.row_stride = padded_stride(4 * p.LK);
        const int threads = pick_threads(p, p.row_stride);
        const size_t smem = (size_t)(threads >> p.gs_log2) * p.row_stride * sizeof(float);
        auto kern = fda::fda_forward_kernel<VT, PT, true>;
        if (int rc = ensure_smem(reinterpret_cast<const void *>(kern), smem)) return rc;
        kern<<<forward_grid(p, threads), threads, smem, st>>>(p);
    } else {
        fda::fda_forward_kernel<VT, PT, false><<<forward_grid(p, fda::kThreads), fda::kThreads, 0, st>>>(p);
    }
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FDA_OK : cuda_fail(e);
}

inline size_t round256(size_t n) { return (n + 255) & ~(size_t)255; }

// Scratch layout: [slab counters [3][B][kMaxSlabs]] [entries [B][rows_per_b*K], 8 bytes each] [dalpha plane].
// The binning part is zero-sized when binning cannot apply to this problem (image of one batch element fits
// the L2 budget, or the entry index would not fit 32 bits, or FDA_BINNING=0).
size_t bin_scratch_bytes(int B, int N, int G, int D, int Q, int K) {
    if (!g_config.binning) return 0;
    if (B <= 0 || N <= 0 || G <= 0 || D <= 0 || Q <= 0 || K <= 0 || K > 8) return 0;
    if ((unsigned long long)N * G * D * 4ull <= l2_keep_budget()) return 0;
    const unsigned long long cap = (unsigned long long)Q * G * K;
    if (cap >= (1ull << 32)) return 0;
    return round256(round256((size_t)3 * B * fda::kMaxSlabs * sizeof(unsigned int)) + (size_t)B * cap * sizeof(uint2));
}

// fp32 plane [B][Q*G][L*K] that carries raw dalpha between launches; only 16-bit offsets need it (with fp32
// offsets the logit slots of grad_sampling_loc_attn hold the same bits).
size_t dalpha_plane_bytes(int B, int G, int L, int Q, int K, int pdt) {
    if (pdt == FDA_DTYPE_F32 || B <= 0 || G <= 0 || L <= 0 || Q <= 0 || K <= 0) return 0;
    return round256((size_t)B * Q * G * L * K * sizeof(float));
}

// Cell-sorted backward: [counters [B*N*G]] [scan tile sums] [entries, 32 bytes per point] [results, 16 bytes per
// point].  Zero when the path is switched off or the problem does not qualify: 16-bit
// values with 32 channels per head only (rows of four lanes, which is what the walk's matrix instructions assume);
// point ids and list positions are 32-bit; FDA_BWD_SORT=1 wants at least a few million points, below that the extra
// launches cost more than they save.
struct SortLayout {
    size_t counters, tile_sums, entries, results, total;
    unsigned long long bins, points;
    unsigned int tiles;
};
SortLayout sort_layout(int B, int N, int G, int D, int L, int Q, int K, int vdt) {
    SortLayout s;
    std::memset(&s, 0, sizeof(s));
    if (g_config.sorted <= 0) return s;
    if (vdt == FDA_DTYPE_F32 || D != 32) return s;
    if (B <= 0 || N <= 0 || G <= 0 || L <= 0 || Q <= 0 || K <= 0 || G >= 65536) return s;
    const unsigned long long bins = (unsigned long long)B * N * G;
    const unsigned long long points = (unsigned long long)B * Q * G * L * K;
    if (bins >= (1ull << 31) || points >= (1ull << 31)) return s;
    // by size: a few million points at least (below that the five extra launches cost more than they save), and ten
    // points per (cell, head) on average -- the walk gathers and reduces once per RUN of equal cells, so it needs runs.
    // Measured per point of one rank's rows, full-size volume: sorted 0.143 / 0.170 ns at 24 / 12 points per cell and
    // head, the slab-binned + plain kernels 0.18 ns whatever the density; the fit a + b / density crosses at 9.5.
    if (g_config.sorted == 1 && (points < (4ull << 20) || (unsigned long long)Q * L * K < 10ull * N)) return s;
    s.bins = bins;
    s.points = points;
    s.tiles = (unsigned int)((bins + fda::kScanTile - 1) / fda::kScanTile);
    s.counters = 0;
    s.tile_sums = round256(bins * sizeof(unsigned int));
    s.entries = s.tile_sums + round256((size_t)s.tiles * sizeof(unsigned int));
    s.results = s.entries + round256(points * 2 * sizeof(float4));
    s.total = s.results + round256(points * sizeof(float4));
    return s;
}

void attach_sorted(fda::Problem &p, const Shape &s, void *scratch, size_t scratch_bytes) {
    if (!scratch || (reinterpret_cast<uintptr_t>(scratch) & 255u)) return;
    const SortLayout lay = sort_layout(s.B, s.N, s.G, s.D, s.L, s.Q, s.K, s.vdt);
    if (lay.total == 0 || scratch_bytes < lay.total) return;
    char *base = static_cast<char *>(scratch);
    p.sort_counters = reinterpret_cast<unsigned int *>(base + lay.counters);
    p.sort_tile_sums = reinterpret_cast<unsigned int *>(base + lay.tile_sums);
    p.sort_entries = reinterpret_cast<float4 *>(base + lay.entries);
    p.sort_results = reinterpret_cast<float4 *>(base + lay.results);
    p.sort_seg = g_config.sort_seg;
    p.bin_allowed = 0;  // this layout replaces the binned one
    p.dalpha = nullptr;
}

// Target size of one slab's share of the fp32 image.
unsigned long long bin_slab_bytes_setting() {
    unsigned long long b = (unsigned long long)(g_config.bin_slab_mb * 1048576.0);
    return b < 4096 ? 4096 : b;
}

// Point the problem at the caller's scratch when it is present and large enough: the slab lists, and for
// 16-bit offsets the dalpha plane behind them (binning is not used without its plane in that case).
void attach_scratch(fda::Problem &p, const Shape &s, void *scratch, size_t scratch_bytes) {
    if (!scratch || !aligned16(scratch)) return;
    const size_t bin_need = bin_scratch_bytes(s.B, s.N, s.G, s.D, s.Q, s.K);
    const size_t plane_need = dalpha_plane_bytes(s.B, s.G, s.L, s.Q, s.K, s.pdt);
    if (scratch_bytes < bin_need + plane_need) return;
    if (plane_need) p.dalpha = reinterpret_cast<float *>(static_cast<char *>(scratch) + bin_need);
    if (bin_need == 0) return;
    p.bin_allowed = 1;
    p.bin_counters = static_cast<unsigned int *>(scratch);
    p.bin_entries = reinterpret_cast<uint2 *>(static_cast<char *>(scratch) +
                                              round256((size_t)3 * s.B * fda::kMaxSlabs * sizeof(unsigned int)));
    p.bin_cap = (unsigned long long)s.Q * s.G * s.K;
    p.bin_slab_bytes = bin_slab_bytes_setting();
}

// Rows of exactly four lanes with two 16-byte reductions per lane (D = 32, 16-bit value): neighbouring
// rows scatter as a team so that every reduction request covers a whole 128-byte line of the image.
template <typename VT>
bool pair_rows(const fda::Problem &p) {
    if (!g_config.pair_rows) return false;
    return fda::Vec16<VT>::kCPL == 8 && p.gs_log2 == 2 && p.lpg == 4;
}

// Sort the largest level's points into slab lists (zero the counters, count, scan, fill).
template <typename PT>
int launch_bin_prepare(const fda::Problem &p, cudaStream_t st) {
    const size_t counter_bytes = (size_t)3 * p.B * fda::kMaxSlabs * sizeof(unsigned int);
    cudaError_t e = cudaMemsetAsync(p.bin_counters, 0, counter_bytes, st);
    if (e != cudaSuccess) return cuda_fail(e);
    const dim3 rows_grid((unsigned)((p.rows_per_b + 255) / 256), (unsigned)p.B, 1);
    fda::fda_bin_count_kernel<PT><<<rows_grid, 256, 0, st>>>(p);
    fda::fda_bin_scan_kernel<<<(unsigned)((p.B + 127) / 128), 128, 0, st>>>(p);
    fda::Problem q = p;
    q.row_stride = padded_stride(4 * p.LK);
    const int threads = pick_threads(q, q.row_stride);
    const size_t smem = (size_t)(threads >> q.gs_log2) * q.row_stride * sizeof(float);
    auto kern = fda::fda_bin_fill_kernel<PT>;
    if (int rc = ensure_smem(reinterpret_cast<const void *>(kern), smem)) return rc;
    kern<<<row_grid(q, threads), threads, smem, st>>>(q);
    e = cudaGetLastError();
    return e == cudaSuccess ? FDA_OK : cuda_fail(e);
}

// The slab-by-slab scatter of the slabs selected by p.slab_part / p.slab_parts.
template <typename VT, typename PT>
int launch_binned_slabs(const fda::Problem &p, cudaStream_t st) {
    // x: blocks striding over one slab's list; y: slab (slabs run one after the other); z: batch element
    // About 16 entries per lane group and slab measured best (full size: 592 / 1184 blocks 43.4 / 42.8 ms per
    // backward; an eighth of the rows: 592 / 296 blocks 6.45 / 6.25 ms).  The host does not know the slab count
    // (the shapes live on the device); it estimates it from the whole image, which the largest level dominates.
    int gx = g_config.bin_grid_x;
    if (gx <= 0) {
        const unsigned long long image_bytes = (unsigned long long)p.N * p.GD * 4ull;
        unsigned long long slabs = (image_bytes + p.bin_slab_bytes - 1) / p.bin_slab_bytes;
        slabs = slabs < 2 ? 2 : (slabs > (unsigned long long)fda::kMaxSlabs ? fda::kMaxSlabs : slabs);
        const unsigned long long groups_per_block = (unsigned long long)(fda::kThreads >> p.gs_log2);
        unsigned long long want = p.bin_cap / slabs / (16ull * groups_per_block);
        gx = (int)(want < 74 ? 74 : (want > 2368 ? 2368 : want));
    }
    const dim3 grid((unsigned)gx, fda::kMaxSlabs, (unsigned)p.B);
    if (pair_rows<VT>(p)) fda::fda_backward_binned_kernel<VT, PT, true><<<grid, fda::kThreads, 0, st>>>(p);
    else fda::fda_backward_binned_kernel<VT, PT, false><<<grid, fda::kThreads, 0, st>>>(p);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FDA_OK : cuda_fail(e);
}

template <typename VT, typename PT>
int launch_binned(fda::Problem p, cudaStream_t st) {
    if (int rc = launch_bin_prepare<PT>(p, st)) return rc;
    return launch_binned_slabs<VT, PT>(p, st);
}

template <typename VT, typename PT>
int launch_binned_part(fda::Problem p, cudaStream_t st) {
    if (p.slab_part == 0)
        if (int rc = launch_bin_prepare<PT>(p, st)) return rc;
    return launch_binned_slabs<VT, PT>(p, st);
}

// Cell-sorted path: the first launch of a sequence sorts the points of ALL levels; every launch walks the part of
// the list that belongs to its levels; the last one writes grad_sampling_loc_attn.
template <typename VT, typename PT>
int launch_sorted(fda::Problem p, cudaStream_t st) {
    if constexpr (std::is_same<VT, float>::value) {
        return FDA_ERR_BAD_DTYPE;  // not reached: the layout is empty for fp32 values
    } else {
        const unsigned long long bins = (unsigned long long)p.B * p.N * p.G;
        const unsigned int tiles = (unsigned int)((bins + fda::kScanTile - 1) / fda::kScanTile);
        if (!p.resume) {
            cudaError_t e = cudaMemsetAsync(p.sort_counters, 0, bins * sizeof(unsigned int), st);
            if (e != cudaSuccess) return cuda_fail(e);
            fda::Problem q = p;
            q.row_stride = padded_stride(4 * p.LK);
            const int threads = pick_threads(q, q.row_stride);
            const size_t smem = (size_t)(threads >> q.gs_log2) * q.row_stride * sizeof(float);
            auto count = fda::fda_sort_pass_kernel<PT, false>;
            auto fill = fda::fda_sort_pass_kernel<PT, true>;
            if (int rc = ensure_smem(reinterpret_cast<const void *>(count), smem)) return rc;
            if (int rc = ensure_smem(reinterpret_cast<const void *>(fill), smem)) return rc;
            count<<<row_grid(q, threads), threads, smem, st>>>(q);
            fda::fda_scan_tile_sums_kernel<<<tiles, fda::kScanThreads, 0, st>>>(p.sort_counters, (size_t)bins, p.sort_tile_sums);
            fda::fda_scan_spine_kernel<<<1, fda::kScanThreads, 0, st>>>(p.sort_tile_sums, tiles);
            fda::fda_scan_apply_kernel<<<tiles, fda::kScanThreads, 0, st>>>(p.sort_counters, (size_t)bins, p.sort_tile_sums);
            fill<<<row_grid(q, threads), threads, smem, st>>>(q);
            e = cudaGetLastError();
            if (e != cudaSuccess) return cuda_fail(e);
        }
        // shared memory of the walk: every warp's span of the list (32 bytes per entry) and every lane's ring of rows
        constexpr int block = 128;
        const int ahead = g_config.sort_ahead;
        const size_t walk_smem = ((size_t)(block / 32) * 8 * (2 * (size_t)p.sort_seg + 1) + (size_t)ahead * fda::kWalkSlot * block) * 16;
        int per_sm = (int)((size_t)227 * 1024 / (walk_smem + 1024));  // resident blocks: shared memory, then registers (3)
        per_sm = per_sm > 3 ? 3 : (per_sm < 1 ? 1 : per_sm);
        int gx = g_config.sort_grid_x;
        if (gx <= 0) gx = (per_sm * sm_count() + p.B - 1) / p.B;
        auto walk = ahead == 2 ? fda::fda_sorted_walk_kernel<VT, block, 3, 2>
                               : (ahead == 3 ? fda::fda_sorted_walk_kernel<VT, block, 3, 3> : fda::fda_sorted_walk_kernel<VT, block, 3, 4>);
        if (int rc = ensure_smem(reinterpret_cast<const void *>(walk), walk_smem)) return rc;
        walk<<<dim3((unsigned)gx, (unsigned)p.B, 1), block, walk_smem, st>>>(p);
        if (p.finalize) {
            fda::Problem q = p;
            q.row_stride = padded_stride(5 * p.LK);
            const int threads = pick_threads(q, q.row_stride);
            const size_t smem = (size_t)(threads >> q.gs_log2) * q.row_stride * sizeof(float);
            auto fin = fda::fda_sort_finalize_kernel<PT>;
            if (int rc = ensure_smem(reinterpret_cast<const void *>(fin), smem)) return rc;
            fin<<<row_grid(q, threads), threads, smem, st>>>(q);
        }
        const cudaError_t e = cudaGetLastError();
        return e == cudaSuccess ? FDA_OK : cuda_fail(e);
    }
}

// Whether fda_backward zero-fills and converts only the rows of the fp32 image that sampling points touch
// (fda_backward_touched.cuh) instead of the whole image.  Worst case (no two points share a row) the two point
// passes write and read 8 rows of D floats per point; the dense passes move the image 2.5 times.  Taken when the
// points can touch at most 60 % of the image.  The slab-binned scatter only adds to touched rows, like the plain
// one; the cell-sorted path is for 10 and more points per cell and head and keeps the dense handling.
bool touched_rows_choice(const Shape &s) {
    if (s.vdt == FDA_DTYPE_F32 || g_config.touched <= 0) return false;
    if (sort_layout(s.B, s.N, s.G, s.D, s.L, s.Q, s.K, s.vdt).total) return false;
    if (g_config.touched >= 2) return true;
    return (double)s.Q * s.L * s.K * 8.0 <= 0.6 * (double)s.N;
}

// kCast = false: zero the touched rows of p.accum; kCast = true: convert them into grad_value.
template <typename VT, typename PT, bool kCast>
int launch_touch_rows(const fda::Problem &p, void *grad_value, cudaStream_t st) {
    if constexpr (std::is_same<VT, float>::value) {
        (void)p; (void)grad_value; (void)st;
        return FDA_ERR_BAD_DTYPE;
    } else {
        const int vecs = p.D / 4;
        const unsigned long long total = (unsigned long long)p.B * p.rows_per_b * p.LK * vecs;
        const unsigned long long blocks = (total + 255) / 256;
        if (blocks > 0x7fffffffull) return FDA_ERR_BAD_SHAPE;
        fda::fda_touch_rows_kernel<VT, PT, kCast><<<(unsigned)blocks, 256, 0, st>>>(p, static_cast<VT *>(grad_value), total, vecs);
        const cudaError_t e = cudaGetLastError();
        return e == cudaSuccess ? FDA_OK : cuda_fail(e);
    }
}

template <typename VT, typename PT>
int launch_backward(fda::Problem p, cudaStream_t st) {
    if (p.sort_counters && !p.binned_elsewhere) return launch_sorted<VT, PT>(p, st);
    if (p.bin_allowed && !p.binned_elsewhere)
        if (int rc = launch_binned<VT, PT>(p, st)) return rc;
    p.row_stride = padded_stride(5 * p.LK);
    const int threads = pick_threads(p, p.row_stride);
    const size_t smem = (size_t)(threads >> p.gs_log2) * p.row_stride * sizeof(float);
    auto kern = pair_rows<VT>(p) ? fda::fda_backward_kernel<VT, PT, true> : fda::fda_backward_kernel<VT, PT, false>;
    if (int rc = ensure_smem(reinterpret_cast<const void *>(kern), smem)) return rc;
    kern<<<row_grid(p, threads), threads, smem, st>>>(p);
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? FDA_OK : cuda_fail(e);
}

#define FDA_DISPATCH(vdt, pdt, CALL)                                                         \
    [&]() -> int {                                                                           \
        if (vdt == FDA_DTYPE_F32) { using VT = float; using PT = float; return CALL; }       \
        if (vdt == FDA_DTYPE_F16 && pdt == FDA_DTYPE_F16) { using VT = __half; using PT = __half; return CALL; } \
        if (vdt == FDA_DTYPE_F16) { using VT = __half; using PT = float; return CALL; }      \
        if (pdt == FDA_DTYPE_BF16) { using VT = __nv_bfloat16; using PT = __nv_bfloat16; return CALL; } \
        { using VT = __nv_bfloat16; using PT = float; return CALL; }                         \
    }()

}  // namespace

namespace fda {
const Config &config() { return g_config; }
void record_cuda_error(int e) { g_last_cuda_error = e; }
}  // namespace fda

extern "C" {

void fda_reload_config(void) { g_config = read_config(); }

const char *fda_status_string(int status) {
    switch (status) {
        case FDA_OK: return "ok";
        case FDA_ERR_NULL_POINTER: return "null pointer argument";
        case FDA_ERR_BAD_DTYPE: return "unsupported dtype (value f32/f16/bf16; packed equal to value, or f32)";
        case FDA_ERR_BAD_LEVELS: return "num_levels must be in 1..5";
        case FDA_ERR_BAD_POINTS: return "num_points must be 4 or 8";
        case FDA_ERR_BAD_HEAD_DIM: return "head_dim must be a multiple of a 16-byte vector and at most 512 bytes";
        case FDA_ERR_BAD_SHAPE: return "non-positive or too large dimension";
        case FDA_ERR_IM2COL_STEP: return "batch must divide im2col_step";
        case FDA_ERR_WORKSPACE: return "workspace missing or too small";
        case FDA_ERR_MISALIGNED: return "tensor base address not 16-byte aligned";
        case FDA_ERR_CUDA: return "CUDA runtime error";
        case FDA_ERR_TOO_LARGE_STATIC: return "problem exceeds a compiled-in capacity";
        default: return "unknown status";
    }
}

int fda_last_cuda_error(void) { return g_last_cuda_error; }

int fda_version(void) { return 1000; }

int fda_forward(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                const void *sampling_loc_attn, void *output,
                int batch, int num_value, int num_heads, int head_dim, int num_levels,
                int num_query, int num_points, int value_dtype, int packed_dtype,
                int im2col_step, int d_stride, int block_thread, int use_reg, void *stream) {
    (void)d_stride; (void)block_thread;
    if (!value || !spatial_shapes || !level_start_index || !sampling_loc_attn || !output) return FDA_ERR_NULL_POINTER;
    const Shape s{batch, num_value, num_heads, head_dim, num_levels, num_query, num_points, value_dtype, packed_dtype};
    if (int rc = validate(s, im2col_step)) return rc;
    if (!aligned16(value) || !aligned16(sampling_loc_attn) || !aligned16(output)) return FDA_ERR_MISALIGNED;
    fda::Problem p = make_problem(s);
    p.value = value; p.shapes = spatial_shapes; p.lsi = level_start_index; p.packed = sampling_loc_attn; p.out = output;
    // Staging choice per shape: with several rows per warp the packed rows of a warp are one
    // contiguous span, which the staged kernel reads with full-width coalesced loads.
    bool stage = !use_reg || p.gs_log2 <= 3;
    const int forced = g_config.forced_variant;
    if (forced == 1 && use_reg) stage = false;
    if (forced == 2) stage = true;
    return FDA_DISPATCH(value_dtype, packed_dtype, (launch_forward<VT, PT>(p, stage, static_cast<cudaStream_t>(stream))));
}

size_t fda_backward_scratch_bytes(int batch, int num_value, int num_heads, int head_dim, int num_levels, int num_query,
                                  int num_points, int packed_dtype) {
    return bin_scratch_bytes(batch, num_value, num_heads, head_dim, num_query, num_points) +
           dalpha_plane_bytes(batch, num_heads, num_levels, num_query, num_points, packed_dtype);
}

int fda_forward_head_group(int num_value, int num_heads, int head_dim, int num_levels, int num_query, int num_points,
                           int value_dtype) {
    if (num_value <= 0 || num_heads <= 0 || head_dim <= 0 || num_levels <= 0 || num_query <= 0 || num_points <= 0) return 0;
    const Shape s{1, num_value, num_heads, head_dim, num_levels, num_query, num_points, value_dtype, FDA_DTYPE_F32};
    return forward_head_group(make_problem(s));
}

size_t fda_backward_sorted_scratch_bytes(int batch, int num_value, int num_heads, int head_dim, int num_levels, int num_query,
                                         int num_points, int value_dtype) {
    return sort_layout(batch, num_value, num_heads, head_dim, num_levels, num_query, num_points, value_dtype).total;
}

int fda_backward_path(int batch, int num_value, int num_heads, int head_dim, int num_levels, int num_query, int num_points,
                      int value_dtype) {
    if (sort_layout(batch, num_value, num_heads, head_dim, num_levels, num_query, num_points, value_dtype).total) return 2;
    return bin_scratch_bytes(batch, num_value, num_heads, head_dim, num_query, num_points) ? 1 : 0;
}

size_t fda_backward_workspace_bytes(int batch, int num_value, int num_heads, int head_dim, int num_levels, int num_query,
                                    int num_points, int value_dtype, int packed_dtype) {
    if (batch <= 0 || num_value <= 0 || num_heads <= 0 || head_dim <= 0) return 0;
    const size_t image = value_dtype == FDA_DTYPE_F32 ? 0 : round256((size_t)batch * num_value * num_heads * head_dim * sizeof(float));
    // fda_backward hands dalpha from launch to launch only when the largest level is slab-binned
    const size_t bin = bin_scratch_bytes(batch, num_value, num_heads, head_dim, num_query, num_points);
    const size_t binned = bin ? bin + dalpha_plane_bytes(batch, num_heads, num_levels, num_query, num_points, packed_dtype) : 0;
    const size_t sorted = sort_layout(batch, num_value, num_heads, head_dim, num_levels, num_query, num_points, value_dtype).total;
    return image + (binned > sorted ? binned : sorted);
}

int fda_backward_accumulate_levels(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                                   const void *sampling_loc_attn, const void *grad_output,
                                   float *accum, void *grad_sampling_loc_attn,
                                   int batch, int num_value, int num_heads, int head_dim, int num_levels,
                                   int num_query, int num_points, int value_dtype, int packed_dtype,
                                   int im2col_step, int level_begin, int level_end, int flags,
                                   void *scratch, size_t scratch_bytes, void *stream) {
    if (!value || !spatial_shapes || !level_start_index || !sampling_loc_attn || !grad_output || !accum || !grad_sampling_loc_attn)
        return FDA_ERR_NULL_POINTER;
    const Shape s{batch, num_value, num_heads, head_dim, num_levels, num_query, num_points, value_dtype, packed_dtype};
    if (int rc = validate(s, im2col_step)) return rc;
    if (level_begin < 0 || level_end > num_levels || level_begin >= level_end) return FDA_ERR_BAD_LEVELS;
    if (!aligned16(value) || !aligned16(sampling_loc_attn) || !aligned16(grad_output) || !aligned16(accum) ||
        !aligned16(grad_sampling_loc_attn))
        return FDA_ERR_MISALIGNED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // an fp32 value accumulates in grad_value itself, which must be zero everywhere the points do not reach
    const bool zero_touched = (flags & FDA_BWD_ZERO_TOUCHED) && value_dtype != FDA_DTYPE_F32;
    if ((flags & FDA_BWD_ZERO_IMAGE) || ((flags & FDA_BWD_ZERO_TOUCHED) && !zero_touched)) {
        const size_t n = (size_t)batch * num_value * num_heads * head_dim;
        cudaError_t e = cudaMemsetAsync(accum, 0, n * sizeof(float), st);
        if (e != cudaSuccess) return cuda_fail(e);
    }
    fda::Problem p = make_problem(s);
    p.value = value; p.shapes = spatial_shapes; p.lsi = level_start_index; p.packed = sampling_loc_attn;
    p.grad_out = grad_output; p.accum = accum; p.grad_packed = grad_sampling_loc_attn;
    if (zero_touched && !(flags & FDA_BWD_ZERO_IMAGE))
        if (int rc = FDA_DISPATCH(value_dtype, packed_dtype, (launch_touch_rows<VT, PT, false>(p, nullptr, st)))) return rc;
    p.level_mask = ((1 << level_end) - 1) & ~((1 << level_begin) - 1);
    p.resume = (flags & FDA_BWD_RESUME) ? 1 : 0;
    p.finalize = (flags & FDA_BWD_FINALIZE) ? 1 : 0;
    // slab-binned handling of the largest level, when the caller gave scratch for it
    attach_scratch(p, s, scratch, scratch_bytes);
    attach_sorted(p, s, scratch, scratch_bytes);
    p.binned_elsewhere = (flags & FDA_BWD_BINNED_DONE) ? 1 : 0;
    if (p.binned_elsewhere && !p.bin_allowed) return FDA_ERR_WORKSPACE;
    return FDA_DISPATCH(value_dtype, packed_dtype, (launch_backward<VT, PT>(p, st)));
}

int fda_backward_bin_plan(const int64_t *spatial_shapes_host, int num_levels, int batch, int num_value, int num_heads,
                          int head_dim, int num_query, int num_points, int *level, int *slabs, int *depth) {
    if (!spatial_shapes_host || num_levels < 1 || num_levels > fda::kMaxLevels) return 0;
    if (bin_scratch_bytes(batch, num_value, num_heads, head_dim, num_query, num_points) == 0) return 0;
    const fda::BinPlan plan = fda::bin_plan_from(spatial_shapes_host, num_levels, num_heads * head_dim, l2_keep_budget(),
                                                 bin_slab_bytes_setting(), (1 << num_levels) - 1, 1);
    if (level) *level = plan.level;
    if (slabs) *slabs = plan.slabs;
    if (depth) *depth = plan.depth;
    return plan.enabled;
}

int fda_backward_binned_part(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                             const void *sampling_loc_attn, const void *grad_output,
                             float *accum, void *grad_sampling_loc_attn,
                             int batch, int num_value, int num_heads, int head_dim, int num_levels,
                             int num_query, int num_points, int value_dtype, int packed_dtype,
                             int im2col_step, int part, int parts, int flags,
                             void *scratch, size_t scratch_bytes, void *stream) {
    if (!value || !spatial_shapes || !level_start_index || !sampling_loc_attn || !grad_output || !accum || !grad_sampling_loc_attn)
        return FDA_ERR_NULL_POINTER;
    const Shape s{batch, num_value, num_heads, head_dim, num_levels, num_query, num_points, value_dtype, packed_dtype};
    if (int rc = validate(s, im2col_step)) return rc;
    if (parts < 1 || part < 0 || part >= parts) return FDA_ERR_BAD_SHAPE;
    if (!aligned16(value) || !aligned16(sampling_loc_attn) || !aligned16(grad_output) || !aligned16(accum) ||
        !aligned16(grad_sampling_loc_attn))
        return FDA_ERR_MISALIGNED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    fda::Problem p = make_problem(s);
    p.value = value; p.shapes = spatial_shapes; p.lsi = level_start_index; p.packed = sampling_loc_attn;
    p.grad_out = grad_output; p.accum = accum; p.grad_packed = grad_sampling_loc_attn;
    attach_scratch(p, s, scratch, scratch_bytes);
    if (!p.bin_allowed) return FDA_ERR_WORKSPACE;
    p.slab_part = part;
    p.slab_parts = parts;
    if ((flags & FDA_BWD_ZERO_IMAGE) && part == 0) {
        const size_t n = (size_t)batch * num_value * num_heads * head_dim;
        cudaError_t e = cudaMemsetAsync(accum, 0, n * sizeof(float), st);
        if (e != cudaSuccess) return cuda_fail(e);
    }
    return FDA_DISPATCH(value_dtype, packed_dtype, (launch_binned_part<VT, PT>(p, st)));
}

int fda_backward_accumulate(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                            const void *sampling_loc_attn, const void *grad_output,
                            float *accum, void *grad_sampling_loc_attn,
                            int batch, int num_value, int num_heads, int head_dim, int num_levels,
                            int num_query, int num_points, int value_dtype, int packed_dtype,
                            int im2col_step, void *stream) {
    return fda_backward_accumulate_levels(value, spatial_shapes, level_start_index, sampling_loc_attn, grad_output, accum,
                                          grad_sampling_loc_attn, batch, num_value, num_heads, head_dim, num_levels,
                                          num_query, num_points, value_dtype, packed_dtype, im2col_step, 0,
                                          num_levels > 0 ? num_levels : 1, FDA_BWD_ZERO_IMAGE | FDA_BWD_FINALIZE,
                                          nullptr, 0, stream);
}

int fda_cast_grad_value(const float *accum, void *grad_value, size_t num_elements, int value_dtype, void *stream) {
    if (!accum || !grad_value) return FDA_ERR_NULL_POINTER;
    if (value_dtype < 0 || value_dtype > 2) return FDA_ERR_BAD_DTYPE;
    if (num_elements % 4 != 0) return FDA_ERR_BAD_SHAPE;
    if (!aligned16(accum) || !aligned16(grad_value)) return FDA_ERR_MISALIGNED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaSuccess;
    if (value_dtype == FDA_DTYPE_F32) {
        if (static_cast<const void *>(accum) != grad_value)
            e = cudaMemcpyAsync(grad_value, accum, num_elements * sizeof(float), cudaMemcpyDeviceToDevice, st);
        return e == cudaSuccess ? FDA_OK : cuda_fail(e);
    }
    const size_t n4 = num_elements / 4;
    if (n4 == 0) return FDA_OK;
    size_t blocks = (n4 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;  // grid-stride; 16 resident blocks of 256 threads cover an SM
    if (value_dtype == FDA_DTYPE_F16)
        fda::fda_cast_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(accum, static_cast<__half *>(grad_value), n4);
    else
        fda::fda_cast_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(accum, static_cast<__nv_bfloat16 *>(grad_value), n4);
    e = cudaGetLastError();
    return e == cudaSuccess ? FDA_OK : cuda_fail(e);
}

int fda_backward_touched_rows(int batch, int num_value, int num_heads, int head_dim, int num_levels, int num_query,
                              int num_points, int value_dtype) {
    if (batch <= 0 || num_value <= 0 || num_heads <= 0 || head_dim <= 0 || num_levels <= 0 || num_query <= 0 || num_points <= 0)
        return 0;
    const Shape s{batch, num_value, num_heads, head_dim, num_levels, num_query, num_points, value_dtype, FDA_DTYPE_F32};
    return touched_rows_choice(s) ? 1 : 0;
}

int fda_cast_grad_value_touched(const float *accum, void *grad_value, const int64_t *spatial_shapes,
                                const int64_t *level_start_index, const void *sampling_loc_attn,
                                int batch, int num_value, int num_heads, int head_dim, int num_levels,
                                int num_query, int num_points, int value_dtype, int packed_dtype, void *stream) {
    if (!accum || !grad_value || !spatial_shapes || !level_start_index || !sampling_loc_attn) return FDA_ERR_NULL_POINTER;
    const Shape s{batch, num_value, num_heads, head_dim, num_levels, num_query, num_points, value_dtype, packed_dtype};
    if (int rc = validate(s, batch)) return rc;
    if (value_dtype == FDA_DTYPE_F32) return FDA_ERR_BAD_DTYPE;  // an fp32 value has no separate image
    if (!aligned16(accum) || !aligned16(grad_value) || !aligned16(sampling_loc_attn)) return FDA_ERR_MISALIGNED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t n = (size_t)batch * num_value * num_heads * head_dim;
    const cudaError_t e = cudaMemsetAsync(grad_value, 0, n * dtype_size(value_dtype), st);
    if (e != cudaSuccess) return cuda_fail(e);
    fda::Problem p = make_problem(s);
    p.shapes = spatial_shapes; p.lsi = level_start_index; p.packed = sampling_loc_attn;
    p.accum = const_cast<float *>(accum);
    return FDA_DISPATCH(value_dtype, packed_dtype, (launch_touch_rows<VT, PT, true>(p, grad_value, st)));
}

int fda_backward(const void *value, const int64_t *spatial_shapes, const int64_t *level_start_index,
                 const void *sampling_loc_attn, const void *grad_output,
                 void *grad_value, void *grad_sampling_loc_attn,
                 void *workspace, size_t workspace_bytes,
                 int batch, int num_value, int num_heads, int head_dim, int num_levels,
                 int num_query, int num_points, int value_dtype, int packed_dtype,
                 int im2col_step, int d_stride, int block_thread, void *stream) {
    (void)d_stride; (void)block_thread;
    if (!grad_value) return FDA_ERR_NULL_POINTER;
    const size_t need = fda_backward_workspace_bytes(batch, num_value, num_heads, head_dim, num_levels, num_query, num_points,
                                                     value_dtype, packed_dtype);
    const size_t n = (size_t)batch * num_value * num_heads * head_dim;
    const size_t image_bytes = value_dtype == FDA_DTYPE_F32 ? 0 : round256(n * sizeof(float));
    float *accum = static_cast<float *>(grad_value);
    if (need > 0 && (!workspace || workspace_bytes < need)) return FDA_ERR_WORKSPACE;
    if (image_bytes > 0) accum = static_cast<float *>(workspace);
    void *scratch = need > image_bytes ? static_cast<char *>(workspace) + image_bytes : nullptr;
    if (!aligned16(grad_value)) return FDA_ERR_MISALIGNED;
    const bool touched = image_bytes > 0 && fda_backward_touched_rows(batch, num_value, num_heads, head_dim, num_levels,
                                                                      num_query, num_points, value_dtype);
    int rc = fda_backward_accumulate_levels(value, spatial_shapes, level_start_index, sampling_loc_attn, grad_output, accum,
                                            grad_sampling_loc_attn, batch, num_value, num_heads, head_dim, num_levels,
                                            num_query, num_points, value_dtype, packed_dtype, im2col_step, 0,
                                            num_levels > 0 ? num_levels : 1,
                                            (touched ? FDA_BWD_ZERO_TOUCHED : FDA_BWD_ZERO_IMAGE) | FDA_BWD_FINALIZE,
                                            scratch, need - image_bytes, stream);
    if (rc != FDA_OK || image_bytes == 0) return rc;
    if (touched)
        return fda_cast_grad_value_touched(accum, grad_value, spatial_shapes, level_start_index, sampling_loc_attn, batch,
                                           num_value, num_heads, head_dim, num_levels, num_query, num_points, value_dtype,
                                           packed_dtype, stream);
    return fda_cast_grad_value(accum, grad_value, n, value_dtype, stream);
}

}  // extern "C"
