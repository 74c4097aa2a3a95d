// RoDe row-decomposition preprocessing on the GPU, plus its host twin.
//
// Specification: the single-thread loop RoDe_preprocess_cpu of the reference
// (Preprocess_opt/_preprocess.cu:340-373).  For row i with pad = row_ptr[i] % vec_len and
// aligned length A = len + pad:
//     A >  seg_len : segments (i, row_ptr[i]), (i, row_ptr[i] - pad + j*seg_len), j = 1, 2, ...
//     last piece   : one more segment if it is >= k_block long; residue row if it is not a
//                    multiple of k_block.
// The reference's device version (count kernel _preprocess.cu:244-274, two CUB scans
// :330-334, fill kernel :275-322) keeps its prefix sums in the output arrays and overwrites
// them in place across thread blocks.  Here the prefix sums live in a separate scratch
// array, so the three kernels below are race-free:
//
//   count_tiles   one CTA per tile of kTile rows: per-row (bn, rn), tile totals -> scratch
//   scan_tiles    one CTA: exclusive scan of the tile totals, n_blk, n_res, end sentinel
//   fill_tiles    one CTA per tile: in-tile exclusive scan + tile offset, then the writes;
//                 rows with many segments are written by a whole warp
//
// HBM traffic: row_ptr is read twice (8 B/row), outputs written once (8 B/segment,
// 4 B/residue row), scratch is 8 B per 1024 rows.
#include <climits>
#include <mutex>

#include "rode_common.cuh"

namespace rode {
namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerThread = 4;
constexpr int kTile = kThreads * kRowsPerThread;  // rows per CTA
constexpr int kWarps = kThreads / 32;
constexpr int kLongRow = 8;  // rows with more segments than this are written by a warp

// The three parameters of the decomposition.  kPow2 = all of them are powers of two (every
// parameter set the reference uses: (512, 32, 4) and (32, 32, 4)): quotients and remainders
// are then shifts and masks.  With run-time divisors the five integer divisions per row made
// the count and fill kernels instruction-bound (about 150 instructions per row).
struct Params {
    int seg_len, k_block, vec_len;
    int seg_shift;  // log2(seg_len) when kPow2
};
template <bool kPow2>
__device__ __forceinline__ int mod_vec(int x, const Params &p) {
    return kPow2 ? (x & (p.vec_len - 1)) : (x % p.vec_len);
}
template <bool kPow2>
__device__ __forceinline__ int mod_block(int x, const Params &p) {
    return kPow2 ? (x & (p.k_block - 1)) : (x % p.k_block);
}

// Number of block segments and residue flag of one row (closed form of the spec loop;
// valid because seg_len % k_block == 0).
template <bool kPow2>
__device__ __forceinline__ void row_counts(int off, int next, const Params &p, int &bn, int &rn) {
    const int a = next - off + mod_vec<kPow2>(off, p);
    if (a > p.seg_len) {
        const int rest = kPow2 ? (a & (p.seg_len - 1)) : (a % p.seg_len);
        const int full = kPow2 ? (a >> p.seg_shift) : (a / p.seg_len);
        bn = full + (rest >= p.k_block ? 1 : 0);
        rn = mod_block<kPow2>(rest, p) != 0 ? 1 : 0;
    } else {
        bn = a >= p.k_block ? 1 : 0;
        rn = mod_block<kPow2>(a, p) != 0 ? 1 : 0;
    }
}

// Inclusive scan of (x, y) over a CTA of kW warps; returns the exclusive prefix of this
// thread and the CTA totals.  smem: 2 * kW ints.
template <int kW = kWarps>
__device__ __forceinline__ void block_exclusive_scan2(int x, int y, int *smem, int &ex, int &ey, int &tx,
                                                      int &ty) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int ix = x, iy = y;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int ux = __shfl_up_sync(0xffffffffu, ix, d);
        const int uy = __shfl_up_sync(0xffffffffu, iy, d);
        if (lane >= d) {
            ix += ux;
            iy += uy;
        }
    }
    if (lane == 31) {
        smem[warp] = ix;
        smem[kW + warp] = iy;
    }
    __syncthreads();
    int wx = 0, wy = 0;
    tx = 0;
    ty = 0;
#pragma unroll
    for (int w = 0; w < kW; ++w) {
        const int sx = smem[w], sy = smem[kW + w];
        if (w < warp) {
            wx += sx;
            wy += sy;
        }
        tx += sx;
        ty += sy;
    }
    ex = wx + ix - x;
    ey = wy + iy - y;
    __syncthreads();
}

template <bool kPow2>
__global__ void __launch_bounds__(kThreads)
count_tiles(Params p, int M, const int *__restrict__ row_ptr, int2 *__restrict__ tile_totals) {
    __shared__ int smem[2 * kWarps];
    const int row0 = blockIdx.x * kTile + threadIdx.x * kRowsPerThread;
    int bsum = 0, rsum = 0;
    if (row0 < M) {
        int off = row_ptr[row0];
#pragma unroll
        for (int i = 0; i < kRowsPerThread; ++i) {
            if (row0 + i < M) {
                const int next = row_ptr[row0 + i + 1];
                int bn, rn;
                row_counts<kPow2>(off, next, p, bn, rn);
                bsum += bn;
                rsum += rn;
                off = next;
            }
        }
    }
    int ex, ey, tx, ty;
    block_exclusive_scan2(bsum, rsum, smem, ex, ey, tx, ty);
    if (threadIdx.x == 0) tile_totals[blockIdx.x] = make_int2(tx, ty);
}

// Single CTA of kScanThreads, kScanPerThread consecutive tiles per thread (8192 tiles, i.e.
// 8.4 M rows, per pass).  Turns tile totals into exclusive tile offsets (in place) and
// publishes n_blk, n_res and, if asked to, the end sentinel st_off[n_blk] = row_ptr[M].
constexpr int kScanThreads = 1024;
constexpr int kScanPerThread = 8;
__global__ void __launch_bounds__(kScanThreads)
scan_tiles(int n_tiles, int M, const int *__restrict__ row_ptr, int2 *__restrict__ tile_totals,
           int *__restrict__ st_off, int *__restrict__ n_blk, int *__restrict__ n_res, bool write_sentinel) {
    __shared__ int smem[2 * (kScanThreads / 32)];
    int carry_b = 0, carry_r = 0;
    for (int base = 0; base < n_tiles; base += kScanThreads * kScanPerThread) {
        const int t0 = base + threadIdx.x * kScanPerThread;
        int2 v[kScanPerThread];
        int sum_b = 0, sum_r = 0;
#pragma unroll
        for (int i = 0; i < kScanPerThread; ++i) {
            v[i] = make_int2(0, 0);
            if (t0 + i < n_tiles) v[i] = tile_totals[t0 + i];
            sum_b += v[i].x;
            sum_r += v[i].y;
        }
        int ex, ey, tx, ty;
        block_exclusive_scan2<kScanThreads / 32>(sum_b, sum_r, smem, ex, ey, tx, ty);
        int run_b = carry_b + ex, run_r = carry_r + ey;
#pragma unroll
        for (int i = 0; i < kScanPerThread; ++i) {
            if (t0 + i < n_tiles) tile_totals[t0 + i] = make_int2(run_b, run_r);
            run_b += v[i].x;
            run_r += v[i].y;
        }
        carry_b += tx;
        carry_r += ty;
    }
    if (threadIdx.x == 0) {
        n_blk[0] = carry_b;
        n_res[0] = carry_r;
        if (write_sentinel) st_off[carry_b] = row_ptr[M];
    }
}

template <bool kPow2>
__global__ void __launch_bounds__(kThreads)
fill_tiles(Params p, int M, const int *__restrict__ row_ptr, const int2 *__restrict__ tile_offsets,
           int *__restrict__ block_r_ind, int *__restrict__ st_off, int *__restrict__ residue_r_ind) {
    __shared__ int smem[2 * kWarps];
    // Long rows of this tile, written cooperatively after the per-thread pass.
    __shared__ int long_row[kTile];
    __shared__ int long_dst[kTile];
    __shared__ int long_cnt[kTile];
    __shared__ int n_long;
    if (threadIdx.x == 0) n_long = 0;

    const int row0 = blockIdx.x * kTile + threadIdx.x * kRowsPerThread;
    int offs[kRowsPerThread + 1];
    int bn[kRowsPerThread], rn[kRowsPerThread];
    int bsum = 0, rsum = 0;
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
        bn[i] = 0;
        rn[i] = 0;
    }
    if (row0 < M) {
        offs[0] = row_ptr[row0];
#pragma unroll
        for (int i = 0; i < kRowsPerThread; ++i) {
            if (row0 + i < M) {
                offs[i + 1] = row_ptr[row0 + i + 1];
                row_counts<kPow2>(offs[i], offs[i + 1], p, bn[i], rn[i]);
                bsum += bn[i];
                rsum += rn[i];
            } else {
                offs[i + 1] = offs[i];
            }
        }
    }
    int ex, ey, tx, ty;
    block_exclusive_scan2(bsum, rsum, smem, ex, ey, tx, ty);  // also orders n_long = 0
    const int2 tile_off = tile_offsets[blockIdx.x];
    int gb = tile_off.x + ex, gr = tile_off.y + ey;

#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
        const int row = row0 + i;
        if (bn[i] > kLongRow) {
            const int slot = atomicAdd(&n_long, 1);  // shared-memory slot counter, order irrelevant
            long_row[slot] = row;
            long_dst[slot] = gb;
            long_cnt[slot] = bn[i];
        } else if (bn[i] > 0) {
            const int off = offs[i];
            const int aligned = off - mod_vec<kPow2>(off, p);
            block_r_ind[gb] = row;
            st_off[gb] = off;
            for (int j = 1; j < bn[i]; ++j) {
                block_r_ind[gb + j] = row;
                st_off[gb + j] = aligned + j * p.seg_len;
            }
        }
        if (rn[i]) residue_r_ind[gr] = row;
        gb += bn[i];
        gr += rn[i];
    }
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int total_long = n_long;
    for (int s = warp; s < total_long; s += kWarps) {
        const int row = long_row[s], dst = long_dst[s], cnt = long_cnt[s];
        const int off = row_ptr[row];
        const int aligned = off - mod_vec<kPow2>(off, p);
        for (int j = lane; j < cnt; j += 32) {
            block_r_ind[dst + j] = row;
            st_off[dst + j] = j == 0 ? off : aligned + j * p.seg_len;
        }
    }
}

int check_params(int seg_len, int k_block, int vec_len, int M, const void *row_ptr) {
    if (seg_len <= 0 || k_block <= 0 || vec_len <= 0)
        return fail(RODE_ERR_INVALID_ARGUMENT, "preprocess: seg_len, k_block, vec_len must be positive");
    if (seg_len % k_block != 0 || k_block % vec_len != 0)
        return fail(RODE_ERR_INVALID_ARGUMENT,
                    "preprocess: need seg_len %% k_block == 0 and k_block %% vec_len == 0 (got %d, %d, %d)",
                    seg_len, k_block, vec_len);
    if (M < 0 || M > INT_MAX - kTile)
        return fail(RODE_ERR_INVALID_ARGUMENT, "preprocess: M = %d outside [0, %d]", M, INT_MAX - kTile);
    if (row_ptr == nullptr) return fail(RODE_ERR_INVALID_ARGUMENT, "preprocess: row_ptr is null");
    return RODE_OK;
}

}  // namespace

// Launches the three kernels; `tile_scratch` holds one int2 per tile.  write_sentinel: also
// store st_off[n_blk] = row_ptr[M] (the C ABI's contract; the reference's device version does
// not, and its callers size st_off without room for it).
int launch_preprocess(int seg_len, int k_block, int vec_len, int M, const int *row_ptr, int *block_r_ind,
                      int *st_off, int *residue_r_ind, int *n_blk, int *n_res, int2 *tile_scratch,
                      cudaStream_t stream, bool write_sentinel = true) {
    const int n_tiles = (M + kTile - 1) / kTile;
    auto pow2 = [](int x) { return (x & (x - 1)) == 0; };
    const bool all_pow2 = pow2(seg_len) && pow2(k_block) && pow2(vec_len);
    Params p = {seg_len, k_block, vec_len, 0};
    while (all_pow2 && (1 << p.seg_shift) < seg_len) ++p.seg_shift;
    if (n_tiles > 0) {
        if (all_pow2)
            count_tiles<true><<<n_tiles, kThreads, 0, stream>>>(p, M, row_ptr, tile_scratch);
        else
            count_tiles<false><<<n_tiles, kThreads, 0, stream>>>(p, M, row_ptr, tile_scratch);
        RODE_CHECK_LAUNCH("rode::count_tiles");
    }
    scan_tiles<<<1, kScanThreads, 0, stream>>>(n_tiles, M, row_ptr, tile_scratch, st_off, n_blk, n_res,
                                               write_sentinel);
    RODE_CHECK_LAUNCH("rode::scan_tiles");
    if (n_tiles > 0) {
        if (all_pow2)
            fill_tiles<true><<<n_tiles, kThreads, 0, stream>>>(p, M, row_ptr, tile_scratch, block_r_ind, st_off,
                                                               residue_r_ind);
        else
            fill_tiles<false><<<n_tiles, kThreads, 0, stream>>>(p, M, row_ptr, tile_scratch, block_r_ind, st_off,
                                                                residue_r_ind);
        RODE_CHECK_LAUNCH("rode::fill_tiles");
    }
    return RODE_OK;
}

int preprocess_tiles(int M) { return (M + kTile - 1) / kTile; }

// Body of the reference-signature entry point RoDe_preprocess (Preprocess_opt/_preprocess.cu:323-339):
// default stream, and nothing is written beyond the n_blk segments and n_res residue rows -- the
// reference's callers allocate nnz / seg_len + M entries for st_off (_preprocess.cu:426-430),
// which has no room for an end sentinel when every row is a whole number of segments.
int preprocess_reference_signature(int seg_len, int k_block, int vec_len, int M, const int *row_ptr,
                                   int *block_r_ind, int *st_off, int *residue_r_ind, int *n_blk, int *n_res,
                                   void *tile_scratch) {
    if (int rc = check_params(seg_len, k_block, vec_len, M, row_ptr)) return rc;
    if (!block_r_ind || !st_off || !residue_r_ind || !n_blk || !n_res)
        return fail(RODE_ERR_INVALID_ARGUMENT, "RoDe_preprocess: an output pointer is null");
    return launch_preprocess(seg_len, k_block, vec_len, M, row_ptr, block_r_ind, st_off, residue_r_ind, n_blk, n_res,
                             static_cast<int2 *>(tile_scratch), nullptr, /*write_sentinel=*/false);
}

// ---------------------------------------------------------------------------------------
// Scratch of rode_preprocess_noalloc: one int2 per tile for up to kNoAllocMaxRows rows,
// resident in every GPU that loads the library (128 KB) until the process exits.  In host
// code this name is only a handle; the device address comes from cudaGetSymbolAddress.
constexpr int kNoAllocMaxRows = 1 << 24;
constexpr int kNoAllocTiles = kNoAllocMaxRows / kTile;
static __device__ __align__(256) int2 g_noalloc_tile_scratch[kNoAllocTiles];

// Device address of the scratch array on the current device, looked up once per device.
int noalloc_scratch(int2 **out) {
    static int2 *address[64] = {nullptr};
    static std::mutex lock;
    int dev = 0;
    RODE_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(RODE_ERR_NO_DEVICE, "device index %d out of range", dev);
    std::lock_guard<std::mutex> guard(lock);
    if (address[dev] == nullptr) {
        void *p = nullptr;
        RODE_CUDA_TRY(cudaGetSymbolAddress(&p, g_noalloc_tile_scratch));
        address[dev] = static_cast<int2 *>(p);
    }
    *out = address[dev];
    return RODE_OK;
}

}  // namespace rode

extern "C" {

int rode_preprocess_workspace_bytes(int M, size_t *bytes) {
    if (bytes == nullptr || M < 0)
        return rode::fail(RODE_ERR_INVALID_ARGUMENT, "preprocess_workspace_bytes: bad argument");
    const size_t tiles = static_cast<size_t>(rode::preprocess_tiles(M));
    *bytes = (tiles > 0 ? tiles : 1) * sizeof(int2);
    return RODE_OK;
}

int rode_preprocess_capacity(int seg_len, int vec_len, int M, long long nnz, long long *max_blocks) {
    if (max_blocks == nullptr || seg_len <= 0 || vec_len <= 0 || M < 0 || nnz < 0)
        return rode::fail(RODE_ERR_INVALID_ARGUMENT, "preprocess_capacity: bad argument");
    *max_blocks = (nnz + static_cast<long long>(vec_len - 1) * M) / seg_len + M;
    return RODE_OK;
}

int rode_preprocess(int seg_len, int k_block, int vec_len, int M, const int *row_ptr, int *block_r_ind,
                    int *st_off, int *residue_r_ind, int *n_blk, int *n_res, void *workspace,
                    size_t workspace_bytes, rode_stream_t stream) {
    if (int rc = rode::check_params(seg_len, k_block, vec_len, M, row_ptr)) return rc;
    if (!block_r_ind || !st_off || !residue_r_ind || !n_blk || !n_res)
        return rode::fail(RODE_ERR_INVALID_ARGUMENT, "preprocess: an output pointer is null");
    size_t need = 0;
    rode_preprocess_workspace_bytes(M, &need);
    if (workspace == nullptr || workspace_bytes < need)
        return rode::fail(RODE_ERR_WORKSPACE, "preprocess: workspace of %zu bytes needed, %zu given", need,
                          workspace ? workspace_bytes : static_cast<size_t>(0));
    if (!rode::aligned_to(workspace, 8))
        return rode::fail(RODE_ERR_WORKSPACE, "preprocess: workspace must be 8-byte aligned");
    return rode::launch_preprocess(seg_len, k_block, vec_len, M, row_ptr, block_r_ind, st_off, residue_r_ind,
                                   n_blk, n_res, static_cast<int2 *>(workspace), stream);
}

int rode_preprocess_noalloc(int seg_len, int k_block, int vec_len, int M, const int *row_ptr, int *block_r_ind,
                            int *st_off, int *residue_r_ind, int *n_blk, int *n_res, rode_stream_t stream) {
    if (int rc = rode::check_params(seg_len, k_block, vec_len, M, row_ptr)) return rc;
    if (!block_r_ind || !st_off || !residue_r_ind || !n_blk || !n_res)
        return rode::fail(RODE_ERR_INVALID_ARGUMENT, "preprocess_noalloc: an output pointer is null");
    if (M > rode::kNoAllocMaxRows)
        return rode::fail(RODE_ERR_INVALID_ARGUMENT,
                          "preprocess_noalloc: M = %d exceeds the built-in scratch (at most %d rows); use "
                          "rode_preprocess with a caller-provided workspace",
                          M, rode::kNoAllocMaxRows);
    int2 *scratch = nullptr;
    if (int rc = rode::noalloc_scratch(&scratch)) return rc;
    // count_tiles rewrites every tile total it later reads, so nothing has to be cleared.
    return rode::launch_preprocess(seg_len, k_block, vec_len, M, row_ptr, block_r_ind, st_off, residue_r_ind,
                                   n_blk, n_res, scratch, stream);
}

int rode_preprocess_cpu(int seg_len, int k_block, int vec_len, int M, const int *row_ptr, int *block_r_ind,
                        int *st_off, int *residue_r_ind, int *n_blk, int *n_res) {
    if (int rc = rode::check_params(seg_len, k_block, vec_len, M, row_ptr)) return rc;
    if (!block_r_ind || !st_off || !residue_r_ind || !n_blk || !n_res)
        return rode::fail(RODE_ERR_INVALID_ARGUMENT, "preprocess_cpu: an output pointer is null");
    int nb = 0, nr = 0;
    for (int row = 0; row < M; ++row) {
        const int off = row_ptr[row];
        const int pad = off % vec_len;
        int left = row_ptr[row + 1] - off + pad;  // aligned length still to place
        int pos = off;                            // where the next segment starts
        while (left > seg_len) {
            block_r_ind[nb] = row;
            st_off[nb++] = pos;
            pos = (pos == off) ? off - pad + seg_len : pos + seg_len;
            left -= seg_len;
        }
        if (left >= k_block) {
            block_r_ind[nb] = row;
            st_off[nb++] = pos;
        }
        if (left % k_block != 0) residue_r_ind[nr++] = row;
    }
    st_off[nb] = row_ptr[M];
    *n_blk = nb;
    *n_res = nr;
    return RODE_OK;
}

}  // extern "C"
