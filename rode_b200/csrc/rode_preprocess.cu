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
// array, so the two kernels below are race-free:
//
//   count_tiles   one CTA per tile of kTile rows: per-row (bn, rn), tile totals -> scratch.  The
//                 CTA that finishes last (a counter in the scratch tells it) turns the totals
//                 into exclusive tile offsets and writes n_blk, n_res and the end sentinel.
//   fill_tiles    one CTA per tile: in-tile exclusive scan + tile offset; the tile's residue rows
//                 and segments are put in order in shared memory and copied out with coalesced
//                 stores; rows with many segments are written by a whole warp.  Launched as a
//                 programmatic dependent of count_tiles: its CTAs read their rows and scan them
//                 while the count grid drains, and wait for it only before they need the tile offset.
//
// HBM traffic: row_ptr is read twice (8 B/row), outputs written once (8 B/segment,
// 4 B/residue row), scratch is 8 B per 2048 rows.
#include <climits>
#include <mutex>

#include "rode_common.cuh"

namespace rode {
namespace {

// CTAs per SM the register budget must allow: the count kernel fits 32 registers (8 CTAs) without
// spilling, the fill kernel 48 (5 CTAs).
#ifndef RODE_PRE_COUNT_MIN_CTAS
#define RODE_PRE_COUNT_MIN_CTAS 8
#endif
#ifndef RODE_PRE_FILL_MIN_CTAS
#define RODE_PRE_FILL_MIN_CTAS 5
#endif
constexpr int kThreads = 256;
#ifndef RODE_PRE_ROWS_PER_THREAD
#define RODE_PRE_ROWS_PER_THREAD 8
#endif
constexpr int kRowsPerThread = RODE_PRE_ROWS_PER_THREAD;
constexpr int kTile = kThreads * kRowsPerThread;  // rows per CTA
constexpr int kWarps = kThreads / 32;
constexpr int kLongRow = 8;  // rows with more segments than this are written by a warp
// Scratch layout: slot 0 = {count of finished count_tiles CTAs, unused}, slot 1 + t = tile t.
constexpr int kScratchHeader = 1;

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
    if constexpr (kPow2) {
        // one form for both cases of the spec loop: with a <= seg_len the quotient is 0 and the
        // remainder is a itself, except a == seg_len, where quotient 1 + remainder 0 gives the same
        // single segment; and (a % seg_len) % k_block == a % k_block because k_block divides seg_len
        bn = (a >> p.seg_shift) + ((a & (p.seg_len - 1)) >= p.k_block ? 1 : 0);
        rn = (a & (p.k_block - 1)) != 0 ? 1 : 0;
    } else if (a > p.seg_len) {
        const int rest = a % p.seg_len;
        bn = a / p.seg_len + (rest >= p.k_block ? 1 : 0);
        rn = rest % p.k_block != 0 ? 1 : 0;
    } else {
        bn = a >= p.k_block ? 1 : 0;
        rn = a % p.k_block != 0 ? 1 : 0;
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

// Rows of one thread: offsets and per-row (bn, rn).  Rows at or beyond M (last tile only) count as
// empty rows that start at the matrix' end.
template <bool kPow2>
__device__ __forceinline__ void load_rows(const Params &p, int M, const int *__restrict__ row_ptr, int row0,
                                          int (&offs)[kRowsPerThread + 1], int (&bn)[kRowsPerThread],
                                          int (&rn)[kRowsPerThread], int &bsum, int &rsum) {
    bsum = 0;
    rsum = 0;
    const bool whole_tile = (static_cast<int>(blockIdx.x) + 1) * kTile <= M;  // CTA-uniform
    if (whole_tile) {
#pragma unroll
        for (int i = 0; i <= kRowsPerThread; ++i) offs[i] = __ldg(row_ptr + row0 + i);  // all independent
#pragma unroll
        for (int i = 0; i < kRowsPerThread; ++i) {
            row_counts<kPow2>(offs[i], offs[i + 1], p, bn[i], rn[i]);
            bsum += bn[i];
            rsum += rn[i];
        }
    } else {
#pragma unroll
        for (int i = 0; i <= kRowsPerThread; ++i) offs[i] = __ldg(row_ptr + min(row0 + i, M));
#pragma unroll
        for (int i = 0; i < kRowsPerThread; ++i) {
            bn[i] = 0;
            rn[i] = 0;
            if (row0 + i < M) row_counts<kPow2>(offs[i], offs[i + 1], p, bn[i], rn[i]);
            bsum += bn[i];
            rsum += rn[i];
        }
    }
}

// Tile totals, then (in the CTA that finishes last) the scan over them.  `scratch` as laid out above;
// the counter is zero when the grid starts and is left at zero.
constexpr int kScanPerThread = 8;  // tiles per thread and pass of the last CTA's scan
template <bool kPow2>
__global__ void __launch_bounds__(kThreads, RODE_PRE_COUNT_MIN_CTAS)
count_tiles(Params p, int M, const int *__restrict__ row_ptr, int2 *__restrict__ scratch, int *__restrict__ st_off,
            int *__restrict__ n_blk, int *__restrict__ n_res, bool write_sentinel) {
    __shared__ int smem[2 * kWarps];
    __shared__ bool is_last;
    int2 *tile_totals = scratch + kScratchHeader;
    int *finished = reinterpret_cast<int *>(scratch);
    {
        const int row0 = blockIdx.x * kTile + threadIdx.x * kRowsPerThread;
        int offs[kRowsPerThread + 1], bn[kRowsPerThread], rn[kRowsPerThread], bsum, rsum;
        load_rows<kPow2>(p, M, row_ptr, row0, offs, bn, rn, bsum, rsum);
        // only the totals are needed here: one warp reduction each, then the warps' sums
        const int wb = __reduce_add_sync(0xffffffffu, bsum), wr = __reduce_add_sync(0xffffffffu, rsum);
        if ((threadIdx.x & 31) == 0) {
            smem[threadIdx.x >> 5] = wb;
            smem[kWarps + (threadIdx.x >> 5)] = wr;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int tx = 0, ty = 0;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) {
                tx += smem[w];
                ty += smem[kWarps + w];
            }
            tile_totals[blockIdx.x] = make_int2(tx, ty);
            __threadfence();  // the total is visible before the count of finished CTAs moves
            is_last = atomicAdd(finished, 1) == static_cast<int>(gridDim.x) - 1;
        }
    }
    __syncthreads();
    // The fill grid may be scheduled once every CTA of this grid has come this far: its CTAs then read
    // and scan their rows while the last CTA scans the tile totals.  (Released at the START of the CTAs
    // instead, the fill grid measured 30 us slower on R-MAT scale 23 with 32-long segments, 98 against
    // 68 us, and 4 us slower on R-MAT scale 21; without the early launch at all every matrix lost 5 us.)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (!is_last) return;
    // Every other CTA has published its total.  Exclusive scan over the tiles, in place.
    __threadfence();
    const int n_tiles = static_cast<int>(gridDim.x);
    int carry_b = 0, carry_r = 0;
    for (int base = 0; base < n_tiles; base += kThreads * kScanPerThread) {
        const int t0 = base + threadIdx.x * kScanPerThread;
        int2 v[kScanPerThread];
        int sum_b = 0, sum_r = 0;
#pragma unroll
        for (int i = 0; i < kScanPerThread; ++i) {
            v[i] = make_int2(0, 0);
            if (t0 + i < n_tiles) v[i] = __ldcg(tile_totals + t0 + i);  // written by other SMs: not through L1
            sum_b += v[i].x;
            sum_r += v[i].y;
        }
        int ex, ey, tx, ty;
        block_exclusive_scan2(sum_b, sum_r, smem, ex, ey, tx, ty);
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
        if (write_sentinel) st_off[carry_b] = __ldg(row_ptr + M);
        *finished = 0;  // ready for the next call on this scratch
    }
}

// M == 0: no tile, only the counts and the sentinel.
__global__ void empty_matrix(const int *__restrict__ row_ptr, int *__restrict__ st_off, int *__restrict__ n_blk,
                             int *__restrict__ n_res, bool write_sentinel) {
    n_blk[0] = 0;
    n_res[0] = 0;
    if (write_sentinel) st_off[0] = row_ptr[0];
}

// Segments of one long row, written by the whole warp.  `row`, `off`, `cnt` are warp-uniform.
template <bool kPow2>
__device__ __forceinline__ void write_long_row(const Params &p, int lane, int row, int off, int cnt,
                                               int *__restrict__ dst_row, int *__restrict__ dst_off) {
    const int aligned = off - mod_vec<kPow2>(off, p);
    for (int j = lane; j < cnt; j += 32) {
        dst_row[j] = row;
        dst_off[j] = j == 0 ? off : aligned + j * p.seg_len;
    }
}

// The listed long rows, taken by the CTA's warps in turn.  The next row's list entry and bounds are
// fetched before the current row is written, so that chain of dependent loads is off the critical path.
template <bool kPow2>
__device__ __forceinline__ void write_long_rows(const Params &p, int lane, int warp, int total, const int *list_row,
                                                const int *list_dst, const int *__restrict__ row_ptr,
                                                int *__restrict__ out_row, int *__restrict__ out_off) {
    int s = warp;
    if (s >= total) return;
    int row = list_row[s], dst = list_dst[s];
    int off = __ldg(row_ptr + row), next = __ldg(row_ptr + row + 1);
    while (true) {
        const int s2 = s + kWarps;
        int row2 = 0, dst2 = 0, off2 = 0, next2 = 0;
        if (s2 < total) {
            row2 = list_row[s2];
            dst2 = list_dst[s2];
            off2 = __ldg(row_ptr + row2);
            next2 = __ldg(row_ptr + row2 + 1);
        }
        int cnt, unused;
        row_counts<kPow2>(off, next, p, cnt, unused);
        write_long_row<kPow2>(p, lane, row, off, cnt, out_row + dst, out_off + dst);
        if (s2 >= total) return;
        s = s2;
        row = row2;
        dst = dst2;
        off = off2;
        next = next2;
    }
}

template <bool kPow2>
__global__ void __launch_bounds__(kThreads, RODE_PRE_FILL_MIN_CTAS)
fill_tiles(Params p, int M, const int *__restrict__ row_ptr, const int2 *__restrict__ scratch,
           int *__restrict__ block_r_ind, int *__restrict__ st_off, int *__restrict__ residue_r_ind) {
    __shared__ int smem[2 * kWarps];
    // The tile's outputs in order: residue rows always, segments when the tile has at most kTile.
    __shared__ int s_res[kTile];
    __shared__ int s_seg_row[kTile];
    __shared__ int s_seg_off[kTile];
    // Rows with more than kLongRow segments are listed and then written by the CTA's warps in turn
    // (on skewed matrices they cluster in the first lanes of a tile).  A staged tile has at most
    // kTile / (kLongRow + 1) of them; a tile that is not staged keeps the list in the staging arrays.
    constexpr int kLongCap = kTile / (kLongRow + 1) + 1;
    __shared__ int s_long_row[kLongCap];
    __shared__ int s_long_dst[kLongCap];
    __shared__ int n_long;
    if (threadIdx.x == 0) n_long = 0;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    const int row0 = blockIdx.x * kTile + threadIdx.x * kRowsPerThread;
    int offs[kRowsPerThread + 1], bn[kRowsPerThread], rn[kRowsPerThread], bsum, rsum;
    load_rows<kPow2>(p, M, row_ptr, row0, offs, bn, rn, bsum, rsum);
    int ex, ey, tx, ty;
    block_exclusive_scan2(bsum, rsum, smem, ex, ey, tx, ty);  // also orders n_long = 0
    const bool staged = tx <= kTile;  // CTA-uniform
    int *list_row = staged ? s_long_row : s_seg_row;
    int *list_dst = staged ? s_long_dst : s_seg_off;

    // ---- residue rows, the list of long rows, and a staged tile's short rows ----------------------
    int lr = ey, lb = ex;
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
        if (rn[i]) s_res[lr] = row0 + i;
        lr += rn[i];
        if (bn[i] > kLongRow) {
            const int slot = atomicAdd(&n_long, 1);  // shared-memory slot counter, order irrelevant
            list_row[slot] = row0 + i;
            list_dst[slot] = lb;
        } else if (staged && bn[i] > 0) {
            const int off = offs[i];
            const int aligned = off - mod_vec<kPow2>(off, p);
            s_seg_row[lb] = row0 + i;
            s_seg_off[lb] = off;
            for (int j = 1; j < bn[i]; ++j) {
                s_seg_row[lb + j] = row0 + i;
                s_seg_off[lb + j] = aligned + j * p.seg_len;
            }
        }
        lb += bn[i];
    }
    __syncthreads();
    const int total_long = n_long;
    if (staged) {
        write_long_rows<kPow2>(p, lane, warp, total_long, list_row, list_dst, row_ptr, s_seg_row, s_seg_off);
        __syncthreads();
    }

    // ---- the tile's place in the outputs: written by the count grid's last CTA --------------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int2 tile_off = __ldcg(scratch + kScratchHeader + blockIdx.x);
    for (int i = threadIdx.x; i < ty; i += kThreads) residue_r_ind[tile_off.y + i] = s_res[i];
    if (staged) {
        for (int i = threadIdx.x; i < tx; i += kThreads) {
            block_r_ind[tile_off.x + i] = s_seg_row[i];
            st_off[tile_off.x + i] = s_seg_off[i];
        }
        return;
    }
    // A tile with more segments than the staging holds (very long rows): straight to the outputs.
    int gb = tile_off.x + ex;
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
        if (bn[i] > 0 && bn[i] <= kLongRow) {
            const int off = offs[i];
            const int aligned = off - mod_vec<kPow2>(off, p);
            block_r_ind[gb] = row0 + i;
            st_off[gb] = off;
            for (int j = 1; j < bn[i]; ++j) {
                block_r_ind[gb + j] = row0 + i;
                st_off[gb + j] = aligned + j * p.seg_len;
            }
        }
        gb += bn[i];
    }
    write_long_rows<kPow2>(p, lane, warp, total_long, list_row, list_dst, row_ptr, block_r_ind + tile_off.x,
                           st_off + tile_off.x);
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

// Launches the two kernels; `scratch` holds kScratchHeader + one int2 per tile.  write_sentinel: also
// store st_off[n_blk] = row_ptr[M] (the C ABI's contract; the reference's device version does
// not, and its callers size st_off without room for it).
template <bool kPow2>
int launch_preprocess_kernels(const Params &p, int n_tiles, int M, const int *row_ptr, int *block_r_ind, int *st_off,
                              int *residue_r_ind, int *n_blk, int *n_res, int2 *scratch, cudaStream_t stream,
                              bool write_sentinel) {
    // the count of finished CTAs: the scratch may be a caller's buffer with any contents
    RODE_CUDA_TRY(cudaMemsetAsync(scratch, 0, sizeof(int2), stream));
    count_tiles<kPow2><<<n_tiles, kThreads, 0, stream>>>(p, M, row_ptr, scratch, st_off, n_blk, n_res, write_sentinel);
    RODE_CHECK_LAUNCH("rode::count_tiles");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int2 *scratch_in = scratch;
    RODE_CUDA_TRY(cudaLaunchKernelEx(&cfg, fill_tiles<kPow2>, p, M, row_ptr, scratch_in, block_r_ind, st_off,
                                     residue_r_ind));
    RODE_CHECK_LAUNCH("rode::fill_tiles");
    return RODE_OK;
}

int launch_preprocess(int seg_len, int k_block, int vec_len, int M, const int *row_ptr, int *block_r_ind,
                      int *st_off, int *residue_r_ind, int *n_blk, int *n_res, int2 *tile_scratch,
                      cudaStream_t stream, bool write_sentinel = true) {
    const int n_tiles = (M + kTile - 1) / kTile;
    auto pow2 = [](int x) { return (x & (x - 1)) == 0; };
    const bool all_pow2 = pow2(seg_len) && pow2(k_block) && pow2(vec_len);
    Params p = {seg_len, k_block, vec_len, 0};
    while (all_pow2 && (1 << p.seg_shift) < seg_len) ++p.seg_shift;
    if (n_tiles == 0) {
        empty_matrix<<<1, 1, 0, stream>>>(row_ptr, st_off, n_blk, n_res, write_sentinel);
        RODE_CHECK_LAUNCH("rode::empty_matrix");
        return RODE_OK;
    }
    if (all_pow2)
        return launch_preprocess_kernels<true>(p, n_tiles, M, row_ptr, block_r_ind, st_off, residue_r_ind, n_blk, n_res,
                                               tile_scratch, stream, write_sentinel);
    return launch_preprocess_kernels<false>(p, n_tiles, M, row_ptr, block_r_ind, st_off, residue_r_ind, n_blk, n_res,
                                            tile_scratch, stream, write_sentinel);
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
// resident in every GPU that loads the library (64 KB) until the process exits.  In host
// code this name is only a handle; the device address comes from cudaGetSymbolAddress.
constexpr int kNoAllocMaxRows = 1 << 24;
constexpr int kNoAllocTiles = kNoAllocMaxRows / kTile;
static __device__ __align__(256) int2 g_noalloc_tile_scratch[kScratchHeader + kNoAllocTiles];

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
    *bytes = (tiles + rode::kScratchHeader) * sizeof(int2);
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
    // count_tiles rewrites every tile total it later reads; the counter is cleared on the stream.
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
