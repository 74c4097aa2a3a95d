// RoDe SpMM for sm_100a:  C[M x n] = S * B  with S in CSR + row-decomposition metadata.
//
// Stands in for the reference's block / residue kernels (RoDe_SpMM/RoDeSpmm.cu:197-476 and
// :41-195) and their launcher (:492-529).  The work split follows the reference's metadata
// (block segments, residue rows); how the work is done is new:
//
//  * A dense-row slice of the column tile (8, 16 or 32 vectors of 16 bytes) is covered by a
//    lane group of L lanes with VPL vectors per lane (LDG.128 each): 4 x 2 for 8 vectors (8 x 1 in
//    the block kernel), 8 x 2 for 16, 32 x 1 for 32.  Two vectors per lane halve the shuffles and the address
//    arithmetic per byte (measured: N = 32 power-law 0.68 -> 0.58 ms, N = 64 R-MAT-21
//    0.99 -> 0.75 ms, N = 64 stencil 0.97 -> 0.75 ms; for 32 vectors no shape beat 32 x 1).
//    A warp holds G = 32/L lane groups.
//  * Gathers are issued in batches of 8 independent LDG.128 per lane; the (column,
//    value) pairs of a chunk of 32 nonzeros are fetched two chunks ahead, stored once into a
//    double-buffered shared-memory tile and read by every lane group as 16-byte broadcast runs
//    (one shuffle per pair element and nonzero costs the SM's load/store data path as much as
//    128 bytes of gathered data).  Bytes in flight per SM = resident warps x 32 x U x 16 B, so the
//    kernels are kept at 64 registers (32 one-warp CTAs per SM, ~131 KB in flight).  Two
//    register buffers per lane (software pipelining) were measured and rejected: 168
//    registers cut the resident warps to 12 and the time went up by 30 %.
//  * spmm_block: one warp per block segment; the G groups take alternate nonzeros and are
//    combined with log2(G) shuffle steps at the end.  The LAST segment of a row also
//    consumes the row's tail (the part shorter than 32 that the reference leaves to its
//    residue kernel), so a row that fits one segment is finished by a single warp and
//    stored with plain vector stores.
//  * Rows cut into several segments: every segment writes its partial row to a workspace
//    slot (slot = segment index); spmm_fixup, ordered after spmm_block on the same stream,
//    sums the slots of each such row in a fixed order (fp64 accumulation) and stores the
//    row.  No floating-point atomics anywhere: results are deterministic.
//  * spmm_rows (L = 32): residue rows that have no block part (aligned length < 32).  A warp
//    takes 32 consecutive residue rows at once: lane j reads the descriptor of row j, so the
//    dependent chain row index -> row pointer -> column -> dense row is paid once per 32
//    rows, not per row.  The nonzeros of the 32 rows form one entry stream that runs through
//    the same batched gather; a row is stored when the stream passes its end.
//    spmm_rows_simple (L < 32): one lane group per residue row; spmm_rows_wide: one warp per
//    row, for lists too short to fill the GPU.
//    Rows of the list without a nonzero are not touched (the reference stores zeros there,
//    RoDeSpmm.cu:185-194, into a C that its contract already wants zero-filled); rows with a
//    block part are skipped (spmm_block finished them).
//  * CTAs are one warp (four in spmm_rows_wide, whose rows are all shorter than 32): a CTA's
//    slot is held until its slowest warp finishes, and segment lengths differ by more than 10x.
//
// Per nonzero the kernels move 8 B of CSR data and 16*L bytes of the dense operand (from
// L1/L2/HBM depending on reuse); per row 4*n bytes of C.  Dense-row offsets are 64-bit.
#include <climits>
#include <type_traits>

#include "rode_common.cuh"

namespace rode {
namespace {

#ifndef RODE_SPMM_CTA_WARPS
#define RODE_SPMM_CTA_WARPS 1
#endif
// Small CTAs: a CTA's slot is held until its slowest warp is done, and segments differ in
// length by more than 10x, so fewer warps per CTA keep more warps resident on average.
constexpr int kCtaWarps = RODE_SPMM_CTA_WARPS;
constexpr int kCtaThreads = 32 * kCtaWarps;
#ifndef RODE_SPMM_WIDE_ROWS_CTA_WARPS
#define RODE_SPMM_WIDE_ROWS_CTA_WARPS 4
#endif
constexpr int kSmallGridWarps = RODE_SPMM_WIDE_ROWS_CTA_WARPS;  // rows (warps) per CTA of spmm_rows_wide

// Shape of a lane group per tile width (in 16-byte vectors: 8, 16 or 32 per dense-row slice):
// L lanes x VPL vectors per lane, encoded as L * 100 + VPL.
// (8 x 1 in the block kernel of the 128-byte tile: a load instruction then covers whole 128-byte lines, 4
// rows per warp, where 4 x 2 covers 8 half lines.  R-MAT 23 N = 32 block kernel 2.19 -> 1.20 ms, R-MAT 21
// N = 96 1.43 -> 0.92 ms, Zipf N = 32 -7 %; uniformly random columns lose 3 %: Pareto 2^20 N = 32 0.354 ->
// 0.365 ms.  The per-row residue kernels measured faster with 4 x 2: R-MAT 23 N = 32 0.756 against 1.079 ms.)
#ifndef RODE_SPMM_SHAPE_8
#define RODE_SPMM_SHAPE_8 801
#endif
// Residue rows of 8-vector tiles (spmm_rows_simple, spmm_rows_wide) may use another shape than the block kernel.
#ifndef RODE_SPMM_ROWS_SHAPE_8
#define RODE_SPMM_ROWS_SHAPE_8 402
#endif
#ifndef RODE_SPMM_SHAPE_16
#define RODE_SPMM_SHAPE_16 802
#endif
#ifndef RODE_SPMM_SHAPE_32
#define RODE_SPMM_SHAPE_32 3201
#endif
// Residue rows of 32-vector tiles may use another shape than the block kernel (3201 selects
// the batched spmm_rows kernel).
#ifndef RODE_SPMM_ROWS_SHAPE_32
#define RODE_SPMM_ROWS_SHAPE_32 3201
#endif
// Widest column tile (in 16-byte vectors) a launch covers; narrower tiles walk the columns
// in several passes over the sparse matrix (grid.y), which shrinks the dense working set of
// each pass.
#ifndef RODE_SPMM_MAX_TILE_VECS
#define RODE_SPMM_MAX_TILE_VECS 32
#endif
// 128-byte tile (N = 32 floats, 16 doubles) with one 32-byte load per lane and 4 lanes per dense row (1) or
// with the 16-byte shapes above (0).  Stencil 128^3 N = 32 0.510 -> 0.401 ms (a load instruction of the
// per-row kernel covers whole lines of 8 rows instead of half lines); the other matrices measure the same
// as with the 8 x 1 block shape.
#ifndef RODE_SPMM_TILE8_WIDE_LOADS
#define RODE_SPMM_TILE8_WIDE_LOADS 1
#endif
// Bytes per load instruction of a lane in the block kernel and the per-row residue kernels:
// 16 (LDG.128) or 32 (the 256-bit loads of sm_100).  The shapes above are given in 16-byte
// vectors; with 32-byte loads a lane group has half as many lanes.
#ifndef RODE_SPMM_VEC_BYTES
#define RODE_SPMM_VEC_BYTES 16
#endif
// How the (column, value) pairs of a chunk reach the lanes that gather with them: 1 = through
// shared memory (the chunk is stored once, every lane group reads its run with 16-byte broadcast
// loads), 0 = by one shuffle per pair and element.  Shuffles and loads share the SM's load/store
// data path, where a shuffle costs as much as 128 bytes of gathered data.
#ifndef RODE_SPMM_PAIRS_IN_SMEM
#define RODE_SPMM_PAIRS_IN_SMEM 1
#endif
// Block kernel: a separate unpredicated form for full chunks of 32 nonzeros (1) or one predicated form (0).
#ifndef RODE_SPMM_FULL_CHUNK_PATH
#define RODE_SPMM_FULL_CHUNK_PATH 1
#endif
// Claim counters of the persistent block kernel: one int per column tile, at the end of the workspace.
constexpr size_t kCounterBytes = 256;
constexpr unsigned kMaxCounterTiles = kCounterBytes / sizeof(int);
// Residue-row kernel of the 512-byte tile as a persistent grid too (1) or one CTA per bundle of rows (0).
#ifndef RODE_SPMM_PERSISTENT_ROWS
#define RODE_SPMM_PERSISTENT_ROWS 1
#endif
// A grid becomes persistent from this many resident waves of work on: with fewer segments per warp
// the claimed order's tail (one long segment claimed last) costs more than the launch gaps it
// saves (measured: gain from about 20 segments per warp, loss below 10).
constexpr int kPersistentMinWaves = 16;
// Block kernel as a persistent grid: CTAs per SM of the one wave that is launched (0 = one CTA per
// segment instead).
#ifndef RODE_SPMM_PERSISTENT_CTAS_PER_SM
#define RODE_SPMM_PERSISTENT_CTAS_PER_SM 32
#endif
// 16-byte units a lane keeps in flight per batch (dense rows per batch = this * 16 / bytes per load / VPL).
constexpr int kLoadsInFlight = 8;

// ---------------------------------------------------------------------------------------
// One warp per block segment; grid.y walks the column tiles of L * VPL vectors.  U = dense
// rows per batch: kLoadsInFlight / VPL for grids that fill the GPU (64 registers keep 32
// warps per SM resident); the whole chunk for small grids, where the time is the
// dependent-batch chain of the longest segment and registers are free.
// One-warp CTAs per SM that the register budget must allow, by 16-byte loads in flight per
// lane: 8 -> 32 CTAs (64 registers), 12 -> 25 (80), 16 -> 20 (96), more -> no limit.
constexpr int min_ctas_per_sm(int loads) { return loads <= 8 ? 32 : loads <= 12 ? 25 : loads <= 16 ? 20 : 1; }

// kRagged: the width is not a multiple of the tile; the last tile's lanes beyond the row's end neither
// load nor store (widths the reference's tiles do not serve: any multiple of 4 columns).
template <typename T, int VB, int L, int VPL, int U, int W, bool kHints, bool kClaim, bool kRagged>
__global__ void __launch_bounds__(32 * W, min_ctas_per_sm(U * VPL * VB / 16) / W)
spmm_block(int m1, int n, const T *__restrict__ values, const int *__restrict__ column_indices,
           const int *__restrict__ row_offsets, const int *__restrict__ block_r_ind,
           const int *__restrict__ st_off, const T *__restrict__ B, T *__restrict__ C, T *__restrict__ partial,
           const unsigned *__restrict__ hot, int hot_flag_word, int *__restrict__ next_segment) {
    using V = typename VecB<T, VB>::type;
    constexpr int kLen = VecB<T, VB>::kLen;
    constexpr int G = 32 / L;             // lane groups, each takes every G-th nonzero
    constexpr int kSteps = 32 / G;        // nonzeros per group per 32-nonzero chunk
    constexpr int NB = (kSteps + U - 1) / U;
    constexpr unsigned kFull = 0xffffffffu;
    // Programmatic dependent launch: as soon as every CTA of this grid has started, the fix-up
    // grid may be scheduled into free slots.  Its warps look for rows that were cut into
    // several segments; those that find none exit at once, the others wait for this grid to
    // complete before they read the workspace.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int g = lane / L, l = lane % L;
    // Chunk staging (two buffers, so one __syncwarp per chunk orders both the reads after the
    // writes and the next-but-one chunk's writes after these reads).  The pair of position t
    // sits at (t % G) * kSteps + t / G: the run of a lane group is contiguous.
    constexpr bool kStage = RODE_SPMM_PAIRS_IN_SMEM != 0 && (kSteps % U == 0) && (U % 4 == 0);
    __shared__ __align__(16) int s_col[kStage ? W : 1][2][32];
    __shared__ __align__(16) T s_val[kStage ? W : 1][2][32];
    const int warp_in_cta = kStage ? (threadIdx.x >> 5) : 0;
    const int stage_slot = (lane % G) * kSteps + lane / G;
    int stage_buf = 0;
    const size_t row_vecs = static_cast<size_t>(n) / kLen;
    const unsigned row_bytes = static_cast<unsigned>(n) * static_cast<unsigned>(sizeof(T));  // n < 2^21 elements
    const size_t col_vec = static_cast<size_t>(blockIdx.y) * L * VPL + l;  // + v * L for vector v
    const V *b_lane = reinterpret_cast<const V *>(B) + col_vec;
    auto inside = [&](int v) { return !kRagged || col_vec + v * L < row_vecs; };
    GatherPolicy policy = {};
    // the word after the bitmap is the library's verdict on this matrix (0: marks would not help)
    if constexpr (kHints) policy = make_gather_policy(__ldg(hot + hot_flag_word) != 0u);

    // Persistent form (next_segment != null, a grid of one resident wave): a warp starts with the
    // segment of its own index and then claims further ones from a counter per column tile, so no
    // warp slot waits for a new CTA to be launched into it (one-warp CTAs of a few microseconds
    // each left a fifth of the slots empty at any time).  The claim is issued before the segment's
    // work and read after it, so its latency is hidden.  Otherwise one segment per warp.
    int seg = blockIdx.x * W + (threadIdx.x >> 5);
    while (seg < m1) {
    int claimed = INT_MAX;
    if constexpr (kClaim) {
        if (next_segment != nullptr && lane == 0)
            claimed = static_cast<int>(gridDim.x) * W + atomicAdd(next_segment + blockIdx.y, 1);
    }
    const int row = __ldg(block_r_ind + seg);
    const int off = __ldg(st_off + seg);
    const int next = (seg + 1 < m1) ? __ldg(st_off + seg + 1) : INT_MAX;
    const int row_begin = __ldg(row_offsets + row);
    const int row_end = __ldg(row_offsets + row + 1);
    const int end = min(row_end, next);
    const bool whole_row = (off == row_begin) && (next >= row_end);

    // (column, value) of this lane's nonzero in the current and in the next chunk
    int c_cur = 0, c_nxt = 0;
    T v_cur = T(0), v_nxt = T(0);
    if (off + lane < end) {
        c_cur = ld_stream(column_indices + off + lane);
        v_cur = ld_stream(values + off + lane);
    }
    if (off + 32 + lane < end) {
        c_nxt = ld_stream(column_indices + off + 32 + lane);
        v_nxt = ld_stream(values + off + 32 + lane);
    }
    // With popularity hints a column index carries its mark in bit 31.  The bitmap word of a
    // column is fetched one chunk after the column itself (which has arrived by then) and one
    // chunk before the column is used, so the lookup adds no exposed latency after the first.
    if constexpr (kHints) c_cur = tag_hot(c_cur, hot_word(hot, c_cur));

    V acc[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) acc[v] = vzero(static_cast<V *>(nullptr));
    for (int base = off; base < end; base += 32) {
        const int cnt = min(32, end - base);
        int c_pre = 0;
        T v_pre = T(0);
        if (base + 64 + lane < end) {  // pairs of the chunk after next
            c_pre = ld_stream(column_indices + base + 64 + lane);
            v_pre = ld_stream(values + base + 64 + lane);
        }
        unsigned w_nxt = 0;
        if constexpr (kHints) w_nxt = hot_word(hot, c_nxt);
        if constexpr (kStage) {
            s_col[warp_in_cta][stage_buf][stage_slot] = c_cur;
            s_val[warp_in_cta][stage_buf][stage_slot] = v_cur;
            __syncwarp();
        }
        // One chunk of the batched gather.  A full chunk (every chunk of a segment but its last) can take
        // a form without bounds: no predicate per gather and no zero-fill of the row buffers (ncu counted
        // 23 warp instructions per gathered row in the predicated form: 4 FMA, 1 load, the rest address,
        // policy, predicate and zero-fill work).
        auto chunk = [&](auto full_tag) {
            constexpr bool kFullChunk = decltype(full_tag)::value;
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                if constexpr (!kFullChunk) {
                    if (b * U * G >= cnt) break;  // warp-uniform
                }
                V buf[U][VPL];
                T vv[U];
                int cc[U];
                if constexpr (kStage) {
                    ld_shared_run<U>(&s_col[warp_in_cta][stage_buf][g * kSteps + b * U], cc);
                    ld_shared_run<U>(&s_val[warp_in_cta][stage_buf][g * kSteps + b * U], vv);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int t = (b * U + u) * G + g;  // position inside the chunk
                    if constexpr (!kStage) {
                        cc[u] = __shfl_sync(kFull, c_cur, t & 31);
                        vv[u] = __shfl_sync(kFull, v_cur, t & 31);
                    }
#pragma unroll
                    for (int v = 0; v < VPL; ++v) {
                        if constexpr (kFullChunk && !kRagged) {
                            buf[u][v] = gather<kHints>(b_lane + v * L, cc[u], row_bytes, policy);
                        } else {
                            buf[u][v] = vzero(static_cast<V *>(nullptr));
                            if ((kFullChunk || t < cnt) && inside(v))
                                buf[u][v] = gather<kHints>(b_lane + v * L, cc[u], row_bytes, policy);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u)
#pragma unroll
                    for (int v = 0; v < VPL; ++v) vfma(acc[v], vv[u], buf[u][v]);
            }
        };
        // (only the 512-byte tile of large grids: R-MAT 21 N = 128 block kernel 0.818 -> 0.787 ms, R-MAT 23
        // step 4.76 -> 4.62 ms; the narrower shapes and the small-grid form measured 1-2 % slower with it)
        constexpr bool kFullChunkPath = RODE_SPMM_FULL_CHUNK_PATH != 0 && L == 32 && U == kLoadsInFlight / VPL;
        if (kFullChunkPath && cnt == 32)
            chunk(std::true_type{});
        else
            chunk(std::false_type{});
        c_cur = kHints ? tag_hot(c_nxt, w_nxt) : c_nxt;
        v_cur = v_nxt;
        c_nxt = c_pre;
        v_nxt = v_pre;
        stage_buf ^= 1;
    }
#pragma unroll
    for (int v = 0; v < VPL; ++v)
#pragma unroll
        for (int w = L; w < 32; w <<= 1) vadd(acc[v], vshfl_xor(kFull, acc[v], w));

    if (g == 0) {
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            if (!inside(v)) continue;
            if (whole_row)
                st_stream(reinterpret_cast<V *>(C) + static_cast<size_t>(row) * row_vecs + col_vec + v * L, acc[v]);
            else
                reinterpret_cast<V *>(partial)[static_cast<size_t>(seg) * row_vecs + col_vec + v * L] = acc[v];
        }
    }
    seg = kClaim ? __shfl_sync(kFull, claimed, 0) : INT_MAX;
    }  // segments of this warp
}

// ---------------------------------------------------------------------------------------
// Sums the workspace slots of every row that was cut into several segments.  A one-warp CTA
// looks at 32 consecutive segments; a lane whose segment is the first of a split row flags
// it, and the warp then adds that row's slots (fp64 accumulation, eight slots in flight per
// lane; the order is fixed by the code, so the result is deterministic).
constexpr int kFixupThreads = 32;
constexpr int kFixupUnroll = 8;  // workspace slots in flight per lane

template <typename T>
__global__ void __launch_bounds__(kFixupThreads)
spmm_fixup(int m1, int n, const int *__restrict__ row_offsets, const int *__restrict__ block_r_ind,
           const int *__restrict__ st_off, const T *__restrict__ partial, T *__restrict__ C) {
    constexpr unsigned kFull = 0xffffffffu;
    const int lane = threadIdx.x;
    const int seg = blockIdx.x * 32 + lane;
    bool head = false;
    int row = 0, count = 0;
    if (seg < m1) {
        row = __ldg(block_r_ind + seg);
        const int off = __ldg(st_off + seg);
        const int next = (seg + 1 < m1) ? __ldg(st_off + seg + 1) : INT_MAX;
        const int row_begin = __ldg(row_offsets + row);
        const int row_end = __ldg(row_offsets + row + 1);
        head = (off == row_begin) && (next < row_end);
        if (head) {
            // number of segments of the row = pieces of (next - aligned start) nonzeros
            const int piece = next - (row_begin - row_begin % 4);
            count = (row_end - (row_begin - row_begin % 4) + piece - 1) / piece;
            // the last piece is a segment only if it is >= 32 long; otherwise it was a
            // residue tail that the previous segment consumed
            const int last_len = row_end - (row_begin - row_begin % 4) - (count - 1) * piece;
            if (last_len < 32) --count;
        }
    }
    unsigned todo = __ballot_sync(kFull, head);
    if (todo == 0) {
        // No split row among these 32 segments: nothing to read from the workspace.  The first
        // CTA still waits for the block grid, so that this grid as a whole cannot complete
        // before spmm_block has completed and flushed its stores: whatever the caller enqueues
        // on the stream afterwards (an event, a copy of C, the next kernel) is then ordered
        // after the block grid through this grid, as with a plain launch.
        if (blockIdx.x == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
        return;
    }
    // Everything above read only the caller's metadata; the workspace is written by the
    // preceding spmm_block grid: wait for it (no-op when launched without the attribute).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    while (todo) {
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        const int first = blockIdx.x * 32 + src;
        const int r = __shfl_sync(kFull, row, src);
        const int cnt = __shfl_sync(kFull, count, src);
        // 4 columns per lane.  Rows narrower than 128 columns leave lanes over: those form
        // 32 / (n/4) groups that take alternate slots and are combined by shuffles.
        const int quads = n / 4;
        const int width = (quads == 8 || quads == 16) ? quads : 32;  // lanes per slot
        const int groups = 32 / width;
        const int g = lane / width, l = lane % width;
        for (int x = l * 4; x < n; x += 128) {
            double acc[4] = {0.0, 0.0, 0.0, 0.0};
            for (int s0 = g; s0 < cnt; s0 += groups * kFixupUnroll) {
                T v[kFixupUnroll][4];
#pragma unroll
                for (int u = 0; u < kFixupUnroll; ++u) {
                    const int s = s0 + u * groups;
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[u][j] = T(0);
                    if (s < cnt) {
                        const T *src_row = partial + static_cast<size_t>(first + s) * n + x;
#pragma unroll
                        for (int j = 0; j < 4; ++j) v[u][j] = src_row[j];
                    }
                }
#pragma unroll
                for (int u = 0; u < kFixupUnroll; ++u)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[j] += static_cast<double>(v[u][j]);
            }
            for (int w = width; w < 32; w <<= 1)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j] += __shfl_xor_sync(kFull, acc[j], w);
            if (g == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) C[static_cast<size_t>(r) * n + x + j] = static_cast<T>(acc[j]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Residue rows without a block part.  One lane group per L consecutive entries of
// residue_r_ind; grid.y walks the column tiles.
template <typename T, int L, bool kRagged>
__global__ void __launch_bounds__(kCtaThreads, (sizeof(T) == 4 ? 32 : 16) / kCtaWarps)  // fp32: 64 registers
spmm_rows(int m2, int rows_per_group, int n, const T *__restrict__ values,
          const int *__restrict__ column_indices, const int *__restrict__ row_offsets,
          const int *__restrict__ residue_r_ind, const T *__restrict__ B, T *__restrict__ C,
          int *__restrict__ next_group) {
    using V = typename Vec16<T>::type;
    constexpr int kLen = Vec16<T>::kLen;
    constexpr int U = (kLoadsInFlight < L) ? kLoadsInFlight : L;  // rows per batch
    constexpr int NB = (L + U - 1) / U;  // batches per L-nonzero chunk
    constexpr int kAlign = 4;            // vec_len of the preprocessing
    constexpr int kBlockK = 32;          // k_block of the preprocessing
    const int lane = threadIdx.x & 31;
    const int l = lane % L;
    const unsigned gmask = group_mask<L>(lane);
    const int gshift = lane & ~(L - 1);
    // chunk staging in shared memory as in spmm_block (one region of L pairs per lane group)
    constexpr bool kStage = RODE_SPMM_PAIRS_IN_SMEM != 0 && (L % U == 0) && (U % 4 == 0);
    __shared__ __align__(16) int s_col[2][kStage ? kCtaThreads : 1];
    __shared__ __align__(16) T s_val[2][kStage ? kCtaThreads : 1];
    const int stage_base = (threadIdx.x / L) * L;  // first slot of this group's region
    int stage_buf = 0;
    // Persistent form (next_group != null, a grid of one resident wave): a lane group starts with
    // the bundle of rows of its own index and claims further bundles from a counter per column
    // tile; the claim is issued before the bundle's work and read after it.
    const long long n_groups = (static_cast<long long>(m2) + rows_per_group - 1) / rows_per_group;
    long long group = (static_cast<long long>(blockIdx.x) * kCtaThreads + threadIdx.x) / L;
    while (group < n_groups) {
    int claimed = INT_MAX;
    constexpr bool kClaim = sizeof(T) == 4;  // fp64: 12 more registers for it cost more than it gains
    if constexpr (kClaim) {
        if (next_group != nullptr && l == 0)
            claimed = static_cast<int>(gridDim.x) * (kCtaThreads / L) + atomicAdd(next_group + blockIdx.y, 1);
    }
    [&]() {
    const int item0 = static_cast<int>(group * rows_per_group);

    // ---- descriptors: lane j of the group owns residue row item0 + j -----------------------
    int row = 0, begin = 0, len = 0;
    if (l < rows_per_group && item0 + l < m2) {
        row = __ldg(residue_r_ind + item0 + l);
        begin = __ldg(row_offsets + row);
        const int end = __ldg(row_offsets + row + 1);
        // aligned length >= k_block: a block part exists and its last segment took the tail
        if (end - begin + (begin % kAlign) < kBlockK) len = end - begin;
    }
    int start = len;  // exclusive prefix sum of len inside the group
#pragma unroll
    for (int d = 1; d < L; d <<= 1) {
        const int up = __shfl_up_sync(gmask, start, d, L);
        if (l >= d) start += up;
    }
    const int total = __shfl_sync(gmask, start, L - 1, L);
    start -= len;

    const size_t row_vecs = static_cast<size_t>(n) / kLen;
    const unsigned row_bytes = static_cast<unsigned>(n) * static_cast<unsigned>(sizeof(T));  // n < 2^21 elements
    const size_t col_vec = static_cast<size_t>(blockIdx.y) * L + l;
    const V *b_lane = reinterpret_cast<const V *>(B) + col_vec;
    V *c_lane = reinterpret_cast<V *>(C) + col_vec;
    const bool inside = !kRagged || col_vec < row_vecs;  // ragged widths: lanes beyond the row's end idle

    // Rows of the list without a nonzero are left alone: C arrives zero-filled (the contract of
    // the reference's entry points), and on graphs with many empty rows the zero rows were half
    // of this kernel's DRAM writes.
    unsigned todo = (__ballot_sync(gmask, len > 0) & gmask) >> gshift;  // rows with nonzeros, in order
    if (todo == 0) return;

    // ---- entry stream: position p -> nonzero index -------------------------------------------------
    auto fetch = [&](int p, int &c, T &v) {  // all lanes of the group call
        int lo = 0;
#pragma unroll
        for (int step = L / 2; step >= 1; step >>= 1) {
            const int s = __shfl_sync(gmask, start, lo + step, L);
            if (s <= p) lo += step;
        }
        const int b0 = __shfl_sync(gmask, begin, lo, L);
        const int s0 = __shfl_sync(gmask, start, lo, L);
        c = 0;
        v = T(0);
        if (p < total) {
            c = ld_stream(column_indices + b0 + (p - s0));
            v = ld_stream(values + b0 + (p - s0));
        }
    };
    int c_cur, c_nxt;
    T v_cur, v_nxt;
    fetch(l, c_cur, v_cur);
    fetch(L + l, c_nxt, v_nxt);

    // ---- consumer state: the row being accumulated -------------------------------------------------
    int cur = __ffs(todo) - 1;
    todo &= todo - 1;
    int cur_row = __shfl_sync(gmask, row, cur, L);
    int cur_end = __shfl_sync(gmask, start, cur, L) + __shfl_sync(gmask, len, cur, L);
    int pos = 0;
    V acc = vzero(static_cast<V *>(nullptr));

    for (int base = 0; base < total; base += L) {
        const int cnt = min(L, total - base);
        int c_pre;
        T v_pre;
        fetch(base + 2 * L + l, c_pre, v_pre);
        if constexpr (kStage) {
            s_col[stage_buf][stage_base + l] = c_cur;
            s_val[stage_buf][stage_base + l] = v_cur;
            __syncwarp(gmask);
        }
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            if (b * U >= cnt) break;  // group-uniform
            V buf[U];
            T vv[U];
            int cc[U];
            if constexpr (kStage) {
                ld_shared_run<U>(&s_col[stage_buf][stage_base + b * U], cc);
                ld_shared_run<U>(&s_val[stage_buf][stage_base + b * U], vv);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = b * U + u;  // position inside the chunk
                if constexpr (!kStage) {
                    cc[u] = __shfl_sync(gmask, c_cur, t, L);
                    vv[u] = __shfl_sync(gmask, v_cur, t, L);
                }
                buf[u] = vzero(static_cast<V *>(nullptr));
                if (t < cnt && inside) buf[u] = ld_dense(dense_row(b_lane, static_cast<unsigned>(cc[u]), row_bytes));
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                vfma(acc, vv[u], buf[u]);
                ++pos;
                if (pos == cur_end) {  // the stream passed the end of a row: store it, start the next
                    if (inside) st_stream(c_lane + static_cast<size_t>(cur_row) * row_vecs, acc);
                    acc = vzero(static_cast<V *>(nullptr));
                    if (todo) {
                        cur = __ffs(todo) - 1;
                        todo &= todo - 1;
                        cur_row = __shfl_sync(gmask, row, cur, L);
                        cur_end = __shfl_sync(gmask, start, cur, L) + __shfl_sync(gmask, len, cur, L);
                    } else {
                        cur_end = INT_MAX;
                    }
                }
            }
        }
        c_cur = c_nxt;
        v_cur = v_nxt;
        c_nxt = c_pre;
        v_nxt = v_pre;
        stage_buf ^= 1;
    }
    }();
    group = kClaim ? __shfl_sync(gmask, claimed, 0, L) : n_groups;
    }  // bundles of this group
}

// ---------------------------------------------------------------------------------------
// Residue rows without a block part, one lane group (L lanes x VPL vectors) per row.  Used
// where a warp holds several groups: there the groups would run different entry streams in
// spmm_rows and diverge, which measured slower (stencil N = 64: 1.43 ms against 0.93 ms),
// while for 32-lane groups the batched kernel wins (R-MAT N = 128: 327 us against 770 us).
#ifndef RODE_SPMM_ROWS_CTA
#define RODE_SPMM_ROWS_CTA 32
#endif
constexpr int kRowsCtaThreads = RODE_SPMM_ROWS_CTA;
// spmm_rows_wide (a warp per row) serves lists of at most this many full waves of warps
#ifndef RODE_SPMM_WIDE_ROWS_WAVES
#define RODE_SPMM_WIDE_ROWS_WAVES 2
#endif

template <typename T, int VB, int L, int VPL, bool kRagged>
__global__ void __launch_bounds__(kRowsCtaThreads, 1024 / kRowsCtaThreads)  // 64 registers: 32 warps per SM
spmm_rows_simple(int m2, int n, const T *__restrict__ values, const int *__restrict__ column_indices,
                 const int *__restrict__ row_offsets, const int *__restrict__ residue_r_ind,
                 const T *__restrict__ B, T *__restrict__ C) {
    using V = typename VecB<T, VB>::type;
    constexpr int kLen = VecB<T, VB>::kLen;
    constexpr int kInFlight = kLoadsInFlight * 16 / VB / VPL;  // dense rows per batch
    constexpr int U = (kInFlight < L) ? kInFlight : L;
    constexpr int kAlign = 4;    // vec_len of the preprocessing
    constexpr int kBlockK = 32;  // k_block of the preprocessing
    const long long item_ll = (static_cast<long long>(blockIdx.x) * kRowsCtaThreads + threadIdx.x) / L;
    if (item_ll >= m2) return;
    const int item = static_cast<int>(item_ll);
    const int lane = threadIdx.x & 31;
    const int l = lane % L;
    const unsigned gmask = group_mask<L>(lane);

    const int row = __ldg(residue_r_ind + item);
    const int begin = __ldg(row_offsets + row);
    const int end = __ldg(row_offsets + row + 1);
    // aligned length >= k_block: a block part exists and its last segment took the tail;
    // no nonzero: the row stays as the caller zero-filled it
    if (end - begin + (begin % kAlign) >= kBlockK || end == begin) return;

    // (this kernel keeps the 64-bit index form of the dense-row address: the 32 x 32 -> 64 bit form of
    // the other kernels measured 2.7 % slower here, stencil N = 64 0.692 -> 0.711 ms)
    const size_t row_vecs = static_cast<size_t>(n) / kLen;
    const size_t col_vec = static_cast<size_t>(blockIdx.y) * L * VPL + l;
    const V *b_lane = reinterpret_cast<const V *>(B) + col_vec;
    auto inside = [&](int v) { return !kRagged || col_vec + v * L < row_vecs; };

    V acc[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) acc[v] = vzero(static_cast<V *>(nullptr));
    // Lane l keeps nonzero l of a chunk of L; the pair is fetched one chunk ahead, so that the
    // fetch overlaps the gathers of the current chunk.
    int c_nxt = 0;
    T v_nxt = T(0);
    if (begin + l < end) {
        c_nxt = ld_stream(column_indices + begin + l);
        v_nxt = ld_stream(values + begin + l);
    }
    // chunk staging in shared memory as in spmm_block (one region of L pairs per lane group; the
    // groups of a warp run rows of different lengths, so they synchronise by group)
    constexpr bool kStage = RODE_SPMM_PAIRS_IN_SMEM != 0 && (L % U == 0) && (U % 4 == 0);
    __shared__ __align__(16) int s_col[2][kStage ? kRowsCtaThreads : 1];
    __shared__ __align__(16) T s_val[2][kStage ? kRowsCtaThreads : 1];
    const int stage_base = (threadIdx.x / L) * L;
    int stage_buf = 0;
    for (int base = begin; base < end; base += L) {
        const int c = c_nxt;
        const T val = v_nxt;
        const int e = base + L + l;
        c_nxt = 0;
        v_nxt = T(0);
        if (e < end) {
            c_nxt = ld_stream(column_indices + e);
            v_nxt = ld_stream(values + e);
        }
        const int cnt = min(L, end - base);
        if constexpr (kStage) {
            s_col[stage_buf][stage_base + l] = c;
            s_val[stage_buf][stage_base + l] = val;
            __syncwarp(gmask);
        }
#pragma unroll
        for (int t0 = 0; t0 < L; t0 += U) {
            if (t0 >= cnt) break;
            int cc[U];
            T vv[U];
            V bb[U][VPL];
            if constexpr (kStage) {
                ld_shared_run<U>(&s_col[stage_buf][stage_base + t0], cc);
                ld_shared_run<U>(&s_val[stage_buf][stage_base + t0], vv);
            } else {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    cc[u] = __shfl_sync(gmask, c, t0 + u, L);
                    vv[u] = __shfl_sync(gmask, val, t0 + u, L);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int v = 0; v < VPL; ++v) {
                    bb[u][v] = vzero(static_cast<V *>(nullptr));
                    if (t0 + u < cnt && inside(v))
                        bb[u][v] = ld_dense(b_lane + static_cast<size_t>(cc[u]) * row_vecs + v * L);
                }
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int v = 0; v < VPL; ++v) vfma(acc[v], vv[u], bb[u][v]);
        }
        stage_buf ^= 1;
    }
#pragma unroll
    for (int v = 0; v < VPL; ++v)
        if (inside(v)) st_stream(reinterpret_cast<V *>(C) + static_cast<size_t>(row) * row_vecs + col_vec + v * L, acc[v]);
}

// ---------------------------------------------------------------------------------------
// The same rows, one WARP per row: for residue lists too short to fill the GPU, where the
// time of the launch is the dependent chain of one row, not throughput.  The 32 lanes fetch
// the row's (fewer than 32) pairs in one coalesced load; the 32 / L lane groups then take
// every (32 / L)-th nonzero each, so that all gathers of the row are in flight at once (L
// per group), and a butterfly over the groups adds the partial rows.  Two dependent memory
// round trips after the row's bounds are known, against up to 32 / L in spmm_rows_simple.
template <typename T, int VB, int L, int VPL, bool kRagged>
__global__ void __launch_bounds__(32 * kSmallGridWarps, 1)
spmm_rows_wide(int m2, int n, const T *__restrict__ values, const int *__restrict__ column_indices,
               const int *__restrict__ row_offsets, const int *__restrict__ residue_r_ind,
               const T *__restrict__ B, T *__restrict__ C) {
    using V = typename VecB<T, VB>::type;
    constexpr int kLen = VecB<T, VB>::kLen;
    constexpr int G = 32 / L;    // lane groups; a group takes at most 32 / G = L nonzeros
    constexpr int kAlign = 4;    // vec_len of the preprocessing
    constexpr int kBlockK = 32;  // k_block of the preprocessing
    constexpr unsigned kFull = 0xffffffffu;
    const int item = blockIdx.x * kSmallGridWarps + (threadIdx.x >> 5);
    if (item >= m2) return;
    const int lane = threadIdx.x & 31;
    const int g = lane / L, l = lane % L;

    const int row = __ldg(residue_r_ind + item);
    const int begin = __ldg(row_offsets + row);
    const int end = __ldg(row_offsets + row + 1);
    if (end - begin + (begin % kAlign) >= kBlockK) return;  // the block part took this row's tail
    const int len = end - begin;                            // < 32
    if (len == 0) return;                                   // stays as the caller zero-filled it

    int c = 0;
    T val = T(0);
    if (lane < len) {
        c = ld_stream(column_indices + begin + lane);
        val = ld_stream(values + begin + lane);
    }
    const size_t row_vecs = static_cast<size_t>(n) / kLen;
    const unsigned row_bytes = static_cast<unsigned>(n) * static_cast<unsigned>(sizeof(T));  // n < 2^21 elements
    const size_t col_vec = static_cast<size_t>(blockIdx.y) * L * VPL + l;
    const V *b_lane = reinterpret_cast<const V *>(B) + col_vec;
    auto inside = [&](int v) { return !kRagged || col_vec + v * L < row_vecs; };

    int cc[L];
    T vv[L];
    V bb[L][VPL];
#pragma unroll
    for (int t = 0; t < L; ++t) {  // nonzero t * G + g
        cc[t] = __shfl_sync(kFull, c, t * G + g);
        vv[t] = __shfl_sync(kFull, val, t * G + g);
    }
#pragma unroll
    for (int t = 0; t < L; ++t)
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
            bb[t][v] = vzero(static_cast<V *>(nullptr));
            if (t * G + g < len && inside(v)) bb[t][v] = ld_dense(dense_row(b_lane, static_cast<unsigned>(cc[t]), row_bytes) + v * L);
        }
    V acc[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
        acc[v] = vzero(static_cast<V *>(nullptr));
#pragma unroll
        for (int t = 0; t < L; ++t) vfma(acc[v], vv[t], bb[t][v]);
#pragma unroll
        for (int d = L; d < 32; d <<= 1) vadd(acc[v], vshfl_xor(kFull, acc[v], d));
    }
    if (g == 0) {
#pragma unroll
        for (int v = 0; v < VPL; ++v)
            if (inside(v)) st_stream(reinterpret_cast<V *>(C) + static_cast<size_t>(row) * row_vecs + col_vec + v * L, acc[v]);
    }
}

template <typename T, int VB, int L, int VPL, bool kRagged>
int launch_rows(int m2, int n, const T *values, const int *col, const int *row_offsets, const int *residue_r_ind,
                const T *B, T *C, int *counters, cudaStream_t s2);

// Block kernel of shape (VB bytes per load, L lanes, VPL loads per lane) and residue-row kernel
// of shape (RVB, RL, RVPL); both cover the same column tile.
template <typename T, int VB, int L, int VPL, int RVB, int RL, int RVPL, bool kRagged>
int launch_shape(int m1, int m2, int k, int n, const T *values, const int *col, const int *row_offsets,
                 const int *block_r_ind, const int *residue_r_ind, const int *st_off, const T *B, T *C,
                 T *partial, int *counters, const unsigned *hot, cudaStream_t s1, cudaStream_t s2) {
    static_assert(L * VPL * VB == RL * RVPL * RVB, "block and residue kernels must cover the same tile");
    constexpr int kTileWidth = L * VPL * VecB<T, VB>::kLen;
    constexpr int U = kLoadsInFlight * 16 / VB / VPL;            // rows per batch, large grids
    constexpr int kChunkSteps = L;                               // nonzeros per group per chunk
    constexpr int kSmallCap = 32 * 16 / VB;                      // small grids: at most 512 bytes per lane in flight
    constexpr int USmall = (kChunkSteps * VPL <= kSmallCap) ? kChunkSteps : kSmallCap / VPL;
    // ragged widths: the last tile is partly empty
    const unsigned tiles = static_cast<unsigned>(kRagged ? (n + kTileWidth - 1) / kTileWidth : n / kTileWidth);
    if (m1 > 0) {
        // Fewer warps than two full waves of 32 per SM: the latency of the longest segment
        // rules, so batches are larger.  CTAs stay one warp: with 4-warp CTAs the Zipf matrix
        // (segments of 32 to 512 nonzeros side by side) ran 0.035 ms instead of 0.029 ms at
        // N = 32 and 0.27 ms instead of 0.06 ms at N = 128.
        const bool small_grid = static_cast<long long>(m1) * tiles <= 2LL * 32 * sm_count();
        // large grids: one resident wave of CTAs whose warps claim segments from counters (one per
        // column tile) at the end of the workspace, zeroed on the stream before the launch
        const int ctas_needed = (m1 + kCtaWarps - 1) / kCtaWarps;
        const int resident = RODE_SPMM_PERSISTENT_CTAS_PER_SM * sm_count();
        // (fp32 only: the fp64 kernels, bound by DRAM on twice the bytes, measured 5 % slower with it)
        const bool persistent = RODE_SPMM_PERSISTENT_CTAS_PER_SM > 0 && sizeof(T) == 4 && !small_grid &&
                                counters != nullptr &&
                                tiles <= kMaxCounterTiles / 2 &&
                                ctas_needed > kPersistentMinWaves * (resident / static_cast<int>(tiles));
        int *claim = nullptr;
        if (persistent) {
            RODE_CUDA_TRY(cudaMemsetAsync(counters, 0, sizeof(int) * tiles, s1));
            claim = counters;
        }
        dim3 grid(persistent ? (resident + tiles - 1) / tiles : ctas_needed, tiles);
        bool launched = false;
        // Popularity hints: block kernel of the 512-byte tile only.  In the residue-row kernel
        // the marks saved DRAM bytes (5.36 -> 4.79 GB on R-MAT scale 23) but the extra registers
        // cost more time than that returned (1.41 -> 1.52 ms).
        if constexpr (L * VPL * VB == 512 && !kRagged) {
            if (hot && !small_grid) {
                spmm_block<T, VB, L, VPL, U, kCtaWarps, true, true, false><<<grid, kCtaThreads, 0, s1>>>(
                    m1, n, values, col, row_offsets, block_r_ind, st_off, B, C, partial, hot, (k + 31) / 32, claim);
                launched = true;
            }
        }
        if (launched) {
        } else if (small_grid && USmall > U) {
            spmm_block<T, VB, L, VPL, USmall, kCtaWarps, false, false, kRagged><<<grid, kCtaThreads, 0, s1>>>(
                m1, n, values, col, row_offsets, block_r_ind, st_off, B, C, partial, nullptr, 0, claim);
        } else {
            spmm_block<T, VB, L, VPL, U, kCtaWarps, false, true, kRagged><<<grid, kCtaThreads, 0, s1>>>(
                m1, n, values, col, row_offsets, block_r_ind, st_off, B, C, partial, nullptr, 0, claim);
        }
        RODE_CHECK_LAUNCH("rode::spmm_block");
        // fix-up as a programmatic dependent of spmm_block: its launch latency and its
        // metadata prologue overlap the tail of the block grid
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((m1 + kFixupThreads - 1) / kFixupThreads);
        cfg.blockDim = dim3(kFixupThreads);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = s1;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const T *partial_in = partial;
        RODE_CUDA_TRY(cudaLaunchKernelEx(&cfg, spmm_fixup<T>, m1, n, row_offsets, block_r_ind, st_off, partial_in,
                                         C));
        RODE_CHECK_LAUNCH("rode::spmm_fixup");
    }
    if (m2 > 0)
        return launch_rows<T, RVB, RL, RVPL, kRagged>(m2, n, values, col, row_offsets, residue_r_ind, B, C, counters, s2);
    return RODE_OK;
}

template <typename T, int VB, int L, int VPL, bool kRagged>
int launch_rows(int m2, int n, const T *values, const int *col, const int *row_offsets, const int *residue_r_ind,
                const T *B, T *C, int *counters, cudaStream_t s2) {
    constexpr int kTileWidth = L * VPL * VecB<T, VB>::kLen;
    const unsigned tiles = static_cast<unsigned>(kRagged ? (n + kTileWidth - 1) / kTileWidth : n / kTileWidth);
    {
        if constexpr (VB == 16 && L == 32 && VPL == 1) {
            // 32 rows per warp when the list is long; fewer (shorter dependent chains, more
            // warps) when the warps would not fill the GPU twice over
            const long long slots = 2LL * 28 * sm_count() * (kCtaThreads / 32);
            int per_group = static_cast<int>((m2 + slots - 1) / slots);
            per_group = per_group < 4 ? 4 : (per_group > 32 ? 32 : per_group);
            const long long groups = (static_cast<long long>(m2) + per_group - 1) / per_group;
            constexpr int kGroupsPerCta = kCtaThreads / 32;
            const long long ctas_needed = (groups + kGroupsPerCta - 1) / kGroupsPerCta;
            const long long resident = static_cast<long long>(RODE_SPMM_PERSISTENT_CTAS_PER_SM) * sm_count();
            const bool persistent = RODE_SPMM_PERSISTENT_ROWS != 0 && sizeof(T) == 4 && counters != nullptr &&
                                    tiles <= kMaxCounterTiles / 2 &&
                                    ctas_needed > kPersistentMinWaves * (resident / tiles);
            int *claim = nullptr;
            if (persistent) {
                claim = counters + kMaxCounterTiles / 2;  // second half: the residue kernel's counters
                RODE_CUDA_TRY(cudaMemsetAsync(claim, 0, sizeof(int) * tiles, s2));
            }
            dim3 grid(static_cast<unsigned>(persistent ? (resident + tiles - 1) / tiles : ctas_needed), tiles);
            spmm_rows<T, 32, kRagged><<<grid, kCtaThreads, 0, s2>>>(m2, per_group, n, values, col, row_offsets,
                                                           residue_r_ind, B, C, claim);
        } else if (static_cast<long long>(m2) * tiles <= RODE_SPMM_WIDE_ROWS_WAVES * 32LL * sm_count()) {
            dim3 grid((m2 + kSmallGridWarps - 1) / kSmallGridWarps, tiles);
            spmm_rows_wide<T, VB, L, VPL, kRagged><<<grid, 32 * kSmallGridWarps, 0, s2>>>(m2, n, values, col, row_offsets,
                                                                                 residue_r_ind, B, C);
        } else {
            constexpr int kRowsPerCta = kRowsCtaThreads / L;
            dim3 grid((m2 + kRowsPerCta - 1) / kRowsPerCta, tiles);
            spmm_rows_simple<T, VB, L, VPL, kRagged><<<grid, kRowsCtaThreads, 0, s2>>>(m2, n, values, col, row_offsets,
                                                                              residue_r_ind, B, C);
        }
        RODE_CHECK_LAUNCH("rode::spmm_rows");
    }
    return RODE_OK;
}

// A shape given in 16-byte vectors (L * 100 + VPL), re-expressed for 32-byte loads: half the
// loads per lane where that number is even, else half the lanes.
constexpr int wide_lanes(int shape) { return (shape % 100) % 2 == 0 ? shape / 100 : shape / 200; }
constexpr int wide_vpl(int shape) { return (shape % 100) % 2 == 0 ? (shape % 100) / 2 : shape % 100; }

template <typename T>
int spmm(int m1, int m2, int k, int n, const T *values, const int *col, const int *row_offsets,
         const int *block_r_ind, const int *residue_r_ind, const int *st_off, const T *B, T *C, void *workspace,
         size_t workspace_bytes, const unsigned *hot, rode_stream_t stream1, rode_stream_t stream2) {
    constexpr int kLen = Vec16<T>::kLen;
    if (m1 < 0 || m2 < 0 || n <= 0) return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: m1, m2 >= 0 and n > 0 required");
    if (hot != nullptr && k <= 0)
        return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: k (the number of columns the bitmap covers) must be positive "
                                               "when hot_columns is given");
    if (n % 4 != 0) return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: n = %d is not a multiple of 4", n);
    if (m1 == 0 && m2 == 0) return RODE_OK;
    if (!values || !col || !row_offsets || !B || !C) return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: null array");
    if (m1 > 0 && (!block_r_ind || !st_off)) return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: null block metadata");
    if (m2 > 0 && !residue_r_ind) return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: null residue metadata");
    if (!aligned_to(B, 16) || !aligned_to(C, 16))
        return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: B and C must be 16-byte aligned");
    if ((n + 8 * kLen - 1) / (8 * kLen) > 65535)
        return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: n = %d exceeds the supported width (%d)", n, 65535 * 8 * kLen);
    size_t need = 0;
    rode_spmm_workspace_bytes(m1, n, static_cast<int>(sizeof(T)), &need);
    // Without block segments the workspace holds the claim counters only and may be left out (the
    // residue kernel then runs one CTA per bundle of rows).
    if (m1 > 0 || workspace != nullptr) {
        if (workspace == nullptr || workspace_bytes < need)
            return fail(RODE_ERR_WORKSPACE, "spmm: workspace of %zu bytes needed, %zu given", need,
                        workspace ? workspace_bytes : static_cast<size_t>(0));
        if (!aligned_to(workspace, 16)) return fail(RODE_ERR_WORKSPACE, "spmm: workspace must be 16-byte aligned");
    }
    T *partial = static_cast<T *>(workspace);
    // the claim counters of the persistent block kernel sit behind the partial rows
    int *counters = workspace != nullptr
                        ? reinterpret_cast<int *>(static_cast<char *>(workspace) + need - kCounterBytes) : nullptr;
    // Widest tile (32, 16 or 8 vectors of 16 bytes) that divides the row.  Shapes are given in
    // 16-byte vectors; with 32-byte loads (operands 32-byte aligned) a group has half the lanes.
    // The batched residue kernel of the widest tile (shape 3201) always loads 16 bytes per lane.
#define RODE_LAUNCH16(shape, rows_shape) RODE_LAUNCH16R(shape, rows_shape, false)
#define RODE_LAUNCH16R(shape, rows_shape, ragged)                                                               \
    launch_shape<T, 16, (shape) / 100, (shape) % 100, 16, (rows_shape) / 100, (rows_shape) % 100, ragged>(      \
        m1, m2, k, n, values, col, row_offsets, block_r_ind, residue_r_ind, st_off, B, C, partial, counters, hot, stream1, \
        stream2)
#define RODE_LAUNCH32(shape, rows_shape, rows_bytes)                                                             \
    launch_shape<T, 32, wide_lanes(shape), wide_vpl(shape), rows_bytes,                                          \
                 (rows_bytes) == 32 ? wide_lanes(rows_shape) : (rows_shape) / 100,                               \
                 (rows_bytes) == 32 ? wide_vpl(rows_shape) : (rows_shape) % 100, false>(                         \
        m1, m2, k, n, values, col, row_offsets, block_r_ind, residue_r_ind, st_off, B, C, partial, counters, hot, stream1, \
        stream2)
    const int vecs = n / kLen;
    // Widths the tiles do not divide (any other multiple of 4 columns; the reference has none of
    // them): the narrowest shape that covers the row, or 512-byte tiles with a partly empty last
    // one.  Always 16-byte loads, no popularity hints.
    if (vecs % 8 != 0) {
        if (vecs < 8) return RODE_LAUNCH16R(RODE_SPMM_SHAPE_8, RODE_SPMM_ROWS_SHAPE_8, true);
        if (vecs < 16) return RODE_LAUNCH16R(RODE_SPMM_SHAPE_16, RODE_SPMM_SHAPE_16, true);
        return RODE_LAUNCH16R(RODE_SPMM_SHAPE_32, RODE_SPMM_ROWS_SHAPE_32, true);
    }
    // 32-byte loads measured no faster than 16-byte ones on any benchmark matrix (the gathers are
    // bound by bytes through L1/L2, not by load instructions), so the default build does not
    // instantiate them.
    if constexpr (RODE_SPMM_VEC_BYTES == 32) {
        if (aligned_to(B, 32) && aligned_to(C, 32) && aligned_to(workspace, 32)) {
            if (vecs % 32 == 0 && RODE_SPMM_MAX_TILE_VECS >= 32) {
                if (RODE_SPMM_ROWS_SHAPE_32 == 3201)
                    return RODE_LAUNCH32(RODE_SPMM_SHAPE_32, RODE_SPMM_ROWS_SHAPE_32, 16);
                return RODE_LAUNCH32(RODE_SPMM_SHAPE_32, RODE_SPMM_ROWS_SHAPE_32, 32);
            }
            if (vecs % 16 == 0) return RODE_LAUNCH32(RODE_SPMM_SHAPE_16, RODE_SPMM_SHAPE_16, 32);
            return RODE_LAUNCH32(RODE_SPMM_SHAPE_8, RODE_SPMM_ROWS_SHAPE_8, 32);
        }
    }
    if (vecs % 32 == 0 && RODE_SPMM_MAX_TILE_VECS >= 32) return RODE_LAUNCH16(RODE_SPMM_SHAPE_32, RODE_SPMM_ROWS_SHAPE_32);
    if (vecs % 16 == 0) return RODE_LAUNCH16(RODE_SPMM_SHAPE_16, RODE_SPMM_SHAPE_16);
    // 128-byte tile: 4 lanes x one 32-byte load cover a whole line per dense row and 8 rows per warp, in
    // the block and the per-row residue kernels alike (operands 32-byte aligned; else the 16-byte shapes)
    if constexpr (RODE_SPMM_TILE8_WIDE_LOADS != 0) {
        if (aligned_to(B, 32) && aligned_to(C, 32) && aligned_to(workspace, 32))
            return launch_shape<T, 32, 4, 1, 32, 4, 1, false>(m1, m2, k, n, values, col, row_offsets, block_r_ind,
                                                              residue_r_ind, st_off, B, C, partial, counters, hot,
                                                              stream1, stream2);
    }
    return RODE_LAUNCH16(RODE_SPMM_SHAPE_8, RODE_SPMM_ROWS_SHAPE_8);
#undef RODE_LAUNCH16
#undef RODE_LAUNCH16R
#undef RODE_LAUNCH32
}

}  // namespace

}  // namespace rode

extern "C" {

int rode_spmm_workspace_bytes(int m1, int n, int elem_size, size_t *bytes) {
    if (bytes == nullptr || m1 < 0 || n < 0 || (elem_size != 4 && elem_size != 8))
        return rode::fail(RODE_ERR_INVALID_ARGUMENT, "spmm_workspace_bytes: bad argument");
    // one partial row per block segment, rounded up to 256 bytes, then the claim counters
    const size_t rows = static_cast<size_t>(m1) * static_cast<size_t>(n) * static_cast<size_t>(elem_size);
    *bytes = (rows + 255) / 256 * 256 + rode::kCounterBytes;
    return RODE_OK;
}

int rode_spmm_f32(int m1, int m2, int k, int n, const float *values, const int *column_indices,
                  const int *row_offsets, const int *block_r_ind, const int *residue_r_ind, const int *st_off,
                  const float *B, float *C, void *workspace, size_t workspace_bytes, rode_stream_t stream1,
                  rode_stream_t stream2) {
    return rode::spmm<float>(m1, m2, k, n, values, column_indices, row_offsets, block_r_ind, residue_r_ind,
                             st_off, B, C, workspace, workspace_bytes, nullptr, stream1, stream2);
}

int rode_spmm_f32_hot(int m1, int m2, int k, int n, const float *values, const int *column_indices,
                      const int *row_offsets, const int *block_r_ind, const int *residue_r_ind, const int *st_off,
                      const float *B, float *C, void *workspace, size_t workspace_bytes,
                      const unsigned *hot_columns, rode_stream_t stream1, rode_stream_t stream2) {
    return rode::spmm<float>(m1, m2, k, n, values, column_indices, row_offsets, block_r_ind, residue_r_ind,
                             st_off, B, C, workspace, workspace_bytes, hot_columns, stream1, stream2);
}

int rode_spmm_f64(int m1, int m2, int k, int n, const double *values, const int *column_indices,
                  const int *row_offsets, const int *block_r_ind, const int *residue_r_ind, const int *st_off,
                  const double *B, double *C, void *workspace, size_t workspace_bytes, rode_stream_t stream1,
                  rode_stream_t stream2) {
    return rode::spmm<double>(m1, m2, k, n, values, column_indices, row_offsets, block_r_ind, residue_r_ind,
                              st_off, B, C, workspace, workspace_bytes, nullptr, stream1, stream2);
}

int rode_spmm_f64_hot(int m1, int m2, int k, int n, const double *values, const int *column_indices,
                      const int *row_offsets, const int *block_r_ind, const int *residue_r_ind, const int *st_off,
                      const double *B, double *C, void *workspace, size_t workspace_bytes,
                      const unsigned *hot_columns, rode_stream_t stream1, rode_stream_t stream2) {
    return rode::spmm<double>(m1, m2, k, n, values, column_indices, row_offsets, block_r_ind, residue_r_ind,
                              st_off, B, C, workspace, workspace_bytes, hot_columns, stream1, stream2);
}

}  // extern "C"
