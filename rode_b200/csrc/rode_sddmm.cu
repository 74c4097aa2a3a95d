// RoDe SDDMM for sm_100a:  out[e] = values[e] * dot(lhs[row(e), :], rhs[col(e), :]).
//
// Stands in for the reference's SDDMMKernel4Block / SDDMMKernel4Residue
// (RoDe_SDDMM/RoDeSddmm.cu:15-203, :206-494) and their launchers (:496-545).  The work
// split follows the reference's metadata (block segments, residue rows); one kernel,
// sddmm_items, serves both lists and every K:
//
//  * A warp takes up to 32 consecutive ITEMS (block segments, or residue rows that have no
//    block part): lane j reads the descriptor of item j, so the dependent chain row index ->
//    row pointer -> column -> dense row is paid once per 32 items.  The nonzeros of the items,
//    concatenated, form one entry stream.  The last segment of a row also covers the row's
//    tail (shorter than 32) that the reference leaves to its residue kernel.
//  * A dense row of length K is covered by a lane group of L lanes, VPL 16-byte loads per
//    lane (K = 4 * L * VPL).  The G = 32/L groups of the warp split the stream into G equal
//    contiguous parts (equal in nonzeros, not in items), so all groups run the same number of
//    iterations and a group walks through its items in order; it keeps the lhs row slice of
//    its current item in registers and prefetches the next item's.
//  * Nonzeros are handled in chunks of L per group (lane l fetches column and value of
//    nonzero l, two chunks ahead) and, inside a chunk, in batches of 8: 8 * VPL independent
//    LDG.128 per lane, one partial dot product per nonzero, then a shuffle reduce that halves
//    the number of live partials at every step (4 + 2 + 1 exchanges, then a butterfly over
//    the remaining lanes).  The finished dot products land in the lanes that hold the
//    matching values, so results are stored coalesced.
//  * Row mode of the residue-row kernel: a warp whose 32 rows hold at least 6 nonzeros on average
//    does not form a stream; its lane groups (8 lanes x 2 loads for K = 64) take the rows one
//    each, neighbouring rows side by side, each row by the plain per-row loop sddmm_one_row.
//    The warp decides from the row lengths it has just loaded (27-point stencil, K = 64:
//    1.26 -> 0.81 ms, rhs rows shared by neighbouring rows now hit in L1; power-law rows,
//    K = 64: 0.51 -> 0.44 ms; graphs with many empty rows keep the stream).
//  * The column indices of a chunk reach the lanes that gather with them through a small
//    double-buffered shared-memory tile (stored once per chunk, read as 16-byte broadcast runs)
//    instead of one shuffle per nonzero: shuffles share the SM's load/store data path with the
//    gathers (block kernel K = 64 on an R-MAT graph 2.29 -> 2.16 ms, power-law residue rows
//    K = 32 0.33 -> 0.26 ms).
//  * sddmm_block: where segments are long (K = 32, 64: up to 543 nonzeros) a segment gets a
//    warp of its own; chunk loads are then plain coalesced loads without any search and the
//    lhs slice never changes (power-law K = 32: 370 us against 744 us through sddmm_items).
//  * One-warp CTAs: a CTA's slot is held until its slowest warp finishes.
//
// Per nonzero: 12 B of CSR data/output plus 4*K bytes of rhs (L1/L2/HBM by reuse); per item
// 4*K bytes of lhs per group that touches it.  No atomics, no workspace in global memory.
#include <climits>
#include <mutex>

#include "rode_common.cuh"

namespace rode {
namespace {

// Shape of a lane group per K: L lanes x VPL 16-byte vectors per lane (K = 4 * L * VPL),
// encoded as L * 100 + VPL.  A batch holds 8 / VPL nonzeros, so a lane always has 8 loads
// in flight.
#ifndef RODE_SDDMM_SHAPE_32
#define RODE_SDDMM_SHAPE_32 801
#endif
#ifndef RODE_SDDMM_SHAPE_64
#define RODE_SDDMM_SHAPE_64 1601
#endif
#ifndef RODE_SDDMM_SHAPE_128
#define RODE_SDDMM_SHAPE_128 3201
#endif
// Shape of a lane group in the row-per-group mode of the residue-row kernel (0 = no such mode),
// and the mean number of nonzeros per row from which a warp uses it.
#ifndef RODE_SDDMM_ROW_SHAPE_32
#define RODE_SDDMM_ROW_SHAPE_32 801
#endif
#ifndef RODE_SDDMM_ROW_SHAPE_64
#define RODE_SDDMM_ROW_SHAPE_64 802
#endif
#ifndef RODE_SDDMM_ROW_SHAPE_128
#define RODE_SDDMM_ROW_SHAPE_128 0
#endif
#ifndef RODE_SDDMM_ROW_MODE_MIN
#define RODE_SDDMM_ROW_MODE_MIN 6
#endif
// 1: the column indices of a chunk reach the lanes of a group through shared memory (stored
// once, read as 16-byte broadcast runs); 0: by one shuffle per nonzero.
#ifndef RODE_SDDMM_COLUMNS_IN_SMEM
#define RODE_SDDMM_COLUMNS_IN_SMEM 1
#endif
// Lane-group sizes L of the stream kernel for which it stages (bit mask: 8 | 16 | 32).
#ifndef RODE_SDDMM_ITEMS_SMEM_MASK
#define RODE_SDDMM_ITEMS_SMEM_MASK (8 | 16 | 32)
#endif
#ifndef RODE_SDDMM_LONG_SEGMENTS_BY_WARP
#define RODE_SDDMM_LONG_SEGMENTS_BY_WARP 1
#endif
constexpr int kLoadsInFlight = 8;  // 16-byte loads per lane per batch
constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ float dot4(const float4 &a, const float4 &b, float acc) {
    return fmaf(a.w, b.w, fmaf(a.z, b.z, fmaf(a.y, b.y, fmaf(a.x, b.x, acc))));
}

// p[u] = this lane's share of the dot product of nonzero u of the batch (u = 0..NB-1).
// Returns the complete dot product of nonzero l / (L / NB) - the same value in the L / NB
// lanes that share those bits.  All L lanes of the group named by gmask take part.
template <int L, int NB>
__device__ __forceinline__ float reduce_batch(float (&p)[NB], int l, unsigned gmask) {
    static_assert(NB <= L, "a batch cannot hold more nonzeros than the group has lanes");
#pragma unroll
    for (int keep = NB / 2, w = L / 2; keep >= 1; keep >>= 1, w >>= 1) {
        const bool upper = (l & w) != 0;
#pragma unroll
        for (int i = 0; i < keep; ++i) {
            const float send = upper ? p[i] : p[i + keep];
            const float mine = upper ? p[i + keep] : p[i];
            p[i] = mine + __shfl_xor_sync(gmask, send, w, L);
        }
    }
    float r = p[0];
#pragma unroll
    for (int w = L / (2 * NB); w >= 1; w >>= 1) r += __shfl_xor_sync(gmask, r, w, L);
    return r;
}

// All nonzeros [begin, end) of ONE row, by the lane group (L lanes x VPL loads per lane) that
// `lane` belongs to; every lane of the group must call with the same row.  Lane l fetches the
// pair of nonzero l of a chunk of L one chunk ahead; batches of kLoadsInFlight loads per lane.
// `stage` = 2 x 32 ints of shared memory owned by this warp (two chunk buffers), `stage_buf` the
// buffer to use next; both are carried from row to row so that a group never stores into a
// buffer that one of its lanes may still read.
template <int L, int VPL, bool kStageAllowed>
__device__ __forceinline__ void sddmm_one_row(int row, int begin, int end, int lane,
                                              const int *__restrict__ column_indices,
                                              const float *__restrict__ values, const float *__restrict__ lhs,
                                              const float *__restrict__ rhs, float *__restrict__ out, int *stage,
                                              int &stage_buf) {
    constexpr int kBatch = (kLoadsInFlight / VPL < L) ? kLoadsInFlight / VPL : L;
    constexpr bool kStage = RODE_SDDMM_COLUMNS_IN_SMEM != 0 && kStageAllowed && (kBatch % 4 == 0);
    constexpr size_t kRowVecs = L * VPL;
    const int l = lane % L;
    const unsigned gmask = group_mask<L>(lane);
    const float4 *rhs_lane = reinterpret_cast<const float4 *>(rhs) + l;
    float4 a[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v)
        a[v] = __ldg(reinterpret_cast<const float4 *>(lhs) + static_cast<size_t>(row) * kRowVecs + v * L + l);
    int c_nxt = 0;
    float v_nxt = 0.f;
    if (begin + l < end) {
        c_nxt = ld_stream(column_indices + begin + l);
        v_nxt = ld_stream(values + begin + l);
    }
    for (int base = begin; base < end; base += L) {
        const int c = c_nxt;
        const float val = v_nxt;
        const int e = base + L + l;
        c_nxt = 0;
        v_nxt = 0.f;
        if (e < end) {
            c_nxt = ld_stream(column_indices + e);
            v_nxt = ld_stream(values + e);
        }
        const int cnt = min(L, end - base);
        float mine = 0.f;
        int *my_stage = stage + stage_buf * 32 + (lane - l);  // this group's region of the buffer
        if constexpr (kStage) {
            my_stage[l] = c;
            __syncwarp(gmask);
            stage_buf ^= 1;
        }
#pragma unroll
        for (int b = 0; b < L / kBatch; ++b) {
            if (b * kBatch < cnt) {  // uniform inside the group
                float4 bb[kBatch][VPL];
                int cc[kBatch];
                if constexpr (kStage) ld_shared_run<kBatch>(my_stage + b * kBatch, cc);
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const int t = b * kBatch + u;
                    if constexpr (!kStage) cc[u] = __shfl_sync(gmask, c, t, L);
#pragma unroll
                    for (int v = 0; v < VPL; ++v) {
                        bb[u][v] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (t < cnt) bb[u][v] = ld_dense(rhs_lane + static_cast<size_t>(cc[u]) * kRowVecs + v * L);
                    }
                }
                float p[kBatch];
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    float d = 0.f;
#pragma unroll
                    for (int v = 0; v < VPL; ++v) d = dot4(a[v], bb[u][v], d);
                    p[u] = d;
                }
                const float r = reduce_batch<L, kBatch>(p, l, gmask);
                const float got = (L == kBatch) ? r : __shfl_sync(gmask, r, (l & (kBatch - 1)) * (L / kBatch), L);
                if ((l / kBatch) == b) mine = got;
            }
        }
        if (base + l < end) st_stream(out + base + l, val * mine);
    }
}

// kSegments: items are block segments (block_r_ind / st_off); otherwise residue rows
// (residue_r_ind) without a block part.
//
// kRagged: the dense rows hold row_vecs_arg <= L * VPL vectors (any K that is a multiple of 4
// up to 4 * L * VPL); vectors beyond the row's end are not loaded and count as zeros.
//
// LB > 0 (residue rows only): a warp whose rows hold at least row_mode_min nonzeros on average
// does not form a stream; its 32 / LB lane groups (LB lanes x VPLB loads) take the rows one
// each, neighbouring rows side by side.  Long residue rows need no balancing over the groups,
// and rows that share columns (stencils, meshes) then find each other's rhs rows in L1; short
// and empty rows (graphs) are better served by the stream, which splits the warp's nonzeros
// evenly.  The warp decides from the row lengths it has just loaded, so no statistic of the
// matrix has to be passed in.
// One-warp CTAs per SM the register allocation must allow: 28 (72 registers).  Left to itself the
// compiler takes 78-80 registers for K = 64 once the chunk staging is in, and the four warps per
// SM that costs outweigh what the staging gains; 64 registers (32 CTAs) spill.
#ifndef RODE_SDDMM_ITEMS_MIN_CTAS
#define RODE_SDDMM_ITEMS_MIN_CTAS 28
#endif
template <int L, int VPL, bool kSegments, bool kRagged = false, int LB = 0, int VPLB = 1>
__global__ void __launch_bounds__(32, kRagged ? 24 : RODE_SDDMM_ITEMS_MIN_CTAS)
sddmm_items(int n_items, int items_per_warp, const int *__restrict__ item_rows, const int *__restrict__ st_off,
            const int *__restrict__ row_offsets, const int *__restrict__ column_indices,
            const float *__restrict__ values, const float *__restrict__ lhs, const float *__restrict__ rhs,
            float *__restrict__ out, int row_vecs_arg, int row_mode_min) {
    constexpr int G = 32 / L;
    constexpr int kBatch = kLoadsInFlight / VPL;  // nonzeros per batch
    const size_t kRowVecs = kRagged ? static_cast<size_t>(row_vecs_arg) : L * VPL;  // float4 per dense row (K / 4)
    constexpr int kAlign = 4;             // vec_len of the preprocessing
    constexpr int kBlockK = 32;           // k_block of the preprocessing
    __shared__ int s_end[32];             // stream position where item j ends
    __shared__ int s_row[32];             // row of item j
    __shared__ __align__(16) int s_col[2][32];  // column indices of the current chunk, two buffers
    int stage_buf = 0;
    const int lane = threadIdx.x;
    const int g = lane / L, l = lane % L;
    const unsigned gmask = group_mask<L>(lane);
    const long long item0 = static_cast<long long>(blockIdx.x) * items_per_warp;
    if (item0 >= n_items) return;

    // ---- descriptors: lane j owns item item0 + j --------------------------------------------
    int row = 0, begin = 0, len = 0;
    if (lane < items_per_warp && item0 + lane < n_items) {
        const int item = static_cast<int>(item0) + lane;
        row = __ldg(item_rows + item);
        if (kSegments) {
            begin = __ldg(st_off + item);
            const int next = (item + 1 < n_items) ? __ldg(st_off + item + 1) : INT_MAX;
            len = min(__ldg(row_offsets + row + 1), next) - begin;
        } else {
            begin = __ldg(row_offsets + row);
            const int end = __ldg(row_offsets + row + 1);
            if (end - begin + (begin % kAlign) < kBlockK) len = end - begin;
        }
    }
    int start = len;  // exclusive prefix sum of len
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(kFull, start, d);
        if (lane >= d) start += up;
    }
    const int total = __shfl_sync(kFull, start, 31);
    s_end[lane] = start;  // inclusive sum = end position
    s_row[lane] = row;
    start -= len;
    const unsigned nonempty = __ballot_sync(kFull, len > 0);
    if (total == 0) return;
    if constexpr (LB > 0 && !kSegments && !kRagged) {
        static_assert(LB * VPLB == L * VPL, "both lane-group shapes must cover the same dense row");
        // (full warps of 32 rows only: short lists give a warp fewer rows than it has groups, and
        // there the stream's even split of the nonzeros is what shortens the dependent chain)
        if (items_per_warp == 32 && total >= row_mode_min * 32) {  // warp-uniform
            constexpr int GB = 32 / LB;
            const int gb = lane / LB;
            for (int j0 = 0; j0 < items_per_warp; j0 += GB) {
                const int j = j0 + gb;  // items_per_warp <= 32, a multiple of GB or the tail is empty
                const int r = __shfl_sync(kFull, row, j & 31);
                const int b0 = __shfl_sync(kFull, begin, j & 31);
                const int n0 = __shfl_sync(kFull, len, j & 31);
                if (j < items_per_warp && n0 > 0)
                    sddmm_one_row<LB, VPLB, ((RODE_SDDMM_ITEMS_SMEM_MASK) & L) != 0>(r, b0, b0 + n0, lane, column_indices, values, lhs, rhs, out, &s_col[0][0],
                                            stage_buf);
            }
            return;
        }
    }
    __syncwarp();

    // ---- this group's contiguous part of the stream: [p0, p1) ----------------------------------
    const int per = (((total + G - 1) / G) + kBatch - 1) & ~(kBatch - 1);
    const int p0 = g * per;
    const int p1 = min(p0 + per, total);
    const int n_chunks = (per + L - 1) / L;  // same for every group

    // stream position p -> (nonzero index, column, value); every lane of the warp calls
    auto fetch = [&](int p, int &e, int &c, float &v) {
        int lo = 0;
#pragma unroll
        for (int step = 16; step >= 1; step >>= 1) {
            const int s = __shfl_sync(kFull, start, lo + step);
            if (s <= p) lo += step;
        }
        const int b0 = __shfl_sync(kFull, begin, lo);
        const int s0 = __shfl_sync(kFull, start, lo);
        e = -1;
        c = 0;
        v = 0.f;
        if (p < p1) {
            e = b0 + (p - s0);
            c = ld_stream(column_indices + e);
            v = ld_stream(values + e);
        }
    };

    const float4 *lhs_lane = reinterpret_cast<const float4 *>(lhs) + l;
    const float4 *rhs_lane = reinterpret_cast<const float4 *>(rhs) + l;
    // vector v of this lane lies inside the dense row
    auto inside = [&](int v) { return !kRagged || static_cast<size_t>(l + v * L) < kRowVecs; };
    auto load_lhs = [&](int item, int v) {
        return inside(v) ? __ldg(lhs_lane + static_cast<size_t>(s_row[item]) * kRowVecs + v * L)
                         : make_float4(0.f, 0.f, 0.f, 0.f);
    };

    // ---- item the group is in, its lhs slice, and the next item's (prefetched) --------------------
    // first item whose end lies beyond p0 = number of items that end at or before p0
    int cur = 0;
#pragma unroll
    for (int gg = 0; gg < G; ++gg) {
        const int cnt = __popc(__ballot_sync(kFull, s_end[lane] <= gg * per));
        if (g == gg) cur = cnt;
    }
    cur = min(cur, 31);
    auto next_nonempty = [&](int after) {  // first non-empty item with index > after, or -1
        const unsigned rest = (after >= 31) ? 0u : (nonempty & (kFull << (after + 1)));
        return __ffs(rest) - 1;
    };
    int cur_end = s_end[cur];
    int nxt = next_nonempty(cur);
    float4 a_cur[VPL], a_nxt[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
        a_cur[v] = load_lhs(cur, v);
        a_nxt[v] = a_cur[v];
        if (nxt >= 0) a_nxt[v] = load_lhs(nxt, v);
    }

    int e_cur, c_cur, e_nxt, c_nxt;
    float v_cur, v_nxt;
    fetch(p0 + l, e_cur, c_cur, v_cur);
    fetch(p0 + L + l, e_nxt, c_nxt, v_nxt);
    int pos = p0;  // stream position of the next nonzero this group multiplies
    for (int ch = 0; ch < n_chunks; ++ch) {
        int e_pre, c_pre;
        float v_pre;
        fetch(p0 + (ch + 2) * L + l, e_pre, c_pre, v_pre);
        const int cnt = min(L, p1 - (p0 + ch * L));  // valid nonzeros of this chunk (may be <= 0)
        float mine = 0.f;
        constexpr bool kStage = RODE_SDDMM_COLUMNS_IN_SMEM != 0 && ((RODE_SDDMM_ITEMS_SMEM_MASK) & L) != 0 && (kBatch % 4 == 0);
        int *my_stage = &s_col[stage_buf][lane - l];  // this group's region of the chunk buffer
        if constexpr (kStage) {
            my_stage[l] = c_cur;
            __syncwarp();  // every group runs the same number of chunks
            stage_buf ^= 1;
        }
#pragma unroll
        for (int b = 0; b < L / kBatch; ++b) {
            if (b * kBatch < cnt) {  // uniform inside the group; no warp-wide shuffles inside
                float4 bb[kBatch][VPL];
                int cc[kBatch];
                if constexpr (kStage) ld_shared_run<kBatch>(my_stage + b * kBatch, cc);
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const int t = b * kBatch + u;
                    if constexpr (!kStage) cc[u] = __shfl_sync(gmask, c_cur, t, L);
#pragma unroll
                    for (int v = 0; v < VPL; ++v) {
                        bb[u][v] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (t < cnt && inside(v))
                            bb[u][v] = ld_dense(rhs_lane + static_cast<size_t>(cc[u]) * kRowVecs + v * L);
                    }
                }
                float p[kBatch];
                if (cur_end - pos >= kBatch) {  // the whole batch lies inside the current item
#pragma unroll
                    for (int u = 0; u < kBatch; ++u) {
                        float d = 0.f;
#pragma unroll
                        for (int v = 0; v < VPL; ++v) d = dot4(a_cur[v], bb[u][v], d);
                        p[u] = d;
                    }
                    pos += kBatch;
                } else {
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    if (pos == cur_end && nxt >= 0) {  // the group enters its next item
                        cur = nxt;
                        cur_end = s_end[cur];
                        nxt = next_nonempty(cur);
#pragma unroll
                        for (int v = 0; v < VPL; ++v) {
                            a_cur[v] = a_nxt[v];
                            if (nxt >= 0) a_nxt[v] = load_lhs(nxt, v);
                        }
                    }
                    float d = 0.f;
#pragma unroll
                    for (int v = 0; v < VPL; ++v) d = dot4(a_cur[v], bb[u][v], d);
                    p[u] = d;
                    ++pos;
                }
                }
                const float r = reduce_batch<L, kBatch>(p, l, gmask);
                // nonzero u of the batch sits in lanes u * (L / kBatch) ..; lane b * kBatch + u wants it
                const float got = (L == kBatch) ? r : __shfl_sync(gmask, r, (l & (kBatch - 1)) * (L / kBatch), L);
                if ((l / kBatch) == b) mine = got;
            }
        }
        if (e_cur >= 0) st_stream(out + e_cur, v_cur * mine);
        e_cur = e_nxt;
        c_cur = c_nxt;
        v_cur = v_nxt;
        e_nxt = e_pre;
        c_nxt = c_pre;
        v_nxt = v_pre;
    }
}

// ---------------------------------------------------------------------------------------
// One warp per block segment (used where segments are long, K = 32 and 64: up to 543
// nonzeros): coalesced chunk loads without any search, the G groups take consecutive
// L-nonzero pieces of each 32-nonzero chunk, the lhs slice stays in registers.
//
// kClaim (grids of one resident wave): a warp starts with the segment of its own index and
// claims further ones from *next_segment; the claim is issued before the segment's work and
// read after it.  One-warp CTAs of one segment each live a few microseconds, and a fifth of the
// warp slots stood empty waiting for the next CTA to be launched into them.
template <int L, int VPL, bool kClaim>
__global__ void __launch_bounds__(32, 32)  // 64 registers: 32 one-warp CTAs per SM
sddmm_block(int m1, const int *__restrict__ block_r_ind, const int *__restrict__ st_off,
            const int *__restrict__ row_offsets, const int *__restrict__ column_indices,
            const float *__restrict__ values, const float *__restrict__ lhs, const float *__restrict__ rhs,
            float *__restrict__ out, int *__restrict__ next_segment) {
    constexpr int kBatch = kLoadsInFlight / VPL;
    constexpr size_t kRowVecs = L * VPL;
    constexpr bool kStage = RODE_SDDMM_COLUMNS_IN_SMEM != 0 && (kBatch % 4 == 0);
    __shared__ __align__(16) int s_col[2][32];  // column indices of the current chunk, two buffers
    int stage_buf = 0;
    const int lane = threadIdx.x;
    const int l = lane % L;
    const int gbase = lane - l;  // first lane (= first nonzero of the chunk) of this group
    const unsigned gmask = group_mask<L>(lane);
    int seg = blockIdx.x;
    while (seg < m1) {
    int claimed = INT_MAX;  // never used in arithmetic: the loop test compares it with m1 as it is
    if constexpr (kClaim) {
        if (lane == 0) claimed = static_cast<int>(gridDim.x) + atomicAdd(next_segment, 1);
    }

    const int row = __ldg(block_r_ind + seg);
    const int off = __ldg(st_off + seg);
    const int next = (seg + 1 < m1) ? __ldg(st_off + seg + 1) : INT_MAX;
    const int end = min(__ldg(row_offsets + row + 1), next);

    const float4 *rhs_lane = reinterpret_cast<const float4 *>(rhs) + l;
    float4 a[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v)
        a[v] = __ldg(reinterpret_cast<const float4 *>(lhs) + static_cast<size_t>(row) * kRowVecs + v * L + l);

    int c_cur = 0, c_nxt = 0;
    float v_cur = 0.f, v_nxt = 0.f;
    if (off + lane < end) {
        c_cur = ld_stream(column_indices + off + lane);
        v_cur = ld_stream(values + off + lane);
    }
    if (off + 32 + lane < end) {
        c_nxt = ld_stream(column_indices + off + 32 + lane);
        v_nxt = ld_stream(values + off + 32 + lane);
    }
    for (int base = off; base < end; base += 32) {
        int c_pre = 0;
        float v_pre = 0.f;
        if (base + 64 + lane < end) {  // pairs of the chunk after next
            c_pre = ld_stream(column_indices + base + 64 + lane);
            v_pre = ld_stream(values + base + 64 + lane);
        }
        const int cnt = min(32, end - base);
        float mine = 0.f;
        if constexpr (kStage) {
            s_col[stage_buf][lane] = c_cur;
            __syncwarp();
        }
#pragma unroll
        for (int b = 0; b < L / kBatch; ++b) {
            if (gbase + b * kBatch < cnt) {  // uniform inside the group
                float4 bb[kBatch][VPL];
                int cc[kBatch];
                if constexpr (kStage) ld_shared_run<kBatch>(&s_col[stage_buf][gbase + b * kBatch], cc);
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    const int t = b * kBatch + u;  // nonzero inside the group's part of the chunk
                    if constexpr (!kStage) cc[u] = __shfl_sync(gmask, c_cur, t, L);
#pragma unroll
                    for (int v = 0; v < VPL; ++v) {
                        bb[u][v] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (gbase + t < cnt)
                            bb[u][v] = ld_dense(rhs_lane + static_cast<size_t>(cc[u]) * kRowVecs + v * L);
                    }
                }
                float p[kBatch];
#pragma unroll
                for (int u = 0; u < kBatch; ++u) {
                    float d = 0.f;
#pragma unroll
                    for (int v = 0; v < VPL; ++v) d = dot4(a[v], bb[u][v], d);
                    p[u] = d;
                }
                const float r = reduce_batch<L, kBatch>(p, l, gmask);
                const float got = (L == kBatch) ? r : __shfl_sync(gmask, r, (l & (kBatch - 1)) * (L / kBatch), L);
                if ((l / kBatch) == b) mine = got;
            }
        }
        if (base + lane < end) st_stream(out + base + lane, v_cur * mine);
        c_cur = c_nxt;
        v_cur = v_nxt;
        c_nxt = c_pre;
        v_nxt = v_pre;
        stage_buf ^= 1;
    }
    seg = kClaim ? __shfl_sync(kFull, claimed, 0) : INT_MAX;
    }  // segments of this warp
}

// ---------------------------------------------------------------------------------------
// Claim counter of the persistent block grid.  The SDDMM entry points carry no workspace, so the
// counters live in a fixed array of the library's device image: kClaimSlots slots of 64 ints
// (32 KB on every GPU that loads the library).  A slot belongs to one (device, stream1, stream2)
// for the life of the process: calls on the same streams are ordered by them and may share
// their counter, calls on other streams get other slots; when all slots are taken a call simply
// runs one CTA per segment.  Nothing is allocated.  (Two host threads that enqueue calls on the
// SAME pair of streams at the same time could interleave one call's counter reset with the
// other's kernel; like the reference, the entry points expect one enqueueing thread per stream.)
#ifndef RODE_SDDMM_PERSISTENT
#define RODE_SDDMM_PERSISTENT 1
#endif
constexpr int kClaimSlots = 128;
constexpr int kClaimInts = 64;
static __device__ __align__(256) int g_claim_counters[kClaimSlots * kClaimInts];

int claim_counters(cudaStream_t s1, cudaStream_t s2, int **out) {
    struct Key {
        int dev;
        cudaStream_t s1, s2;
    };
    static Key keys[kClaimSlots];
    static int n_keys = 0;
    static int *base[64] = {nullptr};  // device address of the array, per device
    static std::mutex lock;
    *out = nullptr;
    int dev = 0;
    RODE_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return RODE_OK;
    std::lock_guard<std::mutex> guard(lock);
    if (base[dev] == nullptr) {
        void *p = nullptr;
        RODE_CUDA_TRY(cudaGetSymbolAddress(&p, g_claim_counters));
        base[dev] = static_cast<int *>(p);
    }
    int slot = -1;
    for (int i = 0; i < n_keys; ++i)
        if (keys[i].dev == dev && keys[i].s1 == s1 && keys[i].s2 == s2) slot = i;
    if (slot < 0 && n_keys < kClaimSlots) {
        slot = n_keys++;
        keys[slot] = {dev, s1, s2};
    }
    if (slot >= 0) *out = base[dev] + slot * kClaimInts;
    return RODE_OK;
}

// Items per warp: 32 when that still gives every SM several waves of warps, fewer otherwise.
int items_per_warp(int n_items, int cap) {
    const long long slots = 4LL * 24 * sm_count();
    long long per = (n_items + slots - 1) / slots;
    per = per < 1 ? 1 : (per > cap ? cap : per);
    return static_cast<int>(per);
}

template <int L, int VPL, int RL, int RVPL>
int launch_k(int m1, int m2, int seg_cap, const int *block_r_ind, const int *residue_r_ind, const int *st_off,
             const int *row_offsets, const int *col, const float *values, const float *lhs, const float *rhs,
             float *out, cudaStream_t s1, cudaStream_t s2) {
    if (m1 > 0) {
        if (seg_cap < 32 && RODE_SDDMM_LONG_SEGMENTS_BY_WARP) {
            const int resident = 32 * sm_count();
            int *claim = nullptr;
            if (RODE_SDDMM_PERSISTENT && m1 > 16 * resident) {  // from about 16 segments per warp on it pays
                if (int rc = claim_counters(s1, s2, &claim)) return rc;
            }
            if (claim != nullptr) {
                RODE_CUDA_TRY(cudaMemsetAsync(claim, 0, sizeof(int), s1));
                sddmm_block<L, VPL, true><<<resident, 32, 0, s1>>>(m1, block_r_ind, st_off, row_offsets, col, values, lhs,
                                                                   rhs, out, claim);
            } else {
                sddmm_block<L, VPL, false><<<m1, 32, 0, s1>>>(m1, block_r_ind, st_off, row_offsets, col, values, lhs, rhs,
                                                              out, nullptr);
            }
            RODE_CHECK_LAUNCH("rode::sddmm_block");
        } else {
            const int per = items_per_warp(m1, seg_cap);
            sddmm_items<L, VPL, true><<<(m1 + per - 1) / per, 32, 0, s1>>>(m1, per, block_r_ind, st_off, row_offsets,
                                                                            col, values, lhs, rhs, out, L * VPL, 0);
            RODE_CHECK_LAUNCH("rode::sddmm_items<segments>");
        }
    }
    if (m2 > 0) {
        const int per = items_per_warp(m2, 32);
        sddmm_items<L, VPL, false, false, RL, RVPL><<<(m2 + per - 1) / per, 32, 0, s2>>>(
            m2, per, residue_r_ind, nullptr, row_offsets, col, values, lhs, rhs, out, L * VPL,
            RODE_SDDMM_ROW_MODE_MIN);
        RODE_CHECK_LAUNCH("rode::sddmm_items<rows>");
    }
    return RODE_OK;
}

// Any other K that is a multiple of 4, up to 256: 32 lanes x 2 vectors per lane, vectors beyond
// the row's end masked.  Both item lists run through sddmm_items (a few segments per warp when
// segments are long).
int launch_ragged(int m1, int m2, int k, const int *block_r_ind, const int *residue_r_ind, const int *st_off,
                  const int *row_offsets, const int *col, const float *values, const float *lhs, const float *rhs,
                  float *out, cudaStream_t s1, cudaStream_t s2) {
    const int row_vecs = k / 4;
    if (m1 > 0) {
        const int per = items_per_warp(m1, 4);
        sddmm_items<32, 2, true, true><<<(m1 + per - 1) / per, 32, 0, s1>>>(m1, per, block_r_ind, st_off, row_offsets,
                                                                             col, values, lhs, rhs, out, row_vecs, 0);
        RODE_CHECK_LAUNCH("rode::sddmm_items<segments, any k>");
    }
    if (m2 > 0) {
        const int per = items_per_warp(m2, 32);
        sddmm_items<32, 2, false, true><<<(m2 + per - 1) / per, 32, 0, s2>>>(m2, per, residue_r_ind, nullptr,
                                                                              row_offsets, col, values, lhs, rhs, out,
                                                                              row_vecs, 0);
        RODE_CHECK_LAUNCH("rode::sddmm_items<rows, any k>");
    }
    return RODE_OK;
}

}  // namespace
}  // namespace rode

extern "C" int rode_sddmm_f32(int m1, int m2, int n, int k, const int *block_r_ind, const int *residue_r_ind,
                              const int *st_off, const int *row_offsets, const int *column_indices,
                              const float *values, const float *lhs, const float *rhs, float *out,
                              rode_stream_t stream1, rode_stream_t stream2) {
    using namespace rode;
    (void)n;
    if (m1 < 0 || m2 < 0) return fail(RODE_ERR_INVALID_ARGUMENT, "sddmm: m1, m2 must be >= 0");
    if (k <= 0 || k % 4 != 0 || k > 256)
        return fail(RODE_ERR_INVALID_ARGUMENT, "sddmm: k = %d unsupported (a multiple of 4, at most 256)", k);
    if (m1 == 0 && m2 == 0) return RODE_OK;
    if (!row_offsets || !column_indices || !values || !lhs || !rhs || !out)
        return fail(RODE_ERR_INVALID_ARGUMENT, "sddmm: null array");
    if (m1 > 0 && (!block_r_ind || !st_off)) return fail(RODE_ERR_INVALID_ARGUMENT, "sddmm: null block metadata");
    if (m2 > 0 && !residue_r_ind) return fail(RODE_ERR_INVALID_ARGUMENT, "sddmm: null residue metadata");
    if (!aligned_to(lhs, 16) || !aligned_to(rhs, 16))
        return fail(RODE_ERR_INVALID_ARGUMENT, "sddmm: lhs and rhs must be 16-byte aligned");
    switch (k) {
        // segments per warp in sddmm_items: few when segments are long (512), 32 when short
        case 32:
            return launch_k<RODE_SDDMM_SHAPE_32 / 100, RODE_SDDMM_SHAPE_32 % 100, RODE_SDDMM_ROW_SHAPE_32 / 100,
                            RODE_SDDMM_ROW_SHAPE_32 % 100>(
                m1, m2, 4, block_r_ind, residue_r_ind, st_off, row_offsets, column_indices, values, lhs, rhs, out,
                stream1, stream2);
        case 64:
            return launch_k<RODE_SDDMM_SHAPE_64 / 100, RODE_SDDMM_SHAPE_64 % 100, RODE_SDDMM_ROW_SHAPE_64 / 100,
                            RODE_SDDMM_ROW_SHAPE_64 % 100>(
                m1, m2, 4, block_r_ind, residue_r_ind, st_off, row_offsets, column_indices, values, lhs, rhs, out,
                stream1, stream2);
        case 128:
            return launch_k<RODE_SDDMM_SHAPE_128 / 100, RODE_SDDMM_SHAPE_128 % 100, RODE_SDDMM_ROW_SHAPE_128 / 100,
                            RODE_SDDMM_ROW_SHAPE_128 == 0 ? 1 : RODE_SDDMM_ROW_SHAPE_128 % 100>(
                m1, m2, 32, block_r_ind, residue_r_ind, st_off, row_offsets, column_indices, values, lhs, rhs, out,
                stream1, stream2);
        default:
            return launch_ragged(m1, m2, k, block_r_ind, residue_r_ind, st_off, row_offsets, column_indices, values,
                                 lhs, rhs, out, stream1, stream2);
    }
}
