// RoDe SDDMM for sm_100a:  out[e] = values[e] * dot(lhs[row(e), :], rhs[col(e), :]).
//
// Stands in for the reference's SDDMMKernel4Block / SDDMMKernel4Residue
// (RoDe_SDDMM/RoDeSddmm.cu:15-203, :206-494) and their launchers (:496-545).  The work
// split follows the reference's metadata (block segments, residue rows); inside a unit:
//
//  * A dense row of length K is covered by L = K/4 lanes, one LDG.128 per lane, so a gather
//    of rhs[col, :] is one coalesced request of 4*K bytes.  K = 32, 64, 128 -> L = 8, 16, 32;
//    a warp holds G = 32/L lane groups.
//  * Nonzeros are handled in chunks of 32 (lane t fetches column and value of nonzero t,
//    two chunks ahead) and, inside a chunk, in batches of 8 per lane group: 8 independent
//    LDG.128 per lane, one partial dot product (this lane's 4 of the K terms) per nonzero,
//    then a shuffle reduce that halves the number of live partials at every step
//    (4 + 2 + 1 exchanges, then a butterfly over the remaining lanes): ~1.2 shuffles per
//    nonzero and only 8 partials in registers.  The finished dot products are handed to
//    the lanes that hold the matching values, so results are stored coalesced.
//  * sddmm_block (K = 32, 64; segments of up to 512 nonzeros): one warp per block segment;
//    the lhs row slice stays in registers.  The last segment of a row also produces the
//    row's tail (shorter than 32) that the reference leaves to its residue kernel.
//    sddmm_rows (K = 32, 64): one lane group per residue row without a block part.
//  * sddmm_stream (K = 128, where segments are only 32 long): a warp takes 32 consecutive
//    items (segments, or residue rows without a block part): lane j reads the descriptor of
//    item j, and the nonzeros of the 32 items run through the gather as one stream, the
//    lhs row being switched (and the next one prefetched) where the stream crosses into the
//    next item.  The dependent chain row index -> row pointer -> column -> dense row is
//    paid once per 32 items.
//  * CTAs are one or two warps: a CTA's slot is held until its slowest warp finishes.
//
// Per nonzero: 12 B of CSR data/output plus 4*K bytes of rhs (L1/L2/HBM by reuse); per item
// 4*K bytes of lhs.  No shared memory, no atomics, no workspace.
#include <climits>

#include "rode_common.cuh"

namespace rode {
namespace {

#ifndef RODE_SDDMM_CTA_WARPS
#define RODE_SDDMM_CTA_WARPS 1
#endif
#ifndef RODE_SDDMM_ROWS_CTA
#define RODE_SDDMM_ROWS_CTA 64
#endif
constexpr int kCtaWarps = RODE_SDDMM_CTA_WARPS;
constexpr int kCtaThreads = 32 * kCtaWarps;
constexpr int kRowsCtaThreads = RODE_SDDMM_ROWS_CTA;
constexpr int kBatch = 8;  // nonzeros per lane group per batch = LDG.128 in flight per lane
constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ float dot4(const float4 &a, const float4 &b) {
    return fmaf(a.w, b.w, fmaf(a.z, b.z, fmaf(a.y, b.y, a.x * b.x)));
}

// p[u] = this lane's share of the dot product of nonzero u of the batch (u = 0..7).
// Returns the complete dot product of nonzero ((l / (L/8)) & 7) - the same value in the
// L/8 lanes that share those bits.  All L lanes of the group named by gmask take part.
template <int L>
__device__ __forceinline__ float reduce_batch(float (&p)[kBatch], int l, unsigned gmask) {
#pragma unroll
    for (int keep = kBatch / 2, w = L / 2; keep >= 1; keep >>= 1, w >>= 1) {
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
    for (int w = L / 16; w >= 1; w >>= 1) r += __shfl_xor_sync(gmask, r, w, L);
    return r;
}

// Dot products of one chunk.  Lane t of the warp holds column `c` of nonzero t; `cnt`
// nonzeros of the chunk are valid.  Group g handles nonzeros g*L .. g*L+L-1 with the lhs
// slice `a`.  Returns, in lane t, the dot product of nonzero t.
template <int L>
__device__ __forceinline__ float chunk_dots(const float4 &a, int c, int cnt, const float4 *__restrict__ rhs_lane,
                                            size_t row_vecs, int lane) {
    const int l = lane % L;
    const int gbase = lane - l;  // first lane (= first nonzero) of this group
    const unsigned gmask = group_mask<L>(lane);
    float mine = 0.f;
#pragma unroll
    for (int b = 0; b < L / kBatch; ++b) {
        if (gbase + b * kBatch >= cnt) break;  // uniform inside the group
        float4 bb[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const int t = b * kBatch + u;  // nonzero inside the group's part of the chunk
            const int cc = __shfl_sync(gmask, c, t, L);
            bb[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (gbase + t < cnt) bb[u] = ld_dense(rhs_lane + static_cast<size_t>(cc) * row_vecs);
        }
        float p[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) p[u] = dot4(a, bb[u]);
        const float r = reduce_batch<L>(p, l, gmask);
        // nonzero u of the batch sits in lanes u * (L/8) ..; lane b*8 + u of the group wants it
        const float got = __shfl_sync(gmask, r, (l & (kBatch - 1)) * (L / kBatch), L);
        if ((l / kBatch) == b) mine = got;
    }
    return mine;
}

// ---------------------------------------------------------------------------------------
template <int L>
__global__ void __launch_bounds__(kCtaThreads)
sddmm_block(int m1, int k, const int *__restrict__ block_r_ind, const int *__restrict__ st_off,
            const int *__restrict__ row_offsets, const int *__restrict__ column_indices,
            const float *__restrict__ values, const float *__restrict__ lhs, const float *__restrict__ rhs,
            float *__restrict__ out) {
    const int seg = blockIdx.x * kCtaWarps + (threadIdx.x >> 5);
    if (seg >= m1) return;
    const int lane = threadIdx.x & 31;
    const int l = lane % L;

    const int row = __ldg(block_r_ind + seg);
    const int off = __ldg(st_off + seg);
    const int next = (seg + 1 < m1) ? __ldg(st_off + seg + 1) : INT_MAX;
    const int end = min(__ldg(row_offsets + row + 1), next);

    const size_t row_vecs = static_cast<size_t>(k) / 4;
    const float4 a = __ldg(reinterpret_cast<const float4 *>(lhs) + static_cast<size_t>(row) * row_vecs + l);
    const float4 *rhs_lane = reinterpret_cast<const float4 *>(rhs) + l;

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
        const float d = chunk_dots<L>(a, c_cur, min(32, end - base), rhs_lane, row_vecs, lane);
        if (base + lane < end) st_stream(out + base + lane, v_cur * d);
        c_cur = c_nxt;
        v_cur = v_nxt;
        c_nxt = c_pre;
        v_nxt = v_pre;
    }
}

// One lane group per residue row without a block part.
template <int L>
__global__ void __launch_bounds__(kRowsCtaThreads)
sddmm_rows(int m2, int k, const int *__restrict__ residue_r_ind, const int *__restrict__ row_offsets,
           const int *__restrict__ column_indices, const float *__restrict__ values,
           const float *__restrict__ lhs, const float *__restrict__ rhs, float *__restrict__ out) {
    constexpr int kAlign = 4;    // vec_len of the preprocessing
    constexpr int kBlockK = 32;  // k_block of the preprocessing
    const int item = (blockIdx.x * kRowsCtaThreads + threadIdx.x) / L;
    if (item >= m2) return;
    const int lane = threadIdx.x & 31;
    const int l = lane % L;
    const unsigned gmask = group_mask<L>(lane);

    const int row = __ldg(residue_r_ind + item);
    const int begin = __ldg(row_offsets + row);
    const int end = __ldg(row_offsets + row + 1);
    // Aligned length >= k_block: the row has a block part whose last segment produced the tail.
    if (end - begin + (begin % kAlign) >= kBlockK || end == begin) return;

    const size_t row_vecs = static_cast<size_t>(k) / 4;
    const float4 a = __ldg(reinterpret_cast<const float4 *>(lhs) + static_cast<size_t>(row) * row_vecs + l);
    const float4 *rhs_lane = reinterpret_cast<const float4 *>(rhs) + l;

    for (int base = begin; base < end; base += L) {
        const int e = base + l;
        int c = 0;
        float v = 0.f;
        if (e < end) {
            c = ld_stream(column_indices + e);
            v = ld_stream(values + e);
        }
        const int cnt = min(L, end - base);
        float mine = 0.f;
#pragma unroll
        for (int b = 0; b < L / kBatch; ++b) {
            if (b * kBatch >= cnt) break;
            float4 bb[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int t = b * kBatch + u;
                const int cc = __shfl_sync(gmask, c, t, L);
                bb[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (t < cnt) bb[u] = ld_dense(rhs_lane + static_cast<size_t>(cc) * row_vecs);
            }
            float p[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) p[u] = dot4(a, bb[u]);
            const float r = reduce_batch<L>(p, l, gmask);
            const float got = __shfl_sync(gmask, r, (l & (kBatch - 1)) * (L / kBatch), L);
            if ((l / kBatch) == b) mine = got;
        }
        if (e < end) st_stream(out + e, v * mine);
    }
}

// ---------------------------------------------------------------------------------------
// K = 128: a warp streams the nonzeros of 32 consecutive items.  kSegments: items are block
// segments (block_r_ind / st_off); otherwise residue rows (residue_r_ind) without block part.
template <bool kSegments>
__global__ void __launch_bounds__(32)
sddmm_stream(int n_items, const int *__restrict__ item_rows, const int *__restrict__ st_off,
             const int *__restrict__ row_offsets, const int *__restrict__ column_indices,
             const float *__restrict__ values, const float *__restrict__ lhs, const float *__restrict__ rhs,
             float *__restrict__ out) {
    constexpr int L = 32;
    constexpr int kAlign = 4;
    constexpr int kBlockK = 32;
    constexpr size_t kRowVecs = 32;  // K / 4
    const int lane = threadIdx.x;
    const long long item0 = static_cast<long long>(blockIdx.x) * 32;
    if (item0 >= n_items) return;

    // ---- descriptors: lane j owns item item0 + j ----------------------------------------
    int row = 0, begin = 0, len = 0;
    if (item0 + lane < n_items) {
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
    start -= len;
    unsigned todo = __ballot_sync(kFull, len > 0);
    if (todo == 0) return;

    // stream position p -> (nonzero index, column, value); all lanes call
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
        if (p < total) {
            e = b0 + (p - s0);
            c = ld_stream(column_indices + e);
            v = ld_stream(values + e);
        }
    };

    const float4 *lhs_lane = reinterpret_cast<const float4 *>(lhs) + lane;
    const float4 *rhs_lane = reinterpret_cast<const float4 *>(rhs) + lane;

    // consumer state: item being processed, its lhs slice, and the next item's (prefetched)
    int cur = __ffs(todo) - 1;
    todo &= todo - 1;
    int cur_end = __shfl_sync(kFull, start, cur) + __shfl_sync(kFull, len, cur);
    float4 a_cur = __ldg(lhs_lane + static_cast<size_t>(__shfl_sync(kFull, row, cur)) * kRowVecs);
    float4 a_nxt = a_cur;
    if (todo) a_nxt = __ldg(lhs_lane + static_cast<size_t>(__shfl_sync(kFull, row, __ffs(todo) - 1)) * kRowVecs);
    int pos = 0;

    int e_cur, c_cur, e_nxt, c_nxt;
    float v_cur, v_nxt;
    fetch(lane, e_cur, c_cur, v_cur);
    fetch(32 + lane, e_nxt, c_nxt, v_nxt);
    for (int base = 0; base < total; base += 32) {
        const int cnt = min(32, total - base);
        int e_pre, c_pre;
        float v_pre;
        fetch(base + 64 + lane, e_pre, c_pre, v_pre);
        float mine = 0.f;
#pragma unroll
        for (int b = 0; b < L / kBatch; ++b) {
            if (b * kBatch >= cnt) break;
            float4 bb[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int t = b * kBatch + u;
                const int cc = __shfl_sync(kFull, c_cur, t);
                bb[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (t < cnt) bb[u] = ld_dense(rhs_lane + static_cast<size_t>(cc) * kRowVecs);
            }
            float p[kBatch];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                if (pos == cur_end) {  // the stream enters the next item: switch the lhs row
                    cur = __ffs(todo) - 1;
                    todo &= todo - 1;
                    cur_end = (cur >= 0) ? __shfl_sync(kFull, start, cur & 31) + __shfl_sync(kFull, len, cur & 31)
                                         : INT_MAX;
                    a_cur = a_nxt;
                    if (todo)
                        a_nxt = __ldg(lhs_lane +
                                      static_cast<size_t>(__shfl_sync(kFull, row, __ffs(todo) - 1)) * kRowVecs);
                }
                p[u] = dot4(a_cur, bb[u]);
                ++pos;
            }
            const float r = reduce_batch<L>(p, lane, kFull);
            const float got = __shfl_sync(kFull, r, (lane & (kBatch - 1)) * (L / kBatch));
            if ((lane / kBatch) == b) mine = got;
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

template <int L>
int launch_k(int m1, int m2, int k, const int *block_r_ind, const int *residue_r_ind, const int *st_off,
             const int *row_offsets, const int *col, const float *values, const float *lhs, const float *rhs,
             float *out, cudaStream_t s1, cudaStream_t s2) {
    if (m1 > 0) {
        sddmm_block<L><<<(m1 + kCtaWarps - 1) / kCtaWarps, kCtaThreads, 0, s1>>>(
            m1, k, block_r_ind, st_off, row_offsets, col, values, lhs, rhs, out);
        RODE_CHECK_LAUNCH("rode::sddmm_block");
    }
    if (m2 > 0) {
        constexpr int kRowsPerCta = kRowsCtaThreads / L;
        sddmm_rows<L><<<(m2 + kRowsPerCta - 1) / kRowsPerCta, kRowsCtaThreads, 0, s2>>>(
            m2, k, residue_r_ind, row_offsets, col, values, lhs, rhs, out);
        RODE_CHECK_LAUNCH("rode::sddmm_rows");
    }
    return RODE_OK;
}

int launch_k128(int m1, int m2, const int *block_r_ind, const int *residue_r_ind, const int *st_off,
                const int *row_offsets, const int *col, const float *values, const float *lhs, const float *rhs,
                float *out, cudaStream_t s1, cudaStream_t s2) {
    if (m1 > 0) {
        sddmm_stream<true><<<(m1 + 31) / 32, 32, 0, s1>>>(m1, block_r_ind, st_off, row_offsets, col, values, lhs,
                                                          rhs, out);
        RODE_CHECK_LAUNCH("rode::sddmm_stream<segments>");
    }
    if (m2 > 0) {
        sddmm_stream<false><<<(m2 + 31) / 32, 32, 0, s2>>>(m2, residue_r_ind, nullptr, row_offsets, col, values,
                                                           lhs, rhs, out);
        RODE_CHECK_LAUNCH("rode::sddmm_stream<rows>");
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
    if (k != 32 && k != 64 && k != 128)
        return fail(RODE_ERR_INVALID_ARGUMENT, "sddmm: k = %d unsupported (32, 64 or 128)", k);
    if (m1 == 0 && m2 == 0) return RODE_OK;
    if (!row_offsets || !column_indices || !values || !lhs || !rhs || !out)
        return fail(RODE_ERR_INVALID_ARGUMENT, "sddmm: null array");
    if (m1 > 0 && (!block_r_ind || !st_off)) return fail(RODE_ERR_INVALID_ARGUMENT, "sddmm: null block metadata");
    if (m2 > 0 && !residue_r_ind) return fail(RODE_ERR_INVALID_ARGUMENT, "sddmm: null residue metadata");
    if (!aligned_to(lhs, 16) || !aligned_to(rhs, 16))
        return fail(RODE_ERR_INVALID_ARGUMENT, "sddmm: lhs and rhs must be 16-byte aligned");
    switch (k) {
        case 32:
            return launch_k<8>(m1, m2, k, block_r_ind, residue_r_ind, st_off, row_offsets, column_indices, values,
                               lhs, rhs, out, stream1, stream2);
        case 64:
            return launch_k<16>(m1, m2, k, block_r_ind, residue_r_ind, st_off, row_offsets, column_indices,
                                values, lhs, rhs, out, stream1, stream2);
        default:
            return launch_k128(m1, m2, block_r_ind, residue_r_ind, st_off, row_offsets, column_indices, values,
                               lhs, rhs, out, stream1, stream2);
    }
}
