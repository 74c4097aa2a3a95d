// RoDe SpMM for sm_100a:  C[M x n] = S * B  with S in CSR + row-decomposition metadata.
//
// Stands in for the reference's block / residue kernels (RoDe_SpMM/RoDeSpmm.cu:197-476 and
// :41-195) and their launcher (:492-529).  The work split follows the reference's metadata
// (one unit per block segment, one per residue row); what each unit does is new:
//
//  * A dense row of the tile is covered by L lanes, 16 bytes per lane (one LDG.128), so a
//    gather of B[col, tile] is one fully coalesced request of 16*L bytes.  L = 8, 16 or 32;
//    a warp holds G = 32/L such lane groups.
//  * spmm_block: one WARP per block segment.  The warp streams the segment's (col, value)
//    pairs 32 at a time (coalesced, prefetched one chunk ahead), group g takes entries
//    g*L .. g*L+L-1 of the chunk, fetches kUnroll dense rows at once per lane and
//    accumulates in registers.  Groups are combined with log2(G) shuffle steps.
//    The LAST segment of a row also consumes the row's tail (the part shorter than 32 that
//    the reference leaves to its residue kernel), so a row that fits one segment is
//    finished by a single warp and stored with plain vector stores.
//  * Rows cut into several segments: every segment writes its partial row to a workspace
//    slot (slot = segment index); spmm_fixup, ordered after spmm_block on the same stream,
//    sums the slots of each such row in segment order (fp64 accumulation) and stores the
//    row.  No floating-point atomics anywhere: results are deterministic.
//  * spmm_residue: one L-lane group per residue row that has NO block part (aligned length
//    < 32); rows with a block part were already finished by spmm_block.  Empty rows in the
//    list are stored as zeros, as the reference does (RoDeSpmm.cu:185-194).
//
// Per nonzero the kernels move 8 B of CSR data and 16*L bytes of the dense operand (from
// L1/L2/HBM depending on reuse); per row 4*n bytes of C.  Dense-row offsets are 64-bit.
#include <climits>

#include "rode_common.cuh"

namespace rode {
namespace {

constexpr int kCtaThreads = 128;
constexpr int kCtaWarps = kCtaThreads / 32;
constexpr int kUnroll = 8;  // dense rows in flight per lane

// acc += sum over the group's first `cnt` entries of value * B[col, slice].
// (c, v) of entry t live in lane t of the group.  `cnt` is uniform across the group, and
// `gmask` names exactly the lanes of the group (groups of one warp may leave early).
template <typename T, int L>
__device__ __forceinline__ void gather_fma(typename Vec16<T>::type &acc, int c, T v, int cnt,
                                           const typename Vec16<T>::type *__restrict__ b_slice, size_t row_vecs,
                                           unsigned gmask) {
    using V = typename Vec16<T>::type;
    constexpr int U = kUnroll < L ? kUnroll : L;
#pragma unroll
    for (int t0 = 0; t0 < L; t0 += U) {
        if (t0 >= cnt) break;
        int cc[U];
        T vv[U];
        V bb[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            cc[u] = __shfl_sync(gmask, c, t0 + u, L);
            vv[u] = __shfl_sync(gmask, v, t0 + u, L);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            bb[u] = vzero(static_cast<V *>(nullptr));
            if (t0 + u < cnt) bb[u] = ld_dense(b_slice + static_cast<size_t>(cc[u]) * row_vecs);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) vfma(acc, vv[u], bb[u]);
    }
}

// One warp per block segment; grid.y walks the column tiles of width L * kLen.
template <typename T, int L>
__global__ void __launch_bounds__(kCtaThreads)
spmm_block(int m1, int n, const T *__restrict__ values, const int *__restrict__ column_indices,
           const int *__restrict__ row_offsets, const int *__restrict__ block_r_ind,
           const int *__restrict__ st_off, const T *__restrict__ B, T *__restrict__ C, T *__restrict__ partial) {
    using V = typename Vec16<T>::type;
    constexpr int kLen = Vec16<T>::kLen;
    const int seg = blockIdx.x * kCtaWarps + (threadIdx.x >> 5);
    if (seg >= m1) return;
    const int lane = threadIdx.x & 31;
    const int g = lane / L, l = lane % L;
    const unsigned gmask = group_mask<L>(lane);

    const int row = __ldg(block_r_ind + seg);
    const int off = __ldg(st_off + seg);
    const int next = (seg + 1 < m1) ? __ldg(st_off + seg + 1) : INT_MAX;
    const int row_begin = __ldg(row_offsets + row);
    const int row_end = __ldg(row_offsets + row + 1);
    const int end = min(row_end, next);
    const bool whole_row = (off == row_begin) && (next >= row_end);

    const size_t row_vecs = static_cast<size_t>(n) / kLen;
    const V *b_slice = reinterpret_cast<const V *>(B) + static_cast<size_t>(blockIdx.y) * L + l;

    V acc = vzero(static_cast<V *>(nullptr));
    int e = off + lane;
    int c = 0;
    T v = T(0);
    if (e < end) {
        c = ld_stream(column_indices + e);
        v = ld_stream(values + e);
    }
    for (int base = off; base < end; base += 32) {
        const int cur_c = c;
        const T cur_v = v;
        e += 32;
        c = 0;
        v = T(0);
        if (e < end) {  // prefetch the next chunk while this one is gathered
            c = ld_stream(column_indices + e);
            v = ld_stream(values + e);
        }
        const int cnt = min(L, max(0, end - base - g * L));
        gather_fma<T, L>(acc, cur_c, cur_v, cnt, b_slice, row_vecs, gmask);
    }
#pragma unroll
    for (int w = L; w < 32; w <<= 1) vadd(acc, vshfl_xor(0xffffffffu, acc, w));

    if (g == 0) {
        const size_t col_vec = static_cast<size_t>(blockIdx.y) * L + l;
        if (whole_row)
            st_stream(reinterpret_cast<V *>(C) + static_cast<size_t>(row) * row_vecs + col_vec, acc);
        else
            reinterpret_cast<V *>(partial)[static_cast<size_t>(seg) * row_vecs + col_vec] = acc;
    }
}

// Sums the workspace slots of every row that was cut into several segments.  One warp
// looks at 32 consecutive segments; a lane whose segment is the first of a split row flags
// it, and the warp then adds that row's slots in segment order.
template <typename T>
__global__ void __launch_bounds__(kCtaThreads)
spmm_fixup(int m1, int n, const int *__restrict__ row_offsets, const int *__restrict__ block_r_ind,
           const int *__restrict__ st_off, const T *__restrict__ partial, T *__restrict__ C) {
    const int lane = threadIdx.x & 31;
    const int seg = (blockIdx.x * kCtaWarps + (threadIdx.x >> 5)) * 32 + lane;
    bool head = false;
    if (seg < m1) {
        const int row = __ldg(block_r_ind + seg);
        const int off = __ldg(st_off + seg);
        const int next = (seg + 1 < m1) ? __ldg(st_off + seg + 1) : INT_MAX;
        head = (off == __ldg(row_offsets + row)) && (next < __ldg(row_offsets + row + 1));
    }
    unsigned todo = __ballot_sync(0xffffffffu, head);
    while (todo) {
        const int src = __ffs(todo) - 1;
        todo &= todo - 1;
        const int first = seg - lane + src;
        const int row = __ldg(block_r_ind + first);
        int last = first + 1;
        while (last < m1 && __ldg(block_r_ind + last) == row) ++last;
        for (int x = lane; x < n; x += 32) {
            double sum = 0.0;
            for (int s = first; s < last; ++s) sum += static_cast<double>(partial[static_cast<size_t>(s) * n + x]);
            C[static_cast<size_t>(row) * n + x] = static_cast<T>(sum);
        }
    }
}

// One L-lane group per residue row without a block part.
template <typename T, int L>
__global__ void __launch_bounds__(kCtaThreads)
spmm_residue(int m2, int n, const T *__restrict__ values, const int *__restrict__ column_indices,
             const int *__restrict__ row_offsets, const int *__restrict__ residue_r_ind,
             const T *__restrict__ B, T *__restrict__ C) {
    using V = typename Vec16<T>::type;
    constexpr int kLen = Vec16<T>::kLen;
    constexpr int kAlign = 4;   // vec_len of the preprocessing
    constexpr int kBlockK = 32; // k_block of the preprocessing
    const int item = (blockIdx.x * kCtaThreads + threadIdx.x) / L;
    if (item >= m2) return;
    const int lane = threadIdx.x & 31;
    const int l = lane % L;
    const unsigned gmask = group_mask<L>(lane);

    const int row = __ldg(residue_r_ind + item);
    const int begin = __ldg(row_offsets + row);
    const int end = __ldg(row_offsets + row + 1);
    // Aligned length >= k_block: the row has a block part, whose last segment already
    // consumed the tail (see spmm_block).
    if (end - begin + (begin % kAlign) >= kBlockK) return;

    const size_t row_vecs = static_cast<size_t>(n) / kLen;
    const size_t col_vec = static_cast<size_t>(blockIdx.y) * L + l;
    const V *b_slice = reinterpret_cast<const V *>(B) + col_vec;

    V acc = vzero(static_cast<V *>(nullptr));
    for (int base = begin; base < end; base += L) {
        const int e = base + l;
        int c = 0;
        T v = T(0);
        if (e < end) {
            c = ld_stream(column_indices + e);
            v = ld_stream(values + e);
        }
        gather_fma<T, L>(acc, c, v, min(L, end - base), b_slice, row_vecs, gmask);
    }
    st_stream(reinterpret_cast<V *>(C) + static_cast<size_t>(row) * row_vecs + col_vec, acc);
}

template <typename T, int L>
int launch_width(int m1, int m2, int n, const T *values, const int *col, const int *row_offsets,
                 const int *block_r_ind, const int *residue_r_ind, const int *st_off, const T *B, T *C,
                 T *partial, cudaStream_t s1, cudaStream_t s2) {
    constexpr int kTileWidth = L * Vec16<T>::kLen;
    const unsigned tiles = static_cast<unsigned>(n / kTileWidth);
    if (m1 > 0) {
        dim3 grid((m1 + kCtaWarps - 1) / kCtaWarps, tiles);
        spmm_block<T, L><<<grid, kCtaThreads, 0, s1>>>(m1, n, values, col, row_offsets, block_r_ind, st_off, B,
                                                       C, partial);
        RODE_CHECK_LAUNCH("rode::spmm_block");
        const int per_cta = kCtaWarps * 32;
        spmm_fixup<T><<<(m1 + per_cta - 1) / per_cta, kCtaThreads, 0, s1>>>(m1, n, row_offsets, block_r_ind,
                                                                            st_off, partial, C);
        RODE_CHECK_LAUNCH("rode::spmm_fixup");
    }
    if (m2 > 0) {
        constexpr int kRowsPerCta = kCtaThreads / L;
        dim3 grid((m2 + kRowsPerCta - 1) / kRowsPerCta, tiles);
        spmm_residue<T, L><<<grid, kCtaThreads, 0, s2>>>(m2, n, values, col, row_offsets, residue_r_ind, B, C);
        RODE_CHECK_LAUNCH("rode::spmm_residue");
    }
    return RODE_OK;
}

template <typename T>
int spmm(int m1, int m2, int k, int n, const T *values, const int *col, const int *row_offsets,
         const int *block_r_ind, const int *residue_r_ind, const int *st_off, const T *B, T *C, void *workspace,
         size_t workspace_bytes, rode_stream_t stream1, rode_stream_t stream2) {
    constexpr int kLen = Vec16<T>::kLen;
    (void)k;
    if (m1 < 0 || m2 < 0 || n <= 0) return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: m1, m2 >= 0 and n > 0 required");
    if (n % (8 * kLen) != 0)
        return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: n = %d is not a multiple of %d", n, 8 * kLen);
    if (m1 == 0 && m2 == 0) return RODE_OK;
    if (!values || !col || !row_offsets || !B || !C) return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: null array");
    if (m1 > 0 && (!block_r_ind || !st_off)) return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: null block metadata");
    if (m2 > 0 && !residue_r_ind) return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: null residue metadata");
    if (!aligned_to(B, 16) || !aligned_to(C, 16))
        return fail(RODE_ERR_INVALID_ARGUMENT, "spmm: B and C must be 16-byte aligned");
    size_t need = 0;
    rode_spmm_workspace_bytes(m1, n, static_cast<int>(sizeof(T)), &need);
    if (need > 0) {
        if (workspace == nullptr || workspace_bytes < need)
            return fail(RODE_ERR_WORKSPACE, "spmm: workspace of %zu bytes needed, %zu given", need,
                        workspace ? workspace_bytes : static_cast<size_t>(0));
        if (!aligned_to(workspace, 16)) return fail(RODE_ERR_WORKSPACE, "spmm: workspace must be 16-byte aligned");
    }
    T *partial = static_cast<T *>(workspace);
    // Widest lane group whose tile divides n.
    if (n % (32 * kLen) == 0)
        return launch_width<T, 32>(m1, m2, n, values, col, row_offsets, block_r_ind, residue_r_ind, st_off, B, C,
                                   partial, stream1, stream2);
    if (n % (16 * kLen) == 0)
        return launch_width<T, 16>(m1, m2, n, values, col, row_offsets, block_r_ind, residue_r_ind, st_off, B, C,
                                   partial, stream1, stream2);
    return launch_width<T, 8>(m1, m2, n, values, col, row_offsets, block_r_ind, residue_r_ind, st_off, B, C,
                              partial, stream1, stream2);
}

}  // namespace
}  // namespace rode

extern "C" {

int rode_spmm_workspace_bytes(int m1, int n, int elem_size, size_t *bytes) {
    if (bytes == nullptr || m1 < 0 || n < 0 || (elem_size != 4 && elem_size != 8))
        return rode::fail(RODE_ERR_INVALID_ARGUMENT, "spmm_workspace_bytes: bad argument");
    *bytes = static_cast<size_t>(m1) * static_cast<size_t>(n) * static_cast<size_t>(elem_size);
    return RODE_OK;
}

int rode_spmm_f32(int m1, int m2, int k, int n, const float *values, const int *column_indices,
                  const int *row_offsets, const int *block_r_ind, const int *residue_r_ind, const int *st_off,
                  const float *B, float *C, void *workspace, size_t workspace_bytes, rode_stream_t stream1,
                  rode_stream_t stream2) {
    return rode::spmm<float>(m1, m2, k, n, values, column_indices, row_offsets, block_r_ind, residue_r_ind,
                             st_off, B, C, workspace, workspace_bytes, stream1, stream2);
}

int rode_spmm_f64(int m1, int m2, int k, int n, const double *values, const int *column_indices,
                  const int *row_offsets, const int *block_r_ind, const int *residue_r_ind, const int *st_off,
                  const double *B, double *C, void *workspace, size_t workspace_bytes, rode_stream_t stream1,
                  rode_stream_t stream2) {
    return rode::spmm<double>(m1, m2, k, n, values, column_indices, row_offsets, block_r_ind, residue_r_ind,
                              st_off, B, C, workspace, workspace_bytes, stream1, stream2);
}

}  // extern "C"
