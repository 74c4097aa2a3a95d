// RoDe SDDMM for sm_100a:  out[e] = values[e] * dot(lhs[row(e), :], rhs[col(e), :]).
//
// Stands in for the reference's SDDMMKernel4Block / SDDMMKernel4Residue
// (RoDe_SDDMM/RoDeSddmm.cu:15-203, :206-494) and their launchers (:496-545).  The work
// split follows the reference's metadata (block segments, residue rows); inside a unit:
//
//  * A dense row of length K is covered by L = K/4 lanes, one LDG.128 per lane, so a gather
//    of rhs[col, :] is one coalesced request of 4*K bytes.  K = 32, 64, 128 -> L = 8, 16, 32.
//  * A lane group works on L nonzeros at a time.  Lane l keeps its slice of the lhs row in
//    registers, forms the partial dot product of its slice with the same slice of each of
//    the L rhs rows (kUnroll rows in flight), and the L x L partials are reduced with a
//    shuffle transpose-reduce (L-1 shuffles) that leaves lane l with the dot product of
//    nonzero l.  Lane l also holds value l, so results are stored coalesced.
//  * sddmm_block: one warp per block segment; its G = 32/L groups take consecutive L-entry
//    pieces of each 32-entry chunk.  The last segment of a row also produces the row's tail
//    (shorter than 32) that the reference leaves to its residue kernel, so the lhs row is
//    read once per segment.
//  * sddmm_residue: one lane group per residue row without a block part (aligned length
//    < 32); other rows in the list were finished by sddmm_block.
//
// Per nonzero: 12 B of CSR data/output plus 4*K bytes of rhs (L1/L2/HBM by reuse); per
// segment 4*K bytes of lhs.  No shared memory, no atomics, no workspace.
#include <climits>

#include "rode_common.cuh"

namespace rode {
namespace {

constexpr int kCtaThreads = 128;
constexpr int kCtaWarps = kCtaThreads / 32;
constexpr int kUnroll = 8;  // rhs rows in flight per lane

__device__ __forceinline__ float dot4(const float4 &a, const float4 &b) {
    return fmaf(a.w, b.w, fmaf(a.z, b.z, fmaf(a.y, b.y, a.x * b.x)));
}

// Dot products of the lhs slice `a` with the rhs rows of the group's first `cnt` entries
// (column of entry t in lane t).  Returns, in lane l of the group, the full dot product of
// entry l (0 for l >= cnt).  `cnt` is uniform across the group.
template <int L>
__device__ __forceinline__ float group_dots(const float4 &a, int c, int cnt, const float4 *__restrict__ rhs_slice,
                                            size_t row_vecs, unsigned gmask, int l) {
    constexpr int U = kUnroll < L ? kUnroll : L;
    float p[L];
#pragma unroll
    for (int t = 0; t < L; ++t) p[t] = 0.f;
#pragma unroll
    for (int t0 = 0; t0 < L; t0 += U) {
        if (t0 >= cnt) break;
        float4 bb[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int cc = __shfl_sync(gmask, c, t0 + u, L);
            bb[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t0 + u < cnt) bb[u] = ld_dense(rhs_slice + static_cast<size_t>(cc) * row_vecs);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) p[t0 + u] = dot4(a, bb[u]);
    }
    // Transpose-reduce: after the step of width w, p[i] of a lane holds the sum over its
    // w-partner class for entry (i | (l & w) bits set so far).
#pragma unroll
    for (int w = L / 2; w >= 1; w >>= 1) {
        const bool upper = (l & w) != 0;
#pragma unroll
        for (int i = 0; i < w; ++i) {
            const float send = upper ? p[i] : p[i + w];
            const float keep = upper ? p[i + w] : p[i];
            p[i] = keep + __shfl_xor_sync(gmask, send, w, L);
        }
    }
    return p[0];
}

template <int L>
__global__ void __launch_bounds__(kCtaThreads)
sddmm_block(int m1, int k, const int *__restrict__ block_r_ind, const int *__restrict__ st_off,
            const int *__restrict__ row_offsets, const int *__restrict__ column_indices,
            const float *__restrict__ values, const float *__restrict__ lhs, const float *__restrict__ rhs,
            float *__restrict__ out) {
    const int seg = blockIdx.x * kCtaWarps + (threadIdx.x >> 5);
    if (seg >= m1) return;
    const int lane = threadIdx.x & 31;
    const int g = lane / L, l = lane % L;
    const unsigned gmask = group_mask<L>(lane);

    const int row = __ldg(block_r_ind + seg);
    const int off = __ldg(st_off + seg);
    const int next = (seg + 1 < m1) ? __ldg(st_off + seg + 1) : INT_MAX;
    const int end = min(__ldg(row_offsets + row + 1), next);

    const size_t row_vecs = static_cast<size_t>(k) / 4;
    const float4 a = __ldg(reinterpret_cast<const float4 *>(lhs) + static_cast<size_t>(row) * row_vecs + l);
    const float4 *rhs_slice = reinterpret_cast<const float4 *>(rhs) + l;

    int e = off + lane;
    int c = 0;
    float v = 0.f;
    if (e < end) {
        c = ld_stream(column_indices + e);
        v = ld_stream(values + e);
    }
    for (int base = off; base < end; base += 32) {
        const int cur_c = c, cur_e = e;
        const float cur_v = v;
        e += 32;
        c = 0;
        v = 0.f;
        if (e < end) {  // prefetch the next chunk while this one is gathered
            c = ld_stream(column_indices + e);
            v = ld_stream(values + e);
        }
        const int cnt = min(L, max(0, end - base - g * L));
        const float d = group_dots<L>(a, cur_c, cnt, rhs_slice, row_vecs, gmask, l);
        if (cur_e < end) st_stream(out + cur_e, cur_v * d);
    }
}

template <int L>
__global__ void __launch_bounds__(kCtaThreads)
sddmm_residue(int m2, int k, const int *__restrict__ residue_r_ind, const int *__restrict__ row_offsets,
              const int *__restrict__ column_indices, const float *__restrict__ values,
              const float *__restrict__ lhs, const float *__restrict__ rhs, float *__restrict__ out) {
    constexpr int kAlign = 4;    // vec_len of the preprocessing
    constexpr int kBlockK = 32;  // k_block of the preprocessing
    const int item = (blockIdx.x * kCtaThreads + threadIdx.x) / L;
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
    const float4 *rhs_slice = reinterpret_cast<const float4 *>(rhs) + l;

    for (int base = begin; base < end; base += L) {
        const int e = base + l;
        int c = 0;
        float v = 0.f;
        if (e < end) {
            c = ld_stream(column_indices + e);
            v = ld_stream(values + e);
        }
        const float d = group_dots<L>(a, c, min(L, end - base), rhs_slice, row_vecs, gmask, l);
        if (e < end) st_stream(out + e, v * d);
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
        constexpr int kRowsPerCta = kCtaThreads / L;
        sddmm_residue<L><<<(m2 + kRowsPerCta - 1) / kRowsPerCta, kCtaThreads, 0, s2>>>(
            m2, k, residue_r_ind, row_offsets, col, values, lhs, rhs, out);
        RODE_CHECK_LAUNCH("rode::sddmm_residue");
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
            return launch_k<32>(m1, m2, k, block_r_ind, residue_r_ind, st_off, row_offsets, column_indices,
                                values, lhs, rhs, out, stream1, stream2);
    }
}
