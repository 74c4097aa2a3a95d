/*
 * rode_b200 — C ABI of the RoDe hot path (row-decomposition preprocessing, SpMM, SDDMM)
 * for NVIDIA B200 (sm_100a).  Shared library: librode_b200.so.
 *
 * Plain C: pointers, ints and sizes only.  Every function returns a status code
 * (RODE_OK == 0) and never throws, prints or exits; rode_last_error() gives a
 * thread-local message for the last non-zero status.  All data pointers are DEVICE
 * pointers unless the name ends in _cpu / says "host".  Launches are asynchronous on the
 * streams passed in; a null stream means the CUDA default stream.
 *
 * Each entry point names the interface of the reference project (Da1sypetals/rode,
 * file:line inside that project) that it stands in for.  The C++ signatures of the
 * reference itself are declared in RoDeSpmm.h, RoDeSddmm.h and RoDePreprocess.h beside
 * this file and are thin wrappers over the functions below.
 *
 * Array contract shared by all compute calls (same as the reference):
 *   row_offsets   int32[M+1]   CSR row pointer
 *   column_indices int32[nnz], values T[nnz]
 *   block_r_ind   int32[m1]    row of every block segment          (preprocess output)
 *   st_off        int32[m1+1]  first nonzero of every segment; st_off[m1] is an end
 *                              sentinel (any value >= row_offsets[M]); this library never
 *                              reads st_off[m1]
 *   residue_r_ind int32[m2]    rows that own a residue             (preprocess output)
 * The metadata must be what the preprocessing produces for the same row_offsets.
 */
#ifndef RODE_B200_H_
#define RODE_B200_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cudaStream_t without pulling in the CUDA headers. */
typedef struct CUstream_st *rode_stream_t;

enum rode_status {
    RODE_OK = 0,
    RODE_ERR_INVALID_ARGUMENT = 1, /* null pointer, negative size, unsupported width, ... */
    RODE_ERR_WORKSPACE = 2,        /* workspace missing or too small                      */
    RODE_ERR_CUDA = 3,             /* a CUDA runtime call or a launch failed              */
    RODE_ERR_NO_DEVICE = 4         /* no usable sm_100 device                             */
};

/* Message for the last non-zero status returned on this thread ("" if none). */
const char *rode_last_error(void);

/* Library version, "major.minor.patch". */
const char *rode_version(void);

/* ------------------------------------------------------------------------------------
 * Row-decomposition preprocessing.
 *
 * rode_preprocess replaces RoDe_preprocess (Preprocess_opt/_preprocess.cu:323-339: count
 * kernel, two CUB scans, fill kernel).  Results are bit-identical to the reference's
 * specification loop RoDe_preprocess_cpu (Preprocess_opt/_preprocess.cu:340-373), and the
 * end sentinel st_off[n_blk] = row_ptr[M] of the reference's host copies
 * (RoDe_SDDMM/main.cu:162) is written too.
 *
 *   seg_len  nonzeros per block segment (512; 32 for SDDMM with K = 128)
 *   k_block  smallest block-part length (32); seg_len % k_block == 0
 *   vec_len  alignment unit of row starts (4); k_block % vec_len == 0
 *   row_ptr  int32[M+1] device
 *   block_r_ind, st_off   device, capacity >= n_blk (+1 for st_off); the bound
 *                         rode_preprocess_capacity() is always enough
 *   residue_r_ind         device, capacity >= min(M, n_res)
 *   n_blk, n_res          device int32[1] each
 *   workspace             device scratch of rode_preprocess_workspace_bytes(M) bytes,
 *                         256-byte aligned; contents are don't-care before and after;
 *                         calls that may run at the same time need a workspace each
 * Unlike the reference, outputs are never used as scratch, so there is no in-place
 * hazard between thread blocks.
 */
int rode_preprocess_workspace_bytes(int M, size_t *bytes);

/* Upper bound of n_blk for a matrix of M rows and nnz nonzeros (host arithmetic only):
 * (nnz + (vec_len-1)*M) / seg_len + M. */
int rode_preprocess_capacity(int seg_len, int vec_len, int M, long long nnz, long long *max_blocks);

int rode_preprocess(int seg_len, int k_block, int vec_len, int M, const int *row_ptr,
                    int *block_r_ind, int *st_off, int *residue_r_ind, int *n_blk, int *n_res,
                    void *workspace, size_t workspace_bytes, rode_stream_t stream);

/* Same decomposition, same outputs, but the library allocates nothing and the caller brings
 * no workspace: the per-tile scratch lives in a fixed array inside the library's device
 * image (64 KB on every GPU that loads the library, kept until the process exits).
 * This entry point has no counterpart in the reference.
 *
 * It is meant for callers that must not, or cannot, obtain device memory at call time:
 * a process that has handed the whole GPU to its own memory pool (a serving engine's
 * arena, a framework's caching allocator with a hard cap), where a cudaMalloc issued by a
 * library can fail or fragment the pool; and callers inside a latency-critical loop, where
 * cudaMalloc / cudaFree would synchronise the whole device and stall every other stream.
 * Those callers also cannot use RoDe_preprocess (it grows a library-owned buffer with
 * cudaMalloc on first use) and may have no spare buffer to pass to rode_preprocess.
 *
 *   Limit     M <= 16,777,216 rows (2^24); larger M returns RODE_ERR_INVALID_ARGUMENT with a
 *             message, before anything is launched.
 *   Set-up    the first call on each device looks up the array's device address (the
 *             device must be current, as for every call); make that first call before any
 *             stream capture begins.  No cudaMalloc, cudaFree or other allocating routine
 *             is called, then or later.  The address is remembered per device ordinal for
 *             the life of the process: after a cudaDeviceReset in the same process it is
 *             stale, so do not call this entry point again after resetting a device.
 *   Sharing   all calls on a device use the same array and it keeps the previous call's
 *             contents.  The caller clears nothing (the call itself zeroes its 8-byte
 *             counter with a memset node on the stream, and every other entry that is read is
 *             written first by the same call), but two calls that overlap in time on one GPU,
 *             e.g. on two streams, race on it: serialise them. */
int rode_preprocess_noalloc(int seg_len, int k_block, int vec_len, int M, const int *row_ptr,
                            int *block_r_ind, int *st_off, int *residue_r_ind, int *n_blk, int *n_res,
                            rode_stream_t stream);

/* Host twin with HOST pointers, replacing RoDe_preprocess_cpu
 * (Preprocess_opt/_preprocess.cu:340-373) and the host loops of
 * RoDe_SDDMM/main.cu:114-163.  Part of the reference's API surface; it is not a fallback
 * for the device path and nothing in this library calls it. */
int rode_preprocess_cpu(int seg_len, int k_block, int vec_len, int M, const int *row_ptr,
                        int *block_r_ind, int *st_off, int *residue_r_ind, int *n_blk, int *n_res);

/* ------------------------------------------------------------------------------------
 * SpMM:  C[M x n] = S[M x k] * B[k x n], S in CSR + RoDe metadata, B and C row-major.
 *
 * Replaces RoDeSpmm_n32 / RoDeSpmm_n128 (RoDe_SpMM/RoDeSpmm.h:4-14, launcher
 * RoDe_SpMM/RoDeSpmm.cu:492-529).  One call serves every width: n may be any multiple
 * of 4 columns, float or double.  Multiples of 32 (float) or 16 (double) are covered by whole
 * lane-group tiles as in the reference; other widths, which the reference does not serve, leave
 * part of the last tile idle and take no popularity hints.  Block segments run on stream1,
 * pure-residue rows on stream2; the caller synchronises both, as with the reference.
 *
 * Differences a caller can observe: every row with at least one nonzero is WRITTEN (not
 * accumulated), without floating-point atomics, so results are deterministic.  Rows without
 * a nonzero are never touched: C must be zero there, which the reference's contract (C
 * zero-filled by the caller) already guarantees.  (The reference stores explicit zeros into
 * the empty rows of its residue list, RoDeSpmm.cu:185-194; with a zero-filled C the result
 * is the same, and on graphs with many empty rows those stores were half of the residue
 * kernel's DRAM writes.)
 *
 * `workspace`: rode_spmm_workspace_bytes(m1, n, sizeof(T)) bytes, 16-byte aligned, contents
 * don't-care before and after the call.  It holds one partial row per block segment (rows
 * split over several segments are summed through it, in a fixed order) and, in its last 256
 * bytes, the counters from which the warps of the large-grid kernels claim their next
 * segment or bundle of rows (those kernels run as one resident wave of CTAs; the library
 * zeroes the counters on the call's streams).  With m1 == 0 the workspace may be null; the
 * residue kernel then runs one CTA per bundle of rows.  Calls that may overlap in time on the
 * GPU must not share a workspace.  Column byte offsets are formed in 64 bits.
 *
 * The metadata must come from the preprocessing with k_block = 32 and vec_len = 4 (any
 * seg_len that is a multiple of 32), the values the reference's kernels are written for
 * (RoDe_SpMM/RoDeSpmm.cu:513,518: 4-wide vectors, 32-nonzero tiles); st_off[m1] is not read.
 */
int rode_spmm_workspace_bytes(int m1, int n, int elem_size, size_t *bytes);

int rode_spmm_f32(int m1, int m2, int k, int n, const float *values, const int *column_indices,
                  const int *row_offsets, const int *block_r_ind, const int *residue_r_ind,
                  const int *st_off, const float *B, float *C, void *workspace,
                  size_t workspace_bytes, rode_stream_t stream1, rode_stream_t stream2);

int rode_spmm_f64(int m1, int m2, int k, int n, const double *values, const int *column_indices,
                  const int *row_offsets, const int *block_r_ind, const int *residue_r_ind,
                  const int *st_off, const double *B, double *C, void *workspace,
                  size_t workspace_bytes, rode_stream_t stream1, rode_stream_t stream2);

/* ------------------------------------------------------------------------------------
 * Column popularity hints for the gathers.  No counterpart in the reference.
 *
 * When the dense operand is many times larger than the L2 and a few columns receive most of
 * the references (power-law graphs), rows that are gathered once push rows that are gathered
 * thousands of times out of the L2.  rode_hot_columns counts the references of every column
 * and marks the most referenced ones whose dense rows (dense_row_bytes each) fit
 * budget_bytes (0 = 60 % of the device's L2).  rode_spmm_f32_hot / _f64_hot then gather
 * marked rows with the L2 policy evict_last and all others with evict_first.  Results are
 * bit-identical to rode_spmm_f32 / _f64; only the DRAM traffic changes.
 *
 * hot_columns: unsigned[rode_hot_columns_words(n_cols)] = one bit per column plus a trailing
 * flag word.  The flag is 0 when the marks would not help (the touched rows nearly fit the
 * budget anyway, or the marked columns get less than twice their share of the references);
 * the SpMM entry points must then be given a null hot_columns pointer, or simply the plain
 * entry points be used.  The hints take effect for n that is a multiple of 128 (float) or
 * 64 (double) and grids of more than two waves of warps; other calls ignore them.
 * workspace: rode_hot_columns_workspace_bytes(n_cols) bytes, 256-byte aligned, only used
 * during the call.
 */
int rode_hot_columns_workspace_bytes(int n_cols, size_t *bytes);
int rode_hot_columns_words(int n_cols, size_t *words);
int rode_hot_columns(long long nnz, int n_cols, const int *column_indices, size_t dense_row_bytes,
                     size_t budget_bytes, unsigned *hot_columns, void *workspace,
                     size_t workspace_bytes, rode_stream_t stream);

int rode_spmm_f32_hot(int m1, int m2, int k, int n, const float *values, const int *column_indices,
                      const int *row_offsets, const int *block_r_ind, const int *residue_r_ind,
                      const int *st_off, const float *B, float *C, void *workspace,
                      size_t workspace_bytes, const unsigned *hot_columns, rode_stream_t stream1,
                      rode_stream_t stream2);

int rode_spmm_f64_hot(int m1, int m2, int k, int n, const double *values, const int *column_indices,
                      const int *row_offsets, const int *block_r_ind, const int *residue_r_ind,
                      const int *st_off, const double *B, double *C, void *workspace,
                      size_t workspace_bytes, const unsigned *hot_columns, rode_stream_t stream1,
                      rode_stream_t stream2);

/* ------------------------------------------------------------------------------------
 * SDDMM:  out[e] = values[e] * dot(lhs[row(e), 0:k], rhs[col(e), 0:k]) for every stored e.
 *
 * Replaces RoDeSDDMM_n32 / RoDeSDDMM_n128 (RoDe_SDDMM/RoDeSddmm.h:4-9, launchers
 * RoDe_SDDMM/RoDeSddmm.cu:496-545).  k: any multiple of 4 up to 256 (the reference has 32
 * and 128; here 32, 64 and 128 have kernels of their own shape, every other k runs a
 * 32-lane x 2-vector form with the vectors beyond the row's end masked);
 * lhs is [M x k], rhs is [n x k], both row-major; out is fp32[nnz] aligned with values.
 * Block segments run on stream1, pure-residue rows on stream2.  A null stream is the
 * default stream (the reference silently skips a kernel whose stream handle is null,
 * RoDeSddmm.cu:503,509; this library does not).  Needs no workspace: the one counter the
 * large-grid block kernel claims its segments from lives in a fixed array of the library's
 * device image (32 KB per GPU), one slot per (device, stream1, stream2) seen by the process;
 * calls on the same streams are ordered by them, calls on other streams use other slots, and
 * beyond 128 distinct stream pairs the kernel runs one CTA per segment instead.  As with the
 * reference, one host thread at a time should enqueue calls on a given pair of streams.
 * Metadata as for SpMM: k_block = 32, vec_len = 4, any seg_len that is a multiple of 32.
 */
int rode_sddmm_f32(int m1, int m2, int n, int k, const int *block_r_ind, const int *residue_r_ind,
                   const int *st_off, const int *row_offsets, const int *column_indices,
                   const float *values, const float *lhs, const float *rhs, float *out,
                   rode_stream_t stream1, rode_stream_t stream2);

#ifdef __cplusplus
}
#endif
#endif /* RODE_B200_H_ */
