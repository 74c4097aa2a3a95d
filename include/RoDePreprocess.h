/*
 * Drop-in C++ declarations of the reference's preprocessing calls.  The reference defines
 * them in Preprocess_opt/_preprocess.cu:323 (RoDe_preprocess, device pointers) and :340
 * (RoDe_preprocess_cpu, host pointers) without a header; callers declare them by hand.
 *
 * RoDe_preprocess: device pointers, runs asynchronously on the default stream, leaves the
 * counts in the device ints n_blk / n_res and writes exactly n_blk entries of block_r_ind
 * and st_off and n_res entries of residue_r_ind, as the reference does: no end sentinel
 * st_off[n_blk], so buffers sized like the reference's callers size them (nnz / N_SEG + M
 * entries, Preprocess_opt/_preprocess.cu:426-430) are large enough.  The SpMM and SDDMM
 * entry points of this library never read st_off[n_blk].  Its scratch (8 bytes per 2048
 * rows) comes from a buffer the library allocates on first use.
 * RoDe_preprocess_cpu: the single-thread host loop.  It also writes the sentinel
 * st_off[n_blk] = row_ptr[M], as the reference's copies of this loop in its SDDMM drivers do
 * (RoDe_SDDMM/main.cu:162; the copy at _preprocess.cu:340-373 does not), so its st_off needs
 * n_blk + 1 entries.
 * Argument order of both: (N_SEG, blockX, vecLen, M, ...) = (seg_len, k_block, vec_len).
 */
#ifndef RODE_B200_RODEPREPROCESS_H_
#define RODE_B200_RODEPREPROCESS_H_

void RoDe_preprocess(int N_SEG, int blockX, int vecLen, int M, const int *row_ptr,
                     int *block_r_ind, int *st_off, int *residue_r_ind, int *n_blk, int *n_res);

void RoDe_preprocess_cpu(int N_SEG, int blockX, int vecLen, int M, const int *row_ptr,
                         int *block_r_ind, int *st_off, int *residue_r_ind, int &n_blk, int &n_res);

#endif /* RODE_B200_RODEPREPROCESS_H_ */
