/*
 * Drop-in C++ declarations of the reference's preprocessing calls.  The reference defines
 * them in Preprocess_opt/_preprocess.cu:323 (RoDe_preprocess, device pointers) and :340
 * (RoDe_preprocess_cpu, host pointers) without a header; callers declare them by hand.
 *
 * RoDe_preprocess: device pointers, runs asynchronously on the default stream, leaves the
 * counts in the device ints n_blk / n_res (as the reference does), and additionally
 * writes the end sentinel st_off[n_blk] = row_ptr[M].  Its scratch (8 bytes per 1024
 * rows) comes from a per-device buffer the library allocates on first use.
 * RoDe_preprocess_cpu: the single-thread host loop, also writing the sentinel.
 * Argument order of both: (N_SEG, blockX, vecLen, M, ...) = (seg_len, k_block, vec_len).
 */
#ifndef RODE_B200_RODEPREPROCESS_H_
#define RODE_B200_RODEPREPROCESS_H_

void RoDe_preprocess(int N_SEG, int blockX, int vecLen, int M, const int *row_ptr,
                     int *block_r_ind, int *st_off, int *residue_r_ind, int *n_blk, int *n_res);

void RoDe_preprocess_cpu(int N_SEG, int blockX, int vecLen, int M, const int *row_ptr,
                         int *block_r_ind, int *st_off, int *residue_r_ind, int &n_blk, int &n_res);

#endif /* RODE_B200_RODEPREPROCESS_H_ */
