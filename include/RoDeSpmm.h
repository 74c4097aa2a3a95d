/*
 * Drop-in C++ declarations of the reference's SpMM entry points
 * (Da1sypetals/rode, RoDe_SpMM/RoDeSpmm.h:4-14), implemented by librode_b200.so as thin
 * wrappers over rode_spmm_f32 / rode_spmm_f64 (rode_b200.h).
 *
 * Same argument order and meaning as the reference:
 *   m1, m2           number of block segments / residue rows
 *   k, n             columns of the sparse matrix (unused) / width of B and C
 *   values, column_indices, row_offsets          CSR arrays (device)
 *   row_indices1, row_indices2, row_seg_st_offsets   block_r_ind, residue_r_ind, st_off
 *   B [k x n], C [M x n]   row-major device arrays; C zero-filled by the caller
 *   stream1, stream2 block work / residue work; the caller synchronises both
 * _n32 accepts any n that is a multiple of 32, _n128 any multiple of 64, as the
 * reference's tiles do.  Failures (bad arguments, launch errors) cannot be returned through
 * a void function: they are recorded and can be read with rode_last_error().
 *
 * Rows cut into several segments are summed through a workspace that the library keeps for
 * these entry points: one growable device buffer per (device, stream1, stream2), allocated on
 * the first call on that pair of streams (cudaMalloc) and re-used afterwards.  Calls on the same
 * streams are ordered by them and share the buffer; calls on other streams get buffers of
 * their own and may overlap on the GPU, as with the reference.  Callers that must not
 * allocate at call time pass their own workspace to rode_spmm_f32 / rode_spmm_f64.
 */
#ifndef RODE_B200_RODESPMM_H_
#define RODE_B200_RODESPMM_H_

#include <cuda_runtime.h>

void RoDeSpmm_n32(int m1, int m2, int k, int n,
                  const float *__restrict__ values,
                  const int *__restrict__ column_indices,
                  const int *__restrict__ row_offsets,
                  const int *__restrict__ row_indices1,
                  const int *__restrict__ row_indices2,
                  const int *__restrict__ row_seg_st_offsets,
                  const float *B, float *C,
                  cudaStream_t stream1, cudaStream_t stream2);

void RoDeSpmm_n128(int m1, int m2, int k, int n,
                   const float *__restrict__ values,
                   const int *__restrict__ column_indices,
                   const int *__restrict__ row_offsets,
                   const int *__restrict__ row_indices1,
                   const int *__restrict__ row_indices2,
                   const int *__restrict__ row_seg_st_offsets,
                   const float *B, float *C,
                   cudaStream_t stream1, cudaStream_t stream2);

void RoDeSpmm_n32(int m1, int m2, int k, int n,
                  const double *__restrict__ values,
                  const int *__restrict__ column_indices,
                  const int *__restrict__ row_offsets,
                  const int *__restrict__ row_indices1,
                  const int *__restrict__ row_indices2,
                  const int *__restrict__ row_seg_st_offsets,
                  const double *B, double *C,
                  cudaStream_t stream1, cudaStream_t stream2);

void RoDeSpmm_n128(int m1, int m2, int k, int n,
                   const double *__restrict__ values,
                   const int *__restrict__ column_indices,
                   const int *__restrict__ row_offsets,
                   const int *__restrict__ row_indices1,
                   const int *__restrict__ row_indices2,
                   const int *__restrict__ row_seg_st_offsets,
                   const double *B, double *C,
                   cudaStream_t stream1, cudaStream_t stream2);

#endif /* RODE_B200_RODESPMM_H_ */
