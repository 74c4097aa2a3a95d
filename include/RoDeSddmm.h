/*
 * Drop-in C++ declarations of the reference's SDDMM entry points
 * (Da1sypetals/rode, RoDe_SDDMM/RoDeSddmm.h:4-9), implemented by librode_b200.so as thin
 * wrappers over rode_sddmm_f32 (rode_b200.h).
 *
 *   out[e] = values[e] * dot(lhs_matrix[row(e), 0:k], rhs_matrix[col(e), 0:k])
 *
 * Same argument order and meaning as the reference; _n32 is the K = 32 entry (metadata
 * from seg_len 512), _n128 the K = 128 entry (seg_len 32).  RoDeSDDMM_n64 (K = 64,
 * seg_len 512) has no counterpart in the reference and serves widths it cannot.
 * A null stream means the default stream (the reference skips the kernel instead,
 * RoDe_SDDMM/RoDeSddmm.cu:503,509).  Failures are recorded for rode_last_error().
 */
#ifndef RODE_B200_RODESDDMM_H_
#define RODE_B200_RODESDDMM_H_

#include <cuda_runtime.h>

void RoDeSDDMM_n32(int m1, int m2, int n, int k,
                   const int *__restrict__ row_indices_block,
                   const int *__restrict__ row_indices_residue,
                   const int *__restrict__ st_offsets,
                   const int *__restrict__ row_offsets,
                   const int *__restrict__ column_indices,
                   const float *__restrict__ values,
                   const float *__restrict__ lhs_matrix,
                   const float *__restrict__ rhs_matrix,
                   float *__restrict__ out,
                   cudaStream_t stream1, cudaStream_t stream2);

void RoDeSDDMM_n128(int m1, int m2, int n, int k,
                    const int *__restrict__ row_indices_block,
                    const int *__restrict__ row_indices_residue,
                    const int *__restrict__ st_offsets,
                    const int *__restrict__ row_offsets,
                    const int *__restrict__ column_indices,
                    const float *__restrict__ values,
                    const float *__restrict__ lhs_matrix,
                    const float *__restrict__ rhs_matrix,
                    float *__restrict__ out,
                    cudaStream_t stream1, cudaStream_t stream2);

void RoDeSDDMM_n64(int m1, int m2, int n, int k,
                   const int *__restrict__ row_indices_block,
                   const int *__restrict__ row_indices_residue,
                   const int *__restrict__ st_offsets,
                   const int *__restrict__ row_offsets,
                   const int *__restrict__ column_indices,
                   const float *__restrict__ values,
                   const float *__restrict__ lhs_matrix,
                   const float *__restrict__ rhs_matrix,
                   float *__restrict__ out,
                   cudaStream_t stream1, cudaStream_t stream2);

#endif /* RODE_B200_RODESDDMM_H_ */
