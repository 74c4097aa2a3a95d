// Host side of librode_b200: status reporting, the per-device workspace cache, and the C++
// entry points with the reference's own signatures (RoDeSpmm.h, RoDeSddmm.h,
// RoDePreprocess.h), each a thin wrapper over the C ABI in rode_b200.h.
#include <cstring>
#include <mutex>

#include "RoDePreprocess.h"
#include "RoDeSddmm.h"
#include "RoDeSpmm.h"
#include "rode_common.cuh"

namespace rode {

char *error_buffer() {
    static thread_local char buf[512] = {0};
    return buf;
}

int fail(int status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), 512, fmt, ap);
    va_end(ap);
    return status;
}

namespace {

// Scratch buffers owned by the library for callers of the reference-signature entry points,
// which carry no workspace argument.  One growable buffer per (purpose, device, stream pair):
// calls on the same streams are ordered by them, so they may share a buffer (the SpMM workspace
// is used by the block kernel on stream1 and, for its claim counters, by the residue kernel on
// stream2, hence both streams are part of the key); calls on other streams may overlap on the GPU
// and get buffers of their own, which keeps the entry points re-entrant like the reference's.  At most kMaxScratch buffers are kept; the least recently
// used one is released when a new key arrives.  Growing or releasing calls cudaFree, which
// waits for work that may still use the buffer.
struct Scratch {
    int kind = 0;
    int dev = -1;
    cudaStream_t stream = nullptr;
    cudaStream_t stream2 = nullptr;
    void *ptr = nullptr;
    size_t bytes = 0;
    unsigned long long last_use = 0;
};
constexpr int kMaxScratch = 32;
enum ScratchKind { kSpmmScratch = 0, kPreprocessScratch = 1 };
Scratch g_scratch[kMaxScratch];
unsigned long long g_scratch_clock = 0;
std::mutex g_scratch_mutex;
// Held from the look-up of a library-owned buffer until the kernels that use it are enqueued.
std::mutex g_enqueue_mutex;

int scratch_for(ScratchKind kind, cudaStream_t stream, cudaStream_t stream2, size_t bytes, void **out) {
    *out = nullptr;
    if (bytes == 0) return RODE_OK;
    int dev = 0;
    RODE_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    Scratch *slot = nullptr, *oldest = &g_scratch[0];
    for (Scratch &s : g_scratch) {
        if (s.ptr && s.kind == kind && s.dev == dev && s.stream == stream && s.stream2 == stream2) {
            slot = &s;
            break;
        }
        if (s.ptr == nullptr ? oldest->ptr != nullptr : (oldest->ptr != nullptr && s.last_use < oldest->last_use))
            oldest = &s;  // a free slot wins over any used one; among used ones the oldest
    }
    if (slot == nullptr) {
        slot = oldest;
        if (slot->ptr) {  // evict: the buffer belongs to another device if slot->dev != dev
            int err = cudaSuccess;
            if (slot->dev != dev) err = cudaSetDevice(slot->dev);
            if (err == cudaSuccess) err = cudaFree(slot->ptr);
            if (slot->dev != dev) cudaSetDevice(dev);
            if (err != cudaSuccess)
                return fail(RODE_ERR_CUDA, "scratch: cudaFree failed: %s", cudaGetErrorString(static_cast<cudaError_t>(err)));
        }
        *slot = Scratch();
        slot->kind = kind;
        slot->dev = dev;
        slot->stream = stream;
        slot->stream2 = stream2;
    }
    if (slot->bytes < bytes) {
        if (slot->ptr) RODE_CUDA_TRY(cudaFree(slot->ptr));
        slot->ptr = nullptr;
        slot->bytes = 0;
        const size_t grown = bytes + bytes / 4;  // head-room against repeated regrowth
        RODE_CUDA_TRY(cudaMalloc(&slot->ptr, grown));
        slot->bytes = grown;
    }
    slot->last_use = ++g_scratch_clock;
    *out = slot->ptr;
    return RODE_OK;
}

template <typename T>
void spmm_entry(int tile, int m1, int m2, int k, int n, const T *values, const int *col, const int *row_offsets,
                const int *blk, const int *res, const int *st, const T *B, T *C, cudaStream_t s1,
                cudaStream_t s2) {
    if (n <= 0 || n % tile != 0) {
        fail(RODE_ERR_INVALID_ARGUMENT, "RoDeSpmm: n = %d is not a multiple of the %d-wide tile", n, tile);
        return;
    }
    size_t need = 0;
    if (rode_spmm_workspace_bytes(m1, n, static_cast<int>(sizeof(T)), &need) != RODE_OK) return;
    // Looking the buffer up and enqueueing the kernels that use it is one step: two host threads
    // that call on the same streams must not interleave their launches on the shared buffer.
    std::lock_guard<std::mutex> enqueue(g_enqueue_mutex);
    void *ws = nullptr;
    if (scratch_for(kSpmmScratch, s1, s2, need, &ws) != RODE_OK) return;
    if (sizeof(T) == 4)
        rode_spmm_f32(m1, m2, k, n, reinterpret_cast<const float *>(values), col, row_offsets, blk, res, st,
                      reinterpret_cast<const float *>(B), reinterpret_cast<float *>(C), ws, need, s1, s2);
    else
        rode_spmm_f64(m1, m2, k, n, reinterpret_cast<const double *>(values), col, row_offsets, blk, res, st,
                      reinterpret_cast<const double *>(B), reinterpret_cast<double *>(C), ws, need, s1, s2);
}

}  // namespace
}  // namespace rode

extern "C" const char *rode_last_error(void) { return rode::error_buffer(); }
extern "C" const char *rode_version(void) { return "0.1.0"; }

// ---- reference-signature C++ entry points ---------------------------------------------

void RoDeSpmm_n32(int m1, int m2, int k, int n, const float *__restrict__ values,
                  const int *__restrict__ column_indices, const int *__restrict__ row_offsets,
                  const int *__restrict__ row_indices1, const int *__restrict__ row_indices2,
                  const int *__restrict__ row_seg_st_offsets, const float *B, float *C, cudaStream_t stream1,
                  cudaStream_t stream2) {
    rode::spmm_entry<float>(32, m1, m2, k, n, values, column_indices, row_offsets, row_indices1, row_indices2,
                            row_seg_st_offsets, B, C, stream1, stream2);
}

void RoDeSpmm_n128(int m1, int m2, int k, int n, const float *__restrict__ values,
                   const int *__restrict__ column_indices, const int *__restrict__ row_offsets,
                   const int *__restrict__ row_indices1, const int *__restrict__ row_indices2,
                   const int *__restrict__ row_seg_st_offsets, const float *B, float *C, cudaStream_t stream1,
                   cudaStream_t stream2) {
    rode::spmm_entry<float>(64, m1, m2, k, n, values, column_indices, row_offsets, row_indices1, row_indices2,
                            row_seg_st_offsets, B, C, stream1, stream2);
}

void RoDeSpmm_n32(int m1, int m2, int k, int n, const double *__restrict__ values,
                  const int *__restrict__ column_indices, const int *__restrict__ row_offsets,
                  const int *__restrict__ row_indices1, const int *__restrict__ row_indices2,
                  const int *__restrict__ row_seg_st_offsets, const double *B, double *C, cudaStream_t stream1,
                  cudaStream_t stream2) {
    rode::spmm_entry<double>(32, m1, m2, k, n, values, column_indices, row_offsets, row_indices1, row_indices2,
                             row_seg_st_offsets, B, C, stream1, stream2);
}

void RoDeSpmm_n128(int m1, int m2, int k, int n, const double *__restrict__ values,
                   const int *__restrict__ column_indices, const int *__restrict__ row_offsets,
                   const int *__restrict__ row_indices1, const int *__restrict__ row_indices2,
                   const int *__restrict__ row_seg_st_offsets, const double *B, double *C, cudaStream_t stream1,
                   cudaStream_t stream2) {
    rode::spmm_entry<double>(64, m1, m2, k, n, values, column_indices, row_offsets, row_indices1, row_indices2,
                             row_seg_st_offsets, B, C, stream1, stream2);
}

namespace {
void sddmm_entry(int expect_k, int m1, int m2, int n, int k, const int *blk, const int *res, const int *st,
                 const int *row_offsets, const int *col, const float *values, const float *lhs, const float *rhs,
                 float *out, cudaStream_t s1, cudaStream_t s2) {
    if (k != expect_k) {
        rode::fail(RODE_ERR_INVALID_ARGUMENT, "RoDeSDDMM_n%d called with k = %d", expect_k, k);
        return;
    }
    rode_sddmm_f32(m1, m2, n, k, blk, res, st, row_offsets, col, values, lhs, rhs, out, s1, s2);
}
}  // namespace

void RoDeSDDMM_n32(int m1, int m2, int n, int k, const int *__restrict__ row_indices_block,
                   const int *__restrict__ row_indices_residue, const int *__restrict__ st_offsets,
                   const int *__restrict__ row_offsets, const int *__restrict__ column_indices,
                   const float *__restrict__ values, const float *__restrict__ lhs_matrix,
                   const float *__restrict__ rhs_matrix, float *__restrict__ out, cudaStream_t stream1,
                   cudaStream_t stream2) {
    sddmm_entry(32, m1, m2, n, k, row_indices_block, row_indices_residue, st_offsets, row_offsets, column_indices,
                values, lhs_matrix, rhs_matrix, out, stream1, stream2);
}

void RoDeSDDMM_n64(int m1, int m2, int n, int k, const int *__restrict__ row_indices_block,
                   const int *__restrict__ row_indices_residue, const int *__restrict__ st_offsets,
                   const int *__restrict__ row_offsets, const int *__restrict__ column_indices,
                   const float *__restrict__ values, const float *__restrict__ lhs_matrix,
                   const float *__restrict__ rhs_matrix, float *__restrict__ out, cudaStream_t stream1,
                   cudaStream_t stream2) {
    sddmm_entry(64, m1, m2, n, k, row_indices_block, row_indices_residue, st_offsets, row_offsets, column_indices,
                values, lhs_matrix, rhs_matrix, out, stream1, stream2);
}

void RoDeSDDMM_n128(int m1, int m2, int n, int k, const int *__restrict__ row_indices_block,
                    const int *__restrict__ row_indices_residue, const int *__restrict__ st_offsets,
                    const int *__restrict__ row_offsets, const int *__restrict__ column_indices,
                    const float *__restrict__ values, const float *__restrict__ lhs_matrix,
                    const float *__restrict__ rhs_matrix, float *__restrict__ out, cudaStream_t stream1,
                    cudaStream_t stream2) {
    sddmm_entry(128, m1, m2, n, k, row_indices_block, row_indices_residue, st_offsets, row_offsets,
                column_indices, values, lhs_matrix, rhs_matrix, out, stream1, stream2);
}

void RoDe_preprocess(int N_SEG, int blockX, int vecLen, int M, const int *row_ptr, int *block_r_ind, int *st_off,
                     int *residue_r_ind, int *n_blk, int *n_res) {
    size_t need = 0;
    if (rode_preprocess_workspace_bytes(M, &need) != RODE_OK) return;
    std::lock_guard<std::mutex> enqueue(rode::g_enqueue_mutex);
    void *ws = nullptr;
    if (rode::scratch_for(rode::kPreprocessScratch, nullptr, nullptr, need, &ws) != RODE_OK) return;
    rode::preprocess_reference_signature(N_SEG, blockX, vecLen, M, row_ptr, block_r_ind, st_off, residue_r_ind, n_blk,
                                         n_res, ws);
}

void RoDe_preprocess_cpu(int N_SEG, int blockX, int vecLen, int M, const int *row_ptr, int *block_r_ind,
                         int *st_off, int *residue_r_ind, int &n_blk, int &n_res) {
    rode_preprocess_cpu(N_SEG, blockX, vecLen, M, row_ptr, block_r_ind, st_off, residue_r_ind, &n_blk, &n_res);
}
