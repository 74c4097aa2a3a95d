// Column popularity hints for the gathers of SpMM and SDDMM.  No counterpart in the reference.
//
// The kernels gather one dense row per nonzero.  When the dense operand is many times larger
// than the L2 and a small set of columns receives most of the references (power-law graphs),
// an LRU-like L2 lets rows that are touched once push out rows that are touched thousands of
// times.  rode_hot_columns marks the most referenced columns whose dense rows fit a byte
// budget; the compute kernels then load marked rows with the L2 policy evict_last and all
// other rows with evict_first (measured on R-MAT scale 23, N = 128: 27.3 -> 22.1 GB of DRAM
// reads in the block kernel).  Hints change cache residency only, never results.
//
//   count_columns      in-degree of every column (one red.add per nonzero)
//   degree_histogram   columns and references per in-degree (degrees >= kBins-1 share a bin)
//   pick_threshold     smallest in-degree d >= 2 such that the columns of in-degree >= d fit
//                      the budget; decides whether hints are worth using at all
//   mark_hot           one bit per column, plus a trailing flag word (1 = use the hints)
//
// The hints are declared useless (flag 0, the kernels then load every row with the default
// policy) when all touched rows nearly fit the budget anyway, or when the marked columns
// receive less than twice their share of the references (no skew to exploit: pinning an
// arbitrary subset would only shrink the cache for the rest).
#include "rode_common.cuh"

namespace rode {
namespace {

constexpr int kBins = 4096;
constexpr int kThreads = 256;

struct HotState {
    int threshold;  // columns of in-degree >= threshold are hot
    int useful;     // 1: kernels apply the hints
    long long hot_columns;
    long long hot_references;
};

__global__ void __launch_bounds__(kThreads)
count_columns(long long nnz, int n_cols, const int *__restrict__ column_indices, int *__restrict__ degree) {
    const long long stride = static_cast<long long>(gridDim.x) * kThreads;
    for (long long e = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x; e < nnz; e += stride) {
        const int c = ld_stream(column_indices + e);
        if (c >= 0 && c < n_cols) atomicAdd(degree + c, 1);
    }
}

// Histogram in shared memory per CTA (millions of columns share the lowest in-degrees), then
// one pass of global adds per CTA.
__global__ void __launch_bounds__(kThreads)
degree_histogram(int n_cols, const int *__restrict__ degree, unsigned *__restrict__ bin_columns,
                 unsigned *__restrict__ bin_references) {
    __shared__ unsigned s_cols[kBins];
    __shared__ unsigned s_refs[kBins];
    for (int b = threadIdx.x; b < kBins; b += kThreads) {
        s_cols[b] = 0;
        s_refs[b] = 0;
    }
    __syncthreads();
    const int stride = gridDim.x * kThreads;
    for (int c = blockIdx.x * kThreads + threadIdx.x; c < n_cols; c += stride) {
        const int d = degree[c];
        if (d > 0) {
            const int bin = d < kBins - 1 ? d : kBins - 1;
            atomicAdd(s_cols + bin, 1u);
            atomicAdd(s_refs + bin, static_cast<unsigned>(d));
        }
    }
    __syncthreads();
    for (int b = threadIdx.x; b < kBins; b += kThreads) {
        if (s_cols[b]) {
            atomicAdd(bin_columns + b, s_cols[b]);
            atomicAdd(bin_references + b, s_refs[b]);
        }
    }
}

// One CTA.  Walks the bins from the highest in-degree down: whole groups of kGroup bins
// first (their sums come from one thread each), single bins inside the group where the
// budget runs out.
constexpr int kGroup = kBins / kThreads;  // bins per thread
__global__ void __launch_bounds__(kThreads)
pick_threshold(long long max_hot_columns, const unsigned *__restrict__ bin_columns,
               const unsigned *__restrict__ bin_references, HotState *__restrict__ state) {
    __shared__ unsigned s_cols[kBins];
    __shared__ unsigned s_refs[kBins];
    __shared__ long long g_cols[kThreads];
    __shared__ long long g_refs[kThreads];
    long long my_cols = 0, my_refs = 0;
    for (int i = 0; i < kGroup; ++i) {
        const int b = threadIdx.x * kGroup + i;
        s_cols[b] = bin_columns[b];
        s_refs[b] = bin_references[b];
        my_cols += s_cols[b];
        my_refs += s_refs[b];
    }
    g_cols[threadIdx.x] = my_cols;
    g_refs[threadIdx.x] = my_refs;
    __syncthreads();
    if (threadIdx.x != 0) return;
    long long touched = 0, references = 0;  // bin 0 (columns without a reference) is never filled
    for (int t = 0; t < kThreads; ++t) {
        touched += g_cols[t];
        references += g_refs[t];
    }
    long long hot = 0, hot_refs = 0;
    int threshold = kBins;  // nothing hot yet
    bool open = true;
    for (int t = kThreads - 1; t >= 0 && open; --t) {
        if (t > 0 && hot + g_cols[t] <= max_hot_columns) {  // the whole group fits
            hot += g_cols[t];
            hot_refs += g_refs[t];
            threshold = t * kGroup;
            continue;
        }
        for (int b = t * kGroup + kGroup - 1; b >= t * kGroup && b >= 2; --b) {
            if (hot + s_cols[b] > max_hot_columns) {
                open = false;
                break;
            }
            hot += s_cols[b];
            hot_refs += s_refs[b];
            threshold = b;
        }
    }
    // useful: the touched rows do not nearly fit the budget anyway, and the hot columns get
    // at least twice their share of the references
    const bool overflow = 2 * touched > 3 * max_hot_columns;
    const bool skewed = hot > 0 && static_cast<double>(hot_refs) * static_cast<double>(touched) >=
                                       2.0 * static_cast<double>(hot) * static_cast<double>(references);
    state->threshold = threshold;
    state->useful = (overflow && skewed) ? 1 : 0;
    state->hot_columns = hot;
    state->hot_references = hot_refs;
}

// A warp turns 1024 columns into 32 words: lane j tests column base + 32 i + j, the ballot is
// word i.
__global__ void __launch_bounds__(kThreads)
mark_hot(int n_cols, const int *__restrict__ degree, const HotState *__restrict__ state,
         unsigned *__restrict__ hot_columns) {
    const int threshold = state->threshold;
    const int n_words = (n_cols + 31) / 32;
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * kThreads + threadIdx.x) >> 5;
    const int n_warps = (gridDim.x * kThreads) >> 5;
    for (int w0 = warp * 32; w0 < n_words; w0 += n_warps * 32) {
        unsigned mine = 0;
#pragma unroll 4
        for (int i = 0; i < 32; ++i) {
            const long long c = (static_cast<long long>(w0) + i) * 32 + lane;
            const bool hot = c < n_cols && degree[c] >= threshold;
            const unsigned word = __ballot_sync(0xffffffffu, hot);
            if (i == lane) mine = word;
        }
        if (w0 + lane < n_words) hot_columns[w0 + lane] = mine;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) hot_columns[n_words] = state->useful ? 1u : 0u;
}

size_t counters_bytes(int n_cols) {
    // degree[n_cols], then the two histograms and the state, each 256-byte aligned
    const size_t deg = (static_cast<size_t>(n_cols) * sizeof(int) + 255) / 256 * 256;
    return deg + 2 * kBins * sizeof(unsigned) + 256;
}

}  // namespace
}  // namespace rode

extern "C" {

int rode_hot_columns_workspace_bytes(int n_cols, size_t *bytes) {
    if (bytes == nullptr || n_cols < 0)
        return rode::fail(RODE_ERR_INVALID_ARGUMENT, "hot_columns_workspace_bytes: bad argument");
    *bytes = rode::counters_bytes(n_cols);
    return RODE_OK;
}

int rode_hot_columns_words(int n_cols, size_t *words) {
    if (words == nullptr || n_cols < 0) return rode::fail(RODE_ERR_INVALID_ARGUMENT, "hot_columns_words: bad argument");
    *words = (static_cast<size_t>(n_cols) + 31) / 32 + 1;
    return RODE_OK;
}

int rode_hot_columns(long long nnz, int n_cols, const int *column_indices, size_t dense_row_bytes,
                     size_t budget_bytes, unsigned *hot_columns, void *workspace, size_t workspace_bytes,
                     rode_stream_t stream) {
    using namespace rode;
    if (nnz < 0 || n_cols < 0 || dense_row_bytes == 0)
        return fail(RODE_ERR_INVALID_ARGUMENT, "hot_columns: nnz, n_cols >= 0 and dense_row_bytes > 0 required");
    if (hot_columns == nullptr || (nnz > 0 && column_indices == nullptr))
        return fail(RODE_ERR_INVALID_ARGUMENT, "hot_columns: null array");
    const size_t need = counters_bytes(n_cols);
    if (workspace == nullptr || workspace_bytes < need)
        return fail(RODE_ERR_WORKSPACE, "hot_columns: workspace of %zu bytes needed, %zu given", need,
                    workspace ? workspace_bytes : static_cast<size_t>(0));
    if (!aligned_to(workspace, 256)) return fail(RODE_ERR_WORKSPACE, "hot_columns: workspace must be 256-byte aligned");
    if (budget_bytes == 0) {  // default: 60 % of this device's L2
        int dev = 0, l2 = 0;
        RODE_CUDA_TRY(cudaGetDevice(&dev));
        RODE_CUDA_TRY(cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev));
        budget_bytes = static_cast<size_t>(l2) / 10 * 6;
    }
    const long long max_hot = static_cast<long long>(budget_bytes / dense_row_bytes);

    char *base = static_cast<char *>(workspace);
    int *degree = reinterpret_cast<int *>(base);
    const size_t deg_bytes = (static_cast<size_t>(n_cols) * sizeof(int) + 255) / 256 * 256;
    unsigned *bin_columns = reinterpret_cast<unsigned *>(base + deg_bytes);
    unsigned *bin_references = bin_columns + kBins;
    HotState *state = reinterpret_cast<HotState *>(bin_references + kBins);
    RODE_CUDA_TRY(cudaMemsetAsync(workspace, 0, need, stream));

    const int resident = 8 * sm_count();
    if (nnz > 0) {
        const long long want = (nnz + kThreads - 1) / kThreads;
        count_columns<<<static_cast<unsigned>(want < resident ? want : resident), kThreads, 0, stream>>>(
            nnz, n_cols, column_indices, degree);
        RODE_CHECK_LAUNCH("rode::count_columns");
    }
    if (n_cols > 0) {
        const int want = (n_cols + kThreads - 1) / kThreads;
        degree_histogram<<<want < resident ? want : resident, kThreads, 0, stream>>>(n_cols, degree, bin_columns,
                                                                                    bin_references);
        RODE_CHECK_LAUNCH("rode::degree_histogram");
    }
    pick_threshold<<<1, kThreads, 0, stream>>>(max_hot, bin_columns, bin_references, state);
    RODE_CHECK_LAUNCH("rode::pick_threshold");
    {
        const int n_words = (n_cols + 31) / 32;
        const int warps = (n_words + 31) / 32;  // a warp writes 32 words per step
        const int want = warps > 0 ? (warps + kThreads / 32 - 1) / (kThreads / 32) : 1;
        mark_hot<<<want < resident ? want : resident, kThreads, 0, stream>>>(n_cols, degree, state, hot_columns);
        RODE_CHECK_LAUNCH("rode::mark_hot");
    }
    return RODE_OK;
}

}  // extern "C"
