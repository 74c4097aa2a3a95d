// Source-level drop-in check: a C++ program written against the reference's declarations
// (RoDeSpmm.h, RoDeSddmm.h and the RoDe_preprocess* functions it defines without a header)
// compiled against include/ and linked with librode_b200.so instead of the reference's
// RoDeSpmm.cu / RoDeSddmm.cu objects.  It follows the call sequence of the reference's own
// driver (RoDe_SDDMM/main.cu:114-163, 460-533: host preprocessing, upload, entry point on two
// streams, synchronise both, compare with a CPU loop) for SDDMM and does the same for SpMM.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "RoDePreprocess.h"
#include "RoDeSddmm.h"
#include "RoDeSpmm.h"

#define CHECK(call)                                                                          \
    do {                                                                                     \
        cudaError_t e_ = (call);                                                             \
        if (e_ != cudaSuccess) {                                                             \
            std::fprintf(stderr, "CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); \
            return 2;                                                                        \
        }                                                                                    \
    } while (0)

static unsigned g_state = 12345u;
static unsigned next_u32() {  // xorshift, so that the inputs do not depend on a C++ library
    g_state ^= g_state << 13;
    g_state ^= g_state >> 17;
    g_state ^= g_state << 5;
    return g_state;
}
static float next_float() { return static_cast<float>(next_u32() % 20001) / 10000.0f - 1.0f; }

template <typename T>
static T *upload(const std::vector<T> &h) {
    T *d = nullptr;
    if (cudaMalloc(&d, (h.size() + 4) * sizeof(T)) != cudaSuccess) return nullptr;
    cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
    return d;
}

int main() {
    const int m = 700, ncols = 900, width = 32;
    std::vector<int> row_ptr(1, 0), col;
    std::vector<float> val;
    for (int i = 0; i < m; ++i) {
        int len = static_cast<int>(next_u32() % 60);
        if (i % 97 == 0) len = 800;   // rows cut into several segments
        if (i % 13 == 0) len = 0;     // empty rows
        std::vector<char> used(ncols, 0);
        int placed = 0;
        while (placed < len) {
            const int c = static_cast<int>(next_u32() % ncols);
            if (!used[c]) {
                used[c] = 1;
                ++placed;
            }
        }
        for (int c = 0; c < ncols; ++c)
            if (used[c]) {
                col.push_back(c);
                val.push_back(next_float());
            }
        row_ptr.push_back(static_cast<int>(col.size()));
    }
    const int nnz = static_cast<int>(col.size());
    std::vector<float> lhs(static_cast<size_t>(m) * width), rhs(static_cast<size_t>(ncols) * width);
    for (auto &x : lhs) x = next_float();
    for (auto &x : rhs) x = next_float();

    // host preprocessing, as the reference's drivers do
    std::vector<int> blk(nnz / 512 + m + 8), st(nnz / 512 + m + 9), res(m);
    int m1 = 0, m2 = 0;
    RoDe_preprocess_cpu(512, 32, 4, m, row_ptr.data(), blk.data(), st.data(), res.data(), m1, m2);

    int *d_rp = upload(row_ptr), *d_col = upload(col), *d_blk = upload(blk), *d_st = upload(st), *d_res = upload(res);
    float *d_val = upload(val), *d_lhs = upload(lhs), *d_rhs = upload(rhs);
    float *d_out = nullptr, *d_C = nullptr;
    CHECK(cudaMalloc(&d_out, sizeof(float) * (nnz + 4)));
    CHECK(cudaMalloc(&d_C, sizeof(float) * m * width));
    CHECK(cudaMemset(d_out, 0, sizeof(float) * (nnz + 4)));
    CHECK(cudaMemset(d_C, 0, sizeof(float) * m * width));

    // device preprocessing must agree with the host one
    int *d_blk2 = nullptr, *d_st2 = nullptr, *d_res2 = nullptr, *d_cnt = nullptr;
    CHECK(cudaMalloc(&d_blk2, sizeof(int) * blk.size()));
    CHECK(cudaMalloc(&d_st2, sizeof(int) * st.size()));
    CHECK(cudaMalloc(&d_res2, sizeof(int) * m));
    CHECK(cudaMalloc(&d_cnt, 2 * sizeof(int)));
    RoDe_preprocess(512, 32, 4, m, d_rp, d_blk2, d_st2, d_res2, d_cnt, d_cnt + 1);
    int counts[2] = {-1, -1};
    CHECK(cudaMemcpy(counts, d_cnt, sizeof(counts), cudaMemcpyDeviceToHost));
    std::vector<int> blk2(m1 + 1), st2(m1 + 1), res2(m2 + 1);
    CHECK(cudaMemcpy(blk2.data(), d_blk2, sizeof(int) * m1, cudaMemcpyDeviceToHost));
    CHECK(cudaMemcpy(st2.data(), d_st2, sizeof(int) * m1, cudaMemcpyDeviceToHost));
    CHECK(cudaMemcpy(res2.data(), d_res2, sizeof(int) * m2, cudaMemcpyDeviceToHost));
    bool same = counts[0] == m1 && counts[1] == m2;
    for (int i = 0; i < m1 && same; ++i) same = blk2[i] == blk[i] && st2[i] == st[i];
    // (the device version writes no end sentinel st_off[m1], like the reference's)
    for (int i = 0; i < m2 && same; ++i) same = res2[i] == res[i];

    cudaStream_t s1, s2;
    CHECK(cudaStreamCreate(&s1));
    CHECK(cudaStreamCreate(&s2));
    RoDeSDDMM_n32(m1, m2, ncols, width, d_blk, d_res, d_st, d_rp, d_col, d_val, d_lhs, d_rhs, d_out, s1, s2);
    RoDeSpmm_n32(m1, m2, ncols, width, d_val, d_col, d_rp, d_blk, d_res, d_st, d_rhs, d_C, s1, s2);
    // a second SpMM on streams of its own, in flight together with the first: the entry points
    // keep no state that two concurrent calls could share (split rows use library scratch)
    cudaStream_t s3, s4;
    float *d_C2 = nullptr;
    CHECK(cudaStreamCreate(&s3));
    CHECK(cudaStreamCreate(&s4));
    CHECK(cudaMalloc(&d_C2, sizeof(float) * m * width));
    CHECK(cudaMemset(d_C2, 0, sizeof(float) * m * width));
    RoDeSpmm_n32(m1, m2, ncols, width, d_val, d_col, d_rp, d_blk, d_res, d_st, d_rhs, d_C2, s3, s4);
    CHECK(cudaStreamSynchronize(s1));
    CHECK(cudaStreamSynchronize(s2));
    CHECK(cudaStreamSynchronize(s3));
    CHECK(cudaStreamSynchronize(s4));
    CHECK(cudaGetLastError());

    std::vector<float> out(nnz), C(static_cast<size_t>(m) * width);
    CHECK(cudaMemcpy(out.data(), d_out, sizeof(float) * nnz, cudaMemcpyDeviceToHost));
    CHECK(cudaMemcpy(C.data(), d_C, sizeof(float) * m * width, cudaMemcpyDeviceToHost));
    std::vector<float> C2(C.size());
    CHECK(cudaMemcpy(C2.data(), d_C2, sizeof(float) * m * width, cudaMemcpyDeviceToHost));
    bool concurrent_same = true;
    for (size_t i = 0; i < C.size() && concurrent_same; ++i) concurrent_same = C[i] == C2[i];
    double worst_sddmm = 0.0, worst_spmm = 0.0;
    for (int i = 0; i < m; ++i) {
        std::vector<double> acc(width, 0.0);
        for (int e = row_ptr[i]; e < row_ptr[i + 1]; ++e) {
            double dot = 0.0;
            for (int k = 0; k < width; ++k) dot += static_cast<double>(lhs[i * width + k]) * rhs[col[e] * width + k];
            worst_sddmm = std::fmax(worst_sddmm, std::fabs(out[e] - val[e] * dot));
            for (int k = 0; k < width; ++k) acc[k] += static_cast<double>(val[e]) * rhs[col[e] * width + k];
        }
        for (int k = 0; k < width; ++k) worst_spmm = std::fmax(worst_spmm, std::fabs(C[i * width + k] - acc[k]));
    }
    const bool ok = same && concurrent_same && worst_sddmm < 2e-5 && worst_spmm < 2e-4;
    std::printf("%s preprocess_same=%d concurrent_same=%d m1=%d m2=%d nnz=%d max_abs_err sddmm=%.3g spmm=%.3g\n",
                ok ? "PASS" : "FAIL", same ? 1 : 0, concurrent_same ? 1 : 0, m1, m2, nnz, worst_sddmm, worst_spmm);
    return ok ? 0 : 1;
}
