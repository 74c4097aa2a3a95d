// Shared host/device helpers of librode_b200 (sm_100a only).
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>

#include "rode_b200.h"

namespace rode {

// Thread-local message behind rode_last_error().
char *error_buffer();
int fail(int status, const char *fmt, ...);

#define RODE_CUDA_TRY(expr)                                                                 \
    do {                                                                                    \
        cudaError_t rode_err_ = (expr);                                                     \
        if (rode_err_ != cudaSuccess)                                                       \
            return ::rode::fail(RODE_ERR_CUDA, "%s failed: %s", #expr,                      \
                                cudaGetErrorString(rode_err_));                             \
    } while (0)

// Launch check that does not clear a sticky error and does not synchronise.
#define RODE_CHECK_LAUNCH(what)                                                             \
    do {                                                                                    \
        cudaError_t rode_err_ = cudaPeekAtLastError();                                      \
        if (rode_err_ != cudaSuccess)                                                       \
            return ::rode::fail(RODE_ERR_CUDA, "launch of %s failed: %s", what,             \
                                cudaGetErrorString(rode_err_));                             \
    } while (0)

// RoDe_preprocess without the end sentinel (rode_preprocess.cu); tile_scratch holds
// rode_preprocess_workspace_bytes(M) bytes.
int preprocess_reference_signature(int seg_len, int k_block, int vec_len, int M, const int *row_ptr,
                                   int *block_r_ind, int *st_off, int *residue_r_ind, int *n_blk, int *n_res,
                                   void *tile_scratch);

inline bool aligned_to(const void *p, size_t a) { return (reinterpret_cast<size_t>(p) % a) == 0; }

// ---------------------------------------------------------------------------------------
// Device-side vector types: what one lane loads with a single instruction, 16 bytes
// (LDG.128) or 32 bytes (the 256-bit loads of sm_100), for either scalar type.
struct __align__(32) f32x8 {
    float4 lo, hi;
};
struct __align__(32) f64x4 {
    double2 lo, hi;
};
template <typename T, int kBytes>
struct VecB;
template <>
struct VecB<float, 16> {
    using type = float4;
    static constexpr int kLen = 4;
};
template <>
struct VecB<double, 16> {
    using type = double2;
    static constexpr int kLen = 2;
};
template <>
struct VecB<float, 32> {
    using type = f32x8;
    static constexpr int kLen = 8;
};
template <>
struct VecB<double, 32> {
    using type = f64x4;
    static constexpr int kLen = 4;
};
template <typename T>
using Vec16 = VecB<T, 16>;

#ifdef __CUDACC__

__device__ __forceinline__ float4 vzero(float4 *) { return make_float4(0.f, 0.f, 0.f, 0.f); }
__device__ __forceinline__ double2 vzero(double2 *) { return make_double2(0.0, 0.0); }

__device__ __forceinline__ void vfma(float4 &acc, float s, const float4 &b) {
    acc.x = fmaf(s, b.x, acc.x);
    acc.y = fmaf(s, b.y, acc.y);
    acc.z = fmaf(s, b.z, acc.z);
    acc.w = fmaf(s, b.w, acc.w);
}
__device__ __forceinline__ void vfma(double2 &acc, double s, const double2 &b) {
    acc.x = fma(s, b.x, acc.x);
    acc.y = fma(s, b.y, acc.y);
}

__device__ __forceinline__ float4 vshfl_xor(unsigned mask, const float4 &v, int lane_mask) {
    return make_float4(__shfl_xor_sync(mask, v.x, lane_mask), __shfl_xor_sync(mask, v.y, lane_mask),
                       __shfl_xor_sync(mask, v.z, lane_mask), __shfl_xor_sync(mask, v.w, lane_mask));
}
__device__ __forceinline__ double2 vshfl_xor(unsigned mask, const double2 &v, int lane_mask) {
    return make_double2(__shfl_xor_sync(mask, v.x, lane_mask), __shfl_xor_sync(mask, v.y, lane_mask));
}
__device__ __forceinline__ void vadd(float4 &a, const float4 &b) {
    a.x += b.x;
    a.y += b.y;
    a.z += b.z;
    a.w += b.w;
}
__device__ __forceinline__ void vadd(double2 &a, const double2 &b) {
    a.x += b.x;
    a.y += b.y;
}

__device__ __forceinline__ f32x8 vzero(f32x8 *) { return {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)}; }
__device__ __forceinline__ f64x4 vzero(f64x4 *) { return {make_double2(0.0, 0.0), make_double2(0.0, 0.0)}; }
__device__ __forceinline__ void vfma(f32x8 &acc, float s, const f32x8 &b) {
    vfma(acc.lo, s, b.lo);
    vfma(acc.hi, s, b.hi);
}
__device__ __forceinline__ void vfma(f64x4 &acc, double s, const f64x4 &b) {
    vfma(acc.lo, s, b.lo);
    vfma(acc.hi, s, b.hi);
}
__device__ __forceinline__ f32x8 vshfl_xor(unsigned mask, const f32x8 &v, int lane_mask) {
    return {vshfl_xor(mask, v.lo, lane_mask), vshfl_xor(mask, v.hi, lane_mask)};
}
__device__ __forceinline__ f64x4 vshfl_xor(unsigned mask, const f64x4 &v, int lane_mask) {
    return {vshfl_xor(mask, v.lo, lane_mask), vshfl_xor(mask, v.hi, lane_mask)};
}
__device__ __forceinline__ void vadd(f32x8 &a, const f32x8 &b) {
    vadd(a.lo, b.lo);
    vadd(a.hi, b.hi);
}
__device__ __forceinline__ void vadd(f64x4 &a, const f64x4 &b) {
    vadd(a.lo, b.lo);
    vadd(a.hi, b.hi);
}

// Read-only gather of a dense-operand vector: cached in L1 and L2 (rows are re-used by
// neighbouring rows of the sparse matrix).
template <typename V>
__device__ __forceinline__ V ld_dense(const V *p) {
    return __ldg(p);
}
// 256-bit read-only loads (sm_100): one instruction and one address per 32 bytes.
__device__ __forceinline__ f32x8 ld_dense(const f32x8 *p) {
    f32x8 v;
    asm("ld.global.nc.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=f"(v.lo.x), "=f"(v.lo.y), "=f"(v.lo.z), "=f"(v.lo.w), "=f"(v.hi.x), "=f"(v.hi.y), "=f"(v.hi.z),
          "=f"(v.hi.w)
        : "l"(p));
    return v;
}
__device__ __forceinline__ f64x4 ld_dense(const f64x4 *p) {
    f64x4 v;
    asm("ld.global.nc.v4.f64 {%0, %1, %2, %3}, [%4];"
        : "=d"(v.lo.x), "=d"(v.lo.y), "=d"(v.hi.x), "=d"(v.hi.y)
        : "l"(p));
    return v;
}

// Gathers steered by column popularity (rode_hot_columns): rows of marked columns are loaded
// with the L2 policy evict_last, all others with evict_first, so that rows touched once do
// not push the popular rows out of the L2.  A column index carries its mark in bit 31.
struct GatherPolicy {
    unsigned long long hot, cold;
};
// steer = false (the bitmap's flag word says that marks would not help on this matrix): both
// classes of rows get the normal priority, i.e. the kernel behaves like the unhinted one.
__device__ __forceinline__ GatherPolicy make_gather_policy(bool steer) {
    GatherPolicy p;
    unsigned long long normal;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p.hot));
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p.cold));
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(normal));
    if (!steer) p.hot = p.cold = normal;
    return p;
}
__device__ __forceinline__ float4 ld_dense_policy(const float4 *p, unsigned long long policy) {
    float4 v;
    asm("ld.global.nc.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %5;"
        : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
        : "l"(p), "l"(policy));
    return v;
}
__device__ __forceinline__ double2 ld_dense_policy(const double2 *p, unsigned long long policy) {
    double2 v;
    asm("ld.global.nc.L2::cache_hint.v2.f64 {%0, %1}, [%2], %3;" : "=d"(v.x), "=d"(v.y) : "l"(p), "l"(policy));
    return v;
}
__device__ __forceinline__ f32x8 ld_dense_policy(const f32x8 *p, unsigned long long policy) {
    f32x8 v;
    asm("ld.global.nc.L2::cache_hint.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8], %9;"
        : "=f"(v.lo.x), "=f"(v.lo.y), "=f"(v.lo.z), "=f"(v.lo.w), "=f"(v.hi.x), "=f"(v.hi.y), "=f"(v.hi.z),
          "=f"(v.hi.w)
        : "l"(p), "l"(policy));
    return v;
}
__device__ __forceinline__ f64x4 ld_dense_policy(const f64x4 *p, unsigned long long policy) {
    f64x4 v;
    asm("ld.global.nc.L2::cache_hint.v4.f64 {%0, %1, %2, %3}, [%4], %5;"
        : "=d"(v.lo.x), "=d"(v.lo.y), "=d"(v.hi.x), "=d"(v.hi.y)
        : "l"(p), "l"(policy));
    return v;
}
// Word of the popularity bitmap that holds column c, and c with its mark moved into bit 31.
__device__ __forceinline__ unsigned hot_word(const unsigned *hot, int c) { return __ldg(hot + (c >> 5)); }
__device__ __forceinline__ int tag_hot(int c, unsigned word) {
    return c | static_cast<int>(((word >> (c & 31)) & 1u) << 31);
}
// Where the dense row of column c (0 <= c < 2^31) starts, seen from a lane's base pointer: one
// 32 x 32 -> 64 bit multiply by the row's byte length instead of 64-bit index arithmetic per gather.
template <typename V>
__device__ __forceinline__ const V *dense_row(const V *lane_base, unsigned c, unsigned row_bytes) {
    return reinterpret_cast<const V *>(reinterpret_cast<const char *>(lane_base) +
                                       static_cast<unsigned long long>(c) * row_bytes);
}
// Gather of the dense-row vector of a column: plain read-only load, or steered by the mark.
template <bool kHints, typename V>
__device__ __forceinline__ V gather(const V *lane_base, int c, unsigned row_bytes, const GatherPolicy &policy) {
    if constexpr (kHints) {
        return ld_dense_policy(dense_row(lane_base, static_cast<unsigned>(c) & 0x7fffffffu, row_bytes),
                               c < 0 ? policy.hot : policy.cold);
    } else {
        return ld_dense(dense_row(lane_base, static_cast<unsigned>(c), row_bytes));
    }
}

// U consecutive entries of a shared-memory array, read with 16-byte loads (all lanes of a group
// read the same address: one broadcast wavefront per load, against one per element with shuffles).
template <int U>
__device__ __forceinline__ void ld_shared_run(const int *p, int (&out)[U]) {
    static_assert(U % 4 == 0, "runs of four");
#pragma unroll
    for (int u = 0; u < U; u += 4) {
        const int4 x = *reinterpret_cast<const int4 *>(p + u);
        out[u] = x.x;
        out[u + 1] = x.y;
        out[u + 2] = x.z;
        out[u + 3] = x.w;
    }
}
template <int U>
__device__ __forceinline__ void ld_shared_run(const float *p, float (&out)[U]) {
    static_assert(U % 4 == 0, "runs of four");
#pragma unroll
    for (int u = 0; u < U; u += 4) {
        const float4 x = *reinterpret_cast<const float4 *>(p + u);
        out[u] = x.x;
        out[u + 1] = x.y;
        out[u + 2] = x.z;
        out[u + 3] = x.w;
    }
}
template <int U>
__device__ __forceinline__ void ld_shared_run(const double *p, double (&out)[U]) {
    static_assert(U % 2 == 0, "runs of two");
#pragma unroll
    for (int u = 0; u < U; u += 2) {
        const double2 x = *reinterpret_cast<const double2 *>(p + u);
        out[u] = x.x;
        out[u + 1] = x.y;
    }
}

// Streaming read of CSR data (touched once): do not let it displace dense rows in L1.
__device__ __forceinline__ int ld_stream(const int *p) { return __ldcs(p); }
__device__ __forceinline__ float ld_stream(const float *p) { return __ldcs(p); }
__device__ __forceinline__ double ld_stream(const double *p) { return __ldcs(p); }

// Streaming store of results (written once, not read again by this kernel).
template <typename V>
__device__ __forceinline__ void st_stream(V *p, const V &v) {
    __stcs(p, v);
}
__device__ __forceinline__ void st_stream(f32x8 *p, const f32x8 &v) {
    __stcs(reinterpret_cast<float4 *>(p), v.lo);
    __stcs(reinterpret_cast<float4 *>(p) + 1, v.hi);
}
__device__ __forceinline__ void st_stream(f64x4 *p, const f64x4 &v) {
    __stcs(reinterpret_cast<double2 *>(p), v.lo);
    __stcs(reinterpret_cast<double2 *>(p) + 1, v.hi);
}

// Lane mask of the L-lane group that `lane` belongs to (L a power of two <= 32).
template <int L>
__device__ __forceinline__ unsigned group_mask(int lane) {
    if constexpr (L == 32) {
        return 0xffffffffu;
    } else {
        return ((1u << L) - 1u) << (lane & ~(L - 1));
    }
}

#endif  // __CUDACC__

// Number of SMs of the current device (looked up once per device; 148 if the query fails).
inline int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cached[dev] = v;
    }
    return cached[dev];
}

}  // namespace rode
