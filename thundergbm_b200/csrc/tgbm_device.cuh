// Device-side helpers shared by the kernels of the histogram tree builder.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

#include "tgbm_common.h"

namespace tgbm {

#define TGBM_CUDA(call)                                                                                   \
    do {                                                                                                  \
        cudaError_t e_ = (call);                                                                          \
        if (e_ != cudaSuccess)                                                                            \
            throw ::tgbm::Error(std::string("CUDA error: ") + cudaGetErrorString(e_) + " in " #call " at " __FILE__ ":" + \
                                std::to_string(__LINE__));                                                \
    } while (0)

// Device memory of the library's buffers (tgbm_devmem.cu): cudaMalloc / cudaFree semantics on top of a per-device pool
// that keeps released blocks.  dev_trim cuts what the pools hold back to their limit (the C entry points call it when
// they return), dev_release_all gives everything unused back to the driver.
void *dev_alloc(size_t bytes);
void dev_free(void *p) noexcept;
void dev_trim() noexcept;
void dev_release_all() noexcept;
// host -> device copy that also runs at the speed of the link when the source is pageable memory (then it returns
// when the data is on the device; from page-locked memory it is cudaMemcpyAsync on `stream`)
void upload_h2d(void *dst, const void *src, size_t bytes, cudaStream_t stream, int n_threads);
int upload_threads();   // host threads one upload may use: TGBM_UPLOAD_THREADS, else half of the cores, at most 8

// RAII device buffer; everything is allocated once at init and reused for every tree.
template <typename T>
struct DevBuf {
    T *p = nullptr;
    size_t n = 0;
    DevBuf() = default;
    DevBuf(const DevBuf &) = delete;
    DevBuf &operator=(const DevBuf &) = delete;
    ~DevBuf() { release(); }
    void release() {
        if (p) dev_free(p);
        p = nullptr;
        n = 0;
    }
    void alloc(size_t count) {
        release();
        n = count;
        if (count) p = static_cast<T *>(dev_alloc(sizeof(T) * count));
    }
    void zero(cudaStream_t s) {
        if (n) TGBM_CUDA(cudaMemsetAsync(p, 0, sizeof(T) * n, s));
    }
    size_t bytes() const { return sizeof(T) * n; }
};

// ---- portable expf ------------------------------------------------------------------------
// Cody-Waite reduction and a degree-5 polynomial written with explicit IEEE fp32 operations
// only, so that a host restatement of the same lines gives the same bits.  Replaces expf in
// the reference's losses (include/thundergbm/objective/regression_obj.h:144-154,
// src/thundergbm/objective/multiclass_obj.cu:22-28).
__host__ __device__ inline float pow2i(int e) {
    union { uint32_t u; float f; } c;
    c.u = (uint32_t)(e + 127) << 23;
    return c.f;
}
__device__ inline float portable_expf(float x) {
    if (!(x <= 88.72283f)) return x != x ? x : __int_as_float(0x7f800000);
    if (x < -103.9f) return 0.0f;
    float n = rintf(__fmul_rn(x, 1.44269504088896341f));
    float r = __fmaf_rn(n, -0.693359375f, x);
    r = __fmaf_rn(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = __fmaf_rn(p, r, 1.3981999507e-3f);
    p = __fmaf_rn(p, r, 8.3334519073e-3f);
    p = __fmaf_rn(p, r, 4.1665795894e-2f);
    p = __fmaf_rn(p, r, 1.6666665459e-1f);
    p = __fmaf_rn(p, r, 5.0000001201e-1f);
    float e = __fadd_rn(__fmaf_rn(p, __fmul_rn(r, r), r), 1.0f);
    int k = (int)n;
    int k1 = k / 2, k2 = k - k1;
    return __fmul_rn(__fmul_rn(e, pow2i(k1)), pow2i(k2));
}

// counter-based hash: LambdaRank partner sampling and the dither of the gradient quantisation
__host__ __device__ inline uint32_t mix32(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    uint64_t z = ((uint64_t)a << 32 | b) * 0x9E3779B97F4A7C15ull + ((uint64_t)c << 32 | d);
    z ^= z >> 30; z *= 0xBF58476D1CE4E5B9ull;
    z ^= z >> 27; z *= 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (uint32_t)(z >> 32);
}

// (g,h) quantisation grid of one boosting round: v_q = floor(v * scale + dither), scale a power of two
struct QuantInfo {
    double sg, sh;          // 2^s
    double inv_sg, inv_sh;  // 2^-s
};

__device__ inline double pow2d(int e) { return __longlong_as_double((long long)(e + 1023) << 52); }

// exponent e with m < 2^e (0 for m == 0); m >= 0 finite
__device__ inline int exp_above(float m) {
    if (m == 0.f) return 0;
    return ilogbf(m) + 1;
}

__device__ inline float q2f(long long v, double inv_scale) { return __double2float_rn((double)v * inv_scale); }

__device__ inline long long shfl_ll(long long v, int src) {
    int lo = __shfl_sync(0xffffffffu, (int)(v & 0xffffffffll), src);
    int hi = __shfl_sync(0xffffffffu, (int)(v >> 32), src);
    return ((long long)hi << 32) | (unsigned int)lo;
}
__device__ inline long long shfl_up_ll(long long v, int d) {
    int lo = __shfl_up_sync(0xffffffffu, (int)(v & 0xffffffffll), d);
    int hi = __shfl_up_sync(0xffffffffu, (int)(v >> 32), d);
    return ((long long)hi << 32) | (unsigned int)lo;
}
__device__ inline long long shfl_xor_ll(long long v, int m) {
    int lo = __shfl_xor_sync(0xffffffffu, (int)(v & 0xffffffffll), m);
    int hi = __shfl_xor_sync(0xffffffffu, (int)(v >> 32), m);
    return ((long long)hi << 32) | (unsigned int)lo;
}

}  // namespace tgbm
