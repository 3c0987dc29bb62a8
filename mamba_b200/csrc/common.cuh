// Shared device/host helpers of libmamba_b200: error reporting, dtype loads, scalar math.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mamba_b200.h"

namespace mb200 {

// ---- error text (thread local), set by every failing entry point -------------------------------
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);
// Makes `device` current; checks that it is an sm_100 part.  Returns MB200_OK or an error code.
int enter_device(int device);
int sm_count(int device);
// Raises the dynamic shared-memory limit of `kernel` on `device` (which must be current) to at least `bytes`; the
// runtime is asked once per (kernel, device) and size increase, later calls only consult a small table.
cudaError_t ensure_dynamic_smem(const void *kernel, int bytes, int device);
// The backward scan's status word (0 = no bounded wait of its kernels has ever run out on the current device).
cudaError_t scan_bwd_status(int *status);

#define MB200_CHECK_ARG(cond, ...)                                     \
    do {                                                               \
        if (!(cond)) return ::mb200::fail(MB200_ERR_BAD_ARG, __VA_ARGS__); \
    } while (0)

// Debug aid: with MB200_DEBUG_SYNC=1 in the environment every launch is followed by a device
// synchronisation and a line on stderr, to find which kernel misbehaves.  Off by default.
bool debug_sync();
void debug_after_launch(const char *what);

#define MB200_CHECK_LAUNCH(what)                                                          \
    do {                                                                                  \
        cudaError_t e__ = cudaGetLastError();                                             \
        if (e__ != cudaSuccess)                                                           \
            return ::mb200::fail(MB200_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e__)); \
        if (::mb200::debug_sync()) ::mb200::debug_after_launch(what);                     \
    } while (0)

// ---- dtype helpers ------------------------------------------------------------------------------
template <typename T> struct DType;
template <> struct DType<float> { static constexpr int code = MB200_F32; };
template <> struct DType<__half> { static constexpr int code = MB200_F16; };
template <> struct DType<__nv_bfloat16> { static constexpr int code = MB200_BF16; };

__host__ __device__ inline int dtype_size(int code) { return code == MB200_F32 ? 4 : 2; }

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Element `i` of a tensor whose dtype is only known at run time (uniform branch; small tensors only).
__device__ __forceinline__ float load_any(const void *p, int dtype, int64_t i)
{
    if (dtype == MB200_F32) return static_cast<const float *>(p)[i];
    if (dtype == MB200_BF16) return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
    return __half2float(static_cast<const __half *>(p)[i]);
}
__device__ __forceinline__ void store_any(void *p, int dtype, int64_t i, float v)
{
    if (dtype == MB200_F32) static_cast<float *>(p)[i] = v;
    else if (dtype == MB200_BF16) static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
    else static_cast<__half *>(p)[i] = __float2half_rn(v);
}

// A 16-byte packet of T widened to floats and back.
template <typename T> struct Vec16 {
    static constexpr int N = 16 / sizeof(T);
    uint4 raw;
    __device__ __forceinline__ void load(const T *p) { raw = *reinterpret_cast<const uint4 *>(p); }
    __device__ __forceinline__ void store(T *p) const { *reinterpret_cast<uint4 *>(p) = raw; }
    __device__ __forceinline__ void unpack(float (&f)[N]) const
    {
        const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int i = 0; i < N; ++i) f[i] = to_float(e[i]);
    }
    __device__ __forceinline__ void pack(const float (&f)[N])
    {
        T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
        for (int i = 0; i < N; ++i) e[i] = from_float<T>(f[i]);
    }
};

// ---- scalar math --------------------------------------------------------------------------------
// softplus with the identity branch above 20 that every site of the path uses.
__device__ __forceinline__ float softplus20(float x) { return x <= 20.f ? log1pf(expf(x)) : x; }
__device__ __forceinline__ float silu(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float fast_silu(float z) { return __fdividef(z, 1.f + __expf(-z)); }
__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
constexpr float kLog2e = 1.4426950408889634f;

// softplus for the streaming kernels: max(x, 0) + log1p(t), t = exp(-|x|) in (0, 1], with
// log1p(t) = 2 atanh(s), s = t / (2 + t) in [0, 1/3], summed to s^13 (truncation < 2e-8 relative).
// Two MUFU operations (ex2, rcp) and a dozen FMA-pipe instructions instead of libm's log1pf(expf()),
// accurate to a few fp32 ulp over the whole range; above 20 the correction is below half an ulp,
// so the result equals x as the thresholded definition requires.
__device__ __forceinline__ float fast_softplus20(float x)
{
    const float t = ex2(-fabsf(x) * kLog2e);
    const float s = __fdividef(t, 2.f + t);
    const float s2 = s * s;
    float p = fmaf(s2, 1.f / 13.f, 1.f / 11.f);
    p = fmaf(p, s2, 1.f / 9.f);
    p = fmaf(p, s2, 1.f / 7.f);
    p = fmaf(p, s2, 1.f / 5.f);
    p = fmaf(p, s2, 1.f / 3.f);
    p = fmaf(p, s2, 1.f);
    return fmaf(2.f * s, p, fmaxf(x, 0.f));
}

// softplus for 16-bit inputs and outputs: max(x, 0) + log2(1 + 2^(-|x| log2 e)) ln 2 with the two MUFU functions and
// four FMA-pipe instructions.  Forming 1 + t costs up to 6e-8 absolute, i.e. a relative error of 6e-8 / softplus(x):
// 2e-4 at x = -8, below 1e-5 from x = -5 up.  That is far inside what a 16-bit dt can express, but not good enough
// for fp32 callers, who get fast_softplus20.  Above 20 the correction is below half an ulp, so the result equals x.
__device__ __forceinline__ float softplus20_lowprec(float x)
{
    float l;
    const float t = ex2(-fabsf(x) * kLog2e);
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l) : "f"(1.f + t));
    return fmaf(l, 0.6931471805599453f, fmaxf(x, 0.f));
}

// silu(z) = h + h tanh(h), h = z/2, with the single-MUFU tanh.approx (relative error 2^-11).  For outputs
// that are rounded to bfloat16 (8 significant bits) the approximation stays below the rounding step.
__device__ __forceinline__ float tanh_approx(float x)
{
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float silu_for_bf16(float z)
{
    const float h = 0.5f * z;
    return fmaf(h, tanh_approx(h), h);
}

// ---- packed fp32 pairs (sm_100 f32x2 instructions: one issue slot for two lanes of work) ----------
__device__ __forceinline__ uint64_t pack2(float lo, float hi)
{
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c)
{
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b)
{
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

}  // namespace mb200
