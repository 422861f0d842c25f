// Shared host/device helpers for the ptb library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "ptb.h"

namespace ptb {

// ---- error reporting -------------------------------------------------------------------------
// The message buffer is thread local, so concurrent host threads do not clobber each other.
char *err_buf();
constexpr int kErrBufLen = 512;

inline int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err_buf(), kErrBufLen, fmt, ap);
    va_end(ap);
    return code;
}

inline int cuda_fail(cudaError_t e, const char *where) {
    snprintf(err_buf(), kErrBufLen, "%s: %s (%d)", where, cudaGetErrorString(e), (int) e);
    return (int) e;
}

#define PTB_REQUIRE(cond, code, ...)                  \
    do {                                              \
        if (!(cond)) return ::ptb::fail((code), __VA_ARGS__); \
    } while (0)

#define PTB_CUDA(expr)                                                \
    do {                                                              \
        cudaError_t _e = (expr);                                      \
        if (_e != cudaSuccess) return ::ptb::cuda_fail(_e, #expr);    \
    } while (0)

#define PTB_LAUNCH_CHECK(name)                                        \
    do {                                                              \
        cudaError_t _e = cudaGetLastError();                          \
        if (_e != cudaSuccess) return ::ptb::cuda_fail(_e, name);     \
    } while (0)

inline bool is_fp8(int dt) { return dt == PTB_E4M3 || dt == PTB_E5M2; }
inline bool is_hp(int dt) { return dt == PTB_F32 || dt == PTB_F16 || dt == PTB_BF16; }
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T> __host__ __device__ inline T cdiv(T a, T b) { return (a + b - 1) / b; }
__host__ __device__ inline int64_t imin(int64_t a, int64_t b) { return a < b ? a : b; }
__host__ __device__ inline int64_t imax(int64_t a, int64_t b) { return a > b ? a : b; }

// ---- device helpers --------------------------------------------------------------------------
template <int FMT> struct Fp8Max;
template <> struct Fp8Max<PTB_E4M3> { static constexpr float v = 448.0f; };
template <> struct Fp8Max<PTB_E5M2> { static constexpr float v = 57344.0f; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// q = cast_rne(clamp(x * scale, -fmax, fmax)).  The multiply is a single fp32 operation (nothing
// to contract it with).  The clamp itself is performed by the conversion: cvt.rn.satfinite maps
// every finite value beyond +-fmax to +-fmax, which is exactly what clamping first would give.
template <int FMT> __device__ __forceinline__ float quant_val(float x, float scale) { return x * scale; }

// two fp32 -> two fp8 bytes (low byte = first value), round-to-nearest-even, finite saturation
template <int FMT> __device__ __forceinline__ uint16_t cvt_fp8x2(float lo, float hi) {
    uint16_t r;
    if constexpr (FMT == PTB_E4M3) {
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(lo), "f"(hi));
    } else {
        asm("cvt.rn.satfinite.e5m2x2.f32 %0, %2, %1;" : "=h"(r) : "f"(lo), "f"(hi));
    }
    return r;
}

template <int FMT> __device__ __forceinline__ uint8_t cvt_fp8(float v) {
    return (uint8_t) (cvt_fp8x2<FMT>(v, 0.0f) & 0xff);
}

template <int FMT> __device__ __forceinline__ float fp8_to_f32(uint8_t b) {
    if constexpr (FMT == PTB_E4M3) {
        __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
        return __half2float(*reinterpret_cast<__half *>(&h));
    } else {
        __half_raw h = __nv_cvt_fp8_to_halfraw(b, __NV_E5M2);
        return __half2float(*reinterpret_cast<__half *>(&h));
    }
}

// scale = fmax / max(amax, eps); scale_inv = 1.0f / scale.  IEEE divisions (__fdiv_rn): the build
// never enables fast-math, and the explicit intrinsic keeps that true under any flag.
template <int FMT>
__device__ __forceinline__ void scale_from_amax(float amax, float eps, float &scale, float &scale_inv) {
    float a   = fmaxf(amax, eps);
    scale     = __fdiv_rn(Fp8Max<FMT>::v, a);
    scale_inv = __fdiv_rn(1.0f, scale);
}

// SwiGLU with routing probability, one element: (up / (1 + exp(-up))) * down * prob in fp32
// (primus_turbo/triton/activation/swiglu_kernel.py:49-55 in the reference).  Every kernel that needs
// the activation calls this one function, so fused and unfused paths agree bit for bit.
__device__ __forceinline__ float swiglu_prob(float up, float down, float prob) {
    const float silu = __fdiv_rn(up, 1.0f + expf(-up));
    return __fmul_rn(__fmul_rn(silu, down), prob);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Dispatch helpers: run `body` with compile-time element type / fp8 format.
#define PTB_SWITCH_HP(dt, T, ...)                                         \
    switch (dt) {                                                         \
    case PTB_F32: { using T = float; __VA_ARGS__; } break;                \
    case PTB_F16: { using T = __half; __VA_ARGS__; } break;               \
    case PTB_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break;       \
    default: return ::ptb::fail(PTB_ERR_ARG, "unsupported high-precision dtype %d", (int) (dt)); \
    }

#define PTB_SWITCH_FP8(dt, FMT, ...)                                      \
    switch (dt) {                                                         \
    case PTB_E4M3: { constexpr int FMT = PTB_E4M3; __VA_ARGS__; } break;  \
    case PTB_E5M2: { constexpr int FMT = PTB_E5M2; __VA_ARGS__; } break;  \
    default: return ::ptb::fail(PTB_ERR_ARG, "unsupported fp8 dtype %d", (int) (dt)); \
    }

} // namespace ptb
