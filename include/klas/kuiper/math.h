/*
 * kuiper/math.h of the runtime shim: the 16-bit math names the extracted kernels call
 * (FStarLang/kuiper include/kuiper/math.h:22-158): kpr_h<op> on `half`, kpr_bf16<op> on
 * `__nv_bfloat16`.  In device code an operation with a native 16-bit instruction uses it; every
 * other one -- and all of them in host code -- is evaluated in f32 and rounded once.
 * Written as inline functions over two small helpers rather than as macro layers.
 */
#ifndef KUIPER_MATH_H
#define KUIPER_MATH_H 1

#include <math.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>

#define HLF_MIN __float2half(6.10352e-5f)
#define HLF_MAX __float2half(65504.0f)
#define HLF_INFINITY __float2half(INFINITY)

__host__ __device__ static inline half __hrcp(half x) { return __float2half(1.0f / __half2float(x)); }

/* f32 round trips */
__host__ __device__ static inline float klas_shim_f32(half x) { return __half2float(x); }
__host__ __device__ static inline float klas_shim_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__host__ __device__ static inline void klas_shim_round(float v, half *out) { *out = __float2half(v); }
__host__ __device__ static inline void klas_shim_round(float v, __nv_bfloat16 *out) { *out = __float2bfloat16(v); }

#define KLAS_SHIM_VIA_F32_1(NAME, T, F32OP) \
    __host__ __device__ static inline T NAME(T x) { T r; klas_shim_round(F32OP(klas_shim_f32(x)), &r); return r; }
#define KLAS_SHIM_VIA_F32_2(NAME, T, F32OP) \
    __host__ __device__ static inline T NAME(T x, T y) { T r; klas_shim_round(F32OP(klas_shim_f32(x), klas_shim_f32(y)), &r); return r; }
/* native 16-bit instruction in device code, f32 round trip on the host */
#ifdef __CUDA_ARCH__
#define KLAS_SHIM_NATIVE_1(NAME, T, NATIVE, F32OP) __device__ static inline T NAME(T x) { return NATIVE(x); }
#else
#define KLAS_SHIM_NATIVE_1(NAME, T, NATIVE, F32OP) KLAS_SHIM_VIA_F32_1(NAME, T, F32OP)
#endif

/* ---- half ---- */
KLAS_SHIM_NATIVE_1(kpr_hsqrt, half, hsqrt, sqrtf)
KLAS_SHIM_NATIVE_1(kpr_hrsqrt, half, hrsqrt, rsqrtf)
KLAS_SHIM_NATIVE_1(kpr_hsin, half, hsin, sinf)
KLAS_SHIM_NATIVE_1(kpr_hcos, half, hcos, cosf)
KLAS_SHIM_NATIVE_1(kpr_hceil, half, hceil, ceilf)
KLAS_SHIM_NATIVE_1(kpr_hfloor, half, hfloor, floorf)
KLAS_SHIM_NATIVE_1(kpr_hlog2, half, hlog2, log2f)
KLAS_SHIM_NATIVE_1(kpr_hexp2, half, hexp2, exp2f)
KLAS_SHIM_NATIVE_1(kpr_hfabs, half, __habs, fabsf)
KLAS_SHIM_VIA_F32_1(kpr_htan, half, tanf)
KLAS_SHIM_VIA_F32_1(kpr_hasin, half, asinf)
KLAS_SHIM_VIA_F32_1(kpr_hacos, half, acosf)
KLAS_SHIM_VIA_F32_1(kpr_hatan, half, atanf)
KLAS_SHIM_VIA_F32_1(kpr_hsinh, half, sinhf)
KLAS_SHIM_VIA_F32_1(kpr_hcosh, half, coshf)
KLAS_SHIM_VIA_F32_1(kpr_htanh, half, tanhf)
KLAS_SHIM_VIA_F32_1(kpr_hround, half, roundf)
KLAS_SHIM_VIA_F32_1(kpr_herf, half, erff)
KLAS_SHIM_VIA_F32_1(kpr_hlog10, half, log10f)
KLAS_SHIM_VIA_F32_2(kpr_hpow, half, powf)
KLAS_SHIM_VIA_F32_2(kpr_hatan2, half, atan2f)
KLAS_SHIM_VIA_F32_2(kpr_hfmin, half, fminf)
KLAS_SHIM_VIA_F32_2(kpr_hfmax, half, fmaxf)
KLAS_SHIM_VIA_F32_2(kpr_hfmod, half, fmodf)
KLAS_SHIM_VIA_F32_2(kpr_hcopysign, half, copysignf)
__host__ __device__ static inline half kpr_hfma(half x, half y, half z)
{
#ifdef __CUDA_ARCH__
    return __hfma(x, y, z);
#else
    return __float2half(fmaf(__half2float(x), __half2float(y), __half2float(z)));
#endif
}

/* ---- bfloat16 ---- */
KLAS_SHIM_NATIVE_1(kpr_bf16sqrt, __nv_bfloat16, hsqrt, sqrtf)
KLAS_SHIM_NATIVE_1(kpr_bf16rsqrt, __nv_bfloat16, hrsqrt, rsqrtf)
KLAS_SHIM_NATIVE_1(kpr_bf16sin, __nv_bfloat16, hsin, sinf)
KLAS_SHIM_NATIVE_1(kpr_bf16cos, __nv_bfloat16, hcos, cosf)
KLAS_SHIM_NATIVE_1(kpr_bf16ceil, __nv_bfloat16, hceil, ceilf)
KLAS_SHIM_NATIVE_1(kpr_bf16floor, __nv_bfloat16, hfloor, floorf)
KLAS_SHIM_NATIVE_1(kpr_bf16log2, __nv_bfloat16, hlog2, log2f)
KLAS_SHIM_NATIVE_1(kpr_bf16exp2, __nv_bfloat16, hexp2, exp2f)
KLAS_SHIM_NATIVE_1(kpr_bf16fabs, __nv_bfloat16, __habs, fabsf)
KLAS_SHIM_NATIVE_1(kpr_bf16exp, __nv_bfloat16, hexp, expf)
KLAS_SHIM_NATIVE_1(kpr_bf16log, __nv_bfloat16, hlog, logf)
KLAS_SHIM_NATIVE_1(kpr_bf16log10, __nv_bfloat16, hlog10, log10f)
KLAS_SHIM_NATIVE_1(kpr_bf16tanh, __nv_bfloat16, htanh, tanhf)
KLAS_SHIM_VIA_F32_1(kpr_bf16tan, __nv_bfloat16, tanf)
KLAS_SHIM_VIA_F32_1(kpr_bf16asin, __nv_bfloat16, asinf)
KLAS_SHIM_VIA_F32_1(kpr_bf16acos, __nv_bfloat16, acosf)
KLAS_SHIM_VIA_F32_1(kpr_bf16atan, __nv_bfloat16, atanf)
KLAS_SHIM_VIA_F32_1(kpr_bf16sinh, __nv_bfloat16, sinhf)
KLAS_SHIM_VIA_F32_1(kpr_bf16cosh, __nv_bfloat16, coshf)
KLAS_SHIM_VIA_F32_1(kpr_bf16round, __nv_bfloat16, roundf)
KLAS_SHIM_VIA_F32_1(kpr_bf16erf, __nv_bfloat16, erff)
KLAS_SHIM_VIA_F32_2(kpr_bf16pow, __nv_bfloat16, powf)
KLAS_SHIM_VIA_F32_2(kpr_bf16atan2, __nv_bfloat16, atan2f)
KLAS_SHIM_VIA_F32_2(kpr_bf16fmin, __nv_bfloat16, fminf)
KLAS_SHIM_VIA_F32_2(kpr_bf16fmax, __nv_bfloat16, fmaxf)
KLAS_SHIM_VIA_F32_2(kpr_bf16fmod, __nv_bfloat16, fmodf)
KLAS_SHIM_VIA_F32_2(kpr_bf16copysign, __nv_bfloat16, copysignf)
__host__ __device__ static inline __nv_bfloat16 kpr_bf16fma(__nv_bfloat16 x, __nv_bfloat16 y, __nv_bfloat16 z)
{
#ifdef __CUDA_ARCH__
    return __hfma(x, y, z);
#else
    return __float2bfloat16(fmaf(__bfloat162float(x), __bfloat162float(y), __bfloat162float(z)));
#endif
}
/* The four arithmetic operations, each rounding to bf16 (the reference's bf16 kernels do all
 * their arithmetic through these: dist/Klas_GEMM_BlockTiling2D.cu:193-199). */
__host__ __device__ static inline __nv_bfloat16 kpr_bf16add(__nv_bfloat16 x, __nv_bfloat16 y) { return x + y; }
__host__ __device__ static inline __nv_bfloat16 kpr_bf16sub(__nv_bfloat16 x, __nv_bfloat16 y) { return x - y; }
__host__ __device__ static inline __nv_bfloat16 kpr_bf16mul(__nv_bfloat16 x, __nv_bfloat16 y) { return x * y; }
__host__ __device__ static inline __nv_bfloat16 kpr_bf16div(__nv_bfloat16 x, __nv_bfloat16 y) { return x / y; }

#endif /* KUIPER_MATH_H */
