/*
 * kuiper/atomics.h of the runtime shim: fetch-and-add on the four element types the extracted
 * kernels reduce with (FStarLang/kuiper include/kuiper/atomics.h:7-59).  Each returns the value
 * found before the addition.  sm_100a has all four natively.
 */
#ifndef KUIPER_ATOMICS_H
#define KUIPER_ATOMICS_H 1

#include <stdint.h>

__device__ static inline uint32_t atomic_add_u32(uint32_t *p, uint32_t v)
{
    return atomicAdd(reinterpret_cast<unsigned int *>(p), static_cast<unsigned int>(v));
}

__device__ static inline uint64_t atomic_add_u64(uint64_t *p, uint64_t v)
{
    static_assert(sizeof(unsigned long long) == sizeof(uint64_t), "64-bit atomics need a 64-bit unsigned long long");
    return atomicAdd(reinterpret_cast<unsigned long long *>(p), static_cast<unsigned long long>(v));
}

__device__ static inline float atomic_add_f32(float *p, float v) { return atomicAdd(p, v); }

__device__ static inline double atomic_add_f64(double *p, double v) { return atomicAdd(p, v); }

#endif /* KUIPER_ATOMICS_H */
