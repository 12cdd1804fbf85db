/*
 * kuiper/vectorops.h of the runtime shim: the 16-byte vector copy the extracted kernels use to
 * move a pack of elements between global and shared memory (FStarLang/kuiper
 * include/kuiper/vectorops.h:7-12).  Both pointers must be 16-byte aligned.
 */
#ifndef KUIPER_VECTOROPS_H
#define KUIPER_VECTOROPS_H 1

#include <stdint.h>

__device__ static inline void vec_memcpy(void *dst, void *src)
{
    const uint4 pack = *static_cast<const uint4 *>(src);   /* one 128-bit load, one 128-bit store */
    *static_cast<uint4 *>(dst) = pack;
}

#endif /* KUIPER_VECTOROPS_H */
