/* Kuiper_GraphDist.h -- prototypes of the reference's all-pairs distance step
 * (FStarLang/kuiper dist/Kuiper_GraphDist.h:6-12), served by libklas_b200.so through the
 * Kuiper_GraphDist compatibility object.  C++ linkage, as in the reference. */
#ifndef Kuiper_GraphDist_H
#define Kuiper_GraphDist_H

#include <kuiper.h>

typedef uint16_t Kuiper_GraphDist_dist;

bool Kuiper_GraphDist_uu___is_D(uint16_t projectee);

/* b <- min(b, a (min,+) a) on size x size device matrices of 16-bit path lengths, 0 = no path. */
void Kuiper_GraphDist_matmul_dist_gpu(uint32_t size, uint16_t *a, uint16_t *b);

#define Kuiper_GraphDist_H_DEFINED
#endif /* Kuiper_GraphDist_H */
