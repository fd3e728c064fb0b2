// Tensor-core flash decode, overlapping-launch geometry: 4 consumer warps per CTA, up to 4 CTAs per SM.
#define TQ_FLASH_WARPS 4
#define TQ_FLASH_MAX_CTAS 4
#define TQ_GEOM w4
#include "flash_mma_impl.cuh"
