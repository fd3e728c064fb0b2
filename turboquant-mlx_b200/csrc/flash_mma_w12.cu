// Tensor-core flash decode, stand-alone geometry: 12 consumer warps per CTA, one CTA per SM.
#define TQ_FLASH_WARPS 12
#define TQ_FLASH_MAX_CTAS 1
#define TQ_GEOM w12
#include "flash_mma_impl.cuh"
