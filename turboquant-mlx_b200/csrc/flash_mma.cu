// Tensor-core flash-decode path (placeholder until the kernel lands).
#include "flash.cuh"
namespace tq {
bool flash_mma_supported(const FlashArgs&) { return false; }
int flash_mma_chunk_multiple() { return 64; }
int launch_flash_mma(const FlashArgs&, int, cudaStream_t) {
  return set_error(TQ_ERR_UNSUPPORTED, "tensor-core flash decode not built");
}
}  // namespace tq
