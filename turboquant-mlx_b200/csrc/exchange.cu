// Peer-to-peer exchange of partial attention states between the GPUs of one node
// (sequence-sharded decode): every rank stores its (m, l, acc) block straight into
// the receive slots of all ranks over NVLink and raises a flag there; a rank starts
// its merge once the flags of all ranks show the current epoch.  Plain peer stores
// and system-scope release / acquire only.  The reference runs on one device and has
// no counterpart.
//
// The pushing kernel never waits; the waiting kernel only waits for pushes, so no two
// kernels wait on one another.  The wait is bounded by a time limit on the GPU-wide
// nanosecond timer (tq_set_peer_wait_limit_ms, 2 s unless changed: ordinary host skew
// between ranks must not trip it) and by an iteration count: when it gives up it writes a
// status word and returns; a merge gated on the same flags then writes NaN, and the host
// reads the status at its next synchronisation point.
#include <atomic>

#include "common.cuh"
#include "flash.cuh"

namespace tq {

static std::atomic<unsigned long long> g_wait_limit_ns{2000ull * 1000ull * 1000ull};
unsigned long long peer_wait_limit_ns() { return g_wait_limit_ns.load(); }

namespace {

constexpr int kMaxPeers = 16;

struct PushArgs {
  const uint4* src;
  int64_t n16;                 // 16-byte chunks
  uint4* dst[kMaxPeers];       // peer p: start of the slot that belongs to this rank
  uint32_t* flag[kMaxPeers];   // peer p: flag word that belongs to this rank
  int n_peers;
  uint32_t epoch;
};

__global__ void __launch_bounds__(256) peer_push_kernel(const PushArgs a) {
  const int p = blockIdx.x;
  uint4* dst = a.dst[p];
  for (int64_t i = threadIdx.x; i < a.n16; i += blockDim.x) dst[i] = a.src[i];
  __threadfence_system();      // this thread's stores are visible system-wide before the flag
  __syncthreads();
  if (threadIdx.x == 0)
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.flag[p]), "r"(a.epoch) : "memory");
}

__global__ void peer_wait_kernel(const uint32_t* flags, int n, uint32_t epoch, int* status,
                                 unsigned long long limit_ns) {
  const int i = threadIdx.x;
  if (i >= n) return;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
  for (uint32_t it = 0; it < (1u << 28); ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + i) : "memory");
    if ((int32_t)(v - epoch) >= 0) return;
    __nanosleep(50);
    unsigned long long t1;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
    if (t1 - t0 > limit_ns) break;
  }
  atomicExch(status, 21 + i);   // rank i never arrived
}

}  // namespace
}  // namespace tq

extern "C" int tq_peer_push(const void* src, int64_t nbytes, void* const* peer_dst, void* const* peer_flags,
                            int n_peers, uint32_t epoch, void* stream) {
  using namespace tq;
  TQ_REQUIRE(src && peer_dst && peer_flags, TQ_ERR_BAD_ARG, "tq_peer_push: NULL pointer");
  TQ_REQUIRE(n_peers >= 1 && n_peers <= kMaxPeers, TQ_ERR_BAD_ARG, "tq_peer_push: 1..%d peers, got %d", kMaxPeers,
             n_peers);
  TQ_REQUIRE(nbytes > 0 && nbytes % 16 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0, TQ_ERR_MISALIGNED,
             "tq_peer_push: the block must be a non-empty multiple of 16 bytes at a 16-byte boundary");
  PushArgs a;
  a.src = static_cast<const uint4*>(src);
  a.n16 = nbytes / 16;
  a.n_peers = n_peers;
  a.epoch = epoch;
  for (int p = 0; p < n_peers; ++p) {
    TQ_REQUIRE(peer_dst[p] && peer_flags[p] && (reinterpret_cast<uintptr_t>(peer_dst[p]) & 15) == 0,
               TQ_ERR_MISALIGNED, "tq_peer_push: peer %d has a NULL or misaligned slot", p);
    a.dst[p] = static_cast<uint4*>(peer_dst[p]);
    a.flag[p] = static_cast<uint32_t*>(peer_flags[p]);
  }
  peer_push_kernel<<<n_peers, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return check_launch("tq_peer_push");
}

extern "C" int tq_peer_wait(const void* flags, int n_ranks, uint32_t epoch, int* status, void* stream) {
  using namespace tq;
  TQ_REQUIRE(flags && status, TQ_ERR_BAD_ARG, "tq_peer_wait: NULL pointer");
  TQ_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeers, TQ_ERR_BAD_ARG, "tq_peer_wait: 1..%d ranks, got %d", kMaxPeers,
             n_ranks);
  peer_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint32_t*>(flags), n_ranks,
                                                                    epoch, status, peer_wait_limit_ns());
  return check_launch("tq_peer_wait");
}

extern "C" int tq_set_peer_wait_limit_ms(int ms) {
  const int prev = (int)(tq::g_wait_limit_ns.load() / 1000000ull);
  if (ms > 0) tq::g_wait_limit_ns.store((unsigned long long)ms * 1000000ull);
  return prev;
}
