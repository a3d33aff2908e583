// Bounded wait on a flag in global (possibly peer) memory, and a kernel that exercises it.
//
// Every wait of this library on another party (an mbarrier fed by TMA or by the tensor core, a flag
// written by another GPU) gives up after a time limit, records a code in the host-mapped status word
// and lets the kernel finish; nothing traps and the context stays usable.  wait_flag_probe is the
// smallest kernel with such a wait: it waits until *flag >= expect.  Tests use it to check the whole
// chain "wait expires -> status word -> Python exception -> next launch works" by simply never
// setting the flag; tools use it as a stream-ordered "wait for a peer" with a deadline.
#include "host_common.cuh"
#include "sm100.cuh"

namespace {
using namespace mb;

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// true when *flag >= expect was observed before the deadline
__device__ __forceinline__ bool wait_flag_bounded(const int* flag, int expect, uint64_t timeout_ns) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (ld_acquire_sys(flag) < expect) {
    if ((++spins & 0x3f) == 0) {
      if (globaltimer_ns() - t0 > timeout_ns) return false;
      __nanosleep(200);
    }
  }
  return true;
}

__global__ void wait_flag_probe_kernel(const int* flag, int expect, unsigned long long timeout_ns, int* status,
                                       int* observed) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const bool ok = wait_flag_bounded(flag, expect, timeout_ns);
    if (!ok) atomicCAS(status, 0, ERR_WAIT_PEER);
    if (observed) *observed = ok ? 1 : 0;
  }
}

}  // namespace

// Waits (on the stream) until *flag >= expect or timeout_ms elapses; on expiry the library status becomes
// ERR_WAIT_PEER.  observed (device int, may be null) receives 1 / 0.  timeout_ms is clamped to 10 s.
extern "C" int mb_wait_flag_probe(const int* flag, int expect, float timeout_ms, int* observed, cudaStream_t st) {
  int* status = mbh::status().dev;
  if (!status) return -4;
  if (timeout_ms < 0.f) timeout_ms = 0.f;
  if (timeout_ms > 10000.f) timeout_ms = 10000.f;
  wait_flag_probe_kernel<<<1, 32, 0, st>>>(flag, expect, static_cast<unsigned long long>(timeout_ms * 1e6), status,
                                           observed);
  return mbh::check_launch("wait_flag_probe");
}
