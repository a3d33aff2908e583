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

// Cross-GPU barrier over a table of per-rank signal pads that every rank can address.  Rank `me` stores the
// epoch into slot [base + me] of every rank's pad and then waits until slot [base + p] of its own pad has reached
// the epoch for every p.  Epochs only grow, so the pads never need clearing between barriers.  The release store
// after a system-scope fence publishes everything earlier kernels of this stream wrote (to local or peer memory);
// the acquire loads order the peers' writes before the kernels that follow on this stream.  Plain peer loads and
// stores only; every wait gives up at the deadline and records ERR_WAIT_PEER.
constexpr int BARRIER_MAX_RANKS = 64;
struct PadTable {
  int* pad[BARRIER_MAX_RANKS];
};

__global__ void symm_barrier_kernel(const PadTable pads, int world, int me, int base, int epoch,
                                    unsigned long long timeout_ns, int* status) {
  const int p = threadIdx.x;
  if (p < world) {
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(pads.pad[p] + base + me), "r"(epoch) : "memory");
    if (!wait_flag_bounded(pads.pad[me] + base + p, epoch, timeout_ns)) atomicCAS(status, 0, ERR_WAIT_PEER);
  }
}

}  // namespace

// Stream-ordered barrier over `world` ranks (this one is `me`).  pads[r] is rank r's signal pad as mapped into
// this process; slots [base, base + world) of every pad belong to this barrier channel; `epoch` must be the same
// on every rank and larger than in the previous call on this channel.  timeout_ms is clamped to 10 minutes.
extern "C" int mb_symm_barrier(void* const* pads, int world, int me, int base, int epoch, float timeout_ms,
                               cudaStream_t st) {
  int* status = mbh::status().dev;
  if (!status) return -4;
  if (world < 1 || world > BARRIER_MAX_RANKS || me < 0 || me >= world) return -3;
  PadTable t;
  for (int r = 0; r < world; ++r) t.pad[r] = static_cast<int*>(pads[r]);
  if (timeout_ms < 1.f) timeout_ms = 1.f;
  if (timeout_ms > 600000.f) timeout_ms = 600000.f;
  symm_barrier_kernel<<<1, BARRIER_MAX_RANKS, 0, st>>>(t, world, me, base, epoch,
                                                       static_cast<unsigned long long>(timeout_ms * 1e6), status);
  return mbh::check_launch("symm_barrier");
}

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
