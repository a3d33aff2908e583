// Expert-parallel token exchange over NVLink peer memory: row scatter to, and row gather from, the
// symmetric buffers of the other ranks of the expert-parallel group.
//
// The reference routes tokens with all_to_all_single, whose split sizes must be read back to the
// host (one synchronisation per MoE block, maester/parallelisms/expert_parallel.py:71-133).  Here
// every rank derives, on the device, the destination (rank, row) of each of its routing slots from
// the all-gathered per-expert counts, and
//   * peer_scatter_rows writes each slot's row straight into the destination rank's expert-major,
//     group-padded buffer (dispatch; and the gradient of combine), and
//   * peer_gather_rows reads each slot's row back from there (combine; and the gradient of dispatch).
// One warp moves one row with 128-bit accesses.  Rows whose destination lies outside the buffer
// capacity are dropped (scatter) or read as zeros (gather) and counted in *overflow.  The kernels
// contain no waits; the caller brackets them with stream-ordered cross-rank barriers.
#include "host_common.cuh"
#include <cuda_bf16.h>

namespace {

constexpr int EP_MAX_PEERS = 16;
struct EpPeers {
  __nv_bfloat16* p[EP_MAX_PEERS];
};

__global__ void __launch_bounds__(256) peer_scatter_rows_kernel(const __nv_bfloat16* __restrict__ src, const EpPeers peers,
                                                               const int* __restrict__ dest_rank,
                                                               const int* __restrict__ dest_row, int n, int dim,
                                                               long long cap_rows, int* __restrict__ overflow) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = dim >> 3;
  for (int i = blockIdx.x * 8 + warp; i < n; i += gridDim.x * 8) {
    const int d = dest_rank[i];
    const long long r = dest_row[i];
    if (r < 0 || r >= cap_rows || d < 0 || d >= EP_MAX_PEERS || peers.p[d] == nullptr) {
      if (lane == 0) atomicAdd(overflow, 1);
      continue;
    }
    const uint4* s = reinterpret_cast<const uint4*>(src + static_cast<long long>(i) * dim);
    uint4* t = reinterpret_cast<uint4*>(peers.p[d] + r * dim);
    for (int v = lane; v < nvec; v += 32) t[v] = s[v];
  }
}

__global__ void __launch_bounds__(256) peer_gather_rows_kernel(__nv_bfloat16* __restrict__ dst, const EpPeers peers,
                                                              const int* __restrict__ src_rank,
                                                              const int* __restrict__ src_row, int n, int dim,
                                                              long long cap_rows, int* __restrict__ overflow) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = dim >> 3;
  for (int i = blockIdx.x * 8 + warp; i < n; i += gridDim.x * 8) {
    const int d = src_rank[i];
    const long long r = src_row[i];
    uint4* t = reinterpret_cast<uint4*>(dst + static_cast<long long>(i) * dim);
    if (r < 0 || r >= cap_rows || d < 0 || d >= EP_MAX_PEERS || peers.p[d] == nullptr) {
      if (lane == 0) atomicAdd(overflow, 1);
      for (int v = lane; v < nvec; v += 32) t[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const uint4* s = reinterpret_cast<const uint4*>(peers.p[d] + r * dim);
    for (int v = lane; v < nvec; v += 32) t[v] = s[v];
  }
}

int fill_peers(EpPeers& pp, void* const* peer_ptrs, int world) {
  if (world < 1 || world > EP_MAX_PEERS) return -3;
  for (int r = 0; r < EP_MAX_PEERS; ++r) pp.p[r] = r < world ? static_cast<__nv_bfloat16*>(peer_ptrs[r]) : nullptr;
  return 0;
}

int grid_rows(int n) {
  const int want = (n + 7) / 8;
  const int cap = mbh::sm_count() * 8;
  return want < cap ? (want > 0 ? want : 1) : cap;
}

}  // namespace

// src: [n, dim] bf16 rows of this rank; peer_ptrs[r]: base of rank r's [cap_rows, dim] buffer.
extern "C" int mb_peer_scatter_rows(const void* src, void* const* peer_ptrs, int world, const int* dest_rank,
                                    const int* dest_row, int n, int dim, long long cap_rows, int* overflow,
                                    cudaStream_t st) {
  if (n <= 0) return 0;
  if (dim & 7) return -3;
  EpPeers pp;
  if (int e = fill_peers(pp, peer_ptrs, world)) return e;
  peer_scatter_rows_kernel<<<grid_rows(n), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(src), pp, dest_rank, dest_row,
                                                         n, dim, cap_rows, overflow);
  return mbh::check_launch("peer_scatter_rows");
}

// dst: [n, dim] bf16 rows of this rank, filled from rank src_rank[i]'s buffer row src_row[i].
extern "C" int mb_peer_gather_rows(void* dst, void* const* peer_ptrs, int world, const int* src_rank,
                                   const int* src_row, int n, int dim, long long cap_rows, int* overflow,
                                   cudaStream_t st) {
  if (n <= 0) return 0;
  if (dim & 7) return -3;
  EpPeers pp;
  if (int e = fill_peers(pp, peer_ptrs, world)) return e;
  peer_gather_rows_kernel<<<grid_rows(n), 256, 0, st>>>(static_cast<__nv_bfloat16*>(dst), pp, src_rank, src_row, n, dim,
                                                        cap_rows, overflow);
  return mbh::check_launch("peer_gather_rows");
}
