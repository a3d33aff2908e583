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

// ---- token-indexed variants: no intermediate [T*k, dim] tensor in sorted-slot order ------------------------
//
// Slot s = t * k + j is the j-th expert choice of token t.  ep_plan turns the all-gathered per-expert counts
// into the destination (rank, row) of every slot: expert e lives on rank e / n_local; on that rank its group
// starts at the padded sizes of the lower local experts, and inside the group the slots of lower source
// ranks come first, each rank's in its own stable order (inv[s] - first sorted position of e).
constexpr int EP_MAX_E = 256;

__global__ void __launch_bounds__(256)
ep_plan_kernel(const int* __restrict__ allc, int ep, int me, int E, int n_local, const int* __restrict__ idx,
               const int* __restrict__ inv, int n_slots, int align, long long cap, int* __restrict__ slot_rank,
               int* __restrict__ slot_row, int* __restrict__ offs) {
  __shared__ int s_base[EP_MAX_E];   // destination row of this rank's first slot of expert e
  __shared__ int s_start[EP_MAX_E];  // first sorted position of expert e among this rank's slots
  __shared__ int s_pad[EP_MAX_E];
  __shared__ int s_mine[EP_MAX_E];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, before = 0;
    for (int r = 0; r < ep; ++r) {
      const int c = allc[r * E + e];
      tot += c;
      if (r < me) before += c;
    }
    s_pad[e] = (tot + align - 1) / align * align;
    s_mine[e] = allc[me * E + e];
    s_base[e] = before;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      s_start[e] = run;
      run += s_mine[e];
    }
    for (int r = 0; r < ep; ++r) {
      int o = 0;
      for (int l = 0; l < n_local; ++l) {
        const int e = r * n_local + l;
        s_base[e] += o;
        if (r == me && blockIdx.x == 0) offs[l] = static_cast<int>(o < cap ? o : cap);
        o += s_pad[e];
      }
      if (r == me && blockIdx.x == 0) offs[n_local] = static_cast<int>(o < cap ? o : cap);
    }
  }
  __syncthreads();
  for (int s = blockIdx.x * blockDim.x + threadIdx.x; s < n_slots; s += gridDim.x * blockDim.x) {
    const int e = idx[s];
    slot_rank[s] = e / n_local;
    slot_row[s] = s_base[e] + (inv[s] - s_start[e]);
  }
}

// Zero the padding rows of this rank's expert-major buffer: rows [offs[l] + rows of expert l, offs[l + 1]) for every
// local expert l.  The rows in front are overwritten by the dispatch, the rows behind the last group are never read,
// so clearing the whole buffer (twice the balanced load) is not needed.  grid = (n_local, row slices).
__global__ void __launch_bounds__(256)
ep_zero_padding_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ allc, int ep, int me, int E, int n_local,
                       const int* __restrict__ offs, int dim, long long cap) {
  const int l = blockIdx.x;
  int tot = 0;
  for (int r = 0; r < ep; ++r) tot += allc[r * E + me * n_local + l];
  long long lo = static_cast<long long>(offs[l]) + tot, hi = offs[l + 1];
  if (hi > cap) hi = cap;
  const int nvec = dim >> 3;
  const uint4 z = make_uint4(0u, 0u, 0u, 0u);
  for (long long r = lo + blockIdx.y; r < hi; r += gridDim.y) {
    uint4* row = reinterpret_cast<uint4*>(buf + r * dim);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) row[v] = z;
  }
}

__device__ __forceinline__ void ep_unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 p = __bfloat1622float2(h[i]);
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
}
__device__ __forceinline__ uint4 ep_pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}
__device__ __forceinline__ bool ep_valid(const EpPeers& peers, int d, long long r, long long cap_rows) {
  return r >= 0 && r < cap_rows && d >= 0 && d < EP_MAX_PEERS && peers.p[d] != nullptr;
}

// peers[slot_rank[s]][slot_row[s]] = x[s / k] * (slot_scale ? slot_scale[s] : 1): one warp per token
__global__ void __launch_bounds__(256)
peer_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const EpPeers peers, const int* __restrict__ slot_rank,
                     const int* __restrict__ slot_row, const float* __restrict__ slot_scale, int T, int k, int dim,
                     long long cap_rows, int* __restrict__ overflow) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = dim >> 3;
  for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(t) * dim);
    for (int j = 0; j < k; ++j) {
      const long long s = static_cast<long long>(t) * k + j;
      const int d = slot_rank[s];
      const long long r = slot_row[s];
      if (!ep_valid(peers, d, r, cap_rows)) {
        if (lane == 0) atomicAdd(overflow, 1);
        continue;
      }
      uint4* dst = reinterpret_cast<uint4*>(peers.p[d] + r * dim);
      if (slot_scale == nullptr) {
        for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
      } else {
        const float w = slot_scale[s];
        for (int v = lane; v < nvec; v += 32) {
          float f[8];
          ep_unpack8(src[v], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] *= w;
          dst[v] = ep_pack8(f);
        }
      }
    }
  }
}

// out[t] = sum_j peers[slot_rank[t*k+j]][slot_row[t*k+j]] * (slot_scale ? slot_scale[t*k+j] : 1), fp32 accumulation
__global__ void __launch_bounds__(256)
peer_combine_kernel(__nv_bfloat16* __restrict__ out, const EpPeers peers, const int* __restrict__ slot_rank,
                    const int* __restrict__ slot_row, const float* __restrict__ slot_scale, int T, int k, int dim,
                    long long cap_rows, int* __restrict__ overflow) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = dim >> 3;
  for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    const __nv_bfloat16* row[8];
    float w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      row[j] = nullptr;
      w[j] = 1.f;
      if (j < k) {
        const long long s = static_cast<long long>(t) * k + j;
        const int d = slot_rank[s];
        const long long r = slot_row[s];
        if (ep_valid(peers, d, r, cap_rows)) {
          row[j] = peers.p[d] + r * dim;
          if (slot_scale) w[j] = slot_scale[s];
        } else if (lane == 0) {
          atomicAdd(overflow, 1);
        }
      }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(t) * dim);
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (row[j] == nullptr) continue;
        float f[8];
        ep_unpack8(reinterpret_cast<const uint4*>(row[j])[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(f[i], w[j], acc[i]);
      }
      dst[v] = ep_pack8(acc);
    }
  }
}

// d[t*k+j] = <peers[slot_rank[t*k+j]][slot_row[t*k+j]], g[t]>
__global__ void __launch_bounds__(256)
peer_slot_dot_kernel(float* __restrict__ out, const EpPeers peers, const int* __restrict__ slot_rank,
                     const int* __restrict__ slot_row, const __nv_bfloat16* __restrict__ g, int T, int k, int dim,
                     long long cap_rows) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = dim >> 3;
  for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    const uint4* gr = reinterpret_cast<const uint4*>(g + static_cast<long long>(t) * dim);
    for (int j = 0; j < k; ++j) {
      const long long s = static_cast<long long>(t) * k + j;
      const int d = slot_rank[s];
      const long long r = slot_row[s];
      float acc = 0.f;
      if (ep_valid(peers, d, r, cap_rows)) {
        const uint4* br = reinterpret_cast<const uint4*>(peers.p[d] + r * dim);
        for (int v = lane; v < nvec; v += 32) {
          float a[8], b[8];
          ep_unpack8(br[v], a);
          ep_unpack8(gr[v], b);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc = fmaf(a[i], b[i], acc);
        }
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) out[s] = acc;
    }
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

// allc: [ep, E] per-expert slot counts of every rank; idx / inv: [n_slots] expert and sorted position of each
// slot of this rank.  Outputs: slot_rank / slot_row [n_slots], offs [n_local + 1] (padded group offsets of this
// rank's experts, clamped to cap).
extern "C" int mb_ep_plan(const int* allc, int ep, int me, int E, int n_local, const int* idx, const int* inv,
                          int n_slots, int align, long long cap, int* slot_rank, int* slot_row, int* offs,
                          cudaStream_t st) {
  if (E < 1 || E > EP_MAX_E || ep < 1 || ep * n_local != E || me < 0 || me >= ep || align < 1) return -3;
  const int want = (n_slots + 255) / 256;
  const int capb = mbh::sm_count() * 4;
  ep_plan_kernel<<<want < 1 ? 1 : (want < capb ? want : capb), 256, 0, st>>>(allc, ep, me, E, n_local, idx, inv, n_slots,
                                                                            align, cap, slot_rank, slot_row, offs);
  return mbh::check_launch("ep_plan");
}

// buf: this rank's [cap, dim] expert-major buffer; allc / offs as for mb_ep_plan.
extern "C" int mb_ep_zero_padding(void* buf, const int* allc, int ep, int me, int E, int n_local, const int* offs,
                                  int dim, long long cap, cudaStream_t st) {
  if ((dim & 7) || n_local < 1 || ep * n_local != E || me < 0 || me >= ep) return -3;
  ep_zero_padding_kernel<<<dim3(n_local, 32), 256, 0, st>>>(static_cast<__nv_bfloat16*>(buf), allc, ep, me, E, n_local,
                                                            offs, dim, cap);
  return mbh::check_launch("ep_zero_padding");
}

extern "C" int mb_peer_dispatch_rows(const void* x, void* const* peer_ptrs, int world, const int* slot_rank,
                                     const int* slot_row, const float* slot_scale, int T, int k, int dim,
                                     long long cap_rows, int* overflow, cudaStream_t st) {
  if (T <= 0) return 0;
  if ((dim & 7) || k < 1) return -3;
  EpPeers pp;
  if (int e = fill_peers(pp, peer_ptrs, world)) return e;
  peer_dispatch_kernel<<<grid_rows(T), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), pp, slot_rank, slot_row,
                                                     slot_scale, T, k, dim, cap_rows, overflow);
  return mbh::check_launch("peer_dispatch_rows");
}

extern "C" int mb_peer_combine_rows(void* out, void* const* peer_ptrs, int world, const int* slot_rank,
                                    const int* slot_row, const float* slot_scale, int T, int k, int dim,
                                    long long cap_rows, int* overflow, cudaStream_t st) {
  if (T <= 0) return 0;
  if ((dim & 7) || k < 1 || k > 8) return -3;
  EpPeers pp;
  if (int e = fill_peers(pp, peer_ptrs, world)) return e;
  peer_combine_kernel<<<grid_rows(T), 256, 0, st>>>(static_cast<__nv_bfloat16*>(out), pp, slot_rank, slot_row, slot_scale,
                                                    T, k, dim, cap_rows, overflow);
  return mbh::check_launch("peer_combine_rows");
}

extern "C" int mb_peer_slot_dot(float* out, void* const* peer_ptrs, int world, const int* slot_rank,
                                const int* slot_row, const void* g, int T, int k, int dim, long long cap_rows,
                                cudaStream_t st) {
  if (T <= 0) return 0;
  if ((dim & 7) || k < 1) return -3;
  EpPeers pp;
  if (int e = fill_peers(pp, peer_ptrs, world)) return e;
  peer_slot_dot_kernel<<<grid_rows(T), 256, 0, st>>>(out, pp, slot_rank, slot_row, static_cast<const __nv_bfloat16*>(g), T,
                                                     k, dim, cap_rows);
  return mbh::check_launch("peer_slot_dot");
}
