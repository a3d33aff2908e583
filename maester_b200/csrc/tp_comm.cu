// Tensor-parallel helpers around the GEMM that is fused with a reduce-scatter (gemm_2cta.cu,
// mb_gemm_bf16_rs): the owner-side sum of the per-rank partial slices, optionally fused with the
// residual add that follows every row-parallel linear in a transformer block.
#include "host_common.cuh"
#include <cuda_bf16.h>

namespace {

// out[i] = (res ? res[i] : 0) + sum_r parts[r * n + i]   (fp32 accumulation, 8 elements per thread)
__global__ void __launch_bounds__(256) sum_partials_kernel(const __nv_bfloat16* __restrict__ parts,
                                                          const __nv_bfloat16* __restrict__ res,
                                                          __nv_bfloat16* __restrict__ out, long long n, int world) {
  const long long nvec = n >> 3;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    if (res) {
      uint4 raw = reinterpret_cast<const uint4*>(res)[v];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] = f.x;
        acc[2 * e + 1] = f.y;
      }
    }
    for (int r = 0; r < world; ++r) {
      uint4 raw = reinterpret_cast<const uint4*>(parts + static_cast<long long>(r) * n)[v];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    reinterpret_cast<uint4*>(out)[v] = o;
  }
}

}  // namespace

// parts: [world, n] bf16 (this rank's buffer, one slot per source rank); res: [n] bf16 or null; out: [n] bf16.
extern "C" int mb_sum_partials(const void* parts, const void* res, void* out, long long n, int world,
                               cudaStream_t st) {
  if (n <= 0) return 0;
  if (n & 7) return -3;
  long long blocks = (n / 8 + 255) / 256;
  const long long cap = static_cast<long long>(mbh::sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  sum_partials_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(parts), static_cast<const __nv_bfloat16*>(res),
      static_cast<__nv_bfloat16*>(out), n, world);
  return mbh::check_launch("sum_partials");
}

namespace {

struct TpPeers {
  const __nv_bfloat16* p[8];
};

// out[row, :] = (res ? res[row, :] : 0) + sum over ranks r of peer_r[(row0 + row), :]   for this rank's rows.
// Every rank holds its full [M, N] partial product in a symmetric buffer; the owner of a row block pulls the
// block from all ranks with 512-byte coalesced reads (the efficient NVLink access size) and adds them in fp32.
__global__ void __launch_bounds__(256) pull_sum_kernel(const TpPeers peers, int world, int first,
                                                      const __nv_bfloat16* __restrict__ res,
                                                      __nv_bfloat16* __restrict__ out, long long row0_elems,
                                                      long long n) {
  const long long nvec = n >> 3;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    if (res) {
      uint4 raw = reinterpret_cast<const uint4*>(res)[v];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] = f.x;
        acc[2 * e + 1] = f.y;
      }
    }
    uint4 raw[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)  // issue all peer loads before using any (NVLink latency)
      if (k < world) raw[k] = reinterpret_cast<const uint4*>(peers.p[(first + k) % world] + row0_elems)[v];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (k < world) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[k]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float2 f = __bfloat1622float2(h[e]);
          acc[2 * e] += f.x;
          acc[2 * e + 1] += f.y;
        }
      }
    }
    uint4 o;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
    reinterpret_cast<uint4*>(out)[v] = o;
  }
}

}  // namespace

// peer_ptrs[r]: rank r's [M, N] bf16 partial product (symmetric memory); this rank owns rows
// [my_rank * M / world, (my_rank + 1) * M / world).  out / res: [M / world, N] bf16.
extern "C" int mb_pull_sum(void* const* peer_ptrs, int world, int my_rank, const void* res, void* out,
                           long long rows_per_rank, long long N, cudaStream_t st) {
  const long long n = rows_per_rank * N;
  if (n <= 0) return 0;
  if ((n & 7) || world < 1 || world > 8) return -3;
  TpPeers pp;
  for (int r = 0; r < 8; ++r) pp.p[r] = r < world ? static_cast<const __nv_bfloat16*>(peer_ptrs[r]) : nullptr;
  long long blocks = (n / 8 + 255) / 256;
  const long long cap = static_cast<long long>(mbh::sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  // start with the local copy so that ranks do not all hit the same peer first
  pull_sum_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(pp, world, my_rank, static_cast<const __nv_bfloat16*>(res),
                                                                static_cast<__nv_bfloat16*>(out),
                                                                static_cast<long long>(my_rank) * n, n);
  return mbh::check_launch("pull_sum");
}
