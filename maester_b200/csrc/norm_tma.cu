// RMSNorm forward / backward as bulk-copy pipelines.
//
// The row-per-warp kernels (elementwise.cu) keep one row of loads in flight per warp and reach about half of the
// copy bandwidth.  Here the memory pipeline does not depend on warp scheduling: one thread of a producer warp streams
// tiles of R consecutive rows (contiguous in memory) into a ring of shared-memory stages with untiled bulk copies
// (cp.async.bulk, completion counted on an mbarrier; no tensor map, no multicast), R consumer warps take one row each
// from shared memory, reduce, and store the result rows straight to global memory with 16-byte stores.  One CTA per
// SM, grid-strided over the tiles.  Every wait is bounded: on expiry the CTA records a status code and leaves.
//
//   forward : y = x * rstd * (w | 1 + w) [+ res],  rstd = rsqrt(mean(x^2) + eps)            (x [, res] are staged)
//   backward: dx = rstd * (w' dy - xhat * mean(xhat w' dy)) [+ dres_add],  dw += dy * xhat   (dy, x [, dres_add] staged)
#include "host_common.cuh"
#include "sm100.cuh"
#include <cuda_bf16.h>

namespace {
using namespace mb;

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};
__device__ __forceinline__ void unpack8(const bf16x8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

constexpr int MAX_STAGES = 4;

// NV: 16-byte vectors per lane (D <= NV * 256), R: rows per tile = consumer warps, NS: streams staged per tile
// (forward: x [, res]; backward: dy, x [, dres_add]), STAGES: ring depth.
template <int NV, int R, int NS, int STAGES>
struct Ring {
  uint64_t* full;
  uint64_t* empty;
  unsigned char* data;
  size_t stream_bytes;  // R * D * 2
  __device__ __forceinline__ unsigned char* at(int stage, int stream) const {
    return data + (static_cast<size_t>(stage) * NS + stream) * stream_bytes;
  }
};

template <int NV, int R, int NS, int STAGES>
__device__ __forceinline__ Ring<NV, R, NS, STAGES> ring_setup(unsigned char* smem, int D) {
  Ring<NV, R, NS, STAGES> r;
  r.full = reinterpret_cast<uint64_t*>(smem);
  r.empty = r.full + MAX_STAGES;
  r.data = smem + 128;
  r.stream_bytes = static_cast<size_t>(R) * D * sizeof(__nv_bfloat16);
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&r.full[s], 1);
      mbar_init(&r.empty[s], R);
    }
    mbar_fence_init();
  }
  __syncthreads();
  return r;
}

// Producer loop (one thread): tile t of this CTA goes to stage it % STAGES.
template <int NV, int R, int NS, int STAGES>
__device__ __forceinline__ void produce(const Ring<NV, R, NS, STAGES>& ring, const __nv_bfloat16* const (&src)[3],
                                        int M, int D, int* status) {
  const int ntiles = (M + R - 1) / R;
  int it = 0;
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
    const int s = it % STAGES;
    if (it >= STAGES && !mbar_wait(&ring.empty[s], ((it / STAGES) - 1) & 1)) {
      atomicCAS(status, 0, ERR_WAIT_EMPTY);
      return;
    }
    const int rows = min(R, M - t * R);
    const uint32_t bytes = static_cast<uint32_t>(rows) * D * sizeof(__nv_bfloat16);
    mbar_expect_tx(&ring.full[s], bytes * NS);
    const size_t off = static_cast<size_t>(t) * R * D;
#pragma unroll
    for (int k = 0; k < NS; ++k) bulk_load(ring.at(s, k), src[k] + off, bytes, &ring.full[s]);
  }
}

template <int NV, int R, bool HAS_RES, int STAGES>
__global__ void __launch_bounds__(32 * (R + 1), 1)
    rmsnorm_fwd_tma_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                           const __nv_bfloat16* __restrict__ res, __nv_bfloat16* __restrict__ y,
                           float* __restrict__ rstd_out, int M, int D, float eps, int unit_offset, int* status) {
  constexpr int NS = HAS_RES ? 2 : 1;
  extern __shared__ __align__(128) unsigned char smem[];
  const auto ring = ring_setup<NV, R, NS, STAGES>(smem, D);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == R) {
    if (lane == 0) {
      const __nv_bfloat16* const src[3] = {x, res, nullptr};
      produce<NV, R, NS, STAGES>(ring, src, M, D, status);
    }
    return;
  }
  const int nvec = D >> 3;
  const float off = unit_offset ? 1.f : 0.f;
  bf16x8 wv[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = lane + 32 * i;
    if (w && v < nvec) {
      wv[i] = reinterpret_cast<const bf16x8*>(w)[v];
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) wv[i].v[e] = __floats2bfloat162_rn(1.f - off, 1.f - off);
    }
  }
  const int ntiles = (M + R - 1) / R;
  int it = 0;
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
    const int s = it % STAGES;
    if (!mbar_wait(&ring.full[s], (it / STAGES) & 1)) {
      atomicCAS(status, 0, ERR_WAIT_FULL);
      return;
    }
    const int row = t * R + warp;
    if (row < M) {
      const bf16x8* xs = reinterpret_cast<const bf16x8*>(ring.at(s, 0) + static_cast<size_t>(warp) * D * 2);
      bf16x8 cur[NV];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int v = lane + 32 * i;
        if (v < nvec) {
          cur[i] = xs[v];
          float f[8];
          unpack8(cur[i], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
        }
      }
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / static_cast<float>(D) + eps);
      if (lane == 0 && rstd_out) rstd_out[row] = rstd;
      bf16x8* yr = reinterpret_cast<bf16x8*>(y + static_cast<size_t>(row) * D);
      MB_CHECK_OR(status, row >= 0 && row < M && NV * 256 >= D, continue);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int v = lane + 32 * i;
        if (v < nvec) {
          float f[8], wf[8];
          unpack8(cur[i], f);
          unpack8(wv[i], wf);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = f[e] * rstd * (wf[e] + off);
          if (HAS_RES) {  // rounded to bf16 before the residual add, as separate ops would do
            const bf16x8 yn = pack8(f);
            float g[8], r[8];
            unpack8(yn, g);
            unpack8(reinterpret_cast<const bf16x8*>(ring.at(s, 1) + static_cast<size_t>(warp) * D * 2)[v], r);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = g[e] + r[e];
          }
          yr[v] = pack8(f);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&ring.empty[s]);
  }
}

template <int NV, int R, bool HAS_ADD, int STAGES>
__global__ void __launch_bounds__(32 * (R + 1), 1)
    rmsnorm_bwd_tma_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                           const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                           const __nv_bfloat16* __restrict__ dres_add, __nv_bfloat16* __restrict__ dx,
                           float* __restrict__ dw, int M, int D, int unit_offset, int* status) {
  constexpr int NS = HAS_ADD ? 3 : 2;
  extern __shared__ __align__(128) unsigned char smem[];
  const auto ring = ring_setup<NV, R, NS, STAGES>(smem, D);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == R) {
    if (lane == 0) {
      const __nv_bfloat16* const src[3] = {dy, x, dres_add};
      produce<NV, R, NS, STAGES>(ring, src, M, D, status);
    }
    return;
  }
  const int nvec = D >> 3;
  const float off = unit_offset ? 1.f : 0.f;
  // the weight row is re-read per row (it stays in L1): the registers go to the dw sums instead
  const bf16x8* wr = reinterpret_cast<const bf16x8*>(w);
  float acc[NV][8];  // this lane's columns of dw, summed over the rows this warp sees
#pragma unroll
  for (int i = 0; i < NV; ++i) {
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[i][e] = 0.f;
  }
  const int ntiles = (M + R - 1) / R;
  int it = 0;
  bool ok = true;
  for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
    const int s = it % STAGES;
    if (!mbar_wait(&ring.full[s], (it / STAGES) & 1)) {
      atomicCAS(status, 0, ERR_WAIT_FULL);
      ok = false;
      break;
    }
    const int row = t * R + warp;
    if (row < M) {
      const size_t roff = static_cast<size_t>(warp) * D * 2;
      const bf16x8* gs = reinterpret_cast<const bf16x8*>(ring.at(s, 0) + roff);
      const bf16x8* xs = reinterpret_cast<const bf16x8*>(ring.at(s, 1) + roff);
      const float rstd = rstd_in[row];
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int v = lane + 32 * i;
        if (v < nvec) {
          float g[8], xf[8], wf[8];
          unpack8(gs[v], g);
          unpack8(xs[v], xf);
          if (w) {
            unpack8(wr[v], wf);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) wf[e] = 1.f - off;
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float xh = xf[e] * rstd;
            dot += g[e] * (wf[e] + off) * xh;
            acc[i][e] += g[e] * xh;
          }
        }
      }
      dot = warp_sum(dot) / static_cast<float>(D);
      bf16x8* dxr = reinterpret_cast<bf16x8*>(dx + static_cast<size_t>(row) * D);
#pragma unroll
      for (int i = 0; i < NV; ++i) {   // second pass over the row: from shared memory again, not from registers
        const int v = lane + 32 * i;
        if (v < nvec) {
          float g[8], xf[8], wf[8], o[8];
          unpack8(gs[v], g);
          unpack8(xs[v], xf);
          if (w) {
            unpack8(wr[v], wf);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) wf[e] = 1.f - off;
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = rstd * (g[e] * (wf[e] + off) - xf[e] * rstd * dot);
          if (HAS_ADD) {
            float a[8];
            unpack8(reinterpret_cast<const bf16x8*>(ring.at(s, 2) + roff)[v], a);
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] += a[e];
          }
          dxr[v] = pack8(o);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&ring.empty[s]);
  }
  if (!dw) return;
  // All consumer warps meet here (the producer warp has left; a warp whose wait ran out comes too, so nobody is
  // left waiting).  Every tile has been consumed and no copy is in flight: the ring's memory is free to hold the
  // warps' column sums, which are then added up and sent to global memory with one vector reduction per 4 columns.
  asm volatile("bar.sync 1, %0;" ::"r"(R * 32) : "memory");
  float* part = reinterpret_cast<float*>(ring.data);   // [R][D]
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = lane + 32 * i;
    if (v < nvec) {
      float4* d = reinterpret_cast<float4*>(part + static_cast<size_t>(warp) * D + v * 8);
      d[0] = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
      d[1] = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
  }
  asm volatile("bar.sync 1, %0;" ::"r"(R * 32) : "memory");
  (void)ok;
  for (int c = threadIdx.x; c < (D >> 2); c += R * 32) {
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < R; ++k) {
      const float4 pv = reinterpret_cast<const float4*>(part + static_cast<size_t>(k) * D)[c];
      sum.x += pv.x; sum.y += pv.y; sum.z += pv.z; sum.w += pv.w;
    }
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dw + c * 4), "f"(sum.x), "f"(sum.y),
                 "f"(sum.z), "f"(sum.w)
                 : "memory");
  }
}

size_t ring_bytes(int R, int D, int NS, int stages) {
  return 128 + static_cast<size_t>(stages) * NS * R * D * sizeof(__nv_bfloat16);
}

}  // namespace

// Returns 1 when the shape is outside what these kernels take (the caller then uses the row-per-warp kernels),
// 0 on success, a negative code on a launch error.
extern "C" int mb_rmsnorm_fwd_tma(const void* x, const void* w, const void* res, void* y, float* rstd, int M, int D,
                                  float eps, int unit_offset, cudaStream_t st) {
  const int nv = (D / 8 + 31) / 32;
  if ((D & 7) || nv > 12 || M < 8 * mbh::sm_count()) return 1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (res && (reinterpret_cast<uintptr_t>(res) & 15)) ||
      (reinterpret_cast<uintptr_t>(y) & 15) || (w && (reinterpret_cast<uintptr_t>(w) & 15)))
    return 1;
  int* status = mbh::status().dev;
  if (!status) return -4;
  constexpr int R = 8;
  const int grid = mbh::sm_count();
#define MB_FWD(NV, HAS_RES, STAGES)                                                                                 \
  do {                                                                                                              \
    const size_t smem = ring_bytes(R, D, (HAS_RES) ? 2 : 1, STAGES);                                                \
    if (smem > 220 * 1024) return 1;                                                                                \
    MB_SET_MAX_SMEM_ONCE((rmsnorm_fwd_tma_kernel<NV, R, HAS_RES, STAGES>), 220 * 1024);                             \
    rmsnorm_fwd_tma_kernel<NV, R, HAS_RES, STAGES><<<grid, 32 * (R + 1), smem, st>>>(                               \
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)res, (__nv_bfloat16*)y, rstd, M, D, \
        eps, unit_offset, status);                                                                                  \
  } while (0)
  if (res) {
    if (nv <= 4) MB_FWD(4, true, 4);
    else if (nv <= 8) MB_FWD(8, true, 3);
    else MB_FWD(12, true, 2);
  } else {
    if (nv <= 4) MB_FWD(4, false, 4);
    else if (nv <= 8) MB_FWD(8, false, 4);
    else MB_FWD(12, false, 4);
  }
#undef MB_FWD
  return mbh::check_launch("rmsnorm_fwd_tma");
}

extern "C" int mb_rmsnorm_bwd_tma(const void* dy, const void* x, const void* w, const float* rstd,
                                  const void* dres_add, void* dx, float* dw, int M, int D, int unit_offset,
                                  cudaStream_t st) {
  const int nv = (D / 8 + 31) / 32;
  if ((D & 7) || nv > 12 || M < 8 * mbh::sm_count()) return 1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(dy) & 15) ||
      (dres_add && (reinterpret_cast<uintptr_t>(dres_add) & 15)) || (reinterpret_cast<uintptr_t>(dx) & 15) ||
      (w && (reinterpret_cast<uintptr_t>(w) & 15)) || (dw && (reinterpret_cast<uintptr_t>(dw) & 15)))
    return 1;
  int* status = mbh::status().dev;
  if (!status) return -4;
  const int grid = mbh::sm_count();
#define MB_BWD(NV, R, HAS_ADD, STAGES)                                                                              \
  do {                                                                                                              \
    const size_t smem = ring_bytes(R, D, (HAS_ADD) ? 3 : 2, STAGES);                                                \
    if (smem > 220 * 1024) return 1;                                                                                \
    MB_SET_MAX_SMEM_ONCE((rmsnorm_bwd_tma_kernel<NV, R, HAS_ADD, STAGES>), 220 * 1024);                             \
    rmsnorm_bwd_tma_kernel<NV, R, HAS_ADD, STAGES><<<grid, 32 * (R + 1), smem, st>>>(                               \
        (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd,                           \
        (const __nv_bfloat16*)dres_add, (__nv_bfloat16*)dx, dw, M, D, unit_offset, status);                         \
  } while (0)
  if (dres_add) {
    if (nv <= 4) MB_BWD(4, 8, true, 3);
    else if (nv <= 8) MB_BWD(8, 4, true, 4);
    else MB_BWD(12, 4, true, 3);
  } else {
    if (nv <= 4) MB_BWD(4, 8, false, 4);
    else if (nv <= 8) MB_BWD(8, 8, false, 3);
    else MB_BWD(12, 8, false, 2);
  }
#undef MB_BWD
  return mbh::check_launch("rmsnorm_bwd_tma");
}
