// Collectives fused with the optimizer over NVLink / NVSwitch peer memory.
//
// fused_rs_adamw_ag: ONE kernel that replaces  reduce-scatter(fp32 grads) -> scale -> AdamW on the
// fp32 master shard -> bf16 cast -> all-gather(bf16 params)  of sharded data parallelism:
//
//   for every element i of this rank's shard
//     g  = sum over ranks of full_grad_r[f(i)]      multimem.ld_reduce through the switch (NVLS), or a
//                                                   loop of peer loads when no multicast mapping exists
//     g *= 1 / divide
//     (p, m, v)[i] <- AdamW(p, m, v, g)             local fp32 shard, decoupled weight decay
//     full_r[f(i)] <- bf16(p)  for every rank r     multimem.st (one store, the switch replicates), or
//                                                   a loop of peer stores
//
// f maps a shard offset to the offset of the same element in the param-major full buffers; it is
// affine per chunk and comes from the chunk table.  The kernel contains no waits: the caller
// brackets it with cross-rank barriers on the stream (all ranks' gradients complete before, all
// stores visible after).  The gradient buffers are read-only here; they are cleared by zero_grad.
#include "host_common.cuh"
#include <stdlib.h>
#include <cuda_bf16.h>

namespace {

struct FusedChunk {
  long long shard_off;  // offset into master / m / v
  long long full_off;   // offset of the same elements in the full (param-major) buffers
  int len;              // multiple of 4
  int tensor;
};
struct FusedTensor {
  float lr_mult;
  float wd;
};
constexpr int MAX_PEERS = 8;
struct PeerPtrs {
  const float* grad[MAX_PEERS];
  __nv_bfloat16* full[MAX_PEERS];
};

__device__ __forceinline__ float4 mc_ld_reduce_f32x4(const float* mc_addr) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc_addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void mc_st_b32x2(void* mc_addr, uint32_t a, uint32_t b) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(mc_addr), "f"(__uint_as_float(a)),
               "f"(__uint_as_float(b))
               : "memory");
}

template <bool MC>
__global__ void __launch_bounds__(256)
fused_rs_adamw_ag_kernel(const float* __restrict__ grad_mc, __nv_bfloat16* __restrict__ full_mc, const PeerPtrs peers,
                         int world, float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                         float* __restrict__ shard_grad_out, const FusedChunk* __restrict__ chunks,
                         const FusedTensor* __restrict__ tensors, int nchunks, const float* __restrict__ lr_ptr,
                         float beta1, float beta2, float eps, float bc1, float bc2_sqrt, float inv_divide) {
  for (int ci = blockIdx.x; ci < nchunks; ci += gridDim.x) {
    const FusedChunk ch = chunks[ci];
    const FusedTensor tt = tensors[ch.tensor];
    const float lr = (*lr_ptr) * tt.lr_mult;
    const float decay = 1.f - lr * tt.wd;
    const float step_size = lr / bc1;
    for (int i = threadIdx.x * 4; i < ch.len; i += blockDim.x * 4) {
      const long long si = ch.shard_off + i, fi = ch.full_off + i;
      float4 g;
      if (MC) {
        g = mc_ld_reduce_f32x4(grad_mc + fi);
      } else {
        g = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int r = 0; r < world; ++r) {
          const float4 t = *reinterpret_cast<const float4*>(peers.grad[r] + fi);
          g.x += t.x; g.y += t.y; g.z += t.z; g.w += t.w;
        }
      }
      float gg[4] = {g.x * inv_divide, g.y * inv_divide, g.z * inv_divide, g.w * inv_divide};
      float4 p4 = *reinterpret_cast<float4*>(master + si);
      float4 m4 = *reinterpret_cast<float4*>(m + si);
      float4 v4 = *reinterpret_cast<float4*>(v + si);
      float pp[4] = {p4.x, p4.y, p4.z, p4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        mm[e] = beta1 * mm[e] + (1.f - beta1) * gg[e];
        vv[e] = beta2 * vv[e] + (1.f - beta2) * gg[e] * gg[e];
        pp[e] = pp[e] * decay - step_size * mm[e] / (sqrtf(vv[e]) / bc2_sqrt + eps);
      }
      *reinterpret_cast<float4*>(master + si) = make_float4(pp[0], pp[1], pp[2], pp[3]);
      *reinterpret_cast<float4*>(m + si) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(v + si) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      if (shard_grad_out) *reinterpret_cast<float4*>(shard_grad_out + si) = make_float4(gg[0], gg[1], gg[2], gg[3]);
      __nv_bfloat162 lo = __floats2bfloat162_rn(pp[0], pp[1]), hi = __floats2bfloat162_rn(pp[2], pp[3]);
      const uint32_t a = *reinterpret_cast<uint32_t*>(&lo), b = *reinterpret_cast<uint32_t*>(&hi);
      if (MC) {
        mc_st_b32x2(full_mc + fi, a, b);
      } else {
        for (int r = 0; r < world; ++r) *reinterpret_cast<uint2*>(peers.full[r] + fi) = make_uint2(a, b);
      }
    }
  }
}

// Plain peer-memory all-gather of bf16 shards into every rank's param-major full buffer (used for the
// first gather after initialisation / checkpoint load, when there is no optimizer step to fuse with).
template <bool MC>
__global__ void __launch_bounds__(256)
push_shards_kernel(const float* __restrict__ master, __nv_bfloat16* __restrict__ full_mc, const PeerPtrs peers, int world,
                   const FusedChunk* __restrict__ chunks, int nchunks) {
  for (int ci = blockIdx.x; ci < nchunks; ci += gridDim.x) {
    const FusedChunk ch = chunks[ci];
    for (int i = threadIdx.x * 4; i < ch.len; i += blockDim.x * 4) {
      const float4 p4 = *reinterpret_cast<const float4*>(master + ch.shard_off + i);
      __nv_bfloat162 lo = __floats2bfloat162_rn(p4.x, p4.y), hi = __floats2bfloat162_rn(p4.z, p4.w);
      const uint32_t a = *reinterpret_cast<uint32_t*>(&lo), b = *reinterpret_cast<uint32_t*>(&hi);
      const long long fi = ch.full_off + i;
      if (MC) {
        mc_st_b32x2(full_mc + fi, a, b);
      } else {
        for (int r = 0; r < world; ++r) *reinterpret_cast<uint2*>(peers.full[r] + fi) = make_uint2(a, b);
      }
    }
  }
}

}  // namespace

// grad_mc / full_mc: multicast addresses of the symmetric gradient / parameter buffers (null when
// the system has no multicast support: then peer_grad / peer_full, arrays of `world` device pointers
// given as host arrays, are used).  shard_grad_out (optional) receives the reduced, scaled gradient.
extern "C" int mb_fused_rs_adamw_ag(const float* grad_mc, void* full_mc, const void* const* peer_grad,
                                    void* const* peer_full, int world, float* master, float* m, float* v,
                                    float* shard_grad_out, const void* chunks, const void* tensors, int nchunks,
                                    const float* lr_ptr, float beta1, float beta2, float eps, float bc1,
                                    float bc2_sqrt, float inv_divide, cudaStream_t st) {
  if (nchunks <= 0) return 0;
  if (world > MAX_PEERS) return -3;
  PeerPtrs pp = {};
  for (int r = 0; r < world; ++r) {
    pp.grad[r] = peer_grad ? static_cast<const float*>(peer_grad[r]) : nullptr;
    pp.full[r] = peer_full ? static_cast<__nv_bfloat16*>(peer_full[r]) : nullptr;
  }
  // Blocks per SM of this kernel.  It usually runs on a side stream beside the backward pass's GEMMs, whose persistent
  // CTAs share the SMs with it: fewer resident warps here leave them more issue slots and cache, at the price of
  // fewer peer loads in flight (MB_FUSED_OPT_BLOCKS_PER_SM, default 8).
  static const int per_sm = []() {
    const char* e = getenv("MB_FUSED_OPT_BLOCKS_PER_SM");
    const int v = e ? atoi(e) : 8;
    return v < 1 ? 1 : (v > 8 ? 8 : v);
  }();
  const int cap = mbh::sm_count() * per_sm;
  const int blocks = nchunks < cap ? nchunks : cap;
  if (grad_mc && full_mc)
    fused_rs_adamw_ag_kernel<true><<<blocks, 256, 0, st>>>(
        grad_mc, static_cast<__nv_bfloat16*>(full_mc), pp, world, master, m, v, shard_grad_out,
        static_cast<const FusedChunk*>(chunks), static_cast<const FusedTensor*>(tensors), nchunks, lr_ptr, beta1,
        beta2, eps, bc1, bc2_sqrt, inv_divide);
  else
    fused_rs_adamw_ag_kernel<false><<<blocks, 256, 0, st>>>(
        nullptr, nullptr, pp, world, master, m, v, shard_grad_out, static_cast<const FusedChunk*>(chunks),
        static_cast<const FusedTensor*>(tensors), nchunks, lr_ptr, beta1, beta2, eps, bc1, bc2_sqrt, inv_divide);
  return mbh::check_launch("fused_rs_adamw_ag");
}

extern "C" int mb_push_shards(const float* master, void* full_mc, void* const* peer_full, int world,
                              const void* chunks, int nchunks, cudaStream_t st) {
  if (nchunks <= 0) return 0;
  if (world > MAX_PEERS) return -3;
  PeerPtrs pp = {};
  for (int r = 0; r < world; ++r) pp.full[r] = peer_full ? static_cast<__nv_bfloat16*>(peer_full[r]) : nullptr;
  const int blocks = nchunks < mbh::sm_count() * 8 ? nchunks : mbh::sm_count() * 8;
  if (full_mc)
    push_shards_kernel<true><<<blocks, 256, 0, st>>>(master, static_cast<__nv_bfloat16*>(full_mc), pp, world,
                                                    static_cast<const FusedChunk*>(chunks), nchunks);
  else
    push_shards_kernel<false><<<blocks, 256, 0, st>>>(master, nullptr, pp, world,
                                                     static_cast<const FusedChunk*>(chunks), nchunks);
  return mbh::check_launch("push_shards");
}
