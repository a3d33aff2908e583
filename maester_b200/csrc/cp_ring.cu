// Helpers of ring context parallelism (the attention kernels themselves are unchanged):
//   * peer_copy: pull a contiguous range from another GPU's memory into local memory with plain 16-byte loads
//     and stores (the K / V chunks of a peer cross NVLink once and are then read locally by the attention kernel);
//   * peer_add_bf16: dst += src for a contiguous bf16 range whose source may be peer memory (the owner of a K / V
//     chunk sums the dK / dV contributions that the other ranks left for it);
//   * attn_merge: combine two partial attention results over the same query rows by their log-sum-exp.
// No waits: callers bracket these with cross-rank barriers on the stream.  No TMA, no multicast.
#include "host_common.cuh"
#include "sm100.cuh"
#include <cuda_bf16.h>
#include <math.h>

namespace {

__global__ void __launch_bounds__(256) peer_copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                                       long long n16) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  // four independent 16-byte loads in flight per thread: NVLink latency is a few microseconds
  for (; i + 3 * stride < n16; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a;
    dst[i + stride] = b;
    dst[i + 2 * stride] = c;
    dst[i + 3 * stride] = d;
  }
  for (; i < n16; i += stride) dst[i] = src[i];
}

__global__ void __launch_bounds__(256) peer_add_bf16_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                                           long long n16) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16; i += stride) {
    uint4 a = dst[i];
    const uint4 b = src[i];
    __nv_bfloat162* ah = reinterpret_cast<__nv_bfloat162*>(&a);
    const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = __bfloat1622float2(ah[e]), y = __bfloat1622float2(bh[e]);
      ah[e] = __floats2bfloat162_rn(x.x + y.x, x.y + y.y);
    }
    dst[i] = a;
  }
}

// acc: fp32 [B, S_acc, H, hd] (rows row_off .. row_off + c are updated); lse: fp32 [B, H, S_acc];
// part: bf16 [B, c, H, hd]; lse_part: fp32 [B, H, c].  One warp per (b, row, h).
// init != 0: acc = part, lse = lse_part (first contribution of these rows).
__global__ void __launch_bounds__(256) attn_merge_kernel(float* __restrict__ acc, float* __restrict__ lse,
                                                        const __nv_bfloat16* __restrict__ part,
                                                        const float* __restrict__ lse_part, int B, int c, int H, int hd,
                                                        int S_acc, int row_off, int init) {
  const long long w = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(B) * c * H;
  if (w >= total) return;
  const int h = static_cast<int>(w % H);
  const long long br = w / H;
  const int row = static_cast<int>(br % c);
  const int b = static_cast<int>(br / c);
  const long long li = (static_cast<long long>(b) * H + h) * S_acc + row_off + row;
  const float l1 = lse_part[(static_cast<long long>(b) * H + h) * c + row];
  float w0, w1, ln;
  if (init) {
    w0 = 0.f;
    w1 = 1.f;
    ln = l1;
  } else {
    const float l0 = lse[li];
    const float m = fmaxf(l0, l1);
    if (m == -INFINITY) {  // neither part attends to anything
      w0 = 0.f;
      w1 = 0.f;
      ln = -INFINITY;
    } else {
      const float e0 = __expf(l0 - m), e1 = __expf(l1 - m);
      ln = m + __logf(e0 + e1);
      w0 = e0 / (e0 + e1);
      w1 = e1 / (e0 + e1);
    }
  }
  float* a = acc + ((static_cast<long long>(b) * S_acc + row_off + row) * H + h) * hd;
  const __nv_bfloat16* p = part + ((static_cast<long long>(b) * c + row) * H + h) * hd;
  for (int i = lane * 2; i < hd; i += 64) {
    const float2 pv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + i));
    float2 av = init ? make_float2(0.f, 0.f) : *reinterpret_cast<float2*>(a + i);
    av.x = av.x * w0 + pv.x * w1;
    av.y = av.y * w0 + pv.y * w1;
    *reinterpret_cast<float2*>(a + i) = av;
  }
  if (lane == 0) lse[li] = ln;
}

// One entry per (parameter, source rank) of a sharded block: `len` elements of 2 bytes from offset `src_off` of rank
// `rank`'s shard buffer to offset `dst_off` of the local staging buffer.  All three are multiples of 8 elements.
struct GatherDesc {
  long long dst_off;
  long long src_off;
  long long len;
  long long rank;
};
struct GatherPeers {
  const uint4* base[8];
};

// grid (entries, slices): slice y of an entry's 16-byte words, eight independent loads in flight per thread.
__global__ void __launch_bounds__(256) peer_gather_kernel(uint4* __restrict__ dst, GatherPeers peers,
                                                         const GatherDesc* __restrict__ descs, long long dst_elems,
                                                         int* status) {
  const GatherDesc d = descs[blockIdx.x];
  MB_CHECK_OR(status, d.rank >= 0 && d.rank < 8 && peers.base[d.rank] && d.dst_off >= 0 && d.src_off >= 0 &&
                          d.len >= 0 && !((d.dst_off | d.src_off | d.len) & 7) && d.dst_off + d.len <= dst_elems,
              return);
  const uint4* __restrict__ src = peers.base[d.rank] + (d.src_off >> 3);
  uint4* __restrict__ out = dst + (d.dst_off >> 3);
  const long long n16 = d.len >> 3;
  const long long stride = static_cast<long long>(gridDim.y) * blockDim.x;
  long long i = static_cast<long long>(blockIdx.y) * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], e = src[i + 3 * stride];
    out[i] = a;
    out[i + stride] = b;
    out[i + 2 * stride] = c;
    out[i + 3 * stride] = e;
  }
  for (; i < n16; i += stride) out[i] = src[i];
}

int copy_grid(long long n16) {
  long long blocks = (n16 + 256 * 4 - 1) / (256 * 4);
  const long long cap = static_cast<long long>(mbh::sm_count());  // one light block per SM beside the attention CTAs
  if (blocks > cap) blocks = cap;
  return static_cast<int>(blocks < 1 ? 1 : blocks);
}

}  // namespace

// dst (local) <- src (local or peer-mapped), nbytes a multiple of 16, both 16-byte aligned.
extern "C" int mb_peer_copy(void* dst, const void* src, long long nbytes, cudaStream_t st) {
  if (nbytes <= 0) return 0;
  if ((nbytes & 15) || (reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) return -3;
  const long long n16 = nbytes >> 4;
  peer_copy_kernel<<<copy_grid(n16), 256, 0, st>>>(static_cast<uint4*>(dst), static_cast<const uint4*>(src), n16);
  return mbh::check_launch("peer_copy");
}

// dst (local bf16) += src (local or peer-mapped bf16), n elements, n % 8 == 0.
extern "C" int mb_peer_add_bf16(void* dst, const void* src, long long n, cudaStream_t st) {
  if (n <= 0) return 0;
  if ((n & 7) || (reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) return -3;
  const long long n16 = n >> 3;
  peer_add_bf16_kernel<<<copy_grid(n16), 256, 0, st>>>(static_cast<uint4*>(dst), static_cast<const uint4*>(src), n16);
  return mbh::check_launch("peer_add_bf16");
}

extern "C" int mb_attn_merge(float* acc, float* lse, const void* part, const float* lse_part, int B, int c, int H,
                             int hd, int S_acc, int row_off, int init, cudaStream_t st) {
  if (B <= 0 || c <= 0) return 0;
  if (hd & 1) return -3;
  const long long warps = static_cast<long long>(B) * c * H;
  const long long blocks = (warps + 7) / 8;
  attn_merge_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(acc, lse, static_cast<const __nv_bfloat16*>(part),
                                                                  lse_part, B, c, H, hd, S_acc, row_off, init);
  return mbh::check_launch("attn_merge");
}

// All-gather of one sharded block into its staging buffer by plain peer loads: `peer_base[r]` is rank r's shard
// buffer (bf16, this rank's own included), `descs` a device array of `ndesc` GatherDesc entries, `slices` the number
// of blocks that share one entry.  Callers make sure with a cross-rank barrier that the shard buffers are final.
extern "C" int mb_peer_gather(void* dst, long long dst_elems, void* const* peer_base, int world, const void* descs,
                              int ndesc, int slices, cudaStream_t st) {
  if (ndesc <= 0) return 0;
  if (world < 1 || world > 8 || slices < 1 || (reinterpret_cast<uintptr_t>(dst) & 15)) return -3;
  GatherPeers peers;
  for (int r = 0; r < 8; ++r) {
    peers.base[r] = r < world ? static_cast<const uint4*>(peer_base[r]) : nullptr;
    if (r < world && (!peer_base[r] || (reinterpret_cast<uintptr_t>(peer_base[r]) & 15))) return -3;
  }
  peer_gather_kernel<<<dim3(ndesc, slices), 256, 0, st>>>(static_cast<uint4*>(dst), peers,
                                                         static_cast<const GatherDesc*>(descs), dst_elems,
                                                         mbh::status().dev);
  return mbh::check_launch("peer_gather");
}
