// Multi-head latent attention (DeepSeek): pack the projections into the attention kernel's layout in one pass.
//
// The reference builds q = [q_nope | rope(q_pe)], k = [k_nope | rope(k_pe) shared by all heads] and v with
// eager slicing, complex-number RoPE, expand and cat (maester/models/deepseek/model.py:118-133, attention.py).
// Here one warp per (token, head) reads
//   q   [T, H, nope + rope]      (output of wq / wq_b)
//   kvb [T, H, nope + vdim]      (output of wkv_b: k_nope | v)
//   kpe [T, rope]                (slice of the wkv_a output, row pitch given)
// and writes the rows of the packed [T, 3, H, P] tensor (q | k | v, head size padded with zeros to P, the head
// size the attention kernel is instantiated for), rotating the rope channels (interleaved pairs) by
// pos[t] * inv_freq[i] computed in fp32.  The backward kernel is the transpose: inverse rotation, the padding
// dropped, and the shared k_pe gradient summed over the heads of a token.
// Every lane moves one 16-byte vector of a row, so nope, rope, vdim must be multiples of 8 and P <= 256.
#include "host_common.cuh"
#include <cuda_bf16.h>

namespace {

__device__ __forceinline__ void mla_unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 p = __bfloat1622float2(h[i]);
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
}
__device__ __forceinline__ uint4 mla_pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}
// rotate the 4 interleaved pairs of one vector; pair j uses frequency index first_pair + j; sign = -1 inverts
__device__ __forceinline__ void mla_rotate(float* f, float pos, const float* __restrict__ inv_freq, int first_pair,
                                           float sign) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float s, c;
    sincosf(pos * inv_freq[first_pair + j], &s, &c);
    s *= sign;
    const float a = f[2 * j], b = f[2 * j + 1];
    f[2 * j] = a * c - b * s;
    f[2 * j + 1] = a * s + b * c;
  }
}

__global__ void __launch_bounds__(256)
mla_pack_fwd_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kvb,
                    const __nv_bfloat16* __restrict__ kpe, long long kpe_pitch, const long long* __restrict__ pos,
                    const float* __restrict__ inv_freq, long long T, int H, int nope, int rope, int vdim, int P,
                    __nv_bfloat16* __restrict__ out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = lane * 8;
  const long long total = T * H;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (long long w = static_cast<long long>(blockIdx.x) * 8 + warp; w < total; w += static_cast<long long>(gridDim.x) * 8) {
    const long long t = w / H;
    const int h = static_cast<int>(w - t * H);
    if (c0 >= P) continue;
    const float p = static_cast<float>(pos[t]);
    const __nv_bfloat16* qrow = q + (t * H + h) * (nope + rope);
    const __nv_bfloat16* kvrow = kvb + (t * H + h) * (nope + vdim);
    __nv_bfloat16* orow = out + t * 3 * H * P + static_cast<long long>(h) * P;
    uint4 qv = zero, kv = zero, vv = zero;
    if (c0 < nope) {
      qv = *reinterpret_cast<const uint4*>(qrow + c0);
      kv = *reinterpret_cast<const uint4*>(kvrow + c0);
    } else if (c0 < nope + rope) {
      float f[8];
      mla_unpack8(*reinterpret_cast<const uint4*>(qrow + c0), f);
      mla_rotate(f, p, inv_freq, (c0 - nope) >> 1, 1.f);
      qv = mla_pack8(f);
      mla_unpack8(*reinterpret_cast<const uint4*>(kpe + t * kpe_pitch + (c0 - nope)), f);
      mla_rotate(f, p, inv_freq, (c0 - nope) >> 1, 1.f);
      kv = mla_pack8(f);
    }
    if (c0 < vdim) vv = *reinterpret_cast<const uint4*>(kvrow + nope + c0);
    *reinterpret_cast<uint4*>(orow + c0) = qv;
    *reinterpret_cast<uint4*>(orow + static_cast<long long>(H) * P + c0) = kv;
    *reinterpret_cast<uint4*>(orow + 2LL * H * P + c0) = vv;
  }
}

// one block per token; warps loop over the heads and keep the k_pe gradient of their heads in registers
__global__ void __launch_bounds__(256)
mla_pack_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const long long* __restrict__ pos,
                    const float* __restrict__ inv_freq, long long T, int H, int nope, int rope, int vdim, int P,
                    __nv_bfloat16* __restrict__ dq, __nv_bfloat16* __restrict__ dkvb, __nv_bfloat16* __restrict__ dkpe) {
  __shared__ float s_kpe[8][256];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = lane * 8;
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    const float p = static_cast<float>(pos[t]);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int h = warp; h < H; h += 8) {
      if (c0 >= P) continue;
      const __nv_bfloat16* grow = dout + t * 3 * H * P + static_cast<long long>(h) * P;
      __nv_bfloat16* dqrow = dq + (t * H + h) * (nope + rope);
      __nv_bfloat16* dkvrow = dkvb + (t * H + h) * (nope + vdim);
      if (c0 < nope) {
        *reinterpret_cast<uint4*>(dqrow + c0) = *reinterpret_cast<const uint4*>(grow + c0);
        *reinterpret_cast<uint4*>(dkvrow + c0) = *reinterpret_cast<const uint4*>(grow + static_cast<long long>(H) * P + c0);
      } else if (c0 < nope + rope) {
        float f[8];
        mla_unpack8(*reinterpret_cast<const uint4*>(grow + c0), f);
        mla_rotate(f, p, inv_freq, (c0 - nope) >> 1, -1.f);
        *reinterpret_cast<uint4*>(dqrow + c0) = mla_pack8(f);
        mla_unpack8(*reinterpret_cast<const uint4*>(grow + static_cast<long long>(H) * P + c0), f);
        mla_rotate(f, p, inv_freq, (c0 - nope) >> 1, -1.f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
      if (c0 < vdim)
        *reinterpret_cast<uint4*>(dkvrow + nope + c0) = *reinterpret_cast<const uint4*>(grow + 2LL * H * P + c0);
    }
    __syncthreads();  // the previous token's reduction is finished
#pragma unroll
    for (int i = 0; i < 8; ++i) s_kpe[warp][c0 + i] = acc[i];
    __syncthreads();
    for (int c = threadIdx.x; c < rope; c += blockDim.x) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s += s_kpe[w][nope + c];
      dkpe[t * rope + c] = __float2bfloat16(s);
    }
  }
}

bool mla_dims_ok(int H, int nope, int rope, int vdim, int P) {
  return H >= 1 && nope >= 0 && rope >= 0 && vdim >= 8 && !(nope & 7) && !(rope & 7) && !(vdim & 7) && !(P & 7) &&
         P <= 256 && nope + rope <= P && vdim <= P;
}

}  // namespace

// out: [T, 3*H*P] bf16.  pos: [T] int64; inv_freq: [rope / 2] fp32; kpe row pitch in elements (multiple of 8).
extern "C" int mb_mla_pack_fwd(const void* q, const void* kvb, const void* kpe, long long kpe_pitch, const long long* pos,
                               const float* inv_freq, long long T, int H, int nope, int rope, int vdim, int P, void* out,
                               cudaStream_t st) {
  if (T <= 0) return 0;
  if (!mla_dims_ok(H, nope, rope, vdim, P) || (kpe_pitch & 7) || (reinterpret_cast<uintptr_t>(kpe) & 15)) return -3;
  const long long want = (T * H + 7) / 8;
  const long long cap = static_cast<long long>(mbh::sm_count()) * 16;
  mla_pack_fwd_kernel<<<static_cast<int>(want < cap ? want : cap), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(kvb), static_cast<const __nv_bfloat16*>(kpe),
      kpe_pitch, pos, inv_freq, T, H, nope, rope, vdim, P, static_cast<__nv_bfloat16*>(out));
  return mbh::check_launch("mla_pack_fwd");
}

// dout: [T, 3*H*P]; dq: [T, H*(nope+rope)]; dkvb: [T, H*(nope+vdim)]; dkpe: [T, rope] (contiguous).
extern "C" int mb_mla_pack_bwd(const void* dout, const long long* pos, const float* inv_freq, long long T, int H, int nope,
                               int rope, int vdim, int P, void* dq, void* dkvb, void* dkpe, cudaStream_t st) {
  if (T <= 0) return 0;
  if (!mla_dims_ok(H, nope, rope, vdim, P)) return -3;
  const long long cap = static_cast<long long>(mbh::sm_count()) * 8;
  mla_pack_bwd_kernel<<<static_cast<int>(T < cap ? T : cap), 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(dout), pos, inv_freq, T, H, nope, rope, vdim, P, static_cast<__nv_bfloat16*>(dq),
      static_cast<__nv_bfloat16*>(dkvb), static_cast<__nv_bfloat16*>(dkpe));
  return mbh::check_launch("mla_pack_bwd");
}
