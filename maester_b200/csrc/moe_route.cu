// Mixture-of-experts routing and row movement without host round trips or sort passes.
//
// The reference routes with a chain of ATen ops: sigmoid / softmax, topk, histc, a stable argsort of the
// T*k expert ids, gathers and a scatter_add (maester/models/moe/moe.py:286-334, 378-398, 497, 522), and pads
// the expert groups with a Triton index kernel (maester/models/moe/kernels.py:15-60).  Here:
//
//   route_topk   one warp per token: score function, biased top-k selection, normalisation, and a
//                per-block histogram of the chosen experts (shared-memory atomics only);
//   route_scan   one block: per-expert exclusive scan of the block histograms, expert totals, the
//                start of each expert in sorted order and in the tile-padded expert-major buffer;
//   route_place  a stable counting sort: every slot computes its rank among the earlier slots of its
//                block with the same expert, which with the scanned bases gives its sorted position
//                and its row in the padded buffer.  No global atomics, so the result is deterministic
//                and equal to a stable argsort.
//
// and three row kernels (one warp per row, 128-bit accesses) used by the dispatch and combine steps
// and by each other's backward passes:
//
//   rows_gather   buf[r] = x[token of the slot that owns row r] * (score), zeros for padding rows
//   rows_combine  out[t] = sum_j buf[row of slot (t, j)] * (score), fp32 accumulation
//   slot_dot      d[s]   = <buf[row of slot s], g[token of s]>            (gradient of the scores)
#include "host_common.cuh"
#include <cuda_bf16.h>
#include <math_constants.h>

namespace {

constexpr int RT_MAX_E = 256;      // experts
constexpr int RT_MAX_K = 8;        // experts per token
constexpr int RT_WARPS = 8;        // warps per block
constexpr int RT_TOK_PER_WARP = 8;
constexpr int RT_TOK_PER_BLOCK = RT_WARPS * RT_TOK_PER_WARP;  // 64 tokens: at most 512 slots per block

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// logits [T, E] fp32 -> scores [T, E], top [T, k] fp32, idx [T, k] int32, block_hist [nblocks, E] int32
__global__ void __launch_bounds__(RT_WARPS * 32)
route_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int k, int softmax,
                  int norm, float scale, int force_balance, float* __restrict__ scores, float* __restrict__ top,
                  int* __restrict__ idx, int* __restrict__ block_hist) {
  __shared__ float s_score[RT_WARPS][RT_MAX_E];
  __shared__ int s_hist[RT_MAX_E];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < E; e += blockDim.x) s_hist[e] = 0;
  __syncthreads();
  const int vpl = (E + 31) >> 5;
  float* sc = s_score[warp];
  for (int i = 0; i < RT_TOK_PER_WARP; ++i) {
    const int t = blockIdx.x * RT_TOK_PER_BLOCK + warp * RT_TOK_PER_WARP + i;
    if (t >= T) break;
    const float* row = logits + static_cast<long long>(t) * E;
    float v[RT_MAX_E / 32], sel[RT_MAX_E / 32];
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < RT_MAX_E / 32; ++j) {
      const int e = lane + 32 * j;
      v[j] = (j < vpl && e < E) ? row[e] : -CUDART_INF_F;
      mx = fmaxf(mx, v[j]);
    }
    if (softmax) {
      mx = warp_max(mx);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < RT_MAX_E / 32; ++j) {
        v[j] = (lane + 32 * j < E && j < vpl) ? __expf(v[j] - mx) : 0.f;
        sum += v[j];
      }
      sum = warp_sum(sum);
      const float r = 1.f / sum;
#pragma unroll
      for (int j = 0; j < RT_MAX_E / 32; ++j) v[j] *= r;
    } else {
#pragma unroll
      for (int j = 0; j < RT_MAX_E / 32; ++j) v[j] = 1.f / (1.f + __expf(-v[j]));
    }
#pragma unroll
    for (int j = 0; j < RT_MAX_E / 32; ++j) {
      const int e = lane + 32 * j;
      if (j < vpl && e < E) {
        sc[e] = v[j];
        scores[static_cast<long long>(t) * E + e] = v[j];
        sel[j] = v[j] + (bias ? bias[e] : 0.f);
      } else {
        sel[j] = -CUDART_INF_F;
      }
    }
    __syncwarp();
    int my_idx = 0;       // lane j < k keeps the j-th choice
    float my_top = 0.f;
    if (force_balance) {
      if (lane < k) {
        my_idx = static_cast<int>((static_cast<long long>(t) * k + lane) % E);
        my_top = sc[my_idx];
      }
    } else {
      for (int c = 0; c < k; ++c) {
        float best = -CUDART_INF_F;
        int be = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < RT_MAX_E / 32; ++j) {
          const int e = lane + 32 * j;
          if (j < vpl && e < E && (sel[j] > best)) {
            best = sel[j];
            be = e;
          }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oe = __shfl_xor_sync(0xffffffffu, be, o);
          if (ob > best || (ob == best && oe < be)) {
            best = ob;
            be = oe;
          }
        }
        if (be == 0x7fffffff) be = c % E;  // every candidate is NaN or -inf: keep the indices in range
        if ((be & 31) == lane) {
#pragma unroll
          for (int j = 0; j < RT_MAX_E / 32; ++j)
            if (j == (be >> 5)) sel[j] = -CUDART_INF_F;
        }
        if (lane == c) {
          my_idx = be;
          my_top = sc[be];
        }
      }
    }
    float sum = warp_sum(lane < k ? my_top : 0.f);
    if (lane < k) {
      if (norm) my_top = my_top / (sum + 1e-20f);
      top[static_cast<long long>(t) * k + lane] = my_top * scale;
      idx[static_cast<long long>(t) * k + lane] = my_idx;
      atomicAdd(&s_hist[my_idx], 1);
    }
    __syncwarp();
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) block_hist[static_cast<long long>(blockIdx.x) * E + e] = s_hist[e];
}

// block_hist becomes the exclusive prefix over blocks; counts / starts / padded offsets per expert
__global__ void __launch_bounds__(RT_MAX_E)
route_scan_kernel(int* __restrict__ block_hist, int nblocks, int E, int align, int* __restrict__ counts,
                  float* __restrict__ counts_f, int* __restrict__ start, int* __restrict__ offs) {
  __shared__ int s_cnt[RT_MAX_E];
  const int e = threadIdx.x;
  if (e < E) {
    int run = 0;
    for (int b = 0; b < nblocks; ++b) {
      const long long at = static_cast<long long>(b) * E + e;
      const int c = block_hist[at];
      block_hist[at] = run;
      run += c;
    }
    s_cnt[e] = run;
    counts[e] = run;
    counts_f[e] = static_cast<float>(run);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0, o = 0;
    for (int i = 0; i < E; ++i) {
      start[i] = s;
      offs[i] = o;
      s += s_cnt[i];
      o += (s_cnt[i] + align - 1) / align * align;
    }
    offs[E] = o;
  }
}

__global__ void __launch_bounds__(256)
route_place_kernel(const int* __restrict__ idx, const float* __restrict__ top, const int* __restrict__ block_base,
                   const int* __restrict__ start, const int* __restrict__ offs, int T, int E, int k,
                   int* __restrict__ order, int* __restrict__ inv, int* __restrict__ slot_row,
                   int* __restrict__ row_slot, float* __restrict__ sorted_scores, int* __restrict__ token_idx,
                   int* __restrict__ sorted_experts) {
  __shared__ int s_e[RT_TOK_PER_BLOCK * RT_MAX_K];
  const int tok0 = blockIdx.x * RT_TOK_PER_BLOCK;
  const int ntok = min(RT_TOK_PER_BLOCK, T - tok0);
  const int n = ntok * k;
  const long long base = static_cast<long long>(tok0) * k;
  for (int s = threadIdx.x; s < n; s += blockDim.x) s_e[s] = idx[base + s];
  __syncthreads();
  for (int s = threadIdx.x; s < n; s += blockDim.x) {
    const int e = s_e[s];
    int rank = 0;
    for (int q = 0; q < s; ++q) rank += (s_e[q] == e);
    const int within = block_base[static_cast<long long>(blockIdx.x) * E + e] + rank;
    const int pos = start[e] + within;
    const int row = offs[e] + within;
    const int slot = static_cast<int>(base) + s;
    order[pos] = slot;
    inv[slot] = pos;
    slot_row[slot] = row;
    row_slot[row] = slot;
    sorted_scores[pos] = top[slot];
    token_idx[pos] = slot / k;
    sorted_experts[pos] = e;
  }
}

// d_logits from d_top (through selection, normalisation, scale) and d_scores (dense, may be null)
__global__ void __launch_bounds__(RT_WARPS * 32)
route_bwd_kernel(const float* __restrict__ d_top, const float* __restrict__ d_scores, const float* __restrict__ scores,
                 const int* __restrict__ idx, int T, int E, int k, int softmax, int norm, float scale,
                 float* __restrict__ d_logits) {
  __shared__ float s_ds[RT_WARPS][RT_MAX_E];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* ds = s_ds[warp];
  for (int t = blockIdx.x * RT_WARPS + warp; t < T; t += gridDim.x * RT_WARPS) {
    const float* srow = scores + static_cast<long long>(t) * E;
    for (int e = lane; e < E; e += 32) ds[e] = d_scores ? d_scores[static_cast<long long>(t) * E + e] : 0.f;
    __syncwarp();
    int my_e = 0;
    float s = 0.f, g = 0.f;
    if (lane < k) {
      my_e = idx[static_cast<long long>(t) * k + lane];
      s = srow[my_e];
      g = d_top[static_cast<long long>(t) * k + lane];
    }
    float dsel = g * scale;
    if (norm) {
      const float S = warp_sum(s) + 1e-20f;
      const float gs = warp_sum(g * s);
      dsel = scale * (g / S - gs / (S * S));
    }
    if (lane < k) ds[my_e] += dsel;  // the k experts of a token are distinct
    __syncwarp();
    float dot = 0.f;
    if (softmax) {
      for (int e = lane; e < E; e += 32) dot += ds[e] * srow[e];
      dot = warp_sum(dot);
    }
    for (int e = lane; e < E; e += 32) {
      const float p = srow[e];
      d_logits[static_cast<long long>(t) * E + e] = softmax ? p * (ds[e] - dot) : ds[e] * p * (1.f - p);
    }
    __syncwarp();
  }
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 p = __bfloat1622float2(h[i]);
    f[2 * i] = p.x;
    f[2 * i + 1] = p.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

// buf[r] = x[row_slot[r] / k] * (slot_scale ? slot_scale[row_slot[r]] : 1); zeros where row_slot[r] < 0
__global__ void __launch_bounds__(256)
rows_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_slot,
                   const float* __restrict__ slot_scale, int k, int rows, int dim, __nv_bfloat16* __restrict__ buf) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = dim >> 3;
  for (int r = blockIdx.x * 8 + warp; r < rows; r += gridDim.x * 8) {
    const int s = row_slot[r];
    uint4* d = reinterpret_cast<uint4*>(buf + static_cast<long long>(r) * dim);
    if (s < 0) {
      for (int v = lane; v < nvec; v += 32) d[v] = make_uint4(0u, 0u, 0u, 0u);
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(s / k) * dim);
    if (slot_scale == nullptr) {
      for (int v = lane; v < nvec; v += 32) d[v] = src[v];
    } else {
      const float w = slot_scale[s];
      for (int v = lane; v < nvec; v += 32) {
        float f[8];
        unpack8(src[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] *= w;
        d[v] = pack8(f);
      }
    }
  }
}

// out[t] = sum_j buf[slot_row[t*k+j]] * (slot_scale ? slot_scale[t*k+j] : 1)
__global__ void __launch_bounds__(256)
rows_combine_kernel(const __nv_bfloat16* __restrict__ buf, const int* __restrict__ slot_row,
                    const float* __restrict__ slot_scale, int k, int T, int dim, long long rows,
                    __nv_bfloat16* __restrict__ out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = dim >> 3;
  for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    int row[RT_MAX_K];
    float w[RT_MAX_K];
#pragma unroll
    for (int j = 0; j < RT_MAX_K; ++j) {
      row[j] = j < k ? slot_row[static_cast<long long>(t) * k + j] : -1;
      w[j] = (j < k && slot_scale) ? slot_scale[static_cast<long long>(t) * k + j] : 1.f;
      if (row[j] >= rows) row[j] = -1;
    }
    uint4* d = reinterpret_cast<uint4*>(out + static_cast<long long>(t) * dim);
    for (int v = lane; v < nvec; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < RT_MAX_K; ++j) {
        if (row[j] < 0) continue;
        float f[8];
        unpack8(reinterpret_cast<const uint4*>(buf + static_cast<long long>(row[j]) * dim)[v], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(f[i], w[j], acc[i]);
      }
      d[v] = pack8(acc);
    }
  }
}

// out[t*k+j] = <buf[slot_row[t*k+j]], g[t]>
__global__ void __launch_bounds__(256)
slot_dot_kernel(const __nv_bfloat16* __restrict__ buf, const int* __restrict__ slot_row,
                const __nv_bfloat16* __restrict__ g, int k, int T, int dim, long long rows, float* __restrict__ out) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = dim >> 3;
  for (int t = blockIdx.x * 8 + warp; t < T; t += gridDim.x * 8) {
    const uint4* gr = reinterpret_cast<const uint4*>(g + static_cast<long long>(t) * dim);
    for (int j = 0; j < k; ++j) {
      const int row = slot_row[static_cast<long long>(t) * k + j];
      float acc = 0.f;
      if (row >= 0 && row < rows) {
        const uint4* br = reinterpret_cast<const uint4*>(buf + static_cast<long long>(row) * dim);
        for (int v = lane; v < nvec; v += 32) {
          float a[8], b[8];
          unpack8(br[v], a);
          unpack8(gr[v], b);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc = fmaf(a[i], b[i], acc);
        }
      }
      acc = warp_sum(acc);
      if (lane == 0) out[static_cast<long long>(t) * k + j] = acc;
    }
  }
}

int row_grid(long long n) {
  const long long want = (n + 7) / 8;
  const long long cap = static_cast<long long>(mbh::sm_count()) * 8;
  return static_cast<int>(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace

// Number of int32 words of scratch that mb_moe_route needs for T tokens and E experts.
extern "C" long long mb_moe_route_scratch_words(int T, int E) {
  const long long nb = (T + RT_TOK_PER_BLOCK - 1) / RT_TOK_PER_BLOCK;
  return nb * E + E;
}

// Routing plan of one MoE block.  logits [T, E] fp32; bias [E] fp32 or null.  Outputs: scores [T, E],
// top [T, k] (normalised, scaled), idx [T, k], counts [E] (int and float), offs [E+1] (padded to `align` rows),
// order / sorted_scores / token_idx / sorted_experts [T*k] (stable expert-major order), inv / slot_row [T*k]
// (slot -> sorted position, slot -> row of the padded buffer), row_slot [rows_cap] (row -> slot, -1 = padding).
extern "C" int mb_moe_route(const float* logits, const float* bias, int T, int E, int k, int softmax, int norm,
                            float scale, int force_balance, int align, long long rows_cap, float* scores, float* top,
                            int* idx, int* counts, float* counts_f, int* offs, int* order, int* inv, int* slot_row,
                            int* row_slot, float* sorted_scores, int* token_idx, int* sorted_experts, int* scratch,
                            cudaStream_t st) {
  if (T <= 0) return 0;
  if (E < 1 || E > RT_MAX_E || k < 1 || k > RT_MAX_K || k > E || align < 1) return -3;
  if (static_cast<long long>(T) * k + static_cast<long long>(E) * (align - 1) > rows_cap) return -3;
  if (static_cast<long long>(T) * k > 0x7fffffffLL) return -3;
  const int nb = (T + RT_TOK_PER_BLOCK - 1) / RT_TOK_PER_BLOCK;
  int* block_hist = scratch;
  int* start = scratch + static_cast<long long>(nb) * E;
  cudaMemsetAsync(row_slot, 0xff, static_cast<size_t>(rows_cap) * sizeof(int), st);
  route_topk_kernel<<<nb, RT_WARPS * 32, 0, st>>>(logits, bias, T, E, k, softmax, norm, scale, force_balance, scores, top,
                                                  idx, block_hist);
  route_scan_kernel<<<1, RT_MAX_E, 0, st>>>(block_hist, nb, E, align, counts, counts_f, start, offs);
  route_place_kernel<<<nb, 256, 0, st>>>(idx, top, block_hist, start, offs, T, E, k, order, inv, slot_row, row_slot,
                                         sorted_scores, token_idx, sorted_experts);
  return mbh::check_launch("moe_route");
}

extern "C" int mb_moe_route_bwd(const float* d_top, const float* d_scores, const float* scores, const int* idx, int T,
                                int E, int k, int softmax, int norm, float scale, float* d_logits, cudaStream_t st) {
  if (T <= 0) return 0;
  if (E < 1 || E > RT_MAX_E || k < 1 || k > RT_MAX_K) return -3;
  const int want = (T + RT_WARPS - 1) / RT_WARPS;
  const int cap = mbh::sm_count() * 8;
  route_bwd_kernel<<<want < cap ? want : cap, RT_WARPS * 32, 0, st>>>(d_top, d_scores, scores, idx, T, E, k, softmax, norm,
                                                                     scale, d_logits);
  return mbh::check_launch("moe_route_bwd");
}

extern "C" int mb_moe_rows_gather(const void* x, const int* row_slot, const float* slot_scale, int k, long long rows,
                                  int dim, void* buf, cudaStream_t st) {
  if (rows <= 0) return 0;
  if ((dim & 7) || k < 1 || rows > 0x7fffffffLL) return -3;
  rows_gather_kernel<<<row_grid(rows), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), row_slot, slot_scale, k,
                                                     static_cast<int>(rows), dim, static_cast<__nv_bfloat16*>(buf));
  return mbh::check_launch("moe_rows_gather");
}

extern "C" int mb_moe_rows_combine(const void* buf, const int* slot_row, const float* slot_scale, int k, int T, int dim,
                                   long long rows, void* out, cudaStream_t st) {
  if (T <= 0) return 0;
  if ((dim & 7) || k < 1 || k > RT_MAX_K) return -3;
  rows_combine_kernel<<<row_grid(T), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(buf), slot_row, slot_scale, k, T, dim,
                                                   rows, static_cast<__nv_bfloat16*>(out));
  return mbh::check_launch("moe_rows_combine");
}

extern "C" int mb_moe_slot_dot(const void* buf, const int* slot_row, const void* g, int k, int T, int dim, long long rows,
                               float* out, cudaStream_t st) {
  if (T <= 0) return 0;
  if ((dim & 7) || k < 1) return -3;
  slot_dot_kernel<<<row_grid(T), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(buf), slot_row,
                                               static_cast<const __nv_bfloat16*>(g), k, T, dim, rows, out);
  return mbh::check_launch("moe_slot_dot");
}
