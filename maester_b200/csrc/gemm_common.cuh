// Pieces shared by the GEMM kernels: parameters, epilogue modes, tile rasterisation, and the
// accumulator-row epilogue (32 fp32 values of one output row -> global memory).
#pragma once
#include "sm100.cuh"

namespace mbg {

enum EpiMode : int {
  EPI_BF16 = 0,      // C(bf16) = alpha*acc
  EPI_F32 = 1,       // C(fp32) = alpha*acc
  EPI_F32_ACC = 2,   // C(fp32) += alpha*acc
  EPI_BF16_ADD = 3,  // C(bf16) = alpha*acc + beta*aux(bf16)
  EPI_F32_RED = 4,   // C(fp32) += alpha*acc with reduction atomics (split-K partial sums; chosen internally)
};

struct GemmParams {
  void* C;
  const void* aux;
  int M, N, K;
  long long ldc, ldaux;
  int epi;
  float alpha;
  float beta;              // scale of aux in EPI_BF16_ADD
  const float* alpha_dev;  // optional device scalar multiplied into alpha
  int* status;
  int splits;              // >1: the contraction is cut into this many ranges, each a separate work unit
  // Row routing of bf16 outputs (GEMM fused with a reduce-scatter over peer memory): output row r belongs to
  // rank r / route_rows and is stored into that rank's buffer route_base[owner], in the slot of THIS
  // rank: row  route_slot * route_rows + r % route_rows.  route_rows == 0 turns routing off.
  void* route_base[8];
  int route_rows;
  int route_slot;
  int group_m;             // CTA-pair kernel: row-tiles per rasterisation group (chosen by the launcher)
  // All-gather fused into the GEMM (CTA-pair kernel, A row-major [M, K] whose M / ag_world-row blocks live on
  // different ranks): the last ag_copiers CTA pairs of the grid do no math; they pull the other ranks' blocks
  // from ag_src[r] into the local A with bulk copies staged through shared memory and count every finished
  // share of a 256-row tile in ag_flags[tile].  The computing pairs start with the local block and wait for
  // a remote tile's counter before its first load.  ag_world == 0 turns this off.
  int ag_world = 0;
  int ag_rank = 0;
  int ag_copiers = 0;
  const void* ag_src[8] = {};
  void* ag_dst = nullptr;
  long long ag_ld = 0;     // row pitch of A in elements (== K: blocks are contiguous)
  int* ag_flags = nullptr; // [M / 256] counters, zeroed by the launcher before the kernel
  // Grouped weight gradients on the CTA-pair kernel: C_g[M, N] (+)= A_g^T B_g where group g owns the rows
  // [grp_offs[g], grp_offs[g + 1]) of the contraction (multiples of 128); C_g starts grp_c_elems after C_{g-1}.
  const int* grp_offs = nullptr;
  int grp_count = 0;
  long long grp_c_elems = 0;
};

// group GROUP_M row-tiles together so that concurrently running CTAs share operand tiles in L2
__device__ __forceinline__ void tile_coords(int t, int tm, int tn, int group_m, int& mt, int& nt) {
  const int group_size = group_m * tn;
  const int g = t / group_size;
  const int first_m = g * group_m;
  const int gm = min(tm - first_m, group_m);
  const int r = t - g * group_size;
  mt = first_m + r % gm;
  nt = r / gm;
}

// Store 32 consecutive accumulator columns [col0, col0+32) of output row `row`.
// `c_off` (elements) shifts the base of fp32 outputs (grouped weight gradients on the CTA-pair kernel).
__device__ __forceinline__ void store_acc_chunk(const GemmParams& p, const uint32_t (&r)[32], float alpha, int row,
                                                int col0, long long c_off = 0) {
  using namespace mb;
  if (row >= p.M || col0 >= p.N) return;
  const bool full_chunk = (col0 + 32 <= p.N);
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
  if (p.epi == EPI_BF16 || p.epi == EPI_BF16_ADD) {
    __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
    if (p.route_rows > 0) {
      const int owner = row / p.route_rows;
      const long long slot_row = static_cast<long long>(p.route_slot) * p.route_rows + (row - owner * p.route_rows);
      crow = reinterpret_cast<__nv_bfloat16*>(p.route_base[owner]) + slot_row * p.ldc + col0;
    }
    if (p.epi == EPI_BF16_ADD) {
      const __nv_bfloat16* arow =
          reinterpret_cast<const __nv_bfloat16*>(p.aux) + static_cast<long long>(row) * p.ldaux + col0;
      if (full_chunk && (p.ldaux & 7) == 0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 a4 = reinterpret_cast<const uint4*>(arow)[j];
          const __nv_bfloat162* ab = reinterpret_cast<const __nv_bfloat162*>(&a4);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float2 f = __bfloat1622float2(ab[e]);
            v[j * 8 + e * 2] += p.beta * f.x;
            v[j * 8 + e * 2 + 1] += p.beta * f.y;
          }
        }
      } else {
        for (int i = 0; i < 32 && col0 + i < p.N; ++i) v[i] += p.beta * __bfloat162float(arow[i]);
      }
    }
    if (full_chunk && (p.ldc & 7) == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 o;
        o.x = pack_bf16(v[j * 8 + 0], v[j * 8 + 1]);
        o.y = pack_bf16(v[j * 8 + 2], v[j * 8 + 3]);
        o.z = pack_bf16(v[j * 8 + 4], v[j * 8 + 5]);
        o.w = pack_bf16(v[j * 8 + 6], v[j * 8 + 7]);
        reinterpret_cast<uint4*>(crow)[j] = o;
      }
    } else {
      for (int i = 0; i < 32 && col0 + i < p.N; ++i) crow[i] = __float2bfloat16(v[i]);
    }
  } else {
    float* crow = reinterpret_cast<float*>(p.C) + c_off + static_cast<long long>(row) * p.ldc + col0;
    if (p.epi == EPI_F32_RED) {
      if (full_chunk && (p.ldc & 3) == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(crow + j * 4), "f"(v[j * 4]),
                       "f"(v[j * 4 + 1]), "f"(v[j * 4 + 2]), "f"(v[j * 4 + 3])
                       : "memory");
      } else {
        for (int i = 0; i < 32 && col0 + i < p.N; ++i) atomicAdd(crow + i, v[i]);
      }
      return;
    }
    if (full_chunk && (p.ldc & 3) == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 o = make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
        if (p.epi == EPI_F32_ACC) {
          float4 old = reinterpret_cast<float4*>(crow)[j];
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        reinterpret_cast<float4*>(crow)[j] = o;
      }
    } else {
      for (int i = 0; i < 32 && col0 + i < p.N; ++i) crow[i] = (p.epi == EPI_F32_ACC ? crow[i] : 0.f) + v[i];
    }
  }
}

}  // namespace mbg
