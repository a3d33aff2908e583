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
  // Hybrid form of the same (CTA-pair kernel, accumulating fp32 output, tail_splits > 0): the first full_tiles tiles
  // (whole waves of the grid) are single work units with a plain read-modify-write epilogue; only the tiles of the
  // last, partial wave are cut into tail_splits ranges each and merged with reduction atomics.
  int full_tiles = 0;
  int tail_splits = 0;
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
  // Gated-linear-unit epilogues (CTA-pair kernel).
  //  glu_mode 1 (forward): B is the fused weight [gate rows | up rows] with glu_F rows each and N = 2 glu_F.  A
  //    tile takes 128 gate rows (even CTA's half of B) and the matching 128 up rows (odd CTA's half), so one
  //    accumulator row holds gate_j and up_j for 128 values of j: the epilogue stores both (C = [gate | up], bf16)
  //    and act(gate_j) * up_j into glu_out [M, glu_F] (row pitch glu_ldo).
  //  glu_mode 2 (backward): the accumulator is d(act) [M, N = glu_F]; the epilogue reads gate_j and up_j from
  //    glu_in [M, 2 glu_F] (row pitch glu_ldi) and stores d(gate_j) = d * up_j * act'(gate_j) and
  //    d(up_j) = d * act(gate_j) into C [M, 2 glu_F].
  // Symmetric rank-k update (C = alpha * A A^T [+ beta * aux], M == N, bf16 out): only the tiles on and below the
  // diagonal are computed; every tile below the diagonal is also stored transposed into its mirror position.
  int syrk = 0;
  // Cross-entropy statistics (CTA-pair kernel, ce_mode 1): C = bf16(alpha * acc) are the logits [M, N] (C may be
  // null: nothing is stored).  For every output row and every 256-column tile the epilogue also stores
  // (max, sum of exp(x - max)) over the tile's valid columns into ce_stats[tile * ce_ld + row], and where
  // ce_labels[row] - ce_v0 falls inside the tile the logit itself into ce_tgt[row] (cleared by the launcher).  Both
  // are taken from the rounded bf16 values, so a later pass over the stored logits sees the same numbers.
  int ce_mode = 0;
  const long long* ce_labels = nullptr;
  long long ce_v0 = 0;
  float2* ce_stats = nullptr;
  long long ce_ld = 0;
  float* ce_tgt = nullptr;
  int glu_mode = 0;
  int glu_act = 0;         // 0: tanh-GELU, 1: SiLU
  int glu_F = 0;
  void* glu_out = nullptr;
  long long glu_ldo = 0;
  const void* glu_in = nullptr;
  long long glu_ldi = 0;
};

__device__ __forceinline__ float tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// act(g) and act'(g) for the gated units (tanh-GELU with the hardware tanh, SiLU)
__device__ __forceinline__ void glu_act_and_grad(int act, float g, float& a, float& da) {
  if (act == 0) {
    const float k = 0.7978845608028654f;
    const float inner = k * (g + 0.044715f * g * g * g);
    const float th = tanh_approx(inner);
    a = 0.5f * g * (1.f + th);
    da = 0.5f * (1.f + th) + 0.5f * g * (1.f - th * th) * k * (1.f + 3.f * 0.044715f * g * g);
  } else {
    const float sg = 1.f / (1.f + __expf(-g));
    a = g * sg;
    da = sg * (1.f + g * (1.f - sg));
  }
}
__device__ __forceinline__ float exp2f_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

// 32 accumulator columns of gate and the matching 32 of up for output row `row`, units j0 .. j0+31:
// stores [gate | up] into C and act(gate) * up into glu_out.  glu_F is a multiple of 128, so chunks are whole.
__device__ __forceinline__ void store_glu_fwd_chunk(const GemmParams& p, const uint32_t (&rg)[32],
                                                    const uint32_t (&ru)[32], float alpha, int row, int j0) {
  using namespace mb;
  if (row >= p.M) return;
  MB_CHECK_OR(p.status, row >= 0 && j0 >= 0 && j0 + 32 <= p.glu_F && p.glu_F <= p.glu_ldo &&
                            (!p.C || 2LL * p.glu_F <= p.ldc), return);
  __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc;
  __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.glu_out) + static_cast<long long>(row) * p.glu_ldo + j0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float g[8], u[8], o[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      g[e] = bf16_round(__uint_as_float(rg[j * 8 + e]) * alpha);  // the activation sees what the backward pass will read
      u[e] = bf16_round(__uint_as_float(ru[j * 8 + e]) * alpha);
      float a, da;
      glu_act_and_grad(p.glu_act, g[e], a, da);
      o[e] = a * u[e];
    }
    uint4 vg, vu, vo;
    vg.x = pack_bf16(g[0], g[1]); vg.y = pack_bf16(g[2], g[3]); vg.z = pack_bf16(g[4], g[5]); vg.w = pack_bf16(g[6], g[7]);
    vu.x = pack_bf16(u[0], u[1]); vu.y = pack_bf16(u[2], u[3]); vu.z = pack_bf16(u[4], u[5]); vu.w = pack_bf16(u[6], u[7]);
    vo.x = pack_bf16(o[0], o[1]); vo.y = pack_bf16(o[2], o[3]); vo.z = pack_bf16(o[4], o[5]); vo.w = pack_bf16(o[6], o[7]);
    if (p.C) {
      reinterpret_cast<uint4*>(crow + j0)[j] = vg;
      reinterpret_cast<uint4*>(crow + p.glu_F + j0)[j] = vu;
    }
    reinterpret_cast<uint4*>(orow)[j] = vo;
  }
}

// 32 accumulator columns of d(act) for output row `row`, units j0 .. j0+31 -> d(gate), d(up) into C [M, 2 glu_F].
__device__ __forceinline__ void store_glu_bwd_chunk(const GemmParams& p, const uint32_t (&r)[32], float alpha, int row,
                                                    int j0) {
  using namespace mb;
  if (row >= p.M || j0 >= p.N) return;
  MB_CHECK_OR(p.status, row >= 0 && j0 >= 0 && j0 + 32 <= p.glu_F && 2LL * p.glu_F <= p.ldc && 2LL * p.glu_F <= p.glu_ldi,
              return);
  const __nv_bfloat16* irow = reinterpret_cast<const __nv_bfloat16*>(p.glu_in) + static_cast<long long>(row) * p.glu_ldi;
  __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 g4 = reinterpret_cast<const uint4*>(irow + j0)[j];
    const uint4 u4 = reinterpret_cast<const uint4*>(irow + p.glu_F + j0)[j];
    const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&g4);
    const __nv_bfloat162* ub = reinterpret_cast<const __nv_bfloat162*>(&u4);
    float dg[8], du[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g = __bfloat1622float2(gb[e]), u = __bfloat1622float2(ub[e]);
      const float d0 = __uint_as_float(r[j * 8 + 2 * e]) * alpha, d1 = __uint_as_float(r[j * 8 + 2 * e + 1]) * alpha;
      float a, da;
      glu_act_and_grad(p.glu_act, g.x, a, da);
      dg[2 * e] = d0 * u.x * da;
      du[2 * e] = d0 * a;
      glu_act_and_grad(p.glu_act, g.y, a, da);
      dg[2 * e + 1] = d1 * u.y * da;
      du[2 * e + 1] = d1 * a;
    }
    uint4 vg, vu;
    vg.x = pack_bf16(dg[0], dg[1]); vg.y = pack_bf16(dg[2], dg[3]); vg.z = pack_bf16(dg[4], dg[5]); vg.w = pack_bf16(dg[6], dg[7]);
    vu.x = pack_bf16(du[0], du[1]); vu.y = pack_bf16(du[2], du[3]); vu.z = pack_bf16(du[4], du[5]); vu.w = pack_bf16(du[6], du[7]);
    reinterpret_cast<uint4*>(crow + j0)[j] = vg;
    reinterpret_cast<uint4*>(crow + p.glu_F + j0)[j] = vu;
  }
}

// 32 accumulator columns [col0, col0 + 32) of output row `row` as logits: optional bf16 store, and the running
// (max m, sum s of exp(x - m)) of the row over this tile; `lab` is the row's label relative to column 0 of the matrix.
__device__ __forceinline__ void ce_stats_chunk(const GemmParams& p, const uint32_t (&r)[32], float alpha, int row,
                                               int col0, long long lab, float& m, float& s) {
  using namespace mb;
  if (row >= p.M || col0 >= p.N) return;
  MB_CHECK_OR(p.status, row >= 0 && col0 >= 0 && (!p.C || static_cast<long long>(min(col0 + 32, p.N)) <= p.ldc), return);
  const int nvalid = min(32, p.N - col0);
  // round once to bf16 pairs (what is stored), then widen again with shifts: the statistics describe the stored values
  uint32_t pk[16];
  float v[32];
  // (every instruction here is paid for in clocks: under the board's power limit the extra work of this epilogue
  // slows the tensor pipe although it runs beside it, so the unit scale skips its multiplies)
  if (alpha == 1.f) {
#pragma unroll
    for (int i = 0; i < 16; ++i) pk[i] = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i)
      pk[i] = pack_bf16(__uint_as_float(r[2 * i]) * alpha, __uint_as_float(r[2 * i + 1]) * alpha);
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    v[2 * i] = __uint_as_float(pk[i] << 16);
    v[2 * i + 1] = __uint_as_float(pk[i] & 0xffff0000u);
  }
  if (p.C) {
    __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
    if (nvalid == 32 && (p.ldc & 7) == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        reinterpret_cast<uint4*>(crow)[j] = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < nvalid) reinterpret_cast<unsigned short*>(crow)[i] = static_cast<unsigned short>(__float_as_uint(v[i]) >> 16);
    }
  }
  float cm = -INFINITY;
  if (nvalid == 32) {
#pragma unroll
    for (int i = 0; i < 32; ++i) cm = fmaxf(cm, v[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      v[i] = i < nvalid ? v[i] : -INFINITY;
      cm = fmaxf(cm, v[i]);
    }
  }
  const float nm = fmaxf(m, cm);
  const float k = 1.4426950408889634f, nmk = nm * k;
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) acc += exp2f_approx(fmaf(v[i], k, -nmk));   // exp(v - nm); columns past N give 0
  s = s * exp2f_approx((m - nm) * k) + acc;   // m == -inf on the first chunk: the factor is 0 and s was 0
  m = nm;
  const long long rel = lab - col0;
  if (rel >= 0 && rel < nvalid) {
    // bit masks instead of a select chain: the compiler turns the chain into an indexed read of v[], which moves
    // the whole array to local memory
    uint32_t t = 0u;
    const uint32_t irel = static_cast<uint32_t>(rel);
#pragma unroll
    for (uint32_t i = 0; i < 32; ++i) t |= __float_as_uint(v[i]) & (0u - static_cast<uint32_t>(i == irel));
    p.ce_tgt[row] = __uint_as_float(t);
  }
}

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

// Lower-triangular tile enumeration: t in [0, T (T + 1) / 2) -> (mt, nt) with nt <= mt, row by row.
__device__ __forceinline__ void tri_coords(int t, int& mt, int& nt) {
  int m = static_cast<int>((sqrtf(8.f * static_cast<float>(t) + 1.f) - 1.f) * 0.5f);
  while ((m + 1) * (m + 2) / 2 <= t) ++m;   // guard the float estimate
  while (m * (m + 1) / 2 > t) --m;
  mt = m;
  nt = t - m * (m + 1) / 2;
}

// Mirror of store_acc_chunk for the symmetric update: the 32 values of row `row`, columns [col0, col0+32), also go
// to C[col0 + i][row].  Across a warp the 32 rows are consecutive, so every store instruction writes 64 contiguous bytes.
__device__ __forceinline__ void store_acc_chunk_mirrored(const GemmParams& p, const uint32_t (&r)[32], float alpha,
                                                         int row, int col0) {
  if (row >= p.M) return;
  __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(p.C);
  const __nv_bfloat16* aux = reinterpret_cast<const __nv_bfloat16*>(p.aux);
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int col = col0 + i;
    if (col >= p.N) break;
    float v = __uint_as_float(r[i]) * alpha;
    // the mirrored element takes the aux value of its own position, so a non-symmetric aux stays exact
    if (p.epi == EPI_BF16_ADD) v += p.beta * __bfloat162float(aux[static_cast<long long>(col) * p.ldaux + row]);
    c[static_cast<long long>(col) * p.ldc + row] = __float2bfloat16(v);
  }
}

// Store 32 consecutive accumulator columns [col0, col0+32) of output row `row`.
// `c_off` (elements) shifts the base of fp32 outputs (grouped weight gradients on the CTA-pair kernel).
__device__ __forceinline__ void store_acc_chunk(const GemmParams& p, const uint32_t (&r)[32], float alpha, int row,
                                                int col0, long long c_off = 0, int epi_unit = -1) {
  using namespace mb;
  if (row >= p.M || col0 >= p.N) return;
  const int epi = epi_unit >= 0 ? epi_unit : p.epi;   // (the hybrid split chooses the epilogue per work unit)
  MB_CHECK_OR(p.status, row >= 0 && col0 >= 0 && static_cast<long long>(min(col0 + 32, p.N)) <= p.ldc, return);
  const bool full_chunk = (col0 + 32 <= p.N);
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
  if (epi == EPI_BF16 || epi == EPI_BF16_ADD) {
    __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
    if (p.route_rows > 0) {
      const int owner = row / p.route_rows;
      const long long slot_row = static_cast<long long>(p.route_slot) * p.route_rows + (row - owner * p.route_rows);
      crow = reinterpret_cast<__nv_bfloat16*>(p.route_base[owner]) + slot_row * p.ldc + col0;
    }
    if (epi == EPI_BF16_ADD) {
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
    if (epi == EPI_F32_RED) {
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
        if (epi == EPI_F32_ACC) {
          float4 old = reinterpret_cast<float4*>(crow)[j];
          o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
        }
        reinterpret_cast<float4*>(crow)[j] = o;
      }
    } else {
      for (int i = 0; i < 32 && col0 + i < p.N; ++i) crow[i] = (epi == EPI_F32_ACC ? crow[i] : 0.f) + v[i];
    }
  }
}

}  // namespace mbg
