// bf16 GEMM on the 5th-generation tensor cores, single-CTA tiles, plain and grouped.
//
//   plain   : C[M,N] = alpha * op(A) * op(B)^T (+ epilogue)
//   grouped : the rows of A (or the contraction range) are partitioned into groups whose padded
//             offsets live on the device, one B (or one C) per group — the expert GEMMs of a
//             mixture-of-experts layer without a host synchronisation on the group sizes.
//
// One persistent CTA per SM walks 128x256 output tiles.  Warp 0 streams operand tiles with TMA into
// a 4-stage shared-memory ring (128-byte swizzle), warp 1 issues tcgen05.mma (M128 N256 K16) into
// one of two 256-column TMEM accumulators, warps 2-5 drain the other accumulator with tcgen05.ld and
// write C, so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Either operand may be K-major (contraction dimension contiguous: A stored [M,K], B stored [N,K])
// or MN-major (A stored [K,M], B stored [K,N]); this covers forward (x W^T), dgrad (dy W) and wgrad
// (dy^T x) of a linear layer without materialising a transpose.
//
// Every mbarrier wait is bounded; on expiry the kernel records a code in the status word, releases
// TMEM and returns.
#include "gemm_common.cuh"
#include "host_common.cuh"

namespace {

using namespace mb;
using namespace mbg;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 8;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;

enum GroupMode : int {
  GROUP_NONE = 0,
  GROUP_ROWS = 1,   // rows of A / C grouped, B stacked per group (forward, dgrad)
  GROUP_CONTR = 2,  // contraction range grouped, C stacked per group (wgrad)
};

struct GroupParams {
  int mode;
  int num_groups;
  const int* offs;           // [num_groups + 1] row offsets, multiples of 128, on the device
  long long b_group_rows;    // rows of one group's B inside the stacked B matrix (GROUP_ROWS)
  long long c_group_elems;   // elements of one group's C (GROUP_CONTR)
};

// One unit of work of the persistent loop, identical for the three warp roles.
struct Work {
  int m0, n0;        // output tile origin (rows / cols of C)
  int a_row0;        // first contraction row of A/B for MN-major grouped wgrad, else 0
  int kblocks;       // number of 64-deep k-blocks
  long long b_row0;  // row offset into the stacked B (GROUP_ROWS)
  long long c_off;   // element offset of C (GROUP_CONTR)
  int m_limit;       // rows < m_limit are valid
};

__device__ __forceinline__ int find_group(const int* offs, int ng, int row) {
  int lo = 0, hi = ng - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (offs[mid] <= row) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ int num_work(const GemmParams& p, const GroupParams& g) {
  const int tn = (p.N + BN - 1) / BN;
  if (g.mode == GROUP_ROWS) return (g.offs[g.num_groups] / BM) * tn;
  const int tm = (p.M + BM - 1) / BM;
  if (g.mode == GROUP_CONTR) return g.num_groups * tm * tn;
  return tm * tn;
}

__device__ __forceinline__ Work get_work(const GemmParams& p, const GroupParams& g, int t) {
  Work w;
  const int tn = (p.N + BN - 1) / BN;
  w.a_row0 = 0;
  w.b_row0 = 0;
  w.c_off = 0;
  w.m_limit = p.M;
  w.kblocks = (p.K + BK - 1) / BK;
  if (g.mode == GROUP_NONE) {
    const int tm = (p.M + BM - 1) / BM;
    int mt, nt;
    tile_coords(t, tm, tn, GROUP_M, mt, nt);
    w.m0 = mt * BM;
    w.n0 = nt * BN;
  } else if (g.mode == GROUP_ROWS) {
    const int mt = t / tn, nt = t - mt * tn;  // column tiles of one row tile run together
    w.m0 = mt * BM;
    w.n0 = nt * BN;
    const int e = find_group(g.offs, g.num_groups, w.m0);
    w.b_row0 = static_cast<long long>(e) * g.b_group_rows;
    w.m_limit = g.offs[g.num_groups];
  } else {
    const int tm = (p.M + BM - 1) / BM;
    const int per = tm * tn;
    const int e = t / per;
    const int r = t - e * per;
    const int mt = r / tn, nt = r - mt * tn;
    w.m0 = mt * BM;
    w.n0 = nt * BN;
    w.a_row0 = g.offs[e];
    w.kblocks = (g.offs[e + 1] - g.offs[e]) / BK;
    w.c_off = static_cast<long long>(e) * g.c_group_elems;
  }
  return w;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p, const GroupParams g) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                        // [STAGES]
  uint64_t* empty = bars + STAGES;              // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;       // [2]
  uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total = num_work(p, g);

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 128);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const Work w = get_work(p, g, t);
        for (int kb = 0; kb < w.kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1)) {
            atomicCAS(p.status, 0, ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d(sa, &tmap_a, &full[s], k0, w.m0);
          } else {
#pragma unroll
            for (int b = 0; b < BM / 64; ++b)
              tma_load_2d(sa + b * (BK * 128), &tmap_a, &full[s], w.m0 + b * 64, w.a_row0 + k0);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tmap_b, &full[s], k0, static_cast<int>(w.b_row0) + w.n0);
          } else {
#pragma unroll
            for (int b = 0; b < BN / 64; ++b)
              tma_load_2d(sb + b * (BK * 128), &tmap_b, &full[s], w.n0 + b * 64,
                          static_cast<int>(w.b_row0) + w.a_row0 + k0);
          }
        }
      }
      // drain: every copy issued above has landed once the matching full barrier phase completed
      const uint32_t issued = it;
      for (uint32_t j = (issued > STAGES ? issued - STAGES : 0); j < issued; ++j)
        mbar_wait(&full[j % STAGES], (j / STAGES) & 1, 20000000ull);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        const Work w = get_work(p, g, t);
        if (w.kblocks == 0) continue;  // empty group: nothing to accumulate
        const uint32_t acc = tcount & 1, acc_ph = (tcount >> 1) & 1;
        ++tcount;
        if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1)) {
          atomicCAS(p.status, 0, ERR_WAIT_ACC_EMPTY);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < w.kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full[s], ph)) {
            atomicCAS(p.status, 0, ERR_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // K-major: 16 elements = 32 B along the swizzled row; MN-major: 16 k-rows = 2048 B
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024)
                                     : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024)
                                     : make_smem_desc(sb + k * 32, 16, 1024);
            umma_bf16_ss(d_tmem, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(&acc_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    const float alpha = p.alpha * (p.alpha_dev ? __ldg(p.alpha_dev) : 1.f);
    uint32_t tcount = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
      const Work w = get_work(p, g, t);
      if (w.kblocks == 0) continue;
      const uint32_t acc = tcount & 1, acc_ph = (tcount >> 1) & 1;
      ++tcount;
      if (!mbar_wait(&acc_full[acc], acc_ph)) {
        atomicCAS(p.status, 0, ERR_WAIT_ACC_FULL);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = w.m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      GemmParams pp = p;
      pp.M = w.m_limit;
      if (w.c_off) {
        pp.C = (p.epi == EPI_BF16 || p.epi == EPI_BF16_ADD)
                   ? static_cast<void*>(reinterpret_cast<__nv_bfloat16*>(p.C) + w.c_off)
                   : static_cast<void*>(reinterpret_cast<float*>(p.C) + w.c_off);
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        store_acc_chunk(pp, r, alpha, row, w.n0 + c * 32);
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

template <bool A_MN, bool B_MN>
int launch(const void* A, const void* B, const GemmParams& p, const GroupParams& g, long long a_rows,
           long long b_rows, long long lda, long long ldb, cudaStream_t stream) {
  // a_rows / b_rows: number of rows of the stored A / B matrices (they differ from M/N/K when grouped)
  CUtensorMap ta, tb;
  int e;
  if (!A_MN) e = mbh::make_tmap_bf16_2d(&ta, A, p.K, a_rows, lda, 64, BM);
  else e = mbh::make_tmap_bf16_2d(&ta, A, p.M, a_rows, lda, 64, BK);
  if (e) return e;
  if (!B_MN) e = mbh::make_tmap_bf16_2d(&tb, B, p.K, b_rows, ldb, 64, BN);
  else e = mbh::make_tmap_bf16_2d(&tb, B, p.N, b_rows, ldb, 64, BK);
  if (e) return e;
  MB_SET_MAX_SMEM_ONCE((gemm_bf16_kernel<A_MN, B_MN>), SMEM_BYTES);
  int grid = mbh::sm_count();
  if (g.mode == GROUP_NONE) {
    const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
    grid = tiles < grid ? tiles : grid;
  }
  gemm_bf16_kernel<A_MN, B_MN><<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p, g);
  return mbh::check_launch("gemm_bf16");
}

int dispatch(const void* A, const void* B, const GemmParams& p, const GroupParams& g, long long a_rows,
             long long b_rows, long long lda, long long ldb, int a_mn, int b_mn, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch<false, false>(A, B, p, g, a_rows, b_rows, lda, ldb, stream);
  if (!a_mn && b_mn) return launch<false, true>(A, B, p, g, a_rows, b_rows, lda, ldb, stream);
  if (a_mn && !b_mn) return launch<true, false>(A, B, p, g, a_rows, b_rows, lda, ldb, stream);
  return launch<true, true>(A, B, p, g, a_rows, b_rows, lda, ldb, stream);
}

}  // namespace

// C[M,N] = alpha * op(A) op(B)^T.  a_mn = 0: A is [M,K] row-major (pitch lda); a_mn = 1: A is [K,M].
// b_mn = 0: B is [N,K] row-major (pitch ldb); b_mn = 1: B is [K,N].  epi: see EpiMode.
// Requirements: bf16 operands, 16-byte aligned bases, pitches multiples of 8 elements.
extern "C" int mb_gemm_bf16(const void* A, const void* B, void* C, const void* aux, int M, int N, int K,
                            long long lda, long long ldb, long long ldc, long long ldaux, int a_mn, int b_mn,
                            int epi, float alpha, float beta, const float* alpha_dev, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -3;
  GemmParams p;
  p.beta = beta;
  p.C = C;
  p.aux = aux;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.ldaux = ldaux;
  p.epi = epi;
  p.alpha = alpha;
  p.alpha_dev = alpha_dev;
  p.status = mbh::status().dev;
  p.splits = 1;
  p.route_rows = 0;
  if (!p.status) return -4;
  GroupParams g = {GROUP_NONE, 0, nullptr, 0, 0};
  return dispatch(A, B, p, g, a_mn ? K : M, b_mn ? K : N, lda, ldb, a_mn, b_mn, stream);
}

// Grouped GEMM over row groups (forward / dgrad of stacked expert weights).
//   A: [rows_cap, K] bf16, rows grouped by offs (device int32 [E+1], multiples of 128; rows beyond
//      offs[E] are ignored);  C: [rows_cap, N]
//   b_mn = 0: B stacked [E*N, K]   -> C_e = A_e B_e^T
//   b_mn = 1: B stacked [E*K, N]   -> C_e = A_e B_e      (K must be a multiple of 64)
extern "C" int mb_gemm_bf16_grouped_rows(const void* A, const void* B, void* C, const int* offs, int num_groups,
                                         int rows_cap, int N, int K, long long lda, long long ldb, long long ldc,
                                         int b_mn, int epi, float alpha, cudaStream_t stream) {
  if (rows_cap <= 0 || N <= 0 || K <= 0 || num_groups <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (rows_cap % 128) || (b_mn && (K % 64))) return -3;
  GemmParams p;
  p.C = C;
  p.aux = nullptr;
  p.M = rows_cap;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.ldaux = 0;
  p.epi = epi;
  p.alpha = alpha;
  p.alpha_dev = nullptr;
  p.beta = 1.f;
  p.status = mbh::status().dev;
  p.splits = 1;
  p.route_rows = 0;
  if (!p.status) return -4;
  GroupParams g = {GROUP_ROWS, num_groups, offs, b_mn ? K : N, 0};
  const long long b_rows = static_cast<long long>(num_groups) * (b_mn ? K : N);
  return dispatch(A, B, p, g, rows_cap, b_rows, lda, ldb, 0, b_mn, stream);
}

// Grouped GEMM over the contraction range (wgrad of stacked expert weights):
//   C_e[M,N] (+)= A_e^T B_e with A: [rows_cap, M] and B: [rows_cap, N] (both stored row-major, rows
//   grouped by offs); C stacked [E, M, N] with pitch ldc.  Groups with no rows are skipped, so use
//   an accumulating epilogue or a zero-initialised C.
extern "C" int mb_gemm_bf16_grouped_contr(const void* A, const void* B, void* C, const int* offs, int num_groups,
                                          int rows_cap, int M, int N, long long lda, long long ldb, long long ldc,
                                          int epi, float alpha, cudaStream_t stream) {
  if (rows_cap <= 0 || N <= 0 || M <= 0 || num_groups <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (rows_cap % 128)) return -3;
  GemmParams p;
  p.C = C;
  p.aux = nullptr;
  p.M = M;
  p.N = N;
  p.K = rows_cap;
  p.ldc = ldc;
  p.ldaux = 0;
  p.epi = epi;
  p.alpha = alpha;
  p.alpha_dev = nullptr;
  p.beta = 1.f;
  p.status = mbh::status().dev;
  p.splits = 1;
  p.route_rows = 0;
  if (!p.status) return -4;
  // Short contractions (rows of one expert) make the accumulating epilogue's load-add-store the long pole of a
  // tile; reduction atomics need no round trip.  Every element receives exactly one addition per call, so the
  // result is the same as with load-add-store.  MB_GROUPED_RED=0 keeps the plain accumulate.
  static const bool use_red = [] {
    const char* e = getenv("MB_GROUPED_RED");
    return !(e && e[0] == '0');
  }();
  if (use_red && epi == EPI_F32_ACC && (ldc & 3) == 0) p.epi = EPI_F32_RED;
  GroupParams g = {GROUP_CONTR, num_groups, offs, 0, static_cast<long long>(M) * ldc};
  return dispatch(A, B, p, g, rows_cap, rows_cap, lda, ldb, 1, 1, stream);
}

extern "C" int mb_status() { return mbh::status().host ? mbh::status().host[0] : -1; }
extern "C" void mb_status_clear() {
  if (mbh::status().host) mbh::status().host[0] = 0;
}
