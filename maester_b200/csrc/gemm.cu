// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = alpha * op(A) * op(B)^T (+ epilogue).
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
#include "host_common.cuh"
#include "sm100.cuh"

namespace {

using namespace mb;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 8;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;

enum EpiMode : int {
  EPI_BF16 = 0,       // C(bf16) = alpha*acc
  EPI_F32 = 1,        // C(fp32) = alpha*acc
  EPI_F32_ACC = 2,    // C(fp32) += alpha*acc
  EPI_BF16_ADD = 3,   // C(bf16) = alpha*acc + aux(bf16)
};

struct GemmParams {
  void* C;
  const void* aux;
  int M, N, K;
  long long ldc, ldaux;
  int epi;
  float alpha;
  const float* alpha_dev;  // optional device scalar multiplied into alpha
  int* status;
};

__device__ __forceinline__ void tile_coords(int t, int tm, int tn, int& mt, int& nt) {
  const int group_size = GROUP_M * tn;
  const int g = t / group_size;
  const int first_m = g * GROUP_M;
  const int gm = min(tm - first_m, GROUP_M);
  const int r = t - g * group_size;
  mt = first_m + r % gm;
  nt = r / gm;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                 // [STAGES]
  uint64_t* empty = bars + STAGES;       // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;      // [2]
  uint64_t* acc_empty = bars + 2 * STAGES + 2; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tm = (p.M + BM - 1) / BM, tn = (p.N + BN - 1) / BN;
  const int num_tiles = tm * tn;
  const int kblocks = (p.K + BK - 1) / BK;

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
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mt, nt;
        tile_coords(t, tm, tn, mt, nt);
        const int m0 = mt * BM, n0 = nt * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
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
            tma_load_2d(sa, &tmap_a, &full[s], k0, m0);
          } else {
#pragma unroll
            for (int b = 0; b < BM / 64; ++b) tma_load_2d(sa + b * (BK * 128), &tmap_a, &full[s], m0 + b * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tmap_b, &full[s], k0, n0);
          } else {
#pragma unroll
            for (int b = 0; b < BN / 64; ++b) tma_load_2d(sb + b * (BK * 128), &tmap_b, &full[s], n0 + b * 64, k0);
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
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tcount) {
        const uint32_t acc = tcount & 1, acc_ph = (tcount >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1)) {
          atomicCAS(p.status, 0, ERR_WAIT_ACC_EMPTY);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
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
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tcount) {
      int mt, nt;
      tile_coords(t, tm, tn, mt, nt);
      const uint32_t acc = tcount & 1, acc_ph = (tcount >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_ph)) {
        atomicCAS(p.status, 0, ERR_WAIT_ACC_FULL);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = mt * BM + q * 32 + lane;
      const int n0 = nt * BN;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      const bool row_ok = row < p.M;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (!row_ok || col0 >= p.N) continue;
        const bool full_chunk = (col0 + 32 <= p.N);
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * alpha;
        if (p.epi == EPI_BF16 || p.epi == EPI_BF16_ADD) {
          __nv_bfloat16* crow = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
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
                  v[j * 8 + e * 2] += f.x;
                  v[j * 8 + e * 2 + 1] += f.y;
                }
              }
            } else {
              for (int i = 0; i < 32 && col0 + i < p.N; ++i) v[i] += __bfloat162float(arow[i]);
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
          float* crow = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
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
            for (int i = 0; i < 32 && col0 + i < p.N; ++i)
              crow[i] = (p.epi == EPI_F32_ACC ? crow[i] : 0.f) + v[i];
          }
        }
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
int launch(const void* A, const void* B, const GemmParams& p, long long lda, long long ldb, cudaStream_t stream) {
  CUtensorMap ta, tb;
  int e;
  if (!A_MN) e = mbh::make_tmap_bf16_2d(&ta, A, p.K, p.M, lda, 64, BM);
  else e = mbh::make_tmap_bf16_2d(&ta, A, p.M, p.K, lda, 64, BK);
  if (e) return e;
  if (!B_MN) e = mbh::make_tmap_bf16_2d(&tb, B, p.K, p.N, ldb, 64, BN);
  else e = mbh::make_tmap_bf16_2d(&tb, B, p.N, p.K, ldb, 64, BK);
  if (e) return e;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemm_bf16_kernel<A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    attr_set = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < mbh::sm_count() ? tiles : mbh::sm_count();
  gemm_bf16_kernel<A_MN, B_MN><<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
  return mbh::check_launch("gemm_bf16");
}

}  // namespace

// C[M,N] = alpha * op(A) op(B)^T.  a_mn = 0: A is [M,K] row-major (pitch lda); a_mn = 1: A is [K,M].
// b_mn = 0: B is [N,K] row-major (pitch ldb); b_mn = 1: B is [K,N].  epi: see EpiMode.
// Requirements: bf16 operands, 16-byte aligned bases, pitches multiples of 8 elements.
extern "C" int mb_gemm_bf16(const void* A, const void* B, void* C, const void* aux, int M, int N, int K,
                            long long lda, long long ldb, long long ldc, long long ldaux, int a_mn, int b_mn,
                            int epi, float alpha, const float* alpha_dev, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -3;
  GemmParams p;
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
  if (!p.status) return -4;
  if (!a_mn && !b_mn) return launch<false, false>(A, B, p, lda, ldb, stream);
  if (!a_mn && b_mn) return launch<false, true>(A, B, p, lda, ldb, stream);
  if (a_mn && !b_mn) return launch<true, false>(A, B, p, lda, ldb, stream);
  return launch<true, true>(A, B, p, lda, ldb, stream);
}

extern "C" int mb_status() { return mbh::status().host ? mbh::status().host[0] : -1; }
extern "C" void mb_status_clear() {
  if (mbh::status().host) mbh::status().host[0] = 0;
}
