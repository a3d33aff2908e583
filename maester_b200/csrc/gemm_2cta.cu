// bf16 GEMM with CTA pairs: C[M,N] = alpha * op(A) * op(B)^T, 256x256 output tile per pair of SMs.
//
// The two CTAs of a cluster share one tcgen05.mma.cta_group::2 (M256 N256 K16) issued by the even
// CTA: each CTA stages its own 128 rows of A and its own 128-row half of B, so per SM only
// 32 KiB of operands enter shared memory per 64-deep k-block (48 KiB for the single-CTA kernel) and
// the tensor core reads half of B from the partner.  That relieves the shared-memory port, which
// the single-CTA 128x256 tile saturates (MMA operand reads + TMA writes).
//
// Per CTA: warp 0 = TMA producer (6-stage ring; loads use .cta_group::2 and complete on the even
// CTA's barrier, no multicast), warp 1 = MMA issuer (even CTA only) + TMEM allocation, warps 2-5 =
// epilogue over this CTA's 128 accumulator rows (two 256-column TMEM buffers, so the epilogue of
// one tile overlaps the main loop of the next).  Operand layouts as in gemm.cu.
// All mbarrier waits are bounded; both CTAs always reach the cluster barriers.
#include "gemm_common.cuh"
#include "host_common.cuh"
#include <stdlib.h>

namespace {
using namespace mb;
using namespace mbg;

constexpr int BM = 128;        // rows per CTA (256 per pair)
constexpr int BN = 256;        // tile columns (each CTA stages BN/2 rows of B)
constexpr int BNH = BN / 2;
constexpr int BK = 64;
#ifndef MB_G2_STAGES
#define MB_G2_STAGES 6
#endif
#ifndef MB_G2_GROUP_M
#define MB_G2_GROUP_M 4
#endif
constexpr int STAGES = MB_G2_STAGES;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BNH * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;  // 32 KiB
constexpr int THREADS = 192;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;  // shared::cluster address of the same offset in the even CTA

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive (+ expected bytes) on the barrier at the same offset in the even CTA of the pair
__device__ __forceinline__ void mbar_expect_tx_leader(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(smem_u32(bar) & PEER_MASK), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & PEER_MASK) : "memory");
}
// TMA load whose completion bytes are counted on the even CTA's barrier (no multicast)
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar) & PEER_MASK), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma2_bf16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n.reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(z), "r"(z), "r"(z), "r"(z), "r"(z),
        "r"(z), "r"(z), "r"(z)
      : "memory");
}
// arrive on the barrier at this offset in both CTAs once all MMAs issued so far have completed
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(mask)
      : "memory");
}

// ---- all-gather fused into the GEMM: untiled bulk copies (no multicast) and the tile counters
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(reinterpret_cast<uint64_t>(gdst)), "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool wait_counter(const int* p, int target) {
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (ld_acquire_gpu(p) < target) {
    if ((++spins & 0x3f) == 0 && globaltimer_ns() - t0 > MB_WAIT_TIMEOUT_NS) return false;
  }
  return true;
}

// Work unit u -> (tile in rasterisation order, slice sp of nsp of the contraction).  Plain split: all tiles' first
// slices run before any second slice.  Hybrid split: the tiles of the whole waves first, one unit each, then the
// slices of the tail tiles.  Grouped weight gradients: sp is the group.
__device__ __forceinline__ void unit_decode(const GemmParams& p, int u, int num_tiles, int splits, int& tile, int& sp,
                                            int& nsp) {
  if (!p.grp_offs && p.tail_splits > 0) {
    if (u < p.full_tiles) {
      tile = u;
      sp = 0;
      nsp = 1;
    } else {
      const int v = u - p.full_tiles, tail = num_tiles - p.full_tiles;
      tile = p.full_tiles + v % tail;
      sp = v / tail;
      nsp = p.tail_splits;
    }
    return;
  }
  tile = u % num_tiles;
  sp = u / num_tiles;
  nsp = splits;
}

// k-block range of a work unit: slice `sp` of a split contraction, or (grouped weight gradients) the rows of group
// `sp`, whose offsets are multiples of 128 rows
__device__ __forceinline__ void unit_krange(const GemmParams& p, int sp, int kblocks, int splits, int& kb0, int& kb1) {
  if (p.grp_offs) {
    kb0 = p.grp_offs[sp] / BK;
    kb1 = p.grp_offs[sp + 1] / BK;
  } else {
    kb0 = sp * kblocks / splits;
    kb1 = (sp + 1) * kblocks / splits;
  }
}

// One thread of a copying CTA: its share of every remote 256-row tile of A, in the order in which the computing
// pairs reach the tiles (next rank's block first).  Shares are contiguous byte ranges; they move through the
// ring of pipeline stages in pieces of at most one stage, loads running STAGES-1 pieces ahead of the stores.
__device__ void ag_copy_rows(const GemmParams& p, uint8_t* smem, uint64_t* bars, int copier, int ncopiers, int tm) {
  const int tiles_per_rank = tm / p.ag_world;
  const long long row_bytes = p.ag_ld * 2;
  const int rows_per = (2 * BM) / ncopiers;                 // rows of each tile handled by this CTA
  const long long share = rows_per * row_bytes;
  const int pieces_per_tile = static_cast<int>((share + STAGE_BYTES - 1) / STAGE_BYTES);
  const int remote_tiles = tiles_per_rank * (p.ag_world - 1);
  const long long n = static_cast<long long>(remote_tiles) * pieces_per_tile;
  bool ok = true;
  auto piece = [&](long long j, const uint8_t*& src, uint8_t*& dst, uint32_t& bytes, int& mt) {
    const int t = static_cast<int>(j / pieces_per_tile), q = static_cast<int>(j % pieces_per_tile);
    const int owner = (p.ag_rank + 1 + t / tiles_per_rank) % p.ag_world;
    const int lt = t % tiles_per_rank;                      // tile inside the owner's block
    mt = owner * tiles_per_rank + lt;
    const long long off = (static_cast<long long>(lt) * 2 * BM + static_cast<long long>(copier) * rows_per) * row_bytes +
                          static_cast<long long>(q) * STAGE_BYTES;
    const long long left = share - static_cast<long long>(q) * STAGE_BYTES;
    bytes = static_cast<uint32_t>(left < STAGE_BYTES ? left : STAGE_BYTES);
    src = static_cast<const uint8_t*>(p.ag_src[owner]) + off;
    dst = static_cast<uint8_t*>(p.ag_dst) + static_cast<long long>(owner) * tiles_per_rank * 2 * BM * row_bytes + off;
  };
  auto issue = [&](long long j) {
    const uint8_t* src;
    uint8_t* dst;
    uint32_t bytes;
    int mt;
    piece(j, src, dst, bytes, mt);
    const int s = static_cast<int>(j % STAGES);
    mbar_expect_tx(&bars[s], bytes);
    bulk_load(smem + s * STAGE_BYTES, src, bytes, &bars[s]);
  };
  long long issued = 0, done = 0;
  for (long long j = 0; j < STAGES - 1 && j < n; ++j, ++issued) issue(j);
  for (long long i = 0; i < n && ok; ++i) {
    const int s = static_cast<int>(i % STAGES);
    if (!mbar_wait(&bars[s], static_cast<uint32_t>((i / STAGES) & 1))) {
      atomicCAS(p.status, 0, ERR_WAIT_PEER);
      ok = false;
      break;
    }
    done = i + 1;
    const uint8_t* src;
    uint8_t* dst;
    uint32_t bytes;
    int mt;
    piece(i, src, dst, bytes, mt);
    bulk_store(dst, smem + s * STAGE_BYTES, bytes);
    tma_store_commit();
    if ((i + 1) % pieces_per_tile == 0) {   // this CTA's share of tile mt is on its way: publish it once it has landed
      tma_store_wait<0>();
      asm volatile("fence.proxy.async;" ::: "memory");
      red_release_gpu_add(p.ag_flags + mt, 1);
    }
    const long long j = i + STAGES - 1;
    if (j < n) {
      tma_store_wait_read<1>();             // the store that last read stage j % STAGES (piece i - 1) is done with it
      issue(j);
      ++issued;
    }
  }
  tma_store_wait<0>();
  // after a timeout: give the loads still in flight one more bounded wait each before the CTA may exit
  for (long long i = done; i < issued; ++i)
    (void)mbar_wait(&bars[i % STAGES], static_cast<uint32_t>((i / STAGES) & 1), 200000000ull);
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                         // [STAGES]  used in the even CTA only
  uint64_t* empty = bars + STAGES;               // [STAGES]  one per CTA
  uint64_t* acc_full = bars + 2 * STAGES;        // [2]       one per CTA
  uint64_t* acc_empty = bars + 2 * STAGES + 2;   // [2]       used in the even CTA only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();        // 0 = even CTA (issues the MMAs), 1 = partner
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
  const int tm = (p.M + 2 * BM - 1) / (2 * BM), tn = (p.N + BN - 1) / BN;
  const int num_tiles = p.syrk ? tm * (tm + 1) / 2 : tm * tn;  // symmetric update: tiles on and below the diagonal
  const int kblocks = (p.K + BK - 1) / BK;
  // work unit u = (tile u % num_tiles, k-range u / num_tiles): all tiles' first ranges run before any
  // second range, so partial sums of one tile rarely meet in the reduction atomics
  const int splits = p.splits > 1 ? p.splits : 1;
  // grouped weight gradients: unit u = (tile u % num_tiles, group u / num_tiles), contraction over the group's rows
  const int num_units = (!p.grp_offs && p.tail_splits > 0)
                            ? p.full_tiles + (num_tiles - p.full_tiles) * p.tail_splits
                            : num_tiles * (p.grp_offs ? p.grp_count : splits);
  // fused all-gather: the last `copiers` pairs copy; the tile order is rotated so that this rank's rows come first
  const int copiers = p.ag_world > 1 ? p.ag_copiers : 0;
  const int gpairs = npairs - copiers;
  const int mt_rot = p.ag_world > 1 ? p.ag_rank * (tm / p.ag_world) : 0;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 2);    // one arrive.expect_tx from each CTA's producer
      mbar_init(&empty[s], 1);   // multicast commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);     // multicast commit
      mbar_init(&acc_empty[a], 256);  // epilogue threads of both CTAs
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc2(tmem_slot, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // partner's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (pair < copiers) {  // lowest block indices: dispatched first
    if (threadIdx.x == 0)
      ag_copy_rows(p, smem, empty, pair * 2 + static_cast<int>(cta), 2 * copiers, tm);
  } else if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int u = pair - copiers; u < num_units && ok; u += gpairs) {
        int mt, nt, tile, sp, nsp;
        unit_decode(p, u, num_tiles, splits, tile, sp, nsp);
        if (p.syrk) tri_coords(tile, mt, nt);
        else tile_coords(tile, tm, tn, p.group_m, mt, nt);
        mt = (mt + mt_rot) % tm;
        if (copiers > 0 && mt / (tm / p.ag_world) != p.ag_rank) {
          // rows of another rank: every copying CTA has to have delivered its share of this tile
          if (!wait_counter(p.ag_flags + mt, 2 * copiers)) {
            atomicCAS(p.status, 0, ERR_WAIT_PEER);
            ok = false;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        int kb0, kb1;
        unit_krange(p, sp, kblocks, nsp, kb0, kb1);
        const int m0 = mt * 2 * BM + static_cast<int>(cta) * BM;
        // gated forward: the even CTA stages 128 gate rows of the fused weight, the odd CTA the matching up rows
        const int n0 = p.glu_mode == 1 ? nt * BNH + static_cast<int>(cta) * p.glu_F : nt * BN + static_cast<int>(cta) * BNH;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1)) {
            atomicCAS(p.status, 0, ERR_WAIT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx_leader(&full[s], STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d_pair(sa, &tmap_a, &full[s], k0, m0);
          } else {
#pragma unroll
            for (int b = 0; b < BM / 64; ++b) tma_load_2d_pair(sa + b * (BK * 128), &tmap_a, &full[s], m0 + b * 64, k0);
          }
          if (!B_MN) {
            tma_load_2d_pair(sb, &tmap_b, &full[s], k0, n0);
          } else {
#pragma unroll
            for (int b = 0; b < BNH / 64; ++b) tma_load_2d_pair(sb + b * (BK * 128), &tmap_b, &full[s], n0 + b * 64, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int u = pair - copiers; u < num_units && ok; u += gpairs) {
        int kb0, kb1, tile, sp, nsp;
        unit_decode(p, u, num_tiles, splits, tile, sp, nsp);
        unit_krange(p, sp, kblocks, nsp, kb0, kb1);
        if (kb0 == kb1) continue;  // a group without rows: no accumulator is produced (the epilogue skips it too)
        const uint32_t acc = tcount & 1, acc_ph = (tcount >> 1) & 1;
        ++tcount;
        if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1)) {
          atomicCAS(p.status, 0, ERR_WAIT_ACC_EMPTY);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
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
            const uint64_t da = A_MN ? make_smem_desc(sa + k * 2048, BK * 128, 1024)
                                     : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc(sb + k * 2048, BK * 128, 1024)
                                     : make_smem_desc(sb + k * 32, 16, 1024);
            umma2_bf16_ss(d_tmem, da, db, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          umma2_commit_both(&empty[s]);
        }
        if (ok) umma2_commit_both(&acc_full[acc]);
      }
    }
  } else {
    const int q = warp & 3;
    const float alpha = p.alpha * (p.alpha_dev ? __ldg(p.alpha_dev) : 1.f);
    uint32_t tcount = 0;
    bool ok = true;
    long long c_off = 0;  // per-unit output base for grouped weight gradients
    for (int u = pair - copiers; u < num_units && ok; u += gpairs) {
      int mt, nt, tile, sp, nsp;
      unit_decode(p, u, num_tiles, splits, tile, sp, nsp);
      if (p.syrk) tri_coords(tile, mt, nt);
      else tile_coords(tile, tm, tn, p.group_m, mt, nt);
      mt = (mt + mt_rot) % tm;
      if (p.grp_offs) {
        int kb0, kb1;
        unit_krange(p, sp, kblocks, nsp, kb0, kb1);
        if (kb0 == kb1) continue;
        c_off = static_cast<long long>(sp) * p.grp_c_elems;
      }
      // hybrid split: whole tiles add to C with a plain read-modify-write, slices of the tail tiles with atomics
      const int epi_unit = (p.tail_splits > 0 && !p.grp_offs) ? (nsp == 1 ? EPI_F32_ACC : EPI_F32_RED) : -1;
      const uint32_t acc = tcount & 1, acc_ph = (tcount >> 1) & 1;
      ++tcount;
      if (!mbar_wait(&acc_full[acc], acc_ph)) {
        atomicCAS(p.status, 0, ERR_WAIT_ACC_FULL);
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = mt * 2 * BM + static_cast<int>(cta) * BM + q * 32 + lane;
      const int n0 = nt * BN;
      const uint32_t taddr = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      if (p.glu_mode == 1) {
#pragma unroll 1
        for (int c = 0; c < BNH / 32; ++c) {  // columns [0, 128): gate units nt*128 .., columns [128, 256): the same up units
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(taddr + c * 32, rg);
          tmem_ld_32x32(taddr + BNH + c * 32, ru);
          tmem_ld_wait();
          store_glu_fwd_chunk(p, rg, ru, alpha, row, nt * BNH + c * 32);
        }
      } else if (p.glu_mode == 2) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          store_glu_bwd_chunk(p, r, alpha, row, n0 + c * 32);
        }
      } else if (p.ce_mode) {
        float m = -INFINITY, s = 0.f;
        const long long lab = row < p.M ? p.ce_labels[row] - p.ce_v0 : -1;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          ce_stats_chunk(p, r, alpha, row, n0 + c * 32, lab, m, s);
        }
        if (row < p.M) p.ce_stats[static_cast<long long>(nt) * p.ce_ld + row] = make_float2(m, s);
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          store_acc_chunk(p, r, alpha, row, n0 + c * 32, c_off, epi_unit);
          if (p.syrk && nt < mt) store_acc_chunk_mirrored(p, r, alpha, row, n0 + c * 32);
        }
      }
      tc_fence_before();
      mbar_arrive_leader(&acc_empty[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the partner may still touch its memory or barriers
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc2(tmem_base, 512);
  }
}


// Rasterisation group: row-tiles swept together across all column tiles.  Measured on B200 over the
// forward / dgrad / wgrad shapes of Gemma-3 4B and Llama-3 8B the throughput is flat in the group size
// (within 2 %) except for very wide outputs with a short contraction (gate|up projection: N = 20480,
// K = 2560), where 8 row-tiles beat 4 by 3.5 %: more rows share each streamed column block of B.
int choose_group_m(int M, int N, int K) {
  if (const char* env = getenv("MB_GEMM_GROUP_M")) {  // manual override for tuning runs (read at every launch)
    const int g = atoi(env);
    if (g > 0) return g;
  }
  (void)M;
  const int tn = (N + BN - 1) / BN;
  return (tn >= 64 && K <= 3072) ? 8 : MB_G2_GROUP_M;
}

template <bool A_MN, bool B_MN>
int launch2(const void* A, const void* B, const GemmParams& p, long long lda, long long ldb, cudaStream_t stream) {
  CUtensorMap ta, tb;
  int e;
  if (!A_MN) e = mbh::make_tmap_bf16_2d(&ta, A, p.K, p.M, lda, 64, BM);
  else e = mbh::make_tmap_bf16_2d(&ta, A, p.M, p.K, lda, 64, BK);
  if (e) return e;
  if (!B_MN) e = mbh::make_tmap_bf16_2d(&tb, B, p.K, p.N, ldb, 64, BNH);
  else e = mbh::make_tmap_bf16_2d(&tb, B, p.N, p.K, ldb, 64, BK);
  if (e) return e;
  GemmParams pp = p;
  pp.group_m = choose_group_m(p.M, p.N, p.K);
  MB_SET_MAX_SMEM_ONCE((gemm_bf16_2cta_kernel<A_MN, B_MN>), SMEM_BYTES);
  const int tm_h = (p.M + 2 * BM - 1) / (2 * BM);
  const int out_tiles = p.syrk ? tm_h * (tm_h + 1) / 2 : tm_h * ((p.N + BN - 1) / BN);
  const int tiles = (!p.grp_offs && p.tail_splits > 0)
                        ? p.full_tiles + (out_tiles - p.full_tiles) * p.tail_splits
                        : out_tiles * (p.grp_offs ? p.grp_count : (p.splits > 1 ? p.splits : 1));
  const int cop = p.ag_world > 1 ? p.ag_copiers : 0;  // pairs that copy instead of computing (fused all-gather)
  const int max_pairs = mbh::sm_count() / 2 - cop;    // every CTA of the grid is resident: waiting on one another is safe
  if (max_pairs < 1) return -3;
  const int pairs = (tiles < max_pairs ? tiles : max_pairs) + cop;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t err = cudaLaunchKernelEx(&cfg, gemm_bf16_2cta_kernel<A_MN, B_MN>, ta, tb, pp);
  if (err != cudaSuccess) {
    fprintf(stderr, "maester_b200: cluster launch of gemm_bf16_2cta failed: %s\n", cudaGetErrorString(err));
    return -100 - static_cast<int>(err);
  }
  return mbh::check_launch("gemm_bf16_2cta");
}

}  // namespace

// Same contract as mb_gemm_bf16 (gemm.cu); uses CTA pairs.
extern "C" int mb_gemm_bf16_2cta(const void* A, const void* B, void* C, const void* aux, int M, int N, int K,
                                 long long lda, long long ldb, long long ldc, long long ldaux, int a_mn, int b_mn,
                                 int epi, float alpha, float beta, const float* alpha_dev, cudaStream_t stream) {
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
  p.beta = beta;
  p.status = mbh::status().dev;
  if (!p.status) return -4;
  p.splits = 1;
  p.route_rows = 0;
  if (epi == EPI_F32_ACC && (ldc & 3) == 0) {
    // Accumulating epilogue (weight gradients): few output tiles and a long contraction leave most of
    // the last wave idle.  Cut the contraction so that tiles x splits fills the waves; partial sums
    // meet in C through reduction atomics.  Cost model: waves x (k-blocks per unit + fixed overhead).
    const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
    const int pairs = mbh::sm_count() / 2;
    const int kblocks = (K + BK - 1) / BK;
    const int overhead = 8;
    long long best = static_cast<long long>((tiles + pairs - 1) / pairs) * (kblocks + overhead);
    for (int s = 2; s <= 16 && s * 8 <= kblocks; ++s) {
      const long long cost = static_cast<long long>((tiles * s + pairs - 1) / pairs) * ((kblocks + s - 1) / s + overhead);
      if (cost * 100 < best * 97) {
        best = cost;
        p.splits = s;
      }
    }
    // Hybrid: whole waves un-cut, only the tiles of the last partial wave cut (fewer atomics, fewer pipeline ramps).
    const int full = (tiles / pairs) * pairs, tail = tiles - full;
    if (full > 0 && tail > 0) {
      int st = pairs / tail;
      if (st > 16) st = 16;
      if (st * 8 > kblocks) st = kblocks / 8;
      if (st >= 2) {
        const long long cost = static_cast<long long>(tiles / pairs) * (kblocks + overhead) +
                               static_cast<long long>((tail * st + pairs - 1) / pairs) * ((kblocks + st - 1) / st + overhead);
        static const bool allow = !(getenv("MB_GEMM_HYBRID_SPLIT") && atoi(getenv("MB_GEMM_HYBRID_SPLIT")) == 0);
        if (allow && cost * 100 < best * 99) {
          p.splits = 1;
          p.full_tiles = full;
          p.tail_splits = st;
        }
      }
    }
    if (p.splits > 1 || p.tail_splits > 0) p.epi = EPI_F32_RED;
  }
  if (!a_mn && !b_mn) return launch2<false, false>(A, B, p, lda, ldb, stream);
  if (!a_mn && b_mn) return launch2<false, true>(A, B, p, lda, ldb, stream);
  if (a_mn && !b_mn) return launch2<true, false>(A, B, p, lda, ldb, stream);
  return launch2<true, true>(A, B, p, lda, ldb, stream);
}

// GEMM fused with a reduce-scatter over NVLink peer memory (row-parallel linears of tensor
// parallelism, and the input-gradient GEMMs of column-parallel ones): every rank computes the full
// [M, N] partial product, and the epilogue stores each 128-row slice of a tile straight into the
// buffer of the rank that owns those rows (M / world consecutive rows per rank), in this rank's slot
// of that buffer [world, M / world, N].  Tile by tile the stores overlap the math of the next tile;
// the owner then sums its world slots (mb_sum_partials).  No atomics: the result is deterministic.
// The caller brackets the launch with cross-rank barriers.
extern "C" int mb_gemm_bf16_rs(const void* A, const void* B, void* const* peer_out, int world, int my_rank, int M,
                               int N, int K, long long lda, long long ldb, long long ldc, int a_mn, int b_mn,
                               float alpha, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 1 || world > 8 || M % world) return -3;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -3;
  GemmParams p;
  p.C = peer_out[my_rank];
  p.aux = nullptr;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  p.ldaux = 0;
  p.epi = EPI_BF16;
  p.alpha = alpha;
  p.alpha_dev = nullptr;
  p.beta = 0.f;
  p.status = mbh::status().dev;
  if (!p.status) return -4;
  p.splits = 1;
  for (int r = 0; r < 8; ++r) p.route_base[r] = r < world ? peer_out[r] : nullptr;
  p.route_rows = M / world;
  p.route_slot = my_rank;
  if (!a_mn && !b_mn) return launch2<false, false>(A, B, p, lda, ldb, stream);
  if (!a_mn && b_mn) return launch2<false, true>(A, B, p, lda, ldb, stream);
  if (a_mn && !b_mn) return launch2<true, false>(A, B, p, lda, ldb, stream);
  return launch2<true, true>(A, B, p, lda, ldb, stream);
}

// All-gather fused into the GEMM (column-parallel linears of tensor parallelism with sequence-sharded
// activations): C = A @ op(B)^T where A is [M, K] row-major and rows [r * M / world, (r + 1) * M / world) belong to
// rank r.  `a_full` is this rank's [M, K] buffer whose own block is already in place; peer_src[r] points at rank
// r's block ([M / world, K], contiguous) in peer-mapped memory.  `copiers` CTA pairs pull the remote blocks over
// NVLink with bulk copies while the other pairs compute, starting with the local rows; a remote 256-row tile is
// consumed as soon as its counter in `flags` ([M / 256] ints, zeroed here) shows that every share has landed.
// The caller makes sure (cross-rank barrier) that the peers' blocks are complete before the launch and are
// not overwritten before all ranks have finished.
namespace {
// Fills the all-gather fields of `p` (whose output / epilogue fields are set by the caller) and launches.
int ag_launch(GemmParams& p, void* a_full, void* const* peer_src, int world, int my_rank, const void* B, long long ldb,
              int b_mn, int copiers, int* flags, cudaStream_t stream) {
  const int M = p.M, K = p.K;
  if (world < 2 || world > 8 || M % (world * 2 * BM) || (K & 7)) return -3;
  if (copiers != 1 && copiers != 2 && copiers != 4 && copiers != 8) return -3;
  if ((ldb & 7) || (reinterpret_cast<uintptr_t>(a_full) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  p.aux = nullptr;
  p.ldaux = 0;
  p.epi = EPI_BF16;
  p.alpha = 1.f;
  p.alpha_dev = nullptr;
  p.beta = 0.f;
  p.status = mbh::status().dev;
  if (!p.status) return -4;
  p.splits = 1;
  p.route_rows = 0;
  p.ag_world = world;
  p.ag_rank = my_rank;
  p.ag_copiers = copiers;
  for (int r = 0; r < 8; ++r) {
    p.ag_src[r] = r < world ? peer_src[r] : nullptr;
    if (r < world && r != my_rank && (!peer_src[r] || (reinterpret_cast<uintptr_t>(peer_src[r]) & 15))) return -3;
  }
  p.ag_dst = a_full;
  p.ag_ld = K;
  p.ag_flags = flags;
  if (cudaMemsetAsync(flags, 0, sizeof(int) * (M / (2 * BM)), stream) != cudaSuccess) return -5;
  if (b_mn) return launch2<false, true>(a_full, B, p, K, ldb, stream);
  return launch2<false, false>(a_full, B, p, K, ldb, stream);
}
}  // namespace

extern "C" int mb_gemm_bf16_ag(void* a_full, void* const* peer_src, int world, int my_rank, const void* B, void* C,
                               int M, int N, int K, long long ldb, long long ldc, int b_mn, int copiers, int* flags,
                               cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  GemmParams p;
  p.C = C;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldc;
  return ag_launch(p, a_full, peer_src, world, my_rank, B, ldb, b_mn, copiers, flags, stream);
}

// The all-gather GEMM with a gated-linear-unit epilogue (GemmParams::glu_mode), for tensor-parallel MLPs:
//  glu_mode 1: B = fused weight [gate rows | up rows] ([2F, K], K-major); C = [gate | up] ([M, 2F], pitch ldc, may be
//              null) and io = act(gate) * up ([M, F], pitch ld_io).
//  glu_mode 2: the gathered A is dy [M, K], B = down-projection weight [K, F] (b_mn layout); io = the saved [gate | up]
//              ([M, 2F], pitch ld_io) and C = d[gate | up] ([M, 2F], pitch ldc).
extern "C" int mb_gemm_bf16_ag_glu(void* a_full, void* const* peer_src, int world, int my_rank, const void* B,
                                   void* C, int M, int F, int K, long long ldb, long long ldc, int copiers, int* flags,
                                   int glu_mode, int act, void* io, long long ld_io, cudaStream_t stream) {
  if (M <= 0 || F <= 0 || K <= 0) return 0;
  if ((glu_mode != 1 && glu_mode != 2) || (ldc & 7) || (ld_io & 7) || (reinterpret_cast<uintptr_t>(io) & 15) ||
      (C && (reinterpret_cast<uintptr_t>(C) & 15)))
    return -3;
  if (glu_mode == 1 ? (F % BNH) != 0 : (F % 32) != 0) return -3;
  if (glu_mode == 2 && !C) return -3;
  GemmParams p;
  p.C = C;
  p.M = M;
  p.N = glu_mode == 1 ? 2 * F : F;
  p.K = K;
  p.ldc = ldc;
  p.glu_mode = glu_mode;
  p.glu_act = act;
  p.glu_F = F;
  if (glu_mode == 1) {
    p.glu_out = io;
    p.glu_ldo = ld_io;
  } else {
    p.glu_in = io;
    p.glu_ldi = ld_io;
  }
  return ag_launch(p, a_full, peer_src, world, my_rank, B, ldb, glu_mode == 2, copiers, flags, stream);
}

// Grouped GEMM over the contraction range on CTA pairs (weight gradients of stacked expert weights):
//   C_g[M, N] (+)= A_g^T B_g with A: [rows_cap, M] and B: [rows_cap, N] row-major, rows grouped by offs (device,
//   multiples of 128); C stacked [num_groups, M, N] with row pitch ldc.  epi: EPI_F32 / EPI_F32_ACC (fp32 output);
//   the accumulating form uses reduction atomics, one addition per element per call.  Groups without rows are skipped.
extern "C" int mb_gemm_bf16_2cta_grouped_contr(const void* A, const void* B, void* C, const int* offs, int num_groups,
                                               int rows_cap, int M, int N, long long lda, long long ldb, long long ldc,
                                               int epi, float alpha, cudaStream_t stream) {
  if (rows_cap <= 0 || N <= 0 || M <= 0 || num_groups <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (rows_cap % 128) || (epi != EPI_F32 && epi != EPI_F32_ACC)) return -3;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  GemmParams p;
  p.C = C;
  p.aux = nullptr;
  p.M = M;
  p.N = N;
  p.K = rows_cap;
  p.ldc = ldc;
  p.ldaux = 0;
  p.epi = (epi == EPI_F32_ACC && (ldc & 3) == 0) ? EPI_F32_RED : epi;
  p.alpha = alpha;
  p.alpha_dev = nullptr;
  p.beta = 1.f;
  p.status = mbh::status().dev;
  if (!p.status) return -4;
  p.splits = 1;
  p.route_rows = 0;
  p.grp_offs = offs;
  p.grp_count = num_groups;
  p.grp_c_elems = static_cast<long long>(M) * ldc;
  return launch2<true, true>(A, B, p, lda, ldb, stream);
}

// Gated linear unit fused into the GEMM epilogue (see GemmParams::glu_mode).
//  forward : gate_up[M, 2F] (may be null) and act_out[M, F] from x[M, K] and the fused weight w[2F, K]:
//            act_out = act(x w_gate^T) * (x w_up^T).  F must be a multiple of 128.
//  backward: d_gate_up[M, 2F] from dy[M, K], the down-projection weight w[K, F] (b_mn layout) and the saved
//            gate_up: d(act) = dy w, then the activation's derivative.  F must be a multiple of 32.
extern "C" int mb_gemm_glu_fwd(const void* x, const void* w, void* gate_up, void* act_out, int M, int F, int K,
                               long long ldx, long long ldw, long long ldgu, long long ldo, int act,
                               cudaStream_t stream) {
  if (M <= 0 || F <= 0 || K <= 0) return 0;
  if ((F % BNH) || (ldx & 7) || (ldw & 7) || (ldgu & 7) || (ldo & 7)) return -3;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      (reinterpret_cast<uintptr_t>(gate_up) & 15) || (reinterpret_cast<uintptr_t>(act_out) & 15))
    return -3;
  GemmParams p;
  p.C = gate_up;
  p.aux = nullptr;
  p.M = M;
  p.N = 2 * F;
  p.K = K;
  p.ldc = ldgu;
  p.ldaux = 0;
  p.epi = EPI_BF16;
  p.alpha = 1.f;
  p.alpha_dev = nullptr;
  p.beta = 0.f;
  p.status = mbh::status().dev;
  if (!p.status) return -4;
  p.splits = 1;
  p.route_rows = 0;
  p.glu_mode = 1;
  p.glu_act = act;
  p.glu_F = F;
  p.glu_out = act_out;
  p.glu_ldo = ldo;
  return launch2<false, false>(x, w, p, ldx, ldw, stream);
}

extern "C" int mb_gemm_glu_bwd(const void* dy, const void* w, const void* gate_up, void* d_gate_up, int M, int F,
                               int K, long long lddy, long long ldw, long long ldgu, long long lddgu, int act,
                               cudaStream_t stream) {
  if (M <= 0 || F <= 0 || K <= 0) return 0;
  if ((F % 32) || (lddy & 7) || (ldw & 7) || (ldgu & 7) || (lddgu & 7)) return -3;
  if ((reinterpret_cast<uintptr_t>(dy) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      (reinterpret_cast<uintptr_t>(gate_up) & 15) || (reinterpret_cast<uintptr_t>(d_gate_up) & 15))
    return -3;
  GemmParams p;
  p.C = d_gate_up;
  p.aux = nullptr;
  p.M = M;
  p.N = F;
  p.K = K;
  p.ldc = lddgu;
  p.ldaux = 0;
  p.epi = EPI_BF16;
  p.alpha = 1.f;
  p.alpha_dev = nullptr;
  p.beta = 0.f;
  p.status = mbh::status().dev;
  if (!p.status) return -4;
  p.splits = 1;
  p.route_rows = 0;
  p.glu_mode = 2;
  p.glu_act = act;
  p.glu_F = F;
  p.glu_in = gate_up;
  p.glu_ldi = ldgu;
  return launch2<false, true>(dy, w, p, lddy, ldw, stream);
}

// Symmetric rank-k update on CTA pairs: C[M, M] = alpha * A A^T (+ beta * aux), A: [M, K] row-major bf16, C and aux
// bf16.  Only the 256x256 tiles on and below the diagonal are computed (about half of the FLOPs of the full product);
// tiles below the diagonal are stored twice, once transposed.  The reference does the same with its Triton kernel
// (maester/optimizers/muon_/syrk.py:9-125).
extern "C" int mb_syrk_bf16(const void* A, void* C, const void* aux, int M, int K, long long lda, long long ldc,
                            long long ldaux, float alpha, float beta, cudaStream_t stream) {
  if (M <= 0 || K <= 0) return 0;
  if ((lda & 7) || (reinterpret_cast<uintptr_t>(A) & 15)) return -3;
  GemmParams p;
  p.C = C;
  p.aux = aux;
  p.M = M;
  p.N = M;
  p.K = K;
  p.ldc = ldc;
  p.ldaux = ldaux;
  p.epi = aux ? EPI_BF16_ADD : EPI_BF16;
  p.alpha = alpha;
  p.alpha_dev = nullptr;
  p.beta = beta;
  p.status = mbh::status().dev;
  if (!p.status) return -4;
  p.splits = 1;
  p.route_rows = 0;
  p.syrk = 1;
  return launch2<false, false>(A, A, p, lda, lda, stream);
}

// Logits with cross-entropy statistics (see GemmParams::ce_mode): logits[M, N] = bf16(scale * h w^T) (may be null),
// stats[tile, row] = (max, sum exp) of every 256-column tile (tile pitch stats_ld >= M rows), tgt[row] = the logit at
// column labels[row] - v0 when that column is in [0, N), else 0.
extern "C" int mb_gemm_ce(const void* h, const void* w, void* logits, const long long* labels, void* stats, float* tgt,
                          int M, int N, int K, long long ldh, long long ldw, long long ldl, long long v0, float scale,
                          long long stats_ld, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((ldh & 7) || (ldw & 7) || (reinterpret_cast<uintptr_t>(h) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      (reinterpret_cast<uintptr_t>(stats) & 7) || stats_ld < M)
    return -3;
  if (logits && (reinterpret_cast<uintptr_t>(logits) & 15)) return -3;
  if (cudaMemsetAsync(tgt, 0, sizeof(float) * static_cast<size_t>(M), stream) != cudaSuccess) return -5;
  GemmParams p;
  p.C = logits;
  p.aux = nullptr;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldc = ldl;
  p.ldaux = 0;
  p.epi = EPI_BF16;
  p.alpha = scale;
  p.alpha_dev = nullptr;
  p.beta = 0.f;
  p.status = mbh::status().dev;
  if (!p.status) return -4;
  p.splits = 1;
  p.route_rows = 0;
  p.ce_mode = 1;
  p.ce_labels = labels;
  p.ce_v0 = v0;
  p.ce_stats = static_cast<float2*>(stats);
  p.ce_ld = stats_ld;
  p.ce_tgt = tgt;
  return launch2<false, false>(h, w, p, ldh, ldw, stream);
}
