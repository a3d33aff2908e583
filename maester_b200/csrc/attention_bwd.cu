// Attention backward on tcgen05, as three kernels:
//   1. delta[b,h,q] = sum_d O[q,d] * dO[q,d]
//   2. dQ kernel   : one CTA per 128 query rows of one (batch, q-head); loops over kv blocks of 64:
//                    S = Q K^T and dP = dO V^T into TMEM, the softmax warps form
//                    dS = P * (dP - delta) * scale (bf16, shared memory), then dQ += dS K.
//   3. dK/dV kernel: one CTA per 128 kv rows of one (batch, kv-head[, half of the head dim when
//                    head_dim = 256]); loops over the q-heads of the GQA group and over query tiles
//                    of 64: S^T = K Q^T, dP^T = V dO^T, P^T and dS^T to shared memory, then
//                    dV += P^T dO and dK += dS^T Q.  The 256-wide head is split in two CTAs because
//                    dK, dV, S^T and dP^T must share the 512 TMEM columns.
// P is recomputed from the saved log-sum-exp.  Masks as in the forward kernel: per-row intervals (kv_start for
// query rows, q_end for kv rows) when given, else window / causal bounds computed here plus an element-wise
// document-id comparison.
// Gradients are written into one packed buffer [T, (H + 2 KV) * hd] (q heads, k heads, v heads).
#include "host_common.cuh"
#include "sm100.cuh"
#include <limits.h>
#include <math.h>
#include <atomic>

namespace {
using namespace mb;

constexpr int BWD_THREADS = 352;     // warps 0-7: element-wise stage (two threads per row), 8: TMA, 9-10: MMA issue
constexpr int EW_THREADS = 256;
constexpr int WARP_TMA = 8, WARP_MMA = 9;
// MMA issue: one thread cannot issue faster than one MMA per ~54 cycles (measured) while an M128 N64 K16 product
// takes 32, so two threads issue, split by role: warp 9 issues the score products (S or S^T) of every block, warp 10
// the dP (dP^T) products and the accumulating products (dQ, or dV and dK).  Every mbarrier therefore still has
// consumers that see all of its phases in order.  Products of different threads that touch the same tensor-memory
// buffer are ordered by "issued" barriers (arrive after issuing, tcgen05 fences on both sides): the pipe executes
// in issue order.
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct BwdParams {
  const float* lse;      // [B,H,S] natural log
  const float* delta;    // [B,H,S]
  __nv_bfloat16* dqkv;   // packed gradients
  long long g_stride;    // row pitch of dqkv (elements)
  const int* doc;        // [B,S] or null
  const int* kv_lo_blk;  // [B, ceil(S/128)] or null   (dQ kernel)
  const int* q_hi_blk;   // [B, ceil(S/128)] or null   (dK/dV kernel): exclusive upper bound on q
  const int* kv_start;   // [B, S] or null: lowest kv index a query row may attend to (window, document start folded in)
  const int* q_end;      // [B, S] or null: exclusive upper bound on the query rows that may attend to a kv row
  int B, S, H, KV;
  int causal, window;
  float scale, scale_log2;
  int* status;
};

// ---------------------------------------------------------------------------------- delta
__global__ void __launch_bounds__(256) attn_delta_kernel(const __nv_bfloat16* __restrict__ o,
                                                        const __nv_bfloat16* __restrict__ dout,
                                                        float* __restrict__ delta, int B, int S, int H, int hd) {
  const long long item = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;  // (b, s, h)
  const int lane = threadIdx.x & 31;
  const long long items = static_cast<long long>(B) * S * H;
  if (item >= items) return;
  const __nv_bfloat16* op = o + item * hd;
  const __nv_bfloat16* dp = dout + item * hd;
  float acc = 0.f;
  for (int c = lane * 2; c < hd; c += 64) {
    float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(op + c));
    float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dp + c));
    acc += a.x * d.x + a.y * d.y;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) {
    const int h = static_cast<int>(item % H);
    const long long bs = item / H;
    const int s = static_cast<int>(bs % S);
    const int b = static_cast<int>(bs / S);
    delta[(static_cast<long long>(b) * H + h) * S + s] = acc;
  }
}


// ---------------------------------------------------------------------------------- dQ kernel
// Per kv block n of 64:  S_n = Q K_n^T and dP_n = dO V_n^T into TMEM (two buffers each); the element-wise
// warps read both, form dS_n = P * (dP - delta) * scale and write it back INTO THE dP BUFFER as packed
// bf16 (tcgen05.st), from where it is the A operand of dQ += dS_n K_n (tcgen05.mma with A in tensor
// memory).  No shared-memory staging of dS, which pays for a second K stage at head size 256; V is
// released as soon as dP_n exists, K only after dQ_n, so the loads for block n+1 run during block n.
constexpr int BKV = 64;

__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

template <int HD, int NSTV>
struct SmemDQ {
  static constexpr int Q_BYTES = 128 * HD * 2;
  static constexpr int KV_BYTES = BKV * HD * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_DO = Q_BYTES;
  static constexpr int OFF_K = 2 * Q_BYTES;              // 2 stages
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;     // NSTV stages
  static constexpr int OFF_BAR = OFF_V + NSTV * KV_BYTES;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

template <int HD, int NSTV>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                   const BwdParams p) {
  using L = SmemDQ<HD, NSTV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* qdo_full = bars;       // 1
  uint64_t* k_full = bars + 1;     // [2]
  uint64_t* k_empty = bars + 3;    // [2]  dQ_n has read K_n
  uint64_t* v_full = bars + 5;     // [2]
  uint64_t* v_empty = bars + 7;    // [2]  dP_n has read V_n
  uint64_t* sdp_full = bars + 9;   // [2]  S_n and dP_n are in tensor memory
  uint64_t* s_empty = bars + 11;   // [2]  the element-wise warps hold S_n in registers
  uint64_t* ds_full = bars + 13;   // [2]  dS_n is in tensor memory
  uint64_t* dp_empty = bars + 15;  // [2]  dQ_n has read dS_n: the dP buffer may be overwritten
  uint64_t* dq_done = bars + 17;   // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.S + 127) / 128;
  const int qb = nqb - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.H / p.KV);
  const int q0 = qb * 128;
  const int kv_end = p.causal ? min(p.S, q0 + 128) : p.S;
  int kv_begin = 0;
  if (p.kv_lo_blk) kv_begin = p.kv_lo_blk[b * nqb + qb];
  else if (p.window >= 0) kv_begin = max(0, q0 - p.window);
  const int jb = kv_begin / BKV, je = (kv_end + BKV - 1) / BKV;
  const int nblk = je - jb;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    prefetch_tmap(&tmap_do);
    mbar_init(qdo_full, 1);
    mbar_init(dq_done, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&sdp_full[i], 2);  // one commit from each issuing thread (S_n and dP_n)
      mbar_init(&s_empty[i], EW_THREADS);
      mbar_init(&ds_full[i], EW_THREADS);
      mbar_init(&dp_empty[i], 1);
    }
    mbar_fence_init();
  }
  if (warp == WARP_MMA) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_dq = tmem_base;
  const uint32_t tmem_s = tmem_base + 256;            // 2 x 64
  const uint32_t tmem_dp = tmem_base + 256 + 2 * BKV; // 2 x 64; dS_n overwrites the start of each half

  if (warp == WARP_TMA) {
    if (lane == 0 && nblk > 0) {
      mbar_expect_tx(qdo_full, 2 * L::Q_BYTES);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        tma_load_4d(smem + L::OFF_Q + c * (128 * 128), &tmap_q, qdo_full, c * 64, h, q0, b);
        tma_load_4d(smem + L::OFF_DO + c * (128 * 128), &tmap_do, qdo_full, c * 64, h, q0, b);
      }
      bool okp = true;
      for (int n = 0; n < nblk && okp; ++n) {
        const int sk = n & 1, sv = n % NSTV;
        if (!mbar_wait(&k_empty[sk], ((n >> 1) & 1) ^ 1)) { okp = false; break; }
        mbar_expect_tx(&k_full[sk], L::KV_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_4d(smem + L::OFF_K + sk * L::KV_BYTES + c * (BKV * 128), &tmap_k, &k_full[sk], c * 64, kvh, (jb + n) * BKV, b);
        if (!mbar_wait(&v_empty[sv], ((n / NSTV) & 1) ^ 1)) { okp = false; break; }
        mbar_expect_tx(&v_full[sv], L::KV_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_4d(smem + L::OFF_V + sv * L::KV_BYTES + c * (BKV * 128), &tmap_v, &v_full[sv], c * 64, kvh, (jb + n) * BKV, b);
      }
      if (!okp) atomicCAS(p.status, 0, ERR_WAIT_EMPTY);
    }
  } else if (warp == WARP_MMA) {
    // ---- issuer A: S_n = Q K_n^T for every block
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, BKV, false, false);
      const uint64_t dq0 = make_smem_desc(smem_u32(smem + L::OFF_Q), 16, 1024);
      bool ok = mbar_wait(qdo_full, 0);
      for (int n = 0; n < nblk && ok; ++n) {
        const int sk_i = n & 1, buf = n & 1;
        const uint32_t ph = (n >> 1) & 1;
        if (!mbar_wait(&k_full[sk_i], ph) || !mbar_wait(&s_empty[buf], ph ^ 1)) {
          ok = false;
          break;
        }
        tc_fence_after();
        // descriptors are built once per tile and stepped by constants (the issuing thread is the bottleneck)
        const uint64_t dk0 = make_smem_desc(smem_u32(smem + L::OFF_K + sk_i * L::KV_BYTES), 16, 1024);
        umma_bf16_ss_c<false>(tmem_s + buf * BKV, dq0, dk0, idesc_s);
#pragma unroll
        for (int k = 1; k < HD / 16; ++k)
          umma_bf16_ss_c<true>(tmem_s + buf * BKV, smem_desc_advance(dq0, (k >> 2) * (128 * 128) + (k & 3) * 32),
                               smem_desc_advance(dk0, (k >> 2) * (BKV * 128) + (k & 3) * 32), idesc_s);
        umma_commit(&sdp_full[buf]);
      }
      if (!ok) atomicCAS(p.status, 0, ERR_WAIT_MISC);
    }
  } else if (warp == WARP_MMA + 1) {
    // ---- issuer B: dP_n = dO V_n^T (one block ahead) and dQ += dS_n K_n
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, BKV, false, false);
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, HD, false, true);
      const uint64_t ddo0 = make_smem_desc(smem_u32(smem + L::OFF_DO), 16, 1024);
      bool ok = mbar_wait(qdo_full, 0);
      auto issue_dp = [&](int n) -> bool {
        const int sv_i = n % NSTV, buf = n & 1;
        if (!mbar_wait(&v_full[sv_i], (n / NSTV) & 1)) return false;
        // (the dP buffer was last read by the dQ product of block n-2, issued earlier by this same thread: no wait)
        tc_fence_after();
        const uint64_t dv0 = make_smem_desc(smem_u32(smem + L::OFF_V + sv_i * L::KV_BYTES), 16, 1024);
        umma_bf16_ss_c<false>(tmem_dp + buf * BKV, ddo0, dv0, idesc_s);
#pragma unroll
        for (int k = 1; k < HD / 16; ++k)
          umma_bf16_ss_c<true>(tmem_dp + buf * BKV, smem_desc_advance(ddo0, (k >> 2) * (128 * 128) + (k & 3) * 32),
                               smem_desc_advance(dv0, (k >> 2) * (BKV * 128) + (k & 3) * 32), idesc_s);
        umma_commit(&v_empty[sv_i]);
        umma_commit(&sdp_full[buf]);
        return true;
      };
      if (ok) ok = issue_dp(0);
      for (int n = 0; n < nblk && ok; ++n) {
        if (n + 1 < nblk) ok = issue_dp(n + 1);
        if (!ok) break;
        const int buf = n & 1;
        // K_n has landed (the other thread waited for it too; this makes the TMA writes visible to this thread's MMAs)
        if (!mbar_wait(&ds_full[buf], (n >> 1) & 1) || !mbar_wait(&k_full[n & 1], (n >> 1) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after();
        // dS_n columns: kv 0..31 packed at the start of the first half of the dP buffer, kv 32..63 at the
        // start of its second half (each element-wise thread overwrites only columns it has read itself)
        const uint64_t dkm0 = make_smem_desc(smem_u32(smem + L::OFF_K + (n & 1) * L::KV_BYTES), BKV * 128, 1024);
        const uint32_t a0 = tmem_dp + buf * BKV;
        umma_bf16_ts(tmem_dq, a0, dkm0, idesc_dq, n != 0);
#pragma unroll
        for (int k = 1; k < BKV / 16; ++k)
          umma_bf16_ts_c<true>(tmem_dq, a0 + (k >> 1) * 32 + (k & 1) * 8, smem_desc_advance(dkm0, k * 2048), idesc_dq);
        // K_n is free once dQ_n has read it (S_n, issued by the other thread, completed before dS_n existed)
        umma_commit(&k_empty[n & 1]);
        if (n == nblk - 1) umma_commit(dq_done);
      }
      if (!ok) atomicCAS(p.status, 0, ERR_WAIT_MISC);
    }
  } else {
    const int half = warp >> 2;  // which 32 of the 64 score columns / which half of the dQ columns
    const int row = (warp & 3) * 32 + lane;
    const int q = q0 + row;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    // masks: one admissible kv interval [lo_q, hi_q] per query row (see the forward kernel); the element-wise
    // document comparison only runs when document ids are given without the interval form
    const int* docb = (p.doc && !p.kv_start) ? p.doc + static_cast<long long>(b) * p.S : nullptr;
    const int dq_doc = (docb && q < p.S) ? docb[q] : 0;
    int lo_q, hi_q;
    if (q >= p.S) {
      lo_q = INT_MAX;
      hi_q = -1;
    } else {
      hi_q = p.causal ? q : p.S - 1;
      if (p.kv_start) lo_q = p.kv_start[static_cast<long long>(b) * p.S + q];
      else lo_q = p.window >= 0 ? max(0, q - p.window) : 0;
    }
    int w_lo_max = lo_q, w_hi_min = hi_q;
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) {
      w_lo_max = max(w_lo_max, __shfl_xor_sync(0xffffffffu, w_lo_max, sh));
      w_hi_min = min(w_hi_min, __shfl_xor_sync(0xffffffffu, w_hi_min, sh));
    }
    const long long stat_idx = (static_cast<long long>(b) * p.H + h) * p.S + q;
    const float lse2 = (q < p.S) ? p.lse[stat_idx] * LOG2E : INFINITY;  // rows past the end give P = 0
    const float delta = (q < p.S) ? p.delta[stat_idx] : 0.f;
    bool ok = true;
    for (int n = 0; n < nblk && ok; ++n) {
      const int buf = n & 1;
      const int kv0 = (jb + n) * BKV;
      if (!mbar_wait(&sdp_full[buf], (n >> 1) & 1)) {
        atomicCAS(p.status, 0, ERR_WAIT_SOFTMAX);
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t rs[32], rp[32];
      tmem_ld_32x32(tmem_s + buf * BKV + half * 32 + lane_sel, rs);
      tmem_ld_32x32(tmem_dp + buf * BKV + half * 32 + lane_sel, rp);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&s_empty[buf]);  // scores are in registers: the MMA warp may refill the S buffer
      const bool need_mask = (docb != nullptr) || kv0 < w_lo_max || kv0 + BKV - 1 > w_hi_min;
      float ds[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float pr = ex2(fmaf(__uint_as_float(rs[i]), p.scale_log2, -lse2));
        ds[i] = pr * (__uint_as_float(rp[i]) - delta) * p.scale;
      }
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kv = kv0 + half * 32 + i;
          bool bad = (kv < lo_q) | (kv > hi_q);
          if (docb && kv < p.S) bad |= docb[kv] != dq_doc;
          if (bad) ds[i] = 0.f;
        }
      }
      uint32_t packed[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) packed[i] = pack_bf16(ds[2 * i], ds[2 * i + 1]);
      tmem_st_32x16(tmem_dp + buf * BKV + half * 32 + lane_sel, packed);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&ds_full[buf]);
    }
    if (ok && nblk > 0 && !mbar_wait(dq_done, 0)) {
      atomicCAS(p.status, 0, ERR_WAIT_ACC_FULL);
      ok = false;
    }
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* grow = p.dqkv + (static_cast<long long>(b) * p.S + q) * p.g_stride + static_cast<long long>(h) * HD +
                            half * (HD / 2);
#pragma unroll 1
      for (int c = 0; c < HD / 64; ++c) {
        uint32_t r[32];
        if (nblk > 0) {
          tmem_ld_32x32(tmem_dq + half * (HD / 2) + c * 32 + lane_sel, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0;
        }
        if (q < p.S) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(r[j * 8 + 0]), __uint_as_float(r[j * 8 + 1]));
            o.y = pack_bf16(__uint_as_float(r[j * 8 + 2]), __uint_as_float(r[j * 8 + 3]));
            o.z = pack_bf16(__uint_as_float(r[j * 8 + 4]), __uint_as_float(r[j * 8 + 5]));
            o.w = pack_bf16(__uint_as_float(r[j * 8 + 6]), __uint_as_float(r[j * 8 + 7]));
            reinterpret_cast<uint4*>(grow + c * 32)[j] = o;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------- dK/dV kernel
// One CTA per 128 kv rows of one (batch, kv head[, half of the head dim when head_dim = 256]); it loops
// over the q-heads of the GQA group and over query tiles of 64:
//   S^T = K Q^T and dP^T = V dO^T into TMEM  ->  P^T and dS^T written back into the same TMEM buffers as
//   packed bf16  ->  dV += P^T dO[:, slice] and dK += dS^T Q[:, slice] with the A operand in tensor memory.
// Shared memory holds K and V (resident) and the query-side tiles split by when they are last needed:
// the channels of this CTA's output slice (needed until dV / dK, two stages) and the other channels
// (needed only for S^T / dP^T, one stage released early).  So the loads of tile n+1 run during tile n.
constexpr int BQ2 = 64;

template <int HD, int DV>
struct SmemKV {
  static constexpr int EARLY = HD - DV;                  // channels not in this CTA's output slice
  static constexpr int KV_BYTES = 128 * HD * 2;
  static constexpr int LATE_BYTES = BQ2 * DV * 2;        // one of Q / dO, slice channels
  static constexpr int EARLY_BYTES = BQ2 * EARLY * 2;    // one of Q / dO, other channels
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = KV_BYTES;
  static constexpr int OFF_QL = 2 * KV_BYTES;            // [2 stages][Q late | dO late]
  static constexpr int OFF_QE = OFF_QL + 2 * 2 * LATE_BYTES;  // [Q early | dO early]
  static constexpr int OFF_STAT = OFF_QE + 2 * EARLY_BYTES;   // [2][2][BQ2] floats
  static constexpr int OFF_BAR = OFF_STAT + 2 * 2 * BQ2 * 4;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

template <int HD, int DV, int NSTQ>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                     const BwdParams p) {
  using L = SmemKV<HD, DV>;
  constexpr int NSPLIT = HD / DV;
  constexpr bool HAS_EARLY = L::EARLY > 0;
  constexpr int LATE_BLKS = DV / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* kv_full = bars;         // 1
  uint64_t* ql_full = bars + 1;     // [2]  slice channels of Q and dO
  uint64_t* ql_empty = bars + 3;    // [2]  dV_n and dK_n have read them
  uint64_t* qe_full = bars + 5;     // 1    other channels
  uint64_t* qe_empty = bars + 6;    // 1    S^T_n and dP^T_n have read them
  uint64_t* sdp_full = bars + 7;    // [2]
  uint64_t* pt_full = bars + 9;     // [2]  P^T_n and dS^T_n are in tensor memory
  uint64_t* acc_free = bars + 11;   // [2]  dV_n and dK_n have read them: the S^T / dP^T buffers are free
  uint64_t* acc_done = bars + 13;   // 1
  uint64_t* stat_bar = bars + 14;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  uint64_t* acc_issued = bars + 18; // [2]  the dV / dK products that read the S^T / dP^T buffers have been issued
  float* stat = reinterpret_cast<float*>(smem + L::OFF_STAT);  // [buf][0: lse2, 1: delta][BQ2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = (p.S + 127) / 128;
  const int kb = blockIdx.x;
  const int kvh = blockIdx.y / NSPLIT, split = blockIdx.y % NSPLIT;
  const int b = blockIdx.z;
  const int G = p.H / p.KV;
  const int kv0 = kb * 128;
  const int dv0 = split * DV;
  const int lb0 = dv0 / 64;  // first 64-channel block of the output slice
  const int q_lo = p.causal ? kv0 : 0;
  int q_hi = p.S;
  if (p.q_hi_blk) q_hi = min(p.S, p.q_hi_blk[b * nkb + kb]);
  else if (p.window >= 0) q_hi = min(p.S, kv0 + 128 + p.window);
  const int ib = q_lo / BQ2, ie = (q_hi + BQ2 - 1) / BQ2;
  const int ntile = max(0, ie - ib);
  const int ntot = ntile * G;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    prefetch_tmap(&tmap_do);
    mbar_init(kv_full, 1);
    mbar_init(acc_done, 1);
    mbar_init(&acc_issued[0], 1);
    mbar_init(&acc_issued[1], 1);
    mbar_init(qe_full, 1);
    mbar_init(qe_empty, 2);   // S^T_n (issuer A) and dP^T_n (issuer B) have read the early region
    for (int i = 0; i < 2; ++i) {
      mbar_init(&ql_full[i], 1);
      mbar_init(&ql_empty[i], 1);
      mbar_init(&sdp_full[i], 2);  // one commit from each issuing thread
      mbar_init(&pt_full[i], EW_THREADS);
      mbar_init(&acc_free[i], 1);
      mbar_init(&stat_bar[i], EW_THREADS);
    }
    mbar_fence_init();
  }
  if (warp == WARP_MMA) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_dk = tmem_base;          // DV <= 128 columns
  const uint32_t tmem_dv = tmem_base + 128;
  const uint32_t tmem_st = tmem_base + 256;    // 2 x 64: S^T, then P^T (packed) at the start of each half
  const uint32_t tmem_dpt = tmem_base + 384;   // 2 x 64: dP^T, then dS^T likewise

  if (warp == WARP_TMA) {
    if (lane == 0 && ntot > 0) {
      mbar_expect_tx(kv_full, 2 * L::KV_BYTES);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        tma_load_4d(smem + L::OFF_K + c * (128 * 128), &tmap_k, kv_full, c * 64, kvh, kv0, b);
        tma_load_4d(smem + L::OFF_V + c * (128 * 128), &tmap_v, kv_full, c * 64, kvh, kv0, b);
      }
      bool okp = true;
      for (int n = 0; n < ntot && okp; ++n) {
        const int g = n / ntile, i = ib + n % ntile;
        const int h = kvh * G + g;
        const int s = n & 1;
        if (!mbar_wait(&ql_empty[s], ((n >> 1) & 1) ^ 1)) { okp = false; break; }
        mbar_expect_tx(&ql_full[s], 2 * L::LATE_BYTES);
#pragma unroll
        for (int c = 0; c < LATE_BLKS; ++c) {
          tma_load_4d(smem + L::OFF_QL + (s * 2 + 0) * L::LATE_BYTES + c * (BQ2 * 128), &tmap_q, &ql_full[s],
                      (lb0 + c) * 64, h, i * BQ2, b);
          tma_load_4d(smem + L::OFF_QL + (s * 2 + 1) * L::LATE_BYTES + c * (BQ2 * 128), &tmap_do, &ql_full[s],
                      (lb0 + c) * 64, h, i * BQ2, b);
        }
        if (HAS_EARLY) {
          if (!mbar_wait(qe_empty, (n & 1) ^ 1)) { okp = false; break; }
          mbar_expect_tx(qe_full, 2 * L::EARLY_BYTES);
#pragma unroll
          for (int c = 0; c < HD / 64; ++c) {
            if (c >= lb0 && c < lb0 + LATE_BLKS) continue;
            const int e = c < lb0 ? c : c - LATE_BLKS;
            tma_load_4d(smem + L::OFF_QE + 0 * L::EARLY_BYTES + e * (BQ2 * 128), &tmap_q, qe_full, c * 64, h, i * BQ2, b);
            tma_load_4d(smem + L::OFF_QE + 1 * L::EARLY_BYTES + e * (BQ2 * 128), &tmap_do, qe_full, c * 64, h, i * BQ2, b);
          }
        }
      }
      if (!okp) atomicCAS(p.status, 0, ERR_WAIT_EMPTY);
    }
  } else if (warp >= WARP_MMA) {
    // issuer A (warp 9): S^T_n = K Q_n^T for every tile.  Issuer B (warp 10): dP^T_n = V dO_n^T (one tile ahead) and
    // dV += P^T_n dO_n, dK += dS^T_n Q_n.
    const bool is_a = warp == WARP_MMA;
    if (lane == 0 && ntot > 0) {
      constexpr uint32_t idesc_st = make_idesc_bf16(128, BQ2, false, false);
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, DV, false, true);
      static_assert(NSPLIT <= 2, "block-to-region mapping below assumes at most two channel splits");
      const uint64_t da0 = make_smem_desc(smem_u32(smem + (is_a ? L::OFF_K : L::OFF_V)), 16, 1024);
      const int which = is_a ? 0 : 1;  // query-side operand: Q for S^T, dO for dP^T
      bool ok = mbar_wait(kv_full, 0);
      // S^T_n (A) or dP^T_n (B): 128 kv rows x BQ2 query columns, contraction over all channels.  The query-side
      // tile sits in two regions: with two channel splits the first LATE_BLKS 64-channel blocks are the slice
      // ("late") region for split 0 and the other ("early") region for split 1, and vice versa.
      auto issue_scores = [&](int n) -> bool {
        const int s = n & 1, buf = n & 1;
        const uint32_t ph = (n >> 1) & 1;
        if (!mbar_wait(&ql_full[s], ph)) return false;
        if (HAS_EARLY && !mbar_wait(qe_full, n & 1)) return false;
        // the buffer was last read by dV_(n-2) / dK_(n-2): issued by B itself, or (for A) announced by B
        if (is_a && n >= 2 && !mbar_wait(&acc_issued[buf], ((n - 2) >> 1) & 1)) return false;
        tc_fence_after();
        const uint64_t late = make_smem_desc(smem_u32(smem + L::OFF_QL + (s * 2 + which) * L::LATE_BYTES), 16, 1024);
        const uint64_t early = HAS_EARLY ? make_smem_desc(smem_u32(smem + L::OFF_QE + which * L::EARLY_BYTES), 16, 1024) : late;
        const uint64_t lo_half = (!HAS_EARLY || split == 0) ? late : early;
        const uint64_t hi_half = (!HAS_EARLY || split == 0) ? early : late;
        const uint32_t d_t = (is_a ? tmem_st : tmem_dpt) + buf * BQ2;
        umma_bf16_ss_c<false>(d_t, da0, lo_half, idesc_st);
#pragma unroll
        for (int k = 1; k < HD / 16; ++k) {
          const int blk = k >> 2, kk = k & 3;
          const bool in_lo = !HAS_EARLY || blk < LATE_BLKS;
          const uint64_t db = smem_desc_advance(in_lo ? lo_half : hi_half,
                                                (in_lo ? blk : blk - LATE_BLKS) * (BQ2 * 128) + kk * 32);
          umma_bf16_ss_c<true>(d_t, smem_desc_advance(da0, blk * (128 * 128) + kk * 32), db, idesc_st);
        }
        if (HAS_EARLY) umma_commit(qe_empty);   // two arrivals per tile: S^T and dP^T have read the early region
        umma_commit(&sdp_full[buf]);            // two arrivals per tile
        return true;
      };
      if (is_a) {
        for (int n = 0; n < ntot && ok; ++n) ok = issue_scores(n);
      } else {
        if (ok) ok = issue_scores(0);
        for (int n = 0; n < ntot && ok; ++n) {
          if (n + 1 < ntot) ok = issue_scores(n + 1);
          if (!ok) break;
          const int s = n & 1, buf = n & 1;
          if (!mbar_wait(&pt_full[buf], (n >> 1) & 1)) {
            ok = false;
            break;
          }
          tc_fence_after();
          // B operands: the [BQ2 x DV] slices of dO / Q (slice channels), MN-major
          const uint64_t dql = make_smem_desc(smem_u32(smem + L::OFF_QL + (s * 2 + 0) * L::LATE_BYTES), BQ2 * 128, 1024);
          const uint64_t ddol = make_smem_desc(smem_u32(smem + L::OFF_QL + (s * 2 + 1) * L::LATE_BYTES), BQ2 * 128, 1024);
          umma_bf16_ts(tmem_dv, tmem_st + buf * BQ2, ddol, idesc_acc, n != 0);
#pragma unroll
          for (int k = 1; k < BQ2 / 16; ++k)
            umma_bf16_ts_c<true>(tmem_dv, tmem_st + buf * BQ2 + (k >> 1) * 32 + (k & 1) * 8,
                                 smem_desc_advance(ddol, k * 2048), idesc_acc);
          umma_bf16_ts(tmem_dk, tmem_dpt + buf * BQ2, dql, idesc_acc, n != 0);
#pragma unroll
          for (int k = 1; k < BQ2 / 16; ++k)
            umma_bf16_ts_c<true>(tmem_dk, tmem_dpt + buf * BQ2 + (k >> 1) * 32 + (k & 1) * 8,
                                 smem_desc_advance(dql, k * 2048), idesc_acc);
          tc_fence_before();
          mbar_arrive(&acc_issued[buf]);  // A may now overwrite the S^T buffer of this parity (it enters the pipe later)
          umma_commit(&ql_empty[s]);
          if (n == ntot - 1) umma_commit(acc_done);
        }
      }
      if (!ok) atomicCAS(p.status, 0, ERR_WAIT_MISC);
    }
  } else {
    // two threads per kv row: each takes 32 of the 64 query columns of a tile
    const int half = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const int kv = kv0 + row;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    // masks: the query rows that may attend to this kv row form the interval [qlo_kv, qhi_kv)
    const int* docb = (p.doc && !p.q_end) ? p.doc + static_cast<long long>(b) * p.S : nullptr;
    const int dk_doc = (docb && kv < p.S) ? docb[kv] : 0;
    int qlo_kv, qhi_kv;
    if (kv >= p.S) {
      qlo_kv = INT_MAX;
      qhi_kv = 0;
    } else {
      qlo_kv = p.causal ? kv : 0;
      if (p.q_end) qhi_kv = min(p.S, p.q_end[static_cast<long long>(b) * p.S + kv]);
      else qhi_kv = p.window >= 0 ? min(p.S, kv + p.window + 1) : p.S;
    }
    int w_qlo_max = qlo_kv, w_qhi_min = qhi_kv;
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) {
      w_qlo_max = max(w_qlo_max, __shfl_xor_sync(0xffffffffu, w_qlo_max, sh));
      w_qhi_min = min(w_qhi_min, __shfl_xor_sync(0xffffffffu, w_qhi_min, sh));
    }
    bool ok = true;
    for (int n = 0; n < ntot && ok; ++n) {
      const int g = n / ntile, i = ib + n % ntile;
      const int h = kvh * G + g;
      const int buf = n & 1;
      const int q0 = i * BQ2;
      // stage lse (log2 domain; +inf past the end, which makes P = 0) and delta of this query tile
      if (threadIdx.x < 2 * BQ2) {
        const int t = threadIdx.x;
        const int qq = q0 + (t & 63);
        const long long idx = (static_cast<long long>(b) * p.H + h) * p.S + qq;
        float val;
        if (t < 64) val = (qq < p.S) ? p.lse[idx] * LOG2E : INFINITY;
        else val = (qq < p.S) ? p.delta[idx] : 0.f;
        stat[buf * 2 * BQ2 + (t >> 6) * BQ2 + (t & 63)] = val;
      }
      mbar_arrive(&stat_bar[buf]);
      if (!mbar_wait(&stat_bar[buf], (n >> 1) & 1) || !mbar_wait(&sdp_full[buf], (n >> 1) & 1)) {
        atomicCAS(p.status, 0, ERR_WAIT_SOFTMAX);
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t rs[32], rp[32];
      tmem_ld_32x32(tmem_st + buf * BQ2 + half * 32 + lane_sel, rs);
      tmem_ld_32x32(tmem_dpt + buf * BQ2 + half * 32 + lane_sel, rp);
      tmem_ld_wait();
      const float4* lse4 = reinterpret_cast<const float4*>(stat + buf * 2 * BQ2 + half * 32);
      const float4* del4 = reinterpret_cast<const float4*>(stat + buf * 2 * BQ2 + BQ2 + half * 32);
      const bool need_mask = (docb != nullptr) || q0 < w_qlo_max || q0 + BQ2 > w_qhi_min;
      float pv[32], ds[32];
#pragma unroll
      for (int j4 = 0; j4 < 8; ++j4) {
        const float4 ls = lse4[j4], dl = del4[j4];
        const float lsv[4] = {ls.x, ls.y, ls.z, ls.w}, dlv[4] = {dl.x, dl.y, dl.z, dl.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j4 * 4 + e;
          const float pr = ex2(fmaf(__uint_as_float(rs[j]), p.scale_log2, -lsv[e]));
          pv[j] = pr;
          ds[j] = pr * (__uint_as_float(rp[j]) - dlv[e]) * p.scale;
        }
      }
      if (need_mask) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int qq = q0 + half * 32 + j;
          bool bad = (qq < qlo_kv) | (qq >= qhi_kv);
          if (docb && qq < p.S) bad |= docb[qq] != dk_doc;
          if (bad) {
            pv[j] = 0.f;
            ds[j] = 0.f;
          }
        }
      }
      uint32_t pk[16], dk16[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        pk[j] = pack_bf16(pv[2 * j], pv[2 * j + 1]);
        dk16[j] = pack_bf16(ds[2 * j], ds[2 * j + 1]);
      }
      // each thread overwrites only columns it has read itself (the first 16 of its 32)
      tmem_st_32x16(tmem_st + buf * BQ2 + half * 32 + lane_sel, pk);
      tmem_st_32x16(tmem_dpt + buf * BQ2 + half * 32 + lane_sel, dk16);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&pt_full[buf]);
    }
    if (ok && ntot > 0 && !mbar_wait(acc_done, 0)) {
      atomicCAS(p.status, 0, ERR_WAIT_ACC_FULL);
      ok = false;
    }
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* base = p.dqkv + (static_cast<long long>(b) * p.S + kv) * p.g_stride;
      __nv_bfloat16* dkrow = base + static_cast<long long>(p.H + kvh) * HD + dv0 + half * (DV / 2);
      __nv_bfloat16* dvrow = base + static_cast<long long>(p.H + p.KV + kvh) * HD + dv0 + half * (DV / 2);
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t src = which == 0 ? tmem_dk : tmem_dv;
        __nv_bfloat16* dst = which == 0 ? dkrow : dvrow;
#pragma unroll 1
        for (int c = 0; c < DV / 64; ++c) {
          uint32_t r[32];
          if (ntot > 0) {
            tmem_ld_32x32(src + half * (DV / 2) + c * 32 + lane_sel, r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0;
          }
          if (kv < p.S) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(r[j * 8 + 0]), __uint_as_float(r[j * 8 + 1]));
              o.y = pack_bf16(__uint_as_float(r[j * 8 + 2]), __uint_as_float(r[j * 8 + 3]));
              o.z = pack_bf16(__uint_as_float(r[j * 8 + 4]), __uint_as_float(r[j * 8 + 5]));
              o.w = pack_bf16(__uint_as_float(r[j * 8 + 6]), __uint_as_float(r[j * 8 + 7]));
              reinterpret_cast<uint4*>(dst + c * 32)[j] = o;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

int make_maps(CUtensorMap* tq, CUtensorMap* tk, CUtensorMap* tv, CUtensorMap* tdo, const void* q, const void* k,
              const void* v, const void* dout, int B, int S, int H, int KV, int HD, long long qs, long long ks,
              long long vs, uint32_t q_rows, uint32_t kv_rows) {
  const uint64_t dq[4] = {(uint64_t)HD, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  const uint64_t sq[3] = {(uint64_t)HD, (uint64_t)qs, (uint64_t)qs * S};
  const uint64_t sdo[3] = {(uint64_t)HD, (uint64_t)H * HD, (uint64_t)H * HD * S};
  const uint32_t bq[4] = {64, 1, q_rows, 1};
  const uint64_t dk[4] = {(uint64_t)HD, (uint64_t)KV, (uint64_t)S, (uint64_t)B};
  const uint64_t sk[3] = {(uint64_t)HD, (uint64_t)ks, (uint64_t)ks * S};
  const uint64_t sv[3] = {(uint64_t)HD, (uint64_t)vs, (uint64_t)vs * S};
  const uint32_t bk[4] = {64, 1, kv_rows, 1};
  if (mbh::make_tmap_bf16_nd(tq, q, 4, dq, sq, bq)) return -2;
  if (mbh::make_tmap_bf16_nd(tdo, dout, 4, dq, sdo, bq)) return -2;
  if (mbh::make_tmap_bf16_nd(tk, k, 4, dk, sk, bk)) return -2;
  if (mbh::make_tmap_bf16_nd(tv, v, 4, dk, sv, bk)) return -2;
  return 0;
}

template <int HD, int NST, int DV, int NSTQ>
int launch_bwd(const void* q, const void* k, const void* v, const void* dout, const BwdParams& p, long long qs,
               long long ks, long long vs, cudaStream_t st) {
  CUtensorMap tq, tk, tv, tdo;
  // ---- dQ
  if (make_maps(&tq, &tk, &tv, &tdo, q, k, v, dout, p.B, p.S, p.H, p.KV, HD, qs, ks, vs, 128, BKV)) return -2;
  using LQ = SmemDQ<HD, NST>;
  MB_SET_MAX_SMEM_ONCE((attn_bwd_dq_kernel<HD, NST>), LQ::TOTAL);
  dim3 g1((p.S + 127) / 128, p.H, p.B);
  attn_bwd_dq_kernel<HD, NST><<<g1, BWD_THREADS, LQ::TOTAL, st>>>(tq, tk, tv, tdo, p);
  int e = mbh::check_launch("attn_bwd_dq");
  if (e) return e;
  // ---- dK/dV
  if (make_maps(&tq, &tk, &tv, &tdo, q, k, v, dout, p.B, p.S, p.H, p.KV, HD, qs, ks, vs, BQ2, 128)) return -2;
  using LK = SmemKV<HD, DV>;
  MB_SET_MAX_SMEM_ONCE((attn_bwd_dkdv_kernel<HD, DV, NSTQ>), LK::TOTAL);
  dim3 g2((p.S + 127) / 128, p.KV * (HD / DV), p.B);
  attn_bwd_dkdv_kernel<HD, DV, NSTQ><<<g2, BWD_THREADS, LK::TOTAL, st>>>(tq, tk, tv, tdo, p);
  return mbh::check_launch("attn_bwd_dkdv");
}

}  // namespace

// q,k (after norm/rope) and v as in mb_attn_fwd; out/dout: [B,S,H,hd] contiguous; lse: [B,H,S];
// delta_ws: fp32 [B,H,S] scratch; dqkv: packed gradient buffer with row pitch g_stride.
extern "C" int mb_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                           const float* lse, float* delta_ws, void* dqkv, const int* doc, const int* kv_lo_blk,
                           const int* q_hi_blk, const int* kv_start, const int* q_end, int B, int S, int H, int KV,
                           int hd, long long q_tok_stride,
                           long long k_tok_stride, long long v_tok_stride, long long g_stride, int causal,
                           int window, float scale, cudaStream_t st) {
  BwdParams p;
  p.lse = lse;
  p.delta = delta_ws;
  p.dqkv = reinterpret_cast<__nv_bfloat16*>(dqkv);
  p.g_stride = g_stride;
  p.doc = doc;
  p.kv_lo_blk = kv_lo_blk;
  p.q_hi_blk = q_hi_blk;
  p.kv_start = kv_start;
  p.q_end = q_end;
  p.B = B;
  p.S = S;
  p.H = H;
  p.KV = KV;
  p.causal = causal;
  p.window = window;
  p.scale = scale;
  p.scale_log2 = scale * LOG2E;
  p.status = mbh::status().dev;
  if (!p.status) return -4;
  if ((kv_start != nullptr) != (q_end != nullptr) || (kv_start && !causal)) return -3;
  if ((q_tok_stride & 7) || (k_tok_stride & 7) || (v_tok_stride & 7) || (g_stride & 7)) return -3;
  const long long items = static_cast<long long>(B) * S * H;
  attn_delta_kernel<<<static_cast<unsigned>((items + 7) / 8), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout), delta_ws, B, S, H, hd);
  int e = mbh::check_launch("attn_delta");
  if (e) return e;
  if (hd == 256) return launch_bwd<256, 1, 128, 1>(q, k, v, dout, p, q_tok_stride, k_tok_stride, v_tok_stride, st);
  if (hd == 128) return launch_bwd<128, 2, 128, 2>(q, k, v, dout, p, q_tok_stride, k_tok_stride, v_tok_stride, st);
  if (hd == 64) return launch_bwd<64, 2, 64, 2>(q, k, v, dout, p, q_tok_stride, k_tok_stride, v_tok_stride, st);
  return -3;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant (declared in maester_b200_noalloc.h; no counterpart in the reference).
// The delta work buffer lives in the library's device image instead of caller-allocated memory.
#include "maester_b200_noalloc.h"

namespace {

static __device__ __align__(256) float g_noalloc_delta[MB_NOALLOC_MAX_ROWS];
static __device__ int g_noalloc_status;

constexpr int NOALLOC_MAX_DEVICES = 64;
struct NoallocDevice {
  std::atomic<bool> ready{false};
  float* delta = nullptr;  // device address of g_noalloc_delta on that GPU
  int* status = nullptr;   // device address of g_noalloc_status
};
NoallocDevice g_noalloc_dev[NOALLOC_MAX_DEVICES];

// Once per device, with that device current.  In host code the array's name is only a handle for
// the runtime; the address a kernel can use has to be asked for.
int noalloc_setup(int dev) {
  NoallocDevice& d = g_noalloc_dev[dev];
  if (d.ready.load(std::memory_order_acquire)) return 0;
  void* p = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_delta);
  if (e != cudaSuccess || !p) {
    fprintf(stderr, "maester_b200: cudaGetSymbolAddress(work array) failed on device %d: %s\n", dev,
            cudaGetErrorString(e));
    return MB_NOALLOC_SETUP_FAILED;
  }
  d.delta = static_cast<float*>(p);
  e = cudaGetSymbolAddress(&p, g_noalloc_status);
  if (e != cudaSuccess || !p) {
    fprintf(stderr, "maester_b200: cudaGetSymbolAddress(status word) failed on device %d: %s\n", dev,
            cudaGetErrorString(e));
    return MB_NOALLOC_SETUP_FAILED;
  }
  d.status = static_cast<int*>(p);
  d.ready.store(true, std::memory_order_release);
  return 0;
}

}  // namespace

extern "C" int mb_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                   const float* lse, void* dqkv, const int* doc, const int* kv_lo_blk,
                                   const int* q_hi_blk, int B, int S, int H, int KV, int hd, long long q_tok_stride,
                                   long long k_tok_stride, long long v_tok_stride, long long g_stride, int causal,
                                   int window, float scale, int* status_out, cudaStream_t st) {
  if (B <= 0 || S <= 0 || H <= 0 || KV <= 0) return -3;
  const long long rows = static_cast<long long>(B) * S * H;
  if (rows > MB_NOALLOC_MAX_ROWS) {
    fprintf(stderr,
            "maester_b200: mb_attn_bwd_noalloc needs B*H*S = %lld work entries but the built-in array holds %d; "
            "use mb_attn_bwd with a caller-provided buffer\n",
            rows, MB_NOALLOC_MAX_ROWS);
    return MB_NOALLOC_TOO_LARGE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return MB_NOALLOC_SETUP_FAILED;
  if (int e = noalloc_setup(dev)) return e;
  const NoallocDevice& d = g_noalloc_dev[dev];

  BwdParams p;
  p.lse = lse;
  p.delta = d.delta;
  p.dqkv = reinterpret_cast<__nv_bfloat16*>(dqkv);
  p.g_stride = g_stride;
  p.doc = doc;
  p.kv_lo_blk = kv_lo_blk;
  p.q_hi_blk = q_hi_blk;
  p.kv_start = nullptr;
  p.q_end = nullptr;
  p.B = B;
  p.S = S;
  p.H = H;
  p.KV = KV;
  p.causal = causal;
  p.window = window;
  p.scale = scale;
  p.scale_log2 = scale * LOG2E;
  p.status = status_out ? status_out : d.status;
  if ((q_tok_stride & 7) || (k_tok_stride & 7) || (v_tok_stride & 7) || (g_stride & 7)) return -3;
  // the kernels read delta[0 .. B*H*S): this launch rewrites exactly that range first
  attn_delta_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(dout), d.delta, B, S, H, hd);
  if (int e = mbh::check_launch("attn_delta(noalloc)")) return e;
  if (hd == 256) return launch_bwd<256, 1, 128, 1>(q, k, v, dout, p, q_tok_stride, k_tok_stride, v_tok_stride, st);
  if (hd == 128) return launch_bwd<128, 2, 128, 2>(q, k, v, dout, p, q_tok_stride, k_tok_stride, v_tok_stride, st);
  if (hd == 64) return launch_bwd<64, 2, 64, 2>(q, k, v, dout, p, q_tok_stride, k_tok_stride, v_tok_stride, st);
  return -3;
}

extern "C" int mb_noalloc_status(void) {
  int code = 0;
  if (cudaMemcpyFromSymbol(&code, g_noalloc_status, sizeof(int)) != cudaSuccess) return MB_NOALLOC_SETUP_FAILED;
  if (code != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_noalloc_status, &zero, sizeof(int)) != cudaSuccess) return MB_NOALLOC_SETUP_FAILED;
  }
  return code;
}
