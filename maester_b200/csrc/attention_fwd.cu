// Flash-style attention forward on tcgen05: causal / sliding-window / same-document masks, GQA.
//
// One CTA handles 128 query rows of one (batch, q-head).  Warp 8 streams Q once and K/V blocks
// through a 2-stage TMA ring; warp 9 issues S = Q K^T into one of two TMEM score buffers and
// O += P V into a TMEM output accumulator.  Warps 0-7 run the online softmax with TWO threads per
// query row (warps w and w+4 share the TMEM lanes of rows 32*(w&3).. and each takes half of the
// score columns): one TMEM read per block kept in registers (the score buffer is released right
// after it), the row maximum exchanged through shared memory (rounded up to bf16 on both sides, so
// both threads use the same reference; any upper bound of the true maximum is a valid reference),
// P (bf16) written into swizzled shared memory for the second MMA, O rescaled in TMEM only when the
// running maximum grew by more than 2^8.  Two warps per scheduler hide each other's latencies.
//
// The mask is   kv <= q  (causal)  AND  q - kv <= window  (inclusive window, if window >= 0)
//           AND doc[q] == doc[kv] (if document ids are given);
// kv blocks outside [kv_lo_blk, causal limit) are skipped, where kv_lo_blk[b, qblock] is a
// conservative per-query-block lower bound computed by the caller.
//
// Every wait is bounded; on expiry the kernel records a status code, frees TMEM and returns.
#include "host_common.cuh"
#include "sm100.cuh"
#include <math.h>

namespace {
using namespace mb;

constexpr int BQ = 128;
constexpr int ATT_THREADS = 320;
constexpr int SOFTMAX_THREADS = 256;
constexpr int WARP_TMA = 8, WARP_MMA = 9;

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
constexpr int KV_STAGES = 2;

struct AttnParams {
  __nv_bfloat16* O;      // [B, S, H, HD] contiguous
  float* lse;            // [B, H, S]
  const int* doc;        // [B, S] or null
  const int* kv_lo_blk;  // [B, ceil(S/BQ)] or null
  int B, S, H, KV;
  int causal, window;    // window < 0: none
  float scale_log2;      // softmax scale * log2(e)
  int* status;
};

template <int HD, int BKV>
struct Smem {
  static constexpr int Q_BYTES = BQ * HD * 2;
  static constexpr int KV_BYTES = BKV * HD * 2;
  static constexpr int P_BYTES = BQ * BKV * 2;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + KV_STAGES * KV_BYTES;
  static constexpr int OFF_P = OFF_V + KV_STAGES * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + 2 * P_BYTES;
  static constexpr int OFF_XCH = OFF_BAR + 256;   // 1 KiB: row-maximum / row-sum exchange between the column halves
  static constexpr int TOTAL = OFF_XCH + 1024 + 1024;
};

template <int HD, int BKV>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  using L = Smem<HD, BKV>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // [2]
  uint64_t* v_full = bars + 3;        // [2]
  uint64_t* v_empty = bars + 5;       // [2]  V stage free: the P V product that read it has completed
  uint64_t* k_empty = bars + 18;      // [2]  K stage free: the Q K^T product that read it has completed (earlier)
  uint64_t* s_full = bars + 7;        // [2]
  uint64_t* s_empty = bars + 9;       // [2]
  uint64_t* p_full = bars + 11;       // [2]
  uint64_t* p_empty = bars + 13;      // [2]
  uint64_t* o_done = bars + 15;       // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.S + BQ - 1) / BQ;
  const int qb = nqb - 1 - blockIdx.x;  // heaviest (latest) query blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.H / p.KV);
  const int q0 = qb * BQ;

  // kv block range for this query block
  int kv_end = p.causal ? min(p.S, q0 + BQ) : p.S;
  int kv_begin = 0;
  if (p.kv_lo_blk) kv_begin = p.kv_lo_blk[b * nqb + qb];
  else if (p.window >= 0) kv_begin = max(0, q0 - p.window);
  const int jb = kv_begin / BKV;
  const int je = (kv_end + BKV - 1) / BKV;
  const int nblk = je - jb;

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], SOFTMAX_THREADS);
      mbar_init(&p_full[i], SOFTMAX_THREADS);
      mbar_init(&p_empty[i], 1);
    }
    mbar_init(o_done, 1);
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
  const uint32_t tmem_o = tmem_base;             // HD columns
  const uint32_t tmem_s = tmem_base + 256;       // 2 x BKV columns (BKV <= 128)

  if (warp == WARP_TMA) {
    // ---------------------------------------------------------------- producer
    if (lane == 0 && nblk > 0) {
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c)
        tma_load_4d(smem + L::OFF_Q + c * (BQ * 128), &tmap_q, q_full, c * 64, h, q0, b);
      // K and V stages are released separately (K as soon as its scores exist, V only after the P V
      // product), and K runs one block ahead of V, so that the load of K for block n+2 starts while
      // block n is still in its softmax: the TMA latency stays off the critical path.
      auto load_k = [&](int n) -> bool {
        const int s = n & 1;
        if (!mbar_wait(&k_empty[s], ((n >> 1) & 1) ^ 1)) return false;
        mbar_expect_tx(&k_full[s], L::KV_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_4d(smem + L::OFF_K + s * L::KV_BYTES + c * (BKV * 128), &tmap_k, &k_full[s], c * 64, kvh, (jb + n) * BKV, b);
        return true;
      };
      auto load_v = [&](int n) -> bool {
        const int s = n & 1;
        if (!mbar_wait(&v_empty[s], ((n >> 1) & 1) ^ 1)) return false;
        mbar_expect_tx(&v_full[s], L::KV_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_4d(smem + L::OFF_V + s * L::KV_BYTES + c * (BKV * 128), &tmap_v, &v_full[s], c * 64, kvh, (jb + n) * BKV, b);
        return true;
      };
      bool okp = true;
      for (int n = 0; n < nblk && okp; ++n) {
        okp = load_k(n);
        if (okp && n >= 1) okp = load_v(n - 1);
      }
      if (okp) okp = load_v(nblk - 1);
      if (!okp) atomicCAS(p.status, 0, ERR_WAIT_EMPTY);
    }
  } else if (warp == WARP_MMA) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(BQ, BKV, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BQ, HD, false, true);
      const uint32_t sq = smem_u32(smem + L::OFF_Q);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) atomicCAS(p.status, 0, ERR_WAIT_FULL);
      auto issue_qk = [&](int n) -> bool {
        const int s = n & 1;
        if (!mbar_wait(&k_full[s], (n >> 1) & 1)) return false;
        if (!mbar_wait(&s_empty[s], ((n >> 1) & 1) ^ 1)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + L::OFF_K + s * L::KV_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t blk = k >> 2, kk = k & 3;  // 64-wide block along head dim, 16-wide step inside
          const uint64_t da = make_smem_desc(sq + blk * (BQ * 128) + kk * 32, 16, 1024);
          const uint64_t db = make_smem_desc(sk + blk * (BKV * 128) + kk * 32, 16, 1024);
          umma_bf16_ss(tmem_s + s * BKV, da, db, idesc_qk, k != 0);
        }
        umma_commit(&s_full[s]);
        umma_commit(&k_empty[s]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int n = 0; n < nblk && ok; ++n) {
        if (n + 1 < nblk) ok = issue_qk(n + 1);
        if (!ok) break;
        const int s = n & 1;
        if (!mbar_wait(&v_full[s], (n >> 1) & 1) || !mbar_wait(&p_full[s], (n >> 1) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sp = smem_u32(smem + L::OFF_P + s * L::P_BYTES);
        const uint32_t sv = smem_u32(smem + L::OFF_V + s * L::KV_BYTES);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint32_t blk = k >> 2, kk = k & 3;
          const uint64_t da = make_smem_desc(sp + blk * (BQ * 128) + kk * 32, 16, 1024);
          // V tile: HD/64 blocks of [BKV rows x 64 channels]; MN-major operand, 16 kv rows per step
          const uint64_t db = make_smem_desc(sv + k * 2048, BKV * 128, 1024);
          umma_bf16_ss(tmem_o, da, db, idesc_pv, (n | k) != 0);
        }
        umma_commit(&v_empty[s]);
        umma_commit(&p_empty[s]);
        umma_commit(o_done);
      }
      if (!ok) atomicCAS(p.status, 0, ERR_WAIT_MISC);
    }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue (warps 0..7)
    constexpr int NC = BKV / 2;  // score columns per thread
    constexpr int OC = HD / 2;   // output columns per thread
    const int half = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const int q = q0 + row;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int col_base = half * NC;
    __nv_bfloat16* xch = reinterpret_cast<__nv_bfloat16*>(smem + L::OFF_XCH);  // [parity][half][128 rows]
    const int* docb = p.doc ? p.doc + static_cast<long long>(b) * p.S : nullptr;
    const int dq = (docb && q < p.S) ? docb[q] : 0;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;  // after a failed wait the thread keeps going (every barrier below is CTA-uniform)
    for (int n = 0; n < nblk; ++n) {
      const int s = n & 1;
      const int kv0 = (jb + n) * BKV;
      if (ok && !mbar_wait(&s_full[s], (n >> 1) & 1)) {
        atomicCAS(p.status, 0, ERR_WAIT_SOFTMAX);
        ok = false;
      }
      tc_fence_after();
      uint32_t r[NC];
#pragma unroll
      for (int c = 0; c < NC / 32; ++c)
        tmem_ld_32x32(tmem_s + s * BKV + col_base + c * 32 + lane_sel, reinterpret_cast<uint32_t(&)[32]>(r[c * 32]));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&s_empty[s]);  // the scores now live in registers
      const bool need_mask = (docb != nullptr) || (kv0 + BKV > p.S) || (p.causal && kv0 + BKV - 1 > q0) ||
                             (p.window >= 0 && (q0 + BQ - 1) - kv0 > p.window);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < NC; ++i) {
          const int kv = kv0 + col_base + i;
          bool bad = kv >= p.S;
          if (p.causal) bad |= kv > q;
          if (p.window >= 0) bad |= (q - kv) > p.window;
          if (docb && kv < p.S) bad |= docb[kv] != dq;
          if (bad) r[i] = 0xFF800000u;  // -inf: exp2 gives exactly 0
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < NC; i += 4) {
        mx4[0] = fmaxf(mx4[0], __uint_as_float(r[i]));
        mx4[1] = fmaxf(mx4[1], __uint_as_float(r[i + 1]));
        mx4[2] = fmaxf(mx4[2], __uint_as_float(r[i + 2]));
        mx4[3] = fmaxf(mx4[3], __uint_as_float(r[i + 3]));
      }
      // both halves round their maximum up to bf16 before use, so the two threads of a row agree
      const __nv_bfloat16 mine = __float2bfloat16_ru(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])));
      xch[(n & 1) * 256 + half * 128 + row] = mine;
      asm volatile("bar.sync 1, 256;" ::: "memory");
      const float mx = fmaxf(__bfloat162float(mine), __bfloat162float(xch[(n & 1) * 256 + (half ^ 1) * 128 + row]));
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      // lazy rescale of the accumulator: only when the maximum moved by more than 2^8
      const bool grow = m_new > m_used + 8.f;
      if (__any_sync(0xffffffffu, grow)) {
        if (n > 0) {
          if (ok && !mbar_wait(o_done, (n - 1) & 1)) {
            atomicCAS(p.status, 0, ERR_WAIT_SOFTMAX);
            ok = false;
          }
          tc_fence_after();
          const float alpha = (m_used == -INFINITY) ? 0.f : ex2(m_used - m_new);
#pragma unroll 1
          for (int c = 0; c < OC / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(tmem_o + half * OC + c * 32 + lane_sel, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(tmem_o + half * OC + c * 32 + lane_sel, o);
          }
          tmem_st_wait();
          l *= alpha;
        }
        m_used = m_new;
      }
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
      // wait until the MMA that read the previous contents of this P buffer has finished
      if (ok && !mbar_wait(&p_empty[s], ((n >> 1) & 1) ^ 1)) {
        atomicCAS(p.status, 0, ERR_WAIT_SOFTMAX);
        ok = false;
      }
      uint8_t* pbuf = smem + L::OFF_P + s * L::P_BYTES;
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < NC / 8; ++c) {  // 8 columns = one 16-byte chunk of the swizzled bf16 tile
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e[i] = ex2(fmaf(__uint_as_float(r[c * 8 + i]), p.scale_log2, -m_safe));
          l4[i & 3] += e[i];
        }
        uint4 o;
        o.x = pack_bf16(e[0], e[1]);
        o.y = pack_bf16(e[2], e[3]);
        o.z = pack_bf16(e[4], e[5]);
        o.w = pack_bf16(e[6], e[7]);
        const int col = col_base + c * 8;
        *reinterpret_cast<uint4*>(pbuf + (col / 64) * (BQ * 128) + swz128(row, (col % 64) / 8)) = o;
      }
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      fence_proxy_async_smem();
      mbar_arrive(&p_full[s]);
    }
    // ---- row sums of the two column halves
    asm volatile("bar.sync 1, 256;" ::: "memory");  // nobody still reads the maximum exchange area
    float* xl = reinterpret_cast<float*>(smem + L::OFF_XCH);  // [half][128 rows]
    xl[half * 128 + row] = l;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    l += xl[(half ^ 1) * 128 + row];
    // ---- epilogue: O / l -> global, log-sum-exp
    if (nblk > 0 && ok) {
      if (!mbar_wait(o_done, (nblk - 1) & 1)) {
        atomicCAS(p.status, 0, ERR_WAIT_ACC_FULL);
        ok = false;
      }
    }
    if (ok) {
      tc_fence_after();
      const float inv_l = (nblk > 0 && l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.O + ((static_cast<long long>(b) * p.S + q) * p.H + h) * HD + half * OC;
#pragma unroll 1
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t o32[32];
        if (nblk > 0) {
          tmem_ld_32x32(tmem_o + half * OC + c * 32 + lane_sel, o32);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o32[i] = 0;
        }
        if (q < p.S) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(o32[v * 8 + 0]) * inv_l, __uint_as_float(o32[v * 8 + 1]) * inv_l);
            o.y = pack_bf16(__uint_as_float(o32[v * 8 + 2]) * inv_l, __uint_as_float(o32[v * 8 + 3]) * inv_l);
            o.z = pack_bf16(__uint_as_float(o32[v * 8 + 4]) * inv_l, __uint_as_float(o32[v * 8 + 5]) * inv_l);
            o.w = pack_bf16(__uint_as_float(o32[v * 8 + 6]) * inv_l, __uint_as_float(o32[v * 8 + 7]) * inv_l);
            reinterpret_cast<uint4*>(orow + c * 32)[v] = o;
          }
        }
      }
      if (half == 0 && q < p.S && p.lse)
        p.lse[(static_cast<long long>(b) * p.H + h) * p.S + q] =
            (nblk > 0 && l > 0.f) ? (m_used * 0.6931471805599453f + logf(l)) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HD, int BKV>
int launch_fwd(const void* q, const void* k, const void* v, const AttnParams& p, long long q_tok_stride,
               long long k_tok_stride, long long v_tok_stride, cudaStream_t st) {
  using L = Smem<HD, BKV>;
  CUtensorMap tq, tk, tv;
  const uint64_t dq[4] = {(uint64_t)HD, (uint64_t)p.H, (uint64_t)p.S, (uint64_t)p.B};
  const uint64_t sq[3] = {(uint64_t)HD, (uint64_t)q_tok_stride, (uint64_t)q_tok_stride * p.S};
  const uint32_t bq[4] = {64, 1, BQ, 1};
  if (mbh::make_tmap_bf16_nd(&tq, q, 4, dq, sq, bq)) return -2;
  const uint64_t dk[4] = {(uint64_t)HD, (uint64_t)p.KV, (uint64_t)p.S, (uint64_t)p.B};
  const uint64_t sk[3] = {(uint64_t)HD, (uint64_t)k_tok_stride, (uint64_t)k_tok_stride * p.S};
  const uint64_t sv[3] = {(uint64_t)HD, (uint64_t)v_tok_stride, (uint64_t)v_tok_stride * p.S};
  const uint32_t bk[4] = {64, 1, BKV, 1};
  if (mbh::make_tmap_bf16_nd(&tk, k, 4, dk, sk, bk)) return -2;
  if (mbh::make_tmap_bf16_nd(&tv, v, 4, dk, sv, bk)) return -2;
  MB_SET_MAX_SMEM_ONCE((attn_fwd_kernel<HD, BKV>), L::TOTAL);
  dim3 grid((p.S + BQ - 1) / BQ, p.H, p.B);
  attn_fwd_kernel<HD, BKV><<<grid, ATT_THREADS, L::TOTAL, st>>>(tq, tk, tv, p);
  return mbh::check_launch("attn_fwd");
}

}  // namespace

// q: [B,S,H,hd] with token stride q_tok_stride (elements) and head stride hd; k, v likewise with KV
// heads.  out: [B,S,H,hd] contiguous bf16, lse: [B,H,S] fp32 (natural log).  window < 0 disables
// the sliding window; doc / kv_lo_blk may be null.
extern "C" int mb_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* doc,
                           const int* kv_lo_blk, int B, int S, int H, int KV, int hd, long long q_tok_stride,
                           long long k_tok_stride, long long v_tok_stride, int causal, int window, float scale,
                           cudaStream_t st) {
  AttnParams p;
  p.O = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.doc = doc;
  p.kv_lo_blk = kv_lo_blk;
  p.B = B;
  p.S = S;
  p.H = H;
  p.KV = KV;
  p.causal = causal;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = mbh::status().dev;
  if (!p.status) return -4;
  if ((q_tok_stride & 7) || (k_tok_stride & 7) || (v_tok_stride & 7)) return -3;
  if (hd == 256) return launch_fwd<256, 64>(q, k, v, p, q_tok_stride, k_tok_stride, v_tok_stride, st);
  if (hd == 128) return launch_fwd<128, 128>(q, k, v, p, q_tok_stride, k_tok_stride, v_tok_stride, st);
  if (hd == 64) return launch_fwd<64, 128>(q, k, v, p, q_tok_stride, k_tok_stride, v_tok_stride, st);
  return -3;
}
