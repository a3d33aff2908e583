// Flash-style attention forward on tcgen05: causal / sliding-window / same-document masks, GQA.
//
// One CTA handles 128 query rows of one (batch, q-head).  Warp 8 streams Q once and K / V blocks through
// two TMA rings.  Warps 9 and 10 issue the MMAs (even / odd kv blocks): S = Q K^T into one of NSB score
// buffers in tensor memory and O += P V into the output accumulator, with P read straight from tensor
// memory (the A operand of the second product is the score buffer itself, overwritten in place with packed
// bf16 probabilities: nothing is staged through shared memory).  The score products run NSB blocks ahead
// of the P V products, so the softmax of a block never waits for the product that frees its buffer.
//
// What set the pace, as measured with an event trace of one CTA: (1) the issuing thread: one thread issues
// at most one MMA per ~54 cycles while an M128 N64 K16 product takes 32, hence two issuing threads whose
// shared-memory descriptors are built once per tile and stepped with one add per instruction; (2) with only
// two score buffers each parity's chain "scores -> softmax -> P V -> next scores" is serial, hence four.
// For head sizes up to 128 there is room in tensor memory to keep Q there as well (QT: HD/2 columns of packed
// bf16, copied once by the softmax warps; the score product then reads no A operand from shared memory); at
// head size 256 O (256 columns) and four score buffers fill tensor memory and Q stays in shared memory.
//
// Warps 0-7 are two softmax sets of four warps (one thread per query row in each set).  The sets take
// alternate kv blocks, so one set's exponentials overlap the other set's tensor-memory reads and
// handshakes.  Both sets accumulate into the same O, so they must use the same reference maximum per row:
// the set that handles block n computes the block maximum, reads the reference the other set published
// for block n-1, raises it only when the maximum grew by more than 2^8 (then it rescales its row of O
// after the earlier P V products have completed), publishes the reference for block n through shared
// memory and a named barrier between the two warps that share the rows, and only then runs its
// exponentials.  Each set keeps its own partial row sum, expressed in the reference it used last; the
// two are combined at the end.
//
// Masks.  kv <= q (causal), q - kv <= window (inclusive, if window >= 0) and "same document" are folded
// into one interval per query row when the caller passes kv_start[b, q] (lowest admissible kv index:
// documents are contiguous runs, so same-document + causal + window is exactly kv_start <= kv <= q);
// blocks that lie inside the interval of every row of a warp skip the mask code.  Without kv_start the
// window / causal bounds are computed here, and a document-id array (any ids, also without the causal
// bound) is compared element by element.  kv blocks outside [kv_lo_blk, causal limit) are skipped.
//
// Every wait is bounded; on expiry the kernel records a status code, frees TMEM and returns.
#include "host_common.cuh"
#include "sm100.cuh"
#include <limits.h>
#include <math.h>

namespace {
using namespace mb;

constexpr int BQ = 128;
constexpr int ATT_THREADS = 352;  // 8 softmax warps, 1 TMA warp, 2 MMA-issuing warps
constexpr int SET_THREADS = 128;
constexpr int WARP_TMA = 8, WARP_MMA = 9;  // warps 9 and 10 issue the MMAs of the even / odd kv blocks

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void named_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void named_arrive(int id, int n) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

struct AttnParams {
  __nv_bfloat16* O;      // [B, S, H, HD] contiguous
  float* lse;            // [B, H, S]
  const int* doc;        // [B, S] or null (element-wise comparison; used when kv_start is null)
  const int* kv_lo_blk;  // [B, ceil(S/BQ)] or null
  const int* kv_start;   // [B, S] or null: lowest kv index each query row may attend to
  int B, S, H, KV;
  int causal, window;    // window < 0: none
  float scale_log2;      // softmax scale * log2(e)
  int* status;
};

// NK / NV: stages of the K and V rings; NSB: score buffers in tensor memory (even, so that a buffer is
// always handled by the same softmax set).
template <int HD, int BKV, int NK_, int NV_, int NSB_, bool QT_>
struct Cfg {
  static constexpr int NK = NK_, NV = NV_, NSB = NSB_;
  static constexpr bool QT = QT_;  // Q lives in tensor memory (A operand of the score product) instead of shared memory
  static constexpr int Q_BYTES = BQ * HD * 2;
  static constexpr int KV_BYTES = BKV * HD * 2;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + NK * KV_BYTES;
  // in tensor-memory mode Q lands in the V ring and moves on before V is loaded; else it has its own buffer
  static constexpr int OFF_Q = QT ? OFF_V : OFF_V + NV * KV_BYTES;
  static constexpr int OFF_BAR = OFF_V + NV * KV_BYTES + (QT ? 0 : Q_BYTES);
  static constexpr int OFF_XCH = OFF_BAR + 512;  // 1 KiB: [2][128] floats, reference maxima / final row sums
  static constexpr int TOTAL = OFF_XCH + 1024 + 1024;  // 512 bytes of barriers, exchange area, alignment slack
  static_assert(HD + (QT ? HD / 2 : 0) + NSB * BKV <= 512, "tensor memory holds 512 columns");
  static_assert(!QT || NV * KV_BYTES >= Q_BYTES, "the V ring doubles as the landing area of Q");
  static_assert(NSB % 2 == 0 && NSB <= 4 && NK <= 4 && NV <= 4, "barrier table layout");
  static_assert(NK % 2 == 0, "a K stage must always be consumed by the same issuing thread (block parity)");
  static_assert(TOTAL <= 232448, "shared memory per CTA");
};

template <int HD, int BKV, int NK, int NV, int NSB, bool QT>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  using L = Cfg<HD, BKV, NK, NV, NSB, QT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars;              // 1
  uint64_t* k_full = bars + 1;          // [NK]
  uint64_t* k_empty = bars + 5;         // [NK]  the Q K^T product that read the stage has completed
  uint64_t* v_full = bars + 9;          // [NV]
  uint64_t* v_empty = bars + 13;        // [NV]  the P V product that read the stage has completed
  uint64_t* s_full = bars + 17;         // [NSB] scores of a block are in tensor memory
  uint64_t* p_full = bars + 21;         // [NSB] probabilities of a block are in tensor memory (128 arrivals)
  uint64_t* pv_done = bars + 25;        // [NSB] the P V product of the block that used the buffer has completed
  uint64_t* q_ready = bars + 29;        // 1     Q has been copied into tensor memory (256 arrivals)
  uint64_t* pv_turn = bars + 31;        // [2]   the P V product of an even / odd block has been issued
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 30);  // (barrier table: 64 slots of 8 bytes)
  float* xch = reinterpret_cast<float*>(smem + L::OFF_XCH);

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
  const int nblk = max(0, je - jb);

  if (threadIdx.x == 0) {
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    mbar_init(q_full, 1);
    mbar_init(q_ready, 2 * SET_THREADS);
    mbar_init(&pv_turn[0], 1);
    mbar_init(&pv_turn[1], 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], SET_THREADS);
      mbar_init(&pv_done[i], 1);
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
  const uint32_t tmem_o = tmem_base;                 // HD columns
  const uint32_t tmem_q = tmem_base + HD;            // HD/2 columns: Q, two bf16 channels per column (QT only)
  const uint32_t tmem_s = tmem_base + HD + (QT ? HD / 2 : 0);   // NSB x BKV columns

  if (warp == WARP_TMA) {
    // ---------------------------------------------------------------- producer
    if (lane == 0 && nblk > 0) {
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c)
        tma_load_4d(smem + L::OFF_Q + c * (BQ * 128), &tmap_q, q_full, c * 64, h, q0, b);
      auto load_k = [&](int n) -> bool {
        const int s = n % NK;
        if (!mbar_wait(&k_empty[s], ((n / NK) & 1) ^ 1)) return false;
        mbar_expect_tx(&k_full[s], L::KV_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_4d(smem + L::OFF_K + s * L::KV_BYTES + c * (BKV * 128), &tmap_k, &k_full[s], c * 64, kvh, (jb + n) * BKV, b);
        return true;
      };
      auto load_v = [&](int n) -> bool {
        const int s = n % NV;
        if (!mbar_wait(&v_empty[s], ((n / NV) & 1) ^ 1)) return false;
        mbar_expect_tx(&v_full[s], L::KV_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_4d(smem + L::OFF_V + s * L::KV_BYTES + c * (BKV * 128), &tmap_v, &v_full[s], c * 64, kvh, (jb + n) * BKV, b);
        return true;
      };
      // K runs NSB blocks ahead of V, like the score products run ahead of the P V products.  Every load only
      // waits for products whose own operands were requested earlier in this sequence, so it cannot deadlock.
      bool okp = true;
      for (int n = 0; n < NSB && n < nblk && okp; ++n) okp = load_k(n);
      if (QT && okp) okp = mbar_wait(q_ready, 0);  // the V ring is free once Q has left it
      for (int n = 0; n < nblk && okp; ++n) {
        okp = load_v(n);
        if (okp && n + NSB < nblk) okp = load_k(n + NSB);
      }
      if (!okp) atomicCAS(p.status, 0, ERR_WAIT_EMPTY);
    }
  } else if (warp >= WARP_MMA) {
    // ---------------------------------------------------------------- MMA issuers
    // One thread cannot issue MMAs faster than one per ~54 cycles (measured), while an M128 N64 K16 product takes
    // 32: two threads issue, warp 9 for the even kv blocks and warp 10 for the odd ones.  Each issues, for its
    // blocks, the score product (NSB blocks ahead) and the P V product.  The P V products must enter the pipe in
    // block order (they accumulate into one O, and a rescale of O sits between the products of block n-1 and n),
    // so the threads take turns: P V of block n is issued only after the other thread has issued that of block n-1.
    const int par = warp - WARP_MMA;
    if (lane == 0 && nblk > par) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(BQ, BKV, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BQ, HD, false, true);
      bool ok = QT ? mbar_wait(q_ready, 0) : mbar_wait(q_full, 0);
      if (!ok) atomicCAS(p.status, 0, ERR_WAIT_FULL);
      tc_fence_after();
      const uint64_t dqa0 = make_smem_desc(smem_u32(smem + L::OFF_Q), 16, 1024);
      auto issue_qk = [&](int n) -> bool {
        const int s = n % NK, buf = n % NSB;
        if (!mbar_wait(&k_full[s], (n / NK) & 1)) return false;
        tc_fence_after();
        // one descriptor per tile, stepped by a constant per instruction: k = 64-channel block (k >> 2) and 16-channel
        // step inside it (k & 3); A: 16 channels of Q = 8 packed tensor-memory columns
        const uint64_t db0 = make_smem_desc(smem_u32(smem + L::OFF_K + s * L::KV_BYTES), 16, 1024);
        const uint32_t d_s = tmem_s + buf * BKV;
        if (QT) {
          umma_bf16_ts_c<false>(d_s, tmem_q, db0, idesc_qk);
#pragma unroll
          for (int k = 1; k < HD / 16; ++k)
            umma_bf16_ts_c<true>(d_s, tmem_q + k * 8, smem_desc_advance(db0, (k >> 2) * (BKV * 128) + (k & 3) * 32), idesc_qk);
        } else {
          umma_bf16_ss_c<false>(d_s, dqa0, db0, idesc_qk);
#pragma unroll
          for (int k = 1; k < HD / 16; ++k)
            umma_bf16_ss_c<true>(d_s, smem_desc_advance(dqa0, (k >> 2) * (BQ * 128) + (k & 3) * 32),
                                 smem_desc_advance(db0, (k >> 2) * (BKV * 128) + (k & 3) * 32), idesc_qk);
        }
        umma_commit(&s_full[buf]);
        umma_commit(&k_empty[s]);
        return true;
      };
      for (int n = par; n < NSB && n < nblk && ok; n += 2) ok = issue_qk(n);
      for (int n = par; n < nblk && ok; n += 2) {
        const int buf = n % NSB, sv_i = n % NV;
        if (!mbar_wait(&p_full[buf], (n / NSB) & 1)) {
          ok = false;
          break;
        }
        if (!mbar_wait(&v_full[sv_i], (n / NV) & 1)) {
          ok = false;
          break;
        }
        // my turn: the other thread has issued the P V product of block n-1
        if (n > 0 && !mbar_wait(&pv_turn[par ^ 1], ((n - 1) >> 1) & 1)) {
          ok = false;
          break;
        }
        tc_fence_after();
        // A: 16 kv columns of P = 8 packed tensor-memory columns; B: V tile, HD/64 blocks of [BKV rows x 64
        // channels], MN-major, 16 kv rows (2048 bytes) per step
        const uint64_t dv0 = make_smem_desc(smem_u32(smem + L::OFF_V + sv_i * L::KV_BYTES), BKV * 128, 1024);
        const uint32_t a_p = tmem_s + buf * BKV;
        umma_bf16_ts(tmem_o, a_p, dv0, idesc_pv, n != 0);
#pragma unroll
        for (int k = 1; k < BKV / 16; ++k)
          umma_bf16_ts_c<true>(tmem_o, a_p + k * 8, smem_desc_advance(dv0, k * 2048), idesc_pv);
        tc_fence_before();
        mbar_arrive(&pv_turn[par]);
        umma_commit(&v_empty[sv_i]);
        umma_commit(&pv_done[buf]);
        // the next score product into this buffer executes after the P V product that read it (same thread, in order)
        if (n + NSB < nblk) ok = issue_qk(n + NSB);
      }
      if (!ok) atomicCAS(p.status, 0, ERR_WAIT_MISC);
    }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue (warps 0..7)
    const int set = warp >> 2;   // which of the two alternating sets
    const int qd = warp & 3;     // lane quarter of tensor memory = 32 query rows
    const int row = qd * 32 + lane;
    const int q = q0 + row;
    const uint32_t lane_sel = static_cast<uint32_t>(qd * 32) << 16;
    const int* docb = (p.doc && !p.kv_start) ? p.doc + static_cast<long long>(b) * p.S : nullptr;
    const int dq = (docb && q < p.S) ? docb[q] : 0;
    // admissible kv interval [lo_q, hi_q] of this row
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
    for (int s = 16; s > 0; s >>= 1) {
      w_lo_max = max(w_lo_max, __shfl_xor_sync(0xffffffffu, w_lo_max, s));
      w_hi_min = min(w_hi_min, __shfl_xor_sync(0xffffffffu, w_hi_min, s));
    }
    // ---- Q: shared memory (128-byte swizzle) -> tensor memory; set 0 takes the first half of the channels
    if (QT && nblk > 0) {
      bool okq = mbar_wait(q_full, 0);
      if (!okq) atomicCAS(p.status, 0, ERR_WAIT_FULL);
      constexpr int QB = HD / 64 / 2 > 0 ? HD / 64 / 2 : 1;  // 64-channel blocks per set
      if (HD >= 128 || set == 0) {
#pragma unroll
        for (int bi = 0; bi < QB; ++bi) {
          const int blk = (HD >= 128 ? set * QB : 0) + bi;
          uint32_t qr[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 v4 = *reinterpret_cast<const uint4*>(smem + L::OFF_Q + blk * (BQ * 128) + swz128(row, j));
            qr[j * 4 + 0] = v4.x;
            qr[j * 4 + 1] = v4.y;
            qr[j * 4 + 2] = v4.z;
            qr[j * 4 + 3] = v4.w;
          }
          tmem_st_32x32(tmem_q + blk * 32 + lane_sel, qr);
        }
        tmem_st_wait();
      }
      tc_fence_before();
      mbar_arrive(q_ready);
    }
    const int bar_mine = 1 + qd * 2 + set, bar_other = 1 + qd * 2 + (set ^ 1);
    float* mref = xch;  // [2][128]: reference maximum (log2 domain) published for block n at [n & 1][row]
    float m_mine = -INFINITY, l = 0.f;
    bool ok = true;  // after a failed wait the thread keeps going (the named barriers below must stay paired)
    for (int n = set; n < nblk; n += 2) {
      const int buf = n % NSB;
      const int kv0 = (jb + n) * BKV;
      const uint32_t tbuf = tmem_s + buf * BKV + lane_sel;
      if (ok && !mbar_wait(&s_full[buf], (n / NSB) & 1)) {
        atomicCAS(p.status, 0, ERR_WAIT_SOFTMAX);
        ok = false;
      }
      tc_fence_after();
      const bool need_mask = (docb != nullptr) || kv0 < w_lo_max || kv0 + BKV - 1 > w_hi_min;
      // ---- scores -> registers, mask, block maximum
      uint32_t r[BKV];
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c)
        tmem_ld_32x32(tbuf + c * 32, reinterpret_cast<uint32_t(&)[32]>(r[c * 32]));
      tmem_ld_wait();
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < BKV; ++i) {
          const int kv = kv0 + i;
          bool bad = (kv < lo_q) | (kv > hi_q);
          if (docb && kv < p.S) bad |= docb[kv] != dq;
          if (bad) r[i] = 0xFF800000u;  // -inf: exp2 gives exactly 0
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < BKV; i += 4) {
        mx4[0] = fmaxf(mx4[0], __uint_as_float(r[i]));
        mx4[1] = fmaxf(mx4[1], __uint_as_float(r[i + 1]));
        mx4[2] = fmaxf(mx4[2], __uint_as_float(r[i + 2]));
        mx4[3] = fmaxf(mx4[3], __uint_as_float(r[i + 3]));
      }
      const float m_blk = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
      // ---- agree on the reference maximum with the other set
      float m_prev = -INFINITY;
      if (n > 0) {
        named_sync(bar_other, 64);  // the other set has published the reference of block n-1
        m_prev = mref[((n - 1) & 1) * 128 + row];
      }
      const float m_new = fmaxf(m_prev, m_blk);
      const bool grow = m_new > m_prev + 8.f;  // lazy: keep the old reference unless the maximum moved by > 2^8
      const bool any_grow = __any_sync(0xffffffffu, grow);
      const float m_use = any_grow ? m_new : m_prev;
      mref[(n & 1) * 128 + row] = m_use;
      if (n + 1 < nblk) named_arrive(bar_mine, 64);
      if (any_grow && n > 0) {
        // rescale this row of O once every earlier P V product has completed (they complete in order)
        if (ok && !mbar_wait(&pv_done[(n - 1) % NSB], ((n - 1) / NSB) & 1)) {
          atomicCAS(p.status, 0, ERR_WAIT_SOFTMAX);
          ok = false;
        }
        tc_fence_after();
        const float alpha = (m_prev == -INFINITY) ? 0.f : ex2(m_prev - m_use);
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_o + c * 32 + lane_sel, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(tmem_o + c * 32 + lane_sel, o);
        }
        tmem_st_wait();
      }
      if (m_mine != m_use) {  // this set's partial row sum follows the reference
        l *= (m_mine == -INFINITY) ? 0.f : ex2(m_mine - m_use);
        m_mine = m_use;
      }
      const float m_safe = (m_use == -INFINITY) ? 0.f : m_use;
      // ---- probabilities (bf16, packed) overwrite the scores in tensor memory
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < BKV / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float e0 = ex2(fmaf(__uint_as_float(r[c * 32 + i]), p.scale_log2, -m_safe));
          const float e1 = ex2(fmaf(__uint_as_float(r[c * 32 + i + 1]), p.scale_log2, -m_safe));
          l4[(i >> 1) & 3] += e0 + e1;
          pk[i >> 1] = pack_bf16(e0, e1);
        }
        tmem_st_32x16(tbuf + c * 16, pk);
      }
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[buf]);
    }
    // ---- combine the two sets' row sums in the final reference
    named_sync(9, 256);  // the reference published for the last block is visible to both sets
    const float m_fin = nblk > 0 ? mref[((nblk - 1) & 1) * 128 + row] : -INFINITY;
    named_sync(9, 256);  // everybody has read it: the exchange area may be reused
    float* xl = xch;     // [2 sets][128 rows]
    xl[set * 128 + row] = (m_mine == -INFINITY || m_fin == -INFINITY) ? 0.f : l * ex2(m_mine - m_fin);
    named_sync(9, 256);
    l = xl[row] + xl[128 + row];
    // ---- epilogue: O / l -> global, log-sum-exp.  Set s writes channels [s * HD/2, (s+1) * HD/2).
    if (nblk > 0 && ok) {
      if (!mbar_wait(&pv_done[(nblk - 1) % NSB], ((nblk - 1) / NSB) & 1)) {
        atomicCAS(p.status, 0, ERR_WAIT_ACC_FULL);
        ok = false;
      }
    }
    if (ok) {
      constexpr int OC = HD / 2;
      tc_fence_after();
      const float inv_l = (nblk > 0 && l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.O + ((static_cast<long long>(b) * p.S + q) * p.H + h) * HD + set * OC;
#pragma unroll 1
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t o32[32];
        if (nblk > 0) {
          tmem_ld_32x32(tmem_o + set * OC + c * 32 + lane_sel, o32);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o32[i] = 0;
        }
        if (q < p.S) {
          MB_CHECK_OR(p.status, q >= 0 && b >= 0 && b < p.B && h >= 0 && h < p.H && set * OC + c * 32 + 32 <= HD, continue);
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
      if (set == 0 && q < p.S && p.lse)
        p.lse[(static_cast<long long>(b) * p.H + h) * p.S + q] =
            (nblk > 0 && l > 0.f) ? (m_fin * 0.6931471805599453f + logf(l)) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    __syncwarp();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HD, int BKV, int NK, int NV, int NSB, bool QT>
int launch_fwd(const void* q, const void* k, const void* v, const AttnParams& p, long long q_tok_stride,
               long long k_tok_stride, long long v_tok_stride, cudaStream_t st) {
  using L = Cfg<HD, BKV, NK, NV, NSB, QT>;
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
  MB_SET_MAX_SMEM_ONCE((attn_fwd_kernel<HD, BKV, NK, NV, NSB, QT>), L::TOTAL);
  dim3 grid((p.S + BQ - 1) / BQ, p.H, p.B);
  attn_fwd_kernel<HD, BKV, NK, NV, NSB, QT><<<grid, ATT_THREADS, L::TOTAL, st>>>(tq, tk, tv, p);
  return mbh::check_launch("attn_fwd");
}

}  // namespace

// q: [B,S,H,hd] with token stride q_tok_stride (elements) and head stride hd; k, v likewise with KV
// heads.  out: [B,S,H,hd] contiguous bf16, lse: [B,H,S] fp32 (natural log).  window < 0 disables
// the sliding window; doc / kv_lo_blk / kv_start may be null.  kv_start (per query row, window and
// document start already folded in) needs causal != 0 and replaces doc.
extern "C" int mb_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* doc,
                           const int* kv_lo_blk, const int* kv_start, int B, int S, int H, int KV, int hd,
                           long long q_tok_stride, long long k_tok_stride, long long v_tok_stride, int causal,
                           int window, float scale, cudaStream_t st) {
  AttnParams p;
  p.O = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.doc = doc;
  p.kv_lo_blk = kv_lo_blk;
  p.kv_start = kv_start;
  p.B = B;
  p.S = S;
  p.H = H;
  p.KV = KV;
  p.causal = causal;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = mbh::status().dev;
  if (!p.status) return -4;
  if (kv_start && !causal) return -3;
  if ((q_tok_stride & 7) || (k_tok_stride & 7) || (v_tok_stride & 7)) return -3;
  // head size 256: Q stays in shared memory so that four score buffers fit into tensor memory next to O (the
  // score products then run ahead of the softmax instead of waiting for the P V product that frees their buffer);
  // K stages = 2 and score buffers = 4 keep every K stage and score buffer with the issuing thread of one parity.
  if (hd == 256) return launch_fwd<256, 64, 2, 3, 4, false>(q, k, v, p, q_tok_stride, k_tok_stride, v_tok_stride, st);
  if (hd == 128) return launch_fwd<128, 64, 4, 4, 4, true>(q, k, v, p, q_tok_stride, k_tok_stride, v_tok_stride, st);
  if (hd == 64) return launch_fwd<64, 64, 4, 4, 4, true>(q, k, v, p, q_tok_stride, k_tok_stride, v_tok_stride, st);
  return -3;
}
