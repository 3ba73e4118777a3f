// Packed-sequence (varlen) flash attention for sm_100a on tcgen05 tensor cores - forward and a
// deterministic backward - with MQA/GQA, causal masking, document boundaries and sliding windows.
//
// It replaces the call the reference makes into the flash-attn package
// (src/scaling/core/nn/attention/attention.py:216-271).  Tokens are packed: q[T, Hq, D], k/v[T, Hkv, D];
// doc_start[t] / doc_end[t] give the token range of the document that token t belongs to, so a query
// at t may attend keys in [max(doc_start[t], t - window), causal ? t : min(doc_end[t] - 1, t + window)].
//
// Forward, one CTA per (128-query tile, head):
//   warp 0      TMA: Q once, then K / V tiles (128 keys) through 2-stage rings
//   warp 1      tcgen05.mma issuer: S = Q K^T (accumulator double-buffered in TMEM) and O_j = P V_j
//   warps 2-5   softmax: thread = query row = TMEM lane; online max / sum in the exp2 domain, P written
//               as bf16 into shared memory in the 128-byte-swizzled K-major layout the next MMA reads,
//               running output kept in registers and rescaled when the row maximum moves
// Backward = three launches, no atomics (bitwise reproducible):
//   fa_bwd_delta   delta[h, t] = sum_d dO * O
//   fa_bwd_dkdv    one CTA per (128-key tile, KV head): loops over the query heads of the group and the
//                  query tiles that see these keys; S^T = K Q^T, dP^T = V dO^T, then dV += P^T dO and
//                  dK += dS^T Q accumulate in TMEM over the whole loop
//   fa_bwd_dq      one CTA per (128-query tile, head): S = Q K^T, dP = dO V^T, dQ += dS K in TMEM
// All waits are bounded; on expiry the CTA raises *status and leaves through the common exit (TMEM freed).
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"

namespace {

// forward: TMA warp, MMA warp and 4 softmax warps with one thread per query row (192 threads) or 8 with two (320)
constexpr int FA_BWD_THREADS = 320;  // backward: TMA warp, MMA warp, 8 warps (two threads share a row, 64 columns each)
constexpr int TILE = 128;          // queries per CTA and keys per step
constexpr int PANEL_BYTES = 16384; // 128 rows x 64 bf16

struct FaParams {
  int T, Hq, Hkv;
  int causal;
  int window;        // < 0: unlimited
  float scale_log2;  // softmax scale * log2(e)
  float scale;       // softmax scale
  const int* doc_start;
  const int* doc_end;
  int ldq_head, ldk_head, ldv_head;  // column offset between heads inside a token row (elements)
  int ldo_head;                      // for dO / O tensor maps in the backward
  void* O;           // [T, Hq, D]
  float* lse2;       // [Hq, T]  log2-domain log-sum-exp of the scaled scores
  const float* delta;  // [Hq, T]
  void* dQ;          // [T, Hq, D]
  void* dK;          // [T, Hkv, D]
  void* dV;          // [T, Hkv, D]
  long lddq_tok, lddk_tok, lddv_tok;     // element strides of the gradient outputs: token rows ...
  int lddq_head, lddk_head, lddv_head;   // ... and heads inside a row
  int* status;
  int fp16;  // element type of q, k, v, o and the gradients: 1 = half, 0 = bf16 (selects the F16 instantiations)
  // dropout on the attention probabilities (DROP instantiations): probability (query t, head h, key k) is kept iff
  // byte (k mod 16) of the Philox block (k / 16, (drop_head0 + h) * T + t, drop_call, step) is >= drop_thr8; kept ones are
  // multiplied by keep_scale = 1 / (1 - drop_thr8 / 256).  rng = {seed, step} in device memory.
  const long long* rng;
  uint32_t drop_call, drop_thr8;
  uint32_t drop_head0;  // index of this call's head 0 among all heads of the layer (tensor-parallel shards differ)
  float keep_scale;
};

// mk[i] = keep (byte >= thr8) or 0 for the 32 keys kbase .. kbase + 31 (kbase a multiple of 32) of query row row_id
__device__ __forceinline__ void drop_mask32(const sb::DropoutRng& st, uint32_t row_id, int kbase, uint32_t thr8,
                                            float keep, float* mk) {
#pragma unroll
  for (int b = 0; b < 2; ++b) {
    const uint4 w = sb::philox4x32(st.key, make_uint4((uint32_t)(kbase >> 4) + b, row_id, st.call, st.step));
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 16; ++i) mk[b * 16 + i] = ((ws[i >> 2] >> ((i & 3) * 8)) & 0xffu) >= thr8 ? keep : 0.f;
  }
}

// byte offset of element (row r, column c) inside a K-major operand made of 64-column panels of
// 128 rows x 128 bytes with the 128-byte swizzle (16-byte chunk index xor (row % 8))
__device__ __forceinline__ uint32_t swz_offset(int r, int c) {
  int panel = c >> 6, cc = c & 63;
  int chunk = (cc >> 3) ^ (r & 7);
  return panel * PANEL_BYTES + r * 128 + chunk * 16 + (cc & 7) * 2;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// two floats as a pair of 16-bit values in the kernels' element type (F16: half, else bf16)
template <bool F16>
__device__ __forceinline__ uint32_t pack16(float a, float b) {
  if constexpr (F16) {
    __half2 t = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
  } else {
    __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&t);
  }
}
// K-major operand descriptor for k-step kk (16 elements per step) of a [128 x (64*panels)] tile
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int kk) {
  return sb::umma_smem_desc(base + (kk >> 2) * PANEL_BYTES + (kk & 3) * 32, 16, 1024);
}
// MN-major operand descriptor for k-step kk (16 rows per step) of a tile stored as [K rows x MN cols],
// MN split in 64-column panels of 16 KiB
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int kk) {
  return sb::umma_smem_desc(base + kk * 2048, PANEL_BYTES, 1024);
}

// Phase timing of the forward softmax warps (debug builds with -DSB200_FA_TIMING only): one thread per CTA adds the
// cycles it spent in each phase of the tile loop to g_fa_phase; sb200_fa_timing reads / clears the totals.
#ifdef SB200_FA_TIMING
__device__ unsigned long long g_fa_phase[10];
#define FA_T(i)                                                                          \
  do {                                                                                   \
    const long long now_ = clock64();                                                    \
    if (timing_thread) atomicAdd(&g_fa_phase[i], (unsigned long long)(now_ - t_last));  \
    t_last = now_;                                                                       \
  } while (0)
#else
#define FA_T(i)
#endif

// allowed key range for query row t
__device__ __forceinline__ void row_range(const FaParams& p, int t, int& lo, int& hi) {
  if (t >= p.T) { lo = 1; hi = 0; return; }
  lo = p.doc_start[t];
  hi = p.causal ? t : p.doc_end[t] - 1;
  if (p.window >= 0) {
    lo = max(lo, t - p.window);
    if (!p.causal) hi = min(hi, t + p.window);
  }
}

// ============================================================================ forward
// D = 64 runs two CTAs per SM (256 TMEM columns and under 113 KB of shared memory each: one S buffer, one V stage),
// so that the softmax of one CTA overlaps the MMAs of the other; D = 128 runs one CTA per SM with S and V double
// buffered.  Softmax per tile: pass 1 takes the row maximum of the raw scores, pass 2 computes
// exp2(score * scale_log2 - max) with one FMA + ex2 per element; tiles that lie fully inside a row's allowed key range
// skip the per-element mask tests.
template <int D> struct FaFwdCfg {
  static constexpr bool TWO = D == 64;             // two CTAs per SM
  static constexpr int SBUF = TWO ? 1 : 2;         // S accumulators in TMEM
  // With two CTAs per SM there is room for three K / V stages per CTA.  K(j + 1) is loaded as soon as S(j) has been
  // multiplied and is used a whole softmax later, so one K stage hides its load; V(j) is needed right after the
  // softmax of tile j and its stage is released only by P V of the tile before, so V gets the second stage.
  static constexpr int KST = TWO ? 1 : 2;          // K stages
  static constexpr int VST = 2;                    // V stages
  static constexpr int TMEM_COLS = TWO ? 256 : 512;
  static constexpr int PANELS = D / 64;
  static constexpr int TILE_BYTES = PANELS * PANEL_BYTES;
  static constexpr int XCH_BYTES = 4096;  // row maxima / sums exchanged between the two threads of a row
  static constexpr int SMEM = TILE_BYTES * (1 + KST + VST) + 2 * PANEL_BYTES + 1024 + 256 + XCH_BYTES;
};

// ROWT = threads per query row: 1 (four softmax warps, thread = row) or 2 (eight softmax warps; warps w and w + 4
// share the rows of a TMEM lane quadrant and take 64 key columns and half of the output columns each; they exchange
// their row maxima through shared memory once per tile and their row sums once at the end).  Twice the warps hide
// the TMEM and arithmetic latencies that two warps per scheduler leave exposed.
template <int D, bool DROP, int ROWT, bool F16 = false>
__global__ void __launch_bounds__(64 + 128 * ROWT, FaFwdCfg<D>::TWO ? 2 : 1)
    fa_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const FaParams p) {
  using Cfg = FaFwdCfg<D>;
  constexpr int PANELS = Cfg::PANELS;
  constexpr int TILE_BYTES = Cfg::TILE_BYTES;
  constexpr int SBUF = Cfg::SBUF, VST = Cfg::VST, KST = Cfg::KST;
  constexpr uint32_t S_COL = 0;               // SBUF buffers of 128 columns
  constexpr uint32_t O_COL = SBUF * TILE;     // two O buffers of D columns
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE_BYTES;           // KST stages
  uint8_t* sV = sK + KST * TILE_BYTES;     // VST stages
  uint8_t* sP = sV + VST * TILE_BYTES;     // 2 panels
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * PANEL_BYTES);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2
  uint64_t* p_full = bars + 11;     // 1
  uint64_t* o_full = bars + 12;     // 2
  uint64_t* s_empty = bars + 14;    // 1 (single S buffer only)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xmax = reinterpret_cast<float*>(bars + 32);  // [tile parity][half][row]
  float* xsum = xmax + 4 * TILE;                      // [half][row]
  volatile int* xseq = reinterpret_cast<volatile int*>(xsum + 2 * TILE);  // [half][row]: tiles published so far

#ifdef SB200_FA_TIMING
  const long long t_entry = clock64();
#endif
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // causal: later query tiles of a document see more keys; they are started first, so that the short ones fill the
  // end of the launch instead of a few long ones determining it
  const int q0 = (p.causal ? gridDim.x - 1 - blockIdx.x : blockIdx.x) * TILE;
  const int h = blockIdx.y;
  const int hk = h / (p.Hq / p.Hkv);

  // key tiles this query tile can see
  int lo_first, hi_first, lo_last, hi_last;
  row_range(p, q0, lo_first, hi_first);
  row_range(p, min(q0 + TILE - 1, p.T - 1), lo_last, hi_last);
  const int kv_begin = (lo_first / TILE);
  const int kv_end = (hi_last / TILE) + 1;  // exclusive
  const int n_tiles = kv_end - kv_begin;

  if (threadIdx.x == 0) {
    sb::mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      sb::mbar_init(&k_full[i], 1);
      sb::mbar_init(&k_empty[i], 1);
      sb::mbar_init(&v_full[i], 1);
      sb::mbar_init(&v_empty[i], 1);
      sb::mbar_init(&s_full[i], 1);
      sb::mbar_init(&o_full[i], 1);
    }
    sb::mbar_init(p_full, 4 * ROWT);
    sb::mbar_init(s_empty, 4 * ROWT);
    *abort_flag = 0;
    sb::mbar_fence_init();
  }
  if (ROWT == 2)
    for (int i = threadIdx.x; i < 2 * TILE; i += blockDim.x) xseq[i] = 0;
  if (warp == 1) {
    sb::tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    sb::tmem_relinquish();
  }
  sb::tc_fence_before();
  __syncthreads();
  sb::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      sb::tma_prefetch_desc(&tmQ);
      sb::tma_prefetch_desc(&tmK);
      sb::tma_prefetch_desc(&tmV);
      sb::mbar_expect_tx(q_full, TILE_BYTES);
#pragma unroll
      for (int pn = 0; pn < PANELS; ++pn) sb::tma_load_2d(sQ + pn * PANEL_BYTES, &tmQ, q_full, h * p.ldq_head + pn * 64, q0);
      for (int j = 0; j < n_tiles; ++j) {
        const int kst = j % KST, vst = j % VST;
        const uint32_t kph = (j / KST) & 1, vph = (j / VST) & 1;
        const int kv0 = (kv_begin + j) * TILE;
        if (!sb::mbar_wait(&k_empty[kst], kph ^ 1, abort_flag)) break;
        sb::mbar_expect_tx(&k_full[kst], TILE_BYTES);
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn)
          sb::tma_load_2d(sK + kst * TILE_BYTES + pn * PANEL_BYTES, &tmK, &k_full[kst], hk * p.ldk_head + pn * 64, kv0);
        if (!sb::mbar_wait(&v_empty[vst], vph ^ 1, abort_flag)) break;
        sb::mbar_expect_tx(&v_full[vst], TILE_BYTES);
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn)
          sb::tma_load_2d(sV + vst * TILE_BYTES + pn * PANEL_BYTES, &tmV, &v_full[vst], hk * p.ldv_head + pn * 64, kv0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = sb::umma_idesc_f16(TILE, TILE, F16 ? 0 : 1, 0, 0);  // S = Q K^T: both K-major
      const uint32_t idesc_o = sb::umma_idesc_f16(TILE, D, F16 ? 0 : 1, 0, 1);     // O = P V: V is MN-major
      const uint32_t q_addr = sb::smem_u32(sQ), p_addr = sb::smem_u32(sP);
      bool ok = sb::mbar_wait(q_full, 0, abort_flag);
      auto issue_s = [&](int j) -> bool {
        const int kst = j % KST, sbuf = j % SBUF;
        if (!sb::mbar_wait(&k_full[kst], (j / KST) & 1, abort_flag)) return false;
        if (SBUF == 1 && j > 0) {  // the softmax threads have read S(j - 1) out of the only buffer
          if (!sb::mbar_wait(s_empty, (j - 1) & 1, abort_flag)) return false;
        }
        sb::tc_fence_after();
        const uint32_t k_addr = sb::smem_u32(sK + kst * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          sb::umma_f16_ss(tmem_base + S_COL + sbuf * TILE, desc_kmajor(q_addr, kk), desc_kmajor(k_addr, kk), idesc_s, kk != 0);
        sb::umma_commit(&s_full[sbuf]);
        sb::umma_commit(&k_empty[kst]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int vst = j % VST, obuf = j & 1;
        if (j + 1 < n_tiles) { if (!issue_s(j + 1)) break; }
        if (!sb::mbar_wait(p_full, j & 1, abort_flag)) break;
        if (!sb::mbar_wait(&v_full[vst], (j / VST) & 1, abort_flag)) break;
        sb::tc_fence_after();
        const uint32_t v_addr = sb::smem_u32(sV + vst * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < TILE / 16; ++kk)
          sb::umma_f16_ss(tmem_base + O_COL + obuf * D, desc_kmajor(p_addr, kk), desc_mnmajor(v_addr, kk), idesc_o, kk != 0);
        sb::umma_commit(&o_full[obuf]);
        sb::umma_commit(&v_empty[vst]);
      }
    }
  } else {
    const int quad = warp & 3;
    const int half = ROWT == 2 ? (warp - 2) >> 2 : 0;  // which key columns and output columns of the row are this thread's
    constexpr int CPT = 4 / ROWT;                      // 32-column chunks of S per thread
    constexpr int DT = D / ROWT;                       // output columns per thread
    const int c_begin = half * CPT, c_end = c_begin + CPT;
    const int r = quad * 32 + lane;   // row inside the tile = TMEM lane
    const int t = q0 + r;
    int lo, hi;
    row_range(p, t, lo, hi);
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float sl2 = p.scale_log2;
    // Hand `mine` to the other thread of this row and take its value: the value goes to `vals[half][row]`, then the
    // row's sequence word is raised to `seq`; the partner's word is awaited with a bound (a partner that left after a
    // failed wait has raised the abort flag).  Returns false when the wait ends without the partner's value.
    auto exchange = [&](float* vals, int seq, float mine, float& other) -> bool {
      volatile float* mine_slot = vals + half * TILE + r;
      *mine_slot = mine;
      __threadfence_block();
      xseq[half * TILE + r] = seq;
      unsigned spins = 0;
      while (xseq[(half ^ 1) * TILE + r] < seq) {
        if (*abort_flag || ++spins > (1u << 26)) {
          *abort_flag = 1;
          return false;
        }
      }
      __threadfence_block();
      other = *(volatile float*)(vals + (half ^ 1) * TILE + r);
      return true;
    };
    float m_raw = -1e30f;   // running maximum of the raw scores (the softmax scale is positive)
    float m = __fmul_rn(m_raw, sl2);  // the same in the exp2 domain; kept as a value of its own so that m - mx is exactly 0
                            // while the maximum does not move (recomputing the product could be fused differently)
    float l = 0.f, alpha_prev = 1.f;
    float o_acc[DT];
#pragma unroll
    for (int i = 0; i < DT; ++i) o_acc[i] = 0.f;
    sb::DropoutRng drng = {};
    if (DROP) drng = sb::dropout_rng(p.rng, p.drop_call);
    const uint32_t drow = (p.drop_head0 + (uint32_t)h) * (uint32_t)p.T + (uint32_t)t;
    bool ok = true;
#ifdef SB200_FA_TIMING
    const bool timing_thread = warp == 2 && lane == 0;
    long long t_last = t_entry;
    FA_T(7);  // prologue: barrier and TMEM set-up until the softmax threads are ready for the first tile
#endif
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int sbuf = j % SBUF;
      const int kv0 = (kv_begin + j) * TILE;
      const uint32_t s_addr = t_lane + S_COL + sbuf * TILE;
      if (!sb::mbar_wait(&s_full[sbuf], (j / SBUF) & 1, abort_flag)) { ok = false; break; }
      sb::tc_fence_after();
      FA_T(0);
      const bool interior = kv0 >= lo && kv0 + TILE - 1 <= hi;  // every key of the tile is allowed for this row
      // pass 1: row maximum (four independent chains: a 128-long dependent chain is not hidden by two warps per scheduler)
      float mx4[4] = {m_raw, m_raw, m_raw, m_raw};
      // With two threads per row a thread's 64 scores fit in registers: they are loaded once (both loads in flight
      // together, one wait), the S buffer is released at once, and both passes work from registers.  With one thread
      // per row the 128 scores are read from TMEM chunk by chunk in each pass.
      constexpr bool KEEP_S = ROWT == 2;
      uint32_t sv[KEEP_S ? CPT : 1][32];
      if (KEEP_S) {
#pragma unroll
        for (int c = 0; c < CPT; ++c) sb::tmem_ld32(s_addr + (c_begin + c) * 32, sv[c]);
        sb::tmem_ld_wait();
        if (SBUF == 1) {
          sb::tc_fence_before();
          __syncwarp();
          if (lane == 0) sb::mbar_arrive(s_empty);
        }
      }
#pragma unroll(KEEP_S ? CPT : 1)
      for (int c = 0; c < CPT; ++c) {
        const int ch = c_begin + c;
        uint32_t vt[32];
        if (!KEEP_S) {
          sb::tmem_ld32(s_addr + ch * 32, vt);
          sb::tmem_ld_wait();
        }
        const uint32_t (&v)[32] = KEEP_S ? sv[KEEP_S ? c : 0] : vt;
        if (interior) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kidx = kv0 + ch * 32 + i;
            if (kidx >= lo && kidx <= hi) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[i]));
          }
        }
      }
      float mx_raw = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      FA_T(1);
      if (ROWT == 2) {
        // the row maximum over all 128 keys: the slots alternate with the tile parity, so a thread that is one tile
        // ahead writes the other slot, and it cannot be two tiles ahead without the partner's value of the tile between
        float other;
        if (!exchange(xmax + (j & 1) * 2 * TILE, j + 1, mx_raw, other)) { ok = false; break; }
        mx_raw = fmaxf(mx_raw, other);
      }
      const float mx = __fmul_rn(mx_raw, sl2);  // never contracted into an FMA with its consumers
      const float alpha = fast_exp2(m - mx);
      FA_T(2);
      // the previous P V must be done before P is overwritten
      if (j > 0) {
        if (!sb::mbar_wait(&o_full[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
        sb::tc_fence_after();
      }
      FA_T(3);
      // pass 2: probabilities -> shared memory (bf16, swizzled K-major), row sum
      float rs4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll(KEEP_S ? CPT : 1)
      for (int c = 0; c < CPT; ++c) {
        const int ch = c_begin + c;
        uint32_t vt[32];
        if (!KEEP_S) {
          sb::tmem_ld32(s_addr + ch * 32, vt);
          sb::tmem_ld_wait();
          if (SBUF == 1 && ch == c_end - 1) {  // this warp's part of S is in registers: the next Q K^T may overwrite it
            sb::tc_fence_before();
            __syncwarp();
            if (lane == 0) sb::mbar_arrive(s_empty);
          }
        }
        const uint32_t (&v)[32] = KEEP_S ? sv[KEEP_S ? c : 0] : vt;
        float pr[32];
        if (interior) {
#pragma unroll
          for (int i = 0; i < 32; ++i) pr[i] = fast_exp2(fmaf(__uint_as_float(v[i]), sl2, -mx));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kidx = kv0 + ch * 32 + i;
            pr[i] = (kidx >= lo && kidx <= hi) ? fast_exp2(fmaf(__uint_as_float(v[i]), sl2, -mx)) : 0.f;
          }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) rs4[i & 3] += pr[i];
        if (DROP) {  // the row sum counts every probability; what reaches P V is the kept part (scaled at the end)
          float mk[32];
          drop_mask32(drng, drow, kv0 + ch * 32, p.drop_thr8, 1.f, mk);
#pragma unroll
          for (int i = 0; i < 32; ++i) pr[i] *= mk[i];
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 u;
          u.x = pack16<F16>(pr[g * 8 + 0], pr[g * 8 + 1]);
          u.y = pack16<F16>(pr[g * 8 + 2], pr[g * 8 + 3]);
          u.z = pack16<F16>(pr[g * 8 + 4], pr[g * 8 + 5]);
          u.w = pack16<F16>(pr[g * 8 + 6], pr[g * 8 + 7]);
          *reinterpret_cast<uint4*>(sP + swz_offset(r, ch * 32 + g * 8)) = u;
        }
      }
      FA_T(4);
      sb::fence_proxy_async_smem();
      sb::tc_fence_before();
      __syncwarp();
      if (lane == 0) sb::mbar_arrive(p_full);
      FA_T(5);
      l = l * alpha + ((rs4[0] + rs4[1]) + (rs4[2] + rs4[3]));
      // fold the previous tile's partial output into the running output
      if (j > 0) {
        const int pst = (j - 1) & 1;
#pragma unroll
        for (int ch = 0; ch < DT / 32; ++ch) {
          uint32_t v[32];
          sb::tmem_ld32(t_lane + O_COL + pst * D + half * DT + ch * 32, v);
          sb::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[ch * 32 + i] = fmaf(o_acc[ch * 32 + i], alpha_prev, __uint_as_float(v[i]));
        }
      }
      alpha_prev = alpha;
      m_raw = mx_raw;
      m = mx;
      FA_T(6);
    }
    if (ok && n_tiles > 0) {
      const int pst = (n_tiles - 1) & 1;
      if (sb::mbar_wait(&o_full[pst], ((n_tiles - 1) >> 1) & 1, abort_flag)) {
        sb::tc_fence_after();
#pragma unroll
        for (int ch = 0; ch < DT / 32; ++ch) {
          uint32_t v[32];
          sb::tmem_ld32(t_lane + O_COL + pst * D + half * DT + ch * 32, v);
          sb::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o_acc[ch * 32 + i] = fmaf(o_acc[ch * 32 + i], alpha_prev, __uint_as_float(v[i]));
        }
        if (ROWT == 2) {  // the two threads of a row add their sums (same running maximum, so they are commensurable)
          float other = 0.f;
          if (!exchange(xsum, n_tiles + 1, l, other)) ok = false;
          l += other;
        }
        if (ok && t < p.T) {
          const float inv = l > 0.f ? (DROP ? p.keep_scale : 1.f) / l : 0.f;
          __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.O) + ((long)t * p.Hq + h) * D + half * DT;
#pragma unroll
          for (int g = 0; g < DT / 8; ++g) {
            uint4 u;
            u.x = pack16<F16>(o_acc[g * 8 + 0] * inv, o_acc[g * 8 + 1] * inv);
            u.y = pack16<F16>(o_acc[g * 8 + 2] * inv, o_acc[g * 8 + 3] * inv);
            u.z = pack16<F16>(o_acc[g * 8 + 4] * inv, o_acc[g * 8 + 5] * inv);
            u.w = pack16<F16>(o_acc[g * 8 + 6] * inv, o_acc[g * 8 + 7] * inv);
            *reinterpret_cast<uint4*>(orow + g * 8) = u;
          }
          if (p.lse2 && half == 0) p.lse2[(long)h * p.T + t] = l > 0.f ? m + log2f(l) : -1e30f;
        }
      }
    }
#ifdef SB200_FA_TIMING
    {
      const long long now_ = clock64();
      if (timing_thread) {
        atomicAdd(&g_fa_phase[8], (unsigned long long)(now_ - t_last));   // last P V, normalisation, output
        atomicAdd(&g_fa_phase[9], 1ull);                                  // CTAs
      }
    }
#endif
  }

  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  sb::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    sb::tc_fence_after();
    sb::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) *p.status = SB_ERR_WAIT_TIMEOUT;
}

// ============================================================================ backward: delta
template <int D, bool F16 = false>
__global__ void fa_bwd_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                    float* __restrict__ delta, int T, int Hq) {
  // D / 8 lanes per (t, h) row, one 16-byte load of O and of dO each: the kernel is a stream over both tensors
  constexpr int LPR = D / 8;
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long row = idx / LPR;
  const int part = (int)(idx - row * LPR);
  const bool valid = row < (long)T * Hq;
  float s = 0.f;
  if (valid) {
    const uint4 a = *reinterpret_cast<const uint4*>(O + row * D + part * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(dO + row * D + part * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 x, y;  // the pointers are typed bf16; with F16 the same 16-bit words hold halves
      if constexpr (F16) {
        x = __half22float2(*reinterpret_cast<const __half2*>(&aw[i]));
        y = __half22float2(*reinterpret_cast<const __half2*>(&bw[i]));
      } else {
        x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[i]));
        y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&bw[i]));
      }
      s = fmaf(x.x, y.x, fmaf(x.y, y.y, s));
    }
  }
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);  // rows do not straddle warps
  if (valid && part == 0) {
    const int t = (int)(row / Hq), h = (int)(row - (long)t * Hq);
    delta[(long)h * T + t] = s;
  }
}

// ============================================================================ backward: dK, dV
// CTA = (key tile, KV head, split of the query-head group).  Per (query head, query tile) that sees the keys:
//   S = Q K^T, dP = dO V^T (TMEM lanes = queries)  ->  threads: P, dS as bf16 [queries x keys] in shared memory
//   ->  dV += P^T dO, dK += dS^T Q, reading the same tiles as MN-major A operands; both accumulate in TMEM
//   (lanes = keys) over the whole loop.  With more than one split the results are written as fp32 partials
//   and summed in a fixed order by fa_bwd_reduce_kernel.
template <int D, bool DROP, bool F16 = false>
__global__ void __launch_bounds__(FA_BWD_THREADS, 1)
    fa_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                       const FaParams p, const int q_tile_end_hint, const int heads_per_split,
                       float* __restrict__ dk_partial, float* __restrict__ dv_partial) {
  constexpr int PANELS = D / 64;
  constexpr int TILE_BYTES = PANELS * PANEL_BYTES;
  constexpr int NS = D == 64 ? 2 : 1;  // stages of the Q / dO ring
  constexpr int TMEM_COLS = 512;
  constexpr uint32_t S_COL = 0, DP_COL = 128, DV_COL = 256, DK_COL = 256 + D;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;               // NS stages
  uint8_t* sdO = sQ + NS * TILE_BYTES;         // NS stages
  uint8_t* sP = sdO + NS * TILE_BYTES;         // P  [queries x keys] 2 panels
  uint8_t* sdS = sP + 2 * PANEL_BYTES;         // dS [queries x keys] 2 panels
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + 2 * PANEL_BYTES);
  uint64_t* kv_full = bars;          // 1
  uint64_t* qdo_full = bars + 1;     // NS
  uint64_t* qdo_empty = bars + 3;    // NS
  uint64_t* sdp_full = bars + 5;     // S and dP ready
  uint64_t* pds_full = bars + 6;     // (count 4) P and dS written
  uint64_t* acc_done = bars + 7;     // dV / dK MMAs of the iteration retired
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kv0 = blockIdx.x * TILE;
  const int hk = blockIdx.y;
  const int split = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  const int h_begin = split * heads_per_split;
  const int n_heads = max(min(group - h_begin, heads_per_split), 0);

  // query tiles that can see this key tile (a superset; the element mask decides)
  const int k_last = min(kv0 + TILE - 1, p.T - 1);
  int q_lo = kv0;
  int q_hi = p.doc_end[k_last] - 1;
  if (!p.causal) {
    q_lo = p.doc_start[kv0 < p.T ? kv0 : p.T - 1];
    if (p.window >= 0) q_lo = max(q_lo, kv0 - p.window);
  }
  if (p.window >= 0) q_hi = min(q_hi, k_last + p.window);
  const int qt_begin = q_lo / TILE;
  const int qt_end = min(q_hi / TILE + 1, q_tile_end_hint);
  const int n_qt = max(qt_end - qt_begin, 0);
  const int n_iter = n_qt * n_heads;

  if (threadIdx.x == 0) {
    sb::mbar_init(kv_full, 1);
    for (int i = 0; i < NS; ++i) {
      sb::mbar_init(&qdo_full[i], 1);
      sb::mbar_init(&qdo_empty[i], 1);
    }
    sb::mbar_init(sdp_full, 1);
    sb::mbar_init(pds_full, 8);
    sb::mbar_init(acc_done, 1);
    *abort_flag = 0;
    sb::mbar_fence_init();
  }
  if (warp == 1) {
    sb::tmem_alloc(tmem_slot, TMEM_COLS);
    sb::tmem_relinquish();
  }
  sb::tc_fence_before();
  __syncthreads();
  sb::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      sb::mbar_expect_tx(kv_full, 2 * TILE_BYTES);
#pragma unroll
      for (int pn = 0; pn < PANELS; ++pn) {
        sb::tma_load_2d(sK + pn * PANEL_BYTES, &tmK, kv_full, hk * p.ldk_head + pn * 64, kv0);
        sb::tma_load_2d(sV + pn * PANEL_BYTES, &tmV, kv_full, hk * p.ldv_head + pn * 64, kv0);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int st = it % NS;
        const uint32_t ph = (it / NS) & 1;
        const int h = hk * group + h_begin + it / n_qt;
        const int q0 = (qt_begin + it % n_qt) * TILE;
        if (!sb::mbar_wait(&qdo_empty[st], ph ^ 1, abort_flag)) break;
        sb::mbar_expect_tx(&qdo_full[st], 2 * TILE_BYTES);
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn) {
          sb::tma_load_2d(sQ + st * TILE_BYTES + pn * PANEL_BYTES, &tmQ, &qdo_full[st], h * p.ldq_head + pn * 64, q0);
          sb::tma_load_2d(sdO + st * TILE_BYTES + pn * PANEL_BYTES, &tmdO, &qdo_full[st], h * p.ldo_head + pn * 64, q0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_nt = sb::umma_idesc_f16(TILE, TILE, F16 ? 0 : 1, 0, 0);  // [q x D] x [keys x D]^T
      const uint32_t idesc_acc = sb::umma_idesc_f16(TILE, D, F16 ? 0 : 1, 1, 1);    // [q x keys]^T x [q x D]: both MN-major
      const uint32_t k_addr = sb::smem_u32(sK), v_addr = sb::smem_u32(sV), p_addr = sb::smem_u32(sP),
                     ds_addr = sb::smem_u32(sdS);
      bool ok = sb::mbar_wait(kv_full, 0, abort_flag);
      // S = Q K^T and dP = dO V^T of iteration it + 1 are issued ahead of the accumulation MMAs of iteration it where
      // the Q / dO ring has a second stage, so that the threads compute P and dS of the next tile while the tensor
      // core accumulates dV and dK of this one
      auto issue_sdp = [&](int it) -> bool {
        const int st = it % NS;
        if (!sb::mbar_wait(&qdo_full[st], (it / NS) & 1, abort_flag)) return false;
        sb::tc_fence_after();
        const uint32_t q_addr = sb::smem_u32(sQ + st * TILE_BYTES), do_addr = sb::smem_u32(sdO + st * TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          sb::umma_f16_ss(tmem_base + S_COL, desc_kmajor(q_addr, kk), desc_kmajor(k_addr, kk), idesc_nt, kk != 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          sb::umma_f16_ss(tmem_base + DP_COL, desc_kmajor(do_addr, kk), desc_kmajor(v_addr, kk), idesc_nt, kk != 0);
        sb::umma_commit(sdp_full);
        return true;
      };
      if (ok && n_iter > 0) ok = issue_sdp(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it % NS;
        const uint32_t q_addr = sb::smem_u32(sQ + st * TILE_BYTES), do_addr = sb::smem_u32(sdO + st * TILE_BYTES);
        if (!sb::mbar_wait(pds_full, it & 1, abort_flag)) break;
        if (NS > 1 && it + 1 < n_iter && !issue_sdp(it + 1)) break;
        sb::tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < TILE / 16; ++kk)
          sb::umma_f16_ss(tmem_base + DV_COL, desc_mnmajor(p_addr, kk), desc_mnmajor(do_addr, kk), idesc_acc, (it | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < TILE / 16; ++kk)
          sb::umma_f16_ss(tmem_base + DK_COL, desc_mnmajor(ds_addr, kk), desc_mnmajor(q_addr, kk), idesc_acc, (it | kk) != 0);
        sb::umma_commit(acc_done);
        sb::umma_commit(&qdo_empty[st]);
        if (NS == 1 && it + 1 < n_iter && !issue_sdp(it + 1)) break;
      }
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;  // which 64 columns of the row this thread handles
    const int r = quad * 32 + lane;  // query row inside the tile while computing P / dS, key row in the epilogue
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    const float sl2 = p.scale_log2, sc = p.scale;
    sb::DropoutRng drng = {};
    if (DROP) drng = sb::dropout_rng(p.rng, p.drop_call);
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int h = hk * group + h_begin + it / n_qt;
      const int q0 = (qt_begin + it % n_qt) * TILE;
      const int t = q0 + r;
      int lo, hi;
      row_range(p, t, lo, hi);
      const float lse = t < p.T ? p.lse2[(long)h * p.T + t] : 0.f;
      const float dls = (t < p.T ? p.delta[(long)h * p.T + t] : 0.f) * sc;
      const bool interior = kv0 >= lo && kv0 + TILE - 1 <= hi;  // every key of the tile is allowed for this row
      if (!sb::mbar_wait(sdp_full, it & 1, abort_flag)) { ok = false; break; }
      sb::tc_fence_after();
#pragma unroll 1
      for (int ch = half * 2; ch < half * 2 + 2; ++ch) {
        uint32_t s[32], dp[32];
        sb::tmem_ld32(t_lane + S_COL + ch * 32, s);
        sb::tmem_ld32(t_lane + DP_COL + ch * 32, dp);
        sb::tmem_ld_wait();
        float pv[32], dsv[32];
        if (DROP) {
          // P V used the kept probabilities times keep_scale: dV takes the same, and dP = dO V^T passes the mask
          float mk[32];
          drop_mask32(drng, (p.drop_head0 + (uint32_t)h) * (uint32_t)p.T + (uint32_t)t, kv0 + ch * 32, p.drop_thr8, p.keep_scale, mk);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kidx = kv0 + ch * 32 + i;
            const float pr = (kidx >= lo && kidx <= hi) ? fast_exp2(fmaf(__uint_as_float(s[i]), sl2, -lse)) : 0.f;
            pv[i] = pr * mk[i];
            dsv[i] = pr * fmaf(__uint_as_float(dp[i]) * mk[i], sc, -dls);
          }
        } else if (interior) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float pr = fast_exp2(fmaf(__uint_as_float(s[i]), sl2, -lse));
            pv[i] = pr;
            dsv[i] = pr * fmaf(__uint_as_float(dp[i]), sc, -dls);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kidx = kv0 + ch * 32 + i;
            const float pr = (kidx >= lo && kidx <= hi) ? fast_exp2(fmaf(__uint_as_float(s[i]), sl2, -lse)) : 0.f;
            pv[i] = pr;
            dsv[i] = pr * fmaf(__uint_as_float(dp[i]), sc, -dls);
          }
        }
        if (it > 0 && ch == half * 2) {
          // P and dS are single buffered: the accumulation MMAs of the previous iteration must have read them
          if (!sb::mbar_wait(acc_done, (it - 1) & 1, abort_flag)) { ok = false; break; }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 u, w;
          u.x = pack16<F16>(pv[g * 8 + 0], pv[g * 8 + 1]);
          u.y = pack16<F16>(pv[g * 8 + 2], pv[g * 8 + 3]);
          u.z = pack16<F16>(pv[g * 8 + 4], pv[g * 8 + 5]);
          u.w = pack16<F16>(pv[g * 8 + 6], pv[g * 8 + 7]);
          w.x = pack16<F16>(dsv[g * 8 + 0], dsv[g * 8 + 1]);
          w.y = pack16<F16>(dsv[g * 8 + 2], dsv[g * 8 + 3]);
          w.z = pack16<F16>(dsv[g * 8 + 4], dsv[g * 8 + 5]);
          w.w = pack16<F16>(dsv[g * 8 + 6], dsv[g * 8 + 7]);
          const uint32_t off = swz_offset(r, ch * 32 + g * 8);
          *reinterpret_cast<uint4*>(sP + off) = u;
          *reinterpret_cast<uint4*>(sdS + off) = w;
        }
      }
      sb::fence_proxy_async_smem();
      sb::tc_fence_before();
      __syncwarp();
      if (lane == 0) sb::mbar_arrive(pds_full);
    }
    // results: TMEM lane = key row
    const int kidx = kv0 + r;
    const bool have = ok && n_iter > 0 && sb::mbar_wait(acc_done, (n_iter - 1) & 1, abort_flag);
    if (have) sb::tc_fence_after();
    if (ok && (have || n_iter == 0)) {
      const long row = (long)kidx * p.Hkv + hk;
#pragma unroll 1
      for (int ch = half; ch < D / 32; ch += 2) {
        uint32_t a[32], b[32];
        if (have) {
          sb::tmem_ld32(t_lane + DV_COL + ch * 32, a);
          sb::tmem_ld32(t_lane + DK_COL + ch * 32, b);
          sb::tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { a[i] = 0u; b[i] = 0u; }
        }
        if (kidx < p.T) {
          if (dk_partial) {
            float* pk = dk_partial + ((long)split * p.T * p.Hkv + row) * D + ch * 32;
            float* pv2 = dv_partial + ((long)split * p.T * p.Hkv + row) * D + ch * 32;
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              *reinterpret_cast<uint4*>(pv2 + g * 4) = make_uint4(a[g * 4], a[g * 4 + 1], a[g * 4 + 2], a[g * 4 + 3]);
              *reinterpret_cast<uint4*>(pk + g * 4) = make_uint4(b[g * 4], b[g * 4 + 1], b[g * 4 + 2], b[g * 4 + 3]);
            }
          } else {
            __nv_bfloat16* dk = reinterpret_cast<__nv_bfloat16*>(p.dK) + (long)kidx * p.lddk_tok +
                                (long)hk * p.lddk_head + ch * 32;
            __nv_bfloat16* dv = reinterpret_cast<__nv_bfloat16*>(p.dV) + (long)kidx * p.lddv_tok +
                                (long)hk * p.lddv_head + ch * 32;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 u, w;
              u.x = pack16<F16>(__uint_as_float(a[g * 8 + 0]), __uint_as_float(a[g * 8 + 1]));
              u.y = pack16<F16>(__uint_as_float(a[g * 8 + 2]), __uint_as_float(a[g * 8 + 3]));
              u.z = pack16<F16>(__uint_as_float(a[g * 8 + 4]), __uint_as_float(a[g * 8 + 5]));
              u.w = pack16<F16>(__uint_as_float(a[g * 8 + 6]), __uint_as_float(a[g * 8 + 7]));
              w.x = pack16<F16>(__uint_as_float(b[g * 8 + 0]), __uint_as_float(b[g * 8 + 1]));
              w.y = pack16<F16>(__uint_as_float(b[g * 8 + 2]), __uint_as_float(b[g * 8 + 3]));
              w.z = pack16<F16>(__uint_as_float(b[g * 8 + 4]), __uint_as_float(b[g * 8 + 5]));
              w.w = pack16<F16>(__uint_as_float(b[g * 8 + 6]), __uint_as_float(b[g * 8 + 7]));
              *reinterpret_cast<uint4*>(dv + g * 8) = u;
              *reinterpret_cast<uint4*>(dk + g * 8) = w;
            }
          }
        }
      }
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  sb::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    sb::tc_fence_after();
    sb::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) *p.status = SB_ERR_WAIT_TIMEOUT;
}

// out[t, h, c] = bf16(sum_s partial[s][t, h, c]) in fixed order; partial rows are dense [T, H, D], the output has
// element strides (ld_tok, ld_head)
template <bool F16 = false>
__global__ void fa_bwd_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, long n,
                                     int splits, int H, int D, long ld_tok, int ld_head) {
  long i = (blockIdx.x * (long)blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < splits; ++s) {
    float4 v = *reinterpret_cast<const float4*>(partial + (long)s * n + i);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  uint2 u;
  u.x = pack16<F16>(acc.x, acc.y);
  u.y = pack16<F16>(acc.z, acc.w);
  const long th = i / D;
  const int c = (int)(i - th * D);
  const long t = th / H;
  const int h = (int)(th - t * H);
  *reinterpret_cast<uint2*>(out + t * ld_tok + (long)h * ld_head + c) = u;
}

// ============================================================================ backward: dQ
// CTA = (query tile, head).  Per key tile: S = Q K^T, dP = dO V^T -> threads: dS (bf16) -> dQ += dS K
template <int D, bool DROP, bool F16 = false>
__global__ void __launch_bounds__(FA_BWD_THREADS, 1)
    fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                     const FaParams p) {
  constexpr int PANELS = D / 64;
  constexpr int TILE_BYTES = PANELS * PANEL_BYTES;
  constexpr int TMEM_COLS = 512;
  constexpr uint32_t S_COL = 0, DP_COL = 128, DQ_COL = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + TILE_BYTES;
  uint8_t* sK = sdO + TILE_BYTES;           // 2 stages
  uint8_t* sV = sK + 2 * TILE_BYTES;        // 2 stages
  uint8_t* sdS = sV + 2 * TILE_BYTES;       // [queries x keys] 2 panels
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + 2 * PANEL_BYTES);
  uint64_t* qdo_full = bars;
  uint64_t* kv_full = bars + 1;    // 2
  uint64_t* kv_empty = bars + 3;   // 2
  uint64_t* sdp_full = bars + 5;
  uint64_t* ds_full = bars + 6;    // count 8
  uint64_t* acc_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = (p.causal ? gridDim.x - 1 - blockIdx.x : blockIdx.x) * TILE;  // longest query tiles first
  const int h = blockIdx.y;
  const int hk = h / (p.Hq / p.Hkv);
  int lo_first, hi_first, lo_last, hi_last;
  row_range(p, q0, lo_first, hi_first);
  row_range(p, min(q0 + TILE - 1, p.T - 1), lo_last, hi_last);
  const int kv_begin = lo_first / TILE;
  const int n_tiles = hi_last / TILE + 1 - kv_begin;

  if (threadIdx.x == 0) {
    sb::mbar_init(qdo_full, 1);
    for (int i = 0; i < 2; ++i) {
      sb::mbar_init(&kv_full[i], 1);
      sb::mbar_init(&kv_empty[i], 1);
    }
    sb::mbar_init(sdp_full, 1);
    sb::mbar_init(ds_full, 8);
    sb::mbar_init(acc_done, 1);
    *abort_flag = 0;
    sb::mbar_fence_init();
  }
  if (warp == 1) {
    sb::tmem_alloc(tmem_slot, TMEM_COLS);
    sb::tmem_relinquish();
  }
  sb::tc_fence_before();
  __syncthreads();
  sb::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      sb::mbar_expect_tx(qdo_full, 2 * TILE_BYTES);
#pragma unroll
      for (int pn = 0; pn < PANELS; ++pn) {
        sb::tma_load_2d(sQ + pn * PANEL_BYTES, &tmQ, qdo_full, h * p.ldq_head + pn * 64, q0);
        sb::tma_load_2d(sdO + pn * PANEL_BYTES, &tmdO, qdo_full, h * p.ldo_head + pn * 64, q0);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const int kv0 = (kv_begin + j) * TILE;
        const int st = j & 1;
        if (!sb::mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1, abort_flag)) break;
        sb::mbar_expect_tx(&kv_full[st], 2 * TILE_BYTES);
#pragma unroll
        for (int pn = 0; pn < PANELS; ++pn) {
          sb::tma_load_2d(sK + st * TILE_BYTES + pn * PANEL_BYTES, &tmK, &kv_full[st], hk * p.ldk_head + pn * 64, kv0);
          sb::tma_load_2d(sV + st * TILE_BYTES + pn * PANEL_BYTES, &tmV, &kv_full[st], hk * p.ldv_head + pn * 64, kv0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_nt = sb::umma_idesc_f16(TILE, TILE, F16 ? 0 : 1, 0, 0);
      const uint32_t idesc_acc = sb::umma_idesc_f16(TILE, D, F16 ? 0 : 1, 0, 1);
      const uint32_t q_addr = sb::smem_u32(sQ), do_addr = sb::smem_u32(sdO), k_base = sb::smem_u32(sK),
                     v_base = sb::smem_u32(sV), ds_addr = sb::smem_u32(sdS);
      bool ok = sb::mbar_wait(qdo_full, 0, abort_flag);
      // S(j) = Q K_j^T and dP(j) = dO V_j^T share one TMEM buffer each; they are issued for tile j + 1 as soon as
      // the threads have read tile j, ahead of dQ += dS_j K_j, so that the threads work on tile j + 1 while the
      // tensor core accumulates dQ of tile j
      auto issue_sdp = [&](int j) -> bool {
        const int st = j & 1;
        if (!sb::mbar_wait(&kv_full[st], (j >> 1) & 1, abort_flag)) return false;
        sb::tc_fence_after();
        const uint32_t k_addr = k_base + st * TILE_BYTES, v_addr = v_base + st * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          sb::umma_f16_ss(tmem_base + S_COL, desc_kmajor(q_addr, kk), desc_kmajor(k_addr, kk), idesc_nt, kk != 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          sb::umma_f16_ss(tmem_base + DP_COL, desc_kmajor(do_addr, kk), desc_kmajor(v_addr, kk), idesc_nt, kk != 0);
        sb::umma_commit(sdp_full);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_sdp(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        if (!sb::mbar_wait(ds_full, j & 1, abort_flag)) break;  // dS(j) is in shared memory, S / dP(j) have been read
        if (j + 1 < n_tiles && !issue_sdp(j + 1)) break;
        sb::tc_fence_after();
        const uint32_t k_addr = k_base + st * TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < TILE / 16; ++kk)
          sb::umma_f16_ss(tmem_base + DQ_COL, desc_kmajor(ds_addr, kk), desc_mnmajor(k_addr, kk), idesc_acc, (j | kk) != 0);
        sb::umma_commit(acc_done);
        sb::umma_commit(&kv_empty[st]);
      }
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;  // which 64 columns of the row this thread handles
    const int r = quad * 32 + lane;
    const int t = q0 + r;
    int lo, hi;
    row_range(p, t, lo, hi);
    const float sl2 = p.scale_log2, sc = p.scale;
    const float lse = t < p.T ? p.lse2[(long)h * p.T + t] : 0.f;
    const float dls = (t < p.T ? p.delta[(long)h * p.T + t] : 0.f) * sc;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    sb::DropoutRng drng = {};
    if (DROP) drng = sb::dropout_rng(p.rng, p.drop_call);
    const uint32_t drow = (p.drop_head0 + (uint32_t)h) * (uint32_t)p.T + (uint32_t)t;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int kv0 = (kv_begin + j) * TILE;
      const bool interior = kv0 >= lo && kv0 + TILE - 1 <= hi;  // every key of the tile is allowed for this row
      if (!sb::mbar_wait(sdp_full, j & 1, abort_flag)) { ok = false; break; }
      sb::tc_fence_after();
#pragma unroll 1
      for (int ch = half * 2; ch < half * 2 + 2; ++ch) {
        uint32_t s[32], dp[32];
        sb::tmem_ld32(t_lane + S_COL + ch * 32, s);
        sb::tmem_ld32(t_lane + DP_COL + ch * 32, dp);
        sb::tmem_ld_wait();
        float dsv[32];
        if (DROP) {
          float mk[32];
          drop_mask32(drng, drow, kv0 + ch * 32, p.drop_thr8, p.keep_scale, mk);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kidx = kv0 + ch * 32 + i;
            const float pr = (kidx >= lo && kidx <= hi) ? fast_exp2(fmaf(__uint_as_float(s[i]), sl2, -lse)) : 0.f;
            dsv[i] = pr * fmaf(__uint_as_float(dp[i]) * mk[i], sc, -dls);
          }
        } else if (interior) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            dsv[i] = fast_exp2(fmaf(__uint_as_float(s[i]), sl2, -lse)) * fmaf(__uint_as_float(dp[i]), sc, -dls);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kidx = kv0 + ch * 32 + i;
            const float pr = (kidx >= lo && kidx <= hi) ? fast_exp2(fmaf(__uint_as_float(s[i]), sl2, -lse)) : 0.f;
            dsv[i] = pr * fmaf(__uint_as_float(dp[i]), sc, -dls);
          }
        }
        if (j > 0 && ch == half * 2) {
          // dS is single buffered: dQ += dS(j - 1) K must have finished reading it (it was issued right behind this
          // tile's S / dP, so the wait is short and the first chunk's arithmetic above already overlapped it)
          if (!sb::mbar_wait(acc_done, (j - 1) & 1, abort_flag)) { ok = false; break; }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w;
          w.x = pack16<F16>(dsv[g * 8 + 0], dsv[g * 8 + 1]);
          w.y = pack16<F16>(dsv[g * 8 + 2], dsv[g * 8 + 3]);
          w.z = pack16<F16>(dsv[g * 8 + 4], dsv[g * 8 + 5]);
          w.w = pack16<F16>(dsv[g * 8 + 6], dsv[g * 8 + 7]);
          *reinterpret_cast<uint4*>(sdS + swz_offset(r, ch * 32 + g * 8)) = w;
        }
      }
      sb::fence_proxy_async_smem();
      sb::tc_fence_before();
      __syncwarp();
      if (lane == 0) sb::mbar_arrive(ds_full);
    }
    if (ok && n_tiles > 0 && sb::mbar_wait(acc_done, (n_tiles - 1) & 1, abort_flag)) {
      sb::tc_fence_after();
      __nv_bfloat16* dq = reinterpret_cast<__nv_bfloat16*>(p.dQ) + (long)t * p.lddq_tok + (long)h * p.lddq_head;
#pragma unroll 1
      for (int ch = half; ch < D / 32; ch += 2) {
        uint32_t a[32];
        sb::tmem_ld32(t_lane + DQ_COL + ch * 32, a);
        sb::tmem_ld_wait();
        if (t < p.T) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 u;
            u.x = pack16<F16>(__uint_as_float(a[g * 8 + 0]), __uint_as_float(a[g * 8 + 1]));
            u.y = pack16<F16>(__uint_as_float(a[g * 8 + 2]), __uint_as_float(a[g * 8 + 3]));
            u.z = pack16<F16>(__uint_as_float(a[g * 8 + 4]), __uint_as_float(a[g * 8 + 5]));
            u.w = pack16<F16>(__uint_as_float(a[g * 8 + 6]), __uint_as_float(a[g * 8 + 7]));
            *reinterpret_cast<uint4*>(dq + ch * 32 + g * 8) = u;
          }
        }
      }
    }
  }

  if (*abort_flag) {
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  sb::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    sb::tc_fence_after();
    sb::tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) *p.status = SB_ERR_WAIT_TIMEOUT;
}

// ============================================================================ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn fa_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(ptr);
  return fn;
}
int g_fa_last_driver_error = 0;
// [T rows, cols] bf16 view with row pitch ld (elements); box = 128 rows x 64 columns, 128-byte swizzle
int fa_tmap(CUtensorMap* tm, const void* base, long T, long cols, long ld) {
  EncodeTiledFn fn = fa_encode_fn();
  if (!fn) return SB_ERR_DRIVER;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)T};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, TILE};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) g_fa_last_driver_error = (int)r;
  return r == CUDA_SUCCESS ? SB_OK : SB_ERR_DRIVER;
}

template <int D> constexpr int fa_fwd_smem() { return FaFwdCfg<D>::SMEM; }
template <int D> constexpr int fa_dkdv_smem() { return (D / 64) * PANEL_BYTES * (2 + 2 * (D == 64 ? 2 : 1)) + 4 * PANEL_BYTES + 1024 + 256; }
template <int D> constexpr int fa_dq_smem() { return (D / 64) * PANEL_BYTES * 6 + 2 * PANEL_BYTES + 1024 + 256; }

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// dropout probability -> threshold on a random byte and the factor of the kept probabilities; p is quantised to 1/256
int fa_dropout(FaParams* p, float dropout_p, const long long* rng, unsigned call, int head0) {
  p->rng = nullptr; p->drop_call = 0; p->drop_thr8 = 0; p->keep_scale = 1.f; p->drop_head0 = (uint32_t)head0;
  if (dropout_p <= 0.f) return SB_OK;
  if (dropout_p >= 1.f || !rng) return SB_ERR_BAD_ARG;
  int thr = (int)(dropout_p * 256.f + 0.5f);
  if (thr < 1) thr = 1;
  if (thr > 255) thr = 255;
  p->rng = rng; p->drop_call = call; p->drop_thr8 = (uint32_t)thr;
  p->keep_scale = 256.f / (float)(256 - thr);
  return SB_OK;
}

template <int D, bool DROP, int ROWT, bool F16>
int fa_launch_fwd_type(dim3 grid, const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                       const FaParams& p, cudaStream_t stream) {
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(fa_fwd_kernel<D, DROP, ROWT, F16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         fa_fwd_smem<D>());
    if (e != cudaSuccess) return (int)e;
    set = true;
  }
  fa_fwd_kernel<D, DROP, ROWT, F16><<<grid, 64 + 128 * ROWT, fa_fwd_smem<D>(), stream>>>(tmQ, tmK, tmV, p);
  SB_CHECK_LAUNCH();
  return SB_OK;
}
template <int D, bool DROP, int ROWT>
int fa_launch_fwd_rowt(dim3 grid, const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                       const FaParams& p, cudaStream_t stream) {
  return p.fp16 ? fa_launch_fwd_type<D, DROP, ROWT, true>(grid, tmQ, tmK, tmV, p, stream)
                : fa_launch_fwd_type<D, DROP, ROWT, false>(grid, tmQ, tmK, tmV, p, stream);
}
template <int D, bool DROP>
int fa_launch_fwd(dim3 grid, const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const FaParams& p,
                  cudaStream_t stream) {
  // two threads per row pay off at head size 128 (one CTA per SM: eight instead of four softmax warps); at 64, two
  // CTAs per SM already give eight.  SB200_FA_ROW_THREADS = 1 | 2 overrides the choice (for measurements).
  static int rowt = 0;
  if (!rowt) {
    const char* e = getenv("SB200_FA_ROW_THREADS");
    const int want = e ? atoi(e) : 0;
    rowt = (want == 1 || want == 2) ? want : (D == 128 ? 2 : 1);
  }
  if (rowt == 1) return fa_launch_fwd_rowt<D, DROP, 1>(grid, tmQ, tmK, tmV, p, stream);
  return fa_launch_fwd_rowt<D, DROP, 2>(grid, tmQ, tmK, tmV, p, stream);
}

template <int D, bool DROP, bool F16>
int fa_launch_bwd_type(int tiles, int splits, int hps, const CUtensorMap& tmQ, const CUtensorMap& tmK,
                       const CUtensorMap& tmV, const CUtensorMap& tmdO, const FaParams& p, float* dk_part,
                       float* dv_part, cudaStream_t stream) {
  static bool set = false;
  if (!set) {
    cudaError_t e = cudaFuncSetAttribute(fa_bwd_dkdv_kernel<D, DROP, F16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         fa_dkdv_smem<D>());
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(fa_bwd_dq_kernel<D, DROP, F16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               fa_dq_smem<D>());
    if (e != cudaSuccess) return (int)e;
    set = true;
  }
  fa_bwd_dkdv_kernel<D, DROP, F16><<<dim3(tiles, p.Hkv, splits), FA_BWD_THREADS, fa_dkdv_smem<D>(), stream>>>(
      tmQ, tmK, tmV, tmdO, p, tiles, hps, dk_part, dv_part);
  SB_CHECK_LAUNCH();
  fa_bwd_dq_kernel<D, DROP, F16><<<dim3(tiles, p.Hq), FA_BWD_THREADS, fa_dq_smem<D>(), stream>>>(tmQ, tmK, tmV, tmdO, p);
  SB_CHECK_LAUNCH();
  return SB_OK;
}
template <int D, bool DROP>
int fa_launch_bwd(int tiles, int splits, int hps, const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV,
                  const CUtensorMap& tmdO, const FaParams& p, float* dk_part, float* dv_part, cudaStream_t stream) {
  return p.fp16 ? fa_launch_bwd_type<D, DROP, true>(tiles, splits, hps, tmQ, tmK, tmV, tmdO, p, dk_part, dv_part, stream)
                : fa_launch_bwd_type<D, DROP, false>(tiles, splits, hps, tmQ, tmK, tmV, tmdO, p, dk_part, dv_part, stream);
}

}  // namespace

#ifdef SB200_FA_TIMING
// out8: host array of 10 counters (cycles summed over one thread of every CTA; the last is the number of CTAs);
// reset != 0 clears them afterwards
SB_API int sb200_fa_timing(unsigned long long* out8, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out8, g_fa_phase, sizeof(g_fa_phase));
  if (e != cudaSuccess) return (int)e;
  if (reset) {
    unsigned long long zero[10] = {};
    e = cudaMemcpyToSymbol(g_fa_phase, zero, sizeof(zero));
  }
  return (int)e;
}
#endif

// CUresult of the last failed tensor-map encode of the attention entry points (0 if none failed)
SB_API int sb200_fa_last_driver_error() { return g_fa_last_driver_error; }

// q: [T, Hq, D] view with token pitch ldq_tok and head pitch ldq_head (elements); k, v likewise; o: [T, Hq, D] contiguous.
// dropout_p > 0 drops attention probabilities (quantised to a multiple of 1/256): rng = device int64[2] {seed, step},
// call = index of this attention inside the step, head0 = index of head 0 among the heads of the whole layer; the
// backward pass is given the same values.
SB_API int sb200_fa_fwd(const void* q, const void* k, const void* v, void* o, float* lse2, const int* doc_start,
                        const int* doc_end, int T, int Hq, int Hkv, int D, long ldq_tok, int ldq_head, long ldk_tok,
                        int ldk_head, long ldv_tok, int ldv_head, int causal, int window, float scale,
                        float dropout_p, const long long* rng, unsigned int call, int head0, int dtype, int* status,
                        cudaStream_t stream) {
  if (T <= 0 || Hq <= 0) return SB_OK;
  if ((D != 64 && D != 128) || Hkv <= 0 || Hq % Hkv) return SB_ERR_BAD_ARG;
  if (dtype != SB_DT_BF16 && dtype != SB_DT_F16) return SB_ERR_BAD_ARG;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return SB_ERR_BAD_ARG;
  if ((ldq_tok % 8) || (ldk_tok % 8) || (ldv_tok % 8) || (ldq_head % 8) || (ldk_head % 8) || (ldv_head % 8))
    return SB_ERR_BAD_ARG;
  CUtensorMap tmQ, tmK, tmV;
  int rc;
  if ((rc = fa_tmap(&tmQ, q, T, (long)(Hq - 1) * ldq_head + D, ldq_tok))) return rc;
  if ((rc = fa_tmap(&tmK, k, T, (long)(Hkv - 1) * ldk_head + D, ldk_tok))) return rc;
  if ((rc = fa_tmap(&tmV, v, T, (long)(Hkv - 1) * ldv_head + D, ldv_tok))) return rc;
  FaParams p = {};
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.window = window;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.doc_start = doc_start; p.doc_end = doc_end;
  p.ldq_head = ldq_head; p.ldk_head = ldk_head; p.ldv_head = ldv_head;
  p.O = o; p.lse2 = lse2; p.status = status; p.fp16 = dtype == SB_DT_F16;
  if ((rc = fa_dropout(&p, dropout_p, rng, call, head0))) return rc;
  dim3 grid((T + TILE - 1) / TILE, Hq);
  if (D == 64) return p.drop_thr8 ? fa_launch_fwd<64, true>(grid, tmQ, tmK, tmV, p, stream)
                                  : fa_launch_fwd<64, false>(grid, tmQ, tmK, tmV, p, stream);
  return p.drop_thr8 ? fa_launch_fwd<128, true>(grid, tmQ, tmK, tmV, p, stream)
                     : fa_launch_fwd<128, false>(grid, tmQ, tmK, tmV, p, stream);
}

// Number of splits of the query-head group the dK/dV kernel uses for this problem (1 = results written directly).
// With more than one split the caller passes a scratch of 2 * splits * T * Hkv * D floats.
SB_API int sb200_fa_bwd_splits(int T, int Hq, int Hkv, int sm_count) {
  if (Hkv <= 0 || Hq % Hkv) return 1;
  const int group = Hq / Hkv;
  const int tiles = (T + TILE - 1) / TILE;
  const long ctas = (long)tiles * Hkv;
  if (group == 1 || ctas >= 2L * sm_count) return 1;
  int want = (int)((2L * sm_count + ctas - 1) / ctas);
  if (want > group) want = group;
  const int hps = (group + want - 1) / want;
  return (group + hps - 1) / hps;
}

// Backward.  o, d_o: [T, Hq, D] contiguous; delta: scratch [Hq, T] floats; dkv_partial: scratch for split
// accumulation (see sb200_fa_bwd_splits), may be null when splits == 1.  The gradients dq [T, Hq, D] and
// dk, dv [T, Hkv, D] have unit stride in D and the given element strides between token rows and heads (multiples
// of 8), so that they can be views into one packed buffer.
SB_API int sb200_fa_bwd_strided(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                const float* lse2, float* delta, float* dkv_partial, int splits, void* dq, void* dk,
                                void* dv, const int* doc_start, const int* doc_end, int T, int Hq, int Hkv, int D,
                                long ldq_tok, int ldq_head, long ldk_tok, int ldk_head, long ldv_tok, int ldv_head,
                                long lddq_tok, int lddq_head, long lddk_tok, int lddk_head, long lddv_tok,
                                int lddv_head, int causal, int window, float scale, float dropout_p,
                                const long long* rng, unsigned int call, int head0, int dtype, int* status,
                                cudaStream_t stream) {
  if ((lddq_tok | lddq_head | lddk_tok | lddk_head | lddv_tok | lddv_head) & 7) return SB_ERR_BAD_ARG;
  if (dtype != SB_DT_BF16 && dtype != SB_DT_F16) return SB_ERR_BAD_ARG;
  if (T <= 0 || Hq <= 0) return SB_OK;
  if ((D != 64 && D != 128) || Hkv <= 0 || Hq % Hkv) return SB_ERR_BAD_ARG;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(d_o) || !aligned16(dq) ||
      !aligned16(dk) || !aligned16(dv))
    return SB_ERR_BAD_ARG;
  CUtensorMap tmQ, tmK, tmV, tmdO;
  int rc;
  if ((rc = fa_tmap(&tmQ, q, T, (long)(Hq - 1) * ldq_head + D, ldq_tok))) return rc;
  if ((rc = fa_tmap(&tmK, k, T, (long)(Hkv - 1) * ldk_head + D, ldk_tok))) return rc;
  if ((rc = fa_tmap(&tmV, v, T, (long)(Hkv - 1) * ldv_head + D, ldv_tok))) return rc;
  if ((rc = fa_tmap(&tmdO, d_o, T, (long)Hq * D, (long)Hq * D))) return rc;
  FaParams p = {};
  p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.causal = causal; p.window = window;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.doc_start = doc_start; p.doc_end = doc_end;
  p.ldq_head = ldq_head; p.ldk_head = ldk_head; p.ldv_head = ldv_head; p.ldo_head = D;
  p.lse2 = const_cast<float*>(lse2); p.delta = delta; p.dQ = dq; p.dK = dk; p.dV = dv; p.status = status;
  p.fp16 = dtype == SB_DT_F16;
  p.lddq_tok = lddq_tok; p.lddk_tok = lddk_tok; p.lddv_tok = lddv_tok;
  p.lddq_head = lddq_head; p.lddk_head = lddk_head; p.lddv_head = lddv_head;
  const int tiles = (T + TILE - 1) / TILE;
  const int group = Hq / Hkv;
  if (splits < 1) splits = 1;
  if (splits > 1 && !dkv_partial) return SB_ERR_BAD_ARG;
  const int hps = (group + splits - 1) / splits;
  float* dk_part = splits > 1 ? dkv_partial : nullptr;
  float* dv_part = splits > 1 ? dkv_partial + (long)splits * T * Hkv * D : nullptr;
  {
    const long threads = (long)T * Hq * (D / 8);
    int blocks = (int)((threads + 255) / 256);
    const __nv_bfloat16* o16 = (const __nv_bfloat16*)o;  // 16-bit words; the F16 instantiations read them as halves
    const __nv_bfloat16* do16 = (const __nv_bfloat16*)d_o;
    if (D == 64) {
      if (p.fp16) fa_bwd_delta_kernel<64, true><<<blocks, 256, 0, stream>>>(o16, do16, delta, T, Hq);
      else fa_bwd_delta_kernel<64, false><<<blocks, 256, 0, stream>>>(o16, do16, delta, T, Hq);
    } else {
      if (p.fp16) fa_bwd_delta_kernel<128, true><<<blocks, 256, 0, stream>>>(o16, do16, delta, T, Hq);
      else fa_bwd_delta_kernel<128, false><<<blocks, 256, 0, stream>>>(o16, do16, delta, T, Hq);
    }
    SB_CHECK_LAUNCH();
  }
  if ((rc = fa_dropout(&p, dropout_p, rng, call, head0))) return rc;
  if (D == 64)
    rc = p.drop_thr8 ? fa_launch_bwd<64, true>(tiles, splits, hps, tmQ, tmK, tmV, tmdO, p, dk_part, dv_part, stream)
                     : fa_launch_bwd<64, false>(tiles, splits, hps, tmQ, tmK, tmV, tmdO, p, dk_part, dv_part, stream);
  else
    rc = p.drop_thr8 ? fa_launch_bwd<128, true>(tiles, splits, hps, tmQ, tmK, tmV, tmdO, p, dk_part, dv_part, stream)
                     : fa_launch_bwd<128, false>(tiles, splits, hps, tmQ, tmK, tmV, tmdO, p, dk_part, dv_part, stream);
  if (rc) return rc;
  if (splits > 1) {
    const long n = (long)T * Hkv * D;
    const int blocks = (int)((n / 4 + 255) / 256);
    if (p.fp16) {
      fa_bwd_reduce_kernel<true><<<blocks, 256, 0, stream>>>(dk_part, (__nv_bfloat16*)dk, n, splits, Hkv, D, lddk_tok,
                                                             lddk_head);
      fa_bwd_reduce_kernel<true><<<blocks, 256, 0, stream>>>(dv_part, (__nv_bfloat16*)dv, n, splits, Hkv, D, lddv_tok,
                                                             lddv_head);
    } else {
      fa_bwd_reduce_kernel<false><<<blocks, 256, 0, stream>>>(dk_part, (__nv_bfloat16*)dk, n, splits, Hkv, D, lddk_tok,
                                                              lddk_head);
      fa_bwd_reduce_kernel<false><<<blocks, 256, 0, stream>>>(dv_part, (__nv_bfloat16*)dv, n, splits, Hkv, D, lddv_tok,
                                                              lddv_head);
    }
    SB_CHECK_LAUNCH();
  }
  return SB_OK;
}

// Same with contiguous gradient outputs.
SB_API int sb200_fa_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse2,
                        float* delta, float* dkv_partial, int splits, void* dq, void* dk, void* dv,
                        const int* doc_start, const int* doc_end, int T,
                        int Hq, int Hkv, int D, long ldq_tok, int ldq_head, long ldk_tok, int ldk_head, long ldv_tok,
                        int ldv_head, int causal, int window, float scale, float dropout_p, const long long* rng,
                        unsigned int call, int head0, int dtype, int* status, cudaStream_t stream) {
  return sb200_fa_bwd_strided(q, k, v, o, d_o, lse2, delta, dkv_partial, splits, dq, dk, dv, doc_start, doc_end, T, Hq,
                              Hkv, D, ldq_tok, ldq_head, ldk_tok, ldk_head, ldv_tok, ldv_head, (long)Hq * D, D,
                              (long)Hkv * D, D, (long)Hkv * D, D, causal, window, scale, dropout_p, rng, call, head0,
                              dtype, status, stream);
}
