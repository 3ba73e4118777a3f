// Attention of a few query tokens against many cached keys (incremental decoding with a KV cache, and any other
// call whose queries and keys have different lengths; src/scaling/core/nn/attention/attention.py:216-271 hands these
// to flash-attn with separate cumulative lengths for queries and keys).
//
// The work is a stream over K and V with a handful of FLOPs per byte, so it runs on plain loads and FMAs, not on the
// tensor cores: one CTA of four warps per (query token, query head); every lane (at head size 128: every pair of
// lanes, half of the dimensions each) walks its own keys with a private running maximum, sum and output accumulator,
// so the loop needs no block-wide synchronisation; the private states are merged once at the end (maximum, rescale,
// sum in a fixed order).
// Forward only: the cache exists in inference.

#include "common.cuh"

namespace {

constexpr int DEC_WARPS = 4;
constexpr int DEC_THREADS = DEC_WARPS * 32;

template <typename T, int D>
__global__ void __launch_bounds__(DEC_THREADS)
    fa_decode_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ out,
                     const int* __restrict__ key_lo, const int* __restrict__ key_hi, int group, long q_ld_tok,
                     long q_ld_head, long k_ld_tok, long k_ld_head, long v_ld_tok, long v_ld_head, long o_ld_tok,
                     long o_ld_head, float scale_log2) {
  constexpr int V = 8;                    // 16-bit elements per 16-byte load
  constexpr int LPK = D / 64;             // lanes that share a key: each owns 64 of the D dimensions
  constexpr int DL = D / LPK;             // dimensions per lane (the accumulator stays in registers)
  constexpr int CH = DL / V;              // loads per row and lane
  constexpr int KPI = DEC_THREADS / LPK;  // keys per iteration of the CTA
  __shared__ float q_s[D];
  __shared__ float red_m[DEC_WARPS], red_l[DEC_WARPS];
  __shared__ float red_acc[DEC_WARPS][D];
  const int t = blockIdx.x, h = blockIdx.y, hk = h / group;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % LPK, slot = threadIdx.x / LPK;
  for (int i = threadIdx.x; i < D; i += DEC_THREADS) q_s[i] = sb::to_f(q[t * q_ld_tok + h * q_ld_head + i]) * scale_log2;
  __syncthreads();
  const int lo = key_lo[t], hi = key_hi[t];
  float m = -INFINITY, l = 0.f;
  float acc[DL];
#pragma unroll
  for (int i = 0; i < DL; ++i) acc[i] = 0.f;
  for (int base = lo; base < hi; base += KPI) {  // the trip count is the same for every thread of the CTA
    const int j = base + slot;
    const bool valid = j < hi;
    float s = 0.f;
    if (valid) {
      const T* kr = k + j * k_ld_tok + hk * k_ld_head + sub * DL;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const sb::Vec16<T> kv = sb::ld16(kr + c * V);
#pragma unroll
        for (int i = 0; i < V; ++i) s = fmaf(q_s[sub * DL + c * V + i], sb::to_f(kv.e[i]), s);
      }
    }
    if (LPK == 2) s += __shfl_xor_sync(0xffffffffu, s, 1);  // the two halves of the dot product
    if (valid) {
      const float m_new = fmaxf(m, s);
      const float corr = exp2f(m - m_new);  // 0 for the first key (m = -inf)
      const float p = exp2f(s - m_new);
      l = l * corr + p;
      m = m_new;
      const T* vr = v + j * v_ld_tok + hk * v_ld_head + sub * DL;
#pragma unroll
      for (int c = 0; c < CH; ++c) {
        const sb::Vec16<T> vv = sb::ld16(vr + c * V);
#pragma unroll
        for (int i = 0; i < V; ++i) acc[c * V + i] = fmaf(acc[c * V + i], corr, p * sb::to_f(vv.e[i]));
      }
    }
  }
  // merge: the maximum over all lanes, every state rescaled to it, then sums in a fixed order
  float mw = m;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, o));
  if (lane == 0) red_m[warp] = mw;
  __syncthreads();
  float mall = red_m[0];
#pragma unroll
  for (int w = 1; w < DEC_WARPS; ++w) mall = fmaxf(mall, red_m[w]);
  const float f = m == -INFINITY ? 0.f : exp2f(m - mall);  // a lane without keys contributes nothing
  float lw = sub == 0 ? l * f : 0.f;                        // lanes that share a key hold the same sum
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lw += __shfl_xor_sync(0xffffffffu, lw, o);
  if (lane == 0) red_l[warp] = lw;
#pragma unroll
  for (int i = 0; i < DL; ++i) {
    float a = acc[i] * f;
#pragma unroll
    for (int o = 16; o >= LPK; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);  // over the lanes with this `sub`
    if (lane < LPK) red_acc[warp][lane * DL + i] = a;
  }
  __syncthreads();
  float lall = 0.f;
#pragma unroll
  for (int w = 0; w < DEC_WARPS; ++w) lall += red_l[w];
  const float inv = lall > 0.f ? 1.f / lall : 0.f;  // no visible key: zeros, like the dense expression
  for (int i = threadIdx.x; i < D; i += DEC_THREADS) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) a += red_acc[w][i];
    out[t * o_ld_tok + h * o_ld_head + i] = sb::from_f<T>(a * inv);
  }
}

}  // namespace

// out[Tq, Hq, D] = softmax(scale * q k^T restricted to keys [key_lo[t], key_hi[t])) v for every query token t.
//   q / out: [Tq, Hq, D], k / v: [Tk, Hkv, D], bf16 or fp16, innermost dimension contiguous; k and v rows 16-byte
//   aligned (strides multiples of 8 elements); Hq a multiple of Hkv; D 64 or 128; key_lo / key_hi: int32 [Tq] with
//   0 <= lo, hi <= Tk (hi <= lo: the token sees no key and its output is zero).
SB_API int sb200_fa_decode(const void* q, const void* k, const void* v, void* out, const int* key_lo, const int* key_hi,
                           int Tq, int Hq, int Hkv, int D, long q_ld_tok, long q_ld_head, long k_ld_tok, long k_ld_head,
                           long v_ld_tok, long v_ld_head, long o_ld_tok, long o_ld_head, float scale, int dtype,
                           cudaStream_t stream) {
  if (Tq <= 0 || Hq <= 0) return SB_OK;
  if (Hkv <= 0 || Hq % Hkv || (D != 64 && D != 128)) return SB_ERR_BAD_ARG;
  if ((k_ld_tok % 8) || (k_ld_head % 8) || (v_ld_tok % 8) || (v_ld_head % 8)) return SB_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) return SB_ERR_BAD_ARG;
  if (dtype != SB_DT_BF16 && dtype != SB_DT_F16) return SB_ERR_BAD_ARG;
  const float scale_log2 = scale * 1.4426950408889634f;
  const dim3 grid(Tq, Hq);
#define SB_DECODE(T_, D_)                                                                                            \
  fa_decode_kernel<T_, D_><<<grid, DEC_THREADS, 0, stream>>>((const T_*)q, (const T_*)k, (const T_*)v, (T_*)out,      \
                                                              key_lo, key_hi, Hq / Hkv, q_ld_tok, q_ld_head, k_ld_tok, \
                                                              k_ld_head, v_ld_tok, v_ld_head, o_ld_tok, o_ld_head,     \
                                                              scale_log2)
  if (dtype == SB_DT_BF16) {
    if (D == 64) SB_DECODE(__nv_bfloat16, 64);
    else SB_DECODE(__nv_bfloat16, 128);
  } else {
    if (D == 64) SB_DECODE(__half, 64);
    else SB_DECODE(__half, 128);
  }
#undef SB_DECODE
  SB_CHECK_LAUNCH();
  return SB_OK;
}
