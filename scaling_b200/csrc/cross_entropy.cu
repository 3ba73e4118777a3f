// Vocab-parallel cross-entropy for sm_100a.
//
// Two kernels so that the tensor-parallel form needs only a tiny all-reduce in between:
//   1. ce_stats: per token, over this rank's vocab shard: max logit, sum exp(x - max),
//      the target's logit when the target id falls into the shard, and (value, index) of
//      the arg-max (for the accuracy metric).
//   2. ce_finalize: given the *global* max / sum / target logit, writes the loss per
//      token and overwrites (or writes) d logits = (softmax - onehot) * coef[token].
// With one rank the two run back to back.  The full-vocab logits are never gathered
// (the reference gathers them and calls F.cross_entropy on fp32 copies:
// src/scaling/transformer/model/losses/cross_entropy.py:24-30,73-86).
#include "common.cuh"

namespace {

constexpr int CE_THREADS = 512;

template <typename T>
__global__ void __launch_bounds__(CE_THREADS)
    ce_stats_kernel(const T* __restrict__ logits, const long* __restrict__ targets, float* __restrict__ row_max,
                    float* __restrict__ row_sum, float* __restrict__ tgt_logit, float* __restrict__ amax_val,
                    long* __restrict__ amax_idx, long N, int V, long ld, long vocab_start) {
  __shared__ float red[33];
  __shared__ float s_best[CE_THREADS / 32];
  __shared__ int s_besti[CE_THREADS / 32];
  long r = blockIdx.x;
  if (r >= N) return;
  const T* x = logits + r * ld;
  constexpr int VEC = sb::Vec16<T>::N;
  float mx = -INFINITY;
  int mi = 0;
  const bool vec = (V % VEC == 0) && (ld % VEC == 0);
  if (vec) {
    for (int c = threadIdx.x * VEC; c < V; c += CE_THREADS * VEC) {
      auto v = sb::ld16(x + c);
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        float f = sb::to_f(v.e[k]);
        if (f > mx) { mx = f; mi = c + k; }
      }
    }
  } else {
    for (int c = threadIdx.x; c < V; c += CE_THREADS) {
      float f = sb::to_f(x[c]);
      if (f > mx) { mx = f; mi = c; }
    }
  }
  // arg-max across the block (lowest index wins ties, like torch.argmax on CPU)
  int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float om = __shfl_xor_sync(0xffffffffu, mx, o);
    int oi = __shfl_xor_sync(0xffffffffu, mi, o);
    if (om > mx || (om == mx && oi < mi)) { mx = om; mi = oi; }
  }
  if (lane == 0) { s_best[w] = mx; s_besti[w] = mi; }
  __syncthreads();
  if (w == 0) {
    float bm = lane < CE_THREADS / 32 ? s_best[lane] : -INFINITY;
    int bi = lane < CE_THREADS / 32 ? s_besti[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float om = __shfl_xor_sync(0xffffffffu, bm, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (om > bm || (om == bm && oi < bi)) { bm = om; bi = oi; }
    }
    if (lane == 0) { s_best[0] = bm; s_besti[0] = bi; }
  }
  __syncthreads();
  float gmax = s_best[0];
  int gidx = s_besti[0];
  float s = 0.f;
  if (vec) {
    for (int c = threadIdx.x * VEC; c < V; c += CE_THREADS * VEC) {
      auto v = sb::ld16(x + c);
#pragma unroll
      for (int k = 0; k < VEC; ++k) s += __expf(sb::to_f(v.e[k]) - gmax);
    }
  } else {
    for (int c = threadIdx.x; c < V; c += CE_THREADS) s += __expf(sb::to_f(x[c]) - gmax);
  }
  s = sb::block_sum(s, red);
  if (threadIdx.x == 0) {
    row_max[r] = gmax;
    row_sum[r] = s;
    long t = targets[r] - vocab_start;
    tgt_logit[r] = (t >= 0 && t < V) ? sb::to_f(x[t]) : 0.f;
    if (amax_val) {
      amax_val[r] = gmax;
      amax_idx[r] = vocab_start + gidx;
    }
  }
}

// loss[r] = log(gsum) + gmax - tgt ; dlogits[r, c] = (exp(x - gmax) / gsum - [c == tgt]) * coef[r] * scale_dev[0]
template <typename T>
__global__ void __launch_bounds__(CE_THREADS)
    ce_finalize_kernel(const T* __restrict__ logits, const long* __restrict__ targets, const float* __restrict__ gmax,
                       const float* __restrict__ gsum, const float* __restrict__ gtgt, const float* __restrict__ coef,
                       float* __restrict__ loss, T* __restrict__ dlogits, long N, int V, long ld, long ldd,
                       long vocab_start, const float* __restrict__ scale_dev) {
  long r = blockIdx.x;
  if (r >= N) return;
  const float m = gmax[r], s = gsum[r];
  if (threadIdx.x == 0 && loss) loss[r] = logf(s) + m - gtgt[r];
  if (!dlogits) return;
  const T* x = logits + r * ld;
  T* d = dlogits + r * ldd;
  const float inv = 1.f / s;
  // scale_dev: the upstream gradient of the loss (a device scalar), applied here instead of in a pass of its own
  const float cf = (coef ? coef[r] : 1.f) * (scale_dev ? *scale_dev : 1.f);
  const long t = targets[r] - vocab_start;
  constexpr int VEC = sb::Vec16<T>::N;
  if ((V % VEC == 0) && (ld % VEC == 0) && (ldd % VEC == 0)) {
    for (int c = threadIdx.x * VEC; c < V; c += CE_THREADS * VEC) {
      auto v = sb::ld16(x + c);
      sb::Vec16<T> o;
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        float p = __expf(sb::to_f(v.e[k]) - m) * inv;
        if (c + k == t) p -= 1.f;
        o.e[k] = sb::from_f<T>(p * cf);
      }
      sb::st16(d + c, o);
    }
  } else {
    for (int c = threadIdx.x; c < V; c += CE_THREADS) {
      float p = __expf(sb::to_f(x[c]) - m) * inv;
      if (c == t) p -= 1.f;
      d[c] = sb::from_f<T>(p * cf);
    }
  }
}

// y[i] = x[i] * (*scale_dev) * scale  (used to apply the upstream gradient to stored d logits)
template <typename T>
__global__ void scale_by_dev_kernel(T* __restrict__ x, const float* __restrict__ scale_dev, float scale, long n) {
  float sc = scale * (scale_dev ? *scale_dev : 1.f);
  constexpr int V = sb::Vec16<T>::N;
  long nv = n / V;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
    auto v = sb::ld16(x + i * V);
#pragma unroll
    for (int k = 0; k < V; ++k) v.e[k] = sb::from_f<T>(sb::to_f(v.e[k]) * sc);
    sb::st16(x + i * V, v);
  }
  for (long i = nv * V + blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    x[i] = sb::from_f<T>(sb::to_f(x[i]) * sc);
}

}  // namespace

SB_API int sb200_ce_stats(const void* logits, const long* targets, float* row_max, float* row_sum, float* tgt_logit,
                          float* amax_val, long* amax_idx, long N, int V, long ld, long vocab_start, int dtype,
                          cudaStream_t stream) {
  if (N <= 0 || V <= 0) return SB_OK;
  SB_DISPATCH_DTYPE(dtype, T, {
    ce_stats_kernel<T><<<(unsigned)N, CE_THREADS, 0, stream>>>((const T*)logits, targets, row_max, row_sum, tgt_logit,
                                                                amax_val, amax_idx, N, V, ld, vocab_start);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
SB_API int sb200_ce_finalize(const void* logits, const long* targets, const float* gmax, const float* gsum,
                             const float* gtgt, const float* coef, float* loss, void* dlogits, long N, int V, long ld,
                             long ldd, long vocab_start, const float* scale_dev, int dtype, cudaStream_t stream) {
  if (N <= 0 || V <= 0) return SB_OK;
  SB_DISPATCH_DTYPE(dtype, T, {
    ce_finalize_kernel<T><<<(unsigned)N, CE_THREADS, 0, stream>>>((const T*)logits, targets, gmax, gsum, gtgt, coef,
                                                                   loss, (T*)dlogits, N, V, ld, ldd, vocab_start,
                                                                   scale_dev);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
SB_API int sb200_scale_by_dev(void* x, const float* scale_dev, float scale, long n, int dtype, cudaStream_t stream) {
  if (n <= 0) return SB_OK;
  SB_DISPATCH_DTYPE(dtype, T, {
    long b = (n / sb::Vec16<T>::N + 256) / 256;
    if (b > 148 * 16) b = 148 * 16;
    scale_by_dev_kernel<T><<<(int)b, 256, 0, stream>>>((T*)x, scale_dev, scale, n);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
