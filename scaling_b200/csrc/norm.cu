// RMSNorm / LayerNorm forward and backward for sm_100a.
//
// One CTA per row in the forward pass (16-byte vector loads, fp32 statistics);
// the backward pass is persistent over rows so that each CTA keeps its share of
// the weight/bias gradient in registers and writes one partial row, which a
// second kernel reduces in a fixed order (deterministic, no atomics).
//
// Behaviour covered: LayerNorm = F.layer_norm with weight (+ optional bias),
// RMSNorm = x * rsqrt(mean(x^2) + eps) * weight (reference:
// src/scaling/core/nn/norm/layernorm.py:84, src/scaling/core/nn/norm/rms_norm.py:47-50).
// Statistics are always accumulated in fp32 (the reference RMSNorm computes in
// the input dtype; fp32 is a strict accuracy improvement).
#include "common.cuh"

namespace {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_ITERS = 8;  // H <= 256 * 8 * 8 = 16384 for 2-byte types

// Forward for rows of at most 32 * V * NV elements: one warp per row, the row stays in registers between the
// statistics and the normalisation (one read of x, one write of y), eight rows in flight per CTA.
template <typename T, bool RMS, int NV>
__global__ void __launch_bounds__(NORM_THREADS)
    norm_fwd_warp_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b, T* __restrict__ y,
                         float* __restrict__ mean_out, float* __restrict__ rstd_out, int M, int H, float eps) {
  constexpr int V = sb::Vec16<T>::N;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_warps = gridDim.x * (NORM_THREADS / 32);
  sb::Vec16<T> wv[NV], bv[NV];
#pragma unroll
  for (int it = 0; it < NV; ++it) {
    const int c = (it * 32 + lane) * V;
    wv[it].u = make_uint4(0, 0, 0, 0);
    bv[it].u = make_uint4(0, 0, 0, 0);
    if (c < H) {
      wv[it] = sb::ld16(w + c);
      if (!RMS && b) bv[it] = sb::ld16(b + c);
    }
  }
  const float inv_h = 1.f / H;
  for (int row = blockIdx.x * (NORM_THREADS / 32) + warp; row < M; row += total_warps) {
    const T* xr = x + (size_t)row * H;
    sb::Vec16<T> xv[NV];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int it = 0; it < NV; ++it) {
      const int c = (it * 32 + lane) * V;
      xv[it].u = make_uint4(0, 0, 0, 0);
      if (c < H) xv[it] = sb::ld16(xr + c);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float f = sb::to_f(xv[it].e[i]);
        s += f;
        ss += f * f;
      }
    }
    float mean = 0.f, rstd;
    if (RMS) {
      rstd = rsqrtf(sb::warp_sum(ss) * inv_h + eps);
    } else {
      mean = sb::warp_sum(s) * inv_h;
      float var = 0.f;  // second pass over the registers: numerically safer than E[x^2] - E[x]^2
#pragma unroll
      for (int it = 0; it < NV; ++it) {
        const int c = (it * 32 + lane) * V;
        if (c < H) {
#pragma unroll
          for (int i = 0; i < V; ++i) {
            const float d = sb::to_f(xv[it].e[i]) - mean;
            var += d * d;
          }
        }
      }
      rstd = rsqrtf(sb::warp_sum(var) * inv_h + eps);
    }
    if (lane == 0) {
      if (!RMS && mean_out) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
    T* yr = y + (size_t)row * H;
#pragma unroll
    for (int it = 0; it < NV; ++it) {
      const int c = (it * 32 + lane) * V;
      if (c < H) {
        sb::Vec16<T> o;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float v = (sb::to_f(xv[it].e[i]) - mean) * rstd * sb::to_f(wv[it].e[i]);
          if (!RMS && b) v += sb::to_f(bv[it].e[i]);
          o.e[i] = sb::from_f<T>(v);
        }
        sb::st16(yr + c, o);
      }
    }
  }
}

template <typename T, bool RMS>
__global__ void __launch_bounds__(NORM_THREADS) norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                                const T* __restrict__ b, T* __restrict__ y,
                                                                float* __restrict__ mean_out,
                                                                float* __restrict__ rstd_out, int M, int H, float eps) {
  __shared__ float red[33];
  constexpr int V = sb::Vec16<T>::N;
  const int row = blockIdx.x;
  if (row >= M) return;
  const T* xr = x + (size_t)row * H;
  T* yr = y + (size_t)row * H;
  const bool vec = (H % V) == 0;
  float s = 0.f, ss = 0.f;
  if (vec) {
    for (int c = threadIdx.x * V; c < H; c += NORM_THREADS * V) {
      auto v = sb::ld16(xr + c);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float f = sb::to_f(v.e[i]);
        s += f;
        ss += f * f;
      }
    }
  } else {
    for (int c = threadIdx.x; c < H; c += NORM_THREADS) {
      float f = sb::to_f(xr[c]);
      s += f;
      ss += f * f;
    }
  }
  float mean = 0.f, rstd;
  if (RMS) {
    ss = sb::block_sum(ss, red);
    rstd = rsqrtf(ss / H + eps);
  } else {
    s = sb::block_sum(s, red);
    mean = s / H;
    // second pass for the variance (numerically safer than E[x^2]-E[x]^2)
    float var = 0.f;
    if (vec) {
      for (int c = threadIdx.x * V; c < H; c += NORM_THREADS * V) {
        auto v = sb::ld16(xr + c);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float d = sb::to_f(v.e[i]) - mean;
          var += d * d;
        }
      }
    } else {
      for (int c = threadIdx.x; c < H; c += NORM_THREADS) {
        float d = sb::to_f(xr[c]) - mean;
        var += d * d;
      }
    }
    var = sb::block_sum(var, red);
    rstd = rsqrtf(var / H + eps);
  }
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mean;
    rstd_out[row] = rstd;
  }
  if (vec) {
    for (int c = threadIdx.x * V; c < H; c += NORM_THREADS * V) {
      auto v = sb::ld16(xr + c);
      auto wv = sb::ld16(w + c);
      sb::Vec16<T> o;
      if (b) {
        auto bv = sb::ld16(b + c);
#pragma unroll
        for (int i = 0; i < V; ++i)
          o.e[i] = sb::from_f<T>((sb::to_f(v.e[i]) - mean) * rstd * sb::to_f(wv.e[i]) + sb::to_f(bv.e[i]));
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) o.e[i] = sb::from_f<T>((sb::to_f(v.e[i]) - mean) * rstd * sb::to_f(wv.e[i]));
      }
      sb::st16(yr + c, o);
    }
  } else {
    for (int c = threadIdx.x; c < H; c += NORM_THREADS) {
      float o = (sb::to_f(xr[c]) - mean) * rstd * sb::to_f(w[c]);
      if (b) o += sb::to_f(b[c]);
      yr[c] = sb::from_f<T>(o);
    }
  }
}

// Backward.  Requires H % V == 0 and H <= NORM_THREADS * V * NORM_MAX_ITERS.
template <typename T, bool RMS>
__global__ void __launch_bounds__(NORM_THREADS)
    norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                    const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ dx,
                    float* __restrict__ dw_partial, float* __restrict__ db_partial, int M, int H) {
  __shared__ float red[33];
  constexpr int V = sb::Vec16<T>::N;
  float dw_acc[NORM_MAX_ITERS][V];
  float db_acc[NORM_MAX_ITERS][V];
#pragma unroll
  for (int it = 0; it < NORM_MAX_ITERS; ++it)
#pragma unroll
    for (int i = 0; i < V; ++i) {
      dw_acc[it][i] = 0.f;
      db_acc[it][i] = 0.f;
    }
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const T* xr = x + (size_t)row * H;
    const T* dyr = dy + (size_t)row * H;
    T* dxr = dx + (size_t)row * H;
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    float sum_g = 0.f, sum_gx = 0.f;
#pragma unroll
    for (int it = 0; it < NORM_MAX_ITERS; ++it) {
      int c = (it * NORM_THREADS + threadIdx.x) * V;
      if (c < H) {
        auto xv = sb::ld16(xr + c);
        auto dv = sb::ld16(dyr + c);
        auto wv = sb::ld16(w + c);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float xh = (sb::to_f(xv.e[i]) - mean) * rstd;
          float d = sb::to_f(dv.e[i]);
          float g = d * sb::to_f(wv.e[i]);
          sum_g += g;
          sum_gx += g * xh;
          dw_acc[it][i] += d * xh;
          if (!RMS) db_acc[it][i] += d;
        }
      }
    }
    sum_gx = sb::block_sum(sum_gx, red) / H;
    if (!RMS) sum_g = sb::block_sum(sum_g, red) / H; else sum_g = 0.f;
#pragma unroll
    for (int it = 0; it < NORM_MAX_ITERS; ++it) {
      int c = (it * NORM_THREADS + threadIdx.x) * V;
      if (c < H) {
        auto xv = sb::ld16(xr + c);
        auto dv = sb::ld16(dyr + c);
        auto wv = sb::ld16(w + c);
        sb::Vec16<T> o;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float xh = (sb::to_f(xv.e[i]) - mean) * rstd;
          float g = sb::to_f(dv.e[i]) * sb::to_f(wv.e[i]);
          o.e[i] = sb::from_f<T>(rstd * (g - sum_g - xh * sum_gx));
        }
        sb::st16(dxr + c, o);
      }
    }
  }
  float* dwp = dw_partial + (size_t)blockIdx.x * H;
  float* dbp = db_partial ? db_partial + (size_t)blockIdx.x * H : nullptr;
#pragma unroll
  for (int it = 0; it < NORM_MAX_ITERS; ++it) {
    int c = (it * NORM_THREADS + threadIdx.x) * V;
    if (c < H) {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        dwp[c + i] = dw_acc[it][i];
        if (!RMS && dbp) dbp[c + i] = db_acc[it][i];
      }
    }
  }
}

// Backward with one warp per row (H <= 32 * V * NV): no block-wide synchronisation, row statistics by
// warp shuffles, every warp keeps its share of dW / dB in registers and writes one partial row.
template <typename T, bool RMS, int NV>
__global__ void __launch_bounds__(NORM_THREADS, 2)
    norm_bwd_warp_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                         const float* __restrict__ mean_in, const float* __restrict__ rstd_in, T* __restrict__ dx,
                         float* __restrict__ dw_partial, float* __restrict__ db_partial, int M, int H) {
  constexpr int V = sb::Vec16<T>::N;
  constexpr int WARPS = NORM_THREADS / 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gw = blockIdx.x * WARPS + warp;
  const int total_warps = gridDim.x * WARPS;
  float dw_acc[NV][V], db_acc[NV][V];
  sb::Vec16<T> wv[NV];  // packed: the row data of an iteration stays in its load format to save registers
#pragma unroll
  for (int it = 0; it < NV; ++it) {
    const int c = (it * 32 + lane) * V;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      dw_acc[it][i] = 0.f;
      db_acc[it][i] = 0.f;
    }
    wv[it].u = make_uint4(0, 0, 0, 0);
    if (c < H) wv[it] = sb::ld16(w + c);
  }
  const float inv_h = 1.f / H;
  for (int row = gw; row < M; row += total_warps) {
    const T* xr = x + (size_t)row * H;
    const T* dyr = dy + (size_t)row * H;
    T* dxr = dx + (size_t)row * H;
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    sb::Vec16<T> xv[NV], dv[NV];
#pragma unroll
    for (int it = 0; it < NV; ++it) {
      const int c = (it * 32 + lane) * V;
      xv[it].u = make_uint4(0, 0, 0, 0);
      dv[it].u = make_uint4(0, 0, 0, 0);
      if (c < H) {
        xv[it] = sb::ld16(xr + c);
        dv[it] = sb::ld16(dyr + c);
      }
    }
    float sum_g = 0.f, sum_gx = 0.f;
#pragma unroll
    for (int it = 0; it < NV; ++it) {
      const int c = (it * 32 + lane) * V;
      if (c < H) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float d = sb::to_f(dv[it].e[i]);
          const float xh = (sb::to_f(xv[it].e[i]) - mean) * rstd;
          const float g = d * sb::to_f(wv[it].e[i]);
          sum_g += g;
          sum_gx += g * xh;
          dw_acc[it][i] += d * xh;
          if (!RMS) db_acc[it][i] += d;
        }
      }
    }
    sum_gx = sb::warp_sum(sum_gx) * inv_h;
    sum_g = RMS ? 0.f : sb::warp_sum(sum_g) * inv_h;
#pragma unroll
    for (int it = 0; it < NV; ++it) {
      const int c = (it * 32 + lane) * V;
      if (c < H) {
        sb::Vec16<T> o;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float xh = (sb::to_f(xv[it].e[i]) - mean) * rstd;
          const float g = sb::to_f(dv[it].e[i]) * sb::to_f(wv[it].e[i]);
          o.e[i] = sb::from_f<T>(rstd * (g - sum_g - xh * sum_gx));
        }
        sb::st16(dxr + c, o);
      }
    }
  }
  // one partial row per CTA: the 8 warps' accumulators are summed in a fixed order through shared memory,
  // one chunk of 32*V columns at a time
  __shared__ float red[WARPS][32 * V];
  float* dwp = dw_partial + (size_t)blockIdx.x * H;
  float* dbp = db_partial ? db_partial + (size_t)blockIdx.x * H : nullptr;
#pragma unroll
  for (int it = 0; it < NV; ++it) {
    const int c0 = it * 32 * V;
#pragma unroll
    for (int pass = 0; pass < (RMS ? 1 : 2); ++pass) {
      if (pass == 1 && !dbp) break;
      __syncthreads();
#pragma unroll
      for (int i = 0; i < V; ++i) red[warp][lane * V + i] = pass == 0 ? dw_acc[it][i] : db_acc[it][i];
      __syncthreads();
      for (int t = threadIdx.x; t < 32 * V; t += NORM_THREADS) {
        if (c0 + t < H) {
          float s = 0.f;
#pragma unroll
          for (int wi = 0; wi < WARPS; ++wi) s += red[wi][t];
          (pass == 0 ? dwp : dbp)[c0 + t] = s;
        }
      }
    }
  }
}

// out[c] (+)= sum_p partial[p][c], fixed order over p.
template <typename T>
__global__ void reduce_partials_kernel(const float* __restrict__ partial, T* __restrict__ out, int P, int H,
                                       int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += partial[(size_t)p * H + c];
  if (accumulate) s += sb::to_f(out[c]);
  out[c] = sb::from_f<T>(s);
}

// Same result layout, parallel over the partial rows: a CTA owns 32 columns, warp w sums rows w, w+32, ...
// and the 32 warp sums are added in a fixed order.  blockIdx.y selects (partial0, out0) or (partial1, out1).
template <typename T>
__global__ void __launch_bounds__(1024)
    reduce_partials_wide_kernel(const float* __restrict__ partial0, T* __restrict__ out0,
                                const float* __restrict__ partial1, T* __restrict__ out1, int P, int H,
                                int accumulate) {
  __shared__ float red[32][33];
  const float* partial = blockIdx.y == 0 ? partial0 : partial1;
  T* out = blockIdx.y == 0 ? out0 : out1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * 32 + lane;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (c < H) {
    int p = warp;
    for (; p + 96 < P; p += 128) {
      s0 += partial[(size_t)p * H + c];
      s1 += partial[(size_t)(p + 32) * H + c];
      s2 += partial[(size_t)(p + 64) * H + c];
      s3 += partial[(size_t)(p + 96) * H + c];
    }
    for (; p < P; p += 32) s0 += partial[(size_t)p * H + c];
  }
  red[warp][lane] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (warp == 0 && c < H) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 32; ++w) s += red[w][lane];
    if (accumulate) s += sb::to_f(out[c]);
    out[c] = sb::from_f<T>(s);
  }
}

}  // namespace

namespace {

template <typename T, int NV>
void launch_norm_fwd_warp(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int M, int H,
                          float eps, int rms, cudaStream_t stream) {
  int ctas = (M + 7) / 8;
  if (ctas > 148 * 8) ctas = 148 * 8;
  if (rms)
    norm_fwd_warp_kernel<T, true, NV><<<ctas, NORM_THREADS, 0, stream>>>((const T*)x, (const T*)w, nullptr, (T*)y, nullptr,
                                                                         rstd, M, H, eps);
  else
    norm_fwd_warp_kernel<T, false, NV><<<ctas, NORM_THREADS, 0, stream>>>((const T*)x, (const T*)w, (const T*)b, (T*)y,
                                                                          mean, rstd, M, H, eps);
}

template <typename T>
void norm_fwd_dispatch(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int M, int H,
                       float eps, int rms, cudaStream_t stream) {
  constexpr int V = sb::Vec16<T>::N;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                         reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
  if (H % V == 0 && H <= 32 * V * 4 && aligned) {
    const int nv = (H + 32 * V - 1) / (32 * V);
    if (nv <= 1) launch_norm_fwd_warp<T, 1>(x, w, b, y, mean, rstd, M, H, eps, rms, stream);
    else if (nv == 2) launch_norm_fwd_warp<T, 2>(x, w, b, y, mean, rstd, M, H, eps, rms, stream);
    else if (nv == 3) launch_norm_fwd_warp<T, 3>(x, w, b, y, mean, rstd, M, H, eps, rms, stream);
    else launch_norm_fwd_warp<T, 4>(x, w, b, y, mean, rstd, M, H, eps, rms, stream);
  } else if (rms) {
    norm_fwd_kernel<T, true><<<M, NORM_THREADS, 0, stream>>>((const T*)x, (const T*)w, nullptr, (T*)y, nullptr, rstd, M,
                                                              H, eps);
  } else {
    norm_fwd_kernel<T, false><<<M, NORM_THREADS, 0, stream>>>((const T*)x, (const T*)w, (const T*)b, (T*)y, mean, rstd,
                                                               M, H, eps);
  }
}

}  // namespace

SB_API int sb200_norm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int M, int H,
                          float eps, int rms, int dtype, cudaStream_t stream) {
  if (M <= 0 || H <= 0) return SB_OK;
  SB_DISPATCH_DTYPE(dtype, T, { norm_fwd_dispatch<T>(x, w, b, y, mean, rstd, M, H, eps, rms, stream); });
  SB_CHECK_LAUNCH();
  return SB_OK;
}

// Number of partial rows the backward pass writes for a problem of M rows; the caller
// provides dw_partial (and db_partial for LayerNorm with bias) of [rows, H] floats.
SB_API int sb200_norm_bwd_partial_rows(int M, int sm_count) {
  int p = sm_count * 2;
  if (p > M) p = M;
  if (p < 1) p = 1;
  return p;
}

// Partial rows (one per CTA) for a problem of M rows of width H: the warp-per-row kernel used for narrow rows
// keeps 8 rows in flight per CTA and is launched with more CTAs than the block-per-row kernel.
SB_API int sb200_norm_bwd_partial_rows_h(int M, int H, int elem_size, int sm_count) {
  const int V = 16 / (elem_size > 0 ? elem_size : 2);
  if (H % V == 0 && H <= 32 * V * 4) {
    int ctas = (M + 15) / 16;
    if (ctas > sm_count * 2) ctas = sm_count * 2;
    if (ctas < 1) ctas = 1;
    return ctas;
  }
  return sb200_norm_bwd_partial_rows(M, sm_count);
}

namespace {

template <typename T, bool RMS, int NV>
void launch_norm_bwd_warp(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                          float* dw_partial, float* db_partial, int M, int H, int partial_rows, cudaStream_t stream) {
  norm_bwd_warp_kernel<T, RMS, NV><<<partial_rows, NORM_THREADS, 0, stream>>>(
      (const T*)dy, (const T*)x, (const T*)w, RMS ? nullptr : mean, rstd, (T*)dx, dw_partial,
      RMS ? nullptr : db_partial, M, H);
}

template <typename T, bool RMS>
int norm_bwd_dispatch(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                      float* dw_partial, float* db_partial, void* dw, void* db, int M, int H, int accumulate,
                      int partial_rows, cudaStream_t stream) {
  constexpr int V = sb::Vec16<T>::N;
  if (H % V != 0 || H > NORM_THREADS * V * NORM_MAX_ITERS) return SB_ERR_BAD_ARG;
  const bool warp_rows = H <= 32 * V * 4;
  const int nv = (H + 32 * V - 1) / (32 * V);
  if (warp_rows && nv <= 1)
    launch_norm_bwd_warp<T, RMS, 1>(dy, x, w, mean, rstd, dx, dw_partial, db_partial, M, H, partial_rows, stream);
  else if (warp_rows && nv <= 2)
    launch_norm_bwd_warp<T, RMS, 2>(dy, x, w, mean, rstd, dx, dw_partial, db_partial, M, H, partial_rows, stream);
  else if (warp_rows && nv <= 3)
    launch_norm_bwd_warp<T, RMS, 3>(dy, x, w, mean, rstd, dx, dw_partial, db_partial, M, H, partial_rows, stream);
  else if (warp_rows && nv <= 4)
    launch_norm_bwd_warp<T, RMS, 4>(dy, x, w, mean, rstd, dx, dw_partial, db_partial, M, H, partial_rows, stream);
  else
    norm_bwd_kernel<T, RMS><<<partial_rows, NORM_THREADS, 0, stream>>>(
        (const T*)dy, (const T*)x, (const T*)w, RMS ? nullptr : mean, rstd, (T*)dx, dw_partial,
        RMS ? nullptr : db_partial, M, H);
  SB_CHECK_LAUNCH();
  const bool want_db = !RMS && db && db_partial;
  reduce_partials_wide_kernel<T><<<dim3((H + 31) / 32, want_db ? 2 : 1), 1024, 0, stream>>>(
      dw_partial, (T*)dw, db_partial, (T*)db, partial_rows, H, accumulate);
  SB_CHECK_LAUNCH();
  return SB_OK;
}

}  // namespace

SB_API int sb200_norm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                          float* dw_partial, float* db_partial, void* dw, void* db, int M, int H, int rms,
                          int accumulate, int partial_rows, int dtype, cudaStream_t stream) {
  if (M <= 0 || H <= 0) return SB_OK;
  SB_DISPATCH_DTYPE(dtype, T, {
    if (rms)
      return norm_bwd_dispatch<T, true>(dy, x, w, mean, rstd, dx, dw_partial, db_partial, dw, db, M, H, accumulate,
                                        partial_rows, stream);
    return norm_bwd_dispatch<T, false>(dy, x, w, mean, rstd, dx, dw_partial, db_partial, dw, db, M, H, accumulate,
                                       partial_rows, stream);
  });
  return SB_OK;
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free variant of the backward pass (declared in sb200_noalloc.h): the partial-sum workspace
// is a static device array instead of caller memory.
#include <mutex>

#include "sb200_noalloc.h"

namespace {

constexpr int NOALLOC_MAX_DEVICES = 64;

// Workspace for the per-CTA partial sums of dW and dB.  In host code these names are only handles for
// cudaGetSymbolAddress; the kernels receive the looked-up device pointers.
static __device__ __align__(256) float g_noalloc_dw_partial[SB200_NOALLOC_MAX_PARTIAL_ROWS * SB200_NOALLOC_MAX_H];
static __device__ __align__(256) float g_noalloc_db_partial[SB200_NOALLOC_MAX_PARTIAL_ROWS * SB200_NOALLOC_MAX_H];

struct NoallocWorkspace {
  float* dw = nullptr;
  float* db = nullptr;
  bool ready = false;
};
NoallocWorkspace g_noalloc_ws[NOALLOC_MAX_DEVICES];
std::mutex g_noalloc_mutex;

// Device addresses of the workspace on the current device, resolved once per device.
int noalloc_workspace(float** dw, float** db) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return SB_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  NoallocWorkspace& ws = g_noalloc_ws[dev];
  if (!ws.ready) {
    e = cudaGetSymbolAddress((void**)&ws.dw, g_noalloc_dw_partial);
    if (e != cudaSuccess) return (int)e;
    e = cudaGetSymbolAddress((void**)&ws.db, g_noalloc_db_partial);
    if (e != cudaSuccess) return (int)e;
    ws.ready = true;
  }
  *dw = ws.dw;
  *db = ws.db;
  return SB_OK;
}

}  // namespace

SB_API int sb200_norm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* mean, const float* rstd,
                                  void* dx, void* dw, void* db, int M, int H, int rms, int accumulate, int dtype,
                                  cudaStream_t stream) {
  if (M <= 0 || H <= 0) return SB_OK;
  if (H > SB200_NOALLOC_MAX_H) return SB_ERR_TOO_LARGE;
  // the kernels use 16-byte loads and stores on the rows and on the weight / gradient vectors: a misaligned pointer
  // would be a device fault (the context is lost), so it is refused here, before anything is launched
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) |
       reinterpret_cast<uintptr_t>(dx) | reinterpret_cast<uintptr_t>(dw) | reinterpret_cast<uintptr_t>(db)) & 15)
    return SB_ERR_BAD_ARG;
  if (!dy || !x || !w || !dx || !dw || !rstd || (!rms && !mean)) return SB_ERR_BAD_ARG;
  float* dw_partial = nullptr;
  float* db_partial = nullptr;
  int rc = noalloc_workspace(&dw_partial, &db_partial);
  if (rc != SB_OK) return rc;
  int rows = M < SB200_NOALLOC_MAX_PARTIAL_ROWS ? M : SB200_NOALLOC_MAX_PARTIAL_ROWS;
  const bool want_db = !rms && db != nullptr;
  SB_DISPATCH_DTYPE(dtype, T, {
    constexpr int V = sb::Vec16<T>::N;
    if (H % V != 0 || H > NORM_THREADS * V * NORM_MAX_ITERS) return SB_ERR_BAD_ARG;
    if (rms)
      norm_bwd_kernel<T, true><<<rows, NORM_THREADS, 0, stream>>>(
          (const T*)dy, (const T*)x, (const T*)w, nullptr, rstd, (T*)dx, dw_partial, nullptr, M, H);
    else
      norm_bwd_kernel<T, false><<<rows, NORM_THREADS, 0, stream>>>(
          (const T*)dy, (const T*)x, (const T*)w, mean, rstd, (T*)dx, dw_partial, want_db ? db_partial : nullptr, M,
          H);
    SB_CHECK_LAUNCH();
    int blocks = (H + 255) / 256;
    reduce_partials_kernel<T><<<blocks, 256, 0, stream>>>(dw_partial, (T*)dw, rows, H, accumulate);
    if (want_db) reduce_partials_kernel<T><<<blocks, 256, 0, stream>>>(db_partial, (T*)db, rows, H, accumulate);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
