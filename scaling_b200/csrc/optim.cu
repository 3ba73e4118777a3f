// Optimizer-side kernels for sm_100a: fused AdamW on a flat fp32 master shard with the
// low-precision write-out, gradient sum-of-squares with a sticky inf/nan flag, and the
// vocab-parallel embedding gather / deterministic scatter.
//
// Behaviour covered (reference files): torch.optim.AdamW over fp32 masters
// (src/scaling/core/optimizer/optimizer.py:62-66,186), per-parameter unscale + norm^2 +
// overflow test (src/scaling/core/optimizer/parameter_group.py:497-511,
// src/scaling/core/optimizer/loss_scaler.py:23-41), fp32 -> bf16 copy back
// (parameter_group.py:428-486), masked embedding lookup
// (src/scaling/core/nn/linear/vocab_parallel_embedding.py:166-189).
#include "common.cuh"

namespace {

// ------------------------------------------------------------------- AdamW
// control[0] = gradient multiplier (1/loss_scale * clip coefficient), control[1] != 0 -> skip step.
template <typename T> struct Vec4 {};  // four consecutive elements as one load / store
template <> struct Vec4<float> { using type = float4; };
template <> struct Vec4<__nv_bfloat16> { using type = uint2; };
template <> struct Vec4<__half> { using type = uint2; };

template <typename T> __device__ __forceinline__ void load4(const T* p, float* v) {
  typename Vec4<T>::type raw = *reinterpret_cast<const typename Vec4<T>::type*>(p);
  const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) v[k] = sb::to_f(e[k]);
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float* v) {
  typename Vec4<T>::type raw;
  T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
  for (int k = 0; k < 4; ++k) e[k] = sb::from_f<T>(v[k]);
  *reinterpret_cast<typename Vec4<T>::type*>(p) = raw;
}

template <typename G, typename P>
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const G* __restrict__ g, P* __restrict__ p_lp, long n, float lr, float beta1, float beta2,
                             float eps, float wd, float bc1, float bc2, const float* __restrict__ control,
                             const float* __restrict__ hyper, int vec_ok) {
  // hyper (optional, device memory): [learning rate, 1 - beta1^t, 1 - beta2^t] - lets a captured CUDA graph
  // be replayed with new values
  if (hyper) {
    lr = hyper[0];
    bc1 = hyper[1];
    bc2 = hyper[2];
  }
  float gmul = 1.f;
  if (control) {
    if (control[1] != 0.f) return;
    gmul = control[0];
  }
  const float inv_bc1 = 1.f / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  const float decay = 1.f - lr * wd;
  const float step = lr * inv_bc1;
  auto update = [&](float& pi, float& mi, float& vi, float gr) {
    gr *= gmul;
    mi = mi * beta1 + (1.f - beta1) * gr;
    vi = vi * beta2 + (1.f - beta2) * gr * gr;
    pi *= decay;
    pi -= step * mi / (sqrtf(vi) * inv_sqrt_bc2 + eps);
  };
  const long tid = blockIdx.x * (long)blockDim.x + threadIdx.x, stride = (long)gridDim.x * blockDim.x;
  long done = 0;
  if (vec_ok) {  // all pointers 16-byte aligned: four elements per thread and step
    const long n4 = n / 4;
    for (long i = tid; i < n4; i += stride) {
      float pv[4], mv[4], vv[4], gv[4];
      load4(p + i * 4, pv);
      load4(m + i * 4, mv);
      load4(v + i * 4, vv);
      load4(g + i * 4, gv);
#pragma unroll
      for (int k = 0; k < 4; ++k) update(pv[k], mv[k], vv[k], gv[k]);
      store4(p + i * 4, pv);
      store4(m + i * 4, mv);
      store4(v + i * 4, vv);
      if (p_lp) store4(p_lp + i * 4, pv);
    }
    done = n4 * 4;
  }
  for (long i = done + tid; i < n; i += stride) {
    float pi = p[i], mi = m[i], vi = v[i];
    update(pi, mi, vi, sb::to_f(g[i]));
    p[i] = pi;
    m[i] = mi;
    v[i] = vi;
    if (p_lp) p_lp[i] = sb::from_f<P>(pi);
  }
}

// ------------------------------------------- sum of squares + inf/nan flag
template <typename G>
__global__ void sumsq_partial_kernel(const G* __restrict__ g, long n, float* __restrict__ partial,
                                     int* __restrict__ flag) {
  __shared__ float red[33];
  float s = 0.f;
  bool bad = false;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    float f = sb::to_f(g[i]);
    if (!isfinite(f)) bad = true;
    s += f * f;
  }
  s = sb::block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
  if (bad && flag) *flag = 1;  // benign race: every writer stores the same value
}
// out[0] = (accumulate ? out[0] : 0) + scale * sum_p partial[p]   (single warp, fixed order)
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int P, float* __restrict__ out, float scale,
                                   int accumulate) {
  float s = 0.f;
  for (int p = threadIdx.x; p < P; p += 32) s += partial[p];
  s = sb::warp_sum(s);
  if (threadIdx.x == 0) out[0] = (accumulate ? out[0] : 0.f) + s * scale;
}

// ------------------------------------------- step control (one thread each)
// Before the all-reduce of the step statistics: stats = [sum of squares (already there), overflow flag, status word].
__global__ void step_pack_kernel(float* __restrict__ stats, const int* __restrict__ flag,
                                 const int* __restrict__ status) {
  stats[1] = flag && *flag ? 1.f : 0.f;
  stats[2] = status && *status ? 1.f : 0.f;
}
// After it: norm = sqrt(stats[0] / replicas) * inv; the step is skipped when any rank saw inf / nan or a device-side
// wait that gave up; control = [gradient multiplier, skip], result = [norm, skip, wait gave up, norm after clipping].
__global__ void step_control_kernel(const float* __restrict__ stats, float inv, float clip, float replicas,
                                    float* __restrict__ control, float* __restrict__ result) {
  const float norm = sqrtf(stats[0] / replicas) * inv;
  const bool timed_out = stats[2] > 0.f;
  const bool bad = stats[1] > 0.f || !isfinite(norm) || timed_out;
  const float coef = (clip > 0.f && norm >= clip) ? clip / norm : 1.f;
  control[0] = bad ? 0.f : coef * inv;
  control[1] = bad ? 1.f : 0.f;
  result[0] = norm;
  result[1] = bad ? 1.f : 0.f;
  result[2] = timed_out ? 1.f : 0.f;
  result[3] = norm * coef;
}
// End of the step: a wait that gave up after the statistics were taken (parameter exchange) still reaches the host.
__global__ void step_status_kernel(const int* __restrict__ status, float* __restrict__ result) {
  if (status && *status) result[2] = 1.f;
}

// --------------------------------------------------------------- embedding
// out[t, :] = W[id - vocab_start, :] when id is inside this rank's shard, else 0.
template <typename T>
__global__ void embedding_fwd_kernel(const long* __restrict__ ids, const T* __restrict__ W, T* __restrict__ out,
                                     long tokens, int H, long vocab_start, long vocab_rows) {
  long t = blockIdx.x;
  if (t >= tokens) return;
  long id = ids[t] - vocab_start;
  bool in = id >= 0 && id < vocab_rows;
  constexpr int V = sb::Vec16<T>::N;
  T* o = out + t * H;
  if (H % V == 0) {
    sb::Vec16<T> z;
    z.u = make_uint4(0, 0, 0, 0);
    for (int c = threadIdx.x * V; c < H; c += blockDim.x * V) sb::st16(o + c, in ? sb::ld16(W + id * H + c) : z);
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x) o[c] = in ? W[id * H + c] : sb::from_f<T>(0.f);
  }
}
// Deterministic backward: ids are sorted (with the permutation `order`); the CTA at the head of
// every run of equal ids sums the rows of that run in order and adds them to dW[id].
template <typename T, typename GW>
__global__ void embedding_bwd_kernel(const long* __restrict__ sorted_ids, const long* __restrict__ order,
                                     const T* __restrict__ dout, GW* __restrict__ dW, long tokens, int H,
                                     long vocab_start, long vocab_rows) {
  long i = blockIdx.x;
  if (i >= tokens) return;
  long id = sorted_ids[i];
  if (i > 0 && sorted_ids[i - 1] == id) return;
  long row = id - vocab_start;
  if (row < 0 || row >= vocab_rows) return;
  long end = i + 1;
  while (end < tokens && sorted_ids[end] == id) ++end;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float s = 0.f;
    for (long j = i; j < end; ++j) s += sb::to_f(dout[order[j] * H + c]);
    dW[row * H + c] = sb::from_f<GW>(sb::to_f(dW[row * H + c]) + s);
  }
}

}  // namespace

// g_dtype: dtype of the gradient; lp_dtype: dtype of the low-precision copy (ignored if p_lp is null)
SB_API int sb200_adamw(float* p, float* m, float* v, const void* g, void* p_lp, long n, float lr, float beta1,
                       float beta2, float eps, float wd, float bc1, float bc2, const float* control,
                       const float* hyper, int g_dtype, int lp_dtype, cudaStream_t stream) {
  if (n <= 0) return SB_OK;
  long b = (n / 4 + 255) / 256;
  if (b > 148 * 8) b = 148 * 8;
  if (b < 1) b = 1;
  const uintptr_t all = reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v) |
                        reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(p_lp);
  const int vec_ok = (all & 15) == 0;
  SB_DISPATCH_DTYPE(g_dtype, G, {
    SB_DISPATCH_DTYPE(lp_dtype, P, {
      adamw_kernel<G, P><<<(int)b, 256, 0, stream>>>(p, m, v, (const G*)g, (P*)p_lp, n, lr, beta1, beta2, eps, wd, bc1,
                                                     bc2, control, hyper, vec_ok);
    });
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}

SB_API int sb200_sumsq_max_partials() { return 1024; }

// partial: scratch of >= sb200_sumsq_max_partials() floats
SB_API int sb200_sumsq(const void* g, long n, float* partial, float* out, int* flag, float scale, int accumulate,
                       int dtype, cudaStream_t stream) {
  long b = (n + 1023) / 1024;
  if (b > 1024) b = 1024;
  if (b < 1) b = 1;
  SB_DISPATCH_DTYPE(dtype, G, {
    sumsq_partial_kernel<G><<<(int)b, 256, 0, stream>>>((const G*)g, n, partial, flag);
  });
  SB_CHECK_LAUNCH();
  sumsq_final_kernel<<<1, 32, 0, stream>>>(partial, (int)b, out, scale, accumulate);
  SB_CHECK_LAUNCH();
  return SB_OK;
}

// The scalar arithmetic of an optimizer step as three one-thread kernels (see the kernels above): `which` = 0 pack
// the overflow flag and the status word into stats before the all-reduce, 1 derive the gradient multiplier, the skip
// flag and the values the host reads, 2 fold a late status into the result.
SB_API int sb200_step_control(int which, float* stats, const int* flag, const int* status, float inv, float clip,
                              float replicas, float* control, float* result, cudaStream_t stream) {
  if (which == 0) step_pack_kernel<<<1, 1, 0, stream>>>(stats, flag, status);
  else if (which == 1) step_control_kernel<<<1, 1, 0, stream>>>(stats, inv, clip, replicas, control, result);
  else if (which == 2) step_status_kernel<<<1, 1, 0, stream>>>(status, result);
  else return SB_ERR_BAD_ARG;
  SB_CHECK_LAUNCH();
  return SB_OK;
}

SB_API int sb200_embedding_fwd(const long* ids, const void* W, void* out, long tokens, int H, long vocab_start,
                               long vocab_rows, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return SB_OK;
  SB_DISPATCH_DTYPE(dtype, T, {
    embedding_fwd_kernel<T><<<(unsigned)tokens, 128, 0, stream>>>(ids, (const T*)W, (T*)out, tokens, H, vocab_start,
                                                                  vocab_rows);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
SB_API int sb200_embedding_bwd(const long* sorted_ids, const long* order, const void* dout, void* dW, long tokens,
                               int H, long vocab_start, long vocab_rows, int dtype, int gw_dtype, cudaStream_t stream) {
  if (tokens <= 0) return SB_OK;
  SB_DISPATCH_DTYPE(dtype, T, {
    SB_DISPATCH_DTYPE(gw_dtype, GW, {
      embedding_bwd_kernel<T, GW><<<(unsigned)tokens, 256, 0, stream>>>(sorted_ids, order, (const T*)dout, (GW*)dW,
                                                                        tokens, H, vocab_start, vocab_rows);
    });
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}

// Make `device` current on the calling host thread.  The library carries its own copy of the CUDA runtime, whose
// per-thread device selection is independent of the one in the host framework; worker threads that the framework
// creates (e.g. for backward passes) call this once before their first launch or tensor-map encode.
SB_API int sb200_bind_device(int device) {
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return (int)e;
  e = cudaFree(nullptr);  // forces the primary context to be current on this thread
  return (int)e;
}
