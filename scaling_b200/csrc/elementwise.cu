// Memory-bound elementwise kernels for sm_100a: SwiGLU, GELU, RoPE, masked softmax,
// dropout + residual add, 2-D transpose.  All use 16-byte vector accesses where the shape allows
// and fp32 math with bf16/fp16/fp32 storage.
//
// Behaviour covered (reference files): silu(a) * g (src/scaling/core/nn/mlp.py:249),
// exact-erf GELU (src/scaling/core/nn/mlp.py:139), rotary embeddings in rotate-half and
// interleaved-pair ("complex") form with position ids and partial rotary dimensions
// (src/scaling/core/nn/rotary.py:117-139, 68-90), softmax(masked_fill(x*scale, mask, -10000))
// (src/scaling/core/nn/masked_softmax/masked_softmax.py:14-34).
#include "common.cuh"

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
// d/dx [x Phi(x)] = Phi(x) + x phi(x).  Phi comes from the rational approximation 7.1.26 of Abramowitz and Stegun of
// erfc (absolute error below 1.5e-7), whose exponential exp(-x^2 / 2) is the one phi needs as well: one ex2, one rcp
// and a dozen FMAs per element, where erff + expf made the backward kernels instruction-bound.
__device__ __forceinline__ float gelu_grad_f(float x) {
  const float z = fabsf(x) * 0.70710678118654752f;
  float t;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, z, 1.f)));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-z * z * 1.4426950408889634f));  // exp(-x^2 / 2)
  const float cdf_neg = 0.5f * poly * t * e;  // Phi(-|x|)
  const float cdf = x >= 0.f ? 1.f - cdf_neg : cdf_neg;
  return fmaf(x * 0.3989422804014327f, e, cdf);
}

// ------------------------------------------------------------------- SwiGLU
// out[m, f] = silu(a[m, f]) * g[m, f]; a, g, out may be column blocks of wider rows.
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ a, const T* __restrict__ g, T* __restrict__ out, long M, int F,
                                  long lda, long ldg, long ldo, float act_scale) {
  constexpr int V = sb::Vec16<T>::N;
  const int fv = F / V;
  long total = M * fv;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    long m = i / fv;
    int c = (int)(i - m * fv) * V;
    auto av = sb::ld16(a + m * lda + c);
    auto gv = sb::ld16(g + m * ldg + c);
    sb::Vec16<T> o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.e[k] = sb::from_f<T>(silu_f(sb::to_f(av.e[k])) * sb::to_f(gv.e[k]) * act_scale);
    sb::st16(out + m * ldo + c, o);
  }
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ a, const T* __restrict__ g,
                                  T* __restrict__ da, T* __restrict__ dg, long M, int F, long lddo, long lda, long ldg,
                                  long ldda, long lddg, float act_scale) {
  constexpr int V = sb::Vec16<T>::N;
  const int fv = F / V;
  long total = M * fv;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    long m = i / fv;
    int c = (int)(i - m * fv) * V;
    auto dv = sb::ld16(dout + m * lddo + c);
    auto av = sb::ld16(a + m * lda + c);
    auto gv = sb::ld16(g + m * ldg + c);
    sb::Vec16<T> oa, og;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float x = sb::to_f(av.e[k]), gg = sb::to_f(gv.e[k]), d = sb::to_f(dv.e[k]) * act_scale;
      float s = sigmoid_f(x);
      float sl = x * s;
      oa.e[k] = sb::from_f<T>(d * gg * (s + sl * (1.f - s)));
      og.e[k] = sb::from_f<T>(d * sl);
    }
    sb::st16(da + m * ldda + c, oa);
    sb::st16(dg + m * lddg + c, og);
  }
}

// --------------------------------------------------------------------- GELU
template <typename T>
__global__ void gelu_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, long n) {
  constexpr int V = sb::Vec16<T>::N;
  long nv = n / V;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
    auto v = sb::ld16(x + i * V);
    sb::Vec16<T> o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.e[k] = sb::from_f<T>(gelu_f(sb::to_f(v.e[k])));
    sb::st16(y + i * V, o);
  }
  // tail
  for (long i = nv * V + blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    y[i] = sb::from_f<T>(gelu_f(sb::to_f(x[i])));
}
template <typename T>
__global__ void gelu_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx, long n) {
  constexpr int V = sb::Vec16<T>::N;
  long nv = n / V;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
    auto v = sb::ld16(x + i * V);
    auto d = sb::ld16(dy + i * V);
    sb::Vec16<T> o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.e[k] = sb::from_f<T>(sb::to_f(d.e[k]) * gelu_grad_f(sb::to_f(v.e[k])));
    sb::st16(dx + i * V, o);
  }
  for (long i = nv * V + blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    dx[i] = sb::from_f<T>(sb::to_f(dy[i]) * gelu_grad_f(sb::to_f(x[i])));
}

// ------------------------------------------------------- dropout + residual
// y = dropout(x) * xs + r * rs, with r optional (the output of a sub-block joining the residual stream:
// src/scaling/transformer/model/layers/layer.py:264-269,283-288; xs / rs carry the u-muP residual scales).  Element g
// (global index: elem_offset + position in this tensor, so that token shards of one tensor draw from one mask)
// is kept iff word (g mod 4) of Philox block (g / 4) is >= thr; kept values are multiplied by keep_scale = 1/(1-p).
// The backward kernel recomputes the mask: dx = dy * mask * keep_scale * xs.
template <typename T, bool BWD>
__global__ void dropout_add_kernel(const T* __restrict__ x, const T* __restrict__ r, T* __restrict__ y, long n,
                                   uint32_t thr, float keep_scale, float xs, float rs,
                                   const long long* __restrict__ rng, uint32_t call, long elem_offset) {
  constexpr int V = sb::Vec16<T>::N;
  const sb::DropoutRng st = sb::dropout_rng(rng, call);
  const long nv = n / V;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
    auto xv = sb::ld16(x + i * V);
    sb::Vec16<T> rv, o;
    if (!BWD && r) rv = sb::ld16(r + i * V);
    const unsigned long long g0 = (unsigned long long)(elem_offset + i * V);
#pragma unroll
    for (int b = 0; b < V / 4; ++b) {
      const uint4 w = sb::dropout_words(st, g0 / 4 + b);
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float kept = ws[k] >= thr ? sb::to_f(xv.e[b * 4 + k]) * keep_scale * xs : 0.f;
        o.e[b * 4 + k] = sb::from_f<T>((!BWD && r) ? kept + sb::to_f(rv.e[b * 4 + k]) * rs : kept);
      }
    }
    sb::st16(y + i * V, o);
  }
  for (long i = nv * V + blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const unsigned long long g = (unsigned long long)(elem_offset + i);
    const uint4 w = sb::dropout_words(st, g / 4);
    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
    const float kept = ws[g & 3] >= thr ? sb::to_f(x[i]) * keep_scale * xs : 0.f;
    y[i] = sb::from_f<T>((!BWD && r) ? kept + sb::to_f(r[i]) * rs : kept);
  }
}
// y = a * as + b * bs (the p = 0 form of the above)
template <typename T>
__global__ void scaled_add_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, long n, float as,
                                  float bs) {
  constexpr int V = sb::Vec16<T>::N;
  long nv = n / V;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
    auto av = sb::ld16(a + i * V);
    auto bv = sb::ld16(b + i * V);
    sb::Vec16<T> o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.e[k] = sb::from_f<T>(sb::to_f(av.e[k]) * as + sb::to_f(bv.e[k]) * bs);
    sb::st16(y + i * V, o);
  }
  for (long i = nv * V + blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
    y[i] = sb::from_f<T>(sb::to_f(a[i]) * as + sb::to_f(b[i]) * bs);
}

// --------------------------------------------------------------------- RoPE
// In place on x[t, h, d] (token stride ld_tok, head stride ld_head).  One CTA per token;
// each thread owns one rotary pair index i and walks the heads, so sin/cos are computed
// once per (token, i).  mode 0: pairs (i, i + rot/2) ("rotate half"); mode 1: pairs (2i, 2i+1).
// sign = +1 forward, -1 backward (the transpose of a rotation is the rotation by -theta).
template <typename T>
__global__ void rope_kernel(T* __restrict__ x, const int* __restrict__ pos, int T_tokens, int n_heads, int rot_dim,
                            long ld_tok, long ld_head, float log2_base, int mode, float sign) {
  int t = blockIdx.x;
  if (t >= T_tokens) return;
  int half = rot_dim >> 1;
  float p = (float)pos[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float inv_freq = exp2f(-log2_base * (2.f * i) / (float)rot_dim);
    float sn, cs;
    sincosf(p * inv_freq, &sn, &cs);
    sn *= sign;
    int i0 = mode == 0 ? i : 2 * i;
    int i1 = mode == 0 ? i + half : 2 * i + 1;
    T* base = x + (long)t * ld_tok;
    for (int h = threadIdx.y; h < n_heads; h += blockDim.y) {
      T* xh = base + h * ld_head;
      float a = sb::to_f(xh[i0]), b = sb::to_f(xh[i1]);
      xh[i0] = sb::from_f<T>(a * cs - b * sn);
      xh[i1] = sb::from_f<T>(b * cs + a * sn);
    }
  }
}

// Vectorised form: a thread owns one 16-byte chunk position of one token, computes the sines and cosines of that
// chunk's frequencies once, and applies them to every head and sub-tensor of the token (the angles depend on the
// position and the frequency only).  A packed [q | k | v] head layout is covered with n_sub = 2, ld_sub = d.
// mode 0: chunk c pairs elements [c*V, c*V + V) with the same range + rot/2; mode 1: chunk c holds V/2 pairs
// (2i, 2i + 1).
template <typename T>
__global__ void rope_vec_kernel(T* __restrict__ x, const int* __restrict__ pos, long total, int n_heads, int n_sub,
                                int n_chunk, int rot_dim, long ld_tok, long ld_head, long ld_sub, float log2_base,
                                int mode, float sign) {
  constexpr int V = sb::Vec16<T>::N;
  const int half = rot_dim >> 1;
  for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % n_chunk);
    const long t = idx / n_chunk;
    const float p = (float)pos[t];
    constexpr int NF = V;  // frequencies per chunk: V in mode 0, V / 2 in mode 1
    float sn[NF], cs[NF];
    const int nf = mode == 0 ? V : V / 2;
#pragma unroll
    for (int i = 0; i < NF; ++i) {
      if (i < nf) {
        const int f = mode == 0 ? c * V + i : c * (V / 2) + i;
        sincosf(p * exp2f(-log2_base * (2.f * (float)f) / (float)rot_dim), &sn[i], &cs[i]);
        sn[i] *= sign;
      }
    }
    T* tok = x + t * ld_tok;
    int h = 0;
    if (mode == 0) {
      // four (head, sub-tensor) slices at a time: eight 16-byte loads in flight per thread before the first store
      const int n_slices = n_heads * n_sub;
      int sl = 0;
      for (; sl + 4 <= n_slices; sl += 4) {
        sb::Vec16<T> a[4], b[4];
        T* base[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          base[j] = tok + ((sl + j) / n_sub) * ld_head + ((sl + j) % n_sub) * ld_sub;
          a[j] = sb::ld16(base[j] + c * V);
          b[j] = sb::ld16(base[j] + half + c * V);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int i = 0; i < V; ++i) {
            const float fa = sb::to_f(a[j].e[i]), fb = sb::to_f(b[j].e[i]);
            a[j].e[i] = sb::from_f<T>(fa * cs[i] - fb * sn[i]);
            b[j].e[i] = sb::from_f<T>(fb * cs[i] + fa * sn[i]);
          }
          sb::st16(base[j] + c * V, a[j]);
          sb::st16(base[j] + half + c * V, b[j]);
        }
      }
      for (; sl < n_slices; ++sl) {  // the slices that do not fill a group of four
        T* bs = tok + (sl / n_sub) * ld_head + (sl % n_sub) * ld_sub;
        sb::Vec16<T> a1 = sb::ld16(bs + c * V), b1 = sb::ld16(bs + half + c * V);
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const float fa = sb::to_f(a1.e[i]), fb = sb::to_f(b1.e[i]);
          a1.e[i] = sb::from_f<T>(fa * cs[i] - fb * sn[i]);
          b1.e[i] = sb::from_f<T>(fb * cs[i] + fa * sn[i]);
        }
        sb::st16(bs + c * V, a1);
        sb::st16(bs + half + c * V, b1);
      }
      h = n_heads;  // mode 0 is done; the loop below serves mode 1
    }
    for (; h < n_heads; ++h) {
      for (int sub = 0; sub < n_sub; ++sub) {
        T* base = tok + h * ld_head + sub * ld_sub;
        if (mode == 0) {
          sb::Vec16<T> a = sb::ld16(base + c * V), b = sb::ld16(base + half + c * V);
#pragma unroll
          for (int i = 0; i < V; ++i) {
            const float fa = sb::to_f(a.e[i]), fb = sb::to_f(b.e[i]);
            a.e[i] = sb::from_f<T>(fa * cs[i] - fb * sn[i]);
            b.e[i] = sb::from_f<T>(fb * cs[i] + fa * sn[i]);
          }
          sb::st16(base + c * V, a);
          sb::st16(base + half + c * V, b);
        } else {
          sb::Vec16<T> a = sb::ld16(base + c * V);
#pragma unroll
          for (int i = 0; i < V / 2; ++i) {
            const float fa = sb::to_f(a.e[2 * i]), fb = sb::to_f(a.e[2 * i + 1]);
            a.e[2 * i] = sb::from_f<T>(fa * cs[i] - fb * sn[i]);
            a.e[2 * i + 1] = sb::from_f<T>(fb * cs[i] + fa * sn[i]);
          }
          sb::st16(base + c * V, a);
        }
      }
    }
  }
}

// ------------------------------------------------------------- column sums
// partial[r][c] = sum over the rows of split r of x[row][c].  A CTA owns a strip of 32 * V columns and one row
// split; warp w takes rows w, w + 8, ... of the split, and the eight warp sums are added in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
    colsum_partial_kernel(const T* __restrict__ x, float* __restrict__ partial, long M, int N, long ld,
                          long rows_per_split) {
  constexpr int V = sb::Vec16<T>::N;
  __shared__ float red[8][32 * V];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = (blockIdx.x * 32 + lane) * V;
  const long r0 = blockIdx.y * rows_per_split;
  long r1 = r0 + rows_per_split;
  if (r1 > M) r1 = M;
  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  if (c < N) {
    long r = r0 + warp;
    // eight independent 16-byte loads per thread before the first add: enough bytes in flight to keep HBM busy
    for (; r + 56 < r1; r += 64) {
      sb::Vec16<T> v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = sb::ld16(x + (r + 8 * j) * ld + c);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] += sb::to_f(v[j].e[i]);
      }
    }
    for (; r + 8 < r1; r += 16) {
      sb::Vec16<T> a = sb::ld16(x + r * ld + c), b = sb::ld16(x + (r + 8) * ld + c);
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] += sb::to_f(a.e[i]) + sb::to_f(b.e[i]);
    }
    for (; r < r1; r += 8) {
      sb::Vec16<T> a = sb::ld16(x + r * ld + c);
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] += sb::to_f(a.e[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < V; ++i) red[warp][lane * V + i] = acc[i];
  __syncthreads();
  for (int t = threadIdx.x; t < 32 * V; t += 256) {
    const int col = blockIdx.x * 32 * V + t;
    if (col < N) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s += red[w][t];
      partial[(long)blockIdx.y * N + col] = s;
    }
  }
}
// GELU backward with the bias gradient in the same pass: dx = dy * gelu'(x) is written and its column sums are taken
// from the registers (the bias gradient of a linear layer with a fused GELU is the column sum of exactly this dx), which
// saves the separate pass that would read dx again.  Same CTA / split layout and summation order as above.
template <typename T>
__global__ void __launch_bounds__(256)
    gelu_bwd_colsum_kernel(const T* __restrict__ dy, const T* __restrict__ x, T* __restrict__ dx,
                           float* __restrict__ partial, long M, int N, long rows_per_split) {
  constexpr int V = sb::Vec16<T>::N;
  __shared__ float red[8][32 * V];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = (blockIdx.x * 32 + lane) * V;
  const long r0 = blockIdx.y * rows_per_split;
  long r1 = r0 + rows_per_split;
  if (r1 > M) r1 = M;
  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  if (c < N) {
    long r = r0 + warp;
    for (; r + 24 < r1; r += 32) {  // four rows per thread in flight
      sb::Vec16<T> d[4], v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        d[j] = sb::ld16(dy + (r + 8 * j) * N + c);
        v[j] = sb::ld16(x + (r + 8 * j) * N + c);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        sb::Vec16<T> o;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          o.e[i] = sb::from_f<T>(sb::to_f(d[j].e[i]) * gelu_grad_f(sb::to_f(v[j].e[i])));
          acc[i] += sb::to_f(o.e[i]);  // the rounded value: what a separate pass over dx would add
        }
        sb::st16(dx + (r + 8 * j) * N + c, o);
      }
    }
    for (; r < r1; r += 8) {
      const sb::Vec16<T> d = sb::ld16(dy + r * N + c), v = sb::ld16(x + r * N + c);
      sb::Vec16<T> o;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        o.e[i] = sb::from_f<T>(sb::to_f(d.e[i]) * gelu_grad_f(sb::to_f(v.e[i])));
        acc[i] += sb::to_f(o.e[i]);
      }
      sb::st16(dx + r * N + c, o);
    }
  }
#pragma unroll
  for (int i = 0; i < V; ++i) red[warp][lane * V + i] = acc[i];
  __syncthreads();
  for (int t = threadIdx.x; t < 32 * V; t += 256) {
    const int col = blockIdx.x * 32 * V + t;
    if (col < N) {
      float s2 = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) s2 += red[w][t];
      partial[(long)blockIdx.y * N + col] = s2;
    }
  }
}
// out[c] = (accumulate ? out[c] : 0) + sum_r partial[r][c], fixed order.  A CTA owns 32 columns; warp w adds rows
// w, w + 8, ... with four loads in flight (one thread per column walking all rows was a chain of dependent L2
// round trips that cost as much as the pass over the matrix), then the eight warp sums are added in order.
template <typename T>
__global__ void __launch_bounds__(256)
    colsum_final_kernel(const float* __restrict__ partial, T* __restrict__ out, int R, int N, int accumulate) {
  __shared__ float red[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (c < N) {
    int r = warp;
    for (; r + 24 < R; r += 32) {
      const float v0 = __ldcg(partial + (long)r * N + c), v1 = __ldcg(partial + (long)(r + 8) * N + c);
      const float v2 = __ldcg(partial + (long)(r + 16) * N + c), v3 = __ldcg(partial + (long)(r + 24) * N + c);
      s += (v0 + v1) + (v2 + v3);
    }
    for (; r < R; r += 8) s += __ldcg(partial + (long)r * N + c);
  }
  red[warp][lane] = s;
  __syncthreads();
  if (warp == 0 && c < N) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][lane];
    if (accumulate) t += sb::to_f(out[c]);
    out[c] = sb::from_f<T>(t);
  }
}

// ----------------------------------------------------------- masked softmax
// x: [rows, cols]; mask (uint8, 1 = masked) addressed as mask[(row / rows_per_mask_div) ...]:
// row r of x uses mask row  (r / (heads * sq)) * sq + (r % sq)  when the mask is [b, 1, sq, sk].
template <typename T>
__global__ void masked_softmax_fwd_kernel(const T* __restrict__ x, const uint8_t* __restrict__ mask, T* __restrict__ y,
                                          long rows, int cols, int heads, int sq, float scale) {
  __shared__ float red[33];
  long r = blockIdx.x;
  if (r >= rows) return;
  const T* xr = x + r * cols;
  T* yr = y + r * cols;
  const uint8_t* mr = nullptr;
  if (mask) {
    long b = r / ((long)heads * sq);
    long q = r % sq;
    mr = mask + (b * sq + q) * cols;
  }
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = sb::to_f(xr[c]) * scale;
    if (mr && mr[c]) v = -10000.f;
    mx = fmaxf(mx, v);
  }
  mx = sb::block_max(mx, red);
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = sb::to_f(xr[c]) * scale;
    if (mr && mr[c]) v = -10000.f;
    s += __expf(v - mx);
  }
  s = sb::block_sum(s, red);
  float inv = 1.f / s;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = sb::to_f(xr[c]) * scale;
    if (mr && mr[c]) v = -10000.f;
    yr[c] = sb::from_f<T>(__expf(v - mx) * inv);
  }
}
// dx = scale * y * (dy - sum(dy * y)); masked positions receive zero gradient.
template <typename T>
__global__ void masked_softmax_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ y,
                                          const uint8_t* __restrict__ mask, T* __restrict__ dx, long rows, int cols,
                                          int heads, int sq, float scale) {
  __shared__ float red[33];
  long r = blockIdx.x;
  if (r >= rows) return;
  const T* yr = y + r * cols;
  const T* dyr = dy + r * cols;
  T* dxr = dx + r * cols;
  const uint8_t* mr = nullptr;
  if (mask) {
    long b = r / ((long)heads * sq);
    long q = r % sq;
    mr = mask + (b * sq + q) * cols;
  }
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) s += sb::to_f(dyr[c]) * sb::to_f(yr[c]);
  s = sb::block_sum(s, red);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float g = scale * sb::to_f(yr[c]) * (sb::to_f(dyr[c]) - s);
    if (mr && mr[c]) g = 0.f;
    dxr[c] = sb::from_f<T>(g);
  }
}

// ------------------------------------------------------------------ transpose
// out[c, r] = in[r, c] for a row-major [R, C] matrix (32x32 tiles through shared memory).
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int R, int C) {
  __shared__ T tile[32][33];
  int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int r = r0 + j, c = c0 + threadIdx.x;
    if (r < R && c < C) tile[j][threadIdx.x] = in[(size_t)r * C + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += blockDim.y) {
    int c = c0 + j, r = r0 + threadIdx.x;
    if (r < R && c < C) out[(size_t)c * R + r] = tile[threadIdx.x][j];
  }
}

inline int grid_for(long work, int threads, int max_blocks = 148 * 16) {
  long b = (work + threads - 1) / threads;
  if (b > max_blocks) b = max_blocks;
  if (b < 1) b = 1;
  return (int)b;
}

}  // namespace

SB_API int sb200_swiglu_fwd(const void* a, const void* g, void* out, long M, int F, long lda, long ldg, long ldo,
                            float act_scale, int dtype, cudaStream_t stream) {
  if (M <= 0 || F <= 0) return SB_OK;
  SB_DISPATCH_DTYPE(dtype, T, {
    constexpr int V = sb::Vec16<T>::N;
    if (F % V || lda % V || ldg % V || ldo % V) return SB_ERR_BAD_ARG;
    swiglu_fwd_kernel<T><<<grid_for(M * (F / V), 256), 256, 0, stream>>>((const T*)a, (const T*)g, (T*)out, M, F, lda,
                                                                           ldg, ldo, act_scale);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
SB_API int sb200_swiglu_bwd(const void* dout, const void* a, const void* g, void* da, void* dg, long M, int F, long lddo,
                            long lda, long ldg, long ldda, long lddg, float act_scale, int dtype, cudaStream_t stream) {
  if (M <= 0 || F <= 0) return SB_OK;
  SB_DISPATCH_DTYPE(dtype, T, {
    constexpr int V = sb::Vec16<T>::N;
    if (F % V || lda % V || ldg % V || lddo % V || ldda % V || lddg % V) return SB_ERR_BAD_ARG;
    swiglu_bwd_kernel<T><<<grid_for(M * (F / V), 256), 256, 0, stream>>>(
        (const T*)dout, (const T*)a, (const T*)g, (T*)da, (T*)dg, M, F, lddo, lda, ldg, ldda, lddg, act_scale);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
SB_API int sb200_gelu_fwd(const void* x, void* y, long n, int dtype, cudaStream_t stream) {
  if (n <= 0) return SB_OK;
  SB_DISPATCH_DTYPE(dtype, T, {
    gelu_fwd_kernel<T><<<grid_for(n / sb::Vec16<T>::N + 1, 256), 256, 0, stream>>>((const T*)x, (T*)y, n);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
SB_API int sb200_gelu_bwd(const void* dy, const void* x, void* dx, long n, int dtype, cudaStream_t stream) {
  if (n <= 0) return SB_OK;
  SB_DISPATCH_DTYPE(dtype, T, {
    gelu_bwd_kernel<T><<<grid_for(n / sb::Vec16<T>::N + 1, 256), 256, 0, stream>>>((const T*)dy, (const T*)x, (T*)dx,
                                                                                     n);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
// y = dropout(x, p) * x_scale + r * r_scale (backward = 0), or dx = dy * mask / (1 - p) * x_scale (backward = 1, r
// unused).  r may be null (plain dropout).  p = 0 needs no random numbers (rng may be null): the call is a scaled add.
// rng: device int64[2] = {seed, step}; call: index of this dropout inside the step; elem_offset: index of x[0] in
// the tensor that the mask is defined on (non-zero for the token shards of sequence parallelism; a multiple of 4).
SB_API int sb200_dropout_add(const void* x, const void* r, void* y, long n, float p, float x_scale, float r_scale,
                             const long long* rng, unsigned int call, long elem_offset, int backward, int dtype,
                             cudaStream_t stream) {
  if (n <= 0) return SB_OK;
  if (p < 0.f || p >= 1.f || (elem_offset & 3)) return SB_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(r) | reinterpret_cast<uintptr_t>(y)) & 15)
    return SB_ERR_BAD_ARG;
  if (p == 0.f) {
    if (backward || !r) return SB_ERR_BAD_ARG;  // nothing to do: the caller passes the tensor through
    SB_DISPATCH_DTYPE(dtype, T, {
      scaled_add_kernel<T><<<grid_for(n / sb::Vec16<T>::N + 1, 256), 256, 0, stream>>>((const T*)x, (const T*)r, (T*)y,
                                                                                      n, x_scale, r_scale);
    });
    SB_CHECK_LAUNCH();
    return SB_OK;
  }
  if (!rng) return SB_ERR_BAD_ARG;
  const double t = (double)p * 4294967296.0;
  const uint32_t thr = t >= 4294967295.0 ? 4294967295u : (uint32_t)t;
  const float keep_scale = 1.f / (1.f - p);
  SB_DISPATCH_DTYPE(dtype, T, {
    const int grid = grid_for(n / sb::Vec16<T>::N + 1, 256);
    if (backward)
      dropout_add_kernel<T, true><<<grid, 256, 0, stream>>>((const T*)x, nullptr, (T*)y, n, thr, keep_scale, x_scale,
                                                            0.f, rng, call, elem_offset);
    else
      dropout_add_kernel<T, false><<<grid, 256, 0, stream>>>((const T*)x, (const T*)r, (T*)y, n, thr, keep_scale,
                                                             x_scale, r_scale, rng, call, elem_offset);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
// In-place rotary embedding of n_sub tensors that share token and head strides and start ld_sub elements apart
// (e.g. the q and k parts of a packed [tokens, heads, 3 * d] projection: n_sub = 2, ld_sub = d).
SB_API int sb200_rope_multi(void* x, const int* pos, int tokens, int n_heads, int rot_dim, long ld_tok, long ld_head,
                            int n_sub, long ld_sub, float base, int mode, int backward, int dtype,
                            cudaStream_t stream) {
  if (tokens <= 0 || n_heads <= 0 || rot_dim <= 0 || n_sub <= 0) return SB_OK;
  if (rot_dim & 1) return SB_ERR_BAD_ARG;
  int half = rot_dim / 2;
  SB_DISPATCH_DTYPE(dtype, T, {
    constexpr int V = sb::Vec16<T>::N;
    const int span = mode == 0 ? half : rot_dim;
    const bool vec = span % V == 0 && ld_tok % V == 0 && ld_head % V == 0 && ld_sub % V == 0 &&
                     (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    if (vec) {
      const int n_chunk = span / V;
      const long total = (long)tokens * n_chunk;
      rope_vec_kernel<T><<<grid_for(total, 128), 128, 0, stream>>>((T*)x, pos, total, n_heads, n_sub, n_chunk, rot_dim,
                                                                   ld_tok, ld_head, ld_sub, log2f(base), mode,
                                                                   backward ? -1.f : 1.f);
    } else {
      int tx = half >= 64 ? 64 : (half >= 32 ? 32 : 16);
      int ty = 256 / tx;
      if (ty > n_heads) ty = n_heads;
      dim3 block(tx, ty);
      for (int sub = 0; sub < n_sub; ++sub)
        rope_kernel<T><<<tokens, block, 0, stream>>>((T*)x + sub * ld_sub, pos, tokens, n_heads, rot_dim, ld_tok,
                                                      ld_head, log2f(base), mode, backward ? -1.f : 1.f);
    }
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
SB_API int sb200_rope(void* x, const int* pos, int tokens, int n_heads, int rot_dim, long ld_tok, long ld_head,
                      float base, int mode, int backward, int dtype, cudaStream_t stream) {
  return sb200_rope_multi(x, pos, tokens, n_heads, rot_dim, ld_tok, ld_head, 1, 0, base, mode, backward, dtype, stream);
}
// Row splits used by sb200_colsum for an [M, N] input; the caller provides `partial` of [splits, N] floats.
SB_API int sb200_colsum_splits(long M, int N, int elem_size, int sm_count) {
  const int V = 16 / (elem_size > 0 ? elem_size : 2);
  const int strips = (N + 32 * V - 1) / (32 * V);
  long r = (6L * sm_count + strips - 1) / strips;  // about six CTAs (48 warps) per SM: the loads of fewer do not cover HBM latency
  const long max_r = (M + 63) / 64;
  if (r > max_r) r = max_r;
  if (r > 128) r = 128;
  if (r < 1) r = 1;
  return (int)r;
}
// dx[M, N] = dy * gelu'(x) and bias_grad[N] (+)= column sums of dx, one pass (contiguous [M, N] tensors, N a multiple
// of 16 bytes; partial: [splits, N] floats with splits from sb200_colsum_splits); deterministic.
SB_API int sb200_gelu_bwd_colsum(const void* dy, const void* x, void* dx, void* bias_grad, float* partial, long M, int N,
                                 int splits, int accumulate, int dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return SB_OK;
  if (splits < 1) return SB_ERR_BAD_ARG;
  SB_DISPATCH_DTYPE(dtype, T, {
    constexpr int V = sb::Vec16<T>::N;
    if (N % V || ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dx)) & 15))
      return SB_ERR_BAD_ARG;
    const int strips = (N + 32 * V - 1) / (32 * V);
    const long rows_per = (M + splits - 1) / splits;
    gelu_bwd_colsum_kernel<T><<<dim3(strips, splits), 256, 0, stream>>>((const T*)dy, (const T*)x, (T*)dx, partial, M, N,
                                                                         rows_per);
    SB_CHECK_LAUNCH();
    colsum_final_kernel<T><<<(N + 31) / 32, 256, 0, stream>>>(partial, (T*)bias_grad, splits, N, accumulate);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
// out[N] (+)= column sums of x[M, N] (row stride ld elements, N and ld multiples of 16 bytes); deterministic.
SB_API int sb200_colsum(const void* x, void* out, float* partial, long M, int N, long ld, int splits, int accumulate,
                        int dtype, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return SB_OK;
  if (splits < 1) return SB_ERR_BAD_ARG;
  SB_DISPATCH_DTYPE(dtype, T, {
    constexpr int V = sb::Vec16<T>::N;
    if (N % V || ld % V || (reinterpret_cast<uintptr_t>(x) & 15)) return SB_ERR_BAD_ARG;
    const int strips = (N + 32 * V - 1) / (32 * V);
    const long rows_per = (M + splits - 1) / splits;
    colsum_partial_kernel<T><<<dim3(strips, splits), 256, 0, stream>>>((const T*)x, partial, M, N, ld, rows_per);
    SB_CHECK_LAUNCH();
    colsum_final_kernel<T><<<(N + 31) / 32, 256, 0, stream>>>(partial, (T*)out, splits, N, accumulate);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
SB_API int sb200_masked_softmax_fwd(const void* x, const uint8_t* mask, void* y, long rows, int cols, int heads, int sq,
                                    float scale, int dtype, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return SB_OK;
  int threads = cols >= 1024 ? 256 : (cols >= 256 ? 128 : 64);
  SB_DISPATCH_DTYPE(dtype, T, {
    masked_softmax_fwd_kernel<T><<<(unsigned)rows, threads, 0, stream>>>((const T*)x, mask, (T*)y, rows, cols, heads,
                                                                          sq, scale);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
SB_API int sb200_masked_softmax_bwd(const void* dy, const void* y, const uint8_t* mask, void* dx, long rows, int cols,
                                    int heads, int sq, float scale, int dtype, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return SB_OK;
  int threads = cols >= 1024 ? 256 : (cols >= 256 ? 128 : 64);
  SB_DISPATCH_DTYPE(dtype, T, {
    masked_softmax_bwd_kernel<T><<<(unsigned)rows, threads, 0, stream>>>((const T*)dy, (const T*)y, mask, (T*)dx, rows,
                                                                          cols, heads, sq, scale);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
SB_API int sb200_transpose(const void* in, void* out, int R, int C, int dtype, cudaStream_t stream) {
  if (R <= 0 || C <= 0) return SB_OK;
  dim3 grid((C + 31) / 32, (R + 31) / 32), block(32, 8);
  SB_DISPATCH_DTYPE(dtype, T, { transpose_kernel<T><<<grid, block, 0, stream>>>((const T*)in, (T*)out, R, C); });
  SB_CHECK_LAUNCH();
  return SB_OK;
}
