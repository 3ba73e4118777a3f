// bf16/fp16 GEMM on the 5th-generation tensor cores (tcgen05) for sm_100a.
//
//   C[M, N] (+)= A * B  (+ bias[N]) (optional GELU), fp32 accumulation in TMEM.
//
// Operand layouts (element = 2 bytes):
//   A "K-major":  stored [M, K] row-major.        A "MN-major": stored [K, M] row-major.
//   B "K-major":  stored [N, K] row-major.        B "MN-major": stored [K, N] row-major.
// so that  forward  Y = X W^T       -> A = X  (K-major),  B = W  (K-major)
//          dgrad    dX = dY W       -> A = dY (K-major),  B = W  (MN-major, W is [N_red, K_out])
//          wgrad    dW = dY^T X     -> A = dY (MN-major), B = X  (MN-major)
// (these are the F.linear forward / autograd GEMMs of the reference's parallel linears,
//  src/scaling/core/nn/linear/column_parallel_linear.py:162, row_parallel_linear.py:169).
//
// Structure: persistent CTAs (one per SM), 128 x BN output tiles, BK = 64.
//   warp 0    TMA producer: cp.async.bulk.tensor tiles (128-byte swizzle) into a ring of stages
//   warp 1    allocates TMEM, issues tcgen05.mma (one elected thread), commits to mbarriers
//   warps 2-5 epilogue: tcgen05.ld the accumulator (TMEM is double buffered, so the epilogue of
//             tile i overlaps the MMAs of tile i+1), bias / GELU / accumulate, 16-byte stores
// All mbarrier waits are bounded; on expiry the CTA sets *status and unwinds (TMEM is freed).
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  void* C;
  void* C_pre;  // optional: pre-activation output (same dtype / ld as C)
  const void* bias;
  int M, N, K;
  long ldc;
  int act;         // 0 none, 1 gelu
  int accumulate;  // C += result
  int ab_fmt;      // 0 fp16, 1 bf16
  int* status;
};

template <int BN> struct GemmCfg {
  static constexpr int STAGES = BN == 256 ? 4 : 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

template <typename OutT> __device__ __forceinline__ void store8(OutT* dst, const float* v);
template <> __device__ __forceinline__ void store8<float>(float* dst, const float* v) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* dst, const float* v) {
  uint4 u;
  __nv_bfloat162 t0 = __floats2bfloat162_rn(v[0], v[1]), t1 = __floats2bfloat162_rn(v[2], v[3]),
                 t2 = __floats2bfloat162_rn(v[4], v[5]), t3 = __floats2bfloat162_rn(v[6], v[7]);
  u.x = *reinterpret_cast<uint32_t*>(&t0);
  u.y = *reinterpret_cast<uint32_t*>(&t1);
  u.z = *reinterpret_cast<uint32_t*>(&t2);
  u.w = *reinterpret_cast<uint32_t*>(&t3);
  *reinterpret_cast<uint4*>(dst) = u;
}
template <> __device__ __forceinline__ void store8<__half>(__half* dst, const float* v) {
  uint4 u;
  __half2 t0 = __floats2half2_rn(v[0], v[1]), t1 = __floats2half2_rn(v[2], v[3]), t2 = __floats2half2_rn(v[4], v[5]),
          t3 = __floats2half2_rn(v[6], v[7]);
  u.x = *reinterpret_cast<uint32_t*>(&t0);
  u.y = *reinterpret_cast<uint32_t*>(&t1);
  u.z = *reinterpret_cast<uint32_t*>(&t2);
  u.w = *reinterpret_cast<uint32_t*>(&t3);
  *reinterpret_cast<uint4*>(dst) = u;
}
template <typename OutT> __device__ __forceinline__ void load8(const OutT* src, float* v) {
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = sb::to_f(src[i]);
}

template <int BN, bool A_MN, bool B_MN, typename OutT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128-byte swizzle atoms
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint64_t* full_bar = bars;                  // [STAGES]
  uint64_t* empty_bar = bars + STAGES;        // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;    // [2]
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM;
  const int n_tiles = (p.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      sb::mbar_init(&full_bar[s], 1);
      sb::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      sb::mbar_init(&tfull_bar[a], 1);
      sb::mbar_init(&tempty_bar[a], 4);  // one arrive per epilogue warp
    }
    *abort_flag = 0;
    sb::mbar_fence_init();
  }
  if (warp == 1) {
    sb::tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    sb::tmem_relinquish();
  }
  sb::tc_fence_before();
  __syncthreads();
  sb::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      sb::tma_prefetch_desc(&tmA);
      sb::tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m_blk = tile / n_tiles, n_blk = tile % n_tiles;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!sb::mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* a_s = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* b_s = a_s + Cfg::A_BYTES;
          sb::mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              sb::tma_load_2d(a_s + j * 8192, &tmA, &full_bar[stage], m_blk * BM + j * 64, kb * BK);
          } else {
            sb::tma_load_2d(a_s, &tmA, &full_bar[stage], kb * BK, m_blk * BM);
          }
          if (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              sb::tma_load_2d(b_s + j * 8192, &tmB, &full_bar[stage], n_blk * BN + j * 64, kb * BK);
          } else {
            sb::tma_load_2d(b_s, &tmB, &full_bar[stage], kb * BK, n_blk * BN);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = sb::umma_idesc_f16(BM, BN, p.ab_fmt, A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!sb::mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        sb::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!sb::mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          sb::tc_fence_after();
          const uint32_t a_addr = sb::smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? sb::umma_smem_desc(a_addr + k * 2048, 8192, 1024)
                                        : sb::umma_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? sb::umma_smem_desc(b_addr + k * 2048, 8192, 1024)
                                        : sb::umma_smem_desc(b_addr + k * 32, 16, 1024);
            sb::umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb | k) != 0);
          }
          sb::umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        sb::umma_commit(&tfull_bar[acc]);  // accumulator ready for the epilogue
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quad = warp & 3;  // TMEM lane quadrant this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    OutT* C = reinterpret_cast<OutT*>(p.C);
    OutT* Cpre = reinterpret_cast<OutT*>(p.C_pre);
    const __nv_bfloat16* bias_bf = reinterpret_cast<const __nv_bfloat16*>(p.bias);
    const __half* bias_h = reinterpret_cast<const __half*>(p.bias);
    const bool vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                        (!p.C_pre || (reinterpret_cast<uintptr_t>(p.C_pre) & 15) == 0);
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int m_blk = tile / n_tiles, n_blk = tile % n_tiles;
      if (!sb::mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) { ok = false; break; }
      sb::tc_fence_after();
      const int row = m_blk * BM + quad * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        uint32_t r[32];
        sb::tmem_ld32(t_row + ch * 32, r);
        sb::tmem_ld_wait();
        const int n0 = n_blk * BN + ch * 32;
        if (row < p.M && n0 < p.N) {
          OutT* crow = C + (long)row * p.ldc + n0;
          OutT* prow = Cpre ? Cpre + (long)row * p.ldc + n0 : nullptr;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int n = n0 + g * 8;
            if (n >= p.N) break;
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[g * 8 + i]);
            const bool full8 = (n + 8 <= p.N);
            if (p.bias) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (full8 || n + i < p.N)
                  v[i] += p.ab_fmt ? __bfloat162float(bias_bf[n + i]) : __half2float(bias_h[n + i]);
            }
            if (p.accumulate) {
              if (full8 && vec_ok) {
                float o[8];
                load8<OutT>(crow + g * 8, o);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += o[i];
              } else {
                for (int i = 0; i < 8 && n + i < p.N; ++i) v[i] += sb::to_f(crow[g * 8 + i]);
              }
            }
            if (prow) {
              if (full8 && vec_ok) store8<OutT>(prow + g * 8, v);
              else
                for (int i = 0; i < 8 && n + i < p.N; ++i) prow[g * 8 + i] = sb::from_f<OutT>(v[i]);
            }
            if (p.act == 1) {
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = gelu_erf(v[i]);
            }
            if (full8 && vec_ok) store8<OutT>(crow + g * 8, v);
            else
              for (int i = 0; i < 8 && n + i < p.N; ++i) crow[g * 8 + i] = sb::from_f<OutT>(v[i]);
          }
        }
      }
      sb::tc_fence_before();
      __syncwarp();
      if (lane == 0) sb::mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) {
    // give copies in flight a bounded time to land before shared memory is released
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

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
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

// 2-D row-major tensor [rows, cols] of 2-byte elements with leading dimension ld (elements);
// box = [box_rows, 64 cols] with the 128-byte swizzle.
int make_tmap_2d(CUtensorMap* tm, const void* base, long rows, long cols, long ld, int box_rows, int fp16) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return SB_ERR_DRIVER;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SB_OK : SB_ERR_DRIVER;
}

template <int BN, bool A_MN, bool B_MN, typename OutT>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int sm_count,
                cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_tcgen05_kernel<BN, A_MN, B_MN, OutT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  int grid = tiles < sm_count ? tiles : sm_count;
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, p);
  SB_CHECK_LAUNCH();
  return SB_OK;
}

template <bool A_MN, bool B_MN, typename OutT>
int dispatch_bn(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int bn, int sm_count,
                cudaStream_t stream) {
  if (bn == 256) return launch_gemm<256, A_MN, B_MN, OutT>(tmA, tmB, p, sm_count, stream);
  return launch_gemm<128, A_MN, B_MN, OutT>(tmA, tmB, p, sm_count, stream);
}

template <typename OutT>
int dispatch_major(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int a_mn, int b_mn, int bn,
                   int sm_count, cudaStream_t stream) {
  if (!a_mn && !b_mn) return dispatch_bn<false, false, OutT>(tmA, tmB, p, bn, sm_count, stream);
  if (!a_mn && b_mn) return dispatch_bn<false, true, OutT>(tmA, tmB, p, bn, sm_count, stream);
  if (a_mn && b_mn) return dispatch_bn<true, true, OutT>(tmA, tmB, p, bn, sm_count, stream);
  return SB_ERR_BAD_ARG;
}

}  // namespace

// C[M,N] (+)= op(A) op(B) + bias, optional GELU.
//   a_mn = 0: A is [M, K] (lda >= K);  a_mn = 1: A is [K, M] (lda >= M)
//   b_mn = 0: B is [N, K] (ldb >= K);  b_mn = 1: B is [K, N] (ldb >= N)
//   in_dtype / out_dtype: SB_DT_* (inputs bf16 or fp16; output bf16, fp16 (fp16 in only) or fp32)
//   status: device int, set to SB_ERR_WAIT_TIMEOUT if a bounded wait expired (may be null)
SB_API int sb200_gemm(const void* A, const void* B, void* C, void* C_pre, const void* bias, int M, int N, int K,
                      long lda, long ldb, long ldc, int a_mn, int b_mn, int act, int accumulate, int in_dtype,
                      int out_dtype, int bn_hint, int sm_count, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return SB_OK;
  if (K <= 0) return SB_ERR_BAD_ARG;
  if (in_dtype != SB_DT_BF16 && in_dtype != SB_DT_F16) return SB_ERR_BAD_ARG;
  if ((lda % 8) || (ldb % 8)) return SB_ERR_BAD_ARG;  // TMA: strides are multiples of 16 bytes
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return SB_ERR_BAD_ARG;
  const int fp16 = in_dtype == SB_DT_F16;
  int bn = bn_hint == 128 || bn_hint == 256 ? bn_hint : (N > 128 ? 256 : 128);
  // prefer the tile width that leaves fewer idle SMs in the last wave
  if (bn_hint == 0 && N > 128) {
    long t256 = (long)((M + BM - 1) / BM) * ((N + 255) / 256);
    long t128 = (long)((M + BM - 1) / BM) * ((N + 127) / 128);
    double w256 = (double)((t256 + sm_count - 1) / sm_count) * 2.0;  // relative time units
    double w128 = (double)((t128 + sm_count - 1) / sm_count) * 1.08;
    bn = w128 < w256 ? 128 : 256;
  }
  CUtensorMap tmA, tmB;
  int rc;
  if (a_mn) rc = make_tmap_2d(&tmA, A, K, M, lda, 64, fp16);
  else rc = make_tmap_2d(&tmA, A, M, K, lda, BM, fp16);
  if (rc) return rc;
  if (b_mn) rc = make_tmap_2d(&tmB, B, K, N, ldb, 64, fp16);
  else rc = make_tmap_2d(&tmB, B, N, K, ldb, bn, fp16);
  if (rc) return rc;
  GemmParams p;
  p.C = C; p.C_pre = C_pre; p.bias = bias; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.act = act;
  p.accumulate = accumulate; p.ab_fmt = fp16 ? 0 : 1; p.status = status;
  if (out_dtype == SB_DT_F32) return dispatch_major<float>(tmA, tmB, p, a_mn, b_mn, bn, sm_count, stream);
  if (out_dtype == SB_DT_BF16 && !fp16)
    return dispatch_major<__nv_bfloat16>(tmA, tmB, p, a_mn, b_mn, bn, sm_count, stream);
  if (out_dtype == SB_DT_F16 && fp16) return dispatch_major<__half>(tmA, tmB, p, a_mn, b_mn, bn, sm_count, stream);
  return SB_ERR_BAD_ARG;
}
