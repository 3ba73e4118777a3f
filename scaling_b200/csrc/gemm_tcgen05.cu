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
//   warps 2-9 epilogue: tcgen05.ld the accumulator (TMEM is double buffered, so the epilogue of
//             tile i overlaps the MMAs of tile i+1); two warps share a TMEM lane quadrant and take half of
//             the columns each.  bias (staged in shared memory) / GELU / optional pre-activation output;
//             16-bit results are packed into a swizzled staging box and leave through TMA stores, which
//             also clip partial tiles.  fp32 output, accumulation into C and unaligned C use 16-byte
//             stores from registers instead.
// Split-K: a work unit is (tile, k-split).  Every split writes its fp32 partial tile to a workspace and
//   bumps a per-tile counter; the CTA that arrives last adds the partials in split order (a fixed
//   order, so results do not depend on timing) and runs the epilogue.  Nothing waits on another CTA.
// All mbarrier waits are bounded; on expiry the CTA sets *status and unwinds (TMEM is freed).
#include <cuda.h>

#include "common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int EPI_WARPS = 8;
constexpr int GEMM_THREADS = 64 + EPI_WARPS * 32;
constexpr int STAGE_BOX_BYTES = 32 * 128;  // one epilogue staging box: 32 rows x 64 16-bit columns

// Fused all-reduce of the output over the tensor-parallel group (see the reducer role in the kernel).  All pointer
// tables are indexed by rank; entry r is rank r's buffer as mapped into this process.
constexpr int AR_MAX_RANKS = 8;
constexpr int REDUCER_THREADS = 128;
struct ArParams {
  void* partial[AR_MAX_RANKS];   // [M, ldc] partial products (this rank writes partial[rank])
  void* out[AR_MAX_RANKS];       // [M, ldc] reduced result, every rank receives all of it
  uint32_t* flags[AR_MAX_RANKS]; // [(W + 1) * flag_stride]: flags[r][q * stride + t] = rank q finished tile t (t owned by
                                 // r); flags[r][W * stride + q] = rank q has finished all its reductions
  void* partial_mc;              // multicast addresses of the two buffers, or null (plain peer loads / stores)
  void* out_mc;
  uint32_t* epoch;               // local: number of completed fused launches on this workspace
  unsigned int* done_ctas;       // local: CTAs of this launch that have finished
  int flag_stride;
  int rank, W;
  unsigned long long timeout_ns;
  // mode 0: all-reduce.  mode 1: reduce-scatter along the rows, rank r keeps rows [r * shard_rows, (r + 1) *
  // shard_rows) in out[rank] ([shard_rows, ld_out], local memory is enough).  mode 2: all-gather of the A operand:
  // every rank pushes its [shard_rows, K] shard a_src into the rows [rank * shard_rows, ...) of partial[q] ([M, K])
  // of every rank q, and the tile loads of a row block wait for its arrival; the output is a plain local GEMM result.
  int mode;
  // partial[] holds two buffers of half_elems elements; launch after launch alternates between them (half = 0 / 1,
  // counted by the host from the last launch with sync_entry).  A buffer is therefore rewritten two launches after
  // it was filled, and no rank can finish a launch before every peer has entered it (it needs their tiles, rows or
  // completion flags): whoever read the buffer has finished by then.  sync_entry = 1 starts a new count: every rank
  // first waits until all ranks have entered this launch.
  long half_elems;
  int half;
  int sync_entry;
  int shard_rows;
  int unit_shift;     // tiles are visited from this one on (modulo their number): a different start on every rank
  long ld_out;
  const void* a_src;
  long lda_src;
};
constexpr int AR_ALLREDUCE = 0, AR_REDUCE_SCATTER = 1, AR_ALLGATHER = 2;

struct GemmParams {
  void* C;
  void* C_pre;  // optional: pre-activation output (same dtype / ld as C)
  const void* bias;
  int M, N, K;
  long ldc;
  int act;         // 0 none, 1 gelu
  int accumulate;  // C += result
  int ab_fmt;      // 0 fp16, 1 bf16 (16-bit operands; also the format of the bias)
  int a8_fmt, b8_fmt;  // 8-bit operands (AB8 instantiations): 0 e4m3, 1 e5m2
  int splits;      // k-splits per tile (1: none)
  int tma_store;   // 1: 16-bit C (and C_pre) leave through the tensor maps tmC / tmP
  float* ws_partial;  // split-K: [tiles * splits][BN / 32][128][32] floats
  int* ws_counter;    // split-K: one arrival counter per tile, zero between launches
  int* status;
  ArParams ar;        // used by the FUSE instantiations only
};

// PAIR: two CTAs of a cluster compute one 256 x BN tile with cta_group::2 MMAs; each CTA loads its own 128 rows of A
// and half of the B rows, which halves the operand bytes every SM pulls from L2 per flop.
template <int BN, bool PAIR> struct GemmCfg {
  static constexpr int CTAS = PAIR ? 2 : 1;
  static constexpr int LOAD_BN = BN / CTAS;  // B rows (output columns) this CTA loads per stage
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = LOAD_BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  // 48 KB stages (a single CTA on a 256-wide tile): four of them and one staging box per epilogue warp; 32 KB stages:
  // five and two staging boxes per warp, so that a warp fills one box while the TMA store still reads the other
  static constexpr int STAGES = STAGE_BYTES == 49152 ? 4 : 5;
  static constexpr int EPI_BUFS = STAGE_BYTES == 49152 ? 1 : 2;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int EPI_BYTES = EPI_WARPS * EPI_BUFS * STAGE_BOX_BYTES;
  static constexpr int BIAS_BYTES = 2 * BN * 2;  // two tiles' worth of 16-bit bias values
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + BIAS_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};
static_assert(GemmCfg<256, false>::SMEM_BYTES <= 232448 && GemmCfg<256, true>::SMEM_BYTES <= 232448, "shared memory");

// Exact-form GELU 0.5 x (1 + erf(x / sqrt 2)) with erf from the rational approximation 7.1.26 of Abramowitz and
// Stegun (absolute error below 1.5e-7, far under the rounding of 16-bit outputs); about a third of the
// instructions of erff, which matters because the epilogue shares the SM with the MMA issue.
__device__ __forceinline__ float gelu_erf(float x) {
  const float z = fabsf(x) * 0.70710678118654752f;
  float t;  // 1 / (1 + p z): the approximate reciprocal is one MUFU instruction, its error (1 ulp) is irrelevant here
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, z, 1.f)));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-z * z * 1.4426950408889634f));
  const float erfc_abs = poly * t * e;            // 1 - erf(|x| / sqrt 2)
  const float cdf_neg = 0.5f * erfc_abs;          // Phi(-|x|)
  return x * (x >= 0.f ? 1.f - cdf_neg : cdf_neg);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, __nv_bfloat16) {
  __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ uint32_t pack2(float a, float b, __half) {
  __half2 t = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&t);
}
__device__ __forceinline__ uint32_t pack2(float a, float, float) { return __float_as_uint(a); }  // unused for fp32
// the two 16-bit bias values packed in w, as floats
__device__ __forceinline__ void bias_pair(uint32_t w, int is_bf16, float& lo, float& hi) {
  if (is_bf16) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x;
    hi = f.y;
  }
}
// Number of CTAs that share the push of one 128-row block in the all-gather mode (the same on every rank and in every
// CTA of a launch: it depends on the grid and the shapes only).
constexpr int GATHER_MAX_GROUPS = 16;
__device__ __forceinline__ int gather_groups(int grid, int blocks, int kvec) {
  int g = grid / (blocks > 0 ? blocks : 1);
  if (g > GATHER_MAX_GROUPS) g = GATHER_MAX_GROUPS;
  if (g > kvec) g = kvec;
  return g < 1 ? 1 : g;
}
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory"); }
__device__ __forceinline__ void red_bar_sync() { asm volatile("bar.sync 2, %0;" ::"n"(REDUCER_THREADS) : "memory"); }
template <typename OutT> __device__ __forceinline__ uint4 multimem_sum16(const void* mc);
template <> __device__ __forceinline__ uint4 multimem_sum16<__nv_bfloat16>(const void* mc) {
  return sb::multimem_ld_reduce_add_bf16x2(mc);
}
template <> __device__ __forceinline__ uint4 multimem_sum16<__half>(const void* mc) {
  return sb::multimem_ld_reduce_add_f16x2(mc);
}
template <> __device__ __forceinline__ uint4 multimem_sum16<float>(const void*) { return make_uint4(0, 0, 0, 0); }

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
template <typename OutT> __device__ __forceinline__ void load8(const OutT* src, float* v);
template <> __device__ __forceinline__ void load8<float>(const float* src, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* src, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(src);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <> __device__ __forceinline__ void load8<__half>(const __half* src, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(src);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

// FUSE: the output is summed over the ranks of a tensor-parallel group inside the kernel.  Every rank runs the same
// launch on its own operands.  The epilogue writes the partial tile to this rank's buffer and flags it at the
// tile's owner (tile number modulo group size); four extra warps per CTA ("reducers") wait until all ranks have
// flagged a tile they own, sum the partial tiles (one multimem.ld_reduce per 16 bytes: the switch adds the
// replicas; or peer loads added in rank order) and store the result to every rank's output (multimem.st or peer
// stores).  Tiles are reduced while later tiles are still being multiplied.  The last CTA of a launch exchanges
// completion flags with the peers, so the kernel ends only when this rank's output is complete.
// AB8: the operands are 8-bit floating point (e4m3 / e5m2, K-major): a k-block is 128 elements = the same 128 bytes per
// row, an MMA instruction covers 32 of them (kind::f8f6f4), everything after the accumulator is unchanged.
template <int BN, bool A_MN, bool B_MN, typename OutT, bool PAIR, bool FUSE, bool AB8 = false>
__global__ void __launch_bounds__(FUSE ? GEMM_THREADS + REDUCER_THREADS : GEMM_THREADS, 1)
    gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmP,
                        const __grid_constant__ CUtensorMap tmA2, const GemmParams p) {
  using Cfg = GemmCfg<BN, PAIR>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int CTAS = Cfg::CTAS;
  constexpr int LOAD_BN = Cfg::LOAD_BN;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128-byte swizzle atoms
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_stage = smem + STAGES * Cfg::STAGE_BYTES;                       // [EPI_WARPS][4 KB]
  uint16_t* sbias = reinterpret_cast<uint16_t*>(epi_stage + Cfg::EPI_BYTES);   // [2][BN] raw 16-bit values
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_stage + Cfg::EPI_BYTES + Cfg::BIAS_BYTES);
  uint64_t* full_bar = bars;                  // [STAGES]
  uint64_t* empty_bar = bars + STAGES;        // [STAGES]
  uint64_t* tfull_bar = bars + 2 * STAGES;    // [2]
  uint64_t* tempty_bar = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // a tile is BM * CTAS rows: with PAIR, CTA `rank` of the cluster owns rows [rank * BM, rank * BM + BM) of it
  const int rank = PAIR ? (int)sb::cluster_ctarank() : 0;
  const int worker = PAIR ? blockIdx.x >> 1 : blockIdx.x;        // index of this CTA (pair) among the workers
  const int num_workers = PAIR ? gridDim.x >> 1 : gridDim.x;
  const int m_tiles = (p.M + BM * CTAS - 1) / (BM * CTAS);
  const int n_tiles = (p.N + BN - 1) / BN;
  constexpr int BKE = AB8 ? 2 * BK : BK;  // elements per k-block (128 bytes per row either way)
  const int num_kb = (p.K + BKE - 1) / BKE;
  const int S = p.splits;
  const int num_units = m_tiles * n_tiles * S;
  const uint32_t epoch = FUSE ? *p.ar.epoch + 1 : 0;  // identifies this launch in the peers' flag words
  const int ushift = FUSE ? p.ar.unit_shift : 0;
  // In the all-gather mode the tile loads wait for a peer (time budget ar.timeout_ns); the roles behind them keep
  // waiting for as long: one spin limit is about three seconds.
  const int wait_rounds = (FUSE && p.ar.mode == AR_ALLGATHER) ? (int)(p.ar.timeout_ns / 2000000000ull) + 2 : 1;
  // position in this worker's sequence -> unit (tile, split); fused launches start at a rank-specific tile
  auto unit_at = [&](int i) { return FUSE ? (i + ushift) % num_units : i; };
  // tile -> (row block of tiles, column block).  Tiles are numbered down groups of RASTER_M tile rows, so the tiles
  // that run at the same time (consecutive numbers) cover about as many tile rows as tile columns and share their A
  // and B panels in L2; numbering them row by row makes every wave sweep the whole of B, which for a wide N (a
  // 12288- or 32000-column weight) is more than L2 holds.  Fused launches keep the row-major numbering that their
  // ownership rules are written in.
  constexpr int RASTER_M = PAIR ? 8 : 16;
  auto tile_mn = [&](int tile) -> int2 {  // .x: tile row, .y: tile column
    if (FUSE) return make_int2(tile / n_tiles, tile % n_tiles);
    const int per_group = RASTER_M * n_tiles;
    const int g = tile / per_group, r = tile - g * per_group;
    const int first = g * RASTER_M;
    const int gm = m_tiles - first < RASTER_M ? m_tiles - first : RASTER_M;
    const int nb = r / gm;
    return make_int2(first + (r - nb * gm), nb);
  };
  // fused launches on the second buffer of the workspace: the gathered operand is read through tmA2, partial tiles
  // are stored through tmP (which no fused reduction uses for a pre-activation output)
  const CUtensorMap* mapA = (FUSE && p.ar.mode == AR_ALLGATHER && p.ar.half) ? &tmA2 : &tmA;
  const CUtensorMap* mapC = (FUSE && p.ar.mode != AR_ALLGATHER && p.ar.half) ? &tmP : &tmC;
  const long hoff = FUSE ? (long)p.ar.half * p.ar.half_elems : 0;  // element offset of the buffer in use

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      sb::mbar_init(&full_bar[s], 1);
      sb::mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      sb::mbar_init(&tfull_bar[a], 1);
      sb::mbar_init(&tempty_bar[a], EPI_WARPS * CTAS);  // one arrive per epilogue warp (of both CTAs of a pair)
    }
    *abort_flag = 0;
    *last_flag = 0;
    sb::mbar_fence_init();
    if (FUSE && p.ar.sync_entry) {
      // first launch of a count: nothing of this launch is written anywhere before every rank has entered it
      const long slot = (long)(p.ar.W + 1) * p.ar.flag_stride;
      if (blockIdx.x == 0)
        for (int q = 0; q < p.ar.W; ++q) sb::st_release_sys(p.ar.flags[q] + slot + p.ar.rank, epoch);
      for (int q = 0; q < p.ar.W; ++q)
        if (!sb::wait_flag_ge(p.ar.flags[p.ar.rank] + slot + q, epoch, p.ar.timeout_ns)) {
          *abort_flag = 1;
          break;
        }
    }
  }
  if (warp == 1) {
    if (PAIR) {
      sb::tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
      sb::tmem_relinquish_pair();
    } else {
      sb::tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
      sb::tmem_relinquish();
    }
  }
  sb::tc_fence_before();
  if (PAIR) sb::cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  else __syncthreads();
  sb::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      sb::tma_prefetch_desc(mapA);
      sb::tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int it = worker; it < num_units && ok; it += num_workers) {
        const int unit = unit_at(it);
        const int tile = unit / S, split = unit - tile * S;
        const int2 mn = tile_mn(tile);
        const int m_blk = mn.x * CTAS + rank, n_blk = mn.y;
        const int kb0 = (int)((long)split * num_kb / S), kb1 = (int)((long)(split + 1) * num_kb / S);
        const int b_col0 = n_blk * BN + rank * LOAD_BN;  // first output column whose B rows this CTA loads
        if (FUSE && p.ar.mode == AR_ALLGATHER && m_blk * BM < p.M) {
          // the rows of this block come from rank `src`: wait until its gather warps have delivered them
          const int src = (m_blk * BM) / p.ar.shard_rows, rb = (m_blk * BM - src * p.ar.shard_rows) / BM;
          const int groups = gather_groups(gridDim.x, (p.ar.shard_rows + BM - 1) / BM, p.K / 8);
          const uint32_t* arrived = p.ar.flags[p.ar.rank] + (long)src * p.ar.flag_stride + rb * groups;
          for (int g = 0; g < groups && ok; ++g)  // one flag per column range of the block
            if (!sb::wait_flag_ge(arrived + g, epoch, p.ar.timeout_ns)) ok = false;
          if (!ok) {
            *abort_flag = 1;
            break;
          }
          sb::fence_proxy_async_global();
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!sb::mbar_wait_rounds(&empty_bar[stage], phase ^ 1, abort_flag, wait_rounds)) { ok = false; break; }
          uint8_t* a_s = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* b_s = a_s + Cfg::A_BYTES;
          if (PAIR) {
            // the leader's barrier counts the bytes of both CTAs; the MMAs it guards read both shared memories
            const uint32_t bar = sb::mapa_u32(&full_bar[stage], 0);
            if (rank == 0) sb::mbar_expect_tx(&full_bar[stage], CTAS * Cfg::STAGE_BYTES);
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                sb::tma_load_2d_pair(a_s + j * 8192, mapA, bar, m_blk * BM + j * 64, kb * BKE);
            } else {
              sb::tma_load_2d_pair(a_s, mapA, bar, kb * BKE, m_blk * BM);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < LOAD_BN / 64; ++j)
                sb::tma_load_2d_pair(b_s + j * 8192, &tmB, bar, b_col0 + j * 64, kb * BKE);
            } else {
              sb::tma_load_2d_pair(b_s, &tmB, bar, kb * BKE, b_col0);
            }
          } else {
            sb::mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
            if (A_MN) {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                sb::tma_load_2d(a_s + j * 8192, mapA, &full_bar[stage], m_blk * BM + j * 64, kb * BKE);
            } else {
              sb::tma_load_2d(a_s, mapA, &full_bar[stage], kb * BKE, m_blk * BM);
            }
            if (B_MN) {
#pragma unroll
              for (int j = 0; j < BN / 64; ++j)
                sb::tma_load_2d(b_s + j * 8192, &tmB, &full_bar[stage], n_blk * BN + j * 64, kb * BKE);
            } else {
              sb::tma_load_2d(b_s, &tmB, &full_bar[stage], kb * BKE, n_blk * BN);
            }
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0 && rank == 0) {  // of a pair, the leader issues the MMAs for both CTAs
      const uint32_t idesc = AB8 ? sb::umma_idesc_f8(BM * CTAS, BN, p.a8_fmt, p.b8_fmt)
                                 : sb::umma_idesc_f16(BM * CTAS, BN, p.ab_fmt, A_MN ? 1u : 0u, B_MN ? 1u : 0u);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int it = worker; it < num_units && ok; it += num_workers) {
        const int unit = unit_at(it);
        const int tile = unit / S, split = unit - tile * S;
        const int kb0 = (int)((long)split * num_kb / S), kb1 = (int)((long)(split + 1) * num_kb / S);
        if (!sb::mbar_wait_rounds(&tempty_bar[acc], acc_phase ^ 1, abort_flag, wait_rounds)) { ok = false; break; }
        sb::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!sb::mbar_wait_rounds(&full_bar[stage], phase, abort_flag, wait_rounds)) { ok = false; break; }
          sb::tc_fence_after();
          const uint32_t a_addr = sb::smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t b_addr = a_addr + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? sb::umma_smem_desc(a_addr + k * 2048, 8192, 1024)
                                        : sb::umma_smem_desc(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? sb::umma_smem_desc(b_addr + k * 2048, 8192, 1024)
                                        : sb::umma_smem_desc(b_addr + k * 32, 16, 1024);
            const uint32_t acc_flag = (kb > kb0) || (k != 0);
            if (AB8) {
              if (PAIR) sb::umma_f8_ss_pair(d_tmem, adesc, bdesc, idesc, acc_flag);
              else sb::umma_f8_ss(d_tmem, adesc, bdesc, idesc, acc_flag);
            } else {
              if (PAIR) sb::umma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, acc_flag);
              else sb::umma_f16_ss(d_tmem, adesc, bdesc, idesc, acc_flag);
            }
          }
          // frees the smem stage (in both CTAs of a pair) once these MMAs retire
          if (PAIR) sb::umma_commit_pair(&empty_bar[stage], 3);
          else sb::umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        // accumulator ready for the epilogue (of both CTAs of a pair: each reads its own TMEM)
        if (PAIR) sb::umma_commit_pair(&tfull_bar[acc], 3);
        else sb::umma_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp < 2 + EPI_WARPS) {
    // ------------------------------------------------------------ epilogue
    const int ew = warp - 2;            // 0 .. EPI_WARPS-1
    const int quad = warp & 3;          // TMEM lane quadrant this warp may access
    const int chalf = ew >> 2;          // which half of the tile's columns this warp owns
    const int et = threadIdx.x - 64;    // epilogue thread index
    constexpr int HALF = BN / 2;
    constexpr int CHUNKS = HALF / 32;   // 32-column chunks per warp
    constexpr bool OUT16 = sizeof(OutT) == 2;
    uint8_t* const stage_base = epi_stage + ew * (Cfg::EPI_BUFS * STAGE_BOX_BYTES);
    int sbuf = 0;  // staging box the next store is built in
    int acc = 0;
    uint32_t acc_phase = 0;
    int bias_buf = 0;
    OutT* C = reinterpret_cast<OutT*>(p.C) + ((FUSE && p.ar.mode != AR_ALLGATHER) ? hoff : 0);
    OutT* Cpre = reinterpret_cast<OutT*>(p.C_pre);
    const uint16_t* bias_raw = reinterpret_cast<const uint16_t*>(p.bias);
    const bool vec_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0) &&
                        (!p.C_pre || (reinterpret_cast<uintptr_t>(p.C_pre) & 15) == 0);
    const bool use_tma = OUT16 && p.tma_store;
    bool ok = true;
    // A warp whose wait expired keeps walking the units without touching data, so that the named barriers
    // below still see all their participants and nobody is left waiting.
    const uint32_t tempty_leader[2] = {PAIR ? sb::mapa_u32(&tempty_bar[0], 0) : 0u,
                                       PAIR ? sb::mapa_u32(&tempty_bar[1], 0) : 0u};
    auto release_acc = [&](int a) {  // this warp has read its part of accumulator `a`
      if (PAIR) sb::mbar_arrive_cluster(tempty_leader[a]);
      else sb::mbar_arrive(&tempty_bar[a]);
    };
    for (int it = worker; it < num_units; it += num_workers) {
      const int unit = unit_at(it);
      const int tile = unit / S;
      const int2 mn = tile_mn(tile);
      const int m_blk = mn.x * CTAS + rank, n_blk = mn.y;
      const int ctile = tile * CTAS + rank;  // this CTA's part of the tile: index of its counter and partial slots
      if (ok && !sb::mbar_wait_rounds(&tfull_bar[acc], acc_phase, abort_flag, wait_rounds)) ok = false;
      sb::tc_fence_after();
      const int row = m_blk * BM + quad * 32 + lane;
      const uint32_t t_acc = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
      const int acc_used = acc;
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }

      if (S > 1) {
        // park this split's partial tile, then find out whether every other split has arrived already
        float* part = p.ws_partial + (((long)ctile * S + (unit - tile * S)) * (BN / 32) * 128 + quad * 32 + lane) * 32;
#pragma unroll 1
        for (int c = 0; c < CHUNKS && ok; ++c) {
          const int ch = chalf * CHUNKS + c;
          uint32_t r[32];
          sb::tmem_ld32(t_acc + ch * 32, r);
          sb::tmem_ld_wait();
          float4* dst = reinterpret_cast<float4*>(part + (long)ch * 128 * 32);
#pragma unroll
          for (int g = 0; g < 8; ++g)
            dst[g] = make_float4(__uint_as_float(r[g * 4]), __uint_as_float(r[g * 4 + 1]), __uint_as_float(r[g * 4 + 2]),
                                 __uint_as_float(r[g * 4 + 3]));
        }
        sb::tc_fence_before();
        __syncwarp();
        if (lane == 0 && ok) release_acc(acc_used);
        __threadfence();
        epi_bar_sync();
        if (et == 0) {
          const int old = atomicAdd(&p.ws_counter[ctile], 1);
          const int last = old == S - 1;
          if (last) p.ws_counter[ctile] = 0;  // every split has arrived: leave the counter clean for the next launch
          *last_flag = last;
        }
        epi_bar_sync();
        if (!*last_flag) continue;
        __threadfence();
        // last arrival: fold the partial tiles of splits 1 .. S-1 into the slot of split 0, in split order, with all
        // epilogue threads striding over the tile (many independent loads in flight); the finishing code below
        // then reads one reduced tile
        {
          float4* slot0 = reinterpret_cast<float4*>(p.ws_partial + (long)ctile * S * (BN / 32) * 128 * 32);
          constexpr int TILE_F4 = (BN / 32) * 128 * 32 / 4;
          for (int i = et; i < TILE_F4; i += EPI_WARPS * 32 * 2) {
            const int j = i + EPI_WARPS * 32;
            float4 a0 = __ldcg(slot0 + i);
            float4 a1 = j < TILE_F4 ? __ldcg(slot0 + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s2 = 1; s2 < S; ++s2) {
              const float4 b0 = __ldcg(slot0 + (long)s2 * TILE_F4 + i);
              a0.x += b0.x; a0.y += b0.y; a0.z += b0.z; a0.w += b0.w;
              if (j < TILE_F4) {
                const float4 b1 = __ldcg(slot0 + (long)s2 * TILE_F4 + j);
                a1.x += b1.x; a1.y += b1.y; a1.z += b1.z; a1.w += b1.w;
              }
            }
            slot0[i] = a0;
            if (j < TILE_F4) slot0[j] = a1;
          }
          __threadfence_block();
          epi_bar_sync();
        }
      }

      // v[0..32) = accumulator values of 32-column chunk `ch` of this thread's row
      auto load_chunk = [&](int ch, float* v) {
        if (S == 1) {
          uint32_t r[32];
          sb::tmem_ld32(t_acc + ch * 32, r);
          sb::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        } else {
          const float4* src = reinterpret_cast<const float4*>(
              p.ws_partial + (((long)ctile * S * (BN / 32) + ch) * 128 + quad * 32 + lane) * 32);
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const float4 f = __ldcg(src + g);
            v[g * 4] = f.x; v[g * 4 + 1] = f.y; v[g * 4 + 2] = f.z; v[g * 4 + 3] = f.w;
          }
        }
      };

      const uint32_t* sb_tile = reinterpret_cast<const uint32_t*>(sbias + bias_buf * BN);  // pairs of columns
      if (p.bias) {
        if (et < BN) {
          const int n = n_blk * BN + et;
          sbias[bias_buf * BN + et] = n < p.N ? bias_raw[n] : (uint16_t)0;
        }
        epi_bar_sync();
        bias_buf ^= 1;
      }

      if (ok) {
      if (use_tma) {
        const int row0 = m_blk * BM + quad * 32;
        // swizzled position of 16-byte chunk j of this lane's row inside the 32 x 128-byte staging box
        const int sw = lane & 7;
#pragma unroll 1
        for (int bx = 0; bx < CHUNKS / 2; ++bx) {
          const int col0 = chalf * HALF + bx * 64;  // first column of this box inside the tile
          const int n0 = n_blk * BN + col0;
          if (n0 >= p.N || row0 >= p.M) break;
          const int passes = Cpre ? 2 : 1;
          for (int pass = 0; pass < passes; ++pass) {
            const bool pre_pass = Cpre && pass == 0;
            // the store that last used this box has finished reading it
            uint8_t* const stage_buf = stage_base + sbuf * STAGE_BOX_BYTES;
            uint8_t* const my_row = stage_buf + lane * 128;
            if (lane == 0) {
              if (Cfg::EPI_BUFS == 2) sb::tma_store_wait_read1();
              else sb::tma_store_wait_read0();
            }
            sbuf ^= Cfg::EPI_BUFS - 1;
            __syncwarp();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              float v[32];
              load_chunk(col0 / 32 + h, v);
              if (p.bias) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                  float lo, hi;
                  bias_pair(sb_tile[(col0 + h * 32) / 2 + i], p.ab_fmt, lo, hi);
                  v[2 * i] += lo;
                  v[2 * i + 1] += hi;
                }
              }
              if (p.act == 1 && !pre_pass) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = gelu_erf(v[i]);
              }
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                uint4 u;
                u.x = pack2(v[g * 8 + 0], v[g * 8 + 1], OutT());
                u.y = pack2(v[g * 8 + 2], v[g * 8 + 3], OutT());
                u.z = pack2(v[g * 8 + 4], v[g * 8 + 5], OutT());
                u.w = pack2(v[g * 8 + 6], v[g * 8 + 7], OutT());
                *reinterpret_cast<uint4*>(my_row + (((h * 4 + g) ^ sw) << 4)) = u;
              }
            }
            sb::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              // accumulate: the memory system adds the box to C (the sum is rounded to the output type there, the
              // product once before it, like a separate "C += product" on 16-bit tensors)
              if (p.accumulate) sb::tma_reduce_add_2d(mapC, stage_buf, n0, row0);
              else sb::tma_store_2d(pre_pass ? &tmP : mapC, stage_buf, n0, row0);
              sb::tma_store_commit();
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < CHUNKS; ++c) {
          const int ch = chalf * CHUNKS + c;
          const int n0 = n_blk * BN + ch * 32;
          if (n0 >= p.N) break;  // warp-uniform
          float r[32];
          load_chunk(ch, r);
          if (row < p.M) {
            OutT* crow = C + (long)row * p.ldc + n0;
            OutT* prow = Cpre ? Cpre + (long)row * p.ldc + n0 : nullptr;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int n = n0 + g * 8;
              if (n >= p.N) break;
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = r[g * 8 + i];
              const bool full8 = (n + 8 <= p.N);
              if (p.bias) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  float lo, hi;
                  bias_pair(sb_tile[(ch * 32 + g * 8) / 2 + i], p.ab_fmt, lo, hi);
                  v[2 * i] += lo;
                  v[2 * i + 1] += hi;
                }
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
      }
      }  // ok
      if (S == 1 && ok) {
        sb::tc_fence_before();
        __syncwarp();
        if (lane == 0) release_acc(acc_used);
      }
      if (FUSE && p.ar.mode != AR_ALLGATHER) {
        // the partial tile is complete in memory before its owner is told so
        if (lane == 0) sb::tma_store_wait_all0();
        __syncwarp();
        __threadfence_system();
        epi_bar_sync();
        if (et == 0) {
          // all-reduce: rotated per CTA of a pair, every CTA owns 1 / W of its tiles; reduce-scatter: by row range
          const int owner = p.ar.mode == AR_REDUCE_SCATTER ? (m_blk * BM) / p.ar.shard_rows : (tile + rank) % p.ar.W;
          if (owner < p.ar.W)  // a block below the last row (odd number of blocks under a CTA pair) has no owner
            sb::st_release_sys(p.ar.flags[owner] + (long)p.ar.rank * p.ar.flag_stride + ctile, epoch);
        }
      }
    }
    // stores in flight read the staging boxes: drain them before shared memory goes away
    if (lane == 0) sb::tma_store_wait_all0();
    __syncwarp();
  }

  else if (FUSE) {
    // ------------------------------------------------------------ reducers
    const int rt = threadIdx.x - (64 + EPI_WARPS * 32);
    const ArParams& ar = p.ar;
    constexpr int VPR = BN / 8;  // 16-byte vectors per tile row
    bool rok = true;
    if (ar.mode == AR_ALLGATHER) {
      // ---------------------------------------------------------- gather: push this rank's rows of A to every rank
      // The destination is the buffer that was not used by the previous launch (see ArParams::half): a rank's
      // copy of it is free as soon as that rank has finished the launch before the previous one, which it has,
      // since this rank could not have finished the previous launch without it.
      if (*abort_flag) rok = false;  // the entry wait of a new count gave up
      const int kvec = p.K / 8;  // 16-byte vectors per row
      const int blocks = (ar.shard_rows + BM - 1) / BM;
      // a 128-row block is pushed by `groups` CTAs, each a range of columns, so that all CTAs of the launch share
      // the work; neighbouring CTAs take the same block: the first blocks (multiplied first by the peers) land first
      const int groups = gather_groups(gridDim.x, blocks, kvec);
      const int cw = (kvec + groups - 1) / groups;  // vectors per row and group
      const uint16_t* src = reinterpret_cast<const uint16_t*>(ar.a_src);
      for (int item = blockIdx.x; item < blocks * groups && rok; item += gridDim.x) {
        const int rb = item / groups, g = item - rb * groups;
        const int r0 = rb * BM;
        const int nrows = ar.shard_rows - r0 < BM ? ar.shard_rows - r0 : BM;
        const int v0 = g * cw;
        const int nv = kvec - v0 < cw ? (kvec - v0 > 0 ? kvec - v0 : 0) : cw;
        const int total = nrows * nv;
        constexpr int UNR = 8;
        for (int base = rt; base < total; base += REDUCER_THREADS * UNR) {
          uint4 v[UNR];
          long doff[UNR];
          bool valid[UNR];
#pragma unroll
          for (int j = 0; j < UNR; ++j) {
            const int idx = base + j * REDUCER_THREADS;
            valid[j] = idx < total;
            const int row = r0 + idx / nv, col = (v0 + idx % nv) * 8;
            doff[j] = hoff + ((long)ar.rank * ar.shard_rows + row) * p.K + col;
            if (valid[j]) v[j] = __ldg(reinterpret_cast<const uint4*>(src + (long)row * ar.lda_src + col));
          }
          if (ar.partial_mc) {
#pragma unroll
            for (int j = 0; j < UNR; ++j)
              if (valid[j]) sb::multimem_st_b128(reinterpret_cast<uint16_t*>(ar.partial_mc) + doff[j], v[j]);
          } else {
            for (int q = 0; q < ar.W; ++q) {
#pragma unroll
              for (int j = 0; j < UNR; ++j)
                if (valid[j]) *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(ar.partial[q]) + doff[j]) = v[j];
            }
          }
        }
        __threadfence_system();  // the piece has landed everywhere before any rank is told so
        red_bar_sync();
        if (rt < ar.W) sb::st_release_sys(ar.flags[rt] + (long)ar.rank * ar.flag_stride + item, epoch);
      }
    } else
    for (int it = worker; it < num_units; it += num_workers) {
      const int unit = unit_at(it);
      const int ctile = unit * CTAS + rank;  // S == 1 in fused launches: unit = tile
      const int m0 = ((unit / n_tiles) * CTAS + rank) * BM, n0 = (unit % n_tiles) * BN;
      const bool scatter = ar.mode == AR_REDUCE_SCATTER;
      // same ownership rule as in the epilogue
      if ((scatter ? m0 / ar.shard_rows : (unit + rank) % ar.W) != ar.rank) continue;
      const long out_shift = scatter ? (long)ar.rank * ar.shard_rows * p.ldc : 0;  // the shard starts at row 0 of out
      if (rok && rt < ar.W) {
        if (!sb::wait_flag_ge(ar.flags[ar.rank] + (long)rt * ar.flag_stride + ctile, epoch, ar.timeout_ns))
          *abort_flag = 1;
      }
      red_bar_sync();
      if (*abort_flag) rok = false;
      if (!rok) continue;
      // several 16-byte pieces per thread and pass: all loads are issued before the first result is needed, which
      // keeps enough bytes in flight to cover the NVLink round trip
      auto piece = [&](int idx, long& off) -> bool {
        const int row = m0 + idx / VPR, col = n0 + (idx % VPR) * 8;
        off = (long)row * p.ldc + col;
        return idx < BM * VPR && row < p.M && col < p.N;
      };
      OutT* out_local = reinterpret_cast<OutT*>(ar.out[ar.rank]);
      if (ar.partial_mc) {
        constexpr int UNR = 8;
        for (int base = rt; base < BM * VPR; base += REDUCER_THREADS * UNR) {
          long off[UNR];
          bool valid[UNR];
          uint4 v[UNR];
#pragma unroll
          for (int j = 0; j < UNR; ++j) {
            valid[j] = piece(base + j * REDUCER_THREADS, off[j]);
            if (valid[j]) v[j] = multimem_sum16<OutT>(reinterpret_cast<const OutT*>(ar.partial_mc) + hoff + off[j]);
          }
          if (scatter) {
#pragma unroll
            for (int j = 0; j < UNR; ++j)
              if (valid[j]) *reinterpret_cast<uint4*>(out_local + (off[j] - out_shift)) = v[j];
          } else {
#pragma unroll
            for (int j = 0; j < UNR; ++j)
              if (valid[j]) sb::multimem_st_b128(reinterpret_cast<OutT*>(ar.out_mc) + off[j], v[j]);
          }
        }
      } else {
        constexpr int UNR = 4;
        for (int base = rt; base < BM * VPR; base += REDUCER_THREADS * UNR) {
          long off[UNR];
          bool valid[UNR];
          float acc[UNR][8];
#pragma unroll
          for (int j = 0; j < UNR; ++j) {
            valid[j] = piece(base + j * REDUCER_THREADS, off[j]);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
          }
          for (int q = 0; q < ar.W; ++q) {  // rank order: the sum is the same on every launch
            uint4 raw[UNR];
#pragma unroll
            for (int j = 0; j < UNR; ++j)
              if (valid[j])
                raw[j] = *reinterpret_cast<const uint4*>(reinterpret_cast<const OutT*>(ar.partial[q]) + hoff + off[j]);
#pragma unroll
            for (int j = 0; j < UNR; ++j)
              if (valid[j]) {
                float v[8];
                load8<OutT>(reinterpret_cast<const OutT*>(&raw[j]), v);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[j][i] += v[i];
              }
          }
          if (scatter) {
#pragma unroll
            for (int j = 0; j < UNR; ++j)
              if (valid[j]) store8<OutT>(out_local + (off[j] - out_shift), acc[j]);
          } else {
            for (int q = 0; q < ar.W; ++q) {
#pragma unroll
              for (int j = 0; j < UNR; ++j)
                if (valid[j]) store8<OutT>(reinterpret_cast<OutT*>(ar.out[q]) + off[j], acc[j]);
            }
          }
        }
      }
    }
    __threadfence_system();  // this CTA's share of the result is visible to the peers before it reports completion
  }

  // ---------------------------------------------------------------- teardown
  if (*abort_flag) {
    // give copies in flight a bounded time to land before shared memory is released
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
  }
  sb::tc_fence_before();
  // a pair leaves together: the leader's MMAs read the peer's shared memory, and both signal each other's barriers
  if (PAIR) sb::cluster_sync_all();
  else __syncthreads();
  if (warp == 1) {
    sb::tc_fence_after();
    if (PAIR) sb::tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
    else sb::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) *p.status = SB_ERR_WAIT_TIMEOUT;
  if (FUSE && threadIdx.x == 0) {
    // All-reduce: the peers write this rank's output, so the last CTA of the launch tells every peer that this rank
    // has finished reducing and waits for the same message from all of them; when the launch ends, every tile of
    // the output has arrived.  The other two forms produce their output locally and need no message at the end
    // (the partial / gathered buffers alternate between launches instead, see ArParams::half).
    const ArParams& ar = p.ar;
    __threadfence_system();
    if (atomicAdd(ar.done_ctas, 1u) == gridDim.x - 1) {
      *ar.done_ctas = 0;
      if (ar.mode == AR_ALLREDUCE) {
        for (int q = 0; q < ar.W; ++q)
          sb::st_release_sys(ar.flags[q] + (long)ar.W * ar.flag_stride + ar.rank, epoch);
        for (int q = 0; q < ar.W; ++q)
          if (!sb::wait_flag_ge(ar.flags[ar.rank] + (long)ar.W * ar.flag_stride + q, epoch, ar.timeout_ns) && p.status)
            *p.status = SB_ERR_WAIT_TIMEOUT;
      }
      *ar.epoch = epoch;
      __threadfence();
    }
  }
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
// fp16 = 2 selects 1-byte elements (8-bit floats move as bytes): the box is then 128 elements wide.
int make_tmap_2d(CUtensorMap* tm, const void* base, long rows, long cols, long ld, int box_rows, int fp16) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return SB_ERR_DRIVER;
  const int esize = fp16 == 2 ? 1 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * esize};
  cuuint32_t box[2] = {(cuuint32_t)(128 / esize), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, fp16 == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                : (fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16), 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? SB_OK : SB_ERR_DRIVER;
}

template <int BN, bool A_MN, bool B_MN, typename OutT, bool PAIR, bool FUSE = false, bool AB8 = false>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmP,
                const GemmParams& p, int sm_count, cudaStream_t stream, const CUtensorMap* tmA2 = nullptr) {
  using Cfg = GemmCfg<BN, PAIR>;
  auto kern = gemm_tcgen05_kernel<BN, A_MN, B_MN, OutT, PAIR, FUSE, AB8>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int rows = BM * Cfg::CTAS;
  const int units = ((p.M + rows - 1) / rows) * ((p.N + BN - 1) / BN) * p.splits;
  const int max_workers = sm_count / Cfg::CTAS;
  const int workers = units < max_workers ? units : max_workers;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(workers * Cfg::CTAS);
  cfg.blockDim = dim3(FUSE ? GEMM_THREADS + REDUCER_THREADS : GEMM_THREADS);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = Cfg::CTAS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = PAIR ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmC, tmP, tmA2 ? *tmA2 : tmA, p);
  if (e != cudaSuccess) return (int)e;
  return SB_OK;
}

// shape: 128 / 256 = tile width of a single CTA; 512 = CTA pair on a 256 x 256 tile
template <bool A_MN, bool B_MN, typename OutT>
int dispatch_bn(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmP,
                const GemmParams& p, int shape, int sm_count, cudaStream_t stream) {
  if (shape == 512) return launch_gemm<256, A_MN, B_MN, OutT, true>(tmA, tmB, tmC, tmP, p, sm_count, stream);
  if (shape == 256) return launch_gemm<256, A_MN, B_MN, OutT, false>(tmA, tmB, tmC, tmP, p, sm_count, stream);
  return launch_gemm<128, A_MN, B_MN, OutT, false>(tmA, tmB, tmC, tmP, p, sm_count, stream);
}

template <typename OutT>
int dispatch_major(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmP,
                   const GemmParams& p, int a_mn, int b_mn, int shape, int sm_count, cudaStream_t stream) {
  if (!a_mn && !b_mn) return dispatch_bn<false, false, OutT>(tmA, tmB, tmC, tmP, p, shape, sm_count, stream);
  if (!a_mn && b_mn) return dispatch_bn<false, true, OutT>(tmA, tmB, tmC, tmP, p, shape, sm_count, stream);
  if (a_mn && b_mn) return dispatch_bn<true, true, OutT>(tmA, tmB, tmC, tmP, p, shape, sm_count, stream);
  return SB_ERR_BAD_ARG;
}

constexpr long WS_COUNTER_BYTES = 4096;  // 1024 tile counters at the head of the workspace

// Tile shape (128, 256, or 512 = CTA pair) and k-splits for an [M, N, K] problem.  The estimate is
// (waves of work units) x (time of one unit); a unit's time is its k-blocks times a per-block cost that reflects
// the operand bytes an SM pulls from L2 per flop (the bound of these kernels), plus a fixed cost per unit and per
// split.  The constants are fitted to measurements of the transformer shapes on a B200.
void choose_shape(int M, int N, int K, int shape_hint, int split_hint, int sm_count, long ws_bytes, int* shape_out,
                  int* splits_out) {
  const int num_kb = (K + BK - 1) / BK;
  double best = 1e30;
  int best_shape = 128, best_s = 1;
  const int shapes[3] = {128, 256, 512};
  for (int si = 0; si < 3; ++si) {
    const int shape = shapes[si];
    if (shape_hint && shape != shape_hint) continue;
    const int bn = shape == 128 ? 128 : 256;
    const int ctas = shape == 512 ? 2 : 1;
    if (!shape_hint && ((bn == 256 && N <= 128) || (ctas == 2 && M <= 128))) continue;
    const long tiles = (long)((M + BM * ctas - 1) / (BM * ctas)) * ((N + bn - 1) / bn);
    const double kb_cost = shape == 128 ? 0.37 : (shape == 256 ? 0.45 : 0.42);  // microseconds per k-block
    const double split_cost = bn == 128 ? 3.5 : 7.0;  // per split: writing and folding one fp32 partial tile
    const int workers = sm_count / ctas;
    for (int s = 1; s <= 16; ++s) {
      if (split_hint > 0 && s != split_hint) continue;
      if (s > 1) {
        if (tiles * ctas > 1024 || num_kb / s < (split_hint > 0 ? 1 : 8)) break;
        const long need = WS_COUNTER_BYTES + tiles * ctas * s * (long)BM * bn * 4;
        if (need > ws_bytes) break;
      }
      const long units = tiles * s;
      const long waves = (units + workers - 1) / workers;
      // fewer busy SMs run at higher clocks and see less contention in L2
      const double busy = (double)(units < workers ? units : workers) * ctas / sm_count;
      const double load = 0.75 + 0.25 * (busy < 1.0 ? busy : 1.0);
      const double unit_time = (double)num_kb / s * kb_cost * load + 1.0 + (s > 1 ? s * split_cost : 0.0);
      const double t = waves * unit_time + 7.0;
      if (t < best * 0.97) { best = t; best_shape = shape; best_s = s; }
    }
  }
  *shape_out = best_shape;
  *splits_out = best_s;
}

// box = [32 rows, 64 columns] of a 16-bit row-major [rows, cols] matrix, 128-byte swizzle (epilogue stores)
int make_tmap_out(CUtensorMap* tm, const void* base, long rows, long cols, long ld, int fp16) {
  return make_tmap_2d(tm, base, rows, cols, ld, 32, fp16);
}

}  // namespace

// C[M,N] (+)= op(A) op(B) + bias, optional GELU.
//   a_mn = 0: A is [M, K] (lda >= K);  a_mn = 1: A is [K, M] (lda >= M)
//   b_mn = 0: B is [N, K] (ldb >= K);  b_mn = 1: B is [K, N] (ldb >= N)
//   in_dtype / out_dtype: SB_DT_* (inputs bf16 or fp16; output bf16, fp16 (fp16 in only) or fp32)
//   bn_hint / split_hint: 0 = choose; otherwise the tile shape (128 / 256 wide single-CTA tiles, 512 = a CTA pair
//              on a 256 x 256 tile) and the number of k-splits to use
//   workspace: optional device scratch for split-K (first 4 KB: tile counters, zero before the first use and
//              left zero by every launch; then fp32 partial tiles); without it no problem is split.  One
//              workspace serves one stream at a time.
//   status: device int, set to SB_ERR_WAIT_TIMEOUT if a bounded wait expired (may be null)
SB_API int sb200_gemm_ws(const void* A, const void* B, void* C, void* C_pre, const void* bias, int M, int N, int K,
                         long lda, long ldb, long ldc, int a_mn, int b_mn, int act, int accumulate, int in_dtype,
                         int out_dtype, int bn_hint, int split_hint, int sm_count, void* workspace, long workspace_bytes,
                         int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return SB_OK;
  if (K <= 0) return SB_ERR_BAD_ARG;
  if (in_dtype != SB_DT_BF16 && in_dtype != SB_DT_F16) return SB_ERR_BAD_ARG;
  if ((lda % 8) || (ldb % 8)) return SB_ERR_BAD_ARG;  // TMA: strides are multiples of 16 bytes
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return SB_ERR_BAD_ARG;
  const int fp16 = in_dtype == SB_DT_F16;
  if (bn_hint != 128 && bn_hint != 256 && bn_hint != 512) bn_hint = 0;
  int shape = 128, splits = 1;
  const bool ws_ok = workspace && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0;
  choose_shape(M, N, K, bn_hint, split_hint, sm_count, ws_ok ? workspace_bytes : 0, &shape, &splits);
  const int bn = shape == 128 ? 128 : 256;
  const int b_rows = shape == 512 ? 128 : bn;  // B rows one CTA loads per stage
  CUtensorMap tmA, tmB, tmC, tmP;
  int rc;
  if (a_mn) rc = make_tmap_2d(&tmA, A, K, M, lda, 64, fp16);
  else rc = make_tmap_2d(&tmA, A, M, K, lda, BM, fp16);
  if (rc) return rc;
  if (b_mn) rc = make_tmap_2d(&tmB, B, K, N, ldb, 64, fp16);
  else rc = make_tmap_2d(&tmB, B, N, K, ldb, b_rows, fp16);
  if (rc) return rc;
  GemmParams p;
  p.C = C; p.C_pre = C_pre; p.bias = bias; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.act = act;
  p.accumulate = accumulate; p.ab_fmt = fp16 ? 0 : 1; p.status = status;
  p.splits = splits;
  p.ws_counter = reinterpret_cast<int*>(workspace);
  p.ws_partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + WS_COUNTER_BYTES);
  const bool out16 = out_dtype != SB_DT_F32;
  p.tma_store = out16 && (!accumulate || (!C_pre && act == 0)) && (ldc % 8 == 0) &&
                (reinterpret_cast<uintptr_t>(C) & 15) == 0 && (!C_pre || (reinterpret_cast<uintptr_t>(C_pre) & 15) == 0);
  tmC = tmA;
  tmP = tmA;  // placeholders when the epilogue stores from registers
  if (p.tma_store) {
    if ((rc = make_tmap_out(&tmC, C, M, N, ldc, fp16))) return rc;
    if (C_pre && (rc = make_tmap_out(&tmP, C_pre, M, N, ldc, fp16))) return rc;
  }
  if (out_dtype == SB_DT_F32) return dispatch_major<float>(tmA, tmB, tmC, tmP, p, a_mn, b_mn, shape, sm_count, stream);
  if (out_dtype == SB_DT_BF16 && !fp16)
    return dispatch_major<__nv_bfloat16>(tmA, tmB, tmC, tmP, p, a_mn, b_mn, shape, sm_count, stream);
  if (out_dtype == SB_DT_F16 && fp16)
    return dispatch_major<__half>(tmA, tmB, tmC, tmP, p, a_mn, b_mn, shape, sm_count, stream);
  return SB_ERR_BAD_ARG;
}

// C[M, N] = A[M, K] B[N, K]^T (+ bias) with 8-bit floating-point operands (a_fmt / b_fmt: 0 = e4m3, 1 = e5m2), fp32
// accumulation on the tensor cores (kind::f8f6f4) and a bf16 or fp32 result; no scaling factors, like a scaled matmul
// with unit scales (src/scaling/core/fp8/fp8_linear.py:34-43).  lda / ldb (elements = bytes) are multiples of 16.
SB_API int sb200_gemm_fp8(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, long lda,
                          long ldb, long ldc, int a_fmt, int b_fmt, int accumulate, int out_dtype, int sm_count,
                          void* workspace, long workspace_bytes, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return SB_OK;
  if (K <= 0 || a_fmt < 0 || a_fmt > 1 || b_fmt < 0 || b_fmt > 1) return SB_ERR_BAD_ARG;
  if (out_dtype != SB_DT_BF16 && out_dtype != SB_DT_F32) return SB_ERR_BAD_ARG;
  if ((lda % 16) || (ldb % 16)) return SB_ERR_BAD_ARG;  // TMA: strides are multiples of 16 bytes
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return SB_ERR_BAD_ARG;
  int shape = 128, splits = 1;
  const bool ws_ok = workspace && (reinterpret_cast<uintptr_t>(workspace) & 15) == 0;
  // a k-block of 128 bytes costs what a 16-bit k-block costs: choose tile and split as for a problem of K / 2
  choose_shape(M, N, (K + 1) / 2, 0, 0, sm_count, ws_ok ? workspace_bytes : 0, &shape, &splits);
  const int bn = shape == 128 ? 128 : 256;
  const int b_rows = shape == 512 ? 128 : bn;
  CUtensorMap tmA, tmB, tmC, tmP;
  int rc;
  if ((rc = make_tmap_2d(&tmA, A, M, K, lda, BM, 2))) return rc;
  if ((rc = make_tmap_2d(&tmB, B, N, K, ldb, b_rows, 2))) return rc;
  GemmParams p = {};
  p.C = C; p.C_pre = nullptr; p.bias = bias; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.act = 0;
  p.accumulate = accumulate; p.ab_fmt = 1; p.a8_fmt = a_fmt; p.b8_fmt = b_fmt; p.status = status;
  p.splits = splits;
  p.ws_counter = reinterpret_cast<int*>(workspace);
  p.ws_partial = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + WS_COUNTER_BYTES);
  p.tma_store = out_dtype == SB_DT_BF16 && !accumulate && (ldc % 8 == 0) && (reinterpret_cast<uintptr_t>(C) & 15) == 0;
  tmC = tmA;
  tmP = tmA;
  if (p.tma_store && (rc = make_tmap_out(&tmC, C, M, N, ldc, 0))) return rc;
  if (out_dtype == SB_DT_F32) {
    if (shape == 512) return launch_gemm<256, false, false, float, true, false, true>(tmA, tmB, tmC, tmP, p, sm_count, stream);
    if (shape == 256) return launch_gemm<256, false, false, float, false, false, true>(tmA, tmB, tmC, tmP, p, sm_count, stream);
    return launch_gemm<128, false, false, float, false, false, true>(tmA, tmB, tmC, tmP, p, sm_count, stream);
  }
  using T = __nv_bfloat16;
  if (shape == 512) return launch_gemm<256, false, false, T, true, false, true>(tmA, tmB, tmC, tmP, p, sm_count, stream);
  if (shape == 256) return launch_gemm<256, false, false, T, false, false, true>(tmA, tmB, tmC, tmP, p, sm_count, stream);
  return launch_gemm<128, false, false, T, false, false, true>(tmA, tmB, tmC, tmP, p, sm_count, stream);
}

// Same without a split-K workspace.
SB_API int sb200_gemm(const void* A, const void* B, void* C, void* C_pre, const void* bias, int M, int N, int K,
                      long lda, long ldb, long ldc, int a_mn, int b_mn, int act, int accumulate, int in_dtype,
                      int out_dtype, int bn_hint, int sm_count, int* status, cudaStream_t stream) {
  return sb200_gemm_ws(A, B, C, C_pre, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, act, accumulate, in_dtype, out_dtype,
                       bn_hint, 0, sm_count, nullptr, 0, status, stream);
}

// Tensor-parallel GEMMs with the collective inside the kernel.  All ranks of the group call this with the same
// shapes and mode and their own operands.  The buffers behind partial_ptrs / out_ptrs / flag_ptrs are symmetric
// allocations mapped into every process (tables of W device pointers in host memory, entry r = rank r's buffer);
// flags: (W + 2) * flag_stride uint32, zero before the first use, flag_stride >= number of 128-row output tiles;
// partial_mc / out_mc: multicast addresses or null; epoch, done_ctas: one uint32 each in local device memory, zero
// before the first use.  bias is given on one rank only in modes 0 and 1 (it is added once to the sum).
// The buffers behind partial_ptrs hold 2 * half_elems elements: two buffers that consecutive launches on a workspace
// use in turn (half = 0, 1, 0, ... on every rank alike).  sync_entry = 1 (with half = 0) starts the alternation anew,
// e.g. at the start of a training step; that launch first waits until all ranks have entered it.
//   mode 0 (all-reduce):     out_ptrs[rank][M, ldc] = sum_r A_r[M, K] op(B_r); partial: [M, ldc] per rank.
//   mode 1 (reduce-scatter): C[M / W, ldc] = rows [rank * M / W, ...) of that sum (C is local memory).
//   mode 2 (all-gather):     C[M, ldc] = act([A_0; A_1; ...; A_{W-1}] op(B) + bias) with A_r the [M / W, K] shard
//                            given as A on rank r; the gathered operand is left in partial_ptrs[rank] ([M, K]).
// Modes 1 and 2 need M to be a multiple of W * 128 rows.
SB_API int sb200_gemm_tp(const void* A, const void* B, void* C, void* C_pre, const void* bias, int M, int N, int K,
                         long lda, long ldb, long ldc, int b_mn, int act, int in_dtype, int mode,
                         void* const* partial_ptrs, void* const* out_ptrs, void* const* flag_ptrs, void* partial_mc,
                         void* out_mc, int flag_stride, uint32_t* epoch, unsigned int* done_ctas, int rank, int W,
                         long half_elems, int half, int sync_entry, double timeout_seconds, int sm_count, int* status,
                         cudaStream_t stream) {
  if (M <= 0 || N <= 0) return SB_OK;
  if (K <= 0 || W < 1 || W > AR_MAX_RANKS || rank < 0 || rank >= W) return SB_ERR_BAD_ARG;
  if (half < 0 || half > 1 || half_elems < 0 || (half_elems & 7)) return SB_ERR_BAD_ARG;
  if ((long)M * (mode == AR_ALLGATHER ? K : ldc) > half_elems && half_elems > 0) return SB_ERR_TOO_LARGE;
  if (in_dtype != SB_DT_BF16 || mode < 0 || mode > 2) return SB_ERR_BAD_ARG;
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (N % 8) || (K % 8)) return SB_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return SB_ERR_BAD_ARG;
  const bool pair = M > BM && N > 128;
  const int bn = pair ? 256 : 128;
  const int rows = pair ? 2 * BM : BM;
  const int m_tiles = (M + rows - 1) / rows, n_tiles = (N + bn - 1) / bn;
  const long ctiles = (long)m_tiles * n_tiles * (pair ? 2 : 1);
  if (ctiles > flag_stride) return SB_ERR_TOO_LARGE;
  if (mode != AR_ALLREDUCE && (M % (W * BM))) return SB_ERR_BAD_ARG;  // a 128-row block belongs to one rank
  if (mode == AR_ALLGATHER && (long)(M / W / BM) * GATHER_MAX_GROUPS > flag_stride) return SB_ERR_TOO_LARGE;
  GemmParams p = {};
  p.bias = bias; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.accumulate = 0; p.ab_fmt = 1; p.status = status;
  p.splits = 1; p.ws_counter = nullptr; p.ws_partial = nullptr; p.tma_store = 1;
  const void* a_operand = A;
  long a_ld = lda;
  if (mode == AR_ALLGATHER) {
    p.C = C; p.C_pre = C_pre; p.act = act;
    a_operand = partial_ptrs[rank];  // the gathered [M, K] operand
    a_ld = K;
    if (C_pre && (reinterpret_cast<uintptr_t>(C_pre) & 15)) return SB_ERR_BAD_ARG;
  } else {
    p.C = partial_ptrs[rank]; p.C_pre = nullptr; p.act = 0;
    if (mode == AR_REDUCE_SCATTER && (!C || (reinterpret_cast<uintptr_t>(C) & 15))) return SB_ERR_BAD_ARG;
  }
  if (!p.C || (reinterpret_cast<uintptr_t>(p.C) & 15)) return SB_ERR_BAD_ARG;
  for (int q = 0; q < AR_MAX_RANKS; ++q) {
    p.ar.partial[q] = q < W ? partial_ptrs[q] : nullptr;
    p.ar.out[q] = q < W && out_ptrs ? out_ptrs[q] : nullptr;
    p.ar.flags[q] = q < W ? reinterpret_cast<uint32_t*>(flag_ptrs[q]) : nullptr;
  }
  if (mode == AR_REDUCE_SCATTER) p.ar.out[rank] = C;
  p.ar.partial_mc = partial_mc; p.ar.out_mc = out_mc; p.ar.epoch = epoch; p.ar.done_ctas = done_ctas;
  // Pushing through the switch's multicast sends every byte over NVLink once, whatever the group size, this GPU's own
  // copy included; with two ranks the plain peer store moves the same bytes and keeps the local copy off the link
  // (measured: 207 us against 235 us for a 4096 x 4096 x 5504 problem).
  if (mode == AR_ALLGATHER && W <= 2) p.ar.partial_mc = nullptr;
  p.ar.flag_stride = flag_stride; p.ar.rank = rank; p.ar.W = W;
  p.ar.half_elems = half_elems; p.ar.half = half; p.ar.sync_entry = sync_entry;
  p.ar.mode = mode; p.ar.shard_rows = mode == AR_ALLREDUCE ? M : M / W; p.ar.ld_out = ldc;
  p.ar.a_src = A; p.ar.lda_src = lda;
  // reduce-scatter: a rank multiplies its own rows last, so that the tiles it has to reduce arrive from the peers
  // while it is still busy; all-gather: it starts with its own rows, which are there first
  const int tiles_per_rank = (m_tiles / W) * n_tiles;
  p.ar.unit_shift = mode == AR_REDUCE_SCATTER ? ((rank + 1) % W) * tiles_per_rank
                  : mode == AR_ALLGATHER ? rank * tiles_per_rank : 0;
  if (timeout_seconds <= 0.0) timeout_seconds = 10.0;
  if (timeout_seconds > 60.0) timeout_seconds = 60.0;  // longest wait a kernel may spin
  p.ar.timeout_ns = (unsigned long long)(timeout_seconds * 1e9);
  CUtensorMap tmA, tmB, tmC, tmP, tmA2;
  int rc;
  if ((rc = make_tmap_2d(&tmA, a_operand, M, K, a_ld, BM, 0))) return rc;
  tmA2 = tmA;
  if (mode == AR_ALLGATHER &&  // the gathered operand in the second buffer
      (rc = make_tmap_2d(&tmA2, reinterpret_cast<const uint16_t*>(a_operand) + half_elems, M, K, a_ld, BM, 0)))
    return rc;
  if (b_mn) rc = make_tmap_2d(&tmB, B, K, N, ldb, 64, 0);
  else rc = make_tmap_2d(&tmB, B, N, K, ldb, pair ? 128 : bn, 0);
  if (rc) return rc;
  if ((rc = make_tmap_out(&tmC, p.C, M, N, ldc, 0))) return rc;
  tmP = tmC;
  if (p.C_pre && (rc = make_tmap_out(&tmP, p.C_pre, M, N, ldc, 0))) return rc;
  if (mode != AR_ALLGATHER &&  // partial tiles in the second buffer
      (rc = make_tmap_out(&tmP, reinterpret_cast<uint16_t*>(p.C) + half_elems, M, N, ldc, 0)))
    return rc;
  using T = __nv_bfloat16;
  if (pair) {
    if (b_mn) return launch_gemm<256, false, true, T, true, true>(tmA, tmB, tmC, tmP, p, sm_count, stream, &tmA2);
    return launch_gemm<256, false, false, T, true, true>(tmA, tmB, tmC, tmP, p, sm_count, stream, &tmA2);
  }
  if (b_mn) return launch_gemm<128, false, true, T, false, true>(tmA, tmB, tmC, tmP, p, sm_count, stream, &tmA2);
  return launch_gemm<128, false, false, T, false, true>(tmA, tmB, tmC, tmP, p, sm_count, stream, &tmA2);
}
