// Data-parallel collectives of the ZeRO-1 optimizer step as plain kernels over NVLink peer memory (sm_100a).
//
// Every rank of the data-parallel group maps the flat gradient and flat parameter buffers of all ranks of the
// group (symmetric allocations: same size and layout everywhere).  The reduce-scatter then is one kernel per rank
// that reads its owned range out of every peer's gradient buffer and adds the pieces in rank order; the
// all-gather is one kernel per rank that stores its updated parameter range into every peer's parameter buffer
// (one multimem store per 16 bytes where the buffers are bound to an NVLink multicast object, so that the switch
// replicates the data).  Ordering between ranks comes from a small barrier kernel on flag words in peer memory.
//
// Behaviour covered (reference): gradient all-reduce / ZeRO partition update and parameter all-gather over the
// data-parallel group (src/scaling/core/optimizer/allreduce.py:16-38,
// src/scaling/core/optimizer/parameter_group.py:439-477).
//
// All waits are bounded: a rank that does not see its peers within the limit records SB_ERR_WAIT_TIMEOUT in
// *status and returns, so the context stays usable and the host can raise.
#include "common.cuh"

namespace {

constexpr int P2P_MAX_RANKS = 16;

struct PeerPtrs {
  void* p[P2P_MAX_RANKS];
};

// Flags: rank r owns an array flags_r[P2P_MAX_RANKS]; flags_r[q] is written by rank q only.  A barrier round
// number lives in local memory and is advanced by the kernel itself, which keeps launches replayable from a graph.
__global__ void p2p_barrier_kernel(PeerPtrs flags, uint32_t* __restrict__ round_word, int rank, int W,
                                   int* __restrict__ status, unsigned long long timeout_ns) {
  __shared__ uint32_t round_s;
  if (threadIdx.x == 0) {
    round_s = *round_word + 1;
    *round_word = round_s;
  }
  __syncthreads();
  const uint32_t round = round_s;
  const int peer = threadIdx.x;
  if (peer >= W) return;
  // everything this GPU wrote before this kernel (earlier kernels of the stream) is ordered before the signal
  __threadfence_system();
  sb::st_release_sys(reinterpret_cast<uint32_t*>(flags.p[peer]) + rank, round);
  const uint32_t* mine = reinterpret_cast<const uint32_t*>(flags.p[rank]) + peer;
  const unsigned long long t0 = sb::globaltimer_ns();
  unsigned spins = 0;
  while ((int32_t)(sb::ld_acquire_sys(mine) - round) < 0) {
    if ((++spins & 0x3ff) == 0 && sb::globaltimer_ns() - t0 > timeout_ns) {
      if (status) *status = SB_ERR_WAIT_TIMEOUT;
      return;
    }
  }
}

// dst[i] = sum over ranks q (ascending) of src_q[offset + i], i in [0, n); 16-byte vectors, fp32 accumulation.
template <typename T>
__global__ void __launch_bounds__(256)
    p2p_reduce_scatter_kernel(PeerPtrs src, T* __restrict__ dst, long offset, long n, int W) {
  constexpr int V = sb::Vec16<T>::N;
  const long nv = n / V;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
    float acc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] = 0.f;
    sb::Vec16<T> v[4];
    for (int q0 = 0; q0 < W; q0 += 4) {  // four peers' loads in flight at a time
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (q0 + j < W) v[j] = sb::ld16(reinterpret_cast<const T*>(src.p[q0 + j]) + offset + i * V);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (q0 + j < W) {
#pragma unroll
          for (int k = 0; k < V; ++k) acc[k] += sb::to_f(v[j].e[k]);
        }
    }
    sb::Vec16<T> o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.e[k] = sb::from_f<T>(acc[k]);
    sb::st16(dst + i * V, o);
  }
  for (long i = nv * V + blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    float a = 0.f;
    for (int q = 0; q < W; ++q) a += sb::to_f(reinterpret_cast<const T*>(src.p[q])[offset + i]);
    dst[i] = sb::from_f<T>(a);
  }
}

__device__ __forceinline__ void multimem_st16(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// Every peer's buffer (and, with a multicast address, all of them at once) receives bytes [offset, offset + n) of
// this rank's buffer.  Byte granularity: offsets and sizes are multiples of 16.
__global__ void __launch_bounds__(256)
    p2p_all_gather_kernel(PeerPtrs dst, const uint8_t* __restrict__ src, uint8_t* __restrict__ mc, long offset, long n,
                          int rank, int W) {
  const long nv = n / 16;
  const uint4* s = reinterpret_cast<const uint4*>(src + offset);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nv; i += (long)gridDim.x * blockDim.x) {
    const uint4 v = s[i];
    if (mc) {
      multimem_st16(mc + offset + i * 16, v);
    } else {
      for (int q = 1; q < W; ++q) {  // start with the next rank so that the ranks do not all hit one peer at once
        const int peer = (rank + q) % W;
        reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(dst.p[peer]) + offset)[i] = v;
      }
    }
  }
}

int fill_ptrs(PeerPtrs* out, void* const* ptrs, int W) {
  if (W < 1 || W > P2P_MAX_RANKS) return SB_ERR_BAD_ARG;
  for (int i = 0; i < P2P_MAX_RANKS; ++i) out->p[i] = i < W ? ptrs[i] : nullptr;
  return SB_OK;
}

}  // namespace

SB_API int sb200_p2p_max_ranks() { return P2P_MAX_RANKS; }

// flag_ptrs: host array of W device pointers, entry q = flag array (P2P_MAX_RANKS uint32, zero-initialised) of rank q
// as mapped on this device.  round_word: one uint32 in local device memory, zero-initialised.
SB_API int sb200_p2p_barrier(void* const* flag_ptrs, uint32_t* round_word, int rank, int W, int* status,
                             double timeout_seconds, cudaStream_t stream) {
  PeerPtrs f;
  int rc = fill_ptrs(&f, flag_ptrs, W);
  if (rc) return rc;
  if (rank < 0 || rank >= W) return SB_ERR_BAD_ARG;
  if (timeout_seconds <= 0.0) timeout_seconds = 10.0;
  if (timeout_seconds > 60.0) timeout_seconds = 60.0;  // longest wait a kernel may spin
  p2p_barrier_kernel<<<1, 32, 0, stream>>>(f, round_word, rank, W, status,
                                           (unsigned long long)(timeout_seconds * 1e9));
  SB_CHECK_LAUNCH();
  return SB_OK;
}

// src_ptrs: host array of W device pointers to the ranks' source buffers (same layout on every rank).
SB_API int sb200_p2p_reduce_scatter(void* const* src_ptrs, void* dst, long offset, long n, int W, int dtype,
                                    int sm_count, cudaStream_t stream) {
  if (n <= 0) return SB_OK;
  PeerPtrs s;
  int rc = fill_ptrs(&s, src_ptrs, W);
  if (rc) return rc;
  SB_DISPATCH_DTYPE(dtype, T, {
    constexpr int V = sb::Vec16<T>::N;
    if (offset % V || (reinterpret_cast<uintptr_t>(dst) & 15)) return SB_ERR_BAD_ARG;
    for (int q = 0; q < W; ++q)
      if (reinterpret_cast<uintptr_t>(src_ptrs[q]) & 15) return SB_ERR_BAD_ARG;
    long blocks = (n / V + 255) / 256;
    if (blocks > sm_count * 8L) blocks = sm_count * 8L;
    if (blocks < 1) blocks = 1;
    p2p_reduce_scatter_kernel<T><<<(int)blocks, 256, 0, stream>>>(s, (T*)dst, offset, n, W);
  });
  SB_CHECK_LAUNCH();
  return SB_OK;
}

// dst_ptrs: host array of W device pointers to the ranks' destination buffers; src = this rank's own buffer;
// multicast: address of the same buffer in the group's multicast mapping, or null to store to each peer in turn.
// offset_bytes and n_bytes are multiples of 16.
SB_API int sb200_p2p_all_gather(void* const* dst_ptrs, const void* src, void* multicast, long offset_bytes, long n_bytes,
                                int rank, int W, int sm_count, cudaStream_t stream) {
  if (n_bytes <= 0 || W <= 1) return SB_OK;
  PeerPtrs d;
  int rc = fill_ptrs(&d, dst_ptrs, W);
  if (rc) return rc;
  if ((offset_bytes | n_bytes) & 15 || (reinterpret_cast<uintptr_t>(src) & 15) ||
      (reinterpret_cast<uintptr_t>(multicast) & 15))
    return SB_ERR_BAD_ARG;
  long blocks = (n_bytes / 16 + 255) / 256;
  if (blocks > sm_count * 4L) blocks = sm_count * 4L;
  if (blocks < 1) blocks = 1;
  p2p_all_gather_kernel<<<(int)blocks, 256, 0, stream>>>(d, (const uint8_t*)src, (uint8_t*)multicast, offset_bytes,
                                                         n_bytes, rank, W);
  SB_CHECK_LAUNCH();
  return SB_OK;
}
