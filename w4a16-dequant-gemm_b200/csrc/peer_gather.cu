// All-gather of the column-parallel GEMM's output slices over NVLink peer memory: the exchange
// step that follows the sharded GEMM (the reference is single-GPU and has no counterpart).
//
// Every rank owns an arena allocated with cudaMalloc and opened by its peers through CUDA IPC.
// One launch per step: CTA p first waits (bounded) until rank p's slice of the step BEFORE THE
// PREVIOUS one has landed here - in steady state it has, long ago - then stores this rank's slice
// into rank p's arena with plain 16-byte peer stores, makes them visible system-wide and posts the
// step number in p's flag array. Ranks therefore stay within two steps of each other and a step
// never waits for a round trip over NVLink. Three slice buffers rotate: step i overwrites the slice
// of step i - 3, and rank p posts step i - 2 only after everything it had queued on its stream for
// the gathered data of step i - 3, so no slice is overwritten while a peer may still read it. A second kernel waits for the slices of the current step (the
// end of a sequence, or whenever the gathered data is needed at once). Step numbers come from a
// device-side counter, so the launches can be replayed from a CUDA graph. No TMA, no multicast,
// no library kernel touches peer memory.
#include "w4b_common.cuh"
#include "w4b_kernels.h"

namespace w4b {
namespace {

// Bounded wait of one thread until *flag >= step; false (and the status word set) when it ran out.
// Once a wait has run out the status word stays set: later waits fail fast instead of taking a
// second each.
__device__ __forceinline__ bool await_flag(const volatile unsigned long long* flag, unsigned long long step,
                                           int* status) {
  const long long t0 = clock64();
  while (*flag < step) {
    if (*reinterpret_cast<volatile int*>(status) != 0) return false;
    __nanosleep(100);
    if (clock64() - t0 > kWaitLimitCycles) {
      atomicExch(status, ST_PEER_TIMEOUT);
      return false;
    }
  }
  __threadfence();  // (kernels that read the slices are ordered after this one by the stream)
  return true;
}

constexpr int PP_THREADS = 1024;

__global__ void __launch_bounds__(PP_THREADS) peer_push_kernel(const PeerPush a) {
  const int p = (int)blockIdx.x;  // the peer this CTA serves
  if (p == a.rank) return;
  const volatile unsigned long long* from_p = reinterpret_cast<const volatile unsigned long long*>(a.flags_local) + p;
  // counters[p]: steps pushed to rank p so far; only this CTA ever writes it
  volatile unsigned long long* ctr = reinterpret_cast<volatile unsigned long long*>(a.counters) + p;
  const unsigned long long step = *ctr + 1ull;
  const uint4* __restrict__ src = reinterpret_cast<const uint4*>(a.src);
  uint4* __restrict__ dst = reinterpret_cast<uint4*>(a.dst[p]);
  // the first two pieces of every thread are loaded before anything is waited for
  const size_t i0 = threadIdx.x, i1 = threadIdx.x + PP_THREADS;
  uint4 v0 = make_uint4(0u, 0u, 0u, 0u), v1 = v0;
  if (i0 < a.n16) v0 = src[i0];
  if (i1 < a.n16) v1 = src[i1];
  if (threadIdx.x == 0 && step > 2) await_flag(from_p, step - 2, a.status);  // rank p is at most two steps behind
  __syncthreads();
  if (i0 < a.n16) dst[i0] = v0;
  if (i1 < a.n16) dst[i1] = v1;
  for (size_t i = i1 + PP_THREADS; i < a.n16; i += 8 * PP_THREADS) {  // the rest of a large slice, eight pieces in flight
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (i + (size_t)u * PP_THREADS < a.n16) v[u] = src[i + (size_t)u * PP_THREADS];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      if (i + (size_t)u * PP_THREADS < a.n16) dst[i + (size_t)u * PP_THREADS] = v[u];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // one system-scope release after the CTA barrier: the slice is visible to rank p before the flag is
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(a.flag_dst[p]), "l"(step) : "memory");
    *ctr = step;
    if (a.wait_now) await_flag(from_p, step, a.status);  // rank p's slice of this step
  }
}

// Waits until every peer's slice of the last pushed step is here.
__global__ void peer_wait_kernel(const void* flags_local, const unsigned long long* counters, int rank, int world,
                                 int* status) {
  const int p = (int)threadIdx.x;
  if (p >= world || p == rank) return;
  const unsigned long long step = *(reinterpret_cast<const volatile unsigned long long*>(counters) + p);
  await_flag(reinterpret_cast<const volatile unsigned long long*>(flags_local) + p, step, status);
}

}  // namespace

// (Launched as a plain stream-ordered kernel: letting the next step's GEMM start beside it - programmatic dependent
// launch - was measured slower, 17.7 against 15.0 us per step on two GPUs.)
cudaError_t peer_push_launch(const PeerPush& p, cudaStream_t stream) {
  peer_push_kernel<<<p.world, PP_THREADS, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t peer_wait_launch(const void* flags_local, const unsigned long long* counters, int rank, int world,
                             int* status, cudaStream_t stream) {
  peer_wait_kernel<<<1, 32, 0, stream>>>(flags_local, counters, rank, world, status);
  return cudaGetLastError();
}

}  // namespace w4b
