// One-shot sum of per-GPU fp32 arrays over NVLink peer memory, for the weight gradient of the
// row-sharded convolution (1.77 MB for [128, 27, 128]): at that size a library all-reduce is
// all fixed cost.  Every GPU owns a buffer that all GPUs of the node have mapped (the same
// layout on each): a control block, then two sets (by parity of the call number) of one slot
// per GPU.
//
//   push:   GPU r copies its array into slot[parity][r] of EVERY GPU's buffer (plain stores over
//           NVLink: no TMA, no multicast), fences at system scope; the last CTA to finish
//           stores the call number into flag[r] of every GPU's control block.
//   reduce: every CTA waits until all flags of ITS OWN buffer have reached the call number --
//           bounded by `timeout_ns`, after which the kernel records status 1 and returns --
//           then sums its share of the slots in GPU order (the same order on every GPU: the
//           results are bit-identical everywhere) and writes fp32 and/or fp16.
//
// The call number lives in the buffer's control block (read by every CTA at kernel start,
// advanced by the last CTA to finish pushing), not in the launch parameters, so a launch can be
// captured in a CUDA graph and replayed.
// Parity makes the slots safe without any further handshake: a GPU can only push call e+2 after
// it has finished reducing e+1, which needed every GPU's flag e+1, which each GPU stores after
// its own reduce of e.  Flags only grow, so there is nothing to reset.
// All CTAs of the grid must be resident at once (they wait for flags that the grid's own last
// CTA stores): the launcher keeps the grid far below one CTA per SM.
#pragma once
#include "ptx.cuh"
#include "rowconv_kernel.cuh"  // status codes
#include <cuda_fp16.h>

namespace cb2 {

constexpr int kPeerMaxWorld = 16;
constexpr int kPeerControlBytes = 4096;   // flags: one int per GPU at 128-byte pitch; CTA counter at 2048; call number at 2304;
                                          // at 2560 four 64-bit global-timer readings of CTA 0 in the last call: start, pushed, flags seen, done

struct PeerReduceParams {
  unsigned char *peer[kPeerMaxWorld];  // every GPU's buffer as mapped here; peer[rank] is this GPU's own
  const float *src;                    // this GPU's array
  float *out32;                        // may be null
  __half *out16;                       // may be null
  long long numel;                     // multiple of 4
  long long slot_bytes;
  int rank, world;
  unsigned long long timeout_ns;
  int *status;
};

__device__ __forceinline__ int ld_acquire_sys(const int *p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int *p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(512) peer_reduce_kernel(const PeerReduceParams p) {
  __shared__ int s_ok;
  // call number of this launch: the last CTA of the previous launch stored the previous one
  const int epoch = *reinterpret_cast<volatile int *>(p.peer[p.rank] + 2304) + 1;
  const int parity = epoch & 1;
  const long long n4 = p.numel / 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const float4 *src4 = reinterpret_cast<const float4 *>(p.src);
  unsigned long long *stamps = reinterpret_cast<unsigned long long *>(p.peer[p.rank] + 2560);
  if (blockIdx.x == 0 && threadIdx.x == 0)
    stamps[0] = global_timer_ns();
  // ---- push: this GPU's array into its slot on every GPU, nearest neighbour in the ring first
  for (int k = 0; k < p.world; ++k) {
    const int dst = (p.rank + 1 + k) % p.world;
    float4 *slot = reinterpret_cast<float4 *>(p.peer[dst] + kPeerControlBytes +
                                              (static_cast<long long>(parity) * p.world + p.rank) * p.slot_bytes);
    for (long long i = first; i < n4; i += stride)
      slot[i] = src4[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (blockIdx.x == 0)
      stamps[1] = global_timer_ns();
    int *counter = reinterpret_cast<int *>(p.peer[p.rank] + 2048);
    const int done = atomicAdd(counter, 1);
    if (done == static_cast<int>(gridDim.x) - 1) {
      // every CTA of this launch has read the call number by now (it did so before pushing)
      *counter = 0;
      *reinterpret_cast<volatile int *>(p.peer[p.rank] + 2304) = epoch;
      __threadfence_system();
      for (int k = 0; k < p.world; ++k)
        st_release_sys(reinterpret_cast<int *>(p.peer[(p.rank + 1 + k) % p.world] + 128 * p.rank), epoch);
    }
    // ---- wait for every GPU's flag in this GPU's own control block
    bool ok = true;
    unsigned long long t0 = 0;
    for (int r = 0; r < p.world && ok; ++r) {
      const int *flag = reinterpret_cast<const int *>(p.peer[p.rank] + 128 * r);
      for (unsigned spin = 0; ld_acquire_sys(flag) - epoch < 0; ++spin) {
        __nanosleep(100);
        if ((spin & 63u) == 63u) {
          const unsigned long long now = global_timer_ns();
          if (t0 == 0)
            t0 = now;
          else if (now - t0 > p.timeout_ns) {
            ok = false;
            break;
          }
        }
      }
    }
    if (blockIdx.x == 0)
      stamps[2] = global_timer_ns();
    if (!ok && p.status)
      atomicCAS(p.status, 0, kStatusWaitTimeout);
    __threadfence_system();
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok)
    return;
  // ---- reduce: slots in GPU order
  const unsigned char *own = p.peer[p.rank] + kPeerControlBytes + static_cast<long long>(parity) * p.world * p.slot_bytes;
  for (long long i = first; i < n4; i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < p.world; ++r) {
      const float4 v = reinterpret_cast<const float4 *>(own + r * p.slot_bytes)[i];
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    if (p.out32)
      reinterpret_cast<float4 *>(p.out32)[i] = acc;
    if (p.out16) {
      const __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
      reinterpret_cast<uint2 *>(p.out16)[i] =
          make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    stamps[3] = global_timer_ns();
}

} // namespace cb2
