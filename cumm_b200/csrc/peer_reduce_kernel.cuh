// Sum of per-GPU fp32 arrays over NVLink peer memory, for the weight gradient of the row-sharded
// convolution (1.77 MB for [128, 27, 128]): at that size a library all-reduce is all fixed cost.
// Every GPU owns a buffer that all GPUs of the node have mapped (the same layout on each): a
// control block, then per parity of the call number W receive slots of one shard each, then per
// parity one result array.
//
//   scatter: GPU r cuts its array into W shards and copies shard s into receive slot r of GPU s
//            (plain stores over NVLink: no TMA, no multicast), fences at system scope; the last
//            CTA to finish stores the call number into flag A[r] of every GPU.
//   reduce:  GPU s waits until all flags A of ITS OWN control block have reached the call number
//            -- bounded by `timeout_ns`, after which the kernel records status 1 and returns --
//            sums its shard over the W receive slots in GPU order and stores the sums into the
//            result array of EVERY GPU; the last CTA stores the call number into flag B[s]
//            everywhere.
//   gather:  every GPU waits (bounded) for all flags B and converts the result array, now complete
//            in its own memory, to fp32 and/or fp16 outputs.
//
// Each element is summed once, by one GPU, in GPU order, and the same sum is delivered to all:
// the results are bit-identical everywhere and do not depend on timing.  A GPU sends and
// receives 2 (W-1)/W of the array instead of the (W-1) arrays of an all-to-all push.
// The call number lives in the buffer's control block (read by every CTA at kernel start,
// advanced by the last CTA to finish scattering), not in the launch parameters, so a launch can
// be captured in a CUDA graph and replayed.
// Parity makes the buffers safe without any further handshake: a GPU can only start call e+2
// after it has finished call e+1, which needed every GPU's flag B of e+1, which each GPU stores
// after its own reduce of e+1 -- and that came after everything it read in call e.  Flags only
// grow, so there is nothing to reset.
// All CTAs of the grid must be resident at once (they wait for flags that the grid's own last
// CTA stores).  The CTAs are small (128 threads, few registers) so that they fit beside the
// persistent convolution kernels of the same step, and the launcher bounds the grid by the
// number of SMs.
#pragma once
#include "ptx.cuh"
#include "rowconv_kernel.cuh"  // status codes
#include <cuda_fp16.h>

namespace cb2 {

constexpr int kPeerMaxWorld = 16;
// control block: flags A, one int per GPU at 128-byte pitch [0, 2048); CTA counters at 2048 (scatter) and
// 2112 (reduce); call number at 2304; at 2560 six 64-bit global-timer readings of CTA 0 in the last call
// (start, scattered, shards seen, reduced, results seen, done); flags B at 4096 + 128 * GPU.
constexpr int kPeerControlBytes = 8192;
constexpr int kPeerThreads = 128;

struct PeerReduceParams {
  unsigned char *peer[kPeerMaxWorld];  // every GPU's buffer as mapped here; peer[rank] is this GPU's own
  const float *src;                    // this GPU's array
  float *out32;                        // may be null
  __half *out16;                       // may be null
  long long numel;                     // multiple of 4
  long long shard_f4;                  // float4 per shard (the last shard may be shorter)
  long long shard_bytes;               // pitch of a receive slot
  long long result_bytes;              // pitch of a result array
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

// Waits until the `world` flags at `flags` (128-byte pitch) have all reached `epoch`.
__device__ __forceinline__ bool peer_wait_flags(const unsigned char *flags, int world, int epoch,
                                                unsigned long long timeout_ns) {
  unsigned long long t0 = 0;
  for (int r = 0; r < world; ++r) {
    const int *flag = reinterpret_cast<const int *>(flags + 128 * r);
    for (unsigned spin = 0; ld_acquire_sys(flag) - epoch < 0; ++spin) {
      __nanosleep(64);
      if ((spin & 63u) == 63u) {
        const unsigned long long now = global_timer_ns();
        if (t0 == 0)
          t0 = now;
        else if (now - t0 > timeout_ns)
          return false;
      }
    }
  }
  return true;
}

__global__ void __launch_bounds__(kPeerThreads) peer_reduce_kernel(const PeerReduceParams p) {
  __shared__ int s_ok;
  unsigned char *own = p.peer[p.rank];
  // call number of this launch: the last CTA of the previous launch stored the previous one
  const int epoch = *reinterpret_cast<volatile int *>(own + 2304) + 1;
  const int parity = epoch & 1;
  const int W = p.world;
  const long long n4 = p.numel / 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long first = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const float4 *src4 = reinterpret_cast<const float4 *>(p.src);
  unsigned long long *stamps = reinterpret_cast<unsigned long long *>(own + 2560);
  const bool lead = blockIdx.x == 0 && threadIdx.x == 0;
  if (lead)
    stamps[0] = global_timer_ns();
  const long long recv_off = kPeerControlBytes + static_cast<long long>(parity) * W * p.shard_bytes;
  const long long result_off = kPeerControlBytes + 2ll * W * p.shard_bytes + static_cast<long long>(parity) * p.result_bytes;

  // ---- scatter: shard s of this GPU's array into receive slot `rank` of GPU s, nearest neighbour first
  for (int k = 0; k < W; ++k) {
    const int dst = (p.rank + 1 + k) % W;
    const long long lo = dst * p.shard_f4;
    long long len = n4 - lo;
    if (len > p.shard_f4)
      len = p.shard_f4;
    float4 *slot = reinterpret_cast<float4 *>(p.peer[dst] + recv_off + p.rank * p.shard_bytes);
    for (long long i = first; i < len; i += stride)
      slot[i] = src4[lo + i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (lead)
      stamps[1] = global_timer_ns();
    int *counter = reinterpret_cast<int *>(own + 2048);
    if (atomicAdd(counter, 1) == static_cast<int>(gridDim.x) - 1) {
      // every CTA of this launch has read the call number by now (it did so before scattering)
      *counter = 0;
      *reinterpret_cast<volatile int *>(own + 2304) = epoch;
      __threadfence_system();
      for (int k = 0; k < W; ++k)
        st_release_sys(reinterpret_cast<int *>(p.peer[(p.rank + 1 + k) % W] + 128 * p.rank), epoch);
    }
    // ---- wait for every GPU's shard in this GPU's own receive slots
    const bool ok = peer_wait_flags(own, W, epoch, p.timeout_ns);
    if (lead)
      stamps[2] = global_timer_ns();
    if (!ok && p.status)
      atomicCAS(p.status, 0, kStatusWaitTimeout);
    __threadfence_system();
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok)
    return;

  // ---- reduce this GPU's shard in GPU order; the sums go to every GPU's result array
  {
    const long long lo = p.rank * p.shard_f4;
    long long len = n4 - lo;
    if (len > p.shard_f4)
      len = p.shard_f4;
    const unsigned char *recv = own + recv_off;
    for (long long i = first; i < len; i += stride) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < W; ++r) {
        const float4 v = __ldcg(reinterpret_cast<const float4 *>(recv + r * p.shard_bytes) + i);
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      for (int k = 0; k < W; ++k)
        reinterpret_cast<float4 *>(p.peer[(p.rank + 1 + k) % W] + result_off)[lo + i] = acc;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (lead)
      stamps[3] = global_timer_ns();
    int *counter = reinterpret_cast<int *>(own + 2112);
    if (atomicAdd(counter, 1) == static_cast<int>(gridDim.x) - 1) {
      *counter = 0;
      __threadfence_system();
      for (int k = 0; k < W; ++k)
        st_release_sys(reinterpret_cast<int *>(p.peer[(p.rank + 1 + k) % W] + 4096 + 128 * p.rank), epoch);
    }
    const bool ok = peer_wait_flags(own + 4096, W, epoch, p.timeout_ns);
    if (lead)
      stamps[4] = global_timer_ns();
    if (!ok && p.status)
      atomicCAS(p.status, 0, kStatusWaitTimeout);
    __threadfence_system();
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok)
    return;

  // ---- gather: the complete sums are in this GPU's own result array
  const float4 *res = reinterpret_cast<const float4 *>(own + result_off);
  for (long long i = first; i < n4; i += stride) {
    const float4 acc = __ldcg(res + i);
    if (p.out32)
      reinterpret_cast<float4 *>(p.out32)[i] = acc;
    if (p.out16) {
      const __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
      reinterpret_cast<uint2 *>(p.out16)[i] =
          make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
    }
  }
  if (lead)
    stamps[5] = global_timer_ns();
}

} // namespace cb2
