// Sum of per-GPU fp32 arrays over NVLink peer memory, for the weight gradient of the row-sharded
// convolution (1.77 MB for [128, 27, 128]): at that size a library all-reduce is all fixed cost,
// and so is every fence and flag round trip over NVLink.  The data therefore carries its own
// flags: a 16-byte line holds two floats, each followed by the call number of the launch that
// wrote it.  An 8-byte half of a line arrives whole or not at all, so a reader that sees the
// current call number beside a float has the float -- no fence at system scope, no counter of
// CTAs and no flag store stands between a store on one GPU and its use on another.  A float4 of
// the array is two neighbouring lines (32 bytes).
// Every GPU owns a buffer that all GPUs of the node have mapped (the same layout on each): a
// control block, then per parity of the call number W receive slots of one shard each, then per
// parity one result array.
//
//   scatter: GPU r cuts its array into W shards and stores shard s, as lines, into receive slot r
//            of GPU s (plain stores over NVLink: no TMA, no multicast).
//   reduce:  GPU s reads the W receive slots of ITS OWN buffer, repeating a load until its lines
//            carry the call number -- bounded by `timeout_ns`, after which the kernel records
//            status 1, stops waiting and runs to its end -- sums in GPU order and stores the sums,
//            as lines, into the result array of EVERY GPU.
//   gather:  every GPU reads the result array in its own buffer the same way and converts it to
//            the fp32 and/or fp16 outputs.
//
// Each element is summed once, by one GPU, in GPU order, and the same sum is delivered to all:
// the results are bit-identical everywhere and do not depend on timing.  A GPU sends and
// receives 2 (W-1)/W of the array, twice over because of the flags.
// The call number lives in the buffer's control block (read by every CTA at kernel start,
// advanced by the last CTA to finish), not in the launch parameters, so a launch can be captured
// in a CUDA graph and replayed.
// Parity makes the buffers safe without any further handshake: a GPU can only finish call e+1
// after it has read every GPU's sums of e+1, which each GPU stores after its own reduce of e+1
// -- and that came after everything it read in call e; so stores of call e+2 never meet a reader
// of call e.  Lines of the same parity left from call e-2 carry another number and read as "not
// yet".  The buffers start out as zeros and the first call has number 1.
// All CTAs of the grid must be resident at once (they wait for lines that other GPUs store only
// after they have seen this GPU's whole scatter).  The launcher bounds the grid by the number of
// SMs; the CTAs are small (128 threads, at most 80 registers).
#pragma once
#include "ptx.cuh"
#include "rowconv_kernel.cuh"  // status codes
#include <cuda_fp16.h>

namespace cb2 {

constexpr int kPeerMaxWorld = 16;
// control block: CTA counter at 2048; call number at 2304; at 2560 six 64-bit global-timer readings
// of thread 0 in the last call (start, scattered, first shard lines seen, reduced, first result
// lines seen, done).
constexpr int kPeerControlBytes = 8192;
constexpr int kPeerThreads = 128;
constexpr int kPeerLineBytesPerF4 = 32;

struct PeerReduceParams {
  unsigned char *peer[kPeerMaxWorld];  // every GPU's buffer as mapped here; peer[rank] is this GPU's own
  const float *src;                    // this GPU's array
  float *out32;                        // may be null
  __half *out16;                       // may be null
  int n4;                              // float4 in the array
  int shard_f4;                        // float4 per shard (the last shard may be shorter)
  long long shard_bytes;               // pitch of a receive slot
  long long result_bytes;              // pitch of a result array
  int rank, world;
  unsigned long long timeout_ns;
  int *status;
};

// a float4 as two lines {x, call, y, call} {z, call, w, call}
__device__ __forceinline__ void peer_store_f4(unsigned char *dst, const float4 &v, int epoch) {
  asm volatile("st.volatile.global.v4.b32 [%0], {%1, %2, %3, %2};" ::"l"(dst), "r"(__float_as_int(v.x)), "r"(epoch),
               "r"(__float_as_int(v.y))
               : "memory");
  asm volatile("st.volatile.global.v4.b32 [%0], {%1, %2, %3, %2};" ::"l"(dst + 16), "r"(__float_as_int(v.z)), "r"(epoch),
               "r"(__float_as_int(v.w))
               : "memory");
}
__device__ __forceinline__ int4 peer_load_line(const unsigned char *src) {
  int4 v;
  asm volatile("ld.volatile.global.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
  return v;
}

// Reads up to N float4 (two lines each) whose loads are all in flight together; a line that does not
// carry `epoch` yet is loaded again until it does or until `timeout_ns` have passed since the first
// miss of this thread (`waited_since`, 0 = none yet).  Returns false on a timeout.
template <int N>
__device__ __forceinline__ bool peer_read_f4(const unsigned char *const (&src)[N], int count, int epoch,
                                             unsigned long long timeout_ns, float4 (&out)[N]) {
  int4 a[N], b[N];
#pragma unroll
  for (int u = 0; u < N; ++u)
    if (u < count) {
      a[u] = peer_load_line(src[u]);
      b[u] = peer_load_line(src[u] + 16);
    }
  bool ok = true;
#pragma unroll
  for (int u = 0; u < N; ++u)
    if (u < count) {
      unsigned long long t0 = 0;
      for (unsigned spin = 1; a[u].y != epoch || a[u].w != epoch || b[u].y != epoch || b[u].w != epoch; ++spin) {
        if ((spin & 15u) == 0) {
          __nanosleep(32);
          const unsigned long long now = global_timer_ns();
          if (t0 == 0)
            t0 = now;
          else if (now - t0 > timeout_ns) {
            ok = false;
            break;
          }
        }
        a[u] = peer_load_line(src[u]);
        b[u] = peer_load_line(src[u] + 16);
      }
      out[u] = make_float4(__int_as_float(a[u].x), __int_as_float(a[u].z), __int_as_float(b[u].x), __int_as_float(b[u].z));
    }
  return ok;
}

__global__ void __launch_bounds__(kPeerThreads, 6) peer_reduce_kernel(const PeerReduceParams p) {
  unsigned char *own = p.peer[p.rank];
  // call number of this launch: the last CTA of the previous launch stored the previous one
  const int epoch = *reinterpret_cast<volatile int *>(own + 2304) + 1;
  const int parity = epoch & 1;
  const int W = p.world;
  const int n4 = p.n4;
  const int stride = static_cast<int>(gridDim.x * blockDim.x);
  const int first = static_cast<int>(blockIdx.x * blockDim.x + threadIdx.x);
  const float4 *src4 = reinterpret_cast<const float4 *>(p.src);
  unsigned long long *stamps = reinterpret_cast<unsigned long long *>(own + 2560);
  const bool lead = first == 0;
  if (lead)
    stamps[0] = global_timer_ns();
  const long long recv_off = kPeerControlBytes + static_cast<long long>(parity) * W * p.shard_bytes;
  const long long result_off = kPeerControlBytes + 2ll * W * p.shard_bytes + static_cast<long long>(parity) * p.result_bytes;
  bool ok = true;

  // ---- scatter: shard s of this GPU's array into receive slot `rank` of GPU s, starting with the next GPU's
  {
    const int shift = ((p.rank + 1) % W) * p.shard_f4;
    for (int i0 = first; i0 < n4; i0 += 4 * stride) {
      float4 v[4];
      int at[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        at[u] = i0 + u * stride;
        if (at[u] < n4) {
          at[u] += shift;
          if (at[u] >= n4)
            at[u] -= n4;
          v[u] = __ldg(src4 + at[u]);
        } else {
          at[u] = -1;
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (at[u] >= 0) {
          const int dst = at[u] / p.shard_f4;
          const int j = at[u] - dst * p.shard_f4;
          peer_store_f4(p.peer[dst] + recv_off + p.rank * p.shard_bytes + static_cast<long long>(j) * kPeerLineBytesPerF4, v[u], epoch);
        }
    }
  }
  if (lead)
    stamps[1] = global_timer_ns();

  // ---- reduce this GPU's shard in GPU order; the sums go to every GPU's result array
  {
    const int lo = p.rank * p.shard_f4;
    const int len = min(p.shard_f4, n4 - lo);
    const unsigned char *recv = own + recv_off;
    for (int j = first; j < len; j += stride) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r0 = 0; r0 < W && ok; r0 += 4) {
        const unsigned char *from[4];
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          from[u] = recv + (r0 + u) * p.shard_bytes + static_cast<long long>(j) * kPeerLineBytesPerF4;
        ok = peer_read_f4<4>(from, W - r0, epoch, p.timeout_ns, v);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (r0 + u < W) {
            acc.x += v[u].x;
            acc.y += v[u].y;
            acc.z += v[u].z;
            acc.w += v[u].w;
          }
      }
      if (lead && j == first)
        stamps[2] = global_timer_ns();
      if (!ok)
        break;
      for (int k = 0; k < W; ++k)
        peer_store_f4(p.peer[(p.rank + 1 + k) % W] + result_off + static_cast<long long>(lo + j) * kPeerLineBytesPerF4, acc, epoch);
    }
  }
  if (lead)
    stamps[3] = global_timer_ns();

  // ---- gather: the sums arrive in this GPU's own result array
  {
    const unsigned char *res = own + result_off;
    for (int i0 = first; i0 < n4 && ok; i0 += 4 * stride) {
      const unsigned char *from[4];
      float4 v[4];
      int count = 0;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        from[u] = res + static_cast<long long>(i0 + u * stride) * kPeerLineBytesPerF4;
        if (i0 + u * stride < n4)
          count = u + 1;
      }
      ok = peer_read_f4<4>(from, count, epoch, p.timeout_ns, v);
      if (lead && i0 == first)
        stamps[4] = global_timer_ns();
      if (!ok)
        break;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * stride;
        if (i >= n4)
          continue;
        if (p.out32)
          reinterpret_cast<float4 *>(p.out32)[i] = v[u];
        if (p.out16) {
          const __half2 lo = __floats2half2_rn(v[u].x, v[u].y), hi = __floats2half2_rn(v[u].z, v[u].w);
          reinterpret_cast<uint2 *>(p.out16)[i] =
              make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
        }
      }
    }
  }
  if (!ok && p.status)
    atomicCAS(p.status, 0, kStatusWaitTimeout);
  __syncthreads();
  if (threadIdx.x == 0) {
    if (lead)
      stamps[5] = global_timer_ns();
    int *counter = reinterpret_cast<int *>(own + 2048);
    // every CTA of this launch read the call number before it counted itself here
    if (atomicAdd(counter, 1) == static_cast<int>(gridDim.x) - 1) {
      *counter = 0;
      *reinterpret_cast<volatile int *>(own + 2304) = epoch;
    }
  }
}

} // namespace cb2
