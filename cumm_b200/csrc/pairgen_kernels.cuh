// Neighbour tables of a sparse convolution, built on the GPU: input-voxel hash table, active
// output voxels of a strided convolution, indices[f, o], neighbour masks, the stable sort of the
// outputs by mask, and the same for the backward direction.
//
// This is the step BEFORE the convolution kernels.  It is not part of cumm itself (its callers
// build these tables with cumm's hash headers, include/tensorview/hash/hash.cu.h:43-263 and
// include/tensorview/hash/ops.h:24-150); the table convention is the one the convolution kernels
// read (include/tensorview/gemm/core/nvrtc_params.h:38-65): indices [kv, N_out] in original row
// order with -1 for a missing neighbour, filter offsets in (z, y, x) row-major order, bit f of a
// row's mask set iff it has a neighbour at offset f, rows sorted by mask value with a STABLE
// sort, active outputs of a strided convolution ordered by their linearised (batch, z, y, x).
// Everything is integer work on HBM-resident arrays: coalesced passes, no tensor cores.
// All loops are bounded: a probe sequence visits at most `capacity` slots and reports a full
// table through the status word instead of spinning.
// None of these kernels triggers programmatic dependent launch (griddepcontrol.launch_dependents):
// the convolution kernels read masks, sort orders and index rows BEFORE their own
// griddepcontrol.wait, which is only sound while whatever wrote those tables has completed in
// the ordinary stream order.  Keep it that way.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace cb2pg {

constexpr unsigned long long kEmptyKey = ~0ULL;
enum : int { kStatusTableFull = 3, kStatusBadCoord = 4 };

struct Geometry {
  int grid[3];    // input grid (z, y, x)
  int ogrid[3];   // output grid
  int ksize[3], stride[3], pad[3], dil[3];
  int kv;
  int batch_size;
};

__device__ __forceinline__ uint32_t mix64(unsigned long long k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdULL;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ULL;
  k ^= k >> 33;
  return static_cast<uint32_t>(k);
}

__device__ __forceinline__ unsigned long long linear_key(int b, int z, int y, int x, const int (&g)[3]) {
  return ((static_cast<unsigned long long>(b) * g[0] + z) * g[1] + y) * g[2] + x;
}

// ---------------------------------------------------------------- hash table: key -> smallest row
__global__ void __launch_bounds__(256) hash_insert_kernel(const int32_t *__restrict__ coords, int n, Geometry g,
                                                          unsigned long long *keys, int *vals, uint32_t cap_mask,
                                                          int *status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n)
    return;
  const int4 c = reinterpret_cast<const int4 *>(coords)[i];
  if (c.x < 0 || c.x >= g.batch_size || c.y < 0 || c.y >= g.grid[0] || c.z < 0 || c.z >= g.grid[1] || c.w < 0 ||
      c.w >= g.grid[2]) {
    atomicCAS(status, 0, kStatusBadCoord);
    return;
  }
  const unsigned long long key = linear_key(c.x, c.y, c.z, c.w, g.grid);
  uint32_t slot = mix64(key) & cap_mask;
  for (uint32_t probe = 0; probe <= cap_mask; ++probe) {
    const unsigned long long prev = atomicCAS(keys + slot, kEmptyKey, key);
    if (prev == kEmptyKey || prev == key) {
      atomicMin(vals + slot, i);  // duplicates resolve to the first row, as a stable sort + search does
      return;
    }
    slot = (slot + 1) & cap_mask;
  }
  atomicCAS(status, 0, kStatusTableFull);
}

__device__ __forceinline__ int hash_find(const unsigned long long *__restrict__ keys, const int *__restrict__ vals,
                                         uint32_t cap_mask, unsigned long long key) {
  uint32_t slot = mix64(key) & cap_mask;
  for (uint32_t probe = 0; probe <= cap_mask; ++probe) {
    const unsigned long long k = __ldg(keys + slot);
    if (k == key)
      return __ldg(vals + slot);
    if (k == kEmptyKey)
      return -1;
    slot = (slot + 1) & cap_mask;
  }
  return -1;
}

// ---------------------------------------------------------------- active outputs of a strided conv
// One thread per input voxel: the output positions that read it, one per filter offset whose
// (in + pad - r * dil) is a multiple of the stride on every axis (for stride 2 that is 8 of the
// 27 offsets; the loops prune whole planes and rows of offsets at once).  New positions are
// appended (unordered) to `list`, one counter update per group of lanes that found one together.
__global__ void __launch_bounds__(256) out_candidates_kernel(const int32_t *__restrict__ coords, int n, Geometry g,
                                                             unsigned long long *set_keys, uint32_t cap_mask,
                                                             unsigned long long *list, int list_cap, int *counter,
                                                             int *status) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n)
    return;
  const int4 c = reinterpret_cast<const int4 *>(coords)[i];
  if (c.x < 0 || c.x >= g.batch_size)
    return;  // reported by the insert kernel
  const int lane = threadIdx.x & 31;
  for (int rz = 0; rz < g.ksize[0]; ++rz) {
    const int nz = c.y + g.pad[0] - rz * g.dil[0];
    if (nz < 0 || nz % g.stride[0] != 0 || nz / g.stride[0] >= g.ogrid[0])
      continue;
    for (int ry = 0; ry < g.ksize[1]; ++ry) {
      const int ny = c.z + g.pad[1] - ry * g.dil[1];
      if (ny < 0 || ny % g.stride[1] != 0 || ny / g.stride[1] >= g.ogrid[1])
        continue;
      for (int rx = 0; rx < g.ksize[2]; ++rx) {
        const int nx = c.w + g.pad[2] - rx * g.dil[2];
        if (nx < 0 || nx % g.stride[2] != 0 || nx / g.stride[2] >= g.ogrid[2])
          continue;
        const unsigned long long key =
            linear_key(c.x, nz / g.stride[0], ny / g.stride[1], nx / g.stride[2], g.ogrid);
        uint32_t slot = mix64(key) & cap_mask;
        bool done = false, fresh = false;
        for (uint32_t probe = 0; probe <= cap_mask && !done; ++probe) {
          const unsigned long long prev = atomicCAS(set_keys + slot, kEmptyKey, key);
          if (prev == key)
            done = true;
          else if (prev == kEmptyKey)
            done = fresh = true;
          else
            slot = (slot + 1) & cap_mask;
        }
        if (!done)
          atomicCAS(status, 0, kStatusTableFull);
        if (fresh) {
          // the lanes that got here together share one counter update
          const unsigned together = __activemask();
          const int leader = __ffs(together) - 1;
          int base = 0;
          if (lane == leader)
            base = atomicAdd(counter, __popc(together));
          base = __shfl_sync(together, base, leader);
          const int at = base + __popc(together & ((1u << lane) - 1u));
          if (at < list_cap)
            list[at] = key;
          else
            atomicCAS(status, 0, kStatusTableFull);
        }
      }
    }
  }
}

__global__ void __launch_bounds__(256) decode_out_coords_kernel(const unsigned long long *__restrict__ keys, int n,
                                                                Geometry g, int32_t *out_coords) {
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= n)
    return;
  unsigned long long k = keys[o];
  const int x = static_cast<int>(k % g.ogrid[2]);
  k /= g.ogrid[2];
  const int y = static_cast<int>(k % g.ogrid[1]);
  k /= g.ogrid[1];
  const int z = static_cast<int>(k % g.ogrid[0]);
  k /= g.ogrid[0];
  reinterpret_cast<int4 *>(out_coords)[o] = make_int4(static_cast<int>(k), z, y, x);
}

// ---------------------------------------------------------------- indices[f, o] and masks
// One thread per output voxel; consecutive threads write consecutive columns of every row of
// the table.  Also writes the row number (the value array of the sort that follows).
__global__ void __launch_bounds__(256) probe_kernel(const int32_t *__restrict__ out_coords, int n_out, Geometry g,
                                                    const unsigned long long *__restrict__ keys,
                                                    const int *__restrict__ vals, uint32_t cap_mask,
                                                    int32_t *indices, uint32_t *mask, int32_t *iota) {
  const int o = blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= n_out)
    return;
  const int4 c = reinterpret_cast<const int4 *>(out_coords)[o];
  uint32_t m = 0;
  int f = 0;
  for (int rz = 0; rz < g.ksize[0]; ++rz) {
    const int z = c.y * g.stride[0] - g.pad[0] + rz * g.dil[0];
    for (int ry = 0; ry < g.ksize[1]; ++ry) {
      const int y = c.z * g.stride[1] - g.pad[1] + ry * g.dil[1];
      for (int rx = 0; rx < g.ksize[2]; ++rx, ++f) {
        const int x = c.w * g.stride[2] - g.pad[2] + rx * g.dil[2];
        int idx = -1;
        if (z >= 0 && z < g.grid[0] && y >= 0 && y < g.grid[1] && x >= 0 && x < g.grid[2])
          idx = hash_find(keys, vals, cap_mask, linear_key(c.x, z, y, x, g.grid));
        indices[static_cast<long long>(f) * n_out + o] = idx;
        if (idx >= 0 && f < 32)
          m |= 1u << f;
      }
    }
  }
  mask[o] = m;
  iota[o] = o;
}

// indices_bwd[f, i] = o for every indices[f, o] = i (the table the input gradient walks)
__global__ void __launch_bounds__(256) invert_table_kernel(const int32_t *__restrict__ indices, int n_out, int kv,
                                                           int n_in, int32_t *indices_bwd) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<long long>(n_out) * kv)
    return;
  const int f = static_cast<int>(t / n_out), o = static_cast<int>(t % n_out);
  const int i = indices[t];
  if (i >= 0 && i < n_in)
    indices_bwd[static_cast<long long>(f) * n_in + i] = o;
}

__global__ void __launch_bounds__(256) mask_from_table_kernel(const int32_t *__restrict__ table, int n, int kv,
                                                              uint32_t *mask, int32_t *iota) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n)
    return;
  uint32_t m = 0;
  for (int f = 0; f < kv && f < 32; ++f)
    if (table[static_cast<long long>(f) * n + j] >= 0)
      m |= 1u << f;
  mask[j] = m;
  iota[j] = j;
}

// Kernel volumes above 32: a row's mask is `words` 32-bit words (word w = offsets 32w .. 32w+31),
// built from the finished table, and rows are sorted as one integer whose LAST word is the most
// significant: one stable radix sort per word, least significant word first, each on the keys
// gathered through the order the previous sorts left.
__global__ void __launch_bounds__(256) mask_words_from_table_kernel(const int32_t *__restrict__ table, int n, int kv,
                                                                    int words, uint32_t *__restrict__ rows) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n)
    return;
  for (int w = 0; w < words; ++w) {
    uint32_t m = 0;
    for (int b = 0; b < 32 && 32 * w + b < kv; ++b)
      if (table[static_cast<long long>(32 * w + b) * n + j] >= 0)
        m |= 1u << b;
    rows[static_cast<long long>(j) * words + w] = m;
  }
}
// key[i] = word w of the row that currently stands at place i; val[i] = that row (order == nullptr:
// the rows are still in their original order)
__global__ void __launch_bounds__(256) gather_word_kernel(const uint32_t *__restrict__ rows, const int32_t *order, int n,
                                                          int words, int w, uint32_t *key, int32_t *val) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n)
    return;
  const int r = order ? order[i] : i;
  key[i] = rows[static_cast<long long>(r) * words + w];
  val[i] = r;
}
// sorted[i, :] = rows[order[i], :]
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint32_t *__restrict__ rows,
                                                          const int32_t *__restrict__ order, int n, int words,
                                                          uint32_t *__restrict__ sorted) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= static_cast<long long>(n) * words)
    return;
  const int i = static_cast<int>(t / words), w = static_cast<int>(t % words);
  sorted[t] = rows[static_cast<long long>(order[i]) * words + w];
}

// A sequence of gather-GEMM-scatter calls (one per filter offset, each with its own pair lists)
// turned into the neighbour table of ONE convolution: table[f, c_inds_f[i]] = a_inds_f[i].
// One thread per pair; `first[f]` = pairs before call f.
constexpr int kSeqMaxCalls = 32;
struct SeqPairLists {
  const int32_t *a_inds[kSeqMaxCalls];  // null = the pair's own position
  const int32_t *c_inds[kSeqMaxCalls];
  long long first[kSeqMaxCalls + 1];
  int count;
};
__global__ void __launch_bounds__(256) seq_scatter_kernel(SeqPairLists L, int n_out, int a_rows, int32_t *__restrict__ table,
                                                          int *status) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= L.first[L.count])
    return;
  int f = 0;
  while (f + 1 < L.count && t >= L.first[f + 1])
    ++f;
  const long long i = t - L.first[f];
  const int o = L.c_inds[f][i];
  const int a = L.a_inds[f] ? L.a_inds[f][i] : (int)i;
  if (o < 0 || o >= n_out || a < 0 || a >= a_rows) {
    atomicCAS(status, 0, 2);  // row index out of range: reported, not dereferenced
    return;
  }
  table[(long long)f * n_out + o] = a;
}

// ---------------------------------------------------------------- stable LSD radix sort, 8 bits per pass
// Three kernels per pass: per-tile digit histograms, one exclusive scan over the (digit, tile)
// matrix, and a scatter in which the warps of a block take turns (in element order) to claim
// their digits' positions, so equal keys keep their order.
constexpr int kSortThreads = 256;
constexpr int kSortItems = 8;
constexpr int kSortTile = kSortThreads * kSortItems;

// Neighbour tables of a DENSE convolution (every grid position is a row, channels last): the
// coordinate rule of the reference's dense iterators, in = out * stride - pad + r * dilation per
// axis (cumm/conv/input_iters.py:2666,2684), written in the layout the row-gather kernels read.
// With them a dense convolution runs through the same kernels as a sparse one whose voxels fill
// the grid.  One thread per (row, filter offset); rows are (batch, z, y, x) row-major.
struct DenseGeometry {
  int batch;
  int in_dims[3], out_dims[3];
  int ksize[3], stride[3], pad[3], dil[3];
  int kv;
};
// forward: indices[f, o] = input row feeding output row o through offset f, or -1
__global__ void __launch_bounds__(256) dense_table_fwd_kernel(DenseGeometry g, long long n_out, int32_t *__restrict__ indices) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_out * g.kv)
    return;
  const int f = (int)(t / n_out);
  const long long o = t % n_out;
  long long rem = o;
  int oc[3];
  for (int a = 2; a >= 0; --a) {
    oc[a] = (int)(rem % g.out_dims[a]);
    rem /= g.out_dims[a];
  }
  const long long b = rem;
  int r[3], fr = f;
  for (int a = 2; a >= 0; --a) {
    r[a] = fr % g.ksize[a];
    fr /= g.ksize[a];
  }
  long long row = b;
  bool ok = true;
  for (int a = 0; a < 3; ++a) {
    const int ic = oc[a] * g.stride[a] - g.pad[a] + r[a] * g.dil[a];
    ok = ok && ic >= 0 && ic < g.in_dims[a];
    row = row * g.in_dims[a] + ic;
  }
  indices[t] = ok ? (int32_t)row : -1;
}
// backward: indices[f, i] = output row that input row i feeds through offset f, or -1
__global__ void __launch_bounds__(256) dense_table_bwd_kernel(DenseGeometry g, long long n_in, int32_t *__restrict__ indices) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_in * g.kv)
    return;
  const int f = (int)(t / n_in);
  const long long i = t % n_in;
  long long rem = i;
  int ic[3];
  for (int a = 2; a >= 0; --a) {
    ic[a] = (int)(rem % g.in_dims[a]);
    rem /= g.in_dims[a];
  }
  const long long b = rem;
  int r[3], fr = f;
  for (int a = 2; a >= 0; --a) {
    r[a] = fr % g.ksize[a];
    fr /= g.ksize[a];
  }
  long long row = b;
  bool ok = true;
  for (int a = 0; a < 3; ++a) {
    const int num = ic[a] + g.pad[a] - r[a] * g.dil[a];
    const int oc = num / g.stride[a];
    ok = ok && num >= 0 && num % g.stride[a] == 0 && oc < g.out_dims[a];
    row = row * g.out_dims[a] + oc;
  }
  indices[t] = ok ? (int32_t)row : -1;
}
// every row carries every offset (the table says which neighbours exist); rows keep their order
__global__ void __launch_bounds__(256) dense_masks_kernel(long long n, int kv, int words, uint32_t *__restrict__ mask,
                                                          int32_t *__restrict__ argsort) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n)
    return;
  argsort[t] = (int32_t)t;
  for (int w = 0; w < words; ++w) {
    const int left = kv - 32 * w;
    mask[t * words + w] = left >= 32 ? 0xffffffffu : (1u << left) - 1u;
  }
}

// OR of the neighbour masks of each run of 128 sorted rows: what the forward kernel reports per
// row tile and the weight gradient reads as its reduced masks.  One warp per tile.
__global__ void __launch_bounds__(256) tile_masks_kernel(const uint32_t *__restrict__ sorted_mask, int n,
                                                         uint32_t *__restrict__ tile_masks) {
  const int tile = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (tile * 128 >= n)
    return;
  uint32_t m = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = tile * 128 + i * 32 + lane;
    if (r < n)
      m |= sorted_mask[r];
  }
  m = __reduce_or_sync(0xffffffffu, m);
  if (lane == 0)
    tile_masks[tile] = m;
}

// the same for several mask words per row: tile_masks[tile, w]
__global__ void __launch_bounds__(256) tile_masks_words_kernel(const uint32_t *__restrict__ sorted_mask, int n, int words,
                                                               uint32_t *__restrict__ tile_masks) {
  const int tile = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (tile * 128 >= n)
    return;
  for (int w = 0; w < words; ++w) {
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = tile * 128 + i * 32 + lane;
      if (r < n)
        m |= sorted_mask[static_cast<long long>(r) * words + w];
    }
    m = __reduce_or_sync(0xffffffffu, m);
    if (lane == 0)
      tile_masks[static_cast<long long>(tile) * words + w] = m;
  }
}

template <typename K>
__global__ void __launch_bounds__(kSortThreads) sort_hist_kernel(const K *__restrict__ keys, int n, int shift,
                                                                 int *hist, int ntiles) {
  __shared__ int h[256];
  h[threadIdx.x] = 0;
  __syncthreads();
  const int base = blockIdx.x * kSortTile;
#pragma unroll
  for (int it = 0; it < kSortItems; ++it) {
    const int idx = base + it * kSortThreads + threadIdx.x;
    if (idx < n)
      atomicAdd(&h[static_cast<int>((keys[idx] >> shift) & 0xff)], 1);
  }
  __syncthreads();
  hist[threadIdx.x * ntiles + blockIdx.x] = h[threadIdx.x];
}

// Exclusive scan, in place, of the (digit, tile) count matrix in digit-major order (all tiles of
// digit 0, then digit 1, ...), `total4` int4 in all (the tail beyond 256 * ntiles is padding whose
// values nobody reads).  One block; every thread owns a contiguous run of int4 that it reads
// twice with several loads in flight: the kernel is a handful of memory latencies long.
__global__ void __launch_bounds__(1024) sort_scan_kernel(int4 *data, int total4) {
  __shared__ int s_sum[1024];
  const int per = (total4 + 1023) / 1024;
  const int lo = min(threadIdx.x * per, total4), hi = min(lo + per, total4);
  int sum = 0;
#pragma unroll 8
  for (int i = lo; i < hi; ++i) {
    const int4 v = data[i];
    sum += v.x + v.y + v.z + v.w;
  }
  // block-wide exclusive scan of the 1024 sums: warp scans, then a scan of the 32 warp totals
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = sum;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d)
      incl += t;
  }
  if (lane == 31)
    s_sum[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const int w = s_sum[lane];
    int wi = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, wi, d);
      if (lane >= d)
        wi += t;
    }
    s_sum[lane] = wi - w;
  }
  __syncthreads();
  int run = s_sum[warp] + incl - sum;
#pragma unroll 8
  for (int i = lo; i < hi; ++i) {
    const int4 v = data[i];
    int4 o;
    o.x = run;
    o.y = run + v.x;
    o.z = o.y + v.y;
    o.w = o.z + v.z;
    run = o.w + v.w;
    data[i] = o;
  }
}

template <typename K, bool HAS_VAL>
__global__ void __launch_bounds__(kSortThreads) sort_scatter_kernel(const K *__restrict__ kin, const int *__restrict__ vin,
                                                                    K *kout, int *vout, int n, int shift,
                                                                    const int *__restrict__ offsets, int ntiles) {
  __shared__ int cnt[256];
  cnt[threadIdx.x] = offsets[threadIdx.x * ntiles + blockIdx.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int base = blockIdx.x * kSortTile;
  for (int it = 0; it < kSortItems; ++it) {
    const int idx = base + it * kSortThreads + threadIdx.x;
    const bool valid = idx < n;
    K key = 0;
    int val = 0;
    if (valid) {
      key = kin[idx];
      if (HAS_VAL)
        val = vin[idx];
    }
    const unsigned digit = valid ? static_cast<unsigned>((key >> shift) & 0xff) : 0x100u + lane;  // invalid: unique
    const unsigned peers = __match_any_sync(0xffffffffu, digit);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    const int leader = __ffs(peers) - 1;
    int claimed = 0;
    for (int w = 0; w < kSortThreads / 32; ++w) {
      __syncthreads();
      if (warp == w && valid && rank == 0) {
        claimed = cnt[digit];
        cnt[digit] = claimed + __popc(peers);
      }
    }
    claimed = __shfl_sync(0xffffffffu, claimed, leader);
    if (valid) {
      kout[claimed + rank] = key;
      if (HAS_VAL)
        vout[claimed + rank] = val;
    }
  }
}

} // namespace cb2pg
