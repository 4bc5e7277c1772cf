// Weight-gradient kernel of the mask-based sparse convolution (and the gather-gather
// "ShuffleAB" GEMM) for sm_100a.
//
//   dW[k, f, c] = alpha * sum_r dout[o_r, k] * X[idx[f, o_r], c] + beta * dW_prev[k, f, c]
//
// The reduction runs over (sorted) rows, so both tcgen05 operands are gathered rows held
// "MN-major": a gathered row is 128-byte-swizzled along its channels and the 128 rows of a
// tile are the K dimension of the MMA.  Work is cut into units (filter offset f, range of
// row tiles); a unit accumulates in TMEM, leaves one fp32 partial [128 x BLOCK_N] in the
// workspace and counts itself in; the unit that completes an offset sets the offset's ready flag.
// The partials of an offset are summed in unit order (the result does not depend on timing)
// by CTAs that have finished their own units and wait, bounded, for that flag: an offset with few
// units by one CTA (the offsets are dealt out over the grid); an offset with many units (the
// centre of a submanifold convolution has one per CTA) by all CTAs, each taking a fixed share
// of the tile's positions.  One launch, no atomics on data.  The wait
// is the only place where a CTA depends on others: like every wait in this library it gives up
// after a second and reports through the status word, and the launcher keeps the grid within
// the number of SMs so that all CTAs run at once (the reference serialises split-K slices through
// an unbounded spinning semaphore, cumm/conv/kernel.py:960-1083).
//
// Semantics follow cumm/gemm/blockmma/mma.py:608-648,722-740 (a row takes part for
// offset f iff the reduced-mask word covering it has bit f), cumm/conv/sparse_iters.py
// :284-316 (A = dout[mask_argsort[r]], B = X[indices[f, mask_argsort[r]]], -1 -> zeros)
// and cumm/conv/kernel.py:890-897 (offsets outside mask_filter are left untouched).
#pragma once
#include "ptx.cuh"
#include "rowconv_kernel.cuh"

namespace cb2 {

enum : int { kWgradMaskConv = 0, kWgradPairList = 1 };
// Row-gather implementations: 16-byte cp.async per chunk, or TMA tile::gather4, four rows per
// request (a row coordinate of -1 is out of bounds and reads as zeros).
enum : int { kGatherCpAsync = 0, kGatherTma4 = 2 };

struct WgradParams {
  const void *dout;        // A rows [*, m_total]  (fp16)
  const void *x;           // B rows [*, n_total]  (fp16)
  const int32_t *indices;  // [kv, n_rows]
  const uint32_t *rmask;   // reduced masks: `words` words (32 filter offsets each) per mask_width sorted rows
  const int32_t *argsort;  // [n_rows]
  const int32_t *a_inds;   // pair-list mode
  const int32_t *b_inds;   //   "
  float *partials;         // workspace: [unit][m_tile][n_tile][128 x BLOCK_N] fp32
  int *ctl;                // workspace, zero between calls: [0] CTAs that have left; [9 + 8 by, 13 + 8 by) bit
                           // masks of the ready offsets of output tile by; from kWgradCtlBase on, per
                           // (f, by) at a pitch of four ints: units arrived
  int *sched;              // workspace header: [0,128) number of row tiles carrying offset f
  const int *lists;        // workspace: per offset, the ordered list of those tiles
  int list_stride;         // ints between two offsets' lists
  int *status;
  void *out;               // dW
  const void *src;         // source for beta (dW itself unless the caller gave another)
  long long ldo;           // elements between consecutive m rows of out
  long long f_stride;      // elements between consecutive f slices
  float alpha, beta;
  int out_f32;
  long long ld_dout, ld_x;
  int n_rows;
  int a_rows, b_rows;
  int m_total, n_total;
  int kv;
  int mask_width;
  int words;               // mask words per chunk of mask_width rows: ceil(kv / 32)
  int rmask_words;         // chunks the reduced-mask array holds
  uint32_t mask_filter;
  int mode;
};

template <int BLOCK_N, int GATHER> struct WgradCfg {
  static constexpr int SA = 3;
  static constexpr int A_BYTES = 128 * 256;                 // 128 rows x (2 x 128 B): M = 128 channels
  static constexpr int B_BYTES = 128 * 2 * BLOCK_N;         // 128 rows x BLOCK_N fp16
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int TMEM_COLS = 2 * BLOCK_N;
  static constexpr int THREADS = 128 + 32 + SA * 128;       // epilogue, mma, 3 gather groups
  static constexpr int FULL_COUNT = GATHER == kGatherCpAsync ? 128 : 1;
  static constexpr int OFF_STAGES = 0;
  static constexpr int OFF_ROWIDX = SA * STAGE_BYTES;       // SA x 2 buffers x 2 operands x 128 ints
  static constexpr int OFF_SCHED = OFF_ROWIDX + SA * 2 * 2 * 128 * 4;  // this CTA's units, then units per offset
  static constexpr int TILE_CAP = 2048;                      // tiles of one CTA staged in shared memory
  static constexpr int OFF_TILES = OFF_SCHED + 1024 * 4;
  static constexpr int OFF_BARS = OFF_TILES + TILE_CAP * 4;
  static constexpr int OFF_MISC = OFF_BARS + 16 * 8;
  static constexpr int SMEM_BYTES = OFF_MISC + 64 + 1024;
};

// Does row tile `tile` (sorted rows [128*tile, 128*tile + 128)) carry filter offset f?  OR of the
// reduced-mask words of offset f's group of 32 over the chunks that cover the tile.
__device__ __forceinline__ bool wgrad_tile_has(const WgradParams &p, int tile, int f) {
  if (p.mode != kWgradMaskConv)
    return true;
  if (!((p.mask_filter >> (f & 31)) & 1u))
    return false;
  const uint32_t *col = p.rmask + (f >> 5);
  if (p.mask_width == 128)  // the usual case: one chunk per tile
    return tile < p.rmask_words && ((__ldg(col + (long long)tile * p.words) >> (f & 31)) & 1u);
  const int r0 = tile * 128;
  int r1 = r0 + 127;
  if (r1 >= p.n_rows)
    r1 = p.n_rows - 1;
  int w0 = r0 / p.mask_width, w1 = r1 / p.mask_width;
  uint32_t v = 0;
  for (int w = w0; w <= w1; ++w)
    if (w < p.rmask_words)
      v |= __ldg(col + (long long)w * p.words);
  return (v >> (f & 31)) & 1u;
}

// ---------------------------------------------------------------- schedule
// The work is the sequence of all (filter offset f, row tile carrying f) pairs, offsets in
// ascending order, tiles in ascending order inside an offset: T steps in all.  CTA c of G takes
// the steps [c*T/G, (c+1)*T/G) -- every CTA the same number, whatever the offsets' shares --
// and each maximal run of one offset inside a CTA's range is a UNIT: it accumulates in TMEM
// and leaves one fp32 partial.  The units of an offset are consecutive in this numbering, and
// there are at most G + kv - 1 of them.
//
// A small planning kernel (one block per offset) writes, per offset, the count and the ordered
// list of its tiles, and clears the control words; the main kernel derives
// everything else from the kv counts.  The plan depends only on the reduced masks, the row
// count and the mask filter, so a caller that runs the same layer again (the next training
// step) may keep it: see `reuse_plan` in the C ABI.
//   sched[f]                      tiles carrying offset f
//   lists[f * list_stride + k]    the k-th of them

// One warp plans for up to 128 offsets: lane l owns offsets 4l .. 4l+3.
constexpr int kWgradMaxOffsets = 128;
// Exclusive prefix sum, in offset order, of four values per lane; `total` = the sum of all.
__device__ __forceinline__ void wgrad_scan4(const int (&v)[4], int (&excl)[4], int &total) {
  const int lane = (int)lane_id();
  const int mine = v[0] + v[1] + v[2] + v[3];
  int incl = mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d)
      incl += t;
  }
  total = __shfl_sync(0xffffffffu, incl, 31);
  int run = incl - mine;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    excl[j] = run;
    run += v[j];
  }
}
// Given the tile counts of this lane's offsets: P = steps before each offset, T = all steps,
// c_first = CTA holding step P, S = units of the offset, U = units before it.
__device__ __forceinline__ void wgrad_plan_warp(const int (&cnt)[4], int G, int (&P)[4], int &T, int (&c_first)[4],
                                                int (&S)[4], int (&U)[4]) {
  wgrad_scan4(cnt, P, T);
  // the CTA holding step x is the largest c with c*T/G <= x, i.e. ceil((x+1)*G/T) - 1
  auto chunk_of = [&](int x) -> int {
    const int c = (int)((((long long)x + 1) * G + T - 1) / T) - 1;
    return c < G - 1 ? c : G - 1;
  };
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    c_first[j] = 0;
    S[j] = 0;
    if (cnt[j] > 0) {
      c_first[j] = chunk_of(P[j]);
      S[j] = chunk_of(P[j] + cnt[j] - 1) - c_first[j] + 1;
    }
  }
  int total_units;
  wgrad_scan4(S, U, total_units);
}

// One block per filter offset: count and list the tiles that carry it.  Warp w owns a
// contiguous span of tiles, so the list comes out in ascending order with one block-wide
// synchronisation per batch of 1024 * K tiles.
__global__ void __launch_bounds__(1024) wgrad_plan_kernel(const WgradParams p, int *lists, int list_stride, int n_ctl) {
  constexpr int K = 4;  // 4096 tiles per batch
  __shared__ int s_w[32];
  const int f = blockIdx.x;
  // the control words start from zero (every later call leaves them at zero again)
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_ctl; i += gridDim.x * blockDim.x)
    p.ctl[i] = 0;
  const int ntiles = (p.n_rows + 127) / 128;
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  grid_dep_launch();  // the main kernel may set itself up meanwhile; it waits before reading the lists
  int *list = lists + (long long)f * list_stride;
  int running = 0;
  for (int base = 0; base < ntiles; base += 1024 * K) {
    bool on[K];
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int t = base + (wid * K + k) * 32 + lane;
      on[k] = t < ntiles && wgrad_tile_has(p, t, f);
    }
    int mine = 0;
#pragma unroll
    for (int k = 0; k < K; ++k)
      mine += __popc(__ballot_sync(0xffffffffu, on[k]));
    __syncthreads();  // s_w of the previous batch has been read
    if (lane == 0)
      s_w[wid] = mine;
    __syncthreads();
    int before = 0, all = 0;
    for (int w = 0; w < 32; ++w) {
      const int v = s_w[w];
      all += v;
      if (w < wid)
        before += v;
    }
    int pos = running + before;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const uint32_t bal = __ballot_sync(0xffffffffu, on[k]);
      if (on[k])
        list[pos + __popc(bal & ((1u << lane) - 1u))] = base + (wid * K + k) * 32 + lane;
      pos += __popc(bal);
    }
    running += all;
  }
  if (threadIdx.x == 0)
    p.sched[f] = running;
}

// Per CTA, in shared memory: s_plan[0] = number of units of this CTA, then five ints per unit
// {f, first list index, one past the last, unit number, offset of its tiles in s_tiles};
// s_tiles = the CTA's tiles in step order (when they fit; otherwise the walk reads the lists).
// The unit number is global: the units of an offset are consecutive.  After the unit records:
// s_plan[kWgradPlanUnits + f] = units of offset f over all CTAs, s_plan[kWgradPlanFirst + f] = the
// first of them.
constexpr int kWgradPlanUnits = 8 + 5 * kWgradMaxOffsets;
constexpr int kWgradPlanFirst = kWgradPlanUnits + kWgradMaxOffsets;
constexpr int kWgradPlanInts = kWgradPlanFirst + kWgradMaxOffsets;  // 904 <= the 1024 reserved
constexpr int kWgradMaxOutTiles = 128; // (m, n) tiles of the weight gradient a launch can have
constexpr int kWgradCtlBase = 8 + 8 * kWgradMaxOutTiles;  // first per-(offset, tile) control word
constexpr int kWgradSharedSumUnits = 16;  // offsets with more units than this are summed by all CTAs together
template <int TILE_CAP>
__device__ __forceinline__ void wgrad_load_plan(const WgradParams &p, const int *lists, int list_stride, int *s_plan,
                                                int *s_tiles) {
  const int G = gridDim.x, c = blockIdx.x;
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    int cnt[4], P[4], c_first[4], S[4], U[4], T;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int f = 4 * lane + j;
      cnt[j] = (f < p.kv) ? __ldg(p.sched + f) : 0;
    }
    wgrad_plan_warp(cnt, G, P, T, c_first, S, U);
    const int b0 = (int)(((long long)c * T) / G), b1 = (int)(((long long)(c + 1) * T) / G);
    int has[4], k0[4], k1[4], len[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int f = 4 * lane + j;
      s_plan[kWgradPlanUnits + f] = S[j];
      s_plan[kWgradPlanFirst + f] = U[j];
      has[j] = (cnt[j] > 0 && c >= c_first[j] && c < c_first[j] + S[j]) ? 1 : 0;
      k0[j] = k1[j] = 0;
      if (has[j]) {
        k0[j] = max(b0, P[j]) - P[j];
        k1[j] = min(b1, P[j] + cnt[j]) - P[j];
        if (k1[j] < k0[j])
          k1[j] = k0[j];
      }
      len[j] = k1[j] - k0[j];
    }
    int slot[4], toff[4], n_units, total_len;
    wgrad_scan4(has, slot, n_units);
    wgrad_scan4(len, toff, total_len);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (has[j]) {
        int *e = s_plan + 8 + 5 * slot[j];
        e[0] = 4 * lane + j;
        e[1] = k0[j];
        e[2] = k1[j];
        e[3] = U[j] + (c - c_first[j]);
        e[4] = toff[j];
      }
    if (lane == 0) {
      s_plan[0] = n_units;
      s_plan[1] = total_len <= TILE_CAP ? 1 : 0;  // tiles are staged in shared memory
    }
  }
  __syncthreads();
  if (s_plan[1]) {
    const int n = s_plan[0];
    for (int j = 0; j < n; ++j) {
      const int *e = s_plan + 8 + 5 * j;
      const int *src = lists + (long long)e[0] * list_stride + e[1];
      for (int i = threadIdx.x; i < e[2] - e[1]; i += blockDim.x)
        s_tiles[e[4] + i] = __ldg(src + i);
    }
  }
  __syncthreads();
}

// Walk this CTA's units.  on_unit(u, f) at unit start, on_tile(tile, f, first_of_unit) for each
// of its tiles, on_unit_end(u, f, n_tiles).  Every role runs the identical walk.
template <class UnitFn, class TileFn, class EndFn>
__device__ __forceinline__ void wgrad_walk(const int *lists, int list_stride, const int *s_plan, const int *s_tiles,
                                           UnitFn on_unit, TileFn on_tile, EndFn on_unit_end) {
  const int n = s_plan[0];
  const bool staged = s_plan[1] != 0;
  for (int j = 0; j < n; ++j) {
    const int *e = s_plan + 8 + 5 * j;
    const int f = e[0], k0 = e[1], k1 = e[2], u = e[3], toff = e[4];
    if (!on_unit(u, f))
      return;
    const int *src = lists + (long long)f * list_stride + k0;
    for (int i = 0; i < k1 - k0; ++i) {
      const int tile = staged ? s_tiles[toff + i] : __ldg(src + i);
      if (!on_tile(tile, f, i == 0))
        return;
    }
    if (!on_unit_end(u, f, k1 - k0))
      return;
  }
}

template <int BLOCK_N, int GATHER>
__global__ void __launch_bounds__(WgradCfg<BLOCK_N, GATHER>::THREADS, 1)
wgrad_kernel(const __grid_constant__ CUtensorMap tmap_dout, const __grid_constant__ CUtensorMap tmap_x,
             const WgradParams p) {
  using Cfg = WgradCfg<BLOCK_N, GATHER>;
  extern __shared__ uint8_t smem_raw[];
  if (threadIdx.x == 0)
    CB2_TRACE_CTA(0, 0);
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t *smem = smem_raw + pad;
  const uint32_t sbase = raw_addr + pad;
  int *rowidx = reinterpret_cast<int *>(smem + Cfg::OFF_ROWIDX);
  int *s_plan = reinterpret_cast<int *>(smem + Cfg::OFF_SCHED);
  int *s_tiles = reinterpret_cast<int *>(smem + Cfg::OFF_TILES);
  volatile int *misc = reinterpret_cast<volatile int *>(smem + Cfg::OFF_MISC);
  volatile int *abort_flag = misc + 1;
  const uint32_t bars = sbase + Cfg::OFF_BARS;
  auto full_s = [&](int s) { return bars + 8u * s; };
  auto empty_s = [&](int s) { return bars + 8u * (3 + s); };
  auto acc_full = [&](int s) { return bars + 8u * (6 + s); };
  auto acc_empty = [&](int s) { return bars + 8u * (8 + s); };
  const uint32_t final_bar = bars + 8u * 10;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles_n = (p.n_total + BLOCK_N - 1) / BLOCK_N;
  const int mt = blockIdx.y / n_tiles_n, nt = blockIdx.y % n_tiles_n;
  const int m0 = mt * 128, n0 = nt * BLOCK_N;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::SA; ++s) {
      mbar_init(full_s(s), Cfg::FULL_COUNT);
      mbar_init(empty_s(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(acc_full(s), 1);
      mbar_init(acc_empty(s), 128);
    }
    mbar_init(final_bar, 1);
    mbar_init_fence();
    misc[1] = 0;
    misc[2] = misc[3] = misc[4] = misc[5] = 1;
#ifndef CB2_TRACE_WGRAD_CTA
#define CB2_TRACE_WGRAD_CTA 0
#endif
    CB2_TRACE_SELECT(blockIdx.x == CB2_TRACE_WGRAD_CTA);
  }
  if (warp == 4) {
    tmem_alloc(sbase + Cfg::OFF_MISC, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (threadIdx.x == 0)
    CB2_TRACE_EVENT(5, 10, 0);
  grid_dep_launch();  // lets the next kernel on the stream be scheduled as soon as SMs free up
  grid_dep_wait();    // counts and lists come from the planning kernel
  wgrad_load_plan<Cfg::TILE_CAP>(p, p.lists, p.list_stride, s_plan, s_tiles);  // contains __syncthreads
  if (threadIdx.x == 0)
    CB2_TRACE_EVENT(5, 11, 0);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = static_cast<uint32_t>(misc[0]);

  auto fail = [&](int code) {
    *abort_flag = 1;
    if (p.status)
      atomicCAS(p.status, 0, code);
  };
  const int gy = gridDim.y;

  // ---- shared by the epilogue warps and the summing phase at the end
  const int *s_units = s_plan + kWgradPlanUnits;
  const int *s_first = s_plan + kWgradPlanFirst;
  constexpr int kTileF4 = 32 * BLOCK_N;  // float4 per [128 x BLOCK_N] tile
  // partial layout: float4 (col/4, row) at index (col/4) * 128 + row, so that the 32 rows of a
  // warp touch 512 contiguous bytes
  auto partial_of = [&](int u) {
    return reinterpret_cast<float4 *>(p.partials) + ((long long)u * gy + blockIdx.y) * kTileF4;
  };
  auto ctl_of = [&](int f) { return p.ctl + kWgradCtlBase + 4 * ((long long)f * gy + blockIdx.y); };
  // dW[m0 + row, f, n0 + 4 * q .. + 3] from four sums
  auto write_out = [&](int f, int row, int q, float4 v) {
    const int m = m0 + row, n = n0 + 4 * q;
    if (m >= p.m_total || n >= p.n_total)
      return;
    const long long off = (long long)m * p.ldo + (long long)f * p.f_stride + n;
    float r[4] = {v.x, v.y, v.z, v.w};
    if (p.out_f32) {
      float *o = reinterpret_cast<float *>(p.out);
      const float *sp = reinterpret_cast<const float *>(p.src);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[off + j] = (p.beta != 0.f) ? __fmaf_rn(p.alpha, r[j], __fmul_rn(p.beta, sp[off + j])) : __fmul_rn(p.alpha, r[j]);
    } else {
      __half *o = reinterpret_cast<__half *>(p.out);
      const __half *sp = reinterpret_cast<const __half *>(p.src);
      __half h[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float t = (p.beta != 0.f) ? __fmaf_rn(p.alpha, r[j], __fmul_rn(p.beta, __half2float(sp[off + j])))
                                        : __fmul_rn(p.alpha, r[j]);
        h[j] = __float2half_rn(t);
      }
      *reinterpret_cast<uint2 *>(o + off) = *reinterpret_cast<const uint2 *>(h);
    }
  };
  if (warp < 4) {
    // ======================= epilogue: one fp32 partial per unit; the unit that completes an
    // offset marks it ready for the summing phase
    const int et = threadIdx.x;
    // Offsets inside the filter that no row tile carries get alpha * 0 + beta * source; CTA c
    // takes those with f = c (mod G).
    for (int f = blockIdx.x; f < p.kv; f += gridDim.x)
      if ((p.mode != kWgradMaskConv || ((p.mask_filter >> (f & 31)) & 1u)) && s_units[f] == 0)
        for (int q = 0; q < BLOCK_N / 4; ++q)
          write_out(f, et, q, make_float4(0.f, 0.f, 0.f, 0.f));
    int acc_use = 0;
    wgrad_walk(
        p.lists, p.list_stride, s_plan, s_tiles, [&](int, int) -> bool { return true; },
        [&](int, int, bool) -> bool { return true; },
        [&](int u, int f, int active) -> bool {
          float4 *dst = partial_of(u) + et;
          if (active == 0) {
            // a unit without tiles (fewer steps than CTAs) still owns a partial: all zeros
            for (int q = 0; q < BLOCK_N / 4; ++q)
              dst[q * 128] = make_float4(0.f, 0.f, 0.f, 0.f);
          } else {
            const int buf = acc_use & 1;
            if (et == 0) {
              CB2_TRACE_EVENT(4, 7, u);
              bool ok = mbar_wait(acc_full(buf), (acc_use >> 1) & 1, abort_flag);
              CB2_TRACE_EVENT(4, 8, u);  // accumulator complete
              misc[2] = ok ? 1 : 0;
              if (!ok)
                fail(kStatusWaitTimeout);
            }
            named_bar_sync(1, 128);
            if (misc[2] == 0)
              return false;
            tc_fence_after();
            const uint32_t trow = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) +
                                  static_cast<uint32_t>(buf * BLOCK_N);
#pragma unroll 1
            for (int round = 0; round < BLOCK_N / 32; ++round) {
              uint32_t v[32];
              tmem_ld32(trow + round * 32, v);
              tmem_ld_wait();
#pragma unroll
              for (int q = 0; q < 8; ++q)
                reinterpret_cast<uint4 *>(dst)[(round * 8 + q) * 128] = make_uint4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
            }
            tc_fence_before();
            mbar_arrive(acc_empty(buf));
            ++acc_use;
          }
          // count the unit in; the one that completes the offset marks it ready
          __threadfence();  // this thread's part of the partial is visible before the unit counts
          named_bar_sync(1, 128);
          if (et == 0) {
            if (atomicAdd(ctl_of(f), 1) == s_units[f] - 1) {
              __threadfence();
              atomicOr(p.ctl + 9 + 8 * blockIdx.y + (f >> 5), 1 << (f & 31));  // ready: every partial of f is in place
            }
            CB2_TRACE_EVENT(4, 9, u);  // partial written
          }
          return true;
        });
  } else if (warp == 4) {
    // ======================= MMA issuer
    constexpr uint32_t idesc = make_idesc(0, true, true, 128, BLOCK_N);
    int step = 0, acc_use = 0;
    bool ok_all = true;
    wgrad_walk(
        p.lists, p.list_stride, s_plan, s_tiles, [&](int, int) -> bool { return true; },
        [&](int tile, int f, bool first) -> bool {
          const int buf = acc_use & 1;
          int ok = 1;
          if (lane == 0) {
            if (first)
              ok = mbar_wait(acc_empty(buf), ((acc_use >> 1) & 1) ^ 1, abort_flag);
            const int stage = step % Cfg::SA;
            CB2_TRACE_EVENT(3, 4, step);  // waiting for data
            if (ok)
              ok = mbar_wait(full_s(stage), (step / Cfg::SA) & 1, abort_flag);
            CB2_TRACE_EVENT(3, 5, step);  // data landed
            if (ok) {
              if constexpr (GATHER == kGatherCpAsync)
                fence_proxy_async_smem();
              tc_fence_after();
              const uint32_t a_base = sbase + Cfg::OFF_STAGES + stage * Cfg::STAGE_BYTES;
              const uint32_t b_base = a_base + Cfg::A_BYTES;
              const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BLOCK_N);
              int rows = p.n_rows - tile * 128;
              if (rows > 128)
                rows = 128;
              const int ksteps = (rows + 15) / 16;
              for (int ks = 0; ks < ksteps; ++ks) {
                const uint64_t adesc = make_smem_desc(a_base + ks * 2048, 128 * 128, 1024);
                const uint64_t bdesc = make_smem_desc(b_base + ks * 2048, 128 * 128, 1024);
                tc_mma<0>(d_tmem, adesc, bdesc, idesc, (first && ks == 0) ? 0u : 1u);
              }
              tc_commit(empty_s(stage));
              CB2_TRACE_EVENT(3, 6, step);  // MMAs issued
            }
          }
          ok = __shfl_sync(0xffffffffu, ok, 0);
          ++step;
          if (!ok) {
            if (lane == 0)
              fail(kStatusWaitTimeout);
            ok_all = false;
            return false;
          }
          return true;
        },
        [&](int, int, int active) -> bool {
          if (active > 0) {
            if (lane == 0)
              tc_commit(acc_full(acc_use & 1));
            __syncwarp();
            ++acc_use;
          }
          return true;
        });
    if (lane == 0 && ok_all) {
      tc_commit(final_bar);
      if (!mbar_wait(final_bar, 0, abort_flag))
        fail(kStatusWaitTimeout);
    }
    __syncwarp();
  } else {
    // ======================= gather both operands: group g owns stage g
    const int g = (warp - 5) >> 2;
    const int gt = threadIdx.x - (5 * 32 + g * 128);
    int *group_rowidx = rowidx + g * 512;
    volatile int *my_flag = misc + 3 + g;
    int step = 0;
    const uint8_t *a_bytes = reinterpret_cast<const uint8_t *>(p.dout);
    const uint8_t *b_bytes = reinterpret_cast<const uint8_t *>(p.x);
    constexpr int CPR_B = BLOCK_N / 8;  // 16-byte chunks per B row (fp16)
    wgrad_walk(
        p.lists, p.list_stride, s_plan, s_tiles, [&](int, int) -> bool { return true; },
        [&](int tile, int f, bool) -> bool {
          const bool mine = (step % Cfg::SA) == g;
          const int use = step / Cfg::SA;
          ++step;
          if (!mine)
            return true;
          const int r = tile * 128 + gt;
          int ia = -1, ib = -1;
          if (r < p.n_rows) {
            if (p.mode == kWgradMaskConv) {
              const uint32_t word = __ldg(p.rmask + (long long)(r / p.mask_width) * p.words + (f >> 5));
              const int o = __ldg(p.argsort + r);  // independent of `word`: both loads are in flight together
              if ((word >> (f & 31)) & 1u) {
                ib = __ldg(p.indices + (long long)f * p.n_rows + o);
                ia = (ib >= 0) ? o : -1;  // a zero B row makes the A row irrelevant
              }
            } else {
              ia = __ldg(p.a_inds + r);
              ib = __ldg(p.b_inds + r);
            }
            if (ia >= p.a_rows || ib >= p.b_rows) {
              fail(kStatusBadIndex);
              ia = ib = -1;
            }
          }
          const uint32_t a_stage = sbase + Cfg::OFF_STAGES + g * Cfg::STAGE_BYTES;
          const uint32_t b_stage = a_stage + Cfg::A_BYTES;
          if constexpr (GATHER == kGatherCpAsync) {
            if (gt == 0) {
              CB2_TRACE_EVENT(g, 1, step - 1 + (ib == 0x7fffffff));  // indices loaded
              bool ok = mbar_wait(empty_s(g), (use & 1) ^ 1, abort_flag);
              CB2_TRACE_EVENT(g, 2, step - 1);             // stage free
              *my_flag = ok ? 1 : 0;
              if (!ok)
                fail(kStatusWaitTimeout);
            }
            int *ridx_a = group_rowidx + (use & 1) * 256;
            int *ridx_b = ridx_a + 128;
            ridx_a[gt] = ia;
            ridx_b[gt] = ib;
            named_bar_sync(2 + g, 128);
            if (*my_flag == 0)
              return false;
            {
              // A rows: 256 B (128 channels of dout starting at m0), 16 chunks per row
              const int c = gt & 15, row0 = gt >> 4;
              const bool col_ok = (m0 + c * 8) < p.m_total;
              const uint32_t dst_c = a_stage + (c >> 3) * (128 * 128);
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                const int row = row0 + i * 8;
                const int ridx = ridx_a[row];
                const uint32_t dst = dst_c + (row >> 3) * 1024 + (row & 7) * 128 + (((c & 7) ^ (row & 7)) << 4);
                const bool valid = col_ok && ridx >= 0;
                const uint8_t *srcp = valid ? a_bytes + ((long long)ridx * p.ld_dout + m0 + c * 8) * 2 : a_bytes;
                cp_async_16(dst, srcp, valid ? 16u : 0u);
              }
            }
            {
              const int c = gt % CPR_B, row0 = gt / CPR_B;
              constexpr int RSTEP = 128 / CPR_B;
              const bool col_ok = (n0 + c * 8) < p.n_total;
              const uint32_t dst_c = b_stage + (c >> 3) * (128 * 128);
#pragma unroll
              for (int i = 0; i < CPR_B; ++i) {
                const int row = row0 + i * RSTEP;
                const int ridx = ridx_b[row];
                const uint32_t dst = dst_c + (row >> 3) * 1024 + (row & 7) * 128 + (((c & 7) ^ (row & 7)) << 4);
                const bool valid = col_ok && ridx >= 0;
                const uint8_t *srcp = valid ? b_bytes + ((long long)ridx * p.ld_x + n0 + c * 8) * 2 : b_bytes;
                cp_async_16(dst, srcp, valid ? 16u : 0u);
              }
            }
            // async arrive when this thread's copies land; the consumer fences (see rowconv kernel)
            cp_async_mbar_arrive_noinc(full_s(g));
          } else {
            if (gt == 0)
              CB2_TRACE_EVENT(g, 1, step - 1 + (ib == 0x7fffffff));  // indices loaded
            if (!mbar_wait_warp(empty_s(g), (use & 1) ^ 1, abort_flag)) {
              if (lane == 0)
                fail(kStatusWaitTimeout);
              return false;
            }
            if (gt == 0) {
              CB2_TRACE_EVENT(g, 2, step - 1);  // stage free
              mbar_arrive_expect_tx(full_s(g), Cfg::STAGE_BYTES);
            }
            // four rows per request and column block; row -1 reads as zeros
            {
              const int a1 = __shfl_down_sync(0xffffffffu, ia, 1), a2 = __shfl_down_sync(0xffffffffu, ia, 2),
                        a3 = __shfl_down_sync(0xffffffffu, ia, 3);
              const int b1 = __shfl_down_sync(0xffffffffu, ib, 1), b2 = __shfl_down_sync(0xffffffffu, ib, 2),
                        b3 = __shfl_down_sync(0xffffffffu, ib, 3);
              if ((lane & 3) == 0) {
#pragma unroll
                for (int ka = 0; ka < 2; ++ka)
                  tma_gather4(a_stage + ka * (128 * 128) + gt * 128, &tmap_dout, full_s(g), m0 + ka * 64, ia, a1, a2, a3);
#pragma unroll
                for (int kb = 0; kb < BLOCK_N / 64; ++kb)
                  tma_gather4(b_stage + kb * (128 * 128) + gt * 128, &tmap_x, full_s(g), n0 + kb * 64, ib, b1, b2, b3);
              }
            }
          }
          if (gt == 0)
            CB2_TRACE_EVENT(g, 3, step - 1);  // copies issued
          return true;
        },
        [&](int, int, int) -> bool { return true; });
    if constexpr (GATHER == kGatherCpAsync)
      cp_async_wait_all();
  }

  // ---------------------------------------------------------------- summing
  // Every role has finished its walk; the whole CTA now sums partials.  Each output element is
  // summed by one thread in unit order -- for the offsets with many units: by sixteen warps, each
  // over every sixteenth unit, whose sums are combined in warp order.
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0)
    CB2_TRACE_CTA(2, global_timer_ns());  // roles done
  if (*abort_flag == 0) {
    const int tid = threadIdx.x;
    float4 *s_part = reinterpret_cast<float4 *>(smem + Cfg::OFF_STAGES);  // the operand stages are idle now
    const long long ustride = (long long)gy * kTileF4;
    // this CTA's share of the offsets with many units: positions [c, c + 1) * kTileF4 / G in runs of 32
    const int q_begin = (int)(((long long)blockIdx.x * kTileF4) / gridDim.x) & ~31;
    const int q_end = blockIdx.x + 1 == gridDim.x ? kTileF4 : ((int)(((long long)(blockIdx.x + 1) * kTileF4) / gridDim.x) & ~31);
    // Which offsets this CTA helps to sum, and which positions of each: worked out once, by one
    // thread per offset, and packed in offset order (a CTA takes part in two or three offsets; a loop
    // over all of them, with its divisions run by every thread, cost more than the sums themselves).
    int *s_take = reinterpret_cast<int *>(smem + Cfg::OFF_ROWIDX);  // the row-index buffers are idle now
    {
      bool take = false;
      int lo = 0, hi = 0;
      unsigned ballot = 0;
      if (tid < 128) {
        const int f = tid;
        if (f < p.kv && s_units[f] > 0) {
          if (s_units[f] > kWgradSharedSumUnits) {
            lo = q_begin, hi = q_end;
            take = q_begin < q_end;
          } else {
            // an offset with few units belongs to a small group of neighbouring CTAs (the groups are
            // dealt out evenly over the grid), each summing an equal run of positions
            const int group = max(1, (int)gridDim.x / p.kv);
            const int member = (int)blockIdx.x - (f * (int)gridDim.x) / p.kv;
            take = member >= 0 && member < group;
            lo = ((member * kTileF4) / group) & ~1;
            hi = member + 1 == group ? kTileF4 : (((member + 1) * kTileF4) / group) & ~1;
          }
        }
        ballot = __ballot_sync(0xffffffffu, take);
        if (lane == 0)
          s_take[384 + warp] = static_cast<int>(ballot);
      }
      __syncthreads();
      if (tid < 128 && take) {
        int rank = __popc(ballot & ((1u << lane) - 1u));
        for (int w = 0; w < warp; ++w)
          rank += __popc(static_cast<uint32_t>(s_take[384 + w]));
        s_take[rank] = tid;
        s_take[128 + rank] = lo;
        s_take[256 + rank] = hi;
      }
      __syncthreads();
    }
    const int n_take = __popc(static_cast<uint32_t>(s_take[384])) + __popc(static_cast<uint32_t>(s_take[385])) +
                       __popc(static_cast<uint32_t>(s_take[386])) + __popc(static_cast<uint32_t>(s_take[387]));
    for (int i = 0; i < n_take; ++i) {
      const int f = s_take[i], lo = s_take[128 + i], hi = s_take[256 + i];
      const int S = s_units[f];
      const bool shared_sum = S > kWgradSharedSumUnits;
      if (tid == 0) {
        // bounded wait for the last unit of f
        const int *flag = p.ctl + 9 + 8 * blockIdx.y + (f >> 5);
        int ok = 1;
        unsigned long long t0 = 0;
        for (unsigned spin = 0; !((static_cast<uint32_t>(ld_acquire_gpu(flag)) >> (f & 31)) & 1u); ++spin) {
          __nanosleep(100);
          if ((spin & 63u) == 63u) {
            const unsigned long long now = global_timer_ns();
            if (t0 == 0)
              t0 = now;
            else if (now - t0 > kWaitLimitNs) {
              ok = 0;
              break;
            }
          }
        }
        if (!ok)
          fail(kStatusWaitTimeout);
        misc[6] = ok;
        CB2_TRACE_EVENT(6, 20, f);  // offset ready
      }
      __syncthreads();
      const bool ok = misc[6] != 0;
      __syncthreads();  // everybody has read the result before thread 0 writes the next one
      if (!ok)
        break;
      const float4 *src = partial_of(s_first[f]);
      if (!shared_sum) {
        // two positions per thread at a time, all units' loads of both in flight together
        for (int q0 = lo + 2 * tid; q0 < hi; q0 += 2 * Cfg::THREADS) {
          float4 acc[2];
#pragma unroll
          for (int g = 0; g < 2; ++g)
            acc[g] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
          for (int j = 0; j < S; ++j) {
            const float4 *sp = src + j * ustride + q0;
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              const float4 v = __ldcg(sp + g);
              acc[g].x += v.x;
              acc[g].y += v.y;
              acc[g].z += v.z;
              acc[g].w += v.w;
            }
          }
#pragma unroll
          for (int g = 0; g < 2; ++g)
            write_out(f, (q0 + g) & 127, (q0 + g) >> 7, acc[g]);
        }
      } else {
        for (int q0 = lo; q0 < hi; q0 += 32) {
          if (warp < 16) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 *sp = src + q0 + lane;
#pragma unroll 8
            for (int j = warp; j < S; j += 16) {
              const float4 v = __ldcg(sp + j * ustride);
              acc.x += v.x;
              acc.y += v.y;
              acc.z += v.z;
              acc.w += v.w;
            }
            s_part[warp * 32 + lane] = acc;
          }
          __syncthreads();
          if (warp == 0) {
            float4 acc = s_part[lane];
#pragma unroll
            for (int w = 1; w < 16; ++w) {
              const float4 v = s_part[w * 32 + lane];
              acc.x += v.x;
              acc.y += v.y;
              acc.z += v.z;
              acc.w += v.w;
            }
            const int q = q0 + lane;
            write_out(f, q & 127, q >> 7, acc);
          }
          __syncthreads();
        }
      }
      if (tid == 0)
        CB2_TRACE_EVENT(6, 21, f);  // summed
    }
  }
  // the last CTA to leave puts every control word back to zero for the next call
  if (threadIdx.x == 0) {
    __threadfence();
    misc[6] = atomicAdd(p.ctl, 1) == (int)(gridDim.x * gridDim.y) - 1 ? 1 : 0;
  }
  __syncthreads();
  if (misc[6]) {
    const int n_ctl = kWgradCtlBase + 4 * p.kv * gy;
    for (int i = threadIdx.x; i < n_ctl; i += Cfg::THREADS)
      p.ctl[i] = 0;
    __threadfence();
  }
  if (threadIdx.x == 0)
    CB2_TRACE_CTA(1, 0);
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

} // namespace cb2
