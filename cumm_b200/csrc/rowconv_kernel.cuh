// Row-gather implicit-GEMM kernel for sm_100a: forward and input-gradient of the
// mask-based sparse convolution, and the gather-GEMM-scatter GEMM (one filter offset with
// explicit row lists).  One persistent CTA per SM takes 128-row tiles of the (sorted)
// output rows from a scheduler warp (global ticket counter, ring of tiles in shared memory);
// for every filter offset present in the tile's OR-ed neighbour mask it gathers the 128
// operand rows into a 128-byte-swizzled shared-memory tile (TMA tile::gather4 for rows of up
// to 128 bytes, 16-byte cp.async for wider ones; missing neighbours read as zeros), brings the
// matching weight slice in by TMA, and one thread issues tcgen05.mma into a TMEM accumulator.
// Eight (fp16) or sixteen (int8) epilogue warps read the accumulator back, apply
// alpha/beta/bias/activation (or the int8 requantisation), stage the tile through shared
// memory and write whole rows to their scattered destinations.  No atomics on data: every
// output row is owned by exactly one tile.
//
// What it computes follows the reference kernel's control flow
// (cumm/conv/kernel.py:825-920, cumm/conv/sparse_iters.py:317-356,
// cumm/gemm/mask_iters.py:971-988, cumm/gemm/out_iters.py:541-553); how it computes it
// does not: the reference stages everything through registers and mma.sync.
#pragma once
#include "ptx.cuh"
#include <cuda.h>
#include <cuda_fp16.h>

namespace cb2 {

enum : int { kModeMaskConv = 0, kModeGatherGemm = 1 };
enum : int { kSrcNone = 0, kSrcRows = 1, kSrcVector = 2 };
enum : int { kStatusOk = 0, kStatusWaitTimeout = 1, kStatusBadIndex = 2 };

struct RowConvParams {
  const void *a;      // operand rows to gather  [a_rows, red]
  void *out;          // destination rows        [*, nn]
  const void *src;    // source rows for beta (same indexing as out) or a length-nn vector
  const float *scale; // int8 requantisation, per output channel
  const float *bias;  //   "
  const int32_t *indices;  // [kv, n_rows] (mask-conv mode)
  const uint32_t *mask;    // [n_rows, mask_words] sorted order
  const int32_t *argsort;  // [n_rows]
  uint32_t *mask_out;      // [tiles, mask_words] or null
  const int32_t *a_inds;   // gather-GEMM mode (null = identity)
  const int32_t *c_inds;   //   "
  int *status;             // device status word (0 = ok)
  int *tickets;            // two zero-initialised ints (next ticket, finished CTAs) or null = static round-robin
  long long lda, ldo, lds; // row strides in elements
  int n_rows;              // rows to produce (sorted positions, or m)
  int a_rows;              // rows available in `a`
  int red;                 // reduction width per filter offset
  int nn;                  // output width
  int kv;
  int mask_words;          // 32-bit words per row mask: ceil(kv / 32), word w covers offsets 32w .. 32w+31
  int mode;
  int src_mode;
  int skip_empty_tiles;    // input-gradient: a tile whose mask is 0 is left untouched
  int reverse_mask;
  uint32_t mask_filter;
  float alpha, beta, act_alpha;
  int act_type;
  uint32_t b_lbo, b_sbo;   // weight-tile descriptor offsets (bytes)
};

#ifndef CB2_ROWCONV_GROUP_THREADS
#define CB2_ROWCONV_GROUP_THREADS 128
#endif
#ifndef CB2_ROWCONV_RING
#define CB2_ROWCONV_RING 12
#endif
#ifndef CB2_ROWCONV_STEP_BUDGET
#define CB2_ROWCONV_STEP_BUDGET 12
#endif
#ifndef CB2_ROWCONV_TICKET_BATCH
#define CB2_ROWCONV_TICKET_BATCH 4
#endif
#ifndef CB2_ROWCONV_EPI_PARTS
#define CB2_ROWCONV_EPI_PARTS 4
#endif

// TMA_GATHER: operand rows are fetched by the TMA unit (tile::gather4, four rows per request,
// one warp per group) instead of 16-byte cp.async issued by 128 threads per group.  The copy
// engine path keeps the load/store queues of the SM free for the other roles.
// MASK_WORDS: mask words per row the ring slots have room for (1: kernel volumes up to 32; 4: up
// to 128, the reference's "dynamic mask" kernels, cumm/gemm/blockmma/mma.py:78-270).
template <int KIND, int NATOM_K, int BLOCK_N, bool B_MN, bool TMA_GATHER, int MASK_WORDS = 1> struct RowConvCfg {
  static constexpr int ES = KIND == 0 ? 2 : 1;            // operand element bytes
  static constexpr int OES = KIND == 0 ? 2 : 1;           // output element bytes
  static constexpr int ATOM_ELEMS = 128 / ES;             // elements per 128-byte swizzle row
  static constexpr int UMMA_K = 32 / ES;
  static constexpr int KRED = NATOM_K * ATOM_ELEMS;       // reduction elements per stage
  static constexpr int TILE_M = 128;
  static constexpr int SA = 3;                            // A stages == producer groups
  static constexpr int A_STAGE_BYTES = TILE_M * 128 * NATOM_K;
  static constexpr int B_SLOT_BYTES = BLOCK_N * 128 * NATOM_K;
  static constexpr int OUT_ROW_BYTES = BLOCK_N * OES;
  static constexpr int STAGING_BYTES = TILE_M * OUT_ROW_BYTES;
  static constexpr int MW = MASK_WORDS;
  static constexpr int RING = MASK_WORDS == 1 ? CB2_ROWCONV_RING : CB2_ROWCONV_RING / 2;  // tile ring slots
  static constexpr int RING_SLOT_INTS = 136 + 128 * MASK_WORDS;  // header; 128 gather rows; 128 output rows / row masks
  // Weight slots: as many as fit (2 to 6).  A tile whose mask carries many offsets needs a new
  // weight tile every step, and with two slots the L2 latency of that load bounds the step.
  static constexpr int FIXED_BYTES = SA * A_STAGE_BYTES + STAGING_BYTES + SA * 2 * 128 * 4 + 128 * 4 +
                                     2 * BLOCK_N * 4 + RING * RING_SLOT_INTS * 4 + (32 + 3 * RING) * 8 + 64 + 1024;
  static constexpr int SB_FIT = (232448 - FIXED_BYTES) / B_SLOT_BYTES;
  static constexpr int SB = SB_FIT < 2 ? 2 : (SB_FIT > 6 ? 6 : SB_FIT);
  static constexpr int NUM_ACC = 2;                       // TMEM accumulators: one fills while one drains
  static constexpr int TMEM_COLS = NUM_ACC * BLOCK_N;     // 128 or 256: power of two >= 32
  // Epilogue: several threads per tile row, each converting its share of the columns.  The
  // conversion is a chain of dependent fixed-latency instructions, so its rate is set by how
  // many warps each SM sub-partition can switch between, not by arithmetic throughput.
  static constexpr int EPI_HALVES = (KIND == 1 && BLOCK_N >= 128) ? CB2_ROWCONV_EPI_PARTS : 2;
  static constexpr int EPI_THREADS = 128 * EPI_HALVES;
  static constexpr int GROUP_THREADS = TMA_GATHER ? 32 : CB2_ROWCONV_GROUP_THREADS;
  static constexpr int FULL_A_COUNT = TMA_GATHER ? 1 : GROUP_THREADS;
  static constexpr int MMA_WARP = EPI_THREADS / 32;
  static constexpr int TMA_WARP = MMA_WARP + 1;
  static constexpr int FIRST_GATHER_WARP = TMA_WARP + 1;
  static constexpr int SCHED_WARP = FIRST_GATHER_WARP + SA * GROUP_THREADS / 32;  // the last warp hands out tiles
  static constexpr int THREADS = (SCHED_WARP + 1) * 32;   // 544
  static constexpr int RING_CONSUMER_WARPS = SCHED_WARP;   // every warp but the scheduler
  // shared memory map (offsets from a 1024-byte aligned base)
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + SA * A_STAGE_BYTES;
  static constexpr int OFF_STAGING = OFF_B + SB * B_SLOT_BYTES;
  static constexpr int OFF_ROWIDX = OFF_STAGING + STAGING_BYTES;     // SA * 2 * 128 ints
  static constexpr int OFF_OUTROW = OFF_ROWIDX + SA * 2 * 128 * 4;   // 128 ints
  static constexpr int OFF_SCALE = OFF_OUTROW + 128 * 4;             // 2 * BLOCK_N floats
  static constexpr int OFF_RING = OFF_SCALE + 2 * BLOCK_N * 4;       // RING slots
  static constexpr int OFF_BARS = OFF_RING + RING * RING_SLOT_INTS * 4;  // 32 + 3 * RING mbarriers
  static constexpr int OFF_MISC = OFF_BARS + (32 + 3 * RING) * 8;                 // tmem ptr, abort, flags
  static constexpr int SMEM_BYTES = OFF_MISC + 64 + 1024;            // + alignment slack
  static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA exceeded");
  static_assert(SB <= 8, "barrier table holds eight weight slots");
};

__device__ __forceinline__ float apply_act(float x, int act_type, float act_alpha) {
  switch (act_type) {
  case 1:
    return fmaxf(x, 0.f);
  case 2:
    return 1.f / (1.f + expf(-x));
  case 3:
    return x >= 0.f ? x : x * act_alpha;
  default:
    return x;
  }
}

// Four floats -> four int8 in one word, round-to-nearest-even, saturating, NaN -> 0 (what
// cvt.rni.sat.s8.f32 returns for each): to int32 first (NaN -> 0, saturating at the int32 range),
// then two saturating packs of two values each -- the reference's packed converter
// (include/tensorview/gemm/math/numeric_convert.h:1107-1138).  Six instructions per four values;
// a clamp-and-magic-add form in the arithmetic pipes took eleven and measured 4 % slower on the
// stride-2 int8 convolution: the kernel is bound by instruction issue, not by a pipe.
__device__ __forceinline__ uint32_t cvt_pack4_s8(float a, float b, float c, float d) {
  int ia, ib, ic, id;
  asm("cvt.rni.s32.f32 %0, %1;" : "=r"(ia) : "f"(a));
  asm("cvt.rni.s32.f32 %0, %1;" : "=r"(ib) : "f"(b));
  asm("cvt.rni.s32.f32 %0, %1;" : "=r"(ic) : "f"(c));
  asm("cvt.rni.s32.f32 %0, %1;" : "=r"(id) : "f"(d));
  uint32_t hi, out;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, 0;" : "=r"(hi) : "r"(id), "r"(ic));       // bytes {c, d}
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(ib), "r"(ia), "r"(hi));  // {a, b, c, d}
  return out;
}

// Tiles are handed out by one scheduler warp per CTA through a small shared-memory ring.
// A slot holds {tile, OR-ed neighbour mask of the tile, the 128 rows the gather starts from,
// the 128 destination rows}.  With `tickets` the scheduler draws tiles from a global counter
// (dynamic scheduling: a tile whose mask carries many offsets costs many steps, and a static
// split leaves the CTAs that own such tiles running long after the others), last tiles of
// the sorted order first because those carry the most offsets.
struct RingView {
  int *slots;
  uint32_t full0, empty0;  // addresses of the first "published" / "released" barrier
  uint32_t landed0;        // first "copies landed" barrier (scheduler only)
  int ring, slot_ints;
  volatile int *abort_flag;
  __device__ __forceinline__ int *slot(int i) const { return slots + i * slot_ints; }
};

// OR of the neighbour masks of a tile's rows, word by word, from the raw mask words of its ring
// slot (warp-collective); returns the number of filter offsets present.
template <int MW>
__device__ __forceinline__ int ring_tile_masks(const RowConvParams &p, const int *sl, int tile, uint32_t (&km)[MW]) {
#pragma unroll
  for (int w = 0; w < MW; ++w)
    km[w] = 0u;
  if (tile < 0 || p.mode != kModeMaskConv) {
    km[0] = 1u;
    return 1;
  }
  const int lane = (int)lane_id();
  int count = 0;
#pragma unroll
  for (int w = 0; w < MW; ++w) {
    if (w < p.mask_words) {
      uint32_t m = 0;
      if constexpr (MW == 1) {
        const int4 m4 = *reinterpret_cast<const int4 *>(sl + 136 + 4 * lane);  // four rows' words in one load
        m = static_cast<uint32_t>(m4.x | m4.y | m4.z | m4.w);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          m |= static_cast<uint32_t>(sl[136 + (i * 32 + lane) * MW + w]);
      }
      m = __reduce_or_sync(0xffffffffu, m) & p.mask_filter;
      const int left = p.kv - 32 * w;  // offsets this word covers
      if (left < 32)
        m &= left > 0 ? (1u << left) - 1u : 0u;
      km[w] = m;
      count += __popc(m);
    }
  }
  return count;
}

// Walks the tiles the scheduler publishes and, inside each, the (filter offset, reduction
// pass) steps.  on_tile(tile, slot, kmask_for_store, has_work) -> bool; on_step(tile, f, kp,
// first, last) -> bool; a false return aborts the walk.  Every consumer warp of the CTA runs
// the identical walk, so their step counters agree.  All 32 lanes take part.
// SINGLE: the walk is run by one thread on its own (no warp-collective operation inside), which
// is what the roles that issue from a single thread anyway use: their time per step is pure
// instruction latency, and the collectives would only add to it.
template <bool SINGLE, int MW, class TileFn, class StepFn>
__device__ __forceinline__ bool walk_steps_impl(const RowConvParams &p, const RingView &rv, int kpasses,
                                                TileFn on_tile, StepFn on_step, long long *prof_c = nullptr,
                                                long long *prof_prev_p = nullptr) {
#ifdef CB2_TRACE
#define CB2_WALK_MARK(i)                                                                                  \
  do {                                                                                                    \
    if (prof_c && (SINGLE || lane_id() == 0)) {                                                           \
      long long t = clock64();                                                                            \
      prof_c[i] += t - *prof_prev_p;                                                                      \
      *prof_prev_p = t;                                                                                   \
    }                                                                                                     \
  } while (0)
#else
#define CB2_WALK_MARK(i) ((void)0)
#endif
  for (int seq = 0;; ++seq) {
    const int si = seq % rv.ring;
    CB2_WALK_MARK(8);  // previous slot released
    if (!(SINGLE ? mbar_wait(rv.full0 + 8u * si, (seq / rv.ring) & 1, rv.abort_flag)
                 : mbar_wait_warp(rv.full0 + 8u * si, (seq / rv.ring) & 1, rv.abort_flag)))
      return false;
    CB2_WALK_MARK(9);  // slot published
    const int *sl = rv.slot(si);
    const int tile = sl[0];
    uint32_t kmask = static_cast<uint32_t>(sl[1]);  // MW == 1: the tile's mask; else: OR of its words
    const uint32_t kmask_store = kmask;
    bool cont = true;
    if (tile >= 0 && !(p.skip_empty_tiles && kmask == 0)) {
      if constexpr (MW == 1) {
        if (p.reverse_mask)
          kmask = __brev(kmask) >> (32 - p.kv);
        cont = on_tile(tile, sl, kmask_store, kmask != 0);
        uint32_t bits = kmask;
        bool first = true;
        while (cont && bits) {
          int f = __ffs(bits) - 1;
          bits &= bits - 1;
          for (int kp = 0; cont && kp < kpasses; ++kp) {
            bool last = (bits == 0) && (kp == kpasses - 1);
            cont = on_step(tile, f, kp, first, last);
            first = false;
          }
        }
      } else {
        // several mask words: offsets in ascending order word by word; with reverse_mask step
        // `pos` (weight offset pos) is taken iff the bit of offset kv - 1 - pos is set, so the
        // words are walked from the last bit down
        uint32_t km[MW];
        int remaining = 0;
#pragma unroll
        for (int w = 0; w < MW; ++w) {
          km[w] = static_cast<uint32_t>(sl[4 + w]);
          remaining += __popc(km[w]);
        }
        cont = on_tile(tile, sl, kmask_store, remaining != 0);
        bool first = true;
        for (int ww = 0; cont && ww < MW; ++ww) {
          const int w = p.reverse_mask ? MW - 1 - ww : ww;
          uint32_t bits = km[w];
          while (cont && bits) {
            const int b = p.reverse_mask ? 31 - __clz(bits) : __ffs(bits) - 1;
            bits &= ~(1u << b);
            const int f = p.reverse_mask ? p.kv - 1 - (32 * w + b) : 32 * w + b;
            --remaining;
            for (int kp = 0; cont && kp < kpasses; ++kp) {
              bool last = (remaining == 0) && (kp == kpasses - 1);
              cont = on_step(tile, f, kp, first, last);
              first = false;
            }
          }
        }
      }
    }
    CB2_WALK_MARK(10);  // steps done
    if (!SINGLE)
      __syncwarp();
    if (SINGLE || lane_id() == 0)
      mbar_arrive(rv.empty0 + 8u * si);
    if (!cont)
      return false;
    if (tile < 0)
      return true;  // end marker
  }
}

template <int MW, class TileFn, class StepFn>
__device__ __forceinline__ bool walk_steps(const RowConvParams &p, const RingView &rv, int kpasses, TileFn on_tile,
                                           StepFn on_step) {
  return walk_steps_impl<false, MW>(p, rv, kpasses, on_tile, on_step);
}
template <int MW, class TileFn, class StepFn>
__device__ __forceinline__ bool walk_steps_single(const RowConvParams &p, const RingView &rv, int kpasses,
                                                  TileFn on_tile, StepFn on_step, long long *prof_c = nullptr,
                                                  long long *prof_prev_p = nullptr) {
  return walk_steps_impl<true, MW>(p, rv, kpasses, on_tile, on_step, prof_c, prof_prev_p);
}

// The scheduler warp: draws tiles and fetches their mask words and row numbers straight into
// a ring slot with 4-byte cp.async.  The slot's "landed" barrier is completed by the copies
// themselves (one asynchronous arrival per lane), so any number of tiles can be in flight and
// each is published -- its OR-ed mask computed once, here -- as soon as ITS words are there.
// Slot layout (ints): [0] tile (-1 = no more tiles), [1] OR-ed mask (with several mask words per
// row: the OR of all of them, and the OR-ed words themselves at [4, 4 + MW)), [2] steps charged
// for the tile (scheduler only), [8,136) rows the gather starts from, from 136 on the destination
// rows in gather-GEMM mode / the rows' raw mask words (MW per row) in conv mode (in conv mode the
// destination rows are the gather rows).
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

// The first batch of tickets is requested at kernel entry (first_ticket_request), long before the
// scheduler can use it: the counter's round trip, and an L2 prefetch of the first tile's words,
// run while the CTA sets up its barriers and tensor memory.
__device__ __forceinline__ int first_ticket_count(int ntiles) {
  const int b = ntiles / ((int)gridDim.x * 4);
  return b < 1 ? 1 : (b > CB2_ROWCONV_TICKET_BATCH ? CB2_ROWCONV_TICKET_BATCH : b);
}

template <int MW>
__device__ __forceinline__ void scheduler_run(const RowConvParams &p, const RingView &rv, int ntiles, int kpasses,
                                              int first_base, int first_cnt) {
  constexpr int STEP_BUDGET = CB2_ROWCONV_STEP_BUDGET;  // steps a CTA may hold (drawn, not finished)
  const int lane = (int)lane_id();
  const bool dynamic = p.tickets != nullptr && gridDim.y == 1;
  const bool conv = p.mode == kModeMaskConv;
  int drawn = 0;
  // Tickets come in batches and the next batch is requested before the current one is used up:
  // the counter's round trip through L2 would otherwise be paid per tile.  Batches shrink to
  // one ticket as the counter nears the end so the tail stays balanced.
  constexpr int MAX_BATCH = CB2_ROWCONV_TICKET_BATCH;
  int cur_base = 0, cur_left = 0, next_base = 0, next_cnt = 0;
  auto request = [&](int seen) {
    int b = (ntiles - seen) / ((int)gridDim.x * 4);
    next_cnt = b < 1 ? 1 : (b > MAX_BATCH ? MAX_BATCH : b);
    if (lane == 0)
      next_base = atomicAdd(p.tickets, next_cnt);
  };
  if (dynamic) {
    next_base = first_base;  // requested at kernel entry (lane 0 holds the counter's answer)
    next_cnt = first_cnt;
  }
  auto draw = [&]() -> int {
    int t;
    if (dynamic) {
      if (cur_left == 0) {
        cur_base = __shfl_sync(0xffffffffu, next_base, 0);
        cur_left = next_cnt;
        next_cnt = 0;
        if (cur_base < ntiles)
          request(cur_base);
      }
      t = cur_base++;
      --cur_left;
    } else {
      t = blockIdx.x + drawn * gridDim.x;
    }
    ++drawn;
    return t;
  };
  const uint32_t slots_addr = smem_u32(rv.slots);
  // Tiles a CTA has drawn but not finished cannot be taken over by an idle CTA, so the
  // look-ahead is bounded by WORK, not by tiles: a CTA draws while the steps it holds (one per
  // offset in a tile's mask) are within STEP_BUDGET.  Until a tile's mask has landed it is
  // charged what the previous tile cost -- tiles arrive heaviest first, so that is an upper
  // estimate -- and the very first one is charged the whole budget: a CTA learns what its
  // first tile weighs before it takes a second.
  int issued = 0, accounted = 0, released = 0, held_steps = 0;
  int guess = (conv && dynamic) ? STEP_BUDGET + 1 : 1;
  // The scheduler's own instructions are what paces a CTA whose tiles carry one offset each: every
  // poll here is made by all lanes at once (a vote instead of a test by one lane and a shuffle), and releases are only looked at when the
  // CTA could not draw otherwise.
  auto account = [&]() {
    while (accounted < issued &&
           __any_sync(0xffffffffu, mbar_poll(rv.landed0 + 8u * (accounted % rv.ring), (accounted / rv.ring) & 1))) {
      int *sl = rv.slot(accounted % rv.ring);
      uint32_t km[MW];
      const int offsets = ring_tile_masks<MW>(p, sl, sl[0], km);
      const int nsteps = (sl[0] >= 0) ? max(1, offsets * kpasses) : 1;
      held_steps += nsteps - sl[2];
      __syncwarp();
      if (lane == 0) {
        uint32_t any = 0;
#pragma unroll
        for (int w = 0; w < MW; ++w) {
          any |= km[w];
          if (MW > 1)
            sl[4 + w] = static_cast<int>(km[w]);
        }
        sl[1] = static_cast<int>(any);
        sl[2] = nsteps;
        CB2_TRACE_EVENT(6, 14, sl[0]);  // tile published
        mbar_arrive(rv.full0 + 8u * (accounted % rv.ring));
      }
      __syncwarp();
      guess = nsteps;
      ++accounted;
    }
  };
  auto account_released = [&]() {
    while (released < accounted &&
           __any_sync(0xffffffffu, mbar_poll(rv.empty0 + 8u * (released % rv.ring), (released / rv.ring) & 1))) {
      held_steps -= rv.slot(released % rv.ring)[2];
      ++released;
    }
  };
  auto can_draw = [&]() { return (held_steps <= STEP_BUDGET || released == issued) && (issued - released < rv.ring); };
  // tables whose tiles can be fetched with two 16-byte copies per lane
  const bool wide_copies = conv && MW == 1 && p.mask_words == 1 &&
                           ((reinterpret_cast<uintptr_t>(p.argsort) | reinterpret_cast<uintptr_t>(p.mask)) & 15u) == 0;
  for (;;) {
    account();
    bool may_draw = can_draw();
    if (!may_draw) {
      account_released();
      may_draw = can_draw();
    }
    if (!may_draw) {
      // first learn what the tiles in flight weigh, then wait for the oldest one to be finished
      const bool ok = accounted < issued
                          ? mbar_wait_warp(rv.landed0 + 8u * (accounted % rv.ring), (accounted / rv.ring) & 1, rv.abort_flag)
                          : mbar_wait_warp(rv.empty0 + 8u * (released % rv.ring), (released / rv.ring) & 1, rv.abort_flag);
      if (!ok)
        return;
      continue;
    }
    const int si = issued % rv.ring;
    const int ticket = draw();
#ifndef CB2_TRACE_TICKET
#define CB2_TRACE_TICKET 0  // 0: follow the CTA that got the heaviest tile
#endif
    if (ticket == CB2_TRACE_TICKET && lane == 0)
      CB2_TRACE_SELECT(1);
    int tile = -1;
    if (ticket < ntiles)
      tile = conv ? (ntiles - 1 - ticket) : ticket;  // the last tiles of the sorted order carry the most offsets
    int *sl = rv.slot(si);
    const uint32_t sa = slots_addr + static_cast<uint32_t>(si * rv.slot_ints) * 4u;
    if (lane == 0) {
      sl[0] = tile;
      sl[2] = guess;
    }
    held_steps += guess;
    if (wide_copies && tile >= 0 && (tile + 1) * 128 <= p.n_rows) {
      cp_async_16(sa + (8 + 4 * lane) * 4, p.argsort + tile * 128 + 4 * lane, 16u);
      cp_async_16(sa + (136 + 4 * lane) * 4, p.mask + tile * 128 + 4 * lane, 16u);
    } else
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int j = i * 32 + lane;
      const int r = tile * 128 + j;
      if (tile >= 0 && r < p.n_rows) {
        if (conv) {
          cp_async_4(sa + (8 + j) * 4, p.argsort + r);
#pragma unroll
          for (int w = 0; w < MW; ++w)
            if (w < p.mask_words)
              cp_async_4(sa + (136 + j * MW + w) * 4, p.mask + (long long)r * p.mask_words + w);
        } else {
          sl[8 + j] = r;
          if (p.c_inds)
            cp_async_4(sa + (136 + j) * 4, p.c_inds + r);
          else
            sl[136 + j] = r;
        }
      } else {
        sl[8 + j] = -1;
#pragma unroll
        for (int w = 0; w < MW; ++w)
          sl[136 + j * MW + w] = conv ? 0 : -1;
      }
    }
    cp_async_mbar_arrive_noinc(rv.landed0 + 8u * si);  // arrives when this lane's copies have landed
    __syncwarp();  // the plain stores above are read by other lanes when the slot is published
    if (lane == 0)
      CB2_TRACE_EVENT(6, 16, tile);  // tile drawn, fetch issued
    ++issued;
    if (tile < 0)
      break;
  }
  // publish what is still in flight (the end marker at the latest)
  while (accounted < issued) {
    if (!mbar_wait_warp(rv.landed0 + 8u * (accounted % rv.ring), (accounted / rv.ring) & 1, rv.abort_flag))
      return;
    account();
  }
  // the last CTA to run out of tiles puts the two counters back to zero for the next launch
  if (dynamic && lane == 0) {
    if (next_cnt != 0)  // an outstanding request must have been served before the counters may be reset
      asm volatile("" ::"r"(next_base) : "memory");
    __threadfence();
    const int done = atomicAdd(p.tickets + 1, 1);
    if (done == (int)(gridDim.x * gridDim.y) - 1) {
      p.tickets[0] = 0;
      p.tickets[1] = 0;
      __threadfence();
    }
  }
  cp_async_wait_all();
}

template <int KIND, int NATOM_K, int BLOCK_N, bool B_MN, bool TMA_GATHER, int MASK_WORDS = 1>
__global__ void __launch_bounds__(RowConvCfg<KIND, NATOM_K, BLOCK_N, B_MN, TMA_GATHER, MASK_WORDS>::THREADS, 1)
rowconv_kernel(const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ CUtensorMap tmap_a,
               const RowConvParams p) {
  using Cfg = RowConvCfg<KIND, NATOM_K, BLOCK_N, B_MN, TMA_GATHER, MASK_WORDS>;
  constexpr int MW = MASK_WORDS;
  extern __shared__ uint8_t smem_raw[];
  if (threadIdx.x == 0)
    CB2_TRACE_CTA(0, 0);
  // Programmatic dependent launch: the next kernel on the stream may be scheduled onto SMs as
  // they free up, and this one may itself have started before its predecessor finished.  What
  // runs ahead is the set-up, the scheduler's tickets and mask words and the first row-index
  // loads -- tables no kernel of this library writes.  Every role calls grid_dep_wait() before
  // it first touches operand rows, weights or the output.
  grid_dep_launch();
  // 1024-byte alignment: required by the 128-byte swizzle atoms of TMA and tcgen05.
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t *smem = smem_raw + pad;
  const uint32_t sbase = raw_addr + pad;

  int *rowidx = reinterpret_cast<int *>(smem + Cfg::OFF_ROWIDX);
  int *outrow = reinterpret_cast<int *>(smem + Cfg::OFF_OUTROW);
  float *s_scale = reinterpret_cast<float *>(smem + Cfg::OFF_SCALE);
  float *s_bias = s_scale + BLOCK_N;
  volatile int *misc = reinterpret_cast<volatile int *>(smem + Cfg::OFF_MISC);
  // misc[0] tmem base, misc[1] abort flag, misc[2..5] per-group wait results
  volatile int *abort_flag = misc + 1;

  const uint32_t bars = sbase + Cfg::OFF_BARS;
  auto full_a = [&](int s) { return bars + 8u * s; };
  auto empty_a = [&](int s) { return bars + 8u * (3 + s); };
  auto acc_full = [&](int s) { return bars + 8u * (6 + s); };
  auto acc_empty = [&](int s) { return bars + 8u * (10 + s); };
  const uint32_t final_bar = bars + 8u * 14;
  auto full_b = [&](int s) { return bars + 8u * (16 + s); };
  auto empty_b = [&](int s) { return bars + 8u * (24 + s); };
  RingView rv;
  rv.slots = reinterpret_cast<int *>(smem + Cfg::OFF_RING);
  rv.full0 = bars + 8u * 32;
  rv.empty0 = bars + 8u * (32 + Cfg::RING);
  rv.landed0 = bars + 8u * (32 + 2 * Cfg::RING);
  rv.ring = Cfg::RING;
  rv.slot_ints = Cfg::RING_SLOT_INTS;
  rv.abort_flag = abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int ntiles = (p.n_rows + 127) / 128;
  const int kpasses = (p.red + Cfg::KRED - 1) / Cfg::KRED;
  const int n0 = blockIdx.y * BLOCK_N;

  // Scheduler warp: ask for the first tickets now; their round trip overlaps the set-up below.
  int early_base = 0, early_cnt = 0;
  if (warp == Cfg::SCHED_WARP && p.tickets != nullptr && gridDim.y == 1) {
    early_cnt = first_ticket_count(ntiles);
    if (lane == 0)
      early_base = atomicAdd(p.tickets, early_cnt);
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::SA; ++s) {
      mbar_init(full_a(s), Cfg::FULL_A_COUNT);
      mbar_init(empty_a(s), 1);
    }
    for (int s = 0; s < Cfg::SB; ++s) {
      mbar_init(full_b(s), 1);
      mbar_init(empty_b(s), 1);
    }
    for (int s = 0; s < Cfg::NUM_ACC; ++s) {
      mbar_init(acc_full(s), 1);
      mbar_init(acc_empty(s), Cfg::EPI_THREADS);
    }
    mbar_init(final_bar, 1);
    for (int s = 0; s < Cfg::RING; ++s) {
      mbar_init(rv.full0 + 8u * s, 1);
      mbar_init(rv.landed0 + 8u * s, 32);  // one copy-completion arrival per scheduler lane
      mbar_init(rv.empty0 + 8u * s, Cfg::RING_CONSUMER_WARPS);
    }
    mbar_init_fence();
    misc[1] = 0;
    misc[2] = misc[3] = misc[4] = misc[5] = 1;
    CB2_TRACE_SELECT(0);
  }
  if (KIND == 1) {
    for (int i = threadIdx.x; i < BLOCK_N; i += blockDim.x) {
      int n = n0 + i;
      s_scale[i] = (n < p.nn && p.scale) ? p.scale[n] : 0.f;
      s_bias[i] = (n < p.nn && p.bias) ? p.bias[n] : 0.f;
    }
  }
  if (warp == Cfg::MMA_WARP) {
    tmem_alloc(sbase + Cfg::OFF_MISC, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == Cfg::SCHED_WARP && early_cnt > 0 && p.mode == kModeMaskConv) {
    // the first tile's sort order and masks: 128 ints each, four 128-byte lines each
    const int first = __shfl_sync(0xffffffffu, early_base, 0);
    const int tile = ntiles - 1 - first;
    if (tile >= 0 && lane < 8) {
      const int r = tile * 128 + (lane & 3) * 32;
      if (r < p.n_rows) {
        const void *line = (lane < 4) ? static_cast<const void *>(p.argsort + r) : static_cast<const void *>(p.mask + (long long)r * p.mask_words);
        asm volatile("prefetch.global.L2 [%0];" ::"l"(line));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = static_cast<uint32_t>(misc[0]);
  if (threadIdx.x == 0)
    CB2_TRACE_EVENT(5, 11, 0);  // set-up done

  auto fail = [&](int code) {
    *abort_flag = 1;
    if (p.status)
      atomicCAS(p.status, 0, code);
  };

  if (warp < Cfg::MMA_WARP) {
    // ======================= epilogue: TMEM -> registers -> staging -> scattered rows
    const int et = threadIdx.x;
    const int erow = et & 127;   // the tile row this thread reads from TMEM (lane quarter = warp & 3)
    const int half = et >> 7;    // which share of the columns
    constexpr int COLS_PER_HALF = BLOCK_N / Cfg::EPI_HALVES;
    uint8_t *staging = smem + Cfg::OFF_STAGING;
    constexpr int CPR = Cfg::OUT_ROW_BYTES / 16;       // 16-byte chunks per output row
    constexpr int SWZ = (CPR >= 8 ? 8 : CPR) - 1;
    constexpr int CH_PER_ROUND = 32 * Cfg::OES / 16;   // chunks produced per 32 columns
    int acc_use = 0;
    bool dep_waited = false;
    CB2_PROF_BEGIN();
    walk_steps<MW>(
        p, rv, kpasses,
        [&](int tile, const int *sl, uint32_t kmask_store, bool has_work) -> bool {
          if (et == 0)
            CB2_PROF_MARK(0);  // walk
          if (!dep_waited) {
            grid_dep_wait();
            dep_waited = true;
          }
          const int o = (p.mode == kModeMaskConv) ? sl[8 + erow] : sl[136 + erow];  // destination row of this thread's tile row
          if (et == 0 && p.mask_out && blockIdx.y == 0) {
            if constexpr (MW == 1) {
              p.mask_out[tile] = kmask_store;
            } else {
              for (int w = 0; w < p.mask_words; ++w)
                p.mask_out[(long long)tile * p.mask_words + w] = static_cast<uint32_t>(sl[4 + w]);
            }
          }
          const int buf = acc_use % Cfg::NUM_ACC;
          if (has_work) {
            if (et == 0) {
              CB2_TRACE_EVENT(4, 7, tile);
              bool ok = mbar_wait(acc_full(buf), (acc_use / Cfg::NUM_ACC) & 1, abort_flag);
              CB2_TRACE_EVENT(4, 8, tile);  // accumulator complete
              misc[2] = ok ? 1 : 0;
              if (!ok)
                fail(kStatusWaitTimeout);
              CB2_PROF_MARK(1);  // accumulator complete
            }
          }
          named_bar_sync(1, Cfg::EPI_THREADS);  // wait result visible; staging free again
          if (et == 0)
            CB2_PROF_MARK(2);  // barrier
          if (has_work && misc[2] == 0)
            return false;
          if (half == 0)
            outrow[erow] = o;
          tc_fence_after();
          const uint32_t trow = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) +
                                static_cast<uint32_t>(buf * BLOCK_N);
          const bool use_src = (p.src_mode != kSrcNone) && (p.beta != 0.f);
          // fast path: out = cvt(acc); everything else goes through the general epilogue
          const bool plain = !use_src && p.act_type == 0 && p.alpha == 1.f;
          constexpr int ROUNDS = COLS_PER_HALF / 32;
#pragma unroll 1
          for (int round = 0; round < ROUNDS; ++round) {
            uint32_t v[32];
            const int col0 = half * COLS_PER_HALF + round * 32;
            if (has_work) {
              tmem_ld32(trow + col0, v);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                v[i] = 0u;
            }
            const int ncol0 = n0 + col0;
            if constexpr (KIND == 0) {
              uint32_t packed[16];
              if (plain) {
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  __half2 h2 = __floats2half2_rn(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                  packed[i / 2] = *reinterpret_cast<uint32_t *>(&h2);
                }
              } else {
                float t[32];
                if (use_src) {
                  if (p.src_mode == kSrcRows) {
                    uint4 srcv[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                      srcv[q] = make_uint4(0, 0, 0, 0);
                    if (o >= 0) {
                      const uint4 *sp = reinterpret_cast<const uint4 *>(
                          reinterpret_cast<const __half *>(p.src) + (long long)o * p.lds + ncol0);
#pragma unroll
                      for (int q = 0; q < 4; ++q)
                        if (ncol0 + q * 8 < p.nn)
                          srcv[q] = __ldg(sp + q);
                    }
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                      const __half2 h = reinterpret_cast<const __half2 *>(srcv)[i / 2];
                      t[i] = __fmaf_rn(p.alpha, __uint_as_float(v[i]), __fmul_rn(p.beta, __low2float(h)));
                      t[i + 1] = __fmaf_rn(p.alpha, __uint_as_float(v[i + 1]), __fmul_rn(p.beta, __high2float(h)));
                    }
                  } else {
                    const __half *bv = reinterpret_cast<const __half *>(p.src);
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                      const float sv = (ncol0 + i < p.nn) ? __half2float(__ldg(bv + ncol0 + i)) : 0.f;
                      t[i] = __fmaf_rn(p.alpha, __uint_as_float(v[i]), __fmul_rn(p.beta, sv));
                    }
                  }
                } else {
#pragma unroll
                  for (int i = 0; i < 32; ++i)
                    t[i] = __fmul_rn(p.alpha, __uint_as_float(v[i]));
                }
                if (p.act_type == 1) {
#pragma unroll
                  for (int i = 0; i < 32; ++i)
                    t[i] = fmaxf(t[i], 0.f);
                } else if (p.act_type != 0) {
#pragma unroll
                  for (int i = 0; i < 32; ++i)
                    t[i] = apply_act(t[i], p.act_type, p.act_alpha);
                }
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                  __half2 h2 = __floats2half2_rn(t[i], t[i + 1]);
                  packed[i / 2] = *reinterpret_cast<uint32_t *>(&h2);
                }
              }
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int c = (col0 / 32) * CH_PER_ROUND + q;
                const int pc = (c & ~SWZ) | ((c ^ erow) & SWZ);
                *reinterpret_cast<uint4 *>(staging + erow * Cfg::OUT_ROW_BYTES + pc * 16) =
                    make_uint4(packed[q * 4], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
              }
            } else {
              uint32_t packed[8];
              float t[32];
              {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  t[i] = __int2float_rn(static_cast<int>(v[i]));
                const float4 *sc4 = reinterpret_cast<const float4 *>(s_scale + col0);
                const float4 *bi4 = reinterpret_cast<const float4 *>(s_bias + col0);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                  const float4 sc = sc4[q], bi = bi4[q];
                  t[4 * q + 0] = __fmaf_rn(sc.x, t[4 * q + 0], bi.x);
                  t[4 * q + 1] = __fmaf_rn(sc.y, t[4 * q + 1], bi.y);
                  t[4 * q + 2] = __fmaf_rn(sc.z, t[4 * q + 2], bi.z);
                  t[4 * q + 3] = __fmaf_rn(sc.w, t[4 * q + 3], bi.w);
                }
              }
              if (use_src) {
                uint4 srcv[2];
                srcv[0] = srcv[1] = make_uint4(0, 0, 0, 0);
                if (o >= 0) {
                  const uint4 *sp = reinterpret_cast<const uint4 *>(
                      reinterpret_cast<const int8_t *>(p.src) + (long long)o * p.lds + ncol0);
#pragma unroll
                  for (int q = 0; q < 2; ++q)
                    if (ncol0 + q * 16 < p.nn)
                      srcv[q] = __ldg(sp + q);
                }
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  t[i] = __fmaf_rn(p.beta, static_cast<float>(reinterpret_cast<const int8_t *>(srcv)[i]), t[i]);
              }
              if (p.act_type == 1) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  t[i] = fmaxf(t[i], 0.f);
              } else if (p.act_type != 0) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                  t[i] = apply_act(t[i], p.act_type, p.act_alpha);
              }
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                packed[i / 4] = cvt_pack4_s8(t[i], t[i + 1], t[i + 2], t[i + 3]);
#pragma unroll
              for (int q = 0; q < 2; ++q) {
                const int c = (col0 / 32) * CH_PER_ROUND + q;
                const int pc = (c & ~SWZ) | ((c ^ erow) & SWZ);
                *reinterpret_cast<uint4 *>(staging + erow * Cfg::OUT_ROW_BYTES + pc * 16) =
                    make_uint4(packed[q * 4], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
              }
            }
          }
          if (has_work) {
            tc_fence_before();
            mbar_arrive(acc_empty(buf));
            ++acc_use;
          }
          if (et == 0) {
            CB2_TRACE_EVENT(4, 12, tile);  // staged
            CB2_PROF_MARK(3);  // TMEM -> staging
          }
          named_bar_sync(1, Cfg::EPI_THREADS);  // staging complete
          if (et == 0)
            CB2_PROF_MARK(4);  // barrier
          // phase 2: CPR threads per row write whole rows
          {
            const int c = et % CPR;
            const int row0 = et / CPR;
            constexpr int RSTEP = Cfg::EPI_THREADS / CPR;
            const int ncol = n0 + c * (16 / Cfg::OES);
            if (ncol < p.nn) {
#pragma unroll 4
              for (int i = 0; i < 128 / RSTEP; ++i) {
                const int row = row0 + i * RSTEP;
                const int orow = outrow[row];
                if (orow >= 0) {
                  const int pc = (c & ~SWZ) | ((c ^ row) & SWZ);
                  uint4 val = *reinterpret_cast<const uint4 *>(staging + row * Cfg::OUT_ROW_BYTES + pc * 16);
                  uint8_t *dst = reinterpret_cast<uint8_t *>(p.out) +
                                 ((long long)orow * p.ldo + ncol) * Cfg::OES;
                  *reinterpret_cast<uint4 *>(dst) = val;
                }
              }
            }
          }
          if (et == 0) {
            CB2_TRACE_EVENT(4, 9, tile);  // rows stored
            CB2_PROF_MARK(5);  // staging -> global
          }
          return true;
        },
        [&](int, int, int, bool, bool) -> bool { return true; });
    if (et == 0)
      CB2_PROF_END2();
  } else if (warp == Cfg::MMA_WARP) {
    // ======================= MMA issuer (one thread walks and issues)
    constexpr uint32_t idesc = make_idesc(KIND, false, B_MN, 128, BLOCK_N);
    int step = 0, acc_use = 0, bcount = 0, last_key = -1, cur_slot = 0;
    bool ok_all = true;
    const uint64_t adesc_base = make_smem_desc(sbase + Cfg::OFF_A, 16, 1024);
    const uint64_t bdesc_base = B_MN ? make_smem_desc(sbase + Cfg::OFF_B, p.b_lbo, p.b_sbo)
                                     : make_smem_desc(sbase + Cfg::OFF_B, 16, 1024);
    CB2_PROF_BEGIN();
    if (lane == 0) {
    walk_steps_single<MW>(
        p, rv, kpasses,
        [&](int, const int *, uint32_t, bool) -> bool {
          CB2_PROF_MARK(7);  // previous slot released, this tile's slot read
          return true;
        },
        [&](int tile, int f, int kp, bool first, bool last) -> bool {
          const int buf = acc_use % Cfg::NUM_ACC;
          int ok = 1;
          {
            CB2_PROF_MARK(0);  // the walk between steps
            if (first)
              ok = mbar_wait(acc_empty(buf), ((acc_use / Cfg::NUM_ACC) & 1) ^ 1, abort_flag);
            CB2_PROF_MARK(1);  // accumulator free
            const int key = f * kpasses + kp;
            if (ok && key != last_key) {
              if (bcount > 0)
                tc_commit(empty_b(cur_slot));
              cur_slot = bcount % Cfg::SB;
              ok = mbar_wait(full_b(cur_slot), (bcount / Cfg::SB) & 1, abort_flag);
              ++bcount;
              last_key = key;
            }
            const int stage = step % Cfg::SA;
            CB2_PROF_MARK(2);  // weight tile present
            CB2_TRACE_EVENT(3, 4, step);  // waiting for rows
            if (ok)
              ok = mbar_wait(full_a(stage), (step / Cfg::SA) & 1, abort_flag);
            CB2_TRACE_EVENT(3, 5, step);  // rows landed
            CB2_PROF_MARK(3);  // rows present
            if (ok) {
              if constexpr (!TMA_GATHER)
                fence_proxy_async_smem();  // gathered rows were written through the generic proxy
              tc_fence_after();
              CB2_PROF_MARK(4);  // fences
              // Descriptors differ from the stage's / slot's base descriptor only in the start
              // address field (bits 0-13, units of 16 bytes), so each one is an add.  This loop is
              // issued by a single thread: every instruction saved here shortens each step.
              const uint64_t adesc0 = adesc_base + static_cast<uint64_t>((stage * Cfg::A_STAGE_BYTES) >> 4);
              const uint64_t bdesc0 = bdesc_base + static_cast<uint64_t>((cur_slot * Cfg::B_SLOT_BYTES) >> 4);
              const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(buf * BLOCK_N);
              const int red_left = p.red - kp * Cfg::KRED;
              constexpr int KSTEPS_FULL = NATOM_K * 4;
              auto issue = [&](int ks, uint32_t acc) {
                const int ka = ks >> 2, kk = ks & 3;
                const uint64_t adesc = adesc0 + static_cast<uint64_t>((ka * (Cfg::TILE_M * 128) + kk * 32) >> 4);
                const uint64_t bdesc =
                    bdesc0 + static_cast<uint64_t>(B_MN ? (((ka * 4 + kk) * (Cfg::UMMA_K * 128)) >> 4)
                                                        : ((ka * (BLOCK_N * 128) + kk * 32) >> 4));
                tc_mma<KIND>(d_tmem, adesc, bdesc, idesc, acc);
              };
              if (red_left >= Cfg::KRED) {
#pragma unroll
                for (int ks = 0; ks < KSTEPS_FULL; ++ks)
                  issue(ks, (first && ks == 0) ? 0u : 1u);
              } else {
                const int ksteps_total = (red_left + Cfg::UMMA_K - 1) / Cfg::UMMA_K;
                for (int ks = 0; ks < ksteps_total; ++ks)
                  issue(ks, (first && ks == 0) ? 0u : 1u);
              }
              CB2_PROF_MARK(5);  // MMAs issued
              tc_commit(empty_a(stage));
              CB2_TRACE_EVENT(3, 6, step);  // MMAs issued
              if (last)
                tc_commit(acc_full(buf));
              CB2_PROF_MARK(6);  // commits
            }
          }
          ++step;
          if (last)
            ++acc_use;
          if (!ok) {
            fail(kStatusWaitTimeout);
            ok_all = false;
            return false;
          }
          return true;
        }
#ifdef CB2_TRACE
        , prof_c, &prof_prev
#endif
        );
      CB2_TRACE_CTA(2, (unsigned long long)step);
      CB2_PROF_END();
      // make sure every MMA has retired before TMEM is released
      if (ok_all) {
        tc_commit(final_bar);
        if (!mbar_wait(final_bar, 0, abort_flag))
          fail(kStatusWaitTimeout);
      }
    }
    __syncwarp();
  } else if (warp == Cfg::TMA_WARP) {
    // ======================= weight tiles by TMA (lane 0 issues)
    int bcount = 0, last_key = -1;
    if (lane == 0) {
    tma_prefetch_desc(&tmap_b);
    grid_dep_wait();
    walk_steps_single<MW>(
        p, rv, kpasses, [&](int, const int *, uint32_t, bool) -> bool { return true; },
        [&](int tile, int f, int kp, bool, bool) -> bool {
          int ok = 1;
          const int key = f * kpasses + kp;
          if (key != last_key) {
            {
              const int slot = bcount % Cfg::SB;
              ok = mbar_wait(empty_b(slot), ((bcount / Cfg::SB) & 1) ^ 1, abort_flag);
              if (ok) {
                const uint32_t dst = sbase + Cfg::OFF_B + slot * Cfg::B_SLOT_BYTES;
                mbar_arrive_expect_tx(full_b(slot), Cfg::B_SLOT_BYTES);
                if constexpr (!B_MN) {
                  // [BLOCK_N rows x 128 B] per reduction atom; rows = output channels
#pragma unroll
                  for (int ka = 0; ka < NATOM_K; ++ka)
                    tma_load_3d(dst + ka * (BLOCK_N * 128), &tmap_b, full_b(slot),
                                kp * Cfg::KRED + ka * Cfg::ATOM_ELEMS, f, n0);
                } else {
                  // [KRED rows x 128 B] per block of ATOM_ELEMS output channels; rows = reduction
#pragma unroll
                  for (int na = 0; na < BLOCK_N / Cfg::ATOM_ELEMS; ++na)
                    tma_load_3d(dst + na * (Cfg::KRED * 128), &tmap_b, full_b(slot),
                                n0 + na * Cfg::ATOM_ELEMS, f, kp * Cfg::KRED);
                }
              }
            }
            ++bcount;
            last_key = key;
          }
          if (!ok) {
            fail(kStatusWaitTimeout);
            return false;
          }
          return true;
        });
    }
    __syncwarp();
  } else if (warp == Cfg::SCHED_WARP) {
    // ======================= scheduler: draws tiles, publishes their masks and row numbers
    scheduler_run<MW>(p, rv, ntiles, kpasses, early_base, early_cnt);
  } else {
    // ======================= operand-row gather: group g owns stage g
    if constexpr (TMA_GATHER) {
      // One warp per group; lane L fetches tile rows 4L .. 4L+3 ("its quad") with one request
      // per 128-byte column block.  A quad none of whose rows has a neighbour at this offset is
      // not requested at all -- for the offsets away from the centre that is most quads, and the
      // copy engine's request rate is what bounds such steps.  The stage therefore keeps the
      // invariant "a quad that was not requested holds zeros": it is cleared once here, and a
      // quad that was filled in the previous use and is not refilled now is cleared again.
      const int g = warp - Cfg::FIRST_GATHER_WARP;
      if (lane == 0)
        tma_prefetch_desc(&tmap_a);
      const uint32_t my_quad = sbase + Cfg::OFF_A + g * Cfg::A_STAGE_BYTES + lane * (4 * 128);
      auto clear_quad = [&]() {
#pragma unroll
        for (int ka = 0; ka < NATOM_K; ++ka)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            st_shared_zero16(my_quad + ka * (Cfg::TILE_M * 128) + i * 16);
      };
      clear_quad();
      fence_proxy_async_smem();
      __syncwarp();
      uint32_t dirty = 0;  // quads of this stage that hold gathered rows
      bool dep_waited = false;
      int step = 0;
      int o[4] = {-1, -1, -1, -1};
      walk_steps<MW>(
          p, rv, kpasses,
          [&](int tile, const int *sl, uint32_t, bool) -> bool {
            const int4 v = *reinterpret_cast<const int4 *>(sl + 8 + lane * 4);
            o[0] = v.x, o[1] = v.y, o[2] = v.z, o[3] = v.w;
            return true;
          },
          [&](int tile, int f, int kp, bool, bool) -> bool {
            const bool mine = (step % Cfg::SA) == g;
            const int use = step / Cfg::SA;
            ++step;
            if (!mine)
              return true;
            int idx[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              idx[r] = -1;
              if (o[r] >= 0) {
                if (p.mode == kModeMaskConv)
                  idx[r] = __ldg(p.indices + (long long)f * p.n_rows + o[r]);
                else
                  idx[r] = p.a_inds ? __ldg(p.a_inds + o[r]) : o[r];
              }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r)
              if (idx[r] >= p.a_rows) {  // reported; the copy engine would read such a row as zeros
                fail(kStatusBadIndex);
                idx[r] = -1;
              }
            if (lane == 0)
              CB2_TRACE_EVENT(g, 1, step - 1 + (idx[0] == 0x7fffffff));  // index loaded
            if (!mbar_wait_warp(empty_a(g), (use & 1) ^ 1, abort_flag)) {
              if (lane == 0)
                fail(kStatusWaitTimeout);
              return false;
            }
            if (!dep_waited) {
              grid_dep_wait();
              dep_waited = true;
            }
            const bool wanted = (idx[0] & idx[1] & idx[2] & idx[3]) >= 0;  // some row index is not -1
            const uint32_t need = __ballot_sync(0xffffffffu, wanted);
            if (((dirty >> lane) & 1u) && !wanted) {
              clear_quad();
              fence_proxy_async_smem();  // generic-proxy stores, read by the tensor core
            }
            __syncwarp();
            if (lane == 0) {
              CB2_TRACE_EVENT(g, 2, step - 1);  // stage free
              mbar_arrive_expect_tx(full_a(g), static_cast<uint32_t>(__popc(need)) * (NATOM_K * 512));
            }
            __syncwarp();
            if (wanted) {
#pragma unroll
              for (int ka = 0; ka < NATOM_K; ++ka)
                tma_gather4(my_quad + ka * (Cfg::TILE_M * 128), &tmap_a, full_a(g),
                            kp * Cfg::KRED + ka * Cfg::ATOM_ELEMS, idx[0], idx[1], idx[2], idx[3]);
            }
            dirty = need;
            if (lane == 0)
              CB2_TRACE_EVENT(g, 3, step - 1);  // copies issued
            return true;
          });
    } else {
      constexpr int GT = Cfg::GROUP_THREADS;
      constexpr int RPT = (128 + GT - 1) / GT;                  // tile rows whose index each thread fetches
      const int g = (warp - Cfg::FIRST_GATHER_WARP) / (GT / 32);  // 0..2
      const int gt = threadIdx.x - (Cfg::FIRST_GATHER_WARP * 32 + g * GT);
      constexpr int CPR = NATOM_K * 8;                  // 16-byte chunks per operand row
      constexpr int RSTEP = GT / CPR;
      const int c = gt % CPR;
      const int row0 = gt / CPR;
      int *group_rowidx = rowidx + g * 256;  // two buffers, alternating per use of the stage
      volatile int *my_flag = misc + 3 + g;
      bool dep_waited = false;
      int step = 0;
      int o[RPT];
#pragma unroll
      for (int r = 0; r < RPT; ++r)
        o[r] = -1;
      const uint8_t *a_bytes = reinterpret_cast<const uint8_t *>(p.a);
      walk_steps<MW>(
          p, rv, kpasses,
          [&](int tile, const int *sl, uint32_t, bool) -> bool {
            // the rows this thread's gathers start from (sort index, or the row itself)
#pragma unroll
            for (int r = 0; r < RPT; ++r)
              o[r] = (gt + r * GT < 128) ? sl[8 + gt + r * GT] : -1;
            return true;
          },
          [&](int tile, int f, int kp, bool, bool) -> bool {
            const bool mine = (step % Cfg::SA) == g;
            const int use = step / Cfg::SA;
            ++step;
            if (!mine)
              return true;
            int idx[RPT];
#pragma unroll
            for (int r = 0; r < RPT; ++r) {
              idx[r] = -1;
              if (o[r] >= 0) {
                if (p.mode == kModeMaskConv)
                  idx[r] = __ldg(p.indices + (long long)f * p.n_rows + o[r]);
                else
                  idx[r] = p.a_inds ? __ldg(p.a_inds + o[r]) : o[r];
              }
            }
#pragma unroll
            for (int r = 0; r < RPT; ++r)
              if (idx[r] >= p.a_rows) {  // never dereference a row the caller did not provide
                fail(kStatusBadIndex);
                idx[r] = -1;
              }
            if (gt == 0) {
              CB2_TRACE_EVENT(g, 1, step - 1 + (idx[0] == 0x7fffffff));  // index loaded
              bool ok = mbar_wait(empty_a(g), (use & 1) ^ 1, abort_flag);
              CB2_TRACE_EVENT(g, 2, step - 1);  // stage free
              *my_flag = ok ? 1 : 0;
              if (!ok)
                fail(kStatusWaitTimeout);
            }
            // Double-buffered: a thread that runs ahead writes the other buffer than the one
            // slower threads of the group may still be reading for the previous use.
            int *my_rowidx = group_rowidx + (use & 1) * 128;
#pragma unroll
            for (int r = 0; r < RPT; ++r)
              if (gt + r * GT < 128)
                my_rowidx[gt + r * GT] = idx[r];
            named_bar_sync(2 + g, Cfg::GROUP_THREADS);
            if (*my_flag == 0)
              return false;
            if (!dep_waited) {
              grid_dep_wait();
              dep_waited = true;
            }
            const uint32_t a_stage = sbase + Cfg::OFF_A + g * Cfg::A_STAGE_BYTES;
            const int byte_off = kp * Cfg::KRED * Cfg::ES + c * 16;
            const bool col_ok = byte_off < p.red * Cfg::ES;
            const uint32_t dst_c = a_stage + (c >> 3) * (Cfg::TILE_M * 128);
#pragma unroll
            for (int i = 0; i < (128 + RSTEP - 1) / RSTEP; ++i) {
              const int row = row0 + i * RSTEP;
              if ((128 % RSTEP) != 0 && row >= 128)
                break;
              const int ridx = my_rowidx[row];
              const uint32_t dst = dst_c + (row >> 3) * 1024 + (row & 7) * 128 + (((c & 7) ^ (row & 7)) << 4);
              const bool valid = col_ok && ridx >= 0;
              const uint8_t *srcp = valid ? a_bytes + ((long long)ridx * p.lda) * Cfg::ES + byte_off : a_bytes;
              cp_async_16(dst, srcp, valid ? 16u : 0u);
            }
            // The barrier is signalled by the copy engine when this thread's copies have landed;
            // the thread itself runs on to its next step.  The consumer makes the data visible
            // to the tensor core with a proxy fence after its wait.
            cp_async_mbar_arrive_noinc(full_a(g));
            if (gt == 0)
              CB2_TRACE_EVENT(g, 3, step - 1);  // copies issued
            return true;
          });
      cp_async_wait_all();
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0)
    CB2_TRACE_CTA(1, 0);
  if (warp == Cfg::MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

} // namespace cb2
