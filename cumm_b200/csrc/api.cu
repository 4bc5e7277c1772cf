// C ABI of the library: argument validation (the checks of the reference's host
// prologues, cumm/gemm/nvrtc_code.py:34-146 and cumm/conv/nvrtc_code.py:20-260), kernel
// selection, TMA descriptor set-up and launches.  No CPU compute path exists here: when
// no kernel fits the descriptor the call fails with CB2_ERR_UNSUPPORTED.
#include "../../include/cumm_b200.h"
#include "rowconv_kernel.cuh"
#include "wgrad_kernel.cuh"
#include "pairgen_kernels.cuh"
#include "peer_reduce_kernel.cuh"

#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#ifndef CB2_DEFAULT_GATHER
#define CB2_DEFAULT_GATHER 2
#endif

namespace {

using namespace cb2;

thread_local std::string g_err;
std::atomic<uint64_t> g_launches{0};
struct LaunchInfo {
  int num_regs = 0, num_threads = 0, smem_bytes = 0;
};
thread_local LaunchInfo g_last_launch;
template <class Kern> int kernel_regs(Kern kern) {
  cudaFuncAttributes attr;
  return cudaFuncGetAttributes(&attr, kern) == cudaSuccess ? attr.numRegs : 0;
}

int set_err(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

#define CB2_CHECK_ARG(cond, ...)                                                                   \
  do {                                                                                             \
    if (!(cond))                                                                                   \
      return set_err(CB2_ERR_INVALID_ARG, __VA_ARGS__);                                            \
  } while (0)
#define CB2_CHECK_RT(cond, ...)                                                                    \
  do {                                                                                             \
    if (!(cond))                                                                                   \
      return set_err(CB2_ERR_RUNTIME, __VA_ARGS__);                                                \
  } while (0)
#define CB2_CUDA(expr)                                                                             \
  do {                                                                                             \
    cudaError_t e__ = (expr);                                                                      \
    if (e__ != cudaSuccess)                                                                        \
      return set_err(CB2_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));               \
  } while (0)

constexpr int kMaxDevices = 64;
constexpr int kTicketSlots = 256;
constexpr size_t kStatusBytes = (16 + 2 * kTicketSlots) * sizeof(int);

struct DeviceState {
  bool ready = false;
  int num_sms = 0;
  int *status = nullptr;
};
DeviceState g_dev[kMaxDevices];
std::mutex g_mu;

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int get_device(DeviceState **out) {
  int dev = 0;
  CB2_CUDA(cudaGetDevice(&dev));
  CB2_CHECK_RT(dev >= 0 && dev < kMaxDevices, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState &st = g_dev[dev];
  if (!st.ready) {
    cudaDeviceProp prop;
    CB2_CUDA(cudaGetDeviceProperties(&prop, dev));
    CB2_CHECK_RT(prop.major == 10, "cumm_b200 kernels are built for sm_100a only; device %d is sm_%d%d",
                 dev, prop.major, prop.minor);
    st.num_sms = prop.multiProcessorCount;
    // word 0: kernel status; from word 16 on: kTicketSlots pairs of scheduling counters
    CB2_CUDA(cudaMalloc(&st.status, kStatusBytes));
    CB2_CUDA(cudaMemset(st.status, 0, kStatusBytes));
    st.ready = true;
  }
  if (!g_encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    CB2_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    CB2_CHECK_RT(fn != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled not available");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  *out = &st;
  return CB2_OK;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// 3-D tensor map over a weight-like tensor [outer, mid, inner] (inner contiguous).
int make_weight_map(CUtensorMap *map, const void *ptr, int es, uint64_t inner, uint64_t mid, uint64_t outer,
                    uint64_t mid_stride_elems, uint64_t outer_stride_elems, uint32_t box_inner,
                    uint32_t box_outer) {
  cuuint64_t dims[3] = {inner, mid, outer};
  cuuint64_t strides[2] = {mid_stride_elems * es, outer_stride_elems * es};
  cuuint32_t box[3] = {box_inner, 1, box_outer};
  cuuint32_t estr[3] = {1, 1, 1};
  CB2_CHECK_ARG(aligned16(ptr), "weight pointer must be 16-byte aligned");
  CB2_CHECK_ARG(strides[0] % 16 == 0 && strides[1] % 16 == 0, "weight strides must be multiples of 16 bytes");
  CUresult r = g_encode(map, es == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                        const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  CB2_CHECK_RT(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return CB2_OK;
}

// 2-D tensor map over gathered operand rows [rows, width] (row stride ld elements); the box is
// one row of 128 bytes, so a gather is one request per (row, column block).
int make_rows_map(CUtensorMap *map, const void *ptr, int es, uint64_t width, uint64_t rows, uint64_t ld) {
  cuuint64_t dims[2] = {width, rows > 0 ? rows : 1};
  cuuint64_t strides[1] = {ld * es};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / es), 1};
  cuuint32_t estr[2] = {1, 1};
  CB2_CHECK_ARG(aligned16(ptr), "operand pointer must be 16-byte aligned");
  CB2_CHECK_ARG(strides[0] % 16 == 0, "operand row stride must be a multiple of 16 bytes");
  CUresult r = g_encode(map, es == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                        const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  CB2_CHECK_RT(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (rows) failed with code %d", (int)r);
  return CB2_OK;
}

// Which row-gather implementation the kernels use: 0 cp.async, otherwise TMA gather4.
int gather_mode() {
  static int mode = -1;
  if (mode < 0) {
    int m = CB2_DEFAULT_GATHER;
    if (const char *v = getenv("CUMM_B200_GATHER"))
      m = atoi(v);
    mode = (m >= 0 && m <= 2) ? m : CB2_DEFAULT_GATHER;
  }
  return mode;
}

// Launch with programmatic stream serialisation: the kernel may be scheduled while its
// predecessor on the stream is still running and synchronises with it through
// griddepcontrol.wait in its own code.  `level` 1 (on by default): the chain of the three
// weight-gradient kernels, the gather-GEMM-scatter calls and the int8 convolutions; level 2
// (only with CUMM_B200_PDL=2): the fp16 convolution row kernels.  CUMM_B200_PDL=0 launches everything the
// ordinary way.
template <class Kern, class... Args>
cudaError_t launch_after(int level, Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                         Args... args) {
  static const int enabled = [] {
    const char *v = getenv("CUMM_B200_PDL");
    return v ? atoi(v) : 1;
  }();
  const bool pdl = enabled >= level;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

template <int KIND, int NATOM_K, int BLOCK_N, bool B_MN, bool TMA_GATHER, int MW = 1>
int launch_rowconv_inst(const CUtensorMap &map, const CUtensorMap &map_a, const RowConvParams &p, int grid_x,
                        int grid_y, cudaStream_t stream) {
  using Cfg = RowConvCfg<KIND, NATOM_K, BLOCK_N, B_MN, TMA_GATHER, MW>;
  auto kern = rowconv_kernel<KIND, NATOM_K, BLOCK_N, B_MN, TMA_GATHER, MW>;
  static std::atomic<uint64_t> configured{0};  // bit per device
  static std::atomic<int> regs{0};
  int dev = 0;
  CB2_CUDA(cudaGetDevice(&dev));
  if (!(configured.load() & (1ull << dev))) {
    CB2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    regs.store(kernel_regs(kern));
    configured.fetch_or(1ull << dev);
  }
  g_last_launch.num_regs = regs.load();
  g_last_launch.num_threads = Cfg::THREADS;
  g_last_launch.smem_bytes = Cfg::SMEM_BYTES;
  // A gather-GEMM-scatter call is one of a run of small kernels (one per filter offset), where
  // overlapping each kernel's set-up with its predecessor's tail nearly halves the run.  For the
  // convolutions it measured +4 % for the int8 kernels (long epilogue tail) and neutral to
  // slightly worse for fp16, so only the former take part by default.
  const int pdl_level = p.mode != kModeMaskConv ? 1 : (KIND == 1 ? 1 : 2);
  CB2_CUDA(launch_after(pdl_level, kern, dim3(grid_x, grid_y), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, stream, map,
                        map_a, p));
  g_launches.fetch_add(1);
  return CB2_OK;
}

struct RowConvPlan {
  int kind;     // 0 f16, 1 s8
  int natom_k;  // 1 or 2
  int block_n;  // 64 or 128
  bool b_mn;
};

// tile_n / tile_k: GemmAlgoDesp::tile_shape[1] / [2] of the caller's descriptor (0 = choose from the
// problem: the narrowest tile that covers the output width / the reduction width).
int plan_rowconv(int kind, int red, int nn, bool b_mn, int tile_n, int tile_k, RowConvPlan *plan) {
  plan->kind = kind;
  plan->b_mn = b_mn;
  const int atom = kind == 0 ? 64 : 128;
  if (tile_n != 0 && tile_n != 64 && tile_n != 128)
    return set_err(CB2_ERR_UNSUPPORTED, "can't find any suitable algo: tile_shape[1] = %d (kernels exist for 64 and 128)",
                   tile_n);
  if (tile_k != 0 && tile_k != atom && !(kind == 0 && tile_k == 2 * atom))
    return set_err(CB2_ERR_UNSUPPORTED, "can't find any suitable algo: tile_shape[2] = %d (kernels exist for %d%s)",
                   tile_k, atom, kind == 0 ? " and 128" : "");
  plan->natom_k = tile_k ? tile_k / atom : ((kind == 0 && red > atom) ? 2 : 1);
  plan->block_n = tile_n ? tile_n : (nn <= 64 ? 64 : 128);
  if (kind == 1 && b_mn)
    return set_err(CB2_ERR_UNSUPPORTED, "int8 is supported for forward only (the reference skips 1-byte "
                                        "dtypes for backward ops)");
  return CB2_OK;
}

int launch_rowconv(const RowConvPlan &pl, const CUtensorMap &map, const CUtensorMap &map_a, bool tma_gather,
                   const RowConvParams &p, int gx, int gy, cudaStream_t s) {
  // Kernel volumes above 32 (several mask words per row): one variant per shape, with the gather
  // path that is the default for its row width.
#define CB2_INST(K, A, N, M)                                                                      \
  if (pl.kind == K && pl.natom_k == A && pl.block_n == N && pl.b_mn == M) {                        \
    if (p.mask_words > 1)                                                                          \
      return launch_rowconv_inst<K, A, N, M, (A == 1), 4>(map, map_a, p, gx, gy, s);               \
    return tma_gather ? launch_rowconv_inst<K, A, N, M, true>(map, map_a, p, gx, gy, s)            \
                      : launch_rowconv_inst<K, A, N, M, false>(map, map_a, p, gx, gy, s);          \
  }
  CB2_INST(0, 1, 64, false)
  CB2_INST(0, 1, 128, false)
  CB2_INST(0, 2, 64, false)
  CB2_INST(0, 2, 128, false)
  CB2_INST(0, 1, 64, true)
  CB2_INST(0, 1, 128, true)
  CB2_INST(0, 2, 64, true)
  CB2_INST(0, 2, 128, true)
  CB2_INST(1, 1, 64, false)
  CB2_INST(1, 1, 128, false)
#undef CB2_INST
  return set_err(CB2_ERR_UNSUPPORTED, "no row-conv kernel for kind=%d natom=%d block_n=%d b_mn=%d", pl.kind,
                 pl.natom_k, pl.block_n, (int)pl.b_mn);
}

// Common tail of the row-gather launches (forward, backward input, ShuffleAC GEMM).
int run_rowconv(DeviceState *dev, RowConvParams &p, int kind, bool b_mn, int tile_n, int tile_k, void *sched_scratch,
                int max_ctas, const void *w_ptr, uint64_t w_inner, uint64_t w_mid, uint64_t w_outer,
                uint64_t w_mid_stride, uint64_t w_outer_stride, cudaStream_t stream) {
  RowConvPlan pl;
  int rc = plan_rowconv(kind, p.red, p.nn, b_mn, tile_n, tile_k, &pl);
  if (rc)
    return rc;
  const int es = kind == 0 ? 2 : 1;
  const int atom = 128 / es;
  const int kred = pl.natom_k * atom;
  CB2_CHECK_ARG(p.n_rows >= 0, "negative row count");
  if (p.n_rows == 0)
    return CB2_OK;
  CB2_CHECK_ARG((p.red * es) % 16 == 0, "reduction width %d is not a multiple of 16 bytes", p.red);
  CB2_CHECK_ARG((p.nn * es) % 16 == 0, "output width %d is not a multiple of 16 bytes", p.nn);
  CB2_CHECK_ARG((p.lda * es) % 16 == 0 && (p.ldo * es) % 16 == 0, "row strides must be multiples of 16 bytes");
  CB2_CHECK_ARG(aligned16(p.a) && aligned16(p.out), "operand pointers must be 16-byte aligned");
  if (p.src_mode == kSrcRows)
    CB2_CHECK_ARG(aligned16(p.src) && (p.lds * es) % 16 == 0, "source rows must be 16-byte aligned");
  CUtensorMap map;
  rc = make_weight_map(&map, w_ptr, es, w_inner, w_mid, w_outer, w_mid_stride, w_outer_stride, atom,
                       b_mn ? kred : pl.block_n);
  if (rc)
    return rc;
  // Operand rows of up to 128 bytes go through the copy engine (one tile::gather4 request per
  // four rows); wider rows need a request per 128-byte column block, at which point the copy
  // engine's request rate, not memory, bounds a step, and 16-byte cp.async is faster.
  // CUMM_B200_GATHER forces one path for every width.
  const bool tma_gather = (getenv("CUMM_B200_GATHER") && p.mask_words == 1) ? gather_mode() != 0 : pl.natom_k == 1;
  CUtensorMap map_a;
  memset(&map_a, 0, sizeof(map_a));
  if (tma_gather) {
    rc = make_rows_map(&map_a, p.a, es, p.red, p.a_rows, p.lda);
    if (rc)
      return rc;
  }
  p.b_lbo = static_cast<uint32_t>(kred * 128);
  p.b_sbo = 1024;
  p.status = dev->status;
  // Dynamic tile scheduling draws from a pair of device counters that the kernel itself
  // returns to zero: the caller's (one pair per argument record, so a captured launch never
  // shares with anybody), else one from the device's pool taken round-robin, so that eager
  // launches that overlap on different streams use different pairs unless more than
  // kTicketSlots are in flight.
  static std::atomic<unsigned> next_slot{0};
  CB2_CHECK_ARG((reinterpret_cast<uintptr_t>(sched_scratch) & 15u) == 0, "sched_scratch must be 16-byte aligned");
  CB2_CHECK_ARG(max_ctas >= 0, "max_ctas must not be negative");
  static const bool static_tiles = getenv("CUMM_B200_STATIC_TILES") != nullptr;
  p.tickets = static_tiles    ? nullptr
              : sched_scratch ? reinterpret_cast<int *>(sched_scratch)
                              : dev->status + 16 + 2 * (next_slot.fetch_add(1) % kTicketSlots);
  const int ntiles = (p.n_rows + 127) / 128;
  const int gy = (p.nn + pl.block_n - 1) / pl.block_n;
  const int sms = (max_ctas > 0 && max_ctas < dev->num_sms) ? max_ctas : dev->num_sms;
  int gx = sms / gy;
  if (gx < 1)
    gx = 1;
  if (gx > ntiles)
    gx = ntiles;
  return launch_rowconv(pl, map, map_a, tma_gather, p, gx, gy, stream);
}

// ---------------------------------------------------------------- weight gradient
struct WgradLayout {
  int block_n, gy, G, slots, list_stride, n_ctl;
  size_t off_ctl, off_partials, off_lists, total;
};

// Workspace of the weight gradient: 512-byte header (tile counts per offset), the control words,
// fp32 partials (one per unit: at most G + kv - 1), and per offset the list of the
// row tiles that carry it.  G = CTAs per (m, n) tile of the launch.
void wgrad_layout(int num_sms, int max_ctas, int m_total, int n_total, long long n_rows, int kv, int tile_n,
                  WgradLayout *L) {
  L->block_n = (tile_n == 64 || tile_n == 128) ? tile_n : (n_total <= 64 ? 64 : 128);
  const int mt = (m_total + 127) / 128, nt = (n_total + L->block_n - 1) / L->block_n;
  L->gy = mt * nt;
  const int sms = (max_ctas > 0 && max_ctas < num_sms) ? max_ctas : num_sms;
  L->G = sms / L->gy;
  if (L->G < 1)
    L->G = 1;
  L->slots = L->G + (kv > 32 ? kv : 32);
  const int kvs = kv > 0 ? kv : 1;
  L->n_ctl = kWgradCtlBase + 4 * kvs * L->gy;
  L->off_ctl = 512;
  L->off_partials = L->off_ctl + ((size_t)L->n_ctl * 4 + 255) / 256 * 256;
  L->off_lists = L->off_partials + (size_t)L->slots * L->gy * 128 * L->block_n * 4;
  const long long ntiles = (n_rows + 127) / 128;
  L->list_stride = (int)((ntiles + 63) / 64 * 64);
  L->total = L->off_lists + (size_t)kvs * L->list_stride * 4;
}

template <int BLOCK_N, int GATHER>
int launch_wgrad_inst(const CUtensorMap &ma, const CUtensorMap &mb, const WgradParams &p, int gx, int gy,
                      cudaStream_t stream) {
  using Cfg = WgradCfg<BLOCK_N, GATHER>;
  auto kern = wgrad_kernel<BLOCK_N, GATHER>;
  static std::atomic<uint64_t> configured{0};
  static std::atomic<int> regs{0};
  int dev = 0;
  CB2_CUDA(cudaGetDevice(&dev));
  if (!(configured.load() & (1ull << dev))) {
    CB2_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    regs.store(kernel_regs(kern));
    configured.fetch_or(1ull << dev);
  }
  g_last_launch.num_regs = regs.load();
  g_last_launch.num_threads = Cfg::THREADS;
  g_last_launch.smem_bytes = Cfg::SMEM_BYTES;
  CB2_CUDA(launch_after(1, kern, dim3(gx, gy), dim3(Cfg::THREADS), Cfg::SMEM_BYTES, stream, ma, mb, p));
  g_launches.fetch_add(1);
  return CB2_OK;
}

int run_wgrad(DeviceState *dev, WgradParams &p, int tile_n, int max_ctas, int reuse_plan, void *workspace,
              size_t workspace_bytes, cudaStream_t stream) {
  CB2_CHECK_RT(tile_n == 0 || tile_n == 64 || tile_n == 128,
               "can't find any suitable algo: tile_shape[1] = %d (kernels exist for 64 and 128)", tile_n);
  CB2_CHECK_ARG(max_ctas >= 0, "max_ctas must not be negative");
  WgradLayout L;
  wgrad_layout(dev->num_sms, max_ctas, p.m_total, p.n_total, p.n_rows, p.kv, tile_n, &L);
  CB2_CHECK_RT(workspace != nullptr && workspace_bytes >= L.total, "workspace at least %zu bytes.", L.total);
  CB2_CHECK_ARG(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, "workspace must be 256-byte aligned");
  CB2_CHECK_RT(L.gy <= kWgradMaxOutTiles, "the weight gradient has %d output tiles of 128 x %d; at most %d are supported",
               L.gy, L.block_n, kWgradMaxOutTiles);
  CB2_CHECK_ARG(p.m_total % 8 == 0 && p.n_total % 8 == 0, "channel counts must be multiples of 8");
  CB2_CHECK_ARG((p.ld_dout * 2) % 16 == 0 && (p.ld_x * 2) % 16 == 0, "row strides must be multiples of 16 bytes");
  CB2_CHECK_ARG(aligned16(p.dout) && aligned16(p.x), "operand pointers must be 16-byte aligned");
  CB2_CHECK_ARG((reinterpret_cast<uintptr_t>(p.out) & 7u) == 0 && (reinterpret_cast<uintptr_t>(p.src) & 7u) == 0 &&
                    p.ldo % 4 == 0 && p.f_stride % 4 == 0,
                "the weight gradient and its row / offset strides must be 8-byte aligned");
  uint8_t *ws = reinterpret_cast<uint8_t *>(workspace);
  p.sched = reinterpret_cast<int *>(ws);
  p.ctl = reinterpret_cast<int *>(ws + L.off_ctl);
  p.partials = reinterpret_cast<float *>(ws + L.off_partials);
  p.lists = reinterpret_cast<const int *>(ws + L.off_lists);
  p.list_stride = L.list_stride;
  p.status = dev->status;
  if (!reuse_plan) {
    // counts and lists of the row tiles per offset; control words to zero
    wgrad_plan_kernel<<<p.kv, 1024, 0, stream>>>(p, reinterpret_cast<int *>(ws + L.off_lists), L.list_stride, L.n_ctl);
    CB2_CUDA(cudaGetLastError());
    g_launches.fetch_add(1);
  }
  CUtensorMap ma, mb;
  int rc = make_rows_map(&ma, p.dout, 2, p.m_total, p.a_rows, p.ld_dout);
  if (rc)
    return rc;
  rc = make_rows_map(&mb, p.x, 2, p.n_total, p.b_rows, p.ld_x);
  if (rc)
    return rc;
  const bool tma = gather_mode() != 0;
  if (L.block_n == 64)
    return tma ? launch_wgrad_inst<64, kGatherTma4>(ma, mb, p, L.G, L.gy, stream)
               : launch_wgrad_inst<64, kGatherCpAsync>(ma, mb, p, L.G, L.gy, stream);
  return tma ? launch_wgrad_inst<128, kGatherTma4>(ma, mb, p, L.G, L.gy, stream)
             : launch_wgrad_inst<128, kGatherCpAsync>(ma, mb, p, L.G, L.gy, stream);
}

// ---------------------------------------------------------------- allocation-free variant
// Scratch for cb2_conv_backward_weight_static: lives in the library image, one copy per GPU
// that loads it, for the life of the process.  In host code this name is only a handle for
// cudaGetSymbolAddress, never a pointer a kernel may be given.
constexpr size_t kStaticScratchBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ int g_static_status[16];

struct StaticState {
  bool ready = false;
  DeviceState dev;  // num_sms, and `status` pointing at g_static_status on that device
  void *scratch = nullptr;
};
StaticState g_static[kMaxDevices];

// Per-device set-up of the allocation-free path, with that device current: resolves the
// device addresses of the two static arrays.  Nothing here allocates.
int get_device_static(StaticState **out) {
  int dev = 0;
  CB2_CUDA(cudaGetDevice(&dev));
  CB2_CHECK_RT(dev >= 0 && dev < kMaxDevices, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  StaticState &st = g_static[dev];
  if (!st.ready) {
    cudaDeviceProp prop;
    CB2_CUDA(cudaGetDeviceProperties(&prop, dev));
    CB2_CHECK_RT(prop.major == 10, "cumm_b200 kernels are built for sm_100a only; device %d is sm_%d%d", dev,
                 prop.major, prop.minor);
    st.dev.num_sms = prop.multiProcessorCount;
    void *scratch = nullptr, *status = nullptr;
    CB2_CUDA(cudaGetSymbolAddress(&scratch, g_static_scratch));
    CB2_CUDA(cudaGetSymbolAddress(&status, g_static_status));
    CB2_CHECK_RT(scratch != nullptr && status != nullptr, "could not resolve the static scratch on device %d", dev);
    st.scratch = scratch;
    st.dev.status = reinterpret_cast<int *>(status);
    st.dev.ready = true;
    st.ready = true;
  }
  if (!g_encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    CB2_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    CB2_CHECK_RT(fn != nullptr && q == cudaDriverEntryPointSuccess, "cuTensorMapEncodeTiled not available");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  *out = &st;
  return CB2_OK;
}

int kind_of(int da, int db, int dc, int is_int8, bool allow_f32_out) {
  if (da == CB2_DTYPE_F16 && db == CB2_DTYPE_F16 &&
      (dc == CB2_DTYPE_F16 || (allow_f32_out && dc == CB2_DTYPE_F32)) && !is_int8)
    return 0;
  if (da == CB2_DTYPE_I8 && db == CB2_DTYPE_I8 && dc == CB2_DTYPE_I8 && is_int8)
    return 1;
  return -1;
}

} // namespace

extern "C" {

#ifdef CB2_TRACE
// Debug builds only: copy the device trace buffer to the host and reset it.
int cb2_debug_read_trace(void *host_dst, size_t bytes) {
  if (bytes != sizeof(cb2::TraceBuf))
    return set_err(CB2_ERR_INVALID_ARG, "trace buffer is %zu bytes", sizeof(cb2::TraceBuf));
  CB2_CUDA(cudaDeviceSynchronize());
  CB2_CUDA(cudaMemcpyFromSymbol(host_dst, cb2::g_trace, bytes));
  static cb2::TraceBuf zero;
  CB2_CUDA(cudaMemcpyToSymbol(cb2::g_trace, &zero, bytes));
  return CB2_OK;
}
#endif

} // extern "C" (reopened below, after the helpers of the table builder)

// ---------------------------------------------------------------- neighbour tables on the GPU
namespace {

struct PairgenLayout {
  cb2pg::Geometry g;
  uint32_t cap_in, cap_set;  // hash capacities (powers of two)
  long long list_cap;        // active outputs a strided conv can have at most
  long long nmax;            // rows the mask sorts may have to hold
  int key_bits;
  int words;                 // mask words per row
  size_t off_in_keys, off_in_vals, off_set_keys, off_list_a, off_list_b, off_m, off_v, off_hist, off_counters, total;
  size_t off_rows, off_k;    // several mask words per row: the unsorted rows, and the key array of a word's sort
};

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

uint32_t pow2_at_least(unsigned long long v) {
  uint32_t c = 64;
  while (c < v && c < (1u << 31))
    c <<= 1;
  return c;
}

int pairgen_layout(const cb2_pairgen_args *a, PairgenLayout *L) {
  CB2_CHECK_ARG(a != nullptr, "null arguments");
  CB2_CHECK_ARG(a->n_in >= 0 && a->batch_size >= 1, "bad n_in / batch_size (%d, %d)", a->n_in, a->batch_size);
  long long kv = 1, cells = a->batch_size;
  for (int i = 0; i < 3; ++i) {
    CB2_CHECK_ARG(a->grid[i] >= 1 && a->ksize[i] >= 1 && a->stride[i] >= 1 && a->dil[i] >= 1 && a->pad[i] >= 0,
                  "bad geometry on axis %d", i);
    L->g.grid[i] = a->grid[i];
    L->g.ksize[i] = a->ksize[i];
    L->g.stride[i] = a->stride[i];
    L->g.pad[i] = a->pad[i];
    L->g.dil[i] = a->dil[i];
    const int span = a->grid[i] + 2 * a->pad[i] - a->dil[i] * (a->ksize[i] - 1) - 1;
    L->g.ogrid[i] = a->subm ? a->grid[i] : (span >= 0 ? span / a->stride[i] + 1 : 0);
    CB2_CHECK_ARG(L->g.ogrid[i] >= 1, "the kernel does not fit the grid on axis %d", i);
    kv *= a->ksize[i];
    cells *= L->g.ogrid[i];
  }
  CB2_CHECK_RT(kv <= 128, "kernel volume %lld is not supported (masks hold up to 128 offsets)", kv);
  if (a->subm)
    for (int i = 0; i < 3; ++i)
      CB2_CHECK_ARG(a->stride[i] == 1, "a submanifold convolution has stride 1");
  L->g.kv = static_cast<int>(kv);
  L->words = static_cast<int>((kv + 31) / 32);
  L->g.batch_size = a->batch_size;
  L->cap_in = pow2_at_least(2ull * static_cast<unsigned long long>(a->n_in));
  // outputs an input can feed: per axis, the offsets r with (in + pad - r * dil) divisible by the stride
  long long per_input = 1;
  for (int i = 0; i < 3; ++i) {
    int gcd = a->stride[i], b = a->dil[i];
    while (b) {
      const int t = gcd % b;
      gcd = b;
      b = t;
    }
    const int period = a->stride[i] / gcd;  // r takes every period-th value
    per_input *= std::min(a->ksize[i], (a->ksize[i] + period - 1) / period);
  }
  L->list_cap = a->subm ? 0 : std::min<long long>(static_cast<long long>(a->n_in) * per_input, cells);
  CB2_CHECK_RT(L->list_cap < (1ll << 30), "too many candidate outputs (%lld)", L->list_cap);
  L->cap_set = a->subm ? 0 : pow2_at_least(2ull * static_cast<unsigned long long>(L->list_cap));
  L->nmax = std::max<long long>(a->subm ? a->n_in : L->list_cap, a->n_in);
  L->key_bits = 1;
  while (L->key_bits < 63 && (1ll << L->key_bits) < cells)
    ++L->key_bits;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off = align256(off + bytes);
    return at;
  };
  L->off_counters = take(256);
  L->off_in_keys = take(static_cast<size_t>(L->cap_in) * 8);
  L->off_in_vals = take(static_cast<size_t>(L->cap_in) * 4);
  L->off_set_keys = take(static_cast<size_t>(L->cap_set) * 8);
  L->off_list_a = take(static_cast<size_t>(L->list_cap) * 8);
  L->off_list_b = take(static_cast<size_t>(L->list_cap) * 8);
  L->off_m = take(static_cast<size_t>(L->nmax) * 4);
  L->off_v = take(static_cast<size_t>(L->nmax) * 4);
  const long long sort_n = std::max<long long>(L->nmax, L->list_cap);
  L->off_hist = take(static_cast<size_t>(256) * ((sort_n + cb2pg::kSortTile - 1) / cb2pg::kSortTile + 1) * 4);
  L->off_rows = L->off_k = 0;
  if (L->words > 1) {
    L->off_rows = take(static_cast<size_t>(L->nmax) * L->words * 4);
    L->off_k = take(static_cast<size_t>(L->nmax) * 4);
  }
  L->total = off;
  return CB2_OK;
}

// Stable ascending sort of n keys (and values) on `bits` low bits, 8 per pass, ping-ponging
// between the result buffers and the scratch buffers.  The unsorted input has to be where
// sort_source() says -- the scratch pair for an odd number of passes, the result pair for an
// even number -- so that the last pass lands in the result buffers.
inline int sort_passes(int bits) { return bits <= 8 ? 1 : (bits + 7) / 8; }
template <typename T> T *sort_source(T *result, T *scratch, int bits) {
  return sort_passes(bits) % 2 ? scratch : result;
}
template <typename K, bool HAS_VAL>
int radix_sort(K *k_result, int *v_result, K *k_scratch, int *v_scratch, int n, int bits, int *hist, cudaStream_t s) {
  if (n <= 0)
    return CB2_OK;
  const int passes = sort_passes(bits);
  const int ntiles = (n + cb2pg::kSortTile - 1) / cb2pg::kSortTile;
  K *ks = sort_source(k_result, k_scratch, bits), *kd = (ks == k_result) ? k_scratch : k_result;
  int *vs = sort_source(v_result, v_scratch, bits), *vd = (vs == v_result) ? v_scratch : v_result;
  for (int p = 0; p < passes; ++p) {
    cb2pg::sort_hist_kernel<K><<<ntiles, cb2pg::kSortThreads, 0, s>>>(ks, n, 8 * p, hist, ntiles);
    cb2pg::sort_scan_kernel<<<1, 1024, 0, s>>>(reinterpret_cast<int4 *>(hist), (256 * ntiles + 3) / 4);
    cb2pg::sort_scatter_kernel<K, HAS_VAL><<<ntiles, cb2pg::kSortThreads, 0, s>>>(ks, vs, kd, vd, n, 8 * p, hist, ntiles);
    CB2_CUDA(cudaGetLastError());
    g_launches.fetch_add(3);
    std::swap(ks, kd);
    std::swap(vs, vd);
  }
  return CB2_OK;
}

// Masks of `words` words per row from a finished table, sorted (see mask_words_from_table_kernel):
// writes mask [n, words] and mask_argsort [n].
int sort_mask_words(const int32_t *table, int n, int kv, int words, uint32_t *rows, uint32_t *k_result,
                    uint32_t *k_scratch, int *v_scratch, uint32_t *mask, int *argsort, int *hist, cudaStream_t s) {
  const unsigned blocks = static_cast<unsigned>((n + 255) / 256);
  cb2pg::mask_words_from_table_kernel<<<blocks, 256, 0, s>>>(table, n, kv, words, rows);
  g_launches.fetch_add(1);
  for (int w = 0; w < words; ++w) {
    const int bits = std::min(32, kv - 32 * w);
    cb2pg::gather_word_kernel<<<blocks, 256, 0, s>>>(rows, w == 0 ? nullptr : argsort, n, words, w,
                                                     sort_source(k_result, k_scratch, bits),
                                                     sort_source(argsort, v_scratch, bits));
    CB2_CUDA(cudaGetLastError());
    g_launches.fetch_add(1);
    const int rc = radix_sort<uint32_t, true>(k_result, argsort, k_scratch, v_scratch, n, bits, hist, s);
    if (rc)
      return rc;
  }
  const long long total = static_cast<long long>(n) * words;
  cb2pg::gather_rows_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(rows, argsort, n, words, mask);
  CB2_CUDA(cudaGetLastError());
  g_launches.fetch_add(1);
  return CB2_OK;
}

int pairgen_common(const cb2_pairgen_args *a, PairgenLayout *L, DeviceState **dev) {
  int rc = get_device(dev);
  if (rc)
    return rc;
  rc = pairgen_layout(a, L);
  if (rc)
    return rc;
  CB2_CHECK_RT(a->in_coords != nullptr || a->n_in == 0, "in_coords must not empty");
  CB2_CHECK_ARG(aligned16(a->in_coords), "in_coords must be 16-byte aligned");
  CB2_CHECK_RT(a->workspace != nullptr && a->workspace_bytes >= L->total, "workspace at least %zu bytes.", L->total);
  CB2_CHECK_ARG(reinterpret_cast<uintptr_t>(a->workspace) % 256 == 0, "workspace must be 256-byte aligned");
  return CB2_OK;
}

} // namespace

extern "C" {

size_t cb2_pairgen_workspace_size(const cb2_pairgen_args *a) {
  PairgenLayout L;
  if (pairgen_layout(a, &L))
    return 0;
  return L.total;
}

int cb2_pairgen_count_outputs(const cb2_pairgen_args *a, int *n_out, void *stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  PairgenLayout L;
  DeviceState *dev;
  int rc = pairgen_common(a, &L, &dev);
  if (rc)
    return rc;
  CB2_CHECK_ARG(n_out != nullptr, "n_out must not be null");
  if (a->subm || a->n_in == 0) {
    *n_out = a->n_in;
    return CB2_OK;
  }
  uint8_t *ws = reinterpret_cast<uint8_t *>(a->workspace);
  int *counter = reinterpret_cast<int *>(ws + L.off_counters);
  unsigned long long *set_keys = reinterpret_cast<unsigned long long *>(ws + L.off_set_keys);
  unsigned long long *list_a = reinterpret_cast<unsigned long long *>(ws + L.off_list_a);
  unsigned long long *list_b = reinterpret_cast<unsigned long long *>(ws + L.off_list_b);
  CB2_CUDA(cudaMemsetAsync(counter, 0, 256, stream));
  CB2_CUDA(cudaMemsetAsync(set_keys, 0xFF, static_cast<size_t>(L.cap_set) * 8, stream));
  cb2pg::out_candidates_kernel<<<(a->n_in + 255) / 256, 256, 0, stream>>>(
      a->in_coords, a->n_in, L.g, set_keys, L.cap_set - 1, sort_source(list_a, list_b, L.key_bits),
      static_cast<int>(L.list_cap), counter, dev->status);
  CB2_CUDA(cudaGetLastError());
  g_launches.fetch_add(1);
  int count = 0;
  CB2_CUDA(cudaMemcpyAsync(&count, counter, sizeof(int), cudaMemcpyDeviceToHost, stream));
  CB2_CUDA(cudaStreamSynchronize(stream));
  CB2_CHECK_RT(count >= 0 && count <= L.list_cap, "active-output count %d out of range", count);
  rc = radix_sort<unsigned long long, false>(list_a, nullptr, list_b, nullptr, count, L.key_bits,
                                             reinterpret_cast<int *>(ws + L.off_hist), stream);
  if (rc)
    return rc;
  *n_out = count;
  return CB2_OK;
}

int cb2_pairgen_run(const cb2_pairgen_args *a, void *stream_v) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  PairgenLayout L;
  DeviceState *dev;
  int rc = pairgen_common(a, &L, &dev);
  if (rc)
    return rc;
  const int n_in = a->n_in;
  const int n_out = a->subm ? n_in : a->n_out;
  CB2_CHECK_ARG(n_out >= 0 && n_out <= L.nmax, "n_out %d out of range", n_out);
  if (n_out == 0)
    return CB2_OK;
  CB2_CHECK_RT(a->indices && a->mask && a->mask_argsort, "error: indices, mask or mask_argsort empty");
  CB2_CHECK_RT(a->subm || a->out_coords, "out_coords must not empty");
  CB2_CHECK_ARG(a->subm || aligned16(a->out_coords), "out_coords must be 16-byte aligned");
  const bool bwd = a->indices_bwd != nullptr;
  CB2_CHECK_RT(!bwd || (a->mask_bwd && a->mask_argsort_bwd), "error: backward mask or mask_argsort empty");
  uint8_t *ws = reinterpret_cast<uint8_t *>(a->workspace);
  unsigned long long *in_keys = reinterpret_cast<unsigned long long *>(ws + L.off_in_keys);
  int *in_vals = reinterpret_cast<int *>(ws + L.off_in_vals);
  uint32_t *m_tmp = reinterpret_cast<uint32_t *>(ws + L.off_m);
  int *v_tmp = reinterpret_cast<int *>(ws + L.off_v);
  int *hist = reinterpret_cast<int *>(ws + L.off_hist);
  CB2_CUDA(cudaMemsetAsync(in_keys, 0xFF, static_cast<size_t>(L.cap_in) * 8, stream));
  CB2_CUDA(cudaMemsetAsync(in_vals, 0x7F, static_cast<size_t>(L.cap_in) * 4, stream));
  cb2pg::hash_insert_kernel<<<(n_in + 255) / 256, 256, 0, stream>>>(a->in_coords, n_in, L.g, in_keys, in_vals,
                                                                     L.cap_in - 1, dev->status);
  const int32_t *out_coords = a->in_coords;
  if (!a->subm) {
    cb2pg::decode_out_coords_kernel<<<(n_out + 255) / 256, 256, 0, stream>>>(
        reinterpret_cast<const unsigned long long *>(ws + L.off_list_a), n_out, L.g, a->out_coords);
    out_coords = a->out_coords;
    g_launches.fetch_add(1);
  }
  const bool wide = L.words > 1;
  uint32_t *rows = reinterpret_cast<uint32_t *>(ws + L.off_rows), *k_res = reinterpret_cast<uint32_t *>(ws + L.off_k);
  // several mask words per row: the probe's one-word mask and row numbers go to scratch, the masks
  // are built from the finished table instead
  cb2pg::probe_kernel<<<(n_out + 255) / 256, 256, 0, stream>>>(
      out_coords, n_out, L.g, in_keys, in_vals, L.cap_in - 1, a->indices,
      wide ? m_tmp : sort_source(a->mask, m_tmp, L.g.kv), wide ? v_tmp : sort_source(a->mask_argsort, v_tmp, L.g.kv));
  CB2_CUDA(cudaGetLastError());
  g_launches.fetch_add(2);
  if (wide)
    rc = sort_mask_words(a->indices, n_out, L.g.kv, L.words, rows, k_res, m_tmp, v_tmp, a->mask, a->mask_argsort, hist,
                         stream);
  else
    rc = radix_sort<uint32_t, true>(a->mask, a->mask_argsort, m_tmp, v_tmp, n_out, L.g.kv, hist, stream);
  if (rc)
    return rc;
  if (a->tile_masks) {
    if (wide)
      cb2pg::tile_masks_words_kernel<<<((n_out + 127) / 128 + 7) / 8, 256, 0, stream>>>(a->mask, n_out, L.words,
                                                                                       a->tile_masks);
    else
      cb2pg::tile_masks_kernel<<<((n_out + 127) / 128 + 7) / 8, 256, 0, stream>>>(a->mask, n_out, a->tile_masks);
    CB2_CUDA(cudaGetLastError());
    g_launches.fetch_add(1);
  }
  if (bwd) {
    CB2_CUDA(cudaMemsetAsync(a->indices_bwd, 0xFF, static_cast<size_t>(L.g.kv) * n_in * 4, stream));
    const long long threads = static_cast<long long>(n_out) * L.g.kv;
    cb2pg::invert_table_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, stream>>>(
        a->indices, n_out, L.g.kv, n_in, a->indices_bwd);
    CB2_CUDA(cudaGetLastError());
    g_launches.fetch_add(1);
    if (wide) {
      rc = sort_mask_words(a->indices_bwd, n_in, L.g.kv, L.words, rows, k_res, m_tmp, v_tmp, a->mask_bwd,
                           a->mask_argsort_bwd, hist, stream);
    } else {
      cb2pg::mask_from_table_kernel<<<(n_in + 255) / 256, 256, 0, stream>>>(
          a->indices_bwd, n_in, L.g.kv, sort_source(a->mask_bwd, m_tmp, L.g.kv),
          sort_source(a->mask_argsort_bwd, v_tmp, L.g.kv));
      CB2_CUDA(cudaGetLastError());
      g_launches.fetch_add(1);
      rc = radix_sort<uint32_t, true>(a->mask_bwd, a->mask_argsort_bwd, m_tmp, v_tmp, n_in, L.g.kv, hist, stream);
    }
    if (rc)
      return rc;
  }
  return CB2_OK;
}

// ---------------------------------------------------------------- a layer's ShuffleAC calls in one launch
struct SeqLayout {
  size_t off_table, off_mask, off_argsort, off_m, off_v, off_hist, off_tickets, total;
};
static void seq_layout(int count, long long n, SeqLayout *L) {
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off = align256(off + bytes);
    return at;
  };
  L->off_tickets = take(256);
  L->off_table = take(static_cast<size_t>(count) * n * 4);
  L->off_mask = take(static_cast<size_t>(n) * 4);
  L->off_argsort = take(static_cast<size_t>(n) * 4);
  L->off_m = take(static_cast<size_t>(n) * 4);
  L->off_v = take(static_cast<size_t>(n) * 4);
  L->off_hist = take(static_cast<size_t>(256) * ((n + cb2pg::kSortTile - 1) / cb2pg::kSortTile + 1) * 4);
  L->total = off;
}

size_t cb2_gemm_sequence_workspace_size(const cb2_gemm_sequence_args *a) {
  if (!a || a->count < 1 || a->count > cb2pg::kSeqMaxCalls || a->n_out_rows < 0)
    return 0;
  SeqLayout L;
  seq_layout(a->count, a->n_out_rows, &L);
  return L.total;
}

int cb2_gemm_sequence_run(const cb2_gemm_sequence_args *a, void *stream_v) {
  CB2_CHECK_ARG(a != nullptr && a->calls != nullptr, "null arguments");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  DeviceState *dev;
  int rc = get_device(&dev);
  if (rc)
    return rc;
  CB2_CHECK_ARG(a->count >= 1 && a->count <= cb2pg::kSeqMaxCalls, "a sequence holds 1 to %d calls", cb2pg::kSeqMaxCalls);
  CB2_CHECK_ARG(a->n_out_rows >= 0, "negative row count");
  const cb2_gemm_args &c0 = a->calls[0];
  CB2_CHECK_RT(c0.ptr_A && c0.ptr_B && c0.ptr_C, "a,b,c must not empty");
  CB2_CHECK_RT(kind_of(c0.dtype_a, c0.dtype_b, c0.dtype_c, 0, false) == 0,
               "can't find any suitable algo for dtypes (%d,%d,%d): only f16,f16,f16 is built", c0.dtype_a, c0.dtype_b,
               c0.dtype_c);
  CB2_CHECK_ARG(c0.k % 8 == 0 && c0.n % 8 == 0, "this m, n, k isn't supported due to misaligned contiguous dim.");
  // what makes the calls one layer
  const long long b_step = a->count > 1 ? (reinterpret_cast<const char *>(a->calls[1].ptr_B) -
                                           reinterpret_cast<const char *>(c0.ptr_B))
                                        : 0;
  cb2pg::SeqPairLists lists;
  memset(&lists, 0, sizeof(lists));
  lists.count = a->count;
  for (int f = 0; f < a->count; ++f) {
    const cb2_gemm_args &c = a->calls[f];
    const bool same = c.shuffle_type == CB2_SHUFFLE_AC && !c.trans_a && !c.trans_c && c.trans_b == c0.trans_b &&
                      c.ptr_A == c0.ptr_A && c.stride_A == c0.stride_A && c.rows_A == c0.rows_A && c.ptr_C == c0.ptr_C &&
                      c.stride_C == c0.stride_C && (c.ptr_D == nullptr || c.ptr_D == c.ptr_C) && !c.d_is_vector &&
                      c.n == c0.n && c.k == c0.k && c.stride_B == c0.stride_B && c.alpha == 1.f && c.beta == 1.f &&
                      c.act_type == CB2_ACT_NONE && c.dtype_a == c0.dtype_a && c.dtype_b == c0.dtype_b &&
                      c.dtype_c == c0.dtype_c && c.m >= 0 && c.indiceBorC != nullptr &&
                      reinterpret_cast<const char *>(c.ptr_B) - reinterpret_cast<const char *>(c0.ptr_B) == f * b_step;
    if (!same)
      return set_err(CB2_ERR_UNSUPPORTED,
                     "call %d of the sequence does not fit the layer form (ShuffleAC, shared A and C, alpha = beta = 1, "
                     "no activation, equally spaced B): run the calls one by one",
                     f);
    lists.a_inds[f] = c.indiceA;
    lists.c_inds[f] = c.indiceBorC;
    lists.first[f + 1] = lists.first[f] + c.m;
  }
  CB2_CHECK_RT(b_step % 2 == 0 && b_step >= 0, "B matrices must be ascending slices of one tensor");
  const int n = a->n_out_rows;
  if (n == 0)
    return CB2_OK;
  SeqLayout L;
  seq_layout(a->count, n, &L);
  CB2_CHECK_RT(a->workspace != nullptr && a->workspace_bytes >= L.total, "workspace at least %zu bytes.", L.total);
  CB2_CHECK_ARG(reinterpret_cast<uintptr_t>(a->workspace) % 256 == 0, "workspace must be 256-byte aligned");
  uint8_t *ws = reinterpret_cast<uint8_t *>(a->workspace);
  int32_t *table = reinterpret_cast<int32_t *>(ws + L.off_table);
  uint32_t *mask = reinterpret_cast<uint32_t *>(ws + L.off_mask);
  int32_t *argsort = reinterpret_cast<int32_t *>(ws + L.off_argsort);
  if (!a->reuse_tables) {
    uint32_t *m_tmp = reinterpret_cast<uint32_t *>(ws + L.off_m);
    int *v_tmp = reinterpret_cast<int *>(ws + L.off_v);
    CB2_CUDA(cudaMemsetAsync(ws + L.off_tickets, 0, 256, stream));
    CB2_CUDA(cudaMemsetAsync(table, 0xFF, static_cast<size_t>(a->count) * n * 4, stream));
    const long long pairs = lists.first[a->count];
    if (pairs > 0)
      cb2pg::seq_scatter_kernel<<<static_cast<unsigned>((pairs + 255) / 256), 256, 0, stream>>>(lists, n, c0.rows_A, table,
                                                                                              dev->status);
    cb2pg::mask_from_table_kernel<<<(n + 255) / 256, 256, 0, stream>>>(table, n, a->count, sort_source(mask, m_tmp, a->count),
                                                                        sort_source(argsort, v_tmp, a->count));
    CB2_CUDA(cudaGetLastError());
    g_launches.fetch_add(2);
    rc = radix_sort<uint32_t, true>(mask, argsort, m_tmp, v_tmp, n, a->count, reinterpret_cast<int *>(ws + L.off_hist), stream);
    if (rc)
      return rc;
  }
  RowConvParams p;
  memset(&p, 0, sizeof(p));
  p.a = c0.ptr_A;
  p.out = c0.ptr_C;
  p.indices = table;
  p.mask = mask;
  p.argsort = argsort;
  p.n_rows = n;
  p.a_rows = c0.rows_A;
  p.red = c0.k;
  p.nn = c0.n;
  p.lda = c0.stride_A;
  p.ldo = c0.stride_C;
  p.kv = a->count;
  p.mask_words = 1;
  p.mode = kModeMaskConv;
  p.mask_filter = 0xffffffffu;
  p.alpha = 1.f;
  p.beta = 1.f;
  p.src = c0.ptr_C;
  p.src_mode = kSrcRows;
  p.lds = c0.stride_C;
  // the weight tensor as [outer, f, inner]: B_f is [n, k] (trans_b) or [k, n]
  const bool b_mn = !c0.trans_b;
  const uint64_t inner = b_mn ? c0.n : c0.k, outer = b_mn ? c0.k : c0.n;
  const uint64_t f_stride = a->count > 1 ? static_cast<uint64_t>(b_step / 2) : inner;
  return run_rowconv(dev, p, 0, b_mn, c0.tile_n, c0.tile_k, ws + L.off_tickets, c0.max_ctas, c0.ptr_B, inner, a->count, outer,
                     f_stride, c0.stride_B, stream);
}

// ---------------------------------------------------------------- tables of a dense convolution
int cb2_dense_tables_run(const cb2_dense_tables_args *a, void *stream_v) {
  CB2_CHECK_ARG(a != nullptr, "null arguments");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  DeviceState *dev;
  int rc = get_device(&dev);
  if (rc)
    return rc;
  cb2pg::DenseGeometry g;
  g.batch = a->batch;
  long long n_in = a->batch, n_out = a->batch, kv = 1;
  CB2_CHECK_ARG(a->batch >= 1, "bad batch %d", a->batch);
  for (int i = 0; i < 3; ++i) {
    CB2_CHECK_ARG(a->in_dims[i] >= 1 && a->out_dims[i] >= 1 && a->ksize[i] >= 1 && a->stride[i] >= 1 &&
                      a->dil[i] >= 1 && a->pad[i] >= 0,
                  "bad geometry on axis %d", i);
    const int span = a->in_dims[i] + 2 * a->pad[i] - a->dil[i] * (a->ksize[i] - 1) - 1;
    CB2_CHECK_ARG(span >= 0 && a->out_dims[i] == span / a->stride[i] + 1,
                  "output extent %d on axis %d does not match input %d, kernel %d, stride %d, padding %d, dilation %d",
                  a->out_dims[i], i, a->in_dims[i], a->ksize[i], a->stride[i], a->pad[i], a->dil[i]);
    g.in_dims[i] = a->in_dims[i];
    g.out_dims[i] = a->out_dims[i];
    g.ksize[i] = a->ksize[i];
    g.stride[i] = a->stride[i];
    g.pad[i] = a->pad[i];
    g.dil[i] = a->dil[i];
    n_in *= a->in_dims[i];
    n_out *= a->out_dims[i];
    kv *= a->ksize[i];
  }
  CB2_CHECK_RT(kv <= 128, "kernel volume %lld: the kernels handle up to 128 filter offsets", kv);
  CB2_CHECK_RT(n_in < (1ll << 31) && n_out < (1ll << 31), "too many rows for 32-bit row indices");
  CB2_CHECK_RT(a->indices_fwd != nullptr, "error: indices empty");
  g.kv = (int)kv;
  const int words = ((int)kv + 31) / 32;
  auto blocks = [](long long n) { return (unsigned)((n + 255) / 256); };
  cb2pg::dense_table_fwd_kernel<<<blocks(n_out * kv), 256, 0, stream>>>(g, n_out, a->indices_fwd);
  g_launches.fetch_add(1);
  if (a->indices_bwd) {
    cb2pg::dense_table_bwd_kernel<<<blocks(n_in * kv), 256, 0, stream>>>(g, n_in, a->indices_bwd);
    g_launches.fetch_add(1);
  }
  if (a->mask_fwd && a->argsort_fwd) {
    cb2pg::dense_masks_kernel<<<blocks(n_out), 256, 0, stream>>>(n_out, (int)kv, words, a->mask_fwd, a->argsort_fwd);
    g_launches.fetch_add(1);
  }
  if (a->mask_bwd && a->argsort_bwd) {
    cb2pg::dense_masks_kernel<<<blocks(n_in), 256, 0, stream>>>(n_in, (int)kv, words, a->mask_bwd, a->argsort_bwd);
    g_launches.fetch_add(1);
  }
  CB2_CUDA(cudaGetLastError());
  return CB2_OK;
}

// ---------------------------------------------------------------- sum over GPUs through peer memory
struct PeerLayout {
  long long shard_f4, shard_bytes, result_bytes;
  size_t total;
};
static void peer_layout(long long numel, int world, PeerLayout *L) {
  const long long n4 = numel / 4;
  L->shard_f4 = (n4 + world - 1) / world;
  // a float4 travels as two 16-byte lines: two floats and two copies of the call number each
  L->shard_bytes = static_cast<long long>(align256(static_cast<size_t>(L->shard_f4) * cb2::kPeerLineBytesPerF4));
  L->result_bytes = static_cast<long long>(align256(static_cast<size_t>(n4) * cb2::kPeerLineBytesPerF4));
  L->total = cb2::kPeerControlBytes + 2 * static_cast<size_t>(world) * L->shard_bytes + 2 * static_cast<size_t>(L->result_bytes);
}

size_t cb2_peer_allreduce_buffer_size(long long numel, int world) {
  if (numel <= 0 || numel % 4 || numel / 4 > 0x3fffffff || world < 1 || world > cb2::kPeerMaxWorld)
    return 0;
  PeerLayout L;
  peer_layout(numel, world, &L);
  return L.total;
}

int cb2_peer_allreduce(const cb2_peer_allreduce_args *a, void *stream_v) {
  CB2_CHECK_ARG(a != nullptr, "null arguments");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  DeviceState *dev;
  int rc = get_device(&dev);
  if (rc)
    return rc;
  CB2_CHECK_ARG(a->world >= 1 && a->world <= cb2::kPeerMaxWorld && a->rank >= 0 && a->rank < a->world,
                "bad rank / world (%d, %d)", a->rank, a->world);
  CB2_CHECK_ARG(a->numel > 0 && a->numel % 4 == 0 && a->numel / 4 <= 0x3fffffff, "numel must be a positive multiple of 4 below 2^32");
  CB2_CHECK_RT(a->peer_buffers && a->src && (a->out_f32 || a->out_f16), "buffers, source and an output must not empty");
  CB2_CHECK_ARG(aligned16(a->src) && aligned16(a->out_f32) && (reinterpret_cast<uintptr_t>(a->out_f16) & 7u) == 0,
                "source and outputs must be 16-byte (fp16: 8-byte) aligned");
  cb2::PeerReduceParams p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < a->world; ++r) {
    CB2_CHECK_RT(a->peer_buffers[r] != nullptr && reinterpret_cast<uintptr_t>(a->peer_buffers[r]) % 256 == 0,
                 "peer buffer %d is null or not 256-byte aligned", r);
    p.peer[r] = reinterpret_cast<unsigned char *>(a->peer_buffers[r]);
  }
  PeerLayout L;
  peer_layout(a->numel, a->world, &L);
  p.src = a->src;
  p.out32 = a->out_f32;
  p.out16 = reinterpret_cast<__half *>(a->out_f16);
  p.n4 = static_cast<int>(a->numel / 4);
  p.shard_f4 = static_cast<int>(L.shard_f4);
  p.shard_bytes = L.shard_bytes;
  p.result_bytes = L.result_bytes;
  p.rank = a->rank;
  p.world = a->world;
  p.timeout_ns = a->timeout_ns ? a->timeout_ns : 1000000000ull;
  p.status = dev->status;
  // every CTA waits for data that other GPUs send only after they have seen this grid's whole
  // scatter: the whole grid must be resident at once, beside whatever else runs (small CTAs)
  static const int max_grid = [] {
    const char *v = getenv("CUMM_B200_PEER_GRID");
    const int g = v ? atoi(v) : 96;
    return g >= 1 ? g : 96;
  }();
  int grid = static_cast<int>(std::min<long long>((a->numel / 4 + cb2::kPeerThreads - 1) / cb2::kPeerThreads, max_grid));
  grid = std::max(1, std::min(grid, dev->num_sms));
  CB2_CHECK_ARG(a->own_sm_smem_bytes >= 0 && a->own_sm_smem_bytes <= 48 * 1024, "own_sm_smem_bytes must be 0 .. 48 KiB");
  cb2::peer_reduce_kernel<<<grid, cb2::kPeerThreads, static_cast<size_t>(a->own_sm_smem_bytes), stream>>>(p);
  CB2_CUDA(cudaGetLastError());
  g_launches.fetch_add(1);
  return CB2_OK;
}

// ---------------------------------------------------------------- the kernel table
static cb2_kernel_desp make_desp(int op_type, int shuffle, bool int8, bool ta, bool tb, int tn, int tk) {
  cb2_kernel_desp d;
  memset(&d, 0, sizeof(d));
  d.op_type = op_type;
  d.shuffle_type = shuffle;
  d.dtype_a = d.dtype_b = d.dtype_c = int8 ? CB2_DTYPE_I8 : CB2_DTYPE_F16;
  d.dacc = int8 ? CB2_DTYPE_I32 : CB2_DTYPE_F32;
  d.dcomp = CB2_DTYPE_F32;
  d.trans_a = ta;
  d.trans_b = tb;
  d.trans_c = 0;
  const int shape[3] = {128, tn, tk};
  for (int i = 0; i < 3; ++i)
    d.tile_shape[i] = d.warp_tile_shape[i] = shape[i];
  d.tensorop[0] = 128;
  d.tensorop[1] = tn;
  d.tensorop[2] = int8 ? 32 : 16;
  d.num_stage = 3;
  d.element_per_access = int8 ? 16 : 8;
  d.split_k_serial = (op_type == CB2_CONV_BACKWARD_WEIGHT || shuffle == CB2_SHUFFLE_AB) ? 1 : 0;
  d.mask_sparse = op_type >= 0 ? 1 : 0;
  d.increment_k_first = op_type >= 0 ? 1 : 0;
  d.is_int8_inference = int8 ? 1 : 0;
  d.min_arch_major = 10;
  d.min_arch_minor = 0;
  return d;
}

static int emit(const cb2_kernel_desp &d, cb2_kernel_desp *out, int capacity, int n) {
  if (out && n < capacity)
    out[n] = d;
  return n + 1;
}

// The variants launch_rowconv and run_wgrad can dispatch to (the CB2_INST list above).
int cb2_enumerate_gemm_desps(cb2_kernel_desp *out, int capacity) {
  int n = 0;
  const int shuffles[2] = {CB2_SHUFFLE_NONE, CB2_SHUFFLE_AC};
  for (int s = 0; s < 2; ++s)
    for (int tb = 1; tb >= 0; --tb)
      for (int tn = 64; tn <= 128; tn += 64)
        for (int tk = 64; tk <= 128; tk += 64)
          n = emit(make_desp(-1, shuffles[s], false, false, tb != 0, tn, tk), out, capacity, n);
  for (int tn = 64; tn <= 128; tn += 64)
    n = emit(make_desp(-1, CB2_SHUFFLE_AB, false, true, false, tn, 128), out, capacity, n);
  return n;
}

int cb2_enumerate_conv_desps(cb2_kernel_desp *out, int capacity) {
  int n = 0;
  // every variant twice: for kernel volumes up to 32, and (dynamic_mask) up to 128
  for (int dyn = 0; dyn <= 1; ++dyn) {
    auto add = [&](cb2_kernel_desp d) {
      d.dynamic_mask = dyn;
      n = emit(d, out, capacity, n);
    };
    // (trans_a, trans_b) per op: cumm/conv/params.py:61-69
    for (int op = CB2_CONV_FORWARD; op <= CB2_CONV_BACKWARD_INPUT; ++op)
      for (int tn = 64; tn <= 128; tn += 64)
        for (int tk = 64; tk <= 128; tk += 64)
          add(make_desp(op, CB2_SHUFFLE_NONE, false, false, op == CB2_CONV_FORWARD, tn, tk));
    for (int tn = 64; tn <= 128; tn += 64) {
      add(make_desp(CB2_CONV_BACKWARD_WEIGHT, CB2_SHUFFLE_NONE, false, true, false, tn, 128));
      add(make_desp(CB2_CONV_FORWARD, CB2_SHUFFLE_NONE, true, false, true, tn, 128));
    }
  }
  return n;
}

const char *cb2_last_error(void) { return g_err.c_str(); }

int cb2_tile_m(void) { return 128; }

uint64_t cb2_launch_count(void) { return g_launches.load(); }

int cb2_last_launch_info(int *num_regs, int *num_threads, int *smem_bytes) {
  if (num_regs)
    *num_regs = g_last_launch.num_regs;
  if (num_threads)
    *num_threads = g_last_launch.num_threads;
  if (smem_bytes)
    *smem_bytes = g_last_launch.smem_bytes;
  return CB2_OK;
}

int cb2_device_status(int *status) {
  DeviceState *dev;
  int rc = get_device(&dev);
  if (rc)
    return rc;
  CB2_CUDA(cudaDeviceSynchronize());
  int v = 0;
  CB2_CUDA(cudaMemcpy(&v, dev->status, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0)  // a kernel that gave up may have left its scheduling counters non-zero: clear everything
    CB2_CUDA(cudaMemset(dev->status, 0, kStatusBytes));
  if (status)
    *status = v;
  return CB2_OK;
}

size_t cb2_gemm_workspace_size(const cb2_gemm_args *a) {
  if (!a || a->shuffle_type != CB2_SHUFFLE_AB)
    return 0;
  DeviceState *dev;
  if (get_device(&dev))
    return 0;
  WgradLayout L;
  wgrad_layout(dev->num_sms, a->max_ctas, a->m, a->n, a->k, 1, a->tile_n, &L);
  return L.total;
}

size_t cb2_conv_workspace_size(const cb2_conv_args *a) {
  if (!a || a->op_type != CB2_CONV_BACKWARD_WEIGHT)
    return 0;
  DeviceState *dev;
  if (get_device(&dev))
    return 0;
  WgradLayout L;
  wgrad_layout(dev->num_sms, a->max_ctas, a->K, a->C, a->N, a->kernel_volume, a->tile_n, &L);
  return L.total;
}

size_t cb2_static_scratch_bytes(void) { return kStaticScratchBytes; }

int cb2_conv_backward_weight_static(const cb2_conv_args *a, void *stream_v) {
  CB2_CHECK_ARG(a != nullptr, "null arguments");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  StaticState *st;
  int rc = get_device_static(&st);
  if (rc)
    return rc;
  CB2_CHECK_RT(a->op_type == CB2_CONV_BACKWARD_WEIGHT, "the static-scratch entry point computes the weight gradient only");
  CB2_CHECK_RT(a->ptr_A && a->ptr_B && a->ptr_C, "input, weight, output must not empty");
  CB2_CHECK_RT(a->indice_ptr && a->mask_ptr && a->mask_argsort_ptr, "error: indices, mask or mask_argsort empty");
  CB2_CHECK_RT(a->kernel_volume >= 1 && a->kernel_volume <= 32, "kernel volume %d is not supported", a->kernel_volume);
  CB2_CHECK_ARG(a->N >= 0 && a->C > 0 && a->K > 0, "bad N,C,K (%d,%d,%d)", a->N, a->C, a->K);
  CB2_CHECK_RT(kind_of(a->dtype_a, a->dtype_b, a->dtype_c, a->is_int8_inference, true) == 0,
               "can't find any suitable algo for dtypes (%d,%d,%d)", a->dtype_a, a->dtype_b, a->dtype_c);
  CB2_CHECK_ARG(a->C % 8 == 0 && a->K % 8 == 0, "fp16 channel counts must be multiples of 8");
  CB2_CHECK_RT(a->mask_width > 0 && (a->mask_width % 128 == 0 || 128 % a->mask_width == 0),
               "error: mask_width must be positive and divide or be a multiple of %d", 128);
  const int need_words = (a->N + a->mask_width - 1) / a->mask_width;
  CB2_CHECK_RT(a->mask_words >= need_words, "reduced mask has %d words, %d needed", a->mask_words, need_words);
  WgradLayout L;
  wgrad_layout(st->dev.num_sms, a->max_ctas, a->K, a->C, a->N, a->kernel_volume, a->tile_n, &L);
  CB2_CHECK_RT(L.total <= kStaticScratchBytes,
               "this problem (K=%d, C=%d, N=%d) needs %zu bytes of scratch; the static scratch holds %zu. Use "
               "cb2_conv_run with a caller-provided workspace instead.",
               a->K, a->C, a->N, L.total, kStaticScratchBytes);
  WgradParams p;
  memset(&p, 0, sizeof(p));
  p.dout = a->ptr_A;
  p.x = a->ptr_B;
  p.indices = a->indice_ptr;
  p.rmask = a->mask_ptr;
  p.argsort = a->mask_argsort_ptr;
  p.ld_dout = a->K;
  p.ld_x = a->C;
  p.n_rows = a->N;
  p.a_rows = a->rows_A;
  p.b_rows = a->rows_B;
  p.m_total = a->K;
  p.n_total = a->C;
  p.kv = a->kernel_volume;
  p.mask_width = a->mask_width;
  p.words = 1;
  p.rmask_words = a->mask_words;
  p.mask_filter = a->mask_filter;
  p.mode = kWgradMaskConv;
  p.out = a->ptr_C;
  p.src = a->ptr_D ? a->ptr_D : a->ptr_C;
  p.ldo = (long long)a->kernel_volume * a->C;
  p.f_stride = a->C;
  p.alpha = a->alpha;
  p.beta = a->beta;
  p.out_f32 = a->dtype_c == CB2_DTYPE_F32 ? 1 : 0;
  // the planning kernel of every call clears the control words the main kernel uses and the main
  // kernel rewrites every partial it later reads, so whatever an earlier call (of any size) left
  // in the scratch does not matter
  return run_wgrad(&st->dev, p, a->tile_n, a->max_ctas, 0, st->scratch, kStaticScratchBytes, stream);
}

int cb2_static_status(int *status) {
  StaticState *st;
  int rc = get_device_static(&st);
  if (rc)
    return rc;
  CB2_CUDA(cudaDeviceSynchronize());
  int v = 0;
  CB2_CUDA(cudaMemcpy(&v, st->dev.status, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0)
    CB2_CUDA(cudaMemset(st->dev.status, 0, sizeof(int)));
  if (status)
    *status = v;
  return CB2_OK;
}

int cb2_gemm_run(const cb2_gemm_args *a, void *stream_v) {
  CB2_CHECK_ARG(a != nullptr, "null arguments");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  DeviceState *dev;
  int rc = get_device(&dev);
  if (rc)
    return rc;
  CB2_CHECK_RT(a->ptr_A && a->ptr_B && a->ptr_C, "a,b,c must not empty");
  CB2_CHECK_RT(!a->trans_c, "trans_c is not supported by the sm_100a kernels");
  const int kind = kind_of(a->dtype_a, a->dtype_b, a->dtype_c, 0, false);
  CB2_CHECK_RT(kind == 0, "can't find any suitable algo for dtypes (%d,%d,%d): only f16,f16,f16 is built",
               a->dtype_a, a->dtype_b, a->dtype_c);
  CB2_CHECK_ARG(a->m >= 0 && a->n > 0 && a->k >= 0, "bad m,n,k (%d,%d,%d)", a->m, a->n, a->k);
  if (a->shuffle_type == CB2_SHUFFLE_AB) {
    CB2_CHECK_RT(a->trans_a && !a->trans_b, "shuffle AB must be nt, i.e. backward weight");
    CB2_CHECK_RT(a->indiceA && a->indiceBorC, "a_inds,b_inds tensor must not empty");
    CB2_CHECK_ARG(a->m % 8 == 0 && a->n % 8 == 0,
                  "this m, n, k isn't supported due to misaligned contiguous dim.");
    WgradParams p;
    memset(&p, 0, sizeof(p));
    p.dout = a->ptr_A;
    p.x = a->ptr_B;
    p.a_inds = a->indiceA;
    p.b_inds = a->indiceBorC;
    p.ld_dout = a->stride_A;
    p.ld_x = a->stride_B;
    p.n_rows = a->k;
    p.a_rows = a->rows_A;
    p.b_rows = a->rows_B;
    p.m_total = a->m;
    p.n_total = a->n;
    p.kv = 1;
    p.mask_width = 128;
    p.words = 1;
    p.mask_filter = 0xffffffffu;
    p.mode = kWgradPairList;
    p.out = a->ptr_C;
    p.src = a->ptr_D ? a->ptr_D : a->ptr_C;
    p.ldo = a->stride_C;
    p.f_stride = 0;
    p.alpha = a->alpha;
    p.beta = a->beta;
    p.out_f32 = 0;
    return run_wgrad(dev, p, a->tile_n, a->max_ctas, a->reuse_plan, a->workspace, a->workspace_bytes, stream);
  }
  CB2_CHECK_RT(a->shuffle_type == CB2_SHUFFLE_AC || a->shuffle_type == CB2_SHUFFLE_NONE, "unknown shuffle type %d",
               a->shuffle_type);
  CB2_CHECK_RT(!a->trans_a, "a of shuffle AB must be row major");
  if (a->shuffle_type == CB2_SHUFFLE_AC)
    CB2_CHECK_RT(a->indiceBorC != nullptr, "a_inds,c_inds tensor must not empty");
  CB2_CHECK_ARG(a->k % 8 == 0 && a->n % 8 == 0, "this m, n, k isn't supported due to misaligned contiguous dim.");
  RowConvParams p;
  memset(&p, 0, sizeof(p));
  p.a = a->ptr_A;
  p.out = a->ptr_C;
  p.a_inds = a->indiceA;
  p.c_inds = a->indiceBorC;
  p.lda = a->stride_A;
  p.ldo = a->stride_C;
  p.n_rows = a->m;
  p.a_rows = a->rows_A;
  p.red = a->k;
  p.nn = a->n;
  p.kv = 1;
  p.mask_words = 1;
  p.mode = kModeGatherGemm;
  p.mask_filter = 0xffffffffu;
  p.alpha = a->alpha;
  p.beta = a->beta;
  p.act_alpha = a->act_alpha;
  p.act_type = a->act_type;
  if (a->beta != 0.f) {
    p.src = a->ptr_D ? a->ptr_D : a->ptr_C;
    p.src_mode = a->d_is_vector ? kSrcVector : kSrcRows;
    p.lds = a->ptr_D ? a->stride_D : a->stride_C;
    if (a->d_is_vector)
      CB2_CHECK_RT(a->ptr_D != nullptr, "d must be a valid bias");
  }
  // B: [n, k] (trans_b) is K-major for the tensor core, [k, n] is MN-major.
  const bool b_mn = !a->trans_b;
  const uint64_t inner = b_mn ? a->n : a->k;
  const uint64_t outer = b_mn ? a->k : a->n;
  return run_rowconv(dev, p, 0, b_mn, a->tile_n, a->tile_k, a->sched_scratch, a->max_ctas, a->ptr_B, inner, 1, outer,
                     a->stride_B, a->stride_B, stream);
}

int cb2_conv_run(const cb2_conv_args *a, void *stream_v) {
  CB2_CHECK_ARG(a != nullptr, "null arguments");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  DeviceState *dev;
  int rc = get_device(&dev);
  if (rc)
    return rc;
  CB2_CHECK_RT(a->ptr_A && a->ptr_B && a->ptr_C, "input, weight, output must not empty");
  CB2_CHECK_RT(a->indice_ptr != nullptr, "error: indices empty");
  CB2_CHECK_RT(a->mask_ptr != nullptr, "error: mask empty");
  CB2_CHECK_RT(a->mask_argsort_ptr != nullptr, "error: mask_argsort empty");
  CB2_CHECK_RT(a->kernel_volume >= 1 && a->kernel_volume <= 128,
               "kernel volume %d: the kernels handle up to 128 filter offsets (four mask words per row)",
               a->kernel_volume);
  CB2_CHECK_RT(a->groups == 1 || a->groups == 0, "groups must be 1");
  CB2_CHECK_ARG(a->N >= 0 && a->C > 0 && a->K > 0, "bad N,C,K (%d,%d,%d)", a->N, a->C, a->K);
  const bool wgrad = a->op_type == CB2_CONV_BACKWARD_WEIGHT;
  const int kind = kind_of(a->dtype_a, a->dtype_b, a->dtype_c, a->is_int8_inference, wgrad);
  CB2_CHECK_RT(kind >= 0, "can't find any suitable algo for dtypes (%d,%d,%d) int8_inference=%d", a->dtype_a,
               a->dtype_b, a->dtype_c, a->is_int8_inference);
  if (kind == 1) {
    CB2_CHECK_RT(a->op_type == CB2_CONV_FORWARD, "int8 inference is forward only");
    CB2_CHECK_RT(a->bias_pointer && a->scale_pointer, "int8 inference must have both scale and bias");
    CB2_CHECK_ARG(a->C % 16 == 0 && a->K % 16 == 0, "int8 channel counts must be multiples of 16");
  } else {
    CB2_CHECK_ARG(a->C % 8 == 0 && a->K % 8 == 0, "fp16 channel counts must be multiples of 8");
  }
  if (wgrad) {
    CB2_CHECK_RT(a->mask_width > 0 && (a->mask_width % 128 == 0 || 128 % a->mask_width == 0),
                 "error: mask_width must be positive and divide or be a multiple of %d", 128);
    const int need_words = (a->N + a->mask_width - 1) / a->mask_width * ((a->kernel_volume + 31) / 32);
    CB2_CHECK_RT(a->mask_words >= need_words, "reduced mask has %d words, %d needed", a->mask_words, need_words);
    WgradParams p;
    memset(&p, 0, sizeof(p));
    p.dout = a->ptr_A;
    p.x = a->ptr_B;
    p.indices = a->indice_ptr;
    p.rmask = a->mask_ptr;
    p.argsort = a->mask_argsort_ptr;
    p.ld_dout = a->K;
    p.ld_x = a->C;
    p.n_rows = a->N;
    p.a_rows = a->rows_A;
    p.b_rows = a->rows_B;
    p.m_total = a->K;
    p.n_total = a->C;
    p.kv = a->kernel_volume;
    p.mask_width = a->mask_width;
    p.words = (a->kernel_volume + 31) / 32;
    p.rmask_words = a->mask_words / p.words;
    p.mask_filter = a->mask_filter;
    p.mode = kWgradMaskConv;
    p.out = a->ptr_C;
    p.src = a->ptr_D ? a->ptr_D : a->ptr_C;
    p.ldo = (long long)a->kernel_volume * a->C;
    p.f_stride = a->C;
    p.alpha = a->alpha;
    p.beta = a->beta;
    p.out_f32 = a->dtype_c == CB2_DTYPE_F32 ? 1 : 0;
    return run_wgrad(dev, p, a->tile_n, a->max_ctas, a->reuse_plan, a->workspace, a->workspace_bytes, stream);
  }
  const bool dgrad = a->op_type == CB2_CONV_BACKWARD_INPUT;
  CB2_CHECK_RT(dgrad || a->op_type == CB2_CONV_FORWARD, "unknown op type %d", a->op_type);
  RowConvParams p;
  memset(&p, 0, sizeof(p));
  p.a = a->ptr_A;
  p.out = a->ptr_C;
  p.indices = a->indice_ptr;
  p.mask = a->mask_ptr;
  p.argsort = a->mask_argsort_ptr;
  p.mask_out = dgrad ? nullptr : a->mask_out_ptr;
  p.n_rows = a->N;
  p.a_rows = a->rows_A;
  p.red = dgrad ? a->K : a->C;
  p.nn = dgrad ? a->C : a->K;
  p.lda = p.red;
  p.ldo = p.nn;
  p.kv = a->kernel_volume;
  p.mask_words = (a->kernel_volume + 31) / 32;
  p.mode = kModeMaskConv;
  p.skip_empty_tiles = dgrad ? 1 : 0;
  p.reverse_mask = (dgrad && a->reverse_mask) ? 1 : 0;
  p.mask_filter = a->mask_filter;
  p.alpha = a->alpha;
  p.beta = a->beta;
  p.act_alpha = a->act_alpha;
  p.act_type = a->act_type;
  if (kind == 1) {
    p.scale = reinterpret_cast<const float *>(a->scale_pointer);
    p.bias = reinterpret_cast<const float *>(a->bias_pointer);
    if (a->beta != 0.f) {
      p.src = a->ptr_D ? a->ptr_D : a->ptr_C;
      p.src_mode = kSrcRows;
      p.lds = p.nn;
    }
  } else if (a->beta != 0.f) {
    p.src = a->ptr_D ? a->ptr_D : a->ptr_C;
    p.src_mode = a->d_is_bias ? kSrcVector : kSrcRows;
    p.lds = p.nn;
  }
  // weight [K, kv, C]: forward reduces over C (K-major B), backward input over K (MN-major B)
  return run_rowconv(dev, p, kind, dgrad, a->tile_n, a->tile_k, a->sched_scratch, a->max_ctas, a->ptr_B, a->C,
                     a->kernel_volume, a->K, a->C, (uint64_t)a->kernel_volume * a->C, stream);
}

} // extern "C"
