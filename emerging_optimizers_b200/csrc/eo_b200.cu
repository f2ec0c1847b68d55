// Host side of libeo_b200.so: argument checks, TMA descriptor construction and kernel launches
// behind the C ABI declared in include/eo_b200.h.
#include "../../include/eo_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

#include "elementwise.cuh"
#include "gemm_sm100.cuh"
#include "gemm_pair_sm100.cuh"
#include "ns_small_sm100.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define EO_CUDA(call)                                                                              \
  do {                                                                                             \
    cudaError_t e_ = (call);                                                                       \
    if (e_ != cudaSuccess) return fail(EO_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_)); \
  } while (0)

// Kernels report bounded-wait failures here; one copy per device that loads the module.
__device__ unsigned int g_device_status = 0;

// Scratch of eo_sumsq_f32_noalloc: per-block partial sums, resident on every device that loads this library
// until the process exits (512 KiB).  Host code must not pass this name to a kernel: on the host it is only a
// handle for cudaGetSymbolAddress, which device_setup() resolves once per device.
constexpr size_t kNoAllocMaxPartials = 65536;
static __device__ __align__(256) double g_noalloc_partials[kNoAllocMaxPartials];

// Tile-scheduler words of eo_gemm_kernel: kSchedSlots pairs {next tile, finished CTAs}, all zero between
// launches.  Consecutive launches take consecutive slots, so kernels that overlap on different streams do not
// share a pair unless more than kSchedSlots launches are in flight at once.
constexpr int kSchedSlots = 1024;
__device__ unsigned int g_sched_words[2 * kSchedSlots];

struct DeviceInfo {
  bool ready = false;
  int sm_count = 0;
  int clock_khz = 0;  // nominal SM clock, to turn the peer-wait budget into cycles
  unsigned int* status_ptr = nullptr;
  unsigned int* sched_ptr = nullptr;
  unsigned int sched_next = 0;
  double* noalloc_partials = nullptr;  // device address of g_noalloc_partials on this device
};
constexpr int kMaxDevices = 64;
DeviceInfo g_dev[kMaxDevices];
std::mutex g_mu;
PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
int g_option_gemm_bm = 0;  // eo_set_option("gemm_tile_m"): 0 = choose per problem, 128 or 256 = force
int g_option_gemm_pair = 1;     // eo_set_option("gemm_pair"): 256-row tiles run on CTA pairs (tcgen05 cta_group::2)
// Tile order of the pair kernel, eo_set_option("gemm_pair_group_m" / "gemm_pair_band"), and L2 policies of its operand
// loads ("gemm_pair_hint_a" / "gemm_pair_hint_b").  Measured on 8192 x 28672 in seconds-long loops: groups of 8 row
// blocks 4 % faster than 16 (32: 15 % slower), bands of 8 tile columns 3 % faster than whole columns; the policies
// made no difference and stay off.
int g_option_pair_group_m = 8;
int g_option_pair_band = 8;
int g_option_pair_hint_a = 0;
int g_option_pair_hint_b = 0;
int g_option_gemm_split_k = 1;  // eo_set_option("gemm_split_k"): the pair kernel may split the K range of its last tiles
int g_option_tp_lower_only = 1;  // eo_set_option("tp_lower_only"): the exchange fills the lower triangle only
int g_option_peer_wait_ms = 10000;  // eo_set_option("peer_wait_ms"): budget of one wait for other ranks' flags

// Workspace of the pair kernel's split tail: partial accumulators and arrival counters, one set per device and
// stream (launches on one stream never overlap), grown on demand and kept until the process exits.
struct SplitWorkspace {
  float* ws = nullptr;
  unsigned int* cnt = nullptr;
  size_t ws_bytes = 0;
  size_t cnt_words = 0;
};
std::map<std::pair<int, cudaStream_t>, SplitWorkspace> g_split_ws;
constexpr size_t kSplitWorkspaceLimit = size_t(4) << 30;
constexpr int kSplitMinBlocks = 48;  // shortest K piece, in 64-element blocks

int split_workspace(cudaStream_t st, size_t ws_bytes, size_t cnt_words, SplitWorkspace* out) {
  int dev = 0;
  EO_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(g_mu);
  SplitWorkspace& w = g_split_ws[std::make_pair(dev, st)];
  if (w.ws_bytes < ws_bytes || w.cnt_words < cnt_words) {
    if (ws_bytes > kSplitWorkspaceLimit)
      return fail(EO_ERR_BAD_ARG, "batch too large for the split-K workspace (%zu bytes); launch it in parts",
                  ws_bytes);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    EO_CUDA(cudaStreamIsCapturing(st, &cap));
    if (cap != cudaStreamCaptureStatusNone)
      return fail(EO_ERR_UNSUPPORTED, "the split-K workspace of this stream has to grow, which cannot happen during "
                                      "stream capture; run the same call once on this stream before capturing");
    // Never shrink either buffer (products of different shapes alternate on a stream).  cudaFree waits for the
    // device, so no kernel still uses the old buffers.
    if (ws_bytes < w.ws_bytes) ws_bytes = w.ws_bytes;
    if (cnt_words < w.cnt_words) cnt_words = w.cnt_words;
    if (w.ws != nullptr) EO_CUDA(cudaFree(w.ws));
    if (w.cnt != nullptr) EO_CUDA(cudaFree(w.cnt));
    w = SplitWorkspace();
    EO_CUDA(cudaMalloc(reinterpret_cast<void**>(&w.ws), ws_bytes));
    w.ws_bytes = ws_bytes;
    EO_CUDA(cudaMalloc(reinterpret_cast<void**>(&w.cnt), cnt_words * sizeof(unsigned int)));
    w.cnt_words = cnt_words;
    EO_CUDA(cudaMemsetAsync(w.cnt, 0, cnt_words * sizeof(unsigned int), st));
  }
  *out = w;
  return EO_OK;
}

int device_setup(DeviceInfo** out) {
  int dev = 0;
  EO_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(EO_ERR_BAD_ARG, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceInfo& d = g_dev[dev];
  if (!d.ready) {
    cudaDeviceProp prop;
    EO_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
      return fail(EO_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library runs on sm_100 only", dev, prop.major,
                  prop.minor);
    d.sm_count = prop.multiProcessorCount;
    EO_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&d.status_ptr), g_device_status));
    EO_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&d.noalloc_partials), g_noalloc_partials));
    EO_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&d.sched_ptr), g_sched_words));
    EO_CUDA(cudaFuncSetAttribute(eo::eo_gemm_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 eo::kGemmSmemBytes));
    EO_CUDA(cudaFuncSetAttribute(eo::eo_gemm_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 eo::kGemmSmemBytes));
    EO_CUDA(cudaFuncSetAttribute(eo::eo_gemm_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 eo::kGemmTpSmemBytes));
    EO_CUDA(cudaFuncSetAttribute(eo::eo_gemm_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 eo::kGemmTpSmemBytes));
    EO_CUDA(cudaFuncSetAttribute(eo::eo_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 eo::kPairSmemBytes));
    d.clock_khz = prop.clockRate;
    EO_CUDA(cudaFuncSetAttribute(eo::eo_ns_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 eo::kSmallSmemBytes));
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      EO_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
      if (fn == nullptr || qres != cudaDriverEntryPointSuccess)
        return fail(EO_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
      g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    }
    d.ready = true;
  }
  *out = &d;
  return EO_OK;
}

// 3-D tiled map over a batch of row-major matrices: dims {inner, rows, batch}, 128-byte swizzle,
// box {box_inner, box_rows, 1}.  Out-of-range parts of a box read as zero.
int make_map(CUtensorMap* map, const void* base, int elem_bytes, uint64_t inner, uint64_t rows, uint64_t batch,
             int64_t ld, int64_t stride, uint32_t box_inner, uint32_t box_rows) {
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return fail(EO_ERR_BAD_ARG, "operand base not 16-byte aligned");
  if ((ld * elem_bytes) % 16 != 0)
    return fail(EO_ERR_BAD_ARG, "leading dimension %lld not a multiple of 16 bytes", (long long)ld);
  if (batch > 1 && (stride * elem_bytes) % 16 != 0)
    return fail(EO_ERR_BAD_ARG, "batch stride %lld not a multiple of 16 bytes", (long long)stride);
  if (ld < static_cast<int64_t>(inner)) return fail(EO_ERR_BAD_ARG, "leading dimension smaller than row length");
  cuuint64_t dims[3] = {inner, rows, batch};
  const uint64_t bstride = (batch > 1) ? static_cast<uint64_t>(stride) : rows * static_cast<uint64_t>(ld);
  cuuint64_t strides[2] = {static_cast<uint64_t>(ld) * elem_bytes, bstride * elem_bytes};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = (elem_bytes == 2) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = g_encode(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(EO_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return EO_OK;
}

// Tensor-parallel Gram exchange of a SYRK launch (see GemmParams::tp_*).
struct TpExchange {
  int world, rank;
  unsigned int seq;
  void* const* partials;       // [world] every rank's partial-tile buffer
  unsigned int* const* flags;  // [world] every rank's flag words, [world][slots] each
  void* const* gram;           // [world] every rank's Gram matrix
  const void* partials_mc;     // multicast alias of the partial-tile buffers, or nullptr
  void* gram_mc;               // multicast alias of the Gram matrices, or nullptr
  int64_t ld_gram;
};

// Tile width of the tensor-parallel Gram exchange (buffer sizes and tile numbering depend on it).
inline int tp_tile_n(int N) { return N > 128 ? 256 : 128; }
inline int tp_total_tiles(int N) {
  const int bn = tp_tile_n(N), tm = (N + eo::kBlockM - 1) / eo::kBlockM, tn = (N + bn - 1) / bn;
  int total = 0;
  for (int j = 0; j < tn; ++j) total += tm - j * (bn / eo::kBlockM);
  return total;
}
inline int tp_slots(int N, int world) { return (tp_total_tiles(N) + world - 1) / world; }

// Split tail of the pair kernel: decided from M, N, K and the triangular flag alone (never from the batch size),
// so that a batched launch and per-matrix launches of the same shape round identically.  It applies when a
// matrix has at least one and a half rounds of 256 x 256 tiles and its last round is so empty that the K range
// of those tiles can be cut into two or more pieces that still fit one round.
void plan_split_tail(int M, int N, int K, int tri, int pairs_max, int* split_s, int* split_rest) {
  *split_s = 1;
  *split_rest = 0;
  const int tm = (M + 255) / 256, tn = (N + 255) / 256;
  long long tiles1 = 0;
  if (tri) {
    for (int j = 0; j < tn; ++j) tiles1 += tm > j ? tm - j : 0;
  } else {
    tiles1 = static_cast<long long>(tm) * tn;
  }
  const int rest = static_cast<int>(tiles1 % pairs_max);
  if (2 * tiles1 >= 3LL * pairs_max && rest > 0) {
    const int num_kb = (K + eo::kBlockK - 1) / eo::kBlockK;
    int s = pairs_max / rest;
    if (s > 8) s = 8;
    // a piece pays for a pipeline fill and a trip of its accumulator through the workspace: keep it long
    if (s > num_kb / kSplitMinBlocks) s = num_kb / kSplitMinBlocks;
    if (s >= 2) {
      *split_s = s;
      *split_rest = rest;
    }
  }
}

// Work-item schedule of the pair kernel for a launch whose tile counts (256 x 256 tiles) are already in `p`.
// Returns the number of work items of the whole batch.
long long fill_pair_schedule(eo::GemmParams& p, int M, int N, int tri, int batch, int split_s, int split_rest) {
  p.pair_group_m = g_option_pair_group_m;
  p.pair_band = (tri && M == N && p.tiles_m == p.tiles_n) ? g_option_pair_band : 0;
  p.pair_hint_a = tri ? 0 : g_option_pair_hint_a;
  p.pair_hint_b = tri ? 0 : g_option_pair_hint_b;
  p.split_first = p.tiles_per_batch - split_rest;
  p.split_s = split_s;
  p.split_items_per_batch = p.split_first + split_rest * split_s;
  return static_cast<long long>(p.split_items_per_batch) * batch;
}

int launch_gemm(const void* A, int a_mn, int64_t lda, int64_t strideA, int64_t planeA, const void* B, int b_mn,
                int64_t ldb, int64_t strideB, int64_t planeB, const void* C, int64_t ldc, int64_t strideC, void* D, int64_t ldd, int64_t strideD,
                int batch, int M, int N, int K, float alpha, float beta, float post_scale, int precision, int d_fp32,
                int round_bf16, int tri, int skip_upper, void* stream, const TpExchange* tp = nullptr,
                int d_multicast = 0, const float* dev_scale = nullptr, int dev_scale_mode = 0) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (batch < 0 || M < 0 || N < 0 || K < 0) return fail(EO_ERR_BAD_ARG, "negative size");
  if (precision != 0 && precision != 1) return fail(EO_ERR_BAD_ARG, "precision must be 0 (bf16) or 1 (split fp32)");
  if (precision == 1 && !d_fp32) return fail(EO_ERR_BAD_ARG, "split-fp32 precision needs an fp32 output");
  if (precision == 1 && (planeA % 8 != 0 || planeB % 8 != 0 || planeA <= 0 || planeB <= 0))
    return fail(EO_ERR_BAD_ARG, "plane strides must be positive multiples of 8 elements");
  if (beta != 0.0f && C == nullptr) return fail(EO_ERR_BAD_ARG, "beta != 0 needs C");
  if (A == nullptr || B == nullptr || (D == nullptr && tp == nullptr)) {
    if (batch == 0 || M == 0 || N == 0) return EO_OK;
    return fail(EO_ERR_BAD_ARG, "null operand");
  }
  if (batch == 0 || M == 0 || N == 0) return EO_OK;
  if (K == 0) return fail(EO_ERR_BAD_ARG, "K == 0 is not supported");

  const int eb = 2;  // operands are bf16 (plain) or bf16 planes (split fp32)
  const int bk = eo::kBlockK;
  const int nplanes = precision == 0 ? 1 : eo::kMaxPlanes;
  eo::GemmMaps maps;
  memset(&maps, 0, sizeof(maps));
  for (int pl = 0; pl < nplanes; ++pl) {
    const void* a_pl = static_cast<const char*>(A) + static_cast<int64_t>(pl) * planeA * eb;
    const void* b_pl = static_cast<const char*>(B) + static_cast<int64_t>(pl) * planeB * eb;
    int rc;
    if (!a_mn)
      rc = make_map(&maps.a[pl], a_pl, eb, K, M, batch, lda, strideA, bk, eo::kBlockM);
    else
      rc = make_map(&maps.a[pl], a_pl, eb, M, K, batch, lda, strideA, bk, bk);
    if (rc) return rc;
    if (!b_mn)
      rc = make_map(&maps.b[pl], b_pl, eb, K, N, batch, ldb, strideB, bk, eo::kBlockM);
    else
      rc = make_map(&maps.b[pl], b_pl, eb, N, K, batch, ldb, strideB, bk, bk);
    if (rc) return rc;
  }

  eo::GemmParams p;
  memset(&p, 0, sizeof(p));
  p.batch = batch;
  p.M = M;
  p.N = N;
  p.K = K;
  p.a_mn = a_mn;
  p.b_mn = b_mn;
  if (precision == 0) {
    p.nterms = 1;
  } else {
    // x = x0 + x1 + x2: keep every product of planes i, j with i + j <= 2, smallest contributions first so
    // that they are not absorbed by the large one in the fp32 accumulator.
    static const int ta[6] = {0, 2, 1, 0, 1, 0};
    static const int tb[6] = {2, 0, 1, 1, 0, 0};
    p.nterms = 6;
    for (int t = 0; t < 6; ++t) {
      p.term_a[t] = ta[t];
      p.term_b[t] = tb[t];
    }
  }
  p.tri = tri;
  p.same_ab = (tri && precision == 0 && A == B && a_mn == b_mn && lda == ldb && strideA == strideB && planeA == planeB) ? 1 : 0;
  p.skip_upper = skip_upper;
  p.c_fp32 = precision;
  p.d_fp32 = d_fp32;
  p.round_bf16 = round_bf16;
  p.C = (beta != 0.0f) ? C : nullptr;
  p.ldc = ldc;
  p.strideC = strideC;
  p.D = D;
  p.ldd = ldd;
  p.strideD = strideD;
  p.alpha = alpha;
  p.beta = beta;
  p.post_scale = post_scale;
  p.status = dev->status_ptr;
  p.dev_scale = dev_scale;
  p.dev_scale_mode = dev_scale_mode;

  // Descriptor geometry.  K-major: rows of 128 bytes along K, eight-row groups 1024 bytes apart,
  // each MMA consumes 32 bytes of a row.  MN-major: rows of 128 bytes along M/N (one per k),
  // eight-k groups 1024 bytes apart, 128-byte-wide M/N atoms bk rows apart; each MMA consumes
  // 32 / elem_bytes k-rows.
  const unsigned int mn_adv = static_cast<unsigned int>((32 / eb) * eo::kRowBytes);
  const unsigned int mn_lbo = static_cast<unsigned int>(bk * eo::kRowBytes);
  p.adv_a = a_mn ? mn_adv : 32u;
  p.adv_b = b_mn ? mn_adv : 32u;
  p.lbo_a = a_mn ? mn_lbo : 0u;
  p.lbo_b = b_mn ? mn_lbo : 0u;
  p.sbo_a = 1024u;
  p.sbo_b = 1024u;

  const int c_eb = p.c_fp32 ? 4 : 2;
  const int d_eb = p.d_fp32 ? 4 : 2;
  bool vec = (reinterpret_cast<uintptr_t>(D) % 16 == 0) && ((ldd * d_eb) % 16 == 0) && ((strideD * d_eb) % 16 == 0);
  if (p.C != nullptr)
    vec = vec && (reinterpret_cast<uintptr_t>(C) % 16 == 0) && ((ldc * c_eb) % 16 == 0) &&
          ((strideC * c_eb) % 16 == 0);
  p.vec_ok = vec ? 1 : 0;

  // Tile height: 256-row tiles (two MMAs per k-step on one B tile) move a third fewer operand bytes per FLOP; they
  // pay off when every SM still gets several tiles and K is long enough to hide the un-overlapped epilogue.
  p.bm = 128;
  p.stages = eo::kStages;
  const int pairs_max = dev->sm_count / 2;
  const bool pair_ok = g_option_gemm_pair && tp == nullptr && !d_multicast && precision == 0 && M >= 256 &&
                       N >= 256 && pairs_max >= 1 && g_option_gemm_bm != 128;
  int split_s = 1, split_rest = 0;
  if (pair_ok && g_option_gemm_split_k) plan_split_tail(M, N, K, tri, pairs_max, &split_s, &split_rest);
  if (split_s > 1) {
    p.bm = 256;
    p.stages = 3;
  } else {
    const int want = g_option_gemm_bm;
    const long long t_wide = (static_cast<long long>((M + 255) / 256) * ((N + 255) / 256)) / (tri ? 2 : 1) * batch;
    const bool fits = precision == 0 && M >= 256 && N >= 256;
    bool good = K >= 1024 && 4 * t_wide >= 3LL * dev->sm_count;
    if (good && tp == nullptr) {
      // Wave quantisation: equal tiles run in rounds of one per SM, so a launch costs ceil(tiles / SMs) tile times.
      // A 128-row tile takes 0.535 of a 256-row tile's time (half the work at about 7 % less per FLOP); take the
      // narrow tiles where their rounds come out shorter (e.g. 448 wide tiles = 4 rounds against 896 narrow
      // tiles = 7 half rounds).
      const long long sms = dev->sm_count;
      const long long tm128 = (M + 127) / 128, tn = (N + 255) / 256;
      const long long t_narrow = (tri ? (tm128 * tn + tn) / 2 : tm128 * tn) * batch;
      const double cost_wide = static_cast<double>((t_wide + sms - 1) / sms);
      const double cost_narrow = 0.535 * static_cast<double>((t_narrow + sms - 1) / sms);
      if (cost_narrow < 0.97 * cost_wide) good = false;
    }
    if (fits && (want == 256 || (want == 0 && good))) {
      p.bm = 256;
      p.stages = 3;
    }
  }
  // Tile width: 256 unless the problem is narrow or the wider tile leaves SMs idle.
  p.tiles_m = (M + p.bm - 1) / p.bm;
  auto count_tiles = [&](int bn, int* tiles_n) {
    *tiles_n = (N + bn - 1) / bn;
    if (!tri) return p.tiles_m * (*tiles_n);
    int total = 0;
    for (int j = 0; j < *tiles_n; ++j) {
      const int first = (j * bn) / p.bm;
      if (first < p.tiles_m) total += p.tiles_m - first;
    }
    return total;
  };
  int tn256 = 0, tn128 = 0;
  const long long t256 = static_cast<long long>(count_tiles(256, &tn256)) * batch;
  const long long t128 = static_cast<long long>(count_tiles(128, &tn128)) * batch;
  bool narrow = p.bm == 128 && ((N <= 128) || (t256 < dev->sm_count && t128 > t256));
  if (tp != nullptr) {
    narrow = tp_tile_n(N) == 128;
    p.tp_world = tp->world;
    p.tp_rank = tp->rank;
    p.tp_seq = tp->seq;
    p.tp_slots = tp_slots(N, tp->world);
    p.tp_total = tp_total_tiles(N);
    p.tp_partials = static_cast<unsigned short*>(tp->partials[tp->rank]);
    p.tp_my_flags = tp->flags[tp->rank];
    p.tp_partials_mc = static_cast<const unsigned short*>(tp->partials_mc);
    p.tp_gram_mc = static_cast<unsigned short*>(tp->gram_mc);
    p.tp_ld = tp->ld_gram;
    p.tp_lower_only = g_option_tp_lower_only;
    // cycles at the nominal clock; the SMs never run faster than that, so the wait is at least as long as asked
    p.tp_wait_cycles = static_cast<long long>(g_option_peer_wait_ms) * dev->clock_khz;
    for (int r = 0; r < tp->world; ++r) {
      p.tp_flags[r] = tp->flags[r] + static_cast<int64_t>(tp->rank) * p.tp_slots;
      p.tp_partials_peer[r] = static_cast<const unsigned short*>(tp->partials[r]);
      p.tp_gram[r] = static_cast<unsigned short*>(tp->gram[r]);
    }
  }
  if (d_multicast) {
    if (tri || precision != 0 || d_fp32 || N % 32 != 0 || !p.vec_ok)
      return fail(EO_ERR_BAD_ARG, "multicast output needs a general bf16 product with N a multiple of 32 and "
                                  "16-byte aligned rows");
    p.d_mc = 1;
  }
  p.bn = narrow ? 128 : 256;
  p.tiles_n = narrow ? tn128 : tn256;
  const long long total = narrow ? t128 : t256;
  if (total > 0x7fffffffLL) return fail(EO_ERR_BAD_ARG, "too many tiles");
  p.total_tiles = static_cast<int>(total);
  p.tiles_per_batch = p.total_tiles / batch;

  {
    std::lock_guard<std::mutex> lock(g_mu);
    p.sched = dev->sched_ptr + 2 * (dev->sched_next % kSchedSlots);
    dev->sched_next++;
  }
  const int grid = p.total_tiles < dev->sm_count ? p.total_tiles : dev->sm_count;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (pair_ok && p.bm == 256 && p.bn == 256) {
    // CTA pairs: one cluster of two CTAs per work item in flight
    const long long items = fill_pair_schedule(p, M, N, tri, batch, split_s, split_rest);
    if (items > 0x3fffffffLL) return fail(EO_ERR_BAD_ARG, "too many tiles");
    p.total_tiles = static_cast<int>(items);
    if (split_rest > 0) {
      const size_t split_tiles = static_cast<size_t>(split_rest) * batch;
      SplitWorkspace w;
      if (int rc = split_workspace(st, split_tiles * split_s * 2 * eo::kSplitHalfFloats * sizeof(float),
                                   split_tiles * 2 * eo::kEpilogueWarps, &w))
        return rc;
      p.split_ws = w.ws;
      p.split_cnt = w.cnt;
      // The kernel leaves its counters at zero, but a launch that gave up a wait may not have: start clean.
      EO_CUDA(cudaMemsetAsync(w.cnt, 0, split_tiles * 2 * eo::kEpilogueWarps * sizeof(unsigned int), st));
    }
    const int pairs = p.total_tiles < pairs_max ? p.total_tiles : pairs_max;
    eo::eo_gemm_pair_kernel<<<2 * pairs, eo::kGemmThreads, eo::kPairSmemBytes, st>>>(maps, p);
  } else if (tp != nullptr) {
    constexpr int threads = eo::kGemmThreads + eo::kTpReducerThreads;
    if (p.bm == 256)
      eo::eo_gemm_kernel<2, true><<<grid, threads, eo::kGemmTpSmemBytes, st>>>(maps, p);
    else
      eo::eo_gemm_kernel<1, true><<<grid, threads, eo::kGemmTpSmemBytes, st>>>(maps, p);
  } else if (p.bm == 256) {
    eo::eo_gemm_kernel<2, false><<<grid, eo::kGemmThreads, eo::kGemmSmemBytes, st>>>(maps, p);
  } else {
    eo::eo_gemm_kernel<1, false><<<grid, eo::kGemmThreads, eo::kGemmSmemBytes, st>>>(maps, p);
  }
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}

}  // namespace

extern "C" {

const char* eo_version(void) { return "eo_b200 0.1.0 sm_100a"; }

const char* eo_last_error(void) { return g_err; }

int eo_debug_pair_schedule(int M, int N, int K, int tri, int batch, int sm_count, int* out, int64_t capacity,
                           int64_t* n_items) {
  if (M < 256 || N < 256 || K < 1 || batch < 1 || sm_count < 2 || n_items == nullptr)
    return fail(EO_ERR_BAD_ARG, "the pair kernel needs M, N >= 256, K, batch >= 1 and at least two SMs");
  if (tri && M != N) return fail(EO_ERR_BAD_ARG, "a triangular product is square");
  eo::GemmParams p;
  memset(&p, 0, sizeof(p));
  p.batch = batch;
  p.M = M;
  p.N = N;
  p.K = K;
  p.tri = tri;
  p.bm = 256;
  p.bn = 256;
  p.tiles_m = (M + 255) / 256;
  p.tiles_n = (N + 255) / 256;
  long long per = 0;
  if (tri) {
    for (int j = 0; j < p.tiles_n; ++j) per += p.tiles_m > j ? p.tiles_m - j : 0;
  } else {
    per = static_cast<long long>(p.tiles_m) * p.tiles_n;
  }
  p.tiles_per_batch = static_cast<int>(per);
  int split_s = 1, split_rest = 0;
  if (g_option_gemm_split_k) plan_split_tail(M, N, K, tri, sm_count / 2, &split_s, &split_rest);
  const long long items = fill_pair_schedule(p, M, N, tri, batch, split_s, split_rest);
  *n_items = items;
  if (out == nullptr) return EO_OK;
  if (capacity < items) return fail(EO_ERR_BAD_ARG, "room for %lld work items needed", items);
  const int num_kb = (K + eo::kBlockK - 1) / eo::kBlockK;
  for (long long w = 0; w < items; ++w) {
    const eo::PairWork wk = eo::decode_pair_work(p, static_cast<int>(w), num_kb);
    int b = 0, ti = 0, tj = 0;
    eo::decode_pair_tile(p, wk.tile, b, ti, tj);
    int* row = out + 6 * w;
    row[0] = b;
    row[1] = ti;
    row[2] = tj;
    row[3] = wk.kb0;
    row[4] = wk.kb1;
    row[5] = wk.slot;
  }
  return EO_OK;
}

int eo_set_option(const char* name, int value) {
  if (name == nullptr) return fail(EO_ERR_BAD_ARG, "option name is NULL");
  if (strcmp(name, "gemm_tile_m") == 0) {
    if (value != 0 && value != 128 && value != 256) return fail(EO_ERR_BAD_ARG, "gemm_tile_m must be 0, 128 or 256");
    g_option_gemm_bm = value;
    return EO_OK;
  }
  if (strcmp(name, "gemm_pair_group_m") == 0) {
    if (value < 1 || value > 64) return fail(EO_ERR_BAD_ARG, "gemm_pair_group_m must be 1..64");
    g_option_pair_group_m = value;
    return EO_OK;
  }
  if (strcmp(name, "gemm_pair_band") == 0) {
    if (value < 0 || value > 64) return fail(EO_ERR_BAD_ARG, "gemm_pair_band must be 0..64");
    g_option_pair_band = value;
    return EO_OK;
  }
  if (strcmp(name, "gemm_pair_hint_a") == 0 || strcmp(name, "gemm_pair_hint_b") == 0) {
    if (value < 0 || value > 2) return fail(EO_ERR_BAD_ARG, "%s must be 0, 1 or 2", name);
    (name[15] == 'a' ? g_option_pair_hint_a : g_option_pair_hint_b) = value;
    return EO_OK;
  }
  if (strcmp(name, "gemm_split_k") == 0) {
    if (value != 0 && value != 1) return fail(EO_ERR_BAD_ARG, "gemm_split_k must be 0 or 1");
    g_option_gemm_split_k = value;
    return EO_OK;
  }
  if (strcmp(name, "gemm_pair") == 0) {
    if (value != 0 && value != 1) return fail(EO_ERR_BAD_ARG, "gemm_pair must be 0 or 1");
    g_option_gemm_pair = value;
    return EO_OK;
  }
  if (strcmp(name, "tp_lower_only") == 0) {
    if (value != 0 && value != 1) return fail(EO_ERR_BAD_ARG, "tp_lower_only must be 0 or 1");
    g_option_tp_lower_only = value;
    return EO_OK;
  }
  if (strcmp(name, "peer_wait_ms") == 0) {
    if (value < 1 || value > 600000) return fail(EO_ERR_BAD_ARG, "peer_wait_ms must be within 1..600000");
    g_option_peer_wait_ms = value;
    return EO_OK;
  }
  return fail(EO_ERR_BAD_ARG, "unknown option %s", name);
}

int eo_read_device_status(uint32_t* host_code, void* stream) {
  if (host_code == nullptr) return fail(EO_ERR_BAD_ARG, "host_code is NULL");
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  EO_CUDA(cudaStreamSynchronize(s));
  unsigned int code = 0;
  EO_CUDA(cudaMemcpyAsync(&code, dev->status_ptr, sizeof(code), cudaMemcpyDeviceToHost, s));
  EO_CUDA(cudaStreamSynchronize(s));
  if (code != 0) {
    // A kernel that gave up may have left its tile-scheduler words non-zero: re-arm all of them.
    EO_CUDA(cudaMemsetAsync(dev->status_ptr, 0, sizeof(code), s));
    EO_CUDA(cudaMemsetAsync(dev->sched_ptr, 0, 2 * kSchedSlots * sizeof(unsigned int), s));
    EO_CUDA(cudaStreamSynchronize(s));
  }
  *host_code = code;
  return EO_OK;
}

int eo_gemm(const void* A, int a_mn_major, int64_t lda, int64_t strideA, int64_t planeA, const void* B,
            int b_mn_major, int64_t ldb, int64_t strideB, int64_t planeB, const void* C, int64_t ldc, int64_t strideC,
            void* D, int64_t ldd, int64_t strideD, int batch, int M, int N, int K, float alpha, float beta,
            float post_scale, int precision, int d_fp32, int round_bf16, void* stream) {
  return launch_gemm(A, a_mn_major, lda, strideA, planeA, B, b_mn_major, ldb, strideB, planeB, C, ldc, strideC, D, ldd, strideD, batch,
                     M, N, K, alpha, beta, post_scale, precision, d_fp32, round_bf16, /*tri=*/0, /*skip_upper=*/0,
                     stream);
}

int eo_gemm_multicast(const void* A, int a_mn_major, int64_t lda, const void* B, int b_mn_major, int64_t ldb,
                      const void* C, int64_t ldc, void* D_multicast, int64_t ldd, int M, int N, int K, float alpha,
                      float beta, void* stream) {
  return launch_gemm(A, a_mn_major, lda, 0, 0, B, b_mn_major, ldb, 0, 0, C, ldc, 0, D_multicast, ldd, 0, 1, M, N, K, alpha,
                     beta, 1.0f, /*precision=*/0, /*d_fp32=*/0, /*round_bf16=*/0, /*tri=*/0, /*skip_upper=*/0, stream,
                     nullptr, /*d_multicast=*/1);
}

int eo_peek_device_status_async(uint32_t* pinned_host_code, void* stream) {
  if (pinned_host_code == nullptr) return fail(EO_ERR_BAD_ARG, "pinned_host_code is NULL");
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  EO_CUDA(cudaMemcpyAsync(pinned_host_code, dev->status_ptr, sizeof(uint32_t), cudaMemcpyDeviceToHost,
                          static_cast<cudaStream_t>(stream)));
  return EO_OK;
}

int eo_syrk(const void* A, int a_trans, int64_t lda, int64_t strideA, int64_t planeA, const void* C, int64_t ldc,
            int64_t strideC, void* D, int64_t ldd, int64_t strideD, int batch, int N, int K, float alpha, float beta,
            int skip_upper, int precision, void* stream) {
  return launch_gemm(A, a_trans, lda, strideA, planeA, A, a_trans, lda, strideA, planeA, C, ldc, strideC, D, ldd, strideD, batch, N, N,
                     K, alpha, beta, 1.0f, precision, /*d_fp32=*/precision, /*round_bf16=*/0, /*tri=*/1, skip_upper,
                     stream);
}

int eo_split_f32(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride, void* planes,
                 int64_t ldo, int64_t strideo, int64_t plane_stride, void* stream) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (batch < 0 || rows < 0 || cols < 0) return fail(EO_ERR_BAD_ARG, "negative size");
  if (batch == 0 || rows == 0 || cols == 0) return EO_OK;
  if (x == nullptr || planes == nullptr) return fail(EO_ERR_BAD_ARG, "null pointer");
  if (ld < cols || ldo < cols) return fail(EO_ERR_BAD_ARG, "leading dimension smaller than cols");
  eo::launch_split3(x, batch, rows, cols, ld, stride, planes, ldo, strideo, plane_stride,
                    static_cast<cudaStream_t>(stream));
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}

size_t eo_sumsq_scratch_bytes(int batch, int64_t rows, int64_t cols) {
  if (batch <= 0) return 0;
  return static_cast<size_t>(batch) * eo::sumsq_blocks_per_matrix(rows, cols) * sizeof(double);
}

int eo_sumsq_f32(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride, double* sumsq,
                 void* scratch, size_t scratch_bytes, void* stream) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (batch < 0 || rows < 0 || cols < 0) return fail(EO_ERR_BAD_ARG, "negative size");
  if (batch == 0) return EO_OK;
  if (sumsq == nullptr) return fail(EO_ERR_BAD_ARG, "sumsq is NULL");
  if (ld < cols) return fail(EO_ERR_BAD_ARG, "ld smaller than cols");
  const size_t need = eo_sumsq_scratch_bytes(batch, rows, cols);
  if (scratch_bytes < need || (need > 0 && scratch == nullptr))
    return fail(EO_ERR_WORKSPACE, "sumsq scratch: need %zu bytes, got %zu", need, scratch_bytes);
  if (rows > 0 && cols > 0 && x == nullptr) return fail(EO_ERR_BAD_ARG, "x is NULL");
  eo::launch_sumsq(x, batch, rows, cols, ld, stride, sumsq, static_cast<double*>(scratch),
                   static_cast<cudaStream_t>(stream));
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}

int eo_cast_sumsq_f32(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride, void* out_bf16,
                      int64_t ldo, int64_t strideo, float eps, double* sumsq, float* scales, void* scratch,
                      size_t scratch_bytes, void* stream) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (batch < 0 || rows < 0 || cols < 0) return fail(EO_ERR_BAD_ARG, "negative size");
  if (batch == 0) return EO_OK;
  if (scales == nullptr || out_bf16 == nullptr) return fail(EO_ERR_BAD_ARG, "null pointer");
  if (ld < cols || ldo < cols) return fail(EO_ERR_BAD_ARG, "leading dimension smaller than cols");
  const size_t need = eo_sumsq_scratch_bytes(batch, rows, cols);
  if (scratch_bytes < need || (need > 0 && scratch == nullptr))
    return fail(EO_ERR_WORKSPACE, "cast_sumsq scratch: need %zu bytes, got %zu", need, scratch_bytes);
  if (rows > 0 && cols > 0 && x == nullptr) return fail(EO_ERR_BAD_ARG, "x is NULL");
  eo::launch_cast_sumsq(x, batch, rows, cols, ld, stride, out_bf16, ldo, strideo, eps, sumsq, scales,
                        static_cast<double*>(scratch), static_cast<cudaStream_t>(stream));
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}

size_t eo_muon_scratch_bytes(int64_t numel) {
  if (numel <= 0) return 0;
  return static_cast<size_t>(eo::sumsq_blocks_per_matrix(numel, 1)) * sizeof(double);
}

int eo_muon_momentum_f32(const float* g, float* m, const float* p, int64_t numel, double momentum, int nesterov,
                         float l2_weight_decay, double* sumsq, void* scratch, size_t scratch_bytes, void* stream) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (numel < 0) return fail(EO_ERR_BAD_ARG, "negative size");
  if (g == nullptr || m == nullptr || sumsq == nullptr) return fail(EO_ERR_BAD_ARG, "null pointer");
  if (l2_weight_decay != 0.0f && p == nullptr) return fail(EO_ERR_BAD_ARG, "l2 weight decay needs p");
  if ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(p)) & 15)
    return fail(EO_ERR_BAD_ARG, "g, m and p must be 16-byte aligned");
  const size_t need = eo_muon_scratch_bytes(numel);
  if (scratch_bytes < need || scratch == nullptr)
    return fail(EO_ERR_WORKSPACE, "muon scratch: need %zu bytes, got %zu", need, scratch_bytes);
  const int nblk = eo::sumsq_blocks_per_matrix(numel, 1);
  eo::MuonEw c{static_cast<float>(momentum), static_cast<float>(1.0 - momentum), l2_weight_decay, nesterov ? 1 : 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  eo::muon_momentum_kernel<<<nblk, eo::kEwThreads, 0, s>>>(g, m, p, numel, c, static_cast<double*>(scratch));
  eo::sumsq_final_kernel<<<1, eo::kEwThreads, 0, s>>>(static_cast<const double*>(scratch), nblk, sumsq);
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}

int eo_muon_normalize_bf16(const float* g, const float* m, const float* p, int64_t numel, double momentum,
                           int nesterov, float l2_weight_decay, const double* sumsq, float eps, void* out,
                           void* stream) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (numel < 0) return fail(EO_ERR_BAD_ARG, "negative size");
  if (numel == 0) return EO_OK;
  if (g == nullptr || m == nullptr || sumsq == nullptr || out == nullptr) return fail(EO_ERR_BAD_ARG, "null pointer");
  if (l2_weight_decay != 0.0f && p == nullptr) return fail(EO_ERR_BAD_ARG, "l2 weight decay needs p");
  if ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(p) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return fail(EO_ERR_BAD_ARG, "g, m, p and out must be 16-byte aligned");
  eo::MuonEw c{static_cast<float>(momentum), static_cast<float>(1.0 - momentum), l2_weight_decay, nesterov ? 1 : 0};
  eo::muon_normalize_kernel<<<eo::ew_blocks(numel, 16), eo::kEwThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      g, m, p, numel, c, sumsq, eps, static_cast<__nv_bfloat16*>(out));
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}

int eo_muon_apply_f32(float* p, const void* update, int update_is_bf16, int64_t numel, float shrink, float scale,
                      float extra_scale, float lr, void* stream) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (numel < 0) return fail(EO_ERR_BAD_ARG, "negative size");
  if (numel == 0) return EO_OK;
  if (p == nullptr || update == nullptr) return fail(EO_ERR_BAD_ARG, "null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int nb = eo::ew_blocks(numel, 8);
  if (update_is_bf16)
    eo::muon_apply_kernel<__nv_bfloat16><<<nb, eo::kEwThreads, 0, s>>>(
        p, static_cast<const __nv_bfloat16*>(update), numel, shrink, scale, extra_scale, lr);
  else
    eo::muon_apply_kernel<float><<<nb, eo::kEwThreads, 0, s>>>(p, static_cast<const float*>(update), numel, shrink,
                                                               scale, extra_scale, lr);
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}

size_t eo_muon_prepare_scratch_bytes(int n, int64_t numel) {
  if (n <= 0 || numel <= 0) return 0;
  return static_cast<size_t>(n) * eo::sumsq_blocks_per_matrix(numel, 1) * sizeof(double);
}

int eo_muon_prepare_batch(int n, const float* const* g, float* const* m, const float* const* p, int64_t numel,
                          double momentum, int nesterov, float l2_weight_decay, float eps, void* out_stack,
                          int64_t slot_stride, double* sumsq, float* dev_scales, void* scratch, size_t scratch_bytes,
                          void* stream) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (n < 0 || numel < 0) return fail(EO_ERR_BAD_ARG, "negative size");
  if (n == 0 || numel == 0) return EO_OK;
  if (g == nullptr || m == nullptr || out_stack == nullptr || sumsq == nullptr)
    return fail(EO_ERR_BAD_ARG, "null pointer");
  if (l2_weight_decay != 0.0f && p == nullptr) return fail(EO_ERR_BAD_ARG, "l2 weight decay needs p");
  if (slot_stride < numel || slot_stride % 8 != 0 || (reinterpret_cast<uintptr_t>(out_stack) & 15))
    return fail(EO_ERR_BAD_ARG, "out_stack must be 16-byte aligned with a slot stride >= numel that is a multiple of 8");
  const size_t need = eo_muon_prepare_scratch_bytes(n, numel);
  if (scratch_bytes < need || scratch == nullptr)
    return fail(EO_ERR_WORKSPACE, "muon prepare scratch: need %zu bytes, got %zu", need, scratch_bytes);
  for (int i = 0; i < n; ++i) {
    uintptr_t bits = reinterpret_cast<uintptr_t>(g[i]) | reinterpret_cast<uintptr_t>(m[i]);
    if (p != nullptr) bits |= reinterpret_cast<uintptr_t>(p[i]);
    if (g[i] == nullptr || m[i] == nullptr || (bits & 15))
      return fail(EO_ERR_BAD_ARG, "tensor %d: g, m and p must be non-null and 16-byte aligned", i);
  }
  const int nblk = eo::sumsq_blocks_per_matrix(numel, 1);
  const eo::MuonEw c{static_cast<float>(momentum), static_cast<float>(1.0 - momentum), l2_weight_decay,
                     nesterov ? 1 : 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  double* partial = static_cast<double*>(scratch);
  for (int i0 = 0; i0 < n; i0 += eo::kMtMax) {
    const int cnt = (n - i0 < eo::kMtMax) ? (n - i0) : eo::kMtMax;
    eo::MtPrepare t;
    memset(&t, 0, sizeof(t));
    for (int i = 0; i < cnt; ++i) {
      t.g[i] = g[i0 + i];
      t.m[i] = m[i0 + i];
      t.p[i] = (p != nullptr) ? p[i0 + i] : nullptr;
    }
    if (dev_scales != nullptr) {
      // deferred normalisation: one pass writes the un-normalised bf16 update; the iteration applies the factors
      eo::muon_momentum_cast_mt_kernel<<<dim3(nblk, cnt), eo::kEwThreads, 0, s>>>(
          t, numel, c, static_cast<__nv_bfloat16*>(out_stack) + static_cast<int64_t>(i0) * slot_stride, slot_stride,
          partial + static_cast<int64_t>(i0) * nblk);
      eo::sumsq_scales_kernel<<<cnt, eo::kEwThreads, 0, s>>>(partial + static_cast<int64_t>(i0) * nblk, nblk, eps,
                                                             sumsq + i0, dev_scales + 2 * static_cast<int64_t>(i0));
      continue;
    }
    eo::muon_momentum_mt_kernel<<<dim3(nblk, cnt), eo::kEwThreads, 0, s>>>(t, numel, c,
                                                                          partial + static_cast<int64_t>(i0) * nblk);
    eo::sumsq_final_kernel<<<cnt, eo::kEwThreads, 0, s>>>(partial + static_cast<int64_t>(i0) * nblk, nblk, sumsq + i0);
    eo::muon_normalize_mt_kernel<<<dim3(eo::ew_blocks(numel, 16), cnt), eo::kEwThreads, 0, s>>>(
        t, numel, c, sumsq + i0, eps, static_cast<__nv_bfloat16*>(out_stack) + static_cast<int64_t>(i0) * slot_stride,
        slot_stride);
  }
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}

int eo_muon_apply_batch(int n, float* const* p, const void* const* update, int update_is_bf16, const int64_t* numel,
                        const float* scale, float shrink, float extra_scale, float lr, int max_blocks_per_tensor,
                        void* stream) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (n < 0) return fail(EO_ERR_BAD_ARG, "negative size");
  if (n == 0) return EO_OK;
  if (p == nullptr || update == nullptr || numel == nullptr || scale == nullptr)
    return fail(EO_ERR_BAD_ARG, "null pointer");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int i0 = 0; i0 < n; i0 += eo::kMtMax) {
    const int cnt = (n - i0 < eo::kMtMax) ? (n - i0) : eo::kMtMax;
    eo::MtApply t;
    memset(&t, 0, sizeof(t));
    int64_t biggest = 0;
    for (int i = 0; i < cnt; ++i) {
      if (p[i0 + i] == nullptr || update[i0 + i] == nullptr || numel[i0 + i] < 0)
        return fail(EO_ERR_BAD_ARG, "tensor %d: null pointer or negative size", i0 + i);
      t.p[i] = p[i0 + i];
      t.u[i] = update[i0 + i];
      t.numel[i] = numel[i0 + i];
      t.scale[i] = scale[i0 + i];
      if (numel[i0 + i] > biggest) biggest = numel[i0 + i];
    }
    int bx = eo::ew_blocks(biggest, 16);
    if (max_blocks_per_tensor > 0 && bx > max_blocks_per_tensor) bx = max_blocks_per_tensor;
    const dim3 grid(bx, cnt);
    if (update_is_bf16)
      eo::muon_apply_mt_kernel<__nv_bfloat16><<<grid, eo::kEwThreads, 0, s>>>(t, shrink, extra_scale, lr);
    else
      eo::muon_apply_mt_kernel<float><<<grid, eo::kEwThreads, 0, s>>>(t, shrink, extra_scale, lr);
  }
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}

namespace {
inline int64_t round_up(int64_t v, int64_t to) { return (v + to - 1) / to * to; }

struct NsLayout {
  int m, n;           // Gram side and contraction length of the wide orientation
  int64_t ldm;        // row stride of A and B
  int64_t a_elems;    // elements of one of A / B (whole batch)
  int64_t ldt;        // row stride of the temporary iterate
  int64_t t_stride;   // batch stride of the temporary iterate
  int64_t t_elems;
};

NsLayout ns_layout(int batch, int rows, int cols) {
  NsLayout L;
  L.m = rows <= cols ? rows : cols;
  L.n = rows <= cols ? cols : rows;
  L.ldm = round_up(L.m, 8);
  L.a_elems = round_up(static_cast<int64_t>(batch) * L.m * L.ldm, 128);
  L.ldt = round_up(cols, 8);
  L.t_stride = round_up(static_cast<int64_t>(rows) * L.ldt, 8);
  L.t_elems = round_up(static_cast<int64_t>(batch) * L.t_stride, 128);
  return L;
}
}  // namespace

size_t eo_newton_schulz_workspace_bytes(int batch, int rows, int cols) {
  if (batch <= 0 || rows <= 0 || cols <= 0) return 0;
  const NsLayout L = ns_layout(batch, rows, cols);
  return static_cast<size_t>(2 * L.a_elems + L.t_elems) * 2;
}

namespace {
// All iterations of a batch of small wide matrices (rows <= 128 <= ... cols) in one persistent kernel.
int launch_ns_small(DeviceInfo* dev, void* X, int batch, int rows, int cols, int64_t ld, int64_t stride,
                    const float* host_abc, int steps, void* T, int64_t ldt, int64_t t_stride, void* out, int out_fp32,
                    int64_t ldo, int64_t strideo, const float* dev_scales, void* stream) {
  eo::SmallMaps maps;
  memset(&maps, 0, sizeof(maps));
  if (int rc = make_map(&maps.x[0], X, 2, cols, rows, batch, ld, stride, 64, 128)) return rc;
  if (int rc = make_map(&maps.x[1], T, 2, cols, rows, batch, ldt, t_stride, 64, 128)) return rc;
  eo::SmallParams p;
  memset(&p, 0, sizeof(p));
  p.batch = batch;
  p.m = rows;
  p.n = cols;
  p.steps = steps;
  for (int i = 0; i < 3 * steps; ++i) p.abc[i] = host_abc[i];
  p.buf[0] = static_cast<unsigned short*>(X);
  p.buf[1] = static_cast<unsigned short*>(T);
  p.ld[0] = ld;
  p.stride[0] = stride;
  p.ld[1] = ldt;
  p.stride[1] = t_stride;
  p.out = out;
  p.ldo = ldo;
  p.strideo = strideo;
  p.out_fp32 = out_fp32;
  p.status = dev->status_ptr;
  p.dev_scale = dev_scales;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    p.sched = dev->sched_ptr + 2 * (dev->sched_next % kSchedSlots);
    dev->sched_next++;
  }
  const int grid = batch < dev->sm_count ? batch : dev->sm_count;
  eo::eo_ns_small_kernel<<<grid, eo::kSmallThreads, eo::kSmallSmemBytes, static_cast<cudaStream_t>(stream)>>>(maps, p);
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}
}  // namespace

int eo_newton_schulz_bf16(void* X, int batch, int rows, int cols, int64_t ld, int64_t stride, const float* host_abc,
                          int steps, int flags, void* out, int out_fp32, int64_t ldo, int64_t strideo,
                          void* workspace, size_t workspace_bytes, const float* dev_scales, void* stream) {
  const int use_syrk = flags & 1;
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (batch < 0 || rows < 0 || cols < 0 || steps < 1) return fail(EO_ERR_BAD_ARG, "bad size or steps < 1");
  if (batch == 0 || rows == 0 || cols == 0) return EO_OK;
  if (X == nullptr || out == nullptr || host_abc == nullptr) return fail(EO_ERR_BAD_ARG, "null pointer");
  const size_t need = eo_newton_schulz_workspace_bytes(batch, rows, cols);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(EO_ERR_WORKSPACE, "newton_schulz workspace: need %zu bytes, got %zu", need, workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(EO_ERR_BAD_ARG, "workspace must be 256-byte aligned");
  const NsLayout L = ns_layout(batch, rows, cols);
  const bool tall = rows > cols;
  char* ws = static_cast<char*>(workspace);
  void* A = ws;
  void* S = ws + L.a_elems * 2;
  void* T = ws + 2 * L.a_elems * 2;
  const int64_t a_stride = static_cast<int64_t>(L.m) * L.ldm;
  const int syrk = use_syrk && (rows % 8 == 0) && (cols % 8 == 0);

  // Matrices whose Gram matrix is a single tile take the fused kernel: A, A^2 and S stay in shared memory.
  const bool small = !(flags & 2) && rows <= 128 && rows <= cols && cols >= 256 && steps <= eo::kSmallMaxSteps;
  if (small)
    return launch_ns_small(dev, X, batch, rows, cols, ld, stride, host_abc, steps, T, L.ldt, L.t_stride, out, out_fp32,
                           ldo, strideo, dev_scales, stream);

  // Iterate buffers: step i reads `cur` and writes `nxt`; the last step writes `out`.
  void* cur = X;
  int64_t cur_ld = ld, cur_stride = stride;
  for (int it = 0; it < steps; ++it) {
    const float a = host_abc[3 * it], b = host_abc[3 * it + 1], c = host_abc[3 * it + 2];
    const bool last = (it == steps - 1);
    int rc;
    // A = X X^T over the wide orientation.  Wide storage: operands K-major; tall storage: MN-major.
    // With deferred normalisation the first iterate is un-normalised: its Gram product takes 1 / norm^2 and its
    // update 1 / norm from the device, after which the iterate is what the normalised input would have given.
    const float* ds = (it == 0) ? dev_scales : nullptr;
    rc = launch_gemm(cur, tall ? 1 : 0, cur_ld, cur_stride, 0, cur, tall ? 1 : 0, cur_ld, cur_stride, 0, nullptr, 0, 0,
                     A, L.ldm, a_stride, batch, L.m, L.m, L.n, 1.0f, 0.0f, 1.0f, 0, 0, 0, syrk, 0, stream, nullptr, 0,
                     ds, 1);
    if (rc) return rc;
    const void* Sop = A;
    float alpha = b, beta = a;
    if (c != 0.0f) {
      // S = b A + c A A (A symmetric)
      rc = launch_gemm(A, 0, L.ldm, a_stride, 0, A, syrk ? 0 : 1, L.ldm, a_stride, 0, A, L.ldm, a_stride, S, L.ldm,
                       a_stride, batch, L.m, L.m, L.m, c, b, 1.0f, 0, 0, 0, syrk, 0, stream);
      if (rc) return rc;
      Sop = S;
      alpha = 1.0f;
    }
    void* dst;
    int64_t dst_ld, dst_stride;
    if (last) {
      dst = out;
      dst_ld = ldo;
      dst_stride = strideo;
    } else {
      // ping-pong between the temporary and the caller's X (which is clobbered from the second step on)
      dst = (cur == X) ? T : X;
      dst_ld = (dst == T) ? L.ldt : ld;
      dst_stride = (dst == T) ? L.t_stride : stride;
    }
    const int d32 = last ? out_fp32 : 0;
    if (!tall) {
      // X' = beta X + alpha S X : A-operand S (m x m, K-major), B-operand X as (n x m): stored m x n, MN-major
      rc = launch_gemm(Sop, 0, L.ldm, a_stride, 0, cur, 1, cur_ld, cur_stride, 0, cur, cur_ld, cur_stride, dst, dst_ld,
                       dst_stride, batch, L.m, L.n, L.m, alpha, beta, 1.0f, 0, d32, d32, 0, 0, stream, nullptr, 0, ds, 2);
    } else {
      // stored transposed (n x m): X'^T = beta X^T + alpha X^T S, S symmetric, both operands K-major
      rc = launch_gemm(cur, 0, cur_ld, cur_stride, 0, Sop, 0, L.ldm, a_stride, 0, cur, cur_ld, cur_stride, dst, dst_ld,
                       dst_stride, batch, L.n, L.m, L.m, alpha, beta, 1.0f, 0, d32, d32, 0, 0, stream, nullptr, 0, ds, 2);
    }
    if (rc) return rc;
    cur = dst;
    cur_ld = dst_ld;
    cur_stride = dst_stride;
  }
  return EO_OK;
}

namespace {
// Workspace of the fp32 driver: bf16 planes of the iterate and of A / S, fp32 A and S, one fp32 temporary iterate.
struct NsF32Layout {
  int m, n;
  int64_t ldxp, xp_stride, xp_plane;  // planes of the iterate, in its storage orientation (rows x cols)
  int64_t ldm, a_stride;              // fp32 A and S
  int64_t ldmp, mp_stride, mp_plane;  // planes of A / S
  int64_t ldt, t_stride;              // fp32 temporary iterate
  size_t off_xp, off_a, off_s, off_mp, off_t, off_parts, total;
  int max_ksplit;  // partial Gram matrices the workspace has room for
};

// K-split of the Gram product of a single small matrix.  A = X X^T of an m x n iterate has only
// ceil(m/128) (ceil(m/128) + 1) / 2 lower-triangle tiles, each a loop over all of n (six plane pairs long on the
// fp32 path): for m = 1024 that is 36 CTAs on `sms` SMs.  Splitting n into S slices that run as the S "batches" of
// one launch fills the machine; the S partial matrices are summed by the pass that splits A into planes anyway.
int ns_f32_ksplit(int batch, int m, int n, int sms) {
  if (batch != 1) return 1;
  const long long tm = (m + 127) / 128;
  const long long tiles = tm * (tm + 1) / 2;
  int S = 1;
  while (S < 8 && tiles * (2 * S) <= sms && n / (2 * S) >= 1024 && n % (2 * S * 8) == 0) S *= 2;
  return S;
}

NsF32Layout ns_f32_layout(int batch, int rows, int cols) {
  NsF32Layout L;
  L.m = rows <= cols ? rows : cols;
  L.n = rows <= cols ? cols : rows;
  L.ldxp = round_up(cols, 8);
  L.xp_stride = static_cast<int64_t>(rows) * L.ldxp;
  L.xp_plane = round_up(static_cast<int64_t>(batch) * L.xp_stride, 128);
  L.ldm = round_up(L.m, 4);
  L.a_stride = static_cast<int64_t>(L.m) * L.ldm;
  L.ldmp = round_up(L.m, 8);
  L.mp_stride = static_cast<int64_t>(L.m) * L.ldmp;
  L.mp_plane = round_up(static_cast<int64_t>(batch) * L.mp_stride, 128);
  L.ldt = round_up(cols, 4);
  L.t_stride = static_cast<int64_t>(rows) * L.ldt;
  size_t off = 0;
  auto take = [&off](size_t bytes) {
    const size_t at = off;
    off += (bytes + 255) / 256 * 256;
    return at;
  };
  L.off_xp = take(static_cast<size_t>(3 * L.xp_plane) * 2);
  L.off_a = take(static_cast<size_t>(batch) * L.a_stride * 4);
  L.off_s = take(static_cast<size_t>(batch) * L.a_stride * 4);
  L.off_mp = take(static_cast<size_t>(3 * L.mp_plane) * 2);
  L.off_t = take(static_cast<size_t>(batch) * L.t_stride * 4);
  // The workspace size must not depend on the device: reserve what a 256-SM part would use (no larger one exists)
  // and let the launch take the smaller of this and what its own SM count asks for.
  L.max_ksplit = ns_f32_ksplit(batch, L.m, L.n, 256);
  L.off_parts = L.max_ksplit > 1 ? take(static_cast<size_t>(L.max_ksplit) * L.a_stride * 4) : off;
  L.total = off;
  return L;
}
}  // namespace

size_t eo_newton_schulz_f32_workspace_bytes(int batch, int rows, int cols) {
  if (batch <= 0 || rows <= 0 || cols <= 0) return 0;
  return ns_f32_layout(batch, rows, cols).total;
}

int eo_newton_schulz_f32(const float* X, int batch, int rows, int cols, int64_t ld, int64_t stride,
                         const float* host_abc, int steps, float* out, int64_t ldo, int64_t strideo, void* workspace,
                         size_t workspace_bytes, void* stream) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (batch < 0 || rows < 0 || cols < 0 || steps < 1) return fail(EO_ERR_BAD_ARG, "bad size or steps < 1");
  if (batch == 0 || rows == 0 || cols == 0) return EO_OK;
  if (X == nullptr || out == nullptr || host_abc == nullptr) return fail(EO_ERR_BAD_ARG, "null pointer");
  if (ld < cols || ldo < cols) return fail(EO_ERR_BAD_ARG, "leading dimension smaller than cols");
  const NsF32Layout L = ns_f32_layout(batch, rows, cols);
  if (workspace == nullptr || workspace_bytes < L.total)
    return fail(EO_ERR_WORKSPACE, "newton_schulz_f32 workspace: need %zu bytes, got %zu", L.total, workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return fail(EO_ERR_BAD_ARG, "workspace must be 256-byte aligned");
  char* ws = static_cast<char*>(workspace);
  void* Xp = ws + L.off_xp;
  float* A = reinterpret_cast<float*>(ws + L.off_a);
  float* S = reinterpret_cast<float*>(ws + L.off_s);
  void* Mp = ws + L.off_mp;
  float* T = reinterpret_cast<float*>(ws + L.off_t);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int tall = rows > cols ? 1 : 0;
  int ksplit = ns_f32_ksplit(batch, L.m, L.n, dev->sm_count);
  if (ksplit > L.max_ksplit) ksplit = L.max_ksplit;
  float* parts = reinterpret_cast<float*>(ws + L.off_parts);

  const float* cur = X;
  int64_t cur_ld = ld, cur_stride = stride;
  for (int it = 0; it < steps; ++it) {
    const float a = host_abc[3 * it], b = host_abc[3 * it + 1], c = host_abc[3 * it + 2];
    int rc;
    // planes of the iterate, in storage orientation
    eo::launch_split3(cur, batch, rows, cols, cur_ld, cur_stride, Xp, L.ldxp, L.xp_stride, L.xp_plane, st);
    EO_CUDA(cudaGetLastError());
    // A = X X^T over the wide orientation, lower triangle computed and mirrored
    if (ksplit > 1) {
      // slices of the contraction dimension as the batches of one launch: n / ksplit columns of the wide
      // orientation apart, which is that many rows of a tall (transposed) storage
      const int kslice = L.n / ksplit;
      const int64_t slice_stride = tall ? static_cast<int64_t>(kslice) * L.ldxp : kslice;
      rc = launch_gemm(Xp, tall, L.ldxp, slice_stride, L.xp_plane, Xp, tall, L.ldxp, slice_stride, L.xp_plane, nullptr,
                       0, 0, parts, L.ldm, L.a_stride, ksplit, L.m, L.m, kslice, 1.0f, 0.0f, 1.0f, 1, 1, 0, 1, 0, stream);
      if (rc) return rc;
      eo::launch_sum_split3(parts, ksplit, L.a_stride, L.m, L.m, L.ldm, A, Mp, L.ldmp, L.mp_plane, st);
    } else {
      rc = launch_gemm(Xp, tall, L.ldxp, L.xp_stride, L.xp_plane, Xp, tall, L.ldxp, L.xp_stride, L.xp_plane, nullptr, 0,
                       0, A, L.ldm, L.a_stride, batch, L.m, L.m, L.n, 1.0f, 0.0f, 1.0f, 1, 1, 0, 1, 0, stream);
      if (rc) return rc;
      eo::launch_split3(A, batch, L.m, L.m, L.ldm, L.a_stride, Mp, L.ldmp, L.mp_stride, L.mp_plane, st);
    }
    EO_CUDA(cudaGetLastError());
    float alpha = b, beta = a;
    if (c != 0.0f) {
      // S = b A + c A A, then its planes replace those of A
      rc = launch_gemm(Mp, 0, L.ldmp, L.mp_stride, L.mp_plane, Mp, 0, L.ldmp, L.mp_stride, L.mp_plane, A, L.ldm,
                       L.a_stride, S, L.ldm, L.a_stride, batch, L.m, L.m, L.m, c, b, 1.0f, 1, 1, 0, 1, 0, stream);
      if (rc) return rc;
      eo::launch_split3(S, batch, L.m, L.m, L.ldm, L.a_stride, Mp, L.ldmp, L.mp_stride, L.mp_plane, st);
      EO_CUDA(cudaGetLastError());
      alpha = 1.0f;
    }
    // The iterate alternates between `out` and the temporary so that the last step lands in `out`.
    const bool to_out = ((steps - 1 - it) % 2) == 0;
    float* dst = to_out ? out : T;
    const int64_t dst_ld = to_out ? ldo : L.ldt, dst_stride = to_out ? strideo : L.t_stride;
    if (!tall) {
      // X' = beta X + alpha S X: S is the K-major A operand, X (m x n row-major) the MN-major B operand
      rc = launch_gemm(Mp, 0, L.ldmp, L.mp_stride, L.mp_plane, Xp, 1, L.ldxp, L.xp_stride, L.xp_plane, cur, cur_ld,
                       cur_stride, dst, dst_ld, dst_stride, batch, L.m, L.n, L.m, alpha, beta, 1.0f, 1, 1, 0, 0, 0, stream);
    } else {
      // stored transposed (n x m): X'^T = beta X^T + alpha X^T S with S symmetric, both operands K-major
      rc = launch_gemm(Xp, 0, L.ldxp, L.xp_stride, L.xp_plane, Mp, 0, L.ldmp, L.mp_stride, L.mp_plane, cur, cur_ld,
                       cur_stride, dst, dst_ld, dst_stride, batch, L.n, L.m, L.m, alpha, beta, 1.0f, 1, 1, 0, 0, 0, stream);
    }
    if (rc) return rc;
    cur = dst;
    cur_ld = dst_ld;
    cur_stride = dst_stride;
  }
  return EO_OK;
}

size_t eo_tp_gram_inbox_bytes(int N, int world) {
  if (N <= 0 || world <= 0) return 0;
  return static_cast<size_t>(world) * tp_slots(N, world) * eo::kBlockM * tp_tile_n(N) * 2;
}

size_t eo_tp_gram_flag_count(int N, int world) {
  if (N <= 0 || world <= 0) return 0;
  return static_cast<size_t>(world) * tp_slots(N, world);
}

int eo_tp_gram_allreduce(const void* X, int x_trans, int64_t ldx, int N, int K, int world, int rank,
                         void* const* partial_ptrs, void* const* flag_ptrs, void* const* gram_ptrs,
                         const void* partials_multicast, void* gram_multicast, int64_t ld_gram, uint32_t seq,
                         void* stream) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (world < 2 || world > 8 || rank < 0 || rank >= world) return fail(EO_ERR_BAD_ARG, "world must be 2..8");
  if (N <= 0 || K <= 0 || N % 8 != 0) return fail(EO_ERR_BAD_ARG, "N must be a positive multiple of 8, K positive");
  if (X == nullptr || partial_ptrs == nullptr || flag_ptrs == nullptr || gram_ptrs == nullptr)
    return fail(EO_ERR_BAD_ARG, "null pointer");
  if (ld_gram < N || ld_gram % 8 != 0) return fail(EO_ERR_BAD_ARG, "ld_gram must be a multiple of 8 and >= N");
  if ((partials_multicast == nullptr) != (gram_multicast == nullptr))
    return fail(EO_ERR_BAD_ARG, "give both multicast aliases or neither");
  for (int r = 0; r < world; ++r) {
    if (partial_ptrs[r] == nullptr || flag_ptrs[r] == nullptr || gram_ptrs[r] == nullptr)
      return fail(EO_ERR_BAD_ARG, "null peer pointer for rank %d", r);
    if ((reinterpret_cast<uintptr_t>(partial_ptrs[r]) | reinterpret_cast<uintptr_t>(gram_ptrs[r])) & 15)
      return fail(EO_ERR_BAD_ARG, "peer buffers must be 16-byte aligned");
  }
  if ((reinterpret_cast<uintptr_t>(partials_multicast) | reinterpret_cast<uintptr_t>(gram_multicast)) & 15)
    return fail(EO_ERR_BAD_ARG, "multicast aliases must be 16-byte aligned");
  unsigned int* flags[8];
  for (int r = 0; r < world; ++r) flags[r] = static_cast<unsigned int*>(flag_ptrs[r]);
  TpExchange tp{world, rank, seq, partial_ptrs, flags, gram_ptrs, partials_multicast, gram_multicast, ld_gram};
  // One launch: the SYRK main loop, the partial tiles and flags from its epilogue, and the owners' reduction
  // into every rank's Gram matrix (both triangles) from the reducer warps of the same CTAs.
  return launch_gemm(X, x_trans, ldx, 0, 0, X, x_trans, ldx, 0, 0, nullptr, 0, 0, nullptr, 0, 0, 1, N, N, K, 1.0f, 0.0f,
                     1.0f, 0, 0, 0, /*tri=*/1, 0, stream, &tp);
}

int eo_tp_gram_mirror(void* gram, int N, int64_t ld_gram, void* stream) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (gram == nullptr || N <= 0 || ld_gram < N) return fail(EO_ERR_BAD_ARG, "bad Gram matrix");
  if (N % 64 == 0 && ld_gram % 8 == 0 && (reinterpret_cast<uintptr_t>(gram) & 15) == 0) {
    const int nb = N / 64;
    eo::mirror_lower64_kernel<<<nb * (nb + 1) / 2, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<unsigned short*>(gram), N, ld_gram);
  } else {
    const int nb = (N + 31) / 32;
    eo::mirror_lower_kernel<<<nb * (nb + 1) / 2, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<unsigned short*>(gram), N, ld_gram);
  }
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}

int eo_multicast_copy(const void* src, void* dst_multicast, size_t bytes, void* stream) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (bytes == 0) return EO_OK;
  if (src == nullptr || dst_multicast == nullptr) return fail(EO_ERR_BAD_ARG, "null pointer");
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst_multicast)) & 15) || bytes % 16 != 0)
    return fail(EO_ERR_BAD_ARG, "multicast copy needs 16-byte aligned pointers and a size that is a multiple of 16");
  const long long nvec = static_cast<long long>(bytes / 16);
  long long blocks = (nvec + 256 * 8 - 1) / (256 * 8);
  if (blocks > 4LL * dev->sm_count) blocks = 4LL * dev->sm_count;
  if (blocks < 1) blocks = 1;
  eo::multicast_copy_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst_multicast), nvec);
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}

size_t eo_sumsq_noalloc_max_partials(void) { return kNoAllocMaxPartials; }

int eo_sumsq_f32_noalloc(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride,
                         double* sumsq, void* stream) {
  {
    // The first library call on a device resolves symbol addresses and sets kernel attributes, which is not
    // allowed while a stream is being captured: refuse that combination instead of failing inside the set-up.
    int cur = 0;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaGetDevice(&cur) == cudaSuccess && cur >= 0 && cur < kMaxDevices &&
        cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &cap) == cudaSuccess &&
        cap != cudaStreamCaptureStatusNone) {
      std::lock_guard<std::mutex> lock(g_mu);
      if (!g_dev[cur].ready)
        return fail(EO_ERR_BAD_ARG, "eo_sumsq_f32_noalloc: the first library call on a device must be made outside "
                                    "stream capture");
    }
  }
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (batch < 0 || rows < 0 || cols < 0) return fail(EO_ERR_BAD_ARG, "negative size");
  if (batch == 0) return EO_OK;
  if (sumsq == nullptr) return fail(EO_ERR_BAD_ARG, "sumsq is NULL");
  if (ld < cols) return fail(EO_ERR_BAD_ARG, "ld smaller than cols");
  if (rows > 0 && cols > 0 && x == nullptr) return fail(EO_ERR_BAD_ARG, "x is NULL");
  const size_t need = static_cast<size_t>(batch) * eo::sumsq_blocks_per_matrix(rows, cols);
  if (need > kNoAllocMaxPartials)
    return fail(EO_ERR_WORKSPACE,
                "eo_sumsq_f32_noalloc: %d matrices of %lld x %lld need %zu partial sums, the built-in scratch holds "
                "%zu; use eo_sumsq_f32 with caller-provided scratch",
                batch, (long long)rows, (long long)cols, need, kNoAllocMaxPartials);
  // Every partial this call reads back is written by it first, so stale contents of the shared array are harmless.
  eo::launch_sumsq(x, batch, rows, cols, ld, stride, sumsq, dev->noalloc_partials, static_cast<cudaStream_t>(stream));
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}

int eo_normalize_f32(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride,
                     const double* sumsq, float eps, int clamp_eps, void* out, int64_t ldo, int64_t strideo,
                     int out_fp32, int round_bf16, void* stream) {
  DeviceInfo* dev = nullptr;
  if (int rc = device_setup(&dev)) return rc;
  if (batch < 0 || rows < 0 || cols < 0) return fail(EO_ERR_BAD_ARG, "negative size");
  if (batch == 0 || rows == 0 || cols == 0) return EO_OK;
  if (x == nullptr || out == nullptr || sumsq == nullptr) return fail(EO_ERR_BAD_ARG, "null pointer");
  if (ld < cols || ldo < cols) return fail(EO_ERR_BAD_ARG, "leading dimension smaller than cols");
  eo::launch_normalize(x, batch, rows, cols, ld, stride, sumsq, eps, clamp_eps, out, ldo, strideo, out_fp32,
                       round_bf16, static_cast<cudaStream_t>(stream));
  EO_CUDA(cudaGetLastError());
  return EO_OK;
}

}  // extern "C"
