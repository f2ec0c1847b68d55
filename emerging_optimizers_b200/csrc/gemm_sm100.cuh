// Persistent, warp-specialised tcgen05 GEMM for sm_100a:
//
//     D[b] = alpha * op(A[b]) * op(B[b])^T + beta * C[b]            (fp32 accumulation in TMEM)
//
// with A given as (M x K), B as (N x K); each operand may be stored K-major (K contiguous) or
// MN-major (M/N contiguous).  With `tri` set the problem is a symmetric rank-k update (A == B,
// M == N): only tiles touching the lower triangle are computed, the lower part is stored and,
// unless `skip_upper`, mirrored into the upper part, so that every output element is written once.
//
// One CTA per SM, 320 threads:
//   warp 0      TMA producer   (global -> 128B-swizzled shared-memory ring, kStages deep)
//   warp 1      MMA issuer     (one elected thread issues tcgen05.mma, accumulators in TMEM)
//   warps 2..9  epilogue       (tcgen05.ld -> alpha/beta -> round -> global stores; two warps per TMEM
//                               lane quarter, so that twice as many C loads and D stores are in flight)
// TMEM holds two 128 x 256 fp32 accumulators so the epilogue of tile t overlaps the main loop of
// tile t+1.  Every wait is bounded; a wait that runs out records a code in the status word and the
// role leaves its loop.
//
// Tensor-parallel Gram mode (template parameter kTp, with `tri`): every rank of a tensor-parallel group runs
// this kernel on its shard and the sum over ranks lands in every rank's Gram matrix before the kernel ends.
// The epilogue writes each bf16 partial tile into the rank's own symmetric buffer and raises a flag in the
// memory of the tile's owner rank (tile t belongs to rank t mod P).  Four extra warps per CTA (warps 10..13)
// are the reducer: for every tile this rank owns they wait (bounded) for the flags of all ranks, read the
// tile with one NVSwitch load-reduce per 16 bytes (fp32 accumulation in the switch, one rounding) -- or, where
// no multicast mapping exists, peer by peer with plain loads -- and store the tile and its mirror image into
// all ranks' Gram matrices with multicast stores (or peer by peer).  Tiles become ready in scheduling order on
// all ranks at about the same time, so the exchange runs behind the main loop of the following tiles.
#pragma once

#include <cuda_bf16.h>

#include "sm100_ptx.cuh"

namespace eo {

constexpr int kBlockM = 128;
constexpr int kMaxBlockN = 256;
constexpr int kRowBytes = 128;  // one swizzle row: 64 bf16 along the contiguous dimension
constexpr int kBlockK = 64;     // K extent of one pipeline stage
constexpr int kMaxPlanes = 3;   // bf16 planes of a split-fp32 operand
constexpr int kStages = 4;       // ring depth with 128-row A tiles (48 KiB stages); 3 with 256-row A tiles (64 KiB)
constexpr int kStageABytes = kBlockM * kRowBytes;     // 16 KiB
constexpr int kStageBBytes = kMaxBlockN * kRowBytes;  // 32 KiB
constexpr int kStageBytes = kStageABytes + kStageBBytes;
#ifndef EO_EPILOGUE_WARPS
#define EO_EPILOGUE_WARPS 8
#endif
constexpr int kEpilogueWarps = EO_EPILOGUE_WARPS;  // 4 or 8: one or two per TMEM lane quarter, alternating 32-column chunks
constexpr int kGemmThreads = 64 + 32 * kEpilogueWarps;
constexpr int kTmemCols = 512;
constexpr int kGroupM = 16;  // row-block group height of the general tile order

constexpr int kTileQueue = 4;  // depth of the in-CTA queue of tile indices handed from the producer to the other roles

// Shared-memory budget: ring + barriers + tile queue + TMEM address slot, plus slack for 1024-byte alignment.
constexpr int kGemmSmemBytes = kStages * kStageBytes + 512 + 1024;

// Tensor-parallel Gram mode: the reducer warps and their staging block of 128 rows x 32 columns (bf16, rows padded
// by 8 elements against bank conflicts when the block is read column-wise for the mirror image).
constexpr int kTpReducerThreads = 128;
constexpr int kTpStagePitch = 32 + 8;
constexpr int kTpStageBytes = kBlockM * kTpStagePitch * 2;
constexpr int kGemmTpSmemBytes = kGemmSmemBytes + kTpStageBytes;
constexpr uint32_t kTpPoison = 0x7FC07FC0u;  // two bf16 NaNs: what a reducer that gave up waiting stores

struct GemmParams {
  int batch, M, N, K;
  int bn;          // tile width: 128 or 256
  int bm;          // tile height: 128, or 256 = two 128-row MMAs per k-step sharing one B tile (one accumulator
                   // each, so the whole of TMEM belongs to one tile): a third fewer operand bytes per FLOP
  int stages;      // ring depth: 4 (bm 128) or 3 (bm 256)
  int a_mn, b_mn;  // operand stored MN-major (1) or K-major (0)
  int nterms;      // operand-plane pairs accumulated into one result (1: plain bf16; 6: split-fp32 product)
  int term_a[6];   // plane of A used by term t
  int term_b[6];   // plane of B used by term t
  int tri;         // symmetric update: lower-triangle tiles only
  int same_ab;     // A and B are the same matrix (SYRK): a tile whose rows lie inside its column range reads
                   // its A operand out of the B tile instead of loading it a second time
  int skip_upper;  // with tri: do not mirror into the upper triangle
  int c_fp32;      // element type of C: fp32 (1) or bf16 (0)
  int d_fp32;      // element type of D
  int round_bf16;  // with d_fp32: round the result to bf16 before widening (keeps the bf16 rounding point)
  int vec_ok;      // C/D rows are 16-byte aligned: the full-chunk fast path may use vector accesses
  const void* C;
  long long ldc, strideC;
  void* D;
  long long ldd, strideD;
  float alpha, beta, post_scale;
  int tiles_m, tiles_n, tiles_per_batch, total_tiles;
  // Shared-memory descriptor geometry (bytes), filled in by the host:
  //   adv_*: start-address advance per MMA instruction (32 bytes of K)
  //   lbo_*/sbo_*: leading / stride byte offsets of the operand's canonical 128B-swizzled layout
  unsigned int adv_a, adv_b, lbo_a, lbo_b, sbo_a, sbo_b;
  unsigned int* status;
  // Work distribution: tiles are handed out through a global counter (`sched[0]`, next tile index), so a CTA
  // that starts late or shares its SM with another kernel simply takes fewer tiles.  `sched[1]` counts CTAs that
  // have finished; the last one zeroes both words for the next launch that uses this slot.
  unsigned int* sched;
  // Tensor-parallel Gram mode (tp_world > 1, with tri; see the head of this file).  Tiles are numbered on the
  // grid of 128-row x bn-column tiles, column block by column block, rows from the diagonal down: tile t is owned
  // by rank t % tp_world and is that rank's slot t / tp_world.
  int tp_world, tp_rank;
  unsigned int tp_seq;              // sequence number of this exchange (flag value that means "tile written")
  int tp_slots, tp_total;           // slots per owner; number of tiles
  unsigned short* tp_partials;      // this rank's partial tiles, [tile][128][bn] bf16 (local memory)
  unsigned int* tp_flags[8];        // per owner rank: this rank's flag words in the owner's memory, [slot]
  const unsigned int* tp_my_flags;  // flag words other ranks raise for the tiles this rank owns, [rank][slot]
  const unsigned short* tp_partials_mc;       // multicast alias of tp_partials (nullptr: read the peers one by one)
  const unsigned short* tp_partials_peer[8];  // every rank's tp_partials
  unsigned short* tp_gram_mc;       // multicast alias of the Gram matrices (nullptr: store to the peers one by one)
  unsigned short* tp_gram[8];       // every rank's Gram matrix, N x tp_ld bf16
  long long tp_ld;
  long long tp_wait_cycles;         // budget of one wait for the other ranks' flags
  int tp_lower_only;                // reducer stores the lower triangle only (the caller mirrors its own copy)
  // D is a multicast address (general product, bf16 D, N a multiple of 32): every store goes to all ranks.
  int d_mc;
  // Deferred Frobenius normalisation: per-matrix factors on the device (two floats per batch entry, see
  // sumsq_scales_kernel).  Mode 1 multiplies alpha by dev_scale[2 b] (the product of two un-normalised operands);
  // mode 2 multiplies alpha * acc + beta * C by dev_scale[2 b + 1] before the result is rounded.
  const float* dev_scale;
  int dev_scale_mode;
  // Split tail of the pair kernel (gemm_pair_sm100.cuh): of every matrix's tiles, those from split_first on are cut
  // into split_s pieces along K.  split_first == tiles_per_batch: nothing is split.
  int split_first;
  int split_s;
  int split_items_per_batch;  // work items per matrix: split_first + (tiles_per_batch - split_first) * split_s
  float* split_ws;            // [split tile][piece][CTA of the pair][128 x 256] fp32 partial accumulators
  unsigned int* split_cnt;    // [split tile][CTA of the pair][epilogue warp] arrivals, zero between launches
  // Tile order and L2 policies of the pair kernel.
  int pair_group_m;  // general products: row-block group height (tiles of a group run column by column)
  int pair_band;     // triangular products: column-band width in tiles (0: column-major through the triangle)
  int pair_hint_a;   // L2 eviction policy of the A / B operand loads: 0 none, 1 evict first, 2 evict last
  int pair_hint_b;
};

__host__ __device__ __forceinline__ void decode_tile(const GemmParams& p, int t, int& b, int& ti, int& tj,
                                            const int bm = kBlockM) {
  b = t / p.tiles_per_batch;
  int r = t - b * p.tiles_per_batch;
  if (p.tri) {
    tj = 0;
    ti = 0;
    for (int j = 0; j < p.tiles_n; ++j) {
      const int first = (j * p.bn) / bm;  // first row block that reaches column block j (bm is a constant here)
      const int cnt = p.tiles_m - first;
      if (r < cnt) {
        tj = j;
        ti = first + r;
        return;
      }
      r -= cnt;
    }
  } else {
    const int per_group = kGroupM * p.tiles_n;
    const int g = r / per_group;
    const int first = g * kGroupM;
    const int rows = min(kGroupM, p.tiles_m - first);
    const int w = r - g * per_group;
    ti = first + (w % rows);
    tj = w / rows;
  }
}

__device__ __forceinline__ void report(const GemmParams& p, unsigned int code) {
  if (p.status != nullptr) atomicCAS(p.status, 0u, code);
}

__device__ __forceinline__ float bf16_bits_to_float(unsigned short h) {
  return __uint_as_float(static_cast<unsigned int>(h) << 16);
}

// Epilogue for one 32-column chunk held by one thread (row `row`, columns col0..col0+31).
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, const uint32_t (&acc)[32], long long batch_c,
                                               long long batch_d, int row, int col0, float alpha, float sum_scale,
                                               const uint4* c_pre = nullptr) {
  // c_pre: the 64 bytes of bf16 C for this chunk, already loaded by the caller (only given for a full, vector-
  // addressable chunk; see the prefetch in the epilogue loop).
  if (row >= p.M) return;
  const bool has_c = (p.beta != 0.0f) && (p.C != nullptr);
  const int ncols = min(32, p.N - col0);
  if (ncols <= 0) return;
  // Number of leading columns this thread stores directly: all of them, or those with col <= row.
  const int ndirect = p.tri ? max(0, min(ncols, row - col0 + 1)) : ncols;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = alpha * __uint_as_float(acc[j]);

  const bool full = (ndirect == 32);
  if (has_c) {
    if (p.c_fp32) {
      const float* c = reinterpret_cast<const float*>(p.C) + batch_c + static_cast<long long>(row) * p.ldc + col0;
      if (full && p.vec_ok) {
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 t = __ldg(reinterpret_cast<const float4*>(c) + q);
          v[4 * q + 0] = fmaf(p.beta, t.x, v[4 * q + 0]);
          v[4 * q + 1] = fmaf(p.beta, t.y, v[4 * q + 1]);
          v[4 * q + 2] = fmaf(p.beta, t.z, v[4 * q + 2]);
          v[4 * q + 3] = fmaf(p.beta, t.w, v[4 * q + 3]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ndirect) v[j] = fmaf(p.beta, c[j], v[j]);
      }
    } else {
      const unsigned short* c =
          reinterpret_cast<const unsigned short*>(p.C) + batch_c + static_cast<long long>(row) * p.ldc + col0;
      if (full && p.vec_ok) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 t = (c_pre != nullptr) ? c_pre[q] : __ldg(reinterpret_cast<const uint4*>(c) + q);
          const unsigned int w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            v[8 * q + 2 * e + 0] = fmaf(p.beta, __uint_as_float(w[e] << 16), v[8 * q + 2 * e + 0]);
            v[8 * q + 2 * e + 1] = fmaf(p.beta, __uint_as_float(w[e] & 0xFFFF0000u), v[8 * q + 2 * e + 1]);
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < ndirect) v[j] = fmaf(p.beta, bf16_bits_to_float(c[j]), v[j]);
      }
    }
  }

  if (sum_scale != 1.0f) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] *= sum_scale;
  }

  if (p.d_fp32) {
    if (p.round_bf16) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(v[j])) * p.post_scale;
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= p.post_scale;
    }
    float* d = reinterpret_cast<float*>(p.D) + batch_d;
    float* drow = d + static_cast<long long>(row) * p.ldd + col0;
    if (full && p.vec_ok) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        reinterpret_cast<float4*>(drow)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ndirect) drow[j] = v[j];
    }
    if (p.tri && !p.skip_upper) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols && col0 + j < row) d[static_cast<long long>(col0 + j) * p.ldd + row] = v[j];
    }
  } else {
    unsigned short h[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) h[j] = __bfloat16_as_ushort(__float2bfloat16_rn(v[j]));
    unsigned short* d = reinterpret_cast<unsigned short*>(p.D) + batch_d;
    unsigned short* drow = d + static_cast<long long>(row) * p.ldd + col0;
    if (full && p.vec_ok) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint4 t;
        t.x = static_cast<unsigned int>(h[8 * q + 0]) | (static_cast<unsigned int>(h[8 * q + 1]) << 16);
        t.y = static_cast<unsigned int>(h[8 * q + 2]) | (static_cast<unsigned int>(h[8 * q + 3]) << 16);
        t.z = static_cast<unsigned int>(h[8 * q + 4]) | (static_cast<unsigned int>(h[8 * q + 5]) << 16);
        t.w = static_cast<unsigned int>(h[8 * q + 6]) | (static_cast<unsigned int>(h[8 * q + 7]) << 16);
        if (p.d_mc)
          multimem_st_16(reinterpret_cast<uint4*>(drow) + q, t);
        else
          reinterpret_cast<uint4*>(drow)[q] = t;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ndirect) drow[j] = h[j];
    }
    if (p.tri && !p.skip_upper) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (j < ncols && col0 + j < row) d[static_cast<long long>(col0 + j) * p.ldd + row] = h[j];
    }
  }
}

// TMA descriptors of up to three bf16 planes per operand.  A plain bf16 product uses plane 0 only; an
// fp32-accurate product stores each fp32 operand as x = p0 + p1 + p2 (three bf16 roundings of the running
// remainder) and accumulates the six largest plane products into the same fp32 accumulator.
struct GemmMaps {
  CUtensorMap a[kMaxPlanes];
  CUtensorMap b[kMaxPlanes];
};

// Tensor-parallel mode: one 32-column chunk of a partial tile, alpha * acc rounded to bf16, 64 contiguous bytes
// per thread at [row_local][col_local .. +32) of the tile image in this rank's partial-tile buffer.
__device__ __forceinline__ void push_chunk(const GemmParams& p, const uint32_t (&acc)[32], unsigned short* tile,
                                           int row_local, int col_local) {
  unsigned short* dst = tile + static_cast<long long>(row_local) * p.bn + col_local;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    unsigned int w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const unsigned int lo = __bfloat16_as_ushort(__float2bfloat16_rn(p.alpha * __uint_as_float(acc[8 * q + 2 * e])));
      const unsigned int hi =
          __bfloat16_as_ushort(__float2bfloat16_rn(p.alpha * __uint_as_float(acc[8 * q + 2 * e + 1])));
      w[e] = lo | (hi << 16);
    }
    reinterpret_cast<uint4*>(dst)[q] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// kHalves = 1: 128-row tiles, four 48 KiB stages, two alternating accumulators.
// kHalves = 2: 256-row tiles (two MMAs per k-step on one B tile), three 64 KiB stages, one accumulator per half.
// kTp: tensor-parallel Gram mode, with four reducer warps after the epilogue warps.
template <int kHalves, bool kTp>
__global__ void __launch_bounds__(kGemmThreads + (kTp ? kTpReducerThreads : 0), 1)
    eo_gemm_kernel(const __grid_constant__ GemmMaps maps, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle atoms are 1024 bytes: align the ring so that descriptor arithmetic holds.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);  // 4 x 48 KiB = 3 x 64 KiB
  uint64_t* full_bar = bars;                     // [kStages]
  uint64_t* empty_bar = bars + kStages;          // [kStages]
  uint64_t* acc_full_bar = bars + 2 * kStages;   // [2]
  uint64_t* acc_empty_bar = acc_full_bar + 2;    // [2]
  uint64_t* tq_full_bar = acc_empty_bar + 2;     // [kTileQueue]
  uint64_t* tq_empty_bar = tq_full_bar + kTileQueue;  // [kTileQueue]
  int* tile_queue = reinterpret_cast<int*>(tq_empty_bar + kTileQueue);  // [kTileQueue]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tile_queue + kTileQueue);
  unsigned int* push_done = tmem_slot + 1;  // [2] epilogue warps that finished writing the tile in accumulator ab
  int* tp_give_up = reinterpret_cast<int*>(push_done + 2);  // reducer: a wait for the other ranks ran out
  // reducer staging block, behind the 512 bytes of barriers and queues (kTp only)
  unsigned short* tp_stage = reinterpret_cast<unsigned short*>(smem + kStages * kStageBytes + 512);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full_bar[s], 1);
      // bm 128: all epilogue warps drain one accumulator; bm 256: half of them drain each of the two
      mbar_init(&acc_empty_bar[s], kHalves == 2 ? kEpilogueWarps / 2 : kEpilogueWarps);
    }
    for (int s = 0; s < kTileQueue; ++s) {
      mbar_init(&tq_full_bar[s], 1);
      mbar_init(&tq_empty_bar[s], 1 + kEpilogueWarps);  // MMA thread + epilogue warps
    }
    push_done[0] = 0u;
    push_done[1] = 0u;
    *tp_give_up = 0;
    mbar_init_fence();
    for (int t = 0; t < p.nterms; ++t) {
      tma_prefetch_desc(&maps.a[p.term_a[t]]);
      tma_prefetch_desc(&maps.b[p.term_b[t]]);
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  constexpr int bk = kBlockK;
  const int num_kb = (p.K + bk - 1) / bk;
  const int num_it = num_kb * p.nterms;  // pipeline iterations per tile
  constexpr int halves = kHalves;                       // MMAs (and accumulators) per k-step and tile
  constexpr int bm = kHalves * kBlockM;                 // tile height
  constexpr int a_bytes = bm * kRowBytes;               // A part of a stage: 16 or 32 KiB
  constexpr int stage_bytes = a_bytes + kStageBBytes;   // 48 or 64 KiB
  constexpr int stages = (kHalves == 2) ? 3 : kStages;  // 192 KiB of ring either way
  const uint32_t stage_tx = static_cast<uint32_t>(a_bytes + p.bn * kRowBytes);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int tq = 0;
      uint32_t tq_phase = 0;
      bool ok = true;
      while (ok) {
        // Take the next tile and publish it to the MMA and epilogue roles (-1: no tiles left).
        int t = static_cast<int>(atomicAdd(p.sched, 1u));
        if (t >= p.total_tiles) t = -1;
        if (!mbar_wait(&tq_empty_bar[tq], tq_phase ^ 1u)) {
          report(p, kStatusTimeoutProducer + 1u);
          break;
        }
        tile_queue[tq] = t;
        mbar_arrive(&tq_full_bar[tq]);
        if (++tq == kTileQueue) {
          tq = 0;
          tq_phase ^= 1u;
        }
        if (t < 0) break;
        int b, ti, tj;
        decode_tile(p, t, b, ti, tj, bm);
        const int m0 = ti * bm;
        const int n0 = tj * p.bn;
        // SYRK tile on the diagonal: its rows are among the rows of the B tile, which then serves both operands.
        const bool a_in_b = p.same_ab && m0 >= n0 && m0 + bm <= n0 + p.bn;
        const uint32_t tx = a_in_b ? static_cast<uint32_t>(p.bn * kRowBytes) : stage_tx;
        int term = 0, kb = 0;
        for (int it = 0; it < num_it; ++it) {
          const CUtensorMap* tmA = &maps.a[p.term_a[term]];
          const CUtensorMap* tmB = &maps.b[p.term_b[term]];
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u)) {
            report(p, kStatusTimeoutProducer);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * stage_bytes;
          uint8_t* sb = sa + a_bytes;
          mbar_expect_tx(&full_bar[stage], tx);
          const int k0 = kb * bk;
          if (a_in_b) {
            // nothing to load for A
          } else if (!p.a_mn) {
            for (int q = 0; q < halves; ++q)  // box {bk, 128, 1}
              tma_load_3d(sa + q * kStageABytes, tmA, &full_bar[stage], k0, m0 + q * kBlockM, b);
          } else {
            // box {bk (M), bk (K), 1}: one 128-byte-wide M atom per copy
            for (int q = 0; q < bm / bk; ++q)
              tma_load_3d(sa + q * bk * kRowBytes, tmA, &full_bar[stage], m0 + q * bk, k0, b);
          }
          if (!p.b_mn) {
            for (int q = 0; q < p.bn / kBlockM; ++q)
              tma_load_3d(sb + q * kStageABytes, tmB, &full_bar[stage], k0, n0 + q * kBlockM, b);
          } else {
            for (int q = 0; q < p.bn / bk; ++q)
              tma_load_3d(sb + q * bk * kRowBytes, tmB, &full_bar[stage], n0 + q * bk, k0, b);
          }
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
          if (++kb == num_kb) {
            kb = 0;
            ++term;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc(1u, p.a_mn != 0, p.b_mn != 0, kBlockM, p.bn);
      int stage = 0;
      uint32_t phase = 0;
      int ab = 0;
      uint32_t aphase = 0;
      int tq = 0;
      uint32_t tq_phase = 0;
      bool ok = true;
      while (ok) {
        if (!mbar_wait(&tq_full_bar[tq], tq_phase)) {
          report(p, kStatusTimeoutMma + 2u);
          break;
        }
        const int t = tile_queue[tq];
        mbar_arrive(&tq_empty_bar[tq]);
        if (++tq == kTileQueue) {
          tq = 0;
          tq_phase ^= 1u;
        }
        if (t < 0) break;
        // Accumulators: bm 128 alternates between the two; bm 256 needs both (rows 0-127 and 128-255 of the tile).
        bool acc_ok = true;
#pragma unroll
        for (int h = 0; h < halves; ++h)
          acc_ok = acc_ok && mbar_wait(&acc_empty_bar[halves == 2 ? h : ab], aphase ^ 1u);
        if (!acc_ok) {
          report(p, kStatusTimeoutMma);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>((halves == 2 ? 0 : ab) * kMaxBlockN);
        // Offset of the A operand inside the stage: its own slot, or its rows inside the B tile (see the producer).
        uint32_t a_off = 0;
        if (p.same_ab) {
          int b, ti, tj;
          decode_tile(p, t, b, ti, tj, bm);
          const int m0 = ti * bm, n0 = tj * p.bn;
          if (m0 >= n0 && m0 + bm <= n0 + p.bn) a_off = static_cast<uint32_t>(a_bytes + (m0 - n0) * kRowBytes);
        }
        for (int it = 0; it < num_it; ++it) {
          if (!mbar_wait(&full_bar[stage], phase)) {
            report(p, kStatusTimeoutMma + 1u);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * stage_bytes);
          const uint32_t sb = sa + static_cast<uint32_t>(a_bytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t db = make_smem_desc(sb + k * p.adv_b, p.lbo_b, p.sbo_b);
#pragma unroll
            for (int h = 0; h < halves; ++h) {
              // rows 128 h .. 128 h + 127 of the A tile start 16 KiB further on, in either operand layout
              const uint64_t da = make_smem_desc(sa + a_off + h * kStageABytes + k * p.adv_a, p.lbo_a, p.sbo_a);
              umma_f16(tmem_d + static_cast<uint32_t>(h * kMaxBlockN), da, db, idesc, (it | k) != 0 ? 1u : 0u);
            }
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (halves == 2) {
          umma_commit(&acc_full_bar[0]);
          umma_commit(&acc_full_bar[1]);
          aphase ^= 1u;
        } else {
          umma_commit(&acc_full_bar[ab]);
          if (++ab == 2) {
            ab = 0;
            aphase ^= 1u;
          }
        }
      }
    }
  } else if (warp < 2 + kEpilogueWarps) {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;          // TMEM lane quarter this warp may read
    const int group = (warp - 2) >> 2;     // first or second set of four warps
    // bm 128: both sets work on the same accumulator and alternate 32-column chunks.
    // bm 256: the first set drains rows 0-127 (accumulator 0), the second rows 128-255 (accumulator 1).
    constexpr bool wide_m = (halves == 2);
    const int chunk0 = wide_m ? 0 : group;
    constexpr int kChunkStep = wide_m ? 1 : kEpilogueWarps / 4;
    int ab = wide_m ? group : 0;
    uint32_t aphase = 0;
    int tq = 0;
    uint32_t tq_phase = 0;
    while (true) {
      if (!mbar_wait(&tq_full_bar[tq], tq_phase)) {
        report(p, kStatusTimeoutEpilogue + 1u);
        break;
      }
      const int t = tile_queue[tq];
      __syncwarp();
      if (lane == 0) mbar_arrive(&tq_empty_bar[tq]);
      if (++tq == kTileQueue) {
        tq = 0;
        tq_phase ^= 1u;
      }
      if (t < 0) break;
      int b, ti, tj;
      decode_tile(p, t, b, ti, tj, bm);
      const int m0 = ti * bm + (wide_m ? group * kBlockM : 0);  // first row this set of warps is responsible for
      const int n0 = tj * p.bn;
      const int row = m0 + quarter * 32 + lane;
      const int warp_last_row = m0 + quarter * 32 + 31;
      const long long batch_c = static_cast<long long>(b) * p.strideC;
      const long long batch_d = static_cast<long long>(b) * p.strideD;
      const int nchunks = p.bn / 32;
      // Prefetch of the bf16 C term (the a X of the update, the b A of the Gram polynomial): a chunk's 64 bytes per
      // thread are requested one chunk ahead - the first chunk's while the tile's last MMAs are still running - so
      // that their L2 latency is not paid once per chunk inside the epilogue, which the 256-row mode cannot overlap
      // with the next tile's main loop.  Only full, vector-addressable chunks; the others load inside epilogue_chunk.
      const bool c_pre_any = !kTp && (p.beta != 0.0f) && (p.C != nullptr) && !p.c_fp32 && p.vec_ok && row < p.M;
      auto c_pre_ok = [&](int c) {
        const int col0 = n0 + c * 32;
        return c_pre_any && c < nchunks && col0 + 32 <= p.N && (!p.tri || row - col0 >= 31);
      };
      auto c_pre_load = [&](int c, uint4 (&dst)[4]) {
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned short*>(p.C) + batch_c +
                                                          static_cast<long long>(row) * p.ldc + n0 + c * 32);
#pragma unroll
        for (int q = 0; q < 4; ++q) dst[q] = __ldg(src + q);
      };
      uint4 c_cur[4], c_nxt[4];
      bool have_cur = c_pre_ok(chunk0);
      if (have_cur) c_pre_load(chunk0, c_cur);
      if (!mbar_wait(&acc_full_bar[ab], aphase)) {
        report(p, kStatusTimeoutEpilogue);
        break;
      }
      tc_fence_after();
      float alpha = p.alpha, sum_scale = 1.0f;
      if (p.dev_scale != nullptr) {
        if (p.dev_scale_mode == 1)
          alpha *= __ldg(p.dev_scale + 2 * b);
        else
          sum_scale = __ldg(p.dev_scale + 2 * b + 1);
      }
      if (kTp) {
        // Write the partial tile into this rank's buffer, then let the last warp working on this accumulator raise
        // the flag at the tile's owner.  Owners and slots are defined on the 128-row tile grid; a 256-row tile is
        // two of those.
        int sub = t;
        bool exists = true;
        if (wide_m) {
          const int tm128 = (p.M + kBlockM - 1) / kBlockM;
          const int ti128 = 2 * ti + group;
          exists = ti128 < tm128;
          sub = tj * tm128 - tj * (tj - 1) + (ti128 - 2 * tj);  // index of tile (ti128, tj) among rows >= 2 tj
        }
        const int owner = sub % p.tp_world;
        const int slot = sub / p.tp_world;
        unsigned short* tile = p.tp_partials + static_cast<long long>(sub) * kBlockM * p.bn;
        if (exists) {
          for (int c = chunk0; c < nchunks; c += kChunkStep) {
            uint32_t acc[32];
            __syncwarp();
            tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                              static_cast<uint32_t>(ab * kMaxBlockN + c * 32),
                          acc);
            tmem_ld_wait();
            push_chunk(p, acc, tile, quarter * 32 + lane, c * 32);
          }
          __threadfence_system();
        }
        __syncwarp();
        if (lane == 0) {
          constexpr unsigned int kWarpsPerAcc = wide_m ? kEpilogueWarps / 2 : kEpilogueWarps;
          if (atomicAdd(&push_done[ab], 1u) == kWarpsPerAcc - 1u) {
            push_done[ab] = 0u;
            if (exists) {
              __threadfence_system();
              st_release_sys_u32(p.tp_flags[owner] + slot, p.tp_seq);
            }
          }
        }
      } else {
        for (int c = chunk0; c < nchunks; c += kChunkStep) {
          const int col0 = n0 + c * 32;
          if (col0 >= p.N) break;
          if (p.tri && col0 > warp_last_row) break;  // whole chunk lies above the diagonal for this warp
          uint32_t acc[32];
          __syncwarp();
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                            static_cast<uint32_t>(ab * kMaxBlockN + c * 32),
                        acc);
          // the next chunk's C values travel while this chunk is read from TMEM and processed
          const bool have_nxt = c_pre_ok(c + kChunkStep);
          if (have_nxt) c_pre_load(c + kChunkStep, c_nxt);
          tmem_ld_wait();
          epilogue_chunk(p, acc, batch_c, batch_d, row, col0, alpha, sum_scale, have_cur ? c_cur : nullptr);
#pragma unroll
          for (int q = 0; q < 4; ++q) c_cur[q] = c_nxt[q];
          have_cur = have_nxt;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty_bar[ab]);
      if (wide_m) {
        aphase ^= 1u;  // the same accumulator again for the next tile
      } else if (++ab == 2) {
        ab = 0;
        aphase ^= 1u;
      }
    }
  } else if (kTp) {
    // ------------------------------------------------------------------ reducer (warps 10..13, kTp only)
    const int rt = static_cast<int>(threadIdx.x) - kGemmThreads;  // 0..127
    const int tm128 = (p.M + kBlockM - 1) / kBlockM;
    const int nsub = p.bn / 32;  // 32-column blocks of a tile
    bool gave_up = false;
    // A unit of reducer work is a quarter (32 rows) of an owned tile when only the lower triangle is stored, so
    // that the tiles of the last wave - whose reduction nothing hides - are spread over four times as many CTAs.
    const int parts = p.tp_lower_only ? 4 : 1;
    for (int unit = blockIdx.x; unit < p.tp_slots * parts; unit += gridDim.x) {
      const int slot = unit / parts, part = unit - slot * parts;
      const int sub = slot * p.tp_world + p.tp_rank;
      if (sub >= p.tp_total) break;
      // tile (ti, tj) on the 128-row grid: column blocks in order, rows from the diagonal down
      int ti = 0, tj = 0;
      {
        int r = sub;
        for (int j = 0; j < p.tiles_n; ++j) {
          const int first = (j * p.bn) / kBlockM;
          const int cnt = tm128 - first;
          if (r < cnt) {
            tj = j;
            ti = first + r;
            break;
          }
          r -= cnt;
        }
      }
      const int m0 = ti * kBlockM, n0 = tj * p.bn;
      // Wait (bounded) until every rank has written its partial of this tile.
      if (!gave_up) {
        if (rt < p.tp_world) {
          const unsigned int* f = p.tp_my_flags + static_cast<long long>(rt) * p.tp_slots + slot;
          const long long t0 = clock64();
          while (static_cast<int>(ld_acquire_sys_u32(f) - p.tp_seq) < 0) {
            if (clock64() - t0 > p.tp_wait_cycles) {
              *tp_give_up = 1;
              report(p, kStatusTimeoutPeer);
              break;
            }
          }
        }
        named_barrier_sync(1, kTpReducerThreads);
        gave_up = (*tp_give_up != 0);
      }
      const long long tile_off = static_cast<long long>(sub) * kBlockM * p.bn;
      if (p.tp_lower_only) {
        // Lower triangle only: consecutive threads take consecutive 16-byte groups of a tile row, so a warp reads
        // and stores whole rows (512 contiguous bytes for 256-column tiles); groups above the diagonal are skipped.
        const int vpr = p.bn / 8;  // groups per tile row
        const int total = (part + 1) * (kBlockM / 4) * vpr;
        for (int v0 = part * (kBlockM / 4) * vpr + rt; v0 < total; v0 += 4 * kTpReducerThreads) {
          uint4 w[4];
          bool use[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int v = v0 + i * kTpReducerThreads;
            const int r = v / vpr, c8 = (v - r * vpr) * 8;
            const int row = m0 + r, col = n0 + c8;
            use[i] = v < total && row < p.N && col <= row;
            if (!use[i]) continue;
            const long long off = tile_off + static_cast<long long>(r) * p.bn + c8;
            if (gave_up) {
              w[i] = make_uint4(kTpPoison, kTpPoison, kTpPoison, kTpPoison);
            } else if (p.tp_partials_mc != nullptr) {
              w[i] = multimem_ld_reduce_bf16x8(p.tp_partials_mc + off);
            } else {
              float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
              for (int src = 0; src < p.tp_world; ++src) {
                const uint4 x = ld_relaxed_sys_16(p.tp_partials_peer[src] + off);
                const unsigned int xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  acc[2 * e] += __uint_as_float(xs[e] << 16);
                  acc[2 * e + 1] += __uint_as_float(xs[e] & 0xFFFF0000u);
                }
              }
              unsigned int o[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                o[e] = static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(acc[2 * e]))) |
                       (static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(acc[2 * e + 1]))) << 16);
              w[i] = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (!use[i]) continue;
            const int v = v0 + i * kTpReducerThreads;
            const int r = v / vpr, c8 = (v - r * vpr) * 8;
            const int row = m0 + r, col = n0 + c8;
            const long long at = static_cast<long long>(row) * p.tp_ld + col;
            if (col + 7 <= row) {
              if (p.tp_gram_mc != nullptr) {
                multimem_st_16(p.tp_gram_mc + at, w[i]);
              } else {
                for (int d = 0; d < p.tp_world; ++d) *reinterpret_cast<uint4*>(p.tp_gram[d] + at) = w[i];
              }
            } else {
              const unsigned int ws[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
              for (int e = 0; e < 8; ++e) {
                if (col + e > row) break;
                const unsigned short h = static_cast<unsigned short>(ws[e >> 1] >> ((e & 1) * 16));
                for (int d = 0; d < p.tp_world; ++d) p.tp_gram[d][at + e] = h;
              }
            }
          }
        }
        continue;
      }
      for (int cb = 0; cb < nsub; ++cb) {
        const int col0 = n0 + cb * 32;
        if (col0 >= p.N || col0 > m0 + kBlockM - 1) break;  // outside the matrix, or wholly above the diagonal
        // ---- sum over ranks of a 128 x 32 block (512 groups of 8 elements, four per thread), staged in shared
        //      memory and stored row-wise where it lies on or below the diagonal
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int v = rt + kTpReducerThreads * i;
          const int r = v >> 2, c8 = (v & 3) * 8;
          const long long off = tile_off + static_cast<long long>(r) * p.bn + cb * 32 + c8;
          uint4 w;
          if (gave_up) {
            w = make_uint4(kTpPoison, kTpPoison, kTpPoison, kTpPoison);
          } else if (p.tp_partials_mc != nullptr) {
            w = multimem_ld_reduce_bf16x8(p.tp_partials_mc + off);
          } else {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int src = 0; src < p.tp_world; ++src) {
              const uint4 x = ld_relaxed_sys_16(p.tp_partials_peer[src] + off);
              const unsigned int xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                acc[2 * e] += __uint_as_float(xs[e] << 16);
                acc[2 * e + 1] += __uint_as_float(xs[e] & 0xFFFF0000u);
              }
            }
            unsigned int o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              o[e] = static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(acc[2 * e]))) |
                     (static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(acc[2 * e + 1]))) << 16);
            w = make_uint4(o[0], o[1], o[2], o[3]);
          }
          *reinterpret_cast<uint4*>(tp_stage + r * kTpStagePitch + c8) = w;
          const int row = m0 + r, col = col0 + c8;
          if (row < p.N && col <= row) {
            const long long at = static_cast<long long>(row) * p.tp_ld + col;
            if (col + 7 <= row) {  // col + 7 <= row < N: the whole group lies inside the lower triangle
              if (p.tp_gram_mc != nullptr) {
                multimem_st_16(p.tp_gram_mc + at, w);
              } else {
                for (int d = 0; d < p.tp_world; ++d) *reinterpret_cast<uint4*>(p.tp_gram[d] + at) = w;
              }
            } else {
              const unsigned int ws[4] = {w.x, w.y, w.z, w.w};
              for (int e = 0; e < 8; ++e) {
                if (col + e > row) break;
                const unsigned short h = static_cast<unsigned short>(ws[e >> 1] >> ((e & 1) * 16));
                for (int d = 0; d < p.tp_world; ++d) p.tp_gram[d][at + e] = h;
              }
            }
          }
        }
        named_barrier_sync(1, kTpReducerThreads);
        // ---- mirror image: element (row, col), col < row, also goes to (col, row); eight rows per group so that
        //      the stores run along the rows of the destination
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int v = rt + kTpReducerThreads * i;
          const int c = v >> 4, r8 = (v & 15) * 8;
          const int col = col0 + c, row = m0 + r8;
          if (col < p.N && row < p.N && col < row + 7) {  // some element of the group lies below the diagonal
            const long long at = static_cast<long long>(col) * p.tp_ld + row;
            const unsigned short* sp = tp_stage + r8 * kTpStagePitch + c;
            if (col < row && row + 7 < p.N) {
              uint4 w;
              w.x = sp[0] | (static_cast<unsigned int>(sp[kTpStagePitch]) << 16);
              w.y = sp[2 * kTpStagePitch] | (static_cast<unsigned int>(sp[3 * kTpStagePitch]) << 16);
              w.z = sp[4 * kTpStagePitch] | (static_cast<unsigned int>(sp[5 * kTpStagePitch]) << 16);
              w.w = sp[6 * kTpStagePitch] | (static_cast<unsigned int>(sp[7 * kTpStagePitch]) << 16);
              if (p.tp_gram_mc != nullptr) {
                multimem_st_16(p.tp_gram_mc + at, w);
              } else {
                for (int d = 0; d < p.tp_world; ++d) *reinterpret_cast<uint4*>(p.tp_gram[d] + at) = w;
              }
            } else {
              for (int e = 0; e < 8; ++e) {
                if (col < row + e && row + e < p.N)
                  for (int d = 0; d < p.tp_world; ++d) p.tp_gram[d][at + e] = sp[e * kTpStagePitch];
              }
            }
          }
        }
        named_barrier_sync(1, kTpReducerThreads);
      }
    }
    // every store of this rank's reducers is visible system-wide before the kernel (and the group barrier the host
    // enqueues behind it) completes
    __threadfence_system();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) {
    // Last CTA out re-arms the scheduler words for the next launch that is given this slot.
    __threadfence();
    if (atomicAdd(p.sched + 1, 1u) == gridDim.x - 1) {
      p.sched[0] = 0u;
      p.sched[1] = 0u;
      __threadfence();
    }
  }
}

// Copy the strict lower triangle of an N x N bf16 matrix onto its upper triangle (32 x 32 blocks through shared
// memory, coalesced on both sides).  blockIdx.x enumerates the blocks on and below the diagonal.
__global__ void __launch_bounds__(256) mirror_lower_kernel(unsigned short* __restrict__ a, int N, long long ld) {
  __shared__ unsigned short tile[32][33];
  const int t = blockIdx.x;  // block (bi, bj), bi >= bj, from the linear index t = bi (bi + 1) / 2 + bj
  int bi = static_cast<int>((sqrtf(8.0f * static_cast<float>(t) + 1.0f) - 1.0f) * 0.5f);
  while (bi * (bi + 1) / 2 > t) --bi;
  while ((bi + 1) * (bi + 2) / 2 <= t) ++bi;
  const int bj = t - bi * (bi + 1) / 2;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int r = ty; r < 32; r += 8) {
    const int row = bi * 32 + r, col = bj * 32 + tx;
    if (row < N && col < N) tile[r][tx] = a[static_cast<long long>(row) * ld + col];
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    // destination element (bj * 32 + r, bi * 32 + tx) takes source (bi * 32 + tx, bj * 32 + r)
    const int drow = bj * 32 + r, dcol = bi * 32 + tx;
    if (drow < N && dcol < N && dcol > drow) a[static_cast<long long>(drow) * ld + dcol] = tile[tx][r];
  }
}

// The same for N a multiple of 64 and 16-byte aligned rows: 64 x 64 blocks, 16-byte loads and stores on both sides
// (eight source rows are gathered from shared memory for every stored group).
__global__ void __launch_bounds__(256) mirror_lower64_kernel(unsigned short* __restrict__ a, int N, long long ld) {
  __shared__ unsigned short tile[64][64 + 2];
  const int t = blockIdx.x;
  int bi = static_cast<int>((sqrtf(8.0f * static_cast<float>(t) + 1.0f) - 1.0f) * 0.5f);
  while (bi * (bi + 1) / 2 > t) --bi;
  while ((bi + 1) * (bi + 2) / 2 <= t) ++bi;
  const int bj = t - bi * (bi + 1) / 2;
  for (int v = threadIdx.x; v < 512; v += 256) {  // source block (bi, bj), rows r, groups of eight columns
    const int r = v >> 3, c8 = (v & 7) * 8;
    const uint4 w = *reinterpret_cast<const uint4*>(a + static_cast<long long>(bi * 64 + r) * ld + bj * 64 + c8);
    const unsigned int ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      tile[r][c8 + 2 * e] = static_cast<unsigned short>(ws[e] & 0xFFFFu);
      tile[r][c8 + 2 * e + 1] = static_cast<unsigned short>(ws[e] >> 16);
    }
  }
  __syncthreads();
  for (int v = threadIdx.x; v < 512; v += 256) {  // destination block (bj, bi): row bj*64 + r takes source column r
    const int r = v >> 3, c8 = (v & 7) * 8;
    const int drow = bj * 64 + r, dcol = bi * 64 + c8;
    unsigned short* dst = a + static_cast<long long>(drow) * ld + dcol;
    if (dcol > drow) {  // the whole group lies above the diagonal
      uint4 w;
      w.x = tile[c8 + 0][r] | (static_cast<unsigned int>(tile[c8 + 1][r]) << 16);
      w.y = tile[c8 + 2][r] | (static_cast<unsigned int>(tile[c8 + 3][r]) << 16);
      w.z = tile[c8 + 4][r] | (static_cast<unsigned int>(tile[c8 + 5][r]) << 16);
      w.w = tile[c8 + 6][r] | (static_cast<unsigned int>(tile[c8 + 7][r]) << 16);
      *reinterpret_cast<uint4*>(dst) = w;
    } else if (dcol + 7 > drow) {  // diagonal block: element by element
      for (int e = 0; e < 8; ++e)
        if (dcol + e > drow) dst[e] = tile[c8 + e][r];
    }
  }
}

// Copy `nvec` 16-byte groups from local memory through a multicast address: every rank mapped by `dst_mc` receives
// them at the same offset.  Consecutive threads store consecutive groups, so a warp emits 512 contiguous bytes.
__global__ void __launch_bounds__(256) multicast_copy_kernel(const uint4* __restrict__ src, uint4* dst_mc,
                                                             long long nvec) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const uint4 v = src[i];
    multimem_st_16(dst_mc + i, v);
  }
}

}  // namespace eo
