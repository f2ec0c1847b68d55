// The GEMM / SYRK of gemm_sm100.cuh on CTA pairs: tcgen05.mma with cta_group::2.
//
// Two CTAs of one TPC (a cluster of two) share every 256 x 256 output tile.  CTA r of the pair holds rows
// 128 r .. 128 r + 127 of the tile: it loads those rows of A and rows 128 r .. of the tile's B operand (its half of
// N) into its own shared memory, and the accumulator for its rows lives in its own TMEM.  One thread of the leader
// CTA (rank 0) issues the MMAs for both: M = 256 across the pair, the B halves are read from both CTAs' shared
// memory by the hardware.  Compared with the 256-row mode of the single-CTA kernel this keeps its operand traffic per
// FLOP (32 KiB per CTA, k-step and 128 x 256 x 64 block) but needs only 256 TMEM columns per tile, so two
// accumulators alternate and the epilogue of tile t overlaps the main loop of tile t + 1, and each SM reads only
// half of B from its shared memory; stages are 32 KiB, so the ring is six deep.
//
// Cross-CTA protocol (all barriers live at the same offsets in both CTAs; "L:" = the leader's copy is used):
//   full[s]      L: operand stage s loaded.  The leader's producer expects 64 KiB; both CTAs' TMA loads count their
//                   bytes on the leader's barrier (cta_group::2 loads, no multicast).
//   empty[s]        stage s free again; the leader's MMA thread commits to its own and to the peer's barrier.
//   acc_full[a]     accumulator a complete; committed to both CTAs likewise.
//   acc_empty[a] L: accumulator a drained; the epilogue warps of both CTAs arrive (the peer's remotely).
//   tq_full[q]      tile index q published; the leader's producer takes tiles from the global counter, writes the
//                   index into both CTAs' queues and arrives on both barriers.
//   tq_empty[q]  L: queue slot q consumed by every role of both CTAs.
// A queue entry is the work-item index, -1 for "no more work", with bit 30 set when the item belongs to a tile on the
// diagonal of a SYRK, whose A rows are the CTA's rows of the B operand and are not loaded a second time.
// Every wait is bounded; a wait that runs out records a code in the status word and the role leaves its loop.
//
// Split tail.  Equal tiles run in rounds of one per pair, and the last round of a launch is usually far from full
// (528 SYRK tiles of an 8192-row Gram matrix on 74 pairs: 7.14 rounds of work take 8).  The launcher can therefore
// cut the K range of the last `tiles mod pairs` tiles of every matrix into `split_s` pieces, which are scheduled as
// work items of their own.  A piece writes its fp32 accumulator to a workspace; per epilogue warp a counter is
// raised, and the warp that raises it last adds the pieces up in piece order (so the result does not depend on who
// finishes last) and runs the normal epilogue.  Nothing waits for anything.  Which tiles are split depends only on
// M, N, K and the triangular flag, never on the batch size, so a batched launch and per-matrix launches agree bit
// for bit.
#pragma once

#include "gemm_sm100.cuh"

namespace eo {

constexpr int kPairStages = 6;
constexpr int kPairStageBytes = 2 * kStageABytes;  // A half (128 x 64 bf16) + B half (128 x 64 bf16)
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 512 + 1024;
constexpr uint32_t kStatusPair = 0x60u;
constexpr int kPairDiagBit = 1 << 30;
constexpr int kSplitHalfFloats = kBlockM * kMaxBlockN;  // one CTA's half of one piece's accumulator (128 KiB)

// One unit of work: a whole tile, or one K piece of a tile of the split tail.
struct PairWork {
  int tile;   // tile index as decode_pair_tile() numbers them (all matrices of the batch)
  int kb0;    // first k-block
  int kb1;    // one past the last k-block
  int slot;   // index of the split tile among all split tiles of the launch, or -1 for a whole tile
  int piece;  // which piece of the split tile
};

// Tile order of the pair kernel (256 x 256 tiles).  The tiles in flight at one time (one per pair, 74 on a B200)
// should touch as few row blocks of the operands as possible: they stream through K together, so an operand block
// shared by several of them comes from DRAM once.  General products: groups of pair_group_m row blocks, column by
// column inside a group.  Triangular products: bands of pair_band tile columns, row by row inside a band, so that
// 74 consecutive tiles form a block of about 9 x 8 tiles instead of two whole tile columns.
__host__ __device__ __forceinline__ void decode_pair_tile(const GemmParams& p, int t, int& b, int& ti, int& tj) {
  b = t / p.tiles_per_batch;
  int r = t - b * p.tiles_per_batch;
  if (p.tri && p.pair_band > 0) {
    const int g = p.pair_band, T = p.tiles_m;
    ti = tj = 0;
    for (int c0 = 0; c0 < T; c0 += g) {
      const int rows = T - c0;
      const int w = rows < g ? rows : g;
      const int tri_cnt = w * (w + 1) / 2;
      const int cnt = tri_cnt + (rows - w) * w;
      if (r < cnt) {
        if (r < tri_cnt) {
          int a = 0;
          while ((a + 1) * (a + 2) / 2 <= r) ++a;
          ti = c0 + a;
          tj = c0 + r - a * (a + 1) / 2;
        } else {
          const int r2 = r - tri_cnt;
          ti = c0 + w + r2 / w;
          tj = c0 + r2 % w;
        }
        return;
      }
      r -= cnt;
    }
  } else if (p.tri) {
    decode_tile(p, t, b, ti, tj, 2 * kBlockM);
  } else {
    const int gm = p.pair_group_m;
    const int per_group = gm * p.tiles_n;
    const int g = r / per_group;
    const int first = g * gm;
    const int rows = min(gm, p.tiles_m - first);
    const int w = r - g * per_group;
    ti = first + (w % rows);
    tj = w / rows;
  }
}

__host__ __device__ __forceinline__ PairWork decode_pair_work(const GemmParams& p, int w, int num_kb) {
  PairWork k;
  const int b = w / p.split_items_per_batch;
  const int r = w - b * p.split_items_per_batch;
  if (r < p.split_first) {
    k.tile = b * p.tiles_per_batch + r;
    k.kb0 = 0;
    k.kb1 = num_kb;
    k.slot = -1;
    k.piece = 0;
  } else {
    const int q = r - p.split_first;
    const int rt = q / p.split_s;
    k.piece = q - rt * p.split_s;
    k.tile = b * p.tiles_per_batch + p.split_first + rt;
    k.kb0 = static_cast<int>(static_cast<long long>(k.piece) * num_kb / p.split_s);
    k.kb1 = static_cast<int>(static_cast<long long>(k.piece + 1) * num_kb / p.split_s);
    k.slot = b * (p.tiles_per_batch - p.split_first) + rt;
  }
  return k;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
    eo_gemm_pair_kernel(const __grid_constant__ GemmMaps maps, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kPairStages * kPairStageBytes);
  uint64_t* full_bar = bars;                           // [kPairStages]
  uint64_t* empty_bar = full_bar + kPairStages;        // [kPairStages]
  uint64_t* acc_full_bar = empty_bar + kPairStages;    // [2]
  uint64_t* acc_empty_bar = acc_full_bar + 2;          // [2]
  uint64_t* tq_full_bar = acc_empty_bar + 2;           // [kTileQueue]
  uint64_t* tq_empty_bar = tq_full_bar + kTileQueue;   // [kTileQueue]
  int* tile_queue = reinterpret_cast<int*>(tq_empty_bar + kTileQueue);  // [kTileQueue]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tile_queue + kTileQueue);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: leader (issues the MMAs, owns the shared barriers), 1: peer
  const bool leader = rank == 0;
  const uint32_t peer = rank ^ 1u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full_bar[s], 1);
      mbar_init(&acc_empty_bar[s], 2 * kEpilogueWarps);  // the epilogue warps of both CTAs
    }
    for (int s = 0; s < kTileQueue; ++s) {
      mbar_init(&tq_full_bar[s], 1);
      // leader: MMA thread + epilogue warps; peer: producer + epilogue warps
      mbar_init(&tq_empty_bar[s], 2 * (1 + kEpilogueWarps));
    }
    mbar_init_fence();
    tma_prefetch_desc(&maps.a[0]);
    tma_prefetch_desc(&maps.b[0]);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers are initialised and TMEM is allocated before anything crosses over
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  constexpr int bk = kBlockK;
  constexpr int bm = 2 * kBlockM;  // pair tile height
  const int num_kb = (p.K + bk - 1) / bk;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int tq = 0;
      uint32_t tq_phase = 0;
      bool ok = true;
      const uint64_t pol_a = l2_policy(p.pair_hint_a), pol_b = l2_policy(p.pair_hint_b);
      auto load = [](void* dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int hint, uint64_t pol) {
        if (hint != 0)
          tma_load_3d_pair_hint(dst, map, bar, c0, c1, c2, pol);
        else
          tma_load_3d_pair(dst, map, bar, c0, c1, c2);
      };
      while (ok) {
        int t;
        if (leader) {
          t = static_cast<int>(atomicAdd(p.sched, 1u));
          if (t >= p.total_tiles) t = -1;
          int entry = t;  // bit 30: the tile lies on the diagonal of a SYRK and A is read from the B operand
          if (t >= 0 && p.same_ab) {
            int b, ti, tj;
            decode_pair_tile(p, decode_pair_work(p, t, num_kb).tile, b, ti, tj);
            if (ti * bm == tj * p.bn) entry |= kPairDiagBit;
          }
          if (!mbar_wait_cluster(&tq_empty_bar[tq], tq_phase ^ 1u)) {
            report(p, kStatusPair + 1u);
            break;
          }
          tile_queue[tq] = entry;
          st_cluster_u32(mapa_u32(smem_u32(&tile_queue[tq]), peer), static_cast<uint32_t>(entry));
          mbar_arrive(&tq_full_bar[tq]);
          mbar_arrive_cluster(mapa_u32(smem_u32(&tq_full_bar[tq]), peer));
        } else {
          if (!mbar_wait_cluster(&tq_full_bar[tq], tq_phase)) {
            report(p, kStatusPair + 2u);
            break;
          }
          t = tile_queue[tq];
          if (t >= 0) t &= ~kPairDiagBit;
          mbar_arrive_cluster(mapa_u32(smem_u32(&tq_empty_bar[tq]), 0u));
        }
        if (++tq == kTileQueue) {
          tq = 0;
          tq_phase ^= 1u;
        }
        if (t < 0) break;
        const PairWork wk = decode_pair_work(p, t, num_kb);
        int b, ti, tj;
        decode_pair_tile(p, wk.tile, b, ti, tj);
        const int m0 = ti * bm + static_cast<int>(rank) * kBlockM;   // this CTA's rows of A
        const int n0 = tj * p.bn + static_cast<int>(rank) * kBlockM;  // this CTA's half of B (rows of op(B))
        // SYRK tile on the diagonal: this CTA's rows of A are its rows of the B operand; load them once.
        const bool a_in_b = p.same_ab && m0 == n0;
        for (int kb = wk.kb0; kb < wk.kb1; ++kb) {
          if (!mbar_wait_cluster(&empty_bar[stage], phase ^ 1u)) {
            report(p, kStatusPair + 3u);
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kPairStageBytes;
          uint8_t* sb = sa + kStageABytes;
          const uint32_t fb = mapa_u32(smem_u32(&full_bar[stage]), 0u);  // the leader's barrier
          if (leader)  // both CTAs' bytes
            mbar_expect_tx(&full_bar[stage], a_in_b ? 2u * kStageABytes : 2u * kPairStageBytes);
          const int k0 = kb * bk;
          if (a_in_b) {
            // nothing to load for A
          } else if (!p.a_mn) {
            load(sa, &maps.a[0], fb, k0, m0, b, p.pair_hint_a, pol_a);  // box {bk, 128, 1}
          } else {
            for (int q = 0; q < kBlockM / bk; ++q)  // box {bk (M), bk (K), 1}
              load(sa + q * bk * kRowBytes, &maps.a[0], fb, m0 + q * bk, k0, b, p.pair_hint_a, pol_a);
          }
          if (!p.b_mn) {
            load(sb, &maps.b[0], fb, k0, n0, b, p.pair_hint_b, pol_b);
          } else {
            for (int q = 0; q < kBlockM / bk; ++q)
              load(sb + q * bk * kRowBytes, &maps.b[0], fb, n0 + q * bk, k0, b, p.pair_hint_b, pol_b);
          }
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (leader && elect_one()) {
      const uint32_t idesc = make_idesc(1u, p.a_mn != 0, p.b_mn != 0, bm, p.bn);
      int stage = 0;
      uint32_t phase = 0;
      int ab = 0;
      uint32_t aphase = 0;
      int tq = 0;
      uint32_t tq_phase = 0;
      bool ok = true;
      while (ok) {
        if (!mbar_wait(&tq_full_bar[tq], tq_phase)) {
          report(p, kStatusPair + 4u);
          break;
        }
        const int entry = tile_queue[tq];
        mbar_arrive(&tq_empty_bar[tq]);
        if (++tq == kTileQueue) {
          tq = 0;
          tq_phase ^= 1u;
        }
        if (entry < 0) break;
        const bool a_in_b = (entry & kPairDiagBit) != 0;
        const PairWork wk = decode_pair_work(p, entry & ~kPairDiagBit, num_kb);
        if (!mbar_wait_cluster(&acc_empty_bar[ab], aphase ^ 1u)) {
          report(p, kStatusPair + 5u);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(ab * kMaxBlockN);
        for (int kb = wk.kb0; kb < wk.kb1; ++kb) {
          if (!mbar_wait_cluster(&full_bar[stage], phase)) {
            report(p, kStatusPair + 6u);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sb = smem_u32(smem + stage * kPairStageBytes) + static_cast<uint32_t>(kStageABytes);
          const uint32_t sa = a_in_b ? sb : sb - static_cast<uint32_t>(kStageABytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = make_smem_desc(sa + k * p.adv_a, p.lbo_a, p.sbo_a);
            const uint64_t db = make_smem_desc(sb + k * p.adv_b, p.lbo_b, p.sbo_b);
            umma_f16_pair(tmem_d, da, db, idesc, ((kb - wk.kb0) | k) != 0 ? 1u : 0u);
          }
          // the stage is free in both CTAs once these MMAs have read it
          umma_commit_pair(smem_u32(&empty_bar[stage]));
          umma_commit_pair(mapa_u32(smem_u32(&empty_bar[stage]), peer));
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair(smem_u32(&acc_full_bar[ab]));
        umma_commit_pair(mapa_u32(smem_u32(&acc_full_bar[ab]), peer));
        if (++ab == 2) {
          ab = 0;
          aphase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;
    constexpr int kChunkStep = kEpilogueWarps / 4;
    int ab = 0;
    uint32_t aphase = 0;
    int tq = 0;
    uint32_t tq_phase = 0;
    while (true) {
      if (!mbar_wait_cluster(&tq_full_bar[tq], tq_phase)) {
        report(p, kStatusPair + 7u);
        break;
      }
      int t = tile_queue[tq];
      if (t >= 0) t &= ~kPairDiagBit;
      __syncwarp();
      if (lane == 0) {
        if (leader)
          mbar_arrive(&tq_empty_bar[tq]);
        else
          mbar_arrive_cluster(mapa_u32(smem_u32(&tq_empty_bar[tq]), 0u));
      }
      if (++tq == kTileQueue) {
        tq = 0;
        tq_phase ^= 1u;
      }
      if (t < 0) break;
      const PairWork wk = decode_pair_work(p, t, num_kb);
      int b, ti, tj;
      decode_pair_tile(p, wk.tile, b, ti, tj);
      const int m0 = ti * bm + static_cast<int>(rank) * kBlockM;
      const int n0 = tj * p.bn;
      const int row = m0 + quarter * 32 + lane;
      const int warp_last_row = m0 + quarter * 32 + 31;
      const long long batch_c = static_cast<long long>(b) * p.strideC;
      const long long batch_d = static_cast<long long>(b) * p.strideD;
      const int nchunks = p.bn / 32;
      float alpha = p.alpha, sum_scale = 1.0f;
      if (p.dev_scale != nullptr) {
        if (p.dev_scale_mode == 1)
          alpha *= __ldg(p.dev_scale + 2 * b);
        else
          sum_scale = __ldg(p.dev_scale + 2 * b + 1);
      }
      if (!mbar_wait_cluster(&acc_full_bar[ab], aphase)) {
        report(p, kStatusPair + 8u);
        break;
      }
      tc_fence_after();
      // a piece's accumulator goes to the workspace as it is: [chunk][row of this CTA's half][32 columns] fp32
      float* const ws_tile =
          wk.slot < 0 ? nullptr
                      : p.split_ws + (static_cast<size_t>(wk.slot) * p.split_s * 2 + rank) * kSplitHalfFloats +
                            static_cast<size_t>(quarter * 32 + lane) * 32;
      constexpr size_t kPieceStride = 2 * static_cast<size_t>(kSplitHalfFloats);
      for (int c = group; c < nchunks; c += kChunkStep) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;
        if (p.tri && col0 > warp_last_row) break;
        uint32_t acc[32];
        __syncwarp();
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                          static_cast<uint32_t>(ab * kMaxBlockN + c * 32),
                      acc);
        tmem_ld_wait();
        if (wk.slot < 0) {
          epilogue_chunk(p, acc, batch_c, batch_d, row, col0, alpha, sum_scale);
        } else {
          float4* dst = reinterpret_cast<float4*>(ws_tile + wk.piece * kPieceStride + static_cast<size_t>(c) * kBlockM * 32);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            __stcg(dst + j, make_float4(__uint_as_float(acc[4 * j]), __uint_as_float(acc[4 * j + 1]),
                                        __uint_as_float(acc[4 * j + 2]), __uint_as_float(acc[4 * j + 3])));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader)
          mbar_arrive(&acc_empty_bar[ab]);
        else
          mbar_arrive_cluster(mapa_u32(smem_u32(&acc_empty_bar[ab]), 0u));
      }
      if (wk.slot >= 0) {
        // The warp whose arrival completes the count owns the sum: pieces are added in piece order, whoever is last.
        __threadfence();
        __syncwarp();
        unsigned int* cnt = p.split_cnt + (static_cast<size_t>(wk.slot) * 2 + rank) * kEpilogueWarps + (warp - 2);
        unsigned int old = 0;
        if (lane == 0) old = atomicAdd(cnt, 1u);
        old = __shfl_sync(0xffffffffu, old, 0);
        if (old == static_cast<unsigned int>(p.split_s - 1)) {
          __threadfence();
          for (int c = group; c < nchunks; c += kChunkStep) {
            const int col0 = n0 + c * 32;
            if (col0 >= p.N) break;
            if (p.tri && col0 > warp_last_row) break;
            uint32_t acc[32];
            const float* src = ws_tile + static_cast<size_t>(c) * kBlockM * 32;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 v = __ldcg(reinterpret_cast<const float4*>(src) + j);
              acc[4 * j] = __float_as_uint(v.x);
              acc[4 * j + 1] = __float_as_uint(v.y);
              acc[4 * j + 2] = __float_as_uint(v.z);
              acc[4 * j + 3] = __float_as_uint(v.w);
            }
            for (int piece = 1; piece < p.split_s; ++piece) {
              const float4* sp = reinterpret_cast<const float4*>(src + piece * kPieceStride);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 v = __ldcg(sp + j);
                acc[4 * j] = __float_as_uint(__uint_as_float(acc[4 * j]) + v.x);
                acc[4 * j + 1] = __float_as_uint(__uint_as_float(acc[4 * j + 1]) + v.y);
                acc[4 * j + 2] = __float_as_uint(__uint_as_float(acc[4 * j + 2]) + v.z);
                acc[4 * j + 3] = __float_as_uint(__uint_as_float(acc[4 * j + 3]) + v.w);
              }
            }
            epilogue_chunk(p, acc, batch_c, batch_d, row, col0, alpha, sum_scale);
          }
          if (lane == 0) *cnt = 0u;  // ready for the next launch on this stream
        }
      }
      if (++ab == 2) {
        ab = 0;
        aphase ^= 1u;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nothing of this CTA is addressed by its partner any more
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.sched + 1, 1u) == gridDim.x - 1) {
      p.sched[0] = 0u;
      p.sched[1] = 0u;
      __threadfence();
    }
  }
}

}  // namespace eo
