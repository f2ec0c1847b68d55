// Second half of the tensor-parallel Gram all-reduce: the owner of a tile waits for the partial tiles that the
// SYRK epilogues of all ranks pushed into its inbox, sums them in fp32, rounds to bf16 once and stores the tile
// and its mirror image into the Gram matrix of every rank (plain stores to local and peer memory).
#pragma once

#include <cuda_bf16.h>

#include "gemm_sm100.cuh"

namespace eo {

constexpr int kTpReduceThreads = 256;

struct TpReduceParams {
  int N;          // Gram matrix is N x N
  int bn;         // tile width used by the pushing kernel
  int world, rank;
  unsigned int seq;
  int tiles_m, tiles_n, total_tiles;
  const unsigned short* inbox;  // local: [world][slots][128][bn] bf16
  const unsigned int* flags;    // local: [world][slots]
  int slots;
  unsigned short* gram[8];      // per rank: N x ld bf16
  long long ld;
  unsigned int* status;
  int mirror;  // 1: also store the mirror image of each tile into every rank's matrix; 0: lower triangle only
               //    (every rank then mirrors its own copy locally, which halves the bytes that cross NVLink)
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kTpReduceThreads) tp_gram_reduce_kernel(const TpReduceParams q) {
  extern __shared__ unsigned short tile_smem[];  // [128][bn + 8] bf16, padded rows against bank conflicts
  __shared__ int give_up;
  const int pitch = q.bn + 8;
  GemmParams dp;  // only the fields decode_tile reads
  dp.tri = 1;
  dp.bn = q.bn;
  dp.tiles_m = q.tiles_m;
  dp.tiles_n = q.tiles_n;
  dp.tiles_per_batch = q.total_tiles;
  const long long tile_elems = static_cast<long long>(kBlockM) * q.bn;

  for (int slot = blockIdx.x; slot < q.slots; slot += gridDim.x) {
    const int t = slot * q.world + q.rank;
    if (t >= q.total_tiles) break;
    // Wait (bounded) for every rank's partial of this tile.
    if (threadIdx.x == 0) give_up = 0;
    __syncthreads();
    if (threadIdx.x < q.world) {
      const unsigned int* f = q.flags + static_cast<long long>(threadIdx.x) * q.slots + slot;
      const long long t0 = clock64();
      while (static_cast<int>(ld_acquire_sys(f) - q.seq) < 0) {
        if (clock64() - t0 > kWaitBudgetCycles) {
          give_up = 1;
          if (q.status != nullptr) atomicCAS(q.status, 0u, kStatusTimeoutPeer);
          break;
        }
      }
    }
    __syncthreads();
    if (give_up) return;

    int b, ti, tj;
    decode_tile(dp, t, b, ti, tj);
    const int m0 = ti * kBlockM, n0 = tj * q.bn;

    // Sum the partials: 8 bf16 (16 bytes) per thread and step.
    const int vec_per_row = q.bn / 8;
    for (int v = threadIdx.x; v < kBlockM * vec_per_row; v += kTpReduceThreads) {
      const int r = v / vec_per_row, c8 = (v - r * vec_per_row) * 8;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int src = 0; src < q.world; ++src) {
        const unsigned short* part =
            q.inbox + (static_cast<long long>(src) * q.slots + slot) * tile_elems + static_cast<long long>(r) * q.bn + c8;
        const uint4 w = *reinterpret_cast<const uint4*>(part);
        const unsigned int ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[2 * e] += __uint_as_float(ws[e] << 16);
          acc[2 * e + 1] += __uint_as_float(ws[e] & 0xFFFF0000u);
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) tile_smem[r * pitch + c8 + e] = __bfloat16_as_ushort(__float2bfloat16_rn(acc[e]));
    }
    __syncthreads();

    // Direct part: elements with col <= row, rows of the tile are contiguous in memory.
    for (int v = threadIdx.x; v < kBlockM * vec_per_row; v += kTpReduceThreads) {
      const int r = v / vec_per_row, c8 = (v - r * vec_per_row) * 8;
      const int row = m0 + r, col = n0 + c8;
      if (row >= q.N || col >= q.N || col > row) continue;
      const bool full = (col + 7 <= row) && (col + 7 < q.N);
      for (int d = 0; d < q.world; ++d) {
        unsigned short* dst = q.gram[d] + static_cast<long long>(row) * q.ld + col;
        if (full) {
          uint4 w;
          const unsigned short* s = &tile_smem[r * pitch + c8];
          w.x = s[0] | (static_cast<unsigned int>(s[1]) << 16);
          w.y = s[2] | (static_cast<unsigned int>(s[3]) << 16);
          w.z = s[4] | (static_cast<unsigned int>(s[5]) << 16);
          w.w = s[6] | (static_cast<unsigned int>(s[7]) << 16);
          *reinterpret_cast<uint4*>(dst) = w;
        } else {
          for (int e = 0; e < 8; ++e)
            if (col + e <= row && col + e < q.N) dst[e] = tile_smem[r * pitch + c8 + e];
        }
      }
    }
    // Mirrored part: element (row, col) with col < row goes to (col, row); rows of the tile run along memory.
    const int rvec = kBlockM / 8;
    for (int v = threadIdx.x; q.mirror && v < q.bn * rvec; v += kTpReduceThreads) {
      const int c = v / rvec, r8 = (v - c * rvec) * 8;
      const int col = n0 + c, row = m0 + r8;
      if (col >= q.N || row >= q.N || col >= row + 7) continue;  // nothing below the diagonal in this group
      const bool full = (col < row) && (row + 7 < q.N);
      for (int d = 0; d < q.world; ++d) {
        unsigned short* dst = q.gram[d] + static_cast<long long>(col) * q.ld + row;
        if (full) {
          uint4 w;
          w.x = tile_smem[(r8 + 0) * pitch + c] | (static_cast<unsigned int>(tile_smem[(r8 + 1) * pitch + c]) << 16);
          w.y = tile_smem[(r8 + 2) * pitch + c] | (static_cast<unsigned int>(tile_smem[(r8 + 3) * pitch + c]) << 16);
          w.z = tile_smem[(r8 + 4) * pitch + c] | (static_cast<unsigned int>(tile_smem[(r8 + 5) * pitch + c]) << 16);
          w.w = tile_smem[(r8 + 6) * pitch + c] | (static_cast<unsigned int>(tile_smem[(r8 + 7) * pitch + c]) << 16);
          *reinterpret_cast<uint4*>(dst) = w;
        } else {
          for (int e = 0; e < 8; ++e)
            if (col < row + e && row + e < q.N) dst[e] = tile_smem[(r8 + e) * pitch + c];
        }
      }
    }
    __syncthreads();
  }
}

// Copy the strict lower triangle of an N x N bf16 matrix onto its upper triangle (32 x 32 blocks through shared
// memory, coalesced on both sides).  blockIdx.x enumerates the blocks on and below the diagonal.
__global__ void __launch_bounds__(256) mirror_lower_kernel(unsigned short* __restrict__ a, int N, long long ld) {
  __shared__ unsigned short tile[32][33];
  // block (bi, bj), bi >= bj, from the linear index t = bi (bi + 1) / 2 + bj
  const int t = blockIdx.x;
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

}  // namespace eo
