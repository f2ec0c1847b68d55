// Whole Newton-Schulz loop for small matrices (m <= 128 rows, wide: m <= n) in ONE persistent kernel.
//
// Per-head / split-QKV blocks are 128 x n: their Gram matrix is a single 128 x 128 tile, so A = X X^T, A^2 and
// S = b A + c A^2 never have to leave the SM.  A CTA takes one matrix at a time (dynamic counter) and runs all
// iterations on it:
//
//   Gram   : first iteration only as a pass of its own: X streamed through a shared-memory ring in 128 x 64
//            boxes (K-major), accumulated in TMEM; the epilogue rounds A to bf16 and writes it into shared
//            memory in the 128B-swizzled operand layout
//   A^2    : tcgen05.mma on the shared-memory copy of A (skipped when c == 0); epilogue writes S likewise
//   S X    : X streamed again, 128 x 128 output tiles (the same boxes now act as MN-major B operands, two
//            N = 64 MMAs per k-step); the epilogue takes the a X term from the boxes still sitting in the ring
//            and overwrites them in place with the new iterate.  While a finished tile is still in the ring
//            it is used twice: a store warp sends it out with TMA stores, and the MMA warp accumulates its
//            contribution to the NEXT iteration's Gram matrix (the boxes are K-major operands of X' X'^T).
//
// so the first iteration reads a matrix twice and every iteration reads it once and writes it once, with no
// launch boundary, no global A / S traffic and no per-launch tail: 11 passes over the matrix for five steps
// instead of 15.  The products are accumulated in the same order as by separate passes, so results are
// bit-identical to the general kernels.  Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2..9 epilogue,
// warp 10 TMA stores.  Every wait is bounded; a wait that runs out records a code in the status word and the
// CTA drains.
#pragma once

#include <cuda_bf16.h>

#include "sm100_ptx.cuh"

namespace eo {

constexpr int kSmallUnitBytes = 128 * 128;  // one TMA box: 128 rows x 64 bf16
constexpr int kSmallUnits = 10;             // ring depth
constexpr int kSmallABytes = 2 * kSmallUnitBytes;  // 128 x 128 bf16 operand (two 64-column atoms)
constexpr int kSmallThreads = 64 + 32 * 8 + 32;
constexpr int kSmallSmemBytes = kSmallUnits * kSmallUnitBytes + 2 * kSmallABytes + 1024 + 1024;
constexpr int kSmallMaxSteps = 16;
constexpr int kSmallAcc = 3;       // TMEM accumulators of 128 columns each, used round-robin by the S X tiles
constexpr int kSmallAccG = 3;      // index of the fourth accumulator: Gram matrix, then A^2, of one iteration
constexpr int kSmallGramLag = 2;   // the Gram MMAs of an S X tile are issued this many tiles behind its S X MMAs
constexpr int kSmallTileN = 128;   // output tile width of the S X product
constexpr uint32_t kStatusSmall = 0x50u;

struct SmallParams {
  int batch, m, n;
  int steps;
  float abc[3 * kSmallMaxSteps];
  unsigned short* buf[2];  // ping-pong iterates: buf[0] holds the input; iteration i reads buf[i & 1]
  long long ld[2], stride[2];  // their layouts (elements)
  void* out;               // result of the last iteration
  long long ldo, strideo;
  int out_fp32;
  unsigned int* sched;   // {next matrix, finished CTAs}
  unsigned int* status;
  // Deferred Frobenius normalisation: when set, buf[0] holds the un-normalised bf16 input and dev_scale[2 b],
  // dev_scale[2 b + 1] = 1 / norm_b^2, 1 / norm_b; the first Gram epilogue and the first update epilogue apply them.
  const float* dev_scale;
};

struct SmallMaps {
  CUtensorMap x[2];  // over buf[0] and buf[1]: dims {n, m, batch}, box {64, 128, 1}, 128B swizzle
};

__device__ __forceinline__ uint32_t swz_offset(int row, int col) {
  // byte offset of element (row, col) of a 128 x 128 bf16 operand stored as two 64-column, 128B-swizzled atoms
  const int atom = col >> 6, unit = (col & 63) >> 3;
  return static_cast<uint32_t>(atom * kSmallUnitBytes + row * 128 + (((unit ^ (row & 7)) << 4)) + ((col & 7) << 1));
}

__global__ void __launch_bounds__(kSmallThreads, 1)
    eo_ns_small_kernel(const __grid_constant__ SmallMaps maps, const SmallParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* a_buf = smem + kSmallUnits * kSmallUnitBytes;
  uint8_t* s_buf = a_buf + kSmallABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_buf + kSmallABytes);
  uint64_t* full_bar = bars;                           // [kSmallUnits] box loaded
  uint64_t* empty_bar = full_bar + kSmallUnits;        // [kSmallUnits] box free again (two arrivals, see below)
  uint64_t* st_ready_bar = empty_bar + kSmallUnits;    // [kSmallUnits] by first box of a tile: new iterate written
  uint64_t* acc_full_bar = st_ready_bar + kSmallUnits;     // [kSmallAcc + 1]
  uint64_t* acc_empty_bar = acc_full_bar + kSmallAcc + 1;  // [kSmallAcc + 1]
  uint64_t* a_ready_bar = acc_empty_bar + kSmallAcc + 1;   // A written to shared memory
  uint64_t* s_ready_bar = a_ready_bar + 1;             // S written to shared memory
  uint64_t* x_ready_bar = s_ready_bar + 1;             // every tile of the next iterate written to global memory
  uint64_t* mq_full_bar = x_ready_bar + 1;             // [2] matrix-index queue
  uint64_t* mq_empty_bar = mq_full_bar + 2;            // [2]
  int* mat_queue = reinterpret_cast<int*>(mq_empty_bar + 2);  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mat_queue + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nk = (p.n + 63) / 64;      // Gram k-blocks
  const int nt = (p.n + kSmallTileN - 1) / kSmallTileN;  // output tiles of the S X product

  // A box is handed back to the producer by two arrivals on its `empty` barrier.  Gram pass of the first
  // iteration: both from the MMA thread (one at once, one when its MMAs have read the box).  S X pass: one from
  // the store thread (TMA store has read the box) and one from the MMA thread (the Gram MMAs of the next iteration
  // have read it); in the last iteration, where neither happens, the store thread arrives twice.
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSmallUnits; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 2);
      mbar_init(&st_ready_bar[s], 8);
    }
    for (int s = 0; s < kSmallAcc + 1; ++s) {
      mbar_init(&acc_full_bar[s], 1);
      mbar_init(&acc_empty_bar[s], 8);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&mq_full_bar[s], 1);
      mbar_init(&mq_empty_bar[s], 10);  // MMA thread, eight epilogue warps, store thread
    }
    mbar_init(a_ready_bar, 8);
    mbar_init(s_ready_bar, 8);
    mbar_init(x_ready_bar, 1);
    mbar_init_fence();
    tma_prefetch_desc(&maps.x[0]);
    tma_prefetch_desc(&maps.x[1]);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto fail = [&](uint32_t code) {
    if (p.status != nullptr) atomicCAS(p.status, 0u, kStatusSmall + code);
  };
  auto next_unit = [](int u) { return (u + 1 == kSmallUnits) ? 0 : u + 1; };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (elect_one()) {
      int unit = 0;
      uint32_t uphase = 0;
      int mq = 0;
      uint32_t mq_phase = 0, x_phase = 0;
      bool ok = true;
      auto load_unit = [&](const CUtensorMap* map, int col, int b) -> bool {
        if (!mbar_wait(&empty_bar[unit], uphase ^ 1u)) {
          fail(1);
          return false;
        }
        mbar_expect_tx(&full_bar[unit], kSmallUnitBytes);
        tma_load_3d(ring + unit * kSmallUnitBytes, map, &full_bar[unit], col, 0, b);
        if (++unit == kSmallUnits) {
          unit = 0;
          uphase ^= 1u;
        }
        return true;
      };
      while (ok) {
        int b = static_cast<int>(atomicAdd(p.sched, 1u));
        if (b >= p.batch) b = -1;
        if (!mbar_wait(&mq_empty_bar[mq], mq_phase ^ 1u)) {
          fail(2);
          break;
        }
        mat_queue[mq] = b;
        mbar_arrive(&mq_full_bar[mq]);
        if (++mq == 2) {
          mq = 0;
          mq_phase ^= 1u;
        }
        if (b < 0) break;
        for (int it = 0; it < p.steps && ok; ++it) {
          const CUtensorMap* map = &maps.x[it & 1];
          if (it > 0) {
            // the previous iteration's output must be complete in global memory before it is read back
            if (!mbar_wait(x_ready_bar, x_phase)) {
              fail(3);
              ok = false;
              break;
            }
            x_phase ^= 1u;
          } else {
            for (int kb = 0; kb < nk && ok; ++kb) ok = load_unit(map, kb * 64, b);  // Gram pass of the input
          }
          for (int t = 0; t < nt && ok; ++t)
            for (int q = 0; q < 2 && ok; ++q) ok = load_unit(map, t * kSmallTileN + q * 64, b);
        }
        // The store thread also arrives on x_ready after the last iteration: consume that phase.
        if (ok && p.steps > 0) {
          if (!mbar_wait(x_ready_bar, x_phase)) {
            fail(3);
            break;
          }
          x_phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc_gram = make_idesc(1u, false, false, 128, 128);  // K-major x K-major
      const uint32_t idesc_sx = make_idesc(1u, false, true, 128, 64);      // S K-major, X box MN-major
      const uint32_t a_addr = smem_u32(a_buf), s_addr = smem_u32(s_buf);
      const uint32_t acc_g = tmem_base + static_cast<uint32_t>(kSmallAccG * 128);
      int unit = 0;
      uint32_t uphase = 0;
      int ab = 0;
      uint32_t aphase = 0, g_phase = 0, a_phase = 0, s_phase = 0;
      uint32_t st_bits = 0;  // phase parity of every st_ready barrier, as seen by this thread
      int mq = 0;
      uint32_t mq_phase = 0;
      bool ok = true;
      auto wait_unit = [&]() -> bool {
        if (!mbar_wait(&full_bar[unit], uphase)) {
          fail(4);
          return false;
        }
        tc_fence_after();
        return true;
      };
      auto advance_unit = [&]() {
        if (++unit == kSmallUnits) {
          unit = 0;
          uphase ^= 1u;
        }
      };
      auto wait_acc_g = [&]() -> bool {  // the epilogue has drained the previous contents of the Gram accumulator
        if (!mbar_wait(&acc_empty_bar[kSmallAccG], g_phase ^ 1u)) {
          fail(6);
          return false;
        }
        tc_fence_after();
        return true;
      };
      auto commit_acc_g = [&]() {
        umma_commit(&acc_full_bar[kSmallAccG]);
        g_phase ^= 1u;
      };
      // X X^T contribution of one 128 x 64 box (K-major operand on both sides)
      auto gram_box = [&](int u, bool first) {
        const uint32_t addr = smem_u32(ring + u * kSmallUnitBytes);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t d = make_smem_desc(addr + k * 32u, 0u, 1024u);
          umma_f16(acc_g, d, d, idesc_gram, (first && k == 0) ? 0u : 1u);
        }
      };
      while (ok) {
        if (!mbar_wait(&mq_full_bar[mq], mq_phase)) {
          fail(5);
          break;
        }
        const int b = mat_queue[mq];
        mbar_arrive(&mq_empty_bar[mq]);
        if (++mq == 2) {
          mq = 0;
          mq_phase ^= 1u;
        }
        if (b < 0) break;
        // ---- Gram matrix of the input: a pass of its own
        if (p.steps > 0) {
          ok = wait_acc_g();
          for (int kb = 0; kb < nk && ok; ++kb) {
            ok = wait_unit();
            if (!ok) break;
            gram_box(unit, kb == 0);
            mbar_arrive(&empty_bar[unit]);
            umma_commit(&empty_bar[unit]);
            advance_unit();
          }
          if (ok) commit_acc_g();
        }
        for (int it = 0; it < p.steps && ok; ++it) {
          const bool quintic = p.abc[3 * it + 2] != 0.0f;
          const bool last = (it == p.steps - 1);
          // ---- A^2 (quintic steps only), into the accumulator the Gram epilogue has just drained
          if (quintic) {
            if (!mbar_wait(a_ready_bar, a_phase)) {
              fail(7);
              ok = false;
              break;
            }
            ok = wait_acc_g();
            if (!ok) break;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint64_t d = make_smem_desc(a_addr + (k >> 2) * kSmallUnitBytes + (k & 3) * 32u, 0u, 1024u);
              umma_f16(acc_g, d, d, idesc_gram, k != 0 ? 1u : 0u);
            }
            commit_acc_g();
          }
          a_phase ^= 1u;
          // ---- S X (S is A itself on cubic steps), with the next iteration's Gram matrix riding behind it
          if (!mbar_wait(s_ready_bar, s_phase)) {
            fail(8);
            ok = false;
            break;
          }
          s_phase ^= 1u;
          if (!last) {
            ok = wait_acc_g();
            if (!ok) break;
          }
          const uint32_t s_op = quintic ? s_addr : a_addr;
          int gunit = unit;   // first box of the oldest tile whose Gram contribution has not been issued yet
          int pending = 0;    // tiles between the S X front and the Gram front
          bool gram_first = true;
          auto gram_tile = [&]() -> bool {
            const int u0 = gunit, u1 = next_unit(u0);
            if (!mbar_wait(&st_ready_bar[u0], (st_bits >> u0) & 1u)) {
              fail(13);
              return false;
            }
            st_bits ^= (1u << u0);
            tc_fence_after();
            gram_box(u0, gram_first);
            gram_box(u1, false);
            gram_first = false;
            umma_commit(&empty_bar[u0]);
            umma_commit(&empty_bar[u1]);
            gunit = next_unit(u1);
            return true;
          };
          for (int t = 0; t < nt && ok; ++t) {
            if (!mbar_wait(&acc_empty_bar[ab], aphase ^ 1u)) {
              fail(6);
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t acc = tmem_base + static_cast<uint32_t>(ab * 128);
            for (int q = 0; q < 2 && ok; ++q) {
              ok = wait_unit();
              if (!ok) break;
              const uint32_t u = smem_u32(ring + unit * kSmallUnitBytes);
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const uint64_t da = make_smem_desc(s_op + (k >> 2) * kSmallUnitBytes + (k & 3) * 32u, 0u, 1024u);
                const uint64_t db = make_smem_desc(u + k * 2048u, 0u, 1024u);
                umma_f16(acc + static_cast<uint32_t>(q * 64), da, db, idesc_sx, k != 0 ? 1u : 0u);
              }
              advance_unit();  // not released here: the epilogue rewrites the box, store thread and Gram MMAs free it
            }
            if (!ok) break;
            umma_commit(&acc_full_bar[ab]);
            if (++ab == kSmallAcc) {
              ab = 0;
              aphase ^= 1u;
            }
            if (!last) {
              ++pending;
              if (pending > kSmallGramLag) {
                ok = gram_tile();
                --pending;
              }
            }
          }
          if (!last) {
            while (ok && pending > 0) {
              ok = gram_tile();
              --pending;
            }
            if (ok) commit_acc_g();
          } else {
            // the store thread consumed this iteration's st_ready phases on its own: keep the parities in step
            int u0 = gunit;
            for (int t = 0; t < nt; ++t) {
              st_bits ^= (1u << u0);
              u0 = next_unit(next_unit(u0));
            }
          }
        }
      }
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ epilogue (warps 2..9)
    const int quarter = warp & 3;
    const int chunk0 = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    int ab = 0;
    uint32_t aphase = 0, g_phase = 0;
    int unit = 0;  // ring position of the next unit, advanced exactly as the producer and the MMA thread do
    int mq = 0;
    uint32_t mq_phase = 0;
    bool ok = true;
    auto release_acc = [&](int which) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty_bar[which]);
    };
    auto load_chunk = [&](int which, int c, uint32_t (&acc)[32]) {
      __syncwarp();
      tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(which * 128 + c * 32),
                    acc);
      tmem_ld_wait();
    };
    auto wait_acc_g = [&]() -> bool {
      if (!mbar_wait(&acc_full_bar[kSmallAccG], g_phase)) {
        fail(10);
        return false;
      }
      g_phase ^= 1u;
      tc_fence_after();
      return true;
    };
    while (ok) {
      if (!mbar_wait(&mq_full_bar[mq], mq_phase)) {
        fail(9);
        break;
      }
      const int b = mat_queue[mq];
      __syncwarp();
      if (lane == 0) mbar_arrive(&mq_empty_bar[mq]);
      if (++mq == 2) {
        mq = 0;
        mq_phase ^= 1u;
      }
      if (b < 0) break;
      if (p.steps > 0) unit = (unit + nk) % kSmallUnits;  // the Gram pass of the input consumed nk units
      const float s_gram = (p.dev_scale != nullptr) ? __ldg(p.dev_scale + 2 * b) : 1.0f;
      const float s_x = (p.dev_scale != nullptr) ? __ldg(p.dev_scale + 2 * b + 1) : 1.0f;
      for (int it = 0; it < p.steps && ok; ++it) {
        const float ca = p.abc[3 * it], cb = p.abc[3 * it + 1], cc = p.abc[3 * it + 2];
        const bool quintic = cc != 0.0f;
        const bool last = (it == p.steps - 1);
        const bool scaled = (it == 0) && (p.dev_scale != nullptr);  // un-normalised iterate: see SmallParams
        // ---- Gram epilogue: A (bf16) into shared memory, operand layout
        ok = wait_acc_g();
        if (!ok) break;
        for (int c = chunk0; c < 4; c += 2) {
          uint32_t acc[32];
          load_chunk(kSmallAccG, c, acc);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            unsigned int w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float g0 = __uint_as_float(acc[8 * q + 2 * e]), g1 = __uint_as_float(acc[8 * q + 2 * e + 1]);
              if (scaled) {
                g0 *= s_gram;
                g1 *= s_gram;
              }
              const unsigned int lo = __bfloat16_as_ushort(__float2bfloat16_rn(g0));
              const unsigned int hi = __bfloat16_as_ushort(__float2bfloat16_rn(g1));
              w[e] = lo | (hi << 16);
            }
            *reinterpret_cast<uint4*>(a_buf + swz_offset(row, c * 32 + q * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(a_ready_bar);
          if (!quintic) mbar_arrive(s_ready_bar);  // cubic step: S is A
        }
        release_acc(kSmallAccG);
        // ---- A^2 epilogue: S = b A + c A^2 into shared memory
        if (quintic) {
          ok = wait_acc_g();
          if (!ok) break;
          for (int c = chunk0; c < 4; c += 2) {
            uint32_t acc[32];
            load_chunk(kSmallAccG, c, acc);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 av = *reinterpret_cast<const uint4*>(a_buf + swz_offset(row, c * 32 + q * 8));
              const unsigned int aw[4] = {av.x, av.y, av.z, av.w};
              unsigned int w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float a0 = __uint_as_float(aw[e] << 16), a1 = __uint_as_float(aw[e] & 0xFFFF0000u);
                const float v0 = fmaf(cb, a0, cc * __uint_as_float(acc[8 * q + 2 * e]));
                const float v1 = fmaf(cb, a1, cc * __uint_as_float(acc[8 * q + 2 * e + 1]));
                w[e] = static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(v0))) |
                       (static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(v1))) << 16);
              }
              *reinterpret_cast<uint4*>(s_buf + swz_offset(row, c * 32 + q * 8)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(s_ready_bar);
          release_acc(kSmallAccG);
        }
        // ---- S X epilogue: X' = a X + alpha (S X), alpha = 1 (quintic) or b (cubic)
        const float alpha = quintic ? 1.0f : cb;
        for (int t = 0; t < nt && ok; ++t) {
          const int u0 = unit, u1 = next_unit(u0);
          unit = next_unit(u1);
          if (!mbar_wait(&acc_full_bar[ab], aphase)) {
            fail(10);
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int c = chunk0 + 2 * h;  // 32-column chunk of the 128-column tile
            const int col0 = t * kSmallTileN + c * 32;
            uint32_t acc[32];
            load_chunk(ab, c, acc);
            // The tile's X values sit in the ring unit the MMA just read (rows = matrix rows, 64 columns per unit,
            // 16-byte groups XOR-swizzled by the row): read a X from there, write the new iterate back in place.
            uint8_t* urow = ring + ((c < 2) ? u0 : u1) * kSmallUnitBytes + row * 128;
            const int g0 = (c & 1) * 4;
            float v[32];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint4 xv = *reinterpret_cast<const uint4*>(urow + (((g0 + q) ^ (row & 7)) << 4));
              const unsigned int ws[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                v[8 * q + 2 * e] = fmaf(ca, __uint_as_float(ws[e] << 16), alpha * __uint_as_float(acc[8 * q + 2 * e]));
                v[8 * q + 2 * e + 1] =
                    fmaf(ca, __uint_as_float(ws[e] & 0xFFFF0000u), alpha * __uint_as_float(acc[8 * q + 2 * e + 1]));
              }
            }
            if (scaled) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] *= s_x;
            }
            if (!last) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                unsigned int w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  w[e] = static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(v[8 * q + 2 * e]))) |
                         (static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(v[8 * q + 2 * e + 1]))) << 16);
                *reinterpret_cast<uint4*>(urow + (((g0 + q) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
              }
            } else if (row < p.m && col0 < p.n) {
              // last iteration: the result leaves in its final dtype, straight from registers
              const int ncols = min(32, p.n - col0);
              if (p.out_fp32) {
                float* o = reinterpret_cast<float*>(p.out) + static_cast<long long>(b) * p.strideo +
                           static_cast<long long>(row) * p.ldo + col0;
                if (ncols == 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
                  for (int q = 0; q < 8; ++q)
                    reinterpret_cast<float4*>(o)[q] = make_float4(__bfloat162float(__float2bfloat16_rn(v[4 * q])),
                                                                  __bfloat162float(__float2bfloat16_rn(v[4 * q + 1])),
                                                                  __bfloat162float(__float2bfloat16_rn(v[4 * q + 2])),
                                                                  __bfloat162float(__float2bfloat16_rn(v[4 * q + 3])));
                } else {
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    if (j < ncols) o[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
                }
              } else {
                unsigned short* o = reinterpret_cast<unsigned short*>(p.out) + static_cast<long long>(b) * p.strideo +
                                    static_cast<long long>(row) * p.ldo + col0;
                if (ncols == 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    unsigned int w[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                      w[e] = static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(v[8 * q + 2 * e]))) |
                             (static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(v[8 * q + 2 * e + 1]))) << 16);
                    reinterpret_cast<uint4*>(o)[q] = make_uint4(w[0], w[1], w[2], w[3]);
                  }
                } else {
#pragma unroll
                  for (int j = 0; j < 32; ++j)
                    if (j < ncols) o[j] = __bfloat16_as_ushort(__float2bfloat16_rn(v[j]));
                }
              }
            }
          }
          // Hand the tile (now holding the new iterate) to the store thread and to the Gram MMAs of the next
          // iteration, then free the accumulator.
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&st_ready_bar[u0]);
          release_acc(ab);
          if (++ab == kSmallAcc) {
            ab = 0;
            aphase ^= 1u;
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ store warp (warp 10)
    if (elect_one()) {
      int unit = 0;
      uint32_t st_bits = 0;  // phase parity of every st_ready barrier, as seen by this thread
      int mq = 0;
      uint32_t mq_phase = 0;
      bool ok = true;
      while (ok) {
        if (!mbar_wait(&mq_full_bar[mq], mq_phase)) {
          fail(11);
          break;
        }
        const int b = mat_queue[mq];
        mbar_arrive(&mq_empty_bar[mq]);
        if (++mq == 2) {
          mq = 0;
          mq_phase ^= 1u;
        }
        if (b < 0) break;
        if (p.steps > 0) unit = (unit + nk) % kSmallUnits;  // the Gram pass of the input consumed nk units
        for (int it = 0; it < p.steps && ok; ++it) {
          const bool last = (it == p.steps - 1);
          const CUtensorMap* map = &maps.x[(it + 1) & 1];
          for (int t = 0; t < nt && ok; ++t) {
            const int u0 = unit, u1 = next_unit(u0);
            unit = next_unit(u1);
            if (!mbar_wait(&st_ready_bar[u0], (st_bits >> u0) & 1u)) {
              fail(12);
              ok = false;
              break;
            }
            st_bits ^= (1u << u0);
            if (!last) {
              tma_store_3d(map, ring + u0 * kSmallUnitBytes, t * kSmallTileN, 0, b);
              tma_store_3d(map, ring + u1 * kSmallUnitBytes, t * kSmallTileN + 64, 0, b);
              tma_store_commit();
              tma_store_wait_read0();  // shared memory has been read; the Gram MMAs give the second arrival
            } else {
              mbar_arrive(&empty_bar[u0]);  // nobody else reads the boxes of the last iteration
              mbar_arrive(&empty_bar[u1]);
            }
            mbar_arrive(&empty_bar[u0]);
            mbar_arrive(&empty_bar[u1]);
          }
          if (!ok) break;
          // Every store of this iteration has landed in global memory: the producer may read the iterate back.
          tma_store_wait0();
          mbar_arrive(x_ready_bar);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
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
