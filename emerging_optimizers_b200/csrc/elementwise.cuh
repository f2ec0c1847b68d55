// HBM-bound passes around the tensor-core kernels: Frobenius sum of squares (two-stage, fixed
// order, float64 accumulation) and the divide-by-norm pass that also narrows fp32 to bf16.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace eo {

constexpr int kEwThreads = 256;
constexpr int kSumsqMaxBlocks = 1024;
constexpr long long kSumsqElemsPerBlock = 32768;

inline int sumsq_blocks_per_matrix(int64_t rows, int64_t cols) {
  const long long total = static_cast<long long>(rows) * cols;
  long long nb = (total + kSumsqElemsPerBlock - 1) / kSumsqElemsPerBlock;
  if (nb < 1) nb = 1;
  if (nb > kSumsqMaxBlocks) nb = kSumsqMaxBlocks;
  return static_cast<int>(nb);
}

__device__ __forceinline__ double block_reduce_sum(double v) {
  __shared__ double warp_sums[kEwThreads / 32];
  for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) warp_sums[warp] = v;
  __syncthreads();
  double total = 0.0;
  if (threadIdx.x == 0) {
    for (int w = 0; w < kEwThreads / 32; ++w) total += warp_sums[w];
  }
  return total;  // valid in thread 0
}

// partial[b * gridDim.x + blockIdx.x] = sum of squares of this block's slice of matrix b.
__global__ void __launch_bounds__(kEwThreads)
    sumsq_partial_kernel(const float* __restrict__ x, long long rows, long long cols, long long ld, long long stride,
                         int vec4, double* __restrict__ partial) {
  const int b = blockIdx.y;
  const float* xb = x + static_cast<long long>(b) * stride;
  double acc = 0.0;
  const long long tid = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * kEwThreads;
  if (vec4) {
    const long long c4 = cols >> 2;
    const long long units = rows * c4;
    for (long long u = tid; u < units; u += nthreads) {
      const long long r = u / c4, c = u - r * c4;
      const float4 v = __ldg(reinterpret_cast<const float4*>(xb + r * ld) + c);
      acc += static_cast<double>(v.x) * v.x + static_cast<double>(v.y) * v.y;
      acc += static_cast<double>(v.z) * v.z + static_cast<double>(v.w) * v.w;
    }
  } else {
    const long long units = rows * cols;
    for (long long u = tid; u < units; u += nthreads) {
      const long long r = u / cols, c = u - r * cols;
      const double v = xb[r * ld + c];
      acc += v * v;
    }
  }
  const double total = block_reduce_sum(acc);
  if (threadIdx.x == 0) partial[static_cast<long long>(b) * gridDim.x + blockIdx.x] = total;
}

// sumsq[b] = sum of partial[b * nblk .. b * nblk + nblk), pairwise inside one block.
__global__ void __launch_bounds__(kEwThreads)
    sumsq_final_kernel(const double* __restrict__ partial, int nblk, double* __restrict__ sumsq) {
  const int b = blockIdx.x;
  double acc = 0.0;
  for (int i = threadIdx.x; i < nblk; i += kEwThreads) acc += partial[static_cast<long long>(b) * nblk + i];
  const double total = block_reduce_sum(acc);
  if (threadIdx.x == 0) sumsq[b] = total;
}

__global__ void __launch_bounds__(kEwThreads)
    normalize_kernel(const float* __restrict__ x, long long rows, long long cols, long long ld, long long stride,
                     const double* __restrict__ sumsq, float eps, int clamp_eps, void* __restrict__ out,
                     long long ldo, long long strideo, int out_fp32, int round_bf16, int vec4) {
  const int b = blockIdx.y;
  const float* xb = x + static_cast<long long>(b) * stride;
  float norm = static_cast<float>(sqrt(sumsq[b]));
  if (clamp_eps) norm = fmaxf(norm, eps);
  const long long tid = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * kEwThreads;
  if (vec4) {
    const long long c4 = cols >> 2;
    const long long units = rows * c4;
    for (long long u = tid; u < units; u += nthreads) {
      const long long r = u / c4, c = u - r * c4;
      const float4 v = __ldg(reinterpret_cast<const float4*>(xb + r * ld) + c);
      float q[4] = {v.x / norm, v.y / norm, v.z / norm, v.w / norm};
      if (out_fp32) {
        if (round_bf16) {
#pragma unroll
          for (int i = 0; i < 4; ++i) q[i] = __bfloat162float(__float2bfloat16_rn(q[i]));
        }
        float* o = reinterpret_cast<float*>(out) + static_cast<long long>(b) * strideo + r * ldo;
        reinterpret_cast<float4*>(o)[c] = make_float4(q[0], q[1], q[2], q[3]);
      } else {
        unsigned short h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __bfloat16_as_ushort(__float2bfloat16_rn(q[i]));
        uint2 t;
        t.x = static_cast<unsigned int>(h[0]) | (static_cast<unsigned int>(h[1]) << 16);
        t.y = static_cast<unsigned int>(h[2]) | (static_cast<unsigned int>(h[3]) << 16);
        unsigned short* o = reinterpret_cast<unsigned short*>(out) + static_cast<long long>(b) * strideo + r * ldo;
        reinterpret_cast<uint2*>(o)[c] = t;
      }
    }
  } else {
    const long long units = rows * cols;
    for (long long u = tid; u < units; u += nthreads) {
      const long long r = u / cols, c = u - r * cols;
      float q = xb[r * ld + c] / norm;
      if (out_fp32) {
        if (round_bf16) q = __bfloat162float(__float2bfloat16_rn(q));
        reinterpret_cast<float*>(out)[static_cast<long long>(b) * strideo + r * ldo + c] = q;
      } else {
        reinterpret_cast<__nv_bfloat16*>(out)[static_cast<long long>(b) * strideo + r * ldo + c] =
            __float2bfloat16_rn(q);
      }
    }
  }
}

// One pass over an fp32 matrix batch that writes it rounded to bf16 (NOT normalised) and leaves per-block partial
// sums of squares of the fp32 values: the first half of a Frobenius normalisation whose division is applied later,
// inside the epilogues of the first Gram and the first update product (see GemmParams::dev_scale).
__global__ void __launch_bounds__(kEwThreads)
    cast_sumsq_kernel(const float* __restrict__ x, long long rows, long long cols, long long ld, long long stride,
                      unsigned short* __restrict__ out, long long ldo, long long strideo, int vec4,
                      double* __restrict__ partial) {
  const int b = blockIdx.y;
  const float* xb = x + static_cast<long long>(b) * stride;
  unsigned short* ob = out + static_cast<long long>(b) * strideo;
  double acc = 0.0;
  const long long tid = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * kEwThreads;
  auto one = [&acc](const float4 v) {
    acc += static_cast<double>(v.x) * v.x + static_cast<double>(v.y) * v.y;
    acc += static_cast<double>(v.z) * v.z + static_cast<double>(v.w) * v.w;
    uint2 t;
    t.x = static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(v.x))) |
          (static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(v.y))) << 16);
    t.y = static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(v.z))) |
          (static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(v.w))) << 16);
    return t;
  };
  if (vec4 && ld == cols && ldo == cols) {
    // Dense rows: the matrix is one contiguous run.  Four grid strides per trip, all loads issued before the first
    // use, so that enough bytes are in flight to reach the HBM bandwidth; no index arithmetic per element.
    const float4* x4 = reinterpret_cast<const float4*>(xb);
    uint2* o2 = reinterpret_cast<uint2*>(ob);
    const long long units = (rows * cols) >> 2;
    long long u = tid;
    for (; u + 3 * nthreads < units; u += 4 * nthreads) {
      const float4 v0 = __ldg(x4 + u), v1 = __ldg(x4 + u + nthreads);
      const float4 v2 = __ldg(x4 + u + 2 * nthreads), v3 = __ldg(x4 + u + 3 * nthreads);
      o2[u] = one(v0);
      o2[u + nthreads] = one(v1);
      o2[u + 2 * nthreads] = one(v2);
      o2[u + 3 * nthreads] = one(v3);
    }
    for (; u < units; u += nthreads) o2[u] = one(__ldg(x4 + u));
  } else if (vec4) {
    const long long c4 = cols >> 2;
    const long long units = rows * c4;
    for (long long u = tid; u < units; u += nthreads) {
      const long long r = u / c4, c = u - r * c4;
      reinterpret_cast<uint2*>(ob + r * ldo)[c] = one(__ldg(reinterpret_cast<const float4*>(xb + r * ld) + c));
    }
  } else {
    const long long units = rows * cols;
    for (long long u = tid; u < units; u += nthreads) {
      const long long r = u / cols, c = u - r * cols;
      const float v = xb[r * ld + c];
      acc += static_cast<double>(v) * v;
      ob[r * ldo + c] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
    }
  }
  const double total = block_reduce_sum(acc);
  if (threadIdx.x == 0) partial[static_cast<long long>(b) * gridDim.x + blockIdx.x] = total;
}

// sumsq[b] as in sumsq_final_kernel, plus the two factors the deferred normalisation needs:
// scales[2 b] = 1 / max(norm, eps)^2 (for X X^T) and scales[2 b + 1] = 1 / max(norm, eps) (for X itself).
__global__ void __launch_bounds__(kEwThreads)
    sumsq_scales_kernel(const double* __restrict__ partial, int nblk, float eps, double* __restrict__ sumsq,
                        float* __restrict__ scales) {
  const int b = blockIdx.x;
  double acc = 0.0;
  for (int i = threadIdx.x; i < nblk; i += kEwThreads) acc += partial[static_cast<long long>(b) * nblk + i];
  const double total = block_reduce_sum(acc);
  if (threadIdx.x == 0) {
    if (sumsq != nullptr) sumsq[b] = total;
    const float inv = 1.0f / fmaxf(static_cast<float>(sqrt(total)), eps);
    scales[2 * b] = inv * inv;
    scales[2 * b + 1] = inv;
  }
}

// Split fp32 into three bf16 planes with x = p0 + p1 + p2 up to 2^-24 relative: p0 = bf16(x),
// p1 = bf16(x - p0), p2 = bf16(x - p0 - p1); both remainders are exact in fp32.
__global__ void __launch_bounds__(kEwThreads)
    split3_kernel(const float* __restrict__ x, long long rows, long long cols, long long ld, long long stride,
                  __nv_bfloat16* __restrict__ out, long long ldo, long long strideo, long long plane_stride) {
  const int b = blockIdx.y;
  const float* xb = x + static_cast<long long>(b) * stride;
  __nv_bfloat16* ob = out + static_cast<long long>(b) * strideo;
  const long long tid = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * kEwThreads;
  const long long units = rows * cols;
  for (long long u = tid; u < units; u += nthreads) {
    const long long r = u / cols, c = u - r * cols;
    const float v = xb[r * ld + c];
    const __nv_bfloat16 h0 = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(h0);
    const __nv_bfloat16 h1 = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(h1);
    const __nv_bfloat16 h2 = __float2bfloat16_rn(r2);
    const long long o = r * ldo + c;
    ob[o] = h0;
    ob[o + plane_stride] = h1;
    ob[o + 2 * plane_stride] = h2;
  }
}

inline void launch_split3(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride,
                          void* out, int64_t ldo, int64_t strideo, int64_t plane_stride, cudaStream_t stream) {
  const long long total = static_cast<long long>(rows) * cols;
  long long nblk = (total + kEwThreads * 4 - 1) / (kEwThreads * 4);
  if (nblk < 1) nblk = 1;
  if (nblk > 4096) nblk = 4096;
  for (int b0 = 0; b0 < batch; b0 += 65535) {
    const int nb = (batch - b0 < 65535) ? (batch - b0) : 65535;
    split3_kernel<<<dim3(static_cast<unsigned>(nblk), nb), kEwThreads, 0, stream>>>(
        x + static_cast<long long>(b0) * stride, rows, cols, ld, stride,
        static_cast<__nv_bfloat16*>(out) + static_cast<long long>(b0) * strideo, ldo, strideo, plane_stride);
  }
}

// Sum of `nparts` fp32 partial matrices (rows x cols, row stride ld, `part_stride` elements apart), in a fixed order,
// written as fp32 and as three bf16 planes: the tail of a K-split product followed by split3 in one pass.
__global__ void __launch_bounds__(kEwThreads)
    sum_split3_kernel(const float* __restrict__ parts, int nparts, long long part_stride, long long rows,
                      long long cols, long long ld, float* __restrict__ sum, __nv_bfloat16* __restrict__ out,
                      long long ldo, long long plane_stride) {
  const long long tid = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * kEwThreads;
  const long long units = rows * cols;
  for (long long u = tid; u < units; u += nthreads) {
    const long long r = u / cols, c = u - r * cols;
    const long long at = r * ld + c;
    float v = parts[at];
    for (int s = 1; s < nparts; ++s) v = __fadd_rn(v, parts[at + s * part_stride]);
    sum[at] = v;
    const __nv_bfloat16 h0 = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(h0);
    const __nv_bfloat16 h1 = __float2bfloat16_rn(r1);
    const float r2 = r1 - __bfloat162float(h1);
    const __nv_bfloat16 h2 = __float2bfloat16_rn(r2);
    const long long o = r * ldo + c;
    out[o] = h0;
    out[o + plane_stride] = h1;
    out[o + 2 * plane_stride] = h2;
  }
}

inline void launch_sum_split3(const float* parts, int nparts, int64_t part_stride, int64_t rows, int64_t cols,
                              int64_t ld, float* sum, void* out, int64_t ldo, int64_t plane_stride,
                              cudaStream_t stream) {
  const long long total = static_cast<long long>(rows) * cols;
  long long nblk = (total + kEwThreads * 4 - 1) / (kEwThreads * 4);
  if (nblk < 1) nblk = 1;
  if (nblk > 4096) nblk = 4096;
  sum_split3_kernel<<<static_cast<unsigned>(nblk), kEwThreads, 0, stream>>>(
      parts, nparts, part_stride, rows, cols, ld, sum, static_cast<__nv_bfloat16*>(out), ldo, plane_stride);
}

// ---------------------------------------------------------------------------------------------
// Muon step, elementwise parts, on flat contiguous fp32 arrays.
//   u(g, m', p) : g' = g + l2 * p;  m' = lerp(m, g', 1 - mu);  u = nesterov ? lerp(g', m', mu) : m'
// with lerp(a, b, w) = |w| < 0.5 ? a + w (b - a) : b - (b - a)(1 - w)   (the formula torch.lerp uses).
// ---------------------------------------------------------------------------------------------
// Written with explicit fused multiply-adds, which is what the compiler makes of torch's expression: the result
// must not depend on how the surrounding code happens to be contracted.
__device__ __forceinline__ float lerp_f32(float a, float b, float w) {
  const float d = __fsub_rn(b, a);
  return (fabsf(w) < 0.5f) ? __fmaf_rn(w, d, a) : __fmaf_rn(-d, __fsub_rn(1.0f, w), b);
}

struct MuonEw {
  float momentum;  // mu
  float one_minus_momentum;  // 1 - mu, rounded once from double (the weight torch.lerp_ receives)
  float l2;        // weight decay added to the gradient (0 unless the l2 method is used)
  int nesterov;
};

__device__ __forceinline__ float muon_update(float g, float m_new, const MuonEw& c) {
  return c.nesterov ? lerp_f32(g, m_new, c.momentum) : m_new;
}

// One float4 of pass 1: the new momentum values (returned through mv) and the sum of squares of the four updates.
__device__ __forceinline__ double muon_momentum_quad(float4 gv, float4& mv, const MuonEw& c) {
  const float w = c.one_minus_momentum;
  mv.x = lerp_f32(mv.x, gv.x, w); mv.y = lerp_f32(mv.y, gv.y, w);
  mv.z = lerp_f32(mv.z, gv.z, w); mv.w = lerp_f32(mv.w, gv.w, w);
  const double u0 = muon_update(gv.x, mv.x, c), u1 = muon_update(gv.y, mv.y, c);
  const double u2 = muon_update(gv.z, mv.z, c), u3 = muon_update(gv.w, mv.w, c);
  return (u0 * u0 + u1 * u1) + (u2 * u2 + u3 * u3);
}

__device__ __forceinline__ float4 muon_add_l2(float4 gv, float4 pv, float l2) {
  // g + l2 * p with one rounding, as torch's add(p, alpha=l2) computes it
  gv.x = __fmaf_rn(l2, pv.x, gv.x); gv.y = __fmaf_rn(l2, pv.y, gv.y);
  gv.z = __fmaf_rn(l2, pv.z, gv.z); gv.w = __fmaf_rn(l2, pv.w, gv.w);
  return gv;
}

// Pass 1: momentum buffer update in place and per-block partial sums of u^2.
__device__ __forceinline__ void muon_momentum_body(const float* __restrict__ g, float* __restrict__ m,
                                                   const float* __restrict__ p, long long numel, const MuonEw& c,
                                                   double* __restrict__ partial_slot) {
  double acc = 0.0;
  const long long tid = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * kEwThreads;
  const long long n4 = numel >> 2;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  const float4* p4 = reinterpret_cast<const float4*>(p);
  float4* m4 = reinterpret_cast<float4*>(m);
  const bool l2 = c.l2 != 0.0f;
  long long i = tid;
  // Two grid strides per trip, every load issued before the first store: the in-place update of m would otherwise
  // order each trip's loads behind the previous trip's store and halve the bytes in flight.
  for (; i + nthreads < n4; i += 2 * nthreads) {
    float4 g0 = __ldg(g4 + i), g1 = __ldg(g4 + i + nthreads);
    float4 m0 = m4[i], m1 = m4[i + nthreads];
    if (l2) {
      g0 = muon_add_l2(g0, __ldg(p4 + i), c.l2);
      g1 = muon_add_l2(g1, __ldg(p4 + i + nthreads), c.l2);
    }
    acc += muon_momentum_quad(g0, m0, c);
    m4[i] = m0;
    acc += muon_momentum_quad(g1, m1, c);
    m4[i + nthreads] = m1;
  }
  for (; i < n4; i += nthreads) {
    float4 gv = __ldg(g4 + i);
    float4 mv = m4[i];
    if (l2) gv = muon_add_l2(gv, __ldg(p4 + i), c.l2);
    acc += muon_momentum_quad(gv, mv, c);
    m4[i] = mv;
  }
  const float w = c.one_minus_momentum;
  for (long long i = (n4 << 2) + tid; i < numel; i += nthreads) {
    float gv = g[i];
    if (c.l2 != 0.0f) gv = __fmaf_rn(c.l2, p[i], gv);
    const float mv = lerp_f32(m[i], gv, w);
    m[i] = mv;
    const double u = muon_update(gv, mv, c);
    acc += u * u;
  }
  const double total = block_reduce_sum(acc);
  if (threadIdx.x == 0) *partial_slot = total;
}

// Pass 1 with the update written out: as muon_momentum_body, plus u itself rounded to bf16 (NOT normalised) into
// `out`.  With the division deferred to the epilogues of the first two products of the iteration (see
// GemmParams::dev_scale) this is the only elementwise pass before Newton-Schulz: g and m are read once.
__device__ __forceinline__ void muon_momentum_cast_body(const float* __restrict__ g, float* __restrict__ m,
                                                        const float* __restrict__ p, long long numel, const MuonEw& c,
                                                        __nv_bfloat16* __restrict__ out,
                                                        double* __restrict__ partial_slot) {
  double acc = 0.0;
  const long long tid = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * kEwThreads;
  const long long n4 = numel >> 2;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  const float4* p4 = reinterpret_cast<const float4*>(p);
  float4* m4 = reinterpret_cast<float4*>(m);
  const bool l2 = c.l2 != 0.0f;
  const float w = c.one_minus_momentum;
  auto quad = [&](float4 gv, float4& mv, long long i) {
    mv.x = lerp_f32(mv.x, gv.x, w); mv.y = lerp_f32(mv.y, gv.y, w);
    mv.z = lerp_f32(mv.z, gv.z, w); mv.w = lerp_f32(mv.w, gv.w, w);
    const float u0 = muon_update(gv.x, mv.x, c), u1 = muon_update(gv.y, mv.y, c);
    const float u2 = muon_update(gv.z, mv.z, c), u3 = muon_update(gv.w, mv.w, c);
    uint2 t;
    t.x = static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(u0))) |
          (static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(u1))) << 16);
    t.y = static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(u2))) |
          (static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(u3))) << 16);
    reinterpret_cast<uint2*>(out)[i] = t;
    const double d0 = u0, d1 = u1, d2 = u2, d3 = u3;
    return (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
  };
  long long i = tid;
  for (; i + nthreads < n4; i += 2 * nthreads) {  // two grid strides per trip, loads first (see muon_momentum_body)
    float4 g0 = __ldg(g4 + i), g1 = __ldg(g4 + i + nthreads);
    float4 m0 = m4[i], m1 = m4[i + nthreads];
    if (l2) {
      g0 = muon_add_l2(g0, __ldg(p4 + i), c.l2);
      g1 = muon_add_l2(g1, __ldg(p4 + i + nthreads), c.l2);
    }
    acc += quad(g0, m0, i);
    m4[i] = m0;
    acc += quad(g1, m1, i + nthreads);
    m4[i + nthreads] = m1;
  }
  for (; i < n4; i += nthreads) {
    float4 gv = __ldg(g4 + i);
    float4 mv = m4[i];
    if (l2) gv = muon_add_l2(gv, __ldg(p4 + i), c.l2);
    acc += quad(gv, mv, i);
    m4[i] = mv;
  }
  for (long long j = (n4 << 2) + tid; j < numel; j += nthreads) {
    float gv = g[j];
    if (l2) gv = __fmaf_rn(c.l2, p[j], gv);
    const float mv = lerp_f32(m[j], gv, w);
    m[j] = mv;
    const float u = muon_update(gv, mv, c);
    out[j] = __float2bfloat16_rn(u);
    acc += static_cast<double>(u) * u;
  }
  const double total = block_reduce_sum(acc);
  if (threadIdx.x == 0) *partial_slot = total;
}

// Pass 2: recompute u from g and the updated momentum buffer, divide by the norm, write bf16.
__device__ __forceinline__ void muon_normalize_body(const float* __restrict__ g, const float* __restrict__ m,
                                                    const float* __restrict__ p, long long numel, const MuonEw& c,
                                                    double sumsq, float eps, __nv_bfloat16* __restrict__ out) {
  const float norm = fmaxf(static_cast<float>(sqrt(sumsq)), eps);
  const long long tid = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * kEwThreads;
  const long long n4 = numel >> 2;
  for (long long i = tid; i < n4; i += nthreads) {
    float4 gv = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c.nesterov) gv = __ldg(reinterpret_cast<const float4*>(g) + i);
    if (c.nesterov && c.l2 != 0.0f) gv = muon_add_l2(gv, __ldg(reinterpret_cast<const float4*>(p) + i), c.l2);
    const float4 mv = __ldg(reinterpret_cast<const float4*>(m) + i);
    const float q0 = muon_update(gv.x, mv.x, c) / norm, q1 = muon_update(gv.y, mv.y, c) / norm;
    const float q2 = muon_update(gv.z, mv.z, c) / norm, q3 = muon_update(gv.w, mv.w, c) / norm;
    uint2 t;
    t.x = static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(q0))) |
          (static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(q1))) << 16);
    t.y = static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(q2))) |
          (static_cast<unsigned int>(__bfloat16_as_ushort(__float2bfloat16_rn(q3))) << 16);
    reinterpret_cast<uint2*>(out)[i] = t;
  }
  for (long long i = (n4 << 2) + tid; i < numel; i += nthreads) {
    float gv = 0.f;
    if (c.nesterov) {
      gv = g[i];
      if (c.l2 != 0.0f) gv = __fmaf_rn(c.l2, p[i], gv);
    }
    out[i] = __float2bfloat16_rn(muon_update(gv, m[i], c) / norm);
  }
}

// Weight update: p <- (p + shrink * p) - lr * ((u * scale) * extra), the operation order of
// `p.add_(p, alpha=shrink)` followed by `p.add_(u * scale * extra, alpha=-lr)`.
__device__ __forceinline__ float muon_apply_one(float pv, float uv, float shrink, float scale, float extra, float lr) {
  // explicit roundings: each add(x, alpha=s) of torch is one fused multiply-add
  if (shrink != 0.0f) pv = __fmaf_rn(shrink, pv, pv);
  const float t = __fmul_rn(__fmul_rn(uv, scale), extra);
  return __fmaf_rn(-lr, t, pv);
}

template <typename U>
__device__ __forceinline__ void muon_apply_body(float* __restrict__ p, const U* __restrict__ u, long long numel,
                                                float shrink, float scale, float extra, float lr) {
  const long long tid = static_cast<long long>(blockIdx.x) * kEwThreads + threadIdx.x;
  const long long nthreads = static_cast<long long>(gridDim.x) * kEwThreads;
  const bool vec = (reinterpret_cast<uintptr_t>(p) % 16 == 0) && (reinterpret_cast<uintptr_t>(u) % (4 * sizeof(U)) == 0);
  const long long n4 = vec ? (numel >> 2) : 0;
  for (long long i = tid; i < n4; i += nthreads) {
    float4 pv = reinterpret_cast<float4*>(p)[i];
    float u0, u1, u2, u3;
    if constexpr (sizeof(U) == 2) {
      const uint2 t = __ldg(reinterpret_cast<const uint2*>(u) + i);
      u0 = __uint_as_float(t.x << 16); u1 = __uint_as_float(t.x & 0xFFFF0000u);
      u2 = __uint_as_float(t.y << 16); u3 = __uint_as_float(t.y & 0xFFFF0000u);
    } else {
      const float4 t = __ldg(reinterpret_cast<const float4*>(u) + i);
      u0 = t.x; u1 = t.y; u2 = t.z; u3 = t.w;
    }
    pv.x = muon_apply_one(pv.x, u0, shrink, scale, extra, lr);
    pv.y = muon_apply_one(pv.y, u1, shrink, scale, extra, lr);
    pv.z = muon_apply_one(pv.z, u2, shrink, scale, extra, lr);
    pv.w = muon_apply_one(pv.w, u3, shrink, scale, extra, lr);
    reinterpret_cast<float4*>(p)[i] = pv;
  }
  for (long long i = (n4 << 2) + tid; i < numel; i += nthreads) {
    float uv;
    if constexpr (sizeof(U) == 2) {
      uv = __bfloat162float(u[i]);
    } else {
      uv = u[i];
    }
    p[i] = muon_apply_one(p[i], uv, shrink, scale, extra, lr);
  }
}

__global__ void __launch_bounds__(kEwThreads)
    muon_momentum_kernel(const float* __restrict__ g, float* __restrict__ m, const float* __restrict__ p,
                         long long numel, MuonEw c, double* __restrict__ partial) {
  muon_momentum_body(g, m, p, numel, c, partial + blockIdx.x);
}

__global__ void __launch_bounds__(kEwThreads)
    muon_normalize_kernel(const float* __restrict__ g, const float* __restrict__ m, const float* __restrict__ p,
                          long long numel, MuonEw c, const double* __restrict__ sumsq, float eps,
                          __nv_bfloat16* __restrict__ out) {
  muon_normalize_body(g, m, p, numel, c, sumsq[0], eps, out);
}

template <typename U>
__global__ void __launch_bounds__(kEwThreads)
    muon_apply_kernel(float* __restrict__ p, const U* __restrict__ u, long long numel, float shrink, float scale,
                      float extra, float lr) {
  muon_apply_body<U>(p, u, numel, shrink, scale, extra, lr);
}

// Multi-tensor variants: blockIdx.y selects a tensor from a table passed by value in the kernel parameters
// (no device-side table, no host-to-device copy); blockIdx.x partitions that tensor as the single-tensor
// kernels do, so results are bit-identical to theirs.
constexpr int kMtMax = 48;

struct MtPrepare {
  const float* g[kMtMax];
  float* m[kMtMax];
  const float* p[kMtMax];
};

struct MtApply {
  float* p[kMtMax];
  const void* u[kMtMax];
  long long numel[kMtMax];
  float scale[kMtMax];
};

__global__ void __launch_bounds__(kEwThreads)
    muon_momentum_mt_kernel(const __grid_constant__ MtPrepare t, long long numel, MuonEw c,
                            double* __restrict__ partial) {
  const int y = blockIdx.y;
  muon_momentum_body(t.g[y], t.m[y], t.p[y], numel, c, partial + static_cast<long long>(y) * gridDim.x + blockIdx.x);
}

__global__ void __launch_bounds__(kEwThreads)
    muon_normalize_mt_kernel(const __grid_constant__ MtPrepare t, long long numel, MuonEw c,
                             const double* __restrict__ sumsq, float eps, __nv_bfloat16* __restrict__ out,
                             long long slot_stride) {
  const int y = blockIdx.y;
  muon_normalize_body(t.g[y], t.m[y], t.p[y], numel, c, sumsq[y], eps, out + static_cast<long long>(y) * slot_stride);
}

__global__ void __launch_bounds__(kEwThreads)
    muon_momentum_cast_mt_kernel(const __grid_constant__ MtPrepare t, long long numel, MuonEw c,
                                 __nv_bfloat16* __restrict__ out, long long slot_stride,
                                 double* __restrict__ partial) {
  const int y = blockIdx.y;
  muon_momentum_cast_body(t.g[y], t.m[y], t.p[y], numel, c, out + static_cast<long long>(y) * slot_stride,
                          partial + static_cast<long long>(y) * gridDim.x + blockIdx.x);
}

template <typename U>
__global__ void __launch_bounds__(kEwThreads)
    muon_apply_mt_kernel(const __grid_constant__ MtApply t, float shrink, float extra, float lr) {
  const int y = blockIdx.y;
  muon_apply_body<U>(t.p[y], static_cast<const U*>(t.u[y]), t.numel[y], shrink, t.scale[y], extra, lr);
}

inline int ew_blocks(long long numel, int per_thread) {
  long long nb = (numel + static_cast<long long>(kEwThreads) * per_thread - 1) / (static_cast<long long>(kEwThreads) * per_thread);
  if (nb < 1) nb = 1;
  if (nb > 4096) nb = 4096;
  return static_cast<int>(nb);
}

inline void launch_sumsq(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride,
                         double* sumsq, double* scratch, cudaStream_t stream) {
  const int nblk = sumsq_blocks_per_matrix(rows, cols);
  const int vec4 = (cols % 4 == 0) && (ld % 4 == 0) && (stride % 4 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0);
  // gridDim.y is limited to 65535: walk the batch in slabs.
  for (int b0 = 0; b0 < batch; b0 += 65535) {
    const int nb = (batch - b0 < 65535) ? (batch - b0) : 65535;
    sumsq_partial_kernel<<<dim3(nblk, nb), kEwThreads, 0, stream>>>(x + static_cast<long long>(b0) * stride, rows, cols,
                                                                    ld, stride, vec4,
                                                                    scratch + static_cast<long long>(b0) * nblk);
  }
  sumsq_final_kernel<<<batch, kEwThreads, 0, stream>>>(scratch, nblk, sumsq);
}

inline void launch_cast_sumsq(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride,
                              void* out, int64_t ldo, int64_t strideo, float eps, double* sumsq, float* scales,
                              double* scratch, cudaStream_t stream) {
  const int nblk = sumsq_blocks_per_matrix(rows, cols);
  const int vec4 = (cols % 4 == 0) && (ld % 4 == 0) && (stride % 4 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(out) % 8 == 0) && (ldo % 4 == 0) && (strideo % 4 == 0);
  for (int b0 = 0; b0 < batch; b0 += 65535) {
    const int nb = (batch - b0 < 65535) ? (batch - b0) : 65535;
    cast_sumsq_kernel<<<dim3(nblk, nb), kEwThreads, 0, stream>>>(
        x + static_cast<long long>(b0) * stride, rows, cols, ld, stride,
        static_cast<unsigned short*>(out) + static_cast<long long>(b0) * strideo, ldo, strideo, vec4,
        scratch + static_cast<long long>(b0) * nblk);
  }
  sumsq_scales_kernel<<<batch, kEwThreads, 0, stream>>>(scratch, nblk, eps, sumsq, scales);
}

inline void launch_normalize(const float* x, int batch, int64_t rows, int64_t cols, int64_t ld, int64_t stride,
                             const double* sumsq, float eps, int clamp_eps, void* out, int64_t ldo, int64_t strideo,
                             int out_fp32, int round_bf16, cudaStream_t stream) {
  const int out_eb = out_fp32 ? 4 : 2;
  const int vec4 = (cols % 4 == 0) && (ld % 4 == 0) && (stride % 4 == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                   (reinterpret_cast<uintptr_t>(out) % 16 == 0) && ((ldo * out_eb) % (4 * out_eb) == 0) &&
                   ((strideo * out_eb) % (4 * out_eb) == 0);
  const long long total = static_cast<long long>(rows) * cols;
  long long nblk = (total / (vec4 ? 4 : 1) + kEwThreads * 4 - 1) / (kEwThreads * 4);
  if (nblk < 1) nblk = 1;
  if (nblk > 2048) nblk = 2048;
  for (int b0 = 0; b0 < batch; b0 += 65535) {
    const int nb = (batch - b0 < 65535) ? (batch - b0) : 65535;
    normalize_kernel<<<dim3(static_cast<unsigned>(nblk), nb), kEwThreads, 0, stream>>>(
        x + static_cast<long long>(b0) * stride, rows, cols, ld, stride, sumsq + b0, eps, clamp_eps,
        static_cast<char*>(out) + static_cast<long long>(b0) * strideo * out_eb, ldo, strideo, out_fp32, round_bf16,
        vec4);
  }
}

}  // namespace eo
