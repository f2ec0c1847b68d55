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
