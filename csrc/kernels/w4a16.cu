// MatMulNBits int4 weight-only projection (block 32, symmetric zp = 8 or packed nibble zero points,
// bf16 or fp32 scales) with in-kernel dequantisation.
//
// Layout is the ONNX contrib operator's: B[N, ceil(K/32), 16] uint8 with the low nibble holding the
// even k, scales[N, ceil(K/32)], optional zero_points[N, ceil(ceil(K/32)/2)] (nibbles), optional bias
// (crates/onnx-runtime-ep-cpu/src/kernels/matmul_nbits.rs:1-17).  The reference needs ~60 GEMV / GEMM
// variants for this operator (crates/onnx-runtime-ep-cuda/src/kernels/matmul_nbits.rs:58-311) plus a
// Marlin-style mma.sync GEMM (marlin_gemm.rs:1-72).  Here:
//   * w4a16_gemv_kernel  -- M <= 8 activations rows per pass: one warp per 4 output columns, each lane
//     streams whole 32-weight blocks with 128-bit loads (one scale per load), nibbles are turned into
//     floats with the 0x4300 bf16 magic-number trick (no int->float conversions), fp32 accumulate;
//   * w4a16_dequant_kernel -- expands W to bf16 [N, K] so larger M runs on the tcgen05 GEMM.
#include "common.cuh"
#include "ogb_kernels.h"

namespace ogb {

constexpr int kGemvCols = 4;     // output columns per warp
constexpr int kGemvWarps = 8;
constexpr int kGemvMaxM = 8;

// 8 nibbles of one 32-bit word -> 8 floats (value = nibble), in k order: low nibble of byte 0 first.
OGB_DEVICE void nibbles_to_float(uint32_t w, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    // bf16 0x4300 = 128.0 with a mantissa step of 1: OR-ing a nibble gives 128 + nibble exactly
    const uint32_t bits = (0x4300u | ((w >> (4 * i)) & 0xFu)) << 16;
    f[i] = __uint_as_float(bits) - 128.0f;
  }
}

template <bool SCALES_F32>
OGB_DEVICE float load_scale(const void* scales, size_t idx) {
  if constexpr (SCALES_F32) return static_cast<const float*>(scales)[idx];
  return __bfloat162float(static_cast<const __nv_bfloat16*>(scales)[idx]);
}

template <bool SCALES_F32>
__global__ void __launch_bounds__(kGemvWarps * 32) w4a16_gemv_kernel(const __nv_bfloat16* __restrict__ x,
                                                                     const uint8_t* __restrict__ qw, const void* __restrict__ scales,
                                                                     const uint8_t* __restrict__ zp, const __nv_bfloat16* __restrict__ bias,
                                                                     __nv_bfloat16* __restrict__ y, int M, int N, int K, int ldx, int ldy) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (blockIdx.x * kGemvWarps + warp) * kGemvCols;
  if (n0 >= N) return;
  const int kb = (K + 31) / 32;
  const int zp_stride = (kb + 1) / 2;
  float acc[kGemvCols][kGemvMaxM];
#pragma unroll
  for (int c = 0; c < kGemvCols; ++c)
#pragma unroll
    for (int m = 0; m < kGemvMaxM; ++m) acc[c][m] = 0.f;

  for (int b = lane; b < kb; b += 32) {
    const int kbase = b * 32;
    // weights, scales and zero points of this k block for the warp's columns (independent 128-bit loads)
    uint4 wq[kGemvCols];
    float sc[kGemvCols], zz[kGemvCols];
#pragma unroll
    for (int c = 0; c < kGemvCols; ++c) {
      const int n = min(n0 + c, N - 1);
      wq[c] = __ldg(reinterpret_cast<const uint4*>(qw + (static_cast<size_t>(n) * kb + b) * 16));
      sc[c] = load_scale<SCALES_F32>(scales, static_cast<size_t>(n) * kb + b);
      zz[c] = 8.f;
      if (zp != nullptr) {
        const uint8_t zb = zp[static_cast<size_t>(n) * zp_stride + (b >> 1)];
        zz[c] = static_cast<float>((b & 1) ? (zb >> 4) : (zb & 0xF));
      }
    }
    float dot[kGemvCols][kGemvMaxM];
    float xsum[kGemvMaxM];
#pragma unroll
    for (int m = 0; m < kGemvMaxM; ++m) {
      xsum[m] = 0.f;
#pragma unroll
      for (int c = 0; c < kGemvCols; ++c) dot[c][m] = 0.f;
    }
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {           // 8 k values per 32-bit word of packed nibbles
      float xs[kGemvMaxM][8];
#pragma unroll
      for (int m = 0; m < kGemvMaxM; ++m) {
        if (m < M) {
          const __nv_bfloat16* xp = x + static_cast<size_t>(m) * ldx + kbase + 8 * wi;
          if (kbase + 8 * wi + 8 <= K) {
            const uint4 q = *reinterpret_cast<const uint4*>(xp);
            float2 f;
            f = unpack_bf16(q.x); xs[m][0] = f.x; xs[m][1] = f.y;
            f = unpack_bf16(q.y); xs[m][2] = f.x; xs[m][3] = f.y;
            f = unpack_bf16(q.z); xs[m][4] = f.x; xs[m][5] = f.y;
            f = unpack_bf16(q.w); xs[m][6] = f.x; xs[m][7] = f.y;
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) xs[m][j] = (kbase + 8 * wi + j < K) ? __bfloat162float(xp[j]) : 0.f;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) xsum[m] += xs[m][j];
        }
      }
#pragma unroll
      for (int c = 0; c < kGemvCols; ++c) {
        const uint32_t word = (wi == 0) ? wq[c].x : (wi == 1) ? wq[c].y : (wi == 2) ? wq[c].z : wq[c].w;
        float f[8];
        nibbles_to_float(word, f);
#pragma unroll
        for (int m = 0; m < kGemvMaxM; ++m) {
          if (m < M) {
#pragma unroll
            for (int i = 0; i < 8; ++i) dot[c][m] += f[i] * xs[m][i];
          }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < kGemvCols; ++c)
#pragma unroll
      for (int m = 0; m < kGemvMaxM; ++m)
        if (m < M) acc[c][m] += sc[c] * (dot[c][m] - zz[c] * xsum[m]);   // sum_k (q - z) s x = s (q.x - z sum x)
  }
#pragma unroll
  for (int c = 0; c < kGemvCols; ++c) {
#pragma unroll
    for (int m = 0; m < kGemvMaxM; ++m) {
      float v = warp_sum(acc[c][m]);
      const int n = n0 + c;
      if (lane == 0 && m < M && n < N) {
        if (bias != nullptr) v += __bfloat162float(bias[n]);
        y[static_cast<size_t>(m) * ldy + n] = __float2bfloat16(v);
      }
    }
  }
}

template <bool SCALES_F32>
__global__ void w4a16_dequant_kernel(const uint8_t* __restrict__ qw, const void* __restrict__ scales,
                                     const uint8_t* __restrict__ zp, __nv_bfloat16* __restrict__ w, int N, int K) {
  const int kb = (K + 31) / 32;
  const int zp_stride = (kb + 1) / 2;
  const size_t total = static_cast<size_t>(N) * kb;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int n = static_cast<int>(i / kb), b = static_cast<int>(i % kb);
    const uint4 w4 = __ldg(reinterpret_cast<const uint4*>(qw + i * 16));
    const float s = load_scale<SCALES_F32>(scales, i);
    float z = 8.f;
    if (zp != nullptr) {
      const uint8_t zb = zp[static_cast<size_t>(n) * zp_stride + (b >> 1)];
      z = static_cast<float>((b & 1) ? (zb >> 4) : (zb & 0xF));
    }
    const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
    __nv_bfloat16* dst = w + static_cast<size_t>(n) * K + b * 32;
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      float f[8];
      nibbles_to_float(words[wi], f);
      if (b * 32 + 8 * wi + 8 <= K && (K % 8) == 0) {
        *reinterpret_cast<uint4*>(dst + 8 * wi) =
            make_uint4(pack_bf16((f[0] - z) * s, (f[1] - z) * s), pack_bf16((f[2] - z) * s, (f[3] - z) * s),
                       pack_bf16((f[4] - z) * s, (f[5] - z) * s), pack_bf16((f[6] - z) * s, (f[7] - z) * s));
      } else {
        for (int j = 0; j < 8; ++j)
          if (b * 32 + 8 * wi + j < K) dst[8 * wi + j] = __float2bfloat16((f[j] - z) * s);
      }
    }
  }
}

}  // namespace ogb

using namespace ogb;

extern "C" int ogb_w4a16_gemv(const void* x, const void* qweight, const void* scales, const void* zp, const void* bias,
                              void* y, int M, int N, int K, int ldx, int ldy, int scales_fp32, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > kGemvMaxM || (ldx % 8) != 0) return -3;
  const int blocks = (N + kGemvWarps * kGemvCols - 1) / (kGemvWarps * kGemvCols);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (scales_fp32)
    w4a16_gemv_kernel<true><<<blocks, kGemvWarps * 32, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const uint8_t*>(qweight), scales, static_cast<const uint8_t*>(zp),
        static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(y), M, N, K, ldx, ldy);
  else
    w4a16_gemv_kernel<false><<<blocks, kGemvWarps * 32, 0, st>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const uint8_t*>(qweight), scales, static_cast<const uint8_t*>(zp),
        static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(y), M, N, K, ldx, ldy);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ogb_w4a16_dequant(const void* qweight, const void* scales, const void* zp, void* w_bf16, int N, int K,
                                 int scales_fp32, void* stream) {
  if (N <= 0 || K <= 0) return 0;
  const size_t total = static_cast<size_t>(N) * ((K + 31) / 32);
  int blocks = static_cast<int>((total + 255) / 256);
  const int cap = ogb_num_sms() * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (scales_fp32)
    w4a16_dequant_kernel<true><<<blocks, 256, 0, st>>>(static_cast<const uint8_t*>(qweight), scales,
                                                      static_cast<const uint8_t*>(zp), static_cast<__nv_bfloat16*>(w_bf16), N, K);
  else
    w4a16_dequant_kernel<false><<<blocks, 256, 0, st>>>(static_cast<const uint8_t*>(qweight), scales,
                                                       static_cast<const uint8_t*>(zp), static_cast<__nv_bfloat16*>(w_bf16), N, K);
  return static_cast<int>(cudaGetLastError());
}
