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
#include <cuda_fp16.h>

#include <algorithm>

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

OGB_DEVICE __half2 as_half2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
OGB_DEVICE uint32_t pack_f16(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
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


// ------------------------------------------------------------------------------------------
// Fused decode-size projection: optional prologue on the activations (RMSNorm, or SiLU(gate)*up), int4
// GEMV, optional residual add in the epilogue.  One launch replaces norm + GEMV, or silu_mul + GEMV +
// residual add (the reference fuses the same neighbours: gate_up+SwiGLU and RMSNorm-prologue GEMVs,
// crates/onnx-runtime-ep-cuda/src/optimizer.rs:27-60).
//
// The kernel is specialised on the row count MT in {1,2,4,8} so the M=1 code stays small: with one
// generic 8-row body the unrolled kernel was dominated by instruction fetch (22-35 us per launch for
// matrices that stream in 1-2 us).  Activations are staged once per CTA in shared memory as bf16 -- after
// the prologue, rounded exactly as the unfused path rounds them -- in chunks of as many values of K as 64 KB hold for the row count (all of K for decode shapes).
// Each warp owns kFusedCols output columns; lanes stride over the 32-weight blocks of a chunk.
//
// Arithmetic: two weights per instruction.  A 32-bit word holds nibbles n0..n7; `(w & 0x000F000F) | 0x64006400` read as
// two fp16 is (1024 + n0, 1024 + n4) and `(w & 0x00F000F0) | 0x54005400` is (64 + n1, 64 + n5) -- no shift needed for
// the odd nibbles -- and the same on w >> 8 gives (n2, n6) and (n3, n7).  One HSUB2 removes the offset and the zero
// point exactly, one HFMA2 multiplies by the matching pair of activations, which are staged as fp16 in the order
// (x0, x4, x1, x5, x2, x6, x3, x7) of every eight.  A block's 32 products are summed in two fp16x2 accumulators (8
// terms each), then go to fp32 for the scale and the sum over blocks, as the reference's fp16 GEMV variants do
// (crates/onnx-runtime-ep-cuda/src/kernels/marlin_gemm.rs:585).  The activations are rounded to bf16 first, exactly as
// the unfused path rounds them; a bf16 value is an fp16 value unless it lies outside +-65504 (clamped) or below 6e-8.
// ------------------------------------------------------------------------------------------
constexpr int kFusedCols = 2;
constexpr int kFusedWarps = 8;

enum : int { kProNone = 0, kProRmsNorm = 1, kProSiluMul = 2 };

struct GemvFusedParams {
  const __nv_bfloat16* x;        // [M, ldx]; kProSiluMul: gate at [0, K), up at [K, 2K)
  const uint8_t* qw;
  const void* scales;
  const uint8_t* zp;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* norm_w;   // kProRmsNorm: [K]
  const __nv_bfloat16* resid;    // optional [M, ldr], added in the epilogue (may alias y)
  __nv_bfloat16* y;              // [M, ldy]
  int M, N, K, ldx, ldy, ldr;
  float eps;
};

// Weights, scale and zero point of one 32-weight block for the C columns starting at n0.
template <int C, bool SCALES_F32>
struct BlockW {
  uint4 wq[C];
  float sc[C], zz[C];
  OGB_DEVICE void load(const GemvFusedParams& p, int n0, int b, int kb, int zp_stride) {
#pragma unroll
    for (int c = 0; c < C; ++c) {
      const int n = min(n0 + c, p.N - 1);
      wq[c] = __ldg(reinterpret_cast<const uint4*>(p.qw + (static_cast<size_t>(n) * kb + b) * 16));
      sc[c] = load_scale<SCALES_F32>(p.scales, static_cast<size_t>(n) * kb + b);
      zz[c] = 8.f;
      if (p.zp != nullptr) {
        const uint8_t zb = p.zp[static_cast<size_t>(n) * zp_stride + (b >> 1)];
        zz[c] = static_cast<float>((b & 1) ? (zb >> 4) : (zb & 0xF));
      }
    }
  }
};

// SPLITK = false: each warp owns kFusedCols columns and walks all of K (wide N, short K).
// SPLITK = true : the CTA owns kSplitCols columns and its 8 warps share the blocks of K, then reduce through
//                 shared memory (narrow N, long K: the down projection), which turns a chain of dependent
//                 loads per lane into one.
constexpr int kSplitCols = 4;

template <int MT, int PRO, bool SCALES_F32, bool SPLITK>
__global__ void __launch_bounds__(kFusedWarps * 32) w4a16_gemv_fused_kernel(const GemvFusedParams p, const int chunk,
                                                                            const int num_tiles) {
  // Persistent over column tiles: a CTA stages the activations once (when all of K fits its shared memory, which is the
  // decode case) and then walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...; the norm statistics, the prologue and the
  // fp16 staging are paid once per CTA instead of once per 16 columns.
  constexpr int C = SPLITK ? kSplitCols : kFusedCols;
  extern __shared__ __align__(16) uint8_t gemv_smem[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(gemv_smem);   // [MT][chunk] fp16 bits in pair order
  __shared__ float rstd_sh[MT];
  __shared__ float red_sh[kFusedWarps][MT];
  __shared__ float part_sh[SPLITK ? kFusedWarps : 1][C][MT];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int K = p.K, N = p.N, M = p.M;
  const int kb = (K + 31) / 32;
  const int zp_stride = (kb + 1) / 2;
  const bool one_chunk = K <= chunk;
  // block index of this lane inside a chunk, and the stride to its next one
  const int j0 = SPLITK ? warp * 32 + lane : lane;
  constexpr int jstep = SPLITK ? kFusedWarps * 32 : 32;
  auto tile_n0 = [&](int tile) { return SPLITK ? tile * C : (tile * kFusedWarps + warp) * C; };

  // The first block's weights do not depend on the activations: request them before the prologue so the
  // DRAM round trip overlaps the norm / staging chain.
  BlockW<C, SCALES_F32> w0;
  const int first_tile = blockIdx.x;
  const bool have_w0 = first_tile < num_tiles && (tile_n0(first_tile) < N) && (j0 < min(kb, chunk / 32));
  if (have_w0) w0.load(p, tile_n0(first_tile), j0, kb, zp_stride);

  if constexpr (PRO == kProRmsNorm) {
    float ss[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) ss[m] = 0.f;
    for (int k = threadIdx.x * 8; k < K; k += blockDim.x * 8) {       // K is a multiple of 8
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        if (m < M) {
          const uint4 q = *reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(m) * p.ldx + k);
          float2 t;
          t = unpack_bf16(q.x); ss[m] += t.x * t.x + t.y * t.y;
          t = unpack_bf16(q.y); ss[m] += t.x * t.x + t.y * t.y;
          t = unpack_bf16(q.z); ss[m] += t.x * t.x + t.y * t.y;
          t = unpack_bf16(q.w); ss[m] += t.x * t.x + t.y * t.y;
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      const float v = warp_sum(ss[m]);
      if (lane == 0) red_sh[warp][m] = v;
    }
    __syncthreads();
    if (threadIdx.x < MT) {
      float t = 0.f;
      for (int w = 0; w < kFusedWarps; ++w) t += red_sh[w][threadIdx.x];
      rstd_sh[threadIdx.x] = rsqrtf(t / static_cast<float>(K) + p.eps);
    }
    __syncthreads();
  }

  for (int tile = first_tile; tile < num_tiles; tile += gridDim.x) {
  const int n0 = tile_n0(tile);
  float acc[C][MT];
#pragma unroll
  for (int c = 0; c < C; ++c)
#pragma unroll
    for (int m = 0; m < MT; ++m) acc[c][m] = 0.f;

  for (int k0 = 0; k0 < K; k0 += chunk) {
    const int klen = min(chunk, K - k0);
    const int klen_pad = (klen + 31) / 32 * 32;
    const bool stage = !one_chunk || tile == first_tile;   // with one chunk the activations stay staged across tiles
    if (stage) {
    if (k0 > 0 || tile != first_tile) __syncthreads();     // every warp is done with what the buffer held
    // stage prologue(x) for this chunk, 8 values per thread per step (K, ldx multiples of 8)
    for (int i = threadIdx.x * 8; i < klen_pad; i += blockDim.x * 8) {
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (m < M && i < klen) {
          const __nv_bfloat16* src = p.x + static_cast<size_t>(m) * p.ldx + k0 + i;
          const uint4 q = *reinterpret_cast<const uint4*>(src);
          if constexpr (PRO == kProNone) {
            o = q;
          } else {
            const uint32_t qa[4] = {q.x, q.y, q.z, q.w};
            uint32_t oa[4];
            uint4 aux;
            if constexpr (PRO == kProSiluMul) aux = *reinterpret_cast<const uint4*>(src + K);
            else aux = *reinterpret_cast<const uint4*>(p.norm_w + k0 + i);
            const uint32_t xa[4] = {aux.x, aux.y, aux.z, aux.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 a = unpack_bf16(qa[e]);
              const float2 bq = unpack_bf16(xa[e]);
              if constexpr (PRO == kProSiluMul) {
                oa[e] = pack_bf16(a.x / (1.f + __expf(-a.x)) * bq.x, a.y / (1.f + __expf(-a.y)) * bq.y);
              } else {
                oa[e] = pack_bf16(a.x * rstd_sh[m] * bq.x, a.y * rstd_sh[m] * bq.y);
              }
            }
            o = make_uint4(oa[0], oa[1], oa[2], oa[3]);
          }
        }
        {
          // bf16 x8 -> fp16 x8 in the pair order of the nibble words
          const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
          float v[8];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 t = unpack_bf16(ow[e]);
            v[2 * e] = fminf(fmaxf(t.x, -65504.f), 65504.f);
            v[2 * e + 1] = fminf(fmaxf(t.y, -65504.f), 65504.f);
          }
          uint4 h;
          h.x = pack_f16(v[0], v[4]); h.y = pack_f16(v[1], v[5]); h.z = pack_f16(v[2], v[6]); h.w = pack_f16(v[3], v[7]);
          *reinterpret_cast<uint4*>(xs + m * chunk + i) = h;
        }
      }
    }
    __syncthreads();
    }
    if (n0 < N) {
      const int b0 = k0 / 32, nb = klen_pad / 32;
      BlockW<C, SCALES_F32> w, wn;
      if (j0 < nb) {
        if (k0 == 0 && tile == first_tile && have_w0) w = w0;
        else w.load(p, n0, b0 + j0, kb, zp_stride);
      }
      for (int j = j0; j < nb; j += jstep) {
        if (j + jstep < nb) wn.load(p, n0, b0 + j + jstep, kb, zp_stride);   // the next block is in flight while this one is used
        __half2 dot[C][MT][2];
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
          for (int m = 0; m < MT; ++m) dot[c][m][0] = dot[c][m][1] = __float2half2_rn(0.f);
        __half2 off_lo[C], off_hi[C];     // what the two magic numbers add, plus the zero point
#pragma unroll
        for (int c = 0; c < C; ++c) {
          off_lo[c] = __float2half2_rn(1024.f + w.zz[c]);
          off_hi[c] = __float2half2_rn(64.f + w.zz[c]);
        }
        const __nv_bfloat16* xb = xs + j * 32;
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          __half2 wv[C][4];
#pragma unroll
          for (int c = 0; c < C; ++c) {
            const uint32_t word = (wi == 0) ? w.wq[c].x : (wi == 1) ? w.wq[c].y : (wi == 2) ? w.wq[c].z : w.wq[c].w;
            const uint32_t w8 = word >> 8;
            wv[c][0] = __hsub2(as_half2((word & 0x000F000Fu) | 0x64006400u), off_lo[c]);
            wv[c][1] = __hsub2(as_half2((word & 0x00F000F0u) | 0x54005400u), off_hi[c]);
            wv[c][2] = __hsub2(as_half2((w8 & 0x000F000Fu) | 0x64006400u), off_lo[c]);
            wv[c][3] = __hsub2(as_half2((w8 & 0x00F000F0u) | 0x54005400u), off_hi[c]);
          }
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            const uint4 q = *reinterpret_cast<const uint4*>(xb + m * chunk + 8 * wi);
            const __half2 xv[4] = {as_half2(q.x), as_half2(q.y), as_half2(q.z), as_half2(q.w)};
#pragma unroll
            for (int c = 0; c < C; ++c)
#pragma unroll
              for (int i = 0; i < 4; ++i) dot[c][m][wi & 1] = __hfma2(wv[c][i], xv[i], dot[c][m][wi & 1]);
          }
        }
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
          for (int m = 0; m < MT; ++m) {
            const float2 d0 = __half22float2(dot[c][m][0]), d1 = __half22float2(dot[c][m][1]);
            acc[c][m] += w.sc[c] * ((d0.x + d0.y) + (d1.x + d1.y));
          }
        w = wn;
      }
    }
  }
  if constexpr (SPLITK) {
#pragma unroll
    for (int c = 0; c < C; ++c)
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float v = warp_sum(acc[c][m]);
        if (lane == 0) part_sh[warp][c][m] = v;
      }
    __syncthreads();
    if (threadIdx.x < C * MT) {
      const int c = threadIdx.x / MT, m = threadIdx.x % MT;
      const int n = n0 + c;
      if (m < M && n < N) {
        float v = 0.f;
        for (int w = 0; w < kFusedWarps; ++w) v += part_sh[w][c][m];
        if (p.bias != nullptr) v += __bfloat162float(p.bias[n]);
        if (p.resid != nullptr) v += __bfloat162float(p.resid[static_cast<size_t>(m) * p.ldr + n]);
        p.y[static_cast<size_t>(m) * p.ldy + n] = __float2bfloat16(v);
      }
    }
    __syncthreads();                                       // part_sh is rewritten by the next tile
  } else {
    if (n0 < N) {
#pragma unroll
    for (int c = 0; c < C; ++c) {
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        float v = warp_sum(acc[c][m]);
        const int n = n0 + c;
        if (lane == 0 && m < M && n < N) {
          if (p.bias != nullptr) v += __bfloat162float(p.bias[n]);
          if (p.resid != nullptr) v += __bfloat162float(p.resid[static_cast<size_t>(m) * p.ldr + n]);
          p.y[static_cast<size_t>(m) * p.ldy + n] = __float2bfloat16(v);
        }
      }
    }
    }
  }
  }
}

template <int MT, int PRO, bool SF32, bool SPLITK>
static int launch_gemv_fused_one(const GemvFusedParams& p, cudaStream_t st) {
  const int per_cta = SPLITK ? kSplitCols : kFusedWarps * kFusedCols;
  const int tiles = (p.N + per_cta - 1) / per_cta;
  // as much of K as 64 KB of shared memory hold for MT rows (a multiple of 32 values): all of it for decode shapes
  const int k_pad = (p.K + 31) / 32 * 32;
  const int chunk = std::min(k_pad, (64 * 1024 / (MT * 2)) / 32 * 32);
  const size_t smem = static_cast<size_t>(MT) * chunk * sizeof(__nv_bfloat16);
  auto kern = w4a16_gemv_fused_kernel<MT, PRO, SF32, SPLITK>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    attr_set = true;
  }
  int ctas_per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas_per_sm, kern, kFusedWarps * 32, smem) != cudaSuccess || ctas_per_sm < 1)
    ctas_per_sm = 1;
  // persistent only when the activations stay staged (one chunk); otherwise one tile per CTA as before
  const int blocks = (p.K <= chunk) ? std::min(tiles, ogb_num_sms() * ctas_per_sm) : tiles;
  kern<<<blocks, kFusedWarps * 32, smem, st>>>(p, chunk, tiles);
  return static_cast<int>(cudaGetLastError());
}

template <int MT, int PRO>
static int launch_gemv_fused(const GemvFusedParams& p, bool scales_fp32, cudaStream_t st) {
  // long K over few columns: share K between the warps of a CTA (see the kernel comment)
  const bool splitk = p.K >= 2048 && p.N <= 4096;
  if (scales_fp32) {
    return splitk ? launch_gemv_fused_one<MT, PRO, true, true>(p, st) : launch_gemv_fused_one<MT, PRO, true, false>(p, st);
  }
  return splitk ? launch_gemv_fused_one<MT, PRO, false, true>(p, st) : launch_gemv_fused_one<MT, PRO, false, false>(p, st);
}

template <int PRO>
static int dispatch_gemv_fused(const GemvFusedParams& p, bool scales_fp32, cudaStream_t st) {
  if (p.M <= 1) return launch_gemv_fused<1, PRO>(p, scales_fp32, st);
  if (p.M <= 2) return launch_gemv_fused<2, PRO>(p, scales_fp32, st);
  if (p.M <= 4) return launch_gemv_fused<4, PRO>(p, scales_fp32, st);
  return launch_gemv_fused<8, PRO>(p, scales_fp32, st);
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

// y[M,N] = prologue(x)[M,K] . dequant(W)^T (+ bias) (+ residual).  prologue: 0 none, 1 RMSNorm with norm_w/eps,
// 2 SiLU(x[:, :K]) * x[:, K:2K].  M <= 8; K and ldx multiples of 8, x 16-byte aligned.  `residual` may alias `y`.
extern "C" int ogb_w4a16_gemv_fused(const void* x, const void* qweight, const void* scales, const void* zp, const void* bias,
                                    const void* norm_w, const void* residual, void* y, int M, int N, int K, int ldx, int ldy,
                                    int ldr, float eps, int prologue, int scales_fp32, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > kGemvMaxM || K <= 0 || (K % 8) != 0 || (ldx % 8) != 0 || (reinterpret_cast<uintptr_t>(x) & 15) != 0) return -3;
  if (prologue == kProRmsNorm && norm_w == nullptr) return -3;
  GemvFusedParams p;
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.qw = static_cast<const uint8_t*>(qweight);
  p.scales = scales;
  p.zp = static_cast<const uint8_t*>(zp);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.norm_w = static_cast<const __nv_bfloat16*>(norm_w);
  p.resid = static_cast<const __nv_bfloat16*>(residual);
  p.y = static_cast<__nv_bfloat16*>(y);
  p.M = M; p.N = N; p.K = K; p.ldx = ldx; p.ldy = ldy; p.ldr = ldr; p.eps = eps;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (prologue) {
    case kProNone: return dispatch_gemv_fused<kProNone>(p, scales_fp32 != 0, st);
    case kProRmsNorm: return dispatch_gemv_fused<kProRmsNorm>(p, scales_fp32 != 0, st);
    case kProSiluMul: return dispatch_gemv_fused<kProSiluMul>(p, scales_fp32 != 0, st);
    default: return -3;
  }
}
