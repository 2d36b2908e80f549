// Device token selection: greedy argmax, the fused temperature -> top-k -> top-p -> min-p ->
// categorical sampler, and greedy speculative verification.
//
// Reference counterparts: greedy_argmax_partials_* / argmax_* (crates/onnx-runtime-ep-cuda/src/
// kernels/device_argmax.rs:10,335-355; crates/onnx-genai-ort/src/device_sampler.rs:126-367) and the
// fused sample_* kernel (device_sampler.rs:369-640), whose filter order (temperature, top-k,
// top-p renormalised over the survivors, min-p, inverse-CDF draw) is kept.  Differences by design:
// the probability mass is carried as 32-bit fixed-point weights w = round(exp(l - max) * 2^30), so
// every threshold search is an exact radix select over integers (no 32-step bisection), the CDF
// walk is a block-wide scan (no serial loop on thread 0), and the result does not depend on the
// summation order.  Ties at a threshold are all kept; the draw walks tokens in index order;
// argmax ties go to the lowest token id (crates/onnx-genai-engine/src/sampling.rs:120-132).
#include "common.cuh"
#include "ogb_kernels.h"

namespace ogb {

constexpr int kSampleThreads = 1024;

struct ArgMax {
  float v;
  int i;
};
OGB_DEVICE ArgMax argmax_better(ArgMax a, ArgMax b) {
  // NaN never wins; lower index wins ties
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
OGB_DEVICE ArgMax warp_argmax(ArgMax a) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = argmax_better(a, b);
  }
  return a;
}
OGB_DEVICE ArgMax block_argmax(ArgMax a, ArgMax* sh /*[32]*/) {
  a = warp_argmax(a);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = a;
  __syncthreads();
  ArgMax r = (lane < nw) ? sh[lane] : ArgMax{-INFINITY, 0x7fffffff};
  r = warp_argmax(r);
  return r;  // identical in every thread
}
OGB_DEVICE ArgMax row_argmax(const __nv_bfloat16* row, int vocab, ArgMax* sh) {
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = __bfloat162float(row[i]);
    if (v > best.v) { best.v = v; best.i = i; }  // strided scan keeps the lowest index per thread on ties
  }
  return block_argmax(best, sh);
}

__global__ void __launch_bounds__(kSampleThreads) argmax_kernel(const __nv_bfloat16* __restrict__ logits,
                                                                 int* __restrict__ out, int vocab, int ld) {
  __shared__ ArgMax sh[32];
  const ArgMax r = row_argmax(logits + static_cast<size_t>(blockIdx.x) * ld, vocab, sh);
  if (threadIdx.x == 0) out[blockIdx.x] = (r.i == 0x7fffffff) ? 0 : r.i;
}

// Block-wide sums over 64-bit integers.
OGB_DEVICE unsigned long long block_sum_u64(unsigned long long v, unsigned long long* sh /*[32]*/) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  unsigned long long r = (lane < nw) ? sh[lane] : 0ull;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  return r;
}

// Radix select over the weights of one row.  Finds the largest threshold T such that
//   measure({ i : w[i] >= T }) >= target
// where measure is the element count (BY_MASS = false, used for top-k) or the summed weight
// (BY_MASS = true, used for top-p).  Only weights >= floor participate.  Weights are < 2^30, so
// five 6-bit digit passes cover them.  Each warp owns a private histogram (64-bit sums kept as
// lo/hi 32-bit words with carry detection, so only native 32-bit shared atomics are used); when
// all 32 lanes of an iteration fall into the same bucket -- the common case, most weights share
// the leading digits -- the warp reduces in registers and lane 0 does one plain add.
constexpr int kDigitBits = 6;
constexpr int kBuckets = 1 << kDigitBits;

struct RadixScratch {
  uint32_t lo[kSampleThreads / 32][kBuckets];
  uint32_t hi[kSampleThreads / 32][kBuckets];
  unsigned long long total[kBuckets];
};

OGB_DEVICE unsigned long long warp_sum_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <bool BY_MASS>
OGB_DEVICE uint32_t radix_threshold(const uint32_t* __restrict__ w, int vocab, uint32_t floor_w,
                                    unsigned long long target, RadixScratch& sc) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t prefix = 0;
  unsigned long long above = 0;  // measure of weights strictly above the current prefix bucket
  for (int shift = 30 - kDigitBits; shift >= 0; shift -= kDigitBits) {
    for (int i = threadIdx.x; i < (kSampleThreads / 32) * kBuckets; i += blockDim.x) {
      (&sc.lo[0][0])[i] = 0u;
      (&sc.hi[0][0])[i] = 0u;
    }
    __syncthreads();
    const uint32_t hi_mask = ~((1u << (shift + kDigitBits)) - 1u);
    const int iters = (vocab + kSampleThreads - 1) / kSampleThreads;
    for (int it = 0; it < iters; ++it) {
      const int i = it * kSampleThreads + threadIdx.x;
      const uint32_t v = (i < vocab) ? w[i] : 0u;
      const bool part = (i < vocab) && v >= floor_w && (v & hi_mask) == prefix;
      const int bucket = part ? static_cast<int>((v >> shift) & (kBuckets - 1)) : kBuckets;
      const unsigned long long val = part ? (BY_MASS ? static_cast<unsigned long long>(v) : 1ull) : 0ull;
      const int b0 = __shfl_sync(0xffffffffu, bucket, 0);
      if (__all_sync(0xffffffffu, bucket == b0)) {
        if (b0 != kBuckets) {
          const unsigned long long tot = warp_sum_u64(val);
          if (lane == 0) {
            const uint32_t add = static_cast<uint32_t>(tot);
            const uint32_t old = sc.lo[warp][b0];
            sc.lo[warp][b0] = old + add;
            sc.hi[warp][b0] += static_cast<uint32_t>(tot >> 32) + ((old + add < old) ? 1u : 0u);
          }
        }
      } else if (part) {
        const uint32_t add = static_cast<uint32_t>(val);
        const uint32_t old = atomicAdd(&sc.lo[warp][bucket], add);
        if (old + add < old) atomicAdd(&sc.hi[warp][bucket], 1u);
      }
      __syncwarp();
    }
    __syncthreads();
    if (threadIdx.x < kBuckets) {
      unsigned long long t = 0;
      for (int wi = 0; wi < kSampleThreads / 32; ++wi)
        t += (static_cast<unsigned long long>(sc.hi[wi][threadIdx.x]) << 32) + sc.lo[wi][threadIdx.x];
      sc.total[threadIdx.x] = t;
    }
    __syncthreads();
    // walk buckets from the top; every thread does the same short walk
    int chosen = 0;
    unsigned long long run = above;
    for (int b = kBuckets - 1; b >= 0; --b) {
      const unsigned long long h = sc.total[b];
      if (run + h >= target) { chosen = b; break; }
      run += h;
    }
    above = run;
    prefix |= static_cast<uint32_t>(chosen) << shift;
    __syncthreads();
  }
  return prefix < floor_w ? floor_w : prefix;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const __nv_bfloat16* __restrict__ logits, int* __restrict__ out, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ uniform, uint32_t* __restrict__ work, int vocab, int ld) {
  __shared__ ArgMax sh_arg[32];
  __shared__ unsigned long long sh_sum[32];
  __shared__ RadixScratch sc;
  __shared__ unsigned long long sh_scan[kSampleThreads / 32];
  __shared__ int sh_pick;
  const int rowi = blockIdx.x;
  const __nv_bfloat16* row = logits + static_cast<size_t>(rowi) * ld;
  const ArgMax best = row_argmax(row, vocab, sh_arg);
  const float temp = temperature[rowi];
  if (!(temp > 0.f) || best.i == 0x7fffffff) {
    if (threadIdx.x == 0) out[rowi] = (best.i == 0x7fffffff) ? 0 : best.i;
    return;
  }
  uint32_t* w = work + static_cast<size_t>(rowi) * vocab;
  const float inv_t = 1.f / temp;
  unsigned long long local = 0;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float l = __bfloat162float(row[i]);
    float e = __expf((l - best.v) * inv_t);   // in (0, 1]; NaN logits get weight 0
    if (!(e >= 0.f)) e = 0.f;
    uint32_t q = static_cast<uint32_t>(e * 1073741824.f + 0.5f);
    if (q > 1073741823u) q = 1073741823u;
    w[i] = q;
    local += q;
  }
  __syncthreads();
  unsigned long long total = block_sum_u64(local, sh_sum);
  uint32_t thr = 1;  // zero-weight tokens never survive

  const int k = top_k[rowi];
  if (k > 0 && k < vocab) {
    thr = radix_threshold<false>(w, vocab, thr, static_cast<unsigned long long>(k), sc);
    unsigned long long s = 0;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) { const uint32_t v = w[i]; s += (v >= thr) ? v : 0u; }
    total = block_sum_u64(s, sh_sum);
  }
  const float p = top_p[rowi];
  if (p > 0.f && p < 1.f) {
    // smallest set of largest weights whose mass reaches p * total (mass renormalised over survivors)
    unsigned long long target = static_cast<unsigned long long>(static_cast<double>(total) * static_cast<double>(p));
    if (target < 1ull) target = 1ull;
    thr = radix_threshold<true>(w, vocab, thr, target, sc);
  }
  const float mp = min_p[rowi];
  if (mp > 0.f) {
    const uint32_t floor_mp = static_cast<uint32_t>(fminf(mp, 1.f) * 1073741824.f);
    if (floor_mp > thr) thr = floor_mp;
  }
  // final mass per warp-contiguous range, then the inverse-CDF draw in token-index order
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per_warp = ((vocab + 31) / 32 + 31) / 32 * 32;  // range length per warp, multiple of 32
  const int wbegin = warp * per_warp;
  const int wend = min(vocab, wbegin + per_warp);
  unsigned long long mine = 0;
  for (int i = wbegin + lane; i < wend; i += 32) { const uint32_t v = w[i]; mine += (v >= thr) ? v : 0u; }
  mine = warp_sum_u64(mine);
  if (lane == 0) sh_scan[warp] = mine;
  if (threadIdx.x == 0) sh_pick = -1;
  __syncthreads();
  if (warp == 0) {
    unsigned long long v = sh_scan[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      unsigned long long n = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += n;
    }
    sh_scan[lane] = v;  // inclusive prefix of warp totals
  }
  __syncthreads();
  const unsigned long long final_total = sh_scan[kSampleThreads / 32 - 1];
  float u = uniform[rowi];
  u = fminf(fmaxf(u, 0.f), 0.99999994f);
  unsigned long long target = static_cast<unsigned long long>(static_cast<double>(u) * static_cast<double>(final_total));
  if (final_total > 0 && target >= final_total) target = final_total - 1;
  const unsigned long long w_incl = sh_scan[warp];
  const unsigned long long w_excl = w_incl - mine;
  if (final_total > 0 && mine > 0 && target >= w_excl && target < w_incl) {
    // this warp owns the draw: walk its range 32 tokens at a time with a warp scan
    unsigned long long run = w_excl;
    for (int base = wbegin; base < wend; base += 32) {
      const int i = base + lane;
      const uint32_t v0 = (i < wend) ? w[i] : 0u;
      const unsigned long long v = (v0 >= thr) ? v0 : 0u;
      unsigned long long incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        unsigned long long n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      const bool hit = v > 0 && target >= run + incl - v && target < run + incl;
      const unsigned ball = __ballot_sync(0xffffffffu, hit);
      if (ball) {
        if (lane == __ffs(ball) - 1) sh_pick = i;
        break;
      }
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) out[rowi] = (sh_pick >= 0) ? sh_pick : best.i;
}

// ------------------------------------------------------------------------------------------
// Vectorised variant of sample_kernel: identical arithmetic and results, but every pass over the
// row uses 16-byte loads (8 logits or 4 weights per thread per iteration), so a pass costs ~4x fewer
// dependent memory round trips.  Requires vocab % 8 == 0, ld % 8 == 0 and 16-byte aligned rows.
// ------------------------------------------------------------------------------------------
template <bool BY_MASS>
OGB_DEVICE uint32_t radix_threshold_vec(const uint32_t* __restrict__ w, int vocab, uint32_t floor_w,
                                        unsigned long long target, RadixScratch& sc) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t prefix = 0;
  unsigned long long above = 0;
  const int nvec = vocab / 4;
  const int iters = (nvec + kSampleThreads - 1) / kSampleThreads;
  for (int shift = 30 - kDigitBits; shift >= 0; shift -= kDigitBits) {
    for (int i = threadIdx.x; i < (kSampleThreads / 32) * kBuckets; i += blockDim.x) {
      (&sc.lo[0][0])[i] = 0u;
      (&sc.hi[0][0])[i] = 0u;
    }
    __syncthreads();
    const uint32_t hi_mask = ~((1u << (shift + kDigitBits)) - 1u);
    for (int it = 0; it < iters; ++it) {
      const int vi = it * kSampleThreads + threadIdx.x;
      uint4 q = make_uint4(0, 0, 0, 0);
      if (vi < nvec) q = reinterpret_cast<const uint4*>(w)[vi];
      const uint32_t vals[4] = {q.x, q.y, q.z, q.w};
      bool parts[4];
      bool any = false;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        parts[e] = (vi < nvec) && vals[e] >= floor_w && (vals[e] & hi_mask) == prefix;
        any |= parts[e];
      }
      if (!__any_sync(0xffffffffu, any)) continue;   // nothing in this stripe belongs to the current prefix
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint32_t v = vals[e];
        const bool part = parts[e];
        const int bucket = part ? static_cast<int>((v >> shift) & (kBuckets - 1)) : kBuckets;
        const unsigned long long val = part ? (BY_MASS ? static_cast<unsigned long long>(v) : 1ull) : 0ull;
        const int b0 = __shfl_sync(0xffffffffu, bucket, 0);
        if (__all_sync(0xffffffffu, bucket == b0)) {
          if (b0 != kBuckets) {
            const unsigned long long tot = warp_sum_u64(val);
            if (lane == 0) {
              const uint32_t add = static_cast<uint32_t>(tot);
              const uint32_t old = sc.lo[warp][b0];
              sc.lo[warp][b0] = old + add;
              sc.hi[warp][b0] += static_cast<uint32_t>(tot >> 32) + ((old + add < old) ? 1u : 0u);
            }
          }
        } else if (part) {
          const uint32_t add = static_cast<uint32_t>(val);
          const uint32_t old = atomicAdd(&sc.lo[warp][bucket], add);
          if (old + add < old) atomicAdd(&sc.hi[warp][bucket], 1u);
        }
        __syncwarp();
      }
    }
    __syncthreads();
    if (threadIdx.x < kBuckets) {
      unsigned long long t = 0;
      for (int wi = 0; wi < kSampleThreads / 32; ++wi)
        t += (static_cast<unsigned long long>(sc.hi[wi][threadIdx.x]) << 32) + sc.lo[wi][threadIdx.x];
      sc.total[threadIdx.x] = t;
    }
    __syncthreads();
    int chosen = 0;
    unsigned long long run = above;
    for (int b = kBuckets - 1; b >= 0; --b) {
      const unsigned long long h = sc.total[b];
      if (run + h >= target) { chosen = b; break; }
      run += h;
    }
    above = run;
    prefix |= static_cast<uint32_t>(chosen) << shift;
    __syncthreads();
  }
  return prefix < floor_w ? floor_w : prefix;
}

__global__ void __launch_bounds__(kSampleThreads, 2)
sample_kernel_vec(const __nv_bfloat16* __restrict__ logits, int* __restrict__ out, const float* __restrict__ temperature,
                  const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
                  const float* __restrict__ uniform, uint32_t* __restrict__ work, int vocab, int ld) {
  __shared__ ArgMax sh_arg[32];
  __shared__ unsigned long long sh_sum[32];
  __shared__ RadixScratch sc;
  __shared__ unsigned long long sh_scan[kSampleThreads / 32];
  __shared__ int sh_pick;
  const int rowi = blockIdx.x;
  const __nv_bfloat16* row = logits + static_cast<size_t>(rowi) * ld;
  // argmax with 8 logits per load; within a thread indices ascend, so ">" keeps the lowest index on ties
  ArgMax best{-INFINITY, 0x7fffffff};
  const int nvec8 = vocab / 8;
  for (int vi = threadIdx.x; vi < nvec8; vi += blockDim.x) {
    const uint4 q = reinterpret_cast<const uint4*>(row)[vi];
    const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16(ws[e]);
      if (f.x > best.v) { best.v = f.x; best.i = vi * 8 + 2 * e; }
      if (f.y > best.v) { best.v = f.y; best.i = vi * 8 + 2 * e + 1; }
    }
  }
  best = block_argmax(best, sh_arg);
  const float temp = temperature[rowi];
  if (!(temp > 0.f) || best.i == 0x7fffffff) {
    if (threadIdx.x == 0) out[rowi] = (best.i == 0x7fffffff) ? 0 : best.i;
    return;
  }
  uint32_t* w = work + static_cast<size_t>(rowi) * vocab;
  const float inv_t = 1.f / temp;
  unsigned long long local = 0;
  for (int vi = threadIdx.x; vi < nvec8; vi += blockDim.x) {
    const uint4 q = reinterpret_cast<const uint4*>(row)[vi];
    const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
    uint32_t o[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16(ws[e]);
      float e0 = __expf((f.x - best.v) * inv_t), e1 = __expf((f.y - best.v) * inv_t);
      if (!(e0 >= 0.f)) e0 = 0.f;
      if (!(e1 >= 0.f)) e1 = 0.f;
      uint32_t q0 = static_cast<uint32_t>(e0 * 1073741824.f + 0.5f), q1 = static_cast<uint32_t>(e1 * 1073741824.f + 0.5f);
      if (q0 > 1073741823u) q0 = 1073741823u;
      if (q1 > 1073741823u) q1 = 1073741823u;
      o[2 * e] = q0;
      o[2 * e + 1] = q1;
      local += q0;
      local += q1;
    }
    reinterpret_cast<uint4*>(w)[2 * vi] = make_uint4(o[0], o[1], o[2], o[3]);
    reinterpret_cast<uint4*>(w)[2 * vi + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
  __syncthreads();
  unsigned long long total = block_sum_u64(local, sh_sum);
  uint32_t thr = 1;
  const int nvec4 = vocab / 4;
  const int k = top_k[rowi];
  if (k > 0 && k < vocab) {
    thr = radix_threshold_vec<false>(w, vocab, thr, static_cast<unsigned long long>(k), sc);
    unsigned long long s = 0;
    for (int vi = threadIdx.x; vi < nvec4; vi += blockDim.x) {
      const uint4 q = reinterpret_cast<const uint4*>(w)[vi];
      s += (q.x >= thr ? q.x : 0u);
      s += (q.y >= thr ? q.y : 0u);
      s += (q.z >= thr ? q.z : 0u);
      s += (q.w >= thr ? q.w : 0u);
    }
    total = block_sum_u64(s, sh_sum);
  }
  const float p = top_p[rowi];
  if (p > 0.f && p < 1.f) {
    unsigned long long target = static_cast<unsigned long long>(static_cast<double>(total) * static_cast<double>(p));
    if (target < 1ull) target = 1ull;
    thr = radix_threshold_vec<true>(w, vocab, thr, target, sc);
  }
  const float mp = min_p[rowi];
  if (mp > 0.f) {
    const uint32_t floor_mp = static_cast<uint32_t>(fminf(mp, 1.f) * 1073741824.f);
    if (floor_mp > thr) thr = floor_mp;
  }
  // identical partition of the row into 32 warp-contiguous ranges as the scalar kernel
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per_warp = ((vocab + 31) / 32 + 31) / 32 * 32;
  const int wbegin = warp * per_warp;
  const int wend = min(vocab, wbegin + per_warp);
  unsigned long long mine = 0;
  for (int i = wbegin + 4 * lane; i < wend; i += 128) {   // per_warp and vocab are multiples of 4
    const uint4 q = *reinterpret_cast<const uint4*>(w + i);
    mine += (q.x >= thr ? q.x : 0u);
    mine += (q.y >= thr ? q.y : 0u);
    mine += (q.z >= thr ? q.z : 0u);
    mine += (q.w >= thr ? q.w : 0u);
  }
  mine = warp_sum_u64(mine);
  if (lane == 0) sh_scan[warp] = mine;
  if (threadIdx.x == 0) sh_pick = -1;
  __syncthreads();
  if (warp == 0) {
    unsigned long long v = sh_scan[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      unsigned long long n = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += n;
    }
    sh_scan[lane] = v;
  }
  __syncthreads();
  const unsigned long long final_total = sh_scan[kSampleThreads / 32 - 1];
  float u = uniform[rowi];
  u = fminf(fmaxf(u, 0.f), 0.99999994f);
  unsigned long long target = static_cast<unsigned long long>(static_cast<double>(u) * static_cast<double>(final_total));
  if (final_total > 0 && target >= final_total) target = final_total - 1;
  const unsigned long long w_incl = sh_scan[warp];
  const unsigned long long w_excl = w_incl - mine;
  if (final_total > 0 && mine > 0 && target >= w_excl && target < w_incl) {
    unsigned long long run = w_excl;
    for (int base = wbegin; base < wend; base += 32) {
      const int i = base + lane;
      const uint32_t v0 = (i < wend) ? w[i] : 0u;
      const unsigned long long v = (v0 >= thr) ? v0 : 0u;
      unsigned long long incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        unsigned long long n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      const bool hit = v > 0 && target >= run + incl - v && target < run + incl;
      const unsigned ball = __ballot_sync(0xffffffffu, hit);
      if (ball) {
        if (lane == __ffs(ball) - 1) sh_pick = i;
        break;
      }
      run += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) out[rowi] = (sh_pick >= 0) ? sh_pick : best.i;
}

// One CTA per sequence: rows [seq*(k+1), seq*(k+1)+k] of the target logits.  Row j predicts the
// token after draft position j-1 (row 0 follows the last committed token).  accept_len = length of
// the longest prefix with draft[j] == argmax(row j); out_tokens[seq, 0..accept_len] = the accepted
// draft tokens followed by the correction / bonus token argmax(row accept_len).
__global__ void __launch_bounds__(kSampleThreads)
spec_verify_greedy_kernel(const __nv_bfloat16* __restrict__ logits, const int* __restrict__ draft, int* __restrict__ accept_len,
                          int* __restrict__ out_tokens, int k, int vocab, int ld) {
  __shared__ ArgMax sh[32];
  __shared__ int best_tok[17];
  const int seq = blockIdx.x;
  for (int j = 0; j <= k; ++j) {
    const ArgMax r = row_argmax(logits + (static_cast<size_t>(seq) * (k + 1) + j) * ld, vocab, sh);
    if (threadIdx.x == 0) best_tok[j] = (r.i == 0x7fffffff) ? 0 : r.i;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    int a = 0;
    while (a < k && draft[seq * k + a] == best_tok[a]) ++a;
    accept_len[seq] = a;
    for (int j = 0; j < a; ++j) out_tokens[seq * (k + 1) + j] = draft[seq * k + j];
    out_tokens[seq * (k + 1) + a] = best_tok[a];
    for (int j = a + 1; j <= k; ++j) out_tokens[seq * (k + 1) + j] = -1;
  }
}

}  // namespace ogb

using namespace ogb;

// ------------------------------------------------------------------------------------------
// Split argmax for few rows: with one CTA per row a batch-1 decode step spends 70 us scanning 152 k logits
// with 2-byte loads.  Here `parts` CTAs share a row, each scans its slice with 16-byte loads and folds its
// best (value, index) into a per-row 64-bit key with atomicMax: the high word is the float in an order-
// preserving integer form, the low word ~index, so the largest value wins and ties go to the lowest index.
// The last CTA of a row to finish decodes the key into the token id and resets the row's words.  The words
// live in the library image, so launches on one device must not overlap (the engine has one stream).
// ------------------------------------------------------------------------------------------
constexpr int kArgmaxMaxRows = 1024;
static __device__ unsigned long long g_argmax_key[kArgmaxMaxRows];
static __device__ unsigned int g_argmax_done[kArgmaxMaxRows];

__global__ void __launch_bounds__(kSampleThreads) argmax_split_kernel(const __nv_bfloat16* __restrict__ logits,
                                                                       int* __restrict__ out, int vocab, int ld, int per_part) {
  __shared__ ArgMax sh[32];
  const int row = blockIdx.y, part = blockIdx.x;
  const __nv_bfloat16* r = logits + static_cast<size_t>(row) * ld;
  const int begin = part * per_part;                       // per_part is a multiple of 8
  const int end = min(vocab, begin + per_part);
  ArgMax best{-INFINITY, 0x7fffffff};
  const int nvec = (end - begin) / 8;
  for (int vi = threadIdx.x; vi < nvec; vi += blockDim.x) {
    const uint4 q = *reinterpret_cast<const uint4*>(r + begin + vi * 8);
    const uint32_t ws[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = unpack_bf16(ws[e]);
      if (f.x > best.v) { best.v = f.x; best.i = begin + vi * 8 + 2 * e; }
      if (f.y > best.v) { best.v = f.y; best.i = begin + vi * 8 + 2 * e + 1; }
    }
  }
  for (int i = begin + nvec * 8 + threadIdx.x; i < end; i += blockDim.x) {
    const float v = __bfloat162float(r[i]);
    if (v > best.v) { best.v = v; best.i = i; }
  }
  best = block_argmax(best, sh);
  if (threadIdx.x == 0) {
    if (best.i != 0x7fffffff) {
      const uint32_t bits = __float_as_uint(best.v);
      const uint32_t ord = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
      atomicMax(&g_argmax_key[row], (static_cast<unsigned long long>(ord) << 32) | (0xffffffffu - static_cast<uint32_t>(best.i)));
    }
    __threadfence();
    if (atomicAdd(&g_argmax_done[row], 1u) == gridDim.x - 1) {
      const unsigned long long key = atomicExch(&g_argmax_key[row], 0ull);
      out[row] = (key == 0ull) ? 0 : static_cast<int>(0xffffffffu - static_cast<uint32_t>(key & 0xffffffffull));
      g_argmax_done[row] = 0;
    }
  }
}

extern "C" int ogb_argmax_bf16(const void* logits, int* out_tokens, int rows, int vocab, int ld, void* stream) {
  if (rows <= 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool vec_ok = (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  int parts = (2 * ogb_num_sms() + rows - 1) / rows;
  if (parts > 16) parts = 16;
  if (parts > vocab / 8192) parts = vocab / 8192;
  if (vec_ok && parts >= 2 && rows <= kArgmaxMaxRows) {
    const int per_part = ((vocab + parts - 1) / parts + 7) / 8 * 8;
    argmax_split_kernel<<<dim3(parts, rows), kSampleThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), out_tokens,
                                                                     vocab, ld, per_part);
    return static_cast<int>(cudaGetLastError());
  }
  argmax_kernel<<<rows, kSampleThreads, 0, st>>>(static_cast<const __nv_bfloat16*>(logits), out_tokens, vocab, ld);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ogb_sample_bf16(const void* logits, int* out_tokens, const float* temperature, const int* top_k,
                               const float* top_p, const float* min_p, const float* uniform, uint32_t* work, int rows,
                               int vocab, int ld, void* stream) {
  if (rows <= 0) return 0;
  if (work == nullptr) return -4;
  const bool vec_ok = (vocab % 8 == 0) && (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0) &&
                      ((reinterpret_cast<uintptr_t>(work) & 15) == 0);
  if (vec_ok) {
    sample_kernel_vec<<<rows, kSampleThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(logits), out_tokens, temperature, top_k, top_p, min_p, uniform, work, vocab, ld);
    return static_cast<int>(cudaGetLastError());
  }
  sample_kernel<<<rows, kSampleThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), out_tokens, temperature, top_k, top_p, min_p, uniform, work, vocab, ld);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ogb_spec_verify_greedy(const void* logits, const int* draft_tokens, int* accept_len, int* out_tokens,
                                      int num_seqs, int k, int vocab, int ld, void* stream) {
  if (num_seqs <= 0) return 0;
  if (k < 0 || k > 16) return -3;
  spec_verify_greedy_kernel<<<num_seqs, kSampleThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), draft_tokens, accept_len, out_tokens, k, vocab, ld);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------------------------------
// Sampler entry point for callers that cannot allocate device memory (see ogb_no_alloc.h).
// ------------------------------------------------------------------------------------------
namespace ogb {
constexpr int kNoAllocMaxRows = 4;
constexpr int kNoAllocMaxVocab = 262144;
// Work area of the fused sampler (one 32-bit weight per logit).  It lives in the library image, so
// every GPU that loads the library carries these 4 MiB until the process exits.
static __device__ __align__(256) uint32_t g_no_alloc_sample_work[kNoAllocMaxRows * kNoAllocMaxVocab];
constexpr int kNoAllocMaxDevices = 64;
static uint32_t* g_no_alloc_work_ptr[kNoAllocMaxDevices] = {};
}  // namespace ogb

extern "C" int ogb_sample_bf16_no_alloc(const void* logits, int* out_tokens, const float* temperature, const int* top_k,
                                        const float* top_p, const float* min_p, const float* uniform, int rows, int vocab,
                                        int ld, void* stream) {
  if (rows <= 0) return 0;
  if (rows > kNoAllocMaxRows || vocab <= 0 || vocab > kNoAllocMaxVocab || ld < vocab) return -3;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kNoAllocMaxDevices) return -4;
  if (g_no_alloc_work_ptr[dev] == nullptr) {
    // In host code the array's name is only a handle; the device address has to be looked up, once
    // per device, with that device current.
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_no_alloc_sample_work);
    if (e != cudaSuccess) return static_cast<int>(e);
    g_no_alloc_work_ptr[dev] = static_cast<uint32_t*>(p);
  }
  // same choice as ogb_sample_bf16: the vectorised kernel when rows are 16-byte aligned (the array itself is
  // 256-byte aligned and a row of it starts at a multiple of vocab * 4 bytes); both kernels pick identical tokens
  const bool vec_ok = (vocab % 8 == 0) && (ld % 8 == 0) && ((reinterpret_cast<uintptr_t>(logits) & 15) == 0);
  if (vec_ok) {
    sample_kernel_vec<<<rows, kSampleThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(logits), out_tokens, temperature, top_k, top_p, min_p, uniform,
        g_no_alloc_work_ptr[dev], vocab, ld);
  } else {
    sample_kernel<<<rows, kSampleThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(logits), out_tokens, temperature, top_k, top_p, min_p, uniform,
        g_no_alloc_work_ptr[dev], vocab, ld);
  }
  return static_cast<int>(cudaGetLastError());
}
