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
// (BY_MASS = true, used for top-p).  Only weights >= floor participate.  Four 8-bit passes.
template <bool BY_MASS>
OGB_DEVICE uint32_t radix_threshold(const uint32_t* __restrict__ w, int vocab, uint32_t floor_w,
                                    unsigned long long target, unsigned long long* hist /*[256]*/) {
  uint32_t prefix = 0;
  unsigned long long above = 0;  // measure of weights strictly above the current prefix bucket
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0ull;
    __syncthreads();
    const uint32_t hi_mask = (shift == 24) ? 0u : (0xffffffffu << (shift + 8));
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      const uint32_t v = w[i];
      if (v >= floor_w && (v & hi_mask) == prefix) {
        atomicAdd(&hist[(v >> shift) & 0xff], BY_MASS ? static_cast<unsigned long long>(v) : 1ull);
      }
    }
    __syncthreads();
    // walk buckets from the top; every thread does the same 256-step walk (cheap, deterministic)
    int chosen = 0;
    unsigned long long run = above;
    for (int b = 255; b >= 0; --b) {
      const unsigned long long h = hist[b];
      if (run + h >= target) { chosen = b; break; }
      run += h;
      if (b == 0) chosen = 0;
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
  __shared__ unsigned long long hist[256];
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
    const uint32_t q = static_cast<uint32_t>(e * 1073741824.f + 0.5f);
    w[i] = q;
    local += q;
  }
  __syncthreads();
  unsigned long long total = block_sum_u64(local, sh_sum);
  uint32_t thr = 1;  // zero-weight tokens never survive

  const int k = top_k[rowi];
  if (k > 0 && k < vocab) {
    thr = radix_threshold<false>(w, vocab, thr, static_cast<unsigned long long>(k), hist);
    unsigned long long s = 0;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) s += (w[i] >= thr) ? w[i] : 0u;
    total = block_sum_u64(s, sh_sum);
  }
  const float p = top_p[rowi];
  if (p > 0.f && p < 1.f) {
    // smallest set of largest weights whose mass reaches p * total (mass renormalised over survivors)
    unsigned long long target = static_cast<unsigned long long>(static_cast<double>(total) * static_cast<double>(p));
    if (target < 1ull) target = 1ull;
    thr = radix_threshold<true>(w, vocab, thr, target, hist);
  }
  const float mp = min_p[rowi];
  if (mp > 0.f) {
    // the maximum weight is always 2^30 (the argmax token)
    const uint32_t floor_mp = static_cast<uint32_t>(fminf(mp, 1.f) * 1073741824.f);
    if (floor_mp > thr) thr = floor_mp;
  }
  // final mass and inverse-CDF draw in token-index order
  const int per = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = threadIdx.x * per;
  const int end = min(vocab, begin + per);
  unsigned long long mine = 0;
  for (int i = begin; i < end; ++i) mine += (w[i] >= thr) ? w[i] : 0u;
  // inclusive scan across threads
  unsigned long long incl = mine;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    unsigned long long n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) sh_scan[warp] = incl;
  if (threadIdx.x == 0) sh_pick = -1;
  __syncthreads();
  if (warp == 0) {
    unsigned long long v = (lane < kSampleThreads / 32) ? sh_scan[lane] : 0ull;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      unsigned long long n = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += n;
    }
    if (lane < kSampleThreads / 32) sh_scan[lane] = v;  // inclusive prefix of warp totals
  }
  __syncthreads();
  const unsigned long long warp_excl = (warp == 0) ? 0ull : sh_scan[warp - 1];
  const unsigned long long final_total = sh_scan[kSampleThreads / 32 - 1];
  const unsigned long long my_incl = warp_excl + incl;
  const unsigned long long my_excl = my_incl - mine;
  float u = uniform[rowi];
  u = fminf(fmaxf(u, 0.f), 0.99999994f);
  unsigned long long target = static_cast<unsigned long long>(static_cast<double>(u) * static_cast<double>(final_total));
  if (final_total > 0 && target >= final_total) target = final_total - 1;
  if (final_total > 0 && mine > 0 && target >= my_excl && target < my_incl) {
    unsigned long long run = my_excl;
    int pick = begin;
    for (int i = begin; i < end; ++i) {
      const uint32_t v = (w[i] >= thr) ? w[i] : 0u;
      if (v > 0 && target < run + v) { pick = i; break; }
      run += v;
    }
    sh_pick = pick;
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

extern "C" int ogb_argmax_bf16(const void* logits, int* out_tokens, int rows, int vocab, int ld, void* stream) {
  if (rows <= 0) return 0;
  argmax_kernel<<<rows, kSampleThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), out_tokens, vocab, ld);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ogb_sample_bf16(const void* logits, int* out_tokens, const float* temperature, const int* top_k,
                               const float* top_p, const float* min_p, const float* uniform, uint32_t* work, int rows,
                               int vocab, int ld, void* stream) {
  if (rows <= 0) return 0;
  if (work == nullptr) return -4;
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
