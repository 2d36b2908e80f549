// Mixture-of-experts routing and data movement around the grouped tcgen05 GEMM.
//
// Reference counterparts: qmoe_route (one CTA per token row, k rounds of block-wide argmax on
// total-order keys, crates/onnx-runtime-ep-cuda/src/kernels/qmoe.rs:56-120), qmoe_group_{init,count,
// prefix,assign} and qmoe_gather_* (qmoe_grouping.rs), qmoe_combine_* (qmoe.rs:22-47).  Router
// semantics follow the metadata's MixtureOfExpertsSpec (score_function softmax, selection top_k,
// normalize_weights; crates/onnx-genai-metadata/src/schema/hardware.rs:64-98).
//   moe_route_topk   one warp per token: softmax over the expert logits, k rounds of warp argmax with
//                    lowest-index tie break, optional renormalisation over the chosen k
//   moe_count / moe_plan / moe_assign   routes -> per-expert counts -> offsets, the 128-row tile table
//                    the grouped GEMM walks, and each route's row in the expert-sorted order
//   moe_gather_rows  activations copied into expert-sorted order
//   moe_combine      out[t] (+)= sum_j w[t,j] * y[row of route (t,j)], j in fixed order (deterministic)
// All routing state stays on the device; nothing here synchronises with the host.
#include "common.cuh"
#include "ogb_kernels.h"

namespace ogb {

constexpr int kMaxExperts = 256;

__global__ void moe_route_topk_kernel(const __nv_bfloat16* __restrict__ logits, int* __restrict__ topk_ids,
                                      float* __restrict__ topk_w, int tokens, int experts, int k, int renormalize, int ld) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  constexpr int PER = kMaxExperts / 32;
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = i * 32 + lane;
    v[i] = (e < experts) ? __bfloat162float(logits[static_cast<size_t>(warp) * ld + e]) : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = (i * 32 + lane < experts) ? __expf(v[i] - mx) : 0.f;
    sum += v[i];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  float chosen_sum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int r = 0; r < k; ++r) {
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = i * 32 + lane;
      if (e < experts && (v[i] > best || (v[i] == best && e < best_e))) { best = v[i]; best_e = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if (lane == r) { my_w = best * inv; my_id = best_e; }
    chosen_sum += best * inv;
    if ((best_e & 31) == lane) v[best_e >> 5] = -1.f;   // remove the winner
  }
  if (lane < k) {
    topk_ids[static_cast<size_t>(warp) * k + lane] = my_id;
    topk_w[static_cast<size_t>(warp) * k + lane] = renormalize ? my_w / chosen_sum : my_w;
  }
}

// counts[e] = routes to local expert e (ids outside [e0, e0 + experts) are other ranks' experts)
__global__ void moe_count_kernel(const int* __restrict__ topk_ids, int* __restrict__ counts, int routes, int e0, int experts) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= routes) return;
  const int e = topk_ids[i] - e0;
  if (e >= 0 && e < experts) atomicAdd(&counts[e], 1);
}

// One CTA: offsets[e] (exclusive prefix), tile table {e, first row, end row, 0} per 128 rows, number of
// tiles, and cursor reset.  meta = {num_mtiles, total_rows}.
__global__ void moe_plan_kernel(const int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ cursor,
                                int* __restrict__ tile_tab, int* __restrict__ meta, int experts, int max_mtiles) {
  __shared__ int s_off[kMaxExperts + 1];
  __shared__ int s_tile[kMaxExperts + 1];
  if (threadIdx.x == 0) {
    int o = 0, t = 0;
    for (int e = 0; e < experts; ++e) {
      s_off[e] = o;
      s_tile[e] = t;
      o += counts[e];
      t += (counts[e] + 127) / 128;
    }
    s_off[experts] = o;
    s_tile[experts] = t;
    meta[0] = min(t, max_mtiles);
    meta[1] = o;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    offsets[e] = s_off[e];
    cursor[e] = 0;
    const int end = s_off[e + 1];
    int t = s_tile[e];
    for (int r = s_off[e]; r < end && t < max_mtiles; r += 128, ++t) {
      tile_tab[4 * t] = e;
      tile_tab[4 * t + 1] = r;
      tile_tab[4 * t + 2] = end;
      tile_tab[4 * t + 3] = 0;
    }
  }
  if (threadIdx.x == 0) offsets[experts] = s_off[experts];
}

__global__ void moe_assign_kernel(const int* __restrict__ topk_ids, const int* __restrict__ offsets, int* __restrict__ cursor,
                                  int* __restrict__ sorted_route, int* __restrict__ route_pos, int routes, int e0, int experts) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= routes) return;
  const int e = topk_ids[i] - e0;
  if (e < 0 || e >= experts) { route_pos[i] = -1; return; }
  const int pos = offsets[e] + atomicAdd(&cursor[e], 1);
  sorted_route[pos] = i;
  route_pos[i] = pos;
}

__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted_route,
                                       const int* __restrict__ meta, __nv_bfloat16* __restrict__ xs, int k, int hidden) {
  const int pos = blockIdx.x;
  if (pos >= meta[1]) return;
  const int token = sorted_route[pos] / k;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(token) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(pos) * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = src[i];
}

__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ ys, const int* __restrict__ route_pos,
                                   const float* __restrict__ topk_w, __nv_bfloat16* __restrict__ out, int k, int hidden,
                                   int accumulate) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (accumulate) {
      const uint4 v = reinterpret_cast<const uint4*>(out + static_cast<size_t>(t) * hidden)[i];
      float2 f;
      f = unpack_bf16(v.x); acc[0] = f.x; acc[1] = f.y;
      f = unpack_bf16(v.y); acc[2] = f.x; acc[3] = f.y;
      f = unpack_bf16(v.z); acc[4] = f.x; acc[5] = f.y;
      f = unpack_bf16(v.w); acc[6] = f.x; acc[7] = f.y;
    }
    for (int j = 0; j < k; ++j) {
      const int pos = route_pos[static_cast<size_t>(t) * k + j];
      if (pos < 0) continue;   // the route's expert lives on another rank
      const float w = topk_w[static_cast<size_t>(t) * k + j];
      const uint4 v = reinterpret_cast<const uint4*>(ys + static_cast<size_t>(pos) * hidden)[i];
      float2 f;
      f = unpack_bf16(v.x); acc[0] += w * f.x; acc[1] += w * f.y;
      f = unpack_bf16(v.y); acc[2] += w * f.x; acc[3] += w * f.y;
      f = unpack_bf16(v.z); acc[4] += w * f.x; acc[5] += w * f.y;
      f = unpack_bf16(v.w); acc[6] += w * f.x; acc[7] += w * f.y;
    }
    reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * hidden)[i] =
        make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
  }
}

}  // namespace ogb

using namespace ogb;

extern "C" int ogb_moe_route_topk(const void* router_logits, int* topk_ids, float* topk_w, int tokens, int experts, int k,
                                  int renormalize, int ld, void* stream) {
  if (tokens <= 0) return 0;
  if (experts > kMaxExperts || k > 32 || k > experts) return -3;
  const int warps_per_block = 8;
  const int blocks = (tokens + warps_per_block - 1) / warps_per_block;
  moe_route_topk_kernel<<<blocks, warps_per_block * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(router_logits), topk_ids, topk_w, tokens, experts, k, renormalize, ld);
  return static_cast<int>(cudaGetLastError());
}

// counts must be zero on entry (the caller clears it); e0 = first expert owned by this rank.
extern "C" int ogb_moe_permute(const int* topk_ids, int* counts, int* offsets, int* cursor, int* sorted_route, int* route_pos,
                               int* tile_tab, int* meta, int tokens, int k, int e0, int experts, int max_mtiles, void* stream) {
  if (tokens <= 0) return 0;
  if (experts > kMaxExperts) return -3;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int routes = tokens * k;
  OGB_CUDA_CHECK(cudaMemsetAsync(counts, 0, sizeof(int) * experts, st));
  moe_count_kernel<<<(routes + 255) / 256, 256, 0, st>>>(topk_ids, counts, routes, e0, experts);
  moe_plan_kernel<<<1, 256, 0, st>>>(counts, offsets, cursor, tile_tab, meta, experts, max_mtiles);
  moe_assign_kernel<<<(routes + 255) / 256, 256, 0, st>>>(topk_ids, offsets, cursor, sorted_route, route_pos, routes, e0, experts);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ogb_moe_gather_rows(const void* x, const int* sorted_route, const int* meta, void* xs, int max_routes, int k,
                                   int hidden, void* stream) {
  if (max_routes <= 0) return 0;
  if (hidden % 8) return -3;
  moe_gather_rows_kernel<<<max_routes, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), sorted_route, meta, static_cast<__nv_bfloat16*>(xs), k, hidden);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ogb_moe_combine(const void* ys, const int* route_pos, const float* topk_w, void* out, int tokens, int k,
                               int hidden, int accumulate, void* stream) {
  if (tokens <= 0) return 0;
  if (hidden % 8) return -3;
  moe_combine_kernel<<<tokens, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(ys), route_pos, topk_w, static_cast<__nv_bfloat16*>(out), k, hidden, accumulate);
  return static_cast<int>(cudaGetLastError());
}
