// Bandwidth-bound glue kernels: embedding gather, (skip-)RMSNorm, SwiGLU, rotary embedding fused
// with the KV-page append, and fp8 page quantisation.
//
// Reference counterparts: skip_rmsnorm_* / rmsnorm_* (crates/onnx-runtime-ep-cuda/src/kernels/
// normalization.rs:1327), rotary_embedding_* (kernels/rotary_embedding.rs:45,620-640),
// gqa_fuse_decode_prep* / gqa_append_cache* (kernels/group_query_attention.rs:33-140), silu_mul_*
// (kernels/elementwise.rs), gather (kernels/gather.rs).  Out-of-range token ids, positions or
// slots set kStatusIndexOutOfRange in the status word and the access is skipped, following the
// capture-error-word convention of that code base.
#include <cuda_fp8.h>
#include "common.cuh"
#include "ogb_kernels.h"

namespace ogb {

// ------------------------------------------------------------------------------------------
// embedding gather: out[t, :] = table[ids[t], :]
// ------------------------------------------------------------------------------------------
__global__ void embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, int hidden, int vocab, int* status) {
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= vocab) {
    if (threadIdx.x == 0) atomicOr(status, kStatusIndexOutOfRange);
    id = 0;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = __ldg(src + i);
}

// ------------------------------------------------------------------------------------------
// RMSNorm with fp32 statistics; optional residual add written back (SkipSimplifiedLayerNorm)
// ------------------------------------------------------------------------------------------
constexpr int kNormThreads = 256;
constexpr int kNormMaxVec = 4;  // cached 16-byte vectors per thread (hidden <= 8192 stays in registers)

__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(__nv_bfloat16* x, const __nv_bfloat16* __restrict__ delta,
                                                                const __nv_bfloat16* __restrict__ weight,
                                                                __nv_bfloat16* __restrict__ out, int hidden, int ldx,
                                                                int ldo, float eps) {
  const int row = blockIdx.x;
  __nv_bfloat16* xr = x + static_cast<size_t>(row) * ldx;
  const __nv_bfloat16* dr = delta ? delta + static_cast<size_t>(row) * hidden : nullptr;
  const int nvec = hidden / 8;
  float cache[kNormMaxVec][8];
  float ss = 0.f;
  int c = 0;
  for (int i = threadIdx.x; i < nvec; i += kNormThreads, ++c) {
    uint4 v = reinterpret_cast<const uint4*>(xr)[i];
    float f[8];
    float2 t;
    t = unpack_bf16(v.x); f[0] = t.x; f[1] = t.y;
    t = unpack_bf16(v.y); f[2] = t.x; f[3] = t.y;
    t = unpack_bf16(v.z); f[4] = t.x; f[5] = t.y;
    t = unpack_bf16(v.w); f[6] = t.x; f[7] = t.y;
    if (dr) {
      uint4 d = reinterpret_cast<const uint4*>(dr)[i];
      t = unpack_bf16(d.x); f[0] += t.x; f[1] += t.y;
      t = unpack_bf16(d.y); f[2] += t.x; f[3] += t.y;
      t = unpack_bf16(d.z); f[4] += t.x; f[5] += t.y;
      t = unpack_bf16(d.w); f[6] += t.x; f[7] += t.y;
      // the residual stream is stored in bf16: round first so the statistics see the stored value
      uint4 w4 = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
      reinterpret_cast<uint4*>(xr)[i] = w4;
      t = unpack_bf16(w4.x); f[0] = t.x; f[1] = t.y;
      t = unpack_bf16(w4.y); f[2] = t.x; f[3] = t.y;
      t = unpack_bf16(w4.z); f[4] = t.x; f[5] = t.y;
      t = unpack_bf16(w4.w); f[6] = t.x; f[7] = t.y;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      ss += f[k] * f[k];
      if (c < kNormMaxVec) cache[c][k] = f[k];
    }
  }
  __shared__ float red[kNormThreads / 32];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kNormThreads / 32; ++i) tot += red[i];
  const float inv = rsqrtf(tot / static_cast<float>(hidden) + eps);
  __nv_bfloat16* orow = out + static_cast<size_t>(row) * ldo;
  c = 0;
  for (int i = threadIdx.x; i < nvec; i += kNormThreads, ++c) {
    float f[8];
    if (c < kNormMaxVec) {
#pragma unroll
      for (int k = 0; k < 8; ++k) f[k] = cache[c][k];
    } else {
      uint4 v = reinterpret_cast<const uint4*>(xr)[i];
      float2 t;
      t = unpack_bf16(v.x); f[0] = t.x; f[1] = t.y;
      t = unpack_bf16(v.y); f[2] = t.x; f[3] = t.y;
      t = unpack_bf16(v.z); f[4] = t.x; f[5] = t.y;
      t = unpack_bf16(v.w); f[6] = t.x; f[7] = t.y;
    }
    uint4 wv = __ldg(reinterpret_cast<const uint4*>(weight) + i);
    float2 w0 = unpack_bf16(wv.x), w1 = unpack_bf16(wv.y), w2 = unpack_bf16(wv.z), w3 = unpack_bf16(wv.w);
    uint4 o4 = make_uint4(pack_bf16(f[0] * inv * w0.x, f[1] * inv * w0.y), pack_bf16(f[2] * inv * w1.x, f[3] * inv * w1.y),
                          pack_bf16(f[4] * inv * w2.x, f[5] * inv * w2.y), pack_bf16(f[6] * inv * w3.x, f[7] * inv * w3.y));
    reinterpret_cast<uint4*>(orow)[i] = o4;
  }
}

// One warp per row, every 16-byte vector of the row held in registers (hidden <= 4096): all loads of
// a row are issued back to back, the statistics never touch shared memory, and a step's ~1300 rows
// fit in a single wave of CTAs.
constexpr int kNormWarpMaxVec = 16;

__global__ void __launch_bounds__(128) rmsnorm_warp_kernel(__nv_bfloat16* x, const __nv_bfloat16* __restrict__ delta,
                                                            const __nv_bfloat16* __restrict__ weight,
                                                            __nv_bfloat16* __restrict__ out, int rows, int hidden, int ldx,
                                                            int ldo, float eps) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  __nv_bfloat16* xr = x + static_cast<size_t>(row) * ldx;
  const int nvec = hidden / 8;
  uint4 v[kNormWarpMaxVec], wq[kNormWarpMaxVec];
#pragma unroll
  for (int c = 0; c < kNormWarpMaxVec; ++c) {
    const int i = lane + 32 * c;
    if (i < nvec) {
      v[c] = reinterpret_cast<const uint4*>(xr)[i];
      wq[c] = __ldg(reinterpret_cast<const uint4*>(weight) + i);   // in flight together with the row itself
    }
  }
  if (delta != nullptr) {
    const __nv_bfloat16* dr = delta + static_cast<size_t>(row) * hidden;
#pragma unroll
    for (int c = 0; c < kNormWarpMaxVec; ++c) {
      const int i = lane + 32 * c;
      if (i < nvec) {
        const uint4 d = reinterpret_cast<const uint4*>(dr)[i];
        float2 a, b;
        a = unpack_bf16(v[c].x); b = unpack_bf16(d.x); v[c].x = pack_bf16(a.x + b.x, a.y + b.y);
        a = unpack_bf16(v[c].y); b = unpack_bf16(d.y); v[c].y = pack_bf16(a.x + b.x, a.y + b.y);
        a = unpack_bf16(v[c].z); b = unpack_bf16(d.z); v[c].z = pack_bf16(a.x + b.x, a.y + b.y);
        a = unpack_bf16(v[c].w); b = unpack_bf16(d.w); v[c].w = pack_bf16(a.x + b.x, a.y + b.y);
        reinterpret_cast<uint4*>(xr)[i] = v[c];   // the residual stream keeps the bf16-rounded sum
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kNormWarpMaxVec; ++c) {
    if (lane + 32 * c < nvec) {
      float2 f;
      f = unpack_bf16(v[c].x); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16(v[c].y); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16(v[c].z); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16(v[c].w); ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / static_cast<float>(hidden) + eps);
  __nv_bfloat16* orow = out + static_cast<size_t>(row) * ldo;
#pragma unroll
  for (int c = 0; c < kNormWarpMaxVec; ++c) {
    const int i = lane + 32 * c;
    if (i < nvec) {
      const uint4 wv = wq[c];
      float2 a, w;
      uint4 o4;
      a = unpack_bf16(v[c].x); w = unpack_bf16(wv.x); o4.x = pack_bf16(a.x * inv * w.x, a.y * inv * w.y);
      a = unpack_bf16(v[c].y); w = unpack_bf16(wv.y); o4.y = pack_bf16(a.x * inv * w.x, a.y * inv * w.y);
      a = unpack_bf16(v[c].z); w = unpack_bf16(wv.z); o4.z = pack_bf16(a.x * inv * w.x, a.y * inv * w.y);
      a = unpack_bf16(v[c].w); w = unpack_bf16(wv.w); o4.w = pack_bf16(a.x * inv * w.x, a.y * inv * w.y);
      reinterpret_cast<uint4*>(orow)[i] = o4;
    }
  }
}

// ------------------------------------------------------------------------------------------
// out[r, j] = silu(gate_up[r, j]) * gate_up[r, inter + j]   (unfused fallback of the GEMM epilogue)
// ------------------------------------------------------------------------------------------
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int inter,
                                size_t total_vec) {
  const int vec_per_row = inter / 8;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total_vec;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t row = i / vec_per_row;
    const int cv = static_cast<int>(i % vec_per_row);
    const uint4 g = reinterpret_cast<const uint4*>(gu + row * 2 * inter)[cv];
    const uint4 u = reinterpret_cast<const uint4*>(gu + row * 2 * inter + inter)[cv];
    const uint32_t gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 a = unpack_bf16(gs[k]), b = unpack_bf16(us[k]);
      o[k] = pack_bf16(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
    }
    reinterpret_cast<uint4*>(out + row * inter)[cv] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ------------------------------------------------------------------------------------------
// RoPE (q and k, in place) + append of k, v to the paged pool.
// One CTA per token; thread = one (head, pair-chunk).  cos_sin: [max_pos, rotary_dim/2, 2] fp32.
// ------------------------------------------------------------------------------------------
template <bool FP8>
__global__ void rope_kv_append_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                      const int* __restrict__ slots, const float* __restrict__ cos_sin,
                                      void* __restrict__ pool, float* __restrict__ scales, int hq, int hkv, int d,
                                      int rotary_dim, int interleaved, int page_size, int64_t num_slots, int max_pos,
                                      int* status) {
  const int t = blockIdx.x;
  int pos = positions[t];
  const int64_t slot = slots[t];  // slot = page * page_size + offset; negative = do not cache
  if (pos < 0 || pos >= max_pos) {
    if (threadIdx.x == 0) atomicOr(status, kStatusIndexOutOfRange);
    pos = 0;
  }
  const bool slot_ok = slot >= 0 && slot < num_slots;  // slot < 0: token is not cached (padding row)
  if (!slot_ok && slot >= num_slots && threadIdx.x == 0) atomicOr(status, kStatusIndexOutOfRange);
  __nv_bfloat16* row = qkv + static_cast<size_t>(t) * (hq + 2 * hkv) * d;
  const int half = rotary_dim / 2;
  const float* cs = cos_sin + static_cast<size_t>(pos) * half * 2;
  // rotate q and k heads
  const int rot_heads = hq + hkv;
  for (int i = threadIdx.x; i < rot_heads * half; i += blockDim.x) {
    const int h = i / half, j = i % half;
    __nv_bfloat16* hp = row + h * d;
    const int i0 = interleaved ? 2 * j : j;
    const int i1 = interleaved ? 2 * j + 1 : j + half;
    const float c = cs[2 * j], s = cs[2 * j + 1];
    const float x0 = __bfloat162float(hp[i0]), x1 = __bfloat162float(hp[i1]);
    hp[i0] = __float2bfloat16(x0 * c - x1 * s);
    hp[i1] = __float2bfloat16(x1 * c + x0 * s);
  }
  __syncthreads();
  if (!slot_ok || pool == nullptr) return;     // pool == nullptr: rotation only (the e4m3 append is its own launch)
  const int64_t page = slot / page_size;
  const int off = static_cast<int>(slot % page_size);
  if constexpr (!FP8) {
    __nv_bfloat16* pl = static_cast<__nv_bfloat16*>(pool);
    const int vec_per_head = d / 8;
    for (int i = threadIdx.x; i < 2 * hkv * vec_per_head; i += blockDim.x) {
      const int kv = i / (hkv * vec_per_head);  // 0 = K, 1 = V
      const int h = (i / vec_per_head) % hkv;
      const int v = i % vec_per_head;
      const uint4 val = reinterpret_cast<const uint4*>(row + (hq + kv * hkv + h) * d)[v];
      __nv_bfloat16* dst = pl + ((((page * hkv + h) * 2 + kv) * page_size + off) * static_cast<int64_t>(d));
      reinterpret_cast<uint4*>(dst)[v] = val;
    }
  }
}

// e4m3 append as its own launch, after the rotation kernel.  One scale per (page, head, K|V), fixed by the
// page's first token (amax * 2 / 448: headroom for the 15 tokens that follow; they saturate to it).  A prefill
// chunk writes many tokens of one page in the same launch, so a token must not read the scale from memory while
// the first token's CTA may still be writing it: when the page's first token is a row of this launch (row
// t - offset carries slot - offset), every token of the page derives the scale from that row's values, which the
// preceding rotation launch has finalised; otherwise the page was started by an earlier launch and the stored
// scale is read.
__global__ void kv_append_fp8_kernel(const __nv_bfloat16* __restrict__ qkv, const int* __restrict__ slots,
                                     uint8_t* __restrict__ pool, float* __restrict__ scales, int hq, int hkv, int d,
                                     int page_size, int64_t num_slots, int fmt, int* status) {
  const float qmax = fmt == 0 ? 448.f : (fmt == 1 ? 127.f : 57344.f);     // fmt 0: e4m3, 1: int8 (symmetric), 2: e5m2
  const int t = blockIdx.x;
  const int64_t slot = slots[t];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, kStatusIndexOutOfRange);
    return;
  }
  const int64_t page = slot / page_size;
  const int off = static_cast<int>(slot % page_size);
  const size_t row_elems = static_cast<size_t>(hq + 2 * hkv) * d;
  const __nv_bfloat16* row = qkv + static_cast<size_t>(t) * row_elems;
  bool first_in_launch = true;
  const __nv_bfloat16* first_row = row;
  if (off != 0) {
    const int t0 = t - off;
    if (t0 >= 0 && slots[t0] == slot - off) first_row = qkv + static_cast<size_t>(t0) * row_elems;
    else first_in_launch = false;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int u = warp; u < 2 * hkv; u += nwarps) {
    const int kv = u / hkv, h = u % hkv;
    const size_t col = static_cast<size_t>(hq + kv * hkv + h) * d;
    float* sc = scales + ((page * hkv + h) * 2 + kv);
    float scale = 0.f;
    if (first_in_launch) {
      float amax = 0.f;
      for (int j = lane; j < d; j += 32) amax = fmaxf(amax, fabsf(__bfloat162float(first_row[col + j])));
      amax = warp_max(amax);
      scale = fmaxf(amax * 2.f, 1e-6f) / qmax;
      if (off == 0 && lane == 0) *sc = scale;
    } else {
      scale = *sc;
      if (!(scale > 0.f)) {                        // a page that was never started: treat this token as its first
        float amax = 0.f;
        for (int j = lane; j < d; j += 32) amax = fmaxf(amax, fabsf(__bfloat162float(row[col + j])));
        amax = warp_max(amax);
        scale = fmaxf(amax * 2.f, 1e-6f) / qmax;
        if (lane == 0) *sc = scale;
      }
    }
    const float inv = 1.f / scale;
    uint8_t* dst = pool + ((((page * hkv + h) * 2 + kv) * page_size + off) * static_cast<int64_t>(d));
    for (int j = lane; j < d; j += 32) {
      float v = __bfloat162float(row[col + j]) * inv;
      v = fminf(fmaxf(v, -qmax), qmax);
      dst[j] = fmt == 0 ? static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3))
               : fmt == 1 ? static_cast<uint8_t>(static_cast<int8_t>(__float2int_rn(v)))
                          : static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2));
    }
  }
}

// ------------------------------------------------------------------------------------------
// page copy (copy-on-write fork) and gather / scatter to a staging buffer (swap out / in)
// ------------------------------------------------------------------------------------------
__global__ void page_copy_kernel(uint8_t* dst_base, const uint8_t* src_base, const int64_t* __restrict__ src_pages,
                                 const int64_t* __restrict__ dst_pages, int64_t page_bytes, int src_indexed,
                                 int dst_indexed) {
  const int i = blockIdx.y;
  const int64_t sp = src_indexed ? src_pages[i] : i;
  const int64_t dp = dst_indexed ? dst_pages[i] : i;
  const uint4* src = reinterpret_cast<const uint4*>(src_base + sp * page_bytes);
  uint4* dst = reinterpret_cast<uint4*>(dst_base + dp * page_bytes);
  const int64_t nvec = page_bytes / 16;
  for (int64_t v = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; v < nvec;
       v += static_cast<int64_t>(gridDim.x) * blockDim.x)
    dst[v] = src[v];
}

// Page moves across every layer in one launch: grid = (blocks per page, pages, layers).  `src_bases` / `dst_bases`
// hold one base address per layer; either side may be pinned host memory (the device reads and writes it over
// PCIe without a staging copy).  Page ids come from the packed step plan as int32 and are bounds-checked: a bad
// id raises kStatusIndexOutOfRange and that page is skipped.
__global__ void page_move_layers_kernel(const uint64_t* __restrict__ dst_bases, const uint64_t* __restrict__ src_bases,
                                        const int* __restrict__ src_pages, const int* __restrict__ dst_pages,
                                        int64_t page_bytes, int64_t src_count, int64_t dst_count, int* status) {
  const int i = blockIdx.y;
  const int64_t sp = src_pages[i], dp = dst_pages[i];
  if (sp < 0 || sp >= src_count || dp < 0 || dp >= dst_count) {
    if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(status, kStatusIndexOutOfRange);
    return;
  }
  const uint8_t* src = reinterpret_cast<const uint8_t*>(src_bases[blockIdx.z]) + sp * page_bytes;
  uint8_t* dst = reinterpret_cast<uint8_t*>(dst_bases[blockIdx.z]) + dp * page_bytes;
  const int64_t first = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if ((page_bytes & 15) == 0) {
    for (int64_t v = first; v < page_bytes / 16; v += step)
      reinterpret_cast<uint4*>(dst)[v] = reinterpret_cast<const uint4*>(src)[v];
  } else {
    for (int64_t v = first; v < page_bytes / 4; v += step)
      reinterpret_cast<uint32_t*>(dst)[v] = reinterpret_cast<const uint32_t*>(src)[v];
  }
}

}  // namespace ogb

using namespace ogb;

extern "C" int ogb_embedding_bf16(const int* ids, const void* table, void* out, int tokens, int hidden, int vocab,
                                  int* status, void* stream) {
  if (tokens <= 0) return 0;
  if (hidden % 8) return -3;
  embedding_kernel<<<tokens, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      ids, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), hidden, vocab, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ogb_rmsnorm_bf16(void* x, const void* delta, const void* weight, void* out, int rows, int hidden, int ldx,
                                int ldo, float eps, void* stream) {
  if (rows <= 0) return 0;
  if (hidden % 8 || ldx % 8 || ldo % 8) return -3;
  if (hidden / 8 <= 32 * kNormWarpMaxVec) {
    rmsnorm_warp_kernel<<<(rows + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(weight),
        static_cast<__nv_bfloat16*>(out), rows, hidden, ldx, ldo, eps);
    return static_cast<int>(cudaGetLastError());
  }
  rmsnorm_kernel<<<rows, kNormThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(delta), static_cast<const __nv_bfloat16*>(weight),
      static_cast<__nv_bfloat16*>(out), hidden, ldx, ldo, eps);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ogb_silu_mul_bf16(const void* gate_up, void* out, int rows, int inter, void* stream) {
  if (rows <= 0) return 0;
  if (inter % 8) return -3;
  const size_t total_vec = static_cast<size_t>(rows) * (inter / 8);
  int blocks = static_cast<int>((total_vec + 255) / 256);
  const int cap = ogb_num_sms() * 8;
  if (blocks > cap) blocks = cap;
  silu_mul_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const __nv_bfloat16*>(gate_up),
                                                                          static_cast<__nv_bfloat16*>(out), inter, total_vec);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ogb_rope_kv_append_bf16(void* qkv, const int* positions, const int* slots, const float* cos_sin,
                                       void* pool, int tokens, int hq, int hkv, int d, int rotary_dim, int interleaved,
                                       int page_size, int64_t num_slots, int max_pos, int* status, void* stream) {
  if (tokens <= 0) return 0;
  if (d % 8 || rotary_dim % 2 || rotary_dim > d) return -3;
  rope_kv_append_kernel<false><<<tokens, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(qkv), positions, slots, cos_sin, pool, nullptr, hq, hkv, d, rotary_dim, interleaved,
      page_size, num_slots, max_pos, status);
  return static_cast<int>(cudaGetLastError());
}

static int launch_rope_kv_append_q8(void* qkv, const int* positions, const int* slots, const float* cos_sin, void* pool,
                                    float* scales, int kv_format, int tokens, int hq, int hkv, int d, int rotary_dim,
                                    int interleaved, int page_size, int64_t num_slots, int max_pos, int* status, void* stream) {
  if (tokens <= 0) return 0;
  if (d % 8 || rotary_dim % 2 || rotary_dim > d || kv_format < 0 || kv_format > 2) return -3;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rope_kv_append_kernel<false><<<tokens, 256, 0, st>>>(static_cast<__nv_bfloat16*>(qkv), positions, slots, cos_sin, nullptr,
                                                      nullptr, hq, hkv, d, rotary_dim, interleaved, page_size, num_slots,
                                                      max_pos, status);
  kv_append_fp8_kernel<<<tokens, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(qkv), slots, static_cast<uint8_t*>(pool), scales,
                                               hq, hkv, d, page_size, num_slots, kv_format, status);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ogb_rope_kv_append_fp8(void* qkv, const int* positions, const int* slots, const float* cos_sin,
                                      void* pool, float* scales, int tokens, int hq, int hkv, int d, int rotary_dim,
                                      int interleaved, int page_size, int64_t num_slots, int max_pos, int* status,
                                      void* stream) {
  return launch_rope_kv_append_q8(qkv, positions, slots, cos_sin, pool, scales, 0, tokens, hq, hkv, d, rotary_dim, interleaved,
                                  page_size, num_slots, max_pos, status, stream);
}
// kv_format 0 = e4m3, 1 = int8, 2 = e5m2; same pool and scale layout
extern "C" int ogb_rope_kv_append_q8(void* qkv, const int* positions, const int* slots, const float* cos_sin, void* pool,
                                     float* scales, int kv_format, int tokens, int hq, int hkv, int d, int rotary_dim,
                                     int interleaved, int page_size, int64_t num_slots, int max_pos, int* status,
                                     void* stream) {
  return launch_rope_kv_append_q8(qkv, positions, slots, cos_sin, pool, scales, kv_format, tokens, hq, hkv, d, rotary_dim,
                                  interleaved, page_size, num_slots, max_pos, status, stream);
}

static int launch_page_copy(void* dst, const void* src, const int64_t* sp, const int64_t* dp, int n, int64_t page_bytes,
                            int si, int di, void* stream) {
  if (n <= 0) return 0;
  if (page_bytes % 16) return -3;
  int bx = static_cast<int>((page_bytes / 16 + 255) / 256);
  if (bx > 64) bx = 64;
  dim3 grid(bx, n);
  page_copy_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint8_t*>(dst),
                                                                         static_cast<const uint8_t*>(src), sp, dp,
                                                                         page_bytes, si, di);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int ogb_kv_page_copy(void* pool, const int64_t* src_pages, const int64_t* dst_pages, int n, int64_t page_bytes,
                                void* stream) {
  return launch_page_copy(pool, pool, src_pages, dst_pages, n, page_bytes, 1, 1, stream);
}
extern "C" int ogb_kv_gather_pages(const void* pool, void* staging, const int64_t* pages, int n, int64_t page_bytes,
                                   void* stream) {
  return launch_page_copy(staging, pool, pages, nullptr, n, page_bytes, 1, 0, stream);
}
extern "C" int ogb_kv_scatter_pages(void* pool, const void* staging, const int64_t* pages, int n, int64_t page_bytes,
                                    void* stream) {
  return launch_page_copy(pool, staging, nullptr, pages, n, page_bytes, 0, 1, stream);
}

// n pages of every one of `layers` page arrays: dst_bases[l] + dst_pages[i] * page_bytes <- src_bases[l] + src_pages[i] * page_bytes.
// The base tables and the index lists are device arrays; the arrays they name may be device or pinned host memory.
extern "C" int ogb_kv_move_pages(const uint64_t* dst_bases, const uint64_t* src_bases, int layers, const int* src_pages,
                                 const int* dst_pages, int n, int64_t page_bytes, int64_t src_count, int64_t dst_count,
                                 int* status, void* stream) {
  if (n <= 0 || layers <= 0) return 0;
  if (page_bytes % 4 || n > 65535 || layers > 65535) return -3;
  const int64_t vecs = (page_bytes % 16 == 0) ? page_bytes / 16 : page_bytes / 4;
  int bx = static_cast<int>((vecs + 255) / 256);
  if (bx > 16) bx = 16;
  if (bx < 1) bx = 1;
  page_move_layers_kernel<<<dim3(bx, n, layers), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      dst_bases, src_bases, src_pages, dst_pages, page_bytes, src_count, dst_count, status);
  return static_cast<int>(cudaGetLastError());
}
