// Operators of hybrid and sparse decoders that are not GEMM-shaped: the recurrent linear-attention state update, the
// depthwise causal convolution with a rolling state, attention over exporter-selected cache positions, and the checked
// sparse row gather.  Each computes in fp32 from fp32 / bf16 / fp16 tensors and follows the statement of the same
// operator in the graph executor (its torch path is the oracle of the tests).  Counterparts in the reference:
// crates/onnx-runtime-ep-cuda/src/kernels/linear_attention.rs, causal_conv_with_state.rs, index_share.rs,
// sparse_kv_gather.rs.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>

#include "common.cuh"
#include "ogb_kernels.h"

namespace ogb {

enum SeqDtype : int { kSeqF32 = 0, kSeqBF16 = 1, kSeqF16 = 2 };

OGB_DEVICE float seq_load(const void* p, size_t i, int dt) {
  if (dt == kSeqF32) return static_cast<const float*>(p)[i];
  if (dt == kSeqBF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}
OGB_DEVICE void seq_store(void* p, size_t i, int dt, float v) {
  if (dt == kSeqF32) static_cast<float*>(p)[i] = v;
  else if (dt == kSeqBF16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16(v);
  else static_cast<__half*>(p)[i] = __float2half(v);
}

// ------------------------------------------------------------------------------------------------------
// Linear attention.  One CTA per (batch, state head, slice of 128 value columns); a thread owns one column of the
// [d_k, d_v] state in registers for the whole sequence.  Per token: the key (and the queries of the heads that read
// this state, and a per-dimension decay if there is one) are staged in shared memory, the state is decayed, the delta
// rule replaces v by beta (v - S^T k), the outer product k v^T is added and every reading head's q^T S is written.
// ------------------------------------------------------------------------------------------------------
struct LinAttnParams {
  const void *q, *k, *v, *past, *decay, *beta;
  void *out, *state_out;
  int B, T, Hq, Nk, Hkv, dv;
  int decay_per_dim;     // 0: decay [B, T, Hkv]; 1: [B, T, Hkv * d_k]
  int beta_heads;        // Hkv or 1
  int use_decay, use_delta;
  float scale;
  int dt;
};

constexpr int kLinCols = 128;
constexpr int kLinMaxGroup = 8;

template <int DK>
__global__ void __launch_bounds__(kLinCols) linear_attention_kernel(LinAttnParams p) {
  const int h = blockIdx.y, b = blockIdx.z;
  const int j = blockIdx.x * kLinCols + threadIdx.x;
  const bool live = j < p.dv;
  // heads that read this state: a contiguous group of query heads, or the one query head a group of states shares
  const int group = p.Hq >= p.Hkv ? p.Hq / p.Hkv : 1;
  const int out_heads = p.Hq >= p.Hkv ? p.Hq : p.Hkv;
  const int q_first = p.Hq >= p.Hkv ? h * group : static_cast<int>(static_cast<long long>(h) * p.Hq / p.Hkv);
  const int out_first = p.Hq >= p.Hkv ? h * group : h;
  const int kh = h / (p.Hkv / p.Nk);
  __shared__ float sk[DK];
  __shared__ float sg[DK];
  __shared__ float sq[kLinMaxGroup][DK];
  float s[DK];
#pragma unroll
  for (int i = 0; i < DK; ++i)
    s[i] = (p.past != nullptr && live) ? seq_load(p.past, ((static_cast<size_t>(b) * p.Hkv + h) * DK + i) * p.dv + j, p.dt) : 0.f;
  for (int t = 0; t < p.T; ++t) {
    const size_t bt = static_cast<size_t>(b) * p.T + t;
    __syncthreads();
    for (int i = threadIdx.x; i < DK; i += kLinCols) {
      sk[i] = seq_load(p.k, (bt * p.Nk + kh) * DK + i, p.dt);
      if (p.use_decay) sg[i] = __expf(seq_load(p.decay, p.decay_per_dim ? (bt * p.Hkv + h) * DK + i : bt * p.Hkv + h, p.dt));
    }
    for (int i = threadIdx.x; i < group * DK; i += kLinCols)
      sq[i / DK][i % DK] = seq_load(p.q, (bt * p.Hq + q_first + i / DK) * DK + i % DK, p.dt);
    __syncthreads();
    if (!live) continue;
    float vt = seq_load(p.v, (bt * p.Hkv + h) * p.dv + j, p.dt);
    if (p.use_decay) {
#pragma unroll
      for (int i = 0; i < DK; ++i) s[i] *= sg[i];
    }
    if (p.use_delta) {
      float r = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i) r += s[i] * sk[i];
      const float bt_ = seq_load(p.beta, p.beta_heads == 1 ? bt : bt * p.Hkv + h, p.dt);
      vt = bt_ * (vt - r);
    }
#pragma unroll
    for (int i = 0; i < DK; ++i) s[i] += sk[i] * vt;
    for (int g = 0; g < group; ++g) {
      float o = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i) o += sq[g][i] * s[i];
      seq_store(p.out, (bt * out_heads + out_first + g) * p.dv + j, p.dt, o * p.scale);
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DK; ++i) seq_store(p.state_out, ((static_cast<size_t>(b) * p.Hkv + h) * DK + i) * p.dv + j, p.dt, s[i]);
  }
}

// ------------------------------------------------------------------------------------------------------
// Causal depthwise convolution over concat(past_state, x): x [B, C, L], weight [C, K], past [B, C, K-1] or null.
// ------------------------------------------------------------------------------------------------------
__global__ void causal_conv_state_kernel(const void* __restrict__ x, const void* __restrict__ w, const void* __restrict__ bias,
                                         const void* __restrict__ past, void* __restrict__ y, void* __restrict__ state_out,
                                         int B, int C, int L, int K, int silu, int dt) {
  const size_t total = static_cast<size_t>(B) * C * L;
  const size_t n_state = static_cast<size_t>(B) * C * (K - 1);
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total + n_state;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const bool is_state = i >= total;
    const size_t e = is_state ? i - total : i;
    const int span = is_state ? K - 1 : L;
    const int l = static_cast<int>(e % span);
    const size_t bc = e / span;
    const int c = static_cast<int>(bc % C);
    // position `pos` of the concatenated sequence: the state's K-1 frames, then x
    auto seq_at = [&](int pos) -> float {
      if (pos < K - 1) return past != nullptr ? seq_load(past, bc * (K - 1) + pos, dt) : 0.f;
      return seq_load(x, bc * L + (pos - (K - 1)), dt);
    };
    if (is_state) {
      seq_store(state_out, e, dt, seq_at(L + l));
      continue;
    }
    float acc = bias != nullptr ? seq_load(bias, c, dt) : 0.f;
    for (int kk = 0; kk < K; ++kk) acc += seq_load(w, static_cast<size_t>(c) * K + kk, dt) * seq_at(l + kk);
    if (silu) acc = acc / (1.f + __expf(-acc));
    seq_store(y, e, dt, acc);
  }
}

// ------------------------------------------------------------------------------------------------------
// Attention over selected cache positions.  One warp per (batch, head, query row); a lane holds D / 32 elements of the
// query and of the output.  `sel` rows are strictly increasing positions with -1 as trailing padding (validated by the
// caller); a position outside [0, total) sets the status word and is skipped.
// ------------------------------------------------------------------------------------------------------
constexpr int kIsMaxPerLane = 8;   // D <= 256

__global__ void __launch_bounds__(128) index_share_attention_kernel(
    const void* __restrict__ q, const void* __restrict__ k, const void* __restrict__ v, const long long* __restrict__ sel,
    const void* __restrict__ bias, void* __restrict__ out, int B, int N, int Nkv, int Sq, int total, int D, int Ksel, int sel_heads,
    long long bias_sb, long long bias_sn, long long bias_sq, long long bias_st, float scale, int dt, int* status) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= static_cast<long long>(B) * N * Sq) return;
  const int sq_ = static_cast<int>(row % Sq);
  const int n = static_cast<int>((row / Sq) % N);
  const int b = static_cast<int>(row / (static_cast<long long>(Sq) * N));
  const int per = D / 32;
  const int kvh = n / (N / Nkv);
  float qv[kIsMaxPerLane], acc[kIsMaxPerLane];
#pragma unroll
  for (int e = 0; e < kIsMaxPerLane; ++e) {
    qv[e] = e < per ? seq_load(q, static_cast<size_t>(row) * D + lane + 32 * e, dt) : 0.f;
    acc[e] = 0.f;
  }
  const long long* srow = sel + ((static_cast<size_t>(b) * sel_heads + (sel_heads == 1 ? 0 : n)) * Sq + sq_) * Ksel;
  float m = -INFINITY, l = 0.f;
  for (int kk = 0; kk < Ksel; ++kk) {
    const long long idx = srow[kk];
    if (idx < 0) break;
    if (idx >= total) {
      if (lane == 0) atomicOr(status, kStatusIndexOutOfRange);
      continue;
    }
    const size_t kv_off = ((static_cast<size_t>(b) * Nkv + kvh) * total + idx) * D;
    float d = 0.f;
#pragma unroll
    for (int e = 0; e < kIsMaxPerLane; ++e)
      if (e < per) d += qv[e] * seq_load(k, kv_off + lane + 32 * e, dt);
    d = warp_sum(d) * scale;
    if (bias != nullptr) d += seq_load(bias, b * bias_sb + n * bias_sn + sq_ * bias_sq + idx * bias_st, dt);
    if (d == -INFINITY) continue;
    const float m_new = fmaxf(m, d);
    const float corr = __expf(m - m_new);      // exp(-inf) = 0 on the first live position
    const float pexp = __expf(d - m_new);
    l = l * corr + pexp;
#pragma unroll
    for (int e = 0; e < kIsMaxPerLane; ++e)
      if (e < per) acc[e] = acc[e] * corr + pexp * seq_load(v, kv_off + lane + 32 * e, dt);
    m = m_new;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int e = 0; e < kIsMaxPerLane; ++e)
    if (e < per) seq_store(out, static_cast<size_t>(row) * D + lane + 32 * e, dt, acc[e] * inv);
}

// ------------------------------------------------------------------------------------------------------
// Sparse row gather: cache [B, G, C, D] and indices [B, G, Q, K] -> [B, G, Q, K, D]; one warp per selected row, bytes
// copied as they are.  An index outside [0, limit) (limit = the row's valid length, or C) sets the status word and
// yields zeros.
// ------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) sparse_kv_gather_kernel(const uint8_t* __restrict__ cache, const long long* __restrict__ idx,
                                                               const long long* __restrict__ lengths, uint8_t* __restrict__ out,
                                                               long long rows, int G, int C, int QK, int row_bytes, int* status) {
  const int lane = threadIdx.x & 31;
  const long long r = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const long long bg = r / QK;
  const int b = static_cast<int>(bg / G);
  const long long limit = lengths != nullptr ? lengths[b] : C;
  const long long i = idx[r];
  uint8_t* dst = out + static_cast<size_t>(r) * row_bytes;
  if (i < 0 || i >= limit || i >= C) {
    if (lane == 0) atomicOr(status, kStatusIndexOutOfRange);
    for (int o = lane; o < row_bytes; o += 32) dst[o] = 0;
    return;
  }
  const uint8_t* src = cache + (static_cast<size_t>(bg) * C + i) * row_bytes;
  if ((row_bytes & 15) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
    for (int o = lane * 16; o < row_bytes; o += 32 * 16) *reinterpret_cast<uint4*>(dst + o) = *reinterpret_cast<const uint4*>(src + o);
  } else {
    for (int o = lane; o < row_bytes; o += 32) dst[o] = src[o];
  }
}

}  // namespace ogb

using namespace ogb;

extern "C" int ogb_linear_attention(const void* q, const void* k, const void* v, const void* past, const void* decay, const void* beta,
                                    void* out, void* state_out, int B, int T, int Hq, int Nk, int Hkv, int dk, int dv, int decay_per_dim,
                                    int beta_heads, int use_decay, int use_delta, float scale, int dtype, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (B <= 0 || Hkv <= 0 || dv <= 0) return 0;
  if (dtype < 0 || dtype > 2 || Nk <= 0 || Hkv % Nk != 0) return -3;
  if (Hq >= Hkv ? (Hq % Hkv != 0 || Hq / Hkv > kLinMaxGroup) : (Hkv % Hq != 0)) return -3;
  if ((use_decay && decay == nullptr) || (use_delta && beta == nullptr)) return -3;
  LinAttnParams p{q, k, v, past, decay, beta, out, state_out, B, T, Hq, Nk, Hkv, dv, decay_per_dim, beta_heads, use_decay, use_delta, scale, dtype};
  const dim3 grid((dv + kLinCols - 1) / kLinCols, Hkv, B);
  switch (dk) {
    case 32: linear_attention_kernel<32><<<grid, kLinCols, 0, stream>>>(p); break;
    case 64: linear_attention_kernel<64><<<grid, kLinCols, 0, stream>>>(p); break;
    case 128: linear_attention_kernel<128><<<grid, kLinCols, 0, stream>>>(p); break;
    default: return -2;      // the caller keeps its own path for other key widths
  }
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ogb_causal_conv_state(const void* x, const void* w, const void* bias, const void* past, void* y, void* state_out, int B,
                                     int C, int L, int K, int silu, int dtype, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (dtype < 0 || dtype > 2 || K < 1) return -3;
  const size_t work = static_cast<size_t>(B) * C * (static_cast<size_t>(L) + K - 1);
  if (work == 0) return 0;
  const int blocks = static_cast<int>(std::min<size_t>((work + 255) / 256, 148 * 16));
  causal_conv_state_kernel<<<blocks, 256, 0, stream>>>(x, w, bias, past, y, state_out, B, C, L, K, silu, dtype);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ogb_index_share_attention(const void* q, const void* k, const void* v, const void* sel, const void* bias, void* out, int B,
                                         int N, int Nkv, int Sq, int total, int D, int Ksel, int sel_heads, const long long* bias_strides,
                                         float scale, int dtype, int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (dtype < 0 || dtype > 2 || Nkv <= 0 || N % Nkv != 0 || (sel_heads != 1 && sel_heads != N)) return -3;
  if (D % 32 != 0 || D > 32 * kIsMaxPerLane) return -2;
  const long long rows = static_cast<long long>(B) * N * Sq;
  if (rows == 0) return 0;
  const long long sb = bias != nullptr ? bias_strides[0] : 0, sn = bias != nullptr ? bias_strides[1] : 0;
  const long long sq = bias != nullptr ? bias_strides[2] : 0, st = bias != nullptr ? bias_strides[3] : 0;
  index_share_attention_kernel<<<static_cast<unsigned>((rows + 3) / 4), 128, 0, stream>>>(
      q, k, v, static_cast<const long long*>(sel), bias, out, B, N, Nkv, Sq, total, D, Ksel, sel_heads, sb, sn, sq, st, scale, dtype, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ogb_sparse_kv_gather(const void* cache, const void* idx, const void* lengths, void* out, int B, int G, int C, int Q, int K,
                                    int row_bytes, int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long rows = static_cast<long long>(B) * G * Q * K;
  if (rows == 0 || row_bytes == 0) return 0;
  sparse_kv_gather_kernel<<<static_cast<unsigned>((rows + 3) / 4), 128, 0, stream>>>(
      static_cast<const uint8_t*>(cache), static_cast<const long long*>(idx), static_cast<const long long*>(lengths),
      static_cast<uint8_t*>(out), rows, G, C, Q * K, row_bytes, status);
  return static_cast<int>(cudaGetLastError());
}
