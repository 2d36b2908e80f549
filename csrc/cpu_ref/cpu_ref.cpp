// CPU kernels: the oracle every GPU kernel is compared against and the executor of the CPU-only
// configuration (tiny int4 model, batch 4).  They restate, in plain C++ with OpenMP and AVX2 where it
// pays, the semantics of the reference's native CPU provider (crates/onnx-runtime-ep-cpu/src/kernels:
// matmul_nbits.rs block-wise int4 dequant "(code - zero_point) * scale", group_query_attention.rs causal
// GQA with fp32 softmax, rotary half/interleaved rotation, (Skip)SimplifiedLayerNormalization with
// fp32 statistics) and of its sampler chain (crates/onnx-genai-engine/src/sampling.rs:120-170:
// temperature, top-k, top-p renormalised over survivors, min-p, inverse-CDF draw; argmax ties go to
// the lowest index).
//
// Order of operations (documented because the GPU kernels are tested against it):
//   matmul_nbits  w[k] = (code - zp) * scale in fp32; element k accumulates x[k] * w[k] into lane k mod 8 by fused
//                 multiply-add, blocks in ascending order; the 8 lanes are reduced once per output
//   rmsnorm       mean of squares in fp32 (ascending, 8 lanes), y = x * rsqrt(ms + eps) * w
//   attention     scores = q.k * scale in fp32, running max + exp2-free expf softmax, out = sum p.v / sum p
//   sampling      30-bit fixed-point weights round(exp((l - max)/T) * 2^30); integer thresholds keep ties;
//                 the draw walks tokens in index order -- bit-identical to the CUDA sampler.
// All tensors are fp32 row-major unless stated.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#if defined(__AVX2__)
#include <immintrin.h>
#endif

namespace {

constexpr int kPage = 16;

inline float hsum8(const float* v) {
  // fixed pairwise order so scalar and AVX2 builds agree
  return ((v[0] + v[4]) + (v[2] + v[6])) + ((v[1] + v[5]) + (v[3] + v[7]));
}

#if defined(__AVX2__)
inline float hsum256(__m256 v) {
  alignas(32) float t[8];
  _mm256_store_ps(t, v);
  return hsum8(t);
}

// 16 packed bytes (32 nibbles: element 2j in the low nibble of byte j) -> 4 x 8 floats in element order
inline void unpack_block(const uint8_t* q, __m256 out[4]) {
  const __m128i bytes = _mm_loadu_si128(reinterpret_cast<const __m128i*>(q));
  const __m128i mask = _mm_set1_epi8(0x0F);
  const __m128i lo = _mm_and_si128(bytes, mask);
  const __m128i hi = _mm_and_si128(_mm_srli_epi16(bytes, 4), mask);
  const __m128i e0 = _mm_unpacklo_epi8(lo, hi);   // elements 0..15
  const __m128i e1 = _mm_unpackhi_epi8(lo, hi);   // elements 16..31
  out[0] = _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(e0));
  out[1] = _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(_mm_srli_si128(e0, 8)));
  out[2] = _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(e1));
  out[3] = _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(_mm_srli_si128(e1, 8)));
}
#endif

}  // namespace

extern "C" {

// y[M,N] = x[M,K] . dequant(W)^T (+ bias).  qweight [N, KB, 16] uint8, scales [N, KB] fp32, zero_points
// [N, ceil(KB/2)] packed nibbles or null (symmetric, zp = 8), KB = ceil(K/32).
int ogb_cpu_matmul_nbits(const float* x, int64_t ldx, const uint8_t* qweight, const float* scales, const uint8_t* zero_points,
                         const float* bias, float* y, int64_t ldy, int M, int N, int K) {
  if (M < 0 || N <= 0 || K <= 0) return -1;
  const int kb = (K + 31) / 32;
  const int zp_stride = (kb + 1) / 2;
  constexpr int kRows = 8;   // activation rows that share one unpack of a weight block
#pragma omp parallel for schedule(static) if (static_cast<int64_t>(N) * K * std::max(M, 1) > 65536)
  for (int n = 0; n < N; ++n) {
    const uint8_t* qrow = qweight + static_cast<int64_t>(n) * kb * 16;
    const float* srow = scales + static_cast<int64_t>(n) * kb;
    for (int m0 = 0; m0 < M; m0 += kRows) {
      const int mr = std::min(kRows, M - m0);
      float lanes[kRows][8];
      for (int m = 0; m < mr; ++m)
        for (int l = 0; l < 8; ++l) lanes[m][l] = 0.f;
      for (int b = 0; b < kb; ++b) {
        float zp = 8.f;
        if (zero_points != nullptr) {
          const uint8_t zb = zero_points[static_cast<int64_t>(n) * zp_stride + (b >> 1)];
          zp = static_cast<float>((b & 1) ? (zb >> 4) : (zb & 0xF));
        }
        const int valid = std::min(32, K - b * 32);
        const float sc = srow[b];
#if defined(__AVX2__)
        if (valid == 32) {
          __m256 w[4];
          unpack_block(qrow + b * 16, w);
          const __m256 z = _mm256_set1_ps(zp), s8 = _mm256_set1_ps(sc);
          for (int j = 0; j < 4; ++j) w[j] = _mm256_mul_ps(_mm256_sub_ps(w[j], z), s8);   // dequantised weights
          for (int m = 0; m < mr; ++m) {
            const float* xr = x + (m0 + m) * ldx + b * 32;
            __m256 acc = _mm256_loadu_ps(lanes[m]);
            acc = _mm256_fmadd_ps(_mm256_loadu_ps(xr), w[0], acc);
            acc = _mm256_fmadd_ps(_mm256_loadu_ps(xr + 8), w[1], acc);
            acc = _mm256_fmadd_ps(_mm256_loadu_ps(xr + 16), w[2], acc);
            acc = _mm256_fmadd_ps(_mm256_loadu_ps(xr + 24), w[3], acc);
            _mm256_storeu_ps(lanes[m], acc);
          }
          continue;
        }
#endif
        for (int e = 0; e < valid; ++e) {
          const uint8_t byte = qrow[b * 16 + (e >> 1)];
          const float wv = (static_cast<float>((e & 1) ? (byte >> 4) : (byte & 0xF)) - zp) * sc;
          for (int m = 0; m < mr; ++m) lanes[m][e & 7] = std::fmaf(x[(m0 + m) * ldx + b * 32 + e], wv, lanes[m][e & 7]);
        }
      }
      for (int m = 0; m < mr; ++m) y[(m0 + m) * ldy + n] = hsum8(lanes[m]) + (bias ? bias[n] : 0.f);
    }
  }
  return 0;
}

// y[M,N] = x[M,K] . w[N,K]^T (+ bias) (+ residual[M,N]); the inner product runs in 8 lanes, ascending k.
int ogb_cpu_gemm(const float* x, int64_t ldx, const float* w, int64_t ldw, const float* bias, const float* residual, int64_t ldr,
                 float* y, int64_t ldy, int M, int N, int K) {
  if (M < 0 || N <= 0 || K <= 0) return -1;
#pragma omp parallel for collapse(2) schedule(static) if (static_cast<int64_t>(M) * N * K > 65536)
  for (int m = 0; m < M; ++m) {
    for (int n = 0; n < N; ++n) {
      const float* xr = x + m * ldx;
      const float* wr = w + n * ldw;
      float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      int k = 0;
#if defined(__AVX2__)
      __m256 acc = _mm256_setzero_ps();
      for (; k + 8 <= K; k += 8) acc = _mm256_fmadd_ps(_mm256_loadu_ps(xr + k), _mm256_loadu_ps(wr + k), acc);
      _mm256_storeu_ps(lanes, acc);
#endif
      for (; k < K; ++k) lanes[k & 7] = std::fmaf(xr[k], wr[k], lanes[k & 7]);
      float v = hsum8(lanes);
      if (bias) v += bias[n];
      if (residual) v += residual[m * ldr + n];
      y[m * ldy + n] = v;
    }
  }
  return 0;
}

// x += delta (optional, written back to x), y = x * rsqrt(mean(x^2) + eps) * w
int ogb_cpu_rmsnorm(float* x, const float* delta, const float* w, float* y, int rows, int hidden, float eps) {
#pragma omp parallel for schedule(static) if (static_cast<int64_t>(rows) * hidden > 32768)
  for (int r = 0; r < rows; ++r) {
    float* xr = x + static_cast<int64_t>(r) * hidden;
    if (delta) {
      const float* dr = delta + static_cast<int64_t>(r) * hidden;
      for (int i = 0; i < hidden; ++i) xr[i] += dr[i];
    }
    float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int i = 0; i < hidden; ++i) lanes[i & 7] = std::fmaf(xr[i], xr[i], lanes[i & 7]);
    const float inv = 1.0f / std::sqrt(hsum8(lanes) / static_cast<float>(hidden) + eps);
    float* yr = y + static_cast<int64_t>(r) * hidden;
    for (int i = 0; i < hidden; ++i) yr[i] = xr[i] * inv * w[i];
  }
  return 0;
}

// out[rows, inter] = silu(gate_up[:, :inter]) * gate_up[:, inter:]
int ogb_cpu_silu_mul(const float* gate_up, int64_t ld, float* out, int rows, int inter) {
#pragma omp parallel for schedule(static) if (static_cast<int64_t>(rows) * inter > 32768)
  for (int r = 0; r < rows; ++r) {
    const float* g = gate_up + r * ld;
    const float* u = g + inter;
    float* o = out + static_cast<int64_t>(r) * inter;
    for (int i = 0; i < inter; ++i) o[i] = g[i] / (1.0f + std::exp(-g[i])) * u[i];
  }
  return 0;
}

// In place on qkv [T, (hq + 2 hkv) * d]: rotate q and k heads (half or interleaved rotation over the first
// rotary_dim elements, cos_sin [max_pos, rotary_dim/2, 2]), then copy k and v into the paged pool
// [pages, hkv, 2, 16, d] at slot = page * 16 + offset (slot < 0: no write).  Returns -2 if a position or a
// slot is out of range (nothing is written for that row).
int ogb_cpu_rope_kv_append(float* qkv, const int32_t* positions, const int32_t* slots, const float* cos_sin, int max_pos,
                           float* pool, int64_t num_pages, int T, int hq, int hkv, int d, int rotary_dim, int interleaved) {
  const int half = rotary_dim / 2;
  const int64_t row = static_cast<int64_t>(hq + 2 * hkv) * d;
  int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad) if (static_cast<int64_t>(T) * row > 32768)
  for (int t = 0; t < T; ++t) {
    const int pos = positions[t];
    if (pos < 0 || pos >= max_pos) { bad |= 1; continue; }
    const float* cs = cos_sin + static_cast<int64_t>(pos) * half * 2;
    float* base = qkv + t * row;
    for (int h = 0; h < hq + hkv; ++h) {
      float* v = base + static_cast<int64_t>(h) * d;
      for (int i = 0; i < half; ++i) {
        const int i0 = interleaved ? 2 * i : i;
        const int i1 = interleaved ? 2 * i + 1 : i + half;
        const float c = cs[2 * i], s = cs[2 * i + 1];
        const float a = v[i0], b = v[i1];
        v[i0] = a * c - b * s;
        v[i1] = b * c + a * s;
      }
    }
    const int slot = slots[t];
    if (slot < 0) continue;
    const int64_t page = slot / kPage;
    const int off = slot % kPage;
    if (page >= num_pages) { bad |= 1; continue; }
    for (int h = 0; h < hkv; ++h) {
      float* kdst = pool + (((page * hkv + h) * 2 + 0) * kPage + off) * d;
      float* vdst = pool + (((page * hkv + h) * 2 + 1) * kPage + off) * d;
      std::memcpy(kdst, base + static_cast<int64_t>(hq + h) * d, sizeof(float) * d);
      std::memcpy(vdst, base + static_cast<int64_t>(hq + hkv + h) * d, sizeof(float) * d);
    }
  }
  return bad ? -2 : 0;
}

// Varlen causal GQA over the paged pool.  Sequence s owns query rows cu_q[s]..cu_q[s+1]; its last row sits
// at position ctx_len[s] - 1.  q rows are the first hq*d columns of a [T, ldq] matrix; out [T, hq*d].
// window > 0 keeps only the last `window` keys of each query, plus the first `sink` keys of the sequence (attention
// sinks); pages between the two are never read, so their table entries may be -1.
int ogb_cpu_paged_attention(const float* q, int64_t ldq, float* out, const float* pool, const int32_t* page_table,
                            int table_stride, const int32_t* ctx_len, const int32_t* cu_q, int num_seqs, int hq, int hkv, int d,
                            float scale, int window, int sink) {
  const int g = hq / hkv;
  std::vector<int64_t> work;   // (seq, row) pairs flattened so OpenMP balances long and short sequences
  for (int s = 0; s < num_seqs; ++s)
    for (int r = cu_q[s]; r < cu_q[s + 1]; ++r) work.push_back((static_cast<int64_t>(s) << 32) | static_cast<uint32_t>(r));
  const int64_t items = static_cast<int64_t>(work.size()) * hq;
#pragma omp parallel
  {
    std::vector<float> scores;
#pragma omp for schedule(dynamic, 4)
    for (int64_t it = 0; it < items; ++it) {
      const int64_t wr = work[it / hq];
      const int h = static_cast<int>(it % hq);
      const int s = static_cast<int>(wr >> 32);
      const int row = static_cast<int>(wr & 0xffffffff);
      const int ctx = ctx_len[s];
      const int qn = cu_q[s + 1] - cu_q[s];
      const int qpos = ctx - qn + (row - cu_q[s]);
      float* o = out + static_cast<int64_t>(row) * hq * d + static_cast<int64_t>(h) * d;
      if (ctx <= 0 || qpos < 0) { std::fill(o, o + d, 0.f); continue; }
      const int k0 = window > 0 ? std::max(0, qpos - window + 1) : 0;
      const int k1 = qpos + 1;
      const int kvh = h / g;
      const float* qv = q + row * ldq + static_cast<int64_t>(h) * d;
      const int32_t* table = page_table + static_cast<int64_t>(s) * table_stride;
      const int ns = (window > 0) ? std::min(std::max(sink, 0), k0) : 0;   // sink keys below the window
      auto key_at = [&](int j) { return j < ns ? j : k0 + (j - ns); };
      const int nk = ns + (k1 - k0);
      scores.resize(nk);
      float mx = -std::numeric_limits<float>::infinity();
      for (int j = 0; j < nk; ++j) {
        const int k = key_at(j);
        const int64_t page = table[k / kPage];
        const float* kv = pool + (((page * hkv + kvh) * 2 + 0) * kPage + (k % kPage)) * d;
        float lanes[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int i = 0; i < d; ++i) lanes[i & 7] = std::fmaf(qv[i], kv[i], lanes[i & 7]);
        const float sc = hsum8(lanes) * scale;
        scores[j] = sc;
        mx = std::max(mx, sc);
      }
      float denom = 0.f;
      std::fill(o, o + d, 0.f);
      for (int j = 0; j < nk; ++j) {
        const int k = key_at(j);
        const float p = std::exp(scores[j] - mx);
        denom += p;
        const int64_t page = table[k / kPage];
        const float* vv = pool + (((page * hkv + kvh) * 2 + 1) * kPage + (k % kPage)) * d;
        for (int i = 0; i < d; ++i) o[i] = std::fmaf(p, vv[i], o[i]);
      }
      const float inv = 1.0f / denom;
      for (int i = 0; i < d; ++i) o[i] *= inv;
    }
  }
  return 0;
}

// Lowest index wins ties; NaN never wins.
int ogb_cpu_argmax(const float* logits, int64_t ld, int32_t* out, int rows, int vocab) {
#pragma omp parallel for schedule(static) if (static_cast<int64_t>(rows) * vocab > 65536)
  for (int r = 0; r < rows; ++r) {
    const float* l = logits + r * ld;
    float best = -std::numeric_limits<float>::infinity();
    int bi = 0;
    bool any = false;
    for (int i = 0; i < vocab; ++i) {
      const float v = l[i];
      if (v != v) continue;
      if (!any || v > best) { best = v; bi = i; any = true; }
    }
    out[r] = bi;
  }
  return 0;
}

// Fused sampler with the device kernel's integer semantics (see the file header).  uniform[r] in [0,1).
int ogb_cpu_sample(const float* logits, int64_t ld, int32_t* out, const float* temperature, const int32_t* top_k,
                   const float* top_p, const float* min_p, const float* uniform, int rows, int vocab) {
#pragma omp parallel for schedule(dynamic, 1) if (rows > 1)
  for (int r = 0; r < rows; ++r) {
    const float* l = logits + r * ld;
    float best = -std::numeric_limits<float>::infinity();
    int bi = -1;
    for (int i = 0; i < vocab; ++i) {
      const float v = l[i];
      if (v != v) continue;
      if (bi < 0 || v > best) { best = v; bi = i; }
    }
    const float t = temperature[r];
    if (!(t > 0.f) || bi < 0) { out[r] = bi < 0 ? 0 : bi; continue; }
    std::vector<uint32_t> w(vocab);
    unsigned long long total = 0;
    for (int i = 0; i < vocab; ++i) {
      float e = std::exp((l[i] - best) / t);
      if (!(e >= 0.f)) e = 0.f;
      double qd = std::floor(static_cast<double>(e) * 1073741824.0 + 0.5);
      uint32_t qv = qd > 1073741823.0 ? 1073741823u : static_cast<uint32_t>(qd);
      w[i] = qv;
      total += qv;
    }
    uint32_t thr = 1;
    std::vector<uint32_t> sorted;
    auto ensure_sorted = [&]() {
      if (sorted.empty()) {
        sorted = w;
        std::sort(sorted.begin(), sorted.end(), std::greater<uint32_t>());
      }
    };
    const int k = top_k[r];
    if (k > 0 && k < vocab) {
      ensure_sorted();
      thr = std::max(thr, sorted[k - 1]);
      total = 0;
      for (int i = 0; i < vocab; ++i) total += (w[i] >= thr) ? w[i] : 0u;
    }
    const float p = top_p[r];
    if (p > 0.f && p < 1.f) {
      unsigned long long target = static_cast<unsigned long long>(static_cast<double>(total) * static_cast<double>(p));
      if (target < 1ull) target = 1ull;
      ensure_sorted();
      unsigned long long run = 0;
      uint32_t at = thr;
      for (int i = 0; i < vocab && sorted[i] >= thr; ++i) {
        run += sorted[i];
        at = sorted[i];
        if (run >= target) break;
      }
      thr = std::max(thr, at);
    }
    const float mp = min_p[r];
    if (mp > 0.f) {
      const uint32_t floor_mp = static_cast<uint32_t>(std::min(mp, 1.0f) * 1073741824.0f);
      thr = std::max(thr, floor_mp);
    }
    unsigned long long final_total = 0;
    for (int i = 0; i < vocab; ++i) final_total += (w[i] >= thr) ? w[i] : 0u;
    if (final_total == 0) { out[r] = bi; continue; }
    float u = uniform[r];
    u = std::min(std::max(u, 0.f), 0.99999994f);
    unsigned long long target = static_cast<unsigned long long>(static_cast<double>(u) * static_cast<double>(final_total));
    if (target >= final_total) target = final_total - 1;
    unsigned long long run = 0;
    int pick = bi;
    for (int i = 0; i < vocab; ++i) {
      if (w[i] < thr) continue;
      run += w[i];
      if (target < run) { pick = i; break; }
    }
    out[r] = pick;
  }
  return 0;
}

// W[N, K] fp32 = dequantised MatMulNBits weight (used by tests and by exporters that need the dense form).
int ogb_cpu_dequant_nbits(const uint8_t* qweight, const float* scales, const uint8_t* zero_points, float* w, int N, int K) {
  const int kb = (K + 31) / 32;
  const int zp_stride = (kb + 1) / 2;
#pragma omp parallel for schedule(static) if (static_cast<int64_t>(N) * K > 65536)
  for (int n = 0; n < N; ++n) {
    for (int k = 0; k < K; ++k) {
      const int b = k / 32, e = k % 32;
      const uint8_t byte = qweight[(static_cast<int64_t>(n) * kb + b) * 16 + (e >> 1)];
      const float code = static_cast<float>((e & 1) ? (byte >> 4) : (byte & 0xF));
      float zp = 8.f;
      if (zero_points) {
        const uint8_t zb = zero_points[static_cast<int64_t>(n) * zp_stride + (b >> 1)];
        zp = static_cast<float>((b & 1) ? (zb >> 4) : (zb & 0xF));
      }
      w[static_cast<int64_t>(n) * K + k] = (code - zp) * scales[static_cast<int64_t>(n) * kb + b];
    }
  }
  return 0;
}

}  // extern "C"
