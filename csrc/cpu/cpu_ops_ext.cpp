// Native CPU backend, second part: the ops beyond a plain dense decoder. Mixture-of-experts
// router and expert block, Gated-DeltaNet (causal conv1d, q/k normalisation and gates, the
// sequential gated delta rule, gated RMSNorm), multi-head latent attention over the compressed
// cache, and GEMMs that keep GGUF block-quantised weights (Q8_0 / Q4_0) packed and take integer
// dot products against activations quantised per 32-element block.
//
// bf16 storage, fp32 arithmetic; every op rounds where the PyTorch oracle of the test-suite rounds
// (ops/{moe,gdn,mla}.py ref_*). Work is split by output index, so results do not depend on the
// thread count.
//
// Reference: src/vt/cpu/cpu_ops.cpp (GDN scan / decode, conv1d, MoE router / combine),
// src/vt/cpu/cpu_mla_attn.cpp, src/vt/cpu/cpu_quant_dot.cpp, src/vt/cpu/cpu_quant_gemm.cpp.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#endif
#include <cstdlib>

#include "cpu_common.h"
#include "cpu_threadpool.h"

using namespace b200cpu;

extern "C" {
void b200cpu_matmul_bt(const uint16_t* A, int64_t lda, const uint16_t* W, int64_t ldw, void* out, int64_t ldo,
                       int out_f32, const uint16_t* bias, const uint16_t* residual, int64_t ldr, int M, int N, int K);
void b200cpu_act_and_mul(const uint16_t* x, int64_t ldx, uint16_t* out, int64_t ldo, int T, int I, int kind);
}

namespace {

inline float silu(float x) { return x / (1.f + std::exp(-x)); }
inline float sigmoid(float x) { return 1.f / (1.f + std::exp(-x)); }
inline float softplus(float x) { return x > 20.f ? x : std::log1p(std::exp(x)); }

}  // namespace

extern "C" {

// ------------------------------------------------------------------------------- MoE router
// Scores = softmax (scoring 0) or sigmoid (1) of the logits; selection runs on score + e_bias,
// optionally restricted to the best `topk_group` of `n_group` expert groups (group score: the sum
// of its two best entries when a bias is present, else its maximum); ties go to the lowest expert
// index; weights are the unbiased scores, renormalised over the k chosen when `renorm`, then
// multiplied by `routed_scale`.
void b200cpu_moe_router_topk(const float* logits, int64_t ld, int T, int E, int k, int renorm, int scoring,
                             const float* e_bias, int n_group, int topk_group, float routed_scale, int32_t* ids,
                             float* w) {
  ThreadPool::instance().parallel_for(T, 4, [&](int64_t t0, int64_t t1) {
    std::vector<float> score(E), sel(E);
    const float ninf = -std::numeric_limits<float>::infinity();
    for (int64_t t = t0; t < t1; ++t) {
      const float* lr = logits + t * ld;
      if (scoring == 0) {
        float mx = lr[0];
        for (int e = 1; e < E; ++e) mx = std::max(mx, lr[e]);
        float sum = 0.f;
        for (int e = 0; e < E; ++e) { score[e] = std::exp(lr[e] - mx); sum += score[e]; }
        for (int e = 0; e < E; ++e) score[e] /= sum;
      } else {
        for (int e = 0; e < E; ++e) score[e] = sigmoid(lr[e]);
      }
      for (int e = 0; e < E; ++e) sel[e] = score[e] + (e_bias ? e_bias[e] : 0.f);
      if (n_group > 1 && topk_group < n_group) {
        const int gs = E / n_group;
        std::vector<float> gscore(n_group);
        for (int g = 0; g < n_group; ++g) {
          float a = ninf, b = ninf;                 // best and second best of the group
          for (int e = g * gs; e < (g + 1) * gs; ++e) {
            if (sel[e] > a) { b = a; a = sel[e]; } else if (sel[e] > b) { b = sel[e]; }
          }
          gscore[g] = e_bias ? a + b : a;
        }
        std::vector<char> keep(n_group, 0);
        for (int j = 0; j < topk_group; ++j) {
          int best = -1;
          for (int g = 0; g < n_group; ++g)
            if (!keep[g] && (best < 0 || gscore[g] > gscore[best])) best = g;
          keep[best] = 1;
        }
        for (int g = 0; g < n_group; ++g)
          if (!keep[g])
            for (int e = g * gs; e < (g + 1) * gs; ++e) sel[e] = ninf;
      }
      float wsum = 0.f;
      for (int j = 0; j < k; ++j) {
        int best = 0;
        for (int e = 1; e < E; ++e)
          if (sel[e] > sel[best]) best = e;
        ids[t * k + j] = best;
        w[t * k + j] = score[best];
        wsum += score[best];
        sel[best] = ninf;
      }
      for (int j = 0; j < k; ++j) {
        float x = w[t * k + j];
        if (renorm && wsum > 0.f) x /= wsum;
        w[t * k + j] = x * routed_scale;
      }
    }
  });
}

// ------------------------------------------------------------------------------- MoE experts
// out[t] = sum over (expert e in [e0, e0 + e_local), slot j with ids[t, j] == e) of
// w[t, j] * down_e(act(gate_e(x_t)) * up_e(x_t)); gate/up and down outputs are rounded to bf16 as
// the grouped GEMMs of the device path round them; the sum is fp32 in ascending (e, j) order with
// one final rounding. Tokens of one expert run as one GEMM over their gathered rows.
void b200cpu_moe_experts(const uint16_t* x, int64_t ldx, const int32_t* ids, const float* w, int T, int k,
                         const uint16_t* w_gate_up, const uint16_t* w_down, int e0, int e_local, int H, int I,
                         int act_kind, uint16_t* out, int64_t ldo) {
  std::vector<float> acc((size_t)T * H, 0.f);
  std::vector<uint16_t> xs, gu, a, y;
  std::vector<int> rows;
  std::vector<float> wts;
  for (int e = 0; e < e_local; ++e) {
    for (int j = 0; j < k; ++j) {
      rows.clear();
      wts.clear();
      for (int t = 0; t < T; ++t)
        if (ids[(size_t)t * k + j] == e + e0) { rows.push_back(t); wts.push_back(w[(size_t)t * k + j]); }
      const int n = (int)rows.size();
      if (n == 0) continue;
      xs.resize((size_t)n * H);
      gu.resize((size_t)n * 2 * I);
      a.resize((size_t)n * I);
      y.resize((size_t)n * H);
      for (int i = 0; i < n; ++i) std::memcpy(xs.data() + (size_t)i * H, x + (size_t)rows[i] * ldx, (size_t)H * 2);
      b200cpu_matmul_bt(xs.data(), H, w_gate_up + (size_t)e * 2 * I * H, H, gu.data(), 2 * I, 0, nullptr, nullptr, 0,
                        n, 2 * I, H);
      b200cpu_act_and_mul(gu.data(), 2 * I, a.data(), I, n, I, act_kind);
      b200cpu_matmul_bt(a.data(), I, w_down + (size_t)e * H * I, I, y.data(), H, 0, nullptr, nullptr, 0, n, H, I);
      ThreadPool::instance().parallel_for(n, 8, [&](int64_t i0, int64_t i1) {
        for (int64_t i = i0; i < i1; ++i) {
          float* dst = acc.data() + (size_t)rows[i] * H;
          const uint16_t* src = y.data() + (size_t)i * H;
          const float wt = wts[i];
          for (int h = 0; h < H; ++h) dst[h] += wt * bf16_to_f32(src[h]);
        }
      });
    }
  }
  ThreadPool::instance().parallel_for(T, 8, [&](int64_t t0, int64_t t1) {
    for (int64_t t = t0; t < t1; ++t)
      for (int h = 0; h < H; ++h) out[t * ldo + h] = f32_to_bf16(acc[(size_t)t * H + h]);
  });
}

// ------------------------------------------------------------------------------- GDN conv1d
// Causal depthwise conv (kernel 4) + SiLU over ragged sequences. conv_state[slot] is [C, 3]: the
// last three inputs of the sequence, oldest first; read when has_init[s], always written back.
// x, out: [T, C] bf16; w: [C, 4] bf16; qsl: [R + 1] token offsets.
void b200cpu_gdn_conv1d(const uint16_t* x, int64_t ldx, const uint16_t* w, uint16_t* conv_state,
                        const int32_t* qsl, const int32_t* slots, const int32_t* has_init, int R, int C,
                        uint16_t* out, int64_t ldo) {
  for (int s = 0; s < R; ++s) {
    const int b = qsl[s], e = qsl[s + 1], L = e - b;
    if (L <= 0) continue;
    uint16_t* st = conv_state + (size_t)slots[s] * C * 3;
    const bool init = has_init[s] != 0;
    ThreadPool::instance().parallel_for(C, 64, [&](int64_t c0, int64_t c1) {
      for (int64_t c = c0; c < c1; ++c) {
        float hist[3];
        for (int i = 0; i < 3; ++i) hist[i] = init ? bf16_to_f32(st[c * 3 + i]) : 0.f;
        const float w0 = bf16_to_f32(w[c * 4]), w1 = bf16_to_f32(w[c * 4 + 1]), w2 = bf16_to_f32(w[c * 4 + 2]),
                    w3 = bf16_to_f32(w[c * 4 + 3]);
        for (int t = 0; t < L; ++t) {
          const float cur = bf16_to_f32(x[(size_t)(b + t) * ldx + c]);
          // the oracle sums seq[i : i + L] * w[:, i] for i = 0..3 starting from zero
          float acc = 0.f + hist[0] * w0;
          acc += hist[1] * w1;
          acc += hist[2] * w2;
          acc += cur * w3;
          out[(size_t)(b + t) * ldo + c] = f32_to_bf16(silu(acc));
          hist[0] = hist[1]; hist[1] = hist[2]; hist[2] = cur;
        }
        for (int i = 0; i < 3; ++i) st[c * 3 + i] = f32_to_bf16(hist[i]);
      }
    });
  }
}

// q, k: L2-normalised per head (eps inside the square root), rounded to bf16; g = -exp(A_log) *
// softplus(a + dt_bias); beta = sigmoid(b). xc: [T, 2 * Hk * 128 + Hv * 128] (q | k | v).
void b200cpu_gdn_post_conv(const uint16_t* xc, int64_t ldx, int T, int Hk, int Hv, const uint16_t* a, int64_t lda,
                           const uint16_t* b, int64_t ldb, const float* A_log, const float* dt_bias, float eps,
                           uint16_t* q, uint16_t* k, float* g, float* beta) {
  ThreadPool::instance().parallel_for(T, 4, [&](int64_t t0, int64_t t1) {
    for (int64_t t = t0; t < t1; ++t) {
      for (int part = 0; part < 2; ++part) {
        uint16_t* dst = part == 0 ? q : k;
        for (int h = 0; h < Hk; ++h) {
          const uint16_t* src = xc + t * ldx + (size_t)(part * Hk + h) * 128;
          float ss = 0.f;
          for (int d = 0; d < 128; ++d) { const float v = bf16_to_f32(src[d]); ss += v * v; }
          const float inv = 1.f / std::sqrt(ss + eps);
          for (int d = 0; d < 128; ++d) dst[((size_t)t * Hk + h) * 128 + d] = f32_to_bf16(bf16_to_f32(src[d]) * inv);
        }
      }
      for (int h = 0; h < Hv; ++h) {
        g[t * Hv + h] = -std::exp(A_log[h]) * softplus(bf16_to_f32(a[t * lda + h]) + dt_bias[h]);
        beta[t * Hv + h] = sigmoid(bf16_to_f32(b[t * ldb + h]));
      }
    }
  });
}

// Sequential gated delta rule over ragged sequences. Per value head with state S [Dv, Dk]:
//   S *= exp(g_t);  u = (v_t - S k_t) * beta_t;  S += u k_t^T;  o_t = S (q_t / sqrt(Dk)).
// q, k: [T, Hk, 128] bf16 (each key head serves Hv / Hk value heads); v: [T, Hv, 128] bf16 with row
// stride ldv; state: [slots, Hv, 128, 128] fp32, read when has_init[s], always written. out fp32.
void b200cpu_gdn_recurrent(const uint16_t* q, const uint16_t* k, const uint16_t* v, int64_t ldv, const float* g,
                           const float* beta, float* state, const int32_t* qsl, const int32_t* slots,
                           const int32_t* has_init, int R, int Hk, int Hv, float* out) {
  const int D = 128, rep = Hv / Hk;
  const float qscale = 1.f / std::sqrt((float)D);
  ThreadPool::instance().parallel_for((int64_t)R * Hv, 1, [&](int64_t i0, int64_t i1) {
    std::vector<float> kf(D), qf(D);
    for (int64_t i = i0; i < i1; ++i) {
      const int s = (int)(i / Hv), h = (int)(i % Hv), hk = h / rep;
      const int b = qsl[s], e = qsl[s + 1];
      if (e <= b) continue;
      float* S = state + ((size_t)slots[s] * Hv + h) * D * D;
      if (!has_init[s]) std::memset(S, 0, sizeof(float) * D * D);
      for (int t = b; t < e; ++t) {
        const float decay = std::exp(g[(size_t)t * Hv + h]), bt = beta[(size_t)t * Hv + h];
        for (int d = 0; d < D; ++d) {
          kf[d] = bf16_to_f32(k[((size_t)t * Hk + hk) * D + d]);
          qf[d] = bf16_to_f32(q[((size_t)t * Hk + hk) * D + d]) * qscale;
        }
        const uint16_t* vt = v + (size_t)t * ldv + (size_t)h * D;
        float* ot = out + ((size_t)t * Hv + h) * D;
        for (int dv = 0; dv < D; ++dv) {
          float* row = S + (size_t)dv * D;
          float kv = 0.f;
          for (int d = 0; d < D; ++d) { row[d] *= decay; kv += row[d] * kf[d]; }
          const float u = (bf16_to_f32(vt[dv]) - kv) * bt;
          float o = 0.f;
          for (int d = 0; d < D; ++d) { row[d] += u * kf[d]; o += row[d] * qf[d]; }
          ot[dv] = o;
        }
      }
    }
  });
}

// out = rmsnorm(x) * w * silu(z) per head of `hd` columns (gate 0) or * sigmoid(z) (gate 1).
void b200cpu_rmsnorm_gated(const uint16_t* x, int64_t ldx, const uint16_t* z, int64_t ldz, const uint16_t* w, float eps,
                           int T, int heads, int hd, int gate, uint16_t* out, int64_t ldo) {
  ThreadPool::instance().parallel_for((int64_t)T * heads, 16, [&](int64_t i0, int64_t i1) {
    for (int64_t i = i0; i < i1; ++i) {
      const int64_t t = i / heads, h = i % heads;
      const uint16_t* xr = x + t * ldx + h * hd;
      const uint16_t* zr = z + t * ldz + h * hd;
      float ss = 0.f;
      for (int d = 0; d < hd; ++d) { const float v = bf16_to_f32(xr[d]); ss += v * v; }
      const float inv = 1.f / std::sqrt(ss / hd + eps);
      for (int d = 0; d < hd; ++d) {
        const float zz = bf16_to_f32(zr[d]);
        const float y = bf16_to_f32(xr[d]) * inv * bf16_to_f32(w[d]) * (gate == 0 ? silu(zz) : sigmoid(zz));
        out[t * ldo + h * hd + d] = f32_to_bf16(y);
      }
    }
  });
}

// ------------------------------------------------------------------------------- MLA attention
// Attention over the compressed cache, keys and values rebuilt per request: cache rows are
// [latent 512 | rope key 64]; w_kvb [H * 256, 512] holds per head [k_nope 128 | v 128] rows. The
// rebuilt k_nope / v are rounded to bf16 (they are GEMM outputs on the device path). q: [T, H, 192]
// (rope applied to the last 64). Causal: query i of a request with L cached rows and n new ones
// sees rows [0, L - n + i]. out: [T, H, 128] fp32.
void b200cpu_mla_attention(const uint16_t* q, int64_t ldq, const uint16_t* cache, const int32_t* block_table,
                           int64_t max_blocks, const int32_t* seq_lens, const int32_t* query_start, int R,
                           const uint16_t* w_kvb, int H, float scale, int block_size, float* out) {
  const int LAT = 512, ROW = 576, ROPE = 64;
  std::vector<float> kv;          // [L, H, 256] rebuilt keys (first 128) and values (last 128)
  std::vector<float> wk((size_t)H * 256 * LAT);
  for (size_t i = 0; i < wk.size(); ++i) wk[i] = bf16_to_f32(w_kvb[i]);
  for (int r = 0; r < R; ++r) {
    const int b = query_start[r], e = query_start[r + 1], L = seq_lens[r], n = e - b;
    if (n <= 0 || L <= 0) continue;
    const int32_t* bt = block_table + (size_t)r * max_blocks;
    auto row_of = [&](int pos) { return cache + ((size_t)bt[pos / block_size] * block_size + pos % block_size) * ROW; };
    kv.resize((size_t)L * H * 256);
    ThreadPool::instance().parallel_for((int64_t)L * H, 8, [&](int64_t i0, int64_t i1) {
      std::vector<float> lat(LAT);
      int64_t last_pos = -1;
      for (int64_t i = i0; i < i1; ++i) {
        const int pos = (int)(i / H), h = (int)(i % H);
        if (pos != last_pos) {
          const uint16_t* cr = row_of(pos);
          for (int c = 0; c < LAT; ++c) lat[c] = bf16_to_f32(cr[c]);
          last_pos = pos;
        }
        float* dst = kv.data() + ((size_t)pos * H + h) * 256;
        const float* wh = wk.data() + (size_t)h * 256 * LAT;
        for (int d = 0; d < 256; ++d) {
          const float* wr = wh + (size_t)d * LAT;
          float s = 0.f;
          for (int c = 0; c < LAT; ++c) s += lat[c] * wr[c];
          dst[d] = round_bf16(s);
        }
      }
    });
    ThreadPool::instance().parallel_for((int64_t)n * H, 1, [&](int64_t i0, int64_t i1) {
      std::vector<float> p(L);
      for (int64_t i = i0; i < i1; ++i) {
        const int t = (int)(i / H), h = (int)(i % H);
        const int visible = L - n + t + 1;
        const uint16_t* qr = q + (size_t)(b + t) * ldq + (size_t)h * 192;
        float qf[192];
        for (int d = 0; d < 192; ++d) qf[d] = bf16_to_f32(qr[d]);
        float mx = -std::numeric_limits<float>::infinity();
        for (int l = 0; l < visible; ++l) {
          const float* kn = kv.data() + ((size_t)l * H + h) * 256;
          const uint16_t* kr = row_of(l) + LAT;
          float s = 0.f;
          for (int d = 0; d < 128; ++d) s += qf[d] * kn[d];
          for (int d = 0; d < ROPE; ++d) s += qf[128 + d] * bf16_to_f32(kr[d]);
          p[l] = s * scale;
          mx = std::max(mx, p[l]);
        }
        float sum = 0.f;
        for (int l = 0; l < visible; ++l) { p[l] = std::exp(p[l] - mx); sum += p[l]; }
        float* o = out + ((size_t)(b + t) * H + h) * 128;
        for (int d = 0; d < 128; ++d) o[d] = 0.f;
        for (int l = 0; l < visible; ++l) {
          const float pl = p[l] / sum;
          const float* vv = kv.data() + ((size_t)l * H + h) * 256 + 128;
          for (int d = 0; d < 128; ++d) o[d] += pl * vv[d];
        }
      }
    });
  }
}

#if defined(__x86_64__)
static bool quant_has_avx2() {
  static const bool ok = [] {
    const char* e = std::getenv("B200CPU_SIMD");
    if (e && !std::strcmp(e, "scalar")) return false;
    return (bool)__builtin_cpu_supports("avx2");
  }();
  return ok;
}
// 32 int8 weights (one block) against 32 int8 activations: |w| as unsigned bytes times a * sign(w),
// pairs summed to 16-bit (at most 2 * 128 * 127, no saturation), then to 32-bit lanes.
__attribute__((target("avx2"))) static inline int32_t dot32_i8(__m256i w, const int8_t* a) {
  const __m256i av = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(a));
  const __m256i p16 = _mm256_maddubs_epi16(_mm256_abs_epi8(w), _mm256_sign_epi8(av, w));
  const __m256i p32 = _mm256_madd_epi16(p16, _mm256_set1_epi16(1));
  const __m128i s = _mm_add_epi32(_mm256_castsi256_si128(p32), _mm256_extracti128_si256(p32, 1));
  const __m128i t = _mm_add_epi32(s, _mm_shuffle_epi32(s, 0x4e));
  return _mm_cvtsi128_si32(_mm_add_epi32(t, _mm_shuffle_epi32(t, 0xb1)));
}
__attribute__((target("avx2"))) static void quant_row_avx2(const uint8_t* wrow, int kind, int nb, const int8_t* qa,
                                                           const float* da, int M, int K, float* acc) {
  const size_t bb = kind == 8 ? 34 : 18;
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  for (int blk = 0; blk < nb; ++blk) {
    const uint8_t* wb = wrow + (size_t)blk * bb;
    uint16_t dh;
    std::memcpy(&dh, wb, 2);
    const float dw = b200cpu::f16_to_f32(dh);
    __m256i wv;
    if (kind == 8) {
      wv = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(wb + 2));
    } else {
      const __m128i raw = _mm_loadu_si128(reinterpret_cast<const __m128i*>(wb + 2));
      const __m128i lo = _mm_and_si128(raw, _mm_set1_epi8(15));
      const __m128i hi = _mm_and_si128(_mm_srli_epi16(raw, 4), _mm_set1_epi8(15));
      wv = _mm256_sub_epi8(_mm256_set_m128i(hi, lo), _mm256_set1_epi8(8));
    }
    for (int m = 0; m < M; ++m) {
      const int32_t isum = dot32_i8(wv, qa + (size_t)m * K + blk * 32);
      acc[m] += dw * da[(size_t)m * nb + blk] * (float)isum;
    }
  }
}
#endif

// ------------------------------------------------------------------------------- block-quant GEMM
// GGUF blocks of 32 weights: Q8_0 = fp16 scale d + 32 int8 (34 bytes), value d * q; Q4_0 = fp16 d +
// 16 bytes of nibbles (18 bytes), element j in the low nibble of byte j, element j + 16 in the
// high nibble, value d * (nibble - 8). Activations are quantised per row and 32-element block to
// int8 with scale amax / 127 (round to nearest), the block dot product is an integer sum, and the
// row sum is fp32: out[m, n] = sum_blocks d_w * d_a * sum_i qw_i * qa_i.
// kind: 8 = Q8_0, 4 = Q4_0. K must be a multiple of 32. out: fp32 [M, N] (out_f32) or bf16.
void b200cpu_matmul_bt_quant(const uint16_t* A, int64_t lda, const uint8_t* Wq, int kind, void* out, int64_t ldo,
                             int out_f32, int M, int N, int K) {
  const int nb = K / 32;
  const size_t bb = kind == 8 ? 34 : 18;
  std::vector<int8_t> qa((size_t)M * K);
  std::vector<float> da((size_t)M * nb);
  ThreadPool::instance().parallel_for(M, 1, [&](int64_t m0, int64_t m1) {
    for (int64_t m = m0; m < m1; ++m)
      for (int blk = 0; blk < nb; ++blk) {
        const uint16_t* src = A + m * lda + blk * 32;
        float amax = 0.f;
        for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(bf16_to_f32(src[i])));
        const float d = amax / 127.f, id = d > 0.f ? 1.f / d : 0.f;
        da[m * nb + blk] = d;
        for (int i = 0; i < 32; ++i) qa[m * K + blk * 32 + i] = (int8_t)std::lrintf(bf16_to_f32(src[i]) * id);
      }
  });
#if defined(__x86_64__)
  if (quant_has_avx2()) {
    // one weight block is decoded once and meets every activation row; the integer block dot is
    // exact, and each output still sums its blocks in ascending order, so the result has the bits
    // of the scalar loop below
    ThreadPool::instance().parallel_for(N, 4, [&](int64_t n0, int64_t n1) {
      std::vector<float> acc(M);
      for (int64_t n = n0; n < n1; ++n) {
        quant_row_avx2(Wq + (size_t)n * nb * bb, kind, nb, qa.data(), da.data(), M, K, acc.data());
        for (int m = 0; m < M; ++m) {
          if (out_f32) ((float*)out)[(size_t)m * ldo + n] = acc[m];
          else ((uint16_t*)out)[(size_t)m * ldo + n] = f32_to_bf16(acc[m]);
        }
      }
    });
    return;
  }
#endif
  ThreadPool::instance().parallel_for(N, 4, [&](int64_t n0, int64_t n1) {
    int8_t wq[32];
    for (int64_t n = n0; n < n1; ++n) {
      const uint8_t* wrow = Wq + (size_t)n * nb * bb;
      for (int m = 0; m < M; ++m) {
        float acc = 0.f;
        for (int blk = 0; blk < nb; ++blk) {
          const uint8_t* wb = wrow + (size_t)blk * bb;
          uint16_t dh;
          std::memcpy(&dh, wb, 2);
          const float dw = f16_to_f32(dh);
          if (kind == 8) {
            std::memcpy(wq, wb + 2, 32);
          } else {
            for (int j = 0; j < 16; ++j) {
              wq[j] = (int8_t)((wb[2 + j] & 15) - 8);
              wq[j + 16] = (int8_t)((wb[2 + j] >> 4) - 8);
            }
          }
          const int8_t* a8 = qa.data() + (size_t)m * K + blk * 32;
          int32_t isum = 0;
          for (int i = 0; i < 32; ++i) isum += (int32_t)wq[i] * (int32_t)a8[i];
          acc += dw * da[(size_t)m * nb + blk] * (float)isum;
        }
        if (out_f32) ((float*)out)[(size_t)m * ldo + n] = acc;
        else ((uint16_t*)out)[(size_t)m * ldo + n] = f32_to_bf16(acc);
      }
    }
  });
}

// fp32 / bf16 rows -> Q8_0 or Q4_0 blocks (the GGUF encoders: Q8_0 scale amax / 127; Q4_0 scale
// max-magnitude value / -8, codes clamp(round(x / d + 8.5 truncated), 0, 15)). For tests and for
// packing weights that arrive unquantised.
void b200cpu_quantize_blocks(const float* x, int64_t n, int kind, uint8_t* out) {
  const int64_t nb = n / 32;
  ThreadPool::instance().parallel_for(nb, 64, [&](int64_t b0, int64_t b1) {
    for (int64_t blk = b0; blk < b1; ++blk) {
      const float* src = x + blk * 32;
      if (kind == 8) {
        uint8_t* dst = out + blk * 34;
        float amax = 0.f;
        for (int i = 0; i < 32; ++i) amax = std::max(amax, std::fabs(src[i]));
        const float d = amax / 127.f, id = d > 0.f ? 1.f / d : 0.f;
        const uint16_t dh = f32_to_f16(d);
        std::memcpy(dst, &dh, 2);
        for (int i = 0; i < 32; ++i) dst[2 + i] = (uint8_t)(int8_t)std::lrintf(src[i] * id);
      } else {
        uint8_t* dst = out + blk * 18;
        float amax = 0.f, mval = 0.f;
        for (int i = 0; i < 32; ++i)
          if (std::fabs(src[i]) > amax) { amax = std::fabs(src[i]); mval = src[i]; }
        const float d = mval / -8.f, id = d != 0.f ? 1.f / d : 0.f;
        const uint16_t dh = f32_to_f16(d);
        std::memcpy(dst, &dh, 2);
        for (int j = 0; j < 16; ++j) {
          const int lo = std::min(15, (int)(src[j] * id + 8.5f));
          const int hi = std::min(15, (int)(src[j + 16] * id + 8.5f));
          dst[2 + j] = (uint8_t)((lo < 0 ? 0 : lo) | ((hi < 0 ? 0 : hi) << 4));
        }
      }
    }
  });
}

}  // extern "C"
