// Native CPU backend: the ops of a dense decoder forward pass on bf16 storage with fp32
// arithmetic, threaded over outputs (see cpu_threadpool.h), AVX2 + FMA inner loops with a
// scalar tier chosen at run time. Rounding points match the PyTorch oracle of the test-suite
// (ops/reference.py): every op rounds to bf16 exactly where the oracle does.
//
// Reference: src/vt/cpu/{cpu_matmul_elem,cpu_ops,cpu_paged_attn,cpu_cache}.cpp.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

#if defined(__x86_64__)
#include <immintrin.h>
#if defined(__linux__)
#include <sys/syscall.h>
#include <unistd.h>
#endif
#endif

#include "cpu_common.h"
#include "cpu_threadpool.h"

namespace b200cpu {

static int simd_cap() {
  static const int cap = [] {
    const char* e = std::getenv("B200CPU_SIMD");
    if (e && !std::strcmp(e, "scalar")) return 0;
    if (e && !std::strcmp(e, "avx2")) return 2;
    if (e && !std::strcmp(e, "avx512")) return 3;
    return 4;
  }();
  return cap;
}
static bool has_avx2() {
#if defined(__x86_64__)
  static const bool ok = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma") && simd_cap() >= 2;
  return ok;
#else
  return false;
#endif
}

// ------------------------------------------------------------------------------- dot products
static float dot_bf16_f32_scalar(const bf16_t* w, const float* a, int K) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};       // same 8-lane order as the vector tier
  int k = 0;
  for (; k + 8 <= K; k += 8)
    for (int j = 0; j < 8; ++j) acc[j] = std::fmaf(bf16_to_f32(w[k + j]), a[k + j], acc[j]);
  float s = ((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]));
  for (; k < K; ++k) s = std::fmaf(bf16_to_f32(w[k]), a[k], s);
  return s;
}

#if defined(__x86_64__)
__attribute__((target("avx2,fma"))) static inline __m256 load_bf16x8(const bf16_t* p) {
  const __m128i h = _mm_loadu_si128(reinterpret_cast<const __m128i*>(p));
  return _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_cvtepu16_epi32(h), 16));
}
__attribute__((target("avx2,fma"))) static inline float hsum8(__m256 v) {
  // ((0+4)+(2+6)) + ((1+5)+(3+7)): fixed order, mirrored by the scalar tier
  const __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
  const __m128 s = _mm_add_ps(lo, hi);                       // 0+4, 1+5, 2+6, 3+7
  const __m128 t = _mm_add_ps(s, _mm_movehl_ps(s, s));       // (0+4)+(2+6), (1+5)+(3+7)
  return _mm_cvtss_f32(_mm_add_ss(t, _mm_shuffle_ps(t, t, 1)));
}
// One weight row against MB activation rows (fp32), K a multiple of 8 handled in the vector
// loop, the tail in scalar.
template <int MB>
__attribute__((target("avx2,fma"))) static void dot_rows_avx2(const bf16_t* w, const float* a, int lda, int K,
                                                              float* out) {
  __m256 acc[MB];
  for (int m = 0; m < MB; ++m) acc[m] = _mm256_setzero_ps();
  int k = 0;
  for (; k + 8 <= K; k += 8) {
    const __m256 wv = load_bf16x8(w + k);
    for (int m = 0; m < MB; ++m) acc[m] = _mm256_fmadd_ps(wv, _mm256_loadu_ps(a + (size_t)m * lda + k), acc[m]);
  }
  for (int m = 0; m < MB; ++m) {
    float s = hsum8(acc[m]);
    for (int kk = k; kk < K; ++kk) s = std::fmaf(bf16_to_f32(w[kk]), a[(size_t)m * lda + kk], s);
    out[m] = s;
  }
}
__attribute__((target("avx2,fma"))) static float dot_bf16_bf16_avx2(const bf16_t* a, const bf16_t* b, int D) {
  __m256 acc = _mm256_setzero_ps();
  int k = 0;
  for (; k + 8 <= D; k += 8) acc = _mm256_fmadd_ps(load_bf16x8(a + k), load_bf16x8(b + k), acc);
  float s = hsum8(acc);
  for (; k < D; ++k) s = std::fmaf(bf16_to_f32(a[k]), bf16_to_f32(b[k]), s);
  return s;
}
__attribute__((target("avx2,fma"))) static void axpy_bf16_avx2(float p, const bf16_t* v, float* acc, int D) {
  const __m256 pv = _mm256_set1_ps(p);
  int k = 0;
  for (; k + 8 <= D; k += 8)
    _mm256_storeu_ps(acc + k, _mm256_fmadd_ps(pv, load_bf16x8(v + k), _mm256_loadu_ps(acc + k)));
  for (; k < D; ++k) acc[k] = std::fmaf(p, bf16_to_f32(v[k]), acc[k]);
}
#endif

#if defined(__x86_64__)
// ------------------------------------------------------------------ AVX-512 BF16 tier (GEMM)
// vdpbf16ps multiplies 32 bf16 pairs and adds them into 16 fp32 lanes, so neither operand is
// widened first and one instruction does the work of four AVX2 FMAs. B200CPU_SIMD=avx2 (or
// scalar) in the environment keeps the narrower tiers, for comparing them.
static bool has_avx512bf16() {
  static const bool ok = __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") &&
                         __builtin_cpu_supports("avx512vl") && __builtin_cpu_supports("avx512bf16");
  return ok && simd_cap() >= 3;
}
#define B200_T512 __attribute__((target("avx512f,avx512bw,avx512vl,avx512bf16,avx2,fma")))
B200_T512 static inline float hsum16(__m512 v) {
  // lanes i and i + 8 first, then the 8-lane order of the other tiers
  const __m256 s = _mm256_add_ps(_mm512_castps512_ps256(v),
                                 _mm256_castpd_ps(_mm512_extractf64x4_pd(_mm512_castps_pd(v), 1)));
  return hsum8(s);
}
// MB activation rows x NB weight rows: MB * NB accumulators stay in registers over the whole K
// loop (6 x 4 = 24 of the 32 vector registers), every 64-byte load of A is used NB times and
// every load of W MB times. Each output's sum runs over K in the same order whatever the block
// it falls in, so results do not depend on the batch size or the thread partition.
template <int MB, int NB>
B200_T512 static void gemm_block_512(const bf16_t* a, int64_t lda, const bf16_t* w, int64_t ldw, int K, float* out) {
  __m512 acc[MB][NB];
  for (int m = 0; m < MB; ++m)
    for (int n = 0; n < NB; ++n) acc[m][n] = _mm512_setzero_ps();
  int k = 0;
  for (; k + 32 <= K; k += 32) {
    __m512bh wv[NB];
    for (int n = 0; n < NB; ++n) wv[n] = (__m512bh)_mm512_loadu_si512(w + n * ldw + k);
    for (int m = 0; m < MB; ++m) {
      const __m512bh av = (__m512bh)_mm512_loadu_si512(a + m * lda + k);
      for (int n = 0; n < NB; ++n) acc[m][n] = _mm512_dpbf16_ps(acc[m][n], av, wv[n]);
    }
  }
  for (int m = 0; m < MB; ++m) {
    if (NB == 4) {
      // four horizontal sums at once, each in hsum16's order: lanes i + (i + 8), then
      // ((0+4)+(2+6)) + ((1+5)+(3+7)) through a 4 x 4 transpose
      __m128 t[4];
      for (int n = 0; n < 4; ++n) {
        const __m256 h = _mm256_add_ps(_mm512_castps512_ps256(acc[m][n]),
                                       _mm256_castpd_ps(_mm512_extractf64x4_pd(_mm512_castps_pd(acc[m][n]), 1)));
        t[n] = _mm_add_ps(_mm256_castps256_ps128(h), _mm256_extractf128_ps(h, 1));
      }
      _MM_TRANSPOSE4_PS(t[0], t[1], t[2], t[3]);
      _mm_storeu_ps(out + m * 4, _mm_add_ps(_mm_add_ps(t[0], t[2]), _mm_add_ps(t[1], t[3])));
      if (k < K)
        for (int n = 0; n < 4; ++n) {
          float s = out[m * 4 + n];
          for (int kk = k; kk < K; ++kk) s = std::fmaf(bf16_to_f32(w[n * ldw + kk]), bf16_to_f32(a[m * lda + kk]), s);
          out[m * 4 + n] = s;
        }
      continue;
    }
    for (int n = 0; n < NB; ++n) {
      float s = hsum16(acc[m][n]);
      for (int kk = k; kk < K; ++kk) s = std::fmaf(bf16_to_f32(w[n * ldw + kk]), bf16_to_f32(a[m * lda + kk]), s);
      out[m * NB + n] = s;
    }
  }
}
template <int NB>
B200_T512 static void gemm_rows_512(int mb, const bf16_t* a, int64_t lda, const bf16_t* w, int64_t ldw, int K,
                                    float* out) {
  switch (mb) {
    case 6: gemm_block_512<6, NB>(a, lda, w, ldw, K, out); break;
    case 5: gemm_block_512<5, NB>(a, lda, w, ldw, K, out); break;
    case 4: gemm_block_512<4, NB>(a, lda, w, ldw, K, out); break;
    case 3: gemm_block_512<3, NB>(a, lda, w, ldw, K, out); break;
    case 2: gemm_block_512<2, NB>(a, lda, w, ldw, K, out); break;
    default: gemm_block_512<1, NB>(a, lda, w, ldw, K, out); break;
  }
}
#endif

#if defined(__x86_64__) && defined(__linux__)
// ------------------------------------------------------------------ AMX tier (GEMM)
// Tile matrix multiply: one TDPBF16PS does a 16 x 16 x 32 bf16 block (fp32 accumulate). The
// weight matrix [N, K] is the row-major operand as it lies in memory; the activations are packed
// once per call into the pair-interleaved layout the second operand needs ([k / 2][m][2]), so the
// product comes out transposed (C^T[n][m]) and the epilogue writes it back row by row. The kernel
// must ask the kernel for permission to use tile state once per process; each worker thread loads
// its own tile configuration.
struct AmxTileCfg {
  uint8_t palette, start_row;
  uint8_t rsv[14];
  uint16_t colsb[16];
  uint8_t rows[16];
} __attribute__((packed));

static bool has_amx() {
  static const bool ok = [] {
    if (simd_cap() < 4) return false;
    if (!__builtin_cpu_supports("amx-tile") || !__builtin_cpu_supports("amx-bf16") || !has_avx2()) return false;
    return syscall(SYS_arch_prctl, 0x1023 /* ARCH_REQ_XCOMP_PERM */, 18 /* XFEATURE_XTILEDATA */) == 0;
  }();
  return ok;
}

#define B200_TAMX __attribute__((target("amx-tile,amx-bf16,avx2,fma")))
// rows [n0, n0 + 32) of W against all of M. wblk: the 32 weight rows (row stride ldw elements);
// ap: packed activations [mblocks][kblocks][16][32]; ct: scratch [32][32] fp32.
B200_TAMX static void amx_block(const bf16_t* w0, const bf16_t* w1, int64_t ldw, const bf16_t* ap, int mblocks,
                                int kblocks, int mb0, float* ct) {
  // tiles 0..3: C (n-half x m-half), 4 / 5: weight rows, 6 / 7: packed activations
  _tile_zero(0); _tile_zero(1); _tile_zero(2); _tile_zero(3);
  const bf16_t* b0 = ap + (size_t)mb0 * kblocks * 512;
  const bool two_m = mb0 + 1 < mblocks;
  const bf16_t* b1 = two_m ? b0 + (size_t)kblocks * 512 : b0;
  // a decode-sized batch streams each weight row once, 64 bytes per k-step from 32 rows that are
  // kilobytes apart: too many streams for the hardware prefetcher, so the lines are asked for ahead
  const bool stream = mblocks <= 2;
  for (int kb = 0; kb < kblocks; ++kb) {
    if (stream && kb + 8 < kblocks) {
      for (int r = 0; r < 16; ++r) {
        _mm_prefetch(reinterpret_cast<const char*>(w0 + r * ldw + (kb + 8) * 32), _MM_HINT_T0);
        _mm_prefetch(reinterpret_cast<const char*>(w1 + r * ldw + (kb + 8) * 32), _MM_HINT_T0);
      }
    }
    _tile_loadd(4, w0 + kb * 32, ldw * 2);
    _tile_loadd(5, w1 + kb * 32, ldw * 2);
    _tile_loadd(6, b0 + (size_t)kb * 512, 64);
    _tile_dpbf16ps(0, 4, 6);
    _tile_dpbf16ps(2, 5, 6);
    if (two_m) {
      _tile_loadd(7, b1 + (size_t)kb * 512, 64);
      _tile_dpbf16ps(1, 4, 7);
      _tile_dpbf16ps(3, 5, 7);
    }
  }
  _tile_stored(0, ct, 128);                 // rows 0..15 (n), columns 0..15 (m)
  _tile_stored(1, ct + 16, 128);            //               columns 16..31
  _tile_stored(2, ct + 16 * 32, 128);       // rows 16..31
  _tile_stored(3, ct + 16 * 32 + 16, 128);
}
B200_TAMX static void amx_load_cfg() {
  AmxTileCfg cfg;
  std::memset(&cfg, 0, sizeof(cfg));
  cfg.palette = 1;
  for (int i = 0; i < 8; ++i) { cfg.colsb[i] = 64; cfg.rows[i] = 16; }
  _tile_loadconfig(&cfg);
}
B200_TAMX static void amx_release() { _tile_release(); }
#endif

static float dot_bf16_bf16(const bf16_t* a, const bf16_t* b, int D) {
#if defined(__x86_64__)
  if (has_avx2()) return dot_bf16_bf16_avx2(a, b, D);
#endif
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int k = 0;
  for (; k + 8 <= D; k += 8)
    for (int j = 0; j < 8; ++j) acc[j] = std::fmaf(bf16_to_f32(a[k + j]), bf16_to_f32(b[k + j]), acc[j]);
  float s = ((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]));
  for (; k < D; ++k) s = std::fmaf(bf16_to_f32(a[k]), bf16_to_f32(b[k]), s);
  return s;
}
static void axpy_bf16(float p, const bf16_t* v, float* acc, int D) {
#if defined(__x86_64__)
  if (has_avx2()) return axpy_bf16_avx2(p, v, acc, D);
#endif
  for (int k = 0; k < D; ++k) acc[k] = std::fmaf(p, bf16_to_f32(v[k]), acc[k]);
}

}  // namespace b200cpu

using namespace b200cpu;

extern "C" {

void b200cpu_set_threads(int n) { ThreadPool::set_num_threads(n); }
int b200cpu_num_threads() { return ThreadPool::instance().size(); }
int b200cpu_simd_tier() {
#if defined(__x86_64__) && defined(__linux__)
  if (has_amx()) return 4;
#endif
#if defined(__x86_64__)
  if (has_avx512bf16()) return 3;
#endif
  return has_avx2() ? 2 : 0;
}

// out[M, N] = A[M, K] W[N, K]^T (+ bias[N]) (+ residual[M, N]); bf16 in, fp32 accumulate, one
// rounding at the end (bf16 or fp32 output). Threads own ranges of output columns; a weight row
// is converted once per block of 8 activation rows.
void b200cpu_matmul_bt(const uint16_t* A, int64_t lda, const uint16_t* W, int64_t ldw, void* out, int64_t ldo,
                       int out_f32, const uint16_t* bias, const uint16_t* residual, int64_t ldr, int M,
                       int N, int K) {
  if (M <= 0 || N <= 0) return;
  ThreadPool& tp = ThreadPool::instance();
#if defined(__x86_64__) && defined(__linux__)
  if (has_amx() && K % 32 == 0 && K >= 32) {
    // every batch size takes this path (rows are padded to 16), so a row's result does not depend
    // on what it is batched with
    const int mblocks = (M + 15) / 16, kblocks = K / 32;
    std::vector<bf16_t> ap((size_t)mblocks * kblocks * 512);
    auto pack = [&](int64_t b0, int64_t b1) {
      for (int64_t mb = b0; mb < b1; ++mb)
        for (int kb = 0; kb < kblocks; ++kb) {
          bf16_t* dst = ap.data() + ((size_t)mb * kblocks + kb) * 512;
          for (int j = 0; j < 16; ++j)
            for (int m = 0; m < 16; ++m) {
              const int64_t row = mb * 16 + m;
              uint32_t pair = 0;
              if (row < M) std::memcpy(&pair, A + row * lda + kb * 32 + 2 * j, 4);
              std::memcpy(dst + j * 32 + m * 2, &pair, 4);
            }
        }
    };
    if (mblocks <= 2) pack(0, mblocks);          // a few kilobytes: not worth waking the pool
    else tp.parallel_for(mblocks, 1, pack);
    const int nblocks = (N + 31) / 32;
    tp.parallel_for(nblocks, 1, [&](int64_t nb0, int64_t nb1) {
      amx_load_cfg();
      alignas(64) float ct[32 * 32];
      std::vector<bf16_t> edge;
      for (int64_t nb = nb0; nb < nb1; ++nb) {
        const int64_t n0 = nb * 32;
        const int nrows = (int)std::min<int64_t>(32, N - n0);
        const bf16_t* w0 = W + n0 * ldw;
        int64_t ld = ldw;
        if (nrows < 32) {                       // last block: its missing rows read as zeros
          edge.assign((size_t)32 * K, 0);
          for (int r = 0; r < nrows; ++r) std::memcpy(edge.data() + (size_t)r * K, W + (n0 + r) * ldw, (size_t)K * 2);
          w0 = edge.data();
          ld = K;
        }
        for (int mb = 0; mb < mblocks; mb += 2) {
          amx_block(w0, w0 + 16 * ld, ld, ap.data(), mblocks, kblocks, mb, ct);
          const int mrows = std::min(32, M - mb * 16);
          for (int i = 0; i < mrows; ++i) {
            const int64_t m = (int64_t)mb * 16 + i;
            for (int j = 0; j < nrows; ++j) {
              const int64_t n = n0 + j;
              float v = ct[j * 32 + i];
              if (bias) v = v + bf16_to_f32(bias[n]);
              if (residual) v = v + bf16_to_f32(residual[m * ldr + n]);
              if (out_f32) reinterpret_cast<float*>(out)[m * ldo + n] = v;
              else reinterpret_cast<uint16_t*>(out)[m * ldo + n] = f32_to_bf16(v);
            }
          }
        }
      }
      amx_release();
    });
    return;
  }
#endif
#if defined(__x86_64__)
  if (has_avx512bf16()) {
    auto store = [&](int64_t m, int64_t n, float v) {
      if (bias) v = v + bf16_to_f32(bias[n]);
      if (residual) v = v + bf16_to_f32(residual[m * ldr + n]);
      if (out_f32) reinterpret_cast<float*>(out)[m * ldo + n] = v;
      else reinterpret_cast<uint16_t*>(out)[m * ldo + n] = f32_to_bf16(v);
    };
    tp.parallel_for(N, 16, [&](int64_t n0, int64_t n1) {
      float tmp[6 * 4];
      for (int64_t n = n0; n < n1; n += 4) {
        const int nb = (int)std::min<int64_t>(4, n1 - n);
        for (int m = 0; m < M; m += 6) {
          const int mb = std::min(6, M - m);
          const bf16_t* a = A + (int64_t)m * lda;
          const bf16_t* w = W + n * ldw;
          switch (nb) {
            case 4: gemm_rows_512<4>(mb, a, lda, w, ldw, K, tmp); break;
            case 3: gemm_rows_512<3>(mb, a, lda, w, ldw, K, tmp); break;
            case 2: gemm_rows_512<2>(mb, a, lda, w, ldw, K, tmp); break;
            default: gemm_rows_512<1>(mb, a, lda, w, ldw, K, tmp); break;
          }
          for (int i = 0; i < mb; ++i)
            for (int j = 0; j < nb; ++j) store(m + i, n + j, tmp[i * nb + j]);
        }
      }
    });
    return;
  }
#endif
  std::vector<float> af((size_t)M * K);
  tp.parallel_for(M, 1, [&](int64_t m0, int64_t m1) {
    for (int64_t m = m0; m < m1; ++m)
      for (int k = 0; k < K; ++k) af[(size_t)m * K + k] = bf16_to_f32(A[m * lda + k]);
  });
  const bool vec = has_avx2();
  tp.parallel_for(N, 16, [&](int64_t n0, int64_t n1) {
    float tmp[8];
    for (int64_t n = n0; n < n1; ++n) {
      const uint16_t* w = W + n * ldw;
      const float b = bias ? bf16_to_f32(bias[n]) : 0.f;
      for (int m = 0; m < M; m += 8) {
        const int mb = std::min(8, M - m);
        const float* a = af.data() + (size_t)m * K;
#if defined(__x86_64__)
        if (vec) {
          switch (mb) {
            case 8: dot_rows_avx2<8>(w, a, K, K, tmp); break;
            case 7: dot_rows_avx2<7>(w, a, K, K, tmp); break;
            case 6: dot_rows_avx2<6>(w, a, K, K, tmp); break;
            case 5: dot_rows_avx2<5>(w, a, K, K, tmp); break;
            case 4: dot_rows_avx2<4>(w, a, K, K, tmp); break;
            case 3: dot_rows_avx2<3>(w, a, K, K, tmp); break;
            case 2: dot_rows_avx2<2>(w, a, K, K, tmp); break;
            default: dot_rows_avx2<1>(w, a, K, K, tmp); break;
          }
        } else
#endif
        {
          for (int i = 0; i < mb; ++i) tmp[i] = dot_bf16_f32_scalar(w, a + (size_t)i * K, K);
        }
        for (int i = 0; i < mb; ++i) {
          float v = tmp[i];
          if (bias) v = v + b;
          if (residual) v = v + bf16_to_f32(residual[(int64_t)(m + i) * ldr + n]);
          if (out_f32) reinterpret_cast<float*>(out)[(int64_t)(m + i) * ldo + n] = v;
          else reinterpret_cast<uint16_t*>(out)[(int64_t)(m + i) * ldo + n] = f32_to_bf16(v);
        }
      }
    }
  });
}

// residual (optional, in place): r = bf16(x + residual); out = bf16(r * rsqrt(mean(r^2) + eps) * (w [+ 1])).
void b200cpu_rmsnorm(const uint16_t* x, int64_t ldx, const uint16_t* w, float eps, uint16_t* residual,
                     int64_t ldr, uint16_t* out, int64_t ldo, int T, int H, int gemma) {
  // a part is worth a thread from about 32 K elements on; decode-sized calls run inline
  ThreadPool::instance().parallel_for(T, std::max(1, 32768 / std::max(1, H)), [&](int64_t t0, int64_t t1) {
    std::vector<float> row(H);
    for (int64_t t = t0; t < t1; ++t) {
      double ss = 0.0;
      for (int i = 0; i < H; ++i) {
        float v = bf16_to_f32(x[t * ldx + i]);
        if (residual) {
          const uint16_t r = f32_to_bf16(v + bf16_to_f32(residual[t * ldr + i]));
          residual[t * ldr + i] = r;
          v = bf16_to_f32(r);
        }
        row[i] = v;
        ss += (double)v * v;
      }
      const float inv = 1.0f / std::sqrt((float)(ss / H) + eps);
      for (int i = 0; i < H; ++i) {
        const float wf = bf16_to_f32(w[i]) + (gemma ? 1.f : 0.f);
        out[t * ldo + i] = f32_to_bf16(row[i] * inv * wf);
      }
    }
  });
}

// x = [gate | up]; out = bf16(act(gate) * up). kind: 0 SiLU, 1 GELU-tanh, 2 GELU-erf.
void b200cpu_act_and_mul(const uint16_t* x, int64_t ldx, uint16_t* out, int64_t ldo, int T, int I, int kind) {
  ThreadPool::instance().parallel_for(T, std::max(1, 16384 / std::max(1, I)), [&](int64_t t0, int64_t t1) {
    for (int64_t t = t0; t < t1; ++t)
      for (int i = 0; i < I; ++i) {
        const float g = bf16_to_f32(x[t * ldx + i]), u = bf16_to_f32(x[t * ldx + I + i]);
        float a;
        if (kind == 0) a = g * (1.f / (1.f + std::exp(-g)));
        else if (kind == 1) a = 0.5f * g * (1.f + std::tanh(0.7978845608028654f * (g + 0.044715f * g * g * g)));
        else a = 0.5f * g * (1.f + std::erf(g * 0.7071067811865476f));
        out[t * ldo + i] = f32_to_bf16(a * u);
      }
  });
}

void b200cpu_embedding(const int64_t* ids, const uint16_t* table, uint16_t* out, int64_t ldo, int T, int H,
                       int64_t vocab_start, int64_t rows, float scale) {
  ThreadPool::instance().parallel_for(T, 8, [&](int64_t t0, int64_t t1) {
    for (int64_t t = t0; t < t1; ++t) {
      const int64_t local = ids[t] - vocab_start;
      if (local < 0 || local >= rows) {
        std::memset(out + t * ldo, 0, (size_t)H * 2);
        continue;
      }
      const uint16_t* src = table + local * H;
      if (scale == 1.f) std::memcpy(out + t * ldo, src, (size_t)H * 2);
      else for (int i = 0; i < H; ++i) out[t * ldo + i] = f32_to_bf16(bf16_to_f32(src[i]) * scale);
    }
  });
}

// Per-head RMSNorm (optional) + rotary embedding on the q and k columns of qkv [T, ld]; q is
// rewritten in place, rotated k and v go to the paged cache [blocks, 2, block_size, Hkv, D] at
// slot_mapping[t] (negative = skip). table: fp32 [max_pos, rot] = [cos | sin].
void b200cpu_rope_kv(uint16_t* qkv, int64_t ld, const int64_t* positions, const float* table, int T, int Hq,
                     int Hkv, int D, int rot, int neox, const uint16_t* q_norm, const uint16_t* k_norm,
                     float eps, int gemma, const int64_t* slot_mapping, uint16_t* kv_cache, int block_size) {
  const int half = rot / 2;
  ThreadPool::instance().parallel_for(T, std::max(1, 32768 / std::max(1, (Hq + Hkv) * D)), [&](int64_t t0, int64_t t1) {
    std::vector<float> buf(D);
    std::vector<uint16_t> krow((size_t)Hkv * D);
    for (int64_t t = t0; t < t1; ++t) {
      const float* cs = table ? table + positions[t] * rot : nullptr;
      auto head = [&](uint16_t* h, const uint16_t* nw, uint16_t* dst) {
        for (int i = 0; i < D; ++i) buf[i] = bf16_to_f32(h[i]);
        if (nw) {
          double ss = 0.0;
          for (int i = 0; i < D; ++i) ss += (double)buf[i] * buf[i];
          const float inv = 1.0f / std::sqrt((float)(ss / D) + eps);
          for (int i = 0; i < D; ++i)
            buf[i] = bf16_to_f32(f32_to_bf16(buf[i] * inv * (bf16_to_f32(nw[i]) + (gemma ? 1.f : 0.f))));
        }
        if (cs) {
          for (int i = 0; i < half; ++i) {
            const int a = neox ? i : 2 * i, b = neox ? i + half : 2 * i + 1;
            const float x1 = buf[a], x2 = buf[b], c = cs[i], s = cs[half + i];
            buf[a] = x1 * c - x2 * s;
            buf[b] = x2 * c + x1 * s;
          }
        }
        for (int i = 0; i < D; ++i) dst[i] = f32_to_bf16(buf[i]);
      };
      uint16_t* row = qkv + t * ld;
      for (int h = 0; h < Hq; ++h) head(row + (size_t)h * D, q_norm, row + (size_t)h * D);
      for (int h = 0; h < Hkv; ++h) head(row + (size_t)(Hq + h) * D, k_norm, krow.data() + (size_t)h * D);
      if (kv_cache && slot_mapping && slot_mapping[t] >= 0) {
        const int64_t slot = slot_mapping[t], blk = slot / block_size, off = slot % block_size;
        uint16_t* kdst = kv_cache + ((blk * 2 + 0) * block_size + off) * (int64_t)Hkv * D;
        uint16_t* vdst = kv_cache + ((blk * 2 + 1) * block_size + off) * (int64_t)Hkv * D;
        std::memcpy(kdst, krow.data(), (size_t)Hkv * D * 2);
        std::memcpy(vdst, row + (size_t)(Hq + Hkv) * D, (size_t)Hkv * D * 2);
      }
    }
  });
}

// Varlen paged attention with a bottom-right aligned causal mask (query t of request r sits at
// position seq_len - q_len + (t - q_start)), optional sliding window and logit soft-cap.
// Threads own (query token, q head) pairs; two-pass softmax in fp32.
void b200cpu_paged_attention(const uint16_t* q, int64_t ldq, const uint16_t* kv_cache, const int32_t* block_table,
                             int64_t max_blocks, const int32_t* seq_lens, const int32_t* q_start, int R, int Hq,
                             int Hkv, int D, int block_size, float scale, float softcap, int window,
                             uint16_t* out, int64_t ldo) {
  const int G = Hq / Hkv;
  std::vector<int> tok_req;
  const int T = q_start[R];
  tok_req.resize(T);
  for (int r = 0; r < R; ++r)
    for (int t = q_start[r]; t < q_start[r + 1]; ++t) tok_req[t] = r;
  ThreadPool::instance().parallel_for((int64_t)T * Hq, 1, [&](int64_t i0, int64_t i1) {
    std::vector<float> s, acc(D);
    for (int64_t idx = i0; idx < i1; ++idx) {
      const int t = (int)(idx / Hq), h = (int)(idx % Hq), r = tok_req[t];
      const int sl = seq_lens[r], ql = q_start[r + 1] - q_start[r];
      uint16_t* o = out + (int64_t)t * ldo + (size_t)h * D;
      if (sl <= 0 || ql <= 0) {
        std::memset(o, 0, (size_t)D * 2);
        continue;
      }
      const int qpos = sl - ql + (t - q_start[r]);
      const int k_lo = window > 0 ? std::max(0, qpos - window + 1) : (window < 0 ? (qpos / -window) * -window : 0),
                k_hi = std::min(sl - 1, qpos);
      const int hk = h / G;
      const uint16_t* qv = q + (int64_t)t * ldq + (size_t)h * D;
      const int32_t* bt = block_table + (int64_t)r * max_blocks;
      const int n = k_hi - k_lo + 1;
      if (n <= 0) {
        std::memset(o, 0, (size_t)D * 2);
        continue;
      }
      s.resize(n);
      float mx = -INFINITY;
      for (int j = 0; j < n; ++j) {
        const int p = k_lo + j;
        const uint16_t* kr = kv_cache + (((int64_t)bt[p / block_size] * 2 + 0) * block_size + p % block_size) *
                                            (int64_t)Hkv * D + (size_t)hk * D;
        float v = dot_bf16_bf16(qv, kr, D) * scale;
        if (softcap > 0.f) v = softcap * std::tanh(v / softcap);
        s[j] = v;
        mx = std::max(mx, v);
      }
      float sum = 0.f;
      for (int j = 0; j < n; ++j) {
        s[j] = std::exp(s[j] - mx);
        sum += s[j];
      }
      std::fill(acc.begin(), acc.end(), 0.f);
      const float inv = 1.f / sum;
      for (int j = 0; j < n; ++j) {
        const int p = k_lo + j;
        const uint16_t* vr = kv_cache + (((int64_t)bt[p / block_size] * 2 + 1) * block_size + p % block_size) *
                                            (int64_t)Hkv * D + (size_t)hk * D;
        axpy_bf16(s[j] * inv, vr, acc.data(), D);
      }
      for (int i = 0; i < D; ++i) o[i] = f32_to_bf16(acc[i]);
    }
  });
}

}  // extern "C"
