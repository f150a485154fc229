// Gated-delta-rule chunked prefill on tcgen05 tensor cores (chunk = 64 tokens, Dk = Dv = 128).
//
// For one (sequence, value head) with per-token decay g, write gate beta, normalised q / k and
// values v, the recurrence  S <- S e^g ; v' = (v - S k) beta ; S <- S + v' (x) k ; o = S q
// is evaluated chunk-wise (WY form). With G = in-chunk cumulative sum of g:
//     A[i,j] = beta_i e^{G_i - G_j} (k_i . k_j)   (j < i),   T = (I + A)^-1
//     u = T (beta v),  w = T (beta e^G k)                                   (per chunk, parallel)
//     v_new = u - w h ;  o = (q e^G) h + mask(e^{G_i - G_j} q_i . k_j) v_new ;
//     h <- h e^{G_last} + k^T (v_new e^{G_last - G})                        (sequential in chunks)
// Reference (same math as FLA's chunk_gated_delta_rule): src/vt/cuda/cuda_gdn.cu:2496-2521
// (formulas), :2554 (GdnChunkWUKernel), :2614 (GdnChunkDeltaHKernel), :2670 (GdnChunkOKernel).
//
// Two kernels, every matrix product an M = 128 tcgen05.mma with operands staged by TMA:
//   gdn_chunk_prep_kernel   grid (chunks, Hv): [K;Q] K^T in one MMA (rows 0-63 = K K^T, rows
//       64-127 = Q K^T), forward substitution for T on CUDA cores, then u^T = V^T T'^T and
//       w^T = K^T T''^T with V / K consumed as MN-major A operands straight from their TMA tiles.
//   gdn_chunk_scan_kernel   grid (sequences * Hv): the state h^T [Dv, Dk] lives in TMEM (fp32)
//       for the whole sequence; per chunk two MMAs against its bf16 copy (w h and q h), an
//       epilogue forming v_new, and two accumulating MMAs (state update, intra-chunk output).
// Rows past the end of a sequence inside its last chunk get beta = 0 and g = 0, which makes
// their u / w rows exactly zero, so neighbouring sequences' tokens in a TMA box are harmless.
#include "api.h"
#include "sm100.cuh"

namespace b200 {

typedef __nv_bfloat16 bf16;

static constexpr int kC = 64;      // chunk length
static constexpr int kD = 128;     // Dk = Dv
static constexpr int kScanThreads = 160;   // 4 compute warps + 1 control warp

struct ScanBars {
  uint64_t load[2];
  uint64_t mma[2];
  uint32_t tmem_base;
  int failed;
};

// byte offset of element (row, col) in a K-major SWIZZLE_128B tile whose rows are 64 bf16
__device__ __forceinline__ uint32_t sw128_off(int row, int col) {
  return (uint32_t)row * 128u + ((((uint32_t)col >> 3) ^ ((uint32_t)row & 7u)) << 4) + ((uint32_t)col & 7u) * 2u;
}

struct PrepParams {
  const float* g;        // [T, Hv]
  const float* beta;     // [T, Hv]
  const bf16* q;         // [T, Hk, 128] normalised (for q')
  const int* chunk_tok0; // [NT]
  const int* chunk_len;  // [NT]
  bf16* u;               // [NT*64, Hv, 128]
  bf16* w;               // [NT*64, Hv, 128]
  bf16* qs;              // [NT*64, Hv, 128]  q e^G Dk^-0.5
  bf16* p;               // [NT, Hv, 64, 64]  masked decayed q k^T (scaled)
  float* gc;             // [NT, Hv, 64]      in-chunk cumulative g
  int Hk, Hv;
  int v_col0;            // column of v head 0 inside the tensor tmV describes
  int* status;
};

__global__ void __launch_bounds__(kScanThreads, 2)
    gdn_chunk_prep_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                          const __grid_constant__ CUtensorMap tmV, PrepParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sKQ = smem;                    // 2 halves x (64 K rows + 64 Q rows) x 128 B
  uint8_t* sV = sKQ + 32768;              // 2 halves x 64 rows x 128 B
  uint8_t* sT1 = sV + 16384;              // [i][j] T beta_j            (B operand, K-major)
  uint8_t* sT2 = sT1 + 8192;              // [i][j] T beta_j e^{G_j}
  float* sA = reinterpret_cast<float*>(sT2 + 8192);     // [64][65]
  float* sT = sA + 64 * 65;                              // [64][65]
  float* sG = sT + 64 * 65;                              // [64]
  float* sBeta = sG + 64;                                // [64]
  ScanBars* bars = reinterpret_cast<ScanBars*>(sBeta + 64);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int n = blockIdx.x, hv = blockIdx.y;
  const int hk = hv / (p.Hv / p.Hk);
  const int tok0 = p.chunk_tok0[n], len = p.chunk_len[n];
  const bool control = (tid == 128);

  if (tid == 0) {
    mbar_init(&bars->load[0], 1);
    mbar_init(&bars->mma[0], 1);
    mbar_init(&bars->mma[1], 1);
    bars->failed = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(&bars->tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  const uint32_t tmem_s = tmem, tmem_u = tmem + 64, tmem_w = tmem + 128;

  if (control) {
    mbar_expect_tx(&bars->load[0], 32768 + 16384);
    for (int h = 0; h < 2; ++h) {
      tma_load_2d(sKQ + h * 16384, &tmK, &bars->load[0], hk * kD + h * 64, tok0);
      tma_load_2d(sKQ + h * 16384 + 8192, &tmQ, &bars->load[0], hk * kD + h * 64, tok0);
      tma_load_2d(sV + h * 8192, &tmV, &bars->load[0], p.v_col0 + hv * kD + h * 64, tok0);
    }
  }
  if (tid < 64) {
    const bool valid = tid < len;
    sG[tid] = valid ? p.g[(size_t)(tok0 + tid) * p.Hv + hv] : 0.f;
    sBeta[tid] = valid ? p.beta[(size_t)(tok0 + tid) * p.Hv + hv] : 0.f;
  }
  __syncthreads();
  if (tid == 0) {
    float acc = 0.f;
    for (int i = 0; i < kC; ++i) { acc += sG[i]; sG[i] = acc; }
  }
  bool ok = true;
  if (control) {
    ok = mbar_wait(&bars->load[0], 0, p.status);
    if (ok) {
      tc_fence_after_sync();
      constexpr uint32_t idesc = umma_idesc_bf16(128, 64, 0, 0);
      const uint32_t a0 = smem_u32(sKQ);
#pragma unroll
      for (int kk = 0; kk < kD / 16; ++kk) {
        const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;
        umma_bf16_ss(tmem_s, umma_desc_k_sw128(a0 + off, 1024), umma_desc_k_sw128(a0 + off, 1024), idesc, kk != 0);
      }
      umma_commit(&bars->mma[0]);
    } else {
      bars->failed = 1;
    }
  }
  __syncthreads();   // sG cumulative sums visible; control has issued (or failed)
  if (tid < 128) p.gc[((size_t)n * p.Hv + hv) * kC + (tid & 63)] = sG[tid & 63];

  if (tid < 128 && !bars->failed) {
    ok = mbar_wait(&bars->mma[0], 0, p.status);
    if (!ok) bars->failed = 1;
  }
  if (tid < 128 && ok && !bars->failed) {
    tc_fence_after_sync();
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    uint32_t r0[32], r1[32];
    tmem_ld_32x32b_x32(tmem_s + lane_off, r0);
    tmem_ld_32x32b_x32(tmem_s + lane_off + 32, r1);
    tmem_ld_wait();
    tc_fence_before_sync();
    if (tid < 64) {
      const int i = tid;
      const float gi = sG[i], bi = sBeta[i];
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        const float kkv = __uint_as_float(j < 32 ? r0[j & 31] : r1[j & 31]);
        sA[i * 65 + j] = (j < i) ? bi * __expf(gi - sG[j]) * kkv : 0.f;
      }
    } else {
      const int i = tid - 64;
      const float gi = sG[i];
      const float scale = 0.08838834764831845f;   // Dk^-0.5
      bf16* prow = p.p + (((size_t)n * p.Hv + hv) * kC + i) * kC;
#pragma unroll
      for (int j8 = 0; j8 < 8; ++j8) {
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j8 * 8 + e * 2;
          const float v0 = __uint_as_float(j < 32 ? r0[j & 31] : r1[j & 31]);
          const float v1 = __uint_as_float((j + 1) < 32 ? r0[(j + 1) & 31] : r1[(j + 1) & 31]);
          const float p0 = (j <= i) ? __expf(gi - sG[j]) * v0 * scale : 0.f;
          const float p1 = (j + 1 <= i) ? __expf(gi - sG[j + 1]) * v1 * scale : 0.f;
          pk[e] = pack_bf16x2(p0, p1);
        }
        reinterpret_cast<uint4*>(prow)[j8] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      // q' = q e^{G_i} Dk^-0.5 into the chunk-indexed buffer
      const float f = __expf(gi) * scale;
      const int tq = tok0 + (i < len ? i : 0);
      const uint4* qrow = reinterpret_cast<const uint4*>(p.q + ((size_t)tq * p.Hk + hk) * kD);
      uint4* qd = reinterpret_cast<uint4*>(p.qs + (((size_t)n * kC + i) * p.Hv + hv) * kD);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        uint4 v = qrow[c];
        float2 a;
        a = unpack_bf16x2(v.x); v.x = pack_bf16x2(a.x * f, a.y * f);
        a = unpack_bf16x2(v.y); v.y = pack_bf16x2(a.x * f, a.y * f);
        a = unpack_bf16x2(v.z); v.z = pack_bf16x2(a.x * f, a.y * f);
        a = unpack_bf16x2(v.w); v.w = pack_bf16x2(a.x * f, a.y * f);
        qd[c] = v;
      }
    }
  }
  __syncthreads();
  const bool failed_a = bars->failed != 0;

  // forward substitution: column c of T = (I + A)^-1 depends only on earlier entries of the
  // same column, so a pair of lanes owns a column (even / odd j) and never waits on others.
  if (tid < 128 && !failed_a) {
    const int c = tid >> 1, half = tid & 1;
    for (int i = 0; i < kC; ++i) {
      float acc = 0.f;   // the loop is empty for i <= c; the shuffle stays warp-uniform
      for (int j = c + half; j < i; j += 2) acc += sA[i * 65 + j] * sT[j * 65 + c];
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      const float v = i < c ? 0.f : (i == c ? 1.f : -acc);
      if (half == 0) sT[i * 65 + c] = v;
      __syncwarp();
    }
  }
  __syncthreads();
  if (tid < 128 && !failed_a) {
    // B operands: row i, 32 columns per thread
    const int i = tid >> 1, j0 = (tid & 1) * 32;
#pragma unroll
    for (int j8 = 0; j8 < 4; ++j8) {
      uint32_t a[4], b[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = j0 + j8 * 8 + e * 2;
        const float t0 = sT[i * 65 + j] * sBeta[j], t1 = sT[i * 65 + j + 1] * sBeta[j + 1];
        a[e] = pack_bf16x2(t0, t1);
        b[e] = pack_bf16x2(t0 * __expf(sG[j]), t1 * __expf(sG[j + 1]));
      }
      const uint32_t off = sw128_off(i, j0 + j8 * 8);
      *reinterpret_cast<uint4*>(sT1 + off) = make_uint4(a[0], a[1], a[2], a[3]);
      *reinterpret_cast<uint4*>(sT2 + off) = make_uint4(b[0], b[1], b[2], b[3]);
    }
    fence_proxy_async_smem();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (control && !failed_a) {
    tc_fence_after_sync();
    constexpr uint32_t idesc = umma_idesc_bf16(128, 64, 1, 0);   // A = V^T / K^T, MN-major
    const uint32_t v0 = smem_u32(sV), k0 = smem_u32(sKQ), t1 = smem_u32(sT1), t2 = smem_u32(sT2);
#pragma unroll
    for (int kk = 0; kk < kC / 16; ++kk) {
      umma_bf16_ss(tmem_u, umma_desc_mn_sw128(v0 + kk * 2048, 8192, 1024),
                   umma_desc_k_sw128(t1 + kk * 32, 1024), idesc, kk != 0);
    }
#pragma unroll
    for (int kk = 0; kk < kC / 16; ++kk) {
      umma_bf16_ss(tmem_w, umma_desc_mn_sw128(k0 + kk * 2048, 16384, 1024),
                   umma_desc_k_sw128(t2 + kk * 32, 1024), idesc, kk != 0);
    }
    umma_commit(&bars->mma[1]);
  }
  if (tid < 128 && !failed_a) {
    ok = mbar_wait(&bars->mma[1], 0, p.status);
    if (ok) {
      tc_fence_after_sync();
      const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        bf16* dst = (which == 0 ? p.u : p.w) + ((size_t)n * kC * p.Hv + hv) * kD + tid;
        const uint32_t base = (which == 0 ? tmem_u : tmem_w) + lane_off;
#pragma unroll
        for (int cb = 0; cb < 2; ++cb) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(base + cb * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c)
            dst[(size_t)(cb * 32 + c) * p.Hv * kD] = __float2bfloat16(__uint_as_float(r[c]));
        }
      }
      tc_fence_before_sync();
    }
  }
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 256);
  }
}

static constexpr size_t kPrepSmem = 32768 + 16384 + 8192 + 8192 + 2 * 64 * 65 * 4 + 2 * 64 * 4 + sizeof(ScanBars) + 1024;

// ---------------------------------------------------------------------------------------
// Sequential scan over the chunks of one (sequence, value head).
// ---------------------------------------------------------------------------------------
struct ScanParams {
  const bf16* u;           // [NT*64, Hv, 128]
  const float* gc;         // [NT, Hv, 64]
  const int* chunk_tok0;   // [NT]
  const int* chunk_len;    // [NT]
  const int* seq_chunk0;   // [n_seq + 1]
  const int* slots;        // [n_seq] state slot (< 0: no state kept)
  const int* has_init;     // [n_seq] or null (= all 1)
  float* state;            // [slots, Hv, Dv, Dk] fp32
  bf16* out;               // [T, Hv, 128]
  int Hk, Hv;
  int* status;
};

static constexpr int kSlotBytes = 16384 * 3 + 8192;   // W, Q', K tiles + P tile

__global__ void __launch_bounds__(kScanThreads, 1)
    gdn_chunk_scan_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmQs,
                          const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmP,
                          ScanParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sH = smem;                       // bf16 h^T: 2 halves x 128 rows x 128 B
  uint8_t* sVs = sH + 32768;                // v_new e^{G_last-G}: 128 rows x 128 B (A, K-major)
  uint8_t* sVo = sVs + 16384;               // v_new
  uint8_t* sSlot = sVo + 16384;             // 2 x {W | Q' | K | P}
  float* sGc = reinterpret_cast<float*>(sSlot + 2 * kSlotBytes);   // [2][64]
  ScanBars* bars = reinterpret_cast<ScanBars*>(sGc + 128);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int s = blockIdx.x / p.Hv, hv = blockIdx.x % p.Hv;
  const int hk = hv / (p.Hv / p.Hk);
  const int n0 = p.seq_chunk0[s], n1 = p.seq_chunk0[s + 1];
  const int nchunks = n1 - n0;
  const bool control = (tid == 128);
  const int slot = p.slots[s];
  const bool init = slot >= 0 && (p.has_init ? p.has_init[s] != 0 : true);

  if (tid == 0) {
    mbar_init(&bars->load[0], 1);
    mbar_init(&bars->load[1], 1);
    mbar_init(&bars->mma[0], 1);
    mbar_init(&bars->mma[1], 1);
    bars->failed = 0;
    mbar_fence_init();
  }
  if (warp == 4) {
    tmem_alloc(&bars->tmem_base, 256);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = bars->tmem_base;
  const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
  const uint32_t tmem_h = tmem, tmem_x = tmem + 128, tmem_o = tmem + 192;

  auto issue_loads = [&](int ci) {
    const int n = n0 + ci;
    uint8_t* base = sSlot + (ci & 1) * kSlotBytes;
    uint64_t* bar = &bars->load[ci & 1];
    mbar_expect_tx(bar, kSlotBytes);
    const int tok0 = p.chunk_tok0[n];
    for (int h = 0; h < 2; ++h) {
      tma_load_2d(base + h * 8192, &tmW, bar, hv * kD + h * 64, n * kC);
      tma_load_2d(base + 16384 + h * 8192, &tmQs, bar, hv * kD + h * 64, n * kC);
      tma_load_2d(base + 32768 + h * 8192, &tmK, bar, hk * kD + h * 64, tok0);
    }
    tma_load_2d(base + 49152, &tmP, bar, 0, (n * p.Hv + hv) * kC);
  };

  int loads_issued = 0, loads_consumed = 0;   // control thread only
  if (control && nchunks > 0) { issue_loads(0); loads_issued = 1; }

  // initial state -> TMEM (row t of h^T = state[slot][hv][t][:])
  if (tid < 128) {
    const float* src = init ? p.state + (((size_t)slot * p.Hv + hv) * kD + tid) * kD : nullptr;
#pragma unroll
    for (int cb = 0; cb < 4; ++cb) {
      uint32_t r[32];
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
        float4 v = src ? *reinterpret_cast<const float4*>(src + cb * 32 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        r[c] = __float_as_uint(v.x); r[c + 1] = __float_as_uint(v.y);
        r[c + 2] = __float_as_uint(v.z); r[c + 3] = __float_as_uint(v.w);
      }
      tmem_st_32x32b_x32(tmem_h + lane_off + cb * 32, r);
    }
    tmem_st_wait();
  }
  tc_fence_before_sync();
  __syncthreads();

  for (int ci = 0; ci < nchunks; ++ci) {
    const int n = n0 + ci;
    const int tok0 = p.chunk_tok0[n], len = p.chunk_len[n];
    uint8_t* slotp = sSlot + (ci & 1) * kSlotBytes;
    float* gcs = sGc + (ci & 1) * 64;
    const uint32_t ph = (ci >> 1) & 1;    // parity of this slot's load barrier
    const uint32_t mph = ci & 1;          // both MMA barriers complete once per chunk

    // ---- phase A: bf16 copy of h for the two products, decay the fp32 state in place
    if (tid < 64) gcs[tid] = p.gc[((size_t)n * p.Hv + hv) * kC + tid];
    if (tid < 128) {
      tc_fence_after_sync();
      const float glast = p.gc[((size_t)n * p.Hv + hv) * kC + kC - 1];
      const float decay = __expf(glast);
#pragma unroll
      for (int cb = 0; cb < 4; ++cb) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_h + lane_off + cb * 32, r);
        tmem_ld_wait();
        uint8_t* hb = sH + (cb >> 1) * 16384;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            pk[e] = pack_bf16x2(__uint_as_float(r[c8 * 8 + e * 2]), __uint_as_float(r[c8 * 8 + e * 2 + 1]));
          *reinterpret_cast<uint4*>(hb + sw128_off(tid, (cb & 1) * 32 + c8 * 8)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
#pragma unroll
        for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * decay);
        tmem_st_32x32b_x32(tmem_h + lane_off + cb * 32, r);
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before_sync();
    }
    __syncthreads();
    if (bars->failed) break;

    // ---- phase B: x = w h, o = q' h
    if (control) {
      if (ci + 1 < nchunks) { issue_loads(ci + 1); loads_issued = ci + 2; }   // that slot's MMAs are done
      const bool got = mbar_wait(&bars->load[ci & 1], ph, p.status);
      if (got) loads_consumed = ci + 1;
      if (got) {
        tc_fence_after_sync();
        constexpr uint32_t idesc = umma_idesc_bf16(128, 64, 0, 0);
        const uint32_t h0 = smem_u32(sH), w0 = smem_u32(slotp), q0 = smem_u32(slotp + 16384);
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t ao = (kk / 4) * 16384 + (kk % 4) * 32, bo = (kk / 4) * 8192 + (kk % 4) * 32;
          umma_bf16_ss(tmem_x, umma_desc_k_sw128(h0 + ao, 1024), umma_desc_k_sw128(w0 + bo, 1024), idesc, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk) {
          const uint32_t ao = (kk / 4) * 16384 + (kk % 4) * 32, bo = (kk / 4) * 8192 + (kk % 4) * 32;
          umma_bf16_ss(tmem_o, umma_desc_k_sw128(h0 + ao, 1024), umma_desc_k_sw128(q0 + bo, 1024), idesc, kk != 0);
        }
        umma_commit(&bars->mma[0]);
      } else {
        bars->failed = 1;
      }
    }
    // ---- phase C: v_new = u - x, staged twice (decayed for the state, plain for the output)
    if (tid < 128) {
      // u[i][tid] for the whole chunk, fetched while the MMAs run
      float uv[64];
      const bf16* ub = p.u + ((size_t)n * kC * p.Hv + hv) * kD + tid;
#pragma unroll
      for (int i = 0; i < 64; ++i) uv[i] = __bfloat162float(ub[(size_t)i * p.Hv * kD]);
      bool ok = mbar_wait(&bars->mma[0], mph, p.status);
      if (!ok) bars->failed = 1;
      if (ok) {
        tc_fence_after_sync();
        const float glast = gcs[kC - 1];
#pragma unroll
        for (int cb = 0; cb < 2; ++cb) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_x + lane_off + cb * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) {
            uint32_t a[4], b[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int i = cb * 32 + c8 * 8 + e * 2;
              const float v0 = uv[i] - __uint_as_float(r[c8 * 8 + e * 2]);
              const float v1 = uv[i + 1] - __uint_as_float(r[c8 * 8 + e * 2 + 1]);
              a[e] = pack_bf16x2(v0 * __expf(glast - gcs[i]), v1 * __expf(glast - gcs[i + 1]));
              b[e] = pack_bf16x2(v0, v1);
            }
            const uint32_t off = sw128_off(tid, cb * 32 + c8 * 8);
            *reinterpret_cast<uint4*>(sVs + off) = make_uint4(a[0], a[1], a[2], a[3]);
            *reinterpret_cast<uint4*>(sVo + off) = make_uint4(b[0], b[1], b[2], b[3]);
          }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
      }
    }
    __syncthreads();
    if (bars->failed) break;

    // ---- phase D: h += (v_new decayed)^T k ; o += v_new^T p^T
    if (control) {
      tc_fence_after_sync();
      constexpr uint32_t idesc_h = umma_idesc_bf16(128, 128, 0, 1);   // B = k, MN-major
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, 64, 0, 0);
      const uint32_t vs0 = smem_u32(sVs), vo0 = smem_u32(sVo);
      const uint32_t k0 = smem_u32(slotp + 32768), p0 = smem_u32(slotp + 49152);
#pragma unroll
      for (int kk = 0; kk < kC / 16; ++kk)
        umma_bf16_ss(tmem_h, umma_desc_k_sw128(vs0 + kk * 32, 1024),
                     umma_desc_mn_sw128(k0 + kk * 2048, 8192, 1024), idesc_h, 1);
#pragma unroll
      for (int kk = 0; kk < kC / 16; ++kk)
        umma_bf16_ss(tmem_o, umma_desc_k_sw128(vo0 + kk * 32, 1024), umma_desc_k_sw128(p0 + kk * 32, 1024),
                     idesc_o, 1);
      umma_commit(&bars->mma[1]);
    }
    // ---- phase E: write o
    if (tid < 128) {
      bool ok = mbar_wait(&bars->mma[1], mph, p.status);
      if (!ok) bars->failed = 1;
      if (ok) {
        tc_fence_after_sync();
        bf16* ob = p.out + ((size_t)tok0 * p.Hv + hv) * kD + tid;
#pragma unroll
        for (int cb = 0; cb < 2; ++cb) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_o + lane_off + cb * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int i = cb * 32 + c;
            if (i < len) ob[(size_t)i * p.Hv * kD] = __float2bfloat16(__uint_as_float(r[c]));
          }
        }
        tc_fence_before_sync();
      }
    }
    __syncthreads();
    if (bars->failed) break;
  }

  // a failed run may leave bulk copies in flight: let them land (bounded) before the CTA ends
  if (control) {
    for (int ci = loads_consumed; ci < loads_issued; ++ci)
      mbar_wait(&bars->load[ci & 1], (ci >> 1) & 1, p.status);
  }
  // final state back to the cache
  if (tid < 128 && slot >= 0 && !bars->failed) {
    tc_fence_after_sync();
    float* dst = p.state + (((size_t)slot * p.Hv + hv) * kD + tid) * kD;
#pragma unroll
    for (int cb = 0; cb < 4; ++cb) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(tmem_h + lane_off + cb * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 32; c += 4)
        *reinterpret_cast<float4*>(dst + cb * 32 + c) =
            make_float4(__uint_as_float(r[c]), __uint_as_float(r[c + 1]), __uint_as_float(r[c + 2]),
                        __uint_as_float(r[c + 3]));
    }
    tc_fence_before_sync();
  }
  __syncthreads();
  if (warp == 4) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 256);
  }
}

static constexpr size_t kScanSmem = 32768 + 16384 + 16384 + 2 * kSlotBytes + 128 * 4 + sizeof(ScanBars) + 1024;

}  // namespace b200

using namespace b200;

// q, k: [T, Hk, 128] bf16 (normalised); v: bf16 rows of stride ldv with head 0 at column
// v_col0; g, beta: [T, Hv] fp32. Work buffers (caller-owned, sized for NT chunks):
// u, w, qs: [NT*64, Hv, 128] bf16; pbuf: [NT, Hv, 64, 64] bf16; gc: [NT, Hv, 64] fp32.
// Chunk tables are device arrays built by the caller from the batch's query_start_loc.
extern "C" int b200_gdn_chunk_scan(const void* q, const void* k, const void* v, long ldv, int v_col0,
                                   const float* g, const float* beta, int T, int Hk, int Hv,
                                   const int* chunk_tok0, const int* chunk_len, int NT,
                                   const int* seq_chunk0, const int* slots, const int* has_init,
                                   int n_seq, float* state, void* u, void* w, void* qs, void* pbuf,
                                   float* gc, void* out, cudaStream_t stream) {
  if (NT <= 0 || n_seq <= 0) return 0;
  if (Hk <= 0 || Hv % Hk || (ldv & 7) || (v_col0 & 7)) return -1;
  CUtensorMap tmQ, tmK, tmV, tmW, tmQs, tmP;
  const auto BF = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const auto SW = CU_TENSOR_MAP_SWIZZLE_128B;
  if (!encode_tmap_2d(&tmQ, q, BF, 2, T, (uint64_t)Hk * kD, (uint64_t)Hk * kD, kC, 64, SW) ||
      !encode_tmap_2d(&tmK, k, BF, 2, T, (uint64_t)Hk * kD, (uint64_t)Hk * kD, kC, 64, SW) ||
      !encode_tmap_2d(&tmV, v, BF, 2, T, (uint64_t)ldv, (uint64_t)ldv, kC, 64, SW) ||
      !encode_tmap_2d(&tmW, w, BF, 2, (uint64_t)NT * kC, (uint64_t)Hv * kD, (uint64_t)Hv * kD, kC, 64, SW) ||
      !encode_tmap_2d(&tmQs, qs, BF, 2, (uint64_t)NT * kC, (uint64_t)Hv * kD, (uint64_t)Hv * kD, kC, 64, SW) ||
      !encode_tmap_2d(&tmP, pbuf, BF, 2, (uint64_t)NT * Hv * kC, kC, kC, kC, 64, SW))
    return -3;
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(gdn_chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPrepSmem);
    cudaFuncSetAttribute(gdn_chunk_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kScanSmem);
  }
  PrepParams pp{};
  pp.g = g; pp.beta = beta; pp.q = (const bf16*)q;
  pp.chunk_tok0 = chunk_tok0; pp.chunk_len = chunk_len;
  pp.u = (bf16*)u; pp.w = (bf16*)w; pp.qs = (bf16*)qs; pp.p = (bf16*)pbuf; pp.gc = gc;
  pp.Hk = Hk; pp.Hv = Hv; pp.v_col0 = v_col0;
  pp.status = device_status_word();
  gdn_chunk_prep_kernel<<<dim3(NT, Hv), kScanThreads, kPrepSmem, stream>>>(tmQ, tmK, tmV, pp);
  if (cudaGetLastError() != cudaSuccess) return -2;
  ScanParams sp{};
  sp.u = (const bf16*)u; sp.gc = gc; sp.chunk_tok0 = chunk_tok0; sp.chunk_len = chunk_len;
  sp.seq_chunk0 = seq_chunk0; sp.slots = slots; sp.has_init = has_init; sp.state = state;
  sp.out = (bf16*)out; sp.Hk = Hk; sp.Hv = Hv; sp.status = pp.status;
  gdn_chunk_scan_kernel<<<n_seq * Hv, kScanThreads, kScanSmem, stream>>>(tmW, tmQs, tmK, tmP, sp);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
