// NVFP4-weight x 16-bit-activation GEMM for decode-sized batches (M <= 128):
// out[M, N] = A[M, K] * dequant(W)[N, K]^T, W = e2m1 nibbles * e4m3 scale per 16 * fp32 global.
//
// The packed weights are the only large stream (K / 2 bytes per row), so the kernel is built
// around keeping them moving: TMA brings 256-row x 256-element packed blocks (32 KB) into a
// ring; sixteen converter warps expand them to f16 with the hardware conversions
// (cvt.rn.f16x2.e2m1x2 for two nibbles, cvt.rn.f16x2.e4m3x2 for two scales, one HMUL2 per two
// elements) straight into 128-byte-swizzled K-major tiles; one thread issues f16 tcgen05 MMAs
// with the (pre-cast f16, zero-padded) batch as the 128-row operand and 256 weight rows as the N
// operand - an MMA instruction costs about the same whatever its N, so the wide side is where the
// weights go. value x block scale is exact in f16 (at most 5 significant bits, magnitude <= 2688);
// the fp32 global scale is applied to the accumulators in the epilogue. Each converter thread
// reads its four block scales of a stage as one word, one stage ahead. Split-K over blockIdx.y
// with fp32 partials.
//
// Reference: src/vt/cuda/cuda_matmul_nvfp4_w4a16.cu (portable wmma W4A16), Marlin dense NVFP4.
#include <cuda_fp16.h>

#include "api.h"
#include "sm100.cuh"

namespace b200 {

using bf16 = __nv_bfloat16;

static constexpr int kWThreads = 19 * 32;   // raw TMA | MMA | act TMA | 16 converter / epilogue warps
static constexpr int kWN = 256;              // weight rows per CTA (the MMA's N)
static constexpr int kRawBytes = kWN * 128;  // 256 rows x 256 nibbles
static constexpr int kSfBytes = kWN * 16;    // 256 rows x 16 block scales (one raw stage)
static constexpr int kExpBytes = kWN * 128;  // 256 rows x 64 f16: one SW128 K-major tile
static constexpr int kActBytes = 128 * 128;  // 128 (padded batch) rows x 64 f16
static constexpr int kMaxRS = 2, kMaxES = 3, kMaxAS = 3;

struct W4SParams {
  int M, N, K;
  bf16* out;
  int ldo;
  const uint8_t* sf;      // [N, K/16] e4m3
  const float* gscale;
  const bf16* bias;
  int splits, ne_per_split;   // stages of 64 k-elements per split (a multiple of 4)
  int sf_tma;             // block scales arrive by TMA with each raw stage (needs K % 256 == 0)
  float* workspace;       // [splits, M, N] fp32 (splits > 1)
  int* status;
};

struct alignas(8) W4SBars {
  uint64_t raw_full[kMaxRS], raw_empty[kMaxRS];
  uint64_t exp_full[kMaxES], exp_empty[kMaxES];
  uint64_t act_full[kMaxAS], act_empty[kMaxAS];
  uint64_t acc_full;
  uint32_t tmem_base;
};

__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// kind::f16 with f16 A and B, f32 accumulation, both K-major.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// Eight e2m1 nibbles (low nibble first) -> four f16x2.
__device__ __forceinline__ void cvt_e2m1x8(uint32_t w, uint32_t (&h)[4]) {
  asm volatile(
      "{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}\n"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}
// Two e4m3 bytes -> f16x2.
__device__ __forceinline__ uint32_t cvt_e4m3x2(uint16_t v) {
  uint32_t r;
  asm volatile("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  return r;
}
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
  __half2 x = *reinterpret_cast<__half2*>(&a), y = *reinterpret_cast<__half2*>(&b);
  __half2 z = __hmul2(x, y);
  return *reinterpret_cast<uint32_t*>(&z);
}

__global__ void __launch_bounds__(kWThreads, 1)
    gemm_w4a16_stream_kernel(const __grid_constant__ CUtensorMap tmW,
                             const __grid_constant__ CUtensorMap tmA,
                             const __grid_constant__ CUtensorMap tmS, W4SParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int RS = kMaxRS, ES = kMaxES, AS = kMaxAS;
  uint8_t* sRaw = smem;
  uint8_t* sExp = sRaw + (size_t)RS * kRawBytes;
  uint8_t* sAct = sExp + (size_t)ES * kExpBytes;
  uint8_t* sSf = sAct + (size_t)AS * kActBytes;      // RS x 4 KB of block scales
  W4SBars* bars = reinterpret_cast<W4SBars*>(sSf + (size_t)RS * kSfBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tn = blockIdx.x, split = blockIdx.y;
  const int n0 = tn * kWN;
  const int ne_total = (p.K + 63) / 64;
  const int e0 = split * p.ne_per_split;
  const int ne = max(0, min(ne_total, e0 + p.ne_per_split) - e0);
  const int k0 = e0 * 64;                           // first element of this split (multiple of 256)
  constexpr uint32_t kTmemCols = kWN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < RS; ++s) {
      mbar_init(&bars->raw_full[s], 1);
      mbar_init(&bars->raw_empty[s], 64);           // 16 warps x 4 sub-stages
    }
    for (int s = 0; s < ES; ++s) {
      mbar_init(&bars->exp_full[s], 16);
      mbar_init(&bars->exp_empty[s], 1);
    }
    for (int s = 0; s < AS; ++s) {
      mbar_init(&bars->act_full[s], 1);
      mbar_init(&bars->act_empty[s], 1);
    }
    mbar_init(&bars->acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, kTmemCols); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ---------------- packed-weight (and scale) producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmW);
      const int nr = (ne + 3) / 4;
      for (int i = 0; i < nr; ++i) {
        const int rs = i % RS;
        if (!mbar_wait_backoff(&bars->raw_empty[rs], ((i / RS) & 1) ^ 1, p.status)) break;
        mbar_expect_tx(&bars->raw_full[rs], kRawBytes + (p.sf_tma ? kSfBytes : 0));
        tma_load_2d(sRaw + (size_t)rs * kRawBytes, &tmW, &bars->raw_full[rs], k0 / 2 + i * 128, n0);
        if (p.sf_tma) tma_load_2d(sSf + (size_t)rs * kSfBytes, &tmS, &bars->raw_full[rs], k0 / 16 + i * 16, n0);
      }
    }
  } else if (warp == 2) {
    // ---------------- activation producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      for (int e = 0; e < ne; ++e) {
        const int as = e % AS;
        if (!mbar_wait_backoff(&bars->act_empty[as], ((e / AS) & 1) ^ 1, p.status)) break;
        mbar_expect_tx(&bars->act_full[as], kActBytes);
        tma_load_2d(sAct + (size_t)as * kActBytes, &tmA, &bars->act_full[as], k0 + e * 64, 0);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: D[128 batch rows, 256 weight rows] ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_f16(128, kWN);
      bool ok = true;
      for (int e = 0; e < ne; ++e) {
        const int es = e % ES, as = e % AS;
        if (!mbar_wait_backoff(&bars->exp_full[es], (e / ES) & 1, p.status) ||
            !mbar_wait_backoff(&bars->act_full[as], (e / AS) & 1, p.status)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint64_t adesc = umma_desc_k_sw128(smem_u32(sAct + (size_t)as * kActBytes), 1024);
        const uint64_t bdesc = umma_desc_k_sw128(smem_u32(sExp + (size_t)es * kExpBytes), 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f16_ss(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (e | k) != 0);
        umma_commit(&bars->exp_empty[es]);
        umma_commit(&bars->act_empty[as]);
      }
      if (ok) umma_commit(&bars->acc_full);
    }
  } else {
    // ---------------- converters (then epilogue) ----------------
    const int cw = warp - 3;                        // 0..15
    const int ct = cw * 32 + lane;                  // 0..511
    const int r = ct & 255;                         // weight row of the tile
    const int h = ct >> 8;                          // which 32 of the stage's 64 elements
    bool ok = true;
    const bool row_in = n0 + r < p.N;
    const uint8_t* sf_row = p.sf + (size_t)(n0 + (row_in ? r : 0)) * (p.K / 16);
    auto scale_pair = [&](int e) -> uint32_t {        // no-TMA fallback: two e4m3 bytes from global
      const int b = k0 / 16 + e * 4 + h * 2;
      return (row_in && e < ne && b < p.K / 16)      // K % 64 == 0: the pair is in range together
                 ? (uint32_t)*reinterpret_cast<const uint16_t*>(sf_row + b) : 0u;
    };
    uint32_t sp_next = p.sf_tma ? 0u : scale_pair(0);
    for (int e = 0; e < ne && ok; ++e) {
      uint32_t sp = sp_next;
      if (!p.sf_tma) sp_next = scale_pair(e + 1);
      const int es = e % ES, ri = e >> 2, rs = ri % RS, sub = e & 3;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->exp_empty[es], ((e / ES) & 1) ^ 1, p.status) &&
                                       mbar_wait(&bars->raw_full[rs], (ri / RS) & 1, p.status));
      if (!ok) break;
      if (p.sf_tma)
        sp = *reinterpret_cast<const uint16_t*>(sSf + (size_t)rs * kSfBytes + r * 16 + sub * 4 + h * 2);
      const uint8_t* raw = sRaw + (size_t)rs * kRawBytes + (size_t)r * 128;
      const int c0 = sub * 2 + h;                   // 16-byte chunk of the raw row (swizzled)
      const uint4 ra = *reinterpret_cast<const uint4*>(raw + ((c0 ^ (r & 7)) << 4));
      const uint32_t s2 = cvt_e4m3x2((uint16_t)sp);
      const uint32_t sc[2] = {__byte_perm(s2, 0, 0x1010), __byte_perm(s2, 0, 0x3232)};
      const uint32_t words[4] = {ra.x, ra.y, ra.z, ra.w};
      uint8_t* dst = sExp + (size_t)es * kExpBytes + (size_t)r * 128;
#pragma unroll
      for (int c = 0; c < 4; ++c) {                 // 8 elements -> one 16-byte chunk of the f16 tile
        uint32_t hh[4];
        cvt_e2m1x8(words[c], hh);
        const uint32_t s = sc[c >> 1];
        *reinterpret_cast<uint4*>(dst + (((h * 4 + c) ^ (r & 7)) << 4)) =
            make_uint4(hmul2_bits(hh[0], s), hmul2_bits(hh[1], s), hmul2_bits(hh[2], s), hmul2_bits(hh[3], s));
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars->exp_full[es]);
        mbar_arrive(&bars->raw_empty[rs]);
      }
    }
    // ---- epilogue: TMEM lane = batch row m, column = weight row n; four warps share a lane
    // quarter and take 64 columns each
    if (ok && ne > 0) ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_full, 0, p.status));
    if (ok) {
      tc_fence_after_sync();
      const int quarter = warp & 3, part = cw >> 2;
      const int m = quarter * 32 + lane;
      const float g = *p.gscale;
      const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        const int col = part * 64 + c * 16;
        uint32_t rr[16];
        if (ne > 0) {
          tmem_ld_32x32b_x16(t_addr + col, rr);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) rr[i] = 0;
        }
        const int n = n0 + col;
        if (m < p.M && n < p.N) {
          float v[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(rr[i]) * g;
          if (p.splits > 1) {
            float* o = p.workspace + ((size_t)split * p.M + m) * p.N + n;
#pragma unroll
            for (int i = 0; i < 16; i += 4)
              if (n + i < p.N) *reinterpret_cast<float4*>(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
          } else {
            bf16* o = p.out + (size_t)m * p.ldo + n;
#pragma unroll
            for (int i = 0; i < 16; i += 8) {
              if (n + i < p.N) {
                if (p.bias) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) v[i + j] += __bfloat162float(p.bias[n + i + j]);
                }
                uint4 w;
                w.x = pack_bf16x2(v[i + 0], v[i + 1]);
                w.y = pack_bf16x2(v[i + 2], v[i + 3]);
                w.z = pack_bf16x2(v[i + 4], v[i + 5]);
                w.w = pack_bf16x2(v[i + 6], v[i + 7]);
                *reinterpret_cast<uint4*>(o + i) = w;
              }
            }
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

__global__ void w4s_splitk_reduce_kernel(const float* __restrict__ ws, int splits, int M, int N, bf16* out,
                                         int ldo, const bf16* __restrict__ bias) {
  const size_t total = (size_t)M * N;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int m = (int)(i / N), n = (int)(i % N);
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += ws[(size_t)s * total + i];
    if (bias) acc += __bfloat162float(bias[n]);
    out[(size_t)m * ldo + n] = __float2bfloat16(acc);
  }
}

// bf16 -> f16 with saturation (the MMA runs in f16; activations beyond the f16 range clamp).
__global__ void __launch_bounds__(256)
    cast_bf16_f16_kernel(const bf16* __restrict__ a, int lda, __half* __restrict__ out, int M, int K) {
  const size_t total = (size_t)M * (K / 8);
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int m = (int)(i / (K / 8)), c = (int)(i % (K / 8));
    const uint4 v = *reinterpret_cast<const uint4*>(a + (size_t)m * lda + c * 8);
    const uint32_t in[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = unpack_bf16x2(in[j]);
      f.x = fminf(fmaxf(f.x, -65504.f), 65504.f);
      f.y = fminf(fmaxf(f.y, -65504.f), 65504.f);
      __half2 h = __floats2half2_rn(f.x, f.y);
      o[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(out + (size_t)m * K + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

// Small-M fused path (M <= 128, K a multiple of 64). workspace: f16 copy of A (M * K * 2 bytes,
// rounded up to 256) followed by fp32 [splits, M, N] split-K partials; returns -4 if it is too
// small for even one split.
int b200_gemm_w4a16(const void* A, int lda, const void* wq, const void* sf, const float* gscale, void* out,
                    int ldo, const void* bias, int M, int N, int K, void* workspace, size_t ws_bytes,
                    cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 128 || (K & 63) || (lda & 7) || (ldo & 7)) return -1;
  if ((reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(workspace)) & 15) return -1;
  const size_t a16_bytes = (((size_t)M * K * 2) + 255) & ~(size_t)255;
  if (!workspace || ws_bytes < a16_bytes) return -4;
  W4SParams p{};
  p.M = M; p.N = N; p.K = K; p.out = (bf16*)out; p.ldo = ldo;
  p.sf = (const uint8_t*)sf; p.gscale = gscale; p.bias = (const bf16*)bias;
  p.status = device_status_word();
  const int sms = b200_num_sms();
  const int tiles_n = (N + kWN - 1) / kWN;
  const int ne_total = (K + 63) / 64;
  // split-K in whole 256-element raw blocks: fill the SMs, at least 8 stages per split
  int splits = 1;
  if (tiles_n < sms) {
    splits = sms / tiles_n;
    if (splits > ne_total / 8) splits = ne_total / 8 > 0 ? ne_total / 8 : 1;
    if (splits > 16) splits = 16;
  }
  const size_t part_room = ws_bytes - a16_bytes;
  while (splits > 1 && (size_t)splits * M * N * 4 > part_room) --splits;
  int ne_per = (ne_total + splits - 1) / splits;
  ne_per = (ne_per + 3) & ~3;
  splits = (ne_total + ne_per - 1) / ne_per;
  p.splits = splits; p.ne_per_split = ne_per;
  p.workspace = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + a16_bytes);

  __half* a16 = reinterpret_cast<__half*>(workspace);
  {
    const size_t total = (size_t)M * (K / 8);
    int blocks = (int)((total + 255) / 256);
    if (blocks > sms * 4) blocks = sms * 4;
    cast_bf16_f16_kernel<<<blocks, 256, 0, stream>>>((const bf16*)A, lda, a16, M, K);
    if (cudaGetLastError() != cudaSuccess) return -2;
  }
  CUtensorMap tmW, tmA, tmS;
  p.sf_tma = ((K & 255) == 0 && (reinterpret_cast<uintptr_t>(sf) & 15) == 0) ? 1 : 0;
  if (!encode_tmap_2d(&tmW, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 2, K / 2, kWN, 128,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  if (!encode_tmap_2d(&tmA, a16, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, M, K, K, 128, 64,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  tmS = tmW;
  if (p.sf_tma && !encode_tmap_2d(&tmS, sf, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 16, K / 16, kWN, 16,
                                  CU_TENSOR_MAP_SWIZZLE_NONE))
    return -3;
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(gemm_w4a16_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
  }
  const size_t smem = (size_t)kMaxRS * kRawBytes + (size_t)kMaxES * kExpBytes + (size_t)kMaxAS * kActBytes +
                      (size_t)kMaxRS * kSfBytes + 1024 + sizeof(W4SBars);
  static_assert((size_t)kMaxRS * kRawBytes + (size_t)kMaxES * kExpBytes + (size_t)kMaxAS * kActBytes +
                        (size_t)kMaxRS * kSfBytes + 1024 + sizeof(W4SBars) <= 224 * 1024, "shared memory budget");
  gemm_w4a16_stream_kernel<<<dim3(tiles_n, splits), kWThreads, smem, stream>>>(tmW, tmA, tmS, p);
  if (cudaGetLastError() != cudaSuccess) return -2;
  if (splits > 1) {
    const size_t total = (size_t)M * N;
    int blocks = (int)((total + 255) / 256);
    if (blocks > sms * 8) blocks = sms * 8;
    w4s_splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(p.workspace, splits, M, N, p.out, ldo, p.bias);
    if (cudaGetLastError() != cudaSuccess) return -2;
  }
  return 0;
}

}  // extern "C"
