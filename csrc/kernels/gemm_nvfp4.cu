// NVFP4 x NVFP4 GEMM (W4A4) on the block-scaled tensor-core path:
//   out[M, N] = (A_q[M, K] * sfa) (W_q[N, K] * sfw)^T * (g_w / g_a)
// A_q, W_q: e2m1 values packed two per byte, K-major; sfa, sfw: one ue4m3 scale per 16 elements in
// the 128 x 4 chunk layout ([rows / 128][K / 64][512 bytes], byte = (r % 32) * 16 + (r / 32) * 4 + k);
// g_w: the weight's fp32 global multiplier, g_a: the activation quantiser's fp32 global scale.
//
// Nothing is converted on the way: TMA brings the packed tiles (128-byte swizzle, 256 elements of K
// per row) and bulk copies bring the scale chunks into a 4-stage ring; one thread copies the scale
// chunks of a stage into tensor memory (tcgen05.cp 32x128b.warpx4: 32 rows x 16 bytes, replicated to
// the four lane quarters, which is what the chunk layout is made for) and issues four
// tcgen05.mma.kind::mxf4nvf4.block_scale.scale_vec::4X instructions (K = 64 each) per stage on a
// 128 x NT accumulator in tensor memory; four warps read it back, apply g_w / g_a (+ bias) and store
// bf16, or fp32 partials when K is split over blockIdx.z.
//
// Reference: src/vt/cuda/cuda_matmul_nvfp4.cu:2579-2652 (native block-scaled MMA) and the CUTLASS
// tactics of src/vt/cuda/nvfp4_cutlass_tactic_impl.cuh:33-80.
#include "api.h"
#include "sm100.cuh"

namespace b200 {

using bf16 = __nv_bfloat16;

static constexpr int kF4Stages = 4;
static constexpr int kF4ABytes = 128 * 128;          // 128 rows x 256 e2m1
static constexpr int kF4SfaBytes = 4 * 512;          // 128 rows x 16 scales (four K = 64 chunks)
static constexpr int kF4Threads = 6 * 32;            // TMA | MMA | 4 epilogue warps

template <int NT>
struct F4Layout {
  static constexpr int b_bytes = NT * 128;
  static constexpr int sfb_bytes = (NT / 128) * kF4SfaBytes;
  static constexpr int stage_bytes = kF4ABytes + b_bytes + kF4SfaBytes + sfb_bytes;
  // tensor memory: accumulator NT columns, then per stage 16 columns of A scales and NT / 8 of B scales
  static constexpr int sf_cols_per_stage = 16 + NT / 8;
  static constexpr int tmem_cols = 512;
};

struct F4Params {
  int M, N, K;
  bf16* out;
  int ldo;
  const uint8_t* sfa;
  const uint8_t* sfw;
  const float* g_w;
  const float* g_a;
  const bf16* bias;
  int splits, stages_per_split;     // stages of 256 k-elements
  float* workspace;                 // [splits, M, N] fp32 when splits > 1
  int* status;
};

struct alignas(8) F4Bars {
  uint64_t full[kF4Stages], empty[kF4Stages];
  uint64_t acc_full;
  uint32_t tmem_base;
};

// Shared-memory descriptor of one scale chunk (32 rows x 16 bytes, no swizzle: 8-row core matrices
// of 128 contiguous bytes, 128 bytes apart).
__device__ __forceinline__ uint64_t sf_chunk_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
  d |= (uint64_t)(128 >> 4) << 16;
  d |= (uint64_t)(128 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <int NT>
__global__ void __launch_bounds__(kF4Threads, 1)
    gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW, F4Params p) {
  using L = F4Layout<NT>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  F4Bars* bars = reinterpret_cast<F4Bars*>(smem + (size_t)kF4Stages * L::stage_bytes);
  auto sA = [&](int s) { return smem + (size_t)s * L::stage_bytes; };
  auto sB = [&](int s) { return sA(s) + kF4ABytes; };
  auto sSfa = [&](int s) { return sB(s) + L::b_bytes; };
  auto sSfb = [&](int s) { return sSfa(s) + kF4SfaBytes; };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * 128, n0 = blockIdx.x * NT, split = blockIdx.z;
  const int total_stages = p.K / 256;
  const int st0 = split * p.stages_per_split;
  const int nst = max(0, min(total_stages, st0 + p.stages_per_split) - st0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kF4Stages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, L::tmem_cols); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmW);
      const size_t chunks_per_rowblock = (size_t)(p.K / 64) * 512;
      for (int i = 0; i < nst; ++i) {
        const int s = i % kF4Stages, st = st0 + i;
        if (!mbar_wait_backoff(&bars->empty[s], ((i / kF4Stages) & 1) ^ 1, p.status)) break;
        mbar_expect_tx(&bars->full[s], L::stage_bytes);
        tma_load_2d(sA(s), &tmA, &bars->full[s], st * 128, m0);
        tma_load_2d(sB(s), &tmW, &bars->full[s], st * 128, n0);
        bulk_load(sSfa(s), p.sfa + (size_t)(m0 / 128) * chunks_per_rowblock + (size_t)st * kF4SfaBytes, kF4SfaBytes,
                  &bars->full[s]);
#pragma unroll
        for (int rb = 0; rb < NT / 128; ++rb)
          bulk_load(sSfb(s) + rb * kF4SfaBytes,
                    p.sfw + (size_t)(n0 / 128 + rb) * chunks_per_rowblock + (size_t)st * kF4SfaBytes, kF4SfaBytes,
                    &bars->full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_nvfp4(128, NT);
      bool ok = true;
      for (int i = 0; i < nst; ++i) {
        const int s = i % kF4Stages;
        if (!mbar_wait_backoff(&bars->full[s], (i / kF4Stages) & 1, p.status)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t t_sfa = tmem_base + NT + s * L::sf_cols_per_stage;
        const uint32_t t_sfb = t_sfa + 16;
        // scale chunks of this stage: A's four K = 64 chunks, then B's per 128-row block
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          tmem_cp_32x128b_warpx4(t_sfa + 4 * j, sf_chunk_desc(smem_u32(sSfa(s) + j * 512)));
#pragma unroll
          for (int rb = 0; rb < NT / 128; ++rb)
            tmem_cp_32x128b_warpx4(t_sfb + (NT / 32) * j + 4 * rb,
                                   sf_chunk_desc(smem_u32(sSfb(s) + rb * kF4SfaBytes + j * 512)));
        }
        const uint64_t adesc = umma_desc_k_sw128(smem_u32(sA(s)), 1024);
        const uint64_t bdesc = umma_desc_k_sw128(smem_u32(sB(s)), 1024);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          umma_nvfp4_ss(tmem_base, adesc + 2 * j, bdesc + 2 * j, idesc, t_sfa + 4 * j, t_sfb + (NT / 32) * j,
                        (i | j) != 0);
        umma_commit(&bars->empty[s]);
      }
      if (ok) umma_commit(&bars->acc_full);
    }
  } else {
    // ---- epilogue: TMEM lane = row of the tile, column = n
    const int q = warp & 3;                       // lane quarter this warp may read
    bool ok = true;
    if (nst > 0) ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_full, 0, p.status));
    if (ok) {
      tc_fence_after_sync();
      const int m = m0 + q * 32 + lane;
      const float scale = *p.g_w / *p.g_a;
      const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < NT / 16; ++c) {
        uint32_t rr[16];
        if (nst > 0) {
          tmem_ld_32x32b_x16(t_addr + c * 16, rr);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) rr[i] = 0;
        }
        const int n = n0 + c * 16;
        if (m < p.M && n < p.N) {
          float v[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(rr[i]) * scale;
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
  if (warp == 1) tmem_dealloc(tmem_base, L::tmem_cols);
}

__global__ void f4_splitk_reduce_kernel(const float* __restrict__ ws, int splits, int M, int N, bf16* out, int ldo,
                                        const bf16* __restrict__ bias) {
  const size_t total = (size_t)M * N;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int m = (int)(i / N), n = (int)(i % N);
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += ws[(size_t)s * total + i];
    if (bias) acc += __bfloat162float(bias[n]);
    out[(size_t)m * ldo + n] = __float2bfloat16(acc);
  }
}

// Row-major block scales [rows, K / 16] -> the 128 x 4 chunk layout, rows padded (with zero scales)
// to a multiple of `pad_rows`.
__global__ void sf_to_chunks_kernel(const uint8_t* __restrict__ sf, long rows, int kb16, uint8_t* __restrict__ out,
                                    long padded_rows) {
  const long total = padded_rows * kb16;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / kb16;
    const int g = (int)(i % kb16);
    const uint8_t v = r < rows ? sf[r * kb16 + g] : (uint8_t)0;
    const size_t o = ((size_t)(r / 128) * (kb16 / 4) + g / 4) * 512 + (size_t)(r % 32) * 16 + (size_t)((r % 128) / 32) * 4 +
                     (g % 4);
    out[o] = v;
  }
}

template <int NT>
static int launch_nvfp4(const CUtensorMap& tmA, const CUtensorMap& tmW, const F4Params& p, int tiles_m, int tiles_n,
                        cudaStream_t stream) {
  using L = F4Layout<NT>;
  constexpr size_t smem = (size_t)kF4Stages * L::stage_bytes + 1024 + sizeof(F4Bars);
  static_assert(smem <= 227 * 1024, "shared memory budget");
  static PerDeviceOnce attr_once;
  if (attr_once.first())
    cudaFuncSetAttribute(gemm_nvfp4_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  gemm_nvfp4_kernel<NT><<<dim3(tiles_n, tiles_m, p.splits), kF4Threads, smem, stream>>>(tmA, tmW, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace b200

using namespace b200;

extern "C" {

// aq / wq: packed e2m1 [M, K / 2] / [N, K / 2]; sfa / sfw: block scales in the chunk layout with rows
// padded to 128 (sfa) and to `n_tile` (sfw); g_w, g_a: device fp32 scalars. K a multiple of 256.
// n_tile: 128 or 256 weight rows per CTA (0 = choose). workspace (fp32 [splits, M, N]) only when K
// is split; without it (or too small) the GEMM runs unsplit.
int b200_gemm_nvfp4(const void* aq, const void* sfa, const float* g_a, const void* wq, const void* sfw,
                    const float* g_w, void* out, int ldo, const void* bias, int M, int N, int K, int n_tile,
                    void* workspace, size_t ws_bytes, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 255) || (N & 7) || (ldo & 7)) return -1;
  if ((reinterpret_cast<uintptr_t>(aq) | reinterpret_cast<uintptr_t>(wq) | reinterpret_cast<uintptr_t>(sfa) |
       reinterpret_cast<uintptr_t>(sfw)) & 15)
    return -1;
  if (n_tile == 0) n_tile = 256;
  if (n_tile != 128 && n_tile != 256) return -1;
  F4Params p{};
  p.M = M; p.N = N; p.K = K; p.out = (bf16*)out; p.ldo = ldo;
  p.sfa = (const uint8_t*)sfa; p.sfw = (const uint8_t*)sfw; p.g_w = g_w; p.g_a = g_a; p.bias = (const bf16*)bias;
  p.status = device_status_word();
  const int sms = b200_num_sms();
  const int tiles_m = (M + 127) / 128, tiles_n = (N + n_tile - 1) / n_tile;
  const int total_stages = K / 256;
  int splits = 1;
  if (tiles_m * tiles_n < sms && workspace) {
    splits = sms / (tiles_m * tiles_n);
    if (splits > total_stages / 4) splits = total_stages / 4 > 0 ? total_stages / 4 : 1;
    if (splits > 16) splits = 16;
    while (splits > 1 && (size_t)splits * M * N * 4 > ws_bytes) --splits;
  }
  int per = (total_stages + splits - 1) / splits;
  splits = (total_stages + per - 1) / per;
  p.splits = splits; p.stages_per_split = per; p.workspace = (float*)workspace;
  CUtensorMap tmA, tmW;
  if (!encode_tmap_2d(&tmA, aq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K / 2, K / 2, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  if (!encode_tmap_2d(&tmW, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 2, K / 2, n_tile, 128,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  const int rc = n_tile == 256 ? launch_nvfp4<256>(tmA, tmW, p, tiles_m, tiles_n, stream)
                               : launch_nvfp4<128>(tmA, tmW, p, tiles_m, tiles_n, stream);
  if (rc) return rc;
  if (splits > 1) {
    const size_t total = (size_t)M * N;
    int blocks = (int)((total + 255) / 256);
    if (blocks > sms * 8) blocks = sms * 8;
    f4_splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(p.workspace, splits, M, N, p.out, ldo, p.bias);
    if (cudaGetLastError() != cudaSuccess) return -2;
  }
  return 0;
}

// Row-major ue4m3 block scales [rows, K / 16] -> chunk layout, rows padded to a multiple of pad_rows
// (128 or 256). out must hold padded_rows * K / 16 bytes. K a multiple of 64.
int b200_nvfp4_sf_to_chunks(const void* sf, long rows, int K, int pad_rows, void* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if ((K & 63) || (pad_rows != 128 && pad_rows != 256)) return -1;
  const long padded = (rows + pad_rows - 1) / pad_rows * pad_rows;
  const long total = padded * (K / 16);
  int blocks = (int)((total + 255) / 256);
  if (blocks > b200_num_sms() * 16) blocks = b200_num_sms() * 16;
  sf_to_chunks_kernel<<<blocks, 256, 0, stream>>>((const uint8_t*)sf, rows, K / 16, (uint8_t*)out, padded);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
