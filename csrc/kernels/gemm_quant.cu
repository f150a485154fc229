// Quantised GEMMs and the kernels that produce their operands.
//
//   fp8 (e4m3) x fp8 -> bf16, per-tensor (optionally per-output-channel) scales: persistent
//   128 x 128 tcgen05 kind::f8f6f4 tiles, TMA ring of 128-byte K blocks (128 elements),
//   accumulators double-buffered in TMEM.     reference: MatmulFp8CublasLt / MatmulFp8Cutlass
//
//   NVFP4 weights (E2M1 pairs packed in bytes, one UE4M3 scale per 16 values, fp32 per-tensor
//   scale) x bf16 activations:
//     small M (<= 256): swap-AB kernel whose four otherwise idle epilogue warps expand each
//       packed 128 x 64 weight block (4 KB + 512 B of scales instead of 16 KB) into the
//       swizzled bf16 tile the MMA reads, so HBM only ever sees 4.5 bits per weight;
//     large M: one pass that expands the matrix to a bf16 scratch, then the bf16 GEMM.
//                                             reference: MatmulNvfp4* W4A16 path, Marlin dense
//
//   producers: bf16 -> fp8 with a static scale (plain, RMSNorm-fused), bf16 -> NVFP4 with
//   per-16 block scales (plain, SiLU-mul-fused), row-major or 128x4-swizzled scale output.
//                                             reference: QuantFp8StaticKernel,
//                                             RmsNormQuantFp8RowKernel, ScaledFp4Quant*,
//                                             SiluAndMulFp4Quant*, SwizzleBlockscaleKernel
#include <cuda_fp8.h>

#include <mutex>
#include <unordered_map>

#include "api.h"
#include "quant_codec.cuh"
#include "sm100.cuh"

namespace b200 {

typedef __nv_bfloat16 bf16;

static constexpr int kQM = 128, kQN = 128, kQKB = 128;   // tile, K bytes per block
static constexpr int kQThreads = 192;
static constexpr int kQMaxStages = 8;

struct QBars {
  uint64_t full[kQMaxStages], empty[kQMaxStages];
  uint64_t raw_full[kQMaxStages];     // W4A16: packed weights landed
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int failed;
};

struct Fp8Params {
  int M, N, K;
  bf16* out;
  int ldo;
  const float* a_scale;      // per-tensor, or [M] with a_scale_per_token
  int a_scale_per_token;
  const float* w_scale;      // per-tensor or per-channel [N]
  int w_scale_per_channel;
  const bf16* bias;
  int tiles_m, tiles_n, stages;
  int splits, kb_per_split;  // split-K: work item w = tile * splits + split; partial sums to `partials`
  float* partials;           // [splits][M][N] fp32 (raw accumulators, scales applied by the reduce)
  int* status;
};

__global__ void __launch_bounds__(kQThreads, 1)
    gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    Fp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kABytes = kQM * kQKB, kBBytes = kQN * kQKB, kStage = kABytes + kBBytes;
  const int stages = p.stages;
  QBars* bars = reinterpret_cast<QBars*>(smem + (size_t)stages * kStage);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n * p.splits;     // work items: (tile, K split)
  const int kblocks_total = (p.K + kQKB - 1) / kQKB;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&bars->acc_full[b], 1); mbar_init(&bars->acc_empty[b], 4); }
    bars->failed = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&bars->tmem_base, 2 * kQN); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_tiles && ok; w += gridDim.x) {
        const int t = w / p.splits, sp = w % p.splits;
        const int tm = t % p.tiles_m, tn = t / p.tiles_m;
        const int kb0 = sp * p.kb_per_split, kb1 = min(kblocks_total, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % stages;
          if (!mbar_wait(&bars->empty[s], ((it / stages) & 1) ^ 1, p.status)) { ok = false; break; }
          uint8_t* a_dst = smem + (size_t)s * kStage;
          mbar_expect_tx(&bars->full[s], kStage);
          tma_load_2d(a_dst, &tmA, &bars->full[s], kb * kQKB, tm * kQM);
          tma_load_2d(a_dst + kABytes, &tmB, &bars->full[s], kb * kQKB, tn * kQN);
        }
      }
      if (!ok) bars->failed = 1;
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_e4m3(kQM, kQN);
      uint32_t it = 0, tc = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < num_tiles && ok; w += gridDim.x, ++tc) {
        const int buf = tc & 1;
        if (!mbar_wait(&bars->acc_empty[buf], ((tc >> 1) & 1) ^ 1, p.status)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * kQN;
        const int sp = w % p.splits;
        const int kb0 = sp * p.kb_per_split, kb1 = min(kblocks_total, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % stages;
          if (!mbar_wait(&bars->full[s], (it / stages) & 1, p.status)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * kStage);
          const uint64_t adesc = umma_desc_k_sw128(a_addr, 1024);
          const uint64_t bdesc = umma_desc_k_sw128(a_addr + kABytes, 1024);
#pragma unroll
          for (int k = 0; k < kQKB / 32; ++k)   // 32 fp8 values = 32 bytes per instruction
            umma_f8f6f4_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, kb != kb0 || k != 0);
          umma_commit(&bars->empty[s]);
        }
        if (ok) umma_commit(&bars->acc_full[buf]);
      }
      if (!ok) bars->failed = 1;
    }
  } else {
    const int quarter = warp & 3;
    uint32_t tc = 0;
    bool ok = true;
    const float sw0 = p.w_scale_per_channel ? 0.f : __ldg(p.w_scale);
    for (int w = blockIdx.x; w < num_tiles && ok; w += gridDim.x, ++tc) {
      const int t = w / p.splits, sp = w % p.splits;
      const int tm = t % p.tiles_m, tn = t / p.tiles_m;
      const int buf = tc & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_full[buf], (tc >> 1) & 1, p.status));
      if (!ok) break;
      tc_fence_after_sync();
      const int row = tm * kQM + quarter * 32 + lane;
      // one scale for the tensor, or one per token (row) when the activations were quantised row-wise
      const float sa = p.a_scale_per_token ? (row < p.M ? p.a_scale[row] : 0.f) : *p.a_scale;
      const uint32_t t_addr = tmem_base + buf * kQN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < kQN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_addr + c * 32, r);
        tmem_ld_wait();
        const int col0 = tn * kQN + c * 32;
        if (p.splits > 1) {
          // raw partial sums; the reduce kernel adds the splits and applies scales and bias
          if (row < p.M && col0 < p.N) {
            float* o = p.partials + ((size_t)sp * p.M + row) * p.N + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              if (col0 + i < p.N)
                *reinterpret_cast<float4*>(o + i) = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]),
                                                                __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
          }
        } else if (row < p.M && col0 < p.N) {
          bf16* o = p.out + (size_t)row * p.ldo + col0;
          // the chunk's channel scales as vectors, fetched before the first store
          float4 swv[8];
#pragma unroll
          for (int i = 0; i < 8; ++i)
            swv[i] = !p.w_scale_per_channel ? make_float4(sw0, sw0, sw0, sw0)
                     : col0 + i * 4 < p.N   ? __ldg(reinterpret_cast<const float4*>(p.w_scale + col0) + i)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
          const float* swf = reinterpret_cast<const float*>(swv);
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            if (col0 + i < p.N) {
              float v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                v[e] = __uint_as_float(r[i + e]) * sa * swf[i + e];
                if (p.bias) v[e] += __bfloat162float(p.bias[col0 + i + e]);
              }
              uint4 w;
              w.x = pack_bf16x2(v[0], v[1]); w.y = pack_bf16x2(v[2], v[3]);
              w.z = pack_bf16x2(v[4], v[5]); w.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(o + i) = w;
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->acc_empty[buf]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * kQN);
}

// ---------------------------------------------------------------------------------------
// NVFP4
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float e2m1_value(uint32_t code) {
  // sign | 2-bit exponent | 1-bit mantissa: 0, .5, 1, 1.5, 2, 3, 4, 6
  const uint32_t mag = code & 7u;
  const float v = mag < 2 ? 0.5f * (float)mag : (float)(2 + (mag & 1)) * (float)(1 << ((mag >> 1) - 1)) * 0.5f;
  return (code & 8u) ? -v : v;
}
// Whole-matrix expansion: packed [N, K/2] + scales [N, K/16] -> bf16 [N, K].
__global__ void nvfp4_dequant_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ sf,
                                     const float* __restrict__ gscale, bf16* __restrict__ out, long N,
                                     int K) {
  const long groups = N * (long)(K / 16);
  const float g = *gscale;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < groups; i += (long)gridDim.x * blockDim.x) {
    const float s = e4m3_to_float(sf[i]) * g;
    const uint2 raw = reinterpret_cast<const uint2*>(packed)[i];   // 8 bytes = 16 values
    uint32_t w[8];
    const uint32_t words[2] = {raw.x, raw.y};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t byte = (words[j >> 2] >> ((j & 3) * 8)) & 0xffu;
      w[j] = pack_bf16x2(e2m1_value(byte & 15u) * s, e2m1_value(byte >> 4) * s);
    }
    uint4* o = reinterpret_cast<uint4*>(out + i * 16);
    o[0] = make_uint4(w[0], w[1], w[2], w[3]);
    o[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// ---------------------------------------------------------------------------------------
// Producers
// ---------------------------------------------------------------------------------------
// out = fp8(x / scale) (optionally after RMSNorm with weight w; gemma adds 1 to w).
__global__ void __launch_bounds__(256)
    quant_fp8_kernel(const bf16* __restrict__ x, long ldx, const bf16* __restrict__ w, float eps, int gemma,
                     const float* __restrict__ scale, uint8_t* __restrict__ out, long ldo, int H) {
  __shared__ float red[32];
  const long t = blockIdx.x;
  const bf16* xr = x + t * ldx;
  float inv = 1.f;
  if (w) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      const float v = __bfloat162float(xr[i]);
      ss += v * v;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) tot += red[i];
    inv = rsqrtf(tot / (float)H + eps);
  }
  const float is = 1.f / *scale;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = __bfloat162float(xr[i]);
    if (w) v = __bfloat162float(__float2bfloat16(v * inv * (__bfloat162float(w[i]) + (gemma ? 1.f : 0.f))));
    out[t * ldo + i] = float_to_e4m3(v * is);
  }
}

// Dynamic per-tensor fp8: pass 1 takes the maximum magnitude of the tensor (bit pattern of a
// non-negative float orders like the unsigned integer, so one atomicMax per block), pass 2 divides
// by amax / 448 and leaves that scale for the GEMM.
__global__ void __launch_bounds__(256)
    absmax_bf16_kernel(const bf16* __restrict__ x, long ldx, long T, int H, unsigned* __restrict__ amax_bits) {
  __shared__ float red[8];
  const int nv = H >> 3;
  const long total = T * (long)nv;
  float m = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / nv;
    const int c = (int)(i % nv);
    const uint4 v = *reinterpret_cast<const uint4*>(x + t * ldx + (long)c * 8);
    const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(wds[j]);
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < (int)(blockDim.x >> 5); ++i) m = fmaxf(m, red[i]);
    if (m > 0.f && !(m != m)) atomicMax(amax_bits, __float_as_uint(m));
  }
}

__global__ void __launch_bounds__(256)
    quant_fp8_dynamic_kernel(const bf16* __restrict__ x, long ldx, const unsigned* __restrict__ amax_bits,
                             float* __restrict__ scale_out, uint8_t* __restrict__ out, long ldo, long T, int H) {
  const float s = fmaxf(__uint_as_float(*amax_bits), 1e-12f) / 448.f;
  const float is = 1.f / s;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = s;
  const int nv = H >> 3;
  const long total = T * (long)nv;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / nv;
    const int c = (int)(i % nv);
    const uint4 v = *reinterpret_cast<const uint4*>(x + t * ldx + (long)c * 8);
    const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(wds[j]);
      const uint32_t two = (uint32_t)float_to_e4m3(f.x * is) | ((uint32_t)float_to_e4m3(f.y * is) << 8);
      if (j < 2) lo |= two << (16 * j); else hi |= two << (16 * (j - 2));
    }
    *reinterpret_cast<uint2*>(out + t * ldo + (long)c * 8) = make_uint2(lo, hi);
  }
}

// NVFP4 activation quant: per 16 values, scale = e4m3(amax / 6 * gs) where gs is the global
// scale (448 * 6 / tensor amax); values = e2m1(x * gs / scale). mode 0: x; mode 1: silu(gate) * up
// with x = [gate | up] rows of width 2K; mode 2: x * sigmoid(gate) with a separate gate tensor. Scales row-major [T, K/16] or in the 128x4-swizzled
// layout of block-scaled MMAs (swizzle = 1).
__global__ void __launch_bounds__(128)
    quant_nvfp4_kernel(const bf16* __restrict__ x, long ldx, const float* __restrict__ gscale,
                       uint8_t* __restrict__ out, uint8_t* __restrict__ sf, long T, int K, int mode,
                       int swizzle, const bf16* __restrict__ gate = nullptr, long ldg = 0) {
  const long groups = T * (long)(K / 16);
  const float gs = *gscale;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < groups; i += (long)gridDim.x * blockDim.x) {
    const long t = i / (K / 16);
    const int gidx = (int)(i % (K / 16));
    const bf16* src = x + t * ldx + (long)gidx * 16;
    float v[16];
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      float a = __bfloat162float(src[e]);
      if (mode == 1) {
        const float u = __bfloat162float(src[K + e]);
        a = __bfloat162float(__float2bfloat16(a / (1.f + __expf(-a)) * u));
      } else if (mode == 2) {
        // attention output gate: x * sigmoid(gate), rounded to bf16 as the separate kernel would
        const float g = __bfloat162float(gate[t * ldg + (long)gidx * 16 + e]);
        a = __bfloat162float(__float2bfloat16(a / (1.f + __expf(-g))));
      }
      v[e] = a;
      amax = fmaxf(amax, fabsf(a));
    }
    const uint8_t sb = float_to_e4m3(amax * gs / 6.f);
    const float sdec = e4m3_to_float(sb);
    const float mul = sdec > 0.f ? gs / sdec : 0.f;
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      w0 |= float_to_e2m1(v[e] * mul) << (e * 4);
      w1 |= float_to_e2m1(v[8 + e] * mul) << (e * 4);
    }
    reinterpret_cast<uint2*>(out)[i] = make_uint2(w0, w1);
    size_t so;
    if (swizzle) {
      // [T/128][K/64][32 rows][4 row-groups][4 k] bytes
      const long rb = t / 128, r = t % 128;
      const int kb = gidx / 4, kk = gidx % 4;
      so = ((size_t)rb * (K / 64) + kb) * 512 + (size_t)(r % 32) * 16 + (size_t)(r / 32) * 4 + kk;
    } else {
      so = (size_t)i;
    }
    sf[so] = sb;
  }
}

// (residual +) RMSNorm -> NVFP4 in one pass over the row: one block per token keeps the row (bf16,
// 16-byte vectors) in shared memory between the sum of squares and the quantisation; the updated
// residual is written back when given, the normalised row itself only when `normed` is given.
// The norm is rmsnorm_kernel's arithmetic (same vector striding, same two-level sum, launched with
// the same thread count) and the quantisation is quant_nvfp4_kernel's, so the fused kernel gives
// the bytes of the two run one after the other.
__device__ __forceinline__ float q_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float q_block_sum(float v, float* red) {
  v = q_warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = q_warp_sum(t);
  __syncthreads();
  return t;
}

__global__ void __launch_bounds__(256)
    rmsnorm_quant_nvfp4_kernel(const bf16* __restrict__ x, long ldx, bf16* residual, const bf16* __restrict__ w,
                               float eps, int gemma, const float* __restrict__ gscale, uint8_t* __restrict__ out,
                               uint8_t* __restrict__ sf, bf16* normed, long T, int K, int swizzle) {
  extern __shared__ uint4 row_cache[];     // K / 8 vectors
  __shared__ float red[32];
  const long t = blockIdx.x;
  const int nv = K >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + t * ldx);
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + t * (long)K) : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    uint4 v = xr[i];
    if (rr) {
      uint4 r = rr[i];
      float2 a, b;
      a = unpack_bf16x2(v.x); b = unpack_bf16x2(r.x); v.x = pack_bf16x2(a.x + b.x, a.y + b.y);
      a = unpack_bf16x2(v.y); b = unpack_bf16x2(r.y); v.y = pack_bf16x2(a.x + b.x, a.y + b.y);
      a = unpack_bf16x2(v.z); b = unpack_bf16x2(r.z); v.z = pack_bf16x2(a.x + b.x, a.y + b.y);
      a = unpack_bf16x2(v.w); b = unpack_bf16x2(r.w); v.w = pack_bf16x2(a.x + b.x, a.y + b.y);
      rr[i] = v;
    }
    row_cache[i] = v;
    float2 f;
    f = unpack_bf16x2(v.x); ss += f.x * f.x + f.y * f.y;
    f = unpack_bf16x2(v.y); ss += f.x * f.x + f.y * f.y;
    f = unpack_bf16x2(v.z); ss += f.x * f.x + f.y * f.y;
    f = unpack_bf16x2(v.w); ss += f.x * f.x + f.y * f.y;
  }
  ss = q_block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)K + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* nrow = normed ? reinterpret_cast<uint4*>(normed + t * (long)K) : nullptr;
  const float g = gemma ? 1.f : 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const uint4 v = row_cache[i];
    const uint4 wv = wr[i];
    uint4 o;
    float2 a, b;
    a = unpack_bf16x2(v.x); b = unpack_bf16x2(wv.x); o.x = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
    a = unpack_bf16x2(v.y); b = unpack_bf16x2(wv.y); o.y = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
    a = unpack_bf16x2(v.z); b = unpack_bf16x2(wv.z); o.z = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
    a = unpack_bf16x2(v.w); b = unpack_bf16x2(wv.w); o.w = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
    row_cache[i] = o;
    if (nrow) nrow[i] = o;
  }
  __syncthreads();               // groups below span vectors written by other threads
  const float gs = *gscale;
  for (int gidx = threadIdx.x; gidx < (K >> 4); gidx += blockDim.x) {
    const uint4 v0 = row_cache[2 * gidx], v1 = row_cache[2 * gidx + 1];
    const uint32_t wds[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    float v[16];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float2 f = unpack_bf16x2(wds[j]);
      v[2 * j] = f.x; v[2 * j + 1] = f.y;
      amax = fmaxf(amax, fabsf(f.x));
      amax = fmaxf(amax, fabsf(f.y));
    }
    const uint8_t sb = float_to_e4m3(amax * gs / 6.f);
    const float sdec = e4m3_to_float(sb);
    const float mul = sdec > 0.f ? gs / sdec : 0.f;
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      w0 |= float_to_e2m1(v[e] * mul) << (e * 4);
      w1 |= float_to_e2m1(v[8 + e] * mul) << (e * 4);
    }
    reinterpret_cast<uint2*>(out)[t * (K / 16) + gidx] = make_uint2(w0, w1);
    sf[swizzle ? nvfp4_sf_chunk_offset(t, gidx, K) : (size_t)t * (K / 16) + gidx] = sb;
  }
}

// out = (sum over splits of partials) * a_scale * w_scale (+ bias), four columns per thread.
__global__ void __launch_bounds__(256)
    fp8_splitk_reduce_kernel(const float* __restrict__ partials, int splits, int M, int N,
                             const float* __restrict__ a_scale, int a_per_token, const float* __restrict__ w_scale,
                             int w_per_channel, const bf16* __restrict__ bias, bf16* __restrict__ out, int ldo) {
  const int nq = N >> 2;
  const size_t total = (size_t)M * nq;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int row = (int)(i / nq), col = (int)(i % nq) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int sp = 0; sp < splits; ++sp) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(partials + ((size_t)sp * M + row) * N + col));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    const float sa = a_per_token ? a_scale[row] : a_scale[0];
    float4 sw = w_per_channel ? *reinterpret_cast<const float4*>(w_scale + col)
                              : make_float4(w_scale[0], w_scale[0], w_scale[0], w_scale[0]);
    acc.x *= sa * sw.x; acc.y *= sa * sw.y; acc.z *= sa * sw.z; acc.w *= sa * sw.w;
    if (bias) {
      const uint2 b = *reinterpret_cast<const uint2*>(bias + col);
      const float2 b0 = unpack_bf16x2(b.x), b1 = unpack_bf16x2(b.y);
      acc.x += b0.x; acc.y += b0.y; acc.z += b1.x; acc.w += b1.y;
    }
    *reinterpret_cast<uint2*>(out + (size_t)row * ldo + col) =
        make_uint2(pack_bf16x2(acc.x, acc.y), pack_bf16x2(acc.z, acc.w));
  }
}

// Split-K scratch of the current device: one 128 x 128 fp32 partial per SM (a split plan never has
// more work items than SMs). Allocated by b200_init_device() or by a first use outside a capture.
static float* fp8_splitk_scratch(cudaStream_t stream) {
  static std::mutex mu;
  static float* g_part[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!g_part[dev]) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) return nullptr;
    float* pp = nullptr;
    if (cudaMalloc(&pp, (size_t)b200_num_sms() * kQM * kQN * sizeof(float)) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    g_part[dev] = pp;
  }
  return g_part[dev];
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_gemm_fp8_pair(const void* A, int lda, const void* W, int ldw, void* out, int ldo,
                       const float* a_scale, const float* w_scale, int w_scale_per_channel, const void* bias,
                       int M, int N, int K, cudaStream_t stream);

int b200_gemm_fp8(const void* A, int lda, const void* W, int ldw, void* out, int ldo, const float* a_scale,
                  const float* w_scale, int w_scale_per_channel, const void* bias, int M, int N, int K,
                  cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 15) || (lda & 15) || (ldw & 15) || (N & 7) || (ldo & 7)) return -1;
  // prefill-sized batches: CTA pairs, 256 x 256 tiles, stream-K (the 128 x 128 kernel below keeps
  // the small batches)
  if (M > 256 && N >= 256)
    return b200_gemm_fp8_pair(A, lda, W, ldw, out, ldo, a_scale, w_scale, w_scale_per_channel, bias, M, N, K,
                              stream);
  CUtensorMap tmA, tmB;
  if (!encode_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, kQM, kQKB, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !encode_tmap_2d(&tmB, W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldw, kQN, kQKB, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  Fp8Params p{};
  p.M = M; p.N = N; p.K = K; p.out = (bf16*)out; p.ldo = ldo;
  p.a_scale = a_scale; p.w_scale = w_scale; p.w_scale_per_channel = w_scale_per_channel & 1;
  p.a_scale_per_token = (w_scale_per_channel >> 1) & 1;
  p.bias = (const bf16*)bias;
  p.tiles_m = (M + kQM - 1) / kQM; p.tiles_n = (N + kQN - 1) / kQN;
  const int kblocks = (K + kQKB - 1) / kQKB;
  p.stages = kblocks + 1 < 6 ? (kblocks + 1 < 2 ? 2 : kblocks + 1) : 6;
  p.status = device_status_word();
  // few tiles and a long K (decode batches against the down projection): split K over the idle
  // SMs, at least four k-blocks per split, partial sums through the per-device scratch
  p.splits = 1;
  p.kb_per_split = kblocks;
  {
    const int tiles0 = p.tiles_m * p.tiles_n, sms = b200_num_sms();
    int splits = sms / tiles0;
    if (splits > kblocks / 4) splits = kblocks / 4;
    if (splits > 16) splits = 16;
    if (splits >= 2 && !(N & 3) && !(ldo & 3)) {
      float* scratch = fp8_splitk_scratch(stream);
      if (scratch) {
        p.kb_per_split = (kblocks + splits - 1) / splits;
        p.splits = (kblocks + p.kb_per_split - 1) / p.kb_per_split;
        p.partials = scratch;
        p.stages = p.kb_per_split + 1 < 6 ? (p.kb_per_split + 1 < 2 ? 2 : p.kb_per_split + 1) : 6;
      }
    }
  }
  const size_t smem = (size_t)p.stages * (kQM * kQKB + kQN * kQKB) + 1024 + sizeof(QBars);
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 6 * 32768 + 2048 + (int)sizeof(QBars));
  }
  const int tiles = p.tiles_m * p.tiles_n * p.splits;
  const int grid = tiles < b200_num_sms() ? tiles : b200_num_sms();
  gemm_fp8_kernel<<<grid, kQThreads, smem, stream>>>(tmA, tmB, p);
  if (cudaGetLastError() != cudaSuccess) return -2;
  if (p.splits > 1) {
    const size_t total = (size_t)M * (N / 4);
    long blocks = (long)((total + 255) / 256);
    if (blocks > (long)b200_num_sms() * 8) blocks = (long)b200_num_sms() * 8;
    fp8_splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, stream>>>(p.partials, p.splits, M, N, a_scale,
                                                                   p.a_scale_per_token, w_scale, p.w_scale_per_channel,
                                                                   (const bf16*)bias, (bf16*)out, ldo);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_fp8_init_device() {
  if (b200_num_sms() <= 0) return -2;
  return fp8_splitk_scratch(nullptr) ? 0 : -2;
}

int b200_nvfp4_dequant(const void* packed, const void* sf, const float* gscale, void* out, long N, int K,
                       cudaStream_t stream) {
  if (N <= 0 || K <= 0) return 0;
  if (K & 15) return -1;
  const long groups = N * (long)(K / 16);
  long blocks = (groups + 255) / 256;
  if (blocks > (long)b200_num_sms() * 16) blocks = (long)b200_num_sms() * 16;
  nvfp4_dequant_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const uint8_t*)packed, (const uint8_t*)sf, gscale,
                                                             (bf16*)out, N, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_quant_fp8(const void* x, long ldx, const void* norm_w, float eps, int gemma, const float* scale,
                   void* out, long ldo, long T, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  quant_fp8_kernel<<<(unsigned)T, 256, 0, stream>>>((const bf16*)x, ldx, (const bf16*)norm_w, eps, gemma, scale,
                                                    (uint8_t*)out, ldo, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// scratch: two words (maximum bits, then the scale = amax / 448 the GEMM reads as a_scale).
int b200_quant_fp8_dynamic(const void* x, long ldx, void* scratch, void* out, long ldo, long T, int H,
                           cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((H & 7) || (ldx & 7) || (ldo & 7) || ((uintptr_t)x & 15) || ((uintptr_t)out & 7)) return -1;
  if (cudaMemsetAsync(scratch, 0, 4, stream) != cudaSuccess) return -2;
  const long vecs = T * (long)(H / 8);
  long blocks = (vecs + 255) / 256;
  if (blocks > (long)b200_num_sms() * 8) blocks = (long)b200_num_sms() * 8;
  absmax_bf16_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const bf16*)x, ldx, T, H, (unsigned*)scratch);
  quant_fp8_dynamic_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const bf16*)x, ldx, (const unsigned*)scratch,
                                                                 (float*)scratch + 1, (uint8_t*)out, ldo, T, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_quant_nvfp4(const void* x, long ldx, const float* gscale, void* out, void* sf, long T, int K, int mode,
                     int swizzle, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((K & 15) || (swizzle && (K & 63))) return -1;
  const long groups = T * (long)(K / 16);
  long blocks = (groups + 127) / 128;
  if (blocks > (long)b200_num_sms() * 32) blocks = (long)b200_num_sms() * 32;
  quant_nvfp4_kernel<<<(unsigned)blocks, 128, 0, stream>>>((const bf16*)x, ldx, gscale, (uint8_t*)out, (uint8_t*)sf,
                                                           T, K, mode, swizzle);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// x * sigmoid(gate) -> NVFP4 (the gated attention output that feeds o_proj).
int b200_quant_nvfp4_gated(const void* x, long ldx, const void* gate, long ldg, const float* gscale, void* out,
                           void* sf, long T, int K, int swizzle, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((K & 15) || (swizzle && (K & 63)) || !gate) return -1;
  const long groups = T * (long)(K / 16);
  long blocks = (groups + 127) / 128;
  if (blocks > (long)b200_num_sms() * 32) blocks = (long)b200_num_sms() * 32;
  quant_nvfp4_kernel<<<(unsigned)blocks, 128, 0, stream>>>((const bf16*)x, ldx, gscale, (uint8_t*)out, (uint8_t*)sf,
                                                           T, K, 2, swizzle, (const bf16*)gate, ldg);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// (residual += x;) RMSNorm -> NVFP4. residual [T, K] contiguous bf16 or null; normed [T, K] bf16 or null.
int b200_rmsnorm_quant_nvfp4(const void* x, long ldx, void* residual, const void* weight, float eps, int gemma,
                             const float* gscale, void* out, void* sf, void* normed, long T, int K, int swizzle,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((K & 15) || (swizzle && (K & 63)) || K > 32768) return -1;
  static PerDeviceOnce attr_once;
  if (attr_once.first())
    cudaFuncSetAttribute(rmsnorm_quant_nvfp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * 4);
  if ((ldx & 7) || ((uintptr_t)x & 15) || ((uintptr_t)weight & 15) || ((uintptr_t)residual & 15) ||
      ((uintptr_t)normed & 15))
    return -1;
  int threads = K / 8 >= 256 ? 256 : ((K / 8 + 31) / 32) * 32;      // as b200_rmsnorm launches its kernel
  if (threads < 32) threads = 32;
  rmsnorm_quant_nvfp4_kernel<<<(unsigned)T, threads, (size_t)K * 2, stream>>>(
      (const bf16*)x, ldx, (bf16*)residual, (const bf16*)weight, eps, gemma, gscale, (uint8_t*)out, (uint8_t*)sf,
      (bf16*)normed, T, K, swizzle);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
