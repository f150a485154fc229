// Row-wise normalisation and element-wise activation kernels (HBM-bound; every access is a
// 16-byte vector, one pass over the data, fp32 math, bf16 storage).
//
//   rmsnorm / fused residual-add + rmsnorm (std and gemma "1+w")   reference:
//       src/vt/cuda/cuda_ops.cu:63 (RmsNormRowKernel), :165 (RmsNormRowFastKernel)
//   layernorm                                                      cuda_layernorm.cu:68
//   silu_and_mul, gelu_tanh_and_mul, relu, add, mul_scalar, softcap, casts
//       cuda_ops.cu:417,463,510,550; cuda_layernorm.cu:164,200; cuda_glue.cu:47-100
//   embedding gather with a bounds flag in the status word         cuda_ops.cu:600
//   gather_rows (logits-row gather before lm_head)
#include "api.h"
#include "quant_codec.cuh"
#include "sm100.cuh"

namespace b200 {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// x: [T, H] bf16 (row stride ldx). If residual != nullptr: residual += x (bf16-rounded) and
// the norm is taken over the updated residual. out may alias x.
__global__ void __launch_bounds__(256)
    rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, int ldx, __nv_bfloat16* residual,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* out, int ldo, int H,
                   float eps, int gemma) {
  __shared__ float red[32];
  extern __shared__ uint4 row_cache[];  // H/8 vectors
  pdl_wait();                 // predecessor grid complete, its writes visible
  pdl_launch_dependents();    // the successor may become resident (it waits the same way)
  const int t = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)t * ldx);
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + (size_t)t * H) : nullptr;
  const int nv = H >> 3;
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
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  uint4* orow = reinterpret_cast<uint4*>(out + (size_t)t * ldo);
  const float g = gemma ? 1.f : 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    uint4 v = row_cache[i];
    uint4 wv = wr[i];
    uint4 o;
    float2 a, b;
    a = unpack_bf16x2(v.x); b = unpack_bf16x2(wv.x); o.x = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
    a = unpack_bf16x2(v.y); b = unpack_bf16x2(wv.y); o.y = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
    a = unpack_bf16x2(v.z); b = unpack_bf16x2(wv.z); o.z = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
    a = unpack_bf16x2(v.w); b = unpack_bf16x2(wv.w); o.w = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
    orow[i] = o;
  }
}

// LayerNorm with affine weight and optional bias; scalar loop (any H).
__global__ void __launch_bounds__(256)
    layernorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                     const __nv_bfloat16* __restrict__ b, __nv_bfloat16* out, int H, float eps) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  const __nv_bfloat16* xr = x + (size_t)t * H;
  float s = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) s += __bfloat162float(xr[i]);
  const float mean = block_sum(s, red) / (float)H;
  float v = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float d = __bfloat162float(xr[i]) - mean;
    v += d * d;
  }
  const float inv = rsqrtf(block_sum(v, red) / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float y = (__bfloat162float(xr[i]) - mean) * inv * __bfloat162float(w[i]);
    if (b) y += __bfloat162float(b[i]);
    out[(size_t)t * H + i] = __float2bfloat16(y);
  }
}

enum ActKind : int { kSilu = 0, kGeluTanh = 1, kGeluErf = 2 };

__device__ __forceinline__ float act_fn(float g, int kind) {
  if (kind == kSilu) return g / (1.f + __expf(-g));
  if (kind == kGeluTanh) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * g * (1.f + tanhf(k0 * (g + k1 * g * g * g)));
  }
  return 0.5f * g * (1.f + erff(g * 0.7071067811865476f));
}

// x: [T, 2*I] = [gate | up] (or, with kind | 0x100, blocks of [128 gate | 128 up]);
// out: [T, I] = act(gate) * up.
__global__ void __launch_bounds__(256)
    act_and_mul_kernel(const __nv_bfloat16* __restrict__ x, int ldx, __nv_bfloat16* out, int I,
                       int T, int kind_flags) {
  pdl_wait();                 // predecessor grid complete, its writes visible
  pdl_launch_dependents();    // the successor may become resident (it waits the same way)
  const int kind = kind_flags & 0xff;
  const bool il = (kind_flags & 0x100) != 0;
  const int nv = I >> 3;
  const size_t total = (size_t)T * nv;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    int t = (int)(idx / nv), i = (int)(idx % nv);
    // interleaved input: blocks of [128 gate | 128 up] instead of [all gate | all up]
    const int goff = il ? ((i * 8) >> 7) * 256 + ((i * 8) & 127) : i * 8;
    const int uoff = il ? goff + 128 : I + i * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(x + (size_t)t * ldx + goff);
    const uint4 u = *reinterpret_cast<const uint4*>(x + (size_t)t * ldx + uoff);
    uint4 o;
    float2 a, b;
    a = unpack_bf16x2(g.x); b = unpack_bf16x2(u.x); o.x = pack_bf16x2(act_fn(a.x, kind) * b.x, act_fn(a.y, kind) * b.y);
    a = unpack_bf16x2(g.y); b = unpack_bf16x2(u.y); o.y = pack_bf16x2(act_fn(a.x, kind) * b.x, act_fn(a.y, kind) * b.y);
    a = unpack_bf16x2(g.z); b = unpack_bf16x2(u.z); o.z = pack_bf16x2(act_fn(a.x, kind) * b.x, act_fn(a.y, kind) * b.y);
    a = unpack_bf16x2(g.w); b = unpack_bf16x2(u.w); o.w = pack_bf16x2(act_fn(a.x, kind) * b.x, act_fn(a.y, kind) * b.y);
    *reinterpret_cast<uint4*>(out + (size_t)t * I + i * 8) = o;
  }
}

// Row-wise dynamic fp8: each token row gets its own scale (max|v| / 448), written to scales[t]
// for the GEMM's epilogue, and the producer of the row runs in the same pass:
//   mode 0  v = x
//   mode 1  v = RMSNorm(x (+ residual, written back)) -- the arithmetic of rmsnorm_kernel, so the
//           normalised row has the bytes the bf16 path would hand to its GEMM
//   mode 2  v = act(gate) * up from [gate | up] rows (kind_flags as act_and_mul_kernel takes them)
// The row (bf16) stays in shared memory between the producer and the quantisation.
__global__ void __launch_bounds__(256)
    rowquant_fp8_kernel(const __nv_bfloat16* __restrict__ x, long ldx, __nv_bfloat16* residual,
                        const __nv_bfloat16* __restrict__ w, float eps, int gemma, int mode, int kind_flags,
                        uint8_t* __restrict__ out, long ldo, float* __restrict__ scales, int K) {
  __shared__ float red[32];
  extern __shared__ uint4 row_cache[];  // K/8 vectors
  const long t = blockIdx.x;
  const int nv = K >> 3;
  float amax = 0.f;
  auto vec_amax = [&](const uint4& v) {
    float2 f;
    f = unpack_bf16x2(v.x); amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    f = unpack_bf16x2(v.y); amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    f = unpack_bf16x2(v.z); amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    f = unpack_bf16x2(v.w); amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
  };
  if (mode == 1) {
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
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)K + eps);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
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
      vec_amax(o);
    }
  } else if (mode == 2) {
    const int kind = kind_flags & 0xff;
    const bool il = (kind_flags & 0x100) != 0;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      const int goff = il ? ((i * 8) >> 7) * 256 + ((i * 8) & 127) : i * 8;
      const int uoff = il ? goff + 128 : K + i * 8;
      const uint4 gt = *reinterpret_cast<const uint4*>(x + t * ldx + goff);
      const uint4 u = *reinterpret_cast<const uint4*>(x + t * ldx + uoff);
      uint4 o;
      float2 a, b;
      a = unpack_bf16x2(gt.x); b = unpack_bf16x2(u.x); o.x = pack_bf16x2(act_fn(a.x, kind) * b.x, act_fn(a.y, kind) * b.y);
      a = unpack_bf16x2(gt.y); b = unpack_bf16x2(u.y); o.y = pack_bf16x2(act_fn(a.x, kind) * b.x, act_fn(a.y, kind) * b.y);
      a = unpack_bf16x2(gt.z); b = unpack_bf16x2(u.z); o.z = pack_bf16x2(act_fn(a.x, kind) * b.x, act_fn(a.y, kind) * b.y);
      a = unpack_bf16x2(gt.w); b = unpack_bf16x2(u.w); o.w = pack_bf16x2(act_fn(a.x, kind) * b.x, act_fn(a.y, kind) * b.y);
      row_cache[i] = o;
      vec_amax(o);
    }
  } else {
    const uint4* xr = reinterpret_cast<const uint4*>(x + t * ldx);
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      const uint4 v = xr[i];
      row_cache[i] = v;
      vec_amax(v);
    }
  }
  // block maximum (every thread re-reads only the vectors it wrote, so no barrier is needed for
  // row_cache itself)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  float m = (lane < nw) ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  const float sc = fmaxf(m, 1e-12f) / 448.f;
  const float is = 1.f / sc;
  if (threadIdx.x == 0) scales[t] = sc;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const uint4 v = row_cache[i];
    const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16x2(wds[j]);
      const uint32_t two = (uint32_t)float_to_e4m3(f.x * is) | ((uint32_t)float_to_e4m3(f.y * is) << 8);
      if (j < 2) lo |= two << (16 * j); else hi |= two << (16 * (j - 2));
    }
    *reinterpret_cast<uint2*>(out + t * ldo + (long)i * 8) = make_uint2(lo, hi);
  }
}

enum EwKind : int { kEwAdd = 0, kEwRelu = 1, kEwMulScalar = 2, kEwSoftcap = 3, kEwSigmoidMul = 4,
                    kEwMul = 5 };

// Generic bf16 element-wise op over n elements (n % 8 == 0). b may be null.
__global__ void __launch_bounds__(256)
    eltwise_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                   __nv_bfloat16* out, size_t n, int kind, float scalar) {
  const size_t nv = n >> 3;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < nv;
       idx += (size_t)gridDim.x * blockDim.x) {
    uint4 va = reinterpret_cast<const uint4*>(a)[idx];
    uint4 vb = b ? reinterpret_cast<const uint4*>(b)[idx] : make_uint4(0, 0, 0, 0);
    uint32_t* pa = reinterpret_cast<uint32_t*>(&va);
    uint32_t* pb = reinterpret_cast<uint32_t*>(&vb);
    uint4 vo;
    uint32_t* po = reinterpret_cast<uint32_t*>(&vo);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 x = unpack_bf16x2(pa[j]), y = unpack_bf16x2(pb[j]), r;
      switch (kind) {
        case kEwAdd: r.x = x.x + y.x; r.y = x.y + y.y; break;
        case kEwRelu: r.x = fmaxf(x.x, 0.f); r.y = fmaxf(x.y, 0.f); break;
        case kEwMulScalar: r.x = x.x * scalar; r.y = x.y * scalar; break;
        case kEwSoftcap: r.x = scalar * tanhf(x.x / scalar); r.y = scalar * tanhf(x.y / scalar); break;
        case kEwSigmoidMul:  // a * sigmoid(b)
          r.x = x.x / (1.f + __expf(-y.x)); r.y = x.y / (1.f + __expf(-y.y)); break;
        default: r.x = x.x * y.x; r.y = x.y * y.y; break;
      }
      po[j] = pack_bf16x2(r.x, r.y);
    }
    reinterpret_cast<uint4*>(out)[idx] = vo;
  }
}

__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ a, float* out, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    out[i] = __bfloat162float(a[i]);
}
__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ a, __nv_bfloat16* out, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(a[i]);
}

// out[t, :] = table[ids[t], :] * scale; an id outside [0, vocab) writes zeros and flags the
// status word (no allocation, no sync: safe inside CUDA graphs). With vocab sharding
// (vocab_start > 0 or a partial table) rows outside the shard are zero without a flag.
__global__ void __launch_bounds__(128)
    embedding_kernel(const int64_t* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                     __nv_bfloat16* out, int H, int64_t vocab_start, int64_t vocab_rows,
                     int64_t vocab_total, float scale, int* status) {
  const int t = blockIdx.x;
  const int64_t id = ids[t];
  const int nv = H >> 3;
  uint4* o = reinterpret_cast<uint4*>(out + (size_t)t * H);
  const int64_t local = id - vocab_start;
  if (id < 0 || id >= vocab_total) {
    if (threadIdx.x == 0 && status) atomicExch(status, (int)kErrBadArg);
  }
  if (local < 0 || local >= vocab_rows || id < 0 || id >= vocab_total) {
    for (int i = threadIdx.x; i < nv; i += blockDim.x) o[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)local * H);
  if (scale == 1.f) {
    for (int i = threadIdx.x; i < nv; i += blockDim.x) o[i] = src[i];
  } else {
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      uint4 v = src[i];
      float2 f;
      f = unpack_bf16x2(v.x); v.x = pack_bf16x2(f.x * scale, f.y * scale);
      f = unpack_bf16x2(v.y); v.y = pack_bf16x2(f.x * scale, f.y * scale);
      f = unpack_bf16x2(v.z); v.z = pack_bf16x2(f.x * scale, f.y * scale);
      f = unpack_bf16x2(v.w); v.w = pack_bf16x2(f.x * scale, f.y * scale);
      o[i] = v;
    }
  }
}

// out[i, :] = x[idx[i], :]  (rows of `bytes_per_row` bytes, multiple of 16)
__global__ void __launch_bounds__(128)
    gather_rows_kernel(const uint8_t* __restrict__ x, const int32_t* __restrict__ idx,
                       uint8_t* out, int row_bytes, int n_src) {
  const int i = blockIdx.x;
  int s = idx[i];
  if (s < 0 || s >= n_src) s = 0;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)s * row_bytes);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)i * row_bytes);
  for (int j = threadIdx.x; j < (row_bytes >> 4); j += blockDim.x) dst[j] = src[j];
}

static inline int ew_grid(size_t work_items) {
  size_t b = (work_items + 255) / 256;
  size_t cap = (size_t)b200_num_sms() * 16;
  return (int)(b < cap ? (b ? b : 1) : cap);
}

}  // namespace b200

using namespace b200;
typedef __nv_bfloat16 bf16;

extern "C" {

int b200_rmsnorm(const void* x, int ldx, void* residual, const void* w, void* out, int ldo, int T,
                 int H, float eps, int gemma, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((H & 7) || (ldx & 7) || (ldo & 7) || H > 32768) return -1;
  int threads = H / 8 >= 256 ? 256 : ((H / 8 + 31) / 32) * 32;
  if (threads < 32) threads = 32;
  return launch_pdl(rmsnorm_kernel, dim3(T), dim3(threads), (size_t)H * 2, stream, (const bf16*)x, ldx,
                    (bf16*)residual, (const bf16*)w, (bf16*)out, ldo, H, eps, gemma) == cudaSuccess ? 0 : -2;
}

// x: mode 0 / 1 rows of K values, mode 2 rows of [gate | up] (2K values). out: fp8 [T, K] (row
// stride ldo bytes), scales: fp32 [T]. Launched with the thread count b200_rmsnorm uses for this
// width, so that mode 1 sums in the same order.
int b200_quant_fp8_rowwise(const void* x, long ldx, void* residual, const void* norm_w, float eps, int gemma,
                           int mode, int kind_flags, void* out, long ldo, void* scales, int T, int K,
                           cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((K & 7) || (ldx & 7) || (ldo & 7) || K > 32768 || mode < 0 || mode > 2) return -1;
  if (((uintptr_t)x & 15) || ((uintptr_t)out & 7) || (mode == 1 && !norm_w)) return -1;
  if (mode == 2 && (kind_flags & 0x100) && (K & 127)) return -1;
  int threads = K / 8 >= 256 ? 256 : ((K / 8 + 31) / 32) * 32;
  if (threads < 32) threads = 32;
  static PerDeviceOnce attr_once;
  if (attr_once.first())
    cudaFuncSetAttribute(rowquant_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * 2);
  rowquant_fp8_kernel<<<T, threads, (size_t)K * 2, stream>>>((const bf16*)x, ldx, (bf16*)residual, (const bf16*)norm_w,
                                                           eps, gemma, mode, kind_flags, (uint8_t*)out, ldo,
                                                           (float*)scales, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_layernorm(const void* x, const void* w, const void* b, void* out, int T, int H, float eps,
                   cudaStream_t stream) {
  if (T <= 0) return 0;
  layernorm_kernel<<<T, 256, 0, stream>>>((const bf16*)x, (const bf16*)w, (const bf16*)b,
                                          (bf16*)out, H, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_act_and_mul(const void* x, int ldx, void* out, int T, int I, int kind,
                     cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((I & 7) || (ldx & 7)) return -1;
  if ((kind & 0x100) && (I & 127)) return -1;      // interleaved layout needs whole blocks
  return launch_pdl(act_and_mul_kernel, dim3(ew_grid((size_t)T * (I / 8))), dim3(256), 0, stream, (const bf16*)x,
                    ldx, (bf16*)out, I, T, kind) == cudaSuccess ? 0 : -2;
}

int b200_eltwise(const void* a, const void* b, void* out, size_t n, int kind, float scalar,
                 cudaStream_t stream) {
  if (n == 0) return 0;
  if (n & 7) return -1;
  eltwise_kernel<<<ew_grid(n / 8), 256, 0, stream>>>((const bf16*)a, (const bf16*)b, (bf16*)out, n,
                                                     kind, scalar);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_cast_bf16_f32(const void* a, void* out, size_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  cast_bf16_to_f32_kernel<<<ew_grid(n), 256, 0, stream>>>((const bf16*)a, (float*)out, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
int b200_cast_f32_bf16(const void* a, void* out, size_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  cast_f32_to_bf16_kernel<<<ew_grid(n), 256, 0, stream>>>((const float*)a, (bf16*)out, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_embedding(const void* ids, const void* table, void* out, int T, int H,
                   int64_t vocab_start, int64_t vocab_rows, int64_t vocab_total, float scale,
                   cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H & 7) return -1;
  embedding_kernel<<<T, 128, 0, stream>>>((const int64_t*)ids, (const bf16*)table, (bf16*)out, H,
                                          vocab_start, vocab_rows, vocab_total, scale,
                                          device_status_word());
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_gather_rows(const void* x, const void* idx, void* out, int n_out, int n_src,
                     int row_bytes, cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (row_bytes & 15) return -1;
  gather_rows_kernel<<<n_out, 128, 0, stream>>>((const uint8_t*)x, (const int32_t*)idx,
                                                (uint8_t*)out, row_bytes, n_src);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
