// Attention preamble fused into one pass over the merged QKV activations:
//   optional per-head RMSNorm on q and k (std or gemma "1+w"), RoPE from a precomputed
//   cos/sin table (NeoX halves or GPT-J pairs, partial rotary), q written back in place,
//   k / v scattered into the paged KV cache by slot.
//
// KV cache layout (one buffer per layer): [num_blocks, 2, block_size, Hkv, D] bf16;
// slot = block * block_size + offset; slot < 0 => skip (CUDA-graph padding rows).
//
// Replaces the reference op chain RmsNorm(per head) -> RopeFromCache -> ReshapeAndCache
// (src/vt/cuda/cuda_ops.cu:783, :964 AttnQkNormRopeGateKernel; cuda_cache.cu:42).
// Also here: MLA cache write (cuda_cache.cu:113 ConcatAndCacheMlaKernel) and the plain
// reshape_and_cache used when K/V arrive already rotated.
#include "api.h"
#include "sm100.cuh"

namespace b200 {

struct RopeKvParams {
  __nv_bfloat16* qkv;  // [T, ld] : q heads | k heads | v heads  (q may carry a gate, see q_stride)
  int ld;
  int q_off, k_off, v_off;  // element offsets of the three sections inside a row
  int q_head_stride;        // elements between consecutive q heads (D, or 2*D with interleaved gate)
  int Hq, Hkv, D, rot;
  const int64_t* positions;  // [T]
  const float* cos_sin;      // [max_pos, rot] : cos[rot/2] | sin[rot/2]
  const __nv_bfloat16* q_norm_w;  // [D] or null
  const __nv_bfloat16* k_norm_w;  // [D] or null
  float eps;
  int gemma;
  int neox;
  const int64_t* slot_mapping;  // [T] or null (no cache write)
  __nv_bfloat16* kv_cache;
  int block_size;
  __nv_bfloat16* q_out;  // optional separate q destination [T, Hq*D]; null => in place
  int vec4;              // D == rot == 128, neox, 8-byte aligned rows: rope_kv_vec4_kernel applies
};

// One warp per (token, head). Heads 0..Hq-1 are q, Hq..Hq+Hkv-1 are k, then Hkv v heads.
__global__ void __launch_bounds__(128) rope_kv_kernel(RopeKvParams p, int T) {
  __shared__ float buf[4][256];
  pdl_wait();                 // predecessor grid complete, its writes visible
  pdl_launch_dependents();    // the successor may become resident (it waits the same way)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nheads = p.Hq + 2 * p.Hkv;
  const long long gw = (long long)blockIdx.x * 4 + warp;
  if (gw >= (long long)T * nheads) return;
  const int t = (int)(gw / nheads);
  const int h = (int)(gw % nheads);
  const int D = p.D;
  float* b = buf[warp];
  __nv_bfloat16* row = p.qkv + (size_t)t * p.ld;

  if (h >= p.Hq + p.Hkv) {
    // ---- V head: straight copy into the cache ----
    if (!p.slot_mapping) return;
    const int64_t slot = p.slot_mapping[t];
    if (slot < 0) return;
    const int hv = h - p.Hq - p.Hkv;
    const __nv_bfloat16* src = row + p.v_off + hv * D;
    const int64_t blk = slot / p.block_size, off = slot % p.block_size;
    __nv_bfloat16* dst =
        p.kv_cache + (((blk * 2 + 1) * p.block_size + off) * p.Hkv + hv) * (int64_t)D;
    for (int i = lane; i < (D >> 3); i += 32)
      reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    return;
  }

  const bool is_q = h < p.Hq;
  __nv_bfloat16* src = is_q ? row + p.q_off + h * p.q_head_stride : row + p.k_off + (h - p.Hq) * D;
  const __nv_bfloat16* nw = is_q ? p.q_norm_w : p.k_norm_w;

  float ss = 0.f;
  for (int i = lane; i < D; i += 32) {
    float v = __bfloat162float(src[i]);
    b[i] = v;
    ss += v * v;
  }
  if (nw) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss / (float)D + p.eps);
    const float g = p.gemma ? 1.f : 0.f;
    for (int i = lane; i < D; i += 32) {
      // Round through bf16 like the unfused chain (norm output is a bf16 tensor).
      b[i] = __bfloat162float(__float2bfloat16(b[i] * inv * (__bfloat162float(nw[i]) + g)));
    }
  }
  __syncwarp();

  __nv_bfloat16* dst;
  if (is_q) {
    dst = p.q_out ? p.q_out + ((size_t)t * p.Hq + h) * D : src;
  } else {
    dst = nullptr;
    if (p.slot_mapping) {
      const int64_t slot = p.slot_mapping[t];
      if (slot >= 0) {
        const int64_t blk = slot / p.block_size, off = slot % p.block_size;
        dst = p.kv_cache + (((blk * 2 + 0) * p.block_size + off) * p.Hkv + (h - p.Hq)) * (int64_t)D;
      }
    }
  }
  const int half = p.rot >> 1;
  const float* cs = p.cos_sin ? p.cos_sin + (size_t)p.positions[t] * p.rot : nullptr;
  for (int i = lane; i < D; i += 32) {
    float v = b[i];
    if (cs && i < p.rot) {
      if (p.neox) {
        const int j = i < half ? i : i - half;
        const float c = cs[j], s = cs[half + j];
        v = i < half ? b[i] * c - b[i + half] * s : b[i] * c + b[i - half] * s;
      } else {
        const int j = i >> 1;
        const float c = cs[j], s = cs[half + j];
        v = (i & 1) ? b[i] * c + b[i - 1] * s : b[i] * c - b[i + 1] * s;
      }
    }
    const __nv_bfloat16 o = __float2bfloat16(v);
    if (dst) dst[i] = o;
    // Keep the rotated k in the activation row too (prefill reads it from the cache only,
    // but the in-place row stays consistent for callers that look at it).
    if (!is_q) src[i] = o;
  }
}

// Vectorised form for 128-dim heads with a full neox rotation (p.vec4): one warp takes kHG
// consecutive heads of one token. Lane l holds dims 4l..4l+3 of a head (one 8-byte load), its
// rotation partner (dim +-64) sits in lane l ^ 16; the token's cos / sin row and cache slot are
// fetched once per warp and the kHG head loads are issued together, so the dependent global
// round trips are paid once per eight heads instead of once per head.
static constexpr int kHG = 8;
__global__ void __launch_bounds__(128) rope_kv_vec4_kernel(RopeKvParams p, int T) {
  pdl_wait();                 // predecessor grid complete, its writes visible
  pdl_launch_dependents();    // the successor may become resident (it waits the same way)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nheads = p.Hq + 2 * p.Hkv;
  const int groups = (nheads + kHG - 1) / kHG;
  const long long gw = (long long)blockIdx.x * 4 + warp;
  if (gw >= (long long)T * groups) return;
  const int t = (int)(gw / groups);
  const int h0 = (int)(gw % groups) * kHG;
  const int nh = min(kHG, nheads - h0);
  __nv_bfloat16* row = p.qkv + (size_t)t * p.ld;
  const int kv0 = p.Hq;              // first k head
  const int v0 = p.Hq + p.Hkv;       // first v head

  const __nv_bfloat16* src[kHG];
  uint2 raw[kHG];
#pragma unroll
  for (int i = 0; i < kHG; ++i) {
    const int h = h0 + i;
    src[i] = h < kv0 ? row + p.q_off + h * p.q_head_stride
                     : (h < v0 ? row + p.k_off + (h - kv0) * 128 : row + p.v_off + (h - v0) * 128);
    if (i < nh) raw[i] = *reinterpret_cast<const uint2*>(src[i] + lane * 4);
  }
  // cache slot of the token (k and v heads) and its rotation row
  __nv_bfloat16* kdst = nullptr;
  __nv_bfloat16* vdst = nullptr;
  if (p.slot_mapping && h0 + nh > kv0) {
    const int64_t slot = p.slot_mapping[t];
    if (slot >= 0) {
      const int64_t blk = slot / p.block_size, off = slot % p.block_size;
      kdst = p.kv_cache + ((blk * 2 + 0) * p.block_size + off) * (int64_t)p.Hkv * 128;
      vdst = p.kv_cache + ((blk * 2 + 1) * p.block_size + off) * (int64_t)p.Hkv * 128;
    }
  }
  float c[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
  if (h0 < v0) {
    const float* cs = p.cos_sin + (size_t)p.positions[t] * 128;
    const int j = (lane & 15) * 4;
    const float4 c4 = *reinterpret_cast<const float4*>(cs + j);
    const float4 s4 = *reinterpret_cast<const float4*>(cs + 64 + j);
    c[0] = c4.x; c[1] = c4.y; c[2] = c4.z; c[3] = c4.w;
    sn[0] = s4.x; sn[1] = s4.y; sn[2] = s4.z; sn[3] = s4.w;
  }
  const float g = p.gemma ? 1.f : 0.f;
#pragma unroll
  for (int i = 0; i < kHG; ++i) {
    if (i >= nh) break;
    const int h = h0 + i;
    if (h >= v0) {                       // v head: straight copy into the cache
      if (vdst) *reinterpret_cast<uint2*>(vdst + (h - v0) * 128 + lane * 4) = raw[i];
      continue;
    }
    const bool is_q = h < kv0;
    const __nv_bfloat16* nw = is_q ? p.q_norm_w : p.k_norm_w;
    const float2 lo = unpack_bf16x2(raw[i].x), hi = unpack_bf16x2(raw[i].y);
    float x[4] = {lo.x, lo.y, hi.x, hi.y};
    if (nw) {
      float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float inv = rsqrtf(ss / 128.f + p.eps);
      const uint2 wr = *reinterpret_cast<const uint2*>(nw + lane * 4);
      const float2 w0 = unpack_bf16x2(wr.x), w1 = unpack_bf16x2(wr.y);
      const float w[4] = {w0.x, w0.y, w1.x, w1.y};
#pragma unroll
      for (int k = 0; k < 4; ++k)
        x[k] = __bfloat162float(__float2bfloat16(x[k] * inv * (w[k] + g)));   // norm output is bf16
    }
    float y[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float other = __shfl_xor_sync(0xffffffffu, x[k], 16);
      y[k] = lane < 16 ? x[k] * c[k] - other * sn[k] : x[k] * c[k] + other * sn[k];
    }
    uint2 o;
    o.x = pack_bf16x2(y[0], y[1]);
    o.y = pack_bf16x2(y[2], y[3]);
    if (is_q) {
      __nv_bfloat16* dst = p.q_out ? p.q_out + ((size_t)t * p.Hq + h) * 128 : const_cast<__nv_bfloat16*>(src[i]);
      *reinterpret_cast<uint2*>(dst + lane * 4) = o;
    } else {
      if (kdst) *reinterpret_cast<uint2*>(kdst + (h - kv0) * 128 + lane * 4) = o;
      // the activation row keeps the rotated k too
      *reinterpret_cast<uint2*>(const_cast<__nv_bfloat16*>(src[i]) + lane * 4) = o;
    }
  }
}

// Plain K/V scatter into the paged cache. k, v: [T, Hkv, D] with row strides ldk / ldv.
__global__ void __launch_bounds__(128)
    reshape_and_cache_kernel(const __nv_bfloat16* __restrict__ k, int ldk,
                             const __nv_bfloat16* __restrict__ v, int ldv,
                             const int64_t* __restrict__ slots, __nv_bfloat16* cache,
                             int block_size, int Hkv, int D) {
  const int t = blockIdx.x;
  const int64_t slot = slots[t];
  if (slot < 0) return;
  const int64_t blk = slot / block_size, off = slot % block_size;
  const int nv = (Hkv * D) >> 3;
  uint4* kd = reinterpret_cast<uint4*>(cache + ((blk * 2 + 0) * block_size + off) * (int64_t)Hkv * D);
  uint4* vd = reinterpret_cast<uint4*>(cache + ((blk * 2 + 1) * block_size + off) * (int64_t)Hkv * D);
  const uint4* ks = reinterpret_cast<const uint4*>(k + (size_t)t * ldk);
  const uint4* vs = reinterpret_cast<const uint4*>(v + (size_t)t * ldv);
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    kd[i] = ks[i];
    vd[i] = vs[i];
  }
}

// MLA latent cache write: cache[slot, :] = [kv_c (Lc) | k_pe (Lr)]; cache is
// [num_blocks, block_size, Lc + Lr].
__global__ void __launch_bounds__(128)
    concat_and_cache_mla_kernel(const __nv_bfloat16* __restrict__ kv_c, int ldc,
                                const __nv_bfloat16* __restrict__ k_pe, int ldr,
                                const int64_t* __restrict__ slots, __nv_bfloat16* cache, int Lc,
                                int Lr) {
  const int t = blockIdx.x;
  const int64_t slot = slots[t];
  if (slot < 0) return;
  __nv_bfloat16* dst = cache + slot * (int64_t)(Lc + Lr);
  for (int i = threadIdx.x; i < Lc; i += blockDim.x) dst[i] = kv_c[(size_t)t * ldc + i];
  for (int i = threadIdx.x; i < Lr; i += blockDim.x) dst[Lc + i] = k_pe[(size_t)t * ldr + i];
}

// Rotary table: out[pos, :] = [cos(pos * inv_freq[j]) * mscale | sin(...) * mscale], fp64 phase.
__global__ void rope_table_kernel(const double* __restrict__ inv_freq, float* out, int max_pos,
                                  int half, float mscale) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)max_pos * half) return;
  const int pos = (int)(idx / half), j = (int)(idx % half);
  const double ph = (double)pos * inv_freq[j];
  out[(size_t)pos * 2 * half + j] = (float)(cos(ph)) * mscale;
  out[(size_t)pos * 2 * half + half + j] = (float)(sin(ph)) * mscale;
}

}  // namespace b200

using namespace b200;
typedef __nv_bfloat16 bf16;

extern "C" {

int b200_rope_kv(void* qkv, int ld, int q_off, int k_off, int v_off, int q_head_stride, int Hq,
                 int Hkv, int D, int rot, const void* positions, const void* cos_sin,
                 const void* q_norm_w, const void* k_norm_w, float eps, int gemma, int neox,
                 const void* slot_mapping, void* kv_cache, int block_size, void* q_out, int T,
                 cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D > 256 || (D & 7) || rot > D || (rot & 1)) return -1;
  RopeKvParams p;
  p.qkv = (bf16*)qkv; p.ld = ld; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off;
  p.q_head_stride = q_head_stride; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.rot = rot;
  p.positions = (const int64_t*)positions; p.cos_sin = (const float*)cos_sin;
  p.q_norm_w = (const bf16*)q_norm_w; p.k_norm_w = (const bf16*)k_norm_w;
  p.eps = eps; p.gemma = gemma; p.neox = neox;
  p.slot_mapping = (const int64_t*)slot_mapping; p.kv_cache = (bf16*)kv_cache;
  p.block_size = block_size; p.q_out = (bf16*)q_out;
  const uintptr_t ptr_bits = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_out) |
                             reinterpret_cast<uintptr_t>(kv_cache) | reinterpret_cast<uintptr_t>(q_norm_w) |
                             reinterpret_cast<uintptr_t>(k_norm_w);
  p.vec4 = (D == 128 && rot == 128 && neox && cos_sin && !((ld | q_off | k_off | v_off | q_head_stride) & 3) &&
            !(ptr_bits & 7) && !(reinterpret_cast<uintptr_t>(cos_sin) & 15)) ? 1 : 0;
  long long warps = (long long)T * (Hq + 2 * Hkv);
  int blocks = (int)((warps + 3) / 4);
  if (p.vec4) {
    const int groups = (Hq + 2 * Hkv + kHG - 1) / kHG;
    const long long w4 = (long long)T * groups;
    return launch_pdl(rope_kv_vec4_kernel, dim3((unsigned)((w4 + 3) / 4)), dim3(128), 0, stream, p, T) == cudaSuccess
               ? 0 : -2;
  }
  return launch_pdl(rope_kv_kernel, dim3(blocks), dim3(128), 0, stream, p, T) == cudaSuccess ? 0 : -2;
}

int b200_reshape_and_cache(const void* k, int ldk, const void* v, int ldv, const void* slots,
                           void* cache, int block_size, int Hkv, int D, int T,
                           cudaStream_t stream) {
  if (T <= 0) return 0;
  if (((Hkv * D) & 7) || (ldk & 7) || (ldv & 7)) return -1;
  reshape_and_cache_kernel<<<T, 128, 0, stream>>>((const bf16*)k, ldk, (const bf16*)v, ldv,
                                                  (const int64_t*)slots, (bf16*)cache, block_size,
                                                  Hkv, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_concat_and_cache_mla(const void* kv_c, int ldc, const void* k_pe, int ldr,
                              const void* slots, void* cache, int Lc, int Lr, int T,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  concat_and_cache_mla_kernel<<<T, 128, 0, stream>>>((const bf16*)kv_c, ldc, (const bf16*)k_pe,
                                                     ldr, (const int64_t*)slots, (bf16*)cache, Lc,
                                                     Lr);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_rope_table(const void* inv_freq_f64, void* out_f32, int max_pos, int half, float mscale,
                    cudaStream_t stream) {
  long long n = (long long)max_pos * half;
  if (n <= 0) return 0;
  rope_table_kernel<<<(int)((n + 255) / 256), 256, 0, stream>>>((const double*)inv_freq_f64,
                                                                (float*)out_f32, max_pos, half,
                                                                mscale);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
