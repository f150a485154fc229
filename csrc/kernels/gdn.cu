// Gated DeltaNet support kernels (HBM-bound, CUDA cores, fp32 math):
//
//   causal depthwise conv1d (K = 4, SiLU) over variable-length sequences with a per-request
//   state of the last three raw inputs, and its single-token update for decode
//       reference: src/vt/cuda/cuda_gdn.cu:328 (CausalConv1dFwdKernel), :709 (Update)
//   post-conv preparation: q/k L2 norm per head, g = -exp(A_log) * softplus(a + dt_bias),
//   beta = sigmoid(b)                                         cuda_gdn.cu:974 (GdnPostConvKernel)
//   packed recurrent decode: one token per request straight from the conv output, state
//   [slots, Hv, Dv, Dk] fp32 updated in place                 cuda_gdn.cu:1778 (GdnPackedDecodeKernel)
//   gated RMSNorm: rmsnorm(x) * w * silu(z)                   cuda_gdn.cu:1315 (RmsNormGatedRowKernel)
//
// The chunked prefill scan lives in gdn_scan.cu.
#include "api.h"
#include "sm100.cuh"

namespace b200 {

typedef __nv_bfloat16 bf16;
static constexpr int kConvK = 4;

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

// ------------------------------------------------------------------------------------
// conv1d forward. Grid (C / 128, ceil(T / kConvTokens)); a thread owns one channel and walks
// the tokens of its block in order, so the three previous inputs stay in registers.
// ------------------------------------------------------------------------------------
static constexpr int kConvTokens = 32;

__global__ void __launch_bounds__(128)
    gdn_conv1d_fwd_kernel(const bf16* __restrict__ x, long ldx, const bf16* __restrict__ w,
                          const bf16* __restrict__ state, const int* __restrict__ qsl,
                          const int* __restrict__ slots, const int* __restrict__ has_init,
                          bf16* __restrict__ out, long ldo, int n_seq, int T, int C) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int t0 = blockIdx.y * kConvTokens;
  if (c >= C || t0 >= T) return;
  const int t1 = min(T, t0 + kConvTokens);
  // sequence of the first token: last s with qsl[s] <= t0
  int lo = 0, hi = n_seq - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (qsl[mid] <= t0) lo = mid; else hi = mid - 1;
  }
  int s = lo;
  const uint2 wv = *reinterpret_cast<const uint2*>(w + (size_t)c * kConvK);
  const float2 w01 = unpack_bf16x2(wv.x), w23 = unpack_bf16x2(wv.y);
  float p1 = 0.f, p2 = 0.f, p3 = 0.f;   // x[t-1], x[t-2], x[t-3]
  int seq_begin = qsl[s], seq_end = qsl[s + 1];
  auto load_window = [&](int t) {
    // previous inputs of token t (first token handled by this thread in sequence s)
    const int pos = t - seq_begin;
    const bool init = has_init ? has_init[s] != 0 : true;
    const int slot = slots[s];
    const bf16* st = state + ((size_t)slot * C + c) * (kConvK - 1);   // [oldest, mid, newest]
    auto prev = [&](int back) -> float {   // input `back` positions before t
      if (pos - back >= 0) return __bfloat162float(x[(size_t)(t - back) * ldx + c]);
      if (!init || slot < 0) return 0.f;
      return __bfloat162float(st[(kConvK - 1) + (pos - back)]);   // pos-back in [-3,-1]
    };
    p1 = prev(1); p2 = prev(2); p3 = prev(3);
  };
  load_window(t0);
  for (int t = t0; t < t1; ++t) {
    while (t >= seq_end && s + 1 < n_seq) {
      ++s;
      seq_begin = qsl[s];
      seq_end = qsl[s + 1];
      if (t < seq_end) load_window(t);
    }
    if (t >= seq_end) break;    // padding rows after the last sequence
    const float xv = __bfloat162float(x[(size_t)t * ldx + c]);
    const float acc = w01.x * p3 + w01.y * p2 + w23.x * p1 + w23.y * xv;
    out[(size_t)t * ldo + c] = __float2bfloat16(silu_f(acc));
    p3 = p2; p2 = p1; p1 = xv;
  }
}

// New state of every sequence = its last three raw inputs (older ones come from the old
// state when the sequence chunk is shorter than three tokens). Runs after the forward pass.
__global__ void __launch_bounds__(128)
    gdn_conv1d_state_kernel(const bf16* __restrict__ x, long ldx, bf16* __restrict__ state,
                            const int* __restrict__ qsl, const int* __restrict__ slots,
                            const int* __restrict__ has_init, int C) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int s = blockIdx.y;
  if (c >= C) return;
  const int slot = slots[s];
  if (slot < 0) return;
  const int b = qsl[s], e = qsl[s + 1], len = e - b;
  if (len <= 0) return;
  const bool init = has_init ? has_init[s] != 0 : true;
  bf16* st = state + ((size_t)slot * C + c) * (kConvK - 1);
  float old[kConvK - 1];
#pragma unroll
  for (int i = 0; i < kConvK - 1; ++i) old[i] = init ? __bfloat162float(st[i]) : 0.f;
  float nw[kConvK - 1];
#pragma unroll
  for (int i = 0; i < kConvK - 1; ++i) {
    // element i of the new window is the input at position len - 3 + i
    const int pos = len - (kConvK - 1) + i;
    nw[i] = pos >= 0 ? __bfloat162float(x[(size_t)(b + pos) * ldx + c]) : old[(kConvK - 1) + pos];
  }
#pragma unroll
  for (int i = 0; i < kConvK - 1; ++i) st[i] = __float2bfloat16(nw[i]);
}

// Decode step: one token per request.
__global__ void __launch_bounds__(128)
    gdn_conv1d_update_kernel(const bf16* __restrict__ x, long ldx, const bf16* __restrict__ w,
                             bf16* __restrict__ state, const int* __restrict__ slots,
                             bf16* __restrict__ out, long ldo, int C) {
  const int c = blockIdx.x * 128 + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C) return;
  const int slot = slots[b];
  if (slot < 0) return;
  bf16* st = state + ((size_t)slot * C + c) * (kConvK - 1);
  const float s0 = __bfloat162float(st[0]), s1 = __bfloat162float(st[1]), s2 = __bfloat162float(st[2]);
  const bf16 xb = x[(size_t)b * ldx + c];
  const float xv = __bfloat162float(xb);
  const uint2 wv = *reinterpret_cast<const uint2*>(w + (size_t)c * kConvK);
  const float2 w01 = unpack_bf16x2(wv.x), w23 = unpack_bf16x2(wv.y);
  const float acc = w01.x * s0 + w01.y * s1 + w23.x * s2 + w23.y * xv;
  out[(size_t)b * ldo + c] = __float2bfloat16(silu_f(acc));
  st[0] = st[1];
  st[1] = st[2];
  st[2] = xb;
}

// ------------------------------------------------------------------------------------
// post-conv: one warp per (token, head) for the q/k L2 norm (D = 128: 4 values per lane),
// plus g / beta for the value heads.
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
    gdn_post_conv_kernel(const bf16* __restrict__ xc, long ld, int T, int Hk, int Hv,
                         const bf16* __restrict__ a, const bf16* __restrict__ b, long ldab,
                         const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                         bf16* __restrict__ q_out, bf16* __restrict__ k_out,
                         float* __restrict__ g, float* __restrict__ beta, float eps) {
  constexpr int D = 128;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const int rows = 2 * Hk;   // q heads then k heads
  for (int r = warp; r < rows; r += 4) {
    const bf16* src = xc + (size_t)t * ld + (size_t)r * D + lane * 4;
    const uint2 v = *reinterpret_cast<const uint2*>(src);
    const float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y);
    float ss = f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss + eps);
    uint2 o;
    o.x = pack_bf16x2(f0.x * inv, f0.y * inv);
    o.y = pack_bf16x2(f1.x * inv, f1.y * inv);
    bf16* dst = (r < Hk ? q_out + ((size_t)t * Hk + r) * D : k_out + ((size_t)t * Hk + (r - Hk)) * D) + lane * 4;
    *reinterpret_cast<uint2*>(dst) = o;
  }
  for (int h = threadIdx.x; h < Hv; h += blockDim.x) {
    const float av = __bfloat162float(a[(size_t)t * ldab + h]);
    const float bv = __bfloat162float(b[(size_t)t * ldab + h]);
    g[(size_t)t * Hv + h] = -__expf(A_log[h]) * softplus_f(av + dt_bias[h]);
    beta[(size_t)t * Hv + h] = sigmoid_f(bv);
  }
}

// ------------------------------------------------------------------------------------
// packed decode. Grid (Dv / 32, B * Hv), 128 threads: a warp owns 8 state rows, 8 lanes per
// row (16 contiguous floats each), 4 rows in flight per pass.
//   S <- S * e^g ; kv = S k ; v' = (v - kv) * beta ; S <- S + v' (x) k ; o = S q * Dk^-0.5
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
    gdn_packed_decode_kernel(const bf16* __restrict__ xc, long ld, const bf16* __restrict__ a,
                             const bf16* __restrict__ b, long ldab, const float* __restrict__ A_log,
                             const float* __restrict__ dt_bias, float* __restrict__ state,
                             const int* __restrict__ slots, bf16* __restrict__ out, int Hk, int Hv,
                             float eps) {
  constexpr int D = 128;
  __shared__ float qs[D], ks[D];
  __shared__ float red[8];
  const int bh = blockIdx.y;
  const int bi = bh / Hv, hv = bh % Hv;
  const int slot = slots[bi];
  if (slot < 0) return;
  const int hk = hv / (Hv / Hk);
  const bf16* row = xc + (size_t)bi * ld;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // q and k of this head: L2 norm in fp32 (threads 0..127 load one element each)
  {
    const float qv = __bfloat162float(row[(size_t)hk * D + tid]);
    const float kv = __bfloat162float(row[(size_t)(Hk + hk) * D + tid]);
    float sq = qv * qv, sk = kv * kv;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sq += __shfl_xor_sync(0xffffffffu, sq, o);
      sk += __shfl_xor_sync(0xffffffffu, sk, o);
    }
    if (lane == 0) { red[warp] = sq; red[4 + warp] = sk; }
    __syncthreads();
    const float tq = red[0] + red[1] + red[2] + red[3];
    const float tk = red[4] + red[5] + red[6] + red[7];
    // the normalised vectors pass through bf16 like the unfused path's q/k tensors
    qs[tid] = __bfloat162float(__float2bfloat16(qv * rsqrtf(tq + eps))) * 0.08838834764831845f;
    ks[tid] = __bfloat162float(__float2bfloat16(kv * rsqrtf(tk + eps)));
    __syncthreads();
  }
  const float av = __bfloat162float(a[(size_t)bi * ldab + hv]);
  const float bv = __bfloat162float(b[(size_t)bi * ldab + hv]);
  const float decay = __expf(-__expf(A_log[hv]) * softplus_f(av + dt_bias[hv]));
  const float be = __bfloat162float(__float2bfloat16(sigmoid_f(bv)));
  const int sub = lane >> 3;       // row within the group of 4
  const int seg = lane & 7;        // 16-float segment of the row
  float kr[16], qr[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) { kr[i] = ks[seg * 16 + i]; qr[i] = qs[seg * 16 + i]; }
  float* S = state + (((size_t)slot * Hv + hv) * D) * D;
  const bf16* vrow = row + (size_t)2 * Hk * D + (size_t)hv * D;
  bf16* orow = out + ((size_t)bi * Hv + hv) * D;
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int dv = blockIdx.x * 32 + warp * 8 + pass * 4 + sub;
    float4* sp = reinterpret_cast<float4*>(S + (size_t)dv * D + seg * 16);
    float4 s4[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) s4[i] = sp[i];
    float* sv = reinterpret_cast<float*>(s4);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) { sv[i] *= decay; dot += sv[i] * kr[i]; }
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
    dot += __shfl_xor_sync(0xffffffffu, dot, 4);
    const float vn = (__bfloat162float(vrow[dv]) - dot) * be;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) { sv[i] += vn * kr[i]; o += sv[i] * qr[i]; }
    o += __shfl_xor_sync(0xffffffffu, o, 1);
    o += __shfl_xor_sync(0xffffffffu, o, 2);
    o += __shfl_xor_sync(0xffffffffu, o, 4);
#pragma unroll
    for (int i = 0; i < 4; ++i) sp[i] = s4[i];
    if (seg == 0) orow[dv] = __float2bfloat16(o);
  }
}

// ------------------------------------------------------------------------------------
// gated RMSNorm over rows of D (<= 1024, multiple of 4): one warp per row. Row r is head
// r % heads of token r / heads; ldx / ldz / ldo are token strides, heads sit D apart.
// gate_kind 0: silu(z), 1: sigmoid(z).
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
    rmsnorm_gated_kernel(const bf16* __restrict__ x, long ldx, const bf16* __restrict__ z, long ldz,
                         const bf16* __restrict__ w, bf16* __restrict__ out, long ldo, long R, int D,
                         float eps, int gate_kind, int heads) {
  const long r = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= R) return;
  const long tok = r / heads;
  const long hoff = (r % heads) * (long)D;
  const bf16* xr = x + tok * ldx + hoff;
  const bf16* zr = z + tok * ldz + hoff;
  bf16* orow = out + tok * ldo + hoff;
  float ss = 0.f;
  for (int i = lane * 4; i < D; i += 128) {
    const uint2 v = *reinterpret_cast<const uint2*>(xr + i);
    const float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y);
    ss += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = rsqrtf(ss / (float)D + eps);
  for (int i = lane * 4; i < D; i += 128) {
    const uint2 v = *reinterpret_cast<const uint2*>(xr + i);
    const uint2 zv = *reinterpret_cast<const uint2*>(zr + i);
    const uint2 wv = *reinterpret_cast<const uint2*>(w + i);
    const float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y);
    const float2 z0 = unpack_bf16x2(zv.x), z1 = unpack_bf16x2(zv.y);
    const float2 w0 = unpack_bf16x2(wv.x), w1 = unpack_bf16x2(wv.y);
    auto gate = [&](float t) { return gate_kind == 0 ? silu_f(t) : sigmoid_f(t); };
    uint2 o;
    o.x = pack_bf16x2(f0.x * inv * w0.x * gate(z0.x), f0.y * inv * w0.y * gate(z0.y));
    o.y = pack_bf16x2(f1.x * inv * w1.x * gate(z1.x), f1.y * inv * w1.y * gate(z1.y));
    *reinterpret_cast<uint2*>(orow + i) = o;
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_gdn_conv1d_fwd(const void* x, long ldx, const void* w, void* conv_state, const int* qsl,
                        const int* slots, const int* has_init, void* out, long ldo, int n_seq,
                        int total_tokens, int C, cudaStream_t stream) {
  if (n_seq <= 0 || total_tokens <= 0) return 0;
  if (x == out || (C & 3)) return -1;
  dim3 grid((C + 127) / 128, (total_tokens + kConvTokens - 1) / kConvTokens);
  gdn_conv1d_fwd_kernel<<<grid, 128, 0, stream>>>((const bf16*)x, ldx, (const bf16*)w,
                                                  (const bf16*)conv_state, qsl, slots, has_init,
                                                  (bf16*)out, ldo, n_seq, total_tokens, C);
  if (cudaGetLastError() != cudaSuccess) return -2;
  dim3 g2((C + 127) / 128, n_seq);
  gdn_conv1d_state_kernel<<<g2, 128, 0, stream>>>((const bf16*)x, ldx, (bf16*)conv_state, qsl, slots,
                                                  has_init, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_gdn_conv1d_update(const void* x, long ldx, const void* w, void* conv_state, const int* slots,
                           void* out, long ldo, int B, int C, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (C & 3) return -1;
  dim3 grid((C + 127) / 128, B);
  gdn_conv1d_update_kernel<<<grid, 128, 0, stream>>>((const bf16*)x, ldx, (const bf16*)w,
                                                     (bf16*)conv_state, slots, (bf16*)out, ldo, C);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_gdn_post_conv(const void* xc, long ld, int T, int Hk, int Hv, int Dk, const void* a,
                       const void* b, long ldab, const float* A_log, const float* dt_bias,
                       void* q_out, void* k_out, float* g, float* beta, float eps,
                       cudaStream_t stream) {
  if (T <= 0) return 0;
  if (Dk != 128 || (ld & 3)) return -1;
  gdn_post_conv_kernel<<<T, 128, 0, stream>>>((const bf16*)xc, ld, T, Hk, Hv, (const bf16*)a,
                                              (const bf16*)b, ldab, A_log, dt_bias, (bf16*)q_out,
                                              (bf16*)k_out, g, beta, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_gdn_packed_decode(const void* xc, long ld, const void* a, const void* b, long ldab,
                           const float* A_log, const float* dt_bias, float* state, const int* slots,
                           void* out, int B, int Hk, int Hv, int Dk, int Dv, float eps,
                           cudaStream_t stream) {
  if (B <= 0) return 0;
  if (Dk != 128 || Dv != 128 || Hk <= 0 || Hv % Hk) return -1;
  dim3 grid(Dv / 32, B * Hv);
  gdn_packed_decode_kernel<<<grid, 128, 0, stream>>>((const bf16*)xc, ld, (const bf16*)a,
                                                     (const bf16*)b, ldab, A_log, dt_bias, state,
                                                     slots, (bf16*)out, Hk, Hv, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_rmsnorm_gated(const void* x, long ldx, const void* z, long ldz, const void* w, void* out,
                       long ldo, long R, int D, float eps, int gate_kind, int heads,
                       cudaStream_t stream) {
  if (R <= 0) return 0;
  if (heads < 1) heads = 1;
  if ((D & 3) || (ldx & 3) || (ldz & 3) || (ldo & 3)) return -1;
  rmsnorm_gated_kernel<<<(unsigned)((R + 3) / 4), 128, 0, stream>>>(
      (const bf16*)x, ldx, (const bf16*)z, ldz, (const bf16*)w, (bf16*)out, ldo, R, D, eps, gate_kind, heads);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
