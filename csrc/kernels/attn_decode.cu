// Paged attention decode (one query token per sequence), GQA-packed, split-KV with a
// deterministic (fixed ascending order) merge. HBM-bound: every K/V byte is read once per
// kv head and shared by the query heads of its group.
//
// Work split: grid (seq, kv head * head-group, kv split). A CTA has 4 warps; each 8-lane
// group owns one token at a time and 16-byte slices of its K and V rows, so a dot product
// needs 3 shuffles and the loads of a warp cover whole 128-byte lines. Up to 4 query heads
// are kept in registers per thread (template HG); larger groups use more CTAs.
//
// Replaces src/vt/cuda/cuda_paged_attn.cu:184 (PagedAttentionKernel), :302
// (PagedAttentionDecodeOptKernel), :430 (PagedAttentionDecodeGqaKernel) and the FA2
// split-KV decode launcher.
#include "api.h"
#include "sm100.cuh"

namespace b200 {

struct DecodeParams {
  const __nv_bfloat16* q;  // [B, Hq*D] row stride ldq
  int ldq;
  __nv_bfloat16* out;      // [B, Hq*D] row stride ldo
  int ldo;
  const __nv_bfloat16* kv_cache;
  const int32_t* block_table;
  int max_blocks;
  const int32_t* seq_lens;
  int Hq, Hkv, block_size;
  float scale, softcap;
  int window;
  int splits;
  float* tmp_o;    // [B, Hq, splits, D]
  float* tmp_lse;  // [B, Hq, splits]  (log2 domain: m + log2(l))
};

template <int D, int HG>
__global__ void __launch_bounds__(128)
    attn_decode_kernel(DecodeParams p) {
  constexpr int NC = D / 64;        // 16-byte chunks per lane for one row (8 lanes per row)
  constexpr int EL = NC * 8;        // elements per lane
  const int b = blockIdx.x;
  const int G = p.Hq / p.Hkv;
  const int groups_per_kv = (G + HG - 1) / HG;
  const int hkv = blockIdx.y / groups_per_kv;
  const int hg0 = (blockIdx.y % groups_per_kv) * HG;   // first q head (within group) of this CTA
  const int nh = min(HG, G - hg0);
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane >> 3, l8 = lane & 7;            // token slot in warp, lane in row

  const int seq_len = p.seq_lens[b];
  int begin = 0;
  if (p.window > 0) begin = max(0, seq_len - p.window);
  else if (p.window < 0) begin = ((seq_len - 1) / -p.window) * -p.window;   // chunked-local: the query's own chunk
  const int span = seq_len - begin;
  int chunk = (span + p.splits - 1) / p.splits;
  chunk = ((chunk + 15) / 16) * 16;
  const int t0 = begin + split * chunk;
  const int t1 = min(seq_len, t0 + chunk);

  // q (scaled) in registers
  float q[HG][EL];
  const float sc = p.scale * 1.4426950408889634f;
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) {
    const int hq = hkv * G + hg0 + min(hh, nh - 1);
    const __nv_bfloat16* qp = p.q + (size_t)b * p.ldq + (size_t)hq * D;
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const uint4 v = *reinterpret_cast<const uint4*>(qp + (c * 8 + l8) * 8);
      float2 f;
      f = unpack_bf16x2(v.x); q[hh][c * 8 + 0] = f.x * sc; q[hh][c * 8 + 1] = f.y * sc;
      f = unpack_bf16x2(v.y); q[hh][c * 8 + 2] = f.x * sc; q[hh][c * 8 + 3] = f.y * sc;
      f = unpack_bf16x2(v.z); q[hh][c * 8 + 4] = f.x * sc; q[hh][c * 8 + 5] = f.y * sc;
      f = unpack_bf16x2(v.w); q[hh][c * 8 + 6] = f.x * sc; q[hh][c * 8 + 7] = f.y * sc;
    }
  }
  float m[HG], l[HG], o[HG][EL];
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) {
    m[hh] = -INFINITY;
    l[hh] = 0.f;
#pragma unroll
    for (int e = 0; e < EL; ++e) o[hh][e] = 0.f;
  }

  const int32_t* bt = p.block_table + (size_t)b * p.max_blocks;
  const size_t tok_stride = (size_t)p.Hkv * D;
  const float cap2 = p.softcap * 1.4426950408889634f;  // softcap in the log2 domain

  // 16 tokens per CTA iteration: warp w, slot `sub` -> token t0 + it*16 + w*4 + sub
  for (int base = t0; base < t1; base += 16) {
    const int tok = base + warp * 4 + sub;
    const bool valid = tok < t1;
    uint4 kreg[NC], vreg[NC];
    if (valid) {
      const int blk = bt[tok / p.block_size];
      const int off = tok % p.block_size;
      const __nv_bfloat16* kp =
          p.kv_cache + ((size_t)(blk * 2 + 0) * p.block_size + off) * tok_stride + (size_t)hkv * D;
      const __nv_bfloat16* vp = kp + (size_t)p.block_size * tok_stride;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        kreg[c] = __ldg(reinterpret_cast<const uint4*>(kp + (c * 8 + l8) * 8));
        vreg[c] = __ldg(reinterpret_cast<const uint4*>(vp + (c * 8 + l8) * 8));
      }
    } else {
#pragma unroll
      for (int c = 0; c < NC; ++c) kreg[c] = vreg[c] = make_uint4(0, 0, 0, 0);
    }
    float kf[EL];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      float2 f;
      f = unpack_bf16x2(kreg[c].x); kf[c * 8 + 0] = f.x; kf[c * 8 + 1] = f.y;
      f = unpack_bf16x2(kreg[c].y); kf[c * 8 + 2] = f.x; kf[c * 8 + 3] = f.y;
      f = unpack_bf16x2(kreg[c].z); kf[c * 8 + 4] = f.x; kf[c * 8 + 5] = f.y;
      f = unpack_bf16x2(kreg[c].w); kf[c * 8 + 6] = f.x; kf[c * 8 + 7] = f.y;
    }
    float s[HG];
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) {
      float a = 0.f;
#pragma unroll
      for (int e = 0; e < EL; ++e) a += q[hh][e] * kf[e];
      a += __shfl_xor_sync(0xffffffffu, a, 1);
      a += __shfl_xor_sync(0xffffffffu, a, 2);
      a += __shfl_xor_sync(0xffffffffu, a, 4);
      if (p.softcap > 0.f) a = cap2 * tanhf(a / cap2);
      s[hh] = valid ? a : -INFINITY;
    }
    float vf[EL];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      float2 f;
      f = unpack_bf16x2(vreg[c].x); vf[c * 8 + 0] = f.x; vf[c * 8 + 1] = f.y;
      f = unpack_bf16x2(vreg[c].y); vf[c * 8 + 2] = f.x; vf[c * 8 + 3] = f.y;
      f = unpack_bf16x2(vreg[c].z); vf[c * 8 + 4] = f.x; vf[c * 8 + 5] = f.y;
      f = unpack_bf16x2(vreg[c].w); vf[c * 8 + 6] = f.x; vf[c * 8 + 7] = f.y;
    }
#pragma unroll
    for (int hh = 0; hh < HG; ++hh) {
      if (s[hh] > m[hh]) {
        const float a = exp2f(m[hh] - s[hh]);  // m = -inf -> 0
        l[hh] *= a;
#pragma unroll
        for (int e = 0; e < EL; ++e) o[hh][e] *= a;
        m[hh] = s[hh];
      }
      const float pr = (s[hh] == -INFINITY) ? 0.f : exp2f(s[hh] - m[hh]);
      l[hh] += pr;
#pragma unroll
      for (int e = 0; e < EL; ++e) o[hh][e] += pr * vf[e];
    }
  }

  // ---- merge the 4 token slots of a warp, then the 4 warps ----
  __shared__ float sm_m[4][HG], sm_l[4][HG];
  __shared__ float sm_o[4][HG][D];
#pragma unroll
  for (int hh = 0; hh < HG; ++hh) {
#pragma unroll
    for (int xo = 8; xo <= 16; xo <<= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m[hh], xo);
      const float l2 = __shfl_xor_sync(0xffffffffu, l[hh], xo);
      const float mn = fmaxf(m[hh], m2);
      const float a1 = (m[hh] == -INFINITY) ? 0.f : exp2f(m[hh] - mn);
      const float a2 = (m2 == -INFINITY) ? 0.f : exp2f(m2 - mn);
      l[hh] = l[hh] * a1 + l2 * a2;
#pragma unroll
      for (int e = 0; e < EL; ++e) {
        const float o2 = __shfl_xor_sync(0xffffffffu, o[hh][e], xo);
        o[hh][e] = o[hh][e] * a1 + o2 * a2;
      }
      m[hh] = mn;
    }
    if (sub == 0) {
      if (l8 == 0) { sm_m[warp][hh] = m[hh]; sm_l[warp][hh] = l[hh]; }
#pragma unroll
      for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int e = 0; e < 8; ++e) sm_o[warp][hh][(c * 8 + l8) * 8 + e] = o[hh][c * 8 + e];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < nh * D; idx += blockDim.x) {
    const int hh = idx / D, d = idx % D;
    float mn = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mn = fmaxf(mn, sm_m[w][hh]);
    float acc = 0.f, ls = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float a = (sm_m[w][hh] == -INFINITY) ? 0.f : exp2f(sm_m[w][hh] - mn);
      acc += sm_o[w][hh][d] * a;
      ls += sm_l[w][hh] * a;
    }
    const int hq = hkv * G + hg0 + hh;
    if (p.splits == 1) {
      p.out[(size_t)b * p.ldo + (size_t)hq * D + d] = __float2bfloat16(ls > 0.f ? acc / ls : 0.f);
    } else {
      const size_t row = ((size_t)b * p.Hq + hq) * p.splits + split;
      p.tmp_o[row * D + d] = ls > 0.f ? acc / ls : 0.f;
      if (d == 0) p.tmp_lse[row] = ls > 0.f ? mn + log2f(ls) : -INFINITY;
    }
  }
}

// Fixed-order merge of split partials: out = sum_s w_s * o_s, w_s = 2^(lse_s - lse_max) / sum.
__global__ void __launch_bounds__(128)
    attn_decode_merge_kernel(const float* __restrict__ tmp_o, const float* __restrict__ tmp_lse,
                             __nv_bfloat16* out, int ldo, int Hq, int D, int splits) {
  const int b = blockIdx.x, h = blockIdx.y;
  const size_t row0 = ((size_t)b * Hq + h) * splits;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, tmp_lse[row0 + s]);
  float den = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float v = tmp_lse[row0 + s];
    den += (v == -INFINITY) ? 0.f : exp2f(v - mx);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float v = tmp_lse[row0 + s];
      const float w = (v == -INFINITY) ? 0.f : exp2f(v - mx);
      acc += w * tmp_o[(row0 + s) * D + d];
    }
    out[(size_t)b * ldo + (size_t)h * D + d] = __float2bfloat16(den > 0.f ? acc / den : 0.f);
  }
}

// Merge two partial attention results with their natural-log LSEs (used by chunked-context
// prefill and MLA). out may alias a.   Reference: cuda_mla_prefill.cu:312 MergeAttnStatesKernel.
__global__ void __launch_bounds__(128)
    merge_attn_states_kernel(const __nv_bfloat16* __restrict__ a, const float* __restrict__ lse_a,
                             const __nv_bfloat16* __restrict__ b, const float* __restrict__ lse_b,
                             __nv_bfloat16* out, float* lse_out, int H, int D) {
  const int t = blockIdx.x, h = blockIdx.y;
  const float la = lse_a[(size_t)t * H + h], lb = lse_b[(size_t)t * H + h];
  const float mx = fmaxf(la, lb);
  float wa, wb;
  if (mx == -INFINITY) { wa = 0.f; wb = 0.f; }
  else {
    const float ea = (la == -INFINITY) ? 0.f : __expf(la - mx);
    const float eb = (lb == -INFINITY) ? 0.f : __expf(lb - mx);
    wa = ea / (ea + eb);
    wb = eb / (ea + eb);
    if (lse_out && threadIdx.x == 0) lse_out[(size_t)t * H + h] = mx + __logf(ea + eb);
  }
  if (mx == -INFINITY && lse_out && threadIdx.x == 0) lse_out[(size_t)t * H + h] = -INFINITY;
  const size_t off = ((size_t)t * H + h) * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x)
    out[off + d] = __float2bfloat16(wa * __bfloat162float(a[off + d]) + wb * __bfloat162float(b[off + d]));
}

template <int D>
static int launch_decode(DecodeParams& p, int B, cudaStream_t stream) {
  const int G = p.Hq / p.Hkv;
  if (G <= 1) {
    dim3 grid(B, p.Hkv, p.splits);
    attn_decode_kernel<D, 1><<<grid, 128, 0, stream>>>(p);
  } else if (G == 2) {
    dim3 grid(B, p.Hkv, p.splits);
    attn_decode_kernel<D, 2><<<grid, 128, 0, stream>>>(p);
  } else {
    constexpr int HG = (D > 128) ? 2 : 4;
    dim3 grid(B, p.Hkv * ((G + HG - 1) / HG), p.splits);
    attn_decode_kernel<D, HG><<<grid, 128, 0, stream>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace b200

using namespace b200;

extern "C" {

// Suggested split count for a batch (the caller fixes it at graph-capture time).
int b200_attn_decode_splits(int B, int Hkv, int G, int D, int max_seq_len) {
  const int HG = (D > 128) ? 2 : 4;
  const int ctas = B * Hkv * ((G + HG - 1) / HG);
  const int target = b200_num_sms() * 4;
  int splits = (target + ctas - 1) / ctas;
  int max_by_len = (max_seq_len + 255) / 256;
  if (splits > max_by_len) splits = max_by_len;
  if (splits > 64) splits = 64;
  if (splits < 1) splits = 1;
  return splits;
}

int b200_attn_decode(const void* q, int ldq, void* out, int ldo, const void* kv_cache,
                     int block_size, int Hq, int Hkv, int D, const void* block_table,
                     int max_blocks, const void* seq_lens, int B, float scale, float softcap,
                     int window, int splits, void* tmp_o, void* tmp_lse, cudaStream_t stream) {
  if (B <= 0) return 0;
  if ((D != 64 && D != 128 && D != 256) || Hq % Hkv || (ldq & 7)) return -1;
  if (splits < 1) splits = 1;
  if (splits > 1 && (!tmp_o || !tmp_lse)) return -1;
  DecodeParams p;
  p.q = (const __nv_bfloat16*)q; p.ldq = ldq; p.out = (__nv_bfloat16*)out; p.ldo = ldo;
  p.kv_cache = (const __nv_bfloat16*)kv_cache; p.block_table = (const int32_t*)block_table;
  p.max_blocks = max_blocks; p.seq_lens = (const int32_t*)seq_lens;
  p.Hq = Hq; p.Hkv = Hkv; p.block_size = block_size; p.scale = scale; p.softcap = softcap;
  p.window = window; p.splits = splits; p.tmp_o = (float*)tmp_o; p.tmp_lse = (float*)tmp_lse;
  int rc;
  if (D == 64) rc = launch_decode<64>(p, B, stream);
  else if (D == 128) rc = launch_decode<128>(p, B, stream);
  else rc = launch_decode<256>(p, B, stream);
  if (rc) return rc;
  if (splits > 1) {
    dim3 grid(B, Hq);
    attn_decode_merge_kernel<<<grid, 128, 0, stream>>>(p.tmp_o, p.tmp_lse, p.out, ldo, Hq, D,
                                                       splits);
    if (cudaGetLastError() != cudaSuccess) return -2;
  }
  return 0;
}

int b200_attn_decode_merge(const void* tmp_o, const void* tmp_lse, void* out, int ldo, int B,
                           int Hq, int D, int splits, cudaStream_t stream) {
  dim3 grid(B, Hq);
  attn_decode_merge_kernel<<<grid, 128, 0, stream>>>((const float*)tmp_o, (const float*)tmp_lse,
                                                     (__nv_bfloat16*)out, ldo, Hq, D, splits);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_merge_attn_states(const void* a, const void* lse_a, const void* b, const void* lse_b,
                           void* out, void* lse_out, int T, int H, int D, cudaStream_t stream) {
  if (T <= 0) return 0;
  dim3 grid(T, H);
  merge_attn_states_kernel<<<grid, 128, 0, stream>>>(
      (const __nv_bfloat16*)a, (const float*)lse_a, (const __nv_bfloat16*)b, (const float*)lse_b,
      (__nv_bfloat16*)out, (float*)lse_out, H, D);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
