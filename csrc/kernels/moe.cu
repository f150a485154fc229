// Mixture-of-experts kernels: router top-k, expert sort (device-side counts, no host sync),
// grouped expert GEMM on tcgen05, weighted combine (optionally scattered to the row owners
// of a tensor-parallel group, i.e. combine + reduce-scatter in one pass).
//
// Grouped GEMM form: for each expert the weight tile is the 128-row MMA operand and the
// tokens routed to that expert are the N operand (up to 256 per chunk), so small per-expert
// batches (decode) stream every expert weight exactly once and large ones (prefill) still
// run full 128 x 256 tiles. Work items (expert, token chunk) are listed on the device.
//
// Reference kernels replaced: src/vt/cuda/cuda_moe.cu:62 (MoeRouterTopKKernel), :197
// (MoeRouterGroupedTopKKernel), :406/:484 (MoeCombine[Gate]Kernel), :547 (MoeSiluMulKernel);
// cuda_matmul_nvfp4.cu:631-676 (hist / offsets / scatter / tile map), :923-1165 (bf16
// grouped GEMM naive / split-K / wmma variants).
#include <float.h>

#include <mutex>
#include <unordered_map>

#include "api.h"
#include "sm100.cuh"

namespace b200 {

// --------------------------------------------------------------------------- router top-k
// One block per token. scoring: 0 softmax, 1 sigmoid. Grouped selection (n_group > 1): the
// experts are split into n_group groups, a group's score is the sum of its two best
// (bias-corrected) scores, only the topk_group best groups stay eligible. Selection uses
// score + bias, the returned weight is the unbiased score. Ties break to the lowest index.
__global__ void __launch_bounds__(256)
    moe_router_topk_kernel(const float* __restrict__ logits, int ld, int E, int k, int renorm,
                           int scoring, const float* __restrict__ e_bias, int n_group,
                           int topk_group, float routed_scale, int32_t* topk_ids, float* topk_w) {
  extern __shared__ float sh[];   // E scores, E selection scores
  float* score = sh;
  float* sel = sh + E;
  __shared__ float red[32];
  __shared__ int redi[32];
  const int t = blockIdx.x;
  const float* x = logits + (size_t)t * ld;
  if (scoring == 0) {
    float mx = -FLT_MAX;
    for (int i = threadIdx.x; i < E; i += blockDim.x) mx = fmaxf(mx, x[i]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    mx = -FLT_MAX;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, red[w]);
    __syncthreads();
    float s = 0.f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
      const float e = expf(x[i] - mx);
      score[i] = e;
      s += e;
    }
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    s = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += red[w];
    const float inv = 1.f / s;
    for (int i = threadIdx.x; i < E; i += blockDim.x) score[i] *= inv;
  } else {
    for (int i = threadIdx.x; i < E; i += blockDim.x) score[i] = 1.f / (1.f + expf(-x[i]));
  }
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x) sel[i] = score[i] + (e_bias ? e_bias[i] : 0.f);
  __syncthreads();
  if (n_group > 1 && topk_group < n_group) {
    // thread g scores group g (n_group is small), thread 0 masks the losers
    __shared__ float gscore[64];
    const int per = E / n_group;
    if ((int)threadIdx.x < n_group) {
      float b0 = -FLT_MAX, b1 = -FLT_MAX;
      for (int i = 0; i < per; ++i) {
        const float v = sel[threadIdx.x * per + i];
        if (v > b0) { b1 = b0; b0 = v; } else if (v > b1) { b1 = v; }
      }
      gscore[threadIdx.x] = e_bias ? b0 + b1 : b0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int pick = 0; pick < n_group - topk_group; ++pick) {
        int worst = -1;
        float wv = FLT_MAX;
        for (int g = n_group - 1; g >= 0; --g)   // ties: drop the highest index first
          if (gscore[g] != FLT_MAX && gscore[g] < wv) { wv = gscore[g]; worst = g; }
        if (worst < 0) break;
        gscore[worst] = FLT_MAX;
        for (int i = 0; i < per; ++i) sel[worst * per + i] = -FLT_MAX;
      }
    }
    __syncthreads();
  }
  float wsum = 0.f;
  for (int j = 0; j < k; ++j) {
    float bv = -FLT_MAX;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < E; i += blockDim.x) {
      const float v = sel[i];
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { red[threadIdx.x >> 5] = bv; redi[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
        if (red[w] > bv || (red[w] == bv && redi[w] < bi)) { bv = red[w]; bi = redi[w]; }
      if (bi >= E) bi = 0;
      topk_ids[(size_t)t * k + j] = bi;
      topk_w[(size_t)t * k + j] = score[bi];
      sel[bi] = -FLT_MAX;
      red[0] = score[bi];
    }
    __syncthreads();
    wsum += red[0];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float denom = (renorm && wsum > 0.f) ? wsum : 1.f;
    for (int j = 0; j < k; ++j) topk_w[(size_t)t * k + j] = topk_w[(size_t)t * k + j] / denom * routed_scale;
  }
}

// ------------------------------------------------------------------------------ expert sort
// meta layout (int32): [0, E) counts | [E, 2E] offsets | [2E+1, 3E+1) cursors | 3E+1 num_chunks
__global__ void moe_hist_kernel(const int32_t* __restrict__ topk_ids, int P, int e0, int e1,
                                int32_t* meta) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  const int e = topk_ids[i];
  if (e >= e0 && e < e1) atomicAdd(&meta[e - e0], 1);
}
__global__ void moe_offsets_kernel(int32_t* meta, int E, int chunk_rows, int32_t* chunk_expert,
                                   int32_t* chunk_row0, int32_t* chunk_n, int max_chunks) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int off = 0, nc = 0;
  for (int e = 0; e < E; ++e) {
    meta[E + e] = off;
    meta[2 * E + 1 + e] = off;
    const int c = meta[e];
    for (int r = 0; r < c && nc < max_chunks; r += chunk_rows) {
      chunk_expert[nc] = e;
      chunk_row0[nc] = off + r;
      chunk_n[nc] = min(chunk_rows, c - r);
      ++nc;
    }
    off += c;
  }
  meta[2 * E] = off;
  meta[3 * E + 1] = nc;
}
// Decode-sized batches: histogram, offsets, chunk table and scatter in ONE block (counts and
// cursors in shared memory) instead of a memset and three launches, one of them a single thread
// walking the experts. E <= 256. The order of the rows inside an expert depends on the atomics,
// which is harmless: every row's product is independent and the combine goes through pair_pos.
__global__ void __launch_bounds__(1024)
    moe_sort_small_kernel(const int32_t* __restrict__ topk_ids, int P, int k, int e0, int e1, int32_t* meta,
                          int chunk_rows, int32_t* chunk_expert, int32_t* chunk_row0, int32_t* chunk_n,
                          int max_chunks, int32_t* sorted_token, int32_t* pair_pos) {
  __shared__ int cnt[256], off[256], cbase[256], cursor[256];
  __shared__ int wsum[8], wcsum[8];
  const int E = e1 - e0, tid = threadIdx.x;
  if (tid < 256) cnt[tid] = 0;
  __syncthreads();
  for (int i = tid; i < P; i += blockDim.x) {
    const int e = topk_ids[i];
    if (e >= e0 && e < e1) atomicAdd(&cnt[e - e0], 1);
  }
  __syncthreads();
  if (tid < 256) {
    // exclusive scans of the counts and of the chunk counts over 256 entries: warp scan + 8 totals
    const int c = tid < E ? cnt[tid] : 0;
    const int nch = (c + chunk_rows - 1) / chunk_rows;
    int a = c, b = nch;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int ta = __shfl_up_sync(0xffffffffu, a, o), tb = __shfl_up_sync(0xffffffffu, b, o);
      if ((tid & 31) >= o) { a += ta; b += tb; }
    }
    if ((tid & 31) == 31) { wsum[tid >> 5] = a; wcsum[tid >> 5] = b; }
    off[tid] = a - c;
    cbase[tid] = b - nch;
  }
  __syncthreads();
  if (tid < 256) {
    int pa = 0, pb = 0;
    for (int w = 0; w < (tid >> 5); ++w) { pa += wsum[w]; pb += wcsum[w]; }
    off[tid] += pa;
    cbase[tid] += pb;
  }
  __syncthreads();
  if (tid < E) {
    const int c = cnt[tid], o = off[tid];
    meta[tid] = c;
    meta[E + tid] = o;
    meta[2 * E + 1 + tid] = o + c;          // where the scatter's cursor ends
    cursor[tid] = o;
    int nc = cbase[tid];
    for (int r = 0; r < c && nc < max_chunks; r += chunk_rows, ++nc) {
      chunk_expert[nc] = tid;
      chunk_row0[nc] = o + r;
      chunk_n[nc] = min(chunk_rows, c - r);
    }
    if (tid == E - 1) {
      meta[2 * E] = o + c;
      meta[3 * E + 1] = min(max_chunks, cbase[tid] + (c + chunk_rows - 1) / chunk_rows);
    }
  }
  __syncthreads();
  for (int i = tid; i < P; i += blockDim.x) {
    const int e = topk_ids[i];
    if (e >= e0 && e < e1) {
      const int pos = atomicAdd(&cursor[e - e0], 1);
      sorted_token[pos] = i / k;
      pair_pos[i] = pos;
    } else {
      pair_pos[i] = -1;
    }
  }
}
__global__ void moe_scatter_kernel(const int32_t* __restrict__ topk_ids, int P, int k, int e0,
                                   int e1, int32_t* meta, int E, int32_t* sorted_token,
                                   int32_t* pair_pos) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= P) return;
  const int e = topk_ids[i];
  if (e >= e0 && e < e1) {
    const int pos = atomicAdd(&meta[2 * E + 1 + (e - e0)], 1);
    sorted_token[pos] = i / k;
    pair_pos[i] = pos;
  } else {
    pair_pos[i] = -1;
  }
}
// xs[pos, :] = x[sorted_token[pos], :] for pos < total (read from meta), rows of H bf16
__global__ void __launch_bounds__(128)
    moe_gather_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const int32_t* sorted_token,
                      const int32_t* meta, int E, __nv_bfloat16* xs, int H) {
  const int pos = blockIdx.x;
  if (pos >= meta[2 * E]) return;
  const uint4* s = reinterpret_cast<const uint4*>(x + (size_t)sorted_token[pos] * ldx);
  uint4* d = reinterpret_cast<uint4*>(xs + (size_t)pos * H);
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) d[i] = s[i];
}

// ------------------------------------------------------------------------------ grouped GEMM
static constexpr int kGBM = 128, kGBK = 64, kGMaxStages = 8;
struct GroupedParams {
  int N, K;                 // per expert: out[rows, N] = xs[rows, K] * W_e[N, K]^T
  __nv_bfloat16* out;       // [P, N] sorted order
  const int32_t* chunk_expert;
  const int32_t* chunk_row0;
  const int32_t* chunk_n;
  const int32_t* meta;
  int E;
  int stages;
  // Gated mode (act_fuse = activation kind + 1): W_e is [gate rows (N/2) | up rows (N/2)]; a CTA
  // takes 128 gate rows and the 128 up rows of the same outputs, keeps one accumulator for each in
  // TMEM (columns [0, np) and [256, 256 + np)) and writes act(gate) * up to out[rows, N / 2], so the
  // merged projection never reaches memory. Both values are rounded to bf16 first, as the separate
  // activation kernel would see them.
  int act_fuse;
  int* status;
};
struct alignas(8) GroupedBars {
  uint64_t full[kGMaxStages], empty[kGMaxStages], acc_full;
  uint32_t tmem_base;
};

// grid: (N / 128, max_chunks). A CTA whose chunk index is past the device-side count exits.
__global__ void __launch_bounds__(192, 1)
    moe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmW,
                            const __grid_constant__ CUtensorMap tmX, GroupedParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  const int chunk = blockIdx.y;
  if (chunk >= p.meta[3 * p.E + 1]) return;
  const int e = p.chunk_expert[chunk], row0 = p.chunk_row0[chunk], rows = p.chunk_n[chunk];
  const int np = (rows + 15) & ~15;                 // UMMA N
  constexpr int kWBytes = kGBM * kGBK * 2;
  constexpr int kXBytes = 256 * kGBK * 2;           // TMA box is always 256 rows
  const bool gated = p.act_fuse != 0;
  const int half_n = p.N >> 1;                      // gated: outputs per expert
  const int kStage = kWBytes * (gated ? 2 : 1) + kXBytes;
  const int stages = p.stages;
  GroupedBars* bars = reinterpret_cast<GroupedBars*>(smem + (size_t)stages * kStage);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tn = blockIdx.x;
  const int nkb = (p.K + kGBK - 1) / kGBK;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
    mbar_init(&bars->acc_full, 1);
    mbar_fence_init();
  }
  const uint32_t tmem_cols = gated ? 512 : 256;
  if (warp == 1) { tmem_alloc(&bars->tmem_base, tmem_cols); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const int x_off = kWBytes * (gated ? 2 : 1);
  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmW);
      tma_prefetch_desc(&tmX);
      for (int i = 0; i < nkb; ++i) {
        const int s = i % stages;
        if (!mbar_wait(&bars->empty[s], ((i / stages) & 1) ^ 1, p.status)) break;
        uint8_t* wd = smem + (size_t)s * kStage;
        mbar_expect_tx(&bars->full[s], kStage);
        tma_load_3d(wd, &tmW, &bars->full[s], i * kGBK, tn * kGBM, e);
        if (gated) tma_load_3d(wd + kWBytes, &tmW, &bars->full[s], i * kGBK, half_n + tn * kGBM, e);
        tma_load_2d(wd + x_off, &tmX, &bars->full[s], i * kGBK, row0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(kGBM, np);
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        const int s = i % stages;
        if (!mbar_wait(&bars->full[s], (i / stages) & 1, p.status)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t wa = smem_u32(smem + (size_t)s * kStage), xa = wa + x_off;
#pragma unroll
        for (int kk = 0; kk < kGBK / 16; ++kk) {
          umma_bf16_ss(tmem_base, umma_desc_k_sw128(wa + kk * 32, 1024),
                       umma_desc_k_sw128(xa + kk * 32, 1024), idesc, (i | kk) != 0);
          if (gated)
            umma_bf16_ss(tmem_base + 256, umma_desc_k_sw128(wa + kWBytes + kk * 32, 1024),
                         umma_desc_k_sw128(xa + kk * 32, 1024), idesc, (i | kk) != 0);
        }
        umma_commit(&bars->empty[s]);
      }
      if (ok) umma_commit(&bars->acc_full);
    }
  } else if (gated) {
    const int quarter = warp & 3;
    bool ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_full, 0, p.status));
    tc_fence_after_sync();
    const int n = tn * kGBM + quarter * 32 + lane;        // output column of this thread
    const uint32_t ta = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int kind = p.act_fuse - 1;
    if (ok) {
      for (int c = 0; c < np / 16; ++c) {
        uint32_t g[16], u[16];
        tmem_ld_32x32b_x16(ta + c * 16, g);
        tmem_ld_32x32b_x16(ta + 256 + c * 16, u);
        tmem_ld_wait();
        if (n < half_n) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int m = c * 16 + i;
            if (m < rows) {
              const float gg = __bfloat162float(__float2bfloat16(__uint_as_float(g[i])));
              const float uu = __bfloat162float(__float2bfloat16(__uint_as_float(u[i])));
              float a;
              if (kind == 0) a = gg / (1.f + __expf(-gg));
              else if (kind == 1) a = 0.5f * gg * (1.f + tanhf(0.7978845608028654f * (gg + 0.044715f * gg * gg * gg)));
              else a = 0.5f * gg * (1.f + erff(gg * 0.7071067811865476f));
              p.out[(size_t)(row0 + m) * half_n + n] = __float2bfloat16(a * uu);
            }
          }
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    bool ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_full, 0, p.status));
    tc_fence_after_sync();
    const int n = tn * kGBM + quarter * 32 + lane;
    const uint32_t ta = tmem_base + ((uint32_t)(quarter * 32) << 16);
    if (ok) {
      for (int c = 0; c < np / 16; ++c) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(ta + c * 16, r);
        tmem_ld_wait();
        if (n < p.N) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int m = c * 16 + i;
            if (m < rows)
              p.out[(size_t)(row0 + m) * p.N + n] = __float2bfloat16(__uint_as_float(r[i]));
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, tmem_cols);
}

// ---------------------------------------------------------------------------------- combine
// out[t, :] = sum_j w[t, j] * y[pair_pos[t, j], :] (+ shared[t, :] * shared_scale[t]) ;
// pairs routed to experts of other ranks (pair_pos < 0) are skipped. fp32 accumulation in
// ascending j, one bf16 rounding. With `peer_recv` set the row is stored into the receive
// slot of its owner rank (combine + reduce-scatter); signalled per 32-row group.
struct CombineParams {
  const __nv_bfloat16* y;
  const int32_t* pair_pos;
  const float* topk_w;
  int k, H, T;
  const __nv_bfloat16* shared;       // optional [T, H]
  const float* shared_gate;          // optional [T] (sigmoid applied by the caller)
  __nv_bfloat16* out;                // [T, H] when not scattering
  int tp_world, tp_rank, rows_per_rank;
  __nv_bfloat16* peer_recv[8];
  uint32_t* peer_rs_flags[8];
  long long recv_parity_stride;
  int rs_flag_parity_stride;
  const uint32_t* op_counter;
};
__global__ void __launch_bounds__(128) moe_combine_kernel(CombineParams p) {
  const int t = blockIdx.x;
  const int nv = p.H >> 3;
  __nv_bfloat16* dst;
  uint32_t par = 0;
  int owner = 0;
  if (p.tp_world > 1 && p.peer_recv[0]) {
    owner = t / p.rows_per_rank;
    par = *p.op_counter & 1;
    dst = p.peer_recv[owner] + par * p.recv_parity_stride +
          ((size_t)p.tp_rank * p.rows_per_rank + (t - owner * p.rows_per_rank)) * p.H;
  } else {
    dst = p.out + (size_t)t * p.H;
  }
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int j = 0; j < p.k; ++j) {
      const int pos = p.pair_pos[(size_t)t * p.k + j];
      if (pos < 0) continue;
      const float w = p.topk_w[(size_t)t * p.k + j];
      const uint4 v = *reinterpret_cast<const uint4*>(p.y + (size_t)pos * p.H + i * 8);
      float2 f;
      f = unpack_bf16x2(v.x); acc[0] += w * f.x; acc[1] += w * f.y;
      f = unpack_bf16x2(v.y); acc[2] += w * f.x; acc[3] += w * f.y;
      f = unpack_bf16x2(v.z); acc[4] += w * f.x; acc[5] += w * f.y;
      f = unpack_bf16x2(v.w); acc[6] += w * f.x; acc[7] += w * f.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    if (p.shared) {
      // routed sum is rounded to bf16 first, then the shared expert is added (reference order)
      const float g = p.shared_gate ? p.shared_gate[t] : 1.f;
      const uint4 s = *reinterpret_cast<const uint4*>(p.shared + (size_t)t * p.H + i * 8);
      float2 a, b;
      a = unpack_bf16x2(o.x); b = unpack_bf16x2(s.x); o.x = pack_bf16x2(a.x + g * b.x, a.y + g * b.y);
      a = unpack_bf16x2(o.y); b = unpack_bf16x2(s.y); o.y = pack_bf16x2(a.x + g * b.x, a.y + g * b.y);
      a = unpack_bf16x2(o.z); b = unpack_bf16x2(s.z); o.z = pack_bf16x2(a.x + g * b.x, a.y + g * b.y);
      a = unpack_bf16x2(o.w); b = unpack_bf16x2(s.w); o.w = pack_bf16x2(a.x + g * b.x, a.y + g * b.y);
    }
    reinterpret_cast<uint4*>(dst)[i] = o;
  }
  if (p.tp_world > 1 && p.peer_recv[0]) {
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      // every 32-row group receives exactly 32 arrivals per source rank: the last token also
      // covers the rows its (partial) group does not have
      uint32_t inc = 1;
      if (t == p.T - 1 && (p.T & 31)) inc += 32 - (p.T & 31);
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(
                       p.peer_rs_flags[owner] + par * p.rs_flag_parity_stride +
                       (t - owner * p.rows_per_rank) / 32),
                   "r"(inc)
                   : "memory");
    }
  }
}

// sigmoid(x . w) per row: gate of the shared expert (Qwen3.5 / 3.6 MoE)
__global__ void __launch_bounds__(128)
    shared_gate_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* w, int H,
                       float* out) {
  __shared__ float red[4];
  const int t = blockIdx.x;
  float s = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x)
    s += __bfloat162float(x[(size_t)t * ldx + i]) * __bfloat162float(w[i]);
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    const float v = red[0] + red[1] + red[2] + red[3];
    out[t] = 1.f / (1.f + expf(-v));
  }
}

}  // namespace b200

using namespace b200;
typedef __nv_bfloat16 bf16;
#define RETL return cudaGetLastError() == cudaSuccess ? 0 : -2

extern "C" {

int b200_moe_router_topk(const void* logits_f32, int ld, int T, int E, int k, int renorm,
                         int scoring, const void* e_bias, int n_group, int topk_group,
                         float routed_scale, void* topk_ids, void* topk_w, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (k > E || n_group > 64 || (n_group > 1 && E % n_group)) return -1;
  moe_router_topk_kernel<<<T, 256, (size_t)2 * E * sizeof(float), stream>>>(
      (const float*)logits_f32, ld, E, k, renorm, scoring, (const float*)e_bias, n_group,
      topk_group, routed_scale, (int32_t*)topk_ids, (float*)topk_w);
  RETL;
}

// Sorts the (token, expert) pairs whose expert is in [e0, e1) by expert.
// meta: int32[3*E_local + 2] (zeroed here); chunk arrays: int32[max_chunks].
int b200_moe_sort(const void* topk_ids, int T, int k, int e0, int e1, void* meta,
                  void* sorted_token, void* pair_pos, void* chunk_expert, void* chunk_row0,
                  void* chunk_n, int max_chunks, cudaStream_t stream) {
  const int P = T * k, E = e1 - e0;
  if (P <= 0) return 0;
  if (E <= 256 && P <= 16384) {
    moe_sort_small_kernel<<<1, 1024, 0, stream>>>((const int32_t*)topk_ids, P, k, e0, e1, (int32_t*)meta, 256,
                                                  (int32_t*)chunk_expert, (int32_t*)chunk_row0, (int32_t*)chunk_n,
                                                  max_chunks, (int32_t*)sorted_token, (int32_t*)pair_pos);
    RETL;
  }
  cudaMemsetAsync(meta, 0, (size_t)(3 * E + 2) * sizeof(int32_t), stream);
  moe_hist_kernel<<<(P + 255) / 256, 256, 0, stream>>>((const int32_t*)topk_ids, P, e0, e1,
                                                       (int32_t*)meta);
  moe_offsets_kernel<<<1, 1, 0, stream>>>((int32_t*)meta, E, 256, (int32_t*)chunk_expert,
                                          (int32_t*)chunk_row0, (int32_t*)chunk_n, max_chunks);
  moe_scatter_kernel<<<(P + 255) / 256, 256, 0, stream>>>((const int32_t*)topk_ids, P, k, e0, e1,
                                                          (int32_t*)meta, E, (int32_t*)sorted_token,
                                                          (int32_t*)pair_pos);
  RETL;
}

int b200_moe_gather(const void* x, int ldx, const void* sorted_token, const void* meta, int E,
                    void* xs, int H, int max_rows, cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  moe_gather_kernel<<<max_rows, 128, 0, stream>>>((const bf16*)x, ldx, (const int32_t*)sorted_token,
                                                  (const int32_t*)meta, E, (bf16*)xs, H);
  RETL;
}

// out[P, N] = grouped(xs[P, K], W[E, N, K]); xs must have at least max_rows + 256 rows allocated.
static int moe_grouped_gemm_impl(const void* xs, int max_rows, const void* W, int E, int N, int K,
                                 void* out, const void* chunk_expert, const void* chunk_row0,
                                 const void* chunk_n, const void* meta, int max_chunks, int act_fuse,
                                 cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  if ((K & 7) || (N & 7)) return -1;
  if (act_fuse && ((N & 1) || ((N / 2) & 7) || act_fuse < 1 || act_fuse > 3)) return -1;
  static std::mutex mu;
  CUtensorMap tmW, tmX;
  if (!encode_tmap_3d(&tmW, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)K, (uint64_t)N,
                      (uint64_t)E, (uint64_t)K * 2, (uint64_t)N * K * 2, kGBK, kGBM, 1,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  if (!encode_tmap_2d(&tmX, xs, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)max_rows + 256,
                      (uint64_t)K, (uint64_t)K, 256, kGBK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  GroupedParams p;
  p.N = N; p.K = K; p.out = (bf16*)out;
  p.chunk_expert = (const int32_t*)chunk_expert; p.chunk_row0 = (const int32_t*)chunk_row0;
  p.chunk_n = (const int32_t*)chunk_n; p.meta = (const int32_t*)meta; p.E = E;
  const int stage = kGBM * kGBK * 2 * (act_fuse ? 2 : 1) + 256 * kGBK * 2;
  int stages = (200 * 1024) / stage;
  if (stages > kGMaxStages) stages = kGMaxStages;
  const int nkb = (K + kGBK - 1) / kGBK;
  if (stages > nkb) stages = nkb < 2 ? 2 : nkb;
  p.stages = stages; p.act_fuse = act_fuse; p.status = device_status_word();
  const size_t smem = (size_t)stages * stage + 1024 + sizeof(GroupedBars);
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(moe_grouped_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         220 * 1024);
  }
  dim3 grid(((act_fuse ? N / 2 : N) + kGBM - 1) / kGBM, max_chunks);
  moe_grouped_gemm_kernel<<<grid, 192, smem, stream>>>(tmW, tmX, p);
  RETL;
}

int b200_moe_grouped_gemm(const void* xs, int max_rows, const void* W, int E, int N, int K,
                          void* out, const void* chunk_expert, const void* chunk_row0,
                          const void* chunk_n, const void* meta, int max_chunks,
                          cudaStream_t stream) {
  return moe_grouped_gemm_impl(xs, max_rows, W, E, N, K, out, chunk_expert, chunk_row0, chunk_n, meta, max_chunks, 0,
                               stream);
}
// Gate / up projection with the gated activation in the epilogue: W [E, 2 I, K] with rows
// [gate (I) | up (I)], out[P, I] = act(xs W_gate^T) * (xs W_up^T). kind: 0 SiLU, 1 GELU-tanh, 2 GELU-erf.
int b200_moe_grouped_gemm_gated(const void* xs, int max_rows, const void* W, int E, int N, int K,
                                void* out, const void* chunk_expert, const void* chunk_row0,
                                const void* chunk_n, const void* meta, int max_chunks, int kind,
                                cudaStream_t stream) {
  return moe_grouped_gemm_impl(xs, max_rows, W, E, N, K, out, chunk_expert, chunk_row0, chunk_n, meta, max_chunks,
                               kind + 1, stream);
}


int b200_moe_combine(const void* y, const void* pair_pos, const void* topk_w, int T, int k, int H,
                     const void* shared, const void* shared_gate, void* out,
                     const B200MoeScatter* sc, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H & 7) return -1;
  CombineParams p{};
  p.y = (const bf16*)y; p.pair_pos = (const int32_t*)pair_pos; p.topk_w = (const float*)topk_w;
  p.k = k; p.H = H; p.T = T; p.shared = (const bf16*)shared; p.shared_gate = (const float*)shared_gate;
  p.out = (bf16*)out;
  if (sc && sc->world > 1) {
    p.tp_world = sc->world; p.tp_rank = sc->rank; p.rows_per_rank = sc->rows_per_rank;
    for (int i = 0; i < sc->world; ++i) {
      p.peer_recv[i] = (bf16*)sc->peer_recv[i];
      p.peer_rs_flags[i] = (uint32_t*)sc->peer_rs_flags[i];
    }
    p.recv_parity_stride = sc->recv_parity_stride;
    p.rs_flag_parity_stride = sc->rs_flag_parity_stride;
    p.op_counter = (const uint32_t*)sc->op_counter;
  }
  moe_combine_kernel<<<T, 128, 0, stream>>>(p);
  RETL;
}

int b200_shared_gate(const void* x, int ldx, const void* w, int T, int H, void* out,
                     cudaStream_t stream) {
  if (T <= 0) return 0;
  shared_gate_kernel<<<T, 128, 0, stream>>>((const bf16*)x, ldx, (const bf16*)w, H, (float*)out);
  RETL;
}

}  // extern "C"
