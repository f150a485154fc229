// Sampler kernels over fp32 logits [n, V] (row stride ld). All reductions are fixed-order
// tree reductions (no float atomics), argmax breaks ties towards the lowest index, and the
// random draw is an exponential race driven by a SplitMix64 counter RNG that the host
// sampler reproduces bit for bit.
//
// Covers the reference's src/vt/cuda/cuda_sample.cu (ApplyTemperature :62, two-stage argmax
// :102/:130, Softmax :220, RandomSample :270, ApplyTopKTopP :367, ApplyPenalties :510,
// ApplyMinP :544, bias / mask / allowed ids :588-621, greedy rejection :647/:671) and
// cuda_combine_tokens.cu (async-scheduling input splice).
#include <float.h>

#include "api.h"
#include "sm100.cuh"

namespace b200 {

static constexpr int kSB = 256;  // threads per block for row kernels
static constexpr float kEps = 1e-5f;

struct ArgPair { float v; int i; };
__device__ __forceinline__ ArgPair arg_better(ArgPair a, ArgPair b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ ArgPair block_argmax(ArgPair a, ArgPair* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = arg_better(a, b);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) sh[warp] = a;
  __syncthreads();
  ArgPair r = (lane < nw) ? sh[lane] : ArgPair{-FLT_MAX, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair b;
    b.v = __shfl_xor_sync(0xffffffffu, r.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, r.i, o);
    r = arg_better(r, b);
  }
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_reduce_sum(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? sh[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_reduce_max(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = (lane < nw) ? sh[lane] : -FLT_MAX;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
  __syncthreads();
  return r;
}
__device__ __forceinline__ int block_reduce_sum_int(int v, int* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  int r = (lane < nw) ? sh[lane] : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  __syncthreads();
  return r;
}

// ---- two-stage argmax ----
__global__ void __launch_bounds__(kSB)
    argmax_partial_kernel(const float* __restrict__ logits, int ld, int V, int blocks_per_row,
                          float* pv, int* pi) {
  __shared__ ArgPair sh[32];
  const int row = blockIdx.y, blk = blockIdx.x;
  const int per = (((V + blocks_per_row - 1) / blocks_per_row) + 3) & ~3;   // multiple of 4
  const int lo = blk * per, hi = min(V, lo + per);
  const float* x = logits + (size_t)row * ld;
  ArgPair a{-FLT_MAX, 0x7fffffff};
  int i0 = lo;
  if (!(ld & 3) && !(reinterpret_cast<uintptr_t>(logits) & 15)) {
    // 16-byte loads over the aligned part of the slice (lo is a multiple of 4)
    const int hi4 = lo + ((hi - lo) & ~3);
    for (int i = lo + threadIdx.x * 4; i < hi4; i += blockDim.x * 4) {
      const float4 q = *reinterpret_cast<const float4*>(x + i);
      const float v[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) a = arg_better(a, ArgPair{v[k] != v[k] ? -FLT_MAX : v[k], i + k});
    }
    i0 = max(lo, hi4);
  }
  for (int i = i0 + threadIdx.x; i < hi; i += blockDim.x) {
    float v = x[i];
    if (v != v) v = -FLT_MAX;
    a = arg_better(a, ArgPair{v, i});
  }
  a = block_argmax(a, sh);
  if (threadIdx.x == 0) {
    pv[row * blocks_per_row + blk] = a.v;
    pi[row * blocks_per_row + blk] = a.i;
  }
}
__global__ void __launch_bounds__(32)
    argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi,
                        int blocks_per_row, int64_t* out, int V) {
  const int row = blockIdx.x;
  ArgPair a{-FLT_MAX, 0x7fffffff};
  for (int i = threadIdx.x; i < blocks_per_row; i += 32)
    a = arg_better(a, ArgPair{pv[row * blocks_per_row + i], pi[row * blocks_per_row + i]});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = arg_better(a, b);
  }
  if (threadIdx.x == 0) out[row] = (a.i >= V || a.i < 0) ? 0 : a.i;
}

// Vocabulary-parallel greedy sampling: each rank reduces its own logits shard to one
// (value, global index) candidate per row; after the candidates of all ranks have been gathered
// ([n][world] pairs, 8 bytes each) the best one wins, ties going to the lowest index, so the
// result equals the argmax over the full row.
__global__ void __launch_bounds__(32)
    argmax_candidate_kernel(const float* __restrict__ pv, const int* __restrict__ pi,
                            int blocks_per_row, int V, int index_base, int2* __restrict__ out) {
  const int row = blockIdx.x;
  ArgPair a{-FLT_MAX, 0x7fffffff};
  for (int i = threadIdx.x; i < blocks_per_row; i += 32)
    a = arg_better(a, ArgPair{pv[row * blocks_per_row + i], pi[row * blocks_per_row + i]});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = arg_better(a, b);
  }
  if (threadIdx.x == 0) {
    const bool ok = a.i >= 0 && a.i < V;
    out[row] = make_int2(__float_as_int(ok ? a.v : -FLT_MAX), ok ? index_base + a.i : 0x7fffffff);
  }
}
__global__ void argmax_combine_kernel(const int2* __restrict__ cand, int n, int world, int V_total,
                                      int64_t* __restrict__ out) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= n) return;
  ArgPair a{-FLT_MAX, 0x7fffffff};
  for (int r = 0; r < world; ++r) {
    const int2 c = cand[(size_t)r * n + row];     // rank-major, as an all-gather along dim 0 lays it out
    a = arg_better(a, ArgPair{__int_as_float(c.x), c.y});
  }
  out[row] = (a.i < 0 || a.i >= V_total) ? 0 : a.i;
}

// ---- temperature: rows with temperature < eps are left untouched (greedy rows) ----
__global__ void temperature_kernel(float* logits, int ld, int V, const float* __restrict__ temp) {
  const int row = blockIdx.y;
  const float t = temp[row];
  if (t < kEps) return;
  const float inv = 1.f / t;
  float* x = logits + (size_t)row * ld;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += gridDim.x * blockDim.x)
    x[i] *= inv;
}

// ---- penalties over (row, token, output_count) triples; every triple is unique ----
__global__ void penalties_kernel(float* logits, int ld, int V, const int* __restrict__ rows,
                                 const int* __restrict__ toks, const int* __restrict__ out_cnt,
                                 int n, const float* __restrict__ rep,
                                 const float* __restrict__ freq, const float* __restrict__ pres) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = rows[i], t = toks[i];
  if (t < 0 || t >= V) return;
  float v = logits[(size_t)r * ld + t];
  const float rp = rep[r];
  v = v > 0.f ? v / rp : v * rp;
  const int c = out_cnt[i];
  v -= freq[r] * (float)c;
  if (c > 0) v -= pres[r];
  logits[(size_t)r * ld + t] = v;
}

// ---- sparse edits: mode 0 add bias, 1 set -inf ----
__global__ void sparse_edit_kernel(float* logits, int ld, int V, const int* __restrict__ rows,
                                   const int* __restrict__ toks, const float* __restrict__ vals,
                                   int n, int mode) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int r = rows[i], t = toks[i];
  if (t < 0 || t >= V) return;
  if (mode == 0) logits[(size_t)r * ld + t] += vals[i];
  else logits[(size_t)r * ld + t] = -INFINITY;
}

// ---- packed bit mask [n, ceil(V/32)] : bit = 1 keeps the token. row_ids maps mask rows to
// logits rows (grammar requests only); allowed-token-ids use the same kernel. ----
__global__ void bitmask_kernel(float* logits, int ld, int V, const int32_t* __restrict__ mask,
                               int words, const int* __restrict__ row_ids) {
  const int mr = blockIdx.y;
  const int row = row_ids ? row_ids[mr] : mr;
  if (row < 0) return;
  float* x = logits + (size_t)row * ld;
  const int32_t* m = mask + (size_t)mr * words;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < V; i += gridDim.x * blockDim.x)
    if (!((m[i >> 5] >> (i & 31)) & 1)) x[i] = -INFINITY;
}

// ---- min-p: drop tokens whose prob < min_p * max prob  <=> logit < max + ln(min_p) ----
__global__ void __launch_bounds__(kSB)
    min_p_kernel(float* logits, int ld, int V, const float* __restrict__ min_p) {
  __shared__ float sh[32];
  const int row = blockIdx.x;
  const float mp = min_p[row];
  if (mp <= 0.f) return;
  float* x = logits + (size_t)row * ld;
  float mx = -FLT_MAX;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, x[i]);
  mx = block_reduce_max(mx, sh);
  const float thr = mx + logf(mp);
  for (int i = threadIdx.x; i < V; i += blockDim.x)
    if (x[i] < thr) x[i] = -INFINITY;
}

// ---- top-k / top-p without a sort ----
// Monotone key: larger float -> larger uint.
__device__ __forceinline__ uint32_t fkey(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float fkey_inv(uint32_t k) {
  uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}
// One block per row. top-k: bitwise radix select of the k-th largest key (count based).
// top-p: bisection on the key for the largest threshold whose kept mass is >= p, mass summed
// with a fixed-order block reduction. Ties at the threshold are all kept (same as the
// sort-based rule for distinct logits).
__global__ void __launch_bounds__(kSB)
    top_k_top_p_kernel(float* logits, int ld, int V, const int* __restrict__ top_k,
                       const float* __restrict__ top_p) {
  __shared__ float shf[32];
  __shared__ int shi[32];
  const int row = blockIdx.x;
  float* x = logits + (size_t)row * ld;
  const int k = top_k ? top_k[row] : 0;
  const float pth = top_p ? top_p[row] : 1.f;
  const bool do_k = (k > 0 && k < V);
  const bool do_p = (pth < 1.f);
  if (!do_k && !do_p) return;
  uint32_t thr_key = 0;
  if (do_k) {
    // find the largest key T such that count(key >= T) >= k
    uint32_t prefix = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = prefix | (1u << bit);
      int c = 0;
      for (int i = threadIdx.x; i < V; i += blockDim.x) c += (fkey(x[i]) >= cand);
      c = block_reduce_sum_int(c, shi);
      if (c >= k) prefix = cand;
    }
    thr_key = prefix;
  }
  if (do_p) {
    float mx = -FLT_MAX;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = x[i];
      if (fkey(v) >= thr_key) mx = fmaxf(mx, v);
    }
    mx = block_reduce_max(mx, shf);
    float tot = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = x[i];
      if (fkey(v) >= thr_key) tot += __expf(v - mx);
    }
    tot = block_reduce_sum(tot, shf);
    const float need = pth * tot;
    // largest key T (>= thr_key) with mass(key >= T) >= need
    uint32_t prefix = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = prefix | (1u << bit);
      float s = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = x[i];
        const uint32_t kk = fkey(v);
        if (kk >= cand && kk >= thr_key) s += __expf(v - mx);
      }
      s = block_reduce_sum(s, shf);
      if (s >= need) prefix = cand;
    }
    if (prefix > thr_key) thr_key = prefix;
  }
  for (int i = threadIdx.x; i < V; i += blockDim.x)
    if (fkey(x[i]) < thr_key) x[i] = -INFINITY;
}

// ---- softmax / log-softmax (out may alias in) ----
__global__ void __launch_bounds__(kSB)
    softmax_kernel(const float* __restrict__ logits, int ld, float* out, int ldo, int V,
                   int log_mode) {
  __shared__ float sh[32];
  const int row = blockIdx.x;
  const float* x = logits + (size_t)row * ld;
  float* o = out + (size_t)row * ldo;
  float mx = -FLT_MAX;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, x[i]);
  mx = block_reduce_max(mx, sh);
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) s += __expf(x[i] - mx);
  s = block_reduce_sum(s, sh);
  if (log_mode) {
    const float lz = mx + logf(s);
    for (int i = threadIdx.x; i < V; i += blockDim.x) o[i] = x[i] - lz;
  } else {
    const float inv = 1.f / s;
    for (int i = threadIdx.x; i < V; i += blockDim.x) o[i] = __expf(x[i] - mx) * inv;
  }
}

// ---- seeded exponential-race sample: argmax_i p_i / (-log u_i) ----
__host__ __device__ inline uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ float race_key(float prob, uint64_t seed, uint64_t step, int col) {
  const uint64_t z = splitmix64(seed ^ splitmix64(step * 0x100000001B3ull + (uint64_t)col));
  const double u = ((double)(z >> 11) + 0.5) * (1.0 / 9007199254740992.0);
  const float e = (float)(-log(u));
  return prob / e;
}
__global__ void __launch_bounds__(kSB)
    random_sample_kernel(const float* __restrict__ probs, int ld, int V,
                         const uint64_t* __restrict__ seeds, const uint64_t* __restrict__ steps,
                         int64_t* out) {
  __shared__ ArgPair sh[32];
  const int row = blockIdx.x;
  const float* x = probs + (size_t)row * ld;
  const uint64_t seed = seeds[row], step = steps[row];
  ArgPair a{-FLT_MAX, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float pr = x[i];
    if (pr > 0.f) a = arg_better(a, ArgPair{race_key(pr, seed, step, i), i});
  }
  a = block_argmax(a, sh);
  if (threadIdx.x == 0) out[row] = (a.i >= V || a.i < 0) ? 0 : a.i;
}

// out[row] = is_greedy ? greedy[row] : random[row]
__global__ void merge_greedy_random_kernel(const int64_t* g, const int64_t* r,
                                           const float* __restrict__ temp, int64_t* out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = temp[i] < kEps ? g[i] : r[i];
}

// ---- logprob + rank of chosen tokens from log-softmax rows ----
__global__ void __launch_bounds__(kSB)
    token_rank_kernel(const float* __restrict__ logprobs, int ld, int V,
                      const int64_t* __restrict__ toks, float* out_lp, int* out_rank) {
  __shared__ int shi[32];
  const int row = blockIdx.x;
  const float* x = logprobs + (size_t)row * ld;
  const int64_t t = toks[row];
  const float v = (t >= 0 && t < V) ? x[t] : -INFINITY;
  int c = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) c += (x[i] > v);
  c = block_reduce_sum_int(c, shi);
  if (threadIdx.x == 0) {
    out_lp[row] = v;
    out_rank[row] = c + 1;
  }
}

// ---- greedy rejection sampling for speculative decoding ----
// target_argmax: [sum(draft)+n] argmax of the target logits at every draft position plus the
// bonus position; cu: [n+1] prefix offsets of draft tokens. out: [n, max_spec+1], -1 padded.
__global__ void greedy_reject_kernel(const int64_t* __restrict__ target_argmax,
                                     const int64_t* __restrict__ draft,
                                     const int* __restrict__ cu_draft, int n, int max_spec,
                                     int64_t* out) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  const int d0 = cu_draft[r], nd = cu_draft[r + 1] - d0;
  const int t0 = d0 + r;  // target rows: nd draft positions + 1 bonus per request
  int64_t* o = out + (size_t)r * (max_spec + 1);
  for (int i = 0; i <= max_spec; ++i) o[i] = -1;
  int i = 0;
  for (; i < nd; ++i) {
    const int64_t tg = target_argmax[t0 + i];
    o[i] = tg;
    if (tg != draft[d0 + i]) return;  // replacement token emitted, stop
  }
  o[nd] = target_argmax[t0 + nd];  // all accepted: bonus token
}

// ---- async-scheduling input splice ----
// input_ids[dst_idx[i]] = last_sampled[src_row[i]]
__global__ void splice_sampled_kernel(int64_t* input_ids, const int* __restrict__ dst_idx,
                                      const int* __restrict__ src_row,
                                      const int64_t* __restrict__ last_sampled, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) input_ids[dst_idx[i]] = last_sampled[src_row[i]];
}
// last_sampled[row_of[i]] = sampled[i]
__global__ void scatter_sampled_kernel(int64_t* last_sampled, const int* __restrict__ row_of,
                                       const int64_t* __restrict__ sampled, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && row_of[i] >= 0) last_sampled[row_of[i]] = sampled[i];
}

}  // namespace b200

using namespace b200;
#define RET_LAUNCH return cudaGetLastError() == cudaSuccess ? 0 : -2

extern "C" {

int b200_argmax_blocks_per_row(int n, int V) {
  int target = b200_num_sms() * 2;
  int bpr = (target + n - 1) / n;
  int maxb = (V + 4095) / 4096;
  if (bpr > maxb) bpr = maxb;
  if (bpr < 1) bpr = 1;
  if (bpr > 64) bpr = 64;
  return bpr;
}

// scratch: float[n*64] + int[n*64]
int b200_argmax(const void* logits, int ld, int n, int V, void* out_i64, void* scratch_f,
                void* scratch_i, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int bpr = b200_argmax_blocks_per_row(n, V);
  dim3 grid(bpr, n);
  argmax_partial_kernel<<<grid, kSB, 0, stream>>>((const float*)logits, ld, V, bpr,
                                                  (float*)scratch_f, (int*)scratch_i);
  argmax_final_kernel<<<n, 32, 0, stream>>>((const float*)scratch_f, (const int*)scratch_i, bpr,
                                            (int64_t*)out_i64, V);
  RET_LAUNCH;
}

// Local stage of the vocabulary-parallel argmax: cand_out[n] (8 bytes each) = best (value,
// index_base + column) of this rank's logits[n, V]; columns at or beyond v_valid are ignored
// (padding of the last shard).
int b200_argmax_candidates(const void* logits, int ld, int n, int V, int v_valid, int index_base,
                           void* cand_out, void* scratch_f, void* scratch_i, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (v_valid > V) v_valid = V;
  if (v_valid <= 0) {   // nothing of the vocabulary lives here: candidates that never win
    argmax_candidate_kernel<<<n, 32, 0, stream>>>(nullptr, nullptr, 0, 0, index_base, (int2*)cand_out);
    RET_LAUNCH;
  }
  const int bpr = b200_argmax_blocks_per_row(n, v_valid);
  dim3 grid(bpr, n);
  argmax_partial_kernel<<<grid, kSB, 0, stream>>>((const float*)logits, ld, v_valid, bpr,
                                                  (float*)scratch_f, (int*)scratch_i);
  argmax_candidate_kernel<<<n, 32, 0, stream>>>((const float*)scratch_f, (const int*)scratch_i, bpr, v_valid,
                                                index_base, (int2*)cand_out);
  RET_LAUNCH;
}
// Final stage: cand[world][n] pairs -> out[n] int64 token ids.
int b200_argmax_combine(const void* cand, int n, int world, int V_total, void* out_i64,
                        cudaStream_t stream) {
  if (n <= 0) return 0;
  argmax_combine_kernel<<<(n + 127) / 128, 128, 0, stream>>>((const int2*)cand, n, world, V_total,
                                                             (int64_t*)out_i64);
  RET_LAUNCH;
}

int b200_apply_temperature(void* logits, int ld, int n, int V, const void* temp,
                           cudaStream_t stream) {
  if (n <= 0) return 0;
  dim3 grid(min(64, (V + 255) / 256), n);
  temperature_kernel<<<grid, 256, 0, stream>>>((float*)logits, ld, V, (const float*)temp);
  RET_LAUNCH;
}

int b200_apply_penalties(void* logits, int ld, int V, const void* rows, const void* toks,
                         const void* out_cnt, int n_entries, const void* rep, const void* freq,
                         const void* pres, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  penalties_kernel<<<(n_entries + 255) / 256, 256, 0, stream>>>(
      (float*)logits, ld, V, (const int*)rows, (const int*)toks, (const int*)out_cnt, n_entries,
      (const float*)rep, (const float*)freq, (const float*)pres);
  RET_LAUNCH;
}

int b200_sparse_edit(void* logits, int ld, int V, const void* rows, const void* toks,
                     const void* vals, int n_entries, int mode, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  sparse_edit_kernel<<<(n_entries + 255) / 256, 256, 0, stream>>>(
      (float*)logits, ld, V, (const int*)rows, (const int*)toks, (const float*)vals, n_entries,
      mode);
  RET_LAUNCH;
}

int b200_apply_bitmask(void* logits, int ld, int V, const void* mask, int n_mask_rows,
                       const void* row_ids, cudaStream_t stream) {
  if (n_mask_rows <= 0) return 0;
  dim3 grid(min(64, (V + 255) / 256), n_mask_rows);
  bitmask_kernel<<<grid, 256, 0, stream>>>((float*)logits, ld, V, (const int32_t*)mask,
                                           (V + 31) / 32, (const int*)row_ids);
  RET_LAUNCH;
}

int b200_apply_min_p(void* logits, int ld, int n, int V, const void* min_p, cudaStream_t stream) {
  if (n <= 0) return 0;
  min_p_kernel<<<n, kSB, 0, stream>>>((float*)logits, ld, V, (const float*)min_p);
  RET_LAUNCH;
}

int b200_apply_top_k_top_p(void* logits, int ld, int n, int V, const void* top_k,
                           const void* top_p, cudaStream_t stream) {
  if (n <= 0) return 0;
  top_k_top_p_kernel<<<n, kSB, 0, stream>>>((float*)logits, ld, V, (const int*)top_k,
                                            (const float*)top_p);
  RET_LAUNCH;
}

int b200_softmax(const void* logits, int ld, void* out, int ldo, int n, int V, int log_mode,
                 cudaStream_t stream) {
  if (n <= 0) return 0;
  softmax_kernel<<<n, kSB, 0, stream>>>((const float*)logits, ld, (float*)out, ldo, V, log_mode);
  RET_LAUNCH;
}

int b200_random_sample(const void* probs, int ld, int n, int V, const void* seeds,
                       const void* steps, void* out_i64, cudaStream_t stream) {
  if (n <= 0) return 0;
  random_sample_kernel<<<n, kSB, 0, stream>>>((const float*)probs, ld, V, (const uint64_t*)seeds,
                                              (const uint64_t*)steps, (int64_t*)out_i64);
  RET_LAUNCH;
}

int b200_merge_greedy_random(const void* g, const void* r, const void* temp, void* out, int n,
                             cudaStream_t stream) {
  if (n <= 0) return 0;
  merge_greedy_random_kernel<<<(n + 255) / 256, 256, 0, stream>>>(
      (const int64_t*)g, (const int64_t*)r, (const float*)temp, (int64_t*)out, n);
  RET_LAUNCH;
}

int b200_token_rank(const void* logprobs, int ld, int n, int V, const void* toks, void* out_lp,
                    void* out_rank, cudaStream_t stream) {
  if (n <= 0) return 0;
  token_rank_kernel<<<n, kSB, 0, stream>>>((const float*)logprobs, ld, V, (const int64_t*)toks,
                                           (float*)out_lp, (int*)out_rank);
  RET_LAUNCH;
}

int b200_greedy_reject(const void* target_argmax, const void* draft, const void* cu_draft, int n,
                       int max_spec, void* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  greedy_reject_kernel<<<(n + 127) / 128, 128, 0, stream>>>(
      (const int64_t*)target_argmax, (const int64_t*)draft, (const int*)cu_draft, n, max_spec,
      (int64_t*)out);
  RET_LAUNCH;
}

int b200_splice_sampled(void* input_ids, const void* dst_idx, const void* src_row,
                        const void* last_sampled, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  splice_sampled_kernel<<<(n + 255) / 256, 256, 0, stream>>>(
      (int64_t*)input_ids, (const int*)dst_idx, (const int*)src_row, (const int64_t*)last_sampled,
      n);
  RET_LAUNCH;
}
int b200_scatter_sampled(void* last_sampled, const void* row_of, const void* sampled, int n,
                         cudaStream_t stream) {
  if (n <= 0) return 0;
  scatter_sampled_kernel<<<(n + 255) / 256, 256, 0, stream>>>(
      (int64_t*)last_sampled, (const int*)row_of, (const int64_t*)sampled, n);
  RET_LAUNCH;
}

uint64_t b200_splitmix64(uint64_t z) { return splitmix64(z); }

}  // extern "C"
