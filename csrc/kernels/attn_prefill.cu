// Paged flash-attention prefill on tcgen05 / TMEM (varlen, causal with bottom-right
// alignment, GQA, sliding window, soft-cap), head_dim 64, 128 or 256.
//
// One CTA = one 128-row query tile of one request and one query head; two CTAs share an SM.
// Per 64-token KV tile:  S = Q K^T  (tcgen05, A = Q smem, B = K smem, both K-major SW128,
// fp32 S in TMEM), softmax with one thread per query row (TMEM lane == row, so no
// cross-thread reductions), P written to smem as bf16 in the UMMA K-major swizzled layout,
// then  PV = P V  with V as an MN-major operand (the pages land in smem exactly as they sit
// in the cache, d contiguous). QK^T of tile j+1 and PV of tile j-1 run on the tensor pipe
// while the softmax warps work on tile j; S is double-buffered in TMEM; O is accumulated in
// TMEM by the tensor pipe and rescaled in place only when a row's reference max is raised
// (lazily, by more than 2^8).
//
// K and V tiles share one ring of three TMA slots, filled in the order the MMA warp consumes them
// (K0 K1 V0 K2 V1 ...); pages are fetched with 3-D TMA boxes
// (64 dims x 1 head x min(block_size, 64) tokens) straight from the paged cache
// [num_blocks, 2, block_size, Hkv, D].
//
// Warp roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer + TMEM owner,
// warps 2..5 softmax + output.
//
// Replaces the reference prefill ladder (src/vt/cuda/cuda_paged_attn.cu:567 PagedFlashKernel,
// :720-1686 wmma variants, and the vendored FA2 path cuda_flash_attn_fa2.cu), none of which
// has an sm_100 tensor-core body.
#include <mutex>
#include <unordered_map>

#include "api.h"
#include "sm100.cuh"

namespace b200 {

static constexpr int kQT = 128;   // query rows per CTA
static constexpr int kKT = 64;    // kv tokens per tile
static constexpr int kRing = 3;   // K/V slots

struct PrefillParams {
  __nv_bfloat16* out;   // [T, Hq*D]
  int ldo;
  float* lse;           // optional [T, Hq] natural-log LSE
  const int32_t* block_table;  // [B, max_blocks]
  int max_blocks;
  const int32_t* seq_lens;     // [B]
  const int32_t* q_start;      // [B+1]
  const int32_t* tile_req;     // [num_tiles]
  const int32_t* tile_q0;      // [num_tiles] first query row of the tile inside its request
  int Hq, Hkv, block_size;
  float scale_log2;            // softmax scale * log2(e)
  float softcap2;              // soft-cap in the log2 domain, 0 = off
  int window;                  // > 0: sliding window (tokens to the left incl. self); < 0: chunked-local
                               // attention with chunks of -window tokens (a query sees its own chunk); 0 = off
  int causal;
  int* status;
};

struct alignas(8) PrefillBars {
  uint64_t q_full;
  uint64_t kv_full[kRing], kv_empty[kRing];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, p_empty, o_full;
  uint32_t tmem_base;
};

__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


// D = 256 keeps two softmax threads per query row (warps w and w + 4 share a TMEM lane
// quarter): both reduce the full score row, each writes half of P and owns half of O.
template <int D>
__global__ void __launch_bounds__(64 + 128 * (D > 128 ? 2 : 1), D > 128 ? 1 : 2)
    attn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ,
                        const __grid_constant__ CUtensorMap tmKV, PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  constexpr int kDH = D / 64;                     // 64-wide halves of the head dim
  constexpr int kSplit = D > 128 ? 2 : 1;         // softmax threads per query row
  constexpr int kDO = D / kSplit;                 // output dims owned by one thread
  constexpr uint32_t kTmemCols = D > 128 ? 512 : 256;
  constexpr int kQHalf = kQT * 128;               // 16 KB: 128 rows x 128 B
  constexpr int kKVHalf = kKT * 128;              // 8 KB: 64 tokens x 128 B
  constexpr int kQBytes = kDH * kQHalf;
  constexpr int kSlotBytes = kDH * kKVHalf;       // one K or V tile
  constexpr int kPBytes = kQT * kKT * 2;          // 16 KB: one K-major half-tile
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + kQBytes;
  uint8_t* sP = sKV + kRing * kSlotBytes;
  PrefillBars* bars = reinterpret_cast<PrefillBars*>(sP + kPBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x, h = blockIdx.y;
  const int hkv = h / (p.Hq / p.Hkv);
  const int req = p.tile_req[tile];
  const int q0 = p.tile_q0[tile];
  const int q_begin = p.q_start[req];
  const int q_len = p.q_start[req + 1] - q_begin;
  const int seq_len = p.seq_lens[req];
  const int ctx_off = seq_len - q_len;          // position of query row 0
  const int rows = min(kQT, q_len - q0);
  // kv range needed by this tile
  const int last_pos = p.causal ? (ctx_off + q0 + rows - 1) : (seq_len - 1);
  int first_pos = 0;
  if (p.window > 0) first_pos = max(0, ctx_off + q0 - p.window + 1);
  else if (p.window < 0) first_pos = ((ctx_off + q0) / -p.window) * -p.window;   // chunk start of the first row
  const int kt0 = first_pos / kKT;
  const int kt1 = last_pos / kKT + 1;           // exclusive
  const int ntiles = kt1 - kt0;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&bars->kv_full[i], 1);
      mbar_init(&bars->kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->s_empty[i], 4 * kSplit);
    }
    mbar_init(&bars->p_full, 4 * kSplit);
    mbar_init(&bars->p_empty, 1);
    mbar_init(&bars->o_full, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t tmem_s0 = tmem_base, tmem_o = tmem_base + 128;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmKV);
      mbar_expect_tx(&bars->q_full, kQBytes);
      for (int dh = 0; dh < kDH; ++dh)
        tma_load_2d(sQ + dh * kQHalf, &tmQ, &bars->q_full, h * D + dh * 64, q_begin + q0);
      const int32_t* bt = p.block_table + (size_t)req * p.max_blocks;
      const int nblk_valid = (seq_len + p.block_size - 1) / p.block_size;
      const int rows_per_load = min(p.block_size, kKT);
      const int loads = kKT / rows_per_load;
      bool ok = true;
      // Load order K0 K1 V0 K2 V1 K3 ... V(n-1): the order in which the MMA warp consumes the
      // tiles, with K one tile further ahead than V (V slots are held until the softmax of their
      // tile is done; K slots turn over as soon as QK^T has run).
      const int nseq = 2 * ntiles;
      for (int sq = 0; sq < nseq && ok; ++sq) {
        int kv, j;
        if (sq == 0) { kv = 0; j = 0; }
        else if (sq == nseq - 1) { kv = 1; j = ntiles - 1; }
        else if (sq & 1) { kv = 0; j = (sq + 1) >> 1; }
        else { kv = 1; j = (sq - 2) >> 1; }
        const int tok0 = (kt0 + j) * kKT;
        const int sl = sq % kRing;
        const uint32_t ph = (sq / kRing) & 1;
        if (!mbar_wait(&bars->kv_empty[sl], ph ^ 1, p.status)) { ok = false; break; }
        uint8_t* dst = sKV + sl * kSlotBytes;
        mbar_expect_tx(&bars->kv_full[sl], kSlotBytes);
        for (int l = 0; l < loads; ++l) {
          const int tk = tok0 + l * rows_per_load;
          const int bi = tk / p.block_size;
          int blk = (bi < nblk_valid) ? bt[bi] : bt[0];
          if (blk < 0) blk = 0;
          const int row = (blk * 2 + kv) * p.block_size + tk % p.block_size;
          for (int dh = 0; dh < kDH; ++dh)
            tma_load_3d(dst + dh * kKVHalf + l * rows_per_load * 128, &tmKV, &bars->kv_full[sl],
                        dh * 64, hkv, row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(kQT, kKT, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(kQT, D, 0, 1);  // B (V) is MN-major
      bool ok = mbar_wait(&bars->q_full, 0, p.status);
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      for (int j = 0; j <= ntiles && ok; ++j) {
        if (j < ntiles) {
          const int it = j == 0 ? 0 : 2 * j - 1, sl = it % kRing, sb = j & 1;   // K(j) in load order
          if (!mbar_wait(&bars->kv_full[sl], (it / kRing) & 1, p.status)) { ok = false; break; }
          if (!mbar_wait(&bars->s_empty[sb], ((j >> 1) & 1) ^ 1, p.status)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t k_addr = smem_u32(sKV + sl * kSlotBytes);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            umma_bf16_ss(tmem_s0 + sb * kKT,
                         umma_desc_k_sw128(q_addr + (kk / 4) * kQHalf + (kk % 4) * 32, 1024),
                         umma_desc_k_sw128(k_addr + (kk / 4) * kKVHalf + (kk % 4) * 32, 1024),
                         idesc_qk, kk != 0);
          }
          umma_commit(&bars->kv_empty[sl]);
          umma_commit(&bars->s_full[sb]);
        }
        if (j >= 1) {
          const int i = j - 1;
          const int it = i == ntiles - 1 ? 2 * ntiles - 1 : 2 * i + 2, sl = it % kRing;       // V(i)
          if (!mbar_wait(&bars->kv_full[sl], (it / kRing) & 1, p.status)) { ok = false; break; }
          if (!mbar_wait(&bars->p_full, i & 1, p.status)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t v_addr = smem_u32(sKV + sl * kSlotBytes);
#pragma unroll
          for (int kk = 0; kk < kKT / 16; ++kk) {
            // V: MN-major; 64-dim blocks are kKVHalf apart, 8-token groups 1024 B apart,
            // 16 tokens per instruction = 2048 B.
            umma_bf16_ss(tmem_o, umma_desc_k_sw128(p_addr + kk * 32, 1024),
                         umma_desc_mn_sw128(v_addr + kk * 2048, kKVHalf, 1024), idesc_pv, (i | kk) != 0);
          }
          umma_commit(&bars->kv_empty[sl]);
          umma_commit(&bars->o_full);     // before p_empty: whoever sees p_empty has this arrival too
          umma_commit(&bars->p_empty);
        }
      }
    }
  } else {
    // ---------------- softmax + output: one thread per query row ----------------
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;               // which half of P / O this thread owns
    const int r = quarter * 32 + lane;              // row inside the tile
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const int q_pos = ctx_off + q0 + r;             // absolute position of this query row
    const int lo = (p.window > 0) ? (q_pos - p.window + 1) : (p.window < 0 ? (q_pos / -p.window) * -p.window : 0);
    const int hi = min(p.causal ? q_pos : (seq_len - 1), seq_len - 1);
    const float sc = p.scale_log2;
    const bool cap = p.softcap2 > 0.f;
    // m: reference maximum of the row in the scaled log2 domain. It is raised lazily: only when a
    // tile exceeds it by more than 2^8, so P stays below 256 and the rescale of O is rare. O is
    // accumulated by the tensor pipe in TMEM across tiles; a raise rescales this thread's row of
    // O in place (TMEM lane == query row, so no other thread is involved).
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    uint8_t* prow = sP + r * 128;
    for (int j = 0; j < ntiles && ok; ++j) {
      const int sb = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[sb], (j >> 1) & 1, p.status));
      if (!ok) break;
      tc_fence_after_sync();
      const int kbase = (kt0 + j) * kKT;
      const uint32_t s_addr = tmem_s0 + sb * kKT + lane_off;
      const bool need_mask = (kbase + kKT - 1 > hi) || (kbase < lo);
      uint32_t s0[32], s1[32];
      tmem_ld_32x32b_x32(s_addr, s0);
      tmem_ld_32x32b_x32(s_addr + 32, s1);
      tmem_ld_wait();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->s_empty[sb]);   // S is in registers now
      // scaled scores (log2 domain), soft-cap, mask
      if (cap || need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float a = __uint_as_float(s0[i]) * sc, b = __uint_as_float(s1[i]) * sc;
          if (cap) {
            a = p.softcap2 * tanhf(a / p.softcap2);
            b = p.softcap2 * tanhf(b / p.softcap2);
          }
          const int ka = kbase + i, kb = kbase + 32 + i;
          if (ka > hi || ka < lo) a = -INFINITY;
          if (kb > hi || kb < lo) b = -INFINITY;
          s0[i] = __float_as_uint(a);
          s1[i] = __float_as_uint(b);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          s0[i] = __float_as_uint(__uint_as_float(s0[i]) * sc);
          s1[i] = __float_as_uint(__uint_as_float(s1[i]) * sc);
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        mx0 = fmaxf(mx0, __uint_as_float(s0[i]));
        mx1 = fmaxf(mx1, __uint_as_float(s1[i]));
      }
      const float tile_max = fmaxf(mx0, mx1);
      float alpha = 1.f;
      bool rescale = false;
      if (tile_max > m + 8.f) {          // also the first finite tile: m == -inf
        if (m != -INFINITY) {
          alpha = ex2_fast(m - tile_max);
          rescale = j > 0;
        }
        m = tile_max;
      }
      const float m_use = (m == -INFINITY) ? 0.f : m;
      // PV of tile j-1 has completed: the P buffer is free and O holds every product so far
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->p_empty, (j & 1) ^ 1, p.status));
      if (!ok) break;
      if (__any_sync(0xffffffffu, rescale)) {
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < kDO / 32; ++c) {
          uint32_t rr[32];
          tmem_ld_32x32b_x32(tmem_o + lane_off + part * kDO + c * 32, rr);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) rr[i] = __float_as_uint(__uint_as_float(rr[i]) * alpha);
          tmem_st_32x32b_x32(tmem_o + lane_off + part * kDO + c * 32, rr);
        }
        tmem_st_wait();
      }
      float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {     // 8 chunks of 8 columns = 16 bytes each
        uint32_t pk[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = (c & 3) * 8 + e * 2;
          const float x0 = __uint_as_float(c < 4 ? s0[i] : s1[i]);
          const float x1 = __uint_as_float(c < 4 ? s0[i + 1] : s1[i + 1]);
          const float p0 = ex2_fast(x0 - m_use), p1 = ex2_fast(x1 - m_use);
          rs0 += p0;
          rs1 += p1;
          pk[e] = pack_bf16x2(p0, p1);
        }
        if (kSplit == 1 || (c >> 2) == part)
          *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l = l * alpha + (rs0 + rs1);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full);
    }
    if (ok && ntiles > 0) {
      // o_full completes once per PV; p_empty of the last iteration showed PV(ntiles-2) complete,
      // so this parity wait can only be satisfied by the last product
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full, (ntiles - 1) & 1, p.status));
      if (ok) tc_fence_after_sync();
    }
    if (ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (size_t)(q_begin + q0 + r) * p.ldo + h * D + part * kDO;
#pragma unroll
      for (int c = 0; c < kDO / 32; ++c) {
        uint32_t rr[32];
        if (ntiles > 0) {
          tmem_ld_32x32b_x32(tmem_o + lane_off + part * kDO + c * 32, rr);   // (whole warp)
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) rr[i] = 0;
        }
        if (r < rows) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(rr[i + 0]) * inv, __uint_as_float(rr[i + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(rr[i + 2]) * inv, __uint_as_float(rr[i + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(rr[i + 4]) * inv, __uint_as_float(rr[i + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(rr[i + 6]) * inv, __uint_as_float(rr[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = w;
          }
        }
      }
    }
    if (ok && r < rows) {
      if (p.lse && part == 0) {
        const float ln2 = 0.6931471805599453f;
        p.lse[(size_t)(q_begin + q0 + r) * p.Hq + h] = l > 0.f ? (m + log2f(l)) * ln2 : -INFINITY;
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

struct KvMapKey {
  const void* p;
  uint64_t rows;
  int hkv, d, box_rows;
  bool operator==(const KvMapKey& o) const {
    return p == o.p && rows == o.rows && hkv == o.hkv && d == o.d && box_rows == o.box_rows;
  }
};
struct KvMapKeyHash {
  size_t operator()(const KvMapKey& k) const {
    return reinterpret_cast<size_t>(k.p) ^ (k.rows * 0x9e3779b97f4a7c15ull) ^
           ((size_t)k.hkv << 40) ^ ((size_t)k.d << 20) ^ (size_t)k.box_rows;
  }
};

template <int D>
static int launch_prefill(const CUtensorMap& tmQ, const CUtensorMap& tmKV, const PrefillParams& p,
                          dim3 grid, cudaStream_t stream) {
  constexpr int kDH = D / 64;
  constexpr size_t smem = (size_t)kDH * 16384 + (size_t)kRing * kDH * 8192 + 16384 + 1024 +
                          sizeof(PrefillBars);
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(attn_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)smem);
  }
  attn_prefill_kernel<D><<<grid, 64 + 128 * (D > 128 ? 2 : 1), smem, stream>>>(tmQ, tmKV, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace b200

using namespace b200;


extern "C" int b200_attn_prefill(const void* q, int ldq, void* out, int ldo, void* lse,
                                 const void* kv_cache, int64_t num_blocks, int block_size, int Hq,
                                 int Hkv, int D, const void* block_table, int max_blocks,
                                 const void* seq_lens, const void* q_start, const void* tile_req,
                                 const void* tile_q0, int num_tiles, int total_q, float scale,
                                 float softcap, int window, int causal, cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (D != 64 && D != 128 && D != 256) return -1;
  if (block_size < 8 || (block_size & 7) || (block_size < kKT && kKT % block_size) ||
      (block_size > kKT && block_size % kKT))
    return -1;
  if ((ldq & 7) || (ldo & 7) || Hq % Hkv) return -1;
  static std::mutex mu;
  static std::unordered_map<KvMapKey, CUtensorMap, KvMapKeyHash> kv_cache_maps;
  CUtensorMap tmQ, tmKV;
  if (!encode_tmap_2d(&tmQ, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)total_q,
                      (uint64_t)Hq * D, (uint64_t)ldq, kQT, 64, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  const int box_rows = block_size < kKT ? block_size : kKT;
  const uint64_t rows = (uint64_t)num_blocks * 2 * block_size;
  {
    KvMapKey key{kv_cache, rows, Hkv, D, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = kv_cache_maps.find(key);
    if (it == kv_cache_maps.end()) {
      if (kv_cache_maps.size() > 4096) kv_cache_maps.clear();   // scratch caches come and go
      CUtensorMap m;
      if (!encode_tmap_3d(&m, kv_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)D,
                          (uint64_t)Hkv, rows, (uint64_t)D * 2, (uint64_t)Hkv * D * 2, 64, 1,
                          (uint32_t)box_rows, CU_TENSOR_MAP_SWIZZLE_128B))
        return -3;
      it = kv_cache_maps.emplace(key, m).first;
    }
    tmKV = it->second;
  }
  PrefillParams p;
  p.out = (__nv_bfloat16*)out; p.ldo = ldo; p.lse = (float*)lse;
  p.block_table = (const int32_t*)block_table; p.max_blocks = max_blocks;
  p.seq_lens = (const int32_t*)seq_lens; p.q_start = (const int32_t*)q_start;
  p.tile_req = (const int32_t*)tile_req; p.tile_q0 = (const int32_t*)tile_q0;
  p.Hq = Hq; p.Hkv = Hkv; p.block_size = block_size;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.softcap2 = softcap * 1.4426950408889634f;
  p.window = window; p.causal = causal;
  p.status = device_status_word();
  dim3 grid(num_tiles, Hq);
  if (D == 256) return launch_prefill<256>(tmQ, tmKV, p, grid, stream);
  return D == 128 ? launch_prefill<128>(tmQ, tmKV, p, grid, stream)
                  : launch_prefill<64>(tmQ, tmKV, p, grid, stream);
}
