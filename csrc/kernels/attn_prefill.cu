// Paged flash-attention prefill on tcgen05 / TMEM (varlen, causal with bottom-right
// alignment, GQA, sliding window, soft-cap), head_dim 64 or 128.
//
// One CTA = one 128-row query tile of one request and one query head. Per 128-token KV
// tile:  S = Q K^T  (tcgen05, A = Q smem, B = K smem, both K-major SW128, fp32 S in TMEM),
// softmax with one thread per query row (TMEM lane == row, so no cross-thread reductions),
// P written to smem as bf16 in the UMMA K-major swizzled layout, then  PV = P V  with V as
// an MN-major operand (the pages land in smem exactly as they sit in the cache, d
// contiguous). QK^T of tile j+1 and PV of tile j-1 run on the tensor pipe while the softmax
// warps work on tile j; S is double-buffered in TMEM; O lives in registers and is
// rescaled when the running max moves.
//
// K/V pages are fetched with 3-D TMA boxes (64 dims x 1 head x min(block_size,128) tokens)
// straight from the paged cache [num_blocks, 2, block_size, Hkv, D].
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
static constexpr int kKT = 128;   // kv tokens per tile

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
  float softcap;               // 0 = off
  int window;                  // sliding window (tokens to the left incl. self), 0 = off
  int causal;
  int* status;
};

struct alignas(8) PrefillBars {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full, p_empty, o_full, o_empty;
  uint32_t tmem_base;
};

template <int D>
__global__ void __launch_bounds__(192, 1)
    attn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ,
                        const __grid_constant__ CUtensorMap tmKV, PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  constexpr int kDH = D / 64;                  // 64-wide halves of the head dim
  constexpr int kHalfBytes = 128 * 128;        // 128 rows x 128 B
  constexpr int kQBytes = kDH * kHalfBytes;
  constexpr int kKVBytes = kDH * kHalfBytes;   // one K or V stage
  constexpr int kPBytes = 2 * kHalfBytes;      // 128 x 128 bf16
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kQBytes;                  // 2 stages
  uint8_t* sV = sK + 2 * kKVBytes;             // 2 stages
  uint8_t* sP = sV + 2 * kKVBytes;
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
  const int kt0 = first_pos / kKT;
  const int kt1 = last_pos / kKT + 1;           // exclusive
  const int ntiles = kt1 - kt0;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->k_full[i], 1);
      mbar_init(&bars->k_empty[i], 1);
      mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->v_empty[i], 1);
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->s_empty[i], 4);
    }
    mbar_init(&bars->p_full, 4);
    mbar_init(&bars->p_empty, 1);
    mbar_init(&bars->o_full, 1);
    mbar_init(&bars->o_empty, 4);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t tmem_s0 = tmem_base, tmem_o = tmem_base + 256;

  const int rows_per_load = min(p.block_size, kKT);
  const int loads_per_tile = kKT / rows_per_load;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmKV);
      mbar_expect_tx(&bars->q_full, kQBytes);
      for (int dh = 0; dh < kDH; ++dh)
        tma_load_2d(sQ + dh * kHalfBytes, &tmQ, &bars->q_full, h * D + dh * 64, q_begin + q0);
      const int32_t* bt = p.block_table + (size_t)req * p.max_blocks;
      const int nblk_valid = (seq_len + p.block_size - 1) / p.block_size;
      bool ok = true;
      for (int j = 0; j < ntiles && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int tok0 = (kt0 + j) * kKT;
        // K then V for this tile
        for (int kv = 0; kv < 2 && ok; ++kv) {
          uint64_t* full = kv ? &bars->v_full[st] : &bars->k_full[st];
          uint64_t* empty = kv ? &bars->v_empty[st] : &bars->k_empty[st];
          if (!mbar_wait(empty, ph ^ 1, p.status)) { ok = false; break; }
          uint8_t* dst = (kv ? sV : sK) + st * kKVBytes;
          mbar_expect_tx(full, kKVBytes);
          for (int l = 0; l < loads_per_tile; ++l) {
            const int tok = tok0 + l * rows_per_load;
            int bi = tok / p.block_size;
            const int off = tok % p.block_size;
            int blk = (bi < nblk_valid) ? bt[bi] : bt[0];
            const int row = (blk * 2 + kv) * p.block_size + off;
            for (int dh = 0; dh < kDH; ++dh)
              tma_load_3d(dst + dh * kHalfBytes + l * rows_per_load * 128, &tmKV, full, dh * 64,
                          hkv, row);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(kQT, kKT, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(kQT, D, 0, 1);  // B (V) is MN-major
      bool ok = mbar_wait(&bars->q_full, 0, p.status);
      for (int j = 0; j <= ntiles && ok; ++j) {
        if (j < ntiles) {
          const int st = j & 1;
          const uint32_t ph = (j >> 1) & 1;
          if (!mbar_wait(&bars->k_full[st], ph, p.status)) { ok = false; break; }
          if (!mbar_wait(&bars->s_empty[st], ph ^ 1, p.status)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK + st * kKVBytes);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk / 4) * kHalfBytes + (kk % 4) * 32;
            umma_bf16_ss(tmem_s0 + st * 128, umma_desc_k_sw128(q_addr + off, 1024),
                         umma_desc_k_sw128(k_addr + off, 1024), idesc_qk, kk != 0);
          }
          umma_commit(&bars->k_empty[st]);
          umma_commit(&bars->s_full[st]);
        }
        if (j >= 1) {
          const int i = j - 1;
          const int st = i & 1;
          const uint32_t ph = (i >> 1) & 1;
          if (!mbar_wait(&bars->v_full[st], ph, p.status)) { ok = false; break; }
          if (!mbar_wait(&bars->p_full, i & 1, p.status)) { ok = false; break; }
          if (!mbar_wait(&bars->o_empty, (i & 1) ^ 1, p.status)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t p_addr = smem_u32(sP), v_addr = smem_u32(sV + st * kKVBytes);
#pragma unroll
          for (int kk = 0; kk < kKT / 16; ++kk) {
            const uint32_t poff = (kk / 4) * kHalfBytes + (kk % 4) * 32;
            // V: MN-major; 64-dim blocks are kHalfBytes apart, 8-token groups 1024 B apart,
            // 16 tokens per instruction = 2048 B.
            umma_bf16_ss(tmem_o, umma_desc_k_sw128(p_addr + poff, 1024),
                         umma_desc_mn_sw128(v_addr + kk * 2048, kHalfBytes, 1024), idesc_pv,
                         kk != 0);
          }
          umma_commit(&bars->v_empty[st]);
          umma_commit(&bars->p_empty);
          umma_commit(&bars->o_full);
        }
      }
    }
  } else {
    // ---------------- softmax + output: one thread per query row ----------------
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;              // row inside the tile
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const int q_pos = ctx_off + q0 + r;             // absolute position of this query row
    const int lo = (p.window > 0) ? (q_pos - p.window + 1) : 0;
    const int hi = p.causal ? q_pos : (seq_len - 1);
    float m = -INFINITY, l = 0.f, alpha_prev = 1.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[st], ph, p.status));
      if (!ok) break;
      tc_fence_after_sync();
      const int kbase = (kt0 + j) * kKT;
      const uint32_t s_addr = tmem_s0 + st * 128 + lane_off;
      const bool need_mask = (kbase + kKT - 1 > hi) || (kbase < lo) || (kbase + kKT > seq_len);
      // pass 1: row max
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kKT / 32; ++c) {
        uint32_t rr[32];
        tmem_ld_32x32b_x32(s_addr + c * 32, rr);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(rr[i]);
          if (p.softcap > 0.f) s = p.softcap * tanhf(s * (p.scale_log2 * 0.6931471805599453f) / p.softcap) / (p.scale_log2 * 0.6931471805599453f);
          const int kp = kbase + c * 32 + i;
          if (need_mask && (kp > hi || kp < lo || kp >= seq_len)) s = -INFINITY;
          mx = fmaxf(mx, s);
        }
      }
      const float m_new = fmaxf(m, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = (m_new == -INFINITY) ? 1.f : exp2f((m - m_new) * p.scale_log2);
      // P buffer must be free (PV of tile j-1 finished reading it)
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->p_empty, (j & 1) ^ 1, p.status));
      if (!ok) break;
      // pass 2: p = exp2((s - m) * scale), row sum, write bf16 P into the swizzled tile
      float rs = 0.f;
      const float moff = m_use * p.scale_log2;
#pragma unroll 1
      for (int c = 0; c < kKT / 32; ++c) {
        uint32_t rr[32];
        tmem_ld_32x32b_x32(s_addr + c * 32, rr);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float s0 = __uint_as_float(rr[i]), s1 = __uint_as_float(rr[i + 1]);
          if (p.softcap > 0.f) {
            const float sc = p.scale_log2 * 0.6931471805599453f;
            s0 = p.softcap * tanhf(s0 * sc / p.softcap) / sc;
            s1 = p.softcap * tanhf(s1 * sc / p.softcap) / sc;
          }
          const int kp = kbase + c * 32 + i;
          float p0 = exp2f(s0 * p.scale_log2 - moff), p1 = exp2f(s1 * p.scale_log2 - moff);
          if (need_mask) {
            if (kp > hi || kp < lo || kp >= seq_len) p0 = 0.f;
            if (kp + 1 > hi || kp + 1 < lo || kp + 1 >= seq_len) p1 = 0.f;
          }
          // Sum what the tensor core will see (bf16-rounded) so rows renormalise exactly.
          const uint32_t pp = pack_bf16x2(p0, p1);
          const float2 pr = unpack_bf16x2(pp);
          rs += pr.x + pr.y;
          pk[i >> 1] = pp;
        }
        // 32 columns = 4 chunks of 16 B in half-tile (c / 2), chunk ids (c & 1) * 4 + 0..3
        uint8_t* half = sP + (c >> 1) * kHalfBytes + r * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = ((c & 1) * 4 + q) ^ (r & 7);
          *reinterpret_cast<uint4*>(half + chunk * 16) =
              make_uint4(pk[q * 4 + 0], pk[q * 4 + 1], pk[q * 4 + 2], pk[q * 4 + 3]);
        }
      }
      l = l * alpha + rs;
      m = m_new;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars->p_full);
        mbar_arrive(&bars->s_empty[st]);
      }
      // deferred accumulate of PV_{j-1}
      if (j >= 1) {
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full, (j - 1) & 1, p.status));
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t rr[32];
          tmem_ld_32x32b_x32(tmem_o + lane_off + c * 32, rr);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            o[c * 32 + i] = o[c * 32 + i] * alpha_prev + __uint_as_float(rr[i]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->o_empty);
      }
      alpha_prev = alpha;
    }
    if (ok && ntiles > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full, (ntiles - 1) & 1, p.status));
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t rr[32];
          tmem_ld_32x32b_x32(tmem_o + lane_off + c * 32, rr);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i)
            o[c * 32 + i] = o[c * 32 + i] * alpha_prev + __uint_as_float(rr[i]);
        }
      }
    }
    if (ok && r < rows) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* dst = p.out + (size_t)(q_begin + q0 + r) * p.ldo + h * D;
#pragma unroll
      for (int i = 0; i < D; i += 8) {
        uint4 w;
        w.x = pack_bf16x2(o[i + 0] * inv, o[i + 1] * inv);
        w.y = pack_bf16x2(o[i + 2] * inv, o[i + 3] * inv);
        w.z = pack_bf16x2(o[i + 4] * inv, o[i + 5] * inv);
        w.w = pack_bf16x2(o[i + 6] * inv, o[i + 7] * inv);
        *reinterpret_cast<uint4*>(dst + i) = w;
      }
      if (p.lse) {
        const float ln2 = 0.6931471805599453f;
        p.lse[(size_t)(q_begin + q0 + r) * p.Hq + h] =
            l > 0.f ? (m * p.scale_log2 + log2f(l)) * ln2 : -INFINITY;
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
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

}  // namespace b200

using namespace b200;

extern "C" int b200_attn_prefill(const void* q, int ldq, void* out, int ldo, void* lse,
                                 const void* kv_cache, int64_t num_blocks, int block_size, int Hq,
                                 int Hkv, int D, const void* block_table, int max_blocks,
                                 const void* seq_lens, const void* q_start, const void* tile_req,
                                 const void* tile_q0, int num_tiles, int total_q, float scale,
                                 float softcap, int window, int causal, cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (D != 64 && D != 128) return -1;
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
  p.softcap = softcap; p.window = window; p.causal = causal;
  p.status = device_status_word();
  dim3 grid(num_tiles, Hq);
  if (D == 128) {
    constexpr size_t smem = (size_t)(2 + 4 * 2 + 2) * 16384 + 1024 + sizeof(PrefillBars);
    static bool set = false;
    if (!set) {
      cudaFuncSetAttribute(attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem);
      set = true;
    }
    attn_prefill_kernel<128><<<grid, 192, smem, stream>>>(tmQ, tmKV, p);
  } else {
    constexpr size_t smem = (size_t)(1 + 4 * 1 + 2) * 16384 + 1024 + sizeof(PrefillBars);
    static bool set = false;
    if (!set) {
      cudaFuncSetAttribute(attn_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem);
      set = true;
    }
    attn_prefill_kernel<64><<<grid, 192, smem, stream>>>(tmQ, tmKV, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
