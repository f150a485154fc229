// Paged decode attention on tcgen05 with swapped operands (head_dim 128 or 256, GQA group <= 16).
//
// One CTA = one (sequence, kv head, kv split). The KV stream is the 128-row MMA operand and
// the few query heads that share the kv head are the narrow N operand, so every K/V byte is
// fetched once by TMA and the tensor pipe does all the dot products:
//
//   S^T[128 tok, 16] = K[128 tok, D] * Q[16, D]^T          (K: K-major A, Q: K-major B)
//   softmax along tokens: TMEM lane == token, so each of the 128 softmax threads owns one
//   token and the per-head max / sum are warp shuffles + a 4-entry smem exchange
//   O^T[D, 16]      += V^T[D, 128 tok] * P^T[16, 128 tok]^T (V: MN-major A straight from the
//                                                            cache layout, P^T: K-major B)
//
// O^T stays in TMEM across tiles (16 fp32 columns); the running max is raised lazily (only
// when a tile exceeds it by more than 2^8), and raising it rescales those 16 columns in
// place. K and V tiles share one TMA ring of 128 x D bf16 slots, filled in the order the MMA warp
// consumes them (K0 K1 V0 K2 V1 ...); two CTAs fit on an SM at head_dim 128. At head_dim 256 the
// P V product runs as two M = 128 instructions (one per half of the head dim), O^T takes two
// 16-column accumulators and one CTA fits on an SM.
//
// Replaces the CUDA-core decode kernels of the reference
// (src/vt/cuda/cuda_paged_attn.cu:302 PagedAttentionDecodeOptKernel, :430 ...GqaKernel) and
// its FA2 split-KV decode launcher.
#include <mutex>
#include <unordered_map>

#include "api.h"
#include "sm100.cuh"

namespace b200 {

static constexpr int kTok = 128;        // tokens per tile
static constexpr int kNQ = 16;          // padded query heads (UMMA N)
static constexpr int kSlots = 3;        // K/V ring slots
template <int D>
struct DecodeTcSmem {
  static constexpr int slot_bytes = kTok * D * 2;      // one K or V tile
  static constexpr int q_bytes = (D / 64) * 2048;      // 16 query rows, 64-element chunks of 2 KB
  static constexpr int p_bytes = 8192;                 // 2 buffers x (2 token halves x 2 KB)
};

struct DecodeTcParams {
  __nv_bfloat16* out;
  int ldo;
  const int32_t* block_table;
  int max_blocks;
  const int32_t* seq_lens;
  int Hq, Hkv, block_size;
  float scale_log2, softcap2;  // softcap in the log2 domain (0 = off)
  int window, splits;
  float* tmp_o;
  float* tmp_lse;
  int* status;
};

struct alignas(8) DecodeTcBars {
  uint64_t q_full;
  uint64_t kv_full[kSlots], kv_empty[kSlots];
  uint64_t s_full[2], s_empty[2];
  uint64_t p_full[2], p_empty[2];
  uint64_t pv_done;
  uint64_t grp;
  uint32_t tmem_base;
  float red_max[2][4][kNQ];
  float red_sum[4][kNQ];
};

__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
      "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
      "r"(r[14]), "r"(r[15])
      : "memory");
}
// Sync of the 4 softmax warps through an mbarrier (count 4) so that, like every other wait
// in this kernel, it is bounded: a hardware named barrier would wait forever if one warp had
// left the loop after a timeout.
__device__ __forceinline__ bool softmax_group_sync(uint64_t* bar, uint32_t& phase, int lane,
                                                   int* status) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
  const bool ok = mbar_wait(bar, phase, status);
  phase ^= 1;
  return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


// GP: the GQA group size rounded up to 4 / 8 / 16; the softmax only touches those columns of
// S^T (the MMA's N stays 16, its minimum at 128 rows).
template <int GP, int D>
__global__ void __launch_bounds__(192, D == 128 ? 2 : 1)
    attn_decode_tc_kernel(const __grid_constant__ CUtensorMap tmQ,
                          const __grid_constant__ CUtensorMap tmKV, DecodeTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  constexpr int kSlotBytes = DecodeTcSmem<D>::slot_bytes;
  constexpr int kQBytes = DecodeTcSmem<D>::q_bytes;
  constexpr int kChunks = D / 64;                    // 64-element (128-byte) chunks of the head dim
  constexpr int kChunkBytes = kTok * 128;            // one chunk of a K / V tile: 128 tokens x 128 bytes
  uint8_t* sKV = smem;                               // kSlots tiles
  uint8_t* sQ = sKV + kSlots * kSlotBytes;           // kChunks x 2 KB
  uint8_t* sP = sQ + kQBytes;                        // 2 buffers * (2 halves * 2 KB)
  DecodeTcBars* bars = reinterpret_cast<DecodeTcBars*>(sP + 8192);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x, hkv = blockIdx.y, split = blockIdx.z;
  const int G = p.Hq / p.Hkv;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(&bars->kv_full[i], 1);
      mbar_init(&bars->kv_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->s_empty[i], 4);
      mbar_init(&bars->p_full[i], 4);
      mbar_init(&bars->p_empty[i], 1);
    }
    mbar_init(&bars->pv_done, 1);
    mbar_init(&bars->grp, 4);
    mbar_fence_init();
  }
  // zero the P^T buffers once: rows >= G are never written and must stay finite
  for (int i = threadIdx.x; i < 8192 / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(sP)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 64);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t tmem_s = tmem_base;        // 2 x 16 columns
  const uint32_t tmem_o = tmem_base + 32;   // 16 columns per 128 rows of the head dim

  // Everything above touches only shared memory and TMEM and may overlap the previous kernel.
  pdl_wait();
  pdl_launch_dependents();
  const int seq_len = p.seq_lens[b];
  int begin = 0;
  if (p.window > 0) begin = max(0, seq_len - p.window);
  else if (p.window < 0 && seq_len > 0) begin = ((seq_len - 1) / -p.window) * -p.window;   // chunked-local
  const int start = (begin / kTok) * kTok;           // tile-aligned start of the kv range
  const int span = max(0, seq_len - start);
  const int tiles_total = (span + kTok - 1) / kTok;
  const int tiles_per_split = (tiles_total + p.splits - 1) / p.splits;
  const int tile0 = split * tiles_per_split;
  const int ntiles = max(0, min(tiles_total, tile0 + tiles_per_split) - tile0);
  const int tok_base = start + tile0 * kTok;

  if (ntiles > 0) {
    if (warp == 0) {
      // ------------------------------ TMA producer ------------------------------
      if (lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmKV);
        mbar_expect_tx(&bars->q_full, kQBytes);
#pragma unroll
        for (int c = 0; c < kChunks; ++c) tma_load_3d(sQ + c * 2048, &tmQ, &bars->q_full, c * 64, hkv * G, b);
        const int32_t* bt = p.block_table + (size_t)b * p.max_blocks;
        const int nblk_valid = (seq_len + p.block_size - 1) / p.block_size;
        const int rows_per_load = min(p.block_size, kTok);
        const int loads = kTok / rows_per_load;
        bool ok = true;
        // Load order K0 K1 V0 K2 V1 K3 ... V(n-1): exactly the order in which the MMA warp
        // consumes the tiles, with K running one tile further ahead than V (a V slot is held
        // until the softmax of its tile is done; K slots turn over as soon as QK has run).
        const int nseq = 2 * ntiles;
        for (int sq = 0; sq < nseq && ok; ++sq) {
          int kv, j;
          if (sq == 0) { kv = 0; j = 0; }
          else if (sq == nseq - 1) { kv = 1; j = ntiles - 1; }
          else if (sq & 1) { kv = 0; j = (sq + 1) >> 1; }
          else { kv = 1; j = (sq - 2) >> 1; }
          const int tok0 = tok_base + j * kTok;
          const int sl = sq % kSlots;
          const uint32_t ph = (sq / kSlots) & 1;
          if (!mbar_wait(&bars->kv_empty[sl], ph ^ 1, p.status)) { ok = false; break; }
          uint8_t* dst = sKV + sl * kSlotBytes;
          mbar_expect_tx(&bars->kv_full[sl], kSlotBytes);
          for (int l = 0; l < loads; ++l) {
            const int tk = tok0 + l * rows_per_load;
            const int bi = tk / p.block_size;
            const int blk = (bi < nblk_valid) ? bt[bi] : bt[0];
            const int row = (blk * 2 + kv) * p.block_size + tk % p.block_size;
#pragma unroll
            for (int c = 0; c < kChunks; ++c)
              tma_load_3d(dst + c * kChunkBytes + l * rows_per_load * 128, &tmKV, &bars->kv_full[sl], c * 64, hkv,
                          row);
          }
        }
      }
    } else if (warp == 1) {
      // ------------------------------ MMA issuer ------------------------------
      if (lane == 0) {
        constexpr uint32_t idesc_qk = umma_idesc_bf16(kTok, kNQ, 0, 0);
        constexpr uint32_t idesc_pv = umma_idesc_bf16(128, kNQ, 1, 0);  // A (V^T) is MN-major
        bool ok = mbar_wait(&bars->q_full, 0, p.status);
        const uint32_t q_addr = smem_u32(sQ);
        for (int j = 0; j <= ntiles && ok; ++j) {
          if (j < ntiles) {
            const int it = j == 0 ? 0 : 2 * j - 1, sl = it % kSlots;     // K(j) in load order
            const uint32_t ph = (it / kSlots) & 1;
            const int sb = j & 1;
            if (!mbar_wait(&bars->kv_full[sl], ph, p.status)) { ok = false; break; }
            if (!mbar_wait(&bars->s_empty[sb], ((j >> 1) & 1) ^ 1, p.status)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t k_addr = smem_u32(sKV + sl * kSlotBytes);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t koff = (kk / 4) * kChunkBytes + (kk % 4) * 32;
              const uint32_t qoff = (kk / 4) * 2048 + (kk % 4) * 32;
              umma_bf16_ss(tmem_s + sb * 16, umma_desc_k_sw128(k_addr + koff, 1024),
                           umma_desc_k_sw128(q_addr + qoff, 1024), idesc_qk, kk != 0);
            }
            umma_commit(&bars->kv_empty[sl]);
            umma_commit(&bars->s_full[sb]);
          }
          if (j >= 1) {
            const int i = j - 1;
            const int it = i == ntiles - 1 ? 2 * ntiles - 1 : 2 * i + 2, sl = it % kSlots;  // V(i)
            const uint32_t ph = (it / kSlots) & 1;
            const int pb = i & 1;
            if (!mbar_wait(&bars->kv_full[sl], ph, p.status)) { ok = false; break; }
            if (!mbar_wait(&bars->p_full[pb], (i >> 1) & 1, p.status)) { ok = false; break; }
            tc_fence_after_sync();
            const uint32_t v_addr = smem_u32(sKV + sl * kSlotBytes);
            const uint32_t p_addr = smem_u32(sP + pb * 4096);
#pragma unroll
            for (int dh = 0; dh < D / 128; ++dh) {       // 128 rows of the head dim per instruction
#pragma unroll
              for (int kk = 0; kk < kTok / 16; ++kk) {
                const uint32_t poff = (kk / 4) * 2048 + (kk % 4) * 32;
                umma_bf16_ss(tmem_o + dh * 16,
                             umma_desc_mn_sw128(v_addr + dh * 2 * kChunkBytes + kk * 2048, kChunkBytes, 1024),
                             umma_desc_k_sw128(p_addr + poff, 1024), idesc_pv, (i | kk) != 0);
              }
            }
            umma_commit(&bars->kv_empty[sl]);
            umma_commit(&bars->pv_done);      // before p_empty: whoever sees p_empty has this arrival too
            umma_commit(&bars->p_empty[pb]);
          }
        }
      }
    } else {
      // ---------------- softmax / correction: thread t owns token t of the tile ----------------
      const int quarter = warp & 3;
      const int t = quarter * 32 + lane;
      const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
      float m[GP], lsum[GP];
#pragma unroll
      for (int g = 0; g < GP; ++g) { m[g] = -INFINITY; lsum[g] = 0.f; }
      const bool capped = p.softcap2 > 0.f;
      bool ok = true;
      uint32_t gphase = 0;
      for (int j = 0; j < ntiles && ok; ++j) {
        const int sb = j & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[sb], (j >> 1) & 1, p.status));
        if (!ok) break;
        tc_fence_after_sync();
        uint32_t r[16];
        tmem_ld_32x32b_x16(tmem_s + sb * 16 + lane_off, r);
        tmem_ld_wait();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->s_empty[sb]);
        const int tok = tok_base + j * kTok + t;
        const bool valid = tok < seq_len && tok >= begin;
        float s[GP];
#pragma unroll
        for (int g = 0; g < GP; ++g) {
          float v = __uint_as_float(r[g]) * p.scale_log2;
          if (capped) v = p.softcap2 * tanhf(v / p.softcap2);
          s[g] = valid ? v : -INFINITY;
        }
        // tile max per head over the 128 tokens: one warp reduction per head, then 4 partials
        {
          float wm[GP];
#pragma unroll
          for (int g = 0; g < GP; ++g) wm[g] = warp_max_f32(s[g]);
          if (lane == 0) {
#pragma unroll
            for (int g = 0; g < GP; ++g) bars->red_max[sb][quarter][g] = wm[g];
          }
        }
        ok = softmax_group_sync(&bars->grp, gphase, lane, p.status);
        if (!ok) break;
        bool rescale = false;
        float alpha[GP];
#pragma unroll
        for (int g = 0; g < GP; ++g) {
          const float tm = fmaxf(fmaxf(bars->red_max[sb][0][g], bars->red_max[sb][1][g]),
                                 fmaxf(bars->red_max[sb][2][g], bars->red_max[sb][3][g]));
          alpha[g] = 1.f;
          if (tm > m[g] + 8.f) {       // raise the reference max lazily (uniform across threads)
            if (m[g] != -INFINITY) {
              alpha[g] = fast_exp2(m[g] - tm);
              rescale = true;
            }
            m[g] = tm;
          }
        }
        // P^T buffer free? (PV of tile j-2 finished reading it.) This also bounds how far
        // pv_done can lag: it has completed at least j-1 times here, so the parity wait of the
        // rescale below (its j-th completion) cannot be satisfied by an older phase.
        const int pb = j & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->p_empty[pb], ((j >> 1) & 1) ^ 1, p.status));
        if (!ok) break;
        if (rescale && j > 0) {
          // all PV products issued so far must have landed before O^T is rescaled in place
          ok = __all_sync(0xffffffffu, mbar_wait(&bars->pv_done, (j - 1) & 1, p.status));
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int dh = 0; dh < D / 128; ++dh) {
            uint32_t o[16];
            tmem_ld_32x32b_x16(tmem_o + dh * 16 + lane_off, o);
            tmem_ld_wait();
#pragma unroll
            for (int g = 0; g < GP; ++g) o[g] = __float_as_uint(__uint_as_float(o[g]) * alpha[g]);
            tmem_st_32x32b_x16(tmem_o + dh * 16 + lane_off, o);
          }
          tmem_st_wait();
#pragma unroll
          for (int g = 0; g < GP; ++g) lsum[g] *= alpha[g];
        }
        uint8_t* pbuf = sP + pb * 4096 + (t >> 6) * 2048;
        const int c = t & 63;
#pragma unroll
        for (int g = 0; g < GP; ++g) {
          if (g < G) {
            const float pv = valid ? fast_exp2(s[g] - m[g]) : 0.f;
            const __nv_bfloat16 pb16 = __float2bfloat16(pv);
            lsum[g] += __bfloat162float(pb16);
            *reinterpret_cast<__nv_bfloat16*>(pbuf + g * 128 + (((c >> 3) ^ (g & 7)) << 4) +
                                              (c & 7) * 2) = pb16;
          }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full[pb]);
      }
      // ---------------- epilogue: O^T / l ----------------
      // pv_done completes once per tile and the loop only guarantees ntiles-2 completions seen
      // (through p_empty), so observe the last two in order: a parity wait two phases ahead
      // would be satisfied by the older phase.
      if (ok && ntiles >= 2)
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->pv_done, (ntiles - 2) & 1, p.status));
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->pv_done, (ntiles - 1) & 1, p.status));
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int g = 0; g < GP; ++g) {
          float v = lsum[g];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0) bars->red_sum[quarter][g] = v;
        }
        ok = softmax_group_sync(&bars->grp, gphase, lane, p.status);
      }
      if (ok) {
#pragma unroll
        for (int dh = 0; dh < D / 128; ++dh) {
          uint32_t o[16];
          tmem_ld_32x32b_x16(tmem_o + dh * 16 + lane_off, o);
          tmem_ld_wait();
          const int d = dh * 128 + t;  // TMEM lane of O^T = head dim index within its half
#pragma unroll
          for (int g = 0; g < GP; ++g) {
            if (g < G) {
              const float l = bars->red_sum[0][g] + bars->red_sum[1][g] + bars->red_sum[2][g] +
                              bars->red_sum[3][g];
              const float v = l > 0.f ? __uint_as_float(o[g]) / l : 0.f;
              const int hq = hkv * G + g;
              if (p.splits == 1) {
                p.out[(size_t)b * p.ldo + (size_t)hq * D + d] = __float2bfloat16(v);
              } else {
                const size_t row = ((size_t)b * p.Hq + hq) * p.splits + split;
                p.tmp_o[row * D + d] = v;
                if (d == 0) p.tmp_lse[row] = l > 0.f ? m[g] + log2f(l) : -INFINITY;
              }
            }
          }
        }
      }
    }
  } else if (warp >= 2) {
    // empty split (or empty sequence): neutral partial / zero output
    for (int d = (warp & 3) * 32 + lane; d < D; d += 128) {
      for (int g = 0; g < G; ++g) {
        const int hq = hkv * G + g;
        if (p.splits == 1) {
          p.out[(size_t)b * p.ldo + (size_t)hq * D + d] = __float2bfloat16(0.f);
        } else {
          const size_t row = ((size_t)b * p.Hq + hq) * p.splits + split;
          p.tmp_o[row * D + d] = 0.f;
          if (d == 0) p.tmp_lse[row] = -INFINITY;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, 64);
}

struct DKey {
  const void* p;
  uint64_t a, b, c;
  bool operator==(const DKey& o) const { return p == o.p && a == o.a && b == o.b && c == o.c; }
};
struct DKeyHash {
  size_t operator()(const DKey& k) const {
    return reinterpret_cast<size_t>(k.p) ^ (k.a * 0x9e3779b97f4a7c15ull) ^ (k.b << 21) ^ (k.c << 42);
  }
};

template <int D>
static cudaError_t launch_decode_tc(int G, dim3 grid, cudaStream_t stream, const CUtensorMap& tmQ,
                                    const CUtensorMap& tmKV, const DecodeTcParams& p) {
  constexpr size_t smem = (size_t)kSlots * DecodeTcSmem<D>::slot_bytes + DecodeTcSmem<D>::q_bytes +
                          DecodeTcSmem<D>::p_bytes + 1024 + sizeof(DecodeTcBars);
  static_assert(smem <= 227 * 1024, "shared memory budget");
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(attn_decode_tc_kernel<4, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(attn_decode_tc_kernel<8, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaFuncSetAttribute(attn_decode_tc_kernel<16, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  if (G <= 4) return launch_pdl(attn_decode_tc_kernel<4, D>, grid, dim3(192), smem, stream, tmQ, tmKV, p);
  if (G <= 8) return launch_pdl(attn_decode_tc_kernel<8, D>, grid, dim3(192), smem, stream, tmQ, tmKV, p);
  return launch_pdl(attn_decode_tc_kernel<16, D>, grid, dim3(192), smem, stream, tmQ, tmKV, p);
}

}  // namespace b200

using namespace b200;


// The merge kernel of the CUDA-core path (attn_decode.cu) combines the split partials.
extern "C" int b200_attn_decode_merge(const void* tmp_o, const void* tmp_lse, void* out, int ldo,
                                      int B, int Hq, int D, int splits, cudaStream_t stream);

extern "C" int b200_attn_decode_tc(const void* q, int ldq, void* out, int ldo,
                                   const void* kv_cache, int64_t num_blocks, int block_size,
                                   int Hq, int Hkv, int D, const void* block_table,
                                   int max_blocks, const void* seq_lens, int B, float scale,
                                   float softcap, int window, int splits, void* tmp_o,
                                   void* tmp_lse, cudaStream_t stream) {
  if (B <= 0) return 0;
  if ((D != 128 && D != 256) || Hq % Hkv || Hq / Hkv > kNQ || (ldq & 7)) return -1;
  if (block_size < 8 || (block_size & 7) || (block_size < kTok && kTok % block_size) ||
      (block_size > kTok && block_size % kTok) || kTok / (block_size < kTok ? block_size : kTok) > 16)
    return -1;
  if (splits < 1) splits = 1;
  if (splits > 1 && (!tmp_o || !tmp_lse)) return -1;
  static std::mutex mu;
  static std::unordered_map<DKey, CUtensorMap, DKeyHash> maps;
  auto get = [&](const DKey& key, auto&& make, CUtensorMap* outm) -> bool {
    std::lock_guard<std::mutex> lock(mu);
    auto it = maps.find(key);
    if (it == maps.end()) {
      CUtensorMap m;
      if (!make(&m)) return false;
      it = maps.emplace(key, m).first;
    }
    *outm = it->second;
    return true;
  };
  CUtensorMap tmQ, tmKV;
  if (!get(DKey{q, (uint64_t)B, (uint64_t)Hq | ((uint64_t)D << 32), (uint64_t)ldq},
           [&](CUtensorMap* m) {
             return encode_tmap_3d(m, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)D,
                                   (uint64_t)Hq, (uint64_t)B, (uint64_t)D * 2, (uint64_t)ldq * 2,
                                   64, kNQ, 1, CU_TENSOR_MAP_SWIZZLE_128B);
           },
           &tmQ))
    return -3;
  const int box_rows = block_size < kTok ? block_size : kTok;
  const uint64_t rows = (uint64_t)num_blocks * 2 * block_size;
  if (!get(DKey{kv_cache, rows, (uint64_t)Hkv | ((uint64_t)D << 32), (uint64_t)box_rows + 7777},
           [&](CUtensorMap* m) {
             return encode_tmap_3d(m, kv_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)D,
                                   (uint64_t)Hkv, rows, (uint64_t)D * 2, (uint64_t)Hkv * D * 2, 64,
                                   1, (uint32_t)box_rows, CU_TENSOR_MAP_SWIZZLE_128B);
           },
           &tmKV))
    return -3;
  DecodeTcParams p;
  p.out = (__nv_bfloat16*)out; p.ldo = ldo;
  p.block_table = (const int32_t*)block_table; p.max_blocks = max_blocks;
  p.seq_lens = (const int32_t*)seq_lens; p.Hq = Hq; p.Hkv = Hkv; p.block_size = block_size;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.softcap2 = softcap * 1.4426950408889634f;
  p.window = window; p.splits = splits;
  p.tmp_o = (float*)tmp_o; p.tmp_lse = (float*)tmp_lse;
  p.status = device_status_word();
  dim3 grid(B, Hkv, splits);
  const int G = Hq / Hkv;
  cudaError_t le;
  if (D == 128) le = launch_decode_tc<128>(G, grid, stream, tmQ, tmKV, p);
  else le = launch_decode_tc<256>(G, grid, stream, tmQ, tmKV, p);
  if (le != cudaSuccess) return -2;
  if (splits > 1)
    return b200_attn_decode_merge(tmp_o, tmp_lse, out, ldo, B, Hq, D, splits, stream);
  return 0;
}
