// Multi-head latent attention (DeepSeek-V2 family) kernels.
//
// Cache: one row of 512 latent + 64 rotary values per token, [num_blocks * block_size, 576].
//
// Decode ("absorbed" form, reference: src/vt/cuda/cuda_mla_decode.cu MlaDecodeStage1/2):
// queries arrive already multiplied by W_UK, q' = [q_nope W_UK (512) | q_pe (64)], and all
// heads attend to the same latent rows (multi-query); V is the first 512 columns of those
// rows. tcgen05 with swapped operands, one CTA = one (sequence, kv split):
//     S^T[128 tok, 16 heads] = C[128 tok, 576] * q'[16, 576]^T
//     O^T[512, 16]          += C[128 tok, 0:512]^T * P^T          (four M = 128 products)
// Every byte of the latent tile is loaded once. Its four 128-column value pieces go through a ring
// of five 32 KB slots and stay there from the S product until the O product of the same tile has
// read them (as the MN-major V^T operand); the 64 rotary columns go through two 16 KB slots that
// are free again as soon as S has read them. The MMA warp issues S(j+1) on the pieces that could be
// prefetched (rotary + the first value piece) while the softmax of tile j runs, then O(j), whose
// four products release the value slots one by one for the rest of tile j+1, then the rest of
// S(j+1). Softmax as in attn_decode_tc.cu: one thread per token, lazily raised running max, O^T
// rescaled in TMEM when it moves.
//
// Prefill helpers (reference: cuda_mla_prefill.cu GatherMlaCache / ConcatMlaNopeRope / PadV):
// gather a request's latent rows into a dense buffer, then build per-head K = [k_nope | k_pe]
// and V padded to 256 columns in the paged layout the head_dim-256 prefill kernel reads.
#include <mutex>
#include <unordered_map>

#include "api.h"
#include "sm100.cuh"

namespace b200 {

typedef __nv_bfloat16 bf16;

static constexpr int kTok = 128;
static constexpr int kNQ = 16;
static constexpr int kLat = 512, kRope = 64, kRow = kLat + kRope;   // 576
static constexpr int kVPieces = 4;         // 128-column value pieces of a row (the rotary 64 columns follow)
static constexpr int kVSlots = 5;          // ring of the value pieces
static constexpr int kRSlots = 2;          // ring of the rotary pieces
static constexpr int kSlots = kVSlots + kRSlots;
static constexpr int kSlotBytes = 128 * 128 * 2;
static constexpr int kRopeBytes = 128 * 64 * 2;
static constexpr int kRingBytes = kVSlots * kSlotBytes + kRSlots * kRopeBytes;
static constexpr int kQBytes = 9 * 2048;   // 9 halves of [16 heads x 64 cols]

struct MlaDecodeParams {
  bf16* out;            // [B, Hq, 512]
  int ldo;              // row stride of out in elements
  const int32_t* block_table;
  int max_blocks;
  const int32_t* seq_lens;
  int Hq, block_size;
  float scale_log2;
  int splits;
  float* tmp_o;         // [B, Hq, splits, 512]
  float* tmp_lse;       // [B, Hq, splits] log2 domain
  int* status;
};

struct alignas(8) MlaBars {
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

__device__ __forceinline__ void mla_tmem_st_x16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
      "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
      "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ bool mla_group_sync(uint64_t* bar, uint32_t& phase, int lane, int* status) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
  const bool ok = mbar_wait(bar, phase, status);
  phase ^= 1;
  return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ float mla_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Ring order shared by producer and consumer: S pieces of tile 0; then for every later tile j
// its S pieces followed by the O pieces of tile j-1; last the O pieces of the final tile.
__global__ void __launch_bounds__(192, 1)
    mla_decode_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmC,
                      MlaDecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sKV = smem;
  uint8_t* sRope = sKV + kVSlots * kSlotBytes;
  uint8_t* sQ = sKV + kRingBytes;
  uint8_t* sP = sQ + kQBytes;                      // 2 buffers x (2 token halves x 2 KB)
  MlaBars* bars = reinterpret_cast<MlaBars*>(sP + 8192);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x, split = blockIdx.y;
  const int G = p.Hq;
  const int seq_len = p.seq_lens[b];
  const int tiles_total = (seq_len + kTok - 1) / kTok;
  const int tiles_per_split = (tiles_total + p.splits - 1) / p.splits;
  const int tile0 = split * tiles_per_split;
  const int ntiles = max(0, min(tiles_total, tile0 + tiles_per_split) - tile0);
  const int tok_base = tile0 * kTok;

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
  for (int i = threadIdx.x; i < 8192 / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(sP)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 128);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  const uint32_t tmem_s = tmem_base;         // 2 x 16 columns
  const uint32_t tmem_o = tmem_base + 32;    // 4 x 16 columns

  if (ntiles > 0) {
    if (warp == 0) {
      if (lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmC);
        mbar_expect_tx(&bars->q_full, kQBytes);
        for (int h = 0; h < 9; ++h) tma_load_3d(sQ + h * 2048, &tmQ, &bars->q_full, h * 64, 0, b);
        const int32_t* bt = p.block_table + (size_t)b * p.max_blocks;
        const int nblk_valid = (seq_len + p.block_size - 1) / p.block_size;
        const int rows_per_load = min(p.block_size, kTok);
        const int loads = kTok / rows_per_load;
        bool ok = true;
        int itv = 0, itr = 0;
        // piece < kVPieces: value columns [128 * piece, +128) into the value ring; piece == kVPieces:
        // the rotary columns [512, 576) into the rotary ring
        auto load_piece = [&](int j, int piece) {
          const bool rope = piece == kVPieces;
          int& it = rope ? itr : itv;
          const int n = rope ? kRSlots : kVSlots;
          const int sl = it % n;
          const uint32_t ph = (it / n) & 1;
          ++it;
          const int bi_ = rope ? kVSlots + sl : sl;                // barrier index
          if (!mbar_wait(&bars->kv_empty[bi_], ph ^ 1, p.status)) { ok = false; return; }
          uint8_t* dst = rope ? sRope + sl * kRopeBytes : sKV + sl * kSlotBytes;
          const int halves = rope ? 1 : 2;
          mbar_expect_tx(&bars->kv_full[bi_], halves * 16384);
          const int tok0 = tok_base + j * kTok;
          for (int l = 0; l < loads; ++l) {
            const int tk = tok0 + l * rows_per_load;
            const int bi = tk / p.block_size;
            const int blk = (bi < nblk_valid) ? bt[bi] : bt[0];
            const int row = (blk < 0 ? 0 : blk) * p.block_size + tk % p.block_size;
            for (int hf = 0; hf < halves; ++hf)
              tma_load_2d(dst + hf * 16384 + l * rows_per_load * 128, &tmC, &bars->kv_full[bi_],
                          piece * 128 + hf * 64, row);
          }
        };
        // per tile: rotary piece first (its slot turns over early), then the value pieces in the
        // order both products read them
        for (int j = 0; j < ntiles && ok; ++j) {
          load_piece(j, kVPieces);
          for (int pc = 0; pc < kVPieces && ok; ++pc) load_piece(j, pc);
        }
      }
    } else if (warp == 1) {
      if (lane == 0) {
        constexpr uint32_t idesc_qk = umma_idesc_bf16(kTok, kNQ, 0, 0);
        constexpr uint32_t idesc_pv = umma_idesc_bf16(128, kNQ, 1, 0);
        bool ok = mbar_wait(&bars->q_full, 0, p.status);
        const uint32_t q_addr = smem_u32(sQ);
        // value piece pc of tile j sits in value slot (4 j + pc) % 5 on that slot's ((4 j + pc) / 5)-th
        // use; the rotary piece of tile j in rotary slot j % 2
        auto s_piece = [&](int j, int pc, bool first) -> bool {      // one piece of S(j) = K(j) Q^T
          const bool rope = pc == kVPieces;
          const int f = rope ? j : kVPieces * j + pc, n = rope ? kRSlots : kVSlots;
          const int sl = f % n, bi_ = rope ? kVSlots + sl : sl;
          if (!mbar_wait(&bars->kv_full[bi_], (f / n) & 1, p.status)) return false;
          tc_fence_after_sync();
          const uint32_t k_addr = smem_u32(rope ? sRope + sl * kRopeBytes : sKV + sl * kSlotBytes);
          const int ksteps = rope ? 4 : 8;
          for (int kk = 0; kk < ksteps; ++kk) {
            const uint32_t koff = (kk / 4) * 16384 + (kk % 4) * 32;
            const uint32_t qoff = (pc * 2 + kk / 4) * 2048 + (kk % 4) * 32;
            umma_bf16_ss(tmem_s + (j & 1) * 16, umma_desc_k_sw128(k_addr + koff, 1024),
                         umma_desc_k_sw128(q_addr + qoff, 1024), idesc_qk, !(first && kk == 0));
          }
          if (rope) umma_commit(&bars->kv_empty[bi_]);    // the value slots stay until O(j) has read them
          return true;
        };
        // S(0): rotary piece, then the value pieces
        ok = ok && mbar_wait(&bars->s_empty[0], 1, p.status);
        ok = ok && s_piece(0, kVPieces, true);
        for (int pc = 0; pc < kVPieces && ok; ++pc) ok = s_piece(0, pc, false);
        if (ok) umma_commit(&bars->s_full[0]);
        for (int j = 0; j < ntiles && ok; ++j) {
          const bool next = j + 1 < ntiles;
          if (next) {
            // what of tile j+1 can be in shared memory already: its rotary piece and one value piece
            const int sb = (j + 1) & 1;
            if (!mbar_wait(&bars->s_empty[sb], (((j + 1) >> 1) & 1) ^ 1, p.status)) { ok = false; break; }
            ok = s_piece(j + 1, kVPieces, true) && s_piece(j + 1, 0, false);
            if (!ok) break;
          }
          // O(j) += V(j)^T P(j)^T, releasing the value slots of tile j one by one
          const int pb = j & 1;
          if (!mbar_wait(&bars->p_full[pb], (j >> 1) & 1, p.status)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t p_addr = smem_u32(sP + pb * 4096);
          for (int pc = 0; pc < kVPieces; ++pc) {
            const int f = kVPieces * j + pc, sl = f % kVSlots;
            const uint32_t v_addr = smem_u32(sKV + sl * kSlotBytes);
#pragma unroll
            for (int kk = 0; kk < kTok / 16; ++kk) {
              const uint32_t poff = (kk / 4) * 2048 + (kk % 4) * 32;
              umma_bf16_ss(tmem_o + pc * 16, umma_desc_mn_sw128(v_addr + kk * 2048, 16384, 1024),
                           umma_desc_k_sw128(p_addr + poff, 1024), idesc_pv, (j | kk) != 0);
            }
            umma_commit(&bars->kv_empty[sl]);
          }
          umma_commit(&bars->pv_done);    // before p_empty: whoever sees p_empty has this arrival too
          umma_commit(&bars->p_empty[pb]);
          if (next) {
            for (int pc = 1; pc < kVPieces && ok; ++pc) ok = s_piece(j + 1, pc, false);
            if (ok) umma_commit(&bars->s_full[(j + 1) & 1]);
          }
        }
      }
    } else {
      const int quarter = warp & 3;
      const int t = quarter * 32 + lane;
      const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
      float m[kNQ], lsum[kNQ];
#pragma unroll
      for (int g = 0; g < kNQ; ++g) { m[g] = -INFINITY; lsum[g] = 0.f; }
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
        const bool valid = tok < seq_len;
        float s[kNQ];
#pragma unroll
        for (int g = 0; g < kNQ; ++g) s[g] = valid ? __uint_as_float(r[g]) * p.scale_log2 : -INFINITY;
        {
          float wm[kNQ];
#pragma unroll
          for (int g = 0; g < kNQ; ++g) wm[g] = warp_max_f32(s[g]);
          if (lane == 0) {
#pragma unroll
            for (int g = 0; g < kNQ; ++g) bars->red_max[sb][quarter][g] = wm[g];
          }
        }
        ok = mla_group_sync(&bars->grp, gphase, lane, p.status);
        if (!ok) break;
        bool rescale = false;
        float alpha[kNQ];
#pragma unroll
        for (int g = 0; g < kNQ; ++g) {
          const float tm = fmaxf(fmaxf(bars->red_max[sb][0][g], bars->red_max[sb][1][g]),
                                 fmaxf(bars->red_max[sb][2][g], bars->red_max[sb][3][g]));
          alpha[g] = 1.f;
          if (tm > m[g] + 8.f) {
            if (m[g] != -INFINITY) {
              alpha[g] = mla_exp2(m[g] - tm);
              rescale = true;
            }
            m[g] = tm;
          }
        }
        const int pb = j & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->p_empty[pb], ((j >> 1) & 1) ^ 1, p.status));
        if (!ok) break;
        // p_empty above means PV(j-2) is complete, so pv_done has completed at least j-1 times
        // and this parity wait (its j-th completion) cannot be satisfied by an older phase
        if (rescale && j > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(&bars->pv_done, (j - 1) & 1, p.status));
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int pc = 0; pc < kVPieces; ++pc) {
            uint32_t o[16];
            tmem_ld_32x32b_x16(tmem_o + pc * 16 + lane_off, o);
            tmem_ld_wait();
#pragma unroll
            for (int g = 0; g < kNQ; ++g) o[g] = __float_as_uint(__uint_as_float(o[g]) * alpha[g]);
            mla_tmem_st_x16(tmem_o + pc * 16 + lane_off, o);
          }
          tmem_st_wait();
#pragma unroll
          for (int g = 0; g < kNQ; ++g) lsum[g] *= alpha[g];
        }
        uint8_t* pbuf = sP + pb * 4096 + (t >> 6) * 2048;
        const int c = t & 63;
#pragma unroll
        for (int g = 0; g < kNQ; ++g) {
          if (g < G) {
            const float pv = valid ? mla_exp2(s[g] - m[g]) : 0.f;
            const bf16 pb16 = __float2bfloat16(pv);
            lsum[g] += __bfloat162float(pb16);
            *reinterpret_cast<bf16*>(pbuf + g * 128 + (((c >> 3) ^ (g & 7)) << 4) + (c & 7) * 2) = pb16;
          }
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->p_full[pb]);
      }
      // observe the last two completions in order (the loop only guarantees ntiles-2 seen)
      if (ok && ntiles >= 2)
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->pv_done, (ntiles - 2) & 1, p.status));
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->pv_done, (ntiles - 1) & 1, p.status));
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int g = 0; g < kNQ; ++g) {
          float v = lsum[g];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0) bars->red_sum[quarter][g] = v;
        }
        ok = mla_group_sync(&bars->grp, gphase, lane, p.status);
      }
      if (ok) {
#pragma unroll
        for (int pc = 0; pc < kVPieces; ++pc) {
          uint32_t o[16];
          tmem_ld_32x32b_x16(tmem_o + pc * 16 + lane_off, o);
          tmem_ld_wait();
          const int d = pc * 128 + t;
#pragma unroll
          for (int g = 0; g < kNQ; ++g) {
            if (g < G) {
              const float l = bars->red_sum[0][g] + bars->red_sum[1][g] + bars->red_sum[2][g] + bars->red_sum[3][g];
              const float v = l > 0.f ? __uint_as_float(o[g]) / l : 0.f;
              if (p.splits == 1) {
                p.out[(size_t)b * p.ldo + (size_t)g * kLat + d] = __float2bfloat16(v);
              } else {
                const size_t row = ((size_t)b * p.Hq + g) * p.splits + split;
                p.tmp_o[row * kLat + d] = v;
                if (d == 0) p.tmp_lse[row] = l > 0.f ? m[g] + log2f(l) : -INFINITY;
              }
            }
          }
        }
      }
    }
  } else if (warp >= 2) {
    const int t = (warp & 3) * 32 + lane;
    for (int g = 0; g < G; ++g) {
      for (int pc = 0; pc < kVPieces; ++pc) {
        const int d = pc * 128 + t;
        if (p.splits == 1) {
          p.out[(size_t)b * p.ldo + (size_t)g * kLat + d] = __float2bfloat16(0.f);
        } else {
          const size_t row = ((size_t)b * p.Hq + g) * p.splits + split;
          p.tmp_o[row * kLat + d] = 0.f;
          if (d == 0) p.tmp_lse[row] = -INFINITY;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, 128);
}

// ---------------------------------------------------------------------------------------
// Prefill helpers
// ---------------------------------------------------------------------------------------
// dense[base[r] + i] = cache row of position i of request r, for whole blocks.
__global__ void __launch_bounds__(128)
    mla_gather_latent_kernel(const bf16* __restrict__ cache, const int32_t* __restrict__ block_table,
                             int max_blocks, const int32_t* __restrict__ seq_lens,
                             const int32_t* __restrict__ dense_base, int block_size, bf16* __restrict__ dense) {
  const int r = blockIdx.y, bi = blockIdx.x;
  const int nblk = (seq_lens[r] + block_size - 1) / block_size;
  if (bi >= nblk) return;
  const int blk = block_table[(size_t)r * max_blocks + bi];
  const uint4* src = reinterpret_cast<const uint4*>(cache + (size_t)(blk < 0 ? 0 : blk) * block_size * kRow);
  uint4* dst = reinterpret_cast<uint4*>(dense + ((size_t)dense_base[r] + (size_t)bi * block_size) * kRow);
  const int n = block_size * kRow / 8;
  for (int i = threadIdx.x; i < n; i += blockDim.x) dst[i] = src[i];
}

// kvb: [N, H, 256] = per head [k_nope 128 | v 128]; dense: [N, 576]. Writes the paged layout
// [N / bs, 2, bs, H, 256]: K = [k_nope | k_pe | 0], V = [v | 0].
__global__ void __launch_bounds__(128)
    mla_assemble_kv_kernel(const bf16* __restrict__ kvb, const bf16* __restrict__ dense,
                           bf16* __restrict__ cache, int H, int block_size) {
  const size_t t = blockIdx.x;
  const size_t blk = t / block_size, off = t % block_size;
  const int lane16 = threadIdx.x & 31;      // 32 uint4 per 256-wide head row
  for (int h = threadIdx.x >> 5; h < H; h += 4) {
    const uint4* src = reinterpret_cast<const uint4*>(kvb + (t * H + h) * 256);
    uint4* kd = reinterpret_cast<uint4*>(cache + (((blk * 2 + 0) * block_size + off) * H + h) * 256);
    uint4* vd = reinterpret_cast<uint4*>(cache + (((blk * 2 + 1) * block_size + off) * H + h) * 256);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    uint4 kv;
    if (lane16 < 16) kv = src[lane16];
    else if (lane16 < 24) kv = reinterpret_cast<const uint4*>(dense + t * kRow + kLat)[lane16 - 16];
    else kv = zero;
    kd[lane16] = kv;
    vd[lane16] = lane16 < 16 ? src[16 + lane16] : zero;
  }
}

// q rows [T, H, 192] (row stride ldq) -> [T, H, 256] zero padded.
__global__ void __launch_bounds__(128)
    mla_pad_q_kernel(const bf16* __restrict__ q, long ldq, bf16* __restrict__ out, int H) {
  const size_t t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  for (int h = threadIdx.x >> 5; h < H; h += 4) {
    const uint4* src = reinterpret_cast<const uint4*>(q + t * ldq + (size_t)h * 192);
    uint4* dst = reinterpret_cast<uint4*>(out + (t * H + h) * 256);
    dst[lane] = lane < 24 ? src[lane] : make_uint4(0, 0, 0, 0);
  }
}

// q_pe (64 values at column 128 of each 192-wide head) -> column 512 of each 576-wide row.
__global__ void __launch_bounds__(128)
    mla_copy_qpe_kernel(const bf16* __restrict__ q, long ldq, bf16* __restrict__ qabs, int H) {
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < H * 8; i += blockDim.x) {
    const int h = i >> 3, c = i & 7;
    reinterpret_cast<uint4*>(qabs + (t * H + h) * kRow + kLat)[c] =
        reinterpret_cast<const uint4*>(q + t * ldq + (size_t)h * 192 + 128)[c];
  }
}

struct MKey {
  const void* p;
  uint64_t a, b;
  bool operator==(const MKey& o) const { return p == o.p && a == o.a && b == o.b; }
};
struct MKeyHash {
  size_t operator()(const MKey& k) const {
    return reinterpret_cast<size_t>(k.p) ^ (k.a * 0x9e3779b97f4a7c15ull) ^ (k.b << 29);
  }
};

}  // namespace b200

using namespace b200;

extern "C" int b200_attn_decode_merge(const void* tmp_o, const void* tmp_lse, void* out, int ldo,
                                      int B, int Hq, int D, int splits, cudaStream_t stream);

extern "C" {

// qabs: [B, Hq, 576] bf16 contiguous; cache: [num_blocks * block_size, 576]; out: [B, Hq, 512]
// (row stride ldo). Hq <= 16.
int b200_mla_decode(const void* qabs, void* out, int ldo, const void* cache, int64_t num_blocks,
                    int block_size, int Hq, const void* block_table, int max_blocks,
                    const void* seq_lens, int B, float scale, int splits, void* tmp_o, void* tmp_lse,
                    cudaStream_t stream) {
  if (B <= 0) return 0;
  if (Hq < 1 || Hq > kNQ) return -1;
  if (block_size < 8 || (block_size & 7) || (block_size < kTok && kTok % block_size) ||
      (block_size > kTok && block_size % kTok) || kTok / (block_size < kTok ? block_size : kTok) > 16)
    return -1;
  if (splits < 1) splits = 1;
  if (splits > 1 && (!tmp_o || !tmp_lse)) return -1;
  static std::mutex mu;
  static std::unordered_map<MKey, CUtensorMap, MKeyHash> maps;
  CUtensorMap tmQ, tmC;
  {
    std::lock_guard<std::mutex> lock(mu);
    MKey kq{qabs, (uint64_t)B, (uint64_t)Hq};
    auto it = maps.find(kq);
    if (it == maps.end()) {
      CUtensorMap m;
      if (!encode_tmap_3d(&m, qabs, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (uint64_t)kRow, (uint64_t)Hq,
                          (uint64_t)B, (uint64_t)kRow * 2, (uint64_t)Hq * kRow * 2, 64, kNQ, 1,
                          CU_TENSOR_MAP_SWIZZLE_128B))
        return -3;
      it = maps.emplace(kq, m).first;
    }
    tmQ = it->second;
    const uint32_t box_rows = block_size < kTok ? block_size : kTok;
    MKey kc{cache, (uint64_t)num_blocks * block_size, (uint64_t)box_rows + 99991};
    it = maps.find(kc);
    if (it == maps.end()) {
      CUtensorMap m;
      if (!encode_tmap_2d(&m, cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                          (uint64_t)num_blocks * block_size, kRow, kRow, box_rows, 64,
                          CU_TENSOR_MAP_SWIZZLE_128B))
        return -3;
      it = maps.emplace(kc, m).first;
    }
    tmC = it->second;
  }
  MlaDecodeParams p;
  p.out = (bf16*)out; p.ldo = ldo;
  p.block_table = (const int32_t*)block_table; p.max_blocks = max_blocks;
  p.seq_lens = (const int32_t*)seq_lens; p.Hq = Hq; p.block_size = block_size;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.splits = splits; p.tmp_o = (float*)tmp_o; p.tmp_lse = (float*)tmp_lse;
  p.status = device_status_word();
  constexpr size_t smem = (size_t)kRingBytes + kQBytes + 8192 + 1024 + sizeof(MlaBars);
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  }
  mla_decode_kernel<<<dim3(B, splits), 192, smem, stream>>>(tmQ, tmC, p);
  if (cudaGetLastError() != cudaSuccess) return -2;
  if (splits > 1) return b200_attn_decode_merge(tmp_o, tmp_lse, out, ldo, B, Hq, kLat, splits, stream);
  return 0;
}

int b200_mla_gather_latent(const void* cache, const void* block_table, int max_blocks,
                           const void* seq_lens, const void* dense_base, int block_size, void* dense,
                           int num_reqs, int max_req_blocks, cudaStream_t stream) {
  if (num_reqs <= 0 || max_req_blocks <= 0) return 0;
  mla_gather_latent_kernel<<<dim3(max_req_blocks, num_reqs), 128, 0, stream>>>(
      (const bf16*)cache, (const int32_t*)block_table, max_blocks, (const int32_t*)seq_lens,
      (const int32_t*)dense_base, block_size, (bf16*)dense);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_mla_assemble_kv(const void* kvb, const void* dense, void* cache, int N, int H, int block_size,
                         cudaStream_t stream) {
  if (N <= 0) return 0;
  mla_assemble_kv_kernel<<<N, 128, 0, stream>>>((const bf16*)kvb, (const bf16*)dense, (bf16*)cache, H,
                                                block_size);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_mla_pad_q(const void* q, long ldq, void* out, int T, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  mla_pad_q_kernel<<<T, 128, 0, stream>>>((const bf16*)q, ldq, (bf16*)out, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_mla_copy_qpe(const void* q, long ldq, void* qabs, int T, int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  mla_copy_qpe_kernel<<<T, 128, 0, stream>>>((const bf16*)q, ldq, (bf16*)qabs, H);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
