// bf16 GEMM  C[M,N] = A[M,K] * W[N,K]^T  (+bias[N]) (+residual[M,N]) on tcgen05 / TMEM.
//
// Two kernels:
//   gemm_bf16_tn_kernel   persistent, 128 x BN output tiles (BN = 128 | 256), TMA-fed
//                         smem ring, accumulators double-buffered in TMEM so the epilogue
//                         of tile i overlaps the main loop of tile i+1. For M > 256.
//   gemm_bf16_swap_kernel small-M ("decode") form: the weight tile is the 128-row MMA
//                         operand and the activations are the N operand (UMMA N = M padded
//                         to 16), so the weight stream is read exactly once; split-K over
//                         blockIdx.y with fp32 partials reduced in fixed order.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (each owns the TMEM lane quarter warp_id % 4).
//
// Replaces the library GEMM calls of the reference (src/vt/cuda/cuda_matmul.cu:284-355
// "MatmulBT" and :219-274), which hand every projection to cuBLASLt.
#include <mutex>
#include <unordered_map>

#include "api.h"
#include "sm100.cuh"

namespace b200 {

static constexpr int kBM = 128;
static constexpr int kBK = 64;
static constexpr int kGemmThreads = 192;
static constexpr int kMaxStages = 12;

struct GemmParams {
  int M, N, K;
  void* out;
  int ldo;
  int out_f32;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int ldr;
  int* status;
  int tiles_m, tiles_n;
  int stages;
  // swap-AB only
  int mp;            // padded M = UMMA N
  int splits;
  int kb_per_split;
  float* workspace;  // [splits, M, N] fp32 partials
  // batched mode (blockIdx.z = batch): W is [batch * N, K], batch b reads the A columns from
  // b * batch_a_cols and writes out + b * batch_out_stride. No split-K.
  int batch_a_cols;
  long long batch_out_stride;
  // ---- fused tensor-parallel modes (all zero when unused) -------------------------------
  // scatter epilogue (GEMM + reduce-scatter): row m of the bf16 partial goes to the rank that
  // owns it (m / rows_per_rank), into that rank's receive buffer slot [parity][tp_rank], and
  // the owner's arrival counter of the 32-row group is bumped with a system-scope release.
  int tp_world, tp_rank, rows_per_rank;
  __nv_bfloat16* peer_recv[8];
  uint32_t* peer_rs_flags[8];
  long long recv_parity_stride;   // elements between the two parities of a receive buffer
  int rs_flag_parity_stride;
  // gather prologue (all-gather + GEMM): A is this rank's copy of the gathered activations,
  // filled by peer stores; the producer waits until every row of a 32-row group has landed.
  const uint32_t* ag_flags;
  long long peer_wait;            // limit of a wait on the gather counters, in cycles
  // The weight operand is not written by earlier work in the stream: its first ring stages may be
  // fetched before the wait on the predecessor kernel (programmatic dependent launch).
  int w_early;
  int ag_flag_parity_stride;
  const uint32_t* op_counter;     // device-side op counter; its low bit selects the parity
  // ---- stream-K (tn kernel only) ---------------------------------------------------------
  // The (tile, k-block) units are cut into gridDim.x equal contiguous ranges. A CTA whose range
  // starts inside a tile writes that fp32 partial to sk_partials[cta] and raises
  // sk_flags[cta * 4 + warp quarter]; the CTA that holds the tile's first k-block adds the
  // partials of the CTAs after it and runs the epilogue, then clears the flags it consumed.
  // fused gated activation (pair kernel, BN = 256): W rows come in blocks of [128 gate | 128 up],
  // so a tile holds both halves of 128 outputs; out[M, N / 2] = act(gate) * up. 0 = off,
  // otherwise activation kind + 1 (1 SiLU, 2 GELU-tanh, 3 GELU-erf).
  int act_fuse;
  // fp8 (e4m3 x e4m3) instantiation of the pair kernel: out = acc * a_scale * w_scale[(n)]
  const float* scale_a;
  const float* scale_w;
  int scale_w_per_channel;
  int scale_a_per_token;     // scale_a is [M], one per row
  int sk;                         // number of leading tiles in the stream-K region (0 = none)
  float* sk_partials;
  uint32_t* sk_flags;
};

// Bounded system-scope acquire wait on a counter another GPU increments.
__device__ __forceinline__ bool wait_counter_ge(const uint32_t* ctr, uint32_t target, int* status,
                                                long long limit) {
  long long t0 = clock64();
  uint32_t it = 0;
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
    if (v >= target) return true;
    if (((++it) & 0xff) == 0 && clock64() - t0 > limit) {
      if (status) atomicExch(status, (int)kErrFlagTimeout);
      return false;
    }
  }
}
__device__ __forceinline__ void signal_counter(uint32_t* ctr) {
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(ctr) : "memory");
}
// Peer stores (generic proxy) must be visible to this SM's TMA reads (async proxy).
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

struct alignas(8) GemmBarriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t failed;
};

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  // Grouped ordering: 16 consecutive M tiles share each N tile while it is L2-hot.
  constexpr int G = 16;
  int per_group = G * tiles_n;
  int g = t / per_group;
  int first_m = g * G;
  int gsz = min(G, tiles_m - first_m);
  int r = t - g * per_group;
  tm = first_m + (r % gsz);
  tn = r / gsz;
}

// Work iterator shared by the three warp roles. Plain mode: whole tiles strided over the workers
// (a worker is a CTA, or a CTA pair in the pair kernel). Stream-K mode: the first p.sk tiles are
// cut into (tile, k-block) units and dealt out as equal contiguous ranges, one per worker; the
// remaining tiles follow as whole tiles. Workers that run whole tiles side by side step through
// K together and share their operand tiles in L2; the stream-K region, where they do not, is
// kept to the ragged part of the problem and runs first so that its fix-up hides under the rest.
struct SegState {
  int sk_tiles, t, stride, u, u1;
};
__device__ __forceinline__ int sk_range_start_w(int w, int units, int nworkers) {
  const int q = units / nworkers, r = units % nworkers;
  return w * q + min(w, r);
}
__device__ __forceinline__ SegState seg_init_w(const GemmParams& p, int kblocks, int worker,
                                               int nworkers) {
  SegState s;
  s.sk_tiles = p.sk;
  s.t = p.sk + worker;
  s.stride = nworkers;
  s.u = sk_range_start_w(worker, p.sk * kblocks, nworkers);
  s.u1 = sk_range_start_w(worker + 1, p.sk * kblocks, nworkers);
  return s;
}
__device__ __forceinline__ bool seg_next(SegState& s, int num_tiles, int kblocks, int& t, int& kb0,
                                         int& kb1) {
  if (s.u < s.u1) {
    t = s.u / kblocks;
    kb0 = s.u - t * kblocks;
    kb1 = min(kblocks, kb0 + (s.u1 - s.u));
    s.u += kb1 - kb0;
    return true;
  }
  if (s.t >= num_tiles) return false;
  t = s.t;
  kb0 = 0;
  kb1 = kblocks;
  s.t += s.stride;
  return true;
}
// Bounded device-scope acquire wait for a stream-K partial flag.
__device__ __forceinline__ bool wait_flag_set(const uint32_t* f, int* status) {
  long long t0 = clock64();
  uint32_t it = 0;
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if (v != 0) return true;
    if (((++it) & 0xff) == 0 && clock64() - t0 > kPeerWaitCycles) {
      if (status) atomicExch(status, (int)kErrFlagTimeout);
      return false;
    }
  }
}

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap tmA,
                        const __grid_constant__ CUtensorMap tmA_alt,
                        const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  constexpr int kABytes = kBM * kBK * 2;
  constexpr int kBBytes = BN * kBK * 2;
  constexpr int kStageBytes = kABytes + kBBytes;
  const int stages = p.stages;
  GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(smem + (size_t)stages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = (p.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], 4);
    }
    bars->failed = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 2 * BN >= 32 ? 2 * BN : 32);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  // Weights that nothing in the stream writes: fetch the weight halves of the first ring stages of
  // this CTA's first segment before waiting on the predecessor kernel.
  int npre = 0;
  if (warp == 0 && lane == 0 && p.w_early && !p.ag_flags) {
    SegState seg0 = seg_init_w(p, kblocks, blockIdx.x, gridDim.x);
    int t0, ka, kz;
    if (seg_next(seg0, num_tiles, kblocks, t0, ka, kz)) {
      int tm0, tn0;
      tile_coords(t0, p.tiles_m, p.tiles_n, tm0, tn0);
      tma_prefetch_desc(&tmB);
      npre = min(kz - ka, stages);
      for (int i = 0; i < npre; ++i) {
        mbar_expect_tx(&bars->full[i], kStageBytes);
        tma_load_2d(smem + (size_t)i * kStageBytes + kABytes, &tmB, &bars->full[i], (ka + i) * kBK, tn0 * BN);
      }
    }
  }
  pdl_wait();                 // predecessor grid complete, its writes visible
  pdl_launch_dependents();    // the successor may become resident (it waits the same way)

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      // gather mode: A has one copy per parity of the op counter, pick the one just written
      const CUtensorMap* ta = (p.ag_flags && ((*p.op_counter - 1) & 1)) ? &tmA_alt : &tmA;
      tma_prefetch_desc(ta);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      SegState seg = seg_init_w(p, kblocks, blockIdx.x, gridDim.x);
      int t, kb0, kb1;
      while (ok && seg_next(seg, num_tiles, kblocks, t, kb0, kb1)) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        if (p.ag_flags) {
          const uint32_t par = (*p.op_counter - 1) & 1;
          for (int g = tm * 4; g < tm * 4 + 4 && ok; ++g) {
            const int need = min(32, p.M - g * 32);
            if (need > 0)
              ok = wait_counter_ge(p.ag_flags + par * p.ag_flag_parity_stride + g, need, p.status, p.peer_wait);
          }
          if (!ok) break;
          fence_proxy_async_global();
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          int s = it % stages;
          uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, p.status)) { ok = false; break; }
          uint8_t* a_dst = smem + (size_t)s * kStageBytes;
          uint8_t* b_dst = a_dst + kABytes;
          if ((int)it >= npre) {  // (the first npre stages already expect their bytes and hold B)
            mbar_expect_tx(&bars->full[s], kStageBytes);
            tma_load_2d(b_dst, &tmB, &bars->full[s], kb * kBK, tn * BN);
          }
          tma_load_2d(a_dst, ta, &bars->full[s], kb * kBK, tm * kBM);
        }
      }
      if (!ok) bars->failed = 1;
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(kBM, BN);
      uint32_t it = 0, tc = 0;
      bool ok = true;
      SegState seg = seg_init_w(p, kblocks, blockIdx.x, gridDim.x);
      int t, kb0, kb1;
      for (; ok && seg_next(seg, num_tiles, kblocks, t, kb0, kb1); ++tc) {
        int buf = tc & 1;
        uint32_t aph = (tc >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[buf], aph ^ 1, p.status)) { ok = false; break; }
        tc_fence_after_sync();
        uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          int s = it % stages;
          uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars->full[s], ph, p.status)) { ok = false; break; }
          tc_fence_after_sync();
          uint32_t a_addr = smem_u32(smem + (size_t)s * kStageBytes);
          uint32_t b_addr = a_addr + kABytes;
          uint64_t adesc = umma_desc_k_sw128(a_addr, 1024);
          uint64_t bdesc = umma_desc_k_sw128(b_addr, 1024);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // +32 bytes per 16-element K step inside the 128-byte swizzle row.
            umma_bf16_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, kb != kb0 || k != 0);
          }
          umma_commit(&bars->empty[s]);
        }
        if (ok) umma_commit(&bars->acc_full[buf]);
      }
      if (!ok) bars->failed = 1;
    }
  } else {
    // ---------------- Epilogue (warps 2..5) ----------------
    const int quarter = warp & 3;
    uint32_t tc = 0;
    bool ok = true;
    SegState seg = seg_init_w(p, kblocks, blockIdx.x, gridDim.x);
    int t, kb0, kb1;
    for (; ok && seg_next(seg, num_tiles, kblocks, t, kb0, kb1); ++tc) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      int buf = tc & 1;
      uint32_t aph = (tc >> 1) & 1;
      ok = mbar_wait(&bars->acc_full[buf], aph, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = tm * kBM + quarter * 32 + lane;
      const uint32_t t_addr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
      if (kb0 > 0) {
        // stream-K partial: raw fp32 accumulators to this CTA's slot, then the flag
        // column-major inside the slot: the 32 lanes of a warp write 32 consecutive floats
        float* dst = p.sk_partials + (size_t)blockIdx.x * kBM * BN + quarter * 32 + lane;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, r);
          tmem_ld_wait();
          if (row < p.M) {       // the owner only reads the rows that exist
#pragma unroll
            for (int i = 0; i < 32; ++i) __stcg(dst + (size_t)(c * 32 + i) * kBM, __uint_as_float(r[i]));
          }
        }
        __threadfence();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          uint32_t one = 1;
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.sk_flags + blockIdx.x * 4 + quarter),
                       "r"(one)
                       : "memory");
          mbar_arrive(&bars->acc_empty[buf]);
        }
        continue;
      }
      // stream-K owner: the CTAs after this one hold the rest of the tile's k-blocks
      int sk_first = 0, sk_last = -1;
      if (kb1 < kblocks) {
        const int tile_end = (t + 1) * kblocks;
        sk_first = blockIdx.x + 1;
        sk_last = blockIdx.x;
        while (sk_last + 1 < (int)gridDim.x &&
               sk_range_start_w(sk_last + 1, p.sk * kblocks, (int)gridDim.x) < tile_end)
          ++sk_last;
        for (int x = sk_first; x <= sk_last && ok; ++x)
          ok = wait_flag_set(p.sk_flags + x * 4 + quarter, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_addr + c * 32, r);
        tmem_ld_wait();
        const int col0 = tn * BN + c * 32;
        if (row < p.M && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          for (int x = sk_first; x <= sk_last; ++x) {
            const float* src = p.sk_partials + (size_t)x * kBM * BN + (size_t)c * 32 * kBM + quarter * 32 + lane;
            float f[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = __ldcg(src + (size_t)i * kBM);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] += f[i];
          }
          if (p.bias) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (col0 + i < p.N) {
                uint4 b = *reinterpret_cast<const uint4*>(p.bias + col0 + i);
                float2 f;
                f = unpack_bf16x2(b.x); v[i + 0] += f.x; v[i + 1] += f.y;
                f = unpack_bf16x2(b.y); v[i + 2] += f.x; v[i + 3] += f.y;
                f = unpack_bf16x2(b.z); v[i + 4] += f.x; v[i + 5] += f.y;
                f = unpack_bf16x2(b.w); v[i + 6] += f.x; v[i + 7] += f.y;
              }
            }
          }
          if (p.residual) {
            const __nv_bfloat16* rr = p.residual + (size_t)row * p.ldr + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (col0 + i < p.N) {
                uint4 b = *reinterpret_cast<const uint4*>(rr + i);
                float2 f;
                f = unpack_bf16x2(b.x); v[i + 0] += f.x; v[i + 1] += f.y;
                f = unpack_bf16x2(b.y); v[i + 2] += f.x; v[i + 3] += f.y;
                f = unpack_bf16x2(b.z); v[i + 4] += f.x; v[i + 5] += f.y;
                f = unpack_bf16x2(b.w); v[i + 6] += f.x; v[i + 7] += f.y;
              }
            }
          }
          if (p.tp_world > 1 && p.peer_recv[0]) {
            const int owner = row / p.rows_per_rank;
            const uint32_t par = *p.op_counter & 1;
            __nv_bfloat16* o = p.peer_recv[owner] + par * p.recv_parity_stride +
                               ((size_t)p.tp_rank * p.rows_per_rank + (row - owner * p.rows_per_rank)) * p.N + col0;  // one slot per rank
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (col0 + i < p.N) {
                uint4 w;
                w.x = pack_bf16x2(v[i + 0], v[i + 1]);
                w.y = pack_bf16x2(v[i + 2], v[i + 3]);
                w.z = pack_bf16x2(v[i + 4], v[i + 5]);
                w.w = pack_bf16x2(v[i + 6], v[i + 7]);
                *reinterpret_cast<uint4*>(o + i) = w;
              }
            }
          } else if (p.out_f32) {
            float* o = reinterpret_cast<float*>(p.out) + (size_t)row * p.ldo + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              if (col0 + i < p.N)
                *reinterpret_cast<float4*>(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
            }
          } else {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.ldo + col0;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (col0 + i < p.N) {
                uint4 w;
                w.x = pack_bf16x2(v[i + 0], v[i + 1]);
                w.y = pack_bf16x2(v[i + 2], v[i + 3]);
                w.z = pack_bf16x2(v[i + 4], v[i + 5]);
                w.w = pack_bf16x2(v[i + 6], v[i + 7]);
                *reinterpret_cast<uint4*>(o + i) = w;
              }
            }
          }
        }
      }
      if (p.tp_world > 1 && p.peer_recv[0]) {
        // this warp's 32 rows x BN columns have been stored to their owner: publish
        __threadfence_system();
        __syncwarp();
        const int row0 = tm * kBM + quarter * 32;
        if (lane == 0 && row0 < p.M) {
          const int owner = row0 / p.rows_per_rank;
          const uint32_t par = *p.op_counter & 1;
          signal_counter(p.peer_rs_flags[owner] + par * p.rs_flag_parity_stride +
                         (row0 - owner * p.rows_per_rank) / 32);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        for (int x = sk_first; x <= sk_last; ++x) p.sk_flags[x * 4 + quarter] = 0;
        mbar_arrive(&bars->acc_empty[buf]);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * BN >= 32 ? 2 * BN : 32);
}

// ---------------------------------------------------------------------------------------
// CTA-pair kernel: a cluster of two CTAs computes a 256 x BN tile with cta_group::2 MMAs.
// Per 64-wide k-block each CTA stages its 128 rows of A and its BN/2 rows of W (32 KB for
// BN = 256, against 48 KB per CTA for the same 128 x 256 outputs in the 1-CTA kernel), so the
// L2 -> shared-memory traffic per FLOP drops by a third. The even CTA issues every MMA; each
// CTA's TMEM holds its 128 rows of the accumulator and its own epilogue warps store them.
// Barriers: full[s] lives in the leader and counts the bytes of both CTAs' loads; empty[s],
// acc_full[b] are signalled in both CTAs by the leader's commits; acc_empty[b] lives in the
// leader and collects the eight epilogue warps of the pair.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void epilogue_store_chunk(const GemmParams& p, float (&v)[32], int row,
                                                     int col0) {
  if (p.bias) {
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      if (col0 + i < p.N) {
        uint4 b = *reinterpret_cast<const uint4*>(p.bias + col0 + i);
        float2 f;
        f = unpack_bf16x2(b.x); v[i + 0] += f.x; v[i + 1] += f.y;
        f = unpack_bf16x2(b.y); v[i + 2] += f.x; v[i + 3] += f.y;
        f = unpack_bf16x2(b.z); v[i + 4] += f.x; v[i + 5] += f.y;
        f = unpack_bf16x2(b.w); v[i + 6] += f.x; v[i + 7] += f.y;
      }
    }
  }
  if (p.residual) {
    const __nv_bfloat16* rr = p.residual + (size_t)row * p.ldr + col0;
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      if (col0 + i < p.N) {
        uint4 b = *reinterpret_cast<const uint4*>(rr + i);
        float2 f;
        f = unpack_bf16x2(b.x); v[i + 0] += f.x; v[i + 1] += f.y;
        f = unpack_bf16x2(b.y); v[i + 2] += f.x; v[i + 3] += f.y;
        f = unpack_bf16x2(b.z); v[i + 4] += f.x; v[i + 5] += f.y;
        f = unpack_bf16x2(b.w); v[i + 6] += f.x; v[i + 7] += f.y;
      }
    }
  }
  if (p.out_f32) {
    float* o = reinterpret_cast<float*>(p.out) + (size_t)row * p.ldo + col0;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      if (col0 + i < p.N)
        *reinterpret_cast<float4*>(o + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    }
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.ldo + col0;
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      if (col0 + i < p.N) {
        uint4 w;
        w.x = pack_bf16x2(v[i + 0], v[i + 1]);
        w.y = pack_bf16x2(v[i + 2], v[i + 3]);
        w.z = pack_bf16x2(v[i + 4], v[i + 5]);
        w.w = pack_bf16x2(v[i + 6], v[i + 7]);
        *reinterpret_cast<uint4*>(o + i) = w;
      }
    }
  }
}

__device__ __forceinline__ float gated_act(float g, int kind) {
  if (kind == 0) return g / (1.f + __expf(-g));
  if (kind == 1) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * g * (1.f + tanhf(k0 * (g + k1 * g * g * g)));
  }
  return 0.5f * g * (1.f + erff(g * 0.7071067811865476f));
}
// act(gate) * up on 32 columns; both inputs are rounded to bf16 first so that the result equals
// a bf16 GEMM followed by the separate activation kernel bit for bit.
__device__ __forceinline__ void epilogue_store_gated(const GemmParams& p, const float (&g)[32],
                                                     const float (&u)[32], int row, int col0) {
  const int kind = p.act_fuse - 1;
  const int n_out = p.N >> 1;
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.ldo + col0;
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    if (col0 + i < n_out) {
      float r[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gg = __bfloat162float(__float2bfloat16(g[i + j]));
        const float uu = __bfloat162float(__float2bfloat16(u[i + j]));
        r[j] = gated_act(gg, kind) * uu;
      }
      uint4 w;
      w.x = pack_bf16x2(r[0], r[1]);
      w.y = pack_bf16x2(r[2], r[3]);
      w.z = pack_bf16x2(r[4], r[5]);
      w.w = pack_bf16x2(r[6], r[7]);
      *reinterpret_cast<uint4*>(o + i) = w;
    }
  }
}

// FP8 = false: bf16 operands, 64 elements per 128-byte smem row. FP8 = true: e4m3 operands
// (kind::f8f6f4), 128 elements per row; everything else (tiles, rings, stream-K) is shared.

template <int BN, bool FP8 = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                          const __grid_constant__ CUtensorMap tmA_alt,
                          const __grid_constant__ CUtensorMap tmB, GemmParams p) {
  constexpr int kBK = FP8 ? 128 : b200::kBK;          // elements per k-block (128 bytes per row)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  constexpr int kABytes = kBM * 128;
  constexpr int kBBytes = (BN / 2) * 128;
  constexpr int kStageBytes = kABytes + kBBytes;
  constexpr uint32_t kTmemCols = 2 * BN;
  const int stages = p.stages;
  GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(smem + (size_t)stages * kStageBytes);
  // scatter epilogue: 4 KB per epilogue warp to turn "lane = row" accumulator chunks into row-
  // contiguous 128-byte pieces before they cross NVLink
  uint8_t* stage_smem = reinterpret_cast<uint8_t*>(bars) + ((sizeof(GemmBarriers) + 127) & ~size_t(127));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;      // tiles_m counts 256-row tiles here
  const int kblocks = (p.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->acc_full[b], 1);
      mbar_init(&bars->acc_empty[b], 8);
    }
    bars->failed = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(&bars->tmem_base, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();            // the peer's barriers exist before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  pdl_wait();                 // predecessor grid complete, its writes visible
  pdl_launch_dependents();    // the successor may become resident (it waits the same way)

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      // gather mode: A has one copy per parity of the op counter, pick the one just written
      const CUtensorMap* ta = (p.ag_flags && ((*p.op_counter - 1) & 1)) ? &tmA_alt : &tmA;
      tma_prefetch_desc(ta);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      SegState seg = seg_init_w(p, kblocks, pair, npairs);
      int t, kb0, kb1;
      while (ok && seg_next(seg, num_tiles, kblocks, t, kb0, kb1)) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
        if (p.ag_flags) {
          // all-gather + GEMM: this CTA's 128 rows of the tile must have landed (four 32-row groups)
          const uint32_t par = (*p.op_counter - 1) & 1;
          const int g0 = (tm * 2 + (int)rank) * 4;
          for (int g = g0; g < g0 + 4 && ok; ++g) {
            const int need = min(32, p.M - g * 32);
            if (need > 0)
              ok = wait_counter_ge(p.ag_flags + par * p.ag_flag_parity_stride + g, need, p.status, p.peer_wait);
          }
          if (!ok) break;
          fence_proxy_async_global();
        }
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          int s = it % stages;
          uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars->empty[s], ph ^ 1, p.status)) { ok = false; break; }
          uint8_t* a_dst = smem + (size_t)s * kStageBytes;
          uint8_t* b_dst = a_dst + kABytes;
          if (rank == 0) mbar_expect_tx(&bars->full[s], 2 * kStageBytes);
          const uint32_t leader_bar = mapa_u32(smem_u32(&bars->full[s]), 0);
          tma_load_2d_pair(a_dst, ta, leader_bar, kb * kBK, tm * 2 * kBM + (int)rank * kBM);
          tma_load_2d_pair(b_dst, &tmB, leader_bar, kb * kBK, tn * BN + (int)rank * (BN / 2));
        }
      }
      if (!ok) bars->failed = 1;
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = FP8 ? umma_idesc_e4m3(2 * kBM, BN) : umma_idesc_bf16(2 * kBM, BN);
      uint32_t it = 0, tc = 0;
      bool ok = true;
      SegState seg = seg_init_w(p, kblocks, pair, npairs);
      int t, kb0, kb1;
      for (; ok && seg_next(seg, num_tiles, kblocks, t, kb0, kb1); ++tc) {
        int buf = tc & 1;
        uint32_t aph = (tc >> 1) & 1;
        if (!mbar_wait(&bars->acc_empty[buf], aph ^ 1, p.status)) { ok = false; break; }
        tc_fence_after_sync();
        uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          int s = it % stages;
          uint32_t ph = (it / stages) & 1;
          if (!mbar_wait(&bars->full[s], ph, p.status)) { ok = false; break; }
          tc_fence_after_sync();
          uint32_t a_addr = smem_u32(smem + (size_t)s * kStageBytes);
          uint32_t b_addr = a_addr + kABytes;
          uint64_t adesc = umma_desc_k_sw128(a_addr, 1024);
          uint64_t bdesc = umma_desc_k_sw128(b_addr, 1024);
#pragma unroll
          for (int k = 0; k < 4; ++k) {     // four 32-byte K steps per 128-byte row
            if (FP8) umma_f8f6f4_ss_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, kb != kb0 || k != 0);
            else umma_bf16_ss_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, kb != kb0 || k != 0);
          }
          umma_commit_pair(&bars->empty[s], 3);
        }
        if (ok) umma_commit_pair(&bars->acc_full[buf], 3);
      }
      if (!ok) bars->failed = 1;
    }
  } else {
    // ---------------- Epilogue (warps 2..5 of both CTAs) ----------------
    const int quarter = warp & 3;
    const int me = blockIdx.x;                        // partial slot / flag owner
    uint32_t tc = 0;
    bool ok = true;
    SegState seg = seg_init_w(p, kblocks, pair, npairs);
    int t, kb0, kb1;
    for (; ok && seg_next(seg, num_tiles, kblocks, t, kb0, kb1); ++tc) {
      int tm, tn;
      tile_coords(t, p.tiles_m, p.tiles_n, tm, tn);
      int buf = tc & 1;
      uint32_t aph = (tc >> 1) & 1;
      ok = mbar_wait(&bars->acc_full[buf], aph, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const int row = tm * 2 * kBM + (int)rank * kBM + quarter * 32 + lane;
      const uint32_t t_addr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
      const uint32_t leader_acc_empty = mapa_u32(smem_u32(&bars->acc_empty[buf]), 0);
      if (kb0 > 0) {
        float* dst = p.sk_partials + (size_t)me * kBM * BN + quarter * 32 + lane;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_addr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) __stcg(dst + (size_t)(c * 32 + i) * kBM, __uint_as_float(r[i]));
        }
        __threadfence();
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          uint32_t one = 1;
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.sk_flags + me * 4 + quarter), "r"(one)
                       : "memory");
          mbar_arrive_cluster(leader_acc_empty);
        }
        continue;
      }
      int sk_first = 0, sk_last = -1;                 // contributing pairs
      if (kb1 < kblocks) {
        const int tile_end = (t + 1) * kblocks;
        sk_first = pair + 1;
        sk_last = pair;
        while (sk_last + 1 < npairs && sk_range_start_w(sk_last + 1, p.sk * kblocks, npairs) < tile_end)
          ++sk_last;
        for (int x = sk_first; x <= sk_last && ok; ++x)
          ok = wait_flag_set(p.sk_flags + (x * 2 + (int)rank) * 4 + quarter, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      float fp8_sa = 1.f, fp8_sw = 1.f;
      if (FP8) {
        fp8_sa = p.scale_a_per_token ? (row < p.M ? __ldg(p.scale_a + row) : 0.f) : __ldg(p.scale_a);
        if (!p.scale_w_per_channel) fp8_sw = __ldg(p.scale_w);
      }
      // accumulator columns [c * 32, c * 32 + 32) of this thread's row, stream-K partials added
      auto load_chunk = [&](int c, float (&v)[32]) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        for (int x = sk_first; x <= sk_last; ++x) {
          const float* src = p.sk_partials + (size_t)(x * 2 + (int)rank) * kBM * BN +
                             (size_t)c * 32 * kBM + quarter * 32 + lane;
          float f[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = __ldcg(src + (size_t)i * kBM);
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] += f[i];
        }
        if (FP8) {
          // scales fetched as vectors ahead of their use: scalar loads between the stores of the
          // previous chunk would each wait out their own latency (one warp per scheduler here)
          const int col = tn * BN + c * 32;
          if (p.scale_w_per_channel) {
            float4 sw[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              sw[i] = col + i * 4 < p.N ? __ldg(reinterpret_cast<const float4*>(p.scale_w + col) + i)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              v[i * 4 + 0] *= fp8_sa * sw[i].x; v[i * 4 + 1] *= fp8_sa * sw[i].y;
              v[i * 4 + 2] *= fp8_sa * sw[i].z; v[i * 4 + 3] *= fp8_sa * sw[i].w;
            }
          } else {
            const float s1 = fp8_sa * fp8_sw;
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= s1;
          }
        }
      };
      if (BN == 256 && p.act_fuse) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float g[32], u[32];
          load_chunk(c, g);
          load_chunk(c + 4, u);
          const int col0 = tn * 128 + c * 32;
          if (row < p.M && col0 < (p.N >> 1)) epilogue_store_gated(p, g, u, row, col0);
        }
      } else if (!FP8 && p.tp_world > 1 && p.peer_recv[0]) {
        // GEMM + reduce-scatter: the bf16 partial rows go to the rank that owns them. Two 32-column
        // accumulator chunks are staged in shared memory (16-byte pieces, XOR-swizzled by row so
        // that neither side has bank conflicts) and leave as 128 contiguous bytes per row, eight
        // lanes to a row, instead of 32 separate 16-byte pieces per store instruction.
        uint8_t* st = stage_smem + (size_t)quarter * 4096;
        const uint32_t par = *p.op_counter & 1;
        const int row_base = tm * 2 * kBM + (int)rank * kBM + quarter * 32;
#pragma unroll 1
        for (int c2 = 0; c2 < BN / 64; ++c2) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float v[32];
            load_chunk(c2 * 2 + h, v);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint4 w;
              w.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
              w.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
              w.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
              w.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
              const int piece = h * 4 + j;
              *reinterpret_cast<uint4*>(st + lane * 128 + ((piece ^ (lane & 7)) << 4)) = w;
            }
          }
          __syncwarp();
          const int piece = lane & 7;
          const int col = tn * BN + c2 * 64 + piece * 8;
#pragma unroll
          for (int rr = 0; rr < 8; ++rr) {
            const int rl = rr * 4 + (lane >> 3);
            const int grow = row_base + rl;
            if (grow < p.M && col < p.N) {
              const uint4 w = *reinterpret_cast<const uint4*>(st + rl * 128 + ((piece ^ (rl & 7)) << 4));
              const int owner = grow / p.rows_per_rank;
              __nv_bfloat16* o = p.peer_recv[owner] + par * p.recv_parity_stride +
                                 ((size_t)p.tp_rank * p.rows_per_rank + (grow - owner * p.rows_per_rank)) * p.N + col;
              *reinterpret_cast<uint4*>(o) = w;
            }
          }
          __syncwarp();
        }
        // this warp's 32 rows x BN columns are on their way to the owner: publish
        __threadfence_system();
        __syncwarp();
        if (lane == 0 && row_base < p.M) {
          const int owner = row_base / p.rows_per_rank;
          signal_counter(p.peer_rs_flags[owner] + par * p.rs_flag_parity_stride +
                         (row_base - owner * p.rows_per_rank) / 32);
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          float v[32];
          load_chunk(c, v);
          const int col0 = tn * BN + c * 32;
          if (row < p.M && col0 < p.N) epilogue_store_chunk(p, v, row, col0);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        for (int x = sk_first; x <= sk_last; ++x) p.sk_flags[(x * 2 + (int)rank) * 4 + quarter] = 0;
        mbar_arrive_cluster(leader_acc_empty);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();            // neither CTA frees while the other still reads its accumulators
  tc_fence_after_sync();
  if (warp == 1) tmem_dealloc_pair(tmem_base, kTmemCols);
}

// ---------------------------------------------------------------------------------------
// Small-M swap-AB split-K kernel.
// TMEM accumulator: lane = weight row (output column n), column = token m.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_bf16_swap_kernel(const __grid_constant__ CUtensorMap tmW,
                          const __grid_constant__ CUtensorMap tmA,
                          const __grid_constant__ CUtensorMap tmA_alt, GemmParams p,
                          uint32_t tmem_cols) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~uintptr_t(1023));
  constexpr int kWBytes = kBM * kBK * 2;
  const int a_bytes = p.mp * kBK * 2;
  // Keep every tile 1024-byte aligned (mp is a multiple of 16 -> a_bytes multiple of 2048).
  const int stage_bytes = kWBytes + a_bytes;
  const int stages = p.stages;
  GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(smem + (size_t)stages * stage_bytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tn = blockIdx.x;
  const int split = blockIdx.y;
  const int bz = blockIdx.z;
  const int kblocks_total = (p.K + kBK - 1) / kBK;
  const int kb0 = split * p.kb_per_split;
  const int kb1 = min(kblocks_total, kb0 + p.kb_per_split);
  const int nkb = kb1 - kb0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->acc_full[0], 1);
    bars->failed = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;
  // Weights that nothing in the stream writes: fill the first ring stages' weight halves while
  // the predecessor kernel is still running; the activation halves follow after the wait.
  int npre = 0;
  if (warp == 0 && lane == 0 && p.w_early && !p.ag_flags) {
    tma_prefetch_desc(&tmW);
    npre = min(nkb, stages);
    for (int i = 0; i < npre; ++i) {
      mbar_expect_tx(&bars->full[i], stage_bytes);
      tma_load_2d(smem + (size_t)i * stage_bytes, &tmW, &bars->full[i], (kb0 + i) * kBK, bz * p.N + tn * kBM);
    }
  }
  pdl_wait();                 // predecessor grid complete, its writes visible
  pdl_launch_dependents();    // the successor may become resident (it waits the same way)

  if (warp == 0) {
    if (lane == 0) {
      const CUtensorMap* ta = (p.ag_flags && ((*p.op_counter - 1) & 1)) ? &tmA_alt : &tmA;
      tma_prefetch_desc(&tmW);
      tma_prefetch_desc(ta);
      bool ag_ok = true;
      if (p.ag_flags) {
        const uint32_t par = (*p.op_counter - 1) & 1;
        for (int g = 0; g * 32 < p.M && ag_ok; ++g)
          ag_ok = wait_counter_ge(p.ag_flags + par * p.ag_flag_parity_stride + g,
                                  min(32, p.M - g * 32), p.status, p.peer_wait);
        fence_proxy_async_global();
      }
      for (int i = 0; i < nkb && ag_ok; ++i) {
        int s = i % stages;
        uint32_t ph = (i / stages) & 1;
        if (!mbar_wait(&bars->empty[s], ph ^ 1, p.status)) { bars->failed = 1; break; }
        uint8_t* w_dst = smem + (size_t)s * stage_bytes;
        uint8_t* a_dst = w_dst + kWBytes;
        if (i >= npre) {         // (the first npre stages already expect their bytes and hold W)
          mbar_expect_tx(&bars->full[s], stage_bytes);
          tma_load_2d(w_dst, &tmW, &bars->full[s], (kb0 + i) * kBK, bz * p.N + tn * kBM);
        }
        tma_load_2d(a_dst, ta, &bars->full[s], bz * p.batch_a_cols + (kb0 + i) * kBK, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(kBM, p.mp);
      bool ok = true;
      for (int i = 0; i < nkb; ++i) {
        int s = i % stages;
        uint32_t ph = (i / stages) & 1;
        if (!mbar_wait(&bars->full[s], ph, p.status)) { ok = false; break; }
        tc_fence_after_sync();
        uint32_t w_addr = smem_u32(smem + (size_t)s * stage_bytes);
        uint32_t a_addr = w_addr + kWBytes;
        uint64_t wdesc = umma_desc_k_sw128(w_addr, 1024);
        uint64_t adesc = umma_desc_k_sw128(a_addr, 1024);
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k)
          umma_bf16_ss(tmem_base, wdesc + 2 * k, adesc + 2 * k, idesc, (i | k) != 0);
        umma_commit(&bars->empty[s]);
      }
      if (ok) umma_commit(&bars->acc_full[0]);
      else bars->failed = 1;
    }
  } else {
    const int quarter = warp & 3;
    bool ok = true;
    if (nkb > 0) ok = mbar_wait(&bars->acc_full[0], 0, p.status);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after_sync();
    const int n = tn * kBM + quarter * 32 + lane;
    const uint32_t t_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    if (ok) {
      float bias_v = 0.f;
      if (p.bias && p.splits == 1 && n < p.N) bias_v = __bfloat162float(p.bias[n]);
      for (int c = 0; c < p.mp / 16; ++c) {
        uint32_t r[16];
        if (nkb > 0) {
          tmem_ld_32x32b_x16(t_addr + c * 16, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = 0;
        }
        if (n < p.N) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            int m = c * 16 + i;
            if (m < p.M) {
              float v = __uint_as_float(r[i]);
              if (p.tp_world > 1 && p.peer_recv[0]) {
                // (rank, k-split) is one virtual source slot of the owner's receive buffer
                const int owner = m / p.rows_per_rank;
                const uint32_t par = *p.op_counter & 1;
                p.peer_recv[owner][par * p.recv_parity_stride +
                                   ((size_t)(p.tp_rank * p.splits + split) * p.rows_per_rank +
                                    (m - owner * p.rows_per_rank)) * p.N + n] = __float2bfloat16(v);
              } else if (p.splits > 1) {
                p.workspace[((size_t)split * p.M + m) * p.N + n] = v;
              } else {
                v += bias_v;
                if (p.residual) v += __bfloat162float(p.residual[(size_t)m * p.ldr + n]);
                const size_t o = (size_t)bz * p.batch_out_stride + (size_t)m * p.ldo + n;
                if (p.out_f32)
                  reinterpret_cast<float*>(p.out)[o] = v;
                else
                  reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16(v);
              }
            }
          }
        }
      }
      if (p.tp_world > 1 && p.peer_recv[0]) {
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const uint32_t par = *p.op_counter & 1;
          for (int g = 0; g * 32 < p.M; ++g) {
            const int row0 = g * 32, owner = row0 / p.rows_per_rank;
            signal_counter(p.peer_rs_flags[owner] + par * p.rs_flag_parity_stride +
                           (row0 - owner * p.rows_per_rank) / 32);
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

// out[m,n] = sum_s ws[s,m,n] (+bias) (+residual), splits summed in ascending order.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, int splits, int M, int N,
                                     void* out, int ldo, int out_f32,
                                     const __nv_bfloat16* __restrict__ bias,
                                     const __nv_bfloat16* __restrict__ residual, int ldr) {
  pdl_wait();                 // predecessor grid complete, its writes visible
  pdl_launch_dependents();    // the successor may become resident (it waits the same way)
  const int n4 = N >> 2;
  const size_t total = (size_t)M * n4;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    int m = (int)(idx / n4);
    int n = (int)(idx % n4) * 4;
    float4 acc = *reinterpret_cast<const float4*>(ws + (size_t)m * N + n);
    for (int s = 1; s < splits; ++s) {
      float4 v = *reinterpret_cast<const float4*>(ws + ((size_t)s * M + m) * N + n);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (bias) {
      uint2 b = *reinterpret_cast<const uint2*>(bias + n);
      float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y);
      acc.x += f0.x; acc.y += f0.y; acc.z += f1.x; acc.w += f1.y;
    }
    if (residual) {
      uint2 b = *reinterpret_cast<const uint2*>(residual + (size_t)m * ldr + n);
      float2 f0 = unpack_bf16x2(b.x), f1 = unpack_bf16x2(b.y);
      acc.x += f0.x; acc.y += f0.y; acc.z += f1.x; acc.w += f1.y;
    }
    if (out_f32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + (size_t)m * ldo + n) = acc;
    } else {
      uint2 w;
      w.x = pack_bf16x2(acc.x, acc.y);
      w.y = pack_bf16x2(acc.z, acc.w);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + (size_t)m * ldo + n) = w;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Host launcher
// ---------------------------------------------------------------------------------------
struct TmapKey {
  const void* p;
  uint64_t rows, cols, ld;
  uint32_t br, bc;
  bool operator==(const TmapKey& o) const {
    return p == o.p && rows == o.rows && cols == o.cols && ld == o.ld && br == o.br && bc == o.bc;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.p);
    h ^= k.rows * 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    h ^= k.cols * 0xc2b2ae3d27d4eb4full + (h << 6) + (h >> 2);
    h ^= k.ld * 0x165667b19e3779f9ull + (h << 6) + (h >> 2);
    h ^= ((uint64_t)k.br << 32 | k.bc) + (h << 6) + (h >> 2);
    return h;
  }
};

static bool get_tmap_bf16(CUtensorMap* out, const void* p, uint64_t rows, uint64_t cols,
                          uint64_t ld, uint32_t br, uint32_t bc) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  TmapKey key{p, rows, cols, ld, br, bc};
  {
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  CUtensorMap m;
  if (!encode_tmap_2d(&m, p, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, rows, cols, ld, br, bc,
                      CU_TENSOR_MAP_SWIZZLE_128B))
    return false;
  std::lock_guard<std::mutex> lock(mu);
  if (cache.size() > 65536) cache.clear();
  cache[key] = m;
  *out = m;
  return true;
}

static constexpr int kSmemBudget = 220 * 1024;

// Stream-K scratch of the current device: one 128 x 256 fp32 partial per CTA plus four flags per
// CTA. b200_init_device() allocates it when a device is set up; a first use that finds none
// allocates it too unless the stream is capturing (a capture that early keeps the plan without
// stream-K). GEMMs that share it must be ordered on one stream (two streams running stream-K
// GEMMs at once would mix their partials).
static bool streamk_scratch(cudaStream_t stream, float** partials, uint32_t** flags) {
  static std::mutex mu;
  static float* g_part[64] = {};
  static uint32_t* g_flags[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (!g_part[dev]) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone)
      return false;
    const size_t n = (size_t)b200_num_sms() * kBM * 256 * sizeof(float);
    float* pp = nullptr;
    uint32_t* ff = nullptr;
    if (cudaMalloc(&pp, n) != cudaSuccess) { cudaGetLastError(); return false; }
    if (cudaMalloc(&ff, (size_t)b200_num_sms() * 4 * sizeof(uint32_t)) != cudaSuccess) {
      cudaGetLastError();
      cudaFree(pp);
      return false;
    }
    cudaMemset(ff, 0, (size_t)b200_num_sms() * 4 * sizeof(uint32_t));
    g_part[dev] = pp;
    g_flags[dev] = ff;
  }
  *partials = g_part[dev];
  *flags = g_flags[dev];
  return true;
}

// Stream-K plan for `tiles` tiles of `kblocks` k-blocks on at most `max_workers` workers.
// Fewer tiles than workers: every tile is cut into the same number of parts (workers that share
// an operand stay in step). Otherwise only the tiles of the ragged last wave are cut.
static void plan_streamk(long tiles, int kblocks, int max_workers, int* nworkers, int* sk_tiles) {
  *nworkers = tiles < max_workers ? (int)tiles : max_workers;
  *sk_tiles = 0;
  if (kblocks < 16 || tiles <= 0) return;
  if (tiles < max_workers) {
    int parts = max_workers / (int)tiles;
    while (parts >= 2 && kblocks / parts < 8) --parts;
    if (parts >= 2) {
      *nworkers = (int)tiles * parts;
      *sk_tiles = (int)tiles;
    }
    // (With 50-88 % of the workers owning a tile, cutting the whole k-range evenly over all workers
    // was measured slower than leaving the rest idle: 71 against 60 us for 32 x 28672 x 4096. The
    // tiles lose their common k-phase and with it the sharing of the activation rows in L2.)
    return;
  }
  const int r = (int)(tiles % max_workers);
  if (r == 0 || r * 100 >= max_workers * 85) return;
  // a sliver of a wave would be cut too finely (one owner summing dozens of partials): take a
  // whole wave into the region with it
  *sk_tiles = ((long)r * kblocks < 8l * max_workers) ? r + max_workers : r;
}

template <int BN>
static int launch_tn(const CUtensorMap& tmA, const CUtensorMap& tmA2, const CUtensorMap& tmB,
                     GemmParams& p, cudaStream_t stream) {
  constexpr int stage_bytes = kBM * kBK * 2 + BN * kBK * 2;
  int stages = (kSmemBudget - 2048) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  int kblocks = (p.K + kBK - 1) / kBK;
  if (stages > kblocks + 1) stages = kblocks + 1;
  if (stages < 2) stages = 2;
  p.stages = stages;
  size_t smem = (size_t)stages * stage_bytes + 1024 + sizeof(GemmBarriers);
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(gemm_bf16_tn_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         kSmemBudget + 4096);
  }
  int tiles = p.tiles_m * p.tiles_n;
  int grid = tiles < b200_num_sms() ? tiles : b200_num_sms();
  if (p.sk) {   // on entry: stream-K wanted; from here on: tiles in the stream-K region
    int sk_tiles = 0;
    plan_streamk(tiles, kblocks, b200_num_sms(), &grid, &sk_tiles);
    if (sk_tiles && !streamk_scratch(stream, &p.sk_partials, &p.sk_flags)) {
      sk_tiles = 0;
      grid = tiles < b200_num_sms() ? tiles : b200_num_sms();
    }
    p.sk = sk_tiles;
  }
  // Tensor-parallel launches use programmatic dependent launch like the rest of the chain: the
  // kernel touches nothing a peer can see before its wait on the predecessor, every CTA of a
  // grid is resident before its dependents may start (the grid never exceeds the SM count), and
  // a kernel only ever waits for work that precedes it in its peers' streams.
  return launch_pdl(gemm_bf16_tn_kernel<BN>, dim3(grid), dim3(kGemmThreads), smem, stream, tmA, tmA2, tmB, p) ==
                 cudaSuccess ? 0 : -2;
}

// CTA-pair launch: clusters of two, as many as can be resident at once (at most one per SM pair).
template <int BN, bool FP8 = false>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmA2, const CUtensorMap& tmB, GemmParams& p,
                       cudaStream_t stream) {
  constexpr int stage_bytes = kBM * 128 + (BN / 2) * 128;
  constexpr int kbk = FP8 ? 128 : kBK;
  // the scatter epilogue stages its stores in 16 KB behind the barriers
  const int epi_bytes = (p.tp_world > 1 && p.peer_recv[0]) ? 16384 + 128 : 0;
  int stages = (kSmemBudget - 2048 - epi_bytes) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  int kblocks = (p.K + kbk - 1) / kbk;
  if (stages > kblocks + 1) stages = kblocks + 1;
  if (stages < 2) stages = 2;
  p.stages = stages;
  size_t smem = (size_t)stages * stage_bytes + 1024 + sizeof(GemmBarriers) + epi_bytes;
  static int max_clusters[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -2;
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // programmatic dependent launch: barriers, TMEM and the cluster handshake are set up while the
  // predecessor drains; the kernel reads and writes nothing global before its pdl_wait()
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = kSmemBudget + 4096;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (!max_clusters[dev]) {
    cudaFuncSetAttribute(gemm_bf16_pair_kernel<BN, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         kSmemBudget + 4096);
    cfg.gridDim = dim3(b200_num_sms() & ~1);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_bf16_pair_kernel<BN, FP8>, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      return -2;
    }
    max_clusters[dev] = n;
  }
  const long tiles = (long)p.tiles_m * p.tiles_n;
  int max_pairs = max_clusters[dev];
  if (max_pairs > b200_num_sms() / 2) max_pairs = b200_num_sms() / 2;
  int pairs = tiles < max_pairs ? (int)tiles : max_pairs;
  if (p.sk) {
    int sk_tiles = 0;
    plan_streamk(tiles, kblocks, max_pairs, &pairs, &sk_tiles);
    if (sk_tiles && !streamk_scratch(stream, &p.sk_partials, &p.sk_flags)) {
      sk_tiles = 0;
      pairs = tiles < max_pairs ? (int)tiles : max_pairs;
    }
    p.sk = sk_tiles;
  }
  cfg.gridDim = dim3(2 * pairs);
  cfg.dynamicSmemBytes = smem;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, gemm_bf16_pair_kernel<BN, FP8>, tmA, tmA2, tmB, p) != cudaSuccess) {
    cudaGetLastError();
    return -2;
  }
  return 0;
}

}  // namespace b200

using namespace b200;

static bool tp_pair_enabled() {
  static const bool on = [] {
    const char* e = getenv("B200_TP_PAIR");
    return !(e && e[0] == '0');
  }();
  return on;
}

static int gemm_bf16_impl(const void* A, int lda, const void* W, int ldw, void* out, int ldo,
                          int out_f32, const void* bias, const void* residual, int ldr, int M,
                          int N, int K, void* workspace, size_t ws_bytes, int force_path,
                          const B200TpGemm* tp, cudaStream_t stream, int act_fuse = 0);


extern "C" int b200_gemm_bf16(const void* A, int lda, const void* W, int ldw, void* out, int ldo,
                              int out_f32, const void* bias, const void* residual, int ldr, int M,
                              int N, int K, void* workspace, size_t ws_bytes, int force_path,
                              cudaStream_t stream) {
  return gemm_bf16_impl(A, lda, W, ldw, out, ldo, out_f32, bias, residual, ldr, M, N, K, workspace,
                        ws_bytes, force_path, nullptr, stream);
}

// Gated-MLP first half in one kernel: out[M, N / 2] = act(A W_gate^T) * (A W_up^T), where W holds
// the gate and up rows interleaved in blocks of 128 ([128 gate | 128 up] per 256 rows) so that
// every 256-column accumulator tile contains both halves of 128 outputs. M > 256 (the CTA-pair
// kernel); smaller batches run the plain GEMM and the interleave-aware activation kernel.
// kind: 0 SiLU, 1 GELU-tanh, 2 GELU-erf. Replaces MatmulBT + SiluAndMul / GeluAndMul of the
// reference (src/vt/cuda/cuda_matmul.cu, cuda_ops.cu) on the prefill-sized path.
extern "C" int b200_gemm_bf16_gated(const void* A, int lda, const void* W, int ldw, void* out,
                                    int ldo, int M, int N, int K, int kind, int force_path,
                                    cudaStream_t stream) {
  if (kind < 0 || kind > 2) return -1;
  return gemm_bf16_impl(A, lda, W, ldw, out, ldo, 0, nullptr, nullptr, 0, M, N, K, nullptr, 0,
                        force_path, nullptr, stream, kind + 1);
}

// e4m3 x e4m3 -> bf16 on the CTA-pair kernel (M > 256): out = (A W^T) * a_scale * w_scale (+ bias).
// Reference: MatmulFp8CublasLt / MatmulFp8Cutlass in src/vt/cuda/cuda_matmul.cu.
extern "C" int b200_gemm_fp8_pair(const void* A, int lda, const void* W, int ldw, void* out, int ldo,
                                  const float* a_scale, const float* w_scale, int w_scale_per_channel,
                                  const void* bias, int M, int N, int K, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 15) || (lda & 15) || (ldw & 15) || (N & 7) || (ldo & 7)) return -1;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.scale_a = a_scale; p.scale_w = w_scale; p.scale_w_per_channel = w_scale_per_channel & 1;
  p.scale_a_per_token = (w_scale_per_channel >> 1) & 1;
  p.status = device_status_word();
  p.sk = 1;
  p.tiles_m = (M + 2 * kBM - 1) / (2 * kBM);
  p.tiles_n = (N + 255) / 256;
  CUtensorMap tA, tB;
  if (!encode_tmap_2d(&tA, A, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K, lda, kBM, 128, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !encode_tmap_2d(&tB, W, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K, ldw, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B))
    return -3;
  return launch_pair<256, true>(tA, tA, tB, p, stream);
}

// Same GEMM with the tensor-parallel prologue / epilogue described by `tp`.
// Returns in *expected_rs the arrival count the owner of a 32-row group must wait for.
extern "C" int b200_gemm_bf16_tp(const void* A, int lda, const void* W, int ldw, void* out,
                                 int ldo, int M, int N, int K, const B200TpGemm* tp,
                                 int* expected_rs, cudaStream_t stream) {
  if (!tp || tp->world < 1 || tp->world > 8) return -1;
  if (tp->scatter && (tp->rows_per_rank <= 0 || (tp->rows_per_rank & 31))) return -1;
  const int tiles_n = (N + 127) / 128;
  const bool swap = (M <= 256);
  if (expected_rs) {
    if (swap) {
      const int kblocks = (K + kBK - 1) / kBK;
      int s = tp->scatter_splits > 0 ? tp->scatter_splits : 1;
      const int kb_per = (kblocks + s - 1) / s;
      s = (kblocks + kb_per - 1) / kb_per;      // the launcher's effective split count
      *expected_rs = tp->world * tiles_n * 4 * s;
    }
    else if (tp_pair_enabled()) {
      *expected_rs = tp->world * (N > 128 ? (N + 255) / 256 : (N + 127) / 128);   // pair tiles
    } else {
      // the tiled path picks BN below; mirror the choice
      const int sms = b200_num_sms();
      int tm = (M + 127) / 128, tn256 = (N + 255) / 256, tn128 = (N + 127) / 128;
      long w256 = ((long)tm * tn256 + sms - 1) / sms, w128 = ((long)tm * tn128 + sms - 1) / sms;
      *expected_rs = tp->world * ((N >= 256 && w256 * 2 * 100 <= w128 * 135) ? tn256 : tn128);
    }
  }
  // gather mode may fuse the gated activation (W rows in [128 gate | 128 up] blocks, out[M, N / 2])
  const int act = (!swap && tp->gather && !tp->scatter && tp_pair_enabled()) ? tp->act_fuse : 0;
  return gemm_bf16_impl(A, lda, W, ldw, out, ldo, tp->scatter ? 0 : tp->out_f32, nullptr, nullptr,
                        0, M, N, K, nullptr, 0, swap ? 2 : 1, tp, stream, act);
}

static int gemm_bf16_impl(const void* A, int lda, const void* W, int ldw, void* out, int ldo,
                          int out_f32, const void* bias, const void* residual, int ldr, int M,
                          int N, int K, void* workspace, size_t ws_bytes, int force_path,
                          const B200TpGemm* tp, cudaStream_t stream, int act_fuse) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  // bit 8 of force_path: W is a constant weight (nothing in the stream writes it)
  const int w_early = (force_path >> 8) & 1;
  force_path &= 0xff;
  if (act_fuse && ((tp && tp->scatter) || M <= 128 || (N & 255) || bias || residual || out_f32)) return -1;
  if (act_fuse && force_path == 0) force_path = 9;      // the gated epilogue lives in the pair kernel
  if ((K & 7) || (lda & 7) || (ldw & 7) || (N & 7) || (ldo & 7) || (residual && (ldr & 7))) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return -1;
  if (tp && tp->scatter && !out) out = const_cast<void*>(A);  // unused by the scatter epilogue
  GemmParams p{};
  p.w_early = (w_early && !tp) ? 1 : 0;
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.out_f32 = out_f32;
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.status = device_status_word();
  p.peer_wait = peer_wait_cycles();
  if (tp) {
    p.tp_world = tp->world;
    p.tp_rank = tp->rank;
    p.rows_per_rank = tp->rows_per_rank;
    p.op_counter = reinterpret_cast<const uint32_t*>(tp->op_counter);
    if (tp->scatter) {
      for (int i = 0; i < tp->world; ++i) {
        p.peer_recv[i] = reinterpret_cast<__nv_bfloat16*>(tp->peer_recv[i]);
        p.peer_rs_flags[i] = reinterpret_cast<uint32_t*>(tp->peer_rs_flags[i]);
      }
      p.recv_parity_stride = tp->recv_parity_stride;
      p.rs_flag_parity_stride = tp->rs_flag_parity_stride;
    }
    if (tp->gather) {
      p.ag_flags = reinterpret_cast<const uint32_t*>(tp->ag_flags);
      p.ag_flag_parity_stride = tp->ag_flag_parity_stride;
    }
  }
  const int sms = b200_num_sms();
  const int kblocks = (K + kBK - 1) / kBK;

  bool use_swap = (M <= 256);
  // Small batches. An MMA instruction takes about the same time whatever its N, so swap-AB (the
  // batch as the narrow N operand) spends one instruction per 128 weight rows x 16 k and becomes
  // issue-bound on wide weight matrices; there the batch goes on the (padded) M side and 256
  // weight rows share an instruction, with stream-K filling the SMs. Measured on B200:
  // N >= 16384: 1-CTA 128 x 256 tiles + stream-K up to 128 rows, CTA pairs above;
  // narrower matrices: swap-AB up to 128 rows, 128 x 128 tiles + stream-K above.
  if (force_path == 0 && !tp && M <= 256) {
    if (N >= 16384) force_path = M <= 128 ? 5 : 9;
    else if (M > 128) force_path = 6;
  }
  if (force_path == 1 || force_path >= 3) use_swap = false;     // an explicit tiling was asked for
  if (force_path == 2 && M <= 256) use_swap = true;

  if (use_swap) {
    int mp = (M + 15) & ~15;
    p.mp = mp;
    p.tiles_n = (N + kBM - 1) / kBM;
    int splits = 1;
    if (p.tiles_n < sms && !(tp && tp->scatter)) {
      splits = sms / p.tiles_n;       // whole CTAs per SM: one wave, never a ragged second one
      int max_by_k = kblocks / 4;
      if (max_by_k < 1) max_by_k = 1;
      if (splits > max_by_k) splits = max_by_k;
      if (splits > 16) splits = 16;
    }
    if (tp && tp->scatter) splits = tp->scatter_splits > 0 ? tp->scatter_splits : 1;
    if (splits > 1 && !(tp && tp->scatter)) {
      size_t need = (size_t)splits * M * N * sizeof(float);
      while (splits > 1 && (workspace == nullptr || need > ws_bytes)) {
        --splits;
        need = (size_t)splits * M * N * sizeof(float);
      }
    }
    int kb_per = (kblocks + splits - 1) / splits;
    splits = (kblocks + kb_per - 1) / kb_per;
    p.splits = splits;
    p.kb_per_split = kb_per;
    p.workspace = reinterpret_cast<float*>(workspace);
    int stage_bytes = kBM * kBK * 2 + mp * kBK * 2;
    int stages = (kSmemBudget - 2048) / stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages > kb_per) stages = kb_per;
    if (stages < 2) stages = 2;
    p.stages = stages;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < mp) tmem_cols <<= 1;
    CUtensorMap tmW, tmA, tmA2;
    if (!get_tmap_bf16(&tmW, W, N, K, ldw, kBM, kBK)) return -3;
    if (!get_tmap_bf16(&tmA, A, M, K, lda, mp, kBK)) return -3;
    tmA2 = tmA;
    if (tp && tp->gather && tp->a_alt && !get_tmap_bf16(&tmA2, tp->a_alt, M, K, lda, mp, kBK)) return -3;
    static PerDeviceOnce attr_once;
    if (attr_once.first()) {
      cudaFuncSetAttribute(gemm_bf16_swap_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kSmemBudget + 4096);
    }
    size_t smem = (size_t)stages * stage_bytes + 1024 + sizeof(GemmBarriers);
    dim3 grid(p.tiles_n, splits);
    if (tp) {
      gemm_bf16_swap_kernel<<<grid, kGemmThreads, smem, stream>>>(tmW, tmA, tmA2, p, tmem_cols);
      if (cudaGetLastError() != cudaSuccess) return -2;
    } else if (launch_pdl(gemm_bf16_swap_kernel, grid, dim3(kGemmThreads), smem, stream, tmW, tmA, tmA2, p,
                          tmem_cols) != cudaSuccess) {
      return -2;
    }
    if (splits > 1 && !(tp && tp->scatter)) {
      size_t total = (size_t)M * (N / 4);
      int blocks = (int)((total + 255) / 256);
      if (blocks > sms * 8) blocks = sms * 8;
      if (tp) {
        splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(p.workspace, splits, M, N, out, ldo,
                                                         out_f32, p.bias, p.residual, ldr);
        if (cudaGetLastError() != cudaSuccess) return -2;
      } else if (launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream, (const float*)p.workspace,
                            splits, M, N, out, ldo, out_f32, p.bias, p.residual, ldr) != cudaSuccess) {
        return -2;
      }
    }
    return 0;
  }

  p.tiles_m = (M + kBM - 1) / kBM;
  int tn256 = (N + 255) / 256, tn128 = (N + 127) / 128;
  long waves256 = ((long)p.tiles_m * tn256 + sms - 1) / sms;
  long waves128 = ((long)p.tiles_m * tn128 + sms - 1) / sms;
  // a 128 x 256 tile runs at about 1.6x the per-tile rate of two 128 x 128 tiles (operand traffic per
  // FLOP), so the wide tile wins unless it needs a third more waves
  bool use256 = (N >= 256 && waves256 * 2 * 100 <= waves128 * 135);
  if (force_path == 3) use256 = false;
  if (force_path == 4) use256 = true;
  // force_path: 0 auto | 1 tiled 1-CTA | 3 / 4 1-CTA with BN 128 / 256 | 5 / 6 1-CTA BN 256 / 128
  // with stream-K | 7 / 8 CTA pairs with 256 x 256 / 256 x 128 tiles | 9 / 10 pairs with stream-K.
  // Plain GEMMs above the small-M range run on CTA pairs; the tensor-parallel prologue and
  // epilogue live in the 1-CTA kernel.
  if (force_path == 5) { use256 = true; p.sk = !tp; }
  if (force_path == 6) { use256 = false; p.sk = !tp; }
  // tensor-parallel shards are narrow (N / world or K / world): few tiles or a ragged last wave
  // are the rule, so the tiled path always plans stream-K there
  if (tp && force_path == 1) p.sk = 1;
  // 256-row pair tiles pad M up to a multiple of 256; where 128-row tiles would do noticeably
  // fewer rows (e.g. M = 1056: 1280 against 1152) the 1-CTA 128 x 256 tile with stream-K is faster
  // (measured 907-1253 against 699-1175 TFLOP/s on the four Llama-8B projections at M = 1056).
  if (force_path == 0 && !tp && !act_fuse && N >= 256) {
    const long rows256 = (long)((M + 255) / 256) * 256, rows128 = (long)((M + 127) / 128) * 128;
    if (rows256 * 100 > rows128 * 108) { force_path = 5; use256 = true; p.sk = 1; }
  }
  // Tensor-parallel GEMMs above the small-M range run on CTA pairs as well (gather prologue,
  // staged scatter epilogue); B200_TP_PAIR=0 keeps them on the 1-CTA tile.
  const bool tp_pair = tp && force_path == 1 && M > 256 && tp_pair_enabled();
  const bool pair_path = tp_pair || (!tp && (force_path == 0 || (force_path >= 7 && force_path <= 10)));
  if (act_fuse && !pair_path) return -1;
  p.act_fuse = act_fuse;
  if (pair_path) {
    const bool bn256 = act_fuse || ((force_path == 0 || tp_pair) ? (N > 128) : (force_path == 7 || force_path == 9));
    p.sk = (force_path == 0 || force_path >= 9 || tp_pair) ? 1 : 0;
    p.tiles_m = (M + 2 * kBM - 1) / (2 * kBM);
    CUtensorMap tA, tA2, tB;
    if (!get_tmap_bf16(&tA, A, M, K, lda, kBM, kBK)) return -3;
    tA2 = tA;
    if (tp && tp->gather && tp->a_alt && !get_tmap_bf16(&tA2, tp->a_alt, M, K, lda, kBM, kBK)) return -3;
    if (bn256) {
      p.tiles_n = tn256;
      if (!get_tmap_bf16(&tB, W, N, K, ldw, 128, kBK)) return -3;
      return launch_pair<256>(tA, tA2, tB, p, stream);
    }
    p.tiles_n = tn128;
    if (!get_tmap_bf16(&tB, W, N, K, ldw, 64, kBK)) return -3;
    return launch_pair<128>(tA, tA2, tB, p, stream);
  }
  CUtensorMap tmA, tmA2, tmB;
  if (!get_tmap_bf16(&tmA, A, M, K, lda, kBM, kBK)) return -3;
  tmA2 = tmA;
  if (tp && tp->gather && tp->a_alt && !get_tmap_bf16(&tmA2, tp->a_alt, M, K, lda, kBM, kBK)) return -3;
  if (use256) {
    p.tiles_n = tn256;
    if (!get_tmap_bf16(&tmB, W, N, K, ldw, 256, kBK)) return -3;
    return launch_tn<256>(tmA, tmA2, tmB, p, stream);
  }
  p.tiles_n = tn128;
  if (!get_tmap_bf16(&tmB, W, N, K, ldw, 128, kBK)) return -3;
  return launch_tn<128>(tmA, tmA2, tmB, p, stream);
}

// Batched small-M GEMM (M <= 256, K a multiple of 64): for b in [0, batch)
//   out[b * out_batch_stride + m * ldo + n] = sum_k A[m * lda + b * a_batch_cols + k] * W[(b * N + n) * ldw + k]
// One launch, grid (N / 128, 1, batch). Used for the per-head W_UK / W_UV products of MLA
// (reference: BatchedMatmulKernelCuda in src/vt/cuda/cuda_matmul.cu).
extern "C" int b200_gemm_bf16_batched(const void* A, int lda, int a_batch_cols, const void* W, int ldw,
                                      void* out, int ldo, long long out_batch_stride, int M, int N,
                                      int K, int batch, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if (M > 256 || (K & 63) || (lda & 7) || (ldw & 7) || (a_batch_cols & 7)) return -1;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W)) & 15) return -1;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.out_f32 = 0;
  p.status = device_status_word();
  p.batch_a_cols = a_batch_cols;
  p.batch_out_stride = out_batch_stride;
  const int mp = (M + 15) & ~15;
  p.mp = mp;
  p.tiles_n = (N + kBM - 1) / kBM;
  p.splits = 1;
  const int kblocks = K / kBK;
  p.kb_per_split = kblocks;
  const int stage_bytes = kBM * kBK * 2 + mp * kBK * 2;
  int stages = (kSmemBudget - 2048) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages > kblocks) stages = kblocks;
  if (stages < 2) stages = 2;
  p.stages = stages;
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < mp) tmem_cols <<= 1;
  CUtensorMap tmW, tmA;
  if (!get_tmap_bf16(&tmW, W, (uint64_t)batch * N, K, ldw, kBM, kBK)) return -3;
  if (!get_tmap_bf16(&tmA, A, M, (uint64_t)lda, lda, mp, kBK)) return -3;
  static PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(gemm_bf16_swap_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         kSmemBudget + 4096);
  }
  const size_t smem = (size_t)stages * stage_bytes + 1024 + sizeof(GemmBarriers);
  gemm_bf16_swap_kernel<<<dim3(p.tiles_n, 1, batch), kGemmThreads, smem, stream>>>(tmW, tmA, tmA, p, tmem_cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// ---------------------------------------------------------------------------------------
// b200_gemm_bf16_smallm_static: the small-M split-K GEMM for callers that cannot allocate.
//
// Some hosts of this library own no allocator they may call at the point where they need a
// GEMM: a plug-in running inside another runtime's callback, a thread that must not touch the
// framework's caching allocator, a C program that links the kernels without torch. The regular
// entry point asks such a caller for a workspace pointer; this one brings its own. The split-K
// partial sums live in a fixed array that is part of the loaded module image, and the sticky
// error word that the kernels' bounded waits report into is a second such symbol. No device or
// host memory is requested here or in anything this function calls: tensor maps are encoded
// on the stack and nothing is cached.
//
// Consequences a caller has to know:
//   * The array is one per device and every call on that device uses it, on whatever stream.
//     Two calls whose execution can overlap (different streams, or different host threads
//     feeding different streams) race on the partial sums. Serialise them.
//   * Nothing in the array has to start at zero: each split overwrites its whole M x N slab
//     before the reduction reads it. The error word starts at zero when the module loads and
//     is never cleared by a call, so one timeout stays visible.
//   * The first call on a device looks up the two symbol addresses and raises the kernel's
//     shared-memory limit. That may make the CUDA runtime load the module. Make that first
//     call ahead of any stream capture on the device.
//   * Shapes whose two-way split does not fit the array are refused (-4), never shrunk to a
//     slower unsplit run behind the caller's back.
// ---------------------------------------------------------------------------------------
namespace b200 {
static __device__ __align__(256) float g_static_splitk_scratch[B200_GEMM_STATIC_SCRATCH_BYTES / 4];
static __device__ int g_static_status_word;

struct StaticGemmDevice {
  float* scratch = nullptr;
  int* status = nullptr;
  bool ready = false;
};
static StaticGemmDevice g_static_dev[64];
static std::mutex g_static_mu;
static thread_local const char* g_static_err = "";
}  // namespace b200

extern "C" const char* b200_gemm_bf16_smallm_static_error(void) { return b200::g_static_err; }

extern "C" int b200_gemm_bf16_smallm_static_status(int* out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || !out) return -1;
  int* word = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (g_static_dev[dev].ready) word = g_static_dev[dev].status;
  }
  if (!word) { *out = 0; return 0; }
  // every stream of the device, non-blocking ones included, must have drained before the read
  if (cudaDeviceSynchronize() != cudaSuccess) return -2;
  return cudaMemcpy(out, word, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -2;
}

extern "C" int b200_gemm_bf16_smallm_static(const void* A, int lda, const void* W, int ldw,
                                            void* out, int ldo, int M, int N, int K,
                                            cudaStream_t stream) {
  g_static_err = "";
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 256) { g_static_err = "M > 256: use b200_gemm_bf16 with a caller-owned workspace"; return -4; }
  if ((K & 7) || (lda & 7) || (ldw & 7) || (N & 7) || (ldo & 7) ||
      ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(W) |
        reinterpret_cast<uintptr_t>(out)) & 15)) {
    g_static_err = "K, N and the leading dimensions must be multiples of 8; pointers 16-byte aligned";
    return -1;
  }
  const size_t slab = (size_t)M * N * sizeof(float);
  if (2 * slab > (size_t)B200_GEMM_STATIC_SCRATCH_BYTES) {
    g_static_err = "2 * M * N * 4 bytes exceeds B200_GEMM_STATIC_SCRATCH_BYTES";
    return -4;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { g_static_err = "no current device"; return -2; }
  StaticGemmDevice sd;
  {
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticGemmDevice& d = g_static_dev[dev];
    if (!d.ready) {
      void* ps = nullptr;
      void* pw = nullptr;
      if (cudaGetSymbolAddress(&ps, g_static_splitk_scratch) != cudaSuccess ||
          cudaGetSymbolAddress(&pw, g_static_status_word) != cudaSuccess || !ps || !pw) {
        g_static_err = "cudaGetSymbolAddress failed for the static scratch";
        return -2;
      }
      if (cudaFuncSetAttribute(gemm_bf16_swap_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kSmemBudget + 4096) != cudaSuccess) {
        g_static_err = "cannot raise the kernel's shared-memory limit";
        return -2;
      }
      d.scratch = reinterpret_cast<float*>(ps);
      d.status = reinterpret_cast<int*>(pw);
      d.ready = true;
    }
    sd = d;
  }
  GemmParams p{};
  p.M = M; p.N = N; p.K = K;
  p.out = out; p.ldo = ldo; p.out_f32 = 0;
  p.status = sd.status;
  const int sms = b200_num_sms();
  const int kblocks = (K + kBK - 1) / kBK;
  const int mp = (M + 15) & ~15;
  p.mp = mp;
  p.tiles_n = (N + kBM - 1) / kBM;
  int splits = 1;
  if (p.tiles_n < sms) {
    splits = sms / p.tiles_n;
    int max_by_k = kblocks / 4;
    if (max_by_k < 1) max_by_k = 1;
    if (splits > max_by_k) splits = max_by_k;
    if (splits > 16) splits = 16;
  }
  while (splits > 1 && (size_t)splits * slab > (size_t)B200_GEMM_STATIC_SCRATCH_BYTES) --splits;
  const int kb_per = (kblocks + splits - 1) / splits;
  splits = (kblocks + kb_per - 1) / kb_per;
  p.splits = splits;
  p.kb_per_split = kb_per;
  p.workspace = sd.scratch;
  const int stage_bytes = kBM * kBK * 2 + mp * kBK * 2;
  int stages = (kSmemBudget - 2048) / stage_bytes;
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages > kb_per) stages = kb_per;
  if (stages < 2) stages = 2;
  p.stages = stages;
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < mp) tmem_cols <<= 1;
  CUtensorMap tmW, tmA;
  if (!encode_tmap_2d(&tmW, W, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, N, K, ldw, kBM, kBK,
                      CU_TENSOR_MAP_SWIZZLE_128B) ||
      !encode_tmap_2d(&tmA, A, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda, mp, kBK,
                      CU_TENSOR_MAP_SWIZZLE_128B)) {
    g_static_err = "tensor map encoding failed";
    return -3;
  }
  const size_t smem = (size_t)stages * stage_bytes + 1024 + sizeof(GemmBarriers);
  dim3 grid(p.tiles_n, splits);
  gemm_bf16_swap_kernel<<<grid, kGemmThreads, smem, stream>>>(tmW, tmA, tmA, p, tmem_cols);
  if (cudaGetLastError() != cudaSuccess) { g_static_err = "kernel launch failed"; return -2; }
  if (splits > 1) {
    const size_t total = (size_t)M * (N / 4);
    int blocks = (int)((total + 255) / 256);
    if (blocks > sms * 8) blocks = sms * 8;
    splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(sd.scratch, splits, M, N, out, ldo, 0,
                                                     nullptr, nullptr, 0);
    if (cudaGetLastError() != cudaSuccess) { g_static_err = "reduce launch failed"; return -2; }
  }
  return 0;
}

// Per-device set-up of everything the launchers would otherwise allocate on first use: the
// stream-K scratch. Call it once per device before the first capture; 0 on success.
extern "C" int b200_fp8_init_device();
extern "C" int b200_init_device() {
  float* p = nullptr;
  uint32_t* f = nullptr;
  if (!streamk_scratch(nullptr, &p, &f)) return -2;
  return b200_fp8_init_device();
}
