// Tensor-parallel fused collectives over NVLink peer memory (one process per GPU).
//
// Sequence-parallel layer flow on `world` ranks, rows (tokens) split into contiguous shards
// of `rows_per_rank`:
//
//   GEMM_A  (o_proj / down_proj, K sharded)   scatter epilogue in gemm_bf16.cu: every partial
//           row is stored straight into its owner's receive slot over NVLink and the owner's
//           arrival counter of that 32-row group is bumped                 [GEMM + reduce-scatter]
//   tp_reduce_norm_gather_kernel (this file)  the owner waits for the `world` partials of a
//           group, sums them in fixed rank order in fp32, adds its residual shard, applies
//           RMSNorm and stores the normalised row into EVERY rank's gather buffer, then
//           bumps that rank's gather counter                  [+ residual + RMSNorm + all-gather]
//   GEMM_C  (qkv / gate_up, N sharded)        gather prologue in gemm_bf16.cu: the TMA
//           producer waits for the gather counters of the rows of a tile      [all-gather + GEMM]
//
// All peer traffic is plain ld/st/red on peer-mapped pointers (CUDA IPC); no TMA touches
// another GPU's memory. Buffers and counters are double-buffered by the parity of a
// device-side op counter so that the kernels can be replayed from a CUDA graph; every wait
// is bounded and reports through the status word.
//
// The reference has no distributed code; these are the collective sites its design note
// lists (.agents/specs/tensor-parallelism.md:291-308) turned into fused kernels.
#include "api.h"
#include "sm100.cuh"

namespace b200 {

struct ReduceNormParams {
  int world, rank, rows_per_rank, M, H;
  const __nv_bfloat16* recv;          // local [2][world][rows_per_rank][H]
  long long recv_parity_stride;
  uint32_t* rs_flags;                 // local [2][rows_per_rank / 32]
  int rs_flag_parity_stride;
  int expected_rs;
  int nsrc;                           // source slots to sum (world x k-splits of the scatter GEMM)
  __nv_bfloat16* residual;            // local shard [rows_per_rank][H], updated in place (may be null)
  const __nv_bfloat16* norm_w;        // [H]
  float eps;
  int gemma;
  __nv_bfloat16* peer_x[8];           // gather buffers [2][M_max][H] on every rank
  long long x_parity_stride;
  uint32_t* peer_ag_flags[8];         // gather counters [2][groups] on every rank
  int ag_flag_parity_stride;
  uint32_t* ag_flags_local;           // == peer_ag_flags[rank]
  int ag_groups;
  uint32_t* op_counter;               // local
  uint32_t* done_counter;             // local
  int* status;
  long long peer_wait;                // limit of the wait on the arrival counters, in cycles
};

__device__ __forceinline__ bool wait_ge_sys(const uint32_t* ctr, uint32_t target, int* status,
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

// One block per owned row.
__global__ void __launch_bounds__(256) tp_reduce_norm_gather_kernel(ReduceNormParams p) {
  __shared__ float red[32];
  __shared__ int s_ok;
  extern __shared__ uint4 row_cache[];  // H/8 vectors
  pdl_wait();                 // the scatter GEMM of this rank is complete
  pdl_launch_dependents();
  const uint32_t k = *p.op_counter;
  const uint32_t par = k & 1, npar = par ^ 1;
  const int rl = blockIdx.x;
  const int row = p.rank * p.rows_per_rank + rl;
  const bool valid = row < p.M;
  if (blockIdx.x == 0) {
    // Gather counters of the other parity: their readers (this rank's GEMMs of the previous op)
    // are done, and their next writers (the peers' reduce kernels two ops from now) cannot start
    // before this rank's next scatter GEMM, which follows this kernel in the stream.
    for (int i = threadIdx.x; i < p.ag_groups; i += blockDim.x)
      p.ag_flags_local[npar * p.ag_flag_parity_stride + i] = 0;
    __threadfence();
  }
  if (threadIdx.x == 0) {
    s_ok = valid ? (wait_ge_sys(p.rs_flags + par * p.rs_flag_parity_stride + rl / 32,
                                (uint32_t)p.expected_rs, p.status, p.peer_wait) ? 1 : 0)
                 : 1;
  }
  __syncthreads();
  if (valid && s_ok) {
    const int nv = p.H >> 3;
    const __nv_bfloat16* base = p.recv + par * p.recv_parity_stride + (size_t)rl * p.H;
    const size_t src_stride = (size_t)p.rows_per_rank * p.H;
    uint4* rr = p.residual ? reinterpret_cast<uint4*>(p.residual + (size_t)rl * p.H) : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int s = 0; s < p.nsrc; ++s) {    // fixed slot order => same bits on every run
        const uint4 v = *reinterpret_cast<const uint4*>(base + s * src_stride + i * 8);
        float2 f;
        f = unpack_bf16x2(v.x); acc[0] += f.x; acc[1] += f.y;
        f = unpack_bf16x2(v.y); acc[2] += f.x; acc[3] += f.y;
        f = unpack_bf16x2(v.z); acc[4] += f.x; acc[5] += f.y;
        f = unpack_bf16x2(v.w); acc[6] += f.x; acc[7] += f.y;
      }
      if (rr) {
        const uint4 r = rr[i];
        float2 f;
        f = unpack_bf16x2(r.x); acc[0] += f.x; acc[1] += f.y;
        f = unpack_bf16x2(r.y); acc[2] += f.x; acc[3] += f.y;
        f = unpack_bf16x2(r.z); acc[4] += f.x; acc[5] += f.y;
        f = unpack_bf16x2(r.w); acc[6] += f.x; acc[7] += f.y;
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      if (rr) rr[i] = o;                    // the residual stream is bf16
      row_cache[i] = o;
      float2 f;
      f = unpack_bf16x2(o.x); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(o.y); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(o.z); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(o.w); ss += f.x * f.x + f.y * f.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
    const float inv = rsqrtf(tot / (float)p.H + p.eps);
    const float g = p.gemma ? 1.f : 0.f;
    const uint4* wr = reinterpret_cast<const uint4*>(p.norm_w);
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      const uint4 v = row_cache[i], wv = wr[i];
      uint4 o;
      float2 a, b;
      a = unpack_bf16x2(v.x); b = unpack_bf16x2(wv.x); o.x = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
      a = unpack_bf16x2(v.y); b = unpack_bf16x2(wv.y); o.y = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
      a = unpack_bf16x2(v.z); b = unpack_bf16x2(wv.z); o.z = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
      a = unpack_bf16x2(v.w); b = unpack_bf16x2(wv.w); o.w = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
      // all-gather: the normalised row goes to every rank (this one included)
      for (int d = 0; d < p.world; ++d)
        reinterpret_cast<uint4*>(p.peer_x[d] + par * p.x_parity_stride + (size_t)row * p.H)[i] = o;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < p.world)
      asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(
                       p.peer_ag_flags[threadIdx.x] + par * p.ag_flag_parity_stride + row / 32)
                   : "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.done_counter, 1u) == gridDim.x - 1) {
      // Last block: every block has consumed its arrival counter. Clear this parity's counters
      // here, by their consumer, and not at the start of a later op: a peer that runs ahead may
      // already be signalling the other parity, and nothing may wipe those arrivals. The next
      // arrivals on THIS parity come from the peers' scatter GEMMs two ops from now, which cannot
      // start before this rank's next scatter GEMM (after this kernel in the stream) has arrived.
      for (int i = 0; i < p.rows_per_rank / 32; ++i) p.rs_flags[par * p.rs_flag_parity_stride + i] = 0;
      *p.done_counter = 0;
      __threadfence();
      atomicAdd(p.op_counter, 1u);   // the next fused op uses the other parity
    }
  }
}

// Local prologue of the first layer: x_full[par] rows = rmsnorm(hidden) for ALL rows (every
// rank holds the full embedding output), gather counters set to "complete", and this rank's
// residual shard initialised. Advances the op counter like the fused kernel does.
__global__ void __launch_bounds__(256)
    tp_first_norm_kernel(const __nv_bfloat16* __restrict__ hidden, __nv_bfloat16* residual_shard,
                         const __nv_bfloat16* __restrict__ w, __nv_bfloat16* x_full,
                         long long x_parity_stride, uint32_t* ag_flags, int ag_flag_parity_stride,
                         int ag_groups, uint32_t* rs_flags, int rs_flag_parity_stride,
                         int rank, int rows_per_rank, int M, int H, float eps, int gemma,
                         uint32_t* op_counter, uint32_t* done_counter) {
  __shared__ float red[32];
  const uint32_t par = *op_counter & 1, npar = par ^ 1;
  const int row = blockIdx.x;
  if (blockIdx.x == 0) {
    // (the reduce-scatter arrival counters are cleared by the reduce kernel that consumed them; a
    // peer that is already past this point may be signalling them for the next op)
    for (int i = threadIdx.x; i < ag_groups; i += blockDim.x) {
      ag_flags[npar * ag_flag_parity_stride + i] = 0;
      ag_flags[par * ag_flag_parity_stride + i] = 32;   // everything is local and complete
    }
  }
  if (row < M) {
    const int nv = H >> 3;
    const uint4* xr = reinterpret_cast<const uint4*>(hidden + (size_t)row * H);
    const int owner = row / rows_per_rank;
    uint4* rs = owner == rank
                    ? reinterpret_cast<uint4*>(residual_shard + (size_t)(row - owner * rows_per_rank) * H)
                    : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      const uint4 v = xr[i];
      if (rs) rs[i] = v;
      float2 f;
      f = unpack_bf16x2(v.x); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(v.y); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(v.z); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(v.w); ss += f.x * f.x + f.y * f.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int wv = 0; wv < (int)(blockDim.x >> 5); ++wv) tot += red[wv];
    const float inv = rsqrtf(tot / (float)H + eps);
    const float g = gemma ? 1.f : 0.f;
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    uint4* orow = reinterpret_cast<uint4*>(x_full + par * x_parity_stride + (size_t)row * H);
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      const uint4 v = xr[i], wv = wr[i];
      uint4 o;
      float2 a, b;
      a = unpack_bf16x2(v.x); b = unpack_bf16x2(wv.x); o.x = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
      a = unpack_bf16x2(v.y); b = unpack_bf16x2(wv.y); o.y = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
      a = unpack_bf16x2(v.z); b = unpack_bf16x2(wv.z); o.z = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
      a = unpack_bf16x2(v.w); b = unpack_bf16x2(wv.w); o.w = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
      orow[i] = o;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(done_counter, 1u) == gridDim.x - 1) {
      *done_counter = 0;
      __threadfence();
      atomicAdd(op_counter, 1u);
    }
  }
}

// out[i, :] = x_gathered[idx[i], :] where x_gathered is the copy selected by the device op
// counter; waits (bounded) until the source row's 32-row group has fully arrived.
__global__ void __launch_bounds__(128)
    tp_gather_rows_kernel(const __nv_bfloat16* __restrict__ x_base, long long x_parity_stride,
                          int H, const int32_t* __restrict__ idx, const uint32_t* ag_flags,
                          int ag_flag_parity_stride, const uint32_t* op_counter, int M,
                          __nv_bfloat16* out, int* status, long long peer_wait) {
  __shared__ int s_ok;
  const uint32_t par = (*op_counter - 1) & 1;
  int src = idx[blockIdx.x];
  if (src < 0 || src >= M) src = 0;
  if (threadIdx.x == 0)
    s_ok = wait_ge_sys(ag_flags + par * ag_flag_parity_stride + src / 32,
                       (uint32_t)min(32, M - (src / 32) * 32), status, peer_wait) ? 1 : 0;
  __syncthreads();
  if (!s_ok) return;
  const uint4* s = reinterpret_cast<const uint4*>(x_base + par * x_parity_stride + (size_t)src * H);
  uint4* d = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * H);
  for (int i = threadIdx.x; i < (H >> 3); i += blockDim.x) d[i] = s[i];
}


// ------------------------------------------------------------------------------------------
// One-shot all-reduce + residual + RMSNorm for small batches (decode-sized steps).
// Every rank holds its partial product [M, H] in a buffer its peers can read; every rank reads all
// `world` partials of every row (its own included) straight from their owners, sums them in rank
// order (so all ranks get the same bits), adds the residual, and normalises. No scatter, no
// gather, one kernel between two GEMMs. Synchronisation: monotonic arrival counters, one per
// source rank, never reset: block 0 tells every peer "my partial number `seq + 1` is complete",
// each block waits until all peers have said the same, and the last block advances `seq`. The
// partial buffers alternate with the op's parity: a rank can only overwrite the buffer of op k
// in its GEMM of op k + 2, which it reaches after the wait of op k + 1, i.e. after every peer has
// finished reading op k.
// ------------------------------------------------------------------------------------------
struct OneShotParams {
  int world, rank, M, H;
  const __nv_bfloat16* peer_partial[8];   // this op's partial buffer on every rank
  const __nv_bfloat16* mc_partial;        // the same buffer through an NVSwitch multicast mapping, or null
  uint32_t* peer_flags[8];                // arrival counters [world] on every rank
  uint32_t* seq;                          // local: completed one-shot ops
  uint32_t* done_counter;                 // local
  __nv_bfloat16* residual;                // [M, H] local, updated in place (may be null)
  const __nv_bfloat16* norm_w;            // null: plain sum, no norm
  __nv_bfloat16* out;                     // [M, H] normalised rows (or the sum when norm_w is null)
  float eps;
  int gemma;
  int* status;
  long long peer_wait;
};

__global__ void __launch_bounds__(256) tp_oneshot_allreduce_norm_kernel(OneShotParams p) {
  __shared__ float red[32];
  __shared__ int s_ok;
  extern __shared__ uint4 row_cache[];
  const uint32_t target = *p.seq + 1;
  if (blockIdx.x == 0 && threadIdx.x < p.world) {
    // the GEMM that wrote this rank's partial is an earlier kernel of this stream: complete and
    // visible at device scope; publish it to the peers
    __threadfence_system();
    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(p.peer_flags[threadIdx.x] + p.rank) : "memory");
  }
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    // wrap-safe comparison of monotonic counters
    const uint32_t* f = p.peer_flags[p.rank] + threadIdx.x;
    long long t0 = clock64();
    uint32_t it = 0;
    while (true) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if ((int32_t)(v - target) >= 0) break;
      if (((++it) & 0xff) == 0 && clock64() - t0 > p.peer_wait) {
        atomicExch(p.status, (int)kErrFlagTimeout);
        s_ok = 0;
        break;
      }
    }
  }
  __syncthreads();
  const int row = blockIdx.x;
  if (s_ok && row < p.M) {
    const int nv = p.H >> 3;
    uint4* rr = p.residual ? reinterpret_cast<uint4*>(p.residual + (size_t)row * p.H) : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      if (p.mc_partial) {
        // NVLS: one load, reduced over all ranks' copies inside the switch (fp32 accumulation, bf16
        // result; the same bits on every rank, as every rank asks the switch for the same sum)
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(p.mc_partial + (size_t)row * p.H + i * 8)
                     : "memory");
        float2 f;
        f = unpack_bf16x2(v.x); acc[0] = f.x; acc[1] = f.y;
        f = unpack_bf16x2(v.y); acc[2] = f.x; acc[3] = f.y;
        f = unpack_bf16x2(v.z); acc[4] = f.x; acc[5] = f.y;
        f = unpack_bf16x2(v.w); acc[6] = f.x; acc[7] = f.y;
      } else {
      // all peers' loads are issued before the first sum: one NVLink round trip, not `world`
      uint4 pv[8];
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r < p.world) pv[r] = *reinterpret_cast<const uint4*>(p.peer_partial[r] + (size_t)row * p.H + i * 8);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        if (r < p.world) {
          const uint4 v = pv[r];
          float2 f;
          f = unpack_bf16x2(v.x); acc[0] += f.x; acc[1] += f.y;
          f = unpack_bf16x2(v.y); acc[2] += f.x; acc[3] += f.y;
          f = unpack_bf16x2(v.z); acc[4] += f.x; acc[5] += f.y;
          f = unpack_bf16x2(v.w); acc[6] += f.x; acc[7] += f.y;
        }
      }
      }
      if (rr) {
        const uint4 r = rr[i];
        float2 f;
        f = unpack_bf16x2(r.x); acc[0] += f.x; acc[1] += f.y;
        f = unpack_bf16x2(r.y); acc[2] += f.x; acc[3] += f.y;
        f = unpack_bf16x2(r.z); acc[4] += f.x; acc[5] += f.y;
        f = unpack_bf16x2(r.w); acc[6] += f.x; acc[7] += f.y;
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      if (rr) rr[i] = o;
      row_cache[i] = o;
      float2 f;
      f = unpack_bf16x2(o.x); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(o.y); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(o.z); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(o.w); ss += f.x * f.x + f.y * f.y;
    }
    uint4* orow = reinterpret_cast<uint4*>(p.out + (size_t)row * p.H);
    if (!p.norm_w) {
      __syncthreads();
      for (int i = threadIdx.x; i < nv; i += blockDim.x) orow[i] = row_cache[i];
    } else {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
      const float inv = rsqrtf(tot / (float)p.H + p.eps);
      const float g = p.gemma ? 1.f : 0.f;
      const uint4* wr = reinterpret_cast<const uint4*>(p.norm_w);
      for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const uint4 v = row_cache[i], wv = wr[i];
        uint4 o;
        float2 a, b;
        a = unpack_bf16x2(v.x); b = unpack_bf16x2(wv.x); o.x = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
        a = unpack_bf16x2(v.y); b = unpack_bf16x2(wv.y); o.y = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
        a = unpack_bf16x2(v.z); b = unpack_bf16x2(wv.z); o.z = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
        a = unpack_bf16x2(v.w); b = unpack_bf16x2(wv.w); o.w = pack_bf16x2(a.x * inv * (b.x + g), a.y * inv * (b.y + g));
        orow[i] = o;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.done_counter, 1u) == gridDim.x - 1) {
      *p.done_counter = 0;
      __threadfence();
      atomicAdd(p.seq, 1u);
    }
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_tp_oneshot_allreduce_norm(const B200TpOneShot* a, cudaStream_t stream) {
  if (!a || a->world < 1 || a->world > 8 || a->M <= 0 || (a->H & 7) || a->H > 32768) return -1;
  OneShotParams p;
  p.world = a->world; p.rank = a->rank; p.M = a->M; p.H = a->H;
  for (int i = 0; i < a->world; ++i) {
    p.peer_partial[i] = (const __nv_bfloat16*)a->peer_partial[i];
    p.peer_flags[i] = (uint32_t*)a->peer_flags[i];
  }
  p.mc_partial = (const __nv_bfloat16*)a->mc_partial;
  p.seq = (uint32_t*)a->seq; p.done_counter = (uint32_t*)a->done_counter;
  p.residual = (__nv_bfloat16*)a->residual; p.norm_w = (const __nv_bfloat16*)a->norm_w;
  p.out = (__nv_bfloat16*)a->out; p.eps = a->eps; p.gemma = a->gemma;
  p.status = device_status_word();
  p.peer_wait = peer_wait_cycles();
  tp_oneshot_allreduce_norm_kernel<<<a->M, 256, (size_t)a->H * 2, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}


int b200_tp_reduce_norm_gather(const B200TpReduce* a, cudaStream_t stream) {
  if (!a || a->world < 1 || a->world > 8 || (a->H & 7) || a->H > 32768 || (a->rows_per_rank & 31))
    return -1;
  ReduceNormParams p;
  p.world = a->world; p.rank = a->rank; p.rows_per_rank = a->rows_per_rank; p.M = a->M; p.H = a->H;
  p.recv = (const __nv_bfloat16*)a->recv; p.recv_parity_stride = a->recv_parity_stride;
  p.rs_flags = (uint32_t*)a->rs_flags; p.rs_flag_parity_stride = a->rs_flag_parity_stride;
  p.expected_rs = a->expected_rs;
  p.nsrc = a->nsrc > 0 ? a->nsrc : a->world;
  p.residual = (__nv_bfloat16*)a->residual; p.norm_w = (const __nv_bfloat16*)a->norm_w;
  p.eps = a->eps; p.gemma = a->gemma;
  for (int i = 0; i < a->world; ++i) {
    p.peer_x[i] = (__nv_bfloat16*)a->peer_x[i];
    p.peer_ag_flags[i] = (uint32_t*)a->peer_ag_flags[i];
  }
  p.x_parity_stride = a->x_parity_stride;
  p.ag_flag_parity_stride = a->ag_flag_parity_stride;
  p.ag_flags_local = (uint32_t*)a->peer_ag_flags[a->rank];
  p.ag_groups = a->ag_groups;
  p.op_counter = (uint32_t*)a->op_counter; p.done_counter = (uint32_t*)a->done_counter;
  p.status = device_status_word();
  p.peer_wait = peer_wait_cycles();
  return launch_pdl(tp_reduce_norm_gather_kernel, dim3(a->rows_per_rank), dim3(256), (size_t)a->H * 2, stream,
                    p) == cudaSuccess ? 0 : -2;
}

int b200_tp_first_norm(const void* hidden, void* residual_shard, const void* w, void* x_full,
                       long long x_parity_stride, void* ag_flags, int ag_flag_parity_stride,
                       int ag_groups, void* rs_flags, int rs_flag_parity_stride, int rank,
                       int rows_per_rank, int M, int H, float eps, int gemma, void* op_counter,
                       void* done_counter, cudaStream_t stream) {
  if (M <= 0 || (H & 7)) return -1;
  tp_first_norm_kernel<<<M, 256, 0, stream>>>(
      (const __nv_bfloat16*)hidden, (__nv_bfloat16*)residual_shard, (const __nv_bfloat16*)w,
      (__nv_bfloat16*)x_full, x_parity_stride, (uint32_t*)ag_flags, ag_flag_parity_stride, ag_groups,
      (uint32_t*)rs_flags, rs_flag_parity_stride, rank, rows_per_rank, M, H, eps, gemma,
      (uint32_t*)op_counter, (uint32_t*)done_counter);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int b200_tp_gather_rows(const void* x_base, long long x_parity_stride, int H, const void* idx,
                        int n, const void* ag_flags, int ag_flag_parity_stride,
                        const void* op_counter, int M, void* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  tp_gather_rows_kernel<<<n, 128, 0, stream>>>(
      (const __nv_bfloat16*)x_base, x_parity_stride, H, (const int32_t*)idx,
      (const uint32_t*)ag_flags, ag_flag_parity_stride, (const uint32_t*)op_counter, M,
      (__nv_bfloat16*)out, device_status_word(), peer_wait_cycles());
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// ---- symmetric heap plumbing: cudaMalloc'd buffers shared between ranks through CUDA IPC ----
void* b200_symm_alloc(size_t bytes) {
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return nullptr;
  cudaMemset(p, 0, bytes);
  cudaDeviceSynchronize();
  return p;
}
int b200_symm_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -2; }
int b200_ipc_get_handle(void* p, void* out64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return -2;
  memcpy(out64, &h, sizeof(h));
  return 0;
}
void* b200_ipc_open(const void* handle64) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return p;
}
int b200_ipc_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -2; }
int b200_memset_async(void* p, int v, size_t bytes, cudaStream_t stream) {
  return cudaMemsetAsync(p, v, bytes, stream) == cudaSuccess ? 0 : -2;
}

}  // extern "C"
