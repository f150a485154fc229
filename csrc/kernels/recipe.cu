// Fused-chain interpreter: one kernel that runs a short program of row-wise steps (load, residual
// add, RMSNorm, gated RMSNorm, activation-multiply, sigmoid gate, fp8 / NVFP4 quantisation, store)
// over every row of its operands, with the intermediate rows held in shared memory instead of
// making a trip through HBM between steps. It is the middle tier of the fusion-recipe catalogue:
// a recipe that has a bespoke kernel runs that; one that has none still runs as ONE launch here;
// and the step-by-step composite of plain kernels stays the oracle.
//
// Every step rounds its result to bf16, as the plain kernel of that step does when it writes its
// output, and the two reductions repeat the summation order of the plain kernels they stand for
// (rmsnorm_kernel: 16-byte vectors strided over the block, then a two-level shuffle sum;
// rmsnorm_gated_kernel: one warp per row, 8-byte vectors). A chain therefore produces the bytes
// of its composite.
//
// One block of 256 threads per row; a row is `width` bf16 values (a multiple of 8; of 16 when the
// chain quantises to NVFP4). With heads > 1 a row is one head of a token: row r reads
// operand + (r / heads) * ld + (r % heads) * width + col.
//
// reference: src/vt/cuda/cuda_ops.cu:1238 (FusedChainInterpKernel), include/vt/fused_recipe.h
#include "api.h"
#include "quant_codec.cuh"
#include "sm100.cuh"

namespace b200 {

typedef __nv_bfloat16 bf16;

enum ChainOp : int {
  kChLoad = 0,         // reg[dst] = operand row
  kChStore = 1,        // operand row = reg[a]
  kChAdd = 2,          // reg[dst] = reg[a] + reg[b]
  kChRmsNorm = 3,      // reg[dst] = reg[a] * rsqrt(mean(a^2) + f) * (w + flag), w = operand vector
  kChRmsNormGated = 4, // reg[dst] = reg[a] * rsqrt(mean(a^2) + f) * w * gate(reg[b]); flag 0 silu, 1 sigmoid
  kChActMul = 5,       // reg[dst] = act(reg[a]) * reg[b]; flag 0 silu, 1 gelu-tanh, 2 gelu-erf
  kChSigmoidMul = 6,   // reg[dst] = reg[a] * sigmoid(reg[b])
  kChQuantFp8 = 7,     // operand row (bytes) = e4m3(reg[a] / *operand2)
  kChQuantNvfp4 = 8,   // operand (packed), operand2 (block scales), *operand3 (global scale); flag 1: chunk layout
};

__device__ __forceinline__ float chain_warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float chain_act(float g, int kind) {
  if (kind == 0) return g / (1.f + __expf(-g));
  if (kind == 1) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    return 0.5f * g * (1.f + tanhf(k0 * (g + k1 * g * g * g)));
  }
  return 0.5f * g * (1.f + erff(g * 0.7071067811865476f));
}

// Sum of squares of a shared-memory row in the order rmsnorm_kernel uses when it is launched for
// this width: nt = min(256, H/8 rounded up to a warp) threads, 16-byte vectors strided by nt.
__device__ float chain_sumsq_block(const bf16* row, int H, float* red) {
  const int nv = H >> 3;
  int nt = nv >= 256 ? 256 : ((nv + 31) / 32) * 32;
  if (nt < 32) nt = 32;
  float ss = 0.f;
  if ((int)threadIdx.x < nt) {
    const uint4* r = reinterpret_cast<const uint4*>(row);
    for (int i = threadIdx.x; i < nv; i += nt) {
      const uint4 v = r[i];
      float2 f;
      f = unpack_bf16x2(v.x); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(v.y); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(v.z); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16x2(v.w); ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = chain_warp_sum(ss);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = nt >> 5;
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = chain_warp_sum(t);
  __syncthreads();
  return t;
}

// Sum of squares in the order of rmsnorm_gated_kernel: one warp, 8-byte vectors strided by 128.
__device__ float chain_sumsq_warp(const bf16* row, int D, float* red) {
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float ss = 0.f;
    for (int i = lane * 4; i < D; i += 128) {
      const uint2 v = *reinterpret_cast<const uint2*>(row + i);
      const float2 f0 = unpack_bf16x2(v.x), f1 = unpack_bf16x2(v.y);
      ss += f0.x * f0.x + f0.y * f0.y + f1.x * f1.x + f1.y * f1.y;
    }
    ss = chain_warp_sum(ss);
    if (lane == 0) red[0] = ss;
  }
  __syncthreads();
  const float t = red[0];
  __syncthreads();
  return t;
}

__global__ void __launch_bounds__(256) fused_chain_kernel(const __grid_constant__ B200Chain prog) {
  extern __shared__ uint4 chain_smem[];
  __shared__ float red[32];
  bf16* regs = reinterpret_cast<bf16*>(chain_smem);
  const int W = prog.width, heads = prog.heads;
  const long r = blockIdx.x;
  const long tok = r / heads;
  const long hoff = (r % heads) * (long)W;
  auto reg = [&](int i) { return regs + (size_t)i * W; };
  auto row_of = [&](int operand) {
    const B200ChainOperand& o = prog.operands[operand];
    return tok * o.ld + hoff + o.col;
  };
  for (int s = 0; s < prog.n_steps; ++s) {
    const B200ChainStep st = prog.steps[s];
    switch (st.op) {
      case kChLoad: {
        const uint4* src = reinterpret_cast<const uint4*>((const bf16*)prog.operands[st.operand].ptr + row_of(st.operand));
        uint4* d = reinterpret_cast<uint4*>(reg(st.dst));
        for (int i = threadIdx.x; i < (W >> 3); i += blockDim.x) d[i] = src[i];
        break;
      }
      case kChStore: {
        uint4* dstp = reinterpret_cast<uint4*>((bf16*)prog.operands[st.operand].ptr + row_of(st.operand));
        const uint4* a = reinterpret_cast<const uint4*>(reg(st.a));
        for (int i = threadIdx.x; i < (W >> 3); i += blockDim.x) dstp[i] = a[i];
        break;
      }
      case kChAdd:
      case kChActMul:
      case kChSigmoidMul: {
        const uint32_t* a = reinterpret_cast<const uint32_t*>(reg(st.a));
        const uint32_t* b = reinterpret_cast<const uint32_t*>(reg(st.b));
        uint32_t* d = reinterpret_cast<uint32_t*>(reg(st.dst));
        for (int i = threadIdx.x; i < (W >> 1); i += blockDim.x) {
          const float2 x = unpack_bf16x2(a[i]), y = unpack_bf16x2(b[i]);
          float2 o;
          if (st.op == kChAdd) {
            o.x = x.x + y.x; o.y = x.y + y.y;
          } else if (st.op == kChActMul) {
            o.x = chain_act(x.x, st.flag) * y.x; o.y = chain_act(x.y, st.flag) * y.y;
          } else {
            o.x = x.x / (1.f + __expf(-y.x)); o.y = x.y / (1.f + __expf(-y.y));
          }
          d[i] = pack_bf16x2(o.x, o.y);
        }
        break;
      }
      case kChRmsNorm: {
        const float ss = chain_sumsq_block(reg(st.a), W, red);
        const float inv = rsqrtf(ss / (float)W + st.f);
        const float g = st.flag ? 1.f : 0.f;
        const uint32_t* a = reinterpret_cast<const uint32_t*>(reg(st.a));
        const uint32_t* w = reinterpret_cast<const uint32_t*>((const bf16*)prog.operands[st.operand].ptr);
        uint32_t* d = reinterpret_cast<uint32_t*>(reg(st.dst));
        for (int i = threadIdx.x; i < (W >> 1); i += blockDim.x) {
          const float2 x = unpack_bf16x2(a[i]), y = unpack_bf16x2(w[i]);
          d[i] = pack_bf16x2(x.x * inv * (y.x + g), x.y * inv * (y.y + g));
        }
        break;
      }
      case kChRmsNormGated: {
        const float ss = chain_sumsq_warp(reg(st.a), W, red);
        const float inv = rsqrtf(ss / (float)W + st.f);
        const uint32_t* a = reinterpret_cast<const uint32_t*>(reg(st.a));
        const uint32_t* z = reinterpret_cast<const uint32_t*>(reg(st.b));
        const uint32_t* w = reinterpret_cast<const uint32_t*>((const bf16*)prog.operands[st.operand].ptr);
        uint32_t* d = reinterpret_cast<uint32_t*>(reg(st.dst));
        const int kind = st.flag;
        auto gate = [&](float t) { return kind == 0 ? t / (1.f + __expf(-t)) : 1.f / (1.f + __expf(-t)); };
        for (int i = threadIdx.x; i < (W >> 1); i += blockDim.x) {
          const float2 x = unpack_bf16x2(a[i]), zz = unpack_bf16x2(z[i]), y = unpack_bf16x2(w[i]);
          d[i] = pack_bf16x2(x.x * inv * y.x * gate(zz.x), x.y * inv * y.y * gate(zz.y));
        }
        break;
      }
      case kChQuantFp8: {
        const float is = 1.f / *(const float*)prog.operands[st.operand2].ptr;
        uint8_t* o = (uint8_t*)prog.operands[st.operand].ptr + row_of(st.operand);
        const bf16* a = reg(st.a);
        for (int i = threadIdx.x; i < W; i += blockDim.x) o[i] = float_to_e4m3(__bfloat162float(a[i]) * is);
        break;
      }
      case kChQuantNvfp4: {
        const float gs = *(const float*)prog.operands[st.operand3].ptr;
        const int K = heads * W;                        // width of the whole quantised row
        uint8_t* packed = (uint8_t*)prog.operands[st.operand].ptr;
        uint8_t* sf = (uint8_t*)prog.operands[st.operand2].ptr;
        const bf16* a = reg(st.a);
        for (int gi = threadIdx.x; gi < (W >> 4); gi += blockDim.x) {
          float v[16];
          float amax = 0.f;
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            v[e] = __bfloat162float(a[gi * 16 + e]);
            amax = fmaxf(amax, fabsf(v[e]));
          }
          const uint8_t sb = float_to_e4m3(amax * gs / 6.f);
          const float sdec = e4m3_to_float(sb);
          const float mul = sdec > 0.f ? gs / sdec : 0.f;
          uint32_t w0 = 0, w1 = 0;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            w0 |= float_to_e2m1(v[e] * mul) << (e * 4);
            w1 |= float_to_e2m1(v[8 + e] * mul) << (e * 4);
          }
          const int gidx = (int)(hoff >> 4) + gi;
          reinterpret_cast<uint2*>(packed)[tok * (K / 16) + gidx] = make_uint2(w0, w1);
          sf[st.flag ? nvfp4_sf_chunk_offset(tok, gidx, K) : (size_t)tok * (K / 16) + gidx] = sb;
        }
        break;
      }
      default: break;
    }
    __syncthreads();
  }
}

}  // namespace b200

using namespace b200;

extern "C" {

// Returns 0, -1 for a program the interpreter cannot run (the caller falls back to the composite),
// -2 for a failed launch.
int b200_fused_chain(const B200Chain* prog, cudaStream_t stream) {
  const B200Chain& p = *prog;
  if (p.rows <= 0) return 0;
  if (p.n_steps < 1 || p.n_steps > B200_CHAIN_MAX_STEPS || p.n_regs < 1 || p.n_regs > 4) return -1;
  if (p.width < 8 || (p.width & 7) || p.width > 32768 || p.heads < 1) return -1;
  const size_t smem = (size_t)p.n_regs * p.width * sizeof(bf16);
  if (smem > 200 * 1024) return -1;
  auto reg_ok = [&](int r) { return r >= 0 && r < p.n_regs; };
  auto opd_ok = [&](int o) { return o >= 0 && o < B200_CHAIN_MAX_OPERANDS && p.operands[o].ptr != nullptr; };
  auto row_ok = [&](int o, int align) {          // 16-byte rows of bf16 (align 8) or of packed bytes
    return opd_ok(o) && !(p.operands[o].ld % align) && !(p.operands[o].col % align) &&
           !((uintptr_t)p.operands[o].ptr & 15);
  };
  for (int s = 0; s < p.n_steps; ++s) {
    const B200ChainStep& st = p.steps[s];
    switch (st.op) {
      case kChLoad: if (!reg_ok(st.dst) || !row_ok(st.operand, 8)) return -1; break;
      case kChStore: if (!reg_ok(st.a) || !row_ok(st.operand, 8)) return -1; break;
      case kChAdd: case kChSigmoidMul: case kChActMul:
        if (!reg_ok(st.dst) || !reg_ok(st.a) || !reg_ok(st.b)) return -1;
        break;
      case kChRmsNorm: if (!reg_ok(st.dst) || !reg_ok(st.a) || !opd_ok(st.operand)) return -1; break;
      case kChRmsNormGated:
        if (!reg_ok(st.dst) || !reg_ok(st.a) || !reg_ok(st.b) || !opd_ok(st.operand)) return -1;
        break;
      case kChQuantFp8: if (!reg_ok(st.a) || !opd_ok(st.operand) || !opd_ok(st.operand2)) return -1; break;
      case kChQuantNvfp4:
        if (!reg_ok(st.a) || !opd_ok(st.operand) || !opd_ok(st.operand2) || !opd_ok(st.operand3)) return -1;
        if ((p.width & 15) || (st.flag && ((p.heads * p.width) & 63))) return -1;
        if ((uintptr_t)p.operands[st.operand].ptr & 7) return -1;
        break;
      default: return -1;
    }
  }
  static PerDeviceOnce attr_once;
  if (attr_once.first())
    cudaFuncSetAttribute(fused_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  fused_chain_kernel<<<(unsigned)p.rows, 256, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // extern "C"
