// Optimizer kernels over flat parameter arenas (one launch for all parameters).
//
//   adamw8bit   block-wise 8-bit AdamW: 256-element blocks, one fp32 absmax per block and moment,
//               power-law companded codes (signed square-root code for m, unsigned fourth-root code
//               for v). Dequantise -> AdamW in fp32 -> requantise -> bf16 parameter write, with
//               optional stochastic rounding and a device-side gradient-clip coefficient, so the
//               step needs no host synchronisation.
//   adamw32     the same update with fp32 moments (reference numerics / small models).
//   ema         shadow = decay * shadow + (1 - decay) * param over the flat arena.
//
// The reference quantises per tensor on the device (src/trainers/adam8bit.rs:101-241) or per
// tensor on the host with percentile clipping (src/trainers/adam8bit_enhanced.rs:42-271); its
// fused CUDA Adam (src/kernels/fused_adam.cu:14-254) is never built. Block-wise scaling bounds
// the quantisation error per 256 values instead of per tensor.
#include "ptx.cuh"
#include "optim_codec.cuh"

using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int kBlock = 256;  // quantisation block, elements

__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}
__device__ __forceinline__ bf16 round_bf16(float v, bool stochastic, uint32_t rnd) {
  if (!stochastic) return __float2bfloat16(v);
  uint32_t bits = __float_as_uint(v);
  if ((bits & 0x7f800000u) == 0x7f800000u) return __float2bfloat16(v);
  bits += rnd & 0xffffu;
  return __ushort_as_bfloat16((unsigned short)(bits >> 16));
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, max_grad_norm, grad_scale;
  uint32_t seed;
  int stochastic;
};

// One warp per 256-element block; each lane owns 8 consecutive elements.
__global__ void adamw8bit_kernel(bf16* __restrict__ param, const bf16* __restrict__ grad,
                                 int8_t* __restrict__ mq, uint8_t* __restrict__ vq,
                                 float* __restrict__ m_absmax, float* __restrict__ v_absmax,
                                 const float* __restrict__ grad_sumsq, long long nblocks,
                                 long long n, AdamArgs a, const float* __restrict__ lr_scale) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  float gs = a.grad_scale;
  if (grad_sumsq) {
    const float ss = *grad_sumsq;
    if (!isfinite(ss)) return;  // non-finite gradients: leave parameters and state untouched
    if (a.max_grad_norm > 0.f) {
      float norm = sqrtf(ss) * a.grad_scale;
      gs *= fminf(1.f, a.max_grad_norm / (norm + 1e-6f));
    }
  }
  for (long long blk = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; blk < nblocks;
       blk += warps) {
    const long long e0 = blk * kBlock + lane * 8;
    const bool live = e0 < n;  // n is padded to a multiple of 8 by the arena
    // optional per-block learning-rate multiplier (per-layer rates, layer rotation): a block
    // whose multiplier is zero is frozen, parameters and moments untouched
    float lr = a.lr;
    if (lr_scale) {
      lr *= lr_scale[blk];
      if (lr == 0.f) continue;
    }
    float p[8], g[8], m[8], v[8];
    if (live) {
      unpack8(*reinterpret_cast<const bf16x8*>(param + e0), p);
      unpack8(*reinterpret_cast<const bf16x8*>(grad + e0), g);
      const float ma = m_absmax[blk], va = v_absmax[blk];
      uint2 mraw = *reinterpret_cast<const uint2*>(mq + e0);
      uint2 vraw = *reinterpret_cast<const uint2*>(vq + e0);
      const int8_t* mb = reinterpret_cast<const int8_t*>(&mraw);
      const uint8_t* vb = reinterpret_cast<const uint8_t*>(&vraw);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        m[j] = decode_m(mb[j], ma);
        v[j] = decode_v(vb[j], va);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) p[j] = g[j] = m[j] = v[j] = 0.f;
    }
    float mmax = 0.f, vmax = 0.f;
    float sv[8];                       // sqrt(v): shared by Adam's denominator and the code of v
    const float inv_bc1 = 1.f / a.bc1, rsqrt_bc2 = rsqrtf(a.bc2), decay = 1.f - lr * a.weight_decay;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gj = g[j] * gs;
      m[j] = a.beta1 * m[j] + (1.f - a.beta1) * gj;
      v[j] = a.beta2 * v[j] + (1.f - a.beta2) * gj * gj;
      mmax = fmaxf(mmax, fabsf(m[j]));
      vmax = fmaxf(vmax, v[j]);
      sv[j] = sqrtf(v[j]);
      const float upd = __fdividef(m[j] * inv_bc1, sv[j] * rsqrt_bc2 + a.eps);
      p[j] = p[j] * decay - lr * upd;
    }
    mmax = warp_max(mmax);
    vmax = warp_max(vmax);
    if (live) {
      const float im = mmax > 0.f ? 1.f / mmax : 0.f, siv = vmax > 0.f ? rsqrtf(vmax) : 0.f;
      uint2 mraw, vraw;
      int8_t* mb = reinterpret_cast<int8_t*>(&mraw);
      uint8_t* vb = reinterpret_cast<uint8_t*>(&vraw);
      bf16x8 po;
      bf16* pb = reinterpret_cast<bf16*>(&po);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        mb[j] = encode_m(m[j], im);
        vb[j] = encode_v_from_sqrt(sv[j], siv);
        pb[j] = round_bf16(p[j], a.stochastic != 0, hash_u32(a.seed ^ (uint32_t)(e0 + j) * 0x9E3779B9u));
      }
      *reinterpret_cast<uint2*>(mq + e0) = mraw;
      *reinterpret_cast<uint2*>(vq + e0) = vraw;
      *reinterpret_cast<bf16x8*>(param + e0) = po;
      if (lane == 0) {
        m_absmax[blk] = mmax;
        v_absmax[blk] = vmax;
      }
    }
  }
}

// The same step with about half the instructions per element (the kernel above is bound by
// instruction issue: ~87 per element, 73 % of the issue slots, DRAM at 35 %): see adam8_update8 /
// adam8_encode8 in optim_codec.cuh. Same codes, same update formula.
__global__ void adamw8bit_pair_kernel(bf16* __restrict__ param, const bf16* __restrict__ grad,
                                      int8_t* __restrict__ mq, uint8_t* __restrict__ vq,
                                      float* __restrict__ m_absmax, float* __restrict__ v_absmax,
                                      const float* __restrict__ grad_sumsq, long long nblocks,
                                      long long n, AdamArgs a, const float* __restrict__ lr_scale) {
  const int lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  float gs = a.grad_scale;
  if (grad_sumsq) {
    const float ss = *grad_sumsq;
    if (!isfinite(ss)) return;  // non-finite gradients: leave parameters and state untouched
    if (a.max_grad_norm > 0.f) {
      float norm = sqrtf(ss) * a.grad_scale;
      gs *= fminf(1.f, a.max_grad_norm / (norm + 1e-6f));
    }
  }
  Adam8Consts k;
  adam8_consts(k, a.beta1, a.beta2, a.eps, a.bc1, a.bc2, gs);
  for (long long blk = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; blk < nblocks;
       blk += warps) {
    const long long e0 = blk * kBlock + lane * 8;
    const bool live = e0 < n;  // n is padded to a multiple of 8 by the arena
    float lr = a.lr;
    if (lr_scale) {
      lr *= lr_scale[blk];
      if (lr == 0.f) continue;
    }
    uint4 pw = make_uint4(0u, 0u, 0u, 0u), gw = pw;
    uint2 mraw = make_uint2(0u, 0u), vraw = mraw;
    if (live) {
      pw = *reinterpret_cast<const uint4*>(param + e0);
      gw = *reinterpret_cast<const uint4*>(grad + e0);
      mraw = *reinterpret_cast<const uint2*>(mq + e0);
      vraw = *reinterpret_cast<const uint2*>(vq + e0);
    }
    const uint32_t gws[4] = {gw.x, gw.y, gw.z, gw.w};
    f32x2 g2[4], m2[4], sv2[4], p2[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) g2[i] = f2_pack_bits(gws[i] << 16, gws[i] & 0xffff0000u);
    float mmax, vmax;
    adam8_update8(k, g2, pw, mraw, vraw, m_absmax[blk], v_absmax[blk], lr, a.weight_decay, m2, sv2, p2,
                  mmax, vmax);
    mmax = warp_max(mmax);
    vmax = warp_max(vmax);
    if (live) {
      uint2 mo, vo;
      uint4 po;
      adam8_encode8(m2, sv2, p2, mmax, vmax, a.stochastic != 0, a.seed, (uint32_t)e0, mo, vo, po);
      *reinterpret_cast<uint2*>(mq + e0) = mo;
      *reinterpret_cast<uint2*>(vq + e0) = vo;
      *reinterpret_cast<uint4*>(param + e0) = po;
      if (lane == 0) {
        m_absmax[blk] = mmax;
        v_absmax[blk] = vmax;
      }
    }
  }
}

// 1: the packed-pair kernel (default), 0: the element-wise one (ERI_B200_ADAMW8_PAIR=0).
int g_adamw8_pair = -1;
bool adamw8_pair() {
  if (g_adamw8_pair < 0) {
    const char* e = getenv("ERI_B200_ADAMW8_PAIR");
    g_adamw8_pair = (e && e[0] == '0') ? 0 : 1;
  }
  return g_adamw8_pair == 1;
}

template <typename PT>
__global__ void adamw32_kernel(PT* __restrict__ param, const PT* __restrict__ grad,
                               float* __restrict__ m, float* __restrict__ v,
                               const float* __restrict__ grad_sumsq, long long n, AdamArgs a) {
  float gs = a.grad_scale;
  if (grad_sumsq) {
    const float ss = *grad_sumsq;
    if (!isfinite(ss)) return;  // non-finite gradients: leave parameters and state untouched
    if (a.max_grad_norm > 0.f) {
      float norm = sqrtf(ss) * a.grad_scale;
      gs *= fminf(1.f, a.max_grad_norm / (norm + 1e-6f));
    }
  }
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float g = (float)grad[i] * gs, p = (float)param[i];
    float mi = a.beta1 * m[i] + (1.f - a.beta1) * g;
    float vi = a.beta2 * v[i] + (1.f - a.beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    float upd = (mi / a.bc1) / (sqrtf(vi / a.bc2) + a.eps);
    p = p * (1.f - a.lr * a.weight_decay) - a.lr * upd;
    if constexpr (sizeof(PT) == 2)
      param[i] = round_bf16(p, a.stochastic != 0, hash_u32(a.seed ^ (uint32_t)i * 0x9E3779B9u));
    else
      param[i] = p;
  }
}

__global__ void ema_kernel(float* __restrict__ shadow, const bf16* __restrict__ param, long long n,
                           float decay) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    shadow[i] = decay * shadow[i] + (1.f - decay) * __bfloat162float(param[i]);
}

__global__ void scale_bf16_kernel(bf16* __restrict__ x, long long n, const float* __restrict__ sumsq,
                                  float max_norm, float extra) {
  float s = extra;
  if (sumsq && max_norm > 0.f) s *= fminf(1.f, max_norm / (sqrtf(*sumsq) + 1e-6f));
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    x[i] = __float2bfloat16(__bfloat162float(x[i]) * s);
}

inline int grid_for(long long n, int block) {
  long long g = (n + block - 1) / block;
  long long cap = 148 * 8;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

extern "C" {

// n: number of elements (multiple of 8); state arrays cover ceil(n/256) blocks.
// grad_sumsq (optional): device fp32 holding the squared global gradient norm (unscaled).
int eri_adamw8bit_step(void* param, const void* grad, void* mq, void* vq, float* m_absmax,
                       float* v_absmax, const float* grad_sumsq, long long n, float lr, float beta1,
                       float beta2, float eps, float weight_decay, int step, float max_grad_norm,
                       float grad_scale, unsigned int seed, int stochastic, void* stream) {
  if (n % 8 != 0 || step < 1) return -1;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.max_grad_norm = max_grad_norm; a.grad_scale = grad_scale; a.seed = seed * 2654435761u + step;
  a.stochastic = stochastic;
  long long nblocks = (n + kBlock - 1) / kBlock;
  auto kern = adamw8_pair() ? adamw8bit_pair_kernel : adamw8bit_kernel;
  kern<<<grid_for(nblocks * 32, 256), 256, 0, (cudaStream_t)stream>>>(
      (bf16*)param, (const bf16*)grad, (int8_t*)mq, (uint8_t*)vq, m_absmax, v_absmax, grad_sumsq,
      nblocks, n, a, nullptr);
  return (int)cudaGetLastError();
}

// Same step with a per-block learning-rate multiplier lr_scale[n / 256] (fp32, may be null).
int eri_adamw8bit_step_scaled(void* param, const void* grad, void* mq, void* vq, float* m_absmax,
                              float* v_absmax, const float* grad_sumsq, long long n, float lr, float beta1,
                              float beta2, float eps, float weight_decay, int step, float max_grad_norm,
                              float grad_scale, unsigned int seed, int stochastic, const float* lr_scale,
                              void* stream) {
  if (step < 1) return -1;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.max_grad_norm = max_grad_norm; a.grad_scale = grad_scale; a.seed = seed * 2654435761u + step;
  a.stochastic = stochastic;
  long long nblocks = (n + kBlock - 1) / kBlock;
  auto kern = adamw8_pair() ? adamw8bit_pair_kernel : adamw8bit_kernel;
  kern<<<grid_for(nblocks * 32, 256), 256, 0, (cudaStream_t)stream>>>(
      (bf16*)param, (const bf16*)grad, (int8_t*)mq, (uint8_t*)vq, m_absmax, v_absmax, grad_sumsq,
      nblocks, n, a, lr_scale);
  return (int)cudaGetLastError();
}

// Chooses the 8-bit AdamW kernel (1: packed pairs, 0: element-wise); returns the previous choice.
int eri_adamw8bit_set_pair_variant(int on) {
  const int prev = adamw8_pair() ? 1 : 0;
  g_adamw8_pair = on ? 1 : 0;
  return prev;
}

int eri_adamw32_step(void* param, const void* grad, float* m, float* v, const float* grad_sumsq,
                     long long n, int param_is_bf16, float lr, float beta1, float beta2, float eps,
                     float weight_decay, int step, float max_grad_norm, float grad_scale,
                     unsigned int seed, int stochastic, void* stream) {
  if (step < 1) return -1;
  AdamArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = 1.f - powf(beta1, (float)step);
  a.bc2 = 1.f - powf(beta2, (float)step);
  a.max_grad_norm = max_grad_norm; a.grad_scale = grad_scale; a.seed = seed * 2654435761u + step;
  a.stochastic = stochastic;
  if (param_is_bf16)
    adamw32_kernel<bf16><<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(
        (bf16*)param, (const bf16*)grad, m, v, grad_sumsq, n, a);
  else
    adamw32_kernel<float><<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(
        (float*)param, (const float*)grad, m, v, grad_sumsq, n, a);
  return (int)cudaGetLastError();
}

int eri_ema_update(float* shadow, const void* param, long long n, float decay, void* stream) {
  ema_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(shadow, (const bf16*)param, n,
                                                                 decay);
  return (int)cudaGetLastError();
}

int eri_scale_bf16(void* x, long long n, const float* sumsq, float max_norm, float extra,
                   void* stream) {
  scale_bf16_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>((bf16*)x, n, sumsq,
                                                                        max_norm, extra);
  return (int)cudaGetLastError();
}

}  // extern "C"
