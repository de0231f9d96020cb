// Memory-bound fused kernels (bf16 storage, fp32 math) for the transformer blocks:
//   norm_modulate   LayerNorm / RMSNorm (+ optional affine) + adaLN (1+scale), shift   fwd + bwd
//   qknorm_rope     per-head RMS QK-norm + interleaved-pair RoPE + head split/concat   fwd + bwd
//   gate_residual   x + gate * y                                                       fwd + bwd
//   activations     GELU(tanh), SiLU, GEGLU, SwiGLU                                    fwd + bwd
//   noise_mix       Philox N(0,1) noise, x_t / target construction, 2x2 patchify
//   mse             weighted MSE forward + gradient in one pass
//   sumsq           sum of squares of a flat buffer (gradient norm)
//
// These replace chains of 3-8 elementwise launches per call site in the reference
// (rms_norm + apply_scale_shift: crates/training/src/flux/runtime.rs:893-922;
//  apply_qk_norm: runtime.rs:1049-1092; rope: src/kernels/rope.cu:13-75;
//  gate/residual: runtime.rs:389-390; adaLN: src/models/mmdit_blocks.rs:238-277).
// All loads and stores are 16-byte vectors; every row is read from DRAM once.
#include "ptx.cuh"

using namespace eri;
typedef __nv_bfloat16 bf16;

#define ERI_LAUNCH_CHECK() return static_cast<int>(cudaGetLastError())

namespace {

constexpr int kMaxVec = 2;  // register-cached 8-element vectors per thread

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// ------------------------------------------------------------------ norm + modulation
// y = (xhat * w + b) * (1 + scale[batch]) + shift[batch]; xhat = (x - mean) * rstd (LayerNorm)
// or x * rstd (RMSNorm). w, b, scale, shift are each optional.
__global__ void __launch_bounds__(1024) norm_modulate_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ scale,
                                         const bf16* __restrict__ shift,
                                         const bf16* __restrict__ weight,
                                         const bf16* __restrict__ bias, bf16* __restrict__ y,
                                         float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                         int rows, int D, int rows_per_batch, int mod_stride,
                                         float eps, int rms) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const int nvec = D >> 3;
  const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)row * D);
  float xv[kMaxVec][8];
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      unpack8(xr[v], xv[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) s += rms ? xv[i][j] * xv[i][j] : xv[i][j];
    }
  }
  float mean = 0.f, rstd;
  if (rms) {
    float ss = block_sum(s, red);
    rstd = rsqrtf(ss / D + eps);
  } else {
    mean = block_sum(s, red) / D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float d = xv[i][j] - mean;
          q += d * d;
        }
      }
    }
    float var = block_sum(q, red) / D;
    rstd = rsqrtf(var + eps);
  }
  if (threadIdx.x == 0) {
    if (mean_out) mean_out[row] = mean;
    if (rstd_out) rstd_out[row] = rstd;
  }
  const int b = row / rows_per_batch;
  const bf16x8* sc = scale ? reinterpret_cast<const bf16x8*>(scale + (size_t)b * mod_stride) : nullptr;
  const bf16x8* sh = shift ? reinterpret_cast<const bf16x8*>(shift + (size_t)b * mod_stride) : nullptr;
  const bf16x8* wv = weight ? reinterpret_cast<const bf16x8*>(weight) : nullptr;
  const bf16x8* bv = bias ? reinterpret_cast<const bf16x8*>(bias) : nullptr;
  bf16x8* yr = reinterpret_cast<bf16x8*>(y + (size_t)row * D);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      float o[8], a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = (xv[i][j] - mean) * rstd;
      if (wv) {
        unpack8(wv[v], a);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] *= a[j];
      }
      if (bv) {
        unpack8(bv[v], a);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += a[j];
      }
      if (sc) {
        unpack8(sc[v], a);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] *= (1.f + a[j]);
      }
      if (sh) {
        unpack8(sh[v], a);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += a[j];
      }
      yr[v] = pack8(o);
    }
  }
}

// Backward. One CTA walks `rows_per_cta` consecutive rows so that the column sums that feed
// d_scale / d_shift / d_weight / d_bias are accumulated in registers and flushed with one
// fp32 atomicAdd per column per CTA (or when the batch index changes).
__global__ void __launch_bounds__(512) norm_modulate_bwd_kernel(
    const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ scale,
    const bf16* __restrict__ weight, const bf16* __restrict__ bias,
    const float* __restrict__ mean_in, const float* __restrict__ rstd_in, bf16* __restrict__ dx,
    float* __restrict__ dscale, float* __restrict__ dshift, float* __restrict__ dweight,
    float* __restrict__ dbias, int rows, int D, int rows_per_batch, int mod_stride, int rms,
    int rows_per_cta) {
  __shared__ float red[32];
  const int nvec = D >> 3;
  const int row0 = blockIdx.x * rows_per_cta;
  const int row1 = min(rows, row0 + rows_per_cta);
  const bool want_mod = dscale != nullptr || dshift != nullptr;
  const bool want_aff = dweight != nullptr || dbias != nullptr;
  float acc_sc[kMaxVec][8], acc_sh[kMaxVec][8], acc_w[kMaxVec][8], acc_b[kMaxVec][8];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc_sc[i][j] = acc_sh[i][j] = acc_w[i][j] = acc_b[i][j] = 0.f;
  int cur_b = row0 / rows_per_batch;

  auto flush_mod = [&](int b) {
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (dscale) atomicAdd(dscale + (size_t)b * D + v * 8 + j, acc_sc[i][j]);
          if (dshift) atomicAdd(dshift + (size_t)b * D + v * 8 + j, acc_sh[i][j]);
          acc_sc[i][j] = acc_sh[i][j] = 0.f;
        }
      }
    }
  };

  for (int row = row0; row < row1; ++row) {
    const int b = row / rows_per_batch;
    if (want_mod && b != cur_b) {
      flush_mod(cur_b);
      cur_b = b;
    }
    const float mean = rms ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    const bf16x8* xr = reinterpret_cast<const bf16x8*>(x + (size_t)row * D);
    const bf16x8* gr = reinterpret_cast<const bf16x8*>(dy + (size_t)row * D);
    const bf16x8* sc = scale ? reinterpret_cast<const bf16x8*>(scale + (size_t)b * mod_stride) : nullptr;
    const bf16x8* wv = weight ? reinterpret_cast<const bf16x8*>(weight) : nullptr;
    const bf16x8* bv = bias ? reinterpret_cast<const bf16x8*>(bias) : nullptr;
    float xh[kMaxVec][8], g[kMaxVec][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float xx[8], gg[8], a[8];
        unpack8(xr[v], xx);
        unpack8(gr[v], gg);
#pragma unroll
        for (int j = 0; j < 8; ++j) xh[i][j] = (xx[j] - mean) * rstd;
        float pre[8];  // value that (1+scale) multiplies
#pragma unroll
        for (int j = 0; j < 8; ++j) pre[j] = xh[i][j];
        float wj[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) wj[j] = 1.f;
        if (wv) {
          unpack8(wv[v], wj);
#pragma unroll
          for (int j = 0; j < 8; ++j) pre[j] *= wj[j];
        }
        if (bv) {
          unpack8(bv[v], a);
#pragma unroll
          for (int j = 0; j < 8; ++j) pre[j] += a[j];
        }
        if (want_mod) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc_sc[i][j] += gg[j] * pre[j];
            acc_sh[i][j] += gg[j];
          }
        }
        if (sc) {
          unpack8(sc[v], a);
#pragma unroll
          for (int j = 0; j < 8; ++j) gg[j] *= (1.f + a[j]);
        }
        if (want_aff) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc_w[i][j] += gg[j] * xh[i][j];
            acc_b[i][j] += gg[j];
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          g[i][j] = gg[j] * wj[j];
          s1 += g[i][j];
          s2 += g[i][j] * xh[i][j];
        }
      }
    }
    float c1 = rms ? 0.f : block_sum(s1, red) / D;
    float c2 = block_sum(s2, red) / D;
    bf16x8* dr = reinterpret_cast<bf16x8*>(dx + (size_t)row * D);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - c1 - xh[i][j] * c2);
        dr[v] = pack8(o);
      }
    }
  }
  if (want_mod) flush_mod(cur_b);
  if (want_aff) {
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (dweight) atomicAdd(dweight + v * 8 + j, acc_w[i][j]);
          if (dbias) atomicAdd(dbias + v * 8 + j, acc_b[i][j]);
        }
      }
    }
  }
}

// ------------------------------------------------------------------ QK-norm + RoPE + split
// Input  qkv : [B, L, 3, H, Dh]  (the QKV projection's output, "b l (k h d)")
// Output q,k,v : [B, Ltot, H, Dh] written at token offset l_off (joint txt||img sequences are
// assembled by two calls). q,k get per-head RMSNorm * scale (optional) and rotation of
// interleaved pairs by the angle table cos/sin [Ltot, Dh/2] (optional).
// One warp per (token, head); each lane owns Dh/32 consecutive elements (an even count).
template <int EPL>  // elements per lane: 2 (Dh=64) or 4 (Dh=128)
__global__ void qknorm_rope_fwd_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ qs,
                                       const bf16* __restrict__ ks, const float* __restrict__ cosT,
                                       const float* __restrict__ sinT, bf16* __restrict__ q,
                                       bf16* __restrict__ k, bf16* __restrict__ v, int B, int L,
                                       int H, int Ltot, int l_off, float eps, int in_tok_stride,
                                       int in_part_stride) {
  constexpr int Dh = EPL * 32;
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int total = B * L * H;
  if (warp >= total) return;
  const int h = warp % H;
  const int l = (warp / H) % L;
  const int b = warp / (H * L);
  const size_t in_base = ((size_t)b * L + l) * in_tok_stride + (size_t)h * Dh + lane * EPL;
  const size_t out_base = (((size_t)b * Ltot + l_off + l) * H + h) * Dh + lane * EPL;
  const float* cr = cosT ? cosT + (size_t)(l_off + l) * (Dh / 2) + lane * (EPL / 2) : nullptr;
  const float* sr = sinT ? sinT + (size_t)(l_off + l) * (Dh / 2) + lane * (EPL / 2) : nullptr;
#pragma unroll
  for (int part = 0; part < 3; ++part) {
    const bf16* src = qkv + in_base + (size_t)part * in_part_stride;
    bf16* dst = (part == 0 ? q : part == 1 ? k : v) + out_base;
    float f[EPL];
    if (EPL == 4) {
      uint2 raw = *reinterpret_cast<const uint2*>(src);
      float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.x));
      float2 c = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw.y));
      f[0] = a.x; f[1] = a.y; f[EPL - 2] = c.x; f[EPL - 1] = c.y;
    } else {
      uint32_t raw = *reinterpret_cast<const uint32_t*>(src);
      float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&raw));
      f[0] = a.x; f[1] = a.y;
    }
    if (part < 2) {
      const bf16* sp = part == 0 ? qs : ks;
      if (sp) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) ss += f[j] * f[j];
        ss = warp_sum(ss);
        float r = rsqrtf(ss / Dh + eps);
#pragma unroll
        for (int j = 0; j < EPL; ++j) f[j] = f[j] * r * __bfloat162float(sp[lane * EPL + j]);
      }
      if (cr) {
#pragma unroll
        for (int p = 0; p < EPL / 2; ++p) {
          float c = cr[p], s = sr[p];
          float a0 = f[2 * p], a1 = f[2 * p + 1];
          f[2 * p] = c * a0 - s * a1;
          f[2 * p + 1] = s * a0 + c * a1;
        }
      }
    }
    if (EPL == 4) {
      uint2 o;
      *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(f[0], f[1]);
      *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(f[EPL - 2], f[EPL - 1]);
      *reinterpret_cast<uint2*>(dst) = o;
    } else {
      *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(f[0], f[1]);
    }
  }
}

template <int EPL, bool SGRAD>
__global__ void qknorm_rope_bwd_kernel(const bf16* __restrict__ dq, const bf16* __restrict__ dk,
                                       const bf16* __restrict__ dv, const bf16* __restrict__ qkv,
                                       const bf16* __restrict__ qs, const bf16* __restrict__ ks,
                                       const float* __restrict__ cosT,
                                       const float* __restrict__ sinT, bf16* __restrict__ dqkv,
                                       float* __restrict__ dqs, float* __restrict__ dks, int B,
                                       int L, int H, int Ltot, int l_off, float eps,
                                       int in_tok_stride, int in_part_stride,
                                       int grad_tok_stride) {
  constexpr int Dh = EPL * 32;
  const int lane = threadIdx.x & 31;
  const int total = B * L * H;
  const int nwarps_grid = (gridDim.x * blockDim.x) >> 5;
  // Scale gradients: every warp keeps its share in registers over its (batch, token, head) items;
  // the CTA adds its warps in shared memory and issues one global atomic per element. (One atomic
  // per element per item put 100 k warps on the same 128 addresses: 1.2 ms per call.)
  // SGRAD = false (frozen scales: LoRA training) keeps the accumulators out of the register budget
  float acc_s[2][SGRAD ? EPL : 1];
  if constexpr (SGRAD) {
#pragma unroll
    for (int j = 0; j < EPL; ++j) acc_s[0][j] = acc_s[1][j] = 0.f;
  }
  for (int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; warp < total;
       warp += SGRAD ? nwarps_grid : total) {   // frozen scales: one item per warp, as many warps as items
  const int h = warp % H;
  const int l = (warp / H) % L;
  const int b = warp / (H * L);
  const size_t in_base = ((size_t)b * L + l) * in_tok_stride + (size_t)h * Dh + lane * EPL;
  const size_t grad_base = ((size_t)b * L + l) * grad_tok_stride + (size_t)h * Dh + lane * EPL;
  const size_t out_base = (((size_t)b * Ltot + l_off + l) * H + h) * Dh + lane * EPL;
  const float* cr = cosT ? cosT + (size_t)(l_off + l) * (Dh / 2) + lane * (EPL / 2) : nullptr;
  const float* sr = sinT ? sinT + (size_t)(l_off + l) * (Dh / 2) + lane * (EPL / 2) : nullptr;
#pragma unroll
  for (int part = 0; part < 3; ++part) {
    const bf16* gsrc = (part == 0 ? dq : part == 1 ? dk : dv) + out_base;
    bf16* dst = dqkv + grad_base + (size_t)part * in_part_stride;
    float g[EPL];
#pragma unroll
    for (int j = 0; j < EPL; j += 2) {
      float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gsrc + j));
      g[j] = a.x; g[j + 1] = a.y;
    }
    if (part < 2) {
      if (cr) {  // transpose of the rotation
#pragma unroll
        for (int p = 0; p < EPL / 2; ++p) {
          float c = cr[p], s = sr[p];
          float a0 = g[2 * p], a1 = g[2 * p + 1];
          g[2 * p] = c * a0 + s * a1;
          g[2 * p + 1] = -s * a0 + c * a1;
        }
      }
      const bf16* sp = part == 0 ? qs : ks;
      float* dsp = part == 0 ? dqs : dks;
      if (sp) {
        const bf16* xsrc = qkv + in_base + (size_t)part * in_part_stride;
        float x[EPL];
#pragma unroll
        for (int j = 0; j < EPL; j += 2) {
          float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xsrc + j));
          x[j] = a.x; x[j + 1] = a.y;
        }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) ss += x[j] * x[j];
        ss = warp_sum(ss);
        float r = rsqrtf(ss / Dh + eps);
        float c2 = 0.f;
        float xh[EPL];
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          xh[j] = x[j] * r;
          float sj = __bfloat162float(sp[lane * EPL + j]);
          if constexpr (SGRAD) {
            if (dsp) acc_s[part][j] += g[j] * xh[j];
          }
          g[j] *= sj;
          c2 += g[j] * xh[j];
        }
        c2 = warp_sum(c2) / Dh;
#pragma unroll
        for (int j = 0; j < EPL; ++j) g[j] = r * (g[j] - xh[j] * c2);
      }
    }
#pragma unroll
    for (int j = 0; j < EPL; j += 2)
      *reinterpret_cast<__nv_bfloat162*>(dst + j) = __floats2bfloat162_rn(g[j], g[j + 1]);
  }
  }
  if constexpr (SGRAD) {
    __shared__ float red[2][Dh];
    for (int i = threadIdx.x; i < 2 * Dh; i += blockDim.x) (&red[0][0])[i] = 0.f;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      if (dqs) atomicAdd(&red[0][lane * EPL + j], acc_s[0][j]);
      if (dks) atomicAdd(&red[1][lane * EPL + j], acc_s[1][j]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < Dh; i += blockDim.x) {
      if (dqs) atomicAdd(dqs + i, red[0][i]);
      if (dks) atomicAdd(dks + i, red[1][i]);
    }
  }
}

// ------------------------------------------------------------------ gate + residual
// out = x + gate[batch] * y   (gate optional: plain add)
__global__ void gate_residual_kernel(const bf16* __restrict__ x, const bf16* __restrict__ y,
                                     const bf16* __restrict__ gate, bf16* __restrict__ out,
                                     size_t nvec, int D, int rows_per_batch, int mod_stride) {
  const int dv = D >> 3;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    float a[8], c[8];
    unpack8(reinterpret_cast<const bf16x8*>(y)[i], c);
    if (gate) {
      size_t row = i / dv;
      int col = (int)(i - row * dv);
      int b = (int)(row / rows_per_batch);
      float g[8];
      unpack8(reinterpret_cast<const bf16x8*>(gate + (size_t)b * mod_stride)[col], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] *= g[j];
    }
    if (x) {
      unpack8(reinterpret_cast<const bf16x8*>(x)[i], a);
#pragma unroll
      for (int j = 0; j < 8; ++j) c[j] += a[j];
    }
    reinterpret_cast<bf16x8*>(out)[i] = pack8(c);
  }
}
// d_gate[b, d] += sum over the batch's tokens of dout * y
__global__ void gate_grad_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ y,
                                 float* __restrict__ dgate, int rows, int D, int rows_per_batch,
                                 int rows_per_cta) {
  const int nvec = D >> 3;
  const int row0 = blockIdx.x * rows_per_cta, row1 = min(rows, row0 + rows_per_cta);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    int cur_b = row0 / rows_per_batch;
    for (int row = row0; row < row1; ++row) {
      int b = row / rows_per_batch;
      if (b != cur_b) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          atomicAdd(dgate + (size_t)cur_b * D + v * 8 + j, acc[j]);
          acc[j] = 0.f;
        }
        cur_b = b;
      }
      float a[8], c[8];
      unpack8(reinterpret_cast<const bf16x8*>(dout + (size_t)row * D)[v], a);
      unpack8(reinterpret_cast<const bf16x8*>(y + (size_t)row * D)[v], c);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += a[j] * c[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(dgate + (size_t)cur_b * D + v * 8 + j, acc[j]);
  }
}

// ------------------------------------------------------------------ activations
// mode 0 GELU(tanh), 1 SiLU. bwd: dx = dy * f'(x)
__global__ void act_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, size_t nvec,
                               int mode) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    float a[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[i], a);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = mode == 0 ? gelu_tanh_f(a[j]) : silu_f(a[j]);
    reinterpret_cast<bf16x8*>(y)[i] = pack8(a);
  }
}
__global__ void act_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                               bf16* __restrict__ dx, size_t nvec, int mode) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    float a[8], g[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[i], a);
    unpack8(reinterpret_cast<const bf16x8*>(dy)[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= mode == 0 ? gelu_tanh_grad_f(a[j]) : silu_grad_f(a[j]);
    reinterpret_cast<bf16x8*>(dx)[i] = pack8(g);
  }
}
// y[r, c] = act(x[r, c]) on row-strided [rows, cols] views.
__global__ void act_fwd_rows_kernel(const bf16* __restrict__ x, long long ld_x, bf16* __restrict__ y, long long ld_y,
                                    int rows, int cols, int mode) {
  const int cv = cols >> 3;
  const size_t n = (size_t)rows * cv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / cv;
    const int c = (int)(i - row * cv) * 8;
    float a[8];
    unpack8(*reinterpret_cast<const bf16x8*>(x + row * ld_x + c), a);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = mode == 0 ? gelu_tanh_f(a[j]) : silu_f(a[j]);
    *reinterpret_cast<bf16x8*>(y + row * ld_y + c) = pack8(a);
  }
}
// The same on row-strided views (a column block of a wider matrix), in place when dx == dy.
__global__ void act_bwd_rows_kernel(const bf16* dy, long long ld_dy, const bf16* __restrict__ x, long long ld_x,
                                    bf16* dx, long long ld_dx, int rows, int cols, int mode) {
  const int cv = cols >> 3;
  const size_t n = (size_t)rows * cv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t row = i / cv;
    const int c = (int)(i - row * cv) * 8;
    float a[8], g[8];
    unpack8(*reinterpret_cast<const bf16x8*>(x + row * ld_x + c), a);
    unpack8(*reinterpret_cast<const bf16x8*>(dy + row * ld_dy + c), g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= mode == 0 ? gelu_tanh_grad_f(a[j]) : silu_grad_f(a[j]);
    *reinterpret_cast<bf16x8*>(dx + row * ld_dx + c) = pack8(g);
  }
}
// Gated linear units on h = [rows, 2F]: out = act(h[:, :F]) * h[:, F:] when act_first,
// else h[:, :F] * act(h[:, F:]).  mode 0 = GELU(tanh) (GEGLU), 1 = SiLU (SwiGLU).
__global__ void glu_fwd_kernel(const bf16* __restrict__ h, bf16* __restrict__ out, int rows, int F,
                               int mode, int act_first) {
  const int fv = F >> 3;
  const size_t n = (size_t)rows * fv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    size_t row = i / fv;
    int c = (int)(i - row * fv);
    const bf16x8* hr = reinterpret_cast<const bf16x8*>(h + row * 2 * (size_t)F);
    float a[8], g[8];
    unpack8(hr[c], a);
    unpack8(hr[fv + c], g);
    if (!act_first) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { float t = a[j]; a[j] = g[j]; g[j] = t; }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = (mode == 0 ? gelu_tanh_f(a[j]) : silu_f(a[j])) * g[j];
    reinterpret_cast<bf16x8*>(out + row * (size_t)F)[c] = pack8(a);
  }
}
__global__ void glu_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ h,
                               bf16* __restrict__ dh, int rows, int F, int mode, int act_first) {
  const int fv = F >> 3;
  const size_t n = (size_t)rows * fv;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    size_t row = i / fv;
    int c = (int)(i - row * fv);
    const bf16x8* hr = reinterpret_cast<const bf16x8*>(h + row * 2 * (size_t)F);
    bf16x8* dr = reinterpret_cast<bf16x8*>(dh + row * 2 * (size_t)F);
    float a[8], g[8], d[8], da[8], dg[8];
    unpack8(hr[act_first ? c : fv + c], a);   // activated half
    unpack8(hr[act_first ? fv + c : c], g);   // linear half
    unpack8(reinterpret_cast<const bf16x8*>(dout + row * (size_t)F)[c], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float f = mode == 0 ? gelu_tanh_f(a[j]) : silu_f(a[j]);
      float fp = mode == 0 ? gelu_tanh_grad_f(a[j]) : silu_grad_f(a[j]);
      da[j] = d[j] * g[j] * fp;
      dg[j] = d[j] * f;
    }
    dr[act_first ? c : fv + c] = pack8(da);
    dr[act_first ? fv + c : c] = pack8(dg);
  }
}

// ------------------------------------------------------------------ Philox noise + mixing
__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
  uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
  uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}
__device__ __forceinline__ void philox4x32(uint64_t seed, uint64_t ctr, uint32_t (&out)[4]) {
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  uint32_t c[4] = {(uint32_t)ctr, (uint32_t)(ctr >> 32), 0x9E3779B9u, 0xBB67AE85u};
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = c[i];
}
__device__ __forceinline__ void normal4(uint64_t seed, uint64_t ctr, float (&z)[4]) {
  uint32_t r[4];
  philox4x32(seed, ctr, r);
  const float inv = 2.3283064365386963e-10f;  // 2^-32
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    float u1 = (r[2 * p] + 0.5f) * inv, u2 = (r[2 * p + 1] + 0.5f) * inv;
    float rad = sqrtf(-2.f * __logf(u1));
    float s, c;
    __sincosf(6.283185307179586f * u2, &s, &c);
    z[2 * p] = rad * c;
    z[2 * p + 1] = rad * s;
  }
}
// x0: [B, C, H, W]. Writes token-major tensors [B, (H/p)*(W/p), C*p*p] ("b c (h ph) (w pw) ->
// b (h w) (c ph pw)"):  x_t = a[b]*x0 + s[b]*eps,  target = ca[b]*eps + cb[b]*x0, and eps itself
// when eps_out is given. If eps_in is given it is used instead of the generator.
__global__ void noise_mix_kernel(const bf16* __restrict__ x0, const bf16* __restrict__ eps_in,
                                 const float* __restrict__ coef,  // [4, B]: a, s, ca, cb
                                 bf16* __restrict__ xt, bf16* __restrict__ target,
                                 bf16* __restrict__ eps_out, int B, int C, int H, int W, int p,
                                 uint64_t seed, uint64_t offset) {
  const size_t per = (size_t)C * H * W;
  const size_t n4 = (size_t)B * per / 4;
  const int Wp = W / p, Hp = H / p;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4;
       i += (size_t)gridDim.x * blockDim.x) {
    float z[4];
    if (!eps_in) normal4(seed, offset + i, z);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      size_t e = i * 4 + j;  // NCHW linear index
      int b = (int)(e / per);
      size_t r = e - (size_t)b * per;
      int c = (int)(r / ((size_t)H * W));
      int hw = (int)(r - (size_t)c * H * W);
      int hh = hw / W, ww = hw - hh * W;
      float xv = __bfloat162float(x0[e]);
      float ev = eps_in ? __bfloat162float(eps_in[e]) : z[j];
      size_t tok = (size_t)(hh / p) * Wp + (ww / p);
      size_t o = ((size_t)b * Hp * Wp + tok) * ((size_t)C * p * p) + (size_t)c * p * p +
                 (hh % p) * p + (ww % p);
      float a = coef[b], s = coef[B + b], ca = coef[2 * B + b], cb = coef[3 * B + b];
      xt[o] = __float2bfloat16(a * xv + s * ev);
      if (target) target[o] = __float2bfloat16(ca * ev + cb * xv);
      if (eps_out) eps_out[o] = __float2bfloat16(ev);
    }
  }
}
__global__ void randn_bf16_kernel(bf16* __restrict__ out, size_t n, uint64_t seed, uint64_t offset,
                                  float mean, float std) {
  const size_t n4 = (n + 3) / 4;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4;
       i += (size_t)gridDim.x * blockDim.x) {
    float z[4];
    normal4(seed, offset + i, z);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (i * 4 + j < n) out[i * 4 + j] = __float2bfloat16(mean + std * z[j]);
  }
}

// ------------------------------------------------------------------ weighted MSE fwd+bwd
// loss += sum_b w[b] * sum_i (p - t)^2 / n ;  dpred = 2 * w[b] * (p - t) * gscale / n
__global__ void mse_fwd_bwd_kernel(const bf16* __restrict__ pred, const bf16* __restrict__ target,
                                   const float* __restrict__ weight, float* __restrict__ loss,
                                   bf16* __restrict__ dpred, size_t n, size_t n_per_batch,
                                   float gscale) {
  __shared__ float red[32];
  float acc = 0.f;
  const float inv_n = 1.f / (float)n;
  const size_t nvec = n >> 3;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    float p[8], t[8];
    unpack8(reinterpret_cast<const bf16x8*>(pred)[i], p);
    unpack8(reinterpret_cast<const bf16x8*>(target)[i], t);
    float w = weight ? weight[(i * 8) / n_per_batch] : 1.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float d = p[j] - t[j];
      acc += w * d * d;
      p[j] = 2.f * w * d * gscale * inv_n;
    }
    if (dpred) reinterpret_cast<bf16x8*>(dpred)[i] = pack8(p);
  }
  float tot = block_sum(acc, red);
  if (threadIdx.x == 0) atomicAdd(loss, tot * inv_n);
}

__global__ void sumsq_kernel(const bf16* __restrict__ x, size_t n, float* __restrict__ out) {
  __shared__ float red[32];
  float acc = 0.f;
  const size_t nvec = n >> 3;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    float a[8];
    unpack8(reinterpret_cast<const bf16x8*>(x)[i], a);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += a[j] * a[j];
  }
  if (blockIdx.x == 0 && threadIdx.x == 0)
    for (size_t i = nvec << 3; i < n; ++i) {
      float a = __bfloat162float(x[i]);
      acc += a * a;
    }
  float tot = block_sum(acc, red);
  if (threadIdx.x == 0) atomicAdd(out, tot);
}

// out[i] = clamp((x[i] + 1) / 2, 0, 1) * 255 as bytes (image post-processing after VAE decode;
// reference: crates/common/vae/src/sdxl.rs:36-50 does the clamp in place on bf16).
__global__ void post_clamp_u8_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ out, size_t n) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x) {
    float v = fminf(fmaxf((__bfloat162float(x[i]) + 1.f) * 0.5f, 0.f), 1.f);
    out[i] = (uint8_t)__float2int_rn(v * 255.f);
  }
}
// Debug allocator poison (reference: crates/core/src/cuda_memory.rs:42-55).
__global__ void poison_fill_kernel(uint32_t* __restrict__ p, size_t nwords, uint32_t pattern) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nwords;
       i += (size_t)gridDim.x * blockDim.x)
    p[i] = pattern;
}

inline int grid_for(size_t n, int block) {
  size_t g = (n + block - 1) / block;
  size_t cap = 148 * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}
inline int row_threads(int D, int max_threads) {
  int nvec = D >> 3;
  int t = ((nvec + 31) / 32) * 32;
  if (t > max_threads) t = (((nvec + kMaxVec - 1) / kMaxVec + 31) / 32) * 32;
  return t < 32 ? 32 : t;
}

}  // namespace

extern "C" {

int eri_norm_modulate_fwd(const void* x, const void* scale, const void* shift, const void* weight,
                          const void* bias, void* y, float* mean, float* rstd, int rows, int D,
                          int rows_per_batch, int mod_stride, float eps, int rms, void* stream) {
  if (D % 8 != 0 || D > 8 * 1024 * kMaxVec) return -1;
  norm_modulate_fwd_kernel<<<rows, row_threads(D, 1024), 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (const bf16*)scale, (const bf16*)shift, (const bf16*)weight,
      (const bf16*)bias, (bf16*)y, mean, rstd, rows, D, rows_per_batch, mod_stride, eps, rms);
  ERI_LAUNCH_CHECK();
}

int eri_norm_modulate_bwd(const void* dy, const void* x, const void* scale, const void* weight,
                          const void* bias, const float* mean, const float* rstd, void* dx,
                          float* dscale, float* dshift, float* dweight, float* dbias, int rows,
                          int D, int rows_per_batch, int mod_stride, int rms, void* stream) {
  if (D % 8 != 0 || D > 8 * 512 * kMaxVec) return -1;
  const bool reduce = dscale || dshift || dweight || dbias;
  const int rpc = reduce ? 8 : 1;
  norm_modulate_bwd_kernel<<<(rows + rpc - 1) / rpc, row_threads(D, 512), 0, (cudaStream_t)stream>>>(
      (const bf16*)dy, (const bf16*)x, (const bf16*)scale, (const bf16*)weight, (const bf16*)bias,
      mean, rstd, (bf16*)dx, dscale, dshift, dweight, dbias, rows, D, rows_per_batch, mod_stride,
      rms, rpc);
  ERI_LAUNCH_CHECK();
}

int eri_qknorm_rope_fwd(const void* qkv, const void* qs, const void* ks, const float* cosT,
                        const float* sinT, void* q, void* k, void* v, int B, int L, int H, int Dh,
                        int Ltot, int l_off, float eps, int in_tok_stride, int in_part_stride,
                        void* stream) {
  const int total = B * L * H;
  const int block = 256;
  const int grid = (total * 32 + block - 1) / block;
  if (Dh == 128)
    qknorm_rope_fwd_kernel<4><<<grid, block, 0, (cudaStream_t)stream>>>(
        (const bf16*)qkv, (const bf16*)qs, (const bf16*)ks, cosT, sinT, (bf16*)q, (bf16*)k,
        (bf16*)v, B, L, H, Ltot, l_off, eps, in_tok_stride, in_part_stride);
  else if (Dh == 64)
    qknorm_rope_fwd_kernel<2><<<grid, block, 0, (cudaStream_t)stream>>>(
        (const bf16*)qkv, (const bf16*)qs, (const bf16*)ks, cosT, sinT, (bf16*)q, (bf16*)k,
        (bf16*)v, B, L, H, Ltot, l_off, eps, in_tok_stride, in_part_stride);
  else
    return -1;
  ERI_LAUNCH_CHECK();
}

int eri_qknorm_rope_bwd(const void* dq, const void* dk, const void* dv, const void* qkv,
                        const void* qs, const void* ks, const float* cosT, const float* sinT,
                        void* dqkv, float* dqs, float* dks, int B, int L, int H, int Dh, int Ltot,
                        int l_off, float eps, int in_tok_stride, int in_part_stride,
                        int grad_tok_stride, void* stream) {
  const int total = B * L * H;
  const int block = 256;
  int grid = (total * 32 + block - 1) / block;
  // with scale gradients the grid is capped (a CTA then loops over its items and reduces once)
  if ((dqs || dks) && grid > 148 * 8) grid = 148 * 8;
#define ERI_QKN_BWD(E, SG)                                                                       \
  qknorm_rope_bwd_kernel<E, SG><<<grid, block, 0, (cudaStream_t)stream>>>(                       \
      (const bf16*)dq, (const bf16*)dk, (const bf16*)dv, (const bf16*)qkv, (const bf16*)qs,      \
      (const bf16*)ks, cosT, sinT, (bf16*)dqkv, dqs, dks, B, L, H, Ltot, l_off, eps,             \
      in_tok_stride, in_part_stride, grad_tok_stride)
  const bool sg = dqs || dks;
  if (Dh == 128) {
    if (sg) ERI_QKN_BWD(4, true); else ERI_QKN_BWD(4, false);
  } else if (Dh == 64) {
    if (sg) ERI_QKN_BWD(2, true); else ERI_QKN_BWD(2, false);
  } else {
    return -1;
  }
#undef ERI_QKN_BWD
  ERI_LAUNCH_CHECK();
}

int eri_gate_residual(const void* x, const void* y, const void* gate, void* out, long long rows,
                      int D, int rows_per_batch, int mod_stride, void* stream) {
  if (D % 8 != 0) return -1;
  size_t nvec = (size_t)rows * (D >> 3);
  gate_residual_kernel<<<grid_for(nvec, 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)x, (const bf16*)y, (const bf16*)gate, (bf16*)out, nvec, D, rows_per_batch,
      mod_stride);
  ERI_LAUNCH_CHECK();
}

int eri_gate_grad(const void* dout, const void* y, float* dgate, int rows, int D,
                  int rows_per_batch, void* stream) {
  if (D % 8 != 0) return -1;
  const int rpc = 32;
  gate_grad_kernel<<<(rows + rpc - 1) / rpc, 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)dout, (const bf16*)y, dgate, rows, D, rows_per_batch, rpc);
  ERI_LAUNCH_CHECK();
}

int eri_act_fwd(const void* x, void* y, long long n, int mode, void* stream) {
  if (n % 8 != 0) return -1;
  act_fwd_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y,
                                                                        n / 8, mode);
  ERI_LAUNCH_CHECK();
}
int eri_act_bwd(const void* dy, const void* x, void* dx, long long n, int mode, void* stream) {
  if (n % 8 != 0) return -1;
  act_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)dy, (const bf16*)x, (bf16*)dx, n / 8, mode);
  ERI_LAUNCH_CHECK();
}
int eri_act_fwd_rows(const void* x, long long ld_x, void* y, long long ld_y, int rows, int cols, int mode,
                     void* stream) {
  if (cols % 8 || ld_x % 8 || ld_y % 8 || ((((uintptr_t)x | (uintptr_t)y) & 15) != 0)) return -1;
  act_fwd_rows_kernel<<<grid_for((size_t)rows * cols / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)x, ld_x, (bf16*)y, ld_y, rows, cols, mode);
  ERI_LAUNCH_CHECK();
}
// dx[r, c] = dy[r, c] * act'(x[r, c]) on row-strided [rows, cols] views (strides in elements, multiples of 8;
// 16-byte aligned bases); dx may be dy.
int eri_act_bwd_rows(const void* dy, long long ld_dy, const void* x, long long ld_x, void* dx, long long ld_dx,
                     int rows, int cols, int mode, void* stream) {
  if (cols % 8 || ld_dy % 8 || ld_x % 8 || ld_dx % 8) return -1;
  if ((((uintptr_t)dy | (uintptr_t)x | (uintptr_t)dx) & 15) != 0) return -1;
  act_bwd_rows_kernel<<<grid_for((size_t)rows * cols / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)dy, ld_dy, (const bf16*)x, ld_x, (bf16*)dx, ld_dx, rows, cols, mode);
  ERI_LAUNCH_CHECK();
}
int eri_glu_fwd(const void* h, void* out, int rows, int F, int mode, int act_first, void* stream) {
  if (F % 8 != 0) return -1;
  glu_fwd_kernel<<<grid_for((size_t)rows * F / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)h, (bf16*)out, rows, F, mode, act_first);
  ERI_LAUNCH_CHECK();
}
int eri_glu_bwd(const void* dout, const void* h, void* dh, int rows, int F, int mode,
                int act_first, void* stream) {
  if (F % 8 != 0) return -1;
  glu_bwd_kernel<<<grid_for((size_t)rows * F / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)dout, (const bf16*)h, (bf16*)dh, rows, F, mode, act_first);
  ERI_LAUNCH_CHECK();
}

int eri_noise_mix(const void* x0, const void* eps_in, const float* coef, void* xt, void* target,
                  void* eps_out, int B, int C, int H, int W, int p, unsigned long long seed,
                  unsigned long long offset, void* stream) {
  size_t n = (size_t)B * C * H * W;
  if (n % 4 != 0 || H % p != 0 || W % p != 0) return -1;
  noise_mix_kernel<<<grid_for(n / 4, 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)x0, (const bf16*)eps_in, coef, (bf16*)xt, (bf16*)target, (bf16*)eps_out, B, C,
      H, W, p, seed, offset);
  ERI_LAUNCH_CHECK();
}
int eri_randn_bf16(void* out, long long n, unsigned long long seed, unsigned long long offset,
                   float mean, float std, void* stream) {
  randn_bf16_kernel<<<grid_for((n + 3) / 4, 256), 256, 0, (cudaStream_t)stream>>>(
      (bf16*)out, (size_t)n, seed, offset, mean, std);
  ERI_LAUNCH_CHECK();
}

// loss must be zeroed by the caller (one fp32).
int eri_mse_fwd_bwd(const void* pred, const void* target, const float* weight, float* loss,
                    void* dpred, long long n, long long n_per_batch, float gscale, void* stream) {
  if (n % 8 != 0 || n_per_batch % 8 != 0) return -1;
  mse_fwd_bwd_kernel<<<grid_for(n / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (const bf16*)pred, (const bf16*)target, weight, loss, (bf16*)dpred, (size_t)n,
      (size_t)n_per_batch, gscale);
  ERI_LAUNCH_CHECK();
}
// out must be zeroed by the caller (one fp32).
int eri_sumsq_bf16(const void* x, long long n, float* out, void* stream) {
  sumsq_kernel<<<grid_for(n / 8 + 1, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)x,
                                                                           (size_t)n, out);
  ERI_LAUNCH_CHECK();
}
int eri_post_clamp_u8(const void* x, void* out, long long n, void* stream) {
  post_clamp_u8_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)x,
                                                                           (uint8_t*)out, n);
  ERI_LAUNCH_CHECK();
}
int eri_poison_fill(void* p, long long nbytes, unsigned int pattern, void* stream) {
  poison_fill_kernel<<<grid_for(nbytes / 4, 256), 256, 0, (cudaStream_t)stream>>>(
      (uint32_t*)p, (size_t)nbytes / 4, pattern);
  ERI_LAUNCH_CHECK();
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Batched transpose of many small bf16 matrices in one launch (the LoRA A / B matrices of every
// adapted linear: backward needs B^T and A^T). grid = (chunks of the largest matrix, matrices).
namespace {
struct TransposeJob {
  const bf16* src;
  bf16* dst;
  int rows, cols;
};
__global__ void batched_transpose_kernel(const TransposeJob* __restrict__ jobs) {
  const TransposeJob j = jobs[blockIdx.y];
  const long long n = (long long)j.rows * j.cols;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // index into dst [cols, rows]
  if (i >= n) return;
  const int c = (int)(i / j.rows), r = (int)(i - (long long)c * j.rows);
  j.dst[i] = j.src[(long long)r * j.cols + c];
}
}  // namespace

extern "C" int eri_batched_transpose(const void* jobs, int n_jobs, int max_elems, void* stream) {
  if (n_jobs < 1) return 0;
  dim3 grid((max_elems + 255) / 256, n_jobs);
  batched_transpose_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const TransposeJob*)jobs);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// out[i] (+)= scale * sum_w slots[w][i]: the owner's side of the weight-gradient reduce-scatter that
// the dW GEMM's row-slab scatter epilogue starts (every rank has pushed its partial slab into slot
// `rank` of this rank's receive buffer). fp32 sum, bf16 in / out, eight elements per thread.
namespace {
__global__ void slot_reduce_kernel(const bf16* __restrict__ slots, bf16* __restrict__ out, int world,
                                   long long n, float scale, int accumulate) {
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < n; i += stride) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int w = 0; w < world; ++w) {
      float f[8];
      unpack8(*reinterpret_cast<const bf16x8*>(slots + (size_t)w * n + i), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= scale;
    if (accumulate) {
      float f[8];
      unpack8(*reinterpret_cast<const bf16x8*>(out + i), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += f[j];
    }
    *reinterpret_cast<bf16x8*>(out + i) = pack8(acc);
  }
}
}  // namespace

extern "C" int eri_slot_reduce(const void* slots, void* out, int world, long long n, float scale,
                               int accumulate, void* stream) {
  if (n % 8 || world < 1) return -1;
  const int block = 256;
  long long blocks = (n / 8 + block - 1) / block;
  if (blocks > 148 * 8) blocks = 148 * 8;
  slot_reduce_kernel<<<(unsigned)blocks, block, 0, (cudaStream_t)stream>>>((const bf16*)slots, (bf16*)out, world, n,
                                                                          scale, accumulate);
  return (int)cudaGetLastError();
}
