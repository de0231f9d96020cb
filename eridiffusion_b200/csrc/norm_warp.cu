// Warp-per-row LayerNorm / RMSNorm + adaLN modulation (forward and input-gradient backward),
// persistent and fed by bulk asynchronous copies.
//
// Each warp owns a two-stage ring in shared memory. One lane issues `cp.async.bulk` row copies
// (global -> shared, completion on an mbarrier) two rows ahead; the warp waits for a row, moves it
// into registers as packed bf16 (one 16-byte shared load per lane per 256 columns), hands the
// stage straight back to the copy engine, and then does its passes over registers: reductions are
// warp shuffles, no block barrier anywhere. With 8-16 warps per SM that keeps 100-190 KB of loads
// in flight per SM, which is what the HBM pipe needs; the CTA-per-row kernels in elementwise.cu
// had only a few rows outstanding per SM and reached a quarter of the copy bandwidth.
// Used when D is a multiple of 8 in [256, 4096] and (backward) no parameter gradients are
// requested; other cases run the kernels in elementwise.cu (same math).
// Reference counterpart: layer_norm / rms_norm followed by separate modulate ops
// (crates/training/src/flux/runtime.rs:2153-2278); its backward is composed from tensor ops.
#include "ptx.cuh"

using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

struct NormArgs {
  const bf16 *x, *dy, *scale, *shift, *weight, *bias;
  const bf16* addend;  // backward only (may be null): added to dx, e.g. the gradient of a residual branch of x
  bf16* out;  // y (forward) or dx (backward)
  float *mean, *rstd;
  int rows, D, rows_per_batch, mod_stride;
  float eps;
  int rms;
  int* err;
};

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// eight bf16 -> four packed fp32 pairs and back
__device__ __forceinline__ void unpack8_f2(const bf16x8& r, f32x2 (&p)[4]) {
  const uint4 u = r.u;
  p[0] = f2_pack_bits(u.x << 16, u.x & 0xffff0000u);
  p[1] = f2_pack_bits(u.y << 16, u.y & 0xffff0000u);
  p[2] = f2_pack_bits(u.z << 16, u.z & 0xffff0000u);
  p[3] = f2_pack_bits(u.w << 16, u.w & 0xffff0000u);
}
__device__ __forceinline__ bf16x8 pack8_f2(const f32x2 (&p)[4]) {
  bf16x8 o;
  o.u = make_uint4(f2_to_bf162(p[0]), f2_to_bf162(p[1]), f2_to_bf162(p[2]), f2_to_bf162(p[3]));
  return o;
}

constexpr int kBarBytes = 1024;  // room for 32 warps x 3 stages of mbarriers
// Ring depth per warp. Three stages for the forward (all rows of a warp in flight at 4608 rows) were
// measured slower in the training step (25.2 against 22.1 us per launch): two it is.
template <bool BWD>
constexpr int kRingStages = 2;

template <int VPL, bool BWD>
__global__ void __launch_bounds__(BWD ? 256 : 384, 1) norm_rows_kernel(const NormArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int NT = BWD ? 2 : 1;
  constexpr int NS = kRingStages<BWD>;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int D = a.D, nvec = D >> 3;
  const uint32_t row_bytes = (uint32_t)D * 2u;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem) + warp * NS;
  uint8_t* ring = smem + kBarBytes + (size_t)warp * NS * NT * row_bytes;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NS; ++s) mbar_init(&bars[s], 1);
    mbar_fence_init();
  }
  __syncwarp();
  const int stride = gridDim.x * nwarps;
  const int row0 = blockIdx.x * nwarps + warp;
  auto issue = [&](int row, int st) {
    mbar_expect_tx(&bars[st], NT * row_bytes);
    bulk_g2s(ring + (size_t)st * NT * row_bytes, a.x + (size_t)row * D, row_bytes, &bars[st]);
    if (BWD)
      bulk_g2s(ring + (size_t)st * NT * row_bytes + row_bytes, a.dy + (size_t)row * D, row_bytes,
               &bars[st]);
  };
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < NS; ++s)
      if (row0 + s * stride < a.rows) issue(row0 + s * stride, s);
  }
  const bf16x8* wv = a.weight ? reinterpret_cast<const bf16x8*>(a.weight) : nullptr;
  const bf16x8* bv = a.bias ? reinterpret_cast<const bf16x8*>(a.bias) : nullptr;
  const float inv_d = 1.f / (float)D;
  int it = 0;
  for (int row = row0; row < a.rows; row += stride, ++it) {
    const int st = it % NS;
    if (!mbar_wait(&bars[st], (uint32_t)((it / NS) & 1))) {
      if (lane == 0) atomicExch(a.err, 1);
      break;
    }
    const bf16x8* sx = reinterpret_cast<const bf16x8*>(ring + (size_t)st * NT * row_bytes);
    // fp32 math runs on packed pairs (one fma / add per two elements): the row is unpacked once
    // into registers, so every later pass is pure FMA-pipe work.
    f32x2 xs[VPL][4];
    f32x2 gs[BWD ? VPL : 1][4];
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int v = lane + 32 * i;
      if (v < nvec) {
        unpack8_f2(sx[v], xs[i]);
        if (BWD) unpack8_f2(sx[nvec + v], gs[i]);
      }
    }
    __syncwarp();
    if (lane == 0 && row + NS * stride < a.rows) {
      fence_proxy_async_smem();  // the warp's reads of this stage precede the copy engine's writes
      issue(row + NS * stride, st);
    }
    const int b = row / a.rows_per_batch;
    const bf16x8* sc =
        a.scale ? reinterpret_cast<const bf16x8*>(a.scale + (size_t)b * a.mod_stride) : nullptr;
    bf16x8* orow = reinterpret_cast<bf16x8*>(a.out + (size_t)row * D);
    const f32x2 zero2 = f2_pack(0.f, 0.f);

    if (!BWD) {
      const bf16x8* sh =
          a.shift ? reinterpret_cast<const bf16x8*>(a.shift + (size_t)b * a.mod_stride) : nullptr;
      f32x2 acc = zero2;
#pragma unroll
      for (int i = 0; i < VPL; ++i)
        if (lane + 32 * i < nvec) {
#pragma unroll
          for (int j = 0; j < 4; ++j) acc = a.rms ? f2_fma(xs[i][j], xs[i][j], acc) : f2_add(acc, xs[i][j]);
        }
      float lo, hi;
      f2_unpack(acc, lo, hi);
      const float s = warp_sum(lo + hi);
      float mean = 0.f, rstd;
      if (a.rms) {
        rstd = rsqrtf(s * inv_d + a.eps);
      } else {
        mean = s * inv_d;
        const f32x2 m2 = f2_pack(mean, mean);
        f32x2 q = zero2;
#pragma unroll
        for (int i = 0; i < VPL; ++i)
          if (lane + 32 * i < nvec) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const f32x2 d = f2_sub(xs[i][j], m2);
              q = f2_fma(d, d, q);
            }
          }
        f2_unpack(q, lo, hi);
        rstd = rsqrtf(warp_sum(lo + hi) * inv_d + a.eps);
      }
      if (lane == 0) {
        if (a.mean) a.mean[row] = mean;
        if (a.rstd) a.rstd[row] = rstd;
      }
      const f32x2 a2 = f2_pack(rstd, rstd), b2 = f2_pack(-mean * rstd, -mean * rstd);
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int v = lane + 32 * i;
        if (v < nvec) {
          f32x2 o[4], t[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = f2_fma(xs[i][j], a2, b2);
          if (wv) {
            unpack8_f2(wv[v], t);
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = f2_mul(o[j], t[j]);
          }
          if (bv) {
            unpack8_f2(bv[v], t);
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = f2_add(o[j], t[j]);
          }
          if (sc) {
            unpack8_f2(sc[v], t);
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = f2_fma(o[j], t[j], o[j]);
          }
          if (sh) {
            unpack8_f2(sh[v], t);
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = f2_add(o[j], t[j]);
          }
          orow[v] = pack8_f2(o);
        }
      }
    } else {
      const float mean = a.rms ? 0.f : a.mean[row];
      const float rstd = a.rstd[row];
      const f32x2 a2 = f2_pack(rstd, rstd), b2 = f2_pack(-mean * rstd, -mean * rstd);
      // first pass: xs <- xhat, gs <- g = dy * (1 + scale) * weight, and the two row sums
      f32x2 s1 = zero2, s2 = zero2;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int v = lane + 32 * i;
        if (v < nvec) {
          f32x2 t[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) xs[i][j] = f2_fma(xs[i][j], a2, b2);
          if (sc) {
            unpack8_f2(sc[v], t);
#pragma unroll
            for (int j = 0; j < 4; ++j) gs[i][j] = f2_fma(gs[i][j], t[j], gs[i][j]);
          }
          if (wv) {
            unpack8_f2(wv[v], t);
#pragma unroll
            for (int j = 0; j < 4; ++j) gs[i][j] = f2_mul(gs[i][j], t[j]);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            s1 = f2_add(s1, gs[i][j]);
            s2 = f2_fma(gs[i][j], xs[i][j], s2);
          }
        }
      }
      float lo, hi;
      f2_unpack(s1, lo, hi);
      const float c1 = a.rms ? 0.f : warp_sum(lo + hi) * inv_d;
      f2_unpack(s2, lo, hi);
      const float c2 = warp_sum(lo + hi) * inv_d;
      // dx = rstd * (g - c1 - xhat * c2)
      const f32x2 k0 = f2_pack(-c1 * rstd, -c1 * rstd), k2 = f2_pack(-c2 * rstd, -c2 * rstd);
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int v = lane + 32 * i;
        if (v < nvec) {
          f32x2 o[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = f2_fma(xs[i][j], k2, f2_fma(gs[i][j], a2, k0));
          orow[v] = pack8_f2(o);
        }
      }
    }
  }
}

// Shared-memory-resident variant: one row buffer per warp and up to 32 warps per CTA, the passes read
// the row from shared memory instead of holding it in registers as fp32. Thirty-two warps of ~60
// registers instead of twelve of ~160: every row of a 4608-row problem is in flight at once (31 rows
// per SM), and on long problems the issue slots are shared by eight warps per scheduler instead of
// three, which is what the register-resident kernel above lacks (it issues 0.4 instructions per cycle
// and scheduler). Statistics in one pass over values shifted by the row's first element (the variance
// as E[(x-k)^2] - E[x-k]^2 does not cancel unless that element is a far outlier); the backward uses
// dx = g*rstd + (x-mean)*(-c2*rstd^2) - c1*rstd with c2 = rstd^2 * mean(g*(x-mean)) folded in.
template <bool BWD>
__global__ void __launch_bounds__(1024, 1) norm_rows_smem_kernel(const NormArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int NT = BWD ? 2 : 1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int D = a.D, nvec = D >> 3;
  const uint32_t row_bytes = (uint32_t)D * 2u;
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem) + warp;
  uint8_t* buf = smem + kBarBytes + (size_t)warp * NT * row_bytes;
  if (lane == 0) {
    mbar_init(bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  const int stride = gridDim.x * nwarps;
  auto issue = [&](int row) {
    mbar_expect_tx(bar, NT * row_bytes);
    bulk_g2s(buf, a.x + (size_t)row * D, row_bytes, bar);
    if (BWD) bulk_g2s(buf + row_bytes, a.dy + (size_t)row * D, row_bytes, bar);
  };
  int row = blockIdx.x * nwarps + warp;
  if (lane == 0 && row < a.rows) issue(row);
  const bf16x8* wv = a.weight ? reinterpret_cast<const bf16x8*>(a.weight) : nullptr;
  const bf16x8* bv = a.bias ? reinterpret_cast<const bf16x8*>(a.bias) : nullptr;
  const bf16x8* sx = reinterpret_cast<const bf16x8*>(buf);
  const float inv_d = 1.f / (float)D;
  const f32x2 zero2 = f2_pack(0.f, 0.f);
  uint32_t phase = 0;
  for (; row < a.rows; row += stride, phase ^= 1u) {
    if (!mbar_wait(bar, phase)) {
      if (lane == 0) atomicExch(a.err, 1);
      break;
    }
    const int b = row / a.rows_per_batch;
    const bf16x8* sc =
        a.scale ? reinterpret_cast<const bf16x8*>(a.scale + (size_t)b * a.mod_stride) : nullptr;
    bf16x8* orow = reinterpret_cast<bf16x8*>(a.out + (size_t)row * D);
    if (!BWD) {
      const bf16x8* sh =
          a.shift ? reinterpret_cast<const bf16x8*>(a.shift + (size_t)b * a.mod_stride) : nullptr;
      const float kshift = a.rms ? 0.f : __bfloat162float(reinterpret_cast<const bf16*>(buf)[0]);
      const f32x2 k2 = f2_pack(kshift, kshift);
      f32x2 s1a = zero2, s1b = zero2, s2a = zero2, s2b = zero2;
#pragma unroll 4
      for (int v = lane; v < nvec; v += 32) {
        f32x2 p[4];
        unpack8_f2(sx[v], p);
#pragma unroll
        for (int j = 0; j < 4; ++j) p[j] = f2_sub(p[j], k2);
        s1a = f2_add(s1a, f2_add(p[0], p[1]));
        s1b = f2_add(s1b, f2_add(p[2], p[3]));
        s2a = f2_fma(p[0], p[0], s2a);
        s2b = f2_fma(p[1], p[1], s2b);
        s2a = f2_fma(p[2], p[2], s2a);
        s2b = f2_fma(p[3], p[3], s2b);
      }
      float lo, hi;
      f2_unpack(f2_add(s1a, s1b), lo, hi);
      const float m1 = warp_sum(lo + hi) * inv_d;
      f2_unpack(f2_add(s2a, s2b), lo, hi);
      const float m2 = warp_sum(lo + hi) * inv_d;
      const float mean = a.rms ? 0.f : kshift + m1;
      const float var = a.rms ? m2 : fmaxf(m2 - m1 * m1, 0.f);
      const float rstd = rsqrtf(var + a.eps);
      if (lane == 0) {
        if (a.mean) a.mean[row] = mean;
        if (a.rstd) a.rstd[row] = rstd;
      }
      const f32x2 a2 = f2_pack(rstd, rstd), b2 = f2_pack(-mean * rstd, -mean * rstd);
#pragma unroll 2
      for (int v = lane; v < nvec; v += 32) {
        f32x2 o[4], t[4];
        unpack8_f2(sx[v], o);
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = f2_fma(o[j], a2, b2);
        if (wv) {
          unpack8_f2(wv[v], t);
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = f2_mul(o[j], t[j]);
        }
        if (bv) {
          unpack8_f2(bv[v], t);
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = f2_add(o[j], t[j]);
        }
        if (sc) {
          unpack8_f2(sc[v], t);
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = f2_fma(o[j], t[j], o[j]);
        }
        if (sh) {
          unpack8_f2(sh[v], t);
#pragma unroll
          for (int j = 0; j < 4; ++j) o[j] = f2_add(o[j], t[j]);
        }
        orow[v] = pack8_f2(o);
      }
    } else {
      const float mean = a.rms ? 0.f : a.mean[row];
      const float rstd = a.rstd[row];
      const f32x2 nm2 = f2_pack(-mean, -mean);
      const bf16x8* sg = sx + nvec;
      // pass 1: sum of g = dy * (1 + scale) * weight and of g * (x - mean)
      f32x2 s1a = zero2, s1b = zero2, s2a = zero2, s2b = zero2;
#pragma unroll 2
      for (int v = lane; v < nvec; v += 32) {
        f32x2 x[4], g[4], t[4];
        unpack8_f2(sx[v], x);
        unpack8_f2(sg[v], g);
        if (sc) {
          unpack8_f2(sc[v], t);
#pragma unroll
          for (int j = 0; j < 4; ++j) g[j] = f2_fma(g[j], t[j], g[j]);
        }
        if (wv) {
          unpack8_f2(wv[v], t);
#pragma unroll
          for (int j = 0; j < 4; ++j) g[j] = f2_mul(g[j], t[j]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) x[j] = f2_add(x[j], nm2);
        s1a = f2_add(s1a, f2_add(g[0], g[1]));
        s1b = f2_add(s1b, f2_add(g[2], g[3]));
        s2a = f2_fma(g[0], x[0], s2a);
        s2b = f2_fma(g[1], x[1], s2b);
        s2a = f2_fma(g[2], x[2], s2a);
        s2b = f2_fma(g[3], x[3], s2b);
      }
      float lo, hi;
      f2_unpack(f2_add(s1a, s1b), lo, hi);
      const float c1 = a.rms ? 0.f : warp_sum(lo + hi) * inv_d;
      f2_unpack(f2_add(s2a, s2b), lo, hi);
      const float c2 = warp_sum(lo + hi) * inv_d * rstd;            // mean(g * xhat)
      // dx = rstd * (g - c1 - xhat * c2) = g * rstd + (x - mean) * (-c2 * rstd^2) - c1 * rstd
      const f32x2 ka = f2_pack(rstd, rstd), kb = f2_pack(-c2 * rstd * rstd, -c2 * rstd * rstd),
                  kc = f2_pack(-c1 * rstd, -c1 * rstd);
#pragma unroll 2
      for (int v = lane; v < nvec; v += 32) {
        f32x2 x[4], g[4], t[4];
        unpack8_f2(sx[v], x);
        unpack8_f2(sg[v], g);
        if (sc) {
          unpack8_f2(sc[v], t);
#pragma unroll
          for (int j = 0; j < 4; ++j) g[j] = f2_fma(g[j], t[j], g[j]);
        }
        if (wv) {
          unpack8_f2(wv[v], t);
#pragma unroll
          for (int j = 0; j < 4; ++j) g[j] = f2_mul(g[j], t[j]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          x[j] = f2_fma(f2_add(x[j], nm2), kb, f2_fma(g[j], ka, kc));
        if (a.addend) {
          unpack8_f2(reinterpret_cast<const bf16x8*>(a.addend + (size_t)row * D)[v], t);
#pragma unroll
          for (int j = 0; j < 4; ++j) x[j] = f2_add(x[j], t[j]);
        }
        orow[v] = pack8_f2(x);
      }
    }
    __syncwarp();
    if (lane == 0 && row + stride < a.rows) {
      fence_proxy_async_smem();  // the warp's reads of the buffer precede the copy engine's writes
      issue(row + stride);
    }
  }
}

int* g_norm_err = nullptr;
int g_norm_sms = 0;

// ERI_B200_NORM_SMEM=0 (or eri_norm_set_smem_variant(0)) keeps the register-resident kernel.
int g_norm_smem = -1;
bool norm_smem_variant() {
  if (g_norm_smem < 0) {
    const char* e = getenv("ERI_B200_NORM_SMEM");
    g_norm_smem = (e && e[0] == '0') ? 0 : 1;
  }
  return g_norm_smem == 1;
}

template <bool BWD>
int launch_rows_smem(const NormArgs& a, cudaStream_t st) {
  constexpr int NT = BWD ? 2 : 1;
  const int per_warp = NT * a.D * 2;
  int warps = (216 * 1024 - kBarBytes) / per_warp;
  if (warps > 32) warps = 32;
  if (warps < 4) return -100;
  const int smem = kBarBytes + warps * per_warp;
  int grid = (a.rows + warps - 1) / warps;
  if (grid > g_norm_sms) grid = g_norm_sms;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(norm_rows_smem_kernel<BWD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             216 * 1024) != cudaSuccess)
      return -101;
    configured = true;
  }
  norm_rows_smem_kernel<BWD><<<grid, warps * 32, smem, st>>>(a);
  return (int)cudaGetLastError();
}

template <bool BWD>
int launch_rows(const NormArgs& a, cudaStream_t st) {
  constexpr int NT = BWD ? 2 : 1;
  const int D = a.D;
  if (norm_smem_variant()) {
    const int code = launch_rows_smem<BWD>(a, st);
    if (code != -100) return code;
  }
  if (a.addend) return -100;   // only the shared-memory-resident kernel adds a second gradient
  const int per_warp = kRingStages<BWD> * NT * D * 2;
  int warps = (200 * 1024 - kBarBytes) / per_warp;
  if (warps > (BWD ? 8 : 12)) warps = BWD ? 8 : 12;
  if (warps < 1) return -100;
  const int smem = kBarBytes + warps * per_warp;
  const int vpl = ((D >> 3) + 31) / 32;
  int grid = (a.rows + warps - 1) / warps;
  if (grid > g_norm_sms) grid = g_norm_sms;
#define ERI_CASE(V)                                                                             \
  do {                                                                                          \
    static bool configured = false;                                                             \
    if (!configured) {                                                                          \
      if (cudaFuncSetAttribute(norm_rows_kernel<V, BWD>,                                        \
                               cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) !=      \
          cudaSuccess)                                                                          \
        return -101;                                                                            \
      configured = true;                                                                        \
    }                                                                                           \
    norm_rows_kernel<V, BWD><<<grid, warps * 32, smem, st>>>(a);                                \
  } while (0)
  if (vpl <= 4) ERI_CASE(4); else if (vpl <= 8) ERI_CASE(8); else if (vpl <= 12) ERI_CASE(12); else ERI_CASE(16);
#undef ERI_CASE
  return (int)cudaGetLastError();
}

int norm_setup() {
  if (!g_norm_err) {
    if (cudaMalloc(&g_norm_err, sizeof(int)) != cudaSuccess) return -3;
    cudaMemset(g_norm_err, 0, sizeof(int));
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_norm_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_norm_sms <= 0) g_norm_sms = 148;
  }
  return 0;
}

}  // namespace

extern "C" {

// Chooses between the shared-memory-resident (1) and the register-resident (0) row kernels; returns
// the previous choice.
int eri_norm_set_smem_variant(int on) {
  const int prev = norm_smem_variant() ? 1 : 0;
  g_norm_smem = on ? 1 : 0;
  return prev;
}

// 0, or 1 when a bounded wait for a row copy ran out (the word is cleared by the read).
int eri_norm_check_error() {
  if (!g_norm_err) return 0;
  int h = 0;
  cudaMemcpy(&h, g_norm_err, sizeof(int), cudaMemcpyDeviceToHost);
  if (h) cudaMemset(g_norm_err, 0, sizeof(int));
  return h;
}

// Returns -100 when the shape is outside this kernel's range (caller uses the general kernel).
int eri_norm_modulate_fwd_warp(const void* x, const void* scale, const void* shift, const void* weight,
                               const void* bias, void* y, float* mean, float* rstd, int rows, int D,
                               int rows_per_batch, int mod_stride, float eps, int rms, void* stream) {
  if (D % 8 || D > 4096 || D < 256) return -100;
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return -100;
  if (norm_setup()) return -3;
  NormArgs a;
  a.x = (const bf16*)x; a.dy = nullptr; a.scale = (const bf16*)scale; a.shift = (const bf16*)shift;
  a.weight = (const bf16*)weight; a.bias = (const bf16*)bias; a.out = (bf16*)y; a.addend = nullptr;
  a.mean = mean; a.rstd = rstd; a.rows = rows; a.D = D; a.rows_per_batch = rows_per_batch;
  a.mod_stride = mod_stride; a.eps = eps; a.rms = rms; a.err = g_norm_err;
  return launch_rows<false>(a, (cudaStream_t)stream);
}

// addend (may be null): a [rows, D] bf16 tensor added to dx, e.g. the gradient that reached x through a
// residual branch, so that autograd has no separate sum to launch.
int eri_norm_modulate_bwd_warp_add(const void* dy, const void* x, const void* scale, const void* weight,
                                   const float* mean, const float* rstd, void* dx, const void* addend, int rows,
                                   int D, int rows_per_batch, int mod_stride, int rms, void* stream);

int eri_norm_modulate_bwd_warp(const void* dy, const void* x, const void* scale, const void* weight,
                               const float* mean, const float* rstd, void* dx, int rows, int D,
                               int rows_per_batch, int mod_stride, int rms, void* stream) {
  return eri_norm_modulate_bwd_warp_add(dy, x, scale, weight, mean, rstd, dx, nullptr, rows, D, rows_per_batch,
                                        mod_stride, rms, stream);
}

int eri_norm_modulate_bwd_warp_add(const void* dy, const void* x, const void* scale, const void* weight,
                                   const float* mean, const float* rstd, void* dx, const void* addend, int rows,
                                   int D, int rows_per_batch, int mod_stride, int rms, void* stream) {
  if (D % 8 || D > 4096 || D < 256) return -100;
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(addend)) & 15) != 0)
    return -100;
  if (norm_setup()) return -3;
  NormArgs a;
  a.addend = (const bf16*)addend;
  a.x = (const bf16*)x; a.dy = (const bf16*)dy; a.scale = (const bf16*)scale; a.shift = nullptr;
  a.weight = (const bf16*)weight; a.bias = nullptr; a.out = (bf16*)dx;
  a.mean = const_cast<float*>(mean); a.rstd = const_cast<float*>(rstd); a.rows = rows; a.D = D;
  a.rows_per_batch = rows_per_batch; a.mod_stride = mod_stride; a.eps = 0.f; a.rms = rms;
  a.err = g_norm_err;
  return launch_rows<true>(a, (cudaStream_t)stream);
}

}  // extern "C"
