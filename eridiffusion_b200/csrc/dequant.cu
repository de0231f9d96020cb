// Weight de-quantisation into a bf16 scratch operand for the tcgen05 GEMM: int8 (one scale per
// output row), int4 and NF4 (two codes per byte, one scale per `block` consecutive elements).
// A frozen base weight stored in 8 or 4 bits is expanded right before the GEMM that consumes it;
// for the layer sizes of the supported models the scratch (<= 75 MB) stays in the 126 MB L2, so the
// GEMM's TMA loads read it back without a DRAM round trip. One thread expands 16 codes (int8) or
// 16 bytes = 32 codes (4-bit) and writes 16-byte vectors.
// Reference: QuantoManager INT8 absmax / INT4 / NF4 (src/memory/quanto.rs:168-426), de-quantised
// with elementwise tensor ops on every use.
#include "ptx.cuh"

using namespace eri;
typedef __nv_bfloat16 bf16;

namespace {

__constant__ float c_nf4[16] = {-1.0f, -0.6961928009986877f, -0.5250730514526367f, -0.39491748809814453f,
                                -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                                0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f,
                                0.33791524171829224f, 0.44070982933044434f, 0.5626170039176941f,
                                0.7229568362236023f, 1.0f};

__global__ void dequant_int8_kernel(const int8_t* __restrict__ q, const float* __restrict__ scale,
                                    bf16* __restrict__ out, long long rows, int cols) {
  const long long vec = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // 16 codes per thread
  const int vpr = cols >> 4;
  if (vec >= rows * vpr) return;
  const long long r = vec / vpr;
  const int c = (int)(vec - r * vpr) << 4;
  const float s = scale[r];
  const uint4 raw = *reinterpret_cast<const uint4*>(q + r * cols + c);
  const int8_t* b = reinterpret_cast<const int8_t*>(&raw);
  float lo[8], hi[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    lo[j] = (float)b[j] * s;
    hi[j] = (float)b[8 + j] * s;
  }
  bf16x8* o = reinterpret_cast<bf16x8*>(out + r * cols + c);
  o[0] = pack8(lo);
  o[1] = pack8(hi);
}

template <bool NF4>
__global__ void dequant_4bit_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scale,
                                    bf16* __restrict__ out, long long nbytes, int block) {
  // The 16-entry code table is read with a different index in every lane: from constant memory
  // that serialises per distinct address (116 us for a 12288 x 3072 weight against 25 us for int4),
  // from shared memory the 16 entries sit in 16 banks.
  __shared__ float s_nf4[16];
  if (NF4) {
    if (threadIdx.x < 16) s_nf4[threadIdx.x] = c_nf4[threadIdx.x];
    __syncthreads();
  }
  const long long vec = (long long)blockIdx.x * blockDim.x + threadIdx.x;   // 16 bytes = 32 codes
  if (vec * 16 >= nbytes) return;
  const uint4 raw = *reinterpret_cast<const uint4*>(q + vec * 16);
  const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
  const long long e0 = vec * 32;                   // first element; block is a multiple of 32
  const float s = scale[e0 / block];
  bf16x8* o = reinterpret_cast<bf16x8*>(out + e0);
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint8_t byte = b[g * 4 + j];
      const int c0 = byte & 0xF, c1 = byte >> 4;   // low nibble is the even element
      v[2 * j] = (NF4 ? s_nf4[c0] : ((float)c0 - 8.f) / 7.f) * s;
      v[2 * j + 1] = (NF4 ? s_nf4[c1] : ((float)c1 - 8.f) / 7.f) * s;
    }
    o[g] = pack8(v);
  }
}

}  // namespace

extern "C" {

// q [rows, cols] int8, scale [rows] fp32 -> out [rows, cols] bf16. cols % 16 == 0.
int eri_dequant_int8(const void* q, const float* scale, void* out, long long rows, int cols, void* stream) {
  if (cols % 16) return -1;
  const long long n = rows * (cols >> 4);
  dequant_int8_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const int8_t*)q, scale, (bf16*)out, rows, cols);
  return (int)cudaGetLastError();
}

// q: packed codes, two per byte (n_elems / 2 bytes); scale [n_elems / block] fp32; kind 0 int4, 1 nf4.
int eri_dequant_4bit(const void* q, const float* scale, void* out, long long n_elems, int block, int kind,
                     void* stream) {
  if (block % 32 || n_elems % 32) return -1;
  const long long nbytes = n_elems / 2, n = nbytes / 16;
  const unsigned grid = (unsigned)((n + 255) / 256);
  if (kind == 1)
    dequant_4bit_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)q, scale, (bf16*)out, nbytes, block);
  else
    dequant_4bit_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint8_t*)q, scale, (bf16*)out, nbytes, block);
  return (int)cudaGetLastError();
}

}  // extern "C"
