// NVFP4 quantisation shared by the stand-alone quantiser and the kernels that emit FP4 directly.
//
// Format: E2M1 codes {0, .5, 1, 1.5, 2, 3, 4, 6} with sign, two per byte (even K index in the low nibble), one
// E4M3 scale per 16 consecutive K elements, one fp32 scale per tensor:
//   tensor_scale = amax / (6 * 448),  block_scale = E4M3(block_amax / (6 * tensor_scale)),
//   code = E2M1(x / (block_scale * tensor_scale)),  all round-to-nearest-even, saturating.
// Block scales live in 512-byte tiles of 128 rows x 4 blocks: tile (r / 128) * ktiles4 + kb / 4, byte
// (r % 32) * 16 + ((r % 128) / 32) * 4 + kb % 4, with the K-tile count padded to a multiple of 4.
#pragma once
#include <cuda_fp8.h>

#include "common.cuh"

namespace sana {

// positive value -> E4M3 bits (round to nearest even, saturating at 448) and back
__device__ __forceinline__ uint32_t e4m3_bits(float v) { return (uint32_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3); }
__device__ __forceinline__ float e4m3_value(uint32_t bits) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)bits, __NV_E4M3)));
}
// two values -> one byte of E2M1 codes (lo in the low nibble), round to nearest even, saturating at 6
__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
  uint16_t r;
  asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %2, %1;\n\tmov.b16 %0, {t, 0};\n\t}" : "=h"(r) : "f"(lo), "f"(hi));
  return (uint32_t)r;
}

// The arithmetic of one 16-block, shared by every kernel that quantises (and restated by the oracle):
//   block scale = E4M3(block_amax * inv6ts),  inv6ts = 1 / (6 * tensor_scale)          (fp32, round to nearest)
//   code        = E2M1(x * inv),              inv    = 1 / (block_scale * tensor_scale), 0 when the scale is 0
// Multiplying by the reciprocal (as Transformer Engine's quantiser does) instead of dividing keeps the inner loop
// to one multiply and half a conversion per element.
struct Fp4Block {
  float inv;         // 1 / (block scale * tensor scale), or 0
  uint32_t sf_byte;  // the block scale as E4M3 bits
};
__device__ __forceinline__ Fp4Block fp4_block_scale(float block_amax, float ts, float inv6ts) {
  Fp4Block b;
  b.sf_byte = e4m3_bits(block_amax * inv6ts);
  const float denom = e4m3_value(b.sf_byte) * ts;
  b.inv = denom > 0.f ? __frcp_rn(denom) : 0.f;
  return b;
}
__device__ __forceinline__ uint32_t fp4_codes8(const float (&f)[8], float inv) {
  return e2m1x2(f[0] * inv, f[1] * inv) | (e2m1x2(f[2] * inv, f[3] * inv) << 8) | (e2m1x2(f[4] * inv, f[5] * inv) << 16) |
         (e2m1x2(f[6] * inv, f[7] * inv) << 24);
}

inline int64_t ktiles4_of(int64_t K) { return ceil_div(ceil_div(K, 64), 4) * 4; }

// Where a producing kernel writes the FP4 image of its bf16 output instead of (or besides) the bf16 tensor.
// The tensor scale is NOT derived from this call's data (that would take a second pass): the kernel uses
// scale_in[1] and accumulates the maximum magnitude of what it produced into amax_out, from which the host
// side derives the scale of a later call (or checks that the one it used was large enough).
struct Fp4Sink {
  unsigned char* q;        // [rows, K / 2] codes, or null: no FP4 output
  unsigned char* sf;       // scale tiles (zero-initialised once by the owner: padding bytes are never written)
  const float* scale_in;   // device floats {amax, tensor_scale}; tensor_scale is used
  float* amax_out;         // device float, atomically raised to max |output| (as bf16), or null
  int K;                   // row length (a multiple of 32)
  int ktiles4;
};

// One lane holds 8 consecutive values of a 16-block (already rounded to bf16), its neighbour lane ^ 1 the other
// 8.  Returns the lane's 8 codes; *scale_byte is the block's E4M3 scale (same in both lanes).
__device__ __forceinline__ uint32_t fp4_quant8_of16(const float (&f)[8], float ts, float inv6ts, uint32_t* scale_byte) {
  float bm = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) bm = fmaxf(bm, fabsf(f[e]));
  bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 1));
  const Fp4Block b = fp4_block_scale(bm, ts, inv6ts);
  *scale_byte = b.sf_byte;
  return fp4_codes8(f, b.inv);
}

// byte offset of the scale of (row r, 16-block kb) in the tiled scale buffer
__device__ __forceinline__ int64_t fp4_sf_offset(int64_t r, int kb, int ktiles4) {
  return ((r >> 7) * ktiles4 + (kb >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (kb & 3);
}

}  // namespace sana
