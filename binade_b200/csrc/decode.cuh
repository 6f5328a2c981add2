// R4 lane-word decode shared by the plain-load kernels and the tensor-core GEMM (device only).
#pragma once

#include "common.cuh"

namespace bn {

// ---------------------------------------------------------------------------------------------
// Exponent lookup. A code byte holds two 4-bit codes (c0 | c1 << 4); the pair table maps it to
// the two exponents already placed in a BF16x2 word: table[c0] << 7 | table[c1] << 23. Code 15
// (escape) maps to exponent bits 0 so that the escape byte can be OR-ed in afterwards. The table
// is replicated once per lane (entry i of lane l at word i * 32 + l): a lookup never conflicts.
// ---------------------------------------------------------------------------------------------
constexpr int LUT_WORDS = 256 * 32;

__device__ __forceinline__ void build_pair_lut(uint32_t *lut, const uint8_t *table) {
  __shared__ uint32_t t16[16];
  if (threadIdx.x < 16) t16[threadIdx.x] = threadIdx.x == 15 ? 0u : (uint32_t)table[threadIdx.x];
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < LUT_WORDS; i += blockDim.x) {
    uint32_t code = i >> 5;
    lut[i] = (t16[code & 15] << 7) | (t16[code >> 4] << 23);
  }
}

// Four weights of one lane word as two BF16x2 words (w01 = weight0 | weight1 << 16, w23 alike).
// raw4: the four raw bytes (sign << 7 | mantissa); c: the uint16 of codes; lut_lane: shared
// address of this lane's column of the pair table.
__device__ __forceinline__ void decode4(uint32_t raw4, uint32_t c, uint32_t lut_lane, uint32_t &w01, uint32_t &w23) {
  uint32_t e01 = lds_u32(lut_lane + ((c << 7) & 0x7F80u));
  uint32_t e23 = lds_u32(lut_lane + ((c >> 1) & 0x7F80u));
  uint32_t p01 = __byte_perm(raw4, 0u, 0x1100);  // bytes b0 b0 b1 b1
  uint32_t p23 = __byte_perm(raw4, 0u, 0x3322);  // bytes b2 b2 b3 b3
  w01 = (p01 & 0x807F807Fu) | e01;
  w23 = (p23 & 0x807F807Fu) | e23;
}

// Patches the escaped weights (code 15) of a flagged tile with the row's next escape bytes, in
// weight order across the warp, and advances the row's escape cursor. Whole warp takes part.
__device__ __forceinline__ void apply_escapes(uint32_t c, const uint8_t *__restrict__ esc, uint32_t &epos, uint32_t lt, uint32_t &w01, uint32_t &w23) {
  uint32_t hit = c & (c >> 1) & (c >> 2) & (c >> 3) & 0x1111u;  // bit 4j: code j == 15
  uint32_t pre, tot;
  warp_scan_small(__popc(hit), lt, pre, tot);
  uint32_t q = epos + pre;
  if (hit & 0x0001u) w01 |= (uint32_t)esc[q++] << 7;
  if (hit & 0x0010u) w01 |= (uint32_t)esc[q++] << 23;
  if (hit & 0x0100u) w23 |= (uint32_t)esc[q++] << 7;
  if (hit & 0x1000u) w23 |= (uint32_t)esc[q++] << 23;
  epos += tot;
}

}  // namespace bn
