// In-register expansion of packed int4 weights into 16-bit float pairs for the
// bandwidth kernels (magic-number trick with deferred bias removal).
#pragma once

#include "common.cuh"

namespace ib200 {

__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) ^ c
  return d;
}

// Per element type: how one packed word becomes four pair registers
// (k0,k4) (k1,k5) (k2,k6) (k3,k7) holding "bias + (q or q^8)", how the staged
// activations are pre-scaled, and the per-k coefficient of the correction sum.
template <typename T>
struct Expand;

template <>
struct Expand<__half> {
  // even pairs: 0x6400 | q        = 1024 + q     (activation as is,   correction 1032 * x)
  // odd pairs : 0x6400 | (q << 4) = 1024 + 16 q  (activation x / 16,  correction 1152 * x/16)
  __device__ static __forceinline__ void magic(bool twos, uint32_t& a, uint32_t& b) {
    a = 0x64006400u ^ (twos ? 0x00080008u : 0u);
    b = 0x64006400u ^ (twos ? 0x00800080u : 0u);
  }
  __device__ static __forceinline__ void word(uint32_t w, uint32_t ma, uint32_t mb, uint32_t (&pair)[4]) {
    const uint32_t hi = w >> 8;
    pair[0] = lop3_and_xor(w, 0x000F000Fu, ma);
    pair[1] = lop3_and_xor(w, 0x00F000F0u, mb);
    pair[2] = lop3_and_xor(hi, 0x000F000Fu, ma);
    pair[3] = lop3_and_xor(hi, 0x00F000F0u, mb);
  }
  __device__ static __forceinline__ uint32_t scale_odd(uint32_t pair) {
    return Elem<__half>::mul2(pair, 0x2C002C00u);  // * 1/16 (exact unless subnormal)
  }
  static constexpr float kEven = 1032.f, kOdd = 1152.f;
};

template <>
struct Expand<__nv_bfloat16> {
  // 0x4300 | q = 128 + q for every pair (7 mantissa bits leave no room for the in-place form)
  __device__ static __forceinline__ void magic(bool twos, uint32_t& a, uint32_t& b) {
    a = b = 0x43004300u ^ (twos ? 0x00080008u : 0u);
  }
  __device__ static __forceinline__ void word(uint32_t w, uint32_t ma, uint32_t, uint32_t (&pair)[4]) {
    pair[0] = lop3_and_xor(w, 0x000F000Fu, ma);
    pair[1] = lop3_and_xor(w >> 4, 0x000F000Fu, ma);
    pair[2] = lop3_and_xor(w >> 8, 0x000F000Fu, ma);
    pair[3] = lop3_and_xor(w >> 12, 0x000F000Fu, ma);
  }
  __device__ static __forceinline__ uint32_t scale_odd(uint32_t pair) { return pair; }
  static constexpr float kEven = 136.f, kOdd = 136.f;
};

template <typename T>
__device__ __forceinline__ float pair_sum(uint32_t pair) {
  return Elem<T>::to_float(uint16_t(pair & 0xFFFF)) + Elem<T>::to_float(uint16_t(pair >> 16));
}

}  // namespace ib200
