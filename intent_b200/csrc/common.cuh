// Shared host/device helpers of the sm_100a quantized-contraction library.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/intent_b200.h"

namespace ib200 {

// ---- host side -----------------------------------------------------------

// Process-wide count of kernels launched by this library.
void note_launch(int count = 1);

inline int cuda_status(cudaError_t error) {
  return error == cudaSuccess ? INTENT_B200_OK : INTENT_B200_ERR_CUDA + static_cast<int>(error);
}

// Returns the status of the launch that was just issued (cudaPeekAtLastError
// would also see sticky errors of unrelated work; cudaGetLastError clears ours).
inline int launch_status() { return cuda_status(cudaGetLastError()); }

// Dry-run observation of a launch: while a sink is installed on the calling thread (intent_b200_observe_begin),
// the main compute kernels' launch sites fill it with what they WOULD launch - the kernel instance's resource
// usage from cudaFuncGetAttributes and the launch plan - and launch nothing.
struct LaunchFacts {
  int valid;
  int registers;        // per thread
  int local_bytes;      // per-thread local memory (register spills land here)
  int static_smem;      // bytes
  int dynamic_smem;     // bytes requested by this launch
  int threads;          // per CTA
  int grid;             // CTAs
  int cluster;          // CTAs per cluster (1 = none)
  char kernel[64];      // kernel family and the plan's distinguishing choice
};
LaunchFacts* observe_sink();
int record_launch(LaunchFacts* sink, const void* kernel, const char* name, int grid, int threads, int dynamic_smem,
                  int cluster);

struct View2 {
  void* p;
  int64_t d0, d1, s0, s1;
};
struct View1 {
  void* p;
  int64_t d0, s0;
};
struct View3 {
  void* p;
  int64_t d0, d1, d2, s0, s1, s2;
};

inline bool contiguous(const View1& v) { return v.d0 <= 1 || v.s0 == 1; }
inline bool contiguous(const View2& v) {
  return (v.d1 <= 1 || v.s1 == 1) && (v.d0 <= 1 || v.s0 == v.d1);
}
inline bool contiguous(const View3& v) {
  return (v.d2 <= 1 || v.s2 == 1) && (v.d1 <= 1 || v.s1 == v.d2) && (v.d0 <= 1 || v.s0 == v.d1 * v.d2);
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define IB200_VIEW1_ARG(p) ib200::View1{p, p##_d0, p##_s0}
#define IB200_VIEW2_ARG(p) ib200::View2{p, p##_d0, p##_d1, p##_s0, p##_s1}
#define IB200_VIEW3_ARG(p) ib200::View3{p, p##_d0, p##_d1, p##_d2, p##_s0, p##_s1, p##_s2}

// ---- device side ---------------------------------------------------------
#ifdef __CUDACC__

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) | c
  return d;
}

__device__ __forceinline__ uint32_t lop3_and_xor_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) ^ c
  return d;
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(selector));
  return d;
}

__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint2 ldg_stream_v2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

// Element-type traits for the 16-bit activation types.
template <typename T>
struct Elem;

template <>
struct Elem<__half> {
  // 0x6400 | q is the half 1024 + q (ulp is 1 at 2^10); subtracting 1032 gives q - 8 exactly.
  static constexpr uint32_t kMagic2 = 0x64006400u;
  static constexpr uint32_t kBias2 = 0x64086408u;  // half2(1032, 1032)
  __device__ static __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  __device__ static __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  __device__ static __forceinline__ float to_float(uint16_t bits) {
    return __half2float(__ushort_as_half(bits));
  }
  __device__ static __forceinline__ uint16_t from_float(float v) {
    return __half_as_ushort(__float2half_rn(v));
  }
  __device__ static __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                  uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

template <>
struct Elem<__nv_bfloat16> {
  // 0x4300 | q is the bfloat16 128 + q (ulp is 1 at 2^7); subtracting 136 gives q - 8 exactly.
  static constexpr uint32_t kMagic2 = 0x43004300u;
  static constexpr uint32_t kBias2 = 0x43084308u;  // bf16x2(136, 136)
  __device__ static __forceinline__ uint32_t sub2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  __device__ static __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
  }
  __device__ static __forceinline__ float to_float(uint16_t bits) {
    return __uint_as_float(static_cast<uint32_t>(bits) << 16);
  }
  __device__ static __forceinline__ uint16_t from_float(float v) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
  }
  __device__ static __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                  uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
};

#endif  // __CUDACC__

// w4a16_table.cu: one small contraction as a table of one problem (kTableDeclined: not that kind of call)
constexpr int kTableDeclined = -77001;
int w4a16_table_single_f16(View2, View2, View2, View2, int, int, void*, int64_t, cudaStream_t);
int w4a16_table_single_bf16(View2, View2, View2, View2, int, int, void*, int64_t, cudaStream_t);
int64_t w4a16_table_single_workspace_bytes(int64_t M, int64_t K, int64_t N);

}  // namespace ib200
