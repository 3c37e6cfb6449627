// Warp-level bf16 MMA (mma.sync m16n8k16, fp32 accumulate) with fragments loaded straight from
// global memory, for the small contractions around the projection path whose operands are streamed
// once and whose output is tiny (k x k, or batch x batch): the kernels are bound by the operand
// stream, not by the tensor pipe, so there is no shared-memory staging.
//
// A contraction index may be permuted freely as long as both operands use the same permutation.
// Each lane therefore loads FOUR consecutive contraction elements (one 16-byte load for float, one
// 8-byte load for bf16) at k0 + 4 * (lane & 3): elements 0-1 go to the fragment slot the ISA names
// k = 2c, 2c+1 and elements 2-3 to the slot it names k = 2c+8, 2c+9.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace gb {

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16x2(__nv_bfloat16 x, __nv_bfloat16 y) {
  __nv_bfloat162 h(x, y);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Four consecutive contraction elements of one operand row as two bf16x2 words (hi) and, for a
// float source, the two words of the residual x - bf16(x) (lo), so that
// hi*hi + lo*hi + hi*lo reproduces the float product to about 2^-16.
struct Quad {
  uint32_t hi[2];
  uint32_t lo[2];
};

template <bool VEC>
__device__ __forceinline__ Quad load_quad(const float* row, long long k, long long k_end, bool row_ok) {
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (row_ok) {
    if (VEC) {
      if (k < k_end) {
        const float4 f = __ldg(reinterpret_cast<const float4*>(row + k));
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
      }
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (k + e < k_end) v[e] = __ldg(row + k + e);
    }
  }
  Quad q;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const __nv_bfloat16 x = __float2bfloat16_rn(v[2 * h]), y = __float2bfloat16_rn(v[2 * h + 1]);
    q.hi[h] = pack_bf16x2(x, y);
    q.lo[h] = pack_bf16x2(__float2bfloat16_rn(v[2 * h] - __bfloat162float(x)),
                          __float2bfloat16_rn(v[2 * h + 1] - __bfloat162float(y)));
  }
  return q;
}

template <bool VEC>
__device__ __forceinline__ Quad load_quad(const __nv_bfloat16* row, long long k, long long k_end, bool row_ok) {
  Quad q;
  q.hi[0] = q.hi[1] = q.lo[0] = q.lo[1] = 0u;
  if (row_ok) {
    if (VEC) {
      if (k < k_end) {
        const uint2 w = __ldg(reinterpret_cast<const uint2*>(row + k));
        q.hi[0] = w.x;
        q.hi[1] = w.y;
      }
    } else {
      const __nv_bfloat16 z = __float2bfloat16_rn(0.f);
      __nv_bfloat16 v[4] = {z, z, z, z};
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (k + e < k_end) v[e] = row[k + e];
      q.hi[0] = pack_bf16x2(v[0], v[1]);
      q.hi[1] = pack_bf16x2(v[2], v[3]);
    }
  }
  return q;
}

}  // namespace gb
